// Host-side file formats of the inference path: config.json, *.safetensors, expert .bin,
// tokenizer.json. No CUDA in here, so all of it is unit-testable without a GPU.
#pragma once
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace tffn {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};
// status codes shared with the C ABI (include/tffn.h)
enum { kOk = 0, kErrInvalid = -1, kErrIO = -2, kErrFormat = -3, kErrShape = -4, kErrCuda = -5, kErrCapacity = -6,
       kErrUnsupported = -7, kErrDevice = -8 };

// Mirrors QwenConfig (inference/include/model/qwen.h:9-23) and qwen_config_from_json
// (inference/src/model/qwen.cu:21-63): same keys, same defaults, head_dim = hidden / heads,
// eos/bos given as a number or as an array whose first element counts.
struct Config {
    int hidden_size = 896, intermediate_size = 4864, num_layers = 24, num_heads = 14, num_kv_heads = 2;
    int head_dim = 64, vocab_size = 151936, max_seq_len = 131072;
    float rms_norm_eps = 1e-6f, rope_theta = 1e6f;
    int eos_token_id = 151645, bos_token_id = 151643;
    bool tie_embeddings = true;
};
Config read_config(const std::string& model_dir);

// What one tensor-parallel rank owns. The reference is single-GPU; these are the slices of its matrices
// (q/k/v rows by head: inference/src/model/qwen.cu:317-319; o_proj columns: :413-415; gate/up rows and down
// columns on the intermediate dimension for the base FFN: :431-437 and for the expert:
// inference/src/model/expert.cu:51-58; LM-head rows on the vocabulary: qwen.cu:450-454).
// Heads are kept together with their kv head: with tp_size <= kv heads every rank takes whole kv groups;
// with more ranks than kv heads, tp_size / kv_heads ranks share a kv head (each computes its K/V row
// itself) and split its query heads as evenly as they go (7 heads over 2 ranks: 3 + 4).
struct TpPartition {
    int tp_rank = 0, tp_size = 1;
    int q_head0 = 0, n_q_heads = 0;    // first global query head, count (all of one kv group when kv heads are shared)
    int kv_head0 = 0, n_kv_heads = 0;  // first global kv head, count
    int i0 = 0, n_i = 0;               // rows of gate/up and columns of down (multiples of 64)
    int v0 = 0, n_v = 0;               // rows of the LM head (multiples of 8)
};
TpPartition tp_partition(const Config& c, int tp_rank, int tp_size);  // kErrUnsupported if the shape does not split

// One memory-mapped .safetensors file: u64 LE header length, JSON header, raw data
// (inference/src/io/safetensors.cpp:41-78). "__metadata__" is skipped.
struct TensorInfo {
    std::string dtype;
    std::vector<int64_t> shape;
    const uint8_t* data = nullptr;
    size_t nbytes = 0;
};
class SafeTensorsFile {
public:
    explicit SafeTensorsFile(const std::string& path);
    ~SafeTensorsFile();
    SafeTensorsFile(const SafeTensorsFile&) = delete;
    SafeTensorsFile& operator=(const SafeTensorsFile&) = delete;
    std::unordered_map<std::string, TensorInfo> tensors;
    std::string path;

private:
    void* map_ = nullptr;
    size_t size_ = 0;
    int fd_ = -1;
};
// Every *.safetensors of a directory, shards in sorted-name order; a name resolves to the
// first shard that holds it (inference/src/io/safetensors.cpp:104-131).
class SafeTensorsDir {
public:
    explicit SafeTensorsDir(const std::string& dir);
    ~SafeTensorsDir();
    bool has(const std::string& name) const;
    const TensorInfo& get(const std::string& name) const;  // throws kErrFormat "Missing tensor"
    // BF16 tensor with exactly `elems` elements, else throws (the reference checks the byte
    // size only: inference/src/model/qwen.cu:69-78)
    const uint16_t* bf16(const std::string& name, size_t elems) const;
    size_t num_shards() const { return shards_.size(); }
    size_t num_tensors() const;

private:
    std::vector<SafeTensorsFile*> shards_;
};

// Expert checkpoint (trainer/include/io/checkpoint.h:12-24; reader inference/src/io/checkpoint.cpp:11-65):
// u32 magic 0x45585054, u32 version, u32 layers, u32 hidden, u32 intermediate, then per layer
// gate[I*H], up[I*H], down[H*I] as little-endian fp32.
constexpr uint32_t kExpertMagic = 0x45585054u;
constexpr uint32_t kExpertVersion = 1u;
struct ExpertHeader {
    uint32_t magic = 0, version = 0, num_layers = 0, hidden = 0, intermediate = 0;
};
class ExpertFile {
public:
    explicit ExpertFile(const std::string& path);  // validates magic and that the file holds every matrix
    ~ExpertFile();
    ExpertHeader hdr;
    // fp32 matrix m (0 gate, 1 up, 2 down) of layer l, memory-mapped
    const float* matrix(int layer, int m) const;
    size_t matrix_elems() const { return (size_t)hdr.hidden * hdr.intermediate; }

private:
    void* map_ = nullptr;
    size_t size_ = 0;
    int fd_ = -1;
};
// Writer of the same format (trainer/src/io/checkpoint.cpp:15-52). mats[l*3+m] -> fp32 [I*H].
void write_expert(const std::string& path, uint32_t layers, uint32_t hidden, uint32_t inter,
                  const float* const* mats);

// Round-to-nearest-even fp32 -> bf16 (what __float2bfloat16 does in the reference's loader).
inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    __builtin_memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline float bf16_to_f32(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    __builtin_memcpy(&f, &u, 4);
    return f;
}

// Reference-compatible tokenizer (inference/src/io/tokenizer.cpp:16-153): vocab + merges +
// added_tokens from tokenizer.json, eos/bos from generation_config.json, per-byte lookup with
// "<0xNN>" fallback, greedy lowest-rank merge loop, decode with the byte-level space marker
// turned back into ' '. It deliberately keeps the reference's behaviour (bytes with no vocab
// entry are dropped).
class Tokenizer {
public:
    void load(const std::string& model_dir);
    std::vector<uint32_t> encode(const std::string& text) const;
    std::string decode(const std::vector<uint32_t>& ids) const;
    // The tokenisation Qwen2's tokenizer.json actually specifies, which the reference's encode() above does not
    // implement (it has no pre-tokenizer and no byte-to-unicode map, so spaces and newlines are dropped:
    // inference/src/io/tokenizer.cpp:86-108; the authors work around it with HF in tools/tokenize_correctly.py):
    // added tokens are cut out verbatim, the rest is split by the Qwen2 pre-tokenizer pattern
    //   (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
    // every piece's UTF-8 bytes go through GPT-2's byte-to-unicode map, and the merges are applied lowest
    // rank first. decode_bpe maps the characters back to bytes.
    std::vector<uint32_t> encode_bpe(const std::string& text) const;
    std::string decode_bpe(const std::vector<uint32_t>& ids) const;
    uint32_t get_id(const std::string& token) const;  // 0 and a warning on stderr when absent
    uint32_t eos_id = 151645, bos_id = 151643, pad_id = 151643;
    size_t vocab_size() const { return token_to_id_.size(); }

private:
    std::unordered_map<std::string, uint32_t> token_to_id_;
    std::unordered_map<uint32_t, std::string> id_to_token_;
    std::vector<std::pair<uint32_t, uint32_t>> merges_;
    std::unordered_map<uint64_t, uint32_t> merge_rank_;
    std::vector<std::string> added_;  // added tokens, longest first
    void bpe_piece(const std::string& bytes, std::vector<uint32_t>& out) const;
};

std::string read_text_file(const std::string& path, bool* ok);

}  // namespace tffn
