/* tffn.h — C ABI of the B200 inference path of tensor-ffn (Qwen2.5 decode with the base FFN
 * plus the expert-FFN delta at every layer).
 *
 * The reference has no FFI layer: its boundary is a set of C++ free functions over plain
 * structs of device pointers, called only from its main() (inference/src/main.cpp:97-204).
 * Each entry point below names the reference function it stands in for. Differences that a
 * binding has to know about:
 *   - the reference prints and calls exit(1) on every error (inference/include/backend/memory.h:5-11);
 *     these functions return a status (0 ok, <0 error) and keep a per-thread message in
 *     tffn_last_error();
 *   - the reference keeps one sequence per QwenModel (KV cache and scratch live inside it,
 *     inference/include/model/qwen.h:59-99); here weights (tffn_model, tffn_expert) are
 *     immutable after load and a tffn_session owns the paged KV cache, scratch and the per-slot
 *     sequence state, so one model serves many sessions and a session serves many sequences;
 *   - token ids and logits cross this boundary in HOST memory; the session moves them.
 * Threading: a session is used by one host thread at a time; different sessions may be used
 * from different threads. All functions are synchronous unless stated.
 */
#ifndef TFFN_H
#define TFFN_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct tffn_model tffn_model;
typedef struct tffn_expert tffn_expert;
typedef struct tffn_session tffn_session;
typedef struct tffn_tokenizer tffn_tokenizer;

enum {
    TFFN_OK = 0,
    TFFN_ERR_INVALID = -1,     /* bad argument */
    TFFN_ERR_IO = -2,          /* file cannot be opened / read */
    TFFN_ERR_FORMAT = -3,      /* bad magic, malformed header, missing tensor, wrong dtype */
    TFFN_ERR_SHAPE = -4,       /* tensor or expert shape does not match the model */
    TFFN_ERR_CUDA = -5,        /* CUDA runtime error, or no CUDA device */
    TFFN_ERR_CAPACITY = -6,    /* KV cache / batch / sequence capacity exceeded */
    TFFN_ERR_UNSUPPORTED = -7, /* shape outside what the kernels support */
    TFFN_ERR_DEVICE = -8       /* a kernel reported a status (bounded wait ran out, index check) */
};

/* QwenConfig (inference/include/model/qwen.h:9-23) */
typedef struct tffn_config {
    int32_t hidden_size, intermediate_size, num_layers, num_heads, num_kv_heads, head_dim;
    int32_t vocab_size, max_position_embeddings;
    float rms_norm_eps, rope_theta;
    int32_t eos_token_id, bos_token_id, tie_embeddings;
} tffn_config;

const char* tffn_last_error(void);
int tffn_version(void);
/* number of CUDA devices visible, 0 without a GPU (never fails) */
int tffn_device_count(void);

/* ---- host-only helpers (no GPU needed) ------------------------------------------------- */
/* qwen_config_from_json (inference/src/model/qwen.cu:21-63) */
int tffn_config_read(const char* model_dir, tffn_config* out);
/* Header of an expert .bin (inference/src/io/checkpoint.cpp:15-31); also checks the file length. */
int tffn_expert_probe(const char* path, uint32_t* version, uint32_t* num_layers, uint32_t* hidden,
                      uint32_t* intermediate);
/* checkpoint_save's file format (trainer/src/io/checkpoint.cpp:15-52): mats[layer*3 + m] points
 * to fp32 [intermediate*hidden], m = 0 gate, 1 up, 2 down. */
int tffn_expert_write(const char* path, uint32_t num_layers, uint32_t hidden, uint32_t intermediate,
                      const float* const* mats);
/* SafeTensorsDir::open / has (inference/src/io/safetensors.cpp:104-131): counts shards and
 * tensors; dtype_out (>= 8 bytes) and nbytes_out describe `name` when it is not NULL. */
int tffn_safetensors_probe(const char* model_dir, const char* name, int32_t* num_shards, int32_t* num_tensors,
                           char* dtype_out, uint64_t* nbytes_out);
/* io::Tokenizer (inference/include/io/tokenizer.h:9-24, inference/src/io/tokenizer.cpp) */
int tffn_tokenizer_load(const char* model_dir, tffn_tokenizer** out);
void tffn_tokenizer_free(tffn_tokenizer* t);
/* returns the number of ids (may exceed cap; only cap are written), <0 on error */
int tffn_tokenizer_encode(const tffn_tokenizer* t, const char* text, uint32_t* ids, int cap);
/* returns the number of bytes of the decoded text (without NUL; may exceed cap), <0 on error */
int tffn_tokenizer_decode(const tffn_tokenizer* t, const uint32_t* ids, int n, char* out, int cap);
/* The byte-level BPE that Qwen2's tokenizer.json specifies (added tokens cut out, NFC, the Qwen2 pre-tokenizer
 * pattern, GPT-2's byte-to-unicode map, merges lowest rank first), same calling convention. The reference's
 * encoder (inference/src/io/tokenizer.cpp:86-135) implements none of this and drops spaces and newlines; its
 * authors tokenise with HF instead (tools/tokenize_correctly.py:11-36). tffn_tokenizer_encode / _decode keep
 * the reference's behaviour id for id; these two are the correct ones, off by default (CLI: --bpe). */
int tffn_tokenizer_encode_bpe(const tffn_tokenizer* t, const char* text, uint32_t* ids, int cap);
int tffn_tokenizer_decode_bpe(const tffn_tokenizer* t, const uint32_t* ids, int n, char* out, int cap);
int tffn_tokenizer_token_id(const tffn_tokenizer* t, const char* token, uint32_t* id);
int tffn_tokenizer_special(const tffn_tokenizer* t, uint32_t* eos, uint32_t* bos, uint32_t* pad);

/* ---- model / expert -------------------------------------------------------------------- */
/* qwen_load minus the KV cache and scratch (inference/src/model/qwen.cu:80-132): reads
 * config.json and every *.safetensors of the directory, uploads the weights to `device`,
 * builds the layouts the kernels stream. tp_rank / tp_size = 0 / 1 loads the whole model; otherwise
 * this process is one rank of a tensor-parallel group and loads only its slices (tffn_tp_partition):
 * query / kv heads, the intermediate dimension of the FFN, rows of the LM head. Such a model needs
 * tffn_session_create_tp. */
int tffn_model_load(const char* model_dir, int device, int tp_rank, int tp_size, tffn_model** out);
void tffn_model_free(tffn_model* m); /* qwen_free (qwen.cu:176-209) */
int tffn_model_config(const tffn_model* m, tffn_config* out);
/* bytes of weight a decode step streams from HBM (every matrix once), with/without an expert */
uint64_t tffn_model_weight_bytes(const tffn_model* m, int with_expert);

/* expert_alloc + checkpoint_load + output_scale (inference/src/model/expert.cu:9-31,
 * inference/src/io/checkpoint.cpp:11-65, inference/src/main.cpp:109-119): fp32 file -> bf16 (RNE)
 * on the device. The shape must match the model. */
int tffn_expert_load(const tffn_model* m, const char* path, float scale, tffn_expert** out);
int tffn_expert_set_scale(tffn_expert* e, float scale); /* ExpertModel::output_scale */
/* expert_forward of the trainer (trainer/src/model/ffn_expert.cu:151-175) on the inference kernels, for
 * training-shaped batches: d_x_norm = DEVICE bf16 [num_layers][batch_tokens][hidden] (the normalised FFN
 * input of every layer), d_out_delta = DEVICE fp32 [num_layers][batch_tokens][hidden] =
 * scale * (bf16(silu(bf16(x Wg^T)) * bf16(x Wu^T)) Wd^T), scale = the expert's output scale (the trainer
 * uses kExpertOutputScale = 0.01: set it with tffn_expert_set_scale). Runs on `stream` (0: the default
 * stream) and returns when the result is complete. */
int tffn_expert_forward(const tffn_expert* e, const void* d_x_norm, float* d_out_delta, int batch_tokens, void* stream);
float tffn_expert_get_scale(const tffn_expert* e);
void tffn_expert_free(tffn_expert* e); /* expert_free (expert.cu:33-42) */

/* ---- session --------------------------------------------------------------------------- */
/* The KV cache + scratch part of qwen_load (qwen.cu:134-171), paged: max_batch sequence slots
 * of up to max_seq tokens each. expert may be NULL (base model only). cuda_stream: a
 * cudaStream_t, or NULL for a stream the session creates. */
int tffn_session_create(const tffn_model* m, const tffn_expert* expert, int max_batch, int max_seq, void* cuda_stream,
                        tffn_session** out);
void tffn_session_free(tffn_session* s);

/* ---- tensor parallelism (the reference is single-GPU: no counterpart) -------------------- */
/* One process per GPU. Rank 0 makes an id (tffn_tp_unique_id, 128 bytes) and hands it to the other
 * ranks by any means; every rank then calls tffn_tp_create (collective: returns when all tp_size
 * ranks have joined), loads its slice with tffn_model_load(dir, device, tp_rank, tp_size) /
 * tffn_expert_load, and creates its session with tffn_session_create_tp. All ranks then make the
 * same tffn_prefill / tffn_decode_step / tffn_decode_run calls with the same arguments; each returns
 * the same tokens (and full logits) on every rank. Inside a step the ranks' partial sums of o_proj
 * and of the down projections (base + scale * expert, summed locally first) are summed over the ranks in
 * fp32 before the one bf16 rounding of the residual add, and the greedy pick exchanges one (max, index)
 * pair per sequence and rank. Launches of up to 128 tokens (decode) exchange the partial sums through peer
 * memory over NVLink: every rank exports an exchange window (CUDA IPC, so the ranks must be processes on one
 * machine whose GPUs have peer access), the projections leave their fp32 partial sums in their own rank's
 * window, and the row kernel that adds the residual and forms the next RMSNorm first hand-shakes with its
 * peers through flags in those windows (bounded wait: a peer that never arrives gives TFFN_ERR_DEVICE
 * status after 10 s, not a hang), then loads every rank's part over NVLink and adds them in rank order; the
 * greedy pick exchanges its candidates the same way. The only stores that cross GPUs are the flags. Larger
 * launches (prefill) use ncclAllReduce. Creating and freeing a tensor-parallel session are collective calls.
 * Sampling and tffn_expert_forward are not available on a tensor-parallel model. NCCL (libnccl.so.2) is
 * opened at run time. */
typedef struct tffn_tp tffn_tp;
int tffn_tp_unique_id(uint8_t* id128);
int tffn_tp_create(const uint8_t* id128, int tp_rank, int tp_size, int device, tffn_tp** out);
void tffn_tp_free(tffn_tp* tp); /* after every session created with it has been freed */
/* Host-only: what rank tp_rank of tp_size owns of a model with this config (only the dimensions of cfg
 * are read): out8 = {first query head, query heads, first kv head, kv heads, first intermediate row,
 * intermediate rows, first LM-head row, LM-head rows}. With more ranks than kv heads, tp_size / kv_heads
 * ranks share a kv head and split its query heads (7 heads over 2 ranks: 3 + 4). */
int tffn_tp_partition(const tffn_config* cfg, int tp_rank, int tp_size, int32_t* out8);
int tffn_session_create_tp(const tffn_model* m, const tffn_expert* expert, int max_batch, int max_seq, void* cuda_stream,
                           tffn_tp* tp, tffn_session** out);
/* on = 0: every all-reduce of this session through NCCL, also the decode-sized ones (all ranks must choose
 * alike); default 1 */
int tffn_session_set_tp_fused(tffn_session* s, int on);
/* qwen_reset (qwen.cu:174) for one slot, or for all with slot = -1: frees the slot's pages. */
int tffn_session_reset(tffn_session* s, int slot);
int tffn_session_seq_len(const tffn_session* s, int slot); /* KVCache::len */
/* 0: plain stream launches. 1: programmatic dependent launch between the batch-1 kernels.
 * 2: 1 + every decode step (batch-1 and batched) replayed from a CUDA graph. Default 1. */
int tffn_session_set_launch_mode(tffn_session* s, int mode);
/* Temperature sampling on the device (the reference samples on the host from a 608 KB logits row per
 * token: sample(), inference/src/main.cpp:52-63). temperature <= 0 restores greedy picks. Otherwise every
 * pick of tffn_prefill / tffn_decode_step / tffn_decode_run is drawn as sample() draws it (float maximum,
 * exp((logit - max) / temperature) in float, sums in double, first index whose running sum reaches
 * r = u * sum), with u from std::uniform_real_distribution<double> over a std::mt19937(seed) that the
 * session owns (the reference's CLI seeds 42): one draw per sampled token, the sequences of a batched
 * step in slot order, the steps of tffn_decode_run in step order. Sampled single-sequence steps run on
 * the batched path. tffn_forward keeps leaving the greedy token. */
int tffn_session_set_sampling(tffn_session* s, float temperature, uint32_t seed);
/* Which path single-token steps take: 1 (default) the fused batch-1 kernels when the shape
 * allows, 0 the batched tensor-core path. */
int tffn_session_set_bs1_path(tffn_session* s, int enable);
/* Keep a copy of the residual stream after every layer of the next tffn_prefill / tffn_forward
 * (up to max_rows token rows); read it with tffn_session_get_hidden. 0 rows = off. */
int tffn_session_capture_hidden(tffn_session* s, int max_rows);
/* dst: bf16 bits [rows, hidden] of layer `layer` from the last captured call; returns rows. */
int tffn_session_get_hidden(tffn_session* s, int layer, uint16_t* dst, int max_rows);

/* qwen_forward for a prompt (inference/src/main.cpp:172-180): appends seq_lens[i] tokens to
 * slot i for i < n_seqs (tokens concatenated in slot order), returns the greedy pick after
 * each prompt's last token in next_tokens[n_seqs] and, if logits_last != NULL, that row's
 * fp32 logits in logits_last[n_seqs, vocab]. */
int tffn_prefill(tffn_session* s, const int32_t* tokens, const int32_t* seq_lens, int n_seqs, int32_t* next_tokens,
                 float* logits_last);
/* qwen_forward with all-row logits, one slot: appends T tokens to `slot` and writes fp32
 * logits[T, vocab] (what the reference's d_logits holds after a call, qwen.cu:450-454). */
int tffn_forward(tffn_session* s, int slot, const int32_t* tokens, int T, float* logits);
/* One step of the decode loop (inference/src/main.cpp:183-197) for slots 0..n_seqs-1:
 * feeds tokens_in[i] (or, if NULL, the slot's previous greedy pick), appends it to the cache,
 * returns the greedy pick in next_tokens[i] and optionally fp32 logits[n_seqs, vocab]. */
int tffn_decode_step(tffn_session* s, const int32_t* tokens_in, int n_seqs, int32_t* next_tokens, float* logits);
/* `steps` greedy steps back to back with no host round trip (each step feeds the previous
 * pick); tokens_out[steps, n_seqs] (host) may be NULL. Asynchronous part ends before return. */
int tffn_decode_run(tffn_session* s, int n_seqs, int steps, int32_t* tokens_out);
/* Device status word (0 = none) and kernel launches issued by the session so far. */
int tffn_session_status(tffn_session* s);
uint64_t tffn_session_launch_count(const tffn_session* s);
/* the stream the session launches on (a cudaStream_t) */
void* tffn_session_stream(const tffn_session* s);

/* ---- kernel-level entry points used by the tests ---------------------------------------- */
/* out[T,N] = X[T,K] * W[N,K]^T on the tensor-core GEMM of the batched path (bf16 bits in,
 * fp32 out, host pointers); splits = 0 lets the launcher choose the K split.
 * Stands in for gemm_bf16 (inference/src/backend/cuda_ops.cu:18-29). */
int tffn_op_gemm(int device, const uint16_t* X, const uint16_t* W, float* out, int T, int N, int K, int splits);
/* The fused batch-1 SwiGLU kernel alone (host pointers, bf16 bits): h_out = bf16(h + FFN(rmsnorm(h)))
 * with FFN = base + expert_scale * expert (packed_expert may be NULL). packed_* use the record
 * layout [I][3][H] = gate row, up row, down column per intermediate index. Stands in for the FFN
 * part of qwen_forward (inference/src/model/qwen.cu:422-447) and expert_forward_layer
 * (inference/src/model/expert.cu:44-59) at T = 1. */
int tffn_op_swiglu_bs1(int device, const uint16_t* h_in, const uint16_t* norm_w, const uint16_t* packed_base,
                       const uint16_t* packed_expert, float expert_scale, float eps, int H, int I, uint16_t* h_out);
/* tffn_op_swiglu_bs1 for callers that must not allocate device memory (no counterpart in the
 * reference, whose every buffer comes from cudaMalloc): a host thread in a latency-critical loop
 * that may not take the allocator's lock or cause a device-wide implicit synchronisation, a plugin
 * inside a process whose device memory is owned and reserved by someone else, a deployment with a
 * memory budget fixed at start-up. All pointers are DEVICE pointers supplied by the caller, each
 * 16-byte aligned (TFFN_ERR_INVALID otherwise); h_io is updated in place. The kernel's scratch is a
 * fixed array inside the library (about 33 KB per GPU that loads it), so hidden <= 2048 (a multiple of
 * 64); larger requests return TFFN_ERR_CAPACITY. The function calls no cudaMalloc / cudaFree; it
 * clears the part of the scratch that must start at zero, launches on `cuda_stream`, and BLOCKS until
 * that stream has finished the call (it synchronises only that stream, nothing device-wide), so it
 * must not be called while the stream is being captured. Calls that could overlap on one GPU share
 * the scratch and must be serialised by the caller. The first call on a device also looks up the
 * array's device address. The calling thread's current device is left as it was. */
int tffn_op_swiglu_bs1_noalloc(int device, void* h_io, const void* norm_w, const void* packed_base,
                               const void* packed_expert, float expert_scale, float eps, int H, int I, void* cuda_stream);
/* Runs a kernel that waits on a barrier nothing signals; returns the device status it
 * recorded (expected: 5). Proves that a wait that runs out returns instead of hanging. */
int tffn_op_wait_selftest(int device);
/* The same for the tensor-parallel hand-shake: one GPU plays rank 0 of a group of two whose peer never
 * signals; the kernel gives up after wait_ms (1..2000) and the recorded status is returned (expected: 7). */
int tffn_op_tp_wait_selftest(int device, int wait_ms);

#ifdef __cplusplus
}
#endif
#endif
