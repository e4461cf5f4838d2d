// Host-side engine: weights on the device (Model, Expert) and the per-session state
// (paged KV cache, block tables, scratch, decode loop). C++ mirror of the reference's
// model:: namespace (inference/include/model/qwen.h, expert.h), behind the C ABI in c_api.cpp.
#pragma once
#include "host_io.h"
#include "kernels.h"
#include <cstdint>
#include <map>
#include <string>
#include <random>
#include <vector>

namespace tffn {

void cuda_check(cudaError_t e, const char* what, const char* file, int line);
#define TFFN_CUDA(x) ::tffn::cuda_check((x), #x, __FILE__, __LINE__)

struct DeviceBuffer {
    void* p = nullptr;
    size_t bytes = 0;
    bool owned = true;  // false: a view into a slab that somebody else frees
    DeviceBuffer() = default;
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    DeviceBuffer(DeviceBuffer&& o) noexcept : p(o.p), bytes(o.bytes), owned(o.owned) { o.p = nullptr; o.bytes = 0; }
    ~DeviceBuffer() { release(); }
    void alloc(size_t n);  // zero-filled
    void alloc_raw(size_t n);  // not filled: for buffers that are overwritten whole before anything reads them
    void view(void* ptr, size_t n) { release(); p = ptr; bytes = n; owned = false; }
    void release();
    template <typename T>
    T* as() const { return (T*)p; }
};

// One FFN (base or expert) of one layer: records [I][3][H] (gate row, up row, down column) for
// the batch-1 kernel and, as strided views of the same records, for the tensor-core GEMM;
// plus down as [H, I] for the GEMM's K-major operand.
struct FfnWeights {
    DeviceBuffer packed;  // bf16 [I][3][H]
    DeviceBuffer down;    // bf16 [H][I]
};

struct LayerWeights {
    DeviceBuffer wqkv, bqkv, wo, attn_norm, ffn_norm;
    bool has_bias = false;
    FfnWeights ffn;
};

// NCCL communicator of a tensor-parallel group (the library is opened at run time; see tp_comm.cpp)
struct TpComm;
TpComm* tp_comm_create(const uint8_t id[128], int rank, int size, int device);
void tp_comm_unique_id(uint8_t id[128]);
void tp_comm_free(TpComm* c);
int tp_comm_size(const TpComm* c);
int tp_comm_rank(const TpComm* c);
void tp_all_reduce_f32(TpComm* c, float* buf, size_t n, cudaStream_t s);                 // in place, sum
void tp_all_gather_bytes(TpComm* c, const void* send, void* recv, size_t bytes, cudaStream_t s);  // recv[rank * bytes ...]
// peer-mapped exchange windows (collective calls; see tp_comm.cpp): peers[] has 8 entries
void tp_window_open(TpComm* c, void* local, void* peers[], cudaStream_t s);
bool tp_window_close(TpComm* c, void* peers[], cudaStream_t s, double timeout_s);

struct Model {
    Config cfg;         // the whole model, as config.json states it
    TpPartition tp;     // this rank's slices (everything when tp_size == 1)
    // this rank's sizes: query heads, kv heads, intermediate rows, LM-head rows
    int nh = 0, nkv = 0, I = 0, V = 0;
    int device = 0, num_sms = 0;
    DeviceBuffer slab;  // the one allocation every weight below is a view of
    DeviceBuffer embed, final_norm, lm_head_own;
    const bf16* lm_head = nullptr;
    std::vector<LayerWeights> layers;
    bool bs1_ok = false;
    uint64_t weight_bytes_base = 0;  // bytes one decode step streams (every matrix once, LM head included)
    static Model* load(const std::string& dir, int device, int tp_rank, int tp_size);
};

struct Expert {
    const Model* model = nullptr;
    float scale = 0.1f;
    DeviceBuffer slab;  // the one allocation the layers' buffers are views of
    std::vector<FfnWeights> layers;
    uint64_t weight_bytes = 0;
    static Expert* load(const Model* m, const std::string& path, float scale);
    // The trainer's expert_forward (trainer/src/model/ffn_expert.cu:151-175) on the inference kernels:
    // d_x device bf16 [layers][T][hidden] (the normalised FFN inputs of every layer), d_out device fp32
    // [layers][T][hidden] = scale * down(silu(gate x) * up x), scale = this expert's output scale.
    void forward_layers(const void* d_x, float* d_out, int T, cudaStream_t stream) const;
};

// kernel classes of the per-launch profile (tffn_session_profile_*)
enum KClass : int {
    KC_EMBED = 0, KC_RMSNORM, KC_GEMM_QKV, KC_ATTENTION, KC_GEMM_OPROJ, KC_GEMM_GATEUP, KC_GEMM_DOWN,
    KC_GEMM_LMHEAD, KC_ARGMAX, KC_ADVANCE, KC_BS1_QKV, KC_BS1_OPROJ, KC_BS1_FFN, KC_BS1_LMHEAD, KC_ALLREDUCE, KC_COUNT
};
const char* kclass_name(int c);

class Session {
public:
    // Runs three batched decode steps of n_seqs slots (the sequences advance) and reports the last one:
    // per kernel launch 7 u64 = class, then min / max over its CTAs of entry, grid-wait return and exit
    // (globaltimer ns). Returns the number of launches. If launch number trace_launch is a tensor-core
    // GEMM, its per-CTA phase timestamps (64 u64 per CTA, see GemmCall::trace; the grid must not exceed
    // trace_ctas CTAs) are returned in trace_out.
    int timeline(int n_seqs, uint64_t* out, int max_launches, int trace_launch = -1, uint64_t* trace_out = nullptr,
                 int trace_ctas = 0);
    void set_profile(bool on);
    // accumulated device time (ms) and launches per class since set_profile(true); returns KC_COUNT
    int read_profile(float* ms, int* counts, int cap);
    Session(const Model* m, const Expert* e, int max_batch, int max_seq, cudaStream_t stream, TpComm* tp = nullptr);
    ~Session();
    void reset(int slot);
    int seq_len(int slot) const { return h_seq_len_[slot]; }
    void prefill(const int32_t* tokens, const int32_t* seq_lens, int n_seqs, int32_t* next_tokens, float* logits_last);
    void forward(int slot, const int32_t* tokens, int T, float* logits);
    void decode_step(const int32_t* tokens_in, int n_seqs, int32_t* next_tokens, float* logits);
    void decode_run(int n_seqs, int steps, int32_t* tokens_out);
    void set_launch_mode(int mode);
    // timing-only: kernel classes (bit = KClass) that the batched path does not launch
    void set_ablation(unsigned mask);
    void set_bs1_path(bool on) { use_bs1_ = on; }
    // tensor parallel: false = every all-reduce through NCCL (all ranks must choose alike)
    void set_tp_fused(bool on);
    // temperature <= 0: greedy. Otherwise every pick is sampled on the device as sample() of the
    // reference does on the host, with draws from a std::mt19937(seed) owned by the session.
    void set_sampling(float temperature, uint32_t seed);
    void capture_hidden(int max_rows);
    int get_hidden(int layer, uint16_t* dst, int max_rows);
    int status();
    uint64_t launch_count() const { return launches_; }
    cudaStream_t stream() const { return stream_; }
    const Model* model() const { return m_; }

private:
    const Model* m_;
    const Expert* e_;
    TpComm* tp_ = nullptr;  // not owned
    DeviceBuffer delta_, tp_pick_send_, tp_pick_recv_, tp_logits_;  // tensor parallel: fp32 partial sums, pick exchange, gathered logits
    // Tensor parallel, launches of at most tp_small_rows_ rows (decode): the projections leave their partial
    // sums in this rank's exchange window, which the peers have mapped, and a row kernel on every rank reads
    // all ranks' parts over NVLink after a flag hand-shake (k_tp_reduce_residual_norm); larger launches
    // (prefill) go through NCCL. Window = flags, pick candidates, then two alternating buffers (o_proj / down)
    // of [tp_small_rows_][H] fp32.
    DeviceBuffer tp_win_, tp_calls_;
    void* tp_peers_[kTpMaxRanks] = {};
    int tp_small_rows_ = 0;
    size_t tp_part_off_[2] = {0, 0};  // in floats, from the window's start
    TpParts tp_parts_[2];
    TpPeerSync tp_sync_, tp_pick_sync_;
    TpPickParts tp_pick_parts_;
    size_t tp_pick_off_ = 0;  // in bytes: [tp_small_rows_] candidates of 8 bytes
    bool tp_fused_ = true;
    void copy_logits_to_host(float* dst, size_t rows);  // rows of logits_ (this rank's vocabulary slice) -> full rows on the host
    int max_batch_, max_seq_, max_pages_per_seq_, num_pages_;
    int cap_tokens_;  // rows of the activation buffers
    cudaStream_t stream_;
    bool own_stream_ = false;
    int launch_mode_ = 1;
    unsigned ablate_mask_ = 0;
    float sample_temp_ = 0.f;
    std::mt19937 sample_rng_{42};
    DeviceBuffer sample_u_;
    double* h_sample_u_ = nullptr;  // pinned staging
    size_t h_sample_cap_ = 0;
    void upload_draws(size_t n);  // n canonical draws -> sample_u_[0..n)
    bool sampling() const { return sample_temp_ > 0.f; }
    bool store_logits_ = true;  // whether the LM head writes its fp32 logits (the greedy pick does not need them)
    bool tl_on_ = false;
    DeviceBuffer tl_buf_;
    std::vector<int> tl_cls_;
    int tl_trace_launch_ = -1;
    DeviceBuffer tl_trace_buf_;
    unsigned long long* tl_next(int cls);
    bool use_bs1_ = true;
    uint64_t launches_ = 0;

    // paged KV cache
    DeviceBuffer k_pool_, v_pool_, block_table_, seq_len_dev_;
    std::vector<int> h_block_table_, h_seq_len_, free_pages_;
    std::vector<int> h_pages_used_;  // pages mapped per slot
    bool table_dirty_ = false;
    KvView kv_;

    // RoPE tables [max_seq, hd/2] (inference/src/model/qwen.cu:120-132)
    DeviceBuffer rope_cos_, rope_sin_;

    // token metadata and activations of the batched path
    DeviceBuffer tokens_, tok_seq_, tok_pos_, row_idx_, picks_, identity_, dec_tokens_;
    DeviceBuffer grp_first_, grp_count_;  // prefill attention: groups of up to 8 consecutive rows of one sequence
    DeviceBuffer h_, xn_, q_, ctx_, act_b_, act_e_, xn_last_, logits_;
    size_t logits_rows_ = 0;
    DeviceBuffer attn_partials_, attn_counters_;
    DeviceBuffer status_, out_ring_, step_counter_;
    int out_ring_cap_ = 0;
    int* h_status_ = nullptr;  // pinned
    int32_t* h_pinned_i32_ = nullptr;
    size_t h_pinned_cap_ = 0;

    // batch-1 path
    DeviceBuffer bs1_h_, bs1_acc_, bs1_q_, bs1_ctx_, bs1_tickets_, bs1_lm_val_, bs1_lm_idx_;
    cudaGraphExec_t bs1_graph_ = nullptr;
    bool bs1_graph_logits_ = false;
    // batched decode steps captured per (sequences, attention splits)
    struct DecGraph { cudaGraphExec_t exec; uint64_t launches; };
    std::map<std::pair<int, int>, DecGraph> dec_graphs_;
    void run_decode_batched(int n_seqs, int max_ctx);
    void drop_graphs();

    // per-launch profile: event pairs around every kernel, resolved in read_profile
    bool profile_ = false;
    struct ProfRec { int cls; cudaEvent_t a, b; };
    std::vector<ProfRec> prof_recs_;
    std::vector<cudaEvent_t> prof_free_;
    float prof_ms_[KC_COUNT] = {0};
    int prof_n_[KC_COUNT] = {0};
    void prof_begin(int cls);
    void prof_end();
    void prof_resolve();

    // hidden-state capture
    DeviceBuffer hidden_;
    int hidden_rows_cap_ = 0, hidden_rows_ = 0;

    GemmWorkspace gemm_ws() const;
    TmapCache* tmaps_ = tmap_cache_create();  // encoded tensor maps of this session's GEMM launches
    AttnWorkspace attn_ws() const;
    void ensure_pages(int slot, int new_len);
    void flush_tables();
    void ensure_logits(size_t rows);
    void ensure_ring(int entries);
    // runs T tokens already staged in tokens_/tok_seq_/tok_pos_ (or decode state when decode=true)
    void run_batched(int T, int n_logit_rows, bool logit_rows_are_all, bool decode, int max_ctx, int n_groups = 0);
    // groups for launch_attention_prefill from the rows' (slot, position) lists; fills pin[0..2*n) and returns n
    static int build_groups(const int* seq, const int* pos, int T, int32_t* first, int32_t* count);
    void run_bs1(bool want_logits);
    void launch_bs1_step(bool want_logits, bool pdl);
    Bs1Ctx bs1_ctx(bool want_logits) const;
    void check_status();
    int32_t* pinned_i32(size_t n);
};

}  // namespace tffn
