// Launchers of the device kernels. Host code (model.cu / session.cu) calls only these.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace tffn {

typedef __nv_bfloat16 bf16;

constexpr int kPageTokens = 32;  // tokens per KV page

// ------------------------------------------------------------------ paged KV cache view
struct KvView {
    bf16* k_pool;            // [L][pages][nkv][kPageTokens][hd]
    bf16* v_pool;
    const int* block_table;  // [max_batch][max_pages_per_seq]
    int max_pages_per_seq;
    int num_pages;           // pages per layer
    size_t layer_stride;     // elements between layers of a pool
    int nkv, hd;
};

// ------------------------------------------------------------------ tensor-core GEMM (batched path)
// out[t, n] = epilogue( sum_k X0[t,k] W0[n,k] , sum_k X1[t,k] W1[n,k] )
enum GemmMode : int {
    GEMM_STORE_F32 = 0,   // out fp32  = a0 (+ alpha * a1)
    GEMM_STORE_BF16 = 1,  // out bf16  = bf16(a0 (+ alpha * a1))
    GEMM_RESIDUAL = 2,    // out bf16 += a0 (+ alpha * a1), i.e. out = bf16(float(out) + sum)
    GEMM_SWIGLU = 3,      // out bf16  = bf16(silu(bf16(a0)) * bf16(a1))   (a0 gate rows, a1 up rows)
    GEMM_QKV = 4,         // q|k|v rows: bias + RoPE + page writes in the epilogue (GemmCall::qkv), no `out`
};
struct GemmQkvEpilogue {
    const bf16* bias;               // [(nh+2nkv)*hd] or null
    const float *rope_cos, *rope_sin;
    const int *tok_seq, *tok_pos;   // per token: sequence slot and position
    float* q_out;                   // fp32 [T, nh*hd]
    KvView kv;
    int layer, nh, max_pos;
};
struct GemmOperand {
    const bf16* W;  // [N, K] row-major, row stride ldw elements
    int64_t ldw;
    const bf16* X;  // [T, K] row-major, row stride ldx elements
    int64_t ldx;
    int K;          // 0 = operand unused
};
constexpr int kTpMaxRanks = 8;  // ranks of a tensor-parallel group

struct GemmCall {
    GemmOperand op[2];
    int N, T;
    int mode;
    float alpha;
    void* out;
    int64_t ldo;
    int x_rows_alloc;  // rows that exist in the X buffers (>= T); the tensor map covers them
    // optional second, independent problem of the same shape in the same launch (e.g. the expert's
    // gate/up next to the base's): its operands and its output; out2 == nullptr means none
    GemmOperand op2[2];
    void* out2;
    float out_scale;  // GEMM_STORE_F32: the stored value is out_scale * sum (0 means 1)
    const GemmQkvEpilogue* qkv;  // GEMM_QKV only
    // GEMM_STORE_F32 only, optional: greedy pick fused into the epilogue. Every CTA leaves, per token, the
    // maximum of its 128 output rows and its index (lowest index among equal maxima) in
    // amax_val / amax_idx [t * ceil(N / 128) + tile]; launch_argmax_tiles combines them. With it `out` may
    // be nullptr: the values themselves are then not stored.
    float* amax_val;
    int* amax_idx;
    // optional device buffer of 64 u64 per CTA: globaltimer (ns) at 0 start, 1 weight boxes requested,
    // 2 dependency wait over, 3 last MMA issued, 4 accumulator complete, 5 epilogue/park done,
    // 6 cluster barrier passed, 7 reduction done, 8 end, 16+i stage i arrived (i < 40)
    unsigned long long* trace;
    int trace_ctas;          // CTAs the trace buffer holds; a larger grid is not traced
    unsigned long long* tl;  // optional 6 u64 of the step timeline (see tl_mark)
    bool pdl;          // launch with programmatic dependent launch (the kernel waits before touching X / out)
};
// Encoded tensor maps of the (buffer, shape, box) combinations a caller keeps launching with: encoding one costs
// microseconds of host time and a decode step needs about 200. Owned by whoever owns the buffers (a session keeps
// one for its lifetime), so entries die with the buffers they describe.
struct TmapCache;
TmapCache* tmap_cache_create();
void tmap_cache_free(TmapCache* c);

struct GemmWorkspace {
    int* status;  // device status word
    int num_sms;
    TmapCache* tmaps = nullptr;  // optional; without it every launch encodes its maps
};
// opt the kernels into their dynamic shared memory sizes (once per device, outside stream capture)
int gemm_prepare();
// returns cudaError (launch) or -1000 if the tensor maps could not be encoded
int launch_gemm(const GemmCall& c, const GemmWorkspace& ws, cudaStream_t stream, int force_splits = 0);

// ------------------------------------------------------------------ row kernels of the batched path
// (pdl: launch with programmatic dependent launch; every kernel here waits before reading its inputs)
// tl: optional 6 u64 of the step timeline (see tl_mark): min / max over the CTAs of entry, grid-wait return, exit
// the row kernels share the step's shared-memory carveout with the large kernels (see prefer_max_shared)
int rows_prepare();
void launch_embed(const int* tokens, const bf16* table, bf16* h, int T, int H, int V, int* status, cudaStream_t s,
                  bool pdl = false, unsigned long long* tl = nullptr);
void launch_rmsnorm(const bf16* x, const bf16* w, bf16* out, int T, int H, float eps, const int* row_idx, cudaStream_t s,
                    bool pdl = false, unsigned long long* tl = nullptr);
// temperature sampling (inference/src/main.cpp:52-63) of R rows of fp32 logits on the device;
// u[step * R + row] = canonical uniform draws in [0, 1), step = *step_counter (0 if nullptr)
void launch_sample(const float* logits, int R, int V, float temperature, const double* u, const int* step_counter, int* out,
                   cudaStream_t s, bool pdl = false, unsigned long long* tl = nullptr);
// Tensor parallel over peer memory (decode-sized launches). Every rank owns an exchange window that the
// other ranks of the group have mapped; kTpFlagBlocks = the largest grid of a kernel that hand-shakes. Block b
// waits for block b of every peer, so all blocks of such a grid have to be resident at once on every rank
// whatever order the hardware starts them in: 128 blocks of 1 024 threads fit the 148 SMs of a B200.
constexpr int kTpFlagBlocks = 128;
struct TpPeerSync {
    unsigned* flags_local;              // this rank's window: [size][kTpFlagBlocks] counters, written by the peers
    unsigned* flags_peer[kTpMaxRanks];  // the same array inside every peer's window
    unsigned* calls;                    // this rank only: [kTpFlagBlocks] calls made so far, per block
    int rank, size;
    unsigned long long wait_ns;         // how long a block waits for its peers before it gives up
};
// the ranks' pick candidates: part[p] = rank p's {maximum, global index} per row as mapped into this process
struct TpPickParts {
    const float2* part[kTpMaxRanks];
};
// per-tile maxima left by the GEMM (GemmCall::amax_val / amax_idx, `tiles` per row) -> argmax per row
// pack (optional, 8 bytes per row): {the row's maximum, idx_offset + its index} for the exchange between
// tensor-parallel ranks, which launch_tp_pick resolves (cand = `ranks` such arrays of R rows back to back)
void launch_argmax_tiles(const float* amax_val, const int* amax_idx, int R, int tiles, int* out, cudaStream_t s,
                         bool pdl = false, unsigned long long* tl = nullptr, void* pack = nullptr, int idx_offset = 0);
// the ranks' partial sums of one exchange: part[p] = rank p's fp32 [rows][H] buffer as mapped into this process
struct TpParts {
    const float* part[kTpMaxRanks];
};
// h += sum over ranks p (in rank order) of part[p][row * H ...], then out = RMSNorm(h) * w (w == nullptr: no
// norm). T <= kTpFlagBlocks rows, H a multiple of 4.
void launch_tp_reduce_residual_norm(bf16* h, const TpParts& parts, const TpPeerSync& sync, const bf16* w, bf16* out, int T, int H,
                                    float eps, int* status, cudaStream_t s, bool pdl = false, unsigned long long* tl = nullptr);
// launch_tp_pick over the candidates every rank left in its own window (launch_argmax_tiles' pack), loaded over
// NVLink after a hand-shake with the peers; R <= 128 * kTpFlagBlocks rows
void launch_tp_pick_peer(const TpPickParts& parts, const TpPeerSync& sync, int R, int* out, int* status, cudaStream_t s,
                         bool pdl = false);
void launch_tp_pick(const void* cand, int ranks, int R, int* out, cudaStream_t s, bool pdl = false);
// tensor parallel: h = bf16(h + delta) and, if w != null, out = rmsnorm(h) * w, per row
void launch_residual_norm(bf16* h, const float* delta, const bf16* w, bf16* out, int T, int H, float eps, cudaStream_t s,
                          bool pdl = false);
// logits fp32 [R, V] -> argmax (lowest index among maxima). scratch (>= 2 * R * 64 floats) and
// counters (>= R ints, zero, left zero) let several blocks share a row; without them one block per row.
void launch_argmax(const float* logits, int R, int V, int* out, float* scratch, size_t scratch_floats, int* counters,
                   int num_counters, int num_sms, cudaStream_t s, bool pdl = false, unsigned long long* tl = nullptr);

// ------------------------------------------------------------------ attention over the paged cache
struct AttnWorkspace {
    float* partials;  // [T*nkv][splits][G*(hd+2)]
    size_t partial_floats;
    int* counters;    // [T*nkv]
    int num_counters;
};
// opt the attention kernels into their dynamic shared memory (once per device, outside stream capture)
int attn_prepare();
// context splits launch_attention will use (a CUDA-graph key: the grid depends on it)
int attention_splits(int T, int nh, int nkv, int hd, int max_ctx, const AttnWorkspace& ws, int num_sms);
// one query token per (t): context = tok_pos[t] + 1 cached tokens of sequence tok_seq[t].
// only_newest_row_fresh (decode): of everything the kernel reads, only q and the cached row at
// tok_pos[t] were written since the last kernel of the stream that was launched WITHOUT programmatic
// dependent launch; the rest may then be fetched before the previous kernel has finished.
void launch_attention(const float* q, KvView kv, int layer, const int* tok_seq, const int* tok_pos, bf16* ctx, int T,
                      int nh, int max_ctx, AttnWorkspace ws, int num_sms, int* status, cudaStream_t s, bool pdl = false,
                      bool only_newest_row_fresh = false, unsigned long long* tl = nullptr,
                      unsigned long long* trace = nullptr, int trace_ctas = 0);  // trace: 16 u64 per CTA, see attn.cu

// Prompt tokens: rows grp_first[g] .. grp_first[g] + grp_count[g] - 1 (at most 8, consecutive positions of
// one sequence) share one pass over that sequence's cache; n_groups groups cover the T rows of the call.
void launch_attention_prefill(const float* q, KvView kv, int layer, const int* tok_seq, const int* tok_pos, const int* grp_first,
                              const int* grp_count, int n_groups, bf16* ctx, int nh, int* status, cudaStream_t s,
                              bool pdl = false, unsigned long long* tl = nullptr);

// ------------------------------------------------------------------ batch-1 fused decode kernels
struct Bs1Layer {
    const bf16 *wqkv, *bqkv;  // [(nh+2nkv)*hd, H] rows q|k|v ; bias or null
    const bf16 *wo;           // [H, nh*hd]
    const bf16 *attn_norm, *ffn_norm;
    const bf16 *ffn_base;     // [I][3][H]: gate row, up row, down column (= row of down^T) per intermediate index
    const bf16 *ffn_expert;   // same layout or null
};
struct Bs1Ctx {
    int H, I, nh, nkv, hd, V;
    float eps, expert_scale;
    const float *rope_cos, *rope_sin;
    int max_pos;
    bf16* h;          // [H] residual stream of this layer: published by the q|k|v kernel, updated by o_proj, read by the FFN
    const bf16* h_in; // [H] residual stream the q|k|v kernel (or the LM head) starts from: the previous layer's `h`
    // The FFN leaves its output as fixed-point sums (see bs1_acc_words): acc_out is where this layer's FFN
    // adds, acc_in what the previous layer's FFN left (null: nothing to fold in). The consumer of the
    // residual stream forms h = bf16(h_in + acc_in) itself; the q|k|v kernel also clears acc_out.
    const long long* acc_in;
    long long* acc_out;
    float* q;         // [nh*hd]
    bf16* ctx;        // [nh*hd]
    int* token;       // device: current input token (slot 0)
    int* seq_len;     // device: cached tokens of the slot = position of the new token
    int slot;
    int* tickets;     // zeroed tickets (LM head)
    float* lm_val;    // [lm_grid] candidates
    int* lm_idx;
    float* logits;    // optional fp32 [V] or null
    int* out_tokens;  // device ring of picks, or null
    int* step_counter;
    int* status;
    int num_sms;
    // optional profiling aid for k_bs1_ffn: 16 u64 per CTA, globaltimer ns at 0 start, 1 rmsnorm done,
    // 2 first record arrived, 3 last record consumed, 4 this CTA's sums added to acc_out
    unsigned long long* trace;
    unsigned long long* tl;  // optional 6 u64 of the step timeline for this launch (see tl_mark)
};
bool bs1_supported(int H, int I, int hd, int nh, int nkv);
// 64-bit words of one FFN accumulator: a few replicas (CTAs spread over them to thin out same-address
// atomics) of H fixed-point sums, value * 2^32 as int64. Integer addition is associative, so the sum of
// the CTAs' contributions does not depend on the order in which the atomics land: results stay
// bit-reproducible although no CTA waits for another.
size_t bs1_acc_words(int H);
// h[i] = bf16(h[i] + acc[i]) and acc cleared: closes a stand-alone launch_bs1_ffn (inside a decode step
// the next kernel folds the sums in instead)
void launch_bs1_ffn_finalize(bf16* h, long long* acc, int H, cudaStream_t s);
int bs1_prepare(int H, bool expert);  // dynamic shared memory opt-in for this shape (outside stream capture)
void launch_bs1_qkv(const Bs1Ctx& c, const Bs1Layer& ly, const bf16* embed, KvView kv, int layer, bool first, cudaStream_t s,
                    bool pdl);
void launch_bs1_oproj(const Bs1Ctx& c, const Bs1Layer& ly, cudaStream_t s, bool pdl);
void launch_bs1_ffn(const Bs1Ctx& c, const Bs1Layer& ly, cudaStream_t s, bool pdl);
void launch_bs1_lmhead(const Bs1Ctx& c, const bf16* final_norm, const bf16* lm_head, cudaStream_t s, bool pdl);

// fp32 -> bf16 (RNE) on device, used by the expert loader (inference/src/io/checkpoint.cpp:33-62)
void launch_cast_f32_bf16(const float* src, bf16* dst, size_t n, cudaStream_t s);
// pack gate/up/down^T rows into the [I][3][H] record layout of the batch-1 FFN kernel
void launch_pack_ffn(const bf16* gate, const bf16* up, const bf16* down, bf16* packed, int I, int H, cudaStream_t s);

// a kernel whose only job is to wait on an mbarrier nothing signals, for the bounded-wait test
void launch_wait_selftest(int* status, cudaStream_t s);

}  // namespace tffn
