// Batch-1 decode as ONE persistent kernel per token (launch mode 3).
//
// The four-kernels-per-layer path (decode_bs1.cu) spends most of a token in kernel boundaries:
// each of its ~100 launches is a latency chain (launch, dependent loads, ticket merges) during which
// HBM idles. Here one CTA per SM stays resident for the whole token:
//   * a producer thread walks the CTA's share of EVERY weight of the step in consumption order
//     (q|k|v row pairs, o_proj rows, base+expert FFN records, finally LM-head rows) and streams it
//     with cp.async.bulk into one shared-memory ring; it never waits for the math, only for a free
//     stage, so the weight stream runs ahead across phase boundaries;
//   * eight consumer warps run the phases of every layer — QKV+bias+RoPE+page write, split-KV
//     attention, o_proj+residual, fused base+expert SwiGLU, partial-sum fold — separated by grid
//     barriers (one atomic + a BOUNDED spin; on time-out a status code is set and every CTA leaves);
//   * the arithmetic and its rounding points are those of decode_bs1.cu (same helpers), i.e. of
//     inference/src/model/qwen.cu:291-458 and inference/src/model/expert.cu:44-59.
// Ring stages are always consumed by the same warp (item q -> stage q % S, warp q % 8, S % 8 == 0).
// Cooperative launch guarantees that all CTAs are co-resident, which the grid barrier needs.
#include "kernels.h"
#include "ptx.cuh"
#include "bs1_common.cuh"
#include "attn_core.cuh"
#include <cooperative_groups.h>

namespace tffn {

namespace {

using namespace bs1;

constexpr int kMegaWarps = 8;                       // consumer warps; warp 8 is the copy producer
constexpr int kMegaThreads = (kMegaWarps + 1) * 32;
constexpr int kMegaConsumers = kMegaWarps * 32;
constexpr int kMegaOprojRows = 2;                   // o_proj rows per ring item
constexpr int kMegaLmRows = 6;                      // LM-head rows per ring item (a stage holds 6 rows)
constexpr int kMegaMaxSplits = 16;                  // attention context splits

struct MegaSmem {
    int stages;
    size_t stage_bytes, scratch_off, ctx_off, bar_off, total;
};
// ring | scratch (attention merge buffers, later the per-warp FFN sums) | merged attention output | barriers
template <int HD, int G>
__host__ __device__ inline MegaSmem mega_smem_layout(int H) {
    MegaSmem s;
    s.stage_bytes = (size_t)H * 12;  // six rows of H bf16: one base + one expert FFN record
    size_t scratch = sizeof(AttnShared<HD, G>);
    const size_t part = (size_t)kMegaWarps * H * 4;
    if (part > scratch) scratch = part;
    scratch = (scratch + 127) / 128 * 128;
    const size_t fixed = scratch + (size_t)H * 2 + 128 + 1024;
    const size_t budget = 224 * 1024;
    int st = (int)((budget - fixed) / s.stage_bytes) / kMegaWarps * kMegaWarps;
    if (st > 32) st = 32;
    s.stages = st;
    s.scratch_off = (s.stage_bytes * (st > 0 ? st : 0) + 127) / 128 * 128;
    s.ctx_off = s.scratch_off + scratch;
    s.bar_off = (s.ctx_off + (size_t)H * 2 + 127) / 128 * 128;
    s.total = s.bar_off + (size_t)(st > 0 ? st : 0) * 16 + 128;
    return s;
}

__device__ __forceinline__ unsigned long long gtime_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// this CTA's share [begin, end) of n things
__device__ __forceinline__ int share_begin(int n, int b, int G) { return (int)(((long long)n * b) / G); }

struct MegaCounts {
    int uA0, nA, rB0, rB1, nB, iC0, nC, vD0, vD1, nD, per_layer;
};
__device__ __forceinline__ MegaCounts mega_counts(const Bs1Ctx& c, int b, int G) {
    MegaCounts m;
    const int U = (c.nh + 2 * c.nkv) * (c.hd / 2);
    m.uA0 = share_begin(U, b, G);
    m.nA = share_begin(U, b + 1, G) - m.uA0;
    m.rB0 = share_begin(c.H, b, G);
    m.rB1 = share_begin(c.H, b + 1, G);
    m.nB = (m.rB1 - m.rB0 + kMegaOprojRows - 1) / kMegaOprojRows;
    m.iC0 = share_begin(c.I, b, G);
    m.nC = share_begin(c.I, b + 1, G) - m.iC0;
    m.vD0 = share_begin(c.V, b, G);
    m.vD1 = share_begin(c.V, b + 1, G);
    m.nD = (m.vD1 - m.vD0 + kMegaLmRows - 1) / kMegaLmRows;
    m.per_layer = m.nA + m.nB + m.nC;
    return m;
}

struct MegaParams {
    Bs1Ctx c;
    const Bs1Layer* layers;  // device array [L]
    int L;
    const bf16 *embed, *final_norm, *lm_head;
    KvView kv;
    float* attn_part;   // [nkv][kMegaMaxSplits][G * (hd + 2)]
    unsigned* barrier;  // grid-barrier arrival counter, zero at launch
};

// Grid barrier over the consumer threads of all CTAs. Returns false (CTA-uniform) after a time-out.
__device__ __forceinline__ bool grid_sync(const MegaParams& p, unsigned& epoch, int* s_abort) {
    asm volatile("bar.sync 1, %0;" ::"n"(kMegaConsumers) : "memory");
    if (threadIdx.x == 0) {
        epoch += 1;
        __threadfence();
        atomicAdd(p.barrier, 1u);
        const unsigned target = epoch * gridDim.x;
        bool ok = false;
        for (uint32_t i = 0; i < kSpinLimit; ++i) {
            if (ld_acquire_u32(p.barrier) >= target) { ok = true; break; }
            if ((i & 255u) == 255u) {
                if (__ldcg(p.c.status) != 0) break;  // another CTA gave up: leave as well
                __nanosleep(64);
            }
        }
        if (!ok) {
            dev_fail(p.c.status, DEV_ERR_GRID_WAIT);
            *s_abort = 1;
        }
        __threadfence();
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kMegaConsumers) : "memory");
    return *s_abort == 0;
}

}  // namespace

}  // namespace tffn

#include "mega_bs1_kernel.inc"

namespace tffn {

namespace {

struct MegaCombo {
    int nch, hd, g;
};

template <int NCH, int HD, int G>
int mega_launch_t(const MegaParams& p, int grid, cudaStream_t s) {
    const MegaSmem L = mega_smem_layout<HD, G>(p.c.H);
    static size_t configured = 0;
    if (configured < L.total) {
        cudaError_t e = cudaFuncSetAttribute(k_bs1_mega<NCH, HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L.total);
        if (e != cudaSuccess) return (int)e;
        configured = L.total;
    }
    void* args[] = {(void*)&p};
    return (int)cudaLaunchCooperativeKernel((const void*)k_bs1_mega<NCH, HD, G>, dim3(grid), dim3(kMegaThreads), args, L.total, s);
}

template <int NCH, int HD, int G>
bool mega_fits_t(int H) {
    const MegaSmem L = mega_smem_layout<HD, G>(H);
    return L.stages >= kMegaWarps && L.total <= 227 * 1024;
}

inline int nch_of(int H) { return (H / 8 + 31) / 32; }

}  // namespace

// shapes with an instantiation: the Qwen2.5 0.5B / 1.5B geometries and the small test shapes
#define TFFN_MEGA_COMBOS(X) X(4, 64, 7) X(6, 128, 6) X(2, 64, 7) X(1, 64, 2) X(1, 128, 2) X(2, 64, 3)

bool bs1_mega_supported(int H, int I, int hd, int nh, int nkv) {
    if (!bs1_supported(H, I, hd, nh, nkv) || nkv < 1) return false;
    const int nch = nch_of(H), g = nh / nkv;
#define X(N, D, GG) \
    if (nch == N && hd == D && g == GG) return mega_fits_t<N, D, GG>(H);
    TFFN_MEGA_COMBOS(X)
#undef X
    return false;
}

size_t bs1_mega_attn_part_floats(int nkv, int hd, int g) { return (size_t)nkv * kMegaMaxSplits * g * (hd + 2); }

int launch_bs1_mega(const Bs1Ctx& c, const Bs1Layer* layers_dev, int L, const bf16* embed, const bf16* final_norm,
                    const bf16* lm_head, KvView kv, float* attn_part, unsigned* barrier, cudaStream_t s) {
    MegaParams p;
    p.c = c;
    p.layers = layers_dev;
    p.L = L;
    p.embed = embed;
    p.final_norm = final_norm;
    p.lm_head = lm_head;
    p.kv = kv;
    p.attn_part = attn_part;
    p.barrier = barrier;
    int grid = c.num_sms;
    if (grid > c.I) grid = c.I;
    if (grid > c.H) grid = c.H;
    cudaError_t e = cudaMemsetAsync(barrier, 0, sizeof(unsigned), s);
    if (e != cudaSuccess) return (int)e;
    const int nch = nch_of(c.H), g = c.nh / c.nkv;
#define X(N, D, GG) \
    if (nch == N && c.hd == D && g == GG) return mega_launch_t<N, D, GG>(p, grid, s);
    TFFN_MEGA_COMBOS(X)
#undef X
    return (int)cudaErrorInvalidValue;
}

}  // namespace tffn
