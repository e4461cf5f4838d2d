// Tensor-core GEMM of the batched path (prefill and decode with more than one token):
//     out[t, n] = epilogue( sum_k X[t,k] * W[n,k] )
// "swap-AB": the weight rows fill the MMA's M = 128 dimension and the tokens are the MMA's N
// (16..256), so a decode step with a few dozen tokens wastes no tensor-core rows and each
// weight byte is streamed from HBM exactly once per token tile.
//
// One CTA = one 128-row x BN-token output tile (optionally one K split of it), 6 warps:
//   warp 0   TMA producer: 128x64 weight box + BNx64 activation box per stage, 128-byte swizzle
//   warp 1   allocates TMEM, issues tcgen05.mma (one thread), commits stages back to the producer
//   warps 2-5 epilogue: tcgen05.ld the fp32 accumulators (lane = weight row, column = token),
//            apply the epilogue and store. With split-K the splits of a tile are one thread-block
//            cluster: partial tiles stay in shared memory and are summed across the cluster over
//            distributed shared memory in rank order, so the result does not depend on
//            scheduling and no partial sum touches HBM.
// Two operand pairs can be accumulated into two TMEM regions (gate|up for the SwiGLU epilogue,
// base|expert for the down projection) and are combined in fp32 in the epilogue.
// It replaces the reference's cublasGemmEx wrappers (inference/src/backend/cuda_ops.cu:18-43)
// and the element-wise kernels around them (silu_mul :58-69, add :152-157,
// k_add_fp32_to_bf16 inference/src/model/qwen.cu:282-285).
#include "kernels.h"
#include "ptx.cuh"
#include "launch.h"
#include <cstdio>
#include <cstring>
#include <functional>
#include <mutex>
#include <unordered_map>

namespace tffn {

namespace {

constexpr int BM = 128;  // weight rows per tile
constexpr int BK = 64;   // K elements per stage (128 bytes of bf16)
constexpr int kGemmThreads = 192;
constexpr int kMaxSmem = 227 * 1024;  // dynamic shared memory a CTA may claim on sm_100
constexpr int kMaxSplits = 16;  // cluster size; above 8 needs the non-portable opt-in (gemm_prepare)

struct GemmDev {
    CUtensorMap tmW[4];  // [problem * 2 + operand pair]
    CUtensorMap tmX[4];
    int kblocks[2];
    int N, T, splits, mode, t_tiles, stages;
    int tile_n;          // output indices per tile: 128, or 64 for GEMM_SWIGLU (64 gate rows + 64 up rows per tile)
    float alpha, out_scale;
    void* out[2];        // per problem
    long long ldo;
    int* status;
    GemmQkvEpilogue qkv;  // GEMM_QKV only
    unsigned long long* trace;  // optional: 64 timestamps (ns) per CTA, see GemmCall::trace
    unsigned long long* tl;     // optional: step timeline of this launch
    float* amax_val;            // GEMM_STORE_F32: per (token, tile) maximum and its index, or nullptr
    int* amax_idx;
};

__device__ __forceinline__ unsigned long long gtime_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TFFN_TRACE(slot)                                                                                            \
    do {                                                                                                            \
        if (p.trace) p.trace[(size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 64 + (slot)] = gtime_ns(); \
    } while (0)

template <int BN>
struct GemmCfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // The ring depth is chosen at launch. A grid of at most one CTA per SM gets the deepest ring
    // that fits (about 190 KB in flight per SM: the HBM latency under load is several microseconds,
    // so the bytes in flight bound the stream); a larger grid of decode-sized tiles gets 4 stages
    // so that two CTAs share an SM.
    static constexpr int MAX_STAGES = (196 * 1024 / STAGE_BYTES) > 10 ? 10 : (196 * 1024 / STAGE_BYTES);
    static constexpr int SHARED_STAGES = (BN <= 64) ? 4 : MAX_STAGES;
    // the epilogue parks one fp32 plane [BN][128] in the (by then idle) stage memory
    static_assert(BN * BM * 4 + BN * 8 <= SHARED_STAGES * STAGE_BYTES, "plane (+ per-token maxima) must fit the smallest ring");
    static constexpr int smem_bytes(int stages) { return stages * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/; }
    static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;  // two accumulators, power of two
};

// ---------------------------------------------------------------------------------------------
// Finalisation of 4 consecutive rows (n .. n+3) of one token column: the epilogues of all modes.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint2 pack_bf16x4(float a, float b, float c, float d) {
    return make_uint2((uint32_t)bf16_bits(a) | ((uint32_t)bf16_bits(b) << 16),
                      (uint32_t)bf16_bits(c) | ((uint32_t)bf16_bits(d) << 16));
}

// What a finalisation reads from global memory besides the accumulators. None of it depends on this
// kernel's own arithmetic, so with split-K (where a warp finishes at most two columns) the epilogue warps
// fetch it while the MMAs still run, instead of paying two or three dependent L2 round trips per column
// after the reduction.
struct FinalizePre {
    bool valid;      // the fields below were fetched
    uint2 residual;  // GEMM_RESIDUAL: the four old bf16 values
    int pos, pg;     // GEMM_QKV: position and page of the token (pg = -1: bad page or position)
    float4 cs, sn;   // GEMM_QKV: the RoPE table entries of this lane's rows
};

// GEMM_QKV: position of token t, its page, and the RoPE entries for rows n .. n+3
__device__ __forceinline__ void prefetch_qkv(const GemmDev& p, int n, int t, FinalizePre& f) {
    const GemmQkvEpilogue& e = p.qkv;
    const int hd = e.kv.hd, half = hd >> 1;
    f.valid = true;
    f.pos = __ldcg(e.tok_pos + t);
    f.pg = -1;
    f.cs = f.sn = make_float4(0.f, 0.f, 0.f, 0.f);
    if (f.pos < 0 || f.pos >= e.max_pos || n >= p.N) return;
    const int seq = __ldcg(e.tok_seq + t);
    const int pg = __ldcg(e.kv.block_table + (size_t)seq * e.kv.max_pages_per_seq + f.pos / kPageTokens);
    f.pg = (pg >= 0 && pg < e.kv.num_pages) ? pg : -1;
    if (n < (e.nh + e.kv.nkv) * hd) {  // q and k rows are rotated
        const int i = (n % hd) % half;
        f.cs = *(const float4*)(e.rope_cos + (size_t)f.pos * half + i);
        f.sn = *(const float4*)(e.rope_sin + (size_t)f.pos * half + i);
    }
}

// GEMM_QKV: round to bf16, add the bias in bf16 (k_add_bias, inference/src/model/qwen.cu:223-226),
// rotate q and k in fp32 at the token's position (k_rope, qwen.cu:232-244) — the RoPE partner rows
// (i <-> i + hd/2) sit hd/8 lanes away in the same warp, because a warp holds all 128 rows of a
// column — keep q in fp32, write k (rounded after the rotation) and v as bf16 into the
// sequence's page (qwen.cu:339-346). Every lane of the warp must call it (shuffles).
__device__ __forceinline__ void finalize_qkv(const GemmDev& p, int n, int t, float4 v, FinalizePre f) {
    const GemmQkvEpilogue& e = p.qkv;
    const int hd = e.kv.hd, half = hd >> 1;
    const int d = n % hd;  // tiles start at multiples of 128 and hd divides 128
    const bool in_range = n < p.N;
    float x[4] = {bf16_round(v.x), bf16_round(v.y), bf16_round(v.z), bf16_round(v.w)};
    if (e.bias && in_range) {
        const uint2 b = *(const uint2*)(e.bias + n);
        x[0] = bf16_round(x[0] + bf16_lo(b.x));
        x[1] = bf16_round(x[1] + bf16_hi(b.x));
        x[2] = bf16_round(x[2] + bf16_lo(b.y));
        x[3] = bf16_round(x[3] + bf16_hi(b.y));
    }
    float xp[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) xp[j] = __shfl_xor_sync(0xffffffffu, x[j], hd >> 3);
    if (!in_range) return;
    if (!f.valid) prefetch_qkv(p, n, t, f);
    if (f.pos < 0 || f.pos >= e.max_pos) {
        dev_fail(p.status, DEV_ERR_BOUNDS);
        return;
    }
    const int nq = e.nh * hd, nk = e.kv.nkv * hd;
    const int kind = n < nq ? 0 : (n < nq + nk ? 1 : 2);
    float o[4] = {x[0], x[1], x[2], x[3]};
    if (kind != 2) {
        const float cs[4] = {f.cs.x, f.cs.y, f.cs.z, f.cs.w}, sn[4] = {f.sn.x, f.sn.y, f.sn.z, f.sn.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = d < half ? x[j] * cs[j] - xp[j] * sn[j] : xp[j] * sn[j] + x[j] * cs[j];
    }
    if (kind == 0) {
        *(float4*)(e.q_out + (size_t)t * nq + n) = make_float4(o[0], o[1], o[2], o[3]);
        return;
    }
    if (f.pg < 0) {
        dev_fail(p.status, DEV_ERR_BOUNDS);
        return;
    }
    const int head = kind == 1 ? (n - nq) / hd : (n - nq - nk) / hd;
    bf16* pool = (kind == 1 ? e.kv.k_pool : e.kv.v_pool) + (size_t)e.layer * e.kv.layer_stride;
    bf16* dst = pool + (((size_t)f.pg * e.kv.nkv + head) * kPageTokens + f.pos % kPageTokens) * hd + d;
    *(uint2*)dst = pack_bf16x4(o[0], o[1], o[2], o[3]);
}

__device__ __forceinline__ bool plain_is_vector(const GemmDev& p, int n) { return (n + 3 < p.N) && ((p.ldo & 3) == 0); }

// GEMM_RESIDUAL: the old values of rows n .. n+3 of token t (read through L2)
__device__ __forceinline__ void prefetch_residual(const GemmDev& p, const void* out, int n, int t, FinalizePre& f) {
    f.valid = n < p.N && plain_is_vector(p, n);
    if (f.valid) f.residual = __ldcg((const uint2*)((const bf16*)out + (size_t)t * (size_t)p.ldo + n));
}

// STORE / RESIDUAL / SWIGLU (the SwiGLU value was formed before the call)
__device__ __forceinline__ void finalize_plain(const GemmDev& p, void* out, int n, int t, float4 v, FinalizePre pre) {
    if (n >= p.N) return;
    const size_t o = (size_t)t * (size_t)p.ldo + n;
    const bool vec = plain_is_vector(p, n);
    const float f[4] = {v.x, v.y, v.z, v.w};
    switch (p.mode) {
        case GEMM_STORE_F32:
            if (!out) break;  // only the fused arg-max was asked for
            if (vec) {
                *(float4*)((float*)out + o) = make_float4(p.out_scale * v.x, p.out_scale * v.y, p.out_scale * v.z, p.out_scale * v.w);
            } else {
                for (int j = 0; j < 4 && n + j < p.N; ++j) ((float*)out)[o + j] = p.out_scale * f[j];
            }
            break;
        case GEMM_RESIDUAL: {
            // h = bf16(float(h) + sum) (k_add_fp32_to_bf16, qwen.cu:282-285); h is read through L2
            bf16* h = (bf16*)out;
            if (vec) {
                const uint2 old = pre.valid ? pre.residual : __ldcg((const uint2*)(h + o));
                *(uint2*)(h + o) = pack_bf16x4(bf16_lo(old.x) + f[0], bf16_hi(old.x) + f[1], bf16_lo(old.y) + f[2],
                                               bf16_hi(old.y) + f[3]);
            } else {
                for (int j = 0; j < 4 && n + j < p.N; ++j) {
                    const float old = __uint_as_float((uint32_t)__ldcg((const unsigned short*)(h + o + j)) << 16);
                    h[o + j] = __float2bfloat16_rn(old + f[j]);
                }
            }
            break;
        }
        default:  // GEMM_STORE_BF16, GEMM_SWIGLU
            if (vec) {
                *(uint2*)((bf16*)out + o) = pack_bf16x4(f[0], f[1], f[2], f[3]);
            } else {
                for (int j = 0; j < 4 && n + j < p.N; ++j) ((bf16*)out)[o + j] = __float2bfloat16_rn(f[j]);
            }
            break;
    }
}

// Fused greedy pick (GEMM_STORE_F32): all 32 lanes of the warp that finished tile column t hold rows
// n .. n+3 of it; the tile's maximum and its index (lowest index among equal maxima: sample(),
// inference/src/main.cpp:45-51) go to amax_val / amax_idx [t][tile].
__device__ __forceinline__ void warp_amax(const GemmDev& p, int n, float4 v, float& best, int& bi) {
    const float f[4] = {v.x, v.y, v.z, v.w};
    best = -INFINITY;
    bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (n + j < p.N && (f[j] > best || (f[j] == best && n + j < bi))) { best = f[j]; bi = n + j; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
}
__device__ __forceinline__ void publish_amax(const GemmDev& p, int n, int t, float4 v, int lane) {
    if (!p.amax_val) return;
    float best;
    int bi;
    warp_amax(p, n, v, best, bi);
    if (lane == 0) {
        p.amax_val[(size_t)t * gridDim.x + blockIdx.x] = best;
        p.amax_idx[(size_t)t * gridDim.x + blockIdx.x] = bi;
    }
}
__device__ __forceinline__ float4 ld_shared_cluster_v4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void add4(float4& a, const float4& b) {
    a.x += b.x;
    a.y += b.y;
    a.z += b.z;
    a.w += b.w;
}

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, (BN <= 64) ? 2 : 1) k_gemm_tc(const __grid_constant__ GemmDev p) {
    using Cfg = GemmCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int STAGES = p.stages;
    uint64_t* full = (uint64_t*)(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int prob = blockIdx.y / p.t_tiles;  // independent problems (base / expert gate-up) share a launch
    const int n0 = blockIdx.x * p.tile_n, t0 = (blockIdx.y % p.t_tiles) * BN;
    const bool halves = p.mode == GEMM_SWIGLU;  // A tile = 64 gate rows over 64 up rows, one accumulator
    void* const out = p.out[prob];
    const int total_kb = p.kblocks[0] + p.kblocks[1];
    const int kb_begin = (int)(((long long)blockIdx.z * total_kb) / p.splits);
    const int kb_end = (int)(((long long)(blockIdx.z + 1) * total_kb) / p.splits);
    const int n_iters = kb_end - kb_begin;
    const bool has0 = kb_begin < p.kblocks[0] && n_iters > 0;
    const bool has1 = kb_end > p.kblocks[0] && p.kblocks[1] > 0 && n_iters > 0;
    constexpr uint32_t tmem_cols = Cfg::TMEM_COLS;

    if (threadIdx.x == 0) {
        TFFN_TRACE(0);
        tl_mark(p.tl, 0);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    FinalizePre pre[2];  // epilogue warps, split-K: operands of the columns they will finish
    pre[0].valid = pre[1].valid = false;

    if (warp == 0) {
        if (lane == 0) {
            prefetch_tmap(&p.tmW[prob * 2]);
            prefetch_tmap(&p.tmX[prob * 2]);
            // Weights do not depend on the previous kernel: the first ring of weight boxes is
            // requested before griddepcontrol.wait, the activation boxes after it.
            const int pre = n_iters < STAGES ? n_iters : STAGES;
            for (int it = 0; it < pre; ++it) {
                const int i = kb_begin + it;
                const int seg = i >= p.kblocks[0] ? 1 : 0;
                const int kb = seg ? i - p.kblocks[0] : i;
                mbar_arrive_expect_tx(&full[it], Cfg::STAGE_BYTES);
                if (halves) {
                    tma_load_2d(smem + it * Cfg::STAGE_BYTES, &p.tmW[prob * 2], kb * BK, n0, &full[it]);
                    tma_load_2d(smem + it * Cfg::STAGE_BYTES + Cfg::A_BYTES / 2, &p.tmW[prob * 2 + 1], kb * BK, n0, &full[it]);
                } else {
                    tma_load_2d(smem + it * Cfg::STAGE_BYTES, &p.tmW[prob * 2 + seg], kb * BK, n0, &full[it]);
                }
            }
            TFFN_TRACE(1);
            pdl_wait();
            TFFN_TRACE(2);
            tl_mark(p.tl, 1);
            for (int it = 0; it < pre; ++it) {
                const int i = kb_begin + it;
                const int seg = i >= p.kblocks[0] ? 1 : 0;
                const int kb = seg ? i - p.kblocks[0] : i;
                tma_load_2d(smem + it * Cfg::STAGE_BYTES + Cfg::A_BYTES, &p.tmX[prob * 2 + seg], kb * BK, t0, &full[it]);
            }
            for (int it = pre; it < n_iters; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, p.status, DEV_ERR_EMPTY_WAIT)) break;
                const int i = kb_begin + it;
                const int seg = i >= p.kblocks[0] ? 1 : 0;
                const int kb = seg ? i - p.kblocks[0] : i;
                uint8_t* a = smem + s * Cfg::STAGE_BYTES;
                uint8_t* b = a + Cfg::A_BYTES;
                mbar_arrive_expect_tx(&full[s], Cfg::STAGE_BYTES);
                if (halves) {
                    tma_load_2d(a, &p.tmW[prob * 2], kb * BK, n0, &full[s]);
                    tma_load_2d(a + Cfg::A_BYTES / 2, &p.tmW[prob * 2 + 1], kb * BK, n0, &full[s]);
                } else {
                    tma_load_2d(a, &p.tmW[prob * 2 + seg], kb * BK, n0, &full[s]);
                }
                tma_load_2d(b, &p.tmX[prob * 2 + seg], kb * BK, t0, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
            bool started[2] = {false, false};
            bool ok = true;
            for (int it = 0; it < n_iters && ok; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                ok = mbar_wait(&full[s], ph, p.status, DEV_ERR_FULL_WAIT);
                if (!ok) break;
                if (it < 12) TFFN_TRACE(16 + it);
                tc_fence_after();
                const int seg = (kb_begin + it) >= p.kblocks[0] ? 1 : 0;
                const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
                const uint32_t b_addr = a_addr + Cfg::A_BYTES;
                const uint32_t d = tmem_base + (uint32_t)(seg * BN);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    umma_bf16(d, umma_desc_k128(a_addr + k * 32), umma_desc_k128(b_addr + k * 32), idesc,
                              (started[seg] || k > 0) ? 1u : 0u);
                started[seg] = true;
                if (it < 12) TFFN_TRACE(28 + it);
                umma_commit(&empty[s]);
            }
            TFFN_TRACE(3);
            umma_commit(acc_full);  // arrives when every MMA above has finished (also on the error path)
        }
    } else {
        // Epilogue warps 2..5 own TMEM lane quarter (warp % 4): thread = one weight row. They combine
        // the two operand pairs (base + alpha * expert) and park ONE fp32 plane [column][row] in the
        // idle stage memory.
        const int q = warp & 3;
        const int row = q * 32 + lane;
        pdl_wait();  // later phases read and write buffers of earlier kernels
        if (p.splits > 1) {
            // split-K: the (at most two) columns this warp will finish are known; fetch their operands now
            const int S = p.splits, cps = BN / S, rank = (int)cluster_ctarank();
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int jj = (warp - 2) + 4 * u, t = t0 + jj * S + rank;
                if (cps <= 8 && jj < cps && t < p.T) {
                    if (p.mode == GEMM_QKV) prefetch_qkv(p, n0 + lane * 4, t, pre[u]);
                    else if (p.mode == GEMM_RESIDUAL) prefetch_residual(p, out, n0 + lane * 4, t, pre[u]);
                }
            }
        }
        // every lane waits (acquire); the outcome is made warp-uniform because tcgen05.ld is .aligned
        bool ok = mbar_wait(acc_full, 0, p.status, DEV_ERR_ACC_WAIT);
        ok = __all_sync(0xffffffffu, ok);
        if (threadIdx.x == 64) TFFN_TRACE(4);
        tc_fence_after();
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const bool dual = p.kblocks[1] > 0;
        const bool live = ok && n_iters > 0;
        float* plane = (float*)smem;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
            if (t0 + c0 >= p.T) break;
            uint32_t v0[16], v1[16];
            if (live && has0) tmem_ld16(lane_addr + (uint32_t)c0, v0);
            if (live && has1) tmem_ld16(lane_addr + (uint32_t)(BN + c0), v1);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float a0 = (live && has0) ? __uint_as_float(v0[j]) : 0.f;
                const float a1 = (live && has1) ? __uint_as_float(v1[j]) : 0.f;
                plane[(size_t)(c0 + j) * BM + row] = dual ? a0 + p.alpha * a1 : a0;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 64) TFFN_TRACE(5);
    // Finalisation is vectorised the other way round from the TMEM layout: a warp takes one column, a
    // lane 4 consecutive rows, so every global access is 8 or 16 bytes per lane and the RoPE partner of
    // a row sits in the same warp. With split-K the splits of one output tile form a thread-block
    // cluster (1,1,splits): after a cluster barrier each rank finalises the columns it owns
    // (column % splits == rank), adding up the parked planes of all ranks in rank order over
    // distributed shared memory (the result does not depend on scheduling). A second cluster barrier
    // keeps every plane alive until its peers have read it; a thread arrives at it as soon as its own
    // remote reads are done and waits only before it leaves, so the barrier's latency hides behind the
    // global stores. (Measured alternatives, both slower per launch: pushing the partial columns into the
    // owners' shared memory with 4-byte remote stores, +3 us; exchanging the planes through an L2
    // workspace, +1 us.)
    if (p.splits > 1) {
        cluster_sync_all();
        if (threadIdx.x == 64) TFFN_TRACE(6);
        if (warp < 2) cluster_arrive();
    }
    constexpr int kWarps = kGemmThreads / 32;
    if (n_iters > 0 && p.splits == 1 && p.mode != GEMM_QKV) {
        // Unsplit tile: every column comes from this CTA's own plane, nothing to wait for, so all six
        // warps (the copy and MMA warps are idle by now) take columns, four in flight per warp.
        const int w = warp;
        const int ncols = min(BN, p.T - t0);
        const float* plane = (const float*)smem;
        if (threadIdx.x == 64) TFFN_TRACE(9);
        if (halves) {
            // rows 0..63 of the tile hold gate, rows 64..127 up, for the same 64 output indices;
            // lane l finishes indices n0 + 2l and n0 + 2l + 1
            bf16* o = (bf16*)out;
            const int nn = n0 + 2 * lane;
            const bool pair = nn + 1 < p.N && (p.ldo & 1) == 0;
#pragma unroll 4
            for (int c = w; c < ncols; c += kWarps) {
                const float2 g = *(const float2*)(plane + (size_t)c * BM + 2 * lane);
                const float2 u = *(const float2*)(plane + (size_t)c * BM + 64 + 2 * lane);
                const float a0 = silu_mul_bf16(g.x, u.x), a1 = silu_mul_bf16(g.y, u.y);
                bf16* dst = o + (size_t)(t0 + c) * (size_t)p.ldo + nn;
                if (pair) {
                    *(uint32_t*)dst = (uint32_t)bf16_bits(a0) | ((uint32_t)bf16_bits(a1) << 16);
                } else {
                    if (nn < p.N) dst[0] = __float2bfloat16_rn(a0);
                    if (nn + 1 < p.N) dst[1] = __float2bfloat16_rn(a1);
                }
            }
        } else {
            const int n = n0 + lane * 4;
            FinalizePre none;
            none.valid = false;
            if (!p.amax_val) {
#pragma unroll 4
                for (int c = w; c < ncols; c += kWarps)
                    finalize_plain(p, out, n, t0 + c, *(const float4*)(plane + (size_t)c * BM + lane * 4), none);
            } else if (warp < 2) {
                // Fused greedy pick: thread = token column, a plain scan down the 128 parked rows (a warp
                // reduction per column would put 64 shuffle chains into every CTA's epilogue). The scan
                // starts at a row that depends on the column so that the lanes hit different banks; the
                // lowest index among equal maxima wins whatever the order.
                for (int c = (int)threadIdx.x; c < ncols; c += 64) {
                    float best = -INFINITY;
                    int bi = 0x7fffffff;
#pragma unroll 8
                    for (int j = 0; j < BM / 4; ++j) {
                        const int r = ((j + c) & (BM / 4 - 1)) * 4;
                        const float4 v = *(const float4*)(plane + (size_t)c * BM + r);
                        const float f[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            const int idx = n0 + r + q4;
                            if (idx < p.N && (f[q4] > best || (f[q4] == best && idx < bi))) { best = f[q4]; bi = idx; }
                        }
                    }
                    p.amax_val[(size_t)(t0 + c) * gridDim.x + blockIdx.x] = best;
                    p.amax_idx[(size_t)(t0 + c) * gridDim.x + blockIdx.x] = bi;
                }
            } else if (out) {
#pragma unroll 4
                for (int c = w - 2; c < ncols; c += kWarps - 2)
                    finalize_plain(p, out, n, t0 + c, *(const float4*)(plane + (size_t)c * BM + lane * 4), none);
            }
        }
    } else if (warp >= 2) {
        const int w = warp - 2;
        const int r4 = lane * 4;
        const int n = n0 + r4;
        const int S = p.splits, cps = BN / S;
        const uint32_t rank = S > 1 ? cluster_ctarank() : 0u;
        const uint32_t plane_local = smem_u32(smem);
        if (threadIdx.x == 64) TFFN_TRACE(9);
        // sum over the ranks' planes of rows row_off .. row_off+3 of tile column c
        auto column_sum = [&](int c, int row_off) {
            const uint32_t off = (uint32_t)(((size_t)c * BM + row_off) * 4);
            if (S == 1) return *(const float4*)(smem + off);
            float4 acc = ld_shared_cluster_v4(map_shared_rank(plane_local + off, 0u));
#pragma unroll 4
            for (int z = 1; z < S; ++z) add4(acc, ld_shared_cluster_v4(map_shared_rank(plane_local + off, (uint32_t)z)));
            return acc;
        };
        auto finish = [&](int t, float4 acc, float4 up, const FinalizePre& f) {
            if (p.mode == GEMM_QKV) {
                finalize_qkv(p, n, t, acc, f);
            } else if (halves) {
                // rows 0..63 of the tile hold gate, rows 64..127 up, for the same 64 output indices
                if (lane < 16)
                    finalize_plain(p, out, n, t,
                                   make_float4(silu_mul_bf16(acc.x, up.x), silu_mul_bf16(acc.y, up.y), silu_mul_bf16(acc.z, up.z),
                                               silu_mul_bf16(acc.w, up.w)), f);
            } else {
                finalize_plain(p, out, n, t, acc, f);
                publish_amax(p, n, t, acc, lane);
            }
        };
        const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (S > 1 && cps <= 8) {
            // at most two columns per warp: all remote reads first, then the arrival, then the stores
            float4 acc[2], up[2];
            bool have[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int jj = w + 4 * u, c = jj * S + (int)rank;
                have[u] = n_iters > 0 && jj < cps && t0 + c < p.T;  // warp-uniform
                acc[u] = have[u] ? column_sum(c, r4) : zero4;
                up[u] = (have[u] && halves && lane < 16) ? column_sum(c, r4 + 64) : zero4;
            }
            cluster_arrive();
            if (threadIdx.x == 64) TFFN_TRACE(10);
#pragma unroll
            for (int u = 0; u < 2; ++u)
                if (have[u]) finish(t0 + (w + 4 * u) * S + (int)rank, acc[u], up[u], pre[u]);
        } else {
            FinalizePre none;
            none.valid = false;
            for (int jj = w; jj < cps && n_iters > 0; jj += 4) {
                const int c = jj * S + (int)rank;
                if (t0 + c >= p.T) break;  // warp-uniform
                const float4 acc = column_sum(c, r4);
                const float4 up = (halves && lane < 16) ? column_sum(c, r4 + 64) : zero4;
                finish(t0 + c, acc, up, none);
            }
            if (S > 1) cluster_arrive();
        }
        if (threadIdx.x == 64) TFFN_TRACE(7);
    }
    if (p.splits > 1) cluster_wait();  // every peer has finished reading this CTA's plane
    if (threadIdx.x == 64) {
        TFFN_TRACE(8);
        tl_mark(p.tl, 2);
    }
    if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

struct TmapKey {
    const void* ptr;
    uint64_t rows, cols, ld;
    uint32_t box_rows;
    bool operator==(const TmapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct TmapKeyHash {
    size_t operator()(const TmapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ (k.rows * 1000003u) ^ (k.cols * 7919u) ^ (k.ld << 20) ^ k.box_rows;
    }
};

bool encode_tmap(CUtensorMap* tm, const bf16* ptr, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_rows);

bool make_tmap(TmapCache* cache, CUtensorMap* tm, const bf16* ptr, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_rows);

// 2-D bf16 tensor [rows, cols] with a row stride, box = box_rows x 64 columns, 128-byte swizzle
bool encode_tmap(CUtensorMap* tm, const bf16* ptr, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld_elems * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)ptr, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace

struct TmapCache {
    std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> maps;
};
TmapCache* tmap_cache_create() { return new TmapCache(); }
void tmap_cache_free(TmapCache* c) { delete c; }

namespace {

bool make_tmap(TmapCache* cache, CUtensorMap* tm, const bf16* ptr, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_rows) {
    if (!cache) return encode_tmap(tm, ptr, rows, cols, ld_elems, box_rows);
    TmapKey key{ptr, rows, cols, ld_elems, box_rows};
    auto it = cache->maps.find(key);
    if (it != cache->maps.end()) {
        *tm = it->second;
        return true;
    }
    if (!encode_tmap(tm, ptr, rows, cols, ld_elems, box_rows)) return false;
    cache->maps.emplace(key, *tm);
    return true;
}

// clusters of `splits` CTAs of k_gemm_tc<BN> with `stages` ring stages that can be resident at once on the
// current device (cudaOccupancyMaxActiveClusters; remembered per configuration)
template <int BN>
int max_active_clusters(const cudaLaunchConfig_t& cfg, int stages, int splits) {
    static std::mutex mu;
    static std::unordered_map<long long, int> seen;
    int dev = 0;
    cudaGetDevice(&dev);
    const long long key = ((long long)dev << 32) | ((long long)stages << 8) | splits;
    std::lock_guard<std::mutex> lock(mu);
    auto it = seen.find(key);
    if (it != seen.end()) return it->second;
    int n = 0;
    cudaLaunchConfig_t q = cfg;
    q.dynamicSmemBytes = GemmCfg<BN>::smem_bytes(stages);
    if (cudaOccupancyMaxActiveClusters(&n, k_gemm_tc<BN>, &q) != cudaSuccess) {
        cudaGetLastError();
        n = 1 << 30;  // unknown: keep the configuration
    }
    seen.emplace(key, n);
    return n;
}

template <int BN>
int launch_bn(const GemmCall& c, const GemmWorkspace& ws, cudaStream_t stream, int force_splits) {
    using Cfg = GemmCfg<BN>;
    GemmDev p;
    memset(&p, 0, sizeof p);
    const int nprob = c.out2 ? 2 : 1;
    const bool halves = c.mode == GEMM_SWIGLU;
    p.tile_n = halves ? BM / 2 : BM;
    if (halves && (c.op[0].K != c.op[1].K || c.op[0].X != c.op[1].X)) return (int)cudaErrorInvalidValue;
    for (int pr = 0; pr < nprob; ++pr)
        for (int i = 0; i < 2; ++i) {
            const GemmOperand& o = pr ? c.op2[i] : c.op[i];
            if (pr == 0) p.kblocks[i] = o.K > 0 ? (o.K + BK - 1) / BK : 0;
            if (o.K <= 0) continue;
            if (pr == 1 && (o.K + BK - 1) / BK != p.kblocks[i]) return (int)cudaErrorInvalidValue;
            if (!make_tmap(ws.tmaps, &p.tmW[pr * 2 + i], o.W, (uint64_t)c.N, (uint64_t)o.K, (uint64_t)o.ldw, halves ? BM / 2 : BM)) return -1000;
            if (!make_tmap(ws.tmaps, &p.tmX[pr * 2 + i], o.X, (uint64_t)(c.x_rows_alloc > c.T ? c.x_rows_alloc : c.T), (uint64_t)o.K,
                           (uint64_t)o.ldx, BN))
                return -1000;
        }
    if (halves) p.kblocks[1] = 0;  // gate and up rows share one accumulator and one pass over K
    for (int i = 1; i < 4; ++i)  // keep unused maps valid
        if (i >= nprob * 2 || (p.kblocks[i & 1] == 0 && !halves)) {
            p.tmW[i] = p.tmW[0];
            p.tmX[i] = p.tmX[0];
        }
    p.N = c.N;
    p.T = c.T;
    p.mode = c.mode;
    p.alpha = c.alpha;
    p.out_scale = c.out_scale == 0.f ? 1.f : c.out_scale;
    p.out[0] = c.out;
    p.out[1] = c.out2 ? c.out2 : c.out;
    p.ldo = c.ldo;
    p.status = ws.status;
    p.trace = c.trace;
    p.tl = c.tl;
    p.amax_val = c.mode == GEMM_STORE_F32 ? c.amax_val : nullptr;
    p.amax_idx = c.amax_idx;
    if (!c.out && !(c.mode == GEMM_STORE_F32 && c.amax_val && c.amax_idx) && c.mode != GEMM_QKV) return (int)cudaErrorInvalidValue;
    if (c.mode == GEMM_QKV) {
        if (!c.qkv || c.op[1].K > 0 || c.out2 || (c.qkv->kv.hd != 64 && c.qkv->kv.hd != 128)) return (int)cudaErrorInvalidValue;
        p.qkv = *c.qkv;
    }
    const int n_tiles = (c.N + p.tile_n - 1) / p.tile_n, t_tiles = (c.T + BN - 1) / BN;
    const int total_kb = p.kblocks[0] + p.kblocks[1];
    const int tiles = n_tiles * t_tiles * nprob;
    p.t_tiles = t_tiles;
    // K splits = cluster size (1, 2, 4, 8 or 16). Inside a decode step one CTA takes in roughly one
    // stage (a 16 KB weight box and its activation box) per 0.5 us whatever the ring depth, about 50 GB/s
    // per SM (measured with the phase stamps; all SMs together about 7 TB/s), so a weight-streaming launch
    // needs about as many CTAs as there are SMs: tiles are split along K until the grid fills the SMs,
    // keeping two k-blocks per split.
    int splits = 1;
    if (force_splits > 0) {
        splits = force_splits;
    } else {
        while (splits < kMaxSplits && tiles * splits * 2 <= ws.num_sms + ws.num_sms / 8 && total_kb / (splits * 2) >= 1) splits *= 2;
        // A long K extent: the stage cadence is a property of the CTA (about 0.45 us per stage), so two
        // CTAs per SM stream twice as much as one until HBM is the limit; keep splitting while every CTA
        // still gets eight k-blocks and the grid fits two per SM (measured at 16 tokens, N 2048, K 22016:
        // 8 splits 49.5 us, half of the 8-CTA clusters waiting for a second wave; 16 splits 18.0 us).
        while (splits < kMaxSplits && tiles * splits * 2 <= 2 * ws.num_sms && total_kb / (splits * 2) >= 8) splits *= 2;
    }
    if (splits != 1 && splits != 2 && splits != 4 && splits != 8 && splits != 16) return (int)cudaErrorInvalidValue;
    if (splits > total_kb) return (int)cudaErrorInvalidValue;
    const bool shared_sm = tiles * splits > ws.num_sms;  // more than one CTA per SM
    p.stages = shared_sm ? Cfg::SHARED_STAGES : Cfg::MAX_STAGES;
    // Many short tiles per SM (the LM head of a small model: 1 187 tiles of 14 k-blocks): what limits such a
    // launch is the set-up and epilogue of every tile, which the other CTAs of the SM have to cover. Three
    // CTAs per SM with 3-stage rings do that better than two with 4 stages (measured inside a decode step,
    // 0.5B shape, 64 tokens: 61 -> 50 us for the 272 MB LM head = 5.4 TB/s).
    if (shared_sm && BN == 64 && splits == 1 && total_kb <= 16 && tiles >= 4 * ws.num_sms) p.stages = 3;
    {
        // No deeper than the k-blocks a CTA streams (but deep enough to park the epilogue plane): the
        // shared memory a CTA does not claim lets CTAs of the next kernel of the stream become resident
        // early under programmatic dependent launch and fetch their weights ahead of their grid wait.
        const int iters = (total_kb + splits - 1) / splits;
        const int plane_stages = (BN * BM * 4 + BN * 8 /* per-token maxima of the fused pick */ + Cfg::STAGE_BYTES - 1) / Cfg::STAGE_BYTES;
        const int want = iters > plane_stages ? iters : plane_stages;
        if (p.stages > want) p.stages = want;
    }
    p.splits = splits;
    cudaLaunchConfig_t cfg = cudaLaunchConfig_t{};
    cfg.gridDim = dim3(n_tiles, t_tiles * nprob, splits);
    if ((long long)n_tiles * t_tiles * nprob * splits > c.trace_ctas) p.trace = nullptr;
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = Cfg::smem_bytes(p.stages);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (splits > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = splits;
        ++na;
    }
    if (c.pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (splits > 1 && !shared_sm) {
        // A cluster lives inside one GPC. With deep rings (one CTA per SM) a GPC of 18 SMs holds two clusters
        // of 8 and leaves two SMs empty, so that 18 clusters need a second wave (seen on the 7B shape over two
        // ranks: q|k|v, 18 clusters of 8 with 7-stage rings, 2 clusters started 14 us late). Ask how many
        // clusters of this launch can be resident at once and, if they are fewer than the grid has, give up
        // ring depth (not below three stages or what the epilogue plane needs) until they all fit. Grids of
        // more CTAs than SMs already run their shallow shared-SM rings and are left alone.
        const int clusters = n_tiles * t_tiles * nprob;
        const int iters = (total_kb + splits - 1) / splits;
        const int plane_stages = (BN * BM * 4 + BN * 8 + Cfg::STAGE_BYTES - 1) / Cfg::STAGE_BYTES;
        const int want_stages = iters < 3 ? iters : 3;
        const int floor_stages = plane_stages > want_stages ? plane_stages : want_stages;  // never below the parked plane
        while (p.stages > floor_stages && max_active_clusters<BN>(cfg, p.stages, splits) < clusters) {
            --p.stages;
            cfg.dynamicSmemBytes = Cfg::smem_bytes(p.stages);
        }
    }
    return (int)cudaLaunchKernelEx(&cfg, k_gemm_tc<BN>, p);
}

}  // namespace

int gemm_prepare() {
    cudaError_t e;
#define TFFN_PREP(BN)                                                                                                 \
    e = cudaFuncSetAttribute(k_gemm_tc<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem); \
    if (e != cudaSuccess) return (int)e;                                                                             \
    e = cudaFuncSetAttribute(k_gemm_tc<BN>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);                     \
    if (e != cudaSuccess) return (int)e;                                                                             \
    e = prefer_max_shared(k_gemm_tc<BN>);                                                                            \
    if (e != cudaSuccess) return (int)e;
    TFFN_PREP(16) TFFN_PREP(32) TFFN_PREP(64) TFFN_PREP(128) TFFN_PREP(256)
#undef TFFN_PREP
    return 0;
}

int launch_gemm(const GemmCall& c, const GemmWorkspace& ws, cudaStream_t stream, int force_splits) {
    if (c.T <= 0 || c.N <= 0 || c.op[0].K <= 0) return (int)cudaErrorInvalidValue;
    // A short K extent with few output tiles (the attention projections of a small model): the grid is
    // filled by splitting K, and the cost of such a launch is the exchange of the partial tiles (measured:
    // 28 KB per CTA over distributed shared memory take 2 to 3.6 us). Halving the token tile (two token
    // tiles, the same split factor, twice the CTAs) halves the plane a CTA parks and the exchange: 14 KB per
    // CTA; the weights are then read twice, the second time from L2 (measured on the 0.5B shape at 64
    // tokens: q|k|v 8.5 -> 7.2 us, o_proj 8.0 -> 7.2 us per launch inside a step).
    {
        const int total_kb = (c.op[0].K + BK - 1) / BK + (c.op[1].K > 0 ? (c.op[1].K + BK - 1) / BK : 0);
        const int n_tiles = (c.N + BM - 1) / BM;
        if (force_splits == 0 && c.mode != GEMM_SWIGLU && !c.out2 && c.T > 32 && c.T <= 64 && total_kb <= 16 &&
            n_tiles * 8 <= ws.num_sms)
            return launch_bn<32>(c, ws, stream, force_splits);
        // A long K extent with as few tiles (the down projection): the largest cluster, 16 splits, is
        // not enough to fill the SMs with 64-token tiles; with 32-token tiles twice as many CTAs (two per SM)
        // stream half as many k-blocks each (measured: 12.6 -> 11.6 us per launch inside a step).
        if (force_splits == 0 && c.mode != GEMM_SWIGLU && !c.out2 && c.T > 32 && c.T <= 64 && total_kb >= 64 &&
            n_tiles * 8 <= ws.num_sms)
            return launch_bn<32>(c, ws, stream, kMaxSplits);
    }
    if (c.T <= 16) return launch_bn<16>(c, ws, stream, force_splits);
    if (c.T <= 32) return launch_bn<32>(c, ws, stream, force_splits);
    if (c.T <= 64) return launch_bn<64>(c, ws, stream, force_splits);
    if (c.T <= 128) return launch_bn<128>(c, ws, stream, force_splits);
    return launch_bn<256>(c, ws, stream, force_splits);
}

}  // namespace tffn
