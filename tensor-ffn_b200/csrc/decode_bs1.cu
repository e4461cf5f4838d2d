// Batch-1 decode: four weight-streaming kernels per layer plus the LM head, all HBM-bound.
//
//   qkv     RMSNorm (recomputed per warp; the row is <= 4 KB) + q|k|v rows + bias + RoPE in
//           registers + K/V written straight into the sequence's page
//   attn    attn.cu (shared with the batched path)
//   oproj   o_proj rows + residual add
//   ffn     ONE kernel: RMSNorm, then each CTA streams its slice of the intermediate dimension
//           as records [gate row | up row | down column] of the base FFN and of the expert
//           FFN side by side (bulk copies into a shared-memory ring, mbarrier-tracked),
//           forms act = silu(g)*u for both, accumulates act_b*down_b + scale*act_e*down_e for
//           all H outputs in registers, and the per-CTA partial sums are folded by a two-level
//           ticket (last CTA of a group, then last group) in a fixed order into the residual
//   lmhead  final RMSNorm + tied LM-head rows streamed through the same kind of ring +
//           arg-max (lowest index among maxima); the last CTA publishes the next token
//
// Every kernel fetches the weights it owns BEFORE griddepcontrol.wait, so with programmatic
// dependent launch the weight stream of kernel n+1 overlaps the tail of kernel n.
// Rounding points follow inference/src/model/qwen.cu:291-458 (see each kernel).
#include "kernels.h"
#include "ptx.cuh"
#include "launch.h"
#include "bs1_common.cuh"

namespace tffn {

namespace {

using namespace bs1;

constexpr int kRowWarps = 4;

__device__ __forceinline__ unsigned long long gtime_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// optional per-CTA phase timestamps (Bs1Ctx::trace, 16 u64 per CTA)
#define BS1_TRACE(c, slot)                                                         \
    do {                                                                           \
        if ((c).trace) (c).trace[(size_t)blockIdx.x * 16 + (slot)] = gtime_ns(); \
    } while (0)  // warps per CTA in the row kernels (qkv, oproj)

// ------------------------------------------------------------------------------------------ qkv
// One warp per RoPE pair: rows (i, i + hd/2) of one head of the concatenated [q|k|v] matrix.
// q,k,v = bf16(x W^T), + bias in bf16, RoPE in fp32 at the token's position, K rounded to bf16
// into the page, V stored as bf16, q kept in fp32 (inference/src/model/qwen.cu:317-346).
template <int NCH>
__global__ void __launch_bounds__(kRowWarps * 32) k_bs1_qkv(Bs1Ctx c, Bs1Layer ly, const bf16* __restrict__ embed,
                                                            KvView kv, int layer, int first) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int H = c.H, hd = c.hd, half = hd >> 1;
    const int unit = blockIdx.x * kRowWarps + warp;
    const int units = (c.nh + 2 * c.nkv) * half;
    pdl_launch_dependents();
    RowRegs<NCH> w0, w1;
    int head = 0, i = 0;
    const bool active = unit < units;
    if (active) {
        head = unit / half;
        i = unit % half;
        const size_t r0 = (size_t)head * hd + i;
        load_row<NCH>(w0, ly.wqkv + r0 * H, H, lane);
        load_row<NCH>(w1, ly.wqkv + (r0 + half) * H, H, lane);
    }
    pdl_wait();
    const bf16* hsrc = c.h;
    if (first) {
        int tok = __ldcg(c.token);
        if (tok < 0 || tok >= c.V) {
            if (threadIdx.x == 0 && blockIdx.x == 0) dev_fail(c.status, DEV_ERR_BOUNDS);
            tok = 0;
        }
        hsrc = embed + (size_t)tok * H;
        if (blockIdx.x == 0 && warp == 0) {  // publish the residual stream for the later kernels
            for (int ch = lane; ch < (H >> 3); ch += 32) ((uint4*)c.h)[ch] = __ldg((const uint4*)hsrc + ch);
        }
    }
    if (!active) return;
    RowRegs<NCH> xn;
    rmsnorm_regs<NCH>(xn, hsrc, ly.attn_norm, H, c.eps, lane);
    float d0 = warp_sum(dot_rows<NCH>(w0, xn));
    float d1 = warp_sum(dot_rows<NCH>(w1, xn));
    if (lane != 0) return;
    const int pos = __ldcg(c.seq_len + c.slot);
    if (pos < 0 || pos >= c.max_pos) {
        dev_fail(c.status, DEV_ERR_BOUNDS);
        return;
    }
    float x0 = bf16_round(d0), x1 = bf16_round(d1);
    if (ly.bqkv) {
        x0 = bf16_round(x0 + __bfloat162float(ly.bqkv[head * hd + i]));
        x1 = bf16_round(x1 + __bfloat162float(ly.bqkv[head * hd + i + half]));
    }
    const int nh = c.nh, nkv = c.nkv;
    if (head < nh + nkv) {
        const float cs = c.rope_cos[(size_t)pos * half + i], sn = c.rope_sin[(size_t)pos * half + i];
        const float r0 = x0 * cs - x1 * sn, r1 = x0 * sn + x1 * cs;
        x0 = r0;
        x1 = r1;
    }
    if (head < nh) {
        c.q[head * hd + i] = x0;
        c.q[head * hd + i + half] = x1;
        return;
    }
    const int kvh = head < nh + nkv ? head - nh : head - nh - nkv;
    const int pg = __ldcg(kv.block_table + (size_t)c.slot * kv.max_pages_per_seq + pos / kPageTokens);
    if (pg < 0 || pg >= kv.num_pages) {
        dev_fail(c.status, DEV_ERR_BOUNDS);
        return;
    }
    bf16* pool = (head < nh + nkv ? kv.k_pool : kv.v_pool) + (size_t)layer * kv.layer_stride;
    bf16* dst = pool + (((size_t)pg * nkv + kvh) * kPageTokens + pos % kPageTokens) * hd;
    dst[i] = __float2bfloat16_rn(x0);
    dst[i + half] = __float2bfloat16_rn(x1);
}

// ------------------------------------------------------------------------------------------ o_proj
// h[n] = bf16(float(h[n]) + ctx . Wo[n,:])   (inference/src/model/qwen.cu:413-419, :282-285)
template <int NCH>
__global__ void __launch_bounds__(kRowWarps * 32) k_bs1_oproj(Bs1Ctx c, Bs1Layer ly) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int H = c.H;
    const int n0 = (blockIdx.x * kRowWarps + warp) * 2;
    pdl_launch_dependents();
    RowRegs<NCH> w0, w1;
    if (n0 < H) load_row<NCH>(w0, ly.wo + (size_t)n0 * H, H, lane);
    if (n0 + 1 < H) load_row<NCH>(w1, ly.wo + (size_t)(n0 + 1) * H, H, lane);
    pdl_wait();
    if (n0 >= H) return;
    RowRegs<NCH> x;
    load_row_act<NCH>(x, c.ctx, H, lane);
    float d0 = warp_sum(dot_rows<NCH>(w0, x));
    float d1 = (n0 + 1 < H) ? warp_sum(dot_rows<NCH>(w1, x)) : 0.f;
    if (lane == 0) {
        c.h[n0] = __float2bfloat16_rn(ld_bf16_cg(c.h + n0) + d0);
        if (n0 + 1 < H) c.h[n0 + 1] = __float2bfloat16_rn(ld_bf16_cg(c.h + n0 + 1) + d1);
    }
}

// ------------------------------------------------------------------------------------------ fused SwiGLU
constexpr int kFfnWarps = 8;          // consumer warps; warp kFfnWarps is the copy producer
constexpr int kFfnThreads = (kFfnWarps + 1) * 32;
constexpr int kFfnGroup = 16;         // CTAs per first-level reduction group

struct FfnSmem {
    int stages;
    size_t stage_bytes;
    size_t ring_off, part_off, bar_off, total;
};
// A stage is always consumed by the same warp (record r -> warp r % kFfnWarps, stage r % stages),
// which needs stages % kFfnWarps == 0: with one parity bit per barrier a warp may only wait for
// the NEXT phase of a stage, never for one two phases ahead of another warp's use.
// The per-warp partial sums reuse the ring once every record has been consumed.
__host__ __device__ inline FfnSmem ffn_smem_layout(int H, bool expert) {
    FfnSmem s;
    s.stage_bytes = (size_t)H * 2 * 3 * (expert ? 2 : 1);
    const size_t part = (size_t)kFfnWarps * H * 4;
    const size_t budget = 200 * 1024;
    int st = (int)(budget / s.stage_bytes) / kFfnWarps * kFfnWarps;
    if (st > 32) st = 32;
    if (st < kFfnWarps) st = kFfnWarps;
    s.stages = st;
    s.ring_off = 0;
    s.part_off = 0;
    size_t ring = s.stage_bytes * st;
    if (ring < part) ring = part;
    s.bar_off = (ring + 127) / 128 * 128;
    s.total = s.bar_off + (size_t)st * 16 + 64;
    return s;
}

// act = bf16(silu(bf16(x.Wg)) * bf16(x.Wu)); out = act.Wd (fp32); expert identical, its fp32
// result scaled by output_scale; ffn = base + expert in fp32; h = bf16(float(h) + ffn)
// (inference/src/model/qwen.cu:422-447, inference/src/model/expert.cu:44-59).
template <int NCH>
__global__ void __launch_bounds__(kFfnThreads, 1) k_bs1_ffn(Bs1Ctx c, Bs1Layer ly) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int H = c.H, I = c.I;
    const bool expert = ly.ffn_expert != nullptr;
    const FfnSmem L = ffn_smem_layout(H, expert);
    uint8_t* ring = smem + L.ring_off;
    float* part = (float*)(smem + L.part_off);
    uint64_t* full = (uint64_t*)(smem + L.bar_off);
    uint64_t* empty = full + L.stages;
    int* s_flag = (int*)(empty + L.stages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x;
    const int i0 = (int)(((long long)I * blockIdx.x) / G), i1 = (int)(((long long)I * (blockIdx.x + 1)) / G);
    const int nrec = i1 - i0;
    const size_t rec_bytes = (size_t)H * 6;

    if (threadIdx.x == 0) {
        for (int s = 0; s < L.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    if (threadIdx.x == 0) BS1_TRACE(c, 0);

    if (warp == kFfnWarps) {
        // producer: the weights do not depend on the previous kernel, so no griddepcontrol.wait here
        if (lane == 0) {
            for (int r = 0; r < nrec; ++r) {
                const int s = r % L.stages;
                const uint32_t ph = (uint32_t)(r / L.stages) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, c.status, DEV_ERR_EMPTY_WAIT)) break;
                uint8_t* dst = ring + (size_t)s * L.stage_bytes;
                mbar_arrive_expect_tx(&full[s], (uint32_t)L.stage_bytes);
                bulk_g2s(dst, (const uint8_t*)ly.ffn_base + (size_t)(i0 + r) * rec_bytes, (uint32_t)rec_bytes, &full[s]);
                if (expert)
                    bulk_g2s(dst + rec_bytes, (const uint8_t*)ly.ffn_expert + (size_t)(i0 + r) * rec_bytes,
                             (uint32_t)rec_bytes, &full[s]);
            }
        }
        return;
    }

    // consumers
    pdl_wait();
    RowRegs<NCH> xn;
    rmsnorm_regs<NCH>(xn, c.h, ly.ffn_norm, H, c.eps, lane);
    if (threadIdx.x == 0) BS1_TRACE(c, 1);
    float acc[NCH * 8];
#pragma unroll
    for (int j = 0; j < NCH * 8; ++j) acc[j] = 0.f;
    const size_t row_bytes = (size_t)H * 2;
    bool ok = true;
    for (int r = warp; r < nrec && ok; r += kFfnWarps) {
        const int s = r % L.stages;
        const uint32_t ph = (uint32_t)(r / L.stages) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(&full[s], ph, c.status, DEV_ERR_FULL_WAIT));
        if (!ok) break;
        if (threadIdx.x == 0 && r == 0) BS1_TRACE(c, 2);
        const uint8_t* st = ring + (size_t)s * L.stage_bytes;
        RowRegs<NCH> wg, wu;
        load_row_smem<NCH>(wg, st, H, lane);
        load_row_smem<NCH>(wu, st + row_bytes, H, lane);
        float gb = dot_rows<NCH>(wg, xn), ub = dot_rows<NCH>(wu, xn), ge = 0.f, ue = 0.f;
        if (expert) {
            load_row_smem<NCH>(wg, st + rec_bytes, H, lane);
            load_row_smem<NCH>(wu, st + rec_bytes + row_bytes, H, lane);
            ge = dot_rows<NCH>(wg, xn);
            ue = dot_rows<NCH>(wu, xn);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            gb += __shfl_xor_sync(0xffffffffu, gb, o);
            ub += __shfl_xor_sync(0xffffffffu, ub, o);
            ge += __shfl_xor_sync(0xffffffffu, ge, o);
            ue += __shfl_xor_sync(0xffffffffu, ue, o);
        }
        const float ab = silu_mul_bf16(gb, ub);
        const float ae = expert ? silu_mul_bf16(ge, ue) * c.expert_scale : 0.f;
        RowRegs<NCH> db;
        load_row_smem<NCH>(db, st + 2 * row_bytes, H, lane);
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const uint32_t u[4] = {db.v[j].x, db.v[j].y, db.v[j].z, db.v[j].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                acc[j * 8 + 2 * k] = fmaf(ab, bf16_lo(u[k]), acc[j * 8 + 2 * k]);
                acc[j * 8 + 2 * k + 1] = fmaf(ab, bf16_hi(u[k]), acc[j * 8 + 2 * k + 1]);
            }
        }
        if (expert) {
            load_row_smem<NCH>(db, st + rec_bytes + 2 * row_bytes, H, lane);
#pragma unroll
            for (int j = 0; j < NCH; ++j) {
                const uint32_t u[4] = {db.v[j].x, db.v[j].y, db.v[j].z, db.v[j].w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    acc[j * 8 + 2 * k] = fmaf(ae, bf16_lo(u[k]), acc[j * 8 + 2 * k]);
                    acc[j * 8 + 2 * k + 1] = fmaf(ae, bf16_hi(u[k]), acc[j * 8 + 2 * k + 1]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
    if (threadIdx.x == 0) BS1_TRACE(c, 3);
    // fold the consumer warps of this CTA (fixed order); the partial sums reuse the ring, so
    // every consumer must be done reading it first
    constexpr int NT = kFfnWarps * 32;
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    const int nchunk = H >> 3;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        const int ch = lane + 32 * j;
        if (ch < nchunk) {
            float4* dst = (float4*)(part + (size_t)warp * H + ch * 8);
            dst[0] = make_float4(acc[j * 8], acc[j * 8 + 1], acc[j * 8 + 2], acc[j * 8 + 3]);
            dst[1] = make_float4(acc[j * 8 + 4], acc[j * 8 + 5], acc[j * 8 + 6], acc[j * 8 + 7]);
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    float* my_part = c.ffn_part + (size_t)blockIdx.x * H;
    for (int col = threadIdx.x; col < H; col += NT) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kFfnWarps; ++w) s += part[(size_t)w * H + col];
        my_part[col] = s;
    }
    if (threadIdx.x == 0) BS1_TRACE(c, 4);
    // level 1: last CTA of the group folds the group's partials
    const int ngroups = (G + kFfnGroup - 1) / kFfnGroup;
    const int grp = blockIdx.x / kFfnGroup;
    const int g_begin = grp * kFfnGroup, g_end = min(G, g_begin + kFfnGroup);
    __threadfence();
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    if (threadIdx.x == 0) {
        const int old = atomicAdd(&c.tickets[1 + grp], 1);
        const int last = old == (g_end - g_begin) - 1;
        if (last) c.tickets[1 + grp] = 0;
        *s_flag = last;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    if (threadIdx.x == 0) BS1_TRACE(c, 5);
    if (!*s_flag) return;
    __threadfence();
    float* gpart = c.ffn_part + (size_t)(G + grp) * H;
    for (int col = threadIdx.x; col < H; col += NT) {
        float v[kFfnGroup];
#pragma unroll
        for (int b = 0; b < kFfnGroup; ++b)  // all loads in flight together, summed in CTA order below
            v[b] = (g_begin + b < g_end) ? __ldcg(c.ffn_part + (size_t)(g_begin + b) * H + col) : 0.f;
        float s = 0.f;
#pragma unroll
        for (int b = 0; b < kFfnGroup; ++b) s += v[b];
        gpart[col] = s;
    }
    if (threadIdx.x == 0) BS1_TRACE(c, 6);
    // level 2: last group folds the group sums into the residual stream
    __threadfence();
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    if (threadIdx.x == 0) {
        const int old = atomicAdd(&c.tickets[0], 1);
        const int last = old == ngroups - 1;
        if (last) c.tickets[0] = 0;
        *s_flag = last;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    if (!*s_flag) return;
    __threadfence();
    for (int col = threadIdx.x; col < H; col += NT) {
        float s = 0.f;
        for (int g0 = 0; g0 < ngroups; g0 += 16) {
            float v[16];
#pragma unroll
            for (int b = 0; b < 16; ++b) v[b] = (g0 + b < ngroups) ? __ldcg(c.ffn_part + (size_t)(G + g0 + b) * H + col) : 0.f;
#pragma unroll
            for (int b = 0; b < 16; ++b) s += v[b];
        }
        c.h[col] = __float2bfloat16_rn(ld_bf16_cg(c.h + col) + s);
    }
    if (threadIdx.x == 0) BS1_TRACE(c, 7);
}

// ------------------------------------------------------------------------------------------ LM head + argmax
constexpr int kLmWarps = 8;
constexpr int kLmThreads = (kLmWarps + 1) * 32;
constexpr int kLmRowsPerStage = 4;

struct LmSmem {
    int stages;
    size_t stage_bytes, bar_off, total;
};
__host__ __device__ inline LmSmem lm_smem_layout(int H) {
    LmSmem s;
    s.stage_bytes = (size_t)kLmRowsPerStage * H * 2;
    int st = (int)((192 * 1024) / s.stage_bytes) / kLmWarps * kLmWarps;  // stages % warps == 0, see ffn_smem_layout
    if (st > 32) st = 32;
    if (st < kLmWarps) st = kLmWarps;
    s.stages = st;
    s.bar_off = (s.stage_bytes * st + 127) / 128 * 128;
    s.total = s.bar_off + (size_t)st * 16 + 64 + kLmWarps * 8;
    return s;
}

// logits = rmsnorm(h) . E^T in fp32 (inference/src/model/qwen.cu:451-454); greedy pick = first
// index of the strict maximum (inference/src/main.cpp:45-51).
template <int NCH>
__global__ void __launch_bounds__(kLmThreads, 1) k_bs1_lmhead(Bs1Ctx c, const bf16* __restrict__ final_norm,
                                                              const bf16* __restrict__ lm_head) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int H = c.H, V = c.V;
    const LmSmem L = lm_smem_layout(H);
    uint64_t* full = (uint64_t*)(smem + L.bar_off);
    uint64_t* empty = full + L.stages;
    int* s_flag = (int*)(empty + L.stages);
    float* s_val = (float*)(s_flag + 2);
    int* s_idx = (int*)(s_val + kLmWarps);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x;
    const int r0 = (int)(((long long)V * blockIdx.x) / G), r1 = (int)(((long long)V * (blockIdx.x + 1)) / G);
    const int nst = (r1 - r0 + kLmRowsPerStage - 1) / kLmRowsPerStage;
    const size_t row_bytes = (size_t)H * 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < L.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kLmWarps) {
        if (lane == 0) {
            for (int r = 0; r < nst; ++r) {
                const int s = r % L.stages;
                const uint32_t ph = (uint32_t)(r / L.stages) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, c.status, DEV_ERR_EMPTY_WAIT)) break;
                const int row = r0 + r * kLmRowsPerStage;
                const int rows = min(kLmRowsPerStage, r1 - row);
                const uint32_t bytes = (uint32_t)(rows * row_bytes);
                mbar_arrive_expect_tx(&full[s], bytes);
                bulk_g2s(smem + (size_t)s * L.stage_bytes, (const uint8_t*)lm_head + (size_t)row * row_bytes, bytes, &full[s]);
            }
        }
        return;
    }

    pdl_wait();
    RowRegs<NCH> xn;
    rmsnorm_regs<NCH>(xn, c.h, final_norm, H, c.eps, lane);
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    bool ok = true;
    for (int r = warp; r < nst && ok; r += kLmWarps) {
        const int s = r % L.stages;
        const uint32_t ph = (uint32_t)(r / L.stages) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(&full[s], ph, c.status, DEV_ERR_FULL_WAIT));
        if (!ok) break;
        const uint8_t* st = smem + (size_t)s * L.stage_bytes;
        const int row = r0 + r * kLmRowsPerStage;
        const int rows = min(kLmRowsPerStage, r1 - row);
        float d[kLmRowsPerStage];
#pragma unroll
        for (int k = 0; k < kLmRowsPerStage; ++k) {
            d[k] = 0.f;
            if (k < rows) {
                RowRegs<NCH> w;
                load_row_smem<NCH>(w, st + (size_t)k * row_bytes, H, lane);
                d[k] = dot_rows<NCH>(w, xn);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int k = 0; k < kLmRowsPerStage; ++k) d[k] += __shfl_xor_sync(0xffffffffu, d[k], o);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
#pragma unroll
        for (int k = 0; k < kLmRowsPerStage; ++k)
            if (k < rows) {
                if (d[k] > best) { best = d[k]; best_i = row + k; }  // rows ascend within a warp: ties keep the lower
                if (c.logits && lane == 0) c.logits[row + k] = d[k];
            }
    }
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    constexpr int NT = kLmWarps * 32;
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    if (threadIdx.x == 0) {
        float bv = s_val[0];
        int bi = s_idx[0];
        for (int w = 1; w < kLmWarps; ++w)
            if (s_val[w] > bv || (s_val[w] == bv && s_idx[w] < bi)) { bv = s_val[w]; bi = s_idx[w]; }
        c.lm_val[blockIdx.x] = bv;
        c.lm_idx[blockIdx.x] = bi;
        __threadfence();
        const int old = atomicAdd(&c.tickets[0], 1);
        if (old == G - 1) {
            c.tickets[0] = 0;
            __threadfence();
            float fv = -INFINITY;
            int fi = 0x7fffffff;
            for (int b = 0; b < G; ++b) {
                const float v = __ldcg(c.lm_val + b);
                const int ix = __ldcg(c.lm_idx + b);
                if (v > fv || (v == fv && ix < fi)) { fv = v; fi = ix; }
            }
            if (fi == 0x7fffffff) fi = 0;
            *c.token = fi;  // input of the next step
            c.seq_len[c.slot] = __ldcg(c.seq_len + c.slot) + 1;
            if (c.out_tokens) {
                const int st = __ldcg(c.step_counter);
                c.out_tokens[st] = fi;
                *c.step_counter = st + 1;
            }
        }
    }
}

}  // namespace

bool bs1_supported(int H, int I, int hd, int nh, int nkv) {
    return H % 8 == 0 && H <= 2048 && (hd == 64 || hd == 128) && nh * hd == H && nh % nkv == 0 && nh / nkv <= 8 && I > 0;
}
size_t bs1_ffn_part_floats(int H, int num_sms) {
    return (size_t)(num_sms + (num_sms + kFfnGroup - 1) / kFfnGroup + 1) * H;
}

namespace {

inline int nch_of(int H) { return (H / 8 + 31) / 32; }

}  // namespace

#define TFFN_NCH_SWITCH(H, STMT)          \
    switch (nch_of(H)) {                  \
        case 1: { constexpr int NCH = 1; STMT; break; } \
        case 2: { constexpr int NCH = 2; STMT; break; } \
        case 3: { constexpr int NCH = 3; STMT; break; } \
        case 4: { constexpr int NCH = 4; STMT; break; } \
        case 5: { constexpr int NCH = 5; STMT; break; } \
        case 6: { constexpr int NCH = 6; STMT; break; } \
        case 7: { constexpr int NCH = 7; STMT; break; } \
        case 8: { constexpr int NCH = 8; STMT; break; } \
        default: break;                   \
    }

int bs1_prepare(int H, bool expert) {
    // the larger of the two FFN layouts covers sessions with and without an expert
    const size_t ffn = ffn_smem_layout(H, expert).total > ffn_smem_layout(H, false).total ? ffn_smem_layout(H, expert).total
                                                                                          : ffn_smem_layout(H, false).total;
    const size_t lm = lm_smem_layout(H).total;
    cudaError_t e1 = cudaSuccess, e2 = cudaSuccess;
    TFFN_NCH_SWITCH(H, {
        e1 = cudaFuncSetAttribute(k_bs1_ffn<NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ffn);
        e2 = cudaFuncSetAttribute(k_bs1_lmhead<NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lm);
    });
    return e1 != cudaSuccess ? (int)e1 : (int)e2;
}

void launch_bs1_qkv(const Bs1Ctx& c, const Bs1Layer& ly, const bf16* embed, KvView kv, int layer, bool first,
                    cudaStream_t s, bool pdl) {
    const int units = (c.nh + 2 * c.nkv) * (c.hd / 2);
    dim3 grid((units + kRowWarps - 1) / kRowWarps), block(kRowWarps * 32);
    TFFN_NCH_SWITCH(c.H, launch_k(k_bs1_qkv<NCH>, grid, block, 0, s, pdl, c, ly, embed, kv, layer, (int)first));
}
void launch_bs1_oproj(const Bs1Ctx& c, const Bs1Layer& ly, cudaStream_t s, bool pdl) {
    dim3 grid((c.H + kRowWarps * 2 - 1) / (kRowWarps * 2)), block(kRowWarps * 32);
    TFFN_NCH_SWITCH(c.H, launch_k(k_bs1_oproj<NCH>, grid, block, 0, s, pdl, c, ly));
}
void launch_bs1_ffn(const Bs1Ctx& c, const Bs1Layer& ly, cudaStream_t s, bool pdl) {
    const FfnSmem L = ffn_smem_layout(c.H, ly.ffn_expert != nullptr);
    int G = c.num_sms < c.I ? c.num_sms : c.I;
    dim3 grid(G), block(kFfnThreads);
    TFFN_NCH_SWITCH(c.H, launch_k(k_bs1_ffn<NCH>, grid, block, L.total, s, pdl, c, ly));
}
void launch_bs1_lmhead(const Bs1Ctx& c, const bf16* final_norm, const bf16* lm_head, cudaStream_t s, bool pdl) {
    const LmSmem L = lm_smem_layout(c.H);
    int G = c.num_sms;
    if (G > c.V) G = c.V;
    dim3 grid(G), block(kLmThreads);
    TFFN_NCH_SWITCH(c.H, launch_k(k_bs1_lmhead<NCH>, grid, block, L.total, s, pdl, c, final_norm, lm_head));
}

}  // namespace tffn
