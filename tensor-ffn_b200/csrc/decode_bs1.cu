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
    __shared__ __align__(16) uint8_t xs[2048 * 2];
    __shared__ float s_red[kRowWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int H = c.H, hd = c.hd, half = hd >> 1;
    const int unit = blockIdx.x * kRowWarps + warp;
    const int units = (c.nh + 2 * c.nkv) * half;
    pdl_launch_dependents();
    if (threadIdx.x == 0) tl_mark(c.tl, 0);
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
    // The position, its page and its RoPE entry were last written before this token's first kernel,
    // which is a full dependency: they can be fetched ahead of the dependency wait as well.
    int pos = 0, pg = 0;
    float cs = 1.f, sn = 0.f, bias0 = 0.f, bias1 = 0.f;
    if (active && lane == 0) {
        pos = __ldcg(c.seq_len + c.slot);
        if (pos >= 0 && pos < c.max_pos) {
            cs = c.rope_cos[(size_t)pos * half + i];
            sn = c.rope_sin[(size_t)pos * half + i];
            pg = __ldcg(kv.block_table + (size_t)c.slot * kv.max_pages_per_seq + pos / kPageTokens);
        }
        if (ly.bqkv) {
            bias0 = __bfloat162float(ly.bqkv[head * hd + i]);
            bias1 = __bfloat162float(ly.bqkv[head * hd + i + half]);
        }
    }
    if (warp == 0) pdl_wait();  // one waiting warp per CTA, see k_bs1_ffn
    __syncthreads();
    if (threadIdx.x == 0) tl_mark(c.tl, 1);
    const bf16* hsrc = c.h_in;
    if (first) {
        int tok = __ldcg(c.token);
        if (tok < 0 || tok >= c.V) {
            if (threadIdx.x == 0 && blockIdx.x == 0) dev_fail(c.status, DEV_ERR_BOUNDS);
            tok = 0;
        }
        hsrc = embed + (size_t)tok * H;
    }
    // The residual stream of this layer = the previous one + the sums its FFN left; block 0 publishes it
    // for the o_proj and FFN kernels, the last block clears the accumulator this layer's FFN will add to
    // (its previous reader, the q|k|v kernel of the layer before, has long finished).
    fold_norm_block<kRowWarps * 32>(hsrc, first ? nullptr : c.acc_in, ly.attn_norm, H, c.eps, blockIdx.x == 0 ? c.h : nullptr, xs,
                                    s_red, (int)threadIdx.x, [] { __syncthreads(); });
    if (blockIdx.x == gridDim.x - 1 && c.acc_out)
        for (int k = threadIdx.x; k < kAccReplicas * H; k += kRowWarps * 32) c.acc_out[k] = 0;
    if (threadIdx.x == 0) tl_mark(c.tl, 2);  // the warps' remaining work is a dot product and a store
    if (!active) return;
    RowRegs<NCH> xn;
    load_row_smem<NCH>(xn, xs, H, lane);
    float d0 = warp_sum(dot_rows<NCH>(w0, xn));
    float d1 = warp_sum(dot_rows<NCH>(w1, xn));
    if (lane != 0) return;
    if (pos < 0 || pos >= c.max_pos) {
        dev_fail(c.status, DEV_ERR_BOUNDS);
        return;
    }
    float x0 = bf16_round(d0), x1 = bf16_round(d1);
    if (ly.bqkv) {
        x0 = bf16_round(x0 + bias0);
        x1 = bf16_round(x1 + bias1);
    }
    const int nh = c.nh, nkv = c.nkv;
    if (head < nh + nkv) {
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
    if (threadIdx.x == 0) tl_mark(c.tl, 0);
    RowRegs<NCH> w0, w1;
    if (n0 < H) load_row<NCH>(w0, ly.wo + (size_t)n0 * H, H, lane);
    if (n0 + 1 < H) load_row<NCH>(w1, ly.wo + (size_t)(n0 + 1) * H, H, lane);
    if (warp == 0) pdl_wait();  // one waiting warp per CTA, see k_bs1_ffn
    __syncthreads();
    if (threadIdx.x == 0) tl_mark(c.tl, 1);
    if (n0 >= H) return;
    RowRegs<NCH> x;
    load_row_act<NCH>(x, c.ctx, H, lane);
    // the old residual values travel together with ctx: one trip to L2 instead of two in a row
    const float h0 = lane == 0 ? ld_bf16_cg(c.h + n0) : 0.f;
    const float h1 = (lane == 0 && n0 + 1 < H) ? ld_bf16_cg(c.h + n0 + 1) : 0.f;
    float d0 = warp_sum(dot_rows<NCH>(w0, x));
    float d1 = (n0 + 1 < H) ? warp_sum(dot_rows<NCH>(w1, x)) : 0.f;
    if (lane == 0) {
        c.h[n0] = __float2bfloat16_rn(h0 + d0);
        if (n0 + 1 < H) c.h[n0 + 1] = __float2bfloat16_rn(h1 + d1);
    }
    if (threadIdx.x == 0) tl_mark(c.tl, 2);
}

// ------------------------------------------------------------------------------------------ fused SwiGLU
// Consumer warps; warp kFfnWarps is the copy producer. A warp takes a chunk of up to four records at a time
// (fewer when the ring is short, see the kernel).
constexpr int kFfnWarps = 9;
constexpr int kFfnThreads = (kFfnWarps + 1) * 32;
constexpr int kSmsLeftToAttention = 4;

struct FfnSmem {
    int stages;
    size_t stage_bytes;
    size_t ring_off, part_off, xs_off, bar_off, total;
};
// One stage holds one record of the base FFN and, next to it, the same record of the expert. Stages
// are not tied to warps: the producer publishes how many records it has issued, and a consumer polls a
// stage's barrier only once its record has been issued (see item_ready). The per-warp partial sums
// reuse the ring once every record has been consumed.
__host__ __device__ inline FfnSmem ffn_smem_layout(int H, bool expert) {
    FfnSmem s;
    s.stage_bytes = (size_t)H * 2 * 3 * (expert ? 2 : 1);
    const size_t part = (size_t)kFfnWarps * H * 4;
    const size_t budget = 200 * 1024;
    int st = (int)(budget / s.stage_bytes);
    if (st > 32) st = 32;
    if (st < 8) st = 8;
    s.stages = st;
    s.ring_off = 0;
    s.part_off = 0;
    size_t ring = s.stage_bytes * st;
    if (ring < part) ring = part;
    s.xs_off = (ring + 127) / 128 * 128;
    s.bar_off = s.xs_off + ((size_t)H * 2 + 127) / 128 * 128;
    s.total = s.bar_off + (size_t)st * 16 + 64;
    return s;
}

// Bounded wait until the producer has issued item `q` (it publishes the count in shared memory). Only
// then may a consumer poll the stage's barrier: a parity wait started before the stage's previous
// occupant has even landed would see the phase before that one and report "complete".
__device__ __forceinline__ bool item_issued(const int* s_issued, int q, int* status) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (*(volatile const int*)s_issued > q) return true;
        if (i > 64) __nanosleep(32);
    }
    dev_fail(status, DEV_ERR_FULL_WAIT);
    return false;
}

// act = bf16(silu(bf16(x.Wg)) * bf16(x.Wu)); out = act.Wd (fp32); expert identical, its fp32
// result scaled by output_scale; ffn = base + expert in fp32; h = bf16(float(h) + ffn)
// (inference/src/model/qwen.cu:422-447, inference/src/model/expert.cu:44-59).
// A warp takes four records at a time: their gate and up rows (16 with the expert, 8 without) are the
// rows of one tensor-core GEMV against the normalised activations; the down columns are then added with
// packed fp32 FMAs into the warp's running sums for all H outputs.
template <int NCH>
__global__ void __launch_bounds__(kFfnThreads, 1) k_bs1_ffn(Bs1Ctx c, Bs1Layer ly) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int H = c.H, I = c.I;
    const bool expert = ly.ffn_expert != nullptr;
    const FfnSmem L = ffn_smem_layout(H, expert);
    uint8_t* ring = smem + L.ring_off;
    float* part = (float*)(smem + L.part_off);
    uint8_t* xs = smem + L.xs_off;
    uint64_t* full = (uint64_t*)(smem + L.bar_off);
    uint64_t* empty = full + L.stages;
    int* s_flag = (int*)(empty + L.stages);
    int* s_issued = s_flag + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x;
    const int i0 = (int)(((long long)I * blockIdx.x) / G), i1 = (int)(((long long)I * (blockIdx.x + 1)) / G);
    const int nrec = i1 - i0;
    const size_t rec_bytes = (size_t)H * 6;
    const int S = L.stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        *s_issued = 0;
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        BS1_TRACE(c, 0);
        tl_mark(c.tl, 0);
    }

    if (warp == kFfnWarps) {
        // producer: the weights do not depend on the previous kernel, so no griddepcontrol.wait here
        if (lane == 0) {
            for (int r = 0; r < nrec; ++r) {
                const int s = r % S;
                const uint32_t ph = (uint32_t)(r / S) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, c.status, DEV_ERR_EMPTY_WAIT)) break;
                uint8_t* dst = ring + (size_t)s * L.stage_bytes;
                mbar_arrive_expect_tx(&full[s], (uint32_t)L.stage_bytes);
                __threadfence_block();
                *(volatile int*)s_issued = r + 1;
                bulk_g2s(dst, (const uint8_t*)ly.ffn_base + (size_t)(i0 + r) * rec_bytes, (uint32_t)rec_bytes, &full[s]);
                if (expert)
                    bulk_g2s(dst + rec_bytes, (const uint8_t*)ly.ffn_expert + (size_t)(i0 + r) * rec_bytes,
                             (uint32_t)rec_bytes, &full[s]);
            }
        }
        return;
    }

    // consumers: one warp waits for the previous kernel, the others follow through the CTA barrier
    constexpr int NT = kFfnWarps * 32;
    if (warp == 0) pdl_wait();
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    {
        RowRegs<NCH> xn;
        rmsnorm_regs<NCH>(xn, c.h, ly.ffn_norm, H, c.eps, lane);
        if (warp == 0) {
#pragma unroll
            for (int j = 0; j < NCH; ++j) {
                const int ch = lane + 32 * j;
                if (ch < (H >> 3)) ((uint4*)xs)[ch] = xn.v[j];
            }
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    if (threadIdx.x == 0) {
        BS1_TRACE(c, 1);
        tl_mark(c.tl, 1);
    }
    unsigned long long acc[NCH * 4];
#pragma unroll
    for (int j = 0; j < NCH * 4; ++j) acc[j] = 0ull;
    const size_t row_bytes = (size_t)H * 2;
    const int g = lane >> 2;
    // the MMA rows this lane loads: with the expert, row g = (record g / 4, {gate_b, up_b, gate_e, up_e}[g % 4])
    // and row g + 8 the same of record 2 + g / 4; without it, row g = (record g / 2, {gate, up}[g % 2])
    const int j_lo = expert ? (g >> 2) : (g >> 1), j_hi = 2 + (g >> 2);
    const size_t koff = expert ? (size_t)(g & 1) * row_bytes + (size_t)((g >> 1) & 1) * rec_bytes : (size_t)(g & 1) * row_bytes;
    // Records per chunk. The ring holds S consecutive records, so only S / CH chunks can be worked on at a
    // time: with four records per chunk a ring of 19 stages (hidden 896) keeps fewer than five of the nine
    // warps busy, one of 8 (hidden 2048) two. Smaller chunks use a part of the 16 MMA rows only (the unused
    // rows repeat the chunk's last record and are dropped), which costs less than idle warps.
    const int CH = S >= 4 * kFfnWarps ? 4 : (S >= 2 * kFfnWarps ? 2 : 1);
    const int nchunks = (nrec + CH - 1) / CH;
    const int nchunk16 = H >> 3;
    bool ok = true;
    for (int ch = warp; ch < nchunks && ok; ch += kFfnWarps) {
        const int r0 = ch * CH, nr = min(CH, nrec - r0);
        for (int j = 0; j < nr && ok; ++j) {
            const int r = r0 + j;
            ok = item_issued(s_issued, r, c.status) && mbar_wait(&full[r % S], (uint32_t)(r / S) & 1u, c.status, DEV_ERR_FULL_WAIT);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (threadIdx.x == 0 && ch == 0) BS1_TRACE(c, 2);
        // records past the end of this CTA's slice stand in as copies of the last one; their results are dropped
        auto stage_of = [&](int j) { return ring + (size_t)((r0 + min(j, nr - 1)) % S) * L.stage_bytes; };
        float v_lo, v_hi = 0.f;
        // with the expert, chunks of one or two records fill the lower eight MMA rows only: the upper half then
        // stays empty instead of loading copies
        if (expert && CH > 2) mma_rows_dot<true>(stage_of(j_lo) + koff, stage_of(j_hi) + koff, H, xs, lane, v_lo, v_hi);
        else mma_rows_dot<false>(stage_of(j_lo) + koff, nullptr, H, xs, lane, v_lo, v_hi);
        // a gate row and its up row are neighbours in g: lane ^ 4
        const float p_lo = __shfl_xor_sync(0xffffffffu, v_lo, 4), p_hi = __shfl_xor_sync(0xffffffffu, v_hi, 4);
        const float a_lo = silu_mul_bf16(v_lo, p_lo), a_hi = silu_mul_bf16(v_hi, p_hi);  // meaningful where g is even
        float act_b[4], act_e[4];
        if (expert) {
            act_b[0] = __shfl_sync(0xffffffffu, a_lo, 0);
            act_e[0] = __shfl_sync(0xffffffffu, a_lo, 8);
            act_b[1] = __shfl_sync(0xffffffffu, a_lo, 16);
            act_e[1] = __shfl_sync(0xffffffffu, a_lo, 24);
            act_b[2] = __shfl_sync(0xffffffffu, a_hi, 0);
            act_e[2] = __shfl_sync(0xffffffffu, a_hi, 8);
            act_b[3] = __shfl_sync(0xffffffffu, a_hi, 16);
            act_e[3] = __shfl_sync(0xffffffffu, a_hi, 24);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                act_b[j] = __shfl_sync(0xffffffffu, a_lo, 8 * j);
                act_e[j] = 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (j < nr) {
                const uint8_t* st = ring + (size_t)((r0 + j) % S) * L.stage_bytes;
                const unsigned long long ab = splat_f32x2(act_b[j]);
                const uint4* db = (const uint4*)(st + 2 * row_bytes);
#pragma unroll
                for (int jj = 0; jj < NCH; ++jj) {
                    const int c16 = lane + 32 * jj;
                    if (c16 < nchunk16) {
                        const uint4 d = db[c16];
                        axpy_bf16x2(acc[jj * 4 + 0], ab, d.x);
                        axpy_bf16x2(acc[jj * 4 + 1], ab, d.y);
                        axpy_bf16x2(acc[jj * 4 + 2], ab, d.z);
                        axpy_bf16x2(acc[jj * 4 + 3], ab, d.w);
                    }
                }
                if (expert) {
                    const unsigned long long ae = splat_f32x2(act_e[j] * c.expert_scale);
                    const uint4* de = (const uint4*)(st + rec_bytes + 2 * row_bytes);
#pragma unroll
                    for (int jj = 0; jj < NCH; ++jj) {
                        const int c16 = lane + 32 * jj;
                        if (c16 < nchunk16) {
                            const uint4 d = de[c16];
                            axpy_bf16x2(acc[jj * 4 + 0], ae, d.x);
                            axpy_bf16x2(acc[jj * 4 + 1], ae, d.y);
                            axpy_bf16x2(acc[jj * 4 + 2], ae, d.z);
                            axpy_bf16x2(acc[jj * 4 + 3], ae, d.w);
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane < nr) mbar_arrive(&empty[(r0 + lane) % S]);
    }
    if (threadIdx.x == 0) BS1_TRACE(c, 3);
    // fold the consumer warps of this CTA (fixed order); the partial sums reuse the ring, so
    // every consumer must be done reading it first
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        const int ch = lane + 32 * j;
        if (ch < nchunk16) {
            float4* dst = (float4*)(part + (size_t)warp * H + ch * 8);
            const float2 p0 = unpack_f32x2(acc[j * 4]), p1 = unpack_f32x2(acc[j * 4 + 1]);
            const float2 p2 = unpack_f32x2(acc[j * 4 + 2]), p3 = unpack_f32x2(acc[j * 4 + 3]);
            dst[0] = make_float4(p0.x, p0.y, p1.x, p1.y);
            dst[1] = make_float4(p2.x, p2.y, p3.x, p3.y);
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    // This CTA's sums join the layer's accumulator as fixed-point integers: fire-and-forget atomics, no
    // ticket, no fence, no CTA waits for another. Integer addition is associative, so the total does
    // not depend on arrival order and the step stays bit-reproducible. Whoever reads the residual stream
    // next (the q|k|v kernel of the next layer, the LM head) adds the total in.
    unsigned long long* acc_out = (unsigned long long*)c.acc_out + (size_t)(blockIdx.x % kAccReplicas) * H;
    for (int col = threadIdx.x; col < H; col += NT) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kFfnWarps; ++w) s += part[(size_t)w * H + col];
        atomicAdd(acc_out + col, (unsigned long long)__float2ll_rn(s * kAccScale));
    }
    if (threadIdx.x == 0) {
        BS1_TRACE(c, 4);
        tl_mark(c.tl, 2);
    }
}

// closes a stand-alone FFN launch: h = bf16(h + sums), sums cleared
__global__ void k_bs1_ffn_finalize(bf16* __restrict__ h, long long* __restrict__ acc, int H) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= H) return;
    h[i] = __float2bfloat16_rn(__bfloat162float(h[i]) + acc_value(acc, H, i));
#pragma unroll
    for (int r = 0; r < kAccReplicas; ++r) acc[(size_t)r * H + i] = 0;
}

// ------------------------------------------------------------------------------------------ LM head + argmax
constexpr int kLmWarps = 8;
constexpr int kLmThreads = (kLmWarps + 1) * 32;
struct LmSmem {
    int stages, rows;  // rows per stage: one tensor-core GEMV tile of 16 rows, or 8 (upper MMA rows empty) for wide models
    size_t stage_bytes, xs_off, bar_off, total;
};
__host__ __device__ inline LmSmem lm_smem_layout(int H) {
    LmSmem s;
    s.rows = (size_t)16 * H * 2 <= 48 * 1024 ? 16 : 8;
    s.stage_bytes = (size_t)s.rows * H * 2;
    int st = (int)((200 * 1024) / s.stage_bytes);
    if (st > 32) st = 32;
    s.stages = st;
    s.xs_off = (s.stage_bytes * st + 127) / 128 * 128;
    s.bar_off = s.xs_off + ((size_t)H * 2 + 127) / 128 * 128;
    s.total = s.bar_off + (size_t)st * 16 + 64 + kLmWarps * 8;
    return s;
}

// logits = rmsnorm(h) . E^T in fp32 (inference/src/model/qwen.cu:451-454); greedy pick = first
// index of the strict maximum (inference/src/main.cpp:45-51). Stages of eight rows go round robin to
// the consumer warps; a stage is one tensor-core GEMV against the normalised activations.
template <int NCH>
__global__ void __launch_bounds__(kLmThreads, 1) k_bs1_lmhead(Bs1Ctx c, const bf16* __restrict__ final_norm,
                                                              const bf16* __restrict__ lm_head) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int H = c.H, V = c.V;
    const LmSmem L = lm_smem_layout(H);
    const int S = L.stages;
    uint8_t* xs = smem + L.xs_off;
    uint64_t* full = (uint64_t*)(smem + L.bar_off);
    uint64_t* empty = full + S;
    int* s_flag = (int*)(empty + S);
    int* s_issued = s_flag + 1;
    float* s_val = (float*)(s_flag + 2);
    int* s_idx = (int*)(s_val + kLmWarps);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x;
    const int r0 = (int)(((long long)V * blockIdx.x) / G), r1 = (int)(((long long)V * (blockIdx.x + 1)) / G);
    const int RS = L.rows;
    const int nst = (r1 - r0 + RS - 1) / RS;
    const size_t row_bytes = (size_t)H * 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        *s_issued = 0;
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    if (threadIdx.x == 0) tl_mark(c.tl, 0);

    if (warp == kLmWarps) {
        if (lane == 0) {
            for (int r = 0; r < nst; ++r) {
                const int s = r % S;
                const uint32_t ph = (uint32_t)(r / S) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, c.status, DEV_ERR_EMPTY_WAIT)) break;
                const int row = r0 + r * RS;
                const int rows = min(RS, r1 - row);
                const uint32_t bytes = (uint32_t)(rows * row_bytes);
                mbar_arrive_expect_tx(&full[s], bytes);
                __threadfence_block();
                *(volatile int*)s_issued = r + 1;
                bulk_g2s(smem + (size_t)s * L.stage_bytes, (const uint8_t*)lm_head + (size_t)row * row_bytes, bytes, &full[s]);
            }
        }
        return;
    }

    constexpr int NT = kLmWarps * 32;
    if (warp == 0) pdl_wait();  // one waiting warp per CTA, see k_bs1_ffn
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    // final residual add (the last layer's FFN sums) + final RMSNorm, by the consumer threads together
    fold_norm_block<NT>(c.h_in, c.acc_in, final_norm, H, c.eps, nullptr, xs, s_val, (int)threadIdx.x,
                        [] { asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory"); });
    if (threadIdx.x == 0) tl_mark(c.tl, 1);
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    const int g = lane >> 2;
    bool ok = true;
    for (int r = warp; r < nst && ok; r += kLmWarps) {
        const int s = r % S;
        const uint32_t ph = (uint32_t)(r / S) & 1u;
        ok = __all_sync(0xffffffffu, item_issued(s_issued, r, c.status) && mbar_wait(&full[s], ph, c.status, DEV_ERR_FULL_WAIT));
        if (!ok) break;
        const uint8_t* st = smem + (size_t)s * L.stage_bytes;
        float d, d_up = 0.f;
        if (RS == 16) mma_rows_dot<true>(st + (size_t)g * row_bytes, st + (size_t)(g + 8) * row_bytes, H, xs, lane, d, d_up);
        else mma_rows_dot<false>(st + (size_t)g * row_bytes, nullptr, H, xs, lane, d, d_up);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        const int row = r0 + r * RS + g;  // rows past the slice's end hold stale data: ignored
        if (row < r1) {
            if (d > best) { best = d; best_i = row; }  // a lane's rows ascend: ties keep the lower index
            if (c.logits && (lane & 3) == 0) c.logits[row] = d;
        }
        if (RS == 16 && row + 8 < r1) {
            if (d_up > best) { best = d_up; best_i = row + 8; }
            if (c.logits && (lane & 3) == 0) c.logits[row + 8] = d_up;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
    if (threadIdx.x == 0) {
        float bv = s_val[0];
        int bi = s_idx[0];
        for (int w = 1; w < kLmWarps; ++w)
            if (s_val[w] > bv || (s_val[w] == bv && s_idx[w] < bi)) { bv = s_val[w]; bi = s_idx[w]; }
        c.lm_val[blockIdx.x] = bv;
        c.lm_idx[blockIdx.x] = bi;
        tl_mark(c.tl, 2);
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
    return H % 64 == 0 && H <= 2048 && (hd == 64 || hd == 128) && nh * hd == H && nh % nkv == 0 && nh / nkv <= 8 && I > 0;
}
size_t bs1_acc_words(int H) { return (size_t)kAccReplicas * H; }
void launch_bs1_ffn_finalize(bf16* h, long long* acc, int H, cudaStream_t s) {
    k_bs1_ffn_finalize<<<(H + 255) / 256, 256, 0, s>>>(h, acc, H);
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
        // one carveout for every kernel of the step, so that they can be resident together
        if (e1 == cudaSuccess) e1 = prefer_max_shared(k_bs1_ffn<NCH>);
        if (e1 == cudaSuccess) e1 = prefer_max_shared(k_bs1_qkv<NCH>);
        if (e1 == cudaSuccess) e1 = prefer_max_shared(k_bs1_oproj<NCH>);
        if (e2 == cudaSuccess) e2 = prefer_max_shared(k_bs1_lmhead<NCH>);
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
    // Every kernel of a layer is resident at once (dependent launches). An attention CTA and an FFN CTA do
    // not fit on one SM together, so a grid of one CTA per SM would leave the CTAs that land behind the
    // attention's without their head start on the weight stream: keep a few SMs out of the grid.
    int G = c.num_sms > 32 ? c.num_sms - kSmsLeftToAttention : c.num_sms;
    if (G > c.I) G = c.I;
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
