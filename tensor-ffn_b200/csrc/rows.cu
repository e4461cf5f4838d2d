// Row-wise kernels of the batched path and load-time helpers. Each states the reference
// kernel whose arithmetic (and rounding points) it reproduces.
#include "kernels.h"
#include "ptx.cuh"
#include "launch.h"

namespace tffn {

namespace {

// h[t,:] = table[tokens[t],:]  (k_embed, inference/src/model/qwen.cu:216-220); ids are bounds-checked.
__global__ void k_embed_rows(const int* __restrict__ tokens, const bf16* __restrict__ table, bf16* __restrict__ h, int T,
                             int H, int V, int* status, unsigned long long* tl) {
    if (threadIdx.x == 0) tl_mark(tl, 0);
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) tl_mark(tl, 1);
    int t = blockIdx.x;
    int tok = __ldcg(tokens + t);
    if (tok < 0 || tok >= V) {
        if (threadIdx.x == 0) dev_fail(status, DEV_ERR_BOUNDS);
        tok = 0;
    }
    const uint4* src = (const uint4*)(table + (size_t)tok * H);
    uint4* dst = (uint4*)(h + (size_t)t * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = __ldg(src + i);
    if (threadIdx.x == 0) tl_mark(tl, 2);
}

// out = bf16(float(x) * rsqrt(mean(x^2) + eps) * float(w))  (k_rmsnorm, inference/src/backend/cuda_ops.cu:75-96)
__global__ void __launch_bounds__(128) k_rmsnorm_rows(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                      bf16* __restrict__ out, int H, float eps,
                                                      const int* __restrict__ row_idx, unsigned long long* tl) {
    if (threadIdx.x == 0) tl_mark(tl, 0);
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) tl_mark(tl, 1);
    const int r = blockIdx.x;
    const int src_row = row_idx ? row_idx[r] : r;
    const uint4* xr = (const uint4*)(x + (size_t)src_row * H);
    // The first 128 16-byte pieces of the row (all of it up to H = 1024) and of the norm weights stay in
    // registers between the two passes; both loads are in flight together.
    const int n16 = H / 8;
    const uint4* wr = (const uint4*)w;
    const bool own = (int)threadIdx.x < n16;
    const uint4 v0 = own ? __ldcg(xr + threadIdx.x) : make_uint4(0, 0, 0, 0);
    const uint4 g0 = own ? __ldg(wr + threadIdx.x) : make_uint4(0, 0, 0, 0);
    float ss = 0.f;
    auto sq = [&](const uint4& q) {
        const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a = bf16_lo(u[j]), b = bf16_hi(u[j]);
            ss += a * a + b * b;
        }
    };
    sq(v0);
    for (int i = threadIdx.x + 128; i < n16; i += 128) sq(__ldcg(xr + i));
    __shared__ float red[4];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = red[0] + red[1] + red[2] + red[3];
    const float rinv = rsqrtf(ss / (float)H + eps);
    uint4* orow = (uint4*)(out + (size_t)r * H);
    auto scale = [&](const uint4& q, const uint4& g) {
        const uint32_t u[4] = {q.x, q.y, q.z, q.w}, gw[4] = {g.x, g.y, g.z, g.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a = bf16_lo(u[j]) * rinv * bf16_lo(gw[j]);
            const float b = bf16_hi(u[j]) * rinv * bf16_hi(gw[j]);
            o[j] = (uint32_t)bf16_bits(a) | ((uint32_t)bf16_bits(b) << 16);
        }
        return make_uint4(o[0], o[1], o[2], o[3]);
    };
    if (own) orow[threadIdx.x] = scale(v0, g0);
    for (int i = threadIdx.x + 128; i < n16; i += 128) orow[i] = scale(__ldcg(xr + i), __ldg(wr + i));
    if (threadIdx.x == 0) tl_mark(tl, 2);
}

// greedy pick: first index of the strict maximum (sample(), inference/src/main.cpp:45-51).
// grid (rows, S): block (r, s) scans slice s of row r; the last block of a row to finish (a ticket, no
// spinning) combines the S partial results, so the pick does not depend on scheduling.
__device__ __forceinline__ void argmax_take(float& best, int& bi, float v, int i) {
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
}
__global__ void __launch_bounds__(256) k_argmax_rows(const float* __restrict__ logits, int V, int S, int* __restrict__ out,
                                                      float* __restrict__ scratch, int* __restrict__ counters,
                                                      unsigned long long* tl) {
    if (threadIdx.x == 0) tl_mark(tl, 0);
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) tl_mark(tl, 1);
    const int r = blockIdx.x, s = blockIdx.y;
    const float* row = logits + (size_t)r * V;
    const int chunk = (((V + S - 1) / S) + 3) & ~3;
    const int v0 = s * chunk, v1 = min(V, v0 + chunk);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    if ((V & 3) == 0) {
        for (int i = v0 + threadIdx.x * 4; i < v1; i += 256 * 4) {  // v1 - v0 is a multiple of 4 here
            const float4 v = __ldcg((const float4*)(row + i));
            argmax_take(best, bi, v.x, i);
            argmax_take(best, bi, v.y, i + 1);
            argmax_take(best, bi, v.z, i + 2);
            argmax_take(best, bi, v.w, i + 3);
        }
    } else {
        for (int i = v0 + threadIdx.x; i < v1; i += 256) argmax_take(best, bi, __ldcg(row + i), i);
    }
    // NaN-free inputs assumed; if every value is -inf the lowest index 0 wins below
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ int s_last;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) argmax_take(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < 8 ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < 8 ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) argmax_take(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (threadIdx.x == 0) {
            if (S == 1) {
                out[r] = (bi == 0x7fffffff) ? 0 : bi;
                s_last = 0;
            } else {
                scratch[((size_t)r * S + s) * 2] = best;
                scratch[((size_t)r * S + s) * 2 + 1] = __int_as_float(bi);
                __threadfence();
                const int old = atomicAdd(&counters[r], 1);
                s_last = (old == S - 1);
                if (s_last) counters[r] = 0;
            }
        }
    }
    __syncthreads();
    if (s_last && threadIdx.x < 32) {
        __threadfence();
        best = -INFINITY;
        bi = 0x7fffffff;
        for (int z = threadIdx.x; z < S; z += 32)
            argmax_take(best, bi, __ldcg(scratch + ((size_t)r * S + z) * 2), __float_as_int(__ldcg(scratch + ((size_t)r * S + z) * 2 + 1)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) argmax_take(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (threadIdx.x == 0) out[r] = (bi == 0x7fffffff) ? 0 : bi;
    }
    if (threadIdx.x == 0) tl_mark(tl, 2);
}

// second half of the greedy pick when the LM-head GEMM left per-tile maxima: one block per row
// (pack: optional {value, idx_offset + index} per row for the exchange between tensor-parallel ranks)
__global__ void __launch_bounds__(256) k_argmax_tiles(const float* __restrict__ val, const int* __restrict__ idx, int tiles,
                                                       int* __restrict__ out, unsigned long long* tl, float2* __restrict__ pack,
                                                       int idx_offset) {
    if (threadIdx.x == 0) tl_mark(tl, 0);
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) tl_mark(tl, 1);
    const int r = blockIdx.x;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < tiles; i += 256)
        argmax_take(best, bi, __ldcg(val + (size_t)r * tiles + i), __ldcg(idx + (size_t)r * tiles + i));
    __shared__ float sv[8];
    __shared__ int si[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) argmax_take(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < 8 ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < 8 ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) argmax_take(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (threadIdx.x == 0) {
            out[r] = (bi == 0x7fffffff) ? 0 : bi;
            if (pack) pack[r] = make_float2(best, __int_as_float(bi == 0x7fffffff ? 0x7fffffff : bi + idx_offset));
            tl_mark(tl, 2);
        }
    }
}

// Tensor parallel: the ranks' candidates {maximum of the rank's vocabulary slice, its global index} ->
// the pick: the largest value, the lowest index among equal values (inference/src/main.cpp:45-51).
__global__ void k_tp_pick(const float2* __restrict__ cand, int ranks, int R, int* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int k = 0; k < ranks; ++k) {
        const float2 c = __ldcg(cand + (size_t)k * R + r);
        argmax_take(best, bi, c.x, __float_as_int(c.y));
    }
    out[r] = (bi == 0x7fffffff) ? 0 : bi;
}

// h = bf16(float(h) + sum) for one row (the residual add of inference/src/model/qwen.cu:282-285) and, when w
// is given, the RMSNorm of the new row (inference/src/backend/cuda_ops.cu:75-96) in the same pass; `sum4(i)`
// returns the four fp32 addends of columns i .. i+3. Block of kRowNormThreads threads (one pass over rows of
// up to 4096 columns, so that all of a thread's loads are in flight at once: they may cross NVLink), H a
// multiple of 4. Shared by the two tensor-parallel row kernels so that they round alike whichever way the
// partial sums travelled.
constexpr int kRowNormThreads = 1024;
template <typename Sum4>
__device__ __forceinline__ void residual_norm_row(bf16* __restrict__ hr, const bf16* __restrict__ w, bf16* __restrict__ outr, int H,
                                                  float eps, float* s_red, Sum4 sum4) {
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < H; i += kRowNormThreads * 4) {
        const float4 acc = sum4(i);
        const uint2 hv = *(const uint2*)(hr + i);
        const float a = bf16_round(bf16_lo(hv.x) + acc.x), b = bf16_round(bf16_hi(hv.x) + acc.y);
        const float c = bf16_round(bf16_lo(hv.y) + acc.z), d = bf16_round(bf16_hi(hv.y) + acc.w);
        *(uint2*)(hr + i) = make_uint2((uint32_t)bf16_bits(a) | ((uint32_t)bf16_bits(b) << 16),
                                       (uint32_t)bf16_bits(c) | ((uint32_t)bf16_bits(d) << 16));
        ss += a * a + b * b + c * c + d * d;
    }
    if (!w) return;
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < kRowNormThreads / 32; ++k) tot += s_red[k];
    const float rinv = rsqrtf(tot / (float)H + eps);
    for (int i = threadIdx.x * 4; i < H; i += kRowNormThreads * 4) {  // each thread re-reads only what it wrote itself
        const uint2 hv = *(const uint2*)(hr + i);
        const uint2 wv = __ldg((const uint2*)(w + i));
        const float x0 = bf16_lo(hv.x) * rinv * bf16_lo(wv.x), x1 = bf16_hi(hv.x) * rinv * bf16_hi(wv.x);
        const float x2 = bf16_lo(hv.y) * rinv * bf16_lo(wv.y), x3 = bf16_hi(hv.y) * rinv * bf16_hi(wv.y);
        *(uint2*)(outr + i) = make_uint2((uint32_t)bf16_bits(x0) | ((uint32_t)bf16_bits(x1) << 16),
                                         (uint32_t)bf16_bits(x2) | ((uint32_t)bf16_bits(x3) << 16));
    }
}

// Tensor parallel, launches that went through NCCL: delta = the all-reduced fp32 sum of the ranks' projection
// outputs. One block per row.
__global__ void __launch_bounds__(kRowNormThreads) k_residual_norm_rows(bf16* __restrict__ h, const float* __restrict__ delta,
                                                             const bf16* __restrict__ w, bf16* __restrict__ out, int H, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_red[kRowNormThreads / 32];
    const int r = blockIdx.x;
    const float* dr = delta + (size_t)r * H;
    residual_norm_row(h + (size_t)r * H, w, out + (size_t)r * H, H, eps, s_red, [&](int i) { return __ldcg((const float4*)(dr + i)); });
}

// ---------------------------------------------------------------- tensor parallel over peer memory
__device__ __forceinline__ void st_relaxed_sys_u32(unsigned* p, unsigned v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Hand-shake of block b with block b of every peer rank: tell them that this rank's kernels before this one
// have completed (so what they stored into this rank's own window is there to be read), then wait until
// every peer has said the same. Flags are call counters that only grow: flags[src rank][block], written by the
// source rank into the destination's window, polled here with system-scope acquire loads. The flag store is a
// relaxed system-scope store, not a release: what it announces was written to THIS GPU's memory by an earlier
// kernel, whose completion the caller's griddepcontrol.wait has already established, so it sits in this GPU's
// L2, the one place every access to this memory goes through, a peer's NVLink load included. A release would
// add a system-wide memory barrier that also waits for the unrelated weight prefetches of the co-resident next
// kernel: measured 3.7 us per exchange (10.8 -> 7.1 us), with identical results. A peer can be at most one call ahead (it needs this rank's next signal to go further), hence the
// "at least" comparison and the two alternating buffers of the callers: a rank overwrites a buffer only after
// a later hand-shake, which its peers enter only when they have finished reading it. The wait is bounded by wall
// time; when it runs out (or the step has already failed) the status word is set and the block goes on with
// whatever the slots hold, so that the kernel returns and the host reads the status.
__device__ __forceinline__ void tp_handshake(const TpPeerSync& a, int* status, unsigned* s_count) {
    const int b = blockIdx.x;
    if (threadIdx.x == 0) {
        const unsigned c0 = a.calls[b] + 1u;
        a.calls[b] = c0;
        *s_count = c0;
    }
    __syncthreads();
    const unsigned cnt = *s_count;
    const int p = (int)threadIdx.x;
    if (p < a.size && p != a.rank) {
        st_relaxed_sys_u32(a.flags_peer[p] + (size_t)a.rank * kTpFlagBlocks + b, cnt);
        const unsigned* mine = a.flags_local + (size_t)p * kTpFlagBlocks + b;
        if (__ldcg(status) == 0) {
            unsigned long long t0 = 0;
            for (unsigned i = 0;; ++i) {
                if ((int)(ld_acquire_sys_u32(mine) - cnt) >= 0) break;
                if ((i & 255u) == 255u) {
                    unsigned long long now;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                    if (t0 == 0) t0 = now;
                    if (now - t0 > a.wait_ns || i > (1u << 30)) {
                        dev_fail(status, DEV_ERR_PEER_WAIT);
                        break;
                    }
                    __nanosleep(100);
                }
            }
        }
    }
    __syncthreads();
}

// k_tp_pick over peer memory: every rank's k_argmax_tiles has left its candidates in its own window; hand-shake,
// load every rank's candidate of the row over NVLink, then the same pick on every rank.
__global__ void __launch_bounds__(128) k_tp_pick_peer(TpPickParts parts, TpPeerSync sync, int R, int* __restrict__ out, int* status) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ unsigned s_count;
    tp_handshake(sync, status, &s_count);
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    float2 c[kTpMaxRanks];
#pragma unroll
    for (int k = 0; k < kTpMaxRanks; ++k)
        if (k < sync.size)
            asm volatile("ld.relaxed.sys.global.v2.f32 {%0, %1}, [%2];" : "=f"(c[k].x), "=f"(c[k].y) : "l"(parts.part[k] + r) : "memory");
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int k = 0; k < kTpMaxRanks; ++k)
        if (k < sync.size) argmax_take(best, bi, c[k].x, __float_as_int(c[k].y));
    out[r] = (bi == 0x7fffffff) ? 0 : bi;
}

__device__ __forceinline__ float4 ld_relaxed_sys_v4(const float* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// Tensor parallel, small launches (decode): the all-reduce, the residual add and the next RMSNorm in one
// kernel, over peer memory. Every rank's projection left its fp32 partial sums in its OWN exchange window
// (plain local stores, complete and visible once that kernel has finished); after the hand-shake, which
// tells the peers exactly that, this block loads its row from every rank's window over NVLink (system-scope
// loads: nothing of an earlier exchange may be served from a cache on this side), adds the parts in rank
// order, the same order on every rank, so that all ranks keep bit-identical residual streams, then
// h = bf16(float(h) + sum) (inference/src/model/qwen.cu:282-285) and, when w is given, the RMSNorm of the new row
// (inference/src/backend/cuda_ops.cu:75-96). No rank ever stores into another rank's partial sums, so no
// store has to be fenced across GPUs. One block per row; all loads of a thread are issued before the adds.
__global__ void __launch_bounds__(kRowNormThreads) k_tp_reduce_residual_norm(bf16* __restrict__ h, TpParts parts, TpPeerSync sync,
                                                                  const bf16* __restrict__ w, bf16* __restrict__ out, int H,
                                                                  float eps, int* status, unsigned long long* tl) {
    if (threadIdx.x == 0) tl_mark(tl, 0);
    pdl_launch_dependents();
    pdl_wait();
    __shared__ unsigned s_count;
    __shared__ float s_red[kRowNormThreads / 32];
    tp_handshake(sync, status, &s_count);
    if (threadIdx.x == 0) tl_mark(tl, 1);  // the peers' parts are there: what follows is the transfer and the arithmetic
    const int r = blockIdx.x;
    const size_t row = (size_t)r * H;
    const int R = sync.size;
    residual_norm_row(h + row, w, out + row, H, eps, s_red, [&](int i) {
        float4 v[kTpMaxRanks];
#pragma unroll
        for (int p = 0; p < kTpMaxRanks; ++p)
            if (p < R) v[p] = ld_relaxed_sys_v4(parts.part[p] + row + i);
        float4 acc = v[0];
#pragma unroll
        for (int p = 1; p < kTpMaxRanks; ++p)
            if (p < R) {
                acc.x += v[p].x;
                acc.y += v[p].y;
                acc.z += v[p].z;
                acc.w += v[p].w;
            }
        return acc;
    });
    if (threadIdx.x == 0) tl_mark(tl, 2);
}

// Temperature sampling on the device, the arithmetic of sample() (inference/src/main.cpp:52-63): float
// maximum, p_i = exp((logit_i - max) / temperature) evaluated in float and summed in double, r = u * sum
// with u the canonical draw of std::uniform_real_distribution<double> (made on the host with the
// reference's std::mt19937), pick = first i whose running sum reaches r (V - 1 if none does). The running
// sum is formed per 32-element group and per warp segment instead of strictly left to right, which moves
// it by rounding errors of the order 1e-16 of the total. One block per row; u[step * rows + row].
__global__ void __launch_bounds__(1024) k_sample_rows(const float* __restrict__ logits, int V, float temperature,
                                                       const double* __restrict__ u, const int* __restrict__ step_counter,
                                                       int* __restrict__ out, unsigned long long* tl) {
    if (threadIdx.x == 0) tl_mark(tl, 0);
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) tl_mark(tl, 1);
    const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float* row = logits + (size_t)r * V;
    const int st = step_counter ? __ldcg(step_counter) : 0;
    const double uu = __ldcg(u + (size_t)st * gridDim.x + r);
    __shared__ float s_mx[32];
    __shared__ double s_seg[32];
    __shared__ int s_warp;
    float mx = -INFINITY;
    for (int i = tid; i < V; i += 1024) mx = fmaxf(mx, __ldcg(row + i));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_mx[warp] = mx;
    __syncthreads();
    mx = s_mx[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    // warp w owns the contiguous segment [w * S, (w + 1) * S), lanes interleaved inside it (coalesced)
    const int S = ((V + 31) / 32 + 31) / 32 * 32;
    const int b0 = warp * S, b1 = min(V, b0 + S);
    auto prob = [&](int i) { return i < b1 ? (double)expf((__ldcg(row + i) - mx) / temperature) : 0.0; };
    double seg = 0.0;
    for (int i = b0 + lane; i < b1; i += 32) seg += prob(i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) seg += __shfl_xor_sync(0xffffffffu, seg, o);
    if (lane == 0) s_seg[warp] = seg;
    if (tid == 0) s_warp = 32;
    __syncthreads();
    // inclusive scan of the 32 segment sums (every warp does it; cheap), total, threshold
    double incl = s_seg[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    const double total = __shfl_sync(0xffffffffu, incl, 31);
    const double rr = uu * total;
    if (warp == 0) {
        const unsigned hit = __ballot_sync(0xffffffffu, incl >= rr);
        if (lane == 0) s_warp = hit ? __ffs(hit) - 1 : 32;
    }
    __syncthreads();
    const int w_hit = s_warp;
    if (w_hit == 32) {
        if (tid == 0) out[r] = V - 1;
    } else if (warp == w_hit) {
        double acc = __shfl_sync(0xffffffffu, incl, w_hit) - s_seg[w_hit];  // running sum before this segment
        int pick = b1 - 1;  // rounding may keep the rescan just below r: then the segment's last element
        for (int i0 = b0; i0 < b1; i0 += 32) {
            double v = prob(i0 + lane);
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double t = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += t;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, acc + v >= rr && i0 + lane < b1);
            if (hit) {
                pick = i0 + __ffs(hit) - 1;
                break;
            }
            acc += __shfl_sync(0xffffffffu, v, 31);
        }
        if (lane == 0) out[r] = pick;
    }
    if (tid == 0) tl_mark(tl, 2);
}

__global__ void k_cast_f32_bf16(const float* __restrict__ src, bf16* __restrict__ dst, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = __float2bfloat16_rn(src[i]);
}

// packed[i][0][:] = gate[i,:], packed[i][1][:] = up[i,:], packed[i][2][h] = down[h, i]
__global__ void k_pack_ffn(const bf16* __restrict__ gate, const bf16* __restrict__ up, const bf16* __restrict__ down,
                           bf16* __restrict__ packed, int I, int H) {
    const int i = blockIdx.x;
    bf16* rec = packed + (size_t)i * 3 * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        rec[h] = gate[(size_t)i * H + h];
        rec[H + h] = up[(size_t)i * H + h];
        rec[2 * H + h] = down[(size_t)h * I + i];
    }
}

__global__ void k_wait_selftest(int* status) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
        // nothing ever arrives on this barrier: the bounded wait every kernel of the library uses
        // (with a short limit here) must give up, record its code and return
        mbar_wait(&bar, 0, status, DEV_ERR_TEST_WAIT, 1u << 14);
    }
}

}  // namespace

int rows_prepare() {
    cudaError_t e = prefer_max_shared(k_embed_rows);
    if (e == cudaSuccess) e = prefer_max_shared(k_rmsnorm_rows);
    if (e == cudaSuccess) e = prefer_max_shared(k_argmax_rows);
    if (e == cudaSuccess) e = prefer_max_shared(k_argmax_tiles);
    if (e == cudaSuccess) e = prefer_max_shared(k_sample_rows);
    if (e == cudaSuccess) e = prefer_max_shared(k_tp_pick);
    if (e == cudaSuccess) e = prefer_max_shared(k_residual_norm_rows);
    if (e == cudaSuccess) e = prefer_max_shared(k_tp_reduce_residual_norm);
    if (e == cudaSuccess) e = prefer_max_shared(k_tp_pick_peer);
    return (int)e;
}

void launch_embed(const int* tokens, const bf16* table, bf16* h, int T, int H, int V, int* status, cudaStream_t s, bool pdl,
                  unsigned long long* tl) {
    launch_k(k_embed_rows, dim3(T), dim3(128), 0, s, pdl, tokens, table, h, T, H, V, status, tl);
}
void launch_rmsnorm(const bf16* x, const bf16* w, bf16* out, int T, int H, float eps, const int* row_idx, cudaStream_t s,
                    bool pdl, unsigned long long* tl) {
    launch_k(k_rmsnorm_rows, dim3(T), dim3(128), 0, s, pdl, x, w, out, H, eps, row_idx, tl);
}
void launch_argmax(const float* logits, int R, int V, int* out, float* scratch, size_t scratch_floats, int* counters,
                   int num_counters, int num_sms, cudaStream_t s, bool pdl, unsigned long long* tl) {
    int S = (4 * num_sms + R - 1) / R;  // about four blocks of 256 threads per SM
    if (S > 64) S = 64;
    if (S > V / 1024) S = V / 1024;
    if (S < 1 || !scratch || !counters || R > num_counters || (size_t)R * S * 2 > scratch_floats) S = 1;
    launch_k(k_argmax_rows, dim3(R, S), dim3(256), 0, s, pdl, logits, V, S, out, scratch, counters, tl);
}
void launch_argmax_tiles(const float* amax_val, const int* amax_idx, int R, int tiles, int* out, cudaStream_t s, bool pdl,
                         unsigned long long* tl, void* pack, int idx_offset) {
    launch_k(k_argmax_tiles, dim3(R), dim3(256), 0, s, pdl, amax_val, amax_idx, tiles, out, tl, (float2*)pack, idx_offset);
}
void launch_tp_pick_peer(const TpPickParts& parts, const TpPeerSync& sync, int R, int* out, int* status, cudaStream_t s, bool pdl) {
    launch_k(k_tp_pick_peer, dim3((R + 127) / 128), dim3(128), 0, s, pdl, parts, sync, R, out, status);
}
void launch_tp_pick(const void* cand, int ranks, int R, int* out, cudaStream_t s, bool pdl) {
    launch_k(k_tp_pick, dim3((R + 127) / 128), dim3(128), 0, s, pdl, (const float2*)cand, ranks, R, out);
}
void launch_residual_norm(bf16* h, const float* delta, const bf16* w, bf16* out, int T, int H, float eps, cudaStream_t s, bool pdl) {
    launch_k(k_residual_norm_rows, dim3(T), dim3(kRowNormThreads), 0, s, pdl, h, delta, w, out, H, eps);
}
void launch_tp_reduce_residual_norm(bf16* h, const TpParts& parts, const TpPeerSync& sync, const bf16* w, bf16* out, int T, int H,
                                    float eps, int* status, cudaStream_t s, bool pdl, unsigned long long* tl) {
    launch_k(k_tp_reduce_residual_norm, dim3(T), dim3(kRowNormThreads), 0, s, pdl, h, parts, sync, w, out, H, eps, status, tl);
}
void launch_sample(const float* logits, int R, int V, float temperature, const double* u, const int* step_counter, int* out,
                   cudaStream_t s, bool pdl, unsigned long long* tl) {
    launch_k(k_sample_rows, dim3(R), dim3(1024), 0, s, pdl, logits, V, temperature, u, step_counter, out, tl);
}
void launch_cast_f32_bf16(const float* src, bf16* dst, size_t n, cudaStream_t s) {
    int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    k_cast_f32_bf16<<<blocks, 256, 0, s>>>(src, dst, n);
}
void launch_pack_ffn(const bf16* gate, const bf16* up, const bf16* down, bf16* packed, int I, int H, cudaStream_t s) {
    k_pack_ffn<<<I, 256, 0, s>>>(gate, up, down, packed, I, H);
}
void launch_wait_selftest(int* status, cudaStream_t s) { k_wait_selftest<<<1, 32, 0, s>>>(status); }

}  // namespace tffn
