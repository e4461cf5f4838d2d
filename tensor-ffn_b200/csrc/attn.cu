// Grouped-query attention of ONE query token over the paged bf16 KV cache (decode; prefill
// runs it per prompt token with a causal context length).
//
// Reference arithmetic (inference/src/model/qwen.cu:349-412): scores = (q . k) / sqrt(hd) with
// q in fp32 and k in bf16, softmax with max-subtraction and exp (cuda_ops.cu:106-126),
// ctx = P V, ctx rounded to bf16; query head qh reads kv head qh * nkv / nh (qwen.cu:252).
// The reference re-expands the whole cache to fp32 per layer and materialises the score matrix.
//
// Here one CTA per (token, kv head, context split) copies its K/V rows once into shared memory
// (16-byte cp.async, two stages in flight, XOR-swizzled so that ldmatrix is conflict-free) and shares
// them between the G = nh / nkv query heads of the group, which form the M dimension of warp-level
// tensor-core tiles: S = Q K^T and O = P V as mma.sync m16n8k16 (bf16 operands, fp32 accumulate).
// G is at most 8, so the 16-row tile is the natural fit: a tcgen05 tile (M >= 64) would be 89%
// padding and put a TMEM round trip between the two contractions of a kernel that is bound by the
// latency of its loads, not by tensor throughput. q and P are fp32 in the reference; each enters the
// MMA as a bf16 pair (hi + lo, 16 mantissa bits): hi in tile rows 0-7, lo in rows 8-15, so one MMA
// yields both partial products in the same thread, which adds them. The softmax is the
// online form in fp32, per 32- or 16-key block of a warp. Splits are merged by the last split to finish
// (a ticket, no spinning), always in split order, so the result does not depend on scheduling.
#include "kernels.h"
#include "ptx.cuh"
#include "launch.h"
#include "attn_core.cuh"

namespace tffn {

namespace {

__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col). Fragment of lane (g = lane / 4, t = lane % 4):
// a0 = A[g][2t, 2t+1], a1 = A[g+8][2t, 2t+1], a2 = A[g][2t+8, 2t+9], a3 = A[g+8][2t+8, 2t+9];
// b0 = B[2t, 2t+1][g], b1 = B[2t+8, 2t+9][g]; c0, c1 = D[g][2t, 2t+1], c2, c3 = D[g+8][2t, 2t+1].
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// (x, y) as two bf16 pairs: hi = bf16(v), lo = bf16(v - hi); x in the low half (the lower k index)
__device__ __forceinline__ void split_bf16x2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
    hi = (uint32_t)__bfloat16_as_ushort(xh) | ((uint32_t)__bfloat16_as_ushort(yh) << 16);
    lo = (uint32_t)bf16_bits(x - __bfloat162float(xh)) | ((uint32_t)bf16_bits(y - __bfloat162float(yh)) << 16);
}

constexpr int kAttnCtaThreads = 256;  // 8 warps: each takes 16 keys of a 128-key stage
constexpr int kAttnWarps = kAttnCtaThreads / 32;

template <int HD>
struct AttnCfg {
    static constexpr int ROW_BYTES = HD * 2;
    static constexpr int GRAN = HD / 8;                // 16-byte granules per cached row
    static constexpr int STAGE_ROWS = 128;             // keys per stage
    static constexpr int NST = 256 / HD;               // stage buffers: 4 at head_dim 64, 2 at 128 (128 KB either way)
    static constexpr int WARP_ROWS = STAGE_ROWS / kAttnWarps;  // 16 keys of a stage per warp
    static constexpr int NT = WARP_ROWS / 8;           // 8-key tiles of S per warp and stage
    static constexpr int KB = WARP_ROWS / 16;          // 16-key steps of P V
    static constexpr int KS = HD / 16;                 // k-steps of Q K^T
    static constexpr int DT = HD / 8;                  // 8-wide tiles of the output row
    static constexpr int STAGE_BYTES = 2 * STAGE_ROWS * ROW_BYTES;  // K then V
    static constexpr int MERGE_FLOATS = kAttnWarps * 8 * (HD + 2);  // per warp and head: max, sum, O[HD]
    static constexpr int SMEM = NST * STAGE_BYTES;                  // the merge buffer reuses the first stage
    static_assert(MERGE_FLOATS * 4 <= STAGE_BYTES, "merge buffer must fit a stage");
    static_assert(NST >= 2 && KB >= 1, "");
};

// One block of 16 cached keys (rows row0 .. row0+15 of a stage buffer, the first n_valid >= 1 of them
// inside the context) for the query-head group held in qh / ql: S = Q K^T, online softmax of head
// lane / 4 (this thread: keys nt * 8 + (lane % 4) * 2 + {0, 1}), O += P V. The whole warp calls it.
template <int HD>
__device__ __forceinline__ void attn_block16(uint32_t kbuf, uint32_t vbuf, int row0, int n_valid,
                                             const uint32_t (&qh)[HD / 16][2], const uint32_t (&ql)[HD / 16][2], float scale,
                                             float& m_run, float& l_run, float (&o)[HD / 8][4], int lane) {
    using C = AttnCfg<HD>;
    const int quad = lane & 3;
    // ---- S = Q K^T for WARP_ROWS keys: NT tiles of 8 keys
    float s[C::NT][4];
#pragma unroll
    for (int nt = 0; nt < C::NT; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        const int row = row0 + nt * 8 + (lane & 7);  // this lane's address row for ldmatrix
#pragma unroll
        for (int kp = 0; kp < C::KS / 2; ++kp) {
            uint32_t b[4];  // B fragments of k-steps 2kp and 2kp + 1 (matrix i = granule 4kp + i)
            const int g = kp * 4 + (lane >> 3);
            ldmatrix_x4(kbuf + (uint32_t)(row * C::ROW_BYTES + ((g ^ (row & 7)) << 4)), b);
            mma_16816(s[nt], qh[2 * kp][0], ql[2 * kp][0], qh[2 * kp][1], ql[2 * kp][1], b[0], b[1]);
            mma_16816(s[nt], qh[2 * kp + 1][0], ql[2 * kp + 1][0], qh[2 * kp + 1][1], ql[2 * kp + 1][1], b[2], b[3]);
        }
    }
    // ---- online softmax of head hrow over these keys (this thread: keys nt * 8 + quad * 2 + {0, 1})
    float mx = kNegBig;
#pragma unroll
    for (int nt = 0; nt < C::NT; ++nt) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const bool live = nt * 8 + quad * 2 + j < n_valid;
            s[nt][j] = live ? (s[nt][j] + s[nt][j + 2]) * scale : kNegBig;  // q_hi . k + q_lo . k
            mx = fmaxf(mx, s[nt][j]);
        }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m_run, mx);  // finite: the first key of the block is in range
    const float corr = __expf(m_run - mn);
    m_run = mn;
    l_run *= corr;
#pragma unroll
    for (int d = 0; d < C::DT; ++d) { o[d][0] *= corr; o[d][1] *= corr; o[d][2] *= corr; o[d][3] *= corr; }
    uint32_t ph[C::NT], pl[C::NT];
#pragma unroll
    for (int nt = 0; nt < C::NT; ++nt) {
        const float p0 = (nt * 8 + quad * 2 < n_valid) ? __expf(s[nt][0] - mn) : 0.f;
        const float p1 = (nt * 8 + quad * 2 + 1 < n_valid) ? __expf(s[nt][1] - mn) : 0.f;
        l_run += p0 + p1;
        split_bf16x2(p0, p1, ph[nt], pl[nt]);
    }
    // ---- O += P V: per 16 keys, per pair of 8-wide output tiles one transposed ldmatrix of V
#pragma unroll
    for (int kb = 0; kb < C::KB; ++kb) {
        const int row = row0 + kb * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
        for (int jp = 0; jp < C::DT / 2; ++jp) {
            uint32_t b[4];  // keys 0-7 / 8-15 of tile 2jp, then of tile 2jp + 1
            const int g = jp * 2 + (lane >> 4);
            ldmatrix_x4_trans(vbuf + (uint32_t)(row * C::ROW_BYTES + ((g ^ (row & 7)) << 4)), b);
            mma_16816(o[2 * jp], ph[2 * kb], pl[2 * kb], ph[2 * kb + 1], pl[2 * kb + 1], b[0], b[1]);
            mma_16816(o[2 * jp + 1], ph[2 * kb], pl[2 * kb], ph[2 * kb + 1], pl[2 * kb + 1], b[2], b[3]);
        }
    }
}

template <int HD>
__global__ void __launch_bounds__(kAttnCtaThreads) k_attn_decode(const float* __restrict__ q, KvView kv, int layer,
                                                              const int* __restrict__ tok_seq,
                                                              const int* __restrict__ tok_pos, bf16* __restrict__ ctx,
                                                              int nh, int G, int splits, int early,
                                                              float* __restrict__ ws, int* __restrict__ counters,
                                                              int* status, unsigned long long* tl,
                                                              unsigned long long* trace) {
    using C = AttnCfg<HD>;
    // optional per-CTA phase stamps (globaltimer ns), 16 per CTA: 0 entry, 1 token data read, 2 first
    // stages requested, 3 grid wait over, 4 first stage landed, 5 all keys processed, 6 partial result
    // written, 7 ticket taken, 8 exit
#define ATTN_TRACE(slot)                                                                              \
    do {                                                                                              \
        if (trace && threadIdx.x == 0) {                                                              \
            unsigned long long t_;                                                                    \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                    \
            trace[(size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 16 + (slot)] = t_;                  \
        }                                                                                             \
    } while (0)
    ATTN_TRACE(0);
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_last;
    // [warp][head][HD + 2]; in the first stage buffer, which is idle once every warp has left the key loop
    float* merge = (float*)smem;

    // With `early` (decode) everything but q and the newest cached row (the one the previous kernel
    // wrote, at position tok_pos[t]) is older than the previous kernel, so token data, block table and
    // the first NST stages of K/V are requested before waiting for it; the newest row follows after.
    if (threadIdx.x == 0) tl_mark(tl, 0);
    pdl_launch_dependents();
    if (!early) pdl_wait();

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int unit = blockIdx.x;  // t * nkv + kvh
    const int nkv = kv.nkv;
    const int t = unit / nkv, kvh = unit % nkv;
    const int split = blockIdx.y;
    const int seq = __ldcg(tok_seq + t);
    const int ctx_len = __ldcg(tok_pos + t) + 1;
    int chunk = (ctx_len + splits - 1) / splits;
    chunk = (chunk + kPageTokens - 1) / kPageTokens * kPageTokens;
    const int c_begin = split * chunk;
    const int c_end = min(ctx_len, c_begin + chunk);
    ATTN_TRACE(1);
    const int* bt = kv.block_table + (size_t)seq * kv.max_pages_per_seq;
    const bf16* kpool = kv.k_pool + (size_t)layer * kv.layer_stride;
    const bf16* vpool = kv.v_pool + (size_t)layer * kv.layer_stride;
    const uint32_t smem_base = smem_u32(smem);
    bool bad = false;

    // Every warp owns rows [warp * 16, warp * 16 + 16) of every stage: it copies them itself and is the
    // only one to read them, so the key loop needs no CTA-wide barrier and the warps run independently.
    // The 16 rows lie in one page; the page ids of the warp's rows in stages 0..31 are fetched up front
    // (lane = stage), so that no copy waits behind a table lookup. Rows past the end of the range (or of
    // a bad page) are zero-filled: their P is 0, and 0 * garbage could be NaN.
    const int wrow0 = warp * C::WARP_ROWS;
    int pg_lane = -1;
    {
        const int tok0 = c_begin + lane * C::STAGE_ROWS + wrow0;
        if (tok0 < c_end) {
            const int pg = __ldg(bt + tok0 / kPageTokens);
            if (pg < 0 || pg >= kv.num_pages) bad = true;
            else pg_lane = pg;
        }
    }
    auto issue_stage = [&](int st) {  // the whole warp calls it
        const int s_begin = c_begin + st * C::STAGE_ROWS + wrow0;  // first key of this warp in the stage
        if (s_begin < c_end) {
            int pg;
            if (st < 32) {
                pg = __shfl_sync(0xffffffffu, pg_lane, st);
            } else {
                pg = __ldg(bt + s_begin / kPageTokens);
                if (pg < 0 || pg >= kv.num_pages) { bad = true; pg = -1; }
            }
            const uint32_t kbuf = smem_base + (uint32_t)((st % C::NST) * C::STAGE_BYTES);
            const uint32_t vbuf = kbuf + (uint32_t)(C::STAGE_ROWS * C::ROW_BYTES);
            const size_t page_off = ((size_t)(pg >= 0 ? pg : 0) * nkv + kvh) * kPageTokens * HD;
#pragma unroll
            for (int i = 0; i < C::WARP_ROWS * C::GRAN / 32; ++i) {
                const int idx = i * 32 + lane;
                const int r = idx / C::GRAN, g = idx % C::GRAN;
                const int row = wrow0 + r, tok = s_begin + r;
                const bool valid = tok < c_end && pg >= 0;
                const size_t off = page_off + (size_t)(tok % kPageTokens) * HD + g * 8;
                const uint32_t dst = (uint32_t)(row * C::ROW_BYTES + ((g ^ (row & 7)) << 4));
                if (!(early && st < C::NST && tok == ctx_len - 1)) {  // the newest row is copied after the wait
                    cp_async16_zfill(kbuf + dst, kpool + off, valid ? 16u : 0u);
                    cp_async16_zfill(vbuf + dst, vpool + off, valid ? 16u : 0u);
                }
            }
        }
        cp_async_commit();
    };
    const int n_stages = c_end > c_begin ? (c_end - c_begin + C::STAGE_ROWS - 1) / C::STAGE_ROWS : 0;
#pragma unroll
    for (int st = 0; st < C::NST; ++st) issue_stage(st);
    ATTN_TRACE(2);
    if (tid == 0 && !early) tl_mark(tl, 1);
    if (early) {
        // page of the newest row (the table entry is in L1 by now: the up-front lookups read it)
        const int newest_pg = ctx_len > 0 ? __ldg(bt + (ctx_len - 1) / kPageTokens) : -1;
        pdl_wait();
        ATTN_TRACE(3);
        if (tid == 0) tl_mark(tl, 1);
        const int rel = ctx_len - 1 - c_begin;  // newest row, relative to this split
        if (rel >= 0 && rel < C::NST * C::STAGE_ROWS && ctx_len - 1 < c_end && (rel % C::STAGE_ROWS) / C::WARP_ROWS == warp &&
            lane < C::GRAN) {
            const int row = rel % C::STAGE_ROWS, g = lane;
            const uint32_t kbuf = smem_base + (uint32_t)((rel / C::STAGE_ROWS) * C::STAGE_BYTES);
            const uint32_t vbuf = kbuf + (uint32_t)(C::STAGE_ROWS * C::ROW_BYTES);
            int pg = newest_pg;
            const bool valid = pg >= 0 && pg < kv.num_pages;
            if (!valid) { bad = true; pg = 0; }
            const size_t off = (((size_t)pg * nkv + kvh) * kPageTokens + (ctx_len - 1) % kPageTokens) * HD + g * 8;
            const uint32_t dst = (uint32_t)(row * C::ROW_BYTES + ((g ^ (row & 7)) << 4));
            cp_async16_zfill(kbuf + dst, kpool + off, valid ? 16u : 0u);
            cp_async16_zfill(vbuf + dst, vpool + off, valid ? 16u : 0u);
        }
        cp_async_commit();
    }

    // Q fragments (A operand; tile row g = hi part of query head g of the group, row g + 8 = its lo
    // part, heads >= G are zero): per k-step the pairs at k = (lane % 4) * 2 and k + 8 of head lane / 4.
    const int hrow = lane >> 2, quad = lane & 3;
    uint32_t qh[C::KS][2], ql[C::KS][2];
    {
        const float* qp = q + (size_t)t * nh * HD + (size_t)(kvh * G + hrow) * HD + quad * 2;
#pragma unroll
        for (int ks = 0; ks < C::KS; ++ks) {
            float2 a = make_float2(0.f, 0.f), b = make_float2(0.f, 0.f);
            if (hrow < G) {
                a = __ldcg((const float2*)(qp + ks * 16));
                b = __ldcg((const float2*)(qp + ks * 16 + 8));
            }
            split_bf16x2(a.x, a.y, qh[ks][0], ql[ks][0]);
            split_bf16x2(b.x, b.y, qh[ks][1], ql[ks][1]);
        }
    }
    const float scale = rsqrtf((float)HD);
    float m_run = kNegBig, l_run = 0.f;  // of head hrow; l_run is this thread's share (summed over the quad at the end)
    float o[C::DT][4];
#pragma unroll
    for (int d = 0; d < C::DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

    // One copy group per stage, committed in stage order (empty past the end of the range), and with
    // `early` one more for the newest row after the first NST: stage st has landed once at most NST - 1
    // younger groups are pending. The first iteration of an early launch also needs the newest row.
    for (int st = 0; st < n_stages; ++st) {
        if (early && st == 0) cp_async_wait<0>();
        else cp_async_wait<C::NST - 1>();
        __syncwarp();  // the lanes' copies of this warp's rows are complete and visible to the warp
        if (st == 0) ATTN_TRACE(4);
        const int w_begin = c_begin + st * C::STAGE_ROWS + warp * C::WARP_ROWS;  // first key of this warp
        if (w_begin < c_end) {
            const uint32_t kbuf = smem_base + (uint32_t)((st % C::NST) * C::STAGE_BYTES);
            const uint32_t vbuf = kbuf + (uint32_t)(C::STAGE_ROWS * C::ROW_BYTES);
            attn_block16<HD>(kbuf, vbuf, warp * C::WARP_ROWS, c_end - w_begin, qh, ql, scale, m_run, l_run, o, lane);
        }
        __syncwarp();  // every lane is done with the warp's rows of this buffer
        issue_stage(st + C::NST);  // commits a group even when there is nothing left to copy
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp has left the key loop: the first stage buffer becomes the merge buffer
    ATTN_TRACE(5);

    // ---- merge the eight warps: (max, sum, O) of head hrow per warp
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    {
        float* mw = merge + (size_t)(warp * 8 + hrow) * (HD + 2);
        if (quad == 0) { mw[0] = m_run; mw[1] = l_run; }
#pragma unroll
        for (int d = 0; d < C::DT; ++d) {
            mw[2 + d * 8 + quad * 2] = o[d][0] + o[d][2];  // P_hi V + P_lo V
            mw[2 + d * 8 + quad * 2 + 1] = o[d][1] + o[d][3];
        }
    }
    __syncthreads();
    float* part = ws + ((size_t)unit * splits + split) * (size_t)(G * (HD + 2));
    bf16* ctx_tok = ctx + (size_t)t * nh * HD;
    for (int idx = tid; idx < G * HD; idx += kAttnCtaThreads) {
        const int g = idx / HD, d = idx % HD;
        float M = kNegBig;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, merge[(size_t)(w * 8 + g) * (HD + 2)]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float* mw = merge + (size_t)(w * 8 + g) * (HD + 2);
            const float wgt = __expf(mw[0] - M);
            L += mw[1] * wgt;
            A += mw[2 + d] * wgt;
        }
        if (splits == 1) {
            ctx_tok[(size_t)(kvh * G + g) * HD + d] = __float2bfloat16_rn(A / L);
        } else {
            part[g * (HD + 2) + 2 + d] = A;
            if (d == 0) { part[g * (HD + 2)] = M; part[g * (HD + 2) + 1] = L; }
        }
    }
    if (bad) dev_fail(status, DEV_ERR_BOUNDS);
    ATTN_TRACE(6);
    if (splits == 1) {
        if (tid == 0) tl_mark(tl, 2);
        return;
    }

    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int old = atomicAdd(&counters[unit], 1);
        s_last = (old == splits - 1);
        if (old == splits - 1) counters[unit] = 0;
    }
    __syncthreads();
    ATTN_TRACE(7);
    if (!s_last) {
        if (tid == 0) tl_mark(tl, 2);
        return;
    }
    __threadfence();
    const float* parts = ws + (size_t)unit * splits * (size_t)(G * (HD + 2));
    constexpr int kMergeSplits = 16;  // up to here: one pass with every load in flight
    if (splits <= kMergeSplits) {
        // weight of split z for head g: exp(m_z - M) / sum_z l_z exp(m_z - M), kept in the (idle) merge buffer
        float* wgt = merge;  // [g][kMergeSplits]
        if (tid < G) {
            float mz[kMergeSplits], lz[kMergeSplits];
#pragma unroll
            for (int z = 0; z < kMergeSplits; ++z) {
                const bool live = z < splits;
                const float* pz = parts + (size_t)(live ? z : 0) * G * (HD + 2) + tid * (HD + 2);
                mz[z] = live ? __ldcg(pz) : kNegBig;
                lz[z] = live ? __ldcg(pz + 1) : 0.f;
            }
            float M = kNegBig, L = 0.f;
#pragma unroll
            for (int z = 0; z < kMergeSplits; ++z) M = fmaxf(M, mz[z]);
#pragma unroll
            for (int z = 0; z < kMergeSplits; ++z) {  // split order
                mz[z] = z < splits ? __expf(mz[z] - M) : 0.f;
                L += lz[z] * mz[z];
            }
#pragma unroll
            for (int z = 0; z < kMergeSplits; ++z) wgt[tid * kMergeSplits + z] = mz[z] / L;
        }
        __syncthreads();
        constexpr int ITERS = (8 * HD + kAttnCtaThreads - 1) / kAttnCtaThreads;  // G <= 8
        float res[ITERS];
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int idx = tid + it * kAttnCtaThreads;
            const bool on = idx < G * HD;
            const int g = on ? idx / HD : 0, d = on ? idx % HD : 0;
            float A = 0.f;
            for (int z0 = 0; z0 < splits; z0 += 4) {
                float az[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    az[j] = (on && z0 + j < splits) ? __ldcg(parts + (size_t)(z0 + j) * G * (HD + 2) + g * (HD + 2) + 2 + d) : 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (z0 + j < splits) A += az[j] * wgt[g * kMergeSplits + z0 + j];
            }
            res[it] = A;
        }
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int idx = tid + it * kAttnCtaThreads;
            if (idx < G * HD) ctx_tok[(size_t)(kvh * G + idx / HD) * HD + idx % HD] = __float2bfloat16_rn(res[it]);
        }
    } else {
        for (int idx = tid; idx < G * HD; idx += kAttnCtaThreads) {
            const int g = idx / HD, d = idx % HD;
            ctx_tok[(size_t)(kvh * G + g) * HD + d] = __float2bfloat16_rn(attn_merge_splits(parts, splits, G, HD, g, d));
        }
    }
    ATTN_TRACE(8);
    if (tid == 0) tl_mark(tl, 2);
#undef ATTN_TRACE
}

// Prefill: one CTA per (group of up to 8 consecutive prompt tokens of ONE sequence, kv head). The eight
// warps are the eight query tokens; the K/V stages (128 keys each, copied by all threads) are shared by
// them, so the cache is read once per 8 tokens instead of once per token; warp w runs the same 16-key
// blocks as the decode kernel over keys 0 .. pos_w (causal), owns its token's whole context and writes
// its output rows itself: no merge.
template <int HD>
__global__ void __launch_bounds__(kAttnCtaThreads) k_attn_prefill(const float* __restrict__ q, KvView kv, int layer,
                                                               const int* __restrict__ tok_seq,
                                                               const int* __restrict__ tok_pos,
                                                               const int* __restrict__ grp_first,
                                                               const int* __restrict__ grp_count, bf16* __restrict__ ctx,
                                                               int nh, int G, int* status, unsigned long long* tl) {
    using C = AttnCfg<HD>;
    extern __shared__ __align__(128) uint8_t smem[];
    if (threadIdx.x == 0) tl_mark(tl, 0);
    pdl_launch_dependents();
    pdl_wait();  // the previous kernel wrote q and the K/V rows of these very tokens
    if (threadIdx.x == 0) tl_mark(tl, 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y, nkv = kv.nkv;
    const int first = __ldcg(grp_first + blockIdx.x), count = __ldcg(grp_count + blockIdx.x);
    const int seq = __ldcg(tok_seq + first);
    const int last_len = __ldcg(tok_pos + first + count - 1) + 1;  // positions ascend within a group
    const bool active = warp < count;
    const int t = first + (active ? warp : 0);
    const int my_len = active ? __ldcg(tok_pos + t) + 1 : 0;
    const int* bt = kv.block_table + (size_t)seq * kv.max_pages_per_seq;
    const bf16* kpool = kv.k_pool + (size_t)layer * kv.layer_stride;
    const bf16* vpool = kv.v_pool + (size_t)layer * kv.layer_stride;
    const uint32_t smem_base = smem_u32(smem);
    bool bad = false;

    auto issue_stage = [&](int st) {  // all 256 threads
        const int s_begin = st * C::STAGE_ROWS;
        if (s_begin < last_len) {
            constexpr int PPS = C::STAGE_ROWS / kPageTokens;
            int pgs[PPS];
#pragma unroll
            for (int j = 0; j < PPS; ++j) {
                const int tok0 = s_begin + j * kPageTokens;
                const int pg = tok0 < last_len ? __ldg(bt + tok0 / kPageTokens) : -1;
                if (tok0 < last_len && (pg < 0 || pg >= kv.num_pages)) bad = true;
                pgs[j] = (pg >= 0 && pg < kv.num_pages) ? pg : -1;
            }
            const uint32_t kbuf = smem_base + (uint32_t)((st % C::NST) * C::STAGE_BYTES);
            const uint32_t vbuf = kbuf + (uint32_t)(C::STAGE_ROWS * C::ROW_BYTES);
            constexpr int ROWS_PER_IT = kAttnCtaThreads / C::GRAN;
            const int row0 = tid / C::GRAN, g = tid % C::GRAN;
#pragma unroll
            for (int i = 0; i < C::STAGE_ROWS / ROWS_PER_IT; ++i) {
                const int row = i * ROWS_PER_IT + row0;
                const int pg = pgs[(i * ROWS_PER_IT) / kPageTokens];
                const bool valid = s_begin + row < last_len && pg >= 0;
                const size_t off = (((size_t)(valid ? pg : 0) * nkv + kvh) * kPageTokens + row % kPageTokens) * HD + g * 8;
                const uint32_t dst = (uint32_t)(row * C::ROW_BYTES + ((g ^ (row & 7)) << 4));
                cp_async16_zfill(kbuf + dst, kpool + off, valid ? 16u : 0u);
                cp_async16_zfill(vbuf + dst, vpool + off, valid ? 16u : 0u);
            }
        }
        cp_async_commit();
    };
    const int n_stages = (last_len + C::STAGE_ROWS - 1) / C::STAGE_ROWS;
#pragma unroll
    for (int st = 0; st < C::NST; ++st) issue_stage(st);

    const int hrow = lane >> 2, quad = lane & 3;
    uint32_t qh[C::KS][2], ql[C::KS][2];
    {
        const float* qp = q + (size_t)t * nh * HD + (size_t)(kvh * G + hrow) * HD + quad * 2;
#pragma unroll
        for (int ks = 0; ks < C::KS; ++ks) {
            float2 a = make_float2(0.f, 0.f), b = make_float2(0.f, 0.f);
            if (active && hrow < G) {
                a = __ldcg((const float2*)(qp + ks * 16));
                b = __ldcg((const float2*)(qp + ks * 16 + 8));
            }
            split_bf16x2(a.x, a.y, qh[ks][0], ql[ks][0]);
            split_bf16x2(b.x, b.y, qh[ks][1], ql[ks][1]);
        }
    }
    const float scale = rsqrtf((float)HD);
    float m_run = kNegBig, l_run = 0.f;
    float o[C::DT][4];
#pragma unroll
    for (int d = 0; d < C::DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

    for (int st = 0; st < n_stages; ++st) {
        cp_async_wait<C::NST - 1>();
        __syncthreads();  // the stage is complete and visible to every warp
        const uint32_t kbuf = smem_base + (uint32_t)((st % C::NST) * C::STAGE_BYTES);
        const uint32_t vbuf = kbuf + (uint32_t)(C::STAGE_ROWS * C::ROW_BYTES);
#pragma unroll 1
        for (int blk = 0; blk < C::STAGE_ROWS / 16; ++blk) {
            const int k0 = st * C::STAGE_ROWS + blk * 16;
            if (k0 >= my_len) break;  // warp-uniform: causal end of this token
            attn_block16<HD>(kbuf, vbuf, blk * 16, my_len - k0, qh, ql, scale, m_run, l_run, o, lane);
        }
        __syncthreads();  // every warp is done with this buffer
        issue_stage(st + C::NST);
    }
    cp_async_wait<0>();
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (active && hrow < G) {
        const float inv = 1.f / l_run;  // my_len >= 1: at least one key
        bf16* dst = ctx + (size_t)t * nh * HD + (size_t)(kvh * G + hrow) * HD + quad * 2;
#pragma unroll
        for (int d = 0; d < C::DT; ++d) {
            const float a = (o[d][0] + o[d][2]) * inv, b = (o[d][1] + o[d][3]) * inv;  // P_hi V + P_lo V
            *(uint32_t*)(dst + d * 8) = (uint32_t)bf16_bits(a) | ((uint32_t)bf16_bits(b) << 16);
        }
    }
    if (bad) dev_fail(status, DEV_ERR_BOUNDS);
    if (tid == 0) tl_mark(tl, 2);
}

template <int HD>
void launch_hd(dim3 grid, cudaStream_t s, bool pdl, const float* q, const KvView& kv, int layer, const int* tok_seq,
               const int* tok_pos, bf16* ctx, int nh, int G, int splits, int early, float* ws, int* counters, int* status,
               unsigned long long* tl, unsigned long long* trace) {
    launch_k(k_attn_decode<HD>, grid, dim3(kAttnCtaThreads), (size_t)AttnCfg<HD>::SMEM, s, pdl, q, kv, layer, tok_seq, tok_pos, ctx,
             nh, G, splits, early, ws, counters, status, tl, trace);
}

template <int HD>
void launch_prefill_hd(dim3 grid, cudaStream_t s, bool pdl, const float* q, const KvView& kv, int layer, const int* tok_seq,
                       const int* tok_pos, const int* grp_first, const int* grp_count, bf16* ctx, int nh, int G, int* status,
                       unsigned long long* tl) {
    launch_k(k_attn_prefill<HD>, grid, dim3(kAttnCtaThreads), (size_t)AttnCfg<HD>::SMEM, s, pdl, q, kv, layer, tok_seq, tok_pos,
             grp_first, grp_count, ctx, nh, G, status, tl);
}

}  // namespace

// The dynamic shared-memory opt-in is a per-device attribute of a kernel: every session makes it for
// its own device (with that device current), outside of stream capture.
int attn_prepare() {
    cudaError_t e = cudaFuncSetAttribute(k_attn_decode<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnCfg<64>::SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_attn_decode<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnCfg<128>::SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_attn_prefill<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnCfg<64>::SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_attn_prefill<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnCfg<128>::SMEM);
    if (e == cudaSuccess) e = prefer_max_shared(k_attn_decode<64>);
    if (e == cudaSuccess) e = prefer_max_shared(k_attn_decode<128>);
    if (e == cudaSuccess) e = prefer_max_shared(k_attn_prefill<64>);
    if (e == cudaSuccess) e = prefer_max_shared(k_attn_prefill<128>);
    return (int)e;
}

constexpr int kMinSplitRows = 1024;

int attention_splits(int T, int nh, int nkv, int hd, int max_ctx, const AttnWorkspace& ws, int num_sms) {
    // One CTA per SM is the target: a CTA holds 128 KB of K/V in flight and its eight warps keep up with
    // what one SM can take in, and a launch without splits needs no merge (a partial write, a ticket and a
    // second read-back cost 4 to 6 us per launch, measured with two and three splits). Splits are used only
    // when there are fewer (token, kv head) units than half the SMs and the context is long: a split
    // must save more key-loop time (about 0.5 us per 128-key stage) than the merge costs, so each split
    // gets at least 1024 keys (batch 1 at a few hundred keys of context: 0.94 -> 0.82 ms per token
    // without splits; halving the minimum for 128-wide heads gained 1.4 us per launch for 32 sequences on a
    // quarter of the 7B shape's heads and cost batch 1 on the 1.5B shape 16 %: 576 -> 483 tok/s).
    const int G = nh / nkv;
    const int units = T * nkv;
    int splits = 1;
    if (units * 2 <= num_sms) {
        splits = num_sms / units;
        const int max_splits = (max_ctx + kMinSplitRows - 1) / kMinSplitRows;
        if (splits > max_splits) splits = max_splits;
        if (splits < 1) splits = 1;
        while (splits > 1 && ((size_t)units * splits * G * (hd + 2) > ws.partial_floats || units > ws.num_counters))
            --splits;
    }
    return splits;
}

void launch_attention(const float* q, KvView kv, int layer, const int* tok_seq, const int* tok_pos, bf16* ctx, int T,
                      int nh, int max_ctx, AttnWorkspace ws, int num_sms, int* status, cudaStream_t s, bool pdl,
                      bool only_newest_row_fresh, unsigned long long* tl, unsigned long long* trace, int trace_ctas) {
    const int early = (pdl && only_newest_row_fresh) ? 1 : 0;
    const int G = nh / kv.nkv;  // at most 8 (checked when the model is loaded)
    const int units = T * kv.nkv;
    const int splits = attention_splits(T, nh, kv.nkv, kv.hd, max_ctx, ws, num_sms);
    dim3 grid(units, splits);
    if ((long long)units * splits > trace_ctas) trace = nullptr;
    if (kv.hd == 64) launch_hd<64>(grid, s, pdl, q, kv, layer, tok_seq, tok_pos, ctx, nh, G, splits, early, ws.partials, ws.counters, status, tl, trace);
    else if (kv.hd == 128) launch_hd<128>(grid, s, pdl, q, kv, layer, tok_seq, tok_pos, ctx, nh, G, splits, early, ws.partials, ws.counters, status, tl, trace);
}

void launch_attention_prefill(const float* q, KvView kv, int layer, const int* tok_seq, const int* tok_pos, const int* grp_first,
                              const int* grp_count, int n_groups, bf16* ctx, int nh, int* status, cudaStream_t s, bool pdl,
                              unsigned long long* tl) {
    const int G = nh / kv.nkv;
    dim3 grid(n_groups, kv.nkv);
    if (kv.hd == 64) launch_prefill_hd<64>(grid, s, pdl, q, kv, layer, tok_seq, tok_pos, grp_first, grp_count, ctx, nh, G, status, tl);
    else if (kv.hd == 128) launch_prefill_hd<128>(grid, s, pdl, q, kv, layer, tok_seq, tok_pos, grp_first, grp_count, ctx, nh, G, status, tl);
}

}  // namespace tffn
