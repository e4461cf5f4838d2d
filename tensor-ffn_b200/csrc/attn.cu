// Grouped-query attention of ONE query token over the paged bf16 KV cache (decode; prefill
// runs it per prompt token with a causal context length).
//
// Reference arithmetic (inference/src/model/qwen.cu:349-412): scores = (q . k) / sqrt(hd) with
// q in fp32 and k in bf16, softmax with max-subtraction and exp (cuda_ops.cu:106-126),
// ctx = P V, ctx rounded to bf16; query head qh reads kv head qh * nkv / nh (qwen.cu:252).
// The reference re-expands the whole cache to fp32 per layer and materialises the score
// matrix; here one CTA per (token, kv head, context split) reads each K/V row once (16-byte
// loads, hd/8 lanes per row) and shares it between the G = nh / nkv query heads of the group,
// with an online softmax in fp32. Splits are merged by the last split to finish (a ticket,
// no spinning), always in split order, so the result does not depend on scheduling.
#include "kernels.h"
#include "ptx.cuh"
#include "launch.h"

namespace tffn {

namespace {

constexpr int kAttnThreads = 128;
constexpr float kNegBig = -1e30f;  // the reference's mask value (qwen.cu:278)

template <int HD, int G>
__global__ void __launch_bounds__(kAttnThreads) k_attn_decode(const float* __restrict__ q, KvView kv, int layer,
                                                              const int* __restrict__ tok_seq,
                                                              const int* __restrict__ tok_pos, bf16* __restrict__ ctx,
                                                              int nh, int splits, float* __restrict__ ws,
                                                              int* __restrict__ counters, int* status) {
    constexpr int LPT = HD / 8;                  // lanes per cached token row (16 bytes each)
    constexpr int NG = kAttnThreads / LPT;       // token rows in flight per CTA
    __shared__ float s_m[NG][G], s_l[NG][G];
    __shared__ float s_acc[NG][G][HD];
    __shared__ int s_last;

    pdl_launch_dependents();
    pdl_wait();

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

    const int grp = threadIdx.x / LPT, sub = threadIdx.x % LPT;
    const float scale = rsqrtf((float)HD);

    float qr[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float4* qp = (const float4*)(q + ((size_t)t * nh + kvh * G + g) * HD + sub * 8);
        float4 a = __ldcg(qp), b = __ldcg(qp + 1);
        qr[g][0] = a.x; qr[g][1] = a.y; qr[g][2] = a.z; qr[g][3] = a.w;
        qr[g][4] = b.x; qr[g][5] = b.y; qr[g][6] = b.z; qr[g][7] = b.w;
    }
    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = kNegBig;
        l[g] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
    }
    const bf16* kpool = kv.k_pool + (size_t)layer * kv.layer_stride;
    const bf16* vpool = kv.v_pool + (size_t)layer * kv.layer_stride;
    const int* bt = kv.block_table + (size_t)seq * kv.max_pages_per_seq;
    bool bad = false;

    // U rows per thread group and iteration: their page lookups and 16-byte K/V loads are all in
    // flight before the first dot product, which hides the HBM latency that a one-row loop pays
    // per row. The trip count is uniform across the warp (the shuffles use the full mask); rows past
    // the end of the range, or with a bad page id, are computed on zeros and then discarded.
    constexpr int U = 4;
    for (int base = c_begin; base < c_end; base += NG * U) {
        int pg[U];
        bool valid[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int tok = base + u * NG + grp;
            valid[u] = tok < c_end;
            pg[u] = valid[u] ? __ldcg(bt + tok / kPageTokens) : 0;
        }
        uint4 kk[U], vv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int tok = base + u * NG + grp;
            if (valid[u] && (pg[u] < 0 || pg[u] >= kv.num_pages)) { bad = true; valid[u] = false; }
            kk[u] = make_uint4(0, 0, 0, 0);
            vv[u] = make_uint4(0, 0, 0, 0);
            if (valid[u]) {
                const size_t off = (((size_t)pg[u] * nkv + kvh) * kPageTokens + tok % kPageTokens) * HD + sub * 8;
                kk[u] = __ldcg((const uint4*)(kpool + off));
                vv[u] = __ldcg((const uint4*)(vpool + off));
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t ku[4] = {kk[u].x, kk[u].y, kk[u].z, kk[u].w};
            float kf[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) { kf[2 * j] = bf16_lo(ku[j]); kf[2 * j + 1] = bf16_hi(ku[j]); }
            float s[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float d = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) d += qr[g][j] * kf[j];
                s[g] = d;
            }
#pragma unroll
            for (int o = LPT / 2; o > 0; o >>= 1)
#pragma unroll
                for (int g = 0; g < G; ++g) s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
            if (!valid[u]) continue;
            const uint32_t vu[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
            float vf[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) { vf[2 * j] = bf16_lo(vu[j]); vf[2 * j + 1] = bf16_hi(vu[j]); }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float sc = s[g] * scale;
                const float mn = fmaxf(m[g], sc);
                const float corr = __expf(m[g] - mn);
                const float p = __expf(sc - mn);
                m[g] = mn;
                l[g] = l[g] * corr + p;
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[g][j] = acc[g][j] * corr + p * vf[j];
            }
        }
    }
    if (bad) dev_fail(status, DEV_ERR_BOUNDS);

    // merge the NG row groups of this CTA
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (sub == 0) { s_m[grp][g] = m[g]; s_l[grp][g] = l[g]; }
#pragma unroll
        for (int j = 0; j < 8; ++j) s_acc[grp][g][sub * 8 + j] = acc[g][j];
    }
    __syncthreads();
    float* part = ws + ((size_t)unit * splits + split) * (size_t)(G * (HD + 2));
    for (int idx = threadIdx.x; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, d = idx % HD;
        float M = kNegBig;
#pragma unroll
        for (int r = 0; r < NG; ++r) M = fmaxf(M, s_m[r][g]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int r = 0; r < NG; ++r) {
            const float w = __expf(s_m[r][g] - M);
            L += s_l[r][g] * w;
            A += s_acc[r][g][d] * w;
        }
        if (splits == 1) {
            ctx[((size_t)t * nh + kvh * G + g) * HD + d] = __float2bfloat16_rn(A / L);
        } else {
            part[g * (HD + 2) + 2 + d] = A;
            if (d == 0) { part[g * (HD + 2)] = M; part[g * (HD + 2) + 1] = L; }
        }
    }
    if (splits == 1) return;

    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int old = atomicAdd(&counters[unit], 1);
        s_last = (old == splits - 1);
        if (old == splits - 1) counters[unit] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* parts = ws + (size_t)unit * splits * (size_t)(G * (HD + 2));
    for (int idx = threadIdx.x; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, d = idx % HD;
        float M = kNegBig, L = 0.f, A = 0.f;
        // 8 splits per round with all loads in flight; a running maximum keeps the merge exact
        for (int z0 = 0; z0 < splits; z0 += 8) {
            float mz[8], lz[8], az[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool live = z0 + j < splits;
                const float* pz = parts + (size_t)(live ? z0 + j : 0) * G * (HD + 2) + g * (HD + 2);
                mz[j] = live ? __ldcg(pz) : kNegBig;
                lz[j] = live ? __ldcg(pz + 1) : 0.f;
                az[j] = live ? __ldcg(pz + 2 + d) : 0.f;
            }
            float Mn = M;
#pragma unroll
            for (int j = 0; j < 8; ++j) Mn = fmaxf(Mn, mz[j]);
            const float corr = __expf(M - Mn);
            L *= corr;
            A *= corr;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float w = __expf(mz[j] - Mn);
                L += lz[j] * w;
                A += az[j] * w;
            }
            M = Mn;
        }
        ctx[((size_t)t * nh + kvh * G + g) * HD + d] = __float2bfloat16_rn(A / L);
    }
}

template <int HD>
bool dispatch_g(int G, dim3 grid, cudaStream_t s, bool pdl, const float* q, const KvView& kv, int layer, const int* tok_seq,
                const int* tok_pos, bf16* ctx, int nh, int splits, float* ws, int* counters, int* status) {
#define TFFN_ATTN_CASE(GG)                                                                                          \
    case GG:                                                                                                       \
        launch_k(k_attn_decode<HD, GG>, grid, dim3(kAttnThreads), 0, s, pdl, q, kv, layer, tok_seq, tok_pos, ctx, nh, \
                 splits, ws, counters, status);                                                                   \
        return true;
    switch (G) {
        TFFN_ATTN_CASE(1)
        TFFN_ATTN_CASE(2)
        TFFN_ATTN_CASE(3)
        TFFN_ATTN_CASE(4)
        TFFN_ATTN_CASE(5)
        TFFN_ATTN_CASE(6)
        TFFN_ATTN_CASE(7)
        TFFN_ATTN_CASE(8)
    }
#undef TFFN_ATTN_CASE
    return false;
}

}  // namespace

int attention_splits(int T, int nh, int nkv, int hd, int max_ctx, const AttnWorkspace& ws, int num_sms) {
    const int G = nh / nkv;
    const int units = T * nkv;
    int splits = 1;
    if (units < 2 * num_sms) {
        splits = (2 * num_sms + units - 1) / units;
        const int max_splits = (max_ctx + 2 * kPageTokens - 1) / (2 * kPageTokens);  // at least 64 rows per split
        if (splits > max_splits) splits = max_splits;
        if (splits < 1) splits = 1;
        while (splits > 1 && ((size_t)units * splits * G * (hd + 2) > ws.partial_floats || units > ws.num_counters))
            --splits;
    }
    return splits;
}

void launch_attention(const float* q, KvView kv, int layer, const int* tok_seq, const int* tok_pos, bf16* ctx, int T,
                      int nh, int max_ctx, AttnWorkspace ws, int num_sms, int* status, cudaStream_t s, bool pdl) {
    const int G = nh / kv.nkv;
    const int units = T * kv.nkv;
    const int splits = attention_splits(T, nh, kv.nkv, kv.hd, max_ctx, ws, num_sms);
    dim3 grid(units, splits);
    bool ok = false;
    if (kv.hd == 64) ok = dispatch_g<64>(G, grid, s, pdl, q, kv, layer, tok_seq, tok_pos, ctx, nh, splits, ws.partials, ws.counters, status);
    else if (kv.hd == 128) ok = dispatch_g<128>(G, grid, s, pdl, q, kv, layer, tok_seq, tok_pos, ctx, nh, splits, ws.partials, ws.counters, status);
    (void)ok;
}

}  // namespace tffn
