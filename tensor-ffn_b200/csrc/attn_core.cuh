// Paged GQA decode attention on the CUDA cores, used by the persistent batch-1 kernel (whose
// 128-thread groups process one context split each), and the merge of context splits that
// k_attn_decode (attn.cu) shares with it: 128 threads process the cached rows [c_begin, c_end) of one (token, kv head) and
// hand the merged (max, sum, weighted V) of every (query head of the group, dim) to `out`.
// Arithmetic follows inference/src/model/qwen.cu:349-412 (see attn.cu).
#pragma once
#include "kernels.h"
#include "ptx.cuh"

namespace tffn {

constexpr int kAttnThreads = 128;
constexpr float kNegBig = -1e30f;  // the reference's mask value (qwen.cu:278)

template <int HD, int G>
struct AttnShared {
    static constexpr int LPT = HD / 8;             // lanes per cached token row (16 bytes each)
    static constexpr int NG = kAttnThreads / LPT;  // token rows in flight
    float m[NG][G], l[NG][G];
    float acc[NG][G][HD];
};

// tid in [0, 128); sync() must be a barrier over exactly those 128 threads; q_tok = fp32 q of this
// token [nh * HD]; bt = the sequence's block-table row. Returns true if a page id was out of range.
template <int HD, int G, typename SyncFn, typename OutFn>
__device__ __forceinline__ bool attn_range(const float* __restrict__ q_tok, const KvView& kv, int layer,
                                           const int* __restrict__ bt, int kvh, int c_begin, int c_end, int tid,
                                           AttnShared<HD, G>& sh, SyncFn sync, OutFn out) {
    constexpr int LPT = AttnShared<HD, G>::LPT;
    constexpr int NG = AttnShared<HD, G>::NG;
    const int grp = tid / LPT, sub = tid % LPT;
    const float scale = rsqrtf((float)HD);

    float qr[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float4* qp = (const float4*)(q_tok + (size_t)(kvh * G + g) * HD + sub * 8);
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
    const int nkv = kv.nkv;
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

    // merge the NG row groups
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (sub == 0) { sh.m[grp][g] = m[g]; sh.l[grp][g] = l[g]; }
#pragma unroll
        for (int j = 0; j < 8; ++j) sh.acc[grp][g][sub * 8 + j] = acc[g][j];
    }
    sync();
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, d = idx % HD;
        float M = kNegBig;
#pragma unroll
        for (int r = 0; r < NG; ++r) M = fmaxf(M, sh.m[r][g]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int r = 0; r < NG; ++r) {
            const float w = __expf(sh.m[r][g] - M);
            L += sh.l[r][g] * w;
            A += sh.acc[r][g][d] * w;
        }
        out(g, d, M, L, A);
    }
    return bad;
}

// merge of `splits` partial results laid out [split][G][HD + 2] = (max, sum, weighted V[HD]) for one
// (query head g, dim d); all loads of a round of R splits are in flight together
template <int R = 8>
__device__ __forceinline__ float attn_merge_splits(const float* __restrict__ parts, int splits, int G, int HD, int g, int d) {
    float M = kNegBig, L = 0.f, A = 0.f;
    const size_t stride = (size_t)G * (HD + 2);
    for (int z0 = 0; z0 < splits; z0 += R) {
        float mz[R], lz[R], az[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const bool live = z0 + j < splits;
            const float* pz = parts + (size_t)(live ? z0 + j : 0) * stride + g * (HD + 2);
            mz[j] = live ? __ldcg(pz) : kNegBig;
            lz[j] = live ? __ldcg(pz + 1) : 0.f;
            az[j] = live ? __ldcg(pz + 2 + d) : 0.f;
        }
        float Mn = M;
#pragma unroll
        for (int j = 0; j < R; ++j) Mn = fmaxf(Mn, mz[j]);
        const float corr = __expf(M - Mn);
        L *= corr;
        A *= corr;
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const float w = __expf(mz[j] - Mn);
            L += lz[j] * w;
            A += az[j] * w;
        }
        M = Mn;
    }
    return A / L;
}
template <int HD, int G, int R = 8>
__device__ __forceinline__ float attn_merge_splits(const float* __restrict__ parts, int splits, int g, int d) {
    return attn_merge_splits<R>(parts, splits, G, HD, g, d);
}

}  // namespace tffn
