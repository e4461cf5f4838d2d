// Core of the paged GQA decode attention, shared by k_attn_decode (attn.cu) and the persistent
// batch-1 kernel: 128 threads process the cached rows [c_begin, c_end) of one (token, kv head) and
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
// With STAGED the rows of [c_begin, c_end) were copied page by page into shared memory beforehand
// (ks / vs: row r of the range at r * HD, see attn_stage_pages) and are read from there.
template <int HD, int G, bool STAGED = false, typename SyncFn, typename OutFn>
__device__ __forceinline__ bool attn_range(const float* __restrict__ q_tok, const KvView& kv, int layer,
                                           const int* __restrict__ bt, int kvh, int c_begin, int c_end, int tid,
                                           AttnShared<HD, G>& sh, SyncFn sync, OutFn out, const bf16* ks = nullptr,
                                           const bf16* vs = nullptr) {
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
            pg[u] = (valid[u] && !STAGED) ? __ldcg(bt + tok / kPageTokens) : 0;
        }
        uint4 kk[U], vv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int tok = base + u * NG + grp;
            if (valid[u] && (pg[u] < 0 || pg[u] >= kv.num_pages)) { bad = true; valid[u] = false; }
            kk[u] = make_uint4(0, 0, 0, 0);
            vv[u] = make_uint4(0, 0, 0, 0);
            if (valid[u]) {
                if (STAGED) {
                    const size_t off = (size_t)(tok - c_begin) * HD + sub * 8;
                    kk[u] = *(const uint4*)(ks + off);
                    vv[u] = *(const uint4*)(vs + off);
                } else {
                    const size_t off = (((size_t)pg[u] * nkv + kvh) * kPageTokens + tok % kPageTokens) * HD + sub * 8;
                    kk[u] = __ldcg((const uint4*)(kpool + off));
                    vv[u] = __ldcg((const uint4*)(vpool + off));
                }
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

// Pages a CTA may stage (K and V each): 64 KB of dynamic shared memory in total, so that two CTAs
// still share an SM next to the merge buffers.
template <int HD>
struct AttnStageCfg {
    static constexpr int PAGE_ELEMS = kPageTokens * HD;
    static constexpr int MAX_PAGES = 32 * 1024 / (PAGE_ELEMS * 2);  // 8 at head_dim 64, 4 at 128
    static constexpr int BYTES = 2 * MAX_PAGES * PAGE_ELEMS * 2 + 16;
};

// Called by warp 0 (all 32 lanes) after `bar` was initialised with count 1 and made visible:
// requests every page of [c_begin, c_end) for one kv head as one contiguous bulk copy per page and
// pool. c_begin is a multiple of the page size. Returns false on a bad page id / too many pages.
template <int HD>
__device__ __forceinline__ bool attn_stage_pages(const KvView& kv, int layer, const int* __restrict__ bt, int kvh, int c_begin,
                                                 int c_end, bf16* ks, bf16* vs, uint64_t* bar, int lane) {
    using C = AttnStageCfg<HD>;
    const int p0 = c_begin / kPageTokens;
    const int np = c_end > c_begin ? (c_end - c_begin + kPageTokens - 1) / kPageTokens : 0;
    int pg = 0;
    bool ok = np <= C::MAX_PAGES;
    if (lane < np && ok) {
        pg = __ldcg(bt + p0 + lane);
        if (pg < 0 || pg >= kv.num_pages) ok = false;
    }
    ok = __all_sync(0xffffffffu, ok);
    if (lane == 0) mbar_arrive_expect_tx(bar, ok ? (uint32_t)(np * 2 * C::PAGE_ELEMS * 2) : 0u);
    __syncwarp();
    if (ok && lane < np) {
        const size_t src = (size_t)layer * kv.layer_stride + ((size_t)pg * kv.nkv + kvh) * (size_t)C::PAGE_ELEMS;
        bulk_g2s(ks + (size_t)lane * C::PAGE_ELEMS, kv.k_pool + src, (uint32_t)(C::PAGE_ELEMS * 2), bar);
        bulk_g2s(vs + (size_t)lane * C::PAGE_ELEMS, kv.v_pool + src, (uint32_t)(C::PAGE_ELEMS * 2), bar);
    }
    return ok;
}

// merge of `splits` partial results laid out [split][G][HD + 2] = (max, sum, weighted V[HD]) for one
// (query head g, dim d); all loads of a round of R splits are in flight together
template <int HD, int G, int R = 8>
__device__ __forceinline__ float attn_merge_splits(const float* __restrict__ parts, int splits, int g, int d) {
    float M = kNegBig, L = 0.f, A = 0.f;
    for (int z0 = 0; z0 < splits; z0 += R) {
        float mz[R], lz[R], az[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const bool live = z0 + j < splits;
            const float* pz = parts + (size_t)(live ? z0 + j : 0) * G * (HD + 2) + g * (HD + 2);
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

}  // namespace tffn
