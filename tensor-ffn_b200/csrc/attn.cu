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
#include "attn_core.cuh"

namespace tffn {

namespace {

template <int HD, int G, bool STAGED>
__global__ void __launch_bounds__(kAttnThreads) k_attn_decode(const float* __restrict__ q, KvView kv, int layer,
                                                              const int* __restrict__ tok_seq,
                                                              const int* __restrict__ tok_pos, bf16* __restrict__ ctx,
                                                              int nh, int splits, float* __restrict__ ws,
                                                              int* __restrict__ counters, int* status) {
    __shared__ AttnShared<HD, G> sh;
    __shared__ int s_last;
    extern __shared__ __align__(128) uint8_t stage_raw[];  // STAGED: K pages | V pages | mbarrier

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
    float* part = ws + ((size_t)unit * splits + split) * (size_t)(G * (HD + 2));
    bf16* ctx_tok = ctx + (size_t)t * nh * HD;
    const int* bt = kv.block_table + (size_t)seq * kv.max_pages_per_seq;
    bf16* ks = (bf16*)stage_raw;
    bf16* vs = ks + AttnStageCfg<HD>::MAX_PAGES * AttnStageCfg<HD>::PAGE_ELEMS;
    bool stage_bad = false;
    if (STAGED) {
        // all K/V rows of this CTA's range are requested up front (one bulk copy per page and pool)
        uint64_t* bar = (uint64_t*)(stage_raw + AttnStageCfg<HD>::BYTES - 16);
        if (threadIdx.x == 0) {
            mbar_init(bar, 1);
            fence_mbar_init();
        }
        __syncthreads();
        if (threadIdx.x < 32) stage_bad = !attn_stage_pages<HD>(kv, layer, bt, kvh, c_begin, c_end, ks, vs, bar, (int)threadIdx.x);
        if (!mbar_wait(bar, 0, status, DEV_ERR_FULL_WAIT)) stage_bad = true;
        stage_bad = __syncthreads_or(stage_bad);
    }
    const bool bad = attn_range<HD, G, STAGED>(
        q + (size_t)t * nh * HD, kv, layer, bt, kvh, c_begin, stage_bad ? c_begin : c_end,
        (int)threadIdx.x, sh, [] { __syncthreads(); },
        [&](int g, int d, float M, float L, float A) {
            if (splits == 1) {
                ctx_tok[(size_t)(kvh * G + g) * HD + d] = __float2bfloat16_rn(A / L);
            } else {
                part[g * (HD + 2) + 2 + d] = A;
                if (d == 0) { part[g * (HD + 2)] = M; part[g * (HD + 2) + 1] = L; }
            }
        },
        ks, vs);
    if (bad || stage_bad) dev_fail(status, DEV_ERR_BOUNDS);
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
        ctx_tok[(size_t)(kvh * G + g) * HD + d] = __float2bfloat16_rn(attn_merge_splits<HD, G>(parts, splits, g, d));
    }
}

template <int HD, bool STAGED>
bool dispatch_g(int G, dim3 grid, cudaStream_t s, bool pdl, const float* q, const KvView& kv, int layer, const int* tok_seq,
                const int* tok_pos, bf16* ctx, int nh, int splits, float* ws, int* counters, int* status) {
#define TFFN_ATTN_CASE(GG)                                                                                          \
    case GG: {                                                                                                     \
        if (STAGED) {                                                                                              \
            static bool configured = false; /* benign race: the call is idempotent */                              \
            if (!configured) {                                                                                     \
                cudaFuncSetAttribute(k_attn_decode<HD, GG, STAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                     AttnStageCfg<HD>::BYTES);                                                     \
                configured = true;                                                                                 \
            }                                                                                                      \
        }                                                                                                          \
        launch_k(k_attn_decode<HD, GG, STAGED>, grid, dim3(kAttnThreads), STAGED ? AttnStageCfg<HD>::BYTES : 0, s, pdl, q, kv, \
                 layer, tok_seq, tok_pos, ctx, nh, splits, ws, counters, status);                                  \
        return true;                                                                                               \
    }
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

AttnPlan attention_plan(int T, int nh, int nkv, int hd, int max_ctx, const AttnWorkspace& ws, int num_sms) {
    const int G = nh / nkv;
    const int units = T * nkv;
    auto fits = [&](int s) { return (size_t)units * s * G * (hd + 2) <= ws.partial_floats && units <= ws.num_counters; };
    AttnPlan plan{1, false};
    if (units < 2 * num_sms) {
        int splits = (2 * num_sms + units - 1) / units;
        const int max_splits = (max_ctx + 2 * kPageTokens - 1) / (2 * kPageTokens);  // at least 64 rows per split
        if (splits > max_splits) splits = max_splits;
        if (splits < 1) splits = 1;
        while (splits > 1 && !fits(splits)) --splits;
        plan.splits = splits;
    }
    // Staged variant: every CTA copies its whole range into shared memory first, so the range must
    // fit the staging buffer; more splits are taken for that as long as the grid stays moderate.
    const int max_pages = hd == 64 ? AttnStageCfg<64>::MAX_PAGES : AttnStageCfg<128>::MAX_PAGES;
    const int ctx_pages = (max_ctx + kPageTokens - 1) / kPageTokens;
    int need = plan.splits;
    while (((ctx_pages + need - 1) / need) > max_pages) ++need;
    // the kernel rounds a split's range up to whole pages: ceil(ceil(ctx / need) / page) pages
    if ((need == 1 || fits(need)) && (long long)units * need <= 16LL * num_sms) {
        plan.splits = need;
        plan.staged = true;
    }
    return plan;
}

void launch_attention(const float* q, KvView kv, int layer, const int* tok_seq, const int* tok_pos, bf16* ctx, int T,
                      int nh, int max_ctx, AttnWorkspace ws, int num_sms, int* status, cudaStream_t s, bool pdl) {
    const int G = nh / kv.nkv;
    const int units = T * kv.nkv;
    const AttnPlan plan = attention_plan(T, nh, kv.nkv, kv.hd, max_ctx, ws, num_sms);
    const int splits = plan.splits;
    dim3 grid(units, splits);
#define TFFN_ATTN_GO(HDV, ST) \
    dispatch_g<HDV, ST>(G, grid, s, pdl, q, kv, layer, tok_seq, tok_pos, ctx, nh, splits, ws.partials, ws.counters, status)
    if (kv.hd == 64) {
        if (plan.staged) TFFN_ATTN_GO(64, true);
        else TFFN_ATTN_GO(64, false);
    } else if (kv.hd == 128) {
        if (plan.staged) TFFN_ATTN_GO(128, true);
        else TFFN_ATTN_GO(128, false);
    }
#undef TFFN_ATTN_GO
}

}  // namespace tffn
