// TEST INFRASTRUCTURE — not part of the product.
//
// CPU restatement of the tensor-ffn inference forward pass (Qwen2.5 decoder with the base
// FFN plus an optional expert-FFN delta at every layer). Scalar C++ with OpenMP over output
// rows. It exists to check the CUDA path and to serve as the timed CPU baseline; nothing in
// the product may link or call it.
//
// Parity status: the reference repository holds no golden vectors or tests for this path.
// This restatement is pinned against outputs of the reference's own GPU code, captured on
// a B200 from a small seeded model and stored as fixtures under tests/golden/ (see
// tests/golden/make_golden.py), and again live on the GPU by the -m gpu tests when the
// compiled reference (oracle/_ref/ref_driver) is present.
//
// Every function cites the reference file:line it follows (paths inside the reference
// project). Rounding points follow the reference exactly; only the summation order inside a
// dot product differs (the reference uses cuBLAS, whose order is not documented).
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

typedef uint16_t bf16;

inline float bf2f(bf16 v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// Round-to-nearest-even fp32 -> bf16, the behaviour of __float2bfloat16
// (inference/src/backend/cuda_ops.cu:138-140, inference/src/io/checkpoint.cpp:47).
inline bf16 f2bf(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16)0x7fff;  // NaN
    u += 0x7fffu + ((u >> 16) & 1u);
    return (bf16)(u >> 16);
}

struct Layer {
    const bf16 *q_proj, *k_proj, *v_proj, *o_proj;
    const bf16 *q_bias, *k_bias, *v_bias;  // may be null
    const bf16 *attn_norm, *ffn_norm;
    const bf16 *gate_proj, *up_proj, *down_proj;
    // expert, bf16 after the loader's fp32->bf16 cast (may be null)
    const bf16 *e_gate, *e_up, *e_down;
};

struct Oracle {
    int H, I, L, nh, nkv, hd, V, max_seq;
    float eps, theta;
    float expert_scale;
    int has_expert;
    const bf16 *embed, *final_norm, *lm_head;
    std::vector<Layer> layers;
    std::vector<float> rope_cos, rope_sin;  // [max_seq, hd/2]
    std::vector<bf16> kcache, vcache;       // [L, max_seq, nkv, hd]
    int kv_len;
    int threads;
};

// dot of a bf16 weight row with a bf16 activation row, fp32 accumulate
// (cublasGemmEx with CUBLAS_COMPUTE_32F, inference/src/backend/cuda_ops.cu:18-43).
inline float dot_bf16(const bf16* w, const bf16* x, int n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int i = 0;
    for (; i + 8 <= n; i += 8)
        for (int j = 0; j < 8; ++j) acc[j] += bf2f(w[i + j]) * bf2f(x[i + j]);
    float s = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
    for (; i < n; ++i) s += bf2f(w[i]) * bf2f(x[i]);
    return s;
}

// out[t, n] = sum_k x[t, k] * W[n, k]     (x bf16 [T,K], W bf16 [N,K], out fp32 [T,N])
void gemm_xwT(const Oracle& o, const bf16* x, const bf16* W, float* out, int T, int N, int K) {
#pragma omp parallel for schedule(static) num_threads(o.threads)
    for (int n = 0; n < N; ++n) {
        const bf16* w = W + (size_t)n * K;
        for (int t = 0; t < T; ++t) out[(size_t)t * N + n] = dot_bf16(w, x + (size_t)t * K, K);
    }
}

// inference/src/backend/cuda_ops.cu:75-96 (k_rmsnorm): fp32 sum of squares,
// r = rsqrt(ss/dim + eps), out = bf16(float(x) * r * float(w)).
void rmsnorm(const bf16* x, const bf16* w, bf16* out, int T, int H, float eps) {
    for (int t = 0; t < T; ++t) {
        const bf16* xr = x + (size_t)t * H;
        float ss = 0.f;
        for (int i = 0; i < H; ++i) {
            float v = bf2f(xr[i]);
            ss += v * v;
        }
        float r = 1.0f / sqrtf(ss / (float)H + eps);
        for (int i = 0; i < H; ++i) out[(size_t)t * H + i] = f2bf(bf2f(xr[i]) * r * bf2f(w[i]));
    }
}

// inference/src/backend/cuda_ops.cu:58-69 (k_silu_mul_bf16)
inline bf16 silu_mul(bf16 g, bf16 u) {
    float gf = bf2f(g), uf = bf2f(u);
    return f2bf((gf / (1.f + expf(-gf))) * uf);
}

// One SwiGLU branch: fp32 [T,H] = (bf16(silu(bf16(x Wg^T)) * bf16(x Wu^T))) Wd^T * alpha
// Base: inference/src/model/qwen.cu:431-437. Expert: inference/src/model/expert.cu:44-59
// (alpha = output_scale applied by the GEMM to the fp32 accumulator).
void swiglu_branch(const Oracle& o, const bf16* x, const bf16* Wg, const bf16* Wu, const bf16* Wd,
                   float alpha, float* out, int T, std::vector<float>& tmp_g, std::vector<float>& tmp_u,
                   std::vector<bf16>& act) {
    int H = o.H, I = o.I;
    tmp_g.resize((size_t)T * I);
    tmp_u.resize((size_t)T * I);
    act.resize((size_t)T * I);
    gemm_xwT(o, x, Wg, tmp_g.data(), T, I, H);
    gemm_xwT(o, x, Wu, tmp_u.data(), T, I, H);
    for (size_t i = 0; i < (size_t)T * I; ++i) act[i] = silu_mul(f2bf(tmp_g[i]), f2bf(tmp_u[i]));
    gemm_xwT(o, act.data(), Wd, out, T, H, I);
    if (alpha != 1.0f)
        for (size_t i = 0; i < (size_t)T * H; ++i) out[i] *= alpha;
}

// inference/src/model/qwen.cu:291-458 (qwen_forward). Appends T tokens to the cache.
// logits: fp32 [T, V] or null; hidden: bf16 [L, T, H] residual stream after each layer, or null;
// argmax_out: int32 [T] greedy pick per row (inference/src/main.cpp:45-51), or null.
int forward(Oracle& o, const int32_t* tokens, int T, float* logits, bf16* hidden, int32_t* argmax_out,
            int last_only) {
    const int H = o.H, I = o.I, nh = o.nh, nkv = o.nkv, hd = o.hd, V = o.V;
    const int past = o.kv_len, total = past + T;
    if (T <= 0 || total > o.max_seq) return -1;
    const int half = hd / 2;

    std::vector<bf16> h((size_t)T * H), hn((size_t)T * H), ctx((size_t)T * nh * hd);
    std::vector<float> qf((size_t)T * nh * hd), kf((size_t)T * nkv * hd), vf((size_t)T * nkv * hd);
    std::vector<float> tmp((size_t)T * H), delta((size_t)T * H), tg, tu;
    std::vector<bf16> act;

    // embed: inference/src/model/qwen.cu:216-220
    for (int t = 0; t < T; ++t) {
        int tok = tokens[t];
        if (tok < 0 || tok >= V) return -2;
        memcpy(&h[(size_t)t * H], o.embed + (size_t)tok * H, (size_t)H * 2);
    }

    for (int l = 0; l < o.L; ++l) {
        const Layer& ly = o.layers[l];
        rmsnorm(h.data(), ly.attn_norm, hn.data(), T, H, o.eps);  // qwen.cu:314

        // q,k,v = bf16(x W^T); += bias in bf16 (qwen.cu:317-326, __hadd at :225)
        gemm_xwT(o, hn.data(), ly.q_proj, qf.data(), T, nh * hd, H);
        gemm_xwT(o, hn.data(), ly.k_proj, kf.data(), T, nkv * hd, H);
        gemm_xwT(o, hn.data(), ly.v_proj, vf.data(), T, nkv * hd, H);
        auto round_bias = [&](std::vector<float>& x, const bf16* b, int D) {
            for (int t = 0; t < T; ++t)
                for (int d = 0; d < D; ++d) {
                    bf16 v = f2bf(x[(size_t)t * D + d]);
                    if (b) v = f2bf(bf2f(v) + bf2f(b[d]));
                    x[(size_t)t * D + d] = bf2f(v);
                }
        };
        round_bias(qf, ly.q_bias, nh * hd);
        round_bias(kf, ly.k_bias, nkv * hd);
        round_bias(vf, ly.v_bias, nkv * hd);

        // RoPE in fp32 at position past+t (qwen.cu:232-244, :333-337)
        auto rope = [&](std::vector<float>& x, int heads) {
            for (int t = 0; t < T; ++t) {
                int pos = past + t;
                for (int hh = 0; hh < heads; ++hh) {
                    float* xh = &x[((size_t)t * heads + hh) * hd];
                    for (int i = 0; i < half; ++i) {
                        float c = o.rope_cos[(size_t)pos * half + i], s = o.rope_sin[(size_t)pos * half + i];
                        float x0 = xh[i], x1 = xh[i + half];
                        xh[i] = x0 * c - x1 * s;
                        xh[i + half] = x0 * s + x1 * c;
                    }
                }
            }
        };
        rope(qf, nh);
        rope(kf, nkv);

        // cache write: K rounded to bf16 after RoPE, V as bf16 (qwen.cu:339-346)
        bf16* kc = &o.kcache[((size_t)l * o.max_seq) * nkv * hd];
        bf16* vc = &o.vcache[((size_t)l * o.max_seq) * nkv * hd];
        for (int t = 0; t < T; ++t)
            for (int d = 0; d < nkv * hd; ++d) {
                kc[(size_t)(past + t) * nkv * hd + d] = f2bf(kf[(size_t)t * nkv * hd + d]);
                vc[(size_t)(past + t) * nkv * hd + d] = f2bf(vf[(size_t)t * nkv * hd + d]);
            }

        // attention (qwen.cu:349-412): scores = q.k / sqrt(hd), mask k > past+t with -1e30,
        // softmax (cuda_ops.cu:106-126), ctx = P V, ctx rounded to bf16. GQA map qwen.cu:252.
        const float scale = 1.f / sqrtf((float)hd);
#pragma omp parallel for collapse(2) schedule(static) num_threads(o.threads)
        for (int t = 0; t < T; ++t)
            for (int qh = 0; qh < nh; ++qh) {
                int kvh = qh * nkv / nh;
                const float* q = &qf[((size_t)t * nh + qh) * hd];
                std::vector<float> sc(total);
                float mx = -1e30f;
                for (int k = 0; k < total; ++k) {
                    float s;
                    if (k > past + t) {
                        s = -1e30f;
                    } else {
                        const bf16* kr = &kc[((size_t)k * nkv + kvh) * hd];
                        float a = 0.f;
                        for (int d = 0; d < hd; ++d) a += q[d] * bf2f(kr[d]);
                        s = a * scale;
                    }
                    sc[k] = s;
                    mx = fmaxf(mx, s);
                }
                float sum = 0.f;
                for (int k = 0; k < total; ++k) {
                    sc[k] = expf(sc[k] - mx);
                    sum += sc[k];
                }
                std::vector<float> acc(hd, 0.f);
                for (int k = 0; k < total; ++k) {
                    float p = sc[k] / sum;
                    if (p == 0.f) continue;
                    const bf16* vr = &vc[((size_t)k * nkv + kvh) * hd];
                    for (int d = 0; d < hd; ++d) acc[d] += p * bf2f(vr[d]);
                }
                for (int d = 0; d < hd; ++d) ctx[((size_t)t * nh + qh) * hd + d] = f2bf(acc[d]);
            }

        // o_proj fp32 out, residual h = bf16(float(h) + o) (qwen.cu:413-419, :282-285)
        gemm_xwT(o, ctx.data(), ly.o_proj, tmp.data(), T, H, nh * hd);
        for (size_t i = 0; i < (size_t)T * H; ++i) h[i] = f2bf(bf2f(h[i]) + tmp[i]);

        // FFN (qwen.cu:422-447): both branches read the same normalised input
        rmsnorm(h.data(), ly.ffn_norm, hn.data(), T, H, o.eps);
        if (o.has_expert && ly.e_gate)
            swiglu_branch(o, hn.data(), ly.e_gate, ly.e_up, ly.e_down, o.expert_scale, delta.data(), T, tg, tu, act);
        swiglu_branch(o, hn.data(), ly.gate_proj, ly.up_proj, ly.down_proj, 1.0f, tmp.data(), T, tg, tu, act);
        if (o.has_expert && ly.e_gate)
            for (size_t i = 0; i < (size_t)T * H; ++i) tmp[i] = tmp[i] + delta[i];  // qwen.cu:440-441
        for (size_t i = 0; i < (size_t)T * H; ++i) h[i] = f2bf(bf2f(h[i]) + tmp[i]);

        if (hidden) memcpy(hidden + ((size_t)l * T) * H, h.data(), (size_t)T * H * 2);
    }

    // final norm + LM head (qwen.cu:451-454); greedy = first strict maximum (main.cpp:45-51)
    rmsnorm(h.data(), o.final_norm, hn.data(), T, H, o.eps);
    int t0 = last_only ? T - 1 : 0;
    int rows = T - t0;
    std::vector<float> lg;
    float* lgp = logits;
    if (!lgp) {
        lg.resize((size_t)rows * V);
        lgp = lg.data();
    }
    gemm_xwT(o, hn.data() + (size_t)t0 * H, o.lm_head, lgp, rows, V, H);
    if (argmax_out)
        for (int r = 0; r < rows; ++r) {
            const float* row = lgp + (size_t)r * V;
            int best = 0;
            for (int i = 1; i < V; ++i)
                if (row[i] > row[best]) best = i;
            argmax_out[r] = best;
        }
    o.kv_len += T;  // qwen.cu:457
    return 0;
}

}  // namespace

extern "C" {

// cfg: H, I, L, nh, nkv, V, max_seq ; head_dim = H / nh (inference/src/model/qwen.cu:31)
void* oracle_create(int H, int I, int L, int nh, int nkv, int V, int max_seq, float eps, float theta) {
    Oracle* o = new Oracle();
    o->H = H; o->I = I; o->L = L; o->nh = nh; o->nkv = nkv; o->hd = H / nh; o->V = V; o->max_seq = max_seq;
    o->eps = eps; o->theta = theta; o->expert_scale = 0.1f; o->has_expert = 0;
    o->embed = o->final_norm = o->lm_head = nullptr;
    o->layers.assign(L, Layer());
    for (auto& ly : o->layers) memset(&ly, 0, sizeof(Layer));
    int half = o->hd / 2;
    // RoPE tables in float (inference/src/model/qwen.cu:120-132)
    o->rope_cos.resize((size_t)max_seq * half);
    o->rope_sin.resize((size_t)max_seq * half);
    for (int pos = 0; pos < max_seq; ++pos)
        for (int i = 0; i < half; ++i) {
            float freq = 1.f / powf(theta, (float)(2 * i) / (float)o->hd);
            o->rope_cos[(size_t)pos * half + i] = cosf(pos * freq);
            o->rope_sin[(size_t)pos * half + i] = sinf(pos * freq);
        }
    o->kcache.assign((size_t)L * max_seq * nkv * o->hd, 0);
    o->vcache.assign((size_t)L * max_seq * nkv * o->hd, 0);
    o->kv_len = 0;
#ifdef _OPENMP
    o->threads = omp_get_max_threads();
#else
    o->threads = 1;
#endif
    return o;
}

void oracle_free(void* p) { delete (Oracle*)p; }

int oracle_threads(void* p) { return ((Oracle*)p)->threads; }
void oracle_set_threads(void* p, int n) {
    if (n > 0) ((Oracle*)p)->threads = n;
}

// which: 0 embed, 1 final_norm, 2 lm_head (pass the embed pointer again when tied)
void oracle_set_global(void* p, int which, const uint16_t* data) {
    Oracle* o = (Oracle*)p;
    if (which == 0) o->embed = data;
    else if (which == 1) o->final_norm = data;
    else if (which == 2) o->lm_head = data;
}

// which: 0 q 1 k 2 v 3 o 4 qb 5 kb 6 vb 7 attn_norm 8 ffn_norm 9 gate 10 up 11 down
//        12 expert gate 13 expert up 14 expert down  (all bf16, caller keeps them alive)
void oracle_set_layer(void* p, int layer, int which, const uint16_t* data) {
    Layer& ly = ((Oracle*)p)->layers[layer];
    const bf16** slots[15] = {&ly.q_proj, &ly.k_proj, &ly.v_proj, &ly.o_proj, &ly.q_bias, &ly.k_bias, &ly.v_bias,
                              &ly.attn_norm, &ly.ffn_norm, &ly.gate_proj, &ly.up_proj, &ly.down_proj,
                              &ly.e_gate, &ly.e_up, &ly.e_down};
    if (which >= 0 && which < 15) *slots[which] = data;
}

void oracle_set_expert(void* p, int enabled, float scale) {
    Oracle* o = (Oracle*)p;
    o->has_expert = enabled;
    o->expert_scale = scale;
}

void oracle_reset(void* p) { ((Oracle*)p)->kv_len = 0; }  // inference/src/model/qwen.cu:174
int oracle_kv_len(void* p) { return ((Oracle*)p)->kv_len; }

int oracle_forward(void* p, const int32_t* tokens, int T, float* logits, uint16_t* hidden, int32_t* argmax_out,
                   int last_only) {
    return forward(*(Oracle*)p, tokens, T, logits, hidden, argmax_out, last_only);
}

// fp32 -> bf16 RNE over an array (the expert loader's cast, inference/src/io/checkpoint.cpp:33-62)
void oracle_f32_to_bf16(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = f2bf(src[i]);
}

// read access to the cache for kernel-level tests: copies [len, nkv, hd] of one layer
void oracle_get_kv(void* p, int layer, uint16_t* k_out, uint16_t* v_out) {
    Oracle* o = (Oracle*)p;
    size_t row = (size_t)o->nkv * o->hd;
    memcpy(k_out, &o->kcache[(size_t)layer * o->max_seq * row], (size_t)o->kv_len * row * 2);
    memcpy(v_out, &o->vcache[(size_t)layer * o->max_seq * row], (size_t)o->kv_len * row * 2);
}

}  // extern "C"
