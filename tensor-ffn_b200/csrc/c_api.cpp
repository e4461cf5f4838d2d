// The C ABI (include/tffn.h): translates exceptions into status codes and keeps the last
// message per thread. No torch types, plain pointers and sizes only.
#include "../../include/tffn.h"
#include "../../include/tffn_diag.h"
#include "engine.h"
#include <cstring>
#include <memory>
#include <vector>

using namespace tffn;

struct tffn_model { Model* m; };
struct tffn_expert { Expert* e; };
struct tffn_session { Session* s; };
struct tffn_tokenizer { Tokenizer t; };
struct tffn_tp { TpComm* c; };

static thread_local std::string g_last_error;
namespace tffn {
void set_last_error(const std::string& msg) { g_last_error = msg; }
}  // namespace tffn

template <typename F>
static int guard(F&& f) {
    try {
        f();
        return TFFN_OK;
    } catch (const Error& e) {
        g_last_error = e.what();
        return e.code;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return TFFN_ERR_INVALID;
    } catch (...) {
        g_last_error = "unknown error";
        return TFFN_ERR_INVALID;
    }
}
static void need(bool ok, const char* what) {
    if (!ok) throw Error(kErrInvalid, what);
}

extern "C" {

const char* tffn_last_error(void) { return g_last_error.c_str(); }
int tffn_version(void) { return 100; }
int tffn_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int tffn_config_read(const char* model_dir, tffn_config* out) {
    return guard([&] {
        need(model_dir && out, "NULL argument");
        Config c = read_config(model_dir);
        out->hidden_size = c.hidden_size; out->intermediate_size = c.intermediate_size; out->num_layers = c.num_layers;
        out->num_heads = c.num_heads; out->num_kv_heads = c.num_kv_heads; out->head_dim = c.head_dim;
        out->vocab_size = c.vocab_size; out->max_position_embeddings = c.max_seq_len;
        out->rms_norm_eps = c.rms_norm_eps; out->rope_theta = c.rope_theta;
        out->eos_token_id = c.eos_token_id; out->bos_token_id = c.bos_token_id; out->tie_embeddings = c.tie_embeddings;
    });
}

int tffn_expert_probe(const char* path, uint32_t* version, uint32_t* num_layers, uint32_t* hidden, uint32_t* intermediate) {
    return guard([&] {
        need(path, "NULL path");
        ExpertFile f(path);
        if (version) *version = f.hdr.version;
        if (num_layers) *num_layers = f.hdr.num_layers;
        if (hidden) *hidden = f.hdr.hidden;
        if (intermediate) *intermediate = f.hdr.intermediate;
    });
}

int tffn_expert_write(const char* path, uint32_t num_layers, uint32_t hidden, uint32_t intermediate, const float* const* mats) {
    return guard([&] {
        need(path && mats && num_layers && hidden && intermediate, "bad argument");
        write_expert(path, num_layers, hidden, intermediate, mats);
    });
}

int tffn_safetensors_probe(const char* model_dir, const char* name, int32_t* num_shards, int32_t* num_tensors, char* dtype_out,
                           uint64_t* nbytes_out) {
    return guard([&] {
        need(model_dir, "NULL directory");
        SafeTensorsDir d(model_dir);
        if (num_shards) *num_shards = (int32_t)d.num_shards();
        if (num_tensors) *num_tensors = (int32_t)d.num_tensors();
        if (name) {
            const TensorInfo& ti = d.get(name);
            if (dtype_out) {
                strncpy(dtype_out, ti.dtype.c_str(), 7);
                dtype_out[7] = 0;
            }
            if (nbytes_out) *nbytes_out = ti.nbytes;
        }
    });
}

int tffn_tokenizer_load(const char* model_dir, tffn_tokenizer** out) {
    return guard([&] {
        need(model_dir && out, "NULL argument");
        std::unique_ptr<tffn_tokenizer> t(new tffn_tokenizer());
        t->t.load(model_dir);
        *out = t.release();
    });
}
void tffn_tokenizer_free(tffn_tokenizer* t) { delete t; }
int tffn_tokenizer_encode(const tffn_tokenizer* t, const char* text, uint32_t* ids, int cap) {
    int n = 0;
    int rc = guard([&] {
        need(t && text, "NULL argument");
        auto v = t->t.encode(text);
        n = (int)v.size();
        for (int i = 0; i < n && i < cap && ids; ++i) ids[i] = v[i];
    });
    return rc < 0 ? rc : n;
}
int tffn_tokenizer_decode(const tffn_tokenizer* t, const uint32_t* ids, int n, char* out, int cap) {
    int len = 0;
    int rc = guard([&] {
        need(t && (ids || n == 0) && n >= 0, "bad argument");
        std::string s = t->t.decode(std::vector<uint32_t>(ids, ids + n));
        len = (int)s.size();
        if (out && cap > 0) {
            int m = len < cap - 1 ? len : cap - 1;
            memcpy(out, s.data(), m);
            out[m] = 0;
        }
    });
    return rc < 0 ? rc : len;
}
int tffn_tokenizer_encode_bpe(const tffn_tokenizer* t, const char* text, uint32_t* ids, int cap) {
    int n = 0;
    int rc = guard([&] {
        need(t && text, "NULL argument");
        auto v = t->t.encode_bpe(text);
        n = (int)v.size();
        for (int i = 0; i < n && i < cap && ids; ++i) ids[i] = v[i];
    });
    return rc < 0 ? rc : n;
}
int tffn_tokenizer_decode_bpe(const tffn_tokenizer* t, const uint32_t* ids, int n, char* out, int cap) {
    int len = 0;
    int rc = guard([&] {
        need(t && (ids || n == 0) && n >= 0, "bad argument");
        std::string s = t->t.decode_bpe(std::vector<uint32_t>(ids, ids + n));
        len = (int)s.size();
        if (out && cap > 0) {
            int m = len < cap - 1 ? len : cap - 1;
            memcpy(out, s.data(), m);
            out[m] = 0;
        }
    });
    return rc < 0 ? rc : len;
}
int tffn_tokenizer_token_id(const tffn_tokenizer* t, const char* token, uint32_t* id) {
    return guard([&] {
        need(t && token && id, "NULL argument");
        *id = t->t.get_id(token);
    });
}
int tffn_tokenizer_special(const tffn_tokenizer* t, uint32_t* eos, uint32_t* bos, uint32_t* pad) {
    return guard([&] {
        need(t, "NULL tokenizer");
        if (eos) *eos = t->t.eos_id;
        if (bos) *bos = t->t.bos_id;
        if (pad) *pad = t->t.pad_id;
    });
}

int tffn_model_load(const char* model_dir, int device, int tp_rank, int tp_size, tffn_model** out) {
    return guard([&] {
        need(model_dir && out, "NULL argument");
        std::unique_ptr<Model> m(Model::load(model_dir, device, tp_rank, tp_size));
        *out = new tffn_model{m.release()};
    });
}
void tffn_model_free(tffn_model* m) {
    if (!m) return;
    delete m->m;
    delete m;
}
int tffn_model_config(const tffn_model* m, tffn_config* out) {
    return guard([&] {
        need(m && out, "NULL argument");
        const Config& c = m->m->cfg;
        out->hidden_size = c.hidden_size; out->intermediate_size = c.intermediate_size; out->num_layers = c.num_layers;
        out->num_heads = c.num_heads; out->num_kv_heads = c.num_kv_heads; out->head_dim = c.head_dim;
        out->vocab_size = c.vocab_size; out->max_position_embeddings = c.max_seq_len;
        out->rms_norm_eps = c.rms_norm_eps; out->rope_theta = c.rope_theta;
        out->eos_token_id = c.eos_token_id; out->bos_token_id = c.bos_token_id; out->tie_embeddings = c.tie_embeddings;
    });
}
uint64_t tffn_model_weight_bytes(const tffn_model* m, int with_expert) {
    if (!m) return 0;
    const Config& c = m->m->cfg;
    uint64_t b = m->m->weight_bytes_base;  // this rank's share under tensor parallelism
    if (with_expert) b += (uint64_t)c.num_layers * 3 * c.hidden_size * m->m->I * 2;
    return b;
}

int tffn_expert_load(const tffn_model* m, const char* path, float scale, tffn_expert** out) {
    return guard([&] {
        need(m && path && out, "NULL argument");
        std::unique_ptr<Expert> e(Expert::load(m->m, path, scale));
        *out = new tffn_expert{e.release()};
    });
}
int tffn_expert_set_scale(tffn_expert* e, float scale) {
    return guard([&] {
        need(e, "NULL expert");
        e->e->scale = scale;
    });
}
float tffn_expert_get_scale(const tffn_expert* e) { return e ? e->e->scale : 0.f; }
int tffn_expert_forward(const tffn_expert* e, const void* d_x_norm, float* d_out_delta, int batch_tokens, void* stream) {
    return guard([&] {
        need(e, "NULL expert");
        e->e->forward_layers(d_x_norm, d_out_delta, batch_tokens, (cudaStream_t)stream);
    });
}
void tffn_expert_free(tffn_expert* e) {
    if (!e) return;
    delete e->e;
    delete e;
}

int tffn_session_create(const tffn_model* m, const tffn_expert* expert, int max_batch, int max_seq, void* cuda_stream,
                        tffn_session** out) {
    return tffn_session_create_tp(m, expert, max_batch, max_seq, cuda_stream, nullptr, out);
}
int tffn_session_create_tp(const tffn_model* m, const tffn_expert* expert, int max_batch, int max_seq, void* cuda_stream,
                           tffn_tp* tp, tffn_session** out) {
    return guard([&] {
        need(m && out, "NULL argument");
        std::unique_ptr<Session> s(new Session(m->m, expert ? expert->e : nullptr, max_batch, max_seq, (cudaStream_t)cuda_stream,
                                               tp ? tp->c : nullptr));
        *out = new tffn_session{s.release()};
    });
}
int tffn_tp_unique_id(uint8_t* id128) {
    return guard([&] {
        need(id128, "NULL argument");
        tp_comm_unique_id(id128);
    });
}
int tffn_tp_create(const uint8_t* id128, int tp_rank, int tp_size, int device, tffn_tp** out) {
    return guard([&] {
        need(id128 && out, "NULL argument");
        *out = new tffn_tp{tp_comm_create(id128, tp_rank, tp_size, device)};
    });
}
void tffn_tp_free(tffn_tp* tp) {
    if (!tp) return;
    tp_comm_free(tp->c);
    delete tp;
}
int tffn_tp_partition(const tffn_config* cfg, int tp_rank, int tp_size, int32_t* out8) {
    return guard([&] {
        need(cfg && out8, "NULL argument");
        Config c;
        c.hidden_size = cfg->hidden_size; c.intermediate_size = cfg->intermediate_size; c.num_layers = cfg->num_layers;
        c.num_heads = cfg->num_heads; c.num_kv_heads = cfg->num_kv_heads; c.head_dim = cfg->head_dim;
        c.vocab_size = cfg->vocab_size;
        const TpPartition p = tp_partition(c, tp_rank, tp_size);
        const int32_t v[8] = {p.q_head0, p.n_q_heads, p.kv_head0, p.n_kv_heads, p.i0, p.n_i, p.v0, p.n_v};
        memcpy(out8, v, sizeof v);
    });
}
void tffn_session_free(tffn_session* s) {
    if (!s) return;
    delete s->s;
    delete s;
}
int tffn_session_reset(tffn_session* s, int slot) {
    return guard([&] {
        need(s, "NULL session");
        s->s->reset(slot);
    });
}
int tffn_session_seq_len(const tffn_session* s, int slot) {
    if (!s || slot < 0) return TFFN_ERR_INVALID;
    int n = -1;
    int rc = guard([&] { n = s->s->seq_len(slot); });
    return rc < 0 ? rc : n;
}
int tffn_session_set_launch_mode(tffn_session* s, int mode) {
    return guard([&] {
        need(s, "NULL session");
        s->s->set_launch_mode(mode);
    });
}
int tffn_session_set_tp_fused(tffn_session* s, int on) {
    return guard([&] {
        need(s, "NULL session");
        s->s->set_tp_fused(on != 0);
    });
}
int tffn_session_set_ablation(tffn_session* s, unsigned mask) {
    return guard([&] {
        need(s, "NULL session");
        s->s->set_ablation(mask);
    });
}
int tffn_session_set_sampling(tffn_session* s, float temperature, uint32_t seed) {
    return guard([&] {
        need(s, "NULL session");
        s->s->set_sampling(temperature, seed);
    });
}
int tffn_session_set_bs1_path(tffn_session* s, int enable) {
    return guard([&] {
        need(s, "NULL session");
        s->s->set_bs1_path(enable != 0);
    });
}
int tffn_session_capture_hidden(tffn_session* s, int max_rows) {
    return guard([&] {
        need(s, "NULL session");
        s->s->capture_hidden(max_rows);
    });
}
int tffn_session_get_hidden(tffn_session* s, int layer, uint16_t* dst, int max_rows) {
    int rows = 0;
    int rc = guard([&] {
        need(s, "NULL session");
        rows = s->s->get_hidden(layer, dst, max_rows);
    });
    return rc < 0 ? rc : rows;
}
int tffn_prefill(tffn_session* s, const int32_t* tokens, const int32_t* seq_lens, int n_seqs, int32_t* next_tokens,
                 float* logits_last) {
    return guard([&] {
        need(s, "NULL session");
        s->s->prefill(tokens, seq_lens, n_seqs, next_tokens, logits_last);
    });
}
int tffn_forward(tffn_session* s, int slot, const int32_t* tokens, int T, float* logits) {
    return guard([&] {
        need(s, "NULL session");
        s->s->forward(slot, tokens, T, logits);
    });
}
int tffn_decode_step(tffn_session* s, const int32_t* tokens_in, int n_seqs, int32_t* next_tokens, float* logits) {
    return guard([&] {
        need(s, "NULL session");
        s->s->decode_step(tokens_in, n_seqs, next_tokens, logits);
    });
}
int tffn_decode_run(tffn_session* s, int n_seqs, int steps, int32_t* tokens_out) {
    return guard([&] {
        need(s, "NULL session");
        s->s->decode_run(n_seqs, steps, tokens_out);
    });
}
int tffn_session_profile(tffn_session* s, int enable) {
    return guard([&] {
        need(s, "NULL session");
        s->s->set_profile(enable != 0);
    });
}
int tffn_session_profile_read(tffn_session* s, float* ms, int32_t* launches, int cap) {
    int n = 0;
    int rc = guard([&] {
        need(s, "NULL session");
        n = s->s->read_profile(ms, launches, cap);
    });
    return rc < 0 ? rc : n;
}
const char* tffn_profile_class_name(int cls) { return kclass_name(cls); }
int tffn_session_timeline(tffn_session* s, int n_seqs, uint64_t* out, int max_launches, int trace_launch,
                          uint64_t* trace_out, int trace_ctas) {
    int n = 0;
    int rc = guard([&] {
        need(s, "NULL session");
        n = s->s->timeline(n_seqs, out, max_launches, trace_launch, trace_out, trace_ctas);
    });
    return rc < 0 ? rc : n;
}
int tffn_session_status(tffn_session* s) {
    int st = 0;
    int rc = guard([&] {
        need(s, "NULL session");
        st = s->s->status();
    });
    return rc < 0 ? rc : st;
}
uint64_t tffn_session_launch_count(const tffn_session* s) { return s ? s->s->launch_count() : 0; }
void* tffn_session_stream(const tffn_session* s) { return s ? (void*)s->s->stream() : nullptr; }

int tffn_op_gemm(int device, const uint16_t* X, const uint16_t* W, float* out, int T, int N, int K, int splits) {
    return tffn_op_gemm_trace(device, X, W, out, T, N, K, splits, nullptr, 0);
}

int tffn_op_gemm_trace(int device, const uint16_t* X, const uint16_t* W, float* out, int T, int N, int K, int splits,
                       uint64_t* trace, int trace_ctas) {
    return guard([&] {
        need(X && W && out && T > 0 && N > 0 && K > 0 && K % 8 == 0, "bad GEMM arguments");
        int ndev = 0;
        if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) throw Error(kErrCuda, "no CUDA device is available");
        TFFN_CUDA(cudaSetDevice(device));
        cudaDeviceProp prop;
        TFFN_CUDA(cudaGetDeviceProperties(&prop, device));
        const int rows = T < 256 ? 256 : T;
        DeviceBuffer dx, dw, dout, status, dtrace;
        if (trace && trace_ctas > 0) dtrace.alloc((size_t)trace_ctas * 64 * 8);
        dx.alloc((size_t)rows * K * 2);
        dw.alloc((size_t)N * K * 2);
        dout.alloc((size_t)T * N * 4);
        status.alloc(4);
        TFFN_CUDA(cudaMemcpy(dx.p, X, (size_t)T * K * 2, cudaMemcpyHostToDevice));
        TFFN_CUDA(cudaMemcpy(dw.p, W, (size_t)N * K * 2, cudaMemcpyHostToDevice));
        GemmCall g;
        memset(&g, 0, sizeof g);
        g.op[0] = {dw.as<bf16>(), K, dx.as<bf16>(), K, K};
        g.N = N; g.T = T; g.mode = GEMM_STORE_F32; g.alpha = 1.f; g.out = dout.p; g.ldo = N; g.x_rows_alloc = rows;
        if (trace && trace_ctas > 0) {
            const int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
            const long long ctas = (long long)((N + 127) / 128) * ((T + bn - 1) / bn) * (splits > 0 ? splits : 8);
            if (ctas > trace_ctas) throw Error(kErrInvalid, "trace buffer too small for this grid");
            g.trace = dtrace.as<unsigned long long>();
            g.trace_ctas = trace_ctas;
        }
        cuda_check((cudaError_t)gemm_prepare(), "gemm_prepare", __FILE__, __LINE__);
        GemmWorkspace ws{status.as<int>(), prop.multiProcessorCount};
        int rc = launch_gemm(g, ws, 0, splits);
        if (rc == -1000) throw Error(kErrCuda, "cuTensorMapEncodeTiled failed or is unavailable");
        if (rc != 0) cuda_check((cudaError_t)rc, "tensor-core GEMM launch", __FILE__, __LINE__);
        TFFN_CUDA(cudaDeviceSynchronize());
        int st = 0;
        TFFN_CUDA(cudaMemcpy(&st, status.p, 4, cudaMemcpyDeviceToHost));
        if (st) throw Error(kErrDevice, "GEMM kernel reported device status " + std::to_string(st));
        TFFN_CUDA(cudaMemcpy(out, dout.p, (size_t)T * N * 4, cudaMemcpyDeviceToHost));
        if (g.trace) TFFN_CUDA(cudaMemcpy(trace, dtrace.p, (size_t)trace_ctas * 64 * 8, cudaMemcpyDeviceToHost));
    });
}

int tffn_op_swiglu_bs1(int device, const uint16_t* h_in, const uint16_t* norm_w, const uint16_t* packed_base,
                       const uint16_t* packed_expert, float expert_scale, float eps, int H, int I, uint16_t* h_out) {
    return tffn_op_swiglu_bs1_trace(device, h_in, norm_w, packed_base, packed_expert, expert_scale, eps, H, I, h_out, nullptr, 0);
}

int tffn_op_swiglu_bs1_trace(int device, const uint16_t* h_in, const uint16_t* norm_w, const uint16_t* packed_base,
                             const uint16_t* packed_expert, float expert_scale, float eps, int H, int I, uint16_t* h_out,
                             uint64_t* trace, int trace_ctas) {
    return guard([&] {
        need(h_in && norm_w && packed_base && h_out && H > 0 && I > 0, "bad arguments");
        int ndev = 0;
        if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) throw Error(kErrCuda, "no CUDA device is available");
        TFFN_CUDA(cudaSetDevice(device));
        if (H % 64 || H > 2048) throw Error(kErrUnsupported, "the batch-1 FFN kernel needs hidden % 64 == 0 and hidden <= 2048");
        cudaDeviceProp prop;
        TFFN_CUDA(cudaGetDeviceProperties(&prop, device));
        cuda_check((cudaError_t)bs1_prepare(H, true), "bs1_prepare", __FILE__, __LINE__);
        DeviceBuffer dh, dw, db, de, acc, status;
        dh.alloc((size_t)H * 2);
        dw.alloc((size_t)H * 2);
        db.alloc((size_t)I * 3 * H * 2);
        TFFN_CUDA(cudaMemcpy(dh.p, h_in, (size_t)H * 2, cudaMemcpyHostToDevice));
        TFFN_CUDA(cudaMemcpy(dw.p, norm_w, (size_t)H * 2, cudaMemcpyHostToDevice));
        TFFN_CUDA(cudaMemcpy(db.p, packed_base, (size_t)I * 3 * H * 2, cudaMemcpyHostToDevice));
        if (packed_expert) {
            de.alloc((size_t)I * 3 * H * 2);
            TFFN_CUDA(cudaMemcpy(de.p, packed_expert, (size_t)I * 3 * H * 2, cudaMemcpyHostToDevice));
        }
        acc.alloc(bs1_acc_words(H) * 8);  // zero-filled
        status.alloc(4);
        Bs1Ctx x;
        memset(&x, 0, sizeof x);
        x.H = H; x.I = I; x.eps = eps; x.expert_scale = expert_scale;
        x.h = dh.as<bf16>(); x.acc_out = acc.as<long long>(); x.status = status.as<int>();
        x.num_sms = prop.multiProcessorCount;
        DeviceBuffer dtrace;
        if (trace && trace_ctas >= prop.multiProcessorCount) {
            dtrace.alloc((size_t)trace_ctas * 16 * 8);
            x.trace = dtrace.as<unsigned long long>();
        }
        Bs1Layer ly;
        memset(&ly, 0, sizeof ly);
        ly.ffn_norm = dw.as<bf16>(); ly.ffn_base = db.as<bf16>(); ly.ffn_expert = packed_expert ? de.as<bf16>() : nullptr;
        // the kernel leaves its result as fixed-point sums; the finalize kernel adds them to h and clears them
        launch_bs1_ffn(x, ly, 0, false);
        launch_bs1_ffn_finalize(x.h, x.acc_out, H, 0);
        if (x.trace) {  // a second, warm launch is the one whose timestamps are returned
            TFFN_CUDA(cudaDeviceSynchronize());
            TFFN_CUDA(cudaMemcpy(dh.p, h_in, (size_t)H * 2, cudaMemcpyHostToDevice));
            TFFN_CUDA(cudaMemset(dtrace.p, 0, dtrace.bytes));
            launch_bs1_ffn(x, ly, 0, false);
            launch_bs1_ffn_finalize(x.h, x.acc_out, H, 0);
        }
        TFFN_CUDA(cudaGetLastError());
        TFFN_CUDA(cudaDeviceSynchronize());
        int st = 0;
        TFFN_CUDA(cudaMemcpy(&st, status.p, 4, cudaMemcpyDeviceToHost));
        if (st) throw Error(kErrDevice, "FFN kernel reported device status " + std::to_string(st));
        TFFN_CUDA(cudaMemcpy(h_out, dh.p, (size_t)H * 2, cudaMemcpyDeviceToHost));
        if (x.trace) TFFN_CUDA(cudaMemcpy(trace, dtrace.p, (size_t)trace_ctas * 16 * 8, cudaMemcpyDeviceToHost));
    });
}

int tffn_op_wait_selftest(int device) {
    int st = 0;
    int rc = guard([&] {
        int ndev = 0;
        if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) throw Error(kErrCuda, "no CUDA device is available");
        TFFN_CUDA(cudaSetDevice(device));
        DeviceBuffer status;
        status.alloc(4);
        launch_wait_selftest(status.as<int>(), 0);
        TFFN_CUDA(cudaGetLastError());
        TFFN_CUDA(cudaDeviceSynchronize());
        TFFN_CUDA(cudaMemcpy(&st, status.p, 4, cudaMemcpyDeviceToHost));
    });
    return rc < 0 ? rc : st;
}

int tffn_op_tp_wait_selftest(int device, int wait_ms) {
    int st = 0;
    int rc = guard([&] {
        int ndev = 0;
        if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) throw Error(kErrCuda, "no CUDA device is available");
        need(wait_ms >= 1 && wait_ms <= 2000, "wait_ms must be 1..2000");
        TFFN_CUDA(cudaSetDevice(device));
        // rank 0 of a group of two whose second rank does not exist: its window is a second local buffer, so the
        // signal lands in this GPU's memory and the flag this rank polls is never written
        const int H = 64, T = 2;
        DeviceBuffer status, win0, win1, calls, h, xn;
        status.alloc(4);
        const size_t flag_floats = (size_t)2 * kTpMaxRanks * kTpFlagBlocks;
        win0.alloc((flag_floats + 2 * T * H) * 4);
        win1.alloc((flag_floats + 2 * T * H) * 4);
        calls.alloc(kTpFlagBlocks * 4);
        h.alloc(T * H * 2);
        xn.alloc(T * H * 2);
        TpPeerSync sy;
        memset(&sy, 0, sizeof sy);
        sy.flags_local = win0.as<unsigned>();
        sy.flags_peer[0] = win0.as<unsigned>();
        sy.flags_peer[1] = win1.as<unsigned>();
        sy.calls = calls.as<unsigned>();
        sy.rank = 0;
        sy.size = 2;
        sy.wait_ns = (unsigned long long)wait_ms * 1000000ull;
        TpParts parts;
        parts.part[0] = win0.as<float>() + flag_floats;
        parts.part[1] = win1.as<float>() + flag_floats;
        for (int p = 2; p < kTpMaxRanks; ++p) parts.part[p] = nullptr;
        launch_tp_reduce_residual_norm(h.as<bf16>(), parts, sy, nullptr, xn.as<bf16>(), T, H, 1e-6f, status.as<int>(), 0);
        TFFN_CUDA(cudaGetLastError());
        TFFN_CUDA(cudaDeviceSynchronize());
        TFFN_CUDA(cudaMemcpy(&st, status.p, 4, cudaMemcpyDeviceToHost));
    });
    return rc < 0 ? rc : st;
}

}  // extern "C"
