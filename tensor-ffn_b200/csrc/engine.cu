#include "engine.h"
#include "launch.h"
#include <algorithm>
#include <cmath>
#include <cstring>
#include <memory>

namespace tffn {

void cuda_check(cudaError_t e, const char* what, const char* file, int line) {
    if (e == cudaSuccess) return;
    char buf[512];
    snprintf(buf, sizeof buf, "CUDA error %s:%d — %s (%s)", file, line, cudaGetErrorString(e), what);
    throw Error(kErrCuda, buf);
}

void DeviceBuffer::alloc(size_t n) {
    release();
    if (n == 0) return;
    TFFN_CUDA(cudaMalloc(&p, n));
    bytes = n;
    // The fill runs on the default stream and returns before it has finished, while the sessions work
    // on non-blocking streams that are not ordered after it: without the wait a buffer's first kernel
    // could run before the fill and have its output zeroed (seen as a rare change of sampled tokens when
    // a session was used right after it was created).
    TFFN_CUDA(cudaMemset(p, 0, n));
    TFFN_CUDA(cudaStreamSynchronize(0));
}
void DeviceBuffer::alloc_raw(size_t n) {
    release();
    if (n == 0) return;
    TFFN_CUDA(cudaMalloc(&p, n));
    bytes = n;
}
void DeviceBuffer::release() {
    if (p && owned) cudaFree(p);
    p = nullptr;
    bytes = 0;
    owned = true;
}

namespace {

void upload(DeviceBuffer& dst, const void* src, size_t bytes) {
    dst.alloc(bytes);
    TFFN_CUDA(cudaMemcpy(dst.p, src, bytes, cudaMemcpyHostToDevice));
    // from pageable memory the call may return once the data is staged: wait for it to reach the device,
    // the streams that will read it are not ordered after the default stream
    TFFN_CUDA(cudaStreamSynchronize(0));
}

// Host-to-device staging for the loaders: the weight files are memory-mapped (pageable), so a plain
// cudaMemcpy would page each tensor in, stage it inside the driver and block. Here the host thread copies the
// next chunk out of the mapping into one of two pinned buffers while the copy engine still moves the previous
// one; everything (copies, the re-layout kernels that follow them) is ordered on one stream and the loader
// waits once at the end.
class Stager {
public:
    explicit Stager(size_t chunk_bytes = (size_t)32 << 20) : chunk_(chunk_bytes) {
        TFFN_CUDA(cudaStreamCreateWithFlags(&s_, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            TFFN_CUDA(cudaMallocHost((void**)&buf_[i], chunk_));
            TFFN_CUDA(cudaEventCreateWithFlags(&ev_[i], cudaEventDisableTiming));
        }
    }
    ~Stager() {
        cudaStreamSynchronize(s_);
        for (int i = 0; i < 2; ++i) {
            if (buf_[i]) cudaFreeHost(buf_[i]);
            if (ev_[i]) cudaEventDestroy(ev_[i]);
        }
        cudaStreamDestroy(s_);
    }
    Stager(const Stager&) = delete;
    Stager& operator=(const Stager&) = delete;
    cudaStream_t stream() const { return s_; }
    void copy(void* dst, const void* src, size_t bytes) {
        for (size_t o = 0; o < bytes; o += chunk_) put((char*)dst + o, (const char*)src + o, std::min(chunk_, bytes - o), 0, 0, 0);
    }
    // `rows` rows of `width` bytes, `src_pitch` bytes apart in the mapping -> dense on the device
    void copy2d(void* dst, const void* src, size_t src_pitch, size_t width, size_t rows) {
        if (width == 0 || rows == 0) return;
        if (src_pitch == width) return copy(dst, src, width * rows);
        if (width > chunk_) throw Error(kErrUnsupported, "a matrix row is longer than the staging buffer");
        const size_t rows_per = chunk_ / width;
        for (size_t r = 0; r < rows; r += rows_per) {
            const size_t nr = std::min(rows_per, rows - r);
            put((char*)dst + r * width, (const char*)src + r * src_pitch, nr * width, src_pitch, width, nr);
        }
    }
    void finish() { TFFN_CUDA(cudaStreamSynchronize(s_)); }

private:
    // one chunk: wait until the pinned buffer's previous transfer has left it, fill it, send it
    void put(void* dst, const char* src, size_t bytes, size_t pitch, size_t width, size_t rows) {
        uint8_t* b = buf_[cur_];
        if (used_[cur_]) TFFN_CUDA(cudaEventSynchronize(ev_[cur_]));
        if (rows == 0) {
            memcpy(b, src, bytes);
        } else {
            for (size_t r = 0; r < rows; ++r) memcpy(b + r * width, src + r * pitch, width);
        }
        TFFN_CUDA(cudaMemcpyAsync(dst, b, bytes, cudaMemcpyHostToDevice, s_));
        TFFN_CUDA(cudaEventRecord(ev_[cur_], s_));
        used_[cur_] = true;
        cur_ ^= 1;
    }
    size_t chunk_;
    cudaStream_t s_ = nullptr;
    uint8_t* buf_[2] = {nullptr, nullptr};
    cudaEvent_t ev_[2] = {nullptr, nullptr};
    bool used_[2] = {false, false};
    int cur_ = 0;
};

// carves 256-byte aligned views out of one allocation
struct Slab {
    DeviceBuffer* mem;
    size_t off = 0;
    void take(DeviceBuffer& dst, size_t bytes) {
        const size_t a = (off + 255) & ~(size_t)255;
        if (a + bytes > mem->bytes) throw Error(kErrInvalid, "weight slab too small (internal size computation)");
        dst.view((char*)mem->p + a, bytes);
        off = a + bytes;
    }
    static size_t padded(size_t bytes) { return (bytes + 255) & ~(size_t)255; }
};

// one block: publish the picks as the next step's inputs, advance the sequence lengths
__global__ void k_decode_advance(const int* __restrict__ picks, int n, int* __restrict__ dec_tokens, int* __restrict__ seq_len,
                                 int* __restrict__ ring, int* __restrict__ step_counter) {
    const int st = *step_counter;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        dec_tokens[i] = picks[i];
        seq_len[i] += 1;
        if (ring) ring[(size_t)st * n + i] = picks[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) *step_counter = st + 1;
}

__global__ void k_copy_rows_bf16(const bf16* __restrict__ src, bf16* __restrict__ dst, size_t n16) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n16) ((uint4*)dst)[i] = ((const uint4*)src)[i];
}

}  // namespace

// ------------------------------------------------------------------------------------------ Expert op
void Expert::forward_layers(const void* d_x, float* d_out, int T, cudaStream_t stream) const {
    if (!d_x || !d_out || T < 1) throw Error(kErrInvalid, "bad expert_forward arguments");
    const Config& c = model->cfg;
    if (model->tp.tp_size != 1) throw Error(kErrUnsupported, "expert_forward is not split across tensor-parallel ranks");
    const int H = c.hidden_size, I = c.intermediate_size;
    TFFN_CUDA(cudaSetDevice(model->device));
    cuda_check((cudaError_t)gemm_prepare(), "gemm_prepare", __FILE__, __LINE__);
    DeviceBuffer act, status;
    act.alloc((size_t)T * I * 2);
    status.alloc(4);
    TFFN_CUDA(cudaMemsetAsync(status.p, 0, 4, stream));
    const GemmWorkspace ws{status.as<int>(), model->num_sms};
    auto run = [&](GemmCall& g) {
        const int rc = launch_gemm(g, ws, stream);
        if (rc == -1000) throw Error(kErrCuda, "cuTensorMapEncodeTiled failed or is unavailable");
        if (rc != 0) cuda_check((cudaError_t)rc, "tensor-core GEMM launch", __FILE__, __LINE__);
    };
    for (size_t l = 0; l < layers.size(); ++l) {
        const bf16* x = (const bf16*)d_x + l * (size_t)T * H;
        const bf16* rec = layers[l].packed.as<bf16>();
        GemmCall g;
        memset(&g, 0, sizeof g);
        g.x_rows_alloc = T;
        g.T = T;
        g.alpha = 1.f;
        // gate | up with the SwiGLU epilogue (gemm_bf16_out x2 + silu_mul_bf16, ffn_expert.cu:162-166)
        g.op[0] = {rec, (int64_t)3 * H, x, H, H};
        g.op[1] = {rec + H, (int64_t)3 * H, x, H, H};
        g.N = I;
        g.mode = GEMM_SWIGLU;
        g.out = act.p;
        g.ldo = I;
        run(g);
        // down projection, fp32 out, scaled (gemm_bf16 + scale_fp32, ffn_expert.cu:167-171)
        g.op[0] = {layers[l].down.as<bf16>(), I, act.as<bf16>(), I, I};
        g.op[1] = {nullptr, 0, nullptr, 0, 0};
        g.N = H;
        g.mode = GEMM_STORE_F32;
        g.out = d_out + l * (size_t)T * H;
        g.ldo = H;
        g.out_scale = scale;
        run(g);
        g.out_scale = 0.f;
    }
    int st = 0;
    TFFN_CUDA(cudaMemcpyAsync(&st, status.p, 4, cudaMemcpyDeviceToHost, stream));
    TFFN_CUDA(cudaStreamSynchronize(stream));
    if (st != 0) throw Error(kErrDevice, "device status " + std::to_string(st) + " in expert_forward");
}

// ------------------------------------------------------------------------------------------ Model
Model* Model::load(const std::string& dir, int device, int tp_rank, int tp_size) {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) throw Error(kErrCuda, "no CUDA device is available");
    if (device < 0 || device >= ndev) throw Error(kErrInvalid, "device index out of range");
    TFFN_CUDA(cudaSetDevice(device));
    std::unique_ptr<Model> m(new Model());
    m->device = device;
    cudaDeviceProp prop;
    TFFN_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10) throw Error(kErrUnsupported, "this library is built for sm_100a (B200) only");
    m->num_sms = prop.multiProcessorCount;
    m->cfg = read_config(dir);
    const Config& c = m->cfg;
    m->tp = tp_partition(c, tp_rank, tp_size);
    const TpPartition& tp = m->tp;
    m->nh = tp.n_q_heads;
    m->nkv = tp.n_kv_heads;
    m->I = tp.n_i;
    m->V = tp.n_v;
    const size_t H = c.hidden_size, Ifull = c.intermediate_size, V = c.vocab_size, hd = c.head_dim;
    const size_t nh_full = c.num_heads;
    const size_t nh = m->nh, nkv = m->nkv, I = m->I;
    if (!(hd == 64 || hd == 128)) throw Error(kErrUnsupported, "head_dim must be 64 or 128");
    if (H % 8 || I % 8) throw Error(kErrUnsupported, "hidden and intermediate sizes must be multiples of 8");
    if (nh / nkv > 8 || nh % nkv != 0) throw Error(kErrUnsupported, "more than 8 query heads per kv head");

    SafeTensorsDir st(dir);
    // this rank's rows of q / k / v (whole heads), columns of o_proj, rows of gate / up, columns of down
    const size_t nq = nh * hd, nk = nkv * hd, nqkv = nq + 2 * nk;
    const size_t q0 = (size_t)tp.q_head0 * hd, k0 = (size_t)tp.kv_head0 * hd;
    const size_t nq_full = nh_full * hd, nk_full = (size_t)c.num_kv_heads * hd;
    const bool has_bias = st.has("model.layers.0.self_attn.q_proj.bias");  // same test as inference/src/model/qwen.cu:99
    // one allocation for every weight (cudaMalloc and its zero-fill once, not ten times per layer)
    {
        size_t total = Slab::padded(V * H * 2) + Slab::padded(H * 2);
        if (!c.tie_embeddings) total += Slab::padded((size_t)m->V * H * 2);
        const size_t per_layer = Slab::padded(nqkv * H * 2) + Slab::padded(nqkv * 2) + Slab::padded(H * nq * 2) + 2 * Slab::padded(H * 2) +
                                 Slab::padded(H * I * 2) + Slab::padded(I * 3 * H * 2);
        total += per_layer * (size_t)c.num_layers + 256;
        m->slab.alloc_raw(total);
    }
    Slab slab{&m->slab};
    Stager up;
    slab.take(m->embed, V * H * 2);
    up.copy(m->embed.p, st.bf16("model.embed_tokens.weight", V * H), V * H * 2);  // replicated: a row gather only
    m->layers.resize(c.num_layers);
    DeviceBuffer gate_tmp, up_tmp;
    gate_tmp.alloc_raw(I * H * 2);
    up_tmp.alloc_raw(I * H * 2);
    for (int l = 0; l < c.num_layers; ++l) {
        LayerWeights& ly = m->layers[l];
        const std::string p = "model.layers." + std::to_string(l) + ".";
        slab.take(ly.wqkv, nqkv * H * 2);
        up.copy(ly.wqkv.as<bf16>(), st.bf16(p + "self_attn.q_proj.weight", nq_full * H) + q0 * H, nq * H * 2);
        up.copy(ly.wqkv.as<bf16>() + nq * H, st.bf16(p + "self_attn.k_proj.weight", nk_full * H) + k0 * H, nk * H * 2);
        up.copy(ly.wqkv.as<bf16>() + (nq + nk) * H, st.bf16(p + "self_attn.v_proj.weight", nk_full * H) + k0 * H, nk * H * 2);
        if (st.has(p + "self_attn.q_proj.bias")) {
            if (!has_bias) throw Error(kErrFormat, "some layers have projection biases and some do not");
            ly.has_bias = true;
            slab.take(ly.bqkv, nqkv * 2);
            up.copy(ly.bqkv.as<bf16>(), st.bf16(p + "self_attn.q_proj.bias", nq_full) + q0, nq * 2);
            up.copy(ly.bqkv.as<bf16>() + nq, st.bf16(p + "self_attn.k_proj.bias", nk_full) + k0, nk * 2);
            up.copy(ly.bqkv.as<bf16>() + nq + nk, st.bf16(p + "self_attn.v_proj.bias", nk_full) + k0, nk * 2);
        }
        slab.take(ly.wo, H * nq * 2);
        up.copy2d(ly.wo.p, st.bf16(p + "self_attn.o_proj.weight", H * nq_full) + q0, nq_full * 2, nq * 2, H);
        slab.take(ly.attn_norm, H * 2);
        up.copy(ly.attn_norm.p, st.bf16(p + "input_layernorm.weight", H), H * 2);
        slab.take(ly.ffn_norm, H * 2);
        up.copy(ly.ffn_norm.p, st.bf16(p + "post_attention_layernorm.weight", H), H * 2);
        // gate and up pass through two scratch matrices (reused by every layer: the copies and the kernel that
        // reads them are ordered on the staging stream), down goes to its place and into the records
        up.copy(gate_tmp.p, st.bf16(p + "mlp.gate_proj.weight", Ifull * H) + (size_t)tp.i0 * H, I * H * 2);
        up.copy(up_tmp.p, st.bf16(p + "mlp.up_proj.weight", Ifull * H) + (size_t)tp.i0 * H, I * H * 2);
        slab.take(ly.ffn.down, H * I * 2);
        up.copy2d(ly.ffn.down.p, st.bf16(p + "mlp.down_proj.weight", H * Ifull) + tp.i0, Ifull * 2, I * 2, H);
        slab.take(ly.ffn.packed, I * 3 * H * 2);
        launch_pack_ffn(gate_tmp.as<bf16>(), up_tmp.as<bf16>(), ly.ffn.down.as<bf16>(), ly.ffn.packed.as<bf16>(), (int)I, (int)H, up.stream());
        TFFN_CUDA(cudaGetLastError());
    }
    slab.take(m->final_norm, H * 2);
    up.copy(m->final_norm.p, st.bf16("model.norm.weight", H), H * 2);
    // LM head: this rank's rows of the vocabulary
    if (c.tie_embeddings) {
        m->lm_head = m->embed.as<bf16>() + (size_t)tp.v0 * H;
    } else {
        slab.take(m->lm_head_own, (size_t)m->V * H * 2);
        up.copy(m->lm_head_own.p, st.bf16("lm_head.weight", V * H) + (size_t)tp.v0 * H, (size_t)m->V * H * 2);
        m->lm_head = m->lm_head_own.as<bf16>();
    }
    up.finish();  // the only wait of the load; the scratch matrices are released after it
    m->bs1_ok = tp_size == 1 && bs1_supported((int)H, (int)I, (int)hd, (int)nh, (int)nkv);
    const uint64_t per_layer = (nqkv * H + H * nq + 3 * I * H) * 2 + 2 * H * 2 + (uint64_t)(m->layers[0].has_bias ? nqkv * 2 : 0);
    m->weight_bytes_base = per_layer * c.num_layers + (uint64_t)m->V * H * 2 + H * 2;
    return m.release();
}

// ------------------------------------------------------------------------------------------ Expert
// Reads only this rank's slice of every matrix from the memory-mapped file (rows of gate / up, columns of
// down): a tensor-parallel rank touches 1 / tp_size of the file (inference/src/io/checkpoint.cpp:40-61 reads
// whole matrices through three device allocations per layer).
Expert* Expert::load(const Model* m, const std::string& path, float scale) {
    if (!m) throw Error(kErrInvalid, "model is NULL");
    TFFN_CUDA(cudaSetDevice(m->device));
    ExpertFile ef(path);
    const Config& c = m->cfg;
    if ((int)ef.hdr.num_layers != c.num_layers || (int)ef.hdr.hidden != c.hidden_size ||
        (int)ef.hdr.intermediate != c.intermediate_size) {
        char buf[256];
        snprintf(buf, sizeof buf, "Expert shape mismatch: checkpoint=%u×%u×%u, model=%d×%d×%d", ef.hdr.num_layers,
                 ef.hdr.hidden, ef.hdr.intermediate, c.num_layers, c.hidden_size, c.intermediate_size);
        throw Error(kErrShape, buf);
    }
    std::unique_ptr<Expert> e(new Expert());
    e->model = m;
    e->scale = scale;
    const size_t H = c.hidden_size, Ifull = c.intermediate_size, I = m->I, i0 = m->tp.i0, n = H * I;
    e->layers.resize(c.num_layers);
    e->slab.alloc_raw((Slab::padded(n * 2) + Slab::padded(n * 3 * 2)) * (size_t)c.num_layers + 256);
    Slab slab{&e->slab};
    Stager up;
    // fp32 matrices arrive in a device scratch buffer and are cast to bf16 on the staging stream, which orders
    // the buffer's reuse; no wait until the end
    DeviceBuffer stage, gate_tmp, up_tmp;
    stage.alloc_raw(n * 4);
    gate_tmp.alloc_raw(n * 2);
    up_tmp.alloc_raw(n * 2);
    for (int l = 0; l < c.num_layers; ++l) {
        FfnWeights& f = e->layers[l];
        slab.take(f.down, n * 2);
        slab.take(f.packed, n * 3 * 2);
        bf16* dst[3] = {gate_tmp.as<bf16>(), up_tmp.as<bf16>(), f.down.as<bf16>()};
        for (int k = 0; k < 3; ++k) {
            DeviceBuffer& sb = stage;
            if (k < 2)  // rows i0 .. i0 + I of [Ifull, H]
                up.copy(sb.p, ef.matrix(l, k) + i0 * H, n * 4);
            else        // columns i0 .. i0 + I of [H, Ifull]
                up.copy2d(sb.p, ef.matrix(l, k) + i0, Ifull * 4, I * 4, H);
            launch_cast_f32_bf16(sb.as<float>(), dst[k], n, up.stream());
            TFFN_CUDA(cudaGetLastError());
        }
        launch_pack_ffn(gate_tmp.as<bf16>(), up_tmp.as<bf16>(), f.down.as<bf16>(), f.packed.as<bf16>(), (int)I, (int)H, up.stream());
        TFFN_CUDA(cudaGetLastError());
    }
    up.finish();
    e->weight_bytes = (uint64_t)c.num_layers * 3 * n * 2;
    return e.release();
}

// ------------------------------------------------------------------------------------------ Session
Session::Session(const Model* m, const Expert* e, int max_batch, int max_seq, cudaStream_t stream, TpComm* tp)
    : m_(m), e_(e), tp_(tp), max_batch_(max_batch), max_seq_(max_seq), stream_(stream) {
    if (!m) throw Error(kErrInvalid, "model is NULL");
    if (m->tp.tp_size > 1) {
        if (!tp) throw Error(kErrInvalid, "the model was loaded as one tensor-parallel rank: the session needs the group's communicator");
        if (tp_comm_size(tp) != m->tp.tp_size || tp_comm_rank(tp) != m->tp.tp_rank)
            throw Error(kErrInvalid, "communicator rank / size differ from the model's tensor-parallel rank / size");
    } else {
        tp_ = nullptr;
    }
    if (e && e->model != m) throw Error(kErrInvalid, "expert was loaded for a different model");
    if (max_batch < 1 || max_batch > 4096) throw Error(kErrInvalid, "max_batch must be in [1, 4096]");
    if (max_seq < 2) throw Error(kErrInvalid, "max_seq must be at least 2");
    TFFN_CUDA(cudaSetDevice(m->device));
    if (!stream_) {
        TFFN_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
        own_stream_ = true;
    }
    const Config& c = m->cfg;
    // this rank's sizes (the whole model without tensor parallelism)
    const size_t H = c.hidden_size, I = m->I, V = c.vocab_size;
    const size_t nh = m->nh, nkv = m->nkv, hd = c.head_dim, L = c.num_layers;

    max_pages_per_seq_ = (max_seq + kPageTokens - 1) / kPageTokens;
    num_pages_ = max_batch * max_pages_per_seq_;
    const size_t layer_stride = (size_t)num_pages_ * nkv * kPageTokens * hd;
    k_pool_.alloc(L * layer_stride * 2);
    v_pool_.alloc(L * layer_stride * 2);
    h_block_table_.assign((size_t)max_batch * max_pages_per_seq_, -1);
    block_table_.alloc(h_block_table_.size() * 4);
    TFFN_CUDA(cudaMemcpy(block_table_.p, h_block_table_.data(), h_block_table_.size() * 4, cudaMemcpyHostToDevice));
    TFFN_CUDA(cudaStreamSynchronize(0));  // staged copies have reached the device before the session's own stream is used
    h_seq_len_.assign(max_batch, 0);
    h_pages_used_.assign(max_batch, 0);
    seq_len_dev_.alloc((size_t)max_batch * 4);
    free_pages_.resize(num_pages_);
    for (int i = 0; i < num_pages_; ++i) free_pages_[i] = num_pages_ - 1 - i;  // pop_back hands out 0,1,2,...
    kv_.k_pool = k_pool_.as<bf16>();
    kv_.v_pool = v_pool_.as<bf16>();
    kv_.block_table = block_table_.as<int>();
    kv_.max_pages_per_seq = max_pages_per_seq_;
    kv_.num_pages = num_pages_;
    kv_.layer_stride = layer_stride;
    kv_.nkv = (int)nkv;
    kv_.hd = (int)hd;

    // RoPE tables in float, as the reference builds them on the host (inference/src/model/qwen.cu:120-132)
    {
        const int half = (int)hd / 2;
        std::vector<float> cs((size_t)max_seq * half), sn((size_t)max_seq * half);
        for (int pos = 0; pos < max_seq; ++pos)
            for (int i = 0; i < half; ++i) {
                float freq = 1.f / powf(c.rope_theta, (float)(2 * i) / (float)hd);
                cs[(size_t)pos * half + i] = cosf(pos * freq);
                sn[(size_t)pos * half + i] = sinf(pos * freq);
            }
        upload(rope_cos_, cs.data(), cs.size() * 4);
        upload(rope_sin_, sn.data(), sn.size() * 4);
    }

    cap_tokens_ = H <= 2048 ? 4096 : 2048;
    if (cap_tokens_ < ((max_batch + 255) / 256) * 256) cap_tokens_ = ((max_batch + 255) / 256) * 256;
    const size_t T = cap_tokens_;
    tokens_.alloc(T * 4);
    tok_seq_.alloc(T * 4);
    tok_pos_.alloc(T * 4);
    row_idx_.alloc(T * 4);
    grp_first_.alloc(T * 4);
    grp_count_.alloc(T * 4);
    picks_.alloc(T * 4);
    dec_tokens_.alloc((size_t)max_batch * 4);
    {
        std::vector<int> id(T);
        for (size_t i = 0; i < T; ++i) id[i] = (int)i;
        upload(identity_, id.data(), T * 4);
    }
    h_.alloc(T * H * 2);
    xn_.alloc(T * H * 2);
    q_.alloc(T * nh * hd * 4);
    ctx_.alloc(T * nh * hd * 2);
    act_b_.alloc(T * I * 2);
    if (e_) act_e_.alloc(T * I * 2);
    xn_last_.alloc(T * H * 2);
    if (tp_) {
        delta_.alloc(T * H * 4);
        // pick exchange: 8 bytes per logits row and rank; sized for the largest launch now, so that no step
        // allocates (a step may be under stream capture)
        tp_pick_send_.alloc(T * 8);
        tp_pick_recv_.alloc(T * 8 * m_->tp.tp_size);
        // exchange window for decode-sized launches (a whole allocation of its own: it is exported to the peers)
        const int R = m_->tp.tp_size;
        if (R > kTpMaxRanks) throw Error(kErrUnsupported, "tensor-parallel groups of more than 8 ranks are not supported");
        tp_small_rows_ = (int)std::min<size_t>(T, kTpFlagBlocks);
        const size_t flag_bytes = (size_t)2 * kTpMaxRanks * kTpFlagBlocks * 4;  // hand-shakes of the reduce and of the pick
        tp_pick_off_ = flag_bytes;
        const size_t pick_bytes = (size_t)kTpMaxRanks * kTpFlagBlocks * 8;
        tp_part_off_[0] = (flag_bytes + pick_bytes) / 4;
        tp_part_off_[1] = tp_part_off_[0] + (size_t)tp_small_rows_ * H;
        size_t win_bytes = (tp_part_off_[1] + (size_t)tp_small_rows_ * H) * 4;
        win_bytes = (std::max<size_t>(win_bytes, (size_t)4 << 20) + ((size_t)2 << 20) - 1) & ~(((size_t)2 << 20) - 1);
        tp_win_.alloc(win_bytes);
        tp_calls_.alloc((size_t)2 * kTpFlagBlocks * 4);
        tp_window_open(tp_, tp_win_.p, tp_peers_, stream_);
        for (int b = 0; b < 2; ++b)
            for (int p = 0; p < kTpMaxRanks; ++p) tp_parts_[b].part[p] = p < R ? (const float*)tp_peers_[p] + tp_part_off_[b] : nullptr;
        tp_sync_.flags_local = (unsigned*)tp_win_.p;
        for (int p = 0; p < kTpMaxRanks; ++p) tp_sync_.flags_peer[p] = p < R ? (unsigned*)tp_peers_[p] : nullptr;
        tp_sync_.calls = tp_calls_.as<unsigned>();
        tp_sync_.rank = m_->tp.tp_rank;
        tp_sync_.size = R;
        tp_sync_.wait_ns = 10ull * 1000 * 1000 * 1000;
        tp_pick_sync_ = tp_sync_;
        tp_pick_sync_.flags_local += (size_t)kTpMaxRanks * kTpFlagBlocks;
        for (int p = 0; p < R; ++p) tp_pick_sync_.flags_peer[p] += (size_t)kTpMaxRanks * kTpFlagBlocks;
        tp_pick_sync_.calls += kTpFlagBlocks;
        for (int p = 0; p < kTpMaxRanks; ++p) tp_pick_parts_.part[p] = p < R ? (const float2*)((const char*)tp_peers_[p] + tp_pick_off_) : nullptr;
    }
    ensure_logits(std::max<size_t>(256, max_batch));
    attn_partials_.alloc((size_t)32 << 20);
    attn_counters_.alloc(16384 * 4);
    status_.alloc(4);
    step_counter_.alloc(4);
    TFFN_CUDA(cudaMallocHost(&h_status_, 4));
    *h_status_ = 0;

    cuda_check((cudaError_t)gemm_prepare(), "gemm_prepare", __FILE__, __LINE__);
    cuda_check((cudaError_t)attn_prepare(), "attn_prepare", __FILE__, __LINE__);
    cuda_check((cudaError_t)rows_prepare(), "rows_prepare", __FILE__, __LINE__);
    cuda_check(prefer_max_shared(k_decode_advance), "carveout", __FILE__, __LINE__);
    if (m->bs1_ok) cuda_check((cudaError_t)bs1_prepare((int)H, true), "bs1_prepare", __FILE__, __LINE__);
    bs1_h_.alloc(2 * H * 2);  // the residual stream alternates between two buffers from layer to layer
    bs1_acc_.alloc(2 * bs1_acc_words((int)H) * 8);
    bs1_q_.alloc(nh * hd * 4);
    bs1_ctx_.alloc(nh * hd * 2);
    bs1_tickets_.alloc(256 * 4);
    bs1_lm_val_.alloc((size_t)m->num_sms * 2 * 4);
    bs1_lm_idx_.alloc((size_t)m->num_sms * 2 * 4);
    (void)V;
}

Session::~Session() {
    cudaSetDevice(m_->device);
    cudaStreamSynchronize(stream_);
    drop_graphs();
    tmap_cache_free(tmaps_);
    if (tp_ && tp_win_.p) {
        // collective, like the constructor: the window may be freed only when no peer has it mapped any more;
        // if a peer does not arrive, the window is left allocated
        if (!tp_window_close(tp_, tp_peers_, stream_, 10.0)) tp_win_.p = nullptr;
    }
    prof_resolve();
    for (cudaEvent_t e : prof_free_) cudaEventDestroy(e);
    if (h_status_) cudaFreeHost(h_status_);
    if (h_pinned_i32_) cudaFreeHost(h_pinned_i32_);
    if (h_sample_u_) cudaFreeHost(h_sample_u_);
    if (own_stream_) cudaStreamDestroy(stream_);
}

int32_t* Session::pinned_i32(size_t n) {
    if (n > h_pinned_cap_) {
        if (h_pinned_i32_) cudaFreeHost(h_pinned_i32_);
        h_pinned_i32_ = nullptr;
        size_t cap = std::max<size_t>(n, 4096);
        TFFN_CUDA(cudaMallocHost(&h_pinned_i32_, cap * 4));
        h_pinned_cap_ = cap;
    }
    return h_pinned_i32_;
}

GemmWorkspace Session::gemm_ws() const {
    GemmWorkspace w;
    w.status = status_.as<int>();
    w.num_sms = m_->num_sms;
    w.tmaps = tmaps_;
    return w;
}
AttnWorkspace Session::attn_ws() const {
    AttnWorkspace w;
    w.partials = attn_partials_.as<float>();
    w.partial_floats = attn_partials_.bytes / 4;
    w.counters = attn_counters_.as<int>();
    w.num_counters = (int)(attn_counters_.bytes / 4);
    return w;
}

void Session::ensure_logits(size_t rows) {
    if (rows <= logits_rows_) return;
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    logits_.alloc(rows * (size_t)m_->V * 4);  // this rank's vocabulary slice
    if (tp_) tp_logits_.alloc(rows * (size_t)m_->V * 4 * m_->tp.tp_size);
    logits_rows_ = rows;
    drop_graphs();  // captured steps hold the old pointer
}
// fp32 logits rows [0, rows) of the last LM-head launch -> host [rows, vocab]. With tensor parallelism
// every rank holds its slice of the vocabulary: the slices are all-gathered on the device and laid out
// side by side by the copies. Asynchronous on the session's stream.
void Session::copy_logits_to_host(float* dst, size_t rows) {
    const size_t V = m_->cfg.vocab_size, Vl = m_->V;
    if (!tp_) {
        TFFN_CUDA(cudaMemcpyAsync(dst, logits_.p, rows * V * 4, cudaMemcpyDeviceToHost, stream_));
        return;
    }
    const int n = m_->tp.tp_size;
    if (Vl * n != V) throw Error(kErrUnsupported, "tensor parallel: the vocabulary does not split evenly, logits cannot be gathered");
    tp_all_gather_bytes(tp_, logits_.p, tp_logits_.p, rows * Vl * 4, stream_);
    for (int r = 0; r < n; ++r)
        TFFN_CUDA(cudaMemcpy2DAsync(dst + (size_t)r * Vl, V * 4, tp_logits_.as<float>() + (size_t)r * rows * Vl, Vl * 4, Vl * 4, rows,
                                    cudaMemcpyDeviceToHost, stream_));
}

void Session::ensure_ring(int entries) {
    if (entries <= out_ring_cap_) return;
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    out_ring_.alloc((size_t)entries * 4);
    out_ring_cap_ = entries;
    drop_graphs();
}

void Session::reset(int slot) {
    if (slot < -1 || slot >= max_batch_) throw Error(kErrInvalid, "slot out of range");
    TFFN_CUDA(cudaSetDevice(m_->device));
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    const int s0 = slot < 0 ? 0 : slot, s1 = slot < 0 ? max_batch_ : slot + 1;
    for (int s = s0; s < s1; ++s) {
        for (int p = h_pages_used_[s] - 1; p >= 0; --p) {
            int& e = h_block_table_[(size_t)s * max_pages_per_seq_ + p];
            if (e >= 0) free_pages_.push_back(e);
            e = -1;
        }
        h_pages_used_[s] = 0;
        h_seq_len_[s] = 0;
    }
    table_dirty_ = true;
    flush_tables();
    TFFN_CUDA(cudaMemcpyAsync(seq_len_dev_.p, h_seq_len_.data(), (size_t)max_batch_ * 4, cudaMemcpyHostToDevice, stream_));
    TFFN_CUDA(cudaStreamSynchronize(stream_));
}

void Session::ensure_pages(int slot, int new_len) {
    if (new_len > max_seq_) {
        char buf[160];
        snprintf(buf, sizeof buf, "KV cache overflow: slot %d would hold %d tokens, capacity %d — increase --max-seq", slot,
                 new_len, max_seq_);
        throw Error(kErrCapacity, buf);
    }
    const int need = (new_len + kPageTokens - 1) / kPageTokens;
    while (h_pages_used_[slot] < need) {
        if (free_pages_.empty()) throw Error(kErrCapacity, "KV page pool exhausted");
        const int pg = free_pages_.back();
        free_pages_.pop_back();
        h_block_table_[(size_t)slot * max_pages_per_seq_ + h_pages_used_[slot]] = pg;
        h_pages_used_[slot]++;
        table_dirty_ = true;
    }
}
void Session::flush_tables() {
    if (!table_dirty_) return;
    // the host vector may change again before the copy runs, so stage it in pinned memory
    int32_t* pin = pinned_i32(h_block_table_.size());
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    memcpy(pin, h_block_table_.data(), h_block_table_.size() * 4);
    TFFN_CUDA(cudaMemcpyAsync(block_table_.p, pin, h_block_table_.size() * 4, cudaMemcpyHostToDevice, stream_));
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    table_dirty_ = false;
}

void Session::set_sampling(float temperature, uint32_t seed) {
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    drop_graphs();  // the pick kernel is part of the captured step
    sample_temp_ = temperature > 0.f ? temperature : 0.f;
    sample_rng_.seed(seed);
}

void Session::upload_draws(size_t n) {
    if (n > h_sample_cap_) {
        TFFN_CUDA(cudaStreamSynchronize(stream_));
        if (h_sample_u_) cudaFreeHost(h_sample_u_);
        h_sample_u_ = nullptr;
        const size_t cap = std::max<size_t>(n, 1024);
        TFFN_CUDA(cudaMallocHost(&h_sample_u_, cap * 8));
        h_sample_cap_ = cap;
        sample_u_.alloc(cap * 8);
        drop_graphs();  // captured steps hold the old address of the draws
    } else {
        TFFN_CUDA(cudaStreamSynchronize(stream_));  // the staging buffer may still feed an earlier copy
    }
    std::uniform_real_distribution<double> canonical(0.0, 1.0);  // r = u * sum, as dist(0, sum) computes it
    for (size_t i = 0; i < n; ++i) h_sample_u_[i] = canonical(sample_rng_);
    TFFN_CUDA(cudaMemcpyAsync(sample_u_.p, h_sample_u_, n * 8, cudaMemcpyHostToDevice, stream_));
}

void Session::set_launch_mode(int mode) {
    if (mode < 0 || mode > 2) throw Error(kErrInvalid, "launch mode must be 0, 1 or 2");
    launch_mode_ = mode;
}

void Session::set_tp_fused(bool on) {
    if (on == tp_fused_) return;
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    tp_fused_ = on;
    drop_graphs();
}
void Session::set_ablation(unsigned mask) {
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    for (auto& kv : dec_graphs_) cudaGraphExecDestroy(kv.second.exec);
    dec_graphs_.clear();
    ablate_mask_ = mask;
}

void Session::capture_hidden(int max_rows) {
    if (max_rows < 0) throw Error(kErrInvalid, "max_rows must be >= 0");
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    hidden_rows_cap_ = max_rows;
    hidden_rows_ = 0;
    if (max_rows > 0) hidden_.alloc((size_t)m_->cfg.num_layers * max_rows * m_->cfg.hidden_size * 2);
    else hidden_.release();
}
int Session::get_hidden(int layer, uint16_t* dst, int max_rows) {
    if (layer < 0 || layer >= m_->cfg.num_layers || !dst) throw Error(kErrInvalid, "bad layer or destination");
    const int rows = std::min(hidden_rows_, max_rows);
    if (rows <= 0) return 0;
    const size_t H = m_->cfg.hidden_size;
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    TFFN_CUDA(cudaMemcpy(dst, hidden_.as<bf16>() + (size_t)layer * hidden_rows_cap_ * H, (size_t)rows * H * 2, cudaMemcpyDeviceToHost));
    return rows;
}

int Session::status() {
    TFFN_CUDA(cudaMemcpyAsync(h_status_, status_.p, 4, cudaMemcpyDeviceToHost, stream_));
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    return *h_status_;
}
void Session::check_status() {
    const int st = status();
    if (st != 0) {
        TFFN_CUDA(cudaMemsetAsync(status_.p, 0, 4, stream_));
        char buf[128];
        snprintf(buf, sizeof buf, "a kernel reported device status %d (1-3: a bounded wait ran out, 4: index out of range)", st);
        throw Error(kErrDevice, buf);
    }
}

// ---------------------------------------------------------------- per-launch profile
const char* kclass_name(int c) {
    static const char* names[KC_COUNT] = {"embed_rows", "rmsnorm_rows", "gemm_tc:qkv", "attn_decode",
                                          "gemm_tc:o_proj", "gemm_tc:gate_up_swiglu", "gemm_tc:down", "gemm_tc:lm_head",
                                          "argmax_rows", "decode_advance", "bs1_qkv", "bs1_oproj", "bs1_ffn", "bs1_lmhead", "tp_all_reduce"};
    return (c >= 0 && c < KC_COUNT) ? names[c] : "?";
}
void Session::set_profile(bool on) {
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    prof_resolve();
    profile_ = on;
    if (on) {
        memset(prof_ms_, 0, sizeof prof_ms_);
        memset(prof_n_, 0, sizeof prof_n_);
    }
}
void Session::prof_begin(int cls) {
    if (!profile_) return;
    if (prof_recs_.size() >= 8192) {
        TFFN_CUDA(cudaStreamSynchronize(stream_));
        prof_resolve();
    }
    ProfRec r;
    r.cls = cls;
    for (cudaEvent_t* e : {&r.a, &r.b}) {
        if (!prof_free_.empty()) {
            *e = prof_free_.back();
            prof_free_.pop_back();
        } else {
            TFFN_CUDA(cudaEventCreate(e));
        }
    }
    TFFN_CUDA(cudaEventRecord(r.a, stream_));
    prof_recs_.push_back(r);
}
void Session::prof_end() {
    if (!profile_) return;
    TFFN_CUDA(cudaEventRecord(prof_recs_.back().b, stream_));
}
void Session::prof_resolve() {
    for (auto& r : prof_recs_) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
            prof_ms_[r.cls] += ms;
            prof_n_[r.cls] += 1;
        }
        prof_free_.push_back(r.a);
        prof_free_.push_back(r.b);
    }
    prof_recs_.clear();
}
int Session::read_profile(float* ms, int* counts, int cap) {
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    prof_resolve();
    for (int i = 0; i < KC_COUNT && i < cap; ++i) {
        if (ms) ms[i] = prof_ms_[i];
        if (counts) counts[i] = prof_n_[i];
    }
    return KC_COUNT;
}

// ---------------------------------------------------------------- batched path (tensor-core GEMMs)
int Session::build_groups(const int* seq, const int* pos, int T, int32_t* first, int32_t* count) {
    int n = 0;
    for (int i = 0; i < T; ++i) {
        const bool extend = n > 0 && count[n - 1] < 8 && seq[i] == seq[i - 1] && pos[i] == pos[i - 1] + 1;
        if (extend) {
            ++count[n - 1];
        } else {
            first[n] = i;
            count[n] = 1;
            ++n;
        }
    }
    return n;
}

void Session::run_batched(int T, int n_logit_rows, bool logit_rows_are_all, bool decode, int max_ctx, int n_groups) {
    const Config& c = m_->cfg;
    // this rank's slice of the heads, of the intermediate dimension and of the LM head (everything without
    // tensor parallelism); the vocabulary of the embedding is always the whole one
    const int H = c.hidden_size, I = m_->I, V = c.vocab_size, Vl = m_->V;
    const int nh = m_->nh, nkv = m_->nkv, hd = c.head_dim;
    const int nqkv = (nh + 2 * nkv) * hd;
    const bool tp = tp_ != nullptr;
    // Tensor parallel: the projections that end a block (o_proj, down) leave fp32 partial sums over this
    // rank's heads / intermediate slice; they are all-reduced in fp32 (NCCL, on this stream, this GPU's own
    // buffer) and only then added into the bf16 residual stream, one rounding as in the single-GPU order
    // (inference/src/model/qwen.cu:282-285). The row kernel that adds them also forms the next RMSNorm.
    auto all_reduce_delta = [&](int rows) {
        prof_begin(KC_ALLREDUCE);
        tp_all_reduce_f32(tp_, delta_.as<float>(), (size_t)rows * H, stream_);
        prof_end();
        launches_++;
    };
    const bool pdl = launch_mode_ >= 1 && !profile_;
    // decode-sized launches: partial sums left in this rank's exchange window, read by every rank's row kernel
    // over NVLink after a flag hand-shake (buffer 0 after o_proj, buffer 1 after down)
    const bool fused = tp && tp_fused_ && T <= tp_small_rows_;
    auto reduce_fused = [&](int which, const bf16* norm_w) {
        prof_begin(KC_ALLREDUCE);
        launch_tp_reduce_residual_norm(h_.as<bf16>(), tp_parts_[which], tp_sync_, norm_w, xn_.as<bf16>(), T, H, c.rms_norm_eps,
                                       status_.as<int>(), stream_, pdl, tl_next(KC_ALLREDUCE));
        prof_end();
        launches_++;
    };
    const int* tokens = decode ? dec_tokens_.as<int>() : tokens_.as<int>();
    const int* tok_seq = decode ? identity_.as<int>() : tok_seq_.as<int>();
    const int* tok_pos = decode ? seq_len_dev_.as<int>() : tok_pos_.as<int>();
    int* status = status_.as<int>();
    const GemmWorkspace gws = gemm_ws();
    // timing-only ablation: a class in the mask is not launched (results are then meaningless)
    auto live = [&](int cls) { return ((ablate_mask_ >> cls) & 1u) == 0; };
    auto gemm = [&](GemmCall& call, int cls) {
        if (!live(cls)) return;
        call.pdl = pdl;
        call.tl = tl_next(cls);
        call.trace = (tl_on_ && (int)tl_cls_.size() - 1 == tl_trace_launch_) ? tl_trace_buf_.as<unsigned long long>() : nullptr;
        call.trace_ctas = (int)(tl_trace_buf_.bytes / (64 * 8));
        prof_begin(cls);
        int rc = launch_gemm(call, gws, stream_);
        prof_end();
        if (rc == -1000) throw Error(kErrCuda, "cuTensorMapEncodeTiled failed or is unavailable");
        if (rc != 0) cuda_check((cudaError_t)rc, "tensor-core GEMM launch", __FILE__, __LINE__);
        launches_++;
    };
    prof_begin(KC_EMBED);
    launch_embed(tokens, m_->embed.as<bf16>(), h_.as<bf16>(), T, H, V, status, stream_, false, tl_next(KC_EMBED));
    prof_end();
    launches_++;
    for (int l = 0; l < c.num_layers; ++l) {
        const LayerWeights& ly = m_->layers[l];
        if (!tp || l == 0) {  // with tensor parallelism the later layers' norm comes out of the residual kernel
            prof_begin(KC_RMSNORM);
            if (live(KC_RMSNORM))
                launch_rmsnorm(h_.as<bf16>(), ly.attn_norm.as<bf16>(), xn_.as<bf16>(), T, H, c.rms_norm_eps, nullptr, stream_, pdl,
                               tl_next(KC_RMSNORM));
            prof_end();
        }
        GemmCall g;
        memset(&g, 0, sizeof g);
        g.x_rows_alloc = cap_tokens_;
        g.T = T;
        g.alpha = 1.f;
        // q|k|v rows in one GEMM; bias, RoPE and the page writes happen in its epilogue
        const bf16* b = ly.has_bias ? ly.bqkv.as<bf16>() : nullptr;
        GemmQkvEpilogue qe;
        qe.bias = b;
        qe.rope_cos = rope_cos_.as<float>();
        qe.rope_sin = rope_sin_.as<float>();
        qe.tok_seq = tok_seq;
        qe.tok_pos = tok_pos;
        qe.q_out = q_.as<float>();
        qe.kv = kv_;
        qe.layer = l;
        qe.nh = nh;
        qe.max_pos = max_seq_;
        g.op[0] = {ly.wqkv.as<bf16>(), H, xn_.as<bf16>(), H, H};
        g.op[1] = {nullptr, 0, nullptr, 0, 0};
        g.N = nqkv;
        g.mode = GEMM_QKV;
        g.qkv = &qe;
        g.out = nullptr;
        g.ldo = nqkv;
        gemm(g, KC_GEMM_QKV);
        g.qkv = nullptr;
        prof_begin(KC_ATTENTION);
        if (live(KC_ATTENTION) && n_groups > 0) {
            // prompt rows: eight consecutive tokens of a sequence share one pass over its cache
            launch_attention_prefill(q_.as<float>(), kv_, l, tok_seq, tok_pos, grp_first_.as<int>(), grp_count_.as<int>(), n_groups,
                                     ctx_.as<bf16>(), nh, status, stream_, pdl, tl_next(KC_ATTENTION));
        } else if (live(KC_ATTENTION)) {
            unsigned long long* tl = tl_next(KC_ATTENTION);
            const bool traced = tl_on_ && (int)tl_cls_.size() - 1 == tl_trace_launch_;
            launch_attention(q_.as<float>(), kv_, l, tok_seq, tok_pos, ctx_.as<bf16>(), T, nh, max_ctx, attn_ws(), m_->num_sms,
                             status, stream_, pdl, decode /* the step's first kernel (embed) is a full dependency */, tl,
                             traced ? tl_trace_buf_.as<unsigned long long>() : nullptr, (int)(tl_trace_buf_.bytes / (16 * 8)));
        }
        prof_end();
        // o_proj + residual
        g.op[0] = {ly.wo.as<bf16>(), nh * hd, ctx_.as<bf16>(), nh * hd, nh * hd};
        g.N = H;
        g.mode = tp ? GEMM_STORE_F32 : GEMM_RESIDUAL;
        g.out = fused ? (void*)((float*)tp_win_.p + tp_part_off_[0]) : tp ? delta_.p : h_.p;
        g.ldo = H;
        gemm(g, KC_GEMM_OPROJ);
        prof_begin(KC_RMSNORM);
        if (fused) {
            prof_end();
            reduce_fused(0, ly.ffn_norm.as<bf16>());
            prof_begin(KC_RMSNORM);
        } else if (tp) {
            prof_end();
            all_reduce_delta(T);
            prof_begin(KC_RMSNORM);
            launch_residual_norm(h_.as<bf16>(), delta_.as<float>(), ly.ffn_norm.as<bf16>(), xn_.as<bf16>(), T, H, c.rms_norm_eps,
                                 stream_, pdl);
        } else if (live(KC_RMSNORM)) {
            launch_rmsnorm(h_.as<bf16>(), ly.ffn_norm.as<bf16>(), xn_.as<bf16>(), T, H, c.rms_norm_eps, nullptr, stream_, pdl,
                           tl_next(KC_RMSNORM));
        }
        prof_end();
        launches_ += 3;
        // gate|up with the SwiGLU epilogue: strided views of the [I][3][H] records; the expert's
        // gate|up rides in the same launch as a second, independent problem
        {
            const bf16* rec = ly.ffn.packed.as<bf16>();
            g.op[0] = {rec, (int64_t)3 * H, xn_.as<bf16>(), H, H};
            g.op[1] = {rec + H, (int64_t)3 * H, xn_.as<bf16>(), H, H};
            g.N = I;
            g.mode = GEMM_SWIGLU;
            g.out = act_b_.p;
            g.ldo = I;
            if (e_) {
                const bf16* erec = e_->layers[l].packed.as<bf16>();
                g.op2[0] = {erec, (int64_t)3 * H, xn_.as<bf16>(), H, H};
                g.op2[1] = {erec + H, (int64_t)3 * H, xn_.as<bf16>(), H, H};
                g.out2 = act_e_.p;
            }
            gemm(g, KC_GEMM_GATEUP);
            g.out2 = nullptr;
        }
        // down projections of base and expert into two accumulators, summed in fp32, + residual
        g.op[0] = {ly.ffn.down.as<bf16>(), I, act_b_.as<bf16>(), I, I};
        if (e_) {
            g.op[1] = {e_->layers[l].down.as<bf16>(), I, act_e_.as<bf16>(), I, I};
            g.alpha = e_->scale;
        } else {
            g.op[1] = {nullptr, 0, nullptr, 0, 0};
        }
        g.N = H;
        g.mode = tp ? GEMM_STORE_F32 : GEMM_RESIDUAL;
        g.out = fused ? (void*)((float*)tp_win_.p + tp_part_off_[1]) : tp ? delta_.p : h_.p;
        g.ldo = H;
        gemm(g, KC_GEMM_DOWN);
        g.alpha = 1.f;
        if (fused) {
            reduce_fused(1, l + 1 < c.num_layers ? m_->layers[l + 1].attn_norm.as<bf16>() : nullptr);
        } else if (tp) {
            all_reduce_delta(T);
            const bf16* next_norm = l + 1 < c.num_layers ? m_->layers[l + 1].attn_norm.as<bf16>() : nullptr;
            prof_begin(KC_RMSNORM);
            launch_residual_norm(h_.as<bf16>(), delta_.as<float>(), next_norm, xn_.as<bf16>(), T, H, c.rms_norm_eps, stream_, pdl);
            prof_end();
            launches_++;
        }
        if (hidden_rows_cap_ > 0) {
            const int rows = std::min(T, hidden_rows_cap_);
            const size_t n16 = (size_t)rows * H / 8;
            k_copy_rows_bf16<<<(unsigned)((n16 + 255) / 256), 256, 0, stream_>>>(
                h_.as<bf16>(), hidden_.as<bf16>() + (size_t)l * hidden_rows_cap_ * H, n16);
            hidden_rows_ = rows;
            launches_++;
        }
    }
    if (n_logit_rows > 0) {
        const int* rows = logit_rows_are_all ? nullptr : row_idx_.as<int>();
        prof_begin(KC_RMSNORM);
        launch_rmsnorm(h_.as<bf16>(), m_->final_norm.as<bf16>(), xn_last_.as<bf16>(), n_logit_rows, H, c.rms_norm_eps, rows, stream_, pdl,
                       tl_next(KC_RMSNORM));
        prof_end();
        GemmCall g;
        memset(&g, 0, sizeof g);
        g.x_rows_alloc = cap_tokens_;
        g.T = n_logit_rows;
        g.alpha = 1.f;
        g.op[0] = {m_->lm_head, H, xn_last_.as<bf16>(), H, H};
        g.N = Vl;  // this rank's rows of the vocabulary
        g.mode = GEMM_STORE_F32;
        g.ldo = Vl;
        // The greedy pick rides in the LM head's epilogue (per-tile maxima, combined by a tiny kernel); the
        // fp32 logits themselves are written only when the caller asked for them. The attention workspace is
        // idle by now and serves as scratch.
        const AttnWorkspace aw = attn_ws();
        const int v_tiles = (Vl + 127) / 128;
        const bool fused_pick = !sampling() && (size_t)n_logit_rows * v_tiles * 2 <= aw.partial_floats;
        if (tp && !fused_pick) throw Error(kErrUnsupported, "tensor parallel: sampling and very large logit batches are not split across ranks");
        if (fused_pick) {
            g.amax_val = aw.partials;
            g.amax_idx = (int*)(aw.partials + (size_t)n_logit_rows * v_tiles);
        }
        g.out = (store_logits_ || !fused_pick) ? logits_.p : nullptr;
        gemm(g, KC_GEMM_LMHEAD);
        prof_begin(KC_ARGMAX);
        if (live(KC_ARGMAX)) {
            if (fused_pick && tp) {
                // every rank's best of its vocabulary slice, exchanged (8 bytes per row and rank), then the same
                // pick on every rank: largest value, lowest global index among equals (main.cpp:45-51)
                const size_t bytes = (size_t)n_logit_rows * 8;
                if (tp_pick_send_.bytes < bytes) throw Error(kErrCapacity, "tensor parallel: more logits rows than the session was sized for");
                if (tp_fused_ && n_logit_rows <= tp_small_rows_) {
                    // candidates left in this rank's window, the pick kernel hand-shakes and loads every rank's: no NCCL call
                    // in a decode step
                    launch_argmax_tiles(g.amax_val, g.amax_idx, n_logit_rows, v_tiles, picks_.as<int>(), stream_, pdl, tl_next(KC_ARGMAX),
                                        (char*)tp_win_.p + tp_pick_off_, m_->tp.v0);
                    launch_tp_pick_peer(tp_pick_parts_, tp_pick_sync_, n_logit_rows, picks_.as<int>(), status_.as<int>(), stream_, pdl);
                    launches_ += 1;
                } else {
                    launch_argmax_tiles(g.amax_val, g.amax_idx, n_logit_rows, v_tiles, picks_.as<int>(), stream_, pdl, tl_next(KC_ARGMAX),
                                        tp_pick_send_.p, m_->tp.v0);
                    tp_all_gather_bytes(tp_, tp_pick_send_.p, tp_pick_recv_.p, bytes, stream_);
                    launch_tp_pick(tp_pick_recv_.p, m_->tp.tp_size, n_logit_rows, picks_.as<int>(), stream_, pdl);
                    launches_ += 2;
                }
            } else if (fused_pick)
                launch_argmax_tiles(g.amax_val, g.amax_idx, n_logit_rows, v_tiles, picks_.as<int>(), stream_, pdl, tl_next(KC_ARGMAX));
            else if (sampling())
                launch_sample(logits_.as<float>(), n_logit_rows, V, sample_temp_, sample_u_.as<double>(),
                              decode ? step_counter_.as<int>() : nullptr, picks_.as<int>(), stream_, pdl, tl_next(KC_ARGMAX));
            else
                launch_argmax(logits_.as<float>(), n_logit_rows, V, picks_.as<int>(), aw.partials, aw.partial_floats, aw.counters,
                              aw.num_counters, m_->num_sms, stream_, pdl, tl_next(KC_ARGMAX));
        }
        prof_end();
        launches_ += 2;
    }
    TFFN_CUDA(cudaGetLastError());
}

// ---------------------------------------------------------------- batch-1 path
Bs1Ctx Session::bs1_ctx(bool want_logits) const {
    const Config& c = m_->cfg;
    Bs1Ctx x;
    memset(&x, 0, sizeof x);
    x.H = c.hidden_size; x.I = c.intermediate_size; x.nh = c.num_heads; x.nkv = c.num_kv_heads; x.hd = c.head_dim;
    x.V = c.vocab_size;
    x.eps = c.rms_norm_eps;
    x.expert_scale = e_ ? e_->scale : 0.f;
    x.rope_cos = rope_cos_.as<float>();
    x.rope_sin = rope_sin_.as<float>();
    x.max_pos = max_seq_;
    x.h = bs1_h_.as<bf16>();
    x.q = bs1_q_.as<float>();
    x.ctx = bs1_ctx_.as<bf16>();
    x.token = dec_tokens_.as<int>();
    x.seq_len = seq_len_dev_.as<int>();
    x.slot = 0;
    x.tickets = bs1_tickets_.as<int>();
    x.lm_val = bs1_lm_val_.as<float>();
    x.lm_idx = bs1_lm_idx_.as<int>();
    x.logits = want_logits ? logits_.as<float>() : nullptr;
    x.out_tokens = out_ring_.as<int>();
    x.step_counter = step_counter_.as<int>();
    x.status = status_.as<int>();
    x.num_sms = m_->num_sms;
    return x;
}

void Session::launch_bs1_step(bool want_logits, bool pdl) {
    const Config& c = m_->cfg;
    Bs1Ctx x = bs1_ctx(want_logits);
    const size_t acc_words = bs1_acc_words(c.hidden_size);
    auto hbuf = [&](int k) { return bs1_h_.as<bf16>() + (size_t)(k & 1) * c.hidden_size; };
    auto accbuf = [&](int k) { return bs1_acc_.as<long long>() + (size_t)(k & 1) * acc_words; };
    for (int l = 0; l < c.num_layers; ++l) {
        // layer l reads the residual stream of layer l - 1 plus the sums its FFN left, and owns the other buffer
        x.h_in = hbuf(l);
        x.h = hbuf(l + 1);
        x.acc_in = l > 0 ? accbuf(l - 1) : nullptr;
        x.acc_out = accbuf(l);
        const LayerWeights& lw = m_->layers[l];
        Bs1Layer ly;
        ly.wqkv = lw.wqkv.as<bf16>();
        ly.bqkv = lw.has_bias ? lw.bqkv.as<bf16>() : nullptr;
        ly.wo = lw.wo.as<bf16>();
        ly.attn_norm = lw.attn_norm.as<bf16>();
        ly.ffn_norm = lw.ffn_norm.as<bf16>();
        ly.ffn_base = lw.ffn.packed.as<bf16>();
        ly.ffn_expert = e_ ? e_->layers[l].packed.as<bf16>() : nullptr;
        x.tl = tl_next(KC_BS1_QKV);
        prof_begin(KC_BS1_QKV);
        // the first kernel of a step is a full dependency: what earlier steps wrote (sequence length,
        // older cache rows) is then stable for every kernel of this step, also ahead of its grid wait
        launch_bs1_qkv(x, ly, m_->embed.as<bf16>(), kv_, l, l == 0, stream_, pdl && l > 0);
        prof_end();
        prof_begin(KC_ATTENTION);
        launch_attention(x.q, kv_, l, identity_.as<int>(), seq_len_dev_.as<int>(), x.ctx, 1, c.num_heads, max_seq_, attn_ws(),
                         m_->num_sms, status_.as<int>(), stream_, pdl, true, tl_next(KC_ATTENTION));
        prof_end();
        x.tl = tl_next(KC_BS1_OPROJ);
        prof_begin(KC_BS1_OPROJ);
        launch_bs1_oproj(x, ly, stream_, pdl);
        prof_end();
        x.tl = tl_next(KC_BS1_FFN);
        // per-CTA phase stamps of this launch if the timeline call asked for it (16 u64 per CTA)
        x.trace = (tl_on_ && (int)tl_cls_.size() - 1 == tl_trace_launch_) ? tl_trace_buf_.as<unsigned long long>() : nullptr;
        prof_begin(KC_BS1_FFN);
        launch_bs1_ffn(x, ly, stream_, pdl);
        prof_end();
    }
    x.h_in = hbuf(c.num_layers);
    x.h = nullptr;
    x.acc_in = accbuf(c.num_layers - 1);
    x.acc_out = nullptr;
    x.tl = tl_next(KC_BS1_LMHEAD);
    prof_begin(KC_BS1_LMHEAD);
    launch_bs1_lmhead(x, m_->final_norm.as<bf16>(), m_->lm_head, stream_, pdl);
    prof_end();
    launches_ += (uint64_t)c.num_layers * 4 + 1;
}

void Session::run_bs1(bool want_logits) {
    if (launch_mode_ == 2 && !profile_) {
        if (!bs1_graph_ || bs1_graph_logits_ != want_logits) {
            if (bs1_graph_) {
                cudaGraphExecDestroy(bs1_graph_);
                bs1_graph_ = nullptr;
            }
            cudaGraph_t graph = nullptr;
            const uint64_t before = launches_;
            TFFN_CUDA(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
            launch_bs1_step(want_logits, true);
            cudaError_t ce = cudaStreamEndCapture(stream_, &graph);
            launches_ = before;
            TFFN_CUDA(ce);
            TFFN_CUDA(cudaGraphInstantiate(&bs1_graph_, graph, 0));
            cudaGraphDestroy(graph);
            bs1_graph_logits_ = want_logits;
        }
        TFFN_CUDA(cudaGraphLaunch(bs1_graph_, stream_));
        launches_ += (uint64_t)m_->cfg.num_layers * 4 + 1;
    } else {
        launch_bs1_step(want_logits, launch_mode_ >= 1);
    }
    TFFN_CUDA(cudaGetLastError());
}

unsigned long long* Session::tl_next(int cls) {
    if (!tl_on_ || (size_t)(tl_cls_.size() + 1) * 48 > tl_buf_.bytes) return nullptr;
    tl_cls_.push_back(cls);
    return tl_buf_.as<unsigned long long>() + (tl_cls_.size() - 1) * 6;
}

int Session::timeline(int n_seqs, uint64_t* out, int max_launches, int trace_launch, uint64_t* trace_out, int trace_ctas) {
    if (!out || max_launches < 1) throw Error(kErrInvalid, "bad timeline arguments");
    const bool want_trace = trace_out && trace_ctas > 0 && trace_launch >= 0;
    if (want_trace) {
        tl_trace_buf_.alloc((size_t)trace_ctas * 64 * 8);
        TFFN_CUDA(cudaMemset(tl_trace_buf_.p, 0, tl_trace_buf_.bytes));
        TFFN_CUDA(cudaStreamSynchronize(0));
    }
    tl_trace_launch_ = want_trace ? trace_launch : -1;
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    drop_graphs();
    tl_buf_.alloc((size_t)max_launches * 48);
    std::vector<uint64_t> init((size_t)max_launches * 6);
    for (size_t i = 0; i < init.size(); ++i) init[i] = (i & 1) ? 0ull : ~0ull;
    tl_on_ = true;
    try {
        for (int rep = 0; rep < 3; ++rep) {  // with graphs the first step captures, the last one is reported
            if (launch_mode_ < 2 || rep == 0) tl_cls_.clear();
            TFFN_CUDA(cudaMemcpy(tl_buf_.p, init.data(), init.size() * 8, cudaMemcpyHostToDevice));
            TFFN_CUDA(cudaStreamSynchronize(0));
            decode_run(n_seqs, 1, nullptr);
        }
    } catch (...) {
        tl_on_ = false;
        tl_trace_launch_ = -1;
        drop_graphs();
        throw;
    }
    tl_on_ = false;
    tl_trace_launch_ = -1;
    drop_graphs();
    if (want_trace) {
        TFFN_CUDA(cudaMemcpy(trace_out, tl_trace_buf_.p, tl_trace_buf_.bytes, cudaMemcpyDeviceToHost));
        tl_trace_buf_.release();
    }
    const int n = (int)tl_cls_.size();
    std::vector<uint64_t> raw((size_t)n * 6);
    TFFN_CUDA(cudaMemcpy(raw.data(), tl_buf_.p, raw.size() * 8, cudaMemcpyDeviceToHost));
    for (int i = 0; i < n; ++i) {
        out[(size_t)i * 7] = (uint64_t)tl_cls_[i];
        for (int j = 0; j < 6; ++j) out[(size_t)i * 7 + 1 + j] = raw[(size_t)i * 6 + j];
    }
    tl_buf_.release();
    return n;
}

void Session::drop_graphs() {
    if (bs1_graph_) cudaGraphExecDestroy(bs1_graph_);
    bs1_graph_ = nullptr;
    for (auto& kv : dec_graphs_) cudaGraphExecDestroy(kv.second.exec);
    dec_graphs_.clear();
}

// one decode step of n_seqs slots on the tensor-core path, then publish picks / advance lengths
void Session::run_decode_batched(int n_seqs, int max_ctx) {
    auto body = [&] {
        run_batched(n_seqs, n_seqs, true, true, max_ctx);
        prof_begin(KC_ADVANCE);
        k_decode_advance<<<1, 256, 0, stream_>>>(picks_.as<int>(), n_seqs, dec_tokens_.as<int>(), seq_len_dev_.as<int>(),
                                                 out_ring_.as<int>(), step_counter_.as<int>());
        prof_end();
        launches_++;
    };
    if (launch_mode_ < 2 || profile_ || hidden_rows_cap_ > 0) {
        body();
        return;
    }
    const Config& c = m_->cfg;
    const int splits = attention_splits(n_seqs, c.num_heads, c.num_kv_heads, c.head_dim, max_ctx, attn_ws(), m_->num_sms);
    const auto key = std::make_pair(n_seqs, splits * 2 + (store_logits_ ? 1 : 0));
    auto it = dec_graphs_.find(key);
    if (it == dec_graphs_.end()) {
        cudaGraph_t graph = nullptr;
        const uint64_t before = launches_;
        TFFN_CUDA(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
        try {
            body();
        } catch (...) {
            cudaStreamEndCapture(stream_, &graph);
            if (graph) cudaGraphDestroy(graph);
            throw;
        }
        cudaError_t ce = cudaStreamEndCapture(stream_, &graph);
        const uint64_t n_launch = launches_ - before;
        launches_ = before;
        TFFN_CUDA(ce);
        cudaGraphExec_t exec = nullptr;
        TFFN_CUDA(cudaGraphInstantiate(&exec, graph, 0));
        cudaGraphDestroy(graph);
        it = dec_graphs_.emplace(key, DecGraph{exec, n_launch}).first;
    }
    TFFN_CUDA(cudaGraphLaunch(it->second.exec, stream_));
    launches_ += it->second.launches;
}

// ---------------------------------------------------------------- public operations
void Session::prefill(const int32_t* tokens, const int32_t* seq_lens, int n_seqs, int32_t* next_tokens, float* logits_last) {
    if (!tokens || !seq_lens || n_seqs < 1 || n_seqs > max_batch_) throw Error(kErrInvalid, "bad prefill arguments");
    TFFN_CUDA(cudaSetDevice(m_->device));
    const int V = m_->cfg.vocab_size;
    size_t total = 0;
    for (int s = 0; s < n_seqs; ++s) {
        if (seq_lens[s] < 1) throw Error(kErrInvalid, "every prompt needs at least one token");
        total += seq_lens[s];
    }
    for (size_t i = 0; i < total; ++i)
        if (tokens[i] < 0 || tokens[i] >= V) throw Error(kErrInvalid, "token id out of range");
    for (int s = 0; s < n_seqs; ++s) ensure_pages(s, h_seq_len_[s] + seq_lens[s]);
    flush_tables();
    ensure_logits(std::max<size_t>(256, n_seqs));
    // flatten (slot, position) in slot order and cut into chunks of at most cap_tokens_ rows
    std::vector<int> f_tok(total), f_seq(total), f_pos(total), f_last(total, -1);
    {
        size_t o = 0;
        for (int s = 0; s < n_seqs; ++s)
            for (int i = 0; i < seq_lens[s]; ++i, ++o) {
                f_tok[o] = tokens[o];
                f_seq[o] = s;
                f_pos[o] = h_seq_len_[s] + i;
                if (i == seq_lens[s] - 1) f_last[o] = s;
            }
    }
    for (size_t c0 = 0; c0 < total; c0 += cap_tokens_) {
        const int T = (int)std::min<size_t>(cap_tokens_, total - c0);
        int32_t* pin = pinned_i32((size_t)T * 6);
        std::vector<int> last_rows, last_slots;
        int max_ctx = 1;
        for (int i = 0; i < T; ++i) {
            pin[i] = f_tok[c0 + i];
            pin[T + i] = f_seq[c0 + i];
            pin[2 * T + i] = f_pos[c0 + i];
            max_ctx = std::max(max_ctx, f_pos[c0 + i] + 1);
            if (f_last[c0 + i] >= 0) {
                last_rows.push_back(i);
                last_slots.push_back(f_last[c0 + i]);
            }
        }
        for (size_t i = 0; i < last_rows.size(); ++i) pin[3 * T + i] = last_rows[i];
        TFFN_CUDA(cudaMemcpyAsync(tokens_.p, pin, (size_t)T * 4, cudaMemcpyHostToDevice, stream_));
        TFFN_CUDA(cudaMemcpyAsync(tok_seq_.p, pin + T, (size_t)T * 4, cudaMemcpyHostToDevice, stream_));
        TFFN_CUDA(cudaMemcpyAsync(tok_pos_.p, pin + 2 * T, (size_t)T * 4, cudaMemcpyHostToDevice, stream_));
        if (!last_rows.empty())
            TFFN_CUDA(cudaMemcpyAsync(row_idx_.p, pin + 3 * T, last_rows.size() * 4, cudaMemcpyHostToDevice, stream_));
        const int n_groups = build_groups(pin + T, pin + 2 * T, T, pin + 4 * T, pin + 5 * T);
        TFFN_CUDA(cudaMemcpyAsync(grp_first_.p, pin + 4 * T, (size_t)n_groups * 4, cudaMemcpyHostToDevice, stream_));
        TFFN_CUDA(cudaMemcpyAsync(grp_count_.p, pin + 5 * T, (size_t)n_groups * 4, cudaMemcpyHostToDevice, stream_));
        store_logits_ = logits_last != nullptr || sampling();
        if (sampling() && !last_rows.empty()) upload_draws(last_rows.size());  // one draw per sequence, slot order
        run_batched(T, (int)last_rows.size(), false, false, max_ctx, n_groups);
        if (!last_rows.empty()) {
            std::vector<int> picks(last_rows.size());
            std::vector<float> rows_host;
            TFFN_CUDA(cudaMemcpyAsync(picks.data(), picks_.p, picks.size() * 4, cudaMemcpyDeviceToHost, stream_));
            if (logits_last) {
                rows_host.resize(last_rows.size() * (size_t)V);
                copy_logits_to_host(rows_host.data(), last_rows.size());
            }
            TFFN_CUDA(cudaStreamSynchronize(stream_));
            for (size_t i = 0; i < last_rows.size(); ++i) {
                if (next_tokens) next_tokens[last_slots[i]] = picks[i];
                int32_t* one = pinned_i32(4);
                one[0] = picks[i];
                TFFN_CUDA(cudaMemcpyAsync(dec_tokens_.as<int>() + last_slots[i], one, 4, cudaMemcpyHostToDevice, stream_));
                if (logits_last) memcpy(logits_last + (size_t)last_slots[i] * V, rows_host.data() + i * (size_t)V, (size_t)V * 4);
                TFFN_CUDA(cudaStreamSynchronize(stream_));
            }
        } else {
            TFFN_CUDA(cudaStreamSynchronize(stream_));
        }
    }
    for (int s = 0; s < n_seqs; ++s) h_seq_len_[s] += seq_lens[s];
    TFFN_CUDA(cudaMemcpyAsync(seq_len_dev_.p, h_seq_len_.data(), (size_t)max_batch_ * 4, cudaMemcpyHostToDevice, stream_));
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    check_status();
}

void Session::forward(int slot, const int32_t* tokens, int T, float* logits) {
    if (!tokens || T < 1 || slot < 0 || slot >= max_batch_) throw Error(kErrInvalid, "bad forward arguments");
    TFFN_CUDA(cudaSetDevice(m_->device));
    const int V = m_->cfg.vocab_size;
    for (int i = 0; i < T; ++i)
        if (tokens[i] < 0 || tokens[i] >= V) throw Error(kErrInvalid, "token id out of range");
    ensure_pages(slot, h_seq_len_[slot] + T);
    flush_tables();
    const int chunk_cap = std::min(cap_tokens_, 512);  // bounds the all-row logits buffer
    if (logits) ensure_logits(std::min(T, chunk_cap));
    // qwen_forward returns logits; the token it leaves for a following decode step is the greedy one
    struct GreedyScope {
        float& t;
        float saved;
        explicit GreedyScope(float& x) : t(x), saved(x) { t = 0.f; }
        ~GreedyScope() { t = saved; }
    } greedy_scope(sample_temp_);
    int last_pick = 0;
    for (int c0 = 0; c0 < T; c0 += chunk_cap) {
        const int n = std::min(chunk_cap, T - c0);
        int32_t* pin = pinned_i32((size_t)n * 5 + 2);  // the last two: row index in, pick out
        for (int i = 0; i < n; ++i) {
            pin[i] = tokens[c0 + i];
            pin[n + i] = slot;
            pin[2 * n + i] = h_seq_len_[slot] + c0 + i;
        }
        const int n_groups = build_groups(pin + n, pin + 2 * n, n, pin + 3 * n, pin + 4 * n);
        TFFN_CUDA(cudaMemcpyAsync(grp_first_.p, pin + 3 * n, (size_t)n_groups * 4, cudaMemcpyHostToDevice, stream_));
        TFFN_CUDA(cudaMemcpyAsync(grp_count_.p, pin + 4 * n, (size_t)n_groups * 4, cudaMemcpyHostToDevice, stream_));
        TFFN_CUDA(cudaMemcpyAsync(tokens_.p, pin, (size_t)n * 4, cudaMemcpyHostToDevice, stream_));
        TFFN_CUDA(cudaMemcpyAsync(tok_seq_.p, pin + n, (size_t)n * 4, cudaMemcpyHostToDevice, stream_));
        TFFN_CUDA(cudaMemcpyAsync(tok_pos_.p, pin + 2 * n, (size_t)n * 4, cudaMemcpyHostToDevice, stream_));
        store_logits_ = logits != nullptr;
        if (logits) {
            run_batched(n, n, true, false, h_seq_len_[slot] + c0 + n, n_groups);
            copy_logits_to_host(logits + (size_t)c0 * V, (size_t)n);
            TFFN_CUDA(cudaMemcpyAsync(pin, picks_.as<int>() + (n - 1), 4, cudaMemcpyDeviceToHost, stream_));
            TFFN_CUDA(cudaStreamSynchronize(stream_));
            last_pick = pin[0];
        } else if (c0 + n < T) {
            run_batched(n, 0, true, false, h_seq_len_[slot] + c0 + n, n_groups);
            TFFN_CUDA(cudaStreamSynchronize(stream_));
        } else {
            // no logits wanted: the LM head still runs for the last row, whose greedy pick feeds a
            // following decode step that passes no tokens
            pin[5 * n] = n - 1;
            TFFN_CUDA(cudaMemcpyAsync(row_idx_.p, pin + 5 * n, 4, cudaMemcpyHostToDevice, stream_));
            run_batched(n, 1, false, false, h_seq_len_[slot] + c0 + n, n_groups);
            TFFN_CUDA(cudaMemcpyAsync(pin + 5 * n + 1, picks_.p, 4, cudaMemcpyDeviceToHost, stream_));
            TFFN_CUDA(cudaStreamSynchronize(stream_));
            last_pick = pin[5 * n + 1];
        }
    }
    h_seq_len_[slot] += T;
    int32_t* pin = pinned_i32(4);
    pin[0] = last_pick;
    TFFN_CUDA(cudaMemcpyAsync(dec_tokens_.as<int>() + slot, pin, 4, cudaMemcpyHostToDevice, stream_));
    TFFN_CUDA(cudaMemcpyAsync(seq_len_dev_.p, h_seq_len_.data(), (size_t)max_batch_ * 4, cudaMemcpyHostToDevice, stream_));
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    check_status();
}

void Session::decode_step(const int32_t* tokens_in, int n_seqs, int32_t* next_tokens, float* logits) {
    if (n_seqs < 1 || n_seqs > max_batch_) throw Error(kErrInvalid, "n_seqs out of range");
    TFFN_CUDA(cudaSetDevice(m_->device));
    const int V = m_->cfg.vocab_size;
    for (int s = 0; s < n_seqs; ++s) ensure_pages(s, h_seq_len_[s] + 1);
    flush_tables();
    int32_t* pin = pinned_i32((size_t)std::max(n_seqs, 4));
    if (tokens_in) {
        for (int s = 0; s < n_seqs; ++s) {
            if (tokens_in[s] < 0 || tokens_in[s] >= V) throw Error(kErrInvalid, "token id out of range");
            pin[s] = tokens_in[s];
        }
        TFFN_CUDA(cudaMemcpyAsync(dec_tokens_.p, pin, (size_t)n_seqs * 4, cudaMemcpyHostToDevice, stream_));
    }
    TFFN_CUDA(cudaMemsetAsync(step_counter_.p, 0, 4, stream_));
    ensure_ring(n_seqs);
    if (logits) ensure_logits(std::max<size_t>(256, n_seqs));
    if (sampling()) upload_draws((size_t)n_seqs);
    const bool bs1 = n_seqs == 1 && use_bs1_ && m_->bs1_ok && !sampling();  // the fused batch-1 LM head picks greedily
    if (bs1) {
        run_bs1(logits != nullptr);
    } else {
        int max_ctx = 1;
        for (int s = 0; s < n_seqs; ++s) max_ctx = std::max(max_ctx, h_seq_len_[s] + 1);
        store_logits_ = logits != nullptr || sampling();
        run_decode_batched(n_seqs, max_ctx);
    }
    TFFN_CUDA(cudaMemcpyAsync(pin, dec_tokens_.p, (size_t)n_seqs * 4, cudaMemcpyDeviceToHost, stream_));
    if (logits) copy_logits_to_host(logits, (size_t)n_seqs);
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    if (next_tokens)
        for (int s = 0; s < n_seqs; ++s) next_tokens[s] = pin[s];
    for (int s = 0; s < n_seqs; ++s) h_seq_len_[s] += 1;
    check_status();
}

void Session::decode_run(int n_seqs, int steps, int32_t* tokens_out) {
    if (n_seqs < 1 || n_seqs > max_batch_ || steps < 1) throw Error(kErrInvalid, "bad decode_run arguments");
    TFFN_CUDA(cudaSetDevice(m_->device));
    for (int s = 0; s < n_seqs; ++s) ensure_pages(s, h_seq_len_[s] + steps);
    flush_tables();
    ensure_ring(n_seqs * steps);
    TFFN_CUDA(cudaMemsetAsync(step_counter_.p, 0, 4, stream_));
    if (sampling()) upload_draws((size_t)n_seqs * steps);  // step-major, slot order within a step
    const bool bs1 = n_seqs == 1 && use_bs1_ && m_->bs1_ok && !sampling();
    int max_ctx = 1;
    for (int s = 0; s < n_seqs; ++s) max_ctx = std::max(max_ctx, h_seq_len_[s] + steps);
    for (int it = 0; it < steps; ++it) {
        if (bs1) {
            run_bs1(false);
        } else {
            store_logits_ = sampling();  // a device-resident loop hands out tokens only; sampling reads the logits
            run_decode_batched(n_seqs, max_ctx);
        }
    }
    if (tokens_out)
        TFFN_CUDA(cudaMemcpyAsync(tokens_out, out_ring_.p, (size_t)n_seqs * steps * 4, cudaMemcpyDeviceToHost, stream_));
    TFFN_CUDA(cudaStreamSynchronize(stream_));
    for (int s = 0; s < n_seqs; ++s) h_seq_len_[s] += steps;
    check_status();
}

}  // namespace tffn
