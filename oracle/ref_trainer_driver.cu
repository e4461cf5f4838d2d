// TEST INFRASTRUCTURE — a thin driver around the UNMODIFIED trainer sources of the reference.
//
// Compiled together with trainer/src/model/ffn_expert.cu, trainer/src/backend/cuda_ops.cu and memory.cpp
// where they lie (see oracle/Makefile, target ref_trainer; nothing is copied) into
// oracle/_ref/ref_trainer_driver. It calls the trainer's own expert_alloc and expert_forward
// (trainer/src/model/ffn_expert.cu:19-68, 151-175) on weights and inputs read from raw files, and writes
// the fp32 deltas, so that the restatement used to check tffn_expert_forward can be pinned to them.
//
// usage: ref_trainer_driver L H I T WEIGHTS.bf16 X.bf16 OUT.f32
//   WEIGHTS.bf16: per layer gate[I*H], up[I*H], down[H*I] (bf16 bits); X.bf16: [L, T, H]; OUT.f32: [L, T, H]
#include "backend/cuda_ops.h"
#include "backend/memory.h"
#include "model/ffn_expert.h"
#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <vector>

static std::vector<uint16_t> slurp(const char* path, size_t n) {
    std::vector<uint16_t> v(n);
    FILE* f = fopen(path, "rb");
    if (!f || fread(v.data(), 2, n, f) != n) { fprintf(stderr, "cannot read %s\n", path); exit(2); }
    fclose(f);
    return v;
}

int main(int argc, char** argv) {
    if (argc != 8) { fprintf(stderr, "usage: ref_trainer_driver L H I T weights x out\n"); return 2; }
    const int L = atoi(argv[1]), H = atoi(argv[2]), I = atoi(argv[3]), T = atoi(argv[4]);
    if (L < 1 || L > model::ExpertFFN::MAX_LAYERS) { fprintf(stderr, "layer count out of range\n"); return 2; }
    const size_t n = (size_t)I * H;
    std::vector<uint16_t> w = slurp(argv[5], (size_t)L * 3 * n), x = slurp(argv[6], (size_t)L * T * H);
    cublasHandle_t cublas;
    if (cublasCreate(&cublas) != CUBLAS_STATUS_SUCCESS) return 3;
    model::ExpertFFN e;
    model::expert_alloc(e, L, H, I, T);
    for (int l = 0; l < L; ++l) {
        backend::host_to_device(e.layers[l].gate_proj, &w[((size_t)l * 3 + 0) * n], n * 2);
        backend::host_to_device(e.layers[l].up_proj, &w[((size_t)l * 3 + 1) * n], n * 2);
        backend::host_to_device(e.layers[l].down_proj, &w[((size_t)l * 3 + 2) * n], n * 2);
    }
    __nv_bfloat16* d_x = (__nv_bfloat16*)backend::device_alloc(x.size() * 2);
    float* d_out = (float*)backend::device_alloc((size_t)L * T * H * 4);
    backend::host_to_device(d_x, x.data(), x.size() * 2);
    model::expert_forward(e, cublas, d_x, d_out, T);
    cudaDeviceSynchronize();
    std::vector<float> out((size_t)L * T * H);
    backend::device_to_host(out.data(), d_out, out.size() * 4);
    FILE* f = fopen(argv[7], "wb");
    if (!f || fwrite(out.data(), 4, out.size(), f) != out.size()) return 4;
    fclose(f);
    backend::device_free(d_x);
    backend::device_free(d_out);
    model::expert_free(e);
    cublasDestroy(cublas);
    return 0;
}
