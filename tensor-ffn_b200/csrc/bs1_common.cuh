// Register-row helpers shared by the batch-1 kernels: a warp holds one row of H bf16 as 16-byte
// chunks (lane owns chunks lane, lane+32, ...), dot products accumulate in fp32, RMSNorm is
// recomputed per warp.
#pragma once
#include "kernels.h"
#include "ptx.cuh"

namespace tffn {
namespace bs1 {

// lane `lane` owns the 16-byte chunks lane, lane+32, ... of a row of H bf16 (H % 8 == 0)
template <int NCH>
struct RowRegs {
    uint4 v[NCH];
};
template <int NCH>
__device__ __forceinline__ void load_row(RowRegs<NCH>& r, const bf16* row, int H, int lane) {
    const uint4* p = (const uint4*)row;
    const int nchunk = H >> 3;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        const int c = lane + 32 * j;
        r.v[j] = (c < nchunk) ? __ldg(p + c) : make_uint4(0, 0, 0, 0);
    }
}
// Activations written by an earlier kernel: read through L2 (ld.global.cg). With programmatic
// dependent launch this CTA can share an SM with the producer grid's CTAs, whose L1 lines for
// the same buffer may predate the update.
template <int NCH>
__device__ __forceinline__ void load_row_act(RowRegs<NCH>& r, const bf16* row, int H, int lane) {
    const uint4* p = (const uint4*)row;
    const int nchunk = H >> 3;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        const int c = lane + 32 * j;
        r.v[j] = (c < nchunk) ? __ldcg(p + c) : make_uint4(0, 0, 0, 0);
    }
}
__device__ __forceinline__ float ld_bf16_cg(const bf16* p) {
    return __uint_as_float((uint32_t)__ldcg((const unsigned short*)p) << 16);
}
template <int NCH>
__device__ __forceinline__ void load_row_smem(RowRegs<NCH>& r, const uint8_t* row, int H, int lane) {
    const uint4* p = (const uint4*)row;
    const int nchunk = H >> 3;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        const int c = lane + 32 * j;
        r.v[j] = (c < nchunk) ? p[c] : make_uint4(0, 0, 0, 0);
    }
}
template <int NCH>
__device__ __forceinline__ float dot_rows(const RowRegs<NCH>& a, const RowRegs<NCH>& b) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        const uint32_t x[4] = {a.v[j].x, a.v[j].y, a.v[j].z, a.v[j].w};
        const uint32_t y[4] = {b.v[j].x, b.v[j].y, b.v[j].z, b.v[j].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            s = fmaf(bf16_lo(x[k]), bf16_lo(y[k]), s);
            s = fmaf(bf16_hi(x[k]), bf16_hi(y[k]), s);
        }
    }
    return s;
}

// xn = bf16( float(x) * rsqrt(mean(x^2)+eps) * float(w) ) for this lane's chunks
// (k_rmsnorm, inference/src/backend/cuda_ops.cu:75-96). Padding chunks stay zero.
template <int NCH>
__device__ __forceinline__ void rmsnorm_regs(RowRegs<NCH>& xn, const bf16* x, const bf16* w, int H, float eps, int lane) {
    RowRegs<NCH> xr, wr;
    load_row_act<NCH>(xr, x, H, lane);
    load_row<NCH>(wr, w, H, lane);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        const uint32_t u[4] = {xr.v[j].x, xr.v[j].y, xr.v[j].z, xr.v[j].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float a = bf16_lo(u[k]), b = bf16_hi(u[k]);
            ss += a * a + b * b;
        }
    }
    ss = warp_sum(ss);
    const float rinv = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        const uint32_t u[4] = {xr.v[j].x, xr.v[j].y, xr.v[j].z, xr.v[j].w};
        const uint32_t g[4] = {wr.v[j].x, wr.v[j].y, wr.v[j].z, wr.v[j].w};
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float a = bf16_lo(u[k]) * rinv * bf16_lo(g[k]);
            const float b = bf16_hi(u[k]) * rinv * bf16_hi(g[k]);
            o[k] = (uint32_t)bf16_bits(a) | ((uint32_t)bf16_bits(b) << 16);
        }
        xn.v[j] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}


}  // namespace bs1
}  // namespace tffn
