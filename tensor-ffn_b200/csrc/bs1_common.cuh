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

// ------------------------------------------------------------------ fixed-point FFN sums
constexpr int kAccReplicas = 2;
constexpr float kAccScale = 4294967296.f;            // 2^32: resolution 2.3e-10, range +-2^31
constexpr float kAccInvScale = 1.f / 4294967296.f;
__device__ __forceinline__ float acc_value(const long long* acc, int H, int i) {
    long long s = 0;
#pragma unroll
    for (int r = 0; r < kAccReplicas; ++r) s += __ldcg(acc + (size_t)r * H + i);
    return __ll2float_rn(s) * kAccInvScale;
}

// Residual stream and its RMSNorm by a block of NT threads: h = bf16(h_in + acc_in) (the residual add of
// inference/src/model/qwen.cu:282-285 with the FFN sums the previous kernel left; acc_in may be null),
// optionally published to `publish`; xn = bf16(h * rsqrt(mean(h^2) + eps) * w) (k_rmsnorm,
// inference/src/backend/cuda_ops.cu:75-96) into shared memory xs[H]. sync() is a barrier over exactly
// those NT threads; s_red holds NT / 32 floats. H <= 2048.
template <int NT, typename SyncFn>
__device__ __forceinline__ void fold_norm_block(const bf16* hsrc, const long long* acc_in, const bf16* w, int H, float eps,
                                                bf16* publish, uint8_t* xs, float* s_red, int tid, SyncFn sync) {
    constexpr int PAIRS = 1024 / NT;
    float a[PAIRS], b[PAIRS];
    uint32_t wv[PAIRS];  // fetched together with h: no second trip to L2 after the reduction
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < PAIRS; ++k) {
        const int i = (tid + k * NT) * 2;
        a[k] = b[k] = 0.f;
        wv[k] = 0u;
        if (i < H) {
            const uint32_t hv = __ldcg((const uint32_t*)(hsrc + i));
            wv[k] = __ldg((const uint32_t*)(w + i));
            a[k] = bf16_lo(hv);
            b[k] = bf16_hi(hv);
            if (acc_in) {
                a[k] = bf16_round(a[k] + acc_value(acc_in, H, i));
                b[k] = bf16_round(b[k] + acc_value(acc_in, H, i + 1));
            }
            if (publish) ((uint32_t*)publish)[i >> 1] = (uint32_t)bf16_bits(a[k]) | ((uint32_t)bf16_bits(b[k]) << 16);
            ss += a[k] * a[k] + b[k] * b[k];
        }
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) s_red[tid >> 5] = ss;
    sync();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < NT / 32; ++k) tot += s_red[k];
    const float rinv = rsqrtf(tot / (float)H + eps);
#pragma unroll
    for (int k = 0; k < PAIRS; ++k) {
        const int i = (tid + k * NT) * 2;
        if (i < H) {
            const float x0 = a[k] * rinv * bf16_lo(wv[k]), x1 = b[k] * rinv * bf16_hi(wv[k]);
            ((uint32_t*)xs)[i >> 1] = (uint32_t)bf16_bits(x0) | ((uint32_t)bf16_bits(x1) << 16);
        }
    }
    sync();
}

// ------------------------------------------------------------------ tensor-core GEMV helpers
// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col). Register layout (g = lane / 4, t = lane % 4):
// a0 = A[g][2t..2t+1], a1 = A[g+8][2t..], a2 = A[g][2t+8..], a3 = A[g+8][2t+8..]; b0 = B[2t..2t+1][g],
// b1 = B[2t+8..][g]; c0,c1 = D[g][2t..2t+1], c2,c3 = D[g+8][2t..2t+1].
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Dot products of weight rows in shared memory with x[K] (bf16 in shared memory) on the tensor cores: a
// batch-1 GEMV does so little arithmetic per byte that what limits a CUDA-core version is instruction
// issue (unpack + FMA per value); here one 16-byte load per lane feeds two MMAs.
// row_lo / row_hi: the row this lane's g = lane / 4 stands for in the lower / upper half of the 16 MMA rows
// (any shared-memory rows, 128-byte aligned, K % 64 == 0); UPPER = false leaves the upper half empty.
// A dot product does not care in which order k is visited, so lane (g, t) reads 16 consecutive bytes
// (8 values) of its row and the same 16 bytes of x and feeds them to two MMAs as that lane's k slots.
// All rows sit at the same offset modulo 128 bytes, so odd rows take the two 64-byte halves of every
// 128-byte block in the opposite order: the eight lanes of a quarter warp then touch 128 distinct bytes
// (no bank conflict). MMA column n is fed by the lanes with g = n, i.e. in that row parity's order, so
// D[g][n] is the wanted sum wherever g and n have the same parity; lane (g, t) holds columns 2t and 2t + 1
// and keeps the matching one. Every lane returns the dot products of its two rows.
template <bool UPPER>
__device__ __forceinline__ void mma_rows_dot(const uint8_t* row_lo, const uint8_t* row_hi, int K, const uint8_t* xs, int lane,
                                             float& d_lo, float& d_hi) {
    const int g = lane >> 2, t = lane & 3, par = g & 1;
    const int o1 = (par ? 64 : 0) + t * 16, o2 = (par ? 0 : 64) + t * 16;
    float c[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) c[i][j] = 0.f;
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    const int nds = K >> 6;
    uint4 a1 = *(const uint4*)(row_lo + o1), a2 = *(const uint4*)(row_lo + o2);
    uint4 b1 = UPPER ? *(const uint4*)(row_hi + o1) : z, b2 = UPPER ? *(const uint4*)(row_hi + o2) : z;
    uint4 x1 = *(const uint4*)(xs + o1), x2 = *(const uint4*)(xs + o2);
#pragma unroll 2
    for (int ds = 0; ds < nds; ++ds) {
        // the next block's loads are in flight while this block's MMAs issue
        const int nx = (ds + 1 < nds ? ds + 1 : ds) * 128;
        const uint4 na1 = *(const uint4*)(row_lo + nx + o1), na2 = *(const uint4*)(row_lo + nx + o2);
        const uint4 nb1 = UPPER ? *(const uint4*)(row_hi + nx + o1) : z, nb2 = UPPER ? *(const uint4*)(row_hi + nx + o2) : z;
        const uint4 nx1 = *(const uint4*)(xs + nx + o1), nx2 = *(const uint4*)(xs + nx + o2);
        mma16816(c[0], a1.x, b1.x, a1.y, b1.y, x1.x, x1.y);
        mma16816(c[1], a1.z, b1.z, a1.w, b1.w, x1.z, x1.w);
        mma16816(c[2], a2.x, b2.x, a2.y, b2.y, x2.x, x2.y);
        mma16816(c[3], a2.z, b2.z, a2.w, b2.w, x2.z, x2.w);
        a1 = na1; a2 = na2; b1 = nb1; b2 = nb2; x1 = nx1; x2 = nx2;
    }
    d_lo = par ? (c[0][1] + c[1][1]) + (c[2][1] + c[3][1]) : (c[0][0] + c[1][0]) + (c[2][0] + c[3][0]);
    d_hi = par ? (c[0][3] + c[1][3]) + (c[2][3] + c[3][3]) : (c[0][2] + c[1][2]) + (c[2][2] + c[3][2]);
}

// acc (two fp32 in one 64-bit register) += a * (lo, hi of a packed bf16 pair): one packed FMA
__device__ __forceinline__ void axpy_bf16x2(unsigned long long& acc, unsigned long long a2, uint32_t w) {
    unsigned long long v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(w << 16), "r"(w & 0xffff0000u));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a2), "l"(v));
}
__device__ __forceinline__ unsigned long long splat_f32x2(float a) {
    unsigned long long v;
    asm("mov.b64 %0, {%1, %1};" : "=l"(v) : "f"(a));
    return v;
}
__device__ __forceinline__ float2 unpack_f32x2(unsigned long long v) {
    float2 r;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
    return r;
}

}  // namespace bs1
}  // namespace tffn
