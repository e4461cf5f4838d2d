// Tensor-core GEMM of the batched path (prefill and decode with more than one token):
//     out[t, n] = epilogue( sum_k X[t,k] * W[n,k] )
// "swap-AB": the weight rows fill the MMA's M = 128 dimension and the tokens are the MMA's N
// (16..256), so a decode step with a few dozen tokens wastes no tensor-core rows and each
// weight byte is streamed from HBM exactly once per token tile.
//
// One CTA = one 128-row x BN-token output tile (optionally one K split of it), 6 warps:
//   warp 0   TMA producer: 128x64 weight box + BNx64 activation box per stage, 128-byte swizzle
//   warp 1   allocates TMEM, issues tcgen05.mma (one thread), commits stages back to the producer
//   warps 2-5 epilogue: tcgen05.ld the fp32 accumulators (lane = weight row, column = token),
//            apply the epilogue and store. With split-K the splits of a tile are one thread-block
//            cluster: partial tiles stay in shared memory and are summed across the cluster over
//            distributed shared memory in rank order, so the result does not depend on
//            scheduling and no partial sum touches HBM.
// Two operand pairs can be accumulated into two TMEM regions (gate|up for the SwiGLU epilogue,
// base|expert for the down projection) and are combined in fp32 in the epilogue.
// It replaces the reference's cublasGemmEx wrappers (inference/src/backend/cuda_ops.cu:18-43)
// and the element-wise kernels around them (silu_mul :58-69, add :152-157,
// k_add_fp32_to_bf16 inference/src/model/qwen.cu:282-285).
#include "kernels.h"
#include "ptx.cuh"
#include <cstdio>
#include <cstring>
#include <functional>
#include <unordered_map>

namespace tffn {

namespace {

constexpr int BM = 128;  // weight rows per tile
constexpr int BK = 64;   // K elements per stage (128 bytes of bf16)
constexpr int kGemmThreads = 192;

struct GemmDev {
    CUtensorMap tmW[2];
    CUtensorMap tmX[2];
    int kblocks[2];
    int N, T, splits, mode;
    float alpha;
    void* out;
    long long ldo;
    int* status;
};

template <int BN>
struct GemmCfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // BN <= 64 (decode): 4 stages keep a CTA under half an SM's shared memory, so two CTAs (or two
    // tiles' splits) are resident per SM and the weight stream has 2 x 64 KB in flight per SM
    static constexpr int STAGES = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 4);
    // split-K parks [accs][BN][128] fp32 partials in the stage memory
    static constexpr bool SPLIT_OK_DUAL = 2 * BN * BM * 4 <= STAGES * STAGE_BYTES;
    static constexpr bool SPLIT_OK_SINGLE = BN * BM * 4 <= STAGES * STAGE_BYTES;
    static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;  // power of two for BN in {16..256}
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void epilogue_apply(const GemmDev& p, int n, int t, float v0, float v1, bool has1) {
    if (n >= p.N || t >= p.T) return;
    size_t o = (size_t)t * (size_t)p.ldo + n;
    switch (p.mode) {
        case GEMM_STORE_F32:
            ((float*)p.out)[o] = has1 ? v0 + p.alpha * v1 : v0;
            break;
        case GEMM_STORE_BF16:
            ((bf16*)p.out)[o] = __float2bfloat16_rn(has1 ? v0 + p.alpha * v1 : v0);
            break;
        case GEMM_RESIDUAL: {
            bf16* h = (bf16*)p.out;
            float d = has1 ? v0 + p.alpha * v1 : v0;
            h[o] = __float2bfloat16_rn(__bfloat162float(h[o]) + d);
            break;
        }
        case GEMM_SWIGLU:
            ((bf16*)p.out)[o] = __float2bfloat16_rn(silu_mul_bf16(v0, v1));
            break;
    }
}

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, (BN <= 64) ? 2 : 1) k_gemm_tc(const __grid_constant__ GemmDev p) {
    using Cfg = GemmCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
    uint64_t* empty = full + Cfg::STAGES;
    uint64_t* acc_full = empty + Cfg::STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BM, t0 = blockIdx.y * BN;
    const int total_kb = p.kblocks[0] + p.kblocks[1];
    const int kb_begin = (int)(((long long)blockIdx.z * total_kb) / p.splits);
    const int kb_end = (int)(((long long)(blockIdx.z + 1) * total_kb) / p.splits);
    const int n_iters = kb_end - kb_begin;
    const bool has0 = kb_begin < p.kblocks[0] && n_iters > 0;
    const bool has1 = kb_end > p.kblocks[0] && p.kblocks[1] > 0 && n_iters > 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            prefetch_tmap(&p.tmW[0]);
            prefetch_tmap(&p.tmX[0]);
            for (int it = 0; it < n_iters; ++it) {
                const int s = it % Cfg::STAGES;
                const uint32_t ph = (uint32_t)(it / Cfg::STAGES) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, p.status, DEV_ERR_EMPTY_WAIT)) break;
                const int i = kb_begin + it;
                const int seg = i >= p.kblocks[0] ? 1 : 0;
                const int kb = seg ? i - p.kblocks[0] : i;
                uint8_t* a = smem + s * Cfg::STAGE_BYTES;
                uint8_t* b = a + Cfg::A_BYTES;
                mbar_arrive_expect_tx(&full[s], Cfg::STAGE_BYTES);
                tma_load_2d(a, &p.tmW[seg], kb * BK, n0, &full[s]);
                tma_load_2d(b, &p.tmX[seg], kb * BK, t0, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
            bool started[2] = {false, false};
            bool ok = true;
            for (int it = 0; it < n_iters && ok; ++it) {
                const int s = it % Cfg::STAGES;
                const uint32_t ph = (uint32_t)(it / Cfg::STAGES) & 1u;
                ok = mbar_wait(&full[s], ph, p.status, DEV_ERR_FULL_WAIT);
                if (!ok) break;
                tc_fence_after();
                const int seg = (kb_begin + it) >= p.kblocks[0] ? 1 : 0;
                const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
                const uint32_t b_addr = a_addr + Cfg::A_BYTES;
                const uint32_t d = tmem_base + (uint32_t)(seg * BN);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    umma_bf16(d, umma_desc_k128(a_addr + k * 32), umma_desc_k128(b_addr + k * 32), idesc,
                              (started[seg] || k > 0) ? 1u : 0u);
                }
                started[seg] = true;
                umma_commit(&empty[s]);
            }
            umma_commit(acc_full);  // arrives when every MMA above has finished (also on the error path)
        }
    } else {
        // epilogue warps 2..5 -> TMEM lane quarter (warp % 4)
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int n = n0 + row;
        // every lane waits (acquire); the outcome is made warp-uniform because tcgen05.ld is .aligned
        bool ok = mbar_wait(acc_full, 0, p.status, DEV_ERR_ACC_WAIT);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const bool dual = p.kblocks[1] > 0;
        if (p.splits == 1) {
            if (ok && n_iters > 0) {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    if (t0 + c0 >= p.T) break;
                    uint32_t v0[16], v1[16];
                    if (has0) tmem_ld16(lane_addr + c0, v0);
                    if (has1) tmem_ld16(lane_addr + BN + c0, v1);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        epilogue_apply(p, n, t0 + c0 + j, has0 ? __uint_as_float(v0[j]) : 0.f,
                                       has1 ? __uint_as_float(v1[j]) : 0.f, dual);
                }
            }
        } else {
            // split-K: park this CTA's partial tile in its own shared memory (the pipeline stages are
            // free: every load was consumed by an MMA that has completed); layout [acc][column][row]
            float* red = (float*)smem;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (t0 + c0 >= p.T) break;
                uint32_t v0[16], v1[16];
                const bool live = ok && n_iters > 0;
                if (live && has0) tmem_ld16(lane_addr + c0, v0);
                if (live && has1) tmem_ld16(lane_addr + BN + c0, v1);
                tc_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    red[(size_t)(c0 + j) * BM + row] = (live && has0) ? __uint_as_float(v0[j]) : 0.f;
                    if (dual) red[(size_t)(BN + c0 + j) * BM + row] = (live && has1) ? __uint_as_float(v1[j]) : 0.f;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (p.splits > 1) {
        // The splits of one output tile form a thread-block cluster (1,1,splits). After the cluster
        // barrier every CTA sums, over all splits in rank order, the columns it owns (column % splits
        // == rank) straight out of its peers' shared memory, and applies the epilogue. A second
        // barrier keeps every CTA's shared memory alive until its peers have finished reading it.
        cluster_sync_all();
        if (warp >= 2) {
            const int q = warp & 3;
            const int row = q * 32 + lane;
            const int n = n0 + row;
            const bool dual = p.kblocks[1] > 0;
            const uint32_t rank = cluster_ctarank();
            const uint32_t red_local = smem_u32(smem);
            uint32_t peer[8];
#pragma unroll
            for (int z = 0; z < 8; ++z) peer[z] = (z < p.splits) ? map_shared_rank(red_local, (uint32_t)z) : 0u;
            for (int c = (int)rank; c < BN; c += p.splits) {
                if (t0 + c >= p.T) break;
                float v0[8], v1[8];
#pragma unroll
                for (int z = 0; z < 8; ++z) {
                    v0[z] = 0.f;
                    v1[z] = 0.f;
                    if (z < p.splits) {
                        v0[z] = ld_shared_cluster_f32(peer[z] + (uint32_t)(((size_t)c * BM + row) * 4));
                        if (dual) v1[z] = ld_shared_cluster_f32(peer[z] + (uint32_t)(((size_t)(BN + c) * BM + row) * 4));
                    }
                }
                float a0 = 0.f, a1 = 0.f;
#pragma unroll
                for (int z = 0; z < 8; ++z) {
                    a0 += v0[z];
                    a1 += v1[z];
                }
                epilogue_apply(p, n, t0 + c, a0, a1, dual);
            }
        }
        cluster_sync_all();
    }
    if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

struct TmapKey {
    const void* ptr;
    uint64_t rows, cols, ld;
    uint32_t box_rows;
    bool operator==(const TmapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct TmapKeyHash {
    size_t operator()(const TmapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ (k.rows * 1000003u) ^ (k.cols * 7919u) ^ (k.ld << 20) ^ k.box_rows;
    }
};

bool encode_tmap(CUtensorMap* tm, const bf16* ptr, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_rows);

// Encoding a tensor map costs microseconds of host time; the same (buffer, shape, box) recurs on
// every step, so encoded maps are kept per thread (a session is used by one thread at a time).
bool make_tmap(CUtensorMap* tm, const bf16* ptr, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_rows) {
    static thread_local std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
    TmapKey key{ptr, rows, cols, ld_elems, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) {
        *tm = it->second;
        return true;
    }
    if (!encode_tmap(tm, ptr, rows, cols, ld_elems, box_rows)) return false;
    if (cache.size() > 65536) cache.clear();
    cache.emplace(key, *tm);
    return true;
}

// 2-D bf16 tensor [rows, cols] with a row stride, box = box_rows x 64 columns, 128-byte swizzle
bool encode_tmap(CUtensorMap* tm, const bf16* ptr, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld_elems * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)ptr, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int BN>
int launch_bn(const GemmCall& c, const GemmWorkspace& ws, cudaStream_t stream, int force_splits) {
    using Cfg = GemmCfg<BN>;
    GemmDev p;
    memset(&p, 0, sizeof p);
    for (int i = 0; i < 2; ++i) {
        const GemmOperand& o = c.op[i];
        p.kblocks[i] = o.K > 0 ? (o.K + BK - 1) / BK : 0;
        if (o.K <= 0) continue;
        if (!make_tmap(&p.tmW[i], o.W, (uint64_t)c.N, (uint64_t)o.K, (uint64_t)o.ldw, BM)) return -1000;
        if (!make_tmap(&p.tmX[i], o.X, (uint64_t)(c.x_rows_alloc > c.T ? c.x_rows_alloc : c.T), (uint64_t)o.K,
                       (uint64_t)o.ldx, BN))
            return -1000;
    }
    if (p.kblocks[1] == 0) {  // keep the unused maps valid for prefetch
        p.tmW[1] = p.tmW[0];
        p.tmX[1] = p.tmX[0];
    }
    p.N = c.N;
    p.T = c.T;
    p.mode = c.mode;
    p.alpha = c.alpha;
    p.out = c.out;
    p.ldo = c.ldo;
    p.status = ws.status;
    const int n_tiles = (c.N + BM - 1) / BM, t_tiles = (c.T + BN - 1) / BN;
    const int total_kb = p.kblocks[0] + p.kblocks[1];
    const int tiles = n_tiles * t_tiles;
    const bool dual = p.kblocks[1] > 0;
    const bool split_ok = dual ? Cfg::SPLIT_OK_DUAL : Cfg::SPLIT_OK_SINGLE;
    // K splits = cluster size (1, 2, 4 or 8): grow while all CTAs stay co-resident (two per SM for
    // the decode tile sizes) and every split keeps at least two k-blocks
    int splits = 1;
    if (force_splits > 0) {
        splits = force_splits;
    } else if (split_ok) {
        const int resident = ws.num_sms * ((BN <= 64) ? 2 : 1);
        while (splits < 8 && tiles * splits * 2 <= resident && total_kb / (splits * 2) >= 2) splits *= 2;
    }
    if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return (int)cudaErrorInvalidValue;
    if (splits > 1 && (!split_ok || splits > total_kb)) return (int)cudaErrorInvalidValue;
    p.splits = splits;
    cudaLaunchConfig_t cfg = cudaLaunchConfig_t{};
    cfg.gridDim = dim3(n_tiles, t_tiles, splits);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = splits;
    cfg.attrs = attr;
    cfg.numAttrs = splits > 1 ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, k_gemm_tc<BN>, p);
}

}  // namespace

int gemm_prepare() {
    cudaError_t e;
#define TFFN_PREP(BN)                                                                                                 \
    e = cudaFuncSetAttribute(k_gemm_tc<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::SMEM_BYTES); \
    if (e != cudaSuccess) return (int)e;
    TFFN_PREP(16) TFFN_PREP(32) TFFN_PREP(64) TFFN_PREP(128) TFFN_PREP(256)
#undef TFFN_PREP
    return 0;
}

int launch_gemm(const GemmCall& c, const GemmWorkspace& ws, cudaStream_t stream, int force_splits) {
    if (c.T <= 0 || c.N <= 0 || c.op[0].K <= 0) return (int)cudaErrorInvalidValue;
    if (c.T <= 16) return launch_bn<16>(c, ws, stream, force_splits);
    if (c.T <= 32) return launch_bn<32>(c, ws, stream, force_splits);
    if (c.T <= 64) return launch_bn<64>(c, ws, stream, force_splits);
    if (c.T <= 128) return launch_bn<128>(c, ws, stream, force_splits);
    return launch_bn<256>(c, ws, stream, force_splits);
}

}  // namespace tffn
