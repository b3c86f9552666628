// Dense GEMMs on the 5th-generation tensor cores (tcgen05) of sm_100a, written with inline PTX.
//
//   gemm_tcgen05      C[M, N]  = epilogue(A[M, K] * B[N, K]^T)     both operands K-major (activations x weights:
//                     forward projections, FFN, input gradients with a pre-transposed weight)
//   gemm_tn_tcgen05   C[N, K] += A[M, N]^T * B[M, K]               both operands MN-major (weight gradients: the
//                     reduction runs over the long row dimension and is split across CTAs)
//
// Structure of a CTA (192 threads): warp 0 / one elected thread issues the TMA loads (cp.async.bulk.tensor, 128-byte
// swizzle, completion on an mbarrier); warp 1 allocates tensor memory and one elected thread issues tcgen05.mma
// (M = 128, N = 128, K = 16 per instruction, fp32 accumulator of 128 lanes x 128 columns in TMEM) and releases each
// shared-memory stage with tcgen05.commit; warps 2-5 are the epilogue: tcgen05.ld of the accumulator (32 lanes per warp),
// bias / ReLU / dropout / cast in registers, vector stores.  Three 32 KB stages per CTA, two CTAs per SM so that one
// CTA's epilogue overlaps the other's main loop (the GEMMs of these models have K = 128..1024, i.e. 2..16 stages, and are
// as much bound by streaming A and C as by the MMAs).
//
// Every wait (mbarrier phases) is bounded: on expiry the waiting thread raises a CTA-wide abort flag and the global status
// word, the producer drains the copies it has in flight, tensor memory is released and the CTA returns.  The host checks
// the status word after synchronising.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "kernels.h"
#include "tc05.cuh"

namespace gt {
namespace {

constexpr int BM = 128, BN = 128, BK = 64, STAGES = 3;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 128;

struct __align__(1024) SharedStorage {
    __nv_bfloat16 a[STAGES][BM * BK];                      // 16 KB per stage
    __nv_bfloat16 b[STAGES][BN * BK];                      // 16 KB per stage
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

__device__ __forceinline__ uint64_t site_seed(const long long* seed, long long stream_id) {
    uint64_t s0 = seed ? (uint64_t)seed[0] : 0x1234567ull, s1 = seed ? (uint64_t)seed[1] : 0ull;
    return s0 + 0x9E3779B97F4A7C15ull * (s1 * 4096ull + (uint64_t)stream_id + 1ull);
}

// Epilogue arithmetic on one 32-column chunk of an accumulator row.  Every condition (bias present, activation, dropout,
// partial tile) is tested once per chunk, never per element: the element loops are branch-free.
__device__ __forceinline__ void epilogue_math(const uint32_t (&r)[32], float (&v)[32], int row, int col0, const GemmArgs& g,
                                              uint64_t sd, float inv_keep) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    const bool full = col0 + 32 <= g.N;
    if (g.bias) {
        if (full && (reinterpret_cast<uintptr_t>(g.bias) & 15) == 0) {      // parameter views are only 4-byte aligned in general
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 b = __ldg(reinterpret_cast<const float4*>(g.bias + col0 + j));
                v[j] += b.x; v[j + 1] += b.y; v[j + 2] += b.z; v[j + 3] += b.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += (col0 + j < g.N) ? g.bias[col0 + j] : 0.f;
        }
    }
    if (g.act == 1) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
    } else if (g.act == 2) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = gelu_f(v[j]);
    }
    if (g.p > 0.f) {
        const uint64_t base = (uint64_t)row * g.N + col0;
        const uint32_t thr = drop_threshold(g.p);
        if ((base & 7) == 0) {                                 // four aligned 8-element chunks: one mask word each
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8) {
                const uint32_t kb = keep_bits8(sd, (base >> 3) + c8, thr);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[c8 * 8 + k] = ((kb >> k) & 1u) ? v[c8 * 8 + k] * inv_keep : 0.f;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = keep_element(sd, base + j, thr) ? v[j] * inv_keep : 0.f;
        }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// C = A * B^T (K-major operands)
// ------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) gemm_nt_kernel(const __grid_constant__ CUtensorMap map_a,
                                                           const __grid_constant__ CUtensorMap map_b, GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    SharedStorage& sh = *reinterpret_cast<SharedStorage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const int nkb = (g.K + BK - 1) / BK;
    volatile int* abort_flag = &sh.abort_flag;

    if (threadIdx.x == 0) {
        sh.abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
        mbar_init(&sh.tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&sh.tmem_base, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        int issued = 0;
        for (int kb = 0; kb < nkb; ++kb) {
            const int s = kb % STAGES;
            if (!mbar_wait(&sh.empty[s], ((kb / STAGES) & 1) ^ 1, abort_flag, g.status, 1)) break;
            mbar_expect_tx(&sh.full[s], (BM + BN) * BK * 2);
            tma_load_2d(sh.a[s], &map_a, kb * BK, m0, &sh.full[s]);
            tma_load_2d(sh.b[s], &map_b, kb * BK, n0, &sh.full[s]);
            issued = kb + 1;
        }
        if (*abort_flag) {
            // drain: every stage whose copy was issued must land before the CTA may exit
            for (int kb = (issued > STAGES ? issued - STAGES : 0); kb < issued; ++kb) {
                const long long t0 = clock64();
                while (!mbar_try_wait(&sh.full[kb % STAGES], (kb / STAGES) & 1) && clock64() - t0 < kWaitCycles) {}
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        const uint32_t idesc = make_idesc(BM, BN, 0, 0);
        bool okay = true;
        for (int kb = 0; kb < nkb && okay; ++kb) {
            const int s = kb % STAGES;
            okay = mbar_wait(&sh.full[s], (kb / STAGES) & 1, abort_flag, g.status, 2);
            if (!okay) break;
            tc_fence_after();
            const uint32_t a_addr = smem_u32(sh.a[s]), b_addr = smem_u32(sh.b[s]);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
                const uint64_t ad = make_desc(a_addr + k * 32, 16, 1024);
                const uint64_t bd = make_desc(b_addr + k * 32, 16, 1024);
                umma_bf16(tmem, ad, bd, idesc, (kb | k) != 0);
            }
            umma_commit(&sh.empty[s]);                    // frees the stage once these MMAs have read it
        }
        if (okay) umma_commit(&sh.tmem_full);
    } else if (warp >= 2) {
        // ---- epilogue: TMEM -> registers -> global ----
        const bool okay = mbar_wait(&sh.tmem_full, 0, abort_flag, g.status, 3);
        tc_fence_after();
        if (okay) {
            const int quad = warp & 3;                     // TMEM lanes [32 * quad, 32 * quad + 32)
            const int row = m0 + quad * 32 + lane;
            const uint64_t sd = site_seed(g.seed, g.stream_id);
            const float inv_keep = g.p > 0.f ? keep_scale(g.p) : 1.f;
            // bf16 results of full-width-aligned tiles go through shared memory (the pipeline stages are free once the
            // accumulator is complete) so that global stores are whole 256-byte row segments instead of one row per lane
            const bool staged = g.c_dtype == DT_BF16 && (g.ldc & 7) == 0 && (g.N & 7) == 0;
            constexpr int kStageStride = BN * 2 + 16;              // bytes per staged row: +16 keeps 16-byte writes conflict-free
            uint8_t* stage = reinterpret_cast<uint8_t*>(sh.a) + (size_t)quad * 32 * kStageStride;
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                __syncwarp();                                 // lanes that skipped the previous chunk rejoin before the aligned load
                tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + c0, r);     // whole warp: sync.aligned
                const int col0 = n0 + c0;
                if (!staged && (row >= g.M || col0 >= g.N)) continue;
                float v[32];
                epilogue_math(r, v, row, col0, g, sd, inv_keep);
                if (staged) {
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(stage + (size_t)lane * kStageStride) + c0;
#pragma unroll
                    for (int j = 0; j < 32; j += 8) st_bf16x8(dst + j, v[j], v[j + 1], v[j + 2], v[j + 3], v[j + 4], v[j + 5], v[j + 6], v[j + 7]);
                    continue;
                }
                const bool full = col0 + 32 <= g.N;
                if (g.c_dtype == DT_BF16) {
                    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(g.c) + (size_t)row * g.ldc + col0;
                    _Pragma("unroll") for (int j = 0; j < 32; ++j)
                        if (col0 + j < g.N) dst[j] = __float2bfloat16(v[j]);
                } else {
                    float* dst = static_cast<float*>(g.c) + (size_t)row * g.ldc + col0;
                    if (full && (g.ldc & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                            if (g.accumulate) {
                                float4 old = *reinterpret_cast<float4*>(dst + j);
                                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                            }
                            *reinterpret_cast<float4*>(dst + j) = o;
                        }
                    } else {
                        _Pragma("unroll") for (int j = 0; j < 32; ++j)
                            if (col0 + j < g.N) dst[j] = g.accumulate ? dst[j] + v[j] : v[j];
                    }
                }
            }
            if (staged) {
                __syncwarp();
                // 16 lanes cover one 256-byte row: two rows per instruction, 16 instructions for the warp's 32 rows
                const int cchunk = lane & 15;
                const bool col_ok = n0 + cchunk * 8 + 8 <= g.N;
#pragma unroll 4
                for (int it = 0; it < 16; ++it) {
                    const int rr = it * 2 + (lane >> 4);
                    const int grow = m0 + quad * 32 + rr;
                    if (grow < g.M && col_ok) {
                        const uint4 val = *reinterpret_cast<const uint4*>(stage + (size_t)rr * kStageStride + cchunk * 16);
                        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(g.c) + (size_t)grow * g.ldc + n0 + cchunk * 8) = val;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// ------------------------------------------------------------------------------------------------------------------
// Persistent variant of C = A * B^T.  One CTA per SM walks the output tiles (n fastest, so CTAs running at the same time share
// the A rows in L2).  Tensor memory holds TWO accumulators (2 x 128 columns): while the epilogue warps drain tile i, the MMA
// thread already accumulates tile i + 1, and the TMA producer runs ahead through a 5-stage ring that is shared by all tiles
// (stage indices and phases continue across tile boundaries).  TMEM allocation, barrier initialisation and pipeline fill are
// paid once per CTA instead of once per tile, which is what bounds the short-K (128..512) GEMMs of these models.
// ------------------------------------------------------------------------------------------------------------------
constexpr int P_STAGES = 5;
constexpr int kStageStrideP = BN * 2 + 16;               // staged C row: +16 bytes keeps 16-byte writes conflict-free

struct __align__(1024) PersistentStorage {
    __nv_bfloat16 a[P_STAGES][BM * BK];
    __nv_bfloat16 b[P_STAGES][BN * BK];
    uint8_t stage_c[4 * 32 * kStageStrideP];
    uint64_t full[P_STAGES];
    uint64_t empty[P_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};


__global__ void __launch_bounds__(kThreads, 1) gemm_nt_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                         const __grid_constant__ CUtensorMap map_b, GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    PersistentStorage& sh = *reinterpret_cast<PersistentStorage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (g.N + BN - 1) / BN, tiles_m = (g.M + BM - 1) / BM;
    const int n_tiles = tiles_n * tiles_m;
    const int nkb = (g.K + BK - 1) / BK;
    volatile int* abort_flag = &sh.abort_flag;

    if (threadIdx.x == 0) {
        sh.abort_flag = 0;
        for (int s = 0; s < P_STAGES; ++s) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sh.tmem_full[b], 1); mbar_init(&sh.tmem_empty[b], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&sh.tmem_base, 2 * kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        int it = 0, issued_from = 0;
        bool okay = true;
        for (int tile = blockIdx.x; tile < n_tiles && okay; tile += gridDim.x) {
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % P_STAGES;
                okay = mbar_wait(&sh.empty[s], ((it / P_STAGES) & 1) ^ 1, abort_flag, g.status, 1);
                if (!okay) break;
                mbar_expect_tx(&sh.full[s], (BM + BN) * BK * 2);
                tma_load_2d(sh.a[s], &map_a, kb * BK, m0, &sh.full[s]);
                tma_load_2d(sh.b[s], &map_b, kb * BK, n0, &sh.full[s]);
            }
        }
        if (*abort_flag) {
            // drain: the copies issued into the last P_STAGES ring slots must land before the CTA may exit
            issued_from = it > P_STAGES ? it - P_STAGES : 0;
            for (int k = issued_from; k < it; ++k) {
                const long long t0 = clock64();
                while (!mbar_try_wait(&sh.full[k % P_STAGES], (k / P_STAGES) & 1) && clock64() - t0 < kWaitCycles) {}
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        const uint32_t idesc = make_idesc(BM, BN, 0, 0);
        int it = 0, ti = 0;
        bool okay = true;
        for (int tile = blockIdx.x; tile < n_tiles && okay; tile += gridDim.x, ++ti) {
            const int b = ti & 1;
            okay = mbar_wait(&sh.tmem_empty[b], ((ti >> 1) & 1) ^ 1, abort_flag, g.status, 2);   // epilogue drained this accumulator
            if (!okay) break;
            tc_fence_after();
            const uint32_t acc = tmem + (uint32_t)(b * BN);
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % P_STAGES;
                okay = mbar_wait(&sh.full[s], (it / P_STAGES) & 1, abort_flag, g.status, 2);
                if (!okay) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(sh.a[s]), b_addr = smem_u32(sh.b[s]);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    umma_bf16(acc, make_desc(a_addr + k * 32, 16, 1024), make_desc(b_addr + k * 32, 16, 1024), idesc, (kb | k) != 0);
                umma_commit(&sh.empty[s]);
            }
            if (okay) umma_commit(&sh.tmem_full[b]);
        }
    } else if (warp >= 2) {
        // ---- epilogue ----
        const int quad = warp & 3;
        const uint64_t sd = site_seed(g.seed, g.stream_id);
        const float inv_keep = g.p > 0.f ? keep_scale(g.p) : 1.f;
        const bool staged = g.c_dtype == DT_BF16 && (g.ldc & 7) == 0 && (g.N & 7) == 0;
        uint8_t* stage = sh.stage_c + (size_t)quad * 32 * kStageStrideP;
        int ti = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++ti) {
            const int b = ti & 1;
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            if (!mbar_wait(&sh.tmem_full[b], (ti >> 1) & 1, abort_flag, g.status, 3)) break;
            tc_fence_after();
            const int row = m0 + quad * 32 + lane;
            const uint32_t acc = tmem + (uint32_t)(b * BN) + ((uint32_t)(quad * 32) << 16);
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                __syncwarp();                                 // lanes that skipped the previous chunk rejoin before the aligned load
                tmem_ld32(acc + c0, r);
                if (c0 + 32 >= BN) {
                    // last chunk read: hand the accumulator back to the MMA thread before the (slow) global stores
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh.tmem_empty[b]);
                }
                const int col0 = n0 + c0;
                if (!staged && (row >= g.M || col0 >= g.N)) continue;
                float v[32];
                epilogue_math(r, v, row, col0, g, sd, inv_keep);
                if (staged) {
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(stage + (size_t)lane * kStageStrideP) + c0;
#pragma unroll
                    for (int j = 0; j < 32; j += 8) st_bf16x8(dst + j, v[j], v[j + 1], v[j + 2], v[j + 3], v[j + 4], v[j + 5], v[j + 6], v[j + 7]);
                    continue;
                }
                if (g.c_dtype == DT_BF16) {
                    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(g.c) + (size_t)row * g.ldc + col0;
                    _Pragma("unroll") for (int j = 0; j < 32; ++j)
                        if (col0 + j < g.N) dst[j] = __float2bfloat16(v[j]);
                } else {
                    float* dst = static_cast<float*>(g.c) + (size_t)row * g.ldc + col0;
                    if (col0 + 32 <= g.N && (g.ldc & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                            if (g.accumulate) {
                                const float4 old = *reinterpret_cast<float4*>(dst + j);
                                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                            }
                            *reinterpret_cast<float4*>(dst + j) = o;
                        }
                    } else {
                        _Pragma("unroll") for (int j = 0; j < 32; ++j)
                            if (col0 + j < g.N) dst[j] = g.accumulate ? dst[j] + v[j] : v[j];
                    }
                }
            }
            if (staged) {
                __syncwarp();
                const int cchunk = lane & 15;
                const bool col_ok = n0 + cchunk * 8 + 8 <= g.N;
#pragma unroll 4
                for (int i2 = 0; i2 < 16; ++i2) {
                    const int rr = i2 * 2 + (lane >> 4);
                    const int grow = m0 + quad * 32 + rr;
                    if (grow < g.M && col_ok) {
                        const uint4 val = *reinterpret_cast<const uint4*>(stage + (size_t)rr * kStageStrideP + cchunk * 16);
                        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(g.c) + (size_t)grow * g.ldc + n0 + cchunk * 8) = val;
                    }
                }
                __syncwarp();                                 // the staging rows are rewritten by the next tile
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 2 * kTmemCols);
}

// ------------------------------------------------------------------------------------------------------------------
// All-gather fused into C = A * B^T.  The rows of A are spread over the ranks of a group: rank p holds rows
// [p * chunk, (p + 1) * chunk) in ITS OWN memory (a symmetric-heap buffer), and every rank needs the product of the whole
// gathered A with its weights.  Instead of all-gathering A and then running a GEMM, each CTA loads its A tiles straight from
// the owner's memory over NVLink with (non-multicast) TMA loads through one tensor map per peer, so the transfer of tile
// i + 1 overlaps the MMAs of tile i and the gathered matrix is never written unless the caller asks for it.
//
// The kernel is A-stationary: a 128-row A tile ([128, K], K <= 512) is fetched ONCE into shared memory and multiplied with
// every 128-column tile of B (the weights stream from L2 through a small ring), because a remote tile must cross the link
// only once.  With K <= 256 two A buffers alternate, so the remote fetch of the next tile runs during the current one.
// Roles (224 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue (two TMEM accumulators, as in the
// persistent kernel), warp 6 optional "copier" that TMA-stores each fetched A tile into a local gathered copy (what backward
// needs for the weight gradient) - the copy rides on data that is already in shared memory.
// m-tiles are dealt round-robin over the peers so all links (and the local HBM) are busy at the same time.
// ------------------------------------------------------------------------------------------------------------------
constexpr int kMaxPeers = 8;
constexpr int kGatherThreads = 224;
constexpr int G_MAX_B = 8;

struct GatherMaps {
    CUtensorMap a[kMaxPeers];
    CUtensorMap out[kMaxPeers];
    CUtensorMap c[kMaxPeers];         // result rows of peer p's block, box 32 rows x 64 columns (TMA-store epilogue)
};

struct GatherCfg {
    int chunk, n_peers, tiles_per_peer, copy_out;
    int nkb, n_abuf, n_b;             // k-blocks per tile, A buffers (1 or 2), B ring stages
    int tma_store;                    // bf16 result through swizzled shared memory + cp.async.bulk.tensor stores
    // epoch channel of the gathered operand (nullable): before the first tile of peer p is fetched the producer waits, bounded,
    // until wait_flags[p] has reached *wait_counter (the owner has published its rows)
    const int* wait_flags; const int* wait_counter; long long max_spins;
    int self;                         // this rank's index in the group: row tiles are walked peer by peer starting with the own rows
};

// Row tile mt -> (peer, first row inside the peer's chunk).  Tiles are ordered peer by peer, starting at this rank and going
// round the group: every CTA first works on rows that are already local, and at any moment the ranks of a group read from
// different owners (rank r is on peer r + k while rank r + 1 is on peer r + 1 + k), so no owner's link is read by all at once.
__device__ __forceinline__ void gather_tile(const GatherCfg& cfg, int mt, int& peer, int& m0) {
    const int slot = mt / cfg.tiles_per_peer;
    peer = cfg.self + slot;
    if (peer >= cfg.n_peers) peer -= cfg.n_peers;
    m0 = (mt - slot * cfg.tiles_per_peer) * BM;
}

struct GatherBars {
    uint64_t a_full[2], a_empty[2];
    uint64_t b_full[G_MAX_B], b_empty[G_MAX_B];
    uint64_t tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(smem_src))
                 : "memory");
}

__global__ void __launch_bounds__(kGatherThreads, 1) gemm_nt_gather_kernel(const __grid_constant__ GatherMaps maps,
                                                                           const __grid_constant__ CUtensorMap map_b, GemmArgs g,
                                                                           GatherCfg cfg) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int kTile = BM * BK * 2;                      // 16 KB
    uint8_t* a_sm = base;                                   // [n_abuf][nkb] tiles
    uint8_t* b_sm = a_sm + (size_t)cfg.n_abuf * cfg.nkb * kTile;
    uint8_t* stage_c = b_sm + (size_t)cfg.n_b * kTile;
    GatherBars& bars = *reinterpret_cast<GatherBars*>(stage_c + 4 * 32 * kStageStrideP);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (g.N + BN - 1) / BN;
    const int n_mtiles = cfg.n_peers * cfg.tiles_per_peer;
    const int nkb = cfg.nkb;
    volatile int* abort_flag = &bars.abort_flag;

    if (threadIdx.x == 0) {
        bars.abort_flag = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars.a_full[i], 1);
            mbar_init(&bars.a_empty[i], cfg.copy_out ? 2 : 1);
            mbar_init(&bars.tmem_full[i], 1);
            mbar_init(&bars.tmem_empty[i], 4);
        }
        for (int s = 0; s < G_MAX_B; ++s) { mbar_init(&bars.b_full[s], 1); mbar_init(&bars.b_empty[s], 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&bars.tmem_base, 2 * kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars.tmem_base;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer: A tiles from the owners' memory, B tiles from the local weights ----
        int ai = 0, it = 0;
        bool okay = true;
        uint32_t ready = cfg.wait_flags ? (1u << cfg.self) : 0xffffffffu;      // peers whose rows are known to be published
        auto load_a = [&](int mt, int idx) -> bool {
            const int buf = idx % cfg.n_abuf;
            if (!mbar_wait(&bars.a_empty[buf], ((idx / cfg.n_abuf) & 1) ^ 1, abort_flag, g.status, 1)) return false;
            int peer, m0;
            gather_tile(cfg, mt, peer, m0);
            if (!((ready >> peer) & 1u)) {
                const int want = *cfg.wait_counter;
                long long spins = 0;
                while (ld_acquire_sys_s32(cfg.wait_flags + peer) < want) {
                    if (*abort_flag) return false;
                    if (++spins > cfg.max_spins) {
                        *abort_flag = 1;
                        if (g.status) atomicExch(g.status, 100 + peer);
                        return false;
                    }
                    __nanosleep(40);
                }
                asm volatile("fence.proxy.async;" ::: "memory");     // the acquire orders the generic proxy; the TMA reads go through the async proxy
                ready |= 1u << peer;
            }
            mbar_expect_tx(&bars.a_full[buf], (uint32_t)nkb * kTile);
            for (int kb = 0; kb < nkb; ++kb)
                tma_load_2d(a_sm + ((size_t)buf * nkb + kb) * kTile, &maps.a[peer], kb * BK, m0, &bars.a_full[buf]);
            return true;
        };
        int a_issued = 0;
        if ((int)blockIdx.x < n_mtiles) { okay = load_a(blockIdx.x, 0); a_issued = okay ? 1 : 0; }
        for (int mt = blockIdx.x; mt < n_mtiles && okay; mt += gridDim.x, ++ai) {
            for (int nt = 0; nt < tiles_n && okay; ++nt) {
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % cfg.n_b;
                    okay = mbar_wait(&bars.b_empty[s], ((it / cfg.n_b) & 1) ^ 1, abort_flag, g.status, 1);
                    if (!okay) break;
                    mbar_expect_tx(&bars.b_full[s], kTile);
                    tma_load_2d(b_sm + (size_t)s * kTile, &map_b, kb * BK, nt * BN, &bars.b_full[s]);
                }
                // the next A tile is requested after the first column tile's weights are on their way (two A buffers), or
                // after the last one (one buffer: the wait below then covers the whole current tile)
                const bool prefetch_now = cfg.n_abuf == 2 ? nt == 0 : nt == tiles_n - 1;
                const int next = mt + gridDim.x;
                if (okay && prefetch_now && next < n_mtiles) {
                    okay = load_a(next, ai + 1);
                    if (okay) a_issued = ai + 2;
                }
            }
        }
        if (*abort_flag) {
            // drain: copies in flight must land before the CTA may exit
            for (int k = (it > cfg.n_b ? it - cfg.n_b : 0); k < it; ++k) {
                const long long t0 = clock64();
                while (!mbar_try_wait(&bars.b_full[k % cfg.n_b], (k / cfg.n_b) & 1) && clock64() - t0 < kWaitCycles) {}
            }
            for (int k = (a_issued > cfg.n_abuf ? a_issued - cfg.n_abuf : 0); k < a_issued; ++k) {
                const long long t0 = clock64();
                while (!mbar_try_wait(&bars.a_full[k % cfg.n_abuf], (k / cfg.n_abuf) & 1) && clock64() - t0 < kWaitCycles) {}
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        const uint32_t idesc = make_idesc(BM, BN, 0, 0);
        int ai = 0, it = 0, ti = 0;
        bool okay = true;
        for (int mt = blockIdx.x; mt < n_mtiles && okay; mt += gridDim.x, ++ai) {
            const int buf = ai % cfg.n_abuf;
            okay = mbar_wait(&bars.a_full[buf], (ai / cfg.n_abuf) & 1, abort_flag, g.status, 2);
            if (!okay) break;
            const uint32_t a_base = smem_u32(a_sm + (size_t)buf * nkb * kTile);
            for (int nt = 0; nt < tiles_n && okay; ++nt, ++ti) {
                const int b = ti & 1;
                okay = mbar_wait(&bars.tmem_empty[b], ((ti >> 1) & 1) ^ 1, abort_flag, g.status, 2);
                if (!okay) break;
                tc_fence_after();
                const uint32_t acc = tmem + (uint32_t)(b * BN);
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % cfg.n_b;
                    okay = mbar_wait(&bars.b_full[s], (it / cfg.n_b) & 1, abort_flag, g.status, 2);
                    if (!okay) break;
                    tc_fence_after();
                    const uint32_t a_addr = a_base + kb * kTile, b_addr = smem_u32(b_sm + (size_t)s * kTile);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_bf16(acc, make_desc(a_addr + k * 32, 16, 1024), make_desc(b_addr + k * 32, 16, 1024), idesc, (kb | k) != 0);
                    umma_commit(&bars.b_empty[s]);
                }
                if (okay) umma_commit(&bars.tmem_full[b]);
            }
            if (okay) umma_commit(&bars.a_empty[buf]);    // every MMA that reads this A buffer has completed
        }
    } else if (warp >= 2 && warp < 6) {
        // ---- epilogue ----
        const int quad = warp & 3;
        const uint64_t sd = site_seed(g.seed, g.stream_id);
        const float inv_keep = g.p > 0.f ? keep_scale(g.p) : 1.f;
        const bool staged = g.c_dtype == DT_BF16 && (g.ldc & 7) == 0 && (g.N & 7) == 0;
        const bool tma_out = cfg.tma_store != 0;
        // TMA-store path: each warp owns two 32 x 64 boxes (4 KB each, 128-byte rows, 128-byte swizzle) of the staging area
        uint8_t* stage = tma_out ? stage_c + (size_t)quad * 8192 : stage_c + (size_t)quad * 32 * kStageStrideP;
        int ti = 0;
        bool okay = true;
        for (int mt = blockIdx.x; mt < n_mtiles && okay; mt += gridDim.x) {
            int peer, m0;
            gather_tile(cfg, mt, peer, m0);
            const long long row_base = (long long)peer * cfg.chunk;
            for (int nt = 0; nt < tiles_n; ++nt, ++ti) {
                const int b = ti & 1, n0 = nt * BN;
                okay = mbar_wait(&bars.tmem_full[b], (ti >> 1) & 1, abort_flag, g.status, 3);
                if (!okay) break;
                tc_fence_after();
                const int lrow = m0 + quad * 32 + lane;
                const long long row = row_base + lrow;
                const uint32_t acc = tmem + (uint32_t)(b * BN) + ((uint32_t)(quad * 32) << 16);
                if (tma_out) {
                    // the boxes of the previous tile must have been read by the TMA engine before they are overwritten
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    __syncwarp();
                }
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    __syncwarp();
                    tmem_ld32(acc + c0, r);
                    if (c0 + 32 >= BN) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bars.tmem_empty[b]);
                    }
                    const int col0 = n0 + c0;
                    if (!staged && (lrow >= cfg.chunk || col0 >= g.N)) continue;
                    float v[32];
                    epilogue_math(r, v, (int)row, col0, g, sd, inv_keep);
                    if (tma_out) {
                        uint8_t* box = stage + (c0 >> 6) * 4096 + lane * 128;
                        const int cbase = (c0 & 63) >> 3;                       // first 16-byte chunk of this 32-column group
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            st_bf16x8(box + (((cbase + j) ^ (lane & 7)) << 4), v[j * 8], v[j * 8 + 1], v[j * 8 + 2], v[j * 8 + 3], v[j * 8 + 4],
                                      v[j * 8 + 5], v[j * 8 + 6], v[j * 8 + 7]);
                        continue;
                    }
                    if (staged) {
                        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(stage + (size_t)lane * kStageStrideP) + c0;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) st_bf16x8(dst + j, v[j], v[j + 1], v[j + 2], v[j + 3], v[j + 4], v[j + 5], v[j + 6], v[j + 7]);
                        continue;
                    }
                    if (g.c_dtype == DT_BF16) {
                        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(g.c) + (size_t)row * g.ldc + col0;
                        _Pragma("unroll") for (int j = 0; j < 32; ++j)
                            if (col0 + j < g.N) dst[j] = __float2bfloat16(v[j]);
                    } else {
                        float* dst = static_cast<float*>(g.c) + (size_t)row * g.ldc + col0;
                        _Pragma("unroll") for (int j = 0; j < 32; ++j)
                            if (col0 + j < g.N) dst[j] = v[j];
                    }
                }
                if (tma_out) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the TMA engine
                    __syncwarp();
                    if (lane == 0 && m0 + quad * 32 < cfg.chunk) {
                        if (n0 < g.N) tma_store_2d(&maps.c[peer], stage, n0, m0 + quad * 32);
                        if (n0 + 64 < g.N) tma_store_2d(&maps.c[peer], stage + 4096, n0 + 64, m0 + quad * 32);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                } else if (staged) {
                    __syncwarp();
                    const int cchunk = lane & 15;
                    const bool col_ok = n0 + cchunk * 8 + 8 <= g.N;
#pragma unroll 4
                    for (int i2 = 0; i2 < 16; ++i2) {
                        const int rr = i2 * 2 + (lane >> 4);
                        const int lr = m0 + quad * 32 + rr;
                        if (lr < cfg.chunk && col_ok) {
                            const uint4 val = *reinterpret_cast<const uint4*>(stage + (size_t)rr * kStageStrideP + cchunk * 16);
                            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(g.c) + (size_t)(row_base + lr) * g.ldc + n0 + cchunk * 8) = val;
                        }
                    }
                    __syncwarp();
                }
            }
        }
        if (tma_out && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    } else if (warp == 6 && lane == 0 && cfg.copy_out) {
        // ---- copier: the fetched A tile also lands in the local gathered matrix (rows past the chunk are clipped by the map) ----
        int ai = 0;
        for (int mt = blockIdx.x; mt < n_mtiles; mt += gridDim.x, ++ai) {
            const int buf = ai % cfg.n_abuf;
            if (!mbar_wait(&bars.a_full[buf], (ai / cfg.n_abuf) & 1, abort_flag, g.status, 4)) break;
            int peer, m0;
            gather_tile(cfg, mt, peer, m0);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            for (int kb = 0; kb < nkb; ++kb) tma_store_2d(&maps.out[peer], a_sm + ((size_t)buf * nkb + kb) * kTile, kb * BK, m0);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");      // shared memory has been read: the buffer may be refilled
            mbar_arrive(&bars.a_empty[buf]);
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 2 * kTmemCols);
}

// ------------------------------------------------------------------------------------------------------------------
// Reduce-scatter fused into C = A * B^T.  Every rank of a group computes a partial product for ALL rows, and rows
// [p * chunk, (p + 1) * chunk) are owned by rank p, which needs the sum of the partials.  The epilogue of this kernel writes
// each finished tile straight into the OWNER's memory (plain peer stores over NVLink, whole 256-byte row segments), into
// slot `my_pos` of the owner's staging area [n_peers][chunk][N]; the transfer therefore overlaps the MMAs of the following
// tiles and the partial product never exists in local memory.  After a group barrier the owner adds its n_peers slots
// (sum_slots_kernel).  Same pipeline as the persistent kernel.
// ------------------------------------------------------------------------------------------------------------------
struct ScatterCfg {
    void* slots[kMaxPeers];           // slots[p] = address of my slot inside rank p's staging area
    int chunk, n_peers;
};

__global__ void __launch_bounds__(kThreads, 1) gemm_nt_scatter_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                      const __grid_constant__ CUtensorMap map_b, GemmArgs g,
                                                                      const __grid_constant__ ScatterCfg cfg) {
    extern __shared__ uint8_t smem_raw[];
    PersistentStorage& sh = *reinterpret_cast<PersistentStorage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (g.N + BN - 1) / BN, tiles_m = (g.M + BM - 1) / BM;
    const int n_tiles = tiles_n * tiles_m;
    const int nkb = (g.K + BK - 1) / BK;
    volatile int* abort_flag = &sh.abort_flag;

    if (threadIdx.x == 0) {
        sh.abort_flag = 0;
        for (int s = 0; s < P_STAGES; ++s) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sh.tmem_full[b], 1); mbar_init(&sh.tmem_empty[b], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&sh.tmem_base, 2 * kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;

    if (warp == 0 && lane == 0) {
        int it = 0;
        bool okay = true;
        for (int tile = blockIdx.x; tile < n_tiles && okay; tile += gridDim.x) {
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % P_STAGES;
                okay = mbar_wait(&sh.empty[s], ((it / P_STAGES) & 1) ^ 1, abort_flag, g.status, 1);
                if (!okay) break;
                mbar_expect_tx(&sh.full[s], (BM + BN) * BK * 2);
                tma_load_2d(sh.a[s], &map_a, kb * BK, m0, &sh.full[s]);
                tma_load_2d(sh.b[s], &map_b, kb * BK, n0, &sh.full[s]);
            }
        }
        if (*abort_flag) {
            for (int k = (it > P_STAGES ? it - P_STAGES : 0); k < it; ++k) {
                const long long t0 = clock64();
                while (!mbar_try_wait(&sh.full[k % P_STAGES], (k / P_STAGES) & 1) && clock64() - t0 < kWaitCycles) {}
            }
        }
    } else if (warp == 1 && lane == 0) {
        const uint32_t idesc = make_idesc(BM, BN, 0, 0);
        int it = 0, ti = 0;
        bool okay = true;
        for (int tile = blockIdx.x; tile < n_tiles && okay; tile += gridDim.x, ++ti) {
            const int b = ti & 1;
            okay = mbar_wait(&sh.tmem_empty[b], ((ti >> 1) & 1) ^ 1, abort_flag, g.status, 2);
            if (!okay) break;
            tc_fence_after();
            const uint32_t acc = tmem + (uint32_t)(b * BN);
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % P_STAGES;
                okay = mbar_wait(&sh.full[s], (it / P_STAGES) & 1, abort_flag, g.status, 2);
                if (!okay) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(sh.a[s]), b_addr = smem_u32(sh.b[s]);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    umma_bf16(acc, make_desc(a_addr + k * 32, 16, 1024), make_desc(b_addr + k * 32, 16, 1024), idesc, (kb | k) != 0);
                umma_commit(&sh.empty[s]);
            }
            if (okay) umma_commit(&sh.tmem_full[b]);
        }
    } else if (warp >= 2) {
        // ---- epilogue: bf16 tile -> shared staging -> the owner's slot, 256-byte row segments ----
        const int quad = warp & 3;
        uint8_t* stage = sh.stage_c + (size_t)quad * 32 * kStageStrideP;
        int ti = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++ti) {
            const int b = ti & 1;
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            if (!mbar_wait(&sh.tmem_full[b], (ti >> 1) & 1, abort_flag, g.status, 3)) break;
            tc_fence_after();
            const uint32_t acc = tmem + (uint32_t)(b * BN) + ((uint32_t)(quad * 32) << 16);
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                __syncwarp();
                tmem_ld32(acc + c0, r);
                if (c0 + 32 >= BN) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh.tmem_empty[b]);
                }
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(stage + (size_t)lane * kStageStrideP) + c0;
#pragma unroll
                for (int j = 0; j < 32; j += 8)
                    st_bf16x8(dst + j, __uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]),
                              __uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]), __uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
            }
            __syncwarp();
            const int cchunk = lane & 15;
            const bool col_ok = n0 + cchunk * 8 + 8 <= g.N;
#pragma unroll 4
            for (int i2 = 0; i2 < 16; ++i2) {
                const int rr = i2 * 2 + (lane >> 4);
                const int grow = m0 + quad * 32 + rr;
                if (grow < g.M && col_ok) {
                    const int owner = grow / cfg.chunk, lrow = grow - owner * cfg.chunk;
                    const uint4 val = *reinterpret_cast<const uint4*>(stage + (size_t)rr * kStageStrideP + cchunk * 16);
                    *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(cfg.slots[owner]) + (size_t)lrow * g.ldc + n0 + cchunk * 8) = val;
                }
            }
            __syncwarp();
        }
        __threadfence_system();                               // the tiles must be visible to the owners after the group barrier
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 2 * kTmemCols);
}

// out[r, :] = sum over slots p (fixed order, fp32 accumulation) of slots[p][r, :]   (bf16 in; bf16 or fp32 out)
template <typename TO>
__global__ void sum_slots_kernel(const __nv_bfloat16* __restrict__ slots, int n_slots, long long slot_elems, TO* __restrict__ out,
                                 int accumulate) {
    const long long n8 = slot_elems / 8;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int p = 0; p < n_slots; ++p) {
            float v[8];
            Vec8<__nv_bfloat16>::load(slots + (size_t)p * slot_elems + i * 8, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += v[j];
        }
        if (accumulate) {
            float o[8];
            Vec8<TO>::load(out + i * 8, o);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += o[j];
        }
        Vec8<TO>::store(out + i * 8, acc);
    }
}

// ------------------------------------------------------------------------------------------------------------------
// C[N, K] += A[M, N]^T * B[M, K]  (MN-major operands, reduction over rows split across gridDim.z)
// ------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a,
                                                           const __grid_constant__ CUtensorMap map_b, GemmTNArgs g, int rows_per_split) {
    extern __shared__ uint8_t smem_raw[];
    SharedStorage& sh = *reinterpret_cast<SharedStorage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k0 = blockIdx.x * BN;                        // output column tile (features of B)
    const int n0 = blockIdx.y * BM;                        // output row tile (features of A)
    const int r_beg = blockIdx.z * rows_per_split;
    const int r_end = min(g.M, r_beg + rows_per_split);
    const int nkb = r_end > r_beg ? (r_end - r_beg + BK - 1) / BK : 0;
    volatile int* abort_flag = &sh.abort_flag;

    if (threadIdx.x == 0) {
        sh.abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
        mbar_init(&sh.tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&sh.tmem_base, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    if (nkb > 0) {
        if (warp == 0 && lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % STAGES;
                if (!mbar_wait(&sh.empty[s], ((kb / STAGES) & 1) ^ 1, abort_flag, g.status, 4)) break;
                mbar_expect_tx(&sh.full[s], (BM + BN) * BK * 2);
                const int r = r_beg + kb * BK;
                // two 64-column boxes per operand: [BK rows][64 cols] each, 128-byte rows
                tma_load_2d(sh.a[s], &map_a, n0, r, &sh.full[s]);
                tma_load_2d(sh.a[s] + BK * 64, &map_a, n0 + 64, r, &sh.full[s]);
                tma_load_2d(sh.b[s], &map_b, k0, r, &sh.full[s]);
                tma_load_2d(sh.b[s] + BK * 64, &map_b, k0 + 64, r, &sh.full[s]);
                issued = kb + 1;
            }
            if (*abort_flag) {
                for (int kb = (issued > STAGES ? issued - STAGES : 0); kb < issued; ++kb) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(&sh.full[kb % STAGES], (kb / STAGES) & 1) && clock64() - t0 < kWaitCycles) {}
                }
            }
        } else if (warp == 1 && lane == 0) {
            const uint32_t idesc = make_idesc(BM, BN, 1, 1);
            bool okay = true;
            for (int kb = 0; kb < nkb && okay; ++kb) {
                const int s = kb % STAGES;
                okay = mbar_wait(&sh.full[s], (kb / STAGES) & 1, abort_flag, g.status, 5);
                if (!okay) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(sh.a[s]), b_addr = smem_u32(sh.b[s]);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    // 16 reduction rows = two 8-row groups of 1024 bytes; the two 64-wide MN blocks are BK * 128 bytes apart
                    const uint64_t ad = make_desc(a_addr + k * 2048, BK * 128, 1024);
                    const uint64_t bd = make_desc(b_addr + k * 2048, BK * 128, 1024);
                    umma_bf16(tmem, ad, bd, idesc, (kb | k) != 0);
                }
                umma_commit(&sh.empty[s]);
            }
            if (okay) umma_commit(&sh.tmem_full);
        } else if (warp >= 2) {
            const bool okay = mbar_wait(&sh.tmem_full, 0, abort_flag, g.status, 6);
            tc_fence_after();
            if (okay) {
                const int quad = warp & 3;
                const int row = n0 + quad * 32 + lane;
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + c0, r);
                    if (row >= g.N) continue;
                    float* dst = g.c + (size_t)row * g.ldc + k0 + c0;
                    if (k0 + c0 + 32 <= g.K && (g.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(g.c) & 15) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)          // 16-byte vector reductions: a quarter of the atomic operations
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j), "f"(__uint_as_float(r[j])),
                                         "f"(__uint_as_float(r[j + 1])), "f"(__uint_as_float(r[j + 2])), "f"(__uint_as_float(r[j + 3]))
                                         : "memory");
                        continue;
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (k0 + c0 + j < g.K) atomicAdd(dst + j, __uint_as_float(r[j]));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// Wide-tile variant of the weight-gradient GEMM: one CTA owns a 256 x 256 tile of C (two 128-row accumulators of 256 columns
// = all 512 TMEM columns) and a slice of the row range.  The 128 x 128 kernel above re-reads A once per column tile and B once
// per row tile of C; for C = [1024, 256] over 169K rows that is 1.4 GB through L2 per product and the kernel runs at the L2's
// speed.  256 x 256 tiles halve that traffic (each 64 KB stage of operands feeds four times the MMA work of a 32 KB stage).
constexpr int TN2_STAGES = 3;
struct __align__(1024) TN2Storage {
    __nv_bfloat16 a[TN2_STAGES][BK * 256];                 // 4 boxes of [BK rows][64 columns], 8 KB each
    __nv_bfloat16 b[TN2_STAGES][BK * 256];
    uint64_t full[TN2_STAGES];
    uint64_t empty[TN2_STAGES];
    uint64_t tmem_full;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void red_add_v4(float* dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)),
                 "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
                 : "memory");
}

__global__ void __launch_bounds__(kThreads, 1) gemm_tn256_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                 const __grid_constant__ CUtensorMap map_b, GemmTNArgs g, int rows_per_split) {
    extern __shared__ uint8_t smem_raw[];
    TN2Storage& sh = *reinterpret_cast<TN2Storage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k0 = blockIdx.x * 256;                       // output column tile (features of B)
    const int n0 = blockIdx.y * 256;                       // output row tile (features of A)
    const int r_beg = blockIdx.z * rows_per_split;
    const int r_end = min(g.M, r_beg + rows_per_split);
    const int nkb = r_end > r_beg ? (r_end - r_beg + BK - 1) / BK : 0;
    volatile int* abort_flag = &sh.abort_flag;

    if (threadIdx.x == 0) {
        sh.abort_flag = 0;
        for (int s = 0; s < TN2_STAGES; ++s) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
        mbar_init(&sh.tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&sh.tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    if (nkb > 0) {
        if (warp == 0 && lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % TN2_STAGES;
                if (!mbar_wait(&sh.empty[s], ((kb / TN2_STAGES) & 1) ^ 1, abort_flag, g.status, 4)) break;
                mbar_expect_tx(&sh.full[s], 2 * BK * 256 * 2);
                const int r = r_beg + kb * BK;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    tma_load_2d(sh.a[s] + i * BK * 64, &map_a, n0 + 64 * i, r, &sh.full[s]);
                    tma_load_2d(sh.b[s] + i * BK * 64, &map_b, k0 + 64 * i, r, &sh.full[s]);
                }
                issued = kb + 1;
            }
            if (*abort_flag) {
                for (int kb = (issued > TN2_STAGES ? issued - TN2_STAGES : 0); kb < issued; ++kb) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(&sh.full[kb % TN2_STAGES], (kb / TN2_STAGES) & 1) && clock64() - t0 < kWaitCycles) {}
                }
            }
        } else if (warp == 1 && lane == 0) {
            const uint32_t idesc = make_idesc(128, 256, 1, 1);
            bool okay = true;
            for (int kb = 0; kb < nkb && okay; ++kb) {
                const int s = kb % TN2_STAGES;
                okay = mbar_wait(&sh.full[s], (kb / TN2_STAGES) & 1, abort_flag, g.status, 5);
                if (!okay) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(sh.a[s]), b_addr = smem_u32(sh.b[s]);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    // 16 reduction rows = two 8-row groups of 1024 bytes; consecutive 64-wide MN blocks are BK * 128 bytes apart
                    const uint64_t bd = make_desc(b_addr + k * 2048, BK * 128, 1024);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint64_t ad = make_desc(a_addr + h * 2 * BK * 128 + k * 2048, BK * 128, 1024);
                        umma_bf16(tmem + (uint32_t)(h * 256), ad, bd, idesc, (kb | k) != 0);
                    }
                }
                umma_commit(&sh.empty[s]);
            }
            if (okay) umma_commit(&sh.tmem_full);
        } else if (warp >= 2) {
            const bool okay = mbar_wait(&sh.tmem_full, 0, abort_flag, g.status, 6);
            tc_fence_after();
            if (okay) {
                const int quad = warp & 3;
                for (int h = 0; h < 2; ++h) {
                    const int row = n0 + h * 128 + quad * 32 + lane;
                    for (int c0 = 0; c0 < 256; c0 += 32) {
                        uint32_t r[32];
                        tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(h * 256 + c0), r);
                        if (row >= g.N) continue;
                        float* dst = g.c + (size_t)row * g.ldc + k0 + c0;           // K % 256 == 0 and 16-byte aligned rows: whole vectors
#pragma unroll
                        for (int j = 0; j < 32; j += 4) red_add_v4(dst + j, r[j], r[j + 1], r[j + 2], r[j + 3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

}  // namespace

// ---- host side: tensor maps ------------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    });
    return fn;
}

// 2D bf16 tensor [rows, cols] with row stride ld (elements); box = [box_rows][box_cols]
bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows, int box_cols) {
    using Key = std::tuple<const void*, int, int, int, int, int>;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    Key key{base, rows, cols, ld, box_rows, box_cols};
    {
        std::lock_guard<std::mutex> lk(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *map = it->second; return true; }
    }
    auto fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    std::lock_guard<std::mutex> lk(mu);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *map;
    return true;
}

namespace {

constexpr size_t kSmemBytes = sizeof(SharedStorage) + 1024;

}  // namespace

bool gemm_tcgen05_supported(int M, int N, int K, int lda, int ldb, int ldc) {
    (void)ldc;
    return M > 0 && N > 0 && K > 0 && (lda % 8) == 0 && (ldb % 8) == 0 && (K % 8) == 0;
}

int gemm_nt_gather(const GemmArgs& g, const void* const* a_peers, int n_peers, int chunk, void* gathered, cudaStream_t s,
                   const GatherWait* wait);

// GT_GEMM_KERNEL: "simple" = one tile per CTA, "persistent" = the tile-walking kernel for every shape (comparison runs)
static char env_kernel() {
    const char* env = getenv("GT_GEMM_KERNEL");
    return env ? env[0] : 0;
}

int gemm_tcgen05(const GemmArgs& g, cudaStream_t s) {
    if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.b) & 15)) return -2;
    CUtensorMap ma, mb;
    if (!make_map(&ma, g.a, g.M, g.K, g.lda, BM, BK)) return -1;
    if (!make_map(&mb, g.b, g.N, g.K, g.ldb, BN, BK)) return -1;
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(gemm_nt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        attr = true;
    }
    static int n_sm = 0;
    static bool simple = false;
    if (n_sm == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        const char* env = getenv("GT_GEMM_KERNEL");
        simple = env && env[0] == 's';                    // "simple": the one-tile-per-CTA kernel (comparison / debugging)
        cudaFuncSetAttribute(gemm_nt_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(PersistentStorage) + 1024));
    }
    // GT_GEMM_KERNEL=a: run local short-K products on the A-stationary kernel of the fused all-gather (one "peer": this GPU).
    // Measured on 169,344 x 256 -> 1024 / 512 / 256 and 512 -> 256: the tile-walking kernel is faster on every shape (0.142 /
    // 0.074 / 0.040 / 0.062 ms against 0.155 / 0.086 / 0.051 / 0.094 ms): neighbouring CTAs work on the same row tile at the same
    // time, so its re-reads of A hit L2, and its ring holds five whole k-steps.
    static const bool a_stationary = env_kernel() == 'a';
    if (!simple && a_stationary && !g.accumulate && g.K <= 512 && g.N > BN) {
        const void* self[1] = {g.a};
        return gemm_nt_gather(g, self, 1, g.M, nullptr, s, nullptr);
    }
    if (simple) {
        dim3 grid((g.N + BN - 1) / BN, (g.M + BM - 1) / BM);
        gemm_nt_kernel<<<grid, kThreads, kSmemBytes, s>>>(ma, mb, g);
    } else {
        const int tiles = ((g.N + BN - 1) / BN) * ((g.M + BM - 1) / BM);
        gemm_nt_persistent_kernel<<<tiles < n_sm ? tiles : n_sm, kThreads, sizeof(PersistentStorage) + 1024, s>>>(ma, mb, g);
    }
    return (int)cudaGetLastError();
}

int gemm_tn_tcgen05(const GemmTNArgs& g, cudaStream_t s) {
    if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.b) & 15)) return -2;
    if ((g.lda % 8) || (g.ldb % 8) || (g.N % 8) || (g.K % 8)) return -3;
    CUtensorMap ma, mb;
    if (!make_map(&ma, g.a, g.M, g.N, g.lda, BK, 64)) return -1;
    if (!make_map(&mb, g.b, g.M, g.K, g.ldb, BK, 64)) return -1;
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(gemm_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        attr = true;
    }
    // 256 x 256 tiles when C has at least four of them (measured at 169K rows: [1024, 256] 0.085 ms against 0.132 ms with 128 x 128
    // tiles; [512, 256] 0.063 against 0.057: too few tiles to fill the SMs without splitting the rows 70-fold).  GT_GEMM_TN=narrow
    // / wide forces one kernel.
    static const char tn_env = getenv("GT_GEMM_TN") ? getenv("GT_GEMM_TN")[0] : 0;
    const bool wide_shape = (g.N % 256) == 0 && (g.K % 256) == 0 && g.M >= 148 * BK && (g.ldc % 4) == 0 && (reinterpret_cast<uintptr_t>(g.c) & 15) == 0;
    if (wide_shape && tn_env != 'n' && ((g.N / 256) * (g.K / 256) >= 4 || tn_env == 'w')) {
        static bool attr2 = false;
        if (!attr2) {
            cudaFuncSetAttribute(gemm_tn256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(TN2Storage) + 1024));
            attr2 = true;
        }
        const int tiles2 = (g.K / 256) * (g.N / 256);
        int splits2 = (148 + tiles2 - 1) / tiles2;
        const int kblocks2 = (g.M + BK - 1) / BK;
        if (splits2 > kblocks2) splits2 = kblocks2;
        const int rows2 = ((kblocks2 + splits2 - 1) / splits2) * BK;
        splits2 = (g.M + rows2 - 1) / rows2;
        if (!g.accumulate) cudaMemsetAsync(g.c, 0, (size_t)g.N * g.ldc * sizeof(float), s);
        dim3 grid2(g.K / 256, g.N / 256, splits2);
        gemm_tn256_kernel<<<grid2, kThreads, sizeof(TN2Storage) + 1024, s>>>(ma, mb, g, rows2);
        return (int)cudaGetLastError();
    }
    const int tiles = ((g.K + BN - 1) / BN) * ((g.N + BM - 1) / BM);
    int splits = (2 * 148 + tiles - 1) / tiles;
    const int kblocks = (g.M + BK - 1) / BK;
    if (splits > kblocks) splits = kblocks;
    if (splits < 1) splits = 1;
    const int rows_per_split = ((kblocks + splits - 1) / splits) * BK;
    splits = (g.M + rows_per_split - 1) / rows_per_split;
    if (!g.accumulate) cudaMemsetAsync(g.c, 0, (size_t)g.N * g.ldc * sizeof(float), s);
    dim3 grid((g.K + BN - 1) / BN, (g.N + BM - 1) / BM, splits);
    gemm_tn_kernel<<<grid, kThreads, kSmemBytes, s>>>(ma, mb, g, rows_per_split);
    return (int)cudaGetLastError();
}


// A rows come from the peers' buffers (a_peers[p]: [chunk, K] bf16, row stride lda); g.a is ignored, g.M = n_peers * chunk.
// gathered != nullptr additionally receives the gathered A ([n_peers * chunk, K], row stride lda).
int gemm_nt_gather(const GemmArgs& g, const void* const* a_peers, int n_peers, int chunk, void* gathered, cudaStream_t s,
                   const GatherWait* wait) {
    if (n_peers < 1 || n_peers > kMaxPeers) return -5;
    const int nkb = (g.K + BK - 1) / BK;
    if (nkb > 8 || (g.K % 8) || (g.lda % 8) || (g.ldb % 8)) return -4;
    if (reinterpret_cast<uintptr_t>(g.b) & 15) return -2;
    GatherMaps maps;
    memset(&maps, 0, sizeof(maps));
    for (int p = 0; p < n_peers; ++p) {
        if (reinterpret_cast<uintptr_t>(a_peers[p]) & 15) return -2;
        if (!make_map(&maps.a[p], a_peers[p], chunk, g.K, g.lda, BM, BK)) return -1;
        if (gathered) {
            const void* base = static_cast<const __nv_bfloat16*>(gathered) + (size_t)p * chunk * g.lda;
            if (reinterpret_cast<uintptr_t>(base) & 15) return -2;
            if (!make_map(&maps.out[p], base, chunk, g.K, g.lda, BM, BK)) return -1;
        }
    }
    CUtensorMap mb;
    if (!make_map(&mb, g.b, g.N, g.K, g.ldb, BN, BK)) return -1;
    const bool tma_store = g.c_dtype == DT_BF16 && (g.ldc % 8) == 0 && (g.N % 8) == 0 && (reinterpret_cast<uintptr_t>(g.c) & 15) == 0 &&
                           ((size_t)chunk * g.ldc * 2) % 16 == 0 && env_kernel() != 'l';      // GT_GEMM_KERNEL=lsu: plain-store epilogue
    if (tma_store)
        for (int p = 0; p < n_peers; ++p)
            if (!make_map(&maps.c[p], static_cast<const __nv_bfloat16*>(g.c) + (size_t)p * chunk * g.ldc, chunk, g.N, g.ldc, 32, 64)) return -1;
    constexpr int kTile = BM * BK * 2;
    const int fixed = 4 * 32 * kStageStrideP + (int)sizeof(GatherBars) + 1024;
    const int slots = (232448 - fixed) / kTile;
    GatherCfg cfg;
    cfg.chunk = chunk; cfg.n_peers = n_peers; cfg.tiles_per_peer = (chunk + BM - 1) / BM; cfg.copy_out = gathered != nullptr;
    cfg.nkb = nkb;
    cfg.tma_store = tma_store ? 1 : 0;
    cfg.wait_flags = wait ? wait->flags : nullptr;
    cfg.wait_counter = wait ? wait->counter : nullptr;
    cfg.max_spins = wait ? wait->max_spins : 0;
    cfg.self = wait ? wait->self : 0;
    if (cfg.self < 0 || cfg.self >= n_peers) return -5;
    // two A buffers whenever they fit: the fetch of the next row tile overlaps the MMAs of the current one (measured: worth more
    // than a deeper ring for the weight tiles)
    cfg.n_abuf = (2 * nkb + 3 <= slots) ? 2 : 1;
    cfg.n_b = slots - cfg.n_abuf * nkb;
    if (cfg.n_b > G_MAX_B) cfg.n_b = G_MAX_B;
    if (cfg.n_b < 2) return -4;
    const int smem = (cfg.n_abuf * nkb + cfg.n_b) * kTile + fixed;
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        cudaFuncSetAttribute(gemm_nt_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    }
    const int n_mtiles = n_peers * cfg.tiles_per_peer;
    gemm_nt_gather_kernel<<<n_mtiles < n_sm ? n_mtiles : n_sm, kGatherThreads, smem, s>>>(maps, mb, g, cfg);
    return (int)cudaGetLastError();
}

// The product's row block p goes to slots[p] (my slot in rank p's staging area, [chunk, N] bf16 with row stride g.ldc).
int gemm_nt_scatter(const GemmArgs& g, void* const* slots, int n_peers, int chunk, cudaStream_t s) {
    if (n_peers < 1 || n_peers > kMaxPeers) return -5;
    if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.b) & 15)) return -2;
    if ((g.N % 8) || (g.ldc % 8) || (g.K % 8) || (g.lda % 8) || (g.ldb % 8)) return -4;
    CUtensorMap ma, mb;
    if (!make_map(&ma, g.a, g.M, g.K, g.lda, BM, BK)) return -1;
    if (!make_map(&mb, g.b, g.N, g.K, g.ldb, BN, BK)) return -1;
    ScatterCfg cfg;
    memset(&cfg, 0, sizeof(cfg));
    for (int p = 0; p < n_peers; ++p) {
        if (reinterpret_cast<uintptr_t>(slots[p]) & 15) return -2;
        cfg.slots[p] = slots[p];
    }
    cfg.chunk = chunk; cfg.n_peers = n_peers;
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        cudaFuncSetAttribute(gemm_nt_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(PersistentStorage) + 1024));
    }
    const int tiles = ((g.N + BN - 1) / BN) * ((g.M + BM - 1) / BM);
    gemm_nt_scatter_kernel<<<tiles < n_sm ? tiles : n_sm, kThreads, sizeof(PersistentStorage) + 1024, s>>>(ma, mb, g, cfg);
    return (int)cudaGetLastError();
}

void sum_slots(const void* slots, int n_slots, long long slot_elems, void* out, int out_dtype, int accumulate, cudaStream_t s) {
    const long long n8 = slot_elems / 8;
    const int blocks = (int)((n8 + 255) / 256 < 148 * 8 ? (n8 + 255) / 256 : 148 * 8);
    if (blocks <= 0) return;
    if (out_dtype == DT_BF16)
        sum_slots_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(slots), n_slots, slot_elems,
                                                              static_cast<__nv_bfloat16*>(out), accumulate);
    else
        sum_slots_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(slots), n_slots, slot_elems, static_cast<float*>(out),
                                                      accumulate);
}

}  // namespace gt
