// Row-wise dense kernels (bandwidth-bound): fused dropout + residual + LayerNorm forward / backward, bias + activation +
// dropout epilogues, masked cross-entropy forward + backward, multi-tensor AdamW with global-norm clipping, casts.
// One warp per row, 16-byte vector accesses, fp32 arithmetic; per-block partial sums for the parameter gradients are
// written to a [n_blocks, d] buffer and folded by reduce_partials (deterministic, no global atomics).
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"

namespace gt {
namespace {

constexpr int kWarps = 4;
constexpr int kMaxCpl = 4;      // up to 4 * 32 * 8 = 1024 features per row

__device__ __forceinline__ uint64_t site_seed(const long long* seed, long long stream_id) {
    uint64_t s0 = seed ? (uint64_t)seed[0] : 0x1234567ull, s1 = seed ? (uint64_t)seed[1] : 0ull;
    return s0 + 0x9E3779B97F4A7C15ull * (s1 * 4096ull + (uint64_t)stream_id + 1ull);
}

__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_grad(float x) {
    return 0.5f * (1.f + erff(x * 0.70710678118654752f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}

// z = x + dropout(y + ybias) for one 8-chunk
template <typename T>
__device__ __forceinline__ void load_z(const T* y, const T* x, const float* ybias, size_t row, int d, int f, float p, uint64_t sd,
                                       float (&z)[8], float (&keep)[8], const float* acc = nullptr, float inv_l = 1.f) {
    float yv[8];
    if (acc) {
        Vec8<float>::load(acc + row * d + f, yv);
#pragma unroll
        for (int k = 0; k < 8; ++k) yv[k] *= inv_l;
    } else {
        Vec8<T>::load(y + row * d + f, yv);
    }
    const float inv = p > 0.f ? keep_scale(p) : 1.f;
    const uint32_t kb = p > 0.f ? keep_bits8(sd, (row * d + f) >> 3, drop_threshold(p)) : 0xffu;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        if (ybias) yv[k] += ybias[f + k];
        keep[k] = ((kb >> k) & 1u) ? inv : 0.f;
        z[k] = yv[k] * keep[k];
    }
    if (x) {
        float xv[8];
        Vec8<T>::load(x + row * d + f, xv);
#pragma unroll
        for (int k = 0; k < 8; ++k) z[k] += xv[k];
    }
}

// Rows in flight per warp: a row is one dependent chain (load -> two warp reductions -> store), so bandwidth comes from
// running several rows' loads at once; narrow rows leave registers for 4 (forward) / 2 (backward) of them.
template <typename T, int CPL>
__global__ void __launch_bounds__(kWarps * 32) ln_fwd_kernel(LayerNormArgs a) {
    constexpr int R = CPL == 1 ? 4 : (CPL == 2 ? 2 : 1);
    const int lane = threadIdx.x & 31, nch = a.d >> 3;
    const uint64_t sd = site_seed(a.seed, a.stream_id);
    const int n_warps = gridDim.x * kWarps;
    for (int row0 = (blockIdx.x * kWarps + (threadIdx.x >> 5)) * R; row0 < a.n; row0 += n_warps * R) {
        float z[R][CPL][8], sum[R], var[R], mean[R], rstd[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            sum[r] = 0.f;
            const int row = row0 + r;
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                const int ch = lane + 32 * i;
                if (row < a.n && ch < nch) {
                    float keep[8];
                    const float inv_l = a.acc ? 1.f / (a.l[(size_t)row * a.H + ((ch << 3) / (a.d / a.H))] + a.eps_l) : 1.f;
                    load_z<T>(static_cast<const T*>(a.y), static_cast<const T*>(a.x), a.ybias, row, a.d, ch << 3, a.p, sd, z[r][i], keep, a.acc, inv_l);
#pragma unroll
                    for (int k = 0; k < 8; ++k) sum[r] += z[r][i][k];
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) z[r][i][k] = 0.f;
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) mean[r] = warp_sum(sum[r]) / a.d;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            var[r] = 0.f;
#pragma unroll
            for (int i = 0; i < CPL; ++i)
                if (lane + 32 * i < nch)
#pragma unroll
                    for (int k = 0; k < 8; ++k) { const float t = z[r][i][k] - mean[r]; var[r] = fmaf(t, t, var[r]); }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) rstd[r] = rsqrtf(warp_sum(var[r]) / a.d + a.eps);
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            const int ch = lane + 32 * i;
            if (ch < nch) {
                const int f = ch << 3;
                float gam[8], bet[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) { gam[k] = a.gamma[f + k]; bet[k] = a.beta[f + k]; }
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (row0 + r < a.n) {
                        float o[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) o[k] = (z[r][i][k] - mean[r]) * rstd[r] * gam[k] + bet[k];
                        Vec8<T>::store(static_cast<T*>(a.out) + (size_t)(row0 + r) * a.d + f, o);
                    }
                }
            }
        }
        if (lane == 0 && a.mean_rstd) {
#pragma unroll
            for (int r = 0; r < R; ++r)
                if (row0 + r < a.n) { a.mean_rstd[2 * (row0 + r)] = mean[r]; a.mean_rstd[2 * (row0 + r) + 1] = rstd[r]; }
        }
    }
}

template <typename T, int CPL>
__global__ void __launch_bounds__(kWarps * 32) ln_bwd_kernel(LayerNormBwdArgs a) {
    constexpr int R = CPL == 1 ? 2 : 1;
    extern __shared__ float smem[];                    // [3][d] block accumulators: dgamma, dbeta, dybias
    const int lane = threadIdx.x & 31, nch = a.d >> 3;
    for (int i = threadIdx.x; i < 3 * a.d; i += blockDim.x) smem[i] = 0.f;
    __syncthreads();
    const uint64_t sd = site_seed(a.seed, a.stream_id);
    const float inv_keep = a.p > 0.f ? keep_scale(a.p) : 1.f;
    const int hd = a.acc ? a.d / a.H : a.d;
    float dgam[CPL][8], dbet[CPL][8], dyb[CPL][8];
#pragma unroll
    for (int i = 0; i < CPL; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) { dgam[i][k] = 0.f; dbet[i][k] = 0.f; dyb[i][k] = 0.f; }
    float gam[CPL][8];
#pragma unroll
    for (int i = 0; i < CPL; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) gam[i][k] = (lane + 32 * i) < nch ? a.gamma[((lane + 32 * i) << 3) + k] : 0.f;
    const int n_warps = gridDim.x * kWarps;
    for (int row0 = (blockIdx.x * kWarps + (threadIdx.x >> 5)) * R; row0 < a.n; row0 += n_warps * R) {
        float zh[R][CPL][8], dzh[R][CPL][8], rstd[R], s1[R], s2[R], inv_l[R][CPL];
        uint32_t keep_bits[R][CPL];                    // dropout mask of the lane's chunk, one bit per element
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = row0 + r;
            const bool live = row < a.n;
            const float mean = live ? a.mean_rstd[2 * row] : 0.f;
            rstd[r] = live ? a.mean_rstd[2 * row + 1] : 0.f;
            s1[r] = 0.f; s2[r] = 0.f;
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                const int ch = lane + 32 * i;
                keep_bits[r][i] = 0u;
                inv_l[r][i] = 1.f;
                if (live && ch < nch) {
                    const int f = ch << 3;
                    float z[8], go[8], keep[8];
                    if (a.acc) inv_l[r][i] = 1.f / (a.l[(size_t)row * a.H + f / hd] + a.eps_l);
                    load_z<T>(static_cast<const T*>(a.y), static_cast<const T*>(a.x), a.ybias, row, a.d, f, a.p, sd, z, keep, a.acc, inv_l[r][i]);
#pragma unroll
                    for (int k = 0; k < 8; ++k) keep_bits[r][i] |= (keep[k] != 0.f ? 1u : 0u) << k;
                    Vec8<T>::load(static_cast<const T*>(a.dout) + (size_t)row * a.d + f, go);
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        zh[r][i][k] = (z[k] - mean) * rstd[r];
                        dzh[r][i][k] = go[k] * gam[i][k];
                        s1[r] += dzh[r][i][k];
                        s2[r] = fmaf(dzh[r][i][k], zh[r][i][k], s2[r]);
                        dgam[i][k] = fmaf(go[k], zh[r][i][k], dgam[i][k]);
                        dbet[i][k] += go[k];
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) { zh[r][i][k] = 0.f; dzh[r][i][k] = 0.f; }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) { s1[r] = warp_sum(s1[r]) / a.d; s2[r] = warp_sum(s2[r]) / a.d; }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = row0 + r;
            const bool live = row < a.n;
            float dl_part[CPL];
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                dl_part[i] = 0.f;
                const int ch = lane + 32 * i;
                if (live && ch < nch) {
                    const int f = ch << 3;
                    float dz[8], dy[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        dz[k] = rstd[r] * (dzh[r][i][k] - s1[r] - zh[r][i][k] * s2[r]);
                        dy[k] = ((keep_bits[r][i] >> k) & 1u) ? dz[k] * inv_keep : 0.f;
                        dyb[i][k] += dy[k];
                    }
                    if (a.acc) {
                        // dacc = dy / (l + eps);  dl[head] = -sum_f dy * acc / (l + eps)^2 (summed over the head's lanes below)
                        float av[8], da[8];
                        Vec8<float>::load(a.acc + (size_t)row * a.d + f, av);
                        float part = 0.f;
#pragma unroll
                        for (int k = 0; k < 8; ++k) { da[k] = dy[k] * inv_l[r][i]; part = fmaf(dy[k], av[k], part); }
                        Vec8<float>::store(a.dacc + (size_t)row * a.d + f, da);
                        dl_part[i] = -part * inv_l[r][i] * inv_l[r][i];
                    } else {
                        Vec8<T>::store(static_cast<T*>(a.dy) + (size_t)row * a.d + f, dy);
                    }
                    if (a.dx) {
                        T* dxp = static_cast<T*>(a.dx) + (size_t)row * a.d + f;
                        if (a.accumulate_dx) {
                            float old[8];
                            Vec8<T>::load(dxp, old);
#pragma unroll
                            for (int k = 0; k < 8; ++k) dz[k] += old[k];
                        }
                        Vec8<T>::store(dxp, dz);
                    }
                }
            }
            if (a.acc) {
                // a head spans (d / H) / 8 consecutive lanes (a power of two): finish dl with xor shuffles, all lanes take part
                const int lph = hd >> 3;
#pragma unroll
                for (int i = 0; i < CPL; ++i) {
                    float v = dl_part[i];
                    for (int o = lph >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(GT_FULL_MASK, v, o);
                    const int ch = lane + 32 * i;
                    if (live && ch < nch && (ch & (lph - 1)) == 0) a.dl[(size_t)row * a.H + (ch << 3) / hd] = v;
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
        int ch = lane + 32 * i;
        if (ch < nch) {
            int f = ch << 3;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                atomicAdd(&smem[f + k], dgam[i][k]);
                atomicAdd(&smem[a.d + f + k], dbet[i][k]);
                atomicAdd(&smem[2 * a.d + f + k], dyb[i][k]);
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < a.d; i += blockDim.x) {
        a.dgamma_part[(size_t)blockIdx.x * a.part_stride + i] = smem[i];
        a.dbeta_part[(size_t)blockIdx.x * a.part_stride + i] = smem[a.d + i];
        if (a.dybias_part) a.dybias_part[(size_t)blockIdx.x * a.part_stride + i] = smem[2 * a.d + i];
    }
}

// ------------------------------------------------------------------------------------------------------------------
// LayerNorm kernels for rows of up to 256 bf16 features whose operands arrive through a per-thread cp.async ring in shared
// memory: a warp keeps the loads of kLnStages - 1 future rows in flight without holding them in registers (a row is a
// dependent chain of load -> two warp reductions -> store, so bandwidth comes only from rows in flight).  Every lane copies and
// later reads only its own chunks: no synchronisation between lanes.  Same arithmetic as ln_fwd_kernel / ln_bwd_kernel.
// ------------------------------------------------------------------------------------------------------------------
constexpr int kLnStages = 8;

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_8(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void unpack_bf16x8(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 x = __bfloat1622float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
}

// ring layout per block: uint4 [stage][slot][thread] followed by float2 [stage][thread] (mean, rstd) and float [stage][thread] (l)
template <bool ACC, bool BWD>
struct LnRing {
    static constexpr int kSlots = (ACC ? 2 : 1) + 1 + (BWD ? 1 : 0);            // y (or acc lo / hi), x, dout
    static constexpr int kThreads = kWarps * 32;
    static constexpr size_t kBytes = (size_t)kLnStages * kThreads * (kSlots * 16 + 8 + 4);
    uint4* data; float2* stat; float* lv;
    __device__ LnRing(uint8_t* base) {
        data = reinterpret_cast<uint4*>(base);
        stat = reinterpret_cast<float2*>(base + (size_t)kLnStages * kThreads * kSlots * 16);
        lv = reinterpret_cast<float*>(base + (size_t)kLnStages * kThreads * (kSlots * 16 + 8));
    }
    __device__ uint4* slot(int stage, int s) const { return data + ((size_t)stage * kSlots + s) * kThreads + threadIdx.x; }
};

template <bool ACC>
__global__ void __launch_bounds__(kWarps * 32) ln_fwd_ring_kernel(LayerNormArgs a) {
    extern __shared__ __align__(16) uint8_t ring_raw[];
    using Ring = LnRing<ACC, false>;
    Ring ring(ring_raw);
    constexpr int NS = kLnStages, SX = ACC ? 2 : 1;
    const int lane = threadIdx.x & 31, nch = a.d >> 3, f = lane << 3;
    const bool active = lane < nch;
    const uint64_t sd = site_seed(a.seed, a.stream_id);
    const float inv_keep = a.p > 0.f ? keep_scale(a.p) : 1.f;
    const int hd = ACC ? a.d / a.H : a.d;
    const __nv_bfloat16* yb16 = static_cast<const __nv_bfloat16*>(a.y);
    const __nv_bfloat16* xb16 = static_cast<const __nv_bfloat16*>(a.x);
    float gam[8], bet[8], ybv[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        gam[k] = active ? a.gamma[f + k] : 0.f;
        bet[k] = active ? a.beta[f + k] : 0.f;
        ybv[k] = (active && a.ybias) ? a.ybias[f + k] : 0.f;
    }
    const int n_warps = gridDim.x * kWarps, w = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int n_k = w < a.n ? (a.n - w + n_warps - 1) / n_warps : 0;
    auto issue = [&](int k) {
        if (k < n_k && active) {
            const size_t row = (size_t)w + (size_t)k * n_warps;
            const int st = k % NS;
            if (ACC) {
                cp_async_16(ring.slot(st, 0), a.acc + row * a.d + f);
                cp_async_16(ring.slot(st, 1), a.acc + row * a.d + f + 4);
                cp_async_4(ring.lv + st * Ring::kThreads + threadIdx.x, a.l + row * a.H + f / hd);
            } else {
                cp_async_16(ring.slot(st, 0), yb16 + row * a.d + f);
            }
            if (a.x) cp_async_16(ring.slot(st, SX), xb16 + row * a.d + f);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int k = 0; k < NS - 1; ++k) issue(k);
    for (int k = 0; k < n_k; ++k) {
        issue(k + NS - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(NS - 1) : "memory");
        const size_t row = (size_t)w + (size_t)k * n_warps;
        const int st = k % NS;
        float z[8];
        float sum = 0.f;
        if (active) {
            float yv[8];
            if (ACC) {
                const float4 lo = *reinterpret_cast<const float4*>(ring.slot(st, 0)), hi = *reinterpret_cast<const float4*>(ring.slot(st, 1));
                const float inv_l = 1.f / (ring.lv[st * Ring::kThreads + threadIdx.x] + a.eps_l);
                yv[0] = lo.x * inv_l; yv[1] = lo.y * inv_l; yv[2] = lo.z * inv_l; yv[3] = lo.w * inv_l;
                yv[4] = hi.x * inv_l; yv[5] = hi.y * inv_l; yv[6] = hi.z * inv_l; yv[7] = hi.w * inv_l;
            } else {
                unpack_bf16x8(*ring.slot(st, 0), yv);
            }
            float xv[8];
            if (a.x) unpack_bf16x8(*ring.slot(st, SX), xv);
            const uint32_t kb = a.p > 0.f ? keep_bits8(sd, (row * a.d + f) >> 3, drop_threshold(a.p)) : 0xffu;
#pragma unroll
            for (int k2 = 0; k2 < 8; ++k2) {
                float v = yv[k2] + ybv[k2];
                v = ((kb >> k2) & 1u) ? v * inv_keep : 0.f;
                z[k2] = a.x ? v + xv[k2] : v;
                sum += z[k2];
            }
        } else {
#pragma unroll
            for (int k2 = 0; k2 < 8; ++k2) z[k2] = 0.f;
        }
        const float mean = warp_sum(sum) / a.d;
        float var = 0.f;
        if (active)
#pragma unroll
            for (int k2 = 0; k2 < 8; ++k2) { const float t = z[k2] - mean; var = fmaf(t, t, var); }
        const float rstd = rsqrtf(warp_sum(var) / a.d + a.eps);
        if (active) {
            float o[8];
#pragma unroll
            for (int k2 = 0; k2 < 8; ++k2) o[k2] = (z[k2] - mean) * rstd * gam[k2] + bet[k2];
            Vec8<__nv_bfloat16>::store(static_cast<__nv_bfloat16*>(a.out) + row * a.d + f, o);
        }
        if (lane == 0 && a.mean_rstd) { a.mean_rstd[2 * row] = mean; a.mean_rstd[2 * row + 1] = rstd; }
    }
}

template <bool ACC>
__global__ void __launch_bounds__(kWarps * 32) ln_bwd_ring_kernel(LayerNormBwdArgs a) {
    extern __shared__ __align__(16) uint8_t ring_raw[];
    using Ring = LnRing<ACC, true>;
    float* acc_sm = reinterpret_cast<float*>(ring_raw);                          // [3][d] block accumulators first, the ring after them
    Ring ring(ring_raw + ((3 * (size_t)a.d * sizeof(float) + 15) & ~size_t(15)));
    constexpr int NS = kLnStages, SX = ACC ? 2 : 1, SD = SX + 1;
    const int lane = threadIdx.x & 31, nch = a.d >> 3, f = lane << 3;
    const bool active = lane < nch;
    for (int i = threadIdx.x; i < 3 * a.d; i += blockDim.x) acc_sm[i] = 0.f;
    __syncthreads();
    const uint64_t sd = site_seed(a.seed, a.stream_id);
    const float inv_keep = a.p > 0.f ? keep_scale(a.p) : 1.f;
    const int hd = ACC ? a.d / a.H : a.d;
    const __nv_bfloat16* yb16 = static_cast<const __nv_bfloat16*>(a.y);
    const __nv_bfloat16* xb16 = static_cast<const __nv_bfloat16*>(a.x);
    const __nv_bfloat16* gob16 = static_cast<const __nv_bfloat16*>(a.dout);
    float gam[8], ybv[8], dgam[8], dbet[8], dyb[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        gam[k] = active ? a.gamma[f + k] : 0.f;
        ybv[k] = (active && a.ybias) ? a.ybias[f + k] : 0.f;
        dgam[k] = 0.f; dbet[k] = 0.f; dyb[k] = 0.f;
    }
    const int n_warps = gridDim.x * kWarps, w = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int n_k = w < a.n ? (a.n - w + n_warps - 1) / n_warps : 0;
    auto issue = [&](int k) {
        if (k < n_k && active) {
            const size_t row = (size_t)w + (size_t)k * n_warps;
            const int st = k % NS;
            if (ACC) {
                cp_async_16(ring.slot(st, 0), a.acc + row * a.d + f);
                cp_async_16(ring.slot(st, 1), a.acc + row * a.d + f + 4);
                cp_async_4(ring.lv + st * Ring::kThreads + threadIdx.x, a.l + row * a.H + f / hd);
            } else {
                cp_async_16(ring.slot(st, 0), yb16 + row * a.d + f);
            }
            if (a.x) cp_async_16(ring.slot(st, SX), xb16 + row * a.d + f);
            cp_async_16(ring.slot(st, SD), gob16 + row * a.d + f);
            cp_async_8(ring.stat + st * Ring::kThreads + threadIdx.x, a.mean_rstd + 2 * row);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int k = 0; k < NS - 1; ++k) issue(k);
    for (int k = 0; k < n_k; ++k) {
        issue(k + NS - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(NS - 1) : "memory");
        const size_t row = (size_t)w + (size_t)k * n_warps;
        const int st = k % NS;
        float zh[8], dzh[8], av[8];
        uint32_t keep_bits = 0u;
        float s1 = 0.f, s2 = 0.f, rstd = 0.f, inv_l = 1.f;
        if (active) {
            const float2 ms = ring.stat[st * Ring::kThreads + threadIdx.x];
            rstd = ms.y;
            float yv[8], go[8], xv[8];
            if (ACC) {
                const float4 lo = *reinterpret_cast<const float4*>(ring.slot(st, 0)), hi = *reinterpret_cast<const float4*>(ring.slot(st, 1));
                inv_l = 1.f / (ring.lv[st * Ring::kThreads + threadIdx.x] + a.eps_l);
                av[0] = lo.x; av[1] = lo.y; av[2] = lo.z; av[3] = lo.w; av[4] = hi.x; av[5] = hi.y; av[6] = hi.z; av[7] = hi.w;
#pragma unroll
                for (int k2 = 0; k2 < 8; ++k2) yv[k2] = av[k2] * inv_l;
            } else {
                unpack_bf16x8(*ring.slot(st, 0), yv);
            }
            if (a.x) unpack_bf16x8(*ring.slot(st, SX), xv);
            unpack_bf16x8(*ring.slot(st, SD), go);
            keep_bits = a.p > 0.f ? keep_bits8(sd, (row * a.d + f) >> 3, drop_threshold(a.p)) : 0xffu;
#pragma unroll
            for (int k2 = 0; k2 < 8; ++k2) {
                float v = yv[k2] + ybv[k2];
                v = ((keep_bits >> k2) & 1u) ? v * inv_keep : 0.f;
                const float z = a.x ? v + xv[k2] : v;
                zh[k2] = (z - ms.x) * rstd;
                dzh[k2] = go[k2] * gam[k2];
                s1 += dzh[k2];
                s2 = fmaf(dzh[k2], zh[k2], s2);
                dgam[k2] = fmaf(go[k2], zh[k2], dgam[k2]);
                dbet[k2] += go[k2];
            }
        }
        s1 = warp_sum(s1) / a.d;
        s2 = warp_sum(s2) / a.d;
        float dl_part = 0.f;
        if (active) {
            float dz[8], dy[8];
#pragma unroll
            for (int k2 = 0; k2 < 8; ++k2) {
                dz[k2] = rstd * (dzh[k2] - s1 - zh[k2] * s2);
                dy[k2] = ((keep_bits >> k2) & 1u) ? dz[k2] * inv_keep : 0.f;
                dyb[k2] += dy[k2];
            }
            if (ACC) {
                float da[8], part = 0.f;
#pragma unroll
                for (int k2 = 0; k2 < 8; ++k2) { da[k2] = dy[k2] * inv_l; part = fmaf(dy[k2], av[k2], part); }
                Vec8<float>::store(a.dacc + row * a.d + f, da);
                dl_part = -part * inv_l * inv_l;
            } else {
                Vec8<__nv_bfloat16>::store(static_cast<__nv_bfloat16*>(a.dy) + row * a.d + f, dy);
            }
            if (a.dx) {
                __nv_bfloat16* dxp = static_cast<__nv_bfloat16*>(a.dx) + row * a.d + f;
                if (a.accumulate_dx) {
                    float old[8];
                    Vec8<__nv_bfloat16>::load(dxp, old);
#pragma unroll
                    for (int k2 = 0; k2 < 8; ++k2) dz[k2] += old[k2];
                }
                Vec8<__nv_bfloat16>::store(dxp, dz);
            }
        }
        if (ACC) {
            const int lph = hd >> 3;
            float v = dl_part;
            for (int o = lph >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(GT_FULL_MASK, v, o);
            if (active && (lane & (lph - 1)) == 0) a.dl[row * a.H + f / hd] = v;
        }
    }
    if (active) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            atomicAdd(&acc_sm[f + k], dgam[k]);
            atomicAdd(&acc_sm[a.d + f + k], dbet[k]);
            atomicAdd(&acc_sm[2 * a.d + f + k], dyb[k]);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < a.d; i += blockDim.x) {
        a.dgamma_part[(size_t)blockIdx.x * a.part_stride + i] = acc_sm[i];
        a.dbeta_part[(size_t)blockIdx.x * a.part_stride + i] = acc_sm[a.d + i];
        if (a.dybias_part) a.dybias_part[(size_t)blockIdx.x * a.part_stride + i] = acc_sm[2 * a.d + i];
    }
}

// out[r, :] = x[r, :] + tab_a[idx_a[r], :] (+ tab_b[idx_b[r], :]): embedding lookups added to a feature matrix in one pass
// (degree / label / token embeddings).  idx < 0 or == pad adds nothing.  Backward of the tables: fp32 atomics per row.
template <typename T>
__global__ void embed_add_kernel(const T* x, const float* tab_a, const long long* idx_a, long long pad_a, const float* tab_b,
                                 const long long* idx_b, long long pad_b, T* out, long long n, int d) {
    const int cpr = d >> 3;
    const long long total = n * cpr;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cpr;
        const int f = (int)(i - r * cpr) << 3;
        float v[8];
        Vec8<T>::load(x + r * d + f, v);
        const long long ia = idx_a[r];
        if (ia >= 0 && ia != pad_a) {
            float e[8];
            Vec8<float>::load(tab_a + ia * d + f, e);
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] += e[k];
        }
        if (tab_b) {
            const long long ib = idx_b[r];
            if (ib >= 0 && ib != pad_b) {
                float e[8];
                Vec8<float>::load(tab_b + ib * d + f, e);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[k] += e[k];
            }
        }
        Vec8<T>::store(out + r * d + f, v);
    }
}

template <typename T>
__global__ void embed_add_bwd_kernel(const T* dout, const long long* idx, long long pad, float* dtab, long long n, int d) {
    const int cpr = d >> 3;
    const long long total = n * cpr;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cpr;
        const long long ix = idx[r];
        if (ix < 0 || ix == pad) continue;
        const int f = (int)(i - r * cpr) << 3;
        float g[8];
        Vec8<T>::load(dout + r * d + f, g);
#pragma unroll
        for (int k = 0; k < 8; ++k) atomicAdd(dtab + ix * d + f + k, g[k]);
    }
}

// UniMP combine in one pass per direction: beta = sigmoid(r . wa + o . wb + b), h = beta r + (1 - beta) o,
// out = dropout(relu(LayerNorm(h))).  wa = W_g[0] + W_g[2], wb = W_g[1] - W_g[2] of the reference's W_g [1, 3 d] applied to
// [r | o | r - o].  Warp per row, d <= 256 (one 8-chunk per lane).  The backward recomputes from r and o.
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) gated_res_fwd_kernel(GatedResArgs a) {
    const int lane = threadIdx.x & 31, nch = a.d >> 3, f = lane << 3;
    const bool active = lane < nch;
    const uint64_t sd = site_seed(a.seed, a.stream_id);
    const float inv_keep = a.p > 0.f ? keep_scale(a.p) : 1.f;
    float wa[8], wb[8], gam[8], bet[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        wa[k] = active ? a.wa[f + k] : 0.f; wb[k] = active ? a.wb[f + k] : 0.f;
        gam[k] = active ? a.gamma[f + k] : 0.f; bet[k] = active ? a.beta[f + k] : 0.f;
    }
    const float gb = a.gate_bias[0];
    for (long long row = blockIdx.x * kWarps + (threadIdx.x >> 5); row < a.n; row += (long long)gridDim.x * kWarps) {
        float rv[8], ov[8], h[8];
        float dot = 0.f;
        if (active) {
            Vec8<T>::load(static_cast<const T*>(a.r) + row * a.d + f, rv);
            Vec8<T>::load(static_cast<const T*>(a.o) + row * a.d + f, ov);
#pragma unroll
            for (int k = 0; k < 8; ++k) dot = fmaf(rv[k], wa[k], fmaf(ov[k], wb[k], dot));
        }
        const float beta_g = 1.f / (1.f + __expf(-(warp_sum(dot) + gb)));
        float sum = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) { h[k] = active ? beta_g * rv[k] + (1.f - beta_g) * ov[k] : 0.f; sum += h[k]; }
        const float mean = warp_sum(sum) / a.d;
        float var = 0.f;
        if (active)
#pragma unroll
            for (int k = 0; k < 8; ++k) { const float t = h[k] - mean; var = fmaf(t, t, var); }
        const float rstd = rsqrtf(warp_sum(var) / a.d + a.eps);
        if (active) {
            const uint32_t kb = a.p > 0.f ? keep_bits8(sd, (uint64_t)(row * a.d + f) >> 3, drop_threshold(a.p)) : 0xffu;
            float out[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float u = fmaxf((h[k] - mean) * rstd * gam[k] + bet[k], 0.f);
                out[k] = ((kb >> k) & 1u) ? u * inv_keep : 0.f;
            }
            Vec8<T>::store(static_cast<T*>(a.out) + row * a.d + f, out);
        }
        if (lane == 0) { a.stats[3 * row] = mean; a.stats[3 * row + 1] = rstd; a.stats[3 * row + 2] = beta_g; }
    }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) gated_res_bwd_kernel(GatedResArgs a) {
    extern __shared__ float smem[];                    // [4][d] + 1: dgamma, dbeta, dwa, dwb, dbias
    const int lane = threadIdx.x & 31, nch = a.d >> 3, f = lane << 3;
    const bool active = lane < nch;
    for (int i = threadIdx.x; i < 4 * a.d + 1; i += blockDim.x) smem[i] = 0.f;
    __syncthreads();
    const uint64_t sd = site_seed(a.seed, a.stream_id);
    const float inv_keep = a.p > 0.f ? keep_scale(a.p) : 1.f;
    float wa[8], wb[8], gam[8], bet[8], dgam[8], dbet[8], dwa[8], dwb[8];
    float dgb = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        wa[k] = active ? a.wa[f + k] : 0.f; wb[k] = active ? a.wb[f + k] : 0.f;
        gam[k] = active ? a.gamma[f + k] : 0.f; bet[k] = active ? a.beta[f + k] : 0.f;
        dgam[k] = 0.f; dbet[k] = 0.f; dwa[k] = 0.f; dwb[k] = 0.f;
    }
    for (long long row = blockIdx.x * kWarps + (threadIdx.x >> 5); row < a.n; row += (long long)gridDim.x * kWarps) {
        const float mean = a.stats[3 * row], rstd = a.stats[3 * row + 1], beta_g = a.stats[3 * row + 2];
        float rv[8], ov[8], zh[8], dzh[8];
        float s1 = 0.f, s2 = 0.f;
        if (active) {
            float go[8];
            Vec8<T>::load(static_cast<const T*>(a.r) + row * a.d + f, rv);
            Vec8<T>::load(static_cast<const T*>(a.o) + row * a.d + f, ov);
            Vec8<T>::load(static_cast<const T*>(a.dout) + row * a.d + f, go);
            const uint32_t kb = a.p > 0.f ? keep_bits8(sd, (uint64_t)(row * a.d + f) >> 3, drop_threshold(a.p)) : 0xffu;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float h = beta_g * rv[k] + (1.f - beta_g) * ov[k];
                zh[k] = (h - mean) * rstd;
                const float u = zh[k] * gam[k] + bet[k];
                const float gz = (u > 0.f && ((kb >> k) & 1u)) ? go[k] * inv_keep : 0.f;   // through dropout and ReLU
                dgam[k] = fmaf(gz, zh[k], dgam[k]);
                dbet[k] += gz;
                dzh[k] = gz * gam[k];
                s1 += dzh[k];
                s2 = fmaf(dzh[k], zh[k], s2);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) { rv[k] = 0.f; ov[k] = 0.f; zh[k] = 0.f; dzh[k] = 0.f; }
        }
        s1 = warp_sum(s1) / a.d;
        s2 = warp_sum(s2) / a.d;
        float dh[8], dbeta_part = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            dh[k] = rstd * (dzh[k] - s1 - zh[k] * s2);
            dbeta_part = fmaf(dh[k], rv[k] - ov[k], dbeta_part);
        }
        const float dlogit = warp_sum(dbeta_part) * beta_g * (1.f - beta_g);
        if (active) {
            float dr[8], dov[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                dr[k] = beta_g * dh[k] + dlogit * wa[k];
                dov[k] = (1.f - beta_g) * dh[k] + dlogit * wb[k];
                dwa[k] = fmaf(dlogit, rv[k], dwa[k]);
                dwb[k] = fmaf(dlogit, ov[k], dwb[k]);
            }
            Vec8<T>::store(static_cast<T*>(a.dr) + row * a.d + f, dr);
            Vec8<T>::store(static_cast<T*>(a.d_o) + row * a.d + f, dov);
        }
        if (lane == 0) dgb += dlogit;
    }
    if (active) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            atomicAdd(&smem[f + k], dgam[k]);
            atomicAdd(&smem[a.d + f + k], dbet[k]);
            atomicAdd(&smem[2 * a.d + f + k], dwa[k]);
            atomicAdd(&smem[3 * a.d + f + k], dwb[k]);
        }
    }
    if (lane == 0) atomicAdd(&smem[4 * a.d], dgb);
    __syncthreads();
    for (int i = threadIdx.x; i < 4 * a.d + 1; i += blockDim.x) a.part[(size_t)blockIdx.x * a.part_stride + i] = smem[i];
}

// Input stage of the models in one pass per direction: out = l2normalize(relu(dropout(LayerNorm(h)))) (dropout AFTER the norm,
// optional L2 normalisation).  Warp per row; the backward recomputes everything from h and the saved (mean, rstd, norm).
template <typename T, int CPL>
__global__ void __launch_bounds__(kWarps * 32) premp_fwd_kernel(PreMpArgs a) {
    const int lane = threadIdx.x & 31, nch = a.d >> 3;
    const uint64_t sd = site_seed(a.seed, a.stream_id);
    const float inv_keep = a.p > 0.f ? keep_scale(a.p) : 1.f;
    for (int row = blockIdx.x * kWarps + (threadIdx.x >> 5); row < a.n; row += gridDim.x * kWarps) {
        float z[CPL][8];
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            const int ch = lane + 32 * i;
            if (ch < nch) {
                Vec8<T>::load(static_cast<const T*>(a.h) + (size_t)row * a.d + (ch << 3), z[i]);
#pragma unroll
                for (int k = 0; k < 8; ++k) sum += z[i][k];
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) z[i][k] = 0.f;
            }
        }
        const float mean = warp_sum(sum) / a.d;
        float var = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i)
            if (lane + 32 * i < nch)
#pragma unroll
                for (int k = 0; k < 8; ++k) { const float t = z[i][k] - mean; var = fmaf(t, t, var); }
        const float rstd = rsqrtf(warp_sum(var) / a.d + a.eps);
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            const int ch = lane + 32 * i;
            if (ch < nch) {
                const int f = ch << 3;
                const uint32_t kb = a.p > 0.f ? keep_bits8(sd, ((uint64_t)row * a.d + f) >> 3, drop_threshold(a.p)) : 0xffu;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    float u = (z[i][k] - mean) * rstd * a.gamma[f + k] + a.beta[f + k];
                    u = ((kb >> k) & 1u) ? u * inv_keep : 0.f;
                    u = fmaxf(u, 0.f);
                    z[i][k] = u;
                    sq = fmaf(u, u, sq);
                }
            }
        }
        const float nrm = a.l2norm ? fmaxf(sqrtf(warp_sum(sq)), 1e-12f) : 1.f;
        const float inv = 1.f / nrm;
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            const int ch = lane + 32 * i;
            if (ch < nch) {
                float o[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = z[i][k] * inv;
                Vec8<T>::store(static_cast<T*>(a.out) + (size_t)row * a.d + (ch << 3), o);
            }
        }
        if (lane == 0 && a.stats) { a.stats[3 * (size_t)row] = mean; a.stats[3 * (size_t)row + 1] = rstd; a.stats[3 * (size_t)row + 2] = nrm; }
    }
}

template <typename T, int CPL>
__global__ void __launch_bounds__(kWarps * 32) premp_bwd_kernel(PreMpArgs a) {
    extern __shared__ float smem[];                    // [2][d] block accumulators: dgamma, dbeta
    const int lane = threadIdx.x & 31, nch = a.d >> 3;
    for (int i = threadIdx.x; i < 2 * a.d; i += blockDim.x) smem[i] = 0.f;
    __syncthreads();
    const uint64_t sd = site_seed(a.seed, a.stream_id);
    const float inv_keep = a.p > 0.f ? keep_scale(a.p) : 1.f;
    float dgam[CPL][8], dbet[CPL][8], gam[CPL][8];
#pragma unroll
    for (int i = 0; i < CPL; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            dgam[i][k] = 0.f; dbet[i][k] = 0.f;
            gam[i][k] = (lane + 32 * i) < nch ? a.gamma[((lane + 32 * i) << 3) + k] : 0.f;
        }
    for (int row = blockIdx.x * kWarps + (threadIdx.x >> 5); row < a.n; row += gridDim.x * kWarps) {
        const float mean = a.stats[3 * (size_t)row], rstd = a.stats[3 * (size_t)row + 1], nrm = a.stats[3 * (size_t)row + 2];
        const float inv = nrm > 1e-12f ? 1.f / nrm : 0.f;
        float zh[CPL][8], go[CPL][8], o[CPL][8], live[CPL][8];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            const int ch = lane + 32 * i;
            if (ch < nch) {
                const int f = ch << 3;
                float hv[8];
                Vec8<T>::load(static_cast<const T*>(a.h) + (size_t)row * a.d + f, hv);
                Vec8<T>::load(static_cast<const T*>(a.dout) + (size_t)row * a.d + f, go[i]);
                const uint32_t kb = a.p > 0.f ? keep_bits8(sd, ((uint64_t)row * a.d + f) >> 3, drop_threshold(a.p)) : 0xffu;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    zh[i][k] = (hv[k] - mean) * rstd;
                    const float keep = ((kb >> k) & 1u) ? inv_keep : 0.f;
                    const float u = (zh[i][k] * gam[i][k] + a.beta[f + k]) * keep;
                    live[i][k] = u > 0.f ? keep : 0.f;                            // ReLU gate times the dropout scale
                    o[i][k] = fmaxf(u, 0.f) * inv;
                    dot = fmaf(o[i][k], go[i][k], dot);
                }
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) { zh[i][k] = 0.f; go[i][k] = 0.f; o[i][k] = 0.f; live[i][k] = 0.f; }
            }
        }
        if (a.l2norm) dot = warp_sum(dot);
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i)
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float gr = a.l2norm ? (go[i][k] - o[i][k] * dot) * inv : go[i][k];
                const float gz = gr * live[i][k];
                dgam[i][k] = fmaf(gz, zh[i][k], dgam[i][k]);
                dbet[i][k] += gz;
                const float dzh = gz * gam[i][k];
                go[i][k] = dzh;
                s1 += dzh;
                s2 = fmaf(dzh, zh[i][k], s2);
            }
        s1 = warp_sum(s1) / a.d;
        s2 = warp_sum(s2) / a.d;
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            const int ch = lane + 32 * i;
            if (ch < nch) {
                float dh[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) dh[k] = rstd * (go[i][k] - s1 - zh[i][k] * s2);
                Vec8<T>::store(static_cast<T*>(a.dh) + (size_t)row * a.d + (ch << 3), dh);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
        const int ch = lane + 32 * i;
        if (ch < nch) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                atomicAdd(&smem[(ch << 3) + k], dgam[i][k]);
                atomicAdd(&smem[a.d + (ch << 3) + k], dbet[i][k]);
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * a.d; i += blockDim.x) a.part[(size_t)blockIdx.x * 2 * a.d + i] = smem[i];
}

// out = dropout(act(in + bias)) on [n, d] (d % 8 == 0), grid-stride over 8-chunks
template <typename T>
__global__ void bias_act_dropout_kernel(const T* in, const float* bias, T* out, long long n_chunks, int d, int act, float p,
                                        const long long* seed, long long stream_id) {
    const uint64_t sd = site_seed(seed, stream_id);
    const float inv = p > 0.f ? keep_scale(p) : 1.f;
    for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x; c < n_chunks; c += (long long)gridDim.x * blockDim.x) {
        long long e = c << 3;
        int f = (int)(e % d);
        float v[8];
        Vec8<T>::load(in + e, v);
        const uint32_t kb = p > 0.f ? keep_bits8(sd, (uint64_t)c, drop_threshold(p)) : 0xffu;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float t = v[k] + (bias ? bias[f + k] : 0.f);
            if (act == 1) t = fmaxf(t, 0.f);
            else if (act == 2) t = gelu_f(t);
            t = ((kb >> k) & 1u) ? t * inv : 0.f;
            v[k] = t;
        }
        Vec8<T>::store(out + e, v);
    }
}

// relu (act 1): `in` is the forward OUTPUT; dz = dout * (out > 0) / (1 - p)  (dropped and inactive units are both zero there)
// gelu (act 2): `in` is the pre-activation without bias; dz = dout * gelu'(in + bias)
// none (act 0): dz = dout * dropmask
template <typename T>
__global__ void bias_act_dropout_bwd_kernel(const T* dout, const T* in, const float* bias, T* dz, long long n_rows, int d, int act,
                                            float p, const long long* seed, long long stream_id, float* dbias_part) {
    extern __shared__ float s_db[];                    // [d]
    for (int i = threadIdx.x; i < d; i += blockDim.x) s_db[i] = 0.f;
    __syncthreads();
    const uint64_t sd = site_seed(seed, stream_id);
    const float inv = p > 0.f ? keep_scale(p) : 1.f;
    const int nch = d >> 3;
    // thread t handles chunk column (t % nch) of rows (t / nch) + k * rows_per_pass: a thread keeps one column group
    const int tpb = blockDim.x;
    const int colc = threadIdx.x % nch;
    const int rsub = threadIdx.x / nch;
    const int rows_per_block_pass = tpb / nch;
    float db[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (rsub < rows_per_block_pass) {
        for (long long row = (long long)blockIdx.x * rows_per_block_pass + rsub; row < n_rows; row += (long long)gridDim.x * rows_per_block_pass) {
            long long e = row * d + (colc << 3);
            float g[8], v[8], o[8];
            Vec8<T>::load(dout + e, g);
            if (act != 0) Vec8<T>::load(in + e, v);
            const uint32_t kb = (act == 0 && p > 0.f) ? keep_bits8(sd, (uint64_t)e >> 3, drop_threshold(p)) : 0xffu;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float t;
                if (act == 1) t = v[k] > 0.f ? g[k] * inv : 0.f;
                else if (act == 2) t = g[k] * gelu_grad(v[k] + (bias ? bias[(colc << 3) + k] : 0.f));
                else t = ((kb >> k) & 1u) ? g[k] * inv : 0.f;
                o[k] = t;
                db[k] += t;
            }
            Vec8<T>::store(dz + e, o);
        }
        if (dbias_part)
#pragma unroll
            for (int k = 0; k < 8; ++k) atomicAdd(&s_db[(colc << 3) + k], db[k]);
    }
    __syncthreads();
    if (dbias_part)
        for (int i = threadIdx.x; i < d; i += blockDim.x) dbias_part[(size_t)blockIdx.x * d + i] = s_db[i];
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) ce_kernel(const T* logits, const long long* labels, const bool* mask, int n, int c,
                                                         float inv_denom, float* loss, T* dlogits) {
    const int row = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (row >= n) return;
    const int lane = threadIdx.x & 31;
    const T* lg = logits + (size_t)row * c;
    T* dl = dlogits ? dlogits + (size_t)row * c : nullptr;
    if (!mask[row]) {
        if (dl) for (int j = lane; j < c; j += 32) dl[j] = from_float<T>(0.f);
        return;
    }
    float mx = -INFINITY;
    for (int j = lane; j < c; j += 32) mx = fmaxf(mx, to_float(lg[j]));
    mx = warp_max(mx);
    float se = 0.f;
    for (int j = lane; j < c; j += 32) se += __expf(to_float(lg[j]) - mx);
    se = warp_sum(se);
    const int y = (int)labels[row];
    const float lse = mx + __logf(se);
    if (lane == 0) atomicAdd(loss, (lse - to_float(lg[y])) * inv_denom);
    if (dl)
        for (int j = lane; j < c; j += 32) {
            float pj = __expf(to_float(lg[j]) - lse);
            dl[j] = from_float<T>((pj - (j == y ? 1.f : 0.f)) * inv_denom);
        }
}

__global__ void adamw_kernel(AdamWArgs a) {
    const float lr = a.hyper[0], b1 = a.hyper[1], b2 = a.hyper[2], eps = a.hyper[3], wd = a.hyper[4];
    const float bc1 = a.hyper[5], bc2 = a.hyper[6];
    // hyper[7] = max gradient norm (<= 0: no clipping), hyper[8] = sum of squared gradients (written by sq_norm)
    float gs = 1.f;
    if (a.hyper[7] > 0.f) gs = fminf(1.f, a.hyper[7] / (sqrtf(a.hyper[8]) + 1e-6f));
    __nv_bfloat16* shadow = static_cast<__nv_bfloat16*>(a.p_bf16);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < a.n; i += (long long)gridDim.x * blockDim.x) {
        float g = a.g[i] * gs, p = a.p[i];
        float m = b1 * a.m[i] + (1.f - b1) * g;
        float v = b2 * a.v[i] + (1.f - b2) * g * g;
        a.m[i] = m;
        a.v[i] = v;
        float decay = a.decay_mask ? a.decay_mask[i] : 1.f;
        p = p * (1.f - lr * wd * decay) - lr * (m / bc1) / (sqrtf(v / bc2) + eps);
        a.p[i] = p;
        if (shadow) shadow[i] = __float2bfloat16(p);
    }
}

__global__ void sq_norm_kernel(const float* g, long long n, float* out) {
    float s = 0.f;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) s = fmaf(g[i], g[i], s);
    s = warp_sum(s);
    __shared__ float ws[32];
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? ws[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) atomicAdd(out, t);
    }
}

__global__ void cast_kernel(const float* in, __nv_bfloat16* out, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16(in[i]);
}

int grid_for(long long work_items, int per_block) {
    long long b = (work_items + per_block - 1) / per_block;
    long long cap = 148LL * 16;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

// Column-wise concatenation with conversion: packed[r, off_i : off_i + w_i] = seg_i[r, :] (dir 0) or the reverse (dir 1).
// One thread moves one 8-element chunk; every width and row stride is a multiple of 8 elements.
template <typename TP>
__global__ void pack_cols_kernel(PackColsArgs a) {
    const int cpr = a.width >> 3;
    const long long total = a.n_rows * cpr;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / cpr;
        int col = (int)(i - row * cpr) << 3;
        TP* pk = static_cast<TP*>(a.packed) + row * a.ld_packed + col;
        int sgi = 0;
        while (sgi + 1 < a.n_seg && col >= a.seg[sgi].width) { col -= a.seg[sgi].width; ++sgi; }
        const PackColSeg& sg = a.seg[sgi];
        float v[8];
        if (a.dir == 0) {
            if (sg.dtype == DT_BF16) Vec8<__nv_bfloat16>::load(static_cast<const __nv_bfloat16*>(sg.p) + row * sg.ld + col, v);
            else Vec8<float>::load(static_cast<const float*>(sg.p) + row * sg.ld + col, v);
            Vec8<TP>::store(pk, v);
        } else {
            Vec8<TP>::load(pk, v);
            if (sg.dtype == DT_BF16) Vec8<__nv_bfloat16>::store(static_cast<__nv_bfloat16*>(sg.p) + row * sg.ld + col, v);
            else Vec8<float>::store(static_cast<float*>(sg.p) + row * sg.ld + col, v);
        }
    }
}

}  // namespace

void pack_cols(const PackColsArgs& a, cudaStream_t s) {
    const long long chunks = a.n_rows * (a.width >> 3);
    if (chunks <= 0) return;
    const int blocks = grid_for(chunks, 256);
    if (a.packed_dtype == DT_BF16) pack_cols_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(a);
    else pack_cols_kernel<float><<<blocks, 256, 0, s>>>(a);
}

int premp_blocks(int n) {
    int b = grid_for(n, kWarps * 8);
    return b > 148 * 8 ? 148 * 8 : b;
}

void premp(const PreMpArgs& a, bool backward, cudaStream_t s) {
    if (a.n <= 0) return;
    const int blocks = backward ? a.n_blocks : premp_blocks(a.n) * 2;
    const size_t sm = backward ? 2 * (size_t)a.d * sizeof(float) : 0;
#define GT_PREMP(T, CPL)                                                                          \
    do {                                                                                          \
        if (backward) premp_bwd_kernel<T, CPL><<<blocks, kWarps * 32, sm, s>>>(a);                \
        else premp_fwd_kernel<T, CPL><<<blocks, kWarps * 32, 0, s>>>(a);                          \
    } while (0)
    if (a.dtype == DT_BF16) { if (a.d <= 256) GT_PREMP(__nv_bfloat16, 1); else if (a.d <= 512) GT_PREMP(__nv_bfloat16, 2); else GT_PREMP(__nv_bfloat16, 4); }
    else                    { if (a.d <= 256) GT_PREMP(float, 1); else if (a.d <= 512) GT_PREMP(float, 2); else GT_PREMP(float, 4); }
#undef GT_PREMP
}

void embed_add(int dtype, const void* x, const float* tab_a, const long long* idx_a, long long pad_a, const float* tab_b,
               const long long* idx_b, long long pad_b, void* out, long long n, int d, cudaStream_t s) {
    if (n <= 0) return;
    const int blocks = grid_for(n * (d / 8), 256);
    if (dtype == DT_BF16)
        embed_add_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), tab_a, idx_a, pad_a, tab_b, idx_b, pad_b,
                                                               static_cast<__nv_bfloat16*>(out), n, d);
    else
        embed_add_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(x), tab_a, idx_a, pad_a, tab_b, idx_b, pad_b,
                                                       static_cast<float*>(out), n, d);
}

void embed_add_bwd(int dtype, const void* dout, const long long* idx, long long pad, float* dtab, long long n, int d, cudaStream_t s) {
    if (n <= 0) return;
    const int blocks = grid_for(n * (d / 8), 256);
    if (dtype == DT_BF16) embed_add_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dout), idx, pad, dtab, n, d);
    else embed_add_bwd_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(dout), idx, pad, dtab, n, d);
}

void gated_residual(const GatedResArgs& a, bool backward, cudaStream_t s) {
    if (a.n <= 0) return;
    if (backward) {
        const size_t sm = (4 * (size_t)a.d + 1) * sizeof(float);
        if (a.dtype == DT_BF16) gated_res_bwd_kernel<__nv_bfloat16><<<a.n_blocks, kWarps * 32, sm, s>>>(a);
        else gated_res_bwd_kernel<float><<<a.n_blocks, kWarps * 32, sm, s>>>(a);
    } else {
        const int blocks = premp_blocks((int)a.n) * 2;
        if (a.dtype == DT_BF16) gated_res_fwd_kernel<__nv_bfloat16><<<blocks, kWarps * 32, 0, s>>>(a);
        else gated_res_fwd_kernel<float><<<blocks, kWarps * 32, 0, s>>>(a);
    }
}

void layer_norm_fwd(const LayerNormArgs& a, cudaStream_t s) {
    if (a.n <= 0) return;
    int blocks = (a.n + kWarps - 1) / kWarps;
    if (blocks > 148 * 16) blocks = 148 * 16;
    static const bool use_ring = [] { const char* e = getenv("GT_LN_RING"); return !(e && e[0] == '0'); }();
    const bool aligned = (reinterpret_cast<uintptr_t>(a.y) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(a.acc) & 15) == 0;
    if (use_ring && a.dtype == DT_BF16 && a.d <= 256 && aligned) {
        // operands through the cp.async ring; 5 blocks of 4 warps per SM fit next to their rings
        int rb = (a.n + kWarps - 1) / kWarps;
        if (rb > 148 * 5) rb = 148 * 5;
        if (a.acc) {
            static bool once = (cudaFuncSetAttribute(ln_fwd_ring_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LnRing<true, false>::kBytes), true);
            (void)once;
            ln_fwd_ring_kernel<true><<<rb, kWarps * 32, LnRing<true, false>::kBytes, s>>>(a);
        } else {
            static bool once = (cudaFuncSetAttribute(ln_fwd_ring_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LnRing<false, false>::kBytes), true);
            (void)once;
            ln_fwd_ring_kernel<false><<<rb, kWarps * 32, LnRing<false, false>::kBytes, s>>>(a);
        }
        return;
    }
    // chunks of 8 features per lane: the kernel is instantiated for 1, 2 or 4 so narrow rows do not pay for wide registers
#define GT_LN_FWD(T)                                                                   \
    do {                                                                               \
        if (a.d <= 256) ln_fwd_kernel<T, 1><<<blocks, kWarps * 32, 0, s>>>(a);         \
        else if (a.d <= 512) ln_fwd_kernel<T, 2><<<blocks, kWarps * 32, 0, s>>>(a);    \
        else ln_fwd_kernel<T, 4><<<blocks, kWarps * 32, 0, s>>>(a);                    \
    } while (0)
    if (a.dtype == DT_BF16) GT_LN_FWD(__nv_bfloat16);
    else GT_LN_FWD(float);
#undef GT_LN_FWD
}

int layer_norm_bwd_blocks(int n) {
    int b = grid_for(n, kWarps * 8);
    return b > 148 * 12 ? 148 * 12 : b;                // enough resident warps to hide the row latency
}

void layer_norm_bwd(const LayerNormBwdArgs& a, cudaStream_t s) {
    if (a.n <= 0) return;
    const size_t sm = 3 * (size_t)a.d * sizeof(float);
    static const bool use_ring = [] { const char* e = getenv("GT_LN_RING"); return !(e && e[0] == '0'); }();
    const bool aligned = (reinterpret_cast<uintptr_t>(a.y) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(a.acc) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.dout) & 15) == 0;
    if (use_ring && a.dtype == DT_BF16 && a.d <= 256 && aligned) {
        const size_t head = (sm + 15) & ~size_t(15);
        if (a.acc) {
            static bool once = (cudaFuncSetAttribute(ln_bwd_ring_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(LnRing<true, true>::kBytes + 4096)), true);
            (void)once;
            ln_bwd_ring_kernel<true><<<a.n_blocks, kWarps * 32, head + LnRing<true, true>::kBytes, s>>>(a);
        } else {
            static bool once = (cudaFuncSetAttribute(ln_bwd_ring_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(LnRing<false, true>::kBytes + 4096)), true);
            (void)once;
            ln_bwd_ring_kernel<false><<<a.n_blocks, kWarps * 32, head + LnRing<false, true>::kBytes, s>>>(a);
        }
        return;
    }
#define GT_LN_BWD(T)                                                                          \
    do {                                                                                      \
        if (a.d <= 256) ln_bwd_kernel<T, 1><<<a.n_blocks, kWarps * 32, sm, s>>>(a);           \
        else if (a.d <= 512) ln_bwd_kernel<T, 2><<<a.n_blocks, kWarps * 32, sm, s>>>(a);      \
        else ln_bwd_kernel<T, 4><<<a.n_blocks, kWarps * 32, sm, s>>>(a);                      \
    } while (0)
    if (a.dtype == DT_BF16) GT_LN_BWD(__nv_bfloat16);
    else GT_LN_BWD(float);
#undef GT_LN_BWD
}

void bias_act_dropout(int dtype, const void* in, const float* bias, void* out, long long n, int d, int act, float p,
                      const long long* seed, long long stream_id, cudaStream_t s) {
    const long long chunks = n * d / 8;
    if (chunks <= 0) return;
    const int blocks = grid_for(chunks, 256);
    if (dtype == DT_BF16)
        bias_act_dropout_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(in), bias,
                                                                      static_cast<__nv_bfloat16*>(out), chunks, d, act, p, seed, stream_id);
    else
        bias_act_dropout_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(in), bias, static_cast<float*>(out), chunks, d,
                                                              act, p, seed, stream_id);
}

int colsum_blocks(long long n) {
    int b = grid_for(n, 64);
    return b > 148 * 4 ? 148 * 4 : b;
}

void bias_act_dropout_bwd(int dtype, const void* dout, const void* in, const float* bias, void* dz, long long n, int d, int act,
                          float p, const long long* seed, long long stream_id, float* dbias_part, int n_blocks, cudaStream_t s) {
    if (n <= 0) return;
    const int nch = d / 8;
    int threads = 256;
    if (nch > threads) threads = ((nch + 31) / 32) * 32;
    const size_t sm = (size_t)d * sizeof(float);
    if (dtype == DT_BF16)
        bias_act_dropout_bwd_kernel<__nv_bfloat16><<<n_blocks, threads, sm, s>>>(
            static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(in), bias, static_cast<__nv_bfloat16*>(dz), n, d,
            act, p, seed, stream_id, dbias_part);
    else
        bias_act_dropout_bwd_kernel<float><<<n_blocks, threads, sm, s>>>(static_cast<const float*>(dout), static_cast<const float*>(in),
                                                                        bias, static_cast<float*>(dz), n, d, act, p, seed, stream_id,
                                                                        dbias_part);
}

void cross_entropy_fwd_bwd(int dtype, const void* logits, const long long* labels, const bool* mask, int n, int c, float inv_denom,
                           float* loss, void* dlogits, cudaStream_t s) {
    if (n <= 0) return;
    const int blocks = (n + kWarps - 1) / kWarps;
    if (dtype == DT_BF16)
        ce_kernel<__nv_bfloat16><<<blocks, kWarps * 32, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), labels, mask, n, c, inv_denom,
                                                                loss, static_cast<__nv_bfloat16*>(dlogits));
    else
        ce_kernel<float><<<blocks, kWarps * 32, 0, s>>>(static_cast<const float*>(logits), labels, mask, n, c, inv_denom, loss,
                                                        static_cast<float*>(dlogits));
}

void adamw_step(const AdamWArgs& a, cudaStream_t s) {
    if (a.n <= 0) return;
    adamw_kernel<<<grid_for(a.n, 256), 256, 0, s>>>(a);
}

void sq_norm(const float* g, long long n, float* out, cudaStream_t s) {
    if (n <= 0) return;
    sq_norm_kernel<<<grid_for(n, 1024), 256, 0, s>>>(g, n, out);
}

void cast_f32_to_bf16(const float* in, void* out, long long n, cudaStream_t s) {
    if (n <= 0) return;
    cast_kernel<<<grid_for(n, 1024), 256, 0, s>>>(in, static_cast<__nv_bfloat16*>(out), n);
}

}  // namespace gt
