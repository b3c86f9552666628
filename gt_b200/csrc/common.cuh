// Shared device helpers of the gt_b200 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define GT_FULL_MASK 0xffffffffu

namespace gt {

// ---- 8-element vector loads / stores -----------------------------------------------------------------------
// Every row kernel moves features in chunks of 8 elements: one 16-byte transaction for bf16, two for fp32.
template <typename T> struct Vec8;

template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
        uint4 u = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 x = __bfloat1622float2(h[i]);
            f[2 * i] = x.x;
            f[2 * i + 1] = x.y;
        }
    }
    // read-only / streaming variant for gathers that are not reused by this thread
    static __device__ __forceinline__ void load_nc(const __nv_bfloat16* p, float (&f)[8]) {
        uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 x = __bfloat1622float2(h[i]);
            f[2 * i] = x.x;
            f[2 * i + 1] = x.y;
        }
    }
    // raw 16-byte register form of a chunk: gathers are held packed and converted on use (4 registers instead of 8)
    using Raw = uint4;
    static __device__ __forceinline__ Raw load_raw(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
    static __device__ __forceinline__ Raw zero_raw() { return make_uint4(0u, 0u, 0u, 0u); }
    static __device__ __forceinline__ void unpack(const Raw& u, float (&f)[8]) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 x = __bfloat1622float2(h[i]);
            f[2 * i] = x.x;
            f[2 * i + 1] = x.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
        uint4 u;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = u;
    }
};

template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
        float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    static __device__ __forceinline__ void load_nc(const float* p, float (&f)[8]) {
        float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p + 4));
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    struct Raw { float4 a, b; };
    static __device__ __forceinline__ Raw load_raw(const float* p) {
        Raw r;
        r.a = __ldg(reinterpret_cast<const float4*>(p));
        r.b = __ldg(reinterpret_cast<const float4*>(p + 4));
        return r;
    }
    static __device__ __forceinline__ Raw zero_raw() {
        Raw r;
        r.a = make_float4(0.f, 0.f, 0.f, 0.f);
        r.b = r.a;
        return r;
    }
    static __device__ __forceinline__ void unpack(const Raw& r, float (&f)[8]) {
        f[0] = r.a.x; f[1] = r.a.y; f[2] = r.a.z; f[3] = r.a.w; f[4] = r.b.x; f[5] = r.b.y; f[6] = r.b.z; f[7] = r.b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
};

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(GT_FULL_MASK, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(GT_FULL_MASK, v, o));
    return v;
}

// Counter-based uniform random number in [0, 1) (stateless: seed, element index, stream id).  Used by the dropout
// epilogues so that forward and backward regenerate the same mask without storing it.
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t idx) {
    uint32_t lo = (uint32_t)idx, hi = (uint32_t)(idx >> 32);
    uint32_t s0 = (uint32_t)seed, s1 = (uint32_t)(seed >> 32);
    uint32_t x = mix32(lo ^ s0) + 0x9e3779b9u * (hi + 1u);
    x = mix32(x ^ s1);
    return (float)(x >> 8) * (1.0f / 16777216.0f);
}

// Dropout masks are drawn per CHUNK of 8 consecutive elements (flattened index i: chunk i >> 3, byte i & 7): three hash rounds
// give 8 random bytes, element k is kept iff byte k >= thr.  The drop probability is therefore quantised to thr / 256 and
// the kept values are scaled by 256 / (256 - thr), so the expectation is exact.  One hash chain per 8 elements instead of
// one per element: the per-element generator made the row kernels instruction-bound.  Every kernel that applies or
// regenerates a mask uses these three functions, so forward and backward always agree.
__device__ __forceinline__ uint32_t drop_threshold(float p) {
    return p > 0.f ? (uint32_t)fminf(p * 256.f + 0.5f, 255.f) : 0u;
}
__device__ __forceinline__ float keep_scale(float p) { return 256.f / (256.f - (float)drop_threshold(p)); }
__device__ __forceinline__ uint32_t keep_bits8(uint64_t seed, uint64_t chunk, uint32_t thr) {
    const uint32_t lo = (uint32_t)chunk, hi = (uint32_t)(chunk >> 32);
    uint32_t x = mix32(lo ^ (uint32_t)seed) + 0x9e3779b9u * (hi + 1u);
    x = mix32(x ^ (uint32_t)(seed >> 32));
    const uint32_t y = mix32(x + 0x68bc21ebu);
    const uint32_t t4 = thr * 0x01010101u;
    const uint32_t a = __vcmpgeu4(x, t4), b = __vcmpgeu4(y, t4);                 // 0xff in every byte that is kept
    return (a & 1u) | ((a >> 7) & 2u) | ((a >> 14) & 4u) | ((a >> 21) & 8u) |
           ((b & 1u) << 4) | ((b >> 3) & 32u) | ((b >> 10) & 64u) | ((b >> 17) & 128u);
}
// mask bit of ONE element (slow path for unaligned chunks)
__device__ __forceinline__ bool keep_element(uint64_t seed, uint64_t idx, uint32_t thr) {
    return (keep_bits8(seed, idx >> 3, thr) >> (idx & 7)) & 1u;
}

}  // namespace gt
