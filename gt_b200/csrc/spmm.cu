// Sparse aggregation out = A @ x on a CSR with fp32 values (the GCN branch and its transpose), and the deterministic
// segmented row sum used by the sparsity-aware reduce-scatter.  One warp per output row; feature rows are read in
// 16-byte chunks, LPR = min(32, pow2ceil(d/8)) lanes per row, several edges per warp iteration when d < 256, fp32
// accumulation.  Bandwidth-bound gather like the attention kernels (replaces cuSPARSE CSR SpMM of the reference,
// gt3d/gt3d/dist/layers.py:53-64, and the ones-valued SpMM of sparse_comm.py:190-202).
#include <stdio.h>

#include "common.cuh"
#include "kernels.h"
#include "noalloc.h"

namespace gt {
namespace {

constexpr int kWarps = 4;

template <typename T, int CPL>
__global__ void __launch_bounds__(kWarps * 32) spmm_kernel(SpmmArgs a, const int* perm_as_idx) {
    const int wid = blockIdx.x * kWarps + (threadIdx.x >> 5);
    int row, beg, end, slot = -1;
    if (a.use_plan) {
        if (wid >= a.plan.n_seg) return;
        row = a.plan.seg_row[wid]; beg = a.plan.seg_beg[wid]; end = a.plan.seg_end[wid]; slot = a.plan.seg_slot[wid];
    } else {
        if (wid >= a.n_out) return;
        row = wid; beg = a.ptr[row]; end = a.ptr[row + 1];
    }
    const int lane = threadIdx.x & 31;
    const int nch = a.d >> 3;
    int lpr = 1;
    while (lpr < nch && lpr < 32) lpr <<= 1;
    const int epw = 32 / lpr, sub = lane / lpr, ll = lane - sub * lpr;
    const T* x = static_cast<const T*>(a.x);
    const size_t ldx = a.ldx ? (size_t)a.ldx : (size_t)a.d, ldo = a.ldo ? (size_t)a.ldo : (size_t)a.d;
    float acc[CPL][8];
    bool act[CPL];
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
        act[i] = (ll + 32 * i) < nch;
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;
    }
    for (int base = beg; base < end; base += 2 * epw) {
        int j[2]; float w[2];
        float xf[2][CPL][8];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            int e = base + u * epw + sub;
            bool ok = e < end;
            j[u] = ok ? a.idx[e] : -1;
            w[u] = ok ? (a.w ? a.w[e] : 1.f) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                if (j[u] >= 0 && act[i]) Vec8<T>::load_nc(x + (size_t)j[u] * ldx + ((ll + 32 * i) << 3), xf[u][i]);
                else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) xf[u][i][k] = 0.f;
                }
            }
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int i = 0; i < CPL; ++i)
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[i][k] = fmaf(w[u], xf[u][i][k], acc[i][k]);
    }
    for (int off = lpr; off < 32; off <<= 1)
#pragma unroll
        for (int i = 0; i < CPL; ++i)
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[i][k] += __shfl_xor_sync(GT_FULL_MASK, acc[i][k], off);
    if (sub != 0) return;
    if (slot >= 0) {
#pragma unroll
        for (int i = 0; i < CPL; ++i)
            if (act[i]) Vec8<float>::store(a.scratch + (size_t)slot * a.d + ((ll + 32 * i) << 3), acc[i]);
        return;
    }
    T* out;
    if (a.push_n > 0) {          // reduce-scatter fused into the store: the row goes into the slot its owner keeps for this rank
        const int owner = row / a.push_rows;
        out = static_cast<T*>(a.push_slot[owner]) + (size_t)(row - owner * a.push_rows) * ldo;
    } else {
        out = static_cast<T*>(a.out) + (size_t)row * ldo;
    }
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
        if (!act[i]) continue;
        T* dst = out + ((ll + 32 * i) << 3);
        if (a.accumulate) {
            float old[8];
            Vec8<T>::load(dst, old);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[i][k] += old[k];
        }
        Vec8<T>::store(dst, acc[i]);
    }
}

// out[row] (+)= sum of the row's slots
template <typename T>
__global__ void spmm_combine_kernel(SpmmArgs a) {
    const int r = blockIdx.x;
    const int row = a.plan.split_rows[r];
    const int s0 = a.plan.split_ptr[r], s1 = a.plan.split_ptr[r + 1];
    const size_t ldo = a.ldo ? (size_t)a.ldo : (size_t)a.d;
    T* out;
    if (a.push_n > 0) {
        const int owner = row / a.push_rows;
        out = static_cast<T*>(a.push_slot[owner]) + (size_t)(row - owner * a.push_rows) * ldo;
    } else {
        out = static_cast<T*>(a.out) + (size_t)row * ldo;
    }
    for (int f = threadIdx.x; f < a.d; f += blockDim.x) {
        float v = a.accumulate ? to_float(out[f]) : 0.f;
        for (int s = s0; s < s1; ++s) v += a.scratch[(size_t)s * a.d + f];
        out[f] = from_float<T>(v);
    }
}

template <typename T>
void launch(const SpmmArgs& a, cudaStream_t s) {
    const int work = a.use_plan ? a.plan.n_seg : a.n_out;
    const int blocks = (work + kWarps - 1) / kWarps;
    const int nch = a.d / 8;
    if (nch <= 32) spmm_kernel<T, 1><<<blocks, kWarps * 32, 0, s>>>(a, nullptr);
    else if (nch <= 64) spmm_kernel<T, 2><<<blocks, kWarps * 32, 0, s>>>(a, nullptr);
    else spmm_kernel<T, 4><<<blocks, kWarps * 32, 0, s>>>(a, nullptr);
    if (a.use_plan && a.plan.n_split > 0) spmm_combine_kernel<T><<<a.plan.n_split, 256, 0, s>>>(a);
}

}  // namespace

void spmm(const SpmmArgs& a, cudaStream_t s) {
    if (a.n_out <= 0) return;
    if (a.dtype == DT_BF16) launch<__nv_bfloat16>(a, s);
    else launch<float>(a, s);
}

void segment_sum_rows(int dtype, const void* rows, const int* perm, const int* ptr, void* out, int n_out, int width, cudaStream_t s) {
    SpmmArgs a{};
    a.dtype = dtype; a.ptr = ptr; a.idx = perm; a.w = nullptr; a.x = rows; a.out = out; a.n_out = n_out; a.d = width; a.accumulate = 0; a.use_plan = 0;
    spmm(a, s);
}

}  // namespace gt

// ---- allocation-free entry point (see noalloc.h) -------------------------------------------------------------------------
// The scratch of the split-row merge as a file-scope device array.  In host code the name `gt_noalloc_scratch` is only a
// handle for the runtime, not a device address: the address is obtained per device with cudaGetSymbolAddress below.
static __device__ __align__(256) float gt_noalloc_scratch[GT_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {};
thread_local char g_noalloc_err[256] = "";

int noalloc_fail(int code, const char* msg, const char* detail = "") {
    snprintf(g_noalloc_err, sizeof(g_noalloc_err), "%s%s", msg, detail);
    return code;
}
}  // namespace

extern "C" const char* gt_noalloc_last_error(void) { return g_noalloc_err; }

extern "C" size_t gt_noalloc_scratch_floats(void) { return (size_t)GT_NOALLOC_SCRATCH_FLOATS; }

extern "C" int gt_spmm_csr_noalloc(int dtype, const int* ptr, const int* idx, const float* w, const void* x, void* out, int n_out, int d,
                                   const int* seg_row, const int* seg_beg, const int* seg_end, const int* seg_slot, int n_seg,
                                   const int* split_rows, const int* split_ptr, int n_split, int n_slots, void* stream) {
    g_noalloc_err[0] = 0;
    if (dtype != gt::DT_F32 && dtype != gt::DT_BF16) return noalloc_fail(GT_NOALLOC_ERR_ARGUMENT, "dtype must be 0 (float32) or 1 (bfloat16)");
    if (n_out < 0 || n_seg < 0 || n_split < 0 || n_slots < 0 || d <= 0 || (d % 8) || d > 1024)
        return noalloc_fail(GT_NOALLOC_ERR_ARGUMENT, "need n_out, n_seg, n_split, n_slots >= 0 and d a multiple of 8 in [8, 1024]");
    if (!ptr || !idx || !x || !out || !seg_row || !seg_beg || !seg_end || !seg_slot || (n_split > 0 && (!split_rows || !split_ptr)))
        return noalloc_fail(GT_NOALLOC_ERR_ARGUMENT, "null pointer argument");
    if ((size_t)n_slots * (size_t)d > (size_t)GT_NOALLOC_SCRATCH_FLOATS) {
        char detail[96];
        snprintf(detail, sizeof(detail), " (requested %d slots x %d floats, capacity %u floats)", n_slots, d, GT_NOALLOC_SCRATCH_FLOATS);
        return noalloc_fail(GT_NOALLOC_ERR_CAPACITY, "split-row scratch exceeds the built-in array", detail);
    }
    if (n_out == 0) return GT_NOALLOC_OK;
    if (n_seg == 0) {            // no entries at all: the product is zero (a fill of the caller's buffer, nothing is allocated)
        cudaError_t ez = cudaMemsetAsync(out, 0, (size_t)n_out * d * (dtype == gt::DT_BF16 ? 2 : 4), static_cast<cudaStream_t>(stream));
        return ez == cudaSuccess ? GT_NOALLOC_OK : noalloc_fail(GT_NOALLOC_ERR_CUDA, "cudaMemsetAsync failed: ", cudaGetErrorString(ez));
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return noalloc_fail(GT_NOALLOC_ERR_CUDA, "cudaGetDevice failed: ", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return noalloc_fail(GT_NOALLOC_ERR_ARGUMENT, "device index out of range");
    if (g_noalloc_ptr[dev] == nullptr) {
        // one-time set-up for this device (the device is current): translate the symbol into its device address
        float* p = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), gt_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr)
            return noalloc_fail(GT_NOALLOC_ERR_CUDA, "cudaGetSymbolAddress(gt_noalloc_scratch) failed: ", cudaGetErrorString(e));
        g_noalloc_ptr[dev] = p;
    }
    gt::SpmmArgs a{};
    a.dtype = dtype; a.ptr = ptr; a.idx = idx; a.w = w; a.x = x; a.out = out; a.n_out = n_out; a.d = d; a.accumulate = 0;
    a.use_plan = 1;
    a.plan.seg_row = seg_row; a.plan.seg_beg = seg_beg; a.plan.seg_end = seg_end; a.plan.seg_slot = seg_slot; a.plan.n_seg = n_seg;
    a.plan.split_rows = split_rows; a.plan.split_ptr = split_ptr; a.plan.n_split = n_split;
    a.scratch = g_noalloc_ptr[dev];
    gt::spmm(a, static_cast<cudaStream_t>(stream));
    e = cudaGetLastError();
    if (e != cudaSuccess) return noalloc_fail(GT_NOALLOC_ERR_CUDA, "kernel launch failed: ", cudaGetErrorString(e));
    return GT_NOALLOC_OK;
}
