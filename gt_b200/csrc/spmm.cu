// Sparse aggregation out = A @ x on a CSR with fp32 values (the GCN branch and its transpose), and the deterministic
// segmented row sum used by the sparsity-aware reduce-scatter.  One warp per output row; feature rows are read in
// 16-byte chunks, LPR = min(32, pow2ceil(d/8)) lanes per row, several edges per warp iteration when d < 256, fp32
// accumulation.  Bandwidth-bound gather like the attention kernels (replaces cuSPARSE CSR SpMM of the reference,
// gt3d/gt3d/dist/layers.py:53-64, and the ones-valued SpMM of sparse_comm.py:190-202).
#include "common.cuh"
#include "kernels.h"

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
                if (j[u] >= 0 && act[i]) Vec8<T>::load_nc(x + (size_t)j[u] * a.d + ((ll + 32 * i) << 3), xf[u][i]);
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
    T* out = static_cast<T*>(a.out) + (size_t)row * a.d;
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
    T* out = static_cast<T*>(a.out) + (size_t)row * a.d;
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
