// gt_spmm_csr_noalloc: sparse aggregation for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference code base; it exists only in this library.
//
// Who needs it.  The regular aggregation (gt::spmm, reached from Python through gt_b200.ops.native.spmm) cuts very long
// rows (hub nodes) into segments and merges the segments' partial sums through a scratch buffer that the Python wrapper
// takes from the framework's caching allocator.  Some hosts of this library cannot do that: a serving process whose device
// memory was handed out completely at start-up, code that runs between other components with a fixed share of the device memory, or a
// C / C++ embedder that links the shared object without any tensor framework behind it.  For them cudaMalloc is either
// forbidden or may fail at an arbitrary moment, and a failed allocation in the middle of a request is worse than a size
// limit that is known in advance.
//
// What it does instead.  The scratch lives in a file-scope `static __device__` array inside the library (see spmm.cu),
// GT_NOALLOC_SCRATCH_FLOATS floats (4 MiB) on every GPU that loads the library, held until the process exits.  The caller
// passes inputs, the output and the segment plan exactly as for gt::spmm; nothing is allocated or freed by the call, neither
// with cudaMalloc / cudaFree nor through any library routine.
//
// Rules of use.
//  * Capacity: n_slots * d must not exceed GT_NOALLOC_SCRATCH_FLOATS; a larger request is rejected with
//    GT_NOALLOC_ERR_CAPACITY and nothing is launched.  gt_noalloc_last_error() returns a readable message.
//  * The plan must agree with n_slots: n_slots has to equal split_ptr[n_split] (= max(seg_slot) + 1), and EVERY seg_slot[i]
//    must be < n_slots.  The check above is made on the host scalar, while the kernels index the scratch with the slot
//    numbers stored in the device arrays, which host code cannot read without a copy: a plan whose slot numbers exceed the
//    declared n_slots writes past the array.  Validate plans on the host before uploading them
//    (gt_b200.utils.checks.validate_segment_plan does).
//  * A plan without segments (n_seg == 0) describes a matrix without entries: the call fills `out` with zeros.
//  * First call on a device: the call looks up the device address of the scratch array (cudaGetSymbolAddress, with that
//    device current) and caches it per device.  Make this first call outside any stream capture.
//  * The scratch is shared by all calls and keeps the previous call's contents.  Every slot a call reads was written by the
//    same call beforehand, so nothing has to be cleared; but two calls whose kernels overlap in time on one GPU (different
//    streams, or different host threads) race on the array.  Serialise them on one stream.
//  * All pointers are device pointers valid on the current device; `stream` is a cudaStream_t (0 = default stream).
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GT_NOALLOC_SCRATCH_FLOATS (1u << 20)

enum {
    GT_NOALLOC_OK = 0,
    GT_NOALLOC_ERR_CAPACITY = 1,   // n_slots * d exceeds the built-in scratch
    GT_NOALLOC_ERR_ARGUMENT = 2,   // bad shape / dtype / null pointer
    GT_NOALLOC_ERR_CUDA = 3        // a CUDA runtime call failed (symbol lookup or launch)
};

// out[r, :] = sum_{e in row r} w[e] * x[idx[e], :]   for a CSR (ptr, idx, w) with n_out rows and feature width d.
// dtype: 0 = float32, 1 = bfloat16 (x and out); w is float32 or NULL (all ones); d % 8 == 0, d <= 1024.
// The plan arrays are those of gt_b200.attention.csr.SegmentPlan (one warp per segment; seg_slot = -1 for rows with a
// single segment, otherwise the slot index; split_rows / split_ptr list the cut rows and their slot ranges).
int gt_spmm_csr_noalloc(int dtype, const int* ptr, const int* idx, const float* w, const void* x, void* out, int n_out, int d,
                        const int* seg_row, const int* seg_beg, const int* seg_end, const int* seg_slot, int n_seg,
                        const int* split_rows, const int* split_ptr, int n_split, int n_slots, void* stream);

// Message of the last failing call of this thread ("" if none).
const char* gt_noalloc_last_error(void);

// Capacity of the built-in scratch in floats (= GT_NOALLOC_SCRATCH_FLOATS).
size_t gt_noalloc_scratch_floats(void);

#ifdef __cplusplus
}
#endif
