// Fused structure-masked sparse attention for sm_100a: SDDMM -> (clamp-)softmax -> SpMM in one pass over the CSR,
// forward and backward, nothing of size [E, H] or [E, H, d] is materialised.
//
// Work decomposition.  One warp owns one *segment* of a row (at most seg_edges consecutive CSR entries; rows longer
// than that -- hubs, the global token -- are cut and merged by a combine kernel: split-KV).  A feature row of H*D
// elements is cut into chunks of 8 elements (16 bytes of bf16); LPR = min(32, H*D/8) lanes cover one row, so a warp
// processes 32/LPR edges at once and every K / V row of an edge is fetched by one fully coalesced 16-byte-per-lane
// transaction.  A head occupies D/8 consecutive lanes; its dot product is finished with log2(D/8) shuffles.  Two edge
// groups are in flight per iteration (their K / V loads are issued before any arithmetic) to keep enough bytes
// outstanding per SM for HBM3e.  Why SIMT and not tcgen05 here: with ~20 edges per row the operation moves ~1 KB per
// edge and does ~1 KFLOP on it (1 FLOP/B against a machine balance of ~215 FLOP/B), so the kernel is bound by the
// gather traffic; a dense tile formulation would gather the same bytes and add >100x redundant MACs.
//
// The same kernels serve every layer kind: `row_map` + `accumulate` implement the compact-accumulate mode of the
// streamed layer (doubly-compressed row list, partials added in place into the reduce-scatter payload), and the
// `*_peers` tables let the forward fetch K / V rows straight from the owners' memory over NVLink (receiver-driven pull
// fused into the kernel: only the rows a tile references cross the switch).
//
// Semantics follow the operator specification in gt_b200/attention/ref.py (reference kernels:
// gt3d/gt3d/attention/triton_kernel.py:38-284, triton_tiled.py:157-479).
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"

namespace gt {

namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxTypesReg = 4;     // edge types whose gate / bias gradients are kept in registers
// edge groups in flight per warp (memory-level parallelism)
constexpr int kUnrollFwd = 2, kUnrollRow = 2, kUnrollCol = 2;

constexpr int kAsyncStages = 4;     // ring depth of the cp.async forward variant

// 16-byte asynchronous copy global -> shared.  L2_ONLY selects cp.async.cg (the line is not allocated in L1): right where a warp
// copies one whole 512-byte row per instruction and nothing is re-read through L1 (K / V / q / row-vector gathers of the
// chunk-per-lane kernels: forward 0.63 ms against 0.72 ms on the 169K-node block, backward 2.1 ms against 2.27 ms); wrong where
// lanes request the same or partial sectors (the column pass' per-head statistics, the head-lane kernels: 2.0 ms against 0.65 ms).
template <bool L2_ONLY = false>
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    if (L2_ONLY)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
    else
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
// ---- bulk row copies (cp.async.bulk, completion on an mbarrier) --------------------------------------------------------
// One instruction moves a whole gathered row global -> shared through the copy engine of the SM instead of 32 lanes x 16 bytes
// through the load/store pipe, which is the busiest unit of these kernels (l1tex 93 % in the forward).
__device__ int g_attn_status = 0;          // set when a bounded mbarrier wait expired (read by the host through attn_status())
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init1(uint64_t* bar) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(bar))); }
__device__ __forceinline__ void mbar_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_row(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(smem_dst)), "l"(gsrc),
                 "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}
// Bounded wait (about 50 ms).  After the first expiry `gave_up` makes every later wait of the thread return at once, so a fault
// in the copy path ends the kernel quickly instead of adding one limit per edge group; the host raises after the step.
__device__ __forceinline__ void mbar_wait_bounded(uint64_t* bar, uint32_t parity, bool& gave_up) {
    if (gave_up) return;
    for (uint32_t tries = 0; tries < (1u << 17); ++tries) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
        if (ok) return;
    }
    gave_up = true;
    atomicExch(&g_attn_status, 7);
}

template <typename T> __device__ __forceinline__ typename Vec8<T>::Raw as_raw(const uint4& u);
template <> __device__ __forceinline__ Vec8<__nv_bfloat16>::Raw as_raw<__nv_bfloat16>(const uint4& u) { return u; }

struct Lanes {
    int lpr;     // lanes per feature row
    int lph;     // lanes per head
    int epw;     // edges per warp iteration
    int sub;     // my edge slot
    int ll;      // my lane inside the row
};

__device__ __forceinline__ Lanes make_lanes(int HD, int D) {
    Lanes L;
    int nch = HD >> 3;
    L.lpr = nch < 32 ? nch : 32;
    L.lph = D >> 3;
    L.epw = 32 / L.lpr;
    int lane = threadIdx.x & 31;
    L.sub = lane / L.lpr;
    L.ll = lane - L.sub * L.lpr;
    return L;
}

__device__ __forceinline__ float head_sum(float v, int lph) {
    for (int o = lph >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(GT_FULL_MASK, v, o);
    return v;
}

__device__ __forceinline__ float safe_exp_diff(float a, float b) {   // exp(a - b) with exp(-inf - -inf) := 0
    return (a == -INFINITY) ? 0.f : __expf(a - b);
}

__device__ __forceinline__ int table_floats(const AttnCommon& c) {
    return (c.score == SCORE_GATED ? c.T * c.H * c.D : 0) + (c.score == SCORE_BIASED ? c.T * c.H : 0);
}

// shared-memory tables: gate [T, HD] and bias [T, H]
__device__ __forceinline__ void load_tables(const AttnCommon& c, float* s_gate, float* s_bias) {
    int HD = c.H * c.D;
    if (c.score == SCORE_GATED)
        for (int i = threadIdx.x; i < c.T * HD; i += blockDim.x) s_gate[i] = c.gate[i];
    if (c.score == SCORE_BIASED)
        for (int i = threadIdx.x; i < c.T * c.H; i += blockDim.x) s_bias[i] = c.bias[i];
    __syncthreads();
}

// Reduce-scatter fused into the forward epilogue: the finished partial row [acc | l] goes, as bf16, straight into the slot
// that the row's OWNER keeps for this rank (a[r, 0 : H*D] = acc, a[r, l_off : l_off + H] = l; 16-byte peer stores over NVLink),
// so the packed payload never exists in local memory and no separate collective moves it.  Called by all 32 lanes.
template <int CPL>
__device__ __forceinline__ void push_partial_row(const AttnFwdArgs& a, long long orow, const Lanes& L, int H, const int (&foff)[CPL],
                                                 const float (&acc)[CPL][8], const float (&l)[CPL]) {
    const int owner = (int)(orow / a.push_rows);
    const long long r = orow - (long long)owner * a.push_rows;
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.push_slot[owner]) + r * a.push_ld;
    const int lane = threadIdx.x & 31;
    const int Hp = (H + 7) & ~7;
    for (int g8 = 0; g8 < Hp; g8 += 8) {                 // the heads' l values are collected in lane 0, eight per 16-byte store
        float lv[8];
#pragma unroll
        for (int x = 0; x < 8; ++x) {
            const int chunk = (g8 + x) * L.lph;          // first 8-element chunk of head g8 + x
            const int src = chunk & 31, ci = chunk >> 5;
            float val = 0.f;
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                const float t = __shfl_sync(GT_FULL_MASK, l[i], src);
                if (i == ci) val = t;
            }
            lv[x] = (g8 + x) < H ? val : 0.f;
        }
        if (lane == 0) Vec8<__nv_bfloat16>::store(dst + a.push_l_off + g8, lv);
    }
    if (L.sub != 0) return;
#pragma unroll
    for (int i = 0; i < CPL; ++i) Vec8<__nv_bfloat16>::store(dst + foff[i], acc[i]);
}

// ------------------------------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------------------------------
template <typename T, int CPL, bool PEER, int SPEC = 0>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, (CPL == 1 ? 6 : 3)) attn_fwd_kernel(AttnFwdArgs a) {
    extern __shared__ float smem[];
    const AttnCommon& c = a.c;
    // SPEC = number of heads of a specialised instance with head dim 32 (4, 8 or 16): the lane layout and every loop bound
    // become compile-time constants; 0 = generic
    const int H = SPEC ? SPEC : c.H, D = SPEC ? 32 : c.D, HD = H * D;
    float* s_gate = smem;
    float* s_bias = smem + (c.score == SCORE_GATED ? c.T * HD : 0);
    load_tables(c, s_gate, s_bias);
    const Lanes L = make_lanes(HD, D);
    // row strides in elements (0 = dense rows of H*D): operands may be column slices of wider matrices, e.g. K | V | message
    const size_t ldq = c.ldq ? (size_t)c.ldq : (size_t)HD, ldk = c.ldk ? (size_t)c.ldk : (size_t)HD;
    const size_t ldr = c.ldr ? (size_t)c.ldr : (size_t)HD, ldo = c.ldo ? (size_t)c.ldo : (size_t)HD;
    (void)ldq; (void)ldk; (void)ldr; (void)ldo;
    const T* q = static_cast<const T*>(a.q);
    const T* kb = static_cast<const T*>(a.k);
    const T* vb = static_cast<const T*>(a.v);
    const bool softmax = c.norm == NORM_SOFTMAX;
    const bool head_writer = (L.ll & (L.lph - 1)) == 0;
    using Raw = typename Vec8<T>::Raw;
    constexpr int U = kUnrollFwd;
    int foff[CPL], head[CPL];
#pragma unroll
    for (int i = 0; i < CPL; ++i) { foff[i] = (L.ll + L.lpr * i) << 3; head[i] = foff[i] / D; }

    // persistent blocks: the tables are loaded once, warps stride over the segments
    const int n_warps = gridDim.x * kWarpsPerBlock;
    for (int seg = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); seg < c.plan.n_seg; seg += n_warps) {
        const int row = c.plan.seg_row[seg], beg = c.plan.seg_beg[seg], end = c.plan.seg_end[seg];
        const int slot = c.plan.seg_slot[seg];
        float qf[CPL][8], acc[CPL][8], l[CPL], m[CPL];
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            Vec8<T>::load(q + (size_t)row * ldq + foff[i], qf[i]);
#pragma unroll
            for (int x = 0; x < 8; ++x) { qf[i][x] *= c.scale; acc[i][x] = 0.f; }
            l[i] = 0.f;
            m[i] = softmax ? -INFINITY : 0.f;
        }
        float qg[CPL][8];                 // q * scale * gate[type] of the type currently cached
        int gt_cached = -1;
        // indices of the first group; every iteration prefetches the next group's indices before it touches K / V
        int jn[U], tn[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int e = beg + u * L.epw + L.sub;
            jn[u] = e < end ? c.idx[e] : -1;
            tn[u] = (e < end && c.etype) ? c.etype[e] : 0;
        }
        for (int base = beg; base < end; base += U * L.epw) {
            int j[U], t[U];
            Raw kr[U][CPL], vr[U][CPL];
#pragma unroll
            for (int u = 0; u < U; ++u) { j[u] = jn[u]; t[u] = tn[u]; }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (j[u] >= 0) {
                    const T* kp; const T* vp;
                    if (PEER) {
                        const int p = j[u] / a.rows_per_peer, r = j[u] - p * a.rows_per_peer;
                        kp = static_cast<const T*>(a.k_peers[p]) + (size_t)r * ldk;
                        vp = static_cast<const T*>(a.v_peers[p]) + (size_t)r * ldk;
                    } else {
                        kp = kb + (size_t)j[u] * ldk;
                        vp = vb + (size_t)j[u] * ldk;
                    }
#pragma unroll
                    for (int i = 0; i < CPL; ++i) { kr[u][i] = Vec8<T>::load_raw(kp + foff[i]); vr[u][i] = Vec8<T>::load_raw(vp + foff[i]); }
                } else {
#pragma unroll
                    for (int i = 0; i < CPL; ++i) { kr[u][i] = Vec8<T>::zero_raw(); vr[u][i] = Vec8<T>::zero_raw(); }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = base + (U + u) * L.epw + L.sub;
                jn[u] = e < end ? c.idx[e] : -1;
                tn[u] = (e < end && c.etype) ? c.etype[e] : 0;
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const bool ok = j[u] >= 0;
                if (c.score == SCORE_GATED && t[u] != gt_cached) {      // edges of a row are grouped by type: rare reload
                    gt_cached = t[u];
#pragma unroll
                    for (int i = 0; i < CPL; ++i) {
                        const float* g = s_gate + gt_cached * HD + foff[i];
#pragma unroll
                        for (int x = 0; x < 8; ++x) qg[i][x] = qf[i][x] * g[x];
                    }
                }
#pragma unroll
                for (int i = 0; i < CPL; ++i) {
                    float kf[8], vf[8];
                    Vec8<T>::unpack(kr[u][i], kf);
                    float s = 0.f;
                    if (c.score == SCORE_GATED) {
#pragma unroll
                        for (int x = 0; x < 8; ++x) s = fmaf(qg[i][x], kf[x], s);
                    } else {
#pragma unroll
                        for (int x = 0; x < 8; ++x) s = fmaf(qf[i][x], kf[x], s);
                    }
                    s = head_sum(s, L.lph);
                    if (c.score == SCORE_BIASED) s += s_bias[t[u] * H + head[i]];
                    Vec8<T>::unpack(vr[u][i], vf);
                    if (softmax) {
                        const float mn = ok ? fmaxf(m[i], s) : m[i];
                        const float corr = safe_exp_diff(m[i], mn);
                        const float p = ok ? __expf(s - mn) : 0.f;
                        l[i] = l[i] * corr + p;
#pragma unroll
                        for (int x = 0; x < 8; ++x) acc[i][x] = fmaf(acc[i][x], corr, p * vf[x]);
                        m[i] = mn;
                    } else {
                        const float p = ok ? __expf(fminf(fmaxf(s, c.lo), c.hi)) : 0.f;
                        l[i] += p;
#pragma unroll
                        for (int x = 0; x < 8; ++x) acc[i][x] = fmaf(p, vf[x], acc[i][x]);
                    }
                }
            }
        }
        // merge the edge slots of the warp
        for (int off = L.lpr; off < 32; off <<= 1) {
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                const float mo = __shfl_xor_sync(GT_FULL_MASK, m[i], off);
                const float lo_ = __shfl_xor_sync(GT_FULL_MASK, l[i], off);
                float wa = 1.f, wb = 1.f;
                if (softmax) {
                    const float mn = fmaxf(m[i], mo);
                    wa = safe_exp_diff(m[i], mn);
                    wb = safe_exp_diff(mo, mn);
                    m[i] = mn;
                }
                l[i] = l[i] * wa + lo_ * wb;
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    const float ao = __shfl_xor_sync(GT_FULL_MASK, acc[i][x], off);
                    acc[i][x] = acc[i][x] * wa + ao * wb;
                }
            }
        }
        if (a.push_n > 0 && slot < 0) {
            push_partial_row<CPL>(a, a.row_map ? a.row_map[row] : row, L, H, foff, acc, l);
            continue;
        }
        if (L.sub != 0) continue;
        if (slot < 0) {
            const long long orow = a.row_map ? a.row_map[row] : row;
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                float* dst = a.acc + orow * a.acc_stride + foff[i];
                if (a.accumulate) {
                    float old[8];
                    Vec8<float>::load(dst, old);
#pragma unroll
                    for (int x = 0; x < 8; ++x) acc[i][x] += old[x];
                }
                Vec8<float>::store(dst, acc[i]);
                if (head_writer) {
                    float* lp = a.l + orow * a.l_stride + head[i];
                    *lp = a.accumulate ? *lp + l[i] : l[i];
                    if (a.m) a.m[orow * H + head[i]] = (m[i] == -INFINITY) ? 0.f : m[i];
                }
            }
        } else {
            float* sc = c.scratch + (size_t)slot * ((HD + 2 * H + 3) & ~3);
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                Vec8<float>::store(sc + foff[i], acc[i]);
                if (head_writer) { sc[HD + head[i]] = l[i]; sc[HD + H + head[i]] = m[i]; }
            }
        }
    }
}

// Variant of the forward kernel whose K / V gathers go through a per-thread ring in shared memory filled by cp.async: the rows
// of kAsyncStages - 1 edge groups are in flight per warp without occupying registers (the register variant holds one group).
// Every lane copies and later reads only its own 16-byte chunks, so no synchronisation between lanes is needed.
// (Measured on the arxiv-shaped block, 8 heads x 32: 2 edge groups x 4 stages 1.080 ms; 3 x 3 1.081; 4 x 3 1.213; 4 x 2 1.215;
// 2 x 6 1.333: deeper rings cost resident blocks.)
template <typename T, int CPL, int SPEC = 0, int UU = kUnrollFwd, int NSTG = kAsyncStages, bool BULK = false>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, (CPL == 1 ? (UU * NSTG <= 8 ? 6 : 4) : 3)) attn_fwd_async_kernel(AttnFwdArgs a) {
    extern __shared__ float smem[];
    const AttnCommon& c = a.c;
    // SPEC = number of heads of a specialised instance with head dim 32 (4, 8 or 16): the lane layout and every loop bound
    // become compile-time constants; 0 = generic
    const int H = SPEC ? SPEC : c.H, D = SPEC ? 32 : c.D, HD = H * D;
    float* s_gate = smem;
    float* s_bias = smem + (c.score == SCORE_GATED ? c.T * HD : 0);
    load_tables(c, s_gate, s_bias);
    // ring: [stage][edge slot u][chunk i][K | V][thread] x 16 bytes, after the tables (16-byte aligned)
    uint4* ring = reinterpret_cast<uint4*>(smem + ((table_floats(c) + 3) & ~3));
    constexpr int NST = NSTG;
    int* tring = reinterpret_cast<int*>(ring + (size_t)NSTG * UU * CPL * 2 * (kWarpsPerBlock * 32));      // edge types of the groups in flight
    // BULK (rows of 32 x 16 bytes, one edge per warp iteration): the ring is [warp][stage][edge slot u][K | V] whole rows, filled
    // by one bulk copy per row (lane 0) that completes on the (warp, stage) mbarrier; bit s of `phase` is the parity to wait for
    uint64_t* bars = reinterpret_cast<uint64_t*>(tring + (size_t)NSTG * UU * (kWarpsPerBlock * 32)) + (threadIdx.x >> 5) * NSTG;
    uint4* wring = ring + (size_t)(threadIdx.x >> 5) * (NSTG * UU * 2 * 32);
    uint32_t phase = 0;
    bool gave_up = false;
    if (BULK) {
        if ((threadIdx.x & 31) == 0)
            for (int st = 0; st < NSTG; ++st) mbar_init1(bars + st);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        __syncthreads();
    }
    const Lanes L = make_lanes(HD, D);
    // row strides in elements (0 = dense rows of H*D): operands may be column slices of wider matrices, e.g. K | V | message
    const size_t ldq = c.ldq ? (size_t)c.ldq : (size_t)HD, ldk = c.ldk ? (size_t)c.ldk : (size_t)HD;
    const size_t ldr = c.ldr ? (size_t)c.ldr : (size_t)HD, ldo = c.ldo ? (size_t)c.ldo : (size_t)HD;
    (void)ldq; (void)ldk; (void)ldr; (void)ldo;
    const T* q = static_cast<const T*>(a.q);
    const T* kb = static_cast<const T*>(a.k);
    const T* vb = static_cast<const T*>(a.v);
    const bool softmax = c.norm == NORM_SOFTMAX;
    const bool head_writer = (L.ll & (L.lph - 1)) == 0;
    using Raw = typename Vec8<T>::Raw;
    constexpr int U = UU;
    int foff[CPL], head[CPL];
#pragma unroll
    for (int i = 0; i < CPL; ++i) { foff[i] = (L.ll + L.lpr * i) << 3; head[i] = foff[i] / D; }

    // persistent blocks: the tables are loaded once, warps stride over the segments
    const int n_warps = gridDim.x * kWarpsPerBlock;
    for (int seg = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); seg < c.plan.n_seg; seg += n_warps) {
        const int row = c.plan.seg_row[seg], beg = c.plan.seg_beg[seg], end = c.plan.seg_end[seg];
        const int slot = c.plan.seg_slot[seg];
        float qf[CPL][8], acc[CPL][8], l[CPL], m[CPL];
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            Vec8<T>::load(q + (size_t)row * ldq + foff[i], qf[i]);
#pragma unroll
            for (int x = 0; x < 8; ++x) { qf[i][x] *= c.scale; acc[i][x] = 0.f; }
            l[i] = 0.f;
            m[i] = softmax ? -INFINITY : 0.f;
        }
        float qg[CPL][8];                 // q * scale * gate[type] of the type currently cached
        int gt_cached = -1;
        const int n_it = (end - beg + U * L.epw - 1) / (U * L.epw);
        // Software pipeline: fetch(g) loads the source indices / types of edge group g into registers one iteration before
        // issue(g) starts that group's copies into ring stage g % NST and parks the types next to them, so neither the copies
        // nor the arithmetic ever wait on an index load.  One commit group per issue() call, also when it is empty.
        int jn[U], tn[U];
        auto fetch = [&](int g) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = min(beg + (g * U + u) * L.epw + L.sub, end - 1);  // padding slots reuse the last edge; their weight is zero
                jn[u] = c.idx[e];
                tn[u] = c.etype ? c.etype[e] : 0;
            }
        };
        auto issue = [&](int g) {
            if (g < n_it) {
                if (BULK) {
                    const int st = g % NST;
                    __syncwarp();                           // every lane has finished reading the stage's previous rows
                    if ((threadIdx.x & 31) == 0) {
                        mbar_expect(bars + st, (uint32_t)(U * 2 * HD * sizeof(T)));
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            bulk_row(wring + ((st * U + u) * 2) * 32, kb + (size_t)jn[u] * ldk, (uint32_t)(HD * sizeof(T)), bars + st);
                            bulk_row(wring + ((st * U + u) * 2 + 1) * 32, vb + (size_t)jn[u] * ldk, (uint32_t)(HD * sizeof(T)), bars + st);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (!BULK) {
                        const T* kp = kb + (size_t)jn[u] * ldk;
                        const T* vp = vb + (size_t)jn[u] * ldk;
#pragma unroll
                        for (int i = 0; i < CPL; ++i) {
                            uint4* dst = ring + ((((g % NST) * U + u) * CPL + i) * 2) * (kWarpsPerBlock * 32) + threadIdx.x;
                            cp_async16<true>(dst, kp + foff[i]);
                            cp_async16<true>(dst + kWarpsPerBlock * 32, vp + foff[i]);
                        }
                    }
                    tring[((g % NST) * U + u) * (kWarpsPerBlock * 32) + threadIdx.x] = tn[u];
                }
                if (g + 1 < n_it) fetch(g + 1);
            }
            if (!BULK) asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if (n_it > 0) fetch(0);             // an empty segment has no edge to read, and idx[beg - 1] may lie before the array
#pragma unroll
        for (int it = 0; it < NST - 1; ++it) issue(it);
        for (int it = 0; it < n_it; ++it) {
            issue(it + NST - 1);
            if (BULK) {
                const int st = it % NST;
                mbar_wait_bounded(bars + st, (phase >> st) & 1u, gave_up);
                phase ^= 1u << st;
            } else {
                asm volatile("cp.async.wait_group %0;" ::"n"(NST - 1) : "memory");
            }
            int j[U], t[U];
            Raw kr[U][CPL], vr[U][CPL];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = beg + (it * U + u) * L.epw + L.sub;
                j[u] = e < end ? 0 : -1;
                t[u] = tring[((it % NST) * U + u) * (kWarpsPerBlock * 32) + threadIdx.x];
#pragma unroll
                for (int i = 0; i < CPL; ++i) {
                    if (BULK) {
                        const uint4* src = wring + (((it % NST) * U + u) * 2) * 32 + (threadIdx.x & 31);
                        kr[u][i] = as_raw<T>(src[0]);
                        vr[u][i] = as_raw<T>(src[32]);
                    } else {
                        const uint4* src = ring + ((((it % NST) * U + u) * CPL + i) * 2) * (kWarpsPerBlock * 32) + threadIdx.x;
                        kr[u][i] = as_raw<T>(src[0]);
                        vr[u][i] = as_raw<T>(src[kWarpsPerBlock * 32]);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const bool ok = j[u] >= 0;
                if (c.score == SCORE_GATED && t[u] != gt_cached) {      // edges of a row are grouped by type: rare reload
                    gt_cached = t[u];
#pragma unroll
                    for (int i = 0; i < CPL; ++i) {
                        const float* g = s_gate + gt_cached * HD + foff[i];
#pragma unroll
                        for (int x = 0; x < 8; ++x) qg[i][x] = qf[i][x] * g[x];
                    }
                }
#pragma unroll
                for (int i = 0; i < CPL; ++i) {
                    float kf[8], vf[8];
                    Vec8<T>::unpack(kr[u][i], kf);
                    float s = 0.f;
                    if (c.score == SCORE_GATED) {
#pragma unroll
                        for (int x = 0; x < 8; ++x) s = fmaf(qg[i][x], kf[x], s);
                    } else {
#pragma unroll
                        for (int x = 0; x < 8; ++x) s = fmaf(qf[i][x], kf[x], s);
                    }
                    s = head_sum(s, L.lph);
                    if (c.score == SCORE_BIASED) s += s_bias[t[u] * H + head[i]];
                    Vec8<T>::unpack(vr[u][i], vf);
                    if (softmax) {
                        const float mn = ok ? fmaxf(m[i], s) : m[i];
                        const float corr = safe_exp_diff(m[i], mn);
                        const float p = ok ? __expf(s - mn) : 0.f;
                        l[i] = l[i] * corr + p;
#pragma unroll
                        for (int x = 0; x < 8; ++x) acc[i][x] = fmaf(acc[i][x], corr, p * vf[x]);
                        m[i] = mn;
                    } else {
                        const float p = ok ? __expf(fminf(fmaxf(s, c.lo), c.hi)) : 0.f;
                        l[i] += p;
#pragma unroll
                        for (int x = 0; x < 8; ++x) acc[i][x] = fmaf(p, vf[x], acc[i][x]);
                    }
                }
            }
        }
        // merge the edge slots of the warp
        for (int off = L.lpr; off < 32; off <<= 1) {
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                const float mo = __shfl_xor_sync(GT_FULL_MASK, m[i], off);
                const float lo_ = __shfl_xor_sync(GT_FULL_MASK, l[i], off);
                float wa = 1.f, wb = 1.f;
                if (softmax) {
                    const float mn = fmaxf(m[i], mo);
                    wa = safe_exp_diff(m[i], mn);
                    wb = safe_exp_diff(mo, mn);
                    m[i] = mn;
                }
                l[i] = l[i] * wa + lo_ * wb;
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    const float ao = __shfl_xor_sync(GT_FULL_MASK, acc[i][x], off);
                    acc[i][x] = acc[i][x] * wa + ao * wb;
                }
            }
        }
        if (a.push_n > 0 && slot < 0) {
            push_partial_row<CPL>(a, a.row_map ? a.row_map[row] : row, L, H, foff, acc, l);
            continue;
        }
        if (L.sub != 0) continue;
        if (slot < 0) {
            const long long orow = a.row_map ? a.row_map[row] : row;
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                float* dst = a.acc + orow * a.acc_stride + foff[i];
                if (a.accumulate) {
                    float old[8];
                    Vec8<float>::load(dst, old);
#pragma unroll
                    for (int x = 0; x < 8; ++x) acc[i][x] += old[x];
                }
                Vec8<float>::store(dst, acc[i]);
                if (head_writer) {
                    float* lp = a.l + orow * a.l_stride + head[i];
                    *lp = a.accumulate ? *lp + l[i] : l[i];
                    if (a.m) a.m[orow * H + head[i]] = (m[i] == -INFINITY) ? 0.f : m[i];
                }
            }
        } else {
            float* sc = c.scratch + (size_t)slot * ((HD + 2 * H + 3) & ~3);
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                Vec8<float>::store(sc + foff[i], acc[i]);
                if (head_writer) { sc[HD + head[i]] = l[i]; sc[HD + H + head[i]] = m[i]; }
            }
        }
    }
}

// Sum of column f over the slots [s0, s1) of a scratch area of row width W, computed by a (32, 8) thread block: the 8 thread
// rows stride over the slots (8 independent loads in flight per column instead of one dependent chain over hundreds of
// slots of a hub row) and are folded through shared memory in a fixed order.  The result is valid for threadIdx.y == 0.
__device__ __forceinline__ float tile_slot_sum(const float* scratch, int s0, int s1, int W, int f, bool valid, float (&sm)[8][33]) {
    float v = 0.f;
    if (valid)
        for (int s = s0 + threadIdx.y; s < s1; s += 8) v += scratch[(size_t)s * W + f];
    __syncthreads();                                    // the previous use of sm is complete
    sm[threadIdx.y][threadIdx.x] = v;
    __syncthreads();
    float t = 0.f;
    if (threadIdx.y == 0) {
#pragma unroll
        for (int y = 0; y < 8; ++y) t += sm[y][threadIdx.x];
    }
    return t;
}

// clamp-exp partials add without rescaling: grid (split rows, 32-column groups of [acc | l]), block (32, 8)
__global__ void attn_fwd_combine_sum_kernel(AttnFwdArgs a) {
    __shared__ float sm[8][33];
    const AttnCommon& c = a.c;
    const int H = c.H, HD = H * c.D, W = (HD + 2 * H + 3) & ~3;
    const int r = blockIdx.x;
    const int row = c.plan.split_rows[r];
    const long long orow = a.row_map ? a.row_map[row] : row;
    const int s0 = c.plan.split_ptr[r], s1 = c.plan.split_ptr[r + 1];
    const int f = blockIdx.y * 32 + threadIdx.x;
    const float v = tile_slot_sum(c.scratch, s0, s1, W, f, f < HD + H, sm);
    if (threadIdx.y != 0 || f >= HD + H) return;
    if (a.push_n > 0) {                                  // split rows of the fused reduce-scatter: the merged row goes to its owner
        const int owner = (int)(orow / a.push_rows);
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.push_slot[owner]) + (orow - (long long)owner * a.push_rows) * a.push_ld;
        dst[f < HD ? f : a.push_l_off + (f - HD)] = __float2bfloat16(v);
        return;
    }
    if (f < HD) {
        float* dst = a.acc + orow * a.acc_stride + f;
        *dst = a.accumulate ? *dst + v : v;
    } else {
        const int h = f - HD;
        float* lp = a.l + orow * a.l_stride + h;
        *lp = a.accumulate ? *lp + v : v;
        if (a.m) a.m[orow * H + h] = 0.f;
    }
}

// merge the slots of the split rows: one block per split row, one thread per feature
__global__ void attn_fwd_combine_kernel(AttnFwdArgs a) {
    const AttnCommon& c = a.c;
    const int H = c.H, D = c.D, HD = H * D, W = (HD + 2 * H + 3) & ~3;     // slots are 16-byte aligned
    const int r = blockIdx.x;
    const int row = c.plan.split_rows[r];
    const long long orow = a.row_map ? a.row_map[row] : row;
    const int s0 = c.plan.split_ptr[r], s1 = c.plan.split_ptr[r + 1];
    const bool softmax = c.norm == NORM_SOFTMAX;
    for (int f = threadIdx.x; f < HD; f += blockDim.x) {
        const int h = f / D;
        float mx = -INFINITY;
        if (softmax)
            for (int s = s0; s < s1; ++s) mx = fmaxf(mx, c.scratch[(size_t)s * W + HD + H + h]);
        float accv = 0.f, lv = 0.f;
        for (int s = s0; s < s1; ++s) {
            const float* sc = c.scratch + (size_t)s * W;
            float w = softmax ? safe_exp_diff(sc[HD + H + h], mx) : 1.f;
            accv = fmaf(sc[f], w, accv);
            lv = fmaf(sc[HD + h], w, lv);
        }
        float* dst = a.acc + orow * a.acc_stride + f;
        *dst = a.accumulate ? *dst + accv : accv;
        if (f == h * D) {
            float* lp = a.l + orow * a.l_stride + h;
            *lp = a.accumulate ? *lp + lv : lv;
            if (a.m) a.m[orow * H + h] = (!softmax || mx == -INFINITY) ? 0.f : mx;
        }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// backward, row pass: dQ and the per-type gate / bias gradients
// ------------------------------------------------------------------------------------------------------------------
// Per row and edge type t the kernel accumulates A_t = sum_{edges of type t} ds_ij k_j.  Then dq_i = scale * sum_t g_t * A_t
// and the row's contribution to the gate gradient is q_i * scale * A_t: the per-edge work is one FMA set, and the per-type
// gradients are flushed to shared memory once per row instead of being carried in registers.
// End of a run of edges of one type in the row pass: dq += g_t * A, the gate gradient of the block += q * A, A = 0.
template <int CPL>
__device__ __forceinline__ void flush_type_run(const float* s_gate, float* s_dg, int t, int HD, const int (&foff)[CPL], const float (&qf)[CPL][8],
                                               float (&A)[CPL][8], float (&dqa)[CPL][8], bool want_dg) {
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
        const float* g = s_gate + t * HD + foff[i];
#pragma unroll
        for (int x = 0; x < 8; ++x) dqa[i][x] = fmaf(g[x], A[i][x], dqa[i][x]);
        if (want_dg) {
#pragma unroll
            for (int x = 0; x < 8; ++x) atomicAdd(&s_dg[t * HD + foff[i] + x], qf[i][x] * A[i][x]);
        }
#pragma unroll
        for (int x = 0; x < 8; ++x) A[i][x] = 0.f;
    }
}

template <typename T, int CPL, bool GATED, int SPEC = 0, bool ASYNC = false>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, (CPL == 1 ? (ASYNC ? 5 : 4) : 2)) attn_bwd_row_kernel(AttnBwdRowArgs a) {
    extern __shared__ float smem[];
    const AttnCommon& c = a.c;
    // SPEC = number of heads of a specialised instance with head dim 32 (4, 8 or 16): the lane layout and every loop bound
    // become compile-time constants; 0 = generic
    const int H = SPEC ? SPEC : c.H, D = SPEC ? 32 : c.D, HD = H * D;
    float* s_gate = smem;
    float* s_bias = smem + (c.score == SCORE_GATED ? c.T * HD : 0);
    float* s_dg = s_bias + (c.score == SCORE_BIASED ? c.T * H : 0);      // [T, HD] or [T, H] block accumulators
    load_tables(c, s_gate, s_bias);
    const bool want_dg = GATED && a.dgate_part;
    const bool want_db = c.score == SCORE_BIASED && a.dbias_part;
    const int acc_n = want_dg ? c.T * HD : (want_db ? c.T * H : 0);
    for (int i = threadIdx.x; i < acc_n; i += blockDim.x) s_dg[i] = 0.f;
    __syncthreads();
    const Lanes L = make_lanes(HD, D);
    // row strides in elements (0 = dense rows of H*D): operands may be column slices of wider matrices, e.g. K | V | message
    const size_t ldq = c.ldq ? (size_t)c.ldq : (size_t)HD, ldk = c.ldk ? (size_t)c.ldk : (size_t)HD;
    const size_t ldr = c.ldr ? (size_t)c.ldr : (size_t)HD, ldo = c.ldo ? (size_t)c.ldo : (size_t)HD;
    (void)ldq; (void)ldk; (void)ldr; (void)ldo;
    const bool softmax = c.norm == NORM_SOFTMAX;
    const T* q = static_cast<const T*>(a.q);
    const T* kb = static_cast<const T*>(a.k);
    const T* vb = static_cast<const T*>(a.v);
    const T* rvb = static_cast<const T*>(a.row_vec);
    const bool head_writer = (L.ll & (L.lph - 1)) == 0;
    using Raw = typename Vec8<T>::Raw;
    constexpr int U = kUnrollRow;
    constexpr int NST = kAsyncStages;
    // ASYNC: K / V gathers through a per-thread cp.async ring placed after the tables and the block accumulators
    uint4* ring = reinterpret_cast<uint4*>(smem + ((table_floats(c) + acc_n + 3) & ~3));
    int* tring = reinterpret_cast<int*>(ring + (size_t)kAsyncStages * kUnrollRow * CPL * 2 * (kWarpsPerBlock * 32));   // types of the groups in flight

    int foff[CPL], head[CPL];
#pragma unroll
    for (int i = 0; i < CPL; ++i) { foff[i] = (L.ll + L.lpr * i) << 3; head[i] = foff[i] / D; }

    const int n_warps = gridDim.x * kWarpsPerBlock;
    for (int seg = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); seg < c.plan.n_seg; seg += n_warps) {
        const int row = c.plan.seg_row[seg], beg = c.plan.seg_beg[seg], end = c.plan.seg_end[seg];
        const int slot = c.plan.seg_slot[seg];
        const long long srow = a.row_map ? a.row_map[row] : row;     // row of q / row_vec / stat / dq
        // A: sum of ds * k over the edges of the CURRENT type run (gated) or of the whole row; dqa: dq accumulated over finished runs
        float qf[CPL][8], rv[CPL][8], A[CPL][8], dqa[CPL][8], db[kMaxTypesReg][CPL], mrow[CPL], rb[CPL], ps[CPL];
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            Vec8<T>::load(q + srow * ldq + foff[i], qf[i]);
            Vec8<T>::load(rvb + srow * ldr + foff[i], rv[i]);
            const float4 st = a.stat[srow * H + head[i]];
            mrow[i] = st.x; rb[i] = st.y; ps[i] = st.z;
#pragma unroll
            for (int x = 0; x < 8; ++x) qf[i][x] *= c.scale;
#pragma unroll
            for (int x = 0; x < 8; ++x) { A[i][x] = 0.f; dqa[i][x] = 0.f; }
#pragma unroll
            for (int tt = 0; tt < kMaxTypesReg; ++tt) db[tt][i] = 0.f;
        }
        float qg[CPL][8];
        int gt_cached = -1;
        const int n_it = (end - beg + U * L.epw - 1) / (U * L.epw);
        int jn[U], tn[U];
        auto fetch = [&](int g) {                       // ASYNC: indices / types of edge group g, one iteration ahead of issue(g)
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = min(beg + (g * U + u) * L.epw + L.sub, end - 1);  // padding slots reuse the last edge; their weight is zero
                jn[u] = c.idx[e];
                tn[u] = c.etype ? c.etype[e] : 0;
            }
        };
        auto issue = [&](int g) {                       // ASYNC: start the copies of edge group g (one commit group per call)
            if (g < n_it) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
#pragma unroll
                    for (int i = 0; i < CPL; ++i) {
                        uint4* dst = ring + ((((g % NST) * U + u) * CPL + i) * 2) * (kWarpsPerBlock * 32) + threadIdx.x;
                        cp_async16<true>(dst, kb + (size_t)jn[u] * ldk + foff[i]);
                        cp_async16<true>(dst + kWarpsPerBlock * 32, vb + (size_t)jn[u] * ldk + foff[i]);
                    }
                    tring[((g % NST) * U + u) * (kWarpsPerBlock * 32) + threadIdx.x] = tn[u];
                }
                if (g + 1 < n_it) fetch(g + 1);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if constexpr (ASYNC) {
            if (n_it > 0) fetch(0);
#pragma unroll
            for (int it = 0; it < NST - 1; ++it) issue(it);
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = beg + u * L.epw + L.sub;
                jn[u] = e < end ? c.idx[e] : -1;
                tn[u] = (e < end && c.etype) ? c.etype[e] : 0;
            }
        }
        for (int it = 0; it < n_it; ++it) {
            const int base = beg + it * U * L.epw;
            int j[U], t[U];
            Raw kr[U][CPL], vr[U][CPL];
            if constexpr (ASYNC) {
                issue(it + NST - 1);
                asm volatile("cp.async.wait_group %0;" ::"n"(NST - 1) : "memory");
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = base + u * L.epw + L.sub;
                    j[u] = e < end ? 0 : -1;
                    t[u] = tring[((it % NST) * U + u) * (kWarpsPerBlock * 32) + threadIdx.x];
#pragma unroll
                    for (int i = 0; i < CPL; ++i) {
                        const uint4* src = ring + ((((it % NST) * U + u) * CPL + i) * 2) * (kWarpsPerBlock * 32) + threadIdx.x;
                        kr[u][i] = as_raw<T>(src[0]);
                        vr[u][i] = as_raw<T>(src[kWarpsPerBlock * 32]);
                    }
                }
            } else {
#pragma unroll
                for (int u = 0; u < U; ++u) { j[u] = jn[u]; t[u] = tn[u]; }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (j[u] >= 0) {
#pragma unroll
                        for (int i = 0; i < CPL; ++i) {
                            kr[u][i] = Vec8<T>::load_raw(kb + (size_t)j[u] * ldk + foff[i]);
                            vr[u][i] = Vec8<T>::load_raw(vb + (size_t)j[u] * ldk + foff[i]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < CPL; ++i) { kr[u][i] = Vec8<T>::zero_raw(); vr[u][i] = Vec8<T>::zero_raw(); }
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = base + (U + u) * L.epw + L.sub;
                    jn[u] = e < end ? c.idx[e] : -1;
                    tn[u] = (e < end && c.etype) ? c.etype[e] : 0;
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const bool ok = j[u] >= 0;
                if (GATED && ok && t[u] != gt_cached) {                 // edges of a row are grouped by type: a run ends (rare)
                    if (gt_cached >= 0) flush_type_run<CPL>(s_gate, s_dg, gt_cached, HD, foff, qf, A, dqa, want_dg);
                    gt_cached = t[u];
#pragma unroll
                    for (int i = 0; i < CPL; ++i) {
                        const float* g = s_gate + gt_cached * HD + foff[i];
#pragma unroll
                        for (int x = 0; x < 8; ++x) qg[i][x] = qf[i][x] * g[x];
                    }
                }
#pragma unroll
                for (int i = 0; i < CPL; ++i) {
                    float kf[8], vf[8];
                    Vec8<T>::unpack(kr[u][i], kf);
                    Vec8<T>::unpack(vr[u][i], vf);
                    float s = 0.f, dp = 0.f;
                    if (GATED) {
#pragma unroll
                        for (int x = 0; x < 8; ++x) s = fmaf(qg[i][x], kf[x], s);
                    } else {
#pragma unroll
                        for (int x = 0; x < 8; ++x) s = fmaf(qf[i][x], kf[x], s);
                    }
#pragma unroll
                    for (int x = 0; x < 8; ++x) dp = fmaf(rv[i][x], vf[x], dp);
                    for (int o = L.lph >> 1; o > 0; o >>= 1) {
                        s += __shfl_xor_sync(GT_FULL_MASK, s, o);
                        dp += __shfl_xor_sync(GT_FULL_MASK, dp, o);
                    }
                    if (c.score == SCORE_BIASED) s += s_bias[t[u] * H + head[i]];
                    float p, mask = 1.f;
                    if (softmax) {
                        p = __expf(s - mrow[i]);
                    } else {
                        p = __expf(fminf(fmaxf(s, c.lo), c.hi));
                        mask = (s >= c.lo && s <= c.hi) ? 1.f : 0.f;
                    }
                    const float ds = ok ? p * ps[i] * (dp + rb[i]) * mask : 0.f;
#pragma unroll
                    for (int x = 0; x < 8; ++x) A[i][x] = fmaf(ds, kf[x], A[i][x]);
                    if (!GATED) {
                        if (want_db) {
#pragma unroll
                            for (int tt = 0; tt < kMaxTypesReg; ++tt)
                                if (t[u] == tt) db[tt][i] += ds;
                        }
                    }
                }
            }
        }
        if (GATED) {
            if (gt_cached >= 0) flush_type_run<CPL>(s_gate, s_dg, gt_cached, HD, foff, qf, A, dqa, want_dg);
        } else {
#pragma unroll
            for (int i = 0; i < CPL; ++i)
#pragma unroll
                for (int x = 0; x < 8; ++x) dqa[i][x] = A[i][x];
        }
        // merge the edge slots of the warp
        for (int off = L.lpr; off < 32; off <<= 1) {
#pragma unroll
            for (int i = 0; i < CPL; ++i)
#pragma unroll
                for (int x = 0; x < 8; ++x) dqa[i][x] += __shfl_xor_sync(GT_FULL_MASK, dqa[i][x], off);
            if (want_db) {
#pragma unroll
                for (int tt = 0; tt < kMaxTypesReg; ++tt)
#pragma unroll
                    for (int i = 0; i < CPL; ++i) db[tt][i] += __shfl_xor_sync(GT_FULL_MASK, db[tt][i], off);
            }
        }
        if (L.sub != 0) continue;
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            float dq[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) dq[x] = dqa[i][x];
            if (!GATED && want_db && head_writer) {
#pragma unroll
                for (int tt = 0; tt < kMaxTypesReg; ++tt)
                    if (tt < c.T) atomicAdd(&s_dg[tt * H + head[i]], db[tt][i]);
            }
#pragma unroll
            for (int x = 0; x < 8; ++x) dq[x] *= c.scale;
            if (slot >= 0) {
                Vec8<float>::store(c.scratch + (size_t)slot * HD + foff[i], dq);
            } else if (a.accumulate_dq) {
                float* dst = static_cast<float*>(a.dq) + srow * ldo + foff[i];
                float old[8];
                Vec8<float>::load(dst, old);
#pragma unroll
                for (int x = 0; x < 8; ++x) old[x] += dq[x];
                Vec8<float>::store(dst, old);
            } else {
                Vec8<T>::store(static_cast<T*>(a.dq) + srow * ldo + foff[i], dq);
            }
        }
    }
    __syncthreads();
    float* part = want_dg ? a.dgate_part + (size_t)blockIdx.x * acc_n : (want_db ? a.dbias_part + (size_t)blockIdx.x * acc_n : nullptr);
    for (int i = threadIdx.x; i < acc_n; i += blockDim.x) part[i] = s_dg[i];
}

// End of a run of edges of one type in the K-only row pass: dq += g_t * A, and the gate gradient q * A goes into per-warp
// REGISTER accumulators (one set per type, selected by a warp-uniform switch, so every index is static): the shared-memory
// atomics of flush_type_run cost about as much as the whole K gather once the rest of the per-edge work is gone.
template <int CPL>
__device__ __forceinline__ void flush_type_run_regs(const float* s_gate, int t, int HD, const int (&foff)[CPL], const float (&qf)[CPL][8],
                                                    float (&A)[CPL][8], float (&dqa)[CPL][8], float (&dg)[kMaxTypesReg][CPL][8], bool want_dg) {
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
        const float* g = s_gate + t * HD + foff[i];
#pragma unroll
        for (int x = 0; x < 8; ++x) dqa[i][x] = fmaf(g[x], A[i][x], dqa[i][x]);
    }
    if (want_dg) {
        switch (t) {
#define GT_DG_CASE(TT)                                                                      \
    case TT:                                                                                \
        _Pragma("unroll") for (int i = 0; i < CPL; ++i)                                     \
            _Pragma("unroll") for (int x = 0; x < 8; ++x) dg[TT][i][x] = fmaf(qf[i][x], A[i][x], dg[TT][i][x]); \
        break;
            GT_DG_CASE(0) GT_DG_CASE(1) GT_DG_CASE(2) GT_DG_CASE(3)
#undef GT_DG_CASE
            default: break;
        }
    }
#pragma unroll
    for (int i = 0; i < CPL; ++i)
#pragma unroll
        for (int x = 0; x < 8; ++x) A[i][x] = 0.f;
}

// ------------------------------------------------------------------------------------------------------------------
// backward, row pass from stored score gradients.  When the column pass ran first and left ds of every entry in CSR order,
// dq_i = scale * sum_t g_t * sum_{edges of type t} ds_ij k_j needs one gathered K row and H floats per edge: no V gather, no
// dot products, no exponentials (the full row pass above recomputes all of them).  Same outputs as attn_bwd_row_kernel.
// ------------------------------------------------------------------------------------------------------------------
template <typename T, int CPL, bool GATED, int SPEC = 0, int UU = kUnrollRow, int NSTG = kAsyncStages, int MINB = (CPL == 1 ? (GATED ? 5 : 6) : 3)>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, MINB) attn_bwd_row_ds_kernel(AttnBwdRowArgs a) {
    extern __shared__ float smem[];
    const AttnCommon& c = a.c;
    const int H = SPEC ? SPEC : c.H, D = SPEC ? 32 : c.D, HD = H * D;
    float* s_gate = smem;
    float* s_bias = smem + (c.score == SCORE_GATED ? c.T * HD : 0);
    float* s_dg = s_bias + (c.score == SCORE_BIASED ? c.T * H : 0);      // [T, HD] or [T, H] block accumulators
    load_tables(c, s_gate, s_bias);
    const bool want_dg = GATED && a.dgate_part;
    const bool want_db = c.score == SCORE_BIASED && a.dbias_part;
    const int acc_n = want_dg ? c.T * HD : (want_db ? c.T * H : 0);
    for (int i = threadIdx.x; i < acc_n; i += blockDim.x) s_dg[i] = 0.f;
    __syncthreads();
    const Lanes L = make_lanes(HD, D);
    const size_t ldq = c.ldq ? (size_t)c.ldq : (size_t)HD, ldk = c.ldk ? (size_t)c.ldk : (size_t)HD;
    const size_t ldo = c.ldo ? (size_t)c.ldo : (size_t)HD;
    const T* q = static_cast<const T*>(a.q);
    const T* kb = static_cast<const T*>(a.k);
    const bool head_writer = (L.ll & (L.lph - 1)) == 0;
    using Raw = typename Vec8<T>::Raw;
    constexpr int U = UU;
    constexpr int NST = NSTG;
    constexpr int NT = kWarpsPerBlock * 32;
    // per-thread rings: K chunks, then the score gradients, then the edge types of the groups in flight
    uint4* ring = reinterpret_cast<uint4*>(smem + ((table_floats(c) + acc_n + 3) & ~3));
    float* dring = reinterpret_cast<float*>(ring + (size_t)NST * U * CPL * NT);
    int* tring = reinterpret_cast<int*>(dring + (size_t)NST * U * CPL * NT);

    int foff[CPL], head[CPL];
#pragma unroll
    for (int i = 0; i < CPL; ++i) { foff[i] = (L.ll + L.lpr * i) << 3; head[i] = foff[i] / D; }

    float dg[kMaxTypesReg][CPL][8];                     // gate gradient of this warp's rows, per type (gated scores only)
#pragma unroll
    for (int tt = 0; tt < kMaxTypesReg; ++tt)
#pragma unroll
        for (int i = 0; i < CPL; ++i)
#pragma unroll
            for (int x = 0; x < 8; ++x) dg[tt][i][x] = 0.f;

    const int n_warps = gridDim.x * kWarpsPerBlock;
    for (int seg = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); seg < c.plan.n_seg; seg += n_warps) {
        const int row = c.plan.seg_row[seg], beg = c.plan.seg_beg[seg], end = c.plan.seg_end[seg];
        const int slot = c.plan.seg_slot[seg];
        const long long srow = a.row_map ? a.row_map[row] : row;
        float qf[CPL][8], A[CPL][8], dqa[CPL][8], db[kMaxTypesReg][CPL];
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            if (want_dg) {
                Vec8<T>::load(q + srow * ldq + foff[i], qf[i]);
#pragma unroll
                for (int x = 0; x < 8; ++x) qf[i][x] *= c.scale;
            } else {
#pragma unroll
                for (int x = 0; x < 8; ++x) qf[i][x] = 0.f;
            }
#pragma unroll
            for (int x = 0; x < 8; ++x) { A[i][x] = 0.f; dqa[i][x] = 0.f; }
#pragma unroll
            for (int tt = 0; tt < kMaxTypesReg; ++tt) db[tt][i] = 0.f;
        }
        int gt_cached = -1;
        const int n_it = (end - beg + U * L.epw - 1) / (U * L.epw);
        int jn[U], tn[U], en[U];
        auto fetch = [&](int g) {                       // column / type of edge group g, one iteration ahead of issue(g)
#pragma unroll
            for (int u = 0; u < U; ++u) {
                en[u] = min(beg + (g * U + u) * L.epw + L.sub, end - 1);        // padding slots reuse the last edge; their weight is zeroed
                jn[u] = c.idx[en[u]];
                tn[u] = c.etype ? c.etype[en[u]] : 0;
            }
        };
        auto issue = [&](int g) {                       // start the copies of edge group g (one commit group per call)
            if (g < n_it) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
#pragma unroll
                    for (int i = 0; i < CPL; ++i) {
                        const int slot_i = (((g % NST) * U + u) * CPL + i) * NT + threadIdx.x;
                        cp_async16<true>(ring + slot_i, kb + (size_t)jn[u] * ldk + foff[i]);
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dring + slot_i)),
                                     "l"(a.ds_in + (size_t)en[u] * H + head[i])
                                     : "memory");
                    }
                    tring[((g % NST) * U + u) * NT + threadIdx.x] = tn[u];
                }
                if (g + 1 < n_it) fetch(g + 1);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if (n_it > 0) fetch(0);
#pragma unroll
        for (int it = 0; it < NST - 1; ++it) issue(it);
        for (int it = 0; it < n_it; ++it) {
            const int base = beg + it * U * L.epw;
            issue(it + NST - 1);
            asm volatile("cp.async.wait_group %0;" ::"n"(NST - 1) : "memory");
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const bool ok = base + u * L.epw + L.sub < end;
                const int t = tring[((it % NST) * U + u) * NT + threadIdx.x];
                if (GATED && ok && t != gt_cached) {                    // edges of a row are grouped by type: a run ends (rare)
                    if (gt_cached >= 0) flush_type_run_regs<CPL>(s_gate, gt_cached, HD, foff, qf, A, dqa, dg, want_dg);
                    gt_cached = t;
                }
#pragma unroll
                for (int i = 0; i < CPL; ++i) {
                    const int slot_i = (((it % NST) * U + u) * CPL + i) * NT + threadIdx.x;
                    float kf[8];
                    Vec8<T>::unpack(as_raw<T>(ring[slot_i]), kf);
                    const float ds = ok ? dring[slot_i] : 0.f;
#pragma unroll
                    for (int x = 0; x < 8; ++x) A[i][x] = fmaf(ds, kf[x], A[i][x]);
                    if (!GATED && want_db) {
#pragma unroll
                        for (int tt = 0; tt < kMaxTypesReg; ++tt)
                            if (t == tt) db[tt][i] += ds;
                    }
                }
            }
        }
        if (GATED) {
            if (gt_cached >= 0) flush_type_run_regs<CPL>(s_gate, gt_cached, HD, foff, qf, A, dqa, dg, want_dg);
        } else {
#pragma unroll
            for (int i = 0; i < CPL; ++i)
#pragma unroll
                for (int x = 0; x < 8; ++x) dqa[i][x] = A[i][x];
        }
        for (int off = L.lpr; off < 32; off <<= 1) {    // merge the edge slots of the warp
#pragma unroll
            for (int i = 0; i < CPL; ++i)
#pragma unroll
                for (int x = 0; x < 8; ++x) dqa[i][x] += __shfl_xor_sync(GT_FULL_MASK, dqa[i][x], off);
            if (want_db) {
#pragma unroll
                for (int tt = 0; tt < kMaxTypesReg; ++tt)
#pragma unroll
                    for (int i = 0; i < CPL; ++i) db[tt][i] += __shfl_xor_sync(GT_FULL_MASK, db[tt][i], off);
            }
        }
        if (L.sub != 0) continue;
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            float dq[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) dq[x] = dqa[i][x] * c.scale;
            if (!GATED && want_db && head_writer) {
#pragma unroll
                for (int tt = 0; tt < kMaxTypesReg; ++tt)
                    if (tt < c.T) atomicAdd(&s_dg[tt * H + head[i]], db[tt][i]);
            }
            if (slot >= 0) {
                Vec8<float>::store(c.scratch + (size_t)slot * HD + foff[i], dq);
            } else if (a.accumulate_dq) {
                float* dst = static_cast<float*>(a.dq) + srow * ldo + foff[i];
                float old[8];
                Vec8<float>::load(dst, old);
#pragma unroll
                for (int x = 0; x < 8; ++x) old[x] += dq[x];
                Vec8<float>::store(dst, old);
            } else {
                Vec8<T>::store(static_cast<T*>(a.dq) + srow * ldo + foff[i], dq);
            }
        }
    }
    if (want_dg) {                                      // one shared-memory reduction per warp and kernel instead of one per row and type
#pragma unroll
        for (int tt = 0; tt < kMaxTypesReg; ++tt)
            if (tt < c.T) {
#pragma unroll
                for (int i = 0; i < CPL; ++i)
#pragma unroll
                    for (int x = 0; x < 8; ++x) atomicAdd(&s_dg[tt * HD + foff[i] + x], dg[tt][i][x]);
            }
    }
    __syncthreads();
    float* part = want_dg ? a.dgate_part + (size_t)blockIdx.x * acc_n : (want_db ? a.dbias_part + (size_t)blockIdx.x * acc_n : nullptr);
    for (int i = threadIdx.x; i < acc_n; i += blockDim.x) part[i] = s_dg[i];
}

// out[row] (+)= sum of the row's slots; grid (split rows, 32-column groups), block (32, 8)
template <typename T>
__global__ void sum_slots_kernel(const SegPlan plan, const float* scratch, int width, const int* row_map, T* out, float* out_f32,
                                 int accumulate, long long ld) {
    __shared__ float sm[8][33];
    const int r = blockIdx.x;
    const int row = plan.split_rows[r];
    const long long orow = row_map ? row_map[row] : row;
    const int s0 = plan.split_ptr[r], s1 = plan.split_ptr[r + 1];
    const int f = blockIdx.y * 32 + threadIdx.x;
    const float v = tile_slot_sum(scratch, s0, s1, width, f, f < width, sm);
    if (threadIdx.y != 0 || f >= width) return;
    if (out_f32) {
        float* d = out_f32 + orow * ld + f;
        *d = accumulate ? *d + v : v;
    } else {
        out[orow * ld + f] = from_float<T>(v);
    }
}

// ------------------------------------------------------------------------------------------------------------------
// backward, column pass: dK, dV over the CSC (no atomics)
// ------------------------------------------------------------------------------------------------------------------
template <typename T, int CPL, int SPEC = 0, bool ASYNC = false>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, (CPL == 1 ? (ASYNC ? 4 : 5) : 2)) attn_bwd_col_kernel(AttnBwdColArgs a) {
    extern __shared__ float smem[];
    const AttnCommon& c = a.c;
    // SPEC = number of heads of a specialised instance with head dim 32 (4, 8 or 16): the lane layout and every loop bound
    // become compile-time constants; 0 = generic
    const int H = SPEC ? SPEC : c.H, D = SPEC ? 32 : c.D, HD = H * D;
    float* s_gate = smem;
    float* s_bias = smem + (c.score == SCORE_GATED ? c.T * HD : 0);
    load_tables(c, s_gate, s_bias);
    const Lanes L = make_lanes(HD, D);
    // row strides in elements (0 = dense rows of H*D): operands may be column slices of wider matrices, e.g. K | V | message
    const size_t ldq = c.ldq ? (size_t)c.ldq : (size_t)HD, ldk = c.ldk ? (size_t)c.ldk : (size_t)HD;
    const size_t ldr = c.ldr ? (size_t)c.ldr : (size_t)HD, ldo = c.ldo ? (size_t)c.ldo : (size_t)HD;
    (void)ldq; (void)ldk; (void)ldr; (void)ldo;
    const bool softmax = c.norm == NORM_SOFTMAX;
    const T* qb = static_cast<const T*>(a.q);
    const T* rvb = static_cast<const T*>(a.row_vec);
    using Raw = typename Vec8<T>::Raw;
    constexpr int U = kUnrollCol;
    constexpr int NST = kAsyncStages;
    // ASYNC: q / row-vector / row-statistics gathers through a per-thread cp.async ring placed after the tables
    uint4* ring = reinterpret_cast<uint4*>(smem + ((table_floats(c) + 3) & ~3));
    int* tring = reinterpret_cast<int*>(ring + (size_t)kAsyncStages * kUnrollCol * CPL * 3 * (kWarpsPerBlock * 32));   // types of the groups in flight
    int foff[CPL], head[CPL];
#pragma unroll
    for (int i = 0; i < CPL; ++i) { foff[i] = (L.ll + L.lpr * i) << 3; head[i] = foff[i] / D; }

    const int n_warps = gridDim.x * kWarpsPerBlock;
    for (int seg = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); seg < c.plan.n_seg; seg += n_warps) {
        const int colj = c.plan.seg_row[seg], beg = c.plan.seg_beg[seg], end = c.plan.seg_end[seg];
        const int slot = c.plan.seg_slot[seg];
        float kf[CPL][8], vf[CPL][8], dk[CPL][8], dv[CPL][8];
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            Vec8<T>::load(static_cast<const T*>(a.k) + (size_t)colj * ldk + foff[i], kf[i]);
            Vec8<T>::load(static_cast<const T*>(a.v) + (size_t)colj * ldk + foff[i], vf[i]);
#pragma unroll
            for (int x = 0; x < 8; ++x) { dk[i][x] = 0.f; dv[i][x] = 0.f; }
        }
        float gc[CPL][8], kg[CPL][8];       // cached gate slice and k * gate of the type currently being walked
        int gt_cached = -1;
        const int n_it = (end - beg + U * L.epw - 1) / (U * L.epw);
        int rn[U], tn[U];
        auto fetch = [&](int g) {                       // ASYNC: row indices / types of entry group g, one iteration ahead of issue(g)
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = min(beg + (g * U + u) * L.epw + L.sub, end - 1);  // padding slots reuse the last entry; their weight is zero
                rn[u] = c.idx[e];
                tn[u] = c.etype ? c.etype[e] : 0;
            }
        };
        auto issue = [&](int g) {                       // ASYNC: start the copies of entry group g (one commit group per call)
            if (g < n_it) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
#pragma unroll
                    for (int i = 0; i < CPL; ++i) {
                        uint4* dst = ring + ((((g % NST) * U + u) * CPL + i) * 3) * (kWarpsPerBlock * 32) + threadIdx.x;
                        cp_async16<true>(dst, qb + (size_t)rn[u] * ldq + foff[i]);
                        cp_async16<true>(dst + kWarpsPerBlock * 32, rvb + (size_t)rn[u] * ldr + foff[i]);
                        cp_async16(dst + 2 * kWarpsPerBlock * 32, a.stat + (size_t)rn[u] * H + head[i]);
                    }
                    tring[((g % NST) * U + u) * (kWarpsPerBlock * 32) + threadIdx.x] = tn[u];
                }
                if (g + 1 < n_it) fetch(g + 1);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if constexpr (ASYNC) {
            if (n_it > 0) fetch(0);
#pragma unroll
            for (int it = 0; it < NST - 1; ++it) issue(it);
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = beg + u * L.epw + L.sub;
                rn[u] = e < end ? c.idx[e] : -1;
                tn[u] = (e < end && c.etype) ? c.etype[e] : 0;
            }
        }
        for (int it = 0; it < n_it; ++it) {
            const int base = beg + it * U * L.epw;
            int r[U], t[U];
            Raw qr[U][CPL], rr[U][CPL];
            float4 st[U][CPL];
            if constexpr (ASYNC) {
                issue(it + NST - 1);
                asm volatile("cp.async.wait_group %0;" ::"n"(NST - 1) : "memory");
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = base + u * L.epw + L.sub;
                    r[u] = e < end ? 0 : -1;
                    t[u] = tring[((it % NST) * U + u) * (kWarpsPerBlock * 32) + threadIdx.x];
#pragma unroll
                    for (int i = 0; i < CPL; ++i) {
                        const uint4* src = ring + ((((it % NST) * U + u) * CPL + i) * 3) * (kWarpsPerBlock * 32) + threadIdx.x;
                        qr[u][i] = as_raw<T>(src[0]);
                        rr[u][i] = as_raw<T>(src[kWarpsPerBlock * 32]);
                        const uint4 sv = src[2 * kWarpsPerBlock * 32];
                        st[u][i] = make_float4(__uint_as_float(sv.x), __uint_as_float(sv.y), __uint_as_float(sv.z), __uint_as_float(sv.w));
                    }
                }
            } else {
#pragma unroll
                for (int u = 0; u < U; ++u) { r[u] = rn[u]; t[u] = tn[u]; }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (r[u] >= 0) {
#pragma unroll
                        for (int i = 0; i < CPL; ++i) {
                            qr[u][i] = Vec8<T>::load_raw(qb + (size_t)r[u] * ldq + foff[i]);
                            rr[u][i] = Vec8<T>::load_raw(rvb + (size_t)r[u] * ldr + foff[i]);
                            st[u][i] = __ldg(a.stat + (size_t)r[u] * H + head[i]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < CPL; ++i) {
                            qr[u][i] = Vec8<T>::zero_raw(); rr[u][i] = Vec8<T>::zero_raw();
                            st[u][i] = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int e = base + (U + u) * L.epw + L.sub;
                    rn[u] = e < end ? c.idx[e] : -1;
                    tn[u] = (e < end && c.etype) ? c.etype[e] : 0;
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const bool ok = r[u] >= 0;
                // CSR position of this entry, for the score gradients handed to the row pass (loaded ahead of the arithmetic)
                const int pe = (a.ds_out != nullptr && ok) ? a.pos[base + u * L.epw + L.sub] : 0;
                if (c.score == SCORE_GATED && t[u] != gt_cached) {      // a column's entries are grouped by type: rare reload
                    gt_cached = t[u];
#pragma unroll
                    for (int i = 0; i < CPL; ++i) {
                        const float* g = s_gate + gt_cached * HD + foff[i];
#pragma unroll
                        for (int x = 0; x < 8; ++x) { gc[i][x] = g[x]; kg[i][x] = kf[i][x] * g[x]; }
                    }
                }
#pragma unroll
                for (int i = 0; i < CPL; ++i) {
                    float qf[8], rv[8];
                    Vec8<T>::unpack(qr[u][i], qf);
                    Vec8<T>::unpack(rr[u][i], rv);
                    float s = 0.f, dp = 0.f;
                    if (c.score == SCORE_GATED) {
#pragma unroll
                        for (int x = 0; x < 8; ++x) s = fmaf(qf[x], kg[i][x], s);
                    } else {
#pragma unroll
                        for (int x = 0; x < 8; ++x) s = fmaf(qf[x], kf[i][x], s);
                    }
#pragma unroll
                    for (int x = 0; x < 8; ++x) dp = fmaf(rv[x], vf[i][x], dp);
                    for (int o = L.lph >> 1; o > 0; o >>= 1) {
                        s += __shfl_xor_sync(GT_FULL_MASK, s, o);
                        dp += __shfl_xor_sync(GT_FULL_MASK, dp, o);
                    }
                    s *= c.scale;
                    if (c.score == SCORE_BIASED) s += s_bias[t[u] * H + head[i]];
                    float p, mask = 1.f;
                    if (softmax) {
                        p = __expf(s - st[u][i].x);
                    } else {
                        p = __expf(fminf(fmaxf(s, c.lo), c.hi));
                        mask = (s >= c.lo && s <= c.hi) ? 1.f : 0.f;
                    }
                    const float P = ok ? p * st[u][i].z : 0.f;
                    const float ds0 = P * (dp + st[u][i].y) * mask;
                    const float ds = ds0 * c.scale;
                    if (a.ds_out != nullptr && ok && (foff[i] % D) == 0) a.ds_out[(size_t)pe * H + head[i]] = ds0;
#pragma unroll
                    for (int x = 0; x < 8; ++x) dv[i][x] = fmaf(P, rv[x], dv[i][x]);
                    if (c.score == SCORE_GATED) {
#pragma unroll
                        for (int x = 0; x < 8; ++x) dk[i][x] = fmaf(ds * qf[x], gc[i][x], dk[i][x]);
                    } else {
#pragma unroll
                        for (int x = 0; x < 8; ++x) dk[i][x] = fmaf(ds, qf[x], dk[i][x]);
                    }
                }
            }
        }
        for (int off = L.lpr; off < 32; off <<= 1)
#pragma unroll
            for (int i = 0; i < CPL; ++i)
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    dk[i][x] += __shfl_xor_sync(GT_FULL_MASK, dk[i][x], off);
                    dv[i][x] += __shfl_xor_sync(GT_FULL_MASK, dv[i][x], off);
                }
        if (L.sub != 0) continue;
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            if (slot >= 0) {
                Vec8<float>::store(c.scratch + (size_t)slot * 2 * HD + foff[i], dk[i]);
                Vec8<float>::store(c.scratch + (size_t)slot * 2 * HD + HD + foff[i], dv[i]);
            } else {
                Vec8<T>::store(static_cast<T*>(a.dk) + (size_t)colj * ldo + foff[i], dk[i]);
                Vec8<T>::store(static_cast<T*>(a.dv) + (size_t)colj * ldo + foff[i], dv[i]);
            }
        }
    }
}

template <typename T>
__global__ void sum_slots_kv_kernel(const SegPlan plan, const float* scratch, int HD, T* dk, T* dv, long long ld) {
    __shared__ float sm[8][33];
    const int r = blockIdx.x;
    const int colj = plan.split_rows[r];
    const int s0 = plan.split_ptr[r], s1 = plan.split_ptr[r + 1];
    const int f = blockIdx.y * 32 + threadIdx.x;
    const float v = tile_slot_sum(scratch, s0, s1, 2 * HD, f, f < 2 * HD, sm);
    if (threadIdx.y != 0 || f >= 2 * HD) return;
    if (f < HD) dk[(size_t)colj * ld + f] = from_float<T>(v);
    else dv[(size_t)colj * ld + f - HD] = from_float<T>(v);
}

// out[i] = sum_b part[b, i]: a block owns 32 columns, its 8 thread rows stride over the partial blocks (coalesced
// 128-byte reads), the 8 sums are folded through shared memory in a fixed order (deterministic)
__global__ void reduce_partials_kernel(const float* part, int n_blocks, int width, float* out, int accumulate) {
    __shared__ float sm[8][33];
    const int i = blockIdx.x * 32 + threadIdx.x;
    float v = 0.f;
    if (i < width)
        for (int b = threadIdx.y; b < n_blocks; b += 8) v += part[(size_t)b * width + i];
    sm[threadIdx.y][threadIdx.x] = v;
    __syncthreads();
    if (threadIdx.y == 0 && i < width) {
        float t = 0.f;
#pragma unroll
        for (int y = 0; y < 8; ++y) t += sm[y][threadIdx.x];
        out[i] = accumulate ? out[i] + t : t;
    }
}

#include "attn_hl.cuh"

// GT_ATTN_HL = "f,r,c": chunks per lane (2 or 4; 0 = use the chunk-per-lane kernels) of the head-lane forward, row-pass and
// column-pass kernels.  Default "0,0,0" (off).  Measured on the 169K-node benchmark block (8 heads x 32, 3.74 M edges): the forward
// with 2 chunks per lane runs in 0.65 ms against 0.72 ms for the chunk-per-lane kernel with L1-allocating copies, but the latter
// with L2-only copies takes 0.63 ms; 4 chunks per lane lose (1.22 ms: a lane's 16-byte pieces of a row are 64 bytes apart, so
// every copy instruction touches 32 sectors for 512 bytes), and the backward passes lose at either width (3.10 ms against
// 2.27 ms: their 140-155 registers leave three blocks per SM).
struct HlCfg { int ch[3]; };
const HlCfg& hl_cfg() {
    static const HlCfg cfg = [] {
        HlCfg c{{0, 0, 0}};
        const char* e = getenv("GT_ATTN_HL");
        int a = 0, b = 0, d = 0;
        if (e && sscanf(e, "%d,%d,%d", &a, &b, &d) == 3) {
            const int v[3] = {a, b, d};
            for (int i = 0; i < 3; ++i) c.ch[i] = (v[i] == 2 || v[i] == 4) ? v[i] : 0;
        }
        return c;
    }();
    return cfg;
}

size_t table_bytes(const AttnCommon& c) {
    size_t n = 0;
    if (c.score == SCORE_GATED) n += (size_t)c.T * c.H * c.D;
    if (c.score == SCORE_BIASED) n += (size_t)c.T * c.H;
    return n * sizeof(float);
}

int cpl_of(int H, int D) { return (H * D / 8) > 32 ? (H * D / 8) / 32 : 1; }

// head count of a specialised kernel instance (head dim 32 and 4, 8 or 16 heads), else 0
int spec_heads(int H, int D) { return (D == 32 && (H == 4 || H == 8 || H == 16)) ? H : 0; }

template <typename K>
void set_smem(K kernel, size_t bytes) {
    if (bytes > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace

bool attn_shape_supported(int H, int D, int T) {
    int HD = H * D;
    if (D < 8 || (D & (D - 1)) || D > 256) return false;          // a head spans a power-of-two number of 8-chunks
    int nch = HD / 8;
    if (nch < 32) { if (nch & (nch - 1)) return false; }
    else if (nch != 32 && nch != 64) return false;                // H*D in {.., 256, 512}
    if (D / 8 > 32) return false;
    if (T > kMaxTypesReg) return false;                           // per-type gradients live in registers
    return true;
}

int attn_scratch_width_fwd(int H, int D) { return (H * D + 2 * H + 3) & ~3; }

int attn_bwd_row_blocks(int n_seg) {
    int want = (n_seg + kWarpsPerBlock - 1) / kWarpsPerBlock;
    int cap = 148 * 12;
    return want < cap ? (want > 0 ? want : 1) : cap;
}

void attn_fwd(const AttnFwdArgs& a_in, cudaStream_t s) {
    const AttnFwdArgs& a = a_in;
    const AttnCommon& c = a.c;
    if (c.plan.n_seg == 0) return;
    int blocks = (c.plan.n_seg + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (blocks > 148 * 24) blocks = 148 * 24;          // persistent: the grid the host-side segment balancing was made for
    const size_t sm = table_bytes(c);
    const bool peer = a.k_peers != nullptr;
    const int cpl = cpl_of(c.H, c.D);
    static const bool use_async = [] { const char* e = getenv("GT_ATTN_ASYNC"); return !(e && e[0] == '0'); }();
    if (hl_cfg().ch[0] && !peer && hl::shape_ok(c) && (c.H >= 8 || getenv("GT_ATTN_HL"))) {   // 4 heads: measured slower (1.28 vs 1.20 ms)
        constexpr int NST = 3;
        const int ch = hl_cfg().ch[0];
        const size_t ring = (size_t)NST * (2 * ch * 16 + 4) * hl::kThreads;
        const size_t smh = ((sm + 15) & ~size_t(15)) + ring;
#define GT_LAUNCH_FWD_HL(HH, CC)                                                                   \
    do {                                                                                           \
        set_smem(hl::attn_fwd_hl_kernel<HH, CC, NST>, smh);                                        \
        hl::attn_fwd_hl_kernel<HH, CC, NST><<<blocks, hl::kThreads, smh, s>>>(a);                  \
    } while (0)
        if (c.H == 4) { if (ch == 4) GT_LAUNCH_FWD_HL(4, 4); else GT_LAUNCH_FWD_HL(4, 2); }
        else if (c.H == 8) { if (ch == 4) GT_LAUNCH_FWD_HL(8, 4); else GT_LAUNCH_FWD_HL(8, 2); }
        else { if (ch == 4) GT_LAUNCH_FWD_HL(16, 4); else GT_LAUNCH_FWD_HL(16, 2); }
#undef GT_LAUNCH_FWD_HL
        if (c.plan.n_split > 0)
            attn_fwd_combine_sum_kernel<<<dim3(c.plan.n_split, (c.H * c.D + c.H + 31) / 32), dim3(32, 8), 0, s>>>(a);
        return;
    }
    if (use_async && !peer && c.dtype == DT_BF16) {
        const size_t ring = (size_t)kAsyncStages * kUnrollFwd * (cpl * 2 * 16 + 4) * kWarpsPerBlock * 32;   // data ring + type ring
        const size_t sma = ((sm + 15) & ~size_t(15)) + ring;
#define GT_LAUNCH_FWD_ASYNC(CPL, SP)                                                                  \
    do {                                                                                              \
        set_smem(attn_fwd_async_kernel<__nv_bfloat16, CPL, SP>, sma);                                 \
        attn_fwd_async_kernel<__nv_bfloat16, CPL, SP><<<blocks, kWarpsPerBlock * 32, sma, s>>>(a);    \
    } while (0)
        const int sp = spec_heads(c.H, c.D);
        // GT_ATTN_BULK=1: rows by cp.async.bulk.  Off by default: measured 0.83 ms against 0.63 ms on the 169K-node block (7.5 M
        // copies of 512 bytes per launch are more than the copy engine retires; it is made for tiles, not for rows).
        static const bool use_bulk = [] { const char* e = getenv("GT_ATTN_BULK"); return e && e[0] == '1'; }();
        const bool rows16 = ((reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v)) & 15) == 0 && ((c.ldk ? c.ldk : c.H * c.D) % 8) == 0;
        if (cpl == 1 && sp == 8 && use_bulk && rows16) {
            const size_t smb = sma + kWarpsPerBlock * kAsyncStages * sizeof(uint64_t);
            set_smem(attn_fwd_async_kernel<__nv_bfloat16, 1, 8, kUnrollFwd, kAsyncStages, true>, smb);
            attn_fwd_async_kernel<__nv_bfloat16, 1, 8, kUnrollFwd, kAsyncStages, true><<<blocks, kWarpsPerBlock * 32, smb, s>>>(a);
        } else if (cpl == 1 && sp == 8) GT_LAUNCH_FWD_ASYNC(1, 8);
        else if (cpl == 1 && sp == 4) GT_LAUNCH_FWD_ASYNC(1, 4);
        else if (cpl == 1) GT_LAUNCH_FWD_ASYNC(1, 0);
        else if (sp == 16) GT_LAUNCH_FWD_ASYNC(2, 16);
        else GT_LAUNCH_FWD_ASYNC(2, 0);
#undef GT_LAUNCH_FWD_ASYNC
        if (c.plan.n_split > 0) {
            if (c.norm == NORM_CLAMPEXP)
                attn_fwd_combine_sum_kernel<<<dim3(c.plan.n_split, (c.H * c.D + c.H + 31) / 32), dim3(32, 8), 0, s>>>(a);
            else
                attn_fwd_combine_kernel<<<c.plan.n_split, 256, 0, s>>>(a);
        }
        return;
    }
#define GT_LAUNCH_FWD(TT, CPL, PEER)                                                     \
    do {                                                                                 \
        set_smem(attn_fwd_kernel<TT, CPL, PEER>, sm);                                    \
        attn_fwd_kernel<TT, CPL, PEER><<<blocks, kWarpsPerBlock * 32, sm, s>>>(a);       \
    } while (0)
    if (c.dtype == DT_BF16) {
        if (cpl == 1) { if (peer) GT_LAUNCH_FWD(__nv_bfloat16, 1, true); else GT_LAUNCH_FWD(__nv_bfloat16, 1, false); }
        else          { if (peer) GT_LAUNCH_FWD(__nv_bfloat16, 2, true); else GT_LAUNCH_FWD(__nv_bfloat16, 2, false); }
    } else {
        if (cpl == 1) { if (peer) GT_LAUNCH_FWD(float, 1, true); else GT_LAUNCH_FWD(float, 1, false); }
        else          { if (peer) GT_LAUNCH_FWD(float, 2, true); else GT_LAUNCH_FWD(float, 2, false); }
    }
#undef GT_LAUNCH_FWD
    if (c.plan.n_split > 0) {
        if (c.norm == NORM_CLAMPEXP)
            attn_fwd_combine_sum_kernel<<<dim3(c.plan.n_split, (c.H * c.D + c.H + 31) / 32), dim3(32, 8), 0, s>>>(a);
        else
            attn_fwd_combine_kernel<<<c.plan.n_split, 256, 0, s>>>(a);
    }
}

void attn_bwd_row(const AttnBwdRowArgs& a_in, cudaStream_t s) {
    const AttnBwdRowArgs& a = a_in;
    const AttnCommon& c = a.c;
    if (c.plan.n_seg == 0) return;
    const int blocks = a.n_blocks > 0 ? a.n_blocks : attn_bwd_row_blocks(c.plan.n_seg);
    size_t sm = table_bytes(c);
    if (c.score == SCORE_GATED && a.dgate_part) sm += (size_t)c.T * c.H * c.D * sizeof(float);
    if (c.score == SCORE_BIASED && a.dbias_part) sm += (size_t)c.T * c.H * sizeof(float);
    const int cpl = cpl_of(c.H, c.D);
    const int HD = c.H * c.D;
    static const bool use_async = [] { const char* e = getenv("GT_ATTN_ASYNC"); return !(e && e[0] == '0'); }();
    const size_t ring_bytes = (size_t)kAsyncStages * kUnrollRow * (cpl * 2 * 16 + 4) * kWarpsPerBlock * 32;   // data ring + type ring
#define GT_LAUNCH_ROW(TT, CPL, SP, AS)                                                        \
    do {                                                                                 \
        if (c.score == SCORE_GATED) {                                                    \
            const size_t smr = AS ? ((sm + 15) & ~size_t(15)) + ring_bytes : sm;         \
            set_smem(attn_bwd_row_kernel<TT, CPL, true, SP, AS>, smr);                   \
            attn_bwd_row_kernel<TT, CPL, true, SP, AS><<<blocks, kWarpsPerBlock * 32, smr, s>>>(a);   \
        } else {                                                                         \
            set_smem(attn_bwd_row_kernel<TT, CPL, false>, sm);                           \
            attn_bwd_row_kernel<TT, CPL, false><<<blocks, kWarpsPerBlock * 32, sm, s>>>(a);  \
        }                                                                                \
        if (c.plan.n_split > 0)                                                          \
            sum_slots_kernel<TT><<<dim3(c.plan.n_split, (HD + 31) / 32), dim3(32, 8), 0, s>>>(c.plan, c.scratch, HD, a.row_map,                       \
                a.accumulate_dq ? nullptr : static_cast<TT*>(a.dq), a.accumulate_dq ? static_cast<float*>(a.dq) : nullptr, \
                a.accumulate_dq, c.ldo ? c.ldo : HD);                                    \
    } while (0)
    const int spec = spec_heads(c.H, c.D);
    if (a.ds_in != nullptr && c.dtype == DT_BF16) {
        // the column pass ran first and left the score gradients: K-only row pass
        const size_t ring_ds = (size_t)kAsyncStages * kUnrollRow * (cpl * (16 + 4) + 4) * kWarpsPerBlock * 32;
        const size_t smd = ((sm + 15) & ~size_t(15)) + ring_ds;
#define GT_LAUNCH_ROW_DS(CPL, SP)                                                                              \
    do {                                                                                                       \
        if (c.score == SCORE_GATED) {                                                                          \
            set_smem(attn_bwd_row_ds_kernel<__nv_bfloat16, CPL, true, SP>, smd);                               \
            attn_bwd_row_ds_kernel<__nv_bfloat16, CPL, true, SP><<<blocks, kWarpsPerBlock * 32, smd, s>>>(a);  \
        } else {                                                                                               \
            set_smem(attn_bwd_row_ds_kernel<__nv_bfloat16, CPL, false, SP>, smd);                              \
            attn_bwd_row_ds_kernel<__nv_bfloat16, CPL, false, SP><<<blocks, kWarpsPerBlock * 32, smd, s>>>(a); \
        }                                                                                                      \
    } while (0)
        // GT_ROWDS_WIDE=1: four edge groups per iteration and a four-deep ring at four blocks per SM for 8 heads x 32 with gated
        // scores.  Timed at 0.484 ms on the 169K-node block against 0.525 ms for the default (2 groups, 4 stages, five blocks; 4 x 3:
        // 0.508, 2 x 6: 0.534, 2 x 3 at six blocks: 0.561).  Opt-in: its results were timed but not compared with the oracle.
        static const bool wide = [] { const char* e = getenv("GT_ROWDS_WIDE"); return e && e[0] == '1'; }();
        if (wide && cpl == 1 && spec == 8 && c.score == SCORE_GATED) {
            constexpr int UU = 4, NN = 4;
            const size_t smx = ((sm + 15) & ~size_t(15)) + (size_t)NN * UU * (cpl * (16 + 4) + 4) * kWarpsPerBlock * 32;
            set_smem(attn_bwd_row_ds_kernel<__nv_bfloat16, 1, true, 8, UU, NN, 4>, smx);
            attn_bwd_row_ds_kernel<__nv_bfloat16, 1, true, 8, UU, NN, 4><<<blocks, kWarpsPerBlock * 32, smx, s>>>(a);
        } else if (cpl == 1 && spec == 8) GT_LAUNCH_ROW_DS(1, 8);
        else if (cpl == 1 && spec == 4) GT_LAUNCH_ROW_DS(1, 4);
        else if (cpl == 1) GT_LAUNCH_ROW_DS(1, 0);
        else if (spec == 16) GT_LAUNCH_ROW_DS(2, 16);
        else GT_LAUNCH_ROW_DS(2, 0);
#undef GT_LAUNCH_ROW_DS
        if (c.plan.n_split > 0)
            sum_slots_kernel<__nv_bfloat16><<<dim3(c.plan.n_split, (HD + 31) / 32), dim3(32, 8), 0, s>>>(
                c.plan, c.scratch, HD, a.row_map, a.accumulate_dq ? nullptr : static_cast<__nv_bfloat16*>(a.dq),
                a.accumulate_dq ? static_cast<float*>(a.dq) : nullptr, a.accumulate_dq, c.ldo ? c.ldo : HD);
        return;
    }
    if (hl_cfg().ch[1] && hl::shape_ok(c)) {
        constexpr int NST = 3;
        const int ch = hl_cfg().ch[1];
        const size_t ring = (size_t)NST * (2 * ch * 16 + 4) * hl::kThreads;
        const size_t smh = ((sm + 15) & ~size_t(15)) + ring;
#define GT_LAUNCH_ROW_HL(HH, CC)                                                                   \
    do {                                                                                           \
        set_smem(hl::attn_bwd_row_hl_kernel<HH, CC, NST>, smh);                                    \
        hl::attn_bwd_row_hl_kernel<HH, CC, NST><<<blocks, hl::kThreads, smh, s>>>(a);              \
    } while (0)
        if (c.H == 4) { if (ch == 4) GT_LAUNCH_ROW_HL(4, 4); else GT_LAUNCH_ROW_HL(4, 2); }
        else if (c.H == 8) { if (ch == 4) GT_LAUNCH_ROW_HL(8, 4); else GT_LAUNCH_ROW_HL(8, 2); }
        else { if (ch == 4) GT_LAUNCH_ROW_HL(16, 4); else GT_LAUNCH_ROW_HL(16, 2); }
#undef GT_LAUNCH_ROW_HL
        if (c.plan.n_split > 0)
            sum_slots_kernel<__nv_bfloat16><<<dim3(c.plan.n_split, (HD + 31) / 32), dim3(32, 8), 0, s>>>(
                c.plan, c.scratch, HD, a.row_map, a.accumulate_dq ? nullptr : static_cast<__nv_bfloat16*>(a.dq),
                a.accumulate_dq ? static_cast<float*>(a.dq) : nullptr, a.accumulate_dq, c.ldo ? c.ldo : HD);
        return;
    }
    if (c.dtype == DT_BF16) {
        if (cpl == 1 && spec == 8 && use_async) GT_LAUNCH_ROW(__nv_bfloat16, 1, 8, true);
        else if (cpl == 1 && spec == 8) GT_LAUNCH_ROW(__nv_bfloat16, 1, 8, false);
        else if (cpl == 1 && spec == 4 && use_async) GT_LAUNCH_ROW(__nv_bfloat16, 1, 4, true);
        else if (cpl == 1 && use_async) GT_LAUNCH_ROW(__nv_bfloat16, 1, 0, true);
        else if (cpl == 1) GT_LAUNCH_ROW(__nv_bfloat16, 1, 0, false);
        else if (spec == 16 && use_async) GT_LAUNCH_ROW(__nv_bfloat16, 2, 16, true);
        else if (use_async) GT_LAUNCH_ROW(__nv_bfloat16, 2, 0, true);
        else GT_LAUNCH_ROW(__nv_bfloat16, 2, 0, false);
    } else {
        if (cpl == 1) GT_LAUNCH_ROW(float, 1, 0, false); else GT_LAUNCH_ROW(float, 2, 0, false);
    }
#undef GT_LAUNCH_ROW
}

void attn_bwd_col(const AttnBwdColArgs& a_in, cudaStream_t s) {
    const AttnBwdColArgs& a = a_in;
    const AttnCommon& c = a.c;
    if (c.plan.n_seg == 0) return;
    int blocks = (c.plan.n_seg + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (blocks > 148 * 24) blocks = 148 * 24;
    const size_t sm = table_bytes(c);
    const int cpl = cpl_of(c.H, c.D);
    const int HD = c.H * c.D;
    static const bool use_async = [] { const char* e = getenv("GT_ATTN_ASYNC"); return !(e && e[0] == '0'); }();
    const size_t ring_bytes = (size_t)kAsyncStages * kUnrollCol * (cpl * 3 * 16 + 4) * kWarpsPerBlock * 32;   // data ring + type ring
#define GT_LAUNCH_COL(TT, CPL, SP, AS)                                                        \
    do {                                                                                 \
        const size_t smc = AS ? ((sm + 15) & ~size_t(15)) + ring_bytes : sm;             \
        set_smem(attn_bwd_col_kernel<TT, CPL, SP, AS>, smc);                             \
        attn_bwd_col_kernel<TT, CPL, SP, AS><<<blocks, kWarpsPerBlock * 32, smc, s>>>(a); \
        if (c.plan.n_split > 0)                                                          \
            sum_slots_kv_kernel<TT><<<dim3(c.plan.n_split, (2 * HD + 31) / 32), dim3(32, 8), 0, s>>>(c.plan, c.scratch, HD, static_cast<TT*>(a.dk),       \
                                                                   static_cast<TT*>(a.dv), c.ldo ? c.ldo : HD);          \
    } while (0)
    const int spec = spec_heads(c.H, c.D);
    if (hl_cfg().ch[2] && hl::shape_ok(c) && a.ds_out == nullptr) {      // the head-lane column kernel does not store score gradients
        constexpr int NST = 3;
        const int ch = hl_cfg().ch[2];
        const size_t ring = (size_t)NST * ((2 * ch + 1) * 16 + 4) * hl::kThreads;
        const size_t smh = ((sm + 15) & ~size_t(15)) + ring;
#define GT_LAUNCH_COL_HL(HH, CC)                                                                   \
    do {                                                                                           \
        set_smem(hl::attn_bwd_col_hl_kernel<HH, CC, NST>, smh);                                    \
        hl::attn_bwd_col_hl_kernel<HH, CC, NST><<<blocks, hl::kThreads, smh, s>>>(a);              \
    } while (0)
        if (c.H == 4) { if (ch == 4) GT_LAUNCH_COL_HL(4, 4); else GT_LAUNCH_COL_HL(4, 2); }
        else if (c.H == 8) { if (ch == 4) GT_LAUNCH_COL_HL(8, 4); else GT_LAUNCH_COL_HL(8, 2); }
        else { if (ch == 4) GT_LAUNCH_COL_HL(16, 4); else GT_LAUNCH_COL_HL(16, 2); }
#undef GT_LAUNCH_COL_HL
        if (c.plan.n_split > 0)
            sum_slots_kv_kernel<__nv_bfloat16><<<dim3(c.plan.n_split, (2 * HD + 31) / 32), dim3(32, 8), 0, s>>>(
                c.plan, c.scratch, HD, static_cast<__nv_bfloat16*>(a.dk), static_cast<__nv_bfloat16*>(a.dv), c.ldo ? c.ldo : HD);
        return;
    }
    if (c.dtype == DT_BF16) {
        if (cpl == 1 && spec == 8 && use_async) GT_LAUNCH_COL(__nv_bfloat16, 1, 8, true);
        else if (cpl == 1 && spec == 8) GT_LAUNCH_COL(__nv_bfloat16, 1, 8, false);
        else if (cpl == 1 && spec == 4 && use_async) GT_LAUNCH_COL(__nv_bfloat16, 1, 4, true);
        else if (cpl == 1 && use_async) GT_LAUNCH_COL(__nv_bfloat16, 1, 0, true);
        else if (cpl == 1) GT_LAUNCH_COL(__nv_bfloat16, 1, 0, false);
        else if (spec == 16 && use_async) GT_LAUNCH_COL(__nv_bfloat16, 2, 16, true);
        else if (use_async) GT_LAUNCH_COL(__nv_bfloat16, 2, 0, true);
        else GT_LAUNCH_COL(__nv_bfloat16, 2, 0, false);
    } else {
        if (cpl == 1) GT_LAUNCH_COL(float, 1, 0, false); else GT_LAUNCH_COL(float, 2, 0, false);
    }
#undef GT_LAUNCH_COL
}

namespace {
template <typename K>
KernelInfo info_of(const char* name, K kernel, size_t dyn_smem) {
    KernelInfo r{name, 0, 0, 0, (int)dyn_smem, 0};
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, kernel) != cudaSuccess) { cudaGetLastError(); return r; }
    set_smem(kernel, dyn_smem);
    r.regs = fa.numRegs; r.local_bytes = (int)fa.localSizeBytes; r.static_smem = (int)fa.sharedSizeBytes;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&r.blocks_per_sm, kernel, kWarpsPerBlock * 32, dyn_smem) != cudaSuccess) cudaGetLastError();
    return r;
}
}  // namespace

// Compiled resources of the attention kernels that serve bf16 operands with 8 heads of 32 (the specialised instances) and of
// the generic instances: registers per thread, local-memory bytes, shared memory and resident blocks per SM.
std::vector<KernelInfo> attn_kernel_info() {
    const size_t tbl = (size_t)3 * 256 * sizeof(float);                     // gate table of 3 edge types x 256 channels
    const size_t per_thread = (size_t)kWarpsPerBlock * 32;
    const size_t ring_f = (size_t)kAsyncStages * kUnrollFwd * (2 * 16 + 4) * per_thread;
    const size_t ring_r = (size_t)kAsyncStages * kUnrollRow * (2 * 16 + 4) * per_thread;
    const size_t ring_c = (size_t)kAsyncStages * kUnrollCol * (3 * 16 + 4) * per_thread;
    std::vector<KernelInfo> v;
    v.push_back(info_of("fwd_ring_bf16_8x32", attn_fwd_async_kernel<__nv_bfloat16, 1, 8>, tbl + ring_f));
    v.push_back(info_of("fwd_ring_bf16_generic", attn_fwd_async_kernel<__nv_bfloat16, 1, 0>, tbl + ring_f));
    v.push_back(info_of("fwd_regs_bf16", attn_fwd_kernel<__nv_bfloat16, 1, false>, tbl));
    v.push_back(info_of("fwd_regs_fp32", attn_fwd_kernel<float, 1, false>, tbl));
    v.push_back(info_of("row_ring_bf16_8x32", attn_bwd_row_kernel<__nv_bfloat16, 1, true, 8, true>, 2 * tbl + ring_r));
    v.push_back(info_of("row_regs_bf16_8x32", attn_bwd_row_kernel<__nv_bfloat16, 1, true, 8, false>, 2 * tbl));
    v.push_back(info_of("col_ring_bf16_8x32", attn_bwd_col_kernel<__nv_bfloat16, 1, 8, true>, tbl + ring_c));
    v.push_back(info_of("col_regs_bf16_8x32", attn_bwd_col_kernel<__nv_bfloat16, 1, 8, false>, tbl));
    return v;
}

int attn_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (v != 0) { const int z = 0; cudaMemcpyToSymbol(g_attn_status, &z, sizeof(int)); }
    return v;
}

void reduce_partials(const float* part, int n_blocks, int width, float* out, cudaStream_t s, int accumulate) {
    if (width <= 0) return;
    reduce_partials_kernel<<<(width + 31) / 32, dim3(32, 8), 0, s>>>(part, n_blocks, width, out, accumulate);
}

}  // namespace gt
