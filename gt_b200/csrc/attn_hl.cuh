// "Head-lane" variants of the fused sparse attention kernels for the common case bf16, head dim 32, clamp-exp normalisation,
// H in {4, 8, 16} heads (included by attn.cu, same namespace and helpers).
//
// The row-per-warp kernels of attn.cu give every lane ONE 16-byte chunk of a feature row, so a warp handles one edge per
// iteration when H * 32 = 256 and spends ~3/4 of its instructions on per-edge bookkeeping that every lane repeats (index and
// type fetch, address arithmetic, ring slots, the exp, the clamp, shuffles that finish a head's dot product).  Here a lane owns
// CH consecutive chunks (CH * 8 channels) of ONE head, LPE = H * 4 / CH lanes cover an edge and a warp walks EPW = 32 / LPE edges
// per iteration: the per-edge bookkeeping is issued once per EPW edges, a head's dot product needs log2(4 / CH) shuffles (none
// for CH = 4), and every (edge, head) pair evaluates its exp exactly once per 4 / CH lanes instead of on four.  The arithmetic on the
// gathered data (unpack + FMA per channel) is unchanged, so the instruction count per edge drops from ~113 to ~36 + 77 / EPW.
// Gathers still go through a per-thread cp.async ring (each lane copies and later reads only its own chunks: no
// synchronisation between lanes); a lane's chunks of one row are consecutive, so the two halves of every 32-byte sector are
// requested by neighbouring instructions of the same lane and the second one hits L1.
//
// Work decomposition, segment plans, scratch layouts of split rows and the combine kernels are those of attn.cu.
#pragma once

namespace hl {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

template <int H, int CH>
struct Geo {
    static constexpr int HD = H * 32;
    static constexpr int C = CH * 8;            // channels per lane
    static constexpr int LPH = 4 / CH;          // lanes per head
    static constexpr int LPE = H * LPH;         // lanes per edge
    static constexpr int EPW = 32 / LPE;        // edges per warp iteration
    static_assert(LPE <= 32 && EPW >= 1, "a warp must hold at least one edge");
};

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
    f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
    f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xffff0000u);
    f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xffff0000u);
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return u;
}

template <int LPH>
__device__ __forceinline__ float head_reduce(float v) {
#pragma unroll
    for (int o = LPH >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(GT_FULL_MASK, v, o);
    return v;
}

// ------------------------------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------------------------------
template <int H, int CH, int NST>
__global__ void __launch_bounds__(kThreads, (CH == 4 ? 3 : 4)) attn_fwd_hl_kernel(AttnFwdArgs a) {
    using G = Geo<H, CH>;
    constexpr int HD = G::HD, C = G::C, LPH = G::LPH, LPE = G::LPE, EPW = G::EPW;
    extern __shared__ float smem[];
    const AttnCommon& c = a.c;
    float* s_gate = smem;
    float* s_bias = smem + (c.score == SCORE_GATED ? c.T * HD : 0);
    load_tables(c, s_gate, s_bias);
    uint4* ring = reinterpret_cast<uint4*>(smem + ((table_floats(c) + 3) & ~3));            // [NST][2 * CH][kThreads]
    int* tring = reinterpret_cast<int*>(ring + (size_t)NST * 2 * CH * kThreads);             // [NST][kThreads]
    const int lane = threadIdx.x & 31;
    const int slot_id = lane / LPE, hl_ = lane - slot_id * LPE;
    const int head = hl_ / LPH, coff = head * 32 + (hl_ - head * LPH) * C;                  // first channel of this lane
    const size_t ldq = c.ldq ? (size_t)c.ldq : (size_t)HD, ldk = c.ldk ? (size_t)c.ldk : (size_t)HD;
    const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(a.q);
    const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(a.k) + coff;
    const __nv_bfloat16* vb = static_cast<const __nv_bfloat16*>(a.v) + coff;
    const bool gated = c.score == SCORE_GATED, biased = c.score == SCORE_BIASED;

    const int n_warps = gridDim.x * kWarps;
    for (int seg = blockIdx.x * kWarps + (threadIdx.x >> 5); seg < c.plan.n_seg; seg += n_warps) {
        const int row = c.plan.seg_row[seg], beg = c.plan.seg_beg[seg], end = c.plan.seg_end[seg];
        const int slot = c.plan.seg_slot[seg];
        const __nv_bfloat16* qrow = q + (size_t)row * ldq + coff;
        float qg[C], acc[C], l = 0.f;
#pragma unroll
        for (int i = 0; i < C; ++i) acc[i] = 0.f;
        auto load_qg = [&](int t) {          // q * scale (* gate of type t)
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float f[8];
                unpack8(__ldg(reinterpret_cast<const uint4*>(qrow + ch * 8)), f);
#pragma unroll
                for (int x = 0; x < 8; ++x) qg[ch * 8 + x] = f[x] * c.scale * (gated ? s_gate[t * HD + coff + ch * 8 + x] : 1.f);
            }
        };
        int gt_cached = -1;
        if (!gated) load_qg(0);
        const int n_it = (end - beg + EPW - 1) / EPW;
        int jn = 0, tn = 0;
        auto fetch = [&](int g) {
            const int e = min(beg + g * EPW + slot_id, end - 1);       // padding slots reuse the last edge; their weight is zero
            jn = c.idx[e];
            tn = c.etype ? c.etype[e] : 0;
        };
        auto issue = [&](int g) {
            if (g < n_it) {
                const __nv_bfloat16* kp = kb + (size_t)jn * ldk;
                const __nv_bfloat16* vp = vb + (size_t)jn * ldk;
                uint4* dst = ring + (size_t)(g % NST) * 2 * CH * kThreads + threadIdx.x;
#pragma unroll
                for (int ch = 0; ch < CH; ++ch) {
                    cp_async16(dst + (2 * ch) * kThreads, kp + ch * 8);
                    cp_async16(dst + (2 * ch + 1) * kThreads, vp + ch * 8);
                }
                tring[(g % NST) * kThreads + threadIdx.x] = tn;
                if (g + 1 < n_it) fetch(g + 1);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if (n_it > 0) fetch(0);
#pragma unroll
        for (int it = 0; it < NST - 1; ++it) issue(it);
        for (int it = 0; it < n_it; ++it) {
            issue(it + NST - 1);
            asm volatile("cp.async.wait_group %0;" ::"n"(NST - 1) : "memory");
            const bool ok = beg + it * EPW + slot_id < end;
            const int t = tring[(it % NST) * kThreads + threadIdx.x];
            if (gated && t != gt_cached) { gt_cached = t; load_qg(t); }
            const uint4* src = ring + (size_t)(it % NST) * 2 * CH * kThreads + threadIdx.x;
            float s0 = 0.f, s1 = 0.f;
            uint4 vraw[CH];
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float kf[8];
                unpack8(src[(2 * ch) * kThreads], kf);
                vraw[ch] = src[(2 * ch + 1) * kThreads];
#pragma unroll
                for (int x = 0; x < 8; x += 2) {
                    s0 = fmaf(qg[ch * 8 + x], kf[x], s0);
                    s1 = fmaf(qg[ch * 8 + x + 1], kf[x + 1], s1);
                }
            }
            float s = head_reduce<LPH>(s0 + s1);
            if (biased) s += s_bias[t * H + head];
            const float p = ok ? __expf(fminf(fmaxf(s, c.lo), c.hi)) : 0.f;
            l += p;
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float vf[8];
                unpack8(vraw[ch], vf);
#pragma unroll
                for (int x = 0; x < 8; ++x) acc[ch * 8 + x] = fmaf(p, vf[x], acc[ch * 8 + x]);
            }
        }
        // merge the edge slots of the warp
#pragma unroll
        for (int off = LPE; off < 32; off <<= 1) {
            l += __shfl_xor_sync(GT_FULL_MASK, l, off);
#pragma unroll
            for (int i = 0; i < C; ++i) acc[i] += __shfl_xor_sync(GT_FULL_MASK, acc[i], off);
        }
        const long long orow = a.row_map ? a.row_map[row] : row;
        if (a.push_n > 0 && slot < 0) {
            // reduce-scatter fused into the epilogue: bf16 [acc | l] row into the slot its owner keeps for this rank
            const int owner = (int)(orow / a.push_rows);
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.push_slot[owner]) + (orow - (long long)owner * a.push_rows) * a.push_ld;
            constexpr int Hp = (H + 7) & ~7;
#pragma unroll
            for (int g8 = 0; g8 < Hp; g8 += 8) {
                float lv[8];
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    const float t = __shfl_sync(GT_FULL_MASK, l, ((g8 + x) < H ? (g8 + x) : 0) * LPH);
                    lv[x] = (g8 + x) < H ? t : 0.f;
                }
                if (lane == 0) *reinterpret_cast<uint4*>(dst + a.push_l_off + g8) = pack8(lv);
            }
            if (slot_id == 0) {
#pragma unroll
                for (int ch = 0; ch < CH; ++ch) {
                    float f[8];
#pragma unroll
                    for (int x = 0; x < 8; ++x) f[x] = acc[ch * 8 + x];
                    *reinterpret_cast<uint4*>(dst + coff + ch * 8) = pack8(f);
                }
            }
            continue;
        }
        if (slot_id != 0) continue;
        const bool head_writer = (hl_ % LPH) == 0;
        if (slot < 0) {
            float* dst = a.acc + orow * a.acc_stride + coff;
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float f[8];
#pragma unroll
                for (int x = 0; x < 8; ++x) f[x] = acc[ch * 8 + x];
                if (a.accumulate) {
                    float old[8];
                    Vec8<float>::load(dst + ch * 8, old);
#pragma unroll
                    for (int x = 0; x < 8; ++x) f[x] += old[x];
                }
                Vec8<float>::store(dst + ch * 8, f);
            }
            if (head_writer) {
                float* lp = a.l + orow * a.l_stride + head;
                *lp = a.accumulate ? *lp + l : l;
                if (a.m) a.m[orow * H + head] = 0.f;
            }
        } else {
            float* sc = c.scratch + (size_t)slot * ((HD + 2 * H + 3) & ~3);
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float f[8];
#pragma unroll
                for (int x = 0; x < 8; ++x) f[x] = acc[ch * 8 + x];
                Vec8<float>::store(sc + coff + ch * 8, f);
            }
            if (head_writer) { sc[HD + head] = l; sc[HD + H + head] = 0.f; }
        }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// backward, row pass: dQ and the per-type gate / bias gradients
// ------------------------------------------------------------------------------------------------------------------
template <int H, int CH, int NST>
__global__ void __launch_bounds__(kThreads, (CH == 4 ? 2 : 3)) attn_bwd_row_hl_kernel(AttnBwdRowArgs a) {
    using G = Geo<H, CH>;
    constexpr int HD = G::HD, C = G::C, LPH = G::LPH, LPE = G::LPE, EPW = G::EPW;
    extern __shared__ float smem[];
    const AttnCommon& c = a.c;
    float* s_gate = smem;
    float* s_bias = smem + (c.score == SCORE_GATED ? c.T * HD : 0);
    float* s_dg = s_bias + (c.score == SCORE_BIASED ? c.T * H : 0);
    load_tables(c, s_gate, s_bias);
    const bool gated = c.score == SCORE_GATED, biased = c.score == SCORE_BIASED;
    const bool want_dg = gated && a.dgate_part, want_db = biased && a.dbias_part;
    const int acc_n = want_dg ? c.T * HD : (want_db ? c.T * H : 0);
    for (int i = threadIdx.x; i < acc_n; i += blockDim.x) s_dg[i] = 0.f;
    __syncthreads();
    uint4* ring = reinterpret_cast<uint4*>(smem + ((table_floats(c) + acc_n + 3) & ~3));
    int* tring = reinterpret_cast<int*>(ring + (size_t)NST * 2 * CH * kThreads);
    const int lane = threadIdx.x & 31;
    const int slot_id = lane / LPE, hl_ = lane - slot_id * LPE;
    const int head = hl_ / LPH, coff = head * 32 + (hl_ - head * LPH) * C;
    const bool head_writer = (hl_ % LPH) == 0;
    const size_t ldq = c.ldq ? (size_t)c.ldq : (size_t)HD, ldk = c.ldk ? (size_t)c.ldk : (size_t)HD;
    const size_t ldr = c.ldr ? (size_t)c.ldr : (size_t)HD, ldo = c.ldo ? (size_t)c.ldo : (size_t)HD;
    const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(a.q);
    const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(a.k) + coff;
    const __nv_bfloat16* vb = static_cast<const __nv_bfloat16*>(a.v) + coff;
    const __nv_bfloat16* rvb = static_cast<const __nv_bfloat16*>(a.row_vec);

    const int n_warps = gridDim.x * kWarps;
    for (int seg = blockIdx.x * kWarps + (threadIdx.x >> 5); seg < c.plan.n_seg; seg += n_warps) {
        const int row = c.plan.seg_row[seg], beg = c.plan.seg_beg[seg], end = c.plan.seg_end[seg];
        const int slot = c.plan.seg_slot[seg];
        const long long srow = a.row_map ? a.row_map[row] : row;
        const __nv_bfloat16* qrow = q + (size_t)srow * ldq + coff;
        float qg[C], rv[C], A[C], dqa[C];
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
            float f[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(rvb + (size_t)srow * ldr + coff + ch * 8)), f);
#pragma unroll
            for (int x = 0; x < 8; ++x) { rv[ch * 8 + x] = f[x]; A[ch * 8 + x] = 0.f; dqa[ch * 8 + x] = 0.f; }
        }
        const float4 st = a.stat[srow * H + head];
        const float rb = st.y, ps = st.z;
        float db[kMaxTypesReg];
#pragma unroll
        for (int tt = 0; tt < kMaxTypesReg; ++tt) db[tt] = 0.f;
        auto load_qg = [&](int t) {
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float f[8];
                unpack8(__ldg(reinterpret_cast<const uint4*>(qrow + ch * 8)), f);
#pragma unroll
                for (int x = 0; x < 8; ++x) qg[ch * 8 + x] = f[x] * c.scale * (gated ? s_gate[t * HD + coff + ch * 8 + x] : 1.f);
            }
        };
        // end of a run of edges of one type: dq += g_t * A, block gate gradient += (q * scale) * A, A = 0
        auto flush = [&](int t) {
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float f[8];
                if (want_dg) unpack8(__ldg(reinterpret_cast<const uint4*>(qrow + ch * 8)), f);
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    const int i = ch * 8 + x;
                    dqa[i] = fmaf(s_gate[t * HD + coff + i], A[i], dqa[i]);
                    if (want_dg) atomicAdd(&s_dg[t * HD + coff + i], f[x] * c.scale * A[i]);
                    A[i] = 0.f;
                }
            }
        };
        int gt_cached = -1;
        if (!gated) load_qg(0);
        const int n_it = (end - beg + EPW - 1) / EPW;
        int jn = 0, tn = 0;
        auto fetch = [&](int g) {
            const int e = min(beg + g * EPW + slot_id, end - 1);
            jn = c.idx[e];
            tn = c.etype ? c.etype[e] : 0;
        };
        auto issue = [&](int g) {
            if (g < n_it) {
                const __nv_bfloat16* kp = kb + (size_t)jn * ldk;
                const __nv_bfloat16* vp = vb + (size_t)jn * ldk;
                uint4* dst = ring + (size_t)(g % NST) * 2 * CH * kThreads + threadIdx.x;
#pragma unroll
                for (int ch = 0; ch < CH; ++ch) {
                    cp_async16(dst + (2 * ch) * kThreads, kp + ch * 8);
                    cp_async16(dst + (2 * ch + 1) * kThreads, vp + ch * 8);
                }
                tring[(g % NST) * kThreads + threadIdx.x] = tn;
                if (g + 1 < n_it) fetch(g + 1);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if (n_it > 0) fetch(0);
#pragma unroll
        for (int it = 0; it < NST - 1; ++it) issue(it);
        for (int it = 0; it < n_it; ++it) {
            issue(it + NST - 1);
            asm volatile("cp.async.wait_group %0;" ::"n"(NST - 1) : "memory");
            const bool ok = beg + it * EPW + slot_id < end;
            const int t = tring[(it % NST) * kThreads + threadIdx.x];
            if (gated && ok && t != gt_cached) {
                if (gt_cached >= 0) flush(gt_cached);
                gt_cached = t;
                load_qg(t);
            }
            const uint4* src = ring + (size_t)(it % NST) * 2 * CH * kThreads + threadIdx.x;
            uint4 kraw[CH];
            float s0 = 0.f, s1 = 0.f, d0 = 0.f, d1 = 0.f;
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float kf[8], vf[8];
                kraw[ch] = src[(2 * ch) * kThreads];
                unpack8(kraw[ch], kf);
                unpack8(src[(2 * ch + 1) * kThreads], vf);
#pragma unroll
                for (int x = 0; x < 8; x += 2) {
                    s0 = fmaf(qg[ch * 8 + x], kf[x], s0);
                    s1 = fmaf(qg[ch * 8 + x + 1], kf[x + 1], s1);
                    d0 = fmaf(rv[ch * 8 + x], vf[x], d0);
                    d1 = fmaf(rv[ch * 8 + x + 1], vf[x + 1], d1);
                }
            }
            float s = head_reduce<LPH>(s0 + s1);
            const float dp = head_reduce<LPH>(d0 + d1);
            if (biased) s += s_bias[t * H + head];
            const float p = __expf(fminf(fmaxf(s, c.lo), c.hi));
            const float mask = (s >= c.lo && s <= c.hi) ? 1.f : 0.f;
            const float ds = ok ? p * ps * (dp + rb) * mask : 0.f;
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float kf[8];
                unpack8(kraw[ch], kf);
#pragma unroll
                for (int x = 0; x < 8; ++x) A[ch * 8 + x] = fmaf(ds, kf[x], A[ch * 8 + x]);
            }
            if (want_db) {
#pragma unroll
                for (int tt = 0; tt < kMaxTypesReg; ++tt)
                    if (t == tt) db[tt] += ds;
            }
        }
        if (gated) {
            if (gt_cached >= 0) flush(gt_cached);
        } else {
#pragma unroll
            for (int i = 0; i < C; ++i) dqa[i] = A[i];
        }
        if (want_db && head_writer) {
#pragma unroll
            for (int tt = 0; tt < kMaxTypesReg; ++tt)
                if (tt < c.T && db[tt] != 0.f) atomicAdd(&s_dg[tt * H + head], db[tt]);
        }
#pragma unroll
        for (int off = LPE; off < 32; off <<= 1)
#pragma unroll
            for (int i = 0; i < C; ++i) dqa[i] += __shfl_xor_sync(GT_FULL_MASK, dqa[i], off);
        if (slot_id != 0) continue;
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
            float f[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) f[x] = dqa[ch * 8 + x] * c.scale;
            if (slot >= 0) {
                Vec8<float>::store(c.scratch + (size_t)slot * HD + coff + ch * 8, f);
            } else if (a.accumulate_dq) {
                float* dst = static_cast<float*>(a.dq) + srow * ldo + coff + ch * 8;
                float old[8];
                Vec8<float>::load(dst, old);
#pragma unroll
                for (int x = 0; x < 8; ++x) old[x] += f[x];
                Vec8<float>::store(dst, old);
            } else {
                *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.dq) + srow * ldo + coff + ch * 8) = pack8(f);
            }
        }
    }
    __syncthreads();
    float* part = want_dg ? a.dgate_part + (size_t)blockIdx.x * acc_n : (want_db ? a.dbias_part + (size_t)blockIdx.x * acc_n : nullptr);
    for (int i = threadIdx.x; i < acc_n; i += blockDim.x) part[i] = s_dg[i];
}

// ------------------------------------------------------------------------------------------------------------------
// backward, column pass: dK, dV over the CSC (no atomics)
// ------------------------------------------------------------------------------------------------------------------
template <int H, int CH, int NST>
__global__ void __launch_bounds__(kThreads, (CH == 4 ? 2 : 3)) attn_bwd_col_hl_kernel(AttnBwdColArgs a) {
    using G = Geo<H, CH>;
    constexpr int HD = G::HD, C = G::C, LPH = G::LPH, LPE = G::LPE, EPW = G::EPW;
    extern __shared__ float smem[];
    const AttnCommon& c = a.c;
    float* s_gate = smem;
    float* s_bias = smem + (c.score == SCORE_GATED ? c.T * HD : 0);
    load_tables(c, s_gate, s_bias);
    const bool gated = c.score == SCORE_GATED, biased = c.score == SCORE_BIASED;
    uint4* ring = reinterpret_cast<uint4*>(smem + ((table_floats(c) + 3) & ~3));            // [NST][2 * CH + 1][kThreads]
    int* tring = reinterpret_cast<int*>(ring + (size_t)NST * (2 * CH + 1) * kThreads);
    const int lane = threadIdx.x & 31;
    const int slot_id = lane / LPE, hl_ = lane - slot_id * LPE;
    const int head = hl_ / LPH, coff = head * 32 + (hl_ - head * LPH) * C;
    const size_t ldq = c.ldq ? (size_t)c.ldq : (size_t)HD, ldk = c.ldk ? (size_t)c.ldk : (size_t)HD;
    const size_t ldr = c.ldr ? (size_t)c.ldr : (size_t)HD, ldo = c.ldo ? (size_t)c.ldo : (size_t)HD;
    const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(a.q) + coff;
    const __nv_bfloat16* rvb = static_cast<const __nv_bfloat16*>(a.row_vec) + coff;

    const int n_warps = gridDim.x * kWarps;
    for (int seg = blockIdx.x * kWarps + (threadIdx.x >> 5); seg < c.plan.n_seg; seg += n_warps) {
        const int colj = c.plan.seg_row[seg], beg = c.plan.seg_beg[seg], end = c.plan.seg_end[seg];
        const int slot = c.plan.seg_slot[seg];
        const __nv_bfloat16* krow = static_cast<const __nv_bfloat16*>(a.k) + (size_t)colj * ldk + coff;
        float kg[C], vf[C], dv[C], dkt[C], dk[C];
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
            float f[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.v) + (size_t)colj * ldk + coff + ch * 8)), f);
#pragma unroll
            for (int x = 0; x < 8; ++x) { vf[ch * 8 + x] = f[x]; dv[ch * 8 + x] = 0.f; dkt[ch * 8 + x] = 0.f; dk[ch * 8 + x] = 0.f; }
        }
        auto load_kg = [&](int t) {          // k (* gate of type t)
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float f[8];
                unpack8(__ldg(reinterpret_cast<const uint4*>(krow + ch * 8)), f);
#pragma unroll
                for (int x = 0; x < 8; ++x) kg[ch * 8 + x] = f[x] * (gated ? s_gate[t * HD + coff + ch * 8 + x] : 1.f);
            }
        };
        auto flush = [&](int t) {            // dk += g_t * sum over the run of ds * q
#pragma unroll
            for (int i = 0; i < C; ++i) { dk[i] = fmaf(gated ? s_gate[t * HD + coff + i] : 1.f, dkt[i], dk[i]); dkt[i] = 0.f; }
        };
        int gt_cached = -1;
        if (!gated) { load_kg(0); gt_cached = 0; }
        const int n_it = (end - beg + EPW - 1) / EPW;
        int rn = 0, tn = 0;
        auto fetch = [&](int g) {
            const int e = min(beg + g * EPW + slot_id, end - 1);
            rn = c.idx[e];
            tn = c.etype ? c.etype[e] : 0;
        };
        auto issue = [&](int g) {
            if (g < n_it) {
                const __nv_bfloat16* qp = qb + (size_t)rn * ldq;
                const __nv_bfloat16* rp = rvb + (size_t)rn * ldr;
                uint4* dst = ring + (size_t)(g % NST) * (2 * CH + 1) * kThreads + threadIdx.x;
#pragma unroll
                for (int ch = 0; ch < CH; ++ch) {
                    cp_async16(dst + (2 * ch) * kThreads, qp + ch * 8);
                    cp_async16(dst + (2 * ch + 1) * kThreads, rp + ch * 8);
                }
                cp_async16(dst + (2 * CH) * kThreads, a.stat + (size_t)rn * H + head);
                tring[(g % NST) * kThreads + threadIdx.x] = tn;
                if (g + 1 < n_it) fetch(g + 1);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if (n_it > 0) fetch(0);
#pragma unroll
        for (int it = 0; it < NST - 1; ++it) issue(it);
        for (int it = 0; it < n_it; ++it) {
            issue(it + NST - 1);
            asm volatile("cp.async.wait_group %0;" ::"n"(NST - 1) : "memory");
            const bool ok = beg + it * EPW + slot_id < end;
            const int t = gated ? tring[(it % NST) * kThreads + threadIdx.x] : 0;
            if (gated && ok && t != gt_cached) {
                if (gt_cached >= 0) flush(gt_cached);
                gt_cached = t;
                load_kg(t);
            }
            const uint4* src = ring + (size_t)(it % NST) * (2 * CH + 1) * kThreads + threadIdx.x;
            uint4 qraw[CH], rraw[CH];
            float s0 = 0.f, s1 = 0.f, d0 = 0.f, d1 = 0.f;
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float qf[8], rf[8];
                qraw[ch] = src[(2 * ch) * kThreads];
                rraw[ch] = src[(2 * ch + 1) * kThreads];
                unpack8(qraw[ch], qf);
                unpack8(rraw[ch], rf);
#pragma unroll
                for (int x = 0; x < 8; x += 2) {
                    s0 = fmaf(qf[x], kg[ch * 8 + x], s0);
                    s1 = fmaf(qf[x + 1], kg[ch * 8 + x + 1], s1);
                    d0 = fmaf(rf[x], vf[ch * 8 + x], d0);
                    d1 = fmaf(rf[x + 1], vf[ch * 8 + x + 1], d1);
                }
            }
            const uint4 sv = src[(2 * CH) * kThreads];
            float s = head_reduce<LPH>(s0 + s1) * c.scale;
            const float dp = head_reduce<LPH>(d0 + d1);
            if (biased) s += s_bias[(c.etype ? tring[(it % NST) * kThreads + threadIdx.x] : 0) * H + head];
            const float p = __expf(fminf(fmaxf(s, c.lo), c.hi));
            const float mask = (s >= c.lo && s <= c.hi) ? 1.f : 0.f;
            const float P = ok ? p * __uint_as_float(sv.z) : 0.f;
            const float ds = P * (dp + __uint_as_float(sv.y)) * mask * c.scale;
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                float qf[8], rf[8];
                unpack8(qraw[ch], qf);
                unpack8(rraw[ch], rf);
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    dv[ch * 8 + x] = fmaf(P, rf[x], dv[ch * 8 + x]);
                    dkt[ch * 8 + x] = fmaf(ds, qf[x], dkt[ch * 8 + x]);
                }
            }
        }
        if (gt_cached >= 0) flush(gt_cached);
#pragma unroll
        for (int off = LPE; off < 32; off <<= 1)
#pragma unroll
            for (int i = 0; i < C; ++i) {
                dk[i] += __shfl_xor_sync(GT_FULL_MASK, dk[i], off);
                dv[i] += __shfl_xor_sync(GT_FULL_MASK, dv[i], off);
            }
        if (slot_id != 0) continue;
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
            float fk[8], fv[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) { fk[x] = dk[ch * 8 + x]; fv[x] = dv[ch * 8 + x]; }
            if (slot >= 0) {
                Vec8<float>::store(c.scratch + (size_t)slot * 2 * HD + coff + ch * 8, fk);
                Vec8<float>::store(c.scratch + (size_t)slot * 2 * HD + HD + coff + ch * 8, fv);
            } else {
                *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.dk) + (size_t)colj * ldo + coff + ch * 8) = pack8(fk);
                *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.dv) + (size_t)colj * ldo + coff + ch * 8) = pack8(fv);
            }
        }
    }
}

inline bool shape_ok(const AttnCommon& c) {
    return c.dtype == DT_BF16 && c.D == 32 && (c.H == 4 || c.H == 8 || c.H == 16) && c.norm == NORM_CLAMPEXP && c.T <= kMaxTypesReg;
}

}  // namespace hl
