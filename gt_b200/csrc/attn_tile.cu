// Tile attention on the 5th-generation tensor cores: the dense part of a block-sparse attention mask.
//
// The gather kernels (attn.cu) move one K row and one V row per edge; where a 128 x 128 tile of the mask holds more than a
// few percent of its entries, loading the tile's 128 K / V rows ONCE and evaluating all 128 x 128 scores on the tensor cores
// is cheaper than gathering.  The host splits a block into such tiles plus a residual edge list; this kernel adds the
// tiles' contribution to the partial results (acc, l, m) that the gather kernels produced for the residual.
//
//   grid  = (row blocks that own at least one tile, head pairs); head dim 32, so a head pair is one 128-byte operand row
//   per half (64 sources) of every column tile of the row block:
//     TMA     K, V pair tiles [64 sources x 64] -> shared memory (two stages)
//     MMA     S_a = Q_a K_a^T, S_b = Q_b K_b^T      (tcgen05.mma, M = 128, N = 64, K = 32; accumulators in tensor memory)
//     8 warps one thread per (row, head): tcgen05.ld of its score row, mask byte -> edge type / no edge, bias, running
//             maximum (softmax) or clamp (clamp-exp), exp, row sum; P as bf16 into shared memory in the operand layout
//     MMA     O_a += P_a V, O_b += P_b V            (M = 128, N = 64, K = 64; the 32 columns of the other head are unused)
//   epilogue: O and the row sums are merged into (acc, l, m) in global memory (log-sum-exp merge for softmax, plain sum
//   for clamp-exp).  A (row block, head pair) is owned by exactly one CTA, so the merge needs no atomics.
//
// Every wait is bounded (status codes 8 producer, 9 MMA, 10 softmax warps); on expiry the CTA drains its copies, releases
// its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.h"
#include "tc05.cuh"

namespace gt {
namespace {

constexpr int TT = 128;                                   // tile edge in the plan (rows = destinations, columns = sources)
constexpr int HC = 64;                                    // sources per step: a tile is processed as two half tiles
constexpr int kTileThreads = 320;                         // warp 0 TMA, warp 1 MMA, warps 2-5 head a, warps 6-9 head b
constexpr int KV_STAGES = 2;
constexpr uint32_t kTileTmemCols = 256;                   // S_a 0..63, S_b 64..127, O_a 128..191, O_b 192..255
constexpr uint32_t COL_S = 0, COL_O = 128;
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;

// 80 KB of shared memory and 256 tensor-memory columns per CTA: two CTAs share an SM, so one CTA's loads, MMAs and epilogue
// overlap the other's softmax arithmetic.
struct __align__(1024) TileStorage {
    __nv_bfloat16 q[TT * 64];                             // [128 rows][2 heads x 32]: 128-byte rows, 128-byte swizzle
    __nv_bfloat16 k[KV_STAGES][HC * 64];                  // [64 sources][2 heads x 32]
    __nv_bfloat16 v[KV_STAGES][HC * 64];
    __nv_bfloat16 p[2][TT * HC];                          // [head][128 rows x 64 sources]: K-major A operand of P V
    uint64_t q_full, kv_full[KV_STAGES], kv_empty[KV_STAGES], s_full, p_full, o_full;
    float bias[2][16];                                    // log2(e) x bias of (edge type, head of the pair); zero without bias
    float wt[2][256];                                     // biased softmax: 2^(bias2 - max bias2) per mask byte, 0 for "no edge"
    float bmax[2];                                        // max over types of log2(e) x bias
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float ex2f(float x) {          // 2^x, 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t mask_byte(const uint32_t (&mw)[16], int col) { return (mw[col >> 2] >> ((col & 3) * 8)) & 255u; }

// Scores are handled in the base-2 domain: s2 = log2(e) * (scale * q.k + bias), weights 2^(s2 - m2).  The row maxima leave
// the kernel in natural units (m = ln 2 * m2).
template <bool BIASED, bool SOFTMAX>
__global__ void __launch_bounds__(kTileThreads, 2) attn_tile_fwd_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                        const __grid_constant__ CUtensorMap map_k,
                                                                        const __grid_constant__ CUtensorMap map_v, AttnTileArgs a) {
    extern __shared__ uint8_t smem_raw[];
    TileStorage& sh = *reinterpret_cast<TileStorage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rb = a.rb_ids[blockIdx.x];
    const int t_beg = a.rb_ptr[blockIdx.x];
    const int nh = 2 * (a.rb_ptr[blockIdx.x + 1] - t_beg);                   // half tiles of this row block
    const int hp = blockIdx.y;
    volatile int* abort_flag = &sh.abort_flag;

    if (threadIdx.x == 0) {
        sh.abort_flag = 0;
        mbar_init(&sh.q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&sh.kv_full[s], 1); mbar_init(&sh.kv_empty[s], 1); }
        mbar_init(&sh.s_full, 1);
        mbar_init(&sh.p_full, 8);                         // one arrival per softmax warp
        mbar_init(&sh.o_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&sh.tmem_base, kTileTmemCols);
    if (warp == 2) {
        const int t = lane & 15, h = lane >> 4;
        const float b2 = (BIASED && a.bias != nullptr && t < a.T) ? kLog2e * a.bias[t * a.H + blockIdx.y * 2 + h] : 0.f;
        sh.bias[h][t] = b2;
        if (BIASED && SOFTMAX) {
            // exp(s + b_t - m) = exp(s - m') * 2^(b2_t - max b2) with m' = m - max b: the per-type factor comes from a table that
            // is indexed with the mask byte itself and holds 0 for "no edge", so the weights need no validity test
            float bm = (t < a.T) ? b2 : -INFINITY;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(GT_FULL_MASK, bm, o));
            if (t == 0) sh.bmax[h] = bm;
            for (int i = t; i < 256; i += 16) sh.wt[h][i] = (i < a.T) ? ex2f(kLog2e * a.bias[i * a.H + blockIdx.y * 2 + h] - bm) : 0.f;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;

    if (nh > 0) {
        if (warp == 0 && lane == 0) {
            // ---- TMA producer ----
            mbar_expect_tx(&sh.q_full, TT * 64 * 2);
            tma_load_2d(sh.q, &map_q, hp * 64, rb * TT, &sh.q_full);
            int issued = 0;
            for (int j = 0; j < nh; ++j) {
                const int s = j % KV_STAGES;
                if (!mbar_wait(&sh.kv_empty[s], ((j / KV_STAGES) & 1) ^ 1, abort_flag, a.status, 8)) break;
                const int src0 = a.tile_cb[t_beg + (j >> 1)] * TT + (j & 1) * HC;
                mbar_expect_tx(&sh.kv_full[s], 2 * HC * 64 * 2);
                tma_load_2d(sh.k[s], &map_k, hp * 64, src0, &sh.kv_full[s]);
                tma_load_2d(sh.v[s], &map_v, hp * 64, src0, &sh.kv_full[s]);
                issued = j + 1;
            }
            if (*abort_flag) {                            // copies in flight must land before the CTA may exit
                const long long t0 = clock64();
                while (!mbar_try_wait(&sh.q_full, 0) && clock64() - t0 < kWaitCycles) {}
                for (int j = (issued > KV_STAGES ? issued - KV_STAGES : 0); j < issued; ++j) {
                    const long long t1 = clock64();
                    while (!mbar_try_wait(&sh.kv_full[j % KV_STAGES], (j / KV_STAGES) & 1) && clock64() - t1 < kWaitCycles) {}
                }
            }
        } else if (warp == 1 && lane == 0) {
            // ---- MMA issuer ----
            const uint32_t idesc_s = make_idesc(TT, HC, 0, 0);        // Q K^T: both operands K-major
            const uint32_t idesc_o = make_idesc(TT, 64, 0, 1);        // P V: P K-major, V MN-major (features contiguous)
            bool okay = mbar_wait(&sh.q_full, 0, abort_flag, a.status, 9);
            const uint32_t q_addr = smem_u32(sh.q);
            for (int j = 0; j < nh && okay; ++j) {
                const int s = j % KV_STAGES;
                okay = mbar_wait(&sh.kv_full[s], (j / KV_STAGES) & 1, abort_flag, a.status, 9);
                if (!okay) break;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(sh.k[s]), v_addr = smem_u32(sh.v[s]);
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks)        // head h occupies bytes [64 h, 64 h + 64) of every 128-byte row
                        umma_bf16(tmem + COL_S + h * HC, make_desc(q_addr + h * 64 + ks * 32, 16, 1024),
                                  make_desc(k_addr + h * 64 + ks * 32, 16, 1024), idesc_s, ks != 0);
                umma_commit(&sh.s_full);
                okay = mbar_wait(&sh.p_full, j & 1, abort_flag, a.status, 9);
                if (!okay) break;
                tc_fence_after();
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t p_addr = smem_u32(sh.p[h]);
#pragma unroll
                    for (int ks = 0; ks < HC / 16; ++ks)  // 16 sources per step: 32 bytes along a P row, V rows [16 ks, 16 ks + 16)
                        umma_bf16(tmem + COL_O + h * 64, make_desc(p_addr + ks * 32, 16, 1024),
                                  make_desc(v_addr + ks * 2048, HC * 128, 1024), idesc_o, (j | ks) != 0);
                }
                umma_commit(&sh.kv_empty[s]);
                umma_commit(&sh.o_full);
            }
        } else if (warp >= 2) {
            // ---- softmax warps: thread = (row, head) ----
            const int hsel = (warp - 2) >> 2;             // 0: first head of the pair, 1: second
            const int quad = warp & 3;                    // tensor-memory lanes [32 quad, 32 quad + 32)
            const int r = quad * 32 + lane;
            const long long grow = (long long)rb * TT + r;
            const int head = hp * 2 + hsel;
            const float* sb = sh.bias[hsel];              // masked entries carry type 255: index with & 15, value unused
            const float* wtab = sh.wt[hsel];
            const float c2 = a.scale * kLog2e, lo2 = a.lo * kLog2e, hi2 = a.hi * kLog2e;
            const uint32_t s_taddr = tmem + COL_S + hsel * HC + ((uint32_t)(quad * 32) << 16);
            const uint32_t o_taddr = tmem + COL_O + hsel * 64 + hsel * 32 + ((uint32_t)(quad * 32) << 16);
            uint8_t* p_row = reinterpret_cast<uint8_t*>(sh.p[hsel]) + r * 128;
            float l_run = 0.f, m_run = SOFTMAX ? -INFINITY : 0.f;             // m_run in the base-2 domain
            // the epilogue reads and rewrites this thread's 128-byte slice of acc: start fetching it now
            if (grow < a.n_rows) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.acc + grow * a.acc_stride + head * 32));
            bool okay = true;
            for (int j = 0; j < nh && okay; ++j) {
                uint32_t mw[16];                          // this row's 64 mask bytes of the half tile
                {
                    const uint4* mp = reinterpret_cast<const uint4*>(a.mask + ((size_t)(t_beg + (j >> 1)) * TT + r) * TT + (j & 1) * HC);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 u = __ldg(mp + i);
                        mw[4 * i] = u.x; mw[4 * i + 1] = u.y; mw[4 * i + 2] = u.z; mw[4 * i + 3] = u.w;
                    }
                }
                okay = __all_sync(GT_FULL_MASK, mbar_wait(&sh.s_full, j & 1, abort_flag, a.status, 10));   // warp-uniform: aligned loads follow
                if (!okay) break;
                tc_fence_after();
                float m_new = m_run, corr = 1.f;
                if (SOFTMAX) {
                    float mx = -INFINITY;
#pragma unroll
                    for (int c0 = 0; c0 < HC; c0 += 16) {
                        uint32_t sr[16];
                        tmem_ld16(s_taddr + c0, sr);
#pragma unroll
                        for (int x = 0; x < 16; ++x) {
                            const uint32_t t = mask_byte(mw, c0 + x);
                            const float s = __uint_as_float(sr[x]) * c2;       // biased scores: the bias offset is a row constant here
                            mx = (t != 255u) ? fmaxf(mx, s) : mx;
                        }
                    }
                    m_new = fmaxf(m_run, mx);
                    corr = (m_run == -INFINITY) ? 0.f : ex2f(m_run - m_new);
                    // the second pass extracts the types again: without this the 64 bias values of the first pass stay live
                    // across the waits below and spill
#pragma unroll
                    for (int i = 0; i < 16; ++i) asm volatile("" : "+r"(mw[i]));
                }
                if (j > 0) {                              // P V of the previous step done: P may be overwritten, O is stable
                    okay = __all_sync(GT_FULL_MASK, mbar_wait(&sh.o_full, (j - 1) & 1, abort_flag, a.status, 10));
                    if (!okay) break;
                    tc_fence_after();
                    if (SOFTMAX && __any_sync(GT_FULL_MASK, corr != 1.f)) {
                        uint32_t orow[32];
                        tmem_ld32(o_taddr, orow);
#pragma unroll
                        for (int x = 0; x < 32; ++x) orow[x] = __float_as_uint(__uint_as_float(orow[x]) * corr);
                        tmem_st32(o_taddr, orow);
                    }
                }
                l_run *= corr;
                // a row without an edge so far has m_new = -inf: its weights are all masked, any finite offset will do
                const float m_off = (SOFTMAX && m_new != -INFINITY) ? m_new : 0.f;
#pragma unroll
                for (int c0 = 0; c0 < HC; c0 += 16) {
                    uint32_t sr[16];
                    tmem_ld16(s_taddr + c0, sr);
                    if (a.dbg_s && blockIdx.x == 0 && blockIdx.y == 0 && j < 2) {
#pragma unroll
                        for (int x = 0; x < 16; ++x) a.dbg_s[((size_t)hsel * TT + r) * TT + j * HC + c0 + x] = __uint_as_float(sr[x]);
                    }
#pragma unroll
                    for (int i = 0; i < 2; ++i) {         // eight weights -> one 16-byte chunk of the P row
                        uint32_t pk[4];
#pragma unroll
                        for (int x = 0; x < 8; x += 2) {
                            float e[2];
#pragma unroll
                            for (int y = 0; y < 2; ++y) {
                                const uint32_t t = mask_byte(mw, c0 + i * 8 + x + y);
                                const float raw = __uint_as_float(sr[i * 8 + x + y]);
                                if (BIASED && SOFTMAX) {
                                    // entries without an edge may exceed the row maximum: cap the exponent, their factor is 0
                                    e[y] = ex2f(fminf(fmaf(raw, c2, -m_off), 0.f)) * wtab[t];
                                } else {
                                    float s;
                                    if (SOFTMAX) s = fmaf(raw, c2, -m_off);
                                    else s = fminf(fmaxf(BIASED ? fmaf(raw, c2, sb[t & 15u]) : raw * c2, lo2), hi2);
                                    e[y] = (t != 255u) ? ex2f(s) : 0.f;
                                }
                                l_run += e[y];
                            }
                            const __nv_bfloat162 h2 = __floats2bfloat162_rn(e[0], e[1]);
                            pk[x >> 1] = *reinterpret_cast<const uint32_t*>(&h2);
                        }
                        *reinterpret_cast<uint4*>(p_row + ((((c0 >> 3) + i) ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
                m_run = m_new;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes of P -> visible to the MMA
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh.p_full);
            }
            if (okay) okay = __all_sync(GT_FULL_MASK, mbar_wait(&sh.o_full, (nh - 1) & 1, abort_flag, a.status, 10));
            if (okay) {
                tc_fence_after();
                uint32_t orow[32];
                tmem_ld32(o_taddr, orow);
                if (grow < a.n_rows && l_run > 0.f) {
                    float* accp = a.acc + grow * a.acc_stride + head * 32;
                    float* lp = a.l + grow * a.l_stride + head;
                    const float lg = *lp;
                    float wa = 1.f, wb = 1.f;
                    if (SOFTMAX) {
                        const float mt = (m_run + (BIASED ? sh.bmax[hsel] : 0.f)) * kLn2, mg = a.m[grow * a.H + head];
                        float mo = mt;
                        if (lg == 0.f) wa = 0.f;
                        else { mo = fmaxf(mg, mt); wa = __expf(mg - mo); wb = __expf(mt - mo); }
                        a.m[grow * a.H + head] = mo;
                    }
                    *lp = wa * lg + wb * l_run;
#pragma unroll
                    for (int x = 0; x < 32; x += 4) {
                        float4 g = *reinterpret_cast<const float4*>(accp + x);
                        g.x = wa * g.x + wb * __uint_as_float(orow[x]);
                        g.y = wa * g.y + wb * __uint_as_float(orow[x + 1]);
                        g.z = wa * g.z + wb * __uint_as_float(orow[x + 2]);
                        g.w = wa * g.w + wb * __uint_as_float(orow[x + 3]);
                        *reinterpret_cast<float4*>(accp + x) = g;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTileTmemCols);
}

template <bool BIASED, bool SOFTMAX>
int launch_tile(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnTileArgs& a, cudaStream_t s) {
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(attn_tile_fwd_kernel<BIASED, SOFTMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(TileStorage) + 1024));
        attr = true;
    }
    dim3 grid(a.n_rb, a.H / 2);
    attn_tile_fwd_kernel<BIASED, SOFTMAX><<<grid, kTileThreads, sizeof(TileStorage) + 1024, s>>>(mq, mk, mv, a);
    return (int)cudaGetLastError();
}

}  // namespace

bool attn_tile_supported(int H, int D, int T) { return D == 32 && H >= 2 && (H % 2) == 0 && T <= 15; }

int attn_tile_fwd(const AttnTileArgs& a, const void* q, const void* k, const void* v, long long ldq, long long ldk, cudaStream_t s) {
    if (!attn_tile_supported(a.H, 32, a.T) || a.n_rb <= 0) return a.n_rb == 0 ? 0 : -3;
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15)) return -2;
    if ((ldq % 8) || (ldk % 8) || (a.acc_stride % 4) || (reinterpret_cast<uintptr_t>(a.acc) & 15) || (reinterpret_cast<uintptr_t>(a.mask) & 15))
        return -2;
    CUtensorMap mq, mk, mv;
    if (!make_map(&mq, q, a.n_rows, a.H * 32, (int)ldq, TT, 64)) return -1;
    if (!make_map(&mk, k, a.n_cols, a.H * 32, (int)ldk, HC, 64)) return -1;
    if (!make_map(&mv, v, a.n_cols, a.H * 32, (int)ldk, HC, 64)) return -1;
    const bool biased = a.score == SCORE_BIASED && a.bias != nullptr, softmax = a.norm == NORM_SOFTMAX;
    if (biased) return softmax ? launch_tile<true, true>(mq, mk, mv, a, s) : launch_tile<true, false>(mq, mk, mv, a, s);
    return softmax ? launch_tile<false, true>(mq, mk, mv, a, s) : launch_tile<false, false>(mq, mk, mv, a, s);
}

}  // namespace gt
