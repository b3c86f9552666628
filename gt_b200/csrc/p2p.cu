// Collectives written as kernels over peer memory (NVLink 5 / NVSwitch): every rank exposes buffers of a symmetric heap,
// and a kernel on the *receiving* GPU reads exactly the bytes it needs from the owners' memory (receiver-driven pull).
// There is no packing step, no send/recv matching and no intermediate copy; reductions accumulate in fp32 in a fixed peer
// order (deterministic).  This is the sm_100a replacement of the reference's NVSHMEM pull collectives
// (gt3d/gt3d/dist/pullcomm/pullcomm.cu:50-108) and of its all-to-all-v sparse collectives.
//
// Ordering between ranks uses epoch flags that live in the symmetric heap: after a rank's producer kernels,
// `signal_peers` publishes the epoch with a system-scope release store into every peer's flag array; `wait_flags` spins
// (bounded) with system-scope acquire loads until every peer has published it.  On expiry the kernel records the peer in
// the status word and returns, so the context stays usable and the host can raise.
#include "common.cuh"
#include "kernels.h"

namespace gt {
namespace {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void signal_kernel(int* const* peer_flags, int n_peers, int my_index, int value) {
    __threadfence_system();
    int p = threadIdx.x;
    if (p < n_peers) st_release_sys(peer_flags[p] + my_index, value);
}

__global__ void wait_kernel(const int* my_flags, int n_peers, int value, long long max_spins, int* status) {
    int p = threadIdx.x;
    if (p >= n_peers) return;
    long long spins = 0;
    while (ld_acquire_sys(my_flags + p) < value) {
        if (++spins > max_spins) {
            atomicExch(status, 100 + p);
            return;
        }
        __nanosleep(64);
    }
}

// Group barrier whose epoch lives in device memory: the kernel itself advances the counter, so the same captured kernel is
// correct on every replay of a CUDA graph.  Thread 0 bumps the epoch, every thread p < n publishes it to peer p (release,
// system scope) and then waits (bounded) until peer p has published the same epoch to this rank.
__global__ void barrier_kernel(int* const* peer_flags, const int* my_flags, int* counter, int n_peers, int my_index,
                               long long max_spins, int* status) {
    __shared__ int epoch;
    if (threadIdx.x == 0) { epoch = *counter + 1; *counter = epoch; }
    __syncthreads();
    __threadfence_system();
    const int p = threadIdx.x;
    if (p >= n_peers) return;
    st_release_sys(peer_flags[p] + my_index, epoch);
    long long spins = 0;
    while (ld_acquire_sys(my_flags + p) < epoch) {
        if (++spins > max_spins) {
            atomicExch(status, 100 + p);
            return;
        }
        __nanosleep(32);
    }
}

// warp per row: out[k] = peers[owner[k]][row[k]]
__global__ void pull_gather_kernel(const void* const* peers, const int* owner, const int* row, uint8_t* out, int n, int row_bytes) {
    const int warps = (blockDim.x >> 5) * gridDim.x;
    const int lane = threadIdx.x & 31;
    const int vec = row_bytes >> 4;
    for (int k = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); k < n; k += warps) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(peers[owner[k]]) + (size_t)row[k] * row_bytes);
        uint4* dst = reinterpret_cast<uint4*>(out + (size_t)k * row_bytes);
        for (int i = lane; i < vec; i += 32) dst[i] = src[i];
    }
}

// warp per owned row: fp32 sum over the peers (fixed order) of the partial rows they hold for it
template <typename T>
__global__ void pull_reduce_kernel(const void* const* peers, int n_peers, const int* src, T* out, int n_rows, int width) {
    const int warps = (blockDim.x >> 5) * gridDim.x;
    const int lane = threadIdx.x & 31;
    const int nch = width >> 3;
    for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n_rows; r += warps) {
        for (int c0 = 0; c0 < nch; c0 += 32) {
            const int ch = c0 + lane;
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int p = 0; p < n_peers; ++p) {
                const int s = src[(size_t)p * n_rows + r];
                if (s >= 0 && ch < nch) {
                    float v[8];
                    Vec8<T>::load(static_cast<const T*>(peers[p]) + (size_t)s * width + (ch << 3), v);
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[k] += v[k];
                }
            }
            if (ch < nch) Vec8<T>::store(out + (size_t)r * width + (ch << 3), acc);
        }
    }
}

// dense all-gather by peer reads: out[p * chunk + i] = peers[p][i]
__global__ void pull_all_gather_kernel(const void* const* peers, int n_peers, uint4* out, long long chunk_vec) {
    const long long total = chunk_vec * n_peers;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int p = (int)(i / chunk_vec);
        const long long o = i - p * chunk_vec;
        out[i] = static_cast<const uint4*>(peers[p])[o];
    }
}

// dense reduce-scatter by peer reads: out[i] = sum_p peers[p][my_index * chunk + i]
template <typename T>
__global__ void pull_reduce_scatter_kernel(const void* const* peers, int n_peers, int my_index, T* out, long long chunk_elems) {
    const long long nch = chunk_elems >> 3;
    for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x; c < nch; c += (long long)gridDim.x * blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int p = 0; p < n_peers; ++p) {
            float v[8];
            Vec8<T>::load(static_cast<const T*>(peers[p]) + my_index * chunk_elems + (c << 3), v);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += v[k];
        }
        Vec8<T>::store(out + (c << 3), acc);
    }
}

// one-shot all-reduce by peer reads (every rank reads every buffer): small / latency-bound payloads such as gradients
template <typename T>
__global__ void pull_all_reduce_kernel(const void* const* peers, int n_peers, T* out, long long n) {
    const long long nch = n >> 3;
    for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x; c < nch; c += (long long)gridDim.x * blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int p = 0; p < n_peers; ++p) {
            float v[8];
            Vec8<T>::load(static_cast<const T*>(peers[p]) + (c << 3), v);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += v[k];
        }
        Vec8<T>::store(out + (c << 3), acc);
    }
}

// Ulysses all-to-all by peer reads, both directions, in 16-byte units.
//   to_heads: out[p * rows + r][:]              = peers[p][r * (n_peers * slab) + me * slab : +slab]     (rows of peer p, my head slab)
//   to_rows : out[r][p * slab : (p + 1) * slab] = peers[p][(me * rows + r) * slab : +slab]               (my rows, peer p's head slab)
// The transposes that the NCCL path does with extra copies happen in the address arithmetic of the reads.
__global__ void pull_all_to_all_kernel(const void* const* peers, int n_peers, int me, long long rows, int slab_vec, int to_heads,
                                       uint4* out) {
    const long long total = rows * n_peers * slab_vec;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int v = (int)(i % slab_vec);
        const long long t = i / slab_vec;
        if (to_heads) {
            const long long r = t % rows;
            const int p = (int)(t / rows);
            out[i] = static_cast<const uint4*>(peers[p])[(r * n_peers + me) * slab_vec + v];
        } else {
            const int p = (int)(t % n_peers);
            const long long r = t / n_peers;
            out[i] = static_cast<const uint4*>(peers[p])[((long long)me * rows + r) * slab_vec + v];
        }
    }
}

// ---- epoch channels: signal without waiting, wait inside the consumer -------------------------------------------------
// A channel is {flags[n] in every member's symmetric heap, one counter in this rank's memory}.  `signal` bumps the counter and
// publishes the new epoch into slot `my_index` of every member's flag array (release, system scope) after this stream's earlier
// kernels (the producers) have completed; it never waits.  A consumer kernel later reads the SAME counter (its own rank signalled
// the same use earlier in stream order) and waits, bounded, until the members it reads from have published that epoch.  The
// counter lives in device memory and is advanced by the kernel itself, so a captured CUDA graph replays correctly.
struct PeerFlags { int* p[8]; };

__global__ void channel_signal_kernel(PeerFlags peers, int n_peers, int my_index, int* counter) {
    __shared__ int epoch;
    if (threadIdx.x == 0) { epoch = *counter + 1; *counter = epoch; }
    __syncthreads();
    __threadfence_system();
    const int p = threadIdx.x;
    if (p < n_peers) st_release_sys(peers.p[p] + my_index, epoch);
}

// Block-wide bounded wait: thread p < n_peers polls flags[p] until it reaches *counter.  Returns after a __syncthreads().
__device__ __forceinline__ void block_wait_channel(const int* flags, const int* counter, int n_peers, long long max_spins, int* status) {
    if (flags != nullptr && (int)threadIdx.x < n_peers) {
        const int want = *counter;
        long long spins = 0;
        while (ld_acquire_sys(flags + threadIdx.x) < want) {
            if (++spins > max_spins) { atomicExch(status, 100 + (int)threadIdx.x); break; }
            __nanosleep(40);
        }
    }
    __syncthreads();
}

// Owner side of the reduce-scatter that the attention / aggregation kernels push into: sums the n_slots bf16 payload rows
// [acc (HD) | l (Hp) | agg (d_agg)] that the row group wrote into this rank's slots and unpacks them (fp32 acc and l, bf16 agg).
__global__ void sum_payload_kernel(const __nv_bfloat16* __restrict__ slots, int n_slots, long long rows, int W, int HD, int H, int l_off,
                                   int agg_off, int d_agg, float* __restrict__ acc, float* __restrict__ l, __nv_bfloat16* __restrict__ agg,
                                   const int* flags, const int* counter, long long max_spins, int* status) {
    block_wait_channel(flags, counter, n_slots, max_spins, status);
    const int cpr = W >> 3;                                   // 8-element chunks per payload row
    const long long total = rows * cpr;
    const long long slot_elems = rows * (long long)W;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cpr;
        const int c = (int)(i - r * cpr) << 3;
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int p = 0; p < n_slots; ++p) {
            float v[8];
            Vec8<__nv_bfloat16>::load(slots + (size_t)p * slot_elems + (size_t)r * W + c, v);
#pragma unroll
            for (int k = 0; k < 8; ++k) s[k] += v[k];
        }
        if (c < HD) {
            Vec8<float>::store(acc + (size_t)r * HD + c, s);
        } else if (c >= l_off && c < l_off + H) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (c - l_off + k < H) l[(size_t)r * H + (c - l_off) + k] = s[k];
        } else if (agg != nullptr && c >= agg_off && c < agg_off + d_agg) {
            Vec8<__nv_bfloat16>::store(agg + (size_t)r * d_agg + (c - agg_off), s);
        }
    }
}

// Backward mirror (an all-gather over the row group, fused with the unpacking): every owner has published the bf16 payload
// gradient [dacc (HD) | dl (Hp) | dagg (d_agg)] of its rows; this rank reads the rows of its whole row block from the owners'
// memory and writes what the backward kernels consume: the row vector (bf16 dacc), the per-(row, head) statistics
// {m = 0, row bias = dl, p scale = 1, 0} and the aggregation gradient.
__global__ void pull_unpack_kernel(PeerFlags src, int n_peers, long long rows_per_peer, int W, int HD, int H, int l_off, int agg_off,
                                   int d_agg, __nv_bfloat16* __restrict__ row_vec, float4* __restrict__ stat, __nv_bfloat16* __restrict__ dagg,
                                   const int* flags, const int* counter, long long max_spins, int* status) {
    block_wait_channel(flags, counter, n_peers, max_spins, status);
    const int cpr = W >> 3;
    const long long total = rows_per_peer * n_peers * cpr;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / cpr;
        const int c = (int)(i - row * cpr) << 3;
        const int p = (int)(row / rows_per_peer);
        const long long r = row - (long long)p * rows_per_peer;
        const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src.p[p]) + (size_t)r * W + c);
        if (c < HD) {
            *reinterpret_cast<uint4*>(row_vec + (size_t)row * HD + c) = raw;
        } else if (c >= l_off && c < l_off + H) {
            float v[8];
            Vec8<__nv_bfloat16>::unpack(raw, v);
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (c - l_off + k < H) stat[(size_t)row * H + (c - l_off) + k] = make_float4(0.f, v[k], 1.f, 0.f);
        } else if (dagg != nullptr && c >= agg_off && c < agg_off + d_agg) {
            *reinterpret_cast<uint4*>(dagg + (size_t)row * d_agg + (c - agg_off)) = raw;
        }
    }
}

// One-GPU form of the same preparation: dacc fp32 [n, HD] -> bf16 row vector, dl fp32 [n, H] -> statistics.
__global__ void attn_bwd_prep_kernel(const float* __restrict__ dacc, const float* __restrict__ dl, long long n, int HD, int H,
                                     __nv_bfloat16* __restrict__ row_vec, float4* __restrict__ stat) {
    const int cpr = (HD >> 3) + ((H + 7) >> 3);
    const long long total = n * cpr;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cpr;
        const int c = (int)(i - r * cpr);
        if (c < (HD >> 3)) {
            float v[8];
            Vec8<float>::load(dacc + (size_t)r * HD + (c << 3), v);
            Vec8<__nv_bfloat16>::store(row_vec + (size_t)r * HD + (c << 3), v);
        } else {
            const int h0 = (c - (HD >> 3)) << 3;
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (h0 + k < H) stat[(size_t)r * H + h0 + k] = make_float4(0.f, dl[(size_t)r * H + h0 + k], 1.f, 0.f);
        }
    }
}

// out (+)= sum of the n_slots bf16 slots after the members of the channel have signalled (GEMM -> reduce-scatter epilogue)
template <typename TO>
__global__ void sum_slots_wait_kernel(const __nv_bfloat16* __restrict__ slots, int n_slots, long long slot_elems, TO* __restrict__ out,
                                      int accumulate, const int* flags, const int* counter, long long max_spins, int* status) {
    block_wait_channel(flags, counter, n_slots, max_spins, status);
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

// Two-shot all-reduce of the flat fp32 gradient buffer over the data-parallel group, as ONE kernel per rank: after the group has
// signalled "gradients final", rank r sums slice r of every member's buffer (peer reads, fixed order, fp32) and stores the
// reduced slice into EVERY member's result buffer (peer stores): 2 n bytes cross this rank's links instead of P n for the
// one-shot form, and no barrier kernel runs.  A second signal / wait pair tells the optimizer that all slices have landed.
__global__ void allreduce_two_shot_kernel(PeerFlags src, PeerFlags dst, int n_peers, int me, long long n, long long chunk,
                                          const int* flags, const int* counter, long long max_spins, int* status) {
    block_wait_channel(flags, counter, n_peers, max_spins, status);
    const long long lo = (long long)me * chunk, hi = lo + chunk < n ? lo + chunk : n;
    for (long long i = lo / 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < hi / 4; i += (long long)gridDim.x * blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < n_peers; ++p) {
            const float4 v = reinterpret_cast<const float4*>(src.p[p])[i];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        for (int p = 0; p < n_peers; ++p) reinterpret_cast<float4*>(dst.p[p])[i] = acc;
    }
}

// bounded wait of one block on a channel (used where the consumer is a library-free kernel that cannot take the wait itself)
__global__ void channel_wait_kernel(const int* flags, const int* counter, int n_peers, long long max_spins, int* status) {
    block_wait_channel(flags, counter, n_peers, max_spins, status);
}

int grid_for(long long items, int per_block) {
    long long b = (items + per_block - 1) / per_block;
    long long cap = 148LL * 8;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

void signal_peers(int* const* peer_flags, int n_peers, int my_index, int value, cudaStream_t s) {
    signal_kernel<<<1, 32, 0, s>>>(peer_flags, n_peers, my_index, value);
}

void wait_flags(const int* my_flags, int n_peers, int value, long long max_spins, int* status, cudaStream_t s) {
    wait_kernel<<<1, 32, 0, s>>>(my_flags, n_peers, value, max_spins, status);
}

void group_barrier(int* const* peer_flags, const int* my_flags, int* counter, int n_peers, int my_index, long long max_spins,
                   int* status, cudaStream_t s) {
    barrier_kernel<<<1, 32, 0, s>>>(peer_flags, my_flags, counter, n_peers, my_index, max_spins, status);
}

void channel_signal(int* const* peer_flags, int n_peers, int my_index, int* counter, cudaStream_t s) {
    PeerFlags pf{};
    for (int p = 0; p < n_peers && p < 8; ++p) pf.p[p] = peer_flags[p];
    channel_signal_kernel<<<1, 32, 0, s>>>(pf, n_peers, my_index, counter);
}

void sum_payload(const void* slots, int n_slots, long long rows, int W, int HD, int H, int l_off, int agg_off, int d_agg, float* acc, float* l,
                 void* agg, const int* flags, const int* counter, long long max_spins, int* status, cudaStream_t s) {
    if (rows <= 0) return;
    sum_payload_kernel<<<grid_for(rows * (W / 8), 1024), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(slots), n_slots, rows, W, HD, H, l_off,
                                                                     agg_off, d_agg, acc, l, static_cast<__nv_bfloat16*>(agg), flags, counter,
                                                                     max_spins, status);
}

void pull_unpack(void* const* src, int n_peers, long long rows_per_peer, int W, int HD, int H, int l_off, int agg_off, int d_agg, void* row_vec,
                 void* stat, void* dagg, const int* flags, const int* counter, long long max_spins, int* status, cudaStream_t s) {
    if (rows_per_peer <= 0) return;
    PeerFlags pf{};
    for (int p = 0; p < n_peers && p < 8; ++p) pf.p[p] = static_cast<int*>(src[p]);
    pull_unpack_kernel<<<grid_for(rows_per_peer * n_peers * (W / 8), 1024), 256, 0, s>>>(
        pf, n_peers, rows_per_peer, W, HD, H, l_off, agg_off, d_agg, static_cast<__nv_bfloat16*>(row_vec), static_cast<float4*>(stat),
        static_cast<__nv_bfloat16*>(dagg), flags, counter, max_spins, status);
}

void attn_bwd_prep(const float* dacc, const float* dl, long long n, int HD, int H, void* row_vec, void* stat, cudaStream_t s) {
    if (n <= 0) return;
    attn_bwd_prep_kernel<<<grid_for(n * (HD / 8 + (H + 7) / 8), 1024), 256, 0, s>>>(dacc, dl, n, HD, H, static_cast<__nv_bfloat16*>(row_vec),
                                                                                    static_cast<float4*>(stat));
}

void sum_slots_wait(const void* slots, int n_slots, long long slot_elems, void* out, int out_dtype, int accumulate, const int* flags,
                    const int* counter, long long max_spins, int* status, cudaStream_t s) {
    const long long n8 = slot_elems / 8;
    if (n8 <= 0) return;
    if (out_dtype == DT_BF16)
        sum_slots_wait_kernel<__nv_bfloat16><<<grid_for(n8, 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(slots), n_slots, slot_elems,
                                                                               static_cast<__nv_bfloat16*>(out), accumulate, flags, counter,
                                                                               max_spins, status);
    else
        sum_slots_wait_kernel<float><<<grid_for(n8, 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(slots), n_slots, slot_elems,
                                                                       static_cast<float*>(out), accumulate, flags, counter, max_spins, status);
}

void allreduce_two_shot(void* const* src, void* const* dst, int n_peers, int me, long long n, const int* flags, const int* counter,
                        long long max_spins, int* status, cudaStream_t s) {
    if (n <= 0) return;
    PeerFlags a{}, b{};
    for (int p = 0; p < n_peers && p < 8; ++p) { a.p[p] = static_cast<int*>(src[p]); b.p[p] = static_cast<int*>(dst[p]); }
    long long chunk = (n + n_peers - 1) / n_peers;
    chunk = (chunk + 3) / 4 * 4;
    allreduce_two_shot_kernel<<<grid_for(chunk / 4, 256), 256, 0, s>>>(a, b, n_peers, me, n, chunk, flags, counter, max_spins, status);
}

void channel_wait(const int* flags, const int* counter, int n_peers, long long max_spins, int* status, cudaStream_t s) {
    channel_wait_kernel<<<1, 32, 0, s>>>(flags, counter, n_peers, max_spins, status);
}

void pull_gather_rows(const void* const* peers, const int* owner, const int* row, void* out, int n, int row_bytes, cudaStream_t s) {
    if (n <= 0) return;
    pull_gather_kernel<<<grid_for(n, 8), 256, 0, s>>>(peers, owner, row, static_cast<uint8_t*>(out), n, row_bytes);
}

void pull_reduce_rows(int dtype, const void* const* peers, int n_peers, const int* src, void* out, int n_rows, int width, cudaStream_t s) {
    if (n_rows <= 0) return;
    if (dtype == DT_BF16)
        pull_reduce_kernel<__nv_bfloat16><<<grid_for(n_rows, 8), 256, 0, s>>>(peers, n_peers, src, static_cast<__nv_bfloat16*>(out), n_rows, width);
    else
        pull_reduce_kernel<float><<<grid_for(n_rows, 8), 256, 0, s>>>(peers, n_peers, src, static_cast<float*>(out), n_rows, width);
}

void pull_all_to_all(const void* const* peers, int n_peers, int me, long long rows, long long slab_bytes, bool to_heads, void* out,
                     cudaStream_t s) {
    const long long vecs = rows * n_peers * (slab_bytes / 16);
    if (vecs <= 0) return;
    pull_all_to_all_kernel<<<grid_for(vecs, 1024), 256, 0, s>>>(peers, n_peers, me, rows, (int)(slab_bytes / 16), to_heads ? 1 : 0,
                                                                static_cast<uint4*>(out));
}

void pull_all_gather(const void* const* peers, int n_peers, void* out, long long chunk_bytes, cudaStream_t s) {
    if (chunk_bytes <= 0) return;
    pull_all_gather_kernel<<<grid_for(chunk_bytes / 16 * n_peers, 1024), 256, 0, s>>>(peers, n_peers, static_cast<uint4*>(out), chunk_bytes / 16);
}

void pull_reduce_scatter(int dtype, const void* const* peers, int n_peers, int my_index, void* out, long long chunk_elems, cudaStream_t s) {
    if (chunk_elems <= 0) return;
    if (dtype == DT_BF16)
        pull_reduce_scatter_kernel<__nv_bfloat16><<<grid_for(chunk_elems / 8, 512), 256, 0, s>>>(peers, n_peers, my_index,
                                                                                                  static_cast<__nv_bfloat16*>(out), chunk_elems);
    else
        pull_reduce_scatter_kernel<float><<<grid_for(chunk_elems / 8, 512), 256, 0, s>>>(peers, n_peers, my_index, static_cast<float*>(out), chunk_elems);
}

void pull_all_reduce(int dtype, const void* const* peers, int n_peers, void* out, long long n, cudaStream_t s) {
    if (n <= 0) return;
    if (dtype == DT_BF16)
        pull_all_reduce_kernel<__nv_bfloat16><<<grid_for(n / 8, 512), 256, 0, s>>>(peers, n_peers, static_cast<__nv_bfloat16*>(out), n);
    else
        pull_all_reduce_kernel<float><<<grid_for(n / 8, 512), 256, 0, s>>>(peers, n_peers, static_cast<float*>(out), n);
}

}  // namespace gt
