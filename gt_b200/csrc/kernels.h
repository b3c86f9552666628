// Host-side launch interface of the gt_b200 kernels.  Everything here is plain C++ (no torch headers): the binding
// translates tensors to these PODs, and the launchers enqueue on the given stream and never allocate.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <vector>

namespace gt {

enum Dtype : int { DT_F32 = 0, DT_BF16 = 1 };
enum Score : int { SCORE_DOT = 0, SCORE_GATED = 1, SCORE_BIASED = 2 };
enum Norm : int { NORM_SOFTMAX = 0, NORM_CLAMPEXP = 1 };

// Work list of a pass: one warp per segment (see gt_b200/attention/csr.py).
struct SegPlan {
    const int* seg_row;
    const int* seg_beg;
    const int* seg_end;
    const int* seg_slot;    // -1: the row has one segment; else index of the segment's scratch slot
    int n_seg;
    const int* split_rows;  // rows cut in several segments
    const int* split_ptr;   // their slot ranges
    int n_split;
};

struct AttnCommon {
    int dtype;              // Dtype of q / k / v / row_vec
    int H, D, T;            // heads, head dim, number of edge types (rows of gate / bias)
    int score, norm;
    float scale, lo, hi;
    const int* idx;         // CSR: source column of every entry;  CSC: destination row of every entry
    const int* etype;       // per entry, nullable
    const float* gate;      // [T, H*D] fp32, nullable
    const float* bias;      // [T, H]   fp32, nullable
    SegPlan plan;
    float* scratch;         // [n_slots, scratch_width] fp32
    // row strides in elements, 0 = dense rows of H*D: q (and the q-side of the passes), k / v, row_vec, and the gradient
    // outputs (dq of the row pass, dk / dv of the column pass).  Operands may be column slices of wider matrices.
    long long ldq, ldk, ldr, ldo;
};

struct AttnFwdArgs {
    AttnCommon c;
    const void* q;          // [n_rows, H*D]
    const void* k;          // [n_cols, H*D]  (ignored when peers are given)
    const void* v;
    // receiver-driven pull over NVLink: column j lives in k_peers[j / rows_per_peer] at row j % rows_per_peer
    const void* const* k_peers;
    const void* const* v_peers;
    int rows_per_peer;
    const int* row_map;     // nullable: output row of every plan row (doubly-compressed row lists)
    float* acc; float* l; float* m;   // outputs (m nullable)
    long long acc_stride, l_stride;   // elements between consecutive output rows
    int accumulate;         // add into acc / l instead of overwriting
    // reduce-scatter fused into the epilogue (clamp-exp partials): output row r belongs to rank r / push_rows of the row group and
    // is stored as bf16 [acc | .. | l] into push_slot[owner] + (r % push_rows) * push_ld; acc / l / m are then unused
    int push_n;             // 0 = off, else the number of owners
    void* push_slot[8];
    int push_rows;          // rows per owner
    long long push_ld;      // bf16 elements per payload row
    int push_l_off;         // column of l inside the payload row (multiple of 8)
};

struct AttnBwdRowArgs {
    AttnCommon c;
    const void* q; const void* k; const void* v;
    const void* row_vec;    // [n_rows, H*D] dtype: dacc (partial form) or dO (normalised form)
    const float4* stat;     // [n_rows, H]: {m, row_bias, p_scale, unused}
    const int* row_map;     // nullable
    void* dq;               // [n_rows, H*D] dtype
    int accumulate_dq;      // dq is fp32 and is added to (streamed layer)
    float* dgate_part;      // [n_blocks, T, H*D] per-block partial sums (nullable)
    float* dbias_part;      // [n_blocks, T, H]   (nullable)
    int n_blocks;           // grid size the partial buffers were sized for
    // nullable: [E, H] fp32 score gradients per CSR entry, written by a column pass that ran first.  The row pass then only
    // gathers K rows and accumulates dq += ds * k (no V gather, no recomputation of the weights); v / row_vec / stat are unused.
    const float* ds_in;
};

struct AttnBwdColArgs {
    AttnCommon c;           // idx = destination row of every CSC entry; plan over the columns
    const void* q; const void* k; const void* v;
    const void* row_vec;
    const float4* stat;
    void* dk; void* dv;     // [n_cols, H*D] dtype
    // nullable pair: the pass stores the score gradient of every entry (before the scale factor) at ds_out[pos[e] * H + head],
    // pos = CSR position of CSC entry e, for a row pass that runs afterwards (AttnBwdRowArgs::ds_in)
    float* ds_out;
    const int* pos;
};

int attn_scratch_width_fwd(int H, int D);              // floats per forward slot
void attn_fwd(const AttnFwdArgs& a, cudaStream_t s);
void attn_bwd_row(const AttnBwdRowArgs& a, cudaStream_t s);
void attn_bwd_col(const AttnBwdColArgs& a, cudaStream_t s);
bool attn_shape_supported(int H, int D, int T);

// Dense tiles of a block-sparse mask on the tensor cores (attn_tile.cu): adds the tiles' contribution to partial results.
struct AttnTileArgs {
    int H, T;               // heads (even, head dim 32), edge types (<= 15)
    int score, norm;        // SCORE_DOT or SCORE_BIASED; either normalisation
    float scale, lo, hi;
    const float* bias;      // [T, H] fp32, nullable
    int n_rb;               // row blocks (of 128 destinations) that own at least one tile
    const int* rb_ids;      // [n_rb] row-block index
    const int* rb_ptr;      // [n_rb + 1] range of tiles of every listed row block
    const int* tile_cb;     // [n_tiles] column-block index (of 128 sources)
    const unsigned char* mask;   // [n_tiles, 128, 128] edge type of (row, column), 255 = no edge
    int n_rows, n_cols;
    float* acc; float* l; float* m;      // partial results of the residual edges, updated in place (m only for softmax)
    long long acc_stride, l_stride;
    int* status;            // device status word of the bounded waits
    float* dbg_s;           // nullable: raw scores of the first tile of CTA (0, 0), [2, 128, 128]
};
bool attn_tile_supported(int H, int D, int T);
int attn_tile_fwd(const AttnTileArgs& a, const void* q, const void* k, const void* v, long long ldq, long long ldk, cudaStream_t s);
struct KernelInfo { const char* name; int regs; int local_bytes; int static_smem; int dyn_smem; int blocks_per_sm; };
std::vector<KernelInfo> attn_kernel_info();            // compiled resources of the main attention kernel instances
int attn_status();                                     // nonzero once after a bounded copy wait of an attention kernel expired (synchronises)
int attn_bwd_row_blocks(int n_seg);                    // grid size attn_bwd_row will use for n_seg segments
// sum of per-block partials: out[i] = sum_b part[b, i]
void reduce_partials(const float* part, int n_blocks, int width, float* out, cudaStream_t s, int accumulate = 0);   // accumulate: out += sum

// ---- sparse aggregation ---------------------------------------------------------------------------------------------
struct SpmmArgs {
    int dtype;              // dtype of x / out
    const int* ptr;         // [n_out + 1]
    const int* idx;         // [E]
    const float* w;         // [E]
    const void* x;          // [n_in, d]
    void* out;              // [n_out, d]
    int n_out, d;
    int accumulate;
    int use_plan;           // 1: one warp per plan segment (hub rows are cut and merged through `scratch`), 0: one warp per row
    SegPlan plan;
    float* scratch;         // [n_slots, d] fp32
    long long ldx, ldo;     // row strides of x / out in elements (0 = d): either may be a column slice of a wider matrix
    // reduce-scatter fused into the store: output row r belongs to rank r / push_rows and is written to
    // push_slot[owner] + (r % push_rows) * ldo instead of `out` (push_slot already points at the column of the slice)
    int push_n; void* push_slot[8]; int push_rows;
};
void spmm(const SpmmArgs& a, cudaStream_t s);
// out[r] = sum_{k in [ptr[r], ptr[r+1])} rows[perm[k]]   (deterministic segmented row sum)
void segment_sum_rows(int dtype, const void* rows, const int* perm, const int* ptr, void* out, int n_out, int width, cudaStream_t s);

// ---- row-wise dense kernels -----------------------------------------------------------------------------------------
struct LayerNormArgs {
    int dtype;              // dtype of y / x / out
    const void* y;          // [n, d] branch output (dropout applied to y + ybias)
    const void* x;          // [n, d] residual, nullable
    const float* ybias;     // [d], nullable
    const float* gamma; const float* beta;
    void* out;              // [n, d]
    float* mean_rstd;       // [n, 2] saved statistics (nullable in inference)
    int n, d; float eps;
    float p;                // dropout probability (0 = none)
    const long long* seed;  // device pointer: {seed, offset}
    long long stream_id;    // distinguishes the dropout sites of a step
    // optional fused attention normalisation: y = acc / (l[head] + eps_l) with acc fp32 [n, d], l fp32 [n, H] (y is ignored)
    const float* acc; const float* l; int H; float eps_l;
};
void layer_norm_fwd(const LayerNormArgs& a, cudaStream_t s);
// out = l2normalize(relu(dropout(LayerNorm(h))))  (input stage of the models); stats [n, 3] = mean, rstd, norm
struct PreMpArgs {
    int dtype; const void* h; const float* gamma; const float* beta; void* out; float* stats;
    int n, d; float eps; float p; const long long* seed; long long stream_id; int l2norm;
    const void* dout; void* dh; float* part; int n_blocks;      // backward: part [n_blocks, 2 d] (dgamma | dbeta)
};
// out = x + tab_a[idx_a] (+ tab_b[idx_b]) row-wise (embedding lookups folded into one pass); tables fp32 [*, d]
void embed_add(int dtype, const void* x, const float* tab_a, const long long* idx_a, long long pad_a, const float* tab_b,
               const long long* idx_b, long long pad_b, void* out, long long n, int d, cudaStream_t s);
void embed_add_bwd(int dtype, const void* dout, const long long* idx, long long pad, float* dtab, long long n, int d, cudaStream_t s);
// UniMP gated residual: out = dropout(relu(LN(beta r + (1 - beta) o))), beta = sigmoid(r . wa + o . wb + b); d <= 256
struct GatedResArgs {
    int dtype; const void* r; const void* o; const float* wa; const float* wb; const float* gate_bias;
    const float* gamma; const float* beta; void* out; float* stats;      // stats [n, 3] = mean, rstd, beta
    long long n; int d; float eps; float p; const long long* seed; long long stream_id;
    const void* dout; void* dr; void* d_o; float* part; int part_stride; int n_blocks;   // backward: part [n_blocks, 4 d + 1]
};
void gated_residual(const GatedResArgs& a, bool backward, cudaStream_t s);
int premp_blocks(int n);
void premp(const PreMpArgs& a, bool backward, cudaStream_t s);

struct LayerNormBwdArgs {
    int dtype;
    const void* dout;       // [n, d]
    const void* y; const void* x; const float* ybias;   // forward inputs (recompute z = x + drop(y + ybias))
    const float* gamma;
    const float* mean_rstd;
    void* dy;               // [n, d] dtype (gradient w.r.t. y, dropout mask applied)
    void* dx;               // [n, d] dtype, nullable; accumulate_dx adds dz to it instead of overwriting
    int accumulate_dx;
    float* dgamma_part; float* dbeta_part; float* dybias_part;   // [n_blocks, d] partials, row stride part_stride (dybias nullable)
    int part_stride;
    int n_blocks;
    int n, d; float p; const long long* seed; long long stream_id;
    // fused attention normalisation (see LayerNormArgs): gradients w.r.t. acc [n, d] and l [n, H] instead of dy
    const float* acc; const float* l; int H; float eps_l; float* dacc; float* dl;
};
void layer_norm_bwd(const LayerNormBwdArgs& a, cudaStream_t s);
int layer_norm_bwd_blocks(int n);

// elementwise epilogue used when a GEMM is not fused: out = drop(act(in + bias))
void bias_act_dropout(int dtype, const void* in, const float* bias, void* out, long long n, int d, int act, float p,
                      const long long* seed, long long stream_id, cudaStream_t s);
// dz = dout * act'(in + bias) * dropmask ; optional per-block bias gradient partials
void bias_act_dropout_bwd(int dtype, const void* dout, const void* in, const float* bias, void* dz, long long n, int d, int act,
                          float p, const long long* seed, long long stream_id, float* dbias_part, int n_blocks, cudaStream_t s);
int colsum_blocks(long long n);

// masked softmax cross-entropy: loss_sum += sum_i mask_i * nll_i / denom ; dlogits = mask_i (softmax - onehot) / denom
void cross_entropy_fwd_bwd(int dtype, const void* logits, const long long* labels, const bool* mask, int n, int c, float inv_denom,
                           float* loss, void* dlogits, cudaStream_t s);

// multi-tensor AdamW over a flat fp32 parameter / gradient / moment space with a device-side LR and clip coefficient
struct AdamWArgs {
    float* p; const float* g; float* m; float* v;
    void* p_bf16;           // optional bf16 shadow of the parameters (nullable)
    long long n;
    const float* hyper;     // device: {lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, max_grad_norm, grad_sq_norm}
    const float* decay_mask;// nullable per-element weight-decay multiplier
};
void adamw_step(const AdamWArgs& a, cudaStream_t s);
// sum of squares of g into out[0] (fp32 atomics over block partials)
void sq_norm(const float* g, long long n, float* out, cudaStream_t s);
void cast_f32_to_bf16(const float* in, void* out, long long n, cudaStream_t s);

// packed[r, :] = concat_i seg_i[r, :] with conversion (dir 0), or seg_i[r, :] = packed[r, off_i : off_i + w_i] (dir 1)
struct PackColSeg { void* p; int width; int dtype; int ld; };
struct PackColsArgs {
    PackColSeg seg[4]; int n_seg;
    void* packed; int packed_dtype; int ld_packed; int width;    // width = sum of the segment widths (<= ld_packed)
    long long n_rows; int dir;
};
void pack_cols(const PackColsArgs& a, cudaStream_t s);

// ---- tcgen05 GEMM -----------------------------------------------------------------------------------------------------
// C[M, N] = A[M, K] * B[N, K]^T  (both operands K-major bf16, fp32 accumulation in tensor memory)
struct GemmArgs {
    const void* a; const void* b; void* c;
    int M, N, K;
    int lda, ldb, ldc;      // elements
    int c_dtype;            // DT_BF16 or DT_F32
    const float* bias;      // [N], nullable
    int act;                // 0 none, 1 relu, 2 gelu
    float p; const long long* seed; long long stream_id;   // dropout epilogue
    int accumulate;         // C += result (fp32 C only)
    int* status;            // device status word: nonzero when a bounded wait expired
};
bool gemm_tcgen05_supported(int M, int N, int K, int lda, int ldb, int ldc);
// returns a CUDA error code or 0; fails (-1) when the tensor maps cannot be encoded
int gemm_tcgen05(const GemmArgs& g, cudaStream_t s);
// C[N, K] = A[M, N]^T * B[M, K]  (weight gradients: reduction over the long row dimension, split across CTAs)
struct GemmTNArgs {
    const void* a; const void* b; float* c;   // bf16 inputs, fp32 output
    int M, N, K; int lda, ldb, ldc;
    int accumulate;
    int* status;
};
int gemm_tn_tcgen05(const GemmTNArgs& g, cudaStream_t s);
// Collective-fused GEMMs over peer memory (symmetric heap).  Return 0, a CUDA error code, or a negative "unsupported" code.
//   gather : C = gathered(A) * B^T where rank p's rows of A are read from a_peers[p] by TMA; optional gathered copy of A
//   scatter: row block p of A * B^T is stored into slots[p] (my slot in rank p's staging area); sum_slots adds the slots
// `wait` (nullable): epoch channel of the gathered operand; the kernel waits per peer, inside its TMA producer, until
// flags[p] >= *counter before it touches peer p's rows (no barrier kernel in front of the GEMM).  `self` = this rank's index.
struct GatherWait { const int* flags; const int* counter; long long max_spins; int self; };
int gemm_nt_gather(const GemmArgs& g, const void* const* a_peers, int n_peers, int chunk, void* gathered, cudaStream_t s,
                   const GatherWait* wait = nullptr);
int gemm_nt_scatter(const GemmArgs& g, void* const* slots, int n_peers, int chunk, cudaStream_t s);
void sum_slots(const void* slots, int n_slots, long long slot_elems, void* out, int out_dtype, int accumulate, cudaStream_t s);

// ---- peer-memory kernels (NVLink) ------------------------------------------------------------------------------------
// out[k] = peers[owner[k]][row[k]]  : receiver-driven gather of rows from the peers' buffers
void pull_gather_rows(const void* const* peers, const int* owner, const int* row, void* out, int n, int row_bytes, cudaStream_t s);
// out[r] = sum over peers p (fixed order) of peers[p][src[p * n_rows + r]] for src >= 0 ; fp32 accumulation
void pull_reduce_rows(int dtype, const void* const* peers, int n_peers, const int* src, void* out, int n_rows, int width, cudaStream_t s);
// dense variants: all-gather / reduce-scatter of equal chunks by direct peer reads
void pull_all_gather(const void* const* peers, int n_peers, void* out, long long chunk_bytes, cudaStream_t s);
// Ulysses all-to-all (rows <-> head slabs) by strided peer reads; slab_bytes % 16 == 0
void pull_all_to_all(const void* const* peers, int n_peers, int me, long long rows, long long slab_bytes, bool to_heads, void* out,
                     cudaStream_t s);
void pull_reduce_scatter(int dtype, const void* const* peers, int n_peers, int my_index, void* out, long long chunk_elems, cudaStream_t s);
// out = sum over peers of their buffers (one-shot all-reduce by peer reads), fp32 or bf16 payload with fp32 accumulation
void pull_all_reduce(int dtype, const void* const* peers, int n_peers, void* out, long long n, cudaStream_t s);
// signal / wait on epoch flags in peer memory with a bounded spin; status != 0 on expiry
void signal_peers(int* const* peer_flags, int n_peers, int my_index, int value, cudaStream_t s);
void wait_flags(const int* my_flags, int n_peers, int value, long long max_spins, int* status, cudaStream_t s);
// signal + wait with a device-resident epoch counter (safe to replay inside a CUDA graph)
void group_barrier(int* const* peer_flags, const int* my_flags, int* counter, int n_peers, int my_index, long long max_spins,
                   int* status, cudaStream_t s);

// ---- epoch channels (signal now, wait inside the consumer) and the collectives built on them ------------------------------
// bump the channel's device-resident epoch and publish it to every member (release, system scope); never waits
void channel_signal(int* const* peer_flags, int n_peers, int my_index, int* counter, cudaStream_t s);
// owner side of the pushed reduce-scatter: wait for the members, sum the n_slots bf16 payload rows [acc | l | agg], unpack
void sum_payload(const void* slots, int n_slots, long long rows, int W, int HD, int H, int l_off, int agg_off, int d_agg, float* acc, float* l,
                 void* agg, const int* flags, const int* counter, long long max_spins, int* status, cudaStream_t s);
// backward mirror: wait, read the owners' bf16 payload gradient rows [dacc | dl | dagg] of the whole row block, unpack into the
// row vector (bf16), the statistics float4 {0, dl, 1, 0} and the aggregation gradient (bf16)
void pull_unpack(void* const* src, int n_peers, long long rows_per_peer, int W, int HD, int H, int l_off, int agg_off, int d_agg, void* row_vec,
                 void* stat, void* dagg, const int* flags, const int* counter, long long max_spins, int* status, cudaStream_t s);
void attn_bwd_prep(const float* dacc, const float* dl, long long n, int HD, int H, void* row_vec, void* stat, cudaStream_t s);
// two-shot all-reduce (reduce my slice from every member, store it to every member) of n fp32 values, n % 4 == 0; waits on the
// channel first.  channel_wait: a one-block bounded wait for consumers that cannot wait themselves.
void allreduce_two_shot(void* const* src, void* const* dst, int n_peers, int me, long long n, const int* flags, const int* counter,
                        long long max_spins, int* status, cudaStream_t s);
void channel_wait(const int* flags, const int* counter, int n_peers, long long max_spins, int* status, cudaStream_t s);
void sum_slots_wait(const void* slots, int n_slots, long long slot_elems, void* out, int out_dtype, int accumulate, const int* flags,
                    const int* counter, long long max_spins, int* status, cudaStream_t s);

}  // namespace gt
