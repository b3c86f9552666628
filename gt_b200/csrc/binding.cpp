// Python binding of the gt_b200 kernels: translates torch tensors into the POD launch arguments of kernels.h and enqueues
// on the current CUDA stream.  No kernel allocates; output and scratch tensors are created by the Python wrappers.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "kernels.h"

namespace {

using torch::Tensor;
using OptT = c10::optional<Tensor>;

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int dt(const Tensor& t) {
    if (t.scalar_type() == torch::kBFloat16) return gt::DT_BF16;
    TORCH_CHECK(t.scalar_type() == torch::kFloat32, "expected a float32 or bfloat16 tensor");
    return gt::DT_F32;
}

template <typename T>
const T* cptr(const OptT& t) { return t.has_value() && t->defined() ? static_cast<const T*>(t->data_ptr()) : nullptr; }

void check_cuda_contig(const Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

gt::SegPlan make_plan(const std::vector<Tensor>& p) {
    TORCH_CHECK(p.size() == 6, "plan = [seg_row, seg_beg, seg_end, seg_slot, split_rows, split_ptr]");
    gt::SegPlan s;
    s.seg_row = p[0].data_ptr<int>(); s.seg_beg = p[1].data_ptr<int>(); s.seg_end = p[2].data_ptr<int>();
    s.seg_slot = p[3].data_ptr<int>(); s.n_seg = (int)p[0].numel();
    s.split_rows = p[4].data_ptr<int>(); s.split_ptr = p[5].data_ptr<int>(); s.n_split = (int)p[4].numel();
    return s;
}

gt::AttnCommon make_common(const Tensor& q, int64_t H, int64_t D, const Tensor& idx, const OptT& etype, const OptT& gate,
                           const OptT& bias, const std::vector<Tensor>& plan, const OptT& scratch, int64_t score, int64_t norm,
                           double scale, double lo, double hi) {
    gt::AttnCommon c{};
    c.dtype = dt(q);
    c.H = (int)H; c.D = (int)D;
    c.T = gate.has_value() && gate->defined() ? (int)gate->size(0) : (bias.has_value() && bias->defined() ? (int)bias->size(0) : 1);
    c.score = (int)score; c.norm = (int)norm;
    c.scale = (float)scale; c.lo = (float)lo; c.hi = (float)hi;
    c.idx = idx.data_ptr<int>();
    c.etype = cptr<int>(etype);
    c.gate = cptr<float>(gate);
    c.bias = cptr<float>(bias);
    c.plan = make_plan(plan);
    c.scratch = scratch.has_value() && scratch->defined() ? scratch->data_ptr<float>() : nullptr;
    TORCH_CHECK(gt::attn_shape_supported(c.H, c.D, c.T), "attention shape (H=", H, ", D=", D, ", T=", c.T, ") not supported by the kernels");
    if (c.score != gt::SCORE_DOT && idx.numel() > 0) TORCH_CHECK(c.etype != nullptr, "gated / biased scores need edge types");
    return c;
}

void attn_fwd(Tensor q, OptT k, OptT v, Tensor idx, OptT etype, OptT gate, OptT bias, std::vector<Tensor> plan, OptT row_map,
              Tensor acc, Tensor l, OptT m, OptT scratch, int64_t H, int64_t D, int64_t score, int64_t norm, double scale, double lo,
              double hi, int64_t acc_stride, int64_t l_stride, bool accumulate, OptT k_peers, OptT v_peers, int64_t rows_per_peer,
              int64_t ldq, int64_t ldk, std::vector<int64_t> push_ptrs, int64_t push_rows, int64_t push_ld, int64_t push_l_off) {
    c10::cuda::CUDAGuard guard(q.device());
    TORCH_CHECK(q.is_cuda(), "q must be a CUDA tensor");
    if (ldq == 0) check_cuda_contig(q, "q");
    gt::AttnFwdArgs a{};
    a.c = make_common(q, H, D, idx, etype, gate, bias, plan, scratch, score, norm, scale, lo, hi);
    a.c.ldq = ldq; a.c.ldk = ldk;
    TORCH_CHECK(ldq % 8 == 0 && ldk % 8 == 0, "row strides must be multiples of 8 elements");
    a.push_n = (int)push_ptrs.size();
    if (a.push_n > 0) {
        TORCH_CHECK(a.push_n <= 8 && norm == gt::NORM_CLAMPEXP && push_rows > 0 && push_ld % 8 == 0 && push_l_off % 8 == 0 && !accumulate,
                    "pushed partials: at most 8 owners, clamp-exp, 16-byte aligned payload columns");
        for (int i = 0; i < a.push_n; ++i) a.push_slot[i] = reinterpret_cast<void*>(push_ptrs[i]);
        a.push_rows = (int)push_rows; a.push_ld = push_ld; a.push_l_off = (int)push_l_off;
    }
    a.q = q.data_ptr();
    a.k = k.has_value() ? k->data_ptr() : nullptr;
    a.v = v.has_value() ? v->data_ptr() : nullptr;
    a.k_peers = k_peers.has_value() ? reinterpret_cast<const void* const*>(k_peers->data_ptr()) : nullptr;
    a.v_peers = v_peers.has_value() ? reinterpret_cast<const void* const*>(v_peers->data_ptr()) : nullptr;
    a.rows_per_peer = (int)rows_per_peer;
    TORCH_CHECK(a.k_peers != nullptr || (a.k != nullptr && a.v != nullptr), "k / v or their peer tables are required");
    a.row_map = cptr<int>(row_map);
    a.acc = a.push_n > 0 ? nullptr : acc.data_ptr<float>(); a.l = a.push_n > 0 ? nullptr : l.data_ptr<float>();
    a.m = m.has_value() && m->defined() ? m->data_ptr<float>() : nullptr;
    a.acc_stride = acc_stride; a.l_stride = l_stride; a.accumulate = accumulate ? 1 : 0;
    gt::attn_fwd(a, stream());
}

// Dense 128 x 128 tiles of the mask on the tensor cores: merges their contribution into (acc, l, m) in place.
void attn_tile_fwd(Tensor q, Tensor k, Tensor v, Tensor rb_ids, Tensor rb_ptr, Tensor tile_cb, Tensor mask, OptT bias, Tensor acc,
                   Tensor l, OptT m, int64_t H, int64_t score, int64_t norm, double scale, double lo, double hi, int64_t ldq, int64_t ldk,
                   Tensor status, OptT dbg_s) {
    c10::cuda::CUDAGuard guard(q.device());
    TORCH_CHECK(q.is_cuda() && q.scalar_type() == torch::kBFloat16 && k.scalar_type() == torch::kBFloat16 && v.scalar_type() == torch::kBFloat16,
                "bf16 CUDA operands expected");
    TORCH_CHECK(mask.scalar_type() == torch::kUInt8 && mask.is_contiguous() && mask.dim() == 3 && mask.size(1) == 128 && mask.size(2) == 128,
                "mask must be uint8 [n_tiles, 128, 128]");
    TORCH_CHECK(tile_cb.numel() == mask.size(0) && rb_ptr.numel() == rb_ids.numel() + 1, "tile plan arrays do not match");
    TORCH_CHECK(acc.scalar_type() == torch::kFloat32 && l.scalar_type() == torch::kFloat32 && acc.stride(-1) == 1 && l.stride(-1) == 1,
                "fp32 partial results expected");
    TORCH_CHECK(score == gt::SCORE_DOT || score == gt::SCORE_BIASED, "tile attention evaluates plain or biased dot-product scores");
    gt::AttnTileArgs a{};
    a.H = (int)H; a.T = bias.has_value() && bias->defined() ? (int)bias->size(0) : 1;
    a.score = (int)score; a.norm = (int)norm; a.scale = (float)scale; a.lo = (float)lo; a.hi = (float)hi;
    a.bias = cptr<float>(bias);
    TORCH_CHECK(gt::attn_tile_supported(a.H, 32, a.T), "tile attention needs an even number of heads of 32 and at most 15 edge types");
    a.n_rb = (int)rb_ids.numel(); a.rb_ids = rb_ids.data_ptr<int>(); a.rb_ptr = rb_ptr.data_ptr<int>();
    a.tile_cb = tile_cb.data_ptr<int>(); a.mask = mask.data_ptr<unsigned char>();
    a.n_rows = (int)q.size(0); a.n_cols = (int)k.size(0);
    a.acc = acc.data_ptr<float>(); a.l = l.data_ptr<float>();
    a.m = m.has_value() && m->defined() ? m->data_ptr<float>() : nullptr;
    TORCH_CHECK(norm != gt::NORM_SOFTMAX || a.m != nullptr, "softmax partials need the row maxima");
    a.acc_stride = acc.stride(0); a.l_stride = l.stride(0);
    a.status = status.data_ptr<int>();
    a.dbg_s = dbg_s.has_value() && dbg_s->defined() ? dbg_s->data_ptr<float>() : nullptr;
    const int64_t hd = H * 32;
    int rc = gt::attn_tile_fwd(a, q.data_ptr(), k.data_ptr(), v.data_ptr(), ldq ? ldq : hd, ldk ? ldk : hd, stream());
    TORCH_CHECK(rc == 0, "tile attention launch failed with code ", rc);
}

int64_t attn_bwd_row_blocks(int64_t n_seg) { return gt::attn_bwd_row_blocks((int)n_seg); }

void attn_bwd_row(Tensor q, Tensor k, Tensor v, Tensor row_vec, Tensor stat, Tensor idx, OptT etype, OptT gate, OptT bias,
                  std::vector<Tensor> plan, OptT row_map, Tensor dq, bool accumulate_dq, OptT dgate_part, OptT dbias_part,
                  int64_t n_blocks, OptT scratch, int64_t H, int64_t D, int64_t score, int64_t norm, double scale, double lo, double hi,
                  int64_t ldq, int64_t ldk, int64_t ldr, int64_t ldo, OptT ds_in) {
    c10::cuda::CUDAGuard guard(q.device());
    gt::AttnBwdRowArgs a{};
    a.ds_in = cptr<float>(ds_in);
    if (a.ds_in) TORCH_CHECK(ds_in->scalar_type() == torch::kFloat32 && ds_in->is_contiguous() && ds_in->numel() == idx.numel() * H,
                             "ds_in must be a contiguous fp32 [E, H] tensor");
    a.c = make_common(q, H, D, idx, etype, gate, bias, plan, scratch, score, norm, scale, lo, hi);
    a.c.ldq = ldq; a.c.ldk = ldk; a.c.ldr = ldr; a.c.ldo = ldo;
    TORCH_CHECK(ldq % 8 == 0 && ldk % 8 == 0 && ldr % 8 == 0 && ldo % 8 == 0, "row strides must be multiples of 8 elements");
    TORCH_CHECK(row_vec.scalar_type() == q.scalar_type(), "row_vec must have the dtype of q");
    a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.row_vec = row_vec.data_ptr();
    a.stat = reinterpret_cast<const float4*>(stat.data_ptr<float>());
    a.row_map = cptr<int>(row_map);
    a.dq = dq.data_ptr(); a.accumulate_dq = accumulate_dq ? 1 : 0;
    a.dgate_part = dgate_part.has_value() && dgate_part->defined() ? dgate_part->data_ptr<float>() : nullptr;
    a.dbias_part = dbias_part.has_value() && dbias_part->defined() ? dbias_part->data_ptr<float>() : nullptr;
    a.n_blocks = (int)n_blocks;
    gt::attn_bwd_row(a, stream());
}

void attn_bwd_col(Tensor q, Tensor k, Tensor v, Tensor row_vec, Tensor stat, Tensor rowidx, OptT etype_t, OptT gate, OptT bias,
                  std::vector<Tensor> plan, Tensor dk, Tensor dv, OptT scratch, int64_t H, int64_t D, int64_t score, int64_t norm,
                  double scale, double lo, double hi, int64_t ldq, int64_t ldk, int64_t ldr, int64_t ldo, OptT ds_out, OptT pos) {
    c10::cuda::CUDAGuard guard(q.device());
    gt::AttnBwdColArgs a{};
    a.ds_out = ds_out.has_value() && ds_out->defined() ? ds_out->data_ptr<float>() : nullptr;
    a.pos = cptr<int>(pos);
    if (a.ds_out) TORCH_CHECK(a.pos != nullptr && ds_out->is_contiguous() && ds_out->numel() == rowidx.numel() * H && pos->numel() == rowidx.numel(),
                              "ds_out must be a contiguous fp32 [E, H] tensor and pos the CSR position of every CSC entry");
    a.c = make_common(q, H, D, rowidx, etype_t, gate, bias, plan, scratch, score, norm, scale, lo, hi);
    a.c.ldq = ldq; a.c.ldk = ldk; a.c.ldr = ldr; a.c.ldo = ldo;
    TORCH_CHECK(ldq % 8 == 0 && ldk % 8 == 0 && ldr % 8 == 0 && ldo % 8 == 0, "row strides must be multiples of 8 elements");
    a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.row_vec = row_vec.data_ptr();
    a.stat = reinterpret_cast<const float4*>(stat.data_ptr<float>());
    a.dk = dk.data_ptr(); a.dv = dv.data_ptr();
    gt::attn_bwd_col(a, stream());
}

void reduce_partials(Tensor part, Tensor out, bool accumulate) {
    c10::cuda::CUDAGuard guard(part.device());
    TORCH_CHECK(out.is_contiguous() && out.scalar_type() == torch::kFloat32, "fp32 contiguous output expected");
    gt::reduce_partials(part.data_ptr<float>(), (int)part.size(0), (int)out.numel(), out.data_ptr<float>(), stream(), accumulate ? 1 : 0);
}

// (name, registers, local bytes, static shared, dynamic shared, resident blocks per SM) of the main attention kernel instances
std::vector<std::tuple<std::string, int64_t, int64_t, int64_t, int64_t, int64_t>> attn_kernel_info() {
    std::vector<std::tuple<std::string, int64_t, int64_t, int64_t, int64_t, int64_t>> out;
    for (const auto& k : gt::attn_kernel_info())
        out.emplace_back(std::string(k.name), k.regs, k.local_bytes, k.static_smem, k.dyn_smem, k.blocks_per_sm);
    return out;
}

int64_t attn_status() { return gt::attn_status(); }

bool attn_shape_supported(int64_t H, int64_t D, int64_t T) { return gt::attn_shape_supported((int)H, (int)D, (int)T); }

void spmm(Tensor ptr, Tensor idx, OptT w, Tensor x, Tensor out, bool accumulate, std::vector<Tensor> plan, OptT scratch,
          std::vector<int64_t> push_ptrs, int64_t push_rows, int64_t push_ld, int64_t n_out) {
    c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0,
                "x must be a CUDA matrix with unit column stride, a row stride that is a multiple of 8 and a 16-byte aligned base");
    TORCH_CHECK(x.size(1) % 8 == 0 && x.size(1) <= 1024, "feature width must be a multiple of 8 and <= 1024");
    gt::SpmmArgs a{};
    a.dtype = dt(x); a.ptr = ptr.data_ptr<int>(); a.idx = idx.data_ptr<int>(); a.w = cptr<float>(w);
    a.x = x.data_ptr(); a.d = (int)x.size(1); a.accumulate = accumulate ? 1 : 0;
    a.ldx = x.stride(0);
    a.push_n = (int)push_ptrs.size();
    if (a.push_n > 0) {
        TORCH_CHECK(a.push_n <= 8 && push_rows > 0 && push_ld % 8 == 0 && !accumulate && n_out > 0, "pushed rows: at most 8 owners, aligned payload rows");
        for (int i = 0; i < a.push_n; ++i) a.push_slot[i] = reinterpret_cast<void*>(push_ptrs[i]);
        a.push_rows = (int)push_rows; a.ldo = push_ld; a.out = nullptr; a.n_out = (int)n_out;
    } else {
        TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1 && out.stride(0) % 8 == 0 && out.size(1) == x.size(1) && out.scalar_type() == x.scalar_type(),
                    "out must be [n_out, d] of x's dtype with unit column stride");
        a.out = out.data_ptr(); a.n_out = (int)out.size(0); a.ldo = out.stride(0);
    }
    a.use_plan = plan.empty() ? 0 : 1;
    if (a.use_plan) a.plan = make_plan(plan);
    a.scratch = scratch.has_value() && scratch->defined() ? scratch->data_ptr<float>() : nullptr;
    gt::spmm(a, stream());
}

void layer_norm_fwd(Tensor y, OptT x, OptT ybias, Tensor gamma, Tensor beta, Tensor out, OptT mean_rstd, double eps, double p,
                    OptT seed, int64_t stream_id, OptT acc, OptT l, double eps_l) {
    c10::cuda::CUDAGuard guard(y.device());
    check_cuda_contig(y, "y");
    TORCH_CHECK(y.size(1) % 8 == 0 && y.size(1) <= 1024, "LayerNorm width must be a multiple of 8 and <= 1024");
    gt::LayerNormArgs a{};
    a.dtype = dt(y); a.y = y.data_ptr(); a.x = x.has_value() && x->defined() ? x->data_ptr() : nullptr;
    a.ybias = cptr<float>(ybias); a.gamma = gamma.data_ptr<float>(); a.beta = beta.data_ptr<float>();
    a.out = out.data_ptr(); a.mean_rstd = mean_rstd.has_value() && mean_rstd->defined() ? mean_rstd->data_ptr<float>() : nullptr;
    a.n = (int)y.size(0); a.d = (int)y.size(1); a.eps = (float)eps; a.p = (float)p;
    a.seed = cptr<long long>(seed); a.stream_id = stream_id;
    a.acc = cptr<float>(acc); a.l = cptr<float>(l); a.H = a.l ? (int)l->size(1) : 1; a.eps_l = (float)eps_l;
    if (a.acc) TORCH_CHECK((a.d / a.H) % 8 == 0 && (((a.d / a.H) / 8) & ((a.d / a.H) / 8 - 1)) == 0, "head width must be 8 * 2^k");
    gt::layer_norm_fwd(a, stream());
}

void embed_add(Tensor x, Tensor tab_a, Tensor idx_a, int64_t pad_a, OptT tab_b, OptT idx_b, int64_t pad_b, Tensor out) {
    c10::cuda::CUDAGuard guard(x.device());
    check_cuda_contig(x, "x");
    TORCH_CHECK(x.size(1) % 8 == 0 && tab_a.scalar_type() == torch::kFloat32 && tab_a.is_contiguous() && idx_a.scalar_type() == torch::kInt64,
                "embed_add: width % 8 == 0, fp32 tables, int64 indices");
    const bool two = tab_b.has_value() && tab_b->defined();
    gt::embed_add(dt(x), x.data_ptr(), tab_a.data_ptr<float>(), idx_a.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(idx_a.data_ptr<int64_t>()) : nullptr,
                  pad_a, two ? tab_b->data_ptr<float>() : nullptr, two ? reinterpret_cast<const long long*>(idx_b->data_ptr<int64_t>()) : nullptr, pad_b,
                  out.data_ptr(), x.size(0), (int)x.size(1), stream());
}

void embed_add_bwd(Tensor dout, Tensor idx, int64_t pad, Tensor dtab) {
    c10::cuda::CUDAGuard guard(dout.device());
    check_cuda_contig(dout, "dout");
    gt::embed_add_bwd(dt(dout), dout.data_ptr(), reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()), pad, dtab.data_ptr<float>(),
                      dout.size(0), (int)dout.size(1), stream());
}

void gated_res_fwd(Tensor r, Tensor o, Tensor wa, Tensor wb, Tensor gate_bias, Tensor gamma, Tensor beta, Tensor out, Tensor stats, double eps,
                   double p, OptT seed, int64_t stream_id) {
    c10::cuda::CUDAGuard guard(r.device());
    check_cuda_contig(r, "r"); check_cuda_contig(o, "o");
    TORCH_CHECK(r.size(1) % 8 == 0 && r.size(1) <= 256, "gated residual kernel: width % 8 == 0 and <= 256");
    gt::GatedResArgs a{};
    a.dtype = dt(r); a.r = r.data_ptr(); a.o = o.data_ptr(); a.wa = wa.data_ptr<float>(); a.wb = wb.data_ptr<float>();
    a.gate_bias = gate_bias.data_ptr<float>(); a.gamma = gamma.data_ptr<float>(); a.beta = beta.data_ptr<float>(); a.out = out.data_ptr();
    a.stats = stats.data_ptr<float>(); a.n = r.size(0); a.d = (int)r.size(1); a.eps = (float)eps; a.p = (float)p;
    a.seed = cptr<long long>(seed); a.stream_id = stream_id;
    gt::gated_residual(a, false, stream());
}

void gated_res_bwd(Tensor r, Tensor o, Tensor dout, Tensor wa, Tensor wb, Tensor gamma, Tensor beta, Tensor stats, Tensor dr, Tensor d_o,
                   Tensor part, double p, OptT seed, int64_t stream_id) {
    c10::cuda::CUDAGuard guard(r.device());
    check_cuda_contig(dout, "dout");
    gt::GatedResArgs a{};
    a.dtype = dt(r); a.r = r.data_ptr(); a.o = o.data_ptr(); a.dout = dout.data_ptr(); a.wa = wa.data_ptr<float>(); a.wb = wb.data_ptr<float>();
    a.gamma = gamma.data_ptr<float>(); a.beta = beta.data_ptr<float>(); a.stats = stats.data_ptr<float>(); a.dr = dr.data_ptr();
    a.d_o = d_o.data_ptr(); a.part = part.data_ptr<float>(); a.part_stride = (int)part.stride(0); a.n_blocks = (int)part.size(0);
    a.n = r.size(0); a.d = (int)r.size(1); a.p = (float)p; a.seed = cptr<long long>(seed); a.stream_id = stream_id;
    gt::gated_residual(a, true, stream());
}

int64_t premp_blocks(int64_t n) { return gt::premp_blocks((int)n); }

void premp_fwd(Tensor h, Tensor gamma, Tensor beta, Tensor out, Tensor stats, double eps, double p, OptT seed, int64_t stream_id, bool l2norm) {
    c10::cuda::CUDAGuard guard(h.device());
    check_cuda_contig(h, "h");
    TORCH_CHECK(h.size(1) % 8 == 0 && h.size(1) <= 1024, "width must be a multiple of 8 and <= 1024");
    gt::PreMpArgs a{};
    a.dtype = dt(h); a.h = h.data_ptr(); a.gamma = gamma.data_ptr<float>(); a.beta = beta.data_ptr<float>(); a.out = out.data_ptr();
    a.stats = stats.data_ptr<float>(); a.n = (int)h.size(0); a.d = (int)h.size(1); a.eps = (float)eps; a.p = (float)p;
    a.seed = cptr<long long>(seed); a.stream_id = stream_id; a.l2norm = l2norm ? 1 : 0;
    gt::premp(a, false, stream());
}

void premp_bwd(Tensor h, Tensor dout, Tensor gamma, Tensor beta, Tensor stats, Tensor dh, Tensor part, double p, OptT seed, int64_t stream_id,
               bool l2norm) {
    c10::cuda::CUDAGuard guard(h.device());
    check_cuda_contig(h, "h"); check_cuda_contig(dout, "dout");
    gt::PreMpArgs a{};
    a.dtype = dt(h); a.h = h.data_ptr(); a.dout = dout.data_ptr(); a.gamma = gamma.data_ptr<float>(); a.beta = beta.data_ptr<float>();
    a.stats = stats.data_ptr<float>(); a.dh = dh.data_ptr(); a.part = part.data_ptr<float>(); a.n_blocks = (int)part.size(0);
    a.n = (int)h.size(0); a.d = (int)h.size(1); a.p = (float)p; a.seed = cptr<long long>(seed); a.stream_id = stream_id;
    a.l2norm = l2norm ? 1 : 0;
    gt::premp(a, true, stream());
}

int64_t layer_norm_bwd_blocks(int64_t n) { return gt::layer_norm_bwd_blocks((int)n); }

void layer_norm_bwd(Tensor dout, Tensor y, OptT x, OptT ybias, Tensor gamma, Tensor mean_rstd, Tensor dy, OptT dx, bool accumulate_dx,
                    Tensor dgamma_part, Tensor dbeta_part, OptT dybias_part, double p, OptT seed, int64_t stream_id, OptT acc, OptT l,
                    double eps_l, OptT dacc, OptT dl) {
    c10::cuda::CUDAGuard guard(y.device());
    gt::LayerNormBwdArgs a{};
    a.dtype = dt(y); a.dout = dout.data_ptr(); a.y = y.data_ptr(); a.x = x.has_value() && x->defined() ? x->data_ptr() : nullptr;
    a.ybias = cptr<float>(ybias); a.gamma = gamma.data_ptr<float>(); a.mean_rstd = mean_rstd.data_ptr<float>();
    a.dy = dy.data_ptr(); a.dx = dx.has_value() && dx->defined() ? dx->data_ptr() : nullptr; a.accumulate_dx = accumulate_dx ? 1 : 0;
    a.dgamma_part = dgamma_part.data_ptr<float>(); a.dbeta_part = dbeta_part.data_ptr<float>();
    a.dybias_part = dybias_part.has_value() && dybias_part->defined() ? dybias_part->data_ptr<float>() : nullptr;
    a.n_blocks = (int)dgamma_part.size(0);
    a.part_stride = (int)dgamma_part.stride(0);
    TORCH_CHECK(dbeta_part.stride(0) == dgamma_part.stride(0), "the partial buffers must share one row stride");
    a.n = (int)y.size(0); a.d = (int)y.size(1); a.p = (float)p; a.seed = cptr<long long>(seed); a.stream_id = stream_id;
    a.acc = cptr<float>(acc); a.l = cptr<float>(l); a.H = a.l ? (int)l->size(1) : 1; a.eps_l = (float)eps_l;
    a.dacc = dacc.has_value() && dacc->defined() ? dacc->data_ptr<float>() : nullptr;
    a.dl = dl.has_value() && dl->defined() ? dl->data_ptr<float>() : nullptr;
    gt::layer_norm_bwd(a, stream());
}

void bias_act_dropout(Tensor in, OptT bias, Tensor out, int64_t act, double p, OptT seed, int64_t stream_id) {
    c10::cuda::CUDAGuard guard(in.device());
    TORCH_CHECK(in.size(-1) % 8 == 0, "width must be a multiple of 8");
    gt::bias_act_dropout(dt(in), in.data_ptr(), cptr<float>(bias), out.data_ptr(), in.numel() / in.size(-1), (int)in.size(-1), (int)act,
                         (float)p, cptr<long long>(seed), stream_id, stream());
}

int64_t colsum_blocks(int64_t n) { return gt::colsum_blocks(n); }

void bias_act_dropout_bwd(Tensor dout, OptT in, OptT bias, Tensor dz, int64_t act, double p, OptT seed, int64_t stream_id, OptT dbias_part) {
    c10::cuda::CUDAGuard guard(dout.device());
    const int d = (int)dout.size(-1);
    TORCH_CHECK(d % 8 == 0 && d <= 8192, "width must be a multiple of 8");
    const long long n = dout.numel() / d;
    const int n_blocks = dbias_part.has_value() && dbias_part->defined() ? (int)dbias_part->size(0) : gt::colsum_blocks(n);
    gt::bias_act_dropout_bwd(dt(dout), dout.data_ptr(), in.has_value() && in->defined() ? in->data_ptr() : nullptr, cptr<float>(bias),
                             dz.data_ptr(), n, d, (int)act, (float)p, cptr<long long>(seed), stream_id,
                             dbias_part.has_value() && dbias_part->defined() ? dbias_part->data_ptr<float>() : nullptr, n_blocks, stream());
}

void cross_entropy(Tensor logits, Tensor labels, Tensor mask, double inv_denom, Tensor loss, OptT dlogits) {
    c10::cuda::CUDAGuard guard(logits.device());
    check_cuda_contig(logits, "logits");
    TORCH_CHECK(labels.scalar_type() == torch::kInt64 && mask.scalar_type() == torch::kBool, "labels int64, mask bool");
    gt::cross_entropy_fwd_bwd(dt(logits), logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                              mask.data_ptr<bool>(), (int)logits.size(0), (int)logits.size(1), (float)inv_denom, loss.data_ptr<float>(),
                              dlogits.has_value() && dlogits->defined() ? dlogits->data_ptr() : nullptr, stream());
}

void adamw_step(Tensor p, Tensor g, Tensor m, Tensor v, OptT p_bf16, Tensor hyper, OptT decay_mask) {
    c10::cuda::CUDAGuard guard(p.device());
    gt::AdamWArgs a{};
    a.p = p.data_ptr<float>(); a.g = g.data_ptr<float>(); a.m = m.data_ptr<float>(); a.v = v.data_ptr<float>();
    a.p_bf16 = p_bf16.has_value() && p_bf16->defined() ? p_bf16->data_ptr() : nullptr;
    a.n = p.numel(); a.hyper = hyper.data_ptr<float>(); a.decay_mask = cptr<float>(decay_mask);
    gt::adamw_step(a, stream());
}

void sq_norm(Tensor g, Tensor out) {
    c10::cuda::CUDAGuard guard(g.device());
    gt::sq_norm(g.data_ptr<float>(), g.numel(), out.data_ptr<float>(), stream());
}

void cast_bf16(Tensor in, Tensor out) {
    c10::cuda::CUDAGuard guard(in.device());
    gt::cast_f32_to_bf16(in.data_ptr<float>(), out.data_ptr(), in.numel(), stream());
}

// parts[i] [n, w_i] (fp32 / bf16, unit column stride) <-> packed [n, sum w_i]; to_packed selects the direction
void pack_cols(std::vector<Tensor> parts, Tensor packed, bool to_packed) {
    c10::cuda::CUDAGuard guard(packed.device());
    TORCH_CHECK(parts.size() >= 1 && parts.size() <= 4, "1..4 parts");
    gt::PackColsArgs a{};
    a.n_seg = (int)parts.size();
    int w = 0;
    for (int i = 0; i < a.n_seg; ++i) {
        Tensor& t = parts[i];
        TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1 && t.size(0) == packed.size(0) && t.size(1) % 8 == 0 && t.stride(0) % 8 == 0 &&
                    (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, "parts must be [n, w] with w, row stride % 8 == 0, 16-byte aligned");
        a.seg[i] = gt::PackColSeg{t.data_ptr(), (int)t.size(1), dt(t), (int)t.stride(0)};
        w += (int)t.size(1);
    }
    TORCH_CHECK(packed.dim() == 2 && packed.stride(1) == 1 && packed.size(1) >= w && packed.stride(0) % 8 == 0, "packed shape");
    a.packed = packed.data_ptr(); a.packed_dtype = dt(packed); a.ld_packed = (int)packed.stride(0); a.width = w;
    a.n_rows = packed.size(0); a.dir = to_packed ? 0 : 1;
    gt::pack_cols(a, stream());
}

// C[M, N] = epilogue(A[M, K] @ B[N, K]^T)
void gemm_nt(Tensor a, Tensor b, Tensor c, OptT bias, int64_t act, double p, OptT seed, int64_t stream_id, bool accumulate, Tensor status) {
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16, "bf16 operands expected");
    TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && c.stride(1) == 1, "row-major operands expected");
    gt::GemmArgs g{};
    g.a = a.data_ptr(); g.b = b.data_ptr(); g.c = c.data_ptr();
    g.M = (int)a.size(0); g.K = (int)a.size(1); g.N = (int)b.size(0);
    TORCH_CHECK(b.size(1) == a.size(1) && c.size(0) == a.size(0) && c.size(1) == b.size(0), "shape mismatch");
    g.lda = (int)a.stride(0); g.ldb = (int)b.stride(0); g.ldc = (int)c.stride(0);
    g.c_dtype = dt(c); g.bias = cptr<float>(bias); g.act = (int)act; g.p = (float)p; g.seed = cptr<long long>(seed);
    g.stream_id = stream_id; g.accumulate = accumulate ? 1 : 0; g.status = status.data_ptr<int>();
    TORCH_CHECK(gt::gemm_tcgen05_supported(g.M, g.N, g.K, g.lda, g.ldb, g.ldc), "GEMM shape / strides not supported (K, lda, ldb % 8)");
    int rc = gt::gemm_tcgen05(g, stream());
    TORCH_CHECK(rc == 0, "tcgen05 GEMM launch failed with code ", rc);
}

// C[N, K] (+)= A[M, N]^T @ B[M, K]
void gemm_tn(Tensor a, Tensor b, Tensor c, bool accumulate, Tensor status) {
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16 && c.scalar_type() == torch::kFloat32,
                "bf16 operands and an fp32 result expected");
    TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && c.is_contiguous(), "row-major operands expected");
    gt::GemmTNArgs g{};
    g.a = a.data_ptr(); g.b = b.data_ptr(); g.c = c.data_ptr<float>();
    g.M = (int)a.size(0); g.N = (int)a.size(1); g.K = (int)b.size(1);
    TORCH_CHECK(b.size(0) == a.size(0) && c.size(0) == a.size(1) && c.size(1) == b.size(1), "shape mismatch");
    g.lda = (int)a.stride(0); g.ldb = (int)b.stride(0); g.ldc = (int)c.stride(0);
    g.accumulate = accumulate ? 1 : 0; g.status = status.data_ptr<int>();
    int rc = gt::gemm_tn_tcgen05(g, stream());
    TORCH_CHECK(rc == 0, "tcgen05 TN GEMM launch failed with code ", rc);
}

// C[g * chunk, N] = epilogue(gathered(A) @ B[N, K]^T): rank p's [chunk, K] rows of A are read from peer_ptrs[p] (addresses
// inside the peers' symmetric heaps, row stride lda) by TMA inside the GEMM; `gathered` (optional) receives the gathered A.
void gemm_nt_gather(std::vector<int64_t> peer_ptrs, int64_t chunk, int64_t k, int64_t lda, Tensor b, Tensor c, OptT bias, int64_t act,
                    double p, OptT seed, int64_t stream_id, OptT gathered, Tensor status, OptT wait_flags, OptT wait_counter, int64_t max_spins,
                    int64_t self_index) {
    c10::cuda::CUDAGuard guard(b.device());
    TORCH_CHECK(b.scalar_type() == torch::kBFloat16 && b.stride(1) == 1 && c.stride(1) == 1, "bf16 row-major operands expected");
    const int n_peers = (int)peer_ptrs.size();
    TORCH_CHECK(b.size(1) == k && c.size(0) == chunk * n_peers && c.size(1) == b.size(0), "shape mismatch");
    gt::GemmArgs g{};
    g.a = nullptr; g.b = b.data_ptr(); g.c = c.data_ptr();
    g.M = (int)(chunk * n_peers); g.K = (int)k; g.N = (int)b.size(0);
    g.lda = (int)lda; g.ldb = (int)b.stride(0); g.ldc = (int)c.stride(0);
    g.c_dtype = dt(c); g.bias = cptr<float>(bias); g.act = (int)act; g.p = (float)p; g.seed = cptr<long long>(seed);
    g.stream_id = stream_id; g.accumulate = 0; g.status = status.data_ptr<int>();
    std::vector<const void*> peers(n_peers);
    for (int i = 0; i < n_peers; ++i) peers[i] = reinterpret_cast<const void*>(peer_ptrs[i]);
    void* gat = nullptr;
    if (gathered.has_value() && gathered->defined()) {
        TORCH_CHECK(gathered->scalar_type() == torch::kBFloat16 && gathered->size(0) == chunk * n_peers && gathered->size(1) == k &&
                    gathered->stride(0) == lda && gathered->stride(1) == 1, "gathered copy must be [g * chunk, K] bf16 with row stride lda");
        gat = gathered->data_ptr();
    }
    gt::GatherWait wait{cptr<int>(wait_flags), cptr<int>(wait_counter), (long long)max_spins, (int)self_index};
    TORCH_CHECK((wait.flags == nullptr) == (wait.counter == nullptr), "wait flags and counter come together");
    int rc = gt::gemm_nt_gather(g, peers.data(), n_peers, (int)chunk, gat, stream(), wait.flags ? &wait : (self_index ? &wait : nullptr));
    TORCH_CHECK(rc == 0, "fused all-gather GEMM failed with code ", rc);
}

// Row block p of A[M, K] @ B[N, K]^T (bf16) is written into slot_ptrs[p] ([chunk, N], row stride ldc) in rank p's memory.
void gemm_nt_scatter(Tensor a, Tensor b, std::vector<int64_t> slot_ptrs, int64_t chunk, int64_t ldc, Tensor status) {
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16, "bf16 operands expected");
    TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && b.size(1) == a.size(1), "row-major operands with equal K expected");
    const int n_peers = (int)slot_ptrs.size();
    TORCH_CHECK(a.size(0) == chunk * n_peers, "A must have n_peers * chunk rows");
    gt::GemmArgs g{};
    g.a = a.data_ptr(); g.b = b.data_ptr(); g.c = nullptr;
    g.M = (int)a.size(0); g.K = (int)a.size(1); g.N = (int)b.size(0);
    g.lda = (int)a.stride(0); g.ldb = (int)b.stride(0); g.ldc = (int)ldc;
    g.c_dtype = gt::DT_BF16; g.status = status.data_ptr<int>();
    std::vector<void*> slots(n_peers);
    for (int i = 0; i < n_peers; ++i) slots[i] = reinterpret_cast<void*>(slot_ptrs[i]);
    int rc = gt::gemm_nt_scatter(g, slots.data(), n_peers, (int)chunk, stream());
    TORCH_CHECK(rc == 0, "fused GEMM reduce-scatter failed with code ", rc);
}

// out (+)= sum over the leading dimension of slots [n, ...] (bf16 slots, fp32 accumulation)
void sum_slots(Tensor slots, Tensor out, bool accumulate) {
    c10::cuda::CUDAGuard guard(slots.device());
    TORCH_CHECK(slots.scalar_type() == torch::kBFloat16 && slots.is_contiguous() && out.is_contiguous(), "contiguous bf16 slots expected");
    const int64_t n = slots.size(0), elems = slots.numel() / n;
    TORCH_CHECK(out.numel() == elems && elems % 8 == 0, "slot size must equal the output size and be a multiple of 8");
    gt::sum_slots(slots.data_ptr(), (int)n, elems, out.data_ptr(), dt(out), accumulate ? 1 : 0, stream());
}

// ---- epoch channels ------------------------------------------------------------------------------------------------------
void channel_signal(std::vector<int64_t> peer_flag_ptrs, int64_t my_index, Tensor counter) {
    c10::cuda::CUDAGuard guard(counter.device());
    TORCH_CHECK(peer_flag_ptrs.size() <= 8, "at most 8 group members");
    std::vector<int*> pf(peer_flag_ptrs.size());
    for (size_t i = 0; i < pf.size(); ++i) pf[i] = reinterpret_cast<int*>(peer_flag_ptrs[i]);
    gt::channel_signal(pf.data(), (int)pf.size(), (int)my_index, counter.data_ptr<int>(), stream());
}

// slots [n_slots, rows, W] bf16 (this rank's staging area) -> acc fp32 [rows, HD], l fp32 [rows, H], agg bf16 [rows, d_agg] (optional)
void sum_payload(Tensor slots, Tensor acc, Tensor l, OptT agg, int64_t l_off, int64_t agg_off, OptT flags, OptT counter, int64_t max_spins,
                 Tensor status) {
    c10::cuda::CUDAGuard guard(slots.device());
    TORCH_CHECK(slots.dim() == 3 && slots.is_contiguous() && slots.scalar_type() == torch::kBFloat16 && slots.size(2) % 8 == 0, "slots [n, rows, W] bf16");
    TORCH_CHECK(acc.is_contiguous() && l.is_contiguous() && acc.size(0) == slots.size(1) && acc.size(1) % 8 == 0 && l_off % 8 == 0 && agg_off % 8 == 0,
                "payload columns must be 16-byte aligned");
    const bool has_agg = agg.has_value() && agg->defined();
    if (has_agg) TORCH_CHECK(agg->is_contiguous() && agg->scalar_type() == torch::kBFloat16 && agg->size(1) % 8 == 0, "agg [rows, d] bf16");
    gt::sum_payload(slots.data_ptr(), (int)slots.size(0), slots.size(1), (int)slots.size(2), (int)acc.size(1), (int)l.size(1), (int)l_off,
                    (int)agg_off, has_agg ? (int)agg->size(1) : 0, acc.data_ptr<float>(), l.data_ptr<float>(), has_agg ? agg->data_ptr() : nullptr,
                    cptr<int>(flags), cptr<int>(counter), max_spins, status.data_ptr<int>(), stream());
}

// peers' payload gradients [rows_per_peer, W] bf16 at src_ptrs -> row_vec bf16 [P * rows, HD], stat fp32 [P * rows, H, 4], dagg bf16 (optional)
void pull_unpack(std::vector<int64_t> src_ptrs, int64_t rows_per_peer, int64_t W, Tensor row_vec, Tensor stat, OptT dagg, int64_t l_off,
                 int64_t agg_off, OptT flags, OptT counter, int64_t max_spins, Tensor status) {
    c10::cuda::CUDAGuard guard(row_vec.device());
    const int n = (int)src_ptrs.size();
    TORCH_CHECK(n >= 1 && n <= 8 && W % 8 == 0 && l_off % 8 == 0 && agg_off % 8 == 0, "at most 8 peers, aligned payload");
    TORCH_CHECK(row_vec.is_contiguous() && row_vec.scalar_type() == torch::kBFloat16 && row_vec.size(0) == rows_per_peer * n && stat.is_contiguous() &&
                stat.scalar_type() == torch::kFloat32 && stat.size(0) == row_vec.size(0) && stat.size(2) == 4, "row_vec [P rows, HD] bf16, stat [P rows, H, 4] fp32");
    const bool has = dagg.has_value() && dagg->defined();
    if (has) TORCH_CHECK(dagg->is_contiguous() && dagg->scalar_type() == torch::kBFloat16 && dagg->size(0) == row_vec.size(0), "dagg [P rows, d] bf16");
    std::vector<void*> src(n);
    for (int i = 0; i < n; ++i) src[i] = reinterpret_cast<void*>(src_ptrs[i]);
    gt::pull_unpack(src.data(), n, rows_per_peer, (int)W, (int)row_vec.size(1), (int)stat.size(1), (int)l_off, (int)agg_off, has ? (int)dagg->size(1) : 0,
                    row_vec.data_ptr(), stat.data_ptr(), has ? dagg->data_ptr() : nullptr, cptr<int>(flags), cptr<int>(counter), max_spins,
                    status.data_ptr<int>(), stream());
}

void attn_bwd_prep(Tensor dacc, Tensor dl, Tensor row_vec, Tensor stat) {
    c10::cuda::CUDAGuard guard(dacc.device());
    TORCH_CHECK(dacc.is_contiguous() && dl.is_contiguous() && row_vec.is_contiguous() && stat.is_contiguous() && dacc.scalar_type() == torch::kFloat32 &&
                dl.scalar_type() == torch::kFloat32 && row_vec.scalar_type() == torch::kBFloat16 && stat.scalar_type() == torch::kFloat32 &&
                dacc.size(1) % 8 == 0, "dacc fp32 [n, HD], dl fp32 [n, H] -> row_vec bf16 [n, HD], stat fp32 [n, H, 4]");
    gt::attn_bwd_prep(dacc.data_ptr<float>(), dl.data_ptr<float>(), dacc.size(0), (int)dacc.size(1), (int)dl.size(1), row_vec.data_ptr(),
                      stat.data_ptr(), stream());
}

void allreduce_two_shot(std::vector<int64_t> src_ptrs, std::vector<int64_t> dst_ptrs, int64_t me, int64_t n, Tensor flags, Tensor counter,
                        int64_t max_spins, Tensor status) {
    c10::cuda::CUDAGuard guard(flags.device());
    const int np = (int)src_ptrs.size();
    TORCH_CHECK(np >= 1 && np <= 8 && dst_ptrs.size() == src_ptrs.size() && n % 4 == 0, "1..8 members, n a multiple of 4");
    std::vector<void*> a(np), b(np);
    for (int i = 0; i < np; ++i) {
        a[i] = reinterpret_cast<void*>(src_ptrs[i]); b[i] = reinterpret_cast<void*>(dst_ptrs[i]);
        TORCH_CHECK((src_ptrs[i] & 15) == 0 && (dst_ptrs[i] & 15) == 0, "buffers must be 16-byte aligned");
    }
    gt::allreduce_two_shot(a.data(), b.data(), np, (int)me, n, flags.data_ptr<int>(), counter.data_ptr<int>(), max_spins, status.data_ptr<int>(),
                           stream());
}

void channel_wait(Tensor flags, Tensor counter, int64_t n_peers, int64_t max_spins, Tensor status) {
    c10::cuda::CUDAGuard guard(flags.device());
    gt::channel_wait(flags.data_ptr<int>(), counter.data_ptr<int>(), (int)n_peers, max_spins, status.data_ptr<int>(), stream());
}

void sum_slots_wait(Tensor slots, Tensor out, bool accumulate, OptT flags, OptT counter, int64_t max_spins, Tensor status) {
    c10::cuda::CUDAGuard guard(slots.device());
    TORCH_CHECK(slots.scalar_type() == torch::kBFloat16 && slots.is_contiguous() && out.is_contiguous(), "contiguous bf16 slots expected");
    const int64_t n = slots.size(0), elems = slots.numel() / n;
    TORCH_CHECK(out.numel() == elems && elems % 8 == 0, "slot size must equal the output size and be a multiple of 8");
    gt::sum_slots_wait(slots.data_ptr(), (int)n, elems, out.data_ptr(), dt(out), accumulate ? 1 : 0, cptr<int>(flags), cptr<int>(counter), max_spins,
                       status.data_ptr<int>(), stream());
}

// ---- symmetric heap: cudaMalloc + CUDA IPC ----------------------------------------------------------------------------
int64_t heap_alloc(int64_t bytes) {
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)bytes);
    TORCH_CHECK(e == cudaSuccess, "cudaMalloc of the symmetric heap failed: ", cudaGetErrorString(e));
    cudaMemset(p, 0, (size_t)bytes);
    return reinterpret_cast<int64_t>(p);
}

void heap_free(int64_t ptr) { cudaFree(reinterpret_cast<void*>(ptr)); }

py::bytes heap_ipc_handle(int64_t ptr) {
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr));
    TORCH_CHECK(e == cudaSuccess, "cudaIpcGetMemHandle failed: ", cudaGetErrorString(e));
    return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
}

int64_t heap_open(py::bytes handle) {
    std::string s = handle;
    TORCH_CHECK(s.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
    cudaIpcMemHandle_t h;
    memcpy(&h, s.data(), sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    TORCH_CHECK(e == cudaSuccess, "cudaIpcOpenMemHandle failed: ", cudaGetErrorString(e));
    return reinterpret_cast<int64_t>(p);
}

void heap_close(int64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }

Tensor tensor_from_ptr(int64_t ptr, std::vector<int64_t> shape, int64_t dtype_code, int64_t device_index) {
    auto dtype = dtype_code == 0 ? torch::kFloat32 : dtype_code == 1 ? torch::kBFloat16 : dtype_code == 2 ? torch::kInt32 : dtype_code == 3 ? torch::kInt64 : torch::kUInt8;
    auto opts = torch::TensorOptions().dtype(dtype).device(torch::kCUDA, (int)device_index);
    return torch::from_blob(reinterpret_cast<void*>(ptr), shape, [](void*) {}, opts);
}

void signal_peers(Tensor peer_flag_ptrs, int64_t my_index, int64_t value) {
    c10::cuda::CUDAGuard guard(peer_flag_ptrs.device());
    gt::signal_peers(reinterpret_cast<int* const*>(peer_flag_ptrs.data_ptr()), (int)peer_flag_ptrs.numel(), (int)my_index, (int)value, stream());
}

void wait_flags(Tensor my_flags, int64_t n_peers, int64_t value, int64_t max_spins, Tensor status) {
    c10::cuda::CUDAGuard guard(my_flags.device());
    gt::wait_flags(my_flags.data_ptr<int>(), (int)n_peers, (int)value, max_spins, status.data_ptr<int>(), stream());
}

void group_barrier(Tensor peer_flag_ptrs, Tensor my_flags, Tensor counter, int64_t my_index, int64_t max_spins, Tensor status) {
    c10::cuda::CUDAGuard guard(my_flags.device());
    gt::group_barrier(reinterpret_cast<int* const*>(peer_flag_ptrs.data_ptr()), my_flags.data_ptr<int>(), counter.data_ptr<int>(),
                      (int)peer_flag_ptrs.numel(), (int)my_index, max_spins, status.data_ptr<int>(), stream());
}

void pull_all_to_all(Tensor peer_ptrs, int64_t me, int64_t rows, int64_t slab_bytes, bool to_heads, Tensor out) {
    c10::cuda::CUDAGuard guard(out.device());
    TORCH_CHECK(slab_bytes % 16 == 0, "head slabs must be a multiple of 16 bytes");
    gt::pull_all_to_all(reinterpret_cast<const void* const*>(peer_ptrs.data_ptr()), (int)peer_ptrs.numel(), (int)me, rows, slab_bytes, to_heads,
                        out.data_ptr(), stream());
}

void pull_gather_rows(Tensor peer_ptrs, Tensor owner, Tensor row, Tensor out) {
    c10::cuda::CUDAGuard guard(out.device());
    const int row_bytes = (int)(out.numel() / std::max<int64_t>(out.size(0), 1) * out.element_size());
    TORCH_CHECK(row_bytes % 16 == 0, "rows must be a multiple of 16 bytes");
    gt::pull_gather_rows(reinterpret_cast<const void* const*>(peer_ptrs.data_ptr()), owner.data_ptr<int>(), row.data_ptr<int>(), out.data_ptr(),
                         (int)out.size(0), row_bytes, stream());
}

void pull_reduce_rows(Tensor peer_ptrs, Tensor src, Tensor out) {
    c10::cuda::CUDAGuard guard(out.device());
    TORCH_CHECK(out.size(1) % 8 == 0, "row width must be a multiple of 8 elements");
    gt::pull_reduce_rows(dt(out), reinterpret_cast<const void* const*>(peer_ptrs.data_ptr()), (int)peer_ptrs.numel(), src.data_ptr<int>(),
                         out.data_ptr(), (int)out.size(0), (int)out.size(1), stream());
}

void pull_all_gather(Tensor peer_ptrs, Tensor out) {
    c10::cuda::CUDAGuard guard(out.device());
    const long long chunk_bytes = (long long)out.numel() * out.element_size() / peer_ptrs.numel();
    TORCH_CHECK(chunk_bytes % 16 == 0, "chunks must be a multiple of 16 bytes");
    gt::pull_all_gather(reinterpret_cast<const void* const*>(peer_ptrs.data_ptr()), (int)peer_ptrs.numel(), out.data_ptr(), chunk_bytes, stream());
}

void pull_reduce_scatter(Tensor peer_ptrs, int64_t my_index, Tensor out) {
    c10::cuda::CUDAGuard guard(out.device());
    TORCH_CHECK(out.numel() % 8 == 0, "chunk must be a multiple of 8 elements");
    gt::pull_reduce_scatter(dt(out), reinterpret_cast<const void* const*>(peer_ptrs.data_ptr()), (int)peer_ptrs.numel(), (int)my_index,
                            out.data_ptr(), out.numel(), stream());
}

void pull_all_reduce(Tensor peer_ptrs, Tensor out) {
    c10::cuda::CUDAGuard guard(out.device());
    TORCH_CHECK(out.numel() % 8 == 0, "payload must be a multiple of 8 elements");
    gt::pull_all_reduce(dt(out), reinterpret_cast<const void* const*>(peer_ptrs.data_ptr()), (int)peer_ptrs.numel(), out.data_ptr(), out.numel(), stream());
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("attn_fwd", &attn_fwd);
    m.def("attn_bwd_row", &attn_bwd_row);
    m.def("attn_bwd_row_blocks", &attn_bwd_row_blocks);
    m.def("attn_bwd_col", &attn_bwd_col);
    m.def("attn_shape_supported", &attn_shape_supported);
    m.def("attn_kernel_info", &attn_kernel_info);
    m.def("reduce_partials", &reduce_partials);
    m.def("spmm", &spmm);
    m.def("layer_norm_fwd", &layer_norm_fwd);
    m.def("layer_norm_bwd", &layer_norm_bwd);
    m.def("layer_norm_bwd_blocks", &layer_norm_bwd_blocks);
    m.def("bias_act_dropout", &bias_act_dropout);
    m.def("bias_act_dropout_bwd", &bias_act_dropout_bwd);
    m.def("colsum_blocks", &colsum_blocks);
    m.def("cross_entropy", &cross_entropy);
    m.def("adamw_step", &adamw_step);
    m.def("sq_norm", &sq_norm);
    m.def("cast_bf16", &cast_bf16);
    m.def("pack_cols", &pack_cols);
    m.def("premp_blocks", &premp_blocks);
    m.def("embed_add", &embed_add);
    m.def("embed_add_bwd", &embed_add_bwd);
    m.def("gated_res_fwd", &gated_res_fwd);
    m.def("gated_res_bwd", &gated_res_bwd);
    m.def("premp_fwd", &premp_fwd);
    m.def("premp_bwd", &premp_bwd);
    m.def("gemm_nt", &gemm_nt);
    m.def("gemm_tn", &gemm_tn);
    m.def("gemm_nt_gather", &gemm_nt_gather);
    m.def("gemm_nt_scatter", &gemm_nt_scatter);
    m.def("sum_slots", &sum_slots);
    m.def("heap_alloc", &heap_alloc);
    m.def("heap_free", &heap_free);
    m.def("heap_ipc_handle", &heap_ipc_handle);
    m.def("heap_open", &heap_open);
    m.def("heap_close", &heap_close);
    m.def("tensor_from_ptr", &tensor_from_ptr);
    m.def("signal_peers", &signal_peers);
    m.def("wait_flags", &wait_flags);
    m.def("group_barrier", &group_barrier);
    m.def("attn_status", &attn_status);
    m.def("attn_tile_fwd", &attn_tile_fwd);
    m.def("channel_signal", &channel_signal);
    m.def("sum_payload", &sum_payload);
    m.def("pull_unpack", &pull_unpack);
    m.def("attn_bwd_prep", &attn_bwd_prep);
    m.def("sum_slots_wait", &sum_slots_wait);
    m.def("allreduce_two_shot", &allreduce_two_shot);
    m.def("channel_wait", &channel_wait);
    m.def("pull_gather_rows", &pull_gather_rows);
    m.def("pull_all_to_all", &pull_all_to_all);
    m.def("pull_reduce_rows", &pull_reduce_rows);
    m.def("pull_all_gather", &pull_all_gather);
    m.def("pull_reduce_scatter", &pull_reduce_scatter);
    m.def("pull_all_reduce", &pull_all_reduce);
}
