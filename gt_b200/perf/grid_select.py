"""White-box time and memory model of one training step on B200 nodes, and the grid chooser built on it.

What the model answers: for a graph ``(N, E_attn, E_gcn, f_in)``, a model ``(d, H, L)`` and ``P`` GPUs, how long does one
epoch take and how many bytes does a rank hold at its peak, for each way of laying the ranks out — the fused 2D grid
``(P_d, P_o)``, the head grid ``(P_d, P_o, P_i)``, the ring ``(P, 1)`` and the streamed (recomputing) layer — and
therefore which layout to run.  It plays the role of the reference's ``gt3d/gt3d/dist/grid_select.py`` (cost functions
``:278-500``, layer models ``:543-930``, memory models ``:705,829,932``, selectors ``:858,990-1039``) with a different
hardware picture:

* one node is 8 GPUs behind NVSwitch: every group that fits in a node sees the same per-rank bandwidth whatever its
  stride, so "placement" only matters for groups that leave the node;
* the dense work runs in bf16 on the tcgen05 GEMM, the sparse work in the gather kernels whose cost is linear in
  (edges, rows, columns) with an L2-resident and an HBM-resident slope (126 MB L2);
* a step is replayed as one CUDA graph, so there is no per-op host floor, only a per-kernel device gap;
* capacity is 180 GB per GPU.

Every constant lives in ``HW`` (defaults measured on B200 or, where marked, nominal) and can be replaced by a JSON
written by ``gt_b200.bench.hw_constants`` / ``gt_b200.bench.kernel_constants`` (``load_constants``).
All functions are pure host arithmetic.
"""
import dataclasses
import json
import math
import os

GB = 2 ** 30
GPUS_PER_NODE = 8
CAPACITY_GB = 180.0
HEADROOM = 0.92

HW = dict(
    hbm_gbs=6550.0,                 # STREAM-style copy, measured
    ew_gbs=4800.0,                  # fused row kernels (LayerNorm / residual / dropout): achieved bytes per second
    kernel_gap_us=1.6,              # device gap between dependent kernels inside a replayed CUDA graph
    l2_bytes=126e6,
    # bf16 GEMM, [rows, d] x [d, n_out]: achieved TFLOP/s by d (fwd, grad-input, grad-weight); rows >= 100K
    gemm_tflops={128: (210.0, 210.0, 120.0), 256: (420.0, 420.0, 260.0), 512: (700.0, 700.0, 450.0)},
    gemm_floor_us=6.0,
    # gather-attention kernels: ns per (edge, row, column) for H*D = 256 bf16; "l2" when K|V of the column block fit in L2
    attn=dict(fwd=dict(l2=(0.25, 1.6, 0.0), hbm=(0.55, 1.6, 0.0)),
              bwd=dict(l2=(0.56, 4.5, 4.0), hbm=(1.20, 4.5, 4.0))),
    attn_ref_width=256,
    spmm=dict(l2=0.12, hbm=0.30, row_ns=0.9),             # ns per edge (d = 256 bf16) and per output row
    # collectives inside an NVSwitch node: latency (us) and per-rank payload rate (GB/s received or sent) at large sizes
    coll=dict(ag=(14.0, 560.0), rs=(14.0, 520.0), a2a=(16.0, 480.0), ar=(18.0, 360.0), p2p=(6.0, 700.0)),
    coll_half_mb=2.0,               # payload at which half the large-size rate is reached
    # collectives issued from inside compute kernels over peer memory (epoch channel + loads / stores over NVLink): flag
    # latency and achieved rate per rank
    fused_coll=dict(alpha_us=6.0, gbs=600.0),
    # arrival skew: ranks reach a wait at different times (unequal blocks, kernel tails on small blocks), and the step runs at the
    # speed of the last one; measured as the share of the layers' time by which multi-rank steps exceed the sum of their parts
    # (0.12 from the 2-, 4- and 8-GPU rows of bench/model_validation_data.py)
    sync_skew=0.12,
    # across nodes: one 400 Gb/s NIC per GPU (nominal; not measured on this pool)
    inter=dict(alpha_us=28.0, gbs=46.0),
    a2a_over_ag=1.25,               # cost of moving the same bytes by all-to-all-v instead of a dense all-gather
    # tensors kept for backward per layer, in units of one bf16 block of the named extent x d
    saved=dict(own=11.0, own_mask=0.0, row=2.0, col=3.0, head_own=14.0, stats_per_row=12.0),
    struct_bytes_per_edge=22.0,     # CSR + CSC (int32 indices, uint8 types, int32 permutation) + segment plans
    # analytic model of a gather pass (attn_theory_ms): fixed ns per row and achieved share of hbm_gbs on long rows, from the
    # regular-block degree sweep of gt_b200.bench.kernel_theory (262,144 rows, 8 x 32 bf16)
    theory=dict(fwd=dict(tau_ns=0.41, bw_eff=0.89), bwd=dict(tau_ns=1.30, bw_eff=0.68)),
)

_DEFAULT_JSON = os.path.join(os.path.dirname(__file__), "b200_constants.json")


def load_constants(path=None):
    """Overlay ``HW`` with a JSON of measured constants (same keys; nested dicts are merged).  Returns the keys replaced."""
    path = path or _DEFAULT_JSON
    if not os.path.exists(path):
        return []
    with open(path) as f:
        new = json.load(f)

    def merge(dst, src):
        for k, v in src.items():
            if isinstance(v, dict) and isinstance(dst.get(k), dict):
                merge(dst[k], v)
            else:
                dst[k] = v if not isinstance(v, list) else tuple(v)
    if "gemm_tflops" in new:
        new["gemm_tflops"] = {int(k): tuple(v) for k, v in new["gemm_tflops"].items()}
        HW["gemm_tflops"] = {}
    merge(HW, {k: v for k, v in new.items() if not k.startswith("_")})
    return sorted(new)


load_constants()


@dataclasses.dataclass
class Graph:
    n: int
    e_attn: int
    e_gcn: int
    f_in: int = 128
    name: str = None
    classes: int = 40
    exp_deg: int = 3
    kappa: float = 0.8             # dispersion of the degree distribution (negative binomial); None: Poisson
    skew: float = 1.0              # sparse-kernel time on this graph's blocks / on random blocks of the same shape (measured)
    token: bool = False            # a global token: one row and one column with n entries each (counted in e_attn)

    @property
    def deg_attn(self):
        return self.e_attn / max(self.n, 1)


@dataclasses.dataclass
class Model:
    hidden: int = 256
    heads: int = 8
    layers: int = 4
    bf16: bool = True
    with_gcn: bool = True
    ffn_mult: int = 2
    sparse_comm: bool = False
    transport: str = "nccl"        # "nccl" or "p2p" (peer-memory kernels: lower latency, pull instead of a2a-v)
    token_dense: bool = False      # the global token as dense terms on the owned rows (parallel/token_dense.py), not as 2 n edges

    @property
    def wire_bytes(self):
        return 2

    @property
    def act_bytes(self):
        return 2 if self.bf16 else 4


@dataclasses.dataclass
class Choice:
    grid: tuple
    ms: float
    gb: float
    family: str = "fused"
    n_sub: int = 1
    fits: bool = True
    ranked: list = dataclasses.field(default_factory=list, repr=False)


# ----------------------------------------------------------------------------------------------------------------------
# primitives
# ----------------------------------------------------------------------------------------------------------------------
def placement(pd, po, pi=1, gpn=GPUS_PER_NODE):
    """``{group: (ranks per node, nodes)}`` for rank = (r P_o + c) P_i + h: the head group is P_i consecutive ranks, the
    row group has stride P_i, the column group stride P_o P_i."""
    def layout(size, stride):
        if size * stride <= gpn:
            return (size, 1)
        per_node = min(max(1, gpn // stride), size)
        return (per_node, max(1, size // per_node))
    return dict(head=layout(pi, 1), row=layout(po, pi), col=layout(pd, po * pi))


def cross_node_groups(pd, po, pi=1, gpn=GPUS_PER_NODE):
    return sum(1 for _, m in placement(pd, po, pi, gpn).values() if m > 1)


def coll_ms(kind, layout, nbytes, transport="nccl"):
    """Time of one collective whose per-rank payload from / to its peers is ``nbytes``; ``layout = (ranks per node, nodes)``."""
    k, m = layout
    g = k * m
    if g <= 1 or nbytes <= 0:
        return 0.0
    alpha, rate = HW["coll"]["p2p" if transport == "p2p" and kind != "a2a" else kind]
    half = HW["coll_half_mb"] * 2 ** 20
    inside = nbytes * (k - 1) / (g - 1)
    t = alpha / 1e3 + (inside + half * (inside > 0)) / (rate * 1e6) if k > 1 else 0.0
    if m > 1:
        outside = nbytes - inside
        t += HW["inter"]["alpha_us"] / 1e3 * math.ceil(math.log2(m) + 1) + outside / (HW["inter"]["gbs"] * 1e6)
    return t


def nonempty_fraction(lam, kappa=0.8):
    """Share of rows with at least one edge in a block when a row has ``lam`` edges there on average (negative-binomial
    degrees with dispersion ``kappa``; Poisson for ``kappa=None``)."""
    if kappa is None or kappa > 1e6:
        return 1.0 - math.exp(-lam)
    return 1.0 - (1.0 + lam / kappa) ** (-kappa)


def sparse_share(g: Graph, p: int):
    """Share of a gathered block's rows that a tile really references when the other grid axis has ``p`` parts: a row is
    touched by its graph edges with the negative-binomial law, and by its 2·exp_deg expander edges uniformly."""
    if p <= 1:
        return 1.0
    graph_deg = max(g.deg_attn - 2 * g.exp_deg, 0.0)
    miss = (1.0 - nonempty_fraction(graph_deg / p, g.kappa)) * (1.0 - 1.0 / p) ** (2 * g.exp_deg)
    return 1.0 - miss


def sparse_coll_ms(kind, layout, nbytes, share, m: Model):
    dense = coll_ms(kind, layout, nbytes, m.transport)
    if not m.sparse_comm or share >= 1.0:
        return dense
    if m.transport == "p2p":                                     # receiver-driven pull of the needed rows
        sparse = coll_ms(kind, layout, nbytes * share, "p2p") * 1.1
    else:
        sparse = coll_ms("a2a", layout, nbytes * share) * HW["a2a_over_ag"]
    return min(dense, sparse)


def fused_coll_ms(nbytes, group, hidden_ms):
    """A collective issued from inside a compute kernel over peer memory: flag latency plus the part of the transfer that the
    issuing kernel (``hidden_ms``) does not cover; nothing for a group of one."""
    if group <= 1 or nbytes <= 0:
        return 0.0
    fc = HW["fused_coll"]
    return fc["alpha_us"] / 1e3 + max(nbytes / (fc["gbs"] * 1e6) - hidden_ms, 0.0)


def gemm_ms(flops, d, which=0):
    tab = HW["gemm_tflops"]
    keys = sorted(tab)
    if d <= keys[0]:
        tf = tab[keys[0]][which] * d / keys[0]
    elif d >= keys[-1]:
        tf = tab[keys[-1]][which]
    else:
        lo = max(k for k in keys if k <= d)
        hi = min(k for k in keys if k >= d)
        w = 0.0 if hi == lo else (d - lo) / (hi - lo)
        tf = tab[lo][which] * (1 - w) + tab[hi][which] * w
    return max(flops / (tf * 1e9), HW["gemm_floor_us"] / 1e3) if flops > 0 else 0.0


def ew_ms(nbytes, n_kernels=1):
    return nbytes / (HW["ew_gbs"] * 1e6) + n_kernels * HW["kernel_gap_us"] / 1e3


def _resident(cols, width_bytes):
    """Weight of the L2-resident slope: 1 while the gathered operand fits in half of L2, falling to 0 at twice L2."""
    ws = cols * width_bytes
    lo, hi = 0.5 * HW["l2_bytes"], 2.0 * HW["l2_bytes"]
    return 1.0 if ws <= lo else 0.0 if ws >= hi else (hi - ws) / (hi - lo)


def attn_ms(e, rows, cols, heads, d_head, direction, skew=1.0):
    """Gather-attention kernels on a block with ``e`` edges, ``rows`` destination rows, ``cols`` source rows."""
    width = heads * d_head
    scale = width / HW["attn_ref_width"]
    w = _resident(cols, 2 * width * 2)                           # K and V rows, bf16
    a, b = HW["attn"][direction]["l2"], HW["attn"][direction]["hbm"]
    ce, cr, cc = (w * x + (1 - w) * y for x, y in zip(a, b))
    n_k = 1 if direction == "fwd" else 3
    return (ce * e * skew + cr * rows + cc * cols) * scale / 1e6 + n_k * HW["kernel_gap_us"] / 1e3


def attn_theory_bytes(e, rows, width, direction, elem=2):
    """Bytes an ideal gather pass without cache reuse moves: per edge the gathered rows and index / type words, per row
    its own operands and results (forward: K and V per edge, q in, fp32 acc + statistics out; backward: twice that per
    edge for the row and the column pass, six operand / result rows per node)."""
    if direction == "fwd":
        return e * (2 * width * elem + 8) + rows * (width * elem + width * 4 + 32)
    return 2 * e * (2 * width * elem + 8) + rows * (6 * width * elem + 64)


def attn_theory_ms(e, rows, heads, d_head, direction):
    """First-principles time of a gather pass on operands larger than L2: a fixed cost per row (the latency of the row's
    pointer / q / result chain, ``tau_ns``) plus the pass's bytes over the achieved share of the memory bandwidth.  Two
    constants per pass instead of the fitted slopes of ``attn_ms``; it extrapolates over widths (bytes scale, ``tau``
    does not) and is exact to a few percent on the forward sweep (reference: ``THEORY`` / ``_theory_pass_ms``,
    ``gt3d/gt3d/perf/grid_select.py:376-426``)."""
    th = HW["theory"][direction]
    nbytes = attn_theory_bytes(e, rows, heads * d_head, direction)
    return (rows * th["tau_ns"] + nbytes / (HW["hbm_gbs"] * th["bw_eff"])) / 1e6


def spmm_ms(e, rows, cols, d, skew=1.0):
    w = _resident(cols, d * 2)
    ce = w * HW["spmm"]["l2"] + (1 - w) * HW["spmm"]["hbm"]
    return (ce * e * skew + HW["spmm"]["row_ns"] * rows) * (d / 256.0) / 1e6 + HW["kernel_gap_us"] / 1e3


# ----------------------------------------------------------------------------------------------------------------------
# layer families
# ----------------------------------------------------------------------------------------------------------------------
def fused_layer_ms(pd, po, g: Graph, m: Model, gpn=GPUS_PER_NODE):
    """(forward parts, backward parts) in ms of one fused layer on the (pd, po) grid: gather x over both groups, project
    on the gathered blocks, SpMM + attention on the tile, one reduce-scatter of ``[acc | l | agg]``, owned-row tail."""
    P = pd * po
    d, H, b, a = m.hidden, m.heads, m.wire_bytes, m.act_bytes
    R, C, O = g.n / pd, g.n / po, g.n / P
    ea, eg = g.e_attn / P, g.e_gcn / P
    if g.token and m.token_dense:
        ea = (g.e_attn - 2 * g.n) / P                        # the token's row and column are not edges (dense terms below)
    elif g.token and P > 1:
        # The token's row lies in ONE row block (n / po entries for each rank of that row group) and its column in ONE column
        # block (n / pd entries per rank of that column group): the rank that has both is the straggler every other rank waits
        # for at the next collective, so the step runs at its speed.
        ea = (g.e_attn - 2 * g.n) / P + g.n / po + g.n / pd
    pl = placement(pd, po, 1, gpn)
    sh_c, sh_r = sparse_share(g, pd), sparse_share(g, po)
    w = (2 * d if m.with_gcn else d) + 2 * H
    proj = 2 * d * d * ((3 if m.with_gcn else 2) * C + R)
    f, bw = {}, {}
    f["gemm"] = gemm_ms(proj, d, 0)
    f["spmm"] = spmm_ms(eg, R, C, d, g.skew) if m.with_gcn else 0.0
    f["attn"] = attn_ms(ea, R, C, H, d // H, "fwd", g.skew)
    f["tail"] = ew_ms(O * d * a * 10, 3) + gemm_ms(2 * O * d * d * 2 * m.ffn_mult, d, 0)
    bw["tail"] = ew_ms(O * d * a * 16, 4) + gemm_ms(2 * O * d * d * 2 * m.ffn_mult, d, 1) + gemm_ms(2 * O * d * d * 2 * m.ffn_mult, d, 2)
    bw["attn"] = attn_ms(ea, R, C, H, d // H, "bwd", g.skew)
    bw["spmm"] = spmm_ms(eg, C, R, d, g.skew) if m.with_gcn else 0.0
    bw["gemm"] = gemm_ms(proj, d, 1) + gemm_ms(proj, d, 2)
    if g.token and m.token_dense:
        # two [O, d] x [d, H] products and one [H, O] x [O, d] product (at the GEMM floor), one cast of x and one update of acc
        # ([O, d] fp32 read + write), a dozen small kernels on [O, H], and two all-reduces of a few hundred numbers per direction
        # (an estimate from the model's primitives: not measured)
        small = coll_ms("ar", (min(P, gpn), max(1, P // gpn)), 4 * (d + H + 8), m.transport)
        f["token"] = 3 * gemm_ms(2 * O * d * H, d, 0) + ew_ms(O * d * (2 + 4 + 8), 16) + 2 * small
        bw["token"] = 6 * gemm_ms(2 * O * d * H, d, 1) + ew_ms(O * d * (4 + 8 + 8), 32) + 2 * small
    if m.transport == "p2p" and not m.sparse_comm and pl["row"][1] == 1 and pl["col"][1] == 1:
        # (both groups within one machine; a group that crosses machines takes the operator off the peer-memory path and the layer
        # runs with NCCL collectives for that group: the branch below is then the estimate)
        # collectives inside the compute kernels (peer memory, epoch channels): the transfer hides behind the kernel that
        # issues it; what remains is the flag latency, the part of the transfer that outlasts the kernel, and the owner-side
        # slot sums / unpacking passes
        f["gather"] = fused_coll_ms((C - O) * d * b, pd, f["gemm"] * 0.75) + fused_coll_ms((R - O) * d * b, po, f["gemm"] * 0.25)
        f["combine"] = fused_coll_ms((R - O) * w * b, po, f["attn"] + f["spmm"]) + (ew_ms(O * w * (po * b + 4), 1) if po > 1 else 0.0)
        bw["combine"] = fused_coll_ms((R - O) * w * b, po, 0.0) + (ew_ms(R * w * (b + 3), 2) if po > 1 else 0.0)
        bw["dx"] = fused_coll_ms((C - O) * d * b, pd, bw["gemm"] * 0.4) + fused_coll_ms((R - O) * d * b, po, bw["gemm"] * 0.1) \
            + ew_ms(O * d * b * (pd + po + 1), (pd > 1) + (po > 1))
    else:
        f["gather"] = sparse_coll_ms("ag", pl["col"], (C - O) * d * b, sh_c, m) + sparse_coll_ms("ag", pl["row"], (R - O) * d * b, sh_r, m)
        f["combine"] = sparse_coll_ms("rs", pl["row"], (R - O) * w * b, sh_r, m) + (ew_ms(R * w * (4 + b), 1) if po > 1 else 0.0)
        bw["combine"] = sparse_coll_ms("ag", pl["row"], (R - O) * w * b, sh_r, m)
        bw["dx"] = sparse_coll_ms("rs", pl["col"], (C - O) * d * b, sh_c, m) + sparse_coll_ms("rs", pl["row"], (R - O) * d * b, sh_r, m) \
            + ew_ms((C + R) * d * a * 2 + O * d * a * 3, 3)
    return f, bw


def fixed_step_ms(P, g: Graph, m: Model, gpn=GPUS_PER_NODE):
    """Work outside the layers: input projection + norm, classifier + loss, gradient all-reduce, clipping + AdamW."""
    O, d = g.n / P, m.hidden
    pre = sum(gemm_ms(2 * O * g.f_in * d, min(g.f_in, d), k) for k in range(3)) + ew_ms(O * (g.f_in + 6 * d) * m.act_bytes, 6)
    head = gemm_ms(2 * O * d * g.classes, d, 0) * 3 + ew_ms(O * g.classes * 4 * 3, 3)
    n_params = m.layers * (12 * d * d + 2 * m.ffn_mult * d * d - 4 * d * d) + g.f_in * d + d * g.classes
    lay = (min(P, gpn), max(1, P // gpn))
    ar = coll_ms("ar", lay, 2 * n_params * 4, m.transport) if P > 1 else 0.0
    opt = ew_ms(n_params * 4 * 7, 3)
    return pre + head + ar + opt


def predict_fused_ms(pd, po, g: Graph, m: Model, gpn=GPUS_PER_NODE, breakdown=False):
    f, bw = fused_layer_ms(pd, po, g, m, gpn)
    fixed = fixed_step_ms(pd * po, g, m, gpn)
    layers = m.layers * (sum(f.values()) + sum(bw.values()))
    skew = HW["sync_skew"] * layers if pd * po > 1 else 0.0
    total = layers + skew + fixed
    if breakdown:
        parts = {k: m.layers * v for k, v in f.items()}
        parts.update({"bwd " + k: m.layers * v for k, v in bw.items()})
        parts["fixed"] = fixed
        parts["arrival skew"] = skew
        return total, parts
    return total


def attn_operator_ms(pd, po, pi, g: Graph, m: Model, family="fused", gpn=GPUS_PER_NODE):
    """Forward + backward of the distributed attention operator alone (projections included), 2D fused or head grid."""
    P = pd * po * pi
    d, H, b = m.hidden, m.heads, m.wire_bytes
    pl = placement(pd, po, pi, gpn)
    sh_c, sh_r = sparse_share(g, pd), sparse_share(g, po)
    O = g.n / P
    if family == "fused":
        R, C = g.n / pd, g.n / po
        ea, w = g.e_attn / P, d + 2 * H
        proj = 2 * d * d * (2 * C + R)
        fwd = sparse_coll_ms("ag", pl["col"], (C - O) * d * b, sh_c, m) + sparse_coll_ms("ag", pl["row"], (R - O) * d * b, sh_r, m) \
            + gemm_ms(proj, d, 0) + attn_ms(ea, R, C, H, d // H, "fwd", g.skew) + sparse_coll_ms("rs", pl["row"], (R - O) * w * b, sh_r, m)
        bwd = sparse_coll_ms("ag", pl["row"], (R - O) * w * b, sh_r, m) + attn_ms(ea, R, C, H, d // H, "bwd", g.skew) \
            + gemm_ms(proj, d, 1) + gemm_ms(proj, d, 2) + sparse_coll_ms("rs", pl["col"], (C - O) * d * b, sh_c, m) \
            + sparse_coll_ms("rs", pl["row"], (R - O) * d * b, sh_r, m) + ew_ms((C + R) * d * 4, 2)
        return fwd + bwd
    Rq, Rkv, ds, Hs = g.n / pd, g.n / po, d / pi, max(H // pi, 1)
    ea, w = g.e_attn / (pd * po), d / pi + 2 * Hs
    a2a = lambda nb: coll_ms("a2a", pl["head"], nb * (1 - 1 / pi)) if pi > 1 else 0.0      # noqa: E731
    fwd = gemm_ms(3 * 2 * O * d * d, d, 0) + 3 * a2a(O * d * b) + 2 * sparse_coll_ms("ag", pl["col"], (Rkv - O * pi) * ds * b, sh_c, m) \
        + sparse_coll_ms("ag", pl["row"], (Rq - O * pi) * ds * b, sh_r, m) + attn_ms(ea, Rq, Rkv, Hs, d // H, "fwd", g.skew) \
        + sparse_coll_ms("rs", pl["row"], (Rq - O * pi) * w * b, sh_r, m) + a2a(O * d * b) + ew_ms(O * d * b * 8, 4)
    bwd = a2a(O * d * b) + sparse_coll_ms("ag", pl["row"], (Rq - O * pi) * w * b, sh_r, m) + attn_ms(ea, Rq, Rkv, Hs, d // H, "bwd", g.skew) \
        + sparse_coll_ms("rs", pl["row"], (Rq - O * pi) * ds * b, sh_r, m) + 2 * sparse_coll_ms("rs", pl["col"], (Rkv - O * pi) * ds * b, sh_c, m) \
        + 3 * a2a(O * d * b) + gemm_ms(3 * 2 * O * d * d, d, 1) + gemm_ms(3 * 2 * O * d * d, d, 2) + ew_ms(O * d * b * 8, 4)
    return fwd + bwd


def head_gcn_ms(pd, po, pi, g: Graph, m: Model, gpn=GPUS_PER_NODE):
    """GCN branch on the head grid: the message projection's d / P_i slice rides in the K | V exchange; SpMM on the slice."""
    P = pd * po * pi
    d, b = m.hidden, m.wire_bytes
    O, Rq, Rkv, ds = g.n / P, g.n / pd, g.n / po, m.hidden / pi
    eg = g.e_gcn / (pd * po)
    pl = placement(pd, po, pi, gpn)
    sh_c, sh_r = sparse_share(g, pd), sparse_share(g, po)
    a2a = lambda nb: coll_ms("a2a", pl["head"], nb * (1 - 1 / pi)) if pi > 1 else 0.0      # noqa: E731
    one_way = gemm_ms(2 * O * d * d, d, 0) + a2a(O * d * b) + sparse_coll_ms("ag", pl["col"], (Rkv - O * pi) * ds * b, sh_c, m) \
        + spmm_ms(eg, Rq, Rkv, ds, g.skew) + sparse_coll_ms("rs", pl["row"], (Rq - O * pi) * ds * b, sh_r, m) + a2a(O * d * b)
    return 2 * one_way + gemm_ms(2 * O * d * d, d, 2)


def _tail_ms(O, m: Model):
    d = m.hidden
    ffn = 2 * O * d * d * 2 * m.ffn_mult
    return ew_ms(O * d * m.act_bytes * 26, 7) + gemm_ms(ffn, d, 0) + gemm_ms(ffn, d, 1) + gemm_ms(ffn, d, 2)


def predict_head_ms(pd, po, pi, g: Graph, m: Model, gpn=GPUS_PER_NODE, breakdown=False):
    P = pd * po * pi
    op = attn_operator_ms(pd, po, pi, g, m, "head", gpn)
    gcn = head_gcn_ms(pd, po, pi, g, m, gpn) if m.with_gcn else 0.0
    tail, fixed = _tail_ms(g.n / P, m), fixed_step_ms(P, g, m, gpn)
    total = m.layers * (op + gcn + tail) + fixed
    if breakdown:
        return total, {"attention operator": m.layers * op, "gcn": m.layers * gcn, "tail": m.layers * tail, "fixed": fixed}
    return total


def ring_layer_ms(P, g: Graph, m: Model, gpn=GPUS_PER_NODE):
    """x-rotating ring on (P, 1): P steps; each re-projects K, V (and the GCN message) of the visiting chunk, runs the
    kernels on a [N/P, N/P] tile; hop h+1 travels while step h computes; backward recomputes and carries dx along."""
    d, H, b = m.hidden, m.heads, m.wire_bytes
    O = g.n / P
    ea, eg = g.e_attn / (P * P), g.e_gcn / (P * P)
    lay = (min(P, gpn), max(1, P // gpn))
    hop = coll_ms("ag", (2, 1) if lay[1] == 1 else (1, 2), O * d * b, "p2p" if m.transport == "p2p" else "nccl")
    nproj = 3 if m.with_gcn else 2
    step_f = gemm_ms(2 * O * d * d * nproj, d, 0) + attn_ms(ea, O, O, H, d // H, "fwd", g.skew) + (spmm_ms(eg, O, O, d, g.skew) if m.with_gcn else 0.0)
    step_b = gemm_ms(2 * O * d * d * nproj, d, 0) + attn_ms(ea, O, O, H, d // H, "bwd", g.skew) + (spmm_ms(eg, O, O, d, g.skew) if m.with_gcn else 0.0) \
        + gemm_ms(2 * O * d * d * nproj, d, 1) + gemm_ms(2 * O * d * d * nproj, d, 2) + ew_ms(O * d * 4 * 3, 2)
    fwd = gemm_ms(2 * O * d * d, d, 0) + P * max(step_f, hop) + hop
    bwd = P * max(step_b, 2 * hop) + 2 * hop + gemm_ms(2 * O * d * d, d, 1) + gemm_ms(2 * O * d * d, d, 2)
    return fwd, bwd


def predict_ring_ms(P, g: Graph, m: Model, gpn=GPUS_PER_NODE, breakdown=False):
    fwd, bwd = ring_layer_ms(P, g, m, gpn)
    tail, fixed = _tail_ms(g.n / P, m), fixed_step_ms(P, g, m, gpn)
    total = m.layers * (fwd + bwd + tail) + fixed
    if breakdown:
        return total, {"ring fwd": m.layers * fwd, "ring bwd": m.layers * bwd, "tail": m.layers * tail, "fixed": fixed}
    return total


def streamed_layer_ms(pd, po, n_sub, g: Graph, m: Model, gpn=GPUS_PER_NODE, overlap=True):
    """Streamed layer: the column block arrives in ``n_sub`` sub-blocks; each is projected, consumed and dropped; backward
    re-gathers and re-projects it.  With ``overlap`` the gather of sub-block s+1 hides behind the compute of s."""
    P = pd * po
    d, H, b = m.hidden, m.heads, m.wire_bytes
    R, C, O = g.n / pd, g.n / po, g.n / P
    cs = C / n_sub
    ea, eg = g.e_attn / P / n_sub, g.e_gcn / P / n_sub
    pl = placement(pd, po, 1, gpn)
    sh_r = sparse_share(g, po)
    sh_s = sparse_share(g, pd * n_sub)
    w = (2 * d if m.with_gcn else d) + 2 * H
    nproj = 3 if m.with_gcn else 2
    live = nonempty_fraction(g.deg_attn / (po * n_sub), g.kappa)              # rows of the tile that a sub-block touches
    gat = sparse_coll_ms("ag", pl["col"], cs * (1 - 1 / pd) * d * b, sh_s, m)
    comp_f = gemm_ms(2 * cs * d * d * nproj, d, 0) + attn_ms(ea, R * live, cs, H, d // H, "fwd", g.skew) + (spmm_ms(eg, R * live, cs, d, g.skew) if m.with_gcn else 0.0)
    comp_b = comp_f + attn_ms(ea, R * live, cs, H, d // H, "bwd", g.skew) + (spmm_ms(eg, cs, R * live, d, g.skew) if m.with_gcn else 0.0) \
        + gemm_ms(2 * cs * d * d * nproj, d, 1) + gemm_ms(2 * cs * d * d * nproj, d, 2)
    rs_sub = sparse_coll_ms("rs", pl["col"], cs * (1 - 1 / pd) * d * b, sh_s, m)
    row = sparse_coll_ms("ag", pl["row"], (R - O) * d * b, sh_r, m) + gemm_ms(2 * R * d * d, d, 0)
    if overlap:
        fwd = row + gat + n_sub * max(comp_f, gat)
        bwd = row + gat + n_sub * max(comp_b, gat + rs_sub) + rs_sub
    else:
        fwd = row + n_sub * (comp_f + gat)
        bwd = row + n_sub * (comp_b + gat + rs_sub)
    fwd += sparse_coll_ms("rs", pl["row"], (R - O) * w * b, sh_r, m)
    bwd += sparse_coll_ms("ag", pl["row"], (R - O) * w * b, sh_r, m) + gemm_ms(2 * R * d * d, d, 1) + gemm_ms(2 * R * d * d, d, 2) \
        + sparse_coll_ms("rs", pl["row"], (R - O) * d * b, sh_r, m)
    return fwd, bwd


def predict_streamed_ms(pd, po, n_sub, g: Graph, m: Model, gpn=GPUS_PER_NODE, overlap=True):
    fwd, bwd = streamed_layer_ms(pd, po, n_sub, g, m, gpn, overlap)
    return m.layers * (fwd + bwd + _tail_ms(g.n / (pd * po), m)) + fixed_step_ms(pd * po, g, m, gpn)


# ----------------------------------------------------------------------------------------------------------------------
# memory
# ----------------------------------------------------------------------------------------------------------------------
def _base_bytes(P, g: Graph, m: Model, replicas=1):
    n_params = m.layers * (8 + 4 * m.ffn_mult) * m.hidden ** 2 + g.f_in * m.hidden
    return g.n / P * g.f_in * m.act_bytes + (g.e_attn + (g.e_gcn if m.with_gcn else 0)) * replicas / P * HW["struct_bytes_per_edge"] \
        + n_params * 4 * 4


def peak_memory_bytes(pd, po, g: Graph, m: Model, n_sub=1, streamed=False, layer_ckpt=False, breakdown=False):
    """Peak bytes per rank of the fused (or streamed) 2D layer: structures + features + parameters/optimizer state +
    L x tensors saved for backward + the transient of one layer's backward."""
    P = pd * po
    d, H, a = m.hidden, m.heads, m.act_bytes
    R, C, O = g.n / pd, g.n / po, g.n / P
    s = HW["saved"]
    base = _base_bytes(P, g, m)
    w = (2 * d if m.with_gcn else d) + 2 * H
    if streamed:
        cs = C / max(n_sub, 1)
        tail = m.layers * (s["own"] * O * d * a)
        sub = 2 * cs * d * a + (3 if m.with_gcn else 2) * cs * d * a
        work = R * d * a * 2 + R * w * 4 + sub + 3 * cs * d * 4 + R * d * 4
        structs = n_sub * R * 17
        total = base + tail + work + structs
        return dict(base=base, owned=tail, transient=work, structs=structs) if breakdown else total
    gathered = (s["col"] if m.with_gcn else s["col"] - 1) * C * d * a + s["row"] * R * d * a + s["stats_per_row"] * R * H
    owned = s["own"] * O * d * a
    transient = R * w * 4 * 2 + R * d * 4 + 3 * C * d * 4
    if layer_ckpt:
        total = base + m.layers * O * d * a + gathered + owned + transient
    else:
        total = base + m.layers * (gathered + owned) + transient
    if breakdown:
        k = 1 if layer_ckpt else m.layers
        return dict(base=base, gathered=k * gathered, owned=k * owned + (m.layers * O * d * a if layer_ckpt else 0), transient=transient)
    return total


def peak_memory_head_bytes(pd, po, pi, g: Graph, m: Model, layer_ckpt=False):
    P = pd * po * pi
    d, a = m.hidden, m.act_bytes
    Hs, ds = max(m.heads // pi, 1), m.hidden / pi
    O, Rq, Rkv = g.n / P, g.n / pd, g.n / po
    s = HW["saved"]
    base = _base_bytes(P, g, m, replicas=pi)
    per_layer = (2 + (1 if m.with_gcn else 0)) * Rkv * ds * a + Rq * ds * a + s["stats_per_row"] * Rq * Hs + s["head_own"] * O * d * a
    transient = Rq * (ds + 2 * Hs) * 4 * 2 + Rq * ds * 4 + 2 * Rkv * ds * 4
    if layer_ckpt:
        return base + m.layers * O * d * a + per_layer + transient
    return base + m.layers * per_layer + transient


def peak_memory_ring_bytes(P, g: Graph, m: Model):
    d, a = m.hidden, m.act_bytes
    O = g.n / P
    base = _base_bytes(P, g, m)
    per_layer = HW["saved"]["own"] * O * d * a + O * (d * 4 + 2 * m.heads * 4)
    transient = 4 * O * d * m.wire_bytes + 6 * O * d * 4
    return base + m.layers * per_layer + transient


# ----------------------------------------------------------------------------------------------------------------------
# selection
# ----------------------------------------------------------------------------------------------------------------------
def attention_edges(num_nodes, num_edges, exp_deg):
    """Attention edges of the Exphormer graph: graph edges (directed count) + self loops + both directions of the expander."""
    return num_edges + num_nodes + 2 * exp_deg * num_nodes


def candidate_grids(world):
    return [(pd, world // pd) for pd in range(1, world + 1) if world % pd == 0]


def candidate_grids_3d(world, heads, max_pi=None):
    out = []
    for pi in range(2, world + 1):
        if world % pi or heads % pi or (max_pi and pi > max_pi):
            continue
        out += [(pd, po, pi) for pd, po in candidate_grids(world // pi)]
    return out


def _rank(cands, capacity_gb, headroom):
    cands.sort(key=lambda c: c.ms)
    for c in cands:
        c.fits = c.gb <= capacity_gb * headroom
    fits = [c for c in cands if c.fits]
    best = fits[0] if fits else None
    if best is not None:
        best.ranked = cands
    return best


def select_grid(world, g: Graph, m: Model, n_sub=1, streamed=False, gpn=GPUS_PER_NODE, capacity_gb=CAPACITY_GB,
                headroom=HEADROOM, layer_ckpt=False):
    """Fastest predicted 2D grid among those that fit in memory.  Raises if none fits (try streaming / checkpointing)."""
    cands = []
    for pd, po in candidate_grids(world):
        gb = peak_memory_bytes(pd, po, g, m, n_sub, streamed, layer_ckpt) / GB
        ms = predict_streamed_ms(pd, po, n_sub, g, m, gpn) if streamed else predict_fused_ms(pd, po, g, m, gpn)
        cands.append(Choice((pd, po), ms, gb, "streamed" if streamed else "fused", n_sub))
    best = _rank(cands, capacity_gb, headroom)
    if best is None:
        raise MemoryError(f"no 2D grid of {world} GPUs fits {capacity_gb * headroom:.0f} GB: smallest needs {min(c.gb for c in cands):.1f} GB")
    return best


def select_grid_streamed(world, g: Graph, m: Model, n_sub_choices=(2, 4, 8, 16, 32, 64, 128), gpn=GPUS_PER_NODE,
                         capacity_gb=CAPACITY_GB, headroom=HEADROOM):
    """Per grid the smallest ``n_sub`` that fits, then the fastest of those; ``None`` if nothing fits."""
    cands = []
    for pd, po in candidate_grids(world):
        for n_sub in n_sub_choices:
            gb = peak_memory_bytes(pd, po, g, m, n_sub, True) / GB
            if gb <= capacity_gb * headroom:
                cands.append(Choice((pd, po), predict_streamed_ms(pd, po, n_sub, g, m, gpn), gb, "streamed", n_sub))
                break
    return _rank(cands, capacity_gb, headroom)


def select_grid_head(world, g: Graph, m: Model, gpn=GPUS_PER_NODE, capacity_gb=CAPACITY_GB, headroom=HEADROOM, max_pi=None):
    cands = [Choice(c, predict_head_ms(*c, g, m, gpn), peak_memory_head_bytes(*c, g, m) / GB, "head")
             for c in candidate_grids_3d(world, m.heads, max_pi)]
    return _rank(cands, capacity_gb, headroom) if cands else None


def select_layout(world, g: Graph, m: Model, gpn=GPUS_PER_NODE, capacity_gb=CAPACITY_GB, headroom=HEADROOM):
    """Best of the fused 2D grids and the head grids (``--head_auto``)."""
    cands = []
    for pd, po in candidate_grids(world):
        cands.append(Choice((pd, po), predict_fused_ms(pd, po, g, m, gpn), peak_memory_bytes(pd, po, g, m) / GB, "fused"))
    for c in candidate_grids_3d(world, m.heads):
        cands.append(Choice(c, predict_head_ms(*c, g, m, gpn), peak_memory_head_bytes(*c, g, m) / GB, "head"))
    best = _rank(cands, capacity_gb, headroom)
    if best is None:
        raise MemoryError(f"no layout of {world} GPUs fits {capacity_gb * headroom:.0f} GB")
    return best


def auto_checkpoint(pd, po, g: Graph, m: Model, capacity_gb=CAPACITY_GB, headroom=HEADROOM):
    """``--auto_ckpt``: per-layer activation checkpointing only when the un-checkpointed layer stack does not fit."""
    return peak_memory_bytes(pd, po, g, m) / GB > capacity_gb * headroom
