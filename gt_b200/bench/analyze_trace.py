"""Analyse the chrome trace of one training epoch (``train_dist --profile`` with ``GT_PROF_TRACE=<prefix>``): GPU busy time
against the wall time of the epoch, the idle gaps between kernels, device time per category of the performance model,
and every collective kernel (NCCL or the package's peer-memory kernels) with its duration, waiting included.  Counterpart
of the reference's ``gt3d/bench/analyze_trace.py``; reads files only.

    python -m gt_b200.bench.analyze_trace trace_rank0.json [trace_rank1.json ...]
"""
import json
import sys

GPU_CATS = ("kernel", "gpu_memcpy", "gpu_memset")


def busy_union(events):
    """Total length of the union of ``(ts, dur)`` intervals (kernels on several streams may overlap)."""
    tot, end = 0.0, None
    for e in sorted(events, key=lambda e: e["ts"]):
        a, b = e["ts"], e["ts"] + e["dur"]
        if end is None or a > end:
            tot += b - a
            end = b
        elif b > end:
            tot += b - end
            end = b
    return tot


def analyze(path, top_gaps=5):
    from ..utils.profiling import categorise
    with open(path) as f:
        ev = json.load(f)["traceEvents"]
    gpu = sorted((e for e in ev if e.get("ph") == "X" and e.get("cat") in GPU_CATS), key=lambda e: e["ts"])
    if not gpu:
        return dict(path=path, kernels=0)
    t0, t1 = gpu[0]["ts"], max(e["ts"] + e["dur"] for e in gpu)
    busy = busy_union(gpu)
    gaps, end = [], gpu[0]["ts"] + gpu[0]["dur"]
    for prev, e in zip(gpu, gpu[1:]):
        if e["ts"] > end:
            gaps.append((e["ts"] - end, prev["name"][:60], e["name"][:60]))
        end = max(end, e["ts"] + e["dur"])
    per_cat = {}
    for e in gpu:
        c = categorise(e["name"]) if e["cat"] == "kernel" else e["cat"]
        per_cat[c] = per_cat.get(c, 0.0) + e["dur"]
    coll = [dict(name=e["name"][:70], start_ms=(e["ts"] - t0) / 1e3, ms=e["dur"] / 1e3) for e in gpu
            if e["cat"] == "kernel" and categorise(e["name"]) == "collective"]
    return dict(path=path, kernels=len(gpu), wall_ms=(t1 - t0) / 1e3, busy_ms=busy / 1e3, idle_ms=(t1 - t0 - busy) / 1e3,
                gaps=len(gaps), largest_gaps=[dict(ms=g / 1e3, after=a, before=b) for g, a, b in sorted(gaps, reverse=True)[:top_gaps]],
                per_category_ms={k: v / 1e3 for k, v in sorted(per_cat.items(), key=lambda kv: -kv[1])},
                collective_ms=sum(c["ms"] for c in coll), collectives=coll)


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 2 if not argv else 0
    out = []
    for path in argv:
        r = analyze(path)
        out.append(r)
        if not r["kernels"]:
            print(f"{path}: no GPU events")
            continue
        print(f"{path}: {r['kernels']} GPU events, wall {r['wall_ms']:.2f} ms, busy {r['busy_ms']:.2f} ms "
              f"({100 * r['busy_ms'] / r['wall_ms']:.1f} %), idle {r['idle_ms']:.2f} ms in {r['gaps']} gaps")
        for cat, ms in r["per_category_ms"].items():
            print(f"    {cat:18s} {ms:9.3f} ms")
        for g in r["largest_gaps"]:
            print(f"    gap {g['ms']:.3f} ms between {g['after']} | {g['before']}")
        print(f"    collectives: {len(r['collectives'])} kernels, {r['collective_ms']:.3f} ms")
        for c in r["collectives"]:
            print(f"      +{c['start_ms']:9.3f} ms  {c['ms']:8.3f} ms  {c['name']}")
    return out


if __name__ == "__main__":
    main()
