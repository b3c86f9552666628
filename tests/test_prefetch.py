"""Input pipeline (pinned host -> staging -> static device tensors) and pipelined scalar reads."""
import pytest
import torch

from gt_b200.train.prefetch import AsyncScalar, InputPrefetcher


def test_prefetcher_and_scalar_ring_on_cpu():
    pre = InputPrefetcher({"x": torch.arange(6.).view(2, 3), "y": torch.tensor([1, 2])}, "cpu")
    out = pre.next()
    assert torch.equal(out["x"], torch.arange(6.).view(2, 3)) and torch.equal(out["y"], torch.tensor([1, 2]))
    pre.next(following={"x": torch.ones(2, 3)})
    assert torch.equal(pre.next()["x"], torch.ones(2, 3)) and pre.static["x"] is out["x"]        # same static tensor, refreshed
    assert pre.bytes_per_step == 6 * 4 + 2 * 8
    ring = AsyncScalar("cpu", slots=2)
    ring.push(torch.tensor(1.5))
    assert ring.pop_previous() is None
    ring.push(torch.tensor(2.5))
    assert ring.pop_previous() == 1.5
    ring.push(torch.tensor(3.5))
    with pytest.raises(RuntimeError):
        ring.push(torch.tensor(4.5))
    assert ring.drain() == [2.5, 3.5]


@pytest.mark.gpu
@pytest.mark.xfail(reason="not yet run on a GPU", strict=False)          # a first-run failure is reported without ending a stop-at-first-failure run
def test_prefetcher_delivers_every_batch_under_overlap():
    dev = torch.device("cuda:0")
    batches = [torch.full((1 << 20,), float(i)).pin_memory() for i in range(6)]
    pre = InputPrefetcher({"x": batches[0]}, dev)
    ring = AsyncScalar(dev)
    got = []
    for i in range(6):
        x = pre.next(following={"x": batches[min(i + 1, 5)]})["x"]     # batch i is in the static tensor; batch i + 1 is being copied
        s = x.sum() / x.numel()
        for _ in range(20):                                 # keep the compute stream busy while the copy stream works
            s = s + (x * 0).sum()
        ring.push(s)
        v = ring.pop_previous()
        if v is not None:
            got.append(v)
    got += ring.drain()
    assert got == [float(i) for i in range(6)]
    with pytest.raises(ValueError):
        InputPrefetcher({"x": torch.zeros(4)}, dev)         # pageable host memory is refused
