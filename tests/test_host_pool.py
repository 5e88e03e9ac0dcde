"""Native host memory pool: allocator logic on any machine, pinned memory and copy / compute overlap on a GPU."""
import gc

import pytest
import torch

from keys_values_b200.utils.host_pool import HostPool


def test_pool_allocates_coalesces_and_falls_back():
    pool = HostPool(1 << 20, pinned=False)
    a, b, c = pool.empty((1000,), torch.float32), pool.empty((3, 5), torch.bfloat16), pool.empty((100_000,), torch.float32)
    a.fill_(3.0)
    b.fill_(1.5)
    c.zero_()
    assert float(a.sum()) == 3000.0 and float(b.float().sum()) == 22.5  # the ranges do not overlap
    s = pool.stats()
    assert s["in_use"] == 4096 + 256 + 400_128 and s["allocations"] == 3
    view = a[10:20]
    del a
    gc.collect()
    assert pool.stats()["in_use"] == s["in_use"]  # a view keeps the range
    assert float(view.sum()) == 30.0
    del view
    gc.collect()
    assert pool.stats()["in_use"] == s["in_use"] - 4096
    big = pool.empty((10_000_000,), torch.float32)  # does not fit: ordinary tensor
    assert big.numel() == 10_000_000 and pool.stats()["fallbacks"] == 1
    hole = pool.empty((512,), torch.float32)  # first fit: reuses the hole in front
    assert pool.stats()["in_use"] == s["in_use"] - 4096 + 2048
    del b, c, hole
    gc.collect()
    s = pool.stats()
    assert s["in_use"] == 0 and s["largest_free"] == s["capacity"]  # all ranges merged back into one
    pool.close()


@pytest.mark.gpu
def test_pool_memory_is_pinned_and_copies_overlap_with_compute():
    dev = torch.device("cuda", 0)
    pool = HostPool(1 << 30, pinned=True)
    n = 64 * 2**20  # 256 MB of fp32
    host = pool.empty((n,), torch.float32)
    assert host.is_pinned()
    src = torch.randn(n, device=dev)
    side = torch.cuda.Stream(device=dev)
    a = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)

    def compute():
        x = a
        for _ in range(12):
            x = x @ a * 0.01
        return x

    def copy():
        with torch.cuda.stream(side):
            host.copy_(src, non_blocking=True)

    def timed(fn):
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        side.synchronize()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1)

    for _ in range(2):
        compute(), copy()
    t_compute, t_copy = min(timed(compute) for _ in range(3)), min(timed(copy) for _ in range(3))
    t_both = min(timed(lambda: (copy(), compute())) for _ in range(3))
    torch.testing.assert_close(host[:1000], src[:1000].cpu())
    back = torch.empty_like(src)
    back.copy_(host, non_blocking=True)
    torch.cuda.synchronize(dev)
    assert torch.equal(back, src)
    # the copy hides behind the GEMMs: both together take clearly less than one after the other
    hidden = (t_compute + t_copy - t_both) / min(t_compute, t_copy)
    print(f"compute {t_compute:.2f} ms, copy {t_copy:.2f} ms ({n * 4 / t_copy / 1e6:.1f} GB/s), together {t_both:.2f} ms, hidden fraction {hidden:.2f}")
    assert hidden > 0.5
    pool.close()
