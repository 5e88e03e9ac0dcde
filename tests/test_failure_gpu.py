"""A device-side wait that runs out: the kernel gives up after its (short) limit, reports through the
status word and returns; the context stays usable. Nothing here faults, traps or hangs the GPU: the
wait is on a flag that no one sets, and it is bounded."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_flag_wait_runs_out_and_reports_status():
    from keys_values_b200.ops import cuda as cu

    dev = torch.device("cuda", 0)
    lib = cu.lib()
    n = 1 << 16
    buf = torch.ones(n, dtype=torch.bfloat16, device=dev)
    flags_mine = torch.zeros(64, dtype=torch.int32, device=dev)
    flags_peer = torch.zeros(64, dtype=torch.int32, device=dev)  # a "peer" that never signals this rank
    sync = torch.zeros(2, dtype=torch.int32, device=dev)
    st = cu.status_word(dev)
    st.zero_()
    bases = (ctypes.c_void_p * 2)(buf.data_ptr(), buf.data_ptr())
    flags = (ctypes.c_void_p * 2)(flags_mine.data_ptr(), flags_peer.data_ptr())
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    rc = lib.kvb_allreduce_mean(bases, flags, 0, 2, ctypes.c_longlong(0), ctypes.c_longlong(n), ctypes.c_float(0.5),
                                ctypes.c_uint(1), ctypes.c_void_p(sync.data_ptr()), 1, 4, ctypes.c_void_p(st.data_ptr()),
                                ctypes.c_double(0.25), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    assert rc == 0
    torch.cuda.synchronize(dev)
    elapsed = time.perf_counter() - t0
    assert elapsed < 5.0, f"the bounded wait took {elapsed:.1f} s"
    assert int(st.item()) == 5  # STATUS_TIMEOUT_PEER_FLAG
    with pytest.raises(cu.NativeError, match="peer"):
        cu.check_status(dev)
    assert int(st.item()) == 0  # cleared by the check
    # the data was not touched and the context is usable
    assert torch.all(buf == 1)
    x = torch.randn(64, 1024, device=dev, dtype=torch.bfloat16)
    y, _ = cu.rmsnorm_fwd(x, None, 1e-6, False)
    torch.cuda.synchronize(dev)
    assert torch.isfinite(y.float()).all()
    cu.check_status(dev)
