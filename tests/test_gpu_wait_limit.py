"""Failure detection on the device, without a fault: a wait that nothing satisfies runs into its
limit, the kernel records the wait site and returns, the host reads LQ_ERR_TIMEOUT, and the
context keeps working.  This is the mechanism every producer/consumer wait of the GEMM kernels
uses (limit 2 s there, 20 ms here); it stands where the reference's "fail loudly, never fall back"
policy (crates/loractl-core/src/config.rs:503-512) meets device code."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_sets_the_status_and_leaves_the_context_usable():
    import loractl_b200 as lb
    from loractl_b200 import _lib as L
    from loractl_b200 import quant as Q

    lib = L.lib()
    dev = torch.device("cuda", 0)
    lb.check_device_status(dev)  # clean to start with
    stream = Q._stream_ptr(dev)
    t0 = time.time()
    L.check(lib.lq_selftest_bounded_wait(20, stream))
    with pytest.raises(L.LqError) as err:
        lb.check_device_status(dev)
    elapsed = time.time() - t0
    assert err.value.status == L.LQ_ERR_TIMEOUT and "wait site 90" in err.value.message
    assert 0.015 <= elapsed < 1.5  # it did wait for its limit, and not for much longer
    lb.check_device_status(dev)  # the word was cleared by the failing check
    # the context is intact: a real contraction runs and is correct afterwards
    w = torch.randn((256, 128), device=dev) * 0.02
    wq = lb.quantize_linear_weight(w, 4, 64)
    x = torch.randn((64, 128), device=dev)
    y = lb.quant_matmul_t(x, wq)
    ref = x @ wq.dequantize(torch.float32).t()
    assert torch.allclose(y, ref, atol=1e-4, rtol=1e-4)
    lb.check_device_status(dev)


def test_selftest_limit_is_validated():
    from loractl_b200 import _lib as L

    assert L.lib().lq_selftest_bounded_wait(0, None) == L.LQ_ERR_INVALID
    assert L.lib().lq_selftest_bounded_wait(5000, None) == L.LQ_ERR_INVALID
