"""The allocation-free split-K contraction, `lq_gemm_bf16_splitk_static`.

Some callers cannot allocate device memory at the point where they need a split contraction
(a stream under graph capture, an allocator callback, a loop whose memory was fixed at
start-up), so this entry point keeps its partial sums in a fixed 16 MiB array inside the
library instead of a caller workspace.  The test calls it through the C ABI and compares it
with the existing `lq_gemm_bf16` split path (caller-provided partials) on the same inputs:
same kernels, same summation order, so the results must agree to the bare-GEMM tolerance of
tests/test_gpu_tc.py (1e-5 of the output's peak).  It does so on two calls in a row with
different shapes and data, so stale contents of the shared array would show, checks an
MN-major case, and checks that a request beyond the array's size is refused by name.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It passes alone in a fresh process and after the rest of the suite.
"""
import numpy as np
import pytest
import torch

from tests.util import dev, host, reldev, seeded

pytestmark = pytest.mark.gpu


def _static(a, b, mn, splits):
    """a: [Mg, Kg], b: [Ng, Kg] logical bf16; mn stores both transposed ([Kg, rows])."""
    from loractl_b200 import _lib as L

    mg, kg = a.shape
    ng = b.shape[0]
    a_st = a.t().contiguous() if mn else a.contiguous()
    b_st = b.t().contiguous() if mn else b.contiguous()
    c = torch.full((mg, ng), float("nan"), dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    rc = L.lib().lq_gemm_bf16_splitk_static(a_st.data_ptr(), b_st.data_ptr(), int(mn), a_st.stride(0),
                                            b_st.stride(0), c.data_ptr(), ng, mg, ng, kg, splits, st)
    return rc, c


def _existing(a, b, mn, splits):
    from tests.test_gpu_tc import run_gemm

    return run_gemm(a, b, int(mn), int(mn), torch.float32, 64, splits)


def test_static_scratch_matches_workspace_path_on_two_calls_in_a_row():
    from loractl_b200 import _lib as L

    cases = [
        # Mg, Ng, Kg, mn, splits
        (1000, 64, 1024, False, 4),
        (520, 128, 640, False, 3),   # smaller, different data: stale partials must not leak in
        (384, 64, 1000, True, 5),
        (1000, 64, 1024, False, 4),  # the first problem again, after the array was reused
        (4100, 128, 512, False, 2),  # many row tiles, two column tiles: the tile raster of the first stage
        (300, 72, 448, False, 3),    # Ng not a multiple of 64: the partial rows are wider than C's
    ]
    first = None
    for i, (mg, ng, kg, mn, splits) in enumerate(cases):
        seed = 11 + (0 if i == 3 else i)
        a = dev(seeded((mg, kg), seed), torch.bfloat16)
        b = dev(seeded((ng, kg), seed + 100), torch.bfloat16)
        rc, got = _static(a, b, mn, splits)
        assert rc == L.LQ_OK, L.lib().lq_last_error()
        torch.cuda.synchronize()
        want = _existing(a, b, mn, splits)
        assert torch.isfinite(got).all()
        assert reldev(host(got), host(want)) <= 1e-5
        ref = a.float() @ b.float().t()
        assert reldev(host(got), host(ref)) <= 1e-5
        if i == 0:
            first = got.clone()
        if i == 3:
            assert torch.equal(got, first)  # deterministic: fixed split ranges, fixed reduction order


def test_static_scratch_call_allocates_no_device_memory():
    """After the one-time set-up call, a call must leave the device's free memory untouched."""
    from loractl_b200 import _lib as L

    a = dev(seeded((512, 768), 3), torch.bfloat16)
    b = dev(seeded((64, 768), 4), torch.bfloat16)
    rc, _ = _static(a, b, False, 4)  # set-up call (symbol address look-up, kernel attributes)
    assert rc == L.LQ_OK, L.lib().lq_last_error()
    torch.cuda.synchronize()
    c = torch.empty((512, 64), dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    free_before, _ = torch.cuda.mem_get_info()
    launches_before = L.lib().lq_kernel_launch_count()
    for _ in range(3):
        rc = L.lib().lq_gemm_bf16_splitk_static(a.data_ptr(), b.data_ptr(), 0, a.stride(0), b.stride(0),
                                                c.data_ptr(), 64, 512, 64, 768, 4, st)
        assert rc == L.LQ_OK, L.lib().lq_last_error()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the allocation-free entry changed the device's free memory"
    assert L.lib().lq_kernel_launch_count() - launches_before == 6  # two kernels per call, nothing else
    assert reldev(host(c), host(a.float() @ b.float().t())) <= 1e-5
    L.check(L.lib().lq_check_device_status(st))  # no bounded wait gave up


def test_static_scratch_rejects_short_row_strides():
    from loractl_b200 import _lib as L

    a = torch.zeros((256, 512), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((64, 512), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((256, 64), dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    rc = L.lib().lq_gemm_bf16_splitk_static(a.data_ptr(), b.data_ptr(), 0, 256, 512, c.data_ptr(), 64, 256, 64, 512,
                                            2, st)
    assert rc == L.LQ_ERR_INVALID  # lda < Kg


def test_static_scratch_limit_is_enforced_by_name():
    from loractl_b200 import _lib as L

    # 8 splits x 8192 rows x 64 padded columns = 4 Mi floats: exactly at the limit is accepted ...
    a = torch.zeros((8192, 512), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((64, 512), dtype=torch.bfloat16, device="cuda")
    rc, c = _static(a, b, False, 8)
    assert rc == L.LQ_OK, L.lib().lq_last_error()
    torch.cuda.synchronize()
    assert float(c.abs().max()) == 0.0
    # ... one more row block is refused, and nothing is launched
    a2 = torch.zeros((8192 + 128, 512), dtype=torch.bfloat16, device="cuda")
    rc, _ = _static(a2, b, False, 8)
    assert rc == L.LQ_ERR_WORKSPACE
    assert b"exceeds the built-in scratch" in L.lib().lq_last_error()
    rc, _ = _static(a, b, False, 9)  # more splits than k-blocks (512 / 64 = 8)
    assert rc == L.LQ_ERR_INVALID
