"""The launch plumbing of the hot calls: inside `lq_linear_fwd/bwd` independent steps are enqueued
on a second stream between an event fork and join.  These tests check what that must not break:
results under a stream capture (replayed) equal the eager ones bit for bit, and calls issued from
two caller streams at once — each with its own workspace and side stream — equal the serial ones."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def make_case(scheme, n, k, m, r, seed):
    import loractl_b200 as lb

    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn((m, k), generator=g, device="cuda") * 0.02
    wq = lb.quantize_linear_weight(w, 4, 64) if scheme == "int4" else lb.fp8_quantize(w, True)
    x = torch.randn((n, k), generator=g, device="cuda").to(torch.bfloat16)
    dy = torch.randn((n, m), generator=g, device="cuda").to(torch.bfloat16)
    a = torch.randn((k, r), generator=g, device="cuda") / k ** 0.5
    b = torch.randn((r, m), generator=g, device="cuda") * 0.01
    return wq, x, dy, a, b


def step(wq, x, dy, a, b, fp8=False):
    from loractl_b200 import quant as Q

    y, h = Q.linear_fwd_raw(wq, x, a, b, 1.5, fp8_compute=fp8)
    dx, da, db = Q.linear_bwd_raw(wq, dy, x, h, a, b, 1.5, fp8_compute=fp8)
    return y, dx, da, db


@pytest.mark.parametrize("scheme,n,fp8", [("int4", 512, False), ("fp8", 384, False), ("fp8", 384, True), ("int4", 8, False)])
def test_captured_step_replays_the_eager_result(scheme, n, fp8):
    import loractl_b200 as lb

    wq, x, dy, a, b = make_case(scheme, n, 512, 768, 16, 1)
    if fp8:
        wq.prepare_fp8_backward()
    eager = [t.clone() for t in step(wq, x, dy, a, b, fp8)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        step(wq, x, dy, a, b, fp8)  # sizes this stream's workspace and creates its fork-join objects
        with torch.cuda.graph(graph, stream=side):
            outs = step(wq, x, dy, a, b, fp8)
    torch.cuda.current_stream().wait_stream(side)
    for t in outs:
        t.fill_(float("nan"))
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    lb.check_device_status()
    for got, want in zip(outs, eager):
        assert torch.equal(got, want)


def test_two_caller_streams_at_once_equal_the_serial_results():
    import loractl_b200 as lb

    cases = [make_case("int4", 640, 512, 1024, 16, s) for s in (2, 3)]
    serial = [[t.clone() for t in step(*c)] for c in cases]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for st in streams:
        st.wait_stream(torch.cuda.current_stream())
    results = [None, None]
    for rep in range(3):  # interleave the enqueues of the two streams
        for i, st in enumerate(streams):
            with torch.cuda.stream(st):
                results[i] = step(*cases[i])
    for st in streams:
        torch.cuda.current_stream().wait_stream(st)
    torch.cuda.synchronize()
    lb.check_device_status()
    for got, want in zip(results, serial):
        for g, w in zip(got, want):
            assert torch.equal(g, w)
