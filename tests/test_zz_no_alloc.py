"""`f8b200_gemm_fp8_static_scratch`: the GEMM entry point whose scheduling words live in the
library's static device array.  It must return the same bits as the workspace entry point,
call after call, allocate nothing, and refuse a 17th stream."""
import pytest
import torch

from float8_experimental_b200 import _native as N

pytestmark = pytest.mark.gpu


def _operands(m, n, k, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(n, k, device="cuda", generator=g).to(torch.float8_e5m2)
    sa, sb = torch.tensor(4.0, device="cuda"), torch.tensor(0.125, device="cuda")
    return a, b, sa, sb


def _run(fn, a, b, sa, sb, out):
    m, k = a.shape
    n = b.shape[0]
    out.fill_(float("nan"))
    fn(a, k, b, k, sa, sb, None, out, n, m, n, k, False)
    return out


@pytest.mark.parametrize("mnk", [(4096, 8192, 512), (8192, 4096, 16384), (300, 520, 64)])
def test_static_scratch_matches_workspace_entry_twice_in_a_row(mnk):
    m, n, k = mnk
    a, b, sa, sb = _operands(m, n, k, seed=m + k)
    want = _run(N.gemm_fp8, a, b, sa, sb, torch.empty(m, n, dtype=torch.bfloat16, device="cuda")).clone()
    got = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    first, second = torch.empty_like(got), torch.empty_like(got)
    _run(N.gemm_fp8_static_scratch, a, b, sa, sb, got)   # also the per-device set-up call
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    torch_before = torch.cuda.memory_allocated()
    _run(N.gemm_fp8_static_scratch, a, b, sa, sb, first)
    _run(N.gemm_fp8_static_scratch, a, b, sa, sb, second)  # straight after, same stream, same slot
    torch.cuda.synchronize()
    # neither call allocated device memory, through torch or behind its back
    assert torch.cuda.memory_allocated() == torch_before
    assert torch.cuda.mem_get_info()[0] == free_before
    assert N.read_device_error() == 0
    assert torch.equal(first.view(torch.int16), want.view(torch.int16))
    assert torch.equal(second.view(torch.int16), want.view(torch.int16))


def test_refused_and_empty_calls_take_no_slot():
    """A call that fails its argument checks, or has nothing to compute, neither looks the array up
    nor claims one of the 16 per-stream slots: twenty such calls on twenty fresh streams leave room
    for the streams of the next test."""
    a, b, sa, sb = _operands(256, 256, 128, seed=9)
    out = torch.empty(256, 256, dtype=torch.bfloat16, device="cuda")
    for _ in range(20):
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            with pytest.raises(N.F8B200Error, match="bad argument"):
                N.gemm_fp8_static_scratch(a, 64, b, 128, sa, sb, None, out, 256, 256, 256, 128, False)  # lda < k
            N.gemm_fp8_static_scratch(a, 128, b, 128, sa, sb, None, out, 256, 0, 256, 128, False)      # m == 0
    torch.cuda.synchronize()
    assert N.read_device_error() == 0


def test_static_scratch_refuses_more_streams_than_slots():
    a, b, sa, sb = _operands(512, 512, 128, seed=3)
    out = torch.empty(512, 512, dtype=torch.bfloat16, device="cuda")
    want = _run(N.gemm_fp8, a, b, sa, sb, torch.empty_like(out)).clone()
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream() for _ in range(20)]
    accepted = refused = 0
    for s in streams:
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            try:
                _run(N.gemm_fp8_static_scratch, a, b, sa, sb, out)
            except N.F8B200Error as err:
                assert "not supported" in str(err)
                refused += 1
                continue
            s.synchronize()
            assert torch.equal(out.view(torch.int16), want.view(torch.int16))
            accepted += 1
    # 16 slots per device; earlier tests of this file may hold one or two of them
    assert 13 <= accepted <= 16 and refused == len(streams) - accepted
    # a stream that already has a slot keeps working after the table is full
    _run(N.gemm_fp8_static_scratch, a, b, sa, sb, out)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    assert N.read_device_error() == 0
