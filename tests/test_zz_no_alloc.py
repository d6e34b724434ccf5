"""`mdy_rmsnorm_bwd_noalloc`: the RMSNorm backward for callers that cannot allocate device memory.

Some hosts of this library cannot call cudaMalloc when the backward runs — a runtime that owns all
device memory and hands out fixed buffers, or code running where the allocator must stay untouched.
For them the float32 partial rows of `dw` live in a fixed array inside the library instead of a
caller-provided buffer.  The test calls the entry point directly through the C ABI, twice in a row with
different inputs (the array keeps the previous call's contents), and requires the same `dx` / `dw` as
`mdy_rmsnorm_bwd` with caller-provided scratch and as the float32 CPU oracle, and that neither the
driver's free-memory figure nor torch's allocator moves across a call.  This file is collected last on
purpose.
"""
import pytest
import torch

from conftest import REL, assert_close
from mdy_triton_b200 import _C
from oracle import eager as E

pytestmark = pytest.mark.gpu


def _inputs(m, n, dt, seed, dev):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, n, generator=g).to(dt).to(dev)
    w = (1 + 0.1 * torch.randn(n, generator=g)).to(dt).to(dev)
    dy = torch.randn(m, n, generator=g).to(dt).to(dev)
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous()
    return x, w, dy, rstd


def _run(noalloc, x, w, dy, rstd):
    lib = _C.lib()
    m, n = x.shape
    code = _C.dtype_code(x)
    st = torch.cuda.current_stream().cuda_stream
    dx = torch.full_like(x, float("nan"))
    dw = torch.full_like(w, float("nan"))
    if noalloc:
        rc = lib.mdy_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                         dw.data_ptr(), m, n, n, n, n, code, code, st)
    else:
        rows = lib.mdy_rmsnorm_bwd_partial_rows(m, n, code)
        partial = torch.empty(rows, n, dtype=torch.float32, device=x.device)
        rc = lib.mdy_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                                 partial.data_ptr(), m, n, n, n, n, code, code, st)
    _C.check(rc, "rmsnorm backward")
    torch.cuda.synchronize()
    return dx, dw


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_noalloc_matches_allocating_entry_point_twice_in_a_row(dt):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    # two different problems back to back: the second must not see the first one's partial rows
    for seed, (m, n) in enumerate([(4096, 2048), (777, 896)]):
        x, w, dy, rstd = _inputs(m, n, dt, 100 + seed, dev)
        dx_ref, dw_ref = _run(False, x, w, dy, rstd)
        dx, dw = _run(True, x, w, dy, rstd)
        assert torch.isfinite(dx).all() and torch.isfinite(dw).all()
        assert_close(dx, dx_ref, REL[dt], "dx")
        assert_close(dw, dw_ref, REL[dt], "dw")
        # same kernels, same grid: the results are in fact identical
        assert torch.equal(dx, dx_ref) and torch.equal(dw, dw_ref)
        # and both agree with the float32 restatement of the reference's backward
        dx_o, dw_o = E.rmsnorm_bwd(dy.cpu(), x.cpu(), w.cpu(), 1e-6)
        assert_close(dx, dx_o, REL[dt], "dx vs oracle")
        assert_close(dw, dw_o, REL[dt], "dw vs oracle")


def test_noalloc_call_leaves_device_memory_untouched():
    """The claim in the entry point's name: across a call (after the first one on the device, which may make
    the driver load the library's device image) the free device memory the driver reports and the bytes
    torch's allocator holds are unchanged."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _C.lib()
    x, w, dy, rstd = _inputs(2048, 4096, torch.bfloat16, 5, dev)
    dx = torch.empty_like(x); dw = torch.empty_like(w)
    code = _C.dtype_code(x)
    st = torch.cuda.current_stream().cuda_stream

    def call():
        return lib.mdy_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                           dw.data_ptr(), 2048, 4096, 4096, 4096, 4096, code, code, st)
    assert call() == 0
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(dev)
    alloc0, reserved0 = torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(dev)
    assert (torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)) == (alloc0, reserved0)
    assert free1 == free0, f"free device memory moved by {free0 - free1} bytes across the calls"


def test_noalloc_odd_shape_takes_the_scalar_path():
    dev = torch.device("cuda", 0)
    x, w, dy, rstd = _inputs(33, 1001, torch.bfloat16, 7, dev)
    dx_ref, dw_ref = _run(False, x, w, dy, rstd)
    dx, dw = _run(True, x, w, dy, rstd)
    assert_close(dx, dx_ref, 1e-2, "dx"); assert_close(dw, dw_ref, 1e-2, "dw")


def test_noalloc_rejects_sizes_beyond_its_scratch():
    """One row of 4 Mi + 8 columns needs one partial row longer than the fixed array.  The buffers passed are
    genuinely that large, so even a library that failed to refuse would stay inside them."""
    lib = _C.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    m, n = 1, (4 << 20) + 8
    assert lib.mdy_rmsnorm_bwd_partial_rows(m, n, _C.MDY_BF16) * n > 4 << 20
    x = torch.zeros(m, n, dtype=torch.bfloat16, device=dev); dy = torch.zeros_like(x); dx = torch.zeros_like(x)
    w = torch.ones(n, dtype=torch.bfloat16, device=dev); dw = torch.zeros_like(w)
    rstd = torch.ones(m, dtype=torch.float32, device=dev)
    before = _C.launch_count()
    rc = lib.mdy_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                     dw.data_ptr(), m, n, n, n, n, _C.MDY_BF16, _C.MDY_BF16, None)
    assert rc == -4 and "limit" in _C.status_string(rc)
    assert _C.launch_count() == before   # nothing was launched
