"""GPU parity tests: the CUDA kernels, reached through the operator API (which calls the C-ABI), against
(1) the golden vectors the reference's own kernels produced and (2) the float32 CPU oracle, on seeded
inputs.  Tolerances: conftest.REL (1e-2 relative for 16-bit I/O, 1e-4 for float32 I/O) and 1e-4 on the
float32 loss."""
import pytest
import torch

from conftest import LOSS_TOL, REL, assert_close, golden_cases
from oracle import eager as E
import mdy_triton.core as core
from mdy_triton.core.cross_entyopy_loss import _FastCrossEntropyLoss, triton_entropy_loss
from mdy_triton_b200 import _C

pytestmark = pytest.mark.gpu
DEV = "cuda"


def g(seed):
    return torch.Generator().manual_seed(seed)


def leaf(t):
    return t.detach().to(DEV).clone().requires_grad_(True)


def loss_close(a, b):
    a, b = float(a), float(b)
    assert abs(a - b) <= LOSS_TOL * max(1.0, abs(b)), (a, b)


# ---------------------------------------------------------------------------------------------- RMSNorm
def run_rmsnorm(x, w, eps, dy):
    xg, wg = leaf(x), leaf(w)
    y = core.triton_rmsnorm(xg, wg, eps)
    y.backward(dy.to(DEV))
    return y, xg.grad, wg.grad


@pytest.mark.parametrize("c", golden_cases("rmsnorm.pt"))
def test_rmsnorm_golden(c):
    y, dx, dw = run_rmsnorm(c["x"], c["w"], c["eps"], c["dy"])
    r = REL[c["x"].dtype]
    assert y.dtype == c["x"].dtype and dw.dtype == c["w"].dtype
    assert_close(y, c["y"], r, "y"); assert_close(dx, c["dx"], r, "dx"); assert_close(dw, c["dw"], r, "dw")


@pytest.mark.parametrize("m,n,dt", [(4096, 896, torch.bfloat16), (4096, 896, torch.float32), (2048, 3584, torch.bfloat16),
                                    (1024, 2048, torch.float16), (1, 4096, torch.bfloat16), (3, 8, torch.float32),
                                    (7, 7, torch.bfloat16), (9, 127, torch.float16),
                                    (9, 129, torch.bfloat16), (64, 3585, torch.bfloat16), (300, 8192, torch.bfloat16),
                                    (40, 16384, torch.bfloat16), (12, 32768, torch.bfloat16), (6, 65536, torch.bfloat16),
                                    (4, 70000, torch.float32), (33, 5120, torch.float32)])
def test_rmsnorm_vs_oracle(m, n, dt):
    gen = g(m * 131 + n)
    x = torch.randn(m, n, generator=gen).to(dt); w = (1 + 0.02 * torch.randn(n, generator=gen)).to(dt)
    dy = torch.randn(m, n, generator=gen).to(dt)
    y, dx, dw = run_rmsnorm(x, w, 1e-6, dy)
    yo, _ = E.rmsnorm_fwd(x, w, 1e-6)
    dxo, dwo = E.rmsnorm_bwd(dy, x, w, 1e-6)
    r = REL[dt]
    assert_close(y, yo, r, "y"); assert_close(dx, dxo, r, "dx")
    assert_close(dw, dwo, max(r, 2e-3) if dt == torch.float32 else r, "dw")


def test_rmsnorm_single_column():
    """N == 1: y = sign(x) * w up to eps; dx cancels to ~0 (it is rounding noise relative to w*dy/rms)."""
    x = torch.tensor([[0.5], [-2.0], [3.0], [1e-2], [-7.0]]); w = torch.tensor([1.5]); dy = torch.randn(5, 1, generator=g(1))
    y, dx, dw = run_rmsnorm(x, w, 1e-6, dy)
    yo, rms = E.rmsnorm_fwd(x, w, 1e-6)
    dxo, dwo = E.rmsnorm_bwd(dy, x, w, 1e-6)
    assert_close(y, yo, 1e-4, "y"); assert_close(dw, dwo, 1e-4, "dw")
    bound = 1e-5 * (w * dy).abs() / rms[:, None]
    assert ((dx.cpu() - dxo).abs() <= bound).all()


def test_rmsnorm_3d_input_strided_rows_and_fp32_weight():
    gen = g(5)
    big = torch.randn(2, 6, 512 + 64, generator=gen).to(torch.bfloat16).to(DEV)
    x = big[..., :512]  # row stride 576: not contiguous, still 16-byte aligned rows
    w = (1 + 0.1 * torch.randn(512, generator=gen)).to(DEV)  # float32 master weight
    xg = x.detach().clone().requires_grad_(True)
    xs = big.detach().clone()[..., :512].requires_grad_(True)
    wg1, wg2 = leaf(w), leaf(w)
    dy = torch.randn(2, 6, 512, generator=gen).to(torch.bfloat16).to(DEV)
    y1 = core.triton_rmsnorm(xg, wg1, 1e-5); y1.backward(dy)
    y2 = core.triton_rmsnorm(xs, wg2, 1e-5); y2.backward(dy)
    assert y1.shape == (2, 6, 512) and wg1.grad.dtype == torch.float32
    assert torch.equal(y1, y2) and torch.equal(wg1.grad, wg2.grad)
    yo, _ = E.rmsnorm_fwd(x.cpu(), w.cpu(), 1e-5)
    dxo, dwo = E.rmsnorm_bwd(dy.cpu(), x.cpu(), w.cpu(), 1e-5)
    assert_close(y1, yo, 1e-2); assert_close(xg.grad, dxo, 1e-2); assert_close(wg1.grad, dwo, 1e-2)


def test_rmsnorm_unaligned_base_takes_scalar_path():
    gen = g(6)
    flat = torch.randn(16 * 64 + 1, generator=gen).to(torch.bfloat16).to(DEV)
    x = flat[1:].view(16, 64)  # base pointer off by 2 bytes
    w = torch.ones(64, dtype=torch.bfloat16, device=DEV)
    y = core.triton_rmsnorm(x, w, 1e-6)
    assert_close(y, E.rmsnorm_fwd(x.cpu(), w.cpu(), 1e-6)[0], 1e-2)


def test_rmsnorm_scale_invariance_full_size():
    """Size-independent property at the Qwen2-7B shape: rmsnorm(4x) == rmsnorm(x) up to eps."""
    x = torch.randn(32768, 3584, device=DEV, dtype=torch.bfloat16, generator=torch.Generator(DEV).manual_seed(2))
    w = torch.ones(3584, device=DEV, dtype=torch.bfloat16)
    y1 = core.triton_rmsnorm(x, w, 1e-6)
    y4 = core.triton_rmsnorm(x * 4, w, 1e-6)
    assert (y1.float() - y4.float()).abs().max() <= 0.04
    ms = y1.float().pow(2).mean(-1)
    assert (ms - 1).abs().max() < 2e-2


# ------------------------------------------------------------------------------------------ add+RMSNorm
def run_add_rmsnorm(x, res, w, eps, dy, dn):
    xg, rg, wg = leaf(x), leaf(res), leaf(w)
    y, nr = core.triton_fused_add_norm(xg, rg, wg, eps)
    torch.autograd.backward([y, nr], [dy.to(DEV), dn.to(DEV)])
    return y, nr, xg.grad, rg.grad, wg.grad


@pytest.mark.parametrize("c", golden_cases("add_rmsnorm.pt"))
def test_add_rmsnorm_golden(c):
    y, nr, dx, dr, dw = run_add_rmsnorm(c["x"], c["res"], c["w"], c["eps"], c["dy"], c["dnew_res"])
    r = REL[c["x"].dtype]
    assert_close(y, c["y"], r, "y"); assert_close(nr, c["new_res"], r, "new_res")
    if c["grads"]:
        assert_close(dx, c["dx"], r, "dx"); assert_close(dr, c["dres"], r, "dres")
        dw_ref = c["dw"].float().sum(0) if c["dw"].dim() == 2 else c["dw"]
        assert_close(dw, dw_ref, r, "dw")


@pytest.mark.parametrize("m,n,dt,eps", [(2048, 4096, torch.bfloat16, 1e-5), (4096, 896, torch.float32, 1e-6),
                                        (512, 2048, torch.float16, 1e-5), (1, 256, torch.bfloat16, 1e-5),
                                        (17, 129, torch.float32, 1e-6), (5, 3585, torch.bfloat16, 1e-6),
                                        (64, 8192, torch.bfloat16, 1e-5), (8, 20480, torch.bfloat16, 1e-5)])
def test_add_rmsnorm_vs_oracle(m, n, dt, eps):
    """Includes hidden sizes > 128, where the reference backward is wrong: checked against the oracle
    (closed form == autograd of `residual + x` followed by RMSNorm)."""
    gen = g(m * 7 + n)
    x = torch.randn(m, n, generator=gen).to(dt); res = torch.randn(m, n, generator=gen).to(dt)
    w = (1 + 0.02 * torch.randn(n, generator=gen)).to(dt)
    dy = torch.randn(m, n, generator=gen).to(dt); dn = torch.randn(m, n, generator=gen).to(dt)
    y, nr, dx, dr, dw = run_add_rmsnorm(x, res, w, eps, dy, dn)
    yo, so, _ = E.add_rmsnorm_fwd(x, res, w, eps)
    r = REL[dt]
    assert_close(y, yo, r, "y"); assert_close(nr, so, r, "new_res")
    # backward consumes the ROUNDED new residual the forward stored
    dxo, dwo = E.add_rmsnorm_bwd(dy, dn, nr.cpu(), w, eps)
    assert_close(dx, dxo, r, "dx"); assert torch.equal(dx, dr)
    assert_close(dw, dwo, max(r, 2e-3), "dw")


def test_add_rmsnorm_unused_outputs():
    x = torch.randn(8, 256, device=DEV, dtype=torch.bfloat16)
    w = torch.ones(256, device=DEV, dtype=torch.bfloat16)
    xg, rg, wg = leaf(x), leaf(x), leaf(w)
    y, nr = core.triton_fused_add_norm(xg, rg, wg, 1e-5)
    y.float().sum().backward()           # new_residual unused -> its gradient is None
    dxo, _ = E.add_rmsnorm_bwd(torch.ones(8, 256), None, nr.cpu(), w.cpu(), 1e-5)
    assert_close(xg.grad, dxo, 1e-2)
    xg, rg, wg = leaf(x), leaf(x), leaf(w)
    y, nr = core.triton_fused_add_norm(xg, rg, wg, 1e-5)
    nr.float().sum().backward()          # y unused
    assert torch.equal(xg.grad, torch.ones_like(xg)) and torch.equal(wg.grad, torch.zeros_like(wg))


# ------------------------------------------------------------------------------------------------- RoPE
def run_rope(c_q, c_k, cos, sin, dq, dk, strided_grad=False):
    # storage layout [B, L, H, D], logical [B, H, L, D] — what q_proj(...).view().transpose(1, 2) yields
    qs = leaf(c_q.transpose(1, 2).contiguous()); ks = leaf(c_k.transpose(1, 2).contiguous())
    q_in = (qs * 1.0).transpose(1, 2); k_in = (ks * 1.0).transpose(1, 2)
    qe, ke = core.fused_apply_rope(q_in, k_in, cos.to(DEV), sin.to(DEV))
    assert qe.data_ptr() == q_in.data_ptr() and ke.data_ptr() == k_in.data_ptr()  # in place
    dq, dk = dq.to(DEV), dk.to(DEV)
    if strided_grad:  # gradient arriving in [B, H, L, D] storage, like an attention backward's
        dq, dk = dq.contiguous(), dk.contiguous()
    qv, kv = qe.detach().clone(), ke.detach().clone()
    torch.autograd.backward([qe, ke], [dq, dk])
    return qv, kv, qs.grad.transpose(1, 2), ks.grad.transpose(1, 2)


@pytest.mark.parametrize("c", golden_cases("rope.pt"))
def test_rope_golden(c):
    qe, ke, gq, gk = run_rope(c["q"], c["k"], c["cos"], c["sin"], c["dq"], c["dk"], strided_grad=True)
    r = REL[c["q"].dtype]
    assert_close(qe, c["q_out"], r, "q"); assert_close(ke, c["k_out"], r, "k")
    assert_close(gq, c["dq_in"], r, "dq"); assert_close(gk, c["dk_in"], r, "dk")


@pytest.mark.parametrize("b,l,qh,kh,d,theta,dt,batch_cs", [
    (4, 1024, 14, 2, 64, 1e6, torch.bfloat16, False),   # Qwen2-0.5B shape
    (4, 1024, 14, 2, 64, 1e6, torch.float32, False),
    (2, 512, 32, 8, 128, 5e5, torch.bfloat16, False),   # Llama-3-8B heads
    (2, 256, 28, 4, 128, 1e6, torch.bfloat16, True),    # Qwen2-7B heads, per-batch positions
    (2, 64, 32, 8, 64, 5e5, torch.float16, False),      # Llama-1B heads
    (1, 3, 1, 1, 2, 1e4, torch.float32, False),         # smallest legal head
    (2, 5, 3, 1, 6, 1e4, torch.bfloat16, False),        # scalar path: D/2 not a multiple of the vector
    (2, 17, 5, 5, 192, 1e4, torch.float32, True),
    (1, 9, 7, 0, 32, 1e4, torch.bfloat16, False),       # no k heads at all
])
def test_rope_vs_oracle(b, l, qh, kh, d, theta, dt, batch_cs):
    gen = g(b * 1000 + l + d)
    q = torch.randn(b, qh, l, d, generator=gen).to(dt); k = torch.randn(b, kh, l, d, generator=gen).to(dt)
    pos = (torch.arange(l)[None] + (torch.arange(b)[:, None] * 3 if batch_cs else 0))
    cos, sin = E.rope_cos_sin(pos, d, theta, dt)
    dq = torch.randn(b, qh, l, d, generator=gen).to(dt); dk = torch.randn(b, kh, l, d, generator=gen).to(dt)
    qe, ke, gq, gk = run_rope(q, k, cos, sin, dq, dk)
    qo, ko = E.rope_fwd(q, k, cos, sin); gqo, gko = E.rope_bwd(dq, dk, cos, sin)
    r = REL[dt]
    assert_close(qe, qo, r, "q"); assert_close(gq, gqo, r, "dq")
    if kh:
        assert_close(ke, ko, r, "k"); assert_close(gk, gko, r, "dk")
    hq, hk = E.hf_rope(q, k, cos, sin)
    assert_close(qe, hq, r, "q vs HF eager")


@pytest.mark.parametrize("d,rd", [(128, 96), (64, 32), (96, 48), (80, 20)])
def test_rope_partial_rotary_dim(d, rd):
    """cos/sin narrower than the head (HuggingFace Phi3 / GLM partial_rotary_factor): the first rotary_dim
    columns of every head are rotated, the others pass through, forward and backward."""
    gen = g(d * 7 + rd)
    b, l, qh, kh = 2, 33, 6, 2
    q = torch.randn(b, l, qh, d, generator=gen).to(torch.bfloat16); k = torch.randn(b, l, kh, d, generator=gen).to(torch.bfloat16)
    dq = torch.randn(b, qh, l, d, generator=gen).to(torch.bfloat16); dk = torch.randn(b, kh, l, d, generator=gen).to(torch.bfloat16)
    cos, sin = E.rope_cos_sin(torch.arange(l)[None], rd, 1e4, torch.bfloat16)
    qs, ks = leaf(q), leaf(k)
    qe, ke = core.fused_apply_rope((qs * 1.0).transpose(1, 2), (ks * 1.0).transpose(1, 2), cos.to(DEV), sin.to(DEV))
    qv, kv = qe.detach().clone(), ke.detach().clone()
    torch.autograd.backward([qe, ke], [dq.to(DEV), dk.to(DEV)])
    qt, kt = q.transpose(1, 2), k.transpose(1, 2)
    qo, ko = E.rope_fwd(qt[..., :rd], kt[..., :rd], cos, sin)
    gq, gk = E.rope_bwd(dq[..., :rd], dk[..., :rd], cos, sin)
    assert_close(qv[..., :rd], qo, 1e-2, "q rotated part"); assert_close(kv[..., :rd], ko, 1e-2, "k rotated part")
    assert torch.equal(qv[..., rd:].cpu(), qt[..., rd:]) and torch.equal(kv[..., rd:].cpu(), kt[..., rd:])
    assert_close(qs.grad.transpose(1, 2)[..., :rd], gq, 1e-2, "dq rotated part")
    assert_close(ks.grad.transpose(1, 2)[..., :rd], gk, 1e-2, "dk rotated part")
    assert torch.equal(qs.grad.transpose(1, 2)[..., rd:].cpu(), dq[..., rd:]) and torch.equal(ks.grad.transpose(1, 2)[..., rd:].cpu(), dk[..., rd:])


def test_rope_head_major_storage_and_unsqueeze_dim_2():
    """q/k stored [B, H, L, D] (head-major) go through the strided path; unsqueeze_dim=2 means the caller's
    tensors are [B, L, H, D]."""
    gen = g(31)
    b, l, qh, kh, d = 2, 33, 6, 2, 64
    q = torch.randn(b, qh, l, d, generator=gen).to(torch.bfloat16); k = torch.randn(b, kh, l, d, generator=gen).to(torch.bfloat16)
    cos, sin = E.rope_cos_sin(torch.arange(l)[None], d, 1e4, torch.bfloat16)
    qo, ko = E.rope_fwd(q, k, cos, sin)
    qd, kd = q.to(DEV).contiguous(), k.to(DEV).contiguous()          # head-major storage
    q1, k1 = core.fused_apply_rope(qd, kd, cos.to(DEV), sin.to(DEV))
    assert q1.data_ptr() == qd.data_ptr()
    assert_close(q1, qo, 1e-2, "q"); assert_close(k1, ko, 1e-2, "k")
    q2 = q.to(DEV).transpose(1, 2).contiguous(); k2 = k.to(DEV).transpose(1, 2).contiguous()   # [B, L, H, D]
    q3, k3 = core.fused_apply_rope(q2, k2, cos.to(DEV), sin.to(DEV), unsqueeze_dim=2)
    assert q3.shape == (b, l, qh, d)
    assert_close(q3.transpose(1, 2), qo, 1e-2, "q, unsqueeze_dim=2"); assert_close(k3.transpose(1, 2), ko, 1e-2, "k, unsqueeze_dim=2")


def test_rope_round_trip_full_size():
    """Llama-3-8B shape (8 x 4096 tokens): backward(forward(x)) == x because cos^2 + sin^2 == 1; and
    memory next to the tensors is untouched."""
    b, l, qh, kh, d = 8, 4096, 32, 8, 128
    gen = torch.Generator(DEV).manual_seed(1)
    pad = 1024
    qbuf = torch.randn(b * l * qh * d + 2 * pad, device=DEV, generator=gen).to(torch.bfloat16)
    kbuf = torch.randn(b * l * kh * d + 2 * pad, device=DEV, generator=gen).to(torch.bfloat16)
    q0, k0 = qbuf.clone(), kbuf.clone()
    q = qbuf[pad:-pad].view(b, l, qh, d).transpose(1, 2); k = kbuf[pad:-pad].view(b, l, kh, d).transpose(1, 2)
    cos, sin = E.rope_cos_sin(torch.arange(l)[None], d, 5e5, torch.float32)
    cos, sin = cos.to(DEV).to(torch.bfloat16), sin.to(DEV).to(torch.bfloat16)
    core.fused_apply_rope(q, k, cos, sin)
    assert torch.equal(qbuf[:pad], q0[:pad]) and torch.equal(qbuf[-pad:], q0[-pad:])
    assert torch.equal(kbuf[:pad], k0[:pad]) and torch.equal(kbuf[-pad:], k0[-pad:])
    assert not torch.equal(qbuf, q0)
    lib = _C.lib()
    st = lambda t: (t.stride(0), t.stride(1), t.stride(2))
    _C.check(lib.mdy_rope(q.data_ptr(), q.data_ptr(), k.data_ptr(), k.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                          b, l, qh, kh, d, 1, *st(q), *st(q), *st(k), *st(k), 1, _C.MDY_BF16,
                          torch.cuda.current_stream().cuda_stream), "mdy_rope")
    torch.cuda.synchronize()
    # two bf16 roundings of O(1) values, cos/sin themselves rounded to bf16
    assert (qbuf.float() - q0.float()).abs().max() < 0.06
    assert (kbuf.float() - k0.float()).abs().max() < 0.06


# ----------------------------------------------------------------------------------------------- SwiGLU
@pytest.mark.parametrize("c", golden_cases("swiglu.pt"))
def test_swiglu_golden(c):
    r = REL[c["dy"].dtype]
    if c["kind"] == "split":
        up, gate = leaf(c["up"]), leaf(c["gate"])
        y = core.triton_fused_up_gate_silu(up, gate); y.backward(c["dy"].to(DEV))
        assert_close(y, c["y"], r, "y"); assert_close(up.grad, c["dup"], r, "dup"); assert_close(gate.grad, c["dgate"], r, "dgate")
    else:
        x = leaf(c["x"])
        y = core.triton_fused_up_gate_silu_no_split(x, c["order"]); y.backward(c["dy"].to(DEV))
        assert_close(y, c["y"], r, "y"); assert_close(x.grad, c["dx"], r, "dx")


@pytest.mark.parametrize("shape,dt", [((4096, 4864), torch.bfloat16), ((2, 512, 4864), torch.float32), ((1024, 14336), torch.bfloat16),
                                      ((3, 1001), torch.float16), ((1, 1), torch.float32), ((5, 7, 9), torch.bfloat16), ((0, 16), torch.bfloat16)])
def test_swiglu_vs_oracle(shape, dt):
    gen = g(sum(shape) + 1)
    up = (torch.randn(*shape, generator=gen) * 2).to(dt); gate = (torch.randn(*shape, generator=gen) * 3).to(dt)
    dy = torch.randn(*shape, generator=gen).to(dt)
    ug, gg = leaf(up), leaf(gate)
    y = core.triton_fused_up_gate_silu(ug, gg); y.backward(dy.to(DEV))
    r = REL[dt]
    if y.numel() == 0:
        assert y.shape == tuple(shape); return
    assert_close(y, E.swiglu_fwd(up, gate), r, "y")
    du, dg = E.swiglu_bwd(dy, up, gate)
    assert_close(ug.grad, du, r, "dup"); assert_close(gg.grad, dg, r, "dgate")


def test_swiglu_strided_halves_and_noncontiguous_dy():
    """up/gate as halves of one projection (row stride 2N) and an expanded (stride-0) upstream gradient,
    which the reference kernel would mis-read."""
    gen = g(77)
    x = torch.randn(64, 2 * 1024, generator=gen).to(torch.bfloat16).to(DEV)
    up, gate = leaf(x[:, :1024]), leaf(x[:, 1024:])
    xs = x.clone().requires_grad_(True)
    y1 = core.triton_fused_up_gate_silu(xs[:, :1024], xs[:, 1024:])
    y2 = core.triton_fused_up_gate_silu(up, gate)
    assert torch.equal(y1, y2)
    y1.sum().backward(); y2.sum().backward()
    assert torch.equal(xs.grad[:, :1024], up.grad) and torch.equal(xs.grad[:, 1024:], gate.grad)
    du, dg = E.swiglu_bwd(torch.ones(64, 1024), x[:, :1024].cpu(), x[:, 1024:].cpu())
    assert_close(up.grad, du, 1e-2); assert_close(gate.grad, dg, 1e-2)
    for order in ("up-gate", "gate-up"):
        xn = x.clone().requires_grad_(True)
        y = core.triton_fused_up_gate_silu_no_split(xn, order)
        u, gt = E.split_no_split(x.cpu(), order)
        assert_close(y, E.swiglu_fwd(u, gt), 1e-2, order)
        y.sum().backward()
        du, dg = E.swiglu_bwd(torch.ones(64, 1024), u, gt)
        gu, gg = E.split_no_split(xn.grad, order)
        assert_close(gu, du, 1e-2); assert_close(gg, dg, 1e-2)


def test_swiglu_linearity_full_size():
    """Qwen2-7B shape: y is linear in `up`, and scaling by 2 is exact in binary floating point."""
    gen = torch.Generator(DEV).manual_seed(2)
    up = torch.randn(32768, 18944, device=DEV, generator=gen, dtype=torch.bfloat16)
    gate = torch.randn(32768, 18944, device=DEV, generator=gen, dtype=torch.bfloat16)
    y1 = core.triton_fused_up_gate_silu(up, gate)
    y2 = core.triton_fused_up_gate_silu(up * 2, gate)
    assert torch.equal(y1 * 2, y2)
    sample = slice(0, 64)
    assert_close(y1[sample], E.swiglu_fwd(up[sample].cpu(), gate[sample].cpu()), 1e-2)


# ---------------------------------------------------------------------------------------- cross-entropy
@pytest.fixture(params=["auto", "smem1024x2", "smem256x8", "smem512x2_small_slices", "row"], autouse=False)
def fused_impl(request):
    """Run a test under every one-pass implementation: the default dispatch (the cluster kernel that stages
    the row slice in shared memory), two other CTA shapes of it, 16 KB slices that force clusters of up to
    8 CTAs, and the row-per-CTA kernel it falls back to."""
    name = request.param
    impl = 1 if name == "row" else 0
    nt, vpc, kb, minb = {"smem1024x2": (1024, 2, 0, 1), "smem256x8": (256, 8, 0, 2),
                         "smem512x2_small_slices": (512, 2, 16, 2)}.get(name, (0, 0, 0, 0))
    _C.set_tunable(_C.TUNE_CE_FUSED_IMPL, impl)
    _C.set_tunable(_C.TUNE_CE_CLUSTER_THREADS, nt)
    _C.set_tunable(_C.TUNE_CE_CLUSTER_VPC, vpc)
    _C.set_tunable(_C.TUNE_CE_CLUSTER_SLICE_KB, kb)
    _C.set_tunable(_C.TUNE_CE_CLUSTER_MINB, minb)
    yield name
    for t in (_C.TUNE_CE_FUSED_IMPL, _C.TUNE_CE_CLUSTER_THREADS, _C.TUNE_CE_CLUSTER_VPC,
              _C.TUNE_CE_CLUSTER_SLICE_KB, _C.TUNE_CE_CLUSTER_MINB):
        _C.set_tunable(t, 0)
    torch.cuda.synchronize()
    assert _C.lib().mdy_last_device_error(1) == 0, "a bounded device-side wait expired"


@pytest.mark.parametrize("c", golden_cases("cross_entropy.pt"))
def test_ce_golden(c, fused_impl):
    lg, lb = c["logits"], c["labels"].to(DEV)
    r = REL[lg.dtype]
    x = leaf(lg)
    losses = _FastCrossEntropyLoss.apply(x, lb, False)
    losses.backward(c["dlosses"].to(DEV))
    assert torch.allclose(losses.cpu(), c["losses"], rtol=LOSS_TOL, atol=LOSS_TOL)
    assert_close(x.grad, c["dlogits"], r, "dlogits")
    # in-place variant writes the same gradient into the logits' storage
    x2 = leaf(lg); xin = x2 * 1.0
    losses2 = _FastCrossEntropyLoss.apply(xin, lb, True)
    losses2.backward(c["dlosses"].to(DEV))
    assert torch.equal(xin.detach(), x.grad)
    # scalar API (one-pass kernel)
    x3 = leaf(lg)
    loss = triton_entropy_loss(x3, lb); loss.backward()
    loss_close(loss, c["loss"])
    if "dlogits_scalar" in c:
        assert_close(x3.grad, c["dlogits_scalar"], r, "dlogits scalar")
    x4 = leaf(lg)
    loss_n = core.fast_cross_entropy_loss(x4.view(1, *lg.shape), lb.view(1, -1), n_items=c["n_items"]); loss_n.backward()
    loss_close(loss_n, c["loss_n"])
    if "dlogits_n" in c:
        assert_close(x4.grad, c["dlogits_n"], r, "dlogits n")
    with torch.no_grad():
        loss_close(triton_entropy_loss(lg.to(DEV), lb), c["loss"])


@pytest.mark.parametrize("m,v,sigma,frac,dt", [
    (256, 151936, 2.0, 0.05, torch.bfloat16),   # Qwen2 vocab
    (128, 128256, 3.0, 0.0, torch.bfloat16),    # Llama-3 vocab
    (128, 152064, 2.0, 0.10, torch.bfloat16),   # Qwen2-7B vocab
    (64, 256000, 4.0, 0.05, torch.bfloat16),
    (64, 32000, 1.0, 0.05, torch.float16),
    (32, 50257, 2.0, 0.1, torch.float32),       # odd vocab, float32
    (16, 1501, 1.0, 0.2, torch.bfloat16),       # row stride not 16-byte aligned -> scalar path
    (8, 5, 1.0, 0.0, torch.float32),
    (4, 1, 1.0, 0.0, torch.float32),
    (1, 8192, 10.0, 0.0, torch.bfloat16),
    (7, 1000, 1.0, 1.0, torch.bfloat16),        # every row ignored
])
def test_ce_vs_oracle(m, v, sigma, frac, dt, fused_impl):
    gen = g(m + v)
    lg = (torch.randn(m, v, generator=gen) * sigma).to(dt)
    lb = torch.randint(0, v, (m,), generator=gen)
    lb[torch.rand(m, generator=gen) < frac] = -100
    dl = torch.randn(m, generator=gen)
    r = REL[dt]
    # float16 gradients of tiny probabilities underflow: allow one subnormal step of the storage format
    atol = 2.0 ** -24 if dt == torch.float16 else 0.0
    lo, lse_o = E.ce_rows(lg, lb)
    # two-phase path
    x = leaf(lg)
    losses = _FastCrossEntropyLoss.apply(x, lb.to(DEV), False); losses.backward(dl.to(DEV))
    assert torch.allclose(losses.cpu(), lo, rtol=LOSS_TOL, atol=LOSS_TOL)
    assert_close(x.grad, E.ce_grad(lg, lb, lse_o, dl), r, "dlogits", atol)
    # one-pass path, in place and not
    n = int((lb != -100).sum())
    for inplace in (False, True):
        x = leaf(lg); xin = x * 1.0
        loss = triton_entropy_loss(xin, lb.to(DEV), inplace=inplace); loss.backward()
        if n == 0:
            assert torch.isnan(loss)  # 0/0, as in the reference
            continue
        loss_close(loss, E.ce_scalar(lg, lb))
        assert_close(x.grad, E.ce_grad(lg, lb, lse_o, torch.tensor(1.0 / n)), r, f"fused dlogits inplace={inplace}", atol)
        if inplace:
            assert torch.equal(xin.detach(), x.grad)
    if n:
        loss_close(E.hf_cross_entropy(lg, lb), E.ce_scalar(lg, lb))


def test_ce_upstream_gradient_scaling(fused_impl):
    """loss * 0.25 (gradient accumulation) must scale the gradient the forward already wrote."""
    gen = g(9)
    lg = (torch.randn(32, 4096, generator=gen) * 2).to(torch.bfloat16); lb = torch.randint(0, 4096, (32,), generator=gen)
    x = leaf(lg)
    (triton_entropy_loss(x, lb.to(DEV)) * 0.25).backward()
    _, lse = E.ce_rows(lg, lb)
    assert_close(x.grad, E.ce_grad(lg, lb, lse, torch.tensor(0.25 / 32)), 1e-2)


def test_ce_float16_with_a_loss_scaler_keeps_small_gradients():
    """float16 logits under a GradScaler: loss * 65536 is what gets differentiated.  The gradient of a rare
    token, (softmax - onehot) / n_items, is below float16's smallest subnormal, but times the scale it is
    representable: it must arrive, not be flushed to zero before the scale is applied."""
    gen = g(11)
    m, v, scale = 64, 32000, 65536.0
    lg = (torch.randn(m, v, generator=gen) * 4).to(torch.float16); lb = torch.randint(0, v, (m,), generator=gen)
    x = leaf(lg)
    (triton_entropy_loss(x, lb.to(DEV)) * scale).backward()
    _, lse = E.ce_rows(lg, lb)
    want = E.ce_grad(lg, lb, lse, torch.tensor(scale / m))
    assert_close(x.grad, want, 1e-2, "scaled float16 dlogits", 2.0 ** -24)
    unscaled = E.ce_grad(lg, lb, lse, torch.tensor(1.0 / m)).abs()
    lost = (unscaled < 2.0 ** -25) & (want.abs() >= 2.0 ** -14)   # flushed without the scale, normal with it
    assert lost.any()
    assert (x.grad.cpu()[lost] != 0).all()


def test_ce_one_pass_gradient_is_handed_out_once():
    """The one-pass path keeps no logits, only the gradient it wrote: a second backward through the same loss
    would rescale the tensor the first one returned, so it raises instead; the per-row function, which the
    reference also offers, can be walked twice."""
    gen = g(12)
    lg = (torch.randn(16, 2048, generator=gen) * 2).to(torch.bfloat16); lb = torch.randint(0, 2048, (16,), generator=gen).to(DEV)
    x = leaf(lg)
    loss = triton_entropy_loss(x, lb)
    (loss * 0.5).backward(retain_graph=True)
    first = x.grad.clone()
    with pytest.raises(RuntimeError, match="once"):
        (loss * 0.5).backward()
    assert torch.equal(x.grad, first)
    x = leaf(lg)
    losses = _FastCrossEntropyLoss.apply(x, lb, False)
    losses.sum().backward(retain_graph=True); g1 = x.grad.clone(); x.grad = None
    losses.sum().backward()
    assert torch.equal(x.grad, g1)


def test_ce_out_of_range_label_and_neg_inf_logits():
    lg = torch.randn(4, 64) * 2
    lg[1, 10:20] = float("-inf")
    lb = torch.tensor([3, 5, 64 + 7, -100])  # row 2: label outside the vocabulary, not -100
    x = leaf(lg)
    losses = _FastCrossEntropyLoss.apply(x, lb.to(DEV), False)
    losses.sum().backward()
    lo, lse = E.ce_rows(lg, lb)
    assert torch.allclose(losses.cpu(), lo, atol=1e-5) and losses[2] == 0
    assert_close(x.grad, E.ce_grad(lg, lb, lse, torch.ones(4)), 1e-4)
    assert torch.isfinite(x.grad).all()


def test_ce_properties_full_size(fused_impl):
    """Llama-3 shape slice at full vocabulary, 8192 rows (2.1 GB of logits): valid rows of dlogits sum to
    ~0 (softmax minus one-hot), ignored rows are exactly 0, the label entry is the only negative one,
    and the one-pass kernel agrees with the two-phase kernels."""
    m, v = 8192, 128256
    gen = torch.Generator(DEV).manual_seed(1)
    lg = (torch.randn(m, v, device=DEV, generator=gen) * 3).to(torch.bfloat16)
    lb = torch.randint(0, v, (m,), device=DEV, generator=gen)
    lb[::16] = -100
    n = int((lb != -100).sum())
    x = lg.clone().requires_grad_(True)
    loss = triton_entropy_loss(x, lb); loss.backward()
    d = x.grad
    assert (d[::16] == 0).all()
    valid = lb != -100
    rows = d[valid].float()
    assert rows.sum(-1).abs().max() * n < 0.05            # each row of (p - onehot) sums to 0
    neg = (rows < 0).sum(-1)
    assert (neg == 1).all()
    idx = lb[valid]
    assert (rows.gather(1, idx[:, None]) < 0).all()
    x2 = lg.clone().requires_grad_(True)
    l2 = _FastCrossEntropyLoss.apply(x2, lb, False)
    (l2.sum() / n).backward()
    loss_close(loss, l2.sum() / n)
    assert_close(d[:512], x2.grad[:512], 1e-2, "fused vs two-phase")
    # oracle on a slice the CPU finishes quickly
    sl = slice(0, 64)
    lo, lse_o = E.ce_rows(lg[sl].cpu(), lb[sl].cpu())
    assert torch.allclose(l2[sl].cpu(), lo, rtol=LOSS_TOL, atol=LOSS_TOL)
    assert_close(d[sl], E.ce_grad(lg[sl].cpu(), lb[sl].cpu(), lse_o, torch.tensor(1.0 / n)), 1e-2)


def test_ce_bounded_wait_runs_out_sets_the_flag_and_poisons_the_loss():
    """Failure detection of the cluster kernel, without faulting anything: a test hook shortens the bound of
    its mbarrier waits to about a millisecond and leaves one chunk of one row unrequested, so the wait for
    it runs out.  The launch must still return, the device must stay usable, the flag must be raised, the
    affected row's loss must be NaN (never a finite wrong number), and the next launch must be correct."""
    import time
    lib = _C.lib()
    gen = g(21)
    m, v = 8, 128256
    lg = (torch.randn(m, v, generator=gen) * 3).to(torch.bfloat16); lb = torch.randint(0, v, (m,), generator=gen)
    lo, lse_o = E.ce_rows(lg, lb)
    x, labels = lg.to(DEV), lb.to(DEV)
    inv = torch.full((1,), 1.0 / m, device=DEV)

    def run():
        dl = torch.empty_like(x); losses = torch.empty(m, device=DEV); lse = torch.empty(m, device=DEV)
        rc = lib.mdy_ce_fused(x.data_ptr(), dl.data_ptr(), labels.data_ptr(), losses.data_ptr(), lse.data_ptr(),
                              inv.data_ptr(), 1.0, m, v, v, _C.MDY_BF16, torch.cuda.current_stream().cuda_stream)
        return rc, dl, losses

    torch.cuda.synchronize()
    assert lib.mdy_last_device_error(1) == 0
    _C.set_tunable(_C.TUNE_CE_WAIT_TEST, 1)
    try:
        t0 = time.perf_counter()
        rc, _, losses = run()
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
    finally:
        _C.set_tunable(_C.TUNE_CE_WAIT_TEST, 0)
    assert rc == 0
    assert elapsed < 1.0, f"the kernel took {elapsed:.2f} s to give up"
    assert lib.mdy_last_device_error(1) == 1, "the expired wait was not flagged"
    assert lib.mdy_last_device_error(0) == 0, "the flag was not cleared"
    losses = losses.cpu()
    assert torch.isnan(losses[0]), "the row whose data never arrived must not get a finite loss"
    assert torch.allclose(losses[1:], lo[1:], rtol=LOSS_TOL, atol=LOSS_TOL)
    # the context is intact: the same launch without the hook is correct
    rc, dl, losses = run()
    torch.cuda.synchronize()
    assert rc == 0 and lib.mdy_last_device_error(1) == 0
    assert torch.allclose(losses.cpu(), lo, rtol=LOSS_TOL, atol=LOSS_TOL)
    assert_close(dl, E.ce_grad(lg, lb, lse_o, torch.tensor(1.0 / m)), 1e-2, "dlogits after the expired wait")


def test_config1_full_size_against_the_cpu_oracle():
    """The Qwen2-0.5B-shaped configuration in full (4 x 1024 tokens, seed 0): float32 on the CPU oracle, the
    bfloat16 cast of the same draw on the GPU.  RMSNorm [4096, 896], RoPE 14 q / 2 kv heads x 64, SwiGLU
    [4096, 4864], cross-entropy [4096, 151936] with 5 % of the labels ignored."""
    gen = g(0)
    dt = torch.bfloat16
    M, H, F, V, B, L, QH, KH, D = 4096, 896, 4864, 151936, 4, 1024, 14, 2, 64
    x = torch.randn(M, H, generator=gen); w = 1 + 0.02 * torch.randn(H, generator=gen); dy = torch.randn(M, H, generator=gen)
    y, dx, dw = run_rmsnorm(x.to(dt), w.to(dt), 1e-6, dy.to(dt))
    yo, _ = E.rmsnorm_fwd(x.to(dt), w.to(dt), 1e-6); dxo, dwo = E.rmsnorm_bwd(dy.to(dt), x.to(dt), w.to(dt), 1e-6)
    assert_close(y, yo, 1e-2, "rmsnorm y"); assert_close(dx, dxo, 1e-2, "rmsnorm dx"); assert_close(dw, dwo, 1e-2, "rmsnorm dw")
    q = torch.randn(B, L, QH, D, generator=gen).to(dt); k = torch.randn(B, L, KH, D, generator=gen).to(dt)
    dq = torch.randn(B, QH, L, D, generator=gen).to(dt); dk = torch.randn(B, KH, L, D, generator=gen).to(dt)
    cos, sin = E.rope_cos_sin(torch.arange(L)[None], D, 1e6, dt)
    qs, ks = leaf(q), leaf(k)
    qe, ke = core.fused_apply_rope((qs * 1.0).transpose(1, 2), (ks * 1.0).transpose(1, 2), cos.to(DEV), sin.to(DEV))
    qv, kv = qe.detach().clone(), ke.detach().clone()
    torch.autograd.backward([qe, ke], [dq.to(DEV), dk.to(DEV)])
    qo, ko = E.rope_fwd(q.transpose(1, 2), k.transpose(1, 2), cos, sin); gq, gk = E.rope_bwd(dq, dk, cos, sin)
    assert_close(qv, qo, 1e-2, "rope q"); assert_close(kv, ko, 1e-2, "rope k")
    assert_close(qs.grad.transpose(1, 2), gq, 1e-2, "rope dq"); assert_close(ks.grad.transpose(1, 2), gk, 1e-2, "rope dk")
    up = torch.randn(M, F, generator=gen).to(dt); gate = torch.randn(M, F, generator=gen).to(dt); sdy = torch.randn(M, F, generator=gen).to(dt)
    ug, gg = leaf(up), leaf(gate)
    sy = core.triton_fused_up_gate_silu(ug, gg); sy.backward(sdy.to(DEV))
    du, dg = E.swiglu_bwd(sdy, up, gate)
    assert_close(sy, E.swiglu_fwd(up, gate), 1e-2, "swiglu y"); assert_close(ug.grad, du, 1e-2, "swiglu dup"); assert_close(gg.grad, dg, 1e-2, "swiglu dgate")
    del ug, gg, sy, du, dg
    lg = (torch.randn(M, V, generator=gen) * 2).to(dt); lb = torch.randint(0, V, (M,), generator=gen)
    lb[torch.rand(M, generator=gen) < 0.05] = -100
    xg = leaf(lg)
    loss = triton_entropy_loss(xg.view(B, L, V), lb.view(B, L).to(DEV)); loss.backward()
    lo, lse = E.ce_rows(lg, lb)
    n = int((lb != -100).sum())
    loss_close(loss, lo.sum() / n)
    want = E.ce_grad(lg, lb, lse, torch.tensor(1.0 / n))
    assert_close(xg.grad, want, 1e-2, "cross-entropy dlogits")


def test_ce_cluster_launch_geometry():
    """The default one-pass launch: clusters are as small as the shared memory allows, the grid is one
    wave of co-resident clusters (or one cluster per row if there are fewer rows), and rows short
    enough for several CTAs per SM get the small-CTA shape."""
    import ctypes
    lib = _C.lib()
    sms = lib.mdy_num_sms()

    def geometry(m, v, dt=torch.bfloat16):
        x = torch.randn(m, v, device=DEV).to(dt).requires_grad_(True)
        triton_entropy_loss(x, torch.randint(0, v, (m,), device=DEV)).backward()
        out = [ctypes.c_int(0) for _ in range(4)]
        _C.check(lib.mdy_ce_last_geometry(*[ctypes.byref(o) for o in out]), "geometry")
        return tuple(o.value for o in out)

    c, ncl, nt, smem = geometry(1024, 128256)          # 250 KB rows: two CTAs per row, one CTA per SM
    assert (c, nt) == (2, 512) and ncl == sms // 2 and 125 * 1024 < smem < 132 * 1024
    c, ncl, nt, smem = geometry(2048, 32000)           # 62.5 KB rows: one CTA per row, three per SM
    assert (c, nt) == (1, 256) and ncl == 3 * sms and smem < 66 * 1024
    c, ncl, nt, smem = geometry(3, 128256)             # fewer rows than co-resident clusters
    assert (c, ncl) == (2, 3)
    c, ncl, nt, smem = geometry(64, 128256, torch.float32)   # 501 KB rows: clusters of eight small CTAs, three per SM
    assert (c, nt) == (8, 256) and ncl <= 3 * sms // 8 and smem < 70 * 1024
    c, ncl, nt, smem = geometry(64, 98304, torch.float32)    # 384 KB rows: still two 192 KB slices, one CTA per SM
    assert (c, nt) == (2, 512)
    assert lib.mdy_last_device_error(1) == 0


# --------------------------------------------------------------------------------------------- max / min
def _first_extreme(x, take_min):
    """Reference result on CPU in float32: the extreme of each row and the first column holding it."""
    xf = x.float().cpu()
    vals = xf.min(-1).values if take_min else xf.max(-1).values
    first = (xf == vals[..., None]).float().argmax(-1)
    return vals, first


@pytest.mark.parametrize("c", golden_cases("maxmin.pt"))
def test_max_min_golden(c):
    """Bit-exact against the reference kernels' stored outputs."""
    from mdy_triton.core import triton_max, triton_min
    x = c["x"].to(DEV)
    for fn, key in ((triton_max, "max"), (triton_min, "min")):
        r = fn(x)
        assert torch.equal(r.values.cpu(), c[key + "_values"]) and torch.equal(r.indices.cpu(), c[key + "_indices"])


@pytest.mark.parametrize("shape,dt", [
    ((64, 7), torch.float32), ((1000, 256), torch.bfloat16), ((33, 257), torch.float16), ((5, 2048), torch.bfloat16),
    ((16, 2056), torch.float32), ((12, 128256), torch.bfloat16), ((3, 50257), torch.float32), ((1, 1), torch.float32),
    ((2, 3, 4096), torch.bfloat16), ((300, 1001), torch.bfloat16),
])
@pytest.mark.parametrize("take_min", [False, True])
def test_max_min_match_torch(shape, dt, take_min):
    from mdy_triton.core import triton_max, triton_min
    # few distinct values, so every row has ties: the index must be the first occurrence
    x = torch.randint(-20, 20, shape, generator=g(sum(shape))).to(dt).to(DEV)
    out = (triton_min if take_min else triton_max)(x)
    vals, first = _first_extreme(x, take_min)
    assert out.func_type == ("triton_min" if take_min else "triton_max")
    assert out.values.dtype == dt and out.indices.dtype == torch.int64 and out.values.shape == x.shape[:-1]
    assert torch.equal(out.values.float().cpu(), vals) and torch.equal(out.indices.cpu(), first)
    y = torch.randn(shape, generator=g(1 + sum(shape))).to(dt).to(DEV)       # continuous values
    v, i = (triton_min if take_min else triton_max)(y)
    t = torch.min(y, -1) if take_min else torch.max(y, -1)
    assert torch.equal(v, t.values) and torch.equal(y.gather(-1, i[..., None])[..., 0], t.values)


def test_max_min_axis_keepdim_strides_and_nan():
    from mdy_triton.core import triton_max, triton_min
    x = torch.randn(6, 50, 40, generator=g(9)).to(DEV)
    for axis in (0, 1, -1, -2):
        for keepdim in (False, True):
            a, b = triton_max(x, axis=axis, keepdim=keepdim), torch.max(x, dim=axis, keepdim=keepdim)
            assert torch.equal(a.values, b.values) and torch.equal(a.indices, b.indices)
            a, b = triton_min(x, axis, keepdim), torch.min(x, dim=axis, keepdim=keepdim)
            assert torch.equal(a.values, b.values) and torch.equal(a.indices, b.indices)
    wide = torch.randn(32, 4096 + 64, generator=g(10)).to(torch.bfloat16).to(DEV)
    view = wide[:, 8:4096 + 8]                                   # row stride larger than the row, 16-byte aligned
    a, b = triton_max(view), torch.max(view, -1)
    assert torch.equal(a.values, b.values) and torch.equal(a.indices, b.indices)
    odd = wide[:, 3:4000]                                        # misaligned rows: scalar path
    a, b = triton_min(odd), torch.min(odd, -1)
    assert torch.equal(a.values, b.values) and torch.equal(a.indices, b.indices)
    n = torch.randn(4, 5000, generator=g(11)).to(DEV)
    n[1, 77] = float("nan"); n[1, 4000] = float("nan"); n[3, 0] = float("inf")
    for fn in (triton_max, triton_min):
        r = fn(n)
        assert torch.isnan(r.values[1]) and r.indices[1] == 77 and not torch.isnan(r.values[[0, 2, 3]]).any()
    assert triton_max(n).indices[3] == 0
    with pytest.raises(RuntimeError):
        triton_max(torch.randn(4, 4))                            # CPU tensor: no fallback


def test_direct_c_abi_calls_with_strides():
    """Call the entry points directly with row strides larger than the row."""
    lib = _C.lib()
    st = torch.cuda.current_stream().cuda_stream
    gen = g(4)
    xb = torch.randn(10, 256 + 32, generator=gen).to(torch.bfloat16).to(DEV)
    w = torch.randn(256, generator=gen).to(torch.bfloat16).to(DEV)
    yb = torch.zeros(10, 256 + 64, dtype=torch.bfloat16, device=DEV)
    rstd = torch.empty(10, dtype=torch.float32, device=DEV)
    _C.check(lib.mdy_rmsnorm_fwd(xb.data_ptr(), w.data_ptr(), yb.data_ptr(), rstd.data_ptr(), 10, 256, 288, 320, 1e-6,
                                 _C.MDY_BF16, _C.MDY_BF16, st), "fwd")
    yo, rms = E.rmsnorm_fwd(xb[:, :256].cpu(), w.cpu(), 1e-6)
    assert_close(yb[:, :256], yo, 1e-2); assert (yb[:, 256:] == 0).all()
    assert_close(rstd, 1.0 / rms, 1e-5)
    # cross-entropy with a padded row stride, split mode and a vocab offset
    v, rs, vs = 1000, 1008, 3000
    lg = (torch.randn(6, rs, generator=gen) * 2).to(torch.bfloat16).to(DEV)
    lb = torch.tensor([3000, 3999, 10, 5000, -100, 3500], device=DEV)
    losses = torch.full((6,), 7.0, device=DEV); lse = torch.full((6,), 7.0, device=DEV)
    _C.check(lib.mdy_ce_fwd(lg.data_ptr(), lb.data_ptr(), losses.data_ptr(), lse.data_ptr(), 6, v, rs, vs, 1, _C.MDY_BF16, st), "ce_fwd")
    lo, lse_o = E.ce_rows(lg[:, :v].cpu(), lb.cpu(), vocab_start=vs, split=True)
    assert torch.allclose(losses.cpu(), lo, atol=1e-4) and torch.allclose(lse.cpu(), lse_o, atol=1e-4)
    dl = torch.randn(6, generator=gen).to(DEV)
    out = torch.full_like(lg, 5.0)
    _C.check(lib.mdy_ce_bwd(dl.data_ptr(), 1, _C.MDY_F32, lg.data_ptr(), out.data_ptr(), lb.data_ptr(), lse.data_ptr(), 6, v, rs, vs, 1,
                            _C.MDY_BF16, st), "ce_bwd")
    assert_close(out[:, :v], E.ce_grad(lg[:, :v].cpu(), lb.cpu(), lse_o, dl.cpu(), vocab_start=vs), 1e-2)
    assert (out[:, v:] == 5.0).all()
    # combine kernel against the oracle
    stats = torch.randn(4, 2, 50, generator=gen).to(DEV)
    lb2 = torch.randint(0, 10, (50,), generator=gen).to(DEV); lb2[::5] = -100
    l_out = torch.empty(50, device=DEV); s_out = torch.empty(50, device=DEV)
    _C.check(lib.mdy_ce_vp_combine(stats.data_ptr(), lb2.data_ptr(), l_out.data_ptr(), s_out.data_ptr(), 4, 50, st), "combine")
    lo, so = E.vp_combine(stats.cpu(), lb2.cpu())
    assert torch.allclose(l_out.cpu(), lo, atol=1e-5) and torch.allclose(s_out.cpu(), so, atol=1e-5)
    assert _C.launch_count() > 0


def test_entry_points_are_cuda_graph_capturable():
    """The C-ABI calls enqueue work only: capturing them on a side stream into a CUDA graph and replaying
    the graph must reproduce the eager results (includes the cluster launch of the one-pass cross-entropy)."""
    lib = _C.lib()
    gen = torch.Generator(DEV).manual_seed(5)
    M, N, V = 256, 2048, 32000
    bf = _C.MDY_BF16
    x = torch.randn(M, N, device=DEV, dtype=torch.bfloat16, generator=gen); w = torch.ones(N, device=DEV, dtype=torch.bfloat16)
    y = torch.empty_like(x); rstd = torch.empty(M, device=DEV)
    up = torch.randn(M, N, device=DEV, dtype=torch.bfloat16, generator=gen); sy = torch.empty_like(up)
    lg = torch.randn(M, V, device=DEV, dtype=torch.bfloat16, generator=gen); dlg = torch.empty_like(lg)
    lb = torch.randint(0, V, (M,), device=DEV, generator=gen)
    losses = torch.empty(M, device=DEV); lse = torch.empty(M, device=DEV); inv = torch.tensor([1.0 / M], device=DEV)

    def enqueue(stream):
        st = stream.cuda_stream
        _C.check(lib.mdy_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), M, N, N, N, 1e-6, bf, bf, st), "n")
        _C.check(lib.mdy_swiglu_fwd(up.data_ptr(), x.data_ptr(), sy.data_ptr(), M, N, N, N, N, bf, st), "s")
        _C.check(lib.mdy_ce_fused(lg.data_ptr(), dlg.data_ptr(), lb.data_ptr(), losses.data_ptr(), lse.data_ptr(), inv.data_ptr(), 1.0,
                                  M, V, V, bf, st), "c")

    enqueue(torch.cuda.current_stream())          # eager (also performs one-time set-up outside capture)
    torch.cuda.synchronize()
    ref = [t.clone() for t in (y, sy, dlg, losses)]
    for t in (y, sy, dlg, losses):
        t.zero_()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            enqueue(side)
    torch.cuda.synchronize()
    assert all(float(t.float().abs().sum()) == 0 for t in (y, sy, losses))   # capture did not execute
    graph.replay()
    torch.cuda.synchronize()
    for got, want in zip((y, sy, dlg, losses), ref):
        assert torch.equal(got, want)


def test_megatron_swiglu_adapter():
    from mdy_triton_b200.core.megatron import swiglu_impl
    gen = g(41)
    x = torch.randn(3, 16, 2 * 256, generator=gen).to(torch.bfloat16); b = torch.randn(2 * 256, generator=gen).to(torch.bfloat16)
    xd = leaf(x)
    y = swiglu_impl(xd, b.to(DEV)); y.float().sum().backward()
    xb = (x.float() + b.float()).to(torch.bfloat16)
    up, gate = E.split_no_split(xb, "gate-up")
    assert_close(y, E.swiglu_fwd(up, gate), 1e-2, "y")
    du, dg = E.swiglu_bwd(torch.ones(3, 16, 256), up, gate)
    gu, gg = E.split_no_split(xd.grad, "gate-up")
    assert_close(gu, du, 1e-2, "dup"); assert_close(gg, dg, 1e-2, "dgate")


def test_operators_on_a_side_stream_and_from_threads():
    """Entry points enqueue on the caller's current stream and keep no per-call host state, so calls from
    several Python threads, each on its own stream, give the same results as serial calls."""
    import threading
    gen = g(51)
    xs = [torch.randn(512, 1024, generator=gen).to(torch.bfloat16).to(DEV) for _ in range(4)]
    w = torch.ones(1024, dtype=torch.bfloat16, device=DEV)
    want = [core.triton_rmsnorm(x, w, 1e-6) for x in xs]
    torch.cuda.synchronize()
    got = [None] * 4

    def work(i):
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            y = core.triton_fused_up_gate_silu(xs[i], xs[i])          # two different operators per thread
            got[i] = (core.triton_rmsnorm(xs[i], w, 1e-6), y)
        s.synchronize()

    ts = [threading.Thread(target=work, args=(i,)) for i in range(4)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    for i in range(4):
        assert torch.equal(got[i][0], want[i])
        assert_close(got[i][1], E.swiglu_fwd(xs[i].cpu(), xs[i].cpu()), 1e-2)


def test_operators_follow_the_tensor_device_not_the_current_device():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    gen = g(52)
    x = torch.randn(64, 512, generator=gen).to(torch.bfloat16)
    w = torch.ones(512, dtype=torch.bfloat16)
    with torch.cuda.device(0):
        y1 = core.triton_rmsnorm(x.to("cuda:1"), w.to("cuda:1"), 1e-6)      # current device 0, tensors on 1
        lg = torch.randn(8, 32000, generator=gen).to(torch.bfloat16).to("cuda:1").requires_grad_(True)
        loss = triton_entropy_loss(lg, torch.randint(0, 32000, (8,), generator=gen).to("cuda:1"))
        loss.backward()
    assert y1.device.index == 1 and lg.grad.device.index == 1
    assert_close(y1, E.rmsnorm_fwd(x, w, 1e-6)[0], 1e-2)
    assert torch.isfinite(lg.grad).all()
