"""Pin the CPU oracle: its float32 restatement must reproduce what the reference's own kernels
produced (golden vectors made by tests/golden/make_golden.py), and the reference kernels themselves
when a reference checkout is present."""
import os

import pytest
import torch

from conftest import REL, assert_close, golden_cases, LOSS_TOL
from oracle import eager as E


def _rel(t):
    # golden outputs are rounded to the I/O dtype; the oracle is unrounded float32
    return REL[t.dtype]


@pytest.mark.parametrize("c", golden_cases("rmsnorm.pt"))
def test_rmsnorm(c):
    y, _ = E.rmsnorm_fwd(c["x"], c["w"], c["eps"])
    dx, dw = E.rmsnorm_bwd(c["dy"], c["x"], c["w"], c["eps"])
    assert_close(c["y"], y, _rel(c["x"]), "y")
    assert_close(c["dx"], dx, _rel(c["x"]), "dx")
    assert_close(c["dw"], dw, _rel(c["x"]), "dw")
    # and the HF eager module the operator replaces
    assert_close(E.hf_rmsnorm(c["x"], c["w"], c["eps"]), y, 1e-5, "hf")


@pytest.mark.parametrize("c", golden_cases("add_rmsnorm.pt"))
def test_add_rmsnorm(c):
    y, s, _ = E.add_rmsnorm_fwd(c["x"], c["res"], c["w"], c["eps"])
    assert_close(c["y"], y, _rel(c["x"]), "y")
    assert_close(c["new_res"], s, _rel(c["x"]), "new_res")
    if c["grads"]:
        dx, dw = E.add_rmsnorm_bwd(c["dy"], c["dnew_res"], s, c["w"], c["eps"])
        assert_close(c["dx"], dx, _rel(c["x"]), "dx")
        assert_close(c["dres"], dx, _rel(c["x"]), "dres")
        dw_ref = c["dw"].float()
        if dw_ref.dim() == 2:  # the reference returns the per-program partials; autograd sums them
            dw_ref = dw_ref.sum(0)
        assert_close(dw_ref, dw, _rel(c["x"]), "dw")
    # closed form == autograd of the HF-style graph, any width
    y2, s2, gx, gr, gw = E.autograd_add_rmsnorm(c["x"], c["res"], c["w"], c["eps"], c["dy"], c["dnew_res"])
    dx, dw = E.add_rmsnorm_bwd(c["dy"], c["dnew_res"], s, c["w"], c["eps"])
    assert_close(dx, gx, 1e-4, "dx vs autograd")
    assert_close(dx, gr, 1e-4, "dres vs autograd")
    assert_close(dw, gw, 1e-4, "dw vs autograd")


@pytest.mark.parametrize("c", golden_cases("rope.pt"))
def test_rope(c):
    qe, ke = E.rope_fwd(c["q"], c["k"], c["cos"], c["sin"])
    gq, gk = E.rope_bwd(c["dq"], c["dk"], c["cos"], c["sin"])
    r = _rel(c["q"])
    assert_close(c["q_out"], qe, r, "q"); assert_close(c["k_out"], ke, r, "k")
    assert_close(c["dq_in"], gq, r, "dq"); assert_close(c["dk_in"], gk, r, "dk")
    if "randcs" not in c["name"] and "batchcs" not in c["name"]:
        hq, hk = E.hf_rope(c["q"], c["k"], c["cos"], c["sin"])  # duplicated-halves tables: HF == kernel form
        assert_close(hq, qe, 1e-5, "hf q"); assert_close(hk, ke, 1e-5, "hf k")


@pytest.mark.parametrize("c", golden_cases("swiglu.pt"))
def test_swiglu(c):
    if c["kind"] == "split":
        up, gate = c["up"], c["gate"]
    else:
        up, gate = E.split_no_split(c["x"], c["order"])
    r = _rel(up)
    assert_close(c["y"], E.swiglu_fwd(up, gate), r, "y")
    du, dg = E.swiglu_bwd(c["dy"], up, gate)
    if c["kind"] == "split":
        assert_close(c["dup"], du, r, "dup"); assert_close(c["dgate"], dg, r, "dgate")
    else:
        gu, gg = E.split_no_split(c["dx"], c["order"])
        assert_close(gu, du, r, "dup"); assert_close(gg, dg, r, "dgate")
    y, au, ag = E.autograd_swiglu(up, gate, c["dy"])
    assert_close(du, au, 1e-4, "dup vs autograd"); assert_close(dg, ag, 1e-4, "dgate vs autograd")


@pytest.mark.parametrize("c", golden_cases("cross_entropy.pt"))
def test_cross_entropy(c):
    lg, lb = c["logits"], c["labels"]
    losses, lse = E.ce_rows(lg, lb)
    assert torch.allclose(c["losses"], losses, rtol=LOSS_TOL, atol=LOSS_TOL)
    assert_close(c["dlogits"], E.ce_grad(lg, lb, lse, c["dlosses"]), _rel(lg), "dlogits")
    assert abs(float(c["loss"]) - float(E.ce_scalar(lg, lb))) <= LOSS_TOL * max(1.0, abs(float(c["loss"])))
    assert abs(float(c["loss_n"]) - float(E.ce_scalar(lg, lb, c["n_items"]))) <= LOSS_TOL * max(1.0, abs(float(c["loss_n"])))
    assert abs(float(E.hf_cross_entropy(lg, lb)) - float(c["loss"])) <= LOSS_TOL * max(1.0, abs(float(c["loss"])))
    if "dlogits_scalar" in c:
        n = torch.count_nonzero(lb != -100)
        assert_close(c["dlogits_scalar"], E.ce_grad(lg, lb, lse, torch.tensor(1.0) / n), _rel(lg), "dlogits scalar")
        assert_close(c["dlogits_n"], E.ce_grad(lg, lb, lse, torch.tensor(1.0 / c["n_items"])), _rel(lg), "dlogits n")


def test_vocab_parallel_combine_matches_full_vocab():
    g = torch.Generator().manual_seed(3)
    m, v, tp = 33, 1504, 4
    lg = torch.randn(m, v, generator=g) * 4
    lb = torch.randint(0, v, (m,), generator=g); lb[::7] = -100
    stats = []
    for r in range(tp):
        lo = r * (v // tp)
        neg, lse = E.ce_rows(lg[:, lo:lo + v // tp], lb, vocab_start=lo, split=True)
        stats.append(torch.stack([lse, neg]))
    losses, lse = E.vp_combine(torch.stack(stats), lb)
    full_losses, full_lse = E.ce_rows(lg, lb)
    assert torch.allclose(losses, full_losses, atol=1e-5) and torch.allclose(lse, full_lse, atol=1e-5)


@pytest.mark.parametrize("c", golden_cases("maxmin.pt"))
def test_max_min(c):
    """Bit-exact: values and first-occurrence indices of the reference's max / min kernels."""
    for take_min, key in ((False, "max"), (True, "min")):
        v, i = E.rowwise_extreme(c["x"], take_min)
        assert torch.equal(v, c[key + "_values"]) and torch.equal(i, c[key + "_indices"])


def test_live_reference_when_present():
    """With a reference checkout at hand, run its kernels now (Triton interpreter) instead of trusting
    only the stored vectors."""
    from oracle import ref_loader as R
    if not R.available():
        pytest.skip("no reference checkout on this machine")
    if os.environ.get("TRITON_INTERPRET") != "1":
        import sys
        if "triton" in sys.modules:
            pytest.skip("triton already imported without TRITON_INTERPRET=1")
    g = torch.Generator().manual_seed(21)
    x = torch.randn(5, 320, generator=g); w = torch.randn(320, generator=g); dy = torch.randn(5, 320, generator=g)
    y, dx, dw = R.rmsnorm(x, w, 1e-6, dy)
    dx2, dw2 = E.rmsnorm_bwd(dy, x, w, 1e-6)
    assert_close(y, E.rmsnorm_fwd(x, w, 1e-6)[0], 1e-5); assert_close(dx, dx2, 1e-4); assert_close(dw, dw2, 1e-4)
    lg = torch.randn(5, 3000, generator=g) * 3; lb = torch.randint(0, 3000, (5,), generator=g); lb[0] = -100
    dl = torch.randn(5, generator=g)
    ls, dlg = R.ce_rows(lg, lb, dl)
    ls2, lse2 = E.ce_rows(lg, lb)
    assert torch.allclose(ls, ls2, atol=1e-5)
    assert_close(dlg, E.ce_grad(lg, lb, lse2, dl), 1e-4)
    xi = torch.randint(-5, 5, (7, 700), generator=g).float()
    for take_min in (False, True):
        v, i = R.extreme(xi, take_min)
        v2, i2 = E.rowwise_extreme(xi, take_min)
        assert torch.equal(v, v2) and torch.equal(i, i2)
