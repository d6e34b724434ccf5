"""Run the reference's own Triton kernels: on CPU under Triton's interpreter, on a GPU natively.
Test infrastructure only.

The reference package cannot be imported as a package (its ``core/__init__.py`` imports a name its
loss module no longer defines), so each kernel file is loaded by path from ``oracle/_ref/``, where
``oracle/make_ref.py`` stages unmodified copies of them (git-ignored; they travel with the working tree to
the GPU machine but never enter the history).

On a GPU (CUDA available and ``TRITON_INTERPRET`` not set to 1) the files are loaded exactly as staged
and Triton's JIT compiles the kernels for the device: this is the reference running natively.

Without a GPU a patched copy of each file is written to a temporary directory because Triton's JIT needs a
source file, with only these host-side shims, none of which touches kernel arithmetic:

  * ``TRITON_INTERPRET=1`` (must be set before ``triton`` is first imported in the process);
  * the ``@triton.autotune`` decorators of ``core/rmsnorm.py`` are removed (the autotuner needs a GPU
    driver; under the interpreter ``num_warps`` has no meaning);
  * ``torch.cuda.device`` / ``torch.cuda.get_device_properties`` are replaced for the duration of a
    call (the host code asks for the SM count and enters a device context);
  * Python bools passed as non-constexpr kernel arguments are wrapped in ``int()``.

Where nothing is staged, ``available()`` is False and callers use the golden vectors in
``tests/golden/`` instead.
"""
from __future__ import annotations

import contextlib
import importlib.util
import os
import re
import sys
import tempfile
import types
from pathlib import Path

_CORE = Path(__file__).resolve().parent / "_ref"
_cache: dict[str, types.ModuleType] = {}
_tmpdir = None


def available() -> bool:
    return (_CORE / "rmsnorm.py").exists()


def native() -> bool:
    """True when the kernels run on a GPU through Triton's JIT (no interpreter, no shims)."""
    import torch
    return torch.cuda.is_available() and os.environ.get("TRITON_INTERPRET") != "1"


def _prepare_env():
    if "triton" in sys.modules and os.environ.get("TRITON_INTERPRET") != "1":
        raise RuntimeError("triton was imported before TRITON_INTERPRET=1 was set")
    os.environ["TRITON_INTERPRET"] = "1"


def _patch(name: str, src: str) -> str:
    if name == "rmsnorm":
        src, n = re.subn(r"@triton\.autotune\(\[.*?key=\['BLOCK_N'\]\)\n", "", src, flags=re.S)
        assert n == 2, "expected two autotune decorators in rmsnorm.py"
    if name == "cross_entyopy_loss":
        a = "M, N, split,"
        b = "M, N, ctx.inplace, "
        assert a in src and b in src
        src = src.replace(a, "M, N, int(split),").replace(b, "M, N, int(ctx.inplace), ")
    return src


def load(name: str) -> types.ModuleType:
    """Load the staged ``mdy_triton/core/<name>.py`` of the reference as an independent module."""
    global _tmpdir
    if name in _cache:
        return _cache[name]
    if not available():
        raise FileNotFoundError(f"no staged reference kernels in {_CORE} (run python -m oracle.make_ref)")
    if native():
        path = _CORE / f"{name}.py"
    else:
        _prepare_env()
        if _tmpdir is None:
            _tmpdir = tempfile.TemporaryDirectory(prefix="mdy_ref_")
        path = Path(_tmpdir.name) / f"ref_{name}.py"
        path.write_text(_patch(name, (_CORE / f"{name}.py").read_text()))
    spec = importlib.util.spec_from_file_location(f"ref_{name}", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _cache[name] = mod
    return mod


@contextlib.contextmanager
def cpu_shims(num_sms: int = 4):
    """Let the reference's host code run without a GPU (see module docstring); nothing is touched when the
    kernels run natively."""
    import torch
    if native():
        yield
        return
    old_dev, old_props = torch.cuda.device, torch.cuda.get_device_properties
    torch.cuda.device = lambda *a, **k: contextlib.nullcontext()
    torch.cuda.get_device_properties = lambda *a, **k: types.SimpleNamespace(multi_processor_count=num_sms)
    try:
        yield
    finally:
        torch.cuda.device, torch.cuda.get_device_properties = old_dev, old_props


# ---- thin callers: inputs are CPU tensors (or device tensors when native), outputs are what the
# ---- reference operator returns

def rmsnorm(x, w, eps, dy):
    """-> y, dx, dw of reference ``triton_rmsnorm`` (core/rmsnorm.py:90)."""
    m = load("rmsnorm")
    x = x.detach().clone().requires_grad_(True); w = w.detach().clone().requires_grad_(True)
    with cpu_shims():
        y = m.triton_rmsnorm(x, w, eps)
        y.backward(dy)
    return y.detach(), x.grad, w.grad


def add_rmsnorm(x, res, w, eps, dy, dnew_res):
    """-> y, new_res, dx, dres, dw of reference ``triton_fused_add_norm`` (core/fused_add_norm.py:97).
    Gradients are only meaningful for hidden sizes up to 128 columns."""
    import torch
    m = load("fused_add_norm")
    x = x.detach().clone().requires_grad_(True); res = res.detach().clone().requires_grad_(True)
    w = w.detach().clone().requires_grad_(True)
    with cpu_shims():
        y, nr = m.triton_fused_add_norm(x, res, w, eps)
        torch.autograd.backward([y, nr], [dy, dnew_res])
    return y.detach(), nr.detach(), x.grad, res.grad, w.grad


def rope(q, k, cos, sin, dq, dk):
    """q,k: [B,L,H,D]-contiguous storage viewed as [B,H,L,D].  -> q_out, k_out, dq_in, dk_in of the
    reference ``fused_apply_rope`` (core/fused_apply_rope.py:140); inputs are not modified."""
    import torch
    m = load("fused_apply_rope")
    def fresh(t):
        return t.detach().transpose(1, 2).contiguous().transpose(1, 2)
    q0 = fresh(q).requires_grad_(True); k0 = fresh(k).requires_grad_(True)
    with cpu_shims():
        # the operator works in place, so hand it a differentiable copy
        qe, ke = m.fused_apply_rope(q0 * 1.0, k0 * 1.0, cos.contiguous(), sin.contiguous())
        qe_val, ke_val = qe.detach().clone(), ke.detach().clone()
        torch.autograd.backward([qe, ke], [fresh(dq).clone(), fresh(dk).clone()])
    return qe_val, ke_val, q0.grad, k0.grad


def swiglu(up, gate, dy):
    """-> y, dup, dgate of reference ``triton_fused_up_gate_silu`` (core/fused_silu.py:233)."""
    m = load("fused_silu")
    up = up.detach().clone().requires_grad_(True); gate = gate.detach().clone().requires_grad_(True)
    with cpu_shims():
        y = m.triton_fused_up_gate_silu(up, gate)
        y.backward(dy.contiguous())
    return y.detach(), up.grad, gate.grad


def swiglu_no_split(x, order, dy):
    """-> y, dx of reference ``triton_fused_up_gate_silu_no_split`` (core/fused_silu.py:234)."""
    m = load("fused_silu")
    x = x.detach().clone().requires_grad_(True)
    with cpu_shims():
        y = m.triton_fused_up_gate_silu_no_split(x, order)
        y.backward(dy.contiguous())
    return y.detach(), x.grad


def ce_rows(logits, labels, dlosses, inplace=False):
    """-> losses, dlogits of reference ``_FastCrossEntropyLoss`` (core/cross_entyopy_loss.py:82-142)."""
    m = load("cross_entyopy_loss")
    lg = logits.detach().clone().requires_grad_(True)
    with cpu_shims():
        x = lg * 1.0 if inplace else lg
        losses = m._FastCrossEntropyLoss.apply(x, labels, inplace)
        losses.backward(dlosses)
    return losses.detach(), lg.grad


def ce_scalar(logits, labels, n_items=None):
    """-> loss, dlogits of reference ``triton_entropy_loss`` (core/cross_entyopy_loss.py:145-149)."""
    m = load("cross_entyopy_loss")
    lg = logits.detach().clone().requires_grad_(True)
    with cpu_shims():
        loss = m.triton_entropy_loss(lg, labels, n_items)
        loss.backward()
    return loss.detach(), lg.grad


def extreme(x, take_min=False, axis=-1, keepdim=False):
    """-> values, indices of reference ``triton_max`` / ``triton_min`` (core/triton_maxmin.py:66-97, :149-179)."""
    m = load("triton_maxmin")
    with cpu_shims():
        r = (m.triton_min if take_min else m.triton_max)(x.detach().clone(), axis, keepdim)
    return r.values, r.indices
