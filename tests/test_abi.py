"""The C-ABI library loads without a GPU, exports every symbol the header declares, and rejects bad
arguments with error codes before touching the device."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

from mdy_triton_b200 import _C

HEADER = Path(__file__).resolve().parent.parent / "include" / "mdy_kernels.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    out = {}
    for m in re.finditer(r"\b(int|int64_t|const char\*)\s+(mdy_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        args = m.group(3).strip()
        n = 0 if args in ("", "void") else len([a for a in args.split(",") if a.strip()])
        out[m.group(2)] = n
    return out


def test_header_declares_what_python_binds():
    decl = declared_functions()
    assert len(decl) >= 19
    assert set(decl) == set(_C.SIGNATURES), set(decl) ^ set(_C.SIGNATURES)
    for name, n in decl.items():
        assert len(_C.SIGNATURES[name][1]) == n, f"{name}: header has {n} args, binding {len(_C.SIGNATURES[name][1])}"


def test_library_exports_every_declared_symbol():
    handle = ctypes.CDLL(str(_C.LIB_PATH))
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} not exported by {_C.LIB_PATH.name}"


def test_info_entry_points():
    lib = _C.lib()
    assert lib.mdy_version() == 1
    assert lib.mdy_launch_count() >= 0
    assert _C.status_string(0) == "ok"
    assert "NULL" in _C.status_string(-1)
    assert lib.mdy_set_tunable(999, 1) == -5
    assert lib.mdy_set_tunable(_C.TUNE_CE_THREADS, 256) == 0 and lib.mdy_get_tunable(_C.TUNE_CE_THREADS) == 256
    assert lib.mdy_set_tunable(_C.TUNE_CE_THREADS, 0) == 0 and lib.mdy_get_tunable(_C.TUNE_CE_THREADS) == 0
    assert lib.mdy_rmsnorm_bwd_partial_rows(0, 128, _C.MDY_BF16) == 1


def test_argument_rejection_needs_no_device():
    lib = _C.lib()
    one = ctypes.c_void_p(16)  # never dereferenced: every call below is rejected first
    assert lib.mdy_rmsnorm_fwd(None, None, None, None, 4, 8, 8, 8, 1e-6, _C.MDY_BF16, _C.MDY_BF16, None) == -1
    assert lib.mdy_rmsnorm_fwd(one, one, one, one, 4, 0, 8, 8, 1e-6, _C.MDY_BF16, _C.MDY_BF16, None) == -3
    assert lib.mdy_rmsnorm_fwd(one, one, one, one, 4, 8, 4, 8, 1e-6, _C.MDY_BF16, _C.MDY_BF16, None) == -3
    assert lib.mdy_rmsnorm_fwd(one, one, one, one, 4, 8, 8, 8, 1e-6, _C.MDY_BF16, 7, None) == -2
    assert lib.mdy_rmsnorm_fwd(one, one, one, one, 0, 8, 8, 8, 1e-6, 9, _C.MDY_BF16, None) == -2
    assert lib.mdy_add_rmsnorm_fwd(one, one, one, one, one, one, -1, 8, 8, 1e-6, 0, 0, None) == -3
    z = [0] * 12
    assert lib.mdy_rope(one, one, one, one, one, one, 1, 4, 2, 2, 7, 1, *z, 0, 0, None) == -3      # odd D
    assert lib.mdy_rope(one, one, one, one, one, one, 2, 4, 2, 2, 8, 3, *z, 0, 0, None) == -5      # cos batch
    assert lib.mdy_rope(None, None, one, one, one, one, 2, 4, 2, 2, 8, 1, *z, 0, 0, None) == -1
    assert lib.mdy_swiglu_fwd(one, one, one, 4, 8, 8, 8, 4, 0, None) == -3                        # y stride < N
    assert lib.mdy_swiglu_bwd(one, one, one, one, None, 4, 8, 8, 8, 8, 8, 8, 0, None) == -1
    assert lib.mdy_ce_fwd(one, one, one, one, 4, 0, 0, 0, 0, 0, None) == -3
    assert lib.mdy_ce_fwd(one, one, one, one, 4, 16, 8, 0, 0, 0, None) == -3                      # stride < V
    assert lib.mdy_ce_bwd(one, 0, 5, one, one, one, one, 4, 16, 16, 0, 1, 0, None) == -2
    assert lib.mdy_ce_fused(one, one, one, one, one, None, 1.0, 4, 16, 16, 3, None) == -2
    assert lib.mdy_ce_fused(one, None, one, one, one, None, 1.0, 4, 16, 16, 0, None) == -1
    assert lib.mdy_ce_vp_combine(one, one, one, one, 0, 4, None) == -3
    assert lib.mdy_scale_inplace(None, 4, None, 0, None) == -1
    assert lib.mdy_rowwise_extreme(None, one, one, 4, 8, 8, 0, 0, None) == -1
    assert lib.mdy_rowwise_extreme(one, one, one, 4, 0, 8, 0, 0, None) == -3                      # empty rows
    assert lib.mdy_rowwise_extreme(one, one, one, 4, 8, 4, 1, 0, None) == -3                      # stride < N
    assert lib.mdy_rowwise_extreme(one, one, one, 4, 8, 8, 0, 5, None) == -2
    assert lib.mdy_rowwise_extreme(None, None, None, 0, 8, 8, 0, 0, None) == 0
    assert lib.mdy_ce_last_geometry(None, None, None, None) == -5                                 # nothing launched yet
    # zero-sized problems are accepted and do nothing
    assert lib.mdy_swiglu_fwd(None, None, None, 0, 8, 8, 8, 8, 0, None) == 0
    assert lib.mdy_ce_fwd(None, None, None, None, 0, 16, 16, 0, 0, 0, None) == 0


def test_operators_refuse_cpu_tensors():
    """No CPU fallback: the Python operators raise instead of computing on the host."""
    import mdy_triton.core as core
    x = torch.randn(4, 16); w = torch.ones(16)
    with pytest.raises(RuntimeError, match="CUDA"):
        core.triton_rmsnorm(x, w, 1e-6)
    with pytest.raises(RuntimeError, match="CUDA"):
        core.triton_fused_add_norm(x, x, w, 1e-6)
    with pytest.raises(RuntimeError, match="CUDA"):
        core.triton_fused_up_gate_silu(x, x)
    with pytest.raises(RuntimeError, match="CUDA"):
        core.triton_fused_up_gate_silu_no_split(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        core.fused_apply_rope(torch.randn(1, 2, 4, 8), torch.randn(1, 1, 4, 8), torch.randn(1, 4, 8), torch.randn(1, 4, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        core.fast_cross_entropy_loss(torch.randn(2, 3, 10), torch.zeros(2, 3, dtype=torch.long))
    with pytest.raises(RuntimeError, match="CUDA"):
        core.triton_entropy_loss(torch.randn(6, 10, requires_grad=True), torch.zeros(6, dtype=torch.long))
    with pytest.raises(RuntimeError, match="CUDA"):
        core.triton_max(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        core.triton_min(x, axis=0, keepdim=True)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_C, "_lib", None)
    monkeypatch.setattr(_C, "LIB_PATH", tmp_path / "libmdy_kernels.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _C.lib()
