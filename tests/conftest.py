import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"

# Where a reference checkout exists, its kernels are run under Triton's interpreter; the switch has to
# be set before anything imports triton.  Machines without the checkout are left untouched.
from oracle import ref_loader as _ref_loader  # noqa: E402

if _ref_loader.available() and not torch.cuda.is_available():
    os.environ.setdefault("TRITON_INTERPRET", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    return torch.load(GOLDEN / name, weights_only=False)


def golden_cases(name):
    """(id, case) pairs for parametrisation."""
    return [pytest.param(c, id=c["name"]) for c in load_golden(name)]


# Tolerances of the parity contract: outputs/gradients in 16-bit I/O within 1e-2 relative, float32
# I/O within 1e-4 relative, the float32 loss within 1e-4.
REL = {torch.bfloat16: 1e-2, torch.float16: 1e-2, torch.float32: 1e-4}
LOSS_TOL = 1e-4


def assert_close(actual, expected, rel, what="", atol=0.0):
    """|a - b| <= rel * (|b| + mean|b|) + atol elementwise: relative error bounded by `rel`, with an
    absolute floor of `rel` times the tensor's typical magnitude for entries that cancel to ~0.  `atol`
    is for outputs whose storage format underflows (float16 gradients below its subnormal step)."""
    a = actual.detach().float().cpu()
    b = expected.detach().float().cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    assert torch.isfinite(a).all(), f"{what}: non-finite values"
    scale = b.abs().mean()
    err = (a - b).abs()
    tol = rel * (b.abs() + scale) + 1e-30 + atol
    bad = err > tol
    if bad.any():
        i = torch.argmax(err / tol)
        raise AssertionError(f"{what}: {int(bad.sum())}/{a.numel()} elements out of tolerance rel={rel}; worst "
                             f"a={a.flatten()[i].item():.6g} b={b.flatten()[i].item():.6g} scale={scale.item():.3g}")


@pytest.fixture(scope="session")
def cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)


def assert_close_device(actual, expected, rel, what="", rows_per_block=2048):
    """`assert_close` for tensors too large to bring to the host: the same bound
    |a - b| <= rel * (|b| + mean|b|), evaluated on the device block of rows by block of rows."""
    assert actual.shape == expected.shape, f"{what}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}"
    a2 = actual.detach().reshape(-1, actual.shape[-1])
    b2 = expected.detach().reshape(-1, expected.shape[-1])
    n = a2.shape[0]
    total = torch.zeros((), dtype=torch.float64, device=b2.device)
    for i in range(0, n, rows_per_block):
        total += b2[i:i + rows_per_block].float().abs().sum(dtype=torch.float64)
    scale = (total / max(1, b2.numel())).float()
    bad = 0
    worst = 0.0
    for i in range(0, n, rows_per_block):
        a = a2[i:i + rows_per_block].float(); b = b2[i:i + rows_per_block].float()
        assert torch.isfinite(a).all(), f"{what}: non-finite values"
        err = (a - b).abs()
        tol = rel * (b.abs() + scale) + 1e-30
        bad += int((err > tol).sum())
        worst = max(worst, float((err / tol).max()))
    assert bad == 0, f"{what}: {bad}/{a2.numel()} elements out of tolerance rel={rel}; worst error/tolerance {worst:.3g}"
