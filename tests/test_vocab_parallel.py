"""Vocab-parallel cross-entropy (spec: reference triton_kernels/cross_entropy/test_ce.py:110-166, 215-279).

CPU: the exchange protocol (sharding bookkeeping, the single all-gather, autograd wiring) runs as two
`gloo` ranks, with the three kernel-calling hooks of `core/vocab_parallel.py` replaced by the float32
oracle — the product code itself never falls back.  GPU: the real kernels are exercised on one device by
walking the shards of every rank in turn (no collective is needed for that), and on two devices under
NCCL when the machine has them.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import LOSS_TOL, assert_close
from oracle import eager as E


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _case(m=48, v=1504, seed=3, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    lg = (torch.randn(m, v, generator=g) * 3).to(dtype)
    lb = torch.randint(0, v, (m,), generator=g); lb[::7] = -100
    dl = torch.randn(m, generator=g)
    return lg, lb, dl


def _install_oracle_hooks():
    """Stand-ins for the three C-ABI calls, so the distributed logic can run without a GPU."""
    from mdy_triton_b200.core import vocab_parallel as vp

    def local_forward(lg, lb, vocab_start, stats):
        neg, lse = E.ce_rows(lg, lb, vocab_start=vocab_start, split=True)
        stats[0].copy_(lse); stats[1].copy_(neg)

    def combine(gathered, lb):
        return E.vp_combine(gathered, lb)

    def local_backward(dlosses, lg, lb, lse, dlogits, vocab_start):
        dlogits.copy_(E.ce_grad(lg, lb, lse, dlosses, vocab_start=vocab_start).to(dlogits.dtype))
        return dlogits

    vp._local_forward, vp._combine, vp._local_backward = local_forward, combine, local_backward
    from mdy_triton_b200 import _C
    _C.require_cuda = lambda *t: t[0].device  # the hooks above run on CPU tensors


def _gloo_worker(rank, world, port, fail_rank, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        _install_oracle_hooks()
        from mdy_triton_b200.core.vocab_parallel import vocab_parallel_cross_entropy, vocab_parallel_entropy_loss
        lg, lb, dl = _case()
        v = lg.shape[1] // world
        shard = lg[:, rank * v:(rank + 1) * v].contiguous().requires_grad_(True)
        if rank == fail_rank:
            raise RuntimeError("injected host-side failure before the collective")
        losses = vocab_parallel_cross_entropy(shard.view(4, 12, v), lb.view(4, 12), None, False)
        losses.view(-1).backward(dl)
        full_losses, full_lse = E.ce_rows(lg, lb)
        full_grad = E.ce_grad(lg, lb, full_lse, dl)
        ok = (losses.shape == (4, 12)
              and torch.allclose(losses.view(-1), full_losses, atol=1e-5)
              and torch.allclose(shard.grad, full_grad[:, rank * v:(rank + 1) * v], atol=1e-6))
        shard2 = lg[:, rank * v:(rank + 1) * v].contiguous().requires_grad_(True)
        loss = vocab_parallel_entropy_loss(shard2, lb)
        ok = ok and abs(float(loss) - float(E.ce_scalar(lg, lb))) < 1e-5
        # the Megatron-facing adapter (reference triton_kernels/megatron_patchs/cross_entropy_losss.py:139-140):
        # same losses, and the gradient lands in the logits' own storage
        from mdy_triton_b200.core.megatron import vocab_parallel_cross_entropy as megatron_ce
        leaf = lg[:, rank * v:(rank + 1) * v].contiguous().requires_grad_(True)
        work = leaf * 1.0                       # the non-leaf tensor a model would hand to the loss
        m_losses = megatron_ce(work.view(4, 12, v), lb.view(4, 12))
        m_losses.view(-1).backward(dl)
        ok = (ok and torch.allclose(m_losses.view(-1), full_losses, atol=1e-5)
              and torch.allclose(leaf.grad, full_grad[:, rank * v:(rank + 1) * v], atol=1e-6)
              and torch.equal(work.detach(), leaf.grad))   # in place: the logits now hold their gradient
        out[rank] = "ok" if ok else "mismatch"
    except Exception as e:  # noqa: BLE001
        out[rank] = f"error: {type(e).__name__}"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run_gloo(world, fail_rank=-1):
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, fail_rank, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        if p.is_alive():
            p.kill()
    return dict(out)


def test_two_gloo_ranks_match_full_vocab_oracle():
    assert _run_gloo(2) == {0: "ok", 1: "ok"}


def test_four_gloo_ranks_match_full_vocab_oracle():
    assert _run_gloo(4) == {0: "ok", 1: "ok", 2: "ok", 3: "ok"}


def test_rank_failing_before_the_collective_is_reported_not_hung():
    """Host-side failure injection: rank 1 raises before the all-gather; rank 0's collective ends with an
    error within the process-group timeout instead of waiting forever."""
    out = _run_gloo(2, fail_rank=1)
    assert out.get(1, "").startswith("error: RuntimeError")
    assert out.get(0, "missing").startswith("error"), out


@pytest.mark.gpu
@pytest.mark.parametrize("v,tp,sigma,dt", [(32000, 8, 1.0, torch.bfloat16), (128256, 2, 4.0, torch.bfloat16),
                                           (151936, 4, 1.0, torch.bfloat16), (256000, 8, 4.0, torch.bfloat16),
                                           (1500, 4, 1.0, torch.float32)])
def test_kernels_over_all_shards_on_one_gpu(v, tp, sigma, dt):
    """The vocab-parallel sweep (four vocabularies, two logit scales) at reduced token count: every rank's local forward,
    the combine kernel and every rank's local backward, run one after the other on a single device."""
    from mdy_triton_b200.core import vocab_parallel as vp
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(3)
    m = 96
    v = (v // tp) * tp
    lg = (torch.randn(m, v, generator=g) * sigma).to(dt)
    lb = torch.randint(0, v, (m,), generator=g); lb[torch.rand(m, generator=g) < 0.05] = -100
    dl = torch.randn(m, generator=g)
    vs = v // tp
    shards = [lg[:, r * vs:(r + 1) * vs].contiguous().to(dev) for r in range(tp)]
    lbd = lb.to(dev)
    gathered = torch.empty(tp, 2, m, dtype=torch.float32, device=dev)
    for r in range(tp):
        vp._local_forward(shards[r], lbd, r * vs, gathered[r])
    losses, lse = vp._combine(gathered, lbd)
    fl, fs = E.ce_rows(lg, lb)
    assert torch.allclose(losses.cpu(), fl, rtol=LOSS_TOL, atol=LOSS_TOL)
    assert torch.allclose(lse.cpu(), fs, rtol=LOSS_TOL, atol=LOSS_TOL)
    full = E.ce_grad(lg, lb, fs, dl)
    for r in range(tp):
        out = shards[r]  # in place, as the reference's --inplace mode
        vp._local_backward(dl.to(dev), shards[r], lbd, lse, out, r * vs)
        assert_close(out, full[:, r * vs:(r + 1) * vs], 1e-2 if dt != torch.float32 else 1e-4, f"rank {r}")


def _nccl_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from mdy_triton_b200.core.vocab_parallel import vocab_parallel_cross_entropy
        lg, lb, dl = _case(m=512, v=32000, dtype=torch.bfloat16)
        v = lg.shape[1] // world
        shard = lg[:, rank * v:(rank + 1) * v].contiguous().to(dev).requires_grad_(True)
        losses = vocab_parallel_cross_entropy(shard, lb.to(dev), None, False)
        losses.backward(dl.to(dev))
        fl, fs = E.ce_rows(lg, lb)
        full = E.ce_grad(lg, lb, fs, dl)[:, rank * v:(rank + 1) * v]
        g = shard.grad.float().cpu()
        ok = torch.allclose(losses.cpu(), fl, rtol=1e-4, atol=1e-4) and bool(((g - full).abs() <= 1e-2 * (full.abs() + full.abs().mean())).all())
        out[rank] = "ok" if ok else "mismatch"
    except Exception as e:  # noqa: BLE001
        out[rank] = f"error: {type(e).__name__}: {e}"
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_two_nccl_ranks_when_two_gpus_are_present():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_nccl_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        if p.is_alive():
            p.kill()
    assert dict(out) == {0: "ok", 1: "ok"}
