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
    # a short limit only where a rank is going to fail on purpose (its peers must notice quickly); otherwise a
    # generous one, so that slow process start-up on a loaded machine is not mistaken for a failure
    limit = 8 if fail_rank >= 0 else 120
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=limit))
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
        p.join(240)
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
        # the one-kernel path: records stored straight into the peer's exchange buffer (mapped through CUDA IPC),
        # four calls in a row on the same buffers, each with other logits: a record left over from two calls
        # earlier (same half of the buffers) would give a wrong loss
        from mdy_triton_b200.core.vocab_parallel import PeerExchange, vocab_parallel_entropy_loss
        from mdy_triton_b200 import _C
        ex = PeerExchange(lg.shape[0], v, torch.bfloat16, dev)
        try:
            n = int((lb != -100).sum())
            for call in range(4):
                lgc = (lg.float() * (1.0 + 0.25 * call)).to(torch.bfloat16)
                flc, fsc = E.ce_rows(lgc, lb)
                want = E.ce_grad(lgc, lb, fsc, torch.tensor(1.0 / n))[:, rank * v:(rank + 1) * v]
                leaf = lgc[:, rank * v:(rank + 1) * v].contiguous().to(dev).requires_grad_(True)
                loss = vocab_parallel_entropy_loss(leaf, lb.to(dev), exchange=ex)
                loss.backward()
                torch.cuda.synchronize()
                g2 = leaf.grad.float().cpu()
                ok = (ok and abs(float(loss) - float(flc.sum() / n)) <= 1e-4 * max(1.0, float(flc.sum() / n))
                      and bool(((g2 - want).abs() <= 1e-2 * (want.abs() + want.abs().mean())).all())
                      and _C.lib().mdy_last_device_error(1) == 0)
        finally:
            ex.close()
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


# ------------------------------------------------------------------ the one-kernel path (mdy_ce_vp_fused)
def _fused_all_ranks_one_gpu(lib, shards, outs, labels, inv_n, xbufs, xrows, epoch):
    """All ranks' shards as virtual ranks of ONE launch on one GPU (the form the exchange takes where there
    are fewer GPUs than ranks).  Returns per-rank (losses, lse)."""
    import ctypes
    from mdy_triton_b200 import _C
    tp = len(shards)
    m, vs = shards[0].shape
    dev = shards[0].device
    losses = [torch.full((m,), float("nan"), device=dev) for _ in range(tp)]
    lse = [torch.full((m,), float("nan"), device=dev) for _ in range(tp)]
    arr = lambda ts: (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    rc = lib.mdy_ce_vp_fused(arr(shards), arr(outs), arr(losses), arr(lse), arr(xbufs), labels.data_ptr(), inv_n.data_ptr(),
                             1.0, m, vs, vs, tp, 0, tp, xrows, epoch, _C.dtype_code(shards[0]),
                             torch.cuda.current_stream().cuda_stream)
    return rc, losses, lse


@pytest.mark.gpu
@pytest.mark.parametrize("v,tp,sigma,dt,m", [
    (32000, 8, 1.0, torch.bfloat16, 300),     # 8 KB slices: four small CTAs per SM
    (128256, 8, 4.0, torch.bfloat16, 200),    # 32 KB slices
    (128256, 2, 4.0, torch.bfloat16, 120),    # 128 KB shard rows: four column slices per rank
    (151936, 4, 1.0, torch.bfloat16, 150),
    (256000, 8, 4.0, torch.bfloat16, 100),    # 64 KB shard rows: two slices per rank, 16 participants
    (128256, 1, 3.0, torch.bfloat16, 160),    # one rank: the exchange is between column slices only
    (8192, 4, 1.0, torch.float32, 64),
    (32000, 4, 2.0, torch.float16, 64),
])
def test_one_kernel_exchange_all_ranks_on_one_gpu(v, tp, sigma, dt, m):
    """mdy_ce_vp_fused against the full-vocabulary oracle: losses, lse and every rank's gradient columns, on three
    calls in a row with different logits (the exchange buffers keep earlier calls' records, told apart by the
    epoch; the third call finds the first call's records in its half of the buffers), the second one in place."""
    from mdy_triton_b200 import _C
    lib = _C.lib()
    dev = torch.device("cuda", 0)
    vs = v // tp
    xrows = 512
    nbytes = lib.mdy_ce_vp_exchange_bytes(xrows, vs, tp, _C.DTYPE_CODE[dt])
    assert nbytes > 0
    xbufs = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(tp)]
    rel = 1e-2 if dt != torch.float32 else 1e-4
    atol = 2.0 ** -24 if dt == torch.float16 else 0.0
    for call, inplace in ((1, False), (2, True), (3, False)):
        g = torch.Generator().manual_seed(100 * call + tp)
        lg = (torch.randn(m, v, generator=g) * sigma).to(dt)
        lb = torch.randint(0, v, (m,), generator=g); lb[torch.rand(m, generator=g) < 0.05] = -100
        n = int((lb != -100).sum())
        inv_n = torch.full((1,), 1.0 / n, device=dev)
        shards = [lg[:, r * vs:(r + 1) * vs].contiguous().to(dev) for r in range(tp)]
        outs = shards if inplace else [torch.full_like(s, float("nan")) for s in shards]
        rc, losses, lse = _fused_all_ranks_one_gpu(lib, shards, outs, lb.to(dev), inv_n, xbufs, xrows, call)
        assert rc == 0, _C.status_string(rc)
        torch.cuda.synchronize()
        assert lib.mdy_last_device_error(1) == 0
        fl, fs = E.ce_rows(lg, lb)
        full = E.ce_grad(lg, lb, fs, torch.tensor(1.0 / n))
        for r in range(tp):
            assert torch.allclose(losses[r].cpu(), fl, rtol=LOSS_TOL, atol=LOSS_TOL), f"losses of rank {r}, call {call}"
            assert torch.allclose(lse[r].cpu(), fs, rtol=LOSS_TOL, atol=LOSS_TOL), f"lse of rank {r}, call {call}"
            assert_close(outs[r], full[:, r * vs:(r + 1) * vs], rel, f"gradient of rank {r}, call {call}", atol)


@pytest.mark.gpu
def test_one_kernel_exchange_gives_up_on_a_missing_record_and_poisons_the_loss():
    """Failure detection without a fault: a test hook keeps one participant from publishing row 0 and shortens
    the bound of the poll, so every rank's wait for that record runs out.  The launch returns, the flag reads 2,
    row 0 has NaN loss on every rank while the other rows are right, and the next call is clean."""
    import time
    from mdy_triton_b200 import _C
    lib = _C.lib()
    dev = torch.device("cuda", 0)
    m, v, tp, dt = 64, 32000, 4, torch.bfloat16
    vs = v // tp
    nbytes = lib.mdy_ce_vp_exchange_bytes(m, vs, tp, _C.DTYPE_CODE[dt])
    xbufs = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(tp)]
    g = torch.Generator().manual_seed(5)
    lg = (torch.randn(m, v, generator=g) * 2).to(dt); lb = torch.randint(0, v, (m,), generator=g)
    inv_n = torch.full((1,), 1.0 / m, device=dev)
    shards = [lg[:, r * vs:(r + 1) * vs].contiguous().to(dev) for r in range(tp)]
    fl, fs = E.ce_rows(lg, lb)
    torch.cuda.synchronize()
    assert lib.mdy_last_device_error(1) == 0
    _C.set_tunable(_C.TUNE_CE_WAIT_TEST, 2)      # participant 1 (rank 1, slice 0) stays silent on row 0
    try:
        t0 = time.perf_counter()
        rc, losses, _ = _fused_all_ranks_one_gpu(lib, shards, [torch.empty_like(s) for s in shards], lb.to(dev), inv_n, xbufs, m, 1)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
    finally:
        _C.set_tunable(_C.TUNE_CE_WAIT_TEST, 0)
    assert rc == 0 and elapsed < 2.0
    assert lib.mdy_last_device_error(1) == 2
    for r in range(tp):
        got = losses[r].cpu()
        assert torch.isnan(got[0])
        healthy = ~torch.isnan(got)
        assert healthy.sum() >= m // 2 and torch.allclose(got[healthy], fl[healthy], rtol=LOSS_TOL, atol=LOSS_TOL)
    outs = [torch.empty_like(s) for s in shards]
    rc, losses, lse = _fused_all_ranks_one_gpu(lib, shards, outs, lb.to(dev), inv_n, xbufs, m, 2)
    torch.cuda.synchronize()
    assert rc == 0 and lib.mdy_last_device_error(1) == 0
    full = E.ce_grad(lg, lb, fs, torch.tensor(1.0 / m))
    for r in range(tp):
        assert torch.allclose(losses[r].cpu(), fl, rtol=LOSS_TOL, atol=LOSS_TOL)
        assert_close(outs[r], full[:, r * vs:(r + 1) * vs], 1e-2, f"rank {r} after the expired wait")


@pytest.mark.gpu
def test_peer_exchange_object_and_fused_loss_single_rank():
    """The public path with one rank: PeerExchange set-up (library-allocated buffer, IPC handle) and
    vocab_parallel_entropy_loss(exchange=...) against the one-pass single-GPU loss."""
    from mdy_triton_b200.core import vocab_parallel as vp
    import mdy_triton.core as core
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(8)
    m, v = 256, 128256
    lg = (torch.randn(m, v, generator=g) * 3).to(torch.bfloat16).to(dev); lb = torch.randint(0, v, (m,), generator=g).to(dev)
    lb[::11] = -100
    ex = vp.PeerExchange(m, v, torch.bfloat16, dev)
    try:
        for _ in range(2):
            a = lg.clone().requires_grad_(True); b = lg.clone().requires_grad_(True)
            la = vp.vocab_parallel_entropy_loss(a, lb, exchange=ex); la.backward()
            lb_ = core.triton_entropy_loss(b, lb); lb_.backward()
            assert abs(float(la) - float(lb_)) <= LOSS_TOL * max(1.0, abs(float(lb_)))
            assert_close(a.grad, b.grad, 1e-2, "gradient")
        # the prepared launcher (fixed buffers, nothing but the C call per step), in place, twice
        n = (lb != -100).sum().float()
        inv = (1.0 / n).reshape(1)
        work = lg.clone()
        launch, losses, _ = vp.fused_launcher(work, lb, work, inv, ex)
        for _ in range(2):
            work.copy_(lg)
            launch()
            assert abs(float(losses.sum() / n) - float(lb_)) <= LOSS_TOL * max(1.0, abs(float(lb_)))
            assert_close(work, b.grad, 1e-2, "gradient from the prepared launcher")
        from mdy_triton_b200 import _C
        assert _C.lib().mdy_last_device_error(1) == 0
    finally:
        ex.close()


@pytest.mark.parametrize("v,tp,want", [
    # vocabulary, ranks -> (column slices per shard row, compute threads, vectors per thread and chunk, CTAs per SM)
    (32000, 8, (1, 64, 8, 8)),       # 8 KB rows: small CTAs, eight per SM
    (32000, 4, (1, 128, 8, 4)),
    (128256, 8, (1, 256, 4, 2)),     # 32 KB slices
    (128256, 1, (4, 512, 4, 1)),     # 250 KB rows: four 64 KB slices
    (151936, 8, (2, 256, 5, 3)),     # two 19 KB slices, one chunk of five, three CTAs per SM
    (256000, 8, (2, 256, 4, 2)),
])
def test_one_kernel_launch_shape_by_shard_length(v, tp, want):
    """The launch shape of mdy_ce_vp_fused is host arithmetic (mdy_ce_vp_geometry): pin the shapes the measured
    configurations run with, and the invariants the kernel relies on, without a GPU."""
    import ctypes
    from mdy_triton_b200 import _C
    lib = _C.lib()
    out = (ctypes.c_int32 * 8)()
    assert lib.mdy_ce_vp_geometry(v // tp, tp, _C.MDY_BF16, out) == 0
    nsub, vps, slot_bytes, nslots, lag, nt, vpc, per_sm = list(out)
    assert (nsub, nt, vpc, per_sm) == want
    assert nsub * tp <= 32                                  # participants of a row: one lane of the exchange warp each
    assert nsub * vps * 8 >= v // tp > (nsub - 1) * vps * 8  # the slices cover the shard row, none is empty
    assert slot_bytes % 128 == 0 and slot_bytes >= vps * 16
    assert 3 <= nslots <= 5 and lag == nslots - 2
    assert per_sm * (nslots * slot_bytes + 4096) <= 227 * 1024
    assert lib.mdy_ce_vp_exchange_bytes(16384, v // tp, tp, _C.MDY_BF16) == 2 * 16384 * tp * nsub * 16


def test_one_kernel_launch_shape_rejects_what_the_kernel_rejects():
    import ctypes
    from mdy_triton_b200 import _C
    lib = _C.lib()
    out = (ctypes.c_int32 * 8)()
    # status codes of include/mdy_kernels.h: -1 null pointer, -2 dtype, -3 size, -4 unsupported
    assert lib.mdy_ce_vp_geometry(4001, 8, _C.MDY_BF16, out) == -4    # not whole 16-byte vectors
    assert lib.mdy_ce_vp_geometry(1 << 20, 8, _C.MDY_BF16, out) == -4  # more than 32 participants
    assert lib.mdy_ce_vp_geometry(4000, 0, _C.MDY_BF16, out) == -3
    assert lib.mdy_ce_vp_geometry(4000, 8, 7, out) == -2
    assert lib.mdy_ce_vp_geometry(4000, 8, _C.MDY_BF16, None) == -1
