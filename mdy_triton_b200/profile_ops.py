"""Run ONE fused operator (forward + backward) a few times on synthetic tensors — the small, single-op
program that profiler captures are taken from (whole-benchmark captures hold tens of GB on the device).

    python -m mdy_triton_b200.profile_ops --op {norm,rmsnorm,rope,swiglu,ce,ce2} [--tokens 16384] [--iters 3]
                                          [--vocab 128256] [--tune ID=VALUE ...]

Shapes are those of the Llama-3-8B-shaped operator set (hidden 4096, 32q/8kv heads x 128, FFN 14336,
vocab 128256) in bf16; `--tokens` rows.  `ce` is the one-pass cross-entropy, `ce2` the two-phase pair
(statistics sweep, then gradient sweep in place) that the per-row API and the vocab-parallel path use;
`--vocab` sets their row length and `--tune` sets launch-shape tunables (ids in include/mdy_kernels.h).
Prints the CUDA-event time per iteration; with `--flush` a 256 MB buffer is overwritten before every
launch so that inputs smaller than the L2 are read from HBM (its time is measured and subtracted).
"""
from __future__ import annotations

import argparse

import torch

from . import _C


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["norm", "rmsnorm", "rope", "swiglu", "ce", "ce2"])
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--tune", action="append", default=[], metavar="ID=VALUE")
    ap.add_argument("--flush", action="store_true")
    a = ap.parse_args()
    for t in a.tune:
        tid, val = t.split("=")
        _C.set_tunable(int(tid), int(val))
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _C.lib()
    st = torch.cuda.current_stream().cuda_stream
    bf = _C.MDY_BF16
    g = torch.Generator(dev).manual_seed(1)
    M = a.tokens

    def rn(*shape):
        return torch.randn(*shape, device=dev, dtype=torch.bfloat16, generator=g)

    if a.op in ("norm", "rmsnorm"):
        N = 4096
        x, res, dy, dn, w = rn(M, N), rn(M, N), rn(M, N), rn(M, N), rn(N)
        y, nres, dx, dw = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x), torch.empty_like(w)
        rstd = torch.empty(M, device=dev)
        part = torch.empty(lib.mdy_rmsnorm_bwd_partial_rows(M, N, bf), N, device=dev)
        if a.op == "norm":
            def run():
                _C.check(lib.mdy_add_rmsnorm_fwd(x.data_ptr(), res.data_ptr(), w.data_ptr(), y.data_ptr(), nres.data_ptr(), rstd.data_ptr(),
                                                 M, N, N, 1e-5, bf, bf, st), "fwd")
                _C.check(lib.mdy_add_rmsnorm_bwd(dy.data_ptr(), dn.data_ptr(), nres.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                                 dw.data_ptr(), part.data_ptr(), M, N, N, bf, bf, st), "bwd")
        else:
            def run():
                _C.check(lib.mdy_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), M, N, N, N, 1e-5, bf, bf, st), "fwd")
                _C.check(lib.mdy_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                                             part.data_ptr(), M, N, N, N, N, bf, bf, st), "bwd")
    elif a.op == "rope":
        L, QH, KH, D = 4096, 32, 8, 128
        B = max(1, M // L)
        q, k, dq, dk = rn(B, L, QH, D), rn(B, L, KH, D), rn(B, L, QH, D), rn(B, L, KH, D)
        dqo, dko = torch.empty_like(q), torch.empty_like(k)
        cos, sin = rn(1, L, D), rn(1, L, D)
        sq = (q.stride(0), q.stride(2), q.stride(1)); sk = (k.stride(0), k.stride(2), k.stride(1))

        def run():
            _C.check(lib.mdy_rope(q.data_ptr(), q.data_ptr(), k.data_ptr(), k.data_ptr(), cos.data_ptr(), sin.data_ptr(), B, L, QH, KH, D, 1,
                                  *sq, *sq, *sk, *sk, 0, bf, st), "fwd")
            _C.check(lib.mdy_rope(dq.data_ptr(), dqo.data_ptr(), dk.data_ptr(), dko.data_ptr(), cos.data_ptr(), sin.data_ptr(), B, L, QH, KH, D,
                                  1, *sq, *sq, *sk, *sk, 1, bf, st), "bwd")
    elif a.op == "swiglu":
        N = 14336
        up, gate, dy = rn(M, N), rn(M, N), rn(M, N)
        y, dup, dgate = torch.empty_like(up), torch.empty_like(up), torch.empty_like(up)

        def run():
            _C.check(lib.mdy_swiglu_fwd(up.data_ptr(), gate.data_ptr(), y.data_ptr(), M, N, N, N, N, bf, st), "fwd")
            _C.check(lib.mdy_swiglu_bwd(dy.data_ptr(), up.data_ptr(), gate.data_ptr(), dup.data_ptr(), dgate.data_ptr(), M, N, N, N, N, N, N,
                                        bf, st), "bwd")
    elif a.op == "ce2":
        V = a.vocab
        lg = rn(M, V).mul_(3)
        lb = torch.randint(0, V, (M,), device=dev, generator=g)
        losses = torch.empty(M, device=dev); lse = torch.empty(M, device=dev); dl = torch.ones(M, device=dev)
        phases = [lambda: _C.check(lib.mdy_ce_fwd(lg.data_ptr(), lb.data_ptr(), losses.data_ptr(), lse.data_ptr(), M, V, V, 0, 0, bf, st), "fwd"),
                  lambda: _C.check(lib.mdy_ce_bwd(dl.data_ptr(), 1, 0, lg.data_ptr(), lg.data_ptr(), lb.data_ptr(), lse.data_ptr(), M, V, V,
                                                  0, 1, bf, st), "bwd")]

        def run():
            for ph in phases:
                ph()
    else:
        V = a.vocab
        lg = rn(M, V).mul_(3)
        lb = torch.randint(0, V, (M,), device=dev, generator=g)
        out = torch.empty_like(lg); losses = torch.empty(M, device=dev); lse = torch.empty(M, device=dev)
        inv = torch.tensor([1.0 / M], device=dev)

        def run():
            _C.check(lib.mdy_ce_fused(lg.data_ptr(), out.data_ptr(), lb.data_ptr(), losses.data_ptr(), lse.data_ptr(), inv.data_ptr(), 1.0,
                                      M, V, V, bf, st), "ce")

    def timed(fn, flush_buf=None):
        fn()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            if flush_buf is not None:
                flush_buf.fill_(1)
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / a.iters * 1e3

    if a.flush and a.op == "ce2":
        buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        base = timed(lambda: None, buf)
        fwd_us, bwd_us = timed(phases[0], buf) - base, timed(phases[1], buf) - base
        nb = M * a.vocab * 2
        print(f"ce2 V={a.vocab} (L2 flushed): statistics sweep {fwd_us:.1f} us {nb / fwd_us / 1e3:.0f} GB/s, "
              f"gradient sweep {bwd_us:.1f} us {2 * nb / bwd_us / 1e3:.0f} GB/s, {M} rows")
        return
    us = timed(run)
    print(f"{a.op}: {us:.1f} us per forward+backward, {M} rows, "
          f"{torch.cuda.memory_allocated(dev) / 1e9:.2f} GB on the device")


if __name__ == "__main__":
    main()
