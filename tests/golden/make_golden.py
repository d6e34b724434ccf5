"""Generate the golden vectors in this directory from the reference's own kernels.

    TRITON_INTERPRET=1 python tests/golden/make_golden.py [file.pt ...]

Needs the reference's kernel files staged by ``python -m oracle.make_ref``.  Each case stores its
seeded inputs and the outputs / gradients the reference operator produced for them when run on CPU
under Triton's interpreter.  The files are small on purpose; they travel with the repository to
machines that have no reference checkout.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")
HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

import torch  # noqa: E402

from oracle import eager as E  # noqa: E402
from oracle import ref_loader as R  # noqa: E402


def gen(seed):
    return torch.Generator().manual_seed(seed)


def randn(g, *shape, dtype=torch.float32, scale=1.0, shift=0.0):
    return (torch.randn(*shape, generator=g) * scale + shift).to(dtype)


def labels_with_ignored(g, m, v, frac):
    lb = torch.randint(0, v, (m,), generator=g)
    lb[torch.rand(m, generator=g) < frac] = -100
    return lb


def case_rmsnorm():
    out = []
    for name, (m, n, eps, dt, seed) in {
        "qwen2_0p5b_f32": (16, 896, 1e-6, torch.float32, 0),
        "qwen2_7b_bf16": (8, 3584, 1e-6, torch.bfloat16, 2),
        "odd_3585_f32": (4, 3585, 1e-6, torch.float32, 5),
        "llama1b_f16": (8, 2048, 1e-5, torch.float16, 4),
    }.items():
        g = gen(seed)
        x = randn(g, m, n, dtype=dt); w = randn(g, n, dtype=dt, scale=0.02, shift=1.0); dy = randn(g, m, n, dtype=dt)
        y, dx, dw = R.rmsnorm(x, w, eps, dy)
        out.append(dict(name=name, eps=eps, x=x, w=w, dy=dy, y=y, dx=dx, dw=dw))
    return out


def case_add_rmsnorm():
    out = []
    for name, (m, n, eps, dt, seed, grads) in {
        "llama3_8b_bf16_fwd": (8, 4096, 1e-5, torch.bfloat16, 1, False),
        "qwen2_0p5b_f32_fwd": (8, 896, 1e-6, torch.float32, 0, False),
        "n96_f32_fwd_bwd": (12, 96, 1e-6, torch.float32, 6, True),
        "n128_bf16_fwd_bwd": (12, 128, 1e-5, torch.bfloat16, 7, True),
    }.items():
        g = gen(seed)
        x = randn(g, m, n, dtype=dt); r = randn(g, m, n, dtype=dt); w = randn(g, n, dtype=dt, scale=0.02, shift=1.0)
        dy = randn(g, m, n, dtype=dt); dn = randn(g, m, n, dtype=dt)
        y, nr, dx, dr, dw = R.add_rmsnorm(x, r, w, eps, dy, dn)
        c = dict(name=name, eps=eps, x=x, res=r, w=w, dy=dy, dnew_res=dn, y=y, new_res=nr, grads=grads)
        if grads:  # the reference backward is only right up to 128 columns
            c.update(dx=dx, dres=dr, dw=dw)
        out.append(c)
    return out


def case_rope():
    out = []
    for name, (b, l, qh, kh, d, theta, dt, seed, rand_cs) in {
        "qwen2_0p5b_f32": (2, 16, 14, 2, 64, 1e6, torch.float32, 0, False),
        "llama3_8b_bf16": (1, 8, 32, 8, 128, 5e5, torch.bfloat16, 1, False),
        "gqa32to1_d192_f32_randcs": (2, 3, 32, 1, 192, 1e4, torch.float32, 8, True),
        "qwen2_7b_bf16_batchcs": (2, 4, 28, 4, 128, 1e6, torch.bfloat16, 2, True),
    }.items():
        g = gen(seed)
        q = randn(g, b, l, qh, d, dtype=dt).transpose(1, 2); k = randn(g, b, l, kh, d, dtype=dt).transpose(1, 2)
        if rand_cs:
            cos = randn(g, b, l, d, dtype=dt); sin = randn(g, b, l, d, dtype=dt)
        else:
            cos, sin = E.rope_cos_sin(torch.arange(l)[None], d, theta, dt)
        dq = randn(g, b, qh, l, d, dtype=dt); dk = randn(g, b, kh, l, d, dtype=dt)
        qe, ke, gq, gk = R.rope(q, k, cos, sin, dq, dk)
        out.append(dict(name=name, q=q.contiguous(), k=k.contiguous(), cos=cos, sin=sin, dq=dq, dk=dk,
                        q_out=qe.contiguous(), k_out=ke.contiguous(), dq_in=gq.contiguous(), dk_in=gk.contiguous()))
    return out


def case_swiglu():
    out = []
    for name, (m, n, dt, seed) in {
        "qwen2_0p5b_f32": (4, 4864, torch.float32, 0),
        "llama3_8b_bf16": (4, 14336, torch.bfloat16, 1),
        "odd_f16": (3, 1001, torch.float16, 9),
    }.items():
        g = gen(seed)
        up = randn(g, m, n, dtype=dt); gate = randn(g, m, n, dtype=dt); dy = randn(g, m, n, dtype=dt)
        y, du, dg = R.swiglu(up, gate, dy)
        out.append(dict(name=name, kind="split", up=up, gate=gate, dy=dy, y=y, dup=du, dgate=dg))
    for name, (m, n, dt, seed, order) in {
        "nosplit_upgate_f32": (4, 512, torch.float32, 10, "up-gate"),
        "nosplit_gateup_bf16": (4, 8192, torch.bfloat16, 11, "gate-up"),
    }.items():
        g = gen(seed)
        x = randn(g, m, 2 * n, dtype=dt); dy = randn(g, m, n, dtype=dt)
        y, dx = R.swiglu_no_split(x, order, dy)
        out.append(dict(name=name, kind="no_split", order=order, x=x, dy=dy, y=y, dx=dx))
    return out


def case_ce():
    out = []
    for name, (m, v, sigma, frac, dt, seed) in {
        "v5000_f32": (8, 5000, 2.0, 0.25, torch.float32, 0),
        "qwen2_v151936_bf16": (3, 151936, 2.0, 0.25, torch.bfloat16, 0),
        "llama3_v128256_bf16": (2, 128256, 3.0, 0.0, torch.bfloat16, 1),
        "v1501_odd_f16": (6, 1501, 1.0, 0.2, torch.float16, 12),
    }.items():
        g = gen(seed)
        lg = randn(g, m, v, dtype=dt, scale=sigma)
        lb = labels_with_ignored(g, m, v, frac)
        if frac > 0:
            lb[0] = -100; lb[1] = v - 1
        dl = torch.randn(m, generator=g)
        losses, dlg = R.ce_rows(lg, lb, dl)
        loss, dlg_s = R.ce_scalar(lg, lb)
        n_given = float(m + 3)
        loss_n, dlg_n = R.ce_scalar(lg, lb, n_given)
        c = dict(name=name, logits=lg, labels=lb, dlosses=dl, losses=losses, dlogits=dlg, loss=loss,
                 n_items=n_given, loss_n=loss_n)
        if v < 100000:  # keep the large-vocab files small: one gradient tensor is enough there
            c.update(dlogits_scalar=dlg_s, dlogits_n=dlg_n)
        out.append(c)
    return out


def case_maxmin():
    out = []
    for name, (shape, dt, seed, ties) in {
        "short_rows_f32": ((37, 200), torch.float32, 20, False),          # reference's short-row kernel (D <= 256)
        "short_rows_ties_bf16": ((64, 256), torch.bfloat16, 21, True),
        # chunked long-row kernel, ragged second chunk.  Rows stay within two chunks of 2048 columns: beyond
        # that the reference kernel skips columns (its column offsets accumulate, triton_maxmin.py:53,136)
        "long_rows_f32": ((5, 4000), torch.float32, 22, False),
        "long_rows_ties_f16": ((6, 4096), torch.float16, 23, True),
        "three_dims_bf16": ((3, 4, 300), torch.bfloat16, 24, False),
    }.items():
        g = gen(seed)
        x = torch.randint(-9, 9, shape, generator=g).to(dt) if ties else randn(g, *shape, dtype=dt)
        vmax, imax = R.extreme(x, False)
        vmin, imin = R.extreme(x, True)
        out.append(dict(name=name, x=x, max_values=vmax, max_indices=imax, min_values=vmin, min_indices=imin))
    return out


def main():
    if not R.available():
        raise SystemExit("no staged reference kernels: run python -m oracle.make_ref first")
    only = set(sys.argv[1:])  # optional: file names to (re)generate; default all
    for fname, fn in {"rmsnorm.pt": case_rmsnorm, "add_rmsnorm.pt": case_add_rmsnorm, "rope.pt": case_rope,
                      "swiglu.pt": case_swiglu, "cross_entropy.pt": case_ce, "maxmin.pt": case_maxmin}.items():
        if only and fname not in only:
            continue
        cases = fn()
        torch.save(cases, HERE / fname)
        print(fname, [c["name"] for c in cases], f"{(HERE / fname).stat().st_size / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
