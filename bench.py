#!/usr/bin/env python
"""Benchmark of the fused-operator path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c1|c2|c3]
                    [--workload opset|llama1b|llama1b-unpatched|llama1b-fused-residual|vpce|op:NAME] [--no-extras]

One step = forward + backward of the fused operator set at one benchmark config (default c2, the
Llama-3-8B-shaped set: add+RMSNorm [32768,4096], RoPE 32q/8kv heads x 128, SwiGLU [32768,14336],
cross-entropy [32768,128256], bf16) on synthetic seeded inputs.  Every rank owns its own 32768-token
shard (tokens are independent: no data-path collective), so the job is weak-scaled.

Printed JSON (rank 0, one line):
  value      aggregate algorithmic HBM GB/s over all ranks, inputs resident in HBM, kernels launched
             through the C-ABI, timed with CUDA events (max over ranks)
  per_op     the same per operator, with its fraction of the measured HBM peak
  roofline   the dominant kernel (one-pass cross-entropy)
  e2e        the same metric through the public operator API with inputs in pinned HOST memory:
             host->device copies of every step's inputs and the device->host read of the loss are
             inside the timed region
  cpu_baseline  the float32 CPU oracle (HF-eager-equivalent math, autograd) on a bounded token sample
and, unless --no-extras is given, further keys that do not change the headline:
  configs    per-operator tables of the other two operator-set configurations (c1, c3)
  token_parallel_with_allreduce  the same step followed by the all-reduce a token-sharded caller needs
             (the RMSNorm weight gradient [hidden] and the loss sum / token count), N > 1 only
  vpce       the vocab-parallel cross-entropy sweep over the N ranks, collective inside the timed region,
             with an on-device check of every case against the full-vocabulary one-GPU loss
  llama1b_train_step  the patched Llama-1B training step (DDP over the N ranks)
  triton_reference    the reference's own Triton kernels timed by the same CUDA-event harness on the same
             tensors (N = 1 only; outside every timed region of this library's kernels)

`--impl reference` times the CPU oracle only (the reference has no CPU implementation of its own; its
Triton kernels need a GPU and are reported under `triton_reference` of the default arm).
`--workload op:NAME` (NAME in norm, rmsnorm, rope, swiglu, ce, ce2, vp) runs ONE operator forward+backward
a few times and prints its time: the small program profiler captures are taken from.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONFIGS = {
    # name: tokens(B, L), hidden, eps, (QH, KH, D, theta), ffn, vocab, sigma, ignored fraction, seed, norm kind
    "c1": dict(desc="Qwen2-0.5B-shaped op set", B=4, L=1024, hidden=896, eps=1e-6, QH=14, KH=2, D=64, theta=1e6,
               ffn=4864, vocab=151936, sigma=2.0, ignored=0.05, seed=0, norm="rmsnorm"),
    "c2": dict(desc="Llama-3-8B-shaped op set", B=8, L=4096, hidden=4096, eps=1e-5, QH=32, KH=8, D=128, theta=5e5,
               ffn=14336, vocab=128256, sigma=3.0, ignored=0.0, seed=1, norm="add_rmsnorm"),
    "c3": dict(desc="Qwen2-7B-shaped op set", B=16, L=2048, hidden=3584, eps=1e-6, QH=28, KH=4, D=128, theta=1e6,
               ffn=18944, vocab=152064, sigma=2.0, ignored=0.10, seed=2, norm="rmsnorm"),
}
OPS = ("norm", "rope", "swiglu", "cross_entropy")
# (operator, direction, OpSet method): the launches of one step, in order.  The one-pass cross-entropy
# computes loss and gradient in a single kernel.
PHASES = (("norm", "fwd", "norm_fwd"), ("norm", "bwd", "norm_bwd"), ("rope", "fwd", "rope_fwd"), ("rope", "bwd", "rope_bwd"),
          ("swiglu", "fwd", "swiglu_fwd"), ("swiglu", "bwd", "swiglu_bwd"), ("cross_entropy", "fwd+bwd", "cross_entropy"))
FALLBACK_PEAK_GBS = 6650.0
NOMINAL_HBM_GBS = 7700.0   # HGX B200 data-sheet figure, reported beside the measured copy bandwidth
# dram__bytes_read.sum + dram__bytes_write.sum of one one-pass cross-entropy launch, from the ncu capture
# summarised under profiles/ (None until a capture exists): bytes per row of the captured case.
CE_TRAFFIC_BYTES_PER_ROW = 499109


def algorithmic_bytes(cfg, tokens, ignored_frac, s=2):
    """Bytes each operator must move for forward+backward (one read or write per tensor element that the
    math needs): norm 5*M*N*s (RMSNorm) or 8*M*N*s (add+RMSNorm, one shared gradient tensor);
    RoPE 4*T*(QH+KH)*D*s + 4*L*D*s (cos/sin broadcast over batch); SwiGLU 8*M*N*s;
    cross-entropy M*V*s*(2 - f_ignored) + 16*M (labels, losses, lse)."""
    M = tokens
    nb = (8 if cfg["norm"] == "add_rmsnorm" else 5) * M * cfg["hidden"] * s
    rb = 4 * M * (cfg["QH"] + cfg["KH"]) * cfg["D"] * s + 4 * cfg["L"] * cfg["D"] * s
    sb = 8 * M * cfg["ffn"] * s
    cb = M * cfg["vocab"] * s * (2 - ignored_frac) + 16 * M
    return {"norm": nb, "rope": rb, "swiglu": sb, "cross_entropy": cb}


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_PEAK_GBS, "fallback (no MEASURED_PEAKS.json beside bench.py)"


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); pw.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load = those in the upper half of the power range seen
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(pw),
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------- device arm
class OpSet:
    """Device buffers of one config shard plus direct C-ABI launches (no autograd, no allocation in the
    timed loop)."""

    def __init__(self, cfg, dev, seed):
        from mdy_triton_b200 import _C
        self.C, self.lib, self.cfg, self.dev = _C, _C.lib(), cfg, dev
        dt = torch.bfloat16
        g = torch.Generator(dev).manual_seed(seed)
        B, L, H = cfg["B"], cfg["L"], cfg["hidden"]
        M = self.M = B * L

        def rn(*shape, scale=1.0):
            t = torch.randn(*shape, device=dev, generator=g, dtype=dt)
            return t if scale == 1.0 else t.mul_(scale)
        # norm
        self.x = rn(M, H); self.res = rn(M, H); self.w = (1 + 0.02 * torch.randn(H, device=dev, generator=g)).to(dt)
        self.y = torch.empty_like(self.x); self.nres = torch.empty_like(self.x)
        self.rstd = torch.empty(M, dtype=torch.float32, device=dev)
        self.dy = rn(M, H); self.dnres = rn(M, H); self.dx = torch.empty_like(self.x); self.dw = torch.empty_like(self.w)
        rows = self.lib.mdy_rmsnorm_bwd_partial_rows(M, H, _C.MDY_BF16)
        self.partial = torch.empty(rows, H, dtype=torch.float32, device=dev)
        # rope: storage [B, L, H, D]
        QH, KH, D = cfg["QH"], cfg["KH"], cfg["D"]
        self.q = rn(B, L, QH, D); self.k = rn(B, L, KH, D)
        self.dq = rn(B, L, QH, D); self.dk = rn(B, L, KH, D)
        self.dq_out = torch.empty_like(self.q); self.dk_out = torch.empty_like(self.k)
        # cos/sin tables the way HF builds them: inv_freq = theta^(-2i/D), emb = cat(freqs, freqs), [1, L, D]
        inv_freq = 1.0 / (cfg["theta"] ** (torch.arange(0, D, 2, dtype=torch.float32, device=dev) / D))
        freqs = torch.arange(L, dtype=torch.float32, device=dev)[None, :, None] * inv_freq
        emb = torch.cat((freqs, freqs), dim=-1)
        self.cos = emb.cos().to(dt).contiguous(); self.sin = emb.sin().to(dt).contiguous()
        # swiglu
        F = cfg["ffn"]
        self.up = rn(M, F); self.gate = rn(M, F); self.sy = torch.empty_like(self.up)
        self.sdy = rn(M, F); self.dup = torch.empty_like(self.up); self.dgate = torch.empty_like(self.up)
        # cross-entropy
        V = cfg["vocab"]
        self.logits = rn(M, V, scale=cfg["sigma"])
        self.labels = torch.randint(0, V, (M,), device=dev, generator=g)
        if cfg["ignored"] > 0:
            self.labels[torch.rand(M, device=dev, generator=g) < cfg["ignored"]] = -100
        self.ignored_frac = float((self.labels == -100).float().mean())
        self.dlogits = torch.empty_like(self.logits)
        self.losses = torch.empty(M, dtype=torch.float32, device=dev); self.lse = torch.empty(M, dtype=torch.float32, device=dev)
        self.inv_n = (1.0 / torch.count_nonzero(self.labels != -100).float()).reshape(1)
        self.stream = torch.cuda.current_stream(dev).cuda_stream

    def _st(self, t):  # (batch, head, position) strides of a [B, L, H, D] storage viewed as [B, H, L, D]
        return t.stride(0), t.stride(2), t.stride(1)

    def norm_fwd(self):
        C, lib, c, st = self.C, self.lib, self.cfg, self.stream
        M, H, bf = self.M, c["hidden"], C.MDY_BF16
        if c["norm"] == "add_rmsnorm":
            C.check(lib.mdy_add_rmsnorm_fwd(self.x.data_ptr(), self.res.data_ptr(), self.w.data_ptr(), self.y.data_ptr(),
                                            self.nres.data_ptr(), self.rstd.data_ptr(), M, H, H, c["eps"], bf, bf, st), "add_rmsnorm_fwd")
        else:
            C.check(lib.mdy_rmsnorm_fwd(self.x.data_ptr(), self.w.data_ptr(), self.y.data_ptr(), self.rstd.data_ptr(), M, H, H, H,
                                        c["eps"], bf, bf, st), "rmsnorm_fwd")

    def norm_bwd(self):
        C, lib, c, st = self.C, self.lib, self.cfg, self.stream
        M, H, bf = self.M, c["hidden"], C.MDY_BF16
        if c["norm"] == "add_rmsnorm":
            C.check(lib.mdy_add_rmsnorm_bwd(self.dy.data_ptr(), self.dnres.data_ptr(), self.nres.data_ptr(), self.w.data_ptr(),
                                            self.rstd.data_ptr(), self.dx.data_ptr(), self.dw.data_ptr(), self.partial.data_ptr(),
                                            M, H, H, bf, bf, st), "add_rmsnorm_bwd")
        else:
            C.check(lib.mdy_rmsnorm_bwd(self.dy.data_ptr(), self.x.data_ptr(), self.w.data_ptr(), self.rstd.data_ptr(),
                                        self.dx.data_ptr(), self.dw.data_ptr(), self.partial.data_ptr(), M, H, H, H, H, bf, bf, st),
                    "rmsnorm_bwd")

    def rope_fwd(self):
        C, lib, c, st = self.C, self.lib, self.cfg, self.stream
        a = (c["B"], c["L"], c["QH"], c["KH"], c["D"], 1)
        C.check(lib.mdy_rope(self.q.data_ptr(), self.q.data_ptr(), self.k.data_ptr(), self.k.data_ptr(), self.cos.data_ptr(),
                             self.sin.data_ptr(), *a, *self._st(self.q), *self._st(self.q), *self._st(self.k), *self._st(self.k),
                             0, C.MDY_BF16, st), "rope fwd")

    def rope_bwd(self):
        C, lib, c, st = self.C, self.lib, self.cfg, self.stream
        a = (c["B"], c["L"], c["QH"], c["KH"], c["D"], 1)
        C.check(lib.mdy_rope(self.dq.data_ptr(), self.dq_out.data_ptr(), self.dk.data_ptr(), self.dk_out.data_ptr(),
                             self.cos.data_ptr(), self.sin.data_ptr(), *a, *self._st(self.dq), *self._st(self.dq_out),
                             *self._st(self.dk), *self._st(self.dk_out), 1, C.MDY_BF16, st), "rope bwd")

    def swiglu_fwd(self):
        C, lib, c, st = self.C, self.lib, self.cfg, self.stream
        M, F = self.M, c["ffn"]
        C.check(lib.mdy_swiglu_fwd(self.up.data_ptr(), self.gate.data_ptr(), self.sy.data_ptr(), M, F, F, F, F, C.MDY_BF16, st), "swiglu_fwd")

    def swiglu_bwd(self):
        C, lib, c, st = self.C, self.lib, self.cfg, self.stream
        M, F = self.M, c["ffn"]
        C.check(lib.mdy_swiglu_bwd(self.sdy.data_ptr(), self.up.data_ptr(), self.gate.data_ptr(), self.dup.data_ptr(),
                                   self.dgate.data_ptr(), M, F, F, F, F, F, F, C.MDY_BF16, st), "swiglu_bwd")

    def cross_entropy(self):
        C, lib, c, st = self.C, self.lib, self.cfg, self.stream
        C.check(lib.mdy_ce_fused(self.logits.data_ptr(), self.dlogits.data_ptr(), self.labels.data_ptr(), self.losses.data_ptr(),
                                 self.lse.data_ptr(), self.inv_n.data_ptr(), 1.0, self.M, c["vocab"], c["vocab"], C.MDY_BF16, st),
                "ce_fused")

    def step(self, events=None):
        for i, (_, _, method) in enumerate(PHASES):
            getattr(self, method)()
            if events is not None:
                events[i + 1].record()


L2_BYTES = 126 * 1024 * 1024


def needs_l2_flush(cfg):
    """True when an operator's working set could stay in the 126 MB L2 between iterations."""
    M = cfg["B"] * cfg["L"]
    smallest = min(M * cfg["hidden"], M * (cfg["QH"] + cfg["KH"]) * cfg["D"], M * cfg["ffn"]) * 2
    return smallest * 3 < 2 * L2_BYTES


def run_device_arm(ops: OpSet, steps, warmup, barrier, flush):
    """Times `steps` steps.  Without flushing, the step is timed as one region (events around the whole
    loop) and every launch group (operator x direction) by events at its boundaries.  With flushing (small
    configs), a 256 MB buffer is overwritten before every launch group, outside its event pair, and a
    step's time is the sum of the groups' times.  Returns total ms, ms per phase, launches."""
    scratch = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=ops.dev) if flush else None
    for _ in range(warmup):
        ops.step()
    torch.cuda.synchronize()
    barrier()
    l0 = ops.C.launch_count()
    n = len(PHASES)
    if not flush:
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(n + 1)] for _ in range(steps)]
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for s in range(steps):
            ev[s][0].record()
            ops.step(ev[s])
        t1.record()
        torch.cuda.synchronize()
        barrier()
        total_ms = t0.elapsed_time(t1)
        phase_ms = [statistics.mean(ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(steps)) for i in range(n)]
    else:
        ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in PHASES] for _ in range(steps)]
        for s in range(steps):
            for i, (_, _, method) in enumerate(PHASES):
                scratch.fill_(s & 0xff)
                ev[s][i][0].record()
                getattr(ops, method)()
                ev[s][i][1].record()
        torch.cuda.synchronize()
        barrier()
        phase_ms = [statistics.mean(ev[s][i][0].elapsed_time(ev[s][i][1]) for s in range(steps)) for i in range(n)]
        total_ms = sum(phase_ms) * steps
    return total_ms, phase_ms, ops.C.launch_count() - l0


def run_graph_replay(ops: OpSet, launches=32, replays=5):
    """Launch-free kernel time of the small configs: each launch group captured `launches` times back to
    back into a CUDA graph and replayed; microseconds per launch group.  The inputs of these configs fit
    the L2, so this is not an HBM figure: it shows what is left when launch latency is taken away."""
    out = []
    side = torch.cuda.Stream(ops.dev)
    saved = ops.stream
    for _, _, method in PHASES:
        graph = torch.cuda.CUDAGraph()
        side.wait_stream(torch.cuda.current_stream(ops.dev))
        with torch.cuda.stream(side):
            ops.stream = side.cuda_stream
            getattr(ops, method)()  # first call outside the capture
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                ops.stream = torch.cuda.current_stream(ops.dev).cuda_stream
                for _ in range(launches):
                    getattr(ops, method)()
        ops.stream = saved
        torch.cuda.synchronize()
        graph.replay()
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(replays):
            graph.replay()
        t1.record()
        torch.cuda.synchronize()
        out.append(t0.elapsed_time(t1) * 1e3 / (replays * launches))
    return out


# --------------------------------------------------------------------------------------------- e2e arm
def run_e2e_arm(ops: OpSet, steps, warmup, barrier):
    """Public operator API (autograd functions of mdy_triton.core) with the step's inputs in pinned host
    memory: H2D of every input, forward+backward of the four operators, D2H of the loss."""
    import mdy_triton.core as core
    cfg, dev = ops.cfg, ops.dev
    names = ["x", "res", "q", "k", "up", "gate", "logits", "labels"]
    host = {n: torch.empty(getattr(ops, n).shape, dtype=getattr(ops, n).dtype, pin_memory=True).copy_(getattr(ops, n)) for n in names}
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    loss_host = torch.empty(1, dtype=torch.float32, pin_memory=True)
    w = ops.w.clone().requires_grad_(True)
    B, L = cfg["B"], cfg["L"]

    def one_step():
        d = {n: getattr(ops, n) for n in names}
        for n in names:
            d[n].copy_(host[n], non_blocking=True)
        x = d["x"].requires_grad_(True)
        if cfg["norm"] == "add_rmsnorm":
            res = d["res"].requires_grad_(True)
            y, nres = core.triton_fused_add_norm(x, res, w, cfg["eps"])
            torch.autograd.backward([y, nres], [ops.dy, ops.dnres])
        else:
            y = core.triton_rmsnorm(x, w, cfg["eps"])
            y.backward(ops.dy)
        q = d["q"].requires_grad_(True); k = d["k"].requires_grad_(True)
        qe, ke = core.fused_apply_rope(q.transpose(1, 2), k.transpose(1, 2), ops.cos, ops.sin)
        torch.autograd.backward([qe, ke], [ops.dq.transpose(1, 2), ops.dk.transpose(1, 2)])
        up = d["up"].requires_grad_(True); gate = d["gate"].requires_grad_(True)
        sy = core.triton_fused_up_gate_silu(up, gate)
        sy.backward(ops.sdy)
        logits = d["logits"].requires_grad_(True)
        loss = core.triton_entropy_loss(logits.view(B, L, -1), d["labels"].view(B, L))
        loss.backward()
        loss_host.copy_(loss.detach().reshape(1), non_blocking=True)
        for n in ("x", "res", "q", "k", "up", "gate", "logits"):
            d[n].requires_grad_(False); d[n].grad = None
        w.grad = None

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    barrier()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        one_step()
    t1.record()
    torch.cuda.synchronize()
    barrier()
    return t0.elapsed_time(t1) / steps, h2d, 4, float(loss_host[0])


# ----------------------------------------------------------------------------------------- CPU baseline
def cpu_oracle_step(cfg, tokens, seed):
    """Forward+backward of the four operators in float32 on the host (HF-eager-equivalent autograd math
    from oracle/eager.py) for `tokens` tokens of the config.  Returns a closure that runs one step."""
    from oracle import eager as E
    g = torch.Generator().manual_seed(seed)
    L = min(cfg["L"], tokens); B = max(1, tokens // L); M = B * L
    H, F, V, D = cfg["hidden"], cfg["ffn"], cfg["vocab"], cfg["D"]
    x = torch.randn(M, H, generator=g); res = torch.randn(M, H, generator=g); w = 1 + 0.02 * torch.randn(H, generator=g)
    dy = torch.randn(M, H, generator=g); dn = torch.randn(M, H, generator=g)
    q = torch.randn(B, cfg["QH"], L, D, generator=g); k = torch.randn(B, cfg["KH"], L, D, generator=g)
    dq = torch.randn(B, cfg["QH"], L, D, generator=g); dk = torch.randn(B, cfg["KH"], L, D, generator=g)
    cos, sin = E.rope_cos_sin(torch.arange(L)[None], D, cfg["theta"])
    up = torch.randn(M, F, generator=g); gate = torch.randn(M, F, generator=g); sdy = torch.randn(M, F, generator=g)
    logits = torch.randn(M, V, generator=g) * cfg["sigma"]
    labels = torch.randint(0, V, (M,), generator=g)
    if cfg["ignored"] > 0:
        labels[torch.rand(M, generator=g) < cfg["ignored"]] = -100
    ign = float((labels == -100).float().mean())

    def step():
        if cfg["norm"] == "add_rmsnorm":
            E.autograd_add_rmsnorm(x, res, w, cfg["eps"], dy, dn)
        else:
            E.autograd_rmsnorm(x, w, cfg["eps"], dy)
        E.autograd_rope(q, k, cos, sin, dq, dk)
        E.autograd_swiglu(up, gate, sdy)
        return E.autograd_ce(logits, labels)[0]

    return step, M, ign


def run_cpu_baseline(cfg, tokens, steps, warmup, seed):
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    step, M, ign = cpu_oracle_step(cfg, tokens, seed)
    for _ in range(warmup):
        step()
    t = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t) / steps
    nbytes = sum(algorithmic_bytes(cfg, M, ign).values())
    return nbytes / dt / 1e9, dt, M, torch.get_num_threads()


# ------------------------------------------------------------------------------------ Llama-1B train step
def fused_share_of_gpu_time(step_fn, steps=2):
    """After the timed region: run `steps` more steps under torch's kernel profiler and return the part of
    the summed GPU kernel time spent in this library's kernels (their names carry the `mdy::` namespace).
    A share taken under a profiler, reported beside the tokens/s, never used for it."""
    try:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(steps):
                step_fn()
            torch.cuda.synchronize()
        total = ours = 0.0
        by_kernel = {}
        for e in prof.key_averages():
            t = float(getattr(e, "device_time_total", 0.0) or getattr(e, "cuda_time_total", 0.0))
            if t <= 0:
                continue
            total += t
            if "mdy::" in e.key:
                ours += t
                short = e.key.split("mdy::", 1)[1].replace("(anonymous namespace)::", "").replace("<unnamed>::", "")
                short = short.split("<")[0].split("(")[0]
                by_kernel[short] = by_kernel.get(short, 0.0) + t
        if total <= 0:
            return None
        return {"share": ours / total, "by_kernel": {k: v / total for k, v in sorted(by_kernel.items(), key=lambda kv: -kv[1])}}
    except Exception as e:  # noqa: BLE001 - profiling support is optional on the box
        return {"error": f"{type(e).__name__}: {e}"[:200]}


def run_llama1b(dev, dist, world, steps, warmup, patched=True, micro_batch=4, seq=4096, fuse_residual=False,
                ddp_bucket_mb=200, profile_share=False):
    """Training-step workload: random-init Llama-style 1B decoder (16 layers, hidden 2048, 32 q / 8 kv heads,
    head_dim 64, FFN 8192, vocab 128256, eps 1e-5, theta 5e5), bf16 parameters with float32 master weights
    and AdamW state, full forward+backward+optimizer step, synthetic tokens uniform in the vocabulary,
    micro-batch 4 x 4096 per GPU, DDP gradient all-reduce over NCCL when world > 1.  Returns a dict."""
    import torch.nn as nn
    if patched:
        import mdy_triton.replace_kernel  # noqa: F401  (the import is the patch)
        mdy_triton.replace_kernel.set_residual_fusion(fuse_residual)
    from transformers import LlamaConfig, LlamaForCausalLM
    from mdy_triton_b200 import _C
    cfg = LlamaConfig(hidden_size=2048, intermediate_size=8192, num_hidden_layers=16, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=64, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0,
                      max_position_embeddings=seq, tie_word_embeddings=False, attn_implementation="sdpa")
    torch.manual_seed(1234)
    torch.cuda.reset_peak_memory_stats(dev)
    with torch.device(dev):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16)
    model.train()
    model.config.use_cache = False
    net = model
    if dist is not None:
        net = nn.parallel.DistributedDataParallel(model, device_ids=[dev.index], gradient_as_bucket_view=True,
                                                  bucket_cap_mb=ddp_bucket_mb)
    params = [p for p in model.parameters() if p.requires_grad]
    master = [p.detach().float().clone() for p in params]          # float32 master weights
    opt = torch.optim.AdamW(master, lr=1e-4, weight_decay=0.01, fused=True)
    g = torch.Generator(dev).manual_seed(7 + (dist.get_rank() if dist is not None else 0))
    ids = torch.randint(0, cfg.vocab_size, (micro_batch, seq), device=dev, generator=g)

    for m_ in master:
        m_.grad = torch.empty_like(m_)                               # float32 gradients, overwritten every step
    master_grads = [m_.grad for m_ in master]

    def step():
        out = net(input_ids=ids, labels=ids)
        out.loss.backward()
        with torch.no_grad():
            torch._foreach_copy_(master_grads, [p_.grad for p_ in params])   # float32 <- bf16, one multi-tensor launch
        for p_ in params:
            p_.grad = None
        opt.step()
        with torch.no_grad():
            torch._foreach_copy_(params, master)                     # bf16 <- float32 master
        return out.loss.detach()

    for _ in range(warmup):
        loss = step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    l0 = _C.launch_count()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        loss = step()
    t1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = t0.elapsed_time(t1) / steps
    if dist is not None:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    fused_launches = (_C.launch_count() - l0) / steps
    share = None
    if profile_share and (dist is None or dist.get_rank() == 0):
        share = fused_share_of_gpu_time(step)
    if dist is not None:
        dist.barrier()
    n_params = sum(p.numel() for p in params)
    res = {"tokens_per_s": world * micro_batch * seq / (ms * 1e-3), "ms_per_step": ms, "loss": float(loss),
           "params": n_params, "patched": patched, "ddp_bucket_mb": ddp_bucket_mb, "fuse_residual": bool(patched and fuse_residual), "tokens_per_gpu": micro_batch * seq, "steps": steps,
           "fused_kernel_launches_per_step": fused_launches,
           "peak_mem_GB": torch.cuda.max_memory_allocated(dev) / 1e9}
    if share is not None:
        res["fused_ops_share_of_gpu_kernel_time"] = share
    del opt, master, master_grads, net, model
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------ vocab-parallel CE sweep
VPCE_TOKENS = 16384
VPCE_VOCABS = (32000, 128256, 151936, 256000)
VPCE_SIGMAS = (1.0, 4.0)


def _vpce_shard(dev, M, vs, sigma, r):
    g = torch.Generator(dev).manual_seed(3 + r)
    return torch.randn(M, vs, device=dev, dtype=torch.bfloat16, generator=g).mul_(sigma)


def run_vpce(dev, dist, world, rank, steps, warmup, check=True):
    """Vocab-parallel sweep: 16384 tokens, vocab in {32000, 128256, 151936, 256000} sharded over the ranks,
    logits N(0, sigma^2) with sigma in {1, 4}, 5 % of the labels -100, bf16.
    Per step and rank ONE kernel (mdy_ce_vp_fused; gradient into a second buffer, `steps` launches timed back to back): statistics sweep, exchange of the per-row records by
    stores into every rank's exchange buffer (peer memory over NVLink), gradient sweep from the slices still
    in shared memory; the exchange is inside the kernel, hence inside the timed region.  Shapes the kernel
    has no geometry for take the three-step path (mdy_ce_fwd in split mode -> one all_gather of [2, M]
    float32 -> mdy_ce_vp_combine -> mdy_ce_bwd, in place, one step per event pair), the collective again inside the
    timed region; each case
    says which path it took.  With `check`, every case's loss and this rank's gradient columns are compared
    on the device with what the one-pass kernel gives on the full vocabulary (all shards side by side on
    this GPU): 1e-4 on the loss, 1e-2 relative on the gradient."""
    from mdy_triton_b200.core import vocab_parallel as vp
    import mdy_triton.core as core
    M = VPCE_TOKENS
    cases = []
    parity = "ok"
    for V in VPCE_VOCABS:
        for sigma in VPCE_SIGMAS:
            vs = V // world
            shard = _vpce_shard(dev, M, vs, sigma, rank)
            gl = torch.Generator(dev).manual_seed(3)                       # labels identical on every rank
            labels = torch.randint(0, vs * world, (M,), device=dev, generator=gl)
            labels[torch.rand(M, device=dev, generator=gl) < 0.05] = -100
            f_ign = float((labels == -100).float().mean())
            n_valid = (labels != -100).sum()
            dl = torch.full((M,), 1.0 / M, device=dev)
            stats = torch.empty(2, M, dtype=torch.float32, device=dev)
            gathered = torch.empty(world, 2, M, dtype=torch.float32, device=dev)
            work = torch.empty_like(shard)
            inv_m = torch.full((1,), 1.0 / M, device=dev)
            try:
                exchange = vp.PeerExchange(M, vs, torch.bfloat16, dev)
            except ValueError:
                exchange = None

            if exchange is not None:
                # out of place (shard -> work), so that repeated launches see the same logits
                launch, fused_losses, _ = vp.fused_launcher(shard, labels, work, inv_m, exchange)

            def timed():
                vp._local_forward(work, labels, vs * rank, stats)
                if dist is not None:
                    dist.all_gather_into_tensor(gathered.view(-1), stats.view(-1))
                else:
                    gathered[0].copy_(stats)
                losses, lse = vp._combine(gathered, labels)
                vp._local_backward(dl, work, labels, lse, work, vs * rank)
                return losses
            ms = []
            if exchange is not None:
                # `steps` launches back to back between one pair of events, like the timed region of the main
                # workload; the buffers and pointer tables are prepared above, so the host only makes the C calls,
                # and a short device-side delay in front of the first event lets it enqueue them before the GPU
                # gets there: the events then bracket device time, not the host's launch latency on an idle GPU.
                # Shards of 131 MB and more: every launch streams more than the L2 holds.
                for i in range(warmup + 3):
                    torch.cuda.synchronize()
                    if dist is not None:
                        dist.barrier()
                    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                    torch.cuda._sleep(200000 + 20000 * steps)
                    e0.record()
                    for _ in range(steps):
                        launch()
                    e1.record()
                    torch.cuda.synchronize()
                    if i >= warmup:
                        ms.append(e0.elapsed_time(e1) / steps)
                losses = fused_losses
            else:
                for i in range(warmup + steps):
                    work.copy_(shard)                                     # restore the logits outside the timed region
                    torch.cuda.synchronize()
                    if dist is not None:
                        dist.barrier()
                    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                    torch.cuda._sleep(200000)
                    e0.record(); losses = timed(); e1.record()
                    torch.cuda.synchronize()
                    if i >= warmup:
                        ms.append(e0.elapsed_time(e1))
            t = statistics.median(ms)
            if dist is not None:
                tt = torch.tensor([t], dtype=torch.float64, device=dev)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                t = float(tt[0])
            loss = float(losses.sum() / n_valid)
            case = {"vocab": vs * world, "sigma": sigma, "ms": t,
                    "path": "one kernel, records stored into peer memory" if exchange is not None else "sweep, all-gather, sweep"}
            alg = M * vs * 2 * (2 - f_ign) * world
            case.update({"algorithmic_GBps": alg / t / 1e6, "loss": loss})
            del work
            if check:
                # the same logits as ONE [M, V] tensor on this GPU, through the one-pass full-vocabulary kernel
                full = torch.empty(M, vs * world, device=dev, dtype=torch.bfloat16)
                for r in range(world):
                    full[:, r * vs:(r + 1) * vs] = shard if r == rank else _vpce_shard(dev, M, vs, sigma, r)
                full.requires_grad_(True)
                ref = core.triton_entropy_loss(full, labels)
                ref.backward()
                # and this rank's gradient against the matching columns of the full-vocabulary gradient
                work2 = shard.clone()
                check_losses = None
                if dist is not None:
                    # the ranks took different times over the reference above; a kernel waits one to two seconds
                    # for its peers' records before it gives up, so let them enter the launch together
                    torch.cuda.synchronize()
                    dist.barrier()
                if exchange is not None:
                    check_losses, _ = vp.fused_loss_and_grad(work2, labels, work2, (1.0 / n_valid.float()).reshape(1), exchange)
                else:
                    vp._local_forward(work2, labels, vs * rank, stats)
                    if dist is not None:
                        dist.all_gather_into_tensor(gathered.view(-1), stats.view(-1))
                    else:
                        gathered[0].copy_(stats)
                    _, lse = vp._combine(gathered, labels)
                    dn = torch.full((M,), 1.0, device=dev) / n_valid
                    vp._local_backward(dn, work2, labels, lse, work2, vs * rank)
                def check_loss_ok(ref_value):
                    if check_losses is None:
                        return True
                    got = float(check_losses.sum() / n_valid)
                    return abs(got - ref_value) <= 1e-4 * max(1.0, abs(ref_value))
                want = full.grad[:, rank * vs:(rank + 1) * vs].float()
                err = (work2.float() - want).abs()
                tol = 1e-2 * (want.abs() + want.abs().mean())
                grad_ok = bool((err <= tol).all())
                if not grad_ok:   # say on stderr where; the JSON line only says ok or not
                    over = err > tol
                    rows_off = over.any(dim=1).nonzero().flatten()
                    print(f"[vpce check] rank {rank} vocab {V} sigma {sigma}: {int(over.sum())} gradient elements off in "
                          f"{rows_off.numel()} rows (first rows {rows_off[:8].tolist()}), largest error / tolerance "
                          f"{float((err / tol).max()):.3g}", file=sys.stderr, flush=True)
                    del over, rows_off
                del work2, want, err, tol
                ref = float(ref.detach())
                case["full_vocab_loss"] = ref
                loss_ok = abs(loss - ref) <= 1e-4 * max(1.0, abs(ref))
                # [loss off, gradient off, loss of the check's own launch off] on any rank
                check_ok = check_loss_ok(ref)
                if not (loss_ok and check_ok):
                    print(f"[vpce check] rank {rank} vocab {V} sigma {sigma}: loss of the timed launches {loss}, of the check's "
                          f"launch {float(check_losses.sum() / n_valid) if check_losses is not None else None}, expected {ref}",
                          file=sys.stderr, flush=True)
                bad = torch.tensor([0 if loss_ok else 1, 0 if grad_ok else 1, 0 if check_ok else 1], device=dev)
                if dist is not None:
                    dist.all_reduce(bad, op=dist.ReduceOp.MAX)
                bad = [int(b) for b in bad]
                if any(bad):
                    parity = (f"MISMATCH at vocab {V} sigma {sigma} (rank 0: {loss} vs {ref}); on some rank: loss of the timed "
                              f"launches off: {bool(bad[0])}, gradient off: {bool(bad[1])}, loss of the check's launch off: {bool(bad[2])}")
                del full, ref
            cases.append(case)
            if exchange is not None:
                exchange.close()
            del shard
            torch.cuda.empty_cache()
    # a bounded wait that expired on ANY rank (each rank has its own flag)
    flag = torch.tensor([_device_error_flag()], device=dev)
    if dist is not None:
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    run_vpce.device_error_flag = int(flag[0])
    return cases, parity


def _device_error_flag():
    """0 unless a bounded device-side wait expired during the run (mdy_last_device_error)."""
    from mdy_triton_b200 import _C
    return int(_C.lib().mdy_last_device_error(1))


def vpce_summary(cases, parity, world, peak):
    val = statistics.mean(c["algorithmic_GBps"] for c in cases)
    for c in cases:
        c["frac_of_peak_per_gpu"] = c["algorithmic_GBps"] / world / peak
    return {"metric": "vocab_parallel_ce_fwd_bwd_algorithmic_hbm_throughput", "value": val, "unit": "GB/s",
            "scaling": "strong", "tokens": VPCE_TOKENS, "frac_of_peak_per_gpu": val / world / peak,
            "parity": parity, "parity_check": "each case: loss and this rank's gradient columns against the one-pass kernel on "
            "the full vocabulary on one GPU (1e-4 on the loss, 1e-2 relative on the gradient)",
            "workload": "16384 tokens, vocab sharded over the GPUs, per-row statistics exchanged inside the timed region, "
                        "launches timed back to back between one pair of events", "device_error_flag": getattr(run_vpce, "device_error_flag", _device_error_flag()), "cases": cases}


# -------------------------------------------------------------------------------- one operator at a time
def run_single_op(args):
    """`--workload op:NAME`: forward + backward of ONE operator a few times on synthetic bf16 tensors of the
    chosen configuration's shapes (`--tokens` rows, `--vocab` / `--hidden` override the row length) and the
    CUDA-event time per iteration.  A small program for profiler captures and for trying launch-shape knobs
    (`--tune ID=VALUE`, ids in mdy_triton_b200/csrc/tunables.h); with `--flush` a 256 MB buffer is overwritten
    before every launch so inputs smaller than the L2 come from HBM (its time is measured and subtracted)."""
    from mdy_triton_b200 import _C
    op = args.workload[3:]
    for t in args.tune:
        tid, val = t.split("=")
        _C.set_tunable(int(tid), int(val))
    cfg = dict(CONFIGS[args.config])
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _C.lib()
    st = torch.cuda.current_stream().cuda_stream
    bf = _C.MDY_BF16
    g = torch.Generator(dev).manual_seed(1)
    M = args.tokens or 16384
    iters = max(1, args.steps)

    def rn(*shape):
        return torch.randn(*shape, device=dev, dtype=torch.bfloat16, generator=g)

    if op in ("norm", "rmsnorm"):
        N = args.hidden or cfg["hidden"]
        x, res, dy, dn, w = rn(M, N), rn(M, N), rn(M, N), rn(M, N), rn(N)
        y, nres, dx, dw = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x), torch.empty_like(w)
        rstd = torch.empty(M, device=dev)
        part = torch.empty(lib.mdy_rmsnorm_bwd_partial_rows(M, N, bf), N, device=dev)
        if op == "norm":
            phases = [lambda: _C.check(lib.mdy_add_rmsnorm_fwd(x.data_ptr(), res.data_ptr(), w.data_ptr(), y.data_ptr(), nres.data_ptr(),
                                                               rstd.data_ptr(), M, N, N, 1e-5, bf, bf, st), "fwd"),
                      lambda: _C.check(lib.mdy_add_rmsnorm_bwd(dy.data_ptr(), dn.data_ptr(), nres.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                                               dx.data_ptr(), dw.data_ptr(), part.data_ptr(), M, N, N, bf, bf, st), "bwd")]
            nbytes = [4 * M * N * 2, 4 * M * N * 2]
        else:
            phases = [lambda: _C.check(lib.mdy_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), M, N, N, N, 1e-5, bf,
                                                           bf, st), "fwd"),
                      lambda: _C.check(lib.mdy_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                                           dw.data_ptr(), part.data_ptr(), M, N, N, N, N, bf, bf, st), "bwd")]
            nbytes = [2 * M * N * 2, 3 * M * N * 2]
    elif op == "rope":
        L, QH, KH, D = cfg["L"], cfg["QH"], cfg["KH"], cfg["D"]
        B = max(1, M // L)
        q, k, dq, dk = rn(B, L, QH, D), rn(B, L, KH, D), rn(B, L, QH, D), rn(B, L, KH, D)
        dqo, dko = torch.empty_like(q), torch.empty_like(k)
        cos, sin = rn(1, L, D), rn(1, L, D)
        sq = (q.stride(0), q.stride(2), q.stride(1)); sk = (k.stride(0), k.stride(2), k.stride(1))
        phases = [lambda: _C.check(lib.mdy_rope(q.data_ptr(), q.data_ptr(), k.data_ptr(), k.data_ptr(), cos.data_ptr(), sin.data_ptr(), B, L,
                                                QH, KH, D, 1, *sq, *sq, *sk, *sk, 0, bf, st), "fwd"),
                  lambda: _C.check(lib.mdy_rope(dq.data_ptr(), dqo.data_ptr(), dk.data_ptr(), dko.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                                B, L, QH, KH, D, 1, *sq, *sq, *sk, *sk, 1, bf, st), "bwd")]
        nbytes = [2 * B * L * (QH + KH) * D * 2 + 2 * L * D * 2] * 2
    elif op == "swiglu":
        N = args.hidden or cfg["ffn"]
        up, gate, dy = rn(M, N), rn(M, N), rn(M, N)
        y, dup, dgate = torch.empty_like(up), torch.empty_like(up), torch.empty_like(up)
        phases = [lambda: _C.check(lib.mdy_swiglu_fwd(up.data_ptr(), gate.data_ptr(), y.data_ptr(), M, N, N, N, N, bf, st), "fwd"),
                  lambda: _C.check(lib.mdy_swiglu_bwd(dy.data_ptr(), up.data_ptr(), gate.data_ptr(), dup.data_ptr(), dgate.data_ptr(), M, N,
                                                      N, N, N, N, N, bf, st), "bwd")]
        nbytes = [3 * M * N * 2, 5 * M * N * 2]
    elif op == "ce2":
        V = args.vocab or cfg["vocab"]
        lg = rn(M, V).mul_(3)
        lb = torch.randint(0, V, (M,), device=dev, generator=g)
        losses = torch.empty(M, device=dev); lse = torch.empty(M, device=dev); dl = torch.ones(M, device=dev)
        phases = [lambda: _C.check(lib.mdy_ce_fwd(lg.data_ptr(), lb.data_ptr(), losses.data_ptr(), lse.data_ptr(), M, V, V, 0, 0, bf, st), "fwd"),
                  lambda: _C.check(lib.mdy_ce_bwd(dl.data_ptr(), 1, 0, lg.data_ptr(), lg.data_ptr(), lb.data_ptr(), lse.data_ptr(), M, V, V,
                                                  0, 1, bf, st), "bwd")]
        nbytes = [M * V * 2, 2 * M * V * 2]
    elif op == "ce":
        V = args.vocab or cfg["vocab"]
        lg = rn(M, V).mul_(3)
        lb = torch.randint(0, V, (M,), device=dev, generator=g)
        out = torch.empty_like(lg); losses = torch.empty(M, device=dev); lse = torch.empty(M, device=dev)
        inv = torch.tensor([1.0 / M], device=dev)
        phases = [lambda: _C.check(lib.mdy_ce_fused(lg.data_ptr(), out.data_ptr(), lb.data_ptr(), losses.data_ptr(), lse.data_ptr(),
                                                    inv.data_ptr(), 1.0, M, V, V, bf, st), "ce")]
        nbytes = [2 * M * V * 2]
    elif op == "vp":
        # the one-kernel vocab-parallel cross-entropy on ONE rank: `--vocab` is the shard width, so this is the
        # per-GPU work of a sharded vocabulary without the peers (the exchange runs through this GPU's own buffer)
        from mdy_triton_b200.core import vocab_parallel as vp
        V = args.vocab or cfg["vocab"] // 8
        lg = rn(M, V).mul_(3)
        lb = torch.randint(0, V, (M,), device=dev, generator=g)
        inv = torch.tensor([1.0 / M], device=dev)
        exchange = vp.PeerExchange(M, V, torch.bfloat16, dev)
        phases = [lambda: vp.fused_loss_and_grad(lg, lb, lg, inv, exchange)]
        nbytes = [2 * M * V * 2]
    else:
        raise SystemExit(f"unknown operator {op!r}")

    buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if args.flush else None

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            if buf is not None:
                buf.fill_(1)
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e3

    base = timed(lambda: None) if buf is not None else 0.0
    res = {"op": op, "rows": M, "flush": bool(args.flush), "tune": args.tune, "phases": []}
    for fn, nb in zip(phases, nbytes):
        us = timed(fn) - base
        res["phases"].append({"us": round(us, 2), "GBps": round(nb / us / 1e3, 1)})
    res["device_GB"] = round(torch.cuda.memory_allocated(dev) / 1e9, 2)
    print(json.dumps(res))


# -------------------------------------------------------------------------------------------------- main
def compact_table(cfg, dev, seed, steps, warmup, barrier, max_over_ranks, peak, rank, graph_replay=True):
    """Per-operator figures of one more operator-set configuration: ms, algorithmic GB/s, fraction of the
    measured peak, forward and backward apart."""
    ops = OpSet(cfg, dev, seed)
    flush = needs_l2_flush(cfg)
    ab = algorithmic_bytes(cfg, ops.M, ops.ignored_frac)
    total_ms, phase_ms, _ = run_device_arm(ops, steps, warmup, barrier, flush)
    per_op_ms = {n: sum(ms for (op, _, _), ms in zip(PHASES, phase_ms) if op == n) for n in OPS}
    ms_per_step = max_over_ranks(total_ms) / steps
    table = {"workload": cfg["desc"], "tokens_per_gpu": ops.M, "l2_flushed": flush, "ms_per_step": ms_per_step,
             "GB/s_per_gpu": sum(ab.values()) / (ms_per_step * 1e-3) / 1e9,
             "frac_of_peak": sum(ab.values()) / (ms_per_step * 1e-3) / 1e9 / peak, "per_op": {}}
    for n in OPS:
        gbs = ab[n] / (per_op_ms[n] * 1e-3) / 1e9
        table["per_op"][n] = {"ms": per_op_ms[n], "GB/s": gbs, "frac_of_peak": gbs / peak}
    for (op, direction, _), ms in zip(PHASES, phase_ms):
        if direction in ("fwd", "bwd"):
            table["per_op"][op][direction + "_ms"] = ms
    table["per_op"]["norm"]["kind"] = cfg["norm"]
    if flush and graph_replay and rank == 0:
        for (op, direction, _), us in zip(PHASES, run_graph_replay(ops)):
            table["per_op"][op].setdefault("graph_replay_us", {})[direction] = us
    del ops
    torch.cuda.empty_cache()
    return table


def run_with_allreduce(ops, dist, steps, warmup):
    """The token-sharded step followed by what a caller that shards tokens must still exchange: ONE all-reduce
    of a float32 vector holding the RMSNorm weight gradient [hidden], the loss sum and the valid-token count."""
    H = ops.cfg["hidden"]
    packed = torch.zeros(H + 2, dtype=torch.float32, device=ops.dev)

    def step():
        ops.step()
        packed[:H].copy_(ops.dw)
        packed[H] = ops.losses.sum()
        packed[H + 1] = 1.0 / ops.inv_n[0]
        dist.all_reduce(packed)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step()
    t1.record()
    torch.cuda.synchronize()
    dist.barrier()
    return t0.elapsed_time(t1) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="print the headline line only (no configs / vpce / llama1b_train_step / triton_reference keys)")
    ap.add_argument("--cpu-tokens", type=int, default=8192)
    ap.add_argument("--workload", default="opset",
                    help="opset (default): the fused operator set; llama1b: only the Llama-1B training step with the patch; "
                         "llama1b-fused-residual: the same with each layer's closing residual add fused into the next RMSNorm; "
                         "llama1b-unpatched: the same with stock HuggingFace modules; vpce: only the vocab-parallel sweep; "
                         "op:NAME: one operator (norm, rmsnorm, rope, swiglu, ce, ce2, vp)")
    ap.add_argument("--profile-share", action="store_true",
                    help="llama1b workloads: after timing, profile two more steps and report the share of GPU kernel time spent in the fused kernels")
    ap.add_argument("--ddp-bucket-mb", type=int, default=200, help="DDP gradient bucket size for the llama1b workloads")
    ap.add_argument("--tokens", type=int, default=0,
                    help="override the tokens per GPU (a multiple of the config's sequence length); smaller "
                         "cases are for profiler captures, not for reported numbers")
    ap.add_argument("--vocab", type=int, default=0, help="op:ce / op:ce2: row length")
    ap.add_argument("--hidden", type=int, default=0, help="op:norm / op:rmsnorm / op:swiglu: row length")
    ap.add_argument("--tune", action="append", default=[], metavar="ID=VALUE", help="op:NAME: set a launch-shape knob")
    ap.add_argument("--flush", action="store_true", help="op:NAME: flush the L2 before every launch")
    args = ap.parse_args()
    if args.workload.startswith("op:"):
        run_single_op(args)
        return
    if args.workload not in ("opset", "llama1b", "llama1b-fused-residual", "llama1b-unpatched", "vpce"):
        raise SystemExit(f"unknown workload {args.workload!r}")
    cfg = dict(CONFIGS[args.config])
    if args.tokens:
        if args.tokens % cfg["L"]:
            raise SystemExit(f"--tokens must be a multiple of the sequence length {cfg['L']}")
        cfg["B"] = args.tokens // cfg["L"]
    warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    workload = (f"{cfg['desc']} fwd+bwd, bf16, seed {cfg['seed']}, {cfg['B']}x{cfg['L']} tokens per GPU: "
                f"{'add+RMSNorm' if cfg['norm'] == 'add_rmsnorm' else 'RMSNorm'} hidden {cfg['hidden']}; RoPE "
                f"{cfg['QH']}q/{cfg['KH']}kv x {cfg['D']}; SwiGLU {cfg['ffn']}; cross-entropy vocab {cfg['vocab']}")
    flush = needs_l2_flush(cfg)
    config = {"workload": workload, "tokens_per_gpu": cfg["B"] * cfg["L"], "sharding": "tokens, one shard per GPU, no collective",
              "l2": ("L2 flushed: a 256 MB buffer is overwritten before every launch group (outside its timed region), the tensors fit L2"
                     if flush else "every tensor streamed per step is larger than the 126 MB L2 (no flush needed)")}
    metric, unit = "fused_opset_fwd_bwd_algorithmic_hbm_throughput", "GB/s"

    if args.impl == "reference":
        if rank != 0:
            return
        gbs, dt, M, cores = run_cpu_baseline(cfg, args.cpu_tokens, max(1, args.steps), max(0, args.warmup), cfg["seed"])
        sample = f"{M} of {cfg['B'] * cfg['L']} tokens per step, all four ops fwd+bwd, float32 autograd on host"
        print(json.dumps({"impl": "reference", "metric": metric, "value": gbs, "unit": unit, "n_gpus": args.gpus,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
                          "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
                          "cpu_baseline": {"value": gbs, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
                          "e2e": {"value": gbs, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                          "gpu_launches": 0}))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the operators)")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v):
        if dist is None:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    peak, peak_src = measured_peak()
    if args.workload == "vpce":
        cases, parity = run_vpce(dev, dist, world, rank, max(3, min(args.steps, 10)), 3)
        if rank == 0:
            out = vpce_summary(cases, parity, world, peak)
            out.update({"n_gpus": world, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                        "config": {"workload": "vocab-parallel cross-entropy sweep: " + out.pop("workload")}})
            print(json.dumps(out))
        if dist is not None:
            dist.destroy_process_group()
        return
    if args.workload != "opset":
        res = run_llama1b(dev, dist, world, max(1, min(args.steps, 10)), 2, patched=args.workload != "llama1b-unpatched",
                          fuse_residual=args.workload == "llama1b-fused-residual", ddp_bucket_mb=args.ddp_bucket_mb, profile_share=args.profile_share)
        if rank == 0:
            print(json.dumps({"metric": "llama1b_train_tokens_per_s", "value": res["tokens_per_s"], "unit": "tokens/s",
                              "n_gpus": world, "steps": res["steps"], "warmup": 2, "ms_per_step": res["ms_per_step"],
                              "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                              "data": "synthetic", "config": {"workload": "random-init Llama-style 1B decoder, 16 layers, hidden "
                              "2048, 32q/8kv heads, FFN 8192, vocab 128256, micro-batch 4 x 4096 per GPU, AdamW on float32 "
                              "master weights, DDP", "patched": res["patched"]}, "detail": res}))
        if dist is not None:
            dist.destroy_process_group()
        return

    ops = OpSet(cfg, dev, cfg["seed"] + rank)
    n_rows = ops.M
    ab = algorithmic_bytes(cfg, ops.M, ops.ignored_frac)
    step_bytes = sum(ab.values())
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    total_ms, phase_ms, launches = run_device_arm(ops, args.steps, warmup, barrier, flush)
    per_op_ms = {n: sum(ms for (op, _, _), ms in zip(PHASES, phase_ms) if op == n) for n in OPS}
    total_ms = max_over_ranks(total_ms)
    ms_per_step = total_ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    per_op = {n: {"ms": per_op_ms[n], "GB/s": ab[n] / (per_op_ms[n] * 1e-3) / 1e9,
                  "frac_of_peak": ab[n] / (per_op_ms[n] * 1e-3) / 1e9 / peak,
                  "frac_of_nominal": ab[n] / (per_op_ms[n] * 1e-3) / 1e9 / NOMINAL_HBM_GBS, "algorithmic_bytes": ab[n]} for n in OPS}
    for (op, direction, _), ms in zip(PHASES, phase_ms):
        if direction in ("fwd", "bwd"):
            per_op[op][direction + "_ms"] = ms
    if flush and rank == 0:
        for (op, direction, _), us in zip(PHASES, run_graph_replay(ops)):
            per_op[op].setdefault("graph_replay_us", {})[direction] = us

    e2e = None
    if not args.no_e2e:
        e_ms, h2d, d2h, loss = run_e2e_arm(ops, min(args.steps, 5), 1, barrier)
        e_ms = max_over_ranks(e_ms)
        e2e = {"value": world * step_bytes / (e_ms * 1e-3) / 1e9, "unit": unit, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": e_ms, "loss": loss}

    clocks = sampler.stop() if rank == 0 else None  # sampled over both timed regions (device arm and e2e arm)
    extras = {}
    extras_on = not args.no_extras and not args.tokens

    def guarded(name, fn):
        """An extra leg must never cost the headline line: its failure is recorded under its key."""
        try:
            extras[name] = fn()
        except Exception as e:  # noqa: BLE001
            extras[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
            torch.cuda.empty_cache()

    if extras_on and dist is not None:
        def with_allreduce():
            ms = max_over_ranks(run_with_allreduce(ops, dist, min(args.steps, 10), 3))
            return {"ms_per_step": ms, "value": world * step_bytes / (ms * 1e-3) / 1e9, "unit": unit,
                    "without_allreduce_ms_per_step": ms_per_step,
                    "collective": f"one all_reduce(SUM) of {cfg['hidden'] + 2} float32 per step (RMSNorm weight gradient, loss sum, token count)"}
        guarded("token_parallel_with_allreduce", with_allreduce)
    if extras_on and world == 1 and rank == 0:
        def triton_reference():
            from oracle import ref_loader, ref_timing
            if not ref_loader.available():
                return {"unavailable": "the reference's kernel files are not staged (python -m oracle.make_ref)"}
            table = ref_timing.time_reference_ops(ops, iters=5, warmup=2, flush=flush)
            for n, row in table.items():
                ours = per_op["cross_entropy" if n.startswith("cross_entropy") else n]["ms"]
                row["ours_ms"] = ours
                row["speedup"] = row["ms"] / ours
            return {"what": "the reference's Triton kernels (JIT-compiled by the installed Triton for this GPU) through the "
                            "reference's own autograd-function host code, same tensors, CUDA events, median of 5",
                    "per_op": table}
        guarded("triton_reference", triton_reference)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        gbs, dt, M, cores = run_cpu_baseline(cfg, args.cpu_tokens, 2, 1, cfg["seed"])
        cpu = {"value": gbs, "unit": unit, "cores": cores, "kind": "port",
               "sample": f"{M} of {n_rows} tokens, all four ops fwd+bwd, float32 autograd on host, {dt:.2f} s per pass"}

    del ops
    torch.cuda.empty_cache()
    if extras_on:
        def other_configs():
            return {name: compact_table(dict(CONFIGS[name]), dev, CONFIGS[name]["seed"] + rank, 10, 3, barrier, max_over_ranks,
                                        peak, rank) for name in sorted(CONFIGS) if name != args.config}
        guarded("configs", other_configs)

        def vpce():
            cases, parity = run_vpce(dev, dist, world, rank, 5, 3)
            return vpce_summary(cases, parity, world, peak)
        guarded("vpce", vpce)
        guarded("llama1b_train_step", lambda: run_llama1b(dev, dist, world, 5, 2, patched=True, ddp_bucket_mb=args.ddp_bucket_mb))

    if rank == 0:
        ce = per_op["cross_entropy"]
        # the capture is of the V = 128256 bf16 kernel; other vocabularies have no capture
        traffic = CE_TRAFFIC_BYTES_PER_ROW * n_rows if (CE_TRAFFIC_BYTES_PER_ROW and cfg["vocab"] == 128256) else None
        out = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": warmup,
               "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
               "data": "synthetic", "config": config, "frac_of_peak": value / world / peak, "per_op": per_op,
               "roofline": {"kernel": "one-pass cross-entropy (mdy_ce_fused)", "bound": "hbm", "achieved": ce["GB/s"], "peak": peak,
                            "peak_source": peak_src, "unit": "GB/s", "frac": ce["GB/s"] / peak, "traffic": traffic},
               "clocks": clocks, "gpu_launches": launches}
        if e2e is not None:
            out["e2e"] = e2e
        if cpu is not None:
            out["cpu_baseline"] = cpu
        out.update(extras)
        print(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
