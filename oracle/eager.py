"""Float32 CPU restatement of the fused operators.  Test infrastructure: see ``oracle/__init__.py``.

Every function takes tensors of any float dtype, upcasts to float32 and returns float32, so it states
what the kernels compute before the final rounding to the I/O dtype.  ``hf_*`` functions restate the
HuggingFace eager modules that the patch replaces (transformers 5.5.0 line numbers); the others restate
the arithmetic of the reference's Triton kernels (paths relative to the reference project).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

IGNORE_INDEX = -100


def _f(t):
    return t.detach().to(torch.float32)


# --------------------------------------------------------------------------------------------------
# RMSNorm — mdy_triton/core/rmsnorm.py:9-25 (forward), :31-50 (backward)
# --------------------------------------------------------------------------------------------------
def rmsnorm_fwd(x, w, eps):
    """y = x / sqrt(mean(x^2) + eps) * w; also returns rms per row (rmsnorm.py:20-25)."""
    x, w = _f(x), _f(w)
    rms = torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return (x / rms) * w, rms.squeeze(-1)


def rmsnorm_bwd(dy, x, w, eps):
    """dx = (w*dy - xhat*mean(xhat*w*dy)) / rms ; dw = sum_rows(xhat*dy) (rmsnorm.py:44-50)."""
    dy, x, w = _f(dy), _f(x), _f(w)
    n = x.shape[-1]
    rms = torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    xhat = x / rms
    wdy = w * dy
    dx = (wdy - (xhat / n) * (xhat * wdy).sum(-1, keepdim=True)) / rms
    dw = (xhat * dy).reshape(-1, n).sum(0)
    return dx, dw


def hf_rmsnorm(x, w, eps):
    """LlamaRMSNorm.forward, transformers/models/llama/modeling_llama.py:60-65 — in float32."""
    x, w = _f(x), _f(w)
    var = x.pow(2).mean(-1, keepdim=True)
    return w * (x * torch.rsqrt(var + eps))


# --------------------------------------------------------------------------------------------------
# add + RMSNorm — mdy_triton/core/fused_add_norm.py:6-26 (forward), :29-55 (backward math)
# --------------------------------------------------------------------------------------------------
def add_rmsnorm_fwd(x, res, w, eps):
    """new_res = x + res (float32); y = rmsnorm(new_res) * w (fused_add_norm.py:14-25)."""
    s = _f(x) + _f(res)
    y, rms = rmsnorm_fwd(s, w, eps)
    return y, s, rms


def add_rmsnorm_bwd(dy, dnew_res, new_res, w, eps):
    """d = rmsnorm_bwd(dy; new_res) + dnew_res for BOTH x and residual (fused_add_norm.py:44-54,
    applied to the whole row — the reference launch covers only the first 128 columns)."""
    dx, dw = rmsnorm_bwd(dy, new_res, w, eps)
    if dnew_res is not None:
        dx = dx + _f(dnew_res)
    return dx, dw


# --------------------------------------------------------------------------------------------------
# RoPE — mdy_triton/core/fused_apply_rope.py:8-46 (forward), :50-90 (backward)
# --------------------------------------------------------------------------------------------------
def rotate_half(x):
    """transformers/models/llama/modeling_llama.py:71-75."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def hf_rope(q, k, cos, sin, unsqueeze_dim=1):
    """apply_rotary_pos_emb, transformers/models/llama/modeling_llama.py:79-101 — in float32."""
    q, k, cos, sin = _f(q), _f(k), _f(cos).unsqueeze(unsqueeze_dim), _f(sin).unsqueeze(unsqueeze_dim)
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin


def rope_fwd(q, k, cos, sin):
    """Kernel form with independent halves of cos/sin (fused_apply_rope.py:24-46):
    o1 = x1*cos1 - x2*sin1, o2 = x2*cos2 + x1*sin2.  q,k: [B,H,L,D]; cos,sin: [B or 1, L, D]."""
    def one(x):
        x = _f(x)
        h = x.shape[-1] // 2
        c, s = _f(cos).unsqueeze(1), _f(sin).unsqueeze(1)
        x1, x2 = x[..., :h], x[..., h:]
        return torch.cat((x1 * c[..., :h] - x2 * s[..., :h], x2 * c[..., h:] + x1 * s[..., h:]), -1)
    return one(q), one(k)


def rope_bwd(dq, dk, cos, sin):
    """d1 = g1*cos1 + g2*sin2, d2 = g2*cos2 - g1*sin1 (fused_apply_rope.py:77-90)."""
    def one(g):
        g = _f(g)
        h = g.shape[-1] // 2
        c, s = _f(cos).unsqueeze(1), _f(sin).unsqueeze(1)
        g1, g2 = g[..., :h], g[..., h:]
        return torch.cat((g1 * c[..., :h] + g2 * s[..., h:], g2 * c[..., h:] - g1 * s[..., :h]), -1)
    return one(dq), one(dk)


def rope_cos_sin(positions, dim, theta, dtype=torch.float32):
    """cos/sin tables the way HF builds them (modeling_llama.py:124-135): inv_freq = theta^(-2i/d),
    emb = cat(freqs, freqs).  positions: [B or 1, L] -> cos, sin [B or 1, L, dim]."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    freqs = positions.to(torch.float32)[..., None] * inv_freq
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


# --------------------------------------------------------------------------------------------------
# SwiGLU — mdy_triton/core/fused_silu.py:8-22 (forward), :25-42 (backward)
# --------------------------------------------------------------------------------------------------
def swiglu_fwd(up, gate):
    """y = up * gate * sigmoid(gate) (fused_silu.py:19-21); equals HF LlamaMLP's
    act_fn(gate_proj(x)) * up_proj(x), modeling_llama.py:115-117."""
    up, gate = _f(up), _f(gate)
    return gate * torch.sigmoid(gate) * up


def swiglu_bwd(dy, up, gate):
    """dup = act*dy ; dgate = (s + act*(1-s)) * up * dy (fused_silu.py:36-40)."""
    dy, up, gate = _f(dy), _f(up), _f(gate)
    s = torch.sigmoid(gate)
    act = s * gate
    return act * dy, (s + act * (1 - s)) * (up * dy)


def split_no_split(x, order):
    """up, gate halves of a fused projection (fused_silu.py:112-117)."""
    n = x.shape[-1] // 2
    return (x[..., :n], x[..., n:]) if order == "up-gate" else (x[..., n:], x[..., :n])


# --------------------------------------------------------------------------------------------------
# cross-entropy — mdy_triton/core/cross_entyopy_loss.py:13-42 (forward), :45-80 (backward), :145-149
# --------------------------------------------------------------------------------------------------
def rowwise_extreme(x, take_min=False):
    """Max (or min) over the last axis with the position of its first occurrence: what the reference's
    ``tl.max / tl.min(..., return_indices=True)`` (core/triton_maxmin.py:32, :114) and its chunked
    update with a strict comparison (:50-63, :133-146) produce.  Values keep the input dtype."""
    xf = _f(x)
    vals = xf.min(-1).values if take_min else xf.max(-1).values
    first = (xf == vals.unsqueeze(-1)).to(torch.int8).argmax(-1)
    return vals.to(x.dtype), first


def ce_rows(logits, labels, vocab_start=0, split=False):
    """Per-row (losses, lse) over the local slice [vocab_start, vocab_start+V) (:20-42).
    Ignored rows: 0, 0.  split=True stores -logit[label] on the owning slice, 0 elsewhere."""
    x = _f(logits).reshape(-1, logits.shape[-1])
    lb = labels.reshape(-1).to(torch.int64)
    v = x.shape[-1]
    lse = torch.logsumexp(x, dim=-1)
    loc = lb - vocab_start
    owned = (loc >= 0) & (loc < v) & (lb != IGNORE_INDEX)
    xl = x.gather(1, loc.clamp(0, v - 1)[:, None]).squeeze(1)
    losses = torch.where(owned, (-xl if split else lse - xl), torch.zeros_like(lse))
    valid = lb != IGNORE_INDEX
    return torch.where(valid, losses, torch.zeros_like(losses)), torch.where(valid, lse, torch.zeros_like(lse))


def ce_grad(logits, labels, lse, dlosses, vocab_start=0):
    """dlogits = (exp(x - lse) - onehot) * dloss; zeros for ignored rows (:56-80)."""
    x = _f(logits).reshape(-1, logits.shape[-1])
    lb = labels.reshape(-1).to(torch.int64)
    m, v = x.shape
    p = torch.exp(x - _f(lse).reshape(-1, 1))
    loc = lb - vocab_start
    owned = (loc >= 0) & (loc < v) & (lb != IGNORE_INDEX)
    rows = torch.nonzero(owned).squeeze(1)
    p[rows, loc[rows]] -= 1.0
    g = _f(dlosses).reshape(-1)
    g = g.expand(m) if g.numel() == 1 else g
    d = p * g[:, None]
    d[lb == IGNORE_INDEX] = 0.0
    return d


def ce_scalar(logits, labels, n_items=None):
    """sum(losses) / n_items with n_items = count(label != -100) by default (:145-149)."""
    losses, _ = ce_rows(logits, labels)
    if n_items is None:
        n_items = torch.count_nonzero(labels != IGNORE_INDEX)
    return losses.sum() / n_items


def hf_cross_entropy(logits, labels, n_items=None):
    """HF fixed_cross_entropy on already-shifted labels, transformers/loss/loss_utils.py:28-44:
    F.cross_entropy(float32 logits, ignore_index=-100, reduction='sum') / n_items (or 'mean')."""
    x = _f(logits).reshape(-1, logits.shape[-1])
    lb = labels.reshape(-1)
    if n_items is None:
        return F.cross_entropy(x, lb, ignore_index=IGNORE_INDEX, reduction="mean")
    return F.cross_entropy(x, lb, ignore_index=IGNORE_INDEX, reduction="sum") / n_items


def vp_combine(stats, labels):
    """Vocab-parallel exchange result, triton_kernels/cross_entropy/test_ce.py:134-142:
    stats [tp, 2, M] (local lse, -x_label or 0) -> lse = logsumexp over ranks, loss = lse + sum(-x_label),
    0 for ignored rows."""
    lb = labels.reshape(-1)
    lse = torch.logsumexp(_f(stats[:, 0]), dim=0)
    losses = lse + _f(stats[:, 1]).sum(0)
    valid = lb != IGNORE_INDEX
    z = torch.zeros_like(lse)
    return torch.where(valid, losses, z), torch.where(valid, lse, z)


# --------------------------------------------------------------------------------------------------
# autograd forms (used for the timed CPU baseline and as an independent check of the closed forms)
# --------------------------------------------------------------------------------------------------
def autograd_rmsnorm(x, w, eps, dy):
    x = _f(x).requires_grad_(True); w = _f(w).requires_grad_(True)
    y = hf_rmsnorm_graph(x, w, eps)
    y.backward(_f(dy))
    return y.detach(), x.grad, w.grad


def hf_rmsnorm_graph(x, w, eps):
    var = x.pow(2).mean(-1, keepdim=True)
    return w * (x * torch.rsqrt(var + eps))


def autograd_add_rmsnorm(x, res, w, eps, dy, dnew_res):
    x = _f(x).requires_grad_(True); res = _f(res).requires_grad_(True); w = _f(w).requires_grad_(True)
    s = x + res
    y = hf_rmsnorm_graph(s, w, eps)
    torch.autograd.backward([y, s], [_f(dy), _f(dnew_res)])
    return y.detach(), s.detach(), x.grad, res.grad, w.grad


def autograd_rope(q, k, cos, sin, dq, dk):
    q = _f(q).requires_grad_(True); k = _f(k).requires_grad_(True)
    c, s = _f(cos).unsqueeze(1), _f(sin).unsqueeze(1)
    qe = q * c + rotate_half(q) * s
    ke = k * c + rotate_half(k) * s
    torch.autograd.backward([qe, ke], [_f(dq), _f(dk)])
    return qe.detach(), ke.detach(), q.grad, k.grad


def autograd_swiglu(up, gate, dy):
    up = _f(up).requires_grad_(True); gate = _f(gate).requires_grad_(True)
    y = F.silu(gate) * up
    y.backward(_f(dy))
    return y.detach(), up.grad, gate.grad


def autograd_ce(logits, labels, n_items=None):
    x = _f(logits).requires_grad_(True)
    loss = _ce_graph(x, labels, n_items)
    loss.backward()
    return loss.detach(), x.grad


def _ce_graph(x, labels, n_items):
    x2 = x.reshape(-1, x.shape[-1])
    lb = labels.reshape(-1)
    if n_items is None:
        n_items = torch.count_nonzero(lb != IGNORE_INDEX)
    return F.cross_entropy(x2, lb, ignore_index=IGNORE_INDEX, reduction="sum") / n_items
