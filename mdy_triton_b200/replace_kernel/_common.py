"""Shared pieces of the per-model patch modules.

The reference writes one copy of each patched ``forward`` per model file
(``mdy_triton/replace_kernel/llama.py:12-190``, ``qwen2.py:14-204``, ...), against transformers
4.45-4.47.  The functions here are built against the signatures of the installed transformers
(5.x: ``past_key_values``, ``logits_to_keep``, decoder layers return a tensor, attention returns two
values); the older tuple-returning layer protocol is kept for installs that still use it.
"""
from __future__ import annotations

import inspect
import os

import torch
import torch.nn.functional as F
from transformers.modeling_outputs import CausalLMOutputWithPast

from ..core.cross_entyopy_loss import fast_cross_entropy_loss
from ..core.fused_add_norm import triton_fused_add_norm
from ..core.fused_apply_rope import fused_apply_rope
from ..core.fused_silu import triton_fused_up_gate_silu, triton_fused_up_gate_silu_no_split
from ..core.rmsnorm import triton_rmsnorm
from ._deferred import DeferredResidual

try:  # transformers >= 4.50
    from transformers.utils import can_return_tuple
except ImportError:  # pragma: no cover
    def can_return_tuple(fn):
        return fn


_fuse_residual = os.environ.get("MDY_FUSE_RESIDUAL", "0") == "1"


def set_residual_fusion(enabled: bool) -> None:
    """Switch the fusion of each layer's closing residual add into the next RMSNorm on or off (default off,
    or the environment variable ``MDY_FUSE_RESIDUAL=1``).  With it on, a patched decoder layer returns a
    :class:`DeferredResidual`; results are unchanged.  It is bypassed under gradient checkpointing and for
    model families whose reference patch keeps add and norm separate (Mistral).  Leave it off with wrappers
    that register hooks on layer outputs (FSDP): a hook would see the materialised sum, not the graph."""
    global _fuse_residual
    _fuse_residual = bool(enabled)


def residual_fusion_enabled() -> bool:
    return _fuse_residual


def _eps_of(norm):
    eps = getattr(norm, "variance_epsilon", None)
    return norm.eps if eps is None else eps


def rmsnorm_forward(self, hidden_state):
    """``<Model>RMSNorm.forward`` (reference llama.py:12-13).  A deferred layer output is added and
    normalised in one kernel."""
    if type(hidden_state) is DeferredResidual:
        branch, residual = hidden_state.parts()
        return triton_fused_add_norm(branch, residual, self.weight, _eps_of(self))[0]
    return triton_rmsnorm(hidden_state, self.weight, _eps_of(self))


def mlp_forward(self, hidden_state):
    """``<Model>MLP.forward`` with separate up/gate projections (reference llama.py:15-17)."""
    return self.down_proj(triton_fused_up_gate_silu(self.up_proj(hidden_state), self.gate_proj(hidden_state)))


def mlp_forward_fused_proj(self, hidden_states):
    """``Phi3MLP.forward``: one ``gate_up_proj`` whose output is ``[gate | up]``
    (transformers phi3 ``gate, up = x.chunk(2, -1)``); reference phi3.py:16-18."""
    return self.down_proj(triton_fused_up_gate_silu_no_split(self.gate_up_proj(hidden_states), "gate-up"))


def _identity(x):
    return x


def make_decoder_layer_forward(original_forward, fuse_add_norm: bool = True):
    """Build a ``<Model>DecoderLayer.forward`` with the post-attention residual add fused into the
    post-attention RMSNorm (reference llama.py:19-84).  ``fuse_add_norm=False`` keeps the two steps
    separate, as the reference does for Mistral (mistral.py:66-72)."""
    params = inspect.signature(original_forward).parameters
    legacy = "past_key_value" in params  # transformers < 4.56 layer protocol: tuple in, tuple out

    def post_attention(self, attn_out, residual):
        drop = getattr(self, "resid_attn_dropout", _identity)
        ln = self.post_attention_layernorm
        if fuse_add_norm:
            return triton_fused_add_norm(drop(attn_out), residual, ln.weight, _eps_of(ln))
        residual = residual + drop(attn_out)
        return ln(residual), residual

    if not legacy:
        def decoder_layer_forward(self, hidden_states, attention_mask=None, position_ids=None,
                                  past_key_values=None, use_cache=False, position_embeddings=None,
                                  **kwargs):
            if type(hidden_states) is DeferredResidual:
                # the previous layer left its closing add to this layer's input norm (one kernel for both)
                branch, residual = hidden_states.parts()
                ln = self.input_layernorm
                hidden_states, residual = triton_fused_add_norm(branch, residual, ln.weight, _eps_of(ln))
            else:
                residual = hidden_states
                hidden_states = self.input_layernorm(hidden_states)
            hidden_states, _ = self.self_attn(
                hidden_states=hidden_states, attention_mask=attention_mask, position_ids=position_ids,
                past_key_values=past_key_values, use_cache=use_cache,
                position_embeddings=position_embeddings, **kwargs)
            hidden_states, residual = post_attention(self, hidden_states, residual)
            hidden_states = getattr(self, "resid_mlp_dropout", _identity)(self.mlp(hidden_states))
            if (_fuse_residual and fuse_add_norm
                    and not (self.training and getattr(self, "gradient_checkpointing", False))):
                return DeferredResidual.wrap(hidden_states, residual)
            return residual + hidden_states
    else:  # pragma: no cover - exercised only with an old transformers install
        def decoder_layer_forward(self, hidden_states, attention_mask=None, position_ids=None,
                                  past_key_value=None, output_attentions=False, use_cache=False,
                                  cache_position=None, position_embeddings=None, **kwargs):
            residual = hidden_states
            hidden_states = self.input_layernorm(hidden_states)
            attn_kwargs = dict(hidden_states=hidden_states, attention_mask=attention_mask,
                               position_ids=position_ids, past_key_value=past_key_value,
                               output_attentions=output_attentions, use_cache=use_cache,
                               cache_position=cache_position)
            if position_embeddings is not None or "position_embeddings" in params:
                attn_kwargs["position_embeddings"] = position_embeddings
            hidden_states, self_attn_weights, present_key_value = self.self_attn(**attn_kwargs)
            hidden_states, residual = post_attention(self, hidden_states, residual)
            hidden_states = self.mlp(hidden_states)
            hidden_states = residual + getattr(self, "resid_mlp_dropout", _identity)(hidden_states)
            outputs = (hidden_states,)
            if output_attentions:
                outputs += (self_attn_weights,)
            if use_cache:
                outputs += (present_key_value,)
            return outputs

    decoder_layer_forward.__doc__ = make_decoder_layer_forward.__doc__
    return decoder_layer_forward


def shifted_labels(labels):
    """labels[..., 1:] followed by one -100 per sequence, so logits need no slicing
    (reference llama.py:165-170, which caches a [-100] column instead of padding)."""
    return F.pad(labels[..., 1:], (0, 1), value=-100)


def make_causal_forward(original_forward, output_cls=CausalLMOutputWithPast, extra_fields=()):
    """Build ``<Model>ForCausalLM.forward``: the stock forward with the loss replaced by the fused
    cross-entropy (reference llama.py:92-184).  ``output_cls`` / ``extra_fields`` let a model family
    return its own output type (Qwen2-VL adds ``rope_deltas``)."""
    params = inspect.signature(original_forward).parameters
    keep_name = "logits_to_keep" if "logits_to_keep" in params else "num_logits_to_keep"

    def _forward(self, input_ids, attention_mask, position_ids, past_key_values, inputs_embeds, labels, use_cache,
                 keep, kwargs):
        if keep is None:
            keep = 0
        n_items = kwargs.pop("num_items_in_batch", None) or kwargs.pop("n_items", None)
        shift = kwargs.pop("shift_labels", None)
        outputs = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                             past_key_values=past_key_values, inputs_embeds=inputs_embeds,
                             use_cache=use_cache, **kwargs)
        hidden_states = outputs[0] if isinstance(outputs, tuple) else outputs.last_hidden_state
        slice_indices = slice(-keep, None) if isinstance(keep, int) else keep
        logits = self.lm_head(hidden_states[:, slice_indices, :])

        loss = None
        if labels is not None or shift is not None:
            if shift is None:
                shift = shifted_labels(labels)
            loss = fast_cross_entropy_loss(logits, shift.to(logits.device), n_items=n_items)

        if isinstance(outputs, tuple):  # legacy return_dict=False path
            output = (logits,) + outputs[1:]
            return (loss,) + output if loss is not None else output
        extra = {f: getattr(outputs, f, None) for f in extra_fields}
        return output_cls(loss=loss, logits=logits,
                          past_key_values=getattr(outputs, "past_key_values", None),
                          hidden_states=getattr(outputs, "hidden_states", None),
                          attentions=getattr(outputs, "attentions", None), **extra)

    # The keep-last-logits argument is an explicit parameter under the installed transformers' name:
    # `generate` inspects the signature to decide whether it may ask for the last position only.
    if keep_name == "logits_to_keep":
        def causal_forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None,
                           inputs_embeds=None, labels=None, use_cache=None, logits_to_keep=0, **kwargs):
            return _forward(self, input_ids, attention_mask, position_ids, past_key_values, inputs_embeds, labels,
                            use_cache, logits_to_keep, kwargs)
    else:  # pragma: no cover - older transformers
        def causal_forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None,
                           inputs_embeds=None, labels=None, use_cache=None, num_logits_to_keep=0, **kwargs):
            return _forward(self, input_ids, attention_mask, position_ids, past_key_values, inputs_embeds, labels,
                            use_cache, num_logits_to_keep, kwargs)

    causal_forward.__doc__ = make_causal_forward.__doc__
    return can_return_tuple(causal_forward)


def patch_family(module, prefix, *, mlp=mlp_forward, rope=True, fuse_add_norm=True,
                 decoder_cls=None, causal_cls=None, norm_cls=None, mlp_cls=None, output_cls=CausalLMOutputWithPast,
                 extra_fields=()):
    """Assign the five patched attributes on a ``transformers.models.<m>.modeling_<m>`` module
    (reference llama.py:186-190).  Idempotent."""
    if getattr(module, "_mdy_patched", False):
        return
    if rope:
        module.apply_rotary_pos_emb = fused_apply_rope
    getattr(module, norm_cls or prefix + "RMSNorm").forward = rmsnorm_forward
    getattr(module, mlp_cls or prefix + "MLP").forward = mlp
    dec = getattr(module, decoder_cls or prefix + "DecoderLayer")
    dec.forward = make_decoder_layer_forward(dec.forward, fuse_add_norm)
    lm = getattr(module, causal_cls or prefix + "ForCausalLM")
    lm.forward = make_causal_forward(lm.forward, output_cls, extra_fields)
    module._mdy_patched = True
