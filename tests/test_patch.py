"""``from mdy_triton.replace_kernel import *`` swaps the HuggingFace attributes the reference swaps
(reference replace_kernel/llama.py:186-190, qwen2.py:200-204), against the installed transformers."""
import inspect

import torch

import mdy_triton.replace_kernel  # noqa: F401  (the import is the patch)
from mdy_triton_b200.core.fused_apply_rope import fused_apply_rope
from mdy_triton_b200.replace_kernel import _common


def _check_family(modname, prefix, rope=True):
    import importlib
    m = importlib.import_module(f"transformers.models.{modname}.modeling_{modname}")
    if rope:
        assert m.apply_rotary_pos_emb is fused_apply_rope
    assert getattr(m, prefix + "RMSNorm").forward is _common.rmsnorm_forward
    assert getattr(m, prefix + "MLP").forward.__module__ == _common.__name__
    dec = getattr(m, prefix + "DecoderLayer").forward
    lm = getattr(m, prefix + "ForCausalLM").forward
    assert dec.__module__ == _common.__name__
    assert "labels" in inspect.signature(lm).parameters
    assert "logits_to_keep" in inspect.signature(lm).parameters   # generate() looks for it by name
    assert "hidden_states" in inspect.signature(dec).parameters
    return m


def test_llama_and_qwen2_are_patched():
    _check_family("llama", "Llama")
    _check_family("qwen2", "Qwen2")


def test_mistral_and_phi3_are_patched():
    _check_family("mistral", "Mistral")
    m = _check_family("phi3", "Phi3")
    assert m.Phi3MLP.forward is _common.mlp_forward_fused_proj


def test_qwen2_vl_text_stack_is_patched():
    import transformers.models.qwen2_vl.modeling_qwen2_vl as m
    assert m.Qwen2VLRMSNorm.forward is _common.rmsnorm_forward
    assert m.Qwen2MLP.forward is _common.mlp_forward
    assert m.Qwen2VLDecoderLayer.forward.__module__ == _common.__name__
    assert "pixel_values" not in inspect.signature(m.Qwen2VLDecoderLayer.forward).parameters
    assert "labels" in inspect.signature(m.Qwen2VLForConditionalGeneration.forward).parameters
    assert m.apply_multimodal_rotary_pos_emb.__module__ == m.__name__   # left alone, as in the reference


def test_reference_import_paths_resolve():
    from mdy_triton.replace_kernel import trigger
    from mdy_triton.replace_kernel.llama import module, trigger as t2
    from mdy_triton.core import (fast_cross_entropy_loss, fused_apply_rope, triton_fused_add_norm,  # noqa: F401
                                 triton_fused_up_gate_silu, triton_fused_up_gate_silu_no_split, triton_max,
                                 triton_min, triton_rmsnorm)
    from mdy_triton.core.cross_entyopy_loss import _FastCrossEntropyLoss, triton_entropy_loss  # noqa: F401
    from mdy_triton.core.rmsnorm import _TritronRMSNorm  # noqa: F401
    from mdy_triton.core.fused_add_norm import _TritronFusedAddRMSNorm  # noqa: F401
    from mdy_triton.core.fused_silu import _FusedSiLU_Unsloth, _FusedSiLUNoSplit  # noqa: F401
    from mdy_triton.core.fused_apply_rope import _FusedApplyRope  # noqa: F401
    assert trigger is None and t2 is None and module.__name__.endswith("modeling_llama")


def test_shifted_labels():
    lb = torch.tensor([[1, 2, 3, 4], [5, 6, -100, 8]])
    out = _common.shifted_labels(lb)
    assert out.tolist() == [[2, 3, 4, -100], [6, -100, 8, -100]]


def test_patched_model_builds_on_cpu_and_refuses_to_run_there():
    """The patch must not break model construction; running on CPU must raise (no fallback)."""
    import pytest
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=128, max_position_embeddings=64)
    model = LlamaForCausalLM(cfg)
    ids = torch.randint(0, 128, (1, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        model(input_ids=ids, labels=ids)


def test_deferred_residual_behaves_like_the_sum():
    """The object a layer returns under residual fusion: every consumer other than the patched norms sees
    branch + residual, with gradients to both parts."""
    from mdy_triton_b200.replace_kernel._deferred import DeferredResidual
    a = torch.randn(2, 3, 4, requires_grad=True)
    r = torch.randn(2, 3, 4, requires_grad=True)
    d = DeferredResidual.wrap(a * 1.0, r * 1.0)
    assert type(d) is DeferredResidual and d.shape == (2, 3, 4) and d.dtype == torch.float32 and d.dim() == 3
    assert d.requires_grad and d.device.type == "cpu" and d.size(-1) == 4 and d.numel() == 24
    y = d * 2
    assert type(y) is torch.Tensor and torch.equal(y, (a + r) * 2)
    y.sum().backward()
    assert torch.equal(a.grad, torch.full_like(a, 2.0)) and torch.equal(r.grad, torch.full_like(r, 2.0))
    assert torch.equal(d[:, -1:, :], (a + r)[:, -1:, :]) and type(d[:, -1:, :]) is torch.Tensor
    assert torch.equal(torch.stack([d, d]), torch.stack([a + r, a + r]))
    assert torch.equal(d.float().detach(), (a + r).detach()) and torch.equal(torch.nn.functional.relu(d), torch.relu(a + r))
    branch, residual = d.parts()
    assert type(branch) is torch.Tensor and torch.equal(branch, a) and torch.equal(residual, r)


def test_residual_fusion_switch():
    from mdy_triton.replace_kernel import residual_fusion_enabled, set_residual_fusion
    before = residual_fusion_enabled()
    set_residual_fusion(True); assert residual_fusion_enabled()
    set_residual_fusion(False); assert not residual_fusion_enabled()
    set_residual_fusion(before)


def test_glm4_is_patched_on_explicit_import_only():
    """The reference's package ``__init__`` does not list glm4; importing the module applies it.  RoPE
    stays stock (reference glm4.py:5-6)."""
    import sys
    import transformers.models.glm.modeling_glm as m
    if "mdy_triton_b200.replace_kernel.glm4" not in sys.modules:
        assert m.GlmRMSNorm.forward is not _common.rmsnorm_forward
    import mdy_triton.replace_kernel.glm4  # noqa: F401
    _check_family("glm", "Glm", rope=False)
    assert m.GlmMLP.forward is _common.mlp_forward_fused_proj
    assert m.apply_rotary_pos_emb is not fused_apply_rope
