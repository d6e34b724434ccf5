"""Patch transformers' Qwen2-VL text stack with the fused kernels at import time
(reference: mdy_triton/replace_kernel/qwen2_vl.py:12-15,183): RMSNorm, MLP, decoder layer and the
conditional-generation forward.  Its multimodal rotary embedding is left alone, as in the reference."""
import importlib

from ._common import patch_family

module = importlib.import_module("transformers.models.qwen2_vl.modeling_qwen2_vl")
patch_family(module, "Qwen2VL", rope=False, mlp_cls="Qwen2MLP",
             norm_cls="Qwen2VLRMSNorm" if hasattr(module, "Qwen2VLRMSNorm") else "Qwen2RMSNorm",
             causal_cls="Qwen2VLForConditionalGeneration", output_cls=module.Qwen2VLCausalLMOutputWithPast,
             extra_fields=("rope_deltas",))

trigger = None
