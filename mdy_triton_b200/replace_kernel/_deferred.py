"""A decoder layer's output ``residual + mlp_out`` whose add has not run yet.

The reference adds the MLP branch to the residual stream at the end of every decoder layer
(``mdy_triton/replace_kernel/llama.py:74``) and the next layer starts by normalising that sum
(``llama.py:40-42``).  With residual fusion switched on (``set_residual_fusion(True)``), a patched layer
returns this tensor subclass instead of the sum: it aliases the MLP branch and carries the residual.  The
next patched layer (or the model's final RMSNorm) takes both parts and runs ONE fused add+RMSNorm kernel,
which saves a pass over the residual stream in the forward and two in the backward per layer.

Anything else that touches the object — a hook, ``output_hidden_states``, user code between the layers —
goes through ``__torch_function__``, which first replaces it by the real sum, so every other consumer sees
the value the stock layer would have returned.
"""
from __future__ import annotations

import torch
from torch.utils._pytree import tree_map

_no_dispatch = torch._C.DisableTorchFunctionSubclass

# Queries that do not depend on the values: answered from the branch tensor (same shape, dtype, device).
_METADATA = {
    torch.Tensor.shape.__get__, torch.Tensor.dtype.__get__, torch.Tensor.device.__get__,
    torch.Tensor.ndim.__get__, torch.Tensor.is_cuda.__get__, torch.Tensor.layout.__get__,
    torch.Tensor.requires_grad.__get__, torch.Tensor.size, torch.Tensor.dim, torch.Tensor.numel,
    torch.Tensor.element_size, torch.Tensor.is_floating_point, torch.Tensor.get_device,
}


class DeferredResidual(torch.Tensor):
    """``branch + residual``, not yet added.  Create with :meth:`wrap`, take apart with :meth:`parts`."""

    @staticmethod
    def wrap(branch: torch.Tensor, residual: torch.Tensor) -> "DeferredResidual":
        with _no_dispatch():
            out = branch.as_subclass(DeferredResidual)  # alias of `branch`, still attached to autograd
        out._mdy_residual = residual
        return out

    def parts(self):
        with _no_dispatch():
            return self.as_subclass(torch.Tensor), self._mdy_residual

    def materialize(self) -> torch.Tensor:
        branch, residual = self.parts()
        return residual + branch

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func in _METADATA:
            with _no_dispatch():
                return func(*args, **kwargs)
        args, kwargs = tree_map(_materialize, (args, kwargs))
        return func(*args, **kwargs)


def _materialize(x):
    return x.materialize() if type(x) is DeferredResidual else x
