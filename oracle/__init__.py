"""CPU oracle for the fused-operator path.  TEST INFRASTRUCTURE ONLY.

Nothing under ``mdy_triton_b200/`` or ``mdy_triton/`` imports this package; only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py`` do, and only as the
checker or as the timed CPU baseline — never as the implementation of an operator.

Contents
  ``eager``       float32 PyTorch restatement of the five operators: the arithmetic of the reference's
                  Triton kernels (cited per function) and of the HuggingFace eager modules they
                  replace.  Runs anywhere.
  ``ref_loader``  loads the reference's own kernel files from a reference checkout and runs them on CPU
                  under Triton's interpreter.  Needs the checkout, so it is used only where one is
                  present: to pin ``eager`` and to generate ``tests/golden/*.pt``.

Parity status: PINNED.  ``eager`` is checked against the reference kernels themselves (run under the
Triton interpreter) by ``tests/test_oracle_pin.py`` when the checkout is present, and against the
golden vectors those kernels produced (``tests/golden/``, made by ``tests/golden/make_golden.py``)
everywhere else.  One exception: the reference's fused add+RMSNorm backward is wrong for hidden
sizes above 128 columns (its launch truncates the row), so above 128 columns that operator's
gradients are pinned to autograd of the eager restatement instead.
"""
