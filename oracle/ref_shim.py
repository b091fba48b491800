"""Load the reference's ``quantized.py`` CPU helpers without JAX.  TEST INFRASTRUCTURE ONLY.

The reference module needs ``jax.numpy`` only for array construction, dtype
names and ``matmul``; NumPy itself serves as the stand-in.  Its Metal launcher
is not importable off macOS, so ``quantized_matmul`` / ``affine_quantized_matmul``
take their CPU route (dequantise + matmul,
src/jax_plugins/silicon/quantized.py:1028-1031,1107-1112).

This only works where the reference checkout is present; it is used by
``tests/golden/make_golden.py`` to generate the committed fixtures and is never
needed at test or run time.
"""

from __future__ import annotations

import importlib.util
import os
import sys
import types

import numpy as np


def load_reference_quantized(reference_root: str):
    path = os.path.join(reference_root, "src", "jax_plugins", "silicon", "quantized.py")
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    saved = {k: sys.modules.get(k) for k in ("jax", "jax.numpy")}
    fake = types.ModuleType("jax")
    fake.numpy = np
    sys.modules["jax"] = fake
    sys.modules["jax.numpy"] = np
    try:
        spec = importlib.util.spec_from_file_location("_reference_quantized", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    return mod
