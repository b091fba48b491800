"""The explicit route into the fused kernels: ``stablehlo.custom_call @qmm_b200.qmm``.

A program that names the kernel it wants does not depend on the pattern matcher recognising how the
dequantisation chain was spelled.  The mechanism is the reference's native-kernel custom call
(src/jax_plugins/silicon/_native_metal.py:34-60,179-196: a primitive that lowers to
``mlir.custom_call(target, operands=..., backend_config=json)``), with its descriptor conventions
(src/pjrt_plugin/runtime/custom_metal_kernel.mm:129-193): a versioned JSON object, validated key by
key, bounded in size.  ``backend_config`` below builds that descriptor; ``call_text`` writes the op in
the textual form the planner (``qmm_plan_compile``) reads; ``lower`` is the lowering rule a JAX
primitive would use where jax is installed.
"""

from __future__ import annotations

import json

TARGET = "qmm_b200.qmm"
VERSION = 1
OPS = ("w8a32_perchannel", "w8a16_perchannel", "i8i8_i32", "w4a16_g128")
MAX_CONFIG_BYTES = 4096


def backend_config(op: str, *, zeros_packed: bool | None = None) -> str:
    """The JSON descriptor of one fused call (compact, ASCII, keys in a fixed order)."""
    if op not in OPS:
        raise ValueError(f"op must be one of {', '.join(OPS)}; got {op!r}")
    desc = {"version": VERSION, "op": op}
    if zeros_packed is not None:
        if op != "w4a16_g128":
            raise ValueError("zeros_packed only applies to w4a16_g128")
        desc["zeros_packed"] = bool(zeros_packed)
    text = json.dumps(desc, separators=(",", ":"), ensure_ascii=True)
    if len(text) > MAX_CONFIG_BYTES:
        raise ValueError("backend_config too large")
    return text


def call_text(result: str, operands, operand_types, result_type: str, config: str) -> str:
    """One ``stablehlo.custom_call`` line: ``%r = stablehlo.custom_call @qmm_b200.qmm(...) {...} : (...) -> ...``."""
    if len(operands) != len(operand_types):
        raise ValueError("one type per operand")
    escaped = config.replace("\\", "\\\\").replace('"', '\\"')
    return (f"    {result} = stablehlo.custom_call @{TARGET}({', '.join(operands)}) "
            f"{{api_version = 1 : i32, backend_config = \"{escaped}\"}} : "
            f"({', '.join(operand_types)}) -> {result_type}")


def module_text(arg_types, result_type: str, config: str, name: str = "jit_qmm") -> str:
    """A module whose ``@main`` is one fused call on its arguments."""
    args = ", ".join(f"%arg{i}: {t}" for i, t in enumerate(arg_types))
    body = call_text("%0", [f"%arg{i}" for i in range(len(arg_types))], list(arg_types), result_type, config)
    return (f"module @{name} {{\n  func.func public @main({args}) -> {result_type} {{\n{body}\n"
            f"    return %0 : {result_type}\n  }}\n}}\n")


def lower(ctx, *operands, config: str):  # pragma: no cover - needs jax
    """Lowering rule for a JAX primitive bound to this route (``mlir.register_lowering(prim, lower,
    platform="qmm_b200")``), the counterpart of ``_lower`` in the reference's ``_native_metal.py``."""
    from jax._src.interpreters import mlir

    return mlir.custom_call(
        TARGET,
        result_types=[mlir.aval_to_ir_type(ctx.module_context, aval) for aval in ctx.avals_out],
        operands=operands,
        backend_config=config,
        api_version=1,
        operand_layouts=[tuple(reversed(range(aval.ndim))) for aval in ctx.avals_in],
        result_layouts=[tuple(reversed(range(aval.ndim))) for aval in ctx.avals_out],
    ).results
