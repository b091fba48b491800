"""Compile-and-run front end for textual StableHLO modules.

``Executable(text)`` hands the module text to ``qmm_plan_compile`` (a
dependency-free C++ reader + dequant-chain matcher inside ``libqmm.so``) and
keeps the resulting launch plan; calling it with CUDA tensors in the order of
``@main``'s arguments runs one fused kernel per matched ``dot_general``.  This
is the part of the reference's compile/execute path
(``PJRT_Client_Compile`` -> parse -> plan -> ``Execute``,
src/pjrt_plugin/api/pjrt_client.cc:178-244, core/mps_executable.mm:9152) that
concerns the quantized matmul; unsupported programs are rejected at compile
time with the offending op named.
"""

from __future__ import annotations

import ctypes
import json

from . import _lib


def weight_only_linears_module(linears, name: str = "jit_layer") -> str:
    """Text of a StableHLO module that applies several int8 per-channel weight-only linears.

    ``linears`` is a list of ``(M, K, N, activation)`` with ``activation`` an integer naming which
    activation argument the linear reads (activations with the same number are one argument).
    ``@main`` takes the distinct activations (bf16 ``[M, K]``) first, then for every linear its
    weight (i8 ``[K, N]``) and scale (f32 ``[N]``), and returns one bf16 ``[M, N]`` per linear:
    ``x @ (convert(w) * broadcast(convert(scale)))``, the form of ``tests/fixtures/cfg5_w8a16.mlir``.
    """
    acts = {}
    for m, k, _n, a in linears:
        if acts.setdefault(a, (m, k)) != (m, k):
            raise ValueError(f"activation {a} is used with two different shapes")
    order = sorted(acts)
    args, body, rets, types = [], [], [], []
    for i, a in enumerate(order):
        m, k = acts[a]
        args.append(f"%arg{i}: tensor<{m}x{k}xbf16>")
    nxt = len(order)
    v = 0
    for m, k, n, a in linears:
        xi, wi, si = order.index(a), nxt, nxt + 1
        nxt += 2
        args += [f"%arg{wi}: tensor<{k}x{n}xi8>", f"%arg{si}: tensor<{n}xf32>"]
        body += [
            f"    %{v} = stablehlo.convert %arg{wi} : (tensor<{k}x{n}xi8>) -> tensor<{k}x{n}xbf16>",
            f"    %{v + 1} = stablehlo.convert %arg{si} : (tensor<{n}xf32>) -> tensor<{n}xbf16>",
            f"    %{v + 2} = stablehlo.broadcast_in_dim %{v + 1}, dims = [1] : (tensor<{n}xbf16>) -> tensor<{k}x{n}xbf16>",
            f"    %{v + 3} = stablehlo.multiply %{v}, %{v + 2} : tensor<{k}x{n}xbf16>",
            f"    %{v + 4} = stablehlo.dot_general %arg{xi}, %{v + 3}, contracting_dims = [1] x [0] : "
            f"(tensor<{m}x{k}xbf16>, tensor<{k}x{n}xbf16>) -> tensor<{m}x{n}xbf16>",
        ]
        rets.append(f"%{v + 4}")
        types.append(f"tensor<{m}x{n}xbf16>")
        v += 5
    head = (f"module @{name} attributes {{mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32}} {{\n"
            f"  func.func public @main({', '.join(args)}) -> ({', '.join(types)}) {{\n")
    return head + "\n".join(body) + f"\n    return {', '.join(rets)} : {', '.join(types)}\n  }}\n}}\n"


class Executable:
    def __init__(self, text: str):
        lib = _lib.load()
        self._lib = lib
        raw = text.encode("utf-8")
        handle = ctypes.c_void_p()
        _lib.check(lib.qmm_plan_compile(raw, len(raw), ctypes.byref(handle)))
        self._h = handle
        self.num_args = lib.qmm_plan_num_args(handle)
        self.num_results = lib.qmm_plan_num_results(handle)
        self.num_steps = lib.qmm_plan_num_steps(handle)
        self.workspace_bytes = lib.qmm_plan_workspace_bytes(handle)
        self._ws = None

    def trace(self) -> list[dict]:
        """The plan's decisions, one dict per ``QMM_PLAN_JSON:`` line."""
        n = self._lib.qmm_plan_trace(self._h, None, 0)
        buf = ctypes.create_string_buffer(n + 1)
        self._lib.qmm_plan_trace(self._h, buf, n + 1)
        out = []
        for line in buf.value.decode().splitlines():
            if line.startswith("QMM_PLAN_JSON:"):
                out.append(json.loads(line[len("QMM_PLAN_JSON:"):]))
        return out

    def __call__(self, args, results):
        """Run the plan: ``args`` / ``results`` are CUDA tensors in @main's order (results pre-allocated)."""
        import torch

        if len(args) != self.num_args or len(results) != self.num_results:
            raise ValueError(f"expected {self.num_args} arguments and {self.num_results} results")
        for t in list(args) + list(results):
            if not t.is_cuda or not t.is_contiguous():
                raise TypeError("arguments and results must be contiguous CUDA tensors")
        ws_ptr, ws_len = None, 0
        if self.workspace_bytes:
            if self._ws is None or self._ws.device != args[0].device:
                self._ws = torch.zeros(self.workspace_bytes, dtype=torch.uint8, device=args[0].device)
            ws_ptr, ws_len = self._ws.data_ptr(), self._ws.numel()
        a = (ctypes.c_void_p * len(args))(*[t.data_ptr() for t in args])
        r = (ctypes.c_void_p * len(results))(*[t.data_ptr() for t in results])
        _lib.check(self._lib.qmm_plan_execute(self._h, a, len(args), r, len(results), ws_ptr, ws_len,
                                              torch.cuda.current_stream().cuda_stream))
        return results

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                self._lib.qmm_plan_destroy(self._h)
                self._h = None
        except Exception:
            pass
