"""Thin host wrappers over the C ABI for the StableHLO-level quantized matmuls.

Each function checks shapes and dtypes, hands raw device pointers and the
current CUDA stream to ``libqmm.so`` and returns a torch tensor that owns the
output memory.  PyTorch is only the allocator and the stream here; all
arithmetic happens in the library's kernels, and a missing library or a
non-CUDA tensor is an error (there is no fallback path).
"""

from __future__ import annotations

import torch

from . import _lib


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is None:
            continue
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise TypeError("quantized-matmul operators run on CUDA tensors only (no CPU fallback)")
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous (row-major)")


def w8a32_perchannel(x: torch.Tensor, w: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """``x @ (w.astype(f32) * scale[None, :])`` with x f32 ``[M,K]``, w int8 ``[K,N]``, scale f32 ``[N]``.

    One fused kernel in place of the reference's convert / broadcast_in_dim /
    multiply / dot_general chain (src/pjrt_plugin/ops/shape_ops.mm:793-829,
    ops/binary_ops.mm:165-193, :1006-1019).
    """
    _need_cuda(x, w, scale)
    if x.dtype != torch.float32 or w.dtype != torch.int8 or scale.dtype != torch.float32:
        raise TypeError("expected x float32, w int8, scale float32")
    lead = x.shape[:-1]
    K = x.shape[-1]
    if w.ndim != 2 or w.shape[0] != K or scale.shape != (w.shape[1],):
        raise ValueError(f"shape mismatch: x {tuple(x.shape)}, w {tuple(w.shape)}, scale {tuple(scale.shape)}")
    N = w.shape[1]
    x2 = x.reshape(-1, K)
    y = torch.empty((x2.shape[0], N), dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().qmm_w8a32_perchannel(x2.data_ptr(), w.data_ptr(), scale.data_ptr(), y.data_ptr(),
                                               x2.shape[0], N, K, _stream_ptr()))
    return y.reshape(*lead, N)


def w8a16_perchannel(x: torch.Tensor, w: torch.Tensor, scale: torch.Tensor, out: torch.Tensor | None = None,
                     out_col_offset: int = 0, independent: bool = False) -> torch.Tensor:
    """bf16 ``x[M,K]`` times int8 ``w[K,N]`` with per-channel f32 ``scale[N]`` -> bf16.

    ``out`` may be a wider ``[M, N_total]`` buffer; the result is written to
    columns ``[out_col_offset, out_col_offset + N)`` (how a rank that holds a
    column shard writes into the gathered output).  ``independent=True`` states
    that nothing still running on the stream writes the operands or touches
    the output (``QMM_GEMM_INDEPENDENT``): the launch is not ordered behind
    its predecessor.
    """
    _need_cuda(x, w, scale, out)
    if x.dtype != torch.bfloat16 or w.dtype != torch.int8 or scale.dtype != torch.float32:
        raise TypeError("expected x bfloat16, w int8, scale float32")
    if x.ndim != 2 or w.ndim != 2 or x.shape[1] != w.shape[0] or scale.shape != (w.shape[1],):
        raise ValueError(f"shape mismatch: x {tuple(x.shape)}, w {tuple(w.shape)}, scale {tuple(scale.shape)}")
    M, K = x.shape
    N = w.shape[1]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        out_col_offset = 0
    if out.dtype != torch.bfloat16 or out.ndim != 2 or out.shape[0] != M or out_col_offset + N > out.shape[1]:
        raise ValueError("bad output buffer")
    ldy = out.shape[1]
    yptr = out.data_ptr() + 2 * out_col_offset
    if independent:
        import ctypes

        ext = _lib.GemmExt(_lib.QMM_GEMM_INDEPENDENT)
        _lib.check(_lib.load().qmm_w8a16_perchannel_ex(x.data_ptr(), w.data_ptr(), scale.data_ptr(), yptr, M, N, K, ldy,
                                                       ctypes.byref(ext), _stream_ptr()))
        return out
    _lib.check(_lib.load().qmm_w8a16_perchannel(x.data_ptr(), w.data_ptr(), scale.data_ptr(), yptr, M, N, K, ldy,
                                                _stream_ptr()))
    return out


def i8_dot(a: torch.Tensor, b: torch.Tensor, row_scale: torch.Tensor | None = None,
           col_scale: torch.Tensor | None = None, want_acc: bool = True):
    """``dot_general(a, b, preferred_element_type=int32)`` for int8/uint8 operands,
    optionally followed by ``acc.astype(f32) * row[:, None] * col[None, :]``.

    Returns ``(acc_int32 or None, out_f32 or None)``.  Replaces the reference's
    IntegerMatMul emulation (src/pjrt_plugin/ops/binary_ops.mm:433-475).
    """
    _need_cuda(a, b, row_scale, col_scale)
    if a.dtype not in (torch.int8, torch.uint8) or b.dtype not in (torch.int8, torch.uint8):
        raise TypeError("operands must be int8 or uint8")
    if a.ndim != 2 or b.ndim != 2 or a.shape[1] != b.shape[0]:
        raise ValueError(f"shape mismatch: a {tuple(a.shape)}, b {tuple(b.shape)}")
    M, K = a.shape
    N = b.shape[1]
    rescale = row_scale is not None or col_scale is not None
    if rescale:
        if row_scale is None or col_scale is None:
            raise ValueError("row_scale and col_scale go together")
        if row_scale.dtype != torch.float32 or col_scale.dtype != torch.float32:
            raise TypeError("scales must be float32")
        if row_scale.shape != (M,) or col_scale.shape != (N,):
            raise ValueError("scale shapes must be [M] and [N]")
    acc = torch.empty((M, N), dtype=torch.int32, device=a.device) if want_acc else None
    out = torch.empty((M, N), dtype=torch.float32, device=a.device) if rescale else None
    if acc is None and out is None:
        raise ValueError("nothing to compute: want_acc is False and no scales were given")
    _lib.check(_lib.load().qmm_i8i8_i32(
        a.data_ptr(), b.data_ptr(), acc.data_ptr() if acc is not None else None,
        row_scale.data_ptr() if rescale else None, col_scale.data_ptr() if rescale else None,
        out.data_ptr() if out is not None else None, M, N, K,
        1 if a.dtype == torch.uint8 else 0, 1 if b.dtype == torch.uint8 else 0, _stream_ptr()))
    return acc, out


class W4Workspace:
    """Scratch for the split-K int4 decode kernel: zeroed once, left zeroed by every call."""

    def __init__(self, device: torch.device):
        self.device = device
        self.buf: torch.Tensor | None = None

    def get(self, nbytes: int) -> torch.Tensor:
        if self.buf is None or self.buf.numel() < nbytes:
            self.buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=self.device)
        return self.buf


_w4_workspaces: dict = {}


def w4a16_g128(x: torch.Tensor, wq: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, *,
               zeros_packed: bool = False, group: int = 128, out: torch.Tensor | None = None,
               workspace: torch.Tensor | None = None, static_weights: bool = False) -> torch.Tensor:
    """int4 group-wise asymmetric weight-only matmul (decode kernel for M <= 32, tcgen05 GEMM above).

    x bf16 ``[M,K]``; wq uint8 ``[K/2,N]`` (low nibble = even k);
    scales bf16 ``[K/group,N]``; zeros uint8 ``[K/group,N]`` or packed
    ``[K/group,N/2]``; returns bf16 ``[M,N]``.  ``static_weights=True`` tells
    the kernel that nothing queued earlier on the stream writes the weights,
    so it may fetch them while the previous kernel is still finishing.
    """
    _need_cuda(x, wq, scales, zeros, out, workspace)
    if x.dtype != torch.bfloat16 or wq.dtype != torch.uint8 or scales.dtype != torch.bfloat16 or zeros.dtype != torch.uint8:
        raise TypeError("expected x bfloat16, wq uint8, scales bfloat16, zeros uint8")
    if x.ndim != 2 or wq.ndim != 2 or 2 * wq.shape[0] != x.shape[1]:
        raise ValueError(f"shape mismatch: x {tuple(x.shape)}, wq {tuple(wq.shape)}")
    M, K = x.shape
    N = wq.shape[1]
    if K % group:
        raise ValueError(f"K ({K}) must be divisible by group ({group})")
    G = K // group
    if scales.shape != (G, N) or zeros.shape != ((G, N // 2) if zeros_packed else (G, N)):
        raise ValueError(f"scales/zeros shapes do not match: {tuple(scales.shape)}, {tuple(zeros.shape)}")
    lib = _lib.load()
    need = lib.qmm_w4a16_g128_workspace_bytes(M, N, K)  # 0 for M > 32: the prefill GEMM needs no scratch
    if workspace is None and need > 0:
        key = (x.device.index,)
        ws = _w4_workspaces.setdefault(key, W4Workspace(x.device))
        workspace = ws.get(need)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    _lib.check(lib.qmm_w4a16_g128(x.data_ptr(), wq.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                  1 if zeros_packed else 0, out.data_ptr(), M, N, K, group,
                                  workspace.data_ptr() if workspace is not None else None,
                                  workspace.numel() if workspace is not None else 0,
                                  _lib.QMM_W4_STATIC_WEIGHTS if static_weights else 0,
                                  _stream_ptr()))
    return out
