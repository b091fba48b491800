"""Host side of the Llama-shaped int4 decode step.

The workload: a Llama-3-8B-architecture decoder (32 layers, d_model 4096, 32
query / 8 KV heads of dim 128, SwiGLU FFN 14336, RMSNorm, RoPE theta 500000,
vocab 128256), random-init, every linear projection quantized to int4 with
asymmetric group-wise (128 along K) parameters, bf16 activations, an
unquantized bf16 lm_head; decode of one token per sequence over a KV cache of
a given context.  All seven projections of a layer go through
``qmm_w4a16_g128``, as four launches: q, k, v share their input, so their
packed weights, scales and zero points are laid side by side along N at load
time and run as one matmul, and likewise gate and up (per output column the
arithmetic is that of the separate projection).  The other operators are the
small kernels of ``csrc/decode_ops.cu``; rope and attention read the q | k | v
slices of the fused output in place.  The KV cache is a read-only input and the step
returns the new K/V rows (the reference has no buffer donation, so a step that
returned an updated cache would copy it whole, src/pjrt_plugin/api/pjrt_api.cc:310).

``DecodeStep`` pre-allocates every buffer, issues the ~320 launches of a step
on the current stream and can capture them in a CUDA graph for replay.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib


@dataclass
class LlamaShape:
    n_layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    eps: float = 1e-5
    group: int = 128

    def linears(self):
        d, hq, hkv = self.d_model, self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        return {"q": (d, hq), "k": (d, hkv), "v": (d, hkv), "o": (hq, d), "gate": (d, self.ffn), "up": (d, self.ffn),
                "down": (self.ffn, d)}

    def weight_bytes_per_step(self, batch: int, context: int) -> int:
        """Algorithmic HBM bytes of one step: packed weights + scales + packed zero points of every
        linear, the KV cache read, and the bf16 lm_head (embedding rows and activations are negligible)."""
        per_layer = 0
        for k, n in self.linears().values():
            g = k // self.group
            per_layer += k * n // 2 + g * n * 2 + g * n // 2
        kv = 2 * batch * self.n_kv_heads * context * self.head_dim * 2
        return self.n_layers * (per_layer + kv) + self.d_model * self.vocab * 2


def random_int4_linear(k: int, n: int, group: int, device, gen) -> dict:
    """Packed nibbles uniform 0-15, bf16 scales U(0.002, 0.01), packed 4-bit zero points uniform 0-15."""
    g = k // group
    return {
        "wq": torch.randint(0, 256, (k // 2, n), dtype=torch.uint8, device=device, generator=gen),
        "s": (torch.rand((g, n), device=device, generator=gen) * 0.008 + 0.002).to(torch.bfloat16),
        "z": torch.randint(0, 256, (g, n // 2), dtype=torch.uint8, device=device, generator=gen),
        "k": k, "n": n,
    }


def fuse_linears(lins: list) -> dict:
    """Projections that share their input, laid side by side along N (packed weights, scales and
    packed zero points all have N as their last axis; every N here is even, so zero-point bytes
    do not straddle a boundary)."""
    assert all(l["k"] == lins[0]["k"] and l["n"] % 2 == 0 for l in lins)
    return {"wq": torch.cat([l["wq"] for l in lins], dim=1).contiguous(),
            "s": torch.cat([l["s"] for l in lins], dim=1).contiguous(),
            "z": torch.cat([l["z"] for l in lins], dim=1).contiguous(),
            "k": lins[0]["k"], "n": sum(l["n"] for l in lins)}


def random_model(shape: LlamaShape, device, seed: int = 4000) -> dict:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)

    def norm_w():
        return (1.0 + 0.1 * torch.randn(shape.d_model, device=device, generator=gen)).to(torch.bfloat16)

    layers = []
    for _ in range(shape.n_layers):
        layer = {name: random_int4_linear(k, n, shape.group, device, gen) for name, (k, n) in shape.linears().items()}
        layer["attn_norm"] = norm_w()
        layer["mlp_norm"] = norm_w()
        layers.append(layer)
    return {
        "embed": (torch.randn((shape.vocab, shape.d_model), device=device, generator=gen)).to(torch.bfloat16),
        "lm_head": (torch.randn((shape.d_model, shape.vocab), device=device, generator=gen) * 0.02).to(torch.bfloat16),
        "final_norm": norm_w(),
        "layers": layers,
    }


class DecodeStep:
    """One decode step of a batch over a fixed-length KV cache."""

    def __init__(self, shape: LlamaShape, model: dict, batch: int, context: int, device):
        self.shape, self.model, self.B, self.L, self.device = shape, model, batch, context, device
        self.lib = _lib.load()
        s, B = shape, batch
        bf16 = torch.bfloat16

        def buf(*dims):
            return torch.empty(dims, dtype=bf16, device=device)

        self.ids = torch.zeros(B, dtype=torch.int32, device=device)
        self.pos = torch.full((B,), context, dtype=torch.int32, device=device)
        self.h = buf(B, s.d_model)        # residual stream
        self.h2 = buf(B, s.d_model)
        self.n = buf(B, s.d_model)        # normed activations
        nq, nkv = s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim
        # one q | k | v row per layer and sequence: the new K/V rows a step returns are slices of it
        self.qkv = buf(s.n_layers, B, nq + 2 * nkv)
        self.new_k = self.qkv[:, :, nq:nq + nkv]
        self.new_v = self.qkv[:, :, nq + nkv:]
        self.attn = buf(B, nq)
        self.o = buf(B, s.d_model)
        self.gate_up = buf(B, 2 * s.ffn)
        self.act = buf(B, s.ffn)
        self.down = buf(B, s.d_model)
        self.logits = buf(B, s.vocab)
        self.fused = [{"qkv": fuse_linears([layer["q"], layer["k"], layer["v"]]),
                       "gate_up": fuse_linears([layer["gate"], layer["up"]])} for layer in model["layers"]]
        need = max(self.lib.qmm_w4a16_g128_workspace_bytes(B, n, k)
                   for k, n in [(s.d_model, nq + 2 * nkv), (nq, s.d_model), (s.d_model, 2 * s.ffn), (s.ffn, s.d_model)])
        self.w4_ws = torch.zeros(need, dtype=torch.uint8, device=device)
        self.attn_ws = torch.empty(max(1, self.lib.qmm_attention_decode_workspace_bytes(B, s.n_heads, s.n_kv_heads,
                                                                                        context)),
                                   dtype=torch.uint8, device=device)
        self.graph = None
        self.launches_per_step = 0

    # -- thin call helpers ------------------------------------------------------
    def _linear(self, x, lin, out, stream):
        _lib.check(self.lib.qmm_w4a16_g128(x.data_ptr(), lin["wq"].data_ptr(), lin["s"].data_ptr(), lin["z"].data_ptr(), 1,
                                           out.data_ptr(), self.B, lin["n"], lin["k"], self.shape.group,
                                           self.w4_ws.data_ptr(), self.w4_ws.numel(), _lib.QMM_W4_STATIC_WEIGHTS,
                                           stream))
        self.launches_per_step += 1

    def _norm(self, x, residual, w, sum_out, out, stream):
        _lib.check(self.lib.qmm_add_rmsnorm_bf16(x.data_ptr(), residual.data_ptr() if residual is not None else None,
                                                 w.data_ptr(), sum_out.data_ptr() if sum_out is not None else None,
                                                 out.data_ptr(), self.B, self.shape.d_model,
                                                 ctypes.c_float(self.shape.eps), stream))
        self.launches_per_step += 1

    def run(self, kcache, vcache):
        """Issue the launches of one step on the current stream.  kcache / vcache:
        lists (one per layer) of bf16 [B, Hkv, L, hd] tensors."""
        s, lib, B = self.shape, self.lib, self.B
        stream = torch.cuda.current_stream().cuda_stream
        self.launches_per_step = 0
        _lib.check(lib.qmm_take_rows_bf16(self.model["embed"].data_ptr(), self.ids.data_ptr(), self.h.data_ptr(), s.vocab,
                                          s.d_model, B, 0, stream))
        self.launches_per_step += 1
        pending = None
        for li, layer in enumerate(self.model["layers"]):
            if pending is None:
                self._norm(self.h, None, layer["attn_norm"], None, self.n, stream)
            else:
                # h <- h2 + down of the previous layer, and its norm, in one launch
                self._norm(self.h2, pending, layer["attn_norm"], self.h, self.n, stream)
            qkv = self.qkv[li]
            nq, nkv, ld = s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim, qkv.shape[1]
            q_ptr = qkv.data_ptr()
            k_ptr, v_ptr = q_ptr + 2 * nq, q_ptr + 2 * (nq + nkv)
            self._linear(self.n, self.fused[li]["qkv"], qkv, stream)
            _lib.check(lib.qmm_rope_bf16(q_ptr, k_ptr, self.pos.data_ptr(), B, s.n_heads, s.n_kv_heads, s.head_dim,
                                         ctypes.c_float(s.rope_theta), ld, ld, stream))
            _lib.check(lib.qmm_attention_decode_bf16(
                q_ptr, kcache[li].data_ptr(), vcache[li].data_ptr(), k_ptr, v_ptr, self.attn.data_ptr(), B, s.n_heads,
                s.n_kv_heads, self.L, s.head_dim, ctypes.c_float(1.0 / (s.head_dim ** 0.5)), ld, ld,
                self.attn_ws.data_ptr(), self.attn_ws.numel(), _lib.QMM_ATTN_STATIC_CACHE, stream))
            self.launches_per_step += 3  # rope + two attention launches
            self._linear(self.attn, layer["o"], self.o, stream)
            self._norm(self.h, self.o, layer["mlp_norm"], self.h2, self.n, stream)
            self._linear(self.n, self.fused[li]["gate_up"], self.gate_up, stream)
            _lib.check(lib.qmm_silu_mul_bf16(self.gate_up.data_ptr(), self.gate_up.data_ptr() + 2 * s.ffn,
                                             self.act.data_ptr(), B, s.ffn, 2 * s.ffn, stream))
            self.launches_per_step += 1
            self._linear(self.act, layer["down"], self.down, stream)
            pending = self.down
        self._norm(self.h2, pending, self.model["final_norm"], self.h, self.n, stream)
        _lib.check(lib.qmm_bf16_matmul_small_m(self.n.data_ptr(), self.model["lm_head"].data_ptr(), self.logits.data_ptr(),
                                               B, s.vocab, s.d_model, stream))
        self.launches_per_step += 1
        return self.logits, self.new_k, self.new_v

    def capture(self, kcache, vcache):
        """Capture one step in a CUDA graph (after one eager warm-up run)."""
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            self.run(kcache, vcache)
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                self.run(kcache, vcache)
        self.graph = g
        return g
