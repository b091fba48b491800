"""CPU oracle for the Llama-shaped int4 decode step.  TEST INFRASTRUCTURE ONLY.

A NumPy restatement of the step the decode workload defines (32-layer
Llama-3-8B architecture at full size; the tests run it at reduced depth and
width): embedding gather, RMSNorm, int4 group-wise weight-only linears, rotary
embedding, grouped-query attention over a KV cache plus the new row, SwiGLU,
residual adds, final norm and a bf16 lm_head.  Activations live in bf16 between
operators (every operator's result is rounded to bf16, as a bf16 JAX program
does on XLA:CPU, see src/pjrt_plugin/ops/registry.h:273-287 of the reference);
inside an operator arithmetic is f32 or better.  The reference has no model of
its own on this path (its benchmarks scan generic float layers,
benchmarks/vs_jax_mps.py:759-807) and no test of it: parity for the step is
UNPINNED; the contract is the stated tolerance against this restatement.
"""

from __future__ import annotations

import numpy as np

from . import qmm_oracle as O

bf = O.round_to_bf16


def take_rows(table, ids, fill=0.0):
    """Row gather with jnp.take's semantics as the reference's fused take kernel implements them:
    negative indices wrap, out-of-range rows get the fill value (README.md:200-202)."""
    V = table.shape[0]
    ids = np.asarray(ids, dtype=np.int64)
    idx = np.where(ids < 0, ids + V, ids)
    ok = (idx >= 0) & (idx < V)
    out = np.where(ok[:, None], table[np.clip(idx, 0, V - 1)], np.float32(fill))
    return out.astype(np.float32)


def rmsnorm(h, w, eps):
    h = h.astype(np.float32)
    inv = 1.0 / np.sqrt(np.mean(h.astype(np.float64) ** 2, axis=-1, keepdims=True) + eps)
    return bf(bf((h * inv).astype(np.float32)) * w.astype(np.float32))


def rope(x, pos, theta):
    """x [B, H, hd]; rotate-half pairing (i, i + hd/2)."""
    B, H, hd = x.shape
    half = hd // 2
    freq = theta ** (-2.0 * np.arange(half, dtype=np.float64) / hd)
    ang = np.asarray(pos, dtype=np.float64)[:, None] * freq[None, :]
    cs, sn = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, c = x[..., :half].astype(np.float64), x[..., half:].astype(np.float64)
    return bf(np.concatenate([a * cs - c * sn, c * cs + a * sn], axis=-1).astype(np.float32))


def attention_decode(q, kcache, vcache, knew, vnew, scale):
    """q [B,Hq,hd]; caches [B,Hkv,L,hd]; new rows [B,Hkv,hd] appended as key L."""
    B, Hq, hd = q.shape
    Hkv = kcache.shape[1]
    R = Hq // Hkv
    out = np.zeros((B, Hq, hd), dtype=np.float32)
    for b in range(B):
        for h in range(Hq):
            kv = h // R
            K = np.concatenate([kcache[b, kv], knew[b, kv][None, :]], axis=0).astype(np.float64)
            V = np.concatenate([vcache[b, kv], vnew[b, kv][None, :]], axis=0).astype(np.float64)
            s = K @ q[b, h].astype(np.float64) * scale
            p = np.exp(s - s.max())
            out[b, h] = (p @ V / p.sum()).astype(np.float32)
    return bf(out)


def silu_mul(gate, up):
    g = gate.astype(np.float64)
    return bf(bf((g / (1.0 + np.exp(-g))).astype(np.float32)) * up.astype(np.float32))


def w4_linear(x, lin):
    """lin = dict(wq uint8 [K/2,N], s f32 [G,N] (bf16 values), z uint8 [G,N])."""
    return bf(O.w4a16_matmul(x, lin["wq"], lin["s"], lin["z"]))


def decode_step(model, ids, pos, kcache, vcache, shape):
    """One decode step.  model: dict with embed, lm_head, final_norm and layers[i] =
    dict(attn_norm, mlp_norm, q, k, v, o, gate, up, down).  Returns logits [B,V],
    new K rows and new V rows [layers, B, Hkv, hd]."""
    B = len(ids)
    Hq, Hkv, hd = shape["n_heads"], shape["n_kv_heads"], shape["head_dim"]
    h = take_rows(model["embed"], ids)
    nk, nv = [], []
    pending = None  # the mlp output waiting to be added to the residual stream
    for li, layer in enumerate(model["layers"]):
        if pending is not None:
            h = bf(h + pending)
        n1 = rmsnorm(h, layer["attn_norm"], shape["eps"])
        q = w4_linear(n1, layer["q"]).reshape(B, Hq, hd)
        k = w4_linear(n1, layer["k"]).reshape(B, Hkv, hd)
        v = w4_linear(n1, layer["v"]).reshape(B, Hkv, hd)
        q, k = rope(q, pos, shape["rope_theta"]), rope(k, pos, shape["rope_theta"])
        nk.append(k)
        nv.append(v)
        a = attention_decode(q, kcache[li], vcache[li], k, v, 1.0 / np.sqrt(hd))
        o = w4_linear(a.reshape(B, Hq * hd), layer["o"])
        h = bf(h + o)
        n2 = rmsnorm(h, layer["mlp_norm"], shape["eps"])
        act = silu_mul(w4_linear(n2, layer["gate"]), w4_linear(n2, layer["up"]))
        pending = w4_linear(act, layer["down"])
    h = bf(h + pending)
    nf = rmsnorm(h, model["final_norm"], shape["eps"])
    logits = bf((nf.astype(np.float64) @ model["lm_head"].astype(np.float64)).astype(np.float32))
    return logits, np.stack(nk), np.stack(nv)
