"""The operators of the int4 decode step and the step itself (reduced depth and
width) against the CPU oracle."""

import ctypes

import numpy as np
import pytest
import torch

from jax_metallib_b200 import _lib, synthetic
from jax_metallib_b200.decode_stack import DecodeStep, LlamaShape, random_model
from oracle import decode_oracle as D
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu


def f32(t):
    return synthetic.bf16_bits_to_f32(t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)).reshape(t.shape)


def bft(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(synthetic.to_bf16_bits(a).view(np.int16))).to(cuda).view(torch.bfloat16)


def stream():
    return torch.cuda.current_stream().cuda_stream


def test_take_rows_wraps_and_fills(cuda):
    lib = _lib.load()
    rng = np.random.default_rng(1)
    table = O.round_to_bf16(rng.standard_normal((50, 64)).astype(np.float32))
    ids = np.array([0, 49, -1, -50, 50, -51, 7], dtype=np.int32)
    out = torch.empty((len(ids), 64), dtype=torch.bfloat16, device=cuda)
    tt, it = bft(table, cuda), torch.from_numpy(ids).to(cuda)  # keep the device copies alive across the launch
    _lib.check(lib.qmm_take_rows_bf16(tt.data_ptr(), it.data_ptr(), out.data_ptr(), 50, 64, len(ids), 0, stream()))
    np.testing.assert_array_equal(f32(out), D.take_rows(table, ids))


@pytest.mark.parametrize("with_residual", [False, True])
def test_add_rmsnorm(cuda, with_residual):
    lib = _lib.load()
    rng = np.random.default_rng(2)
    B, Dm = 5, 4096
    x = O.round_to_bf16(rng.standard_normal((B, Dm)).astype(np.float32) * 3)
    r = O.round_to_bf16(rng.standard_normal((B, Dm)).astype(np.float32))
    w = O.round_to_bf16(1 + 0.1 * rng.standard_normal(Dm).astype(np.float32))
    s_out = torch.empty((B, Dm), dtype=torch.bfloat16, device=cuda)
    n_out = torch.empty((B, Dm), dtype=torch.bfloat16, device=cuda)
    xt, rt, wt = bft(x, cuda), bft(r, cuda), bft(w, cuda)
    _lib.check(lib.qmm_add_rmsnorm_bf16(xt.data_ptr(), rt.data_ptr() if with_residual else None, wt.data_ptr(),
                                        s_out.data_ptr() if with_residual else None, n_out.data_ptr(), B, Dm,
                                        ctypes.c_float(1e-5), stream()))
    h = O.round_to_bf16(x + r) if with_residual else x
    if with_residual:
        np.testing.assert_array_equal(f32(s_out), h)
    assert O.max_rel_err(f32(n_out), D.rmsnorm(h, w, 1e-5)) <= 1e-2


@pytest.mark.parametrize("fused", [False, True])
def test_rope(cuda, fused):
    lib = _lib.load()
    rng = np.random.default_rng(3)
    B, Hq, Hkv, hd = 4, 8, 2, 128
    q = O.round_to_bf16(rng.standard_normal((B, Hq, hd)).astype(np.float32))
    k = O.round_to_bf16(rng.standard_normal((B, Hkv, hd)).astype(np.float32))
    pos = np.array([0, 1, 2047, 100000], dtype=np.int32)
    pt = torch.from_numpy(pos).to(cuda)
    if fused:
        # q | k | v side by side in one buffer, as a fused projection writes them
        buf = torch.zeros((B, (Hq + 2 * Hkv) * hd), dtype=torch.bfloat16, device=cuda)
        buf[:, :Hq * hd] = bft(q, cuda).reshape(B, -1)
        buf[:, Hq * hd:(Hq + Hkv) * hd] = bft(k, cuda).reshape(B, -1)
        qt, kt = buf[:, :Hq * hd], buf[:, Hq * hd:(Hq + Hkv) * hd]
        ld = buf.shape[1]
        _lib.check(lib.qmm_rope_bf16(qt.data_ptr(), kt.data_ptr(), pt.data_ptr(), B, Hq, Hkv, hd,
                                     ctypes.c_float(500000.0), ld, ld, stream()))
        assert float(buf[:, (Hq + Hkv) * hd:].abs().max()) == 0.0  # the v slice is untouched
    else:
        qt, kt = bft(q, cuda), bft(k, cuda)
        _lib.check(lib.qmm_rope_bf16(qt.data_ptr(), kt.data_ptr(), pt.data_ptr(), B, Hq, Hkv, hd,
                                     ctypes.c_float(500000.0), Hq * hd, Hkv * hd, stream()))
    assert O.max_rel_err(f32(qt).reshape(q.shape), D.rope(q, pos, 500000.0)) <= 1e-2
    assert O.max_rel_err(f32(kt).reshape(k.shape), D.rope(k, pos, 500000.0)) <= 1e-2
    np.testing.assert_array_equal(f32(qt).reshape(q.shape)[0], q[0])  # position 0 is the identity


def test_silu_mul(cuda):
    lib = _lib.load()
    rng = np.random.default_rng(4)
    B, F = 3, 14336
    g = O.round_to_bf16(rng.standard_normal((B, F)).astype(np.float32) * 4)
    u = O.round_to_bf16(rng.standard_normal((B, F)).astype(np.float32))
    out = torch.empty((B, F), dtype=torch.bfloat16, device=cuda)
    gt, ut = bft(g, cuda), bft(u, cuda)
    _lib.check(lib.qmm_silu_mul_bf16(gt.data_ptr(), ut.data_ptr(), out.data_ptr(), B, F, F, stream()))
    assert O.max_rel_err(f32(out), D.silu_mul(g, u)) <= 1e-2


@pytest.mark.parametrize("B,Hq,Hkv,L", [(8, 32, 8, 2048), (3, 4, 1, 300), (2, 8, 8, 128), (2, 16, 2, 1), (2, 8, 2, 0),
                                        (1, 6, 2, 65), (2, 8, 1, 1000), (16, 32, 8, 63), (1, 5, 1, 4099)])
def test_attention_decode(cuda, B, Hq, Hkv, L):
    lib = _lib.load()
    rng = np.random.default_rng(5)
    hd = 128
    q = O.round_to_bf16(rng.standard_normal((B, Hq, hd)).astype(np.float32))
    kc = O.round_to_bf16(rng.standard_normal((B, Hkv, L, hd)).astype(np.float32))
    vc = O.round_to_bf16(rng.standard_normal((B, Hkv, L, hd)).astype(np.float32))
    kn = O.round_to_bf16(rng.standard_normal((B, Hkv, hd)).astype(np.float32))
    vn = O.round_to_bf16(rng.standard_normal((B, Hkv, hd)).astype(np.float32))
    out = torch.empty((B, Hq, hd), dtype=torch.bfloat16, device=cuda)
    ws = torch.empty(max(1, lib.qmm_attention_decode_workspace_bytes(B, Hq, Hkv, L)), dtype=torch.uint8, device=cuda)
    kct = bft(kc, cuda) if L else torch.empty(1, dtype=torch.bfloat16, device=cuda)
    vct = bft(vc, cuda) if L else torch.empty(1, dtype=torch.bfloat16, device=cuda)
    qt, knt, vnt = bft(q, cuda), bft(kn, cuda), bft(vn, cuda)
    _lib.check(lib.qmm_attention_decode_bf16(qt.data_ptr(), kct.data_ptr(), vct.data_ptr(), knt.data_ptr(),
                                             vnt.data_ptr(), out.data_ptr(), B, Hq, Hkv, L, hd,
                                             ctypes.c_float(1 / np.sqrt(hd)), Hq * hd, Hkv * hd, ws.data_ptr(),
                                             ws.numel(), 0, stream()))
    torch.cuda.synchronize()
    assert lib.qmm_device_status() == 0
    ref = D.attention_decode(q, kc, vc, kn, vn, 1 / np.sqrt(hd))
    assert O.max_rel_err(f32(out), ref) <= 1e-2
    # the same through slices of one fused q | k | v buffer
    fused = torch.zeros((B, (Hq + 2 * Hkv) * hd), dtype=torch.bfloat16, device=cuda)
    fused[:, :Hq * hd] = qt.reshape(B, -1)
    fused[:, Hq * hd:(Hq + Hkv) * hd] = knt.reshape(B, -1)
    fused[:, (Hq + Hkv) * hd:] = vnt.reshape(B, -1)
    out2 = torch.empty_like(out)
    ld = fused.shape[1]
    _lib.check(lib.qmm_attention_decode_bf16(fused.data_ptr(), kct.data_ptr(), vct.data_ptr(),
                                             fused[:, Hq * hd:].data_ptr(), fused[:, (Hq + Hkv) * hd:].data_ptr(),
                                             out2.data_ptr(), B, Hq, Hkv, L, hd, ctypes.c_float(1 / np.sqrt(hd)), ld, ld,
                                             ws.data_ptr(), ws.numel(), _lib.QMM_ATTN_STATIC_CACHE, stream()))
    torch.cuda.synchronize()
    assert torch.equal(out, out2)


def test_attention_decode_peaked_softmax(cuda):
    """One cache row dominates (a score far above the rest) and sits in the ragged last tile."""
    lib = _lib.load()
    rng = np.random.default_rng(6)
    B, Hq, Hkv, L, hd = 1, 4, 1, 200, 128
    q = O.round_to_bf16(rng.standard_normal((B, Hq, hd)).astype(np.float32))
    kc = O.round_to_bf16(rng.standard_normal((B, Hkv, L, hd)).astype(np.float32) * 0.1)
    kc[0, 0, 199] = O.round_to_bf16(q[0, 1] * 8)  # head 1 attends to row 199 almost exclusively
    vc = O.round_to_bf16(rng.standard_normal((B, Hkv, L, hd)).astype(np.float32))
    kn = O.round_to_bf16(rng.standard_normal((B, Hkv, hd)).astype(np.float32) * 0.1)
    vn = O.round_to_bf16(rng.standard_normal((B, Hkv, hd)).astype(np.float32))
    out = torch.empty((B, Hq, hd), dtype=torch.bfloat16, device=cuda)
    ws = torch.empty(lib.qmm_attention_decode_workspace_bytes(B, Hq, Hkv, L), dtype=torch.uint8, device=cuda)
    kct, vct, qt, knt, vnt = bft(kc, cuda), bft(vc, cuda), bft(q, cuda), bft(kn, cuda), bft(vn, cuda)
    _lib.check(lib.qmm_attention_decode_bf16(qt.data_ptr(), kct.data_ptr(), vct.data_ptr(), knt.data_ptr(),
                                             vnt.data_ptr(), out.data_ptr(), B, Hq, Hkv, L, hd,
                                             ctypes.c_float(1 / np.sqrt(hd)), Hq * hd, Hkv * hd, ws.data_ptr(),
                                             ws.numel(), 0, stream()))
    torch.cuda.synchronize()
    assert lib.qmm_device_status() == 0
    ref = D.attention_decode(q, kc, vc, kn, vn, 1 / np.sqrt(hd))
    assert O.max_rel_err(f32(out), ref) <= 1e-2
    assert O.max_rel_err(f32(out)[0, 1], vc[0, 0, 199]) <= 2e-2


@pytest.mark.parametrize("M,K,N", [(8, 4096, 128256), (1, 64, 64), (16, 512, 1024), (5, 128, 192)])
def test_bf16_matmul_small_m(cuda, M, K, N):
    lib = _lib.load()
    rng = np.random.default_rng(6)
    x = O.round_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    w = O.round_to_bf16(rng.standard_normal((K, N)).astype(np.float32) * 0.05)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=cuda)
    xt, wt = bft(x, cuda), bft(w, cuda)
    _lib.check(lib.qmm_bf16_matmul_small_m(xt.data_ptr(), wt.data_ptr(), y.data_ptr(), M, N, K, stream()))
    torch.cuda.synchronize()
    assert lib.qmm_device_status() == 0
    ref = (x.astype(np.float64) @ w.astype(np.float64)).astype(np.float32)
    assert O.max_rel_err(f32(y), ref) <= 1e-2


def test_decode_step_reduced_model_matches_oracle(cuda):
    shape = LlamaShape(n_layers=2, d_model=512, n_heads=4, n_kv_heads=1, ffn=1024, vocab=1024)
    B, L = 3, 300
    model = random_model(shape, cuda, seed=4000)
    gen = torch.Generator(device=cuda)
    gen.manual_seed(7)
    kc = [torch.randn((B, 1, L, 128), device=cuda, generator=gen).to(torch.bfloat16) for _ in range(2)]
    vc = [torch.randn((B, 1, L, 128), device=cuda, generator=gen).to(torch.bfloat16) for _ in range(2)]
    step = DecodeStep(shape, model, B, L, cuda)
    step.ids.copy_(torch.tensor([5, 1023, 77], dtype=torch.int32))
    logits, nk, nv = step.run(kc, vc)
    torch.cuda.synchronize()
    assert _lib.load().qmm_device_status() == 0

    def lin(l):
        zp = l["z"].cpu().numpy()
        return {"wq": l["wq"].cpu().numpy(), "s": f32(l["s"]), "z": O.unpack_u4_pairs_last(zp)}

    omodel = {"embed": f32(model["embed"]), "lm_head": f32(model["lm_head"]), "final_norm": f32(model["final_norm"]),
              "layers": [{**{k: lin(v) for k, v in layer.items() if isinstance(v, dict)},
                          "attn_norm": f32(layer["attn_norm"]), "mlp_norm": f32(layer["mlp_norm"])}
                         for layer in model["layers"]]}
    oshape = dict(n_heads=4, n_kv_heads=1, head_dim=128, eps=shape.eps, rope_theta=shape.rope_theta)
    ref_logits, ref_k, ref_v = D.decode_step(omodel, [5, 1023, 77], [L] * B, [f32(t) for t in kc], [f32(t) for t in vc], oshape)
    assert O.max_rel_err(f32(nk).reshape(ref_k.shape), ref_k) <= 1e-2
    assert O.max_rel_err(f32(nv).reshape(ref_v.shape), ref_v) <= 1e-2
    # two layers of bf16 round trips: the end-to-end bound is looser than a single linear's
    assert O.max_rel_err(f32(logits), ref_logits) <= 3e-2
    # the captured graph replays to the same result
    step.capture(kc, vc)
    step.graph.replay()
    torch.cuda.synchronize()
    assert O.max_rel_err(f32(step.logits), ref_logits) <= 3e-2
