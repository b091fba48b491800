"""Host logic of the N-sharded linears, two ranks over gloo on the CPU.

The CUDA kernel cannot run here, so the local matmul is replaced by the oracle;
what is under test is the sharding bookkeeping, the all-gather and the
``[P, M, N/P]`` -> ``[M, N]`` addressing, plus the behaviour when a rank is
missing (bounded process-group timeout, error instead of a hang)."""

import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jax_metallib_b200 import tp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_matmul(x, w, scale):
    from oracle import qmm_oracle as O

    y = O.w8_perchannel_matmul(x.float().numpy(), w.numpy(), scale.numpy())
    return torch.from_numpy(O.round_to_bf16(y)).to(torch.bfloat16)


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    try:
        M, K, N = 16, 64, 96
        rng = np.random.default_rng(5)  # same on every rank: replicated activations, one global weight
        x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16)
        w = torch.from_numpy(rng.integers(-127, 128, size=(K, N), dtype=np.int64).astype(np.int8))
        scale = torch.from_numpy(rng.uniform(0.005, 0.02, size=(N,)).astype(np.float32))
        a, b = tp.shard_bounds(N, world, rank)
        lin = tp.ColumnShardedLinear(w[:, a:b].contiguous(), scale[a:b].contiguous(), N)
        gathered = lin.forward(x, matmul=_oracle_matmul)
        assert gathered.shape == (world, M, N // world)
        logical = tp.gathered_to_logical(gathered)
        full = _oracle_matmul(x, w, scale)
        assert torch.equal(logical, full), "gathered output differs from the unsharded result"
        torch.save(logical, os.path.join(result_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_column_sharding_and_gather(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a = torch.load(tmp_path / "rank0.pt")
    b = torch.load(tmp_path / "rank1.pt")
    assert torch.equal(a, b)


def _exchange_worker(rank, world, port, result_dir):
    # GatherExchange over gloo ranks: the slot/linear bookkeeping and the [P, M, N/P] buffers, with the
    # oracle in place of the CUDA kernel
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    try:
        M, K = 16, 64
        shapes = {"a": (M, 96), "b": (M, 32)}
        rng = np.random.default_rng(6)
        x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16)
        ex = tp.GatherExchange(shapes, "cpu", depth=2)
        assert ex.mode == "collective" and ex.world == world
        for use in range(3):  # slots alternate; the third use overwrites slot 0
            slot = use & 1
            for name, (_, n) in shapes.items():
                w = torch.from_numpy(rng.integers(-127, 128, size=(K, n), dtype=np.int64).astype(np.int8))
                scale = torch.from_numpy(rng.uniform(0.005, 0.02, size=(n,)).astype(np.float32))
                a, b = tp.shard_bounds(n, world, rank)
                out = ex.linear(name, slot, x, w[:, a:b].contiguous(), scale[a:b].contiguous(), matmul=_oracle_matmul)
                assert out.shape == (world, M, n // world)
                assert torch.equal(ex.logical(name, slot), _oracle_matmul(x, w, scale))
                assert torch.equal(tp.gathered_view(out)[:, rank, :], _oracle_matmul(x, w[:, a:b], scale[a:b]))
        ex.finish()
        # the symmetric-memory modes are refused on CPU ranks, unknown modes everywhere
        for mode in ("fused", "mcast", "peer", "copy"):
            try:
                tp.GatherExchange(shapes, "cpu", depth=2, mode=mode)
            except ValueError as exc:
                assert "CUDA" in str(exc)
            else:
                raise AssertionError(f"mode {mode!r} accepted on CPU ranks")
        try:
            tp.GatherExchange(shapes, "cpu", depth=2, mode="ring")
        except ValueError as exc:
            assert "unknown exchange mode" in str(exc)
        else:
            raise AssertionError("unknown mode accepted")
        with open(os.path.join(result_dir, f"ok{rank}"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_exchange_bookkeeping(tmp_path):
    port = _free_port()
    mp.spawn(_exchange_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_exchange_layout_plan():
    blocks, sig, total = tp.plan_layout({"qkv": (4096, 10240), "o": (4096, 8192)}, world=8, depth=2)
    assert blocks[(0, "qkv")].offset == 0 and blocks[(0, "qkv")].block_bytes == 4096 * 1280 * 2
    assert blocks[(0, "o")].offset == 4096 * 10240 * 2
    assert blocks[(1, "qkv")].offset == 4096 * (10240 + 8192) * 2
    assert sig == 2 * 4096 * (10240 + 8192) * 2 and total >= sig + 2 * 2 * 8 * 4 and total % 256 == 0
    assert all(b.offset % 256 == 0 for b in blocks.values())
    with pytest.raises(ValueError):
        tp.plan_layout({"x": (4, 10)}, world=4, depth=1)
    with pytest.raises(ValueError):
        tp.plan_layout({"x": (4, 8)}, world=4, depth=0)


def test_shard_bounds_and_errors():
    assert tp.shard_bounds(10240, 8, 3) == (3840, 5120)
    assert [tp.shard_bounds(8, 2, r) for r in range(2)] == [(0, 4), (4, 8)]
    with pytest.raises(ValueError):
        tp.shard_bounds(10, 4, 0)
    with pytest.raises(ValueError):
        tp.shard_bounds(8, 2, 2)
    g = torch.arange(2 * 3 * 4).reshape(2, 3, 4)
    logical = tp.gathered_to_logical(g)
    assert logical.shape == (3, 8)
    assert torch.equal(logical[1], torch.cat([g[0, 1], g[1, 1]]))
    view = tp.gathered_view(g)  # [M, P, N/P] without a copy
    assert view.shape == (3, 2, 4) and view.data_ptr() == g.data_ptr()
    assert torch.equal(view[1, 1], g[1, 1])


def _absent_peer_worker(rank, world, port, result_dir):
    # rank 1 never joins the collective: rank 0 must get an error within the timeout, not hang
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        if rank == 1:
            return  # leaves between steps, with nothing in flight
        y = torch.ones(4, 8)
        out = torch.empty(2 * 4 * 8)
        try:
            dist.all_gather_into_tensor(out, y.view(-1))
            outcome = "completed"
        except Exception as e:  # noqa: BLE001
            outcome = "error:" + type(e).__name__
        with open(os.path.join(result_dir, "outcome.txt"), "w") as f:
            f.write(outcome)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_missing_rank_gives_an_error_not_a_hang(tmp_path):
    port = _free_port()
    import time

    ctx = mp.spawn(_absent_peer_worker, args=(2, port, str(tmp_path)), nprocs=2, join=False)
    deadline = time.time() + 90
    while time.time() < deadline:
        try:
            if ctx.join(timeout=5):
                break
        except Exception:  # a rank that exits with the collective's error is the expected outcome
            break
    for p in ctx.processes:
        if p.is_alive():
            p.terminate()
            pytest.fail("a rank was still waiting after the process-group timeout")
    assert (tmp_path / "outcome.txt").read_text().startswith("error:")
