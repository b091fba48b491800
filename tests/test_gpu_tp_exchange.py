"""The gathered-output exchange of the column-sharded linears on two GPUs: one process per GPU,
NCCL for the rendezvous, every available exchange mode compared with the CPU oracle of the
unsharded linear on both ranks.  Skipped on a box with one GPU."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    import torch.distributed as dist

    from jax_metallib_b200 import _lib, synthetic, tp
    from oracle import qmm_oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # NCCL is only the rendezvous here
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        M, K = 1024, 512
        shapes = {"a": (M, 2560), "b": (M, 512)}
        rng = np.random.default_rng(11)  # the same global problem on every rank
        x_h = synthetic.bf16_bits_to_f32(synthetic.to_bf16_bits(rng.standard_normal((M, K)).astype(np.float32)))
        x = torch.from_numpy(x_h).to(device).to(torch.bfloat16)
        modes_seen = []
        for mode in ("auto", "mcast", "peer", "copy", "collective"):
            try:
                ex = tp.GatherExchange(shapes, device, depth=2, mode=mode)
            except RuntimeError:
                if mode != "mcast":
                    raise
                modes_seen.append("mcast-unavailable")   # no multicast address on this system (every rank agrees)
                continue
            modes_seen.append(ex.mode)
            for use in range(3):
                slot = use & 1
                for name, (_, n) in shapes.items():
                    w_h = rng.integers(-127, 128, size=(K, n), dtype=np.int64).astype(np.int8)
                    s_h = rng.uniform(0.005, 0.02, size=(n,)).astype(np.float32)
                    a, b = tp.shard_bounds(n, world, rank)
                    w = torch.from_numpy(np.ascontiguousarray(w_h[:, a:b])).to(device)
                    s = torch.from_numpy(np.ascontiguousarray(s_h[a:b])).to(device)
                    ex.linear(name, slot, x, w, s, independent=(mode != "collective"))
                    ex.finish()
                    torch.cuda.synchronize()
                    assert _lib.load().qmm_device_status() == 0
                    got = ex.logical(name, slot).float().cpu().numpy()
                    ref = O.w8_perchannel_matmul(x_h, w_h, s_h)
                    err = O.max_rel_err(got, ref)
                    assert err <= 1e-2, (mode, ex.mode, name, use, err)
                    dist.barrier()  # nobody overwrites a slot a peer is still reading
            if ex.mode in ("fused", "mcast", "peer"):
                assert int(ex.signal_words("a", 0)[0]) == 2 and int(ex.signal_words("a", 1)[1]) == 1
            ex.close()
            del ex
        with open(os.path.join(result_dir, f"modes{rank}.txt"), "w") as f:
            f.write(",".join(modes_seen))
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_two_gpu_exchange_modes_match_the_unsharded_oracle(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    m0 = (tmp_path / "modes0.txt").read_text()
    assert m0 == (tmp_path / "modes1.txt").read_text()
    print("exchange modes used:", m0)
