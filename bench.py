#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Headline workload (every N): the tensor-parallel int8 per-channel weight-only
linears with Llama-3-70B shapes — 80 layers of QKV 8192->10240, O 8192->8192,
gate+up 8192->2x28672, down 28672->8192 on bf16 activations [4096, 8192]
(random-init weights, seeded synthetic inputs).  One step = one pass over all
320 linears.  With N ranks the weights are column-sharded along N, every rank
computes its [4096, N/P] slice and the slices are all-gathered with NCCL
(strong scaling: total work is fixed).  ``value`` is prefill TFLOP/s of the
whole job, timed on the device with inputs resident in HBM; ``e2e`` is the same
metric with the step's activations copied from pinned host memory and the
last layer's result copied back inside the timed region.

At N = 1 the JSON line also carries, under ``detail``, the other workloads of
the path (decode int4 GEMV in GB/s, int8 x int8 GEMM in TOP/s, the small f32
case in microseconds), each with its own roofline fraction, and a CPU baseline
(the NumPy oracle timed on the host cores on a bounded sample).

``--impl reference`` times the reference's CPU route for this path — the
oracle restatement, since neither jaxlib's CPU backend nor the Metal plugin
can be installed here — on the same metric.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# SMs left to the multicast copy kernel of --exchange mcast: a rank's own egress is 1/P of the gathered
# bytes (6.9 GB per step at P = 8), so a few CTAs keep up; the links are loaded by what arrives.
MCAST_CTAS = 8
# SMs left to the all-gather kernel when the exchange is an NCCL collective (--exchange collective).
# Measured at N = 2 (40 layers): NCCL's own choice with no SMs reserved 1786 TFLOP/s (its CTAs queue
# behind the resident GEMM CTAs and delay the next launch), 8 reserved 1660 (the gather becomes the
# bottleneck), 16: 1967, 32: 1996.
NCCL_CTAS = 32
M_TOKENS = 4096
D_MODEL, FFN, QKV = 8192, 28672, 10240
N_LAYERS = 80
METRIC = "prefill_tflops_int8_weight_only_linears"


def layer_shapes():
    """(name, K, N, activation) for the four linears of a layer."""
    return [("qkv", D_MODEL, QKV, "x"), ("o", D_MODEL, D_MODEL, "x"), ("gate_up", D_MODEL, 2 * FFN, "x"),
            ("down", FFN, D_MODEL, "h")]


def flops_per_layer(m=M_TOKENS):
    return sum(2.0 * m * k * n for _, k, n, _ in layer_shapes())


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                        bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                        source="measured")
        except Exception:
            pass
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ----------------------------------------------------------------------------
# clocks sampled during the timed region
# ----------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return

        def reader():
            for line in self.proc.stdout:
                self.lines.append((time.time(), line.strip()))

        self.thread = threading.Thread(target=reader, daemon=True)
        self.thread.start()

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return None
        time.sleep(0.15)
        self.proc.terminate()  # the exact child this object started
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, smax, reasons = [], [], set()
        for ts, line in self.lines:
            if ts < t0 or ts > t1 + 0.2:
                continue
            f = [p.strip() for p in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------
# CPU baseline (oracle port) — also the --impl reference arm
# ----------------------------------------------------------------------------
def workload_config(world, layers, extra=None):
    """The ``config`` object both arms print (the reference arm runs a bounded sample of it)."""
    cfg = {"workload": f"int8 per-channel weight-only linears, Llama-3-70B shapes, {layers} layers x "
                       "(qkv 8192->10240, o 8192->8192, gate_up 8192->57344, down 28672->8192), "
                       "bf16 activations [4096,8192]",
           "layers": layers, "parallelism": f"tp{world}",
           "l2": "every launch reads a different weight matrix (>= 67 MB each at N = 1), inputs exceed L2"}
    if extra:
        cfg.update(extra)
    return cfg


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:  # noqa: BLE001
        return os.cpu_count() or 1


def pin_host_threads():
    """Use every host core for the CPU arm whatever the launcher exported (torch.distributed.run
    sets OMP_NUM_THREADS=1 for its children).  Must run before NumPy is imported."""
    n = str(host_cores())
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = n


class CpuLinears:
    """The NumPy oracle of one layer's four weight-only int8 linears on the host cores.

    A pass keeps the workload's M = 4096 rows and full K and takes one column slice (N / col_div
    columns) of each of the four weights, so dequantisation and GEMM work stay in the workload's
    own proportion; the slice is what bounds the time of a step."""

    def __init__(self, col_div: int):
        import numpy as np

        from jax_metallib_b200 import synthetic

        self.col_div = col_div
        rng = np.random.default_rng(5000)
        self.problems = []
        for _name, k, n, _act in layer_shapes():
            nc = max(16, n // col_div)
            x = synthetic.bf16_bits_to_f32(synthetic.to_bf16_bits(rng.standard_normal((M_TOKENS, k)).astype(np.float32)))
            w = rng.integers(-127, 128, size=(k, nc), dtype=np.int64).astype(np.int8)
            s = rng.uniform(0.005, 0.02, size=(nc,)).astype(np.float32)
            self.problems.append((x, w, s))
        self.flops = sum(2.0 * M_TOKENS * w.shape[0] * w.shape[1] for _, w, _ in self.problems)

    def one_pass(self):
        from oracle import qmm_oracle as O

        for x, w, s in self.problems:
            wf = O.w8_perchannel_dequant(w, s)  # fp32 dequantise
            y = x @ wf                            # f32 dot (BLAS, all host threads)
            O.f32_to_bf16_bits(y)                 # round to the declared result type

    def sample_text(self, passes, dt):
        return (f"M=4096 rows, full K, 1/{self.col_div} of the columns of each of one layer's four weights per step "
                f"({self.flops / 1e12:.3f} TFLOP), fp32 dequantise + NumPy matmul + bf16 rounding, "
                f"{passes} timed steps, {dt:.3f} s each")


def cpu_linears_tflops(steps: int, warmup: int, col_div: int = 16):
    """Time `steps` passes after `warmup` untimed ones; returns (cpu_baseline dict, seconds per step)."""
    try:
        from threadpoolctl import threadpool_limits
    except Exception:  # noqa: BLE001
        threadpool_limits = None
    prob = CpuLinears(col_div)
    cores = host_cores()

    def run():
        for _ in range(warmup):
            prob.one_pass()
        t0 = time.perf_counter()
        for _ in range(steps):
            prob.one_pass()
        return (time.perf_counter() - t0) / steps

    if threadpool_limits is not None:
        with threadpool_limits(limits=cores):
            dt = run()
    else:
        dt = run()
    return dict(value=prob.flops / dt / 1e12, unit="TFLOP/s", cores=cores, kind="port",
                sample=prob.sample_text(steps, dt)), dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    pin_host_threads()
    # --steps and --warmup are the passes really run; the column slice keeps the whole run within minutes
    # (a pass over 1/16 of the columns is about 1.8 s on 16 cores)
    base, dt = cpu_linears_tflops(steps=max(1, args.steps), warmup=max(0, args.warmup), col_div=16)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": max(1, args.steps), "warmup": max(0, args.warmup), "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus, args.layers),
        "note": "reference CPU route = NumPy oracle port on the host cores (jaxlib's CPU backend and the Metal "
                "plugin are not installable offline); each step is a bounded sample of the workload, see "
                "cpu_baseline.sample; the CPU rate does not depend on n_gpus",
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------
def build_weights(torch, synthetic, device, rank, world, layers):
    """Column shard of every layer's four weights, generated on the device."""
    from jax_metallib_b200 import tp

    gen = synthetic.torch_generator(device, 5, rank)
    weights = []
    for _l in range(layers):
        layer = []
        for name, k, n, act in layer_shapes():
            lo, hi = tp.shard_bounds(n, world, rank)
            ns = hi - lo
            w = synthetic.device_int8((k, ns), device, gen)
            s = synthetic.device_uniform((ns,), 0.005, 0.02, device, gen)
            layer.append((name, k, n, ns, act, w, s))
        weights.append(layer)
    return weights


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one w8a16_kernel launch at M = 4096, by
# (K, N), from the ncu captures summarised in profiles/w8a16_kernel_dram_traffic.md.  Shapes that
# were not captured are scaled by FLOPs from the nearest captured shape of the same K and said so.
MEASURED_TRAFFIC = {
    (8192, 10240): 417.29e6, (8192, 8192): 339.71e6, (8192, 57344): 2020.91e6, (28672, 8192): 1304.28e6,  # full width
    (8192, 5120): 231.95e6, (8192, 4096): 199.90e6, (8192, 28672): 1065.67e6, (28672, 4096): 794.24e6,    # N / 2
    (8192, 2560): 115.98e6, (8192, 2048): 85.28e6, (8192, 14336): 545.10e6, (28672, 2048): 295.03e6,      # N / 4
    (8192, 1280): 164.82e6, (8192, 1024): 77.20e6, (8192, 7168): 295.67e6, (28672, 1024): 266.00e6,       # N / 8
}


def launch_traffic(k, ns):
    """(bytes, how) for one launch of [4096, k] x [k, ns]."""
    if (k, ns) in MEASURED_TRAFFIC:
        return MEASURED_TRAFFIC[(k, ns)], "ncu"
    same_k = [(n2, b) for (k2, n2), b in MEASURED_TRAFFIC.items() if k2 == k]
    if same_k:
        n2, b = min(same_k, key=lambda t: abs(t[0] - ns))
        return b * ns / n2, "scaled"
    return None, "none"


def check_last_layer(torch, dist, ex, layer, slot, acts, rank, world, device):
    """Outside the timed region: four rows of every 256-row tile of the last layer's four gathered
    outputs against the CPU oracle of the unsharded linear.  Each rank computes the reference of its
    own columns, the references are all-gathered, and every rank compares all P blocks of its own
    copy of the gathered buffer (so the exchange is checked on every rank)."""
    import numpy as np

    from jax_metallib_b200 import synthetic, tp
    from oracle import qmm_oracle as O

    rows = np.array(sorted({t * 256 + o for t in range(M_TOKENS // 256) for o in (3, 100, 131, 250)}))
    rows_t = torch.from_numpy(rows).to(device)
    worst = 0.0
    ok = True
    for name, k, n, ns, act, w, s in layer:
        xs = synthetic.bf16_bits_to_f32(acts[act][rows_t].contiguous().view(torch.int16).cpu().numpy().view(np.uint16))
        w_h, s_h = w.cpu().numpy(), s.cpu().numpy()
        ref = np.empty((len(rows), ns), np.float32)
        for c0 in range(0, ns, 4096):
            ref[:, c0:c0 + 4096] = O.w8_perchannel_matmul(xs, w_h[:, c0:c0 + 4096], s_h[c0:c0 + 4096])
        ref_t = torch.from_numpy(ref).to(device)
        if world > 1:
            allref = torch.empty((world,) + tuple(ref_t.shape), dtype=torch.float32, device=device)
            dist.all_gather_into_tensor(allref.view(-1), ref_t.view(-1))
        else:
            allref = ref_t.unsqueeze(0)
        logical_ref = tp.gathered_to_logical(allref).cpu().numpy()  # [rows, N] of the unsharded linear
        got = tp.gathered_to_logical(ex.out(name, slot)[:, rows_t, :].contiguous())  # [rows, N]
        got = synthetic.bf16_bits_to_f32(got.contiguous().view(torch.int16).cpu().numpy().view(np.uint16))
        err = O.max_rel_err(got, logical_ref)
        worst = max(worst, err)
        ok = ok and err <= 1e-2 and bool(np.all(np.abs(got - logical_ref) <= np.abs(logical_ref) * 2.0**-7
                                                + 1e-3 * np.max(np.abs(logical_ref))))
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    worst_t = torch.tensor([worst], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        dist.all_reduce(worst_t, op=dist.ReduceOp.MAX)
    return bool(int(flag.item())), float(worst_t.item()), len(rows)


def run_gpu(args):
    import torch
    import torch.distributed as dist

    from jax_metallib_b200 import _lib, ops, synthetic, tp

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    lib = _lib.load()
    if world > 1:
        if args.exchange == "collective":
            # The GEMM keeps one CTA per SM resident for a whole launch; leave the all-gather its own SMs.
            os.environ.setdefault("NCCL_MAX_CTAS", str(NCCL_CTAS))
            os.environ.setdefault("NCCL_MIN_CTAS", str(NCCL_CTAS))
        dist.init_process_group("nccl", device_id=device)
    peaks = measured_peaks()
    layers = args.layers
    # --shard-of P (single GPU): rank 0's share of a P-way sharded run, without the exchange
    shard_world = args.shard_of if world == 1 else world
    shard_rank = 0 if world == 1 else rank

    weights = build_weights(torch, synthetic, device, shard_rank, shard_world, layers)
    x_host = torch.randn((M_TOKENS, D_MODEL), dtype=torch.float32).to(torch.bfloat16).pin_memory()
    h_host = torch.randn((M_TOKENS, FFN), dtype=torch.float32).to(torch.bfloat16).pin_memory()
    acts = {"x": x_host.to(device), "h": h_host.to(device)}
    # gathered outputs [P, M, N/P] per linear kind, two slots each (layer parity): the exchange of a
    # layer may run under the whole of the next layer
    shapes = {name: (M_TOKENS, n // (shard_world if world == 1 else 1)) for name, k, n, act in layer_shapes()}
    def reserve(mode):
        return args.copy_ctas if mode in ("mcast", "peer") else NCCL_CTAS

    ex = tp.GatherExchange(shapes, device, depth=2, mode=args.exchange, reserve_ctas=reserve(args.exchange))
    result_host = torch.empty((world, M_TOKENS, shapes["down"][1] // world), dtype=torch.bfloat16).pin_memory()
    launches = [0]

    def step(ex=None):
        # Every launch reads activations and weights that nothing on the stream writes, and writes a
        # slot whose previous use lies eight launches back: the launches are independent of their
        # predecessors, so each may fill the SMs that the last round of the one before leaves idle.
        ex = ex or exchange[0]
        for li, layer in enumerate(weights):
            for name, k, n, ns, act, w, s in layer:
                ex.linear(name, li & 1, acts[act], w, s, independent=True)
                launches[0] += 1
        ex.finish()  # every block of every rank has arrived in this rank's buffers

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    exchange = [ex]
    tuned = None
    if world > 1 and args.exchange == "auto" and ex.mode == "fused":
        # Three ways to fill the gathered buffers are available here: multimem stores in the GEMM's
        # epilogue (fused), a small multicast copy kernel per finished block on a side stream (mcast),
        # copy-engine peer copies (copy).  Which one is fastest depends on N: time two steps of each
        # before the measurement and keep the fastest, the same choice on every rank.
        times = {}
        for mode in ("fused", "mcast", "peer", "copy"):
            cand = ex if mode == "fused" else tp.GatherExchange(shapes, device, depth=2, mode=mode, reserve_ctas=reserve(mode))
            step(cand)
            barrier()
            c0 = torch.cuda.Event(enable_timing=True)
            c1 = torch.cuda.Event(enable_timing=True)
            c0.record()
            step(cand)
            step(cand)
            c1.record()
            barrier()
            t = torch.tensor([c0.elapsed_time(c1) / 2], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times[mode] = float(t.item())
            if mode != "fused":
                cand.close()
                del cand
        tuned = {"ms_per_step": times, "chosen": min(times, key=times.get)}
        if tuned["chosen"] != "fused":
            ex.close()
            ex = tp.GatherExchange(shapes, device, depth=2, mode=tuned["chosen"], reserve_ctas=reserve(tuned["chosen"]))
        exchange[0] = ex
        torch.cuda.empty_cache()

    # ---- resident-input timing -------------------------------------------------
    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    launches[0] = 0
    t_wall0 = time.time()
    ev0 = torch.cuda.Event(enable_timing=True)
    ev1 = torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    ms = ev0.elapsed_time(ev1)
    timed_launches = launches[0]
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    rank_flops = sum(2.0 * M_TOKENS * k * ns for layer in weights for _, k, _, ns, _, _, _ in layer)
    total_flops = rank_flops * world  # = flops_per_layer() * layers unless --shard-of cut it
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    # ---- end-to-end timing (host activations in, last result out) ---------------
    last_slot = (layers - 1) & 1
    h2d = x_host.numel() * 2 + h_host.numel() * 2
    d2h = result_host.numel() * 2
    if world == 1:
        # Through the runtime layer's C ABI (what a PJRT plugin's callbacks call): host buffers are
        # uploaded with BufferFromHostBuffer, every layer is one Execute of a compiled StableHLO module
        # with its four linears, the last layer's `down` output comes back with ToHostBuffer, and the
        # step ends when that transfer's event is ready.  Weights are device-resident views.
        import numpy as np

        from jax_metallib_b200 import runtime
        from jax_metallib_b200.stablehlo import weight_only_linears_module

        rt = runtime.Client()
        exe = rt.compile(weight_only_linears_module(
            [(M_TOKENS, k, ns, 0 if act == "x" else 1) for _, k, _, ns, act, _, _ in weights[0]]))
        layer_bufs = []
        for layer in weights:
            bufs = []
            for _, k, _, ns, _, w, s in layer:
                bufs.append(rt.view_of_device_memory(w.data_ptr(), _lib.QMM_S8, (k, ns), local_rank, keepalive=w))
                bufs.append(rt.view_of_device_memory(s.data_ptr(), _lib.QMM_F32, (ns,), local_rank, keepalive=s))
            layer_bufs.append(bufs)
        x_np = x_host.view(torch.int16).numpy().view(np.uint16)
        h_np = h_host.view(torch.int16).numpy().view(np.uint16)
        res_np = result_host.view(torch.int16).numpy().view(np.uint16).reshape(M_TOKENS, -1)

        def e2e_step():
            xb = rt.buffer_from_host(x_np, local_rank, dtype=_lib.QMM_BF16)
            hb = rt.buffer_from_host(h_np, local_rank, dtype=_lib.QMM_BF16)
            outs = None
            for bufs in layer_bufs:
                if outs is not None:
                    for o in outs:
                        o.destroy()  # stream-ordered free behind the launch that produced it
                outs, _ = exe.execute([xb, hb] + bufs, want_event=False)
            ev = outs[3].to_host(res_np)
            ev.await_(60000)
            for o in outs:
                o.destroy()
            xb.destroy()
            hb.destroy()

        torch.cuda.synchronize()
        e2e_step()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        e2e_ms = (time.perf_counter() - t0) * 1e3  # every step ends with a host-visible completion
        e2e_launches = args.steps * layers * 4
        e2e_api = ("qmm_rt_buffer_from_host -> qmm_rt_executable_execute (one compiled four-linear StableHLO module per "
                   "layer) -> qmm_rt_buffer_to_host, host wall clock around steps that each end with an awaited event")
        # what the runtime path computed is checked as well (the last layer's `down` output, rows sampled)
        rt_down = torch.from_numpy(res_np.view(np.int16).copy()).view(torch.bfloat16)
    else:
        def e2e_step():
            acts["x"].copy_(x_host, non_blocking=True)
            acts["h"].copy_(h_host, non_blocking=True)
            step()
            result_host.copy_(ex.out("down", last_slot), non_blocking=True)

        e2e_step()
        barrier()
        ee0 = torch.cuda.Event(enable_timing=True)
        ee1 = torch.cuda.Event(enable_timing=True)
        ee0.record()
        for _ in range(args.steps):
            e2e_step()
        ee1.record()
        barrier()
        e2e_ms = ee0.elapsed_time(ee1)
        t = torch.tensor([e2e_ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
        e2e_api = ("tp.GatherExchange.linear per linear (qmm_w8a16_perchannel_ex) with pinned-host activations copied in "
                   "and the gathered `down` output copied out every step; CUDA events, max over ranks")
        rt_down = None
    e2e_value = total_flops / (e2e_ms / args.steps * 1e-3) / 1e12

    status = lib.qmm_device_status()
    if status != 0:
        raise SystemExit(f"device status word is 0x{status:x}: a kernel gave up waiting")

    # ---- parity of what was just timed (outside the timed region) -----------------
    checked, worst_err, n_rows = check_last_layer(torch, dist, ex, weights[-1], last_slot, acts, rank, world, device)
    if rt_down is not None:
        # the runtime path ran the same last layer on the same inputs: bit-identical to the direct path
        same = bool(torch.equal(rt_down.to(device), ex.out("down", last_slot)[0]))
        checked = checked and same
        if not same:
            print("[rank 0] the runtime path's output differs from the direct path's", file=sys.stderr)
    if not checked:
        print(f"[rank {rank}] PARITY CHECK FAILED: max relative error {worst_err:.3e}", file=sys.stderr)

    line = None
    if rank == 0:
        peak = peaks["bf16_tflops_sustained"]
        # average launch duration over the timed region (CUDA events on the launching stream; the
        # launches overlap each other's tails, so they are not timed one by one)
        launch_ms = ms_per_step * args.steps / max(1, timed_launches)
        achieved = rank_flops * args.steps / max(1, timed_launches) / (launch_ms * 1e-3) / 1e12
        traffic, how = 0.0, set()
        for _, k, _, ns, _, _, _ in weights[0]:
            b, h = launch_traffic(k, ns)
            how.add(h)
            traffic = None if (b is None or traffic is None) else traffic + b / len(weights[0])
        if ex.mode == "fused":
            par = ("weights column-sharded along N; the GEMM epilogue stores each output element once with "
                   "multimem.st to an NVSwitch multicast address, which places it in block r of every rank's "
                   "[P, M, N/P] buffer (no separate all-gather); per-launch completion signals, bounded wait "
                   "for all of them at the end of a step")
        elif ex.mode == "mcast":
            par = ("weights column-sharded along N; every finished [M, N/P] block is copied to the NVSwitch multicast "
                   "address of the gathered [P, M, N/P] buffer by a small kernel (--copy-ctas CTAs) on a side stream (multimem.st, "
                   "512-byte runs), overlapped with the next GEMMs, which leave those SMs free; per-launch completion "
                   "signals, bounded wait for all of them at the end of a step")
        elif ex.mode == "peer":
            par = ("weights column-sharded along N; every finished [M, N/P] block is stored into every peer's gathered "
                   "[P, M, N/P] buffer over NVLink by a small kernel (--copy-ctas CTAs) on a side stream, overlapped "
                   "with the next GEMMs, which leave those SMs free; per-launch completion signals, bounded wait for "
                   "all of them at the end of a step")
        elif ex.mode == "copy":
            par = ("weights column-sharded along N; outputs gathered into [P, M, N/P] by copy-engine peer copies "
                   "of each finished [M, N/P] block into every peer's symmetric buffer, overlapped on side "
                   "streams, one 4-byte NCCL all-reduce per step as the rendezvous")
        elif ex.mode == "collective":
            par = "weights column-sharded along N; outputs gathered by NCCL all-gather overlapped on a second stream"
        else:
            par = "single GPU" + (f", rank 0's share of a {shard_world}-way sharded run (no exchange)" if shard_world > 1 else "")
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world, layers),
            "exchange": {"mode": ex.mode, "detail": par, "chosen_by_timing": tuned},
            "checked": checked,
            "check": {"rows": n_rows, "linears": 4, "max_rel_err": worst_err, "tolerance": 1e-2,
                      "what": "last layer's four gathered outputs, four rows of every 256-row tile, all columns, "
                              "against the CPU oracle of the unsharded linear, on every rank"},
            "roofline": {"bound": "tensor", "kernel": "w8a16_kernel (tcgen05 kind::f16, in-kernel int8->bf16)",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_source": f"{peaks['source']} bf16_tflops_sustained (burst {peaks['bf16_tflops']})",
                         "launch_ms_mean": launch_ms,
                         "traffic": traffic, "traffic_unit": "DRAM bytes per launch (mean of a layer's four)",
                         "traffic_source": "+".join(sorted(how))},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": e2e_api},
            "gpu_launches": timed_launches,
            "clocks": clocks,
        }
        if ex.why_not_fused:
            line["exchange"]["note"] = ex.why_not_fused
    if world == 1 and rank == 0 and not args.no_detail:
        time.sleep(2.0)  # let the power-capped clocks of the timed region recover before the small kernels
        del weights, ex
        if rt_down is not None:
            for bufs in layer_bufs:
                for b in bufs:
                    b.destroy()
            del layer_bufs, bufs, exe
            rt.destroy()
        torch.cuda.empty_cache()
        line["detail"] = run_detail(torch, ops, synthetic, lib, device, peaks)
        base, _ = cpu_linears_tflops(steps=6, warmup=1)
        line["cpu_baseline"] = base
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if checked else 1


def run_detail(torch, ops, synthetic, lib, device, peaks, items=None):
    """The other workloads of the path.  The kernels here run for microseconds,
    so a sequence of launches is captured in a CUDA graph and the graph is
    replayed: the device time per launch is then free of host launch overhead.
    Timing is by CUDA events on the replaying stream."""
    detail = {}
    hbm = peaks["hbm_gbs"]
    stream = torch.cuda.Stream()
    want = (lambda name: True) if not items else (lambda name: name in items)

    def graph_time(launch, n_launches, replays=20, warm_replays=3):
        """launch(i) issues the i-th kernel; returns mean microseconds per kernel."""
        with torch.cuda.stream(stream):
            launch(0)  # first call outside capture (function attributes, lazy init)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(n_launches):
                    launch(i)
            for _ in range(warm_replays):
                g.replay()
            stream.synchronize()
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(replays):
                g.replay()
            e1.record(stream)
            stream.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (replays * n_launches)

    if want("int4_decode"):
        _detail_int4_decode(torch, ops, synthetic, lib, device, hbm, graph_time, detail)
    if want("int4_prefill"):
        _detail_int4_prefill(torch, ops, synthetic, device, peaks, detail)
    if want("int8_dot"):
        _detail_int8_dot(torch, synthetic, lib, device, peaks, graph_time, detail)
    if items is not None and "operator_api_sweep" in items:  # not part of the default run
        _detail_operator_api_sweep(torch, synthetic, lib, device, graph_time, detail)
    if items is not None and "int4_decode_sweep" in items:  # not part of the default run
        _detail_int4_sweep(torch, ops, synthetic, lib, device, graph_time, detail)
    if want("llama_decode"):
        _detail_llama_decode(torch, synthetic, device, hbm, stream, detail)
    if want("operator_api"):
        _detail_operator_api(torch, synthetic, lib, device, hbm, graph_time, detail)
    if want("small_f32"):
        _detail_small_f32(torch, synthetic, lib, device, hbm, graph_time, detail)
    return detail


def _detail_int4_decode(torch, ops, synthetic, lib, device, hbm, graph_time, detail):
    # decode int4 g128 GEMV: rotate through enough weight copies that no launch finds its weights in L2
    K, N, G = 4096, 14336, 32
    copies = 12  # 12 x 30.5 MB > 2 x L2
    gen = synthetic.torch_generator(device, 3, 0)
    wqs = [torch.randint(0, 256, (K // 2, N), dtype=torch.uint8, device=device, generator=gen) for _ in range(copies)]
    sc = synthetic.device_uniform((G, N), 0.002, 0.01, device, gen, torch.bfloat16)
    zp = torch.randint(0, 256, (G, N // 2), dtype=torch.uint8, device=device, generator=gen)
    ws = torch.zeros(lib.qmm_w4a16_g128_workspace_bytes(16, N, K), dtype=torch.uint8, device=device)
    for M in (1, 4, 16):
        x = synthetic.device_normal((M, K), device, gen, torch.bfloat16)
        y = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        us = graph_time(lambda i: ops.w4a16_g128(x, wqs[i % copies], sc, zp, zeros_packed=True, out=y, workspace=ws,
                                                   static_weights=True),
                        copies * 2)
        us_warm = graph_time(lambda i: ops.w4a16_g128(x, wqs[0], sc, zp, zeros_packed=True, out=y, workspace=ws,
                                                        static_weights=True),
                             copies * 2)
        nbytes = K * N // 2 + G * N * 2 + G * N // 2 + M * K * 2 + M * N * 2
        gbs = nbytes / (us * 1e-6) / 1e9
        detail[f"int4_g128_decode_M{M}"] = {
            "us": us, "bytes": nbytes, "GB/s": gbs, "frac_of_measured_hbm": gbs / hbm, "frac_of_8TBs": gbs / 8000.0,
            "us_warm_l2_single_copy": us_warm,
            "note": f"{copies} rotating weight copies (cold L2), zero points packed 4-bit, CUDA-graph replay"}
    del wqs


def _detail_int4_prefill(torch, ops, synthetic, device, peaks, detail):
    # int4 g128 weight-only matmul at prefill sizes: the tcgen05 GEMM with in-kernel nibble dequantisation
    K, N, G = 4096, 14336, 32
    gen = synthetic.torch_generator(device, 3, 50)
    copies = 6  # 6 x 29 MB of packed weights; the activations (33 MB at M = 4096) add to the L2 pressure
    wqs = [torch.randint(0, 256, (K // 2, N), dtype=torch.uint8, device=device, generator=gen) for _ in range(copies)]
    sc = synthetic.device_uniform((G, N), 0.002, 0.01, device, gen, torch.bfloat16)
    zp = torch.randint(0, 256, (G, N // 2), dtype=torch.uint8, device=device, generator=gen)
    for M in (512, 4096):
        x = synthetic.device_normal((M, K), device, gen, torch.bfloat16)
        y = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        for i in range(3):
            ops.w4a16_g128(x, wqs[i % copies], sc, zp, zeros_packed=True, out=y)
        torch.cuda.synchronize()
        reps = 24
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            ops.w4a16_g128(x, wqs[i % copies], sc, zp, zeros_packed=True, out=y)
        e1.record()
        e1.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        tf = 2.0 * M * K * N / (us * 1e-6) / 1e12
        detail[f"int4_g128_prefill_M{M}"] = {
            "us": us, "TFLOP/s": tf, "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"],
            "note": "w8a16_kernel<4>: tcgen05 kind::f16 after in-kernel nibble dequantisation; back-to-back launches "
                    "(dependent, so they do not overlap), rotating weight copies"}
    del wqs


def _detail_int4_sweep(torch, ops, synthetic, lib, device, graph_time, detail):
    # M = 1 int4 g128 matmul over a range of sizes: time = fixed cost + bytes / streaming rate
    gen = synthetic.torch_generator(device, 3, 7)
    ws = torch.zeros(lib.qmm_w4a16_g128_workspace_bytes(8, 28672, 16384), dtype=torch.uint8, device=device)
    rows = []
    for K, N in [(128, 256), (2048, 14336), (4096, 14336), (8192, 14336), (16384, 14336), (4096, 4096), (4096, 28672)]:
        G = K // 128
        copies = max(2, min(12, (300 << 20) // max(1, K * N // 2)))
        wqs = [torch.randint(0, 256, (K // 2, N), dtype=torch.uint8, device=device, generator=gen) for _ in range(copies)]
        sc = synthetic.device_uniform((G, N), 0.002, 0.01, device, gen, torch.bfloat16)
        zp = torch.randint(0, 256, (G, N // 2), dtype=torch.uint8, device=device, generator=gen)
        x = synthetic.device_normal((1, K), device, gen, torch.bfloat16)
        y = torch.empty((1, N), dtype=torch.bfloat16, device=device)
        us = graph_time(lambda i: ops.w4a16_g128(x, wqs[i % copies], sc, zp, zeros_packed=True, out=y, workspace=ws,
                                                   static_weights=True), copies * 2)
        nbytes = K * N // 2 + G * N * 2 + G * N // 2
        rows.append({"K": K, "N": N, "MB": nbytes / 1e6, "us": us, "TB/s": nbytes / us / 1e6})
        del wqs
    detail["int4_g128_decode_M1_size_sweep"] = rows


def _detail_operator_api_sweep(torch, synthetic, lib, device, graph_time, detail):
    # affine 4-bit g64, f16, M = 4 over a range of sizes: time = fixed cost + bytes / streaming rate
    gen = synthetic.torch_generator(device, 6, 9)
    st = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
    rows = []
    M, gs = 4, 64
    for K, N in [(4096, 2368), (4096, 14336), (4096, 28672), (8192, 28672), (8192, 57344)]:
        wbytes = N * K // 2
        copies = max(2, min(10, (300 << 20) // wbytes))
        x = synthetic.device_normal((M, K), device, gen, torch.float16)
        y = torch.empty((M, N), dtype=torch.float16, device=device)
        ws = [torch.randint(0, 256, (wbytes,), dtype=torch.uint8, device=device, generator=gen) for _ in range(copies)]
        sc = synthetic.device_uniform((N, K // gs), 0.002, 0.01, device, gen)
        bi = synthetic.device_uniform((N, K // gs), -0.05, 0.05, device, gen)

        def run(i):
            assert lib.qmm_affine_matmul(x.data_ptr(), ws[i % copies].data_ptr(), sc.data_ptr(), bi.data_ptr(),
                                         y.data_ptr(), M, N, K, 4, gs, 1, st()) == 0

        us = graph_time(run, copies * 2)
        nbytes = wbytes + 2 * N * (K // gs) * 4
        rows.append({"K": K, "N": N, "MB": nbytes / 1e6, "us": us, "TB/s": nbytes / us / 1e6})
        del ws
    detail["operator_api_affine_4bit_g64_M4_size_sweep"] = rows


def _detail_operator_api(torch, synthetic, lib, device, hbm, graph_time, detail):
    # the operator-API formats at a decode-sized shape: f16 activations [M, 4096] x packed weights [14336, 4096]
    M, K, N = 4, 4096, 14336
    gen = synthetic.torch_generator(device, 6, 0)
    x = synthetic.device_normal((M, K), device, gen, torch.float16)
    y = torch.empty((M, N), dtype=torch.float16, device=device)
    st = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
    QMM_F16 = 1
    cases = []
    for bits, gs in ((4, 64), (8, 64)):
        wbytes = N * K * bits // 8
        copies = max(2, (300 << 20) // wbytes)
        ws = [torch.randint(0, 256, (wbytes,), dtype=torch.uint8, device=device, generator=gen) for _ in range(copies)]
        sc = synthetic.device_uniform((N, K // gs), 0.002, 0.01, device, gen)
        bi = synthetic.device_uniform((N, K // gs), -0.05, 0.05, device, gen)

        def run(i, ws=ws, sc=sc, bi=bi, bits=bits, gs=gs, copies=copies):
            assert lib.qmm_affine_matmul(x.data_ptr(), ws[i % copies].data_ptr(), sc.data_ptr(), bi.data_ptr(),
                                         y.data_ptr(), M, N, K, bits, gs, QMM_F16, st()) == 0

        cases.append((f"affine_{bits}bit_g{gs}", run, copies, wbytes + 2 * N * (K // gs) * 4))
    for mode, name, gs, wb in ((0, "mxfp4", 32, 4), (1, "mxfp8", 32, 8), (2, "nvfp4", 16, 4)):
        wbytes = N * K * wb // 8
        copies = max(2, (300 << 20) // wbytes)
        # element codes and scale codes below the NaN patterns
        ws = [torch.randint(0, 0x70, (wbytes,), dtype=torch.uint8, device=device, generator=gen) for _ in range(copies)]
        sc = torch.randint(0x70, 0x7C, (N, K // gs), dtype=torch.uint8, device=device, generator=gen)

        def run(i, ws=ws, sc=sc, mode=mode, copies=copies):
            assert lib.qmm_mx_matmul(x.data_ptr(), ws[i % copies].data_ptr(), sc.data_ptr(), y.data_ptr(), M, N, K,
                                     mode, QMM_F16, st()) == 0

        cases.append((name, run, copies, wbytes + N * (K // gs)))
    for name, run, copies, nbytes in cases:
        us = graph_time(run, copies * 2)
        detail[f"operator_api_{name}_M{M}_{N}x{K}"] = {
            "us": us, "bytes": nbytes, "GB/s": nbytes / (us * 1e-6) / 1e9,
            "frac_of_measured_hbm": nbytes / (us * 1e-6) / 1e9 / hbm,
            "note": ("affine_ring_kernel" if name.startswith("affine") else "mx_ring_kernel") +
                    " (mma.sync on the packed codes, per-warp TMA rings); rotating weight copies (cold L2), CUDA-graph replay"}


def _detail_int8_dot(torch, synthetic, lib, device, peaks, graph_time, detail):
    # int8 x int8 -> int32 with fused rescale
    Mi, Ki, Ni = 2048, 4096, 4096
    gen = synthetic.torch_generator(device, 2, 0)
    a = synthetic.device_int8((Mi, Ki), device, gen)
    bs = [synthetic.device_int8((Ki, Ni), device, gen) for _ in range(10)]  # 160 MB of B operands
    row = synthetic.device_uniform((Mi,), 0.01, 0.05, device, gen)
    col = synthetic.device_uniform((Ni,), 0.005, 0.02, device, gen)
    out = torch.empty((Mi, Ni), dtype=torch.float32, device=device)

    def run_i8(i):
        st = lib.qmm_i8i8_i32(a.data_ptr(), bs[i % 10].data_ptr(), None, row.data_ptr(), col.data_ptr(),
                              out.data_ptr(), Mi, Ni, Ki, 0, 0, torch.cuda.current_stream().cuda_stream)
        assert st == 0

    us = graph_time(run_i8, 20, replays=10)
    tops = 2.0 * Mi * Ni * Ki / (us * 1e-6) / 1e12
    lib_peak = _int8_library_peak(torch, device)
    detail["int8_library_peak"] = lib_peak
    detail["int8_dot_2048x4096x4096_f32_rescale"] = {
        "us": us, "TOP/s": tops, "frac_of_measured_int8": tops / lib_peak["burst_TOPs"] if lib_peak.get("burst_TOPs") else None,
        "frac_of_2x_measured_bf16_burst": tops / (2 * peaks["bf16_tflops"]),
        "note": "fused float(acc)*row*col epilogue, f32 output only; 10 rotating B operands; measured int8 peak = "
                "the library int8 GEMM of int8_library_peak (burst, as this kernel is timed in isolation)"}
    del bs
    # the same M and N at four times the K: separates the per-launch fixed cost from the main-loop rate
    Kl = 16384
    al = synthetic.device_int8((Mi, Kl), device, gen)
    bl = [synthetic.device_int8((Kl, Ni), device, gen) for _ in range(3)]  # 192 MB of B operands

    def run_long(i):
        st = lib.qmm_i8i8_i32(al.data_ptr(), bl[i % 3].data_ptr(), None, row.data_ptr(), col.data_ptr(),
                              out.data_ptr(), Mi, Ni, Kl, 0, 0, torch.cuda.current_stream().cuda_stream)
        assert st == 0

    us_l = graph_time(run_long, 6, replays=10)
    tops_l = 2.0 * Mi * Ni * Kl / (us_l * 1e-6) / 1e12
    detail["int8_dot_2048x16384x4096_f32_rescale"] = {
        "us": us_l, "TOP/s": tops_l,
        "frac_of_measured_int8": tops_l / lib_peak["burst_TOPs"] if lib_peak.get("burst_TOPs") else None,
        "frac_of_2x_measured_bf16_burst": tops_l / (2 * peaks["bf16_tflops"]),
        "main_loop_us_per_4096_k": (us_l - us) / 3.0, "fixed_us_per_launch": us - (us_l - us) / 3.0,
        "note": "context for the line above: same M and N, K x 4"}
    del bl


def _int8_library_peak(torch, device):
    """A library int8 GEMM (torch._int_mm, 8192^3, int32 result) as the int8 tensor-core denominator:
    best of 10 (burst) and back to back for 4 s (sustained), the recipe the bf16 peaks of
    MEASURED_PEAKS.json were taken with.  Timing only: nothing of it is on the product path."""
    n = 8192
    try:
        a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device)
        b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device)
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        ops_per = 2.0 * n * n * n
        reps = max(10, int(4000.0 / best))
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch._int_mm(a, b)
        e1.record()
        e1.synchronize()
        sustained = e0.elapsed_time(e1) / reps
        del a, b
        return {"burst_TOPs": ops_per / (best * 1e-3) / 1e12, "sustained_TOPs": ops_per / (sustained * 1e-3) / 1e12,
                "how": "torch._int_mm int8 8192^3 -> int32: best of 10 (burst), back to back for 4 s (sustained)"}
    except Exception as exc:  # noqa: BLE001
        return {"burst_TOPs": None, "sustained_TOPs": None, "how": f"torch._int_mm unavailable: {exc!r}"}


def _detail_llama_decode(torch, synthetic, device, hbm, stream, detail):
    # Llama-3-8B-shaped int4 decode step, batch 8, KV context 2048 (random weights and cache)
    from jax_metallib_b200.decode_stack import DecodeStep, LlamaShape, random_model

    shape = LlamaShape()
    B, L = 8, 2048
    model = random_model(shape, device, seed=4000)
    gen = synthetic.torch_generator(device, 4, 1)
    kc = [torch.randn((B, shape.n_kv_heads, L, shape.head_dim), device=device, generator=gen).to(torch.bfloat16)
          for _ in range(shape.n_layers)]
    vc = [torch.randn((B, shape.n_kv_heads, L, shape.head_dim), device=device, generator=gen).to(torch.bfloat16)
          for _ in range(shape.n_layers)]
    step = DecodeStep(shape, model, B, L, device)
    step.ids.copy_(torch.randint(0, shape.vocab, (B,), device=device, generator=gen).to(torch.int32))
    g = step.capture(kc, vc)
    with torch.cuda.stream(stream):
        for _ in range(3):
            g.replay()
        stream.synchronize()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        reps = 20
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1) / reps
    step_bytes = shape.weight_bytes_per_step(B, L)
    detail["llama3_8b_int4_decode_b8_ctx2048"] = {
        "ms_per_step": ms, "tokens_per_s": B / (ms * 1e-3), "launches_per_step": step.launches_per_step,
        "bytes_per_step": step_bytes, "GB/s": step_bytes / (ms * 1e-3) / 1e9,
        "frac_of_measured_hbm": step_bytes / (ms * 1e-3) / 1e9 / hbm,
        "ceiling_tokens_per_s_at_measured_hbm": B / (step_bytes / (hbm * 1e9)),
        "note": "one CUDA-graph replay per step: embedding gather, 32 layers (7 int4 g128 linears as 4 launches: q|k|v and gate|up side by side along N; RMSNorm, RoPE, "
                "GQA attention over a read-only bf16 KV cache, SwiGLU), final norm and bf16 lm_head all inside the "
                "timed step; the step returns logits and the new K/V rows; 6.8 GB touched per step exceeds L2"}
    del model, kc, vc, step, g
    torch.cuda.empty_cache()


def _detail_small_f32(torch, synthetic, lib, device, hbm, graph_time, detail):
    # small f32 case (launch-latency bound)
    c = synthetic.config1()
    x1 = torch.from_numpy(c["x"]).to(device)
    w1 = torch.from_numpy(c["w"]).to(device)
    s1 = torch.from_numpy(c["scale"]).to(device)
    y1 = torch.empty((32, 1024), dtype=torch.float32, device=device)

    def run_c1(i):
        st = lib.qmm_w8a32_perchannel(x1.data_ptr(), w1.data_ptr(), s1.data_ptr(), y1.data_ptr(), 32, 1024, 1024,
                                      torch.cuda.current_stream().cuda_stream)
        assert st == 0

    us = graph_time(run_c1, 50)
    nbytes = 32 * 1024 * 4 * 2 + 1024 * 1024 + 4096
    detail["int8_weight_only_f32_32x1024x1024"] = {
        "us": us, "GB/s": nbytes / (us * 1e-6) / 1e9, "frac_of_measured_hbm": nbytes / (us * 1e-6) / 1e9 / hbm,
        "note": "1.3 MB problem (fits L2): back-to-back launches in a CUDA graph; latency bound"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=N_LAYERS, help="layers in the pass (the workload names 80)")
    ap.add_argument("--copy-ctas", type=int, default=MCAST_CTAS,
                    help="SMs left to the multicast copy kernel of --exchange mcast (the GEMM keeps the rest)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "fused", "mcast", "peer", "copy", "collective"],
                    help="how the outputs are gathered at N > 1 (auto: fused multimem stores when the symmetric "
                         "allocation has a multicast address, else peer copies, else the NCCL all-gather)")
    ap.add_argument("--shard-of", type=int, default=1, choices=[1, 2, 4, 8],
                    help="single GPU only: run rank 0's share of a P-way sharded pass (no exchange)")
    ap.add_argument("--no-detail", action="store_true", help="skip the per-workload detail and the CPU baseline")
    ap.add_argument("--detail-only", action="store_true",
                    help="run only the per-workload detail (small case for profiling) and print it as JSON")
    ap.add_argument("--detail-items", default="",
                    help="comma-separated subset of int4_decode,int4_prefill,int8_dot,llama_decode,operator_api,small_f32 (and int4_decode_sweep, operator_api_sweep, "
                         "which is not part of the default run)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    pin_host_threads()  # the CPU baseline leg uses every host core whatever the launcher exported
    if args.detail_only:
        import torch

        from jax_metallib_b200 import _lib, ops, synthetic

        device = torch.device("cuda", 0)
        torch.cuda.set_device(device)
        items = [x for x in args.detail_items.split(",") if x] or None
        print(json.dumps({"detail": run_detail(torch, ops, synthetic, _lib.load(), device, measured_peaks(), items)}))
        return 0
    return run_gpu(args)


if __name__ == "__main__":
    sys.exit(main())
