"""Benchmark: 27B-class Q4_K_M decode tokens/s through the packed-quant matmul path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A *step* is one decode token step (batch B, default 1) through the 64-layer stack of
``ferric_b200.stack`` -- per layer the fused q|k|v, o, gate|up+SwiGLU (Q4_K) and down (Q6_K)
products with their norms; 13.36 GB of weights streamed per step, sharded tensor-parallel over N
GPUs with two f32 all-reduces per layer.  Weights are synthetic (random-init blocks of the named
shapes and value distributions, generated on the device); the working set per GPU is far larger
than L2, so every step reads its weights from HBM.

Prints ONE JSON line (rank 0).  `value` is device-timed with inputs resident; `e2e` is the same
step driven through host buffers (pinned-host -> device copy of the activations, device -> host
read of the result, every step).  `roofline` is measured live for the dominant kernel, the Q4_K
gate|up GEMV.  `cpu_baseline` times the CPU oracle port on this box's host cores on a bounded
sample.  ``--impl reference`` runs only that CPU path, in the same units.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_LAYERS, HIDDEN, N_FF, Q_OUT, KV_OUT = 64, 5120, 17408, 5120, 1024
WORKLOAD = ("configs[4] at batch {b}: 64 x configs[1] layer (q|k|v 7168x5120, o 5120x5120, gate|up 34816x5120 Q4_K; "
            "down 5120x17408 Q6_K), f32 activations")
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch kernels directly instead of replaying a CUDA graph")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-matrix table")
    ap.add_argument("--shard-of", type=int, default=0, metavar="N",
                    help="diagnostic, 1 GPU only: time rank 0's shard of an N-way tensor-parallel plan with the exchange "
                         "replaced by nothing (what N GPUs would reach if the exchange were free); not a valid result")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--no-chain", action="store_true",
                    help="launch the norms and activation preparation as kernels of their own (8 launches per layer) instead of "
                         "inside the products' launches (4 per layer)")
    ap.add_argument("--chain", action="store_true", help="force the chained form wherever it applies (also across ranks)")
    ap.add_argument("--no-parity", action="store_true", help="N > 1: skip the sharded-against-unsharded parity stage")
    ap.add_argument("--prefill", type=int, default=0, metavar="M",
                    help="time only the tensor-core prefill product (Q4_K x bf16, M activation rows) and print its line")
    ap.add_argument("--prefill-rows", type=int, default=17408, help="weight rows of the --prefill matrix")
    ap.add_argument("--prefill-cols", type=int, default=5120, help="columns (K) of the --prefill matrix")
    ap.add_argument("--prefill-type", type=int, default=12, choices=[12, 13, 14, 8], help="ggml type of the --prefill matrix")
    ap.add_argument("--allreduce", default="auto", choices=["auto", "push", "fused", "wide", "nccl"],
                    help="N > 1: the library's own exchange over peer memory (push: the products store into every rank's memory; "
                         "fused: signalled buffers read by the peers; wide: the two-step pushed all-reduce of the batched decode path, batch > 8), "
                         "NCCL through torch.distributed, or (default) the library's own")
    return ap.parse_args()


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ------------------------------------------------------------------------------------------------
# CPU leg: the oracle port of the reference's CPU path, all host threads, on a bounded sample.
# ------------------------------------------------------------------------------------------------
class CpuLayer:
    """ONE layer's four products on the host cores through the oracle port (weights built once)."""

    def __init__(self, batch: int):
        from ferric_b200 import synth
        from oracle import oracle as O

        self.O, self.cores, self.batch = O, os.cpu_count() or 1, batch
        mats = [(synth.GGML_Q4_K, Q_OUT + 2 * KV_OUT, HIDDEN), (synth.GGML_Q4_K, HIDDEN, Q_OUT),
                (synth.GGML_Q4_K, 2 * N_FF, HIDDEN), (synth.GGML_Q6_K, HIDDEN, N_FF)]
        self.data = [(ty, r, c, synth.matrix(ty, r, c, seed=4 + i), synth.activations(batch, c, seed=4 + i))
                     for i, (ty, r, c) in enumerate(mats)]

    def seconds(self, mode_name: str = "dequant_dot", threads: int = 0) -> float:
        O = self.O
        mode = {"dequant_dot": O.MODE_DEQUANT_DOT, "fused": O.MODE_FUSED}[mode_name]
        t0 = time.perf_counter()
        for ty, r, c, raw, x in self.data:
            y = O.matmul_q(raw, ty, r, c, x, threads=threads or self.cores, mode=mode)
            if r == 2 * N_FF:
                O.swiglu(y, N_FF)
        return time.perf_counter() - t0


def run_reference(args):
    """`--impl reference`: the reference's CPU implementation of the path (oracle port; the Rust
    reference cannot be built in this image), timed on the host cores in the bench's own units."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    batch = args.batch
    times = []
    layer = CpuLayer(batch)
    cores = layer.cores
    spent = 0.0
    for i in range(args.warmup + args.steps):
        t = layer.seconds()
        spent += t
        if i >= args.warmup:
            times.append(t)
        if spent > 120 and len(times) >= 3:  # keep the whole run within a few minutes
            break
    per_layer = statistics.median(times)
    step_s = per_layer * args.layers
    value = batch / step_s
    sample = (f"1 of {args.layers} layers per step (4 products, 208.8 MB of weights), dequantise-then-dot order, "
              f"{cores} threads; step time = {args.layers} x layer time")
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        # the same workload keys as the GPU arm's line (the host cores run the unsharded layer whatever --gpus says)
        "config": {"workload": WORKLOAD.format(b=batch), "batch": batch, "layers": args.layers, "parallelism": f"tp{args.gpus}",
                   "host": f"cpu, {cores} threads"},
        "sampled_ms_per_step": per_layer * 1e3,
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# clocks during the timed region (read-only NVML queries)
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self._nv:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    from ferric_b200 import Context, QMatrix, TPGroup
    from ferric_b200.stack import DecodeStack, TPPlan

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback on this path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG", "WARN")   # quiet by default; a caller's own setting (e.g. INFO) is kept
        # No NVLink multicast bindings: nothing here needs in-switch reduction, and a rank must never leave while its
        # memory is bound to a multicast object.
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    ctx = Context(local)
    plan = TPPlan.make(world, rank, HIDDEN, N_FF, Q_OUT, KV_OUT)
    if args.shard_of > 1 and world == 1:
        plan = TPPlan.make(args.shard_of, 0, HIDDEN, N_FF, Q_OUT, KV_OUT)
    def exchange_for(batch):
        """(all_reduce callable, exchange group, name) for a batch size.  `auto`: the library's own pushed exchange
        up to batch 4 (up to batch 8 from 4 GPUs on: measured 1306 against 1027 tokens/s at 8 GPUs, but 904 against 957
        at 2), NCCL above that."""
        if world == 1:
            if args.shard_of > 1 and args.chain and batch <= 4:
                # diagnostic: rank 0's shard with the chained pushed exchange, the "group" being this rank alone
                grp = TPGroup(ctx, 0, 1, batch, HIDDEN)
                grp.connect([grp.export()])
                return None, grp, "push"
            return ((lambda t: None) if args.shard_of > 1 else None), None, "none"
        kind = args.allreduce
        if kind == "auto":
            kind = "push" if batch <= (8 if world >= 4 else 4) else "wide" if batch > 8 else "nccl"
        if batch > 8 and kind in ("push", "fused"):
            kind = "wide"        # the GEMV's exchanges serve up to 8 rows
        if kind == "nccl":
            return (lambda t: dist.all_reduce(t)), None, kind
        grp = TPGroup(ctx, rank, world, batch, HIDDEN)
        grp.connect_with_torch_distributed()
        return None, grp, kind

    chain = False if args.no_chain else (True if args.chain else None)
    parity = None
    if world > 1 and not args.no_parity:
        parity = tp_parity_check(torch, dist, ctx, world, rank, dev, exchange_for, chain)

    allreduce, group, ar_name = exchange_for(B)
    stack = DecodeStack(ctx, plan, n_layers=args.layers, batch=B, all_reduce=allreduce, group=group, push=(ar_name == "push"),
                        chain=chain)
    stack.build_synthetic(seed=4)
    g = torch.Generator(device=dev).manual_seed(4)
    x0 = torch.randn((B, HIDDEN), device=dev, generator=g)
    if world > 1:
        dist.broadcast(x0, 0)
    stack.h.copy_(x0)
    # Captured graphs hold the address of the context's activation scratch, and growing the scratch moves it:
    # size it once for the largest batch measured below, before anything is captured.
    L0 = stack.layers[0]
    ctx.reserve_scratch(max(w.scratch_bytes(max(B, 64)) for w in (L0.wqkv, L0.wo, L0.wgu, L0.wdown)))
    if not args.no_graph:
        stack.capture()
    else:
        stack.step()
    launches_per_step = stack.launches_per_step

    # ---- device-timed: inputs resident ----------------------------------------------------
    for _ in range(W):
        stack.h.copy_(x0)
        stack.run()
    # The K-step block is timed (CUDA events, max over ranks) as often as fills half a second, at least three times;
    # the reported step time is the median block.
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    block_ms = []
    with ClockSampler(local) as clocks:
        while len(block_ms) < 3 or (sum(block_ms) < 500.0 and len(block_ms) < 25):
            barrier()
            ev0.record()
            for _ in range(K):
                stack.run()
            ev1.record()
            torch.cuda.synchronize(dev)
            barrier()
            block_ms.append(max_over_ranks(ev0.elapsed_time(ev1)))
    elapsed_ms = statistics.median(block_ms)
    finite = bool(torch.isfinite(stack.h).all().item())
    if group is not None:
        group.check()      # raises if any bounded wait on a peer ran out
    ms_per_step = elapsed_ms / K
    value = B * 1e3 / ms_per_step

    # ---- the other batch sizes of the configuration, same weights, same timing rules ------------
    other_batches = {}
    if not args.no_extras:
        for b in (1, 8, 64):
            if b == B:
                continue
            ar2, g2, name2 = exchange_for(b)
            st2 = DecodeStack(ctx, plan, n_layers=args.layers, batch=b, all_reduce=ar2, group=g2, push=(name2 == "push"), chain=chain)
            for L in stack.layers:
                st2.add_layer(L.wqkv, L.wo, L.wgu, L.wdown)
            st2.reserve()
            xb = torch.randn((b, HIDDEN), device=dev, generator=g)
            if world > 1:
                dist.broadcast(xb, 0)
            st2.h.copy_(xb)
            if not args.no_graph:
                st2.capture()
            for _ in range(3):
                st2.h.copy_(xb)
                st2.run()
            barrier()
            k2 = max(5, min(K, 20))
            ev0.record()
            for _ in range(k2):
                st2.run()
            ev1.record()
            torch.cuda.synchronize(dev)
            barrier()
            ms2 = max_over_ranks(ev0.elapsed_time(ev1)) / k2
            if g2 is not None:
                g2.check()
            other_batches[str(b)] = {"tokens_per_s": b * 1e3 / ms2, "ms_per_step": ms2, "steps": k2, "all_reduce": name2,
                                     "launches_per_step": int(st2.launches_per_step),
                                     "finite": bool(torch.isfinite(st2.h).all().item())}
            st2.layers = []     # the matrices belong to the first stack
            st2.graph = None
            del st2

    # ---- end to end: host buffers in and out, every step -----------------------------------
    xh = torch.empty((B, HIDDEN), dtype=torch.float32).pin_memory()
    yh = torch.empty((B, HIDDEN), dtype=torch.float32).pin_memory()
    xh.copy_(x0.cpu())
    for _ in range(3):
        stack.step_host(xh, yh)
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        stack.step_host(xh, yh)
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    e2e = {"value": B * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": xh.numel() * 4,
           "d2h_bytes_per_step": yh.numel() * 4, "ms_per_step": e2e_s * 1e3 / K}

    # ---- roofline of the dominant kernel: the Q4_K gate|up GEMV with the SwiGLU epilogue ----
    # 64 distinct 100 MB matrices in turn (always cold in L2), launched from a CUDA graph so the host
    # is out of the loop; CUDA events on the launching stream bracket 3 replays.
    peak, peak_kind = measured_peak()
    L0 = stack.layers[0]
    xr = torch.randn((B, HIDDEN), device=dev, generator=g)
    if B > 8:      # the tensor-core decode kernel prepares its own activation form: time the whole product
        def gate_up_pass():
            for L in stack.layers:
                L.wgu.try_matmul_swiglu(xr, out=stack.f)
        roof_kernel = "tc_prep_kernel + gemv_tc_kernel + tc_finish_kernel<swiglu>"
    else:
        m = L0.wgu.prepare(xr)

        def gate_up_pass():
            for L in stack.layers:
                L.wgu.matmul_prepared(m, out=stack.f, swiglu=True)
        roof_kernel = "gemv_q4k_kernel<swiglu>"

    with ClockSampler(local) as roof_clocks:
        us_per_launch = graph_time_us(torch, ctx, gate_up_pass, reps=9) / len(stack.layers)
    algo_bytes = L0.wgu.nbytes() + B * HIDDEN * 4 + B * plan.ff_rows * 4
    achieved = algo_bytes / (us_per_launch * 1e-6) / 1e9
    traffic = None
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            t = json.load(f).get("gemv_q4k_swiglu", {})
            if t.get("rows") == L0.wgu.rows() and t.get("cols") == L0.wgu.cols() and t.get("m") == B:
                traffic = t.get("dram_bytes_per_launch")
    except Exception:
        pass
    roofline = {"kernel": roof_kernel, "shape": [L0.wgu.rows(), L0.wgu.cols(), B], "bound": "hbm",
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_kind,
                "algorithmic_bytes_per_launch": algo_bytes, "us_per_launch": us_per_launch, "traffic": traffic,
                "timing": "median of 9 graph replays of 64 launches over 64 distinct matrices", "clocks": roof_clocks.summary()}

    # whole-step HBM efficiency, for context: weight bytes per step per GPU / device time
    step_gbs = stack.weight_bytes_per_step() / (ms_per_step * 1e-3) / 1e9

    extras = None
    if rank == 0 and world == 1 and not args.no_extras:
        with ClockSampler(local) as extra_clocks:
            extras = per_matrix_table(torch, ctx, stack, QMatrix, B, peak)
            if B == 1 and stack.plan.world == 1:      # the same four products at 64 activation rows
                extras.update(per_matrix_table(torch, ctx, stack, QMatrix, 64, peak, suffix="_m64"))
            extras.update(other_configs(torch, ctx, QMatrix, peak))
            extras["prefill_q4k_bf16_34816x5120"] = {f"m{m}": prefill_case(torch, ctx, QMatrix, stack.layers[0].wgu, m, 9)
                                                     for m in (128, 512, 2048)}
            extras["prefill_q6k_bf16_5120x17408"] = {f"m{m}": prefill_case(torch, ctx, QMatrix, stack.layers[0].wdown, m, 9)
                                                     for m in (512, 2048)}
        extras["timing"] = "every entry: median of 9 individually timed replays (CUDA events)"
        extras["clocks"] = extra_clocks.summary()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        layer = CpuLayer(B)
        cores = layer.cores
        t_layer = min(layer.seconds() for _ in range(3))
        t_fused = min(layer.seconds("fused") for _ in range(2))
        t_one = layer.seconds(threads=1)
        cpu = {"value": B / (t_layer * args.layers), "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"1 of {args.layers} layers (208.8 MB of weights), best of 3, dequantise-then-dot order, "
                         f"{cores} threads; step time = {args.layers} x layer time",
               "fused_order_value": B / (t_fused * args.layers),
               "one_thread_value": B / (t_one * args.layers)}

    if rank == 0:
        line = {
            "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD.format(b=B), "batch": B, "layers": args.layers,
                       "parallelism": f"tp{world}", "cuda_graph": not args.no_graph,
                       "launch_form": ("chained: one launch per matrix, norms / residual adds / activation preparation inside them"
                                       if stack.chain else "one kernel per stage"),
                       "l2": f"{stack.weight_bytes_per_step() / 1e9:.2f} GB of weights per GPU per step, larger than L2",
                       "all_reduce": ar_name, **({"diagnostic": f"rank 0's shard of tp{args.shard_of}, no exchange: not a result"}
                                                  if args.shard_of > 1 and world == 1 else {})},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": int(launches_per_step * K), "launches_per_step": int(launches_per_step),
            "clocks": clocks.summary(), "step_weight_gbs_per_gpu": step_gbs, "output_finite": finite,
            "timed_blocks": {"blocks": len(block_ms), "ms_per_block_median": elapsed_ms, "ms_per_block_min": min(block_ms),
                             "ms_per_block_max": max(block_ms)},
            "parity_check": parity,
            "other_batches": other_batches,
            "extras": extras,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave in order: no captured graph (they may hold NCCL work), nothing in flight, then the collective teardown.
        # Tearing a process group down has been seen to block for minutes; a watchdog ends the process if it does.
        stack.graph = None
        barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        watchdog = threading.Timer(60.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
        torch.cuda.synchronize(dev)
        dist.destroy_process_group()
        watchdog.cancel()
        os._exit(0)        # the exchange groups' peer mappings are released with the process
    stack.close()


def tp_parity_check(torch, dist, ctx, world, rank, dev, exchange_for, chain):
    """N > 1, outside every timed region: two full-shape layers, cut into this run's shards, run through the exchange
    the timed run uses at batch 1, 8 and 64, against the same two layers run unsharded on rank 0.  The bytes are drawn
    on rank 0 and broadcast, so every rank cuts the same tensors.  Compared element by element, bar 1e-4 + 1e-3 |ref|:
    the stack's result, the RMS-normalised residual stream after the last layer (values of order one, like the
    activations the bar is stated for).  The raw residual stream grows to ~1e4 with these random-init weights, so an
    absolute 1e-4 on it would be below one f32 ulp; it is compared against 1e-4 + 1e-3 max|ref| instead."""
    from ferric_b200 import QMatrix, synth
    from ferric_b200.stack import DecodeStack, TPPlan

    layers = 2
    plan = TPPlan.make(world, rank, HIDDEN, N_FF, Q_OUT, KV_OUT)
    plan1 = TPPlan.make(1, 0, HIDDEN, N_FF, Q_OUT, KV_OUT)
    shapes = {"q": (12, Q_OUT, HIDDEN), "k": (12, KV_OUT, HIDDEN), "v": (12, KV_OUT, HIDDEN), "o": (12, HIDDEN, Q_OUT),
              "gate": (12, N_FF, HIDDEN), "up": (12, N_FF, HIDDEN), "down": (14, HIDDEN, N_FF)}

    def cut(raw, ty, rows, cols, row0, nrows, col0, ncols):
        vals, bb = synth.BLOCK[ty]
        return raw.view(rows, cols // vals, bb)[row0:row0 + nrows, col0 // vals:(col0 + ncols) // vals, :].contiguous().view(-1)

    def build(p, full):
        qkv = torch.cat([cut(full["q"], 12, Q_OUT, HIDDEN, p.q_row0, p.q_rows, 0, HIDDEN),
                         cut(full["k"], 12, KV_OUT, HIDDEN, p.kv_row0, p.kv_rows, 0, HIDDEN),
                         cut(full["v"], 12, KV_OUT, HIDDEN, p.kv_row0, p.kv_rows, 0, HIDDEN)])
        gu = torch.cat([cut(full["gate"], 12, N_FF, HIDDEN, p.ff_row0, p.ff_rows, 0, HIDDEN),
                        cut(full["up"], 12, N_FF, HIDDEN, p.ff_row0, p.ff_rows, 0, HIDDEN)])
        return (QMatrix.from_device_bytes(ctx, qkv, 12, p.q_rows + 2 * p.kv_rows, HIDDEN),
                QMatrix.from_device_bytes(ctx, cut(full["o"], 12, HIDDEN, Q_OUT, 0, HIDDEN, p.q_row0, p.q_rows), 12, HIDDEN, p.q_rows),
                QMatrix.from_device_bytes(ctx, gu, 12, 2 * p.ff_rows, HIDDEN),
                QMatrix.from_device_bytes(ctx, cut(full["down"], 14, HIDDEN, N_FF, 0, HIDDEN, p.ff_row0, p.ff_rows), 14, HIDDEN, p.ff_rows))

    sharded, whole = [], []
    for l in range(layers):
        full = {}
        for i, (name, (ty, r, c)) in enumerate(shapes.items()):
            t = synth.matrix_on_device(ty, r, c, 9000 + 16 * l + i, dev)
            dist.broadcast(t, 0)
            full[name] = t
        sharded.append(build(plan, full))
        if rank == 0:
            whole.append(build(plan1, full))
        del full
    result = {"world": world, "layers": layers, "batches": [], "all_reduce": {}, "worst_ratio": 0.0, "worst_ratio_maxnorm": 0.0,
              "bar": "worst_ratio: element-wise |sharded - unsharded| / (1e-4 + 1e-3 |unsharded|) on rank 0's normalised residual "
                     "stream after the layers (the stack's result); worst_ratio_maxnorm: max|sharded - unsharded| / "
                     "(1e-4 + 1e-3 max|unsharded|) on the raw residual stream"}
    g = torch.Generator(device=dev).manual_seed(77)
    for b in (1, 8, 64):
        x = torch.randn((b, HIDDEN), device=dev, generator=g)
        dist.broadcast(x, 0)
        ar, grp, name = exchange_for(b)
        st = DecodeStack(ctx, plan, n_layers=layers, batch=b, all_reduce=ar, group=grp, push=(name == "push"), chain=chain)
        for mats in sharded:
            st.add_layer(*mats)
        st.reserve()
        st.h.copy_(x)
        got = st.step().clone()
        got_n = st.xn.clone()
        torch.cuda.synchronize(dev)
        if grp is not None:
            grp.check()
        dist.barrier()
        if rank == 0:
            ref_st = DecodeStack(ctx, plan1, n_layers=layers, batch=b, chain=chain)
            for mats in whole:
                ref_st.add_layer(*mats)
            ref_st.reserve()
            ref_st.h.copy_(x)
            ref = ref_st.step().clone()
            ref_n = ref_st.xn.clone()
            torch.cuda.synchronize(dev)
            ratio = float(((got_n - ref_n).abs().double() / (1e-4 + 1e-3 * ref_n.abs().double())).max().item())
            ratio_max = float(((got - ref).abs().double().max() / (1e-4 + 1e-3 * ref.abs().max().double())).item())
            result["worst_ratio"] = max(result["worst_ratio"], ratio)
            result["worst_ratio_maxnorm"] = max(result["worst_ratio_maxnorm"], ratio_max)
            ref_st.layers = []
        result["batches"].append(b)
        result["all_reduce"][str(b)] = name + ("+chain" if st.chain else "")
        st.layers = []
        dist.barrier()
    for mats in sharded + whole:
        for w in mats:
            w.close()
    flag = torch.tensor([result["worst_ratio"]], dtype=torch.float64, device=dev)
    dist.broadcast(flag, 0)
    result["worst_ratio"] = float(flag.item())
    result["ok"] = bool(result["worst_ratio"] <= 1.0)
    return result


def graph_time_us(torch, ctx, fn, reps=9):
    """Microseconds for one call of `fn` (a sequence of launches on the context), replayed from a CUDA graph: 3 warm-up
    replays, then the median of `reps` (at least 9) replays, each bracketed by its own pair of CUDA events."""
    dev = ctx.device
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        ctx.use_torch_stream()
        fn()
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        ctx.use_torch_stream()
        fn()
    ctx.use_torch_stream()
    for _ in range(3):
        gr.replay()
    torch.cuda.synchronize(dev)
    reps = max(reps, 9)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    for e0, e1 in evs:
        e0.record()
        gr.replay()
        e1.record()
    torch.cuda.synchronize(dev)
    return statistics.median(e0.elapsed_time(e1) for e0, e1 in evs) * 1e3


def per_matrix_table(torch, ctx, stack, QMatrix, B, peak, suffix=""):
    """GB/s of each product of the layer (prepare + product), cold: cycling over all layers' copies.  With a suffix the
    table is taken at that many activation rows on buffers of its own (the tensor-core decode kernel's range)."""
    out = {}
    p = stack.plan
    dev = stack.h.device
    xh = torch.randn((B, p.hidden), device=dev)
    xf = torch.randn((B, p.ff_rows), device=dev)
    if suffix:
        qkv, o = torch.empty((B, stack.qkv.shape[1]), device=dev), torch.empty((B, stack.o.shape[1]), device=dev)
        f, d = torch.empty((B, stack.f.shape[1]), device=dev), torch.empty((B, stack.d.shape[1]), device=dev)
        ctx.reserve_scratch(max(getattr(stack.layers[0], a).scratch_bytes(B) for a in ("wqkv", "wo", "wgu", "wdown")))
    else:
        qkv, o, f, d = stack.qkv, stack.o, stack.f, stack.d
    cases = [("qkv_q4k_7168x5120", "wqkv", xh, qkv), ("o_q4k_5120x5120", "wo", qkv[:, :p.q_rows], o),
             ("gate_up_swiglu_q4k_34816x5120", "wgu", xh, f), ("down_q6k_5120x17408", "wdown", xf, d)]
    for name, attr, x, y in cases:
        name += suffix
        def once():
            for L in stack.layers:
                w = getattr(L, attr)
                if attr == "wgu":
                    w.try_matmul_swiglu(x, out=y)
                else:
                    w.matmul(x, out=y)
        us = graph_time_us(torch, ctx, once) / len(stack.layers)
        w = getattr(stack.layers[0], attr)
        nbytes = w.nbytes() + x.shape[0] * x.shape[1] * 4 + y.numel() * 4
        out[name] = {"us": us, "GB/s": nbytes / us / 1e3, "frac_of_peak": nbytes / us / 1e3 / peak, "launches": 2}
    return out


def other_configs(torch, ctx, QMatrix, peak):
    """The single-matrix configurations: configs[0] (Q4_K 4096x4096 GEMV, cold: 32 copies = 302 MB cycled, more than
    twice L2), configs[2] (Q6_K 151936x5120 output head at batch 1 and 64; 638 MB, larger than L2 by itself) and
    configs[3] (Q4_K 17408x5120 prefill at M = 128 / 512 / 2048)."""
    from ferric_b200 import synth
    dev = torch.device("cuda", ctx.device)
    out = {}
    # configs[0]
    rows = cols = 4096
    ws = [QMatrix.from_device_bytes(ctx, synth.matrix_on_device(12, rows, cols, 100 + i, dev), 12, rows, cols) for i in range(32)]
    x = torch.randn((1, cols), device=dev)
    y = torch.empty((1, rows), device=dev)

    def cycle():
        for w in ws:
            w.matmul(x, out=y)
    us = graph_time_us(torch, ctx, cycle) / len(ws)
    nbytes = ws[0].nbytes() + 4 * cols + 4 * rows
    out["config0_q4k_4096x4096_m1_cold"] = {"us": us, "GB/s": nbytes / us / 1e3, "frac_of_peak": nbytes / us / 1e3 / peak,
                                            "launches": 2}
    for w in ws:
        w.close()
    # configs[2]
    rows, cols = 151936, 5120
    head = QMatrix.from_device_bytes(ctx, synth.matrix_on_device(14, rows, cols, 2, dev), 14, rows, cols)
    for b in (1, 64):
        x = torch.randn((b, cols), device=dev)
        y = torch.empty((b, rows), device=dev)
        us = graph_time_us(torch, ctx, lambda: head.matmul(x, out=y))
        nbytes = head.nbytes() + 4 * b * cols + 4 * b * rows
        out[f"config2_head_q6k_151936x5120_m{b}"] = {"us": us, "GB/s": nbytes / us / 1e3, "frac_of_peak": nbytes / us / 1e3 / peak,
                                                     "TFLOP/s": 2.0 * b * rows * cols / us / 1e6}
    head.close()
    # configs[3]
    rows, cols = 17408, 5120
    gate = QMatrix.from_device_bytes(ctx, synth.matrix_on_device(12, rows, cols, 3, dev), 12, rows, cols)
    out["config3_prefill_q4k_bf16_17408x5120"] = {f"m{m}": prefill_case(torch, ctx, QMatrix, gate, m, 9) for m in (128, 512, 2048)}
    gate.close()
    # Q8_0 GEMV (the third format of the path): gate-sized matrix, 32 copies cycled (2.96 GB, far more than L2)
    rows, cols = 17408, 5120
    ws = [QMatrix.from_device_bytes(ctx, synth.matrix_on_device(8, rows, cols, 300 + i, dev), 8, rows, cols) for i in range(32)]
    x = torch.randn((1, cols), device=dev)
    y = torch.empty((1, rows), device=dev)

    def cycle8():
        for w in ws:
            w.matmul(x, out=y)
    us = graph_time_us(torch, ctx, cycle8) / len(ws)
    nbytes = ws[0].nbytes() + 4 * cols + 4 * rows
    out["gemv_q8_0_17408x5120_m1_cold"] = {"us": us, "GB/s": nbytes / us / 1e3, "frac_of_peak": nbytes / us / 1e3 / peak, "launches": 1}
    for w in ws:
        w.close()
    return out


def bf16_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, 1400.0, "fallback"


def prefill_case(torch, ctx, QMatrix, w, m, reps):
    """TFLOP/s of y[m, rows] = x[m, cols] . W^T on the tensor cores (weights dequantised to bf16 in the kernel): the
    median of `reps` (at least 9) individually timed launches after 3 warm-up launches.
    x (bf16) and y (f32) are resident; the weights of one matrix (100 MB at full size) are re-read from L2/HBM."""
    dev = torch.device("cuda", ctx.device)
    x = torch.randn((m, w.cols()), device=dev).to(torch.bfloat16)
    y = torch.empty((m, w.rows()), device=dev, dtype=torch.float32)
    for _ in range(3):
        w.matmul_bf16(x, out=y)
    assert w.gemm_status() == 0
    reps = max(reps, 9)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    for e0, e1 in evs:
        e0.record()
        w.matmul_bf16(x, out=y)
        e1.record()
    torch.cuda.synchronize(dev)
    us = statistics.median(e0.elapsed_time(e1) for e0, e1 in evs) * 1e3
    tf = 2.0 * m * w.rows() * w.cols() / us / 1e6
    burst, sustained, kind = bf16_peaks()
    return {"us": us, "TFLOP/s": tf, "frac_of_bf16_peak": tf / burst, "frac_of_sustained_bf16_peak": tf / sustained,
            "peak_source": kind, "finite": bool(torch.isfinite(y).all().item())}


def run_prefill(args):
    """One line for the prefill configuration alone (also the command the tensor-pipe profile is taken with)."""
    import torch
    from ferric_b200 import Context, QMatrix, synth
    torch.cuda.set_device(0)
    ctx = Context(0)
    rows, cols, m, ty = args.prefill_rows, args.prefill_cols, args.prefill, args.prefill_type
    raw = synth.matrix_on_device(ty, rows, cols, 1, torch.device("cuda:0"))
    w = QMatrix.from_device_bytes(ctx, raw, ty, rows, cols)
    with ClockSampler(0) as clocks:
        r = prefill_case(torch, ctx, QMatrix, w, m, max(args.steps, 1))
    burst, _, kind = bf16_peaks()
    print(json.dumps({
        "metric": "prefill_tflops", "value": r["TFLOP/s"], "unit": "TFLOP/s", "n_gpus": 1, "steps": max(args.steps, 1),
        "warmup": 3, "ms_per_step": r["us"] / 1e3, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{ {12: 'Q4_K', 13: 'Q5_K', 14: 'Q6_K', 8: 'Q8_0'}[ty] } [{rows}x{cols}] x bf16 [{m}x{cols}] -> f32, weights dequantised in-kernel"},
        "roofline": {"kernel": "gemm_q_bf16_kernel", "bound": "tensor", "achieved": r["TFLOP/s"], "peak": burst,
                     "unit": "TFLOP/s", "frac": r["TFLOP/s"] / burst, "peak_source": kind, "traffic": None},
        "gpu_launches": max(args.steps, 1), "clocks": clocks.summary(), "output_finite": r["finite"]}), flush=True)


def main():
    args = parse_args()
    if args.prefill:
        run_prefill(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
