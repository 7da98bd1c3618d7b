#!/usr/bin/env python
"""Benchmark of the NativeBit packed-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch M] [--impl ours|reference]

Workload (one "step"): the FFN decode matvecs of the 2.2B configuration — per layer gate and
up (6912 x 2560) and down (2560 x 6912), 3-bit indices, block 128, fp16 K=8 codebooks, bf16
activations at batch M — over 26 layers of distinct synthetic weights (691 MB, larger than L2, so
every matrix streams from HBM).  At batch 1 the 78 matvecs of a step are ONE launch of the
persistent multi-matrix kernel (nativebit_b200.MatvecGroup); at larger batches, and for the
per-layer all-reduce chain reported beside it, one CUDA graph of 78 single-matrix launches.
Metric: achieved HBM GB/s = algorithmic bytes / time.

With N > 1 ranks (torchrun) the same stack is tensor-parallel: every rank generates the same global
weights and keeps its shard (gate/up rows, down input blocks); the partial down outputs of all
layers are summed across ranks after the launch.  `value` is the whole job's algorithmic bytes over
the slowest rank's time ("strong" scaling: total work fixed).  Every N > 1 run checks its summed
outputs against the unsharded matvecs computed on the same GPU and exits non-zero on a mismatch.

`--impl reference` times the reference's CPU PyTorch path (restated in oracle/nb_oracle.py) on
the host cores over a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, FFN, LAYERS, BITS, BLOCK = 2560, 6912, 26, 3, 128
METRIC, UNIT = "dequant_matvec_hbm_gbs", "GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one 6912 x 2560 batch-1 launch, from one ncu capture
# (algorithmic bytes: 8 866 304)
NCU_TRAFFIC_B1 = 8912128
# the same sum for one launch of the group kernel over a step's 78 matrices: 225,413,376 B captured on a launch over
# 20 matrices of 6912 x 2560 (algorithmic 177,326,080 B), scaled by algorithmic bytes to the step's 691,571,712 B
NCU_TRAFFIC_STEP = 879112166


def alg_bytes(m, n, k, bits=BITS):
    return n * k * bits // 8 + (n * k // BLOCK) * (1 << bits) * 2 + m * k * 2 + m * n * 2


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU every few milliseconds while the timed region
    runs (NVML, read-only), with `nvidia-smi --query-gpu` as the fallback."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None
        self.thread, self.stop_flag, self.samples, self.reasons, self.max_mhz = None, False, [], set(), None

    def _nvml_loop(self, nv, handle):
        bits = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                for name, bit in bits.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[self.index]) if vis and vis.split(",")[self.index].isdigit() else self.index
            handle = nv.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            if self.samples:
                out.update(sm_mhz=statistics.median(self.samples), sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons),
                           samples=len(self.samples))
            return out
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [c.strip() for c in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ----------------------------------------------------------------------------- CPU arms
def cpu_sample(batch: int, repeats: int):
    """One layer's gate, up and down matvec through the reference's CPU PyTorch path."""
    import numpy as np
    import torch
    from oracle import nb_oracle as o
    torch.set_num_threads(os.cpu_count() or 1)
    mats = []
    for j, (n, k) in enumerate(((FFN, HIDDEN), (FFN, HIDDEN), (HIDDEN, FFN))):
        packed, cb, _ = o.make_packed_linear(n, k, BITS, seed=j)
        x = o.make_activation(batch, k, seed=j)
        mats.append((torch.from_numpy(x), torch.from_numpy(packed), torch.from_numpy(cb.astype(np.float32)), n, k))
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        for x, p, c, n, k in mats:
            o.torch_reference_forward(x, p, c, n, k)
        times.append(time.perf_counter() - t0)
    nbytes = sum(alg_bytes(batch, n, k) for *_, n, k in mats)
    return nbytes, times, torch.get_num_threads()


def workload_config(m, world):
    return {"workload": f"2.2B FFN decode matvecs (gate/up 6912x2560, down 2560x6912) x {LAYERS} layers, "
                        f"3-bit block-128 K=8 fp16 codebooks, bf16 activations batch {m} (configs[1])",
            "l2": "weights of one step total 691 MB (> 126 MB L2); every matrix is read once per step, 77 other "
                  "matrices between two reads of it",
            "parallelism": f"tp{world}" if world > 1 else "single"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    nbytes, _, cores = cpu_sample(args.batch, max(1, args.warmup))
    nbytes, times, cores = cpu_sample(args.batch, args.steps)
    t = sum(times) / len(times)
    val = nbytes / t / 1e9
    sample = "per step: gate+up+down matvec of ONE layer (1/26 of the GPU arm's step), unpack+gather+matmul each call"
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.batch, args.gpus),
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ----------------------------------------------------------------------------- GPU arm
N_BLOCKS, MIN_TIMED_S = 20, 0.5


def run_ours(args):
    import torch
    import torch.distributed as dist
    import nativebit_b200 as nbt
    from nativebit_b200 import ops, synthetic, tp

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    m = args.batch
    use_group = m <= 8 and not args.chain          # one launch per step, if the activations fit its shared memory (1..4 rows here)

    # ---- weights: every rank generates the same global matrices (seed 10 * layer + j) and keeps its shard
    ch0, ch_n = tp.ffn_shard_plan(FFN, world, rank)            # hidden channels of this rank
    shapes = [("gate", ch_n, HIDDEN), ("up", ch_n, HIDDEN), ("down", HIDDEN, ch_n)]
    check_layers = (0, LAYERS - 1) if world > 1 else ()
    layers, full_layers = [], {}
    for l in range(LAYERS):
        mods, full = {}, {}
        for j, name in enumerate(("gate", "up", "down")):
            n, k = (FFN, HIDDEN) if name != "down" else (HIDDEN, FFN)
            p, c = synthetic.synthetic_packed(n, k, BITS, seed=10 * l + j, device=dev)
            if l in check_layers:
                full[name] = (p, c)
            if world > 1:
                if name != "down":
                    p, c = tp.slice_rows(p, c, n, k, BITS, ch0, ch_n, BLOCK)
                else:
                    p, c = tp.slice_cols(p, c, n, k, BITS, ch0 // BLOCK, ch_n // BLOCK, BLOCK)
            mods[name] = nbt.PackedLinear(p, c, *(((ch_n, HIDDEN) if name != "down" else (HIDDEN, ch_n))), bits=BITS)
        layers.append(mods)
        if full:
            full_layers[l] = full
    # the step's inputs live in one device buffer and its outputs in another, so that the end-to-end leg moves each
    # with a single copy
    h_full = synthetic.synthetic_activation(m, FFN, 2, dev)
    io_in = torch.empty(m * HIDDEN + m * ch_n, dtype=torch.bfloat16, device=dev)
    x = io_in[:m * HIDDEN].view(m, HIDDEN)
    h = io_in[m * HIDDEN:].view(m, ch_n)
    x.copy_(synthetic.synthetic_activation(m, HIDDEN, 1, dev))
    h.copy_(h_full[:, ch0:ch0 + ch_n])
    # with more than one rank the partial down outputs are summed in fp32
    down_dtype = torch.bfloat16 if world == 1 else torch.float32
    gu_bytes = LAYERS * m * ch_n * 2
    down_bytes = LAYERS * m * HIDDEN * (2 if world == 1 else 4)
    io_out = torch.empty(2 * gu_bytes + down_bytes, dtype=torch.uint8, device=dev)
    y_gate = io_out[:gu_bytes].view(torch.bfloat16).view(LAYERS, m, ch_n)
    y_up = io_out[gu_bytes:2 * gu_bytes].view(torch.bfloat16).view(LAYERS, m, ch_n)
    y_down = io_out[2 * gu_bytes:].view(down_dtype).view(LAYERS, m, HIDDEN)
    ws = ops.workspace(dev, 8 << 20)
    oneshot = None
    if world > 1 and args.allreduce in ("oneshot", "fused"):
        from nativebit_b200.comm import OneShotAllReduce
        oneshot = OneShotAllReduce(LAYERS * m * HIDDEN, dev)

    def all_reduce(t):
        if oneshot is not None:
            oneshot(t)
        else:
            dist.all_reduce(t)

    stream = torch.cuda.Stream(device=dev)
    side = torch.cuda.Stream(device=dev)
    ws_side = torch.zeros(8 << 20, dtype=torch.uint8, device=dev)

    def run_lin(lin, src, dst, wsp):
        ops.gemv(src, lin.packed_indices, lin.codebook, BITS, BLOCK, lin.out_features, lin.in_features, out=dst, ws=wsp)

    # ---- path A: the whole step as one launch of the persistent kernel (+ one sum over the ranks)
    group = None
    if use_group:
        items = [(mods[nm], x, out[l]) for l, mods in enumerate(layers) for nm, out in (("gate", y_gate), ("up", y_up))]
        items += [(mods["down"], h, y_down[l]) for l, mods in enumerate(layers)]
        try:
            group = nbt.MatvecGroup(items)
        except RuntimeError:                       # too many activation rows for the kernel's shared memory: the graph of launches
            use_group = False

    def group_step():
        group.run()
        if world > 1:
            all_reduce(y_down)

    # ---- path B: one launch per matrix, gate || up on two streams, down after both, the down output of a
    # layer summed over the ranks before the next layer (the order a decoder imposes); one CUDA graph
    def launch_chain(xin, hin):
        cur = torch.cuda.current_stream()
        for l, mods in enumerate(layers):
            side.wait_stream(cur)
            run_lin(mods["gate"], xin, y_gate[l], ws)
            with torch.cuda.stream(side):
                run_lin(mods["up"], xin, y_up[l], ws_side)
            cur.wait_stream(side)
            run_lin(mods["down"], hin, y_down[l], ws)
            if world > 1:
                all_reduce(y_down[l])

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        launch_chain(x, h)                     # warm the kernels / NCCL before capture
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            launch_chain(x, h)
    step_fn = group_step if use_group else graph.replay
    launches_per_step = (1 + (1 if world > 1 else 0)) if use_group else 3 * LAYERS + (LAYERS if world > 1 else 0)
    step_bytes_rank = sum(alg_bytes(m, n, k) for _, n, k in shapes) * LAYERS

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_blocks(fn, steps, blocks):
        """`blocks` back-to-back blocks of `steps` calls, each block timed with CUDA events on the launching
        stream, a barrier + synchronize on both sides of the whole region; per block the max over ranks."""
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
        barrier()
        with torch.cuda.stream(stream):
            ev[0].record(stream)
            for b in range(blocks):
                for _ in range(steps):
                    fn()
                ev[b + 1].record(stream)
        barrier()
        t = torch.tensor([ev[b].elapsed_time(ev[b + 1]) for b in range(blocks)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def timed(fn, steps):
        return sum(timed_blocks(fn, steps, 1))

    # ---- device-resident throughput (the `value`): at least N_BLOCKS blocks of `steps` steps and MIN_TIMED_S seconds
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            step_fn()
    probe = timed(step_fn, args.steps)
    blocks = max(args.blocks, int(args.min_timed_s * 1e3 / max(probe, 1e-3)) + 1)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    block_ms = timed_blocks(step_fn, args.steps, blocks)
    if sum(block_ms) < args.min_timed_s * 1e3:      # the probe ran slower than the steady state: take the region again, longer
        blocks = int(blocks * args.min_timed_s * 1e3 / max(sum(block_ms), 1e-3) * 1.1) + 1
        block_ms = timed_blocks(step_fn, args.steps, blocks)
    clocks = sampler.stop() if rank == 0 else None
    if group is not None:
        group.check()
    total_bytes = torch.tensor([float(step_bytes_rank)], device=dev)
    if world > 1:
        dist.all_reduce(total_bytes)
    step_bytes = float(total_bytes)
    ms_per_step = statistics.median(block_ms) / args.steps
    value = step_bytes / (ms_per_step * 1e-3) / 1e9
    timing = {"blocks": blocks, "steps_per_block": args.steps, "timed_region_ms": sum(block_ms),
              "ms_per_step_median_block": ms_per_step, "ms_per_step_mean": sum(block_ms) / (blocks * args.steps),
              "ms_per_step_min_block": min(block_ms) / args.steps, "ms_per_step_max_block": max(block_ms) / args.steps}
    # the other way of issuing the same step, for the record
    other = None
    if use_group:
        with torch.cuda.stream(stream):
            for _ in range(3):
                graph.replay()
        t_chain = statistics.median(timed_blocks(graph.replay, args.steps, 5)) / args.steps
        other = {"graph_of_78_launches_ms_per_step": t_chain, "graph_of_78_launches_GBps": step_bytes / (t_chain * 1e-3) / 1e9,
                 "exchange": "per-layer all-reduce inside the graph" if world > 1 else "none"}

    # ---- N > 1: the sharded, summed outputs against the unsharded matvecs computed on this GPU
    tp_check = None
    if world > 1:
        with torch.cuda.stream(stream):
            step_fn()
        stream.synchronize()
        worst = {"gate_up": 0.0, "down": 0.0}
        for l, full in full_layers.items():
            for nm, ysh in (("gate", y_gate), ("up", y_up)):
                ref = ops.gemv(x, full[nm][0], full[nm][1], BITS, BLOCK, FFN, HIDDEN, out_dtype=torch.float32, ordered=True)
                err = (ysh[l].float() - ref[:, ch0:ch0 + ch_n]).abs().max() / ref.abs().max()
                worst["gate_up"] = max(worst["gate_up"], float(err))
            ref = ops.gemv(h_full, full["down"][0], full["down"][1], BITS, BLOCK, HIDDEN, FFN, out_dtype=torch.float32, ordered=True)
            worst["down"] = max(worst["down"], float((y_down[l].float() - ref).abs().max() / ref.abs().max()))
        ok = worst["gate_up"] <= 2.0 ** -7 and worst["down"] <= 2e-5          # bf16 outputs / fp32 sums
        flag = torch.tensor([int(ok)], device=dev)
        errs = torch.tensor([worst["gate_up"], worst["down"]], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        dist.all_reduce(errs, op=dist.ReduceOp.MAX)
        if oneshot is not None:
            oneshot.check()
        tp_check = {"ok": bool(flag.item() == 1), "layers_checked": list(full_layers), "gate_up_rel_err_bf16_out": float(errs[0]),
                    "down_sum_rel_err": float(errs[1]), "against": "unsharded matvecs of the same global weights on every rank's GPU"}
        full_layers.clear()

    # ---- end to end through the public API with host buffers: inputs from pinned host memory, results back to it
    in_host = io_in.cpu().pin_memory()
    out_host = torch.empty(io_out.numel(), dtype=torch.uint8).pin_memory()

    def e2e_step():
        io_in.copy_(in_host, non_blocking=True)
        if use_group:
            group_step()
        else:
            for l, mods in enumerate(layers):
                y_gate[l] = mods["gate"](x)
                y_up[l] = mods["up"](x)
                y_down[l] = mods["down"](h).to(y_down.dtype)
                if world > 1:
                    all_reduce(y_down[l])
        out_host.copy_(io_out, non_blocking=True)
        torch.cuda.current_stream().synchronize()          # the caller reads the results of every step

    with torch.cuda.stream(stream):
        for _ in range(3):
            e2e_step()
    e2e_steps = max(1, min(args.steps, 20))
    ms_e2e = statistics.median(timed_blocks(e2e_step, e2e_steps, 5)) / e2e_steps
    e2e_value = step_bytes / (ms_e2e * 1e-3) / 1e9
    h2d = in_host.numel() * 2
    d2h = out_host.numel()

    # ---- roofline of the dominant kernel and the per-kernel figures (1 GPU only)
    roofline, extra = None, {}
    if world == 1:
        peak, peak_src = measured_peak()
        kb = alg_bytes(m, FFN, HIDDEN)
        gate_up = [(mods[nm]) for mods in layers for nm in ("gate", "up")]          # 52 copies, 461 MB > L2
        yb = torch.empty(m, FFN, dtype=torch.bfloat16, device=dev)
        yb2 = torch.empty_like(yb)

        def capture(n_chains):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                with torch.cuda.graph(g, stream=stream):
                    if n_chains == 2:
                        side.wait_stream(stream)
                    for i, lin in enumerate(gate_up):
                        if n_chains == 2 and i % 2:
                            with torch.cuda.stream(side):
                                run_lin(lin, x, yb2, ws_side)
                        else:
                            run_lin(lin, x, yb, ws)
                    if n_chains == 2:
                        stream.wait_stream(side)
                for _ in range(3):
                    g.replay()
            return g

        g2 = capture(2)
        g1 = capture(1)
        reps = max(5, args.steps)
        ms_k = timed(g2.replay, reps) / (reps * len(gate_up))
        ms_k1 = timed(g1.replay, reps) / (reps * len(gate_up))
        single = {"kernel": "nb::gemv_kernel<3,%d,%d> 6912x2560 batch %d, one launch per matrix" % (2 if m > 8 else 1, 1 if m == 1 else 8, m),
                  "algorithmic_bytes": kb,
                  "one_chain_us": ms_k1 * 1e3, "one_chain_GBps": kb / (ms_k1 * 1e-3) / 1e9, "one_chain_frac": kb / (ms_k1 * 1e-3) / 1e9 / peak,
                  "two_chains_us": ms_k * 1e3, "two_chains_GBps": kb / (ms_k * 1e-3) / 1e9, "two_chains_frac": kb / (ms_k * 1e-3) / 1e9 / peak}
        if m == 1:
            # the same chain on the decode step's kernel: one nb_gemv_stream launch per matrix over the stream-layout
            # copies (programmatic dependent launches: a kernel's first weight requests overlap the drain of the one before)
            yf = torch.empty(FFN, dtype=torch.float32, device=dev)
            g3 = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                for lin in gate_up[:2]:
                    ops.gemv_stream(ops.PRO_NONE, x, lin.stream_weight(), BITS, FFN, HIDDEN, yf)
                with torch.cuda.graph(g3, stream=stream):
                    for lin in gate_up:
                        ops.gemv_stream(ops.PRO_NONE, x, lin.stream_weight(), BITS, FFN, HIDDEN, yf)
                for _ in range(3):
                    g3.replay()
            ms_k3 = timed(g3.replay, reps) / (reps * len(gate_up))
            single.update({"stream_layout_chain_kernel": "nb::tile_gemv_kernel<3,1> (nb_gemv_stream), one launch per matrix, one chain",
                           "stream_layout_chain_us": ms_k3 * 1e3, "stream_layout_chain_GBps": kb / (ms_k3 * 1e-3) / 1e9,
                           "stream_layout_chain_frac": kb / (ms_k3 * 1e-3) / 1e9 / peak})
        if use_group:
            # the persistent kernel on the two FFN shapes alone: 52 gate/up matrices, 26 down matrices per launch
            per = {}
            for tag, its, n, k in (("6912x2560", [(lin, x, y_gate[i // 2] if i % 2 == 0 else y_up[i // 2]) for i, lin in enumerate(gate_up)], FFN, HIDDEN),
                                   ("2560x6912", [(mods["down"], h, y_down[l]) for l, mods in enumerate(layers)], HIDDEN, FFN)):
                g = nbt.MatvecGroup(its)
                with torch.cuda.stream(stream):
                    for _ in range(3):
                        g.run()
                t = statistics.median(timed_blocks(g.run, 10, 5)) / 10 / len(its)
                per[tag] = {"us_per_matrix": t * 1e3, "GBps": alg_bytes(1, n, k) / (t * 1e-3) / 1e9,
                            "frac": alg_bytes(1, n, k) / (t * 1e-3) / 1e9 / peak, "matrices_per_launch": len(its)}
                g.check()
                del g
            # four activation rows per matrix (configs[1] at batch 4): rows ride in the MMA's columns
            if m == 1:
                x4 = synthetic.synthetic_activation(4, HIDDEN, 7, dev)
                h4 = synthetic.synthetic_activation(4, FFN, 8, dev)
                yg4 = torch.empty(len(gate_up), 4, FFN, dtype=torch.bfloat16, device=dev)
                yd4 = torch.empty(LAYERS, 4, HIDDEN, dtype=torch.bfloat16, device=dev)
                for tag, its, n, k in (("6912x2560_b4", [(lin, x4, yg4[i]) for i, lin in enumerate(gate_up)], FFN, HIDDEN),
                                       ("2560x6912_b4", [(mods["down"], h4, yd4[l]) for l, mods in enumerate(layers)], HIDDEN, FFN)):
                    g = nbt.MatvecGroup(its)
                    with torch.cuda.stream(stream):
                        for _ in range(3):
                            g.run()
                    t = statistics.median(timed_blocks(g.run, 10, 5)) / 10 / len(its)
                    per[tag] = {"us_per_matrix": t * 1e3, "GBps": alg_bytes(4, n, k) / (t * 1e-3) / 1e9,
                                "frac": alg_bytes(4, n, k) / (t * 1e-3) / 1e9 / peak, "matrices_per_launch": len(its)}
                    del g
                del x4, h4, yg4, yd4
            # the other index widths of the format (2-bit K=4, 4-bit K=16), 26 matrices of 6912 x 2560 per launch
            for wb in (2, 4):
                its = []
                for i in range(LAYERS):
                    p2, c2 = synthetic.synthetic_packed(FFN, HIDDEN, wb, seed=500 + i, device=dev)
                    its.append((nbt.PackedLinear(p2, c2, FFN, HIDDEN, bits=wb), x, y_gate[i]))
                g = nbt.MatvecGroup(its)
                with torch.cuda.stream(stream):
                    for _ in range(3):
                        g.run()
                t = statistics.median(timed_blocks(g.run, 10, 5)) / 10 / len(its)
                ab = alg_bytes(1, FFN, HIDDEN, wb)
                per[f"6912x2560_{wb}bit"] = {"us_per_matrix": t * 1e3, "GBps": ab / (t * 1e-3) / 1e9, "frac": ab / (t * 1e-3) / 1e9 / peak,
                                             "matrices_per_launch": len(its), "algorithmic_bytes": ab}
                del g, its
            roofline = {"bound": "hbm", "achieved": value, "peak": peak, "unit": "GB/s", "frac": value / peak,
                        "traffic": NCU_TRAFFIC_STEP if m == 1 else None,
                        "kernel": "nb::group_kernel<3>, one launch = the 78 matrices of a step",
                        "us_per_launch": ms_per_step * 1e3, "algorithmic_bytes": int(step_bytes), "peak_source": peak_src,
                        "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch over 20 matrices of 6912x2560 "
                                          "(one ncu capture), scaled by algorithmic bytes to the 78 matrices of a step",
                        "per_shape_within_one_launch": per, "single_matrix_kernel": single,
                        "frac_of_nominal_8TBs": value / 8000.0}
        else:
            ach = kb / (ms_k * 1e-3) / 1e9
            roofline = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                        "traffic": NCU_TRAFFIC_B1 if m == 1 else None, "kernel": single["kernel"], "us_per_launch": ms_k * 1e3,
                        "algorithmic_bytes": kb, "peak_source": peak_src, "single_matrix_kernel": single,
                        "frac_of_nominal_8TBs": ach / 8000.0}
        # other batch sizes of configs[1], the single-matrix kernel, for the record
        for mb in (1, 4, 16):
            xb = synthetic.synthetic_activation(mb, HIDDEN, 3, dev)
            hb = synthetic.synthetic_activation(mb, FFN, 4, dev)
            ob1 = torch.empty(mb, FFN, dtype=torch.bfloat16, device=dev)
            ob2 = torch.empty(mb, HIDDEN, dtype=torch.bfloat16, device=dev)
            for tag, key, src, dst, n, k in (("6912x2560", "gate", xb, ob1, FFN, HIDDEN), ("2560x6912", "down", hb, ob2, HIDDEN, FFN)):
                gk = torch.cuda.CUDAGraph()
                with torch.cuda.stream(stream):
                    lins = [mods[key] for mods in layers] * 2
                    for lin in lins[:2]:
                        run_lin(lin, src, dst, ws)
                    stream.synchronize()
                    with torch.cuda.graph(gk, stream=stream):
                        for lin in lins:
                            ops.gemv(src, lin.packed_indices, lin.codebook, BITS, BLOCK, n, k, out=dst, ws=ws)
                    for _ in range(3):
                        gk.replay()
                t = timed(gk.replay, 5) / (5 * len(lins))
                gbs = alg_bytes(mb, n, k) / (t * 1e-3) / 1e9
                extra[f"{tag}_b{mb}"] = {"us": round(t * 1e3, 3), "GB/s": round(gbs, 1), "frac": round(gbs / peak, 4)}
    del group

    # ---- CPU baseline on the host cores (rank 0, N=1 only)
    cpu = None
    if world == 1 and not args.no_cpu:
        nbytes, times, cores = cpu_sample(m, 4)
        t = min(times[1:]) if len(times) > 1 else times[0]
        cpu = {"value": nbytes / t / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": "gate+up+down matvec of one layer (3 of the step's 78 matvecs), best of 3 after 1 warm-up; "
                         "reference CPU PyTorch path: unpack + gather + matmul per call"}

    # ---- prefill dequant-GEMM (configs[2]): 2048 tokens against both FFN shapes on the tensor cores
    prefill = None
    if world == 1 and not args.no_prefill:
        prefill = {}
        pk_bf16 = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("bf16_tflops", 1590.0) \
            if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 1590.0
        for n, k, key in ((FFN, HIDDEN, "gate"), (HIDDEN, FFN, "down")):
            lin = layers[0][key]
            xp = synthetic.synthetic_activation(2048, k, 5, dev)
            yp = torch.empty(2048, n, dtype=torch.bfloat16, device=dev)
            wbf = ops.dequant(lin.packed_indices, lin.codebook, BITS, BLOCK, (n, k), torch.bfloat16)
            wst = lin.stream_weight()
            calls = {"fused": lambda: ops.gemm_prefill_fused(xp, wst, BITS, n, k, out=yp),
                     "dequant_then_gemm": lambda: ops.gemm_prefill(xp, lin.packed_indices, lin.codebook, BITS, BLOCK, n, k, out=yp),
                     "gemm_only": lambda: ops.gemm_bf16(xp, wbf),
                     "library_gemm_on_dense": lambda: torch.matmul(xp, wbf.T)}
            t = {}
            with torch.cuda.stream(stream):
                for fn in calls.values():
                    for _ in range(3):
                        fn()
            for name, fn in calls.items():
                t[name] = timed(fn, 20) / 20
            fl = 2.0 * 2048 * n * k
            prefill[f"2048x{n}x{k}"] = {
                "fused_dequant_in_kernel_us": round(t["fused"] * 1e3, 1), "dequant_then_gemm_us": round(t["dequant_then_gemm"] * 1e3, 1),
                "gemm_only_us": round(t["gemm_only"] * 1e3, 1), "library_gemm_on_dense_us": round(t["library_gemm_on_dense"] * 1e3, 1),
                "TFLOPs_fused": round(fl / (t["fused"] * 1e-3) / 1e12, 1),
                "frac_of_measured_bf16_peak_fused": round(fl / (t["fused"] * 1e-3) / 1e12 / pk_bf16, 3),
                "TFLOPs_gemm_only": round(fl / (t["gemm_only"] * 1e-3) / 1e12, 1),
                "frac_of_measured_bf16_peak_gemm_only": round(fl / (t["gemm_only"] * 1e-3) / 1e12 / pk_bf16, 3),
                "weight_operand": "exact fp16 codebook entries; bf16 activations converted to fp16 (exact in range)"}
            if ops.prefill_status(dev) != 0:
                raise RuntimeError("a bounded wait of the prefill kernel ran out")
            del wbf, xp, yp
        # a decoder layer's four packed linears at 128 fp32 activation rows (the prefill of a 128-token prompt: the
        # residual stream is fp32 and enters the tensor cores as two fp16 terms), replayed from a CUDA graph
        per128 = {}
        for j, (nm, n, k) in enumerate((("qkv", 3 * HIDDEN, HIDDEN), ("out_proj", HIDDEN, HIDDEN), ("gate_up", 2 * FFN, HIDDEN),
                                        ("down", HIDDEN, FFN))):
            p2, c2 = synthetic.synthetic_packed(n, k, BITS, seed=900 + j, device=dev)
            lin = nbt.PackedLinear(p2, c2, n, k, bits=BITS)
            xr = synthetic.synthetic_activation(128, k, 6, dev).float()
            with torch.cuda.stream(stream):
                for _ in range(2):
                    lin(xr)
                stream.synchronize()
                gq = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gq, stream=stream):
                    for _ in range(10):
                        lin(xr)
                for _ in range(2):
                    gq.replay()
            per128[nm] = round(timed(gq.replay, 5) / 50 * 1e3, 2)
            del gq, lin, p2, c2
        per128["layer_total_us"] = round(sum(per128.values()), 1)
        prefill["128_rows_fp32_us"] = per128

    # ---- the full 2.2B packed decoder (configs[3]): 128-token prompt, 256 greedy tokens, batch 1
    decode = None
    if not args.no_decode:
        from nativebit_b200 import generate as G
        del layers, y_gate, y_up, y_down
        torch.cuda.empty_cache()
        cfg = G.ModelConfig()
        model = G.PackedGPT.random_init(cfg, seed=0, device=dev, tp_rank=rank, tp_size=world)
        if world > 1 and args.allreduce in ("oneshot", "fused"):
            model.enable_oneshot_allreduce(max_batch=1)
        if world > 1 and args.allreduce == "fused":
            model.enable_fused_allreduce(max_batch=1)
        gen = torch.Generator().manual_seed(0)
        prompt = torch.randint(0, cfg.vocab_size, (128,), generator=gen)
        # self-check before timing: the logits of the prompt's last token from the batched (tensor-core) prefill
        # against the same token reached by single-token decode steps (the GEMV kernels); with N > 1 also
        # against the unsharded model built on this GPU from the same seed
        pr = prompt.to(dev).reshape(1, -1)
        sess = G.DecodeSession(model, 1)
        sess.prefill(pr)
        lg_prefill = sess.logits.float().clone()
        sess2 = G.DecodeSession(model, 1, use_graph=False)
        sess2.prefill(pr[:, :96])
        for j in range(96, 128):
            sess2.token.copy_(pr[:, j].reshape(sess2.token.shape))     # teacher forcing: the prompt's token
            sess2.step()
        torch.cuda.synchronize()
        scale = float(lg_prefill.abs().max())
        errs = [float((sess2.logits.float() - lg_prefill).abs().max()) / scale]
        names = ["prefill_vs_stepwise_rel_err"]
        same_token = True
        del sess2
        if world > 1:
            full = G.PackedGPT.random_init(cfg, seed=0, device=dev)
            s1 = G.DecodeSession(full, 1, use_graph=False)
            s1.prefill(pr)
            errs.append(float((s1.logits.float() - lg_prefill).abs().max()) / float(s1.logits.abs().max()))
            names.append("tp_vs_single_gpu_rel_err")
            same_token = bool(torch.equal(s1.logits.argmax(-1), lg_prefill.argmax(-1)))
            del s1, full
            torch.cuda.empty_cache()
        errs_t = torch.tensor(errs, device=dev)
        flag = torch.tensor([int(same_token)], device=dev)
        if world > 1:
            dist.all_reduce(errs_t, op=dist.ReduceOp.MAX)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        checks = {nm: float(errs_t[i]) for i, nm in enumerate(names)}
        if world > 1:
            checks["tp_vs_single_gpu_next_token_equal"] = bool(flag.item() == 1)
        checks["gate"] = "2e-3 of max |logit|"
        checks["ok"] = bool(float(errs_t.max()) <= 2e-3 and flag.item() == 1)
        del sess
        res = G.benchmark(model, prompt, n_generate=256, n_runs=2)
        t = torch.tensor([res["per_token_ms"], res["prefill_ms"]], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        per_tok_ms, prefill_ms = float(t[0]), float(t[1])
        lin_bytes = cfg.n_layers * (alg_bytes(1, 3 * HIDDEN, HIDDEN) + alg_bytes(1, HIDDEN, HIDDEN) +
                                    2 * alg_bytes(1, FFN, HIDDEN) + alg_bytes(1, HIDDEN, FFN))
        head_bytes = cfg.vocab_size * HIDDEN * 2
        decode = {"tokens_per_s": 1e3 / per_tok_ms, "per_token_ms": per_tok_ms, "prefill_ms_128_tokens": prefill_ms,
                  "n_generate": 256, "batch": 1, "tp": world,
                  "allreduce": ("none" if world == 1 else args.allreduce),
                  "packed_linear_bytes_per_token": lin_bytes, "lm_head_bytes_per_token": head_bytes,
                  "weight_GBps": (lin_bytes + head_bytes) / (per_tok_ms * 1e-3) / 1e9,
                  "model": "26 layers, hidden 2560, 32 heads, FFN 6912, vocab 32000, random-init 3-bit packed linears",
                  "self_check": checks}
        del model
        torch.cuda.empty_cache()
        # the 2-bit (K=4) model of the same shape, decode speed only
        cfg2 = G.ModelConfig(bits=2)
        model2 = G.PackedGPT.random_init(cfg2, seed=0, device=dev, tp_rank=rank, tp_size=world)
        if world > 1 and args.allreduce in ("oneshot", "fused"):
            model2.enable_oneshot_allreduce(max_batch=1)
        if world > 1 and args.allreduce == "fused":
            model2.enable_fused_allreduce(max_batch=1)
        res2 = G.benchmark(model2, prompt, n_generate=128, n_runs=1)
        t2 = torch.tensor([res2["per_token_ms"]], device=dev)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        decode["two_bit"] = {"tokens_per_s": 1e3 / float(t2), "per_token_ms": float(t2), "n_generate": 128}
        del model2

    # ---- serving sweep (configs[4]): batch 1/8/32/64 decode after a 512-token prompt, 3-bit and 2-bit
    serving = None
    compact = world == 8 and not args.serving and not args.no_decode      # the 8-GPU line always carries batch 8 and 64
    if args.serving or compact:
        from nativebit_b200 import generate as G
        serving = {"prompt_tokens": 512, "n_generate": 64, "tp": world,
                   "linears": "1 sequence: nb_gemv_stream; 2..8: nb_gemv_stream_rows (the rows in the MMA columns, one weight pass); 9..16: fused GEMV; more: the tensor-core kernel that dequantises inside (exact fp16 weights)"}
        for bits in (3, 2):
            cfg = G.ModelConfig(bits=bits)
            model = G.PackedGPT.random_init(cfg, seed=0, device=dev, tp_rank=rank, tp_size=world)
            if world > 1 and args.allreduce in ("oneshot", "fused"):
                model.enable_oneshot_allreduce(max_batch=64)
            if world > 1 and args.allreduce == "fused":
                model.enable_fused_allreduce(max_batch=8)
            prompt = torch.randint(0, cfg.vocab_size, (512,), generator=torch.Generator().manual_seed(1))
            for b in ((8, 64) if compact else (1, 8, 32, 64)):
                res = G.benchmark(model, prompt, n_generate=64, n_runs=1, batch_size=b)
                t = torch.tensor([res["per_token_ms"]], device=dev)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                serving[f"{bits}bit_b{b}"] = {"ms_per_step": round(float(t), 3), "tokens_per_s": round(b * 1e3 / float(t), 1)}
            del model
            torch.cuda.empty_cache()

    failed = (tp_check is not None and not tp_check["ok"]) or (decode is not None and not decode["self_check"]["ok"])
    if rank == 0:
        cfgd = workload_config(m, world)
        cfgd["launch"] = ("one launch of the persistent multi-matrix kernel per step (nativebit_b200.MatvecGroup)" if use_group else
                          "one CUDA graph of 78 kernels per step; gate and up of a layer on two streams, down after both")
        if world > 1:
            cfgd["exchange"] = ("one sum over the ranks of all layers' partial down outputs per step (the layers of this workload are "
                                "independent); the per-layer exchange of a decoder is the `other_issue_order` and `decode` figures"
                                if use_group else "all-reduce of the down output after every layer") + f"; {args.allreduce}"
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f16xf16->f32",
                "data": "synthetic", "config": cfgd, "timing": timing,
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": ms_e2e,
                        "api": ("nativebit_b200.MatvecGroup.run()" if use_group else "PackedLinear.forward per matrix") +
                               ", inputs copied from pinned host memory and every output copied back to it, stream synchronised, each step"},
                "gpu_launches": launches_per_step * args.steps * blocks,
                "clocks": clocks}
        if other is not None:
            line["other_issue_order"] = other
        if tp_check is not None:
            line["tp_check"] = tp_check
        if roofline is not None:
            line["roofline"] = roofline
            line["per_shape"] = extra
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if decode is not None:
            line["decode"] = decode
        if prefill is not None:
            line["prefill"] = prefill
        if serving is not None:
            line["serving"] = serving
        print(json.dumps(line))
    if world > 1:
        # NCCL communicators cannot be torn down while CUDA graphs that captured their kernels are
        # alive (destroy_process_group blocks); everything is released with the process instead.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(1 if failed else 0)
    if failed:
        sys.exit(1)


def run_kernel_only(args):
    """A few plain launches of one shape over weight copies larger than L2 — the small case
    that profiler captures are taken on (python bench.py --kernel-only N K M)."""
    import torch
    from nativebit_b200 import ops, synthetic
    n, k, m = args.kernel_only
    dev = torch.device("cuda", 0)
    copies = max(2, int(160e6 // (n * k * 3 // 8)) + 1)
    ws = [synthetic.synthetic_packed(n, k, BITS, seed=i, device=dev) for i in range(copies)]
    x = synthetic.synthetic_activation(m, k, 0, dev)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    wsp = ops.workspace(dev, 8 << 20)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for rep in range(3):
        e0.record()
        for p, c in ws:
            ops.gemv(x, p, c, BITS, BLOCK, n, k, out=y, ws=wsp)
        e1.record()
        torch.cuda.synchronize()
    print(json.dumps({"kernel_only": [n, k, m], "copies": copies, "us_per_launch_stream": e0.elapsed_time(e1) * 1e3 / copies}))


def run_group_only(args):
    """A few launches of the persistent kernel over N_MATS matrices of 6912 x 2560 (distinct weights, more than
    L2 from 10 matrices up) — the small case that profiler captures are taken on
    (python bench.py --group-only N_MATS)."""
    import torch
    import nativebit_b200 as nbt
    from nativebit_b200 import synthetic
    dev = torch.device("cuda", 0)
    x = synthetic.synthetic_activation(1, HIDDEN, 1, dev)
    y = torch.empty(args.group_only, 1, FFN, dtype=torch.bfloat16, device=dev)
    items = []
    for i in range(args.group_only):
        p, c = synthetic.synthetic_packed(FFN, HIDDEN, BITS, seed=i, device=dev)
        items.append((nbt.PackedLinear(p, c, FFN, HIDDEN, bits=BITS), x, y[i]))
    grp = nbt.MatvecGroup(items)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for rep in range(3):
        e0.record()
        grp.run()
        e1.record()
        torch.cuda.synchronize()
    grp.check()
    us = e0.elapsed_time(e1) * 1e3
    print(json.dumps({"group_only": args.group_only, "us_per_launch": us, "us_per_matrix": us / args.group_only,
                      "GBps": args.group_only * alg_bytes(1, FFN, HIDDEN) / us / 1e3}))


def run_gemm_only(args):
    """A few plain launches of the prefill GEMM on one shape, first the dequant kernel + tcgen05 GEMM, then the
    kernel that dequantises inside the tensor-core pipeline — the small case that profiler captures are taken
    on (python bench.py --gemm-only M N K)."""
    import torch
    from nativebit_b200 import ops, synthetic
    m, n, k = args.gemm_only
    dev = torch.device("cuda", 0)
    p, c = synthetic.synthetic_packed(n, k, BITS, seed=0, device=dev)
    x = synthetic.synthetic_activation(m, k, 0, dev)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for rep in range(3):
        e0.record()
        for _ in range(4):
            ops.gemm_prefill(x, p, c, BITS, BLOCK, n, k, out=y)
        e1.record()
        torch.cuda.synchronize()
    two = e0.elapsed_time(e1) * 1e3 / 4
    from nativebit_b200 import stream as S
    w = S.stream_pack(p, c, BITS, n, k)
    for rep in range(3):
        e0.record()
        for _ in range(4):
            ops.gemm_prefill_fused(x, w, BITS, n, k, out=y)
        e1.record()
        torch.cuda.synchronize()
    print(json.dumps({"gemm_only": [m, n, k], "us_per_call_dequant_plus_gemm": two, "us_per_call_fused": e0.elapsed_time(e1) * 1e3 / 4,
                      "status": ops.prefill_status(dev)}))


def run_decode_only(args):
    """Prefill and a few graph-replayed decode steps of the 2.2B packed decoder at batch 1; the last step
    runs between cudaProfilerStart/Stop, so a profiler started with --profile-from-start off sees the
    launches of exactly one step (python bench.py --decode-only STEPS)."""
    import time
    import torch
    from nativebit_b200 import generate as G
    dev = torch.device("cuda", 0)
    cfg = G.ModelConfig()
    model = G.PackedGPT.random_init(cfg, seed=0, device=dev)
    prompt = torch.randint(0, cfg.vocab_size, (1, 128), generator=torch.Generator().manual_seed(0)).to(dev)
    sess = G.DecodeSession(model, 1)
    sess.prefill(prompt)
    for _ in range(3):
        sess.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.decode_only):
        sess.step()
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) / args.decode_only * 1e3
    torch.cuda.profiler.start()
    sess.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    sess.check()
    print(json.dumps({"decode_only": args.decode_only, "per_token_ms": ms}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--blocks", type=int, default=N_BLOCKS, help="timed blocks of --steps steps each (the median block is reported)")
    ap.add_argument("--min-timed-s", type=float, default=MIN_TIMED_S,
                    help="lower bound of the timed region in seconds (more blocks are added to reach it; 0 for short profiling runs)")
    ap.add_argument("--chain", action="store_true", help="time the graph of one launch per matrix instead of the persistent kernel")
    ap.add_argument("--allreduce", default="oneshot", choices=["oneshot", "fused", "nccl"],
                    help="tensor-parallel all-reduce of the decoder: the one-shot peer-memory kernel (default, the fastest "
                         "measured), folded into the packed GEMVs (peer-memory push + gather; the one-shot kernel where that "
                         "does not apply), or NCCL")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 2048-token prefill GEMM leg")
    ap.add_argument("--serving", action="store_true", help="add the batch 1/8/32/64, 3-bit and 2-bit decode sweep (configs[4])")
    ap.add_argument("--no-decode", action="store_true", help="skip the 2.2B decoder leg")
    ap.add_argument("--decode-only", type=int, default=0, metavar="STEPS",
                    help="time STEPS decode steps of the 2.2B decoder at batch 1 and exit (profiling case)")
    ap.add_argument("--group-only", type=int, default=0, metavar="N_MATS",
                    help="launch the persistent kernel over N_MATS 6912x2560 matrices a few times and exit (profiling case)")
    ap.add_argument("--gemm-only", type=int, nargs=3, metavar=("M", "N", "K"), default=None,
                    help="launch the prefill GEMM on one shape a few times and exit (profiling case)")
    ap.add_argument("--kernel-only", type=int, nargs=3, metavar=("N", "K", "M"), default=None,
                    help="launch one GEMV shape a few times and exit (profiling case)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.decode_only:
        run_decode_only(args)
    elif args.group_only:
        run_group_only(args)
    elif args.gemm_only:
        run_gemm_only(args)
    elif args.kernel_only:
        run_kernel_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
