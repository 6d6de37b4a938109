#!/usr/bin/env python
"""Benchmark of the B200 quantized matrix-product path.

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--impl reference]

A step is one pass of the decode (or prefill) layer set: every projection of
every layer of the named model shape against synthetic Q8_0 activations.  The
metric is the reference benchmark's own (hearth-llm/examples/benchk.rs:162,
:198): packed weight bytes streamed per second.  With N > 1 every weight is
row-sharded over the ranks (rank r holds rows [r*ceil(n/N), ...)) and each step
ends with an NCCL all-gather of the output slices, so the total work is fixed
("strong" scaling).  Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from hearth_b200 import synth  # noqa: E402

DEFAULT_WORKLOAD = "c4_pq2_27b_decode"
METRIC = "quant GEMV weight-stream bandwidth"
UNIT = "GB/s"
PREFILL_METRIC = "prefill GEMM throughput (2*M*N*K int8 ops)"
PREFILL_UNIT = "TOPS"


def is_prefill(cfg: dict) -> bool:
    return cfg["seq_len"] >= 128


def total_ops(cfg: dict) -> float:
    return 2.0 * cfg["seq_len"] * cfg["layers"] * sum(r * k for _, r, k in cfg["shapes"])


def tensor_peak(hb=None):
    """Dense int8 peak is not in MEASURED_PEAKS.json: measure it on the GPU in use (a bare run of kind::i8 MMAs on
    every SM, hb200_measure_i8_peak).  Without the library: 2 x the measured sustained bf16 figure."""
    if hb is not None:
        try:
            return hb.measure_i8_peak(), "measured on this GPU: bare tcgen05.mma kind::i8 128x256x32 on every SM (hb200_measure_i8_peak)"
        except Exception as e:  # noqa: BLE001 - fall through to the derived figure, and say so
            print(f"bench: int8 peak measurement failed ({e}); using 2 x bf16", file=sys.stderr)
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return 2.0 * float(d["bf16_tflops_sustained"]), "2 x measured sustained bf16 (MEASURED_PEAKS.json bf16_tflops_sustained)"
    return 2.0 * 1400.0, "2 x fallback sustained bf16 (1.4 PFLOP/s)"


def cpu_model() -> str:
    try:
        for ln in open("/proc/cpuinfo"):
            if ln.startswith("model name"):
                return ln.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


from hearth_b200.sharding import ShardPlan, shard_rows  # noqa: E402


def algorithmic_bytes(cfg: dict) -> dict:
    """Per step: packed weights + Q8_0 activations + f32 outputs (whole job, all ranks together)."""
    m = cfg["seq_len"]
    w = a = o = 0
    for _, n_rows, n_cols in cfg["shapes"]:
        w += n_rows * synth.row_bytes(cfg["dtype"], n_cols)
        a += m * n_cols * 4 if cfg["dtype"] in (12, 14) else m * (n_cols // 32) * 34  # K-quants read f32 activations
        o += m * n_rows * 4
    L = cfg["layers"]
    return {"weights": w * L, "activations": a * L, "outputs": o * L}


# ------------------------------------------------------------------------------------------ CPU arm

class CpuArm:
    """The restated reference CPU path (SIMD arms + row-splitting pool) on a bounded sample of the workload."""

    def __init__(self, cfg: dict, threads: int, sample_layers: int):
        from oracle import oracle as O
        O.build()
        self.O, self.cfg = O, cfg
        self.S = O.simd()
        self.threads = self.S.hs_pool_start(threads)  # <= 0: physical cores, the reference's dense rule (pool.rs:150-152)
        self.mats = []
        for li in range(sample_layers):
            for ti, (_, n_rows, n_cols) in enumerate(cfg["shapes"]):
                w = synth.weights(cfg["dtype"], n_rows, n_cols, seed=4000 + 10 * li + ti)
                a = synth.activations(cfg["seq_len"], n_cols, seed=5000 + 10 * li + ti)
                if cfg["dtype"] not in (12, 14):  # K-quants take the f32 rows as they are
                    a = O.quantize_q8_0(a)
                self.mats.append((w, a, n_rows, n_cols, np.zeros((cfg["seq_len"], n_rows), dtype=np.float32)))
        self.nbytes = sum(w.size for w, *_ in self.mats)
        self.ops = 2.0 * cfg["seq_len"] * sum(n_rows * n_cols for _, _, n_rows, n_cols, _ in self.mats)
        self.kernel = self.S.hs_selected_kernel(cfg["dtype"]).decode()
        self.desc = (f"{sample_layers} layer(s) x {len(cfg['shapes'])} projections of the workload, M={cfg['seq_len']}, "
                     f"{self.nbytes / 1e6:.1f} MB of weights per pass; arm={self.kernel}; {self.threads} threads of "
                     f"{self.S.hs_logical_cores()} logical CPUs; C restatement of the reference's SIMD kernels and pool")
        t_end = time.perf_counter() + 0.3  # time-based warm-up, as benchk does (benchk.rs:172-182)
        self.one_pass()
        while time.perf_counter() < t_end:
            self.one_pass()

    def one_pass(self) -> float:
        t0 = time.perf_counter()
        run = self.O.simd_matmul_kquant_f32 if self.cfg["dtype"] in (12, 14) else self.O.simd_dot_rows_batched
        for w, a, n_rows, n_cols, out in self.mats:
            run(self.cfg["dtype"], w, a, n_rows, n_cols, out)
        return time.perf_counter() - t0

    def gbs(self, passes: int = 2) -> float:
        return self.nbytes / min(self.one_pass() for _ in range(passes)) / 1e9

    def close(self):
        self.S.hs_pool_stop()


def run_reference(args, cfg, rank):
    """The reference arm: the reference's CPU implementation of the path (here its C restatement, because the
    Rust original cannot be built) on all physical cores; a step is one pass over a one-layer sample."""
    if rank != 0:
        return
    arm = CpuArm(cfg, 0, 1)
    t0 = time.perf_counter()
    times = []
    for i in range(args.warmup + args.steps):
        t = arm.one_pass()
        if i >= args.warmup:
            times.append(t)
        if time.perf_counter() - t0 > 150:
            break
    arm.close()
    sec = statistics.median(times)
    value = arm.nbytes / sec / 1e9
    metric, unit = METRIC, UNIT
    if is_prefill(cfg):
        metric, unit, value = PREFILL_METRIC, PREFILL_UNIT, arm.ops / sec / 1e12
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": len(times),
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 x {1,2}-bit -> int32, fp32 scales", "data": "synthetic",
        "config": {"workload": args.workload, "tokens": cfg["seq_len"], "sample": arm.desc},
        "cpu_baseline": {"value": value, "unit": unit, "cores": arm.threads, "kind": "port", "sample": arm.desc},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------ GPU arm

def run_ours(args, cfg, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from hearth_b200 import api as hb

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    hb.init(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    M = cfg["seq_len"]
    dtype = cfg["dtype"]
    stream = torch.cuda.Stream(device=dev)

    # ---- resident data: this rank's row shard of every weight, one activation per distinct input width
    weights, acts = [], {}
    slice_rows = 0
    for li in range(cfg["layers"]):
        for ti, (_, n_rows, n_cols) in enumerate(cfg["shapes"]):
            lo, hi = shard_rows(n_rows, rank, world)
            packed = synth.weights_torch(dtype, hi - lo, n_cols, seed=1000 * (li + 1) + 10 * ti + rank, device=dev)
            weights.append((hb.Weight.upload_dev(dtype, hi - lo, n_cols, packed), -(-n_rows // world)))
            del packed
            slice_rows += -(-n_rows // world)
    torch.cuda.synchronize()
    # One activation per input-sharing group of each layer, as in the model: q|k|v read one vector, o another,
    # gate|up a third, down a fourth (hearth-llm/src/model/mod.rs:527-775).
    group_of = {"q": 0, "k": 0, "v": 0, "o": 1, "gate": 2, "up": 2, "down": 3}

    # outputs: one packed buffer per rank [M, slice_rows]; gathered into [world, M, slice_rows]
    out_local = torch.zeros((M, slice_rows), dtype=torch.float32, device=dev)
    out_all = torch.zeros((world * M, slice_rows), dtype=torch.float32, device=dev) if world > 1 else None  # [world][M][slice]
    batch = hb.Batch()
    off = 0
    i = 0
    for li in range(cfg["layers"]):
        for ti, (name, n_rows, n_cols) in enumerate(cfg["shapes"]):
            W, pad_rows = weights[i]
            i += 1
            key = (li, group_of.get(name, ti))
            if key not in acts:
                acts[key] = hb.Act(M, n_cols)
            if W.n_rows > 0:
                batch.add(W, acts[key], M, out_local[:, off:], ld_out=slice_rows)
            off += pad_rows
    batch.seal()
    # all inputs of a step in one pinned host buffer, outputs in another (the end-to-end leg copies both every step)
    rng = np.random.Generator(np.random.PCG64(4242))
    x_pinned = torch.from_numpy(rng.standard_normal(batch.input_floats, dtype=np.float32)).pin_memory()
    out_pinned = torch.zeros((M, slice_rows), dtype=torch.float32).pin_memory()
    batch.run_host(x_pinned.numpy(), out_local, out_pinned.numpy())  # uploads and quantizes the activations once
    launches_per_step = batch.launch_count

    # Fused gather (N > 1, up to four tokens): a second recording of the same ops whose outputs go straight into
    # every rank's assembled [M, sum of n_rows] buffer.
    fused = None
    use_fused = world > 1 and args.gather == "fused" and M <= 4
    if use_fused:
        full_cols = sum(n for _, n, _ in cfg["shapes"]) * cfg["layers"]
        mine = hb.PeerBuffer.alloc(M * full_cols)
        handles = [None] * world
        dist.all_gather_object(handles, mine.handle)
        bufs = [mine if r == rank else hb.PeerBuffer.open(handles[r], M * full_cols) for r in range(world)]
        full_local = mine.tensor(dev).view(M, full_cols)
        fused = hb.Batch()
        fused.set_peers(rank, bufs, wait=True)
        coff, i = 0, 0
        for li in range(cfg["layers"]):
            for ti, (name, n_rows, n_cols) in enumerate(cfg["shapes"]):
                W, _ = weights[i]
                i += 1
                lo, hi = shard_rows(n_rows, rank, world)
                if hi > lo:
                    fused.add(W, acts[(li, group_of.get(name, ti))], M, full_local[:, coff + lo:], ld_out=full_cols)
                coff += n_rows
        fused.seal()
        launches_per_step = fused.launch_count

    def step_nccl():
        batch.launch(stream)
        if world > 1:
            with torch.cuda.stream(stream):
                dist.all_gather_into_tensor(out_all, out_local)

    def step_fused():
        fused.launch(stream)

    step = step_fused if use_fused else step_nccl

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        t_end = time.perf_counter() + 0.7
    # An untimed burst of the same steps first, so that the clock sampler (100 ms period) has samples
    # under load on both sides of the timed region; rank 0 decides when it ends.
    burst = 0
    while burst < 4000 and not args.quick:
        step()
        burst += 1
        if burst % 50 == 0:
            stream.synchronize()
            flag = torch.tensor([1.0 if (rank == 0 and time.perf_counter() >= t_end) else 0.0], device=dev)
            if world > 1:
                dist.broadcast(flag, 0)
            if flag.item() > 0:
                break
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    for _ in range(0 if args.quick else 50):
        step()
    barrier()
    ms_nccl = None
    if use_fused:  # the same steps with the collective instead, for comparison
        hb.check_status()
        for _ in range(5):
            step_nccl()
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            step_nccl()
        e1.record(stream)
        barrier()
        ms_nccl = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([ms, ms_nccl or 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_nccl = float(t[0].item()), (float(t[1].item()) if ms_nccl else None)
    ms_per_step = ms / args.steps

    # ---- end to end through the host-buffer entry point: every step copies all inputs from pinned host memory,
    # quantizes, runs the recorded batch, (all-gathers) and copies the results back to pinned host memory.
    e2e_ms, h2d, d2h = None, 0, 0
    if not args.quick:
        xh, oh = x_pinned.numpy(), out_pinned.numpy()
        out_all_pinned = torch.zeros((world * M, slice_rows), dtype=torch.float32).pin_memory() if world > 1 else None
        empty = np.zeros(0, dtype=np.float32)
        full_pinned = torch.zeros((M, full_cols), dtype=torch.float32).pin_memory() if use_fused else None

        def e2e_step():
            if world == 1:
                batch.run_host(xh, out_local, oh)
            elif use_fused:
                fused.run_host(xh, full_local, full_pinned.numpy())  # the kernel itself assembles every rank's outputs
            else:
                batch.run_host(xh, out_local, empty)           # inputs in, compute; results stay on the device
                dist.all_gather_into_tensor(out_all, out_local)
                out_all_pinned.copy_(out_all, non_blocking=True)
                torch.cuda.synchronize()
        e2e_steps = max(1, min(args.steps, 20 if M <= 4 else 3))
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        tt = torch.tensor([dt], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt.item()) / e2e_steps * 1e3
        h2d = batch.input_floats * 4
        d2h = (full_pinned.numel() if use_fused else (out_all_pinned.numel() if world > 1 else out_pinned.numel())) * 4

    if rank == 0:
        ab = algorithmic_bytes(cfg)
        total_alg = ab["weights"] + ab["activations"] + ab["outputs"]
        value = ab["weights"] / (ms_per_step * 1e-3) / 1e9
        peak, peak_src = measured_peaks()
        per_rank_alg = total_alg / world
        achieved = per_rank_alg / (ms_per_step * 1e-3) / 1e9
        metric, unit = METRIC, UNIT
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "kernel": hb.selected_kernel(dtype, M), "peak_source": peak_src,
                "algorithmic_bytes_per_launch": per_rank_alg}
        if dtype in (42, 142) and M <= 4:
            # dram__bytes_read + dram__bytes_write of gemv_dp4a_kernel<Q2_0> from the ncu capture summarised in
            # profiles/gemv_dp4a_q2_0__c1_1p7b_decode.md (1.7B layer set, 1.008 x its algorithmic bytes), scaled to this
            # launch by algorithmic bytes: every launch streams each weight byte exactly once.
            roof["traffic"] = 1.008 * per_rank_alg
            roof["traffic_source"] = "ncu capture of the same kernel on the 1.7B layer set, scaled by algorithmic bytes"
        if is_prefill(cfg):
            metric, unit = PREFILL_METRIC, PREFILL_UNIT
            value = total_ops(cfg) / (ms_per_step * 1e-3) / 1e12
            tpeak, tsrc = tensor_peak(hb)
            per_rank_tops = value / world
            roof = {"bound": "tensor", "achieved": per_rank_tops, "peak": tpeak, "unit": "TOP/s", "frac": per_rank_tops / tpeak,
                    "traffic": None, "kernel": hb.selected_kernel(dtype, M), "peak_source": tsrc,
                    "ops_per_step": total_ops(cfg), "weight_stream_gbs": ab["weights"] / (ms_per_step * 1e-3) / 1e9}
        line = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 x {1,2}-bit -> int32, fp32 scales", "data": "synthetic",
            "config": {"workload": args.workload, "format": {41: "Q1_0", 43: "Q1_0_G128", 42: "Q2_0", 142: "PQ2_0", 143: "PTQ1_0", 8: "Q8_0", 12: "Q4_K", 14: "Q6_K"}.get(dtype, str(dtype)),
                       "tokens": M, "layers": cfg["layers"], "matrices_per_step": cfg["layers"] * len(cfg["shapes"]),
                       "weight_bytes": ab["weights"], "parallelism": f"rows/{world}" + ((" + outputs stored to all ranks from the kernel (peer stores, flag exchange)" if use_fused
                                                                else " + NCCL all-gather of output slices") if world > 1 else ""),
                       "l2": "per-GPU inputs exceed the 126 MB L2" if ab["weights"] / world > 126e6 else "inputs fit in L2",
                       "launch": "one recorded batch (work list) per step"},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": roof,
            "e2e": ({"value": (total_ops(cfg) / (e2e_ms * 1e-3) / 1e12) if is_prefill(cfg) else ab["weights"] / (e2e_ms * 1e-3) / 1e9, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                     "ms_per_step": e2e_ms, "call": "hb200_batch_run_host: the step's inputs up, list quantize, recorded batch, every output back; pinned host buffers; single-token steps run as eight pipelined runs (upload, compute and readback streams)"} if e2e_ms else None),
        }
        if ms_nccl:
            line["nccl_allgather_variant"] = {"ms_per_step": ms_nccl / args.steps,
                                              "value": ab["weights"] / (ms_nccl / args.steps * 1e-3) / 1e9, "unit": UNIT}
        if world == 1 and not args.no_cpu and not args.quick:
            arm = CpuArm(cfg, 0, 1)
            t0 = time.perf_counter()
            best = arm.gbs(2)
            while time.perf_counter() - t0 < 8.0:  # bounded: about ten seconds of CPU work
                best = max(best, arm.gbs(2))
            # one thread, as the reference's benchk measures its kernels (300 ms warm-up, best of two passes,
            # hearth-llm/examples/benchk.rs:172-198)
            threads_used, desc, nbytes, ops = arm.threads, arm.desc, arm.nbytes, arm.ops
            arm.S.hs_pool_start(1)
            t1 = time.perf_counter() + 0.3
            while time.perf_counter() < t1:
                arm.one_pass()
            single = arm.gbs(2)
            arm.close()
            if is_prefill(cfg):  # same unit as the line: ops of the sample / time
                best = best * 1e9 / nbytes * ops / 1e12
                single = single * 1e9 / nbytes * ops / 1e12
            line["cpu_baseline"] = {"value": best, "unit": unit, "cores": threads_used, "kind": "port", "sample": desc,
                                    "single_thread": single, "cpu_model": cpu_model()}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(synth.CONFIGS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: 'fused' stores every output into all ranks' buffers from the kernel (peer stores + flag "
                         "exchange); 'nccl' runs an all-gather of the output slices after the kernel")
    ap.add_argument("--quick", action="store_true",
                    help="kernel timing only: no clock-sampling burst, no end-to-end leg, no CPU leg (for profiler runs)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = synth.CONFIGS[args.workload]
    if args.impl == "reference":
        run_reference(args, cfg, rank)
        return
    if world != args.gpus:
        if args.gpus > 1 and world == 1:
            raise SystemExit("bench.py: launch with torch.distributed.run for --gpus > 1")
    run_ours(args, cfg, rank, world, local_rank)


if __name__ == "__main__":
    main()
