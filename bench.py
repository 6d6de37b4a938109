#!/usr/bin/env python
"""Benchmark of the B200 quantized matrix-product path.

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--impl reference]

A step is one pass of the decode (or prefill) layer set: every projection of
every layer of the named model shape against synthetic Q8_0 activations.  The
metric is the reference benchmark's own (hearth-llm/examples/benchk.rs:162,
:198): packed weight bytes streamed per second.  With N > 1 every weight is
row-sharded over the ranks (rank r holds rows [r*ceil(n/N), ...)); by default the
decode kernel itself stores every output into all ranks' buffers over NVLink
(peer stores and a flag exchange; --gather nccl runs an NCCL all-gather of the
output slices after the kernel instead), so the total work is fixed ("strong"
scaling).  What the ranks assemble is compared across ranks and with the CPU
checker before anything is timed.  The default run also times the other
workloads of the metric (prefill, the 8B and 1.7B decode sets, the K-quant
configuration) and reports them under "secondary".  Prints one JSON line on
rank 0.
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

GROUP_OF = {"q": 0, "k": 0, "v": 0, "o": 1, "gate": 2, "up": 2, "down": 3}
FORMAT_NAME = {41: "Q1_0", 43: "Q1_0_G128", 42: "Q2_0", 142: "PQ2_0", 143: "PTQ1_0", 8: "Q8_0", 12: "Q4_K", 14: "Q6_K"}
NOMINAL_HBM_GBS = 8000.0  # the figure the path's brief quotes its decode target against

# Workloads timed after the headline one and reported under "secondary" (device-timed, inputs resident):
# the prefill half of the metric, the decode shapes the 70 % target is quoted on, the 1.7B sets, the K-quant
# configuration at its three token counts, a Q8_0-weight set, and the single 6144 x 2048 matvec.
SECONDARY_1GPU = ["c2_q1_8b_prefill", "c2_q1_8b_decode", "c2_q2_8b_decode", "c1_q1_1p7b_decode", "c1_q2_1p7b_decode",
                  "c3_q4k_m1", "c3_q4k_m8", "c3_q4k_m32", "c3_q6k_m1", "c3_q6k_m8", "c3_q6k_m32", "c1_q8_1p7b_decode",
                  "c4_pq2_27b_m32", "c0_q1_single_x160"]
SECONDARY_MULTI = ["c4_pq2_27b_m32"]


def weight_seed(li: int, ti: int, rank: int) -> int:
    return 1000 * (li + 1) + 10 * ti + rank


class Workload:
    """One configuration resident on this rank: its row shard of every weight, one activation per input-sharing group
    of each layer (q|k|v read one vector, o another, gate|up a third, down a fourth, hearth-llm/src/model/mod.rs:527-775)
    and the recorded batch that writes a packed [M, slice_rows] buffer."""

    def __init__(self, hb, torch, cfg, rank, world, dev):
        self.hb, self.torch, self.cfg, self.rank, self.world, self.dev = hb, torch, cfg, rank, world, dev
        M, dtype = cfg["seq_len"], cfg["dtype"]
        self.M = M
        self.weights, self.acts, self.act_offset = [], {}, {}
        self.slice_rows = 0
        for li in range(cfg["layers"]):
            for ti, (_, n_rows, n_cols) in enumerate(cfg["shapes"]):
                lo, hi = shard_rows(n_rows, rank, world)
                packed = synth.weights_torch(dtype, hi - lo, n_cols, seed=weight_seed(li, ti, rank), device=dev)
                self.weights.append((hb.Weight.upload_dev(dtype, hi - lo, n_cols, packed), -(-n_rows // world)))
                del packed
                self.slice_rows += -(-n_rows // world)
        torch.cuda.synchronize()
        self.out_local = torch.zeros((M, self.slice_rows), dtype=torch.float32, device=dev)
        self.batch = hb.Batch()
        off, i, x_off = 0, 0, 0
        for li in range(cfg["layers"]):
            for ti, (name, n_rows, n_cols) in enumerate(cfg["shapes"]):
                W, pad_rows = self.weights[i]
                i += 1
                key = (li, GROUP_OF.get(name, ti))
                if W.n_rows > 0:
                    if key not in self.acts:
                        self.acts[key] = hb.Act(M, n_cols)
                        self.act_offset[key] = x_off            # the batch lists inputs in order of first use, 16-byte aligned
                        x_off = (x_off + M * n_cols + 3) & ~3
                    self.batch.add(W, self.acts[key], M, self.out_local[:, off:], ld_out=self.slice_rows)
                off += pad_rows
        self.batch.seal()
        assert self.batch.input_floats == x_off, (self.batch.input_floats, x_off)
        rng = np.random.Generator(np.random.PCG64(4242))
        self.x_pinned = torch.from_numpy(rng.standard_normal(max(x_off, 1), dtype=np.float32)).pin_memory()
        self.out_pinned = torch.zeros((M, self.slice_rows), dtype=torch.float32).pin_memory()
        # uploads and quantizes the activations once, so that device-only steps have their inputs resident
        self.batch.run_host(self.x_pinned.numpy(), self.out_local, self.out_pinned.numpy())

    def free(self):
        self.batch.free()
        for a in self.acts.values():
            a.free()
        for W, _ in self.weights:
            W.free()
        self.weights, self.acts = [], {}
        del self.out_local
        self.torch.cuda.empty_cache()


def roofline_of(hb, cfg, ms_per_step, world):
    """(metric, unit, value, roofline dict) of one device-timed step of cfg."""
    ab = algorithmic_bytes(cfg)
    total_alg = ab["weights"] + ab["activations"] + ab["outputs"]
    kernel = hb.selected_kernel(cfg["dtype"], cfg["seq_len"])
    if is_prefill(cfg):
        value = total_ops(cfg) / (ms_per_step * 1e-3) / 1e12
        tpeak, tsrc = tensor_peak(hb)
        per_rank = value / world
        return PREFILL_METRIC, PREFILL_UNIT, value, {
            "bound": "tensor", "achieved": per_rank, "peak": tpeak, "unit": "TOP/s", "frac": per_rank / tpeak, "traffic": None,
            "kernel": kernel, "peak_source": tsrc, "ops_per_step": total_ops(cfg),
            "weight_stream_gbs": ab["weights"] / (ms_per_step * 1e-3) / 1e9}
    peak, peak_src = measured_peaks()
    per_rank_alg = total_alg / world
    achieved = per_rank_alg / (ms_per_step * 1e-3) / 1e9
    return METRIC, UNIT, ab["weights"] / (ms_per_step * 1e-3) / 1e9, {
        "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        "frac_of_nominal_8tbs": achieved / NOMINAL_HBM_GBS, "traffic": None, "kernel": kernel, "peak_source": peak_src,
        "algorithmic_bytes_per_launch": per_rank_alg}


def time_secondary(hb, torch, dist, name, rank, world, dev, stream, steps):
    """Device-timed steps of one more workload (weights generated, timed, freed).  N > 1: row shards + NCCL gather; the
    layer set then runs as eight recorded batches of consecutive layers, and the all-gather of each batch's output
    slices runs on a second stream under the kernels of the next one (at 32 tokens the outputs are 428 MB per step: gathered
    in one piece behind the last kernel they cost as much as a rank's share of the compute at eight ranks)."""
    cfg = synth.CONFIGS[name]
    n_parts = 8 if (world > 1 and cfg["layers"] >= 8) else 1
    parts = []
    for k in range(n_parts):
        c = dict(cfg)
        c["layers"] = cfg["layers"] * (k + 1) // n_parts - cfg["layers"] * k // n_parts
        parts.append(Workload(hb, torch, c, rank, world, dev))
    wl = parts[0]
    outs_all = [torch.zeros((world * p.M, p.slice_rows), dtype=torch.float32, device=dev) for p in parts] if world > 1 else None
    comm = torch.cuda.Stream(device=dev) if world > 1 else None
    done = [torch.cuda.Event() for _ in parts]

    def step():
        for k, p in enumerate(parts):
            p.batch.launch(stream)
            if world > 1:
                done[k].record(stream)
                comm.wait_event(done[k])
                with torch.cuda.stream(comm):
                    dist.all_gather_into_tensor(outs_all[k], p.out_local)
        if world > 1:
            stream.wait_stream(comm)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(3):
        step()
    barrier()
    hb.check_status()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    launches = sum(p.batch.launch_count for p in parts)
    for p in parts:
        p.free()
    metric, unit, value, roof = roofline_of(hb, cfg, ms, world)
    ab = algorithmic_bytes(cfg)
    entry = {"workload": name, "format": FORMAT_NAME.get(cfg["dtype"], str(cfg["dtype"])), "tokens": cfg["seq_len"],
             "metric": metric, "value": value, "unit": unit, "ms_per_step": ms, "steps": steps, "gpu_launches_per_step": launches,
             "weight_bytes": ab["weights"], "kernel": roof["kernel"],
             "roofline": {k: roof[k] for k in ("bound", "achieved", "peak", "unit", "frac") if k in roof},
             "l2": "per-GPU inputs exceed the 126 MB L2" if ab["weights"] / world > 126e6 else "inputs fit in L2"}
    if "frac_of_nominal_8tbs" in roof:
        entry["roofline"]["frac_of_nominal_8tbs"] = roof["frac_of_nominal_8tbs"]
    if world > 1:
        entry["gather"] = f"NCCL all-gather of output slices, {n_parts} pieces, each under the kernels of the next piece"
    if name.startswith("c0_q1_single_x"):
        n = cfg["layers"]
        entry["note"] = (f"the single 6144 x 2048 Q1_0 matvec (1.77 MB, shorter than a launch and L2-resident when repeated) is "
                         f"timed as one launch over {n} distinct copies of the weight ({ab['weights'] / 1e6:.0f} MB, more than "
                         f"twice the L2), and reported per matrix")
        entry["us_per_matrix"] = ms * 1e3 / n
    return entry


def time_producers(hb, torch, dev, stream, steps=5):
    """Device-timed activation producers, one launch each over an input larger than the L2 (the shapes of an 8B model,
    4096 or 12288 tokens): the Q8_0 quantizer (hearth-quant/src/q8_0.rs:20-51) alone and fused behind the RMS norm, the
    gated activation and the Hadamard rotation (hearth-llm/src/ops.rs:489, :273; model/qwen35.rs:924-943).  Algorithmic
    bytes per element: the f32 inputs read, one int8 and 2 x 4 / 32 bytes of block values written."""
    peak, _ = measured_peaks()
    out = []

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def entry(name, kernel, ms, n_elem, in_bytes_per_elem, shape):
        alg = n_elem * (in_bytes_per_elem + 1.25)
        gbs = alg / (ms * 1e-3) / 1e9
        return {"producer": name, "kernel": kernel, "shape": shape, "launches_per_step": 1, "ms_per_step": ms,
                "algorithmic_bytes_per_step": alg,
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak}}

    gen = torch.Generator(device=dev)
    gen.manual_seed(77)
    M, K = 4096, 12288  # 201 MB of f32 per input
    x = torch.randn((M, K), generator=gen, device=dev, dtype=torch.float32)
    up = torch.randn((M, K), generator=gen, device=dev, dtype=torch.float32)
    act = hb.Act(M, K)
    ms = timed(lambda: act.quantize(M, x_dev=x, stream=stream))
    out.append(entry("quantize_q8_0", "quantize_q8_0_kernel", ms, M * K, 4, f"[{M}][{K}]"))
    ms = timed(lambda: act.silu_mul_q8(x, up, M, stream=stream))
    out.append(entry("silu_mul_q8", "silu_mul_q8_kernel", ms, M * K, 8, f"2 x [{M}][{K}]"))
    act.free()
    del x, up
    M, K = 12288, 4096
    x = torch.randn((M, K), generator=gen, device=dev, dtype=torch.float32)
    act = hb.Act(M, K)
    wt = torch.rand((K,), generator=gen, device=dev, dtype=torch.float32) + 0.5
    ms = timed(lambda: act.rms_norm_q8(x, wt, 1e-6, M, stream=stream))
    out.append(entry("rms_norm_q8", "rms_norm_q8_kernel", ms, M * K, 4, f"[{M}][{K}]"))
    signs = torch.where(torch.rand((K,), generator=gen, device=dev) < 0.5, -1.0, 1.0).to(torch.float32)
    ms = timed(lambda: act.hadamard_quantize(M, 256, x_dev=x, signs_dev=signs, stream=stream))
    out.append(entry("hadamard_quantize_q8_0", "hadamard_quantize_kernel", ms, M * K, 4, f"[{M}][{K}], blocks of 256"))
    act.free()
    hb.check_status()
    return out


def time_f32act(hb, torch, dev, stream, steps=5):
    """The f32-activation matvec (the arithmetic of the reference's GPU shader, hearth-compute/src/shaders/q1_0_matmul.wgsl:38-97,
    dispatched by GpuCompute::dequant_matmul_cached, hearth-compute/src/lib.rs:104-251) at the 8B gate shape, one token:
    40 distinct 12288 x 4096 Q1_0 weights (283 MB, more than twice the L2), one launch each per step."""
    peak, _ = measured_peaks()
    n_rows, n_cols, n = 12288, 4096, 40
    ws = [hb.Weight.upload_dev(41, n_rows, n_cols, synth.weights_torch(41, n_rows, n_cols, 900 + i, dev)) for i in range(n)]
    x = torch.randn((1, n_cols), device=dev, dtype=torch.float32)
    out = torch.zeros((1, n_rows), device=dev, dtype=torch.float32)

    def step():
        for w in ws:
            hb.dequant_matmul_f32act_dev(w, x, 1, out, stream=stream)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    wbytes = n * n_rows * (n_cols // 128) * 18
    for w in ws:
        w.free()
    hb.check_status()
    gbs = wbytes / (ms * 1e-3) / 1e9
    return {"workload": "f32act_q1_12288x4096_m1_x40", "format": "Q1_0", "tokens": 1, "metric": METRIC, "value": gbs, "unit": UNIT,
            "ms_per_step": ms, "us_per_matrix": ms * 1e3 / n, "steps": steps, "gpu_launches_per_step": n, "weight_bytes": wbytes,
            "kernel": "f32act_q1_0",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak},
            "l2": "per-GPU inputs exceed the 126 MB L2",
            "note": "f32 activations, the shader's 128-leaf reduction tree per block; one launch per matrix"}


def shared_pinned(torch, name, n_floats, rank, world, dist):
    """One float32 host buffer shared by all ranks of the node (a file in /dev/shm mapped by every process) and
    page-locked in each of them, so that each rank's readback lands in its own part of ONE host buffer.
    Returns (numpy array, page-locked?, cleanup)."""
    import mmap
    nbytes = max(n_floats, 1) * 4
    path = os.path.join("/dev/shm", name)
    if rank == 0:
        with open(path, "wb") as f:
            f.truncate(nbytes)
    if world > 1:
        dist.barrier()
    f = open(path, "r+b")
    mm = mmap.mmap(f.fileno(), nbytes)
    f.close()
    arr = np.frombuffer(mm, dtype=np.float32, count=n_floats)
    rt = torch.cuda.cudart()
    try:
        registered = int(rt.cudaHostRegister(arr.ctypes.data, nbytes, 0)) == 0
    except RuntimeError:
        registered = False

    def cleanup():
        if registered:
            rt.cudaHostUnregister(arr.ctypes.data)
        if world > 1:
            dist.barrier()
        if rank == 0:
            try:
                os.unlink(path)
            except OSError:
                pass
    return arr, registered, cleanup


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

    wl = Workload(hb, torch, cfg, rank, world, dev)
    batch, acts, weights, out_local, slice_rows = wl.batch, wl.acts, wl.weights, wl.out_local, wl.slice_rows
    x_pinned, out_pinned = wl.x_pinned, wl.out_pinned
    out_all = torch.zeros((world * M, slice_rows), dtype=torch.float32, device=dev) if world > 1 else None  # [world][M][slice]
    launches_per_step = batch.launch_count

    # Fused gather (N > 1, up to four tokens): a second recording of the same ops whose outputs go straight into
    # every rank's assembled [M, sum of n_rows] buffer.  Every buffer holds two such areas, written by alternate
    # launches, so a rank that runs one step ahead never overwrites what a slower rank still reads.
    fused = None
    use_fused = world > 1 and args.gather == "fused" and M <= 4
    full_cols = sum(n for _, n, _ in cfg["shapes"]) * cfg["layers"]
    area = (M * full_cols + 3) & ~3
    if use_fused:
        mine = hb.PeerBuffer.alloc(2 * area)
        handles = [None] * world
        dist.all_gather_object(handles, mine.handle)
        bufs = [mine if r == rank else hb.PeerBuffer.open(handles[r], 2 * area) for r in range(world)]
        full_both = mine.tensor(dev)
        full_area0 = full_both[:M * full_cols].view(M, full_cols)
        fused = hb.Batch()
        fused.set_peers(rank, bufs, wait=True, area_floats=area)
        coff, i = 0, 0
        for li in range(cfg["layers"]):
            for ti, (name, n_rows, n_cols) in enumerate(cfg["shapes"]):
                W, _ = weights[i]
                i += 1
                lo, hi = shard_rows(n_rows, rank, world)
                if hi > lo:
                    fused.add(W, acts[(li, GROUP_OF.get(name, ti))], M, full_area0[:, coff + lo:], ld_out=full_cols)
                coff += n_rows
        fused.seal()
        launches_per_step = fused.launch_count

        def full_latest():
            a = fused.peer_area
            return full_both[a * area:a * area + M * full_cols].view(M, full_cols)

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

    # ---- N > 1: what the ranks assembled is checked before anything is timed.  Every rank must hold the same bits,
    # and rank 0 recomputes whole row shards of three matrices (first, middle and last rank's) with the CPU checker
    # from the seeds the shards were generated with.
    multi_check, assembled_host = None, None
    if world > 1:
        hb.check_status()
        if use_fused:
            mine_full = full_latest().clone()
        else:
            g = out_all.view(world, M, slice_rows)
            parts, off = [], 0
            for li in range(cfg["layers"]):
                for ti, (name, n_rows, n_cols) in enumerate(cfg["shapes"]):
                    chunk = -(-n_rows // world)
                    for r in range(world):
                        lo, hi = shard_rows(n_rows, r, world)
                        if hi > lo:
                            parts.append(g[r][:, off:off + (hi - lo)])
                    off += chunk
            mine_full = torch.cat(parts, dim=1).contiguous()
        ref_full = mine_full.clone()
        dist.broadcast(ref_full, 0)
        diff = (mine_full.view(torch.int32) != ref_full.view(torch.int32)).sum().to(torch.float64).reshape(1)
        nan_count = torch.isnan(mine_full).sum().to(torch.float64).reshape(1)
        dist.all_reduce(diff, op=dist.ReduceOp.MAX)
        dist.all_reduce(nan_count, op=dist.ReduceOp.MAX)
        identical = float(diff.item()) == 0.0 and float(nan_count.item()) == 0.0
        rows_checked, oracle_ok = 0, True
        if rank == 0 and dtype not in (12, 14):
            from oracle import oracle as O  # the CPU checker, used as a checker
            O.build()
            n_l, n_t = cfg["layers"], len(cfg["shapes"])
            picks = [(0, min(1, n_t - 1), 0), (n_l // 2, min(4, n_t - 1), world // 2), (n_l - 1, n_t - 1, world - 1)]
            col_of = {}
            coff = 0
            for li in range(n_l):
                for ti, (_, n_rows, _) in enumerate(cfg["shapes"]):
                    col_of[(li, ti)] = coff
                    coff += n_rows
            host_full = assembled_host = mine_full.cpu().numpy()
            xh = x_pinned.numpy()
            for li, ti, r in picks:
                name, n_rows, n_cols = cfg["shapes"][ti]
                lo, hi = shard_rows(n_rows, r, world)
                if hi <= lo:
                    continue
                hi = min(hi, lo + 512)
                w = synth.weights_torch(dtype, shard_rows(n_rows, r, world)[1] - lo, n_cols, seed=weight_seed(li, ti, r), device=dev)
                w = w.cpu().numpy().reshape(-1, synth.row_bytes(dtype, n_cols))[:hi - lo]
                xo = wl.act_offset[(li, GROUP_OF.get(name, ti))]
                q8 = O.quantize_q8_0(xh[xo:xo + M * n_cols].reshape(M, n_cols))
                want = O.dot_rows_batched(dtype, np.ascontiguousarray(w), q8, hi - lo, n_cols)
                c0 = col_of[(li, ti)] + lo
                got = np.ascontiguousarray(host_full[:, c0:c0 + (hi - lo)])
                oracle_ok = oracle_ok and bool((got.view(np.uint32) == want.view(np.uint32)).all())
                rows_checked += hi - lo
        flag = torch.tensor([1.0 if oracle_ok else 0.0, float(rows_checked)], dtype=torch.float64, device=dev)
        dist.broadcast(flag, 0)
        oracle_ok, rows_checked = bool(flag[0].item() > 0), int(flag[1].item())
        multi_check = {"ranks_identical": identical, "oracle_rows_checked": rows_checked, "oracle_bits_equal": oracle_ok,
                       "assembled_floats": int(mine_full.numel())}
        del mine_full, ref_full
        if not identical or not oracle_ok:
            if rank == 0:
                print(json.dumps({"error": "multi-GPU value check failed", "multi_gpu_check": multi_check}))
            dist.barrier()
            raise SystemExit(3)

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

    # ---- end to end through the host-buffer entry point: every step copies this rank's inputs from pinned host
    # memory, quantizes, runs the recorded batch and copies the results back to pinned host memory.  The consumer is
    # the host, so with N > 1 no device-side gather is needed: every rank reads back only the rows it computed, into
    # its own part of ONE page-locked host buffer shared by all ranks ([rank][M][slice]); the step is complete when
    # every rank's part has landed (barrier at the end of the timed region, maximum over ranks).
    e2e_ms, h2d, d2h, e2e_note = None, 0, 0, None
    if not args.quick:
        xh = x_pinned.numpy()
        cleanup = None
        if world == 1:
            oh = out_pinned.numpy()
        else:
            shared, registered, cleanup = shared_pinned(torch, f"hb200_bench_{os.environ.get('MASTER_PORT', '0')}",
                                                        world * M * slice_rows, rank, world, dist)
            oh = shared[rank * M * slice_rows:(rank + 1) * M * slice_rows].reshape(M, slice_rows)
            e2e_note = ("every rank reads back its own row slices into its part of one shared page-locked host buffer"
                        if registered else "shared host buffer could not be page-locked; pageable copies")

        # Inputs are replicated on the ranks.  Up to four ranks every rank uploads all of them, pipelined under its compute.
        # At eight ranks that upload (8.4 MB per rank, eight at a time through one host) takes twice as long as a rank's
        # share of the compute - measured: 0.422 ms end to end at four ranks, 0.440 at eight - so there every rank uploads
        # 1/G of the inputs and one NCCL all-gather assembles them on the devices before hb200_batch_run_dev: the host
        # links carry every input once per step.  (At four ranks that form measured slower, 0.49 ms: upload, collective
        # and compute run one after the other.)
        shard_inputs = world >= 8
        if shard_inputs:
            nfl = batch.input_floats
            per = -(-nfl // world)
            xg = torch.zeros(per * world, dtype=torch.float32, device=dev)
            lo, hi = rank * per, min((rank + 1) * per, nfl)

            def e2e_step():
                with torch.cuda.stream(stream):
                    if hi > lo:
                        xg[lo:hi].copy_(x_pinned[lo:hi], non_blocking=True)
                    dist.all_gather_into_tensor(xg, xg[rank * per:(rank + 1) * per])
                batch.run_dev(xg, out_local, oh, x_stream=stream)
            e2e_note = (e2e_note or "") + "; every rank uploads 1/G of the inputs, one NCCL all-gather assembles them on the devices (hb200_batch_run_dev)"
        else:
            def e2e_step():
                batch.run_host(xh, out_local, oh)
        e2e_steps = max(1, min(args.steps, 20 if M <= 4 else 3))
        for _ in range(2):
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
        # bytes summed over the ranks: every rank uploads every input (activations are replicated), each output once
        counts = torch.tensor([float(max(hi - lo, 0) * 4 if shard_inputs else batch.input_floats * 4), float(M * slice_rows * 4)],
                              dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(counts, op=dist.ReduceOp.SUM)
        h2d, d2h = int(counts[0].item()), int(counts[1].item())
        if world > 1:
            barrier()
            if rank == 0 and assembled_host is not None:
                # the shared host buffer must now hold, rank by rank, the rows the device-side assembly holds
                same, off, col = True, 0, 0
                parts = shared.reshape(world, M, slice_rows)
                for li in range(cfg["layers"]):
                    for ti, (name, n_rows, n_cols) in enumerate(cfg["shapes"]):
                        for r in range(world):
                            lo, hi = shard_rows(n_rows, r, world)
                            if hi > lo:
                                same = same and bool((parts[r][:, off:off + (hi - lo)].view(np.uint32) ==
                                                      assembled_host[:, col + lo:col + hi].view(np.uint32)).all())
                        off += -(-n_rows // world)
                        col += n_rows
                multi_check["host_buffer_equals_device_assembly"] = same
            cleanup()

    # ---- the other workloads of the metric
    secondary = []
    if not args.quick and not args.no_secondary and args.workload == DEFAULT_WORKLOAD:
        for name in (SECONDARY_1GPU if world == 1 else SECONDARY_MULTI):
            c2 = synth.CONFIGS[name]
            k = 3 if c2["seq_len"] >= 128 else (10 if c2["seq_len"] > 4 else 20)
            try:
                secondary.append(time_secondary(hb, torch, dist, name, rank, world, dev, stream, k))
            except Exception as e:  # noqa: BLE001 - one failed extra workload must not lose the headline line
                secondary.append({"workload": name, "error": f"{type(e).__name__}: {e}"})
        if world == 1:
            try:
                secondary.append(time_f32act(hb, torch, dev, stream))
            except Exception as e:  # noqa: BLE001
                secondary.append({"workload": "f32act_q1_12288x4096_m1_x40", "error": f"{type(e).__name__}: {e}"})

    producers = None
    if world == 1 and not args.quick and not args.no_secondary and args.workload == DEFAULT_WORKLOAD:
        try:
            producers = time_producers(hb, torch, dev, stream)
        except Exception as e:  # noqa: BLE001
            producers = [{"error": f"{type(e).__name__}: {e}"}]

    if rank == 0:
        ab = algorithmic_bytes(cfg)
        metric, unit, value, roof = roofline_of(hb, cfg, ms_per_step, world)
        if dtype in (42, 142) and M <= 4:
            # dram__bytes_read + dram__bytes_write of gemv_dp4a_kernel<Q2_0> from the ncu capture summarised in
            # profiles/gemv_dp4a_q2_0__c1_1p7b_decode.md (1.7B layer set, 1.008 x its algorithmic bytes), scaled to this
            # launch by algorithmic bytes: every launch streams each weight byte exactly once.
            roof["traffic"] = 1.008 * roof["algorithmic_bytes_per_launch"]
            roof["traffic_source"] = "ncu capture of the same kernel on the 1.7B layer set, scaled by algorithmic bytes"
        line = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 x {1,2}-bit -> int32, fp32 scales", "data": "synthetic",
            "config": {"workload": args.workload, "format": FORMAT_NAME.get(dtype, str(dtype)),
                       "tokens": M, "layers": cfg["layers"], "matrices_per_step": cfg["layers"] * len(cfg["shapes"]),
                       "weight_bytes": ab["weights"], "parallelism": f"rows/{world}" + ((" + outputs stored to all ranks from the kernel (peer stores, flag exchange, two output areas)" if use_fused
                                                                else " + NCCL all-gather of output slices") if world > 1 else ""),
                       "l2": "per-GPU inputs exceed the 126 MB L2" if ab["weights"] / world > 126e6 else "inputs fit in L2",
                       "launch": "one recorded batch (work list) per step"},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": roof,
            "e2e": ({"value": (total_ops(cfg) / (e2e_ms * 1e-3) / 1e12) if is_prefill(cfg) else ab["weights"] / (e2e_ms * 1e-3) / 1e9, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                     "ms_per_step": e2e_ms, "bytes_counted": "summed over ranks",
                     "call": "hb200_batch_run_host on every rank: the step's inputs up, list quantize, recorded batch, the rank's own outputs back; pinned host buffers; single-token steps run as six pipelined runs with short first and last ones (upload, compute and readback streams)"
                             + ("; " + e2e_note if e2e_note else "")} if e2e_ms else None),
        }
        if multi_check:
            line["multi_gpu_check"] = multi_check
        if ms_nccl:
            line["nccl_allgather_variant"] = {"ms_per_step": ms_nccl / args.steps,
                                              "value": ab["weights"] / (ms_nccl / args.steps * 1e-3) / 1e9, "unit": UNIT}
        if secondary:
            line["secondary"] = secondary
        if producers:
            line["producers"] = producers
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
    ap.add_argument("--no-secondary", action="store_true", help="skip the extra workloads reported under 'secondary'")
    ap.add_argument("--quick", action="store_true",
                    help="kernel timing only: no clock-sampling burst, no end-to-end leg, no CPU leg (for profiler runs)")
    ap.add_argument("--producers-only", action="store_true",
                    help="time only the activation producers (quantizer, fused norm / activation / rotation) on one GPU")
    args = ap.parse_args()
    if args.producers_only:
        import torch
        from hearth_b200 import api as hb
        hb.init(0)
        dev = torch.device("cuda:0")
        torch.cuda.set_device(dev)
        stream = torch.cuda.current_stream()
        k = max(1, min(args.steps, 5))
        print(json.dumps({"producers": time_producers(hb, torch, dev, stream, steps=k),
                          "f32act": time_f32act(hb, torch, dev, stream, steps=k)}), flush=True)
        return
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
