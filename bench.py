#!/usr/bin/env python
"""MoE-layer throughput benchmark (tokens/s) for the sm_100a MoE block.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape 120b|20b] [--tokens ROWS] [--zipf S] [--tp G] [--parallel tp|dp]
                    [--case headline|tokens|collectives|quantizer]

A step is one pass of the MoE block (router, top-4 + softmax, permutation,
MLP1 + SwiGLU, MLP2, weighted combine) over one batch of synthetic bf16 rows.
At N = 1 the workload is the GPT-OSS-120B-shape layer (128 experts, hidden and
intermediate 2880, MXFP4 weights) at 1856 rows.  At N > 1 the ranks form
tensor-parallel groups of min(N, 4) GPUs (the reference's deployments: TP2 x DP4
for the 20B model, TP4 x DP2 for the 120B one): every rank owns 1856 rows, the
block runs on the group's union with the intermediate dimension sharded, rows are
all-gathered before and reduce-scattered after by this library's peer-memory
kernels; more GPUs than one group add independent replicas.  `--parallel dp`
runs N independent replicas instead.  The value is rows of all ranks per second.

One JSON line is printed by rank 0.  `value` is device-resident throughput
(CUDA events on the launching stream), `e2e` goes through the host-buffer entry points
(moe_forward_host_submit/_wait, three batches in flight, every rank of a TP group with its own rows) with
pinned host buffers (every step's copies inside the timed region), `roofline` describes the
dominant kernel (the MLP1 grouped GEMM) from per-stage CUDA events, `parity` compares rank 0's
first rows of the result that travelled back through the host call with the CPU oracle, and
`cpu_baseline` times the reference's own CPU forward() on the host cores over a
bounded sample of the same workload.

--impl reference times that CPU code alone (oracle/_ref when the reference
binary is present, else this repository's C restatement of it).

--case selects the secondary measurements (one JSON line per sub-case; the headline
line above is what the contract reads):
  tokens        one GPU: rows in {1, 32, 256, 1856, 8192} (or --rows), uniform or --zipf S routing
  collectives   N GPUs (torchrun): all-gather / reduce-scatter of bf16 [T, 2880] for T in
                {64, 256, 1536, 1856, 8192}, peer-memory kernels vs NCCL
  quantizer     one GPU: the load-time fp32 -> MXFP4 quantiser over 2^28 values
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
SHAPES = {"120b": dict(E=128, H=2880, D=2880, K=4, name="GPT-OSS-120B"),
          "20b": dict(E=32, H=2880, D=2880, K=4, name="GPT-OSS-20B")}
CPU_SAMPLE_TOKENS = 32
PARITY_ROWS = 64
# dram read+write bytes / algorithmic bytes of the expert MLP kernel, from an ncu capture of a 4x smaller case
# (20B shape, 464 rows: the same rows per expert); traffic is proportional to the weights streamed
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.027


def tp_size_for(n_gpus: int, parallel: str, tp_arg: int) -> int:
    """TP group size at N GPUs: the reference's deployments (TP2 x DP4 for 20B, TP4 x DP2 for 120B,
    getp-csrc/getp_run.cpp:1850-1853) cap the group at 4; more GPUs add data-parallel replicas of it."""
    if n_gpus == 1 or parallel == "dp":
        return 1
    tp = tp_arg if tp_arg > 0 else min(n_gpus, 4)
    assert n_gpus % tp == 0
    return tp


def workload_config(shape: dict, tokens: int, n_gpus: int, parallel: str = "tp", tp_arg: int = 0,
                    zipf: float | None = None) -> dict:
    tp = tp_size_for(n_gpus, parallel, tp_arg)
    if n_gpus == 1:
        par = "tp1"
    elif tp > 1:
        par = (f"tp{tp} x dp{n_gpus // tp}: intermediate dimension sharded over {tp} GPUs, every rank owns {tokens} "
               f"rows, the block runs on the group's union of {tp * tokens} rows; all-gather before and "
               f"reduce-scatter after by peer-memory kernels over NVLink; groups are independent replicas")
    else:
        par = f"tp1 x dp{n_gpus} (independent replicas, no collective)"
    wbytes = shape["E"] * (3 * shape["H"] * shape["D"]) * 17 // 32
    return {
        "workload": f"{shape['name']}-shape MoE layer (E={shape['E']}, top-{shape['K']}, hidden {shape['H']}, "
                    f"intermediate {shape['D']}, MXFP4 weights, E8M0 scales), {tokens} bf16 rows per GPU, seed 0"
                    + (f", router bias for Zipf({zipf}) expert popularity" if zipf else ""),
        "rows_per_gpu": tokens,
        "parallelism": par,
        "l2_policy": f"inputs larger than L2: {wbytes / 1e9:.2f} GB of expert weights are streamed every step "
                     f"(L2 is 126 MB)",
    }


def peaks() -> tuple[float, float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            m = json.load(f)
        return float(m["hbm_gbs"]), float(m.get("bf16_tflops_sustained", m["bf16_tflops"])), "measured"
    return 6650.0, 1400.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid: str | None):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        cmd = ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20"]
        if uuid:
            cmd += ["-i", uuid]
        try:
            self.p = subprocess.Popen(cmd, stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0])); smax.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.f.close()
        os.unlink(self.f.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # "under load": samples in the upper half of the observed power range
        thr = (min(power) + max(power)) / 2
        loaded = [c for c, w in zip(sm, power) if w >= thr] or sm
        return {"sm_mhz": float(np.median(loaded)), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


def _oracle():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle
    return oracle


def cpu_reference_arm(layer, tokens_bits, steps: int, warmup: int):
    """Times the reference CPU path on `tokens_bits` (a bounded sample) with all the host's physical cores
    (set explicitly: a launcher such as torchrun exports OMP_NUM_THREADS=1 to its children).  Returns
    (tokens/s, kind, cores, ms per pass, outputs of the last pass as (logits, idx, w, out))."""
    oracle = _oracle()
    n = tokens_bits.shape[0]
    cores = oracle.host_cores()
    if oracle.reference_available():
        ref = oracle.Reference(layer)
        ref.set_threads(cores)
        ref.prepare(tokens_bits)          # load-time dequantisation, not part of the forward
        run, kind, cores = (lambda: ref.forward(tokens_bits)), "reference", ref.threads()
    else:
        port = oracle.Port()
        port.set_threads(cores)
        run, kind, cores = (lambda: port.moe_layer(layer, tokens_bits)), "port", port.threads()
    last = None
    for _ in range(warmup):
        last = run()
    t0 = time.perf_counter()
    for _ in range(steps):
        last = run()
    dt = time.perf_counter() - t0
    return steps * n / dt, kind, cores, dt / steps * 1e3, last


def parity_figures(synth, got_bits, ref_out, got_idx, ref_idx, ref_logits, got_f32=None, tp: int = 1) -> dict:
    """Raw error figures of `got_bits` (bf16 bit patterns) against the oracle's float output for the same rows.
    Rows whose expert selection differs from the oracle's are counted and left out of the output figures
    (allowed only where the oracle's own logits are within 1e-5 at the place that differs).  In a TP group
    every rank's partial travels as bf16 and the sum is rounded once more (as in the reference,
    getp_run.cpp:3206-3246): the max-abs bound grows by half a bf16 ulp of the largest output per rounding."""
    same = (got_idx == ref_idx).all(axis=1)
    k = ref_idx.shape[1]
    srt = np.sort(ref_logits, axis=1)[:, ::-1]
    near_tie = (srt[:, :k] - srt[:, 1:k + 1]).min(axis=1) < 1e-5
    got = synth.bf16_bits_to_f32(got_bits).astype(np.float64)[same]
    ref = ref_out.astype(np.float64)[same]
    err = np.abs(got - ref)
    rms = float(np.sqrt((ref ** 2).mean()))
    floor = np.abs(synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(ref.astype(np.float32))).astype(np.float64) - ref)
    max_bound = 2e-2 * max(1.0, rms) + ((tp + 1) * 2.0 ** -9 * float(np.abs(ref).max()) if tp > 1 else 0.0)
    out = {"rows": int(len(same)), "selection_mismatches": int((~same).sum()),
           "selection_mismatches_with_clear_gap": int((~same & ~near_tie).sum()),
           "max_abs": float(err.max()), "rms_ref": rms, "max_abs_over_rms": float(err.max() / rms),
           "mean_rel": float(err.mean() / np.abs(ref).mean()),
           "max_abs_of_bf16_rounding_alone": float(floor.max()),
           "bounds": "mean_rel <= 5e-3; max_abs <= 2e-2 * max(1, rms_ref)"
                     + (f" + {tp + 1} x 2^-9 x max|ref| (bf16 partials of {tp} ranks and their rounded sum)" if tp > 1 else ""),
           "max_abs_bound": max_bound,
           "within_bounds": bool(err.mean() / np.abs(ref).mean() <= 5e-3 and err.max() <= max_bound
                                 and not (~same & ~near_tie).any())}
    if got_f32 is not None:
        e32 = np.abs(got_f32.astype(np.float64)[same] - ref)
        out["f32_before_rounding"] = {"max_abs": float(e32.max()), "max_abs_over_rms": float(e32.max() / rms),
                                      "mean_rel": float(e32.mean() / np.abs(ref).mean())}
    return out


# --------------------------------------------------------------------------------------------------
# secondary cases
# --------------------------------------------------------------------------------------------------

def case_tokens(args, shape):
    """Token-count sweep on one GPU, uniform or skewed routing: time per block against the roofline of the
    algorithmic work (bytes of the experts that received rows / measured HBM rate, flops / measured bf16 rate)."""
    import torch
    pkg = importlib.import_module("gpt-oss_b200")
    synth = pkg.synth
    E, H, D, K = shape["E"], shape["H"], shape["D"], shape["K"]
    hbm, tc, _ = peaks()
    layer = synth.make_layer(E, H, D, seed=0, zipf_s=args.zipf)
    rows = [int(x) for x in (args.rows or "1,32,256,1856,8192").split(",")]
    blk = pkg.MoeBlock(H, D, E, top_k=K, max_rows=max(rows))
    blk.load_layer(0, layer)
    stream = torch.cuda.current_stream()
    for T in rows:
        tokens = synth.make_tokens(T, H, seed=0)
        d_t = torch.from_numpy(tokens.view(np.int16)).cuda()
        d_o = torch.empty_like(d_t)
        for _ in range(max(args.warmup, 3)):
            blk.forward(0, d_t.data_ptr(), T, d_o.data_ptr(), 0, stream.cuda_stream)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            blk.forward(0, d_t.data_ptr(), T, d_o.data_ptr(), 0, stream.cuda_stream)
        e1.record(stream)
        torch.cuda.synchronize()
        blk.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        counts = blk.debug(pkg.DBG_COUNTS)
        active = int((counts > 0).sum())
        # the same call captured once in a CUDA graph and replayed (the call is stream-ordered work only): what a
        # caller pays per layer when it does not launch the kernels one by one from the host
        side = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            blk.forward(0, d_t.data_ptr(), T, d_o.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(args.steps):
            g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        blk.synchronize()
        ms_graph = e0.elapsed_time(e1) / args.steps
        flops, nbytes = synth.algorithmic_work(T, H, D, E, K, active)
        roof_ms = max(nbytes / hbm / 1e6, flops / tc / 1e9)
        print(json.dumps({"case": "tokens", "shape": shape["name"], "zipf": args.zipf, "rows": T, "ms_per_block": ms,
                          "ms_per_block_cuda_graph": ms_graph,
                          "tokens_per_s": T / ms * 1e3, "active_experts": active,
                          "max_rows_per_expert": int(counts.max()), "roofline_ms": roof_ms,
                          "frac_of_roofline": roof_ms / ms}), flush=True)
    blk.close()


def case_quantizer(args):
    """The load-time quantiser alone: 4 bytes read and 17/32 byte written per element."""
    import torch
    pkg = importlib.import_module("gpt-oss_b200")
    hbm, _, _ = peaks()
    n = 1 << 28
    src = torch.randn(n, device="cuda", dtype=torch.float32)
    codes = torch.empty(n // 2, dtype=torch.uint8, device="cuda")
    scales = torch.empty(n // 32, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream()
    run = lambda: pkg.quantize_mxfp4(src.data_ptr(), n, codes.data_ptr(), scales.data_ptr(), stream.cuda_stream)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        run()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    nbytes = n * 4 + n // 2 + n // 32
    print(json.dumps({"case": "quantizer", "elements": n, "ms": ms, "algorithmic_bytes": nbytes,
                      "achieved_gbs": nbytes / ms / 1e6, "hbm_peak_gbs": hbm,
                      "frac_of_measured_hbm": nbytes / ms / 1e6 / hbm}), flush=True)


def case_collectives(args):
    """All-gather and reduce-scatter of bf16 [T, 2880] alone over all the GPUs of the launch (one TP group)."""
    import torch
    import torch.distributed as dist
    pkg = importlib.import_module("gpt-oss_b200")
    tpmod = importlib.import_module("gpt-oss_b200.tp")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    gloo = dist.new_group(backend="gloo")
    H = 2880
    rows = [int(x) for x in (args.rows or "64,256,1536,1856,8192").split(",")]
    # T is the gathered row count; every rank contributes T / world rows.  The handle only lends its symmetric
    # buffers: a small layer whose intermediate size every group size up to 8 can split on 32-element blocks.
    blk = pkg.MoeBlock(H, 256, 8, max_rows=max(rows) + world, tp_size=world, tp_rank=rank, device=local)
    tpmod.attach_group(blk, rank, gloo)
    stream = torch.cuda.current_stream()

    def timed(fn):
        for _ in range(5):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(args.steps):
            fn()
        b.record(stream)
        torch.cuda.synchronize(); dist.barrier()
        t = torch.tensor([a.elapsed_time(b) / args.steps], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for T in rows:
        rl = max(T // world, 1)
        src = torch.randn((rl, H), device="cuda").to(torch.bfloat16)
        full = torch.empty((rl * world, H), dtype=torch.bfloat16, device="cuda")
        part = torch.randn((rl * world, H), device="cuda").to(torch.bfloat16)
        out = torch.empty((rl, H), dtype=torch.bfloat16, device="cuda")
        sp = stream.cuda_stream
        res = {
            "allgather_ms": {"peer_kernels": timed(lambda: blk.tp_allgather(src.data_ptr(), rl, sp)),
                             "nccl": timed(lambda: dist.all_gather_into_tensor(full, src))},
            "reduce_scatter_ms": {"peer_kernels": timed(lambda: blk.tp_reduce_scatter(rl, out.data_ptr(), sp)),
                                  "nccl": timed(lambda: dist.reduce_scatter_tensor(out, part))},
        }
        blk.synchronize()
        if rank == 0:
            per_dir = (world - 1) * rl * H * 2
            res.update({"case": "collectives", "gpus": world, "rows_gathered": rl * world,
                        "bytes_per_rank_per_direction": per_dir,
                        "allgather_gbs": {k: per_dir / v / 1e6 for k, v in res["allgather_ms"].items()},
                        "reduce_scatter_gbs": {k: per_dir / v / 1e6 for k, v in res["reduce_scatter_ms"].items()}})
            print(json.dumps(res), flush=True)
    blk.close()
    dist.destroy_process_group()


# --------------------------------------------------------------------------------------------------
# headline
# --------------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="120b", choices=sorted(SHAPES))
    ap.add_argument("--tokens", type=int, default=1856, help="rows per GPU")
    ap.add_argument("--zipf", type=float, default=None, help="router bias for Zipf(s) expert popularity")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parallel", default="tp", choices=["tp", "dp"],
                    help="at N > 1: tensor-parallel groups (default) or N independent replicas")
    ap.add_argument("--tp", type=int, default=0, help="TP group size (default min(N, 4))")
    ap.add_argument("--case", default="headline", choices=["headline", "tokens", "collectives", "quantizer"])
    ap.add_argument("--rows", default=None, help="--case tokens / collectives: comma-separated row counts")
    args = ap.parse_args()
    shape = SHAPES[args.shape]
    if args.case == "tokens":
        return case_tokens(args, shape)
    if args.case == "quantizer":
        return case_quantizer(args)
    if args.case == "collectives":
        return case_collectives(args)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    warmup = max(args.warmup, 3)
    pkg = importlib.import_module("gpt-oss_b200")
    synth = pkg.synth
    E, H, D, K = shape["E"], shape["H"], shape["D"], shape["K"]
    T = args.tokens
    cfg = workload_config(shape, T, args.gpus, args.parallel, args.tp, args.zipf)

    if args.impl == "reference":
        if rank != 0:
            return
        layer = synth.make_layer(E, H, D, seed=0, zipf_s=args.zipf)
        sample = synth.make_tokens(T, H, seed=0)[:CPU_SAMPLE_TOKENS]
        tps, kind, cores, ms, _ = cpu_reference_arm(layer, sample, max(args.steps, 1), min(warmup, 3))
        sample_desc = (f"first {CPU_SAMPLE_TOKENS} of the {T} rows per step, fp32 weights dequantised beforehand "
                       f"(as the reference loads them), {cores} OpenMP threads")
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample_desc},
            "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}))
        return

    import torch
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    tp = tp_size_for(world, args.parallel, args.tp)
    layer = synth.make_layer(E, H, D, seed=0, zipf_s=args.zipf)
    tokens = synth.make_tokens(T, H, seed=rank)
    blk = pkg.MoeBlock(H, D, E, top_k=K, max_rows=T * tp, tp_size=tp, tp_rank=rank % tp, device=local_rank)
    blk.load_layer(0, layer)
    tp_group = None
    if tp > 1:
        tpmod = importlib.import_module("gpt-oss_b200.tp")
        for ranks in tpmod.tp_groups(world, tp):          # every rank takes part in creating every group
            g_gloo = dist.new_group(ranks=ranks, backend="gloo")
            g_nccl = dist.new_group(ranks=ranks, backend="nccl")
            if rank in ranks:
                tp_group = g_nccl
                tpmod.attach_group(blk, rank % tp, g_gloo)
    Dl = blk.Dl
    Tu = T * tp                      # rows the block sees on every rank
    d_t = torch.from_numpy(tokens.view(np.int16)).cuda()
    d_o = torch.empty_like(d_t)
    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream

    def step():
        if tp > 1:
            blk.tp_forward(0, d_t.data_ptr(), T, d_o.data_ptr(), 0, sp)
        else:
            blk.forward(0, d_t.data_ptr(), T, d_o.data_ptr(), 0, sp)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    blk.synchronize()
    launches0 = blk.launches()

    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid)
    except Exception:
        pass
    sampler = ClockSampler(uuid) if rank == 0 else None

    # ---- A: device-resident throughput ------------------------------------
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(); torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize(); barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    gpu_launches = blk.launches() - launches0
    blk.synchronize()

    # ---- B: the same steps with per-stage events (roofline of the top kernel)
    blk.profile(True)
    for _ in range(args.steps):
        step()
    stage_ms, ncalls = blk.profile_collect()
    blk.profile(False)
    counts = blk.debug(pkg.DBG_COUNTS)
    active = int((counts > 0).sum())

    # ---- C: end to end through the host-buffer entry points -----------------
    # Every step copies its rows in from pinned host memory and its result back out: submit/wait, up to three
    # batches in flight, so the copies of neighbouring steps overlap the block of this one (what a serving
    # loop does).  In a TP group every rank submits its own rows, in the same order.
    n_pin = 3
    pin_in = [pkg.PinnedBuffer((T, H), np.uint16) for _ in range(n_pin)]
    pin_out = [pkg.PinnedBuffer((T, H), np.uint16) for _ in range(n_pin)]
    for b in pin_in:
        b.array[:] = tokens
    host_cpu = {"submit_s": 0.0, "wait_s": 0.0}

    def host_steps(n):
        tickets = []
        for i in range(n):
            if len(tickets) == n_pin:
                t_a = time.perf_counter()
                blk.forward_host_wait(tickets.pop(0))
                host_cpu["wait_s"] += time.perf_counter() - t_a
            t_a = time.perf_counter()
            tickets.append(blk.forward_host_submit(0, pin_in[i % n_pin].array, pin_out[i % n_pin].array))
            host_cpu["submit_s"] += time.perf_counter() - t_a
        for t in tickets:
            blk.forward_host_wait(t)

    host_steps(3)
    barrier(); torch.cuda.synchronize()
    host_cpu["submit_s"] = host_cpu["wait_s"] = 0.0
    t0 = time.perf_counter()
    host_steps(args.steps)
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()

    # ---- C2: the copies of those steps alone (no block), all ranks at once: what host<->device traffic allows ----
    c_in, c_out = torch.cuda.Stream(), torch.cuda.Stream()
    pin_t = [torch.from_numpy(b.array.view(np.int16)) for b in pin_in]       # views of the pinned buffers
    pout_t = [torch.from_numpy(b.array.view(np.int16)) for b in pin_out]
    n_copy = min(args.steps, 50)

    def copy_steps(n):
        for i in range(n):
            with torch.cuda.stream(c_in):
                d_t.copy_(pin_t[i % n_pin], non_blocking=True)
            with torch.cuda.stream(c_out):
                pout_t[i % n_pin].copy_(d_o, non_blocking=True)
        c_in.synchronize(); c_out.synchronize()

    saved_out = pin_out[(args.steps - 1) % n_pin].array[:min(PARITY_ROWS, T)].copy()   # the last step's rows, before the probe overwrites them
    copy_steps(3)
    barrier(); torch.cuda.synchronize()
    t0 = time.perf_counter()
    copy_steps(n_copy)
    copy_s = max_over_ranks(time.perf_counter() - t0)
    barrier()

    # ---- parity: rank 0's first rows, as they came back through the host call, against the CPU oracle ----
    parity = None
    if rank == 0:
        nrow = min(PARITY_ROWS, T)
        got_bits = saved_out[:nrow]
        got_idx = blk.debug(pkg.DBG_TOPK_IDX)[:nrow]        # rank 0's rows are the first rows of the union
        port = _oracle().Port()
        port.set_threads(_oracle().host_cores())
        ref_logits, ref_idx, _, ref_out = port.moe_layer(layer, tokens[:nrow])
        got_f32 = None
        if tp == 1:
            blk.forward(0, d_t.data_ptr(), T, 0, pkg.FWD_PARTIAL_F32, sp)
            torch.cuda.synchronize()
            got_f32 = blk.debug(pkg.DBG_OUT_F32)[:nrow]
        parity = parity_figures(synth, got_bits, ref_out, got_idx, ref_idx, ref_logits, got_f32, tp)
        parity["against"] = "C restatement of run.cpp:657-748 (pinned bit-exact to the reference's forward())"

    # ---- D (TP only): the two collectives alone, this library's peer-memory kernels vs NCCL ----
    coll = None
    if tp > 1:
        def timed(fn, n):
            for _ in range(3):
                fn()
            barrier(); torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(n):
                fn()
            b.record(stream)
            torch.cuda.synchronize(); barrier()
            return max_over_ranks(a.elapsed_time(b)) / n
        n = min(args.steps, 50)
        bt = d_t.view(torch.bfloat16)
        g_full = torch.empty((Tu, H), dtype=torch.bfloat16, device="cuda")
        g_part = torch.randn((Tu, H), dtype=torch.float32, device="cuda").to(torch.bfloat16)
        g_out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
        ours_ag = timed(lambda: blk.tp_allgather(d_t.data_ptr(), T, sp), n)
        ours_rs = timed(lambda: blk.tp_reduce_scatter(T, d_o.data_ptr(), sp), n)
        nccl_ag = timed(lambda: dist.all_gather_into_tensor(g_full, bt, group=tp_group), n)
        nccl_rs = timed(lambda: dist.reduce_scatter_tensor(g_out, g_part, group=tp_group), n)
        per_dir = (tp - 1) / tp * Tu * H * 2     # bytes each rank sends (and receives) per collective
        coll = {"rows_per_rank": T, "bytes_per_rank_per_direction": per_dir,
                "allgather_ms": {"ours": ours_ag, "nccl": nccl_ag},
                "reduce_scatter_ms": {"ours": ours_rs, "nccl": nccl_rs},
                "allgather_gbs_per_direction": {"ours": per_dir / ours_ag / 1e6, "nccl": per_dir / nccl_ag / 1e6},
                "reduce_scatter_gbs_per_direction": {"ours": per_dir / ours_rs / 1e6, "nccl": per_dir / nccl_rs / 1e6},
                "nvlink_peer_copy_measured_gbs": 770.0}
    loss_like = float(synth.bf16_bits_to_f32(saved_out[:4]).sum())  # the result was read back
    clocks = sampler.stop() if sampler else None

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    hbm_peak, tc_peak, peak_kind = peaks()
    ms_step = ms_total / args.steps
    value = world * T / (ms_step * 1e-3)
    P = Tu * K
    R1 = 2 * Dl                      # this rank's MLP1 rows per expert
    # the expert MLP kernel (MLP1 + SwiGLU + MLP2 in one launch; its time is the profile's "mlp1" stage, the
    # "mlp2" stage is then empty): weights, scales and biases of both matrices once, the
    # two e4m3 terms of every gathered row in, the fp16 expert outputs out.  The SwiGLU rows in between are
    # written and read back inside the launch and are not counted.
    mlp_bytes = (active * (R1 * H // 2 + R1 * H // 32 + R1 * 2) + active * (H * Dl // 2 + H * Dl // 32 + H * 2)
                 + P * H * 2 + P * H * 2)
    mlp_flops = 2.0 * P * R1 * H + 2.0 * P * H * Dl
    mlp_s = stage_ms["mlp1"] / max(ncalls, 1) * 1e-3
    achieved = mlp_bytes / mlp_s / 1e9
    flops, nbytes = synth.algorithmic_work(Tu, H, D, E, K, active)
    if tp > 1:                       # per rank: 1/tp of the expert weights and flops, all of the rows
        flops = (flops - Tu * 2 * H * E) / tp + Tu * 2 * H * E
        nbytes = active * synth.weight_bytes_per_expert(H, D) / tp + Tu * H * 2 * 2 + E * H * 4
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "e4m3 (high+low terms of bf16) x mxfp4 -> fp32 accumulate (bf16 in/out)", "data": "synthetic",
        "config": cfg,
        "e2e": {"value": world * T * args.steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": T * H * 2,
                "d2h_bytes_per_step": T * H * 2, "ms_per_step": e2e_s / args.steps * 1e3,
                "api": "moe_forward_host_submit/_wait, 3 batches in flight, pinned buffers",
                "host_cpu_us_per_step": {"submit": host_cpu["submit_s"] / args.steps * 1e6,
                                         "wait": host_cpu["wait_s"] / args.steps * 1e6},
                "copies_alone_ms_per_step": copy_s / n_copy * 1e3,
                "copies_alone_note": "the same host->device and device->host copies on two streams with no block in "
                                     "between, all ranks at once: the floor that host memory and PCIe set for a step"},
        "gpu_launches": gpu_launches,
        "clocks": clocks,
        "roofline": {"kernel": "expert_gemm_kernel (grouped MLP1 + SwiGLU + MLP2, one launch)", "bound": "hbm",
                     "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": mlp_bytes * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE,
                     "traffic_source": "ncu capture of a 4x smaller case scaled by bytes processed",
                     "peak_source": peak_kind, "bytes_per_launch": mlp_bytes,
                     "ms_per_launch": mlp_s * 1e3,
                     "tensor_tflops": mlp_flops / mlp_s / 1e12, "tensor_peak_tflops": tc_peak,
                     "tensor_frac": mlp_flops / mlp_s / 1e12 / tc_peak},
        "block_roofline": {"flops": flops, "bytes": nbytes, "active_experts": active,
                           "hbm_bound_ms": nbytes / hbm_peak / 1e6, "tensor_bound_ms": flops / tc_peak / 1e9,
                           "frac_of_min_time": max(nbytes / hbm_peak / 1e6, flops / tc_peak / 1e9) / ms_step},
        "stage_ms": {k: v / max(ncalls, 1) for k, v in stage_ms.items()},
        "stage_ms_note": "'router' is the one launch that routes (router GEMM, top-k, softmax, histogram) and 'mlp1' the one launch of the expert MLP kernel (MLP1 + SwiGLU + MLP2); 'topk' and 'mlp2' launch nothing and are 0",
        "parity": parity,
        "checksum": loss_like,
    }
    if coll is not None:
        out["collectives"] = coll
        out["stage_notes"] = ("tensor-parallel call: the all-gather push runs beside 'router' on a side stream and its "
                              "arrival wait is inside 'topk'; the reduce-scatter (peer stores from the combine, arrival "
                              "wait, slot sum) is inside 'combine'")
    if args.gpus == 1 and not args.no_cpu_baseline:
        sample = tokens[:CPU_SAMPLE_TOKENS]
        tps, kind, cores, _, ref_last = cpu_reference_arm(layer, sample, 2, 1)
        out["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": cores, "kind": kind,
                               "sample": f"first {CPU_SAMPLE_TOKENS} of the {T} rows, 2 timed passes after 1 warm-up, "
                                         f"fp32 weights dequantised beforehand, {cores} OpenMP threads"}
        # the outputs of that very run are the second anchor of the parity figures
        r_logits, r_idx, _, r_out = ref_last
        n = CPU_SAMPLE_TOKENS
        out["parity"]["against_timed_cpu_run"] = dict(
            parity_figures(synth, saved_out[:n], r_out,
                           blk.debug(pkg.DBG_TOPK_IDX)[:n], r_idx, r_logits), kind=kind)
    print(json.dumps(out))
    for b in pin_in + pin_out:
        b.free()
    blk.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
