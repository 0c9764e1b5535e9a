#!/usr/bin/env python
"""MoE-layer throughput benchmark (tokens/s) for the sm_100a MoE block.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one pass of the MoE block (router, top-4 + softmax, permutation,
MLP1 + SwiGLU, MLP2, weighted combine) over one batch of synthetic bf16 rows.
At N = 1 the workload is the GPT-OSS-120B-shape layer (128 experts, hidden and
intermediate 2880, MXFP4 weights) at 1856 rows.  At N > 1 each rank runs a
replica of that workload on its own rows (data parallel, no collective on the
data path) and the value is the sum over ranks.

One JSON line is printed by rank 0.  `value` is device-resident throughput
(CUDA events on the launching stream), `e2e` goes through the host-buffer entry points
(moe_forward_host_submit/_wait, three batches in flight, every rank of a TP group with its own rows) with
pinned host buffers (every step's copies inside the timed region), `roofline` describes the
dominant kernel (the MLP1 grouped GEMM) from per-stage CUDA events, and
`cpu_baseline` times the reference's own CPU forward() on the host cores over a
bounded sample of the same workload.

--impl reference times that CPU code alone (oracle/_ref when the reference
binary is present, else this repository's C restatement of it).
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
SHAPE = dict(E=128, H=2880, D=2880, K=4)
CPU_SAMPLE_TOKENS = 32
# dram read+write bytes / algorithmic bytes of the MLP1 kernel, from the ncu capture summarised in
# profiles/expert_gemm_mxf8f6f4_20bshape_t464.md (small case; traffic is proportional to the weights streamed)
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.034


def tp_size_for(n_gpus: int, parallel: str, tp_arg: int) -> int:
    """TP group size at N GPUs: the reference's deployments (TP2 x DP4 for 20B, TP4 x DP2 for 120B,
    getp-csrc/getp_run.cpp:1850-1853) cap the group at 4; more GPUs add data-parallel replicas of it."""
    if n_gpus == 1 or parallel == "dp":
        return 1
    tp = tp_arg if tp_arg > 0 else min(n_gpus, 4)
    assert n_gpus % tp == 0
    return tp


def workload_config(tokens: int, n_gpus: int, parallel: str = "tp", tp_arg: int = 0) -> dict:
    tp = tp_size_for(n_gpus, parallel, tp_arg)
    if n_gpus == 1:
        par = "tp1"
    elif tp > 1:
        par = (f"tp{tp} x dp{n_gpus // tp}: intermediate dimension sharded over {tp} GPUs, every rank owns {tokens} "
               f"rows, the block runs on the group's union of {tp * tokens} rows; all-gather before and "
               f"reduce-scatter after by peer-memory kernels over NVLink; groups are independent replicas")
    else:
        par = f"tp1 x dp{n_gpus} (independent replicas, no collective)"
    return {
        "workload": f"GPT-OSS-120B-shape MoE layer (E=128, top-4, hidden 2880, intermediate 2880, MXFP4 "
                    f"weights, E8M0 scales), {tokens} bf16 rows per GPU, seed 0",
        "rows_per_gpu": tokens,
        "parallelism": par,
        "l2_policy": "inputs larger than L2: 1.69 GB of expert weights are streamed every step (L2 is 126 MB)",
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


def cpu_reference_arm(layer, tokens_bits, steps: int, warmup: int):
    """Times the reference CPU path on `tokens_bits` (a bounded sample); returns
    (tokens/s, kind, cores)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle
    n = tokens_bits.shape[0]
    if oracle.reference_available():
        ref = oracle.Reference(layer)
        ref.prepare(tokens_bits)          # load-time dequantisation, not part of the forward
        run, kind, cores = (lambda: ref.forward(tokens_bits)), "reference", ref.threads()
    else:
        port = oracle.Port()
        run, kind, cores = (lambda: port.moe_layer(layer, tokens_bits)), "port", port.threads()
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = time.perf_counter() - t0
    return steps * n / dt, kind, cores, dt / steps * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=1856)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parallel", default="tp", choices=["tp", "dp"],
                    help="at N > 1: tensor-parallel groups (default) or N independent replicas")
    ap.add_argument("--tp", type=int, default=0, help="TP group size (default min(N, 4))")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    warmup = max(args.warmup, 3)
    pkg = importlib.import_module("gpt-oss_b200")
    synth = pkg.synth
    E, H, D, K = SHAPE["E"], SHAPE["H"], SHAPE["D"], SHAPE["K"]
    T = args.tokens
    cfg = workload_config(T, args.gpus, args.parallel, args.tp)

    if args.impl == "reference":
        if rank != 0:
            return
        layer = synth.make_layer(E, H, D, seed=0)
        sample = synth.make_tokens(T, H, seed=0)[:CPU_SAMPLE_TOKENS]
        tps, kind, cores, ms = cpu_reference_arm(layer, sample, max(args.steps, 1), min(warmup, 3))
        sample_desc = (f"first {CPU_SAMPLE_TOKENS} of the {T} rows per step, fp32 weights dequantised beforehand "
                       f"(as the reference loads them)")
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
    layer = synth.make_layer(E, H, D, seed=0)
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

    def host_steps(n):
        tickets = []
        for i in range(n):
            if len(tickets) == n_pin:
                blk.forward_host_wait(tickets.pop(0))
            tickets.append(blk.forward_host_submit(0, pin_in[i % n_pin].array, pin_out[i % n_pin].array))
        for t in tickets:
            blk.forward_host_wait(t)

    host_steps(3)
    barrier(); torch.cuda.synchronize()
    t0 = time.perf_counter()
    host_steps(args.steps)
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()

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
    loss_like = float(synth.bf16_bits_to_f32(pin_out[(args.steps - 1) % n_pin].array[:4]).sum())  # the result was read back
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
    mlp1_bytes = active * (R1 * H // 2 + R1 * H // 32 + R1 * 2) + P * H * 2 + P * Dl * 2
    mlp1_flops = 2.0 * P * R1 * H
    mlp1_s = stage_ms["mlp1"] / max(ncalls, 1) * 1e-3
    achieved = mlp1_bytes / mlp1_s / 1e9
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
                "api": "moe_forward_host_submit/_wait, 3 batches in flight, pinned buffers"},
        "gpu_launches": gpu_launches,
        "clocks": clocks,
        "roofline": {"kernel": "expert_gemm_kernel<1> (MLP1 grouped GEMM + SwiGLU)", "bound": "hbm",
                     "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": mlp1_bytes * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE,
                     "traffic_source": "ncu capture of a 4x smaller case scaled by bytes processed",
                     "peak_source": peak_kind, "bytes_per_launch": mlp1_bytes,
                     "ms_per_launch": mlp1_s * 1e3,
                     "tensor_tflops": mlp1_flops / mlp1_s / 1e12, "tensor_peak_tflops": tc_peak,
                     "tensor_frac": mlp1_flops / mlp1_s / 1e12 / tc_peak},
        "block_roofline": {"flops": flops, "bytes": nbytes, "active_experts": active,
                           "hbm_bound_ms": nbytes / hbm_peak / 1e6, "tensor_bound_ms": flops / tc_peak / 1e9,
                           "frac_of_min_time": max(nbytes / hbm_peak / 1e6, flops / tc_peak / 1e9) / ms_step},
        "stage_ms": {k: v / max(ncalls, 1) for k, v in stage_ms.items()},
        "checksum": loss_like,
    }
    if coll is not None:
        out["collectives"] = coll
        out["stage_notes"] = ("tensor-parallel call: the all-gather push runs beside 'router' on a side stream and its "
                              "arrival wait is inside 'topk'; the reduce-scatter (peer stores from the combine, arrival "
                              "wait, slot sum) is inside 'combine'")
    if args.gpus == 1 and not args.no_cpu_baseline:
        sample = tokens[:CPU_SAMPLE_TOKENS]
        tps, kind, cores, _ = cpu_reference_arm(layer, sample, 2, 1)
        out["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": cores, "kind": kind,
                               "sample": f"first {CPU_SAMPLE_TOKENS} of the {T} rows, 2 timed passes after 1 warm-up, "
                                         f"fp32 weights dequantised beforehand"}
    print(json.dumps(out))
    for b in pin_in + pin_out:
        b.free()
    blk.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
