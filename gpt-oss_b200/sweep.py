"""Secondary measurements of the MoE block (bench.py stays the headline).

    python -m gpt-oss_b200.sweep tokens [--zipf 1.2]     one GPU: rows in {1, 32, 256, 1856, 8192}
    python -m gpt-oss_b200.sweep quantizer               one GPU: fp32 -> MXFP4 of 2^28 values (1 GiB), GB/s
    torchrun --nproc-per-node N -m gpt-oss_b200.sweep collectives
                                                          N GPUs: all-gather / reduce-scatter of bf16
                                                          [T, 2880], T in {64, 256, 1536, 1856, 8192},
                                                          peer-memory kernels vs NCCL

`tokens` covers the skewed-routing case: with --zipf the router bias makes expert popularity
follow Zipf(s), so a few experts receive almost every row (many token tiles) while most receive
none or a few; rows per expert decide how full the 64-row token tiles are.  One JSON line per
case: time per block from CUDA events, the roofline time of the algorithmic work (bytes of the
experts that received rows / measured HBM rate, flops / measured bf16 rate) and their ratio.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        m = json.load(open(p))
        return float(m["hbm_gbs"]), float(m.get("bf16_tflops_sustained", m["bf16_tflops"]))
    return 6650.0, 1400.0


def sweep_tokens(args):
    import torch
    pkg = importlib.import_module("gpt-oss_b200")
    synth = pkg.synth
    E, H, D, K = args.experts, 2880, 2880, 4
    hbm, tc = _peaks()
    layer = synth.make_layer(E, H, D, seed=0, zipf_s=args.zipf)
    rows = [int(x) for x in args.rows.split(",")]
    blk = pkg.MoeBlock(H, D, E, top_k=K, max_rows=max(rows))
    blk.load_layer(0, layer)
    stream = torch.cuda.current_stream()
    for T in rows:
        tokens = synth.make_tokens(T, H, seed=0)
        d_t = torch.from_numpy(tokens.view(np.int16)).cuda()
        d_o = torch.empty_like(d_t)
        for _ in range(5):
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
        tiles = int(((counts + 63) // 64).sum())
        flops, nbytes = synth.algorithmic_work(T, H, D, E, K, active)
        roof_ms = max(nbytes / hbm / 1e6, flops / tc / 1e9)
        print(json.dumps({"case": "tokens", "zipf": args.zipf, "rows": T, "ms_per_block": ms,
                          "tokens_per_s": T / ms * 1e3, "active_experts": active, "token_tiles": tiles,
                          "max_rows_per_expert": int(counts.max()), "roofline_ms": roof_ms,
                          "frac_of_roofline": roof_ms / ms}), flush=True)
    blk.close()


def sweep_quantizer(args):
    """The load-time quantiser alone: 4 bytes read and 17/32 byte written per element."""
    import torch
    pkg = importlib.import_module("gpt-oss_b200")
    hbm, _ = _peaks()
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


def sweep_collectives(args):
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
    rows = [int(x) for x in args.rows.split(",")]
    # T is the gathered row count; every rank contributes T / world rows
    blk = pkg.MoeBlock(H, 32 * world, 8, max_rows=max(rows) + world, tp_size=world, tp_rank=rank, device=local)
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["tokens", "collectives", "quantizer"])
    ap.add_argument("--zipf", type=float, default=None)
    ap.add_argument("--rows", default=None)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--experts", type=int, default=128, help="tokens: experts of the layer (32 = the 20B shape)")
    args = ap.parse_args()
    sys.path.insert(0, ROOT)
    if args.what == "quantizer":
        sweep_quantizer(args)
    elif args.what == "tokens":
        args.rows = args.rows or "1,32,256,1856,8192"
        sweep_tokens(args)
    else:
        args.rows = args.rows or "64,256,1536,1856,8192"
        sweep_collectives(args)


if __name__ == "__main__":
    main()
