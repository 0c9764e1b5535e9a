"""Multi-rank parity check of moe_tp_forward, run as one process per GPU by
tests/test_tp_multi_gpu.py (python -m torch.distributed.run --nproc-per-node N tests/tp_check.py).
Each rank owns `rows_local` rows; the group's union goes through the oracle on the CPU and every
rank compares its own slice."""
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def main():
    import torch
    import torch.distributed as dist
    import oracle
    pkg = importlib.import_module("gpt-oss_b200")
    tp = importlib.import_module("gpt-oss_b200.tp")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dist.init_process_group("gloo")
    torch.cuda.set_device(local)
    E, H, D, rows_local = 16, 256, 320, 50
    layer = pkg.synth.make_layer(E, H, D, seed=7)
    union = pkg.synth.make_tokens(rows_local * world, H, seed=8)
    sl_mine = slice(rank * rows_local, (rank + 1) * rows_local)
    mine = union[sl_mine]
    blk = pkg.MoeBlock(H, D, E, max_rows=rows_local * world, tp_size=world, tp_rank=rank, device=local)
    blk.load_layer(0, layer)
    tp.attach_group(blk, rank)
    _, ref_i, _, ref_out = oracle.Port().moe_layer(layer, union)
    d_t = torch.from_numpy(mine.view(np.int16).copy()).cuda()
    d_o = torch.zeros_like(d_t)
    stream = torch.cuda.current_stream().cuda_stream
    for it in range(3):                      # repeated calls exercise the epoch flags and buffer reuse
        blk.tp_forward(0, d_t.data_ptr(), rows_local, d_o.data_ptr(), 0, stream)
    torch.cuda.synchronize()
    blk.synchronize()
    assert np.array_equal(blk.debug(pkg.DBG_TOPK_IDX), ref_i), "routing of the union differs"
    got = pkg.synth.bf16_bits_to_f32(d_o.cpu().numpy().view(np.uint16)).astype(np.float64)
    ref = ref_out[rank * rows_local:(rank + 1) * rows_local].astype(np.float64)
    err = np.abs(got - ref)
    rms = max(1.0, float(np.sqrt((ref ** 2).mean())))
    mean_rel = err.mean() / np.abs(ref).mean()
    # bf16 partial payloads add one rounding per rank on top of the single-GPU path
    assert mean_rel <= 5e-3, mean_rel
    assert err.max() <= 2e-2 * rms, (err.max(), rms)
    # the all-gather alone: every rank's gather buffer ends up holding the union, in rank order
    blk.tp_allgather(d_t.data_ptr(), rows_local, stream)
    torch.cuda.synchronize()
    blk.synchronize()
    blk.rows = rows_local * world
    assert np.array_equal(blk.debug(pkg.DBG_GATHER), union), "all-gather buffer differs from the union of the ranks' rows"
    # The three steps as separate calls (the reference's own order: ring_allgather_rows_bf16, the MLPs into
    # e_agg_g, the owner-slice reduce-scatter; getp_run.cpp:2958-3246), four times in a row on different rows,
    # so that buffers and epoch flags are reused while their contents change.  The reduce-scatter's output must
    # be, bit for bit, the fp32 sum in rank order of the ranks' bf16 partials, and match the oracle.
    gather_ptr, partial_ptr = blk.tp_buffer(pkg.TP_BUF_GATHER), blk.tp_buffer(pkg.TP_BUF_PARTIAL)
    port = oracle.Port()
    unions = [pkg.synth.make_tokens(rows_local * world, H, seed=30 + it) for it in range(4)]
    d_ins = [torch.from_numpy(np.ascontiguousarray(u[sl_mine]).view(np.int16).copy()).cuda() for u in unions]
    d_rss = [torch.zeros_like(d) for d in d_ins]
    for it in range(4):                       # no host synchronisation between the steps or the rounds
        blk.tp_allgather(d_ins[it].data_ptr(), rows_local, stream)
        blk.forward(0, gather_ptr, rows_local * world, partial_ptr, 0, stream)
        blk.tp_reduce_scatter(rows_local, d_rss[it].data_ptr(), stream)
    torch.cuda.synchronize()
    blk.synchronize()
    blk.rows = rows_local * world
    assert np.array_equal(blk.debug(pkg.DBG_GATHER), unions[-1]), "gathered rows differ from the union"
    my_partial = torch.from_numpy(blk.debug(pkg.DBG_TP_PARTIAL).view(np.uint8).copy())    # gloo carries bytes
    parts = [torch.empty_like(my_partial) for _ in range(world)]
    dist.all_gather(parts, my_partial)
    acc = np.zeros((rows_local, H), dtype=np.float32)
    for r in range(world):                    # fp32 adds in rank order, as the kernel does
        acc = acc + pkg.synth.bf16_bits_to_f32(parts[r].numpy().view(np.uint16).reshape(-1, H)[sl_mine])
    assert np.array_equal(d_rss[-1].cpu().numpy().view(np.uint16), pkg.synth.f32_to_bf16_bits(acc)), \
        "reduce-scatter is not the rank-ordered fp32 sum of the ranks' bf16 partials"
    for it in range(4):
        _, _, _, ref_it = port.moe_layer(layer, unions[it])
        ref_rows = ref_it[sl_mine].astype(np.float64)
        e = np.abs(pkg.synth.bf16_bits_to_f32(d_rss[it].cpu().numpy().view(np.uint16)).astype(np.float64) - ref_rows)
        r_rms = max(1.0, float(np.sqrt((ref_rows ** 2).mean())))
        # every rank's partial travels as bf16 and the sum is rounded once more: up to half an ulp (2^-9 relative)
        # of a value of the output's magnitude per rounding, on top of the single-GPU bound
        bound = 2e-2 * r_rms + (world + 1) * 2.0 ** -9 * np.abs(ref_rows).max()
        assert e.mean() / np.abs(ref_rows).mean() <= 5e-3 and e.max() <= bound, (it, e.mean(), e.max(), bound)
    # all-reduce (ring_allreduce_sum_bf16, tp_ring.hpp:253-331): every rank ends with the rank-ordered fp32 sum
    rng = np.random.default_rng(100 + rank)
    n_el = rows_local * world * H
    for it in range(3):
        mine_f = rng.normal(0, 1, size=n_el).astype(np.float32)
        mine_b = pkg.synth.f32_to_bf16_bits(mine_f)
        d_buf = torch.from_numpy(mine_b.view(np.int16).copy()).cuda()
        blk.tp_allreduce(d_buf.data_ptr(), n_el, stream)
        torch.cuda.synchronize()
        blk.synchronize()
        allb = [torch.empty(n_el * 2, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(allb, torch.from_numpy(mine_b.view(np.uint8).copy()))
        acc = np.zeros(n_el, dtype=np.float32)
        for r in range(world):
            acc = acc + pkg.synth.bf16_bits_to_f32(allb[r].numpy().view(np.uint16))
        assert np.array_equal(d_buf.cpu().numpy().view(np.uint16), pkg.synth.f32_to_bf16_bits(acc)), f"all-reduce round {it}"
    # the reference's calling form over the group: x <- x + MoE(rmsnorm(x) * gain) on each rank's rows
    x_bits, gain_bits = pkg.synth.make_residual(rows_local * world, H, seed=9)
    xf, gf = pkg.synth.bf16_bits_to_f32(x_bits), pkg.synth.bf16_bits_to_f32(gain_bits)
    _, b_logits, b_idx, _, b_agg, b_xo = oracle.Port().moe_block(layer, xf, gf, t_as_bf16=True)
    sl = slice(rank * rows_local, (rank + 1) * rows_local)
    d_x = torch.from_numpy(x_bits[sl].view(np.int16).copy()).cuda()
    d_g = torch.from_numpy(gain_bits.view(np.int16).copy()).cuda()
    blk.block(0, d_x.data_ptr(), d_g.data_ptr(), rows_local, 0, stream)
    torch.cuda.synchronize()
    blk.synchronize()
    same = (np.sort(blk.debug(pkg.DBG_TOPK_IDX), axis=1) == np.sort(b_idx, axis=1)).all(axis=1)
    srt = np.sort(b_logits, axis=1)[:, ::-1]
    assert ((srt[:, 3] - srt[:, 4])[~same] < 1e-5).all(), "block form: routing differs with a clear logit gap"
    got_x = pkg.synth.bf16_bits_to_f32(d_x.cpu().numpy().view(np.uint16)).astype(np.float64)
    ok_rows = same[sl]
    b_err = np.abs(got_x - b_xo[sl])[ok_rows]
    b_rms = max(1.0, float(np.sqrt((b_agg.astype(np.float64) ** 2).mean())))
    bound = (2e-2 * b_rms + 2.0 ** -8 * np.abs(b_xo[sl]))[ok_rows]
    assert (b_err <= bound).all(), float((b_err - bound).max())
    # host buffers, three batches in flight on every rank: the bits of the blocking call
    batches = [pkg.synth.make_tokens(rows_local * world, H, seed=20 + i)[sl] for i in range(5)]
    want = [blk.tp_forward_host(0, np.ascontiguousarray(b), np.empty_like(b)).copy() for b in batches]
    pin_i = [pkg.PinnedBuffer(b.shape, np.uint16) for b in batches]
    pin_o = [pkg.PinnedBuffer(b.shape, np.uint16) for b in batches]
    for p_, b in zip(pin_i, batches):
        p_.array[:] = b
    tickets = []
    for i in range(len(batches)):
        if len(tickets) == 3:
            blk.forward_host_wait(tickets.pop(0))
        tickets.append(blk.forward_host_submit(0, pin_i[i].array, pin_o[i].array))
    for t in tickets:
        blk.forward_host_wait(t)
    for i, w_ in enumerate(want):
        assert np.array_equal(pin_o[i].array, w_), f"pipelined batch {i} differs from the blocking call"
    dist.barrier()
    print(f"rank {rank}: tp_forward ok, mean rel {mean_rel:.2e}, max abs {err.max():.3e} (rms {rms:.2f})", flush=True)
    blk.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
