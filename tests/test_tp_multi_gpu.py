"""Tensor-parallel path on real GPUs: one process per GPU (torchrun), peer memory over NVLink.
Needs at least two GPUs; ranks that wait on one another are never run on one GPU."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _gpus():
    import torch
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.parametrize("n", [2, 4])
def test_tp_forward_matches_oracle(n):
    if _gpus() < n:
        pytest.skip(f"needs {n} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + n), os.path.join(ROOT, "tests", "tp_check.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    print(res.stdout[-2000:])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("tp_forward ok") == n


def test_one_process_one_thread_per_gpu(pkg, synth, port):
    """The reference's own process model (one process, one host thread per GPU after hipSetDevice,
    getp_run.cpp:3514-3517): two handles on two devices of THIS process, connected with raw peer pointers
    (moe_tp_attach_ptr, what include/moe_b200_shim.hpp's moe_b200_connect_group does), each driven by its own
    thread.  Every kernel attribute the library needs must therefore have been set on both devices."""
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    import ctypes as C
    import threading
    import numpy as np
    import torch
    tp, E, H, D, rows_local = 2, 16, 256, 320, 50
    layer = synth.make_layer(E, H, D, seed=7)
    union = synth.make_tokens(rows_local * tp, H, seed=8)
    _, ref_i, _, ref_out = port.moe_layer(layer, union)
    blks = [pkg.MoeBlock(H, D, E, max_rows=rows_local * tp, tp_size=tp, tp_rank=r, device=r) for r in range(tp)]
    results, errors = [None] * tp, []
    try:
        for b in blks:
            b.load_layer(0, layer)
        lib = pkg.lib()
        for r in range(tp):
            for which in range(pkg.TP_N_BUFS):
                blks[r]._check(lib.moe_tp_attach_ptr(blks[r].h, which, 1 - r, C.c_void_p(blks[1 - r].tp_buffer(which)), 1 - r))

        def worker(r):
            try:
                torch.cuda.set_device(r)
                dev = torch.device("cuda", r)
                mine = union[r * rows_local:(r + 1) * rows_local]
                d_t = torch.from_numpy(mine.view(np.int16).copy()).to(dev)
                d_o = torch.zeros_like(d_t)
                s = torch.cuda.current_stream(dev).cuda_stream
                for _ in range(3):
                    blks[r].tp_forward(0, d_t.data_ptr(), rows_local, d_o.data_ptr(), 0, s)
                torch.cuda.synchronize(dev)
                blks[r].synchronize()
                results[r] = (d_o.cpu().numpy().view(np.uint16), blks[r].debug(pkg.DBG_TOPK_IDX))
            except Exception as e:           # surfaced by the main thread
                errors.append((r, repr(e)))

        threads = [threading.Thread(target=worker, args=(r,)) for r in range(tp)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=120)
        assert not errors, errors
        for r in range(tp):
            out_bits, idx = results[r]
            assert np.array_equal(idx, ref_i), f"rank {r}: routing of the union differs"
            got = synth.bf16_bits_to_f32(out_bits).astype(np.float64)
            ref = ref_out[r * rows_local:(r + 1) * rows_local].astype(np.float64)
            err = np.abs(got - ref)
            assert err.mean() / np.abs(ref).mean() <= 5e-3
            assert err.max() <= 2e-2 * max(1.0, float(np.sqrt((ref ** 2).mean())))
    finally:
        for b in blks:
            b.close()


def test_tp_forward_single_rank_group(pkg, synth, port):
    """tp_size = 1 runs the same launch sequence (push, flags, block, pull) on one GPU."""
    import numpy as np
    import torch
    E, H, D, T = 8, 128, 128, 37
    layer = synth.make_layer(E, H, D, seed=61)
    tokens = synth.make_tokens(T, H, seed=62)
    _, _, _, ref = port.moe_layer(layer, tokens)
    blk = pkg.MoeBlock(H, D, E, max_rows=T)
    try:
        blk.load_layer(0, layer)
        d_t = torch.from_numpy(tokens.view(np.int16)).cuda()
        d_o = torch.zeros_like(d_t)
        for _ in range(2):
            blk.tp_forward(0, d_t.data_ptr(), T, d_o.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        blk.synchronize()
        got = synth.bf16_bits_to_f32(d_o.cpu().numpy().view(np.uint16)).astype(np.float64)
        err = np.abs(got - ref)
        assert err.mean() / np.abs(ref).mean() <= 5e-3 and err.max() <= 2e-2 * max(1.0, float(np.sqrt((ref ** 2).mean())))
        # the stand-alone reduce-scatter on a group of one: the owner's slice of the partial buffer, value for value
        d_plain = torch.zeros_like(d_t)
        blk.forward(0, d_t.data_ptr(), T, d_plain.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
        blk.forward(0, d_t.data_ptr(), T, blk.tp_buffer(pkg.TP_BUF_PARTIAL), 0, torch.cuda.current_stream().cuda_stream)
        d_rs = torch.zeros_like(d_t)
        blk.tp_reduce_scatter(T, d_rs.data_ptr(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        blk.synchronize()
        assert np.array_equal(d_rs.cpu().numpy(), d_plain.cpu().numpy())
        assert np.array_equal(blk.debug(pkg.DBG_TP_PARTIAL).view(np.int16), d_plain.cpu().numpy())
        # all-reduce over a group of one leaves the values as they are
        d_ar = d_plain.clone()
        blk.tp_allreduce(d_ar.data_ptr(), T * H - (T * H) % 8, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        blk.synchronize()
        assert np.array_equal(d_ar.cpu().numpy(), d_plain.cpu().numpy())
    finally:
        blk.close()


def test_peer_that_never_arrives_is_reported_not_hung(pkg, synth):
    """Failure detection without a fault: a rank waits for a peer flag that nothing sets.  The
    device-side wait is bounded (about a second); it records a status bit, the kernel returns,
    the host call reports MOE_ERR_TIMEOUT, and the context keeps working.  (The reference's
    tp_group_barrier spins forever in that situation, getp-csrc/nccl.hpp:133-135.)
    Both handles live on one GPU; only rank 0 ever launches, so no two kernels wait on each other."""
    import numpy as np
    import torch
    E, H, D, T = 8, 128, 128, 16
    layer = synth.make_layer(E, H, D, seed=71)
    r0 = pkg.MoeBlock(H, D, E, max_rows=2 * T, tp_size=2, tp_rank=0)
    r1 = pkg.MoeBlock(H, D, E, max_rows=2 * T, tp_size=2, tp_rank=1)   # the silent peer
    try:
        r0.load_layer(0, layer)
        lib = pkg.lib()
        import ctypes as C
        for which in range(pkg.TP_N_BUFS):
            r0._check(lib.moe_tp_attach_ptr(r0.h, which, 1, C.c_void_p(r1.tp_buffer(which)), 0))
        rows = torch.from_numpy(synth.make_tokens(T, H, seed=72).view(np.int16)).cuda()
        r0.tp_allgather(rows.data_ptr(), T, torch.cuda.current_stream().cuda_stream)
        with pytest.raises(pkg.MoeError) as ei:
            r0.synchronize()
        assert ei.value.code == 4                      # MOE_ERR_TIMEOUT
        assert "0x80" in str(ei.value)                 # the peer-wait bit of the status word
        # the push itself happened: the silent peer's gather buffer holds rank 0's rows in slot 0
        r1.rows = T
        got = r1.debug(pkg.DBG_GATHER)
        assert np.array_equal(got, rows.cpu().numpy().view(np.uint16))
        # and the context is still usable: a plain forward on a fresh single-rank handle works
        solo = pkg.MoeBlock(H, D, E, max_rows=T)
        solo.load_layer(0, layer)
        out = solo.forward_host(0, rows.cpu().numpy().view(np.uint16))
        assert np.isfinite(synth.bf16_bits_to_f32(out)).all()
        solo.close()
    finally:
        r0.close()
        r1.close()
