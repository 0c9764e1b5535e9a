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
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("tp_forward ok") == n


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
    finally:
        blk.close()
