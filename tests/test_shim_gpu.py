"""The drop-in boundary seen from the reference's side: a C++ caller that uses the reference runtime's own
names (GPUTransformer with state.x / weights.rms_ffn_w, TPGroup, tp_init, tp_group_barrier, moe_gpu_120b) is
compiled against include/moe_b200_shim.hpp and run as one process with one host thread per GPU; its updated
residual rows are checked against the CPU oracle.  With one GPU the group has one rank; with two or more the
two-rank group runs as well."""
import os
import shutil
import subprocess

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

CUDA_INC, CUDA_LIB = "/usr/local/cuda/include", "/usr/local/cuda/lib64"


def _build(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None or not os.path.exists(os.path.join(CUDA_INC, "cuda_runtime.h")):
        pytest.skip("no host compiler or CUDA headers")
    exe = tmp_path / "shim_caller"
    libdir = os.path.join(ROOT, "gpt-oss_b200")
    subprocess.run([gxx, "-std=c++17", "-O1", "-pthread", "-I" + os.path.join(ROOT, "include"), "-I" + CUDA_INC,
                    os.path.join(ROOT, "tests", "shim", "shim_caller.cpp"), "-L" + libdir, "-lmoe_b200",
                    "-L" + CUDA_LIB, "-lcudart", "-Wl,-rpath," + libdir, "-Wl,-rpath," + CUDA_LIB, "-o", str(exe)], check=True)
    return exe


@pytest.mark.parametrize("tp", [1, 2])
def test_reference_style_caller_through_the_shim(tp, tmp_path, pkg, synth, port):
    import torch
    if torch.cuda.device_count() < tp:
        pytest.skip(f"needs {tp} GPUs")
    pkg.lib()                      # the library must be built
    exe = _build(tmp_path)
    E, H, D, T = 16, 256, 320, 96
    layer = synth.make_layer(E, H, D, seed=17)
    x_bits, gain_bits = synth.make_residual(T, H, seed=18)
    for k in ("w1_codes", "w1_scales", "b1", "w2_codes", "w2_scales", "b2"):
        np.ascontiguousarray(layer[k]).tofile(tmp_path / f"{k}.bin")
    np.ascontiguousarray(layer["router_w"], dtype=np.float32).tofile(tmp_path / "router_w.bin")
    np.ascontiguousarray(layer["router_b"], dtype=np.float32).tofile(tmp_path / "router_b.bin")
    x_bits.tofile(tmp_path / "x.bin")
    gain_bits.tofile(tmp_path / "gain.bin")
    (tmp_path / "cfg.txt").write_text(f"{E} {H} {D} {T}\n")
    res = subprocess.run([str(exe), str(tmp_path), str(tp)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    got = synth.bf16_bits_to_f32(np.fromfile(tmp_path / "x_out.bin", dtype=np.uint16).reshape(T, H)).astype(np.float64)
    x, gain = synth.bf16_bits_to_f32(x_bits), synth.bf16_bits_to_f32(gain_bits)
    _, logits, idx, _, agg, xo = port.moe_block(layer, x, gain, t_as_bf16=True)
    rms = max(1.0, float(np.sqrt((agg.astype(np.float64) ** 2).mean())))
    err = np.abs(got - xo)
    bound = 2e-2 * rms + 2.0 ** -8 * np.abs(xo)
    srt = np.sort(logits, axis=1)[:, ::-1]
    clear = (srt[:, :4] - srt[:, 1:5]).min(axis=1) >= 1e-5       # rows whose selection cannot legitimately differ
    assert (err[clear] <= bound[clear]).all(), float((err - bound)[clear].max())
    assert clear.mean() > 0.95
    upd = np.abs((got - x) - agg)[clear].mean() / np.abs(agg[clear]).mean()
    assert upd <= 0.1, upd
