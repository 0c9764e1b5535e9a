"""GPU parity of the load-time MXFP4 quantiser (byte work: bit-exact) and of loading a layer from fp32."""
import os

import numpy as np
import pytest

from conftest import GOLDEN_DIR

pytestmark = pytest.mark.gpu


def gpu_quantize(pkg, vals):
    import torch
    n = vals.size
    nblk = (n + 31) // 32
    d_v = torch.from_numpy(np.ascontiguousarray(vals, dtype=np.float32)).cuda()
    d_c = torch.full((nblk * 16,), 0xAB, dtype=torch.uint8, device="cuda")
    d_s = torch.full((nblk,), 0xCD, dtype=torch.uint8, device="cuda")
    pkg.quantize_mxfp4(d_v.data_ptr(), n, d_c.data_ptr(), d_s.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return d_c.cpu().numpy(), d_s.cpu().numpy()


def test_quantizer_golden_edge_cases(pkg, synth):
    z = np.load(os.path.join(GOLDEN_DIR, "quant_edge_cases.npz"))
    codes, scales = gpu_quantize(pkg, z["values"])
    assert np.array_equal(scales, z["scales"])
    assert np.array_equal(codes, z["codes"])


@pytest.mark.parametrize("n", [1, 31, 32, 33, 4096, 32 * 5000 + 17])
def test_quantizer_matches_oracle(n, pkg, port):
    rng = np.random.default_rng(n)
    v = (rng.standard_normal(n) * np.exp(rng.uniform(-25, 25, n))).astype(np.float32)
    if n >= 4096:
        v[64:96] = 0.0
        v[200] = np.nan                      # a NaN never becomes the block maximum and encodes as code 0
    pc, ps = port.quantize(v)
    gc, gs = gpu_quantize(pkg, v)
    assert np.array_equal(gs, ps) and np.array_equal(gc, pc)


def test_quantizer_full_size_properties(pkg, synth, port):
    """One expert's MLP1 matrix at full size (5760 x 2880 fp32, 66 MB): quantising the exact decode of
    MXFP4 weights gives back values that decode to the same floats (a block whose largest code is 3 or
    less moves to the next lower scale; its values stay representable), and the scales never exceed the
    original ones."""
    layer = synth.make_layer(1, 2880, 2880, seed=5)
    w = synth.dequant_mxfp4(layer["w1_codes"][0], layer["w1_scales"][0]).astype(np.float32)
    gc, gs = gpu_quantize(pkg, w.reshape(-1))
    back = port.dequant(gc.reshape(-1, 16), gs.reshape(-1, 1)).reshape(w.shape)
    assert np.array_equal(back, w)
    assert (gs.reshape(layer["w1_scales"][0].shape) <= layer["w1_scales"][0]).all()


def test_load_layer_f32_equals_load_layer(pkg, synth):
    """A layer loaded from the fp32 decode of its MXFP4 tensors gives the same output bits."""
    E, H, D, T = 8, 128, 160, 50
    layer = synth.make_layer(E, H, D, seed=33)
    tokens = synth.make_tokens(T, H, seed=34)
    a = pkg.MoeBlock(H, D, E, max_rows=T)
    b = pkg.MoeBlock(H, D, E, max_rows=T)
    try:
        a.load_layer(0, layer)
        w1 = synth.dequant_mxfp4(layer["w1_codes"], layer["w1_scales"])
        w2 = synth.dequant_mxfp4(layer["w2_codes"], layer["w2_scales"])
        b.load_layer_f32(0, w1, synth.bf16_bits_to_f32(layer["b1"]), w2, synth.bf16_bits_to_f32(layer["b2"]),
                         layer["router_w"], layer["router_b"])
        assert np.array_equal(a.forward_host(0, tokens), b.forward_host(0, tokens))
    finally:
        a.close()
        b.close()
