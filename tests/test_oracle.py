"""Pins the CPU restatement (oracle/moe_oracle.c) to the reference.

* against the committed outputs of the reference's own forward()
  (tests/golden/*.npz, produced by tests/golden/make_golden.py);
* against that binary run live on further seeds, where oracle/_ref exists;
* the MXFP4 decode against a direct numpy evaluation of the format.
"""
import hashlib
import os

import numpy as np
import pytest

import oracle
from conftest import GOLDEN_DIR, golden_block_cases, golden_cases

LAYER_KEYS = ("w1_codes", "w1_scales", "b1", "w2_codes", "w2_scales", "b2", "router_w", "router_b")


def load_case(name, synth):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    E, H, D, T = int(z["E"]), int(z["H"]), int(z["D"]), int(z["T"])
    zipf = float(z["zipf"])
    if "tokens" in z.files:
        layer = {k: z[k] for k in LAYER_KEYS}
        layer.update(E=E, H=H, D=D)
        tokens = z["tokens"]
    else:
        layer = synth.make_layer(E, H, D, seed=int(z["layer_seed"]), zipf_s=None if zipf < 0 else zipf)
        tokens = synth.make_tokens(T, H, seed=int(z["token_seed"]))
    h = hashlib.sha256()
    for k in LAYER_KEYS:
        h.update(np.ascontiguousarray(layer[k]).tobytes())
    h.update(np.ascontiguousarray(tokens).tobytes())
    assert h.hexdigest() == str(z["digest"]), "synthetic generator drifted from the fixture"
    return layer, tokens, z


@pytest.mark.parametrize("name", golden_cases())
def test_port_matches_reference_golden(name, synth, port):
    layer, tokens, z = load_case(name, synth)
    logits, idx, w, out = port.moe_layer(layer, tokens)
    # bit-exact: same operations, same order, same libm as the reference binary
    assert np.array_equal(logits, z["logits"])
    assert np.array_equal(idx, z["topk_i"])
    assert np.array_equal(w, z["topk_v"])
    assert np.array_equal(out, z["out"])


@pytest.mark.skipif(not oracle.reference_available(), reason="oracle/_ref not built")
@pytest.mark.parametrize("E,H,D,T,seed", [(4, 64, 32, 7, 5), (8, 96, 128, 19, 6), (32, 64, 64, 64, 7)])
def test_port_matches_reference_live(E, H, D, T, seed, synth, port):
    layer = synth.make_layer(E, H, D, seed=seed)
    tokens = synth.make_tokens(T, H, seed=seed + 100)
    ref = oracle.Reference(layer)
    ref.prepare(tokens)
    r = ref.forward(tokens)
    ref.close()
    p = port.moe_layer(layer, tokens)
    for a, b in zip(p, r):
        assert np.array_equal(a, b)


def test_shard_partials_sum_to_full_block(synth, port):
    """Tensor-parallel split of the intermediate dimension (shards need not fall on
    scale-block boundaries; MLP2 bias added once): partial outputs add up to the
    unsharded block."""
    layer = synth.make_layer(8, 64, 96, seed=3)
    tokens = synth.make_tokens(12, 64, seed=4)
    _, idx, w, full = port.moe_layer(layer, tokens)
    parts = []
    for r, (d0, d1) in enumerate([(0, 24), (24, 72), (72, 96)]):
        _, i2, w2, o = port.moe_layer(layer, tokens, shard=(d0, d1), add_b2=(r == 0))
        assert np.array_equal(i2, idx) and np.array_equal(w2, w)
        parts.append(o.astype(np.float64))
    np.testing.assert_allclose(parts[0] + parts[1] + parts[2], full, rtol=1e-5, atol=1e-5)


def test_mxfp4_decode(synth, port):
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 256, size=(5, 7, 48), dtype=np.uint8)
    scales = rng.integers(100, 140, size=(5, 7, 3), dtype=np.uint8)
    assert np.array_equal(port.dequant(codes, scales), synth.dequant_mxfp4(codes, scales))
    # every code, low nibble = even element
    allc = np.arange(256, dtype=np.uint8).reshape(16, 16)
    sc = np.full((16, 1), 127, dtype=np.uint8)
    v = port.dequant(allc, sc)
    lut = synth.E2M1_VALUES
    assert np.array_equal(v[:, 0::2], lut[allc & 0xF]) and np.array_equal(v[:, 1::2], lut[allc >> 4])


def test_topk_ties_prefer_lower_index(port):
    logits = np.array([[1.0, 3.0, 3.0, 2.0, 3.0, 0.5, 2.0, -1.0]], dtype=np.float32)
    idx, w = port.topk_softmax(logits, 4)
    assert idx.tolist() == [[1, 2, 4, 3]]
    e = np.exp(np.array([0, 0, 0, -1.0]))
    np.testing.assert_allclose(w[0], e / e.sum(), rtol=1e-6)


def load_block_case(name, synth):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    layer = {k: z[k] for k in LAYER_KEYS}
    layer.update(E=int(z["E"]), H=int(z["H"]), D=int(z["D"]))
    return layer, z


@pytest.mark.parametrize("name", golden_block_cases())
def test_block_with_rmsnorm_matches_reference_golden(name, synth, port):
    layer, z = load_block_case(name, synth)
    x, gain = synth.bf16_bits_to_f32(z["x"]), synth.bf16_bits_to_f32(z["gain"])
    t, logits, idx, w, agg, xo = port.moe_block(layer, x, gain)
    assert np.array_equal(t, z["t"])          # rmsnorm, run.cpp:320-333
    assert np.array_equal(logits, z["logits"])
    assert np.array_equal(idx, z["topk_i"])
    assert np.array_equal(w, z["topk_v"])
    assert np.array_equal(agg, z["e_agg"])
    assert np.array_equal(xo, x + z["e_agg"])  # residual, run.cpp:744-747


@pytest.mark.skipif(not oracle.reference_available(), reason="oracle/_ref not built")
def test_block_with_rmsnorm_matches_reference_live(synth, port):
    layer = synth.make_layer(8, 96, 64, seed=71)
    xb, gb = synth.make_residual(9, 96, seed=72)
    x, gain = synth.bf16_bits_to_f32(xb), synth.bf16_bits_to_f32(gb)
    ref = oracle.Reference(layer)
    r = ref.forward_block(x, gain)
    ref.close()
    p = port.moe_block(layer, x, gain)
    for a, b in zip(p[:5], r):
        assert np.array_equal(a, b)


def test_quantizer_matches_reference_golden(synth, port):
    """The MXFP4 quantiser restatement against committed outputs of the reference's own source
    (getp-csrc/memory/mxfp4.hpp:113-217), bit for bit, and the decode of those bytes."""
    z = np.load(os.path.join(GOLDEN_DIR, "quant_edge_cases.npz"))
    vals = synth.make_quantizer_inputs(seed=1)
    assert np.array_equal(vals.view(np.uint32), z["values"].view(np.uint32)), "generator drifted from the fixture"
    codes, scales = port.quantize(vals)
    assert np.array_equal(codes, z["codes"]) and np.array_equal(scales, z["scales"])
    n = vals.size
    pad = (-n) % 32
    back = port.dequant(codes.reshape(-1, 16), scales.reshape(-1, 1)).reshape(-1)[:n]
    # Scale byte 0 (only the block of denormals reaches it, through the clamp) is the one encoding the two
    # decoders read differently: the reference forms the scale by a shift into the exponent field
    # (mxfp4.hpp:53), which gives 0 there, where E8M0 means 2^-127.
    live = np.repeat(scales != 0, 32)[:n]
    assert (~live).sum() == 32
    assert np.array_equal(back.view(np.uint32)[live], z["dequant"].view(np.uint32)[live])
    # the quantisation error is bounded by half the coarsest step (1 x scale above 4, clipping at 6)
    sc = np.repeat(np.exp2(scales.astype(np.float64) - 127), 32)[:n]
    inside = (np.abs(vals) <= 6 * sc) & live
    assert (np.abs(back.astype(np.float64) - vals)[inside] <= 1.0 * sc[inside]).all()
    assert pad == 19


@pytest.mark.skipif(not oracle.reference_quantizer_available(), reason="oracle/_ref/libref_mxfp4.so not built")
def test_quantizer_matches_reference_live(port):
    rng = np.random.default_rng(7)
    v = (rng.standard_normal(32 * 300 + 5) * np.exp(rng.uniform(-20, 20, 32 * 300 + 5))).astype(np.float32)
    ref = oracle.ReferenceQuantizer()
    rc, rs = ref.quantize(v)
    pc, ps = port.quantize(v)
    assert np.array_equal(pc, rc) and np.array_equal(ps, rs)
