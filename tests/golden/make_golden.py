"""Regenerates tests/golden/*.npz from the reference's own CPU forward().

Run in a checkout that has the reference sources (oracle/Makefile compiles
run.cpp's CPU part into oracle/_ref/libref_moe.so):

    python tests/golden/make_golden.py

Each fixture holds the outputs of the reference binary (router logits, top-k
indices, softmax weights, block output e_agg) for one seeded synthetic layer.
The block_* fixtures go through forward()'s own RMSNorm
(residual rows x and a gain vector in, state.t and e_agg out).
Small cases also store their inputs; the GPT-OSS-20B-shape case stores the
seeds and a SHA-256 of the regenerated inputs instead (423 MB of weights).
"""
import hashlib
import importlib.util
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402

_spec = importlib.util.spec_from_file_location("synth", os.path.join(ROOT, "gpt-oss_b200", "synth.py"))
synth = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(synth)

CASES = [
    # name, E, H, D, T, layer seed, token seed, zipf, store inputs
    ("tiny_e8_h64_d64_t16", 8, 64, 64, 16, 11, 12, None, True),
    ("ragged_e8_h128_d96_t33", 8, 128, 96, 33, 21, 22, None, True),
    ("zipf_e16_h96_d160_t40", 16, 96, 160, 40, 31, 32, 1.2, True),
    ("onetoken_e8_h64_d64_t1", 8, 64, 64, 1, 41, 42, None, True),
    ("shape20b_e32_h2880_d2880_t16", 32, 2880, 2880, 16, 0, 0, None, False),
]

# The block with its own RMSNorm and the residual add (forward(), run.cpp:657-747): name, E, H, D, T, seeds
BLOCK_CASES = [
    ("block_e8_h64_d64_t12", 8, 64, 64, 12, 51, 52),
    ("block_e16_h128_d96_t33", 16, 128, 96, 33, 61, 62),
]

LAYER_KEYS = ("w1_codes", "w1_scales", "b1", "w2_codes", "w2_scales", "b2", "router_w", "router_b")


def inputs_digest(layer, tokens) -> str:
    h = hashlib.sha256()
    for k in LAYER_KEYS:
        h.update(np.ascontiguousarray(layer[k]).tobytes())
    h.update(np.ascontiguousarray(tokens).tobytes())
    return h.hexdigest()


def main():
    oracle.build(quiet=False)
    here = os.path.dirname(os.path.abspath(__file__))
    only_blocks = "--blocks" in sys.argv  # leave the older fixtures untouched
    for name, E, H, D, T, ls, ts, zipf, store in ([] if only_blocks else CASES):
        layer = synth.make_layer(E, H, D, seed=ls, zipf_s=zipf)
        tokens = synth.make_tokens(T, H, seed=ts)
        ref = oracle.Reference(layer)
        ref.prepare(tokens)
        logits, idx, w, out = ref.forward(tokens)
        ref.close()
        blob = dict(E=E, H=H, D=D, T=T, layer_seed=ls, token_seed=ts,
                    zipf=-1.0 if zipf is None else zipf,
                    digest=inputs_digest(layer, tokens),
                    logits=logits, topk_i=idx, topk_v=w, out=out)
        if store:
            blob.update({k: layer[k] for k in LAYER_KEYS})
            blob["tokens"] = tokens
        path = os.path.join(here, name + ".npz")
        np.savez_compressed(path, **blob)
        print(f"{name}: {os.path.getsize(path)} bytes, out rms {np.sqrt((out ** 2).mean()):.4f}")
    for name, E, H, D, T, ls, xs in BLOCK_CASES:
        layer = synth.make_layer(E, H, D, seed=ls)
        x_bits, gain_bits = synth.make_residual(T, H, seed=xs)
        ref = oracle.Reference(layer)
        t, logits, idx, w, agg = ref.forward_block(synth.bf16_bits_to_f32(x_bits), synth.bf16_bits_to_f32(gain_bits))
        ref.close()
        blob = dict(E=E, H=H, D=D, T=T, x=x_bits, gain=gain_bits, t=t, logits=logits, topk_i=idx, topk_v=w, e_agg=agg)
        blob.update({k: layer[k] for k in LAYER_KEYS})
        path = os.path.join(here, name + ".npz")
        np.savez_compressed(path, **blob)
        print(f"{name}: {os.path.getsize(path)} bytes, e_agg rms {np.sqrt((agg ** 2).mean()):.4f}")
    # the reference's own MXFP4 quantiser (getp-csrc/memory/mxfp4.hpp:113-217) on edge-case inputs
    vals = synth.make_quantizer_inputs(seed=1)
    q = oracle.ReferenceQuantizer()
    codes, scales = q.quantize(vals)
    back = q.dequantize(codes, scales, vals.size)
    path = os.path.join(here, "quant_edge_cases.npz")
    np.savez_compressed(path, values=vals, codes=codes, scales=scales, dequant=back)
    print(f"quant_edge_cases: {os.path.getsize(path)} bytes, {vals.size} values")


if __name__ == "__main__":
    main()
