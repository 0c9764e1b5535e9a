"""Checkpoint ingest from the reference's flat fp32 file (Config header + tensors in the order of
memory_map_weights, run.cpp:206-247).  The writer below restates that order independently of the library:
it appends the tensors one after the other exactly as the reference maps them."""
import ctypes as C
import os

import numpy as np
import pytest


def write_bin(path, cfg, rng):
    """cfg: dict with the reference's Config fields.  Returns the per-layer MoE tensors that were written."""
    V, H, E, K, D, L = cfg["vocab_size"], cfg["hidden_dim"], cfg["n_experts"], cfg["experts_per_token"], \
        cfg["intermediate_dim"], cfg["n_layers"]
    hd, nq, nkv = cfg["head_dim"], cfg["n_attn_heads"], cfg["n_kv_heads"]
    header = np.zeros(15, dtype=np.int32)
    header[:11] = [V, H, E, K, D, L, hd, nq, nkv, cfg["seq_len"], cfg["initial_context_length"]]
    header[11:13] = np.array([cfg["rope_theta"], cfg["rope_scaling_factor"]], dtype=np.float32).view(np.int32)
    header[13] = cfg["sliding_window"]
    header[14] = np.array([cfg["swiglu_limit"]], dtype=np.float32).view(np.int32)[0]
    qkv = hd * nq + 2 * hd * nkv
    t = {}
    def rnd(*shape, scale=0.05):
        return (rng.standard_normal(shape) * scale).astype(np.float32)
    order = [("token_embedding_table", rnd(V, H)), ("out", rnd(V, H)), ("rms_attn_w", rnd(L, H)),
             ("rms_ffn_w", 1.0 + rnd(L, H)), ("rms_out_w", rnd(H)), ("w_qkv", rnd(L, qkv, H)), ("b_qkv", rnd(L, qkv)),
             ("w_o", rnd(L, H, hd * nq)), ("b_o", rnd(L, H)), ("attn_sinks", rnd(L, nq)),
             ("w_router", rnd(L, E, H)), ("b_router", rnd(L, E)),
             ("w_mlp1", rnd(L, E, 2 * D, H)), ("b_mlp1", rnd(L, E, 2 * D, scale=0.02)),
             ("w_mlp2", rnd(L, E, H, D)), ("b_mlp2", rnd(L, E, H, scale=0.02))]
    with open(path, "wb") as f:
        f.write(header.tobytes())
        for name, arr in order:
            f.write(np.ascontiguousarray(arr).tobytes())
            t[name] = arr
    return header, t


CFG = dict(vocab_size=37, hidden_dim=128, n_experts=8, experts_per_token=4, intermediate_dim=96, n_layers=3,
           head_dim=16, n_attn_heads=4, n_kv_heads=2, seq_len=64, initial_context_length=64, rope_theta=150000.0,
           rope_scaling_factor=32.0, sliding_window=8, swiglu_limit=7.0)


def test_offsets_follow_the_reference_mapping(tmp_path, pkg):
    lib = pkg.lib()
    path = str(tmp_path / "model.bin")
    header, t = write_bin(path, CFG, np.random.default_rng(3))
    flat = np.fromfile(path, dtype=np.float32)
    names = ["rms_ffn_w", "w_router", "b_router", "w_mlp1", "b_mlp1", "w_mlp2", "b_mlp2"]
    for layer in range(CFG["n_layers"]):
        off = (C.c_longlong * 7)()
        total = C.c_longlong()
        assert lib.moe_bin_layer_offsets(header.ctypes.data_as(C.c_void_p), layer, off, C.byref(total)) == 0
        assert total.value == flat.size
        for i, name in enumerate(names):
            want = t[name][layer].ravel()
            assert np.array_equal(flat[off[i]:off[i] + want.size], want), (layer, name)
    off = (C.c_longlong * 7)()
    assert lib.moe_bin_layer_offsets(header.ctypes.data_as(C.c_void_p), CFG["n_layers"], off, None) != 0


@pytest.mark.gpu
def test_layer_loaded_from_bin_equals_layer_loaded_from_arrays(tmp_path, pkg, synth):
    path = str(tmp_path / "model.bin")
    _, t = write_bin(path, CFG, np.random.default_rng(4))
    H, E, D = CFG["hidden_dim"], CFG["n_experts"], CFG["intermediate_dim"]
    tokens = synth.make_tokens(50, H, seed=5)
    a = pkg.MoeBlock(H, D, E, max_rows=64)
    b = pkg.MoeBlock(H, D, E, max_rows=64)
    try:
        layer = 1
        gain = a.load_layer_from_bin(0, path, file_layer=layer)
        assert np.array_equal(gain, t["rms_ffn_w"][layer])
        b.load_layer_f32(0, t["w_mlp1"][layer], t["b_mlp1"][layer], t["w_mlp2"][layer], t["b_mlp2"][layer],
                         t["w_router"][layer], t["b_router"][layer])
        assert np.array_equal(a.forward_host(0, tokens), b.forward_host(0, tokens))
        with pytest.raises(pkg.MoeError):                      # dimensions of the file must be the handle's
            c = pkg.MoeBlock(H, D + 32, E, max_rows=8)
            try:
                c.load_layer_from_bin(0, path, file_layer=0)
            finally:
                c.close()
        with pytest.raises(pkg.MoeError):
            a.load_layer_from_bin(0, os.path.join(str(tmp_path), "missing.bin"))
    finally:
        a.close()
        b.close()
