"""GPU parity tests: the CUDA path through the C ABI against the CPU oracle.

Tolerances (floating point path, stated once here):
  * expert selection: exact, given identical fp32 logits (moe_route_topk on the
    oracle's logits).  In the full path the logits come from a tensor-core sum
    and may differ from the oracle's double-precision sum by ~1e-6; a token's
    selection may then differ only where the oracle's own gap between the last
    selected and first rejected logit is below 1e-5.
  * block output (bf16): mean relative error (mean|a-b| / mean|b|) <= 5e-3 and
    max|a-b| <= 2e-2 * max(1, rms(b)).  For outputs of unit scale or below (all
    small fixtures) that is the literal 2e-2, and check_output asserts the literal
    bound there.  At the benchmark's weight scales the layer output has rms ~37
    and peaks near 200, where half a bf16 ulp is already 0.5, so an absolute 2e-2
    cannot be met by ANY bf16 result (check_output measures and prints that floor:
    the error of the oracle's own output rounded to bf16); the bound is therefore
    taken relative to the output's rms, and the raw figures are printed.
  * a token whose selection differs from the oracle's (only allowed at a near-tie,
    see above) is left out of the output comparison; every other row is compared,
    and the number of such tokens is bounded (near_tie_allowance).
  * the fp32 output kept before the final rounding: max|a-b| <= 1e-2 * max(1, rms(b))
    (the SwiGLU output feeds MLP2 as two e4m3 terms, i.e. with about 8 significant bits,
    as the reference GPU path does by rounding it to bf16).
"""
import hashlib
import os

import numpy as np
import pytest

from conftest import GOLDEN_DIR, golden_block_cases, golden_cases, load_pkg

pytestmark = pytest.mark.gpu

LAYER_KEYS = ("w1_codes", "w1_scales", "b1", "w2_codes", "w2_scales", "b2", "router_w", "router_b")


def _load_case(name, synth):
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
    return layer, tokens, z


def near_tie_allowance(n_tokens):
    """How many tokens may select differently from the oracle because of a near-tie at the cut."""
    return max(2, n_tokens // 500)


def check_selection(idx, ref_idx, ref_logits):
    """Exact match (same experts in the same order), except tokens where the oracle's own logits are within
    1e-5 of each other at the place that differs (the cut, or two neighbours inside the selection); their
    number is bounded.  Returns a mask of the rows that match exactly."""
    same = (idx == ref_idx).all(axis=1)
    k = idx.shape[1]
    for t in np.nonzero(~same)[0]:
        s = np.sort(ref_logits[t])[::-1]
        gaps = s[:k] - s[1:k + 1]                     # between neighbours of the selection, the last one at the cut
        assert gaps.min() < 1e-5, f"token {t}: selection differs with clear logit gaps {gaps}"
    assert (~same).sum() <= near_tie_allowance(len(idx)), f"{(~same).sum()} tokens select differently from the oracle"
    return same


def check_output(out_bits, out_f32, ref, synth, rows=None, label=""):
    """Both bounds on the rows of `rows` (a mask; default all).  Prints the raw figures."""
    got = synth.bf16_bits_to_f32(out_bits).astype(np.float64)
    ref = ref.astype(np.float64)
    if rows is not None:
        got, ref = got[rows], ref[rows]
        out_f32 = None if out_f32 is None else out_f32[rows]
    err = np.abs(got - ref)
    mean_rel = err.mean() / max(np.abs(ref).mean(), 1e-30)
    rms = np.sqrt((ref ** 2).mean())
    floor = np.abs(synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(ref.astype(np.float32))).astype(np.float64) - ref).max()
    msg = (f"{label} rows {len(ref)}: max abs {err.max():.4g} (bf16 rounding of the oracle itself: {floor:.4g}), "
           f"rms(ref) {rms:.4g}, max abs / rms {err.max() / max(rms, 1e-30):.3g}, mean rel {mean_rel:.3g}")
    e32max = None
    if out_f32 is not None:
        e32max = np.abs(out_f32.astype(np.float64) - ref).max()
        msg += f", fp32 output max abs {e32max:.4g} ({e32max / max(rms, 1e-30):.3g} x rms)"
    print(msg)
    assert mean_rel <= 5e-3, f"mean relative error {mean_rel}"
    assert err.max() <= 2e-2 * max(1.0, rms), f"max abs error {err.max()} at rms {rms}"
    if rms <= 1.0:
        assert err.max() <= 2e-2, f"max abs error {err.max()} above the literal 2e-2 at rms {rms}"
    if e32max is not None:
        assert e32max <= 1e-2 * max(1.0, rms), f"fp32 output max abs error {e32max} at rms {rms}"
    return mean_rel, err.max()


def run_block(pkg, layer, tokens, flags=0, max_rows=None, keep_f32=True):
    blk = pkg.MoeBlock(layer["H"], layer["D"], layer["E"], max_rows=max_rows or max(tokens.shape[0], 1),
                       keep_f32=keep_f32)
    blk.load_layer(0, layer)
    out = blk.forward_host(0, tokens, flags=flags)
    return blk, out


@pytest.mark.parametrize("flags", [0, 1, 4, 8], ids=["tcgen05", "simt", "split_router", "split_mlp"])
@pytest.mark.parametrize("name", golden_cases())
def test_golden_fixture(name, flags, pkg, synth):
    layer, tokens, z = _load_case(name, synth)
    blk, out = run_block(pkg, layer, tokens, flags=flags)
    try:
        logits = blk.debug(pkg.DBG_LOGITS)
        np.testing.assert_allclose(logits, z["logits"], rtol=0, atol=2e-5 * max(1.0, np.abs(z["logits"]).max()))
        idx = blk.debug(pkg.DBG_TOPK_IDX)
        same = check_selection(idx, z["topk_i"], z["logits"])
        np.testing.assert_allclose(blk.debug(pkg.DBG_TOPK_W)[same], z["topk_v"][same], rtol=2e-5, atol=1e-7)
        check_output(out, blk.debug(pkg.DBG_OUT_F32), z["out"], synth, rows=same, label=name)
    finally:
        blk.close()


def test_selection_exact_on_oracle_logits(pkg, synth, port):
    """Expert choice is bit-exact whenever the fp32 logits are identical."""
    import torch
    rng = np.random.default_rng(5)
    for E in (8, 32, 128):
        T = 777
        logits = rng.normal(0, 1, size=(T, E)).astype(np.float32)
        logits[5, :] = 0.25               # all tied: lowest indices win, in order
        logits[6, 3] = logits[6, 1]       # pairwise ties
        logits[7, E - 1] = logits[7].max()
        ref_i, ref_w = port.topk_softmax(logits, 4)
        blk = pkg.MoeBlock(64, 64, E, max_rows=T)
        try:
            d_l = torch.from_numpy(logits).cuda()
            d_i = torch.empty((T, 4), dtype=torch.int32, device="cuda")
            d_w = torch.empty((T, 4), dtype=torch.float32, device="cuda")
            blk.route_topk(d_l.data_ptr(), T, d_i.data_ptr(), d_w.data_ptr(), torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            assert np.array_equal(d_i.cpu().numpy(), ref_i)
            np.testing.assert_allclose(d_w.cpu().numpy(), ref_w, rtol=2e-6, atol=1e-8)
        finally:
            blk.close()


def test_routing_invariants(pkg, synth):
    """The invariants the reference's own routing benchmark verifies on the host
    (getp-csrc/tests/bench_route_and_pack_fused_kernel.cpp:133-183)."""
    E, H, D, T, K = 16, 64, 64, 333, 4
    layer = synth.make_layer(E, H, D, seed=9, zipf_s=1.2)
    tokens = synth.make_tokens(T, H, seed=10)
    blk, _ = run_block(pkg, layer, tokens)
    try:
        idx = blk.debug(pkg.DBG_TOPK_IDX)
        counts, offsets = blk.debug(pkg.DBG_COUNTS), blk.debug(pkg.DBG_OFFSETS)
        pair_row, row_token = blk.debug(pkg.DBG_PAIR_ROW), blk.debug(pkg.DBG_ROW_TOKEN)
        assert (np.sort(idx, axis=1)[:, 1:] != np.sort(idx, axis=1)[:, :-1]).all()  # K distinct experts
        assert np.array_equal(counts, np.bincount(idx.ravel(), minlength=E))
        assert np.array_equal(offsets, np.concatenate([[0], np.cumsum(counts)]))
        assert (counts == 0).any() or True
        for t in range(T):
            for k in range(K):
                e, r = idx[t, k], pair_row[t, k]
                assert offsets[e] <= r < offsets[e] + counts[e]
                assert row_token[r] == t
        for e in range(E):
            seg = row_token[offsets[e]:offsets[e + 1]]
            assert (np.diff(seg) > 0).all()  # ascending token order inside an expert
        assert sorted(pair_row.ravel().tolist()) == list(range(T * K))
    finally:
        blk.close()


@pytest.mark.parametrize("E,H,D,T,zipf", [
    (8, 128, 128, 5, None),      # fewer rows than one MMA column group
    (8, 256, 192, 100, None),    # K tail (192 = 128 + 64), ragged counts
    (4, 128, 64, 300, None),     # every expert above the 96-row token tile
    (32, 160, 96, 47, 1.2),      # skewed: empty experts and crowded ones
    (8, 64, 544, 64, None),      # MLP1 rows 1088 = 4*256 + 64: half-empty last row block
])
def test_shapes_against_oracle(E, H, D, T, zipf, pkg, synth, port):
    layer = synth.make_layer(E, H, D, seed=E + T, zipf_s=zipf)
    tokens = synth.make_tokens(T, H, seed=H + T)
    ref_logits, ref_i, ref_w, ref_out = port.moe_layer(layer, tokens)
    for flags in (0, 1, 4, 8):
        blk, out = run_block(pkg, layer, tokens, flags=flags)
        try:
            same = check_selection(blk.debug(pkg.DBG_TOPK_IDX), ref_i, ref_logits)
            check_output(out, blk.debug(pkg.DBG_OUT_F32), ref_out, synth, rows=same)
        finally:
            blk.close()


@pytest.mark.parametrize("E,T", [(128, 1), (128, 130), (128, 1000), (128, 3000), (128, 10000), (32, 700), (24, 257),
                                 (6, 100), (256, 300)])
def test_router_forms_against_oracle(E, T, pkg, synth, port):
    """Router logits, selection, weights and histogram of the fused cluster kernel (1 to 8 k slices per token
    tile, by row count) and of the two-launch form (always taken above 128 experts), each against the oracle."""
    H, D = 576, 64   # nine 64-wide k chunks: eight slices leave some CTAs of a cluster without a chunk
    layer = synth.make_layer(E, H, D, seed=3 * E + T, zipf_s=1.1)
    tokens = synth.make_tokens(T, H, seed=T)
    ref_logits, ref_i, ref_w, _ = port.moe_layer(layer, tokens)
    for flags in (0, pkg.FWD_SPLIT_ROUTER):
        blk, _ = run_block(pkg, layer, tokens, flags=flags)
        try:
            logits = blk.debug(pkg.DBG_LOGITS)
            np.testing.assert_allclose(logits, ref_logits, rtol=0, atol=2e-5 * max(1.0, np.abs(ref_logits).max()))
            idx = blk.debug(pkg.DBG_TOPK_IDX)
            same = check_selection(idx, ref_i, ref_logits)
            np.testing.assert_allclose(blk.debug(pkg.DBG_TOPK_W)[same], ref_w[same], rtol=2e-5, atol=1e-7)
            assert np.array_equal(blk.debug(pkg.DBG_COUNTS), np.bincount(idx.ravel(), minlength=E))
        finally:
            blk.close()


@pytest.mark.parametrize("E,H,D,T,K", [
    (8, 128, 64, 150, 2),     # two experts per token: the kernels' forms for any K
    (16, 192, 96, 90, 6),
    (8, 4096, 256, 70, 4),    # the widest row the quantiser takes (its 8-vector form)
    (8, 3200, 256, 33, 4),
])
def test_other_top_k_and_wide_rows(E, H, D, T, K, pkg, synth, port):
    layer = synth.make_layer(E, H, D, seed=E + T + K)
    tokens = synth.make_tokens(T, H, seed=H + K)
    ref_logits, ref_i, ref_w, ref_out = port.moe_layer(layer, tokens, top_k=K)
    blk = pkg.MoeBlock(H, D, E, top_k=K, max_rows=T, keep_f32=True)
    try:
        blk.load_layer(0, layer)
        out = blk.forward_host(0, tokens)
        same = check_selection(blk.debug(pkg.DBG_TOPK_IDX), ref_i, ref_logits)
        np.testing.assert_allclose(blk.debug(pkg.DBG_TOPK_W)[same], ref_w[same], rtol=2e-5, atol=1e-7)
        check_output(out, blk.debug(pkg.DBG_OUT_F32), ref_out, synth, rows=same, label=f"E={E} H={H} K={K}")
        assert np.array_equal(blk.debug(pkg.DBG_COUNTS), np.bincount(blk.debug(pkg.DBG_TOPK_IDX).ravel(), minlength=E))
    finally:
        blk.close()


def test_shape20b_64_tokens(pkg, synth, port):
    """GPT-OSS-20B-shape layer, 64 tokens, seed 0: the reference's CPU-runnable case."""
    layer = synth.make_layer(32, 2880, 2880, seed=0)
    tokens = synth.make_tokens(64, 2880, seed=0)
    ref_logits, ref_i, ref_w, ref_out = port.moe_layer(layer, tokens)
    blk, out = run_block(pkg, layer, tokens)
    try:
        idx = blk.debug(pkg.DBG_TOPK_IDX)
        assert check_selection(idx, ref_i, ref_logits).all()
        assert np.array_equal(idx, ref_i)
        mean_rel, max_abs = check_output(out, blk.debug(pkg.DBG_OUT_F32), ref_out, synth, label="20B shape T=64")
        print(f"20B shape T=64: mean rel {mean_rel:.3e}, max abs {max_abs:.3e}, ref rms {np.sqrt((ref_out**2).mean()):.2f}")
        # the plain CUDA-core GEMM (fp16 operands) and the tensor-core GEMM agree to bf16 precision
        out_simt = synth.bf16_bits_to_f32(blk.forward_host(0, tokens, flags=pkg.FWD_SIMT_GEMM))
        d = np.abs(out_simt - synth.bf16_bits_to_f32(out))
        assert d.mean() / np.abs(out_simt).mean() < 5e-3 and d.max() <= 2.0  # two bf16 ulps at |y| < 256
    finally:
        blk.close()


@pytest.fixture(scope="module")
def layer_120b(synth):
    """The benchmark's layer: 120B shape, seed 0 (about a minute of host time, so it is made once)."""
    return synth.make_layer(128, 2880, 2880, seed=0)


@pytest.mark.parametrize("zipf", [None, 1.2], ids=["uniform", "zipf1.2"])
def test_headline_shape_sampled_rows_against_oracle(zipf, layer_120b, pkg, synth, port):
    """The configuration every benchmark number is quoted on (120B shape, 1856 rows, seed 0), with uniform
    and with Zipf(1.2) routing: the whole batch runs on the GPU, and 64 sampled rows are compared with the
    oracle run on those rows alone (a row's result depends on no other row: run.cpp:657-748 is a loop over
    tokens)."""
    E, H, D, T = 128, 2880, 2880, 1856
    layer = dict(layer_120b)
    if zipf is not None:
        layer["router_b"] = synth.zipf_router_bias(E, zipf)
    tokens = synth.make_tokens(T, H, seed=0)
    sample = np.sort(np.random.default_rng(2).choice(T, size=64, replace=False))
    ref_logits, ref_i, ref_w, ref_out = port.moe_layer(layer, tokens[sample])
    blk, out = run_block(pkg, layer, tokens, keep_f32=True)
    try:
        logits = blk.debug(pkg.DBG_LOGITS)[sample]
        np.testing.assert_allclose(logits, ref_logits, rtol=0, atol=2e-5 * max(1.0, np.abs(ref_logits).max()))
        same = check_selection(blk.debug(pkg.DBG_TOPK_IDX)[sample], ref_i, ref_logits)
        np.testing.assert_allclose(blk.debug(pkg.DBG_TOPK_W)[sample][same], ref_w[same], rtol=2e-5, atol=1e-7)
        check_output(out[sample], blk.debug(pkg.DBG_OUT_F32)[sample], ref_out, synth, rows=same,
                     label=f"120B shape T={T} {'zipf' if zipf else 'uniform'}")
        counts = blk.debug(pkg.DBG_COUNTS)
        assert counts.sum() == 4 * T
        if zipf is not None:
            assert counts.max() > T // 2 and (counts == 0).any()   # the skew the case is about
    finally:
        blk.close()


@pytest.mark.parametrize("zipf", [None, 1.2], ids=["uniform", "zipf1.2"])
def test_one_launch_and_two_launch_mlp_agree_bitwise(zipf, layer_120b, pkg, synth):
    """MLP1 and MLP2 in one launch (an MLP2 item waits, inside the kernel, for the MLP1 items of its token tile)
    against the same kernel launched once per phase: the arithmetic is the same, so every output bit must be;
    a tile read before it was complete would show here.  Full benchmark size, several passes."""
    E, H, D, T = 128, 2880, 2880, 1856
    layer = dict(layer_120b)
    if zipf is not None:
        layer["router_b"] = synth.zipf_router_bias(E, zipf)
    blk = pkg.MoeBlock(H, D, E, max_rows=T)
    try:
        blk.load_layer(0, layer)
        for seed in range(3):
            tokens = synth.make_tokens(T, H, seed=40 + seed)
            two = blk.forward_host(0, tokens, flags=pkg.FWD_SPLIT_MLP).copy()
            for _ in range(3):
                one = blk.forward_host(0, tokens)
                assert np.array_equal(one, two)
    finally:
        blk.close()


def test_full_size_properties(layer_120b, pkg, synth):
    """120B-shape layer at 1856 rows: properties that need no CPU run.
    Row order does not matter (a permuted batch gives the permuted output, bit
    for bit), repeated rows give repeated outputs, and two runs agree."""
    E, H, D, T = 128, 2880, 2880, 1856
    layer = layer_120b
    tokens = synth.make_tokens(T, H, seed=0)
    tokens[100] = tokens[7]
    tokens[1855] = tokens[7]
    blk, out = run_block(pkg, layer, tokens, keep_f32=False)
    try:
        out2 = blk.forward_host(0, tokens)
        assert np.array_equal(out, out2)
        assert np.array_equal(out[100], out[7]) and np.array_equal(out[1855], out[7])
        perm = np.random.default_rng(1).permutation(T)
        outp = blk.forward_host(0, tokens[perm])
        assert np.array_equal(outp, out[perm])
        counts = blk.debug(pkg.DBG_COUNTS)
        assert counts.sum() == 4 * T
        f = synth.bf16_bits_to_f32(out)
        assert np.isfinite(f).all() and 5.0 < np.sqrt((f.astype(np.float64) ** 2).mean()) < 200.0
    finally:
        blk.close()


def test_device_pointer_api_and_errors(pkg, synth, port):
    import torch
    E, H, D, T = 8, 128, 128, 40
    layer = synth.make_layer(E, H, D, seed=77)
    tokens = synth.make_tokens(T, H, seed=78)
    _, _, _, ref_out = port.moe_layer(layer, tokens)
    blk = pkg.MoeBlock(H, D, E, max_rows=64, keep_f32=True)
    try:
        with pytest.raises(pkg.MoeError) as ei:   # no weights yet
            blk.forward_host(0, tokens)
        assert ei.value.code == 6
        blk.load_layer(0, layer)
        d_t = torch.from_numpy(tokens.view(np.int16)).cuda()
        d_o = torch.empty_like(d_t)
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            blk.forward(0, d_t.data_ptr(), T, d_o.data_ptr(), 0, stream.cuda_stream)
        stream.synchronize()
        blk.synchronize()
        check_output(d_o.cpu().numpy().view(np.uint16), blk.debug(pkg.DBG_OUT_F32), ref_out, synth)
        with pytest.raises(pkg.MoeError) as ei:   # more rows than the handle was sized for
            blk.forward(0, d_t.data_ptr(), 65, d_o.data_ptr())
        assert ei.value.code == 1
        bad = dict(layer)
        bad["w1_scales"] = layer["w1_scales"].copy()
        bad["w1_scales"][0, 0, 0] = 255           # E8M0 NaN
        with pytest.raises(pkg.MoeError) as ei:
            blk.load_layer(0, bad)
        assert ei.value.code == 5
    finally:
        blk.close()


@pytest.mark.parametrize("tp", [2, 4])
def test_tp_shard_partials_sum_to_full_block(tp, pkg, synth, port):
    """Tensor-parallel shards of the intermediate dimension (one handle per rank, here all on
    one GPU): every rank routes identically, and the ranks' fp32 partial outputs add up to the
    unsharded block (MLP2 bias contributed by rank 0 only)."""
    E, H, D, T = 8, 256, 320, 90          # 320 = 10 scale blocks: uneven 32-aligned shards for tp 4
    layer = synth.make_layer(E, H, D, seed=55)
    tokens = synth.make_tokens(T, H, seed=56)
    _, ref_i, _, ref_out = port.moe_layer(layer, tokens)
    total = np.zeros((T, H), dtype=np.float64)
    covered = 0
    for r in range(tp):
        blk = pkg.MoeBlock(H, D, E, max_rows=T, tp_size=tp, tp_rank=r, keep_f32=True)
        try:
            assert blk.d0 == covered
            covered += blk.Dl
            blk.load_layer(0, layer)
            out = blk.forward_host(0, tokens)        # bf16 of the partial; the fp32 partial is kept too
            assert np.array_equal(blk.debug(pkg.DBG_TOPK_IDX), ref_i)
            part = blk.debug(pkg.DBG_OUT_F32).astype(np.float64)
            d0, d1 = blk.d0, blk.d0 + blk.Dl
            _, _, _, ref_part = port.moe_layer(layer, tokens, shard=(d0, d1), add_b2=(r == 0))
            rms = max(1.0, float(np.sqrt((ref_part.astype(np.float64) ** 2).mean())))
            assert np.abs(part - ref_part).max() <= 1e-2 * rms
            total += part
        finally:
            blk.close()
    assert covered == D
    err = np.abs(total - ref_out)
    assert err.mean() / np.abs(ref_out).mean() <= 5e-3
    assert err.max() <= 1e-2 * max(1.0, float(np.sqrt((ref_out.astype(np.float64) ** 2).mean())))


# ---- the block in the reference's calling form: x <- x + MoE(rmsnorm(x) * gain) ----

def check_block_form(pkg, synth, port, layer, x_bits, gain_bits, ref=None):
    """moe_block() against the oracle.  t must equal the oracle's bf16-rounded RMSNorm but for rare
    one-ulp (bf16) differences (the kernel's fp32 products against the oracle's double ones); the
    updated rows x must be the oracle's x + e_agg within the block tolerance plus one bf16 rounding of
    the sum (2^-8 relative)."""
    import torch
    T, H = x_bits.shape
    x, gain = synth.bf16_bits_to_f32(x_bits), synth.bf16_bits_to_f32(gain_bits)
    if ref is None:
        ref = port.moe_block(layer, x, gain, t_as_bf16=True)
    t_ref, logits_ref, idx_ref, _, agg_ref, xo_ref = ref
    blk = pkg.MoeBlock(H, layer["D"], layer["E"], max_rows=T)
    try:
        blk.load_layer(0, layer)
        d_x = torch.from_numpy(x_bits.view(np.int16).copy()).cuda()
        d_g = torch.from_numpy(gain_bits.view(np.int16).copy()).cuda()
        blk.block(0, d_x.data_ptr(), d_g.data_ptr(), T, 0, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        blk.synchronize()
        t_got = blk.debug(pkg.DBG_TNORM)
        t_want = synth.f32_to_bf16_bits(t_ref)
        diff = t_got.astype(np.int32) - t_want.astype(np.int32)
        assert np.abs(diff).max() <= 1, "normalised rows differ by more than one bf16 ulp"
        assert (diff != 0).mean() <= 2e-3, f"{(diff != 0).mean():.2%} of the normalised rows differ"
        same = check_selection(blk.debug(pkg.DBG_TOPK_IDX), idx_ref, logits_ref)
        got = synth.bf16_bits_to_f32(d_x.cpu().numpy().view(np.uint16)).astype(np.float64)
        err = np.abs(got - xo_ref)[same]
        rms = np.sqrt((agg_ref[same].astype(np.float64) ** 2).mean())
        bound = (2e-2 * max(1.0, rms) + 2.0 ** -8 * np.abs(xo_ref))[same]
        assert (err <= bound).all(), f"max excess {(err - bound).max()}"
        upd = np.abs((got - x) - agg_ref)[same].mean() / max(np.abs(agg_ref[same]).mean(), 1e-30)
        # the update itself, seen through the rounding of the sum: coarse, but catches a missing residual or bias
        assert upd <= 0.1, f"mean relative error of the update {upd}"
    finally:
        blk.close()


@pytest.mark.parametrize("name", golden_block_cases())
def test_block_form_golden(name, pkg, synth, port):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    layer = {k: z[k] for k in LAYER_KEYS}
    layer.update(E=int(z["E"]), H=int(z["H"]), D=int(z["D"]))
    # the reference's CPU forward keeps t in fp32; rounding t to bf16 as its GPU path does is the oracle's switch
    x, gain = synth.bf16_bits_to_f32(z["x"]), synth.bf16_bits_to_f32(z["gain"])
    ref32 = port.moe_block(layer, x, gain, t_as_bf16=False)
    assert np.array_equal(ref32[0], z["t"]) and np.array_equal(ref32[4], z["e_agg"])
    check_block_form(pkg, synth, port, layer, z["x"], z["gain"])


def test_block_form_20b_shape(pkg, synth, port):
    layer = synth.make_layer(32, 2880, 2880, seed=3)
    x_bits, gain_bits = synth.make_residual(48, 2880, seed=4)
    check_block_form(pkg, synth, port, layer, x_bits, gain_bits)


def test_host_pipeline_submit_wait(pkg, synth):
    """Batches in flight through submit/wait give the same bits as the blocking call, in any overlap;
    a fourth submit without a wait is refused and the handle stays usable."""
    E, H, D = 16, 256, 320
    layer = synth.make_layer(E, H, D, seed=90)
    batches = [synth.make_tokens(rows, H, seed=91 + i) for i, rows in enumerate((70, 128, 1, 99, 128, 33, 64))]
    blk = pkg.MoeBlock(H, D, E, max_rows=128)
    try:
        blk.load_layer(0, layer)
        want = [blk.forward_host(0, b).copy() for b in batches]
        pin_in = [pkg.PinnedBuffer(b.shape, np.uint16) for b in batches]
        pin_out = [pkg.PinnedBuffer(b.shape, np.uint16) for b in batches]
        for p, b in zip(pin_in, batches):
            p.array[:] = b
        tickets = []
        for i in range(len(batches)):
            if len(tickets) == 3:
                blk.forward_host_wait(tickets.pop(0))
            tickets.append(blk.forward_host_submit(0, pin_in[i].array, pin_out[i].array))
        for t in tickets:
            blk.forward_host_wait(t)
        for i, w in enumerate(want):
            assert np.array_equal(pin_out[i].array, w), f"batch {i}"
        # three in flight, a fourth is refused
        ts = [blk.forward_host_submit(0, pin_in[i].array, pin_out[i].array) for i in range(3)]
        with pytest.raises(pkg.MoeError) as ei:
            blk.forward_host_submit(0, pin_in[3].array, pin_out[3].array)
        assert ei.value.code == 6
        for t in ts:
            blk.forward_host_wait(t)
        blk.forward_host_wait(ts[0])          # waiting twice is harmless
        t = blk.forward_host_submit(0, pin_in[3].array, pin_out[3].array)
        blk.forward_host_wait(t)
        assert np.array_equal(pin_out[3].array, want[3])
        for p in pin_in + pin_out:
            p.free()
    finally:
        blk.close()


def test_forward_in_a_cuda_graph(pkg, synth):
    """The per-layer call is stream-ordered work only (no allocation, no host synchronisation), so a caller
    can capture it once and replay it per step (the reference launches every kernel of every layer from the
    host, getp_run.cpp:3313-3367).  A replay on new rows gives the bits of a direct call."""
    import torch
    E, H, D, T = 16, 256, 320, 96
    layer = synth.make_layer(E, H, D, seed=41)
    a, b = synth.make_tokens(T, H, seed=42), synth.make_tokens(T, H, seed=43)
    blk = pkg.MoeBlock(H, D, E, max_rows=T)
    try:
        blk.load_layer(0, layer)
        want_a, want_b = blk.forward_host(0, a).copy(), blk.forward_host(0, b).copy()
        d_t = torch.from_numpy(a.view(np.int16).copy()).cuda()
        d_o = torch.zeros_like(d_t)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            blk.forward(0, d_t.data_ptr(), T, d_o.data_ptr(), 0, s.cuda_stream)   # first call outside the capture
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            blk.forward(0, d_t.data_ptr(), T, d_o.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
        for rows, want in ((a, want_a), (b, want_b), (a, want_a)):
            d_t.copy_(torch.from_numpy(rows.view(np.int16).copy()))
            d_o.zero_()
            g.replay()
            torch.cuda.synchronize()
            assert np.array_equal(d_o.cpu().numpy().view(np.uint16), want)
        blk.synchronize()
    finally:
        blk.close()


def test_expert_output_beyond_fp16_is_reported(pkg, synth):
    """The per-(token, expert) MLP2 outputs wait for the combine in fp16; a magnitude above 65504 is an
    error code, not a silent infinity, and the handle keeps working."""
    E, H, D, T = 8, 128, 128, 20
    layer = synth.make_layer(E, H, D, seed=51)
    tokens = synth.make_tokens(T, H, seed=52)
    bad = dict(layer)
    bad["b2"] = layer["b2"].copy()
    bad["b2"][:, 5] = synth.f32_to_bf16_bits(np.float32(1.0e5))
    blk = pkg.MoeBlock(H, D, E, max_rows=T, n_layers=2)
    try:
        blk.load_layer(0, layer)
        blk.load_layer(1, bad)
        good = blk.forward_host(0, tokens).copy()
        with pytest.raises(pkg.MoeError) as ei:
            blk.forward_host(1, tokens)
        assert ei.value.code == 8
        assert np.array_equal(blk.forward_host(0, tokens), good)
    finally:
        blk.close()
