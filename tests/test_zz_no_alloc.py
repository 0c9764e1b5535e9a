"""moe_route_static: routing for callers that must not touch the CUDA allocator.

Some users of this library run in a place where cudaMalloc is off limits when
a routing decision is needed: a serving loop whose device memory was handed
out once at start-up by a pool that owns the rest of the GPU, or a
latency-critical thread that cannot take the device-wide synchronisation a
cudaMalloc implies.  For them the router's split-k scratch is a fixed 8 MiB
array inside the library's device image; the entry point allocates nothing and
writes only into buffers the caller passes.

The check: its logits, expert indices and routing weights equal what the
regular entry point (moe_forward, read back through moe_get_debug) produces
for the same rows, on two calls in a row with different batches (the array
keeps the first call's contents, which the second must not be disturbed by).
This file sorts last so that a run that stops at the first failure has already
run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_route_static_matches_regular_path_twice(pkg, synth):
    import torch
    E, H, D = 32, 2880, 64
    layer = synth.make_layer(E, H, D, seed=91)
    blk = pkg.MoeBlock(H, D, E, max_rows=700)
    try:
        blk.load_layer(0, layer)
        stream = torch.cuda.current_stream().cuda_stream
        for call, T in enumerate((700, 333)):       # the second, smaller call sees the first one's leftovers
            tokens = synth.make_tokens(T, H, seed=92 + call)
            d_t = torch.from_numpy(tokens.view(np.int16)).cuda()
            d_o = torch.empty_like(d_t)
            blk.forward(0, d_t.data_ptr(), T, d_o.data_ptr(), 0, stream)
            torch.cuda.synchronize()
            ref_logits = blk.debug(pkg.DBG_LOGITS)
            ref_idx, ref_w = blk.debug(pkg.DBG_TOPK_IDX), blk.debug(pkg.DBG_TOPK_W)

            logits = torch.full((T, E), float("nan"), dtype=torch.float32, device="cuda")
            idx = torch.full((T, 4), -1, dtype=torch.int32, device="cuda")
            w = torch.full((T, 4), float("nan"), dtype=torch.float32, device="cuda")
            blk.route_static(0, d_t.data_ptr(), T, logits.data_ptr(), idx.data_ptr(), w.data_ptr(), stream)
            torch.cuda.synchronize()
            blk.synchronize()
            got = logits.cpu().numpy()
            # same kernels; the k-slices may be grouped differently, so allow the logit tolerance of the GPU tests
            np.testing.assert_allclose(got, ref_logits, rtol=0, atol=2e-5 * max(1.0, float(np.abs(ref_logits).max())))
            same = (np.sort(idx.cpu().numpy(), axis=1) == np.sort(ref_idx, axis=1)).all(axis=1)
            for t in np.nonzero(~same)[0]:           # only a near-tie at the cut may differ
                s = np.sort(ref_logits[t])[::-1]
                assert s[3] - s[4] < 1e-5
            ok = same & (idx.cpu().numpy() == ref_idx).all(axis=1)
            np.testing.assert_allclose(w.cpu().numpy()[ok], ref_w[ok], rtol=2e-5, atol=1e-7)
            assert ok.mean() > 0.99
    finally:
        blk.close()


def test_route_static_sliced_to_fit_after_a_larger_call(pkg, synth, port):
    """A batch whose usual number of k-slices does not fit the fixed array (256 experts x 2368 rows: four slices
    of 606 208 floats against 2 097 152) is routed with fewer, longer slices.  It runs right after a larger batch
    that filled more of the array, and both are checked against the CPU oracle as well as against the regular
    entry point.  The call must leave the amount of free device memory as it found it."""
    import torch
    E, H, D = 256, 512, 64
    layer = synth.make_layer(E, H, D, seed=95)
    blk = pkg.MoeBlock(H, D, E, max_rows=4000)
    try:
        blk.load_layer(0, layer)
        stream = torch.cuda.current_stream().cuda_stream
        for call, T in enumerate((4000, 2368)):
            tokens = synth.make_tokens(T, H, seed=96 + call)
            ref_logits, ref_i, ref_w, _ = port.moe_layer(layer, tokens)
            d_t = torch.from_numpy(tokens.view(np.int16)).cuda()
            d_o = torch.empty_like(d_t)
            blk.forward(0, d_t.data_ptr(), T, d_o.data_ptr(), 0, stream)
            torch.cuda.synchronize()
            reg_logits, reg_idx = blk.debug(pkg.DBG_LOGITS), blk.debug(pkg.DBG_TOPK_IDX)
            logits = torch.full((T, E), float("nan"), dtype=torch.float32, device="cuda")
            idx = torch.full((T, 4), -1, dtype=torch.int32, device="cuda")
            w = torch.full((T, 4), float("nan"), dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            blk.route_static(0, d_t.data_ptr(), T, logits.data_ptr(), idx.data_ptr(), w.data_ptr(), stream)
            torch.cuda.synchronize()
            blk.synchronize()
            assert torch.cuda.mem_get_info()[0] == free_before, "moe_route_static changed the free device memory"
            got, got_i, got_w = logits.cpu().numpy(), idx.cpu().numpy(), w.cpu().numpy()
            tol = 2e-5 * max(1.0, float(np.abs(ref_logits).max()))
            np.testing.assert_allclose(got, ref_logits, rtol=0, atol=tol)
            np.testing.assert_allclose(got, reg_logits, rtol=0, atol=tol)
            srt = np.sort(ref_logits, axis=1)[:, ::-1]
            near_tie = (srt[:, :4] - srt[:, 1:5]).min(axis=1) < 1e-5
            for other in (ref_i, reg_idx):
                differ = (got_i != other).any(axis=1)
                assert (near_tie | ~differ).all(), "selection differs from the oracle where its logits are clearly apart"
                assert differ.sum() <= max(2, T // 500)
            ok = (got_i == ref_i).all(axis=1)
            np.testing.assert_allclose(got_w[ok], ref_w[ok], rtol=2e-5, atol=1e-7)
    finally:
        blk.close()


def test_route_static_rejects_oversize(pkg, synth):
    import torch
    E, H, D = 256, 64, 64
    rows = (2 << 20) // E + 1                        # one row past the fixed scratch
    layer = synth.make_layer(E, H, D, seed=93)
    blk = pkg.MoeBlock(H, D, E, max_rows=rows)
    try:
        blk.load_layer(0, layer)
        t = torch.zeros((rows, H), dtype=torch.int16, device="cuda")
        logits = torch.empty((rows, E), dtype=torch.float32, device="cuda")
        idx = torch.empty((rows, 4), dtype=torch.int32, device="cuda")
        w = torch.empty((rows, 4), dtype=torch.float32, device="cuda")
        with pytest.raises(pkg.MoeError) as ei:
            blk.route_static(0, t.data_ptr(), rows, logits.data_ptr(), idx.data_ptr(), w.data_ptr())
        assert ei.value.code == 1 and "8 MiB" in str(ei.value)
        blk.route_static(0, t.data_ptr(), rows - 1, logits.data_ptr(), idx.data_ptr(), w.data_ptr())
        torch.cuda.synchronize()
    finally:
        blk.close()
