"""Python harness around libmoe_b200.so, the sm_100a MoE block.

The product is the C-ABI library (include/moe_b200.h) and the C++ shim that
recreates the reference's entry points (include/moe_b200_shim.hpp).  This module
only loads the library through ctypes so that tests and bench.py can drive it;
there is no Python or CPU implementation behind it: if the library is missing
or the device is not a B200, calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import synth  # noqa: F401  (re-exported for tests and bench)

HERE = os.path.dirname(os.path.abspath(__file__))
# MOE_B200_LIB selects another build of the same library (e.g. one compiled with extra flags).
LIB_PATH = os.environ.get("MOE_B200_LIB") or os.path.join(HERE, "libmoe_b200.so")

MOE_OK = 0
ERR_NAMES = {1: "INVALID", 2: "CUDA", 3: "NOMEM", 4: "TIMEOUT", 5: "SCALE_RANGE", 6: "STATE", 7: "NO_SM100", 8: "Y_RANGE"}

CFG_KEEP_F32_OUT = 1
FWD_SIMT_GEMM = 1
FWD_PARTIAL_F32 = 2
FWD_SPLIT_ROUTER = 4
FWD_SPLIT_MLP = 8

DBG_LOGITS, DBG_TOPK_IDX, DBG_TOPK_W, DBG_COUNTS, DBG_OFFSETS, DBG_PAIR_ROW, DBG_ROW_TOKEN, DBG_OUT_F32, \
    DBG_STATUS, DBG_HBUF, DBG_YBUF, DBG_GATHER, DBG_TNORM, DBG_TP_PARTIAL = range(14)

EXPORTS = [
    "moe_create", "moe_destroy", "moe_load_layer", "moe_shard_range", "moe_forward", "moe_forward_host",
    "moe_synchronize", "moe_host_alloc", "moe_host_free", "moe_route_topk", "moe_get_debug",
    "moe_last_error", "moe_strerror", "moe_launch_count", "moe_profile_enable", "moe_profile_collect",
    "moe_route_static", "moe_block", "moe_forward_host_submit", "moe_forward_host_wait",
    "moe_quantize_mxfp4", "moe_load_layer_f32", "moe_tp_export", "moe_tp_attach_ipc", "moe_tp_buffer", "moe_tp_attach_ptr",
    "moe_tp_forward", "moe_tp_forward_host", "moe_tp_allgather", "moe_tp_reduce_scatter", "moe_tp_allreduce",
    "moe_load_layer_from_bin", "moe_bin_layer_offsets",
]
TP_BUF_GATHER, TP_BUF_PARTIAL, TP_BUF_FLAGS, TP_BUF_TOPK_IDX, TP_BUF_TOPK_W = range(5)
TP_N_BUFS = 5
TP_HANDLE_BYTES = 64
STAGES = ("router", "topk", "index", "gather", "mlp1", "mlp2", "combine")


class MoeConfig(C.Structure):
    _fields_ = [("hidden_dim", C.c_int), ("intermediate_dim", C.c_int), ("n_experts", C.c_int),
                ("experts_per_token", C.c_int), ("n_layers", C.c_int), ("swiglu_limit", C.c_float),
                ("swiglu_alpha", C.c_float), ("max_rows", C.c_int), ("tp_size", C.c_int), ("tp_rank", C.c_int),
                ("device", C.c_int), ("flags", C.c_uint)]


class MoeError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"moe_b200 error {code} ({ERR_NAMES.get(code, '?')}): {msg}")
        self.code = code


_lib = None


def lib() -> C.CDLL:
    """Loads the C-ABI library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(f"{LIB_PATH} missing: run `python -m gpt-oss_b200.build` "
                                    "(or __graft_entry__.build()); there is no fallback path")
        L = C.CDLL(LIB_PATH)
        L.moe_create.argtypes = [C.POINTER(MoeConfig), C.POINTER(C.c_void_p)]
        L.moe_destroy.argtypes = [C.c_void_p]
        L.moe_load_layer.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 8
        L.moe_shard_range.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.moe_forward.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_uint, C.c_void_p]
        L.moe_forward_host.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_uint]
        L.moe_synchronize.argtypes = [C.c_void_p]
        L.moe_host_alloc.argtypes = [C.c_size_t]
        L.moe_host_alloc.restype = C.c_void_p
        L.moe_host_free.argtypes = [C.c_void_p]
        L.moe_route_topk.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.moe_get_debug.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t]
        L.moe_last_error.argtypes = [C.c_void_p]
        L.moe_last_error.restype = C.c_char_p
        L.moe_strerror.argtypes = [C.c_int]
        L.moe_strerror.restype = C.c_char_p
        L.moe_launch_count.argtypes = [C.c_void_p]
        L.moe_launch_count.restype = C.c_longlong
        L.moe_route_static.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_void_p]
        L.moe_tp_export.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.moe_tp_attach_ipc.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.moe_tp_buffer.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_void_p)]
        L.moe_tp_attach_ptr.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.moe_tp_forward.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_uint, C.c_void_p]
        L.moe_tp_forward_host.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_uint]
        L.moe_tp_allgather.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.moe_tp_reduce_scatter.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        L.moe_load_layer_from_bin.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_int, C.c_void_p]
        L.moe_bin_layer_offsets.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        L.moe_tp_allreduce.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        L.moe_forward_host_submit.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_uint,
                                              C.POINTER(C.c_longlong)]
        L.moe_forward_host_wait.argtypes = [C.c_void_p, C.c_longlong]
        L.moe_quantize_mxfp4.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]
        L.moe_load_layer_f32.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 6
        L.moe_block.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_uint, C.c_void_p]
        L.moe_profile_enable.argtypes = [C.c_void_p, C.c_int]
        L.moe_profile_collect.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_int)]
        _lib = L
    return _lib


def shard_range(inter: int, tp_size: int, tp_rank: int) -> tuple[int, int]:
    s, n = C.c_int(), C.c_int()
    rc = lib().moe_shard_range(inter, tp_size, tp_rank, C.byref(s), C.byref(n))
    if rc != MOE_OK:
        raise MoeError(rc, "moe_shard_range")
    return s.value, n.value


def quantize_mxfp4(src_ptr: int, n_elems: int, codes_ptr: int, scales_ptr: int, stream: int = 0):
    """Device pointers: fp32 [n] -> e2m1 codes [ceil(n/32)*16] and E8M0 scales [ceil(n/32)]."""
    rc = lib().moe_quantize_mxfp4(C.c_void_p(src_ptr), n_elems, C.c_void_p(codes_ptr), C.c_void_p(scales_ptr),
                                  C.c_void_p(stream))
    if rc != MOE_OK:
        raise MoeError(rc, "moe_quantize_mxfp4")


class PinnedBuffer:
    """Page-locked host memory from moe_host_alloc, viewed as a numpy array."""

    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape)) * self.dtype.itemsize
        self.ptr = lib().moe_host_alloc(self.nbytes)
        if not self.ptr:
            raise MemoryError("moe_host_alloc failed")
        buf = (C.c_uint8 * self.nbytes).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=self.dtype).reshape(self.shape)

    def free(self):
        if self.ptr:
            self.array = None
            lib().moe_host_free(self.ptr)
            self.ptr = None


class MoeBlock:
    """One handle of the C-ABI library (one GPU, one TP rank)."""

    def __init__(self, hidden: int, inter: int, n_experts: int, top_k: int = 4, n_layers: int = 1,
                 max_rows: int = 2048, tp_size: int = 1, tp_rank: int = 0, device: int = 0,
                 keep_f32: bool = False, limit: float = 7.0, alpha: float = 1.702):
        self.L = lib()
        self.cfg = MoeConfig(hidden, inter, n_experts, top_k, n_layers, limit, alpha, max_rows, tp_size,
                             tp_rank, device, CFG_KEEP_F32_OUT if keep_f32 else 0)
        self.h = C.c_void_p()
        rc = self.L.moe_create(C.byref(self.cfg), C.byref(self.h))
        if rc != MOE_OK:
            msg = self.L.moe_last_error(self.h).decode() if self.h else "moe_create"
            if self.h:
                self.L.moe_destroy(self.h)
                self.h = C.c_void_p()
            raise MoeError(rc, msg)
        self.H, self.D, self.E, self.K = hidden, inter, n_experts, top_k
        self.d0, self.Dl = shard_range(inter, tp_size, tp_rank)
        self.rows = 0

    def _check(self, rc: int):
        if rc != MOE_OK:
            raise MoeError(rc, self.L.moe_last_error(self.h).decode())

    def load_layer(self, idx: int, layer: dict):
        arrs = [np.ascontiguousarray(layer[k]) for k in
                ("w1_codes", "w1_scales", "b1", "w2_codes", "w2_scales", "b2")]
        arrs.append(np.ascontiguousarray(layer["router_w"], dtype=np.float32))
        arrs.append(np.ascontiguousarray(layer["router_b"], dtype=np.float32))
        E, H, D = self.E, self.H, self.D
        want = [(E, 2 * D, H // 2), (E, 2 * D, H // 32), (E, 2 * D), (E, H, D // 2), (E, H, D // 32), (E, H),
                (E, H), (E,)]
        for a, w in zip(arrs, want):
            assert a.shape == w, (a.shape, w)
        self._check(self.L.moe_load_layer(self.h, idx, *[a.ctypes.data_as(C.c_void_p) for a in arrs]))

    def forward_host(self, layer: int, t_bits: np.ndarray, out: np.ndarray | None = None,
                     flags: int = 0) -> np.ndarray:
        """bf16 bit patterns [rows, H] in host memory -> bf16 bit patterns [rows, H]."""
        t_bits = np.ascontiguousarray(t_bits, dtype=np.uint16)
        rows = t_bits.shape[0]
        if out is None:
            out = np.empty_like(t_bits)
        self._check(self.L.moe_forward_host(self.h, layer, t_bits.ctypes.data_as(C.c_void_p), rows,
                                            out.ctypes.data_as(C.c_void_p), flags))
        self.rows = rows
        return out

    def load_layer_f32(self, layer: int, w1: np.ndarray, b1: np.ndarray, w2: np.ndarray, b2: np.ndarray,
                       router_w: np.ndarray, router_b: np.ndarray):
        """fp32 expert tensors (w1 [E,2D,H], b1 [E,2D], w2 [E,H,D], b2 [E,H]) quantised to MXFP4 on the GPU."""
        arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in (w1, b1, w2, b2, router_w, router_b)]
        self._check(self.L.moe_load_layer_f32(self.h, layer, *[a.ctypes.data_as(C.c_void_p) for a in arrs]))

    def load_layer_from_bin(self, layer: int, path: str, file_layer: int = 0) -> np.ndarray:
        """Loads the MoE tensors of one layer of a checkpoint in the reference's flat fp32 layout; returns the
        layer's pre-MoE RMSNorm gain (fp32 [H])."""
        gain = np.empty(self.H, dtype=np.float32)
        self._check(self.L.moe_load_layer_from_bin(self.h, layer, path.encode(), file_layer, gain.ctypes.data_as(C.c_void_p)))
        return gain

    def forward_host_submit(self, layer: int, t_bits: np.ndarray, out: np.ndarray, flags: int = 0) -> int:
        """Starts one batch (host arrays, ideally PinnedBuffer.array, kept alive until the wait) and returns
        its ticket; up to three batches may be in flight."""
        assert t_bits.dtype == np.uint16 and t_bits.flags.c_contiguous and out.flags.c_contiguous
        ticket = C.c_longlong(-1)
        self._check(self.L.moe_forward_host_submit(self.h, layer, t_bits.ctypes.data_as(C.c_void_p), t_bits.shape[0],
                                                   out.ctypes.data_as(C.c_void_p), flags, C.byref(ticket)))
        self.rows = t_bits.shape[0] * self.cfg.tp_size
        return ticket.value

    def forward_host_wait(self, ticket: int):
        self._check(self.L.moe_forward_host_wait(self.h, C.c_longlong(ticket)))

    def forward(self, layer: int, t_ptr: int, rows: int, out_ptr: int, flags: int = 0, stream: int = 0):
        """Device pointers; stream-ordered, does not wait."""
        self._check(self.L.moe_forward(self.h, layer, C.c_void_p(t_ptr), rows, C.c_void_p(out_ptr), flags,
                                       C.c_void_p(stream)))
        self.rows = rows

    def block(self, layer: int, x_ptr: int, rms_w_ptr: int, rows_local: int, flags: int = 0, stream: int = 0):
        """x <- x + MoE(rmsnorm(x) * w), in place, device pointers (the reference's moe_gpu form)."""
        self._check(self.L.moe_block(self.h, layer, C.c_void_p(x_ptr), C.c_void_p(rms_w_ptr), rows_local, flags,
                                     C.c_void_p(stream)))
        self.rows = rows_local * self.cfg.tp_size

    def synchronize(self):
        self._check(self.L.moe_synchronize(self.h))

    def route_topk(self, logits_ptr: int, rows: int, idx_ptr: int, w_ptr: int, stream: int = 0):
        self._check(self.L.moe_route_topk(self.h, C.c_void_p(logits_ptr), rows, C.c_void_p(idx_ptr),
                                          C.c_void_p(w_ptr), C.c_void_p(stream)))

    def route_static(self, layer: int, t_ptr: int, rows: int, logits_ptr: int, idx_ptr: int, w_ptr: int,
                     stream: int = 0):
        """Router + top-k + softmax with the library's fixed scratch array; allocates nothing."""
        self._check(self.L.moe_route_static(self.h, layer, C.c_void_p(t_ptr), rows, C.c_void_p(logits_ptr),
                                            C.c_void_p(idx_ptr), C.c_void_p(w_ptr), C.c_void_p(stream)))

    # ---- tensor-parallel group -------------------------------------------------------------
    def tp_export_all(self) -> bytes:
        """The IPC handles of this rank's symmetric buffers, TP_N_BUFS x 64 bytes."""
        out = b""
        for which in range(TP_N_BUFS):
            buf = C.create_string_buffer(TP_HANDLE_BYTES)
            self._check(self.L.moe_tp_export(self.h, which, buf))
            out += buf.raw
        return out

    def tp_attach_all(self, rank: int, blob: bytes):
        """Attaches rank `rank`'s buffers from the bytes its tp_export_all() returned."""
        assert len(blob) == TP_N_BUFS * TP_HANDLE_BYTES
        for which in range(TP_N_BUFS):
            part = blob[which * TP_HANDLE_BYTES:(which + 1) * TP_HANDLE_BYTES]
            self._check(self.L.moe_tp_attach_ipc(self.h, which, rank, C.c_char_p(part)))

    def tp_buffer(self, which: int) -> int:
        p = C.c_void_p()
        self._check(self.L.moe_tp_buffer(self.h, which, C.byref(p)))
        return p.value

    def tp_forward(self, layer: int, t_ptr: int, rows_local: int, out_ptr: int, flags: int = 0, stream: int = 0):
        self._check(self.L.moe_tp_forward(self.h, layer, C.c_void_p(t_ptr), rows_local, C.c_void_p(out_ptr), flags,
                                          C.c_void_p(stream)))
        self.rows = rows_local * self.cfg.tp_size

    def tp_forward_host(self, layer: int, t_bits: np.ndarray, out: np.ndarray, flags: int = 0) -> np.ndarray:
        rows = t_bits.shape[0]
        self._check(self.L.moe_tp_forward_host(self.h, layer, t_bits.ctypes.data_as(C.c_void_p), rows,
                                               out.ctypes.data_as(C.c_void_p), flags))
        self.rows = rows * self.cfg.tp_size
        return out

    def tp_allgather(self, src_ptr: int, rows_local: int, stream: int = 0):
        self._check(self.L.moe_tp_allgather(self.h, C.c_void_p(src_ptr), rows_local, C.c_void_p(stream)))

    def tp_reduce_scatter(self, rows_local: int, out_ptr: int, stream: int = 0):
        self._check(self.L.moe_tp_reduce_scatter(self.h, rows_local, C.c_void_p(out_ptr), C.c_void_p(stream)))

    def tp_allreduce(self, buf_ptr: int, n_elems: int, stream: int = 0):
        """In place: bf16 buffer <- sum over the ranks of the group (fp32 adds in rank order)."""
        self._check(self.L.moe_tp_allreduce(self.h, C.c_void_p(buf_ptr), n_elems, C.c_void_p(stream)))

    def debug(self, which: int) -> np.ndarray:
        T, E, K, H = self.rows, self.E, self.K, self.H
        shape, dt = {
            DBG_LOGITS: ((T, E), np.float32), DBG_TOPK_IDX: ((T, K), np.int32), DBG_TOPK_W: ((T, K), np.float32),
            DBG_COUNTS: ((E,), np.int32), DBG_OFFSETS: ((E + 1,), np.int32), DBG_PAIR_ROW: ((T, K), np.int32),
            DBG_ROW_TOKEN: ((T * K,), np.int32), DBG_OUT_F32: ((T, H), np.float32),
            DBG_STATUS: ((1,), np.uint32), DBG_YBUF: ((T * K, H), np.float16),
            DBG_GATHER: ((T, H), np.uint16), DBG_TNORM: ((T // self.cfg.tp_size, H), np.uint16),
            DBG_TP_PARTIAL: ((T, H), np.uint16)}[which]
        out = np.empty(shape, dtype=dt)
        self._check(self.L.moe_get_debug(self.h, which, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def profile(self, on: bool):
        self._check(self.L.moe_profile_enable(self.h, int(on)))

    def profile_collect(self) -> tuple[dict, int]:
        """Summed milliseconds per stage and the number of profiled calls."""
        ms = (C.c_float * len(STAGES))()
        n = C.c_int()
        self._check(self.L.moe_profile_collect(self.h, ms, C.byref(n)))
        return {k: float(ms[i]) for i, k in enumerate(STAGES)}, n.value

    def launches(self) -> int:
        return int(self.L.moe_launch_count(self.h))

    def close(self):
        if self.h:
            self.L.moe_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
