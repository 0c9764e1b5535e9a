"""TEST INFRASTRUCTURE ONLY: ctypes front end of the two CPU checkers.

* ``Port``      -> oracle/libmoe_oracle.so, this repository's C restatement
                   (moe_oracle.c) of the reference MoE block, run.cpp:657-748.
* ``Reference`` -> oracle/_ref/libref_moe.so, the reference's own run.cpp
                   forward() driven on a one-layer in-memory model
                   (ref_driver.inc.cpp).  Present only where oracle/Makefile
                   could read the reference checkout, or where the prebuilt
                   binary travelled with the tree.

Only tests/, the smoke check and the CPU-baseline legs of bench.py may import
this module; the product library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "libmoe_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libref_moe.so")
REF_MXFP4_SO = os.path.join(HERE, "_ref", "libref_mxfp4.so")


def reference_dir() -> str:
    """Where the reference checkout is looked for: MOE_REFERENCE_DIR, else a directory named
    `reference` beside this repository."""
    return os.environ.get("MOE_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(quiet: bool = True) -> None:
    """Compile the checkers (the reference one only where its sources exist)."""
    subprocess.run(["make", "-C", HERE, "all", f"REF={reference_dir()}"], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _ptr(a: np.ndarray, ty):
    return a.ctypes.data_as(C.POINTER(ty))


def _bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _prep(layer: dict) -> dict:
    """Contiguous views in the dtypes the C side expects; biases widened to f32."""
    out = {k: np.ascontiguousarray(layer[k]) for k in
           ("w1_codes", "w1_scales", "w2_codes", "w2_scales")}
    out["b1"] = np.ascontiguousarray(_bf16_to_f32(layer["b1"]))
    out["b2"] = np.ascontiguousarray(_bf16_to_f32(layer["b2"]))
    out["router_w"] = np.ascontiguousarray(layer["router_w"], dtype=np.float32)
    out["router_b"] = np.ascontiguousarray(layer["router_b"], dtype=np.float32)
    return out


class Port:
    """The C restatement.  Inputs: a layer dict from synth.make_layer and bf16 bit
    patterns [T, H]; outputs float32 logits [T,E], int32 top-k [T,K], float32
    weights [T,K] and the float32 block output [T,H]."""

    def __init__(self):
        if not os.path.exists(PORT_SO):
            build()
        self.lib = C.CDLL(PORT_SO)
        self.lib.oracle_moe_layer_shard.restype = C.c_int
        self.lib.oracle_num_threads.restype = C.c_int

    def threads(self) -> int:
        return int(self.lib.oracle_num_threads())

    def set_threads(self, n: int) -> None:
        self.lib.oracle_set_num_threads(int(n))

    def dequant(self, codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
        codes = np.ascontiguousarray(codes)
        scales = np.ascontiguousarray(scales)
        out = np.empty(codes.shape[:-1] + (codes.shape[-1] * 2,), dtype=np.float32)
        self.lib.oracle_mxfp4_dequant(_ptr(codes, C.c_uint8), _ptr(scales, C.c_uint8),
                                      C.c_size_t(out.size), _ptr(out, C.c_float))
        return out

    def quantize(self, values: np.ndarray):
        """fp32 values (flattened) -> (codes uint8 [ceil(n/32)*16], scales uint8 [ceil(n/32)])."""
        v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        nblk = (v.size + 31) // 32
        codes = np.empty(nblk * 16, dtype=np.uint8)
        scales = np.empty(nblk, dtype=np.uint8)
        self.lib.oracle_mxfp4_quantize.restype = None
        self.lib.oracle_mxfp4_quantize(_ptr(v, C.c_float), C.c_size_t(v.size), _ptr(codes, C.c_uint8),
                                       _ptr(scales, C.c_uint8))
        return codes, scales

    def topk_softmax(self, logits: np.ndarray, k: int = 4):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        T, E = logits.shape
        idx = np.empty((T, k), dtype=np.int32)
        w = np.empty((T, k), dtype=np.float32)
        self.lib.oracle_topk_softmax(_ptr(logits, C.c_float), T, E, k,
                                     _ptr(idx, C.c_int), _ptr(w, C.c_float))
        return idx, w

    def moe_layer(self, layer: dict, t_bits: np.ndarray, top_k: int = 4,
                  limit: float = 7.0, shard: tuple[int, int] | None = None,
                  add_b2: bool = True):
        p = _prep(layer)
        t = np.ascontiguousarray(_bf16_to_f32(t_bits))
        T, H = t.shape
        E, D = layer["E"], layer["D"]
        d0, d1 = shard if shard is not None else (0, D)
        logits = np.empty((T, E), dtype=np.float32)
        idx = np.empty((T, top_k), dtype=np.int32)
        w = np.empty((T, top_k), dtype=np.float32)
        out = np.empty((T, H), dtype=np.float32)
        rc = self.lib.oracle_moe_layer_shard(
            _ptr(t, C.c_float), T, H, D, E, top_k, C.c_float(limit),
            _ptr(p["w1_codes"], C.c_uint8), _ptr(p["w1_scales"], C.c_uint8), _ptr(p["b1"], C.c_float),
            _ptr(p["w2_codes"], C.c_uint8), _ptr(p["w2_scales"], C.c_uint8), _ptr(p["b2"], C.c_float),
            _ptr(p["router_w"], C.c_float), _ptr(p["router_b"], C.c_float),
            d0, d1, int(add_b2),
            _ptr(logits, C.c_float), _ptr(idx, C.c_int), _ptr(w, C.c_float), _ptr(out, C.c_float))
        if rc != 0:
            raise RuntimeError(f"oracle_moe_layer_shard failed: {rc}")
        return logits, idx, w, out


    def moe_block(self, layer: dict, x: np.ndarray, gain: np.ndarray, top_k: int = 4, limit: float = 7.0,
                  t_as_bf16: bool = False):
        """x [T,H] and gain [H] as float32 values.  Returns t, logits, idx, w, e_agg, x_out."""
        p = _prep(layer)
        x = np.ascontiguousarray(x, dtype=np.float32)
        gain = np.ascontiguousarray(gain, dtype=np.float32)
        T, H = x.shape
        E, D = layer["E"], layer["D"]
        t = np.empty((T, H), dtype=np.float32)
        logits = np.empty((T, E), dtype=np.float32)
        idx = np.empty((T, top_k), dtype=np.int32)
        w = np.empty((T, top_k), dtype=np.float32)
        agg = np.empty((T, H), dtype=np.float32)
        xo = np.empty((T, H), dtype=np.float32)
        self.lib.oracle_moe_block.restype = C.c_int
        rc = self.lib.oracle_moe_block(
            _ptr(x, C.c_float), _ptr(gain, C.c_float), T, H, D, E, top_k, C.c_float(limit),
            _ptr(p["w1_codes"], C.c_uint8), _ptr(p["w1_scales"], C.c_uint8), _ptr(p["b1"], C.c_float),
            _ptr(p["w2_codes"], C.c_uint8), _ptr(p["w2_scales"], C.c_uint8), _ptr(p["b2"], C.c_float),
            _ptr(p["router_w"], C.c_float), _ptr(p["router_b"], C.c_float), int(t_as_bf16),
            _ptr(t, C.c_float), _ptr(logits, C.c_float), _ptr(idx, C.c_int), _ptr(w, C.c_float),
            _ptr(agg, C.c_float), _ptr(xo, C.c_float))
        if rc != 0:
            raise RuntimeError(f"oracle_moe_block failed: {rc}")
        return t, logits, idx, w, agg, xo


def host_cores() -> int:
    """Physical cores this process may run on (what the timed CPU baseline uses)."""
    try:
        import psutil
        n = psutil.cpu_count(logical=False) or 0
    except Exception:
        n = 0
    allowed = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    return max(1, min(n, allowed) if n else allowed)


def reference_available() -> bool:
    return os.path.exists(REF_SO)


def reference_quantizer_available() -> bool:
    return os.path.exists(REF_MXFP4_SO)


class ReferenceQuantizer:
    """The reference's own MXFP4 quantiser and decoder (getp-csrc/memory/mxfp4.hpp:41-57, :113-217),
    its kernel body run on 32 host threads."""

    def __init__(self):
        if not os.path.exists(REF_MXFP4_SO):
            build()
        if not os.path.exists(REF_MXFP4_SO):
            raise FileNotFoundError(REF_MXFP4_SO)
        self.lib = C.CDLL(REF_MXFP4_SO)
        self.lib.ref_mxfp4_quantize.restype = C.c_int
        self.lib.ref_mxfp4_dequantize.restype = None

    def quantize(self, values: np.ndarray):
        v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        nblk = (v.size + 31) // 32
        codes = np.empty(nblk * 16, dtype=np.uint8)
        scales = np.empty(nblk, dtype=np.uint8)
        rc = self.lib.ref_mxfp4_quantize(_ptr(v, C.c_float), C.c_size_t(v.size), _ptr(codes, C.c_uint8),
                                         _ptr(scales, C.c_uint8))
        if rc != 0:
            raise RuntimeError(f"ref_mxfp4_quantize failed: {rc}")
        return codes, scales

    def dequantize(self, codes: np.ndarray, scales: np.ndarray, n: int) -> np.ndarray:
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        scales = np.ascontiguousarray(scales, dtype=np.uint8)
        out = np.empty(n, dtype=np.float32)
        self.lib.ref_mxfp4_dequantize(_ptr(codes, C.c_uint8), _ptr(scales, C.c_uint8), C.c_size_t(n),
                                      _ptr(out, C.c_float))
        return out


class Reference:
    """The reference's own forward() (run.cpp:528-756) on a one-layer model."""

    def __init__(self, layer: dict, top_k: int = 4, limit: float = 7.0):
        if not os.path.exists(REF_SO):
            build()
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        self.lib = C.CDLL(REF_SO)
        self.lib.ref_moe_create.restype = C.c_void_p
        self.lib.ref_moe_forward.restype = C.c_long
        self.lib.ref_moe_prepare.restype = C.c_int
        self.lib.ref_moe_num_threads.restype = C.c_int
        self.layer = layer
        self.k = top_k
        self.p = _prep(layer)  # keeps the borrowed arrays alive
        p = self.p
        self.h = C.c_void_p(self.lib.ref_moe_create(
            layer["H"], layer["D"], layer["E"], top_k, C.c_float(limit),
            _ptr(p["w1_codes"], C.c_uint8), _ptr(p["w1_scales"], C.c_uint8), _ptr(p["b1"], C.c_float),
            _ptr(p["w2_codes"], C.c_uint8), _ptr(p["w2_scales"], C.c_uint8), _ptr(p["b2"], C.c_float),
            _ptr(p["router_w"], C.c_float), _ptr(p["router_b"], C.c_float)))
        if not self.h:
            raise MemoryError("ref_moe_create failed")

    def threads(self) -> int:
        return int(self.lib.ref_moe_num_threads())

    def set_threads(self, n: int) -> None:
        self.lib.ref_moe_set_num_threads(int(n))

    def prepare(self, t_bits: np.ndarray) -> int:
        """Dequantise the experts these rows will use (load-time work in the
        reference); returns how many experts are now resident."""
        t = np.ascontiguousarray(_bf16_to_f32(t_bits))
        return int(self.lib.ref_moe_prepare(self.h, _ptr(t, C.c_float), t.shape[0]))

    def forward(self, t_bits: np.ndarray):
        t = np.ascontiguousarray(_bf16_to_f32(t_bits))
        T, H = t.shape
        E = self.layer["E"]
        logits = np.empty((T, E), dtype=np.float32)
        idx = np.empty((T, self.k), dtype=np.int32)
        w = np.empty((T, self.k), dtype=np.float32)
        out = np.empty((T, H), dtype=np.float32)
        bad = self.lib.ref_moe_forward(self.h, _ptr(t, C.c_float), T, _ptr(logits, C.c_float),
                                       _ptr(idx, C.c_int), _ptr(w, C.c_float), _ptr(out, C.c_float))
        if bad != 0:
            raise RuntimeError(f"reference RMSNorm did not reproduce the injected rows "
                               f"({bad} elements differ)")
        return logits, idx, w, out

    def forward_block(self, x: np.ndarray, gain: np.ndarray):
        """forward() with its own RMSNorm: x [T,H], gain [H] float32.  Returns t, logits, idx, w, e_agg."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        gain = np.ascontiguousarray(gain, dtype=np.float32)
        T, H = x.shape
        E = self.layer["E"]
        t = np.empty((T, H), dtype=np.float32)
        logits = np.empty((T, E), dtype=np.float32)
        idx = np.empty((T, self.k), dtype=np.int32)
        w = np.empty((T, self.k), dtype=np.float32)
        agg = np.empty((T, H), dtype=np.float32)
        self.lib.ref_moe_forward_block.restype = None
        self.lib.ref_moe_forward_block(self.h, _ptr(x, C.c_float), _ptr(gain, C.c_float), T, _ptr(t, C.c_float),
                                       _ptr(logits, C.c_float), _ptr(idx, C.c_int), _ptr(w, C.c_float),
                                       _ptr(agg, C.c_float))
        return t, logits, idx, w, agg

    def close(self):
        if self.h:
            self.lib.ref_moe_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
