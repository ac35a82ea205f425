"""ctypes bindings of the CPU checker (oracle/oracle.cpp) and, when built, of the reference's own CPU sources
(oracle/_ref/libtqref.so). TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and bench.py's CPU baseline;
the shipped package never imports this module.

All arrays are numpy, C-contiguous. GGUF type ids: Q4_K 12, IQ4_NL 20, IQ3_S 21, IQ4_XS 23, NVFP4G 323.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

Q4_K, IQ4_NL, IQ3_S, IQ4_XS, NVFP4G = 12, 20, 21, 23, 323
SOFTMAX, SIGMOID, SOFTMAX_WEIGHT, SQRT_SOFTPLUS = 1, 2, 3, 4

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C")


def _opt(a, dtype):
    if a is None:
        return None
    a = np.ascontiguousarray(a, dtype=dtype)
    return a.ctypes.data_as(C.c_void_p), a


def _vp(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class _Lib:
    def __init__(self, path: str, prefix: str):
        self.path, self.p = path, prefix
        self.lib = C.CDLL(path)
        L, p = self.lib, prefix
        getattr(L, p + "half_to_float").restype = C.c_float
        getattr(L, p + "half_to_float").argtypes = [C.c_uint16]
        getattr(L, p + "e4m3_to_float").restype = C.c_float
        getattr(L, p + "e4m3_to_float").argtypes = [C.c_uint8]
        getattr(L, p + "dequant").argtypes = [C.c_uint32, C.c_void_p, _f32p, C.c_int64]
        getattr(L, p + "route").argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, _f32p, C.c_void_p, _i32p, _f32p]
        getattr(L, p + "expert_ffn").argtypes = [_f32p, C.c_int, _f32p, _f32p, _f32p, C.c_int, C.c_float, C.c_int, _f32p]
        getattr(L, p + "expert_ffn").restype = None

    def half_to_float(self, h: int) -> float:
        return getattr(self.lib, self.p + "half_to_float")(h)

    def e4m3_to_float(self, b: int) -> float:
        return getattr(self.lib, self.p + "e4m3_to_float")(b)

    def dequant(self, type_id: int, raw: np.ndarray, n: int) -> np.ndarray:
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        out = np.empty(n, np.float32)
        rc = getattr(self.lib, self.p + "dequant")(type_id, raw.ctypes.data_as(C.c_void_p), out, n)
        if rc:
            raise ValueError(f"dequant: unsupported type {type_id} or bad length {n}")
        return out

    def route(self, gating, logits, k, norm=True, scale=0.0, sel_bias=None):
        """logits [tokens][experts] -> (ids [tokens][k] int32, weights [tokens][k] f32)."""
        logits = np.ascontiguousarray(logits, np.float32)
        if logits.ndim == 1:
            logits = logits[None]
        t, e = logits.shape
        ids = np.empty((t, k), np.int32)
        w = np.empty((t, k), np.float32)
        b = None if sel_bias is None else np.ascontiguousarray(sel_bias, np.float32)
        fn = getattr(self.lib, self.p + "route")
        for i in range(t):
            if fn(gating, e, k, int(bool(norm)), float(scale), logits[i], _vp(b), ids[i], w[i]):
                raise ValueError("route: bad shape or gating")
        return ids, w

    def expert_ffn(self, x, wg, wu, wd, clamp=0.0, clamp_gate=False):
        x = np.ascontiguousarray(x, np.float32)
        wg, wu, wd = (np.ascontiguousarray(a, np.float32) for a in (wg, wu, wd))
        ff, hidden = wg.shape
        out = np.empty(hidden, np.float32)
        getattr(self.lib, self.p + "expert_ffn")(x, hidden, wg, wu, wd, ff, clamp, int(clamp_gate), out)
        return out


class Oracle(_Lib):
    def __init__(self):
        super().__init__(_build.build_oracle(), "orc_")
        L = self.lib
        L.orc_block_elems.argtypes = [C.c_uint32]
        L.orc_block_bytes.argtypes = [C.c_uint32]
        L.orc_router_logits.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int, _f32p, C.c_int]
        L.orc_router_logits.restype = None
        L.orc_router_logits_f64.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int, _f64p, C.c_int]
        L.orc_router_logits_f64.restype = None
        L.orc_dispatch.argtypes = [_i32p, C.c_int, C.c_int, _i32p, _i32p, _i32p]
        L.orc_dispatch.restype = None
        L.orc_combine.argtypes = [_f32p, C.c_int, _f32p, C.c_int, _f32p]
        L.orc_combine.restype = None
        L.orc_moe_layer.argtypes = [C.c_int] * 7 + [C.c_float] + [C.c_void_p] * 3 + \
            [C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p] + \
            [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_void_p, C.c_int, C.c_void_p] + \
            [_i32p, _f32p, _i32p, _i32p, _i32p, _f32p, C.c_int]

    def block_elems(self, t): return self.lib.orc_block_elems(t)
    def block_bytes(self, t): return self.lib.orc_block_bytes(t)

    def router_logits(self, w, x, f64=False):
        w, x = np.ascontiguousarray(w, np.float32), np.ascontiguousarray(x, np.float32)
        e, h = w.shape
        t = x.shape[0]
        out = np.empty((t, e), np.float64 if f64 else np.float32)
        (self.lib.orc_router_logits_f64 if f64 else self.lib.orc_router_logits)(w, x, h, e, t, out, e)
        return out

    def dispatch(self, ids, experts):
        ids = np.ascontiguousarray(ids, np.int32).reshape(-1)
        counts = np.empty(experts, np.int32)
        offsets = np.empty(experts + 1, np.int32)
        perm = np.full(ids.size, -1, np.int32)
        self.lib.orc_dispatch(ids, ids.size, experts, counts, offsets, perm)
        return counts, offsets, perm

    def combine(self, weights, expert_outs, out):
        weights = np.ascontiguousarray(weights, np.float32)
        expert_outs = np.ascontiguousarray(expert_outs, np.float32)
        self.lib.orc_combine(weights, weights.size, expert_outs, out.size, out)
        return out

    def moe_layer(self, *, x, router_w, topk, ff, gating, norm, scale, types, gate, up, down, experts,
                  sel_bias=None, shared=None, shared_gate_vec=None, logits_in=None, threads=0):
        """Whole layer on the CPU. gate/up/down: raw GGUF block bytes (uint8 arrays) of the stacked experts;
        shared: optional (gate, up, down) raw bytes of one always-on expert; types: (gate, up, down) GGUF ids.
        Returns dict(logits, ids, weights, counts, offsets, perm, out)."""
        x = np.ascontiguousarray(x, np.float32)
        t, h = x.shape
        keep = []

        def opt(a, dt):
            if a is None:
                return None
            a = np.ascontiguousarray(a, dt)
            keep.append(a)
            return a.ctypes.data_as(C.c_void_p)

        logits_out = np.empty((t, experts), np.float32)
        ids = np.empty((t, topk), np.int32)
        w = np.empty((t, topk), np.float32)
        counts = np.empty(experts, np.int32)
        offsets = np.empty(experts + 1, np.int32)
        perm = np.full(t * topk, -1, np.int32)
        out = np.empty((t, h), np.float32)
        ld = 0
        if logits_in is not None:
            logits_in = np.ascontiguousarray(logits_in, np.float32)
            ld = logits_in.shape[1]
        sh = shared or (None, None, None)
        rc = self.lib.orc_moe_layer(
            t, h, experts, topk, ff, gating, int(bool(norm)), float(scale),
            opt(router_w, np.float32), opt(sel_bias, np.float32), opt(x, np.float32),
            types[0], opt(gate, np.uint8), types[1], opt(up, np.uint8), types[2], opt(down, np.uint8),
            int(shared is not None), opt(sh[0], np.uint8), opt(sh[1], np.uint8), opt(sh[2], np.uint8),
            opt(shared_gate_vec, np.float32), opt(logits_in, np.float32), ld, logits_out.ctypes.data_as(C.c_void_p),
            ids, w, counts, offsets, perm, out, threads or (os.cpu_count() or 1))
        if rc:
            raise ValueError("moe_layer: bad argument")
        return dict(logits=logits_out, ids=ids, weights=w, counts=counts, offsets=offsets, perm=perm, out=out)


class Reference(_Lib):
    """The reference's CPU sources compiled in place; available only where oracle/_ref/libtqref.so was built."""

    def __init__(self, path: str):
        super().__init__(path, "ref_")
        self.lib.ref_moe_layer.argtypes = [C.c_int] * 7 + [C.c_float] + [C.c_void_p] * 2 + \
            [C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p] + \
            [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_void_p, C.c_int] + \
            [_i32p, _f32p, _f32p, C.c_int]

    def moe_layer(self, *, x, topk, ff, gating, norm, scale, types, gate, up, down, experts, logits_in,
                  sel_bias=None, shared=None, shared_gate_vec=None, threads=0):
        x = np.ascontiguousarray(x, np.float32)
        t, h = x.shape
        keep = []

        def opt(a, dt):
            if a is None:
                return None
            a = np.ascontiguousarray(a, dt)
            keep.append(a)
            return a.ctypes.data_as(C.c_void_p)

        logits_in = np.ascontiguousarray(logits_in, np.float32)
        ids = np.empty((t, topk), np.int32)
        w = np.empty((t, topk), np.float32)
        out = np.empty((t, h), np.float32)
        sh = shared or (None, None, None)
        rc = self.lib.ref_moe_layer(
            t, h, experts, topk, ff, gating, int(bool(norm)), float(scale), opt(sel_bias, np.float32), opt(x, np.float32),
            types[0], opt(gate, np.uint8), types[1], opt(up, np.uint8), types[2], opt(down, np.uint8),
            int(shared is not None), opt(sh[0], np.uint8), opt(sh[1], np.uint8), opt(sh[2], np.uint8),
            opt(shared_gate_vec, np.float32), opt(logits_in, np.float32), logits_in.shape[1], ids, w, out,
            threads or (os.cpu_count() or 1))
        if rc:
            raise ValueError("ref_moe_layer: bad argument")
        return dict(ids=ids, weights=w, out=out)


_oracle = None
_reference = None


def oracle() -> Oracle:
    global _oracle
    if _oracle is None:
        _oracle = Oracle()
    return _oracle


def reference() -> Reference | None:
    """The compiled reference, or None when it cannot be had (no checkout here and no prebuilt library)."""
    global _reference
    if _reference is None:
        path = _build.build_ref()
        if path is None:
            return None
        _reference = Reference(path)
    return _reference


class ReferencePool:
    """The reference's production CPU expert pool (CpuMissPool) compiled in place: oracle/_ref/libtqrefpool.so. It is what
    bench.py times as the CPU arm; its numerics are the reference's int8 / bf16 ones, so it is not a parity checker."""

    def __init__(self, path: str):
        self.lib = C.CDLL(path)
        self.lib.refpool_create.argtypes = [C.c_int] * 3
        self.lib.refpool_layer.argtypes = [C.c_int] * 5 + [_f32p, _i32p, _f32p, C.c_void_p] + [C.c_void_p] * 3 + [C.c_int] + [C.c_void_p] * 3 + [_f32p]
        self.threads = 0

    def create(self, threads: int, hidden: int, ff: int):
        """threads workers pinned to CPUs 1 .. threads; the calling thread is pinned to CPU 0 (the pool's own policy)"""
        rc = self.lib.refpool_create(threads, hidden, ff)
        if rc:
            raise ValueError(f"refpool_create failed ({rc}): one pool shape per process")
        self.threads = threads

    def layer(self, *, x, ids, weights, ff, types, gate, up, down, experts, shared=None):
        x = np.ascontiguousarray(x, np.float32)
        ids = np.ascontiguousarray(ids, np.int32)
        weights = np.ascontiguousarray(weights, np.float32)
        t, h = x.shape
        keep = [np.ascontiguousarray(a, np.uint8) for a in (gate, up, down)]
        sh = [np.ascontiguousarray(a, np.uint8) for a in shared] if shared is not None else [None] * 3
        ty = (C.c_uint32 * 3)(*types)
        out = np.empty((t, h), np.float32)
        rc = self.lib.refpool_layer(t, h, experts, ids.shape[1], ff, x, ids, weights, C.cast(ty, C.c_void_p),
                                    *[_vp(a) for a in keep], int(shared is not None), *[_vp(a) for a in sh], out)
        if rc:
            raise ValueError(f"refpool_layer failed ({rc})")
        return out


_pool = None


def reference_pool() -> ReferencePool | None:
    """The compiled production CPU pool of the reference, or None when it cannot be had (no checkout here and no prebuilt
    library, or not an x86 host)."""
    global _pool
    if _pool is None:
        path = _build.build_ref_pool()
        if path is None:
            return None
        _pool = ReferencePool(path)
    return _pool
