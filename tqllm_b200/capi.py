"""ctypes binding of libb2moe.so (the C ABI declared in include/b2moe.h).

The library is built in-tree by `python -m tqllm_b200.build`. There is no fallback: when the shared library is missing
or fails to load, importing this module raises, and every compute call returns a status that `check` turns into an
exception. Device pointers are passed as integers (`tensor.data_ptr()`).
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb2moe.so")

OK, ERR_SHAPE, ERR_ALIGN, ERR_FORMAT, ERR_NULL, ERR_WORKSPACE, ERR_CUDA, ERR_CAPACITY = range(8)
F32, F16, BF16 = 0, 1, 2
Q4_K, IQ4_NL, IQ3_S, IQ4_XS, NVFP4G = 12, 20, 21, 23, 323
IQ3_S_X4 = 0x1015        # bank layout of IQ3_S blocks as 4-bit codes (b2moe_type)
FAMILY = {"auto": 0, "generic": 1, "decode": 2, "gemm": 3}
SOFTMAX, SIGMOID = 1, 2


class B2moeError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {status_string(status)} (status {status})")


class Bank(C.Structure):
    _fields_ = [("data", C.c_void_p), ("aux", C.c_void_p), ("type", C.c_uint32), ("experts", C.c_int32),
                ("rows", C.c_int32), ("cols", C.c_int32)]


class PlanView(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("counts", "offsets", "active", "perm", "passes", "total")]


class Layer(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("experts", C.c_int32), ("topk", C.c_int32), ("ff", C.c_int32),
                ("gating", C.c_int32), ("norm", C.c_int32), ("scale", C.c_float), ("has_shared", C.c_int32),
                ("router_w", C.c_void_p), ("sel_bias", C.c_void_p), ("shared_gate_vec", C.c_void_p),
                ("gate", Bank), ("up", Bank), ("down", Bank), ("sh_gate", Bank), ("sh_up", Bank), ("sh_down", Bank)]


class LayerWs(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in ("logits", "ids", "weights", "shared_weights", "plan", "act", "y", "scratch", "expert_scratch", "total")]


# name -> (restype, argtypes): every symbol include/b2moe.h declares
_vp, _i32, _i64, _u32, _f32, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_float, C.c_size_t
SIGNATURES = {
    "b2moe_status_string": (C.c_char_p, [_i32]),
    "b2moe_abi_version": (_i32, []),
    "b2moe_codebooks": (None, [_vp, _vp]),
    "b2moe_raw_bytes": (_sz, [_u32, _i32, _i32]),
    "b2moe_bank_bytes": (_sz, [_u32, _i32, _i32]),
    "b2moe_bank_aux_bytes": (_sz, [_u32, _i32, _i32]),
    "b2moe_bank_load": (_i32, [_u32, _vp, _i32, _i32, _i32, _vp, _vp, _vp]),
    "b2moe_dequant_dump": (_i32, [C.POINTER(Bank), _vp, _vp]),
    "b2moe_router": (_i32, [_vp, _vp, _vp, _i32, _vp, _i32, _i32, _i32, _i32, _vp]),
    "b2moe_topk_softmax": (_i32, [_vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _f32, _vp]),
    "b2moe_topk_softmax2": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _vp]),
    "b2moe_route_sigmoid": (_i32, [_vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _f32, _i32, _vp]),
    "b2moe_plan_ints": (_i64, [_i32, _i32, _i32]),
    "b2moe_plan_view_of": (None, [_i32, _i32, _i32, C.POINTER(PlanView)]),
    "b2moe_dispatch_workspace_bytes": (_sz, [_i32, _i32]),
    "b2moe_dispatch": (_i32, [_vp, _i32, _i32, _i32, _i32, _vp, _vp, _sz, _vp]),
    "b2moe_dispatch_range": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _sz, _vp]),
    "b2moe_ep_local_ids": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp]),
    "b2moe_ep_reduce": (_i32, [_vp, _i32, _vp, _vp, _i32, _i32, _vp, _i32, _vp]),
    "b2moe_ep_peer_lists": (_i32, [_vp, _i32, _i32, _vp, _i32, _i32, _vp, _vp, _vp, _vp]),
    "b2moe_ep_pack": (_i32, [_vp, _i32, _vp, _vp, _i32, _i32, _vp, _vp, _i32, _i32, _vp, _vp]),
    "b2moe_ep_unpack": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "b2moe_ep_return_reduce": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp, _i32, _i32, _vp, _i32, _vp]),
    "b2moe_peer_alloc": (_i32, [_sz, C.POINTER(_vp), _vp]),
    "b2moe_peer_open": (_i32, [_vp, C.POINTER(_vp)]),
    "b2moe_peer_close": (_i32, [_vp]),
    "b2moe_peer_free": (_i32, [_vp]),
    "b2moe_peer_put": (_i32, [_vp, _sz, _sz, _vp, _vp, _vp, _i32, _i32, _vp]),
    "b2moe_peer_wait": (_i32, [_vp, _i32, _i32, _vp, _vp]),
    "b2moe_route_dispatch": (_i32, [_i32, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _f32, _i32, _i32, _i32, _vp, _vp, _sz, _vp]),
    "b2moe_plan_to_groups": (_i32, [_vp, _i32, _i32, _i32, _vp, _vp, _vp]),
    "b2moe_expert_workspace_bytes": (_sz, [_u32, _i32, _i32, _i32]),
    "b2moe_expert_gateup_swiglu": (_i32, [C.POINTER(Bank)] * 4 + [_vp, _i32, _vp, _i32, _i32, _i32, _vp, _vp, _sz, _vp]),
    "b2moe_expert_down": (_i32, [C.POINTER(Bank)] * 2 + [_vp, _vp, _i32, _i32, _i32, _vp, _vp, _sz, _vp]),
    "b2moe_expert_down_sparse": (_i32, [C.POINTER(Bank)] * 2 + [_vp, _vp, _i32, _i32, _i32, _i64, _vp, _vp, _sz, _vp]),
    "b2moe_expert_gateup_swiglu_sparse": (_i32, [C.POINTER(Bank)] * 4 + [_vp, _i32, _vp, _i32, _i32, _i32, _i64, _vp, _vp, _sz, _vp]),
    "b2moe_expert_matvec_workspace_bytes": (_sz, [C.POINTER(Bank), _i32, _i32]),
    "b2moe_expert_gemm_gateup_workspace_bytes": (_sz, [C.POINTER(Bank), _i32, _i32, _i32]),
    "b2moe_plan_from_groups": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "b2moe_expert_matvec": (_i32, [C.POINTER(Bank), _vp, _i32, _vp, _i32, _vp, _i32, _i32, _i32, _vp, _sz, _vp]),
    "b2moe_expert_gemm": (_i32, [C.POINTER(Bank), _vp, _i32, _vp, _i32, _vp, _vp, _i32, _i32, _i32, _vp, _sz, _vp]),
    "b2moe_expert_gemm_gateup": (_i32, [C.POINTER(Bank)] * 2 + [_vp, _i32, _vp, _i32, _vp, _vp, _i32, _i32, _vp, _sz, _vp]),
    "b2moe_bank_pack_host": (_i32, [_u32, _vp, _i32, _i32, _i32, _vp, _vp]),
    "b2moe_sum_rows": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "b2moe_swiglu": (_i32, [_vp, _vp, _i32, _vp, _i32, _i64, _vp]),
    "b2moe_dequant_dump_as": (_i32, [C.POINTER(Bank), _vp, _i32, _vp, _sz, _vp]),
    "b2moe_static_scratch_bytes": (_sz, []),
    "b2moe_expert_down_static": (_i32, [C.POINTER(Bank)] * 2 + [_vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "b2moe_combine": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _i32, _vp]),
    "b2moe_combine_residual": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _i32, _vp]),
    "b2moe_gguf_open": (_i32, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "b2moe_gguf_close": (None, [_vp]),
    "b2moe_gguf_tensor_count": (_i32, [_vp]),
    "b2moe_gguf_tensor_name": (_i32, [_vp, _i32, C.c_char_p, _i32]),
    "b2moe_gguf_tensor": (_i32, [_vp, C.c_char_p, C.POINTER(C.c_uint32), C.POINTER(C.c_int64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "b2moe_gguf_expert_slice": (_i32, [_vp, C.c_char_p, _i32, _i32, C.POINTER(C.c_uint32), C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                       C.POINTER(C.c_void_p), C.POINTER(C.c_uint64)]),
    "b2moe_gguf_expert_bank": (_i32, [_vp, C.c_char_p, _i32, _i32, C.c_uint32, _vp, _vp]),
    "b2moe_count": (_i32, [_vp, _vp, _i32, _i32, _vp]),
    "b2moe_place_experts": (_i32, [_vp, _i32, _i32, _vp, _vp]),
    "b2moe_harness_select": (None, [_i32, _i32]),
    "b2moe_harness_wait_probe": (None, [_i32, _u32]),
    "b2moe_harness_skip_staging": (None, [_i32]),
    "b2moe_harness_overlap": (None, [_i32]),
    "b2moe_harness_ring": (None, [_i32, _i32, _i32]),
    "b2moe_harness_column_split": (None, [_i32]),
    "b2moe_harness_launches": (C.c_uint64, []),
    "b2moe_layer_workspace": (_i32, [C.POINTER(Layer), _i32, C.POINTER(LayerWs)]),
    "b2moe_layer_forward": (_i32, [C.POINTER(Layer), _vp, _i32, _i32, _vp, _i32, _vp, _sz, _vp]),
    "b2moe_layer_forward_residual": (_i32, [C.POINTER(Layer), _vp, _i32, _i32, _vp, _vp, _i32, _vp, _sz, _vp]),
}

if not os.path.isfile(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is missing: build it with `python -m tqllm_b200.build` (there is no fallback path)")
lib = C.CDLL(LIB_PATH)
for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here = the library does not export a declared symbol
    _fn.restype, _fn.argtypes = _res, _args


def status_string(status: int) -> str:
    return lib.b2moe_status_string(status).decode()


def check(status: int, where: str) -> None:
    if status != OK:
        raise B2moeError(status, where)


def codebooks():
    grid = (C.c_uint32 * 512)()
    kv = (C.c_int8 * 16)()
    lib.b2moe_codebooks(grid, kv)
    return list(grid), list(kv)


class family:
    """Every expert product inside the block takes the named kernel family ("generic", "decode", "gemm") where it supports
    the shape; `item_tokens` = 256 selects the wide work items of the grouped GEMM. Harness hook: process-wide."""

    def __init__(self, name: str, item_tokens: int = 0):
        self.name, self.item_tokens = name, item_tokens

    def __enter__(self):
        lib.b2moe_harness_select(FAMILY[self.name], self.item_tokens)
        return self

    def __exit__(self, *a):
        lib.b2moe_harness_select(0, 0)
