"""The C ABI without a GPU: the shared library loads, exports every symbol include/b2moe.h declares, its host
arithmetic (sizes, plan layout, status strings) is right, and bad arguments are rejected before any launch."""
import ctypes as C
import os
import re

import pytest

from tqllm_b200 import capi, gen_tables, synth
from tqllm_b200.capi import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b2moe.h")).read()
    return re.findall(r"^B2MOE_API [\w \*]+?\b(b2moe_\w+)\(", text, flags=re.M)


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/b2moe.h but not exported"
        assert n in capi.SIGNATURES, f"{n} has no ctypes signature"
    assert set(capi.SIGNATURES) == set(names)
    assert lib.b2moe_abi_version() == 1


def test_status_strings():
    assert capi.status_string(0) == "ok"
    assert len({capi.status_string(i) for i in range(8)}) == 8
    assert capi.status_string(99) == "unknown status"


def test_sizes():
    for t, (elems, nbytes) in synth.BLOCK.items():
        assert lib.b2moe_raw_bytes(t, 32, 1024) == 32 * (1024 // elems) * nbytes
        moved = 32 * (1024 // 128) * 4 if t == 323 else 0          # NVFP4G: the tensor scale moves to the aux array
        assert lib.b2moe_bank_bytes(t, 32, 1024) == lib.b2moe_raw_bytes(t, 32, 1024) - moved     # no padding
        assert lib.b2moe_bank_bytes(t, 19, 1024) == lib.b2moe_raw_bytes(t, 32, 1024) - moved     # rows pad to 16
        assert lib.b2moe_raw_bytes(t, 32, 1000) == 0
    assert lib.b2moe_raw_bytes(7, 32, 1024) == 0 and lib.b2moe_bank_bytes(7, 32, 1024) == 0
    assert lib.b2moe_bank_aux_bytes(323, 19, 256) == 32 * 4 and lib.b2moe_bank_aux_bytes(12, 19, 256) == 0
    assert lib.b2moe_raw_bytes(23, 64, 1408) == 0 and lib.b2moe_raw_bytes(20, 64, 1408) == 64 * 44 * 18


def test_plan_layout():
    v = capi.PlanView()
    lib.b2moe_plan_view_of(8, 20, 5, C.byref(v))
    assert (v.counts, v.offsets, v.active, v.perm, v.passes, v.total) == (4, 13, 23, 32, 57, 67)
    assert lib.b2moe_plan_ints(8, 20, 5) == 67 and lib.b2moe_plan_ints(0, 20, 5) == 0


def test_codebooks_match_the_table_source():
    grid, kv = capi.codebooks()
    g2, k2 = gen_tables.tables()
    assert grid == g2 and kv == k2


def test_layer_workspace_is_host_arithmetic():
    L = capi.Layer()
    L.hidden, L.experts, L.topk, L.ff, L.has_shared = 2048, 512, 10, 512, 1
    ws = capi.LayerWs()
    assert lib.b2moe_layer_workspace(C.byref(L), 64, C.byref(ws)) == 0
    assert ws.act - ws.plan >= lib.b2moe_plan_ints(512, 640, 64) * 4
    assert ws.total >= ws.y + 704 * 2048 * 4 and ws.logits == 0 and all(getattr(ws, f) % 256 == 0 for f, _ in ws._fields_)
    L.topk = 0
    assert lib.b2moe_layer_workspace(C.byref(L), 64, C.byref(ws)) == capi.ERR_SHAPE


def test_arguments_are_rejected_before_any_launch():
    """null / misaligned / bad-shape arguments return their status codes on a box with no GPU at all"""
    assert lib.b2moe_router(None, None, None, capi.BF16, None, 9, 64, 8, 1, None) == capi.ERR_NULL
    assert lib.b2moe_router(16, None, 16, capi.BF16, 16, 9, 60, 8, 1, None) == capi.ERR_SHAPE
    assert lib.b2moe_router(16, None, 17, capi.BF16, 16, 9, 64, 8, 1, None) == capi.ERR_ALIGN
    assert lib.b2moe_topk_softmax(16, 9, 16, 16, None, 8, 9, 1, 0.0, None) == capi.ERR_SHAPE
    assert lib.b2moe_topk_softmax(16, 9, 16, 16, None, 5000, 2, 1, 0.0, None) == capi.ERR_SHAPE
    assert lib.b2moe_route_sigmoid(None, 8, None, 16, 16, 8, 2, 1, 0.0, 1, None) == capi.ERR_NULL
    assert lib.b2moe_dispatch(None, 4, 2, 8, 0, 16, None, 0, None) == capi.ERR_NULL
    assert lib.b2moe_dispatch(16, 4, 2, 8, 3, 16, None, 0, None) == capi.ERR_SHAPE
    assert lib.b2moe_bank_load(99, 16, 1, 16, 256, 16, None, None) == capi.ERR_FORMAT
    assert lib.b2moe_bank_load(12, 16, 1, 16, 100, 16, None, None) == capi.ERR_SHAPE
    assert lib.b2moe_bank_load(323, 16, 1, 16, 256, 16, None, None) == capi.ERR_NULL      # NVFP4G needs aux
    bank = capi.Bank(16, None, 12, 4, 32, 256)
    bad = capi.Bank(8, None, 12, 4, 32, 256)
    assert lib.b2moe_dequant_dump(C.byref(bank), None, None) == capi.ERR_NULL
    assert lib.b2moe_dequant_dump(C.byref(bad), 16, None) == capi.ERR_ALIGN
    up_other = capi.Bank(16, None, 21, 4, 32, 256)
    assert lib.b2moe_expert_gateup_swiglu(C.byref(bank), C.byref(up_other), None, None, 16, capi.BF16, 16, 2, 2, 0, 16, None, 0, None) == capi.ERR_FORMAT
    iq = capi.Bank(16, None, 21, 4, 32, 256)
    assert lib.b2moe_expert_workspace_bytes(21, 64, 2048, capi.F32) >= 64 * 2048 * 2 + 64 * 4   # one scaled fp16 term per value + 2^-e per row
    # every format: at least the scaled fp16 copy of the rows + one float per row that the tensor-core GEMM takes
    for t in (12, 20, 21, 23, 323):
        assert lib.b2moe_expert_workspace_bytes(t, 64, 16384, capi.F32) >= 64 * 16384 * 2 + 64 * 4
    assert lib.b2moe_expert_workspace_bytes(12, 0, 2048, capi.BF16) == 0
    assert lib.b2moe_expert_down(C.byref(iq), None, 16, 16, 2, 2, 0, 16, None, 0, None) == capi.ERR_NULL        # needs scratch
    assert lib.b2moe_expert_down(C.byref(iq), None, 16, 16, 2, 2, 0, 16, 32, 64, None) == capi.ERR_WORKSPACE
    assert lib.b2moe_combine(16, None, 16, None, 2, 2, 30, 0, 16, capi.F32, None) == capi.ERR_SHAPE
    # the peer-memory exchange: pointer, size and alignment checks come before any CUDA call
    assert lib.b2moe_peer_put(None, 0, 64, 16, 16, 16, 2, 1, None) == capi.ERR_NULL
    assert lib.b2moe_peer_put(16, 0, 60, 16, 16, 16, 2, 1, None) == capi.ERR_SHAPE         # bytes: a multiple of 16
    assert lib.b2moe_peer_put(16, 8, 64, 16, 16, 16, 2, 1, None) == capi.ERR_SHAPE         # stride: a multiple of 16
    assert lib.b2moe_peer_put(24, 0, 64, 16, 16, 16, 2, 1, None) == capi.ERR_ALIGN
    assert lib.b2moe_peer_put(16, 0, 64, 16, 16, 16, 0, 1, None) == capi.ERR_SHAPE
    assert lib.b2moe_peer_wait(None, 2, 1, 16, None) == capi.ERR_NULL
    assert lib.b2moe_peer_wait(16, 0, 1, 16, None) == capi.ERR_SHAPE
    assert lib.b2moe_peer_alloc(0, C.byref(C.c_void_p()), (C.c_uint8 * 64)()) == capi.ERR_SHAPE
    assert lib.b2moe_peer_open(None, C.byref(C.c_void_p())) == capi.ERR_NULL
    assert lib.b2moe_peer_close(None) == capi.ERR_NULL and lib.b2moe_peer_free(None) == capi.ERR_NULL
    with pytest.raises(capi.B2moeError):
        capi.check(capi.ERR_WORKSPACE, "x")


def test_load_aware_placement_balances_a_zipf_histogram():
    """b2moe_place_experts: a permutation, equal expert counts per rank, never worse than contiguous blocks, deterministic."""
    import numpy as np
    from tqllm_b200 import moe
    rng = np.random.default_rng(5)
    for experts, ranks in ((128, 8), (128, 2), (512, 4), (16, 16)):
        counts = (1e6 / np.arange(1, experts + 1) ** 1.2).astype(np.uint64)
        rng.shuffle(counts)
        order, load = moe.place_experts(counts, ranks)
        per = experts // ranks
        assert sorted(order.tolist()) == list(range(experts))
        got = np.array([counts[order[r * per:(r + 1) * per]].sum() for r in range(ranks)])
        assert np.array_equal(got, load)
        contiguous = counts.reshape(ranks, per).sum(1)
        assert load.max() <= contiguous.max()
        if per > 1:
            # longest-first bound; a rank that holds the heaviest expert still has to take per - 1 more (the lightest ones)
            assert load.max() <= max(counts.max() + np.sort(counts)[:per - 1].sum(), 1.34 * counts.sum() / ranks)
        order2, _ = moe.place_experts(counts, ranks)
        assert np.array_equal(order, order2)
    assert lib.b2moe_place_experts(None, 8, 2, None, None) != 0
    c = np.ones(10, np.uint64)
    o = np.empty(10, np.int32)
    assert lib.b2moe_place_experts(c.ctypes.data, 10, 3, o.ctypes.data, None) != 0               # 10 experts do not split over 3 ranks
