"""GPU: b2moe_expert_down_static, the down product for callers that cannot hand the library any scratch memory (an
engine plugin that owns no device memory, code inside a stream capture). It must give the results of
b2moe_expert_down, call after call, although its scratch is one fixed array inside the library that keeps the
previous call's contents. This file sorts last on purpose: it runs after every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

from make_golden import layer_inputs
from tqllm_b200 import synth

pytestmark = pytest.mark.gpu


def down_both_ways(shape, experts, tokens, seed):
    from tqllm_b200 import capi, moe
    from tqllm_b200.capi import lib
    layer, x = layer_inputs(shape, experts, tokens, seed)
    dev = moe.MoeLayer.from_synth(layer, experts=experts)
    xd = x.cuda()
    logits = moe.router(dev.router_w, xd)
    ids, w, _ = moe.topk_softmax(logits, experts, shape.topk, shape.scale)
    plan = moe.dispatch(ids, experts, tokens)
    act = moe.expert_gateup_swiglu(dev.gate, dev.up, xd, plan, dev.sh[0], dev.sh[1])
    want = moe.expert_down(dev.down, act, plan, dev.sh[2])
    got = torch.zeros_like(want)
    # one call first so that the module's one-time look-up of the array is behind us; then the driver's own figure of free
    # device memory (which also sees an allocation made behind torch's back) must not move over a second call
    rc = lib.b2moe_expert_down_static(C.byref(dev.down.c), C.byref(dev.sh[2].c), act.data_ptr(), plan.buf.data_ptr(), tokens, shape.topk,
                                      tokens, got.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == capi.OK, capi.status_string(rc)
    torch.cuda.synchronize()
    got.zero_()
    before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
    rc = lib.b2moe_expert_down_static(C.byref(dev.down.c), C.byref(dev.sh[2].c), act.data_ptr(), plan.buf.data_ptr(), tokens, shape.topk,
                                      tokens, got.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == capi.OK, capi.status_string(rc)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.cuda.mem_get_info()[0] == free_before
    assert int(plan.buf[3]) == 0
    return got.cpu().numpy(), want.cpu().numpy()


def test_static_scratch_down_matches_workspace_down_twice():
    big = synth.LayerShape("noalloc-a", 512, 16, 4, 512, shared=True, types=(21, 21, 21))
    small = synth.LayerShape("noalloc-b", 256, 8, 2, 256, shared=True, types=(21, 21, 21))
    # two calls in a row: the second is smaller, so the shared array still holds rows of the first beyond its own
    for shape, experts, tokens, seed in ((big, 16, 40, 1), (small, 8, 5, 2), (big, 16, 40, 3)):
        got, want = down_both_ways(shape, experts, tokens, seed)
        ref = np.sqrt((want.astype(np.float64) ** 2).mean())
        assert np.abs(got - want).max() <= 1e-2 * ref          # the layer-output tolerance of the other tests
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))   # in fact the same kernel: the same bits


def test_static_scratch_rejects_oversize_and_serves_other_formats():
    from tqllm_b200 import capi
    from tqllm_b200.capi import lib
    assert lib.b2moe_static_scratch_bytes() == 16 << 20
    # 70,000 assignments x 256 columns x 2 bytes (fp16 operand rows) > 16 MiB: refused before anything is launched
    bank = capi.Bank(256, None, 21, 4, 32, 256)
    rc = lib.b2moe_expert_down_static(C.byref(bank), None, 256, 256, 7000, 10, 0, 256, None)
    assert rc == capi.ERR_CAPACITY
    assert lib.b2moe_expert_down_static(C.byref(bank), None, None, 256, 4, 2, 0, 256, None) == capi.ERR_NULL
    # a Q4_K bank (tensor-core GEMM: its fp16 rows go to the same array) matches the ordinary entry point
    shape = synth.LayerShape("noalloc-q4k", 256, 8, 2, 256, shared=True, types=(12, 12, 12))
    got, want = down_both_ways(shape, 8, 6, 4)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
