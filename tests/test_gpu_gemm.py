"""GPU: the tcgen05 grouped GEMM (every bank format, experts holding many tokens) against the exact fp32 generic path
of the same library and, end to end, against the oracle.

The GEMM rounds the decoded weights and the activations to fp16 and sums in fp32; the generic path is exact fp32
(src/experts/moe.cpp:115-155 order). Tolerance: max |err| / RMS(reference) <= 1e-2, the bound of the layer tests;
observed values are about 3e-3."""
import numpy as np
import pytest
import torch

from make_golden import layer_inputs
from test_gpu_layer import run_case
from tqllm_b200 import synth
from util import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-2


def forced_path(name, item_tokens=0):
    """the kernel family of every expert product inside the block (b2moe_harness_select)"""
    from tqllm_b200 import capi
    return capi.family(name, item_tokens)


def products(shape, experts, tokens, seed, path, item_tokens=0, iq3s_layout="codes"):
    from tqllm_b200 import moe
    layer, x = layer_inputs(shape, experts, tokens, seed)
    dev = moe.MoeLayer.from_synth(layer, experts=experts, iq3s_layout=iq3s_layout)
    xd = x.cuda()
    logits = moe.router(dev.router_w, xd)
    ids, w, _ = moe.topk_softmax(logits, experts, shape.topk, shape.scale)
    plan = moe.dispatch(ids, experts, tokens if shape.shared else 0)
    sh = dev.sh if shape.shared else (None, None, None)
    with forced_path(path, item_tokens):
        act = moe.expert_gateup_swiglu(dev.gate, dev.up, xd, plan, sh[0], sh[1])
        y = moe.expert_down(dev.down, act, plan, sh[2])
    torch.cuda.synchronize()
    assert int(plan.buf[3]) == 0, "a bounded wait ran out"
    return act.cpu().numpy(), y.cpu().numpy()


# (types, hidden, ff, experts, topk, tokens, shared, act dtype): token tiles of 128 + a ragged rest, partial row blocks
# (ff = 320: 20 row tiles = 2.5 blocks), a 64-column tail chunk (IQ4_NL down with K = 320), a shared expert
GEMM_CASES = (
    ((12, 12, 12), 512, 256, 4, 2, 300, True, "bf16"),
    ((21, 21, 21), 512, 256, 4, 2, 150, True, "f32"),
    ((21, 21, 21), 512, 256, 4, 2, 140, True, "bf16", "gguf"),
    ((23, 23, 20), 512, 320, 3, 2, 200, False, "bf16"),
    ((20, 20, 20), 256, 192, 2, 1, 270, True, "bf16"),
    ((323, 323, 323), 512, 256, 4, 3, 130, True, "bf16"),
    ((12, 12, 12), 256, 256, 8, 2, 5, True, "f32"),
)


@pytest.mark.parametrize("case", GEMM_CASES, ids=[f"{c[0][0]}-{c[0][2]}-t{c[5]}" + (f"-{c[8]}" if len(c) > 8 else "") for c in GEMM_CASES])
def test_gemm_matches_exact_path(case):
    types, hidden, ff, experts, topk, tokens, shared, dt = case[:8]
    lay = case[8] if len(case) > 8 else "codes"                  # IQ3_S banks: 4-bit codes (default) or the GGUF-sized layout
    shape = synth.LayerShape("gemm", hidden, experts, topk, ff, shared=shared, types=types, act_dtype=dt)
    act_g, y_g = products(shape, experts, tokens, 7, "gemm", iq3s_layout=lay)
    act_x, y_x = products(shape, experts, tokens, 7, "generic", iq3s_layout=lay)
    assert rel_err(act_g, act_x) <= TOL
    assert rel_err(y_g, y_x) <= TOL
    # the same call again: the same bits
    act_2, y_2 = products(shape, experts, tokens, 7, "gemm", iq3s_layout=lay)
    assert np.array_equal(act_g.view(np.uint32), act_2.view(np.uint32)) and np.array_equal(y_g.view(np.uint32), y_2.view(np.uint32))


@pytest.mark.parametrize("types", ((12, 12, 12), (21, 21, 21), (23, 23, 20), (323, 323, 323)), ids=("q4k", "iq3s", "iq4xs-nl", "nvfp4"))
def test_gemm_layer_against_oracle(orc, types):
    """whole layer with the GEMM forced, 40 tokens per expert on average"""
    shape = synth.LayerShape("gemm-layer", 512, 8, 2, 256, shared=True, types=types)
    with forced_path("gemm"):
        err = run_case(orc, shape, 8, 160, 31)
    assert err <= TOL


def test_full_size_c2_gemm_agrees_with_decode_kernels():
    """benchmark shape (512 experts, hidden 2048, IQ3_S), 512 tokens: two independent tensor-core paths, same sums"""
    from tqllm_b200 import moe
    shape = synth.CONFIGS["c2"]
    layer = synth.make_layer(shape, 5, "cuda")
    dev = moe.MoeLayer.from_synth(layer)
    x = synth.make_tokens(shape, 512, 6, "cuda")
    outs = {}
    for path in ("decode", "gemm"):
        with forced_path(path):
            outs[path] = dev.forward(x).float().cpu().numpy()
        assert dev.artefacts()["status"] == 0          # no bounded wait ran out
    assert rel_err(outs["gemm"], outs["decode"]) <= TOL
    assert np.isfinite(outs["gemm"]).all()


def test_token_order_does_not_change_a_token():
    """c3 shape (NVFP4G, 512 experts), 640 tokens: reversing the batch reverses the outputs bit for bit — a token's sums
    do not depend on its column in the MMA tile or on its neighbours"""
    from tqllm_b200 import moe
    shape = synth.CONFIGS["c3"]
    layer = synth.make_layer(shape, 8, "cuda")
    dev = moe.MoeLayer.from_synth(layer)
    x = synth.make_tokens(shape, 640, 9, "cuda")
    with forced_path("gemm"):
        a = dev.forward(x).float().cpu().numpy()
        b = dev.forward(torch.flip(x, dims=(0,)).contiguous()).float().cpu().numpy()
    assert np.array_equal(a.view(np.uint32), b[::-1].copy().view(np.uint32))


def test_gemm_layer_sigmoid_bias_routing(orc):
    """the c4 routing (sigmoid scores, selection bias, renormalised weights, no shared expert) over Q4_K banks, GEMM forced"""
    shape = synth.LayerShape("gemm-c4", 768, 16, 4, 512, gating=2, sel_bias=True, types=(12, 12, 12))
    with forced_path("gemm"):
        err = run_case(orc, shape, 16, 200, 77)
    assert err <= TOL


@pytest.mark.parametrize("case", (GEMM_CASES[0], GEMM_CASES[3], GEMM_CASES[5]), ids=("q4k", "iq4xs-nl", "nvfp4"))
def test_gemm_256_token_items_match_exact_path(case):
    """the 256-token item variant (one accumulator set, two B stages), forced: token tiles of 256 + a ragged rest"""
    types, hidden, ff, experts, topk, tokens, shared, dt = case[:8]
    shape = synth.LayerShape("gemm-wide", hidden, experts, topk, ff, shared=shared, types=types, act_dtype=dt)
    act_g, y_g = products(shape, experts, 3 * tokens, 11, "gemm", item_tokens=256)
    act_x, y_x = products(shape, experts, 3 * tokens, 11, "generic")
    assert rel_err(act_g, act_x) <= TOL
    assert rel_err(y_g, y_x) <= TOL
