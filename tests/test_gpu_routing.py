"""GPU routing through the C ABI. Protocol of the reference's device test (tests/moe_device.cu:32-74): the router dot
is checked against an fp64 dot; the device top-k must equal the CPU moe_route (oracle) run on the DEVICE's own
logits; weights within 3e-6. A mismatch is accepted only when the CPU's own selection keys differ by <= 4 ulp (the
near-tie audit), and the tests state how many such ties they saw (0 for these seeds)."""
import numpy as np
import pytest
import torch

import oracle as O
from util import audit_ids

pytestmark = pytest.mark.gpu


def cpu_keys(gating, logits, bias):
    x = logits.astype(np.float32)
    if gating == O.SOFTMAX:
        e = np.exp(x - x.max(-1, keepdims=True))
        p = e / e.sum(-1, keepdims=True)
    else:
        p = 1 / (1 + np.exp(-x))
    return (p if bias is None else p + bias).astype(np.float32)


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16, torch.float16))
# the last two sizes take the shared-memory tile kernel (bf16, 256 tokens or more): ragged token and row tiles, and the c3 prefill shape
@pytest.mark.parametrize("n,h,e", ((1, 256, 8), (5, 1024, 32), (64, 2048, 512), (19, 512, 100), (300, 96, 70), (1024, 2048, 512)))
def test_router_logits_vs_fp64(orc, dtype, n, h, e):
    from tqllm_b200 import moe
    g = torch.Generator()
    g.manual_seed(n + h + e)
    w = torch.randn(e, h, generator=g) * 0.02
    sg = torch.randn(h, generator=g) * 0.02
    x = torch.randn(n, h, generator=g).to(dtype)
    logits = moe.router(w.cuda(), x.cuda(), sg.cuda()).cpu().numpy()
    want = orc.router_logits(torch.cat([w, sg[None]]).numpy(), x.float().numpy(), f64=True)
    assert np.abs(logits - want).max() < 3e-6 * max(1.0, np.abs(want).max())
    # without the shared-gate row the extra column is left alone
    l2 = moe.router(w.cuda(), x.cuda(), None).cpu().numpy()
    assert np.array_equal(l2[:, :e], logits[:, :e]) and np.all(l2[:, e] == 0)


@pytest.mark.parametrize("e,k,n", ((8, 2, 4), (32, 4, 64), (512, 10, 64), (128, 8, 300), (1000, 8, 7), (2000, 6, 3)))
def test_topk_softmax_matches_cpu_route_on_device_logits(orc, e, k, n):
    from tqllm_b200 import moe
    g = torch.Generator()
    g.manual_seed(e * 7 + k)
    logits = torch.randn(n, e + 1, generator=g) * 2.0
    for scale in (0.0, 2.5):
        ids, w, sw = moe.topk_softmax(logits.cuda(), e, k, scale, shared=True)
        ids, w, sw = ids.cpu().numpy(), w.cpu().numpy(), sw.cpu().numpy()
        cid, cw = orc.route(O.SOFTMAX, logits[:, :e].numpy(), k, True, scale)
        ties = audit_ids(ids, cid, cpu_keys(O.SOFTMAX, logits[:, :e].numpy(), None))
        assert ties == 0
        assert np.abs(w - cw).max() < 3e-6 * max(1.0, scale)
        assert np.abs(sw - 1 / (1 + np.exp(-logits[:, e].numpy().astype(np.float64)))).max() < 3e-6
        assert np.abs(w.sum(-1) - (scale or 1.0)).max() < 1e-5


@pytest.mark.parametrize("e,k,n", ((512, 10, 17), (256, 8, 1), (1000, 8, 5)))
def test_two_routings_in_one_launch_equal_two_calls(e, k, n):
    """The reference's moe_topk2 (src/experts/moe.cu:160-166): this layer's routing and the next layer's predicted one."""
    from tqllm_b200 import moe
    g = torch.Generator()
    g.manual_seed(e + n)
    la, lb = (torch.randn(n, e + 1, generator=g) * 2.0).cuda(), (torch.randn(n, e + 1, generator=g) * 2.0).cuda()
    (i1, w1, s1), (i2, w2, s2) = moe.topk_softmax2(la, lb, e, k, 1.0, shared=True)
    for logits, got in ((la, (i1, w1, s1)), (lb, (i2, w2, s2))):
        want = moe.topk_softmax(logits, e, k, 1.0, shared=True)
        for a, b in zip(got, want):
            assert torch.equal(a, b)


def test_topk_ties_and_extremes(orc):
    from tqllm_b200 import moe
    rows = np.zeros((4, 17), np.float32)
    rows[0, :16] = 0.5                                   # all equal: lowest indices win
    rows[1, :16] = [10000, -10000, 10000, 0, 3, 3, 3, 3] * 2
    rows[2, :16] = -10000
    rows[2, 5] = 10000
    rows[3, :16] = np.arange(16) * 1e-3
    ids, w, _ = moe.topk_softmax(torch.from_numpy(rows).cuda(), 16, 4, 0.0, shared=True)
    cid, cw = orc.route(O.SOFTMAX, rows[:, :16], 4, True, 0.0)
    assert np.array_equal(ids.cpu().numpy(), cid)
    assert list(ids[0].cpu().numpy()) == [0, 1, 2, 3]
    assert np.isfinite(w.cpu().numpy()).all() and np.abs(w.cpu().numpy() - cw).max() < 3e-6


@pytest.mark.parametrize("e,k,n,norm,scale", ((16, 4, 9, True, 0.0), (256, 8, 16, True, 1.0), (288, 8, 33, True, 2.5), (64, 6, 5, False, 2.0)))
def test_sigmoid_bias_route(orc, e, k, n, norm, scale):
    from tqllm_b200 import moe
    g = torch.Generator()
    g.manual_seed(e + k)
    logits = torch.randn(n, e, generator=g) * 3
    bias = torch.randn(e, generator=g) * 0.1
    for b in (None, bias):
        ids, w = moe.route_sigmoid(logits.cuda(), e, k, None if b is None else b.cuda(), norm, scale)
        cid, cw = orc.route(O.SIGMOID, logits.numpy(), k, norm, scale, None if b is None else b.numpy())
        ties = audit_ids(ids.cpu().numpy(), cid, cpu_keys(O.SIGMOID, logits.numpy(), None if b is None else b.numpy()))
        assert ties == 0
        assert np.abs(w.cpu().numpy() - cw).max() < 3e-6 * max(1.0, scale)


def test_sigmoid_known_answers(orc):
    """the reference's routing KATs (tests/moe.cpp:155-236) on the device"""
    from tqllm_b200 import moe
    logits = torch.tensor([[2., 1., 0., -1.]]).cuda()
    ids, w = moe.route_sigmoid(logits, 4, 2, None, False, 1.0)
    assert list(ids[0].cpu().numpy()) == [0, 1]
    ids, w = moe.route_sigmoid(logits, 4, 2, torch.tensor([0., 0., 0., 100.]).cuda(), False, 1.0)
    assert int(ids[0, 0]) == 3 and abs(float(w[0, 0]) - 1 / (1 + np.exp(1.0))) < 1e-6
    ids, w = moe.route_sigmoid(torch.tensor([[-200., -300., -400., -500.]]).cuda(), 4, 4, None, True, 0.0)
    assert np.isfinite(w.cpu().numpy()).all() and list(ids[0].cpu().numpy()) == [0, 1, 2, 3]
    ids, _ = moe.route_sigmoid(torch.full((1, 8), 0.5).cuda(), 8, 3, None, False, 0.0)
    assert list(ids[0].cpu().numpy()) == [0, 1, 2]
