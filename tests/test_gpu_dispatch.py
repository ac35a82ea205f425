"""GPU dispatch through the C ABI: counts, offsets, active list and the stable permutation must equal the oracle's
counting sort exactly, on the single-block path (decode sizes), the multi-block path (prefill sizes up to 65,536
assignments), with skipped (-1) ids, with the shared expert appended, with every assignment on one expert."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def check(orc, ids, experts, shared):
    from tqllm_b200 import moe
    n, k = ids.shape
    plan = moe.dispatch(torch.from_numpy(ids).cuda(), experts, n if shared else 0)
    counts, offsets, perm = orc.dispatch(ids, experts)
    A = n * k
    got_counts = plan.counts.cpu().numpy()
    got_off = plan.offsets.cpu().numpy()
    assert np.array_equal(got_counts[:experts], counts) and got_counts[experts] == (n if shared else 0)
    assert np.array_equal(got_off[:experts + 1], offsets) and got_off[experts + 1] == offsets[-1] + (n if shared else 0)
    grouped = int(offsets[-1])
    gp = plan.perm.cpu().numpy()
    assert np.array_equal(gp[:grouped], perm[:grouped])
    if shared:
        assert np.array_equal(gp[grouped:grouped + n], A + np.arange(n))
    act = np.flatnonzero(got_counts > 0)
    assert plan.n_active == act.size and np.array_equal(plan.active.cpu().numpy()[:act.size], act)
    assert int(plan.buf[1]) == grouped + (n if shared else 0)
    # pass list: active experts from last to first, ceil(count / 8) passes each
    per = [-(-int(got_counts[e]) // 8) for e in act[::-1]]
    want = np.concatenate([[0], np.cumsum(per)]).astype(np.int32)
    assert np.array_equal(plan.passes.cpu().numpy()[:act.size + 1], want) and int(plan.buf[2]) == want[-1] and int(plan.buf[3]) == 0
    return plan


@pytest.mark.parametrize("n,k,e", ((1, 10, 512), (4, 10, 512), (64, 10, 512), (64, 4, 32), (16, 8, 256), (100, 8, 7), (819, 10, 512)))
@pytest.mark.parametrize("shared", (False, True))
def test_small_path(orc, n, k, e, shared):
    rng = np.random.default_rng(n * k + e)
    ids = np.stack([rng.permutation(e)[:k] if k <= e else rng.integers(0, e, k) for _ in range(n)]).astype(np.int32)
    check(orc, ids, e, shared)


@pytest.mark.parametrize("n,k,e", ((4096, 10, 512), (8192, 8, 128), (2048, 8, 256), (1500, 6, 1100)))
def test_large_path(orc, n, k, e):
    rng = np.random.default_rng(n + e)
    p = 1.0 / np.arange(1, e + 1) ** 1.2                 # Zipf-like skew: a hot expert gets many times the mean
    ids = rng.choice(e, size=(n, k), p=p / p.sum()).astype(np.int32)
    check(orc, ids, e, True)
    check(orc, ids, e, False)


def test_skipped_and_degenerate(orc):
    rng = np.random.default_rng(0)
    ids = rng.integers(-1, 9, size=(50, 4)).astype(np.int32)
    ids[3] = -1
    check(orc, ids, 9, False)
    check(orc, np.full((7, 3), -1, np.int32), 5, True)           # nothing routed: only the shared expert is active
    check(orc, np.full((300, 8), 2, np.int32), 4, False)         # every assignment on one expert
    big = np.full((5000, 8), -1, np.int32)
    big[::3, 0] = 1
    check(orc, big, 3, True)


def test_plan_to_groups_is_ordered_moe_group(orc):
    from tqllm_b200 import moe
    rng = np.random.default_rng(4)
    ids = np.stack([rng.permutation(16)[:4] for _ in range(33)]).astype(np.int32)
    plan = check(orc, ids, 16, False)
    counts, groups = moe.plan_to_groups(plan)
    counts, groups = counts.cpu().numpy(), groups.cpu().numpy()
    flat = ids.reshape(-1)
    for e in range(16):
        want = np.flatnonzero(flat == e)
        assert counts[e] == want.size and np.array_equal(groups[e, :want.size], want)


def test_repeatable_bits(orc):
    from tqllm_b200 import moe
    rng = np.random.default_rng(9)
    ids = torch.from_numpy(rng.integers(0, 512, size=(4096, 10)).astype(np.int32)).cuda()
    a = moe.dispatch(ids, 512, 4096).buf.clone()
    b = moe.dispatch(ids, 512, 4096).buf.clone()
    assert torch.equal(a, b)
