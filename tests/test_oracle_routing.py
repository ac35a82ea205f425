"""The oracle's routing against the reference: the known-answer cases of the reference's tests/moe.cpp restated,
an independent max-scan router, the committed golden routings (outputs of the reference's moe_route), and random
cases against the compiled reference."""
import numpy as np
import pytest

import oracle as O


def indep_route(gating, logits, k, norm, scale, bias):
    """independent statement: repeated max scan, first maximum wins (the shape of tests/moe.cpp:112-151)"""
    x = np.asarray(logits, np.float32)
    if gating == 1:
        e = np.exp((x - x.max()).astype(np.float32)).astype(np.float32)
        s = np.float32(0)
        for v in e:
            s = np.float32(s + v)
        p = (e / s).astype(np.float32)
    else:
        p = (np.float32(1) / (np.float32(1) + np.exp(-x).astype(np.float32))).astype(np.float32)
    key = p.copy() if bias is None else (p + np.asarray(bias, np.float32)).astype(np.float32)
    ids = []
    for _ in range(k):
        i = int(np.argmax(key))          # argmax returns the first maximum = the lowest index
        ids.append(i)
        key[i] = -np.inf
    w = p[ids].astype(np.float32)
    if norm:
        s = np.float32(0)
        for v in w:
            s = np.float32(s + v)
        w = (w / max(s, np.float32(6.103515625e-5))).astype(np.float32)
    if scale not in (0.0, 1.0):
        w = (w * np.float32(scale)).astype(np.float32)
    return np.array(ids, np.int32), w


def test_bias_changes_selection_not_weights(orc):
    logits = np.array([2, 1, 0, -1], np.float32)
    ids, w = orc.route(O.SIGMOID, logits, 2, norm=False, scale=1.0)
    assert list(ids[0]) == [0, 1]
    ids, w = orc.route(O.SIGMOID, logits, 2, norm=False, scale=1.0, sel_bias=np.array([0, 0, 0, 100], np.float32))
    assert ids[0][0] == 3
    assert abs(w[0][0] - 1 / (1 + np.exp(1.0))) < 1e-6 and w[0][0] < 0.5


def test_ties_take_lowest_index(orc):
    ids, _ = orc.route(O.SIGMOID, np.full(8, 0.5, np.float32), 3, norm=False)
    assert list(ids[0]) == [0, 1, 2]


def test_underflow_gives_no_nan(orc):
    _, w = orc.route(O.SIGMOID, np.array([-200, -300, -400, -500], np.float32), 4, norm=True)
    assert np.isfinite(w).all()


def test_scale_zero_and_one_are_identity(orc):
    logits = np.array([3, 1, -1, -3], np.float32)
    a = orc.route(O.SIGMOID, logits, 2, norm=True, scale=0.0)
    b = orc.route(O.SIGMOID, logits, 2, norm=True, scale=1.0)
    c = orc.route(O.SIGMOID, logits, 2, norm=True, scale=2.5)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    assert abs(c[1][0][0] - 2.5 * b[1][0][0]) < 1e-6
    assert abs(b[1].sum() - 1) < 1e-6 and abs(c[1].sum() - 2.5) < 1e-6


def test_glm_shape_selection_follows_biased_probs(orc):
    logits = (np.sin(np.arange(288) * 0.7) * 3).astype(np.float32)
    bias = (0.001 * (np.arange(288) % 7)).astype(np.float32)
    ids, w = orc.route(O.SIGMOID, logits, 8, norm=True, scale=2.5, sel_bias=bias)
    p = 1 / (1 + np.exp(-logits.astype(np.float64)))
    key = p + bias
    assert all(key[ids[0][i - 1]] >= key[ids[0][i]] for i in range(1, 8))
    want = p[ids[0]] / p[ids[0]].sum() * 2.5
    assert np.abs(w[0] - want).max() < 1e-5
    i2, w2 = indep_route(2, logits, 8, True, 2.5, bias)
    assert np.array_equal(ids[0], i2) and np.abs(w[0] - w2).max() < 1e-6


def test_random_routing_vs_independent(orc):
    rng = np.random.default_rng(5)
    for gating in (1, 2):
        for norm in (False, True):
            for biased in (False, True):
                for _ in range(100):
                    e = int(rng.integers(2, 62))
                    k = int(rng.integers(1, e + 1))
                    scale = float(rng.uniform(0, 4))
                    logits = rng.uniform(-8, 8, e).astype(np.float32)
                    bias = rng.uniform(-1, 1, e).astype(np.float32) if biased else None
                    ids, w = orc.route(gating, logits, k, norm, scale, bias)
                    i2, w2 = indep_route(gating, logits, k, norm, scale, bias)
                    assert np.array_equal(ids[0], i2)
                    assert np.abs(w[0] - w2).max() <= 2e-6 * max(1.0, scale)


def test_committed_golden_routings(orc, golden):
    g = golden["route"]
    for i in range(int(g["n"])):
        gating, norm, k = (int(v) for v in g[f"cfg_{i}"])
        bias = g[f"bias_{i}"]
        ids, w = orc.route(gating, g[f"logits_{i}"], k, norm, float(g[f"scale_{i}"]), bias if bias.size else None)
        assert np.array_equal(ids[0], g[f"ids_{i}"]), i
        assert np.array_equal(w[0].view(np.uint32), g[f"w_{i}"].view(np.uint32)), i


def test_random_routing_vs_compiled_reference(orc, ref):
    rng = np.random.default_rng(11)
    for gating in (1, 2, 3, 4):
        for _ in range(100):
            e = int(rng.integers(2, 300))
            k = int(rng.integers(1, min(e, 20) + 1))
            logits = rng.uniform(-8, 8, e).astype(np.float32)
            bias = rng.uniform(-1, 1, e).astype(np.float32) if rng.random() < 0.5 else None
            norm, scale = bool(rng.integers(0, 2)), float(rng.choice([0, 1, 2.5]))
            a, b = orc.route(gating, logits, k, norm, scale, bias), ref.route(gating, logits, k, norm, scale, bias)
            assert np.array_equal(a[0], b[0])
            assert np.array_equal(a[1].view(np.uint32), b[1].view(np.uint32))


def test_bad_shapes(orc):
    with pytest.raises(ValueError):
        orc.route(O.SOFTMAX, np.zeros(4, np.float32), 5)
    with pytest.raises(ValueError):
        orc.route(0, np.zeros(4, np.float32), 2)


def test_dispatch_is_stable_counting_sort(orc):
    rng = np.random.default_rng(3)
    ids = rng.integers(-1, 9, size=(50, 4)).astype(np.int32)
    counts, offsets, perm = orc.dispatch(ids, 9)
    flat = ids.reshape(-1)
    assert counts.sum() == (flat >= 0).sum() and offsets[-1] == counts.sum()
    for e in range(9):
        seg = perm[offsets[e]:offsets[e + 1]]
        assert np.array_equal(seg, np.flatnonzero(flat == e))
    counts, offsets, perm = orc.dispatch(np.full((3, 2), -1, np.int32), 4)
    assert counts.sum() == 0 and np.all(perm == -1)
