"""The oracle's whole-layer composition against the committed golden layers (outputs of the reference's own CPU
functions) and, live, against the reference compiled in place."""
import numpy as np
import pytest

from make_golden import layer_cases, layer_inputs, sha
from util import same_bits

CASES = layer_cases()


def run_oracle(orc, shape, experts, layer, x, logits=None):
    return orc.moe_layer(x=x.float().numpy(), router_w=layer.router_w.numpy(), topk=shape.topk, ff=shape.ff, gating=shape.gating,
                         norm=shape.norm, scale=shape.scale, types=shape.types, gate=layer.raw[0].numpy(),
                         up=layer.raw[1].numpy(), down=layer.raw[2].numpy(), experts=experts,
                         sel_bias=None if layer.sel_bias is None else layer.sel_bias.numpy(),
                         shared=None if layer.shared_raw is None else tuple(t.numpy() for t in layer.shared_raw),
                         logits_in=logits)


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_golden_layer(orc, golden, case):
    name, shape, experts, tokens, seed = case
    layer, x = layer_inputs(shape, experts, tokens, seed)
    g = golden["layer"]
    if sha(layer.router_w.numpy(), *[t.numpy() for t in layer.raw], x.float().numpy()) != str(g[f"{name}_sha"]):
        pytest.fail("the synthetic generator no longer reproduces the fixture's inputs: regenerate tests/golden")
    res = run_oracle(orc, shape, experts, layer, x)
    assert same_bits(res["logits"], g[f"{name}_logits"])
    assert np.array_equal(res["ids"], g[f"{name}_ids"])
    assert same_bits(res["weights"], g[f"{name}_w"])
    assert same_bits(res["out"], g[f"{name}_out"])
    # the dispatch artefacts are self-consistent with the ids
    flat = res["ids"].reshape(-1)
    for e in range(experts):
        assert np.array_equal(res["perm"][res["offsets"][e]:res["offsets"][e + 1]], np.flatnonzero(flat == e))


@pytest.mark.parametrize("case", CASES[:5], ids=[c[0] for c in CASES[:5]])
def test_layer_vs_compiled_reference(orc, ref, case):
    name, shape, experts, tokens, seed = case
    layer, x = layer_inputs(shape, experts, tokens, seed + 1000)
    res = run_oracle(orc, shape, experts, layer, x)
    r = ref.moe_layer(x=x.float().numpy(), topk=shape.topk, ff=shape.ff, gating=shape.gating, norm=shape.norm, scale=shape.scale,
                      types=shape.types, gate=layer.raw[0].numpy(), up=layer.raw[1].numpy(), down=layer.raw[2].numpy(),
                      experts=experts, logits_in=res["logits"], sel_bias=None if layer.sel_bias is None else layer.sel_bias.numpy(),
                      shared=None if layer.shared_raw is None else tuple(t.numpy() for t in layer.shared_raw))
    assert np.array_equal(res["ids"], r["ids"]) and same_bits(res["weights"], r["weights"]) and same_bits(res["out"], r["out"])


def test_expert_ffn_vs_naive_and_reference(orc, ref):
    rng = np.random.default_rng(1)
    h, f = 8, 6
    x = rng.standard_normal(h).astype(np.float32)
    wg, wu, wd = (rng.standard_normal(s).astype(np.float32) for s in ((f, h), (f, h), (h, f)))
    g, u = wg.astype(np.float64) @ x, wu.astype(np.float64) @ x
    want = wd.astype(np.float64) @ (g / (1 + np.exp(-g)) * u)
    got = orc.expert_ffn(x, wg, wu, wd)
    assert np.abs(got - want).max() < 1e-5
    for clamp, cg in ((0.0, False), (0.5, False), (0.5, True)):
        assert same_bits(orc.expert_ffn(x, wg, wu, wd, clamp, cg), ref.expert_ffn(x, wg, wu, wd, clamp, cg))


def test_combine(orc):
    out = np.zeros(4, np.float32)
    orc.combine(np.array([0.25, 0.75], np.float32), np.array([[1, 2, 3, 4], [4, 3, 2, 1]], np.float32), out)
    assert np.allclose(out, [3.25, 2.75, 2.25, 1.75])
