"""Expert parallelism on CPU ranks (gloo, world size 2 and 3): the real orchestration and exchanges of
tqllm_b200.ep with the oracle as the compute backend must reproduce the unsplit oracle layer, including uneven
expert blocks, a shared expert, sigmoid + bias routing; and a rank that never joins is detected by the timeout."""
import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tqllm_b200 import ep, synth


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def case(name):
    S = synth.LayerShape
    return {
        "softmax_shared": (S("ep-a", 256, 8, 3, 256, shared=True, types=(21, 21, 21)), 8, 5),
        "sigmoid_bias": (S("ep-b", 256, 6, 2, 256, gating=synth.SIGMOID, sel_bias=True, types=(12, 12, 12)), 6, 4),
        "gated_shared": (S("ep-c", 256, 8, 3, 256, shared=True, types=(21, 21, 21)), 8, 4),
    }[name]


def gate_vector(name):
    if name != "gated_shared":
        return None
    g = torch.Generator()
    g.manual_seed(77)
    return torch.randn(256, generator=g) * 0.1


def skewed_order(E, world):
    """a placement as b2moe_place_experts gives it for a histogram with one hot expert per contiguous block's start"""
    from tqllm_b200 import moe
    counts = np.array([1000 // (1 + (e * 7) % E) for e in range(E)], np.uint64)
    order, _ = moe.place_experts(counts, world)
    return order


def worker(rank, world, port, name, out_dir, a2a=False, placed=False):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from ep_oracle_backend import OracleEpBackend
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=60))
    shape, E, T = case(name)
    layer = synth.make_layer(shape, 31, "cpu", experts=E)
    if placed:                                      # the experts stacked in a load-aware order before the rank blocks are cut
        layer = synth.permute_experts(layer, skewed_order(E, world))
    x = synth.make_tokens(shape, T * world, 31, "cpu")[rank * T:(rank + 1) * T]
    fwd = ep.ep_forward_a2a if a2a else ep.ep_forward
    out = fwd(OracleEpBackend(shape, layer, E, world, rank, gate_vector(name)), ep.TorchComm(), x)
    np.save(os.path.join(out_dir, f"out{rank}.npy"), out.numpy())
    dist.destroy_process_group()


@pytest.mark.parametrize("name,world", (("softmax_shared", 2), ("softmax_shared", 3), ("sigmoid_bias", 2), ("gated_shared", 2)))
@pytest.mark.parametrize("a2a", (False, True), ids=("allgather", "alltoall"))
def test_ep_matches_unsplit_oracle(orc, tmp_path, name, world, a2a):
    port = free_port()
    mp.spawn(worker, args=(world, port, name, str(tmp_path), a2a), nprocs=world, join=True)
    shape, E, T = case(name)
    layer = synth.make_layer(shape, 31, "cpu", experts=E)
    x = synth.make_tokens(shape, T * world, 31, "cpu")
    want = orc.moe_layer(x=x.float().numpy(), router_w=layer.router_w.numpy(), topk=shape.topk, ff=shape.ff, gating=shape.gating,
                         norm=shape.norm, scale=shape.scale, types=shape.types, gate=layer.raw[0].numpy(), up=layer.raw[1].numpy(),
                         down=layer.raw[2].numpy(), experts=E, sel_bias=None if layer.sel_bias is None else layer.sel_bias.numpy(),
                         shared=None if layer.shared_raw is None else tuple(t.numpy() for t in layer.shared_raw),
                         shared_gate_vec=None if gate_vector(name) is None else gate_vector(name).numpy())["out"]
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    rms = np.sqrt((want.astype(np.float64) ** 2).mean())
    assert np.abs(got - want).max() <= 1e-5 * rms        # only the order of the fp32 partial sums differs


@pytest.mark.parametrize("a2a", (False, True), ids=("allgather", "alltoall"))
def test_ep_with_a_load_aware_placement_matches_the_unplaced_layer(orc, tmp_path, a2a):
    """experts stacked in the order b2moe_place_experts returns, then split over the ranks: the layer's output is that of
    the layer in its original order (routing only renames the experts)"""
    name, world = "softmax_shared", 2
    port = free_port()
    mp.spawn(worker, args=(world, port, name, str(tmp_path), a2a, True), nprocs=world, join=True)
    shape, E, T = case(name)
    assert sorted(skewed_order(E, world).tolist()) == list(range(E)) and not np.array_equal(skewed_order(E, world), np.arange(E))
    layer = synth.make_layer(shape, 31, "cpu", experts=E)
    x = synth.make_tokens(shape, T * world, 31, "cpu")
    want = orc.moe_layer(x=x.float().numpy(), router_w=layer.router_w.numpy(), topk=shape.topk, ff=shape.ff, gating=shape.gating,
                         norm=shape.norm, scale=shape.scale, types=shape.types, gate=layer.raw[0].numpy(), up=layer.raw[1].numpy(),
                         down=layer.raw[2].numpy(), experts=E, sel_bias=None,
                         shared=tuple(t.numpy() for t in layer.shared_raw), shared_gate_vec=None)["out"]
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    rms = np.sqrt((want.astype(np.float64) ** 2).mean())
    assert np.abs(got - want).max() <= 1e-5 * rms


def test_expert_ranges_partition():
    for E in (8, 128, 256, 512, 7):
        for G in (1, 2, 3, 4, 8):
            blocks = [ep.expert_range(E, G, r) for r in range(G)]
            assert blocks[0][0] == 0 and sum(c for _, c in blocks) == E
            assert all(blocks[i][0] + blocks[i][1] == blocks[i + 1][0] for i in range(G - 1))
            assert max(c for _, c in blocks) - min(c for _, c in blocks) <= 1


def lonely(rank, world, port, q):
    """rank 0 of a 2-rank group whose peer never joins: the rendezvous must fail within its timeout, not hang"""
    try:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=2,
                                timeout=datetime.timedelta(seconds=3))
        q.put("joined")
    except Exception as e:  # noqa: BLE001
        q.put("timeout:" + type(e).__name__)


def test_missing_rank_is_detected_on_the_host():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=lonely, args=(0, 2, free_port(), q))
    p.start()
    p.join(60)
    assert not p.is_alive()
    assert q.get(timeout=5).startswith("timeout:")
