"""GPU: the expert-parallel compute phases (C ABI: b2moe_ep_local_ids, b2moe_dispatch_range, the grouped kernels,
b2moe_combine over local ids, b2moe_ep_reduce) with all ranks emulated on one device and the exchanges done by tensor
copies — how the reference tests its two-rank split (tests/ep_split.cu:87-151). The split result must equal the
unsplit layer: ids exactly, outputs up to the order of the fp32 partial sums when both sides run the same kernel
family (b2moe_harness_select pins it: a rank with a quarter of the experts would otherwise cross the
tokens-per-expert threshold of the tensor-core GEMM, whose fp16 operands round differently), and within the layer
tolerance with the default choice."""
import numpy as np
import pytest
import torch

from ep_oracle_backend import slice_raw
from make_golden import layer_inputs
from tqllm_b200 import synth
from util import rel_err

pytestmark = pytest.mark.gpu


def run_split(shape, E, T, world, seed, gate_vec=None):
    from tqllm_b200 import ep, moe
    layer, x = layer_inputs(shape, E, T * world, seed)
    full = moe.MoeLayer.from_synth(layer, experts=E, shared_gate_vec=gate_vec)
    xd = x.cuda()
    want = full.forward(xd).cpu().numpy()
    want_ids = full.artefacts()["ids"].cpu().numpy()
    H, F = shape.hidden, shape.ff
    ranks = []
    for r in range(world):
        first, count = ep.expert_range(E, world, r)
        raw = tuple(slice_raw(layer.raw[i], shape.types[i], (F, F, H)[i], (H, H, F)[i], first, count) for i in range(3))
        loc = moe.MoeLayer(shape, layer.router_w[first:first + count], raw, layer.shared_raw, experts=count, shared_gate_vec=gate_vec)
        ranks.append(ep.CudaEpLayer(loc, layer.router_w.cuda(), E, world, r, out_dtype=torch.float32,
                                    sel_bias_all=None if layer.sel_bias is None else layer.sel_bias.cuda()))
    routed = [rk.route_local(xd[r * T:(r + 1) * T]) for r, rk in enumerate(ranks)]
    ids_all = torch.cat([i for i, _ in routed]).contiguous()
    w_all = torch.cat([w for _, w in routed]).contiguous()
    assert np.array_equal(ids_all.cpu().numpy(), want_ids)
    parts = [rk.partial_sums(xd, ids_all, w_all) for rk in ranks]
    # the packed-record form of the same exchange (one pack launch per rank, one unpack launch) gives the same partial sums
    if ranks[0].can_pack(xd, ids_all.shape[1]):
        rec_all = torch.cat([rk.pack_all(xd[r * T:(r + 1) * T].contiguous(), *routed[r]) for r, rk in enumerate(ranks)]).contiguous()
        for r, rk in enumerate(ranks):
            want_parts = parts[r][0].clone()
            got_parts, _ = rk.partial_sums_packed(rec_all, ids_all.shape[1], xd.dtype)
            assert torch.equal(got_parts, want_parts)
    outs = []
    for h, rk in enumerate(ranks):
        recv = torch.stack([parts[r][0][h * T:(h + 1) * T] for r in range(world)]).contiguous()
        outs.append(rk.finish(recv, parts[h][1]).cpu().numpy())
    return np.concatenate(outs), want


def run_split_a2a(shape, E, T, world, seed, gate_vec=None):
    """the all-to-all dispatch with every rank on this device: the exchanges are slices of the ranks' send buffers"""
    from tqllm_b200 import ep, moe
    layer, x = layer_inputs(shape, E, T * world, seed)
    full = moe.MoeLayer.from_synth(layer, experts=E, shared_gate_vec=gate_vec)
    xd = x.cuda()
    want = full.forward(xd).cpu().numpy()
    H, F = shape.hidden, shape.ff
    ranks = []
    for r in range(world):
        first, count = ep.expert_range(E, world, r)
        raw = tuple(slice_raw(layer.raw[i], shape.types[i], (F, F, H)[i], (H, H, F)[i], first, count) for i in range(3))
        loc = moe.MoeLayer(shape, layer.router_w[first:first + count], raw, layer.shared_raw, experts=count, shared_gate_vec=gate_vec)
        ranks.append(ep.CudaEpLayer(loc, layer.router_w.cuda(), E, world, r, out_dtype=torch.float32,
                                    sel_bias_all=None if layer.sel_bias is None else layer.sel_bias.cuda()))
    st = []
    for r, rk in enumerate(ranks):
        xl = xd[r * T:(r + 1) * T].contiguous()
        ids, w = rk.route_local(xl)
        ids, w = ids.clone(), w.clone()
        counts, pos, lst = (t.clone() for t in rk.peer_lists(ids))
        n = [int(v) for v in counts.cpu()]
        off = torch.zeros(world + 1, dtype=torch.int32)
        off[1:] = torch.cumsum(torch.tensor(n, dtype=torch.int32), 0)
        send = rk.pack_records(xl, ids, w, lst, off.cuda(), sum(n)).clone()
        st.append(dict(n=n, off=[int(v) for v in off], offd=off.cuda(), pos=pos, send=send, sw=None if rk.shared_w is None else rk.shared_w.clone()))
    outs = []
    backs = [[None] * world for _ in range(world)]
    for p, rk in enumerate(ranks):                      # rank p receives segment p of every rank's send buffer, in rank order
        segs = [st[r]["send"][st[r]["off"][p]:st[r]["off"][p + 1]] for r in range(world)]
        recv_n = [s_.shape[0] for s_ in segs]
        recv = torch.cat(segs).contiguous()
        parts, shared = rk.partial_sums_records(recv, sum(recv_n), sum(recv_n[:p]), T)
        assert int(rk.buf["plan"][3]) == 0
        st[p]["shared"] = None if shared is None else shared.clone()
        o = 0
        for r in range(world):
            backs[r][p] = parts[o:o + recv_n[r]].clone()
            o += recv_n[r]
    for r, rk in enumerate(ranks):
        back = torch.cat(backs[r]).contiguous()
        rk.shared_w = st[r]["sw"]
        outs.append(rk.finish_records(back, st[r]["pos"], st[r]["offd"], st[r]["shared"]).cpu().numpy())
    sent = sum(sum(s_["n"]) for s_ in st)
    return np.concatenate(outs), want, sent


@pytest.mark.parametrize("world", (2, 4))
@pytest.mark.parametrize("types,gating,shared,topk", (((21, 21, 21), 1, True, 2), ((12, 12, 12), 2, False, 4)))
def test_alltoall_dispatch_equals_unsplit(world, types, gating, shared, topk):
    from tqllm_b200 import capi
    shape = synth.LayerShape("ep-a2a", 512, 16, topk, 256, gating=gating, sel_bias=gating == 2, shared=shared, types=types)
    with capi.family("decode"):
        got, want, sent = run_split_a2a(shape, 16, 7, world, 80 + world)
    assert rel_err(got, want) <= 1e-5
    assert sent <= world * world * 7                    # never more records than the all-gather moves
    if topk == 2 and world == 4:
        assert sent < world * world * 7                 # two experts cannot sit on four ranks: some token rows stay home


@pytest.mark.parametrize("world", (2, 4))
@pytest.mark.parametrize("types,gating,shared", (((21, 21, 21), 1, True), ((12, 12, 12), 2, False), ((23, 23, 20), 1, True)))
def test_split_equals_unsplit(world, types, gating, shared):
    from tqllm_b200 import capi
    ff = 256 if types[2] != 20 else 96
    shape = synth.LayerShape("ep-gpu", 512, 16, 4, ff, gating=gating, sel_bias=gating == 2, shared=shared, types=types)
    with capi.family("decode"):
        got, want = run_split(shape, 16, 6, world, 50 + world)
    assert rel_err(got, want) <= 1e-5


def test_split_with_gated_shared_expert():
    """a shared expert scaled by sigmoid(v . x): every rank weighs the shared rows of its own tokens exactly as one GPU does"""
    from tqllm_b200 import capi
    g = torch.Generator()
    g.manual_seed(12)
    v = torch.randn(512, generator=g) * 0.05
    shape = synth.LayerShape("ep-gated", 512, 16, 4, 256, shared=True, types=(21, 21, 21))
    with capi.family("decode"):
        got, want = run_split(shape, 16, 6, 4, 61, gate_vec=v)
        plain, _ = run_split(shape, 16, 6, 4, 61)
    assert rel_err(got, want) <= 1e-5
    assert rel_err(plain, want) > 1e-3          # the gate matters: without it the result is a different one


@pytest.mark.parametrize("types", ((21, 21, 21), (12, 12, 12)))
def test_split_default_paths_within_layer_tolerance(types):
    shape = synth.LayerShape("ep-gpu-auto", 512, 16, 4, 256, shared=True, types=types)
    got, want = run_split(shape, 16, 6, 4, 77)
    assert rel_err(got, want) <= 1e-2


def test_uneven_blocks_and_idle_rank():
    """7 experts over 4 ranks (blocks of 2, 2, 2, 1), and a rank whose experts nobody routed to"""
    from tqllm_b200 import capi
    with capi.family("decode"):
        shape = synth.LayerShape("ep-uneven", 512, 7, 2, 256, shared=True, types=(21, 21, 21))
        got, want = run_split(shape, 7, 3, 4, 9)
        assert rel_err(got, want) <= 1e-5
        shape = synth.LayerShape("ep-idle", 512, 16, 1, 256, types=(21, 21, 21))
        got, want = run_split(shape, 16, 1, 4, 10)          # one token, one expert: three ranks have nothing to do
        assert rel_err(got, want) <= 1e-5


class OneRankComm:
    """world of one: the exchanges are copies (the graphed forward must give the bits of the direct one)"""
    world, rank = 1, 0

    def buffer(self, shape, dtype, device=None):
        return torch.empty(shape, dtype=dtype, device=device)

    def all_gather(self, t, out=None):
        if out is None:
            return t.clone()
        out.copy_(t)
        return out

    def all_to_all(self, t, out=None):
        if out is None:
            return t.clone()
        out.copy_(t)
        return out


def test_graphed_compute_phases_equal_direct_launches():
    from tqllm_b200 import ep, moe
    shape = synth.LayerShape("ep-graph", 512, 16, 4, 256, shared=True, types=(21, 21, 21))
    layer, x = layer_inputs(shape, 16, 24, 3)
    loc = moe.MoeLayer.from_synth(layer, experts=16)
    rk = ep.CudaEpLayer(loc, layer.router_w.cuda(), 16, 1, 0, out_dtype=torch.float32)
    comm = OneRankComm()
    xd = x.cuda()
    want = ep.ep_forward(rk, comm, xd).clone()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        gf = ep.GraphedEpForward(rk, comm, xd)
        got1 = gf().clone()
        xd.copy_(torch.flip(xd, dims=(0,)))              # new contents at the same address
        got2 = gf().clone()
    side.synchronize()
    assert torch.equal(got1, want)
    assert torch.equal(got2, torch.flip(want, dims=(0,)))


def test_peer_memory_exchange_world_of_one_equals_copies():
    """the put / wait kernels through the rank's own inbox: the same bits as plain copies, direct and graphed, and the
    sequence numbers keep step over repeated exchanges"""
    from tqllm_b200 import ep, moe
    shape = synth.LayerShape("ep-peer", 512, 16, 4, 256, shared=True, types=(21, 21, 21))
    layer, x = layer_inputs(shape, 16, 24, 5)
    loc = moe.MoeLayer.from_synth(layer, experts=16)
    rk = ep.CudaEpLayer(loc, layer.router_w.cuda(), 16, 1, 0, out_dtype=torch.float32)
    xd = x.cuda()
    want = ep.ep_forward(rk, OneRankComm(), xd).clone()
    pc = ep.PeerComm()
    try:
        for _ in range(3):
            got = ep.ep_forward(rk, pc, xd).clone()
            assert torch.equal(got, want)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            gf = ep.GraphedEpForward(rk, pc, xd)
            g1 = gf().clone()
            g2 = gf().clone()
        side.synchronize()
        assert torch.equal(g1, want) and torch.equal(g2, want)
        pc.check()
    finally:
        pc.close()


def test_peer_wait_runs_out_and_reports_the_sender():
    """a counter that nobody raises: the wait returns within its bound and names the sender in the status word (no trap, the
    context stays usable)"""
    from tqllm_b200 import capi
    lib = capi.lib
    counters = torch.zeros(4, dtype=torch.int32, device="cuda")
    counters[0] = 7
    counters[1] = 7
    counters[3] = 9
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    capi.check(lib.b2moe_peer_wait(counters.data_ptr(), 4, 7, status.data_ptr(), st), "b2moe_peer_wait")
    torch.cuda.synchronize()
    assert int(status.item()) == 1 + 2                      # sender 2 never arrived; 0, 1 and 3 (already past 7) did
    status.zero_()
    counters[2] = 7
    capi.check(lib.b2moe_peer_wait(counters.data_ptr(), 4, 7, status.data_ptr(), st), "b2moe_peer_wait")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
