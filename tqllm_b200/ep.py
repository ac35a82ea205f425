"""Expert parallelism over the GPUs of one box: rank r of G owns a contiguous block of experts, tokens stay
data-parallel, router weights and the shared expert are replicated.

Per layer (the G-rank generalisation of the reference's two-rank `--split experts` path, fn_layer_forward.cpp:475-503,
924-976, with NCCL all-gather / all-to-all in place of its grouped send / recv, tp_comm.cpp:94-101):

  1. route      every rank routes its own T tokens (router + top-k);
  2. dispatch   exchange: all ranks gather every rank's activation rows, routed ids and weights, packed into one
                record per token so that it is ONE all-gather (with top-k spread over G ranks nearly every token has an
                expert on every rank, so the dispatch all-to-all at fixed capacity T is an all-gather);
  3. experts    ids outside the rank's block become -1; the usual dispatch -> gate/up + SwiGLU -> down runs on the
                G*T tokens for the local experts, the shared expert only for the rank's own tokens; a combine over
                the local assignments (slot order) leaves one fp32 partial sum per token;
  4. combine    exchange: all-to-all returns slice h of the partial sums to home rank h, which adds the G slices in
                ascending rank order (deterministic) plus its shared expert.

For batches where gathering every token on every rank is too much (prefill), `ep_forward_a2a` is the all-to-all form of
steps 2 - 4: a rank sends a token only to the ranks that own one of its routed experts (and always to itself, so that
its shared expert finds every own token in the local batch); a count exchange gives both sides the exact sizes, so there
is no fixed capacity and no overflow rule (the reference's two-rank exchange caps the result rows and computes the
overflow locally, src/models/qwen/qwen4exp/decode_rules.hpp:210, which needs every expert resident on every rank).
The partial sums travel home by the reverse all-to-all and are added in ascending peer order.

The orchestration below is backend-agnostic (phases + a communicator) so that the same code runs on NCCL, on gloo
with a CPU backend in the tests, and in-process with all ranks on one GPU (the reference tests EP the same way,
tests/ep_split.cu:87-151). The CUDA backend calls the C ABI only.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist


def expert_range(experts: int, world: int, rank: int) -> tuple[int, int]:
    """(first, count) of the contiguous expert block rank `rank` owns; blocks differ by at most one expert"""
    base, extra = divmod(experts, world)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


class TorchComm:
    """all-gather / all-to-all over a torch.distributed process group (NCCL on GPUs, gloo on CPU)"""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def buffer(self, shape, dtype, device=None) -> torch.Tensor:
        """a result buffer for all_gather / all_to_all (PeerComm hands out its inboxes here)"""
        return torch.empty(shape, dtype=dtype, device=device)

    def all_gather(self, t: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """[n, ...] per rank -> [world * n, ...] in rank order"""
        if out is None:
            out = torch.empty((self.world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        try:
            dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        except (RuntimeError, NotImplementedError):
            parts = list(out.chunk(self.world))
            dist.all_gather(parts, t.contiguous(), group=self.group)
        return out

    def all_to_all(self, t: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """[world, ...]: slice r goes to rank r; returns [world, ...] with slice r received from rank r"""
        if out is None:
            out = torch.empty_like(t)
        try:
            dist.all_to_all_single(out, t.contiguous(), group=self.group)
        except (RuntimeError, NotImplementedError):
            reqs = []
            for r in range(self.world):
                if r == self.rank:
                    out[r].copy_(t[r])
                else:
                    reqs.append(dist.isend(t[r].contiguous(), r, group=self.group))
                    reqs.append(dist.irecv(out[r], r, group=self.group))
            for q in reqs:
                q.wait()
        return out

    def all_to_all_v(self, t: torch.Tensor, send_counts, recv_counts) -> torch.Tensor:
        """rows of t in peer segments of send_counts rows -> the rows received, in peer segments of recv_counts rows"""
        out = torch.empty((sum(recv_counts),) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        try:
            dist.all_to_all_single(out, t.contiguous(), list(recv_counts), list(send_counts), group=self.group)
        except (RuntimeError, NotImplementedError):
            so, ro = [0], [0]
            for c in send_counts:
                so.append(so[-1] + c)
            for c in recv_counts:
                ro.append(ro[-1] + c)
            reqs = []
            for p in range(self.world):
                if p == self.rank:
                    out[ro[p]:ro[p + 1]].copy_(t[so[p]:so[p + 1]])
                else:
                    if send_counts[p]:
                        reqs.append(dist.isend(t[so[p]:so[p + 1]].contiguous(), p, group=self.group))
                    if recv_counts[p]:
                        reqs.append(dist.irecv(out[ro[p]:ro[p + 1]], p, group=self.group))
            for q in reqs:
                q.wait()
        return out


class _LibraryMemory:
    """device memory owned by the library, handed to torch through the CUDA array interface (uint8)"""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerComm:
    """The two fixed-size exchanges of the all-gather path over peer memory instead of library collectives: every rank owns
    an inbox with one slot per sender; a sender stores its block into every receiver's inbox and raises a counter there
    (b2moe_peer_put), a receiver waits, bounded, for all counters (b2moe_peer_wait). One process per GPU on one node. The
    process group is used for set-up only (the 64-byte memory handles). all_gather / all_to_all write into a tensor obtained
    from buffer() (or into an inbox of their own when none is given) and return it; the result stays valid until the next
    exchange into the same buffer. The kernels number the exchanges themselves (device counters), so a sequence of layer
    calls with their exchanges can be captured into a CUDA graph and replayed (`capturable`)."""
    capturable = True

    def __init__(self, group=None):
        from . import capi
        self.capi, self.lib = capi, capi.lib
        self.group = group
        # without a process group: a world of one (the exchanges then run through the rank's own inbox)
        self.world, self.rank = (dist.get_world_size(group), dist.get_rank(group)) if dist.is_initialized() else (1, 0)
        self.dev = torch.device("cuda", torch.cuda.current_device())
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.inboxes, self.own, self.opened = {}, [], []

    def _symmetric(self, nbytes: int):
        """a zeroed allocation of nbytes on every rank -> (own pointer, [every rank's pointer as seen from here])"""
        ptr, handle = C.c_void_p(), (C.c_uint8 * 64)()
        failed = int(self.lib.b2moe_peer_alloc(nbytes, C.byref(ptr), handle) != 0)
        if not failed:
            self.own.append(ptr.value)
        if self.world == 1:
            if failed:
                raise self.capi.B2moeError(self.capi.ERR_CUDA, "b2moe_peer_alloc failed")
            return ptr.value, [ptr.value]
        # a rank that failed still takes part in the two collectives below, so that all ranks give up together
        mine = torch.tensor(list(handle), dtype=torch.uint8, device=self.dev)
        every = torch.empty(self.world * 64, dtype=torch.uint8, device=self.dev)
        dist.all_gather_into_tensor(every, mine, group=self.group)
        every = every.cpu().view(self.world, 64)
        ptrs = []
        for p in range(self.world if not failed else 0):
            if p == self.rank:
                ptrs.append(ptr.value)
                continue
            q, h = C.c_void_p(), (C.c_uint8 * 64)(*every[p].tolist())
            if self.lib.b2moe_peer_open(h, C.byref(q)) != 0:
                failed = 1
                ptrs.append(0)
            else:
                self.opened.append(q.value)
                ptrs.append(q.value)
        bad = torch.tensor([failed], dtype=torch.int32, device=self.dev)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX, group=self.group)      # every rank learns of a failure: they give up together
        if int(bad):
            raise self.capi.B2moeError(self.capi.ERR_CUDA, "an inbox could not be allocated or a peer's memory handle could not be opened")
        return ptr.value, ptrs

    def buffer(self, shape, dtype, device=None) -> torch.Tensor:
        """an exchange result buffer: world slots of numel / world elements each (collective: every rank, same order)"""
        nbytes = int(torch.Size(shape).numel()) * torch.empty(0, dtype=dtype).element_size()
        assert nbytes % (16 * self.world) == 0
        slot = nbytes // self.world
        box, boxes = self._symmetric(nbytes)
        cnt, cnts = self._symmetric(max(256, 4 * (self.world + 1)))
        t = torch.as_tensor(_LibraryMemory(box, nbytes), device=self.dev).view(dtype).view(shape)
        self.inboxes[t.data_ptr()] = {
            "tensor": t, "slot": slot, "counters": cnt,
            "dst": torch.tensor([boxes[p] + self.rank * slot for p in range(self.world)], dtype=torch.int64, device=self.dev),
            "flags": torch.tensor([cnts[p] + 4 * self.rank for p in range(self.world)], dtype=torch.int64, device=self.dev),
            "tickets": torch.zeros(self.world + 2, dtype=torch.int32, device=self.dev)}
        return t

    def _exchange(self, t: torch.Tensor, stride: int, nbytes: int, out: torch.Tensor) -> torch.Tensor:
        b = self.inboxes[out.data_ptr()]
        assert nbytes == b["slot"] and t.is_contiguous()
        st = torch.cuda.current_stream().cuda_stream
        self.capi.check(self.lib.b2moe_peer_put(t.data_ptr(), stride, nbytes, b["dst"].data_ptr(), b["flags"].data_ptr(), b["tickets"].data_ptr(),
                                                self.world, 0, st), "b2moe_peer_put")
        self.capi.check(self.lib.b2moe_peer_wait(b["counters"], self.world, 0, self.status.data_ptr(), st), "b2moe_peer_wait")
        return out

    def _own_buffer(self, kind, shape, dtype):
        key = (kind, tuple(shape), dtype)
        if key not in self.inboxes:
            self.inboxes[key] = self.buffer(shape, dtype)
        return self.inboxes[key]

    def all_gather(self, t: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """every rank's t (same shape everywhere) stacked along dim 0 in rank order"""
        if out is None:
            out = self._own_buffer("ag", (self.world * t.shape[0],) + tuple(t.shape[1:]), t.dtype)
        return self._exchange(t, 0, t.numel() * t.element_size(), out)

    def all_to_all(self, t: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """t[p] goes to rank p; out[q] = what rank q sent here"""
        if out is None:
            out = self._own_buffer("a2a", tuple(t.shape), t.dtype)
        n = t[0].numel() * t.element_size()
        return self._exchange(t, n, n, out)

    def check(self):
        """raises if a wait ran out (reads one int from the device: call it outside timed regions)"""
        v = int(self.status.item())
        if v:
            raise self.capi.B2moeError(self.capi.ERR_CUDA, f"the exchange with rank {v - 1} did not arrive within the wait's bound")

    def close(self):
        torch.cuda.synchronize()
        for q in self.opened:
            self.lib.b2moe_peer_close(q)
        self.inboxes.clear()
        for q in self.own:
            self.lib.b2moe_peer_free(q)
        self.opened, self.own = [], []


def pack_tokens(x: torch.Tensor, ids: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """one byte record per token: its activation row, its k routed ids and its k routing weights -> uint8 [n][record]"""
    n = x.shape[0]
    xb, ib, wb = x.shape[1] * x.element_size(), ids.shape[1] * 4, w.shape[1] * 4
    if out is None:
        out = torch.empty(n, xb + ib + wb, dtype=torch.uint8, device=x.device)
    out[:, :xb].copy_(x.contiguous().view(torch.uint8).view(n, xb))
    out[:, xb:xb + ib].copy_(ids.contiguous().view(torch.uint8).view(n, ib))
    out[:, xb + ib:].copy_(w.contiguous().view(torch.uint8).view(n, wb))
    return out


def unpack_tokens(rec: torch.Tensor, hidden: int, topk: int, x_dtype, x=None, ids=None, w=None):
    """the inverse of pack_tokens for [N][record] gathered records -> (x [N][hidden], ids [N][k] int32, w [N][k] f32)"""
    N = rec.shape[0]
    xb, ib = hidden * torch.empty((), dtype=x_dtype).element_size(), topk * 4
    if x is None:
        x = torch.empty(N, hidden, dtype=x_dtype, device=rec.device)
        ids = torch.empty(N, topk, dtype=torch.int32, device=rec.device)
        w = torch.empty(N, topk, dtype=torch.float32, device=rec.device)
    x.view(torch.uint8).view(N, xb).copy_(rec[:, :xb])
    ids.view(torch.uint8).view(N, ib).copy_(rec[:, xb:xb + ib])
    w.view(torch.uint8).view(N, ib).copy_(rec[:, xb + ib:])
    return x, ids, w


def ep_forward(backend, comm, x_local: torch.Tensor) -> torch.Tensor:
    """one expert-parallel layer forward for this rank's tokens; `backend` supplies the three compute phases"""
    ids, weights = backend.route_local(x_local)
    if getattr(backend, "can_pack", None) and backend.can_pack(x_local, ids.shape[1]):      # one pack and one unpack launch
        rec_all = comm.all_gather(backend.pack_all(x_local, ids, weights))
        parts, shared = backend.partial_sums_packed(rec_all, ids.shape[1], x_local.dtype)
    else:
        rec_all = comm.all_gather(pack_tokens(x_local, ids, weights))
        x_all, ids_all, w_all = unpack_tokens(rec_all, x_local.shape[1], ids.shape[1], x_local.dtype)
        parts, shared = backend.partial_sums(x_all, ids_all, w_all)
    recv = comm.all_to_all(parts.view(comm.world, x_local.shape[0], -1))
    return backend.finish(recv, shared)


def ep_forward_a2a(backend, comm, x_local: torch.Tensor) -> torch.Tensor:
    """one expert-parallel layer forward with the all-to-all dispatch (two host reads of G counts per layer)"""
    G, r, T = comm.world, comm.rank, x_local.shape[0]
    ids, weights = backend.route_local(x_local)
    counts, pos, lst = backend.peer_lists(ids)                       # device: [G], [G][T], [G][T]
    recv_counts = comm.all_to_all(counts.view(G, 1)).view(G)
    send_n, recv_n = [int(v) for v in counts.cpu()], [int(v) for v in recv_counts.cpu()]
    offsets = torch.zeros(G + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(torch.tensor(send_n, dtype=torch.int32), 0)
    offsets = offsets.to(counts.device)
    send = backend.pack_records(x_local, ids, weights, lst, offsets, sum(send_n))
    recv = comm.all_to_all_v(send, send_n, recv_n)
    parts, shared = backend.partial_sums_records(recv, sum(recv_n), sum(recv_n[:r]), T)
    back = comm.all_to_all_v(parts, recv_n, send_n)
    return backend.finish_records(back, pos, offsets, shared)


def phase_times(backend, comm, x_local: torch.Tensor, reps: int = 20) -> dict:
    """mean microseconds of every phase of one expert-parallel layer on this rank (CUDA events on the current stream, every
    rank must call it): route, pack + all-gather + unpack, the local expert products, the all-to-all of the partial sums,
    the rank-ordered reduce. The sum is a direct-launch layer; the graphed step is faster by the launch overheads."""
    ev = lambda: torch.cuda.Event(enable_timing=True)
    names = ("route", "dispatch_exchange", "local_experts", "combine_exchange", "reduce")
    acc = dict.fromkeys(names, 0.0)
    for it in range(reps + 2):
        e = [ev() for _ in range(6)]
        e[0].record()
        ids, weights = backend.route_local(x_local)
        e[1].record()
        packed = bool(getattr(backend, "can_pack", None)) and backend.can_pack(x_local, ids.shape[1])
        rec_all = comm.all_gather(backend.pack_all(x_local, ids, weights) if packed else pack_tokens(x_local, ids, weights))
        if not packed:
            x_all, ids_all, w_all = unpack_tokens(rec_all, x_local.shape[1], ids.shape[1], x_local.dtype)
        e[2].record()
        parts, shared = backend.partial_sums_packed(rec_all, ids.shape[1], x_local.dtype) if packed else backend.partial_sums(x_all, ids_all, w_all)
        e[3].record()
        recv = comm.all_to_all(parts.view(comm.world, x_local.shape[0], -1))
        e[4].record()
        backend.finish(recv, shared)
        e[5].record()
        torch.cuda.synchronize()
        if it >= 2:
            for i, n in enumerate(names):
                acc[n] += e[i].elapsed_time(e[i + 1]) * 1e3 / reps
    return acc


class CudaEpLayer:
    """The three compute phases of one rank on the device, through the C ABI. `layer` holds ONLY this rank's experts
    (a tqllm_b200.moe.MoeLayer built from the rank's slice of the stacked banks) plus the replicated router weight
    over ALL experts."""

    def __init__(self, layer, router_w_all: torch.Tensor, experts_total: int, world: int, rank: int, out_dtype=torch.bfloat16,
                 sel_bias_all: torch.Tensor | None = None):
        from . import capi
        self.capi, self.lib = capi, capi.lib
        self.layer, self.shape = layer, layer.shape
        self.router_w, self.sel_bias = router_w_all, sel_bias_all
        self.E, self.world, self.rank = experts_total, world, rank
        self.first, self.count = expert_range(experts_total, world, rank)
        assert layer.experts == self.count
        self.out_dtype = out_dtype
        self.buf = {}

    def _b(self, name, shape, dtype):
        t = self.buf.get(name)
        if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype:
            t = torch.zeros(shape, dtype=dtype, device=self.router_w.device)
            self.buf[name] = t
        return t

    def _st(self):
        return torch.cuda.current_stream().cuda_stream

    def route_local(self, x):
        from . import moe
        lib, sh = self.lib, self.shape
        n = x.shape[0]
        logits = self._b("logits", (n, self.E + 1), torch.float32)
        ids = self._b("ids", (n, sh.topk), torch.int32)
        w = self._b("w", (n, sh.topk), torch.float32)
        dt = moe._DT[x.dtype]
        # a gated shared expert (weight = sigmoid(v . x), the router's extra logits column): the weights of this rank's own tokens
        gate_vec = self.layer.shared_gate_vec if self.layer.sh is not None else None
        if gate_vec is not None and sh.gating != self.capi.SOFTMAX:
            raise self.capi.B2moeError(self.capi.ERR_SHAPE, "the sigmoid routing family adds its shared expert unscaled")
        self.shared_w = self._b("shared_w", (n,), torch.float32) if gate_vec is not None else None
        self.capi.check(lib.b2moe_router(self.router_w.data_ptr(), None if gate_vec is None else gate_vec.data_ptr(), x.data_ptr(), dt,
                                         logits.data_ptr(), self.E + 1, sh.hidden, self.E, n, self._st()), "b2moe_router")
        if sh.gating == self.capi.SOFTMAX:
            self.capi.check(lib.b2moe_topk_softmax(logits.data_ptr(), self.E + 1, ids.data_ptr(), w.data_ptr(),
                                                   None if self.shared_w is None else self.shared_w.data_ptr(), self.E, sh.topk, n,
                                                   sh.scale, self._st()), "b2moe_topk_softmax")
        else:
            bias = None if self.sel_bias is None else self.sel_bias.data_ptr()
            self.capi.check(lib.b2moe_route_sigmoid(logits.data_ptr(), self.E + 1, bias, ids.data_ptr(), w.data_ptr(), self.E, sh.topk,
                                                    int(sh.norm), sh.scale, n, self._st()), "b2moe_route_sigmoid")
        return ids, w

    def live_estimate(self, nominal: int) -> int:
        """expected number of the nominal n * topk assignments whose expert lives on this rank (uniform routing): the kernel
        family of the expert products is chosen from it (b2moe_expert_*_sparse)"""
        return min(nominal, max(1, -(-nominal * self.count // self.E)))

    def partial_sums(self, x_all, ids_all, w_all):
        N, k = ids_all.shape
        local = self._b("local", (N, k), torch.int32)
        self.capi.check(self.lib.b2moe_ep_local_ids(ids_all.data_ptr(), local.data_ptr(), N * k, self.first, self.count, self._st()), "ep_local_ids")
        return self._local_products(x_all, local, w_all)

    # one launch each instead of three strided copies (and a fourth for the local ids): the packed token records of the all-gather
    def can_pack(self, x, k):
        return (x.shape[1] * x.element_size()) % 16 == 0 and (8 * k) % 16 == 0

    def pack_all(self, x, ids, w, out=None):
        n, k = ids.shape
        xb = x.shape[1] * x.element_size()
        if out is None:
            out = torch.empty(n, xb + 8 * k, dtype=torch.uint8, device=x.device)
        lst = self.buf.get("own_list")
        if lst is None or lst.numel() != n:
            lst = torch.arange(n, dtype=torch.int32, device=x.device)
            self.buf["own_list"], self.buf["own_offsets"] = lst, torch.tensor([0, n], dtype=torch.int32, device=x.device)
        self.capi.check(self.lib.b2moe_ep_pack(x.data_ptr(), xb, ids.data_ptr(), w.data_ptr(), k, n, lst.data_ptr(), self.buf["own_offsets"].data_ptr(),
                                               1, n, out.data_ptr(), self._st()), "b2moe_ep_pack")
        return out

    def partial_sums_packed(self, rec_all, k, x_dtype):
        N, H = rec_all.shape[0], self.shape.hidden
        x_all, local, w_all = self._b("x_all", (N, H), x_dtype), self._b("local", (N, k), torch.int32), self._b("w_all", (N, k), torch.float32)
        self.capi.check(self.lib.b2moe_ep_unpack(rec_all.data_ptr(), N, H * x_all.element_size(), k, self.first, self.count, x_all.data_ptr(),
                                                 local.data_ptr(), w_all.data_ptr(), self._st()), "b2moe_ep_unpack")
        return self._local_products(x_all, local, w_all)

    def _local_products(self, x_all, local, w_all):
        from . import moe
        lib, sh, L = self.lib, self.shape, self.layer
        N, k = local.shape
        T = N // self.world
        A = N * k
        has_sh = L.sh is not None
        shared_n = N if has_sh else 0                      # buffer rows for the shared expert (token-indexed)
        pv = self.capi.PlanView()
        lib.b2moe_plan_view_of(self.count, A, T if has_sh else 0, C.byref(pv))
        plan = self._b("plan", (pv.total,), torch.int32)
        dws = self._b("dws", (max(lib.b2moe_dispatch_workspace_bytes(self.count, A), 16),), torch.uint8)
        self.capi.check(lib.b2moe_dispatch_range(local.data_ptr(), N, k, self.count, self.rank * T, T if has_sh else 0, plan.data_ptr(),
                                                 dws.data_ptr(), dws.numel(), self._st()), "b2moe_dispatch_range")
        act = self._b("act", (A + shared_n, sh.ff), torch.float32)
        y = self._b("y", (A + shared_n, sh.hidden), torch.float32)
        dt = moe._DT[x_all.dtype]
        eg = lib.b2moe_expert_workspace_bytes(L.gate.type, N, sh.hidden, dt)
        ed = lib.b2moe_expert_workspace_bytes(L.down.type, A + shared_n, sh.ff, self.capi.F32)
        ews = self._b("ews", (max(eg, ed, 16),), torch.uint8)
        br = lambda b: C.byref(b.c)
        shg, shu, shd = (br(L.sh[0]), br(L.sh[1]), br(L.sh[2])) if has_sh else (None, None, None)
        live = self.live_estimate(N * k)                 # this rank owns count / experts_total of the experts: so many ids are not -1
        self.capi.check(lib.b2moe_expert_gateup_swiglu_sparse(br(L.gate), br(L.up), shg, shu, x_all.data_ptr(), dt, plan.data_ptr(), N, k,
                                                              shared_n, live, act.data_ptr(), ews.data_ptr(), ews.numel(), self._st()), "gateup")
        self.capi.check(lib.b2moe_expert_down_sparse(br(L.down), shd, act.data_ptr(), plan.data_ptr(), N, k, shared_n, live, y.data_ptr(),
                                                     ews.data_ptr(), ews.numel(), self._st()), "down")
        parts = self._b("parts", (N, sh.hidden), torch.float32)
        self.capi.check(lib.b2moe_combine(y.data_ptr(), local.data_ptr(), w_all.data_ptr(), None, N, k, sh.hidden, 0, parts.data_ptr(),
                                          self.capi.F32, self._st()), "b2moe_combine")
        shared = y[A + self.rank * T:A + (self.rank + 1) * T] if has_sh else None
        return parts, shared

    # ---- all-to-all dispatch ----
    def _bounds(self):
        b = self.buf.get("bounds")
        if b is None:
            b = torch.tensor([expert_range(self.E, self.world, p)[0] for p in range(self.world)] + [self.E], dtype=torch.int32,
                             device=self.router_w.device)
            self.buf["bounds"] = b
        return b

    def peer_lists(self, ids):
        n, k = ids.shape
        G = self.world
        counts, pos, lst = self._b("pl_counts", (G,), torch.int32), self._b("pl_pos", (G, n), torch.int32), self._b("pl_list", (G, n), torch.int32)
        self.capi.check(self.lib.b2moe_ep_peer_lists(ids.data_ptr(), n, k, self._bounds().data_ptr(), G, self.rank, counts.data_ptr(),
                                                     pos.data_ptr(), lst.data_ptr(), self._st()), "b2moe_ep_peer_lists")
        return counts, pos, lst

    def pack_records(self, x, ids, w, lst, offsets, records):
        n, k = ids.shape
        xb = x.shape[1] * x.element_size()
        out = torch.empty(max(records, 1), xb + 8 * k, dtype=torch.uint8, device=x.device)[:records]
        self.capi.check(self.lib.b2moe_ep_pack(x.data_ptr(), xb, ids.data_ptr(), w.data_ptr(), k, n, lst.data_ptr(), offsets.data_ptr(),
                                               self.world, records, out.data_ptr(), self._st()), "b2moe_ep_pack")
        return out

    def partial_sums_records(self, recv, records, self_off, T):
        """the local expert products over the received records; the shared expert for the T records at self_off (the rank's own tokens)"""
        from . import moe
        lib, sh, L = self.lib, self.shape, self.layer
        k, H = sh.topk, sh.hidden
        x_dtype = torch.bfloat16 if sh.act_dtype != "f32" else torch.float32
        xb = H * (2 if x_dtype != torch.float32 else 4)
        N = max(records, 1)
        x = torch.empty(N, H, dtype=x_dtype, device=recv.device)
        ids = torch.full((N, k), -1, dtype=torch.int32, device=recv.device)
        w = torch.zeros(N, k, dtype=torch.float32, device=recv.device)
        self.capi.check(lib.b2moe_ep_unpack(recv.data_ptr(), records, xb, k, self.first, self.count, x.data_ptr(), ids.data_ptr(), w.data_ptr(),
                                            self._st()), "b2moe_ep_unpack")
        has_sh = L.sh is not None
        A, shared_n = N * k, (N if has_sh else 0)
        pv = self.capi.PlanView()
        lib.b2moe_plan_view_of(self.count, A, T if has_sh else 0, C.byref(pv))
        plan = torch.zeros(pv.total, dtype=torch.int32, device=recv.device)
        dws = torch.empty(max(lib.b2moe_dispatch_workspace_bytes(self.count, A), 16), dtype=torch.uint8, device=recv.device)
        self.capi.check(lib.b2moe_dispatch_range(ids.data_ptr(), N, k, self.count, self_off if has_sh else 0, T if has_sh else 0, plan.data_ptr(),
                                                 dws.data_ptr(), dws.numel(), self._st()), "b2moe_dispatch_range")
        act = torch.empty(A + shared_n, sh.ff, dtype=torch.float32, device=recv.device)
        y = torch.empty(A + shared_n, H, dtype=torch.float32, device=recv.device)
        dt = moe._DT[x_dtype]
        eg = lib.b2moe_expert_workspace_bytes(L.gate.type, N, H, dt)
        ed = lib.b2moe_expert_workspace_bytes(L.down.type, A + shared_n, sh.ff, self.capi.F32)
        ews = torch.empty(max(eg, ed, 16), dtype=torch.uint8, device=recv.device)
        br = lambda b: C.byref(b.c)
        shg, shu, shd = (br(L.sh[0]), br(L.sh[1]), br(L.sh[2])) if has_sh else (None, None, None)
        live = self.live_estimate(N * k)
        self.capi.check(lib.b2moe_expert_gateup_swiglu_sparse(br(L.gate), br(L.up), shg, shu, x.data_ptr(), dt, plan.data_ptr(), N, k, shared_n,
                                                              live, act.data_ptr(), ews.data_ptr(), ews.numel(), self._st()), "gateup")
        self.capi.check(lib.b2moe_expert_down_sparse(br(L.down), shd, act.data_ptr(), plan.data_ptr(), N, k, shared_n, live, y.data_ptr(),
                                                     ews.data_ptr(), ews.numel(), self._st()), "down")
        parts = torch.empty(N, H, dtype=torch.float32, device=recv.device)
        self.capi.check(lib.b2moe_combine(y.data_ptr(), ids.data_ptr(), w.data_ptr(), None, N, k, H, 0, parts.data_ptr(), self.capi.F32,
                                          self._st()), "b2moe_combine")
        self.buf["plan"] = plan
        shared = y[A + self_off:A + self_off + T] if has_sh else None
        return parts[:records], shared

    def finish_records(self, back, pos, offsets, shared):
        from . import moe
        G, T = pos.shape
        H = self.shape.hidden
        out = self._b("out", (T, H), self.out_dtype)
        sw = getattr(self, "shared_w", None) if shared is not None else None
        self.capi.check(self.lib.b2moe_ep_return_reduce(back.data_ptr(), pos.data_ptr(), offsets.data_ptr(), G,
                                                        None if shared is None else shared.data_ptr(), None if sw is None else sw.data_ptr(),
                                                        T, H, out.data_ptr(), moe._DT[self.out_dtype], self._st()), "b2moe_ep_return_reduce")
        return out

    def finish(self, recv, shared):
        G, T, H = recv.shape
        out = self._b("out", (T, H), self.out_dtype)
        from . import moe
        sw = getattr(self, "shared_w", None) if shared is not None else None
        self.capi.check(self.lib.b2moe_ep_reduce(recv.data_ptr(), G, None if shared is None else shared.data_ptr(),
                                                 None if sw is None else sw.data_ptr(), T, H, out.data_ptr(), moe._DT[self.out_dtype],
                                                 self._st()), "b2moe_ep_reduce")
        return out


class GraphedEpForward:
    """ep_forward for a CUDA backend with the three compute phases replayed as CUDA graphs (one launch each instead of
    about ten) and the two collectives issued between them in the ordinary way: no collective is ever captured. The input
    tensor and every exchange buffer keep their addresses; `x_local` must be the same tensor at every call."""

    def __init__(self, backend: CudaEpLayer, comm, x_local: torch.Tensor):
        self.backend, self.comm, self.x = backend, comm, x_local
        G, T = comm.world, x_local.shape[0]
        dev = x_local.device
        stream = torch.cuda.current_stream()
        # eager pass: allocates the backend's buffers and gives the exchange buffers their shapes
        ids, w = backend.route_local(x_local)
        k = ids.shape[1]
        packed = bool(getattr(backend, "can_pack", None)) and backend.can_pack(x_local, k)
        self.rec = backend.pack_all(x_local, ids, w) if packed else pack_tokens(x_local, ids, w)
        self.rec_all = comm.buffer((G * T, self.rec.shape[1]), torch.uint8, dev)
        self.x_all = torch.empty((G * T,) + tuple(x_local.shape[1:]), dtype=x_local.dtype, device=dev)
        self.ids_all = torch.empty((G * T, k), dtype=ids.dtype, device=dev)
        self.w_all = torch.empty((G * T, k), dtype=w.dtype, device=dev)
        comm.all_gather(self.rec, self.rec_all)

        def local_phase():
            if packed:
                return backend.partial_sums_packed(self.rec_all, k, x_local.dtype)
            unpack_tokens(self.rec_all, x_local.shape[1], k, x_local.dtype, self.x_all, self.ids_all, self.w_all)
            return backend.partial_sums(self.x_all, self.ids_all, self.w_all)
        parts, shared = local_phase()
        self.recv = comm.buffer((G, T, parts.shape[1]), parts.dtype, dev)
        comm.all_to_all(parts.view(G, T, -1), self.recv)
        backend.finish(self.recv, shared)
        stream.synchronize()
        self.g_route, self.g_part, self.g_fin = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.g_route, stream=stream):             # route + pack
            self.ids, self.w = backend.route_local(x_local)
            if packed:
                backend.pack_all(x_local, self.ids, self.w, self.rec)
            else:
                pack_tokens(x_local, self.ids, self.w, self.rec)
        with torch.cuda.graph(self.g_part, stream=stream):              # unpack + local experts + partial sums
            self.parts, self.shared = local_phase()
        with torch.cuda.graph(self.g_fin, stream=stream):
            self.out = backend.finish(self.recv, self.shared)

    def __call__(self) -> torch.Tensor:
        c = self.comm
        self.g_route.replay()
        c.all_gather(self.rec, self.rec_all)
        self.g_part.replay()
        c.all_to_all(self.parts.view(c.world, self.x.shape[0], -1), self.recv)
        self.g_fin.replay()
        return self.out
