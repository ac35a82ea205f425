"""CPU stand-in for the three compute phases of tqllm_b200.ep (route_local / partial_sums / finish), built on the
oracle: it lets the gloo tests run the real expert-parallel orchestration and exchanges without a GPU. Test code."""
import numpy as np
import torch

import oracle
from tqllm_b200 import ep, synth


def slice_raw(raw, type_id, rows, cols, first, count):
    b = synth.raw_bytes(type_id, rows, cols)
    return raw[first * b:(first + count) * b]


class OracleEpBackend:
    def __init__(self, shape, layer, experts_total, world, rank, shared_gate_vec=None):
        self.orc = oracle.oracle()
        self.gate_vec = None if shared_gate_vec is None else shared_gate_vec.numpy().astype(np.float32)
        self.shape, self.layer, self.E, self.world, self.rank = shape, layer, experts_total, world, rank
        self.first, self.count = ep.expert_range(experts_total, world, rank)
        H, F = shape.hidden, shape.ff
        tg, tu, td = shape.types
        self.w = []
        for e in range(self.first, self.first + self.count):
            g = self.orc.dequant(tg, slice_raw(layer.raw[0], tg, F, H, e, 1).numpy(), F * H).reshape(F, H)
            u = self.orc.dequant(tu, slice_raw(layer.raw[1], tu, F, H, e, 1).numpy(), F * H).reshape(F, H)
            d = self.orc.dequant(td, slice_raw(layer.raw[2], td, H, F, e, 1).numpy(), H * F).reshape(H, F)
            self.w.append((g, u, d))
        self.sh = None
        if layer.shared_raw is not None:
            self.sh = (self.orc.dequant(tg, layer.shared_raw[0].numpy(), F * H).reshape(F, H),
                       self.orc.dequant(tu, layer.shared_raw[1].numpy(), F * H).reshape(F, H),
                       self.orc.dequant(td, layer.shared_raw[2].numpy(), H * F).reshape(H, F))

    def route_local(self, x):
        logits = self.orc.router_logits(self.layer.router_w.numpy(), x.float().numpy())
        bias = None if self.layer.sel_bias is None else self.layer.sel_bias.numpy()
        ids, w = self.orc.route(self.shape.gating, logits, self.shape.topk, self.shape.norm, self.shape.scale, bias)
        return torch.from_numpy(ids), torch.from_numpy(w)

    def partial_sums(self, x_all, ids_all, w_all):
        xs, ids, w = x_all.float().numpy(), ids_all.numpy(), w_all.numpy()
        N, k = ids.shape
        T = N // self.world
        parts = np.zeros((N, self.shape.hidden), np.float32)
        for t in range(N):
            for s in range(k):
                e = ids[t, s] - self.first
                if 0 <= e < self.count:
                    parts[t] += w[t, s] * self.orc.expert_ffn(xs[t], *self.w[e])
        shared = None
        if self.sh is not None:
            shared = np.stack([self.orc.expert_ffn(xs[self.rank * T + t], *self.sh) for t in range(T)])
            if self.gate_vec is not None:          # shared weight = sigmoid(v . x) of the rank's own tokens
                s = xs[self.rank * T:(self.rank + 1) * T] @ self.gate_vec
                shared = shared * (1.0 / (1.0 + np.exp(-s)))[:, None].astype(np.float32)
            shared = torch.from_numpy(shared.astype(np.float32))
        return torch.from_numpy(parts), shared

    def finish(self, recv, shared):
        out = torch.zeros_like(recv[0])
        for r in range(recv.shape[0]):
            out += recv[r]
        if shared is not None:
            out += shared
        return out

    # ---- all-to-all dispatch (numpy restatement of b2moe_ep_peer_lists / pack / unpack / return_reduce) ----
    def peer_lists(self, ids):
        ids = ids.numpy()
        n = ids.shape[0]
        G = self.world
        bounds = [ep.expert_range(self.E, G, p)[0] for p in range(G)] + [self.E]
        counts, pos, lst = np.zeros(G, np.int32), np.full((G, n), -1, np.int32), np.zeros((G, n), np.int32)
        for p in range(G):
            flag = ((ids >= bounds[p]) & (ids < bounds[p + 1])).any(1) | (p == self.rank)
            toks = np.nonzero(flag)[0]
            counts[p] = len(toks)
            pos[p, toks] = np.arange(len(toks))
            lst[p, :len(toks)] = toks
        return torch.from_numpy(counts), torch.from_numpy(pos), torch.from_numpy(lst)

    def pack_records(self, x, ids, w, lst, offsets, records):
        k, H = ids.shape[1], x.shape[1]
        rows = []
        off = offsets.numpy()
        for p in range(self.world):
            for j in range(off[p + 1] - off[p]):
                t = int(lst[p, j])
                rows.append(np.concatenate([x[t].float().numpy(), ids[t].numpy().astype(np.float32), w[t].numpy()]))
        return torch.from_numpy(np.stack(rows).astype(np.float32)) if rows else torch.zeros(0, H + 2 * k)

    def partial_sums_records(self, recv, records, self_off, T):
        k, H = self.shape.topk, self.shape.hidden
        r = recv.numpy()
        xs, ids, w = r[:, :H], r[:, H:H + k].astype(np.int64), r[:, H + k:]
        parts = np.zeros((records, H), np.float32)
        for j in range(records):
            for s in range(k):
                e = ids[j, s] - self.first
                if 0 <= e < self.count:
                    parts[j] += w[j, s] * self.orc.expert_ffn(xs[j], *self.w[e])
        shared = None
        if self.sh is not None:
            own = xs[self_off:self_off + T]
            shared = np.stack([self.orc.expert_ffn(own[t], *self.sh) for t in range(T)])
            if self.gate_vec is not None:
                shared = shared * (1.0 / (1.0 + np.exp(-(own @ self.gate_vec))))[:, None].astype(np.float32)
            shared = torch.from_numpy(shared.astype(np.float32))
        return torch.from_numpy(parts), shared

    def finish_records(self, back, pos, offsets, shared):
        G, T = pos.shape
        out = torch.zeros(T, back.shape[1])
        for t in range(T):
            for p in range(G):
                q = int(pos[p, t])
                if q >= 0:
                    out[t] += back[int(offsets[p]) + q]
        if shared is not None:
            out += shared
        return out
