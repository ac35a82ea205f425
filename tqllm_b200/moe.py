"""Host-side harness over the C ABI: torch tensors own the device memory, every computation goes through libb2moe.so.

This is the Python mirror used by the tests and the benchmark; tqLLM itself binds the same C ABI from C++ through the
adapter in tqllm_b200/adapter/. Names follow the reference's: banks of stacked experts, routing ids / weights, the
dispatch plan (counts, offsets, permutation), the layer forward.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import capi
from .capi import check, lib

_DT = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


class DeviceBank:
    """One stacked expert matrix [experts * rows][cols] in bank layout on the device."""

    def __init__(self, type_id: int, raw: torch.Tensor, experts: int, rows: int, cols: int):
        assert raw.is_cuda and raw.dtype == torch.uint8
        if raw.numel() != experts * lib.b2moe_raw_bytes(type_id, rows, cols) or raw.numel() == 0:
            raise capi.B2moeError(capi.ERR_SHAPE, "DeviceBank: raw byte count does not match the shape")
        self.type, self.experts, self.rows, self.cols = type_id, experts, rows, cols
        self.data = torch.empty(experts * lib.b2moe_bank_bytes(type_id, rows, cols), dtype=torch.uint8, device=raw.device)
        aux_bytes = lib.b2moe_bank_aux_bytes(type_id, rows, cols)
        self.aux = torch.empty(experts * aux_bytes // 4, dtype=torch.float32, device=raw.device) if aux_bytes else None
        check(lib.b2moe_bank_load(type_id, raw.data_ptr(), experts, rows, cols, self.data.data_ptr(), _ptr(self.aux), _stream()),
              "b2moe_bank_load")
        self.c = capi.Bank(self.data.data_ptr(), _ptr(self.aux), type_id, experts, rows, cols)

    @classmethod
    def from_packed(cls, type_id: int, data, aux, experts: int, rows: int, cols: int, device="cuda"):
        """a bank that was packed on the host (b2moe_bank_pack_host, b2moe_gguf_expert_bank): one upload, no device repack"""
        self = cls.__new__(cls)
        self.type, self.experts, self.rows, self.cols = type_id, experts, rows, cols
        if len(data) != lib.b2moe_bank_bytes(type_id, experts * rows, cols):
            raise capi.B2moeError(capi.ERR_SHAPE, "DeviceBank.from_packed: byte count does not match the shape")
        self.data = torch.as_tensor(data).to(device)
        self.aux = None if aux is None else torch.as_tensor(aux).to(device)
        self.c = capi.Bank(self.data.data_ptr(), _ptr(self.aux), type_id, experts, rows, cols)
        return self

    def dequant(self) -> torch.Tensor:
        out = torch.empty(self.experts * self.rows, self.cols, dtype=torch.float32, device=self.data.device)
        check(lib.b2moe_dequant_dump(C.byref(self.c), out.data_ptr(), _stream()), "b2moe_dequant_dump")
        return out


def router(router_w, x, shared_gate=None, ld=None):
    n, h = x.shape
    e = router_w.shape[0]
    ld = ld or e + 1
    logits = torch.zeros(n, ld, dtype=torch.float32, device=x.device)
    check(lib.b2moe_router(router_w.data_ptr(), _ptr(shared_gate), x.data_ptr(), _DT[x.dtype], logits.data_ptr(), ld, h, e, n, _stream()),
          "b2moe_router")
    return logits


def topk_softmax(logits, experts, k, scale=0.0, shared=False):
    n, ld = logits.shape
    ids = torch.empty(n, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(n, k, dtype=torch.float32, device=logits.device)
    sw = torch.empty(n, dtype=torch.float32, device=logits.device) if shared else None
    check(lib.b2moe_topk_softmax(logits.data_ptr(), ld, ids.data_ptr(), w.data_ptr(), _ptr(sw), experts, k, n, scale, _stream()),
          "b2moe_topk_softmax")
    return ids, w, sw



def topk_softmax2(logits, logits2, experts, k, scale=0.0, shared=False):
    """Two routings of the same tokens in one launch (the reference's moe_topk2): returns ((ids, w, sw), (ids2, w2, sw2))."""
    n, ld = logits.shape
    assert logits2.shape == logits.shape
    out = []
    for _ in range(2):
        out.append((torch.empty(n, k, dtype=torch.int32, device=logits.device), torch.empty(n, k, dtype=torch.float32, device=logits.device),
                    torch.empty(n, dtype=torch.float32, device=logits.device) if shared else None))
    (i1, w1, s1), (i2, w2, s2) = out
    check(lib.b2moe_topk_softmax2(logits.data_ptr(), i1.data_ptr(), w1.data_ptr(), _ptr(s1), logits2.data_ptr(), i2.data_ptr(), w2.data_ptr(),
                                  _ptr(s2), ld, experts, k, n, scale, _stream()), "b2moe_topk_softmax2")
    return out

def route_sigmoid(logits, experts, k, bias=None, norm=True, scale=0.0):
    n, ld = logits.shape
    ids = torch.empty(n, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(n, k, dtype=torch.float32, device=logits.device)
    check(lib.b2moe_route_sigmoid(logits.data_ptr(), ld, _ptr(bias), ids.data_ptr(), w.data_ptr(), experts, k, int(norm), scale, n,
                                  _stream()), "b2moe_route_sigmoid")
    return ids, w


def count_ids(ids: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """counts[e] += occurrences of e in ids (the reference's moe_count): counts is an int64 device tensor [experts]"""
    assert counts.dtype == torch.int64 and ids.dtype == torch.int32
    check(lib.b2moe_count(ids.data_ptr(), counts.data_ptr(), ids.numel(), counts.numel(), _stream()), "b2moe_count")
    return counts


def place_experts(counts, ranks: int):
    """Load-aware placement from a routing histogram: (order, rank_load) with order[r * per + i] = the expert in slot i of
    rank r (host arithmetic, b2moe_place_experts); feed `order` to synth.permute_experts or the loader's equivalent."""
    import numpy as np
    c = np.ascontiguousarray(np.asarray(counts.cpu() if hasattr(counts, "cpu") else counts), dtype=np.uint64)
    order = np.empty(c.size, np.int32)
    load = np.empty(ranks, np.uint64)
    check(lib.b2moe_place_experts(c.ctypes.data, c.size, ranks, order.ctypes.data, load.ctypes.data), "b2moe_place_experts")
    return order, load


class Plan:
    """Device dispatch plan with views of its arrays."""

    def __init__(self, experts: int, n: int, topk: int, shared_tokens: int, device):
        self.experts, self.n, self.topk, self.shared_tokens = experts, n, topk, shared_tokens
        v = capi.PlanView()
        lib.b2moe_plan_view_of(experts, n * topk, shared_tokens, C.byref(v))
        self.view = v
        self.buf = torch.zeros(v.total, dtype=torch.int32, device=device)

    @property
    def n_active(self): return int(self.buf[0])
    @property
    def counts(self): return self.buf[self.view.counts:self.view.counts + self.experts + 1]
    @property
    def offsets(self): return self.buf[self.view.offsets:self.view.offsets + self.experts + 2]
    @property
    def active(self): return self.buf[self.view.active:self.view.active + self.experts + 1]
    @property
    def perm(self): return self.buf[self.view.perm:self.view.passes]
    @property
    def passes(self): return self.buf[self.view.passes:self.view.total]


def dispatch(ids: torch.Tensor, experts: int, shared_tokens: int = 0) -> Plan:
    n, k = ids.shape
    plan = Plan(experts, n, k, shared_tokens, ids.device)
    wsb = lib.b2moe_dispatch_workspace_bytes(experts, n * k)
    ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=ids.device)
    check(lib.b2moe_dispatch(ids.data_ptr(), n, k, experts, shared_tokens, plan.buf.data_ptr(), ws.data_ptr(), ws.numel(), _stream()),
          "b2moe_dispatch")
    return plan


def plan_to_groups(plan: Plan):
    counts = torch.zeros(plan.experts, dtype=torch.int32, device=plan.buf.device)
    groups = torch.full((plan.experts, plan.n), -1, dtype=torch.int32, device=plan.buf.device)
    check(lib.b2moe_plan_to_groups(plan.buf.data_ptr(), plan.n, plan.topk, plan.experts, counts.data_ptr(), groups.data_ptr(), _stream()),
          "b2moe_plan_to_groups")
    return counts, groups


def _scratch(nbytes: int, device):
    return torch.empty(nbytes, dtype=torch.uint8, device=device) if nbytes else None


def _bref(b: DeviceBank | None):
    return C.byref(b.c) if b is not None else None


def expert_gateup_swiglu(gate, up, x, plan: Plan, sh_gate=None, sh_up=None):
    total = plan.n * plan.topk + plan.shared_tokens
    act = torch.zeros(total, gate.rows, dtype=torch.float32, device=x.device)
    ws = _scratch(lib.b2moe_expert_workspace_bytes(gate.type, plan.n, gate.cols, _DT[x.dtype]), x.device)
    check(lib.b2moe_expert_gateup_swiglu(_bref(gate), _bref(up), _bref(sh_gate), _bref(sh_up), x.data_ptr(), _DT[x.dtype],
                                         plan.buf.data_ptr(), plan.n, plan.topk, plan.shared_tokens, act.data_ptr(),
                                         _ptr(ws), 0 if ws is None else ws.numel(), _stream()), "b2moe_expert_gateup_swiglu")
    return act


def expert_down(down, act, plan: Plan, sh_down=None):
    y = torch.zeros(act.shape[0], down.rows, dtype=torch.float32, device=act.device)
    ws = _scratch(lib.b2moe_expert_workspace_bytes(down.type, act.shape[0], down.cols, capi.F32), act.device)
    check(lib.b2moe_expert_down(_bref(down), _bref(sh_down), act.data_ptr(), plan.buf.data_ptr(), plan.n, plan.topk,
                                plan.shared_tokens, y.data_ptr(), _ptr(ws), 0 if ws is None else ws.numel(), _stream()),
          "b2moe_expert_down")
    return y


def combine(y, weights, n, topk, hidden, shared_tokens=0, shared_weights=None, ids=None, out_dtype=torch.float32):
    out = torch.empty(n, hidden, dtype=out_dtype, device=y.device)
    check(lib.b2moe_combine(y.data_ptr(), _ptr(ids), weights.data_ptr(), _ptr(shared_weights), n, topk, hidden, shared_tokens,
                            out.data_ptr(), _DT[out_dtype], _stream()), "b2moe_combine")
    return out


class MoeLayer:
    """A resident MoE layer: router weight, expert banks (+ shared expert), and a workspace sized for `max_tokens`."""

    def __init__(self, shape, router_w, raw, shared_raw=None, sel_bias=None, shared_gate_vec=None, experts=None,
                 device="cuda", iq3s_layout="codes"):
        """iq3s_layout: "codes" loads IQ3_S blocks into the 4-bit-code bank layout (capi.IQ3_S_X4: 21.8 % more HBM, decode
        kernels without a codebook lookup), "gguf" into the layout of the GGUF block size."""
        E = experts or shape.experts
        self.shape, self.experts, self.device = shape, E, torch.device(device)
        H, F = shape.hidden, shape.ff
        dev = lambda t: None if t is None else t.to(self.device).contiguous()
        self.router_w, self.sel_bias, self.shared_gate_vec = dev(router_w), dev(sel_bias), dev(shared_gate_vec)
        assert iq3s_layout in ("codes", "gguf")
        tg, tu, td = (capi.IQ3_S_X4 if (t == capi.IQ3_S and iq3s_layout == "codes") else t for t in shape.types)
        self.gate = DeviceBank(tg, dev(raw[0]), E, F, H)
        self.up = DeviceBank(tu, dev(raw[1]), E, F, H)
        self.down = DeviceBank(td, dev(raw[2]), E, H, F)
        self.sh = None
        if shared_raw is not None:
            self.sh = (DeviceBank(tg, dev(shared_raw[0]), 1, F, H), DeviceBank(tu, dev(shared_raw[1]), 1, F, H),
                       DeviceBank(td, dev(shared_raw[2]), 1, H, F))
        self._finish()

    def _finish(self):
        shape, E, H, F = self.shape, self.experts, self.shape.hidden, self.shape.ff
        L = capi.Layer()
        L.hidden, L.experts, L.topk, L.ff = H, E, shape.topk, F
        L.gating, L.norm, L.scale, L.has_shared = shape.gating, int(shape.norm), shape.scale, int(self.sh is not None)
        L.router_w, L.sel_bias, L.shared_gate_vec = _ptr(self.router_w), _ptr(self.sel_bias), _ptr(self.shared_gate_vec)
        L.gate, L.up, L.down = self.gate.c, self.up.c, self.down.c
        if self.sh:
            L.sh_gate, L.sh_up, L.sh_down = self.sh[0].c, self.sh[1].c, self.sh[2].c
        self.c = L
        self.ws, self.ws_view, self.ws_tokens = None, None, 0

    @classmethod
    def from_gguf(cls, path, shape, layer_index=0, first_expert=0, experts=None, device="cuda", iq3s_layout="codes"):
        """Experts [first_expert, first_expert + experts) of layer `layer_index` of a GGUF checkpoint (tensor names
        blk.N.ffn_{gate,up,down}_exps.weight, router blk.N.ffn_gate_inp.weight, optional blk.N.ffn_{gate,up,down}_shexp.weight):
        the banks are packed on the host by the library's reader and uploaded once."""
        import numpy as np
        from . import gguf
        pre = f"blk.{layer_index}."
        with gguf.GgufExperts(path) as g:
            names = g.names()
            t, (h, e_all, _), off, _ = g.tensor(pre + "ffn_gate_inp.weight")
            assert t == 0 and h == shape.hidden, "router must be an F32 [hidden, experts] tensor"
            E = experts or e_all - first_expert
            router = np.array(np.memmap(path, np.float32, "r", off, (e_all, h))[first_expert:first_expert + E])
            codes = iq3s_layout == "codes"
            banks = [g.expert_bank(pre + f"ffn_{m}_exps.weight", first_expert, E, codes) for m in ("gate", "up", "down")]
            shared = None
            if pre + "ffn_gate_shexp.weight" in names:
                shared = [g.expert_bank(pre + f"ffn_{m}_shexp.weight", 0, 1, codes) for m in ("gate", "up", "down")]
        self = cls.__new__(cls)
        self.shape, self.experts, self.device = shape, E, torch.device(device)
        self.router_w, self.sel_bias, self.shared_gate_vec = torch.from_numpy(router).to(device), None, None
        mk = lambda b, n: DeviceBank.from_packed(b[0], b[3], b[4], n, b[1], b[2], device)
        self.gate, self.up, self.down = (mk(b, E) for b in banks)
        self.sh = tuple(mk(b, 1) for b in shared) if shared else None
        self._finish()
        return self

    @classmethod
    def from_synth(cls, layer, device="cuda", experts=None, shared_gate_vec=None, iq3s_layout="codes"):
        return cls(layer.shape, layer.router_w, layer.raw, layer.shared_raw, layer.sel_bias, shared_gate_vec,
                   experts=experts or layer.router_w.shape[0], device=device, iq3s_layout=iq3s_layout)

    def reserve(self, n: int):
        if self.ws is not None and self.ws_tokens == n:
            return
        v = capi.LayerWs()
        check(lib.b2moe_layer_workspace(C.byref(self.c), n, C.byref(v)), "b2moe_layer_workspace")
        self.ws = torch.zeros(v.total, dtype=torch.uint8, device=self.device)
        self.ws_view, self.ws_tokens = v, n

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None, out_dtype=torch.float32, residual: torch.Tensor | None = None) -> torch.Tensor:
        """out = layer(x), or residual + layer(x) when a residual [n][hidden] of the output's dtype is given (it may be `out`)"""
        n = x.shape[0]
        self.reserve(n)
        if out is None:
            out = torch.empty(n, self.shape.hidden, dtype=out_dtype if residual is None else residual.dtype, device=self.device)
        if residual is None:
            check(lib.b2moe_layer_forward(C.byref(self.c), x.data_ptr(), _DT[x.dtype], n, out.data_ptr(), _DT[out.dtype],
                                          self.ws.data_ptr(), self.ws.numel(), _stream()), "b2moe_layer_forward")
        else:
            assert residual.dtype == out.dtype and residual.shape == out.shape
            check(lib.b2moe_layer_forward_residual(C.byref(self.c), x.data_ptr(), _DT[x.dtype], n, residual.data_ptr(), out.data_ptr(),
                                                   _DT[out.dtype], self.ws.data_ptr(), self.ws.numel(), _stream()), "b2moe_layer_forward_residual")
        return out

    def artefacts(self) -> dict:
        """The routing / dispatch intermediates of the last forward, read back from the workspace."""
        v, n, k, E = self.ws_view, self.ws_tokens, self.shape.topk, self.experts

        def view(off, count, dtype):
            return self.ws[off:off + count * 4].view(dtype)

        pv = capi.PlanView()
        sh = n if self.sh else 0
        lib.b2moe_plan_view_of(E, n * k, sh, C.byref(pv))
        plan = view(v.plan, pv.total, torch.int32)
        return dict(
            logits=view(v.logits, n * (E + 1), torch.float32).reshape(n, E + 1),
            ids=view(v.ids, n * k, torch.int32).reshape(n, k),
            weights=view(v.weights, n * k, torch.float32).reshape(n, k),
            shared_weights=view(v.shared_weights, n, torch.float32),
            n_active=int(plan[0]),
            counts=plan[pv.counts:pv.counts + E + 1], offsets=plan[pv.offsets:pv.offsets + E + 2],
            active=plan[pv.active:pv.active + E + 1], perm=plan[pv.perm:pv.passes], passes=plan[pv.passes:pv.total],
            status=int(plan[3]),
            act=view(v.act, (n * k + sh) * self.shape.ff, torch.float32).reshape(n * k + sh, self.shape.ff),
            y=view(v.y, (n * k + sh) * self.shape.hidden, torch.float32).reshape(n * k + sh, self.shape.hidden),
        )
