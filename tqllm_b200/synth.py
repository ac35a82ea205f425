"""Seeded synthetic workloads for the MoE layer: shapes of the five benchmark configurations, weight generators and
this package's own quantisers fp32 -> GGUF block bytes (Q4_K, IQ3_S, IQ4_XS, IQ4_NL, NVFP4G).

The reference ships no quantiser for these types and gguf-py only decodes them, so the encoders here are this
package's own: simple round-to-nearest encoders whose only contract is validity (finite fp16 scale fields, codes in
range, the byte layout ggml defines). The decode side is what is graded; these bytes go unchanged to both the CPU
checker and the CUDA kernels. Everything is torch and runs on whichever device the input lives on.

Block layouts (as decoded by the reference, src/formats/weight/dequant.cpp:80-99, 137-150, 177-192, 352-360, 397-409):
  Q4_K   144 B / 256: d f16, dmin f16, scales[12] (8 x 6-bit scale, 8 x 6-bit min), qs[128]
  IQ3_S  110 B / 256: d f16, qs[64], qh[8], signs[32], scales[4]
  IQ4_XS 136 B / 256: d f16, scales_h u16, scales_l[4], qs[128]
  IQ4_NL  18 B / 32 : d f16, qs[16]
  NVFP4G  76 B / 128: f32 tensor scale, 8 x E4M3 group scales, 64 B of E2M1 pairs
"""
from __future__ import annotations

import dataclasses
import math

import torch

Q4_K, IQ4_NL, IQ3_S, IQ4_XS, NVFP4G = 12, 20, 21, 23, 323
BLOCK = {Q4_K: (256, 144), IQ3_S: (256, 110), IQ4_XS: (256, 136), IQ4_NL: (32, 18), NVFP4G: (128, 76)}
TYPE_NAME = {Q4_K: "Q4_K", IQ3_S: "IQ3_S", IQ4_XS: "IQ4_XS", IQ4_NL: "IQ4_NL", NVFP4G: "NVFP4G"}
SOFTMAX, SIGMOID = 1, 2


def raw_bytes(type_id: int, rows: int, cols: int) -> int:
    elems, nbytes = BLOCK[type_id]
    assert cols % elems == 0, f"{TYPE_NAME[type_id]}: cols {cols} is not a multiple of {elems}"
    return rows * (cols // elems) * nbytes


# ------------------------------------------------------------------------------------------------ codebooks ----
_tables = None


def codebooks():
    """(iq3s_grid int64 [512][4] magnitudes, kvalues_iq4nl int64 [16]) from the build-time table source."""
    global _tables
    if _tables is None:
        from . import gen_tables
        grid, kv = gen_tables.tables()
        g = torch.tensor(grid, dtype=torch.int64)
        _tables = (torch.stack([(g >> (8 * j)) & 255 for j in range(4)], dim=1), torch.tensor(kv, dtype=torch.int64))
    return _tables


_iq3_lut = None


def _iq3s_nearest_lut(device):
    """[8^4] -> index of the nearest IQ3_S grid entry, for four magnitude levels l (magnitude 2l+1)."""
    global _iq3_lut
    if _iq3_lut is None:
        grid, _ = codebooks()
        lv = torch.arange(8)
        combos = torch.stack(torch.meshgrid(lv, lv, lv, lv, indexing="ij"), dim=-1).reshape(-1, 4) * 2 + 1  # [4096][4]
        d = ((combos[:, None, :] - grid[None, :, :]).float() ** 2).sum(-1)
        _iq3_lut = d.argmin(1)
    return _iq3_lut.to(device)


def _f16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16)


def _u8(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.uint8)


def _bytes_of(x: torch.Tensor) -> torch.Tensor:
    """little-endian bytes of each element, appended as a last dim"""
    return x.contiguous().view(torch.uint8).reshape(*x.shape, x.element_size())


# ------------------------------------------------------------------------------------------------ quantisers ----
def quantize_q4k(w: torch.Tensor) -> torch.Tensor:
    rows, cols = w.shape
    x = w.float().reshape(rows, cols // 256, 8, 32)
    mn = (-x.amin(-1)).clamp_min(0)
    rng = x.amax(-1) + mn
    sub = rng / 15
    d = _f16(sub.amax(-1) / 63).float()
    dmin = _f16(mn.amax(-1) / 63).float()
    sc = torch.where(d[..., None] > 0, (sub / d[..., None].clamp_min(1e-30)).round(), torch.zeros_like(sub)).clamp(0, 63)
    m = torch.where(dmin[..., None] > 0, (mn / dmin[..., None].clamp_min(1e-30)).round(), torch.zeros_like(mn)).clamp(0, 63)
    d1 = (d[..., None] * sc)[..., None]
    m1 = (dmin[..., None] * m)[..., None]
    q = torch.where(d1 > 0, ((x + m1) / d1.clamp_min(1e-30)).round(), torch.zeros_like(x)).clamp(0, 15).to(torch.int64)
    sc, m = sc.to(torch.int64), m.to(torch.int64)
    s = torch.empty(rows, cols // 256, 12, dtype=torch.int64, device=w.device)
    s[..., 0:4] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    s[..., 4:8] = m[..., 0:4] | ((m[..., 4:8] >> 4) << 6)
    s[..., 8:12] = (sc[..., 4:8] & 15) | ((m[..., 4:8] & 15) << 4)
    q = q.reshape(rows, cols // 256, 4, 2, 32)
    qs = (q[..., 0, :] | (q[..., 1, :] << 4)).reshape(rows, cols // 256, 128)
    out = torch.cat([_bytes_of(_f16(d)), _bytes_of(_f16(dmin)), _u8(s), _u8(qs)], dim=-1)
    return out.reshape(-1)


def quantize_iq3s(w: torch.Tensor) -> torch.Tensor:
    rows, cols = w.shape
    x = w.float().reshape(rows, cols // 256, 8, 32)
    amax = x.abs().amax(-1)
    db0 = amax / 14.0
    d = _f16(db0.amax(-1) / 31.0).float()
    s4 = torch.where(d[..., None] > 0, ((db0 / d[..., None].clamp_min(1e-30) - 1) / 2).round(), torch.zeros_like(db0)).clamp(0, 15)
    db = (d[..., None] * (1 + 2 * s4))[..., None]
    lv = torch.where(db > 0, ((x.abs() / db.clamp_min(1e-30) - 1) / 2).round(), torch.zeros_like(x)).clamp(0, 7).to(torch.int64)
    lv = lv.reshape(rows, cols // 256, 8, 8, 4)
    key = ((lv[..., 0] * 8 + lv[..., 1]) * 8 + lv[..., 2]) * 8 + lv[..., 3]
    idx = _iq3s_nearest_lut(w.device)[key]                                   # [rows][nb][8][8] 9-bit grid indices
    neg = (x < 0).to(torch.int64).reshape(rows, cols // 256, 8, 8, 4)
    nib = neg[..., 0] | (neg[..., 1] << 1) | (neg[..., 2] << 2) | (neg[..., 3] << 3)       # 4 sign bits per entry
    signs = (nib[..., 0::2] | (nib[..., 1::2] << 4)).reshape(rows, cols // 256, 32)
    qs = (idx & 255).reshape(rows, cols // 256, 64)
    sh = torch.arange(8, device=w.device)
    qh = ((idx >> 8) << sh).sum(-1)                                          # [rows][nb][8]
    s4 = s4.to(torch.int64)
    scales = s4[..., 0::2] | (s4[..., 1::2] << 4)
    out = torch.cat([_bytes_of(_f16(d)), _u8(qs), _u8(qh), _u8(signs), _u8(scales)], dim=-1)
    return out.reshape(-1)


def _iq4_codes(x: torch.Tensor, dl: torch.Tensor) -> torch.Tensor:
    """nearest IQ4_NL table entry of x / dl (dl broadcast over the last dim)"""
    _, kv = codebooks()
    kv = kv.to(x.device).float()
    t = torch.where(dl != 0, x / torch.where(dl != 0, dl, torch.ones_like(dl)), torch.zeros_like(x))
    mid = (kv[1:] + kv[:-1]) / 2
    return torch.bucketize(t.contiguous(), mid)


def _iq4_scale(x: torch.Tensor) -> torch.Tensor:
    """per last-dim block: the scale that maps the largest-magnitude element onto the table's end (-127 or 113)"""
    i = x.abs().argmax(-1, keepdim=True)
    v = x.gather(-1, i).squeeze(-1)
    return torch.where(v < 0, v / -127.0, v / 113.0)


def quantize_iq4nl(w: torch.Tensor) -> torch.Tensor:
    rows, cols = w.shape
    x = w.float().reshape(rows, cols // 32, 32)
    d = _f16(_iq4_scale(x)).float()
    c = _iq4_codes(x, d[..., None])
    qs = c[..., :16] | (c[..., 16:] << 4)
    return torch.cat([_bytes_of(_f16(d)), _u8(qs)], dim=-1).reshape(-1)


def quantize_iq4xs(w: torch.Tensor) -> torch.Tensor:
    rows, cols = w.shape
    x = w.float().reshape(rows, cols // 256, 8, 32)
    sub = _iq4_scale(x)                                                       # >= 0
    d = _f16(sub.amax(-1) / 31.0).float()
    l = torch.where(d[..., None] > 0, (sub / d[..., None].clamp_min(1e-30)).round(), torch.zeros_like(sub)).clamp(0, 31)
    ls = (l + 32).to(torch.int64)
    dl = (d[..., None] * l)[..., None]
    c = _iq4_codes(x, dl.expand_as(x))
    qs = (c[..., :16] | (c[..., 16:] << 4)).reshape(rows, cols // 256, 128)
    sl = (ls[..., 0::2] & 15) | ((ls[..., 1::2] & 15) << 4)
    sh = ((ls >> 4) << (2 * torch.arange(8, device=w.device))).sum(-1)
    shb = torch.stack([sh & 255, sh >> 8], dim=-1)
    return torch.cat([_bytes_of(_f16(d)), _u8(shb), _u8(sl), _u8(qs)], dim=-1).reshape(-1)


def quantize_nvfp4g(w: torch.Tensor) -> torch.Tensor:
    rows, cols = w.shape
    x = w.float().reshape(rows, cols // 128, 8, 16)
    g = (x.abs().amax() / (6.0 * 448.0)).clamp_min(1e-30).float()            # one fp32 scale for the tensor
    sc8 = (x.abs().amax(-1) / (6.0 * g)).clamp(0, 448).to(torch.float8_e4m3fn)
    sc = sc8.float()
    t = torch.where(sc[..., None] > 0, x / (sc[..., None] * g).clamp_min(1e-30), torch.zeros_like(x))
    lv = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], device=w.device)
    mid = (lv[1:] + lv[:-1]) / 2
    code = torch.bucketize(t.abs().contiguous(), mid) | ((t < 0).to(torch.int64) << 3)
    qs = (code[..., 0::2] | (code[..., 1::2] << 4)).reshape(rows, cols // 128, 64)
    gb = _bytes_of(g.reshape(1, 1).expand(rows, cols // 128).contiguous())
    return torch.cat([gb, sc8.view(torch.uint8), _u8(qs)], dim=-1).reshape(-1)


QUANTIZE = {Q4_K: quantize_q4k, IQ3_S: quantize_iq3s, IQ4_XS: quantize_iq4xs, IQ4_NL: quantize_iq4nl, NVFP4G: quantize_nvfp4g}


def quantize(type_id: int, w: torch.Tensor) -> torch.Tensor:
    """fp32 [rows][cols] -> uint8 raw GGUF block bytes, rows contiguous"""
    out = QUANTIZE[type_id](w)
    assert out.numel() == raw_bytes(type_id, *w.shape)
    return out


def random_blocks(type_id: int, blocks: int, gen: torch.Generator, blocks_per_row: int = 1) -> torch.Tensor:
    """Random block bytes with finite, moderate fp16 / scale fields (the reference's test idiom,
    tests/moe_device.cu:121-138): every code pattern occurs, which the quantisers above do not guarantee.
    NVFP4G carries one fp32 tensor scale per row (the reference's loader rejects rows whose blocks disagree,
    src/formats/weight/q4.cpp:512,518), so its blocks need `blocks_per_row`."""
    elems, nbytes = BLOCK[type_id]
    raw = torch.randint(0, 256, (blocks, nbytes), generator=gen, dtype=torch.int64).to(torch.uint8)
    halves = {Q4_K: [0, 2], IQ3_S: [0], IQ4_XS: [0], IQ4_NL: [0], NVFP4G: []}[type_id]
    for off in halves:
        v = (torch.rand(blocks, generator=gen) * 4.9e-2 + 1e-3) * (torch.randint(0, 2, (blocks,), generator=gen) * 2 - 1)
        raw[:, off:off + 2] = _bytes_of(v.to(torch.float16))
    if type_id == NVFP4G:
        assert blocks % blocks_per_row == 0
        g = torch.rand(blocks // blocks_per_row, generator=gen) * 1e-3 + 1e-5
        raw[:, 0:4] = _bytes_of(g.float().repeat_interleave(blocks_per_row))
        sc = raw[:, 4:12]
        sc[(sc & 0x7F) == 0x7F] = 0x38                                       # no E4M3 NaN
    return raw.reshape(-1)


# ------------------------------------------------------------------------------------------------ configs ----
@dataclasses.dataclass
class LayerShape:
    name: str
    hidden: int
    experts: int
    topk: int
    ff: int
    gating: int = SOFTMAX
    norm: bool = True
    scale: float = 0.0
    shared: bool = False
    types: tuple = (Q4_K, Q4_K, Q4_K)          # gate, up, down GGUF ids
    sel_bias: bool = False
    act_dtype: str = "bf16"                    # dtype of the activations handed to the layer

    def expert_bytes(self) -> int:
        """GGUF block bytes of one expert's gate + up + down: the unit the HBM roofline counts"""
        return raw_bytes(self.types[0], self.ff, self.hidden) + raw_bytes(self.types[1], self.ff, self.hidden) + \
            raw_bytes(self.types[2], self.hidden, self.ff)


CONFIGS = {
    "c1": LayerShape("c1-q4k-h1024-e32-k4-f512", 1024, 32, 4, 512, types=(Q4_K, Q4_K, Q4_K), act_dtype="f32"),
    "c2": LayerShape("c2-flashnext-iq3s-h2048-e512-k10-f512", 2048, 512, 10, 512, shared=True, types=(IQ3_S,) * 3),
    "c3": LayerShape("c3-flashnext-nvfp4-h2048-e512-k10-f512", 2048, 512, 10, 512, shared=True, types=(NVFP4G,) * 3),
    "c4": LayerShape("c4-minimax-q4k-h3072-e256-k8-f1536", 3072, 256, 8, 1536, gating=SIGMOID, sel_bias=True,
                     types=(Q4_K,) * 3),
    "c5": LayerShape("c5-glm-iq4xs-h4096-e128-k8-f1408", 4096, 128, 8, 1408, types=(IQ4_XS, IQ4_XS, IQ4_NL)),
}


@dataclasses.dataclass
class Layer:
    shape: LayerShape
    router_w: torch.Tensor                     # f32 [E][H]
    sel_bias: torch.Tensor | None              # f32 [E]
    raw: tuple                                 # (gate, up, down) uint8 raw blocks of the stacked experts
    shared_raw: tuple | None                   # (gate, up, down) of the always-on expert


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def make_layer(shape: LayerShape, seed: int, device="cpu", experts: int | None = None, router_scale: float = 1.0,
               zipf: float = 0.0, chunk_experts: int = 16) -> Layer:
    """Weights N(0, 0.02) quantised expert by expert (chunked so a 512-expert layer fits beside its fp32 source).
    `experts` overrides the expert count (small parity cases); `router_scale` multiplies the router weight (c2: solved
    so the top-k softmax mass is about 0.6); `zipf` adds log(rank^-s)-shaped selection pressure through the router bias
    row handled by the caller."""
    E = experts or shape.experts
    H, F = shape.hidden, shape.ff
    g = _gen(seed, device)
    router = torch.randn(E, H, generator=g, device=device) * 0.02 * router_scale
    bias = (torch.randn(E, generator=g, device=device) * 0.1) if shape.sel_bias else None

    def stack(type_id, rows, cols, n):
        parts = []
        for e0 in range(0, n, chunk_experts):
            m = min(chunk_experts, n - e0)
            w = torch.randn(m * rows, cols, generator=g, device=device) * 0.02
            parts.append(quantize(type_id, w))
        return torch.cat(parts)

    raw = (stack(shape.types[0], F, H, E), stack(shape.types[1], F, H, E), stack(shape.types[2], H, F, E))
    shared = None
    if shape.shared:
        shared = (stack(shape.types[0], F, H, 1), stack(shape.types[1], F, H, 1), stack(shape.types[2], H, F, 1))
    return Layer(shape, router, bias, raw, shared)


def permute_experts(layer: Layer, order) -> Layer:
    """The same layer with its experts stacked in `order` (order[i] = the expert that takes position i): router rows,
    selection bias and the raw blocks of the three banks move together, so the layer computes the same function and a
    routed id i now means the former expert order[i]. Used to apply a load-aware placement (b2moe_place_experts)."""
    shape = layer.shape
    order = torch.as_tensor(order, dtype=torch.long, device=layer.router_w.device)
    E = layer.router_w.shape[0]
    assert sorted(order.tolist()) == list(range(E))
    H, F = shape.hidden, shape.ff
    raws = []
    for i, (rows, cols) in enumerate(((F, H), (F, H), (H, F))):
        per = raw_bytes(shape.types[i], rows, cols)
        raws.append(layer.raw[i].view(E, per)[order].reshape(-1).contiguous())
    return Layer(shape, layer.router_w[order].contiguous(), None if layer.sel_bias is None else layer.sel_bias[order].contiguous(),
                 tuple(raws), layer.shared_raw)


def make_tokens(shape: LayerShape, tokens: int, seed: int, device="cpu") -> torch.Tensor:
    """activations N(0,1); rounded to bf16 (and returned as bf16) unless the config feeds fp32"""
    g = _gen(seed ^ 0x5DEECE66D, device)
    x = torch.randn(tokens, shape.hidden, generator=g, device=device)
    return x if shape.act_dtype == "f32" else x.to(torch.bfloat16)


def solve_router_scale(shape: LayerShape, target_mass: float = 0.6, seed: int = 7) -> float:
    """Scale s of the router weight N(0, 0.02 s) for which the mean top-k softmax mass over N(0,1) tokens is
    `target_mass` (bisection on the CPU; logits are then N(0, 0.02 s sqrt(H)))."""
    g = _gen(seed, "cpu")
    z = torch.randn(512, shape.experts, generator=g)
    sigma0 = 0.02 * math.sqrt(shape.hidden)
    lo, hi = 0.01, 100.0
    for _ in range(40):
        mid = math.sqrt(lo * hi)
        mass = torch.softmax(z * sigma0 * mid, -1).topk(shape.topk, -1).values.sum(-1).mean().item()
        lo, hi = (mid, hi) if mass < target_mass else (lo, mid)
    return math.sqrt(lo * hi)
