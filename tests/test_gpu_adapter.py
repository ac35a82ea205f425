"""GPU: the WeightFormat adapter driven through the reference's own interface (tests/adapter_driver.cpp, built against the
reference's weight_format.hpp / moe_kernels.cuh by tests/adapter_build.py where that checkout exists; the built program
travels with the tree). Protocol of the reference's device test of this interface (tests/moe_device.cu:117-219): grouped
calls against per-row fp32 references, expert_gemm* equal to expert_matvec*, a row slice of the stacked bank used as a
matrix of its own, n in {1, 5, 17}, -1 ids skipped. Outputs are bf16 / fp16 as in the reference, so the bound is the
rounding of the output type on top of the layer tolerance."""
import os
import struct
import subprocess

import numpy as np
import pytest
import torch

import adapter_build
from tqllm_b200 import synth

pytestmark = pytest.mark.gpu
DRIVER = adapter_build.DRIVER


def bf16_to_f32(a):
    return (a.astype(np.uint32) << 16).view(np.float32)


@pytest.mark.skipif(not os.path.isfile(DRIVER), reason="adapter driver not built (needs the reference checkout at build time)")
@pytest.mark.parametrize("type_id,codes,experts,rows,cols,n,topk", ((21, 1, 6, 80, 512, 5, 3), (21, 0, 4, 48, 256, 1, 2), (12, 0, 5, 64, 768, 17, 2),
                                                                       (23, 0, 3, 32, 256, 5, 2), (323, 0, 4, 32, 256, 17, 3)))
def test_adapter_calls_match_fp32_references(orc, tmp_path, type_id, codes, experts, rows, cols, n, topk):
    g = torch.Generator()
    g.manual_seed(1000 + n + type_id)
    wg = torch.randn(experts * rows, cols, generator=g) * 0.05
    wu = torch.randn(experts * rows, cols, generator=g) * 0.05
    raw_g, raw_u = synth.quantize(type_id, wg).numpy(), synth.quantize(type_id, wu).numpy()
    A = n * topk
    x = (torch.randn(n, cols, generator=g)).to(torch.float16).numpy()
    xa = (torch.randn(A, cols, generator=g)).to(torch.float16).numpy()
    ids = torch.stack([torch.randperm(experts, generator=g)[:topk] for _ in range(n)]).to(torch.int32).numpy()
    if A > 3:
        ids.reshape(-1)[2] = -1                                   # a skipped assignment
    w = torch.rand(n, topk, generator=g).numpy().astype(np.float32)
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(fin, "wb") as f:
        f.write(struct.pack("8i", type_id, experts, rows, cols, n, topk, codes, 0))
        for a in (raw_g, raw_u, x, xa, ids, w):
            f.write(np.ascontiguousarray(a).tobytes())
    r = subprocess.run([DRIVER, str(fin), str(fout)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    buf = open(fout, "rb").read()
    off = 0

    def take(count, dt):
        nonlocal off
        a = np.frombuffer(buf, dt, count, off)
        off += a.nbytes
        return a
    flags = take(4, np.int32)
    assert flags[0] == 1 and flags[1] == 1
    assert flags[3] == 1, "moe_topk2 differs from two moe_topk calls"
    pick = int(flags[2])
    u16 = lambda c: take(c, np.uint16)
    y_tok, y_pei, yg, yu = (bf16_to_f32(u16(A * rows)).reshape(A, rows) for _ in range(4))
    act2 = u16(A * rows).view(np.float16).astype(np.float32).reshape(A, rows)
    y_gemm = bf16_to_f32(u16(A * rows)).reshape(A, rows)
    act_f = u16(A * rows).view(np.float16).astype(np.float32).reshape(A, rows)
    ssum = bf16_to_f32(u16(n * rows)).reshape(n, rows)
    y_dense = bf16_to_f32(u16(n * rows)).reshape(n, rows)
    deq = u16(rows * cols).view(np.float16).astype(np.float32).reshape(rows, cols)
    threw = take(1, np.int32)[0]
    assert threw == 1
    # fp64 references from the oracle's exact dequantisation
    Wg = orc.dequant(type_id, raw_g, experts * rows * cols).reshape(experts, rows, cols).astype(np.float64)
    Wu = orc.dequant(type_id, raw_u, experts * rows * cols).reshape(experts, rows, cols).astype(np.float64)
    xf, xaf = x.astype(np.float64), xa.astype(np.float64)
    flat = ids.reshape(-1)
    live = flat >= 0
    ref_g = np.stack([Wg[max(e, 0)] @ xf[a // topk] for a, e in enumerate(flat)])
    ref_u = np.stack([Wu[max(e, 0)] @ xf[a // topk] for a, e in enumerate(flat)])
    ref_pei = np.stack([Wu[max(e, 0)] @ xaf[a] for a, e in enumerate(flat)])

    def close(got, want, tol=2e-2, rel=2.0 ** -7):
        """the layer tolerance on the RMS plus the rounding of the bf16 / fp16 rows the reference's interface prescribes"""
        rms = max(np.sqrt((want[live] ** 2).mean()), 1e-30)
        excess = np.abs(got[live] - want[live]) - rel * np.abs(want[live])
        assert excess.max() <= tol * rms, excess.max() / rms
    close(y_tok, ref_g); close(yg, ref_g); close(yu, ref_u); close(y_pei, ref_pei); close(y_gemm, ref_g)
    assert np.array_equal(y_tok[live], yg[live]) and np.array_equal(y_tok[live], y_gemm[live])     # one kernel, three ways in
    # skipped rows stay as the caller left them (filled with 0x7f7f = a large bf16 marker)
    assert np.all(y_tok[~live] > 1e30) if (~live).any() else True
    silu = lambda v: v / (1 + np.exp(-v))
    close(act_f, silu(ref_g) * ref_u, 3e-2)
    close(act2, silu(ref_g) * ref_u, 3e-2)                       # the unfused route rounds gate and up to bf16 first
    # moe_sum: weighted rows of the live assignments (the marker rows carry weight only where skipped: mask them)
    yt = np.where(live[:, None], y_tok, 0.0).reshape(n, topk, rows)
    wm = np.where(live.reshape(n, topk), w, 0.0)
    if live.all():
        want = (wm[:, :, None] * yt).sum(1)
        assert np.abs(ssum - want).max() <= 2e-2 * max(np.sqrt((want ** 2).mean()), 1e-30)
    # a row slice of the stacked bank is a matrix of its own: dense matvec of expert `pick` for every token, and its dequant
    want_dense = xf @ Wg[pick].T
    assert np.abs(y_dense - want_dense).max() <= 2e-2 * np.sqrt((want_dense ** 2).mean())
    assert np.abs(deq - Wg[pick]).max() <= 2 ** -10 * np.abs(Wg[pick]).max()
    for a, e in enumerate(flat):
        if e == pick:
            assert np.array_equal(y_tok[a], y_dense[a // topk])    # grouped == row-sliced, bit for bit
