"""The GGUF expert reader and bank packer (b2moe_gguf_*, host code): a checkpoint written by the package's own minimal
GGUF writer from seeded synthetic experts is opened, listed, sliced per expert and per rank block, and packed into banks
that equal b2moe_bank_pack_host of the same raw rows; broken files and wrong requests are refused."""
import os
import struct

import numpy as np
import pytest
import torch

from tqllm_b200 import capi, gguf, synth
from tqllm_b200.capi import lib


def layer_file(tmp_path, cfg="c1", experts=6, seed=3):
    shape = synth.CONFIGS[cfg]
    layer = synth.make_layer(shape, seed, experts=experts)
    H, F = shape.hidden, shape.ff
    names = ("blk.0.ffn_gate_exps.weight", "blk.0.ffn_up_exps.weight", "blk.0.ffn_down_exps.weight")
    dims = ((H, F, experts), (H, F, experts), (F, H, experts))
    tensors = [("blk.0.ffn_gate_inp.weight", 0, (H, experts), layer.router_w.numpy().tobytes())]
    tensors += [(n, shape.types[i], dims[i], layer.raw[i].numpy().tobytes()) for i, n in enumerate(names)]
    path = str(tmp_path / "layer.gguf")
    gguf.write_gguf(path, tensors, kv=(("general.architecture", "synthetic-moe"), ("synthetic.expert_count", experts),
                                       ("synthetic.rope_scale", 1.5), ("synthetic.list", [1, 2, 3])))
    return path, shape, layer, names, dims


@pytest.mark.parametrize("cfg", ("c1", "c2", "c5"))
def test_slices_and_banks_match_the_raw_rows(tmp_path, cfg):
    experts = 6
    path, shape, layer, names, dims = layer_file(tmp_path, cfg, experts)
    with gguf.GgufExperts(path) as g:
        assert g.names() == ["blk.0.ffn_gate_inp.weight", *names]
        t, d, off, nb = g.tensor("blk.0.ffn_gate_inp.weight")
        assert t == 0 and d == (shape.hidden, experts, 1) and nb == 0          # F32 is not an expert block format
        for i, n in enumerate(names):
            raw = layer.raw[i].numpy()
            t, d, off, nb = g.tensor(n)
            assert t == shape.types[i] and d == dims[i] and nb == raw.size and off % 32 == 0
            per = raw.size // experts
            for e in (0, experts - 1):
                tt, rows, cols, view = g.expert_slice(n, e)
                assert (tt, rows, cols) == (t, dims[i][1], dims[i][0])
                assert np.array_equal(view, raw[e * per:(e + 1) * per])
            # a rank's block of experts -> a finished bank, in both IQ3_S layouts where that applies
            first, count = 2, 3
            for codes in ((True, False) if t == 21 else (True,)):
                bank_type, rows, cols, data, aux = g.expert_bank(n, first, count, iq3s_as_codes=codes)
                want = np.empty_like(data)
                waux = np.empty_like(aux) if aux is not None else None
                block = np.ascontiguousarray(raw[first * per:(first + count) * per])
                assert lib.b2moe_bank_pack_host(bank_type, block.ctypes.data, count, rows, cols, want.ctypes.data,
                                                waux.ctypes.data if waux is not None else None) == 0
                assert np.array_equal(data, want) and (aux is None or np.array_equal(aux, waux))
                assert bank_type == (capi.IQ3_S_X4 if (t == 21 and codes) else t)


def test_wrong_requests_and_broken_files_are_refused(tmp_path):
    import ctypes as C
    path, shape, layer, names, dims = layer_file(tmp_path, "c1", 4)
    with gguf.GgufExperts(path) as g:
        for bad in (lambda: g.expert_slice(names[0], 4), lambda: g.expert_slice(names[0], 3, 2), lambda: g.expert_slice(names[0], -1),
                    lambda: g.expert_slice("blk.0.ffn_gate_inp.weight", 0), lambda: g.tensor("no.such.tensor")):
            with pytest.raises(Exception):
                bad()
        data = np.empty(16, np.uint8)
        assert lib.b2moe_gguf_expert_bank(g._h, names[0].encode(), 0, 1, 23, data.ctypes.data, None) != 0     # IQ4_XS bank from a Q4_K tensor
    blob = open(path, "rb").read()
    cases = {"magic": b"GGUX" + blob[4:], "version": blob[:4] + struct.pack("<I", 7) + blob[8:], "truncated header": blob[:40],
             "truncated data": blob[:len(blob) // 2], "tensor count": blob[:8] + struct.pack("<Q", 1 << 30) + blob[16:]}
    for what, b in cases.items():
        p = str(tmp_path / "bad.gguf")
        open(p, "wb").write(b)
        h = C.c_void_p()
        rc = lib.b2moe_gguf_open(p.encode(), C.byref(h))
        if rc == 0:                     # the header may still parse: then the truncated tensor must be refused at the slice
            assert what == "truncated data", what
            raw, nb = C.c_void_p(), C.c_uint64()
            assert lib.b2moe_gguf_expert_slice(h, names[2].encode(), 0, 1, None, None, None, C.byref(raw), C.byref(nb)) != 0
            lib.b2moe_gguf_close(h)
        else:
            assert not h.value, what
    h = C.c_void_p()
    assert lib.b2moe_gguf_open(str(tmp_path / "missing.gguf").encode(), C.byref(h)) != 0
