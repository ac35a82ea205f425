"""The oracle's block decoders against every golden vector there is for them: the committed fixture (gguf-py values,
NVFP4G from the reference), the reference's own tests/data/kquant_golden.bin when that checkout is present, gguf-py
live when importable, and the reference's dequantize_host compiled in place."""
import os
import struct

import numpy as np
import pytest
import torch

from tqllm_b200 import synth
from util import same_bits

TYPES = (12, 21, 23, 20, 323)
_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_GOLDEN = os.path.join(os.environ.get("TQLLM_REFERENCE") or os.path.join(os.path.dirname(_ROOT), "reference"), "tests", "data", "kquant_golden.bin")


@pytest.mark.parametrize("t", TYPES)
def test_committed_golden(orc, golden, t):
    raw, vals = golden["dequant"][f"raw_{t}"], golden["dequant"][f"vals_{t}"]
    assert same_bits(orc.dequant(t, raw, vals.size), vals)


@pytest.mark.skipif(not os.path.isfile(REF_GOLDEN), reason="reference checkout absent")
def test_reference_golden_file(orc):
    buf = open(REF_GOLDEN, "rb").read()
    off, seen = 0, set()
    while off < len(buf):
        t, blocks, nbytes, elems = struct.unpack_from("<4I", buf, off)
        off += 16
        raw = np.frombuffer(buf, np.uint8, blocks * nbytes, off)
        off += blocks * nbytes
        vals = np.frombuffer(buf, np.float32, blocks * elems, off)
        off += 4 * blocks * elems
        if orc.block_elems(t):
            assert orc.block_bytes(t) == nbytes and orc.block_elems(t) == elems
            assert same_bits(orc.dequant(t, raw, vals.size), vals), f"type {t}"
            seen.add(t)
    assert seen == {12, 21, 23, 20}


@pytest.mark.parametrize("t", (12, 21, 23, 20))
def test_against_gguf_py(orc, t):
    gguf = pytest.importorskip("gguf")
    qt = {12: gguf.GGMLQuantizationType.Q4_K, 21: gguf.GGMLQuantizationType.IQ3_S, 23: gguf.GGMLQuantizationType.IQ4_XS,
          20: gguf.GGMLQuantizationType.IQ4_NL}[t]
    g = torch.Generator()
    g.manual_seed(t)
    raw = synth.random_blocks(t, 40, g).numpy()
    want = gguf.quants.dequantize(raw, qt).astype(np.float32).reshape(-1)
    assert same_bits(orc.dequant(t, raw, want.size), want)


@pytest.mark.parametrize("t", TYPES)
def test_against_compiled_reference(orc, ref, t):
    g = torch.Generator()
    g.manual_seed(100 + t)
    elems, _ = synth.BLOCK[t]
    raw = synth.random_blocks(t, 64, g, 2 if t == 323 else 1).numpy()
    assert same_bits(orc.dequant(t, raw, 64 * elems), ref.dequant(t, raw, 64 * elems))
    w = torch.randn(32, 512, generator=g) * 0.02
    raw = synth.quantize(t, w).numpy()
    assert same_bits(orc.dequant(t, raw, w.numel()), ref.dequant(t, raw, w.numel()))


def test_half_and_e4m3_tables(orc, ref):
    for h in range(0, 65536, 7):
        a, b = orc.half_to_float(h), ref.half_to_float(h)
        assert (np.isnan(a) and np.isnan(b)) or np.float32(a).view(np.uint32) == np.float32(b).view(np.uint32), h
    for b8 in range(256):
        a, b = orc.e4m3_to_float(b8), ref.e4m3_to_float(b8)
        assert (np.isnan(a) and np.isnan(b)) or a == b
    # spot values of the E4M3 code (1.0, largest finite 448, smallest subnormal 2^-9, NaN)
    assert orc.e4m3_to_float(0x38) == 1.0 and orc.e4m3_to_float(0x7E) == 448.0 and orc.e4m3_to_float(0x01) == 2.0 ** -9
    assert np.isnan(orc.e4m3_to_float(0x7F)) and orc.e4m3_to_float(0xB8) == -1.0


def test_bad_arguments(orc):
    with pytest.raises(ValueError):
        orc.dequant(999, np.zeros(16, np.uint8), 256)
    with pytest.raises(ValueError):
        orc.dequant(12, np.zeros(144, np.uint8), 100)


@pytest.mark.parametrize("t", TYPES)
def test_quantisers_are_valid(orc, t):
    """our own encoders: right byte count, finite values, error far below the weight scale"""
    g = torch.Generator()
    g.manual_seed(7)
    w = torch.randn(48, 1024, generator=g) * 0.02
    raw = synth.quantize(t, w).numpy()
    assert raw.size == synth.raw_bytes(t, 48, 1024)
    v = orc.dequant(t, raw, w.numel())
    assert np.isfinite(v).all()
    rel = np.sqrt(((v - w.numpy().ravel()) ** 2).mean()) / 0.02
    assert rel < (0.25 if t == 21 else 0.15), rel
    z = synth.quantize(t, torch.zeros(16, 256)).numpy()
    assert np.all(orc.dequant(t, z, 16 * 256) == 0)
