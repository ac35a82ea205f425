"""Bank layout arithmetic on the CPU: the pack_word / decode_unit functions of tqllm_b200/csrc/formats.cuh are
__host__ __device__, so tests/host_formats.cu compiles them for the host; pack + decode must reproduce the oracle's
fp32 values bit for bit, for random blocks (every code pattern) and ragged row counts."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest
import torch

from tqllm_b200 import gen_tables, synth
from util import same_bits

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "_build", "host_formats.so")
TILE = {12: (256, 2304), 21: (256, 1760), 23: (256, 2176), 20: (32, 288), 323: (128, 1152), 0x1015: (256, 2144)}
RAW = lambda t: 21 if t == 0x1015 else t    # 0x1015: IQ3_S blocks in the 4-bit-code bank layout


@pytest.fixture(scope="module")
def shim():
    src = os.path.join(HERE, "host_formats.cu")
    hdr = os.path.join(os.path.dirname(HERE), "tqllm_b200", "csrc", "formats.cuh")
    gen_tables.write()
    if not os.path.isfile(SO) or os.path.getmtime(SO) < max(os.path.getmtime(src), os.path.getmtime(hdr)):
        os.makedirs(os.path.dirname(SO), exist_ok=True)
        subprocess.run(["nvcc", "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a",
                        src, "-o", SO], check=True)
    return C.CDLL(SO)


@pytest.mark.parametrize("t", (12, 21, 23, 20, 323, 0x1015))
@pytest.mark.parametrize("rows,cols", ((16, 256), (19, 512), (40, 768), (1, 256)))
def test_pack_decode_matches_oracle(orc, shim, t, rows, cols):
    g = torch.Generator()
    g.manual_seed(rows * 1000 + cols + t)
    elems, _ = synth.BLOCK[RAW(t)]
    raw = synth.random_blocks(RAW(t), rows * cols // elems, g, cols // elems).numpy()
    kt, tile = TILE[t]
    bank = np.zeros(((rows + 15) // 16) * (cols // kt) * tile, np.uint8)
    out = np.zeros(rows * cols, np.float32)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    assert shim.host_pack_decode(t, vp(raw), rows, cols, vp(bank), vp(out)) == 0
    assert same_bits(out, orc.dequant(RAW(t), raw, rows * cols))


def test_tile_bytes_equal_block_bytes():
    """the bank adds no padding: a 16-row tile holds exactly 16 rows of GGUF blocks (NVFP4G: minus the per-block copy
    of the fp32 tensor scale, which moves to the per-row aux array)"""
    for t, (kt, tile) in TILE.items():
        if t == 0x1015:                       # the code layout trades bytes for decode work: 134 per 256 weights
            assert tile == 16 * 134
            continue
        elems, nbytes = synth.BLOCK[t]
        assert tile == 16 * (kt // elems) * (nbytes - (4 if t == 323 else 0)) and tile % 16 == 0
