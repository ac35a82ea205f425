"""GPU: bank load + fp32 dump through the C ABI must equal the oracle's dequantisation bit for bit (all five formats,
random blocks so every code pattern occurs, quantised Gaussian weights, ragged row counts, several experts)."""
import numpy as np
import pytest
import torch

from tqllm_b200 import synth
from util import same_bits

pytestmark = pytest.mark.gpu
TYPES = (12, 21, 23, 20, 323, 0x1015)       # 0x1015: IQ3_S blocks in the 4-bit-code bank layout
RAW = lambda t: 21 if t == 0x1015 else t    # the GGUF type whose blocks the bank is loaded from


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("experts,rows,cols", ((1, 16, 256), (3, 19, 512), (2, 48, 1024), (5, 1, 256)))
def test_dump_equals_oracle_random_blocks(orc, t, experts, rows, cols):
    from tqllm_b200 import moe
    g = torch.Generator()
    g.manual_seed(t * 31 + rows)
    elems, _ = synth.BLOCK[RAW(t)]
    raw = synth.random_blocks(RAW(t), experts * rows * cols // elems, g, cols // elems)
    bank = moe.DeviceBank(t, raw.cuda(), experts, rows, cols)
    got = bank.dequant().cpu().numpy().reshape(-1)
    assert same_bits(got, orc.dequant(RAW(t), raw.numpy(), experts * rows * cols))


@pytest.mark.parametrize("t", TYPES)
def test_dump_equals_oracle_quantised_weights(orc, t):
    from tqllm_b200 import moe
    g = torch.Generator()
    g.manual_seed(t)
    w = torch.randn(4 * 64, 1024, generator=g) * 0.02
    raw = synth.quantize(RAW(t), w)
    bank = moe.DeviceBank(t, raw.cuda(), 4, 64, 1024)
    assert same_bits(bank.dequant().cpu().numpy().reshape(-1), orc.dequant(RAW(t), raw.numpy(), w.numel()))


@pytest.mark.parametrize("t", TYPES)
def test_committed_golden_blocks(golden, t):
    """the golden blocks (gguf-py / reference values) through the device path"""
    from tqllm_b200 import moe
    raw, vals = golden["dequant"][f"raw_{RAW(t)}"], golden["dequant"][f"vals_{RAW(t)}"]
    elems, nbytes = synth.BLOCK[RAW(t)]
    blocks = raw.size // nbytes
    per_row = 4 if t == 323 else 1
    bank = moe.DeviceBank(t, torch.from_numpy(raw.copy()).cuda(), 1, blocks // per_row, elems * per_row)
    assert same_bits(bank.dequant().cpu().numpy().reshape(-1), vals)


def test_idempotent_and_deterministic(orc):
    from tqllm_b200 import moe
    g = torch.Generator()
    g.manual_seed(5)
    raw = synth.random_blocks(21, 2 * 32 * 2, g).cuda()
    a = moe.DeviceBank(21, raw, 2, 32, 512)
    b = moe.DeviceBank(21, raw, 2, 32, 512)
    assert torch.equal(a.data, b.data) and torch.equal(a.dequant(), b.dequant())
