"""The reference's production CPU expert pool (CpuMissPool, compiled in place into oracle/_ref/libtqrefpool.so) runs one
IQ3_S layer and lands near the fp32 oracle: it is the CPU arm the benchmark times, so it must compute the same layer.
Its numerics are the reference's own (activations rounded to fp16 and quantised to int8 per 32 values, bf16 expert outputs),
hence the loose bound. Runs in a child process: the pool pins the calling thread to CPU 0 and its workers never stop."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHILD = r"""
import sys
sys.path.insert(0, %r); sys.path.insert(0, %r)
import numpy as np
import oracle
from make_golden import layer_inputs
from tqllm_b200 import synth
pool = oracle.reference_pool()
if pool is None:
    print("SKIP"); sys.exit(0)
orc = oracle.oracle()
shape = synth.LayerShape("pool", 512, 8, 3, 256, shared=True, types=(21, 21, 21))
layer, x = layer_inputs(shape, 8, 20, 5)
res = orc.moe_layer(x=x.float().numpy(), router_w=layer.router_w.numpy(), topk=3, ff=256, gating=1, norm=True, scale=0.0, types=shape.types,
                    gate=layer.raw[0].numpy(), up=layer.raw[1].numpy(), down=layer.raw[2].numpy(), experts=8,
                    shared=tuple(t.numpy() for t in layer.shared_raw))
pool.create(2, 512, 256)
out = pool.layer(x=x.float().numpy(), ids=res["ids"], weights=res["weights"], ff=256, types=shape.types, gate=layer.raw[0].numpy(),
                 up=layer.raw[1].numpy(), down=layer.raw[2].numpy(), experts=8, shared=tuple(t.numpy() for t in layer.shared_raw))
ref = res["out"].astype(np.float64)
err = np.abs(out - ref).max() / np.sqrt((ref ** 2).mean())
print("ERR", err)
"""


def test_production_pool_computes_the_layer():
    code = CHILD % (ROOT, os.path.join(ROOT, "tests", "golden"))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    if "SKIP" in r.stdout:
        pytest.skip("no reference checkout and no prebuilt pool library (or not an x86 host)")
    err = float(r.stdout.split("ERR")[1].split()[0])
    assert err < 5e-2, err
