"""Shared helpers of the parity tests."""
import numpy as np


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(bits(a), bits(b))


def rel_err(out, ref):
    """max abs error normalised by the RMS of the reference output: the layer-output tolerance metric (<= 1e-2)"""
    ref = np.asarray(ref, np.float64)
    return float(np.abs(np.asarray(out, np.float64) - ref).max() / max(np.sqrt((ref ** 2).mean()), 1e-30))


def ulp_gap(a, b):
    """distance in fp32 ulps between two same-sign floats"""
    return abs(int(np.float32(a).view(np.int32)) - int(np.float32(b).view(np.int32)))


def audit_ids(dev_ids, cpu_ids, cpu_logits_row_probs, max_ulps=4):
    """Every position where the device and the CPU top-k disagree must be a near-tie of the CPU's own selection keys
    (gap <= max_ulps): the protocol of the reference's device routing test plus a tie audit. Returns the number of
    audited near-ties; raises AssertionError on a real mismatch."""
    ties = 0
    for t in range(dev_ids.shape[0]):
        if np.array_equal(dev_ids[t], cpu_ids[t]):
            continue
        keys = cpu_logits_row_probs[t]
        for a, b in zip(dev_ids[t], cpu_ids[t]):
            if a != b:
                assert ulp_gap(keys[a], keys[b]) <= max_ulps, f"token {t}: device picked {a}, CPU {b}, keys {keys[a]} {keys[b]}"
                ties += 1
    return ties
