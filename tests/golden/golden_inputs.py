"""Inputs of the golden vectors, made by integer arithmetic only so that the script that ran the reference's
kernels on a GPU and the CPU test that compares the plain implementation with their outputs build the very
same numbers on any machine."""
import numpy as np

CASES = {
    "rms": dict(n=5, hidden=200, eps=1e-5),
    "rope": dict(n=9, heads=3, kv_heads=1, head=64, theta=10000.0, positions=[0, 1, 2, 17, 63, 64, 200, 511, 1000]),
    "silu": dict(n=4, d=172),
    "attn": dict(heads=4, kv_heads=2, head=64, block=16, ctx=[5, 40, 530]),
}


def values(n, seed, scale=1.0):
    """n float32 values in [-scale, scale): a 64-bit linear congruential sequence, top 24 bits."""
    out = np.empty(n, dtype=np.float32)
    s = np.uint64(seed * 2654435761 + 12345)
    a, c = np.uint64(6364136223846793005), np.uint64(1442695040888963407)
    with np.errstate(over="ignore"):
        for i in range(n):
            s = s * a + c
            out[i] = (float(s >> np.uint64(40)) / float(1 << 24) * 2.0 - 1.0) * scale
    return out
