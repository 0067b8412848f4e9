"""Shared helpers of the test-suite: seeded inputs and bit-level comparisons."""
import numpy as np
import torch


def config0_inputs(n, seed=0, steps=5, scale=8.0):
    """Single-chunk case of the benchmark: p ~ N(0, 0.02), m ~ N(0, 1e-4),
    v = |N(0, 1e-6)|, g = fp16(N(0, 1e-3) * scale); one CPU generator, drawn in
    this order (same as tests/golden/make_golden.py)."""
    g = torch.Generator().manual_seed(seed)
    p = torch.randn(n, generator=g) * 0.02
    m = torch.randn(n, generator=g) * 1e-4
    v = (torch.randn(n, generator=g) * 1e-6).abs()
    grads = [(torch.randn(n, generator=g) * 1e-3 * scale).half() for _ in range(steps)]
    return p, m, v, grads


def checksum(t):
    a = t.detach().cpu().numpy()
    bits = a.view(np.uint32 if a.dtype.itemsize == 4 else np.uint16)
    return [int(np.bitwise_xor.reduce(bits)), int(bits.astype(np.uint64).sum(dtype=np.uint64))]


def ulp_diff_f32(a, b):
    """Max distance in units of the last place between two float32 arrays
    (monotone integer mapping of the bit patterns)."""
    a = np.ascontiguousarray(a, dtype=np.float32).view(np.int32).astype(np.int64)
    b = np.ascontiguousarray(b, dtype=np.float32).view(np.int32).astype(np.int64)
    a = np.where(a < 0, -(a & 0x7fffffff), a)
    b = np.where(b < 0, -(b & 0x7fffffff), b)
    return int(np.abs(a - b).max()) if a.size else 0


def ulp_diff_f16(a, b):
    a = np.ascontiguousarray(a).view(np.int16).astype(np.int64)
    b = np.ascontiguousarray(b).view(np.int16).astype(np.int64)
    a = np.where(a < 0, -(a & 0x7fff), a)
    b = np.where(b < 0, -(b & 0x7fff), b)
    return int(np.abs(a - b).max()) if a.size else 0


def n_bit_mismatch(a, b):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    it = np.uint32 if a.dtype.itemsize == 4 else np.uint16
    return int((a.view(it) != b.view(it)).sum())
