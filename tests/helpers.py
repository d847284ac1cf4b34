"""Shared input generators and comparison helpers for the parity tests."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def h16(a):
    return np.ascontiguousarray(a, dtype=np.float32).astype(np.float16)


def wkv_inputs(B, T, H, seed=0):
    """Inputs of the op-level WKV benchmark configuration: r,k,v ~ N(0,1); the decay target is
    exp(-exp(x)), x ~ U(-6,-0.5), expressed as the raw pre-activation the kernels consume;
    kk = L2-normalised N(0,1) per head, a = -kk, b = kk * sigmoid(U(-3,3)).  All rounded to fp16."""
    rng = np.random.default_rng(seed)
    C_ = H * 64
    shape = (B * T, C_)
    r, k, v = (h16(rng.standard_normal(shape)) for _ in range(3))
    x = rng.uniform(-6.0, -0.5, shape)
    p = np.clip(np.exp(x + 0.5), 1e-6, 1 - 1e-6)
    w = h16(np.clip(np.log(p / (1 - p)), -12, 12))
    kk = rng.standard_normal((B * T, H, 64))
    kk /= np.linalg.norm(kk, axis=-1, keepdims=True)
    a = h16(-kk.reshape(shape))
    b = h16((kk * (1 / (1 + np.exp(-rng.uniform(-3, 3, kk.shape))))).reshape(shape))
    return r, w, k, v, a, b


def pattern_value(index, scale, bias):
    """The file-free deterministic generator of the reference's kernel tests
    (test/cuda_non4096_kernels_test.cpp:20-24)."""
    index = np.asarray(index)
    return (np.sin((index % 97).astype(np.float32) * np.float32(0.173)) * np.float32(scale)
            + np.cos((index % 53).astype(np.float32) * np.float32(0.071)) * np.float32(scale * 0.5) + np.float32(bias)).astype(np.float32)


def ulp_diff16(a, b):
    """Distance in fp16 units-in-the-last-place between two float16 arrays (monotone integer map)."""
    def key(x):
        u = np.ascontiguousarray(x, np.float16).view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - u, u)
    return np.abs(key(a) - key(b))


from oracle.oracle import ref_lib  # noqa: E402,F401  (the reference's own kernels built under oracle/_ref/)
