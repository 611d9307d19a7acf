"""Seeded input generators shared by make_golden.py and the tests.

numpy's legacy RandomState streams are frozen, so the same seed gives the same bits on every
numpy version; fixtures that leave out x and dy are rebuilt from here.
"""
import numpy as np


def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def gen_inputs(seed, b, L, h, d, lo, hi, per_head=False):
    """x, dy ~ N(0,1) fp32 [b,L,h,d]; a = sigmoid(U(lo,hi)) fp32 [b,L,h] or [h]."""
    rs = np.random.RandomState(seed)
    x = rs.standard_normal((b, L, h, d)).astype(np.float32)
    dy = rs.standard_normal((b, L, h, d)).astype(np.float32)
    shape = (h,) if per_head else (b, L, h)
    a = sigmoid(lo + (hi - lo) * rs.random_sample(shape)).astype(np.float32)
    return x, a, dy
