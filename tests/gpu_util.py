"""Helpers for the GPU tests: direct C-ABI calls on sentinel-filled, canary-padded buffers."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from sharq_b200 import _lib

CANARY = 0xA5
SENTINEL = 0xCD
PAD = 256


class Buf:
    """A device byte buffer of `n` bytes filled with a sentinel and followed by a canary."""

    def __init__(self, n: int, device="cuda:0"):
        self.n = int(n)
        self.t = torch.full((self.n + PAD,), SENTINEL, dtype=torch.uint8, device=device)
        self.t[self.n:] = CANARY

    @property
    def ptr(self):
        return ctypes.c_void_p(self.t.data_ptr())

    def get(self) -> np.ndarray:
        torch.cuda.synchronize()
        h = self.t.cpu().numpy()
        assert (h[self.n:] == CANARY).all(), "kernel wrote past the end of an output buffer"
        return h[: self.n].copy()


def dptr(t: torch.Tensor):
    return ctypes.c_void_p(t.data_ptr())


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def call(name: str, *args):
    _lib.check(getattr(_lib.lib(), name)(*args))


def sizes5(m, n, k):
    out = (ctypes.c_int64 * 5)()
    call("sharq_get_fused_sparse_residual_buffer_sizes", m, n, k, out)
    return [int(v) for v in out]
