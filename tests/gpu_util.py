"""Helpers for the GPU parity tests: numpy bit patterns <-> device memory, and error metrics."""
import numpy as np


def dev(arr):
    """Uploads a numpy array as raw bytes (the C ABI only sees pointers and sizes)."""
    import torch

    a = np.ascontiguousarray(arr)
    return torch.from_numpy(a.view(np.uint8).reshape(-1).copy()).cuda()


def empty(nbytes, fill=0xAB):
    import torch

    return torch.full((int(nbytes),), fill, dtype=torch.uint8, device="cuda")


def host(t, np_dtype, shape=None):
    a = t.cpu().numpy().view(np_dtype)
    return a.reshape(shape) if shape is not None else a


def rel_err(got, want):
    """Max relative error with the reference's near-zero floor (device/cpu/parity/parity.go:47,86-92)."""
    got = got.astype(np.float64).ravel()
    want = want.astype(np.float64).ravel()
    both_tiny = (np.abs(got) < 1e-11) & (np.abs(want) < 1e-11)
    denom = np.maximum(np.abs(want), 1e-30)
    e = np.abs(got - want) / denom
    e[both_tiny] = 0
    return float(e.max()) if e.size else 0.0


def ulp16_diff(got_bits, want_bits):
    """Distance in units of the last place between two arrays of 16-bit float patterns (same sign assumed)."""
    g = got_bits.astype(np.int32)
    w = want_bits.astype(np.int32)
    g = np.where(g & 0x8000, 0x8000 - g, g)
    w = np.where(w & 0x8000, 0x8000 - w, w)
    return np.abs(g - w)
