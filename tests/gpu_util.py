"""Helpers for the GPU parity tests."""
import numpy as np
import torch


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.view(dtype) if t.element_size() == torch.empty((), dtype=dtype).element_size() and t.dtype != dtype else t.to(dtype)
    return t.cuda()


def f16(a_u16):
    """uint16 bit patterns -> torch float16 CUDA tensor"""
    return torch.from_numpy(np.ascontiguousarray(a_u16).view(np.float16)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.detach().cpu().numpy()


def rel_max_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-30))
