"""Helpers shared by the GPU parity tests (torch <-> numpy views, package import, reference-on-GPU lib)."""
import ctypes as C
import importlib
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def package():
    return importlib.import_module("canopy-foundry_b200")


def bf16_to_u16(t):
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def u16_to_bf16(a, device="cuda"):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(device).view(torch.bfloat16)


def randn_bf16(shape, std=1.0, seed=0, device="cuda", outlier_frac=0.0, outlier_mul=20.0):
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std
    if outlier_frac > 0:
        mask = torch.rand(shape, generator=g, device=device) < outlier_frac
        x = torch.where(mask, x * outlier_mul, x)
    return x.to(torch.bfloat16)


def f32_scalar(v=0.0, device="cuda"):
    """A 16-byte aligned device float (first element of a 4-float block)."""
    import torch
    t = torch.zeros(4, dtype=torch.float32, device=device)
    t[0] = v
    return t


def rel_fro(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


class RefGpu:
    """The reference's own CUDA operators compiled for sm_100a (oracle/_ref/libref_gpu.so)."""

    def __init__(self):
        path = os.path.join(ROOT, "oracle", "_ref", "libref_gpu.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)

    def call(self, name, *args):
        fn = getattr(self.lib, name)
        fn.restype = C.c_int
        conv = []
        import torch
        for a in args:
            if isinstance(a, torch.Tensor):
                conv.append(C.c_void_p(a.data_ptr()))
            elif isinstance(a, float):
                conv.append(C.c_float(a))
            elif isinstance(a, int):
                conv.append(C.c_longlong(a) if abs(a) > 2**31 - 1 else C.c_int(a))
            elif a is None:
                conv.append(C.c_void_p(None))
            else:
                conv.append(a)
        rc = fn(*conv)
        assert rc == 0, f"{name} -> {rc}"


def ref_gpu_or_none():
    try:
        return RefGpu()
    except (FileNotFoundError, OSError):
        return None


def stream_ptr():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)
