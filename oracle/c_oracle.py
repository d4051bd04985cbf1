"""Build and call the plain-C checker (``colsum_oracle.c``).  Test infrastructure only."""

from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "colsum_oracle.c")
_LIB = os.path.join(_HERE, "libcolsum_oracle.so")
_handle = None


def build(force: bool = False) -> str:
    """gcc -O2 -fopenmp the C file next to this module; returns the library path."""
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(_SRC):
        cmd = ["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-o", _LIB, _SRC, "-lm"]
        subprocess.run(cmd, check=True)
    return _LIB


def _lib():
    global _handle
    if _handle is None:
        _handle = ctypes.CDLL(build())
        _handle.colsum_oracle_f32.restype = ctypes.c_int
        _handle.colsum_oracle_f32.argtypes = [
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
            ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
            ctypes.c_double, ctypes.c_int, ctypes.c_int]
        _handle.colsum_oracle_threads.restype = ctypes.c_int
    return _handle


def threads() -> int:
    return int(_lib().colsum_oracle_threads())


def colsum_c(query: torch.Tensor, key: torch.Tensor, scale: Optional[float] = None,
             is_causal: bool = False, cls_len: Optional[int] = None) -> np.ndarray:
    """(B, Sk) float64 column means; inputs of any float dtype are upcast to fp32."""
    q = query.detach().cpu().to(torch.float32).contiguous()
    k = key.detach().cpu().to(torch.float32).contiguous()
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    if scale is None:
        scale = 1.0 / (D ** 0.5)
    out = np.zeros((B, Sk), dtype=np.float64)
    rc = _lib().colsum_oracle_f32(q.data_ptr(), k.data_ptr(), out.ctypes.data,
                                  B, H, Sq, Sk, D, float(scale), int(bool(is_causal)),
                                  0 if cls_len is None else int(cls_len))
    if rc != 0:
        raise RuntimeError(f"colsum_oracle_f32 failed with {rc}")
    return out
