"""Helpers for the -m gpu parity tests: device tensors live in torch (memory plumbing only); all
compute goes through the C ABI on the runtime's own stream."""
import numpy as np
import torch

import effect_torch_b200 as et

_rt = None


def runtime() -> et.Runtime:
    global _rt
    if _rt is None:
        _rt = et.Runtime(0)
    return _rt


def dev(array, dtype=None):
    """numpy -> device tensor, visible to the runtime's stream before returning."""
    a = np.ascontiguousarray(array if dtype is None else np.asarray(array, dtype=dtype))
    t = torch.from_numpy(a).cuda()
    torch.cuda.synchronize()
    return t


def empty(shape, dtype=torch.float32):
    t = torch.zeros(shape, dtype=dtype, device="cuda")
    torch.cuda.synchronize()
    return t


def host(t) -> np.ndarray:
    """Waits for the runtime's stream (raising any device-side status), then copies back."""
    runtime().synchronize()
    return t.cpu().numpy()
