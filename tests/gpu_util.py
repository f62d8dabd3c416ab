"""Helpers for the GPU parity tests: device buffers via torch (plumbing only),
storage-bit conversions, and the norm-wise error the tolerances are stated in."""
import numpy as np
import torch

from pyc_b200 import abi, backend, workloads

# Norm-wise tolerances, max|gpu - ref| / max|ref| against the fp32 CPU result.
TOL = {abi.DTYPE_F32: 1e-5, abi.DTYPE_BF16: 2e-2, abi.DTYPE_F16: 2e-2}


def round_to(dtype, x):
    """fp32 array -> (storage array to upload, the rounded values widened back to fp32)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dtype == abi.DTYPE_F32:
        return x, x
    if dtype == abi.DTYPE_BF16:
        bits = workloads.to_bf16_bits(x)
        return bits, workloads.bf16_bits_to_f32(bits)
    h = x.astype(np.float16)
    return h.view(np.uint16), h.astype(np.float32)


def to_device(storage):
    a = np.ascontiguousarray(storage)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(a.copy()).cuda()


def empty_device(dtype, shape):
    td = torch.float32 if dtype == abi.DTYPE_F32 else torch.int16
    return torch.zeros(tuple(shape), dtype=td, device="cuda")


def to_host_f32(dtype, t):
    a = t.cpu().numpy()
    if dtype == abi.DTYPE_F32:
        return a
    if dtype == abi.DTYPE_BF16:
        return workloads.bf16_bits_to_f32(a.view(np.uint16))
    return a.view(np.float16).astype(np.float32)


def rel_err(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / max(np.abs(want).max(), 1e-30))


def dev_tensor(t, dtype, shape=None):
    return backend.make_tensor(t.data_ptr(), t.numel() * t.element_size(), dtype, shape or tuple(t.shape))


def sync_ok():
    torch.cuda.synchronize()
    st = backend.device_status()
    assert st == 0, f"a kernel wait timed out: status 0x{st:x}"
