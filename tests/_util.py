"""Helpers shared by the tests: NumPy <-> torch conversion for the three float types and thin
wrappers that run the library on device copies of NumPy arrays (through the C ABI)."""
from __future__ import annotations

import ml_dtypes
import numpy as np

from cubek_b200 import ComputeClient, ElemType, QuantScheme, QuantStore, TensorHandleRef, dequantize, quantize
from cubek_b200 import _ffi

bfloat16 = ml_dtypes.bfloat16
NP_FLOAT = {ElemType.F32: np.dtype(np.float32), ElemType.F16: np.dtype(np.float16), ElemType.BF16: np.dtype(bfloat16)}


def elem_of(dtype) -> ElemType:
    dtype = np.dtype(dtype)
    for k, v in NP_FLOAT.items():
        if v == dtype:
            return k
    raise TypeError(dtype)


def to_device(a: np.ndarray):
    import torch

    a = np.ascontiguousarray(a)
    if a.dtype == np.dtype(bfloat16):
        return torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    if a.dtype == np.dtype(np.uint32):
        return torch.from_numpy(a.view(np.int32)).cuda()
    return torch.from_numpy(a).cuda()


def to_numpy(t, dtype) -> np.ndarray:
    import torch

    dtype = np.dtype(dtype)
    if dtype == np.dtype(bfloat16):
        return t.view(torch.int16).cpu().numpy().view(bfloat16)
    if dtype == np.dtype(np.uint32):
        return t.view(torch.int32).cpu().numpy().view(np.uint32)
    return t.cpu().numpy().astype(dtype, copy=False)


def empty_device(shape, dtype):
    import torch

    dtype = np.dtype(dtype)
    tdt = {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16,
           np.dtype(bfloat16): torch.bfloat16, np.dtype(np.uint32): torch.int32,
           np.dtype(np.int8): torch.int8, np.dtype(np.uint8): torch.uint8}[dtype]
    # Filled with a pattern so that elements a kernel fails to write are caught.
    t = torch.empty(tuple(shape), dtype=tdt, device="cuda")
    t.view(torch.uint8).fill_(0xA5)
    return t


def code_dtype(scheme: QuantScheme) -> np.dtype:
    from cubek_b200 import QuantValue

    if scheme.store == QuantStore.U32:
        return np.dtype(np.uint32)
    return np.dtype(np.int8) if scheme.value in (QuantValue.Q8F, QuantValue.Q8S) else np.dtype(np.uint8)


def workspace(nbytes: int = 256):
    import torch

    return torch.zeros(max(nbytes, 256), dtype=torch.uint8, device="cuda")


def gpu_compute_scales(x: np.ndarray, scheme: QuantScheme) -> np.ndarray:
    import torch

    elem = elem_of(x.dtype)
    dx = to_device(x)
    ds = empty_device(scheme.scales_shape(x.shape), x.dtype)
    ws = workspace()
    quantize.compute_scales(ComputeClient.current(), TensorHandleRef.from_torch(dx), TensorHandleRef.from_torch(ds),
                            scheme, elem, TensorHandleRef.from_torch(ws))
    torch.cuda.synchronize()
    return to_numpy(ds, x.dtype)


def gpu_quantize(x: np.ndarray, scale: np.ndarray, scheme: QuantScheme):
    import torch

    elem = elem_of(x.dtype)
    dx, dscale = to_device(x), to_device(scale)
    dq = empty_device(scheme.packed_shape(x.shape), code_dtype(scheme))
    dos = empty_device(scale.shape, NP_FLOAT[ElemType(int(scheme.param))])
    quantize.launch_ref(ComputeClient.current(), TensorHandleRef.from_torch(dx), TensorHandleRef.from_torch(dq),
                        TensorHandleRef.from_torch(dscale), TensorHandleRef.from_torch(dos), scheme, elem)
    torch.cuda.synchronize()
    return to_numpy(dq, code_dtype(scheme)), to_numpy(dos, NP_FLOAT[ElemType(int(scheme.param))])


def gpu_quantize_dynamic(x: np.ndarray, scheme: QuantScheme):
    import torch

    elem = elem_of(x.dtype)
    dx = to_device(x)
    dq = empty_device(scheme.packed_shape(x.shape), code_dtype(scheme))
    pdt = NP_FLOAT[ElemType(int(scheme.param))]
    dos = empty_device(scheme.scales_shape(x.shape), pdt)
    tin = _ffi.CTensor(TensorHandleRef.from_torch(dx))
    need = _ffi.lib().qk_workspace_bytes_for(tin.ref(), _ffi.c_scheme(scheme), int(elem))
    ws = workspace(int(need))
    quantize.launch_dynamic(ComputeClient.current(), TensorHandleRef.from_torch(dx), TensorHandleRef.from_torch(dq),
                            TensorHandleRef.from_torch(dos), scheme, elem, TensorHandleRef.from_torch(ws))
    torch.cuda.synchronize()
    return to_numpy(dq, code_dtype(scheme)), to_numpy(dos, pdt)


def gpu_dequantize(values: np.ndarray, params: np.ndarray, scheme: QuantScheme, out_dtype) -> np.ndarray:
    import torch

    elem = elem_of(out_dtype)
    dv, dp = to_device(values), to_device(params)
    shape = tuple(values.shape[:-1]) + (values.shape[-1] * scheme.num_quants(),)
    do = empty_device(shape, out_dtype)
    dequantize.launch_ref(ComputeClient.current(), TensorHandleRef.from_torch(dv), TensorHandleRef.from_torch(do),
                          TensorHandleRef.from_torch(dp), scheme, elem)
    torch.cuda.synchronize()
    return to_numpy(do, out_dtype)


def assert_bits_equal(a: np.ndarray, b: np.ndarray, what: str = ""):
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    assert a.dtype == b.dtype, f"{what}: dtype {a.dtype} vs {b.dtype}"
    if a.tobytes() != b.tobytes():
        ai = a.reshape(-1).view(np.uint8).reshape(a.size, -1)
        bi = b.reshape(-1).view(np.uint8).reshape(b.size, -1)
        bad = np.nonzero((ai != bi).any(axis=1))[0]
        i = int(bad[0])
        raise AssertionError(f"{what}: {bad.size} of {a.size} elements differ; first at flat index {i}: "
                             f"{a.reshape(-1)[i]!r} vs {b.reshape(-1)[i]!r}")
