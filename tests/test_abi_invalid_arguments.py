"""Every entry point turns a malformed call into a validation status (1..9) before it makes a CUDA
call: a valid description of a call is corrupted in one to three ways (rank, extents, element size,
null pointers, misaligned pointers, mismatched shapes, scheme fields out of range, non-contiguous codes)
and the status must never be QK_OK nor a CUDA error.  No device memory is involved: addresses are made
up and never dereferenced by the validation."""
import ctypes as C

import numpy as np
from hypothesis import given, settings, strategies as st

from cubek_b200 import ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue, _ffi

LIB = _ffi.lib()
U32, NAT = QuantStore.U32, QuantStore.Native


def tensor(addr, shape, strides, elem_size, rank=None):
    t = _ffi.QkTensor()
    n = max(len(shape), 1)
    t._keep = ((C.c_int64 * n)(*shape), (C.c_int64 * n)(*strides))
    t.ptr = C.c_void_p(addr)
    t.rank = len(shape) if rank is None else rank
    t.shape, t.strides = t._keep
    t.elem_size = elem_size
    return t


def strides_of(shape):
    out, acc = [], 1
    for s in reversed(shape):
        out.append(acc)
        acc *= s
    return list(reversed(out))


CORRUPTIONS = ["rank0", "rank9", "neg_extent", "elem_size", "null_in", "null_out", "misaligned", "codes_shape",
               "scales_shape", "value", "store", "mode", "param", "level", "block_zero", "block_rank", "block_nq",
               "last_dim_nq", "dtype", "null_scheme"]


@settings(max_examples=300, deadline=None)
@given(st.data())
def test_corrupted_calls_are_rejected_by_validation(data):
    store = data.draw(st.sampled_from([U32, NAT]))
    value = data.draw(st.sampled_from([QuantValue.Q8S, QuantValue.Q4S, QuantValue.Q2F] if store == U32
                                      else [QuantValue.Q8S, QuantValue.E2M1, QuantValue.E4M3]))
    blocked = data.draw(st.booleans())
    scheme = QuantScheme(value=value, store=store, level=QuantLevel.block([32]) if blocked else QuantLevel.Tensor)
    nq = scheme.num_quants()
    rows, cols = data.draw(st.integers(1, 9)), 32 * data.draw(st.integers(1, 4))
    fdt = data.draw(st.sampled_from([ElemType.F32, ElemType.F16, ElemType.BF16]))
    fsize = 4 if fdt == ElemType.F32 else 2
    csize = 4 if store == U32 else 1
    shape, cshape = [rows, cols], [rows, cols // nq]
    sshape = [rows, cols // 32] if blocked else [1]
    kinds = data.draw(st.lists(st.sampled_from(CORRUPTIONS), min_size=1, max_size=3, unique=True))

    sch = _ffi.c_scheme(scheme)
    a_in, a_codes, a_scale, a_oscale, a_out = 0x100000, 0x200000, 0x300000, 0x400000, 0x500000
    in_shape, in_strides, in_size, in_rank = list(shape), strides_of(shape), fsize, None
    c_shape, c_strides = list(cshape), strides_of(cshape)
    s_shape = list(sshape)
    dtype = int(fdt)
    scheme_ptr = C.byref(sch)
    for k in kinds:
        if k == "rank0":
            in_rank = 0
        elif k == "rank9":
            in_rank = 9
        elif k == "neg_extent":
            in_shape[0] = -in_shape[0]
        elif k == "elem_size":
            in_size = 3
        elif k == "null_in":
            a_in = a_out = 0                           # the float tensor of either direction
        elif k == "null_out":
            a_codes = 0
        elif k == "misaligned":
            a_in += 1
            a_out += 1
        elif k == "codes_shape":
            c_shape[-1] += 1
            c_strides = strides_of(c_shape)
        elif k == "scales_shape":
            s_shape = [s + 1 for s in s_shape]
        elif k == "value":
            sch.value = 17
        elif k == "store":
            sch.store = 5
        elif k == "mode":
            sch.mode = 1
        elif k == "param":
            sch.param = 9
        elif k == "level":
            sch.level = 3
        elif k == "block_zero":
            sch.level, sch.block_rank = 1, 1
            sch.block[0] = 0
        elif k == "block_rank":
            sch.level, sch.block_rank = 1, 3          # more block dims than tensor dims
            for i in range(3):
                sch.block[i] = 32
        elif k == "block_nq":
            if nq == 1:
                sch.value = 99                         # every block size suits one value per item
            else:
                sch.level, sch.block_rank = 1, 1
                sch.block[0] = nq + 1                  # not a multiple of num_quants
        elif k == "last_dim_nq":
            if nq == 1:
                in_size = 3
            else:
                in_shape[-1] += 1
                in_strides = strides_of(in_shape)
        elif k == "dtype":
            dtype = 7
        elif k == "null_scheme":
            scheme_ptr = None

    t_in = tensor(a_in, in_shape, in_strides, in_size, in_rank)
    t_codes = tensor(a_codes, c_shape, c_strides, csize)
    t_scale = tensor(a_scale, s_shape, strides_of(s_shape), fsize)
    t_oscale = tensor(a_oscale, s_shape, strides_of(s_shape), 4)
    t_out = tensor(a_out, in_shape, in_strides, in_size, in_rank)
    ws = C.c_void_p(0x600000)
    calls = {
        "qk_quantize": lambda: LIB.qk_quantize(C.byref(t_in), C.byref(t_codes), C.byref(t_scale), C.byref(t_oscale),
                                               scheme_ptr, dtype, None),
        "qk_quantize_dynamic": lambda: LIB.qk_quantize_dynamic(C.byref(t_in), C.byref(t_codes), C.byref(t_oscale), scheme_ptr,
                                                               dtype, ws, 1 << 20, None),
        "qk_dequantize": lambda: LIB.qk_dequantize(C.byref(t_codes), C.byref(t_out), C.byref(t_oscale), scheme_ptr, dtype, None),
    }
    for name, call in calls.items():
        rc = call()
        assert 1 <= rc <= 9, f"{name} returned {rc} for corruptions {kinds} ({value.name}, {store.name}, blocked={blocked})"
