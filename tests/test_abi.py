"""The C ABI without a GPU: the library loads, exports every symbol the header declares, and
rejects bad arguments with the status that stands for the reference's panic / assert / Err —
all before any CUDA call is made."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

from cubek_b200 import (ComputeClient, ElemType, LaunchError, QuantLevel, QuantPanic, QuantParam, QuantScheme,
                        QuantStore, QuantValue, TensorHandleRef, dequantize, quantize)
from cubek_b200 import _ffi

INCLUDE = Path(__file__).resolve().parent.parent / "include"
HEADER = INCLUDE / "cubek_quant_b200.h"
TESTING_HEADER = INCLUDE / "cubek_quant_b200_testing.h"
CLIENT = ComputeClient(0, 0)


def declared_symbols(header=HEADER):
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(qk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(str(_ffi.LIB_PATH))
    names = declared_symbols()
    assert len(names) >= 15
    for name in names + declared_symbols(TESTING_HEADER):
        assert hasattr(lib, name), f"{name} declared in a header but not exported"


def test_binding_covers_the_headers():
    assert set(_ffi.EXPORTED_SYMBOLS) == set(declared_symbols())
    assert set(_ffi.TESTING_SYMBOLS) == set(declared_symbols(TESTING_HEADER))
    # the public header carries no process-wide knobs
    assert not any("tuning" in n or "testing" in n for n in declared_symbols())


def test_version_and_strerror():
    assert b"sm_100a" in _ffi.lib().qk_version()
    assert _ffi.strerror(0) == "ok"
    assert "block size" in _ffi.strerror(_ffi.QK_ERR_BLOCK_SIZE)


def test_scheme_constants_match_host_mirror():
    lo, hi = C.c_float(), C.c_float()
    for v in QuantValue:
        assert _ffi.lib().qk_value_range(int(v), C.byref(lo), C.byref(hi)) == 0
        assert (lo.value, hi.value) == v.range()
        for store in QuantStore:
            s = QuantScheme(value=v, store=store)
            assert _ffi.lib().qk_num_quants(_ffi.c_scheme(s)) == s.num_quants()
    assert _ffi.lib().qk_value_range(99, C.byref(lo), C.byref(hi)) == _ffi.QK_ERR_UNSUPPORTED_SCHEME


def fake(shape, elem_size, addr=0x10000, strides=None):
    """A handle with a plausible aligned address; validation never dereferences it."""
    return TensorHandleRef.from_raw_parts(addr, shape, elem_size, strides)


def test_native_store_rejects_4_and_2_bit_values():
    # panic!("{value:?} is not supported for native quantization"), quantize.rs:213-219
    for v in (QuantValue.Q4F, QuantValue.Q4S, QuantValue.Q2F, QuantValue.Q2S):
        sch = QuantScheme(value=v, store=QuantStore.Native)
        with pytest.raises(QuantPanic) as e:
            quantize.launch_ref(CLIENT, fake((4, 32), 4), fake((4, 32), 1), fake((1,), 4), fake((1,), 4), sch,
                                ElemType.F32)
        assert e.value.status == _ffi.QK_ERR_UNSUPPORTED_SCHEME
        with pytest.raises(QuantPanic):
            dequantize.launch_ref(CLIENT, fake((4, 32), 1), fake((4, 32), 4), fake((1,), 4), sch, ElemType.F32)


def test_block_size_must_be_divisible_by_num_quants():
    # assert!(block_size.is_multiple_of(div)), lib.rs:28-31 via quantize.rs:305
    sch = QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([4]))
    with pytest.raises(QuantPanic) as e:
        quantize.launch_ref(CLIENT, fake((4, 32), 4), fake((4, 4), 4), fake((4, 8), 4), fake((4, 8), 4), sch,
                            ElemType.F32)
    assert e.value.status == _ffi.QK_ERR_BLOCK_SIZE


def test_shape_checks():
    sch = QuantScheme(value=QuantValue.Q8S)
    with pytest.raises(QuantPanic) as e:   # packed last dim * 4 != input last dim
        quantize.launch_ref(CLIENT, fake((4, 32), 4), fake((4, 7), 4), fake((1,), 4), fake((1,), 4), sch, ElemType.F32)
    assert e.value.status == _ffi.QK_ERR_SHAPE
    blk = QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([16]))
    with pytest.raises(QuantPanic) as e:   # scales must be [4, 2]
        quantize.launch_ref(CLIENT, fake((4, 32), 4), fake((4, 8), 4), fake((4, 4), 4), fake((4, 2), 4), blk,
                            ElemType.F32)
    assert e.value.status == _ffi.QK_ERR_SHAPE


def test_dtype_layout_alignment_and_null():
    sch = QuantScheme(value=QuantValue.Q8S)
    args = dict(output=fake((4, 8), 4), scale=fake((1,), 4), out_scale=fake((1,), 4))
    with pytest.raises(QuantPanic) as e:   # bf16 declared, 4-byte elements given
        quantize.launch_ref(CLIENT, fake((4, 32), 4), args["output"], args["scale"], args["out_scale"], sch,
                            ElemType.BF16)
    assert e.value.status == _ffi.QK_ERR_DTYPE
    # the repack's output is the one tensor that must be contiguous
    import ctypes as C2
    src, dst = _ffi.c_tensors(fake((8, 16), 4, strides=(1, 8)), fake((32, 4), 4, strides=(1, 32)))
    shape = (C2.c_int64 * 2)(32, 16)
    assert _ffi.lib().qk_into_contiguous_packed(src.ref(), dst.ref(), shape, 2, 4, None) == _ffi.QK_ERR_LAYOUT
    # ... and its shapes must be the packed forms of `shape`
    src, dst = _ffi.c_tensors(fake((8, 16), 4, strides=(1, 8)), fake((32, 5), 4))
    assert _ffi.lib().qk_into_contiguous_packed(src.ref(), dst.ref(), shape, 2, 4, None) == _ffi.QK_ERR_SHAPE
    with pytest.raises(LaunchError) as e:
        quantize.launch_ref(CLIENT, fake((4, 32), 4, addr=0x10002), args["output"], args["scale"],
                            args["out_scale"], sch, ElemType.F32)
    assert e.value.status == _ffi.QK_ERR_ALIGN
    with pytest.raises(LaunchError) as e:
        quantize.launch_ref(CLIENT, fake((4, 32), 4, addr=0), args["output"], args["scale"], args["out_scale"], sch,
                            ElemType.F32)
    assert e.value.status == _ffi.QK_ERR_NULL


def test_per_tensor_dynamic_needs_workspace():
    sch = QuantScheme(value=QuantValue.Q8S)
    with pytest.raises(LaunchError) as e:
        quantize.launch_dynamic(CLIENT, fake((4, 32), 4), fake((4, 8), 4), fake((1,), 4), sch, ElemType.F32, None)
    assert e.value.status == _ffi.QK_ERR_WORKSPACE
    assert _ffi.lib().qk_workspace_bytes() >= 4


def test_empty_tensor_is_a_no_op():
    sch = QuantScheme(value=QuantValue.Q8S)
    quantize.launch_ref(CLIENT, fake((0, 32), 4), fake((0, 8), 4), fake((1,), 4), fake((1,), 4), sch, ElemType.F32)
    dequantize.launch_ref(CLIENT, fake((0, 8), 4), fake((0, 32), 4), fake((1,), 4), sch, ElemType.F32)


def test_host_roundtrip_staging_size():
    sch = QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32]))
    t = _ffi.CTensor(fake((14336, 4096), 2))
    n = _ffi.lib().qk_host_roundtrip_staging_bytes(t.ref(), _ffi.c_scheme(sch), int(ElemType.BF16))
    lib = _ffi.lib()
    slots, slice_kib = lib.qk_get_tuning(_ffi.TUNE_SLOTS), lib.qk_get_tuning(_ffi.TUNE_SLICE_KIB)
    assert (slots, slice_kib) == (4, 0)                          # 0: slices sized by the call, 16 MiB for this one
    slice_bytes = 16 << 20
    assert slots * slice_bytes < n < slots * 3 * slice_bytes     # input + codes + scales + restored per slot
    # a call of many tensors takes larger slices (a sixteenth of its input, at most 64 MiB)
    many = _ffi.CTensorArray([fake((14336, 4096), 2) for _ in range(16)])
    n16 = lib.qk_host_roundtrip_staging_bytes_batch(many.count, many.array, _ffi.c_scheme(sch), int(ElemType.BF16))
    assert slots * (64 << 20) < n16 < slots * 3 * (64 << 20)
    try:
        lib.qk_set_tuning(_ffi.TUNE_SLICE_KIB, 4096)             # an explicit size is taken as given
        n4 = lib.qk_host_roundtrip_staging_bytes_batch(many.count, many.array, _ffi.c_scheme(sch), int(ElemType.BF16))
        assert slots * (4 << 20) < n4 < slots * 3 * (4 << 20)
    finally:
        lib.qk_set_tuning(_ffi.TUNE_SLICE_KIB, 0)


def test_device_header_probe_library_is_built():
    """The test kernel of the public device header is compiled together with the library (sm_100a) and
    exports its one entry point; it is only run on a GPU (tests/test_gpu_device_api.py)."""
    import ctypes
    from pathlib import Path

    probe = Path(__file__).resolve().parent / "device_api" / "libdevice_api_probe.so"
    assert probe.exists(), "run `python -m cubek_b200.build`"
    assert hasattr(ctypes.CDLL(str(probe)), "probe_dequantize")
