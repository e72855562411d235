"""The entry points only enqueue work on the caller's stream (no allocation, no synchronisation), so a
sequence of calls can be captured into a CUDA graph after one warm-up call and replayed on new data."""
import numpy as np
import pytest
import torch

from cubek_b200 import (ComputeClient, ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue, TensorHandleRef,
                        dequantize, quantize)
from oracle import oracle as O
from tests._cases import FLOATS, random_tensor
from tests._util import assert_bits_equal, code_dtype, elem_of, empty_device, to_device, to_numpy

pytestmark = pytest.mark.gpu
H = TensorHandleRef.from_torch

CASES = [
    ("bf16", QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32])), (256, 1024), 1 << 16),
    ("f16", QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([16])), (128, 512), 1 << 16),
    ("f32", QuantScheme(value=QuantValue.Q8S), (512, 1024), 1 << 16),     # per tensor, one cooperative launch
    ("f32", QuantScheme(value=QuantValue.Q8S), (512, 1024), 256),         # per tensor, absmax kernel + quantize kernel
    ("f32", QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([24])), (64, 96), 1 << 16),   # general kernels
]


@pytest.mark.parametrize("fname,scheme,shape,ws_bytes", CASES)
def test_capture_and_replay(fname, scheme, shape, ws_bytes):
    F = FLOATS[fname]
    elem = elem_of(F)
    x0, x1 = random_tensor(shape, F, 11), random_tensor(shape, F, 12) * np.float32(3).astype(F)
    dx = to_device(x0)
    dq = empty_device(scheme.packed_shape(shape), code_dtype(scheme))
    ds = empty_device(scheme.scales_shape(shape), np.float32)
    do = empty_device(shape, F)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")

    def enqueue():
        client = ComputeClient.current()
        quantize.launch_dynamic(client, H(dx), H(dq), H(ds), scheme, elem, H(ws))
        dequantize.launch_ref(client, H(dq), H(do), H(ds), scheme, elem)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        enqueue()                       # warm-up outside the capture (module loading, one-time attributes)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        enqueue()
    for x in (x1, x0):
        dx.copy_(to_device(x))
        dq.view(torch.uint8).fill_(0xA5)
        do.view(torch.uint8).fill_(0xA5)
        graph.replay()
        torch.cuda.synchronize()
        oc, os_ = O.quantize_dynamic(x, scheme)
        assert_bits_equal(to_numpy(dq, code_dtype(scheme)), oc, "codes")
        assert_bits_equal(to_numpy(ds, np.float32), os_, "scales")
        assert_bits_equal(to_numpy(do, F), O.dequantize(oc, os_, scheme, F), "restored")
