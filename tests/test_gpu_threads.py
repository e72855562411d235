"""Host threads calling the library at the same time, each on a stream of its own: the entry points keep
no per-call state outside their arguments, so every thread gets the bits of a lone call."""
import threading

import numpy as np
import pytest
import torch

from cubek_b200 import (ComputeClient, ElemType, QuantLevel, QuantScheme, QuantStore, QuantValue, TensorHandleRef,
                        dequantize, quantize)
from oracle import oracle as O
from tests._cases import FLOATS, random_tensor
from tests._util import assert_bits_equal, code_dtype, empty_device, to_device, to_numpy

pytestmark = pytest.mark.gpu
H = TensorHandleRef.from_torch

JOBS = [
    ("bf16", ElemType.BF16, QuantScheme(value=QuantValue.Q4S, level=QuantLevel.block([32])), (512, 1024)),
    ("f32", ElemType.F32, QuantScheme(value=QuantValue.Q8S), (256, 2048)),
    ("f16", ElemType.F16, QuantScheme(value=QuantValue.E2M1, store=QuantStore.Native, level=QuantLevel.block([16])), (300, 512)),
    ("f32", ElemType.F32, QuantScheme(value=QuantValue.Q2S, level=QuantLevel.block([64])), (128, 4096)),
    ("bf16", ElemType.BF16, QuantScheme(value=QuantValue.Q8S, level=QuantLevel.block([24])), (64, 96)),   # general kernels
    ("f16", ElemType.F16, QuantScheme(value=QuantValue.Q8F), (1000, 36)),
]


def test_concurrent_host_threads():
    rounds = 25
    device = torch.cuda.current_device()
    results, errors = {}, []

    def work(j):
        try:
            torch.cuda.set_device(device)
            fname, elem, scheme, shape = JOBS[j]
            F = FLOATS[fname]
            stream = torch.cuda.Stream()
            client = ComputeClient(device, stream.cuda_stream)
            with torch.cuda.stream(stream):
                xs = [to_device(random_tensor(shape, F, 7000 + 100 * j + r)) for r in range(rounds)]
                dq = [empty_device(scheme.packed_shape(shape), code_dtype(scheme)) for _ in range(rounds)]
                ds = [empty_device(scheme.scales_shape(shape), np.float32) for _ in range(rounds)]
                do = [empty_device(shape, F) for _ in range(rounds)]
                ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
                stream.synchronize()
                for r in range(rounds):
                    quantize.launch_dynamic(client, H(xs[r]), H(dq[r]), H(ds[r]), scheme, elem, H(ws))
                    dequantize.launch_ref(client, H(dq[r]), H(do[r]), H(ds[r]), scheme, elem)
                stream.synchronize()
            results[j] = (xs, dq, ds, do)
        except Exception as e:   # surfaced by the main thread
            errors.append((j, repr(e)))

    threads = [threading.Thread(target=work, args=(j,)) for j in range(len(JOBS))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    torch.cuda.synchronize()
    for j, (fname, elem, scheme, shape) in enumerate(JOBS):
        F = FLOATS[fname]
        xs, dq, ds, do = results[j]
        for r in (0, rounds // 2, rounds - 1):
            oc, os_ = O.quantize_dynamic(to_numpy(xs[r], F), scheme)
            assert_bits_equal(to_numpy(dq[r], code_dtype(scheme)), oc, "codes")
            assert_bits_equal(to_numpy(ds[r], np.float32), os_, "scales")
            assert_bits_equal(to_numpy(do[r], F), O.dequantize(oc, os_, scheme, F), "restored")
