"""``cubek_quant::quantize`` for B200: same entry point, argument order and error behaviour as
the reference's ``launch_ref`` (crates/cubek-quant/src/quantize.rs:174-221), executed by
hand-written sm_100a kernels through the C ABI."""
from __future__ import annotations

from . import _ffi
from .scheme import ElemType, QuantScheme
from .tensor import ComputeClient, TensorHandleRef


def launch_ref(client: ComputeClient, input: TensorHandleRef, output: TensorHandleRef,
               scale: TensorHandleRef, out_scale: TensorHandleRef, scheme: QuantScheme,
               input_elem: ElemType) -> None:
    """Quantize ``input`` with the given scales.

    ``scale`` is typed like the input ("scale is computed based on input float dtype, but stored
    based on qparams precision", quantize.rs:262); ``out_scale`` receives it cast to
    ``scheme.param``; ``output`` is the quantized tensor (u32 words of shape ``[.., n/num_quants]``
    or native bytes).  Enqueues on ``client.stream`` and returns; raises ``QuantPanic`` where the
    reference panics and ``LaunchError`` where it returns ``Err``.
    """
    ti, to, ts, tos = _ffi.c_tensors(input, output, scale, out_scale)
    sch = _ffi.c_scheme(scheme)
    _ffi.check(_ffi.lib().qk_quantize(ti.ref(), to.ref(), ts.ref(), tos.ref(), sch, int(input_elem),
                                      client.stream))


def compute_scales(client: ComputeClient, input: TensorHandleRef, scale: TensorHandleRef,
                   scheme: QuantScheme, input_elem: ElemType, workspace: TensorHandleRef | None = None) -> None:
    """The caller-side step of the reference flow: absmax (``cubek_reduce`` ``MaxAbs``,
    crates/cubek-reduce/src/instructions/maxabs.rs:31-87) and ``scale = 2*absmax/(q_max-q_min)``
    (crates/cubek-quant/tests/suite/symmetric.rs:35-38).  ``scale`` is typed like the input."""
    ti, ts = _ffi.c_tensors(input, scale)
    ws_ptr, ws_bytes = (workspace.handle, workspace.shape[0] * workspace.elem_size) if workspace else (None, 0)
    _ffi.check(_ffi.lib().qk_compute_scales(ti.ref(), ts.ref(), _ffi.c_scheme(scheme), int(input_elem),
                                            ws_ptr, ws_bytes, client.stream))


def launch_dynamic(client: ComputeClient, input: TensorHandleRef, output: TensorHandleRef,
                   out_scale: TensorHandleRef, scheme: QuantScheme, input_elem: ElemType,
                   workspace: TensorHandleRef | None = None) -> None:
    """``compute_scales`` + ``launch_ref`` fused (one pass per block; two per tensor), with
    identical results."""
    ti, to, tos = _ffi.c_tensors(input, output, out_scale)
    ws_ptr, ws_bytes = (workspace.handle, workspace.shape[0] * workspace.elem_size) if workspace else (None, 0)
    _ffi.check(_ffi.lib().qk_quantize_dynamic(ti.ref(), to.ref(), tos.ref(), _ffi.c_scheme(scheme),
                                              int(input_elem), ws_ptr, ws_bytes, client.stream))


def absmax(client: ComputeClient, input: TensorHandleRef, input_elem: ElemType, absmax_out: int) -> None:
    """Shard-local absmax into one f32 at device address ``absmax_out``."""
    (ti,) = _ffi.c_tensors(input)
    _ffi.check(_ffi.lib().qk_absmax_f32(ti.ref(), int(input_elem), absmax_out, client.stream))


def launch_from_absmax(client: ComputeClient, input: TensorHandleRef, output: TensorHandleRef,
                       out_scale: TensorHandleRef, absmax_ptr: int, scheme: QuantScheme,
                       input_elem: ElemType) -> None:
    """Per-tensor quantize with the scale derived on the device from a (reduced) absmax."""
    ti, to, tos = _ffi.c_tensors(input, output, out_scale)
    _ffi.check(_ffi.lib().qk_quantize_from_absmax(ti.ref(), to.ref(), tos.ref(), absmax_ptr,
                                                  _ffi.c_scheme(scheme), int(input_elem), client.stream))


class PreparedDynamic:
    """``launch_dynamic`` with the argument marshalling done once.

    Building the C structs costs more host time than a small tensor takes on the device; callers
    that quantize the same buffers repeatedly (or loop over many tensors) prepare the call once
    and invoke it with no Python-side allocation."""

    def __init__(self, client: ComputeClient, input: TensorHandleRef, output: TensorHandleRef,
                 out_scale: TensorHandleRef, scheme: QuantScheme, input_elem: ElemType,
                 workspace: TensorHandleRef | None = None):
        self._keep = _ffi.c_tensors(input, output, out_scale)
        self._scheme = _ffi.c_scheme(scheme)
        ws_ptr, ws_bytes = (workspace.handle, workspace.shape[0] * workspace.elem_size) if workspace else (None, 0)
        self._args = (self._keep[0].ref(), self._keep[1].ref(), self._keep[2].ref(), self._scheme, int(input_elem),
                      ws_ptr, ws_bytes, client.stream)
        self._fn = _ffi.lib().qk_quantize_dynamic

    def __call__(self) -> None:
        status = self._fn(*self._args)
        if status:
            _ffi.check(status)


class PreparedScales:
    """``compute_scales`` with the argument marshalling done once."""

    def __init__(self, client: ComputeClient, input: TensorHandleRef, scale: TensorHandleRef, scheme: QuantScheme,
                 input_elem: ElemType, workspace: TensorHandleRef | None = None):
        self._keep = _ffi.c_tensors(input, scale)
        self._scheme = _ffi.c_scheme(scheme)
        ws_ptr, ws_bytes = (workspace.handle, workspace.shape[0] * workspace.elem_size) if workspace else (None, 0)
        self._args = (self._keep[0].ref(), self._keep[1].ref(), self._scheme, int(input_elem), ws_ptr, ws_bytes, client.stream)
        self._fn = _ffi.lib().qk_compute_scales

    def __call__(self) -> None:
        status = self._fn(*self._args)
        if status:
            _ffi.check(status)


class PreparedRef:
    """``launch_ref`` (quantize with given scales) with the argument marshalling done once."""

    def __init__(self, client: ComputeClient, input: TensorHandleRef, output: TensorHandleRef, scale: TensorHandleRef,
                 out_scale: TensorHandleRef, scheme: QuantScheme, input_elem: ElemType):
        self._keep = _ffi.c_tensors(input, output, scale, out_scale)
        self._scheme = _ffi.c_scheme(scheme)
        self._args = tuple(k.ref() for k in self._keep) + (self._scheme, int(input_elem), client.stream)
        self._fn = _ffi.lib().qk_quantize

    def __call__(self) -> None:
        status = self._fn(*self._args)
        if status:
            _ffi.check(status)


class PreparedDynamicBatch:
    """Fused quantize of a set of tensors with one launch per group of up to 64 compatible tensors
    (``qk_quantize_dynamic_batch``); same results as ``launch_dynamic`` per tensor."""

    def __init__(self, client: ComputeClient, inputs, outputs, out_scales, scheme: QuantScheme,
                 input_elem: ElemType, workspace: TensorHandleRef | None = None):
        self._in, self._out, self._sc = (_ffi.CTensorArray(inputs), _ffi.CTensorArray(outputs),
                                         _ffi.CTensorArray(out_scales))
        if not (self._in.count == self._out.count == self._sc.count):
            raise ValueError("inputs, outputs and out_scales must have the same length")
        self._scheme = _ffi.c_scheme(scheme)
        ws_ptr, ws_bytes = (workspace.handle, workspace.shape[0] * workspace.elem_size) if workspace else (None, 0)
        self._args = (self._in.count, self._in.array, self._out.array, self._sc.array, self._scheme, int(input_elem),
                      ws_ptr, ws_bytes, client.stream)
        self._fn = _ffi.lib().qk_quantize_dynamic_batch

    def __call__(self) -> None:
        status = self._fn(*self._args)
        if status:
            _ffi.check(status)


def launch_dynamic_batch(client: ComputeClient, inputs, outputs, out_scales, scheme: QuantScheme,
                         input_elem: ElemType, workspace: TensorHandleRef | None = None) -> None:
    PreparedDynamicBatch(client, inputs, outputs, out_scales, scheme, input_elem, workspace)()
