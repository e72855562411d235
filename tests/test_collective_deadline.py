"""`qk_allreduce_max_f32` / `qk_allreduce_max_f32_deadline` against a fake collective table (no NCCL, no GPU, nothing
left waiting on a device): the enqueue of a non-blocking communicator, a communicator that reports an asynchronous
error, a collective whose peer never joins (the stream never drains) and the plain success path."""
import ctypes as C
import time

import pytest

from cubek_b200 import _ffi

NCCL_SUCCESS, NCCL_INTERNAL_ERROR, NCCL_IN_PROGRESS = 0, 3, 7
CUDA_NOT_READY = 600
COMM, STREAM = 0x1234, 0x5678


class FakeCollectives:
    def __init__(self, enqueue=(NCCL_SUCCESS,), async_states=(NCCL_SUCCESS,), drained_after=0):
        self.enqueue, self.async_states, self.drained_after = list(enqueue), list(async_states), drained_after
        self.calls, self.queries, self.polls = [], 0, 0
        self.allreduce = _ffi.ALLREDUCE_HOOK(self._allreduce)
        self.async_error = _ffi.ASYNC_ERROR_HOOK(self._async_error)
        self.stream_query = _ffi.STREAM_QUERY_HOOK(self._stream_query)

    def _allreduce(self, send, recv, count, dtype, op, comm, stream):
        self.calls.append((send, recv, count, dtype, op, comm, stream))
        return self.enqueue[0]

    def _async_error(self, comm, out):
        assert comm == COMM
        state = self.async_states[min(self.polls, len(self.async_states) - 1)]
        self.polls += 1
        out[0] = state
        return NCCL_SUCCESS

    def _stream_query(self, stream):
        assert stream == STREAM
        self.queries += 1
        return 0 if self.drained_after is not None and self.queries > self.drained_after else CUDA_NOT_READY

    def install(self):
        _ffi.lib().qk_testing_set_collective_hooks(C.cast(self.allreduce, C.c_void_p), C.cast(self.async_error, C.c_void_p),
                                                   C.cast(self.stream_query, C.c_void_p))


@pytest.fixture
def hooks():
    made = []

    def make(**kw):
        f = FakeCollectives(**kw)
        f.install()
        made.append(f)
        return f

    yield make
    _ffi.lib().qk_testing_set_collective_hooks(None, None, None)


BUF = (C.c_float * 4)(1, 2, 3, 4)


def test_enqueue_only_form_passes_max_of_f32(hooks):
    f = hooks()
    assert _ffi.lib().qk_allreduce_max_f32(C.addressof(BUF), 4, COMM, STREAM) == 0
    (send, recv, count, dtype, op, comm, stream), = f.calls
    assert send == recv == C.addressof(BUF) and count == 4
    assert (dtype, op) == (7, 2)          # ncclFloat32, ncclMax
    assert (comm, stream) == (COMM, STREAM)
    assert f.queries == 0                 # does not wait for completion


def test_deadline_form_returns_once_the_stream_has_drained(hooks):
    f = hooks(drained_after=3)
    assert _ffi.lib().qk_allreduce_max_f32_deadline(C.addressof(BUF), 4, COMM, STREAM, 2000) == 0
    assert f.queries == 4


def test_a_rank_that_never_joins_ends_in_timeout_not_in_a_hang(hooks):
    f = hooks(drained_after=None)         # the collective never completes
    t0 = time.perf_counter()
    status = _ffi.lib().qk_allreduce_max_f32_deadline(C.addressof(BUF), 4, COMM, STREAM, 150)
    waited = time.perf_counter() - t0
    assert status == _ffi.QK_ERR_TIMEOUT
    assert 0.1 < waited < 2.0
    assert "deadline" in _ffi.strerror(status)
    with pytest.raises(_ffi.LaunchError):
        _ffi.check(status)


def test_asynchronous_communicator_error_is_reported(hooks):
    hooks(async_states=(NCCL_SUCCESS, NCCL_SUCCESS, NCCL_INTERNAL_ERROR), drained_after=None)
    assert _ffi.lib().qk_allreduce_max_f32_deadline(C.addressof(BUF), 4, COMM, STREAM, 5000) == _ffi.QK_ERR_NCCL


def test_non_blocking_communicator_enqueue_in_progress(hooks):
    # ncclAllReduce answers ncclInProgress; the communicator leaves that state after two polls
    f = hooks(enqueue=(NCCL_IN_PROGRESS,), async_states=(NCCL_IN_PROGRESS, NCCL_IN_PROGRESS, NCCL_SUCCESS), drained_after=0)
    assert _ffi.lib().qk_allreduce_max_f32_deadline(C.addressof(BUF), 4, COMM, STREAM, 2000) == 0
    assert f.polls >= 3
    # ... or never does
    hooks(enqueue=(NCCL_IN_PROGRESS,), async_states=(NCCL_IN_PROGRESS,), drained_after=0)
    assert _ffi.lib().qk_allreduce_max_f32_deadline(C.addressof(BUF), 4, COMM, STREAM, 100) == _ffi.QK_ERR_TIMEOUT


def test_failed_enqueue_and_null_arguments(hooks):
    hooks(enqueue=(NCCL_INTERNAL_ERROR,))
    assert _ffi.lib().qk_allreduce_max_f32(C.addressof(BUF), 4, COMM, STREAM) == _ffi.QK_ERR_NCCL
    assert _ffi.lib().qk_allreduce_max_f32(None, 4, COMM, STREAM) == _ffi.QK_ERR_NULL
    assert _ffi.lib().qk_allreduce_max_f32_deadline(C.addressof(BUF), 4, None, STREAM, 10) == _ffi.QK_ERR_NULL
