/*
 * cubek_quant_b200 - hooks for tests and measurements.  NOT part of the drop-in interface: nothing here
 * replaces anything of the reference, and production callers have no use for it.  The symbols are exported by
 * the same shared library.
 */
#ifndef CUBEK_QUANT_B200_TESTING_H
#define CUBEK_QUANT_B200_TESTING_H

#include "cubek_quant_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Process-wide launch knobs (keys: 0 threads per CTA, 1 CTAs per SM, 2 force the reference-arithmetic route,
 * 3 force the layout-general kernels, 4 programmatic dependent launch on/off, 5 / 6 grid size of the quantize /
 * dequantize kernels in waves, 7 cooperative per-tensor kernel on/off, 8 staging of the quantize input through
 * shared memory with bulk copies: 0 units below 64 bytes, 1 always, 2 never, 9 / 10 input KiB per slice (0: sized by the call, 16-64 MiB) and
 * staging slots (1..8) of qk_roundtrip_host; change them only between calls, and size the staging area after,
 * 11 ring depth (2..4 tiles of 16 KB) of the staged quantize variant, 12 rows the one-launch per-tensor kernel keeps
 * in shared memory (< 0: as many as fit), 13 largest tensor in MiB that takes that kernel).  They exist so that tests can force every
 * route onto the same inputs and measurements can compare routes; they change behaviour for every thread of the
 * process. */
void qk_set_tuning(int key, int value);
int qk_get_tuning(int key);

/* Replaces the functions qk_allreduce_max_f32[_deadline] call, so that the deadline and error paths can be tested on
 * the host with no communicator and no GPU left waiting:
 *   allreduce(sendbuf, recvbuf, count, datatype, op, comm, stream) -> ncclResult_t
 *   async_error(comm, ncclResult_t *out) -> ncclResult_t
 *   stream_query(stream) -> 0 when the stream has drained, 600 (cudaErrorNotReady) while work is pending
 * Null pointers restore the real ones (NCCL resolved at run time, cudaStreamQuery). */
void qk_testing_set_collective_hooks(int (*allreduce)(const void *, void *, size_t, int, int, void *, void *),
                                     int (*async_error)(void *, int *), int (*stream_query)(void *));

#ifdef __cplusplus
}
#endif
#endif /* CUBEK_QUANT_B200_TESTING_H */
