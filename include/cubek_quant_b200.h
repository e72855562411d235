/*
 * cubek_quant_b200 — C ABI of the B200 (sm_100a) quantize / dequantize library.
 *
 * Every entry point replaces one interface of the reference crate `cubek-quant`
 * (paths below are relative to the reference checkout).  All functions are
 * asynchronous on the caller's CUDA stream, allocate no device memory, never
 * synchronise the device and return a status code instead of panicking.
 *
 * Pointers inside QkTensor are DEVICE pointers unless a function says otherwise.
 */
#ifndef CUBEK_QUANT_B200_H
#define CUBEK_QUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scheme: mirrors `cubecl_common::quant::scheme` as re-exported at
 *      crates/cubek-quant/src/lib.rs:14 -------------------------------------------- */

/* Float element types of inputs, outputs and params (`ElemType::Float(..)` passed as
 * `input_elem` at crates/cubek-quant/src/quantize.rs:181; Flex32 is treated as F32). */
typedef enum { QK_F32 = 0, QK_F16 = 1, QK_BF16 = 2 } QkDType;

/* `QuantValue` (crates/cubek-quant/tests/suite/mod.rs:18-38, quantize.rs:192-198). */
typedef enum {
    QK_Q8F = 0, QK_Q8S = 1, QK_Q4F = 2, QK_Q4S = 3, QK_Q2F = 4, QK_Q2S = 5,
    QK_E4M3 = 6, QK_E5M2 = 7, QK_E2M1 = 8
} QkValue;

/* `QuantStore` (quantize.rs:187, :199). */
typedef enum { QK_STORE_NATIVE = 0, QK_STORE_U32 = 1 } QkStore;

/* `QuantParam` (symmetric.rs:65); the value is a QkDType. */
typedef enum { QK_PARAM_F32 = 0, QK_PARAM_F16 = 1, QK_PARAM_BF16 = 2 } QkParam;

/* `QuantLevel` (symmetric.rs:61, :202). */
typedef enum { QK_LEVEL_TENSOR = 0, QK_LEVEL_BLOCK = 1 } QkLevel;

/* `QuantMode` (symmetric.rs:25). */
typedef enum { QK_MODE_SYMMETRIC = 0 } QkMode;

/* `QuantScheme { value, param, store, level, mode }`.  `block` holds `block_rank` u8
 * extents (as `BlockSize` does); they are right-aligned to the tensor rank and
 * left-padded with 1, like `BlockSize::to_dim_vec` (layout/scales.rs:239). */
typedef struct {
    int32_t value;       /* QkValue */
    int32_t param;       /* QkParam */
    int32_t store;       /* QkStore */
    int32_t level;       /* QkLevel */
    int32_t mode;        /* QkMode  */
    int32_t block_rank;  /* 0 for QK_LEVEL_TENSOR */
    uint8_t block[8];
} QkScheme;

/* The fields the reference reads from `TensorHandleRef` (`handle`, `shape`, `strides`,
 * `elem_size`: layout/scales.rs:213-215, quantize.rs:234-239).  Strides in elements.
 * `shape`/`strides` are host arrays of `rank` entries, 1 <= rank <= QK_MAX_RANK. */
#define QK_MAX_RANK 8
typedef struct {
    void *ptr;
    int32_t rank;
    const int64_t *shape;
    const int64_t *strides;
    int32_t elem_size;
} QkTensor;

/* ---- status codes.  The "panic class" (1..4) stands for the reference's `panic!` /
 *      `assert!` sites; the rest map to `Err(LaunchError)`. ------------------------- */
enum {
    QK_OK = 0,
    QK_ERR_UNSUPPORTED_SCHEME = 1, /* quantize.rs:203-206, :218, :273, :324; dequantize.rs:205-208, :226, :278, :330 */
    QK_ERR_BLOCK_SIZE = 2,         /* lib.rs:28-31 */
    QK_ERR_SHAPE = 3,              /* last dim not a multiple of num_quants, or shapes that disagree */
    QK_ERR_DTYPE = 4,              /* elem_size does not match the declared element type */
    QK_ERR_LAYOUT = 5,             /* a tensor this entry point needs contiguous is not */
    QK_ERR_ALIGN = 6,              /* pointer not aligned to its element / word size */
    QK_ERR_NULL = 7,
    QK_ERR_WORKSPACE = 8,          /* workspace missing or too small */
    QK_ERR_TOO_LARGE = 9,          /* more elements than the entry point supports */
    QK_ERR_NCCL = 10,              /* an NCCL call failed, the communicator reports an asynchronous error, or NCCL is absent */
    QK_ERR_TIMEOUT = 11,           /* a host-side deadline ran out (qk_allreduce_max_f32_deadline) */
    QK_ERR_DEVICE = 12,            /* a kernel gave up on a bounded wait: see qk_device_error */
    QK_ERR_CUDA = 1000             /* QK_ERR_CUDA + cudaError_t */
};

/* Quantized values per stored item: 32/bits for QK_STORE_U32; 2 for native E2M1 (two fp4
 * codes per byte), else 1.  `QuantScheme::num_quants` (quantize.rs:144, :290).  0 if invalid. */
int qk_num_quants(const QkScheme *scheme);

/* `QuantValue::range()` (quantize.rs:243, :296).  Returns QK_OK or QK_ERR_UNSUPPORTED_SCHEME. */
int qk_value_range(int value, float *lo, float *hi);

/*
 * Replaces `cubek_quant::quantize::launch_ref` (quantize.rs:174-221), same argument order.
 *   input     float tensor of type `input_dtype`; may be strided (contiguous ones, and ones whose rows are
 *             contiguous and a constant 16-byte-aligned stride apart, take the fast kernels)
 *   output    quantized tensor: u32 words of shape [.., n/num_quants] (QK_STORE_U32), or
 *             1-byte items (QK_STORE_NATIVE: i8, e4m3, e5m2; fp4 pairs of shape [.., n/2]); may be strided (the
 *             reference writes it through `linear_view(output, 1)`, quantize.rs:316): contiguous ones take the
 *             fast kernels
 *   scale     scales typed `input_dtype`: shape [1] per tensor, else one per block
 *             (its strides are honoured)
 *   out_scale receives the scales cast to the param type; same shape/strides rules
 */
int qk_quantize(const QkTensor *input, const QkTensor *output, const QkTensor *scale,
                const QkTensor *out_scale, const QkScheme *scheme, int input_dtype,
                void *stream);

/*
 * Replaces `cubek_quant::dequantize::launch_ref` (dequantize.rs:171-229), same argument order.
 *   values  quantized tensor (as written by qk_quantize); may be strided
 *   output  float tensor of type `output_dtype`, shape = unpacked shape; may be strided
 *   params  scales typed as the scheme's param
 */
int qk_dequantize(const QkTensor *values, const QkTensor *output, const QkTensor *params,
                  const QkScheme *scheme, int output_dtype, void *stream);

/*
 * The caller-side half of the reference flow: absmax per tensor / per block
 * (`cubek_reduce::reduce::<_, MaxAbs>`, crates/cubek-reduce/src/lib.rs:93-131,
 * instructions/maxabs.rs:31-87) followed by `scale = 2*absmax / (q_max - q_min)`
 * (crates/cubek-quant/tests/suite/symmetric.rs:35-38, :175-178).  Writes `scale`
 * typed `input_dtype`, ready to be handed to qk_quantize.
 * Per tensor it needs 4 bytes of device workspace; per block none.
 */
int qk_compute_scales(const QkTensor *input, const QkTensor *scale, const QkScheme *scheme,
                      int input_dtype, void *workspace, size_t workspace_bytes, void *stream);

/*
 * Axis reductions: `cubek_reduce::reduce::<R, Inst>(client, input, output, axis, strategy, ..)`
 * (crates/cubek-reduce/src/lib.rs:93-131) for the instructions MaxAbs, Max and Min
 * (instructions/maxabs.rs:31-87, max.rs, min.rs).  `output` has the input's shape with extent 1 at `axis`
 * (`valid_output_shape`, lib.rs:142-160) and the input's element type, which is also the accumulator type of these
 * instructions in the reference; every result is one of the inputs, hence exact.  Max / Min start from the lowest /
 * highest finite value of the type (their null accumulators).  Both tensors may be strided.
 *
 * `strategy` mirrors `ReduceStrategy { use_planes, shared }` (strategy.rs:7-16): shared = all threads of a CTA
 * reduce one output item together; else use_planes = one warp per item; else one thread per item.  NULL lets the
 * library choose by shape.  The result does not depend on it.
 */
typedef enum { QK_REDUCE_MAXABS = 0, QK_REDUCE_MAX = 1, QK_REDUCE_MIN = 2 } QkReduceInst;
typedef struct {
    int32_t use_planes;
    int32_t shared;
} QkReduceStrategy;
int qk_reduce(const QkTensor *input, const QkTensor *output, int axis, int inst, const QkReduceStrategy *strategy,
              int dtype, void *stream);
/* qk_reduce with QK_REDUCE_MAXABS and the default strategy: the absmax step callers of the quantize path run. */
int qk_reduce_maxabs(const QkTensor *input, const QkTensor *output, int axis, int dtype, void *stream);

/*
 * Fused form of qk_compute_scales + qk_quantize with identical results: per block one
 * pass (absmax, scale, round, clamp, pack in registers); per tensor two passes (grid-wide
 * absmax, then quantize).  `out_scale` is typed as the scheme's param.
 */
int qk_quantize_dynamic(const QkTensor *input, const QkTensor *output, const QkTensor *out_scale,
                        const QkScheme *scheme, int input_dtype,
                        void *workspace, size_t workspace_bytes, void *stream);

/*
 * Sets of tensors (e.g. the weights of a model): the same results as calling
 * qk_quantize_dynamic / qk_dequantize once per tensor, but consecutive tensors that need the same
 * kernel go out as ONE launch (up to 64 tensors each), so that small tensors do not pay a launch
 * gap each.  `inputs`, `outputs`, ... are host arrays of `count` QkTensor.  Per-tensor schemes need
 * 4 bytes of workspace per tensor (at least qk_workspace_bytes()); per-block schemes as
 * qk_quantize_dynamic.  No reference counterpart: the reference launches tensor by tensor.
 */
int qk_quantize_dynamic_batch(int count, const QkTensor *inputs, const QkTensor *outputs,
                              const QkTensor *out_scales, const QkScheme *scheme, int input_dtype,
                              void *workspace, size_t workspace_bytes, void *stream);
int qk_dequantize_batch(int count, const QkTensor *values, const QkTensor *outputs, const QkTensor *params,
                        const QkScheme *scheme, int output_dtype, void *stream);

/*
 * Per-tensor quantize split for tensors sharded over several GPUs: phase 1 leaves the
 * shard's absmax as one f32 in `absmax_out` (device); the caller max-reduces that scalar
 * across ranks (qk_allreduce_max_f32 or any allreduce); phase 2 quantizes with the scale
 * derived on the device from the reduced absmax.  No reference counterpart: the reference
 * is single-device.
 */
int qk_absmax_f32(const QkTensor *input, int input_dtype, float *absmax_out, void *stream);
int qk_quantize_from_absmax(const QkTensor *input, const QkTensor *output, const QkTensor *out_scale,
                            const float *absmax, const QkScheme *scheme, int input_dtype, void *stream);

/* The same split for a set of row-sharded tensors: `absmax_out` / `absmax` hold one f32 per tensor, so a
 * single all-reduce(MAX) of `count` scalars serves the whole set; the quantize launches take up to 64
 * tensors each. */
int qk_absmax_batch(int count, const QkTensor *inputs, int input_dtype, float *absmax_out, void *stream);
int qk_quantize_from_absmax_batch(int count, const QkTensor *inputs, const QkTensor *outputs,
                                  const QkTensor *out_scales, const float *absmax, const QkScheme *scheme,
                                  int input_dtype, void *stream);

/* ncclAllReduce(buf, buf, count, ncclFloat32, ncclMax, comm, stream) on a library-resolved
 * NCCL (libnccl.so.2 already loaded in the process, else dlopen).  `comm` is an ncclComm_t.
 * Enqueues and returns; on a non-blocking communicator it waits (at most 10 s) for the enqueue itself to leave
 * ncclInProgress. */
int qk_allreduce_max_f32(float *buf, size_t count, void *comm, void *stream);

/* The same exchange with a host-side deadline, for callers that must find out when a rank never joins: after the
 * enqueue the call polls `ncclCommGetAsyncError(comm)` and the stream until the collective has completed, the
 * communicator reports an error (QK_ERR_NCCL) or `timeout_ms` has passed (QK_ERR_TIMEOUT).  It blocks the calling
 * thread, never the device; after QK_ERR_TIMEOUT or QK_ERR_NCCL the communicator is the caller's to abort
 * (ncclCommAbort) - the library does not own it.  With a non-blocking communicator (ncclConfig_t.blocking = 0) the
 * enqueue itself is covered by the deadline too. */
int qk_allreduce_max_f32_deadline(float *buf, size_t count, void *comm, void *stream, int timeout_ms);

/*
 * qk_quantize_dynamic for callers that cannot allocate.  (No counterpart in the reference, whose
 * callers always own a memory pool.)
 *
 * Who this is for: code that is handed finished input and output buffers but has no allocator of
 * its own and may not touch the CUDA one - a plug-in running inside a host application that has
 * already carved up the whole device between its components, a callback on a latency-critical
 * thread where the device-wide synchronisation hidden in cudaMalloc / cudaFree is not acceptable,
 * or a process whose memory budget is fixed and audited at start-up.  Such a caller has nowhere
 * to get the workspace that qk_quantize_dynamic asks for.
 *
 * Here the scratch lives in a fixed array inside the library image: qk_noalloc_scratch_bytes()
 * bytes (64 KiB) per GPU that loads the library, held until the process exits.  The call performs
 * no cudaMalloc, cudaFree or other allocating call; input, output and out_scale are still the
 * caller's buffers.  Results are bit-identical to qk_quantize_dynamic.
 *
 *  - Limit: per-tensor schemes and the streaming per-block layouts work at any tensor size (they
 *    need at most one cell of scratch).  Layouts that take the general kernels (N-d blocks, block
 *    sizes that are not a power of two, ragged sizes) stage one input-typed scale per block in the
 *    array; if those do not fit (256 bytes + scales > 64 KiB) the call returns QK_ERR_TOO_LARGE
 *    and launches nothing.
 *  - First call on a device: looks up the array's device address (once per device, with that
 *    device current).  Make that first call during set-up, before any CUDA stream capture begins.
 *  - Sharing: every call on a GPU uses the same array, on whatever stream it is given.  Two calls
 *    whose kernels can overlap on the GPU (different streams, no dependency between them) race on
 *    it; order them with events or keep them on one stream.  The array keeps the previous call's
 *    contents; the part that must start at zero is cleared by each call.
 */
int qk_quantize_dynamic_noalloc(const QkTensor *input, const QkTensor *output, const QkTensor *out_scale,
                                const QkScheme *scheme, int input_dtype, void *stream);
size_t qk_noalloc_scratch_bytes(void);

/* Device workspace for the per-tensor paths (a fixed, small size: 8 KiB).  With at least 4 bytes
 * they still work, through two launches instead of one. */
size_t qk_workspace_bytes(void);
/* Workspace for qk_quantize_dynamic on this input: qk_workspace_bytes() plus, per block, room
 * to stage F-typed scales when the layout is not the streaming one (N-d blocks, ragged sizes). */
size_t qk_workspace_bytes_for(const QkTensor *input, const QkScheme *scheme, int input_dtype);

/*
 * Round trip through HOST buffers: copies `input` (host) to the device in slices, runs
 * qk_quantize_dynamic then qk_dequantize per slice on internal streams, and copies codes,
 * scales and the restored tensor back to host memory.  Slices are whole rows, so results
 * equal the device entry points' for per-block schemes; per-tensor schemes run as one slice.
 * `staging` is a caller-provided DEVICE buffer of at least qk_host_roundtrip_staging_bytes().
 * Blocks until the results are in host memory.
 */
int qk_roundtrip_host(const QkTensor *input, const QkTensor *codes, const QkTensor *out_scale,
                      const QkTensor *restored, const QkScheme *scheme, int input_dtype,
                      void *staging, size_t staging_bytes, int device);
size_t qk_host_roundtrip_staging_bytes(const QkTensor *input, const QkScheme *scheme, int input_dtype);
/* The same for a set of tensors in host memory: the slices of all tensors share one ring of staging slots, so that
 * copies of neighbouring tensors overlap (small tensors - one slice each - would otherwise run upload, kernels and
 * download one after the other).  Slices hold a sixteenth of the call's input, between 16 and 64 MiB, and four of them
 * are in flight: the staging buffer is 0.2 to 0.7 GB.  Results equal qk_roundtrip_host per tensor.  No reference
 * counterpart. */
int qk_roundtrip_host_batch(int count, const QkTensor *inputs, const QkTensor *codes, const QkTensor *out_scales,
                            const QkTensor *restored, const QkScheme *scheme, int input_dtype,
                            void *staging, size_t staging_bytes, int device);
size_t qk_host_roundtrip_staging_bytes_batch(int count, const QkTensor *inputs, const QkScheme *scheme, int input_dtype);

/*
 * Rewrites a packed quantized tensor whose packing does not run along its last dim as a contiguous row-major tensor
 * packed along the last dim: `into_contiguous_packed(client, data, shape, packing, ..)` as called by
 * `MatmulInputHandleRef::into_contiguous` for quantized operands (crates/cubek-matmul/src/base.rs:489-541; packing =
 * num_quants for QK_STORE_U32, 2 for native e2m1x2).  A column-major operand - the transposed view of a tensor
 * quantized along its rows, which the matmul addresses as `(row / packing, col)`
 * (crates/cubek-matmul/src/components/global/memory/layout.rs:131-134) - becomes the row-major operand addressed as
 * `(row, col / packing)`.
 *   input   packed tensor, any strides; its packing runs along its contiguous dim (stride 1); that dim's extent is
 *           ceil(shape[d] / packing), the others equal `shape`; elem_size 4 (u32 words) or 1 (e2m1x2 bytes)
 *   output  contiguous, `shape` with the last dim ceil-divided by `packing`, same elem_size
 *   shape   the logical (unpacked) shape, `rank` entries
 */
int qk_into_contiguous_packed(const QkTensor *input, const QkTensor *output, const int64_t *shape, int rank, int packing,
                              void *stream);

const char *qk_strerror(int status);
const char *qk_version(void);

/* Reads AND CLEARS (synchronously: the call waits for the device) the error flag of the current device: `*flag_out`
 * is non-zero if, since the last call, a kernel gave up on a bounded wait and left its output unwritten.  Only the
 * quantize variant that stages its input through shared memory with bulk copies has such waits.  Entry points
 * are asynchronous and cannot report this themselves: callers that need the guarantee call this after
 * synchronising the stream.  qk_roundtrip_host, which synchronises anyway, checks the flag itself and returns
 * QK_ERR_DEVICE. */
int qk_device_error(int *flag_out);

/* Number of kernels this library has launched in the calling process (for accounting). */
uint64_t qk_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* CUBEK_QUANT_B200_H */
