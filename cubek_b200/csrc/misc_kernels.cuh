// Declarations for the per-tensor absmax reduction and the layout-general fallback kernels.
#pragma once

#include "common.cuh"

namespace qk {

// Host-built description of the scales layout, mirroring BlockScaledLayout /
// PerTensorLayout (crates/cubek-quant/src/layout/scales.rs:66-160).
struct GeneralLayout {
    int rank;
    int per_tensor;
    long long shape[QK_MAX_RANK];          // unpacked value shape
    long long block[QK_MAX_RANK];          // block extents, left-padded with 1
    long long scale_strides[QK_MAX_RANK];  // strides of the scales tensor (elements)
    // strides of the second scales tensor of a quantize call (`out_scale`); the reference builds
    // one view per scales handle (crates/cubek-quant/src/quantize.rs:313, :317)
    long long out_scale_strides[QK_MAX_RANK];
    // strides (elements) of the float tensor: the input of quantize / compute_scales, the output of
    // dequantize.  The reference reaches it through `linear_view`, which honours strides.
    long long data_strides[QK_MAX_RANK];
    int data_contiguous;
    // strides (stored items) of the quantized tensor, whose shape is `shape` with the last dim divided by
    // num_quants.  The reference writes / reads it through `linear_view(.., 1)` (quantize.rs:316), so it may be a
    // strided view too (a transposed matmul operand).
    long long values_strides[QK_MAX_RANK];
    int values_contiguous;
    FastDiv packed_last_div;   // shape[rank - 1] / num_quants
    // Tensors of fewer than 2^31 elements take 32-bit index arithmetic with one multiply-high per
    // division (the 64-bit div/mod chain costs several hundred instructions per stored item).
    int fits31;
    FastDiv shape_div[QK_MAX_RANK];
    FastDiv block_div[QK_MAX_RANK];
};

// Fills fits31 / shape_div / block_div / packed_last_div from rank, shape, block and num_quants.
void finish_layout(GeneralLayout &layout, int nq = 1);

struct GeneralQuantArgs {
    GeneralLayout layout;
    const void *in;
    void *out;
    const void *scale_in;
    void *out_scale;
    const float *absmax;
    long long nitems;  // stored items (u32 words or native bytes)
    int nq, kind, fdt, param;
    float lo, hi, range;
    int force_exact;   // 1: IEEE division for every element (filled by the launcher from the launch knobs)
    int vector_bytes;  // 16 / 8: an item's elements are read as vectors of that size; 0: one by one (filled by the launcher)
};

struct GeneralDequantArgs {
    GeneralLayout layout;
    const void *values;
    const void *params;
    void *out;
    long long nitems;
    int nq, kind, fdt, param;
    int vector_bytes;  // like GeneralQuantArgs::vector_bytes, for the stores
};

struct GeneralScalesArgs {
    GeneralLayout layout;
    const void *in;
    void *scale_out;
    long long nblocks;
    int fdt;
    float range;
};

// absmax of `n` elements max-reduced into `*cell` (bit pattern of a non-negative f32).  The cell
// must hold zero (or an earlier partial result) beforehand; `zero_first` clears it on the stream.
// `row_stride` (optional): rows of whole 16-byte chunks, a constant number of bytes apart, 16-byte aligned.
cudaError_t launch_absmax(int fdt, const void *in, long long n, unsigned int *cell, const LaunchCfg &cfg,
                          cudaStream_t stream, bool zero_first = true, const RowStride *row_stride = nullptr);
// absmax of every tensor of a batch in one launch.  `chunk_end` counts 16-byte chunks across the batch;
// every tensor must start on a 16-byte boundary and hold a whole number of chunks.  `cells[i]` must be
// zero (or hold an earlier partial result) beforehand.
constexpr int QK_ABSMAX_BATCH = 128;
struct AbsmaxBatchArgs {
    const void *in[QK_ABSMAX_BATCH];
    long long chunk_end[QK_ABSMAX_BATCH];
    int ntensors;
    unsigned int *cells;
};
cudaError_t launch_absmax_batch(int fdt, const AbsmaxBatchArgs &args, const LaunchCfg &cfg, cudaStream_t stream);
cudaError_t launch_finalize_scale(const unsigned int *cell, void *scale_out, int fdt, float range,
                                  cudaStream_t stream);
cudaError_t launch_general_quantize(const GeneralQuantArgs &a, const LaunchCfg &cfg, cudaStream_t stream);
cudaError_t launch_general_dequantize(const GeneralDequantArgs &a, const LaunchCfg &cfg, cudaStream_t stream);
cudaError_t launch_general_scales(const GeneralScalesArgs &a, const LaunchCfg &cfg, cudaStream_t stream);
// absmax of a strided tensor into `*cell` (cleared first on the stream).
cudaError_t launch_absmax_strided(const GeneralLayout &layout, const void *in, int fdt, long long n, unsigned int *cell,
                                  const LaunchCfg &cfg, cudaStream_t stream);

// max |x| over `len` elements of stride `inner`, for every (outer, inner) position.
// `into_contiguous_packed` (repack.cu): gathers the fields of a packed tensor whose packing runs along `packed_dim`
// into a contiguous row-major tensor packed along the last dim.
struct RepackArgs {
    int rank, packed_dim, packing, bits, item_bytes;
    long long shape[QK_MAX_RANK];        // logical (unpacked) shape
    long long in_strides[QK_MAX_RANK];   // strides of the packed input (items)
    const void *in;
    void *out;
    long long nitems_out;
};
cudaError_t launch_repack(const RepackArgs &a, const LaunchCfg &cfg, cudaStream_t stream);
// Axis reductions (reduce.cu).  inst: 0 MaxAbs, 1 Max, 2 Min.
cudaError_t launch_reduce_contiguous(int fdt, int inst, const void *in, void *out, long long outer, long long len,
                                     long long inner, int units_per_item, const LaunchCfg &cfg, cudaStream_t stream);
cudaError_t launch_reduce_strided(int fdt, int inst, const QkTensor *input, const QkTensor *output, int axis,
                                  const LaunchCfg &cfg, cudaStream_t stream);

}  // namespace qk
