// Quantize kernels instantiated for f32 inputs.
#include "quantize_inst.cuh"

namespace qk {
cudaError_t launch_quantize_f32(int kind, int unit_bytes, bool dyn, bool clamp, int sub, const QuantArgs &args,
                               const LaunchCfg &cfg, cudaStream_t stream)
{
    return launch_quantize_t<QK_F32>(kind, unit_bytes, dyn, clamp, sub, args, cfg, stream);
}
cudaError_t launch_block_scales_f32(const void *in, void *scale_out, long long nunits, int unit_bytes, int lg,
                                     float range, float inv_range, const RowStride &rs, const LaunchCfg &cfg,
                                     cudaStream_t stream)
{
    return launch_block_scales_t<QK_F32>(in, scale_out, nunits, unit_bytes, lg, range, inv_range, rs, cfg, stream);
}
cudaError_t launch_quantize_tensor_f32(int kind, QuantTensorArgs &args, int partials_capacity, const LaunchCfg &cfg,
                                      cudaStream_t stream)
{
    return launch_quantize_tensor_t<QK_F32>(kind, args, partials_capacity, cfg, stream);
}
cudaError_t launch_block_scales_2d_f32(const void *in, void *scale_out, long long rows, long long cols, int block_rows,
                                      int block_cols, float range, float inv_range, const LaunchCfg &cfg,
                                      cudaStream_t stream)
{
    return launch_block_scales_2d_t<QK_F32>(in, scale_out, rows, cols, block_rows, block_cols, range, inv_range, cfg, stream);
}
}  // namespace qk
