// Quantize kernels instantiated for f16 inputs.
#include "quantize_inst.cuh"

namespace qk {
cudaError_t launch_quantize_f16(int kind, bool dyn, const QuantArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    return launch_quantize_t<QK_F16>(kind, dyn, args, cfg, stream);
}
cudaError_t launch_block_scales_f16(const void *in, void *scale_out, long long nchunks, int lg, float range,
                                   const LaunchCfg &cfg, cudaStream_t stream)
{
    return launch_block_scales_t<QK_F16>(in, scale_out, nchunks, lg, range, cfg, stream);
}
}  // namespace qk
