// Kernel instantiation + launch for one float type; included by quantize_f32.cu,
// quantize_f16.cu and quantize_bf16.cu so that the three compile in parallel.
#pragma once

#include "quantize_kernels.cuh"

namespace qk {

template <int FDT, int KIND, bool DYN>
static cudaError_t launch_one(const QuantArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    constexpr int UNR = 64 / Unit<FDT, KIND>::IN_BYTES;
    const int threads = cfg.threads;
    long long need = (args.nunits + (long long)threads * UNR - 1) / ((long long)threads * UNR);
    const long long cap = (long long)cfg.sm_count * cfg.ctas_per_sm;
    if (need > cap) need = cap;
    if (need < 1) need = 1;
    quantize_kernel<FDT, KIND, DYN><<<(int)need, threads, 0, stream>>>(args);
    return cudaGetLastError();
}

template <int FDT, bool DYN>
static cudaError_t launch_kind(int kind, const QuantArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    switch (kind) {
    case KIND_PACK8: return launch_one<FDT, KIND_PACK8, DYN>(args, cfg, stream);
    case KIND_PACK4: return launch_one<FDT, KIND_PACK4, DYN>(args, cfg, stream);
    case KIND_PACK2: return launch_one<FDT, KIND_PACK2, DYN>(args, cfg, stream);
    case KIND_I8: return launch_one<FDT, KIND_I8, DYN>(args, cfg, stream);
    case KIND_E2M1: return launch_one<FDT, KIND_E2M1, DYN>(args, cfg, stream);
    case KIND_E4M3: return launch_one<FDT, KIND_E4M3, DYN>(args, cfg, stream);
    case KIND_E5M2: return launch_one<FDT, KIND_E5M2, DYN>(args, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

template <int FDT>
static cudaError_t launch_quantize_t(int kind, bool dyn, const QuantArgs &args, const LaunchCfg &cfg,
                                     cudaStream_t stream)
{
    return dyn ? launch_kind<FDT, true>(kind, args, cfg, stream) : launch_kind<FDT, false>(kind, args, cfg, stream);
}

template <int FDT>
static cudaError_t launch_block_scales_t(const void *in, void *scale_out, long long nchunks, int lg, float range,
                                         const LaunchCfg &cfg, cudaStream_t stream)
{
    const int threads = cfg.threads;
    long long need = (nchunks + (long long)threads * 4 - 1) / ((long long)threads * 4);
    const long long cap = (long long)cfg.sm_count * cfg.ctas_per_sm;
    if (need > cap) need = cap;
    if (need < 1) need = 1;
    block_scales_kernel<FDT><<<(int)need, threads, 0, stream>>>(in, scale_out, nchunks, lg, range);
    return cudaGetLastError();
}

}  // namespace qk
