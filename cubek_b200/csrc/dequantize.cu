// Dequantize kernels instantiated for every (float type, stored-code kind).
#include "dequantize_kernels.cuh"

namespace qk {

template <int FDT, int KIND>
static cudaError_t launch_one(const DequantArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    const int threads = cfg.threads;
    long long need = (args.nunits + (long long)threads * 4 - 1) / ((long long)threads * 4);
    const long long cap = (long long)cfg.sm_count * cfg.ctas_per_sm;
    if (need > cap) need = cap;
    if (need < 1) need = 1;
    dequantize_kernel<FDT, KIND><<<(int)need, threads, 0, stream>>>(args);
    return cudaGetLastError();
}

template <int FDT>
static cudaError_t launch_kind(int kind, const DequantArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    switch (kind) {
    case KIND_PACK8: return launch_one<FDT, KIND_PACK8>(args, cfg, stream);
    case KIND_PACK4: return launch_one<FDT, KIND_PACK4>(args, cfg, stream);
    case KIND_PACK2: return launch_one<FDT, KIND_PACK2>(args, cfg, stream);
    case KIND_I8: return launch_one<FDT, KIND_I8>(args, cfg, stream);
    case KIND_E2M1: return launch_one<FDT, KIND_E2M1>(args, cfg, stream);
    case KIND_E4M3: return launch_one<FDT, KIND_E4M3>(args, cfg, stream);
    case KIND_E5M2: return launch_one<FDT, KIND_E5M2>(args, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_dequantize(int fdt, int kind, const DequantArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    switch (fdt) {
    case QK_F32: return launch_kind<QK_F32>(kind, args, cfg, stream);
    case QK_F16: return launch_kind<QK_F16>(kind, args, cfg, stream);
    case QK_BF16: return launch_kind<QK_BF16>(kind, args, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

int dequant_unit_elems(int fdt, int kind)
{
    const int size = (fdt == QK_F32) ? 4 : 2;
    return cmax(32 / size, kind_elems_per_u32(kind));
}

}  // namespace qk
