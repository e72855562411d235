// Dequantize kernels instantiated for every (float type, stored-code kind, unit size).
#include "dequantize_kernels.cuh"

namespace qk {

template <typename Kernel> static int resident_ctas_per_sm(Kernel kernel, int threads)
{
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, 0) != cudaSuccess || n < 1) n = 1;
    return n;
}

template <int FDT, int KIND, int OB, bool TILES, int SUB = 1>
static cudaError_t launch_tiles(const DequantArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    const int threads = cfg.threads;
    static const int occ256 = resident_ctas_per_sm(dequantize_kernel<FDT, KIND, OB, TILES, SUB>, 256);
    // The write-heavy kernel runs faster as many short CTAs than as one persistent wave (CTAs
    // drift apart, so loads, arithmetic and stores of different CTAs overlap): 12 waves by default
    // (bf16 q4 batch: 5750 GB/s as one wave, 6480 at 8 waves, 6540 at 12).
    // Short launches (the shards of an 8-way split: 0.5 GB of output per launch) want fewer, longer CTAs: at least
    // one and a half rounds of 4 units per thread, down to 4 waves (6100 GB/s at 12 waves, 6350 at 6, 6390 at 4).
    int waves = cfg.dequant_waves > 0 ? cfg.dequant_waves : 1;
    const long long fit = args.nunits / ((long long)cfg.sm_count * occ256 * threads * 6);
    if (fit < waves) waves = (int)(fit > 4 ? fit : (waves < 4 ? waves : 4));
    const int per_sm = (cfg.ctas_per_sm > 0) ? cfg.ctas_per_sm : occ256 * waves;
    long long need = (args.nunits + (long long)threads * 4 - 1) / ((long long)threads * 4);
    const long long cap = (long long)cfg.sm_count * per_sm;
    if (need > cap) need = cap;
    if (need < 1) need = 1;
    return launch_kernel(dequantize_kernel<FDT, KIND, OB, TILES, SUB>, (int)need, threads, stream, cfg.pdl != 0, args);
}

template <int FDT, int KIND, int OB>
static cudaError_t launch_one(int sub, const DequantArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    if constexpr (OB == 64 && FDT != QK_F32 && DUnitT<FDT, KIND, 64>::IW % 2 == 0) {
        if (sub == 2 && !args.b2.enabled) return launch_tiles<FDT, KIND, OB, false, 2>(args, cfg, stream);
    }
    if (sub != 1) return cudaErrorInvalidValue;
    return args.b2.enabled ? launch_tiles<FDT, KIND, OB, true>(args, cfg, stream)
                           : launch_tiles<FDT, KIND, OB, false>(args, cfg, stream);
}

template <int FDT, int KIND>
static cudaError_t launch_unit(int out_bytes, int sub, const DequantArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    constexpr int MINB = min_dequant_bytes(FDT, KIND);
    if (out_bytes == 64) return launch_one<FDT, KIND, 64>(sub, args, cfg, stream);
    if constexpr (MINB < 64) {
        if (out_bytes == MINB) return launch_one<FDT, KIND, MINB>(sub, args, cfg, stream);
    }
    return cudaErrorInvalidValue;
}

template <int FDT>
static cudaError_t launch_kind(int kind, int out_bytes, int sub, const DequantArgs &args, const LaunchCfg &cfg,
                               cudaStream_t stream)
{
    switch (kind) {
    case KIND_PACK8: return launch_unit<FDT, KIND_PACK8>(out_bytes, sub, args, cfg, stream);
    case KIND_PACK4: return launch_unit<FDT, KIND_PACK4>(out_bytes, sub, args, cfg, stream);
    case KIND_PACK2: return launch_unit<FDT, KIND_PACK2>(out_bytes, sub, args, cfg, stream);
    case KIND_I8: return launch_unit<FDT, KIND_I8>(out_bytes, sub, args, cfg, stream);
    case KIND_E2M1: return launch_unit<FDT, KIND_E2M1>(out_bytes, sub, args, cfg, stream);
    case KIND_E4M3: return launch_unit<FDT, KIND_E4M3>(out_bytes, sub, args, cfg, stream);
    case KIND_E5M2: return launch_unit<FDT, KIND_E5M2>(out_bytes, sub, args, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_dequantize(int fdt, int kind, int out_bytes, int sub, const DequantArgs &args, const LaunchCfg &cfg,
                              cudaStream_t stream)
{
    switch (fdt) {
    case QK_F32: return launch_kind<QK_F32>(kind, out_bytes, sub, args, cfg, stream);
    case QK_F16: return launch_kind<QK_F16>(kind, out_bytes, sub, args, cfg, stream);
    case QK_BF16: return launch_kind<QK_BF16>(kind, out_bytes, sub, args, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace qk
