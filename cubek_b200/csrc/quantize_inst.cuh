// Kernel instantiation + launch for one float type; included by quantize_f32.cu,
// quantize_f16.cu and quantize_bf16.cu so that the three compile in parallel.
#pragma once

#include <mutex>

#include "quantize_kernels.cuh"

namespace qk {

// Grids are whole waves of resident CTAs (or fewer CTAs when the tensor is small): a partial
// last wave leaves SMs idle while the others finish (measured: 3 or 6 CTAs/SM for a kernel that
// holds 3 run at 6500 GB/s, 4 or 8 at 5100-6100).
template <typename Kernel> static int resident_ctas_per_sm(Kernel kernel, int threads)
{
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, 0) != cudaSuccess || n < 1) n = 1;
    return n;
}

template <int FDT, int KIND, int UB, bool DYN, bool CLAMP, int SUB = 1, bool LG0 = false, bool ONE_SITE = false>
static cudaError_t launch_one(const QuantArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    constexpr int UNR = (UB >= 64) ? 2 : 4;
    const int threads = cfg.threads;
    static const int occ256 = resident_ctas_per_sm(quantize_kernel<FDT, KIND, UB, DYN, CLAMP, SUB, LG0, ONE_SITE>, 256);
    const int per_sm = (cfg.ctas_per_sm > 0) ? cfg.ctas_per_sm : occ256 * (cfg.quant_waves > 0 ? cfg.quant_waves : 1);
    long long need = (args.nunits + (long long)threads * UNR - 1) / ((long long)threads * UNR);
    const long long cap = (long long)cfg.sm_count * per_sm;
    if (need > cap) need = cap;
    if (need < 1) need = 1;
    // cfg.staged: 0 = units below 64 bytes, 1 = always, 2 = never
    if constexpr (SUB == 1 && !LG0 && !ONE_SITE) {
        if ((cfg.staged == 1 || (cfg.staged == 0 && UB < 64)) && threads == 256 && !args.rs.enabled) {
            // bulk-copy staged variant: cfg.stages x 16 KB stages + barriers per CTA, a whole number of waves
            const int nstages = cfg.stages < 2 ? 2 : (cfg.stages > QK_MAX_STAGES ? QK_MAX_STAGES : cfg.stages);
            const int SMEM = nstages * QK_TILE_BYTES + QK_MAX_STAGES * 8;
            int dev = 0;
            if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
            // The opt-in to more than 48 KiB of dynamic shared memory is a per-device attribute of the kernel.
            struct Occupancy {
                int per_sm[QK_MAX_STAGES + 1];
                bool ready;
            };
            static Occupancy occupancy[64];
            static std::mutex occupancy_mutex;
            int occ_staged;
            {
                std::lock_guard<std::mutex> lock(occupancy_mutex);
                Occupancy &o = occupancy[dev];
                if (!o.ready) {
                    cudaFuncSetAttribute(quantize_staged_kernel<FDT, KIND, UB, DYN, CLAMP>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         QK_MAX_STAGES * QK_TILE_BYTES + QK_MAX_STAGES * 8);
                    for (int n = 0; n <= QK_MAX_STAGES; ++n) {
                        o.per_sm[n] = 1;
                        if (n >= 2 &&
                            (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o.per_sm[n], quantize_staged_kernel<FDT, KIND, UB, DYN, CLAMP>,
                                                                           256, n * QK_TILE_BYTES + QK_MAX_STAGES * 8) != cudaSuccess ||
                             o.per_sm[n] < 1))
                            o.per_sm[n] = 1;
                    }
                    o.ready = true;
                }
                occ_staged = o.per_sm[nstages];
            }
            int *flag = stage_error_flag();
            if (flag != nullptr) {
                long long tiles = args.t[args.ntensors - 1].tile_end;
                const long long cap2 = (long long)cfg.sm_count * occ_staged;
                if (tiles > cap2) tiles = cap2;
                if (tiles < 1) tiles = 1;
                cudaLaunchConfig_t lc = {};
                lc.gridDim = dim3((unsigned)tiles, 1, 1);
                lc.blockDim = dim3(256, 1, 1);
                lc.dynamicSmemBytes = SMEM;
                lc.stream = stream;
                cudaLaunchAttribute attr[1];
                attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr[0].val.programmaticStreamSerializationAllowed = 1;
                lc.attrs = attr;
                lc.numAttrs = cfg.pdl ? 1 : 0;
                return cudaLaunchKernelEx(&lc, quantize_staged_kernel<FDT, KIND, UB, DYN, CLAMP>, args, flag, nstages);
            }
        }
    }
    QuantArgs split_args = args;
    split_args.split = make_pass_split(args.nunits, need, threads, UNR);
    return launch_kernel(quantize_kernel<FDT, KIND, UB, DYN, CLAMP, SUB, LG0, ONE_SITE>, (int)need, threads, stream, cfg.pdl != 0,
                         split_args);
}

// The fused form with one block per unit (lg == 0) and 64-byte units has a kernel of its own without the
// shuffle rounds; smaller units keep the staged route, which takes lg at run time.
template <int FDT, int KIND, int UB>
static cudaError_t launch_mode(bool dyn, bool clamp, int sub, const QuantArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    if constexpr (UB == 64 && FDT != QK_F32 && (UB / 2) >= min_unit_bytes(FDT, KIND)) {
        if (sub == 2) {
            if (!dyn) return launch_one<FDT, KIND, UB, false, true, 2, true>(args, cfg, stream);
            return clamp ? launch_one<FDT, KIND, UB, true, true, 2, true>(args, cfg, stream)
                         : launch_one<FDT, KIND, UB, true, false, 2, true>(args, cfg, stream);
        }
    }
    if (sub != 1) return cudaErrorInvalidValue;
    if (!dyn) {
        // per tensor from absmax cells, 16-bit inputs, 64-byte units: the one-site walk (see common.cuh)
        if constexpr (UB == 64 && FDT != QK_F32) {
            if (args.absmax != nullptr && cfg.staged != 1) return launch_one<FDT, KIND, UB, false, true, 1, false, true>(args, cfg, stream);
        }
        return launch_one<FDT, KIND, UB, false, true>(args, cfg, stream);
    }
    if constexpr (UB == 64) {
        if (args.lg_units_per_block == 0)
            return clamp ? launch_one<FDT, KIND, UB, true, true, 1, true>(args, cfg, stream)
                         : launch_one<FDT, KIND, UB, true, false, 1, true>(args, cfg, stream);
    }
    if (clamp) return launch_one<FDT, KIND, UB, true, true>(args, cfg, stream);
    return launch_one<FDT, KIND, UB, true, false>(args, cfg, stream);
}

template <int FDT, int KIND>
static cudaError_t launch_unit(int unit_bytes, bool dyn, bool clamp, int sub, const QuantArgs &args, const LaunchCfg &cfg,
                               cudaStream_t stream)
{
    constexpr int MINB = min_unit_bytes(FDT, KIND);
    if (unit_bytes == 64) return launch_mode<FDT, KIND, 64>(dyn, clamp, sub, args, cfg, stream);
    if constexpr (MINB < 32) {
        if (unit_bytes == 32) return launch_mode<FDT, KIND, 32>(dyn, clamp, sub, args, cfg, stream);
    }
    if constexpr (MINB < 64) {
        if (unit_bytes == MINB) return launch_mode<FDT, KIND, MINB>(dyn, clamp, sub, args, cfg, stream);
    }
    return cudaErrorInvalidValue;
}

template <int FDT>
static cudaError_t launch_quantize_t(int kind, int unit_bytes, bool dyn, bool clamp, int sub, const QuantArgs &args,
                                     const LaunchCfg &cfg, cudaStream_t stream)
{
    switch (kind) {
    case KIND_PACK8: return launch_unit<FDT, KIND_PACK8>(unit_bytes, dyn, clamp, sub, args, cfg, stream);
    case KIND_PACK4: return launch_unit<FDT, KIND_PACK4>(unit_bytes, dyn, clamp, sub, args, cfg, stream);
    case KIND_PACK2: return launch_unit<FDT, KIND_PACK2>(unit_bytes, dyn, clamp, sub, args, cfg, stream);
    case KIND_I8: return launch_unit<FDT, KIND_I8>(unit_bytes, dyn, clamp, sub, args, cfg, stream);
    case KIND_E2M1: return launch_unit<FDT, KIND_E2M1>(unit_bytes, dyn, clamp, sub, args, cfg, stream);
    case KIND_E4M3: return launch_unit<FDT, KIND_E4M3>(unit_bytes, dyn, clamp, sub, args, cfg, stream);
    case KIND_E5M2: return launch_unit<FDT, KIND_E5M2>(unit_bytes, dyn, clamp, sub, args, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

template <int FDT, int KIND, bool CLAMP>
static cudaError_t launch_tensor_clamp(QuantTensorArgs &args, int partials_capacity, const LaunchCfg &cfg,
                                     cudaStream_t stream)
{
    constexpr int MAX_SMEM = QK_TENSOR_SMEM_ROWS * QK_TENSOR_ROW_BYTES;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    // The opt-in to more than 48 KiB of dynamic shared memory is a per-device attribute of the kernel.
    static int occupancy[64];
    static std::mutex occupancy_mutex;
    int occ;
    {
        std::lock_guard<std::mutex> lock(occupancy_mutex);
        if (occupancy[dev] == 0) {
            int n = 0;
            if (cudaFuncSetAttribute(quantize_tensor_kernel<FDT, KIND, 64, CLAMP>, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM) !=
                    cudaSuccess ||
                cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quantize_tensor_kernel<FDT, KIND, 64, CLAMP>, 256, MAX_SMEM) != cudaSuccess ||
                n < 1) {
                (void)cudaGetLastError();
                n = -1;
            }
            occupancy[dev] = n;
        }
        occ = occupancy[dev];
    }
    if (occ < 1) return cudaErrorInvalidValue;
    long long need = (args.nunits + 256ll * 2 - 1) / (256ll * 2);
    const long long cap = (long long)cfg.sm_count * occ;   // all CTAs must be resident (grid barrier)
    if (need > cap) need = cap;
    if (need < 1) need = 1;
    if (need > partials_capacity) return cudaErrorInvalidValue;
    // the same row arithmetic as the kernel's
    const long long row_units = need * 256;
    const int nrows = (int)((args.nunits + row_units - 1) / row_units);
    const int reg_row = nrows - 4;
    int smem_rows = cfg.tensor_smem_rows >= 0 ? cfg.tensor_smem_rows : QK_TENSOR_SMEM_ROWS;
    if (smem_rows > QK_TENSOR_SMEM_ROWS) smem_rows = QK_TENSOR_SMEM_ROWS;
    if (smem_rows > reg_row) smem_rows = reg_row > 0 ? reg_row : 0;
    args.smem_rows = smem_rows;
    void *params[] = {&args};
    return cudaLaunchCooperativeKernel(reinterpret_cast<void *>(quantize_tensor_kernel<FDT, KIND, 64, CLAMP>), dim3((unsigned)need),
                                       dim3(256), params, (size_t)smem_rows * QK_TENSOR_ROW_BYTES, stream);
}

template <int FDT, int KIND>
static cudaError_t launch_tensor_one(QuantTensorArgs &args, int partials_capacity, const LaunchCfg &cfg, cudaStream_t stream)
{
    const bool clamp = need_clamp(FDT, KIND, true, args.lo == -args.hi, args.param);
    return clamp ? launch_tensor_clamp<FDT, KIND, true>(args, partials_capacity, cfg, stream)
                 : launch_tensor_clamp<FDT, KIND, false>(args, partials_capacity, cfg, stream);
}

template <int FDT>
static cudaError_t launch_quantize_tensor_t(int kind, QuantTensorArgs &args, int partials_capacity,
                                            const LaunchCfg &cfg, cudaStream_t stream)
{
    switch (kind) {
    case KIND_PACK8: return launch_tensor_one<FDT, KIND_PACK8>(args, partials_capacity, cfg, stream);
    case KIND_PACK4: return launch_tensor_one<FDT, KIND_PACK4>(args, partials_capacity, cfg, stream);
    case KIND_PACK2: return launch_tensor_one<FDT, KIND_PACK2>(args, partials_capacity, cfg, stream);
    case KIND_I8: return launch_tensor_one<FDT, KIND_I8>(args, partials_capacity, cfg, stream);
    case KIND_E2M1: return launch_tensor_one<FDT, KIND_E2M1>(args, partials_capacity, cfg, stream);
    case KIND_E4M3: return launch_tensor_one<FDT, KIND_E4M3>(args, partials_capacity, cfg, stream);
    case KIND_E5M2: return launch_tensor_one<FDT, KIND_E5M2>(args, partials_capacity, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

template <int FDT, int UB>
static cudaError_t launch_block_scales_unit(const void *in, void *scale_out, long long nunits, int lg, float range,
                                            float inv_range, const RowStride &rs, const LaunchCfg &cfg, cudaStream_t stream)
{
    constexpr int UNR = (UB >= 64) ? 2 : 4;
    const int threads = 256;
    static const int occ = resident_ctas_per_sm(block_scales_kernel<FDT, UB>, 256);
    long long need = (nunits + (long long)threads * UNR - 1) / ((long long)threads * UNR);
    const long long cap = (long long)cfg.sm_count * occ;
    if (need > cap) need = cap;
    if (need < 1) need = 1;
    const int aligned32 = ((reinterpret_cast<uintptr_t>(in) & 31u) == 0 && (!rs.enabled || rs.row_bytes % 32 == 0)) ? 1 : 0;
    return launch_kernel(block_scales_kernel<FDT, UB>, (int)need, threads, stream, cfg.pdl != 0, in, scale_out, nunits, lg,
                         range, inv_range, aligned32, rs, make_pass_split(nunits, need, threads, UNR));
}

template <int FDT>
static cudaError_t launch_block_scales_t(const void *in, void *scale_out, long long nunits, int unit_bytes, int lg,
                                         float range, float inv_range, const RowStride &rs, const LaunchCfg &cfg,
                                         cudaStream_t stream)
{
    switch (unit_bytes) {
    case 64: return launch_block_scales_unit<FDT, 64>(in, scale_out, nunits, lg, range, inv_range, rs, cfg, stream);
    case 32: return launch_block_scales_unit<FDT, 32>(in, scale_out, nunits, lg, range, inv_range, rs, cfg, stream);
    case 16: return launch_block_scales_unit<FDT, 16>(in, scale_out, nunits, lg, range, inv_range, rs, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

template <int FDT>
static cudaError_t launch_block_scales_2d_t(const void *in, void *scale_out, long long rows, long long cols,
                                            int block_rows, int block_cols, float range, float inv_range,
                                            const LaunchCfg &cfg, cudaStream_t stream)
{
    const long long tiles = ((rows + block_rows - 1) / block_rows) * (cols / block_cols);
    const long long chunks = (long long)block_rows * block_cols * ((FDT == QK_F32) ? 4 : 2) / 16;
    const int cta_per_tile = chunks >= 1024 ? 1 : 0;
    long long need = cta_per_tile ? tiles : (tiles + 7) / 8;   // else 8 warps per CTA, one tile per warp
    const long long cap = (long long)cfg.sm_count * 8;
    if (need > cap) need = cap;
    if (need < 1) need = 1;
    return launch_kernel(block_scales_2d_kernel<FDT>, (int)need, 256, stream, cfg.pdl != 0, in, scale_out, rows, cols,
                         block_rows, block_cols, range, inv_range, cta_per_tile);
}

}  // namespace qk
