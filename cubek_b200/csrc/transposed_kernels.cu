// Quantize / dequantize of a TRANSPOSED matrix view: a logical [R, C] float tensor whose element (r, c)
// sits at c * ld + r (the view `w.t()` of a row-major [C, R] matrix).  Blocks and packed words run along
// the logical last dim, i.e. across memory rows, so the streaming kernels' contiguous units do not exist
// here.  Instead consecutive lanes take consecutive logical rows r for the same run of columns: every
// element load / store of a warp is one contiguous segment of a memory row (coalesced), each lane gathers
// its unit in registers, and the arithmetic, the scale handling and the layout of codes and scales are
// those of the streaming kernels (the quantized tensor and the scales are contiguous in logical order).
//
// The reference reaches such a tensor through `linear_view`, which honours strides
// (crates/cubek-quant/src/quantize.rs:234-239); results are identical to quantizing a contiguous copy.
#include "dequantize_kernels.cuh"
#include "quantize_kernels.cuh"

namespace qk {

template <int FDT> __device__ __forceinline__ uint32_t load_elem_bits(const char *p)
{
    if constexpr (FDT == QK_F32) return __ldg(reinterpret_cast<const unsigned int *>(p));
    else return __ldg(reinterpret_cast<const unsigned short *>(p));
}

// Work item w -> (column unit cu, logical row r) with r fastest, so that a warp covers 32 consecutive rows.
struct TransposedIndex {
    unsigned r, cu;
    long long li;   // unit index in logical (row-major) order
};
__device__ __forceinline__ TransposedIndex transposed_index(const Transposed &tr, unsigned w)
{
    TransposedIndex t;
    t.cu = fastdiv(w, tr.rows);
    t.r = w - t.cu * tr.rows.div;
    t.li = (long long)t.r * tr.units_per_row + t.cu;
    return t;
}

template <int FDT, int KIND, int UB, bool DYN, bool CLAMP>
__global__ void __launch_bounds__(256) quantize_transposed_kernel(const QuantArgs a)
{
    using UT = UnitT<FDT, KIND, UB>;
    constexpr int RAW = UT::RAW;
    constexpr int U = UT::U;
    constexpr int ESZ = UT::ESZ;
    using F = typename ElemOf<FDT>::type;
    const QuantTensor &T = a.t[0];
    const char *in = static_cast<const char *>(T.in);
    const bool aligned32 = a.aligned32 != 0;
    const int lg = a.lg_units_per_block;   // 0 (a unit is a block) or -1 (per tensor)
    pdl_entry();
    float tensor_scale = 0.0f;
    bool have_tensor_scale = false;
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < a.nunits;
         w += (long long)gridDim.x * blockDim.x) {
        const TransposedIndex ix = transposed_index(a.tr, (unsigned)w);
        const char *p = in + ((long long)ix.cu * U * a.tr.ld + ix.r) * ESZ;
        const long long step = a.tr.ld * ESZ;
        uint32_t raw[RAW];
        if constexpr (FDT == QK_F32) {
#pragma unroll
            for (int i = 0; i < U; ++i) raw[i] = load_elem_bits<FDT>(p + i * step);
        } else {
#pragma unroll
            for (int i = 0; i < U; i += 2)
                raw[i / 2] = load_elem_bits<FDT>(p + i * step) | (load_elem_bits<FDT>(p + (i + 1) * step) << 16);
        }
        float scale_f;
        long long sidx = 0;
        bool starts;
        if constexpr (DYN) {
            sidx = ix.li;
            starts = true;
            scale_f = fused_unit_scale<FDT, RAW>(raw, 0, a.range, a.inv_range);
        } else if (lg < 0) {
            if (!have_tensor_scale) {
                have_tensor_scale = true;
                tensor_scale = tensor_unit_scale<FDT>(a, T, 0);
            }
            scale_f = tensor_scale;
            starts = (ix.li == 0);
        } else {
            sidx = ix.li;
            starts = true;
            scale_f = static_cast<float>(static_cast<const F *>(T.scale_in)[sidx]);
        }
        finish_unit<FDT, KIND, UB, DYN, CLAMP>(a, T, raw, scale_f, sidx, starts, ix.li, true, aligned32);
    }
}

// 16-bit types, even number of rows, even ld, 4-byte aligned base: a lane takes TWO adjacent logical rows and
// reads them with one 32-bit load per column (128 bytes per warp instead of 64), then separates the two
// units with byte permutes.  `a.tr.rows` holds rows / 2 here; a.nunits counts row pairs x column units.
template <int FDT, int KIND, int UB, bool DYN, bool CLAMP>
__global__ void __launch_bounds__(256) quantize_transposed_pair_kernel(const QuantArgs a)
{
    using UT = UnitT<FDT, KIND, UB>;
    constexpr int RAW = UT::RAW;
    constexpr int U = UT::U;
    static_assert(FDT != QK_F32, "pairs of rows are for 16-bit types");
    using F = typename ElemOf<FDT>::type;
    const QuantTensor &T = a.t[0];
    const char *in = static_cast<const char *>(T.in);
    const bool aligned32 = a.aligned32 != 0;
    const int lg = a.lg_units_per_block;
    pdl_entry();
    float tensor_scale = 0.0f;
    bool have_tensor_scale = false;
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < a.nunits;
         w += (long long)gridDim.x * blockDim.x) {
        const unsigned cu = fastdiv((unsigned)w, a.tr.rows);
        const unsigned r = 2u * ((unsigned)w - cu * a.tr.rows.div);
        const char *p = in + ((long long)cu * U * a.tr.ld + r) * 2;
        const long long step = a.tr.ld * 2;
        uint32_t raw[2][RAW];
#pragma unroll
        for (int i = 0; i < U; i += 2) {
            const uint32_t w0 = __ldg(reinterpret_cast<const unsigned int *>(p + i * step));         // (row r, row r+1) at column i
            const uint32_t w1 = __ldg(reinterpret_cast<const unsigned int *>(p + (i + 1) * step));   // ... at column i+1
            raw[0][i / 2] = __byte_perm(w0, w1, 0x5410);
            raw[1][i / 2] = __byte_perm(w0, w1, 0x7632);
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const long long li = (long long)(r + k) * a.tr.units_per_row + cu;
            float scale_f;
            long long sidx = 0;
            bool starts;
            if constexpr (DYN) {
                sidx = li;
                starts = true;
                scale_f = fused_unit_scale<FDT, RAW>(raw[k], 0, a.range, a.inv_range);
            } else if (lg < 0) {
                if (!have_tensor_scale) {
                    have_tensor_scale = true;
                    tensor_scale = tensor_unit_scale<FDT>(a, T, 0);
                }
                scale_f = tensor_scale;
                starts = (li == 0);
            } else {
                sidx = li;
                starts = true;
                scale_f = static_cast<float>(static_cast<const F *>(T.scale_in)[sidx]);
            }
            finish_unit<FDT, KIND, UB, DYN, CLAMP>(a, T, raw[k], scale_f, sidx, starts, li, true, aligned32);
        }
    }
}

template <int FDT, int KIND, int OB>
__global__ void __launch_bounds__(256) dequantize_transposed_kernel(const DequantArgs a)
{
    using DU = DUnitT<FDT, KIND, OB>;
    constexpr int IW = DU::IW;
    constexpr int E = DU::E;
    constexpr int ESZ = DU::ESZ;
    constexpr int OREG_PER_WORD = DU::EPW * ESZ / 4;
    const DequantTensor &T = a.t[0];
    const int lg = a.lg_units_per_block;
    pdl_entry();
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < a.nunits;
         w += (long long)gridDim.x * blockDim.x) {
        const TransposedIndex ix = transposed_index(a.tr, (unsigned)w);
        const uint32_t *vals = static_cast<const uint32_t *>(T.values) + ix.li * IW;
        uint32_t words[IW];
#pragma unroll
        for (int j = 0; j < IW; ++j) words[j] = __ldg(vals + j);
        const long long si = (lg < 0) ? 0 : ix.li;
        const float s = round_to<FDT>(load_dyn(T.params, a.param, si));
        uint32_t s2 = 0;
        if constexpr (FDT != QK_F32) s2 = h2_pack<FDT>(s, s);
        uint32_t o[DU::OREG];
#pragma unroll
        for (int j = 0; j < IW; ++j) dequant_word<FDT, KIND>(words[j], s, s2, o + j * OREG_PER_WORD);
        char *p = static_cast<char *>(T.out) + ((long long)ix.cu * E * a.tr.ld + ix.r) * ESZ;
        const long long step = a.tr.ld * ESZ;
        if constexpr (FDT == QK_F32) {
#pragma unroll
            for (int i = 0; i < E; ++i) *reinterpret_cast<uint32_t *>(p + i * step) = o[i];
        } else {
#pragma unroll
            for (int i = 0; i < E; i += 2) {
                *reinterpret_cast<unsigned short *>(p + i * step) = (unsigned short)(o[i / 2] & 0xFFFFu);
                *reinterpret_cast<unsigned short *>(p + (i + 1) * step) = (unsigned short)(o[i / 2] >> 16);
            }
        }
    }
}

// The same pairing of rows for the 16-bit output of dequantize: one 32-bit store per column and lane.
template <int FDT, int KIND, int OB>
__global__ void __launch_bounds__(256) dequantize_transposed_pair_kernel(const DequantArgs a)
{
    using DU = DUnitT<FDT, KIND, OB>;
    constexpr int IW = DU::IW;
    constexpr int E = DU::E;
    constexpr int OREG_PER_WORD = DU::EPW * 2 / 4;
    static_assert(FDT != QK_F32, "pairs of rows are for 16-bit types");
    const DequantTensor &T = a.t[0];
    const int lg = a.lg_units_per_block;
    pdl_entry();
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < a.nunits;
         w += (long long)gridDim.x * blockDim.x) {
        const unsigned cu = fastdiv((unsigned)w, a.tr.rows);
        const unsigned r = 2u * ((unsigned)w - cu * a.tr.rows.div);
        uint32_t o[2][DU::OREG];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const long long li = (long long)(r + k) * a.tr.units_per_row + cu;
            const uint32_t *vals = static_cast<const uint32_t *>(T.values) + li * IW;
            const float s = round_to<FDT>(load_dyn(T.params, a.param, (lg < 0) ? 0 : li));
            const uint32_t s2 = h2_pack<FDT>(s, s);
#pragma unroll
            for (int j = 0; j < IW; ++j) dequant_word<FDT, KIND>(__ldg(vals + j), s, s2, o[k] + j * OREG_PER_WORD);
        }
        char *p = static_cast<char *>(T.out) + ((long long)cu * E * a.tr.ld + r) * 2;
        const long long step = a.tr.ld * 2;
#pragma unroll
        for (int i = 0; i < E; i += 2) {
            *reinterpret_cast<uint32_t *>(p + i * step) = __byte_perm(o[0][i / 2], o[1][i / 2], 0x5410);        // column i of both rows
            *reinterpret_cast<uint32_t *>(p + (i + 1) * step) = __byte_perm(o[0][i / 2], o[1][i / 2], 0x7632);  // column i + 1
        }
    }
}

// ---- launchers ----------------------------------------------------------------------------------
template <typename Kernel> static int resident(Kernel kernel)
{
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, 256, 0) != cudaSuccess || n < 1) n = 1;
    return n;
}

template <typename Kernel, typename Args>
static cudaError_t launch_waves(Kernel kernel, const Args &args, long long nunits, const LaunchCfg &cfg, cudaStream_t stream)
{
    long long need = (nunits + 255) / 256;
    const long long cap = (long long)cfg.sm_count * resident(kernel) * 4;   // a few waves: the threads are short-lived
    if (need > cap) need = cap;
    if (need < 1) need = 1;
    return launch_kernel(kernel, (int)need, 256, stream, cfg.pdl != 0, args);
}

template <int FDT, int KIND, int UB>
static cudaError_t quantize_mode(bool dyn, bool clamp, const QuantArgs &a, const LaunchCfg &cfg, cudaStream_t stream)
{
    if constexpr (FDT != QK_F32) {
        if (a.tr.pairs) {
            if (!dyn) return launch_waves(quantize_transposed_pair_kernel<FDT, KIND, UB, false, true>, a, a.nunits, cfg, stream);
            if (clamp) return launch_waves(quantize_transposed_pair_kernel<FDT, KIND, UB, true, true>, a, a.nunits, cfg, stream);
            return launch_waves(quantize_transposed_pair_kernel<FDT, KIND, UB, true, false>, a, a.nunits, cfg, stream);
        }
    }
    if (!dyn) return launch_waves(quantize_transposed_kernel<FDT, KIND, UB, false, true>, a, a.nunits, cfg, stream);
    if (clamp) return launch_waves(quantize_transposed_kernel<FDT, KIND, UB, true, true>, a, a.nunits, cfg, stream);
    return launch_waves(quantize_transposed_kernel<FDT, KIND, UB, true, false>, a, a.nunits, cfg, stream);
}

template <int FDT, int KIND>
static cudaError_t quantize_unit(int unit_bytes, bool dyn, bool clamp, const QuantArgs &a, const LaunchCfg &cfg,
                                 cudaStream_t stream)
{
    constexpr int MINB = min_unit_bytes(FDT, KIND);
    if (unit_bytes == 64) return quantize_mode<FDT, KIND, 64>(dyn, clamp, a, cfg, stream);
    if constexpr (MINB <= 32) {
        if (unit_bytes == 32) return quantize_mode<FDT, KIND, 32>(dyn, clamp, a, cfg, stream);
    }
    return cudaErrorInvalidValue;
}

template <int FDT>
static cudaError_t quantize_kind(int kind, int unit_bytes, bool dyn, bool clamp, const QuantArgs &a, const LaunchCfg &cfg,
                                 cudaStream_t stream)
{
    switch (kind) {
    case KIND_PACK8: return quantize_unit<FDT, KIND_PACK8>(unit_bytes, dyn, clamp, a, cfg, stream);
    case KIND_PACK4: return quantize_unit<FDT, KIND_PACK4>(unit_bytes, dyn, clamp, a, cfg, stream);
    case KIND_PACK2: return quantize_unit<FDT, KIND_PACK2>(unit_bytes, dyn, clamp, a, cfg, stream);
    case KIND_I8: return quantize_unit<FDT, KIND_I8>(unit_bytes, dyn, clamp, a, cfg, stream);
    case KIND_E2M1: return quantize_unit<FDT, KIND_E2M1>(unit_bytes, dyn, clamp, a, cfg, stream);
    case KIND_E4M3: return quantize_unit<FDT, KIND_E4M3>(unit_bytes, dyn, clamp, a, cfg, stream);
    case KIND_E5M2: return quantize_unit<FDT, KIND_E5M2>(unit_bytes, dyn, clamp, a, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_quantize_transposed(int fdt, int kind, int unit_bytes, bool dyn, bool clamp, const QuantArgs &args,
                                       const LaunchCfg &cfg, cudaStream_t stream)
{
    switch (fdt) {
    case QK_F32: return quantize_kind<QK_F32>(kind, unit_bytes, dyn, clamp, args, cfg, stream);
    case QK_F16: return quantize_kind<QK_F16>(kind, unit_bytes, dyn, clamp, args, cfg, stream);
    case QK_BF16: return quantize_kind<QK_BF16>(kind, unit_bytes, dyn, clamp, args, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

template <int FDT, int KIND>
static cudaError_t dequantize_unit(int out_bytes, const DequantArgs &a, const LaunchCfg &cfg, cudaStream_t stream)
{
    constexpr int MINB = min_dequant_bytes(FDT, KIND);
    if constexpr (FDT != QK_F32) {
        if (a.tr.pairs) {
            if (out_bytes == 64) return launch_waves(dequantize_transposed_pair_kernel<FDT, KIND, 64>, a, a.nunits, cfg, stream);
            if constexpr (MINB <= 32) {
                if (out_bytes == 32) return launch_waves(dequantize_transposed_pair_kernel<FDT, KIND, 32>, a, a.nunits, cfg, stream);
            }
            return cudaErrorInvalidValue;
        }
    }
    if (out_bytes == 64) return launch_waves(dequantize_transposed_kernel<FDT, KIND, 64>, a, a.nunits, cfg, stream);
    if constexpr (MINB <= 32) {
        if (out_bytes == 32) return launch_waves(dequantize_transposed_kernel<FDT, KIND, 32>, a, a.nunits, cfg, stream);
    }
    return cudaErrorInvalidValue;
}

template <int FDT>
static cudaError_t dequantize_kind(int kind, int out_bytes, const DequantArgs &a, const LaunchCfg &cfg, cudaStream_t stream)
{
    switch (kind) {
    case KIND_PACK8: return dequantize_unit<FDT, KIND_PACK8>(out_bytes, a, cfg, stream);
    case KIND_PACK4: return dequantize_unit<FDT, KIND_PACK4>(out_bytes, a, cfg, stream);
    case KIND_PACK2: return dequantize_unit<FDT, KIND_PACK2>(out_bytes, a, cfg, stream);
    case KIND_I8: return dequantize_unit<FDT, KIND_I8>(out_bytes, a, cfg, stream);
    case KIND_E2M1: return dequantize_unit<FDT, KIND_E2M1>(out_bytes, a, cfg, stream);
    case KIND_E4M3: return dequantize_unit<FDT, KIND_E4M3>(out_bytes, a, cfg, stream);
    case KIND_E5M2: return dequantize_unit<FDT, KIND_E5M2>(out_bytes, a, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_dequantize_transposed(int fdt, int kind, int out_bytes, const DequantArgs &args, const LaunchCfg &cfg,
                                         cudaStream_t stream)
{
    switch (fdt) {
    case QK_F32: return dequantize_kind<QK_F32>(kind, out_bytes, args, cfg, stream);
    case QK_F16: return dequantize_kind<QK_F16>(kind, out_bytes, args, cfg, stream);
    case QK_BF16: return dequantize_kind<QK_BF16>(kind, out_bytes, args, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace qk
