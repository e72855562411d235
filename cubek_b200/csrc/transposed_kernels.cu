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

// The unit(s) of one lane: U consecutive logical columns of row r0 (and r0 + 1 with PAIR), one element
// (or one pair of rows) per memory row, packed in registers exactly like a contiguous unit.
template <int FDT, int UB, bool PAIR>
__device__ __forceinline__ void gather_units(const char *in, long long ld, unsigned cu, unsigned r0, bool active,
                                             uint32_t (*raw)[UB / 4])
{
    constexpr int ESZ = FInfo<FDT>::SIZE;
    constexpr int U = UB / ESZ;
    constexpr int RAW = UB / 4;
    constexpr int NR = PAIR ? 2 : 1;
    if (!active) {
#pragma unroll
        for (int k = 0; k < NR; ++k)
#pragma unroll
            for (int i = 0; i < RAW; ++i) raw[k][i] = 0u;
        return;
    }
    const char *p = in + ((long long)cu * U * ld + r0) * ESZ;
    const long long step = ld * ESZ;
    if constexpr (FDT == QK_F32) {
#pragma unroll
        for (int i = 0; i < U; ++i) raw[0][i] = load_elem_bits<FDT>(p + i * step);
    } else if constexpr (PAIR) {
#pragma unroll
        for (int i = 0; i < U; i += 2) {
            const uint32_t w0 = __ldg(reinterpret_cast<const unsigned int *>(p + i * step));        // rows r0, r0+1 at column i
            const uint32_t w1 = __ldg(reinterpret_cast<const unsigned int *>(p + (i + 1) * step));  // ... at column i+1
            raw[0][i / 2] = __byte_perm(w0, w1, 0x5410);
            raw[1][i / 2] = __byte_perm(w0, w1, 0x7632);
        }
    } else {
#pragma unroll
        for (int i = 0; i < U; i += 2)
            raw[0][i / 2] = load_elem_bits<FDT>(p + i * step) | (load_elem_bits<FDT>(p + (i + 1) * step) << 16);
    }
}

// Quantize.  A CTA takes a tile of RT logical rows x 8 column units: warp w the unit column ct*8 + w, lane l
// the row(s) rt*RT + l (16-bit types with an even number of rows, an even ld and a 4-byte aligned base:
// PAIR, two adjacent rows per lane read with one 32-bit load per column and separated with byte permutes).
// The codes of a lane are only 4-32 bytes and lie a whole logical row from its neighbours', so codes and
// scales of the tile go through shared memory and leave as runs of 8 units per logical row (32-256 bytes
// contiguous) instead of half-filled sectors.  `a.tr.rows` divides by the number of row tiles; a.nunits
// counts tiles, row tiles fastest (CTAs that run together then read neighbouring pieces of the same memory rows).
template <int FDT, int KIND, int UB, bool DYN, bool CLAMP, bool PAIR>
__global__ void __launch_bounds__(256) quantize_transposed_kernel(const QuantArgs a)
{
    using UT = UnitT<FDT, KIND, UB>;
    constexpr int RAW = UT::RAW;
    constexpr int U = UT::U;
    constexpr int OW = UT::OW;
    constexpr int ESZ = UT::ESZ;
    constexpr int NR = PAIR ? 2 : 1;          // rows per lane
    constexpr int RT = 32 * NR;               // rows per tile
    constexpr int CT = 8;                     // column units per tile (one per warp)
    constexpr int ROW_WORDS = CT * OW;        // code words of one tile row
    static_assert(!PAIR || FDT != QK_F32, "pairs of rows are for 16-bit types");
    using F = typename ElemOf<FDT>::type;
    __shared__ uint32_t codes_s[RT][ROW_WORDS + 1];   // +1: lanes write one column of this array
    __shared__ float scales_s[RT][CT + 1];
    __shared__ float amax_s[RT][CT + 1];
    const QuantTensor &T = a.t[0];
    const char *in = static_cast<const char *>(T.in);
    const int lg = a.lg_units_per_block;      // -1 per tensor; else a block is 2^lg units (1, 2, 4 or 8 warps of the tile)
    const int lgb = lg < 0 ? 0 : lg;
    const unsigned R = a.tr.nrows, upr = a.tr.units_per_row;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_entry();
    float tensor_scale = 0.0f;
    if (!DYN && lg < 0) tensor_scale = tensor_unit_scale<FDT>(a, T, 0);

    for (long long tile = blockIdx.x; tile < a.nunits; tile += gridDim.x) {
        const unsigned ct = fastdiv((unsigned)tile, a.tr.rows);
        const unsigned rt = (unsigned)tile - ct * a.tr.rows.div;
        const unsigned cu = ct * CT + warp;
        const unsigned r0 = rt * RT + lane * NR;
        const bool active = cu < upr && r0 < R;
        uint32_t raw[NR][RAW];
        gather_units<FDT, UB, PAIR>(in, a.tr.ld, cu, r0, active, raw);
        float amax[NR];
        if constexpr (DYN) {
            // absmax of a block: the unit's own; blocks of several units add the other warps' through shared memory
#pragma unroll
            for (int k = 0; k < NR; ++k) amax[k] = unit_absmax<FDT, RAW>(raw[k]);
            if (lgb > 0) {
#pragma unroll
                for (int k = 0; k < NR; ++k) amax_s[lane * NR + k][warp] = amax[k];
                __syncthreads();
                const int first = warp & ~((1 << lgb) - 1);
#pragma unroll
                for (int k = 0; k < NR; ++k)
                    for (int j = 0; j < (1 << lgb); ++j) amax[k] = fmaxf(amax[k], amax_s[lane * NR + k][first + j]);
            }
        }
#pragma unroll
        for (int k = 0; k < NR; ++k) {
            float scale_f;
            if constexpr (DYN) {
                scale_f = round_to<FDT>(div_by_range(2.0f * amax[k], a.range, a.inv_range));
            } else if (lg < 0) {
                scale_f = tensor_scale;
            } else {
                scale_f = active ? static_cast<float>(static_cast<const F *>(T.scale_in)[(long long)(r0 + k) * (upr >> lgb) + (cu >> lgb)])
                                 : 1.0f;
            }
            // write_scale (crates/cubek-quant/src/quantize.rs:83-98): cast to the param type, divide by that value
            const float s_fs = (a.param == QK_F32) ? scale_f : round_to_dyn(a.param, scale_f);
            const float sc = (a.param == QK_F32) ? scale_f : round_to<FDT>(s_fs);
            uint32_t w[OW];
            if (kind_allows_fast<FDT, KIND>() && !a.force_exact && scale_is_safe(sc))
                quantize_unit_fast<FDT, KIND, UB, CLAMP, DYN>(raw[k], sc, a.lo, a.hi, w);
            else quantize_unit_exact<FDT, KIND, UB>(raw[k], sc, a.lo, a.hi, w);
#pragma unroll
            for (int j = 0; j < OW; ++j) codes_s[lane * NR + k][warp * OW + j] = w[j];
            if ((warp & ((1 << lgb) - 1)) == 0) scales_s[lane * NR + k][warp >> lgb] = s_fs;
            if (lg < 0 && tile == 0 && threadIdx.x == 0 && k == 0) store_dyn(T.out_scale, a.param, 0, s_fs);
        }
        __syncthreads();
        // rows of the tile leave as contiguous runs
        uint32_t *out = static_cast<uint32_t *>(T.out);
        for (int j = threadIdx.x; j < RT * ROW_WORDS; j += 256) {
            const int row = j / ROW_WORDS, col = j % ROW_WORDS;
            const unsigned grow = rt * RT + row, gcu = ct * CT + col / OW;
            if (grow < R && gcu < upr) out[((long long)grow * upr + ct * CT) * OW + col] = codes_s[row][col];
        }
        if (lg >= 0) {
            const int per_row = CT >> lgb;      // blocks of one tile row
            for (int j = threadIdx.x; j < RT * per_row; j += 256) {
                const int row = j / per_row, c = j % per_row;
                const unsigned grow = rt * RT + row, gcu = ct * CT + (c << lgb);
                if (grow < R && gcu < upr)
                    store_dyn(T.out_scale, a.param, (long long)grow * (upr >> lgb) + (gcu >> lgb), scales_s[row][c]);
            }
        }
        __syncthreads();   // the tile buffers are reused
    }
}

// Scales only (the two-call form) of a transposed matrix whose blocks are one unit long: same tiles, the
// F-typed scales leave as runs of 8 per logical row.
template <int FDT, int UB, bool PAIR>
__global__ void __launch_bounds__(256) scales_transposed_kernel(const void *in_, void *scale_out, const Transposed tr,
                                                                long long ntiles, float range, float inv_range, int lgb)
{
    constexpr int RAW = UB / 4;
    constexpr int NR = PAIR ? 2 : 1;
    constexpr int RT = 32 * NR;
    constexpr int CT = 8;
    using F = typename ElemOf<FDT>::type;
    __shared__ float scales_s[RT][CT + 1];
    const char *in = static_cast<const char *>(in_);
    const unsigned R = tr.nrows, upr = tr.units_per_row;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_entry();
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const unsigned ct = fastdiv((unsigned)tile, tr.rows);
        const unsigned rt = (unsigned)tile - ct * tr.rows.div;
        const unsigned cu = ct * CT + warp;
        const unsigned r0 = rt * RT + lane * NR;
        uint32_t raw[NR][RAW];
        gather_units<FDT, UB, PAIR>(in, tr.ld, cu, r0, cu < upr && r0 < R, raw);
#pragma unroll
        for (int k = 0; k < NR; ++k) scales_s[lane * NR + k][warp] = unit_absmax<FDT, RAW>(raw[k]);   // absmax per unit
        __syncthreads();
        const int per_row = CT >> lgb;      // blocks of 2^lgb units
        for (int j = threadIdx.x; j < RT * per_row; j += 256) {
            const int row = j / per_row, c = j % per_row;
            const unsigned grow = rt * RT + row, gcu = ct * CT + (c << lgb);
            if (grow < R && gcu < upr) {
                float amax = 0.0f;
                for (int u = 0; u < (1 << lgb); ++u) amax = fmaxf(amax, scales_s[row][(c << lgb) + u]);
                static_cast<F *>(scale_out)[(long long)grow * (upr >> lgb) + (gcu >> lgb)] =
                    static_cast<F>(round_to<FDT>(div_by_range(2.0f * amax, range, inv_range)));
            }
        }
        __syncthreads();
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
        const long long si = (lg < 0) ? 0 : (long long)ix.r * (a.tr.units_per_row >> lg) + (ix.cu >> lg);
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
            const long long si = (lg < 0) ? 0 : (long long)(r + k) * (a.tr.units_per_row >> lg) + (cu >> lg);
            const float s = round_to<FDT>(load_dyn(T.params, a.param, si));
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

template <typename Kernel>
static cudaError_t launch_tiles(Kernel kernel, const QuantArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    long long need = args.nunits;   // tiles
    const long long cap = (long long)cfg.sm_count * resident(kernel) * 4;
    if (need > cap) need = cap;
    if (need < 1) need = 1;
    return launch_kernel(kernel, (int)need, 256, stream, cfg.pdl != 0, args);
}

template <int FDT, int KIND, int UB, bool PAIR>
static cudaError_t quantize_pairing(bool dyn, bool clamp, const QuantArgs &a, const LaunchCfg &cfg, cudaStream_t stream)
{
    if (!dyn) return launch_tiles(quantize_transposed_kernel<FDT, KIND, UB, false, true, PAIR>, a, cfg, stream);
    if (clamp) return launch_tiles(quantize_transposed_kernel<FDT, KIND, UB, true, true, PAIR>, a, cfg, stream);
    return launch_tiles(quantize_transposed_kernel<FDT, KIND, UB, true, false, PAIR>, a, cfg, stream);
}

template <int FDT, int KIND, int UB>
static cudaError_t quantize_mode(bool dyn, bool clamp, const QuantArgs &a, const LaunchCfg &cfg, cudaStream_t stream)
{
    if constexpr (FDT != QK_F32) {
        if (a.tr.pairs) return quantize_pairing<FDT, KIND, UB, true>(dyn, clamp, a, cfg, stream);
    }
    return quantize_pairing<FDT, KIND, UB, false>(dyn, clamp, a, cfg, stream);
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

template <int FDT, int UB>
static cudaError_t scales_pairing(const void *in, void *scale_out, const Transposed &tr, long long ntiles, float range,
                                  float inv_range, int lgb, const LaunchCfg &cfg, cudaStream_t stream)
{
    long long need = ntiles;
    if constexpr (FDT != QK_F32) {
        if (tr.pairs) {
            const long long cap = (long long)cfg.sm_count * resident(scales_transposed_kernel<FDT, UB, true>) * 4;
            if (need > cap) need = cap;
            return launch_kernel(scales_transposed_kernel<FDT, UB, true>, (int)need, 256, stream, cfg.pdl != 0, in, scale_out, tr,
                                 ntiles, range, inv_range, lgb);
        }
    }
    const long long cap = (long long)cfg.sm_count * resident(scales_transposed_kernel<FDT, UB, false>) * 4;
    if (need > cap) need = cap;
    return launch_kernel(scales_transposed_kernel<FDT, UB, false>, (int)need, 256, stream, cfg.pdl != 0, in, scale_out, tr,
                         ntiles, range, inv_range, lgb);
}

cudaError_t launch_scales_transposed(int fdt, int unit_bytes, int lgb, const void *in, void *scale_out, const Transposed &tr,
                                     long long ntiles, float range, float inv_range, const LaunchCfg &cfg, cudaStream_t stream)
{
    if (ntiles < 1 || (unit_bytes != 64 && unit_bytes != 32) || lgb < 0 || lgb > 3) return cudaErrorInvalidValue;
    switch (fdt) {
    case QK_F32:
        return unit_bytes == 64 ? scales_pairing<QK_F32, 64>(in, scale_out, tr, ntiles, range, inv_range, lgb, cfg, stream)
                                : scales_pairing<QK_F32, 32>(in, scale_out, tr, ntiles, range, inv_range, lgb, cfg, stream);
    case QK_F16:
        return unit_bytes == 64 ? scales_pairing<QK_F16, 64>(in, scale_out, tr, ntiles, range, inv_range, lgb, cfg, stream)
                                : scales_pairing<QK_F16, 32>(in, scale_out, tr, ntiles, range, inv_range, lgb, cfg, stream);
    case QK_BF16:
        return unit_bytes == 64 ? scales_pairing<QK_BF16, 64>(in, scale_out, tr, ntiles, range, inv_range, lgb, cfg, stream)
                                : scales_pairing<QK_BF16, 32>(in, scale_out, tr, ntiles, range, inv_range, lgb, cfg, stream);
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
