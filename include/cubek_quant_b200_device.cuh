/*
 * Device-side helpers for CUDA kernels that consume quantized tensors in place (for instance the
 * operand loader of a matmul): the counterparts of the `pub` cube functions of the reference,
 *
 *   dequantize_symmetric                   crates/cubek-quant/src/dequantize.rs:22-25
 *   dequantize_symmetric_packed_values     crates/cubek-quant/src/dequantize.rs:31-39
 *   dequantize_symmetric_packed_value_at   crates/cubek-quant/src/dequantize.rs:46-54
 *   dequantize_symmetric_packed_value      crates/cubek-quant/src/dequantize.rs:61-84
 *   unpack_q                               crates/cubek-quant/src/dequantize.rs:86-118
 *   ScalesLayout / PerTensorLayout / BlockScaledLayout   crates/cubek-quant/src/layout/scales.rs:15-195
 *
 * Those are generic device functions of the reference's kernel language and cannot cross a C ABI;
 * this header gives CUDA code the same operations with the same results: header only, no link
 * dependency on libcubek_quant_b200.so.  Every function returns the bits `qk_dequantize` writes for
 * the same codes and scales: codes are widened exactly, the scale is cast to F first, and the product
 * is rounded once to F (there is no addition, so contraction cannot change a result).
 *
 * The scheme is a compile-time argument, as in the reference (`#[comptime] scheme`): VALUE is a
 * QkValue, STORE a QkStore.  F is float, __half or __nv_bfloat16; FS (the scale type) likewise.
 */
#ifndef CUBEK_QUANT_B200_DEVICE_CUH
#define CUBEK_QUANT_B200_DEVICE_CUH

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "cubek_quant_b200.h"

namespace cubek_quant_b200 {

/* ---- scheme arithmetic at compile time (QuantValue::size_bits, QuantScheme::num_quants) ---------- */
__host__ __device__ constexpr int size_bits(int value)
{
    return (value == QK_Q8F || value == QK_Q8S || value == QK_E4M3 || value == QK_E5M2) ? 8
           : (value == QK_Q4F || value == QK_Q4S || value == QK_E2M1)                   ? 4
                                                                                        : 2;
}
/* Quantized values per stored item: 32 / bits for u32 words; native items hold one value, or two for
 * e2m1 (one byte of two fp4 codes). */
__host__ __device__ constexpr int num_quants(int value, int store)
{
    return store == QK_STORE_U32 ? 32 / size_bits(value) : (value == QK_E2M1 ? 2 : 1);
}
/* The stored item: a u32 word, or one byte for native stores. */
template <int STORE> struct Stored { using type = uint32_t; };
template <> struct Stored<QK_STORE_NATIVE> { using type = uint8_t; };

/* ---- float casts -------------------------------------------------------------------------------- */
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename F> __device__ __forceinline__ F from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

/* `Line::cast_from(scale) * value` in F: the scale is narrowed (or widened) to F, and the product of
 * two F values, computed exactly in f32 (at most 22 significant bits for the 16-bit types; one f32
 * rounding for F = float), is rounded once to F. */
template <typename F, typename FS> __device__ __forceinline__ F dequantize_symmetric(F value, FS scale)
{
    const float s = to_f32(from_f32<F>(to_f32(scale)));
    return from_f32<F>(s * to_f32(value));
}

/* ---- unpack_q: the codes of one stored item as exact f32 values, element 0 first ------------------- */
template <int VALUE, int STORE>
__device__ __forceinline__ void unpack_q(typename Stored<STORE>::type item, float *out)
{
    constexpr int BITS = size_bits(VALUE);
    if constexpr (STORE == QK_STORE_U32) {
        /* element i in bits [i*BITS, (i+1)*BITS), two's complement (quantize.rs:61-81) */
#pragma unroll
        for (int i = 0; i < 32 / BITS; ++i) {
            const int32_t field = (int32_t)(item << (32 - BITS - i * BITS)) >> (32 - BITS);   // sign-extends
            out[i] = (float)field;
        }
    } else if constexpr (VALUE == QK_Q8F || VALUE == QK_Q8S) {
        out[0] = (float)(int8_t)item;
    } else if constexpr (VALUE == QK_E2M1) {
        /* one byte = two fp4 codes, even element in the low nibble */
        uint32_t h2;
        const uint16_t b = item;
        asm("{\n\t.reg .b8 t;\n\tcvt.u8.u16 t, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, t;\n\t}" : "=r"(h2) : "h"(b));
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&h2));
        out[0] = f.x;
        out[1] = f.y;
    } else {
        uint32_t h2;
        const uint16_t b = item;
        if constexpr (VALUE == QK_E4M3) asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(b));
        else asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(h2) : "h"(b));
        out[0] = __low2float(*reinterpret_cast<const __half2 *>(&h2));
    }
}

/* ---- scale indexing ------------------------------------------------------------------------------- */
/* Maps the linear index of an unpacked element (row-major over `shape`) to its scale, as the
 * reference's ScalesLayout does: PerTensorLayout -> always element 0; BlockScaledLayout -> per dim
 * `coordinate / block`, combined with the strides of the scales tensor. */
template <typename FS> struct ScalesView {
    const FS *scales;
    int rank;                       /* 0 = per tensor */
    uint32_t shape[QK_MAX_RANK];    /* unpacked shape of the values */
    uint32_t block[QK_MAX_RANK];    /* block extents, left-padded with 1 to `rank` */
    int64_t strides[QK_MAX_RANK];   /* strides of the scales tensor, in elements */

    __device__ __forceinline__ int64_t to_source_pos(uint32_t element) const
    {
        int64_t pos = 0;
        for (int d = rank - 1; d >= 0; --d) {
            const uint32_t c = element % shape[d];
            element /= shape[d];
            pos += (int64_t)(c / block[d]) * strides[d];
        }
        return pos;
    }
    /* True for the first element of a block (the one `write_scale` stores the scale at). */
    __device__ __forceinline__ bool is_block_start(uint32_t element) const
    {
        bool start = true;
        for (int d = rank - 1; d >= 0; --d) {
            const uint32_t c = element % shape[d];
            element /= shape[d];
            start = start && (c % block[d] == 0);
        }
        return start;
    }
    __device__ __forceinline__ FS operator[](uint32_t element) const { return scales[to_source_pos(element)]; }
};

/* Host-side construction (scales_view / scales_layout, layout/scales.rs:205-258).  `values_shape` is the
 * shape of the quantized tensor (last dim in stored items); `scales_strides` the strides of the scales tensor. */
template <typename FS>
inline ScalesView<FS> make_scales_view(const FS *scales, const QkScheme &scheme, int rank, const int64_t *values_shape,
                                       const int64_t *scales_strides)
{
    ScalesView<FS> v{};
    v.scales = scales;
    if (scheme.level == QK_LEVEL_TENSOR) {
        v.rank = 0;
        return v;
    }
    v.rank = rank;
    const int nq = num_quants(scheme.value, scheme.store);
    for (int d = 0; d < rank; ++d) {
        v.shape[d] = (uint32_t)(d == rank - 1 ? values_shape[d] * nq : values_shape[d]);
        const int bi = d - (rank - scheme.block_rank);
        v.block[d] = bi >= 0 ? scheme.block[bi] : 1u;
        v.strides[d] = scales_strides[d];
    }
    return v;
}

/* ---- packed values ---------------------------------------------------------------------------------- */
/* dequantize_symmetric_packed_value: LINE stored items (`values`, a "line") at line position `position`
 * -> LINE * num_quants floats in `out`, element order.  Item i uses the scale of unpacked element
 * (position * LINE + i) * num_quants, as the reference does (dequantize.rs:75). */
template <typename F, typename FS, int VALUE, int STORE, int LINE>
__device__ __forceinline__ void dequantize_symmetric_packed_value(const typename Stored<STORE>::type *values,
                                                                  const ScalesView<FS> &scales, uint32_t position, F *out)
{
    constexpr int NQ = num_quants(VALUE, STORE);
#pragma unroll
    for (int i = 0; i < LINE; ++i) {
        float q[NQ];
        unpack_q<VALUE, STORE>(values[i], q);
        const FS scale = scales[(position * LINE + i) * NQ];
        const float s = to_f32(from_f32<F>(to_f32(scale)));
#pragma unroll
        for (int j = 0; j < NQ; ++j) out[i * NQ + j] = from_f32<F>(s * q[j]);
    }
}

/* dequantize_symmetric_packed_value_at: same, argument order of the reference. */
template <typename F, typename FS, int VALUE, int STORE, int LINE>
__device__ __forceinline__ void dequantize_symmetric_packed_value_at(uint32_t position,
                                                                     const typename Stored<STORE>::type *values,
                                                                     const ScalesView<FS> &scales, F *out)
{
    dequantize_symmetric_packed_value<F, FS, VALUE, STORE, LINE>(values, scales, position, out);
}

/* dequantize_symmetric_packed_values: reads line `position` of the quantized tensor itself. */
template <typename F, typename FS, int VALUE, int STORE, int LINE>
__device__ __forceinline__ void dequantize_symmetric_packed_values(uint32_t position,
                                                                   const typename Stored<STORE>::type *tensor,
                                                                   const ScalesView<FS> &scales, F *out)
{
    typename Stored<STORE>::type line[LINE];
#pragma unroll
    for (int i = 0; i < LINE; ++i) line[i] = tensor[(size_t)position * LINE + i];
    dequantize_symmetric_packed_value_at<F, FS, VALUE, STORE, LINE>(position, line, scales, out);
}

}  /* namespace cubek_quant_b200 */

#endif
