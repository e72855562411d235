// Dequantize kernels: unpack / sign-extend (or native decode), multiply by the scale in F.
//
// Replaces dequantize_symmetric_packed_kernel / dequantize_symmetric_native_kernel of the
// reference (crates/cubek-quant/src/dequantize.rs:121-167; unpack_q :86-118; the product
// `cast<F>(scale) * value` :22-25).  There is no addition in the element arithmetic, so a
// fused multiply-add cannot change a result: outputs are bit-exact.
#pragma once

#include "common.cuh"

namespace qk {

struct DequantArgs {
    const void *values;   // u32 words or native bytes
    const void *params;   // param-typed scales, contiguous, one per block (or one)
    void *out;            // F-typed output
    long long nunits;     // dequant units in the tensor
    int lg_units_per_block;  // log2(units per block); -1 = per tensor
    int param;            // QkParam
    int aligned32;        // output base 32-byte aligned (256-bit stores allowed)
};

// One dequant unit is 32 bytes of output (64 for f32 from 2-bit codes).
template <int FDT, int KIND> struct DUnit {
    static constexpr int EPW = kind_elems_per_u32(KIND);
    static constexpr int ELEMS = cmax(32 / FInfo<FDT>::SIZE, EPW);
    static constexpr int IN_WORDS = ELEMS / EPW;                   // 1, 2 or 4
    static constexpr int OUT_BYTES = ELEMS * FInfo<FDT>::SIZE;     // 32 or 64
};

// Decode the EPW codes of one stored word into f32 (exact).
template <int KIND> __device__ __forceinline__ void decode_word(uint32_t w, float *q)
{
    if constexpr (KIND == KIND_PACK8 || KIND == KIND_I8) {
        // bias to unsigned, drop the byte into the mantissa of 2^23, subtract 2^23 + 128.
        const uint32_t b = w ^ 0x80808080u;
        q[0] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7650)) - 8388736.0f;
        q[1] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7651)) - 8388736.0f;
        q[2] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7652)) - 8388736.0f;
        q[3] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7653)) - 8388736.0f;
    } else if constexpr (KIND == KIND_PACK4) {
        const uint32_t b = w ^ 0x88888888u;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            q[i] = __uint_as_float(((b >> (4 * i)) & 0xFu) | 0x4B000000u) - 8388616.0f;
    } else if constexpr (KIND == KIND_PACK2) {
        const uint32_t b = w ^ 0xAAAAAAAAu;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            q[i] = __uint_as_float(((b >> (2 * i)) & 0x3u) | 0x4B000000u) - 8388610.0f;
    } else if constexpr (KIND == KIND_E2M1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t h2 = cvt_f16x2_from_e2m1x2((w >> (8 * i)) & 0xFFu);
            float2 f = __half22float2(*reinterpret_cast<__half2 *>(&h2));
            q[2 * i] = f.x;
            q[2 * i + 1] = f.y;
        }
    } else {  // KIND_E4M3 / KIND_E5M2
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t two = (w >> (16 * i)) & 0xFFFFu;
            uint32_t h2 = (KIND == KIND_E4M3) ? cvt_f16x2_from_e4m3x2(two) : cvt_f16x2_from_e5m2x2(two);
            float2 f = __half22float2(*reinterpret_cast<__half2 *>(&h2));
            q[2 * i] = f.x;
            q[2 * i + 1] = f.y;
        }
    }
}

template <int FDT, int KIND>
__global__ void __launch_bounds__(256) dequantize_kernel(const DequantArgs a)
{
    using DU = DUnit<FDT, KIND>;
    constexpr int E = DU::ELEMS;
    constexpr int IW = DU::IN_WORDS;
    constexpr int EPW = DU::EPW;
    constexpr int UNR = 4;

    const uint32_t *vals = static_cast<const uint32_t *>(a.values);
    char *out = static_cast<char *>(a.out);
    const int lg = a.lg_units_per_block;
    const bool aligned32 = a.aligned32 != 0;
    float tensor_scale = 0.0f;
    if (lg < 0) tensor_scale = round_to<FDT>(load_dyn(a.params, a.param, 0));

    const long long stride = (long long)gridDim.x * blockDim.x * UNR;
    for (long long base = (long long)blockIdx.x * blockDim.x * UNR + threadIdx.x; base - threadIdx.x < a.nunits;
         base += stride) {
        uint32_t w[UNR][IW];
        float s[UNR];
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            const long long idx = base + (long long)k * blockDim.x;
            const bool valid = idx < a.nunits;
            if constexpr (IW == 1) {
                w[k][0] = valid ? __ldg(vals + idx) : 0u;
            } else if constexpr (IW == 2) {
                uint2 t = valid ? __ldg(reinterpret_cast<const uint2 *>(vals) + idx) : make_uint2(0u, 0u);
                w[k][0] = t.x;
                w[k][1] = t.y;
            } else {
                uint4 t = valid ? __ldg(reinterpret_cast<const uint4 *>(vals) + idx) : make_uint4(0u, 0u, 0u, 0u);
                w[k][0] = t.x;
                w[k][1] = t.y;
                w[k][2] = t.z;
                w[k][3] = t.w;
            }
            // cast<F>(scale): the param-typed scale narrowed (or widened) to F.
            s[k] = (lg < 0) ? tensor_scale : (valid ? round_to<FDT>(load_dyn(a.params, a.param, idx >> lg)) : 0.0f);
        }
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            const long long idx = base + (long long)k * blockDim.x;
            if (idx >= a.nunits) continue;
            float q[E];
#pragma unroll
            for (int j = 0; j < IW; ++j) decode_word<KIND>(w[k][j], q + j * EPW);
            uint32_t o[DU::OUT_BYTES / 4];
            if constexpr (FDT == QK_F32) {
#pragma unroll
                for (int i = 0; i < E; ++i) o[i] = __float_as_uint(s[k] * q[i]);
            } else if constexpr (FDT == QK_BF16) {
#pragma unroll
                for (int i = 0; i < E; i += 2) o[i / 2] = pack_bf16x2(s[k] * q[i], s[k] * q[i + 1]);
            } else {
#pragma unroll
                for (int i = 0; i < E; i += 2) o[i / 2] = pack_f16x2(s[k] * q[i], s[k] * q[i + 1]);
            }
            char *dst = out + idx * DU::OUT_BYTES;
            if (aligned32) {
#pragma unroll
                for (int v = 0; v < DU::OUT_BYTES / 32; ++v) {
                    Vec32 t;
#pragma unroll
                    for (int i = 0; i < 8; ++i) t.w[i] = o[8 * v + i];
                    stg256_stream(dst + 32 * v, t);
                }
            } else {
#pragma unroll
                for (int v = 0; v < DU::OUT_BYTES / 16; ++v) {
                    Vec16 t;
#pragma unroll
                    for (int i = 0; i < 4; ++i) t.w[i] = o[4 * v + i];
                    stg128_stream(dst + 16 * v, t);
                }
            }
        }
    }
}

cudaError_t launch_dequantize(int fdt, int kind, const DequantArgs &args, const LaunchCfg &cfg,
                              cudaStream_t stream);
int dequant_unit_elems(int fdt, int kind);

}  // namespace qk
