// Dequantize kernels: unpack / sign-extend (or native decode), multiply by the scale in F.
//
// Replaces dequantize_symmetric_packed_kernel / dequantize_symmetric_native_kernel of the
// reference (crates/cubek-quant/src/dequantize.rs:121-167; unpack_q :86-118; the product
// `cast<F>(scale) * value` :22-25).  There is no addition in the element arithmetic, so a
// fused multiply-add cannot change a result: outputs are bit-exact.
//
// Output dominates the traffic (2-4 bytes written per 0.25-1 byte read), so a thread produces
// 32 or 64 contiguous bytes with 256-bit stores.  For f16 / bf16 outputs the codes are turned
// into packed F x2 values directly: a biased field b dropped into the mantissa of 2^k gives
// F(2^k + b) exactly; subtracting the bias and multiplying by the scale are packed operations
// whose single rounding is the reference's rounding (the product of two F values is exact in
// the multiplier and rounded once).
#pragma once

#include "common.cuh"
#include "quantize_kernels.cuh"  // packed helpers

namespace qk {

struct DequantTensor {
    const void *values;  // u32 words or native bytes
    const void *params;  // param-typed scales, contiguous, one per block (or one)
    void *out;           // F-typed output
    long long unit_end;  // units in this and all earlier tensors of the batch
};

// One tensor, or a batch of tensors sharing scheme, float type and unit geometry.
struct DequantArgs {
    DequantTensor t[QK_MAX_BATCH];
    int ntensors;
    long long nunits;        // dequant units in the whole batch
    int lg_units_per_block;  // log2(units per block); -1 = per tensor
    Blocks2D b2;             // [rows, cols] tiles instead of runs
    RowStride rs;            // row-strided output (one tensor per launch)
    Transposed tr;           // transposed output (dequantize_transposed_kernel only)
    int param;               // QkParam
    int aligned32;           // every output base 32-byte aligned (256-bit stores allowed)
};

// One dequant unit: OB bytes of output produced by one thread.
template <int FDT, int KIND, int OB> struct DUnitT {
    static constexpr int ESZ = FInfo<FDT>::SIZE;
    static constexpr int EPW = kind_elems_per_u32(KIND);
    static constexpr int E = OB / ESZ;          // elements
    static constexpr int IW = E / EPW;          // input words: 1, 2, 4 or 8
    static constexpr int OREG = OB / 4;         // output registers
    static_assert(E % EPW == 0 && IW >= 1, "a unit must consume whole stored words");
};

// Smallest dequant unit: 32 bytes of output, or one stored word if that is more.
__host__ __device__ constexpr int min_dequant_bytes(int fdt, int kind)
{
    return cmax(32, kind_elems_per_u32(kind) * ((fdt == QK_F32) ? 4 : 2));
}

// Decode the EPW codes of one stored word into f32 (exact).
template <int KIND> __device__ __forceinline__ void decode_word_f32(uint32_t w, float *q)
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
        const uint32_t ev = b & 0x0F0F0F0Fu, od = (b >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            q[2 * i] = __uint_as_float(__byte_perm(ev, 0x4B000000u, 0x7650 + i)) - 8388616.0f;
            q[2 * i + 1] = __uint_as_float(__byte_perm(od, 0x4B000000u, 0x7650 + i)) - 8388616.0f;
        }
    } else if constexpr (KIND == KIND_PACK2) {
        const uint32_t b = w ^ 0xAAAAAAAAu;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t f = (b >> (2 * j)) & 0x03030303u;   // elements j, j+4, j+8, j+12
#pragma unroll
            for (int i = 0; i < 4; ++i)
                q[j + 4 * i] = __uint_as_float(__byte_perm(f, 0x4B000000u, 0x7650 + i)) - 8388610.0f;
        }
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

// One stored word -> EPW/2 registers of packed F x2 outputs (element order), scale applied.
// `s` is the scale as f32 (already narrowed to F), `s2` the same value as packed F x2.
template <int FDT, int KIND>
__device__ __forceinline__ void dequant_word(uint32_t w, float s, uint32_t s2, uint32_t *o)
{
    constexpr int EPW = kind_elems_per_u32(KIND);
    if constexpr (FDT == QK_F32) {
        float q[EPW];
        decode_word_f32<KIND>(w, q);
#pragma unroll
        for (int i = 0; i < EPW; ++i) o[i] = __float_as_uint(s * q[i]);
    } else if constexpr (KIND == KIND_PACK4 || KIND == KIND_PACK2 ||
                         ((KIND == KIND_PACK8 || KIND == KIND_I8) && FDT == QK_F16)) {
        // F(2^k + b) for a biased field b: 0x4300 | b = 128 + b (bf16, b < 128),
        // 0x6400 | b = 1024 + b (f16, b < 1024).
        constexpr uint32_t BASE = (FDT == QK_BF16) ? 0x43004300u : 0x64006400u;
        constexpr float BASE_F = (FDT == QK_BF16) ? 128.0f : 1024.0f;
        constexpr int BITS = kind_bits(KIND);
        const uint32_t bias2 = h2_const<FDT>(BASE_F + (float)(1 << (BITS - 1)));
        if constexpr (BITS == 8) {
            const uint32_t b = w ^ 0x80808080u;
            // bytes (0,1) -> halves of o[0]; bytes (2,3) -> o[1]
            const uint32_t p0 = __byte_perm(b, BASE, 0x7150);           // [b0, BASE.b1, b1, BASE.b3]
            const uint32_t p1 = __byte_perm(b, BASE, 0x7352);           // [b2, BASE.b1, b3, BASE.b3]
            o[0] = h2_mul<FDT>(h2_sub<FDT>(p0, bias2), s2);
            o[1] = h2_mul<FDT>(h2_sub<FDT>(p1, bias2), s2);
        } else if constexpr (BITS == 4) {
            const uint32_t b = w ^ 0x88888888u;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                // byte k holds elements 2k (low nibble) and 2k+1 (high nibble)
                const uint32_t byte = __byte_perm(b, 0u, 0x4440 + k);
                const uint32_t p = ((byte * 0x1001u) & 0x000F000Fu) | BASE;
                o[k] = h2_mul<FDT>(h2_sub<FDT>(p, bias2), s2);
            }
        } else {
            const uint32_t b = w ^ 0xAAAAAAAAu;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                // nibble k holds elements 2k (low 2 bits) and 2k+1 (high 2 bits)
                const uint32_t nib = (b >> (4 * k)) & 0xFu;
                const uint32_t p = ((nib * 0x4001u) & 0x00030003u) | BASE;
                o[k] = h2_mul<FDT>(h2_sub<FDT>(p, bias2), s2);
            }
        }
    } else if constexpr (KIND == KIND_E2M1 && FDT == QK_F16) {
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = h2_mul<FDT>(cvt_f16x2_from_e2m1x2(__byte_perm(w, 0u, 0x4440 + k)), s2);
    } else {
        // bf16 8-bit codes (9-bit biased values do not fit a bf16 mantissa), bf16 fp4 and fp8:
        // decode to f32, multiply (exact product), narrow once.
        if constexpr (KIND == KIND_PACK8 || KIND == KIND_I8) {
            // the same decode as decode_word_f32, two elements per instruction (add / mul.rn.f32x2)
            const uint32_t b = w ^ 0x80808080u;
#pragma unroll
            for (int i = 0; i < 4; i += 2) {
                float q0, q1, r0, r1;
                add2(__uint_as_float(__byte_perm(b, 0x4B000000u, 0x7650 + i)), __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7651 + i)),
                     -8388736.0f, q0, q1);
                mul2(q0, q1, s, r0, r1);
                o[i / 2] = h2_pack<FDT>(r0, r1);
            }
        } else {
            float q[EPW];
            decode_word_f32<KIND>(w, q);
#pragma unroll
            for (int i = 0; i < EPW; i += 2) o[i / 2] = h2_pack<FDT>(s * q[i], s * q[i + 1]);
        }
    }
}

// TILES selects the [rows, cols] tile scale indexing at compile time: folding it into the common
// kernel costs 16 registers and with them one resident CTA per SM.
// SUB = 2: the unit holds two blocks (16-bit types, blocks of 32 bytes, f32 params): its two scales are fetched with
// one 8-byte load and each half of the unit is multiplied by its own.
template <int FDT, int KIND, int OB, bool TILES, int SUB = 1>
__global__ void __launch_bounds__(256) dequantize_kernel(const DequantArgs a)
{
    using DU = DUnitT<FDT, KIND, OB>;
    constexpr int IW = DU::IW;
    constexpr int EPW = DU::EPW;
    constexpr int OREG_PER_WORD = EPW * DU::ESZ / 4;
    constexpr int UNR = 4;
    static_assert(SUB == 1 || (IW % 2 == 0 && !TILES), "two blocks per unit need an even number of words");

    const int lg = a.lg_units_per_block;
    const bool aligned32 = a.aligned32 != 0;
    pdl_entry();
    int ti = 0;  // tensor of the batch this thread is in (only ever moves forward)

    const long long stride = (long long)gridDim.x * blockDim.x * UNR;
    for (long long base = (long long)blockIdx.x * blockDim.x * UNR + threadIdx.x; base - threadIdx.x < a.nunits;
         base += stride) {
        uint32_t w[UNR][IW];
        float s[UNR][SUB];
        char *dst[UNR];
        const bool full = base - threadIdx.x + (long long)blockDim.x * UNR <= a.nunits;
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            const long long idx = base + (long long)k * blockDim.x;
            const bool valid = full || idx < a.nunits;
            if (valid) {
                while (ti + 1 < a.ntensors && idx >= a.t[ti].unit_end) ++ti;
                const DequantTensor &T = a.t[ti];
                const long long li = idx - (ti ? a.t[ti - 1].unit_end : 0);
                const uint32_t *vals = static_cast<const uint32_t *>(T.values);
                long long offset = li * OB;
                if (a.rs.enabled) {
                    const unsigned row = fastdiv((unsigned)li, a.rs.units_per_row);
                    offset = (long long)row * a.rs.row_bytes + (long long)((unsigned)li - row * a.rs.units_per_row.div) * OB;
                }
                dst[k] = static_cast<char *>(T.out) + offset;
                if constexpr (IW == 1) {
                    w[k][0] = __ldg(vals + li);
                } else if constexpr (IW == 2) {
                    const uint2 t = __ldg(reinterpret_cast<const uint2 *>(vals) + li);
                    w[k][0] = t.x;
                    w[k][1] = t.y;
                } else {
#pragma unroll
                    for (int v = 0; v < IW / 4; ++v) {
                        const uint4 t = __ldg(reinterpret_cast<const uint4 *>(vals) + li * (IW / 4) + v);
                        w[k][4 * v] = t.x;
                        w[k][4 * v + 1] = t.y;
                        w[k][4 * v + 2] = t.z;
                        w[k][4 * v + 3] = t.w;
                    }
                }
                // cast<F>(scale): the param-typed scale narrowed (or widened) to F.
                if constexpr (SUB == 2) {
                    const float2 p = __ldg(reinterpret_cast<const float2 *>(T.params) + li);
                    s[k][0] = round_to<FDT>(p.x);
                    s[k][SUB - 1] = round_to<FDT>(p.y);
                } else {
                    long long si;
                    if constexpr (TILES) {
                        bool unused;
                        si = (long long)blocks2d_scale_index(a.b2, (unsigned)li, &unused);
                    } else {
                        si = (lg < 0) ? 0 : (li >> lg);
                    }
                    if (a.param == QK_F32) s[k][0] = round_to<FDT>(__ldg(static_cast<const float *>(T.params) + si));
                    else s[k][0] = round_to<FDT>(load_dyn(T.params, a.param, si));
                }
            } else {
#pragma unroll
                for (int j = 0; j < IW; ++j) w[k][j] = 0u;
#pragma unroll
                for (int j = 0; j < SUB; ++j) s[k][j] = 0.0f;
                dst[k] = nullptr;
            }
        }
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            const long long idx = base + (long long)k * blockDim.x;
            if (!(full || idx < a.nunits)) continue;
            uint32_t o[DU::OREG];
            uint32_t s2[SUB];
#pragma unroll
            for (int j = 0; j < SUB; ++j) {
                s2[j] = 0;
                if constexpr (FDT != QK_F32) s2[j] = h2_pack<FDT>(s[k][j], s[k][j]);
            }
#pragma unroll
            for (int j = 0; j < IW; ++j) {
                constexpr int HALF = (SUB == 2) ? IW / 2 : IW;
                const int b = (SUB == 2 && j >= HALF) ? SUB - 1 : 0;
                dequant_word<FDT, KIND>(w[k][j], s[k][b], s2[b], o + j * OREG_PER_WORD);
            }
            if (aligned32) {
#pragma unroll
                for (int v = 0; v < OB / 32; ++v) {
                    Vec32 t;
#pragma unroll
                    for (int i = 0; i < 8; ++i) t.w[i] = o[8 * v + i];
                    stg256_stream(dst[k] + 32 * v, t);
                }
            } else {
#pragma unroll
                for (int v = 0; v < OB / 16; ++v) {
                    Vec16 t;
#pragma unroll
                    for (int i = 0; i < 4; ++i) t.w[i] = o[4 * v + i];
                    stg128_stream(dst[k] + 16 * v, t);
                }
            }
        }
    }
}

// `sub`: blocks per unit, 1 or 2.
cudaError_t launch_dequantize(int fdt, int kind, int out_bytes, int sub, const DequantArgs &args, const LaunchCfg &cfg,
                              cudaStream_t stream);
cudaError_t launch_dequantize_transposed(int fdt, int kind, int out_bytes, const DequantArgs &args, const LaunchCfg &cfg,
                                         cudaStream_t stream);

}  // namespace qk
