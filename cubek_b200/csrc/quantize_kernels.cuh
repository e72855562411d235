// Quantize kernels: symmetric scale, round, clamp, pack (u32 store) or native cast.
//
// Replaces quantize_symmetric_packed_kernel / quantize_symmetric_native_kernel of the
// reference (crates/cubek-quant/src/quantize.rs:100-171).  The reference gives each thread
// one u32 and resolves the scale index with a div/mod chain per thread; here a thread owns
// a "unit" of consecutive elements (16..64 bytes of input, whole output words), blocks are
// power-of-two runs of units, and in the fused form the absmax of a block is reduced with
// warp shuffles so that the data is read exactly once.
#pragma once

#include "common.cuh"

namespace qk {

struct QuantArgs {
    const void *in;          // F-typed input, contiguous
    void *out;               // u32 words or native bytes
    const void *scale_in;    // F-typed scales (given-scale form); contiguous, one per block
    void *out_scale;         // param-typed scales out (may alias nothing else)
    const float *absmax;     // per tensor: absmax scalar on the device (overrides scale_in)
    long long nunits;        // units in the tensor
    int lg_units_per_block;  // log2(units per block); -1 = per tensor
    int param;               // QkParam of out_scale
    float lo, hi, range;     // clamp bounds, hi - lo
    int force_exact;         // 1: reference arithmetic for every unit
    int aligned32;           // input base is 32-byte aligned (256-bit loads allowed)
};

// -------------------------------------------------------------------------------------
// Loading one unit (16 / 32 / 64 contiguous bytes) with 128- or 256-bit streaming loads.
// -------------------------------------------------------------------------------------
template <int IN_BYTES> struct RawUnit { Vec16 v[IN_BYTES / 16]; };

template <int IN_BYTES>
__device__ __forceinline__ void load_unit(RawUnit<IN_BYTES> &u, const char *p, bool valid, bool aligned32)
{
    if (!valid) {
#pragma unroll
        for (int i = 0; i < IN_BYTES / 16; ++i) u.v[i] = Vec16{{0u, 0u, 0u, 0u}};
        return;
    }
    if constexpr (IN_BYTES == 16) {
        u.v[0] = ldg128_stream(p);
    } else {
        if (aligned32) {
#pragma unroll
            for (int i = 0; i < IN_BYTES / 32; ++i) {
                Vec32 t = ldg256_stream(p + 32 * i);
                u.v[2 * i] = Vec16{{t.w[0], t.w[1], t.w[2], t.w[3]}};
                u.v[2 * i + 1] = Vec16{{t.w[4], t.w[5], t.w[6], t.w[7]}};
            }
        } else {
#pragma unroll
            for (int i = 0; i < IN_BYTES / 16; ++i) u.v[i] = ldg128_stream(p + 16 * i);
        }
    }
}

// -------------------------------------------------------------------------------------
// Element arithmetic on one unit.
// -------------------------------------------------------------------------------------

// 1.5 * 2^23: adding it to |v| < 2^22 rounds v to an integer (half to even) and leaves
// that integer, in two's complement, in the low mantissa bits.
#define QK_MAGIC 12582912.0f
#define QK_MAGIC_BITS 0x4B400000u

// Fast quotient RN_F(x / s) for a scale in the safe exponent window, given r = RN(1/s).
//   f32: q0 = x*r; q1 = fma(fma(-s, q0, x), r, q0) is the correctly rounded quotient when r
//        is the correctly rounded reciprocal and nothing under/overflows.  With a caller
//        supplied scale the first guess is clamped so that a huge quotient ends as +-inf or
//        a huge finite value of the right sign (never NaN); it is clamped afterwards anyway.
//   f16/bf16: x and s carry 11 / 8 significant bits, so x/s is never closer than 2^-23 /
//        2^-17 (relative) to a rounding boundary of F, and the f32 product x*r (error
//        < 2^-22.9) rounds to the same F value as the exact quotient for every |x/s| in
//        [1/8, 1024] (checked exhaustively on the host); outside it the code is 0 or clamped.
template <int FDT, bool BOUNDED>
__device__ __forceinline__ float fast_quotient(float x, float s, float r, float lo, float hi)
{
    float q0 = x * r;
    if constexpr (FDT == QK_F32) {
        if constexpr (!BOUNDED) q0 = fminf(fmaxf(q0, lo - 2.0f), hi + 2.0f);
        float e = __fmaf_rn(-s, q0, x);
        return __fmaf_rn(e, r, q0);
    } else {
        return q0;  // narrowed to F by the caller
    }
}

template <int FDT, int KIND, bool BOUNDED>
__device__ __forceinline__ void quantize_unit(const float *x, float s, float lo, float hi, bool fast,
                                              uint32_t *outw)
{
    constexpr int U = Unit<FDT, KIND>::ELEMS;
    constexpr int OW = Unit<FDT, KIND>::OUT_WORDS;
    constexpr int EPW = kind_elems_per_u32(KIND);
    float c[U];  // clamped, integral values

    if (fast) {
        const float r = __frcp_rn(s);
        float t[U];
#pragma unroll
        for (int i = 0; i < U; ++i) t[i] = fast_quotient<FDT, BOUNDED>(x[i], s, r, lo, hi);
        if constexpr (FDT == QK_BF16) {
#pragma unroll
            for (int i = 0; i < U; i += 2) {
                uint32_t p = pack_bf16x2(t[i], t[i + 1]);
                t[i] = bf16_lo_to_f32(p);
                t[i + 1] = bf16_hi_to_f32(p);
            }
        } else if constexpr (FDT == QK_F16) {
#pragma unroll
            for (int i = 0; i < U; i += 2) {
                uint32_t p = pack_f16x2(t[i], t[i + 1]);
                float2 f = __half22float2(*reinterpret_cast<__half2 *>(&p));
                t[i] = f.x;
                t[i + 1] = f.y;
            }
        }
        // clamp first (the bounds are integers, so clamp and round commute), then round.
#pragma unroll
        for (int i = 0; i < U; ++i) c[i] = fminf(fmaxf(t[i], lo), hi);
    } else {
#pragma unroll
        for (int i = 0; i < U; ++i) c[i] = quantize_exact<FDT>(x[i], s, lo, hi);
    }

    if constexpr (KIND == KIND_PACK8 || KIND == KIND_I8) {
#pragma unroll
        for (int w = 0; w < OW; ++w) {
            uint32_t b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) b[i] = __float_as_uint(c[4 * w + i] + QK_MAGIC);
            uint32_t l = __byte_perm(b[0], b[1], 0x0040);
            uint32_t h = __byte_perm(b[2], b[3], 0x0040);
            outw[w] = __byte_perm(l, h, 0x5410);
        }
    } else if constexpr (KIND == KIND_PACK4 || KIND == KIND_PACK2) {
        // Bias every code to be non-negative (q + 2^(bits-1)), add the shifted float bit
        // patterns, remove the constant part, then flip the top bit of every field to get
        // back to two's complement.
        constexpr int BITS = kind_bits(KIND);
        constexpr uint32_t BIAS = 1u << (BITS - 1);
        constexpr uint32_t FLIP = (BITS == 4) ? 0x88888888u : 0xAAAAAAAAu;
        uint32_t kconst = 0;
#pragma unroll
        for (int i = 0; i < EPW; ++i) kconst += (QK_MAGIC_BITS << (i * BITS));
#pragma unroll
        for (int w = 0; w < OW; ++w) {
            uint32_t acc = 0;
#pragma unroll
            for (int i = 0; i < EPW; ++i) {
                uint32_t b = __float_as_uint(c[EPW * w + i] + (QK_MAGIC + (float)BIAS));
                acc += b << (i * BITS);
            }
            outw[w] = (acc - kconst) ^ FLIP;
        }
    } else if constexpr (KIND == KIND_E2M1) {
#pragma unroll
        for (int w = 0; w < OW; ++w) {
            uint32_t by[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float a = (c[8 * w + 2 * i] + QK_MAGIC) - QK_MAGIC;
                float b = (c[8 * w + 2 * i + 1] + QK_MAGIC) - QK_MAGIC;
                by[i] = cvt_e2m1x2(a, b);
            }
            uint32_t l = __byte_perm(by[0], by[1], 0x0040);
            uint32_t h = __byte_perm(by[2], by[3], 0x0040);
            outw[w] = __byte_perm(l, h, 0x5410);
        }
    } else {  // KIND_E4M3 / KIND_E5M2
#pragma unroll
        for (int w = 0; w < OW; ++w) {
            uint32_t hw[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float a = rintf(c[4 * w + 2 * i]);
                float b = rintf(c[4 * w + 2 * i + 1]);
                hw[i] = (KIND == KIND_E4M3) ? cvt_e4m3x2(a, b) : cvt_e5m2x2(a, b);
            }
            outw[w] = __byte_perm(hw[0], hw[1], 0x5410);
        }
    }
}

// Scales outside this window (zero, subnormal-ish, huge, negative, NaN) take the reference
// arithmetic: the shortcuts above assume 1/s and x*(1/s) stay inside the normal range.
__device__ __forceinline__ bool scale_is_safe(float s)
{
    return s >= 7.888609052e-31f /* 2^-100 */ && s <= 1.267650600e+30f /* 2^100 */;
}

// E5M2 clamps at +-57344, outside the window the half-precision shortcut was checked on.
template <int FDT, int KIND> __host__ __device__ constexpr bool kind_allows_fast()
{
    return !(KIND == KIND_E5M2 && FDT != QK_F32);
}

// -------------------------------------------------------------------------------------
// The kernel.  DYN = true: scale from the block's own absmax (one pass, fused).
// DYN = false: scale given (tensor of F, one per block) or derived from a device absmax.
// -------------------------------------------------------------------------------------
template <int FDT, int KIND, bool DYN>
__global__ void __launch_bounds__(256) quantize_kernel(const QuantArgs a)
{
    using UT = Unit<FDT, KIND>;
    constexpr int U = UT::ELEMS;
    constexpr int IN_BYTES = UT::IN_BYTES;
    constexpr int OW = UT::OUT_WORDS;
    constexpr int UNR = 64 / IN_BYTES;  // units in flight per thread (64 bytes of loads)
    using F = typename ElemOf<FDT>::type;

    const char *in = static_cast<const char *>(a.in);
    uint32_t *out = static_cast<uint32_t *>(a.out);
    const bool aligned32 = a.aligned32 != 0;
    const int lg = a.lg_units_per_block;

    // Per tensor with a device absmax: derive the scale once per thread.
    float tensor_scale = 0.0f;
    if constexpr (!DYN) {
        if (lg < 0) {
            tensor_scale = a.absmax ? scale_from_absmax<FDT>(*a.absmax, a.range)
                                    : static_cast<float>(static_cast<const F *>(a.scale_in)[0]);
        }
    }

    const long long stride = (long long)gridDim.x * blockDim.x * UNR;
    for (long long base = (long long)blockIdx.x * blockDim.x * UNR + threadIdx.x; base - threadIdx.x < a.nunits;
         base += stride) {
        RawUnit<IN_BYTES> raw[UNR];
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            const long long idx = base + (long long)k * blockDim.x;
            load_unit<IN_BYTES>(raw[k], in + idx * IN_BYTES, idx < a.nunits, aligned32);
        }
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            const long long idx = base + (long long)k * blockDim.x;
            const bool valid = idx < a.nunits;
            float x[U];
#pragma unroll
            for (int v = 0; v < UT::IN_VEC16; ++v) widen16<FDT>(raw[k].v[v], x + v * FInfo<FDT>::PER16);

            float scale_f;
            if constexpr (DYN) {
                float amax = 0.0f;
#pragma unroll
                for (int i = 0; i < U; ++i) amax = fmaxf(amax, fabsf(x[i]));
                // Blocks are aligned runs of 2^lg lanes; every lane of the warp takes part.
#pragma unroll
                for (int m = 1; m < 32; m <<= 1)
                    if (m < (1 << lg)) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
                scale_f = scale_from_absmax<FDT>(amax, a.range);
            } else {
                scale_f = (lg < 0) ? tensor_scale
                                   : (valid ? static_cast<float>(static_cast<const F *>(a.scale_in)[idx >> lg]) : 1.0f);
            }
            // write_scale: the scale is cast to the param type, stored, and that value (cast
            // back to F) is the divisor (crates/cubek-quant/src/quantize.rs:83-98).
            const float s_fs = round_to_dyn(a.param, scale_f);
            const float s = round_to<FDT>(s_fs);
            if (valid) {
                if (lg < 0) {
                    if (idx == 0) store_dyn(a.out_scale, a.param, 0, s_fs);
                } else if ((idx & ((1ll << lg) - 1)) == 0) {
                    store_dyn(a.out_scale, a.param, idx >> lg, s_fs);
                }
            }
            const bool fast = kind_allows_fast<FDT, KIND>() && !a.force_exact && scale_is_safe(s);
            uint32_t w[OW];
            quantize_unit<FDT, KIND, DYN>(x, s, a.lo, a.hi, fast, w);
            if (valid) {
                if constexpr (OW == 1) stg32_stream(out + idx, w[0]);
                else stg64_stream(out + idx * 2, w[0], w[1]);
            }
        }
    }
}

// -------------------------------------------------------------------------------------
// Scales only (per block), for the two-call form: absmax over each block then the scale
// formula, written as F.  Same unit/shuffle geometry as the fused kernel (KIND fixed to
// the 16-byte unit).
// -------------------------------------------------------------------------------------
template <int FDT>
__global__ void __launch_bounds__(256) block_scales_kernel(const void *in_, void *scale_out, long long nchunks,
                                                           int lg_chunks_per_block, float range)
{
    using F = typename ElemOf<FDT>::type;
    constexpr int PER = FInfo<FDT>::PER16;
    constexpr int UNR = 4;
    const char *in = static_cast<const char *>(in_);
    const int lg = lg_chunks_per_block;
    const long long stride = (long long)gridDim.x * blockDim.x * UNR;
    for (long long base = (long long)blockIdx.x * blockDim.x * UNR + threadIdx.x; base - threadIdx.x < nchunks;
         base += stride) {
        Vec16 raw[UNR];
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            const long long idx = base + (long long)k * blockDim.x;
            raw[k] = (idx < nchunks) ? ldg128_stream(in + idx * 16) : Vec16{{0u, 0u, 0u, 0u}};
        }
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            const long long idx = base + (long long)k * blockDim.x;
            float x[PER];
            widen16<FDT>(raw[k], x);
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < PER; ++i) amax = fmaxf(amax, fabsf(x[i]));
#pragma unroll
            for (int m = 1; m < 32; m <<= 1)
                if (m < (1 << lg)) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
            if (idx < nchunks && (idx & ((1ll << lg) - 1)) == 0)
                static_cast<F *>(scale_out)[idx >> lg] = static_cast<F>(scale_from_absmax<FDT>(amax, range));
        }
    }
}

// Host-side launchers, one translation unit per float type.
cudaError_t launch_quantize(int fdt, int kind, bool dyn, const QuantArgs &args, const LaunchCfg &cfg,
                            cudaStream_t stream);
cudaError_t launch_block_scales(int fdt, const void *in, void *scale_out, long long nchunks, int lg,
                                float range, const LaunchCfg &cfg, cudaStream_t stream);

// Elements per unit for (float type, kind), for the host-side geometry checks.
int unit_elems(int fdt, int kind);

}  // namespace qk
