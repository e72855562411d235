// Quantize kernels: symmetric scale, round, clamp, pack (u32 store) or native cast.
//
// Replaces quantize_symmetric_packed_kernel / quantize_symmetric_native_kernel of the
// reference (crates/cubek-quant/src/quantize.rs:100-171).  The reference gives each thread
// one u32 and resolves the scale index with a div/mod chain per thread; here a thread owns
// a "unit" of consecutive elements (16..64 bytes of input, whole output words), blocks are
// power-of-two runs of units, and in the fused form the absmax of a block is reduced in
// registers (plus warp shuffles when a block spans several lanes) so that the data is read
// exactly once.
//
// The path is HBM bound only if the arithmetic stays cheap: at 6.5 TB/s a bf16 -> q4 kernel
// consumes ~9 elements per clock per SM, which leaves ~7 ALU-pipe lane-instructions per
// element.  The element arithmetic below is therefore written per float type:
//   * f32: exact division as x*r corrected by two FMAs (r = RN(1/s)), rounding by adding
//     1.5*2^23, packing with shifts-as-multiplies;
//   * f16 / bf16: the product x*r in f32 narrowed by one cvt.rn.{f16,bf16}x2.f32 gives the
//     correctly rounded quotient in F (see fast path notes); clamp, round-to-integer and the
//     code bias are then done two elements at a time in packed {f16,bf16}x2 arithmetic.
// A slow route with the reference arithmetic spelled out (true division, rintf) handles
// scales outside the window where those shortcuts are proven, and is what the tests compare
// the fast route against.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace qk {

// A launch covers one tensor or a batch of tensors that share the scheme, float type and unit
// geometry.  Units are numbered across the batch; `unit_end` is the running total.
// (128 per launch, a 6 KB kernel argument, was measured on 8-way shards of a 225-tensor set and on single-tensor
// calls: no faster anywhere, 2 % slower on the shards.)
#ifndef QK_MAX_BATCH_TENSORS
#define QK_MAX_BATCH_TENSORS 64
#endif
constexpr int QK_MAX_BATCH = QK_MAX_BATCH_TENSORS;

struct QuantTensor {
    const void *in;        // F-typed input, contiguous
    void *out;             // u32 words or native bytes
    const void *scale_in;  // F-typed scales (given-scale form); contiguous, one per block
    void *out_scale;       // param-typed scales out
    long long unit_end;    // units in this and all earlier tensors of the batch
    long long tile_end;    // 16 KB tiles in this and all earlier tensors (staged kernels; tiles do not span tensors)
};

struct QuantArgs {
    QuantTensor t[QK_MAX_BATCH];
    int ntensors;
    const float *absmax;     // per tensor: absmax scalars on the device, one per tensor of the batch
                             // (overrides scale_in)
    long long nunits;        // units in the whole batch
    int lg_units_per_block;  // log2(units per block); -1 = per tensor
    Blocks2D b2;             // [rows, cols] tiles instead of runs (given-scale form only)
    RowStride rs;            // row-strided input (direct kernel only)
    Transposed tr;           // transposed input (quantize_transposed_kernel only)
    int param;               // QkParam of out_scale
    float lo, hi, range;     // clamp bounds, hi - lo
    float inv_range;         // RN(1 / range), computed on the host
    int force_exact;         // 1: reference arithmetic for every unit
    int aligned32;           // every input and output base is 32-byte aligned (256-bit accesses allowed)
    PassSplit split;         // full passes of the grid (filled by the launcher once the grid is known)
};

// A unit: UB bytes of input handled by one thread.
template <int FDT, int KIND, int UB> struct UnitT {
    static constexpr int ESZ = FInfo<FDT>::SIZE;
    static constexpr int U = UB / ESZ;                      // elements
    static constexpr int EPW = kind_elems_per_u32(KIND);    // elements per output word
    static constexpr int OW = U / EPW;                      // output words (1, 2, 4 or 8)
    static constexpr int RAW = UB / 4;                      // 32-bit registers of input
    static_assert(U % EPW == 0 && OW >= 1, "a unit must fill whole output words");
};

// Smallest unit for (float type, kind): one 128-bit access and one output word.
__host__ __device__ constexpr int min_unit_bytes(int fdt, int kind)
{
    return cmax(16, kind_elems_per_u32(kind) * ((fdt == QK_F32) ? 4 : 2));
}

// 1.5 * 2^23: adding it to |v| < 2^22 rounds v to an integer (half to even) and leaves that
// integer, in two's complement, in the low mantissa bits.
#define QK_MAGIC 12582912.0f
#define QK_MAGIC_BITS 0x4B400000u

// ---- packed half helpers ----------------------------------------------------------------
template <int FDT> __device__ __forceinline__ uint32_t h2_absmax(uint32_t a, uint32_t b)
{
    uint32_t r;  // magnitude = max(|a|,|b|) per half; the sign bit is the xor of the signs
    if constexpr (FDT == QK_BF16) asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    else asm("max.xorsign.abs.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
template <int FDT> __device__ __forceinline__ uint32_t h2_add(uint32_t a, uint32_t b)
{
    uint32_t r;
    if constexpr (FDT == QK_BF16) asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    else asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
template <int FDT> __device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b)
{
    uint32_t r;
    if constexpr (FDT == QK_BF16) asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    else asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
template <int FDT> __device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b)
{
    uint32_t r;
    if constexpr (FDT == QK_BF16) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    else asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
template <int FDT> __device__ __forceinline__ uint32_t h2_min(uint32_t a, uint32_t b)
{
    uint32_t r;
    if constexpr (FDT == QK_BF16) asm("min.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    else asm("min.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
template <int FDT> __device__ __forceinline__ uint32_t h2_max(uint32_t a, uint32_t b)
{
    uint32_t r;
    if constexpr (FDT == QK_BF16) asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    else asm("max.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
// Two f32 -> packed F x2 (lo in bits 0..15), round to nearest even.
template <int FDT> __device__ __forceinline__ uint32_t h2_pack(float lo, float hi)
{
    if constexpr (FDT == QK_BF16) return pack_bf16x2(lo, hi);
    else return pack_f16x2(lo, hi);
}
// A small integer-valued constant as packed F x2 (both halves).
template <int FDT> __device__ __forceinline__ uint32_t h2_const(float v) { return h2_pack<FDT>(v, v); }

// Two f32 products with one packed instruction (mul.rn.f32x2: one issue slot for both lanes' pair).
__device__ __forceinline__ void mul2(float a0, float a1, float b, float &o0, float &o1)
{
#ifdef QK_NO_F32X2
    o0 = a0 * b;
    o1 = a1 * b;
#else
    asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmul.rn.f32x2 rc, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rc;\n\t}"
        : "=f"(o0), "=f"(o1)
        : "f"(a0), "f"(a1), "f"(b));
#endif
}

// Two fused multiply-adds / sums with one packed instruction each (IEEE per lane, like the scalar forms).
__device__ __forceinline__ void fma2(float a0, float a1, float b0, float b1, float c0, float c1, float &o0, float &o1)
{
#ifdef QK_NO_F32X2
    o0 = __fmaf_rn(a0, b0, c0);
    o1 = __fmaf_rn(a1, b1, c1);
#else
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(o0), "=f"(o1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
#endif
}
__device__ __forceinline__ void add2(float a0, float a1, float b, float &o0, float &o1)
{
#ifdef QK_NO_F32X2
    o0 = a0 + b;
    o1 = a1 + b;
#else
    asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tadd.rn.f32x2 rc, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rc;\n\t}"
        : "=f"(o0), "=f"(o1)
        : "f"(a0), "f"(a1), "f"(b));
#endif
}

template <int FDT> __device__ __forceinline__ float h_lo_to_f32(uint32_t p)
{
    if constexpr (FDT == QK_BF16) return bf16_lo_to_f32(p);
    else return __low2float(*reinterpret_cast<const __half2 *>(&p));   // half selected by the instruction
}
template <int FDT> __device__ __forceinline__ float h_hi_to_f32(uint32_t p)
{
    if constexpr (FDT == QK_BF16) return bf16_hi_to_f32(p);
    else return __high2float(*reinterpret_cast<const __half2 *>(&p));
}

// Element i of the raw registers, widened to f32.
template <int FDT> __device__ __forceinline__ float raw_elem(const uint32_t *raw, int i)
{
    if constexpr (FDT == QK_F32) return __uint_as_float(raw[i]);
    else return (i & 1) ? h_hi_to_f32<FDT>(raw[i >> 1]) : h_lo_to_f32<FDT>(raw[i >> 1]);
}

// absmax of the unit as f32 (exact: it is one of the inputs).  NaNs are ignored.
template <int FDT, int RAW> __device__ __forceinline__ float unit_absmax(const uint32_t *raw)
{
    if constexpr (FDT == QK_F32) {
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < RAW; i += 2) m = fmax3(m, fabsf(__uint_as_float(raw[i])), fabsf(__uint_as_float(raw[i + 1])));
        return m;
    } else {
        uint32_t m = raw[0];
#pragma unroll
        for (int i = 1; i < RAW; ++i) m = h2_absmax<FDT>(m, raw[i]);
        m = h2_absmax<FDT>(m, m >> 16) & 0x7fffu;  // low half: max(|lo|, |hi|)
        return h_lo_to_f32<FDT>(m);
    }
}

// ---- scale arithmetic (once per unit) -------------------------------------------------------

// (2*absmax) / range, correctly rounded.  Inside [2^-100, 2^100] the quotient is obtained as
// q0 = a*inv, q = fma(fma(-range, q0, a), inv, q0) with inv = RN(1/range): exhaustively equal to
// IEEE division for every f32 `a` in that window and every range of a supported value type.
__device__ __forceinline__ float div_by_range(float a, float range, float inv_range)
{
    if (a >= 7.888609052e-31f && a <= 1.267650600e+30f) {
        const float q0 = a * inv_range;
        return __fmaf_rn(__fmaf_rn(-range, q0, a), inv_range, q0);
    }
    return __fdiv_rn(a, range);
}

// Scales outside this window (zero, tiny, huge, negative, NaN) take the reference arithmetic:
// the shortcuts assume 1/s and x*(1/s) stay inside the normal range.
__device__ __forceinline__ bool scale_is_safe(float s)
{
    return s >= 7.888609052e-31f /* 2^-100 */ && s <= 1.267650600e+30f /* 2^100 */;
}

// Every kind takes the shortcuts.  E5M2 clamps at +-57344, beyond the window of the integer kinds: for
// 16-bit inputs the half-precision shortcut was checked on the host up to |x/s| = 2^18, overflow of
// f16 to infinity included (the clamp then gives the bound either way).
template <int FDT, int KIND> __host__ __device__ constexpr bool kind_allows_fast()
{
#ifdef QK_ROUND_HALF_AWAY
    return false;   // the shortcuts round halves to even
#else
    return true;
#endif
}

// ---- packing of integral f32 values -----------------------------------------------------------
// `c` holds integral (or to-be-rounded, already clamped) f32 values in element order.
template <int KIND, int U> __device__ __forceinline__ void pack_from_f32(const float *c, uint32_t *outw)
{
    constexpr int EPW = kind_elems_per_u32(KIND);
    constexpr int OW = U / EPW;
    if constexpr (KIND == KIND_PACK8 || KIND == KIND_I8) {
#pragma unroll
        for (int w = 0; w < OW; ++w) {
            uint32_t b[4];
#pragma unroll
            for (int i = 0; i < 4; i += 2) {
                float m0, m1;
                if constexpr (U >= 16) add2(c[4 * w + i], c[4 * w + i + 1], QK_MAGIC, m0, m1);
                else m0 = c[4 * w + i] + QK_MAGIC, m1 = c[4 * w + i + 1] + QK_MAGIC;
                b[i] = __float_as_uint(m0), b[i + 1] = __float_as_uint(m1);
            }
            const uint32_t l = __byte_perm(b[0], b[1], 0x0040);
            const uint32_t h = __byte_perm(b[2], b[3], 0x0040);
            outw[w] = __byte_perm(l, h, 0x5410);
        }
    } else if constexpr (KIND == KIND_PACK4 || KIND == KIND_PACK2) {
        // Bias every code to be non-negative (q + 2^(bits-1)), sum the shifted float bit
        // patterns (shifts as multiplies, which run on the FMA pipe), remove the constant part,
        // then flip the top bit of every field to return to two's complement.
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
            for (int i = 0; i < EPW; ++i)
                acc += __float_as_uint(c[EPW * w + i] + (QK_MAGIC + (float)BIAS)) * (1u << (i * BITS));
            outw[w] = (acc - kconst) ^ FLIP;
        }
    } else if constexpr (KIND == KIND_E2M1) {
#pragma unroll
        for (int w = 0; w < OW; ++w) {
            uint32_t by[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // round to integer; keep the sign of a zero result (-0.3 -> -0, code 0b1000)
                const float a = copysignf((c[8 * w + 2 * i] + QK_MAGIC) - QK_MAGIC, c[8 * w + 2 * i]);
                const float b = copysignf((c[8 * w + 2 * i + 1] + QK_MAGIC) - QK_MAGIC, c[8 * w + 2 * i + 1]);
                by[i] = cvt_e2m1x2(a, b);
            }
            const uint32_t l = __byte_perm(by[0], by[1], 0x0040);
            const uint32_t h = __byte_perm(by[2], by[3], 0x0040);
            outw[w] = __byte_perm(l, h, 0x5410);
        }
    } else {  // KIND_E4M3 / KIND_E5M2
#pragma unroll
        for (int w = 0; w < OW; ++w) {
            uint32_t hw[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float a = rintf(c[4 * w + 2 * i]);
                const float b = rintf(c[4 * w + 2 * i + 1]);
                hw[i] = (KIND == KIND_E4M3) ? cvt_e4m3x2(a, b) : cvt_e5m2x2(a, b);
            }
            outw[w] = __byte_perm(hw[0], hw[1], 0x5410);
        }
    }
}

// ---- reference arithmetic route ---------------------------------------------------------------
template <int FDT, int KIND, int UB>
__device__ void quantize_unit_exact(const uint32_t *raw, float s, float lo, float hi, uint32_t *outw)
{
    using UT = UnitT<FDT, KIND, UB>;
    float c[UT::U];
#pragma unroll
    for (int i = 0; i < UT::U; ++i) c[i] = quantize_exact<FDT>(raw_elem<FDT>(raw, i), s, lo, hi);
    pack_from_f32<KIND, UT::U>(c, outw);
}

// ---- fast route ---------------------------------------------------------------------------------
// Valid for scale_is_safe(s) and finite inputs.  CLAMP = false is used by the fused form when
// |x/s| cannot reach hi + 0.5 (see need_clamp()).
//   f32 quotient: q0 = x*r, q = fma(fma(-s, q0, x), r, q0) with r = RN(1/s) is the correctly
//     rounded quotient.  With a caller-supplied scale (BOUNDED = false) the first guess is
//     clamped so that a huge quotient ends as +-inf or a huge value of the right sign (never NaN).
//   f16 / bf16 quotient: x and s carry 11 / 8 significant bits, so x/s is never closer than
//     2^-23 / 2^-17 (relative) to a rounding boundary of F; the f32 product x*r rounds to the
//     same F value as the exact quotient for every |x/s| in [1/8, 2^18] (checked exhaustively on
//     the host for all pairs; the property depends on the two significands only); outside that
//     range the code is 0 or the clamp bound either way.
template <int FDT, int KIND, int UB, bool CLAMP, bool BOUNDED>
__device__ __forceinline__ void quantize_unit_fast(const uint32_t *raw, float s, float lo, float hi, uint32_t *outw)
{
    using UT = UnitT<FDT, KIND, UB>;
    constexpr int U = UT::U;
    constexpr int EPW = UT::EPW;
    constexpr int OW = UT::OW;
    const float r = __frcp_rn(s);

    if constexpr (FDT == QK_F32) {
        float c[U];
        const float ms = -s;
#pragma unroll
        for (int i = 0; i < U; i += 2) {
            const float x0 = __uint_as_float(raw[i]), x1 = __uint_as_float(raw[i + 1]);
            float q0, q1, e0, e1, t0, t1;
            constexpr bool PACKED = (UB >= 64);   // the packed forms want register pairs: smaller units have none to spare
            if constexpr (PACKED) mul2(x0, x1, r, q0, q1);
            else q0 = x0 * r, q1 = x1 * r;
            if constexpr (!BOUNDED) {
                q0 = fminf(fmaxf(q0, lo - 2.0f), hi + 2.0f);
                q1 = fminf(fmaxf(q1, lo - 2.0f), hi + 2.0f);
            }
            if constexpr (PACKED) {
                fma2(ms, ms, q0, q1, x0, x1, e0, e1);
                fma2(e0, e1, r, r, q0, q1, t0, t1);
            } else {
                e0 = __fmaf_rn(ms, q0, x0), e1 = __fmaf_rn(ms, q1, x1);
                t0 = __fmaf_rn(e0, r, q0), t1 = __fmaf_rn(e1, r, q1);
            }
            // The 4- and 2-bit packs add shifted bit patterns: a NaN would carry into the fields of its neighbours, so
            // the unclamped form still takes the minimum with the upper bound (which a NaN does not survive).
            constexpr bool ADDS = (KIND == KIND_PACK4 || KIND == KIND_PACK2);
            c[i] = CLAMP ? fminf(fmaxf(t0, lo), hi) : (ADDS ? fminf(t0, hi) : t0);
            c[i + 1] = CLAMP ? fminf(fmaxf(t1, lo), hi) : (ADDS ? fminf(t1, hi) : t1);
        }
        pack_from_f32<KIND, U>(c, outw);
    } else if constexpr ((KIND == KIND_E4M3 || KIND == KIND_E5M2) && FDT == QK_F16) {
        // f16 quotients stay packed: clamp, round to integer and convert two at a time (the integer rounding comes
        // before the cast, as in the reference; e4m3's bound 448 is inside the range of the magic-number rounding,
        // e5m2's 57344 is not and takes cvt.rni).
        const uint32_t lo2 = h2_const<FDT>(lo), hi2 = h2_const<FDT>(hi), magic = h2_const<FDT>(1536.0f);
#pragma unroll
        for (int w = 0; w < OW; ++w) {
            uint32_t hw[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float q0, q1;
                mul2(raw_elem<FDT>(raw, 4 * w + 2 * j), raw_elem<FDT>(raw, 4 * w + 2 * j + 1), r, q0, q1);
                uint32_t p = h2_min<FDT>(h2_max<FDT>(h2_pack<FDT>(q0, q1), lo2), hi2);
                if constexpr (KIND == KIND_E4M3) {
                    const uint32_t q = h2_sub<FDT>(h2_add<FDT>(p, magic), magic);
                    p = (q & 0x7fff7fffu) | (p & 0x80008000u);   // keep the sign of zero
                    hw[j] = cvt_e4m3x2_from_f16x2(p);
                } else {
                    hw[j] = cvt_e5m2x2_from_f16x2(f16x2_rint(p));
                }
            }
            outw[w] = __byte_perm(hw[0], hw[1], 0x5410);
        }
    } else if constexpr (KIND == KIND_E4M3 || KIND == KIND_E5M2) {
        float c[U];
#pragma unroll
        for (int i = 0; i < U; i += 2) {
            float q0, q1;
            mul2(raw_elem<FDT>(raw, i), raw_elem<FDT>(raw, i + 1), r, q0, q1);
            const uint32_t p = h2_pack<FDT>(q0, q1);
            c[i] = fminf(fmaxf(h_lo_to_f32<FDT>(p), lo), hi);
            c[i + 1] = fminf(fmaxf(h_hi_to_f32<FDT>(p), lo), hi);
        }
        pack_from_f32<KIND, U>(c, outw);
    } else {
        // Packed route.  Quotients are narrowed to F two at a time; which two elements share a
        // register is chosen per kind so that the output word can be assembled with left shifts
        // only: element j and element j + EPW/2 of a word for the integer packs, neighbours
        // (2j, 2j+1) for fp4 bytes and for bf16 8-bit codes.
        const uint32_t lo2 = h2_const<FDT>(lo), hi2 = h2_const<FDT>(hi);
        constexpr bool SPLIT_PAIRS = (KIND == KIND_PACK4 || KIND == KIND_PACK2 ||
                                      ((KIND == KIND_PACK8 || KIND == KIND_I8) && FDT == QK_F16));
#pragma unroll
        for (int w = 0; w < OW; ++w) {
            uint32_t p[EPW / 2];
#pragma unroll
            for (int j = 0; j < EPW / 2; ++j) {
                const int e0 = w * EPW + (SPLIT_PAIRS ? j : 2 * j);
                const int e1 = w * EPW + (SPLIT_PAIRS ? j + EPW / 2 : 2 * j + 1);
                float q0, q1;
                mul2(raw_elem<FDT>(raw, e0), raw_elem<FDT>(raw, e1), r, q0, q1);
                uint32_t q = h2_pack<FDT>(q0, q1);
                if constexpr (CLAMP) q = h2_min<FDT>(h2_max<FDT>(q, lo2), hi2);
                else if constexpr (KIND == KIND_PACK4 || KIND == KIND_PACK2) q = h2_min<FDT>(q, hi2);   // NaN -> hi, see above
                p[j] = q;
            }
            if constexpr (KIND == KIND_PACK4 || KIND == KIND_PACK2) {
                // F(192 + b) = 0x4340 + b (bf16), F(1536 + b) = 0x6600 + b (f16) for small b >= 0.
                constexpr int BITS = kind_bits(KIND);
                constexpr float BIAS = (float)(1 << (BITS - 1));
                constexpr uint32_t HBITS = (FDT == QK_BF16) ? 0x43404340u : 0x66006600u;
                constexpr uint32_t FLIP = (BITS == 4) ? 0x88888888u : 0xAAAAAAAAu;
                const uint32_t magic = h2_const<FDT>(((FDT == QK_BF16) ? 192.0f : 1536.0f) + BIAS);
                uint32_t kconst = 0, acc = 0;
#pragma unroll
                for (int j = 0; j < EPW / 2; ++j) {
                    kconst += HBITS << (j * BITS);
                    acc += h2_add<FDT>(p[j], magic) * (1u << (j * BITS));
                }
                outw[w] = (acc - kconst) ^ FLIP;
            } else if constexpr (KIND == KIND_PACK8 || KIND == KIND_I8) {
                if constexpr (FDT == QK_F16) {
                    // low byte of each half = q + 128; p[0] = (e0, e2), p[1] = (e1, e3)
                    const uint32_t magic = h2_const<FDT>(1536.0f + 128.0f);
                    const uint32_t a = h2_add<FDT>(p[0], magic), b = h2_add<FDT>(p[1], magic);
                    outw[w] = __byte_perm(a, b, 0x6240) ^ 0x80808080u;
                } else {
                    // bf16 cannot hold 9-bit integers: finish in f32.
                    uint32_t b[4];
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        float m0, m1;
                        add2(bf16_lo_to_f32(p[j]), bf16_hi_to_f32(p[j]), QK_MAGIC, m0, m1);
                        b[2 * j] = __float_as_uint(m0), b[2 * j + 1] = __float_as_uint(m1);
                    }
                    const uint32_t l = __byte_perm(b[0], b[1], 0x0040);
                    const uint32_t h = __byte_perm(b[2], b[3], 0x0040);
                    outw[w] = __byte_perm(l, h, 0x5410);
                }
            } else {  // KIND_E2M1: p[j] = (e_2j, e_2j+1) -> byte j
                const uint32_t magic = h2_const<FDT>((FDT == QK_BF16) ? 192.0f : 1536.0f);
                uint32_t by[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t q = h2_sub<FDT>(h2_add<FDT>(p[j], magic), magic);   // round to integer
                    q = (q & 0x7fff7fffu) | (p[j] & 0x80008000u);                // keep the sign of zero
                    by[j] = cvt_e2m1x2(h_lo_to_f32<FDT>(q), h_hi_to_f32<FDT>(q));
                }
                const uint32_t l = __byte_perm(by[0], by[1], 0x0040);
                const uint32_t h = __byte_perm(by[2], by[3], 0x0040);
                outw[w] = __byte_perm(l, h, 0x5410);
            }
        }
    }
}

// Whether the fused form must clamp: with scale = 2*absmax/(hi-lo) taken from the same data,
// |x/s| <= (hi-lo)/2 * (1 + e) where e covers the narrowing of the scale to F and to the param
// type.  For symmetric ranges and f32 params that never reaches hi + 0.5, except for 8-bit codes
// of bf16 inputs (127 * (1 + 2^-9) narrows to 127.5, which rounds to 128).  Everything else
// (the "F" ranges, whose positive bound is one short; half-precision params; given scales) clamps.
__host__ __device__ constexpr bool need_clamp(int fdt, int kind, bool dyn, bool symmetric, int param)
{
    if (!dyn || !symmetric || param != QK_F32) return true;
    if (kind == KIND_E4M3 || kind == KIND_E5M2) return true;
    if (fdt == QK_BF16 && (kind == KIND_PACK8 || kind == KIND_I8)) return true;
    return false;
}

// -------------------------------------------------------------------------------------
// Loading / storing one unit.
// -------------------------------------------------------------------------------------
template <int UB> __device__ __forceinline__ void load_unit(uint32_t *raw, const char *p, bool aligned32)
{
    if constexpr (UB == 16) {
        const Vec16 v = ldg128_stream(p);
#pragma unroll
        for (int i = 0; i < 4; ++i) raw[i] = v.w[i];
    } else {
        if (aligned32) {
#pragma unroll
            for (int k = 0; k < UB / 32; ++k) {
                const Vec32 v = ldg256_stream(p + 32 * k);
#pragma unroll
                for (int i = 0; i < 8; ++i) raw[8 * k + i] = v.w[i];
            }
        } else {
#pragma unroll
            for (int k = 0; k < UB / 16; ++k) {
                const Vec16 v = ldg128_stream(p + 16 * k);
#pragma unroll
                for (int i = 0; i < 4; ++i) raw[4 * k + i] = v.w[i];
            }
        }
    }
}

template <int OW> __device__ __forceinline__ void store_words(uint32_t *dst, const uint32_t *w, bool aligned32)
{
    if constexpr (OW == 1) {
        stg32_stream(dst, w[0]);
    } else if constexpr (OW == 2) {
        stg64_stream(dst, w[0], w[1]);
    } else if constexpr (OW == 4) {
        stg128_stream(dst, Vec16{{w[0], w[1], w[2], w[3]}});
    } else {
        static_assert(OW == 8, "1, 2, 4 or 8 output words");
        if (aligned32) {
            stg256_stream(dst, Vec32{{w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]}});
        } else {
            stg128_stream(dst, Vec16{{w[0], w[1], w[2], w[3]}});
            stg128_stream(dst + 4, Vec16{{w[4], w[5], w[6], w[7]}});
        }
    }
}

// -------------------------------------------------------------------------------------
// Pieces shared by the direct and the staged kernel.
// -------------------------------------------------------------------------------------

// Scale of a fused unit: absmax of its block (the unit's own registers, then the lanes that share the
// block: aligned runs of 2^lg lanes; every lane of the warp takes part), then the scale formula.
// LG0: the block is the unit (lg == 0 known at compile time): no shuffle rounds, no tests for them.
// NaN elements do not take part (maxima return the other operand), as in the reference's MaxAbs
// (crates/cubek-reduce/src/instructions/maxabs.rs:62-63).
template <int FDT, int RAW, bool LG0 = false>
__device__ __forceinline__ float fused_unit_scale(const uint32_t *raw, int lg, float range, float inv_range)
{
    float amax = unit_absmax<FDT, RAW>(raw);
    if constexpr (!LG0) {
#pragma unroll
        for (int m = 1; m < 32; m <<= 1)
            if (m < (1 << lg)) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    }
    return round_to<FDT>(div_by_range(2.0f * amax, range, inv_range));
}

// Scale of a per-tensor launch (given as a tensor of one F, or derived from a device absmax cell).
template <int FDT>
__device__ __forceinline__ float tensor_unit_scale(const QuantArgs &a, const QuantTensor &T, int tensor)
{
    using F = typename ElemOf<FDT>::type;
    return a.absmax ? round_to<FDT>(div_by_range(2.0f * a.absmax[tensor], a.range, a.inv_range))
                    : static_cast<float>(static_cast<const F *>(T.scale_in)[0]);
}

// write_scale, quantize, store: the scale is cast to the param type, stored by the unit that starts
// the block (unit 0 for per tensor), and that value cast back to F is the divisor
// (crates/cubek-quant/src/quantize.rs:83-98).  SUB = 2: the unit holds two blocks (halves of the unit), each
// with its own scale; `sidx` is then the index of the first of the two (f32 params, 8-byte aligned scales).
template <int FDT, int KIND, int UB, bool DYN, bool CLAMP, int SUB = 1>
__device__ __forceinline__ void finish_unit(const QuantArgs &a, const QuantTensor &T, const uint32_t *raw,
                                            const float *scale_f, long long sidx, bool starts, long long li, bool valid,
                                            bool aligned32)
{
    constexpr int OW = UnitT<FDT, KIND, UB>::OW;
    constexpr int RAW = UnitT<FDT, KIND, UB>::RAW;
    static_assert(SUB == 1 || (SUB == 2 && OW % 2 == 0), "a half unit must fill whole output words");
    float s_fs[SUB], s[SUB];
#pragma unroll
    for (int j = 0; j < SUB; ++j) {
        s_fs[j] = (a.param == QK_F32) ? scale_f[j] : round_to_dyn(a.param, scale_f[j]);
        s[j] = (a.param == QK_F32) ? scale_f[j] : round_to<FDT>(s_fs[j]);
    }
    if (valid && starts) {
        if constexpr (SUB == 1) store_dyn(T.out_scale, a.param, sidx, s_fs[0]);
        else *reinterpret_cast<float2 *>(static_cast<float *>(T.out_scale) + sidx) = make_float2(s_fs[0], s_fs[1]);
    }
    uint32_t w[OW];
#pragma unroll
    for (int j = 0; j < SUB; ++j) {
        if (kind_allows_fast<FDT, KIND>() && !a.force_exact && scale_is_safe(s[j]))
            quantize_unit_fast<FDT, KIND, UB / SUB, CLAMP, DYN>(raw + j * (RAW / SUB), s[j], a.lo, a.hi, w + j * (OW / SUB));
        else
            quantize_unit_exact<FDT, KIND, UB / SUB>(raw + j * (RAW / SUB), s[j], a.lo, a.hi, w + j * (OW / SUB));
    }
    if (valid) store_words<OW>(static_cast<uint32_t *>(T.out) + li * OW, w, aligned32);
}

// -------------------------------------------------------------------------------------
// The kernel.  DYN = true: scale from the block's own absmax (one pass, fused).
// DYN = false: scale given (tensor of F, one per block) or derived from a device absmax.
// -------------------------------------------------------------------------------------
// Resident CTAs per SM the register allocation must allow: 3 (at most 85 registers), 4 for the fused
// two-blocks-per-unit form, which fits 64 registers with at most a few spilled words.
#ifndef QK_GIVEN_MIN_CTAS
#define QK_GIVEN_MIN_CTAS 3
#endif
#ifndef QK_SUB2_MIN_CTAS
#define QK_SUB2_MIN_CTAS 4
#endif
#define QK_MIN_CTAS(DYN, SUB) ((DYN) ? ((SUB) == 2 ? QK_SUB2_MIN_CTAS : 3) : QK_GIVEN_MIN_CTAS)
// SUB = 2: two blocks per unit (16-bit types).  LG0: one block per unit, known at compile time.
// Units are walked in grid-wide passes (see PassSplit).
// ONE_SITE: the pass body is inlined once instead of twice (see QK_WALK_PASSES_ONE_SITE).
template <int FDT, int KIND, int UB, bool DYN, bool CLAMP, int SUB = 1, bool LG0 = false, bool ONE_SITE = false>
__global__ void __launch_bounds__(256, QK_MIN_CTAS(DYN, SUB)) quantize_kernel(const QuantArgs a)
{
    using UT = UnitT<FDT, KIND, UB>;
    constexpr int RAW = UT::RAW;
    constexpr int UNR = (UB >= 64) ? 2 : 4;  // units in flight per thread (128 bytes; 64 for 16-byte units)
    using F = typename ElemOf<FDT>::type;

    const bool aligned32 = a.aligned32 != 0;
    const int lg = (LG0 || SUB == 2) ? 0 : a.lg_units_per_block;
    pdl_entry();

    int ti = 0;                 // tensor of the batch this thread is in (only ever moves forward)
    int scale_ti = -1;          // tensor `tensor_scale` belongs to
    float tensor_scale = 0.0f;  // per tensor: one scale for the whole tensor

    // One pass over UNR units of this thread.  `full`: all of them exist.  Otherwise a unit may lie past the end
    // (it is loaded as zeros and stores nothing), and rows of 32 units that lie past the end entirely are skipped
    // by their whole warp.
    auto pass = [&](const long long (&idx)[UNR], const bool full) {
        uint32_t raw[UNR][RAW];
        int tk[UNR];
        long long lidx[UNR];
        // Given block scales are fetched together with the data, so that the two latencies overlap
        // (loaded after the data, they cost a second round trip per iteration: 5.6 -> 6.1 TB/s on f32 q4).
        float given[UNR][SUB];
        long long given_idx[UNR];
        bool given_starts[UNR];
        const bool block_scales_given = !DYN && (lg >= 0 || a.b2.enabled);
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
#pragma unroll
            for (int j = 0; j < SUB; ++j) given[k][j] = 1.0f;
            given_idx[k] = 0;
            given_starts[k] = false;
            if (full || idx[k] < a.nunits) {
                while (ti + 1 < a.ntensors && idx[k] >= a.t[ti].unit_end) ++ti;
                tk[k] = ti;
                lidx[k] = idx[k] - (ti ? a.t[ti - 1].unit_end : 0);
                long long offset = lidx[k] * UB;
                if (a.rs.enabled) {
                    const unsigned row = fastdiv((unsigned)lidx[k], a.rs.units_per_row);
                    offset = (long long)row * a.rs.row_bytes +
                             (long long)((unsigned)lidx[k] - row * a.rs.units_per_row.div) * UB;
                }
                load_unit<UB>(raw[k], static_cast<const char *>(a.t[ti].in) + offset, aligned32);
                if constexpr (!DYN && SUB == 2) {
                    // the unit's two scales are neighbours: one 32-bit load (16-bit types only)
                    given_idx[k] = 2 * lidx[k];
                    given_starts[k] = true;
                    const uint32_t pair = __ldg(reinterpret_cast<const uint32_t *>(a.t[ti].scale_in) + lidx[k]);
                    given[k][0] = h_lo_to_f32<FDT>(pair);
                    given[k][SUB - 1] = h_hi_to_f32<FDT>(pair);
                } else if constexpr (!DYN) {
                    if (block_scales_given) {
                        if (a.b2.enabled) {
                            given_idx[k] = blocks2d_scale_index(a.b2, (unsigned)lidx[k], &given_starts[k]);
                        } else {
                            given_idx[k] = lidx[k] >> lg;
                            given_starts[k] = (lidx[k] & ((1ll << lg) - 1)) == 0;
                        }
                        given[k][0] = static_cast<float>(static_cast<const F *>(a.t[ti].scale_in)[given_idx[k]]);
                    }
                }
            } else {
                tk[k] = ti;
                lidx[k] = 0;
#pragma unroll
                for (int i = 0; i < RAW; ++i) raw[k][i] = 0u;
            }
        }
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            if (!full && idx[k] - (threadIdx.x & 31) >= a.nunits) continue;   // the whole row lies past the end
            const bool valid = full || idx[k] < a.nunits;
            const QuantTensor &T = a.t[tk[k]];
            const long long li = lidx[k];

            float scale_f[SUB];
            long long sidx = 0;      // index of the unit's scale
            bool starts = false;     // the unit is the first of its block
            if constexpr (DYN && SUB == 2) {
                sidx = 2 * li;
                starts = true;
                scale_f[0] = fused_unit_scale<FDT, RAW / 2, true>(raw[k], 0, a.range, a.inv_range);
                scale_f[1] = fused_unit_scale<FDT, RAW / 2, true>(raw[k] + RAW / 2, 0, a.range, a.inv_range);
            } else if constexpr (DYN) {
                sidx = LG0 ? li : (li >> lg);
                starts = LG0 ? true : ((li & ((1ll << lg) - 1)) == 0);
                scale_f[0] = fused_unit_scale<FDT, RAW, LG0>(raw[k], lg, a.range, a.inv_range);
            } else if (SUB == 1 && lg < 0 && !a.b2.enabled) {
                if (scale_ti != tk[k]) {
                    scale_ti = tk[k];
                    tensor_scale = tensor_unit_scale<FDT>(a, T, scale_ti);
                }
                scale_f[0] = tensor_scale;
                starts = (li == 0);
            } else {
                sidx = given_idx[k];
                starts = given_starts[k];
#pragma unroll
                for (int j = 0; j < SUB; ++j) scale_f[j] = given[k][j];
            }
            finish_unit<FDT, KIND, UB, DYN, CLAMP, SUB>(a, T, raw[k], scale_f, sidx, starts, li, valid, aligned32);
        }
    };

    if constexpr (ONE_SITE) QK_WALK_PASSES_ONE_SITE(a.split.full_passes, a.nunits, UNR, pass);
    else QK_WALK_PASSES(a.split.full_passes, a.nunits, UNR, pass);
}

// -------------------------------------------------------------------------------------
// The same kernel with the input staged through shared memory by the bulk-copy engine:
// one thread issues `cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes` for
// 16 KB tiles into a ring of `nstages` tiles, the CTA waits on the stage's mbarrier, copies its units
// to registers, releases the stage (one __syncthreads, then the refill is issued) and does the
// arithmetic while the other tiles are in flight.
//
// Measured against the direct loads: slower for 64-byte units (a thread's 64 bytes sit 64 bytes
// apart in shared memory: 4-way bank conflicts; 5115 vs 5713 GB/s on bf16 q4), faster for 16- and
// 32-byte units, where the direct kernel has too few bytes in flight per thread (4341 vs 3771 GB/s on
// f16 e2m1 block 16).  The launcher therefore stages units below 64 bytes and loads 64-byte units
// directly; a tuning key forces either route, and the parity tests run both.
//
// Ring depth: these small-unit kernels are bound by instruction issue, not by bytes in flight, so
// resident warps matter more than a deep ring.  Two tiles per CTA (32 KB) leave room for the 5 CTAs
// per SM the 48 registers allow; 3 / 4 tiles allow 4 / 3.  f16 e2m1 block 16, batch of 8 tensors:
// 5244 / 5178 / 4917 GB/s with 2 / 3 / 4 tiles.  Forcing 6 CTAs per SM (40 registers) spills and
// drops to 4949 GB/s.
//
// Every mbarrier wait is bounded: after ~2^22 polls a thread records the failure in
// `*a_error` and leaves the kernel instead of spinning forever.
// -------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbarrier_init(uint64_t *bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbarrier_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbarrier_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(smem_addr(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_load_1d(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

constexpr int QK_MAX_STAGES = 4;     // ring depth is a launch parameter: 2..QK_MAX_STAGES
constexpr int QK_TILE_BYTES = 16384;

template <int FDT, int KIND, int UB, bool DYN, bool CLAMP>
__global__ void __launch_bounds__(256) quantize_staged_kernel(const QuantArgs a, int *a_error, int nstages)
{
    using UT = UnitT<FDT, KIND, UB>;
    constexpr int RAW = UT::RAW;
    constexpr int UPT = QK_TILE_BYTES / (256 * UB);   // units per thread per tile: 1, 2 or 4
    constexpr int TILE_UNITS = 256 * UPT;
    using F = typename ElemOf<FDT>::type;
    extern __shared__ __align__(128) unsigned char stage_mem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(stage_mem + nstages * QK_TILE_BYTES);

    const bool aligned32 = a.aligned32 != 0;
    const int lg = a.lg_units_per_block;
    const long long ntiles = a.t[a.ntensors - 1].tile_end;
    if (threadIdx.x == 0) {
        for (int s = 0; s < nstages; ++s) mbarrier_init(&full[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_entry();

    // Tiles are numbered across the batch; a tile lies in one tensor.  Both walkers only move forward.
    int ti_issue = 0, ti = 0;
    auto issue = [&](long long tile, int s) {
        while (ti_issue + 1 < a.ntensors && tile >= a.t[ti_issue].tile_end) ++ti_issue;
        const QuantTensor &T = a.t[ti_issue];
        const long long tile0 = ti_issue ? a.t[ti_issue - 1].tile_end : 0;
        const long long units = T.unit_end - (ti_issue ? a.t[ti_issue - 1].unit_end : 0);
        const long long u0 = (tile - tile0) * TILE_UNITS;
        long long nu = units - u0;
        if (nu > TILE_UNITS) nu = TILE_UNITS;
        const uint32_t bytes = (uint32_t)(nu * UB);
        mbarrier_expect_tx(&full[s], bytes);
        bulk_load_1d(stage_mem + s * QK_TILE_BYTES, static_cast<const char *>(T.in) + u0 * UB, bytes, &full[s]);
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < nstages; ++s) {
            const long long t = blockIdx.x + (long long)s * gridDim.x;
            if (t < ntiles) issue(t, s);
        }
    }
    int scale_ti = -1;
    float tensor_scale = 0.0f;

    int next_stage = 0;          // the ring position of the coming iteration
    uint32_t next_parity = 0;    // flips every time the ring wraps
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int s = next_stage;
        const uint32_t parity = next_parity;
        if (++next_stage == nstages) {
            next_stage = 0;
            next_parity ^= 1u;
        }
        int polls = 0;
        while (!mbarrier_try_wait(&full[s], parity)) {
            if (++polls > (1 << 22)) {
                atomicExch(a_error, 1);
                return;
            }
        }
        while (ti + 1 < a.ntensors && tile >= a.t[ti].tile_end) ++ti;
        const QuantTensor &T = a.t[ti];
        const long long nunits_t = T.unit_end - (ti ? a.t[ti - 1].unit_end : 0);
        const long long u0 = (tile - (ti ? a.t[ti - 1].tile_end : 0)) * TILE_UNITS;
        uint32_t raw[UPT][RAW];
#pragma unroll
        for (int k = 0; k < UPT; ++k) {
            const long long li = u0 + k * 256 + threadIdx.x;
            const Vec16 *src = reinterpret_cast<const Vec16 *>(stage_mem + s * QK_TILE_BYTES + (k * 256 + threadIdx.x) * UB);
#pragma unroll
            for (int v = 0; v < UB / 16; ++v) {
                const Vec16 t = (li < nunits_t) ? src[v] : Vec16{{0u, 0u, 0u, 0u}};
#pragma unroll
                for (int i = 0; i < 4; ++i) raw[k][4 * v + i] = t.w[i];
            }
        }
        __syncthreads();   // every thread holds its units: the stage can be refilled
        if (threadIdx.x == 0) {
            const long long t = tile + (long long)nstages * gridDim.x;
            if (t < ntiles) issue(t, s);
        }
#pragma unroll
        for (int k = 0; k < UPT; ++k) {
            const long long li = u0 + k * 256 + threadIdx.x;
            const bool valid = li < nunits_t;
            float scale_f[1];
            long long sidx = 0;
            bool starts = false;
            if constexpr (DYN) {
                sidx = li >> lg;
                starts = (li & ((1ll << lg) - 1)) == 0;
                scale_f[0] = fused_unit_scale<FDT, RAW>(raw[k], lg, a.range, a.inv_range);
            } else if (lg < 0 && !a.b2.enabled) {
                if (scale_ti != ti) {
                    scale_ti = ti;
                    tensor_scale = tensor_unit_scale<FDT>(a, T, ti);
                }
                scale_f[0] = tensor_scale;
                starts = (li == 0);
            } else {
                if (a.b2.enabled) {
                    sidx = blocks2d_scale_index(a.b2, (unsigned)li, &starts);
                } else {
                    sidx = li >> lg;
                    starts = (li & ((1ll << lg) - 1)) == 0;
                }
                scale_f[0] = valid ? static_cast<float>(static_cast<const F *>(T.scale_in)[sidx]) : 1.0f;
            }
            finish_unit<FDT, KIND, UB, DYN, CLAMP>(a, T, raw[k], scale_f, sidx, starts, li, valid, aligned32);
        }
    }
}

// -------------------------------------------------------------------------------------
// Per tensor, fused in ONE cooperative launch: absmax over the whole tensor, a grid-wide
// barrier, then quantize.  Every CTA leaves its partial absmax in `partials[blockIdx.x]`
// (no atomics, nothing to clear), and after the barrier every CTA reduces those partials.
//
// The tensor is walked in rows of gridDim.x * 256 units; a thread owns one unit of every row.
// The first pass has four rows (256 bytes per thread) in flight.  What a thread read last it
// keeps for the second pass: the final four rows in registers, the `smem_rows` rows before
// them in shared memory (a thread-private spill area, laid out [row][16-byte chunk][thread],
// so the accesses are conflict free).  With 2 CTAs per SM and 5 x 16 KiB of shared memory
// each, 9 of the 14 rows of a 64 MiB tensor never leave the SM.  The other rows are read
// again newest first (the likeliest to be in the 126 MB L2), two rows ahead of the
// arithmetic.  Results are bit-identical to absmax_kernel + quantize_kernel.
// Must be launched cooperatively with a grid that is resident all at once.
// -------------------------------------------------------------------------------------
struct QuantTensorArgs {
    const void *in;
    void *out;
    void *out_scale;
    float *partials;     // gridDim.x floats of scratch
    long long nunits;
    int param;
    float lo, hi, range, inv_range;
    int force_exact;
    int aligned32;
    int smem_rows;       // rows kept in dynamic shared memory (16 KiB each)
};

// More shared memory than this leaves the L1 too small to track the loads in flight (7 rows: first pass 25 % slower).
constexpr int QK_TENSOR_SMEM_ROWS = 5;
constexpr int QK_TENSOR_ROW_BYTES = 256 * 64;

template <int FDT, int KIND, int UB, bool CLAMP>
__global__ void __launch_bounds__(256, 2) quantize_tensor_kernel(const QuantTensorArgs a)
{
    static_assert(UB == 64, "64-byte units");
    using UT = UnitT<FDT, KIND, UB>;
    constexpr int RAW = UT::RAW;
    constexpr int OW = UT::OW;
    extern __shared__ uint4 kept_rows[];
    const char *in = static_cast<const char *>(a.in);
    uint32_t *out = static_cast<uint32_t *>(a.out);
    const bool aligned32 = a.aligned32 != 0;
    const long long row_units = (long long)gridDim.x * 256;
    const long long first = (long long)blockIdx.x * 256 + threadIdx.x;
    const int nrows = (int)((a.nunits + row_units - 1) / row_units);   // >= 1; units of rows >= nrows are out of range
    // Rows are taken four at a time, counted so that the last four end the tensor: the first group starts at a
    // negative row when nrows is not a multiple of 4.
    const int reg_row = nrows - 4;                                              // rows reg_row .. reg_row + 3 stay in registers
    const int start_row = -((4 - (nrows & 3)) & 3);
    const int kept_row = reg_row > a.smem_rows ? reg_row - a.smem_rows : (reg_row > 0 ? 0 : reg_row);   // rows [kept_row, reg_row) stay in shared memory

    auto fetch = [&](uint32_t (&raw)[RAW], int row) {
        const long long idx = (long long)row * row_units + first;
        if (row >= 0 && idx < a.nunits) {
            load_unit<UB>(raw, in + idx * UB, aligned32);
        } else {
#pragma unroll
            for (int i = 0; i < RAW; ++i) raw[i] = 0u;
        }
    };

    // ---- pass 1: absmax ---------------------------------------------------------------------------
    float amax = 0.0f;
    uint32_t held[4][RAW];
    for (int row = start_row; row <= reg_row; row += 4) {
#pragma unroll
        for (int k = 0; k < 4; ++k) fetch(held[k], row + k);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            amax = fmaxf(amax, unit_absmax<FDT, RAW>(held[k]));
            if (row < reg_row && row + k >= kept_row) {
                uint4 *slot = kept_rows + (size_t)(row + k - kept_row) * (RAW / 4) * 256 + threadIdx.x;
#pragma unroll
                for (int j = 0; j < RAW / 4; ++j)
                    slot[j * 256] = make_uint4(held[k][4 * j], held[k][4 * j + 1], held[k][4 * j + 2], held[k][4 * j + 3]);
            }
        }
    }
    __shared__ float warp_max[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    if (lane == 0) warp_max[warp] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float v = warp_max[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) v = fmaxf(v, warp_max[i]);
        a.partials[blockIdx.x] = v;
    }
    __threadfence();
    cooperative_groups::this_grid().sync();

    // ---- every CTA reduces the partials --------------------------------------------------
    float v = 0.0f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) v = fmaxf(v, __ldcg(a.partials + i));
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    if (lane == 0) warp_max[warp] = v;   // no warp reads the first round's values after the grid barrier
    __syncthreads();
    v = warp_max[lane & 7];
#pragma unroll
    for (int m = 4; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    const float scale_f = round_to<FDT>(div_by_range(2.0f * v, a.range, a.inv_range));
    const float s_fs = (a.param == QK_F32) ? scale_f : round_to_dyn(a.param, scale_f);
    const float s = (a.param == QK_F32) ? scale_f : round_to<FDT>(s_fs);
    if (blockIdx.x == 0 && threadIdx.x == 0) store_dyn(a.out_scale, a.param, 0, s_fs);
    const bool fast = kind_allows_fast<FDT, KIND>() && !a.force_exact && scale_is_safe(s);

    auto emit = [&](const uint32_t (&raw)[RAW], int row) {
        const long long idx = (long long)row * row_units + first;
        uint32_t w[OW];
        if (fast) quantize_unit_fast<FDT, KIND, UB, CLAMP, true>(raw, s, a.lo, a.hi, w);
        else quantize_unit_exact<FDT, KIND, UB>(raw, s, a.lo, a.hi, w);
        if (row >= 0 && idx < a.nunits) store_words<OW>(out + idx * OW, w, aligned32);
    };

    // ---- pass 2: quantize, newest data first ------------------------------------------------------
    emit(held[3], reg_row + 3);
    emit(held[2], reg_row + 2);
    // the newest rows that were not kept come from L2 while the kept ones are worked on
    int next_row = kept_row - 1;
    fetch(held[2], next_row);
    fetch(held[3], next_row - 1);
    emit(held[1], reg_row + 1);
    emit(held[0], reg_row);
    for (int row = reg_row - 1; row >= kept_row; --row) {
        const uint4 *slot = kept_rows + (size_t)(row - kept_row) * (RAW / 4) * 256 + threadIdx.x;
#pragma unroll
        for (int j = 0; j < RAW / 4; ++j) {
            const uint4 q = slot[j * 256];
            held[0][4 * j] = q.x, held[0][4 * j + 1] = q.y, held[0][4 * j + 2] = q.z, held[0][4 * j + 3] = q.w;
        }
        emit(held[0], row);
    }
    while (next_row >= 0) {   // the two register pairs take turns
        int row = next_row;
        next_row -= 2;
        fetch(held[0], next_row);
        fetch(held[1], next_row - 1);
        emit(held[2], row);
        emit(held[3], row - 1);
        if (next_row < 0) break;
        row = next_row;
        next_row -= 2;
        fetch(held[2], next_row);
        fetch(held[3], next_row - 1);
        emit(held[0], row);
        emit(held[1], row - 1);
    }
}

// -------------------------------------------------------------------------------------
// Scales only (per block), for the two-call form: absmax over each block then the scale
// formula, written as F.  A thread reduces UB contiguous bytes (64 when blocks are made of whole
// 64-byte units, else 32 or 16) in registers; blocks are aligned runs of 2^lg lanes, finished with
// lg shuffle rounds (f32 blocks of 128 elements: 3 rounds on 64-byte units instead of 5 on
// 16-byte chunks).
// -------------------------------------------------------------------------------------
template <int FDT, int UB>
__global__ void __launch_bounds__(256) block_scales_kernel(const void *in_, void *scale_out, long long nunits,
                                                           int lg_units_per_block, float range, float inv_range,
                                                           int aligned32, const RowStride rs, const PassSplit split)
{
    using F = typename ElemOf<FDT>::type;
    constexpr int RAW = UB / 4;
    constexpr int UNR = (UB >= 64) ? 2 : 4;
    const char *in = static_cast<const char *>(in_);
    const int lg = lg_units_per_block;
    pdl_entry();
    auto pass = [&](const long long (&idx)[UNR], const bool full) {
        uint32_t raw[UNR][RAW];
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            if (full || idx[k] < nunits) {
                long long offset = idx[k] * UB;
                if (rs.enabled) {
                    const unsigned row = fastdiv((unsigned)idx[k], rs.units_per_row);
                    offset = (long long)row * rs.row_bytes + (long long)((unsigned)idx[k] - row * rs.units_per_row.div) * UB;
                }
                load_unit<UB>(raw[k], in + offset, aligned32 != 0);
            } else {
#pragma unroll
                for (int i = 0; i < RAW; ++i) raw[k][i] = 0u;
            }
        }
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            if (!full && idx[k] - (threadIdx.x & 31) >= nunits) continue;   // the whole row lies past the end
            float amax = unit_absmax<FDT, RAW>(raw[k]);
#pragma unroll
            for (int m = 1; m < 32; m <<= 1)
                if (m < (1 << lg)) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
            if ((full || idx[k] < nunits) && (idx[k] & ((1ll << lg) - 1)) == 0)
                static_cast<F *>(scale_out)[idx[k] >> lg] =
                    static_cast<F>(round_to<FDT>(div_by_range(2.0f * amax, range, inv_range)));
        }
    };
    QK_WALK_PASSES(split.full_passes, nunits, UNR, pass);
}

// -------------------------------------------------------------------------------------
// Scales of [block_rows, block_cols] tiles.  A tile is reduced by one warp (small tiles) or by a
// whole CTA (tiles of 1024 chunks = 16 KB and more), with four independent 128-bit loads in
// flight per thread along the rows of the tile.  Tiles at the bottom edge are clipped.
// -------------------------------------------------------------------------------------
template <int FDT>
__global__ void __launch_bounds__(256) block_scales_2d_kernel(const void *in_, void *scale_out, long long rows,
                                                              long long cols, int block_rows, int block_cols,
                                                              float range, float inv_range, int cta_per_tile)
{
    using F = typename ElemOf<FDT>::type;
    constexpr int PER = FInfo<FDT>::PER16;
    const char *in = static_cast<const char *>(in_);
    const int lane = threadIdx.x & 31;
    const int group = cta_per_tile ? 256 : 32;                       // threads that share a tile
    const int rank_in_group = cta_per_tile ? threadIdx.x : lane;
    const long long team = cta_per_tile ? blockIdx.x : (((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    const long long nteams = cta_per_tile ? gridDim.x : (((long long)gridDim.x * blockDim.x) >> 5);
    const long long ncb = cols / block_cols, nrb = (rows + block_rows - 1) / block_rows;
    const int chunks_per_row = block_cols / PER;
    __shared__ float warp_max[8];
    pdl_entry();
    for (long long t = team; t < nrb * ncb; t += nteams) {
        const long long rb = t / ncb, cb = t % ncb;
        const long long r0 = rb * block_rows;
        const int nr = (int)((rows - r0 < block_rows) ? rows - r0 : block_rows);
        const int nchunks = nr * chunks_per_row;
        float amax = 0.0f;
        for (int c0 = rank_in_group; c0 < nchunks; c0 += 4 * group) {
            uint32_t raw[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = c0 + group * j;
                if (c < nchunks) {
                    const int r = c / chunks_per_row, cc = c - r * chunks_per_row;
                    load_unit<16>(raw[j], in + ((r0 + r) * cols + cb * block_cols + (long long)cc * PER) * FInfo<FDT>::SIZE,
                                  false);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) raw[j][i] = 0u;
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) amax = fmaxf(amax, unit_absmax<FDT, 4>(raw[j]));
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        if (cta_per_tile) {
            __syncthreads();   // warp_max of the previous tile has been read
            if (lane == 0) warp_max[threadIdx.x >> 5] = amax;
            __syncthreads();
            if (threadIdx.x == 0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, warp_max[i]);
            }
        }
        if (rank_in_group == 0)
            static_cast<F *>(scale_out)[t] = static_cast<F>(round_to<FDT>(div_by_range(2.0f * amax, range, inv_range)));
    }
}

// Host-side launchers, one translation unit per float type.
// `sub`: blocks per unit, 1 or 2 (2: fused form of 16-bit types with 64-byte units and blocks of 32 bytes).
cudaError_t launch_quantize(int fdt, int kind, int unit_bytes, bool dyn, bool clamp, int sub, const QuantArgs &args,
                            const LaunchCfg &cfg, cudaStream_t stream);
// Transposed matrix views (transposed_kernels.cu): one tensor; blocks of 1, 2, 4 or 8 units (lg 0..3) or per tensor (lg -1).
cudaError_t launch_quantize_transposed(int fdt, int kind, int unit_bytes, bool dyn, bool clamp, const QuantArgs &args,
                                       const LaunchCfg &cfg, cudaStream_t stream);
// `lgb`: a block is 2^lgb units (0..3).
cudaError_t launch_scales_transposed(int fdt, int unit_bytes, int lgb, const void *in, void *scale_out, const Transposed &tr,
                                     long long ntiles, float range, float inv_range, const LaunchCfg &cfg, cudaStream_t stream);
// Device flag the staged kernels set when a bounded wait gives up (address of the current device).
int *stage_error_flag();
// `unit_bytes` in {16, 32, 64}; `lg` = log2(units per block), at most 5.
cudaError_t launch_block_scales(int fdt, const void *in, void *scale_out, long long nunits, int unit_bytes, int lg,
                                float range, float inv_range, const RowStride &rs, const LaunchCfg &cfg, cudaStream_t stream);
cudaError_t launch_block_scales_2d(int fdt, const void *in, void *scale_out, long long rows, long long cols,
                                   int block_rows, int block_cols, float range, float inv_range, const LaunchCfg &cfg,
                                   cudaStream_t stream);
// Cooperative per-tensor launch (64-byte units).  `partials_capacity` floats are available at
// args.partials; returns cudaErrorInvalidValue if the resident grid needs more.
cudaError_t launch_quantize_tensor(int fdt, int kind, QuantTensorArgs &args, int partials_capacity,
                                   const LaunchCfg &cfg, cudaStream_t stream);

}  // namespace qk
