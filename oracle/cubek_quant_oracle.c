/*
 * CPU oracle for the cubek-quant symmetric quantize / dequantize path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of the
 * reference crate so that the CUDA kernels can be checked bit for bit.  It is never
 * linked into, loaded by or called from the shipped library; only the test-suite,
 * the smoke check and the benchmark's CPU-baseline leg use it.
 *
 * PARITY UNPINNED.  The reference (Rust + the CubeCL JIT, an un-vendored git
 * dependency pinned at rev e7515bb10bbc16f1fff6c32803938a1da95affed) cannot be
 * compiled or run where this oracle is built, and its own tests hold no bit-exact
 * vectors (only a round-trip tolerance, crates/cubek-quant/tests/suite/symmetric.rs:130-140
 * and :272-283).  The oracle is therefore pinned against (1) that tolerance contract on
 * the reference's 24 test cases, and (2) an independent NumPy/ml_dtypes restatement.
 * The choices the reference leaves to its JIT back end are fixed here as:
 *   - `Line::round` is round-half-to-even (nearbyintf in the default rounding mode); built with
 *     -DOQ_ROUND_HALF_AWAY (liboracle_half_away.so) it rounds halves away from zero instead, the one
 *     other lowering a back end could plausibly choose;
 *   - arithmetic on f16 / bf16 lines is the correctly rounded result in that type
 *     (computed as the f32 operation followed by one round-to-nearest-even narrowing;
 *     f32 carries >= 2p+2 bits for both types, so the double rounding is innocuous);
 *   - a NaN quotient (0/0, i.e. an all-zero block with scale 0) quantizes to code 0;
 *   - the fp4 cast is OCP e2m1, round-to-nearest-even, saturating at +-6, even element
 *     in the low nibble of each byte.
 *
 * Reference lines restated (paths relative to the reference checkout):
 *   quantize element     crates/cubek-quant/src/quantize.rs:19-31   (x / scale, round, clamp)
 *   pack into u32        crates/cubek-quant/src/quantize.rs:61-81
 *   scale write + cast   crates/cubek-quant/src/quantize.rs:83-98
 *   packed kernel        crates/cubek-quant/src/quantize.rs:128-171
 *   native kernel        crates/cubek-quant/src/quantize.rs:100-126
 *   unpack + sign-extend crates/cubek-quant/src/dequantize.rs:86-118
 *   dequantize element   crates/cubek-quant/src/dequantize.rs:22-25  (cast(scale) * q)
 *   packed kernel        crates/cubek-quant/src/dequantize.rs:121-148 (one scale per u32, :73)
 *   native kernel        crates/cubek-quant/src/dequantize.rs:151-167
 *   scale index          crates/cubek-quant/src/layout/scales.rs:144-160 (to_source_pos)
 *   block-start election crates/cubek-quant/src/layout/scales.rs:179-195
 *   block % nq assert    crates/cubek-quant/src/lib.rs:20-33
 *   absmax               crates/cubek-reduce/src/instructions/maxabs.rs:31-87
 *   scale formula        crates/cubek-quant/tests/suite/symmetric.rs:35-38, :175-178
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- enums shared (by value) with include/cubek_quant_b200.h ---------------------- */
enum { OQ_F32 = 0, OQ_F16 = 1, OQ_BF16 = 2 };
enum { OQ_Q8F = 0, OQ_Q8S, OQ_Q4F, OQ_Q4S, OQ_Q2F, OQ_Q2S, OQ_E4M3, OQ_E5M2, OQ_E2M1 };
enum { OQ_STORE_NATIVE = 0, OQ_STORE_U32 = 1 };
enum { OQ_LEVEL_TENSOR = 0, OQ_LEVEL_BLOCK = 1 };

enum {
    OQ_OK = 0,
    OQ_ERR_UNSUPPORTED = 1,
    OQ_ERR_BLOCK_SIZE = 2,
    OQ_ERR_SHAPE = 3,
};

#define OQ_MAX_RANK 8

/* ---- scalar type helpers ------------------------------------------------------------ */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* f32 -> bf16, round to nearest even; NaN stays NaN (quiet). */
static inline uint16_t f32_to_bf16(float f)
{
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float f16_to_f32(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
static inline uint16_t f32_to_f16(float f) { _Float16 v = (_Float16)f; uint16_t h; memcpy(&h, &v, 2); return h; }

static inline int dtype_size(int dt) { return dt == OQ_F32 ? 4 : 2; }

/* Load element i of a buffer of float type `dt`, widened (exactly) to f32. */
static inline float load_as_f32(const void *p, int dt, int64_t i)
{
    switch (dt) {
    case OQ_F32: return ((const float *)p)[i];
    case OQ_F16: return f16_to_f32(((const uint16_t *)p)[i]);
    default:     return bf16_to_f32(((const uint16_t *)p)[i]);
    }
}

/* Round an f32 value to float type `dt` (nearest even) and return it widened back to f32. */
static inline float round_to(int dt, float v)
{
    switch (dt) {
    case OQ_F32: return v;
    case OQ_F16: return f16_to_f32(f32_to_f16(v));
    default:     return bf16_to_f32(f32_to_bf16(v));
    }
}

static inline void store_from_f32(void *p, int dt, int64_t i, float v)
{
    switch (dt) {
    case OQ_F32: ((float *)p)[i] = v; break;
    case OQ_F16: ((uint16_t *)p)[i] = f32_to_f16(v); break;
    default:     ((uint16_t *)p)[i] = f32_to_bf16(v); break;
    }
}

/* ---- scheme constants (cubecl-common `QuantValue::range` / `size_bits`) -------------- */

int oq_value_bits(int value)
{
    switch (value) {
    case OQ_Q8F: case OQ_Q8S: case OQ_E4M3: case OQ_E5M2: return 8;
    case OQ_Q4F: case OQ_Q4S: case OQ_E2M1: return 4;
    case OQ_Q2F: case OQ_Q2S: return 2;
    default: return 0;
    }
}

int oq_value_range(int value, float *lo, float *hi)
{
    switch (value) {
    case OQ_Q8F: *lo = -128.f; *hi = 127.f; return 0;
    case OQ_Q8S: *lo = -127.f; *hi = 127.f; return 0;
    case OQ_Q4F: *lo = -8.f;   *hi = 7.f;   return 0;
    case OQ_Q4S: *lo = -7.f;   *hi = 7.f;   return 0;
    case OQ_Q2F: *lo = -2.f;   *hi = 1.f;   return 0;
    case OQ_Q2S: *lo = -1.f;   *hi = 1.f;   return 0;
    case OQ_E4M3: *lo = -448.f; *hi = 448.f; return 0;
    case OQ_E5M2: *lo = -57344.f; *hi = 57344.f; return 0;
    case OQ_E2M1: *lo = -6.f;  *hi = 6.f;   return 0;
    default: return -1;
    }
}

/* Quantized values held by one stored item: 32/bits for the u32 store, 2 for native fp4
 * (two codes per byte), 1 for the other native stores. */
int oq_num_quants(int value, int store)
{
    int bits = oq_value_bits(value);
    if (bits == 0) return 0;
    if (store == OQ_STORE_U32) return 32 / bits;
    return value == OQ_E2M1 ? 2 : 1;
}

/* ---- small float formats used by the native store ------------------------------------ */

/* OCP e2m1: magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6; bit 3 is the sign.  Round to nearest,
 * ties to the code with an even mantissa bit, saturate at 6.  NaN maps to +0. */
static inline uint8_t f32_to_e2m1(float v)
{
    uint8_t sign = (f32_bits(v) >> 31) ? 8u : 0u;
    float a = fabsf(v);
    uint8_t m;
    if (!(a == a)) return 0;
    if (a <= 0.25f) m = 0;            /* tie 0.25 -> 0   (even)  */
    else if (a < 0.75f) m = 1;        /* 0.5                     */
    else if (a <= 1.25f) m = 2;       /* ties 0.75, 1.25 -> 1    */
    else if (a < 1.75f) m = 3;        /* 1.5                     */
    else if (a <= 2.5f) m = 4;        /* ties 1.75, 2.5 -> 2     */
    else if (a < 3.5f) m = 5;         /* 3                       */
    else if (a <= 5.0f) m = 6;        /* ties 3.5, 5 -> 4        */
    else m = 7;                       /* 6 (saturating)          */
    return sign | m;
}

static inline float e2m1_to_f32(uint8_t code)
{
    static const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    float v = mag[code & 7u];
    return (code & 8u) ? -v : v;
}

/* Generic small binary float encode (exponent bits E, mantissa bits M, bias B), RNE, clamped
 * to +-max_finite.  Used for e4m3 (fn: no inf, max 448) and e5m2 (max 57344). */
static inline uint8_t f32_to_fp8(float v, int E, int M, int bias, float max_finite)
{
    uint8_t sign = (f32_bits(v) >> 31) ? 0x80u : 0u;
    float a = fabsf(v);
    if (!(a == a)) return (uint8_t)(sign | 0x7fu);
    if (a > max_finite) a = max_finite;
    if (a == 0.f) return sign;
    int e;
    (void)frexpf(a, &e);              /* a = f * 2^e, f in [0.5,1) -> exponent of leading bit = e-1 */
    int ue = e - 1;
    int min_e = 1 - bias;             /* smallest normal exponent */
    if (ue < min_e) ue = min_e;       /* subnormal: fixed quantum */
    float quantum = ldexpf(1.f, ue - M);
    float q = nearbyintf(a / quantum);  /* exact scaling by a power of two, RNE */
    float r = q * quantum;
    if (r > max_finite) r = max_finite;
    /* re-derive fields from the rounded value */
    (void)frexpf(r, &e);
    ue = e - 1;
    uint32_t expf, man;
    if (r == 0.f) return sign;
    if (ue < min_e) { expf = 0; man = (uint32_t)(r / ldexpf(1.f, min_e - M)); }
    else { expf = (uint32_t)(ue + bias); man = (uint32_t)(r / ldexpf(1.f, ue - M)) - (1u << M); }
    (void)E;
    return (uint8_t)(sign | (expf << M) | man);
}

static inline float fp8_to_f32(uint8_t code, int E, int M, int bias)
{
    uint32_t expf = (code >> M) & ((1u << E) - 1u);
    uint32_t man = code & ((1u << M) - 1u);
    float v;
    if (expf == 0) v = ldexpf((float)man, 1 - bias - M);
    else v = ldexpf((float)(man + (1u << M)), (int)expf - bias - M);
    return (code & 0x80u) ? -v : v;
}

/* ---- scale index: BlockScaledLayout::to_source_pos ----------------------------------- */

typedef struct {
    int rank;
    int64_t shape[OQ_MAX_RANK];          /* unpacked value shape */
    int64_t block[OQ_MAX_RANK];          /* block dims, left-padded with 1 (to_dim_vec) */
    int64_t scale_strides[OQ_MAX_RANK];  /* strides of the scales tensor, in elements */
    int per_tensor;
} oq_layout;

static int make_layout(oq_layout *L, const int64_t *shape, int rank, int level,
                       const uint8_t *block, int block_rank, const int64_t *scale_strides)
{
    if (rank < 1 || rank > OQ_MAX_RANK) return OQ_ERR_SHAPE;
    L->rank = rank;
    L->per_tensor = (level == OQ_LEVEL_TENSOR);
    for (int d = 0; d < rank; ++d) {
        L->shape[d] = shape[d];
        L->block[d] = 1;
        L->scale_strides[d] = scale_strides ? scale_strides[d] : 0;
    }
    if (!L->per_tensor) {
        if (block_rank < 1 || block_rank > rank) return OQ_ERR_BLOCK_SIZE;
        for (int i = 0; i < block_rank; ++i) {
            uint8_t b = block[i];
            if (b == 0) return OQ_ERR_BLOCK_SIZE;
            L->block[rank - block_rank + i] = b;
        }
    }
    return OQ_OK;
}

/* Walk the dims last to first, dividing the linear position by each extent; every
 * coordinate is divided by its block extent and weighted by the scales stride. */
static inline int64_t scale_pos(const oq_layout *L, int64_t pos, int *is_start)
{
    if (L->per_tensor) { if (is_start) *is_start = (pos == 0); return 0; }
    int64_t offs = pos, sp = 0;
    int start = 1;
    for (int d = L->rank - 1; d >= 0; --d) {
        int64_t coord = offs % L->shape[d];
        offs /= L->shape[d];
        sp += (coord / L->block[d]) * L->scale_strides[d];
        start &= (coord % L->block[d]) == 0;
    }
    if (is_start) *is_start = start;
    return sp;
}

static int64_t numel(const int64_t *shape, int rank)
{
    int64_t n = 1;
    for (int d = 0; d < rank; ++d) n *= shape[d];
    return n;
}

/* ---- element arithmetic -------------------------------------------------------------- */

/* clamp(round(x / s)) evaluated in float type `fdt`; returns the integral value as f32. */
static inline float quantize_value(float x, float s, int fdt, float lo, float hi)
{
    float t = round_to(fdt, x / s);
#ifdef OQ_ROUND_HALF_AWAY
    float r = roundf(t);        /* the other plausible lowering of `Line::round`: halves away from zero */
#else
    float r = nearbyintf(t);
#endif
    if (!(r == r)) return 0.f;
    r = r < lo ? lo : r;
    r = r > hi ? hi : r;
    return r;
}

/* ---- public entry points ------------------------------------------------------------- */

/*
 * Scales from data: absmax per tensor / per block, then scale = (2*absmax)/(hi-lo)
 * evaluated in f32 and narrowed to the input float type.  `scale_out` is typed `fdt`
 * and laid out through `scale_strides` (per tensor: one element).
 */
int oq_compute_scales(const void *input, int fdt, const int64_t *shape, int rank,
                      int value, int level, const uint8_t *block, int block_rank,
                      void *scale_out, const int64_t *scale_strides)
{
    float lo, hi;
    oq_layout L;
    int rc;
    if (oq_value_range(value, &lo, &hi)) return OQ_ERR_UNSUPPORTED;
    if ((rc = make_layout(&L, shape, rank, level, block, block_rank, scale_strides))) return rc;
    const int64_t n = numel(shape, rank);
    const float denom = hi - lo;

    if (L.per_tensor) {
        float amax = 0.f;
#pragma omp parallel for reduction(max : amax) schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            float a = fabsf(load_as_f32(input, fdt, i));
            if (a > amax) amax = a;
        }
        store_from_f32(scale_out, fdt, 0, (2.f * amax) / denom);
        return OQ_OK;
    }

    /* Per block: fast route when blocks run along the last dim only and rows split evenly
     * (the blocks are then consecutive runs of the linear index). */
    int last_only = 1;
    for (int d = 0; d < rank - 1; ++d) last_only &= (L.block[d] == 1);
    const int64_t B = L.block[rank - 1];
    if (last_only && shape[rank - 1] % B == 0) {
        const int64_t nb = n / B;
#pragma omp parallel for schedule(static)
        for (int64_t b = 0; b < nb; ++b) {
            float amax = 0.f;
            for (int64_t i = 0; i < B; ++i) {
                float a = fabsf(load_as_f32(input, fdt, b * B + i));
                if (a > amax) amax = a;
            }
            store_from_f32(scale_out, fdt, scale_pos(&L, b * B, 0), (2.f * amax) / denom);
        }
        return OQ_OK;
    }

    /* General N-d blocks: accumulate the absmax of every block in f32 scratch held in the
     * output itself is not possible for 16-bit outputs, so run block by block. */
    {
        int64_t nblk[OQ_MAX_RANK], total = 1;
        for (int d = 0; d < rank; ++d) { nblk[d] = (shape[d] + L.block[d] - 1) / L.block[d]; total *= nblk[d]; }
#pragma omp parallel for schedule(static)
        for (int64_t bi = 0; bi < total; ++bi) {
            int64_t bc[OQ_MAX_RANK], rem = bi, ext[OQ_MAX_RANK], cnt = 1;
            for (int d = rank - 1; d >= 0; --d) { bc[d] = rem % nblk[d]; rem /= nblk[d]; }
            for (int d = 0; d < rank; ++d) {
                int64_t startc = bc[d] * L.block[d];
                ext[d] = shape[d] - startc < L.block[d] ? shape[d] - startc : L.block[d];
                cnt *= ext[d];
            }
            float amax = 0.f;
            int64_t sp = 0;
            for (int d = 0; d < rank; ++d) sp += bc[d] * L.scale_strides[d];
            for (int64_t k = 0; k < cnt; ++k) {
                int64_t r = k, lin = 0, mul = 1;
                int64_t coord[OQ_MAX_RANK];
                for (int d = rank - 1; d >= 0; --d) { coord[d] = bc[d] * L.block[d] + r % ext[d]; r /= ext[d]; }
                for (int d = rank - 1; d >= 0; --d) { lin += coord[d] * mul; mul *= shape[d]; }
                float a = fabsf(load_as_f32(input, fdt, lin));
                if (a > amax) amax = a;
            }
            store_from_f32(scale_out, fdt, sp, (2.f * amax) / denom);
        }
    }
    return OQ_OK;
}

/*
 * quantize::launch_ref.  `shape` is the unpacked (input) shape; `scale` is typed `fdt`
 * (the input float type), `out_scale` is typed `param` (the scheme's param type).
 * Output: u32 words (store U32), i8 / fp8 bytes, or fp4 pairs in bytes (store Native).
 */
int oq_quantize(const void *input, int fdt, const int64_t *shape, int rank,
                const void *scale, const int64_t *scale_strides,
                int value, int store, int param, int level,
                const uint8_t *block, int block_rank,
                void *output, void *out_scale)
{
    float lo, hi;
    oq_layout L;
    int rc;
    if (oq_value_range(value, &lo, &hi)) return OQ_ERR_UNSUPPORTED;
    const int bits = oq_value_bits(value);
    const int nq = oq_num_quants(value, store);
    if (store == OQ_STORE_NATIVE &&
        !(value == OQ_Q8F || value == OQ_Q8S || value == OQ_E4M3 || value == OQ_E5M2 || value == OQ_E2M1))
        return OQ_ERR_UNSUPPORTED;                       /* quantize.rs:213-219 */
    if ((rc = make_layout(&L, shape, rank, level, block, block_rank, scale_strides))) return rc;
    if (!L.per_tensor && (L.block[rank - 1] % nq) != 0) return OQ_ERR_BLOCK_SIZE;   /* lib.rs:20-33 */
    if (shape[rank - 1] % nq != 0) return OQ_ERR_SHAPE;
    const int64_t n = numel(shape, rank);
    const int64_t items = n / nq;
    const uint32_t mask = (bits == 32) ? 0xffffffffu : ((1u << bits) - 1u);

#pragma omp parallel for schedule(static)
    for (int64_t w = 0; w < items; ++w) {
        const int64_t pos = w * nq;
        int is_start;
        const int64_t sp = scale_pos(&L, pos, &is_start);
        /* write_scale: cast the F-typed scale to the param type; that value is stored and,
         * cast back to F, is the divisor. */
        const float s_fs = round_to(param, load_as_f32(scale, fdt, sp));
        if (is_start) store_from_f32(out_scale, param, sp, s_fs);
        const float s = round_to(fdt, s_fs);

        if (store == OQ_STORE_U32) {
            uint32_t word = 0;
            for (int i = 0; i < nq; ++i) {
                float c = quantize_value(load_as_f32(input, fdt, pos + i), s, fdt, lo, hi);
                word |= ((uint32_t)(int32_t)c & mask) << (i * bits);
            }
            ((uint32_t *)output)[w] = word;
        } else if (value == OQ_E2M1) {
            float c0 = quantize_value(load_as_f32(input, fdt, pos), s, fdt, lo, hi);
            float c1 = quantize_value(load_as_f32(input, fdt, pos + 1), s, fdt, lo, hi);
            ((uint8_t *)output)[w] = (uint8_t)(f32_to_e2m1(c0) | (f32_to_e2m1(c1) << 4));
        } else {
            float c = quantize_value(load_as_f32(input, fdt, pos), s, fdt, lo, hi);
            if (value == OQ_E4M3) ((uint8_t *)output)[w] = f32_to_fp8(c, 4, 3, 7, 448.f);
            else if (value == OQ_E5M2) ((uint8_t *)output)[w] = f32_to_fp8(c, 5, 2, 15, 57344.f);
            else ((int8_t *)output)[w] = (int8_t)(int32_t)c;
        }
    }
    return OQ_OK;
}

/*
 * dequantize::launch_ref.  `shape` is the unpacked (output) shape; `values` holds
 * numel/nq stored items; `params` is typed `param`; output is typed `odt`.
 */
int oq_dequantize(const void *values, const int64_t *shape, int rank,
                  const void *params, const int64_t *scale_strides,
                  int value, int store, int param, int level,
                  const uint8_t *block, int block_rank,
                  int odt, void *output)
{
    float lo, hi;
    oq_layout L;
    int rc;
    if (oq_value_range(value, &lo, &hi)) return OQ_ERR_UNSUPPORTED;
    const int bits = oq_value_bits(value);
    const int nq = oq_num_quants(value, store);
    if (store == OQ_STORE_NATIVE &&
        !(value == OQ_Q8F || value == OQ_Q8S || value == OQ_E4M3 || value == OQ_E5M2 || value == OQ_E2M1))
        return OQ_ERR_UNSUPPORTED;                       /* dequantize.rs:218-226 */
    if ((rc = make_layout(&L, shape, rank, level, block, block_rank, scale_strides))) return rc;
    if (shape[rank - 1] % nq != 0) return OQ_ERR_SHAPE;
    const int64_t n = numel(shape, rank);
    const int64_t items = n / nq;
    const uint32_t mask = (1u << bits) - 1u;
    const int32_t sign_bit = 1 << (bits - 1), two_pow_n = 1 << bits;

#pragma omp parallel for schedule(static)
    for (int64_t w = 0; w < items; ++w) {
        const int64_t pos = w * nq;
        const float s = round_to(odt, load_as_f32(params, param, scale_pos(&L, pos, 0)));
        if (store == OQ_STORE_U32) {
            const uint32_t word = ((const uint32_t *)values)[w];
            for (int i = 0; i < nq; ++i) {
                int32_t raw = (int32_t)((word >> (i * bits)) & mask);
                int32_t q = raw - (raw >= sign_bit ? two_pow_n : 0);
                store_from_f32(output, odt, pos + i, s * round_to(odt, (float)q));
            }
        } else if (value == OQ_E2M1) {
            const uint8_t b = ((const uint8_t *)values)[w];
            store_from_f32(output, odt, pos, s * e2m1_to_f32(b & 0xf));
            store_from_f32(output, odt, pos + 1, s * e2m1_to_f32(b >> 4));
        } else {
            float q;
            if (value == OQ_E4M3) q = fp8_to_f32(((const uint8_t *)values)[w], 4, 3, 7);
            else if (value == OQ_E5M2) q = fp8_to_f32(((const uint8_t *)values)[w], 5, 2, 15);
            else q = (float)((const int8_t *)values)[w];
            store_from_f32(output, odt, pos, s * round_to(odt, q));
        }
    }
    return OQ_OK;
}

int oq_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oq_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* Single-value probes used by the tests to pin the small-format tables. */
uint8_t oq_f32_to_e2m1(float v) { return f32_to_e2m1(v); }
float oq_e2m1_to_f32(uint8_t c) { return e2m1_to_f32(c); }
uint8_t oq_f32_to_e4m3(float v) { return f32_to_fp8(v, 4, 3, 7, 448.f); }
uint8_t oq_f32_to_e5m2(float v) { return f32_to_fp8(v, 5, 2, 15, 57344.f); }
float oq_e4m3_to_f32(uint8_t c) { return fp8_to_f32(c, 4, 3, 7); }
float oq_e5m2_to_f32(uint8_t c) { return fp8_to_f32(c, 5, 2, 15); }
uint16_t oq_f32_to_bf16(float v) { return f32_to_bf16(v); }
uint16_t oq_f32_to_f16(float v) { return f32_to_f16(v); }
