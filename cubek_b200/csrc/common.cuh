// Shared device helpers for the sm_100a quantize / dequantize kernels.
//
// Numeric contract (restating crates/cubek-quant/src/quantize.rs:19-31 and
// dequantize.rs:22-25 of the reference): every operation on a line of float type F is
// the correctly rounded result in F.  For f16 / bf16 that is the f32 operation followed
// by one round-to-nearest-even narrowing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cubek_quant_b200.h"

namespace qk {

// Stored-code kinds the kernels are specialised on.  Q8F/Q8S (and so on) share a kind and
// differ only in the clamp bounds passed at launch.
enum Kind : int {
    KIND_PACK8 = 0,  // 4 x 8-bit two's-complement codes per u32
    KIND_PACK4 = 1,  // 8 x 4-bit codes per u32
    KIND_PACK2 = 2,  // 16 x 2-bit codes per u32
    KIND_I8 = 3,     // native i8
    KIND_E2M1 = 4,   // native fp4, two codes per byte (even element in the low nibble)
    KIND_E4M3 = 5,   // native fp8 e4m3
    KIND_E5M2 = 6,   // native fp8 e5m2
    KIND_COUNT = 7
};

template <int FDT> struct ElemOf;
template <> struct ElemOf<QK_F32> { using type = float; };
template <> struct ElemOf<QK_F16> { using type = __half; };
template <> struct ElemOf<QK_BF16> { using type = __nv_bfloat16; };

template <int FDT> struct FInfo {
    static constexpr int SIZE = (FDT == QK_F32) ? 4 : 2;
    static constexpr int PER16 = 16 / SIZE;  // elements in one 128-bit access
};

// Elements that fill one 32-bit word of output for a kind.
__host__ __device__ constexpr int kind_elems_per_u32(int kind)
{
    return (kind == KIND_PACK4 || kind == KIND_E2M1) ? 8 : (kind == KIND_PACK2) ? 16 : 4;
}
__host__ __device__ constexpr int kind_bits(int kind)
{
    return (kind == KIND_PACK4 || kind == KIND_E2M1) ? 4 : (kind == KIND_PACK2) ? 2 : 8;
}
__host__ __device__ constexpr int cmax(int a, int b) { return a > b ? a : b; }

// ---- raw memory access ----------------------------------------------------------------

struct alignas(16) Vec16 { uint32_t w[4]; };
struct alignas(32) Vec32 { uint32_t w[8]; };

// Streaming 128-bit load: read-only path, do not keep the line in L1.
__device__ __forceinline__ Vec16 ldg128_stream(const void *p)
{
    Vec16 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3])
                 : "l"(p));
    return r;
}

// Streaming 256-bit load (sm_100 and later).  The address must be 32-byte aligned.
__device__ __forceinline__ Vec32 ldg256_stream(const void *p)
{
    Vec32 r;
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]),
                   "=r"(r.w[5]), "=r"(r.w[6]), "=r"(r.w[7])
                 : "l"(p));
    return r;
}

__device__ __forceinline__ void stg32_stream(void *p, uint32_t v)
{
    asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void stg64_stream(void *p, uint32_t a, uint32_t b)
{
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void stg128_stream(void *p, const Vec16 &v)
{
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]),
                 "r"(v.w[2]), "r"(v.w[3])
                 : "memory");
}
// 256-bit store (sm_100 and later); 32-byte aligned address.
__device__ __forceinline__ void stg256_stream(void *p, const Vec32 &v)
{
    asm volatile("st.global.cs.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.w[0]),
                 "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]), "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]),
                 "r"(v.w[7])
                 : "memory");
}

// ---- float type conversions -------------------------------------------------------------

__device__ __forceinline__ float bf16_lo_to_f32(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi_to_f32(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

// Two f32 -> packed bf16x2 / f16x2, round to nearest even; `lo` lands in bits 0..15.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Round an f32 to type FDT and widen it back.
template <int FDT> __device__ __forceinline__ float round_to(float v)
{
    if constexpr (FDT == QK_F32) return v;
    else if constexpr (FDT == QK_F16) return __half2float(__float2half_rn(v));
    else return __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float round_to_dyn(int dt, float v)
{
    if (dt == QK_F32) return v;
    if (dt == QK_F16) return __half2float(__float2half_rn(v));
    return __bfloat162float(__float2bfloat16_rn(v));
}

// Element i of a buffer of float type `dt`, widened to f32.
__device__ __forceinline__ float load_dyn(const void *p, int dt, int64_t i)
{
    if (dt == QK_F32) return reinterpret_cast<const float *>(p)[i];
    if (dt == QK_F16) return __half2float(reinterpret_cast<const __half *>(p)[i]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
}
__device__ __forceinline__ void store_dyn(void *p, int dt, int64_t i, float v)
{
    if (dt == QK_F32) reinterpret_cast<float *>(p)[i] = v;
    else if (dt == QK_F16) reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
}

// Widen the 16 bytes of `v` (PER16 elements of type FDT) to f32.
template <int FDT> __device__ __forceinline__ void widen16(const Vec16 &v, float *out)
{
    if constexpr (FDT == QK_F32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = __uint_as_float(v.w[i]);
    } else if constexpr (FDT == QK_BF16) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = bf16_lo_to_f32(v.w[i]);
            out[2 * i + 1] = bf16_hi_to_f32(v.w[i]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&v.w[i]));
            out[2 * i] = f.x;
            out[2 * i + 1] = f.y;
        }
    }
}

// Maximum of three f32 in one instruction (sm_100); a NaN operand is ignored, like fmaxf.
__device__ __forceinline__ float fmax3(float a, float b, float c)
{
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// ---- scale arithmetic -----------------------------------------------------------------

// `Line::round` of the reference (crates/cubek-quant/src/quantize.rs:27) is lowered by its external JIT back end.
// The default here is round-half-to-even; a build with -DQK_ROUND_HALF_AWAY rounds halves away from zero instead
// (every unit then takes the reference-arithmetic route: the shortcut arithmetic is built on half-to-even).
#ifdef QK_ROUND_HALF_AWAY
#define QK_ROUND(t) roundf(t)
#else
#define QK_ROUND(t) rintf(t)
#endif

// clamp(round(t)); a NaN quotient (0/0) gives code 0.
__device__ __forceinline__ float round_clamp(float t, float lo, float hi)
{
    float r = QK_ROUND(t);
    r = fminf(fmaxf(r, lo), hi);
    return (t != t) ? 0.0f : r;
}

// Reference arithmetic, one element, no shortcuts: RN_F(x / s), round, clamp.
template <int FDT> __device__ __forceinline__ float quantize_exact(float x, float s, float lo, float hi)
{
    return round_clamp(round_to<FDT>(__fdiv_rn(x, s)), lo, hi);
}

// ---- fp4 / fp8 conversions (Blackwell cvt instructions) -----------------------------------

// Two f32 -> one byte of e2m1 codes, round to nearest even, saturating; `lo` -> low nibble.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi)
{
    uint16_t r;
    asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}"
        : "=h"(r)
        : "f"(hi), "f"(lo));
    return r;
}
// One byte of e2m1 codes -> f16x2 (low nibble -> low half).  Exact.
__device__ __forceinline__ uint32_t cvt_f16x2_from_e2m1x2(uint32_t byte)
{
    uint32_t r;
    uint16_t b = (uint16_t)byte;
    asm("{\n\t.reg .b8 t;\n\tcvt.u8.u16 t, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, t;\n\t}" : "=r"(r) : "h"(b));
    return r;
}
// Two f32 -> two fp8 codes in the low 16 bits; `lo` -> low byte.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi)
{
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t cvt_e5m2x2(float lo, float hi)
{
    uint16_t r;
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
// f16x2 -> two fp8 codes in the low 16 bits (low half -> low byte), round to nearest even, saturating.
__device__ __forceinline__ uint32_t cvt_e4m3x2_from_f16x2(uint32_t p)
{
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(r) : "r"(p));
    return r;
}
__device__ __forceinline__ uint32_t cvt_e5m2x2_from_f16x2(uint32_t p)
{
    uint16_t r;
    asm("cvt.rn.satfinite.e5m2x2.f16x2 %0, %1;" : "=h"(r) : "r"(p));
    return r;
}
// Both halves of an f16x2 rounded to integers (ties to even); the sign of a zero result is kept.
__device__ __forceinline__ uint32_t f16x2_rint(uint32_t p)
{
    uint32_t r;
    asm("{\n\t.reg .f16 l, h;\n\tmov.b32 {l, h}, %1;\n\tcvt.rni.f16.f16 l, l;\n\tcvt.rni.f16.f16 h, h;\n\tmov.b32 %0, {l, h};\n\t}"
        : "=r"(r)
        : "r"(p));
    return r;
}
__device__ __forceinline__ uint32_t cvt_f16x2_from_e4m3x2(uint32_t two_bytes)
{
    uint32_t r;
    uint16_t b = (uint16_t)two_bytes;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(b));
    return r;
}
__device__ __forceinline__ uint32_t cvt_f16x2_from_e5m2x2(uint32_t two_bytes)
{
    uint32_t r;
    uint16_t b = (uint16_t)two_bytes;
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(r) : "h"(b));
    return r;
}

// ---- programmatic dependent launch ----------------------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may become resident
// while the previous kernel of the stream is still draining; it must not touch global memory
// before `griddepcontrol.wait`, which returns once the previous grid has completed and its
// writes are visible.  Signalling `launch_dependents` first lets the *next* kernel do the same
// with respect to this one.  Both instructions are no-ops for a normal launch.  For back-to-back
// launches of 20-30 us kernels this hides the 3-5 us between the end of one grid and the first
// instruction of the next.
__device__ __forceinline__ void pdl_entry()
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}


template <typename... KArgs, typename... Args>
static inline cudaError_t launch_kernel(void (*kernel)(KArgs...), int grid, int threads, cudaStream_t stream, bool pdl,
                                        Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- 2-D blocks ---------------------------------------------------------------------------------
// Division of a 31-bit unsigned number by a run-time constant with one multiply-high.
struct FastDiv {
    unsigned mul, shift, div;
};
static inline FastDiv make_fastdiv(unsigned d)
{
    FastDiv f;
    f.div = d;
    unsigned s = 0;
    while ((1ull << s) < d) ++s;
    f.shift = s;
    f.mul = (unsigned)((((1ull << s) - d) << 32) / d + 1);
    return f;
}
__device__ __forceinline__ unsigned fastdiv(unsigned n, const FastDiv &f)
{
    return (unsigned)(((unsigned long long)__umulhi(n, f.mul) + n) >> f.shift);
}

// Scale geometry of a matrix quantized in [block_rows, block_cols] tiles (the layout quantized
// matmul inputs use, crates/cubek-matmul/src/components/global/memory/layout.rs:213-262): units are
// runs along a row; unit `u` lies in row u / units_per_row and block column (u % units_per_row) >> lg.
struct Blocks2D {
    int enabled;
    FastDiv units_per_row;
    FastDiv block_rows;
    unsigned scales_per_row;
    int lg_units_per_block_col;
};
// Scale index of unit `u`, and whether the unit is the first of its tile.
__device__ __forceinline__ unsigned blocks2d_scale_index(const Blocks2D &b, unsigned u, bool *is_start)
{
    const unsigned row = fastdiv(u, b.units_per_row);
    const unsigned cu = u - row * b.units_per_row.div;
    const unsigned rb = fastdiv(row, b.block_rows);
    *is_start = (row - rb * b.block_rows.div == 0) && ((cu & ((1u << b.lg_units_per_block_col) - 1u)) == 0);
    return rb * b.scales_per_row + (cu >> b.lg_units_per_block_col);
}

// A float tensor whose rows are contiguous but `row_bytes` apart (a column slice of a wider matrix, padded
// rows): unit u lies in row u / units_per_row.  One tensor per launch.
struct RowStride {
    int enabled;
    FastDiv units_per_row;
    long long row_bytes;
};

// A transposed matrix view: logical [rows, cols], element (r, c) at c * ld + r (elements).  Work items are
// numbered with r fastest; `units_per_row` units make one logical row.  One tensor per launch.
struct Transposed {
    int enabled;
    int pairs;      // 16-bit types: a lane takes two adjacent rows
    FastDiv rows;   // dequantize: rows (or row pairs) per column unit; quantize: row tiles
    unsigned nrows; // logical rows
    long long ld;
    unsigned units_per_row;
};

// ---- work split ---------------------------------------------------------------------------------
// The persistent streaming kernels (one wave of CTAs, many passes each) walk their units in passes of
// gridDim.x * 256 * UNR consecutive units: CTA b takes the b-th run of 256 * UNR units of a pass, so that at any
// moment the grid reads one contiguous window of memory.  The passes that are full for EVERY CTA run in a loop
// without bounds checks; what is left (less than one pass) is dealt out in rows of 32 units, one row per warp and
// round, over all warps of the grid.
struct PassSplit {
    long long full_passes;   // passes in which every thread of the grid has UNR valid units
};
static inline PassSplit make_pass_split(long long nunits, long long grid, int threads, int unr)
{
    PassSplit s;
    s.full_passes = nunits / (grid * threads * unr);
    return s;
}
// Calls `pass(idx, true)` once per full pass with this thread's UNR unit indices, then `pass(idx, false)` once with
// its units of the remainder (units past `nunits` included) unless its whole row of the first round of the
// remainder lies past the end.  The two call sites give two inlined copies of the body: with the literal `true`
// the one in the loop keeps no bounds checks at all.
#define QK_WALK_PASSES(FULL_PASSES, NUNITS, UNR, PASS)                                                              \
    do {                                                                                                            \
        const long long qk_per_cta = (long long)blockDim.x * (UNR);                                                 \
        const long long qk_per_pass = qk_per_cta * gridDim.x;                                                       \
        long long qk_base = (long long)blockIdx.x * qk_per_cta + threadIdx.x;                                       \
        for (long long qk_p = 0; qk_p < (FULL_PASSES); ++qk_p, qk_base += qk_per_pass) {                            \
            long long qk_idx[UNR];                                                                                  \
            _Pragma("unroll") for (int qk_k = 0; qk_k < (UNR); ++qk_k) qk_idx[qk_k] = qk_base + qk_k * blockDim.x;  \
            PASS(qk_idx, true);                                                                                     \
        }                                                                                                           \
        const long long qk_rest = (FULL_PASSES) * qk_per_pass + (long long)blockIdx.x * blockDim.x + threadIdx.x;   \
        if (qk_rest - (threadIdx.x & 31) < (NUNITS)) {                                                              \
            long long qk_idx[UNR];                                                                                  \
            _Pragma("unroll") for (int qk_k = 0; qk_k < (UNR); ++qk_k)                                              \
                qk_idx[qk_k] = qk_rest + (long long)qk_k * gridDim.x * blockDim.x;                                  \
            PASS(qk_idx, false);                                                                                    \
        }                                                                                                           \
    } while (0)

// The same walk through ONE call site (`full` is then a run-time value and the body keeps its bounds checks, but
// exists once).  Measured per kernel: the per-tensor quantize of 16-bit inputs from absmax cells ran 7 % faster
// this way in batched launches (fewer exposed load stalls), every other quantize kernel 3-7 % slower.
#define QK_WALK_PASSES_ONE_SITE(FULL_PASSES, NUNITS, UNR, PASS)                                                      \
    do {                                                                                                            \
        const long long qk_per_cta = (long long)blockDim.x * (UNR);                                                 \
        const long long qk_per_pass = qk_per_cta * gridDim.x;                                                       \
        const long long qk_rest = (FULL_PASSES) * qk_per_pass + (long long)blockIdx.x * blockDim.x + threadIdx.x;   \
        for (long long qk_p = 0; qk_p <= (FULL_PASSES); ++qk_p) {                                                   \
            const bool qk_full = qk_p < (FULL_PASSES);                                                              \
            if (!qk_full && qk_rest - (threadIdx.x & 31) >= (NUNITS)) break;                                        \
            long long qk_idx[UNR];                                                                                  \
            _Pragma("unroll") for (int qk_k = 0; qk_k < (UNR); ++qk_k)                                              \
                qk_idx[qk_k] = qk_full ? qk_p * qk_per_pass + blockIdx.x * qk_per_cta + qk_k * blockDim.x + threadIdx.x \
                                       : qk_rest + (long long)qk_k * gridDim.x * blockDim.x;                        \
            PASS(qk_idx, qk_full);                                                                                  \
        }                                                                                                           \
    } while (0)

// ---- launch bookkeeping -----------------------------------------------------------------

struct LaunchCfg {
    int threads;      // threads per CTA
    int ctas_per_sm;  // grid cap = SM count * ctas_per_sm; 0 = resident CTAs per SM * waves
    int quant_waves;  // grid cap of the quantize kernels, in waves of resident CTAs
    int dequant_waves;
    int sm_count;
    int force_exact;  // 1: every unit takes the reference-arithmetic route
    int pdl;          // 1: launch with programmatic stream serialization
    int staged;       // 1: quantize reads its input through the shared-memory bulk-copy pipeline
    int stages;       // ring depth of that pipeline (2..4 tiles of 16 KB per CTA)
    int tensor_smem_rows;  // rows the one-launch per-tensor kernel keeps in shared memory; < 0 = as many as fit
};

}  // namespace qk
