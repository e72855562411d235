// Axis reductions MaxAbs, Max and Min: the instructions of `cubek_reduce::reduce`
// (crates/cubek-reduce/src/lib.rs:93-131; instructions/maxabs.rs, max.rs, min.rs) that the callers of the
// quantize path use for scales and ranges.  Every result is one of the inputs (or the instruction's null
// accumulator), so it is exact in the input type, which is also the accumulator type of these instructions in the
// reference (crates/cubek-reduce/src/instructions/mixed.rs:42-48), and independent of the order of evaluation;
// NaN elements do not take part.
//
// `ReduceStrategy { use_planes, shared }` (strategy.rs:7-16) chooses who reduces one output item: every unit by
// itself, a plane (warp), or all units of a cube (CTA) together.  The two memory layouts are the reference's
// line modes (config.rs:71-79): "parallel" - the reduced axis is the contiguous one - and "perpendicular" - the
// contiguous axis is kept and vectorised, the loop runs over the reduced axis.
//   parallel:       1, 32 or 256 threads walk one row with 128-bit loads, four in flight per thread;
//   perpendicular:  a thread owns a 16-byte column of `inner` and walks the reduced axis (coalesced across the
//                   warp); with `shared` the 8 warps of a CTA split the reduced axis and combine in shared memory;
//   any strides:    one thread per output item through the strides (same results, not tuned).
#include "common.cuh"
#include "misc_kernels.cuh"

namespace qk {

enum { INST_MAXABS = 0, INST_MAX = 1, INST_MIN = 2 };

template <int INST> __device__ __forceinline__ float red2(float a, float b)
{
    if constexpr (INST == INST_MAXABS) return fmaxf(a, fabsf(b));
    else if constexpr (INST == INST_MAX) return fmaxf(a, b);
    else return fminf(a, b);
}
template <int INST> __device__ __forceinline__ float merge2(float a, float b)   // two accumulators
{
    if constexpr (INST == INST_MIN) return fminf(a, b);
    else return fmaxf(a, b);
}
// Null accumulator: 0 for MaxAbs; the lowest / highest FINITE value of the type for Max / Min (`min_value()` /
// `max_value()`, max.rs:33-39, min.rs).
template <int FDT, int INST> __device__ __forceinline__ float null_acc()
{
    if constexpr (INST == INST_MAXABS) return 0.0f;
    constexpr float big = (FDT == QK_F32) ? 3.402823466e+38f : (FDT == QK_F16) ? 65504.0f : 3.3895313892515355e+38f;
    return INST == INST_MAX ? -big : big;
}

template <int FDT, int INST> __device__ __forceinline__ float reduce_chunk(float acc, const Vec16 &v)
{
    constexpr int PER = FInfo<FDT>::PER16;
    float x[PER];
    widen16<FDT>(v, x);
#pragma unroll
    for (int i = 0; i < PER; ++i) acc = red2<INST>(acc, x[i]);
    return acc;
}

// ---- parallel: rows of `len` contiguous elements, GROUP threads per row --------------------------------------
template <int FDT, int INST, int GROUP>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const void *in_, void *out, long long rows, long long len, int vector_ok)
{
    constexpr int PER = FInfo<FDT>::PER16;
    constexpr int ESZ = FInfo<FDT>::SIZE;
    const char *in = static_cast<const char *>(in_);
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long group = tid / GROUP, ngroups = ((long long)gridDim.x * blockDim.x) / GROUP;
    const int rank = (int)(tid % GROUP);
    __shared__ float warp_acc[8];
    pdl_entry();
    for (long long r = group; r < rows; r += ngroups) {
        float acc = null_acc<FDT, INST>();
        const long long base = r * len;
        if (vector_ok) {
            const long long nchunk = len / PER;
            long long c = rank;
            for (; c + 3 * GROUP < nchunk; c += 4 * GROUP) {
                Vec16 v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = ldg128_stream(in + (base + (c + (long long)j * GROUP) * PER) * ESZ);
#pragma unroll
                for (int j = 0; j < 4; ++j) acc = reduce_chunk<FDT, INST>(acc, v[j]);
            }
            for (; c < nchunk; c += GROUP) acc = reduce_chunk<FDT, INST>(acc, ldg128_stream(in + (base + c * PER) * ESZ));
        } else {
            for (long long i = rank; i < len; i += GROUP) acc = red2<INST>(acc, load_dyn(in_, FDT, base + i));
        }
        if constexpr (GROUP >= 32) {
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) acc = merge2<INST>(acc, __shfl_xor_sync(0xffffffffu, acc, m));
        }
        if constexpr (GROUP == 256) {
            __syncthreads();   // warp_acc of the previous row has been read
            if ((threadIdx.x & 31) == 0) warp_acc[threadIdx.x >> 5] = acc;
            __syncthreads();
            if (threadIdx.x == 0) {
#pragma unroll
                for (int i = 1; i < 8; ++i) acc = merge2<INST>(acc, warp_acc[i]);
            }
        }
        if (rank == 0) store_dyn(out, FDT, r, acc);
    }
}

// ---- perpendicular: [outer, len, inner] with `inner` contiguous; columns of one 16-byte vector -----------------
// SPLIT = false: a thread walks the whole reduced axis of its column.  SPLIT = true: a CTA takes 32 neighbouring
// columns, its 8 warps take every 8th step of the reduced axis, shared memory combines them.
template <int FDT, int INST, bool SPLIT>
__global__ void __launch_bounds__(256) reduce_columns_kernel(const void *in_, void *out_, long long outer, long long len,
                                                             long long inner_vecs)
{
    constexpr int PER = FInfo<FDT>::PER16;
    constexpr int ESZ = FInfo<FDT>::SIZE;
    const char *in = static_cast<const char *>(in_);
    char *out = static_cast<char *>(out_);
    const long long ncols = outer * inner_vecs;
    const long long row_bytes = inner_vecs * 16;          // one step along the reduced axis
    __shared__ float part[8][32][PER + 1];
    pdl_entry();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long first = SPLIT ? (long long)blockIdx.x * 32 + lane : (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long step = SPLIT ? (long long)gridDim.x * 32 : (long long)gridDim.x * blockDim.x;
    const long long cols_padded = SPLIT ? (ncols + 31) / 32 * 32 : ncols;
    for (long long col = first; col < cols_padded; col += step) {
        float acc[PER];
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] = null_acc<FDT, INST>();
        if (col < ncols) {
            const long long o = col / inner_vecs, v = col - o * inner_vecs;
            const char *p = in + (o * len * inner_vecs + v) * 16;
            const long long k0 = SPLIT ? warp : 0, dk = SPLIT ? 8 : 1;
            long long k = k0;
            for (; k + 3 * dk < len; k += 4 * dk) {
                Vec16 t[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) t[j] = ldg128_stream(p + (k + j * dk) * row_bytes);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float x[PER];
                    widen16<FDT>(t[j], x);
#pragma unroll
                    for (int i = 0; i < PER; ++i) acc[i] = red2<INST>(acc[i], x[i]);
                }
            }
            for (; k < len; k += dk) {
                float x[PER];
                widen16<FDT>(ldg128_stream(p + k * row_bytes), x);
#pragma unroll
                for (int i = 0; i < PER; ++i) acc[i] = red2<INST>(acc[i], x[i]);
            }
        }
        if constexpr (SPLIT) {
            __syncthreads();
#pragma unroll
            for (int i = 0; i < PER; ++i) part[warp][lane][i] = acc[i];
            __syncthreads();
            if (warp == 0) {
#pragma unroll
                for (int w = 1; w < 8; ++w)
#pragma unroll
                    for (int i = 0; i < PER; ++i) acc[i] = merge2<INST>(acc[i], part[w][lane][i]);
            }
        }
        if (col < ncols && (!SPLIT || warp == 0)) {
            Vec16 r;
            if constexpr (FDT == QK_F32) {
#pragma unroll
                for (int i = 0; i < 4; ++i) r.w[i] = __float_as_uint(acc[i]);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    r.w[i] = (FDT == QK_BF16) ? pack_bf16x2(acc[2 * i], acc[2 * i + 1]) : pack_f16x2(acc[2 * i], acc[2 * i + 1]);
            }
            *reinterpret_cast<Vec16 *>(out + col * 16) = r;
        }
    }
}

// ---- any strides: one thread per output item --------------------------------------------------------------------
struct ReduceStrided {
    int rank, axis;
    long long shape[QK_MAX_RANK];
    long long in_strides[QK_MAX_RANK];
    long long out_strides[QK_MAX_RANK];
};

template <int INST>
__global__ void __launch_bounds__(256) reduce_strided_kernel(const ReduceStrided g, const void *in, void *out, int fdt,
                                                             long long nout, float null_value)
{
    pdl_entry();
    for (long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x; o < nout; o += (long long)gridDim.x * blockDim.x) {
        long long rem = o, ioff = 0, ooff = 0;
        for (int d = g.rank - 1; d >= 0; --d) {
            if (d == g.axis) continue;
            const long long c = rem % g.shape[d];
            rem /= g.shape[d];
            ioff += c * g.in_strides[d];
            ooff += c * g.out_strides[d];
        }
        float acc = null_value;
        for (long long k = 0; k < g.shape[g.axis]; ++k) acc = red2<INST>(acc, load_dyn(in, fdt, ioff + k * g.in_strides[g.axis]));
        store_dyn(out, fdt, ooff, acc);
    }
}

namespace {

template <typename K> int resident(K kernel)
{
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, 256, 0) != cudaSuccess || n < 1) n = 1;
    return n;
}

template <int FDT, int INST>
cudaError_t launch_typed(const void *in, void *out, long long outer, long long len, long long inner, int units_per_item,
                         const LaunchCfg &cfg, cudaStream_t stream)
{
    constexpr int ESZ = FInfo<FDT>::SIZE, PER = FInfo<FDT>::PER16;
    const bool pdl = cfg.pdl != 0;
    const bool base16 = (reinterpret_cast<uintptr_t>(in) & 15u) == 0;
    if (inner == 1) {
        const int vector_ok = (len % PER == 0) && base16;
        // who reduces one row: a thread, a warp or a CTA; by default the smallest group that still keeps whole
        // 128-bit loads busy on every lane
        int group = units_per_item;
        if (group == 0) group = (len * ESZ >= 32768) ? 256 : (len * ESZ >= 512 ? 32 : 1);
        const long long threads_needed = outer * group;
        if (group == 256) {
            static const int occ = resident(reduce_rows_kernel<FDT, INST, 256>);
            long long grid = outer, cap = (long long)cfg.sm_count * occ;
            if (grid > cap) grid = cap;
            return launch_kernel(reduce_rows_kernel<FDT, INST, 256>, (int)(grid < 1 ? 1 : grid), 256, stream, pdl, in, out, outer, len, vector_ok);
        }
        long long grid = (threads_needed + 255) / 256;
        if (group == 32) {
            static const int occ = resident(reduce_rows_kernel<FDT, INST, 32>);
            const long long cap = (long long)cfg.sm_count * occ;
            if (grid > cap) grid = cap;
            return launch_kernel(reduce_rows_kernel<FDT, INST, 32>, (int)(grid < 1 ? 1 : grid), 256, stream, pdl, in, out, outer, len, vector_ok);
        }
        static const int occ = resident(reduce_rows_kernel<FDT, INST, 1>);
        const long long cap = (long long)cfg.sm_count * occ;
        if (grid > cap) grid = cap;
        return launch_kernel(reduce_rows_kernel<FDT, INST, 1>, (int)(grid < 1 ? 1 : grid), 256, stream, pdl, in, out, outer, len, vector_ok);
    }
    // perpendicular, vectorised over `inner`
    const long long inner_vecs = inner / PER;
    const long long ncols = outer * inner_vecs;
    bool split = units_per_item == 256;
    if (units_per_item == 0) split = ncols < (long long)cfg.sm_count * 1024 && len >= 64;   // too few columns to fill the GPU
    if (split) {
        static const int occ = resident(reduce_columns_kernel<FDT, INST, true>);
        long long grid = (ncols + 31) / 32, cap = (long long)cfg.sm_count * occ;
        if (grid > cap) grid = cap;
        return launch_kernel(reduce_columns_kernel<FDT, INST, true>, (int)(grid < 1 ? 1 : grid), 256, stream, pdl, in, out, outer, len, inner_vecs);
    }
    static const int occ = resident(reduce_columns_kernel<FDT, INST, false>);
    long long grid = (ncols + 255) / 256, cap = (long long)cfg.sm_count * occ * 4;
    if (grid > cap) grid = cap;
    return launch_kernel(reduce_columns_kernel<FDT, INST, false>, (int)(grid < 1 ? 1 : grid), 256, stream, pdl, in, out, outer, len, inner_vecs);
}

template <int INST>
cudaError_t launch_inst(int fdt, const void *in, void *out, long long outer, long long len, long long inner, int units_per_item,
                        const LaunchCfg &cfg, cudaStream_t stream)
{
    switch (fdt) {
    case QK_F32: return launch_typed<QK_F32, INST>(in, out, outer, len, inner, units_per_item, cfg, stream);
    case QK_F16: return launch_typed<QK_F16, INST>(in, out, outer, len, inner, units_per_item, cfg, stream);
    case QK_BF16: return launch_typed<QK_BF16, INST>(in, out, outer, len, inner, units_per_item, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

float null_value_of(int fdt, int inst)
{
    if (inst == INST_MAXABS) return 0.0f;
    const float big = (fdt == QK_F32) ? 3.402823466e+38f : (fdt == QK_F16) ? 65504.0f : 3.3895313892515355e+38f;
    return inst == INST_MAX ? -big : big;
}

}  // namespace

// Contiguous [outer, len, inner] view.  `units_per_item`: 1, 32 or 256 threads per output item, 0 = chosen here.
// The perpendicular layout needs `inner` to hold whole 16-byte vectors and 16-byte aligned bases; the caller falls
// back to the strided kernel otherwise.
cudaError_t launch_reduce_contiguous(int fdt, int inst, const void *in, void *out, long long outer, long long len,
                                     long long inner, int units_per_item, const LaunchCfg &cfg, cudaStream_t stream)
{
    switch (inst) {
    case INST_MAXABS: return launch_inst<INST_MAXABS>(fdt, in, out, outer, len, inner, units_per_item, cfg, stream);
    case INST_MAX: return launch_inst<INST_MAX>(fdt, in, out, outer, len, inner, units_per_item, cfg, stream);
    case INST_MIN: return launch_inst<INST_MIN>(fdt, in, out, outer, len, inner, units_per_item, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_reduce_strided(int fdt, int inst, const QkTensor *input, const QkTensor *output, int axis,
                                  const LaunchCfg &cfg, cudaStream_t stream)
{
    ReduceStrided g;
    g.rank = input->rank;
    g.axis = axis;
    long long nout = 1;
    for (int d = 0; d < QK_MAX_RANK; ++d) {
        g.shape[d] = d < input->rank ? input->shape[d] : 1;
        g.in_strides[d] = d < input->rank ? input->strides[d] : 0;
        g.out_strides[d] = d < input->rank ? output->strides[d] : 0;
        if (d < input->rank && d != axis) nout *= input->shape[d];
    }
    long long grid = (nout + 255) / 256;
    const long long cap = (long long)cfg.sm_count * 8;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    const bool pdl = cfg.pdl != 0;
    const float nv = null_value_of(fdt, inst);
    switch (inst) {
    case INST_MAXABS: return launch_kernel(reduce_strided_kernel<INST_MAXABS>, (int)grid, 256, stream, pdl, g, input->ptr, output->ptr, fdt, nout, nv);
    case INST_MAX: return launch_kernel(reduce_strided_kernel<INST_MAX>, (int)grid, 256, stream, pdl, g, input->ptr, output->ptr, fdt, nout, nv);
    case INST_MIN: return launch_kernel(reduce_strided_kernel<INST_MIN>, (int)grid, 256, stream, pdl, g, input->ptr, output->ptr, fdt, nout, nv);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace qk
