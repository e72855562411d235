// max |x| along one axis: the `MaxAbs` instruction of `cubek_reduce::reduce`
// (crates/cubek-reduce/src/lib.rs:93-131, instructions/maxabs.rs:31-87), which callers of the
// quantize path use to obtain absmax before the scale formula.  The result is one of the inputs'
// magnitudes, so it is exact in the input type (the reference accumulates in the input type,
// crates/cubek-reduce/src/precision.rs).  NaNs are ignored.
//
// Two layouts, like the reference's "parallel" and "perpendicular" line modes (config.rs:71-79):
//   * reduce along the last (contiguous) axis: one warp per row, 128-bit loads, shuffle reduction;
//   * reduce along another axis: one thread per output element, consecutive threads on consecutive
//     addresses, a loop over the reduced axis.
#include "common.cuh"
#include "quantize_kernels.cuh"

namespace qk {

template <int FDT>
__global__ void __launch_bounds__(256) maxabs_last_axis_kernel(const void *in_, void *out, long long rows, long long len,
                                                               int vector_ok)
{
    constexpr int PER = FInfo<FDT>::PER16;
    const char *in = static_cast<const char *>(in_);
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    pdl_entry();
    for (long long r = warp; r < rows; r += nwarps) {
        float amax = 0.0f;
        const long long base = r * len;
        if (vector_ok) {
            const long long nchunk = len / PER;
            for (long long c = lane; c < nchunk; c += 32) {
                uint32_t raw[4];
                load_unit<16>(raw, in + (base + c * PER) * FInfo<FDT>::SIZE, false);
                amax = fmaxf(amax, unit_absmax<FDT, 4>(raw));
            }
        } else {
            for (long long i = lane; i < len; i += 32) amax = fmaxf(amax, fabsf(load_dyn(in_, FDT, base + i)));
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        if (lane == 0) store_dyn(out, FDT, r, amax);
    }
}

__global__ void __launch_bounds__(256) maxabs_inner_axis_kernel(const void *in, void *out, int fdt, long long outer,
                                                                long long len, long long inner)
{
    const long long total = outer * inner;
    pdl_entry();
    for (long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x; o < total;
         o += (long long)gridDim.x * blockDim.x) {
        const long long oi = o / inner, ii = o % inner;
        const long long base = oi * len * inner + ii;
        float amax = 0.0f;
        for (long long k = 0; k < len; ++k) amax = fmaxf(amax, fabsf(load_dyn(in, fdt, base + k * inner)));
        store_dyn(out, fdt, o, amax);
    }
}

cudaError_t launch_maxabs(int fdt, const void *in, void *out, long long outer, long long len, long long inner,
                          const LaunchCfg &cfg, cudaStream_t stream)
{
    const bool pdl = cfg.pdl != 0;
    // one wave of resident CTAs (these kernels hold 6 CTAs of 256 threads per SM)
    auto resident = [](auto kernel) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, 256, 0) != cudaSuccess || n < 1) n = 1;
        return n;
    };
    static const int occ_last[3] = {resident(maxabs_last_axis_kernel<QK_F32>), resident(maxabs_last_axis_kernel<QK_F16>),
                                    resident(maxabs_last_axis_kernel<QK_BF16>)};
    static const int occ_inner = resident(maxabs_inner_axis_kernel);
    const int per_sm = (inner == 1) ? occ_last[fdt == QK_F32 ? 0 : fdt == QK_F16 ? 1 : 2] : occ_inner;
    const long long cap = (long long)cfg.sm_count * (cfg.ctas_per_sm > 0 ? cfg.ctas_per_sm : per_sm);
    if (inner == 1) {
        const int esz = (fdt == QK_F32) ? 4 : 2;
        const int per = 16 / esz;
        const int vector_ok = (len % per == 0) && ((reinterpret_cast<uintptr_t>(in) & 15u) == 0);
        long long grid = (outer + 7) / 8;   // 8 warps per CTA
        if (grid > cap) grid = cap;
        if (grid < 1) grid = 1;
        switch (fdt) {
        case QK_F32: return launch_kernel(maxabs_last_axis_kernel<QK_F32>, (int)grid, 256, stream, pdl, in, out, outer, len, vector_ok);
        case QK_F16: return launch_kernel(maxabs_last_axis_kernel<QK_F16>, (int)grid, 256, stream, pdl, in, out, outer, len, vector_ok);
        default: return launch_kernel(maxabs_last_axis_kernel<QK_BF16>, (int)grid, 256, stream, pdl, in, out, outer, len, vector_ok);
        }
    }
    long long grid = (outer * inner + 255) / 256;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    return launch_kernel(maxabs_inner_axis_kernel, (int)grid, 256, stream, pdl, in, out, fdt, outer, len, inner);
}

}  // namespace qk
