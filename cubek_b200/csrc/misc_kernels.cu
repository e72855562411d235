// Per-tensor absmax (grid-wide reduction) and the layout-general fallback kernels.
//
// absmax: stands in for `cubek_reduce::reduce::<_, MaxAbs>` used by callers of the
// reference (crates/cubek-reduce/src/instructions/maxabs.rs:31-87).  The reference's shared
// strategy gives ONE cube to each output element (crates/cubek-reduce/src/config.rs:192-206),
// i.e. a whole-tensor absmax runs on one SM; here every SM streams its
// slice, reduces with warp shuffles and a shared-memory step, and merges with one atomicMax
// on the bit pattern of the (non-negative) float, which orders like an unsigned integer.
//
// general kernels: any rank <= 8, N-d blocks, strided scales, sizes that do not fill whole
// units.  They restate BlockScaledLayout::to_source_pos / is_block_start
// (crates/cubek-quant/src/layout/scales.rs:144-195) per stored item, as the reference does.
#include "misc_kernels.cuh"
#include "quantize_kernels.cuh"   // unit_absmax

namespace qk {

// CTAs of 256 threads of `kernel` that one SM holds at a time.
template <typename Kernel> static int resident_ctas(Kernel kernel)
{
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, 256, 0) != cudaSuccess || n < 1) n = 1;
    return n;
}

// ---------------------------------------------------------------------------------------
// absmax
// ---------------------------------------------------------------------------------------
template <int FDT>
__global__ void __launch_bounds__(256) absmax_kernel(const void *in_, long long n, unsigned int *cell, const RowStride rs,
                                                     const PassSplit split)
{
    constexpr int PER = FInfo<FDT>::PER16;
    constexpr int UNR = 4;
    const char *in = static_cast<const char *>(in_);
    const long long nchunks = n / PER;
    float amax = 0.0f;
    pdl_entry();

    auto pass = [&](const long long (&idx)[UNR], const bool full) {
        Vec16 raw[UNR];
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            long long offset = idx[k] * 16;
            if (rs.enabled) {   // rows of whole 16-byte chunks, `row_bytes` apart
                const unsigned row = fastdiv((unsigned)idx[k], rs.units_per_row);
                offset = (long long)row * rs.row_bytes + (long long)((unsigned)idx[k] - row * rs.units_per_row.div) * 16;
            }
            raw[k] = (full || idx[k] < nchunks) ? ldg128_stream(in + offset) : Vec16{{0u, 0u, 0u, 0u}};
        }
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            float x[PER];
            widen16<FDT>(raw[k], x);
#pragma unroll
            for (int i = 0; i < PER; i += 2) amax = fmax3(amax, fabsf(x[i]), fabsf(x[i + 1]));
        }
    };
    QK_WALK_PASSES(split.full_passes, nchunks, UNR, pass);
    // ragged tail (fewer than PER elements)
    if (blockIdx.x == 0 && threadIdx.x == 0)
        for (long long i = nchunks * PER; i < n; ++i) amax = fmaxf(amax, fabsf(load_dyn(in_, FDT, i)));

#pragma unroll
    for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    __shared__ float warp_max[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) warp_max[warp] = amax;
    __syncthreads();
    if (warp == 0) {
        float v = (lane < (int)(blockDim.x >> 5)) ? warp_max[lane] : 0.0f;
#pragma unroll
        for (int m = 4; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
        if (lane == 0) atomicMax(cell, __float_as_uint(v));
    }
}

// One launch for a batch of tensors.  Chunks are numbered across the batch and walked in grid-wide passes like
// every other streaming kernel (the grid reads one contiguous window of memory at any moment; contiguous spans
// per CTA read 5 % slower).  A thread keeps the running absmax of the tensor it is in and walks the table of
// tensors forward; when a warp crosses into the next tensor it flushes into the CTA's cells in shared memory
// (shards of a few MB are smaller than a pass, so that happens in every pass: with one global atomic per warp
// and flush, 9472 warps hammering a handful of cells made the kernel 2.3 x slower on 8-way shards), and the CTA
// hands its cells to the global ones once, at the end.
template <int FDT>
__global__ void __launch_bounds__(256) absmax_batch_kernel(const AbsmaxBatchArgs a, const PassSplit split)
{
    constexpr int UNR = 4;
    __shared__ unsigned int cta_cells[QK_ABSMAX_BATCH];
    for (int i = threadIdx.x; i < a.ntensors; i += blockDim.x) cta_cells[i] = 0u;
    __syncthreads();
    const long long total = a.chunk_end[a.ntensors - 1];
    pdl_entry();
    int ti = 0, cur = -1;
    float amax = 0.0f;
    long long ti_begin = 0, ti_end = a.chunk_end[0];
    const char *ti_in = static_cast<const char *>(a.in[0]);

    auto flush = [&](int next) {
        // the warp enters another tensor: lanes still in the old one contribute through a warp reduction when
        // they all agree, else one by one
        const int c0 = __shfl_sync(0xffffffffu, cur, 0);
        if (__all_sync(0xffffffffu, cur == c0)) {
            float m = amax;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
            if ((threadIdx.x & 31) == 0 && c0 >= 0 && m > 0.0f) atomicMax(cta_cells + c0, __float_as_uint(m));
        } else if (cur >= 0 && amax > 0.0f) {
            atomicMax(cta_cells + cur, __float_as_uint(amax));
        }
        cur = next;
        amax = 0.0f;
    };
    auto pass = [&](const long long (&idx)[UNR], const bool full) {
        Vec16 raw[UNR];
        int tk[UNR];
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            if (full || idx[k] < total) {
                while (idx[k] >= ti_end) {   // forward only: a thread's chunk indices grow
                    ++ti;
                    ti_begin = ti_end;
                    ti_end = a.chunk_end[ti];
                    ti_in = static_cast<const char *>(a.in[ti]);
                }
                raw[k] = ldg128_stream(ti_in + (idx[k] - ti_begin) * 16);
                tk[k] = ti;
            } else {
                raw[k] = Vec16{{0u, 0u, 0u, 0u}};
                tk[k] = -1;   // nothing to add, nothing to flush
            }
        }
#pragma unroll
        for (int k = 0; k < UNR; ++k) {
            if (__any_sync(0xffffffffu, tk[k] >= 0 && tk[k] != cur)) flush(tk[k] >= 0 ? tk[k] : cur);
            amax = fmaxf(amax, unit_absmax<FDT, 4>(raw[k].w));
        }
    };
    QK_WALK_PASSES(split.full_passes, total, UNR, pass);
    __syncwarp();
    flush(-1);
    __syncthreads();
    for (int i = threadIdx.x; i < a.ntensors; i += blockDim.x) {
        const unsigned int v = cta_cells[i];
        if (v != 0u) atomicMax(a.cells + i, v);
    }
}

cudaError_t launch_absmax_batch(int fdt, const AbsmaxBatchArgs &args, const LaunchCfg &cfg, cudaStream_t stream)
{
    if (args.ntensors < 1) return cudaSuccess;
    const long long total = args.chunk_end[args.ntensors - 1];
    if (total == 0) return cudaSuccess;
    // One wave of resident CTAs: a partial second wave would take as long as a full one.
    static const int occ[3] = {resident_ctas(absmax_batch_kernel<QK_F32>), resident_ctas(absmax_batch_kernel<QK_F16>),
                               resident_ctas(absmax_batch_kernel<QK_BF16>)};
    long long need = (total + 1023) / 1024;
    const long long cap = (long long)cfg.sm_count * (cfg.ctas_per_sm > 0 ? cfg.ctas_per_sm : occ[fdt == QK_F32 ? 0 : fdt == QK_F16 ? 1 : 2]);
    if (need > cap) need = cap;
    const bool pdl = cfg.pdl != 0;
    const PassSplit split = make_pass_split(total, need, 256, 4);
    switch (fdt) {
    case QK_F32: return launch_kernel(absmax_batch_kernel<QK_F32>, (int)need, 256, stream, pdl, args, split);
    case QK_F16: return launch_kernel(absmax_batch_kernel<QK_F16>, (int)need, 256, stream, pdl, args, split);
    default: return launch_kernel(absmax_batch_kernel<QK_BF16>, (int)need, 256, stream, pdl, args, split);
    }
}

// Scalar route for inputs whose base is not 16-byte aligned.
__global__ void __launch_bounds__(256) absmax_scalar_kernel(const void *in, int fdt, long long n, unsigned int *cell)
{
    float amax = 0.0f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        amax = fmaxf(amax, fabsf(load_dyn(in, fdt, i)));
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    if ((threadIdx.x & 31) == 0) atomicMax(cell, __float_as_uint(amax));
}

__device__ __forceinline__ long long data_index(const GeneralLayout &L, long long pos);

__global__ void __launch_bounds__(256) absmax_strided_kernel(const GeneralLayout L, const void *in, int fdt, long long n,
                                                             unsigned int *cell)
{
    float amax = 0.0f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        amax = fmaxf(amax, fabsf(load_dyn(in, fdt, data_index(L, i))));
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    if ((threadIdx.x & 31) == 0) atomicMax(cell, __float_as_uint(amax));
}

__global__ void finalize_scale_kernel(const unsigned int *cell, void *scale_out, int fdt, float range)
{
    const float amax = __uint_as_float(*cell);
    const float s = __fdiv_rn(2.0f * amax, range);
    store_dyn(scale_out, fdt, 0, s);
}

// `cfg` with the grid cap set to one wave of resident CTAs of `kernel` (unless a tuning key fixed it).
template <typename Kernel> static LaunchCfg one_wave(const LaunchCfg &cfg, Kernel kernel)
{
    LaunchCfg c = cfg;
    if (c.ctas_per_sm <= 0) c.ctas_per_sm = resident_ctas(kernel);
    return c;
}

static int grid_for(long long work_items, int per_cta, const LaunchCfg &cfg)
{
    long long need = (work_items + per_cta - 1) / per_cta;
    long long cap = (long long)cfg.sm_count * (cfg.ctas_per_sm > 0 ? cfg.ctas_per_sm : 8);
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

cudaError_t launch_absmax(int fdt, const void *in, long long n, unsigned int *cell, const LaunchCfg &cfg,
                          cudaStream_t stream, bool zero_first, const RowStride *row_stride)
{
    RowStride rs;
    rs.enabled = 0;
    rs.units_per_row = make_fastdiv(1u);
    rs.row_bytes = 0;
    if (row_stride) rs = *row_stride;
    if (zero_first) {
        cudaError_t e = cudaMemsetAsync(cell, 0, sizeof(unsigned int), stream);
        if (e != cudaSuccess) return e;
    }
    if (n == 0) return cudaSuccess;
    const int threads = 256;
    if ((reinterpret_cast<uintptr_t>(in) & 15u) != 0 && !rs.enabled) {
        absmax_scalar_kernel<<<grid_for(n, threads * 8, one_wave(cfg, absmax_scalar_kernel)), threads, 0, stream>>>(in, fdt, n, cell);
        return cudaGetLastError();
    }
    const int per = (fdt == QK_F32) ? 4 : 8;
    // One wave of resident CTAs (the f32 instance holds 6 per SM, the 16-bit ones 8): with a fixed 8 per SM the
    // f32 kernel ran a third of a second wave and took 110 us instead of 78 us on 470 MB.
    static const int occ[3] = {resident_ctas(absmax_kernel<QK_F32>), resident_ctas(absmax_kernel<QK_F16>),
                               resident_ctas(absmax_kernel<QK_BF16>)};
    LaunchCfg wave = cfg;
    if (wave.ctas_per_sm <= 0) wave.ctas_per_sm = occ[fdt == QK_F32 ? 0 : fdt == QK_F16 ? 1 : 2];
    const int grid = grid_for(n / per + 1, threads * 4, wave);
    const bool pdl = cfg.pdl != 0;
    const PassSplit split = make_pass_split(n / per, grid, threads, 4);
    switch (fdt) {
    case QK_F32: return launch_kernel(absmax_kernel<QK_F32>, grid, threads, stream, pdl, in, n, cell, rs, split);
    case QK_F16: return launch_kernel(absmax_kernel<QK_F16>, grid, threads, stream, pdl, in, n, cell, rs, split);
    default: return launch_kernel(absmax_kernel<QK_BF16>, grid, threads, stream, pdl, in, n, cell, rs, split);
    }
}

cudaError_t launch_absmax_strided(const GeneralLayout &layout, const void *in, int fdt, long long n, unsigned int *cell,
                                  const LaunchCfg &cfg, cudaStream_t stream)
{
    cudaError_t e = cudaMemsetAsync(cell, 0, sizeof(unsigned int), stream);
    if (e != cudaSuccess || n == 0) return e;
    absmax_strided_kernel<<<grid_for(n, 256 * 8, one_wave(cfg, absmax_strided_kernel)), 256, 0, stream>>>(layout, in, fdt, n, cell);
    return cudaGetLastError();
}

cudaError_t launch_finalize_scale(const unsigned int *cell, void *scale_out, int fdt, float range,
                                  cudaStream_t stream)
{
    finalize_scale_kernel<<<1, 1, 0, stream>>>(cell, scale_out, fdt, range);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// layout-general kernels
// ---------------------------------------------------------------------------------------

// Scale index of linear element `pos` and whether `pos` starts a block.
__device__ __forceinline__ long long general_scale_pos(const GeneralLayout &L, long long pos, bool *is_start,
                                                       long long *out_pos = nullptr)
{
    if (L.per_tensor) {
        *is_start = (pos == 0);
        if (out_pos) *out_pos = 0;
        return 0;
    }
    if (L.fits31) {
        unsigned offs = (unsigned)pos;
        long long sp = 0, sp_out = 0;
        bool start = true;
        for (int d = L.rank - 1; d >= 0; --d) {
            const unsigned q = fastdiv(offs, L.shape_div[d]);
            const unsigned coord = offs - q * L.shape_div[d].div;
            offs = q;
            const unsigned b = fastdiv(coord, L.block_div[d]);
            sp += (long long)b * L.scale_strides[d];
            sp_out += (long long)b * L.out_scale_strides[d];
            start = start && (coord - b * L.block_div[d].div == 0);
        }
        *is_start = start;
        if (out_pos) *out_pos = sp_out;
        return sp;
    }
    long long offs = pos, sp = 0, sp_out = 0;
    bool start = true;
    for (int d = L.rank - 1; d >= 0; --d) {
        const long long coord = offs % L.shape[d];
        offs /= L.shape[d];
        sp += (coord / L.block[d]) * L.scale_strides[d];
        sp_out += (coord / L.block[d]) * L.out_scale_strides[d];
        start = start && (coord % L.block[d] == 0);
    }
    *is_start = start;
    if (out_pos) *out_pos = sp_out;
    return sp;
}

// Offset (elements) of linear element `pos` of the float tensor.
__device__ __forceinline__ long long data_index(const GeneralLayout &L, long long pos)
{
    if (L.data_contiguous) return pos;
    if (L.fits31) {
        unsigned offs = (unsigned)pos;
        long long idx = 0;
        for (int d = L.rank - 1; d >= 0; --d) {
            const unsigned q = fastdiv(offs, L.shape_div[d]);
            idx += (long long)(offs - q * L.shape_div[d].div) * L.data_strides[d];
            offs = q;
        }
        return idx;
    }
    long long offs = pos, idx = 0;
    for (int d = L.rank - 1; d >= 0; --d) {
        idx += (offs % L.shape[d]) * L.data_strides[d];
        offs /= L.shape[d];
    }
    return idx;
}

// Offset (stored items) of item `item` of the quantized tensor (linear index over the packed shape).
__device__ __forceinline__ long long values_index(const GeneralLayout &L, long long item)
{
    if (L.values_contiguous) return item;
    const int last = L.rank - 1;
    if (L.fits31) {
        unsigned offs = (unsigned)item;
        unsigned q = fastdiv(offs, L.packed_last_div);
        long long idx = (long long)(offs - q * L.packed_last_div.div) * L.values_strides[last];
        offs = q;
        for (int d = last - 1; d >= 0; --d) {
            q = fastdiv(offs, L.shape_div[d]);
            idx += (long long)(offs - q * L.shape_div[d].div) * L.values_strides[d];
            offs = q;
        }
        return idx;
    }
    long long offs = item;
    const long long plast = (long long)L.packed_last_div.div;
    long long idx = (offs % plast) * L.values_strides[last];
    offs /= plast;
    for (int d = last - 1; d >= 0; --d) {
        idx += (offs % L.shape[d]) * L.values_strides[d];
        offs /= L.shape[d];
    }
    return idx;
}

// Native element encode of an integral, clamped value.
__device__ __forceinline__ uint32_t encode_native(int kind, float c)
{
    if (kind == KIND_I8) return (uint32_t)(int)c & 0xFFu;
    if (kind == KIND_E4M3) return cvt_e4m3x2(c, 0.0f) & 0xFFu;
    return cvt_e5m2x2(c, 0.0f) & 0xFFu;
}

// One element: RN_F(x / s), round, clamp.  With a scale inside the window of the shortcuts the quotient comes from
// the reciprocal like in the streaming kernels (f32: two correction steps, exactly rounded, first guess clamped so
// that a huge quotient keeps its sign; 16-bit types: the f32 product narrowed to F), else from IEEE division.
template <int FDT> __device__ __forceinline__ float general_quantize_one(float x, float s, float r, bool fast, float lo, float hi)
{
    if (!fast) return quantize_exact<FDT>(x, s, lo, hi);
    float t;
    if constexpr (FDT == QK_F32) {
        const float q0 = fminf(fmaxf(x * r, lo - 2.0f), hi + 2.0f);
        t = __fmaf_rn(__fmaf_rn(-s, q0, x), r, q0);
    } else {
        t = round_to<FDT>(x * r);
    }
    return round_clamp(t, lo, hi);
}

template <int FDT> __global__ void __launch_bounds__(256) general_quantize_kernel(const GeneralQuantArgs a)
{
    using F = typename ElemOf<FDT>::type;
    const int bits = kind_bits(a.kind);
    const uint32_t mask = (1u << bits) - 1u;
    const F *in = static_cast<const F *>(a.in);
    for (long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x; item < a.nitems;
         item += (long long)gridDim.x * blockDim.x) {
        const long long pos = item * a.nq;
        bool is_start;
        long long sp_out;
        const long long sp = general_scale_pos(a.layout, pos, &is_start, &sp_out);
        float scale_f;
        if (a.absmax) scale_f = round_to<FDT>(__fdiv_rn(2.0f * (*a.absmax), a.range));
        else scale_f = static_cast<float>(static_cast<const F *>(a.scale_in)[sp]);
        const float s_fs = round_to_dyn(a.param, scale_f);
        if (is_start) store_dyn(a.out_scale, a.param, sp_out, s_fs);
        const float s = round_to<FDT>(s_fs);
#ifdef QK_ROUND_HALF_AWAY
        const bool fast = false;   // the shortcuts were proven for halves-to-even only
#else
        const bool fast = !a.force_exact && scale_is_safe(s);
#endif
        const float r = fast ? __frcp_rn(s) : 0.0f;

        // the nq elements of an item are consecutive along the last dim
        const long long d0 = data_index(a.layout, pos);
        const long long dstep = a.layout.data_contiguous ? 1 : a.layout.data_strides[a.layout.rank - 1];
        if (a.kind <= KIND_PACK2) {
            uint32_t word = 0;
            if (a.vector_bytes == 16) {
                // contiguous, 16-byte aligned data: the item's elements arrive 16 bytes at a time
                constexpr int PER = 16 / (int)sizeof(F);
                const uint4 *p = reinterpret_cast<const uint4 *>(in + d0);
                for (int c0 = 0; c0 < a.nq; c0 += PER) {
                    const uint4 v = __ldg(p + c0 / PER);
                    const uint32_t raw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < PER; ++j) {
                        const float c = general_quantize_one<FDT>(raw_elem<FDT>(raw, j), s, r, fast, a.lo, a.hi);
                        word |= ((uint32_t)(int)c & mask) << ((c0 + j) * bits);
                    }
                }
            } else if (a.vector_bytes == 8) {   // four 16-bit elements
                const uint2 v = __ldg(reinterpret_cast<const uint2 *>(in + d0));
                const uint32_t raw[2] = {v.x, v.y};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float c = general_quantize_one<FDT>(raw_elem<FDT>(raw, j), s, r, fast, a.lo, a.hi);
                    word |= ((uint32_t)(int)c & mask) << (j * bits);
                }
            } else {
                for (int i = 0; i < a.nq; ++i) {
                    const float c = general_quantize_one<FDT>(static_cast<float>(in[d0 + i * dstep]), s, r, fast, a.lo, a.hi);
                    word |= ((uint32_t)(int)c & mask) << (i * bits);
                }
            }
            static_cast<uint32_t *>(a.out)[values_index(a.layout, item)] = word;
        } else if (a.kind == KIND_E2M1) {
            const float c0 = general_quantize_one<FDT>(static_cast<float>(in[d0]), s, r, fast, a.lo, a.hi);
            const float c1 = general_quantize_one<FDT>(static_cast<float>(in[d0 + dstep]), s, r, fast, a.lo, a.hi);
            static_cast<uint8_t *>(a.out)[values_index(a.layout, item)] = (uint8_t)cvt_e2m1x2(c0, c1);
        } else {
            const float c = general_quantize_one<FDT>(static_cast<float>(in[d0]), s, r, fast, a.lo, a.hi);
            static_cast<uint8_t *>(a.out)[values_index(a.layout, item)] = (uint8_t)encode_native(a.kind, c);
        }
    }
}

template <int FDT> __global__ void __launch_bounds__(256) general_dequantize_kernel(const GeneralDequantArgs a)
{
    using F = typename ElemOf<FDT>::type;
    const int bits = kind_bits(a.kind);
    const uint32_t mask = (1u << bits) - 1u;
    const int sign_bit = 1 << (bits - 1), two_pow_n = 1 << bits;
    F *out = static_cast<F *>(a.out);
    for (long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x; item < a.nitems;
         item += (long long)gridDim.x * blockDim.x) {
        const long long pos = item * a.nq;
        bool is_start;
        const long long sp = general_scale_pos(a.layout, pos, &is_start);
        const float s = round_to<FDT>(load_dyn(a.params, a.param, sp));
        const long long d0 = data_index(a.layout, pos);
        const long long dstep = a.layout.data_contiguous ? 1 : a.layout.data_strides[a.layout.rank - 1];
        if (a.kind <= KIND_PACK2) {
            const uint32_t word = static_cast<const uint32_t *>(a.values)[values_index(a.layout, item)];
            auto value = [&](int i) {
                const int raw = (int)((word >> (i * bits)) & mask);
                return s * (float)(raw - (raw >= sign_bit ? two_pow_n : 0));
            };
            if (a.vector_bytes == 16) {
                // contiguous, 16-byte aligned output: the item's elements leave 16 bytes at a time
                constexpr int PER = 16 / (int)sizeof(F);
                uint4 *p = reinterpret_cast<uint4 *>(out + d0);
                for (int c0 = 0; c0 < a.nq; c0 += PER) {
                    uint32_t r[4];
                    if constexpr (FDT == QK_F32) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) r[j] = __float_as_uint(value(c0 + j));
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) r[j] = h2_pack<FDT>(value(c0 + 2 * j), value(c0 + 2 * j + 1));
                    }
                    p[c0 / PER] = make_uint4(r[0], r[1], r[2], r[3]);
                }
            } else if (a.vector_bytes == 8) {   // four 16-bit elements
                if constexpr (FDT != QK_F32)
                    *reinterpret_cast<uint2 *>(out + d0) = make_uint2(h2_pack<FDT>(value(0), value(1)), h2_pack<FDT>(value(2), value(3)));
            } else {
                for (int i = 0; i < a.nq; ++i) out[d0 + i * dstep] = static_cast<F>(value(i));
            }
        } else if (a.kind == KIND_E2M1) {
            uint32_t h2 = cvt_f16x2_from_e2m1x2(static_cast<const uint8_t *>(a.values)[values_index(a.layout, item)]);
            float2 f = __half22float2(*reinterpret_cast<__half2 *>(&h2));
            out[d0] = static_cast<F>(s * f.x);
            out[d0 + dstep] = static_cast<F>(s * f.y);
        } else {
            const uint32_t b = static_cast<const uint8_t *>(a.values)[values_index(a.layout, item)];
            float q;
            if (a.kind == KIND_I8) q = (float)(int)(int8_t)b;
            else {
                uint32_t h2 = (a.kind == KIND_E4M3) ? cvt_f16x2_from_e4m3x2(b) : cvt_f16x2_from_e5m2x2(b);
                q = __half22float2(*reinterpret_cast<__half2 *>(&h2)).x;
            }
            out[d0] = static_cast<F>(s * q);
        }
    }
}

// One thread per block of the scales tensor: absmax over the (possibly clipped) N-d block.  The block is
// walked row by row (runs along the last dim) with an odometer over the other dims, so the element loop
// has no division.
template <int FDT> __global__ void __launch_bounds__(256) general_scales_kernel(const GeneralScalesArgs a)
{
    using F = typename ElemOf<FDT>::type;
    constexpr int PER = 16 / (int)sizeof(F);
    const F *in = static_cast<const F *>(a.in);
    const bool aligned_base = reinterpret_cast<uintptr_t>(a.in) % 16 == 0;
    const GeneralLayout &L = a.layout;
    const int last = L.rank - 1;
    for (long long bi = (long long)blockIdx.x * blockDim.x + threadIdx.x; bi < a.nblocks;
         bi += (long long)gridDim.x * blockDim.x) {
        int ext[QK_MAX_RANK], at[QK_MAX_RANK];
        long long rem = bi, sp = 0, lin = 0, mul = 1, rows = 1;
        long long stride[QK_MAX_RANK];
        for (int d = L.rank - 1; d >= 0; --d) {
            const long long nb = (L.shape[d] + L.block[d] - 1) / L.block[d];
            const long long bc = rem % nb;
            rem /= nb;
            const long long start = bc * L.block[d];
            ext[d] = (int)((L.shape[d] - start < L.block[d]) ? L.shape[d] - start : L.block[d]);
            stride[d] = L.data_contiguous ? mul : L.data_strides[d];
            mul *= L.shape[d];
            lin += start * stride[d];
            sp += bc * L.scale_strides[d];
            at[d] = 0;
            if (d != last) rows *= ext[d];
        }
        float amax = 0.0f;
        for (long long r = 0; r < rows; ++r) {
            if (aligned_base && stride[last] == 1 && ext[last] % PER == 0 && lin % PER == 0) {
                // a run of whole, aligned 16-byte chunks
                const uint4 *p = reinterpret_cast<const uint4 *>(in + lin);
                for (int k = 0; k < ext[last] / PER; ++k) {
                    const uint4 v = __ldg(p + k);
                    const uint32_t raw[4] = {v.x, v.y, v.z, v.w};
                    amax = fmaxf(amax, unit_absmax<FDT, 4>(raw));
                }
            } else {
                for (int k = 0; k < ext[last]; ++k) amax = fmaxf(amax, fabsf(static_cast<float>(in[lin + k * stride[last]])));
            }
            // next row of the block: advance the odometer over dims last-1 .. 0
            for (int d = last - 1; d >= 0; --d) {
                lin += stride[d];
                if (++at[d] < ext[d]) break;
                lin -= (long long)ext[d] * stride[d];
                at[d] = 0;
            }
        }
        static_cast<F *>(a.scale_out)[sp] = static_cast<F>(__fdiv_rn(2.0f * amax, a.range));
    }
}

void finish_layout(GeneralLayout &L, int nq)
{
    long long n = 1;
    bool ok = true;
    for (int d = 0; d < L.rank; ++d) {
        n *= L.shape[d];
        ok = ok && L.shape[d] >= 1 && L.shape[d] < (1ll << 31) && L.block[d] >= 1 && L.block[d] < (1ll << 31) && n < (1ll << 31);
    }
    L.fits31 = ok ? 1 : 0;
    for (int d = 0; d < QK_MAX_RANK; ++d) {
        L.shape_div[d] = make_fastdiv((ok && d < L.rank) ? (unsigned)L.shape[d] : 1u);
        L.block_div[d] = make_fastdiv((ok && d < L.rank) ? (unsigned)L.block[d] : 1u);
    }
    const long long plast = (L.rank >= 1 && nq >= 1) ? L.shape[L.rank - 1] / nq : 1;
    L.packed_last_div = make_fastdiv((plast >= 1 && plast < (1ll << 31)) ? (unsigned)plast : 1u);
}

cudaError_t launch_general_quantize(const GeneralQuantArgs &a, const LaunchCfg &cfg, cudaStream_t stream)
{
    if (a.nitems == 0) return cudaSuccess;
    GeneralQuantArgs args = a;
    args.force_exact = cfg.force_exact;
    // packed kinds on contiguous, 16-byte aligned data read an item's elements as 16-byte (or one 8-byte) vectors
    const int item_bytes = a.nq * (a.fdt == QK_F32 ? 4 : 2);
    args.vector_bytes = 0;
    if (a.kind <= KIND_PACK2 && a.layout.data_contiguous && reinterpret_cast<uintptr_t>(a.in) % 16 == 0)
        args.vector_bytes = (item_bytes % 16 == 0) ? 16 : (item_bytes == 8 ? 8 : 0);
    switch (a.fdt) {
    case QK_F32:
        general_quantize_kernel<QK_F32><<<grid_for(a.nitems, 256, one_wave(cfg, general_quantize_kernel<QK_F32>)), 256, 0, stream>>>(args);
        break;
    case QK_F16:
        general_quantize_kernel<QK_F16><<<grid_for(a.nitems, 256, one_wave(cfg, general_quantize_kernel<QK_F16>)), 256, 0, stream>>>(args);
        break;
    default:
        general_quantize_kernel<QK_BF16><<<grid_for(a.nitems, 256, one_wave(cfg, general_quantize_kernel<QK_BF16>)), 256, 0, stream>>>(args);
        break;
    }
    return cudaGetLastError();
}
cudaError_t launch_general_dequantize(const GeneralDequantArgs &a, const LaunchCfg &cfg, cudaStream_t stream)
{
    if (a.nitems == 0) return cudaSuccess;
    GeneralDequantArgs args = a;
    // packed kinds into contiguous, 16-byte aligned output write an item's elements as 16-byte (or one 8-byte) vectors
    const int item_bytes = a.nq * (a.fdt == QK_F32 ? 4 : 2);
    args.vector_bytes = 0;
    if (a.kind <= KIND_PACK2 && a.layout.data_contiguous && reinterpret_cast<uintptr_t>(a.out) % 16 == 0)
        args.vector_bytes = (item_bytes % 16 == 0) ? 16 : (item_bytes == 8 ? 8 : 0);
    switch (a.fdt) {
    case QK_F32:
        general_dequantize_kernel<QK_F32><<<grid_for(a.nitems, 256, one_wave(cfg, general_dequantize_kernel<QK_F32>)), 256, 0, stream>>>(args);
        break;
    case QK_F16:
        general_dequantize_kernel<QK_F16><<<grid_for(a.nitems, 256, one_wave(cfg, general_dequantize_kernel<QK_F16>)), 256, 0, stream>>>(args);
        break;
    default:
        general_dequantize_kernel<QK_BF16><<<grid_for(a.nitems, 256, one_wave(cfg, general_dequantize_kernel<QK_BF16>)), 256, 0, stream>>>(args);
        break;
    }
    return cudaGetLastError();
}
cudaError_t launch_general_scales(const GeneralScalesArgs &a, const LaunchCfg &cfg, cudaStream_t stream)
{
    if (a.nblocks == 0) return cudaSuccess;
    switch (a.fdt) {
    case QK_F32:
        general_scales_kernel<QK_F32><<<grid_for(a.nblocks, 256, one_wave(cfg, general_scales_kernel<QK_F32>)), 256, 0, stream>>>(a);
        break;
    case QK_F16:
        general_scales_kernel<QK_F16><<<grid_for(a.nblocks, 256, one_wave(cfg, general_scales_kernel<QK_F16>)), 256, 0, stream>>>(a);
        break;
    default:
        general_scales_kernel<QK_BF16><<<grid_for(a.nblocks, 256, one_wave(cfg, general_scales_kernel<QK_BF16>)), 256, 0, stream>>>(a);
        break;
    }
    return cudaGetLastError();
}

}  // namespace qk
