// `into_contiguous_packed`: a packed quantized tensor whose packing runs along another dim than the last (a
// column-major matmul operand keeps `num_quants` values per item along its rows) is rewritten as a contiguous
// row-major tensor packed along the last dim - what `MatmulInputHandleRef::into_contiguous` does to quantized
// operands before a kernel that wants them contiguous (crates/cubek-matmul/src/base.rs:489-541: packing =
// num_quants for u32 stores, 2 for native e2m1x2).  The function itself lives in the reference's external kernel
// library; this restates its contract from those call sites: field `i` of output item (.., r, cw) is the value
// at logical position (.., r, cw * packing + i), fetched from the input item that holds it.  Positions past the
// logical extent (a last dim that is not a multiple of the packing) are filled with zero bits.
#include "common.cuh"
#include "misc_kernels.cuh"

namespace qk {

template <typename Item>
__global__ void __launch_bounds__(256) repack_kernel(const RepackArgs a)
{
    const Item *in = static_cast<const Item *>(a.in);
    Item *out = static_cast<Item *>(a.out);
    const int last = a.rank - 1;
    const long long out_last = (a.shape[last] + a.packing - 1) / a.packing;
    const uint32_t mask = (a.bits == 32) ? 0xffffffffu : ((1u << a.bits) - 1u);
    pdl_entry();
    for (long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x; o < a.nitems_out;
         o += (long long)gridDim.x * blockDim.x) {
        // coordinates of the output item; `base` gathers the input offset of every dim but the packed one
        long long rem = o / out_last;
        const long long cw = o - rem * out_last;
        long long coord[QK_MAX_RANK];
        for (int d = last - 1; d >= 0; --d) {
            coord[d] = rem % a.shape[d];
            rem /= a.shape[d];
        }
        uint32_t word = 0;
        for (int i = 0; i < a.packing; ++i) {
            coord[last] = cw * a.packing + i;
            if (coord[last] >= a.shape[last]) break;
            long long off = 0;
            int field = 0;
            for (int d = 0; d < a.rank; ++d) {
                long long c = coord[d];
                if (d == a.packed_dim) {
                    field = (int)(c % a.packing);
                    c /= a.packing;
                }
                off += c * a.in_strides[d];
            }
            const uint32_t v = ((uint32_t)in[off] >> (field * a.bits)) & mask;
            word |= v << (i * a.bits);
        }
        out[o] = (Item)word;
    }
}

cudaError_t launch_repack(const RepackArgs &a, const LaunchCfg &cfg, cudaStream_t stream)
{
    long long grid = (a.nitems_out + 255) / 256;
    const long long cap = (long long)cfg.sm_count * 8;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    const bool pdl = cfg.pdl != 0;
    if (a.item_bytes == 4) return launch_kernel(repack_kernel<uint32_t>, (int)grid, 256, stream, pdl, a);
    return launch_kernel(repack_kernel<uint8_t>, (int)grid, 256, stream, pdl, a);
}

}  // namespace qk
