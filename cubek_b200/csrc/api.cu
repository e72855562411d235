// C ABI: argument validation (every `panic!` / `assert!` site of the reference becomes a
// status code), launch geometry and dispatch.  Host-side counterpart of
// `quantize::launch_ref` / `quantize_packed` / `quantize_native`
// (crates/cubek-quant/src/quantize.rs:174-326), `dequantize::launch_ref` and helpers
// (crates/cubek-quant/src/dequantize.rs:171-332) and `scales_layout`
// (crates/cubek-quant/src/layout/scales.rs:220-258).
#include <atomic>
#include <cstdio>
#include <cstring>
#include <dlfcn.h>

#include <chrono>
#include <thread>

#include "../../include/cubek_quant_b200_testing.h"
#include "dequantize_kernels.cuh"
#include "misc_kernels.cuh"
#include "quantize_kernels.cuh"

namespace qk {

cudaError_t launch_quantize_f32(int, int, bool, bool, int, const QuantArgs &, const LaunchCfg &, cudaStream_t);
cudaError_t launch_quantize_f16(int, int, bool, bool, int, const QuantArgs &, const LaunchCfg &, cudaStream_t);
cudaError_t launch_quantize_bf16(int, int, bool, bool, int, const QuantArgs &, const LaunchCfg &, cudaStream_t);
cudaError_t launch_block_scales_f32(const void *, void *, long long, int, int, float, float, const RowStride &, const LaunchCfg &, cudaStream_t);
cudaError_t launch_block_scales_f16(const void *, void *, long long, int, int, float, float, const RowStride &, const LaunchCfg &, cudaStream_t);
cudaError_t launch_block_scales_bf16(const void *, void *, long long, int, int, float, float, const RowStride &, const LaunchCfg &, cudaStream_t);

cudaError_t launch_block_scales_2d_f32(const void *, void *, long long, long long, int, int, float, float, const LaunchCfg &, cudaStream_t);
cudaError_t launch_block_scales_2d_f16(const void *, void *, long long, long long, int, int, float, float, const LaunchCfg &, cudaStream_t);
cudaError_t launch_block_scales_2d_bf16(const void *, void *, long long, long long, int, int, float, float, const LaunchCfg &, cudaStream_t);

cudaError_t launch_block_scales_2d(int fdt, const void *in, void *scale_out, long long rows, long long cols,
                                   int block_rows, int block_cols, float range, float inv_range, const LaunchCfg &cfg,
                                   cudaStream_t stream)
{
    switch (fdt) {
    case QK_F32: return launch_block_scales_2d_f32(in, scale_out, rows, cols, block_rows, block_cols, range, inv_range, cfg, stream);
    case QK_F16: return launch_block_scales_2d_f16(in, scale_out, rows, cols, block_rows, block_cols, range, inv_range, cfg, stream);
    case QK_BF16: return launch_block_scales_2d_bf16(in, scale_out, rows, cols, block_rows, block_cols, range, inv_range, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_quantize_tensor_f32(int, QuantTensorArgs &, int, const LaunchCfg &, cudaStream_t);
cudaError_t launch_quantize_tensor_f16(int, QuantTensorArgs &, int, const LaunchCfg &, cudaStream_t);
cudaError_t launch_quantize_tensor_bf16(int, QuantTensorArgs &, int, const LaunchCfg &, cudaStream_t);

cudaError_t launch_quantize_tensor(int fdt, int kind, QuantTensorArgs &args, int partials_capacity, const LaunchCfg &cfg,
                                   cudaStream_t stream)
{
    switch (fdt) {
    case QK_F32: return launch_quantize_tensor_f32(kind, args, partials_capacity, cfg, stream);
    case QK_F16: return launch_quantize_tensor_f16(kind, args, partials_capacity, cfg, stream);
    case QK_BF16: return launch_quantize_tensor_bf16(kind, args, partials_capacity, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_quantize(int fdt, int kind, int unit_bytes, bool dyn, bool clamp, int sub, const QuantArgs &args,
                            const LaunchCfg &cfg, cudaStream_t stream)
{
    switch (fdt) {
    case QK_F32: return launch_quantize_f32(kind, unit_bytes, dyn, clamp, sub, args, cfg, stream);
    case QK_F16: return launch_quantize_f16(kind, unit_bytes, dyn, clamp, sub, args, cfg, stream);
    case QK_BF16: return launch_quantize_bf16(kind, unit_bytes, dyn, clamp, sub, args, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_block_scales(int fdt, const void *in, void *scale_out, long long nunits, int unit_bytes, int lg,
                                float range, float inv_range, const RowStride &rs, const LaunchCfg &cfg, cudaStream_t stream)
{
    switch (fdt) {
    case QK_F32: return launch_block_scales_f32(in, scale_out, nunits, unit_bytes, lg, range, inv_range, rs, cfg, stream);
    case QK_F16: return launch_block_scales_f16(in, scale_out, nunits, unit_bytes, lg, range, inv_range, rs, cfg, stream);
    case QK_BF16: return launch_block_scales_bf16(in, scale_out, nunits, unit_bytes, lg, range, inv_range, rs, cfg, stream);
    default: return cudaErrorInvalidValue;
    }
}

// ---- process-wide knobs (measurement only) and counters ------------------------------------
enum { TUNE_THREADS = 0, TUNE_CTAS_PER_SM = 1, TUNE_FORCE_EXACT = 2, TUNE_FORCE_GENERAL = 3, TUNE_PDL = 4,
       TUNE_QUANT_WAVES = 5, TUNE_DEQUANT_WAVES = 6, TUNE_COOP_TENSOR = 7, TUNE_STAGED = 8, TUNE_SLICE_KIB = 9,
       TUNE_SLOTS = 10, TUNE_STAGES = 11, TUNE_TENSOR_SMEM_ROWS = 12, TUNE_COOP_MAX_MIB = 13, TUNE_COUNT = 14 };
static std::atomic<int> g_tune[TUNE_COUNT] = {{256}, {0}, {0}, {0}, {1}, {1}, {12}, {1}, {0}, {0}, {4}, {2}, {-1}, {256}};
static std::atomic<uint64_t> g_launches{0};
static std::atomic<int> g_sm_count[64];

// Flag the staged kernels raise when a bounded mbarrier wait gives up.  One per device image of this
// translation unit; the host needs its device address (once per device, with that device current).
static __device__ int g_stage_error;
static std::atomic<int *> g_stage_error_addr[64];

int *stage_error_flag()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    int *p = g_stage_error_addr[dev].load();
    if (p) return p;
    void *addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_stage_error) != cudaSuccess) return nullptr;
    g_stage_error_addr[dev].store(static_cast<int *>(addr));
    return static_cast<int *>(addr);
}

static int sm_count_of_current_device()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = g_sm_count[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev].store(n, std::memory_order_relaxed);
    return n;
}

static LaunchCfg current_cfg()
{
    LaunchCfg c;
    c.threads = g_tune[TUNE_THREADS].load();
    c.ctas_per_sm = g_tune[TUNE_CTAS_PER_SM].load();
    c.force_exact = g_tune[TUNE_FORCE_EXACT].load();
    c.pdl = g_tune[TUNE_PDL].load();
    c.quant_waves = g_tune[TUNE_QUANT_WAVES].load();
    c.staged = g_tune[TUNE_STAGED].load();
    c.stages = g_tune[TUNE_STAGES].load();
    c.tensor_smem_rows = g_tune[TUNE_TENSOR_SMEM_ROWS].load();
    c.dequant_waves = g_tune[TUNE_DEQUANT_WAVES].load();
    c.sm_count = sm_count_of_current_device();
    return c;
}

static inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? QK_OK : QK_ERR_CUDA + (int)e; }
static inline void count_launch(int n = 1) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

// ---- scheme helpers ----------------------------------------------------------------------------
static int dtype_size(int dt) { return dt == QK_F32 ? 4 : (dt == QK_F16 || dt == QK_BF16) ? 2 : 0; }

static int value_bits(int value)
{
    switch (value) {
    case QK_Q8F: case QK_Q8S: case QK_E4M3: case QK_E5M2: return 8;
    case QK_Q4F: case QK_Q4S: case QK_E2M1: return 4;
    case QK_Q2F: case QK_Q2S: return 2;
    default: return 0;
    }
}

static int num_quants(const QkScheme *s)
{
    const int bits = value_bits(s->value);
    if (bits == 0) return 0;
    if (s->store == QK_STORE_U32) return 32 / bits;
    if (s->store == QK_STORE_NATIVE) return s->value == QK_E2M1 ? 2 : 1;
    return 0;
}

static int kind_of(const QkScheme *s)
{
    if (s->store == QK_STORE_U32) {
        const int bits = value_bits(s->value);
        return bits == 8 ? KIND_PACK8 : bits == 4 ? KIND_PACK4 : KIND_PACK2;
    }
    switch (s->value) {
    case QK_Q8F: case QK_Q8S: return KIND_I8;
    case QK_E2M1: return KIND_E2M1;
    case QK_E4M3: return KIND_E4M3;
    case QK_E5M2: return KIND_E5M2;
    default: return -1;
    }
}

// The checks `launch_ref` performs by pattern matching (quantize.rs:185-220).
static int check_scheme(const QkScheme *s)
{
    if (value_bits(s->value) == 0) return QK_ERR_UNSUPPORTED_SCHEME;
    if (s->store != QK_STORE_U32 && s->store != QK_STORE_NATIVE) return QK_ERR_UNSUPPORTED_SCHEME;
    if (s->mode != QK_MODE_SYMMETRIC) return QK_ERR_UNSUPPORTED_SCHEME;
    if (dtype_size(s->param) == 0) return QK_ERR_UNSUPPORTED_SCHEME;
    if (s->level != QK_LEVEL_TENSOR && s->level != QK_LEVEL_BLOCK) return QK_ERR_UNSUPPORTED_SCHEME;
    if (s->store == QK_STORE_NATIVE && kind_of(s) < 0) return QK_ERR_UNSUPPORTED_SCHEME;  // Q4*/Q2* native
    if (s->level == QK_LEVEL_BLOCK) {
        if (s->block_rank < 1 || s->block_rank > 8) return QK_ERR_BLOCK_SIZE;
        for (int i = 0; i < s->block_rank; ++i)
            if (s->block[i] == 0) return QK_ERR_BLOCK_SIZE;
    }
    return QK_OK;
}

static long long numel(const QkTensor *t)
{
    long long n = 1;
    for (int d = 0; d < t->rank; ++d) n *= t->shape[d];
    return n;
}

static bool is_contiguous(const QkTensor *t)
{
    long long expect = 1;
    for (int d = t->rank - 1; d >= 0; --d) {
        if (t->shape[d] != 1 && t->strides[d] != expect) return false;
        expect *= t->shape[d];
    }
    return true;
}

// A view whose strides are a permutation of a dense row-major layout (a transposed matrix, a permuted
// N-d tensor): its elements fill `numel` consecutive positions from `ptr`, so an order-independent
// reduction may walk the memory instead of the view.
static bool is_dense_permutation(const QkTensor *t)
{
    int order[QK_MAX_RANK];
    int n = 0;
    for (int d = 0; d < t->rank; ++d) {
        if (t->shape[d] == 1) continue;
        if (t->strides[d] <= 0) return false;
        order[n++] = d;
    }
    for (int i = 1; i < n; ++i)   // insertion sort by stride
        for (int j = i; j > 0 && t->strides[order[j]] < t->strides[order[j - 1]]; --j) {
            const int tmp = order[j];
            order[j] = order[j - 1];
            order[j - 1] = tmp;
        }
    long long expect = 1;
    for (int i = 0; i < n; ++i) {
        if (t->strides[order[i]] != expect) return false;
        expect *= t->shape[order[i]];
    }
    return true;
}

// Rows (runs along the last dim) contiguous, rows a constant number of elements apart: a column slice
// of a wider matrix, a matrix with padded rows.  Leading dims must step uniformly over the rows.
static bool is_row_strided(const QkTensor *t, long long *row_stride)
{
    const int r = t->rank;
    if (r < 2 || (t->shape[r - 1] != 1 && t->strides[r - 1] != 1)) return false;
    long long expect = 0;
    for (int d = r - 2; d >= 0; --d) {
        if (t->shape[d] == 1) continue;
        if (expect == 0) {
            if (t->strides[d] < t->shape[r - 1]) return false;
            *row_stride = t->strides[d];
        } else if (t->strides[d] != expect) {
            return false;
        }
        expect = (expect == 0 ? t->strides[d] : expect) * t->shape[d];
    }
    return expect != 0;
}

// A transposed matrix: rank 2, element (r, c) at c * ld + r with ld >= rows.
static bool is_transposed_matrix(const QkTensor *t, long long *ld)
{
    if (t->rank != 2 || t->shape[0] < 2 || t->shape[1] < 2) return false;
    if (t->strides[0] != 1 || t->strides[1] < t->shape[0]) return false;
    *ld = t->strides[1];
    return true;
}

// Tile geometry of the transposed quantize / scales kernels: tiles of 32 (64 with row pairs) rows x 8 units.
static long long fill_transposed_tiles(Transposed &tr, const QkTensor *t, long long ld, int fsize, long long unit_elems)
{
    const bool pairs = fsize == 2 && t->shape[0] % 2 == 0 && ld % 2 == 0 && (reinterpret_cast<uintptr_t>(t->ptr) & 3u) == 0;
    const long long rows_per_tile = pairs ? 64 : 32;
    const long long row_tiles = (t->shape[0] + rows_per_tile - 1) / rows_per_tile;
    const long long unit_tiles = (t->shape[1] / unit_elems + 7) / 8;
    tr.enabled = 1;
    tr.pairs = pairs ? 1 : 0;
    tr.rows = make_fastdiv((unsigned)row_tiles);
    tr.nrows = (unsigned)t->shape[0];
    tr.ld = ld;
    tr.units_per_row = (unsigned)(t->shape[1] / unit_elems);
    return row_tiles * unit_tiles;
}

static int check_tensor(const QkTensor *t, int elem_size)
{
    if (!t || !t->shape || !t->strides) return QK_ERR_NULL;
    if (t->rank < 1 || t->rank > QK_MAX_RANK) return QK_ERR_SHAPE;
    for (int d = 0; d < t->rank; ++d)
        if (t->shape[d] < 0) return QK_ERR_SHAPE;
    if (t->elem_size != elem_size) return QK_ERR_DTYPE;
    if (numel(t) > 0) {
        if (!t->ptr) return QK_ERR_NULL;
        if (reinterpret_cast<uintptr_t>(t->ptr) % (uintptr_t)elem_size) return QK_ERR_ALIGN;
    }
    return QK_OK;
}

// Everything the launchers need to know about one call, derived from the handles the way
// `scales_layout` / `shape_divmod_quant` do (layout/scales.rs:220-258).
struct Geometry {
    int rank = 0, nq = 0, kind = 0;
    long long n = 0;                 // unpacked elements
    long long block[QK_MAX_RANK];    // left-padded with 1
    long long shape[QK_MAX_RANK];    // unpacked shape
    bool per_tensor = true;
    bool last_dim_blocks = false;    // blocks only along the last dim, rows split evenly
    bool blocks_2d = false;          // [block_rows, B] tiles over the last two dims (cols split evenly)
    long long block_rows = 1;        // tile extent along dim rank-2
    long long cols = 0;              // extent of the last dim
    long long B = 0;                 // block extent along the last dim
    long long nscales = 1;
};

// `values` is the quantized tensor; `unpacked` the float one.  Shapes must agree as
// unpacked = packed with the last dim multiplied by num_quants.
static int build_geometry(Geometry &g, const QkScheme *s, const QkTensor *unpacked, const QkTensor *values)
{
    g.nq = num_quants(s);
    g.kind = kind_of(s);
    g.rank = unpacked->rank;
    if (values && values->rank != unpacked->rank) return QK_ERR_SHAPE;
    for (int d = 0; d < g.rank; ++d) {
        g.shape[d] = unpacked->shape[d];
        g.block[d] = 1;
        if (values) {
            const long long want = (d == g.rank - 1) ? values->shape[d] * g.nq : values->shape[d];
            if (want != unpacked->shape[d]) return QK_ERR_SHAPE;
        }
    }
    if (unpacked->shape[g.rank - 1] % g.nq != 0) return QK_ERR_SHAPE;
    g.n = numel(unpacked);
    g.per_tensor = (s->level == QK_LEVEL_TENSOR);
    g.nscales = 1;
    if (!g.per_tensor) {
        if (s->block_rank > g.rank) return QK_ERR_BLOCK_SIZE;
        for (int i = 0; i < s->block_rank; ++i) g.block[g.rank - s->block_rank + i] = s->block[i];
        g.B = g.block[g.rank - 1];
        g.last_dim_blocks = (g.shape[g.rank - 1] % g.B == 0);
        for (int d = 0; d < g.rank - 1; ++d) g.last_dim_blocks = g.last_dim_blocks && g.block[d] == 1;
        g.cols = g.shape[g.rank - 1];
        if (!g.last_dim_blocks && g.rank >= 2 && g.block[g.rank - 2] > 1 && g.cols % g.B == 0) {
            // Tiles over the last two dims; leading dims may be flattened into rows only if no tile
            // would straddle two matrices.
            bool ok = (g.rank == 2) || (g.shape[g.rank - 2] % g.block[g.rank - 2] == 0);
            for (int d = 0; d < g.rank - 2; ++d) ok = ok && g.block[d] == 1;
            g.blocks_2d = ok;
            g.block_rows = g.block[g.rank - 2];
        }
        for (int d = 0; d < g.rank; ++d) g.nscales *= (g.shape[d] + g.block[d] - 1) / g.block[d];
    }
    return QK_OK;
}

// A scales tensor must hold one element per tensor, or one per block with the rank of the values.
static int check_scales_shape(const Geometry &g, const QkTensor *sc)
{
    if (g.per_tensor) return numel(sc) == 1 ? QK_OK : QK_ERR_SHAPE;
    if (sc->rank != g.rank) return QK_ERR_SHAPE;
    for (int d = 0; d < g.rank; ++d)
        if (sc->shape[d] != (g.shape[d] + g.block[d] - 1) / g.block[d]) return QK_ERR_SHAPE;
    return QK_OK;
}

static void fill_layout(GeneralLayout &L, const Geometry &g, const QkTensor *scales, const QkTensor *out_scales,
                        const QkTensor *data, const QkTensor *values = nullptr)
{
    L.data_contiguous = (!data || is_contiguous(data)) ? 1 : 0;
    L.values_contiguous = (!values || is_contiguous(values)) ? 1 : 0;
    L.rank = g.rank;
    L.per_tensor = g.per_tensor ? 1 : 0;
    for (int d = 0; d < QK_MAX_RANK; ++d) {
        L.shape[d] = d < g.rank ? g.shape[d] : 1;
        L.block[d] = d < g.rank ? g.block[d] : 1;
        L.scale_strides[d] = (!g.per_tensor && scales && d < g.rank) ? scales->strides[d] : 0;
        L.out_scale_strides[d] = (!g.per_tensor && out_scales && d < g.rank) ? out_scales->strides[d] : 0;
        L.data_strides[d] = (data && d < g.rank) ? data->strides[d] : 0;
        L.values_strides[d] = (values && d < g.rank) ? values->strides[d] : 0;
    }
    finish_layout(L, g.nq);
}

static int log2_exact(long long v)
{
    if (v <= 0 || (v & (v - 1))) return -1;
    int lg = 0;
    while ((1ll << lg) < v) ++lg;
    return lg;
}

static bool aligned(const void *p, unsigned a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// The streaming kernels need whole units, power-of-two blocks made of whole units along the
// last dim, contiguous scales and vector-aligned bases.  Picks the unit (64 bytes when blocks
// and the tensor allow, else the smallest unit of the kind); returns log2(units per block), -1
// for per tensor, or -2 when the call has to take the layout-general kernels.
// `*sub` (optional) is set to the blocks per unit: 2 when 16-bit blocks of 32 bytes may run as halves of 64-byte
// units (f32 params, scales out 8-byte aligned, given scales 4-byte aligned), else 1.
static int fast_quantize_lg(const Geometry &g, int fdt, const QkTensor *in, const QkTensor *out,
                            const QkTensor *scale, const QkTensor *out_scale, int *unit_bytes, int *sub = nullptr,
                            bool fused = false, int param = QK_F32)
{
    if (sub) *sub = 1;
    if (g_tune[TUNE_FORCE_GENERAL].load()) return -2;
    if (!is_contiguous(out)) return -2;   // a strided quantized tensor (a transposed matmul operand): general kernels
    const int esz = dtype_size(fdt);
    if (!aligned(in->ptr, 16)) return -2;
    long long row_stride = 0;
    const bool strided_rows = !is_contiguous(in);
    if (strided_rows) {
        // rows of whole units, every row 16-byte aligned, no tiles over two dims
        if (!is_row_strided(in, &row_stride) || (row_stride * esz) % 16 != 0 || g.blocks_2d) return -2;
    }
    if (!g.per_tensor) {
        if (!g.last_dim_blocks && !g.blocks_2d) return -2;
        if (scale && !is_contiguous(scale)) return -2;
        if (out_scale && !is_contiguous(out_scale)) return -2;
    }
    const int candidates[3] = {64, 32, min_unit_bytes(fdt, g.kind)};
    for (int ci = 0; ci < 3; ++ci) {
        const int ub = candidates[ci];
        if (ub < min_unit_bytes(fdt, g.kind)) continue;
        const int U = ub / esz;
        if (g.n % U != 0) continue;
        if (strided_rows && (g.shape[g.rank - 1] % U != 0 || g.n / U >= (1ll << 31))) continue;
        const int out_words = U / kind_elems_per_u32(g.kind);
        const int out_align = out_words >= 4 ? 16 : 4 * out_words;
        if (!aligned(out->ptr, out_align)) continue;
        *unit_bytes = ub;
        if (g.per_tensor) return -1;
        if (sub && (fused || (scale && aligned(scale->ptr, 4))) && ub == 64 && esz == 2 && U == 2 * g.B && !g.blocks_2d &&
            !strided_rows && param == QK_F32 && 32 >= min_unit_bytes(fdt, g.kind) && out_scale && aligned(out_scale->ptr, 8)) {
            *sub = 2;
            return 0;
        }
        if (g.B % U != 0) continue;
        const int lg = log2_exact(g.B / U);
        if (lg < 0 || (lg > 5 && !g.blocks_2d)) continue;
        if (g.blocks_2d && g.n / U >= (1ll << 31)) continue;
        return lg;
    }
    return -2;
}

// Tile geometry for the streaming kernels (units of `unit_elems` elements).
static Blocks2D make_blocks2d(const Geometry &g, int unit_elems, int lg)
{
    Blocks2D b;
    b.enabled = g.blocks_2d ? 1 : 0;
    b.units_per_row = make_fastdiv((unsigned)(g.blocks_2d ? g.cols / unit_elems : 1));
    b.block_rows = make_fastdiv((unsigned)(g.blocks_2d ? g.block_rows : 1));
    b.scales_per_row = (unsigned)(g.blocks_2d ? g.cols / g.B : 1);
    b.lg_units_per_block_col = lg < 0 ? 0 : lg;
    return b;
}

static int fast_dequantize_lg(const Geometry &g, int fdt, const QkTensor *values, const QkTensor *out,
                              const QkTensor *params, int *out_bytes, int *sub, int param)
{
    *sub = 1;
    if (g_tune[TUNE_FORCE_GENERAL].load()) return -2;
    if (!is_contiguous(values)) return -2;
    const int esz = dtype_size(fdt);
    if (!aligned(out->ptr, 16)) return -2;
    long long row_stride = 0;
    const bool strided_rows = !is_contiguous(out);
    if (strided_rows && (!is_row_strided(out, &row_stride) || (row_stride * esz) % 16 != 0 || g.blocks_2d)) return -2;
    if (!g.per_tensor && ((!g.last_dim_blocks && !g.blocks_2d) || !is_contiguous(params))) return -2;
    const int candidates[2] = {64, min_dequant_bytes(fdt, g.kind)};
    for (int ci = 0; ci < 2; ++ci) {
        const int ob = candidates[ci];
        const int E = ob / esz;
        if (g.n % E != 0) continue;
        if (strided_rows && (g.shape[g.rank - 1] % E != 0 || g.n / E >= (1ll << 31))) continue;
        const int in_words = E / kind_elems_per_u32(g.kind);
        if (!aligned(values->ptr, in_words >= 4 ? 16 : 4 * in_words)) continue;
        *out_bytes = ob;
        if (g.per_tensor) return -1;
        // 16-bit blocks of 32 bytes: two per 64-byte unit (f32 params fetched as one 8-byte load)
        if (ob == 64 && esz == 2 && E == 2 * g.B && !g.blocks_2d && !strided_rows && param == QK_F32 &&
            aligned(params->ptr, 8) && (E / kind_elems_per_u32(g.kind)) % 2 == 0) {
            *sub = 2;
            return 0;
        }
        if (g.B % E != 0) continue;
        const int lg = log2_exact(g.B / E);
        if (lg < 0) continue;
        if (g.blocks_2d && g.n / E >= (1ll << 31)) continue;
        return lg;
    }
    return -2;
}

// Layout of a strided float tensor for the whole-tensor absmax (no blocks, no scales).
static GeneralLayout strided_data_layout(const QkTensor *t)
{
    GeneralLayout L;
    L.rank = t->rank;
    L.per_tensor = 1;
    L.data_contiguous = 0;
    L.values_contiguous = 1;
    for (int d = 0; d < QK_MAX_RANK; ++d) {
        L.shape[d] = d < t->rank ? t->shape[d] : 1;
        L.data_strides[d] = d < t->rank ? t->strides[d] : 0;
        L.block[d] = 1;
        L.values_strides[d] = 0;
        L.scale_strides[d] = L.out_scale_strides[d] = 0;
    }
    finish_layout(L);
    return L;
}

// absmax of any float tensor into `*cell`: in memory order for contiguous and densely permuted views, row by
// row for row-strided ones (whole 16-byte chunks per row), element by element through the strides otherwise.
static cudaError_t absmax_of(const QkTensor *t, int dtype, long long n, unsigned int *cell, const LaunchCfg &cfg,
                             cudaStream_t stream, bool zero_first)
{
    if (is_contiguous(t) || is_dense_permutation(t)) return launch_absmax(dtype, t->ptr, n, cell, cfg, stream, zero_first);
    const int fsize = dtype_size(dtype);
    const int per16 = 16 / fsize;
    const long long cols = t->shape[t->rank - 1];
    long long row_stride = 0;
    if (is_row_strided(t, &row_stride) && aligned(t->ptr, 16) && (row_stride * fsize) % 16 == 0 && cols % per16 == 0 &&
        n / per16 < (1ll << 31)) {
        RowStride rs;
        rs.enabled = 1;
        rs.units_per_row = make_fastdiv((unsigned)(cols / per16));
        rs.row_bytes = row_stride * fsize;
        return launch_absmax(dtype, t->ptr, n, cell, cfg, stream, zero_first, &rs);
    }
    const GeneralLayout L = strided_data_layout(t);
    return launch_absmax_strided(L, t->ptr, dtype, n, cell, cfg, stream);   // clears the cell itself
}

// absmax of `count` tensors into `cells[0..count)` (already zero): tensors that are contiguous, start on
// a 16-byte boundary and hold whole 16-byte chunks share launches of up to QK_ABSMAX_BATCH tensors; the
// others get a launch each.
static int absmax_into_cells(int count, const QkTensor *inputs, const bool *skip, int input_dtype, unsigned int *cells,
                             const LaunchCfg &cfg, cudaStream_t stream)
{
    const int fsize = dtype_size(input_dtype);
    const int per16 = 16 / fsize;
    AbsmaxBatchArgs b;
    b.ntensors = 0;
    b.cells = nullptr;
    int rc;
    auto flush = [&]() -> int {
        if (b.ntensors == 0) return QK_OK;
        count_launch();
        const cudaError_t e = launch_absmax_batch(input_dtype, b, cfg, stream);
        b.ntensors = 0;
        return cuda_status(e);
    };
    for (int i = 0; i < count; ++i) {
        if (skip && skip[i]) {
            if ((rc = flush())) return rc;   // cells of one launch are consecutive
            continue;
        }
        if ((rc = check_tensor(&inputs[i], fsize))) return rc;
        const long long n = numel(&inputs[i]);
        if (n == 0) {
            if ((rc = flush())) return rc;
            continue;
        }
        if (!is_contiguous(&inputs[i]) && !is_dense_permutation(&inputs[i])) {
            if ((rc = flush())) return rc;
            count_launch();
            const cudaError_t e = absmax_of(&inputs[i], input_dtype, n, cells + i, cfg, stream, false);
            if (e != cudaSuccess) return cuda_status(e);
            continue;
        }
        const bool chunkable = (n % per16 == 0) && aligned(inputs[i].ptr, 16);
        if (!chunkable) {
            if ((rc = flush())) return rc;
            count_launch();
            const cudaError_t e = launch_absmax(input_dtype, inputs[i].ptr, n, cells + i, cfg, stream, false);
            if (e != cudaSuccess) return cuda_status(e);
            continue;
        }
        if (b.ntensors == QK_ABSMAX_BATCH && (rc = flush())) return rc;
        if (b.ntensors == 0) b.cells = cells + i;
        b.in[b.ntensors] = inputs[i].ptr;
        b.chunk_end[b.ntensors] = (b.ntensors ? b.chunk_end[b.ntensors - 1] : 0) + n / per16;
        b.ntensors += 1;
    }
    return flush();
}

// Streaming launches are collected here: consecutive tensors that share the kernel
// specialisation and geometry go out as one launch (up to QK_MAX_BATCH tensors).
struct QuantBatch {
    QuantArgs a;
    int fdt = -1, kind = -1, unit_bytes = 0, sub = 1;
    bool dyn = false, clamp = false;
    QuantBatch() { a.ntensors = 0; a.nunits = 0; a.absmax = nullptr; a.b2.enabled = 0; a.rs.enabled = 0; a.tr.enabled = 0; }
};
struct DequantBatch {
    DequantArgs a;
    int fdt = -1, kind = -1, out_bytes = 0, sub = 1;
    DequantBatch() { a.ntensors = 0; a.nunits = 0; a.b2.enabled = 0; a.rs.enabled = 0; a.tr.enabled = 0; }
};

static int flush_quant(QuantBatch &b, const LaunchCfg &cfg, cudaStream_t stream)
{
    if (b.a.ntensors == 0) return QK_OK;
    count_launch();
    const cudaError_t e = launch_quantize(b.fdt, b.kind, b.unit_bytes, b.dyn, b.clamp, b.sub, b.a, cfg, stream);
    b.a.ntensors = 0;
    b.a.nunits = 0;
    b.a.absmax = nullptr;
    return cuda_status(e);
}

static int flush_dequant(DequantBatch &b, const LaunchCfg &cfg, cudaStream_t stream)
{
    if (b.a.ntensors == 0) return QK_OK;
    count_launch();
    const cudaError_t e = launch_dequantize(b.fdt, b.kind, b.out_bytes, b.sub, b.a, cfg, stream);
    b.a.ntensors = 0;
    b.a.nunits = 0;
    return cuda_status(e);
}

static int quantize_common(const QkTensor *input, const QkTensor *output, const QkTensor *scale,
                           const QkTensor *out_scale, const float *absmax, bool dynamic, void *gen_scales,
                           const QkScheme *scheme, int input_dtype, cudaStream_t stream, QuantBatch *batch = nullptr);
static int dequantize_common(const QkTensor *values, const QkTensor *output, const QkTensor *params,
                             const QkScheme *scheme, int output_dtype, cudaStream_t stream, DequantBatch *batch = nullptr);
static int try_quantize_tensor_coop(const QkTensor *input, const QkTensor *output, const QkTensor *out_scale,
                                    const QkScheme *scheme, int input_dtype, void *workspace, size_t workspace_bytes,
                                    cudaStream_t stream);

}  // namespace qk

using namespace qk;

// =============================================================================================
// C ABI
// =============================================================================================
extern "C" {

int qk_num_quants(const QkScheme *scheme) { return scheme ? num_quants(scheme) : 0; }

int qk_value_range(int value, float *lo, float *hi)
{
    float l, h;
    switch (value) {
    case QK_Q8F: l = -128.f; h = 127.f; break;
    case QK_Q8S: l = -127.f; h = 127.f; break;
    case QK_Q4F: l = -8.f; h = 7.f; break;
    case QK_Q4S: l = -7.f; h = 7.f; break;
    case QK_Q2F: l = -2.f; h = 1.f; break;
    case QK_Q2S: l = -1.f; h = 1.f; break;
    case QK_E4M3: l = -448.f; h = 448.f; break;
    case QK_E5M2: l = -57344.f; h = 57344.f; break;
    case QK_E2M1: l = -6.f; h = 6.f; break;
    default: return QK_ERR_UNSUPPORTED_SCHEME;
    }
    if (lo) *lo = l;
    if (hi) *hi = h;
    return QK_OK;
}

size_t qk_workspace_bytes(void) { return 8192; }

size_t qk_workspace_bytes_for(const QkTensor *input, const QkScheme *scheme, int input_dtype)
{
    // Per tensor: the partial absmax of every resident CTA (or, with less than that, one cell and
    // the two-kernel route).  Per block: the fused kernel needs nothing; layouts that fall back to
    // the general kernels stage F-typed scales 256 bytes into the workspace.
    size_t bytes = 256;
    if (input && scheme && dtype_size(input_dtype) != 0 && check_scheme(scheme) == QK_OK && input->shape &&
        input->rank >= 1 && input->rank <= QK_MAX_RANK) {
        Geometry g;
        if (build_geometry(g, scheme, input, nullptr) == QK_OK && !g.per_tensor)
            bytes += (size_t)g.nscales * (size_t)dtype_size(input_dtype);
    }
    if (bytes < qk_workspace_bytes()) bytes = qk_workspace_bytes();
    return (bytes + 255) & ~(size_t)255;
}

int qk_quantize(const QkTensor *input, const QkTensor *output, const QkTensor *scale, const QkTensor *out_scale,
                const QkScheme *scheme, int input_dtype, void *stream)
{
    if (!scale) return QK_ERR_NULL;
    return quantize_common(input, output, scale, out_scale, nullptr, false, nullptr, scheme, input_dtype,
                           static_cast<cudaStream_t>(stream));
}

int qk_dequantize(const QkTensor *values, const QkTensor *output, const QkTensor *params, const QkScheme *scheme,
                  int output_dtype, void *stream)
{
    return dequantize_common(values, output, params, scheme, output_dtype, static_cast<cudaStream_t>(stream));
}

int qk_dequantize_batch(int count, const QkTensor *values, const QkTensor *outputs, const QkTensor *params,
                        const QkScheme *scheme, int output_dtype, void *stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (count < 0) return QK_ERR_SHAPE;
    if (count == 0) return QK_OK;
    if (!values || !outputs || !params || !scheme) return QK_ERR_NULL;
    DequantBatch batch;
    for (int i = 0; i < count; ++i) {
        const int rc = dequantize_common(&values[i], &outputs[i], &params[i], scheme, output_dtype, stream, &batch);
        if (rc != QK_OK) {
            flush_dequant(batch, current_cfg(), stream);
            return rc;
        }
    }
    return flush_dequant(batch, current_cfg(), stream);
}

int qk_quantize_dynamic_batch(int count, const QkTensor *inputs, const QkTensor *outputs, const QkTensor *out_scales,
                              const QkScheme *scheme, int input_dtype, void *workspace, size_t workspace_bytes,
                              void *stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (count < 0) return QK_ERR_SHAPE;
    if (count == 0) return QK_OK;
    if (!inputs || !outputs || !out_scales || !scheme) return QK_ERR_NULL;
    int rc = check_scheme(scheme);
    if (rc) return rc;
    const LaunchCfg cfg = current_cfg();
    QuantBatch batch;
    if (scheme->level == QK_LEVEL_TENSOR) {
        // One absmax cell per tensor at the front of the workspace, cleared once; every tensor's
        // absmax is reduced into its cell, then the quantize launches read them by tensor index.
        if (!workspace || workspace_bytes < sizeof(unsigned int) * (size_t)count) return QK_ERR_WORKSPACE;
        if (!aligned(workspace, 4)) return QK_ERR_ALIGN;
        const int fsize = dtype_size(input_dtype);
        if (fsize == 0) return QK_ERR_DTYPE;
        unsigned int *cells = static_cast<unsigned int *>(workspace);
        const size_t cells_bytes = (sizeof(unsigned int) * (size_t)count + 255) & ~(size_t)255;
        bool pending[QK_MAX_BATCH * 16];
        if (count > (int)(sizeof(pending) / sizeof(pending[0]))) return QK_ERR_TOO_LARGE;
        int npending = 0;
        for (int i = 0; i < count; ++i) {
            pending[i] = true;
            // Only a lone tensor gains from the cooperative kernel (fewer launches, second pass from L2);
            // for a set, one batched absmax launch plus batched quantize launches are faster (measured on
            // 8 x 64 MB f32: 5440 vs 5340 GB/s; on the 225-tensor Llama-shaped set: 9.2 vs 10.2 ms).
            if (count == 1 && workspace_bytes > cells_bytes) {
                rc = try_quantize_tensor_coop(&inputs[i], &outputs[i], &out_scales[i], scheme, input_dtype,
                                              static_cast<char *>(workspace) + cells_bytes, workspace_bytes - cells_bytes,
                                              stream);
                if (rc == QK_OK) pending[i] = false;
                else if (rc != QK_ERR_TOO_LARGE) return rc;
            }
            npending += pending[i] ? 1 : 0;
        }
        if (npending == 0) return QK_OK;
        cudaError_t e = cudaMemsetAsync(cells, 0, sizeof(unsigned int) * (size_t)count, stream);
        if (e != cudaSuccess) return cuda_status(e);
        count_launch();
        {
            bool done[QK_MAX_BATCH * 16];
            for (int i = 0; i < count; ++i) done[i] = !pending[i];
            if ((rc = absmax_into_cells(count, inputs, done, input_dtype, cells, cfg, stream))) return rc;
        }
        for (int i = 0; i < count; ++i) {
            if (!pending[i]) continue;
            rc = quantize_common(&inputs[i], &outputs[i], nullptr, &out_scales[i],
                                 reinterpret_cast<const float *>(cells + i), false, nullptr, scheme, input_dtype, stream,
                                 &batch);
            if (rc != QK_OK) {
                flush_quant(batch, cfg, stream);
                return rc;
            }
        }
        return flush_quant(batch, cfg, stream);
    }
    for (int i = 0; i < count; ++i) {
        void *gen_scales = nullptr;
        if (workspace && workspace_bytes >= qk_workspace_bytes_for(&inputs[i], scheme, input_dtype))
            gen_scales = static_cast<char *>(workspace) + 256;
        rc = quantize_common(&inputs[i], &outputs[i], nullptr, &out_scales[i], nullptr, true, gen_scales, scheme,
                             input_dtype, stream, &batch);
        if (rc != QK_OK) {
            flush_quant(batch, cfg, stream);
            return rc;
        }
    }
    return flush_quant(batch, cfg, stream);
}

int qk_compute_scales(const QkTensor *input, const QkTensor *scale, const QkScheme *scheme, int input_dtype,
                      void *workspace, size_t workspace_bytes, void *stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!input || !scale || !scheme) return QK_ERR_NULL;
    int rc = check_scheme(scheme);
    if (rc) return rc;
    const int fsize = dtype_size(input_dtype);
    if (fsize == 0) return QK_ERR_DTYPE;
    if ((rc = check_tensor(input, fsize))) return rc;
    if ((rc = check_tensor(scale, fsize))) return rc;
    Geometry g;
    if ((rc = build_geometry(g, scheme, input, nullptr))) return rc;
    if ((rc = check_scales_shape(g, scale))) return rc;
    const bool contiguous = is_contiguous(input);
    float lo, hi;
    qk_value_range(scheme->value, &lo, &hi);
    const float range = hi - lo;
    const LaunchCfg cfg = current_cfg();

    if (g.per_tensor) {
        if (!workspace || workspace_bytes < sizeof(unsigned int)) return QK_ERR_WORKSPACE;
        if (!aligned(workspace, 4)) return QK_ERR_ALIGN;
        unsigned int *cell = static_cast<unsigned int *>(workspace);
        count_launch(g.n > 0 ? 3 : 2);
        const cudaError_t e = absmax_of(input, input_dtype, g.n, cell, cfg, stream, true);
        if (e != cudaSuccess) return cuda_status(e);
        return cuda_status(launch_finalize_scale(cell, scale->ptr, input_dtype, range, stream));
    }
    if (g.n == 0) return QK_OK;
    const int per16 = 16 / fsize;
    long long row_stride = 0;
    const bool strided_rows = !contiguous && is_row_strided(input, &row_stride) && (row_stride * fsize) % 16 == 0;
    if (!g_tune[TUNE_FORCE_GENERAL].load() && (contiguous || strided_rows) && g.last_dim_blocks && aligned(input->ptr, 16) &&
        is_contiguous(scale)) {
        // the largest per-thread unit that blocks are made of, with at most 32 lanes per block
        for (int ub = 64; ub >= 16; ub >>= 1) {
            const long long U = ub / fsize;
            if (g.B % U != 0) continue;
            const int lg = log2_exact(g.B / U);
            if (lg < 0 || lg > 5) continue;
            if (strided_rows && g.n / U >= (1ll << 31)) continue;
            RowStride rs;
            rs.enabled = strided_rows ? 1 : 0;
            rs.units_per_row = make_fastdiv(strided_rows ? (unsigned)(g.cols / U) : 1u);
            rs.row_bytes = strided_rows ? row_stride * fsize : 0;
            count_launch();
            return cuda_status(launch_block_scales(input_dtype, input->ptr, scale->ptr, g.n / U, ub, lg, range,
                                                   1.0f / range, rs, cfg, stream));
        }
    }
    if (!g_tune[TUNE_FORCE_GENERAL].load() && contiguous && g.blocks_2d && g.B % per16 == 0 && aligned(input->ptr, 16) &&
        is_contiguous(scale)) {
        count_launch();
        return cuda_status(launch_block_scales_2d(input_dtype, input->ptr, scale->ptr, g.n / g.cols, g.cols,
                                                  (int)g.block_rows, (int)g.B, range, 1.0f / range, cfg, stream));
    }
    long long ld = 0;
    if (!g_tune[TUNE_FORCE_GENERAL].load() && is_transposed_matrix(input, &ld) && g.last_dim_blocks && is_contiguous(scale)) {
        for (int ub = 64; ub >= 32; ub >>= 1) {
            const long long U = ub / fsize;
            const int lgb = (g.B % U == 0) ? log2_exact(g.B / U) : -1;
            if (lgb < 0 || lgb > 3 || g.n / U >= (1ll << 31)) continue;
            Transposed tr;
            const long long ntiles = fill_transposed_tiles(tr, input, ld, fsize, U);
            count_launch();
            return cuda_status(launch_scales_transposed(input_dtype, ub, lgb, input->ptr, scale->ptr, tr, ntiles, range,
                                                        1.0f / range, cfg, stream));
        }
    }
    GeneralScalesArgs a;
    fill_layout(a.layout, g, scale, nullptr, input);
    a.in = input->ptr;
    a.scale_out = scale->ptr;
    a.nblocks = g.nscales;
    a.fdt = input_dtype;
    a.range = range;
    count_launch();
    return cuda_status(launch_general_scales(a, cfg, stream));
}

int qk_quantize_dynamic(const QkTensor *input, const QkTensor *output, const QkTensor *out_scale,
                        const QkScheme *scheme, int input_dtype, void *workspace, size_t workspace_bytes,
                        void *stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!input || !scheme) return QK_ERR_NULL;
    int rc = check_scheme(scheme);
    if (rc) return rc;
    if (scheme->level == QK_LEVEL_TENSOR) {
        if (!workspace || workspace_bytes < sizeof(unsigned int)) return QK_ERR_WORKSPACE;
        if (!aligned(workspace, 4)) return QK_ERR_ALIGN;
        const int fsize = dtype_size(input_dtype);
        if (fsize == 0) return QK_ERR_DTYPE;
        if ((rc = check_tensor(input, fsize))) return rc;
        unsigned int *cell = static_cast<unsigned int *>(workspace);
        const long long n = numel(input);
        rc = try_quantize_tensor_coop(input, output, out_scale, scheme, input_dtype, workspace, workspace_bytes, stream);
        if (rc != QK_ERR_TOO_LARGE) return rc;   // done, or a real error; TOO_LARGE = route not applicable
        count_launch(n > 0 ? 2 : 1);
        const cudaError_t e = absmax_of(input, input_dtype, n, cell, current_cfg(), stream, true);
        if (e != cudaSuccess) return cuda_status(e);
        return quantize_common(input, output, nullptr, out_scale, reinterpret_cast<const float *>(cell), false,
                               nullptr, scheme, input_dtype, stream);
    }
    // Per block: fused kernel, or (general layouts) scales staged in the workspace.
    void *gen_scales = nullptr;
    if (workspace && workspace_bytes >= qk_workspace_bytes_for(input, scheme, input_dtype))
        gen_scales = static_cast<char *>(workspace) + 256;
    return quantize_common(input, output, nullptr, out_scale, nullptr, true, gen_scales, scheme, input_dtype, stream);
}

int qk_reduce(const QkTensor *input, const QkTensor *output, int axis, int inst, const QkReduceStrategy *strategy,
              int dtype, void *stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!input || !output) return QK_ERR_NULL;
    if (inst != QK_REDUCE_MAXABS && inst != QK_REDUCE_MAX && inst != QK_REDUCE_MIN) return QK_ERR_UNSUPPORTED_SCHEME;
    const int fsize = dtype_size(dtype);
    if (fsize == 0) return QK_ERR_DTYPE;
    int rc;
    if ((rc = check_tensor(input, fsize))) return rc;
    if ((rc = check_tensor(output, fsize))) return rc;
    // validate_axis / valid_output_shape (crates/cubek-reduce/src/lib.rs:134-160)
    if (axis < 0 || axis >= input->rank) return QK_ERR_SHAPE;
    if (output->rank != input->rank) return QK_ERR_SHAPE;
    for (int d = 0; d < input->rank; ++d)
        if (output->shape[d] != (d == axis ? 1 : input->shape[d])) return QK_ERR_SHAPE;
    long long outer = 1, inner = 1;
    for (int d = 0; d < axis; ++d) outer *= input->shape[d];
    for (int d = axis + 1; d < input->rank; ++d) inner *= input->shape[d];
    const long long len = input->shape[axis];
    if (outer * inner == 0) return QK_OK;
    // `ReduceStrategy` (strategy.rs:7-16): shared -> a CTA per item, else planes -> a warp per item, else a thread
    int units = 0;
    if (strategy) units = strategy->shared ? 256 : (strategy->use_planes ? 32 : 1);
    const LaunchCfg cfg = current_cfg();
    count_launch();
    const int per16 = 16 / fsize;
    const bool contiguous = is_contiguous(input) && is_contiguous(output);
    const bool vectors_ok = inner == 1 || (inner % per16 == 0 && aligned(input->ptr, 16) && aligned(output->ptr, 16));
    if (contiguous && vectors_ok && !g_tune[TUNE_FORCE_GENERAL].load())
        return cuda_status(launch_reduce_contiguous(dtype, inst, input->ptr, output->ptr, outer, len, inner, units, cfg, stream));
    return cuda_status(launch_reduce_strided(dtype, inst, input, output, axis, cfg, stream));
}

int qk_reduce_maxabs(const QkTensor *input, const QkTensor *output, int axis, int dtype, void *stream)
{
    return qk_reduce(input, output, axis, QK_REDUCE_MAXABS, nullptr, dtype, stream);
}

int qk_absmax_f32(const QkTensor *input, int input_dtype, float *absmax_out, void *stream)
{
    if (!input || !absmax_out) return QK_ERR_NULL;
    const int fsize = dtype_size(input_dtype);
    if (fsize == 0) return QK_ERR_DTYPE;
    int rc = check_tensor(input, fsize);
    if (rc) return rc;
    if (!aligned(absmax_out, 4)) return QK_ERR_ALIGN;
    const long long n = numel(input);
    count_launch(n > 0 ? 2 : 1);
    return cuda_status(absmax_of(input, input_dtype, n, reinterpret_cast<unsigned int *>(absmax_out), current_cfg(),
                                 static_cast<cudaStream_t>(stream), true));
}

int qk_absmax_batch(int count, const QkTensor *inputs, int input_dtype, float *absmax_out, void *stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (count < 0) return QK_ERR_SHAPE;
    if (count == 0) return QK_OK;
    if (!inputs || !absmax_out) return QK_ERR_NULL;
    const int fsize = dtype_size(input_dtype);
    if (fsize == 0) return QK_ERR_DTYPE;
    if (!aligned(absmax_out, 4)) return QK_ERR_ALIGN;
    const LaunchCfg cfg = current_cfg();
    cudaError_t e = cudaMemsetAsync(absmax_out, 0, sizeof(float) * (size_t)count, stream);
    if (e != cudaSuccess) return cuda_status(e);
    count_launch();
    return absmax_into_cells(count, inputs, nullptr, input_dtype, reinterpret_cast<unsigned int *>(absmax_out), cfg, stream);
}

int qk_quantize_from_absmax_batch(int count, const QkTensor *inputs, const QkTensor *outputs, const QkTensor *out_scales,
                                  const float *absmax, const QkScheme *scheme, int input_dtype, void *stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (count < 0) return QK_ERR_SHAPE;
    if (count == 0) return QK_OK;
    if (!inputs || !outputs || !out_scales || !absmax || !scheme) return QK_ERR_NULL;
    if (scheme->level != QK_LEVEL_TENSOR) return QK_ERR_UNSUPPORTED_SCHEME;
    QuantBatch batch;
    for (int i = 0; i < count; ++i) {
        const int rc = quantize_common(&inputs[i], &outputs[i], nullptr, &out_scales[i], absmax + i, false, nullptr, scheme,
                                       input_dtype, stream, &batch);
        if (rc != QK_OK) {
            flush_quant(batch, current_cfg(), stream);
            return rc;
        }
    }
    return flush_quant(batch, current_cfg(), stream);
}

int qk_quantize_from_absmax(const QkTensor *input, const QkTensor *output, const QkTensor *out_scale,
                            const float *absmax, const QkScheme *scheme, int input_dtype, void *stream)
{
    if (!absmax || !scheme) return QK_ERR_NULL;
    if (scheme->level != QK_LEVEL_TENSOR) return QK_ERR_UNSUPPORTED_SCHEME;
    return quantize_common(input, output, nullptr, out_scale, absmax, false, nullptr, scheme, input_dtype,
                           static_cast<cudaStream_t>(stream));
}

// ---- NCCL, resolved at run time so that the library has no link-time NCCL dependency -----------
}  // extern "C"

namespace {

typedef int (*allreduce_fn)(const void *, void *, size_t, int, int, void *, void *);
typedef int (*async_error_fn)(void *, int *);
typedef int (*stream_query_fn)(void *);

std::atomic<allreduce_fn> g_allreduce{nullptr};
std::atomic<async_error_fn> g_async_error{nullptr};
std::atomic<stream_query_fn> g_stream_query{nullptr};
std::atomic<bool> g_hooks_set{false};

int real_stream_query(void *stream) { return (int)cudaStreamQuery(static_cast<cudaStream_t>(stream)); }

void *nccl_symbol(const char *name)
{
    void *sym = dlsym(RTLD_DEFAULT, name);
    if (!sym) {
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (h) sym = dlsym(h, name);
    }
    return sym;
}

bool resolve_collectives()
{
    if (g_allreduce.load() && g_async_error.load() && g_stream_query.load()) return true;
    if (g_hooks_set.load()) return false;   // hooks are installed as a complete set
    void *ar = nccl_symbol("ncclAllReduce");
    void *ae = nccl_symbol("ncclCommGetAsyncError");
    if (!ar || !ae) return false;
    g_allreduce.store(reinterpret_cast<allreduce_fn>(ar));
    g_async_error.store(reinterpret_cast<async_error_fn>(ae));
    g_stream_query.store(real_stream_query);
    return true;
}

constexpr int kNcclSuccess = 0, kNcclInProgress = 7;   // nccl.h: ncclResult_t
constexpr int kCudaNotReady = 600;                     // cudaErrorNotReady

// Enqueue, then (wait_done) poll until the stream has drained.  `timeout_ms` bounds every wait.
int allreduce_max(float *buf, size_t count, void *comm, void *stream, int timeout_ms, bool wait_done)
{
    if (!buf || !comm) return QK_ERR_NULL;
    if (!resolve_collectives()) return QK_ERR_NCCL;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
    const auto expired = [&] { return std::chrono::steady_clock::now() >= deadline; };
    // ncclFloat32 = 7, ncclMax = 2 (nccl.h: ncclDataType_t, ncclRedOp_t)
    int rc = g_allreduce.load()(buf, buf, count, 7, 2, comm, stream);
    while (rc == kNcclInProgress) {   // non-blocking communicator: the enqueue itself is still pending
        int state = kNcclSuccess;
        if (g_async_error.load()(comm, &state) != kNcclSuccess) return QK_ERR_NCCL;
        if (state == kNcclSuccess) { rc = kNcclSuccess; break; }
        if (state != kNcclInProgress) return QK_ERR_NCCL;
        if (expired()) return QK_ERR_TIMEOUT;
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    if (rc != kNcclSuccess) return QK_ERR_NCCL;
    if (!wait_done) return QK_OK;
    for (;;) {
        int state = kNcclSuccess;
        if (g_async_error.load()(comm, &state) != kNcclSuccess) return QK_ERR_NCCL;
        if (state != kNcclSuccess && state != kNcclInProgress) return QK_ERR_NCCL;
        const int q = g_stream_query.load()(stream);
        if (q == 0) return QK_OK;
        if (q != kCudaNotReady) return QK_ERR_CUDA + q;
        if (expired()) return QK_ERR_TIMEOUT;
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

}  // namespace

extern "C" {

int qk_allreduce_max_f32(float *buf, size_t count, void *comm, void *stream)
{
    return allreduce_max(buf, count, comm, stream, 10000, false);
}

int qk_allreduce_max_f32_deadline(float *buf, size_t count, void *comm, void *stream, int timeout_ms)
{
    return allreduce_max(buf, count, comm, stream, timeout_ms, true);
}

void qk_testing_set_collective_hooks(int (*allreduce)(const void *, void *, size_t, int, int, void *, void *),
                                     int (*async_error)(void *, int *), int (*stream_query)(void *))
{
    const bool set = allreduce && async_error && stream_query;
    g_hooks_set.store(set);
    g_allreduce.store(set ? allreduce : nullptr);
    g_async_error.store(set ? async_error : nullptr);
    g_stream_query.store(set ? stream_query : nullptr);
}

int qk_into_contiguous_packed(const QkTensor *input, const QkTensor *output, const int64_t *shape, int rank, int packing,
                              void *stream)
{
    if (!input || !output || !shape) return QK_ERR_NULL;
    if (rank < 1 || rank > QK_MAX_RANK || input->rank != rank || output->rank != rank) return QK_ERR_SHAPE;
    if (input->elem_size != output->elem_size || (input->elem_size != 4 && input->elem_size != 1)) return QK_ERR_DTYPE;
    const int item_bits = input->elem_size * 8;
    if (packing < 1 || item_bits % packing != 0) return QK_ERR_SHAPE;
    int rc;
    if ((rc = check_tensor(input, input->elem_size))) return rc;
    if ((rc = check_tensor(output, output->elem_size))) return rc;
    // The packing of the input runs along its contiguous dim (the last one of stride 1 among dims of extent > 1).
    int packed_dim = rank - 1;
    for (int d = rank - 1; d >= 0; --d)
        if (input->strides[d] == 1 && input->shape[d] != 1) { packed_dim = d; break; }
    RepackArgs a;
    a.rank = rank;
    a.packed_dim = packed_dim;
    a.packing = packing;
    a.bits = item_bits / packing;
    a.item_bytes = input->elem_size;
    a.nitems_out = 1;
    for (int d = 0; d < QK_MAX_RANK; ++d) {
        a.shape[d] = d < rank ? shape[d] : 1;
        a.in_strides[d] = d < rank ? input->strides[d] : 0;
        if (d >= rank) continue;
        if (shape[d] < 0) return QK_ERR_SHAPE;
        const long long in_want = (d == packed_dim) ? (shape[d] + packing - 1) / packing : shape[d];
        const long long out_want = (d == rank - 1) ? (shape[d] + packing - 1) / packing : shape[d];
        if (input->shape[d] != in_want || output->shape[d] != out_want) return QK_ERR_SHAPE;
        a.nitems_out *= out_want;
    }
    if (!is_contiguous(output)) return QK_ERR_LAYOUT;
    if (a.nitems_out == 0) return QK_OK;
    a.in = input->ptr;
    a.out = output->ptr;
    count_launch();
    return cuda_status(launch_repack(a, current_cfg(), static_cast<cudaStream_t>(stream)));
}

const char *qk_strerror(int status)
{
    switch (status) {
    case QK_OK: return "ok";
    case QK_ERR_UNSUPPORTED_SCHEME: return "unsupported quantization scheme";
    case QK_ERR_BLOCK_SIZE: return "block size must be non-zero, fit the tensor rank and be divisible by num_quants";
    case QK_ERR_SHAPE: return "shape mismatch (last dim must be a multiple of num_quants; scales must hold one value per block)";
    case QK_ERR_DTYPE: return "element size does not match the declared element type";
    case QK_ERR_LAYOUT: return "tensor layout not supported by this entry point";
    case QK_ERR_ALIGN: return "pointer is not aligned to its element size";
    case QK_ERR_NULL: return "null argument";
    case QK_ERR_WORKSPACE: return "workspace missing or too small";
    case QK_ERR_TOO_LARGE: return "size beyond what this entry point supports";
    case QK_ERR_NCCL: return "NCCL call failed, communicator in error, or NCCL not found";
    case QK_ERR_TIMEOUT: return "deadline passed before the collective completed";
    case QK_ERR_DEVICE: return "a kernel gave up on a bounded wait and left its output unwritten";
    default:
        if (status >= QK_ERR_CUDA) return cudaGetErrorString((cudaError_t)(status - QK_ERR_CUDA));
        return "unknown status";
    }
}

#ifdef QK_ROUND_HALF_AWAY
const char *qk_version(void) { return "cubek-quant-b200 0.2.0 (sm_100a, round half away from zero)"; }
#else
const char *qk_version(void) { return "cubek-quant-b200 0.2.0 (sm_100a)"; }
#endif

uint64_t qk_launch_count(void) { return g_launches.load(); }

int qk_device_error(int *flag_out)
{
    if (!flag_out) return QK_ERR_NULL;
    int *p = stage_error_flag();
    if (!p) return QK_ERR_CUDA;
    cudaError_t e = cudaMemcpy(flag_out, p, sizeof(int), cudaMemcpyDeviceToHost);   // synchronises
    if (e != cudaSuccess) return cuda_status(e);
    if (*flag_out != 0) e = cudaMemset(p, 0, sizeof(int));                          // read and clear
    return cuda_status(e);
}

void qk_set_tuning(int key, int value)
{
    if (key >= 0 && key < TUNE_COUNT) g_tune[key].store(value);
}
int qk_get_tuning(int key) { return (key >= 0 && key < TUNE_COUNT) ? g_tune[key].load() : -1; }

}  // extern "C"

namespace qk {

// Shared body of qk_quantize / qk_quantize_dynamic / qk_quantize_from_absmax.
static int quantize_common(const QkTensor *input, const QkTensor *output, const QkTensor *scale,
                           const QkTensor *out_scale, const float *absmax, bool dynamic, void *gen_scales,
                           const QkScheme *scheme, int input_dtype, cudaStream_t stream, QuantBatch *batch)
{
    if (!input || !output || !out_scale || !scheme) return QK_ERR_NULL;
    int rc = check_scheme(scheme);
    if (rc) return rc;
    const int fsize = dtype_size(input_dtype);
    if (fsize == 0) return QK_ERR_DTYPE;
    if ((rc = check_tensor(input, fsize))) return rc;
    if ((rc = check_tensor(output, scheme->store == QK_STORE_U32 ? 4 : 1))) return rc;
    if (scale && (rc = check_tensor(scale, fsize))) return rc;
    if ((rc = check_tensor(out_scale, dtype_size(scheme->param)))) return rc;
    Geometry g;
    if ((rc = build_geometry(g, scheme, input, output))) return rc;
    // check_block_size_compat (crates/cubek-quant/src/lib.rs:20-33)
    if (!g.per_tensor && g.B % g.nq != 0) return QK_ERR_BLOCK_SIZE;
    if (scale && (rc = check_scales_shape(g, scale))) return rc;
    if ((rc = check_scales_shape(g, out_scale))) return rc;
    // Both tensors may be strided: the reference reaches them through `linear_view` (quantize.rs:311, :316).
    if (g.n == 0) return QK_OK;

    float lo, hi;
    qk_value_range(scheme->value, &lo, &hi);
    const LaunchCfg cfg = current_cfg();
    int unit_bytes = 0, sub = 1;
    const int lg = fast_quantize_lg(g, input_dtype, input, output, scale, out_scale, &unit_bytes, &sub, dynamic,
                                    scheme->param);
    // Tiles over two dims cannot be reduced inside one thread group: the fused form first writes the
    // tile scales (one warp per tile) into the workspace, then runs the given-scale kernel.
    const void *tile_scales = nullptr;
    if (lg >= -1 && g.blocks_2d && dynamic) {
        const int per16 = 16 / fsize;
        if (!gen_scales) return QK_ERR_WORKSPACE;
        if (g.B % per16 == 0) {
            if (batch && (rc = flush_quant(*batch, cfg, stream))) return rc;
            count_launch();
            const cudaError_t e = launch_block_scales_2d(input_dtype, input->ptr, gen_scales, g.n / g.cols, g.cols,
                                                         (int)g.block_rows, (int)g.B, hi - lo, 1.0f / (hi - lo), cfg, stream);
            if (e != cudaSuccess) return cuda_status(e);
            tile_scales = gen_scales;
            dynamic = false;
        }
    }
    if (lg >= -1 && !(g.blocks_2d && dynamic)) {
        QuantBatch local;
        QuantBatch &b = batch ? *batch : local;
        const bool symmetric = (lo == -hi);
        const bool clamp = need_clamp(input_dtype, g.kind, dynamic, symmetric, scheme->param);
        const long long nunits = g.n / (unit_bytes / fsize);
        long long row_stride = 0;
        const bool strided_rows = !is_contiguous(input) && is_row_strided(input, &row_stride);
        const int a32 = (aligned(input->ptr, 32) && aligned(output->ptr, 32) &&
                         (!strided_rows || (row_stride * fsize) % 32 == 0)) ? 1 : 0;
        // A tensor joins the pending launch only if it needs the very same kernel and constants;
        // per-tensor absmax cells must be consecutive (the kernel indexes them by tensor).
        const bool joins = !g.blocks_2d && !b.a.b2.enabled &&   // tile geometry is per launch
                           !strided_rows && !b.a.rs.enabled &&  // and so is a row stride
                           b.a.ntensors > 0 && b.a.ntensors < QK_MAX_BATCH && b.fdt == input_dtype &&
                           b.kind == g.kind && b.unit_bytes == unit_bytes && b.sub == sub && b.dyn == dynamic && b.clamp == clamp &&
                           b.a.lg_units_per_block == lg && b.a.param == scheme->param && b.a.lo == lo && b.a.hi == hi &&
                           b.a.force_exact == cfg.force_exact &&
                           ((absmax == nullptr && b.a.absmax == nullptr) ||
                            (absmax != nullptr && b.a.absmax != nullptr && absmax == b.a.absmax + b.a.ntensors));
        if (!joins) {
            if ((rc = flush_quant(b, cfg, stream))) return rc;
            b.fdt = input_dtype;
            b.kind = g.kind;
            b.unit_bytes = unit_bytes;
            b.sub = sub;
            b.dyn = dynamic;
            b.clamp = clamp;
            b.a.absmax = absmax;
            b.a.lg_units_per_block = lg;
            b.a.param = scheme->param;
            b.a.lo = lo;
            b.a.hi = hi;
            b.a.range = hi - lo;
            b.a.inv_range = 1.0f / (hi - lo);
            b.a.force_exact = cfg.force_exact;
            b.a.aligned32 = 1;
            b.a.b2 = make_blocks2d(g, unit_bytes / fsize, lg);
            b.a.rs.enabled = strided_rows ? 1 : 0;
            b.a.rs.units_per_row = make_fastdiv(strided_rows ? (unsigned)(g.shape[g.rank - 1] / (unit_bytes / fsize)) : 1u);
            b.a.rs.row_bytes = strided_rows ? row_stride * fsize : 0;
        }
        QuantTensor &t = b.a.t[b.a.ntensors];
        t.in = input->ptr;
        t.out = output->ptr;
        t.scale_in = tile_scales ? tile_scales : (scale ? scale->ptr : nullptr);
        t.out_scale = out_scale->ptr;
        b.a.nunits += nunits;
        t.unit_end = b.a.nunits;
        const long long tile_units = QK_TILE_BYTES / unit_bytes;
        t.tile_end = (b.a.ntensors ? b.a.t[b.a.ntensors - 1].tile_end : 0) + (nunits + tile_units - 1) / tile_units;
        b.a.aligned32 &= a32;
        b.a.ntensors += 1;
        return batch ? QK_OK : flush_quant(b, cfg, stream);
    }
    if (batch && (rc = flush_quant(*batch, cfg, stream))) return rc;

    // Transposed matrix views: units gathered across memory rows, coalesced over the logical rows.
    long long ld = 0;
    if (!g_tune[TUNE_FORCE_GENERAL].load() && is_contiguous(output) && is_transposed_matrix(input, &ld) && !g.blocks_2d &&
        (g.per_tensor || (g.last_dim_blocks && is_contiguous(out_scale) && (!scale || is_contiguous(scale)))) &&
        !(dynamic && g.per_tensor)) {
        for (int ub = 64; ub >= 32; ub >>= 1) {
            if (ub < min_unit_bytes(input_dtype, g.kind)) break;
            const long long U = ub / fsize;
            // a block is 1, 2, 4 or 8 units: the warps of one tile row of the kernel
            int lgb = -1;
            if (!g.per_tensor) {
                lgb = (g.B % U == 0) ? log2_exact(g.B / U) : -1;
                if (lgb < 0 || lgb > 3) continue;
            }
            if (g.shape[1] % U != 0) continue;
            const int out_words = (int)(U / kind_elems_per_u32(g.kind));
            if (!aligned(output->ptr, out_words >= 4 ? 16 : 4 * out_words)) continue;
            if (g.n / U >= (1ll << 31) || g.shape[0] >= (1ll << 31)) continue;
            QuantBatch one;
            one.a.ntensors = 1;
            one.a.nunits = g.n / U;
            one.a.absmax = absmax;
            one.a.lg_units_per_block = lgb;
            one.a.param = scheme->param;
            one.a.lo = lo;
            one.a.hi = hi;
            one.a.range = hi - lo;
            one.a.inv_range = 1.0f / (hi - lo);
            one.a.force_exact = cfg.force_exact;
            one.a.aligned32 = aligned(output->ptr, 32) ? 1 : 0;
            one.a.nunits = fill_transposed_tiles(one.a.tr, input, ld, fsize, U);   // the kernel walks tiles
            one.a.t[0].in = input->ptr;
            one.a.t[0].out = output->ptr;
            one.a.t[0].scale_in = scale ? scale->ptr : nullptr;
            one.a.t[0].out_scale = out_scale->ptr;
            one.a.t[0].unit_end = one.a.nunits;
            one.a.t[0].tile_end = 0;
            // always clamped here: the clamp also keeps a NaN element inside its own code
            const bool clamp = true;
            count_launch();
            return cuda_status(launch_quantize_transposed(input_dtype, g.kind, ub, dynamic, clamp, one.a, cfg, stream));
        }
    }

    // Layout-general route.
    GeneralQuantArgs a;
    const void *scale_ptr = scale ? scale->ptr : nullptr;
    QkTensor staged;
    int64_t staged_strides[QK_MAX_RANK], staged_shape[QK_MAX_RANK];
    if (dynamic) {
        // Scales are computed first into caller-provided workspace (contiguous, F-typed).
        if (!gen_scales) return QK_ERR_WORKSPACE;
        int64_t st = 1;
        for (int d = g.rank - 1; d >= 0; --d) {
            staged_shape[d] = (g.shape[d] + g.block[d] - 1) / g.block[d];
            staged_strides[d] = st;
            st *= staged_shape[d];
        }
        staged.ptr = gen_scales;
        staged.rank = g.rank;
        staged.shape = staged_shape;
        staged.strides = staged_strides;
        staged.elem_size = fsize;
        GeneralScalesArgs sa;
        fill_layout(sa.layout, g, &staged, nullptr, input);
        sa.in = input->ptr;
        sa.scale_out = gen_scales;
        sa.nblocks = g.nscales;
        sa.fdt = input_dtype;
        sa.range = hi - lo;
        count_launch();
        cudaError_t e = launch_general_scales(sa, cfg, stream);
        if (e != cudaSuccess) return cuda_status(e);
        scale_ptr = gen_scales;
        fill_layout(a.layout, g, &staged, out_scale, input, output);
    } else {
        fill_layout(a.layout, g, scale, out_scale, input, output);
    }
    a.in = input->ptr;
    a.out = output->ptr;
    a.scale_in = scale_ptr;
    a.out_scale = out_scale->ptr;
    a.absmax = absmax;
    a.nitems = g.n / g.nq;
    a.nq = g.nq;
    a.kind = g.kind;
    a.fdt = input_dtype;
    a.param = scheme->param;
    a.lo = lo;
    a.hi = hi;
    a.range = hi - lo;
    count_launch();
    return cuda_status(launch_general_quantize(a, cfg, stream));
}

// Shared body of qk_dequantize / qk_dequantize_batch.
static int dequantize_common(const QkTensor *values, const QkTensor *output, const QkTensor *params,
                             const QkScheme *scheme, int output_dtype, cudaStream_t stream, DequantBatch *batch)
{
    if (!values || !output || !params || !scheme) return QK_ERR_NULL;
    int rc = check_scheme(scheme);
    if (rc) return rc;
    const int fsize = dtype_size(output_dtype);
    if (fsize == 0) return QK_ERR_DTYPE;
    if ((rc = check_tensor(output, fsize))) return rc;
    if ((rc = check_tensor(values, scheme->store == QK_STORE_U32 ? 4 : 1))) return rc;
    if ((rc = check_tensor(params, dtype_size(scheme->param)))) return rc;
    Geometry g;
    if ((rc = build_geometry(g, scheme, output, values))) return rc;
    if ((rc = check_scales_shape(g, params))) return rc;
    if (g.n == 0) return QK_OK;

    const LaunchCfg cfg = current_cfg();
    int out_bytes = 0, sub = 1;
    const int lg = fast_dequantize_lg(g, output_dtype, values, output, params, &out_bytes, &sub, scheme->param);
    if (lg >= -1) {
        DequantBatch local;
        DequantBatch &b = batch ? *batch : local;
        long long row_stride = 0;
        const bool strided_rows = !is_contiguous(output) && is_row_strided(output, &row_stride);
        const bool joins = !g.blocks_2d && !b.a.b2.enabled && !strided_rows && !b.a.rs.enabled &&
                           b.a.ntensors > 0 && b.a.ntensors < QK_MAX_BATCH && b.fdt == output_dtype &&
                           b.kind == g.kind && b.out_bytes == out_bytes && b.sub == sub && b.a.lg_units_per_block == lg &&
                           b.a.param == scheme->param;
        if (!joins) {
            if ((rc = flush_dequant(b, cfg, stream))) return rc;
            b.fdt = output_dtype;
            b.kind = g.kind;
            b.out_bytes = out_bytes;
            b.sub = sub;
            b.a.lg_units_per_block = lg;
            b.a.param = scheme->param;
            b.a.aligned32 = 1;
            b.a.b2 = make_blocks2d(g, out_bytes / fsize, lg);
            b.a.rs.enabled = strided_rows ? 1 : 0;
            b.a.rs.units_per_row = make_fastdiv(strided_rows ? (unsigned)(g.shape[g.rank - 1] / (out_bytes / fsize)) : 1u);
            b.a.rs.row_bytes = strided_rows ? row_stride * fsize : 0;
        }
        DequantTensor &t = b.a.t[b.a.ntensors];
        t.values = values->ptr;
        t.params = params->ptr;
        t.out = output->ptr;
        b.a.nunits += g.n / (out_bytes / fsize);
        t.unit_end = b.a.nunits;
        b.a.aligned32 &= (aligned(output->ptr, 32) && (!strided_rows || (row_stride * fsize) % 32 == 0)) ? 1 : 0;
        b.a.ntensors += 1;
        return batch ? QK_OK : flush_dequant(b, cfg, stream);
    }
    if (batch && (rc = flush_dequant(*batch, cfg, stream))) return rc;
    long long ld = 0;
    if (!g_tune[TUNE_FORCE_GENERAL].load() && is_contiguous(values) && is_transposed_matrix(output, &ld) && !g.blocks_2d &&
        (g.per_tensor || (g.last_dim_blocks && is_contiguous(params)))) {
        for (int ob = 64; ob >= 32; ob >>= 1) {
            if (ob < min_dequant_bytes(output_dtype, g.kind)) break;
            const long long E = ob / fsize;
            int lgb = -1;
            if (!g.per_tensor) {
                lgb = (g.B % E == 0) ? log2_exact(g.B / E) : -1;
                if (lgb < 0 || lgb > 3) continue;
            }
            if (g.shape[1] % E != 0) continue;
            const int in_words = (int)(E / kind_elems_per_u32(g.kind));
            if (!aligned(values->ptr, 4 * (in_words >= 4 ? 4 : in_words))) continue;
            if (g.n / E >= (1ll << 31) || g.shape[0] >= (1ll << 31)) continue;
            DequantBatch one;
            one.a.ntensors = 1;
            one.a.nunits = g.n / E;
            one.a.lg_units_per_block = lgb;
            one.a.param = scheme->param;
            one.a.aligned32 = 0;
            const bool pairs = fsize == 2 && g.shape[0] % 2 == 0 && ld % 2 == 0 && aligned(output->ptr, 4);
            one.a.tr.enabled = 1;
            one.a.tr.pairs = pairs ? 1 : 0;
            one.a.tr.rows = make_fastdiv((unsigned)(pairs ? g.shape[0] / 2 : g.shape[0]));
            one.a.tr.nrows = (unsigned)g.shape[0];
            one.a.tr.ld = ld;
            one.a.tr.units_per_row = (unsigned)(g.shape[1] / E);
            if (pairs) one.a.nunits /= 2;     // work items; every item writes two units
            one.a.t[0].values = values->ptr;
            one.a.t[0].params = params->ptr;
            one.a.t[0].out = output->ptr;
            one.a.t[0].unit_end = one.a.nunits;
            count_launch();
            return cuda_status(launch_dequantize_transposed(output_dtype, g.kind, ob, one.a, cfg, stream));
        }
    }
    GeneralDequantArgs a;
    fill_layout(a.layout, g, params, nullptr, output, values);
    a.values = values->ptr;
    a.params = params->ptr;
    a.out = output->ptr;
    a.nitems = g.n / g.nq;
    a.nq = g.nq;
    a.kind = g.kind;
    a.fdt = output_dtype;
    a.param = scheme->param;
    count_launch();
    return cuda_status(launch_general_dequantize(a, cfg, stream));
}

// Per tensor in one cooperative launch (absmax, grid barrier, quantize; second pass served from
// L2).  Returns QK_ERR_TOO_LARGE when the route does not apply (geometry, workspace, tuning) and
// the caller should take the two-kernel route; any other status is final.
static int try_quantize_tensor_coop(const QkTensor *input, const QkTensor *output, const QkTensor *out_scale,
                                    const QkScheme *scheme, int input_dtype, void *workspace, size_t workspace_bytes,
                                    cudaStream_t stream)
{
    if (!g_tune[TUNE_COOP_TENSOR].load() || g_tune[TUNE_FORCE_GENERAL].load()) return QK_ERR_TOO_LARGE;
    if (!input || !output || !out_scale) return QK_ERR_NULL;
    const int fsize = dtype_size(input_dtype);
    int rc;
    if ((rc = check_tensor(input, fsize))) return rc;
    if ((rc = check_tensor(output, scheme->store == QK_STORE_U32 ? 4 : 1))) return rc;
    if ((rc = check_tensor(out_scale, dtype_size(scheme->param)))) return rc;
    Geometry g;
    if ((rc = build_geometry(g, scheme, input, output))) return rc;
    if ((rc = check_scales_shape(g, out_scale))) return rc;
    if (!is_contiguous(input) || !is_contiguous(output)) return QK_ERR_TOO_LARGE;
    const int U = 64 / fsize;
    if (g.n == 0 || g.n % U != 0 || !aligned(input->ptr, 16) || !aligned(output->ptr, 16) || !aligned(workspace, 4))
        return QK_ERR_TOO_LARGE;
    // Measured against absmax + quantize as two launches: 24 vs 32 us at 64 MiB, 50 vs 53 at 112 MiB, 91 vs 95 at
    // 256 MiB, 217 vs 212 at 512 MiB (the second pass comes from HBM there and the two-launch route has more CTAs).
    if ((size_t)g.n * fsize > (size_t)g_tune[TUNE_COOP_MAX_MIB].load() << 20) return QK_ERR_TOO_LARGE;
    float lo, hi;
    qk_value_range(scheme->value, &lo, &hi);
    const LaunchCfg cfg = current_cfg();
    QuantTensorArgs a;
    a.in = input->ptr;
    a.out = output->ptr;
    a.out_scale = out_scale->ptr;
    a.partials = static_cast<float *>(workspace);
    a.nunits = g.n / U;
    a.param = scheme->param;
    a.lo = lo;
    a.hi = hi;
    a.range = hi - lo;
    a.inv_range = 1.0f / (hi - lo);
    a.force_exact = cfg.force_exact;
    a.aligned32 = (aligned(input->ptr, 32) && aligned(output->ptr, 32)) ? 1 : 0;
    const cudaError_t e = launch_quantize_tensor(input_dtype, g.kind, a, (int)(workspace_bytes / sizeof(float)), cfg, stream);
    if (e == cudaErrorInvalidValue) {
        (void)cudaGetLastError();
        return QK_ERR_TOO_LARGE;   // workspace smaller than the resident grid: two-kernel route
    }
    count_launch();
    return cuda_status(e);
}

}  // namespace qk
