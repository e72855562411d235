// Round trip through host buffers: slices of whole rows travel host -> device, are quantized
// (fused absmax + scale + pack) and dequantized on the device, and codes, scales and restored
// values travel back.  Four staging slots on four streams overlap the copies in both
// directions with the kernels.  This is the call a host-resident caller of the reference's
// test flow makes (create_tensor_from_slice -> quantize -> dequantize -> read_one_tensor,
// crates/cubek-quant/tests/suite/symmetric.rs:32-127), as one entry point.
#include <mutex>

#include "../../include/cubek_quant_b200_testing.h"
#include "common.cuh"
#include "misc_kernels.cuh"

namespace qk {
int *stage_error_flag();   // device address of the flag the staged kernels raise (api.cu)
}

namespace {

constexpr int kMaxSlots = 8;
// Staging slots in flight (tuning key 10, default 4) and input bytes per slice (key 9, KiB; 0, the default, sizes
// slices by the call: a sixteenth of the input bytes of all its tensors, between 16 and 64 MiB).
// Every slice costs about 30 us of copy set-up (one upload, three downloads), and the first slice's upload and the
// last one's downloads are overlapped with nothing.  On a 117 MB bf16 tensor 1 / 4 / 8 / 16 MiB slices took
// 5.8 / 4.2 / 3.7 / 3.6 ms, against 3.3 ms for the downloads alone at the link's rate with both directions busy;
// on 1.74 GB (28 tensors) 16 / 32 / 64 MiB slices took 55.7 / 53.8 / 52.6 ms against 51.5 ms for the copies alone.
int slot_count()
{
    const int v = qk_get_tuning(10);
    return v < 1 ? 1 : (v > kMaxSlots ? kMaxSlots : v);
}
size_t slice_target_bytes(size_t total_input_bytes)
{
    const int kib = qk_get_tuning(9);
    if (kib > 0) return (size_t)(kib < 64 ? 64 : kib) << 10;
    const size_t lo = (size_t)16 << 20, hi = (size_t)64 << 20;
    const size_t t = total_input_bytes / 16;
    return t < lo ? lo : (t > hi ? hi : t);
}
size_t total_input_bytes(int count, const QkTensor *inputs, int fsize)
{
    size_t total = 0;
    for (int i = 0; i < count; ++i) {
        if (!inputs[i].shape || inputs[i].rank < 1 || inputs[i].rank > QK_MAX_RANK) continue;
        size_t n = 1;
        for (int d = 0; d < inputs[i].rank; ++d) n *= (size_t)(inputs[i].shape[d] > 0 ? inputs[i].shape[d] : 0);
        total += n * (size_t)fsize;
    }
    return total;
}

struct DeviceStreams {
    cudaStream_t stream[kMaxSlots] = {};
    bool ready = false;
};
DeviceStreams g_streams[64];
std::mutex g_streams_mutex;

int dtype_size(int dt) { return dt == QK_F32 ? 4 : (dt == QK_F16 || dt == QK_BF16) ? 2 : 0; }

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Plan {
    int ok = 0;
    long long rows = 0, cols = 0;       // input viewed as rows x cols (cols = last dim)
    long long slice_rows = 0;           // rows per slice
    long long scales_per_row = 0;       // sliced block schemes: scales in one row
    long long slice_scales = 1;         // scales held by one slice (whole tensor when unsliced)
    bool sliced = false;
    int nq = 0;
    size_t in_row = 0, code_row = 0, scale_row = 0, out_row = 0;  // bytes per row
    size_t slot_bytes = 0, in_off = 0, code_off = 0, scale_off = 0, out_off = 0, ws_off = 0;
    bool per_tensor = false;
};

// Slices are whole rows; for block schemes the blocks must lie along the last dim and divide it,
// so that no block straddles a slice.  Anything else runs as a single slice.
Plan make_plan(const QkTensor *input, const QkScheme *scheme, int input_dtype, size_t slice_target)
{
    Plan p;
    const int fsize = dtype_size(input_dtype);
    p.nq = qk_num_quants(scheme);
    if (!input || !input->shape || input->rank < 1 || input->rank > QK_MAX_RANK || fsize == 0 || p.nq == 0) return p;
    p.cols = input->shape[input->rank - 1];
    p.rows = 1;
    for (int d = 0; d < input->rank - 1; ++d) p.rows *= input->shape[d];
    if (p.cols <= 0 || p.rows <= 0 || p.cols % p.nq) return p;
    p.per_tensor = scheme->level == QK_LEVEL_TENSOR;
    bool sliceable = !p.per_tensor;
    if (!p.per_tensor) {
        const int br = scheme->block_rank;
        if (br < 1 || br > input->rank) return p;
        for (int i = 0; i < br - 1; ++i) sliceable = sliceable && scheme->block[i] == 1;
        const long long B = scheme->block[br - 1];
        if (B == 0) return p;
        sliceable = sliceable && (p.cols % B == 0);
        p.scales_per_row = (p.cols + B - 1) / B;
        if (!sliceable) {
            // N-d blocks: one slice, scales counted over the whole tensor.
            long long ns = 1;
            for (int d = 0; d < input->rank; ++d) {
                const int bi = d - (input->rank - br);
                const long long b = bi >= 0 ? scheme->block[bi] : 1;
                ns *= (input->shape[d] + b - 1) / b;
            }
            p.slice_scales = ns;
        }
    }
    p.in_row = (size_t)p.cols * fsize;
    p.code_row = (size_t)(p.cols / p.nq) * (scheme->store == QK_STORE_U32 ? 4 : 1);
    p.scale_row = (size_t)p.scales_per_row * dtype_size(scheme->param);
    p.out_row = p.in_row;
    if (sliceable) {
        p.slice_rows = (long long)(slice_target / p.in_row);
        if (p.slice_rows < 1) p.slice_rows = 1;
        if (p.slice_rows > p.rows) p.slice_rows = p.rows;
        p.slice_scales = p.scales_per_row * p.slice_rows;
        p.sliced = p.slice_rows < p.rows;
    } else {
        p.slice_rows = p.rows;
    }
    p.in_off = 0;
    p.code_off = align_up(p.in_off + p.in_row * p.slice_rows, 256);
    p.scale_off = align_up(p.code_off + p.code_row * p.slice_rows, 256);
    p.out_off = align_up(p.scale_off + (size_t)p.slice_scales * dtype_size(scheme->param), 256);
    p.ws_off = align_up(p.out_off + p.out_row * p.slice_rows, 256);
    // workspace: absmax cell (+ staged scales for general layouts)
    size_t ws_bytes = 256 + (size_t)p.slice_scales * fsize;
    if (ws_bytes < qk_workspace_bytes()) ws_bytes = qk_workspace_bytes();
    p.slot_bytes = align_up(p.ws_off + ws_bytes, 256);
    p.ok = 1;
    return p;
}

}  // namespace

extern "C" {

size_t qk_host_roundtrip_staging_bytes(const QkTensor *input, const QkScheme *scheme, int input_dtype)
{
    return qk_host_roundtrip_staging_bytes_batch(1, input, scheme, input_dtype);
}

size_t qk_host_roundtrip_staging_bytes_batch(int count, const QkTensor *inputs, const QkScheme *scheme, int input_dtype)
{
    if (!scheme || !inputs || count < 1) return 0;
    size_t slot = 0;
    bool sliced = false;
    long long nslices = 0;
    const size_t slice_target = slice_target_bytes(total_input_bytes(count, inputs, dtype_size(input_dtype)));
    for (int i = 0; i < count; ++i) {
        const Plan p = make_plan(&inputs[i], scheme, input_dtype, slice_target);
        if (!p.ok) return 0;
        if (p.slot_bytes > slot) slot = p.slot_bytes;
        sliced = sliced || p.sliced;
        nslices += (p.rows + p.slice_rows - 1) / p.slice_rows;
    }
    const int slots = (nslices > 1) ? slot_count() : 1;
    return slot * slots;
}

int qk_roundtrip_host(const QkTensor *input, const QkTensor *codes, const QkTensor *out_scale,
                      const QkTensor *restored, const QkScheme *scheme, int input_dtype, void *staging,
                      size_t staging_bytes, int device)
{
    if (!input || !codes || !out_scale || !restored) return QK_ERR_NULL;
    return qk_roundtrip_host_batch(1, input, codes, out_scale, restored, scheme, input_dtype, staging, staging_bytes, device);
}

int qk_roundtrip_host_batch(int count, const QkTensor *inputs, const QkTensor *codes, const QkTensor *out_scales,
                            const QkTensor *restored, const QkScheme *scheme, int input_dtype, void *staging,
                            size_t staging_bytes, int device)
{
    if (count < 0) return QK_ERR_SHAPE;
    if (count == 0) return QK_OK;
    if (!inputs || !codes || !out_scales || !restored || !scheme || !staging) return QK_ERR_NULL;
    if (device < 0 || device >= 64) return QK_ERR_SHAPE;
    if (count > 4096) return QK_ERR_TOO_LARGE;
    // Every tensor's slices pass through the same ring of staging slots, so the upload of one tensor's first slice
    // overlaps the downloads of the previous tensor's last ones (tensors of one slice would otherwise run
    // upload, kernels and download strictly one after the other).
    size_t slot_bytes = 0;
    long long nslices = 0;
    const size_t slice_target = slice_target_bytes(total_input_bytes(count, inputs, dtype_size(input_dtype)));
    for (int i = 0; i < count; ++i) {
        const Plan p = make_plan(&inputs[i], scheme, input_dtype, slice_target);
        if (!p.ok) return QK_ERR_SHAPE;
        if (!inputs[i].ptr || !codes[i].ptr || !out_scales[i].ptr || !restored[i].ptr) return QK_ERR_NULL;
        if (p.slot_bytes > slot_bytes) slot_bytes = p.slot_bytes;
        nslices += (p.rows + p.slice_rows - 1) / p.slice_rows;
    }
    const int slots = (nslices > 1) ? slot_count() : 1;
    if (staging_bytes < slot_bytes * slots) return QK_ERR_WORKSPACE;

    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return QK_ERR_CUDA + (int)e;
    cudaStream_t *streams;
    {
        std::lock_guard<std::mutex> lock(g_streams_mutex);
        DeviceStreams &ds = g_streams[device];
        if (!ds.ready) {
            for (int i = 0; i < kMaxSlots; ++i) {
                e = cudaStreamCreateWithFlags(&ds.stream[i], cudaStreamNonBlocking);
                if (e != cudaSuccess) return QK_ERR_CUDA + (int)e;
            }
            ds.ready = true;
        }
        streams = ds.stream;
    }

    const int fsize = dtype_size(input_dtype);
    const int psize = dtype_size(scheme->param);
    const int csize = scheme->store == QK_STORE_U32 ? 4 : 1;
    int status = QK_OK;
    long long slice = 0;
    for (int ti = 0; ti < count && status == QK_OK; ++ti) {
        const QkTensor *input = &inputs[ti];
        const Plan p = make_plan(input, scheme, input_dtype, slice_target);
        const int rank = input->rank;
        for (long long r0 = 0; r0 < p.rows && status == QK_OK; r0 += p.slice_rows, ++slice) {
            const long long nr = (p.rows - r0 < p.slice_rows) ? p.rows - r0 : p.slice_rows;
            const int slot = (int)(slice % slots);
            cudaStream_t st = streams[slot];
            char *base = static_cast<char *>(staging) + (size_t)slot * slot_bytes;

            // The slot's previous work is ordered before this slice by stream order.
            e = cudaMemcpyAsync(base + p.in_off, static_cast<const char *>(input->ptr) + (size_t)r0 * p.in_row,
                                (size_t)nr * p.in_row, cudaMemcpyHostToDevice, st);
            if (e != cudaSuccess) { status = QK_ERR_CUDA + (int)e; break; }

            // Device views of this slice.  A sliced tensor is [nr, cols]; a single slice keeps the
            // caller's shape so that N-d blocks still apply.
            int64_t shp_in[QK_MAX_RANK], shp_code[QK_MAX_RANK], shp_scale[QK_MAX_RANK];
            int64_t str_in[QK_MAX_RANK], str_code[QK_MAX_RANK], str_scale[QK_MAX_RANK];
            int vr;
            QkScheme sch = *scheme;
            if (!p.sliced) {
                vr = rank;
                for (int d = 0; d < rank; ++d) {
                    shp_in[d] = input->shape[d];
                    shp_code[d] = codes[ti].shape[d];
                }
                if (p.per_tensor) { shp_scale[0] = 1; }
                else for (int d = 0; d < rank; ++d) shp_scale[d] = out_scales[ti].shape[d];
            } else {
                vr = 2;
                shp_in[0] = nr; shp_in[1] = p.cols;
                shp_code[0] = nr; shp_code[1] = p.cols / p.nq;
                shp_scale[0] = nr; shp_scale[1] = p.scales_per_row;
                sch.block_rank = 1;
                sch.block[0] = scheme->block[scheme->block_rank - 1];
            }
            const int sr = p.per_tensor ? 1 : vr;
            auto fill_strides = [](int64_t *str, const int64_t *shp, int r) {
                int64_t acc = 1;
                for (int d = r - 1; d >= 0; --d) { str[d] = acc; acc *= shp[d]; }
            };
            fill_strides(str_in, shp_in, vr);
            fill_strides(str_code, shp_code, vr);
            fill_strides(str_scale, shp_scale, sr);
            QkTensor t_in{base + p.in_off, vr, shp_in, str_in, fsize};
            QkTensor t_code{base + p.code_off, vr, shp_code, str_code, csize};
            QkTensor t_scale{base + p.scale_off, sr, shp_scale, str_scale, psize};
            QkTensor t_out{base + p.out_off, vr, shp_in, str_in, fsize};

            status = qk_quantize_dynamic(&t_in, &t_code, &t_scale, &sch, input_dtype, base + p.ws_off,
                                         p.slot_bytes - p.ws_off, st);
            if (status != QK_OK) break;
            status = qk_dequantize(&t_code, &t_out, &t_scale, &sch, input_dtype, st);
            if (status != QK_OK) break;

            e = cudaMemcpyAsync(static_cast<char *>(codes[ti].ptr) + (size_t)r0 * p.code_row, base + p.code_off,
                                (size_t)nr * p.code_row, cudaMemcpyDeviceToHost, st);
            if (e == cudaSuccess) {
                const size_t sbytes = p.sliced ? (size_t)nr * p.scale_row : (size_t)p.slice_scales * psize;
                const size_t soff = p.sliced ? (size_t)r0 * p.scale_row : 0;
                e = cudaMemcpyAsync(static_cast<char *>(out_scales[ti].ptr) + soff, base + p.scale_off, sbytes,
                                    cudaMemcpyDeviceToHost, st);
            }
            if (e == cudaSuccess)
                e = cudaMemcpyAsync(static_cast<char *>(restored[ti].ptr) + (size_t)r0 * p.out_row, base + p.out_off,
                                    (size_t)nr * p.out_row, cudaMemcpyDeviceToHost, st);
            if (e != cudaSuccess) status = QK_ERR_CUDA + (int)e;
        }
    }
    for (int i = 0; i < slots; ++i) {
        e = cudaStreamSynchronize(streams[i]);
        if (e != cudaSuccess && status == QK_OK) status = QK_ERR_CUDA + (int)e;
    }
    // The results are claimed to be in host memory: a kernel that gave up on a bounded wait must not pass silently.
    // (Read on one of the internal streams: a copy on the default stream would wait for other threads' work.)
    if (status == QK_OK) {
        int flag = 0;
        int *dev_flag = qk::stage_error_flag();
        if (dev_flag) {
            e = cudaMemcpyAsync(&flag, dev_flag, sizeof(int), cudaMemcpyDeviceToHost, streams[0]);
            if (e == cudaSuccess) e = cudaStreamSynchronize(streams[0]);
            if (e != cudaSuccess) status = QK_ERR_CUDA + (int)e;
            else if (flag != 0) status = QK_ERR_DEVICE;
        }
    }
    return status;
}

}  // extern "C"
