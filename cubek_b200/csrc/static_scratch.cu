// qk_quantize_dynamic_noalloc: the fused quantize for callers that have no device memory to
// hand over as workspace and are not allowed to obtain any.
//
// The per-tensor path needs a few bytes of scratch on the device (the cell every CTA max-reduces
// its absmax into), and layouts that take the general kernels stage their scales there.  The
// ordinary entry point asks the caller for that workspace.  This one keeps it in a fixed array that
// is part of the library image, so the call path contains no allocation at all.
#include <mutex>

#include "common.cuh"

#define QK_STATIC_SCRATCH_BYTES (64 * 1024)

// One copy per GPU that loads the library, resident until the process exits.  Shared by every call
// on that GPU; it keeps whatever the previous call left in it.
static __device__ __align__(256) unsigned char g_static_scratch[QK_STATIC_SCRATCH_BYTES];

namespace {

std::mutex g_mutex;
void *g_scratch_address[64];
bool g_scratch_ready[64];

// `g_static_scratch` is only a stand-in on the host side: its device address has to be asked for,
// once per device, with that device current.
int scratch_of_current_device(void **out)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return QK_ERR_CUDA + (int)e;
    if (dev < 0 || dev >= 64) return QK_ERR_TOO_LARGE;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch_ready[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return QK_ERR_CUDA + (int)e;
        if (p == nullptr) return QK_ERR_NULL;
        g_scratch_address[dev] = p;
        g_scratch_ready[dev] = true;
    }
    *out = g_scratch_address[dev];
    return QK_OK;
}

}  // namespace

extern "C" {

size_t qk_noalloc_scratch_bytes(void) { return QK_STATIC_SCRATCH_BYTES; }

int qk_quantize_dynamic_noalloc(const QkTensor *input, const QkTensor *output, const QkTensor *out_scale,
                                const QkScheme *scheme, int input_dtype, void *stream)
{
    if (!input || !output || !out_scale || !scheme) return QK_ERR_NULL;
    void *scratch = nullptr;
    const int rc = scratch_of_current_device(&scratch);
    if (rc != QK_OK) return rc;
    // The absmax cell is re-zeroed by the per-tensor path on every call; staged scales are fully
    // rewritten before they are read.  Nothing else of the array's old contents is ever read.
    const int status = qk_quantize_dynamic(input, output, out_scale, scheme, input_dtype, scratch,
                                           QK_STATIC_SCRATCH_BYTES, stream);
    // The only way the fixed array can be too small: a layout that stages more scales than fit.
    return status == QK_ERR_WORKSPACE ? QK_ERR_TOO_LARGE : status;
}

}  // extern "C"
