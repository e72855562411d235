// Test kernel for include/cubek_quant_b200_device.cuh: every thread dequantizes one line of stored items
// with dequantize_symmetric_packed_values and writes the floats in element order.  Built into
// libdevice_api_probe.so by cubek_b200/build.py; used only by tests/test_gpu_device_api.py.
#include <cuda_runtime.h>

#include "../../include/cubek_quant_b200_device.cuh"

namespace cq = cubek_quant_b200;

template <typename F, typename FS, int VALUE, int STORE, int LINE>
__global__ void probe_kernel(const void *values, cq::ScalesView<FS> scales, F *out, long long nlines)
{
    using Item = typename cq::Stored<STORE>::type;
    constexpr int NQ = cq::num_quants(VALUE, STORE);
    const long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= nlines) return;
    F tmp[LINE * NQ];
    cq::dequantize_symmetric_packed_values<F, FS, VALUE, STORE, LINE>((uint32_t)p, static_cast<const Item *>(values), scales, tmp);
#pragma unroll
    for (int i = 0; i < LINE * NQ; ++i) out[p * LINE * NQ + i] = tmp[i];
}

struct Call {
    const void *values;
    const void *scales;
    void *out;
    long long nlines;
    const QkScheme *scheme;
    int rank;
    const int64_t *values_shape, *scales_strides;
    cudaStream_t stream;
};

template <typename F, typename FS, int VALUE, int STORE, int LINE> static int run(const Call &c)
{
    const cq::ScalesView<FS> view =
        cq::make_scales_view(static_cast<const FS *>(c.scales), *c.scheme, c.rank, c.values_shape, c.scales_strides);
    const int threads = 128;
    const long long blocks = (c.nlines + threads - 1) / threads;
    if (blocks == 0) return 0;
    probe_kernel<F, FS, VALUE, STORE, LINE><<<(unsigned)blocks, threads, 0, c.stream>>>(c.values, view, static_cast<F *>(c.out), c.nlines);
    return (int)cudaGetLastError();
}

template <typename F, typename FS, int VALUE, int STORE> static int by_line(const Call &c, int line)
{
    if (line == 1) return run<F, FS, VALUE, STORE, 1>(c);
    if (line == 4) return run<F, FS, VALUE, STORE, 4>(c);
    return -1;
}

template <typename F, typename FS> static int by_scheme(const Call &c, int line)
{
    const int v = c.scheme->value;
    if (c.scheme->store == QK_STORE_U32) {
        switch (v) {
        case QK_Q8F: return by_line<F, FS, QK_Q8F, QK_STORE_U32>(c, line);
        case QK_Q8S: return by_line<F, FS, QK_Q8S, QK_STORE_U32>(c, line);
        case QK_Q4F: return by_line<F, FS, QK_Q4F, QK_STORE_U32>(c, line);
        case QK_Q4S: return by_line<F, FS, QK_Q4S, QK_STORE_U32>(c, line);
        case QK_Q2F: return by_line<F, FS, QK_Q2F, QK_STORE_U32>(c, line);
        case QK_Q2S: return by_line<F, FS, QK_Q2S, QK_STORE_U32>(c, line);
        default: return -1;
        }
    }
    switch (v) {
    case QK_Q8F: case QK_Q8S: return by_line<F, FS, QK_Q8S, QK_STORE_NATIVE>(c, line);
    case QK_E2M1: return by_line<F, FS, QK_E2M1, QK_STORE_NATIVE>(c, line);
    case QK_E4M3: return by_line<F, FS, QK_E4M3, QK_STORE_NATIVE>(c, line);
    case QK_E5M2: return by_line<F, FS, QK_E5M2, QK_STORE_NATIVE>(c, line);
    default: return -1;
    }
}

// Returns 0, a cudaError_t, or -1 for a combination the probe was not built for.
extern "C" int probe_dequantize(const void *values, const void *scales, void *out, long long nlines, int line,
                                const QkScheme *scheme, int fdt, int rank, const int64_t *values_shape,
                                const int64_t *scales_strides, void *stream)
{
    const Call c{values, scales, out, nlines, scheme, rank, values_shape, scales_strides, static_cast<cudaStream_t>(stream)};
    const int p = scheme->param;
    if (fdt == QK_F32 && p == QK_F32) return by_scheme<float, float>(c, line);
    if (fdt == QK_F16 && p == QK_F32) return by_scheme<__half, float>(c, line);
    if (fdt == QK_BF16 && p == QK_F32) return by_scheme<__nv_bfloat16, float>(c, line);
    if (fdt == QK_F16 && p == QK_F16) return by_scheme<__half, __half>(c, line);
    if (fdt == QK_BF16 && p == QK_BF16) return by_scheme<__nv_bfloat16, __nv_bfloat16>(c, line);
    if (fdt == QK_F32 && p == QK_BF16) return by_scheme<float, __nv_bfloat16>(c, line);
    return -1;
}
