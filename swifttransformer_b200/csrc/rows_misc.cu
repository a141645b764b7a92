// Small row-wise kernels.
//
// concat_rows:   out[r] = [ a[r] | b[r] ] in the activation type (a: float or the activation type, width wa; b: wb).
// scale_softcap: x <- cap * tanh(x * scale / cap) in place on float rows (cap <= 0: x <- x * scale).
#include "common.cuh"

template <typename TA, typename T>
__global__ void concat_rows_kernel(const TA* __restrict__ a, int wa, const T* __restrict__ b, int wb, T* __restrict__ out,
                                   size_t total) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int w = wa + wb;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / w;
        const int e = (int)(i % w);
        out[i] = e < wa ? from_f32<T>(load1_cg(a + r * wa + e)) : from_f32<T>(load1_cg(b + r * wb + (e - wa)));
    }
}

ST_EXPORT int st_concat_rows(const void* a, int a_f32, int wa, const void* b, int wb, void* out, int n_rows, int dtype,
                             void* stream) {
    if (n_rows <= 0) return 0;
    const size_t total = (size_t)n_rows * (wa + wb);
    int grid = (int)((total + 255) / 256);
    if (grid > st_sm_count() * 16) grid = st_sm_count() * 16;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0)
        return st_launch_pdl("concat_rows", concat_rows_kernel<float, float>, dim3(grid), dim3(256), 0, s, (const float*)a, wa,
                             (const float*)b, wb, (float*)out, total);
    if (dtype != 1) return ST_ERR_BAD_DTYPE;
    if (a_f32)
        return st_launch_pdl("concat_rows", concat_rows_kernel<float, bf16>, dim3(grid), dim3(256), 0, s, (const float*)a, wa,
                             (const bf16*)b, wb, (bf16*)out, total);
    return st_launch_pdl("concat_rows", concat_rows_kernel<bf16, bf16>, dim3(grid), dim3(256), 0, s, (const bf16*)a, wa,
                         (const bf16*)b, wb, (bf16*)out, total);
}

__global__ void scale_softcap_kernel(float* __restrict__ x, size_t total, float scale, float cap) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float v = __ldcg(x + i) * scale;
        x[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
    }
}

ST_EXPORT int st_scale_softcap(float* x, long long total, float scale, float cap, void* stream) {
    if (total <= 0) return 0;
    int grid = (int)((total + 255) / 256);
    if (grid > st_sm_count() * 16) grid = st_sm_count() * 16;
    return st_launch_pdl("scale_softcap", scale_softcap_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, x,
                         (size_t)total, scale, cap);
}
