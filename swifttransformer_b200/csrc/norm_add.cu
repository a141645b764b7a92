// Two elementwise kernels of blocks that normalise a sub-layer's OUTPUT before the residual sum, and of
// gated feed-forwards.
//
// norm_add:   x[r] += mult * gain * y[r] / sqrt(mean(y[r]^2) + eps)      (gain: one number, read from the device)
//             optionally act[r] = x[r] in the activation type, for the sub-layer that reads x next.
//             x is the float residual stream; statistics and the sum are float for every storage type.
// gated_act:  out[r][j] = act(gu[r][j]) * gu[r][inner + j]               (gu = the fused gate | up product)
#include "common.cuh"

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
norm_add_kernel(float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ gain, float mult, float eps,
                int width, const int* __restrict__ positions, TO* __restrict__ act) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    if (positions && positions[r] < 0) return;          // padding token of a fixed-shape step
    const T* yr = y + (size_t)r * width;
    float* xr = x + (size_t)r * width;
    float ss = 0.f;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        const float v = to_f32(yr[e]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float k = rsqrtf(ss / (float)width + eps) * gain[0] * mult;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        const float v = xr[e] + k * to_f32(yr[e]);
        xr[e] = v;
        if (act) act[(size_t)r * width + e] = from_f32<TO>(v);
    }
}

ST_EXPORT int st_norm_add(float* x, const void* y, const float* gain, float mult, float eps, int n_rows, int width,
                          const int* positions, void* act, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) return ST_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    int block = (width + 31) / 32 * 32;
    if (block > 256) block = 256;
    if (dtype == 0)
        norm_add_kernel<float, float><<<n_rows, block, 0, s>>>(x, (const float*)y, gain, mult, eps, width, positions, (float*)act);
    else if (dtype == 1)
        norm_add_kernel<bf16, bf16><<<n_rows, block, 0, s>>>(x, (const bf16*)y, gain, mult, eps, width, positions, (bf16*)act);
    else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, int inner, size_t total, int act) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t r = i / inner, j = i % inner;
        const T* row = gu + r * 2 * inner;
        out[i] = from_f32<T>(apply_act(to_f32(row[j]), act) * to_f32(row[inner + j]));
    }
}

ST_EXPORT int st_gated_act(const void* gu, void* out, int n_rows, int inner, int act, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (inner <= 0 || act < 0 || act > 4) return ST_ERR_BAD_ARG;
    const size_t total = (size_t)n_rows * inner;
    int grid = (int)((total + 255) / 256);
    if (grid > st_sm_count() * 16) grid = st_sm_count() * 16;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0) gated_act_kernel<float><<<grid, 256, 0, s>>>((const float*)gu, (float*)out, inner, total, act);
    else if (dtype == 1) gated_act_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)gu, (bf16*)out, inner, total, act);
    else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}
