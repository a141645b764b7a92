// Two elementwise kernels of blocks that normalise a sub-layer's OUTPUT before the residual sum, and of
// gated feed-forwards.
//
// norm_add:   x[r] += mult * gain * y[r] / sqrt(mean(y[r]^2) + eps)      (gain: one number, read from the device)
//             optionally act[r] = x[r] in the activation type, for the sub-layer that reads x next.
//             x is the float residual stream; statistics and the sum are float for every storage type.
// gated_act:  out[r][j] = act(gu[r][j]) * gu[r][inner + j]               (gu = the fused gate | up product)
#include "common.cuh"

template <typename T, typename TO, bool VEC>
__global__ void __launch_bounds__(256)
norm_add_kernel(float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ gain, float mult, float eps,
                int width, const int* __restrict__ positions, TO* __restrict__ act) {
    __shared__ float scratch[32];
    ST_PDL_TRIGGER();
    const int r = blockIdx.x;
    if (positions && positions[r] < 0) return;          // padding token of a fixed-shape step
    const T* yr = y + (size_t)r * width;
    float* xr = x + (size_t)r * width;
    float ss = 0.f;
    if (VEC) {
        for (int e = threadIdx.x * 4; e < width; e += blockDim.x * 4) {
            const float4 v = load4(yr + e);
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
    } else {
        for (int e = threadIdx.x; e < width; e += blockDim.x) {
            const float v = to_f32(yr[e]);
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float k = rsqrtf(ss / (float)width + eps) * gain[0] * mult;
    if (VEC) {
        for (int e = threadIdx.x * 4; e < width; e += blockDim.x * 4) {
            const float4 v = load4(yr + e), o = load4(xr + e);
            const float4 n = make_float4(o.x + k * v.x, o.y + k * v.y, o.z + k * v.z, o.w + k * v.w);
            store4(xr + e, n);
            if (act) store4(act + (size_t)r * width + e, n);
        }
    } else {
        for (int e = threadIdx.x; e < width; e += blockDim.x) {
            const float v = xr[e] + k * to_f32(yr[e]);
            xr[e] = v;
            if (act) act[(size_t)r * width + e] = from_f32<TO>(v);
        }
    }
}

ST_EXPORT int st_norm_add(float* x, const void* y, const float* gain, float mult, float eps, int n_rows, int width,
                          const int* positions, void* act, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) return ST_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = width % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(act);
    int block = ((vec ? width / 4 : width) + 31) / 32 * 32;
    if (block > 256) block = 256;
    if (dtype == 0) {
        if (vec) norm_add_kernel<float, float, true><<<n_rows, block, 0, s>>>(x, (const float*)y, gain, mult, eps, width, positions, (float*)act);
        else norm_add_kernel<float, float, false><<<n_rows, block, 0, s>>>(x, (const float*)y, gain, mult, eps, width, positions, (float*)act);
    } else if (dtype == 1) {
        if (vec) norm_add_kernel<bf16, bf16, true><<<n_rows, block, 0, s>>>(x, (const bf16*)y, gain, mult, eps, width, positions, (bf16*)act);
        else norm_add_kernel<bf16, bf16, false><<<n_rows, block, 0, s>>>(x, (const bf16*)y, gain, mult, eps, width, positions, (bf16*)act);
    } else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}

// VEC: inner % 8 == 0 and 16-byte aligned rows: eight outputs per thread
template <typename T, bool VEC>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, int inner, size_t total, int act) {
    ST_PDL_TRIGGER();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    if (VEC) {
        for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < total; i += stride * 8) {
            const size_t r = i / inner, j = i % inner;
            const T* row = gu + r * 2 * inner + j;
            const float4 g0 = load4(row), g1 = load4(row + 4), u0 = load4(row + inner), u1 = load4(row + inner + 4);
            store4(out + i, make_float4(apply_act(g0.x, act) * u0.x, apply_act(g0.y, act) * u0.y,
                                        apply_act(g0.z, act) * u0.z, apply_act(g0.w, act) * u0.w));
            store4(out + i + 4, make_float4(apply_act(g1.x, act) * u1.x, apply_act(g1.y, act) * u1.y,
                                            apply_act(g1.z, act) * u1.z, apply_act(g1.w, act) * u1.w));
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
            const size_t r = i / inner, j = i % inner;
            const T* row = gu + r * 2 * inner;
            out[i] = from_f32<T>(apply_act(to_f32(row[j]), act) * to_f32(row[inner + j]));
        }
    }
}

ST_EXPORT int st_gated_act(const void* gu, void* out, int n_rows, int inner, int act, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (inner <= 0 || act < 0 || act > 4) return ST_ERR_BAD_ARG;
    const size_t total = (size_t)n_rows * inner;
    const bool vec = inner % 8 == 0 && aligned16(gu) && aligned16(out);
    const size_t work = vec ? total / 8 : total;
    int grid = (int)((work + 255) / 256);
    if (grid > st_sm_count() * 16) grid = st_sm_count() * 16;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0) {
        if (vec) gated_act_kernel<float, true><<<grid, 256, 0, s>>>((const float*)gu, (float*)out, inner, total, act);
        else gated_act_kernel<float, false><<<grid, 256, 0, s>>>((const float*)gu, (float*)out, inner, total, act);
    } else if (dtype == 1) {
        if (vec) gated_act_kernel<bf16, true><<<grid, 256, 0, s>>>((const bf16*)gu, (bf16*)out, inner, total, act);
        else gated_act_kernel<bf16, false><<<grid, 256, 0, s>>>((const bf16*)gu, (bf16*)out, inner, total, act);
    } else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}
