// Gated linear recurrence with the forget gate tied to the input gate (the HGRN2 form), per head:
//
//   S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T        S: [dim, vd] float, kept per request
//   o_t = S_t^T q_t
//   f_t = lower + (1 - lower) * sigmoid(z_t + bias)    per head and channel
//   q_t = silu(projection)
//   out_t = o_t / sqrt(mean(o_t^2) + eps) * weight      over the head's vd values
//
// One block per (request of the step, head) owns that head's state for the whole launch: it loads it,
// walks through the request's tokens of this step in order and stores it back.  Tokens are taken in groups
// of GROUP: all threads prepare the group's gates and queries (float arithmetic on the projection's
// values), then thread j carries column j of S through the group's tokens without meeting the others, and
// the group's outputs are normalised a warp per token.
#include "common.cuh"

#define HG_GROUP 16

template <typename T>
__global__ void __launch_bounds__(1024)
hgrn2_scan_kernel(const T* __restrict__ proj, int ld, int q_off, int f_off, int v_off,
                  const float* __restrict__ f_bias, const float* __restrict__ lower,
                  const float* __restrict__ norm_w, float eps, float* __restrict__ state, T* __restrict__ out,
                  const int* __restrict__ positions, const int* __restrict__ q_start,
                  const int* __restrict__ slots, int nh, int dim, int vd) {
    extern __shared__ float smem[];
    const int b = blockIdx.x, h = blockIdx.y;
    const int first = q_start[b], n = q_start[b + 1] - first;
    // padding of a fixed-shape step: a request without tokens, or one whose tokens stand at position -1
    if (n <= 0 || positions[first] < 0) return;
    float* S = smem;                                      // [dim][vd]
    float* sq = S + (size_t)dim * vd;                     // [GROUP][dim]
    float* sf = sq + HG_GROUP * dim;                      // [GROUP][dim]
    float* sv = sf + HG_GROUP * dim;                      // [GROUP][vd]
    float* so = sv + HG_GROUP * vd;                       // [GROUP][vd]
    float* st = state + ((size_t)slots[b] * nh + h) * dim * vd;
    const int tid = threadIdx.x, nt = blockDim.x;
    for (int e = tid; e < dim * vd; e += nt) S[e] = st[e];
    const int lane = tid & 31, warp = tid >> 5, nwarp = nt >> 5;
    for (int r0 = 0; r0 < n; r0 += HG_GROUP) {
        const int rn = min(HG_GROUP, n - r0);
        __syncthreads();                                  // the group before has been written out
        for (int e = tid; e < rn * dim; e += nt) {
            const int k = e / dim, i = e % dim;
            const T* row = proj + (size_t)(first + r0 + k) * ld;
            const float zq = to_f32(row[q_off + h * dim + i]);
            const float zf = to_f32(row[f_off + h * dim + i]) + f_bias[h * dim + i];
            const float lo = lower[h * dim + i];
            sq[e] = zq / (1.f + expf(-zq));
            sf[e] = lo + (1.f - lo) * (1.f / (1.f + expf(-zf)));
        }
        for (int e = tid; e < rn * vd; e += nt) {
            const int k = e / vd, j = e % vd;
            sv[e] = to_f32(proj[(size_t)(first + r0 + k) * ld + v_off + h * vd + j]);
        }
        __syncthreads();
        for (int j = tid; j < vd; j += nt) {
            for (int k = 0; k < rn; ++k) {
                const float v = sv[k * vd + j];
                const float* f = sf + k * dim;
                const float* qq = sq + k * dim;
                float o = 0.f;
                for (int i = 0; i < dim; ++i) {
                    const float s = fmaf(f[i], S[i * vd + j], (1.f - f[i]) * v);
                    S[i * vd + j] = s;
                    o = fmaf(s, qq[i], o);
                }
                so[k * vd + j] = o;
            }
        }
        __syncthreads();
        for (int k = warp; k < rn; k += nwarp) {
            float ss = 0.f;
            for (int j = lane; j < vd; j += 32) ss += so[k * vd + j] * so[k * vd + j];
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)vd + eps);
            T* orow = out + ((size_t)(first + r0 + k) * nh + h) * vd;
            for (int j = lane; j < vd; j += 32) orow[j] = from_f32<T>(so[k * vd + j] * inv * norm_w[j]);
        }
    }
    __syncthreads();
    for (int e = tid; e < dim * vd; e += nt) st[e] = S[e];
}

static size_t hgrn2_smem(int dim, int vd) {
    return ((size_t)dim * vd + 2 * HG_GROUP * dim + 2 * HG_GROUP * vd) * sizeof(float);
}

// proj: [tokens, ld] with the query, gate and value projections at column offsets q_off, f_off, v_off
// state: [slots, nh, dim, vd] float; out: [tokens, nh * vd]
ST_EXPORT int st_hgrn2_scan(const void* proj, int ld, int q_off, int f_off, int v_off, const float* f_bias,
                            const float* lower, const float* norm_w, float eps, float* state, void* out,
                            const int* positions, const int* q_start, const int* slots, int n_seqs, int nh, int dim,
                            int vd, int dtype, void* stream) {
    if (n_seqs <= 0) return 0;
    if (nh <= 0 || dim <= 0 || vd <= 0) return ST_ERR_BAD_ARG;
    const size_t smem = hgrn2_smem(dim, vd);
    if (smem > 200 * 1024) return ST_ERR_TOO_LARGE;
    int threads = (vd + 31) / 32 * 32;
    if (threads < 128) threads = 128;
    if (threads > 1024) threads = 1024;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_seqs, nh);
#define HG_LAUNCH(T)                                                                                                  \
    do {                                                                                                              \
        if (smem > 48 * 1024) {                                                                                       \
            cudaError_t e = cudaFuncSetAttribute(hgrn2_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                                 (int)smem);                                                          \
            if (e != cudaSuccess) return (int)e;                                                                      \
        }                                                                                                             \
        hgrn2_scan_kernel<T><<<grid, threads, smem, s>>>((const T*)proj, ld, q_off, f_off, v_off, f_bias, lower,      \
                                                         norm_w, eps, state, (T*)out, positions, q_start, slots, nh, dim, vd); \
    } while (0)
    if (dtype == 0) HG_LAUNCH(float);
    else if (dtype == 1) HG_LAUNCH(bf16);
    else return ST_ERR_BAD_DTYPE;
#undef HG_LAUNCH
    return st_launch_status();
}
