// Short causal convolutions over time, one filter per channel, with the last
// taps-1 inputs of every request kept in a state slot so that a request may
// arrive in portions cut anywhere.
//
//   y[t][c] = sum_j w[c][j] * u[t - taps + 1 + j][c]          (zeros before position 0)
//
// The state of a request holds the inputs at positions len-(taps-1) .. len-1
// in that order (zero where the position is negative: a fresh slot is all
// zeros, which is exactly "nothing before the sequence's start").
//
// Who may touch the state: within one launch the tokens of a request read the
// old state while its new state has to be written.  `conv_residual` gives the
// first token of a request in the step to the thread that also owns the
// request's state for that channel: it computes the outputs of the first
// taps-1 tokens itself (the only ones that read the state) and then writes the
// new state; all other threads read the step's own rows only.  A kernel that
// reads the state in many threads (the fused q/k/v preparation of
// diff_attention.cu) leaves it unchanged and is followed by
// `conv_state_update`, where one thread per (request, channel) reads all it
// needs before it writes.
#include "common.cuh"

#define CONV_MAX_TAPS 8

template <int V, typename T> __device__ __forceinline__ void load_v(const T* p, float* v) {
    // through L2 only: the rows were written by the kernel just before (see the note on programmatic launch)
    if (V == 4) { const float4 f = load4_cg(p); v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w; }
    else v[0] = load1_cg(p);
}
template <int V, typename T> __device__ __forceinline__ void store_v(T* p, const float* v) {
    if (V == 4) store4(p, make_float4(v[0], v[1], v[2], v[3]));
    else p[0] = from_f32<T>(v[0]);
}

// out[t][c] = (residual ? in[t][c] : 0) + conv(in)[t][c];  in: float residual rows or activations.
// A thread owns V neighbouring channels (V = 4: 16-byte accesses, channels % 4 == 0).
template <typename TI, typename TO, int V>
__global__ void __launch_bounds__(128)
conv_residual_kernel(const TI* __restrict__ in, const float* __restrict__ w, float* __restrict__ state,
                     TO* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                     const int* __restrict__ q_start, const int* __restrict__ slots, int channels, int taps,
                     int residual) {
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    const int t = blockIdx.x;
    float wv[V][CONV_MAX_TAPS];
    if (c < channels) {                                 // the filters: no kernel writes them, fetched before the wait
#pragma unroll
        for (int v = 0; v < V; ++v)
#pragma unroll
            for (int j = 0; j < CONV_MAX_TAPS; ++j)     // (constant bounds: the filters stay in registers)
                wv[v][j] = j < taps ? w[(size_t)(c + v) * taps + j] : 0.f;
    }
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    if (c >= channels || positions[t] < 0) return;      // padding token of a fixed-shape step
    const int b = seq_of_token[t];
    const int first = q_start[b], n = q_start[b + 1] - first, i = t - first;
    const int keep = taps - 1;
    if (i >= keep) {
        float y[V], x[V];
#pragma unroll
        for (int v = 0; v < V; ++v) y[v] = 0.f;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) {
            if (j < taps) {
                load_v<V>(in + (size_t)(t - keep + j) * channels + c, x);
#pragma unroll
                for (int v = 0; v < V; ++v) y[v] = fmaf(wv[v][j], x[v], y[v]);
            }
        }
#pragma unroll
        for (int v = 0; v < V; ++v) y[v] += residual ? x[v] : 0.f;      // x holds the token's own row (j = taps - 1)
        store_v<V>(out + (size_t)t * channels + c, y);
        return;
    }
    if (i != 0) return;                                 // done by the thread of the request's first token
    // u = old state followed by the first rows of the step: u[keep + k] is the step's token k
    float* st = state + (size_t)slots[b] * keep * channels + c;
    float u[2 * CONV_MAX_TAPS][V];
    const int m = n < keep ? n : keep;                  // tokens that read the state
    for (int j = 0; j < keep; ++j) load_v<V>(st + (size_t)j * channels, u[j]);
    for (int k = 0; k < m; ++k) load_v<V>(in + (size_t)(first + k) * channels + c, u[keep + k]);
    for (int k = 0; k < m; ++k) {
        float y[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
            y[v] = 0.f;      // (the filters once more from memory: indexing wv by a variable would move it out of registers)
            for (int j = 0; j < taps; ++j) y[v] = fmaf(w[(size_t)(c + v) * taps + j], u[k + j][v], y[v]);
            y[v] += residual ? u[keep + k][v] : 0.f;
        }
        store_v<V>(out + (size_t)(first + k) * channels + c, y);
    }
    // the last `keep` inputs of old state + all n rows
    for (int j = 0; j < keep; ++j) {
        const int src = n + j;                          // index into (state, rows of the step)
        float x[V];
        if (src < keep) {
#pragma unroll
            for (int v = 0; v < V; ++v) x[v] = u[src][v];
        } else {
            load_v<V>(in + (size_t)(first + src - keep) * channels + c, x);
        }
        store_v<V>(st + (size_t)j * channels, x);
    }
}

// state <- the last taps-1 rows of (state, the request's rows of this step), for every request of the step
template <typename TI>
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const TI* __restrict__ in, int ld, float* __restrict__ state,
                         const int* __restrict__ positions, const int* __restrict__ q_start,
                         const int* __restrict__ slots, int channels, int taps) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    const int first = q_start[b], n = q_start[b + 1] - first;
    // padding of a fixed-shape step: a request without tokens, or one whose tokens stand at position -1
    if (c >= channels || n <= 0 || positions[first] < 0) return;
    const int keep = taps - 1;
    float* st = state + (size_t)slots[b] * keep * channels + c;
    float v[CONV_MAX_TAPS];
    for (int j = 0; j < keep; ++j) {
        const int src = n + j;
        v[j] = src < keep ? st[(size_t)src * channels] : to_f32(in[(size_t)(first + src - keep) * ld + c]);
    }
    for (int j = 0; j < keep; ++j) st[(size_t)j * channels] = v[j];
}

// in: [n_tokens, channels] float (in_f32) or the storage type; out: [n_tokens, channels] storage type `dtype`
ST_EXPORT int st_conv_residual(const void* in, int in_f32, const float* w, float* state, void* out,
                               const int* positions, const int* seq_of_token, const int* q_start, const int* slots,
                               int n_tokens, int channels, int taps, int residual, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (channels <= 0 || taps < 1) return ST_ERR_BAD_ARG;
    if (taps > CONV_MAX_TAPS) return ST_ERR_TOO_LARGE;
    if (dtype != 0 && dtype != 1) return ST_ERR_BAD_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = channels % 4 == 0 && aligned16(in) && aligned16(out) && aligned16(state);
    const int per_block = vec ? 128 * 4 : 128;
    dim3 grid(n_tokens, (channels + per_block - 1) / per_block);
#define CONV_LAUNCH(TI, TO)                                                                                           \
    do {                                                                                                              \
        if (vec) return st_launch_pdl("conv", conv_residual_kernel<TI, TO, 4>, grid, dim3(128), 0, s, (const TI*)in, w, state, \
                                      (TO*)out, positions, seq_of_token, q_start, slots, channels, taps, residual);   \
        return st_launch_pdl("conv", conv_residual_kernel<TI, TO, 1>, grid, dim3(128), 0, s, (const TI*)in, w, state, \
                             (TO*)out, positions, seq_of_token, q_start, slots, channels, taps, residual);            \
    } while (0)
    if (dtype == 0) CONV_LAUNCH(float, float);
    else if (in_f32) CONV_LAUNCH(float, bf16);
    else CONV_LAUNCH(bf16, bf16);
#undef CONV_LAUNCH
}

// in: [rows, ld] of which the first `channels` columns are the convolution's inputs
ST_EXPORT int st_conv_state_update(const void* in, int ld, float* state, const int* positions, const int* q_start,
                                   const int* slots, int n_seqs, int channels, int taps, int dtype, void* stream) {
    if (n_seqs <= 0 || taps <= 1) return 0;
    if (channels <= 0 || ld < channels) return ST_ERR_BAD_ARG;
    if (taps > CONV_MAX_TAPS) return ST_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((channels + 255) / 256, n_seqs);
    if (dtype == 0) conv_state_update_kernel<float><<<grid, 256, 0, s>>>((const float*)in, ld, state, positions, q_start, slots, channels, taps);
    else if (dtype == 1) conv_state_update_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)in, ld, state, positions, q_start, slots, channels, taps);
    else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}
