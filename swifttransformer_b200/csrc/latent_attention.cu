// Latent attention over a paged cache of per-token latents.
//
// Per token the cache holds one row [c | k_rot]: c, the RMS-normed latent of kr numbers, and k_rot, a rotated key
// part of `rot` numbers shared by all heads.  Head h's keys and values are linear maps of c (k_h = Uk_h c,
// v_h = Uv_h c); the kernels here work in the latent space: the query of head h arrives already multiplied by
// Uk_h^T (kr numbers) followed by its own rotated part, so that
//
//   s_j   = scale * (q_lat . c_j + q_rot . k_rot_j)                  over the keys j <= the query's position
//   p     = exp(s_j - m) / (sum_j exp(s_j - m) + exp(sink_h - m))    the sink has no key and no value
//   o_lat = gate * sum_j p_j c_j                                     gate = sigmoid of the head's gate logit
//
// and head h's result is Uv_h o_lat, a product the caller does for all tokens at once.
//
// latent_prepare:  from the fused projection [dq | dkv | gates] of the step's tokens: RMS norm of the query latent
//                  (out, in the activation type), RMS norm of the key/value latent and rotation of the shared key
//                  part by position, both written to the token's page.
// latent_q_rotate: rotation of every head's rotated query part into the latent-space query rows.
// latent_attention_plain: one block per (token, head), float arithmetic for either storage type, key tiles
//                  aligned to absolute positions: a row's result does not depend on how the request was cut
//                  into steps or on what else is in the batch.
//
// Rotation ("halves" layout): of the first rot_dims dimensions, i is paired with i + rot_dims/2 and the pair
// (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * inv_freq[i], angle in float.
#include "latent_attention.cuh"

#define LP_THREADS 128

template <typename T>
__global__ void __launch_bounds__(LP_THREADS)
latent_prepare_kernel(const T* __restrict__ proj, int ld, int q_rank, const float* __restrict__ q_w,
                      const float* __restrict__ kv_w, float eps, const float* __restrict__ inv_freq, int rot_dims,
                      T* __restrict__ cq, T* __restrict__ pool, LatentCache cache, const int* __restrict__ positions,
                      const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                      const int* __restrict__ block_table, int write_kv, int* __restrict__ status) {
    __shared__ float scratch[32];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    const int pos = positions[t];
    if (pos < 0) return;
    const T* row = proj + (size_t)t * ld;
    const int kr = cache.kr, rot = cache.rot;
    float ss = 0.f;
    for (int e = threadIdx.x; e < q_rank; e += LP_THREADS) {
        const float v = load1_cg(row + e);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float rq = rsqrtf(ss / (float)q_rank + eps);
    for (int e = threadIdx.x; e < q_rank; e += LP_THREADS)
        cq[(size_t)t * q_rank + e] = from_f32<T>(load1_cg(row + e) * rq * q_w[e]);
    if (!write_kv) return;
    const T* kv = row + q_rank;
    ss = 0.f;
    for (int e = threadIdx.x; e < kr; e += LP_THREADS) {
        const float v = load1_cg(kv + e);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float rk = rsqrtf(ss / (float)kr + eps);
    const int page = block_table[(size_t)slots[seq_of_token[t]] * cache.max_pages + pos / cache.page_size];
    if (page < 0) {
        if (status && threadIdx.x == 0) *status = 1;
        return;
    }
    T* dst = latent_row(pool, cache, page, pos % cache.page_size);
    for (int e = threadIdx.x; e < kr; e += LP_THREADS) dst[e] = from_f32<T>(load1_cg(kv + e) * rk * kv_w[e]);
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += LP_THREADS) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        const float u = load1_cg(kv + kr + i), v = load1_cg(kv + kr + i + half);
        dst[kr + i] = from_f32<T>(u * cs - v * sn);
        dst[kr + i + half] = from_f32<T>(v * cs + u * sn);
    }
    for (int e = rot_dims + threadIdx.x; e < rot; e += LP_THREADS) dst[kr + e] = kv[kr + e];
}

ST_EXPORT int st_latent_prepare(const void* proj, int ld, int q_rank, const float* q_w, const float* kv_w, float eps,
                                const float* inv_freq, int rot_dims, void* cq, void* pool, long long page_stride,
                                long long entry_offset, const int* positions, const int* seq_of_token,
                                const int* slots, const int* block_table, int max_pages, int n_tokens, int kr, int rot,
                                int page_size, int write_kv, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (q_rank <= 0 || kr <= 0 || rot < 0 || rot_dims < 0 || rot_dims > rot || rot_dims % 2) return ST_ERR_BAD_SIZE;
    LatentCache c{max_pages, page_size, kr, rot, page_stride, entry_offset};
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0)
        return st_launch_pdl("latent_prepare", latent_prepare_kernel<float>, dim3(n_tokens), dim3(LP_THREADS), 0, s,
                             (const float*)proj, ld, q_rank, q_w, kv_w, eps, inv_freq, rot_dims, (float*)cq, (float*)pool,
                             c, positions, seq_of_token, slots, block_table, write_kv, status);
    if (dtype == 1)
        return st_launch_pdl("latent_prepare", latent_prepare_kernel<bf16>, dim3(n_tokens), dim3(LP_THREADS), 0, s,
                             (const bf16*)proj, ld, q_rank, q_w, kv_w, eps, inv_freq, rot_dims, (bf16*)cq, (bf16*)pool, c,
                             positions, seq_of_token, slots, block_table, write_kv, status);
    return ST_ERR_BAD_DTYPE;
}

// q: [tokens, nh * (dim + rot)] as the up-projection left it; q_lat: [tokens, nh, kr + rot], whose last `rot`
// numbers per head this kernel writes (the first kr are the product of the head's unrotated part with Uk_h).
template <typename T>
__global__ void __launch_bounds__(LP_THREADS)
latent_q_rotate_kernel(const T* __restrict__ q, T* __restrict__ q_lat, const int* __restrict__ positions,
                       const float* __restrict__ inv_freq, int rot_dims, int nh, int dim, int rot, int kr) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    const int pos = positions[t];
    if (pos < 0) return;
    const int half = rot_dims / 2, per = half + (rot - rot_dims);
    for (int i = threadIdx.x; i < nh * per; i += LP_THREADS) {
        const int h = i / per, j = i % per;
        const T* src = q + ((size_t)t * nh + h) * (dim + rot) + dim;
        T* dst = q_lat + ((size_t)t * nh + h) * (kr + rot) + kr;
        if (j < half) {
            float sn, cs;
            sincosf((float)pos * inv_freq[j], &sn, &cs);
            const float u = load1_cg(src + j), v = load1_cg(src + j + half);
            dst[j] = from_f32<T>(u * cs - v * sn);
            dst[j + half] = from_f32<T>(v * cs + u * sn);
        } else {
            dst[rot_dims + j - half] = src[rot_dims + j - half];
        }
    }
}

ST_EXPORT int st_latent_q_rotate(const void* q, void* q_lat, const int* positions, const float* inv_freq, int rot_dims,
                                 int n_tokens, int nh, int dim, int rot, int kr, int dtype, void* stream) {
    if (n_tokens <= 0 || rot <= 0) return 0;
    if (rot_dims < 0 || rot_dims > rot || rot_dims % 2) return ST_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0)
        return st_launch_pdl("latent_q_rotate", latent_q_rotate_kernel<float>, dim3(n_tokens), dim3(LP_THREADS), 0, s,
                             (const float*)q, (float*)q_lat, positions, inv_freq, rot_dims, nh, dim, rot, kr);
    if (dtype == 1)
        return st_launch_pdl("latent_q_rotate", latent_q_rotate_kernel<bf16>, dim3(n_tokens), dim3(LP_THREADS), 0, s,
                             (const bf16*)q, (bf16*)q_lat, positions, inv_freq, rot_dims, nh, dim, rot, kr);
    return ST_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------------------------------------
#define LKT 128          // keys per tile = threads per block
#define LVMAX 8          // latent dimensions per thread: kr <= LKT * LVMAX

template <typename T>
__global__ void __launch_bounds__(LKT)
latent_attention_plain_kernel(const T* __restrict__ q_lat, const T* __restrict__ pool, LatentCache cache,
                              T* __restrict__ out, const int* __restrict__ items, const int* __restrict__ positions,
                              const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                              const int* __restrict__ block_table, const float* __restrict__ sink,
                              const T* __restrict__ gates, int gate_ld, int nh, float scale, int* __restrict__ status) {
    extern __shared__ float smem[];
    float* sq = smem;                       // [kr + rot]
    float* sp = smem + cache.kr + cache.rot;  // [LKT]
    __shared__ float scratch[32];
    const int h = blockIdx.y;
    const float snk = sink ? sink[h] : -INFINITY;
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = items ? items[blockIdx.x] : blockIdx.x;
    if (t < 0) return;
    const int pos = positions[t];
    if (pos < 0) return;
    const int kr = cache.kr, kd = cache.kr + cache.rot, ps = cache.page_size;
    const int* bt = block_table + (size_t)slots[seq_of_token[t]] * cache.max_pages;
    for (int e = threadIdx.x; e < kd; e += LKT) sq[e] = load1_cg(q_lat + ((size_t)t * nh + h) * kd + e);
    __syncthreads();
    float acc[LVMAX];
#pragma unroll
    for (int c = 0; c < LVMAX; ++c) acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int hi = pos + 1;
    for (int base = 0; base < hi; base += LKT) {
        const int j = base + threadIdx.x;
        float sc = -INFINITY;
        if (j < hi) {
            const int page = bt[j / ps];
            if (page >= 0) {
                const T* krow = latent_row(pool, cache, page, j % ps);
                float d = 0.f;
                for (int e = 0; e < kd; ++e) d = fmaf(sq[e], load1_cg(krow + e), d);
                sc = d * scale;
            } else if (status) {
                *status = 1;
            }
        }
        const float n = fmaxf(m, block_max(sc, scratch));
        const float p = sc > -INFINITY ? expf(sc - n) : 0.f;
        const float corr = m == -INFINITY ? 0.f : expf(m - n);
        l = l * corr + block_sum(p, scratch);
        m = n;
        sp[threadIdx.x] = p;
        __syncthreads();
        const int j_end = min(LKT, hi - base);
#pragma unroll
        for (int c = 0; c < LVMAX; ++c) {
            const int e = threadIdx.x + c * LKT;
            if (e >= kr) continue;
            float x = acc[c] * corr;
            for (int jj = 0; jj < j_end; ++jj) {
                const int key = base + jj;
                const int page = bt[key / ps];
                if (page < 0) continue;
                x = fmaf(sp[jj], load1_cg(latent_row(pool, cache, page, key % ps) + e), x);
            }
            acc[c] = x;
        }
        __syncthreads();
    }
    // the sink: one more term in the denominator
    const float mf = fmaxf(m, snk);
    const float corr = m == -INFINITY ? 0.f : expf(m - mf);
    l = l * corr + (snk > -INFINITY ? expf(snk - mf) : 0.f);
    float g = 1.f;
    if (gates) g = 1.f / (1.f + expf(-load1_cg(gates + (size_t)t * gate_ld + h)));
    const float k = l > 0.f ? corr * g / l : 0.f;
#pragma unroll
    for (int c = 0; c < LVMAX; ++c) {
        const int e = threadIdx.x + c * LKT;
        if (e < kr) out[((size_t)t * nh + h) * kr + e] = from_f32<T>(acc[c] * k);
    }
}

// q_lat [tokens, nh, kr + rot]; out [tokens, nh, kr]; gates: the gate logit of (token t, head h) at gates[t * gate_ld + h]
// (null: no gate); sink [nh] float (null: none); items: the tokens to serve (-1: none), null: all of them.
ST_EXPORT int st_latent_attention_plain(const void* q_lat, const void* pool, long long page_stride, long long entry_offset,
                                        void* out, const int* items, const int* positions, const int* seq_of_token,
                                        const int* slots, const int* block_table, int max_pages, int n_tokens, int nh,
                                        int kr, int rot, int page_size, const float* sink, const void* gates, int gate_ld,
                                        float scale, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (kr <= 0 || rot < 0 || nh <= 0) return ST_ERR_BAD_SIZE;
    if (kr > LKT * LVMAX || nh > 65535) return ST_ERR_TOO_LARGE;
    LatentCache c{max_pages, page_size, kr, rot, page_stride, entry_offset};
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(kr + rot + LKT) * sizeof(float);
    const dim3 grid(n_tokens, nh);
    if (dtype == 0)
        return st_launch_pdl("latent_plain", latent_attention_plain_kernel<float>, grid, dim3(LKT), smem, s,
                             (const float*)q_lat, (const float*)pool, c, (float*)out, items, positions, seq_of_token, slots,
                             block_table, sink, (const float*)gates, gate_ld, nh, scale, status);
    if (dtype == 1)
        return st_launch_pdl("latent_plain", latent_attention_plain_kernel<bf16>, grid, dim3(LKT), smem, s,
                             (const bf16*)q_lat, (const bf16*)pool, c, (bf16*)out, items, positions, seq_of_token, slots,
                             block_table, sink, (const bf16*)gates, gate_ld, nh, scale, status);
    return ST_ERR_BAD_DTYPE;
}
