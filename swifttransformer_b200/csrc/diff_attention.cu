// Differential attention over a paged cache: every query head carries two
// score maps (two queries, two keys per key/value head) over one set of values.
//
//   s_a  = cap * tanh(scale * (q_a . k_a) / cap)          a = 1, 2   (cap <= 0: no cap)
//   p_a  = softmax of s_a over the visible keys
//   o    = p_1 V - lambda * p_2 V
//   out  = o / sqrt(mean(o^2) + eps) * out_scale           (over the head's value dimensions)
//
// Visible keys of the query at position p: lo..p with lo = floor(p / block) * block when the mask is
// block-diagonal (block > 0; blocks are counted from position 0 of the request), max(0, p - window + 1)
// with a window, else 0.
//
// Cache layout (one page of one cache entry; kd = 2 * dim, the two maps' keys side by side):
//   keys   [kv_head][position in page][kd]     at offset 0
//   values [kv_head][position in page][vd]     at offset nkv * page_size * kd
// kd and vd need not be equal.  Pages of an entry are `page_stride` elements apart.
//
// This file holds the preparation of q, k and v (short convolution over time, per-map RMS norm with a
// shared weight, rotation of pairs of dimensions by position, cache write) and the plain attention kernel
// (float arithmetic for either storage type, key tiles aligned to absolute positions: a row's result does not
// depend on how the request was cut into steps or on what else is in the batch).
#include "diff_attention.cuh"

#define CONV_MAX_TAPS 8
#define PREP_THREADS 256

// One warp per unit of a token: a unit is one map of one query head (dim channels), one map of one key head
// (dim channels) or one value head (vd channels).  A lane owns pairs of neighbouring channels, so that a
// rotated pair stays in one thread.
//
// proj:  [n_tokens, ld] the fused projection q | k | v as the product left it (before the convolution)
// conv_w: [channels, taps] float, channels = nh*2*dim + nkv*2*dim + nkv*vd in the projection's order
// state: [slots, taps-1, channels] float: read only (conv_state_update moves it afterwards), or, with move_state
// (steps in which every request brings exactly one token), moved on here
template <typename T>
__global__ void __launch_bounds__(PREP_THREADS)
diff_qkv_prepare_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ conv_w,
                        float* __restrict__ state, int move_state, int taps, const float* __restrict__ q_norm,
                        const float* __restrict__ k_norm, float eps, const float* __restrict__ inv_freq, int rot_dims,
                        T* __restrict__ q_out, T* __restrict__ pool, DiffCache cache,
                        const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                        const int* __restrict__ q_start, const int* __restrict__ slots,
                        const int* __restrict__ block_table, int nh, int dim, int write_kv, int* __restrict__ status) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    const int pos = positions[t];
    if (pos < 0) return;
    const int b = seq_of_token[t];
    const int slot = slots[b];
    const int i = t - q_start[b];                         // the token's place in its portion
    const int nkv = cache.nkv, vd = cache.vd;
    const int q_units = nh * 2, k_units = nkv * 2, units = q_units + k_units + nkv;
    const int channels = (q_units + k_units) * dim + nkv * vd;
    const int keep = taps - 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int page = block_table[(size_t)slot * cache.max_pages + pos / cache.page_size];
    const int pip = pos % cache.page_size;
    if (page < 0 && write_kv && status && threadIdx.x == 0 && blockIdx.y == 0) *status = 1;
    float* st = state + (size_t)slot * keep * channels;
    for (int u = blockIdx.y * nwarp + warp; u < units; u += nwarp * gridDim.y) {
        const bool is_q = u < q_units, is_k = !is_q && u < q_units + k_units;
        const int width = (is_q || is_k) ? dim : vd;
        const int ch0 = is_q ? u * dim : is_k ? q_units * dim + (u - q_units) * dim
                                              : (q_units + k_units) * dim + (u - q_units - k_units) * vd;
        // at most 4 pairs per lane: widths up to 256
        float x0[4], x1[4];
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            x0[r] = x1[r] = 0.f;
            const int e = 2 * (lane + 32 * r);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                if (e + half >= width) continue;
                const int c = ch0 + e + half;
                float y = 0.f, vv[CONV_MAX_TAPS];
                for (int j = 0; j < taps; ++j) {
                    const int back = keep - j;            // the input `back` positions before this token
                    float v;
                    // (through L2 only: the kernel just before wrote the projection)
                    if (back <= i) v = load1_cg(proj + (size_t)(t - back) * ld + c);
                    else v = __ldcg(st + (size_t)(keep - (back - i)) * channels + c);   // zero before the request's start
                    vv[j] = v;
                    y = fmaf(conv_w[(size_t)c * taps + j], v, y);
                }
                // every request brings one token: this thread alone reads and writes the channel's state
                if (move_state)
                    for (int j = 0; j < keep; ++j) st[(size_t)j * channels + c] = vv[j + 1];
                if (half) x1[r] = y; else x0[r] = y;
                ss += y * y;
            }
        }
        if (is_q || is_k) {
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)dim + eps);
            const float* g = is_q ? q_norm : k_norm;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int e = 2 * (lane + 32 * r);
                if (e >= dim) continue;
                float a = x0[r] * inv * g[e];
                float bb = e + 1 < dim ? x1[r] * inv * g[e + 1] : 0.f;
                if (e + 1 < rot_dims) {
                    float sn, cs;
                    sincosf((float)pos * inv_freq[e >> 1], &sn, &cs);
                    const float ra = a * cs - bb * sn, rb = bb * cs + a * sn;
                    a = ra; bb = rb;
                }
                x0[r] = a; x1[r] = bb;
            }
        }
        T* dst;
        if (is_q) dst = q_out + ((size_t)t * q_units + u) * dim;
        else if (!write_kv || page < 0) continue;
        else if (is_k) dst = cache_keys(pool, cache, page, (u - q_units) >> 1, pip) + ((u - q_units) & 1) * dim;
        else dst = cache_values(pool, cache, page, u - q_units - k_units, pip);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = 2 * (lane + 32 * r);
            if (e < width) dst[e] = from_f32<T>(x0[r]);
            if (e + 1 < width) dst[e + 1] = from_f32<T>(x1[r]);
        }
    }
}

ST_EXPORT int st_diff_qkv_prepare(const void* proj, int ld, const float* conv_w, float* state, int move_state, int taps,
                                  const float* q_norm, const float* k_norm, float eps, const float* inv_freq,
                                  int rot_dims, void* q_out, void* pool, long long page_stride, long long entry_offset,
                                  const int* positions, const int* seq_of_token, const int* q_start, const int* slots,
                                  const int* block_table, int max_pages, int n_tokens, int nh, int nkv, int dim, int vd,
                                  int page_size, int write_kv, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || dim <= 0 || vd <= 0 || page_size <= 0 || taps < 1 || rot_dims < 0 ||
        rot_dims > dim || rot_dims % 2)
        return ST_ERR_BAD_ARG;
    if (taps > CONV_MAX_TAPS || dim > 256 || vd > 256) return ST_ERR_TOO_LARGE;
    const DiffCache c = {max_pages, page_size, nkv, 2 * dim, vd, page_stride, entry_offset};
    cudaStream_t s = (cudaStream_t)stream;
    // a warp per unit (a map of a head, or a value head); few tokens: the units of a token spread over blocks
    const int units = 2 * nh + 3 * nkv, per_block = PREP_THREADS / 32;
    const int groups = n_tokens >= 2 * st_sm_count() ? 1 : (units + per_block - 1) / per_block;
    if (dtype == 0)
        return st_launch_pdl("diff_prepare", diff_qkv_prepare_kernel<float>, dim3(n_tokens, groups), dim3(PREP_THREADS), 0, s,
                             (const float*)proj, ld, conv_w, state, move_state, taps, q_norm, k_norm, eps, inv_freq, rot_dims,
                             (float*)q_out, (float*)pool, c, positions, seq_of_token, q_start, slots, block_table, nh, dim,
                             write_kv, status);
    else if (dtype == 1)
        return st_launch_pdl("diff_prepare", diff_qkv_prepare_kernel<bf16>, dim3(n_tokens, groups), dim3(PREP_THREADS), 0, s,
                             (const bf16*)proj, ld, conv_w, state, move_state, taps, q_norm, k_norm, eps, inv_freq, rot_dims,
                             (bf16*)q_out, (bf16*)pool, c, positions, seq_of_token, q_start, slots, block_table, nh, dim,
                             write_kv, status);
    else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}

// ------------------------------------------------------------------------------------------------
// Plain differential attention: one block per (query token, head); `items` lists the tokens to serve
// (n_tokens of them, -1: none), or is null for tokens 0..n_tokens-1.
#define KT 128   // keys per tile == threads per block

template <typename T>
__global__ void __launch_bounds__(KT)
diff_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ pool, DiffCache cache, T* __restrict__ out,
                            const int* __restrict__ items, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                            const int* __restrict__ slots, const int* __restrict__ block_table, int nh, int dim,
                            float scale, float cap, int block, int window, float lambda, float eps, float out_scale,
                            int* __restrict__ status) {
    extern __shared__ float smem[];
    float* sq = smem;                 // [2 * dim] the two queries
    float* sp1 = smem + 2 * dim;      // [KT] weights of the tile, map 1
    float* sp2 = sp1 + KT;            // [KT] map 2
    __shared__ float scratch[32];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = items ? items[blockIdx.x] : blockIdx.x, h = blockIdx.y;
    if (t < 0) return;                                  // padding of the item list
    const int pos = positions[t];
    if (pos < 0) return;
    const int nkv = cache.nkv, vd = cache.vd, kd = cache.kd, ps = cache.page_size;
    const int kvh = h / (nh / nkv);
    const int* bt = block_table + (size_t)slots[seq_of_token[t]] * cache.max_pages;
    for (int e = threadIdx.x; e < kd; e += KT) sq[e] = load1_cg(q + ((size_t)t * nh + h) * kd + e);
    __syncthreads();
    const int lo = first_visible(pos, block, window), hi = pos + 1;
    float a1[2] = {0.f, 0.f}, a2[2] = {0.f, 0.f};     // vd <= 2 * KT
    float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.f, l2 = 0.f;
    for (int base = (lo / KT) * KT; base < hi; base += KT) {
        const int j = base + threadIdx.x;
        const bool seen = j >= lo && j < hi;
        float s1 = -INFINITY, s2 = -INFINITY;
        if (seen) {
            const int page = bt[j / ps];
            if (page >= 0) {
                const T* krow = cache_keys(pool, cache, page, kvh, j % ps);
                float d1 = 0.f, d2 = 0.f;
                for (int e = 0; e < dim; ++e) {
                    d1 = fmaf(sq[e], load1_cg(krow + e), d1);
                    d2 = fmaf(sq[dim + e], load1_cg(krow + dim + e), d2);
                }
                s1 = soft_cap(d1 * scale, cap);
                s2 = soft_cap(d2 * scale, cap);
            } else if (status) {
                *status = 1;
            }
        }
        const float n1 = fmaxf(m1, block_max(s1, scratch)), n2 = fmaxf(m2, block_max(s2, scratch));
        const float p1 = s1 > -INFINITY ? expf(s1 - n1) : 0.f, p2 = s2 > -INFINITY ? expf(s2 - n2) : 0.f;
        const float c1 = m1 == -INFINITY ? 0.f : expf(m1 - n1), c2 = m2 == -INFINITY ? 0.f : expf(m2 - n2);
        l1 = l1 * c1 + block_sum(p1, scratch);
        l2 = l2 * c2 + block_sum(p2, scratch);
        m1 = n1; m2 = n2;
        sp1[threadIdx.x] = p1;
        sp2[threadIdx.x] = p2;
        __syncthreads();
        const int j_begin = max(0, lo - base), j_end = min(KT, hi - base);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int e = threadIdx.x + c * KT;
            if (e >= vd) continue;
            float x1 = a1[c] * c1, x2 = a2[c] * c2;
            for (int jj = j_begin; jj < j_end; ++jj) {
                const int key = base + jj;
                const int page = bt[key / ps];
                if (page < 0) continue;
                const float v = load1_cg(cache_values(pool, cache, page, kvh, key % ps) + e);
                x1 = fmaf(sp1[jj], v, x1);
                x2 = fmaf(sp2[jj], v, x2);
            }
            a1[c] = x1; a2[c] = x2;
        }
        __syncthreads();
    }
    const float i1 = l1 > 0.f ? 1.f / l1 : 0.f, i2 = l2 > 0.f ? 1.f / l2 : 0.f;
    float o[2], ss = 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int e = threadIdx.x + c * KT;
        o[c] = e < vd ? a1[c] * i1 - lambda * (a2[c] * i2) : 0.f;
        ss += o[c] * o[c];
    }
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)vd + eps) * out_scale;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int e = threadIdx.x + c * KT;
        if (e < vd) out[((size_t)t * nh + h) * vd + e] = from_f32<T>(o[c] * r);
    }
}

// ------------------------------------------------------------------------------------------------
// The same per (token, head) for bfloat16 with 16-byte accesses, for single tokens and short portions, where
// the keys and values are read once and the kernel is bound by their way from memory: each of the four warps
// takes every fourth key of a tile of 128, its lanes side by side along the key's row (the two maps' dot
// products by shuffles) and then along the value row (a lane owns four neighbouring value dimensions, the rows'
// addresses wait in shared memory); the softmax over the tile is done a thread per key, and the warps' partial
// sums meet at the end.  dim % 8 == 0, vd % 4 == 0,
// vd <= 512.  Tiles are aligned to absolute positions as in the plain kernel.
#define DA_VPASS 2      // value dimensions per lane: 4 * DA_VPASS * 32 >= vd (vd <= 256)
#define DA_QPASS 2      // and of the 2 * dim query / key elements: dim <= 128
#define DA_THREADS 512  // sixteen warps: four per scheduler hide one another's waits (a block per SM is the usual launch)
#define DA_WARPS (DA_THREADS / 32)
#define DA_BATCH (KT / DA_WARPS)   // a warp's keys of a tile: all their rows are asked for before the first is used

__global__ void __launch_bounds__(DA_THREADS)
diff_attention_single_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, DiffCache cache,
                             bf16* __restrict__ out, const int* __restrict__ items, const int* __restrict__ positions,
                             const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                             const int* __restrict__ block_table, int nh, int dim, float scale, float cap, int block,
                             int window, float lambda, float eps, float out_scale, int* __restrict__ status) {
    extern __shared__ __align__(16) float smem[];
    __shared__ float scratch[32];
    __shared__ const bf16* srow[KT];                     // the value row of each key of the tile (null: not seen)
    __shared__ const bf16* skrow[KT];                    // and its key row
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = items ? items[blockIdx.x] : blockIdx.x, h = blockIdx.y;
    if (t < 0) return;
    const int pos = positions[t];
    if (pos < 0) return;
    const int nkv = cache.nkv, vd = cache.vd, kd = cache.kd, ps = cache.page_size;
    float* sq = smem;                 // [2 * dim]
    float* sp1 = sq + kd;             // [KT]
    float* sp2 = sp1 + KT;            // [KT]
    float* so = sp2 + KT;             // [warps][2 maps][vd]
    const int kvh = h / (nh / nkv);
    const int* bt = block_table + (size_t)slots[seq_of_token[t]] * cache.max_pages;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int e = threadIdx.x; e < kd; e += DA_THREADS) sq[e] = load1_cg(q + ((size_t)t * nh + h) * kd + e);
    __syncthreads();
    const int lo = first_visible(pos, block, window), hi = pos + 1;
    float a1[DA_VPASS][4], a2[DA_VPASS][4];
#pragma unroll
    for (int p = 0; p < DA_VPASS; ++p)
#pragma unroll
        for (int x = 0; x < 4; ++x) a1[p][x] = a2[p][x] = 0.f;
    float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.f, l2 = 0.f;
    // this lane's share of the two queries: four neighbouring elements of the 2 * dim per pass of 128
    float qr[DA_QPASS][4];
#pragma unroll
    for (int p = 0; p < DA_QPASS; ++p)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int g = p * 128 + 4 * lane + x;
            qr[p][x] = g < kd ? sq[g] : 0.f;
        }
    for (int base = (lo / KT) * KT; base < hi; base += KT) {
        // where the tile's keys and values lie: a thread per key (the look-ups of a tile run side by side)
        if (threadIdx.x < KT) {
            const int j = base + threadIdx.x;
            const bf16 *kr = nullptr, *vr = nullptr;
            if (j >= lo && j < hi) {
                const int page = bt[j / ps];
                if (page >= 0) {
                    kr = cache_keys(pool, cache, page, kvh, j % ps);
                    vr = cache_values(pool, cache, page, kvh, j % ps);
                } else if (status) {
                    *status = 1;
                }
            }
            skrow[threadIdx.x] = kr;
            srow[threadIdx.x] = vr;
        }
        __syncthreads();
        // scores: a warp takes every fourth key of the tile, its lanes side by side along the key's row; the rows of
        // four keys are asked for before the first is used
        for (int jj0 = warp; jj0 < KT; jj0 += DA_WARPS * DA_BATCH) {
            float4 kk[DA_BATCH][DA_QPASS];
#pragma unroll
            for (int u = 0; u < DA_BATCH; ++u) {
                const bf16* krow = skrow[jj0 + DA_WARPS * u];
#pragma unroll
                for (int p = 0; p < DA_QPASS; ++p) {
                    const int g = p * 128 + 4 * lane;
                    kk[u][p] = (krow && g < kd) ? load4_cg(krow + g) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int u = 0; u < DA_BATCH; ++u) {
                float d1 = 0.f, d2 = 0.f;
#pragma unroll
                for (int p = 0; p < DA_QPASS; ++p) {
                    const int g = p * 128 + 4 * lane;
                    const float4 k = kk[u][p];
                    const float d = fmaf(qr[p][0], k.x, fmaf(qr[p][1], k.y, fmaf(qr[p][2], k.z, qr[p][3] * k.w)));
                    if (g < dim) d1 += d; else d2 += d;
                }
                d1 = warp_sum(d1);
                d2 = warp_sum(d2);
                if (lane == 0) {
                    const bool seen = skrow[jj0 + DA_WARPS * u] != nullptr;
                    sp1[jj0 + DA_WARPS * u] = seen ? soft_cap(d1 * scale, cap) : -INFINITY;
                    sp2[jj0 + DA_WARPS * u] = seen ? soft_cap(d2 * scale, cap) : -INFINITY;
                }
            }
        }
        // the same keys' value rows are asked for now and wait in registers while the block does the softmax
        float4 vv[DA_BATCH][DA_VPASS];
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u) {
            const bf16* vr = srow[warp + DA_WARPS * u];
#pragma unroll
            for (int p = 0; p < DA_VPASS; ++p) {
                const int e = p * 128 + 4 * lane;
                vv[u][p] = (vr && e < vd) ? load4_cg(vr + e) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        __syncthreads();
        const bool holds = threadIdx.x < KT;              // the softmax over the tile: a thread per key
        const float s1 = holds ? sp1[threadIdx.x] : -INFINITY, s2 = holds ? sp2[threadIdx.x] : -INFINITY;
        const float n1 = fmaxf(m1, block_max(s1, scratch)), n2 = fmaxf(m2, block_max(s2, scratch));
        const float p1 = s1 > -INFINITY ? expf(s1 - n1) : 0.f, p2 = s2 > -INFINITY ? expf(s2 - n2) : 0.f;
        const float c1 = m1 == -INFINITY ? 0.f : expf(m1 - n1), c2 = m2 == -INFINITY ? 0.f : expf(m2 - n2);
        l1 = l1 * c1 + block_sum(p1, scratch);
        l2 = l2 * c2 + block_sum(p2, scratch);
        m1 = n1; m2 = n2;
        if (holds) {                 // (block_sum above has met all threads since the scores were read)
            sp1[threadIdx.x] = p1;
            sp2[threadIdx.x] = p2;
        }
        __syncthreads();
#pragma unroll
        for (int p = 0; p < DA_VPASS; ++p)
#pragma unroll
            for (int x = 0; x < 4; ++x) { a1[p][x] *= c1; a2[p][x] *= c2; }
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u) {
            const int jj = warp + DA_WARPS * u;
            const float w1 = sp1[jj], w2 = sp2[jj];       // zero for a key that is not seen
#pragma unroll
            for (int p = 0; p < DA_VPASS; ++p) {
                const float4 v = vv[u][p];
                a1[p][0] = fmaf(w1, v.x, a1[p][0]); a1[p][1] = fmaf(w1, v.y, a1[p][1]);
                a1[p][2] = fmaf(w1, v.z, a1[p][2]); a1[p][3] = fmaf(w1, v.w, a1[p][3]);
                a2[p][0] = fmaf(w2, v.x, a2[p][0]); a2[p][1] = fmaf(w2, v.y, a2[p][1]);
                a2[p][2] = fmaf(w2, v.z, a2[p][2]); a2[p][3] = fmaf(w2, v.w, a2[p][3]);
            }
        }
        __syncthreads();
    }
    // the warps' partial sums meet (in warp order), then the difference of the maps and its norm
#pragma unroll
    for (int p = 0; p < DA_VPASS; ++p) {
        const int e = p * 128 + 4 * lane;
        if (e < vd) {
            *reinterpret_cast<float4*>(so + (warp * 2 + 0) * vd + e) = make_float4(a1[p][0], a1[p][1], a1[p][2], a1[p][3]);
            *reinterpret_cast<float4*>(so + (warp * 2 + 1) * vd + e) = make_float4(a2[p][0], a2[p][1], a2[p][2], a2[p][3]);
        }
    }
    __syncthreads();
    const float i1 = l1 > 0.f ? 1.f / l1 : 0.f, i2 = l2 > 0.f ? 1.f / l2 : 0.f;
    const int e = threadIdx.x;                            // vd <= 256 <= threads
    float o = 0.f;
    if (e < vd) {
        float x1 = 0.f, x2 = 0.f;
        for (int w = 0; w < DA_WARPS; ++w) { x1 += so[(w * 2 + 0) * vd + e]; x2 += so[(w * 2 + 1) * vd + e]; }
        o = x1 * i1 - lambda * (x2 * i2);
    }
    const float ss = block_sum(o * o, scratch);
    const float r = rsqrtf(ss / (float)vd + eps) * out_scale;
    if (e < vd) out[((size_t)t * nh + h) * vd + e] = __float2bfloat16_rn(o * r);
}

ST_EXPORT int st_diff_attention_single_applies(int dim, int vd) {
    return dim > 0 && vd > 0 && dim % 8 == 0 && vd % 4 == 0 && vd <= 128 * DA_VPASS && 2 * dim <= 128 * DA_QPASS;
}

// bfloat16 only; `items` as for the plain kernel
ST_EXPORT int st_diff_attention_single(const void* q, const void* pool, long long page_stride, long long entry_offset,
                                       void* out, const int* items, const int* positions, const int* seq_of_token,
                                       const int* slots, const int* block_table, int max_pages, int n_tokens, int nh,
                                       int nkv, int dim, int vd, int page_size, float scale, float cap, int block,
                                       int window, float lambda, float eps, float out_scale, int* status, void* stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0) return ST_ERR_BAD_ARG;
    if (!st_diff_attention_single_applies(dim, vd)) return ST_ERR_BAD_SIZE;
    const DiffCache c = {max_pages, page_size, nkv, 2 * dim, vd, page_stride, entry_offset};
    const size_t smem = (size_t)(2 * dim + 2 * KT + 2 * DA_WARPS * vd) * sizeof(float);
    if (smem > 48 * 1024) return ST_ERR_TOO_LARGE;
    return st_launch_pdl("diff_single", diff_attention_single_kernel, dim3(n_tokens, nh), dim3(DA_THREADS), smem, (cudaStream_t)stream,
                         (const bf16*)q, (const bf16*)pool, c, (bf16*)out, items, positions, seq_of_token, slots,
                         block_table, nh, dim, scale, cap, block, window, lambda, eps, out_scale, status);
}

ST_EXPORT int st_diff_attention_plain(const void* q, const void* pool, long long page_stride, long long entry_offset,
                                      void* out, const int* items, const int* positions, const int* seq_of_token,
                                      const int* slots,
                                      const int* block_table, int max_pages, int n_tokens, int nh, int nkv, int dim,
                                      int vd, int page_size, float scale, float cap, int block, int window,
                                      float lambda, float eps, float out_scale, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || dim <= 0 || vd <= 0 || page_size <= 0) return ST_ERR_BAD_ARG;
    if (vd > 2 * KT || dim > 1024) return ST_ERR_TOO_LARGE;
    const DiffCache c = {max_pages, page_size, nkv, 2 * dim, vd, page_stride, entry_offset};
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, nh);
    const size_t smem = (size_t)(2 * dim + 2 * KT) * sizeof(float);
    if (dtype == 0)
        return st_launch_pdl("diff_plain", diff_attention_plain_kernel<float>, grid, dim3(KT), smem, s, (const float*)q,
                             (const float*)pool, c, (float*)out, items, positions, seq_of_token, slots, block_table, nh, dim,
                             scale, cap, block, window, lambda, eps, out_scale, status);
    else if (dtype == 1)
        return st_launch_pdl("diff_plain", diff_attention_plain_kernel<bf16>, grid, dim3(KT), smem, s, (const bf16*)q,
                             (const bf16*)pool, c, (bf16*)out, items, positions, seq_of_token, slots, block_table, nh, dim,
                             scale, cap, block, window, lambda, eps, out_scale, status);
    else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}
