// Grouped matrix products: many products of the same shape of weights, each over its own rows.
//
//   c[row, g * c_goff + n] = epilogue( sum_k a[arow, g * a_goff + k] * w[g][n][k] )        w[g] stored [out, in]
//
// Two ways to say which rows a group has:
//   * every group takes all n_rows rows (the heads of an attention layer, each with a matrix of its own on its own
//     columns of a: a_goff / c_goff are the column offsets from one head to the next); grid.z walks the groups;
//   * a group takes the rows offsets[g]..offsets[g+1]-1 of a sorted list (the experts of a mixture): the launch walks
//     row tiles (tile_group[i], tile_row0[i]) made on the device, arow = a_rows[row] / a_row_div where a_rows is
//     given (the sorted (token, choice) items, a_row_div choices per token), else the row itself.
// Epilogue: none, or "gated": w[g] holds 2 * n_out rows, gate rows first, and c = act(gate) * up.
//
// gemm_grouped_mma: bfloat16 on the warp-level tensor cores (mma.sync m16n8k16, float accumulation): tiles of 64 rows
// x 64 outputs x 64 of k, four warps of 32 x 32 each, rows gathered and weights streamed by 16-byte asynchronous
// copies in three stages (two tiles of k under way per block: steps of few tokens are bound by the weights' way from
// memory, and what a block has in flight decides the rate); k, the row strides and the group offsets must be multiples of 8 elements.
// gemm_grouped_plain: float arithmetic for either storage type; every output element is one chain of fused
// multiply-adds over k in ascending order whatever rows share its tile (the 32-bit path, and the plain twin).
#include "common.cuh"
#include "mma_sync.cuh"

struct GroupedShape {
    int n_rows, n_out, k_dim, gated, act;
    long long lda, a_goff, ldc, c_goff, w_gstride;
    const int* offsets;        // null: every group takes all rows
    const int* tile_group;
    const int* tile_row0;
    const int* a_rows;
    int a_row_div;
};

#define GG_BM 64
#define GG_BN 64
#define GG_BK 16

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
gemm_grouped_plain_kernel(const T* __restrict__ a, const T* __restrict__ w, TO* __restrict__ c, GroupedShape sh) {
    __shared__ float sa[GG_BK][GG_BM + 4];
    __shared__ float sw[GG_BK][GG_BN + 4];
    __shared__ float su[GG_BK][GG_BN + 4];
    __shared__ int srow[GG_BM];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    int g, row0, row_end;
    if (sh.offsets) {
        g = __ldcg(sh.tile_group + blockIdx.y);
        if (g < 0) return;
        row0 = __ldcg(sh.tile_row0 + blockIdx.y);
        row_end = min(row0 + GG_BM, __ldcg(sh.offsets + g + 1));
    } else {
        g = blockIdx.z;
        row0 = blockIdx.y * GG_BM;
        row_end = min(row0 + GG_BM, sh.n_rows);
    }
    if (threadIdx.x < GG_BM) {
        const int r = row0 + threadIdx.x;
        int ar = -1;
        if (r < row_end) ar = sh.a_rows ? __ldcg(sh.a_rows + r) / sh.a_row_div : r;
        srow[threadIdx.x] = ar;
    }
    __syncthreads();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int col0 = blockIdx.x * GG_BN;
    const T* wg = w + (long long)g * sh.w_gstride;
    float acc[4][4], acu[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = acu[i][j] = 0.f;
    for (int k0 = 0; k0 < sh.k_dim; k0 += GG_BK) {
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = threadIdx.x + it * 256;
            const int r = idx / GG_BK, kk = idx % GG_BK;
            const int k = k0 + kk;
            const int ar = srow[r], wr = col0 + r;
            sa[kk][r] = (ar >= 0 && k < sh.k_dim) ? load1_cg(a + (long long)ar * sh.lda + g * sh.a_goff + k) : 0.f;
            const bool ok = wr < sh.n_out && k < sh.k_dim;
            sw[kk][r] = ok ? to_f32(wg[(long long)wr * sh.k_dim + k]) : 0.f;
            if (sh.gated) su[kk][r] = ok ? to_f32(wg[(long long)(sh.n_out + wr) * sh.k_dim + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GG_BK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = sw[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
            if (sh.gated) {
#pragma unroll
                for (int j = 0; j < 4; ++j) wv[j] = su[kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acu[i][j] = fmaf(av[i], wv[j], acu[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        if (r >= row_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = col0 + tx * 4 + j;
            if (n >= sh.n_out) continue;
            float v = acc[i][j];
            if (sh.gated) {
                // both products are rounded to the storage type first, as two separate products would leave them
                v = apply_act(to_f32(from_f32<T>(v)), sh.act) * to_f32(from_f32<T>(acu[i][j]));
            }
            c[(long long)r * sh.ldc + g * sh.c_goff + n] = from_f32<TO>(v);
        }
    }
}

ST_EXPORT int st_gemm_grouped_plain(const void* a, const void* w, void* c, int n_groups, int n_rows, int n_out, int k_dim,
                                    int gated, int act, long long lda, long long a_goff, long long ldc, long long c_goff,
                                    long long w_gstride, const int* offsets, const int* tile_group, const int* tile_row0,
                                    int n_tiles, const int* a_rows, int a_row_div, int dtype, int out_f32, void* stream) {
    if (n_groups <= 0 || n_out <= 0) return 0;
    if (k_dim <= 0 || (offsets && (!tile_group || !tile_row0 || n_tiles <= 0)) || (a_rows && a_row_div <= 0)) return ST_ERR_BAD_ARG;
    if (!offsets && n_rows <= 0) return 0;
    GroupedShape sh{n_rows, n_out, k_dim, gated, act, lda, a_goff, ldc, c_goff, w_gstride, offsets, tile_group, tile_row0,
                    a_rows, a_row_div};
    dim3 grid((n_out + GG_BN - 1) / GG_BN, offsets ? n_tiles : (n_rows + GG_BM - 1) / GG_BM, offsets ? 1 : n_groups);
    if (grid.y > 65535 || grid.z > 65535) return ST_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0)
        return st_launch_pdl("gemm_grouped", gemm_grouped_plain_kernel<float, float>, grid, dim3(256), 0, s, (const float*)a,
                             (const float*)w, (float*)c, sh);
    if (dtype != 1) return ST_ERR_BAD_DTYPE;
    if (out_f32)
        return st_launch_pdl("gemm_grouped", gemm_grouped_plain_kernel<bf16, float>, grid, dim3(256), 0, s, (const bf16*)a,
                             (const bf16*)w, (float*)c, sh);
    return st_launch_pdl("gemm_grouped", gemm_grouped_plain_kernel<bf16, bf16>, grid, dim3(256), 0, s, (const bf16*)a,
                         (const bf16*)w, (bf16*)c, sh);
}

#define GM_BK 64
#define GM_LD (GM_BK + 8)
#define GM_STAGES 3

template <typename TO, bool GATED, int BN>
__global__ void __launch_bounds__(128)
gemm_grouped_mma_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, TO* __restrict__ c, GroupedShape sh) {
    extern __shared__ __align__(16) unsigned char gm_smem[];
    constexpr int WROWS = GATED ? 2 * BN : BN;
    bf16 (*sa)[GG_BM][GM_LD] = reinterpret_cast<bf16 (*)[GG_BM][GM_LD]>(gm_smem);
    bf16 (*sw)[WROWS][GM_LD] = reinterpret_cast<bf16 (*)[WROWS][GM_LD]>(gm_smem + sizeof(bf16) * GM_STAGES * GG_BM * GM_LD);
    __shared__ int srow[GG_BM];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    int g, row0, row_end;
    if (sh.offsets) {
        g = __ldcg(sh.tile_group + blockIdx.y);
        if (g < 0) return;
        row0 = __ldcg(sh.tile_row0 + blockIdx.y);
        row_end = min(row0 + GG_BM, __ldcg(sh.offsets + g + 1));
    } else {
        g = blockIdx.z;
        row0 = blockIdx.y * GG_BM;
        row_end = min(row0 + GG_BM, sh.n_rows);
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < GG_BM) {
        const int r = row0 + tid;
        int ar = -1;
        if (r < row_end) ar = sh.a_rows ? __ldcg(sh.a_rows + r) / sh.a_row_div : r;
        srow[tid] = ar;
    }
    __syncthreads();
    const int col0 = blockIdx.x * BN;
    const bf16* wg = w + (long long)g * sh.w_gstride;
    const bf16* ag = a + g * sh.a_goff;
    auto load = [&](int k0, int stage) {
        // 64 rows x 8 chunks of 8 per operand
        for (int ch = tid; ch < GG_BM * 8; ch += 128) {
            const int r = ch >> 3, kc = (ch & 7) * 8;
            const int ar = srow[r];
            const bool ok = ar >= 0 && k0 + kc < sh.k_dim;
            cp_async16(&sa[stage][r][kc], ok ? ag + (long long)ar * sh.lda + k0 + kc : a, ok);
        }
        for (int ch = tid; ch < BN * 8 * (GATED ? 2 : 1); ch += 128) {
            const int r = ch >> 3, kc = (ch & 7) * 8;
            const int n = col0 + (r & (BN - 1)) + (r >= BN ? sh.n_out : 0);
            const bool ok = col0 + (r & (BN - 1)) < sh.n_out && k0 + kc < sh.k_dim;
            cp_async16(&sw[stage][r][kc], ok ? wg + (long long)n * sh.k_dim + k0 + kc : w, ok);
        }
    };
    constexpr int NJ = BN / 16;          // 8-wide output tiles of a warp (its half of the block's columns)
    float acc[2][NJ][4], acu[GATED ? 2 : 1][NJ][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < NJ; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[i][j][e] = 0.f;
                if (GATED) acu[i][j][e] = 0.f;
            }
    const int wm = (warp & 1) * 32, wn = (warp >> 1) * (BN / 2);
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
    const int n_k = (sh.k_dim + GM_BK - 1) / GM_BK;
    // three stages: two tiles of k under way while one is multiplied (a group is committed every turn, so that
    // "all but the newest" always means the tile about to be used)
#pragma unroll
    for (int p = 0; p < GM_STAGES - 1; ++p) {
        if (p < n_k) load(p * GM_BK, p);
        cp_async_commit();
    }
    for (int kt = 0; kt < n_k; ++kt) {
        const int stage = kt % GM_STAGES;
        cp_async_wait<GM_STAGES - 2>();
        __syncthreads();
        if (kt + GM_STAGES - 1 < n_k) load((kt + GM_STAGES - 1) * GM_BK, (kt + GM_STAGES - 1) % GM_STAGES);
        cp_async_commit();
#pragma unroll
        for (int kk = 0; kk < GM_BK; kk += 16) {
            uint32_t af[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                ldmatrix_x4(af[i][0], af[i][1], af[i][2], af[i][3], &sa[stage][wm + i * 16 + a_row][kk + a_col]);
#pragma unroll
            for (int jp = 0; jp < NJ / 2; ++jp) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, &sw[stage][wn + jp * 16 + b_row][kk + b_col]);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mma_bf16(acc[i][2 * jp], af[i], b0, b1);
                    mma_bf16(acc[i][2 * jp + 1], af[i], b2, b3);
                }
                if (GATED) {
                    ldmatrix_x4(b0, b1, b2, b3, &sw[stage][BN + wn + jp * 16 + b_row][kk + b_col]);
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        mma_bf16(acu[i][2 * jp], af[i], b0, b1);
                        mma_bf16(acu[i][2 * jp + 1], af[i], b2, b3);
                    }
                }
            }
        }
    }
    const int gq = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < NJ; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = row0 + wm + i * 16 + gq + (e >> 1) * 8;
                const int n = col0 + wn + j * 8 + 2 * tq + (e & 1);
                if (r >= row_end || n >= sh.n_out) continue;
                float v = acc[i][j][e];
                if (GATED) v = apply_act(to_f32(from_f32<bf16>(v)), sh.act) * to_f32(from_f32<bf16>(acu[i][j][e]));
                c[(long long)r * sh.ldc + g * sh.c_goff + n] = from_f32<TO>(v);
            }
}

ST_EXPORT int st_gemm_grouped_mma_applies(int k_dim, long long lda, long long a_goff, long long w_gstride) {
    return k_dim > 0 && k_dim % 8 == 0 && lda % 8 == 0 && a_goff % 8 == 0 && w_gstride % 8 == 0;
}

ST_EXPORT int st_gemm_grouped_mma(const void* a, const void* w, void* c, int n_groups, int n_rows, int n_out, int k_dim,
                                  int gated, int act, long long lda, long long a_goff, long long ldc, long long c_goff,
                                  long long w_gstride, const int* offsets, const int* tile_group, const int* tile_row0,
                                  int n_tiles, const int* a_rows, int a_row_div, int out_f32, void* stream) {
    if (n_groups <= 0 || n_out <= 0) return 0;
    if ((offsets && (!tile_group || !tile_row0 || n_tiles <= 0)) || (a_rows && a_row_div <= 0)) return ST_ERR_BAD_ARG;
    if (!offsets && n_rows <= 0) return 0;
    if (!st_gemm_grouped_mma_applies(k_dim, lda, a_goff, w_gstride) || !aligned16(a) || !aligned16(w)) return ST_ERR_BAD_SIZE;
    GroupedShape sh{n_rows, n_out, k_dim, gated, act, lda, a_goff, ldc, c_goff, w_gstride, offsets, tile_group, tile_row0,
                    a_rows, a_row_div};
    dim3 grid((n_out + GG_BN - 1) / GG_BN, offsets ? n_tiles : (n_rows + GG_BM - 1) / GG_BM, offsets ? 1 : n_groups);
    if (grid.y > 65535 || grid.z > 65535) return ST_ERR_TOO_LARGE;
    // launches of few blocks (steps of few tokens, bound by the weights' way from memory) take tiles of 32 outputs:
    // twice the blocks, so that every SM pulls weights
    const bool narrow = (long long)grid.x * grid.y * grid.z < 2LL * st_sm_count();
    if (narrow) grid.x = (n_out + 31) / 32;
    cudaStream_t s = (cudaStream_t)stream;
    auto smem_of = [](int bn, bool g) { return sizeof(bf16) * GM_STAGES * (GG_BM + (g ? 2 : 1) * bn) * GM_LD; };
    static bool set = false;
    if (!set) {
#define GM_SET(TO, G, BN) cudaFuncSetAttribute(gemm_grouped_mma_kernel<TO, G, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_of(BN, G))
        GM_SET(float, true, 64); GM_SET(bf16, true, 64); GM_SET(float, false, 64); GM_SET(bf16, false, 64);
        GM_SET(float, true, 32); GM_SET(bf16, true, 32); GM_SET(float, false, 32); GM_SET(bf16, false, 32);
#undef GM_SET
        set = true;
    }
#define GM_LAUNCH(TO, G, BN)                                                                                          \
    return st_launch_pdl("gemm_grouped", gemm_grouped_mma_kernel<TO, G, BN>, grid, dim3(128), smem_of(BN, G), s,      \
                         (const bf16*)a, (const bf16*)w, (TO*)c, sh)
    if (narrow) {
        if (gated) { if (out_f32) GM_LAUNCH(float, true, 32); GM_LAUNCH(bf16, true, 32); }
        if (out_f32) GM_LAUNCH(float, false, 32);
        GM_LAUNCH(bf16, false, 32);
    }
    if (gated) { if (out_f32) GM_LAUNCH(float, true, 64); GM_LAUNCH(bf16, true, 64); }
    if (out_f32) GM_LAUNCH(float, false, 64);
    GM_LAUNCH(bf16, false, 64);
#undef GM_LAUNCH
}

ST_EXPORT int st_gemm_grouped_tile_rows() { return GG_BM; }
