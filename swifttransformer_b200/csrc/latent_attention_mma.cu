// Latent attention on the warp-level tensor cores (bfloat16): the kernel for prompt portions and for single tokens.
//
// All heads read the same cached rows [c | k_rot], so the rows of the query tile are (token, head) pairs: 64
// consecutive pairs of one request's tokens of the step, in the order the latent-space queries lie in memory
// ([token][head][kr + rot]).  A single decoded token of a model with H heads is a tile of H rows; a prompt portion
// of n tokens is ceil(n * H / 64) tiles, and every row carries its own causal limit (its token's position).
//
// Per tile of 32 keys (aligned to absolute positions, so a row's sums do not depend on how the request was cut):
//   S = Q K^T        eight warps: four groups of 16 rows x two halves of 16 keys, mma.sync m16n8k16 over kr + rot
//   softmax          float, running maximum and sums per row (the halves meet through shared memory)
//   O += P V         V is the first kr numbers of the very rows that were the keys: the warp of (row group, half)
//                    owns 16 rows x half of the value columns; P goes through shared memory as bfloat16
// and at the end the sink joins the denominator, the gate multiplies, and the row is stored.
// The key tiles arrive by 16-byte asynchronous copies, two stages.  NP: into how many parts the 32 keys of a tile (for
// S) and the value columns (for O) are cut among the warps of a row group: 2 (eight warps) is what is instantiated; 4
// (sixteen warps, a warp's accumulator 16 x kr/4) was measured at kr 512 and was no faster.  NT: value
// columns per warp / 8 (the block covers NT * 8 * NP >= kr columns; the template keeps the accumulator in registers).
#include "latent_attention.cuh"
#include "mma_sync.cuh"
#include "tcgen05.cuh"

#define LM_ROWS 64
#define LM_KEYS 32
#define LM_PLD 40          // row stride of the P tile in elements
#define LM_LAZY 8.f        // how far (log2) a row's maximum may run ahead of the reference before the row is rescaled

// one row of the cache into shared memory as a bulk copy that completes on an mbarrier (both addresses 16-byte
// aligned, the size a multiple of 16 bytes)
__device__ __forceinline__ void bulk_row_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t mbar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(mbar) : "memory");
}

__device__ __forceinline__ void ldmatrix_x2_s(uint32_t& r0, uint32_t& r1, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}

template <int NT, int NP>
__global__ void __launch_bounds__(NP * 128, 1)
latent_attention_mma_kernel(const bf16* __restrict__ q_lat, const bf16* __restrict__ pool, LatentCache cache,
                            bf16* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ q_start,
                            const int* __restrict__ start_pos, const int* __restrict__ slots,
                            const int* __restrict__ block_table, int n_seqs, const float* __restrict__ sink,
                            const bf16* __restrict__ gates, int gate_ld, int nh, float scale_log2, int lds, int kdp,
                            int n_splits, float* __restrict__ partial, int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);                 // [64][lds]
    bf16* sK = sQ + LM_ROWS * lds;                                // [2][32][lds]
    bf16* sP = sK + 2 * LM_KEYS * lds;                            // [64][LM_PLD]
    float* smax = reinterpret_cast<float*>(sP + LM_ROWS * LM_PLD);  // [NP][64]
    float* ssum = smax + NP * LM_ROWS;                            // [NP][64]
    __shared__ int s_req, s_tile;
    __shared__ __align__(8) uint64_t s_bar[2];          // "this stage's key rows have landed"
    constexpr int LM_THREADS = NP * 128, KW = LM_KEYS / NP, NKT = KW / 8;   // keys and key n-tiles of a warp
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, rg = warp & 3, half = warp >> 2;
    const int g = lane >> 2, tq = lane & 3;
    const int kr = cache.kr, kd = cache.kr + cache.rot, ps = cache.page_size;

    // zero the tiles once: the columns between kd and the padded width are read by the products
    for (int i = tid * 8; i < (LM_ROWS + 2 * LM_KEYS) * lds; i += LM_THREADS * 8)
        *reinterpret_cast<uint4*>(sQ + i) = make_uint4(0, 0, 0, 0);
    if (tid == 0) {
        int tile = gridDim.x - 1 - blockIdx.x, req = -1;      // the last tiles of a request have the longest key ranges: first
        for (int i = 0; i < n_seqs; ++i) {
            const int rows = (q_start[i + 1] - q_start[i]) * nh;
            const int tiles = (rows + LM_ROWS - 1) / LM_ROWS;
            if (tile < tiles) { req = i; break; }
            tile -= tiles;
        }
        s_req = req;
        s_tile = tile;
        tc_mbar_init(tc_smem(&s_bar[0]), 1);
        tc_mbar_init(tc_smem(&s_bar[1]), 1);
        tc_mbar_init_fence();
    }
    tc_fence_async_smem();                              // the zeros above before the bulk copies into the same rows
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    __syncthreads();
    const int b = s_req;
    if (b < 0) return;
    const int tok0 = q_start[b], n_rows = (q_start[b + 1] - tok0) * nh, r0 = s_tile * LM_ROWS;
    if (positions[tok0] < 0) return;                    // a padding request of a fixed-shape step
    const int start = start_pos[b];
    const int* bt = block_table + (size_t)slots[b] * cache.max_pages;
    const int last_row = min(r0 + LM_ROWS, n_rows) - 1;
    const int hi = start + last_row / nh + 1;           // keys 0 .. hi-1 are seen by some row of the tile
    const int chunks = kd / 8;

    // the queries: the tile's rows are consecutive in memory
    {
        const bf16* src = q_lat + ((size_t)tok0 * nh + r0) * kd;
        const int rows_here = last_row - r0 + 1;
        for (int c = tid; c < LM_ROWS * chunks; c += LM_THREADS) {
            const int r = c / chunks, ch = c - r * chunks;
            cp_async16(sQ + r * lds + ch * 8, src + (size_t)r * kd + ch * 8, r < rows_here);
        }
    }
    // The key rows of a tile arrive as bulk copies, one per row, issued by the lanes of warp 0 (a lane per key: the 32
    // page look-ups go out together) and completing on the stage's mbarrier; rows past the tile's last key keep what
    // an earlier tile left there (finite numbers, and every weight on them is zero).
    const uint32_t row_bytes = (uint32_t)kd * sizeof(bf16);
    auto load_keys = [&](int kt, int stage) {
        if (warp != 0) return;
        const int j = kt * LM_KEYS + lane;
        bool ok = j < hi;
        const bf16* src = pool;
        if (ok) {
            const int page = bt[j / ps];
            if (page >= 0) src = latent_row(pool, cache, page, j % ps);
            else { ok = false; if (status) *status = 1; }
        }
        const uint32_t bar = tc_smem(&s_bar[stage]);
        const unsigned live = __ballot_sync(0xffffffffu, ok);
        if (lane == 0) tc_mbar_expect_tx(bar, __popc(live) * row_bytes);
        __syncwarp();
        if (ok) bulk_row_copy(smem_u32(sK + (stage * LM_KEYS + lane) * lds), src, row_bytes, bar);
    };
    // the tile's key range, cut over blockIdx.y into parts of whole key tiles
    const int all_kt = (hi + LM_KEYS - 1) / LM_KEYS;
    const int per = (all_kt + n_splits - 1) / n_splits;
    const int kt_begin = blockIdx.y * per, n_kt = min(all_kt, kt_begin + per);
    if (kt_begin < n_kt) load_keys(kt_begin, 0);
    cp_async_commit();

    const int row_a = rg * 16 + g, row_b = row_a + 8;
    const int pos_a = r0 + row_a <= last_row ? start + (r0 + row_a) / nh : -1;
    const int pos_b = r0 + row_b <= last_row ? start + (r0 + row_b) / nh : -1;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    // lane-dependent parts of the ldmatrix addresses
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;      // A operands, and V (transposed)
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;      // K as the B operand

    for (int kt = kt_begin; kt < n_kt; ++kt) {
        const int stage = (kt - kt_begin) & 1;
        cp_async_wait<0>();              // the queries (first turn)
        if (!tc_wait(tc_smem(&s_bar[stage]), ((kt - kt_begin) >> 1) & 1) && status) *status = 6;   // gave up: the step is invalid
        __syncthreads();                 // this tile has landed, and every warp is through with the tile before
        if (kt + 1 < n_kt) load_keys(kt + 1, stage ^ 1);      // into the stage the tile before was read from
        cp_async_commit();
        const bf16* kb = sK + stage * LM_KEYS * lds;
        float s[NKT][4];
        {
            // two steps of k per turn on accumulators of their own: independent chains of products
            float s2[NKT][4];
#pragma unroll
            for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] = s2[nt][e] = 0.f;
            const uint32_t qa = smem_u32(sQ + (rg * 16 + a_row) * lds + a_col);
            const uint32_t ka = NKT == 2 ? smem_u32(kb + (half * KW + b_row) * lds + b_col)
                                         : smem_u32(kb + (half * KW + (lane & 7)) * lds + ((lane >> 3) & 1) * 8);
#pragma unroll 2
            for (int k0 = 0; k0 < kdp; k0 += 32) {
                uint32_t a[4], a2[4], b0, b1, b2 = 0, b3 = 0, c0, c1, c2 = 0, c3 = 0;
                ldmatrix_x4_s(a[0], a[1], a[2], a[3], qa + k0 * 2);
                ldmatrix_x4_s(a2[0], a2[1], a2[2], a2[3], qa + k0 * 2 + 32);
                if (NKT == 2) {
                    ldmatrix_x4_s(b0, b1, b2, b3, ka + k0 * 2);
                    ldmatrix_x4_s(c0, c1, c2, c3, ka + k0 * 2 + 32);
                } else {
                    ldmatrix_x2_s(b0, b1, ka + k0 * 2);
                    ldmatrix_x2_s(c0, c1, ka + k0 * 2 + 32);
                }
                mma_bf16(s[0], a, b0, b1);
                mma_bf16(s2[0], a2, c0, c1);
                if (NKT == 2) {
                    mma_bf16(s[NKT - 1], a, b2, b3);
                    mma_bf16(s2[NKT - 1], a2, c2, c3);
                }
            }
#pragma unroll
            for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] += s2[nt][e];
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = kt * LM_KEYS + half * KW + nt * 8 + 2 * tq + (e & 1);
                const int limit = e < 2 ? pos_a : pos_b;
                const float v = j <= limit ? s[nt][e] * scale_log2 : -INFINITY;
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        }
        if (tq == 0) {
            smax[half * LM_ROWS + row_a] = mx[0];
            smax[half * LM_ROWS + row_b] = mx[1];
        }
        __syncthreads();
        float corr[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = i ? row_b : row_a;
            float mn = m[i];
#pragma unroll
            for (int p = 0; p < NP; ++p) mn = fmaxf(mn, smax[p * LM_ROWS + row]);
            // m is the reference the row's weights are taken against, not its exact maximum: it moves only when the
            // maximum has grown by more than LM_LAZY (in powers of two), so that the accumulator is rarely rescaled;
            // weights stay below 2^LM_LAZY, and the reference cancels in the end like a maximum does
            if (m[i] == -INFINITY) {
                corr[i] = 1.f;                 // nothing accumulated yet
                m[i] = mn;
            } else if (mn > m[i] + LM_LAZY) {
                corr[i] = fast_exp2(m[i] - mn);
                m[i] = mn;
            } else {
                corr[i] = 1.f;
            }
        }
        float add[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < NKT; ++nt) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = s[nt][e] == -INFINITY ? 0.f : fast_exp2(s[nt][e] - m[e >> 1]);
                add[e >> 1] += p[e];
            }
            const int col = half * KW + nt * 8 + 2 * tq;
            *reinterpret_cast<uint32_t*>(sP + row_a * LM_PLD + col) = pack_bf16(p[0], p[1]);
            *reinterpret_cast<uint32_t*>(sP + row_b * LM_PLD + col) = pack_bf16(p[2], p[3]);
        }
        l[0] = l[0] * corr[0] + add[0];
        l[1] = l[1] * corr[1] + add[1];
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {     // only when a row's maximum moved
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            uint32_t a[4];
            ldmatrix_x4(a[0], a[1], a[2], a[3], sP + (rg * 16 + a_row) * LM_PLD + kk * 16 + a_col);
            const uint32_t va = smem_u32(kb + (kk * 16 + a_row) * lds + half * NT * 8 + a_col);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans_s(b0, b1, b2, b3, va + np * 32);
                mma_bf16(o[2 * np], a, b0, b1);
                mma_bf16(o[2 * np + 1], a, b2, b3);
            }
        }
        // no barrier here: the next turn's first one stands between these reads and the next writes
    }
    // the halves' sums meet; the sink joins the denominator; the gate multiplies
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    if (tq == 0) {
        ssum[half * LM_ROWS + row_a] = l[0];
        ssum[half * LM_ROWS + row_b] = l[1];
    }
    __syncthreads();
    auto part_sum = [&](int row) {
        float t = 0.f;
#pragma unroll
        for (int p = 0; p < NP; ++p) t += ssum[p * LM_ROWS + row];
        return t;
    };
    if (n_splits > 1) {
        // this part's maximum, sum and unnormalised rows go to scratch; latent_merge finishes the rows
        float* base = partial + ((size_t)blockIdx.x * n_splits + blockIdx.y) * LM_ROWS * (NT * 8 * NP + 2);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = i ? row_b : row_a;
            if (r0 + row > last_row) continue;
            float* dst = base + (size_t)row * (NT * 8 * NP + 2);
            if (half == 0 && tq == 0) { dst[0] = m[i]; dst[1] = part_sum(row); }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int col = half * NT * 8 + nt * 8 + 2 * tq;
                if (col < kr) *reinterpret_cast<float2*>(dst + 2 + col) = make_float2(o[nt][2 * i], o[nt][2 * i + 1]);
            }
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = i ? row_b : row_a;
        if (r0 + row > last_row) continue;
        const int tok = tok0 + (r0 + row) / nh, h = (r0 + row) % nh;
        const float snk = sink ? sink[h] * 1.4426950408889634f : -INFINITY;
        const float mf = fmaxf(m[i], snk);
        const float c = m[i] == -INFINITY ? 0.f : exp2f(m[i] - mf);
        const float den = part_sum(row) * c + (snk > -INFINITY ? exp2f(snk - mf) : 0.f);
        float gate = 1.f;
        if (gates) gate = 1.f / (1.f + expf(-load1_cg(gates + (size_t)tok * gate_ld + h)));
        const float k = den > 0.f ? c * gate / den : 0.f;
        bf16* dst = out + ((size_t)tok * nh + h) * kr;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int col = half * NT * 8 + nt * 8 + 2 * tq;
            if (col < kr)
                *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(o[nt][2 * i] * k, o[nt][2 * i + 1] * k);
        }
    }
}

// Finishes the rows of tiles whose key range was cut into parts: the parts' maxima, sums and unnormalised rows
// are combined, the sink joins the denominator, the gate multiplies.  One block per (tile, row): a thread owns pairs
// of columns and asks for all parts' values at once.
#define LM_MERGE_THREADS 128
#define LM_MAX_SPLITS 64
__global__ void __launch_bounds__(LM_MERGE_THREADS)
latent_merge_kernel(const float* __restrict__ partial, int n_splits, int dvp, bf16* __restrict__ out,
                    const int* __restrict__ positions, const int* __restrict__ q_start, int n_seqs,
                    const float* __restrict__ sink, const bf16* __restrict__ gates, int gate_ld, int nh, int kr) {
    __shared__ int s_req, s_tile;
    __shared__ float s_w[LM_MAX_SPLITS];
    __shared__ float s_k;
    if (threadIdx.x == 0) {
        int tile = gridDim.x - 1 - blockIdx.x, req = -1;      // as in the attention kernel
        for (int i = 0; i < n_seqs; ++i) {
            const int rows = (q_start[i + 1] - q_start[i]) * nh;
            const int tiles = (rows + LM_ROWS - 1) / LM_ROWS;
            if (tile < tiles) { req = i; break; }
            tile -= tiles;
        }
        s_req = req;
        s_tile = tile;
    }
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    __syncthreads();
    const int b = s_req;
    if (b < 0) return;
    const int tok0 = q_start[b], n_rows = (q_start[b + 1] - tok0) * nh, r0 = s_tile * LM_ROWS;
    const int row = blockIdx.y;
    if (positions[tok0] < 0 || r0 + row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const size_t stride = (size_t)LM_ROWS * (dvp + 2);
    const float* pr = partial + (size_t)blockIdx.x * n_splits * stride + (size_t)row * (dvp + 2);
    const int tok = tok0 + (r0 + row) / nh, h = (r0 + row) % nh;
    if (threadIdx.x < 32) {
        // a lane per part (two turns): maxima, weights, the denominator
        const float snk = sink ? sink[h] * 1.4426950408889634f : -INFINITY;
        float ms[2], ls[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int sp = lane + 32 * u;
            ms[u] = sp < n_splits ? __ldcg(pr + sp * stride) : -INFINITY;
            ls[u] = sp < n_splits ? __ldcg(pr + sp * stride + 1) : 0.f;
        }
        const float mf = fmaxf(snk, warp_max(fmaxf(ms[0], ms[1])));
        float den = 0.f;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const float w = ms[u] > -INFINITY ? exp2f(ms[u] - mf) : 0.f;
            s_w[lane + 32 * u] = w;
            den += w * ls[u];
        }
        den = warp_sum(den) + (snk > -INFINITY ? exp2f(snk - mf) : 0.f);
        float gate = 1.f;
        if (gates) gate = 1.f / (1.f + expf(-load1_cg(gates + (size_t)tok * gate_ld + h)));
        if (lane == 0) s_k = den > 0.f ? gate / den : 0.f;
    }
    __syncthreads();
    const float k = s_k;
    bf16* dst = out + ((size_t)tok * nh + h) * kr;
    for (int col = 2 * threadIdx.x; col < kr; col += 2 * LM_MERGE_THREADS) {
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll 8
        for (int sp = 0; sp < n_splits; ++sp) {                 // every part wrote its rows (zeros if it was empty)
            const float2 v = __ldcg(reinterpret_cast<const float2*>(pr + sp * stride + 2 + col));
            acc.x = fmaf(s_w[sp], v.x, acc.x);
            acc.y = fmaf(s_w[sp], v.y, acc.y);
        }
        *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(acc.x * k, acc.y * k);
    }
}

// the launch's shape for a latent width: parts per row group, value n-tiles per warp (0: not taken)
static int lm_np(int kr) { (void)kr; return 2; }
static int lm_nt(int kr) {
    const int sizes[] = {2, 4, 6, 8, 12, 16, 24, 32};    // 32 ... 512 columns
    for (int nt : sizes)
        if (nt * 16 >= kr) return nt;
    return 0;
}
static int lm_dv(int kr) { return lm_nt(kr) * 8 * lm_np(kr); }
static int lm_row_stride(int kr, int rot) {
    const int kdp = (kr + rot + 31) / 32 * 32, dv = lm_dv(kr);
    return (kdp > dv ? kdp : dv) + 8;
}
static size_t lm_smem(int kr, int rot) {
    return (size_t)(LM_ROWS + 2 * LM_KEYS) * lm_row_stride(kr, rot) * sizeof(bf16) + LM_ROWS * LM_PLD * sizeof(bf16) +
           2 * lm_np(kr) * LM_ROWS * sizeof(float);
}

// bfloat16; kr a multiple of 16 up to 512; kr + rot a multiple of 8; the tiles must fit the shared memory of an SM
ST_EXPORT int st_latent_attention_mma_applies(int kr, int rot) {
    if (kr <= 0 || kr % 16 || rot < 0 || (kr + rot) % 8 || !lm_nt(kr)) return 0;
    return lm_smem(kr, rot) <= 200 * 1024;
}

static long long lm_tiles(int n_tokens, int n_seqs, int nh) {
    return ((long long)n_tokens * nh + LM_ROWS - 1) / LM_ROWS + n_seqs;
}

// Into how many parts the key ranges of a step of this shape are cut: one when the tiles fill the device by
// themselves (prompt portions), else as many as bring the launch to about a block per SM, 16 at most.  It depends on
// the step's shape only (never on lengths), so a recorded step keeps it.
ST_EXPORT int st_latent_attention_mma_splits(int n_tokens, int n_seqs, int nh) {
    const long long tiles = lm_tiles(n_tokens, n_seqs, nh);
    long long n = st_sm_count() / (tiles > 0 ? tiles : 1);
    return (int)(n < 1 ? 1 : n > 16 ? 16 : n);
}

// floats of scratch a launch with n_splits > 1 needs
ST_EXPORT long long st_latent_attention_mma_scratch(int n_tokens, int n_seqs, int nh, int kr, int n_splits) {
    if (n_splits <= 1) return 0;
    return lm_tiles(n_tokens, n_seqs, nh) * n_splits * LM_ROWS * (lm_dv(kr) + 2);
}

ST_EXPORT int st_latent_attention_mma(const void* q_lat, const void* pool, long long page_stride, long long entry_offset,
                                      void* out, const int* positions, const int* q_start, const int* start_pos,
                                      const int* slots, const int* block_table, int max_pages, int n_tokens, int n_seqs,
                                      int nh, int kr, int rot, int page_size, const float* sink, const void* gates,
                                      int gate_ld, float scale, int n_splits, float* partial, int* status, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (!st_latent_attention_mma_applies(kr, rot) || page_stride % 8 || entry_offset % 8) return ST_ERR_BAD_SIZE;
    if (!aligned16(q_lat) || !aligned16(pool) || n_splits < 1 || n_splits > 64 || (n_splits > 1 && !partial)) return ST_ERR_BAD_ARG;
    LatentCache c{max_pages, page_size, kr, rot, page_stride, entry_offset};
    const int nt = lm_nt(kr), np = lm_np(kr), lds = lm_row_stride(kr, rot), kdp = (kr + rot + 31) / 32 * 32;
    const size_t smem = lm_smem(kr, rot);
    const long long tiles = lm_tiles(n_tokens, n_seqs, nh);
    if (tiles > 0x7fffffff) return ST_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    const float scale_log2 = scale * 1.4426950408889634f;
    int rc = ST_ERR_BAD_SIZE;
#define LM_LAUNCH(NTV, NPV)                                                                                          \
    if (nt == NTV && np == NPV) {                                                                                    \
        static bool set = false;                                                                                     \
        if (!set) {                                                                                                  \
            cudaFuncSetAttribute(latent_attention_mma_kernel<NTV, NPV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            set = true;                                                                                              \
        }                                                                                                            \
        rc = st_launch_pdl("latent_mma", latent_attention_mma_kernel<NTV, NPV>, dim3((unsigned)tiles, n_splits), dim3(NPV * 128), \
                           smem, s, (const bf16*)q_lat, (const bf16*)pool, c, (bf16*)out, positions, q_start, start_pos,  \
                           slots, block_table, n_seqs, sink, (const bf16*)gates, gate_ld, nh, scale_log2, lds, kdp,      \
                           n_splits, partial, status);                                                               \
    }
    LM_LAUNCH(2, 2) LM_LAUNCH(4, 2) LM_LAUNCH(6, 2) LM_LAUNCH(8, 2)
    LM_LAUNCH(12, 2) LM_LAUNCH(16, 2) LM_LAUNCH(24, 2) LM_LAUNCH(32, 2)
#undef LM_LAUNCH
    if (rc != 0 || n_splits == 1) return rc;
    return st_launch_pdl("latent_merge", latent_merge_kernel, dim3((unsigned)tiles, LM_ROWS), dim3(LM_MERGE_THREADS), 0, s,
                         (const float*)partial, n_splits, nt * 8 * np, (bf16*)out, positions, q_start, n_seqs, sink,
                         (const bf16*)gates, gate_ld, nh, kr);
}
