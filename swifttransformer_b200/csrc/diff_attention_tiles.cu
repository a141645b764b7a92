// Differential attention for prompt portions on the warp-level tensor cores (mma.sync m16n8k16, bfloat16 in,
// float accumulate): one block per (64 query rows of one request, query head).
//
// Eight warps: warps 0-3 carry map 1 of rows 0-15 / 16-31 / 32-47 / 48-63, warps 4-7 map 2 of the same rows.
// All eight read the same key tile (64 keys, the two maps' keys side by side) and the same value tile from
// shared memory, filled by 16-byte asynchronous copies from the pages (two stages: the next tile lands while
// this one is multiplied).  Each warp keeps S = Q K^T of its map, the running maximum and sum and
// O = P V (16 x vd) in registers.  At the end the map-2 warps hand their normalised O to the map-1 warps through
// shared memory, which form o = O1 - lambda O2, normalise each row over vd and store it.
//
// Sizes are template arguments rounded up (dim to 32/64/128, vd to 32/64/128/256) with the padding columns
// zero in shared memory; dim and vd themselves must be multiples of 8 (16-byte pieces).  Scores, the cap, the
// softmax and the final norm are float; the cap's tanh and the weights' exponentials use the fast exp2.
#include "diff_attention.cuh"
#include "mma_sync.cuh"

#define DT_ROWS 64      // query rows per block
#define DT_KEYS 64      // keys per tile
#define DT_THREADS 256

// x: a score times log2(e); returns log2(e) * cap * tanh(score / cap) by tanh(y) = 1 - 2 / (1 + e^(2y)) with the
// fast exponential and division (cap_l2 = log2(e) * cap, two_over_cap = 2 / cap_l2; cap_l2 <= 0: no cap)
__device__ __forceinline__ float fast_cap(float x, float cap_l2, float two_over_cap) {
    if (cap_l2 <= 0.f) return x;
    const float e = fast_exp2(x * two_over_cap * 1.4426950408889634f);
    return cap_l2 * (1.f - __fdividef(2.f, 1.f + e));
}

template <int DIMT, int VDT>
struct DiffTileSmem {
    static constexpr int K_LD = 2 * DIMT + 8;       // elements per key row (both maps), padded against bank conflicts
    static constexpr int V_LD = VDT + 8;
    static constexpr int STAGE = DT_KEYS * (K_LD + V_LD);
    static constexpr size_t BYTES = 2 * (size_t)STAGE * sizeof(bf16);
};

template <int DIMT, int VDT>
__device__ __forceinline__ void load_kv_tile(bf16* stage, const bf16* __restrict__ pool, const DiffCache& cache,
                                             const int* __restrict__ bt, int kvh, int key0, int lo, int hi, int dim,
                                             int* __restrict__ status) {
    using L = DiffTileSmem<DIMT, VDT>;
    bf16* sk = stage;
    bf16* sv = stage + DT_KEYS * L::K_LD;
    constexpr int KC = 2 * DIMT / 8, VC = VDT / 8;      // 16-byte pieces per row
    const int vd = cache.vd, ps = cache.page_size;
    // four threads per key row: one look-up of the row's page, then the row's pieces in turn
    const int row = threadIdx.x >> 2;
    const int key = key0 + row;
    int page = -1;
    if (key >= lo && key <= hi) {
        page = bt[key / ps];
        if (page < 0 && status) *status = 1;            // a hole in the block table: the key counts as zeros
    }
    const bf16* krow = page >= 0 ? cache_keys(pool, cache, page, kvh, key % ps) : nullptr;
    const bf16* vrow = page >= 0 ? cache_values(pool, cache, page, kvh, key % ps) : nullptr;
    for (int c = threadIdx.x & 3; c < KC + VC; c += 4) {
        if (c < KC) {
            const int map = c / (DIMT / 8), e = (c % (DIMT / 8)) * 8;
            bf16* dst = sk + row * L::K_LD + map * DIMT + e;
            if (page >= 0 && e < dim) cp_async16(dst, krow + map * dim + e, true);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        } else {
            const int e = (c - KC) * 8;
            bf16* dst = sv + row * L::V_LD + e;
            if (page >= 0 && e < vd) cp_async16(dst, vrow + e, true);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
}

template <int DIMT, int VDT>
__global__ void __launch_bounds__(DT_THREADS)
diff_attention_tiles_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, DiffCache cache,
                            bf16* __restrict__ out, const int* __restrict__ tiles, int halves,
                            const int* __restrict__ q_start, const int* __restrict__ start_pos,
                            const int* __restrict__ slots, const int* __restrict__ block_table, int nh, int dim,
                            float scale, float cap, int block, int window, float lambda, float eps, float out_scale,
                            int* __restrict__ status) {
    using L = DiffTileSmem<DIMT, VDT>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    ST_PDL_TRIGGER();
    const int tile = blockIdx.x / halves, part = blockIdx.x % halves;
    const int req = tiles[2 * tile], off = tiles[2 * tile + 1] + part * DT_ROWS;
    const int first = q_start[req], n_new = q_start[req + 1] - first;
    if (off >= n_new) return;                           // padding tile, or the part lies past the request's tokens
    const int h = blockIdx.y, nkv = cache.nkv, vd = cache.vd;
    const int kvh = h / (nh / nkv);
    const int start = start_pos[req];
    const int* bt = block_table + (size_t)slots[req] * cache.max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int map = warp >> 2, row0 = (warp & 3) * 16;
    const int rows_here = min(DT_ROWS, n_new - off);
    const int p_first = start + off, p_last = p_first + rows_here - 1;
    const int lo = first_visible(p_first, block, window), hi = p_last;

    // this thread's two query rows (g and g + 8 of the warp's sixteen)
    int pos[2], vis[2];
    bool live[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + g + 8 * r;
        live[r] = row < rows_here;
        pos[r] = p_first + row;
        vis[r] = first_visible(pos[r], block, window);
    }
    // what decides whether a key tile needs a mask for this warp's sixteen rows
    const bool w_all_live = row0 + 15 < rows_here;
    const int w_pos_min = p_first + row0, w_vis_max = first_visible(p_first + row0 + 15, block, window);
    // Q fragments of the warp's map, from global memory (once)
    uint32_t qa[DIMT / 16][4];
#pragma unroll
    for (int ks = 0; ks < DIMT / 16; ++ks)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int r = x & 1, col = ks * 16 + 2 * tq + 8 * (x >> 1);
            const int row = row0 + g + 8 * r;
            uint32_t v = 0;
            if (live[r] && col < dim)
                v = __ldcg(reinterpret_cast<const uint32_t*>(q + ((size_t)(first + off + row) * nh + h) * 2 * dim + map * dim + col));
            qa[ks][x] = v;
        }

    float o[VDT / 8][4];
#pragma unroll
    for (int nt = 0; nt < VDT / 8; ++nt)
#pragma unroll
        for (int x = 0; x < 4; ++x) o[nt][x] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    // scores are kept in units of log2(e): s' = log2(e) * cap * tanh(scale * qk / cap), so that the weights are exp2
    const float LOG2E = 1.4426950408889634f;
    const float scale_l2 = scale * LOG2E, cap_l2 = cap * LOG2E, two_over_cap = cap > 0.f ? 2.f / cap_l2 : 0.f;

    const int kt_first = lo / DT_KEYS, kt_last = hi / DT_KEYS;
    load_kv_tile<DIMT, VDT>(smem, pool, cache, bt, kvh, kt_first * DT_KEYS, lo, hi, dim, status);
    cp_async_commit();
    for (int kt = kt_first; kt <= kt_last; ++kt) {
        bf16* stage = smem + ((kt - kt_first) & 1) * L::STAGE;
        if (kt < kt_last)
            load_kv_tile<DIMT, VDT>(smem + ((kt + 1 - kt_first) & 1) * L::STAGE, pool, cache, bt, kvh, (kt + 1) * DT_KEYS,
                                    lo, hi, dim, status);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* sk = stage + map * DIMT;
        const bf16* sv = stage + DT_KEYS * L::K_LD;
        const int key0 = kt * DT_KEYS;
        // S = Q K^T for the tile's 64 keys
        float s[DT_KEYS / 8][4];
#pragma unroll
        for (int nt = 0; nt < DT_KEYS / 8; ++nt) {
#pragma unroll
            for (int x = 0; x < 4; ++x) s[nt][x] = 0.f;
#pragma unroll
            for (int ks = 0; ks < DIMT / 16; ++ks) {
                const bf16* kp = sk + (nt * 8 + g) * L::K_LD + ks * 16 + 2 * tq;
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kp);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kp + 8);
                mma_bf16(s[nt], qa[ks], b0, b1);
            }
        }
        // scale, cap, mask; running maximum.  A tile that lies wholly inside the range of every row of the warp
        // needs no mask.
        float tmax[2] = {-INFINITY, -INFINITY};
        if (w_all_live && key0 + DT_KEYS - 1 <= w_pos_min && key0 >= w_vis_max) {
#pragma unroll
            for (int nt = 0; nt < DT_KEYS / 8; ++nt)
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float v = fast_cap(s[nt][x] * scale_l2, cap_l2, two_over_cap);
                    s[nt][x] = v;
                    tmax[x >> 1] = fmaxf(tmax[x >> 1], v);
                }
        } else {
#pragma unroll
            for (int nt = 0; nt < DT_KEYS / 8; ++nt)
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const int r = x >> 1, key = key0 + nt * 8 + 2 * tq + (x & 1);
                    const bool seen = live[r] && key >= vis[r] && key <= pos[r];
                    const float v = seen ? fast_cap(s[nt][x] * scale_l2, cap_l2, two_over_cap) : -INFINITY;
                    s[nt][x] = v;
                    tmax[r] = fmaxf(tmax[r], v);
                }
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
            const float m_new = fmaxf(m[r], tmax[r]);
            corr[r] = m[r] == -INFINITY ? 0.f : fast_exp2(m[r] - m_new);
            m[r] = m_new;
        }
        float tsum[2] = {0.f, 0.f};
        uint32_t pa[DT_KEYS / 16][4];
#pragma unroll
        for (int nt = 0; nt < DT_KEYS / 8; ++nt) {
            float p[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int r = x >> 1;
                p[x] = s[nt][x] == -INFINITY ? 0.f : fast_exp2(s[nt][x] - m[r]);
                tsum[r] += p[x];
            }
            pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
            pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            tsum[r] += __shfl_xor_sync(0xffffffffu, tsum[r], 1);
            tsum[r] += __shfl_xor_sync(0xffffffffu, tsum[r], 2);
            l[r] = l[r] * corr[r] + tsum[r];
        }
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {     // a maximum of the warp's rows moved
#pragma unroll
            for (int nt = 0; nt < VDT / 8; ++nt) {
                o[nt][0] *= corr[0]; o[nt][1] *= corr[0];
                o[nt][2] *= corr[1]; o[nt][3] *= corr[1];
            }
        }
        // O += P V: V [key][vd] is the k-major operand, read transposed
#pragma unroll
        for (int ks = 0; ks < DT_KEYS / 16; ++ks)
#pragma unroll
            for (int nt2 = 0; nt2 < VDT / 16; ++nt2) {
                uint32_t b0, b1, b2, b3;
                const bf16* vp = sv + (ks * 16 + (lane & 15)) * L::V_LD + nt2 * 16 + (lane >> 4) * 8;
                ldmatrix_x4_trans(b0, b1, b2, b3, vp);
                mma_bf16(o[2 * nt2], pa[ks], b0, b1);
                mma_bf16(o[2 * nt2 + 1], pa[ks], b2, b3);
            }
        __syncthreads();            // the stage may be refilled
    }
    cp_async_wait<0>();
    __syncthreads();
    // map 2 hands its normalised result over; map 1 combines, normalises over vd and stores
    float* so = reinterpret_cast<float*>(smem_raw);      // [64][VDT + 1]
    const float inv[2] = {l[0] > 0.f ? 1.f / l[0] : 0.f, l[1] > 0.f ? 1.f / l[1] : 0.f};
    if (map == 1) {
#pragma unroll
        for (int nt = 0; nt < VDT / 8; ++nt)
#pragma unroll
            for (int x = 0; x < 4; ++x)
                so[(row0 + g + 8 * (x >> 1)) * (VDT + 1) + nt * 8 + 2 * tq + (x & 1)] = o[nt][x] * inv[x >> 1];
    }
    __syncthreads();
    if (map == 0) {
        float ss[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < VDT / 8; ++nt)
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int r = x >> 1;
                const float v = o[nt][x] * inv[r] - lambda * so[(row0 + g + 8 * r) * (VDT + 1) + nt * 8 + 2 * tq + (x & 1)];
                o[nt][x] = v;
                ss[r] = fmaf(v, v, ss[r]);
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], 1);
            ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], 2);
            ss[r] = rsqrtf(ss[r] / (float)vd + eps) * out_scale;
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (!live[r]) continue;
            bf16* orow = out + ((size_t)(first + off + row0 + g + 8 * r) * nh + h) * vd;
#pragma unroll
            for (int nt = 0; nt < VDT / 8; ++nt) {
                const int e = nt * 8 + 2 * tq;
                if (e < vd)
                    *reinterpret_cast<uint32_t*>(orow + e) = pack_bf16(o[nt][2 * r] * ss[r], o[nt][2 * r + 1] * ss[r]);
            }
        }
    }
}

template <int DIMT, int VDT>
static int launch_diff_tiles(const void* q, const void* pool, const DiffCache& c, void* out, const int* tiles, int n_tiles,
                             int tile_rows, const int* q_start, const int* start_pos, const int* slots,
                             const int* block_table, int nh, int dim, float scale, float cap, int block, int window,
                             float lambda, float eps, float out_scale, int* status, cudaStream_t s) {
    using L = DiffTileSmem<DIMT, VDT>;
    size_t smem = L::BYTES;
    const size_t hand = (size_t)DT_ROWS * (VDT + 1) * sizeof(float);
    if (hand > smem) smem = hand;
    auto kern = diff_attention_tiles_kernel<DIMT, VDT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int halves = (tile_rows + DT_ROWS - 1) / DT_ROWS;
    kern<<<dim3(n_tiles * halves, nh), DT_THREADS, smem, s>>>((const bf16*)q, (const bf16*)pool, c, (bf16*)out, tiles, halves,
                                                             q_start, start_pos, slots, block_table, nh, dim, scale, cap,
                                                             block, window, lambda, eps, out_scale, status);
    return st_launch_status();
}

ST_EXPORT int st_diff_attention_tiles_applies(int dim, int vd) {
    return dim > 0 && vd > 0 && dim % 8 == 0 && vd % 8 == 0 && dim <= 128 && vd <= 256;
}

// tiles: int32 [n_tiles][2] = (request of the step, offset of a tile of `tile_rows` query rows among its new tokens);
// a tile whose offset lies past the request's tokens is padding
ST_EXPORT int st_diff_attention_tiles(const void* q, const void* pool, long long page_stride, long long entry_offset,
                                      void* out, const int* tiles, int n_tiles, int tile_rows, const int* q_start,
                                      const int* start_pos, const int* slots, const int* block_table, int max_pages,
                                      int nh, int nkv, int dim, int vd, int page_size, float scale, float cap, int block,
                                      int window, float lambda, float eps, float out_scale, int* status, void* stream) {
    if (n_tiles <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || tile_rows <= 0) return ST_ERR_BAD_ARG;
    if (!st_diff_attention_tiles_applies(dim, vd)) return ST_ERR_BAD_SIZE;
    const DiffCache c = {max_pages, page_size, nkv, 2 * dim, vd, page_stride, entry_offset};
    cudaStream_t s = (cudaStream_t)stream;
#define DT_ARGS q, pool, c, out, tiles, n_tiles, tile_rows, q_start, start_pos, slots, block_table, nh, dim, scale, cap, block, \
                window, lambda, eps, out_scale, status, s
#define DT_PICK_V(DIMT)                                                    \
    do {                                                                   \
        if (vd <= 32) return launch_diff_tiles<DIMT, 32>(DT_ARGS);         \
        if (vd <= 64) return launch_diff_tiles<DIMT, 64>(DT_ARGS);         \
        if (vd <= 128) return launch_diff_tiles<DIMT, 128>(DT_ARGS);       \
        return launch_diff_tiles<DIMT, 256>(DT_ARGS);                      \
    } while (0)
    if (dim <= 32) DT_PICK_V(32);
    if (dim <= 64) DT_PICK_V(64);
    DT_PICK_V(128);
#undef DT_PICK_V
#undef DT_ARGS
}
