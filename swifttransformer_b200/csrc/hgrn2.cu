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

// ------------------------------------------------------------------------------------------------
// The same recurrence with the state in registers and the work of a head spread over blocks: a block of four
// warps owns a few columns of S for one (request, head); LANES lanes (8 or 32) share a column, each with R
// consecutive rows of it in registers (dim <= LANES * R), and meet by shuffles for o = S^T q.  Many small blocks:
// every step of the recurrence waits for the one before, and only other warps on the same scheduler hide that.
// The blocks of a head cannot normalise its output (each sees a slice of it): they leave o in float and
// `hgrn2_norm_kernel` follows.  Per token the order of the sums is fixed, whatever the portion or the batch.
template <int R, int LANES> struct HcLayout {
    static constexpr int CPW = 32 / LANES;                  // columns a warp owns
    static constexpr int COLS = 4 * CPW;                    // columns a block (four warps) owns
    static constexpr int LS = R == 4 ? 4 : (R > 4 ? R + 4 : R + 1);   // floats between consecutive lanes' rows (bank spread)
    static constexpr int ROW = LANES * LS;                  // floats per token
    static constexpr int DIMP = LANES * R;                  // dim rounded up
};

template <typename T, int R, int LANES>
__global__ void __launch_bounds__(128)
hgrn2_cols_kernel(const T* __restrict__ proj, int ld, int q_off, int f_off, int v_off, const float* __restrict__ f_bias,
                  const float* __restrict__ lower, const float* __restrict__ gates, float* __restrict__ state,
                  float* __restrict__ o_raw, const int* __restrict__ positions, const int* __restrict__ q_start,
                  const int* __restrict__ slots, int nh, int dim, int vd) {
    using L = HcLayout<R, LANES>;
    constexpr int DIMP = L::DIMP, COLS = L::COLS, CPW = L::CPW;
    constexpr int TOK_PASS = 128 / DIMP, PASSES = HG_GROUP / TOK_PASS;      // 128 threads cover 128 / DIMP tokens a pass
    constexpr int VTOK = 128 / COLS, VPASSES = VTOK >= HG_GROUP ? 1 : HG_GROUP / VTOK;
    __shared__ __align__(16) float sq[HG_GROUP * L::ROW];
    __shared__ __align__(16) float sf[HG_GROUP * L::ROW];
    __shared__ float sv[HG_GROUP * COLS];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int first = q_start[b], n = q_start[b + 1] - first;
    if (n <= 0 || positions[first] < 0) return;           // padding of a fixed-shape step
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int l = lane / CPW, cw = warp * CPW + lane % CPW, col = c0 + cw;
    float* st = state + ((size_t)slots[b] * nh + h) * dim * vd;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = l * R + r;
        S[r] = (i < dim && col < vd) ? __ldcg(st + (size_t)i * vd + col) : 0.f;
    }
    // what this thread prepares of every group: row i of the gates and queries of the tokens k0, k0 + TOK_PASS, ...,
    // and some values; the raw projections of the NEXT group are fetched before this group's recurrence runs
    const int i_mine = tid % DIMP, k0 = tid / DIMP;
    const bool row_live = i_mine < dim;
    const float fb = row_live ? f_bias[h * dim + i_mine] : 0.f, lo = row_live ? lower[h * dim + i_mine] : 0.f;
    const int at_mine = (i_mine / R) * L::LS + i_mine % R;
    const int vk = tid / COLS, vj = c0 + tid % COLS;
    float zq[PASSES], zf[PASSES], zv[VPASSES];
    auto fetch = [&](int r0) {
        const int rn = min(HG_GROUP, n - r0);
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int k = k0 + p * TOK_PASS;
            zq[p] = zf[p] = 0.f;
            if (k < rn && row_live) {
                if (gates) {                                  // silu(q) and the gate, prepared for all tokens at once
                    const float* grow = gates + (size_t)(first + r0 + k) * 2 * nh * dim + h * dim + i_mine;
                    zq[p] = __ldcg(grow);
                    zf[p] = __ldcg(grow + nh * dim);
                } else {
                    const T* row = proj + (size_t)(first + r0 + k) * ld + h * dim + i_mine;
                    zq[p] = load1_cg(row + q_off);              // through L2 only: the product just before wrote them
                    zf[p] = load1_cg(row + f_off);
                }
            }
        }
#pragma unroll
        for (int p = 0; p < VPASSES; ++p) {
            const int k = vk + p * VTOK;
            zv[p] = (k < rn && vj < vd) ? load1_cg(proj + (size_t)(first + r0 + k) * ld + v_off + h * vd + vj) : 0.f;
        }
    };
    fetch(0);
    for (int r0 = 0; r0 < n; r0 += HG_GROUP) {
        const int rn = min(HG_GROUP, n - r0);
        __syncthreads();                                  // the group before has been read
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int k = k0 + p * TOK_PASS;
            float qv = 0.f, fv = 1.f;                     // rows past dim: nothing written, nothing read
            if (row_live && gates) {
                qv = zq[p];
                fv = zf[p];
            } else if (row_live) {
                qv = zq[p] / (1.f + expf(-zq[p]));
                fv = lo + (1.f - lo) * (1.f / (1.f + expf(-(zf[p] + fb))));
            }
            sq[k * L::ROW + at_mine] = qv;
            sf[k * L::ROW + at_mine] = fv;
        }
#pragma unroll
        for (int p = 0; p < VPASSES; ++p)
            if (vk + p * VTOK < HG_GROUP) sv[(vk + p * VTOK) * COLS + tid % COLS] = zv[p];
        __syncthreads();
        if (r0 + HG_GROUP < n) fetch(r0 + HG_GROUP);
#pragma unroll 4
        for (int k = 0; k < rn; ++k) {
            const float v = sv[k * COLS + cw];
            const float* fp = sf + k * L::ROW + l * L::LS;
            const float* qp = sq + k * L::ROW + l * L::LS;
            float f[R], qq[R];
            if (R % 4 == 0) {
#pragma unroll
                for (int r = 0; r < R; r += 4) {
                    *reinterpret_cast<float4*>(f + r) = *reinterpret_cast<const float4*>(fp + r);
                    *reinterpret_cast<float4*>(qq + r) = *reinterpret_cast<const float4*>(qp + r);
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) { f[r] = fp[r]; qq[r] = qp[r]; }
            }
            float o = 0.f, o2 = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                S[r] = fmaf(f[r], S[r] - v, v);               // f S + (1 - f) v
                if (r & 1) o2 = fmaf(S[r], qq[r], o2);
                else o = fmaf(S[r], qq[r], o);
            }
            o += o2;
#pragma unroll
            for (int d = CPW; d < 32; d <<= 1) o += __shfl_xor_sync(0xffffffffu, o, d);
            if (l == 0 && col < vd) o_raw[((size_t)(first + r0 + k) * nh + h) * vd + col] = o;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = l * R + r;
        if (i < dim && col < vd) st[(size_t)i * vd + col] = S[r];
    }
}

// The form for long portions: a warp owns FOUR neighbouring columns, all 32 lanes share each of them (R rows per
// lane, dim <= 32 R).  The gates and queries a lane loads serve its four columns, the four column sums are reduced
// together (the lanes pass on the half they do not keep: six shuffles for four sums), and the tokens of a group are
// unrolled so that the chains of different tokens overlap: few warps with much to do each, where the warp per
// column has many warps that each spend most instructions on loads and shuffles.
#define HW_C 4

template <typename T, int R>
__global__ void __launch_bounds__(128)
hgrn2_wide_kernel(const T* __restrict__ proj, int ld, int q_off, int f_off, int v_off, const float* __restrict__ f_bias,
                  const float* __restrict__ lower, const float* __restrict__ gates, float* __restrict__ state,
                  float* __restrict__ o_raw, const int* __restrict__ positions, const int* __restrict__ q_start,
                  const int* __restrict__ slots, int nh, int dim, int vd) {
    using L = HcLayout<R, 32>;
    constexpr int DIMP = L::DIMP, COLS = 4 * HW_C;           // four warps, four columns each
    constexpr int TOK_PASS = 128 / DIMP, PASSES = HG_GROUP / TOK_PASS;
    constexpr int VTOK = 128 / COLS, VPASSES = HG_GROUP / VTOK;
    __shared__ __align__(16) float sq[HG_GROUP * L::ROW];
    __shared__ __align__(16) float sf[HG_GROUP * L::ROW];
    __shared__ __align__(16) float sv[HG_GROUP * COLS];
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int first = q_start[b], n = q_start[b + 1] - first;
    if (n <= 0 || positions[first] < 0) return;           // padding of a fixed-shape step
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col0 = c0 + warp * HW_C;                    // the warp's first column
    float* st = state + ((size_t)slots[b] * nh + h) * dim * vd;
    float S[R][HW_C];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < HW_C; ++c) {
            const int i = lane * R + r;
            S[r][c] = (i < dim && col0 + c < vd) ? __ldcg(st + (size_t)i * vd + col0 + c) : 0.f;
        }
    const int i_mine = tid % DIMP, k0 = tid / DIMP;
    const bool row_live = i_mine < dim;
    const float fb = row_live ? f_bias[h * dim + i_mine] : 0.f, lo = row_live ? lower[h * dim + i_mine] : 0.f;
    const int at_mine = (i_mine / R) * L::LS + i_mine % R;
    const int vk = tid / COLS, vj = c0 + tid % COLS;
    float zq[PASSES], zf[PASSES], zv[VPASSES];
    auto fetch = [&](int r0) {
        const int rn = min(HG_GROUP, n - r0);
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int k = k0 + p * TOK_PASS;
            zq[p] = zf[p] = 0.f;
            if (k < rn && row_live) {
                if (gates) {
                    const float* grow = gates + (size_t)(first + r0 + k) * 2 * nh * dim + h * dim + i_mine;
                    zq[p] = __ldcg(grow);
                    zf[p] = __ldcg(grow + nh * dim);
                } else {
                    const T* row = proj + (size_t)(first + r0 + k) * ld + h * dim + i_mine;
                    zq[p] = load1_cg(row + q_off);
                    zf[p] = load1_cg(row + f_off);
                }
            }
        }
#pragma unroll
        for (int p = 0; p < VPASSES; ++p) {
            const int k = vk + p * VTOK;
            zv[p] = (k < rn && vj < vd) ? load1_cg(proj + (size_t)(first + r0 + k) * ld + v_off + h * vd + vj) : 0.f;
        }
    };
    fetch(0);
    const bool up16 = lane & 16, up8 = lane & 8;
    const int my_col = col0 + (up16 ? 2 : 0) + (up8 ? 1 : 0);   // the column whose sum this lane ends up with
    for (int r0 = 0; r0 < n; r0 += HG_GROUP) {
        const int rn = min(HG_GROUP, n - r0);
        __syncthreads();
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int k = k0 + p * TOK_PASS;
            float qv = 0.f, fv = 1.f;
            if (row_live && gates) {
                qv = zq[p];
                fv = zf[p];
            } else if (row_live) {
                qv = zq[p] / (1.f + expf(-zq[p]));
                fv = lo + (1.f - lo) * (1.f / (1.f + expf(-(zf[p] + fb))));
            }
            sq[k * L::ROW + at_mine] = qv;
            sf[k * L::ROW + at_mine] = fv;
        }
#pragma unroll
        for (int p = 0; p < VPASSES; ++p) sv[(vk + p * VTOK) * COLS + tid % COLS] = zv[p];
        __syncthreads();
        if (r0 + HG_GROUP < n) fetch(r0 + HG_GROUP);
#pragma unroll 4
        for (int k = 0; k < rn; ++k) {
            const float4 v4 = *reinterpret_cast<const float4*>(sv + k * COLS + warp * HW_C);
            const float v[HW_C] = {v4.x, v4.y, v4.z, v4.w};
            const float* fp = sf + k * L::ROW + lane * L::LS;
            const float* qp = sq + k * L::ROW + lane * L::LS;
            float f[R], qq[R];
            if (R % 4 == 0) {
#pragma unroll
                for (int r = 0; r < R; r += 4) {
                    *reinterpret_cast<float4*>(f + r) = *reinterpret_cast<const float4*>(fp + r);
                    *reinterpret_cast<float4*>(qq + r) = *reinterpret_cast<const float4*>(qp + r);
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) { f[r] = fp[r]; qq[r] = qp[r]; }
            }
            float o[HW_C] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int c = 0; c < HW_C; ++c) {
                    S[r][c] = fmaf(f[r], S[r][c] - v[c], v[c]);       // f S + (1 - f) v
                    o[c] = fmaf(S[r][c], qq[r], o[c]);
                }
            // four sums over 32 lanes: halves pass on the pair they do not keep, then quarters, then within eight lanes
            const float g0 = __shfl_xor_sync(0xffffffffu, up16 ? o[0] : o[2], 16);
            const float g1 = __shfl_xor_sync(0xffffffffu, up16 ? o[1] : o[3], 16);
            const float a = (up16 ? o[2] : o[0]) + g0, bb = (up16 ? o[3] : o[1]) + g1;
            float c1 = (up8 ? bb : a) + __shfl_xor_sync(0xffffffffu, up8 ? a : bb, 8);
            c1 += __shfl_xor_sync(0xffffffffu, c1, 4);
            c1 += __shfl_xor_sync(0xffffffffu, c1, 2);
            c1 += __shfl_xor_sync(0xffffffffu, c1, 1);
            if ((lane & 7) == 0 && my_col < vd) o_raw[((size_t)(first + r0 + k) * nh + h) * vd + my_col] = c1;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < HW_C; ++c) {
            const int i = lane * R + r;
            if (i < dim && col0 + c < vd) st[(size_t)i * vd + col0 + c] = S[r][c];
        }
}

// gates[t] = (silu(q projection) | lower + (1 - lower) sigmoid(gate projection + bias)) for every token and channel
// at once: float [tokens, 2 * channels]; for long portions, where the recurrence's blocks would each repeat it
template <typename T>
__global__ void __launch_bounds__(256)
hgrn2_gates_kernel(const T* __restrict__ proj, int ld, int q_off, int f_off, const float* __restrict__ f_bias,
                   const float* __restrict__ lower, float* __restrict__ gates, const int* __restrict__ positions,
                   int channels) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    if (positions[t] < 0) return;
    const T* row = proj + (size_t)t * ld;
    float* g = gates + (size_t)t * 2 * channels;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        const float zq = load1_cg(row + q_off + c), zf = load1_cg(row + f_off + c) + f_bias[c], lo = lower[c];
        g[c] = zq / (1.f + expf(-zq));
        g[channels + c] = lo + (1.f - lo) * (1.f / (1.f + expf(-zf)));
    }
}

// out[t][h] = o_raw[t][h] / sqrt(mean(o_raw[t][h]^2) + eps) * norm_w, a warp per (token, head)
template <typename T>
__global__ void __launch_bounds__(256)
hgrn2_norm_kernel(const float* __restrict__ o_raw, const float* __restrict__ norm_w, float eps, T* __restrict__ out,
                  const int* __restrict__ positions, int n_tokens, int nh, int vd) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= n_tokens * nh || positions[unit / nh] < 0) return;
    const float* row = o_raw + (size_t)unit * vd;
    float ss = 0.f;
    for (int j = lane; j < vd; j += 32) { const float v = __ldcg(row + j); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)vd + eps);
    for (int j = lane; j < vd; j += 32) out[(size_t)unit * vd + j] = from_f32<T>(__ldcg(row + j) * inv * norm_w[j]);
}

static size_t hgrn2_smem(int dim, int vd) {
    return ((size_t)dim * vd + 2 * HG_GROUP * dim + 2 * HG_GROUP * vd) * sizeof(float);
}

// proj: [tokens, ld] with the query, gate and value projections at column offsets q_off, f_off, v_off
// state: [slots, nh, dim, vd] float; out: [tokens, nh * vd]
// o_raw: float scratch [tokens, nh * vd] for the form with the state in registers (dim <= 128), or null for the
// form with one block per head and the state in shared memory; gates: float scratch [tokens, 2 * nh * dim] or null:
// with it the gates and queries are prepared by a kernel of their own (worth it for long portions)
ST_EXPORT int st_hgrn2_scan(const void* proj, int ld, int q_off, int f_off, int v_off, const float* f_bias,
                            const float* lower, const float* norm_w, float eps, float* state, void* out, float* o_raw,
                            float* gates, const int* positions, const int* q_start, const int* slots, int n_tokens, int n_seqs, int nh,
                            int dim, int vd, int dtype, void* stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (nh <= 0 || dim <= 0 || vd <= 0) return ST_ERR_BAD_ARG;
    if (dtype != 0 && dtype != 1) return ST_ERR_BAD_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
    if (o_raw && dim <= 128) {
        if (gates) {
            const int rc = dtype == 0
                ? st_launch_pdl("hgrn2_gates", hgrn2_gates_kernel<float>, dim3(n_tokens), dim3(256), 0, s, (const float*)proj,
                                ld, q_off, f_off, f_bias, lower, gates, positions, nh * dim)
                : st_launch_pdl("hgrn2_gates", hgrn2_gates_kernel<bf16>, dim3(n_tokens), dim3(256), 0, s, (const bf16*)proj,
                                ld, q_off, f_off, f_bias, lower, gates, positions, nh * dim);
            if (rc) return rc;
        }
#define HC_LAUNCH(T, R, LANES)                                                                                        \
    rc = st_launch_pdl("hgrn2_cols", hgrn2_cols_kernel<T, R, LANES>,                                                  \
                       dim3(n_seqs, nh, (vd + HcLayout<R, LANES>::COLS - 1) / HcLayout<R, LANES>::COLS), dim3(128), 0, s, \
                       (const T*)proj, ld, q_off, f_off, v_off, f_bias, lower, (const float*)gates, state, o_raw,     \
                       positions, q_start, slots, nh, dim, vd)
    // Long portions: the wide form (32 lanes per column, four columns per warp).  Steps of few tokens per request
    // are bound by reading and writing the state: eight lanes per column with many rows each, four columns side by
    // side per warp.
    const bool long_portions = n_tokens > 4 * n_seqs;
#define HW_LAUNCH(T, R)                                                                                               \
    rc = st_launch_pdl("hgrn2_wide", hgrn2_wide_kernel<T, R>, dim3(n_seqs, nh, (vd + 4 * HW_C - 1) / (4 * HW_C)), dim3(128), \
                       0, s, (const T*)proj, ld, q_off, f_off, v_off, f_bias, lower, (const float*)gates, state, o_raw, \
                       positions, q_start, slots, nh, dim, vd)
#define HC_PICK(T)                                                    \
    do {                                                              \
        if (dim <= 8) HC_LAUNCH(T, 1, 8);                             \
        else if (dim <= 16) HC_LAUNCH(T, 2, 8);                       \
        else if (dim <= 32 && long_portions) HW_LAUNCH(T, 1);         \
        else if (dim <= 32) HC_LAUNCH(T, 4, 8);                       \
        else if (dim <= 64 && long_portions) HW_LAUNCH(T, 2);         \
        else if (dim <= 64) HC_LAUNCH(T, 8, 8);                       \
        else if (long_portions) HW_LAUNCH(T, 4);                      \
        else HC_LAUNCH(T, 16, 8);                                     \
    } while (0)
        int rc = 0;
        if (dtype == 0) HC_PICK(float); else HC_PICK(bf16);
#undef HC_PICK
#undef HC_LAUNCH
#undef HW_LAUNCH
        if (rc) return rc;
        const int units = n_tokens * nh;
        if (dtype == 0)
            return st_launch_pdl("hgrn2_norm", hgrn2_norm_kernel<float>, dim3((units + 7) / 8), dim3(256), 0, s,
                                 (const float*)o_raw, norm_w, eps, (float*)out, positions, n_tokens, nh, vd);
        return st_launch_pdl("hgrn2_norm", hgrn2_norm_kernel<bf16>, dim3((units + 7) / 8), dim3(256), 0, s,
                             (const float*)o_raw, norm_w, eps, (bf16*)out, positions, n_tokens, nh, vd);
    }
    const size_t smem = hgrn2_smem(dim, vd);
    if (smem > 200 * 1024) return ST_ERR_TOO_LARGE;
    int threads = (vd + 31) / 32 * 32;
    if (threads < 128) threads = 128;
    if (threads > 1024) threads = 1024;
    dim3 grid(n_seqs, nh);
#define HG_LAUNCH(T)                                                                                                  \
    do {                                                                                                              \
        if (smem > 48 * 1024) {                                                                                       \
            cudaError_t e = cudaFuncSetAttribute(hgrn2_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                                 (int)smem);                                                          \
            if (e != cudaSuccess) return (int)e;                                                                      \
        }                                                                                                             \
        hgrn2_scan_kernel<T><<<grid, threads, smem, s>>>((const T*)proj, ld, q_off, f_off, v_off, f_bias, lower,      \
                                                         norm_w, eps, state, (T*)out, positions, q_start, slots, nh,  \
                                                         dim, vd);                                                    \
    } while (0)
    if (dtype == 0) HG_LAUNCH(float);
    else HG_LAUNCH(bf16);
#undef HG_LAUNCH
    return st_launch_status();
}
