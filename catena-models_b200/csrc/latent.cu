// Latent attention: keys and values of all heads are read out of one small latent row per token, and only that row
// (plus one turned key part that all heads share) is cached.
//
//   per token      c_q = norm(W_dq h) w_q ;  [c' | r] = W_dkv h ;  c = norm(c') w_kv ;  r turned by the position
//   cache entry    [c (KR) | r (R) | zeros up to EC]                         one per token, for all heads
//   per head       q = [q_plain (D) | q_turn (R)] = W_uq c_q ;  q_turn turned by the position
//                  score(i, j) = (q_plain_i . (W_uk c_j) + q_turn_i . r_j) * scale
//                              = ((W_uk^T q_plain_i) . c_j + q_turn_i . r_j) * scale        (the product moved to the query)
//                  o_i = W_uv (sum_j p_ij c_j)                                               (and out of the sum)
//
// so a head's query against the cache is the row [W_uk^T q_plain | q_turn] of E = KR + R channels, every head meets the
// same cache entries, and the weighted sum runs over the latents.  The two per-head products (W_uk^T on the queries,
// W_uv on the sums) are `head_linear`.  Norms, angles, scores, softmax and the sums over them are float.
//
// Every kind of step writes its entries first and then reads all keys from the cache: whole prompts, portions,
// single tokens and mixed batches are one code path.  Rows of padding (tok_seq < 0) are left alone.
#include "common.cuh"
#include "latent.h"
#include <math.h>

// ------------------------------------------------------------------------------ entries and query latent
// One block per row of the step.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const LatentArgs a) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const long long t = blockIdx.x;
    const int b = a.tok_seq[t];
    T* copy = a.ckv && !a.no_entry ? (T*)a.ckv + t * a.EC : nullptr;
    if (b < 0) {
        if (copy)
            for (int c = threadIdx.x; c < a.EC; c += blockDim.x) copy[c] = from_f32<T>(0.f);
        return;
    }
    const T* row = (const T*)a.proj + t * a.ld_proj;
    // the query latent
    {
        const T* x = row + a.q_off;
        float ss = 0.f;
        for (int c = threadIdx.x; c < a.QR; c += blockDim.x) {
            const float v = to_f32(x[c]);
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.f / sqrtf(ss / (float)a.QR + a.eps);
        T* o = (T*)a.cq + t * a.QR;
        for (int c = threadIdx.x; c < a.QR; c += blockDim.x) o[c] = from_f32<T>((to_f32(x[c]) * inv) * a.wq_norm[c]);
    }
    if (a.no_entry) return;
    // the cache entry
    const int pos = a.tok_pos[t];
    const int page = a.ptab[(long long)a.seq_slot[b] * a.ptab_stride + pos / PAGE_TOKENS];
    T* entry = (T*)a.pool + ((long long)page * PAGE_TOKENS + pos % PAGE_TOKENS) * a.EC;
    const T* x = row + a.kv_off;
    float ss = 0.f;
    for (int c = threadIdx.x; c < a.KR; c += blockDim.x) {
        const float v = to_f32(x[c]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)a.KR + a.eps);
    for (int c = threadIdx.x; c < a.KR; c += blockDim.x) entry[c] = from_f32<T>((to_f32(x[c]) * inv) * a.wkv_norm[c]);
    const T* r = x + a.KR;
    for (int i = threadIdx.x; i < (a.R + 1) / 2; i += blockDim.x) {
        if (2 * i + 1 >= a.R) {                       // an odd last channel has no partner
            entry[a.KR + 2 * i] = r[2 * i];
            continue;
        }
        float sn, cs;
        sincosf((float)pos * a.rate[i], &sn, &cs);
        sn *= a.mag;
        cs *= a.mag;
        const float u = to_f32(r[2 * i]), v = to_f32(r[2 * i + 1]);
        entry[a.KR + 2 * i] = from_f32<T>(u * cs - v * sn);
        entry[a.KR + 2 * i + 1] = from_f32<T>(v * cs + u * sn);
    }
    for (int c = a.KR + a.R + threadIdx.x; c < a.EC; c += blockDim.x) entry[c] = from_f32<T>(0.f);
    if (copy) {
        __syncthreads();                               // the entry is complete (every thread reads what others wrote)
        for (int c = threadIdx.x; c < a.EC; c += blockDim.x) copy[c] = entry[c];
    }
}

// The prompt form's operands: per row, queries, keys and values of every head in heads of HD channels, as the attention
// kernels over keys and values take them: q = [q_plain | q_turn turned | 0], k = [W_uk c | the row's turned key part | 0],
// v = [W_uv c | 0].  One block per row; the row's angles are formed once and serve every head.  VEC: eight channels per
// access (every size a multiple of 8, rows and buffers aligned to match).
#define LX_MAX_PAIRS 256
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
latent_expand_kernel(const LatentArgs a) {
    __shared__ float cs_tab[LX_MAX_PAIRS], sn_tab[LX_MAX_PAIRS];
    pdl_trigger();
    pdl_wait();
    const long long t = blockIdx.x;
    const int H = a.H, D = a.D, R = a.R, DV = a.DV, HD = a.HD;
    T* out = (T*)a.qkv + t * a.ld_qkv;
    const bool pad = a.tok_seq[t] < 0;
    const T* q = (const T*)a.q + t * a.ldq;
    const T* kvu = (const T*)a.kvu + t * a.ld_kvu;
    const T* r = (const T*)a.ckv + t * a.EC + a.KR;
    const float pos = pad ? 0.f : (float)a.tok_pos[t];
    for (int i = threadIdx.x; i < R / 2; i += blockDim.x) {
        sincosf(pos * a.rate[i], &sn_tab[i], &cs_tab[i]);
        sn_tab[i] *= a.mag;
        cs_tab[i] *= a.mag;
    }
    __syncthreads();
    const int n = H * HD;
    if (VEC) {
        const int n8 = n >> 3;
        for (int e8 = threadIdx.x; e8 < 3 * n8; e8 += blockDim.x) {
            const int which = e8 / n8, hc = (e8 - which * n8) * 8, h = hc / HD, c = hc - h * HD;
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (!pad) {
                if (which == 0) {
                    if (c < D + R) load8f<T>(q + h * (D + R) + c, v);
                    if (c >= D && c < D + R) {
                        const int i0 = (c - D) >> 1;
#pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            const float cs = cs_tab[i0 + p], sn = sn_tab[i0 + p], u = v[2 * p], w = v[2 * p + 1];
                            v[2 * p] = u * cs - w * sn;
                            v[2 * p + 1] = w * cs + u * sn;
                        }
                    }
                } else if (which == 1) {
                    if (c < D) load8f<T>(kvu + h * D + c, v);
                    else if (c < D + R) load8f<T>(r + (c - D), v);
                } else if (c < DV) load8f<T>(kvu + H * D + h * DV + c, v);
            }
            store8f<T>(out + (long long)e8 * 8, v);
        }
        return;
    }
    for (int e = threadIdx.x; e < 3 * n; e += blockDim.x) {
        const int which = e / n, hc = e - which * n, h = hc / HD, c = hc - h * HD;
        float v = 0.f;
        if (!pad) {
            if (which == 0) {
                if (c < D) v = to_f32(q[h * (D + R) + c]);
                else if (c < D + R) {
                    const int i = (c - D) >> 1;
                    const T* pair = q + h * (D + R) + D + 2 * i;
                    if (2 * i + 1 >= R) v = to_f32(pair[0]);          // an odd last channel has no partner
                    else {
                        const float u = to_f32(pair[0]), w = to_f32(pair[1]);
                        v = ((c - D) & 1) ? w * cs_tab[i] + u * sn_tab[i] : u * cs_tab[i] - w * sn_tab[i];
                    }
                }
            } else if (which == 1) {
                if (c < D) v = to_f32(kvu[h * D + c]);
                else if (c < D + R) v = to_f32(r[c - D]);
            } else if (c < DV) v = to_f32(kvu[H * D + h * DV + c]);
        }
        out[e] = from_f32<T>(v);
    }
}

extern "C" int cm_latent_expand(int dt, const LatentArgs* args, cudaStream_t st) {
    const LatentArgs& a = *args;
    if (a.rows <= 0) return CM_OK;
    if (a.HD < a.D + a.R || a.HD < a.DV || !a.ckv || !a.kvu || !a.qkv || !a.q || a.R / 2 > LX_MAX_PAIRS)
        CM_REFUSE("latent_expand: heads of %d channels for %d + %d and %d", a.HD, a.D, a.R, a.DV);
    const bool vec = ((a.D | a.R | a.DV | a.HD | a.KR | a.EC) % 8 == 0) && ((a.ldq | a.ld_kvu | a.ld_qkv) % 8 == 0) &&
                     (((uintptr_t)a.q | (uintptr_t)a.kvu | (uintptr_t)a.ckv | (uintptr_t)a.qkv) & 15) == 0 && dt == DT_BF16;
    if (dt == DT_F32) cm_launch(latent_expand_kernel<float, false>, (unsigned)a.rows, 256, 0, st, a);
    else if (dt == DT_BF16 && vec) cm_launch(latent_expand_kernel<bf16, true>, (unsigned)a.rows, 256, 0, st, a);
    else if (dt == DT_BF16) cm_launch(latent_expand_kernel<bf16, false>, (unsigned)a.rows, 256, 0, st, a);
    else return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// The turned part of every head's query, moved behind the place of the query against the latent:
// qa[t][h][KR + 2i, 2i + 1] = turn(q[t][h][D + 2i, 2i + 1]).  One thread per pair.
template <typename T>
__global__ void latent_query_turn_kernel(const LatentArgs a) {
    pdl_trigger();
    pdl_wait();
    const int half = (a.R + 1) / 2;
    const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (idx >= a.rows * a.H * half) return;
    const int i = (int)(idx % half);
    const long long th = idx / half;
    const int h = (int)(th % a.H);
    const long long t = th / a.H;
    if (a.tok_seq[t] < 0) return;
    const T* q = (const T*)a.q + t * a.ldq + (long long)h * (a.D + a.R) + a.D;
    float* o = a.qa + t * a.ldqa + (long long)h * a.E + a.KR;
    if (2 * i + 1 >= a.R) {
        o[2 * i] = to_f32(q[2 * i]);
        return;
    }
    float sn, cs;
    sincosf((float)a.tok_pos[t] * a.rate[i], &sn, &cs);
    sn *= a.mag;
    cs *= a.mag;
    const float u = to_f32(q[2 * i]), v = to_f32(q[2 * i + 1]);
    o[2 * i] = u * cs - v * sn;
    o[2 * i + 1] = v * cs + u * sn;
}

extern "C" int cm_latent_prepare(int dt, const LatentArgs* args, cudaStream_t st) {
    const LatentArgs& a = *args;
    if (a.rows <= 0) return CM_OK;
    if (a.EC < a.KR + a.R || a.EC % 8) CM_REFUSE("latent_prepare: entries of %d for %d + %d channels (a multiple of 8)", a.EC, a.KR, a.R);
    if (dt == DT_F32) cm_launch(latent_prepare_kernel<float>, (unsigned)a.rows, 128, 0, st, a);
    else if (dt == DT_BF16) cm_launch(latent_prepare_kernel<bf16>, (unsigned)a.rows, 128, 0, st, a);
    else return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

extern "C" int cm_latent_query_turn(int dt, const LatentArgs* args, cudaStream_t st) {
    const LatentArgs& a = *args;
    const long long n = a.rows * a.H * ((a.R + 1) / 2);
    if (n <= 0) return CM_OK;
    const unsigned grid = (unsigned)((n + 255) / 256);
    if (dt == DT_F32) cm_launch(latent_query_turn_kernel<float>, grid, 256, 0, st, a);
    else if (dt == DT_BF16) cm_launch(latent_query_turn_kernel<bf16>, grid, 256, 0, st, a);
    else return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// ------------------------------------------------------------------------------ a matrix per head
// y[t][h * ys + n] = sum_k x[t][h * xs + k] * w[h][n][k]: every head's channels of a row meet the head's own matrix
// (a block-diagonal product).  Tiles of 64 rows x 64 columns, a thread 4 x 4, float sums in the order of k.
#define HL_TM 64
#define HL_TN 64
#define HL_BK 16
template <typename TX, typename T, typename TY>
__global__ void __launch_bounds__(256)
head_linear_kernel(TY* __restrict__ y, const TX* __restrict__ x, const T* __restrict__ w, long long rows, int N, int K,
                   long long ldx, long long ldy, int xs, int ys) {
    __shared__ float sx[HL_BK][HL_TM + 4];
    __shared__ float sw[HL_BK][HL_TN + 4];
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.z;
    const long long r0 = (long long)blockIdx.y * HL_TM;
    const int n0 = blockIdx.x * HL_TN;
    const TX* xh = x + (long long)h * xs;
    const T* wh = w + (long long)h * N * K;
    const int tid = threadIdx.x, tr = tid / 16, tc = tid % 16;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HL_BK) {
        for (int e = tid; e < HL_TM * HL_BK; e += 256) {
            const int r = e / HL_BK, kk = e % HL_BK;
            sx[kk][r] = (r0 + r < rows && k0 + kk < K) ? to_f32(xh[(r0 + r) * ldx + k0 + kk]) : 0.f;
        }
        for (int e = tid; e < HL_TN * HL_BK; e += 256) {
            const int n = e / HL_BK, kk = e % HL_BK;
            sw[kk][n] = (n0 + n < N && k0 + kk < K) ? to_f32(wh[(long long)(n0 + n) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HL_BK; ++kk) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = sx[kk][tr * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = sw[kk][tc * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long r = r0 + tr * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tc * 4 + j;
            if (n < N) y[r * ldy + (long long)h * ys + n] = from_f32<TY>(acc[i][j]);
        }
    }
}

// The same for a few rows (single-token steps): the tiles above would be nearly empty.  A warp owns one output column of
// one head: its lanes walk the matrix row once and meet up to HL_FEW rows of x with it; sums over lanes by shuffles.
#define HL_FEW 8
template <typename TX, typename T, typename TY>
__global__ void __launch_bounds__(256)
head_linear_few_kernel(TY* __restrict__ y, const TX* __restrict__ x, const T* __restrict__ w, long long rows, int N, int K,
                       long long ldx, long long ldy, int xs, int ys) {
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.y, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= N) return;
    const T* wr = w + ((long long)h * N + n) * K;
    const TX* xh = x + (long long)h * xs;
    for (long long r0 = 0; r0 < rows; r0 += HL_FEW) {
        float acc[HL_FEW];
#pragma unroll
        for (int r = 0; r < HL_FEW; ++r) acc[r] = 0.f;
        for (int k = lane; k < K; k += 32) {
            const float wv = to_f32(wr[k]);
#pragma unroll
            for (int r = 0; r < HL_FEW; ++r)
                if (r0 + r < rows) acc[r] = fmaf(to_f32(xh[(r0 + r) * ldx + k]), wv, acc[r]);
        }
#pragma unroll
        for (int r = 0; r < HL_FEW; ++r) {
            const float v = warp_sum(acc[r]);
            if (lane == 0 && r0 + r < rows) y[(r0 + r) * ldy + (long long)h * ys + n] = from_f32<TY>(v);
        }
    }
}

// x_f32 / y_f32: the rows read / written are float whatever the matrices' dtype (sums that stay unrounded between two steps).
extern "C" int cm_head_linear(int dt, void* y, const void* x, const void* w, long long rows, int H, int N, int K, long long ldx,
                              long long ldy, int xs, int ys, int x_f32, int y_f32, cudaStream_t st) {
    if (rows <= 0 || H <= 0 || N <= 0) return CM_OK;
    if (H > 65535) CM_REFUSE("head_linear: %d heads", H);
    const bool few = rows <= 2 * HL_FEW;
    dim3 grid(few ? (N + 7) / 8 : (N + HL_TN - 1) / HL_TN, few ? H : (unsigned)((rows + HL_TM - 1) / HL_TM), few ? 1 : H);
#define HL_LAUNCH(TX, TW, TY) \
    do {                                                                                                                    \
        if (few) cm_launch(head_linear_few_kernel<TX, TW, TY>, grid, 256, 0, st, (TY*)y, (const TX*)x, (const TW*)w, rows, N, K, ldx, ldy, xs, ys); \
        else cm_launch(head_linear_kernel<TX, TW, TY>, grid, 256, 0, st, (TY*)y, (const TX*)x, (const TW*)w, rows, N, K, ldx, ldy, xs, ys);         \
    } while (0)
    if (dt == DT_F32) HL_LAUNCH(float, float, float);
    else if (dt == DT_BF16 && x_f32 && y_f32) HL_LAUNCH(float, bf16, float);
    else if (dt == DT_BF16 && x_f32) HL_LAUNCH(float, bf16, bf16);
    else if (dt == DT_BF16 && y_f32) HL_LAUNCH(bf16, bf16, float);
    else if (dt == DT_BF16) HL_LAUNCH(bf16, bf16, bf16);
    else return CM_ERR_DTYPE;
#undef HL_LAUNCH
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// ------------------------------------------------------------------------------ attention over the latent cache
// CUDA-core form.  A sequence's rows of the step are (token i, head h) pairs, row = i * H + h; all of them meet the same
// keys, so a block takes LA_ROWS consecutive rows (a few tokens times all or some heads) and walks key tiles of LA_KT cache
// entries from position 0 (or its split's first key) to the position of its last row.  A warp owns four rows: lane j forms the
// scores of key j of the tile, maxima and sums are warp reductions, and in the weighted sum lane l owns the latent's channels
// l, l + 32, ...  Masks are selections on positions.  A tile's entries at or behind the sequence's end are zeros in shared memory
// (what the cache holds there is not the sequence's).
#define LA_ROWS 32
#define LA_KT 32
#define LA_THREADS 256

template <typename T, int KRL>
__global__ void __launch_bounds__(LA_THREADS)
latent_attn_kernel(const LatentArgs a) {
    extern __shared__ __align__(16) float sm[];
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.z, split = blockIdx.y;
    const int s0 = a.seq_start[b], n_tok = a.seq_start[b + 1] - s0;
    const int H = a.H, E = a.E, KR = a.KR;
    const int n_rows = n_tok * H;
    const int r0 = blockIdx.x * LA_ROWS;
    if (r0 >= n_rows) return;
    const int pos0 = a.seq_pos0[b], end = a.seq_end[b];
    const int EQ = (E + 3) & ~3, EK = E | 1;          // pitches: queries read as float4, keys by lanes without conflicts
    float* sq = sm;                                   // [LA_ROWS][EQ]
    float* sk = sq + LA_ROWS * EQ;                    // [LA_KT][EK]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the block's queries, as floats times the scale
    for (int e = threadIdx.x; e < LA_ROWS * EQ; e += LA_THREADS) {
        const int m = e / EQ, c = e - m * EQ, r = r0 + m;
        float v = 0.f;
        if (r < n_rows && c < E) v = a.qa[(long long)(s0 + r / H) * a.ldqa + (long long)(r % H) * E + c] * a.scale;
        sq[e] = v;
    }
    int row_pos[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const int r = r0 + warp * 4 + m;
        row_pos[m] = r < n_rows ? pos0 + r / H : -1;
    }
    const bool warp_live = r0 + warp * 4 < n_rows;    // a warp without rows (fewer heads than the block has rows) only fetches
    const int last_row = min(n_rows, r0 + LA_ROWS) - 1;
    const int k_first = a.splits > 1 ? split * a.chunk : 0;
    const int k_last = min(pos0 + last_row / H, a.splits > 1 ? k_first + a.chunk - 1 : 0x7fffffff);     // inclusive
    float mx[4], sum[4], acc[4][KRL];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        mx[m] = -INFINITY;
        sum[m] = 0.f;
#pragma unroll
        for (int ci = 0; ci < KRL; ++ci) acc[m][ci] = 0.f;
    }
    const int* ptab = a.ptab + (long long)a.seq_slot[b] * a.ptab_stride;
    const bool vec8 = a.EC % 8 == 0 && E % 8 == 0;
    for (int k0 = k_first; k0 <= k_last; k0 += LA_KT) {
        __syncthreads();                              // the tile before is no longer read (and the queries are in place)
        if (vec8) {
            const int E8 = E >> 3;
            for (int e = threadIdx.x; e < LA_KT * E8; e += LA_THREADS) {
                const int j = e / E8, c = (e - j * E8) * 8, kp = k0 + j;
                float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (kp < end) load8f<T>((const T*)a.pool + ((long long)ptab[kp / PAGE_TOKENS] * PAGE_TOKENS + kp % PAGE_TOKENS) * a.EC + c, v);
#pragma unroll
                for (int x = 0; x < 8; ++x) sk[j * EK + c + x] = v[x];
            }
        } else {
            for (int e = threadIdx.x; e < LA_KT * E; e += LA_THREADS) {
                const int j = e / E, c = e - j * E, kp = k0 + j;
                sk[j * EK + c] = kp < end ? to_f32(((const T*)a.pool)[((long long)ptab[kp / PAGE_TOKENS] * PAGE_TOKENS + kp % PAGE_TOKENS) * a.EC + c]) : 0.f;
            }
        }
        __syncthreads();
        if (!warp_live) continue;                     // warp-uniform: the block's barriers stand at the loop's head
        // scores of key k0 + lane against the warp's four rows
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        const float* kr = sk + lane * EK;
        const float* qr = sq + (warp * 4) * EQ;
        for (int c = 0; c < EQ; c += 4) {
            const float k_0 = kr[c], k_1 = c + 1 < E ? kr[c + 1] : 0.f, k_2 = c + 2 < E ? kr[c + 2] : 0.f, k_3 = c + 3 < E ? kr[c + 3] : 0.f;
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const float4 q4 = *reinterpret_cast<const float4*>(qr + m * EQ + c);
                s[m] = fmaf(q4.x, k_0, s[m]);
                s[m] = fmaf(q4.y, k_1, s[m]);
                s[m] = fmaf(q4.z, k_2, s[m]);
                s[m] = fmaf(q4.w, k_3, s[m]);
            }
        }
        const int kp = k0 + lane;
        float p[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const bool seen = kp <= row_pos[m] && kp <= k_last;
            const float sc = seen ? s[m] : -INFINITY;
            const float m_new = fmaxf(mx[m], warp_max(sc));
            const float ref = m_new == -INFINITY ? 0.f : m_new;
            const float f = expf(mx[m] - ref);            // 0 for a row that has seen nothing yet
            p[m] = seen ? expf(sc - ref) : 0.f;
            sum[m] = sum[m] * f + warp_sum(p[m]);
            mx[m] = m_new;
#pragma unroll
            for (int ci = 0; ci < KRL; ++ci) acc[m][ci] *= f;
        }
        // the weighted sum over the tile's latents
        const int n_keys = min(LA_KT, k_last - k0 + 1);
        for (int j = 0; j < n_keys; ++j) {
            float pj[4];
#pragma unroll
            for (int m = 0; m < 4; ++m) pj[m] = __shfl_sync(0xffffffffu, p[m], j);
            const float* vr = sk + j * EK;
#pragma unroll
            for (int ci = 0; ci < KRL; ++ci) {
                const int c = lane + 32 * ci;
                const float v = c < KR ? vr[c] : 0.f;
#pragma unroll
                for (int m = 0; m < 4; ++m) acc[m][ci] = fmaf(pj[m], v, acc[m][ci]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const int r = r0 + warp * 4 + m;
        if (r >= n_rows) continue;
        const long long t = s0 + r / H;
        const int h = r % H;
        if (a.splits > 1) {
            float* part = a.parts + ((t * H + h) * a.splits + split) * (2 + KR);
            if (lane == 0) {
                part[0] = mx[m];
                part[1] = sum[m];
            }
#pragma unroll
            for (int ci = 0; ci < KRL; ++ci) {
                const int c = lane + 32 * ci;
                if (c < KR) part[2 + c] = acc[m][ci];
            }
        } else {
            const float g = a.gate ? sigmoid_f32(to_f32(((const T*)a.gate)[t * a.ld_gate + h])) : 1.f;
            const float f = g / sum[m];
            float* o = a.out + t * a.ldo + (long long)h * KR;
#pragma unroll
            for (int ci = 0; ci < KRL; ++ci) {
                const int c = lane + 32 * ci;
                if (c < KR) o[c] = acc[m][ci] * f;
            }
        }
    }
}

// The splits of a row merged in their order, normalised and gated.  One block per (row, head): the splits' weights
// exp(maximum - the row's maximum) are formed once, then every thread adds up its channels over the splits, with loads
// that do not wait for one another.
#define LA_MAX_SPLITS 1024
#define LA_MERGE_THREADS 128
template <typename T>
__global__ void __launch_bounds__(LA_MERGE_THREADS)
latent_attn_merge_kernel(const LatentArgs a) {
    __shared__ float ws[LA_MAX_SPLITS];
    __shared__ float red[LA_MERGE_THREADS / 32];
    pdl_trigger();
    pdl_wait();
    const long long idx = blockIdx.x;
    const long long t = idx / a.H;
    const int h = (int)(idx - t * a.H), KR = a.KR, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (a.tok_seq[t] < 0) return;
    const long long stride = 2 + KR;
    const float* part = a.parts + idx * a.splits * stride;
    float mx = -INFINITY;
    for (int s = tid; s < a.splits; s += LA_MERGE_THREADS) mx = fmaxf(mx, part[s * stride]);
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < LA_MERGE_THREADS / 32; ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    for (int s = tid; s < a.splits; s += LA_MERGE_THREADS) {
        const float m = part[s * stride];
        ws[s] = m == -INFINITY ? 0.f : expf(m - mx);
    }
    __syncthreads();
    // the sum in the splits' order, by every thread for itself: no exchange, and the same digits in every thread
    float sum = 0.f;
    for (int s = 0; s < a.splits; ++s) sum = fmaf(part[s * stride + 1], ws[s], sum);
    const float g = a.gate ? sigmoid_f32(to_f32(((const T*)a.gate)[t * a.ld_gate + h])) : 1.f;
    const float f = g / sum;
    float* o = a.out + t * a.ldo + (long long)h * KR;
    for (int c = tid; c < KR; c += LA_MERGE_THREADS) {
        float v = 0.f;
#pragma unroll 8
        for (int s = 0; s < a.splits; ++s) v = fmaf(part[s * stride + 2 + c], ws[s], v);
        o[c] = v * f;
    }
}

int cm_latent_attn_merge(int dt, const LatentArgs* args, cudaStream_t st) {
    const LatentArgs& a = *args;
    if (a.splits > LA_MAX_SPLITS) CM_REFUSE("latent_attn: %d splits", a.splits);
    const unsigned mgrid = (unsigned)(a.rows * a.H);
    if (dt == DT_F32) cm_launch(latent_attn_merge_kernel<float>, mgrid, LA_MERGE_THREADS, 0, st, a);
    else if (dt == DT_BF16) cm_launch(latent_attn_merge_kernel<bf16>, mgrid, LA_MERGE_THREADS, 0, st, a);
    else return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

extern "C" int cm_latent_attn(int dt, const LatentArgs* args, cudaStream_t st) {
    const LatentArgs& a = *args;
    if (a.rows <= 0 || a.B <= 0 || a.max_len <= 0) return CM_OK;
    if (a.E != a.KR + a.R || a.KR < 1 || a.KR > 512) CM_REFUSE("latent_attn: latents of %d channels (up to 512)", a.KR);
    if (a.splits < 1 || a.splits > LA_MAX_SPLITS || (a.splits > 1 && (!a.parts || a.chunk < LA_KT || a.chunk % LA_KT)))
        CM_REFUSE("latent_attn: %d splits of %d keys", a.splits, a.chunk);
    const int EQ = (a.E + 3) & ~3, EK = a.E | 1;
    const size_t smem = (size_t)(LA_ROWS * EQ + LA_KT * EK) * sizeof(float);
    if (smem > 200 * 1024) CM_REFUSE("latent_attn: rows of %d channels do not fit shared memory", a.E);
    dim3 grid((unsigned)(((long long)a.max_len * a.H + LA_ROWS - 1) / LA_ROWS), a.splits, a.B);
    const int krl = a.KR <= 128 ? 4 : (a.KR <= 256 ? 8 : 16);
#define LA_LAUNCH(TT, N)                                                                                            \
    do {                                                                                                            \
        if (smem > 48 * 1024)                                                                                       \
            cudaFuncSetAttribute(latent_attn_kernel<TT, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        cm_launch(latent_attn_kernel<TT, N>, grid, LA_THREADS, smem, st, a);                                        \
    } while (0)
    if (dt == DT_F32) {
        if (krl == 4) LA_LAUNCH(float, 4); else if (krl == 8) LA_LAUNCH(float, 8); else LA_LAUNCH(float, 16);
    } else if (dt == DT_BF16) {
        if (krl == 4) LA_LAUNCH(bf16, 4); else if (krl == 8) LA_LAUNCH(bf16, 8); else LA_LAUNCH(bf16, 16);
    } else
        return CM_ERR_DTYPE;
#undef LA_LAUNCH
    CM_CHECK_LAUNCH();
    if (a.splits > 1) return cm_latent_attn_merge(dt, args, st);
    return CM_OK;
}
