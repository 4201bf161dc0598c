// Routed feed-forward (mixture of experts) without a look from the host: a router kernel scores the
// experts of every token and picks the best `top`; the (token, choice) pairs are put into the order of
// their experts by counting (a list of row tiles, each of one expert, comes with it); two grouped
// products then run the experts over their own rows only.  Everything a launch needs to know about the
// routing it reads from device memory, so a step of given shape launches the same kernels with the same
// arguments whatever the router decides, and can be recorded into a graph.
//
//   scores      s = gate(W_r h) in float (gate: sigmoid or softmax over the experts);
//               the `top` largest, lowest index first among equals; weights = the chosen scores,
//               optionally divided by their sum
//   experts     a = act(W_gate x) * (W_up x), y = W_down a, with x = weight * h (the weight on the
//               expert's INPUT) or x = h and y = weight * y (the weight on its output)
//   result      one row of y per pair, float, in the order of the experts; dest[token * top + choice] says
//               where a pair's row is, and the consumer adds a token's rows in the order of its choices.
//
// A pair's result does not depend on which tile it lands in (every output is one dot product in a fixed
// order), so the order of the pairs inside an expert, which comes from atomic counters, changes nothing.
#include "common.cuh"
#include <math.h>

#define MOE_TM 32
#define MOE_TN 64
#define MOE_BK 16
#define MOE_THREADS 256
#define MOE_MAX_GROUPS 64          // groups of experts a router can have

// ------------------------------------------------------------------------------ routing
// How a token's experts are chosen from its E router logits, and what their weights are.
struct RouteRule {
    int softmax_gate;          // scores: softmax over the experts (1) or a sigmoid of each logit (0)
    int renormalize;           // weights divided by (their sum + renorm_eps)
    float renorm_eps;
    float scale;               // factor on the weights
    const float* correction;   // null, or [E]: added to the scores for the choice only; the weights are the scores themselves
    int groups, keep;          // groups > 0: the experts form `groups` equal groups of neighbours, a group's score is the sum of
    int group_best;            // its `group_best` largest choice scores (1: its largest), and only experts of the best `keep`
                               // groups can be chosen
    int real;                  // experts real .. E-1 are identity experts: they get a weight but no rows (their output is the input)
};

// One thread's walk for one token.  sc [E]: logits in, scores out (overwritten).  ch: [E] scratch for the choice scores when
// the rule has a correction or groups, else the same array as sc.  Writes ids and wts [top]; counts every chosen real expert.
__device__ void choose_experts(float* sc, float* ch, int E, int top, const RouteRule& r, int* ids, float* wts, int* counts) {
    if (r.softmax_gate) {
        float mx = -INFINITY, den = 0.f;
        for (int e = 0; e < E; ++e) mx = fmaxf(mx, sc[e]);
        for (int e = 0; e < E; ++e) den += expf(sc[e] - mx);
        for (int e = 0; e < E; ++e) sc[e] = expf(sc[e] - mx) / den;
    } else {
        for (int e = 0; e < E; ++e) sc[e] = sigmoid_f32(sc[e]);
    }
    if (ch != sc)
        for (int e = 0; e < E; ++e) ch[e] = sc[e] + (r.correction ? r.correction[e] : 0.f);
    if (r.groups > 0) {
        // the `keep` best groups stay open: a group is closed if `keep` others have a larger best choice score (or an
        // equal one and a lower index); a closed group's choice scores count as minus infinity
        const int n = E / r.groups;
        float best[MOE_MAX_GROUPS];
        const int nb = min(max(r.group_best, 1), n);
        for (int g = 0; g < r.groups; ++g) {
            if (nb == 1) {
                best[g] = -INFINITY;
                for (int e = g * n; e < (g + 1) * n; ++e) best[g] = fmaxf(best[g], ch[e]);
                continue;
            }
            // the sum of the nb largest: each pass takes the largest not yet taken (the lower index among equals)
            unsigned long long taken = 0ull;                    // n <= 64 experts a group
            float sum = 0.f;
            for (int j = 0; j < nb; ++j) {
                int at = -1;
                float bv = -INFINITY;
                for (int e = 0; e < n; ++e)
                    if (!((taken >> e) & 1ull) && (at < 0 || ch[g * n + e] > bv)) {
                        bv = ch[g * n + e];
                        at = e;
                    }
                taken |= 1ull << at;
                sum += bv;
            }
            best[g] = sum;
        }
        for (int g = 0; g < r.groups; ++g) {
            int ahead = 0;
            for (int o = 0; o < r.groups; ++o)
                if (o != g && (best[o] > best[g] || (best[o] == best[g] && o < g))) ++ahead;
            if (ahead >= r.keep)
                for (int e = g * n; e < (g + 1) * n; ++e) ch[e] = -INFINITY;
        }
    }
    float total = 0.f;
    for (int j = 0; j < top; ++j) {
        int best = 0;
        float bv = -INFINITY;
        for (int e = 0; e < E; ++e)
            if (ch[e] > bv) {
                bv = ch[e];
                best = e;
            }
        ids[j] = best;
        wts[j] = sc[best];
        total += sc[best];
        ch[best] = -INFINITY;
        if (best < r.real) atomicAdd(counts + best, 1);
    }
    if (r.renormalize)
        for (int j = 0; j < top; ++j) wts[j] /= total + r.renorm_eps;
    if (r.scale != 1.f)
        for (int j = 0; j < top; ++j) wts[j] *= r.scale;
}

// One block per token.  ids[p] = expert of pair p (-1 for rows of padding), wts[p] its weight.
template <typename T>
__global__ void __launch_bounds__(128)
moe_router_kernel(int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ counts,
                  const T* __restrict__ h, const T* __restrict__ wr, const int* __restrict__ tok_seq, int W, int E,
                  int top, RouteRule rule) {
    extern __shared__ float score[];              // [E], and [E] choice scores when the rule needs them
    pdl_trigger();
    pdl_wait();
    const long long t = blockIdx.x;
    if (tok_seq && tok_seq[t] < 0) {
        for (int j = threadIdx.x; j < top; j += blockDim.x) ids[t * top + j] = -1;
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* hr = h + t * W;
    for (int e = warp; e < E; e += 4) {
        const T* w = wr + (long long)e * W;
        float acc = 0.f;
        for (int c = lane; c < W; c += 32) acc = fmaf(to_f32(w[c]), to_f32(hr[c]), acc);
        acc = warp_sum(acc);
        if (lane == 0) score[e] = acc;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    const bool two = rule.correction || rule.groups > 0;
    choose_experts(score, two ? score + E : score, E, top, rule, ids + t * top, wts + t * top, counts);
}

// One block, one thread's walk over the experts: where each expert's rows begin (a multiple of tile_rows: an
// expert's rows fill whole row tiles, the last one partly), and the list of row tiles.  plan: [0] number of
// tiles, then per tile (expert, first row, rows); tile_group[t]: the expert of row tile t (0 for tiles that no
// expert uses).  cursor[e] = the first row of expert e.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int* __restrict__ cursor, int* __restrict__ plan,
                                int* __restrict__ tile_group, int E, int tile_rows, int max_tiles) {
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x != 0) return;
    int n = 0;
    for (int e = 0; e < E; ++e) {
        const int c = counts[e];
        cursor[e] = n * tile_rows;
        for (int r = 0; r < c; r += tile_rows) {
            plan[1 + 3 * n] = e;
            plan[2 + 3 * n] = n * tile_rows;
            plan[3 + 3 * n] = min(tile_rows, c - r);
            tile_group[n] = e;
            ++n;
        }
    }
    plan[0] = n;
    for (; n < max_tiles; ++n) tile_group[n] = 0;
}

// perm[sorted row] = pair, dest[pair] = sorted row (-1 for pairs of padding rows).
__global__ void moe_scatter_kernel(int* __restrict__ perm, int* __restrict__ dest, int* __restrict__ cursor,
                                   const int* __restrict__ ids, long long P, int real) {
    pdl_trigger();
    pdl_wait();
    const long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (p >= P) return;
    const int e = ids[p];
    int pos = -1;
    if (e >= 0 && e < real) {
        pos = atomicAdd(cursor + e, 1);
        perm[pos] = (int)p;
    }
    dest[p] = pos;
}

// xs[dest[p]] = T(h[p / top] * (apply_weight ? wts[p] : 1)): the experts' inputs in the order of the experts.
template <typename T>
__global__ void moe_gather_kernel(T* __restrict__ xs, const T* __restrict__ h, const int* __restrict__ dest,
                                  const float* __restrict__ wts, int top, int K, int apply_weight) {
    pdl_trigger();
    pdl_wait();
    const long long p = blockIdx.x;
    const int d = dest[p];
    if (d < 0) return;
    const float w = apply_weight ? wts[p] : 1.f;
    const T* src = h + (p / top) * K;
    T* dst = xs + (long long)d * K;
    for (int c = threadIdx.x; c < K; c += blockDim.x) dst[c] = from_f32<T>(to_f32(src[c]) * w);
}

extern "C" int cm_moe_gather(int dt, void* xs, const void* h, const int* dest, const float* wts, long long pairs,
                             int top, int K, int apply_weight, cudaStream_t st) {
    if (pairs <= 0) return CM_OK;
    if (dt == DT_F32)
        cm_launch(moe_gather_kernel<float>, (unsigned)pairs, 128, 0, st, (float*)xs, (const float*)h, dest, wts, top, K, apply_weight);
    else if (dt == DT_BF16)
        cm_launch(moe_gather_kernel<bf16>, (unsigned)pairs, 128, 0, st, (bf16*)xs, (const bf16*)h, dest, wts, top, K, apply_weight);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// Everything above in one block, for the few rows of a decode step: scores, the best `top`, counts, the list of
// row tiles, the order of the pairs, and (with xs) the experts' inputs in that order.  One launch instead of five.
#define MOE_SMALL_ROWS 64
#define MOE_SMALL_SCORES 8192
template <typename T>
__global__ void __launch_bounds__(256)
moe_route_small_kernel(int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ perm, int* __restrict__ dest,
                       int* __restrict__ counts_out, int* __restrict__ plan, int* __restrict__ tile_group,
                       const T* __restrict__ h, const T* __restrict__ wr, const int* __restrict__ tok_seq, int rows, int W,
                       int E, int top, RouteRule rule, int tile_rows, int max_tiles,
                       T* __restrict__ xs, int apply_weight) {
    extern __shared__ float score[];              // [rows][E] (twice when the rule needs choice scores), then E counts and E cursors
    const bool two = rule.correction || rule.groups > 0;
    int* counts = reinterpret_cast<int*>(score + (two ? 2 : 1) * rows * E);
    const int real = rule.real;
    int* cursor = counts + E;
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    for (int pe = warp; pe < rows * E; pe += 8) {
        const int t = pe / E, e = pe - t * E;
        const T* w = wr + (long long)e * W;
        const T* hr = h + (long long)t * W;
        float acc = 0.f;
        for (int c = lane; c < W; c += 32) acc = fmaf(to_f32(w[c]), to_f32(hr[c]), acc);
        acc = warp_sum(acc);
        if (lane == 0) score[pe] = acc;
    }
    __syncthreads();
    for (int t = threadIdx.x; t < rows; t += blockDim.x) {
        if (tok_seq && tok_seq[t] < 0) {
            for (int j = 0; j < top; ++j) ids[t * top + j] = -1;
            continue;
        }
        float* sc = score + t * E;
        choose_experts(sc, two ? sc + rows * E : sc, E, top, rule, ids + t * top, wts + t * top, counts);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int n = 0;
        for (int e = 0; e < real; ++e) {              // identity experts get no rows
            const int c = counts[e];
            counts_out[e] = c;
            cursor[e] = n * tile_rows;
            for (int r = 0; r < c; r += tile_rows) {
                plan[1 + 3 * n] = e;
                plan[2 + 3 * n] = n * tile_rows;
                plan[3 + 3 * n] = min(tile_rows, c - r);
                tile_group[n] = e;
                ++n;
            }
        }
        plan[0] = n;
        for (; n < max_tiles; ++n) tile_group[n] = 0;
    }
    __syncthreads();
    const int P = rows * top;
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        int pos = -1;
        if (e >= 0 && e < real) {
            pos = atomicAdd(cursor + e, 1);
            perm[pos] = p;
        }
        dest[p] = pos;
    }
    if (!xs) return;
    __syncthreads();                              // dest and wts of this block's own writes
    for (int p = warp; p < P; p += 8) {
        const int d = dest[p];
        if (d < 0) continue;
        const float w = apply_weight ? wts[p] : 1.f;
        const T* src = h + (long long)(p / top) * W;
        T* dst = xs + (long long)d * W;
        for (int c = lane; c < W; c += 32) dst[c] = from_f32<T>(to_f32(src[c]) * w);
    }
}

// Row tiles that `pairs` rows of `E` experts can need at most, each expert's rows starting a tile of its own.
static int max_tiles_for(long long pairs, int E, int tile_rows) {
    const long long full = (pairs + tile_rows - 1) / tile_rows;
    return (int)(full + (pairs < E ? pairs : E));
}

// work: int32 scratch of E' (counts) + E' (cursor) + 1 + 3 * max_tiles (plan) + max_tiles (tile_group) entries, E' = E - identity;
// perm: max_tiles * tile_rows entries (sorted rows), dest: P entries.  tile_rows: 32 for the CUDA-core grouped
// products of this file, 128 for the tensor-core grouped product.
// xs (or null): the experts' inputs [max_tiles * tile_rows][W] in the order of the experts, h times the pair's weight
// when apply_weight (cm_moe_gather as part of this call).
// E counts every router output; the last `identity` of them are identity experts (no matrices, no rows: their pairs get
// dest -1 and a weight, see cm_moe_identity).  correction (or null), groups, keep, scale, renorm_eps: see RouteRule.
extern "C" int cm_moe_route(int dt, int* ids, float* wts, int* perm, int* dest, int* work, const void* h, const void* wr,
                            const int* tok_seq, long long rows, int W, int E, int top, int softmax_gate,
                            int renormalize, int tile_rows, void* xs, int apply_weight, const float* correction, int groups,
                            int keep, int identity, float scale, float renorm_eps, int group_best, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    if (groups > 0 && (group_best < 1 || E / groups > 64 && group_best > 1))
        CM_REFUSE("moe_route: the sum of the %d best of a group of %d experts", group_best, E / groups);
    if (top < 1 || top > E) CM_REFUSE("moe_route: %d of %d experts", top, E);
    if (identity < 0 || identity >= E) CM_REFUSE("moe_route: %d identity experts of %d", identity, E);
    if (groups < 0 || groups > MOE_MAX_GROUPS || (groups > 0 && (E % groups || keep < 1 || keep > groups || keep * (E / groups) < top)))
        CM_REFUSE("moe_route: %d groups of which %d stay open, for %d of %d experts", groups, keep, top, E);
    const bool two = correction || groups > 0;
    if ((size_t)E * sizeof(float) * (two ? 2 : 1) > 48 * 1024) CM_REFUSE("moe_route: %d experts", E);
    if (tile_rows != MOE_TM && tile_rows != 128) CM_REFUSE("moe_route: row tiles of %d (32 or 128)", tile_rows);
    RouteRule rule;
    rule.softmax_gate = softmax_gate;
    rule.renormalize = renormalize;
    rule.renorm_eps = renorm_eps;
    rule.scale = scale;
    rule.correction = correction;
    rule.groups = groups;
    rule.keep = keep;
    rule.group_best = group_best;
    rule.real = E - identity;
    // the scratch is laid out for the experts that get rows (the Python side sizes it by their number)
    const int ER = rule.real;
    const int max_tiles = max_tiles_for(rows * top, ER, tile_rows);
    int *counts = work, *cursor = work + ER, *plan = work + 2 * ER, *tile_group = plan + 1 + 3 * max_tiles;
    if (rows <= MOE_SMALL_ROWS && rows * E * (two ? 2 : 1) <= MOE_SMALL_SCORES && (dt == DT_F32 || dt == DT_BF16)) {
        const size_t small = ((size_t)rows * E * (two ? 2 : 1)) * sizeof(float) + 2 * (size_t)E * sizeof(int);
        if (dt == DT_F32)
            cm_launch(moe_route_small_kernel<float>, 1, 256, small, st, ids, wts, perm, dest, counts, plan, tile_group,
                      (const float*)h, (const float*)wr, tok_seq, (int)rows, W, E, top, rule, tile_rows,
                      max_tiles, (float*)xs, apply_weight);
        else
            cm_launch(moe_route_small_kernel<bf16>, 1, 256, small, st, ids, wts, perm, dest, counts, plan, tile_group,
                      (const bf16*)h, (const bf16*)wr, tok_seq, (int)rows, W, E, top, rule, tile_rows,
                      max_tiles, (bf16*)xs, apply_weight);
        CM_CHECK_LAUNCH();
        return CM_OK;
    }
    if (cudaMemsetAsync(counts, 0, (size_t)ER * sizeof(int), st) != cudaSuccess) {
        cm_set_error("moe_route: memset failed");
        return CM_ERR_LAUNCH;
    }
    const size_t smem = (size_t)E * sizeof(float) * (two ? 2 : 1);
    if (dt == DT_F32)
        cm_launch(moe_router_kernel<float>, (unsigned)rows, 128, smem, st, ids, wts, counts, (const float*)h, (const float*)wr,
                  tok_seq, W, E, top, rule);
    else if (dt == DT_BF16)
        cm_launch(moe_router_kernel<bf16>, (unsigned)rows, 128, smem, st, ids, wts, counts, (const bf16*)h, (const bf16*)wr,
                  tok_seq, W, E, top, rule);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    cm_launch(moe_plan_kernel, 1, 32, 0, st, counts, cursor, plan, tile_group, ER, tile_rows, max_tiles);
    CM_CHECK_LAUNCH();
    const long long P = rows * top;
    cm_launch(moe_scatter_kernel, (unsigned)((P + 255) / 256), 256, 0, st, perm, dest, cursor, ids, P, rule.real);
    CM_CHECK_LAUNCH();
    if (xs) return cm_moe_gather(dt, xs, h, dest, wts, P, top, W, apply_weight, st);
    return CM_OK;
}

// y[t] = (the sum of the weights of token t's pairs whose expert is an identity expert, id >= real) * h[t], float.
template <typename T>
__global__ void moe_identity_kernel(float* __restrict__ y, const T* __restrict__ h, const int* __restrict__ ids,
                                    const float* __restrict__ wts, int top, int real, int K) {
    pdl_trigger();
    pdl_wait();
    const long long t = blockIdx.x;
    float w = 0.f;
    for (int j = 0; j < top; ++j)
        if (ids[t * top + j] >= real) w += wts[t * top + j];
    for (int c = threadIdx.x; c < K; c += blockDim.x) y[t * K + c] = w * to_f32(h[t * K + c]);
}

extern "C" int cm_moe_identity(int dt, float* y, const void* h, const int* ids, const float* wts, long long rows, int top,
                               int real, int K, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    if (dt == DT_F32)
        cm_launch(moe_identity_kernel<float>, (unsigned)rows, 128, 0, st, y, (const float*)h, ids, wts, top, real, K);
    else if (dt == DT_BF16)
        cm_launch(moe_identity_kernel<bf16>, (unsigned)rows, 128, 0, st, y, (const bf16*)h, ids, wts, top, real, K);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

extern "C" int cm_moe_max_tiles(long long pairs, int E, int tile_rows) { return max_tiles_for(pairs, E, tile_rows); }

// ------------------------------------------------------------------------------ grouped products
// UP:   a[row] = act(Wg_e x) * (Wu_e x) for the sorted rows of a tile; x = h[token of the pair] (times the
//       pair's weight when scale_input); w: [E][2 F][K] (gate rows, then up rows); out a: [P][F], sorted order.
// DOWN: y[row] = Wd_e a[row] (times the pair's weight when scale_output); w: [E][N][K]; out y: [rows][N] float,
//       sorted order as well (dest[pair] says where a pair's row is).
// A block computes MOE_TM rows x MOE_TN columns; a thread 4 rows x 2 columns (and both halves for UP).
template <typename T, bool UP>
__global__ void __launch_bounds__(MOE_THREADS)
moe_grouped_kernel(void* __restrict__ out, const T* __restrict__ x, const T* __restrict__ w,
                   const int* __restrict__ plan, const int* __restrict__ perm, const float* __restrict__ wts,
                   int top, int N, int K, int apply_weight, int act, float limit) {
    __shared__ float xs[MOE_BK][MOE_TM + 1];
    __shared__ float ws[UP ? 2 : 1][MOE_BK][MOE_TN + 1];
    __shared__ int src_row[MOE_TM];
    __shared__ float row_w[MOE_TM];
    pdl_trigger();
    pdl_wait();
    const int tile = blockIdx.x;
    if (tile >= plan[0]) return;
    const int e = plan[1 + 3 * tile], row0 = plan[2 + 3 * tile], n_rows = plan[3 + 3 * tile];
    const int n0 = blockIdx.y * MOE_TN;
    const int tid = threadIdx.x;
    if (tid < MOE_TM) {
        const int p = tid < n_rows ? perm[row0 + tid] : -1;
        src_row[tid] = p < 0 ? -1 : (UP ? p / top : row0 + tid);
        row_w[tid] = p < 0 ? 0.f : wts[p];
    }
    __syncthreads();
    const int tr = tid / 32, tc = tid % 32;          // rows tr * 4 .. + 3, columns tc * 2, tc * 2 + 1
    float acc[UP ? 2 : 1][4][2];
#pragma unroll
    for (int h = 0; h < (UP ? 2 : 1); ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[h][i][0] = acc[h][i][1] = 0.f;
    const T* we = w + (long long)e * (UP ? 2 : 1) * N * K;
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
        for (int i = tid; i < MOE_TM * MOE_BK; i += MOE_THREADS) {
            const int r = i / MOE_BK, kk = i % MOE_BK;
            float v = 0.f;
            if (src_row[r] >= 0 && k0 + kk < K) {
                v = to_f32(x[(long long)src_row[r] * K + k0 + kk]);
                if (UP && apply_weight) v = rounded<T>(v * row_w[r]);       // the expert's input as it would be stored
            }
            xs[kk][r] = v;
        }
        for (int i = tid; i < MOE_TN * MOE_BK; i += MOE_THREADS) {
            const int c = i / MOE_BK, kk = i % MOE_BK;
            const bool in = n0 + c < N && k0 + kk < K;
            ws[0][kk][c] = in ? to_f32(we[(long long)(n0 + c) * K + k0 + kk]) : 0.f;
            if (UP) ws[1][kk][c] = in ? to_f32(we[(long long)(N + n0 + c) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_BK; ++kk) {
            float xv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = xs[kk][tr * 4 + i];
#pragma unroll
            for (int h = 0; h < (UP ? 2 : 1); ++h) {
                const float w0 = ws[h][kk][tc * 2], w1 = ws[h][kk][tc * 2 + 1];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[h][i][0] = fmaf(xv[i], w0, acc[h][i][0]);
                    acc[h][i][1] = fmaf(xv[i], w1, acc[h][i][1]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = tr * 4 + i;
        if (r >= n_rows) continue;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int n = n0 + tc * 2 + c;
            if (n >= N) continue;
            if (UP) {
                const float g = acc[0][i][c], u = acc[1][i][c];
                reinterpret_cast<T*>(out)[(long long)(row0 + r) * N + n] = from_f32<T>(gated_act(g, u, act, limit));
            } else {
                float y = acc[0][i][c];
                if (apply_weight) y *= row_w[r];
                reinterpret_cast<float*>(out)[(long long)(row0 + r) * N + n] = y;
            }
        }
    }
}

template <typename T>
static int launch_grouped(bool up, void* out, const void* x, const void* w, const int* work, const int* perm,
                          const float* wts, int E, int top, int max_tiles, int N, int K, int apply_weight, int act, float limit,
                          cudaStream_t st) {
    const int* plan = work + 2 * E;
    dim3 grid(max_tiles, (N + MOE_TN - 1) / MOE_TN);
    if (up)
        cm_launch(moe_grouped_kernel<T, true>, grid, MOE_THREADS, 0, st, out, (const T*)x, (const T*)w, plan, perm, wts, top, N,
                  K, apply_weight, act, limit);
    else
        cm_launch(moe_grouped_kernel<T, false>, grid, MOE_THREADS, 0, st, out, (const T*)x, (const T*)w, plan, perm, wts, top, N,
                  K, apply_weight, act, limit);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// up != 0: the gated first product (N = the experts' inner width, K = the model's width);
// up == 0: the second product (N = the model's width, K = the inner width), rows of float by pair.
extern "C" int cm_moe_grouped(int dt, int up, void* out, const void* x, const void* w, const int* work,
                              const int* perm, const float* wts, int E, int top, int max_tiles, int N, int K,
                              int apply_weight, int act, float limit, cudaStream_t st) {
    if (max_tiles <= 0) return CM_OK;
    if (dt == DT_F32) return launch_grouped<float>(up != 0, out, x, w, work, perm, wts, E, top, max_tiles, N, K, apply_weight, act, limit, st);
    if (dt == DT_BF16) return launch_grouped<bf16>(up != 0, out, x, w, work, perm, wts, E, top, max_tiles, N, K, apply_weight, act, limit, st);
    return CM_ERR_DTYPE;
}
