// Difference-of-two-maps attention over a paged cache, with the short causal taps and the partial
// rotation that come between its projections and its scores.
//
//   taps      y_t[c] = sum_j w[c][j] * u_(t - K + 1 + j)[c],  u = projection + bias, zeros before position 0;
//             the last K values of u of every sequence are its state (float, a ring), so a step may begin anywhere
//   rotation  of the leading `rot` channels of every vector of `sub` channels of q and k: channel i against
//             channel i + rot/2, angle = float(position) * rate[i], sine and cosine times `mag`
//   cache     a key/value head g holds, per position, a key row [map 1 | map 2] of 2 D channels and a value
//             row of DV channels, each in an entry of HDC channels of this layer's pages
//   scores    two maps per query head over the same values: s_m = (q_m . k_m) * scale, m = 1, 2; a key at
//             position j is visible to a query at position i when j <= i and (i - j < window or j < keep;
//             window <= 0: every j <= i); softmax per map in float
//   output    o = a_1 - lambda * a_2;  o <- o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate)
//
// Keys and values of the step are written to the cache before the scores are formed, and every key is
// read from there, whatever the kind of step: whole prompts, portions and single tokens run the same
// code.  (The cache keeps every position: a window with kept first tokens is not a ring.)
// Rows whose tok_seq is negative are padding: they touch nothing.
#include "common.cuh"
#include "diffattn.h"
#include <math.h>

struct TapRotArgs {
    const void* proj;            // [T][ldp] activations: q | k | v channels from column 0 on
    long long ldp;
    const float* bias;           // [C] or null
    const float* taps;           // [C][K]
    float* state;                // [slots][state_stride]: a ring of K rows of C channels; position s lies in row s % K
    long long state_stride;
    void* q_out;                 // [T][ldq] activations: the queries after taps and rotation
    long long ldq;
    void* pool;                  // this layer's pages [2][pages][G][PAGE_TOKENS][HDC], or null when KC = VC = 0
    long long pages;
    const int* ptab;
    long long ptab_stride;
    const float* rate;           // [rot / 2], or null for no rotation
    float mag;
    const int *tok_seq, *tok_pos, *seq_start, *seq_pos0, *seq_slot;
    int T, B, QC, KC, VC, K, sub, rot, G, KW, DV, HDC;
    int one_token_each;          // every sequence brings one token on top of held ones: the state moves on in the same launch
    // further forms, all off at 0
    int interleaved;             // the rotation pairs channel 2i with 2i + 1 (rate[i]) instead of i with i + rot/2
    int value_from_key;          // no value channels (VC = 0): a position's value row is its key row before the rotation
    int ring;                    // > 0: the pages are a ring of this many entries; position p lies in entry p % ring, and of a
                                 // step only the last `ring` positions of a sequence are written
    int no_store;                // the cache is left as it is (the caller writes the step's rows later)
    int rows_out;                // q_out rows hold [q | turned k | v] (ldq >= QC + KC + value channels), not the queries alone
    int from_zero;               // every sequence of the step starts at position 0: nothing reads the filter's state, so the
                                 // pairs form writes it in the same launch
};

#define TR_THREADS 128
#define TR_MAXK CM_MAX_CONV_TAPS

template <typename T>
__device__ __forceinline__ float tap_input(const TapRotArgs& a, int c, int t, int pos, int p0, int s, const float* st) {
    // what the filter of channel c reads at position s <= pos of the token in row t
    if (s >= p0) return to_f32(((const T*)a.proj)[(long long)(t - (pos - s)) * a.ldp + c]) + (a.bias ? a.bias[c] : 0.f);
    if (s >= 0) return st[(long long)(s % a.K) * (a.QC + a.KC + a.VC) + c];
    return 0.f;
}

template <typename T>
__device__ __forceinline__ float tap_sum(const TapRotArgs& a, int c, int t, int pos, int p0, const float* st) {
    const int K = a.K;
    const float* w = a.taps + (long long)c * K;
    float y = 0.f;
    if (pos - (K - 1) >= p0) {                     // every tap reads a row of this step: the usual case, kept short
        const float bias = a.bias ? a.bias[c] : 0.f;
        const T* u = (const T*)a.proj + (long long)(t - (K - 1)) * a.ldp + c;
#pragma unroll 4
        for (int j = 0; j < K; ++j) y = fmaf(w[j], to_f32(u[(long long)j * a.ldp]) + bias, y);
        return y;
    }
    for (int j = 0; j < K; ++j) y = fmaf(w[j], tap_input<T>(a, c, t, pos, p0, pos - K + 1 + j, st), y);
    return y;
}

// One thread per channel and TOK tokens (grid x walks the tokens TOK at a time).  The state of a sequence is a ring
// of K rows: the projected row of position s lies in row s % K.  A single token reads positions pos - K + 1 ..
// pos - 1 and then writes row pos % K, which held position pos - K: nobody reads what it writes, so the state moves
// on in the same launch.  TOK > 1 (long steps): a thread forms its tokens' results side by side before it stores
// any, so that their loads are in flight together; a block per token was bound by the waves of short blocks.
template <typename T, int TOK>
__global__ void __launch_bounds__(TR_THREADS)
tap_rotate_store_kernel(const TapRotArgs a) {
    pdl_trigger();
    pdl_wait();
    const int C = a.QC + a.KC + a.VC;
    const int c = blockIdx.y * TR_THREADS + threadIdx.x;
    if (c >= C) return;
    const int half = a.rot >> 1;
    const int cr = c < a.QC ? c : c - a.QC;           // channel within q, or within k | v
    const int e = cr % max(a.sub, 1);
    const bool turned = c < a.QC + a.KC && a.rate && e < a.rot, low = a.interleaved ? !(e & 1) : e < half;
    const int partner = a.interleaved ? (low ? c + 1 : c - 1) : (low ? c + half : c - half);
    const int pair = a.interleaved ? e >> 1 : (low ? e : e - half);
    float y[TOK], other[TOK];
    int bs[TOK];
#pragma unroll
    for (int i = 0; i < TOK; ++i) {
        const int t = blockIdx.x * TOK + i;
        bs[i] = t < a.T ? a.tok_seq[t] : -1;
        y[i] = other[i] = 0.f;
        if (bs[i] < 0) continue;
        const int pos = a.tok_pos[t], p0 = a.seq_pos0[bs[i]];
        const float* st = a.state + (long long)a.seq_slot[bs[i]] * a.state_stride;
        y[i] = tap_sum<T>(a, c, t, pos, p0, st);
        if (turned) other[i] = tap_sum<T>(a, partner, t, pos, p0, st);
    }
#pragma unroll
    for (int i = 0; i < TOK; ++i) {
        const int t = blockIdx.x * TOK + i, b = bs[i];
        if (b < 0) continue;
        const int pos = a.tok_pos[t];
        float v = y[i];
        if (turned) {
            float sn, cs;
            sincosf((float)pos * a.rate[pair], &sn, &cs);
            sn *= a.mag;
            cs *= a.mag;
            v = low ? v * cs - other[i] * sn : v * cs + other[i] * sn;
        }
        if (c < a.QC) {
            ((T*)a.q_out)[(long long)t * a.ldq + c] = from_f32<T>(v);
        } else {
            if (a.rows_out) {
                // the step's rows side by side: turned keys behind the queries, values behind the keys
                T* o = (T*)a.q_out + (long long)t * a.ldq + a.QC;
                if (cr < a.KC) {
                    o[cr] = from_f32<T>(v);
                    if (a.value_from_key) o[a.KC + cr] = from_f32<T>(y[i]);
                } else {
                    o[cr] = from_f32<T>(v);
                }
            }
            bool keep = !a.no_store;
            int entry = pos;
            if (a.ring > 0) {
                const int end = a.seq_pos0[b] + a.seq_start[b + 1] - a.seq_start[b];
                keep = keep && pos >= end - a.ring;
                entry = pos % a.ring;
            }
            if (keep) {
                const int page = a.ptab[(long long)a.seq_slot[b] * a.ptab_stride + entry / PAGE_TOKENS], row = entry % PAGE_TOKENS;
                if (cr < a.KC) {
                    const int g = cr / a.KW, off = cr - g * a.KW;
                    kv_tile((T*)a.pool, 0, a.pages, page, g, a.G, a.HDC)[(long long)row * a.HDC + off] = from_f32<T>(v);
                    if (a.value_from_key)
                        kv_tile((T*)a.pool, 1, a.pages, page, g, a.G, a.HDC)[(long long)row * a.HDC + off] = from_f32<T>(y[i]);
                } else {
                    const int cv = cr - a.KC, g = cv / a.DV, off = cv - g * a.DV;
                    kv_tile((T*)a.pool, 1, a.pages, page, g, a.G, a.HDC)[(long long)row * a.HDC + off] = from_f32<T>(v);
                }
            }
        }
        if (a.one_token_each && a.K > 1) {
            float* st = a.state + (long long)a.seq_slot[b] * a.state_stride;
            st[(long long)(pos % a.K) * C + c] = tap_input<T>(a, c, t, pos, a.seq_pos0[b], pos, st);
        }
    }
}

// Two neighbouring channels as floats, and back: one 4-byte access for bfloat16, one 8-byte access for float.
__device__ __forceinline__ float2 load_pair(const bf16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
__device__ __forceinline__ float2 load_pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ void store_pair(bf16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }
__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }

// The interleaved form for long steps: a thread owns the channels c, c + 1 (a rotation pair, so nobody forms a partner's
// filter a second time) and TP_TOK consecutive rows.  The rows' filter inputs overlap: TP_TOK + K - 1 rows are fetched for
// TP_TOK results, each as one access for both channels.  Rows of a step lie side by side per sequence, so the input of
// position s >= p0 of the sequence of row t at position pos is row t - (pos - s); what is older comes from the state (a
// sequence that stands at p0 > 0) or is zero.
#define TP_TOK 8
template <typename T, int K>
__global__ void __launch_bounds__(TR_THREADS)
tap_rotate_pairs_kernel(const TapRotArgs a) {
    // what every thread of the block needs to know of the block's rows, looked up once: sequence (-1: padding), position, the
    // sequence's first position of the step and its end, its slot, and the page of the row's cache entry (-1: not written)
    __shared__ int r_seq[TP_TOK], r_pos[TP_TOK], r_p0[TP_TOK], r_end[TP_TOK], r_slot[TP_TOK], r_page[TP_TOK];
    pdl_trigger();
    pdl_wait();
    const int C = a.QC + a.KC + a.VC;
    const int c = 2 * (blockIdx.y * TR_THREADS + threadIdx.x);
    const int t0 = blockIdx.x * TP_TOK;
    if (threadIdx.x < TP_TOK) {
        const int i = threadIdx.x, t = t0 + i;
        int b = t < a.T ? a.tok_seq[t] : -1, pos = 0, p0 = 0, end = 0, slot = 0, page = -1;
        if (b >= 0) {
            pos = a.tok_pos[t];
            p0 = a.seq_pos0[b];
            end = p0 + a.seq_start[b + 1] - a.seq_start[b];
            slot = a.seq_slot[b];
            const bool keep = a.pool && !a.no_store && (a.ring <= 0 || pos >= end - a.ring);
            const int entry = a.ring > 0 ? pos % a.ring : pos;
            if (keep) page = a.ptab[(long long)slot * a.ptab_stride + entry / PAGE_TOKENS];
        }
        r_seq[i] = b; r_pos[i] = pos; r_p0[i] = p0; r_end[i] = end; r_slot[i] = slot; r_page[i] = page;
    }
    __syncthreads();
    if (c >= C) return;
    const int cr = c < a.QC ? c : c - a.QC;
    const int e = cr % max(a.sub, 1);
    const bool turned = c < a.QC + a.KC && a.rate && e < a.rot;
    const float rate = turned ? a.rate[e >> 1] : 0.f;
    const float b0 = a.bias ? a.bias[c] : 0.f, b1 = a.bias ? a.bias[c + 1] : 0.f;
    float w0[K], w1[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
        w0[j] = a.taps[(long long)c * K + j];
        w1[j] = a.taps[(long long)(c + 1) * K + j];
    }
    float2 u[TP_TOK + K - 1];
#pragma unroll
    for (int r = 0; r < TP_TOK + K - 1; ++r) {
        const int row = t0 - (K - 1) + r;
        u[r] = make_float2(0.f, 0.f);
        if (row >= 0 && row < a.T) {
            u[r] = load_pair((const T*)a.proj + (long long)row * a.ldp + c);
            u[r].x += b0;
            u[r].y += b1;
        }
    }
    // where a key pair lies inside its entry: the same for every row
    const bool is_key = c >= a.QC && cr < a.KC;
    const int g = c < a.QC ? 0 : (is_key ? cr / a.KW : (cr - a.KC) / max(a.DV, 1));
    const int off = c < a.QC ? 0 : (is_key ? cr - g * a.KW : cr - a.KC - g * a.DV);
#pragma unroll
    for (int i = 0; i < TP_TOK; ++i) {
        const int t = t0 + i;
        if (r_seq[i] < 0) continue;
        const int pos = r_pos[i], p0 = r_p0[i];
        float y0 = 0.f, y1 = 0.f;
#pragma unroll
        for (int j = 0; j < K; ++j) {
            const int s = pos - (K - 1) + j;
            float x0 = u[i + j].x, x1 = u[i + j].y;
            if (s < p0) {
                x0 = x1 = 0.f;
                if (s >= 0) {
                    const float* st = a.state + (long long)r_slot[i] * a.state_stride + (long long)(s % K) * C + c;
                    x0 = st[0];
                    x1 = st[1];
                }
            }
            y0 = fmaf(w0[j], x0, y0);
            y1 = fmaf(w1[j], x1, y1);
        }
        if (a.from_zero && K > 1 && pos >= r_end[i] - (K - 1)) {
            // the filter's state after the step: the projected rows of the sequence's last K - 1 positions
            float* st = a.state + (long long)r_slot[i] * a.state_stride + (long long)(pos % K) * C + c;
            st[0] = u[i + K - 1].x;
            st[1] = u[i + K - 1].y;
        }
        float v0 = y0, v1 = y1;
        if (turned) {
            float sn, cs;
            sincosf((float)pos * rate, &sn, &cs);
            sn *= a.mag;
            cs *= a.mag;
            v0 = y0 * cs - y1 * sn;
            v1 = y1 * cs + y0 * sn;
        }
        if (c < a.QC) {
            store_pair((T*)a.q_out + (long long)t * a.ldq + c, v0, v1);
            continue;
        }
        if (a.rows_out) {
            T* o = (T*)a.q_out + (long long)t * a.ldq + a.QC;
            store_pair(o + cr, v0, v1);
            if (is_key && a.value_from_key) store_pair(o + a.KC + cr, y0, y1);
        }
        const int page = r_page[i];
        if (page < 0) continue;
        const int entry = a.ring > 0 ? pos % a.ring : pos;
        const long long at = (long long)(entry % PAGE_TOKENS) * a.HDC + off;
        if (is_key) {
            store_pair(kv_tile((T*)a.pool, 0, a.pages, page, g, a.G, a.HDC) + at, v0, v1);
            if (a.value_from_key) store_pair(kv_tile((T*)a.pool, 1, a.pages, page, g, a.G, a.HDC) + at, y0, y1);
        } else {
            store_pair(kv_tile((T*)a.pool, 1, a.pages, page, g, a.G, a.HDC) + at, v0, v1);
        }
    }
}

// Whether the pairs form can run: interleaved pairs, a long step, and every size and pitch even so that two channels are one
// access (heads, key and value rows, the entry size, the pitches of the rows in and out; bases aligned to two elements).
template <typename T>
static bool tap_pairs_fit(const TapRotArgs& a) {
    const uintptr_t two = 2 * sizeof(T);
    if (!a.interleaved || a.one_token_each || a.T < 64 || a.K > 4) return false;
    if ((a.QC | a.KC | a.VC | a.sub | a.rot | a.KW | a.DV | a.HDC) & 1) return false;
    if ((a.ldp | a.ldq) & 1) return false;
    return !(((uintptr_t)a.proj | (uintptr_t)a.q_out | (uintptr_t)a.pool) % two);
}

template <typename T>
static void launch_tap_pairs(const TapRotArgs& a, cudaStream_t st) {
    const int C = a.QC + a.KC + a.VC;
    dim3 grid((a.T + TP_TOK - 1) / TP_TOK, (C / 2 + TR_THREADS - 1) / TR_THREADS);
    switch (a.K) {
    case 1: cm_launch(tap_rotate_pairs_kernel<T, 1>, grid, TR_THREADS, 0, st, a); break;
    case 2: cm_launch(tap_rotate_pairs_kernel<T, 2>, grid, TR_THREADS, 0, st, a); break;
    case 3: cm_launch(tap_rotate_pairs_kernel<T, 3>, grid, TR_THREADS, 0, st, a); break;
    default: cm_launch(tap_rotate_pairs_kernel<T, 4>, grid, TR_THREADS, 0, st, a); break;
    }
}

// The state after a step of several tokens: the projected rows of the sequence's last K - 1 positions that the
// step brought go to their rows of the ring (older ones lie there already).  A launch of its own, behind the
// outputs: a long step overwrites rows that its first tokens read.
template <typename T>
__global__ void __launch_bounds__(TR_THREADS)
tap_state_kernel(const TapRotArgs a) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.y;
    const int c = blockIdx.x * TR_THREADS + threadIdx.x;
    const int C = a.QC + a.KC + a.VC, K = a.K;
    if (c >= C) return;
    const int s0 = a.seq_start[b], n = a.seq_start[b + 1] - s0;
    if (n <= 0) return;
    const int p0 = a.seq_pos0[b], end = p0 + n;
    float* st = a.state + (long long)a.seq_slot[b] * a.state_stride;
    const float bias = a.bias ? a.bias[c] : 0.f;
    for (int s = max(p0, end - (K - 1)); s < end; ++s)
        st[(long long)(s % K) * C + c] = to_f32(((const T*)a.proj)[(long long)(s0 + s - p0) * a.ldp + c]) + bias;
}

extern "C" int cm_tap_rotate_store(int dt, const TapRotArgs* args, cudaStream_t st) {
    TapRotArgs a = *args;
    if (a.T <= 0) return CM_OK;
    const int C = a.QC + a.KC + a.VC;
    if (a.K < 1 || a.K > TR_MAXK) CM_REFUSE("tap_rotate_store: %d taps (1 to %d)", a.K, TR_MAXK);
    if (a.rate && (a.rot % 2 || a.rot > a.sub || a.sub <= 0 || a.QC % a.sub || a.KC % a.sub))
        CM_REFUSE("tap_rotate_store: %d turned channels in vectors of %d", a.rot, a.sub);
    if ((a.KC || a.VC) && (!a.pool || a.KW > a.HDC || a.DV > a.HDC || a.KC != a.G * a.KW || a.VC != a.G * a.DV))
        CM_REFUSE("tap_rotate_store: %d key and %d value channels do not fit %d heads of %d", a.KC, a.VC, a.G, a.HDC);
    if (a.K > 1 && (!a.state || a.state_stride < (long long)a.K * C)) CM_REFUSE("tap_rotate_store: a state row of %lld floats is too short", a.state_stride);
    if (a.value_from_key && a.VC) CM_REFUSE("tap_rotate_store: values that are the keys come without value channels");
    if (a.interleaved && a.rate && a.rot % 2) CM_REFUSE("tap_rotate_store: %d turned channels in pairs", a.rot);
    if (a.ring < 0 || a.ring % PAGE_TOKENS) CM_REFUSE("tap_rotate_store: a ring of %d entries (whole pages)", a.ring);
    const bool many = a.T >= 512 && !a.one_token_each;               // long steps: four tokens a thread
    dim3 grid(many ? (a.T + 3) / 4 : a.T, (C + TR_THREADS - 1) / TR_THREADS), sgrid((C + TR_THREADS - 1) / TR_THREADS, a.B);
    const bool inline_state = a.from_zero && (dt == DT_F32 ? tap_pairs_fit<float>(a) : tap_pairs_fit<bf16>(a));
    if (!inline_state) a.from_zero = 0;
    if (dt == DT_F32) {
        if (tap_pairs_fit<float>(a)) launch_tap_pairs<float>(a, st);
        else if (many) cm_launch(tap_rotate_store_kernel<float, 4>, grid, TR_THREADS, 0, st, a);
        else cm_launch(tap_rotate_store_kernel<float, 1>, grid, TR_THREADS, 0, st, a);
        CM_CHECK_LAUNCH();
        if (!a.one_token_each && a.K > 1 && !inline_state) cm_launch(tap_state_kernel<float>, sgrid, TR_THREADS, 0, st, a);
    } else if (dt == DT_BF16) {
        if (tap_pairs_fit<bf16>(a)) launch_tap_pairs<bf16>(a, st);
        else if (many) cm_launch(tap_rotate_store_kernel<bf16, 4>, grid, TR_THREADS, 0, st, a);
        else cm_launch(tap_rotate_store_kernel<bf16, 1>, grid, TR_THREADS, 0, st, a);
        CM_CHECK_LAUNCH();
        if (!a.one_token_each && a.K > 1 && !inline_state) cm_launch(tap_state_kernel<bf16>, sgrid, TR_THREADS, 0, st, a);
    } else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// ================================================================================ the two maps
__device__ __forceinline__ bool da_visible(int kpos, int qpos, int window, int keep) {
    return kpos <= qpos && (window <= 0 || qpos - kpos < window || kpos < keep);
}

// what a query's two finished maps become: a lane holds channels lane, lane + 32, ... of both
template <typename T, int NJ>
__device__ __forceinline__ void da_finish(const DiffAttnArgs& a, long long t, int h, const float* acc1, const float* acc2,
                                          float l1, float l2) {
    const int lane = threadIdx.x & 31;
    const float i1 = 1.f / l1, i2 = 1.f / l2;
    float o[NJ], ss = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        o[j] = (lane + 32 * j < a.DV) ? acc1[j] * i1 - a.lambda * (acc2[j] * i2) : 0.f;
        ss = fmaf(o[j], o[j], ss);
    }
    ss = warp_sum(ss);
    float f = a.out_scale / sqrtf(ss / (float)a.DV + a.eps);
    if (a.gate) f *= sigmoid_f32(to_f32(((const T*)a.gate)[t * a.ldg + h]));
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int d = lane + 32 * j;
        if (d < a.DV) ((T*)a.ctx)[t * a.ldc + (long long)h * a.DV + d] = from_f32<T>(o[j] * f);
    }
}

// -------------------------------------------------------------------------------- many rows a sequence
// One block = DA_BQ queries of one head of one sequence (warp w owns queries 4w .. 4w + 3); keys come in
// tiles of 32 from the cache: the tiles that hold kept first tokens, then those the block's windows reach.
// A lane is a key for the scores and a set of channels for the value sums.
#define DA_BQ 32
#define DA_BK 32
#define DA_QPW 4
#define DA_THREADS 256

template <typename T, int NJ>
__global__ void __launch_bounds__(DA_THREADS)
diff_attn_tile_kernel(const DiffAttnArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int D2 = 2 * a.D, ldk = D2 + 1, DV = a.DV;
    float* Qs = smem;                            // [DA_BQ][2D + 1]
    float* Ks = Qs + DA_BQ * ldk;                // [DA_BK][2D + 1]
    float* Vs = Ks + DA_BK * ldk;                // [DA_BK][DV]
    float* Ps = Vs + DA_BK * DV;                 // [2][DA_BQ][DA_BK + 1]
    const int b = blockIdx.z, h = blockIdx.y, g = h / (a.H / a.G);
    const int s0 = a.seq_start[b], n_new = a.seq_start[b + 1] - s0;
    const int p0 = a.seq_pos0[b], len = p0 + n_new;
    const int q0 = p0 + blockIdx.x * DA_BQ;
    if (q0 >= len) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nq = min(DA_BQ, len - q0), q_last = q0 + nq - 1;
    const int* prow = a.ptab + (long long)a.seq_slot[b] * a.ptab_stride;
    for (int e = threadIdx.x; e < DA_BQ * D2; e += DA_THREADS) {
        const int r = e / D2, d = e - r * D2;
        Qs[r * ldk + d] = r < nq ? to_f32(((const T*)a.q)[(long long)(s0 + q0 - p0 + r) * a.ldq + (long long)h * D2 + d]) : 0.f;
    }
    float m1[DA_QPW], l1[DA_QPW], m2[DA_QPW], l2[DA_QPW], acc1[DA_QPW][NJ], acc2[DA_QPW][NJ];
#pragma unroll
    for (int i = 0; i < DA_QPW; ++i) {
        m1[i] = m2[i] = -INFINITY;
        l1[i] = l2[i] = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) acc1[i][j] = acc2[i][j] = 0.f;
    }
    // tiles [0, kept_end) hold kept first tokens; the windows begin in tile win_tile
    const int win_first = a.window > 0 ? max(0, q0 - a.window + 1) : 0;
    const int kept_end = a.window > 0 ? min(a.keep, q_last + 1) : 0;
    const int win_k0 = win_first / DA_BK * DA_BK;
    for (int k0 = 0; k0 <= q_last; k0 += DA_BK) {
        if (k0 >= kept_end && k0 < win_k0) {                 // nothing of this tile is seen: on to the windows
            k0 = win_k0 - DA_BK;
            continue;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < DA_BK * D2; e += DA_THREADS) {
            const int r = e / D2, d = e - r * D2, kp = k0 + r;
            float x = 0.f;
            if (kp < len)
                x = to_f32(kv_tile((const T*)a.pool, 0, a.pages, prow[kp / PAGE_TOKENS], g, a.G, a.HDC)[(long long)(kp % PAGE_TOKENS) * a.HDC + d]);
            Ks[r * ldk + d] = x;
        }
        for (int e = threadIdx.x; e < DA_BK * DV; e += DA_THREADS) {
            const int r = e / DV, d = e - r * DV, kp = k0 + r;
            float x = 0.f;
            if (kp < len)
                x = to_f32(kv_tile((const T*)a.pool, 1, a.pages, prow[kp / PAGE_TOKENS], g, a.G, a.HDC)[(long long)(kp % PAGE_TOKENS) * a.HDC + d]);
            Vs[r * DV + d] = x;
        }
        __syncthreads();
        const int kpos = k0 + lane;
        const float* kr = Ks + lane * ldk;
#pragma unroll
        for (int i = 0; i < DA_QPW; ++i) {
            const int qi = warp * DA_QPW + i, qpos = q0 + qi;
            const float* qr = Qs + qi * ldk;
            float s1 = 0.f, s2 = 0.f;
            for (int d = 0; d < a.D; ++d) {
                s1 = fmaf(qr[d], kr[d], s1);
                s2 = fmaf(qr[a.D + d], kr[a.D + d], s2);
            }
            const bool vis = qi < nq && kpos < len && da_visible(kpos, qpos, a.window, a.keep);
            s1 = vis ? s1 * a.scale : -INFINITY;
            s2 = vis ? s2 * a.scale : -INFINITY;
            const float x1 = fmaxf(m1[i], warp_max(s1)), x2 = fmaxf(m2[i], warp_max(s2));
            float p1 = 0.f, p2 = 0.f, f1 = 1.f, f2 = 1.f;
            if (x1 != -INFINITY) {                   // both maps see the same keys
                p1 = vis ? expf(s1 - x1) : 0.f;
                p2 = vis ? expf(s2 - x2) : 0.f;
                f1 = expf(m1[i] - x1);
                f2 = expf(m2[i] - x2);
            }
            l1[i] = l1[i] * f1 + warp_sum(p1);
            l2[i] = l2[i] * f2 + warp_sum(p2);
            m1[i] = x1;
            m2[i] = x2;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                acc1[i][j] *= f1;
                acc2[i][j] *= f2;
            }
            Ps[qi * (DA_BK + 1) + lane] = p1;
            Ps[(DA_BQ + qi) * (DA_BK + 1) + lane] = p2;
        }
        __syncwarp();
        for (int kk = 0; kk < DA_BK; ++kk) {
            float vv[NJ];
#pragma unroll
            for (int j = 0; j < NJ; ++j) vv[j] = (lane + 32 * j < DV) ? Vs[kk * DV + lane + 32 * j] : 0.f;
#pragma unroll
            for (int i = 0; i < DA_QPW; ++i) {
                const float p1 = Ps[(warp * DA_QPW + i) * (DA_BK + 1) + kk];
                const float p2 = Ps[(DA_BQ + warp * DA_QPW + i) * (DA_BK + 1) + kk];
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    acc1[i][j] = fmaf(p1, vv[j], acc1[i][j]);
                    acc2[i][j] = fmaf(p2, vv[j], acc2[i][j]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < DA_QPW; ++i) {
        const int qi = warp * DA_QPW + i;
        if (qi < nq) da_finish<T, NJ>(a, (long long)s0 + q0 - p0 + qi, h, acc1[i], acc2[i], l1[i], l2[i]);
    }
}

// -------------------------------------------------------------------------------- a row at a time
// One block = one row (token), one head (or four heads of one key/value head) and one share of the row's visible keys: the tiles of 32 keys that hold
// kept first tokens or lie in the row's window are dealt out in turns to the warps of `splits` blocks.  Each warp
// keeps running maxima and sums of its own; a block merges its warps in warp order, and (with more than one
// share) leaves maxima, sums and value sums in `parts`, which diff_attn_merge_kernel adds in share order.  A lane is
// a key for the scores (its key's row read from the cache, 16 bytes at a time where the layout allows) and a set
// of channels for the value sums.
#define DR_WARPS 4

// a key row [map 1 | map 2] against R heads' query vectors (Qs: R rows of 2 D floats)
template <typename T, int R>
__device__ __forceinline__ void da_key_dots(const T* kr, const float* Qs, int D, bool vec, float* s1, float* s2) {
#pragma unroll
    for (int r = 0; r < R; ++r) s1[r] = s2[r] = 0.f;
    if (vec) {
        for (int d = 0; d < D; d += 8) {
            float k1[8], k2[8];
            load8f<T>(kr + d, k1);
            load8f<T>(kr + D + d, k2);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float* q = Qs + r * 2 * D;
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    s1[r] = fmaf(q[d + x], k1[x], s1[r]);
                    s2[r] = fmaf(q[D + d + x], k2[x], s2[r]);
                }
            }
        }
    } else {
        for (int d = 0; d < D; ++d) {
            const float k1 = to_f32(kr[d]), k2 = to_f32(kr[D + d]);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                s1[r] = fmaf(Qs[r * 2 * D + d], k1, s1[r]);
                s2[r] = fmaf(Qs[r * 2 * D + D + d], k2, s2[r]);
            }
        }
    }
}

// R: query heads of one key/value head that a block takes together (they read the same keys and values).
template <typename T, int NJ, int R>
__global__ void __launch_bounds__(DR_WARPS * 32)
diff_attn_row_kernel(const DiffAttnArgs a, float* __restrict__ parts, int splits) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int D2 = 2 * a.D, DV = a.DV;
    float* Qs = smem;                            // [R][2D]
    float* Ms = Qs + R * D2;                     // [DR_WARPS][R][4]: m1, l1, m2, l2
    float* As = Ms + DR_WARPS * R * 4;           // [DR_WARPS][R][2][DV]
    const long long t = blockIdx.y;
    const int h0 = blockIdx.x * R, g = h0 / (a.H / a.G), share = blockIdx.z;
    const int b = a.tok_seq[t];
    if (b < 0) return;
    const int qpos = a.tok_pos[t];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int* prow = a.ptab + (long long)a.seq_slot[b] * a.ptab_stride;
    for (int d = threadIdx.x; d < R * D2; d += DR_WARPS * 32) Qs[d] = to_f32(((const T*)a.q)[t * a.ldq + (long long)h0 * D2 + d]);
    __syncthreads();
    float m1[R], m2[R], l1[R], l2[R], acc1[R][NJ], acc2[R][NJ];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        m1[r] = m2[r] = -INFINITY;
        l1[r] = l2[r] = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) acc1[r][j] = acc2[r][j] = 0.f;
    }
    const int last_tile = qpos / 32;
    const int kept_tiles = a.window > 0 ? min((min(a.keep, qpos + 1) + 31) / 32, last_tile + 1) : 0;
    const int win_tile = a.window > 0 ? max(kept_tiles, max(0, qpos - a.window + 1) / 32) : 0;
    const int n_tiles = kept_tiles + (last_tile - win_tile + 1);
    const bool vec = a.D % 8 == 0 && a.HDC % 8 == 0 && ((uintptr_t)a.pool & 15) == 0;
    for (int idx = share * DR_WARPS + warp; idx < n_tiles; idx += splits * DR_WARPS) {
        const int tile = idx < kept_tiles ? idx : win_tile + idx - kept_tiles;
        const int kpos = tile * 32 + lane;
        const bool vis = da_visible(kpos, qpos, a.window, a.keep);
        const unsigned seen = __ballot_sync(0xffffffffu, vis);
        if (!seen) continue;                     // no key of this tile is seen
        const int page = kpos <= qpos ? prow[kpos / PAGE_TOKENS] : 0;
        float s1[R], s2[R], p1[R], p2[R];
#pragma unroll
        for (int r = 0; r < R; ++r) s1[r] = s2[r] = 0.f;
        if (vis)
            da_key_dots<T, R>(kv_tile((const T*)a.pool, 0, a.pages, page, g, a.G, a.HDC) + (long long)(kpos % PAGE_TOKENS) * a.HDC,
                              Qs, a.D, vec, s1, s2);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float v1 = vis ? s1[r] * a.scale : -INFINITY, v2 = vis ? s2[r] * a.scale : -INFINITY;
            const float x1 = fmaxf(m1[r], warp_max(v1)), x2 = fmaxf(m2[r], warp_max(v2));
            p1[r] = vis ? expf(v1 - x1) : 0.f;
            p2[r] = vis ? expf(v2 - x2) : 0.f;
            const float f1 = expf(m1[r] - x1), f2 = expf(m2[r] - x2);
            l1[r] = l1[r] * f1 + warp_sum(p1[r]);
            l2[r] = l2[r] * f2 + warp_sum(p2[r]);
            m1[r] = x1;
            m2[r] = x2;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                acc1[r][j] *= f1;
                acc2[r][j] *= f2;
            }
        }
        // a tile of 32 keys lies within one page of 64
        const int tile_page = __shfl_sync(0xffffffffu, page, __ffs(seen) - 1);
        const T* vt = kv_tile((const T*)a.pool, 1, a.pages, tile_page, g, a.G, a.HDC) + (long long)((tile * 32) % PAGE_TOKENS) * a.HDC;
#pragma unroll 2
        for (int kk = 0; kk < 32; ++kk) {
            if (!((seen >> kk) & 1u)) continue;  // an unseen key's values may never have been written
            const T* vr = vt + (long long)kk * a.HDC;
            float v[NJ];
#pragma unroll
            for (int j = 0; j < NJ; ++j) v[j] = lane + 32 * j < DV ? to_f32(vr[lane + 32 * j]) : 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float q1 = __shfl_sync(0xffffffffu, p1[r], kk), q2 = __shfl_sync(0xffffffffu, p2[r], kk);
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    acc1[r][j] = fmaf(q1, v[j], acc1[r][j]);
                    acc2[r][j] = fmaf(q2, v[j], acc2[r][j]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (lane == 0) {
            float* ms = Ms + (warp * R + r) * 4;
            ms[0] = m1[r];
            ms[1] = l1[r];
            ms[2] = m2[r];
            ms[3] = l2[r];
        }
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int d = lane + 32 * j;
            if (d < DV) {
                As[((warp * R + r) * 2) * DV + d] = acc1[r][j];
                As[((warp * R + r) * 2 + 1) * DV + d] = acc2[r][j];
            }
        }
    }
    __syncthreads();
    // warp w merges head w, w + DR_WARPS, ... of the block's heads over the warps' partial results, in warp order
    for (int r = warp; r < R; r += DR_WARPS) {
        float M1 = -INFINITY, M2 = -INFINITY;
        for (int w = 0; w < DR_WARPS; ++w) {
            M1 = fmaxf(M1, Ms[(w * R + r) * 4]);
            M2 = fmaxf(M2, Ms[(w * R + r) * 4 + 2]);
        }
        float L1 = 0.f, L2 = 0.f, o1[NJ], o2[NJ];
#pragma unroll
        for (int j = 0; j < NJ; ++j) o1[j] = o2[j] = 0.f;
        for (int w = 0; w < DR_WARPS; ++w) {
            const float* ms = Ms + (w * R + r) * 4;
            if (ms[0] == -INFINITY) continue;    // a warp that saw no tile
            const float f1 = expf(ms[0] - M1), f2 = expf(ms[2] - M2);
            L1 = fmaf(ms[1], f1, L1);
            L2 = fmaf(ms[3], f2, L2);
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int d = lane + 32 * j;
                if (d < DV) {
                    o1[j] = fmaf(As[((w * R + r) * 2) * DV + d], f1, o1[j]);
                    o2[j] = fmaf(As[((w * R + r) * 2 + 1) * DV + d], f2, o2[j]);
                }
            }
        }
        const int h = h0 + r;
        if (splits == 1) {
            da_finish<T, NJ>(a, t, h, o1, o2, L1, L2);
            continue;
        }
        float* part = parts + ((t * a.H + h) * splits + share) * (long long)(4 + 2 * DV);
        if (lane == 0) {
            part[0] = M1;
            part[1] = L1;
            part[2] = M2;
            part[3] = L2;
        }
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int d = lane + 32 * j;
            if (d < DV) {
                part[4 + d] = o1[j];
                part[4 + DV + d] = o2[j];
            }
        }
    }
}

// The shares of a row and head, added in share order; one warp per (row, head).
template <typename T, int NJ>
__global__ void __launch_bounds__(32)
diff_attn_merge_kernel(const DiffAttnArgs a, const float* __restrict__ parts, int splits) {
    pdl_trigger();
    pdl_wait();
    const long long t = blockIdx.y;
    const int h = blockIdx.x, lane = threadIdx.x, DV = a.DV;
    if (a.tok_seq[t] < 0) return;
    const float* part = parts + (t * a.H + h) * splits * (long long)(4 + 2 * DV);
    float M1 = -INFINITY, M2 = -INFINITY;
    for (int s = 0; s < splits; ++s) {
        M1 = fmaxf(M1, part[s * (4 + 2 * DV)]);
        M2 = fmaxf(M2, part[s * (4 + 2 * DV) + 2]);
    }
    float L1 = 0.f, L2 = 0.f, o1[NJ], o2[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) o1[j] = o2[j] = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float* ps = part + s * (long long)(4 + 2 * DV);
        if (ps[0] == -INFINITY) continue;        // a share without a visible tile
        const float f1 = expf(ps[0] - M1), f2 = expf(ps[2] - M2);
        L1 = fmaf(ps[1], f1, L1);
        L2 = fmaf(ps[3], f2, L2);
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int d = lane + 32 * j;
            if (d < DV) {
                o1[j] = fmaf(ps[4 + d], f1, o1[j]);
                o2[j] = fmaf(ps[4 + DV + d], f2, o2[j]);
            }
        }
    }
    da_finish<T, NJ>(a, t, h, o1, o2, L1, L2);
}

template <typename T, int NJ>
static int da_launch(const DiffAttnArgs& a, int rows_form, int max_len, float* parts, int splits, cudaStream_t st) {
    if (rows_form) {
        // the query heads of a key/value head four at a time where their number allows it (the binding counts blocks by the same rule)
        const int R = (a.H / a.G) % 4 == 0 ? 4 : 1;
        const size_t smem = ((size_t)R * 2 * a.D + DR_WARPS * R * 4 + (size_t)DR_WARPS * R * 2 * a.DV) * sizeof(float);
        if (R == 4) {
            if (smem > 48 * 1024) cudaFuncSetAttribute(diff_attn_row_kernel<T, NJ, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            cm_launch(diff_attn_row_kernel<T, NJ, 4>, dim3(a.H / 4, a.T, splits), DR_WARPS * 32, smem, st, a, parts, splits);
        } else {
            if (smem > 48 * 1024) cudaFuncSetAttribute(diff_attn_row_kernel<T, NJ, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            cm_launch(diff_attn_row_kernel<T, NJ, 1>, dim3(a.H, a.T, splits), DR_WARPS * 32, smem, st, a, parts, splits);
        }
        if (splits > 1) {
            CM_CHECK_LAUNCH();
            cm_launch(diff_attn_merge_kernel<T, NJ>, dim3(a.H, a.T), 32, 0, st, a, (const float*)parts, splits);
        }
    } else {
        const size_t smem = ((size_t)(DA_BQ + DA_BK) * (2 * a.D + 1) + (size_t)DA_BK * a.DV + 2 * DA_BQ * (DA_BK + 1)) * sizeof(float);
        if (smem > 200 * 1024) CM_REFUSE("diff_attn: heads of 2 x %d and %d channels do not fit shared memory", a.D, a.DV);
        if (smem > 48 * 1024) cudaFuncSetAttribute(diff_attn_tile_kernel<T, NJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cm_launch(diff_attn_tile_kernel<T, NJ>, dim3((max_len + DA_BQ - 1) / DA_BQ, a.H, a.B), DA_THREADS, smem, st, a);
    }
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// rows_form: one block per row, head and share of the keys (steps of one or few tokens a sequence), `splits` shares
// with `parts` [T][H][splits][4 + 2 DV] floats between the two launches (splits 1: one launch, no parts); else tiles
// of 32 queries, launched for sequences of up to max_len new tokens.
extern "C" int cm_diff_attn(int dt, const DiffAttnArgs* args, int rows_form, int max_len, float* parts, int splits,
                            cudaStream_t st) {
    const DiffAttnArgs a = *args;
    if (a.T <= 0 || a.B <= 0) return CM_OK;
    if (a.D <= 0 || a.DV <= 0 || a.DV > CM_MAX_HEAD_DIM || 2 * a.D > a.HDC || a.DV > a.HDC)
        CM_REFUSE("diff_attn: heads of 2 x %d key and %d value channels in entries of %d (values up to %d)", a.D, a.DV, a.HDC, CM_MAX_HEAD_DIM);
    if (a.G <= 0 || a.H % a.G) CM_REFUSE("diff_attn: %d query heads over %d key heads", a.H, a.G);
    if (!rows_form && max_len <= 0) return CM_OK;
    if (splits < 1 || (splits > 1 && !parts)) CM_REFUSE("diff_attn: %d shares need their scratch", splits);
    const int nj = (a.DV + 31) / 32;
#define DA_DISPATCH(TT)                                                                    \
    do {                                                                                   \
        if (nj <= 1) return da_launch<TT, 1>(a, rows_form, max_len, parts, splits, st);    \
        if (nj == 2) return da_launch<TT, 2>(a, rows_form, max_len, parts, splits, st);    \
        if (nj == 3) return da_launch<TT, 3>(a, rows_form, max_len, parts, splits, st);    \
        if (nj == 4) return da_launch<TT, 4>(a, rows_form, max_len, parts, splits, st);    \
        if (nj <= 6) return da_launch<TT, 6>(a, rows_form, max_len, parts, splits, st);    \
        return da_launch<TT, 8>(a, rows_form, max_len, parts, splits, st);                 \
    } while (0)
    if (dt == DT_F32) DA_DISPATCH(float);
    if (dt == DT_BF16) DA_DISPATCH(bf16);
#undef DA_DISPATCH
    return CM_ERR_DTYPE;
}
