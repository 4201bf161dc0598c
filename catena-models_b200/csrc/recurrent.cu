// Mixers with a matrix-valued state per head that is carried from token to token:
//
//   decay mix      o_t = (S + diag(u) k_t v_t^T)^T r_t ;  S <- diag(w_t) S + k_t v_t^T
//                  (per-channel decay w_t in (0, 1) that depends on the token, bonus u for the present token)
//   matrix memory  m' = max(f + m, i) ;  S <- e^(f + m - m') S + e^(i - m') k v^T ;  n likewise with k alone ;
//                  o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)         (log-domain gates i, f with a running maximum m)
//   constant decay S <- w S + k v^T ;  o = S^T q                      (one decay w in (0, 1] per head, the same for
//                  every token; q, k and v may pass through silu on their way in: lightning attention)
//
// followed by the unit norm of each head's output, the channel weights and the output gate.  State, gates,
// decays and all sums are float whatever the activation type.  The state lives in per-slot rows of a float
// array; a step starts from what is stored there (zeros for a new sequence) and leaves its last state, so
// whole prompts, portions of prompts and single tokens run the same code and give the same numbers.  A block
// owns some columns of one head's state for one sequence and walks the sequence's rows of the step in order;
// rows that belong to no sequence (padding) are never touched.
//
// Beside it: the token shift (each projection reads its own blend of the present and the previous
// token's input), the low-rank decay network, and the capped gate pre-activations.
#include "common.cuh"
#include "recurrent.h"
#include <math.h>

// ------------------------------------------------------------------------------ token shift
// out[s][t] = T(h[t] + (prev[t] - h[t]) * mu[s]) for s < S, prev[t] = h[t - 1] within a sequence's rows of
// the step, and the stored previous input (the head of the sequence's state row) for its first row.
template <typename T>
__global__ void shift_mix_kernel(T* __restrict__ out, const T* __restrict__ h, const float* __restrict__ mu,
                                 const float* __restrict__ state, long long state_stride,
                                 const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                 const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot, int S,
                                 long long rows, int W) {
    pdl_trigger();
    pdl_wait();
    const long long t = blockIdx.x;
    const int b = tok_seq[t];
    if (b < 0) return;
    const bool first = tok_pos[t] == seq_pos0[b];
    const float* sp = state + (long long)seq_slot[b] * state_stride;
    const T* hp = h + (t - 1) * W;
    const T* hr = h + t * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float x = to_f32(hr[c]);
        const float d = (first ? sp[c] : to_f32(hp[c])) - x;
        for (int s = 0; s < S; ++s) out[((long long)s * rows + t) * W + c] = from_f32<T>(fmaf(d, mu[(long long)s * W + c], x));
    }
}

extern "C" int cm_shift_mix(int dt, void* out, const void* h, const float* mu, const float* state,
                            long long state_stride, const int* tok_seq, const int* tok_pos, const int* seq_pos0,
                            const int* seq_slot, int S, long long rows, int W, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    const int threads = W >= 1024 ? 256 : 128;
    if (dt == DT_F32)
        cm_launch(shift_mix_kernel<float>, (unsigned)rows, threads, 0, st, (float*)out, (const float*)h, mu, state,
                  state_stride, tok_seq, tok_pos, seq_pos0, seq_slot, S, rows, W);
    else if (dt == DT_BF16)
        cm_launch(shift_mix_kernel<bf16>, (unsigned)rows, threads, 0, st, (bf16*)out, (const bf16*)h, mu, state,
                  state_stride, tok_seq, tok_pos, seq_pos0, seq_slot, S, rows, W);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// ------------------------------------------------------------------------- small row products
// A warp's dot products of one weight row with RT rows of x (float sums, lanes stride the columns).
#define RP_ROWS 4
#define RP_THREADS 256
template <typename T>
__device__ __forceinline__ void warp_row_dots(const T* __restrict__ wrow, const T* __restrict__ x, long long ldx,
                                              int n_rows, int W, float* acc) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int r = 0; r < RP_ROWS; ++r) acc[r] = 0.f;
    if (W % 8 == 0 && ldx % 8 == 0) {                  // 16-byte accesses: eight columns a lane and round
        for (int c = lane * 8; c < W; c += 256) {
            float wv[8], xv[8];
            load8f<T>(wrow + c, wv);
#pragma unroll
            for (int r = 0; r < RP_ROWS; ++r)
                if (r < n_rows) {
                    load8f<T>(x + r * ldx + c, xv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[r] = fmaf(wv[i], xv[i], acc[r]);
                }
        }
#pragma unroll
        for (int r = 0; r < RP_ROWS; ++r) acc[r] = warp_sum(acc[r]);
        return;
    }
    for (int c = lane; c < W; c += 32) {
        const float wv = to_f32(wrow[c]);
#pragma unroll
        for (int r = 0; r < RP_ROWS; ++r)
            if (r < n_rows) acc[r] = fmaf(wv, to_f32(x[r * ldx + c]), acc[r]);
    }
#pragma unroll
    for (int r = 0; r < RP_ROWS; ++r) acc[r] = warp_sum(acc[r]);
}

// A decay per token and channel out of a low-rank network, in float.  kind 0 (decay mix): w = exp(-exp(W2 tanh(W1 x) + w0));
// kind 1 (gated linear attention): w = sigmoid(W2 (W1 x) + w0)^(1/tau), formed as exp(log sigmoid(z) / tau).
// x [rows][W], W1 [R][W], W2 stored transposed [R][C] (neighbouring threads read neighbouring channels), w0 [C];
// out [rows][C] float.
__device__ __forceinline__ float log_sigmoid_f32(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float decay_of(float z, int kind, float inv_tau) {
    return kind == 1 ? expf(log_sigmoid_f32(z) * inv_tau) : expf(-expf(z));
}

template <typename T>
__global__ void __launch_bounds__(RP_THREADS)
lowrank_decay_kernel(float* __restrict__ out, const T* __restrict__ x, const T* __restrict__ w1,
                     const T* __restrict__ w2, const float* __restrict__ w0, long long rows, int W, int R, int C, int kind,
                     float inv_tau) {
    extern __shared__ float th[];                     // [RP_ROWS][R]
    pdl_trigger();
    pdl_wait();
    const long long row0 = (long long)blockIdx.x * RP_ROWS;
    const int n_rows = (int)min((long long)RP_ROWS, rows - row0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < R; r += RP_THREADS / 32) {
        float acc[RP_ROWS];
        warp_row_dots<T>(w1 + (long long)r * W, x + row0 * W, W, n_rows, W, acc);
        if (lane == 0)
            for (int i = 0; i < RP_ROWS; ++i) th[i * R + r] = kind == 1 ? acc[i] : tanhf(acc[i]);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_rows * C; e += RP_THREADS) {
        const int i = e / C, c = e - i * C;
        float z = 0.f;
        for (int r = 0; r < R; ++r) z = fmaf(to_f32(w2[(long long)r * C + c]), th[i * R + r], z);
        out[(row0 + i) * C + c] = decay_of(z + w0[c], kind, inv_tau);
    }
}

extern "C" int cm_lowrank_decay(int dt, float* out, const void* x, const void* w1, const void* w2, const float* w0,
                                long long rows, int W, int R, int C, int kind, float tau, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    if (kind == 1 && !(tau > 0.f)) CM_REFUSE("lowrank_decay: tau %f", tau);
    const float inv_tau = kind == 1 ? 1.f / tau : 0.f;
    const size_t smem = (size_t)RP_ROWS * R * sizeof(float);
    if (smem > 48 * 1024) CM_REFUSE("lowrank_decay: rank %d is too large", R);
    const unsigned grid = (unsigned)((rows + RP_ROWS - 1) / RP_ROWS);
    if (dt == DT_F32)
        cm_launch(lowrank_decay_kernel<float>, grid, RP_THREADS, smem, st, out, (const float*)x, (const float*)w1,
                  (const float*)w2, w0, rows, W, R, C, kind, inv_tau);
    else if (dt == DT_BF16)
        cm_launch(lowrank_decay_kernel<bf16>, grid, RP_THREADS, smem, st, out, (const bf16*)x, (const bf16*)w1,
                  (const bf16*)w2, w0, rows, W, R, C, kind, inv_tau);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// The decay network through the runtime's products (ranks that fill a tensor-core tile): tanh in place on the
// first product's result, and w = exp(-exp(z + w0)) from the second product's float result.
template <typename T>
__global__ void tanh_inplace_kernel(T* __restrict__ x, long long n) {
    pdl_trigger();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] = from_f32<T>(tanhf(to_f32(x[i])));
}

__global__ void decay_from_logits_kernel(float* __restrict__ out, const float* __restrict__ z, const float* __restrict__ w0,
                                         long long n, int C, int kind, float inv_tau) {
    pdl_trigger();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = decay_of(z[i] + w0[i % C], kind, inv_tau);
}

extern "C" int cm_tanh_inplace(int dt, void* x, long long n, cudaStream_t st) {
    if (n <= 0) return CM_OK;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    if (dt == DT_F32) cm_launch(tanh_inplace_kernel<float>, grid, 256, 0, st, (float*)x, n);
    else if (dt == DT_BF16) cm_launch(tanh_inplace_kernel<bf16>, grid, 256, 0, st, (bf16*)x, n);
    else return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

extern "C" int cm_decay_from_logits(float* out, const float* z, const float* w0, long long rows, int C, int kind, float tau,
                                    cudaStream_t st) {
    const long long n = rows * C;
    if (n <= 0) return CM_OK;
    if (kind == 1 && !(tau > 0.f)) CM_REFUSE("decay_from_logits: tau %f", tau);
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    cm_launch(decay_from_logits_kernel, grid, 256, 0, st, out, z, w0, n, C, kind, kind == 1 ? 1.f / tau : 0.f);
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// Capped gate pre-activations of the matrix memory: z = W h + b for 2 * H rows of W (input gates, then
// forget gates); out[t][o] = cap * tanh(z / cap), and the logarithm of its sigmoid for the forget gates.
template <typename T>
__global__ void __launch_bounds__(RP_THREADS)
capped_gates_kernel(float* __restrict__ out, const T* __restrict__ x, const T* __restrict__ w,
                    const float* __restrict__ bias, float cap, long long rows, int W, int H) {
    pdl_trigger();
    pdl_wait();
    const long long row0 = (long long)blockIdx.x * RP_ROWS;
    const int n_rows = (int)min((long long)RP_ROWS, rows - row0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int o = warp; o < 2 * H; o += RP_THREADS / 32) {
        float acc[RP_ROWS];
        warp_row_dots<T>(w + (long long)o * W, x + row0 * W, W, n_rows, W, acc);
        if (lane == 0)
            for (int i = 0; i < n_rows; ++i) {
                float g = cap * tanhf((acc[i] + bias[o]) / cap);
                if (o >= H) g = log_sigmoid_f32(g);
                out[(row0 + i) * 2 * H + o] = g;
            }
    }
}

extern "C" int cm_capped_gates(int dt, float* out, const void* x, const void* w, const float* bias, float cap,
                               long long rows, int W, int H, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    const unsigned grid = (unsigned)((rows + RP_ROWS - 1) / RP_ROWS);
    if (dt == DT_F32)
        cm_launch(capped_gates_kernel<float>, grid, RP_THREADS, 0, st, out, (const float*)x, (const float*)w, bias, cap, rows, W, H);
    else if (dt == DT_BF16)
        cm_launch(capped_gates_kernel<bf16>, grid, RP_THREADS, 0, st, out, (const bf16*)x, (const bf16*)w, bias, cap, rows, W, H);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// ------------------------------------------------------------------------------ the scan
#define SCAN_THREADS 128
#define SCAN_MAX_ROWS 32          // rows of the step that a block stages at a time

template <int N>
__device__ __forceinline__ void load_run(const float* p, float* out) {
    if constexpr (N % 4 == 0) {
#pragma unroll
        for (int x = 0; x < N; x += 4) {
            const float4 t = *reinterpret_cast<const float4*>(p + x);
            out[x] = t.x; out[x + 1] = t.y; out[x + 2] = t.z; out[x + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int x = 0; x < N; x += 2) {
            const float2 t = *reinterpret_cast<const float2*>(p + x);
            out[x] = t.x; out[x + 1] = t.y;
        }
    }
}

// MODE 0: decay mix.  MODE 1: matrix memory.  MODE 2: constant decay per head (a.decay [H]).  MODE 3: a decay per token and key
// channel as MODE 0 has it, applied before the output is read: S <- diag(w_t) S + k_t v_t^T, o_t = S^T q_t (gated linear
// attention).  A block owns some columns of one head's S for one sequence and
// walks the sequence's rows of the step in order.  Thread (column c, part ks) keeps S[i][c] for the RPT key
// channels i = ks * RPT ... in registers.  For the matrix memory the block's last column is the normaliser n: it
// is the column of S whose value channel is constantly one (n <- a n + b k, and its output is n . q), so it needs
// no code of its own; every block keeps a copy, and all copies see the same operations.
// The block stages the operands of up to SCAN_MAX_ROWS rows in shared memory at a time (as floats: q times its
// scale, k, the decay, its columns of v), so the latency of global memory is paid once per group of rows.  For the
// matrix memory the first warp then walks the gates of the group (the running maximum is a chain; the
// exponentials of all rows are formed side by side).  The walk of the state over the group needs no barrier, no
// exchange and no exponential: a thread leaves its part of every row's output in shared memory, and once the
// group is through, the parts of a column are added in index order and divided by the normaliser.  Columns do
// not depend on each other, so the split over blocks changes no number, and an element of S sees the same
// operations in the same order whatever the number of parts.  Outputs go to `raw` in float; the unit norm over a
// head's columns, the channel weights and the gate follow in head_norm_gate_kernel.
template <typename T, int MODE, int RPT>
__global__ void __launch_bounds__(SCAN_THREADS)
matrix_scan_kernel(const ScanArgs a, int TB) {
    extern __shared__ __align__(16) float sm[];
    pdl_trigger();
    pdl_wait();
    const int hd = blockIdx.x, cb = blockIdx.y, b = blockIdx.z;
    const int s0 = a.seq_start[b], s1 = a.seq_start[b + 1];
    if (s1 <= s0) return;
    const int D = a.D, DV = a.DV, KS = a.KS, H = a.H;
    const int Dp = KS * RPT;                          // a staged row's pitch: the parts' runs of channels, D <= Dp
    const int cols = SCAN_THREADS / KS;               // columns of the block, the normaliser's among them
    const int real = MODE == 1 ? cols - 1 : cols;     // columns of S proper
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ks = threadIdx.x % KS, c = threadIdx.x / KS, j = cb * real + c;
    const bool is_n = MODE == 1 && c == real;
    const bool active = is_n || j < DV;
    const int i0 = ks * RPT;
    float* sq = sm;                                   // [TB][Dp]
    float* sk = sq + (size_t)TB * Dp;                 // [TB][Dp]
    float* sw = sk + (size_t)TB * Dp;                 // [TB][Dp]  (MODE 0)
    constexpr bool CH = MODE == 0 || MODE == 3;       // a decay per token and key channel
    float* sv = sw + (CH ? (size_t)TB * Dp : 0);      // [TB][cols]
    float* sg = sv + (size_t)TB * cols;               // [TB][4]: MODE 1: a = e^(f + m - m'), b = e^(i - m'), e^(-m')
    float* part = sg + (size_t)TB * 4;                // [TB][KS][cols] partial outputs
    const long long per_head = (long long)D * DV + (MODE == 1 ? D + 1 : 0);
    float* st = a.state + (long long)a.seq_slot[b] * a.state_stride + a.state_offset + hd * per_head;
    float S[RPT], U[RPT];
#pragma unroll
    for (int it = 0; it < RPT; ++it) {
        const int i = i0 + it;
        S[it] = (active && i < D) ? (is_n ? st[(long long)D * DV + i] : st[(long long)i * DV + j]) : 0.f;
        U[it] = (MODE == 0 && i < D) ? a.bonus[hd * D + i] : 0.f;
    }
    float m = MODE == 1 ? st[(long long)D * DV + D] : 0.f;      // the first warp carries it
    const T* Q = (const T*)a.q + (long long)hd * D;
    const T* K = (const T*)a.k + (long long)hd * D;
    const T* V = (const T*)a.v + (long long)hd * DV + (long long)cb * real;
    const float* Wd = a.decay + (CH ? (long long)hd * D : 0);
    const float w_head = MODE == 2 ? a.decay[hd] : 1.f;
    const bool act = MODE == 2 && a.qkv_act;
    const long long ldw = CH ? (long long)H * D : 2LL * H;
    float* R = a.raw + (long long)hd * DV + (long long)cb * real;
    const long long ldr = (long long)H * DV;
    const int n_cols = max(0, min(real, DV - cb * real));
    // 16-byte accesses to q, k and the decay: heads of a multiple of 8 channels in rows and buffers aligned to match
    const bool vec8 = D % 8 == 0 && a.ldq % 8 == 0 && a.ldk % 8 == 0 && (ldw % 8 == 0 || !CH) &&
                      (((uintptr_t)a.q | (uintptr_t)a.k) & 15) == 0 && (!CH || ((uintptr_t)a.decay & 31) == 0);
    // channels past D of a staged row are read by the last part's vector accesses: they hold zeros
    for (int e = threadIdx.x; e < TB * (Dp - D); e += SCAN_THREADS) {
        const int tt = e / (Dp - D), i = D + e - tt * (Dp - D);
        sq[(size_t)tt * Dp + i] = 0.f;
        sk[(size_t)tt * Dp + i] = 0.f;
        if (CH) sw[(size_t)tt * Dp + i] = 0.f;
    }
    for (long long t0 = s0; t0 < s1; t0 += TB) {
        const int nt = (int)min((long long)TB, s1 - t0);
        __syncthreads();                 // the group before is no longer read
        if (vec8) {
            // eight channels per access, four accesses of each operand in flight before the first is stored
            const int D8 = D >> 3, n8 = nt * D8;
            for (int e0 = threadIdx.x; e0 < n8; e0 += 4 * SCAN_THREADS) {
                float fq[4][8], fk[4][8], fw[4][8];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int e = e0 + u * SCAN_THREADS;
                    if (e < n8) {
                        const int tt = e / D8, i = (e - tt * D8) * 8;
                        load8f<T>(Q + (t0 + tt) * a.ldq + i, fq[u]);
                        load8f<T>(K + (t0 + tt) * a.ldk + i, fk[u]);
                        if (CH) load8f<float>(Wd + (t0 + tt) * ldw + i, fw[u]);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int e = e0 + u * SCAN_THREADS;
                    if (e < n8) {
                        const int tt = e / D8, i = (e - tt * D8) * 8;
                        if (act) {
#pragma unroll
                            for (int x = 0; x < 8; ++x) {
                                fq[u][x] *= sigmoid_f32(fq[u][x]);
                                fk[u][x] *= sigmoid_f32(fk[u][x]);
                            }
                        }
#pragma unroll
                        for (int x = 0; x < 8; ++x) fq[u][x] *= a.q_scale;
                        store8f<float>(sq + (size_t)tt * Dp + i, fq[u]);
                        store8f<float>(sk + (size_t)tt * Dp + i, fk[u]);
                        if (CH) store8f<float>(sw + (size_t)tt * Dp + i, fw[u]);
                    }
                }
            }
        } else {
            for (int e = threadIdx.x; e < nt * D; e += SCAN_THREADS) {
                const int tt = e / D, i = e - tt * D;
                float fq = to_f32(Q[(t0 + tt) * a.ldq + i]), fk = to_f32(K[(t0 + tt) * a.ldk + i]);
                if (act) {
                    fq *= sigmoid_f32(fq);
                    fk *= sigmoid_f32(fk);
                }
                sq[(size_t)tt * Dp + i] = fq * a.q_scale;
                sk[(size_t)tt * Dp + i] = fk;
                if (CH) sw[(size_t)tt * Dp + i] = Wd[(t0 + tt) * ldw + i];
            }
        }
        for (int e = threadIdx.x; e < nt * cols; e += SCAN_THREADS) {
            const int tt = e / cols, cc = e - tt * cols;
            float fv = (MODE == 1 && cc == real) ? 1.f : (cc < n_cols ? to_f32(V[(t0 + tt) * a.ldv + cc]) : 0.f);
            if (act) fv *= sigmoid_f32(fv);
            sv[e] = fv;
        }
        if (MODE == 1 && warp == 0) {
            // the gates of the group: lane tt fetches row tt's pair; the running maximum is a chain over the rows, which
            // every lane walks (keeping its own row's values); the exponentials of all rows are then formed side by side
            const float g_i = lane < nt ? Wd[(t0 + lane) * ldw + hd] : 0.f;
            const float g_f = lane < nt ? Wd[(t0 + lane) * ldw + H + hd] : 0.f;
            float mm = m, my_a = 0.f, my_b = 0.f, my_m = 0.f;
            for (int tt = 0; tt < nt; ++tt) {
                const float ig = __shfl_sync(0xffffffffu, g_i, tt), fg = __shfl_sync(0xffffffffu, g_f, tt);
                const float m_new = fmaxf(fg + mm, ig);
                if (tt == lane) {
                    my_a = fg + mm - m_new;
                    my_b = ig - m_new;
                    my_m = -m_new;
                }
                mm = m_new;
            }
            if (lane < nt) {
                sg[4 * lane] = expf(my_a);
                sg[4 * lane + 1] = expf(my_b);
                sg[4 * lane + 2] = expf(my_m);
            }
            m = mm;
        }
        __syncthreads();
        // the state's walk over the group: no barrier, no exchange; a thread leaves its part of every row's output
#pragma unroll 4
        for (int tt = 0; tt < nt; ++tt) {
            float q[RPT], k[RPT], w[RPT];
            load_run<RPT>(sq + (size_t)tt * Dp + i0, q);
            load_run<RPT>(sk + (size_t)tt * Dp + i0, k);
            if (CH) load_run<RPT>(sw + (size_t)tt * Dp + i0, w);
            const float vj = sv[tt * cols + c];
            const float af = MODE == 1 ? sg[4 * tt] : w_head, bv = MODE == 1 ? sg[4 * tt + 1] * vj : vj;
            float acc = 0.f;
#pragma unroll
            for (int it = 0; it < RPT; ++it) {
                const float x = k[it] * bv;
                if (MODE == 0) {
                    acc = fmaf(fmaf(U[it], x, S[it]), q[it], acc);
                    S[it] = fmaf(w[it], S[it], x);
                } else {
                    S[it] = fmaf(MODE == 3 ? w[it] : af, S[it], x);
                    acc = fmaf(S[it], q[it], acc);
                }
            }
            part[((size_t)tt * KS + ks) * cols + c] = acc;
        }
        __syncthreads();
        // a column's parts are added in index order; the matrix memory divides by its normaliser
        for (int e = threadIdx.x; e < nt * real; e += SCAN_THREADS) {
            const int tt = e / real, cc = e - tt * real;
            if (cc >= n_cols) continue;
            float o = 0.f;
            for (int x = 0; x < KS; ++x) o += part[((size_t)tt * KS + x) * cols + cc];
            if (MODE == 1) {
                float dot = 0.f;
                for (int x = 0; x < KS; ++x) dot += part[((size_t)tt * KS + x) * cols + real];
                o /= fmaxf(fabsf(dot), sg[4 * tt + 2]) + 1e-6f;
            }
            R[(t0 + tt) * ldr + cc] = o;
        }
    }
#pragma unroll
    for (int it = 0; it < RPT; ++it) {
        const int i = i0 + it;
        if (i < D) {
            if (is_n) {
                if (cb == 0) st[(long long)D * DV + i] = S[it];
            } else if (active) {
                st[(long long)i * DV + j] = S[it];
            }
        }
    }
    if (MODE == 1) {
        if (cb == 0 && threadIdx.x == 0) st[(long long)D * DV + D] = m;
    } else if (MODE == 0 && hd == 0 && cb == 0 && a.shift_src) {
        const T* last = (const T*)a.shift_src + (long long)(s1 - 1) * a.W;
        float* keep = a.state + (long long)a.seq_slot[b] * a.state_stride;
        for (int e = threadIdx.x; e < a.W; e += SCAN_THREADS) keep[e] = to_f32(last[e]);
    }
}

// out[t][head] = T(raw / rms(raw over the head's columns) * norm_w * act(g)); act = silu (MODE 0) or sigmoid (MODE 1).
// One warp per (row, head).  Rows of padding hold whatever `raw` held; nothing reads them.
template <typename T, int MODE>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const ScanArgs a) {
    pdl_trigger();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (idx >= a.rows * a.H) return;
    const long long t = idx / a.H;
    const int hd = (int)(idx - t * a.H), lane = threadIdx.x & 31, DV = a.DV;
    const float* r = a.raw + t * ((long long)a.H * DV) + (long long)hd * DV;
    float ss = 0.f;
    for (int c = lane; c < DV; c += 32) ss = fmaf(r[c], r[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)DV + a.eps);
    const T* G = (const T*)a.g + t * a.ldg + (long long)hd * DV;
    T* O = (T*)a.out + t * a.ldo + (long long)hd * DV;
    for (int c = lane; c < DV; c += 32) {
        const float gz = to_f32(G[c]);
        const float act = MODE == 0 ? gz * sigmoid_f32(gz) : sigmoid_f32(gz);
        O[c] = from_f32<T>(((r[c] * inv) * a.norm_w[hd * DV + c]) * act);
    }
}

// The unit norm, channel weights and gate over `raw` (see head_norm_gate_kernel): act 0 silu, 1 sigmoid.
int cm_scan_norm_gate(int dt, int act, const ScanArgs& a, cudaStream_t st) {
    ScanArgs n = a;
    if (a.norm_all_heads) {                      // the norm over all heads of a row together is the norm of one head that spans the row
        n.DV = a.H * a.DV;
        n.H = 1;
    }
    dim3 egrid((unsigned)((n.rows * n.H + 3) / 4));
    if (dt == DT_F32 && act == 0) cm_launch(head_norm_gate_kernel<float, 0>, egrid, 128, 0, st, n);
    else if (dt == DT_F32) cm_launch(head_norm_gate_kernel<float, 1>, egrid, 128, 0, st, n);
    else if (dt == DT_BF16 && act == 0) cm_launch(head_norm_gate_kernel<bf16, 0>, egrid, 128, 0, st, n);
    else if (dt == DT_BF16) cm_launch(head_norm_gate_kernel<bf16, 1>, egrid, 128, 0, st, n);
    else return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// mode 0: decay mix, mode 1: matrix memory, mode 2: constant decay per head.  B sequences; rows of the step are found
// through seq_start.
extern "C" int cm_matrix_scan(int dt, int mode, const ScanArgs* args, int B, cudaStream_t st) {
    ScanArgs a = *args;
    if (B <= 0 || a.rows <= 0) return CM_OK;
    if (a.D <= 0 || a.DV <= 0 || a.D > 1024) CM_REFUSE("matrix_scan: head sizes %d x %d (keys up to 1024)", a.D, a.DV);
    if (!a.raw) CM_REFUSE("matrix_scan: the float buffer for the heads' raw outputs is missing");
    if (mode < 0 || mode > 3) CM_REFUSE("matrix_scan: mode %d", mode);
    // Channels per thread (a power of two from 2 to 32) and parts per column (a power of two up to 32): as many
    // channels as leave the grid with a block per SM.  The walk is bound by its latency per row, not by arithmetic,
    // so what counts is how many SMs walk at once (measured on B200, 2,048 rows, one sequence, 8 heads of 64 x 128 /
    // 16 heads of 64 x 64, us at 2 / 4 / 8 / 16 / 32 channels: 541 / 407 / 619 / 959 / 1255 and 293 / 331 / 509 / 769 / 1229).
    auto parts_for = [&](int r) { int k = 1; while (k * r < a.D) k *= 2; return k; };
    auto blocks = [&](int k) {
        const int real = SCAN_THREADS / k - (mode == 1 ? 1 : 0);
        return real < 1 ? 0LL : (long long)a.H * ((a.DV + real - 1) / real) * B;
    };
    int rpt = 32;
    while (rpt > 2 && parts_for(rpt / 2) <= 32 && blocks(parts_for(rpt)) < 148) rpt /= 2;
    // ... and, while a thread still has more than four channels, with nearly two: several sequences in a step give the
    // schedulers warps to choose from (2,048 rows as 4 / 8 sequences, matrix memory: 288 -> 197 and 203 -> 187 us)
    while (rpt > 4 && parts_for(rpt / 2) <= 32 && blocks(parts_for(rpt)) < 256) rpt /= 2;
    const int ks = parts_for(rpt);
    if (ks > 32) CM_REFUSE("matrix_scan: heads of %d key channels (up to 1024)", a.D);
    a.KS = ks;
    const int cols = SCAN_THREADS / ks, real = cols - (mode == 1 ? 1 : 0);
    const int row_floats = (mode == 0 || mode == 3 ? 3 : 2) * ks * rpt + cols + 4 + SCAN_THREADS;
    int tb = 12288 / row_floats;                          // about 48 KB of staged rows
    tb = tb < 1 ? 1 : (tb > SCAN_MAX_ROWS ? SCAN_MAX_ROWS : tb);
    const size_t smem = (size_t)tb * row_floats * sizeof(float);
    dim3 grid(a.H, (a.DV + real - 1) / real, B);
    // the norm over all heads of a row together is the norm of one head that spans the row
    ScanArgs n = a;
    if (a.norm_all_heads) {
        n.DV = a.H * a.DV;
        n.H = 1;
    }
    dim3 egrid((unsigned)((n.rows * n.H + 3) / 4));
#define SCAN_LAUNCH(TT, M, R)                                                                                    \
    do {                                                                                                         \
        if (smem > 48 * 1024)                                                                                    \
            cudaFuncSetAttribute(matrix_scan_kernel<TT, M, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        cm_launch(matrix_scan_kernel<TT, M, R>, grid, SCAN_THREADS, smem, st, a, tb);                                \
    } while (0)
#define SCAN_RPT(TT, M)                             \
    do {                                            \
        if (rpt == 2) SCAN_LAUNCH(TT, M, 2);        \
        else if (rpt == 4) SCAN_LAUNCH(TT, M, 4);   \
        else if (rpt == 8) SCAN_LAUNCH(TT, M, 8);   \
        else if (rpt == 16) SCAN_LAUNCH(TT, M, 16); \
        else SCAN_LAUNCH(TT, M, 32);                \
    } while (0)
    if (dt == DT_F32 && mode == 0) { SCAN_RPT(float, 0); CM_CHECK_LAUNCH(); cm_launch(head_norm_gate_kernel<float, 0>, egrid, 128, 0, st, n); }
    else if (dt == DT_F32 && mode == 1) { SCAN_RPT(float, 1); CM_CHECK_LAUNCH(); cm_launch(head_norm_gate_kernel<float, 1>, egrid, 128, 0, st, n); }
    else if (dt == DT_BF16 && mode == 0) { SCAN_RPT(bf16, 0); CM_CHECK_LAUNCH(); cm_launch(head_norm_gate_kernel<bf16, 0>, egrid, 128, 0, st, n); }
    else if (dt == DT_BF16 && mode == 1) { SCAN_RPT(bf16, 1); CM_CHECK_LAUNCH(); cm_launch(head_norm_gate_kernel<bf16, 1>, egrid, 128, 0, st, n); }
    else if (dt == DT_F32 && mode == 2) { SCAN_RPT(float, 2); CM_CHECK_LAUNCH(); cm_launch(head_norm_gate_kernel<float, 1>, egrid, 128, 0, st, n); }
    else if (dt == DT_BF16 && mode == 2) { SCAN_RPT(bf16, 2); CM_CHECK_LAUNCH(); cm_launch(head_norm_gate_kernel<bf16, 1>, egrid, 128, 0, st, n); }
    else if (dt == DT_F32 && mode == 3) { SCAN_RPT(float, 3); CM_CHECK_LAUNCH(); cm_launch(head_norm_gate_kernel<float, 0>, egrid, 128, 0, st, n); }
    else if (dt == DT_BF16 && mode == 3) { SCAN_RPT(bf16, 3); CM_CHECK_LAUNCH(); cm_launch(head_norm_gate_kernel<bf16, 0>, egrid, 128, 0, st, n); }
    else return CM_ERR_DTYPE;
#undef SCAN_RPT
#undef SCAN_LAUNCH
    CM_CHECK_LAUNCH();
    return CM_OK;
}
