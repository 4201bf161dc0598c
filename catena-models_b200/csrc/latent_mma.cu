// The latent attention of single-token steps on the tensor cores (bfloat16 caches): mma.sync m16n8k16 for the scores of
// 16 heads against a tile of cache entries and for the weights' product with the same entries' latents.
//
// All heads of a sequence meet the same entries, so the heads are the rows of the products: one block = one sequence,
// one run of keys (a split) and 16 heads.  A tile is LM_KT = 32 entries, copied whole (cp.async) into shared memory
// rows padded by 16 bytes; the next tile is copied into a second buffer while the present one is multiplied.  Each of
// the four warps forms the scores of the 16 heads against eight of the tile's keys over all E = KR + R channels and
// leaves them in shared memory; then every warp takes the whole tile's scores [16 x LM_KT], masks, keeps the running
// maximum and sum in float (each warp for itself: the same numbers in all four), and adds
// P [16 x LM_KT] x latents [LM_KT x its own quarter of the KR channels] to its output tile in registers.  The queries
// come as float rows [W_uk^T q_plain | q_turn] and are rounded to bfloat16 on their way into shared memory; the scale
// multiplies the float scores.  Splits leave (maximum, sum, unnormalised sums) as the CUDA-core form does, and the same
// merge kernel finishes them.
#include "common.cuh"
#include "latent.h"
#include <math.h>

#define LM_KT 32
#define LM_THREADS 128
#define LM_PAD 8
#define LM_LDS (LM_KT + 8)                     // pitch (floats) of the tile's scores in shared memory

__device__ __forceinline__ void lm_copy16(void* dst, const void* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;                 // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void lm_copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void lm_copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void lm_ldsm_x4(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lm_ldsm_x4_trans(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lm_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float lm_exp2(float x) {          // -inf gives 0, as the masks need
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t lm_pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// The pitches (elements) of a query row and of an entry in shared memory.  EP: the channels the score products walk
// (E up to a multiple of 32; what lies behind E is zeros on both sides); an entry's row also covers the 4 * NT * 8
// channels that the warps' output tiles span.  Both are odd multiples of 16 bytes: ldmatrix meets no bank twice.
static inline int lm_ep(int E) { return (E + 31) & ~31; }
static inline int lm_ldk(int E, int nt) { return max(lm_ep(E), 4 * nt * 8) + LM_PAD; }

// NT: output tiles of 8 channels per warp (4 warps x NT x 8 >= KR).
template <int NT>
__global__ void __launch_bounds__(LM_THREADS)
latent_attn_mma_kernel(const LatentArgs a) {
    extern __shared__ __align__(16) unsigned char lm_smem[];
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.z, split = blockIdx.y, hg = blockIdx.x;
    const int H = a.H, E = a.E, KR = a.KR, EC = a.EC;
    const int EP = (E + 31) & ~31, LDQ = EP + LM_PAD, LDK = max(EP, 4 * NT * 8) + LM_PAD;
    bf16* Qs = reinterpret_cast<bf16*>(lm_smem);          // [16][LDQ]
    bf16* Ks = Qs + 16 * LDQ;                             // [2][LM_KT][LDK]
    float* Ss = reinterpret_cast<float*>(Ks + 2 * LM_KT * LDK);      // [16][LM_LDS]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const long long t = a.seq_start[b];                   // the sequence's one row of the step
    const int pos = a.seq_pos0[b], end = a.seq_end[b];
    // the 16 heads' queries, rounded; zeros for heads past H and channels past E (eight threads a head)
    {
        const int m = tid >> 3, h = hg * 16 + m;
        const float* src = a.qa + t * a.ldqa + (long long)h * E;
        for (int c = tid & 7; c < LDQ; c += 8) Qs[m * LDQ + c] = __float2bfloat16_rn((h < H && c < E) ? src[c] : 0.f);
    }
    // what no copy writes (channels from EC on) is zeros once and for all
    for (int e = tid; e < 2 * LM_KT * (LDK - EC); e += LM_THREADS) {
        const int j = e / (LDK - EC), c = EC + e - j * (LDK - EC);
        Ks[j * LDK + c] = __float2bfloat16_rn(0.f);
    }
    const int k_first = a.splits > 1 ? split * a.chunk : 0;
    const int k_last = min(pos, a.splits > 1 ? k_first + a.chunk - 1 : 0x7fffffff);        // inclusive
    const float scale_log2 = a.scale * 1.4426950408889634f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
    const int* ptab = a.ptab + (long long)a.seq_slot[b] * a.ptab_stride;
    const int C8 = EC >> 3;
    const int ch0 = warp * NT * 8;                        // the warp's first output channel
    // A tile's entries into buffer `buf`, 16 bytes a copy, four threads an entry; entries at or behind the sequence's end
    // become zeros.  A tile starts at a multiple of LM_KT and so lies within one page: its page index is read from the
    // table a round ahead, and no copy waits for a load.
    static_assert(PAGE_TOKENS % LM_KT == 0 && LM_THREADS == 4 * LM_KT, "a tile within a page, four threads an entry");
    auto fetch = [&](int k0, int buf, int page) {
        const int j = tid >> 2, kp = k0 + j;
        const bool valid = kp < end && kp <= k_last;
        const bf16* src = (const bf16*)a.pool + (valid ? ((long long)page * PAGE_TOKENS + kp % PAGE_TOKENS) * EC : 0);
        bf16* dst = Ks + (buf * LM_KT + j) * LDK;
        for (int c8 = tid & 3; c8 < C8; c8 += 4) lm_copy16(dst + c8 * 8, src + (valid ? c8 * 8 : 0), valid);
        lm_copy_commit();
    };
    const bool any = k_first <= k_last;
    int page_next = 0;
    if (any) {
        fetch(k_first, 0, ptab[k_first / PAGE_TOKENS]);
        if (k_first + LM_KT <= k_last) page_next = ptab[(k_first + LM_KT) / PAGE_TOKENS];
    }
    int buf = 0;
    for (int k0 = k_first; k0 <= k_last; k0 += LM_KT, buf ^= 1) {
        // the other buffer's tile was multiplied before the barrier that ended the round before this one
        const bool more = k0 + LM_KT <= k_last;
        if (more) {
            fetch(k0 + LM_KT, buf ^ 1, page_next);
            if (k0 + 2 * LM_KT <= k_last) page_next = ptab[(k0 + 2 * LM_KT) / PAGE_TOKENS];
        }
        if (more) lm_copy_wait<1>(); else lm_copy_wait<0>();
        __syncthreads();                                  // every thread's copies of this tile (and the queries) are in place
        const bf16* Kt = Ks + buf * LM_KT * LDK;
        // ---- scores of the 16 heads against the warp's eight keys of the tile, over all channels; two steps of 16
        //      channels a matrix load of the keys
        {
            float sw[4] = {0.f, 0.f, 0.f, 0.f};
            for (int kk = 0; kk < EP / 32; ++kk) {
                uint32_t kb[4], qf[4];
                lm_ldsm_x4(kb, Kt + (warp * 8 + (lane & 7)) * LDK + kk * 32 + 8 * (lane >> 3));
                lm_ldsm_x4(qf, Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDQ + kk * 32 + 8 * (lane >> 4));
                lm_mma(sw, qf, kb[0], kb[1]);
                lm_ldsm_x4(qf, Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDQ + kk * 32 + 16 + 8 * (lane >> 4));
                lm_mma(sw, qf, kb[2], kb[3]);
            }
            *reinterpret_cast<float2*>(Ss + g * LM_LDS + warp * 8 + 2 * t4) = make_float2(sw[0], sw[1]);
            *reinterpret_cast<float2*>(Ss + (g + 8) * LM_LDS + warp * 8 + 2 * t4) = make_float2(sw[2], sw[3]);
        }
        __syncthreads();
        // every warp takes all of the tile's scores, laid out as the products leave them
        float s[LM_KT / 8][4];
#pragma unroll
        for (int j = 0; j < LM_KT / 8; ++j) {
            const float2 lo = *reinterpret_cast<const float2*>(Ss + g * LM_LDS + j * 8 + 2 * t4);
            const float2 hi = *reinterpret_cast<const float2*>(Ss + (g + 8) * LM_LDS + j * 8 + 2 * t4);
            s[j][0] = lo.x; s[j][1] = lo.y; s[j][2] = hi.x; s[j][3] = hi.y;
        }
        // ---- mask (every head stands at the same position), running maximum
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < LM_KT / 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = k0 + 8 * j + 2 * t4 + (i & 1);
                s[j][i] = key <= k_last ? s[j][i] : -INFINITY;
                mx[i >> 1] = fmaxf(mx[i >> 1], s[j][i]);
            }
        float alpha[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h] * scale_log2);      // scale > 0: the order of scores is kept
            m_use[h] = m_new == -INFINITY ? 0.f : m_new;
            alpha[h] = lm_exp2(m_run[h] - m_use[h]);
            m_run[h] = m_new;
        }
        float rs[2] = {0.f, 0.f};
        uint32_t pf[LM_KT / 16][4];                       // P as the A operand, steps of 16 keys
#pragma unroll
        for (int j = 0; j < LM_KT / 8; ++j) {
            const float p0 = lm_exp2(fmaf(s[j][0], scale_log2, -m_use[0])), p1 = lm_exp2(fmaf(s[j][1], scale_log2, -m_use[0]));
            const float p2 = lm_exp2(fmaf(s[j][2], scale_log2, -m_use[1])), p3 = lm_exp2(fmaf(s[j][3], scale_log2, -m_use[1]));
            rs[0] += p0 + p1;
            rs[1] += p2 + p3;
            pf[j >> 1][(j & 1) * 2] = lm_pack(p0, p1);       // rows g
            pf[j >> 1][(j & 1) * 2 + 1] = lm_pack(p2, p3);   // rows g + 8
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + rs[h];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            o[j][0] *= alpha[0];
            o[j][1] *= alpha[0];
            o[j][2] *= alpha[1];
            o[j][3] *= alpha[1];
        }
        // ---- the warp's channels of P x latents
#pragma unroll
        for (int kk = 0; kk < LM_KT / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < NT / 2; ++dp) {         // channel tiles 2dp, 2dp + 1
                uint32_t vb[4];
                lm_ldsm_x4_trans(vb, Kt + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDK + ch0 + dp * 16 + 8 * (lane >> 4));
                lm_mma(o[2 * dp], pf[kk], vb[0], vb[1]);
                lm_mma(o[2 * dp + 1], pf[kk], vb[2], vb[3]);
            }
        }
        __syncthreads();                                  // this buffer is refilled in the next round
    }
    // ---- the rows' sums over the quad, then parts or the finished rows
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int h = hg * 16 + g + 8 * half;
        if (h >= H) continue;
        if (a.splits > 1) {
            float* part = a.parts + ((t * H + h) * a.splits + split) * (2 + KR);
            if (warp == 0 && t4 == 0) {
                part[0] = m_run[half] * 0.6931471805599453f;      // the maximum as a natural exponent, as the merge takes it
                part[1] = l_run[half];
            }
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int c = ch0 + 8 * j + 2 * t4 + i;
                    if (c < KR) part[2 + c] = o[j][2 * half + i];
                }
        } else {
            const float gt = a.gate ? sigmoid_f32(to_f32(((const bf16*)a.gate)[t * a.ld_gate + h])) : 1.f;
            const float f = gt / l_run[half];
            float* out = a.out + t * a.ldo + (long long)h * KR;
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int c = ch0 + 8 * j + 2 * t4 + i;
                    if (c < KR) out[c] = o[j][2 * half + i] * f;
                }
        }
    }
}

// A step in which every sequence brings one token (rows = B, row b of sequence b at seq_start[b]); bfloat16 cache.
extern "C" int cm_latent_attn_mma(const LatentArgs* args, cudaStream_t st) {
    const LatentArgs& a = *args;
    if (a.rows <= 0 || a.B <= 0) return CM_OK;
    if (a.E != a.KR + a.R || a.KR < 1 || a.KR > 512 || a.EC % 8 || a.EC < a.E || ((uintptr_t)a.pool & 15))
        CM_REFUSE("latent_attn_mma: latents of %d channels (up to 512) in entries of %d (a multiple of 8, 16-byte aligned)", a.KR, a.EC);
    if (a.splits < 1 || (a.splits > 1 && (!a.parts || a.chunk < LM_KT || a.chunk % LM_KT)))
        CM_REFUSE("latent_attn_mma: %d splits of %d keys", a.splits, a.chunk);
    const int nt = a.KR <= 128 ? 4 : (a.KR <= 256 ? 8 : 16);
    const size_t smem = (size_t)(16 * (lm_ep(a.E) + LM_PAD) + 2 * LM_KT * lm_ldk(a.E, nt)) * sizeof(bf16) + 16 * LM_LDS * sizeof(float);
    dim3 grid((unsigned)((a.H + 15) / 16), a.splits, a.B);
#define LM_LAUNCH(N)                                                                                               \
    do {                                                                                                           \
        if (smem > 48 * 1024)                                                                                      \
            cudaFuncSetAttribute(latent_attn_mma_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        cm_launch(latent_attn_mma_kernel<N>, grid, LM_THREADS, smem, st, a);                                       \
    } while (0)
    if (nt == 4) LM_LAUNCH(4); else if (nt == 8) LM_LAUNCH(8); else LM_LAUNCH(16);
#undef LM_LAUNCH
    CM_CHECK_LAUNCH();
    if (a.splits > 1) return cm_latent_attn_merge(DT_BF16, args, st);
    return CM_OK;
}
