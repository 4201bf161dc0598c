// Row-wise kernels for models whose residual stream is kept in float whatever the activation type:
// a norm that reads float rows and writes activations, the residual sum of several terms fused with
// the norm of whatever runs next, and the concatenation [x; x0] that a looped stack feeds to the
// projection at the start of a pass.
//
// The norm is a root-mean-square norm (kind 0) or a dynamic tanh (kind 1: y = tanh(alpha x) * w + b, which takes
// no statistics of the row; alpha is read from the device).
//
// A row is held in shared memory between the two passes over it (sum of squares, then scaling), so the
// width is bounded by shared memory only.  All sums are float and run in a fixed order.
#include "common.cuh"

#define R32_THREADS 256
#define R32_MAX_TERMS 4

// One term of a residual sum: rows of `per_row` consecutive pieces each (a routed feed-forward leaves
// one piece per chosen expert), stored as float or as activations, times a constant.
struct ResidualTerm {
    const void* p;
    const int* index;      // null: piece j of row r is row r * per_row + j; else row index[r * per_row + j] (negative: none)
    const float* weights;  // null, or a factor per piece: weights[r * per_row + j] (a routed feed-forward's weights on its experts' outputs)
    float scale;
    int per_row;
    int is_f32;
};
struct ResidualTerms {
    ResidualTerm t[R32_MAX_TERMS];
    int n;
};

template <typename T>
__device__ __forceinline__ float term_at(const ResidualTerm& t, long long i) {
    return t.is_f32 ? reinterpret_cast<const float*>(t.p)[i] : to_f32(reinterpret_cast<const T*>(t.p)[i]);
}

#define NORM_RMS 0
#define NORM_DYT 1

// y = T((x * inv) * w), inv = 1 / sqrt(mean(x^2) + eps); or T(tanh(alpha x) * w + b); x float.
template <typename T>
__global__ void __launch_bounds__(R32_THREADS)
norm_f32in_kernel(T* __restrict__ y, const float* __restrict__ x, const float* __restrict__ w, int H, float eps,
                  int kind, const float* __restrict__ alpha, const float* __restrict__ shift) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const float* xr = x + (long long)blockIdx.x * H;
    if (kind == NORM_DYT) {
        const float al = alpha[0];
        T* yd = y + (long long)blockIdx.x * H;
        for (int c = threadIdx.x; c < H; c += R32_THREADS) yd[c] = from_f32<T>(fmaf(tanhf(al * xr[c]), w[c], shift[c]));
        return;
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += R32_THREADS) {
        const float v = xr[c];
        row[c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
    T* yr = y + (long long)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += R32_THREADS) yr[c] = from_f32<T>((row[c] * inv) * w[c]);
}

// sum_i scale_i * sum_j (weights_i[j]) term_i[row * per_row_i + j] at column c: the terms are added to each other in their order.
template <typename T>
__device__ __forceinline__ float terms_at(const ResidualTerms& terms, long long r, int H, int c) {
    float add = 0.f;
    for (int i = 0; i < terms.n; ++i) {
        const ResidualTerm& t = terms.t[i];
        float s = 0.f;
        for (int j = 0; j < t.per_row; ++j) {
            const long long piece = t.index ? t.index[r * t.per_row + j] : r * t.per_row + j;
            if (piece >= 0) {
                const float v = term_at<T>(t, piece * H + c);
                s = t.weights ? fmaf(t.weights[r * t.per_row + j], v, s) : s + v;
            }
        }
        add += t.scale * s;
    }
    return add;
}

// h += sum_i scale_i * sum_j term_i[row * per_row_i + j] (+ bias);  n = T(norm(h) * w) when n is given.
// The terms are added to each other first, in their order, and their sum to h: x + (mixer + feed-forward).
template <typename T>
__global__ void __launch_bounds__(R32_THREADS)
residual_add_norm_kernel(float* __restrict__ h, T* __restrict__ n_out, ResidualTerms terms,
                         const float* __restrict__ bias, const float* __restrict__ w, int H, float eps,
                         int kind, const float* __restrict__ alpha, const float* __restrict__ shift) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const long long r = blockIdx.x;
    float* hr = h + r * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += R32_THREADS) {
        float v = hr[c] + terms_at<T>(terms, r, H, c);
        if (bias) v += bias[c];
        hr[c] = v;
        row[c] = v;
        ss += v * v;
    }
    if (!n_out) return;
    T* nr = n_out + r * H;
    if (kind == NORM_DYT) {                          // every thread reads back what it stored itself
        const float al = alpha[0];
        for (int c = threadIdx.x; c < H; c += R32_THREADS) nr[c] = from_f32<T>(fmaf(tanhf(al * row[c]), w[c], shift[c]));
        return;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += R32_THREADS) nr[c] = from_f32<T>((row[c] * inv) * w[c]);
}

// The norm behind the sum (a post-norm layer), optionally followed by an average over the depth of the stack:
//   x = norm(h_scale * h + terms) * w
//   without `hist`:  h <- x
//   with `hist` [n_hist][rows][H] (entry j at hist + j * hist_stride): entry n_hist - 1 <- x, and
//                    h <- sum over j < n_hist of coef[j] * entry j          (j ascending; the last entry is x itself)
//   n_out <- T(h) when given: the rows as the next reader's products take them.
template <typename T>
__global__ void __launch_bounds__(R32_THREADS)
postnorm_residual_kernel(float* __restrict__ h, T* __restrict__ n_out, ResidualTerms terms, float h_scale,
                         const float* __restrict__ w, int H, float eps, float* __restrict__ hist, long long hist_stride,
                         int n_hist, const float* __restrict__ coef) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const long long r = blockIdx.x;
    float* hr = h + r * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += R32_THREADS) {
        const float v = fmaf(h_scale, hr[c], terms_at<T>(terms, r, H, c));
        row[c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += R32_THREADS) {     // every thread reads back what it stored itself
        float x = (row[c] * inv) * w[c];
        if (hist) {
            hist[(long long)(n_hist - 1) * hist_stride + r * H + c] = x;
            float mix = 0.f;
            for (int j = 0; j + 1 < n_hist; ++j) mix = fmaf(coef[j], hist[(long long)j * hist_stride + r * H + c], mix);
            x = fmaf(coef[n_hist - 1], x, mix);
        }
        hr[c] = x;
        if (n_out) n_out[r * H + c] = from_f32<T>(x);
    }
}

// out[r] = T([a[r]; b[r]]) for float rows a and b of width H: the input of a projection over both.
template <typename T>
__global__ void concat_cast_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b,
                                   long long rows, int H) {
    pdl_trigger();
    pdl_wait();
    const long long total = rows * 2 * H;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / (2 * H);
        const int c = (int)(i - r * 2 * H);
        out[i] = from_f32<T>(c < H ? a[r * H + c] : b[r * H + c - H]);
    }
}

static int row_smem(int H, size_t* out) {
    *out = (size_t)H * sizeof(float);
    if (*out > 200 * 1024) CM_REFUSE("a row of %d floats does not fit shared memory", H);
    return CM_OK;
}

extern "C" int cm_norm_f32in(int dt, void* y, const float* x, const float* w, int rows, int H, float eps,
                             int kind, const float* alpha, const float* shift, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    if (kind == NORM_DYT && (!alpha || !shift)) CM_REFUSE("norm_f32in: a dynamic tanh needs its alpha and its shift");
    size_t smem;
    if (row_smem(H, &smem) != CM_OK) return CM_ERR_SHAPE;
    if (dt == DT_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(norm_f32in_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cm_launch(norm_f32in_kernel<float>, rows, R32_THREADS, smem, st, (float*)y, x, w, H, eps, kind, alpha, shift);
    } else if (dt == DT_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(norm_f32in_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cm_launch(norm_f32in_kernel<bf16>, rows, R32_THREADS, smem, st, (bf16*)y, x, w, H, eps, kind, alpha, shift);
    } else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

static void fill_terms(ResidualTerms& terms, int n_terms, const void* const* term_ptr, const float* term_scale,
                       const int* term_per_row, const int* term_is_f32, const int* const* term_index,
                       const float* const* term_weights) {
    terms.n = n_terms;
    for (int i = 0; i < R32_MAX_TERMS; ++i) {
        terms.t[i].p = i < n_terms ? term_ptr[i] : nullptr;
        terms.t[i].index = i < n_terms ? term_index[i] : nullptr;
        terms.t[i].weights = i < n_terms ? term_weights[i] : nullptr;
        terms.t[i].scale = i < n_terms ? term_scale[i] : 0.f;
        terms.t[i].per_row = i < n_terms ? term_per_row[i] : 0;
        terms.t[i].is_f32 = i < n_terms ? term_is_f32[i] : 0;
    }
}

// terms: n_terms entries of (pointer, scale, pieces per row, stored as float?, index of the pieces or null, a weight per
// piece or null) in parallel arrays.
extern "C" int cm_residual_add_norm(int dt, float* h, void* n_out, int n_terms, const void* const* term_ptr,
                                    const float* term_scale, const int* term_per_row, const int* term_is_f32,
                                    const int* const* term_index, const float* const* term_weights, const float* bias,
                                    const float* w, int rows, int H, float eps, int kind, const float* alpha,
                                    const float* shift, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    if (n_terms < 0 || n_terms > R32_MAX_TERMS) CM_REFUSE("residual_add_norm: %d terms (at most %d)", n_terms, R32_MAX_TERMS);
    if (n_out && !w) CM_REFUSE("residual_add_norm: a norm needs its weight");
    if (n_out && kind == NORM_DYT && (!alpha || !shift)) CM_REFUSE("residual_add_norm: a dynamic tanh needs its alpha and its shift");
    size_t smem;
    if (row_smem(H, &smem) != CM_OK) return CM_ERR_SHAPE;
    ResidualTerms terms;
    fill_terms(terms, n_terms, term_ptr, term_scale, term_per_row, term_is_f32, term_index, term_weights);
    if (dt == DT_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(residual_add_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cm_launch(residual_add_norm_kernel<float>, rows, R32_THREADS, smem, st, h, (float*)n_out, terms, bias, w, H, eps, kind, alpha, shift);
    } else if (dt == DT_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(residual_add_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cm_launch(residual_add_norm_kernel<bf16>, rows, R32_THREADS, smem, st, h, (bf16*)n_out, terms, bias, w, H, eps, kind, alpha, shift);
    } else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

// The post-norm sum (postnorm_residual_kernel); terms as for cm_residual_add_norm.  coef: n_hist floats on the device.
extern "C" int cm_postnorm_residual(int dt, float* h, void* n_out, int n_terms, const void* const* term_ptr,
                                    const float* term_scale, const int* term_per_row, const int* term_is_f32,
                                    const int* const* term_index, const float* const* term_weights, float h_scale,
                                    const float* w, int rows, int H, float eps, float* hist, long long hist_stride,
                                    int n_hist, const float* coef, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    if (n_terms < 0 || n_terms > R32_MAX_TERMS) CM_REFUSE("postnorm_residual: %d terms (at most %d)", n_terms, R32_MAX_TERMS);
    if (!w) CM_REFUSE("postnorm_residual: the norm needs its weight");
    if (hist && (n_hist < 1 || !coef)) CM_REFUSE("postnorm_residual: an average over %d entries needs its coefficients", n_hist);
    size_t smem;
    if (row_smem(H, &smem) != CM_OK) return CM_ERR_SHAPE;
    ResidualTerms terms;
    fill_terms(terms, n_terms, term_ptr, term_scale, term_per_row, term_is_f32, term_index, term_weights);
    if (dt == DT_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(postnorm_residual_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cm_launch(postnorm_residual_kernel<float>, rows, R32_THREADS, smem, st, h, (float*)n_out, terms, h_scale, w, H, eps, hist,
                  hist_stride, n_hist, coef);
    } else if (dt == DT_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(postnorm_residual_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cm_launch(postnorm_residual_kernel<bf16>, rows, R32_THREADS, smem, st, h, (bf16*)n_out, terms, h_scale, w, H, eps, hist,
                  hist_stride, n_hist, coef);
    } else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}

extern "C" int cm_concat_cast(int dt, void* out, const float* a, const float* b, long long rows, int H, cudaStream_t st) {
    if (rows <= 0) return CM_OK;
    const long long total = rows * 2 * H;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dt == DT_F32)
        cm_launch(concat_cast_kernel<float>, blocks, 256, 0, st, (float*)out, a, b, rows, H);
    else if (dt == DT_BF16)
        cm_launch(concat_cast_kernel<bf16>, blocks, 256, 0, st, (bf16*)out, a, b, rows, H);
    else
        return CM_ERR_DTYPE;
    CM_CHECK_LAUNCH();
    return CM_OK;
}
