// Layer norm (a weight, and a bias where the caller has one) over rows of the 32-bit residual stream, and the form
// that a block with norms on both sides of its sublayers needs: the sublayer's output is normed, added to the residual stream, and the new row is
// normed again for the sublayer that follows, in one pass over the row.
//
//   ln(z)[i] = (z[i] - mean(z)) / sqrt(mean((z - mean(z))^2) + eps) * w[i]
//
// All statistics are 32-bit, mean first and then the squared deviations (two passes: a difference of large sums
// would lose the small variances of a normed stream).  One block per row; a thread touches the same elements in
// every pass, so that a row may be normed in place and the second norm may read the row the first pass wrote.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int LN_THREADS = 1024;   // at most; see ln_threads

struct RowStats { float mean, rstd; };

template <typename F>
__device__ __forceinline__ RowStats row_stats(F value, int n, float eps, float* scratch)
{
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += value(i);
    const float mean = block_sum(s, scratch) / (float)n;
    float d2 = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float d = value(i) - mean; d2 = fmaf(d, d, d2); }
    const float var = block_sum(d2, scratch) / (float)n;
    return {mean, 1.0f / sqrtf(var + eps)};
}

template <typename OT>
__global__ void __launch_bounds__(LN_THREADS) layernorm_kernel(
    const float* x, const int* __restrict__ rows, const void* __restrict__ w, int w_dtype,
    const void* __restrict__ bias, int b_dtype, float eps, OT* out, int hidden)
{
    __shared__ float scratch[33];
    fx_pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (long)(rows ? rows[r] : r) * hidden;
    const RowStats st = row_stats([&](int i) { return xr[i]; }, hidden, eps, scratch);
    OT* o = out + (long)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = (xr[i] - st.mean) * st.rstd * load_any(w, w_dtype, i);
        if (bias) v += load_any(bias, b_dtype, i);
        o[i] = from_f32<OT>(v);
    }
}

// z = s1 * y1 (+ s2 * y2);  h += ln(z) * w_post;  x_out = ln(h) * w_next (if asked for).
template <typename OT>
__global__ void __launch_bounds__(LN_THREADS) layernorm_residual_kernel(
    float* h, const void* __restrict__ y1, int y1_dtype, float s1, const void* __restrict__ y2,
    int y2_dtype, float s2, const void* __restrict__ w_post, int wp_dtype, float eps, const void* __restrict__ w_next,
    int wn_dtype, float eps_next, OT* __restrict__ x_out, int hidden)
{
    __shared__ float scratch[33];
    fx_pdl_wait();
    const long base = (long)blockIdx.x * hidden;
    auto z = [&](int i) {
        float v = s1 * load_any(y1, y1_dtype, base + i);
        if (y2) v = fmaf(s2, load_any(y2, y2_dtype, base + i), v);
        return v;
    };
    const RowStats st = row_stats(z, hidden, eps, scratch);
    float* hr = h + base;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        hr[i] = hr[i] + (z(i) - st.mean) * st.rstd * load_any(w_post, wp_dtype, i);
    if (!w_next) return;
    // the same thread wrote hr[i] that reads it here
    const RowStats sn = row_stats([&](int i) { return hr[i]; }, hidden, eps_next, scratch);
    OT* o = x_out + base;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        o[i] = from_f32<OT>((hr[i] - sn.mean) * sn.rstd * load_any(w_next, wn_dtype, i));
}

__global__ void scale_kernel(float* __restrict__ x, long n, float s)
{
    fx_pdl_wait();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) x[i] *= s;
}

// Few rows (a decode step) leave the kernel's time to the trips of one block through its row: more threads, fewer.
inline int ln_threads(int hidden, int n_rows)
{
    const int per = n_rows >= 256 ? 8 : 2;      // elements a thread; many rows fill the machine with smaller blocks
    int n = ((hidden + per - 1) / per + 31) / 32 * 32;
    return n < 64 ? 64 : (n > LN_THREADS ? LN_THREADS : n);
}

}  // namespace

extern "C" int fx_layernorm(const float* x, const int* rows, const void* w, int w_dtype, const void* bias, int b_dtype,
                            float eps, void* out, int out_dtype, int n_rows, int hidden, void* stream)
{
    if (n_rows <= 0) return FX_OK;
    if (hidden <= 0) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == FX_F32) fx_launch_pdl(layernorm_kernel<float>, n_rows, ln_threads(hidden, n_rows), 0, s, x, rows, w, w_dtype, bias, b_dtype, eps, (float*)out, hidden);
    else if (out_dtype == FX_BF16) fx_launch_pdl(layernorm_kernel<bf16>, n_rows, ln_threads(hidden, n_rows), 0, s, x, rows, w, w_dtype, bias, b_dtype, eps, (bf16*)out, hidden);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}

extern "C" int fx_layernorm_residual(float* h, const void* y1, int y1_dtype, float s1, const void* y2, int y2_dtype,
                                     float s2, const void* w_post, int wp_dtype, float eps, const void* w_next,
                                     int wn_dtype, float eps_next, void* x_out, int x_dtype, int n_rows, int hidden,
                                     void* stream)
{
    if (n_rows <= 0) return FX_OK;
    if (hidden <= 0 || !y1 || !w_post || (w_next && !x_out)) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (!w_next || x_dtype == FX_F32)
        fx_launch_pdl(layernorm_residual_kernel<float>, n_rows, ln_threads(hidden, n_rows), 0, s, h, y1, y1_dtype, s1, y2, y2_dtype, s2,
                      w_post, wp_dtype, eps, w_next, wn_dtype, eps_next, (float*)x_out, hidden);
    else if (x_dtype == FX_BF16)
        fx_launch_pdl(layernorm_residual_kernel<bf16>, n_rows, ln_threads(hidden, n_rows), 0, s, h, y1, y1_dtype, s1, y2, y2_dtype, s2,
                      w_post, wp_dtype, eps, w_next, wn_dtype, eps_next, (bf16*)x_out, hidden);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}

extern "C" int fx_scale(float* x, long n, float scale, void* stream)
{
    if (n <= 0) return FX_OK;
    long blocks = fx_cdiv(n, 256);
    if (blocks > 4096) blocks = 4096;
    fx_launch_pdl(scale_kernel, (unsigned)blocks, 256, 0, (cudaStream_t)stream, x, n, scale);
    return fx_launch_status();
}
