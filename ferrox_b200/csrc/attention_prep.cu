// What stands between an attention mixer's projections and its attention kernel, for the mixers that do more
// there than rotate: queries and keys normed per head, a query temperature that grows with the position, keys
// and values of different widths; and the latent form, in which a position stores one normed latent vector and one
// rotated key part that all heads share.  All norms, angles, rotations and temperatures are 32-bit arithmetic;
// the rows keep the element type of the projections.
#include "common.cuh"
#include "api.h"

namespace {

// ---------------------------------------------------------------------------------------------------------------
// Rows of [q heads | k heads | v heads] (head widths D, D, V).  Per head, in place:
//   q <- q / sqrt(mean(q^2) + eps) * wq * (1 + coef * ln(floor((pos + 1) / every) + 1))
//   k <- k / sqrt(mean(k^2) + eps) * wk                      (wq, wk: [D], shared by the heads; null: no norm)
// then k and v go to the pages, [page][kv head][position][D] and [page][kv head][position][V].
// v_eps >= 0: every value head is divided by its root mean square first, v / sqrt(mean(v^2) + v_eps), no weight,
// and is cached so.
// One block a token, a warp a head.
template <typename T>
__global__ void qk_norm_store_kernel(T* __restrict__ qkv, long ld, const int* __restrict__ positions,
                                     const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                     const void* __restrict__ wq, const void* __restrict__ wk, int w_dtype, float eps,
                                     float temp_coef, int temp_every, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     const int* __restrict__ block_table, int table_width, int page_size, int H, int G,
                                     int D, int V, int write_cache, int* __restrict__ status, float v_eps)
{
    fx_pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int pos = positions[t];
    T* row = qkv + (long)t * ld;
    long place = -1;      // (page, kv head 0, position in the page) as one index
    if (write_cache) {
        const int page = block_table[(long)seq_slot[token_seq[t]] * table_width + pos / page_size];
        if (page < 0) { if (threadIdx.x == 0 && status) atomicExch(status, 2); }
        else place = (long)page * G * page_size + (pos % page_size);
    }
    float temp = 1.f;
    if (temp_every > 0) temp = 1.0f + temp_coef * logf((float)((pos + 1) / temp_every + 1));
    for (int u = warp; u < H + G; u += n_warps) {
        const bool is_q = u < H;
        T* x = row + (long)u * D;
        const void* w = is_q ? wq : wk;
        float r = 1.f;
        if (w) {
            float ss = 0.f;
            for (int i = lane; i < D; i += 32) { const float v = to_f32(x[i]); ss = fmaf(v, v, ss); }
            ss = warp_sum(ss);
            r = sqrtf(ss / (float)D + eps);
        }
        const float mult = is_q ? temp : 1.f;
        T* kp = (!is_q && place >= 0) ? k_pages + (place + (long)(u - H) * page_size) * D : nullptr;
        for (int i = lane; i < D; i += 32) {
            float v = to_f32(x[i]);
            if (w) v = v / r * load_any(w, w_dtype, i);
            const T o = from_f32<T>(v * mult);
            x[i] = o;
            if (kp) kp[i] = o;
        }
    }
    if (place < 0) return;
    const T* v = row + (long)(H + G) * D;
    if (v_eps >= 0.f) {
        for (int g = warp; g < G; g += n_warps) {
            const T* x = v + (long)g * V;
            float ss = 0.f;
            for (int i = lane; i < V; i += 32) { const float f = to_f32(x[i]); ss = fmaf(f, f, ss); }
            ss = warp_sum(ss);
            const float r = sqrtf(ss / (float)V + v_eps);
            T* vp = v_pages + (place + (long)g * page_size) * V;
            for (int i = lane; i < V; i += 32) vp[i] = from_f32<T>(to_f32(x[i]) / r);
        }
        return;
    }
    for (int idx = threadIdx.x; idx < G * V; idx += blockDim.x) {
        const int g = idx / V, i = idx - g * V;
        v_pages[(place + (long)g * page_size) * V + i] = v[idx];
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The latent form.  Per token: `dkv` = [C latent | R rotated key part] as projected, `q` = H heads of [D | R].
//   c <- dkv[:C] / sqrt(mean(dkv[:C]^2) + eps) * wc            -> pages[position][0:C]
//   k_rot <- pairs (2i, 2i+1) of the first rot_dims of dkv[C:] turned by the position's angles, the rest as it is
//                                                               -> pages[position][C:C+R]
//   q's D part of every head                                    -> q_plain[head][token][0:D]      (head by head)
//   q's R part of every head, turned the same way               -> q_full[head][token][C:C+R]
// q_full's first C columns are filled afterwards by the product of q_plain with the keys' read-out matrix, so that a
// score is one dot product of C + R elements against a cached row.  cos_sin: [tokens][rot_dims / 2][2].
// q_plain == nullptr: the queries stay token rows and only their rotated parts are turned, in place (the form in
// which keys and values are read out of the latent before the attention).
// One block a token.
template <typename T>
__global__ void latent_prep_kernel(T* __restrict__ q, long ldq, const T* __restrict__ dkv, long ld_dkv,
                                   const int* __restrict__ positions, const int* __restrict__ token_seq,
                                   const int* __restrict__ seq_slot, const void* __restrict__ wc, int w_dtype, float eps,
                                   const float* __restrict__ cos_sin, int rot_dims, T* __restrict__ q_plain,
                                   T* __restrict__ q_full, T* __restrict__ pages, const int* __restrict__ block_table,
                                   int table_width, int page_size, int n_tokens, int H, int D, int R, int C,
                                   int write_cache, int* __restrict__ status, int pairing)
{
    // pairing 1: neighbours (2i, 2i + 1); 0: halves (i, i + rot_dims / 2).  Thread i < half turns pair i; the
    // threads beyond copy element rot_dims + (i - half).
    __shared__ float scratch[33];
    fx_pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rot_dims >> 1;
    const float* cs = cos_sin + (long)t * half * 2;
    const int W = C + R;
    const T* d = dkv + (long)t * ld_dkv;
    T* dst = nullptr;
    if (write_cache) {
        const int page = block_table[(long)seq_slot[token_seq[t]] * table_width + pos / page_size];
        if (page < 0) { if (threadIdx.x == 0 && status) atomicExch(status, 2); }
        else dst = pages + ((long)page * page_size + (pos % page_size)) * W;
    }
    // queries: the plain part head by head, the rotated part into its place behind the latent columns
    T* qr = q + (long)t * ldq;
    if (q_plain)
        for (int idx = threadIdx.x; idx < H * D; idx += blockDim.x) {
            const int h = idx / D, i = idx - h * D;
            q_plain[((long)h * n_tokens + t) * D + i] = qr[(long)h * (D + R) + i];
        }
    for (int idx = threadIdx.x; idx < H * (R - half); idx += blockDim.x) {
        const int h = idx / (R - half), i = idx - h * (R - half);
        T* x = qr + (long)h * (D + R) + D;
        T* o = q_plain ? q_full + ((long)h * n_tokens + t) * W + C : x;   // no head-by-head copy: turned where it lies
        if (i < half) {
            const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
            const float a = to_f32(x[ia]), b = to_f32(x[ib]), c = cs[2 * i], s = cs[2 * i + 1];
            o[ia] = from_f32<T>(a * c - b * s);
            o[ib] = from_f32<T>(b * c + a * s);
        } else {
            o[half + i] = x[half + i];      // beyond the rotated pairs: element rot_dims + (i - half)
        }
    }
    if (!dst) return;    // (uniform across the block)
    float ss = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) { const float v = to_f32(d[i]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    const float r = sqrtf(ss / (float)C + eps);
    for (int i = threadIdx.x; i < C; i += blockDim.x)
        dst[i] = from_f32<T>(to_f32(d[i]) / r * load_any(wc, w_dtype, i));
    for (int i = threadIdx.x; i < R - half; i += blockDim.x) {
        const T* x = d + C;
        if (i < half) {
            const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
            const float a = to_f32(x[ia]), b = to_f32(x[ib]), c = cs[2 * i], s = cs[2 * i + 1];
            dst[C + ia] = from_f32<T>(a * c - b * s);
            dst[C + ib] = from_f32<T>(b * c + a * s);
        } else {
            dst[C + half + i] = x[half + i];
        }
    }
}

// out[t, :] = x[t, :] / sqrt(mean(x[t, :]^2) + eps) * w over rows with strides; one block a row.
template <typename TI, typename TO>
__global__ void rmsnorm_rows_kernel(const TI* __restrict__ x, long ldx, const void* __restrict__ w, int w_dtype, float eps,
                                    TO* __restrict__ out, long ldo, int n)
{
    __shared__ float scratch[33];
    fx_pdl_wait();
    const TI* xr = x + (long)blockIdx.x * ldx;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = to_f32(xr[i]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    const float r = sqrtf(ss / (float)n + eps);
    TO* o = out + (long)blockIdx.x * ldo;
    for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = from_f32<TO>(to_f32(xr[i]) / r * load_any(w, w_dtype, i));
}

// out[t][h * V + v] = in[t * in_ldt + h * in_ldh + v] * (gate ? sigmoid(gate[t][h * V + v]) : 1): rows laid out head
// by head ([h][t][v]: in_ldh = tokens * V, in_ldt = V) back into token rows, with the output gate of the mixer applied
// (gate_per_head: one gate a head, gate[t][h], instead of one an element)
// on the way; or token rows gated where they lie (in == out, in_ldt = ldo, in_ldh = V).
template <typename T>
__global__ void heads_to_tokens_kernel(const T* in, long in_ldt, long in_ldh, const T* __restrict__ gate, long ldg, T* out,
                                       long ldo, int n_tokens, int H, int V, int gate_per_head)
{
    fx_pdl_wait();
    const long total = (long)n_tokens * H * V;
    for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
        const int t = (int)(idx / (H * V));
        const int c = (int)(idx - (long)t * H * V);
        const int h = c / V, v = c - h * V;
        float x = to_f32(in[(long)t * in_ldt + (long)h * in_ldh + v]);
        if (gate) x *= 1.0f / (1.0f + expf(-to_f32(gate[(long)t * ldg + (gate_per_head ? h : c)])));
        out[(long)t * ldo + c] = from_f32<T>(x);
    }
}

int threads_for_width(int n) {
    int t = 32;
    while (t < n && t < 256) t <<= 1;
    return t;
}

}  // namespace

extern "C" int fx_qk_norm_store(void* qkv, int dtype, long ld, const int* positions, const int* token_seq,
                                const int* seq_slot, const void* wq, const void* wk, int w_dtype, float eps,
                                float temp_coef, int temp_every, void* k_pages, void* v_pages, const int* block_table,
                                int table_width, int page_size, int n_tokens, int n_heads, int n_kv_heads, int key_dim,
                                int value_dim, int write_cache, int* status, float v_eps, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (key_dim <= 0 || value_dim <= 0 || page_size <= 0 || n_heads <= 0 || n_kv_heads <= 0) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int nt = 32 * (n_heads + n_kv_heads > 8 ? 8 : n_heads + n_kv_heads);
#define FX_GO(T)                                                                                                      \
    fx_launch_pdl(qk_norm_store_kernel<T>, n_tokens, nt, 0, s, (T*)qkv, ld, positions, token_seq, seq_slot, wq, wk,  \
                  w_dtype, eps, temp_coef, temp_every, (T*)k_pages, (T*)v_pages, block_table, table_width, page_size, \
                  n_heads, n_kv_heads, key_dim, value_dim, write_cache, status, v_eps)
    if (dtype == FX_F32) FX_GO(float);
    else if (dtype == FX_BF16) FX_GO(bf16);
    else return FX_ERR_DTYPE;
#undef FX_GO
    return fx_launch_status();
}

extern "C" int fx_latent_prep(void* q, long ldq, const void* dkv, long ld_dkv, int dtype, const int* positions,
                              const int* token_seq, const int* seq_slot, const void* wc, int w_dtype, float eps,
                              const float* cos_sin, int rot_dims, void* q_plain, void* q_full, void* pages,
                              const int* block_table, int table_width, int page_size, int n_tokens, int n_heads,
                              int plain_dim, int rot_dim, int rank, int write_cache, int* status, int pairing,
                              void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (pairing < 0 || pairing > 1) return FX_ERR_SIZE;
    if (rot_dims % 2 || rot_dims > rot_dim || rot_dims < 0 || plain_dim <= 0 || rank <= 0 || page_size <= 0)
        return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int nt = threads_for_width(n_heads * plain_dim > rank ? n_heads * plain_dim : rank);
#define FX_GO(T)                                                                                                      \
    fx_launch_pdl(latent_prep_kernel<T>, n_tokens, nt, 0, s, (T*)q, ldq, (const T*)dkv, ld_dkv, positions,      \
                  token_seq, seq_slot, wc, w_dtype, eps, cos_sin, rot_dims, (T*)q_plain, (T*)q_full, (T*)pages,       \
                  block_table, table_width, page_size, n_tokens, n_heads, plain_dim, rot_dim, rank, write_cache, status, pairing)
    if (dtype == FX_F32) FX_GO(float);
    else if (dtype == FX_BF16) FX_GO(bf16);
    else return FX_ERR_DTYPE;
#undef FX_GO
    return fx_launch_status();
}

extern "C" int fx_rmsnorm_rows(const void* x, int x_dtype, long ldx, const void* w, int w_dtype, float eps, void* out,
                               int out_dtype, long ldo, int n_rows, int n, void* stream)
{
    if (n_rows <= 0 || n <= 0) return FX_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int nt = threads_for_width(n);
#define FX_GO(TI, TO)                                                                                                 \
    fx_launch_pdl(rmsnorm_rows_kernel<TI, TO>, n_rows, nt, 0, s, (const TI*)x, ldx, w, w_dtype, eps, (TO*)out, ldo, n)
    if (x_dtype == FX_F32 && out_dtype == FX_F32) FX_GO(float, float);
    else if (x_dtype == FX_F32 && out_dtype == FX_BF16) FX_GO(float, bf16);
    else if (x_dtype == FX_BF16 && out_dtype == FX_BF16) FX_GO(bf16, bf16);
    else if (x_dtype == FX_BF16 && out_dtype == FX_F32) FX_GO(bf16, float);
    else return FX_ERR_DTYPE;
#undef FX_GO
    return fx_launch_status();
}

extern "C" int fx_heads_to_tokens(const void* in, long in_ldt, long in_ldh, const void* gate, long ldg, void* out, long ldo,
                                  int dtype, int n_tokens, int n_heads, int width, int gate_per_head, void* stream)
{
    if (n_tokens <= 0 || n_heads <= 0 || width <= 0) return FX_OK;
    cudaStream_t s = (cudaStream_t)stream;
    long blocks = fx_cdiv((long)n_tokens * n_heads * width, 256);
    if (blocks > fx_sm_count() * 16L) blocks = fx_sm_count() * 16L;
    if (dtype == FX_F32)
        fx_launch_pdl(heads_to_tokens_kernel<float>, (unsigned)blocks, 256, 0, s, (const float*)in, in_ldt, in_ldh, (const float*)gate, ldg,
                      (float*)out, ldo, n_tokens, n_heads, width, gate_per_head);
    else if (dtype == FX_BF16)
        fx_launch_pdl(heads_to_tokens_kernel<bf16>, (unsigned)blocks, 256, 0, s, (const bf16*)in, in_ldt, in_ldh, (const bf16*)gate, ldg,
                      (bf16*)out, ldo, n_tokens, n_heads, width, gate_per_head);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}
