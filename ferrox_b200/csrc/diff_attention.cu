// What an attention mixer with a short convolution behind its projections does between the fused product and the
// attention kernel, and what differential attention does after it.
//
// fx_conv_rotary_store, one block a (token, head).  The row as projected is [q heads | k heads | v heads]; on every channel
//
//   y_t[c] = sum_j w[c, j] u_(t - taps + 1 + j)[c]          (zeros before the request's start; no input added)
//
// with the inputs before the step's first token taken from the request's state slot (tail [slots, taps - 1,
// channels], 32-bit, oldest first: the framework's convention for short convolutions).  Then the first rot_dims
// elements of every q and k head are turned by the token's angles (cos_sin [tokens][rot_dims / 2][2], which carry
// any factor on cos and sin; pairs (i, i + rot_dims / 2) or neighbours), q goes to q_out and k and v to the pages
// (k [pages, k heads, page, head_dim], v [pages, v heads, page, value_dim]).  Sums and rotation are 32-bit; the
// element type is that of the projected rows.  A step of one token a request (update_tail) also moves the tail on;
// other steps call fx_conv_tail_update on the projected rows afterwards.  A prompt's portion (64 tokens or more)
// goes in runs of up to 16 tokens a block instead, whose rows are staged once in shared memory
// (conv_rotary_store_run_kernel).
//
// fx_diff_combine, one warp a (token, head).  The attention ran over twice as many query heads as the mixer has:
// for the heads hg = 0 .. group - 1 of kv head g, map j of head g * group + hg is row (2 g + j) * group + hg of the
// attention's output.  out = rms(a1 - lambda a2) * post over the head's values, without a weight.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int MAX_TAPS = 16;
constexpr int RUN_MAX = 16;      // tokens a block of the prompt form takes

template <typename T>
__global__ void __launch_bounds__(128) conv_rotary_store_kernel(
    const T* __restrict__ proj, long ldp, const void* __restrict__ w, int w_dtype, int taps, float* tail,
    const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
    const float* __restrict__ cos_sin, int rot_dims, int pairing, T* __restrict__ q_out, long ldq,
    T* __restrict__ k_pages, T* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
    int page_size, int n_q_heads, int n_k_heads, int head_dim, int n_v_heads, int value_dim, int write_cache,
    int update_tail, int* __restrict__ status)
{
    // one block a (token, head): q heads, then k heads, then v heads
    fx_pdl_wait();
    const int t = blockIdx.x, head = blockIdx.y;
    const int b = token_seq[t];
    const int pos = positions[t];
    const int slot = seq_slot[b];
    const int qk = (n_q_heads + n_k_heads) * head_dim, C = qk + n_v_heads * value_dim;
    const bool is_v = head >= n_q_heads + n_k_heads;
    const int width = is_v ? value_dim : head_dim;
    const int c0 = is_v ? qk + (head - n_q_heads - n_k_heads) * value_dim : head * head_dim;    // the head's first channel
    // how many rows before t belong to the same entry (at most taps - 1 matter)
    int own = 0;
    while (own < taps - 1 && t - own - 1 >= 0 && token_seq[t - own - 1] == b) ++own;
    float* tl = tail + (long)slot * (taps - 1) * C;
    const T* row = proj + (long)t * ldp;
    auto conv = [&](int c) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;
            float v;
            if (back <= own) v = to_f32(row[c - (long)back * ldp]);
            else v = tl[(long)(taps - 1 - (back - own)) * C + c];
            acc = fmaf(load_any(w, w_dtype, (long)c * taps + j), v, acc);
        }
        return acc;
    };
    T* dst = nullptr;      // where the head's elements go
    if (head < n_q_heads) {
        dst = q_out + (long)t * ldq + (long)head * head_dim;
    } else if (write_cache) {
        const int page = block_table[(long)slot * table_width + pos / page_size];
        if (page < 0) { if (threadIdx.x == 0 && status) atomicExch(status, 2); }
        else if (is_v) dst = v_pages + (((long)page * n_v_heads + (head - n_q_heads - n_k_heads)) * page_size + (pos % page_size)) * value_dim;
        else dst = k_pages + (((long)page * n_k_heads + (head - n_q_heads)) * page_size + (pos % page_size)) * head_dim;
    }
    const int rot = (is_v || !cos_sin) ? 0 : rot_dims, half = rot >> 1;
    const float* cs = cos_sin ? cos_sin + (long)t * (rot_dims >> 1) * 2 : nullptr;
    if (dst) {
        // element i of the head; the first of a rotated pair does both, its partner is skipped
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            if (i < rot) {
                if (pairing ? (i & 1) : (i >= half)) continue;
                const int p = pairing ? i >> 1 : i, i1 = pairing ? i + 1 : i + half;
                const float a = conv(c0 + i), bb = conv(c0 + i1), c = cs[2 * p], s = cs[2 * p + 1];
                dst[i] = from_f32<T>(a * c - bb * s);
                dst[i1] = from_f32<T>(bb * c + a * s);
            } else {
                dst[i] = from_f32<T>(conv(c0 + i));
            }
        }
    }
    if (update_tail && taps > 1) {
        // (the caller's promise that every entry brings exactly one token: this block is the only reader of its
        // channels' tail in the whole step, and moves it on by the token's own row once all its sums are made)
        __syncthreads();
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const int c = c0 + i;
            for (int j = 0; j + 1 < taps - 1; ++j) tl[(long)j * C + c] = tl[(long)(j + 1) * C + c];
            tl[(long)(taps - 2) * C + c] = to_f32(row[c]);
        }
    }
}

// The same for a prompt's portion: one block a (run of tokens, head).  The run's projected rows of the head, with the
// taps - 1 rows before them, are staged once in shared memory (32-bit) beside the head's taps, so that every input
// is read from memory once; the (token, element) pairs of the run are then shared out over the threads.  Inputs
// before an entry's first row of the step come from the slot's tail as ever.
template <typename T>
__global__ void __launch_bounds__(128) conv_rotary_store_run_kernel(
    const T* __restrict__ proj, long ldp, const void* __restrict__ w, int w_dtype, int taps, const float* __restrict__ tail,
    const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
    const float* __restrict__ cos_sin, int rot_dims, int pairing, T* __restrict__ q_out, long ldq,
    T* __restrict__ k_pages, T* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
    int page_size, int n_tokens, int run, int n_q_heads, int n_k_heads, int head_dim, int n_v_heads, int value_dim,
    int write_cache, int* __restrict__ status)
{
    extern __shared__ float run_s[];      // [run + taps - 1][width] rows, then [width][taps] weights
    fx_pdl_wait();
    const int head = blockIdx.y;
    const int t0 = blockIdx.x * run, t1 = min(n_tokens, t0 + run);
    const int first = max(0, t0 - (taps - 1));      // the first staged row
    const int qk = (n_q_heads + n_k_heads) * head_dim, C = qk + n_v_heads * value_dim;
    const bool is_q = head < n_q_heads, is_v = head >= n_q_heads + n_k_heads;
    const int width = is_v ? value_dim : head_dim;
    const int c0 = is_v ? qk + (head - n_q_heads - n_k_heads) * value_dim : head * head_dim;    // the head's first channel
    float* w_s = run_s + (long)(run + taps - 1) * width;
    for (int idx = threadIdx.x; idx < (t1 - first) * width; idx += blockDim.x) {
        const int r = idx / width, i = idx - r * width;
        run_s[idx] = to_f32(proj[(long)(first + r) * ldp + c0 + i]);
    }
    for (int idx = threadIdx.x; idx < width * taps; idx += blockDim.x) w_s[idx] = load_any(w, w_dtype, (long)c0 * taps + idx);
    // what the run's tokens need beside their rows, worked out once a token: how many rows before it belong to the same
    // entry (at most taps - 1 matter), its slot's tail, and where the head's elements go
    __shared__ int own_s[RUN_MAX];
    __shared__ const float* tl_s[RUN_MAX];
    __shared__ T* dst_s[RUN_MAX];
    if (threadIdx.x < t1 - t0) {
        const int t = t0 + threadIdx.x;
        const int b = token_seq[t];
        const int slot = seq_slot[b];
        int own = 0;
        while (own < taps - 1 && t - own - 1 >= 0 && token_seq[t - own - 1] == b) ++own;
        own_s[threadIdx.x] = own;
        tl_s[threadIdx.x] = tail + (long)slot * (taps - 1) * C + c0;
        T* dst = nullptr;
        if (is_q) {
            dst = q_out + (long)t * ldq + (long)head * head_dim;
        } else if (write_cache) {
            const int pos = positions[t];
            const int page = block_table[(long)slot * table_width + pos / page_size];
            if (page < 0) { if (status) atomicExch(status, 2); }
            else if (is_v) dst = v_pages + (((long)page * n_v_heads + (head - n_q_heads - n_k_heads)) * page_size + (pos % page_size)) * value_dim;
            else dst = k_pages + (((long)page * n_k_heads + (head - n_q_heads)) * page_size + (pos % page_size)) * head_dim;
        }
        dst_s[threadIdx.x] = dst;
    }
    __syncthreads();
    const int rot = (is_v || !cos_sin) ? 0 : rot_dims, half = rot >> 1;
    for (int idx = threadIdx.x; idx < (t1 - t0) * width; idx += blockDim.x) {
        const int tt = idx / width, i = idx - tt * width, t = t0 + tt;
        int i1 = -1, p = 0;      // the partner of a rotated element and the pair's index
        if (i < rot) {
            if (pairing ? (i & 1) : (i >= half)) continue;      // (its partner does both)
            p = pairing ? i >> 1 : i;
            i1 = pairing ? i + 1 : i + half;
        }
        T* dst = dst_s[tt];
        if (!dst) continue;
        const int own = own_s[tt];
        const float* tl = tl_s[tt];
        float a = 0.f, bb = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;      // this tap's input lies `back` tokens before t
            float va, vb = 0.f;
            if (back <= own) {
                const float* r = run_s + (long)(t - back - first) * width;
                va = r[i];
                if (i1 >= 0) vb = r[i1];
            } else {
                const float* r = tl + (long)(taps - 1 - (back - own)) * C;
                va = r[i];
                if (i1 >= 0) vb = r[i1];
            }
            a = fmaf(w_s[i * taps + j], va, a);
            if (i1 >= 0) bb = fmaf(w_s[i1 * taps + j], vb, bb);
        }
        if (i1 >= 0) {
            const float* cs = cos_sin + ((long)t * (rot_dims >> 1) + p) * 2;
            dst[i] = from_f32<T>(a * cs[0] - bb * cs[1]);
            dst[i1] = from_f32<T>(bb * cs[0] + a * cs[1]);
        } else {
            dst[i] = from_f32<T>(a);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(128) diff_combine_kernel(const T* __restrict__ attn, long lda, T* __restrict__ out,
                                                           long ldo, int n_tokens, int n_heads, int group, int V,
                                                           float lambda, float eps, float post)
{
    fx_pdl_wait();
    const int lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= (long)n_tokens * n_heads) return;
    const int t = (int)(item / n_heads), h = (int)(item - (long)t * n_heads);
    const int g = h / group, hg = h - g * group;
    const T* a1 = attn + (long)t * lda + ((long)(2 * g) * group + hg) * V;
    const T* a2 = attn + (long)t * lda + ((long)(2 * g + 1) * group + hg) * V;
    float ss = 0.f;
    for (int i = lane; i < V; i += 32) {
        const float d = to_f32(a1[i]) - lambda * to_f32(a2[i]);
        ss = fmaf(d, d, ss);
    }
    ss = warp_sum(ss);
    const float r = post / sqrtf(ss / (float)V + eps);
    T* o = out + (long)t * ldo + (long)h * V;
    for (int i = lane; i < V; i += 32) o[i] = from_f32<T>((to_f32(a1[i]) - lambda * to_f32(a2[i])) * r);
}

}  // namespace

extern "C" int fx_conv_rotary_store(const void* proj, int dtype, long ldp, const void* w, int w_dtype, int taps,
                                    float* tail, const int* positions, const int* token_seq, const int* seq_slot,
                                    const float* cos_sin, int rot_dims, int pairing, void* q_out, long ldq,
                                    void* k_pages, void* v_pages, const int* block_table, int table_width,
                                    int page_size, int n_tokens, int n_q_heads, int n_k_heads, int head_dim,
                                    int n_v_heads, int value_dim, int write_cache, int update_tail, int* status,
                                    void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (taps < 1 || taps > MAX_TAPS || rot_dims < 0 || rot_dims % 2 || rot_dims > head_dim || pairing < 0 ||
        pairing > 1 || page_size <= 0 || head_dim <= 0 || value_dim <= 0 || n_q_heads <= 0 || n_k_heads <= 0 ||
        n_v_heads <= 0 || proj == q_out)
        return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int widest = head_dim > value_dim ? head_dim : value_dim;
    if (!update_tail && n_tokens >= 64) {
        // a prompt's portion: runs of tokens whose rows a block stages once (as many as 40 KB of shared memory hold)
        int run = (int)(40 * 1024 / 4 / widest) - 2 * taps;
        run = run > RUN_MAX ? RUN_MAX : run;
        if (run >= 4) {
            const dim3 rgrid((unsigned)fx_cdiv(n_tokens, run), n_q_heads + n_k_heads + n_v_heads);
            const size_t smem = ((size_t)(run + taps - 1) * widest + (size_t)widest * taps) * sizeof(float);
#define FX_RUN(T)                                                                                                     \
    fx_launch_pdl(conv_rotary_store_run_kernel<T>, rgrid, 128, smem, s, (const T*)proj, ldp, w, w_dtype, taps,         \
                  (const float*)tail, positions, token_seq, seq_slot, cos_sin, rot_dims, pairing, (T*)q_out, ldq,     \
                  (T*)k_pages, (T*)v_pages, block_table, table_width, page_size, n_tokens, run, n_q_heads, n_k_heads, \
                  head_dim, n_v_heads, value_dim, write_cache, status)
            if (dtype == FX_F32) FX_RUN(float);
            else if (dtype == FX_BF16) FX_RUN(bf16);
            else return FX_ERR_DTYPE;
#undef FX_RUN
            return fx_launch_status();
        }
    }
    const dim3 grid(n_tokens, n_q_heads + n_k_heads + n_v_heads);
    const int nt = widest <= 32 ? 32 : widest <= 64 ? 64 : 128;
#define FX_GO(T)                                                                                                      \
    fx_launch_pdl(conv_rotary_store_kernel<T>, grid, nt, 0, s, (const T*)proj, ldp, w, w_dtype, taps, tail,           \
                  positions, token_seq, seq_slot, cos_sin, rot_dims, pairing, (T*)q_out, ldq, (T*)k_pages,            \
                  (T*)v_pages, block_table, table_width, page_size, n_q_heads, n_k_heads, head_dim, n_v_heads,        \
                  value_dim, write_cache, update_tail, status)
    if (dtype == FX_F32) FX_GO(float);
    else if (dtype == FX_BF16) FX_GO(bf16);
    else return FX_ERR_DTYPE;
#undef FX_GO
    return fx_launch_status();
}

extern "C" int fx_diff_combine(const void* attn, long lda, void* out, long ldo, int dtype, int n_tokens, int n_heads,
                               int group, int value_dim, float lambda, float eps, float post, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (n_heads <= 0 || group <= 0 || n_heads % group || value_dim <= 0) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)fx_cdiv((long)n_tokens * n_heads, 4);
    if (dtype == FX_F32)
        fx_launch_pdl(diff_combine_kernel<float>, blocks, 128, 0, s, (const float*)attn, lda, (float*)out, ldo,
                      n_tokens, n_heads, group, value_dim, lambda, eps, post);
    else if (dtype == FX_BF16)
        fx_launch_pdl(diff_combine_kernel<bf16>, blocks, 128, 0, s, (const bf16*)attn, lda, (bf16*)out, ldo, n_tokens,
                      n_heads, group, value_dim, lambda, eps, post);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}
