// Attention of every query token over its own request's cache pages: one kernel
// for whole prompts, portions of prompts and single decoded tokens alike.
//
// The query at absolute position p of a request sees the keys at positions
// max(0, p - W + 1) .. p of that request (W = window, 0 = all), found through
// the request's block table: position t lives in page table[t / page_size] at
// offset t % page_size.  K and V of the tokens of this step were written to the
// pages before this kernel runs, so earlier steps' keys and this portion's keys
// are read the same way, and the mask is a function of absolute positions only.
//
// One warp per (token, head).  Keys are taken in blocks of 32 aligned to absolute
// positions; lane j scores key j of the block with the full 32-bit dot product,
// the block's maximum and sum update a running (m, l) pair, and the 32 lanes then
// share out the head dimension for the sum of p * V.  The order of every sum is
// fixed by (p, W) alone: the result does not depend on how the tokens were cut
// into steps, on the batch, or on which pages hold the keys.
//
// Reference: online softmax crates/ferrox-core/src/attention.rs:146-175; head h
// reads kv head h / (n_heads / n_kv_heads), scale 1/sqrt(head_dim) :432-449; window
// = the last W positions, the query's own included :484-524; pages :572-610.
// CUDA-core arithmetic throughout: this is the 32-bit path and the fallback of the
// bfloat16 path.
//
// Keys and values may differ in width (key_dim <= 640, value_dim <= 512) and in the distance between two
// positions of a page (ldk, ldv): values that are the leading part of the cached key rows (one latent vector a
// position, read by every head) are ldv = ldk with v_pages = k_pages.  Queries and outputs are addressed by a
// token stride and a head stride, so that rows laid out head by head ([head][token][dim]) are read as they lie.
// `slopes` (optional, one per head): the score of key j for the query at position i is lowered by
// slopes[h] * (i - j), a bias that grows with the distance.
// `keep_first` (with a window): the first keep_first positions of the request stay visible beside the window; they
// are taken first, in blocks of 32 from position 0, then the window's keys as ever.
// `sinks` (optional, one per head): exp(sinks[h]) is added to the softmax's denominator, once, unscaled.
// `value_share` (>= 1): that many consecutive key heads read one value head (value head = key head / value_share;
// the value pages hold n_kv_heads / value_share heads), for attention maps of their own keys over shared values.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_DK = 640;
constexpr int MAX_DV = 512;

template <typename T, int NV>
__global__ void __launch_bounds__(WARPS * 32) paged_attention_kernel(
    const T* __restrict__ q, long ldq, long ldqh, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
    long ldk, long ldv, const int* __restrict__ block_table, int table_width, int page_size,
    const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
    T* __restrict__ out, long ldo, long ldoh, int n_heads, int n_kv_heads, int key_dim, int value_dim, int window,
    float scale, float softcap, const float* __restrict__ slopes, int keep_first, const float* __restrict__ sinks,
    int value_share)
{
    __shared__ float q_s[WARPS][MAX_DK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * WARPS + warp;
    if (h >= n_heads) return;  // whole warp leaves; no block-wide barrier below
    const int kvh = h / (n_heads / n_kv_heads);
    const int vh = kvh / value_share, n_v_heads = n_kv_heads / value_share;   // key heads that read one value head
    const int pos = positions[t];
    const int* table = block_table + (long)seq_slot[token_seq[t]] * table_width;
    const T* qh = q + (long)t * ldq + (long)h * ldqh;
    for (int i = lane; i < key_dim; i += 32) q_s[warp][i] = to_f32(qh[i]);
    __syncwarp();
    const float slope = slopes ? slopes[h] : 0.f;

    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float m = -INFINITY, l = 0.f;
    float acc[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[i] = 0.f;

    // the kept first positions that the window no longer covers: keys 0 .. kept_end - 1
    const int kept_end = keep_first < lo ? keep_first : lo;
    const int kept_blocks = (kept_end + 31) / 32;
    const int win_kb = (lo / 32) * 32;
    const int n_blocks = kept_blocks + (pos - win_kb) / 32 + 1;
    for (int blk = 0; blk < n_blocks; ++blk) {
        const bool kept = blk < kept_blocks;
        const int kb = kept ? blk * 32 : win_kb + (blk - kept_blocks) * 32;
        const int key = kb + lane;
        bool valid = kept ? key < kept_end : (key >= lo && key <= pos);
        long place = -1;      // (page, kv head, position in the page) as one index
        long vplace = -1;     // the same for the value head
        float s = -INFINITY;
        const int page = valid ? table[key / page_size] : -1;
        valid = valid && page >= 0;  // a position without a page is skipped, never dereferenced
        if (valid) {
            place = ((long)page * n_kv_heads + kvh) * page_size + (key % page_size);
            vplace = ((long)page * n_v_heads + vh) * page_size + (key % page_size);
            const T* kr = k_pages + place * ldk;
            float dot = 0.f;
            for (int i = 0; i < key_dim; ++i) dot = fmaf(q_s[warp][i], to_f32(kr[i]), dot);
            s = dot * scale;
            if (softcap > 0.f) s = softcap * tanhf(s / softcap);   // soft cap: scores stay inside (-cap, cap)
            s -= slope * (float)(pos - key);                       // the distance bias
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;  // no key of this block is readable (uniform across the warp)
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < NV; ++i) acc[i] *= alpha;
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long bj = __shfl_sync(0xffffffffu, vplace, j);
            if (bj < 0) continue;  // uniform across the warp
            const T* vr = v_pages + bj * ldv;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int d = lane + 32 * i;
                if (d < value_dim) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
        m = m_new;
    }
    if (sinks && m != -INFINITY) {
        // a learned number per head in the denominator: it has no key and no value, and counts once
        const float sk = sinks[h], mm = fmaxf(m, sk), f = expf(m - mm);
        l = l * f + expf(sk - mm);
#pragma unroll
        for (int i = 0; i < NV; ++i) acc[i] *= f;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* o = out + (long)t * ldo + (long)h * ldoh;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = lane + 32 * i;
        if (d < value_dim) o[d] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T>
int launch_paged(const void* q, long ldq, long ldqh, const void* k_pages, const void* v_pages, long ldk, long ldv,
                 const int* block_table, int table_width, int page_size, const int* positions, const int* token_seq,
                 const int* seq_slot, void* out, long ldo, long ldoh, int n_tokens, int n_heads, int n_kv_heads,
                 int key_dim, int value_dim, int window, float scale, float softcap, const float* slopes, int keep_first,
                 const float* sinks, int value_share, cudaStream_t s)
{
    dim3 grid(n_tokens, (unsigned)fx_cdiv(n_heads, WARPS));
#define FX_GO(NV)                                                                                                     \
    paged_attention_kernel<T, NV><<<grid, WARPS * 32, 0, s>>>((const T*)q, ldq, ldqh, (const T*)k_pages,              \
        (const T*)v_pages, ldk, ldv, block_table, table_width, page_size, positions, token_seq, seq_slot, (T*)out,    \
        ldo, ldoh, n_heads, n_kv_heads, key_dim, value_dim, window, scale, softcap, slopes, keep_first, sinks,        \
        value_share)
    if (value_dim <= 64) FX_GO(2);
    else if (value_dim <= 128) FX_GO(4);
    else if (value_dim <= 256) FX_GO(8);
    else FX_GO(16);
#undef FX_GO
    return fx_launch_status();
}

}  // namespace

// The general form.  Pages: element d of position s of kv head g of page p lies at ((p * n_kv_heads + g) * page_size
// + s) * ldk + d in k_pages, likewise with ldv in v_pages.
extern "C" int fx_paged_attention_ex(const void* q, long ldq, long ldqh, const void* k_pages, const void* v_pages,
                                     long ldk, long ldv, int dtype, const int* block_table, int table_width,
                                     int page_size, const int* positions, const int* token_seq, const int* seq_slot,
                                     void* out, long ldo, long ldoh, int n_tokens, int n_heads, int n_kv_heads,
                                     int key_dim, int value_dim, int window, float scale, float softcap,
                                     const float* slopes, int keep_first, const float* sinks, int value_share,
                                     void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (value_share < 1) value_share = 1;
    if (n_kv_heads % value_share) return FX_ERR_SIZE;
    if (keep_first < 0 || window <= 0) keep_first = 0;
    if (key_dim > MAX_DK || value_dim > MAX_DV || key_dim <= 0 || value_dim <= 0 || n_kv_heads <= 0 ||
        n_heads % n_kv_heads || ldk < key_dim || ldv < value_dim)
        return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FX_F32)
        return launch_paged<float>(q, ldq, ldqh, k_pages, v_pages, ldk, ldv, block_table, table_width, page_size,
                                   positions, token_seq, seq_slot, out, ldo, ldoh, n_tokens, n_heads, n_kv_heads,
                                   key_dim, value_dim, window, scale, softcap, slopes, keep_first, sinks, value_share, s);
    if (dtype == FX_BF16)
        return launch_paged<bf16>(q, ldq, ldqh, k_pages, v_pages, ldk, ldv, block_table, table_width, page_size,
                                  positions, token_seq, seq_slot, out, ldo, ldoh, n_tokens, n_heads, n_kv_heads,
                                  key_dim, value_dim, window, scale, softcap, slopes, keep_first, sinks, value_share, s);
    return FX_ERR_DTYPE;
}

// Keys and values of one width, rows of [head][dim] a token.
extern "C" int fx_paged_attention(const void* q, long ldq, const void* k_pages, const void* v_pages, int dtype,
                                  const int* block_table, int table_width, int page_size, const int* positions,
                                  const int* token_seq, const int* seq_slot, void* out, long ldo, int n_tokens,
                                  int n_heads, int n_kv_heads, int head_dim, int window, float scale, float softcap,
                                  void* stream)
{
    return fx_paged_attention_ex(q, ldq, head_dim, k_pages, v_pages, head_dim, head_dim, dtype, block_table, table_width,
                                 page_size, positions, token_seq, seq_slot, out, ldo, head_dim, n_tokens, n_heads,
                                 n_kv_heads, head_dim, head_dim, window, scale, softcap, nullptr, 0, nullptr, 1, stream);
}
