// Attention over pages in its general form, in bfloat16 on the tensor cores: keys and values of different widths
// (values may be the leading part of the cached key rows), queries and outputs addressed by a token stride and a
// head stride, an optional bias slope[h] * (i - j) taken off the scores, a window.  The operation of
// fx_paged_attention_ex (attention_generic.cu), for prompt portions and for decoded tokens alike.
//
// A tile is 64 ROWS, a row being a (token, query head) pair: consecutive tokens of one request times the query
// heads that share one kv head (at most 64 of them a tile).  With many heads on one kv head (a latent cache that
// all heads read: one kv head) a tile is a few tokens times all heads, so that a block of keys, once in shared
// memory, serves every head; with one token a request (decoding) a tile is that token's heads.  Every row carries
// its own position, window edge and slope.  4 warps of 16 rows; with NSPLIT = 2 a second set of 4 warps takes the
// other half of the value columns (it repeats the scores, which are the smaller product when values are wide).
// Keys in blocks of 32 by cp.async, two buffers; S = Q K^T and O += P V by mma.sync.m16n8k16 (bf16 in, f32 out);
// scores, bias, softmax and sums are 32-bit, P is rounded to bfloat16 for the second product.  Q stays in shared
// memory (key rows of up to 640 elements do not fit the registers).
//
// Work items: `items` int32 [n, 5] = (first flat token, tokens, entry, first query head, heads) from the host for
// prompt portions; items == nullptr: one token a tile, grid = (tokens, kv heads x head chunks), the entry from
// token_seq, so that a captured decode step replays unchanged.  Positions are read from `positions` either way.
// In that form a token's visible keys may be cut into n_splits runs (fx_split_range: equal runs, whatever the
// context length), one block each, so that a step of few tokens fills the machine; a block then leaves its
// unnormalised sums and its (maximum, sum) in scratch and a second kernel adds a row's runs up.
//
// keep_first (with a window): the first keep_first positions of a request stay visible to every query beside its
// window.  The key blocks that hold them and lie wholly before the first window block are taken first (blocks
// 0 .. n_kept - 1 of the loop), then the window's blocks; of a decoding token's runs, run 0 takes them.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int BQ = 64;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct GArgs {
    const bf16* q; long ldq, ldqh;
    const bf16* k_pages; const bf16* v_pages; long ldk, ldv;
    long k_page_stride, k_head_stride, v_page_stride, v_head_stride;   // element (page, kv head, position, d) lies at
                                                                       // page * page_stride + head * head_stride + position * ld + d
    const int* block_table; int table_width, page_size;
    const int* positions; const int* token_seq; const int* seq_slot;
    const int* items;
    bf16* out; long ldo, ldoh;
    int n_heads, n_kv_heads, key_dim, value_dim, window;
    int keep_first;   // (window > 0) positions 0 .. keep_first - 1 stay visible beside the window
    float scale_log2e;
    const float* slopes;
    int alias;        // the values are the leading columns of the key rows: one copy in shared memory serves both
    int part_cols;    // value columns a set of 4 warps takes (a multiple of 16)
    int n_splits;     // > 1 (only without items): blockIdx.z takes one run of the token's keys
    float* part_o;    // [tokens][heads][n_splits][value_dim] unnormalised sums, relative to the run's maximum
    float* part_ml;   // [tokens][heads][n_splits][2] the run's maximum (in units of log2 e) and its sum
    float softcap;    // c > 0: the scaled scores pass through c tanh(s / c); cap_log2e = c log2 e
    float cap_log2e, scale_over_cap;
    const float* sinks;   // (optional, one per head) exp(sinks[h]) joins the softmax's denominator once
    int value_share;      // consecutive key heads that read one value head
};

// DVMAX: most value columns one warp accumulates.  NSPLIT: sets of 4 warps that share out the value columns.
// BKEY: keys a block of the loop holds.
template <int DVMAX, int NSPLIT, int BKEY>
__global__ void __launch_bounds__(128 * NSPLIT) general_attention_kernel(GArgs a)
{
    constexpr int NTHREADS = 128 * NSPLIT;
    extern __shared__ __align__(16) uint8_t smem[];
    const int pk = a.key_dim * 2 + 16, pv = a.value_dim * 2 + 16;   // bytes per row, 16 of padding against bank conflicts
    uint8_t* q_s = smem;                                  // [BQ][pk]
    uint8_t* k_s = q_s + BQ * pk;                         // [2][BKEY][pk]
    uint8_t* v_s = a.alias ? k_s : k_s + 2 * BKEY * pk;   // [2][BKEY][pv]
    const int pvv = a.alias ? pk : pv;
    const uint32_t q_u = (uint32_t)__cvta_generic_to_shared(q_s);
    const uint32_t k_u = (uint32_t)__cvta_generic_to_shared(k_s);
    const uint32_t v_u = (uint32_t)__cvta_generic_to_shared(v_s);

    const int warp = (threadIdx.x >> 5) & 3, part = threadIdx.x >> 7, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int group = a.n_heads / a.n_kv_heads;
    int tok0, n_tok, entry, head0, n_h;
    if (a.items) {
        const int* it = a.items + (long)blockIdx.x * 5;
        tok0 = it[0]; n_tok = it[1]; entry = it[2]; head0 = it[3]; n_h = it[4];
    } else {
        const int chunks = (group + BQ - 1) / BQ;
        const int kv = blockIdx.y / chunks, c = blockIdx.y - kv * chunks;
        tok0 = blockIdx.x; n_tok = 1; entry = a.token_seq[tok0];
        head0 = kv * group + c * BQ;
        n_h = min(BQ, group - c * BQ);
    }
    fx_pdl_wait();
    const int kvh = head0 / group;
    const int pos0 = a.positions[tok0];
    const int rows = n_tok * n_h;
    const int* table = a.block_table + (long)a.seq_slot[entry] * a.table_width;
    const int kchunks = a.key_dim / 8, vchunks = a.value_dim / 8;   // 16-byte chunks per row
    int last_pos = pos0 + n_tok - 1;
    int key_lo = (a.window > 0 && pos0 - a.window + 1 > 0) ? pos0 - a.window + 1 : 0;   // first key any row may see
    int keep = a.keep_first;   // kept first positions this block takes
    if (a.n_splits > 1) {      // (one token a tile) this block's run of the token's keys
        int k_begin, k_end;
        fx_split_range(pos0, key_lo, blockIdx.z, a.n_splits, 0, k_begin, k_end);
        if (k_begin >= k_end) return;      // nothing of this run is visible: the merge skips it by the same rule
        if (blockIdx.z > 0) keep = 0;      // (run 0 always has keys: it begins at the token's first visible key)
        key_lo = k_begin; last_pos = k_end - 1;
    }
    const int kb_begin = (key_lo / BKEY) * BKEY;
    // key blocks of the kept first positions that lie wholly before the first window block (what of them falls into
    // a window block is admitted there by the mask)
    const int n_kept = (min(keep, kb_begin) + BKEY - 1) / BKEY;
    const int n_blocks = n_kept + (last_pos - kb_begin) / BKEY + 1;
    auto block_start = [&](int blk) { return blk < n_kept ? blk * BKEY : kb_begin + (blk - n_kept) * BKEY; };

    // ---- Q rows -> shared memory (rows past the tile's end are zero) ----------------
    for (int c = threadIdx.x; c < BQ * kchunks; c += NTHREADS) {
        const int r = c / kchunks, ch = c - r * kchunks;
        const int rr = min(r, rows - 1);
        const bf16* src = a.q + (long)(tok0 + rr / n_h) * a.ldq + (long)(head0 + rr % n_h) * a.ldqh + ch * 8;
        cp_async16(q_u + r * pk + ch * 16, src, r < rows ? 16 : 0);
    }
    auto load_kv = [&](int blk, int buf) {
        const int kb = block_start(blk);
        for (int c = threadIdx.x; c < BKEY * kchunks; c += NTHREADS) {
            const int r = c / kchunks, ch = c - r * kchunks;
            const int key = kb + r;
            int page = -1;
            if (key <= last_pos && (key >= key_lo || key < keep)) page = table[key / a.page_size];
            const bool ok = page >= 0;
            const long at = ok ? (long)page * a.k_page_stride + (long)kvh * a.k_head_stride + (long)(key % a.page_size) * a.ldk : 0;
            cp_async16(k_u + (buf * BKEY + r) * pk + ch * 16, a.k_pages + at + ch * 8, ok ? 16 : 0);
        }
        if (a.alias) return;
        for (int c = threadIdx.x; c < BKEY * vchunks; c += NTHREADS) {
            const int r = c / vchunks, ch = c - r * vchunks;
            const int key = kb + r;
            int page = -1;
            if (key <= last_pos && (key >= key_lo || key < keep)) page = table[key / a.page_size];
            const bool ok = page >= 0;
            const long at = ok ? (long)page * a.v_page_stride + (long)(kvh / a.value_share) * a.v_head_stride + (long)(key % a.page_size) * a.ldv : 0;
            cp_async16(v_u + (buf * BKEY + r) * pv + ch * 16, a.v_pages + at + ch * 8, ok ? 16 : 0);
        }
    };
    load_kv(0, 0);
    cp_commit();

    constexpr int ON = DVMAX / 8;      // n-tiles of this warp's share of the output
    const int ks_n = a.key_dim / 16;
    const int col0 = part * a.part_cols;                              // this warp's first value column
    const int my_cols = min(a.part_cols, a.value_dim - col0);         // and how many it has (may be <= 0)
    float o[ON][4];
#pragma unroll
    for (int i = 0; i < ON; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g + 8 of this warp's 16
    const int qrow0 = warp * 16;
    const int r0 = qrow0 + g, r1 = r0 + 8;
    // each row's own position, first visible key and slope (in units of log2 e)
    const int p_row0 = pos0 + min(r0, rows - 1) / n_h, p_row1 = pos0 + min(r1, rows - 1) / n_h;
    const int lo0 = max(a.window > 0 ? p_row0 - a.window + 1 : 0, key_lo), lo1 = max(a.window > 0 ? p_row1 - a.window + 1 : 0, key_lo);
    const int hi0 = min(p_row0, last_pos), hi1 = min(p_row1, last_pos);      // each row's last visible key here
    float sl0 = 0.f, sl1 = 0.f;
    if (a.slopes) {
        sl0 = a.slopes[head0 + min(r0, rows - 1) % n_h] * 1.4426950408889634f;
        sl1 = a.slopes[head0 + min(r1, rows - 1) % n_h] * 1.4426950408889634f;
    }
    // the warp's rows cover the tokens of rows qrow0 .. qrow0 + 15
    const int w_first = pos0 + min(qrow0, rows - 1) / n_h, w_last = min(last_pos, pos0 + min(qrow0 + 15, rows - 1) / n_h);
    const int w_lo = max(key_lo, (a.window > 0 && w_first - a.window + 1 > 0) ? w_first - a.window + 1 : 0);

    for (int blk = 0; blk < n_blocks; ++blk) {
        const int buf = blk & 1;
        if (blk + 1 < n_blocks) load_kv(blk + 1, buf ^ 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();

        const int kb = block_start(blk);
        const bool warp_active = qrow0 < rows && my_cols > 0 && kb <= w_last && (kb + BKEY - 1 >= w_lo || kb < keep);
        if (warp_active) {
            // ---- S = Q K^T : 16 x 32 per warp ---------------------------------------
            float s[BKEY / 8][4];
#pragma unroll
            for (int j = 0; j < BKEY / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll 4
            for (int ks = 0; ks < ks_n; ++ks) {
                uint32_t a0, a1, a2, a3;
                ldsm4(q_u + (qrow0 + (lane & 15)) * pk + (ks * 16 + (lane >> 4) * 8) * 2, a0, a1, a2, a3);
#pragma unroll
                for (int j = 0; j < BKEY / 16; ++j) {
                    uint32_t b0, b1, b2, b3;
                    const int krow = j * 16 + (lane & 7) + (lane >> 4) * 8;
                    ldsm4(k_u + (buf * BKEY + krow) * pk + (ks * 16 + ((lane >> 3) & 1) * 8) * 2, b0, b1, b2, b3);
                    mma16816(s[2 * j], a0, a1, a2, a3, b0, b1);
                    mma16816(s[2 * j + 1], a0, a1, a2, a3, b2, b3);
                }
            }
            // ---- scale, distance bias, mask by absolute position, online softmax (all in units of log2 e) ----
            float mx0 = -INFINITY, mx1 = -INFINITY;
            if (a.softcap > 0.f) {
                // the cap: c tanh(scale s / c), then in units of log2 e like the uncapped scores times scale_log2e
                const float back = a.cap_log2e / a.scale_log2e;
#pragma unroll
                for (int j = 0; j < BKEY / 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[j][e] = back * tanhf(s[j][e] * a.scale_over_cap);
                }
            }
#pragma unroll
            for (int j = 0; j < BKEY / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = kb + j * 8 + 2 * t4 + e;
                    s[j][e] = (key > hi0 || (key < lo0 && key >= keep)) ? -INFINITY
                                                          : fmaf(-sl0, (float)(p_row0 - key), s[j][e] * a.scale_log2e);
                    s[j][2 + e] = (key > hi1 || (key < lo1 && key >= keep)) ? -INFINITY
                                                              : fmaf(-sl1, (float)(p_row1 - key), s[j][2 + e] * a.scale_log2e);
                    mx0 = fmaxf(mx0, s[j][e]);
                    mx1 = fmaxf(mx1, s[j][2 + e]);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            // a row that sees no key yet keeps m = -inf: use 0 as the reference so that exp2 stays finite
            const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
            const float al0 = m0 == -INFINITY ? 0.f : exp2f(m0 - ref0);
            const float al1 = m1 == -INFINITY ? 0.f : exp2f(m1 - ref1);
            float sum0 = 0.f, sum1 = 0.f;
            uint32_t p[BKEY / 8][2];
#pragma unroll
            for (int j = 0; j < BKEY / 8; ++j) {
                const float e0 = exp2f(s[j][0] - ref0), e1 = exp2f(s[j][1] - ref0);
                const float e2 = exp2f(s[j][2] - ref1), e3 = exp2f(s[j][3] - ref1);
                sum0 += e0 + e1; sum1 += e2 + e3;
                p[j][0] = pack_bf16(e0, e1);
                p[j][1] = pack_bf16(e2, e3);
            }
            sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
            sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
            l0 = l0 * al0 + sum0; l1 = l1 * al1 + sum1;
            m0 = mn0; m1 = mn1;
#pragma unroll
            for (int i = 0; i < ON; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
            // ---- O += P V ------------------------------------------------------------
#pragma unroll
            for (int kk = 0; kk < BKEY / 16; ++kk) {
                const uint32_t a0 = p[2 * kk][0], a1 = p[2 * kk][1], a2 = p[2 * kk + 1][0], a3 = p[2 * kk + 1][1];
#pragma unroll
                for (int i = 0; i < ON / 2; ++i) {
                    if (i * 16 < my_cols) {
                        uint32_t b0, b1, b2, b3;
                        const int vrow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                        ldsm4t(v_u + (buf * BKEY + vrow) * pvv + (col0 + i * 16 + (lane >> 4) * 8) * 2, b0, b1, b2, b3);
                        mma16816(o[2 * i], a0, a1, a2, a3, b0, b1);
                        mma16816(o[2 * i + 1], a0, a1, a2, a3, b2, b3);
                    }
                }
            }
        }
        __syncthreads();   // everyone is done with this buffer before it is loaded again
    }
    cp_wait<0>();

    if (a.n_splits > 1) {
        // ---- this run's sums as they are, for the merge ------------------------------
        const long row0 = ((long)tok0 * a.n_heads + head0 + min(r0, rows - 1)) * a.n_splits + blockIdx.z;
        const long row1 = ((long)tok0 * a.n_heads + head0 + min(r1, rows - 1)) * a.n_splits + blockIdx.z;
        if (part == 0 && t4 == 0 && qrow0 < rows) {
            if (r0 < rows) { a.part_ml[row0 * 2] = m0; a.part_ml[row0 * 2 + 1] = l0; }
            if (r1 < rows) { a.part_ml[row1 * 2] = m1; a.part_ml[row1 * 2 + 1] = l1; }
        }
#pragma unroll
        for (int i = 0; i < ON; ++i) {
            const int col = i * 8 + 2 * t4;
            if (col < my_cols) {
                if (r0 < rows) *reinterpret_cast<float2*>(a.part_o + row0 * a.value_dim + col0 + col) = make_float2(o[i][0], o[i][1]);
                if (r1 < rows) *reinterpret_cast<float2*>(a.part_o + row1 * a.value_dim + col0 + col) = make_float2(o[i][2], o[i][3]);
            }
        }
        return;
    }
    // ---- normalise and store ---------------------------------------------------------
    float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    if (a.sinks) {
        // the head's sink in the denominator, once: sums and maximum brought to the larger of the two references
        const float k0 = a.sinks[head0 + min(r0, rows - 1) % n_h] * 1.4426950408889634f;
        const float k1 = a.sinks[head0 + min(r1, rows - 1) % n_h] * 1.4426950408889634f;
        if (l0 > 0.f) { const float mm = fmaxf(m0, k0), f = exp2f(m0 - mm); inv0 = f / (l0 * f + exp2f(k0 - mm)); }
        if (l1 > 0.f) { const float mm = fmaxf(m1, k1), f = exp2f(m1 - mm); inv1 = f / (l1 * f + exp2f(k1 - mm)); }
    }
    bf16* o0 = a.out + (long)(tok0 + min(r0, rows - 1) / n_h) * a.ldo + (long)(head0 + min(r0, rows - 1) % n_h) * a.ldoh + col0;
    bf16* o1 = a.out + (long)(tok0 + min(r1, rows - 1) / n_h) * a.ldo + (long)(head0 + min(r1, rows - 1) % n_h) * a.ldoh + col0;
#pragma unroll
    for (int i = 0; i < ON; ++i) {
        const int col = i * 8 + 2 * t4;
        if (col < my_cols) {
            if (r0 < rows) *reinterpret_cast<uint32_t*>(o0 + col) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
            if (r1 < rows) *reinterpret_cast<uint32_t*>(o1 + col) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
        }
    }
}

// One block a (token, head): the runs of a token's keys added up, each weighted by 2^(its maximum - the largest).
__global__ void general_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                     const int* __restrict__ positions, bf16* __restrict__ out, long ldo, long ldoh,
                                     int n_heads, int value_dim, int n_splits, int window, const float* __restrict__ sinks)
{
    fx_pdl_wait();
    const int tkn = blockIdx.x, h = blockIdx.y;
    const long base = ((long)tkn * n_heads + h) * n_splits;
    const int pos = positions[tkn];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    auto has_keys = [&](int s) { int b, e; fx_split_range(pos, lo, s, n_splits, 0, b, e); return b < e; };
    float mm = -INFINITY;
    for (int s = 0; s < n_splits; ++s)
        if (has_keys(s)) mm = fmaxf(mm, part_ml[(base + s) * 2]);
    float sunk = 0.f;        // the head's sink: a term of the denominator that no run holds
    if (sinks && mm != -INFINITY) {
        const float sk = sinks[h] * 1.4426950408889634f;
        mm = fmaxf(mm, sk);
        sunk = exp2f(sk - mm);
    }
    for (int e = threadIdx.x; e < value_dim; e += blockDim.x) {
        float ll = sunk, acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            if (!has_keys(s)) continue;
            const float ms = part_ml[(base + s) * 2];
            if (ms == -INFINITY) continue;
            const float w = exp2f(ms - mm);
            ll += part_ml[(base + s) * 2 + 1] * w;
            acc += part_o[(base + s) * value_dim + e] * w;
        }
        out[(long)tkn * ldo + (long)h * ldoh + e] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
    }
}

template <int DVMAX, int NSPLIT, int BKEY>
int launch(dim3 grid, size_t smem, cudaStream_t s, const GArgs& a)
{
    auto kern = general_attention_kernel<DVMAX, NSPLIT, BKEY>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    fx_launch_pdl(kern, grid, dim3(128 * NSPLIT), smem, s, a);
    if (a.n_splits > 1)
        fx_launch_pdl(general_merge_kernel, dim3(grid.x, a.n_heads), dim3(64), 0, s, (const float*)a.part_o,
                      (const float*)a.part_ml, a.positions, a.out, a.ldo, a.ldoh, a.n_heads, a.value_dim, a.n_splits,
                      a.window, a.sinks);
    return fx_launch_status();
}

}  // namespace

static size_t general_smem(int key_dim, int value_dim, int alias, int bkey)
{
    return (size_t)(BQ + 2 * bkey) * (key_dim * 2 + 16) + (alias ? 0 : (size_t)2 * bkey * (value_dim * 2 + 16));
}

// Keys a block of the loop: 64 where an SM then still holds three blocks of threads, else 32 (the kernel lives on
// the warps an SM holds: with 64 keys and two blocks an SM, rows of 192 + 128 elements took 1.6 times as long).
static int general_bkey(int key_dim, int value_dim, int alias)
{
    return general_smem(key_dim, value_dim, alias, 64) + 1024 <= 75 * 1024 ? 64 : 32;
}

// Whether fx_general_attention takes these sizes (the caller goes to fx_paged_attention_ex otherwise): 0, or how
// many of its blocks an SM holds.
extern "C" int fx_general_attention_ok(int key_dim, int value_dim, int alias)
{
    if (key_dim <= 0 || value_dim <= 0 || key_dim % 16 || value_dim % 16 || key_dim > 640 || value_dim > 512) return 0;
    const size_t smem = general_smem(key_dim, value_dim, alias, general_bkey(key_dim, value_dim, alias));
    if (smem > 220 * 1024) return 0;
    const int fit = (int)((227 * 1024) / (smem + 1024));
    return fit > 4 ? 4 : fit;
}

// items: int32 [n_items, 5] = (first flat token, tokens, entry, first query head, heads), heads of one kv head,
// tokens x heads <= 64; or nullptr: one token a tile, n_items = tokens.  bfloat16 only.
// softcap c > 0: the scaled scores pass through c tanh(s / c) before bias and softmax.  sinks (optional, one per
// head): exp(sinks[h]) joins the denominator once (with runs: in the merge).  value_share >= 1: that many consecutive
// key heads read one value head (value head = key head / value_share).
// kv_strides: nullptr for pages laid out [page][kv head][position][ld]; else (k page stride, k head stride, v page
// stride, v head stride) in elements, for keys and values that lie otherwise (rows of all heads side by side).
extern "C" int fx_general_attention(const void* q, long ldq, long ldqh, const void* k_pages, const void* v_pages, long ldk,
                                    long ldv, const long* kv_strides, const int* block_table, int table_width, int page_size,
                                    const int* positions, const int* token_seq, const int* seq_slot, const int* items,
                                    int n_items, void* out, long ldo, long ldoh, int n_heads, int n_kv_heads,
                                    int key_dim, int value_dim, int window, float scale, const float* slopes,
                                    int n_splits, float* part_o, float* part_ml, int keep_first, float softcap,
                                    const float* sinks, int value_share, void* stream)
{
    if (n_items <= 0) return FX_OK;
    if (value_share < 1) value_share = 1;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads || n_kv_heads % value_share) return FX_ERR_SIZE;
    const long kps = kv_strides ? kv_strides[0] : (long)n_kv_heads * page_size * ldk, khs = kv_strides ? kv_strides[1] : (long)page_size * ldk;
    const long vps = kv_strides ? kv_strides[2] : (long)(n_kv_heads / value_share) * page_size * ldv, vhs = kv_strides ? kv_strides[3] : (long)page_size * ldv;
    const int alias = v_pages == k_pages && ldv == ldk && kps == vps && khs == vhs && value_dim <= key_dim;
    if (!fx_general_attention_ok(key_dim, value_dim, alias)) return FX_ERR_SIZE;
    if (kps % 8 || khs % 8 || vps % 8 || vhs % 8) return FX_ERR_ALIGN;
    if (ldq % 8 || ldqh % 8 || ldk % 8 || ldv % 8 || ldo % 2 || ldoh % 2 || (uintptr_t)q % 16 || (uintptr_t)k_pages % 16 ||
        (uintptr_t)v_pages % 16 || (uintptr_t)out % 4)
        return FX_ERR_ALIGN;
    GArgs a;
    a.q = (const bf16*)q; a.ldq = ldq; a.ldqh = ldqh;
    a.k_pages = (const bf16*)k_pages; a.v_pages = (const bf16*)v_pages; a.ldk = ldk; a.ldv = ldv;
    a.k_page_stride = kps; a.k_head_stride = khs; a.v_page_stride = vps; a.v_head_stride = vhs;
    a.block_table = block_table; a.table_width = table_width; a.page_size = page_size;
    a.positions = positions; a.token_seq = token_seq; a.seq_slot = seq_slot; a.items = items;
    a.out = (bf16*)out; a.ldo = ldo; a.ldoh = ldoh;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.key_dim = key_dim; a.value_dim = value_dim; a.window = window;
    a.keep_first = (window > 0 && keep_first > 0) ? keep_first : 0;
    a.scale_log2e = scale * 1.4426950408889634f; a.slopes = slopes; a.alias = alias;
    a.softcap = softcap > 0.f ? softcap : 0.f;
    a.cap_log2e = a.softcap * 1.4426950408889634f; a.scale_over_cap = a.softcap > 0.f ? scale / a.softcap : 0.f;
    a.sinks = sinks; a.value_share = value_share;
    a.n_splits = n_splits > 1 ? n_splits : 1; a.part_o = part_o; a.part_ml = part_ml;
    if (a.n_splits > 1 && (items || !part_o || !part_ml || a.n_splits > 65535)) return FX_ERR_SIZE;
    const int bkey = general_bkey(key_dim, value_dim, alias);
    const size_t smem = general_smem(key_dim, value_dim, alias, bkey);
    const int group = n_heads / n_kv_heads;
    dim3 grid = items ? dim3(n_items) : dim3(n_items, n_kv_heads * ((group + BQ - 1) / BQ), a.n_splits);
    cudaStream_t s = (cudaStream_t)stream;
    if (value_dim <= 64) { a.part_cols = 64; return bkey == 64 ? launch<64, 1, 64>(grid, smem, s, a) : launch<64, 1, 32>(grid, smem, s, a); }
    if (value_dim <= 128) { a.part_cols = 128; return bkey == 64 ? launch<128, 1, 64>(grid, smem, s, a) : launch<128, 1, 32>(grid, smem, s, a); }
    a.part_cols = ((value_dim / 2 + 15) / 16) * 16;
    if (value_dim <= 256) return bkey == 64 ? launch<128, 2, 64>(grid, smem, s, a) : launch<128, 2, 32>(grid, smem, s, a);
    return launch<256, 2, 32>(grid, smem, s, a);
}
