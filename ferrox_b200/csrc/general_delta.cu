// The generalized delta rule: per head a matrix state S [dim (keys), dim (values)] that every token decays channel by
// channel, from which it removes part of what its unit key reads, and to which it adds its key and value:
//
//   u = k / sqrt(sum k^2 + 1e-6)
//   S <- diag(w) S - (a * u) (u^T S) + k v^T          (both terms read the state of the token before)
//   o = S^T r
//
// with a decay w and a removal rate a per head and key channel.  A column of S (one value index) never meets another
// column: with d = u . S[:, j],  S[i, j] <- w_i S[i, j] - a_i u_i d + k_i v_j  and  o_j = S[:, j] . r.  So, as in the
// other state mixers (linear_state.cu), a group of R lanes owns one column for a whole step, with its rows in
// registers, and the tokens of a request are taken one after the other in the same order of operations however the
// request was cut into steps.  State [slots, H, dim (values), dim (keys)], 32-bit, column by column.  Everything here
// is 32-bit CUDA-core arithmetic: state, decays, rates, unit keys and the dot products with the state.
//
// fx_general_delta_prep makes u, a u and w of every (token, head) from the projections' 32-bit rows:
//   w = exp(-rate * sigmoid(W2 tanh(w1_out) + w0)),  a = sigmoid(a_pre + a_bias).
// fx_general_delta_scan runs the recurrence: grid (entries, heads, column groups), 128 threads; the tokens' rows
// (r, k, u, a u, w and the values of the block's columns) travel into shared memory eight tokens at a time by
// cp.async, the next chunk while this one is worked on.
#include "common.cuh"
#include "api.h"

namespace {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// first row r with token_seq[r] >= b
__device__ __forceinline__ int first_row_of(const int* __restrict__ token_seq, int n_tokens, int b)
{
    int lo = 0, hi = n_tokens;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (token_seq[mid] < b) lo = mid + 1; else hi = mid;
    }
    return lo;
}

constexpr int GP_THREADS = 128;
constexpr int GP_RC = 64;           // low-rank channels a pass
constexpr int GP_MAX_TT = 8;        // tokens a block
constexpr int GP_ITEMS = GP_MAX_TT * 256 / GP_THREADS;

constexpr int GP_LD = GP_RC + 4;    // floats between two rows of W2 in shared memory

// One block: `tt_n` tokens of one head.  The head's rows of W2 pass through shared memory GP_RC columns at a time
// (read along their rows, so the loads coalesce, and kept GP_RC + 4 floats apart, so that eight threads, one key
// channel each, read 16 bytes each from all 32 banks); every (token, channel) sums its products in the order of the
// low-rank index, whatever the block holds beside it.
__global__ void __launch_bounds__(GP_THREADS) general_delta_prep_kernel(
    const float* __restrict__ k, long ldk, const float* __restrict__ a_pre, long lda, const float* __restrict__ w1_out,
    long ldw1, const void* __restrict__ w2, int w2_dtype, const void* __restrict__ w0, int w0_dtype,
    const void* __restrict__ a_bias, int ab_dtype, float rate, float* __restrict__ u, float* __restrict__ au,
    float* __restrict__ w, int n_tokens, int H, int D, int rank, int tt_n)
{
    extern __shared__ __align__(16) float gp_s[];
    float* w2_s = gp_s;                              // [D][GP_LD]
    float* th_s = w2_s + D * GP_LD;                  // [tt_n][GP_RC]: tanh of the tokens' low-rank rows
    float* len_s = th_s + GP_MAX_TT * GP_RC;         // [tt_n]: the keys' lengths
    fx_pdl_wait();
    const int t0 = blockIdx.x * tt_n, h = blockIdx.y;
    const int nt = min(tt_n, n_tokens - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int tt = warp; tt < nt; tt += GP_THREADS / 32) {
        const float* kr = k + (long)(t0 + tt) * ldk + (long)h * D;
        float ss = 0.f;
        for (int i = lane; i < D; i += 32) ss = fmaf(kr[i], kr[i], ss);
        for (int x = 16; x > 0; x >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, x);
        if (lane == 0) len_s[tt] = sqrtf(ss + 1e-6f);
    }
    const int items = nt * D;
    const bool vec4 = rank % 4 == 0 && (uintptr_t)w2 % 16 == 0;
    float z[GP_ITEMS];
#pragma unroll
    for (int n = 0; n < GP_ITEMS; ++n) z[n] = 0.f;
    for (int rc0 = 0; rc0 < rank; rc0 += GP_RC) {
        const int nr = min(GP_RC, rank - rc0);
        __syncthreads();
        if (vec4) {     // four columns a load
            for (int idx = threadIdx.x; idx < D * (GP_RC / 4); idx += GP_THREADS) {
                const int i = idx / (GP_RC / 4), r = (idx - i * (GP_RC / 4)) * 4;
                const long at = ((long)h * D + i) * rank + rc0 + r;
                float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
                if (r < nr) {    // (nr is a multiple of 4 here)
                    if (w2_dtype == FX_F32) {
                        f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w2) + at);
                    } else {
                        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(w2) + at);
                        f.x = __uint_as_float(raw.x << 16); f.y = __uint_as_float(raw.x & 0xffff0000u);
                        f.z = __uint_as_float(raw.y << 16); f.w = __uint_as_float(raw.y & 0xffff0000u);
                    }
                }
                *reinterpret_cast<float4*>(w2_s + i * GP_LD + r) = f;
            }
        } else {
            for (int idx = threadIdx.x; idx < D * GP_RC; idx += GP_THREADS) {
                const int i = idx / GP_RC, r = idx - i * GP_RC;
                w2_s[i * GP_LD + r] = r < nr ? load_any(w2, w2_dtype, ((long)h * D + i) * rank + rc0 + r) : 0.f;
            }
        }
        for (int idx = threadIdx.x; idx < nt * GP_RC; idx += GP_THREADS) {
            const int tt = idx / GP_RC, r = idx - tt * GP_RC;
            th_s[idx] = r < nr ? tanhf(w1_out[(long)(t0 + tt) * ldw1 + rc0 + r]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int n = 0; n < GP_ITEMS; ++n) {
            const int idx = threadIdx.x + n * GP_THREADS;
            if (idx < items) {
                const int tt = idx / D, i = idx - tt * D;
                const float4* wr = reinterpret_cast<const float4*>(w2_s + i * GP_LD);
                const float4* tr = reinterpret_cast<const float4*>(th_s + tt * GP_RC);
                float acc = z[n];
                for (int r4 = 0; r4 < (nr + 3) >> 2; ++r4) {     // (zeros beyond nr in both rows)
                    const float4 ww = wr[r4], th = tr[r4];
                    acc = fmaf(ww.x, th.x, acc); acc = fmaf(ww.y, th.y, acc);
                    acc = fmaf(ww.z, th.z, acc); acc = fmaf(ww.w, th.w, acc);
                }
                z[n] = acc;
            }
        }
    }
#pragma unroll
    for (int n = 0; n < GP_ITEMS; ++n) {
        const int idx = threadIdx.x + n * GP_THREADS;
        if (idx < items) {
            const int tt = idx / D, i = idx - tt * D, c = h * D + i;
            const long t = t0 + tt;
            const float zz = z[n] + load_any(w0, w0_dtype, c);
            const float a = sigmoid_f(a_pre[t * lda + c] + load_any(a_bias, ab_dtype, c));
            const float uu = k[t * ldk + c] / len_s[tt];
            const long at = t * H * D + c;
            u[at] = uu;
            au[at] = a * uu;
            w[at] = expf(-rate * sigmoid_f(zz));
        }
    }
}

constexpr int GD_THREADS = 128;
constexpr int GD_CH = 8;       // tokens a chunk
constexpr int GD_MAX_D = 256;

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct GdArgs {
    const float* src[5];   // rows of r, k, u, a u, w: the head's D elements of token t at src[i] + t * ld[i] + h * D
    long ld[5];
    const float* v; long ldv;
    float* state;          // [slots, H, D, D]
    float* out; long ldo;  // [T, H * D]
    const int *token_seq, *seq_slot;
    int n_tokens, H, D, R;
    int vec;               // rows may be copied 16 bytes at a time
};

// Shared memory: two buffers of [5][GD_CH][DP] rows and [GD_CH][cols] values, then [GD_CH][128] read-out shares.
template <int RPL>
__global__ void __launch_bounds__(GD_THREADS) general_delta_scan_kernel(const GdArgs a)
{
    extern __shared__ __align__(16) float sm[];
    fx_pdl_wait_only();
    const int b = blockIdx.x, h = blockIdx.y;
    const int R = a.R, cols = GD_THREADS / R, D = a.D, DP = R * RPL;
    const int part = threadIdx.x % R, cl = threadIdx.x / R;
    const int col0 = blockIdx.z * cols, col = col0 + cl;
    const int r0 = first_row_of(a.token_seq, a.n_tokens, b), r1 = first_row_of(a.token_seq, a.n_tokens, b + 1);
    if (r1 <= r0) return;
    const bool live = col < D;
    float* sp = a.state + (((long)a.seq_slot[b] * a.H + h) * D + (live ? col : 0)) * D;
    const int buf_floats = GD_CH * (5 * DP + cols);
    float* rd_s = sm + 2 * buf_floats;
    const uint32_t sm_u = (uint32_t)__cvta_generic_to_shared(sm);

    float S[RPL];
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
        const int row = (i >> 2) * 4 * R + part * 4 + (i & 3);
        S[i] = (live && row < D) ? sp[row] : 0.f;
    }
    // what lies beyond the head's D rows and the block's live columns stays zero in both buffers
    for (int idx = threadIdx.x; idx < 2 * buf_floats; idx += GD_THREADS) sm[idx] = 0.f;
    __syncthreads();

    // Staging.  Thread t copies piece t, t + 128, ... of a chunk; a piece's (token, place in the row) moves on by the
    // same step every time, so the quotient and the remainder are taken once here and carried from piece to piece.
    const int pw = a.vec ? D >> 2 : D;                   // pieces a row: 16 bytes each, or one element
    const int p_tt0 = threadIdx.x / pw, p_i0 = threadIdx.x - p_tt0 * pw;
    const int p_dq = GD_THREADS / pw, p_dr = GD_THREADS - p_dq * pw;
    const int nc = min(cols, D - col0);                  // the block's live columns
    const int v_tt0 = threadIdx.x / nc, v_c0 = threadIdx.x - v_tt0 * nc;
    const int v_dq = GD_THREADS / nc, v_dr = GD_THREADS - v_dq * nc;
    const float* srcp[5];
#pragma unroll
    for (int arr = 0; arr < 5; ++arr) srcp[arr] = a.src[arr] + (long)h * D;
    const float* vp = a.v + (long)h * D + col0;
    auto issue = [&](int c0, int nt, int buf) {
        const uint32_t base = sm_u + (uint32_t)(buf * buf_floats) * 4u;
        for (int tt = p_tt0, i = p_i0; tt < nt;) {
            const int e = a.vec ? i * 4 : i;
#pragma unroll
            for (int arr = 0; arr < 5; ++arr) {
                const uint32_t dst = base + (uint32_t)((arr * GD_CH + tt) * DP + e) * 4u;
                const float* src = srcp[arr] + (long)(c0 + tt) * a.ld[arr] + e;
                if (a.vec) cp_async16(dst, src); else cp_async4(dst, src);
            }
            tt += p_dq; i += p_dr;
            if (i >= pw) { i -= pw; ++tt; }
        }
        for (int tt = v_tt0, c = v_c0; tt < nt;) {
            cp_async4(base + (uint32_t)(5 * GD_CH * DP + tt * cols + c) * 4u, vp + (long)(c0 + tt) * a.ldv + c);
            tt += v_dq; c += v_dr;
            if (c >= nc) { c -= nc; ++tt; }
        }
    };

    issue(r0, min(GD_CH, r1 - r0), 0);
    cp_commit();
    int buf = 0;
    for (int c0 = r0; c0 < r1; c0 += GD_CH, buf ^= 1) {
        const int nt = min(GD_CH, r1 - c0);
        if (c0 + GD_CH < r1) {
            issue(c0 + GD_CH, min(GD_CH, r1 - c0 - GD_CH), buf ^ 1);
            cp_commit();
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        const float* bs = sm + buf * buf_floats;
        const float* r_s = bs;
        const float* k_s = bs + GD_CH * DP;
        const float* u_s = bs + 2 * GD_CH * DP;
        const float* au_s = bs + 3 * GD_CH * DP;
        const float* w_s = bs + 4 * GD_CH * DP;
        const float* v_s = bs + 5 * GD_CH * DP;
        for (int tt = 0; tt < nt; ++tt) {
            const int o = tt * DP;
            // d = u . S (the old state); four partial sums, then the column's lanes
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
            for (int i = 0; i < RPL; i += 4) {
                const float4 uu = *reinterpret_cast<const float4*>(&u_s[o + (i >> 2) * 4 * R + part * 4]);
                d0 = fmaf(S[i], uu.x, d0); d1 = fmaf(S[i + 1], uu.y, d1);
                d2 = fmaf(S[i + 2], uu.z, d2); d3 = fmaf(S[i + 3], uu.w, d3);
            }
            float d = (d0 + d1) + (d2 + d3);
            for (int x = R >> 1; x > 0; x >>= 1) d += __shfl_xor_sync(0xffffffffu, d, x);
            const float vt = v_s[tt * cols + cl];
            float q0 = 0.f, q1 = 0.f, q2 = 0.f, q3 = 0.f;
#pragma unroll
            for (int i = 0; i < RPL; i += 4) {
                const int at = o + (i >> 2) * 4 * R + part * 4;
                const float4 ww = *reinterpret_cast<const float4*>(&w_s[at]);
                const float4 aa = *reinterpret_cast<const float4*>(&au_s[at]);
                const float4 kk = *reinterpret_cast<const float4*>(&k_s[at]);
                const float4 rr = *reinterpret_cast<const float4*>(&r_s[at]);
                S[i] = fmaf(ww.x, S[i], fmaf(-aa.x, d, kk.x * vt));
                S[i + 1] = fmaf(ww.y, S[i + 1], fmaf(-aa.y, d, kk.y * vt));
                S[i + 2] = fmaf(ww.z, S[i + 2], fmaf(-aa.z, d, kk.z * vt));
                S[i + 3] = fmaf(ww.w, S[i + 3], fmaf(-aa.w, d, kk.w * vt));
                q0 = fmaf(S[i], rr.x, q0); q1 = fmaf(S[i + 1], rr.y, q1);
                q2 = fmaf(S[i + 2], rr.z, q2); q3 = fmaf(S[i + 3], rr.w, q3);
            }
            // this lane's share of the read-out; the lanes' shares are added up after the chunk, eight tokens'
            // reductions side by side, instead of one chain of shuffles in every token's way
            rd_s[tt * GD_THREADS + threadIdx.x] = (q0 + q1) + (q2 + q3);
        }
        float rd[GD_CH];
#pragma unroll
        for (int tt = 0; tt < GD_CH; ++tt) rd[tt] = tt < nt ? rd_s[tt * GD_THREADS + threadIdx.x] : 0.f;   // (its own writes)
        for (int x = R >> 1; x > 0; x >>= 1) {
#pragma unroll
            for (int tt = 0; tt < GD_CH; ++tt) rd[tt] += __shfl_xor_sync(0xffffffffu, rd[tt], x);
        }
        if (live && part == 0) {
#pragma unroll
            for (int tt = 0; tt < GD_CH; ++tt)
                if (tt < nt) a.out[(long)(c0 + tt) * a.ldo + (long)h * D + col] = rd[tt];
        }
        __syncthreads();     // everyone is done with this buffer before the chunk after next is copied into it
    }
    fx_pdl_trigger();
    if (live) {
#pragma unroll
        for (int i = 0; i < RPL; ++i) {
            const int row = (i >> 2) * 4 * R + part * 4 + (i & 3);
            if (row < D) sp[row] = S[i];
        }
    }
}

template <int RPL>
int launch_gd(const GdArgs& a, int n_entries, cudaStream_t s)
{
    const int cols = GD_THREADS / a.R, DP = a.R * RPL;
    const size_t smem = ((size_t)2 * GD_CH * (5 * DP + cols) + GD_CH * GD_THREADS) * sizeof(float);
    auto kern = general_delta_scan_kernel<RPL>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(n_entries, a.H, (unsigned)fx_cdiv(a.D, cols));
    // a prompt's recurrence starts on an empty device (see fx_launch_pdl_if); a decode step's is set up early
    fx_launch_pdl_if(a.n_tokens < 8 * n_entries, kern, grid, dim3(GD_THREADS), smem, s, a);
    return fx_launch_status();
}

}  // namespace

extern "C" int fx_general_delta_prep(const float* k, long ldk, const float* a_pre, long lda, const float* w1_out,
                                     long ldw1, const void* w2, int w2_dtype, const void* w0, int w0_dtype,
                                     const void* a_bias, int ab_dtype, float rate, float* u, float* au, float* w,
                                     int n_tokens, int H, int D, int rank, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (H <= 0 || H > 65535 || D <= 0 || D > GD_MAX_D || rank <= 0) return FX_ERR_SIZE;
    // few tokens (a decode step): a block a token, so that every head's slice of W2 is read by as many blocks as there
    // are tokens and the step is spread over the device; many: eight tokens share one reading of the slice
    const int tt_n = n_tokens >= 64 ? GP_MAX_TT : 1;
    const size_t smem = ((size_t)D * GP_LD + GP_MAX_TT * GP_RC + GP_MAX_TT) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(general_delta_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    fx_launch_pdl(general_delta_prep_kernel, dim3((unsigned)fx_cdiv(n_tokens, tt_n), H), dim3(GP_THREADS), smem,
                  (cudaStream_t)stream, k, ldk, a_pre, lda, w1_out, ldw1, w2, w2_dtype, w0, w0_dtype, a_bias, ab_dtype, rate,
                  u, au, w, n_tokens, H, D, rank, tt_n);
    return fx_launch_status();
}

extern "C" int fx_general_delta_scan(const float* r, long ldr, const float* k, long ldk, const float* v, long ldv,
                                     const float* u, const float* au, const float* w, float* state, float* out, long ldo,
                                     const int* token_seq, const int* seq_slot, int n_tokens, int n_entries, int H, int D,
                                     void* stream)
{
    if (n_tokens <= 0 || n_entries <= 0) return FX_OK;
    if (H <= 0 || H > 65535 || D <= 0 || D > GD_MAX_D) return FX_ERR_SIZE;
    // lanes per column: at least 4, and enough for at most 32 rows a lane; few requests leave most schedulers without
    // a warp, so columns are then shared by more lanes (shorter chains, more warps), as in fx_state_scan
    int R = 4;
    while ((D + R - 1) / R > 32) R *= 2;
    auto warps = [&](int rr) { return (long)n_entries * H * fx_cdiv(D, GD_THREADS / rr) * (GD_THREADS / 32); };
    while (R < 16 && (D + 2 * R - 1) / (2 * R) >= 4 && warps(R) < 6L * fx_sm_count()) R *= 2;
    const int rpl = (((D + R - 1) / R) + 3) & ~3;
    GdArgs a;
    a.src[0] = r; a.src[1] = k; a.src[2] = u; a.src[3] = au; a.src[4] = w;
    a.ld[0] = ldr; a.ld[1] = ldk; a.ld[2] = a.ld[3] = a.ld[4] = (long)H * D;
    a.v = v; a.ldv = ldv; a.state = state; a.out = out; a.ldo = ldo;
    a.token_seq = token_seq; a.seq_slot = seq_slot; a.n_tokens = n_tokens; a.H = H; a.D = D; a.R = R;
    a.vec = D % 4 == 0 && ldr % 4 == 0 && ldk % 4 == 0;
    for (int i = 0; i < 5; ++i) a.vec = a.vec && (uintptr_t)a.src[i] % 16 == 0;
    cudaStream_t s = (cudaStream_t)stream;
    switch (rpl) {
        case 4: return launch_gd<4>(a, n_entries, s);
        case 8: return launch_gd<8>(a, n_entries, s);
        case 12: return launch_gd<12>(a, n_entries, s);
        case 16: return launch_gd<16>(a, n_entries, s);
        case 20: return launch_gd<20>(a, n_entries, s);
        case 24: return launch_gd<24>(a, n_entries, s);
        case 28: return launch_gd<28>(a, n_entries, s);
        case 32: return launch_gd<32>(a, n_entries, s);
        default: return FX_ERR_SIZE;
    }
}
