// Mixers that carry a matrix state per head from token to token instead of reading old keys:
//
//   plain decay:  S <- d S + k v^T                      o = S^T q      (decayed linear attention)
//   delta rule:   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;   o = S^T q      (gated delta rule)
//
// S is [dim, vdim] per (request, head), 32-bit, in the cache manager's state slots, stored column by column
// ([vdim][dim]): a column of S never meets another column, so a thread group owns one column for a whole step and
// the tokens of a request are taken one after the other, in the same order of operations however the request was
// cut into steps.  Everything here is 32-bit CUDA-core arithmetic: the state, the decays and the dot products with
// the state are what the designs that use these mixers ask to be kept in 32 bits.
//
// Kernels: fx_delta_prep (short causal convolution + SiLU of the projected q, k, v rows with the convolution's tail
// from the state slot, unit length per head, the gates beta and g), fx_conv_tail_update (the last taps - 1 inputs of
// every request of the step become its new tail), fx_state_scan (the recurrences above), fx_gated_group_norm (RMS
// norm over groups of the read-out, times a weight, times an activation of a gate row).
//
// A step's tokens are flat rows sorted by entry (token_seq ascending); an entry's rows are found by binary search.
#include "common.cuh"
#include "api.h"

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

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

// ------------------------------------------------------------------------------------------------------------
// Gated delta rule, what comes before the recurrence.
//   proj row: [ q (G*D) | k (G*D) | v (H*V) | ... ]  as projected
//   conv: y[c] = sum_j w[c, j] x_{t - (taps-1-j)}[c]; inputs before the step come from tail[slot] ([taps-1][C],
//   oldest first; zeros at the start of a request)
//   out row (32-bit): [ q / |q| * D^-1/2 | k / |k| | v ]  after SiLU;  |x| = sqrt(sum x^2 + 1e-6) per head
//   beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias))   from ba = [ b (H) | a (H) ] (32-bit)
constexpr int MAX_TAPS = 16;

constexpr int PREP_THREADS = 256;

// Grid (tokens, units): unit u < 2G is one q or k head (convolution, SiLU, unit length); the units after them are
// slices of PREP_THREADS value channels; unit 0 also makes the token's gates.
template <typename T>
__global__ void __launch_bounds__(PREP_THREADS) delta_prep_kernel(
    const T* __restrict__ proj, long ldp, const void* __restrict__ conv_w, int cw_dtype, int taps,
    const float* tail, const float* __restrict__ ba, long ldba, const float* __restrict__ a_log,
    const float* __restrict__ dt_bias, const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
    float* __restrict__ out, float* __restrict__ beta, float* __restrict__ g, int G, int D, int H, int V,
    float* tail_new)
{
    extern __shared__ float row_s[];   // D floats
    __shared__ float scratch[33];
    fx_pdl_wait();
    const int t = blockIdx.x, u = blockIdx.y;
    const int C = 2 * G * D + H * V;
    const int b = token_seq[t];
    // how many rows before t belong to the same entry (at most taps - 1 matter)
    int own = 0;
    while (own < taps - 1 && t - own - 1 >= 0 && token_seq[t - own - 1] == b) ++own;
    const float* tl = tail + (long)seq_slot[b] * (taps - 1) * C;
    auto conv = [&](int c) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;          // this tap's input lies `back` tokens before t
            float x;
            if (back <= own) x = to_f32(proj[(long)(t - back) * ldp + c]);
            else x = tl[(long)(taps - 1 - (back - own)) * C + c];
            acc = fmaf(load_any(conv_w, cw_dtype, (long)c * taps + j), x, acc);
        }
        // tail_new (the caller's promise that every entry brings exactly one token): this thread is then the only
        // reader of the channel's tail in the whole step, and moves it on by the token's input itself
        if (tail_new && taps > 1) {
            float* tn = tail_new + (long)seq_slot[b] * (taps - 1) * C;
            for (int j = 0; j + 1 < taps - 1; ++j) tn[(long)j * C + c] = tn[(long)(j + 1) * C + c];
            tn[(long)(taps - 2) * C + c] = to_f32(proj[(long)t * ldp + c]);
        }
        return silu_f(acc);
    };
    float* o = out + (long)t * C;
    if (u < 2 * G) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < D; i += blockDim.x) { const float x = conv(u * D + i); row_s[i] = x; ss = fmaf(x, x, ss); }
        ss = block_sum(ss, scratch);
        float inv = 1.0f / sqrtf(ss + 1e-6f);
        if (u < G) inv *= 1.0f / sqrtf((float)D);
        for (int i = threadIdx.x; i < D; i += blockDim.x) o[u * D + i] = row_s[i] * inv;   // (its own writes)
    } else {
        const int c = 2 * G * D + (u - 2 * G) * PREP_THREADS + threadIdx.x;
        if (c < C) o[c] = conv(c);
    }
    if (u == 0) {
        for (int hd = threadIdx.x; hd < H; hd += blockDim.x) {
            const float* r = ba + (long)t * ldba;
            beta[(long)t * H + hd] = sigmoid_f(r[hd]);
            // The decay is raised to the power of the distance a memory travels: an error of one unit in its last
            // place grows a thousandfold over a thousand tokens.  Its three transcendental steps are therefore taken
            // in 64 bits and rounded once (a handful of values a token).
            const double sp = log1p(exp((double)(r[H + hd] + dt_bias[hd])));
            g[(long)t * H + hd] = (float)exp(-exp((double)a_log[hd]) * sp);
        }
    }
}

// The convolution's tail after the step: the last taps - 1 inputs of every entry, from its rows of this step and,
// where the entry brought fewer, from the old tail.  One block per entry; a thread reads all it needs of a channel
// before it writes.
template <typename T>
__global__ void __launch_bounds__(256) conv_tail_update_kernel(
    const T* __restrict__ proj, long ldp, int C, int taps, float* __restrict__ tail,
    const int* __restrict__ token_seq, const int* __restrict__ seq_slot, int n_tokens)
{
    fx_pdl_wait();
    const int b = blockIdx.x;
    const int r0 = first_row_of(token_seq, n_tokens, b), r1 = first_row_of(token_seq, n_tokens, b + 1);
    const int n = r1 - r0, keep = taps - 1;
    if (n <= 0) return;
    float* tl = tail + (long)seq_slot[b] * keep * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float v[MAX_TAPS];
        for (int j = 0; j < keep; ++j) {
            const int rel = n - keep + j;     // index among the entry's rows; negative: before the step
            v[j] = rel >= 0 ? to_f32(proj[(long)(r0 + rel) * ldp + c]) : tl[(long)(j + n) * C + c];
        }
        for (int j = 0; j < keep; ++j) tl[(long)j * C + c] = v[j];
    }
}

// ------------------------------------------------------------------------------------------------------------
// The recurrence.  Grid (entries, heads, column groups); 128 threads; R lanes share a column, each with RPL rows
// of it in registers (rows in runs of four: lane p of a column holds rows 4 R i + 4 p + {0..3}, so that shared
// memory is read in conflict-free 16-byte pieces and the state in contiguous ones).  Tokens are staged CH at a
// time in shared memory.
constexpr int SCAN_THREADS = 128;
constexpr int CH = 8;
constexpr int MAX_DP = 256;    // padded dim (R * RPL)

struct ScanArgs {
    const void *q, *k, *v;       // rows of q [G*D], k [G*D], v [H*V]
    long ldq, ldk, ldv;
    int dtype;                   // element type of q, k, v
    int act;                     // 1: SiLU applied when q, k, v are read
    const float* g;  long g_ld;  // decay of (token, head): g[t * g_ld + h]   (g_ld = 0: one per head)
    const float* beta;           // [T, H] (delta rule) or null
    float* state;                // [slots, H, V, D]
    float* out;  long ldo;       // [T, H*V]
    const int *token_seq, *seq_slot;
    int n_tokens, H, G, D, V, R;
};

template <typename T>
__device__ __forceinline__ float load_act(const void* p, long i, int act)
{
    const float x = to_f32(reinterpret_cast<const T*>(p)[i]);
    return act ? silu_f(x) : x;
}

template <int RPL, bool DELTA, typename T>
__global__ void __launch_bounds__(SCAN_THREADS) state_scan_kernel(const ScanArgs a)
{
    __shared__ __align__(16) float k_s[CH][MAX_DP];
    __shared__ __align__(16) float q_s[CH][MAX_DP];
    __shared__ float v_s[CH][SCAN_THREADS];
    __shared__ float g_s[CH], b_s[CH];
    __shared__ float rd_s[CH][SCAN_THREADS];
    fx_pdl_wait_only();    // the kernel after this one starts when the loop over the tokens is over
    const int b = blockIdx.x, h = blockIdx.y;
    const int R = a.R, cols = SCAN_THREADS / R;
    const int part = threadIdx.x % R, cl = threadIdx.x / R;
    const int col = blockIdx.z * cols + cl;
    const int col0 = blockIdx.z * cols;
    const int r0 = first_row_of(a.token_seq, a.n_tokens, b), r1 = first_row_of(a.token_seq, a.n_tokens, b + 1);
    if (r1 <= r0) return;
    const int D = a.D, V = a.V, DP = R * RPL;
    const int kvh = h / (a.H / a.G);
    const bool live = col < V;
    float* sp = a.state + (((long)a.seq_slot[b] * a.H + h) * V + (live ? col : 0)) * D;

    float S[RPL];
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
        const int row = (i >> 2) * 4 * R + part * 4 + (i & 3);
        S[i] = (live && row < D) ? sp[row] : 0.f;
    }

    // The next chunk's q, k, v rows, decays and gates travel into registers while this chunk is worked on (all
    // loads of a chunk are issued together: one trip to memory a chunk, hidden behind the arithmetic).  Token tt of
    // the chunk: thread i takes elements i and i + 128 of its k and q rows; every load is unconditional, from an
    // index clamped into the chunk, so that nothing keeps the compiler from issuing them all before the first is
    // used; what lies outside is never stored.
    constexpr int NV = CH * 32 / SCAN_THREADS;
    const T* Kp = reinterpret_cast<const T*>(a.k) + (long)kvh * D;
    const T* Qp = reinterpret_cast<const T*>(a.q) + (long)kvh * D;
    const T* Vp = reinterpret_cast<const T*>(a.v) + (long)h * V + col0;
    T kr[2 * CH], qr[2 * CH], vr[NV];
    float gr = 0.f, br = 1.f;
    const bool wide = DP > SCAN_THREADS;                       // rows of more than 128 elements: a second half
    const int i0 = min((int)threadIdx.x, D - 1), i1 = min((int)threadIdx.x + SCAN_THREADS, D - 1);
    const int cshift = 31 - __clz(cols);                       // cols is a power of two
    auto fetch = [&](int c0, int nt) {
#pragma unroll
        for (int tt = 0; tt < CH; ++tt) {
            const long t = c0 + min(tt, nt - 1);
            kr[tt] = __ldg(Kp + t * a.ldk + i0);
            qr[tt] = __ldg(Qp + t * a.ldq + i0);
        }
        if (wide) {
#pragma unroll
            for (int tt = 0; tt < CH; ++tt) {
                const long t = c0 + min(tt, nt - 1);
                kr[CH + tt] = __ldg(Kp + t * a.ldk + i1);
                qr[CH + tt] = __ldg(Qp + t * a.ldq + i1);
            }
        }
#pragma unroll
        for (int e = 0; e < NV; ++e) {
            const int idx = min((int)threadIdx.x + e * SCAN_THREADS, nt * cols - 1);
            const int tt = idx >> cshift, c = min(idx - (tt << cshift), V - 1 - col0);
            vr[e] = __ldg(Vp + (long)(c0 + tt) * a.ldv + c);
        }
        const long t = c0 + min((int)threadIdx.x, nt - 1);
        gr = __ldg(a.g + t * a.g_ld + h);
        if (DELTA) br = __ldg(a.beta + t * a.H + h);
    };
    auto widen = [&](T x) { const float f = to_f32(x); return a.act ? silu_f(f) : f; };
    auto stash = [&](int nt) {
        const int i = threadIdx.x;
        if (i < DP) {
#pragma unroll
            for (int tt = 0; tt < CH; ++tt) {
                k_s[tt][i] = i < D ? widen(kr[tt]) : 0.f;
                q_s[tt][i] = i < D ? widen(qr[tt]) : 0.f;
            }
        }
        if (wide && i + SCAN_THREADS < DP) {
#pragma unroll
            for (int tt = 0; tt < CH; ++tt) {
                k_s[tt][i + SCAN_THREADS] = i + SCAN_THREADS < D ? widen(kr[CH + tt]) : 0.f;
                q_s[tt][i + SCAN_THREADS] = i + SCAN_THREADS < D ? widen(qr[CH + tt]) : 0.f;
            }
        }
#pragma unroll
        for (int e = 0; e < NV; ++e) {
            const int idx = threadIdx.x + e * SCAN_THREADS;
            if (idx < nt * cols) {
                const int tt = idx >> cshift, c = idx - (tt << cshift);
                v_s[tt][c] = col0 + c < V ? widen(vr[e]) : 0.f;
            }
        }
        if (threadIdx.x < nt) { g_s[threadIdx.x] = gr; b_s[threadIdx.x] = br; }
    };
    fetch(r0, min(CH, r1 - r0));
    for (int c0 = r0; c0 < r1; c0 += CH) {
        const int nt = min(CH, r1 - c0);
        __syncthreads();             // the chunk before is done with the staged rows
        stash(nt);
        __syncthreads();
        if (c0 + CH < r1) fetch(c0 + CH, min(CH, r1 - c0 - CH));
        for (int tt = 0; tt < nt; ++tt) {
            const float gt = g_s[tt];
            float u = v_s[tt][cl];
            // (four partial sums a dot product: the chain of dependent additions is a quarter as long)
            if (DELTA) {
                float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
                for (int i = 0; i < RPL; i += 4) {
                    const float4 kk = *reinterpret_cast<const float4*>(&k_s[tt][(i >> 2) * 4 * R + part * 4]);
                    S[i] *= gt; S[i + 1] *= gt; S[i + 2] *= gt; S[i + 3] *= gt;
                    d0 = fmaf(S[i], kk.x, d0); d1 = fmaf(S[i + 1], kk.y, d1);
                    d2 = fmaf(S[i + 2], kk.z, d2); d3 = fmaf(S[i + 3], kk.w, d3);
                }
                float dot = (d0 + d1) + (d2 + d3);
                for (int o = R >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                u = b_s[tt] * (u - dot);
            }
            float r0s = 0.f, r1s = 0.f, r2s = 0.f, r3s = 0.f;
#pragma unroll
            for (int i = 0; i < RPL; i += 4) {
                const int at = (i >> 2) * 4 * R + part * 4;
                const float4 kk = *reinterpret_cast<const float4*>(&k_s[tt][at]);
                const float4 qq = *reinterpret_cast<const float4*>(&q_s[tt][at]);
                if (DELTA) {
                    S[i] = fmaf(kk.x, u, S[i]); S[i + 1] = fmaf(kk.y, u, S[i + 1]);
                    S[i + 2] = fmaf(kk.z, u, S[i + 2]); S[i + 3] = fmaf(kk.w, u, S[i + 3]);
                } else {
                    S[i] = fmaf(gt, S[i], kk.x * u); S[i + 1] = fmaf(gt, S[i + 1], kk.y * u);
                    S[i + 2] = fmaf(gt, S[i + 2], kk.z * u); S[i + 3] = fmaf(gt, S[i + 3], kk.w * u);
                }
                r0s = fmaf(S[i], qq.x, r0s); r1s = fmaf(S[i + 1], qq.y, r1s);
                r2s = fmaf(S[i + 2], qq.z, r2s); r3s = fmaf(S[i + 3], qq.w, r3s);
            }
            // this lane's share of the read-out; the lanes' shares are added up after the chunk, eight tokens'
            // reductions side by side, instead of one chain of shuffles in every token's way
            rd_s[tt][threadIdx.x] = (r0s + r1s) + (r2s + r3s);
        }
        float rd[CH];
#pragma unroll
        for (int tt = 0; tt < CH; ++tt) rd[tt] = rd_s[tt][threadIdx.x];     // (its own writes)
        for (int o = R >> 1; o > 0; o >>= 1) {
#pragma unroll
            for (int tt = 0; tt < CH; ++tt) rd[tt] += __shfl_xor_sync(0xffffffffu, rd[tt], o);
        }
        if (live && part == 0) {
#pragma unroll
            for (int tt = 0; tt < CH; ++tt)
                if (tt < nt) a.out[(long)(c0 + tt) * a.ldo + (long)h * V + col] = rd[tt];
        }
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

int g_scan_lanes = 0;

template <int RPL, typename T>
void launch_scan(const ScanArgs& a, int n_entries, cudaStream_t s)
{
    const int cols = SCAN_THREADS / a.R;
    dim3 grid(n_entries, a.H, (unsigned)fx_cdiv(a.V, cols));
    // a prompt's recurrence starts on an empty device (see fx_launch_pdl_if); a decode step's is set up early
    const bool early = a.n_tokens < 8 * (int)grid.x;
    if (a.beta) fx_launch_pdl_if(early, state_scan_kernel<RPL, true, T>, grid, SCAN_THREADS, 0, s, a);
    else fx_launch_pdl_if(early, state_scan_kernel<RPL, false, T>, grid, SCAN_THREADS, 0, s, a);
}

template <typename T>
int scan_for(const ScanArgs& a, int rpl, int n_entries, cudaStream_t s)
{
    switch (rpl) {
        case 4: launch_scan<4, T>(a, n_entries, s); break;
        case 8: launch_scan<8, T>(a, n_entries, s); break;
        case 12: launch_scan<12, T>(a, n_entries, s); break;
        case 16: launch_scan<16, T>(a, n_entries, s); break;
        case 20: launch_scan<20, T>(a, n_entries, s); break;
        case 24: launch_scan<24, T>(a, n_entries, s); break;
        case 28: launch_scan<28, T>(a, n_entries, s); break;
        case 32: launch_scan<32, T>(a, n_entries, s); break;
        default: return FX_ERR_SIZE;
    }
    return fx_launch_status();
}

// ------------------------------------------------------------------------------------------------------------
// out[t, grp, i] = x[t, grp, i] / sqrt(mean_i x^2 + eps) * w[grp * w_stride + i] * act(gate[t, grp, i]); act 0: SiLU,
// 1: sigmoid.  w_stride 0: the groups share one weight vector; width: a weight for every element of the row.
template <typename GT, typename OT>
__global__ void __launch_bounds__(128) gated_group_norm_kernel(
    const float* __restrict__ x, const GT* __restrict__ gate, long ldg, const void* __restrict__ w, int w_dtype,
    float eps, int act, OT* __restrict__ out, int groups, int width, long w_stride)
{
    __shared__ float scratch[33];
    fx_pdl_wait();
    const int t = blockIdx.x, grp = blockIdx.y;
    const float* xr = x + ((long)t * groups + grp) * width;
    const GT* gr = gate + (long)t * ldg + (long)grp * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    OT* o = out + ((long)t * groups + grp) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float gv = to_f32(gr[i]);
        o[i] = from_f32<OT>(xr[i] * inv * load_any(w, w_dtype, (long)grp * w_stride + i) * (act ? sigmoid_f(gv) : silu_f(gv)));
    }
}

// The same for narrow groups (up to 64 elements): a warp a group, four groups a block, no barrier.
template <typename GT, typename OT>
__global__ void __launch_bounds__(128) gated_group_norm_warp_kernel(
    const float* __restrict__ x, const GT* __restrict__ gate, long ldg, const void* __restrict__ w, int w_dtype,
    float eps, int act, OT* __restrict__ out, int groups, int width, long w_stride)
{
    fx_pdl_wait();
    const int t = blockIdx.x, grp = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (grp >= groups) return;
    const float* xr = x + ((long)t * groups + grp) * width;
    const GT* gr = gate + (long)t * ldg + (long)grp * width;
    float ss = 0.f;
    for (int i = lane; i < width; i += 32) ss = fmaf(xr[i], xr[i], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    OT* o = out + ((long)t * groups + grp) * width;
    for (int i = lane; i < width; i += 32) {
        const float gv = to_f32(gr[i]);
        o[i] = from_f32<OT>(xr[i] * inv * load_any(w, w_dtype, (long)grp * w_stride + i) * (act ? sigmoid_f(gv) : silu_f(gv)));
    }
}

}  // namespace

extern "C" int fx_delta_prep(const void* proj, int dtype, long ldp, const void* conv_w, int cw_dtype, int taps,
                             const float* tail, const float* ba, long ldba, const float* a_log, const float* dt_bias,
                             const int* token_seq, const int* seq_slot, float* out, float* beta, float* g,
                             int n_tokens, int G, int D, int H, int V, int update_tail, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (taps < 1 || taps > MAX_TAPS || G <= 0 || H % G || D <= 0 || D > 8192) return FX_ERR_SIZE;
    float* tail_new = update_tail ? const_cast<float*>(tail) : nullptr;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)D * 4;
    const long units = 2L * G + fx_cdiv((long)H * V, PREP_THREADS);
    if (units > 65535) return FX_ERR_SIZE;
    dim3 grid(n_tokens, (unsigned)units);
    if (dtype == FX_F32)
        fx_launch_pdl(delta_prep_kernel<float>, grid, PREP_THREADS, smem, s, (const float*)proj, ldp, conv_w, cw_dtype, taps,
                      tail, ba, ldba, a_log, dt_bias, token_seq, seq_slot, out, beta, g, G, D, H, V, tail_new);
    else if (dtype == FX_BF16)
        fx_launch_pdl(delta_prep_kernel<bf16>, grid, PREP_THREADS, smem, s, (const bf16*)proj, ldp, conv_w, cw_dtype, taps,
                      tail, ba, ldba, a_log, dt_bias, token_seq, seq_slot, out, beta, g, G, D, H, V, tail_new);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}

extern "C" int fx_conv_tail_update(const void* proj, int dtype, long ldp, int channels, int taps, float* tail,
                                   const int* token_seq, const int* seq_slot, int n_tokens, int n_entries, void* stream)
{
    if (n_tokens <= 0 || n_entries <= 0 || taps <= 1) return FX_OK;
    if (taps > MAX_TAPS) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FX_F32) fx_launch_pdl(conv_tail_update_kernel<float>, n_entries, 256, 0, s, (const float*)proj, ldp, channels, taps, tail, token_seq, seq_slot, n_tokens);
    else if (dtype == FX_BF16) fx_launch_pdl(conv_tail_update_kernel<bf16>, n_entries, 256, 0, s, (const bf16*)proj, ldp, channels, taps, tail, token_seq, seq_slot, n_tokens);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}

// Lanes that share a state column, fixed for measurements (0: chosen by the launcher); returns the old setting.
extern "C" int fx_set_scan_lanes(int lanes)
{
    const int was = g_scan_lanes;
    g_scan_lanes = lanes;
    return was;
}

// beta null: plain decay (g_ld may be 0: g holds one decay per head); else the delta rule.
extern "C" int fx_state_scan(const void* q, long ldq, const void* k, long ldk, const void* v, long ldv, int dtype, int act,
                             const float* g, long g_ld, const float* beta, float* state, float* out, long ldo,
                             const int* token_seq, const int* seq_slot, int n_tokens, int n_entries, int H, int G, int D,
                             int V, void* stream)
{
    if (n_tokens <= 0 || n_entries <= 0) return FX_OK;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0 || D > MAX_DP) return FX_ERR_SIZE;
    // lanes per column: at least 4, and enough for at most 32 rows a lane; rows a lane in steps of 4
    int R = 4;
    while ((D + R - 1) / R > 32) R *= 2;
    // Few requests leave most schedulers without a warp, and a warp alone issues an instruction every four cycles
    // (each waits for the one before): columns are then shared by more lanes (up to 16, at least 4 rows each), which
    // shortens every warp's chain and makes more warps, until there are three for every two schedulers (measured on a
    // B200, 16 heads of 128 x 128: one prompt of 2,048 tokens 1.2 ms a layer with 4 lanes, 0.95 with 8, 0.91 with 16;
    // four prompts of 512 tokens 0.37 ms with 4 lanes, 0.5 with 8).  Only the grouping of a dot product's partial
    // sums depends on it.
    auto warps = [&](int r) { return (long)n_entries * H * fx_cdiv(V, SCAN_THREADS / r) * (SCAN_THREADS / 32); };
    while (R < 16 && (D + 2 * R - 1) / (2 * R) >= 4 && warps(R) < 6L * fx_sm_count()) R *= 2;
    if (g_scan_lanes >= 4 && g_scan_lanes <= 32 && (D + g_scan_lanes - 1) / g_scan_lanes <= 32 &&
        (D + g_scan_lanes - 1) / g_scan_lanes >= 1 && (g_scan_lanes & (g_scan_lanes - 1)) == 0)
        R = g_scan_lanes;
    const int rpl = (((D + R - 1) / R) + 3) & ~3;
    ScanArgs a;
    a.q = q; a.k = k; a.v = v; a.ldq = ldq; a.ldk = ldk; a.ldv = ldv; a.dtype = dtype; a.act = act;
    a.g = g; a.g_ld = g_ld; a.beta = beta; a.state = state; a.out = out; a.ldo = ldo;
    a.token_seq = token_seq; a.seq_slot = seq_slot; a.n_tokens = n_tokens; a.H = H; a.G = G; a.D = D; a.V = V; a.R = R;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FX_F32) return scan_for<float>(a, rpl, n_entries, s);
    if (dtype == FX_BF16) return scan_for<bf16>(a, rpl, n_entries, s);
    return FX_ERR_DTYPE;
}

extern "C" int fx_gated_group_norm(const float* x, const void* gate, int gate_dtype, long ldg, const void* w, int w_dtype,
                                   float eps, int act, void* out, int out_dtype, int n_tokens, int groups, int width,
                                   long w_stride, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (groups <= 0 || width <= 0) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const bool narrow = width <= 64;
    dim3 grid(n_tokens, narrow ? (unsigned)fx_cdiv(groups, 4) : groups);
#define FX_GO(GT, OT)                                                                                                     \
    do {                                                                                                                  \
        if (narrow) fx_launch_pdl(gated_group_norm_warp_kernel<GT, OT>, grid, 128, 0, s, x, (const GT*)gate, ldg, w, w_dtype, \
                                  eps, act, (OT*)out, groups, width, w_stride);                                         \
        else fx_launch_pdl(gated_group_norm_kernel<GT, OT>, grid, 128, 0, s, x, (const GT*)gate, ldg, w, w_dtype, eps, act, \
                           (OT*)out, groups, width, w_stride);                                                          \
    } while (0)
    if (gate_dtype == FX_F32 && out_dtype == FX_F32) FX_GO(float, float);
    else if (gate_dtype == FX_F32 && out_dtype == FX_BF16) FX_GO(float, bf16);
    else if (gate_dtype == FX_BF16 && out_dtype == FX_BF16) FX_GO(bf16, bf16);
    else return FX_ERR_DTYPE;
#undef FX_GO
    return fx_launch_status();
}
