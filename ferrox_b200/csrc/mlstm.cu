// The matrix memory of an mLSTM mixer: per (request, head) a state S [dim, vdim], a normaliser n [dim] and the
// running maximum m of the gates' logarithms,
//
//   i_t = cap tanh((i~_t + b_i) / cap)                     log input gate
//   f_t = logsigmoid(cap tanh((f~_t + b_f) / cap))         log forget gate
//   m_t = max(f_t + m_(t-1), i_t)                          (m starts at 0)
//   S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,    n_t likewise with k_t alone
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// over the tokens of every entry of the step, in order, whatever the cut.  A column of S (one value index) never
// meets another: a group of R lanes owns one column for the whole step, its rows in registers (lane p holds rows
// p, p + R, ...); every lane also carries the rows of n that match its rows of S, so that n . q comes out of the
// same pass.  n and m are the same for every column; so that no block reads what another has already moved on,
// each block of columns (blockIdx.z) keeps a copy of its own of both in the state: n [slots, H, Z, D] and
// m [slots, H, Z] with Z = fx_mlstm_column_blocks(D, V), all copies equal.  Tokens are
// staged CH at a time in shared memory: the gates of the chunk's tokens are worked out by one thread each, the
// chain of maxima by one thread, the three exponentials of a token by one thread each, so that the loop over the
// tokens holds multiply-adds only.  Everything is 32-bit; the products that made q, k, v and the gates' inputs
// were written in 32 bits.
//
// State layout: S [slots, H, V, D] (column by column), n [slots, H, Z, D], m [slots, H, Z]; zeroed at admission.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int ML_THREADS = 128;
constexpr int CH = 8;
constexpr int MAX_D = 512;

__device__ __forceinline__ int first_row_of(const int* __restrict__ token_seq, int n_tokens, int b)
{
    int lo = 0, hi = n_tokens;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (token_seq[mid] < b) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// log(sigmoid(x)) without overflow on either side
__device__ __forceinline__ float logsigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

struct MlstmArgs {
    const float *q, *k, *v;        // rows: q, k [H*D], v [H*V]
    long ldq, ldk, ldv;
    const float* gates; long ldg;  // gates[t * ldg + h] = i~, gates[t * ldg + H + h] = f~
    const void *i_bias, *f_bias; int bias_dtype;
    float cap, q_scale;
    float *S, *n, *m;
    float* out; long ldo;          // [T, H*V]
    const int *token_seq, *seq_slot;
    int n_tokens, H, D, V, R;
};

template <int RPL>
__global__ void __launch_bounds__(ML_THREADS) mlstm_scan_kernel(const MlstmArgs a)
{
    __shared__ float k_s[CH][MAX_D];
    __shared__ float q_s[CH][MAX_D];
    __shared__ float v_s[CH][ML_THREADS];
    __shared__ float gi_s[CH], gf_s[CH], keep_s[CH], take_s[CH], floor_s[CH], m_s[CH + 1];
    fx_pdl_wait_only();
    const int b = blockIdx.x, h = blockIdx.y;
    const int R = a.R, cols = ML_THREADS / R;
    const int part = threadIdx.x % R, cl = threadIdx.x / R;
    const int col0 = blockIdx.z * cols, col = col0 + cl;
    const int r0 = first_row_of(a.token_seq, a.n_tokens, b), r1 = first_row_of(a.token_seq, a.n_tokens, b + 1);
    if (r1 <= r0) return;
    const int D = a.D, V = a.V, H = a.H;
    const bool live = col < V;
    const long slot = a.seq_slot[b];
    float* sp = a.S + ((slot * H + h) * V + (live ? col : 0)) * D;
    const long copy = (slot * H + h) * gridDim.z + blockIdx.z;      // this block's copy of n and m
    float* np = a.n + copy * D;
    float S[RPL], N[RPL];
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
        const int row = part + i * R;
        S[i] = (live && row < D) ? sp[row] : 0.f;
        N[i] = row < D ? np[row] : 0.f;
    }
    if (threadIdx.x == 0) m_s[0] = a.m[copy];
    const float bi = load_any(a.i_bias, a.bias_dtype, h), bf = load_any(a.f_bias, a.bias_dtype, h);
    const float inv_cap = 1.0f / a.cap;

    for (int c0 = r0; c0 < r1; c0 += CH) {
        const int nt = min(CH, r1 - c0);
        __syncthreads();      // the chunk before is done with the staged rows (and m_s[0] is set)
        for (int idx = threadIdx.x; idx < nt * D; idx += ML_THREADS) {
            const int tt = idx / D, i = idx - tt * D;
            k_s[tt][i] = a.k[(long)(c0 + tt) * a.ldk + (long)h * D + i];
            q_s[tt][i] = a.q[(long)(c0 + tt) * a.ldq + (long)h * D + i] * a.q_scale;
        }
        for (int idx = threadIdx.x; idx < nt * cols; idx += ML_THREADS) {
            const int tt = idx / cols, c = idx - tt * cols;
            v_s[tt][c] = col0 + c < V ? a.v[(long)(c0 + tt) * a.ldv + (long)h * V + col0 + c] : 0.f;
        }
        if (threadIdx.x < nt) {
            const float* g = a.gates + (long)(c0 + threadIdx.x) * a.ldg;
            gi_s[threadIdx.x] = a.cap * tanhf((g[h] + bi) * inv_cap);
            gf_s[threadIdx.x] = logsigmoid_f(a.cap * tanhf((g[H + h] + bf) * inv_cap));
        }
        __syncthreads();
        if (threadIdx.x == 0) {      // the chain of maxima: an addition and a maximum a token
            float m = m_s[0];
            for (int tt = 0; tt < nt; ++tt) { m = fmaxf(gf_s[tt] + m, gi_s[tt]); m_s[tt + 1] = m; }
        }
        __syncthreads();
        if (threadIdx.x < nt) {
            const int tt = threadIdx.x;
            keep_s[tt] = expf(gf_s[tt] + m_s[tt] - m_s[tt + 1]);
            take_s[tt] = expf(gi_s[tt] - m_s[tt + 1]);
            floor_s[tt] = expf(-m_s[tt + 1]);
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float keep = keep_s[tt], take = take_s[tt], vj = v_s[tt][cl];
            float num = 0.f, den = 0.f;
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                const int row = part + i * R;      // rows beyond D hold zeros: their k and q are never read
                const float kk = row < D ? take * k_s[tt][row] : 0.f;
                const float qq = row < D ? q_s[tt][row] : 0.f;
                S[i] = fmaf(kk, vj, keep * S[i]);
                N[i] = fmaf(keep, N[i], kk);
                num = fmaf(S[i], qq, num);
                den = fmaf(N[i], qq, den);
            }
            for (int o = R >> 1; o > 0; o >>= 1) {
                num += __shfl_xor_sync(0xffffffffu, num, o);
                den += __shfl_xor_sync(0xffffffffu, den, o);
            }
            if (live && part == 0)
                a.out[(long)(c0 + tt) * a.ldo + (long)h * V + col] = num / (fmaxf(fabsf(den), floor_s[tt]) + 1e-6f);
        }
        __syncthreads();
        if (threadIdx.x == 0) m_s[0] = m_s[nt];
    }
    fx_pdl_trigger();
    if (live) {
#pragma unroll
        for (int i = 0; i < RPL; ++i) {
            const int row = part + i * R;
            if (row < D) sp[row] = S[i];
        }
    }
    if (cl == 0) {
#pragma unroll
        for (int i = 0; i < RPL; ++i) {
            const int row = part + i * R;
            if (row < D) np[row] = N[i];
        }
    }
    if (threadIdx.x == 0) a.m[copy] = m_s[0];
}

int lanes_for(int D)
{
    int R = 4;
    while (R < 32 && (D + R - 1) / R > 32) R <<= 1;
    return R;
}

}  // namespace

// Blocks of columns a head's state is shared out over (the copies of n and m the state keeps).
extern "C" int fx_mlstm_column_blocks(int D, int V)
{
    if (D <= 0 || V <= 0 || D > MAX_D) return 0;
    const int cols = ML_THREADS / lanes_for(D);
    return (V + cols - 1) / cols;
}

extern "C" int fx_mlstm_scan(const float* q, long ldq, const float* k, long ldk, const float* v, long ldv,
                             const float* gates, long ldg, const void* i_bias, const void* f_bias, int bias_dtype,
                             float cap, float q_scale, float* S, float* n, float* m, float* out, long ldo,
                             const int* token_seq, const int* seq_slot, int n_tokens, int n_entries, int H, int D,
                             int V, int copies, void* stream)
{
    if (n_tokens <= 0 || n_entries <= 0) return FX_OK;
    if (H <= 0 || D <= 0 || V <= 0 || D > MAX_D || !(cap > 0.f)) return FX_ERR_SIZE;
    if (copies != fx_mlstm_column_blocks(D, V)) return FX_ERR_SIZE;     // the state was laid out for another grid
    MlstmArgs a;
    a.q = q; a.k = k; a.v = v; a.ldq = ldq; a.ldk = ldk; a.ldv = ldv; a.gates = gates; a.ldg = ldg;
    a.i_bias = i_bias; a.f_bias = f_bias; a.bias_dtype = bias_dtype; a.cap = cap; a.q_scale = q_scale;
    a.S = S; a.n = n; a.m = m; a.out = out; a.ldo = ldo; a.token_seq = token_seq; a.seq_slot = seq_slot;
    a.n_tokens = n_tokens; a.H = H; a.D = D; a.V = V; a.R = lanes_for(D);
    const int rpl = (D + a.R - 1) / a.R;
    dim3 grid(n_entries, H, fx_mlstm_column_blocks(D, V));
    cudaStream_t s = (cudaStream_t)stream;
    // a prompt's recurrence starts on an empty device (see fx_launch_pdl_if); a decode step's is set up early
    const bool early = n_tokens < 8 * n_entries;
#define FX_GO(RPL) fx_launch_pdl_if(early, mlstm_scan_kernel<RPL>, grid, ML_THREADS, 0, s, a)
    if (rpl <= 4) FX_GO(4);
    else if (rpl <= 8) FX_GO(8);
    else if (rpl <= 12) FX_GO(12);
    else if (rpl <= 16) FX_GO(16);
    else if (rpl <= 24) FX_GO(24);
    else FX_GO(32);
#undef FX_GO
    return fx_launch_status();
}
