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
// meets another: a group of R lanes owns one column for the whole step, its rows in registers (in runs of four);
// every lane also carries the rows of n that match its rows of S, so that n . q comes out of the
// same pass.  n and m are the same for every column; so that no block reads what another has already moved on,
// each block of columns (blockIdx.z) keeps a copy of its own of both in the state: n [slots, H, Z, D] and
// m [slots, H, Z] with Z = fx_mlstm_column_blocks(D, V), all copies equal.  Tokens are
// staged CH at a time in shared memory (the next chunk's rows travel into registers meanwhile).  A fifth warp owns no
// column: a chunk ahead of the others it works out the gates (a lane a token), runs the chain of maxima over
// shuffles and takes the three exponentials of every token, so that the loop over the tokens holds multiply-adds
// only and never waits for a transcendental; the read-outs' reductions over a
// column's lanes are made for the whole chunk together.  Everything is 32-bit; the products that made q, k, v and the gates' inputs
// were written in 32 bits.
//
// State layout: S [slots, H, V, D] (column by column), n [slots, H, Z, D], m [slots, H, Z]; zeroed at admission.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int ML_THREADS = 128;               // threads that own state columns
constexpr int ML_BLOCK = ML_THREADS + 32;     // and one more warp that works out the gates a chunk ahead
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

// Rows in runs of four: lane p of a column holds rows 4 R (i / 4) + 4 p + (i % 4), i < RPL, so that k and q are
// read from shared memory in conflict-free 16-byte pieces.  DP = R * RPL >= D is the padded height (zeros beyond D).
// PRE: elements of every k and q row of the next chunk that a thread brings into registers while this chunk is
// worked on (1: DP <= 128, 2: DP <= 256); 0: the rows are read when they are staged.
template <int RPL, int PRE>
__global__ void __launch_bounds__(ML_BLOCK) mlstm_scan_kernel(const MlstmArgs a)
{
    __shared__ __align__(16) float k_s[CH][MAX_D];
    __shared__ __align__(16) float q_s[CH][MAX_D];
    __shared__ float v_s[CH][ML_THREADS];
    __shared__ float keep_s[2][CH], take_s[2][CH], floor_s[2][CH];      // two chunks: the gate warp runs one ahead
    __shared__ float num_s[CH][ML_THREADS], den_s[CH][ML_THREADS];      // a thread's partial read-outs of the chunk
    fx_pdl_wait_only();
    const int b = blockIdx.x, h = blockIdx.y;
    const int R = a.R, cols = ML_THREADS / R;
    const int part = threadIdx.x % R, cl = threadIdx.x / R;
    const int col0 = blockIdx.z * cols, col = col0 + cl;
    const int r0 = first_row_of(a.token_seq, a.n_tokens, b), r1 = first_row_of(a.token_seq, a.n_tokens, b + 1);
    if (r1 <= r0) return;
    const int D = a.D, V = a.V, H = a.H, DP = R * RPL;
    const bool worker = threadIdx.x < ML_THREADS;      // the last warp owns no column
    const bool live = worker && col < V;
    const long slot = a.seq_slot[b];
    float* sp = a.S + ((slot * H + h) * V + (live ? col : 0)) * D;
    const long copy = (slot * H + h) * gridDim.z + blockIdx.z;      // this block's copy of n and m
    float* np = a.n + copy * D;
    float S[RPL], N[RPL];
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
        const int row = (i >> 2) * 4 * R + part * 4 + (i & 3);
        S[i] = (live && row < D) ? sp[row] : 0.f;
        N[i] = (worker && row < D) ? np[row] : 0.f;
    }
    float m_run = a.m[copy];      // the running maximum (the gate warp moves it on and writes it back)
    const float bi = load_any(a.i_bias, a.bias_dtype, h), bf = load_any(a.f_bias, a.bias_dtype, h);
    const float inv_cap = 1.0f / a.cap;
    const float* Kp = a.k + (long)h * D;
    const float* Qp = a.q + (long)h * D;
    const float* Vp = a.v + (long)h * V + col0;

    // what a thread brings of a chunk: elements t and t + 128 of every token's k and q row, two of the chunk's
    // values, and (threads below CH) one token's gate inputs; all loads are unconditional, from indices clamped into
    // the chunk, so that they are issued together
    float kr[PRE ? PRE * CH : 1], qr[PRE ? PRE * CH : 1], vr[2], gir = 0.f, gfr = 0.f;
    const int i0 = min((int)threadIdx.x, D - 1), i1 = min((int)threadIdx.x + ML_THREADS, D - 1);
    auto fetch = [&](int c0, int nt) {
        if (PRE) {
#pragma unroll
            for (int tt = 0; tt < CH; ++tt) {
                const long t = c0 + min(tt, nt - 1);
                kr[tt] = __ldg(Kp + t * a.ldk + i0);
                qr[tt] = __ldg(Qp + t * a.ldq + i0);
            }
            if (PRE == 2) {
#pragma unroll
                for (int tt = 0; tt < CH; ++tt) {
                    const long t = c0 + min(tt, nt - 1);
                    kr[CH + tt] = __ldg(Kp + t * a.ldk + i1);
                    qr[CH + tt] = __ldg(Qp + t * a.ldq + i1);
                }
            }
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int idx = min((int)threadIdx.x + e * ML_THREADS, nt * cols - 1);
            const int tt = idx / cols, c = min(idx - tt * cols, V - 1 - col0);
            vr[e] = __ldg(Vp + (long)(c0 + tt) * a.ldv + c);
        }
    };
    // The gate warp, a chunk ahead of the others: a lane a token works out the two gates, the chain of maxima runs over
    // shuffles, and a lane a token takes the three exponentials.
    auto gates_of = [&](int c0, int nt, int buf) {
        const int lane = threadIdx.x - ML_THREADS;
        const float* g = a.gates + (long)(c0 + min(lane, nt - 1)) * a.ldg;
        gir = __ldg(g + h);
        gfr = __ldg(g + H + h);
        const float gi = a.cap * tanhf((gir + bi) * inv_cap);
        const float gf = logsigmoid_f(a.cap * tanhf((gfr + bf) * inv_cap));
        float m = m_run, m_before = 0.f, m_after = 0.f;
        for (int tt = 0; tt < nt; ++tt) {
            const float f = __shfl_sync(0xffffffffu, gf, tt), i = __shfl_sync(0xffffffffu, gi, tt);
            const float mn = fmaxf(f + m, i);
            if (lane == tt) { m_before = m; m_after = mn; }
            m = mn;
        }
        m_run = m;
        if (lane < nt) {
            keep_s[buf][lane] = expf(gf + m_before - m_after);
            take_s[buf][lane] = expf(gi - m_after);
            floor_s[buf][lane] = expf(-m_after);
        }
    };
    if (worker) fetch(r0, min(CH, r1 - r0));
    else gates_of(r0, min(CH, r1 - r0), 0);
    for (int c0 = r0, buf = 0; c0 < r1; c0 += CH, buf ^= 1) {
        const int nt = min(CH, r1 - c0);
        __syncthreads();      // the chunk before is done with the staged rows; this chunk's gates are in place
        if (!worker) {
            // (the other warps stage and work on this chunk meanwhile; the buffer written now was last read in the
            // chunk before this one)
            __syncthreads();
            if (c0 + CH < r1) gates_of(c0 + CH, min(CH, r1 - c0 - CH), buf ^ 1);
            continue;
        }
        if (PRE) {
            const int i = threadIdx.x;
            if (i < DP) {
#pragma unroll
                for (int tt = 0; tt < CH; ++tt) {
                    k_s[tt][i] = i < D ? kr[tt] : 0.f;
                    q_s[tt][i] = i < D ? qr[tt] * a.q_scale : 0.f;
                }
            }
            if (PRE == 2 && i + ML_THREADS < DP) {
#pragma unroll
                for (int tt = 0; tt < CH; ++tt) {
                    k_s[tt][i + ML_THREADS] = i + ML_THREADS < D ? kr[CH + tt] : 0.f;
                    q_s[tt][i + ML_THREADS] = i + ML_THREADS < D ? qr[CH + tt] * a.q_scale : 0.f;
                }
            }
        } else {
            for (int idx = threadIdx.x; idx < nt * DP; idx += ML_THREADS) {
                const int tt = idx / DP, i = idx - tt * DP;
                k_s[tt][i] = i < D ? Kp[(long)(c0 + tt) * a.ldk + i] : 0.f;
                q_s[tt][i] = i < D ? Qp[(long)(c0 + tt) * a.ldq + i] * a.q_scale : 0.f;
            }
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int idx = threadIdx.x + e * ML_THREADS;
            if (idx < nt * cols) {
                const int tt = idx / cols, c = idx - tt * cols;
                v_s[tt][c] = col0 + c < V ? vr[e] : 0.f;
            }
        }
        __syncthreads();
        if (c0 + CH < r1) fetch(c0 + CH, min(CH, r1 - c0 - CH));
        // (the loop over the tokens is not unrolled: its body is the whole column's update, and eight copies of
        // it do not fit the instruction cache)
#pragma unroll 1
        for (int tt = 0; tt < nt; ++tt) {
            {
                const float keep = keep_s[buf][tt], take = take_s[buf][tt], tv = take * v_s[tt][cl];
                // (four partial sums a dot product: the chain of dependent additions is a quarter as long)
                float n0 = 0.f, n1 = 0.f, n2 = 0.f, n3 = 0.f, d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
                for (int i = 0; i < RPL; i += 4) {
                    const int at = (i >> 2) * 4 * R + part * 4;
                    const float4 kk = *reinterpret_cast<const float4*>(&k_s[tt][at]);
                    const float4 qq = *reinterpret_cast<const float4*>(&q_s[tt][at]);
                    S[i] = fmaf(kk.x, tv, keep * S[i]);             N[i] = fmaf(take, kk.x, keep * N[i]);
                    S[i + 1] = fmaf(kk.y, tv, keep * S[i + 1]);     N[i + 1] = fmaf(take, kk.y, keep * N[i + 1]);
                    S[i + 2] = fmaf(kk.z, tv, keep * S[i + 2]);     N[i + 2] = fmaf(take, kk.z, keep * N[i + 2]);
                    S[i + 3] = fmaf(kk.w, tv, keep * S[i + 3]);     N[i + 3] = fmaf(take, kk.w, keep * N[i + 3]);
                    n0 = fmaf(S[i], qq.x, n0); n1 = fmaf(S[i + 1], qq.y, n1);
                    n2 = fmaf(S[i + 2], qq.z, n2); n3 = fmaf(S[i + 3], qq.w, n3);
                    d0 = fmaf(N[i], qq.x, d0); d1 = fmaf(N[i + 1], qq.y, d1);
                    d2 = fmaf(N[i + 2], qq.z, d2); d3 = fmaf(N[i + 3], qq.w, d3);
                }
                num_s[tt][threadIdx.x] = (n0 + n1) + (n2 + n3);
                den_s[tt][threadIdx.x] = (d0 + d1) + (d2 + d3);
            }
        }
        float num[CH], den[CH];
#pragma unroll
        for (int tt = 0; tt < CH; ++tt) { num[tt] = num_s[tt][threadIdx.x]; den[tt] = den_s[tt][threadIdx.x]; }   // (its own writes)
        // the read-outs of the chunk: all reductions over a column's lanes together, then the division
        for (int o = R >> 1; o > 0; o >>= 1) {
#pragma unroll
            for (int tt = 0; tt < CH; ++tt) {
                num[tt] += __shfl_xor_sync(0xffffffffu, num[tt], o);
                den[tt] += __shfl_xor_sync(0xffffffffu, den[tt], o);
            }
        }
        if (live && part == 0) {
#pragma unroll
            for (int tt = 0; tt < CH; ++tt)
                if (tt < nt)
                    a.out[(long)(c0 + tt) * a.ldo + (long)h * V + col] = num[tt] / (fmaxf(fabsf(den[tt]), floor_s[buf][tt]) + 1e-6f);
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
    if (worker && cl == 0) {
#pragma unroll
        for (int i = 0; i < RPL; ++i) {
            const int row = (i >> 2) * 4 * R + part * 4 + (i & 3);
            if (row < D) np[row] = N[i];
        }
    }
    if (threadIdx.x == ML_THREADS) a.m[copy] = m_run;
}

// rows a lane holds: a multiple of four
int rows_per_lane(int D, int R) { return (int)fx_cdiv(D, 4 * R) * 4; }

int lanes_for(int D)
{
    int R = 4;
    while (R < 32 && rows_per_lane(D, R) > 16) R <<= 1;
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
    const int rpl = rows_per_lane(D, a.R);
    if (rpl > 16) return FX_ERR_SIZE;
    const int dp = a.R * rpl;
    const int pre = dp <= ML_THREADS ? 1 : dp <= 2 * ML_THREADS ? 2 : 0;      // elements of a row a thread prefetches
    dim3 grid(n_entries, H, fx_mlstm_column_blocks(D, V));
    cudaStream_t s = (cudaStream_t)stream;
    // a prompt's recurrence starts on an empty device (see fx_launch_pdl_if); a decode step's is set up early
    const bool early = n_tokens < 8 * n_entries;
#define FX_GO(RPL)                                                                                                    \
    do {                                                                                                              \
        if (pre == 1) fx_launch_pdl_if(early, mlstm_scan_kernel<RPL, 1>, grid, ML_BLOCK, 0, s, a);                    \
        else if (pre == 2) fx_launch_pdl_if(early, mlstm_scan_kernel<RPL, 2>, grid, ML_BLOCK, 0, s, a);               \
        else fx_launch_pdl_if(early, mlstm_scan_kernel<RPL, 0>, grid, ML_BLOCK, 0, s, a);                             \
    } while (0)
    switch (rpl) {
        case 4: FX_GO(4); break;
        case 8: FX_GO(8); break;
        case 12: FX_GO(12); break;
        default: FX_GO(16); break;
    }
#undef FX_GO
    return fx_launch_status();
}
