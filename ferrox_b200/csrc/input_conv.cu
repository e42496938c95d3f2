// A causal convolution over time on every channel of a mixer's input, added to the input itself:
//
//   out[t, c] = x[t, c] + sum_j w[c, j] * x[t - (taps - 1) + j, c]        (zeros before the request's start)
//
// (add_input = 0: the sum alone, for a convolution that stands in its input's place, as the one behind the
// projections of an attention mixer)
//
// over the tokens of one request.  The taps - 1 inputs before a step's first token come from the request's state
// slot (`tail` [slots, taps - 1, channels], 32-bit, oldest first), so a request may be cut into steps anywhere;
// after the step the last taps - 1 inputs of every entry become its tail (fx_conv_tail_update, linear_state.cu; a
// step of one token a request moves the tail on in this kernel).  The sum is 32-bit, taken in the order of the
// taps; the rows keep the element type of the mixer's input.
//
// Also here: the embedding with a learned position vector, the soft cap of the logits, the squared ReLU.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int CONV_THREADS = 256;
constexpr int CONV_MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(CONV_THREADS) input_conv_kernel(
    const T* __restrict__ x, long ldx, const void* __restrict__ w, int w_dtype, int taps, float* tail,
    const int* __restrict__ token_seq, const int* __restrict__ seq_slot, T* __restrict__ out, long ldo, int C,
    int update_tail, int add_input)
{
    fx_pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
    if (c >= C) return;
    const int b = token_seq[t];
    // how many rows before t belong to the same entry (at most taps - 1 matter)
    int own = 0;
    while (own < taps - 1 && t - own - 1 >= 0 && token_seq[t - own - 1] == b) ++own;
    float* tl = tail + (long)seq_slot[b] * (taps - 1) * C;
    const float xt = to_f32(x[(long)t * ldx + c]);
    float acc = add_input ? xt : 0.f;     // (a convolution that replaces its input: the sum alone)
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;          // this tap's input lies `back` tokens before t
        float v;
        if (back == 0) v = xt;
        else if (back <= own) v = to_f32(x[(long)(t - back) * ldx + c]);
        else v = tl[(long)(taps - 1 - (back - own)) * C + c];
        acc = fmaf(load_any(w, w_dtype, (long)c * taps + j), v, acc);
    }
    out[(long)t * ldo + c] = from_f32<T>(acc);
    // (the caller's promise that every entry brings exactly one token: this thread is then the only reader of the
    // channel's tail in the whole step, and moves it on by the token's input itself)
    if (update_tail && taps > 1) {
        for (int j = 0; j + 1 < taps - 1; ++j) tl[(long)j * C + c] = tl[(long)(j + 1) * C + c];
        tl[(long)(taps - 2) * C + c] = xt;
    }
}

template <typename T, typename PT>
__global__ void embed_pos_kernel(const T* __restrict__ table, const int* __restrict__ ids, const PT* __restrict__ pos_table,
                                 const int* __restrict__ positions, float* __restrict__ out, int hidden, int vocab,
                                 int n_positions, int* __restrict__ status)
{
    fx_pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t], p = positions[t];
    const bool ok = id >= 0 && id < vocab, pok = p >= 0 && p < n_positions;
    if (threadIdx.x == 0 && status) {
        if (!ok) atomicExch(status, 1);
        else if (!pok) atomicExch(status, 4);
    }
    const T* row = table + (long)(ok ? id : 0) * hidden;
    const PT* prow = pos_table + (long)(pok ? p : 0) * hidden;
    float* o = out + (long)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        o[i] = (ok && pok) ? to_f32(row[i]) + to_f32(prow[i]) : 0.f;
}

__global__ void softcap_kernel(float* __restrict__ x, long n, float cap)
{
    fx_pdl_wait();
    const float inv = 1.0f / cap;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}

template <typename T>
__global__ void relu_square_kernel(T* __restrict__ x, long ld, int n)
{
    fx_pdl_wait();
    T* r = x + (long)blockIdx.x * ld;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
        const float v = fmaxf(to_f32(r[i]), 0.f);
        r[i] = from_f32<T>(v * v);
    }
}

}  // namespace

extern "C" int fx_input_conv(const void* x, int dtype, long ldx, const void* w, int w_dtype, int taps, float* tail,
                             const int* token_seq, const int* seq_slot, void* out, long ldo, int n_tokens, int channels,
                             int update_tail, int add_input, void* stream)
{
    if (n_tokens <= 0 || channels <= 0) return FX_OK;
    if (taps < 1 || taps > CONV_MAX_TAPS || x == out) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, (unsigned)fx_cdiv(channels, CONV_THREADS));
    if (dtype == FX_F32)
        fx_launch_pdl(input_conv_kernel<float>, grid, CONV_THREADS, 0, s, (const float*)x, ldx, w, w_dtype, taps, tail,
                      token_seq, seq_slot, (float*)out, ldo, channels, update_tail, add_input);
    else if (dtype == FX_BF16)
        fx_launch_pdl(input_conv_kernel<bf16>, grid, CONV_THREADS, 0, s, (const bf16*)x, ldx, w, w_dtype, taps, tail,
                      token_seq, seq_slot, (bf16*)out, ldo, channels, update_tail, add_input);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}

extern "C" int fx_embed_pos(const void* table, int dtype, const int* ids, const void* pos_table, int pos_dtype,
                            const int* positions, float* out, int n_tokens, int hidden, int vocab, int n_positions,
                            int* status, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    cudaStream_t s = (cudaStream_t)stream;
    int nt = 32;
    while (nt < hidden && nt < 256) nt <<= 1;
#define FX_GO(T, PT)                                                                                                \
    fx_launch_pdl(embed_pos_kernel<T, PT>, n_tokens, nt, 0, s, (const T*)table, ids, (const PT*)pos_table, positions, \
                  out, hidden, vocab, n_positions, status)
    if (dtype == FX_F32 && pos_dtype == FX_F32) FX_GO(float, float);
    else if (dtype == FX_BF16 && pos_dtype == FX_BF16) FX_GO(bf16, bf16);
    else if (dtype == FX_F32 && pos_dtype == FX_BF16) FX_GO(float, bf16);
    else if (dtype == FX_BF16 && pos_dtype == FX_F32) FX_GO(bf16, float);
    else return FX_ERR_DTYPE;
#undef FX_GO
    return fx_launch_status();
}

extern "C" int fx_softcap(float* x, long n, float cap, void* stream)
{
    if (n <= 0) return FX_OK;
    if (!(cap > 0.f)) return FX_ERR_SIZE;
    long blocks = fx_cdiv(n, 256);
    if (blocks > 4096) blocks = 4096;
    fx_launch_pdl(softcap_kernel, (unsigned)blocks, 256, 0, (cudaStream_t)stream, x, n, cap);
    return fx_launch_status();
}

extern "C" int fx_relu_square(void* x, int dtype, long ld, int rows, int n, void* stream)
{
    if (rows <= 0 || n <= 0) return FX_OK;
    cudaStream_t s = (cudaStream_t)stream;
    long by = fx_cdiv(n, 256 * 4);
    if (by > 64) by = 64;
    dim3 grid(rows, (unsigned)by);
    if (dtype == FX_F32) fx_launch_pdl(relu_square_kernel<float>, grid, 256, 0, s, (float*)x, ld, n);
    else if (dtype == FX_BF16) fx_launch_pdl(relu_square_kernel<bf16>, grid, 256, 0, s, (bf16*)x, ld, n);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}
