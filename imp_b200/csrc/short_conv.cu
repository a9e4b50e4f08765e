// A short causal convolution over time on each channel, added to its own input, and a normalised polynomial as
// activation.
//
//   add_conv    out[t, c] = x[t, c] + sum_j w[j, c] * x[t - taps + 1 + j, c]   (j < taps; the last tap is the token itself;
//               the weight is held tap by tap, [taps][C], so that neighbouring channels are neighbouring words)
//               Tokens before the step's portion come from the request's state, which holds its last taps - 1 inputs
//               ([slot][taps - 1][C] float32, the newest last, zeros at a request's start).  In a step of single tokens the
//               kernel also shifts the state; otherwise imp_gdr_conv_state follows (it must not run before every token of
//               the portion has read the old state).
//   polynorm    out[t, :] = a z / rms(z) + b z^2 / rms(z^2) + c z^3 / rms(z^3) + e, powers element by element,
//               rms(u) = sqrt(mean(u^2) + eps) over the row; the three sums and the result in 32-bit.
#include "common.cuh"

namespace {

constexpr int SC_BLOCK = 256;
constexpr int SC_MAX_TAPS = 64;

template <typename TA>
__global__ void __launch_bounds__(SC_BLOCK) add_conv_kernel(TA* __restrict__ out, const TA* __restrict__ x, int64_t ld, const float* __restrict__ w,
                                                            int taps, float* __restrict__ state, const int* __restrict__ seq_of_token,
                                                            const int* __restrict__ q_start, const int* __restrict__ slots, int n_seqs, int C,
                                                            int shift_state, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0 || seq >= n_seqs) {
        if (threadIdx.x == 0) imp_report(status, IMP_BAD_SEQUENCE);
        return;
    }
    const int start = q_start[seq];
    const int lt = (int)t - start;                       // the token's place in its portion
    float* st = state + (int64_t)slots[seq] * (taps - 1) * C;
    for (int c = blockIdx.y * SC_BLOCK + threadIdx.x; c < C; c += gridDim.y * SC_BLOCK) {
        const float own = to_float(x[t * ld + c]);
        float acc = own;
        for (int j = 0; j < taps; ++j) {
            const int s = lt - (taps - 1) + j;           // which input, counted from the portion's first token
            const float v = s >= 0 ? (j == taps - 1 ? own : to_float(x[(int64_t)(start + s) * ld + c])) : st[(int64_t)(taps - 1 + s) * C + c];
            acc = fmaf(w[(int64_t)j * C + c], v, acc);
        }
        out[t * (int64_t)C + c] = from_float<TA>(acc);
        if (shift_state) {                               // one token a sequence: this thread alone reads and writes its channel
            for (int i = 0; i + 1 < taps - 1; ++i) st[(int64_t)i * C + c] = st[(int64_t)(i + 1) * C + c];
            if (taps > 1) st[(int64_t)(taps - 2) * C + c] = own;
        }
    }
}


// Eight neighbouring channels a thread, 16-byte loads and stores (32 bytes where the type is float32): rows of the input, of
// the state and of the weight are all read as whole vectors.  C a multiple of 8, every row 16-byte aligned.
struct F8 {
    float v[8];
};
__device__ __forceinline__ F8 load8(const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    return F8{{a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w}};
}
__device__ __forceinline__ F8 load8(const __nv_bfloat16* p) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y)),
                 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.z)), d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.w));
    return F8{{a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y}};
}
__device__ __forceinline__ void store8(float* p, const F8& f) {
    *reinterpret_cast<float4*>(p) = make_float4(f.v[0], f.v[1], f.v[2], f.v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f.v[4], f.v[5], f.v[6], f.v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const F8& f) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f.v[0], f.v[1]), b = __floats2bfloat162_rn(f.v[2], f.v[3]), c = __floats2bfloat162_rn(f.v[4], f.v[5]),
                   d = __floats2bfloat162_rn(f.v[6], f.v[7]);
    uint4 u;
    u.x = *reinterpret_cast<uint32_t*>(&a), u.y = *reinterpret_cast<uint32_t*>(&b), u.z = *reinterpret_cast<uint32_t*>(&c), u.w = *reinterpret_cast<uint32_t*>(&d);
    *reinterpret_cast<uint4*>(p) = u;
}

template <typename TA>
__global__ void __launch_bounds__(SC_BLOCK) add_conv_vec_kernel(TA* __restrict__ out, const TA* __restrict__ x, int64_t ld, const float* __restrict__ w,
                                                                int taps, float* __restrict__ state, const int* __restrict__ seq_of_token,
                                                                const int* __restrict__ q_start, const int* __restrict__ slots, int n_seqs, int C,
                                                                int shift_state, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0 || seq >= n_seqs) {
        if (threadIdx.x == 0 && blockIdx.y == 0) imp_report(status, IMP_BAD_SEQUENCE);
        return;
    }
    const int c = (blockIdx.y * SC_BLOCK + threadIdx.x) * 8;
    if (c >= C) return;
    const int start = q_start[seq];
    const int lt = (int)t - start;
    float* st = state + (int64_t)slots[seq] * (taps - 1) * C;
    const F8 own = load8(x + t * ld + c);
    F8 acc = own;
    for (int j = 0; j < taps; ++j) {                     // j ascending, as in the kernel of single channels: the same sum
        const int s = lt - (taps - 1) + j;
        const F8 v = s >= 0 ? (j == taps - 1 ? own : load8(x + (int64_t)(start + s) * ld + c)) : load8(st + (int64_t)(taps - 1 + s) * C + c);
        const F8 wv = load8(w + (int64_t)j * C + c);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc.v[i] = fmaf(wv.v[i], v.v[i], acc.v[i]);
    }
    store8(out + t * (int64_t)C + c, acc);
    if (shift_state) {
        for (int i = 0; i + 1 < taps - 1; ++i) store8(st + (int64_t)i * C + c, load8(st + (int64_t)(i + 1) * C + c));
        if (taps > 1) store8(st + (int64_t)(taps - 2) * C + c, own);
    }
}

// Steps of several tokens a sequence: a thread walks SC_TOK neighbouring tokens of the step for its eight channels.  The rows it
// needs (the tokens' own and the TAPS - 1 before the first) are asked for at once and read once, the taps' weights stay in
// registers; a token near its portion's start takes the missing inputs from its request's state.  The sum runs over the taps in
// the order of the other forms.  TAPS at compile time, so that every row and weight has a register of its own.
constexpr int SC_TOK = 4;
template <typename TA, int TAPS>
__global__ void __launch_bounds__(SC_BLOCK) add_conv_tile_kernel(TA* __restrict__ out, const TA* __restrict__ x, int64_t ld, const float* __restrict__ w,
                                                                 const float* __restrict__ state, const int* __restrict__ seq_of_token,
                                                                 const int* __restrict__ q_start, const int* __restrict__ slots, int n_tokens, int n_seqs,
                                                                 int C, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = (blockIdx.y * SC_BLOCK + threadIdx.x) * 8;
    if (c >= C) return;
    const int t0 = blockIdx.x * SC_TOK;
    F8 rows[SC_TOK + TAPS - 1];
#pragma unroll
    for (int i = 0; i < SC_TOK + TAPS - 1; ++i) {
        const int r = t0 - (TAPS - 1) + i;
        if (r >= 0 && r < n_tokens) rows[i] = load8(x + (int64_t)r * ld + c);
    }
    F8 wv[TAPS];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wv[j] = load8(w + (int64_t)j * C + c);
#pragma unroll
    for (int i = 0; i < SC_TOK; ++i) {
        const int t = t0 + i;
        if (t < n_tokens) {
            const int seq = seq_of_token[t];
            if (seq < 0 || seq >= n_seqs) {
                if (threadIdx.x == 0 && blockIdx.y == 0) imp_report(status, IMP_BAD_SEQUENCE);
            } else {
                const int lt = t - q_start[seq];
                F8 acc = rows[i + TAPS - 1];
#pragma unroll
                for (int j = 0; j < TAPS; ++j) {
                    const int s = lt - (TAPS - 1) + j;     // s >= 0: row t - (TAPS - 1) + j of the step belongs to this sequence
                    F8 v = rows[i + j];
                    if (s < 0) v = load8(state + ((int64_t)slots[seq] * (TAPS - 1) + (TAPS - 1 + s)) * C + c);
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc.v[k] = fmaf(wv[j].v[k], v.v[k], acc.v[k]);
                }
                store8(out + (int64_t)t * C + c, acc);
            }
        }
    }
}

template <typename TA>
static bool launch_conv_tile(void* out, const void* x, int64_t ld, const float* w, int taps, const float* state, const int* seq_of_token, const int* q_start,
                             const int* slots, int n_tokens, int n_seqs, int C, int* status, cudaStream_t s) {
    const dim3 grid((unsigned)((n_tokens + SC_TOK - 1) / SC_TOK), (unsigned)((C / 8 + SC_BLOCK - 1) / SC_BLOCK));
#define IMP_CONV_TILE(T)                                                                                                                          \
    case T:                                                                                                                                       \
        imp_launch(add_conv_tile_kernel<TA, T>, grid, dim3(SC_BLOCK), 0, s, (TA*)out, (const TA*)x, ld, w, state, seq_of_token, q_start, slots, \
                   n_tokens, n_seqs, C, status);                                                                                                  \
        return true
    switch (taps) {
        IMP_CONV_TILE(2);
        IMP_CONV_TILE(3);
        IMP_CONV_TILE(4);
        IMP_CONV_TILE(5);
        IMP_CONV_TILE(6);
        default: return false;
    }
#undef IMP_CONV_TILE
}

template <typename TA>
__global__ void __launch_bounds__(SC_BLOCK) polynorm_kernel(TA* __restrict__ out, const TA* __restrict__ z, int64_t ld, int n, const float* __restrict__ coef,
                                                            float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int64_t t = blockIdx.x;
    const TA* row = z + t * ld;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < n; i += SC_BLOCK) {
        const float v = to_float(row[i]), v2 = v * v;
        s2 += v2;
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v2 * v2, v2, s6);
    }
    const float a = coef[0] * rsqrtf(block_sum(s2, scratch) / (float)n + eps);
    const float b = coef[1] * rsqrtf(block_sum(s4, scratch) / (float)n + eps);
    const float c = coef[2] * rsqrtf(block_sum(s6, scratch) / (float)n + eps);
    const float e = coef[3];
    TA* orow = out + t * (int64_t)n;
    for (int i = threadIdx.x; i < n; i += SC_BLOCK) {
        const float v = to_float(row[i]);
        orow[i] = from_float<TA>(fmaf(v, fmaf(v, fmaf(v, c, b), a), e));    // a v + b v^2 + c v^3 + e
    }
}

}  // namespace

// x [T, ld] and out [T, C] dense, of the activation type; w float32 [taps, C]; state float32 [slots][taps - 1][C].
IMP_API int imp_add_conv(void* out, const void* x, int64_t ld, const float* w, int taps, float* state, const int* seq_of_token, const int* q_start,
                         const int* slots, int n_tokens, int n_seqs, int C, int shift_state, int dtype, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(out && x && w && seq_of_token && q_start && slots && C > 0 && ld >= C, "imp_add_conv: bad argument");
    IMP_CHECK_ARG(taps >= 1 && taps <= SC_MAX_TAPS && (taps == 1 || state), "imp_add_conv: 1 to %d taps, and a state where there is more than one", SC_MAX_TAPS);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t el = dtype == IMP_F32 ? 4 : 2;
    if (C % 8 == 0 && (ld * el) % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)state % 16 == 0) {
        if (!shift_state && n_tokens >= 64) {    // portions of prompts: the form that walks several tokens a thread
            const bool done = dtype == IMP_F32 ? launch_conv_tile<float>(out, x, ld, w, taps, state, seq_of_token, q_start, slots, n_tokens, n_seqs, C, status, s)
                                               : launch_conv_tile<__nv_bfloat16>(out, x, ld, w, taps, state, seq_of_token, q_start, slots, n_tokens, n_seqs, C,
                                                                                 status, s);
            if (done) IMP_RETURN_LAUNCH();
        }
        const dim3 vgrid((unsigned)n_tokens, (unsigned)((C / 8 + SC_BLOCK - 1) / SC_BLOCK));
        if (dtype == IMP_F32)
            imp_launch(add_conv_vec_kernel<float>, vgrid, dim3(SC_BLOCK), 0, s, (float*)out, (const float*)x, ld, w, taps, state, seq_of_token, q_start,
                       slots, n_seqs, C, shift_state, status);
        else
            imp_launch(add_conv_vec_kernel<__nv_bfloat16>, vgrid, dim3(SC_BLOCK), 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, ld, w, taps, state,
                       seq_of_token, q_start, slots, n_seqs, C, shift_state, status);
        IMP_RETURN_LAUNCH();
    }
    const dim3 grid((unsigned)n_tokens, (unsigned)std::min((C + SC_BLOCK - 1) / SC_BLOCK, 64));
    if (dtype == IMP_F32)
        imp_launch(add_conv_kernel<float>, grid, dim3(SC_BLOCK), 0, s, (float*)out, (const float*)x, ld, w, taps, state, seq_of_token, q_start, slots,
                   n_seqs, C, shift_state, status);
    else
        imp_launch(add_conv_kernel<__nv_bfloat16>, grid, dim3(SC_BLOCK), 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, ld, w, taps, state,
                   seq_of_token, q_start, slots, n_seqs, C, shift_state, status);
    IMP_RETURN_LAUNCH();
}

// z [T, ld], out [T, n] dense, of the activation type; coef float32 [4] = (a, b, c, e).
IMP_API int imp_polynorm(void* out, const void* z, int64_t ld, int n_tokens, int n, const float* coef, float eps, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(out && z && coef && n > 0 && ld >= n, "imp_polynorm: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == IMP_F32) imp_launch(polynorm_kernel<float>, dim3(n_tokens), dim3(SC_BLOCK), 0, s, (float*)out, (const float*)z, ld, n, coef, eps);
    else imp_launch(polynorm_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(SC_BLOCK), 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)z, ld, n, coef, eps);
    IMP_RETURN_LAUNCH();
}
