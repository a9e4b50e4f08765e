// The gated delta rule: a recurrent token mixer with one matrix state S [D, Dv] per head.
//
// Per token and value head h (reading the query / key head h / (H / G)):
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// with g in (0, 1) a decay and beta in (0, 1) a step size, both per head and token.  q, k and v come out
// of a short causal convolution over time per channel (taps - 1 earlier inputs are part of a request's
// state) followed by silu; q and k are then unit vectors per head and q carries D^(-1/2).
//
// Four kernels, all 32-bit arithmetic on 32-bit state whatever the activation type:
//   gdr_prepare     one warp per token and head: convolution + silu of its channels, unit q and k; beta and decay
//   gdr_conv_state  the last taps - 1 inputs of every sequence of the batch go to its state slot
//   gdr_scan        the recurrence; a CTA owns 32 value columns of one head of one sequence and walks
//                   the sequence's new tokens in order; eight lanes share a column, each holding an
//                   eighth of it in registers, so no state travels between tokens but through registers;
//                   the tokens' inputs arrive through a two-deep cp.async ring
//   gdr_output      per head: o / rms(o) * w * silu(gate)
// Every column of S evolves independently of the others, which is what the scan kernel's split rests on.
// A token's result depends on the tokens before it only through S and the convolution's inputs, and the
// order of every sum is fixed by the sizes alone: cutting a prompt into portions changes no bit.
#include <algorithm>

#include "common.cuh"

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ------------------------------------------------------------------------------------- prepare
// proj: [T, ld] activations, columns [q: G*D | k: G*D | v: H*Dv | gate: H*Dv | b: H | a: H].
// conv_w: [C, taps] float32 with C = 2*G*D + H*Dv (the last tap is the current token's).
// conv_state: [slots, taps - 1, C] float32: the inputs of the taps - 1 tokens before the portion.
// A warp makes one head of one token (a q head, a k head or a v head: convolution, silu, and for q and k the unit
// norm, summed inside the warp), or a token's H step sizes and decays; a CTA holds four warps and there are no
// block-wide steps, so a decode step of a few tokens still spreads over the device and a prompt's rows stream.
constexpr int GP_BLOCK = 128;
constexpr int GP_MAX_D = 256;

// TAPS: the convolution's taps at compile time (0: read from `taps_rt`), so that a channel's loads go out together.
template <typename TA, int TAPS>
__global__ void __launch_bounds__(GP_BLOCK) gdr_prepare_kernel(
    const TA* __restrict__ proj, int64_t ld, const float* __restrict__ conv_w, int taps_rt, float* __restrict__ conv_state,
    const int* __restrict__ seq_of_token, const int* __restrict__ q_start, const int* __restrict__ slots, int n_tokens, int n_seqs,
    int G, int D, int H, int Dv, const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* __restrict__ qn,
    float* __restrict__ kn, float* __restrict__ vc, float* __restrict__ beta, float* __restrict__ decay, int update_state, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int taps = TAPS ? TAPS : taps_rt;
    const int lane = threadIdx.x & 31;
    const int units = 2 * G + H + 1;
    const int64_t item = (int64_t)blockIdx.x * (GP_BLOCK / 32) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_tokens * units) return;
    const int t = (int)(item / units), unit = (int)(item - (int64_t)t * units);
    const int nqk = G * D, C = 2 * nqk + H * Dv;
    const int seq = seq_of_token[t];
    if (seq < 0 || seq >= n_seqs) {
        if (lane == 0 && unit == 0) imp_report(status, IMP_BAD_SEQUENCE);
        return;
    }
    if (unit == 2 * G + H) {
        for (int hh = lane; hh < H; hh += 32) {
            const TA* row = proj + (int64_t)t * ld + C + H * Dv;
            const float b = to_float(row[hh]), a = to_float(row[H + hh]);
            beta[(int64_t)t * H + hh] = 1.f / (1.f + expf(-b));
            decay[(int64_t)t * H + hh] = expf(-expf(a_log[hh]) * softplus_f(a + dt_bias[hh]));
        }
        return;
    }
    const int start = q_start[seq];
    const int n = t - start;                 // index of the token inside its portion
    float* st = conv_state + (int64_t)slots[seq] * (taps - 1) * C;
    // update_state (every sequence of the step brings one token): the thread that read a channel's earlier inputs
    // also shifts them down and appends the new one, and no separate pass over the state is needed
    auto channel = [&](int c) {
        float acc = 0.f;
        if constexpr (TAPS > 0) {
            float x[TAPS], w[TAPS];
#pragma unroll
            for (int j = 0; j < TAPS; ++j) {
                const int idx = n - (TAPS - 1) + j;
                x[j] = idx >= 0 ? to_float(proj[(int64_t)(start + idx) * ld + c]) : st[(int64_t)(TAPS - 1 + idx) * C + c];
                w[j] = conv_w[(int64_t)c * TAPS + j];
            }
#pragma unroll
            for (int j = 0; j < TAPS; ++j) {
                if (update_state && j >= 1) st[(int64_t)(j - 1) * C + c] = x[j];
                acc = fmaf(w[j], x[j], acc);
            }
        } else {
            for (int j = 0; j < taps; ++j) {
                const int idx = n - (taps - 1) + j;
                const float x = idx >= 0 ? to_float(proj[(int64_t)(start + idx) * ld + c]) : st[(int64_t)(taps - 1 + idx) * C + c];
                if (update_state && j >= 1) st[(int64_t)(j - 1) * C + c] = x;
                acc = fmaf(conv_w[(int64_t)c * taps + j], x, acc);
            }
        }
        return silu_f(acc);
    };
    if (unit >= 2 * G) {                     // a value head: no norm
        const int hh = unit - 2 * G;
        for (int d = lane; d < Dv; d += 32) vc[(int64_t)t * H * Dv + hh * Dv + d] = channel(2 * nqk + hh * Dv + d);
        return;
    }
    // a q or k head: up to eight channels a lane, unit norm over the head
    float x[GP_MAX_D / 32], ss = 0.f;
#pragma unroll
    for (int i = 0; i < GP_MAX_D / 32; ++i) {
        const int d = lane + i * 32;
        x[i] = d < D ? channel(unit * D + d) : 0.f;
        ss = fmaf(x[i], x[i], ss);
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss + 1e-6f) * (unit < G ? rsqrtf((float)D) : 1.f);
    float* dst = unit < G ? qn + (int64_t)t * nqk + unit * D : kn + (int64_t)t * nqk + (unit - G) * D;
#pragma unroll
    for (int i = 0; i < GP_MAX_D / 32; ++i) {
        const int d = lane + i * 32;
        if (d < D) dst[d] = x[i] * r;
    }
}

// New state of every sequence in the batch: the inputs of its last taps - 1 tokens (older ones shift down).
template <typename TA>
__global__ void gdr_conv_state_kernel(const TA* __restrict__ proj, int64_t ld, float* __restrict__ conv_state, int taps, int C,
                                      const int* __restrict__ q_start, const int* __restrict__ slots, int n_seqs) {
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C || seq >= n_seqs) return;
    const int start = q_start[seq], n = q_start[seq + 1] - start;
    if (n <= 0) return;
    float* st = conv_state + (int64_t)slots[seq] * (taps - 1) * C;
    for (int i = 0; i < taps - 1; ++i) {   // ascending: entry i reads entry i + n, never one already rewritten
        const int idx = n - (taps - 1) + i;
        st[(int64_t)i * C + c] = idx >= 0 ? to_float(proj[(int64_t)(start + idx) * ld + c]) : st[(int64_t)(i + n) * C + c];
    }
}

// ---------------------------------------------------------------------------------------- scan
constexpr int GS_COLS = 32;          // value columns per CTA
constexpr int GS_LANES = 8;          // lanes that share a column
constexpr int GS_BLOCK = GS_COLS * GS_LANES;

__device__ __forceinline__ void gs_cp_async16(void* dst, const void* src, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
                 "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void gs_cp_async4(void* dst, const void* src, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
                 "r"(valid ? 4 : 0) : "memory");
}

// DPL: key dimensions per lane (D <= 8 * DPL).  Lane r of a column holds dimensions [r * DPL, (r + 1) * DPL) of its
// column of S in registers.  (Eight lanes a column: with four, a CTA's four warps had a scheduler each and every
// dependent instruction waited out its latency, 730 cycles a token at D = 128; two warps a scheduler hide part of it.
// Sixteen lanes and a fourth round of shuffles measured slower again: a 2,048-token prompt of four layers 7.1 against 6.6 ms.)
//
// The state's layout in memory is this kernel's own: per (slot, head, block of 32 columns) DPL planes of 256 floats,
// plane i holding element (dimension r * DPL + i, column c) at c * 8 + r, which is the thread's own index.  A warp so
// reads and writes 128 contiguous bytes per plane, and dimensions beyond D and columns beyond Dv are zeros that stay
// zeros.  imp_gdr_state_floats() gives the size per slot.  The new tokens' q, k, v, decay and beta travel through a two-deep ring of chunks in shared
// memory (cp.async; the next chunk is on its way while this one is computed); outputs leave a chunk at a time.
//
// Per token, with a = S^T k, c = S^T q (both on the state before the token) and kq = k . q:
//     u = beta (v - g a);   o = g c + u kq;   S <- g S + k u^T
// which is the recurrence's read-out S_new^T q written so that both reductions over the key dimension start from
// the old state at once: one round of shuffles per token on the critical path instead of two.
template <int DPL, bool VEC>
__global__ void __launch_bounds__(GS_BLOCK, 1) gdr_scan_kernel(
    const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vc, const float* __restrict__ beta,
    const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ out, const int* __restrict__ q_start,
    const int* __restrict__ slots, int G, int D, int H, int Dv) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int ROW = DPL + 4;                          // padded so that the eight lanes' 16-byte reads miss each other's banks
    constexpr int CH = DPL <= 16 ? 16 : 8;                // tokens per chunk
    __shared__ __align__(16) float k_s[2][CH][GS_LANES * ROW];
    __shared__ __align__(16) float q_s[2][CH][GS_LANES * ROW];
    __shared__ float v_s[2][CH][GS_COLS];
    __shared__ float g_s[2][CH], b_s[2][CH];
    __shared__ float o_s[CH][GS_COLS];
    const int tid = threadIdx.x, r = tid & (GS_LANES - 1), ci = tid / GS_LANES;
    const int col0 = blockIdx.x * GS_COLS;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int hk = h / (H / G);
    const int start = q_start[seq], n = q_start[seq + 1] - start;
    if (n <= 0) return;
    float* S = state + ((((int64_t)slots[seq] * H + h) * gridDim.x + blockIdx.x) * DPL) * GS_BLOCK + tid;
    float s[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) s[i] = S[i * GS_BLOCK];
    const int nqk = G * D;
    const int64_t hv = (int64_t)H * Dv;
    auto load_chunk = [&](int t0, int buf) {
        const int nt = min(CH, n - t0);
        if (VEC) {
            constexpr int V4 = GS_LANES * DPL / 4;                      // 16-byte pieces of a (padded) row: 4 dimensions, all inside one lane's run
            for (int e = tid; e < CH * V4; e += GS_BLOCK) {
                const int tt = e / V4, d = (e - tt * V4) * 4;
                const bool ok = tt < nt && d < D;
                const int64_t src = ok ? (int64_t)(start + t0 + tt) * nqk + hk * D + d : 0;
                const int dst = (d / DPL) * ROW + d % DPL;
                gs_cp_async16(&k_s[buf][tt][dst], kn + src, ok);
                gs_cp_async16(&q_s[buf][tt][dst], qn + src, ok);
            }
        } else {
            for (int e = tid; e < CH * GS_LANES * DPL; e += GS_BLOCK) {
                const int tt = e / (GS_LANES * DPL), d = e - tt * (GS_LANES * DPL);
                const bool ok = tt < nt && d < D;
                const int64_t src = ok ? (int64_t)(start + t0 + tt) * nqk + hk * D + d : 0;
                const int dst = (d / DPL) * ROW + d % DPL;
                gs_cp_async4(&k_s[buf][tt][dst], kn + src, ok);
                gs_cp_async4(&q_s[buf][tt][dst], qn + src, ok);
            }
        }
        for (int e = tid; e < CH * GS_COLS; e += GS_BLOCK) {
            const int tt = e / GS_COLS, c = e - tt * GS_COLS;
            const bool ok = tt < nt && col0 + c < Dv;
            gs_cp_async4(&v_s[buf][tt][c], vc + (ok ? (int64_t)(start + t0 + tt) * hv + (int64_t)h * Dv + col0 + c : 0), ok);
        }
        if (tid < CH) {
            const bool ok = tid < nt;
            const int64_t src = ok ? (int64_t)(start + t0 + tid) * H + h : 0;
            gs_cp_async4(&g_s[buf][tid], decay + src, ok);
            gs_cp_async4(&b_s[buf][tid], beta + src, ok);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    load_chunk(0, 0);
    int buf = 0;
    for (int t0 = 0; t0 < n; t0 += CH, buf ^= 1) {
        const int nt = min(CH, n - t0);
        if (t0 + CH < n) {
            load_chunk(t0 + CH, buf ^ 1);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float g = g_s[buf][tt], b = b_s[buf][tt], v = v_s[buf][tt][ci];
            const float4* k4 = reinterpret_cast<const float4*>(&k_s[buf][tt][r * ROW]);
            const float4* q4 = reinterpret_cast<const float4*>(&q_s[buf][tt][r * ROW]);
            float a0 = 0.f, a1 = 0.f, c0 = 0.f, c1 = 0.f, e0 = 0.f, e1 = 0.f;
#pragma unroll
            for (int i = 0; i < DPL / 4; ++i) {
                const float4 kk = k4[i], qq = q4[i];
                a0 = fmaf(s[4 * i], kk.x, a0);     a1 = fmaf(s[4 * i + 1], kk.y, a1);
                a0 = fmaf(s[4 * i + 2], kk.z, a0); a1 = fmaf(s[4 * i + 3], kk.w, a1);
                c0 = fmaf(s[4 * i], qq.x, c0);     c1 = fmaf(s[4 * i + 1], qq.y, c1);
                c0 = fmaf(s[4 * i + 2], qq.z, c0); c1 = fmaf(s[4 * i + 3], qq.w, c1);
                e0 = fmaf(kk.x, qq.x, e0);         e1 = fmaf(kk.y, qq.y, e1);
                e0 = fmaf(kk.z, qq.z, e0);         e1 = fmaf(kk.w, qq.w, e1);
            }
            float a = a0 + a1, c = c0 + c1, kq = e0 + e1;
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            c += __shfl_xor_sync(0xffffffffu, c, 1);
            kq += __shfl_xor_sync(0xffffffffu, kq, 1);
            a += __shfl_xor_sync(0xffffffffu, a, 2);
            c += __shfl_xor_sync(0xffffffffu, c, 2);
            kq += __shfl_xor_sync(0xffffffffu, kq, 2);
            a += __shfl_xor_sync(0xffffffffu, a, 4);
            c += __shfl_xor_sync(0xffffffffu, c, 4);
            kq += __shfl_xor_sync(0xffffffffu, kq, 4);
            const float u = b * (v - g * a);
#pragma unroll
            for (int i = 0; i < DPL / 4; ++i) {
                const float4 kk = k4[i];
                s[4 * i] = fmaf(kk.x, u, g * s[4 * i]);
                s[4 * i + 1] = fmaf(kk.y, u, g * s[4 * i + 1]);
                s[4 * i + 2] = fmaf(kk.z, u, g * s[4 * i + 2]);
                s[4 * i + 3] = fmaf(kk.w, u, g * s[4 * i + 3]);
            }
            if (r == 0) o_s[tt][ci] = fmaf(u, kq, g * c);
        }
        __syncthreads();
        for (int e = tid; e < nt * GS_COLS; e += GS_BLOCK) {
            const int tt = e / GS_COLS, c = e - tt * GS_COLS;
            if (col0 + c < Dv) out[(int64_t)(start + t0 + tt) * hv + (int64_t)h * Dv + col0 + c] = o_s[tt][c];
        }
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) S[i * GS_BLOCK] = s[i];
}

// -------------------------------------------------------------------------------------- output
// y[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * w[h * w_head_stride + :] * act(gate[t, h, :]); a warp per (token, head).
// w may be null (no weight); w_head_stride 0: one weight vector for all heads; act: 0 silu, 1 sigmoid.
template <typename TA>
__global__ void gdr_output_kernel(TA* __restrict__ y, const float* __restrict__ o, const TA* __restrict__ gate, int64_t gate_ld,
                                  const float* __restrict__ w, int w_head_stride, int act, float eps, int n_tokens, int H, int Dv) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_tokens * H) return;
    const int64_t t = item / H;
    const int h = (int)(item - t * H);
    const float* x = o + (t * H + h) * Dv;
    float ss = 0.f;
    for (int d = lane; d < Dv; d += 32) ss = fmaf(x[d], x[d], ss);
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)Dv + eps);
    const TA* gt = gate + t * gate_ld + (int64_t)h * Dv;
    const float* wh = w ? w + (int64_t)h * w_head_stride : nullptr;
    TA* dst = y + (t * H + h) * Dv;
    for (int d = lane; d < Dv; d += 32) {
        const float g = to_float(gt[d]);
        const float a = act == 0 ? silu_f(g) : 1.f / (1.f + expf(-g));
        dst[d] = from_float<TA>(x[d] * r * (wh ? wh[d] : 1.f) * a);
    }
}

// ------------------------------------------------------------------------------------ launchers
// update_state: the step brings one token per sequence (n_tokens == n_seqs) and the kernel also writes the
// convolution's new state; otherwise imp_gdr_conv_state has to follow.
IMP_API int imp_gdr_prepare(const void* proj, int64_t ld, const float* conv_w, int taps, float* conv_state,
                            const int* seq_of_token, const int* q_start, const int* slots, int n_tokens, int n_seqs, int G, int D,
                            int H, int Dv, const float* a_log, const float* dt_bias, float* qn, float* kn, float* vc, float* beta,
                            float* decay, int update_state, int act_dtype, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(proj && conv_w && conv_state && seq_of_token && q_start && slots && a_log && dt_bias && qn && kn && vc && beta && decay,
                  "imp_gdr_prepare: null pointer");
    IMP_CHECK_ARG(G > 0 && H > 0 && H % G == 0 && D > 0 && D <= GP_MAX_D && Dv > 0 && taps >= 1,
                  "imp_gdr_prepare: bad sizes (heads %d over %d key heads, key size %d of at most %d)", H, G, D, GP_MAX_D);
    IMP_CHECK_ARG(!update_state || n_tokens == n_seqs, "imp_gdr_prepare: the state is updated in place only when every sequence brings one token");
    IMP_CHECK_ARG(ld >= (int64_t)2 * G * D + 2 * (int64_t)H * Dv + 2 * H, "imp_gdr_prepare: the projection's rows are too short");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t items = (int64_t)n_tokens * (2 * G + H + 1);
    const int64_t ctas = (items + GP_BLOCK / 32 - 1) / (GP_BLOCK / 32);
    IMP_CHECK_ARG(ctas <= 0x7fffffff, "imp_gdr_prepare: too many tokens");
    const dim3 grid((unsigned)ctas);
#define GDR_PREPARE(TA, TAPS)                                                                                                      \
    imp_launch(gdr_prepare_kernel<TA, TAPS>, grid, dim3(GP_BLOCK), 0, s, (const TA*)proj, ld, conv_w, taps, conv_state, seq_of_token, \
               q_start, slots, n_tokens, n_seqs, G, D, H, Dv, a_log, dt_bias, qn, kn, vc, beta, decay, update_state, status)
#define GDR_PREPARE_T(TA)                       \
    do {                                        \
        if (taps == 4) GDR_PREPARE(TA, 4);      \
        else if (taps == 3) GDR_PREPARE(TA, 3); \
        else if (taps == 2) GDR_PREPARE(TA, 2); \
        else GDR_PREPARE(TA, 0);                \
    } while (0)
    if (act_dtype == IMP_F32) GDR_PREPARE_T(float);
    else GDR_PREPARE_T(__nv_bfloat16);
#undef GDR_PREPARE_T
#undef GDR_PREPARE
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_gdr_conv_state(const void* proj, int64_t ld, float* conv_state, int taps, int C, const int* q_start, const int* slots,
                               int n_seqs, int act_dtype, void* stream) {
    if (n_seqs == 0 || taps <= 1) return 0;
    IMP_CHECK_ARG(proj && conv_state && q_start && slots && C > 0 && n_seqs <= 65535, "imp_gdr_conv_state: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((C + 127) / 128, n_seqs);
    if (act_dtype == IMP_F32)
        imp_launch(gdr_conv_state_kernel<float>, grid, dim3(128), 0, s, (const float*)proj, ld, conv_state, taps, C, q_start, slots, n_seqs);
    else
        imp_launch(gdr_conv_state_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, (const __nv_bfloat16*)proj, ld, conv_state, taps, C,
                   q_start, slots, n_seqs);
    IMP_RETURN_LAUNCH();
}

// Key dimensions a lane holds for key size D (eight lanes a column).
static int gdr_dims_per_lane(int D) { return D <= 32 ? 4 : D <= 64 ? 8 : D <= 128 ? 16 : 32; }

// Floats of one request's state S for H heads of D x Dv in the scan kernel's layout (padded to whole lanes and column blocks).
IMP_API int64_t imp_gdr_state_floats(int H, int D, int Dv) {
    return (int64_t)H * ((Dv + GS_COLS - 1) / GS_COLS) * gdr_dims_per_lane(D) * GS_BLOCK;
}

// state: [slots, imp_gdr_state_floats(H, D, Dv)] float32 in the kernel's own layout, zero at a request's start, updated in
// place; out: [n_tokens, H * Dv] float32.
IMP_API int imp_gdr_scan(const float* qn, const float* kn, const float* vc, const float* beta, const float* decay, float* state,
                         float* out, const int* q_start, const int* slots, int n_seqs, int G, int D, int H, int Dv, void* stream) {
    if (n_seqs == 0) return 0;
    IMP_CHECK_ARG(qn && kn && vc && beta && decay && state && out && q_start && slots, "imp_gdr_scan: null pointer");
    IMP_CHECK_ARG(G > 0 && H % G == 0 && D > 0 && Dv > 0 && H <= 65535 && n_seqs <= 65535, "imp_gdr_scan: bad sizes");
    if (D > 256) {
        imp_set_error("imp_gdr_scan: key size %d exceeds 256", D);
        return IMP_ERR_UNSUPPORTED;
    }
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((Dv + GS_COLS - 1) / GS_COLS, H, n_seqs);
    // 16-byte copies of q and k rows need rows that start on 16 bytes: D a multiple of 4 and aligned buffers
    const bool vec = D % 4 == 0 && (uintptr_t)qn % 16 == 0 && (uintptr_t)kn % 16 == 0;
    // Launched as an ordinary dependent, without the programmatic attribute: its CTAs hold three quarters of an SM's
    // registers, and resident early (waiting for the kernels before them) they starved those kernels: a 2,048-token
    // prompt of four layers took 8.1 instead of 6.7 ms.
#define GDR_SCAN(DPL)                                                                                                          \
    do {                                                                                                                       \
        if (vec) gdr_scan_kernel<DPL, true><<<grid, GS_BLOCK, 0, s>>>(qn, kn, vc, beta, decay, state, out, q_start, slots, G, D, H, Dv); \
        else gdr_scan_kernel<DPL, false><<<grid, GS_BLOCK, 0, s>>>(qn, kn, vc, beta, decay, state, out, q_start, slots, G, D, H, Dv);    \
    } while (0)
    switch (gdr_dims_per_lane(D)) {
        case 4: GDR_SCAN(4); break;
        case 8: GDR_SCAN(8); break;
        case 16: GDR_SCAN(16); break;
        default: GDR_SCAN(32); break;
    }
#undef GDR_SCAN
    IMP_RETURN_LAUNCH();
}


// The same read-out with one norm over the whole row: y[t, :] = o[t, :] / sqrt(mean over all n of o^2 + eps) * w * act(gate[t, :]),
// the heads side by side (n = H * Dv); a CTA per token, sums in 32-bit in an order the row's size fixes.
template <typename TA>
__global__ void __launch_bounds__(256) lsr_output_row_kernel(TA* __restrict__ y, const float* __restrict__ o, const TA* __restrict__ gate, int64_t gate_ld,
                                                             const float* __restrict__ w, int act, float eps, int n) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int64_t t = blockIdx.x;
    const float* x = o + t * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
    const float r = rsqrtf(block_sum(ss, scratch) / (float)n + eps);
    const TA* gt = gate + t * gate_ld;
    TA* dst = y + t * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float g = to_float(gt[i]);
        const float a = act == 0 ? silu_f(g) : 1.f / (1.f + expf(-g));
        dst[i] = from_float<TA>(x[i] * r * (w ? w[i] : 1.f) * a);
    }
}

// Rows whose size is a multiple of 4: four neighbouring values a thread and pass (16-byte loads of the read-out and the weight,
// 8-byte loads of a 16-bit gate), 512 threads a token.
template <typename TA>
__global__ void __launch_bounds__(512) lsr_output_row_vec_kernel(TA* __restrict__ y, const float* __restrict__ o, const TA* __restrict__ gate, int64_t gate_ld,
                                                                 const float* __restrict__ w, int act, float eps, int n) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int64_t t = blockIdx.x;
    const float* x = o + t * n;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < n; i += 512 * 4) {
        const float4 v = *reinterpret_cast<const float4*>(x + i);
        ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
    }
    const float r = rsqrtf(block_sum(ss, scratch) / (float)n + eps);
    const TA* gt = gate + t * gate_ld;
    TA* dst = y + t * n;
    for (int i = threadIdx.x * 4; i < n; i += 512 * 4) {
        const float4 v = *reinterpret_cast<const float4*>(x + i);
        const float4 ww = w ? *reinterpret_cast<const float4*>(w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        float g[4], out[4];
        if constexpr (sizeof(TA) == 4) {
            const float4 gv = *reinterpret_cast<const float4*>(gt + i);
            g[0] = gv.x, g[1] = gv.y, g[2] = gv.z, g[3] = gv.w;
        } else {
            const uint2 u = *reinterpret_cast<const uint2*>(gt + i);
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
            g[0] = a.x, g[1] = a.y, g[2] = b.x, g[3] = b.y;
        }
        const float xs[4] = {v.x, v.y, v.z, v.w}, ws[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float a = act == 0 ? silu_f(g[k]) : 1.f / (1.f + expf(-g[k]));
            out[k] = xs[k] * r * ws[k] * a;
        }
        if constexpr (sizeof(TA) == 4) {
            *reinterpret_cast<float4*>(dst + i) = make_float4(out[0], out[1], out[2], out[3]);
        } else {
            __nv_bfloat162 a = __floats2bfloat162_rn(out[0], out[1]), b = __floats2bfloat162_rn(out[2], out[3]);
            uint2 u;
            u.x = *reinterpret_cast<uint32_t*>(&a), u.y = *reinterpret_cast<uint32_t*>(&b);
            *reinterpret_cast<uint2*>(dst + i) = u;
        }
    }
}

// The read-out's norm and gate.  w: float32 weight or null; w_head_stride: 0 for one vector [Dv] shared by the heads, Dv for
// a vector [H * Dv]; gate_act: 0 silu, 1 sigmoid.
IMP_API int imp_gdr_output_ex(void* y, const float* o, const void* gate, int64_t gate_ld, const float* w, int w_head_stride, int gate_act,
                              float eps, int n_tokens, int H, int Dv, int act_dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(y && o && gate && H > 0 && Dv > 0 && (gate_act == 0 || gate_act == 1) && (w_head_stride == 0 || w_head_stride == Dv),
                  "imp_gdr_output: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t items = (int64_t)n_tokens * H;
    const dim3 grid((unsigned)((items + 7) / 8));
    if (act_dtype == IMP_F32)
        imp_launch(gdr_output_kernel<float>, grid, dim3(256), 0, s, (float*)y, o, (const float*)gate, gate_ld, w, w_head_stride, gate_act, eps,
                   n_tokens, H, Dv);
    else
        imp_launch(gdr_output_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (__nv_bfloat16*)y, o, (const __nv_bfloat16*)gate, gate_ld, w,
                   w_head_stride, gate_act, eps, n_tokens, H, Dv);
    IMP_RETURN_LAUNCH();
}

// The read-out normalised over the whole row of n = H * Dv values (w: float32 [n] or null; gate_act: 0 silu, 1 sigmoid).
IMP_API int imp_lsr_output_row(void* y, const float* o, const void* gate, int64_t gate_ld, const float* w, int gate_act, float eps, int n_tokens,
                               int n, int act_dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(y && o && gate && n > 0 && gate_ld >= n && (gate_act == 0 || gate_act == 1), "imp_lsr_output_row: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t el = act_dtype == IMP_F32 ? 4 : 2;
    if (n % 4 == 0 && gate_ld % 4 == 0 && (uintptr_t)o % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)gate % (4 * el) == 0 && (uintptr_t)y % (4 * el) == 0) {
        if (act_dtype == IMP_F32)
            imp_launch(lsr_output_row_vec_kernel<float>, dim3(n_tokens), dim3(512), 0, s, (float*)y, o, (const float*)gate, gate_ld, w, gate_act, eps, n);
        else
            imp_launch(lsr_output_row_vec_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(512), 0, s, (__nv_bfloat16*)y, o, (const __nv_bfloat16*)gate, gate_ld, w,
                       gate_act, eps, n);
        IMP_RETURN_LAUNCH();
    }
    if (act_dtype == IMP_F32)
        imp_launch(lsr_output_row_kernel<float>, dim3(n_tokens), dim3(256), 0, s, (float*)y, o, (const float*)gate, gate_ld, w, gate_act, eps, n);
    else
        imp_launch(lsr_output_row_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, s, (__nv_bfloat16*)y, o, (const __nv_bfloat16*)gate, gate_ld, w,
                   gate_act, eps, n);
    IMP_RETURN_LAUNCH();
}


IMP_API int imp_gdr_output(void* y, const float* o, const void* gate, int64_t gate_ld, const float* w, float eps, int n_tokens, int H,
                           int Dv, int act_dtype, void* stream) {
    IMP_CHECK_ARG(w, "imp_gdr_output: bad argument");
    return imp_gdr_output_ex(y, o, gate, gate_ld, w, 0, 0, eps, n_tokens, H, Dv, act_dtype, stream);
}

// ====================================================================================================
// The general form of these recurrences: a matrix state S [D, Dv] per head that decays per key channel,
// loses one direction and gains one outer product per token,
//     S <- diag(w) S - p (z^T S) + kw v^T,      o = S^T q      (the read-out sees the token's own write)
// with w, p, z, kw, q vectors over the key dimension.  Three mixers are instances of it:
//     retention              w = a constant per head, p = z = 0, kw = k
//     delta rule, decay per  w = g (per head and key channel), z = g k, p = kw = beta k
//       key channel            (S <- g S; u = beta (v - S^T k); S <- S + k u^T)
//     generalised delta      w per head and key channel, z = u (the unit key), p = a u, kw = k
// Everything is 32-bit arithmetic on 32-bit state.  The work is split as in gdr_scan_kernel (a CTA owns 32 value
// columns of one head of one sequence, eight lanes a column) and the state has that kernel's layout.  Per column,
// with a = z . s and c = (q w) . s on the old column s, and the column-independent qp = q . p, qk = q . kw
// (made once per token and head by the prepare kernels):
//     s <- w s - p a + kw v;      o = c - qp a + qk v
// so the two sums over the key dimension start from the old state together: one round of shuffles per token.
enum { LSR_RETENTION = 0, LSR_DELTA = 1, LSR_GENERAL = 2 };

// Rows of one token in the ring, by mode: k (kw), q always; w for the modes with a decay per channel; p and z for the
// general form.
__host__ __device__ constexpr int lsr_rows(int mode) { return mode == LSR_RETENTION ? 2 : mode == LSR_DELTA ? 3 : 5; }
__host__ __device__ constexpr int lsr_chunk(int dpl) { return dpl <= 8 ? 16 : 8; }

// kw, q, w, p, z: [T, H, D] float32 (w, p, z only where the mode reads them); v: [T, H, Dv]; scal: [T, H, 2] = (qk, qp);
// head_decay: [H] (LSR_RETENTION).  In LSR_DELTA kw is the plain key k, p and z are formed from it (z = w k, p = beta k),
// and scal = (beta q . k, beta).
template <int DPL, bool VEC, int MODE>
__global__ void __launch_bounds__(GS_BLOCK, 1) lsr_scan_kernel(
    const float* __restrict__ kw, const float* __restrict__ q, const float* __restrict__ w, const float* __restrict__ p,
    const float* __restrict__ z, const float* __restrict__ v, const float* __restrict__ scal, const float* __restrict__ head_decay,
    float* __restrict__ state, float* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ slots, int D, int H,
    int Dv) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int ROW = DPL + 4;
    constexpr int CH = lsr_chunk(DPL);
    constexpr int NR = lsr_rows(MODE);
    constexpr int TOK = NR * GS_LANES * ROW;            // floats of one token's vectors in the ring
    extern __shared__ __align__(16) float lsr_smem[];
    float* vec_s = lsr_smem;                              // [2][CH][NR][GS_LANES * ROW]
    float* v_s = vec_s + 2 * CH * TOK;                    // [2][CH][GS_COLS]
    float* sc_s = v_s + 2 * CH * GS_COLS;                 // [2][CH][2]
    float* o_s = sc_s + 2 * CH * 2;                       // [CH][GS_COLS]
    const int tid = threadIdx.x, r = tid & (GS_LANES - 1), ci = tid / GS_LANES;
    const int col0 = blockIdx.x * GS_COLS;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int start = q_start[seq], n = q_start[seq + 1] - start;
    if (n <= 0) return;
    float* S = state + ((((int64_t)slots[seq] * H + h) * gridDim.x + blockIdx.x) * DPL) * GS_BLOCK + tid;
    float s[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) s[i] = S[i * GS_BLOCK];
    const float hd = MODE == LSR_RETENTION ? head_decay[h] : 1.f;
    const int64_t hD = (int64_t)H * D, hv = (int64_t)H * Dv;
    const float* src_of[5] = {kw, q, MODE == LSR_RETENTION ? kw : w, MODE == LSR_GENERAL ? p : kw, MODE == LSR_GENERAL ? z : kw};   // the first lsr_rows(MODE) are read
    auto load_chunk = [&](int t0, int buf) {
        const int nt = min(CH, n - t0);
        float* base = vec_s + (size_t)buf * CH * TOK;
        if (VEC) {
            constexpr int V4 = GS_LANES * DPL / 4;
            for (int e = tid; e < CH * V4; e += GS_BLOCK) {
                const int tt = e / V4, d = (e - tt * V4) * 4;
                const bool ok = tt < nt && d < D;
                const int64_t src = ok ? (int64_t)(start + t0 + tt) * hD + (int64_t)h * D + d : 0;
                const int dst = (d / DPL) * ROW + d % DPL;
#pragma unroll
                for (int a = 0; a < NR; ++a) gs_cp_async16(base + (size_t)tt * TOK + a * (GS_LANES * ROW) + dst, src_of[a] + src, ok);
            }
        } else {
            for (int e = tid; e < CH * GS_LANES * DPL; e += GS_BLOCK) {
                const int tt = e / (GS_LANES * DPL), d = e - tt * (GS_LANES * DPL);
                const bool ok = tt < nt && d < D;
                const int64_t src = ok ? (int64_t)(start + t0 + tt) * hD + (int64_t)h * D + d : 0;
                const int dst = (d / DPL) * ROW + d % DPL;
#pragma unroll
                for (int a = 0; a < NR; ++a) gs_cp_async4(base + (size_t)tt * TOK + a * (GS_LANES * ROW) + dst, src_of[a] + src, ok);
            }
        }
        for (int e = tid; e < CH * GS_COLS; e += GS_BLOCK) {
            const int tt = e / GS_COLS, c = e - tt * GS_COLS;
            const bool ok = tt < nt && col0 + c < Dv;
            gs_cp_async4(v_s + ((size_t)buf * CH + tt) * GS_COLS + c, v + (ok ? (int64_t)(start + t0 + tt) * hv + (int64_t)h * Dv + col0 + c : 0), ok);
        }
        if (tid < CH * 2) {
            const int tt = tid >> 1;
            const bool ok = tt < nt;
            gs_cp_async4(sc_s + ((size_t)buf * CH + tt) * 2 + (tid & 1), scal + (ok ? ((int64_t)(start + t0 + tt) * H + h) * 2 + (tid & 1) : 0), ok);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    load_chunk(0, 0);
    int buf = 0;
    for (int t0 = 0; t0 < n; t0 += CH, buf ^= 1) {
        const int nt = min(CH, n - t0);
        if (t0 + CH < n) {
            load_chunk(t0 + CH, buf ^ 1);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float* tok = vec_s + ((size_t)buf * CH + tt) * TOK + r * ROW;
            const float4* k4 = reinterpret_cast<const float4*>(tok);
            const float4* q4 = reinterpret_cast<const float4*>(tok + GS_LANES * ROW);
            const float4* w4 = reinterpret_cast<const float4*>(tok + 2 * GS_LANES * ROW);
            const float4* p4 = reinterpret_cast<const float4*>(tok + 3 * GS_LANES * ROW);
            const float4* z4 = reinterpret_cast<const float4*>(tok + 4 * GS_LANES * ROW);
            const float vv = v_s[((size_t)buf * CH + tt) * GS_COLS + ci];
            const float qk = sc_s[((size_t)buf * CH + tt) * 2], qp = sc_s[((size_t)buf * CH + tt) * 2 + 1];
            float a0 = 0.f, a1 = 0.f, c0 = 0.f, c1 = 0.f;
#pragma unroll
            for (int i = 0; i < DPL / 4; ++i) {
                const float4 qq = q4[i];
                if (MODE == LSR_RETENTION) {
                    c0 = fmaf(s[4 * i], qq.x, c0);     c1 = fmaf(s[4 * i + 1], qq.y, c1);
                    c0 = fmaf(s[4 * i + 2], qq.z, c0); c1 = fmaf(s[4 * i + 3], qq.w, c1);
                } else {
                    const float4 ww = w4[i];
                    // the decayed column is formed first, as the recurrence states it: both sums read w s
                    const float d0 = ww.x * s[4 * i], d1 = ww.y * s[4 * i + 1], d2 = ww.z * s[4 * i + 2], d3 = ww.w * s[4 * i + 3];
                    c0 = fmaf(d0, qq.x, c0); c1 = fmaf(d1, qq.y, c1);
                    c0 = fmaf(d2, qq.z, c0); c1 = fmaf(d3, qq.w, c1);
                    if (MODE == LSR_DELTA) {
                        const float4 kk = k4[i];       // a = k . (w s)
                        a0 = fmaf(d0, kk.x, a0); a1 = fmaf(d1, kk.y, a1);
                        a0 = fmaf(d2, kk.z, a0); a1 = fmaf(d3, kk.w, a1);
                    } else {
                        const float4 zz = z4[i];       // the unit key: a = u . s on the state before the decay
                        a0 = fmaf(s[4 * i], zz.x, a0);     a1 = fmaf(s[4 * i + 1], zz.y, a1);
                        a0 = fmaf(s[4 * i + 2], zz.z, a0); a1 = fmaf(s[4 * i + 3], zz.w, a1);
                    }
                }
            }
            float a = a0 + a1, c = c0 + c1;
            if (MODE != LSR_RETENTION) {
                a += __shfl_xor_sync(0xffffffffu, a, 1);
                a += __shfl_xor_sync(0xffffffffu, a, 2);
                a += __shfl_xor_sync(0xffffffffu, a, 4);
            }
            c += __shfl_xor_sync(0xffffffffu, c, 1);
            c += __shfl_xor_sync(0xffffffffu, c, 2);
            c += __shfl_xor_sync(0xffffffffu, c, 4);
#pragma unroll
            for (int i = 0; i < DPL / 4; ++i) {
                const float4 kk = k4[i];
                if (MODE == LSR_RETENTION) {
                    s[4 * i] = fmaf(kk.x, vv, hd * s[4 * i]);
                    s[4 * i + 1] = fmaf(kk.y, vv, hd * s[4 * i + 1]);
                    s[4 * i + 2] = fmaf(kk.z, vv, hd * s[4 * i + 2]);
                    s[4 * i + 3] = fmaf(kk.w, vv, hd * s[4 * i + 3]);
                } else if (MODE == LSR_DELTA) {
                    const float4 ww = w4[i];
                    const float u = qp * (vv - a);     // qp holds beta: s <- w s + k beta (v - a)
                    s[4 * i] = fmaf(kk.x, u, ww.x * s[4 * i]);
                    s[4 * i + 1] = fmaf(kk.y, u, ww.y * s[4 * i + 1]);
                    s[4 * i + 2] = fmaf(kk.z, u, ww.z * s[4 * i + 2]);
                    s[4 * i + 3] = fmaf(kk.w, u, ww.w * s[4 * i + 3]);
                } else {
                    const float4 ww = w4[i], pp = p4[i];
                    s[4 * i] = fmaf(kk.x, vv, fmaf(-pp.x, a, ww.x * s[4 * i]));
                    s[4 * i + 1] = fmaf(kk.y, vv, fmaf(-pp.y, a, ww.y * s[4 * i + 1]));
                    s[4 * i + 2] = fmaf(kk.z, vv, fmaf(-pp.z, a, ww.z * s[4 * i + 2]));
                    s[4 * i + 3] = fmaf(kk.w, vv, fmaf(-pp.w, a, ww.w * s[4 * i + 3]));
                }
            }
            if (r == 0) {
                float o;
                if (MODE == LSR_RETENTION) o = fmaf(qk, vv, hd * c);
                else if (MODE == LSR_DELTA) o = fmaf(qk, vv - a, c);
                else o = fmaf(qk, vv, fmaf(-qp, a, c));
                o_s[tt * GS_COLS + ci] = o;
            }
        }
        __syncthreads();
        for (int e = tid; e < nt * GS_COLS; e += GS_BLOCK) {
            const int tt = e / GS_COLS, c = e - tt * GS_COLS;
            if (col0 + c < Dv) out[(int64_t)(start + t0 + tt) * hv + (int64_t)h * Dv + col0 + c] = o_s[tt * GS_COLS + c];
        }
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) S[i * GS_BLOCK] = s[i];
}

static size_t lsr_smem_bytes(int dpl, int mode) {
    const int ch = lsr_chunk(dpl), tok = lsr_rows(mode) * GS_LANES * (dpl + 4);
    return (size_t)(2 * ch * tok + 2 * ch * GS_COLS + 2 * ch * 2 + ch * GS_COLS) * sizeof(float);
}

template <int DPL, bool VEC, int MODE>
static cudaError_t lsr_launch(dim3 grid, cudaStream_t s, const float* kw, const float* q, const float* w, const float* p, const float* z,
                              const float* v, const float* scal, const float* head_decay, float* state, float* out, const int* q_start,
                              const int* slots, int D, int H, int Dv) {
    const size_t smem = lsr_smem_bytes(DPL, MODE);
    static bool raised = false;   // per instantiation
    if (!raised && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(lsr_scan_kernel<DPL, VEC, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        raised = true;
    }
    // an ordinary dependent launch, as gdr_scan: CTAs that hold most of an SM's registers must not become resident early
    lsr_scan_kernel<DPL, VEC, MODE><<<grid, GS_BLOCK, smem, s>>>(kw, q, w, p, z, v, scal, head_decay, state, out, q_start, slots, D, H, Dv);
    return cudaGetLastError();
}

// mode: 0 retention (head_decay [H]; w, p, z unused), 1 delta rule with a decay per key channel (kw = k, w = g,
// scal = (beta q . k, beta); p, z unused), 2 the general form.  state: [slots, imp_gdr_state_floats(H, D, Dv)], zero at a request's start, updated in place.
// All vectors are [n_tokens, H, D] float32, v and out [n_tokens, H, Dv], scal [n_tokens, H, 2] = (q . kw, q . p).
IMP_API int imp_lsr_scan(int mode, const float* kw, const float* q, const float* w, const float* p, const float* z, const float* v,
                         const float* scal, const float* head_decay, float* state, float* out, const int* q_start, const int* slots,
                         int n_seqs, int D, int H, int Dv, void* stream) {
    if (n_seqs == 0) return 0;
    IMP_CHECK_ARG(kw && q && v && scal && state && out && q_start && slots, "imp_lsr_scan: null pointer");
    IMP_CHECK_ARG(mode >= 0 && mode <= 2, "imp_lsr_scan: unknown mode %d", mode);
    IMP_CHECK_ARG(mode == LSR_RETENTION ? head_decay != nullptr : w != nullptr, "imp_lsr_scan: the mode's decay is missing");
    IMP_CHECK_ARG(mode != LSR_GENERAL || (p && z), "imp_lsr_scan: the general form reads p and z");
    IMP_CHECK_ARG(D > 0 && Dv > 0 && H > 0 && H <= 65535 && n_seqs <= 65535, "imp_lsr_scan: bad sizes");
    if (D > 256) {
        imp_set_error("imp_lsr_scan: key size %d exceeds 256", D);
        return IMP_ERR_UNSUPPORTED;
    }
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((Dv + GS_COLS - 1) / GS_COLS, H, n_seqs);
    bool vec = D % 4 == 0;
    for (const float* ptr : {kw, q, w, p, z})
        if (ptr && (uintptr_t)ptr % 16) vec = false;
    cudaError_t e;
#define LSR_SCAN_M(DPL, MODE)                                                                                                      \
    e = vec ? lsr_launch<DPL, true, MODE>(grid, s, kw, q, w, p, z, v, scal, head_decay, state, out, q_start, slots, D, H, Dv)      \
            : lsr_launch<DPL, false, MODE>(grid, s, kw, q, w, p, z, v, scal, head_decay, state, out, q_start, slots, D, H, Dv)
#define LSR_SCAN(DPL)                                   \
    do {                                                \
        if (mode == LSR_RETENTION) LSR_SCAN_M(DPL, 0);  \
        else if (mode == LSR_DELTA) LSR_SCAN_M(DPL, 1); \
        else LSR_SCAN_M(DPL, 2);                        \
    } while (0)
    switch (gdr_dims_per_lane(D)) {
        case 4: LSR_SCAN(4); break;
        case 8: LSR_SCAN(8); break;
        case 16: LSR_SCAN(16); break;
        default: LSR_SCAN(32); break;
    }
#undef LSR_SCAN
#undef LSR_SCAN_M
    if (e != cudaSuccess) {
        imp_set_error("imp_lsr_scan: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// ------------------------------------------------------------------------ prepare kernels of the general scan
// One warp per (token, head) makes that head's vectors for imp_lsr_scan from the rows of the mixer's input product,
// everything after the projections in 32-bit.  Up to LP_MAX_D / 32 key channels a lane.
constexpr int LP_MAX_D = 256;
constexpr int LP_PER = LP_MAX_D / 32;

// Retention: proj columns [q: H*D | k: H*D | v: H*Dv | ...]; q = f(q projected), kw = f(k) * k_scale, v = f(v), scal = (q . kw, 0);
// f the identity (act 0) or silu (act 1), in 32-bit.
template <typename TA> __device__ __forceinline__ float lp_silu(float x) { return __fdividef(x, 1.f + __expf(-x)); }   // 16-bit inputs: the fast forms are far below their rounding
template <> __device__ __forceinline__ float lp_silu<float>(float x) { return silu_f(x); }
template <typename TA>
__global__ void __launch_bounds__(GP_BLOCK) retention_prepare_kernel(const TA* __restrict__ proj, int64_t ld, int n_tokens, int H, int D, int Dv,
                                                                     float k_scale, int act, float* __restrict__ q, float* __restrict__ kw,
                                                                     float* __restrict__ v, float* __restrict__ scal) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (GP_BLOCK / 32) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_tokens * H) return;
    const int64_t t = item / H;
    const int h = (int)(item - t * H);
    const TA* row = proj + t * ld;
    float dot = 0.f;
    for (int d = lane; d < D; d += 32) {
        float qq = to_float(row[h * D + d]), kk = to_float(row[(int64_t)H * D + h * D + d]);
        if (act == 1) qq = lp_silu<TA>(qq), kk = lp_silu<TA>(kk);
        kk *= k_scale;
        q[(t * H + h) * D + d] = qq;
        kw[(t * H + h) * D + d] = kk;
        dot = fmaf(qq, kk, dot);
    }
    for (int d = lane; d < Dv; d += 32) {
        const float vv = to_float(row[(int64_t)2 * H * D + h * Dv + d]);
        v[(t * H + h) * Dv + d] = act == 1 ? lp_silu<TA>(vv) : vv;
    }
    dot = warp_sum(dot);
    if (lane == 0) {
        scal[(t * H + h) * 2] = dot;
        scal[(t * H + h) * 2 + 1] = 0.f;
    }
}

// Generalised delta rule: proj columns [r: H*D | k: H*D | v: H*D | gate: H*D | a: H*D | ...]; dlog [T, H*D] float32 is the
// decay's pre-activation without its bias w0.
//   w = exp(-decay_scale * sigmoid(dlog + w0));  a = sigmoid(a_raw + a_bias);  u = k / sqrt(sum k^2 + unit_eps)
//   q = r, kw = k, z = u, p = a u, scal = (q . k, q . p)
template <typename TA>
__global__ void __launch_bounds__(GP_BLOCK) gdelta_prepare_kernel(const TA* __restrict__ proj, int64_t ld, const float* __restrict__ dlog,
                                                                  const float* __restrict__ w0, const float* __restrict__ a_bias,
                                                                  float decay_scale, float unit_eps, int n_tokens, int H, int D,
                                                                  float* __restrict__ q, float* __restrict__ kw, float* __restrict__ w,
                                                                  float* __restrict__ p, float* __restrict__ z, float* __restrict__ v,
                                                                  float* __restrict__ scal) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (GP_BLOCK / 32) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_tokens * H) return;
    const int64_t t = item / H;
    const int h = (int)(item - t * H);
    const int64_t HD = (int64_t)H * D;
    const TA* row = proj + t * ld + (int64_t)h * D;
    float kk[LP_PER], ss = 0.f;
#pragma unroll
    for (int i = 0; i < LP_PER; ++i) {
        const int d = lane + i * 32;
        kk[i] = d < D ? to_float(row[HD + d]) : 0.f;
        ss = fmaf(kk[i], kk[i], ss);
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss + unit_eps);
    float qk = 0.f, qp = 0.f;
    const int64_t o = (t * H + h) * D;
#pragma unroll
    for (int i = 0; i < LP_PER; ++i) {
        const int d = lane + i * 32;
        if (d < D) {
            const float r = to_float(row[d]);
            const float a = 1.f / (1.f + expf(-(to_float(row[4 * HD + d]) + a_bias[h * D + d])));
            const float sg = 1.f / (1.f + expf(-(dlog[t * HD + h * D + d] + w0[h * D + d])));
            const float u = kk[i] * inv;
            q[o + d] = r;
            kw[o + d] = kk[i];
            w[o + d] = expf(-decay_scale * sg);
            z[o + d] = u;
            p[o + d] = a * u;
            v[o + d] = to_float(row[2 * HD + d]);
            qk = fmaf(r, kk[i], qk);
            qp = fmaf(r, a * u, qp);
        }
    }
    qk = warp_sum(qk);
    qp = warp_sum(qp);
    if (lane == 0) {
        scal[(t * H + h) * 2] = qk;
        scal[(t * H + h) * 2 + 1] = qp;
    }
}

// The delta rule with a decay per key channel: proj columns [q: G*D | k: G*D | v: H*Dv | beta: H | ...]; q, k, v pass the
// causal convolution (as in gdr_prepare_kernel; conv_state [slots, taps - 1, C], C = 2*G*D + H*Dv) and silu; q and k become
// unit vectors, q times D^(-1/2); dpre [T, H*D] float32 is the decay's pre-activation without dt_bias:
//   g = exp(-exp(a_log[h]) * softplus(dpre + dt_bias));  beta = sigmoid(.)
// Outputs per value head (reading key head h / (H / G)): kw = k, q, w = g, v, scal = (beta q . k, beta).
// A CTA per (token, key head): its warps make the key head's q and k channels once, together, and then take the value
// heads of that key head in turn (a warp per value head, up to GC_MAX_WARPS at a time).
constexpr int GC_MAX_WARPS = 8;
template <typename TA, int TAPS>
__global__ void __launch_bounds__(GC_MAX_WARPS * 32) gdrc_prepare_kernel(
    const TA* __restrict__ proj, int64_t ld, const float* __restrict__ conv_w, int taps_rt, const float* __restrict__ conv_state,
    const int* __restrict__ seq_of_token, const int* __restrict__ q_start, const int* __restrict__ slots, int n_tokens, int n_seqs, int G,
    int D, int H, int Dv, const float* __restrict__ dpre, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
    float unit_eps, float* __restrict__ q, float* __restrict__ kw, float* __restrict__ w, float* __restrict__ v, float* __restrict__ scal,
    int* status) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float qk_s[2 * LP_MAX_D];
    const int taps = TAPS ? TAPS : taps_rt;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int t = (int)(blockIdx.x / G), hk = (int)(blockIdx.x - (int64_t)t * G);
    const int per_key = H / G;
    const int nqk = G * D, C = 2 * nqk + H * Dv;
    const int seq = seq_of_token[t];
    if (seq < 0 || seq >= n_seqs) {
        if (threadIdx.x == 0 && hk == 0) imp_report(status, IMP_BAD_SEQUENCE);
        return;
    }
    const int start = q_start[seq];
    const int n = t - start;
    const float* st = conv_state + (int64_t)slots[seq] * (taps - 1) * C;
    auto channel = [&](int c) {
        float acc = 0.f;
        if constexpr (TAPS > 0) {
            float x[TAPS], cw[TAPS];
#pragma unroll
            for (int j = 0; j < TAPS; ++j) {
                const int idx = n - (TAPS - 1) + j;
                x[j] = idx >= 0 ? to_float(proj[(int64_t)(start + idx) * ld + c]) : st[(int64_t)(TAPS - 1 + idx) * C + c];
                cw[j] = conv_w[(int64_t)c * TAPS + j];
            }
#pragma unroll
            for (int j = 0; j < TAPS; ++j) acc = fmaf(cw[j], x[j], acc);
        } else {
            for (int j = 0; j < taps; ++j) {
                const int idx = n - (taps - 1) + j;
                const float x = idx >= 0 ? to_float(proj[(int64_t)(start + idx) * ld + c]) : st[(int64_t)(taps - 1 + idx) * C + c];
                acc = fmaf(conv_w[(int64_t)c * taps + j], x, acc);
            }
        }
        return silu_f(acc);
    };
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) qk_s[i] = channel(i < D ? hk * D + i : nqk + hk * D + (i - D));
    __syncthreads();
    float qq[LP_PER], kk[LP_PER], sq = 0.f, sk = 0.f;
#pragma unroll
    for (int i = 0; i < LP_PER; ++i) {
        const int d = lane + i * 32;
        qq[i] = d < D ? qk_s[d] : 0.f;
        kk[i] = d < D ? qk_s[D + d] : 0.f;
        sq = fmaf(qq[i], qq[i], sq);
        sk = fmaf(kk[i], kk[i], sk);
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float rq = rsqrtf(sq + unit_eps) * rsqrtf((float)D), rk = rsqrtf(sk + unit_eps);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < LP_PER; ++i) {
        qq[i] *= rq;
        kk[i] *= rk;
        dot = fmaf(qq[i], kk[i], dot);
    }
    dot = warp_sum(dot);
    for (int h = hk * per_key + warp; h < (hk + 1) * per_key; h += n_warps) {
        const float beta = 1.f / (1.f + expf(-to_float(proj[(int64_t)t * ld + C + h])));
        const float rate = expf(a_log[h]);
        const int64_t o = ((int64_t)t * H + h) * D;
#pragma unroll
        for (int i = 0; i < LP_PER; ++i) {
            const int d = lane + i * 32;
            if (d < D) {
                q[o + d] = qq[i];
                kw[o + d] = kk[i];
                w[o + d] = expf(-rate * softplus_f(dpre[(int64_t)t * H * D + h * D + d] + dt_bias[h * D + d]));
            }
        }
        for (int d = lane; d < Dv; d += 32) v[((int64_t)t * H + h) * Dv + d] = channel(2 * nqk + h * Dv + d);
        if (lane == 0) {
            scal[((int64_t)t * H + h) * 2] = beta * dot;
            scal[((int64_t)t * H + h) * 2 + 1] = beta;
        }
    }
}

static unsigned lp_grid(int64_t items) { return (unsigned)((items + GP_BLOCK / 32 - 1) / (GP_BLOCK / 32)); }

IMP_API int imp_retention_prepare_ex(const void* proj, int64_t ld, int n_tokens, int H, int D, int Dv, float k_scale, int act, float* q, float* kw,
                                     float* v, float* scal, int act_dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(proj && q && kw && v && scal && H > 0 && D > 0 && Dv > 0 && ld >= (int64_t)2 * H * D + (int64_t)H * Dv && (act == 0 || act == 1),
                  "imp_retention_prepare: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(lp_grid((int64_t)n_tokens * H));
    if (act_dtype == IMP_F32)
        imp_launch(retention_prepare_kernel<float>, grid, dim3(GP_BLOCK), 0, s, (const float*)proj, ld, n_tokens, H, D, Dv, k_scale, act, q, kw, v, scal);
    else
        imp_launch(retention_prepare_kernel<__nv_bfloat16>, grid, dim3(GP_BLOCK), 0, s, (const __nv_bfloat16*)proj, ld, n_tokens, H, D, Dv, k_scale, act,
                   q, kw, v, scal);
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_retention_prepare(const void* proj, int64_t ld, int n_tokens, int H, int D, int Dv, float k_scale, float* q, float* kw, float* v,
                                  float* scal, int act_dtype, void* stream) {
    return imp_retention_prepare_ex(proj, ld, n_tokens, H, D, Dv, k_scale, 0, q, kw, v, scal, act_dtype, stream);
}

IMP_API int imp_gdelta_prepare(const void* proj, int64_t ld, const float* dlog, const float* w0, const float* a_bias, float decay_scale,
                               float unit_eps, int n_tokens, int H, int D, float* q, float* kw, float* w, float* p, float* z, float* v,
                               float* scal, int act_dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(proj && dlog && w0 && a_bias && q && kw && w && p && z && v && scal, "imp_gdelta_prepare: null pointer");
    IMP_CHECK_ARG(H > 0 && D > 0 && D <= LP_MAX_D && ld >= (int64_t)5 * H * D, "imp_gdelta_prepare: bad sizes (key size %d of at most %d)", D, LP_MAX_D);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(lp_grid((int64_t)n_tokens * H));
    if (act_dtype == IMP_F32)
        imp_launch(gdelta_prepare_kernel<float>, grid, dim3(GP_BLOCK), 0, s, (const float*)proj, ld, dlog, w0, a_bias, decay_scale, unit_eps, n_tokens,
                   H, D, q, kw, w, p, z, v, scal);
    else
        imp_launch(gdelta_prepare_kernel<__nv_bfloat16>, grid, dim3(GP_BLOCK), 0, s, (const __nv_bfloat16*)proj, ld, dlog, w0, a_bias, decay_scale,
                   unit_eps, n_tokens, H, D, q, kw, w, p, z, v, scal);
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_gdrc_prepare(const void* proj, int64_t ld, const float* conv_w, int taps, const float* conv_state, const int* seq_of_token,
                             const int* q_start, const int* slots, int n_tokens, int n_seqs, int G, int D, int H, int Dv, const float* dpre,
                             const float* a_log, const float* dt_bias, float unit_eps, float* q, float* kw, float* w, float* v, float* scal,
                             int act_dtype, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(proj && conv_w && conv_state && seq_of_token && q_start && slots && dpre && a_log && dt_bias && q && kw && w && v && scal,
                  "imp_gdrc_prepare: null pointer");
    IMP_CHECK_ARG(G > 0 && H > 0 && H % G == 0 && D > 0 && D <= LP_MAX_D && Dv > 0 && taps >= 1,
                  "imp_gdrc_prepare: bad sizes (heads %d over %d key heads, key size %d of at most %d)", H, G, D, LP_MAX_D);
    IMP_CHECK_ARG(ld >= (int64_t)2 * G * D + (int64_t)H * Dv + H, "imp_gdrc_prepare: the projection's rows are too short");
    cudaStream_t s = (cudaStream_t)stream;
    IMP_CHECK_ARG((int64_t)n_tokens * G <= 0x7fffffff, "imp_gdrc_prepare: too many tokens");
    const dim3 grid((unsigned)((int64_t)n_tokens * G));
    // a warp per value head of the key head, and enough threads for the key head's 2 D channels to be made in one or two rounds
    const int n_warps = std::max(std::min(H / G, GC_MAX_WARPS), std::min((D + 31) / 32, 4));
#define GDRC_PREPARE(TA, TAPS)                                                                                                          \
    imp_launch(gdrc_prepare_kernel<TA, TAPS>, grid, dim3(32 * n_warps), 0, s, (const TA*)proj, ld, conv_w, taps, conv_state, seq_of_token, q_start, \
               slots, n_tokens, n_seqs, G, D, H, Dv, dpre, a_log, dt_bias, unit_eps, q, kw, w, v, scal, status)
#define GDRC_PREPARE_T(TA)                       \
    do {                                         \
        if (taps == 4) GDRC_PREPARE(TA, 4);      \
        else if (taps == 3) GDRC_PREPARE(TA, 3); \
        else if (taps == 2) GDRC_PREPARE(TA, 2); \
        else GDRC_PREPARE(TA, 0);                \
    } while (0)
    if (act_dtype == IMP_F32) GDRC_PREPARE_T(float);
    else GDRC_PREPARE_T(__nv_bfloat16);
#undef GDRC_PREPARE_T
#undef GDRC_PREPARE
    IMP_RETURN_LAUNCH();
}
