// Between a q,k,v product and the paged attention kernels, for attention whose heads are normalised, rotated in
// part, scaled per head and whose values are normalised; and the small kernels of blocks that combine two mixers
// or gate their heads.
//
//   qkv_prepare      per token: q heads  -> RMS norm with a weight shared by the heads (optional), rotation of the
//                    first `rot` entries (pairs i, i + rot/2, or neighbours 2i, 2i + 1), times a number per head (optional) -> q_out, padded
//                    to the cache's head size; k heads -> norm, rotation -> K page; v heads -> divided by their
//                    root mean square (optional) -> V page.  Key and value heads may have different sizes: the
//                    cache's head size is the larger one, the rest of a row is zeros.  With v_share = n, n neighbouring key
//                    heads read one value head (the product holds Hkv / n of them) and each caches a copy of it.
//   diff_combine     two softmax maps per head over the same values: o = a1 - lambda * a2, o / rms(o) * out_scale
//   head_gate        y[t, h, :] *= sigmoid(g[t, h])
//   rms_pair_mean    out = ca * a / rms(a) * wa + cb * b / rms(b) * wb   (two branch outputs, each normalised over the width)
//   gated_act        out = act(gate) * up for gelu (tanh form) and silu over [gate | up] rows
//   act_rows         out[t, :] = act(x[t, c0 : c0 + n])  (a slice of a product's rows made dense, tanh or identity)
// Norm statistics, angles, the rotation and the per-head factors are 32-bit; results are rounded once.
#include "common.cuh"

constexpr int QP_BLOCK = 256;
constexpr int QP_WARPS = QP_BLOCK / 32;
constexpr int QP_UNITS = 16;     // units of one token a CTA takes, two a warp: the token's angles are made once for all of them
constexpr int QP_MAX_D = 512;

// A CTA per (token, group of QP_UNITS units), a warp per unit; units: Hq query heads, then Hkv key heads, then Hkv value
// heads; PER entries of a head a lane (the cache's head size is at most 32 * PER).
// proj: [T, ld] with columns [q: Hq*D | k: Hkv*D | v: Hkv*Dv | ...].  inv_freq: [rot/2] float32 (angle = pos * inv_freq[i]).
template <typename TA, int PER>
__global__ void __launch_bounds__(QP_BLOCK) qkv_prepare_kernel(
    const TA* __restrict__ proj, int64_t ld, int n_tokens, int Hq, int Hkv, int D, int Dv, int Dc, const float* __restrict__ q_norm_w,
    const float* __restrict__ k_norm_w, float eps, int v_norm, const float* __restrict__ inv_freq, int rot, int pairing, int v_share,
    const float* __restrict__ head_mult, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ block_table, int bt_stride, int n_seqs, TA* __restrict__ q_out, int64_t q_ld, TA* __restrict__ k_cache,
    TA* __restrict__ v_cache, int page_size, int num_pages, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float rot_s[QP_WARPS][32 * PER];
    __shared__ float cos_s[16 * PER], sin_s[16 * PER];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int units = Hq + 2 * Hkv;
    const int64_t t = blockIdx.x;
    const int seq = seq_of_token[t], pos = positions[t];
    if (seq < 0 || seq >= n_seqs || pos < 0 || pos / page_size >= bt_stride) {
        if (threadIdx.x == 0 && blockIdx.y == 0) imp_report(status, seq < 0 || seq >= n_seqs ? IMP_BAD_SEQUENCE : IMP_BAD_POSITION);
        return;
    }
    const int half = rot / 2;
    const int u_begin = blockIdx.y * QP_UNITS, u_end = min(units, u_begin + QP_UNITS);
    if (rot > 0 && u_begin < Hq + Hkv) {     // a group of value heads rotates nothing
        for (int i = threadIdx.x; i < half; i += QP_BLOCK) sincosf((float)pos * inv_freq[i], &sin_s[i], &cos_s[i]);
    }
    __syncthreads();
    const int page = block_table[(int64_t)seq * bt_stride + pos / page_size];
    for (int unit = u_begin + warp; unit < u_end; unit += QP_WARPS) {
        const bool is_q = unit < Hq, is_v = unit >= Hq + Hkv;
        const int head = is_q ? unit : is_v ? unit - Hq - Hkv : unit - Hq;
        const int n = is_v ? Dv : D;
        const TA* src = proj + t * ld + (is_q ? (int64_t)head * D : is_v ? (int64_t)Hq * D + (int64_t)Hkv * D + (int64_t)(head / v_share) * Dv
                                                                         : (int64_t)Hq * D + (int64_t)head * D);
        TA* dst;
        if (is_q) {
            dst = q_out + t * q_ld + (int64_t)head * Dc;
        } else {
            if (page < 0 || page >= num_pages) {
                if (lane == 0) imp_report(status, IMP_BAD_PAGE);
                continue;
            }
            TA* cache = is_v ? v_cache : k_cache;
            if (!cache) continue;
            dst = cache + (((int64_t)page * Hkv + head) * page_size + pos % page_size) * Dc;   // pages are [page][kv head][slot][entry]
        }
        float x[PER], ss = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + i * 32;
            x[i] = d < n ? to_float(src[d]) : 0.f;
            ss = fmaf(x[i], x[i], ss);
        }
        const float* nw = is_q ? q_norm_w : is_v ? nullptr : k_norm_w;
        const bool normed = is_v ? v_norm != 0 : nw != nullptr;
        if (normed) {
            ss = warp_sum(ss);
            const float r = rsqrtf(ss / (float)n + eps);
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int d = lane + i * 32;
                if (d < n) x[i] = x[i] * r * (nw ? nw[d] : 1.f);
            }
        }
        if (!is_v && rot > 0 && pairing == 1) {
            // neighbours: entry 2i pairs with 2i + 1, which the next lane holds, at angle pos * inv_freq[i]
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int d = lane + i * 32;
                const float partner = __shfl_xor_sync(0xffffffffu, x[i], 1);
                if (d < rot) {
                    const float sn = sin_s[d >> 1], cs = cos_s[d >> 1];
                    x[i] = (d & 1) ? x[i] * cs + partner * sn : x[i] * cs - partner * sn;
                }
            }
        } else if (!is_v && rot > 0) {
            // entry d < rot/2 pairs with d + rot/2, which another lane holds: the head goes through shared memory once
            float* row = rot_s[warp];
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int d = lane + i * 32;
                if (d < rot) row[d] = x[i];
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int d = lane + i * 32;
                if (d < rot) {
                    const int fi = d < half ? d : d - half;
                    const float partner = row[d < half ? d + half : d - half];
                    const float sn = sin_s[fi], cs = cos_s[fi];
                    // (u, v) -> (u cos - v sin, v cos + u sin)
                    x[i] = d < half ? x[i] * cs - partner * sn : x[i] * cs + partner * sn;
                }
            }
            __syncwarp();     // the row is written again for the warp's next unit
        }
        const float mult = (is_q && head_mult) ? head_mult[head] : 1.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + i * 32;
            if (d < Dc) dst[d] = from_float<TA>(d < n ? x[i] * mult : 0.f);
        }
    }
}

// y[t, h, :] *= sigmoid(g[t, h]); a warp per (token, head).
template <typename TA>
__global__ void head_gate_kernel(TA* __restrict__ y, int64_t y_ld, const TA* __restrict__ g, int64_t g_ld, int n_tokens, int H, int Dv) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_tokens * H) return;
    const int64_t t = item / H;
    const int h = (int)(item - t * H);
    const float s = 1.f / (1.f + expf(-to_float(g[t * g_ld + h])));
    TA* row = y + t * y_ld + (int64_t)h * Dv;
    for (int d = lane; d < Dv; d += 32) row[d] = from_float<TA>(to_float(row[d]) * s);
}

// out[r] = ca * a[r] / rms(a[r]) * wa + cb * b[r] / rms(b[r]) * wb; one block per row, the two sums of squares in 32-bit.
template <typename TA>
__global__ void __launch_bounds__(256) rms_pair_mean_kernel(TA* __restrict__ out, const TA* __restrict__ a, const float* __restrict__ wa, float ca,
                                                            const TA* __restrict__ b, const float* __restrict__ wb, float cb, int d, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int64_t r = blockIdx.x;
    const TA* ar = a + r * d;
    const TA* br = b + r * d;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float x = to_float(ar[i]), y = to_float(br[i]);
        sa = fmaf(x, x, sa);
        sb = fmaf(y, y, sb);
    }
    const float ra = rsqrtf(block_sum(sa, scratch) / (float)d + eps) * ca;
    const float rb = rsqrtf(block_sum(sb, scratch) / (float)d + eps) * cb;
    TA* o = out + r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_float<TA>(fmaf(to_float(ar[i]) * ra, wa[i], to_float(br[i]) * rb * wb[i]));
}

// out[t, f] = act(gate) * up over rows [gate | up] (block == 0) or runs of `block` gate entries followed by their up entries.
// act: 0 silu, 1 gelu (tanh form).
template <typename T>
__global__ void gated_act_kernel(T* __restrict__ out, const T* __restrict__ gu, int64_t n_tokens, int F, int block, int act) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t total = n_tokens * (int64_t)F;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / F;
        const int f = (int)(i - t * F);
        const int gi = block ? (f / block) * 2 * block + f % block : f;
        const int ui = block ? gi + block : F + f;
        const float g = to_float(gu[t * 2 * F + gi]);
        const float u = to_float(gu[t * 2 * F + ui]);
        const float a = gate_act_f(g, act);
        out[i] = from_float<T>(a * u);
    }
}

// out[t, j] = act(x[t, j]) for j < n: a dense copy of a slice of wider rows.  act: 0 identity, 1 tanh.
template <typename T>
__global__ void act_rows_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t ld, int64_t n_tokens, int n, int act) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t total = n_tokens * (int64_t)n;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / n;
        const float v = to_float(x[t * ld + (i - t * n)]);
        out[i] = from_float<T>(act == 1 ? tanhf(v) : v);
    }
}


// attn [T, ld] holds, per token, G groups x 2 maps x R query heads of Dc entries (the order the paged attention kernels
// want: the R heads of a map of a group share that map's key head).  Head h = g * R + j of the result:
//   o = a[g, 0, j] - lambda * a[g, 1, j] over the first Dv entries;  y[t, h, :] = o / sqrt(mean(o^2) + eps) * out_scale.
// A warp per (token, head); the difference and the norm in 32-bit.
template <typename TA>
__global__ void diff_combine_kernel(TA* __restrict__ y, const TA* __restrict__ attn, int64_t ld, int n_tokens, int G, int R, int Dc, int Dv,
                                    const float* __restrict__ lambda, float eps, float out_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int H = G * R;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_tokens * H) return;
    const int64_t t = item / H;
    const int h = (int)(item - t * H), g = h / R, j = h - g * R;
    const TA* a1 = attn + t * ld + ((int64_t)(g * 2) * R + j) * Dc;
    const TA* a2 = a1 + (int64_t)R * Dc;
    const float lam = lambda[0];
    float o[QP_MAX_D / 32], ss = 0.f;
#pragma unroll
    for (int i = 0; i < QP_MAX_D / 32; ++i) {
        const int d = lane + i * 32;
        o[i] = d < Dv ? fmaf(-lam, to_float(a2[d]), to_float(a1[d])) : 0.f;
        ss = fmaf(o[i], o[i], ss);
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)Dv + eps) * out_scale;
    TA* dst = y + (t * H + h) * Dv;
#pragma unroll
    for (int i = 0; i < QP_MAX_D / 32; ++i) {
        const int d = lane + i * 32;
        if (d < Dv) dst[d] = from_float<TA>(o[i] * r);
    }
}

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a), u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

// The same with four neighbouring entries a lane (8-byte loads of 16-bit values): Dv and Dc multiples of 4, rows 8-byte aligned.
template <typename TA>
__global__ void diff_combine_vec_kernel(TA* __restrict__ y, const TA* __restrict__ attn, int64_t ld, int n_tokens, int G, int R, int Dc, int Dv,
                                        const float* __restrict__ lambda, float eps, float out_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int H = G * R;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_tokens * H) return;
    const int64_t t = item / H;
    const int h = (int)(item - t * H), g = h / R, j = h - g * R;
    const TA* a1 = attn + t * ld + ((int64_t)(g * 2) * R + j) * Dc;
    const TA* a2 = a1 + (int64_t)R * Dc;
    const float lam = lambda[0];
    float4 o[QP_MAX_D / 128];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < QP_MAX_D / 128; ++i) {
        const int d = (lane + i * 32) * 4;
        o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (d < Dv) {
            const float4 p = load4(a1 + d), q = load4(a2 + d);
            o[i] = make_float4(fmaf(-lam, q.x, p.x), fmaf(-lam, q.y, p.y), fmaf(-lam, q.z, p.z), fmaf(-lam, q.w, p.w));
        }
        ss += (o[i].x * o[i].x + o[i].y * o[i].y) + (o[i].z * o[i].z + o[i].w * o[i].w);
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)Dv + eps) * out_scale;
    TA* dst = y + (t * H + h) * Dv;
#pragma unroll
    for (int i = 0; i < QP_MAX_D / 128; ++i) {
        const int d = (lane + i * 32) * 4;
        if (d < Dv) store4(dst + d, make_float4(o[i].x * r, o[i].y * r, o[i].z * r, o[i].w * r));
    }
}

IMP_API int imp_qkv_prepare_ex(const void* proj, int64_t ld, int n_tokens, int Hq, int Hkv, int D, int Dv, int Dc, const float* q_norm_w,
                               const float* k_norm_w, float eps, int v_norm, const float* inv_freq, int rot, int pairing, int v_share,
                               const float* head_mult, const int* positions, const int* seq_of_token, const int* block_table, int bt_stride,
                               int n_seqs, void* q_out, int64_t q_ld, void* k_cache, void* v_cache, int page_size, int num_pages, int act_dtype,
                               int* status, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(proj && positions && seq_of_token && block_table && q_out, "imp_qkv_prepare: null pointer");
    IMP_CHECK_ARG(Hq > 0 && Hkv > 0 && D > 0 && Dv > 0 && Dc >= D && Dc >= Dv && Dc <= QP_MAX_D,
                  "imp_qkv_prepare: head sizes %d / %d must fit the cache's %d (at most %d)", D, Dv, Dc, QP_MAX_D);
    IMP_CHECK_ARG(rot >= 0 && rot % 2 == 0 && rot <= D && (rot == 0 || inv_freq), "imp_qkv_prepare: the rotated part must be even and within the head");
    IMP_CHECK_ARG((q_norm_w == nullptr) == (k_norm_w == nullptr), "imp_qkv_prepare: q and k are normalised together or not at all");
    IMP_CHECK_ARG((pairing == 0 || pairing == 1) && v_share > 0 && Hkv % v_share == 0, "imp_qkv_prepare: pairing is 0 (halves) or 1 (neighbours); v_share divides the key heads");
    IMP_CHECK_ARG(ld >= (int64_t)(Hq + Hkv) * D + (int64_t)(Hkv / v_share) * Dv && q_ld >= (int64_t)Hq * Dc, "imp_qkv_prepare: rows too short");
    IMP_CHECK_ARG(page_size > 0 && num_pages > 0, "imp_qkv_prepare: bad cache geometry");
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((unsigned)n_tokens, (unsigned)((Hq + 2 * Hkv + QP_UNITS - 1) / QP_UNITS));
#define QP_LAUNCH(TA, PER)                                                                                                                    \
    imp_launch(qkv_prepare_kernel<TA, PER>, grid, dim3(QP_BLOCK), 0, s, (const TA*)proj, ld, n_tokens, Hq, Hkv, D, Dv, Dc, q_norm_w, k_norm_w, eps, \
               v_norm, inv_freq, rot, pairing, v_share, head_mult, positions, seq_of_token, block_table, bt_stride, n_seqs, (TA*)q_out, q_ld, (TA*)k_cache,     \
               (TA*)v_cache, page_size, num_pages, status)
#define QP_LAUNCH_PER(TA)                       \
    do {                                        \
        if (Dc <= 64) QP_LAUNCH(TA, 2);         \
        else if (Dc <= 128) QP_LAUNCH(TA, 4);   \
        else if (Dc <= 256) QP_LAUNCH(TA, 8);   \
        else QP_LAUNCH(TA, 16);                 \
    } while (0)
    if (act_dtype == IMP_F32) QP_LAUNCH_PER(float);
    else QP_LAUNCH_PER(__nv_bfloat16);
#undef QP_LAUNCH_PER
#undef QP_LAUNCH
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_qkv_prepare(const void* proj, int64_t ld, int n_tokens, int Hq, int Hkv, int D, int Dv, int Dc, const float* q_norm_w,
                            const float* k_norm_w, float eps, int v_norm, const float* inv_freq, int rot, const float* head_mult,
                            const int* positions, const int* seq_of_token, const int* block_table, int bt_stride, int n_seqs, void* q_out,
                            int64_t q_ld, void* k_cache, void* v_cache, int page_size, int num_pages, int act_dtype, int* status,
                            void* stream) {
    return imp_qkv_prepare_ex(proj, ld, n_tokens, Hq, Hkv, D, Dv, Dc, q_norm_w, k_norm_w, eps, v_norm, inv_freq, rot, 0, 1, head_mult, positions,
                              seq_of_token, block_table, bt_stride, n_seqs, q_out, q_ld, k_cache, v_cache, page_size, num_pages, act_dtype, status,
                              stream);
}

// y [T, G * R * Dv] dense; attn rows `ld` apart; lambda: one float32 on the device.
IMP_API int imp_diff_combine(void* y, const void* attn, int64_t ld, int n_tokens, int G, int R, int Dc, int Dv, const float* lambda, float eps,
                             float out_scale, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(y && attn && lambda && G > 0 && R > 0 && Dv > 0 && Dv <= Dc && Dc <= QP_MAX_D && ld >= (int64_t)2 * G * R * Dc,
                  "imp_diff_combine: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t items = (int64_t)n_tokens * G * R;
    const dim3 grid((unsigned)((items + 7) / 8));
    const size_t el = dtype == IMP_F32 ? 4 : 2;
    if (Dv % 4 == 0 && Dc % 4 == 0 && (ld * el) % (4 * el) == 0 && (uintptr_t)attn % (4 * el) == 0 && (uintptr_t)y % (4 * el) == 0) {
        if (dtype == IMP_F32)
            imp_launch(diff_combine_vec_kernel<float>, grid, dim3(256), 0, s, (float*)y, (const float*)attn, ld, n_tokens, G, R, Dc, Dv, lambda, eps, out_scale);
        else
            imp_launch(diff_combine_vec_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (__nv_bfloat16*)y, (const __nv_bfloat16*)attn, ld, n_tokens, G, R, Dc,
                       Dv, lambda, eps, out_scale);
        IMP_RETURN_LAUNCH();
    }
    if (dtype == IMP_F32)
        imp_launch(diff_combine_kernel<float>, grid, dim3(256), 0, s, (float*)y, (const float*)attn, ld, n_tokens, G, R, Dc, Dv, lambda, eps, out_scale);
    else
        imp_launch(diff_combine_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (__nv_bfloat16*)y, (const __nv_bfloat16*)attn, ld, n_tokens, G, R, Dc, Dv,
                   lambda, eps, out_scale);
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_head_gate(void* y, int64_t y_ld, const void* g, int64_t g_ld, int n_tokens, int H, int Dv, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(y && g && H > 0 && Dv > 0 && y_ld >= (int64_t)H * Dv && g_ld >= H, "imp_head_gate: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t items = (int64_t)n_tokens * H;
    const dim3 grid((unsigned)((items + 7) / 8));
    if (dtype == IMP_F32) imp_launch(head_gate_kernel<float>, grid, dim3(256), 0, s, (float*)y, y_ld, (const float*)g, g_ld, n_tokens, H, Dv);
    else imp_launch(head_gate_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (__nv_bfloat16*)y, y_ld, (const __nv_bfloat16*)g, g_ld, n_tokens, H, Dv);
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_rms_pair_mean(void* out, const void* a, const float* wa, float ca, const void* b, const float* wb, float cb, int n_rows, int d,
                              float eps, int dtype, void* stream) {
    if (n_rows == 0) return 0;
    IMP_CHECK_ARG(out && a && b && wa && wb && d > 0, "imp_rms_pair_mean: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == IMP_F32)
        imp_launch(rms_pair_mean_kernel<float>, dim3(n_rows), dim3(256), 0, s, (float*)out, (const float*)a, wa, ca, (const float*)b, wb, cb, d, eps);
    else
        imp_launch(rms_pair_mean_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)a, wa, ca,
                   (const __nv_bfloat16*)b, wb, cb, d, eps);
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_gated_act(void* out, const void* gate_up, int n_tokens, int F, int block, int act, int dtype, void* stream) {
    if (n_tokens == 0 || F == 0) return 0;
    IMP_CHECK_ARG(out && gate_up && n_tokens > 0 && F > 0 && block >= 0 && (block == 0 || F % block == 0) && (act == 0 || act == 1),
                  "imp_gated_act: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t total = (int64_t)n_tokens * F;
    const dim3 grid((unsigned)std::min<int64_t>((total + 255) / 256, 65535));
    if (dtype == IMP_F32) imp_launch(gated_act_kernel<float>, grid, dim3(256), 0, s, (float*)out, (const float*)gate_up, (int64_t)n_tokens, F, block, act);
    else imp_launch(gated_act_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, (int64_t)n_tokens, F, block, act);
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_act_rows(void* out, const void* x, int64_t ld, int n_tokens, int n, int act, int dtype, void* stream) {
    if (n_tokens == 0 || n == 0) return 0;
    IMP_CHECK_ARG(out && x && n > 0 && ld >= n && (act == 0 || act == 1), "imp_act_rows: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t total = (int64_t)n_tokens * n;
    const dim3 grid((unsigned)std::min<int64_t>((total + 255) / 256, 65535));
    if (dtype == IMP_F32) imp_launch(act_rows_kernel<float>, grid, dim3(256), 0, s, (float*)out, (const float*)x, ld, (int64_t)n_tokens, n, act);
    else imp_launch(act_rows_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, ld, (int64_t)n_tokens, n, act);
    IMP_RETURN_LAUNCH();
}

// dst[t, h, 0:n] = src[t, h, 0:n] out of heads of `ds` entries: the heads' first n columns as dense rows.
template <typename T>
__global__ void gather_head_cols_kernel(T* __restrict__ dst, const T* __restrict__ src, int64_t n_tokens, int H, int ds, int n) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t total = n_tokens * (int64_t)H * n;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t th = i / n;
        dst[i] = src[th * ds + (i - th * n)];
    }
}

IMP_API int imp_gather_head_cols(void* dst, const void* src, int n_tokens, int H, int ds, int n, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(dst && src && H > 0 && n > 0 && ds >= n, "imp_gather_head_cols: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t total = (int64_t)n_tokens * H * n;
    const dim3 grid((unsigned)std::min<int64_t>((total + 255) / 256, 65535));
    if (dtype == IMP_F32) imp_launch(gather_head_cols_kernel<float>, grid, dim3(256), 0, s, (float*)dst, (const float*)src, (int64_t)n_tokens, H, ds, n);
    else imp_launch(gather_head_cols_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (__nv_bfloat16*)dst, (const __nv_bfloat16*)src, (int64_t)n_tokens, H, ds, n);
    IMP_RETURN_LAUNCH();
}
