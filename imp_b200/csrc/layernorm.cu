// Layer norm with a weight and an optional bias, fused with the residual sum, and the small kernels that go
// with a stream whose branches carry a factor per column.
//
//   h  = m h + s (.) branch      (m: a constant, 1 unless given; s: 32-bit factor per column, optional; branch optional)
//   y  = (h - mean(h)) / sqrt(var(h) + eps) * w (+ b),   var = mean((h - mean)^2)
//
// write_h: 0 leaves the stream as it is, 1 stores the sum (pre-norm: the stream is the sum), 2 stores y in 32-bit
// (post-norm: the normalised sum is the stream).
//
// The residual stream is 32-bit; mean, variance and the scaling are 32-bit.  One block per row with a
// fixed block size; the row is held in registers between the passes (up to LN_MAX_PER_THREAD values a
// thread, the rest re-read), so the order of every sum depends on the width alone.
#include "common.cuh"

constexpr int LN_BLOCK = 256;
constexpr int LN_KEEP = 16;   // values a thread keeps in registers: rows up to 4096 wide are read once

template <typename TA, typename TW>
__global__ void __launch_bounds__(LN_BLOCK) add_layernorm_kernel(float* __restrict__ h, const TA* __restrict__ branch,
                                                                 const float* __restrict__ col_scale, const TW* __restrict__ w,
                                                                 TA* __restrict__ out, const int* __restrict__ rows, int d, float eps,
                                                                 int write_h, float h_mult, const TW* __restrict__ bias) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int64_t src = rows ? rows[r] : r;
    float* hrow = h + src * d;
    const TA* brow = branch ? branch + src * d : nullptr;
    float keep[LN_KEEP];
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < LN_KEEP; ++e) {
        const int i = threadIdx.x + e * LN_BLOCK;
        float v = 0.f;
        if (i < d) {
            v = hrow[i] * h_mult;
            if (brow) v = col_scale ? fmaf(col_scale[i], to_float(brow[i]), v) : v + to_float(brow[i]);
            if (write_h == 1 && brow) hrow[i] = v;
        }
        keep[e] = v;
        sum += v;
    }
    for (int i = threadIdx.x + LN_KEEP * LN_BLOCK; i < d; i += LN_BLOCK) {
        float v = hrow[i] * h_mult;
        if (brow) v = col_scale ? fmaf(col_scale[i], to_float(brow[i]), v) : v + to_float(brow[i]);
        if (write_h == 1 && brow) hrow[i] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)d;
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < LN_KEEP; ++e) {
        const int i = threadIdx.x + e * LN_BLOCK;
        if (i < d) {
            const float c = keep[e] - mean;
            ss = fmaf(c, c, ss);
        }
    }
    const bool stored = write_h == 1 && brow;   // beyond the kept part the row is read again: from h if it was stored, else recomputed
    for (int i = threadIdx.x + LN_KEEP * LN_BLOCK; i < d; i += LN_BLOCK) {
        float v = stored ? hrow[i] : hrow[i] * h_mult;
        if (brow && !stored) v = col_scale ? fmaf(col_scale[i], to_float(brow[i]), v) : v + to_float(brow[i]);
        const float c = v - mean;
        ss = fmaf(c, c, ss);
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)d + eps);
    TA* orow = out + (int64_t)r * d;
#pragma unroll
    for (int e = 0; e < LN_KEEP; ++e) {
        const int i = threadIdx.x + e * LN_BLOCK;
        if (i < d) {
            const float y = fmaf((keep[e] - mean) * inv, to_float(w[i]), bias ? to_float(bias[i]) : 0.f);
            orow[i] = from_float<TA>(y);
            if (write_h == 2) hrow[i] = y;
        }
    }
    // the part of the row that is read again is normalised in place only after every thread has read what it needs:
    // each thread rewrites the entries it alone reads
    for (int i = threadIdx.x + LN_KEEP * LN_BLOCK; i < d; i += LN_BLOCK) {
        float v = stored ? hrow[i] : hrow[i] * h_mult;
        if (brow && !stored) v = col_scale ? fmaf(col_scale[i], to_float(brow[i]), v) : v + to_float(brow[i]);
        const float y = fmaf((v - mean) * inv, to_float(w[i]), bias ? to_float(bias[i]) : 0.f);
        orow[i] = from_float<TA>(y);
        if (write_h == 2) hrow[i] = y;
    }
}

template <typename T> struct Vec4 {};
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&a);
        u.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

// Rows whose width is a multiple of 4, up to 256 x NV x 4 columns: the row is read once with 16-byte loads issued together,
// kept in registers (NV float4 a thread) and written from there.
template <typename TA, typename TW, int NV>
__global__ void __launch_bounds__(LN_BLOCK) add_layernorm_vec_kernel(float* __restrict__ h, const TA* __restrict__ branch,
                                                                     const float* __restrict__ col_scale, const TW* __restrict__ w,
                                                                     TA* __restrict__ out, const int* __restrict__ rows, int d, float eps,
                                                                     int write_h, float h_mult, const TW* __restrict__ bias) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int64_t src = rows ? rows[r] : r;
    float* hrow = h + src * d;
    const TA* brow = branch ? branch + src * d : nullptr;
    float4 v[NV];
#pragma unroll
    for (int e = 0; e < NV; ++e) {
        const int i = (threadIdx.x + e * LN_BLOCK) * 4;
        v[e] = i < d ? Vec4<float>::load(hrow + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        v[e].x *= h_mult, v[e].y *= h_mult, v[e].z *= h_mult, v[e].w *= h_mult;
    }
    if (brow) {
#pragma unroll
        for (int e = 0; e < NV; ++e) {
            const int i = (threadIdx.x + e * LN_BLOCK) * 4;
            if (i < d) {
                const float4 b = Vec4<TA>::load(brow + i);
                if (col_scale) {
                    const float4 s = Vec4<float>::load(col_scale + i);
                    v[e].x = fmaf(s.x, b.x, v[e].x), v[e].y = fmaf(s.y, b.y, v[e].y), v[e].z = fmaf(s.z, b.z, v[e].z), v[e].w = fmaf(s.w, b.w, v[e].w);
                } else {
                    v[e].x += b.x, v[e].y += b.y, v[e].z += b.z, v[e].w += b.w;
                }
                if (write_h == 1) Vec4<float>::store(hrow + i, v[e]);
            }
        }
    }
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < NV; ++e) sum += (v[e].x + v[e].y) + (v[e].z + v[e].w);
    const float mean = block_sum(sum, scratch) / (float)d;
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < NV; ++e) {
        const int i = (threadIdx.x + e * LN_BLOCK) * 4;
        if (i < d) {
            const float a = v[e].x - mean, b = v[e].y - mean, c = v[e].z - mean, g = v[e].w - mean;
            ss += (a * a + b * b) + (c * c + g * g);
        }
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)d + eps);
    TA* orow = out + (int64_t)r * d;
#pragma unroll
    for (int e = 0; e < NV; ++e) {
        const int i = (threadIdx.x + e * LN_BLOCK) * 4;
        if (i < d) {
            const float4 ww = Vec4<TW>::load(w + i);
            const float4 bb = bias ? Vec4<TW>::load(bias + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 y = make_float4(fmaf((v[e].x - mean) * inv, ww.x, bb.x), fmaf((v[e].y - mean) * inv, ww.y, bb.y),
                                         fmaf((v[e].z - mean) * inv, ww.z, bb.z), fmaf((v[e].w - mean) * inv, ww.w, bb.w));
            Vec4<TA>::store(orow + i, y);
            if (write_h == 2) Vec4<float>::store(hrow + i, y);
        }
    }
}

template <typename TA, typename TW>
static cudaError_t launch_layernorm(float* h, const void* branch, const float* col_scale, const void* w, void* out, const int* rows, int n, int d,
                                    float eps, int write_h, float h_mult, const void* bias_v, cudaStream_t s) {
    const TW* bias = (const TW*)bias_v;
    const dim3 grid(n), block(LN_BLOCK);
    const bool vec = d % 4 == 0 && d <= LN_BLOCK * 4 * 8 && (uintptr_t)h % 16 == 0 && (uintptr_t)branch % 8 == 0 && (uintptr_t)out % 8 == 0 &&
                     (uintptr_t)w % 16 == 0 && (uintptr_t)col_scale % 16 == 0 && (uintptr_t)bias_v % 16 == 0;
    if (vec) {
        const int nv = (d / 4 + LN_BLOCK - 1) / LN_BLOCK;
        if (nv <= 1) return imp_launch(add_layernorm_vec_kernel<TA, TW, 1>, grid, block, 0, s, h, (const TA*)branch, col_scale, (const TW*)w, (TA*)out, rows, d, eps, write_h, h_mult, bias);
        if (nv <= 2) return imp_launch(add_layernorm_vec_kernel<TA, TW, 2>, grid, block, 0, s, h, (const TA*)branch, col_scale, (const TW*)w, (TA*)out, rows, d, eps, write_h, h_mult, bias);
        if (nv <= 4) return imp_launch(add_layernorm_vec_kernel<TA, TW, 4>, grid, block, 0, s, h, (const TA*)branch, col_scale, (const TW*)w, (TA*)out, rows, d, eps, write_h, h_mult, bias);
        return imp_launch(add_layernorm_vec_kernel<TA, TW, 8>, grid, block, 0, s, h, (const TA*)branch, col_scale, (const TW*)w, (TA*)out, rows, d, eps, write_h, h_mult, bias);
    }
    return imp_launch(add_layernorm_kernel<TA, TW>, grid, block, 0, s, h, (const TA*)branch, col_scale, (const TW*)w, (TA*)out, rows, d, eps, write_h, h_mult, bias);
}

// h: [*, d] float32 stream, taken times h_mult; branch (optional, dense [*, d] of the activation type) is added, times
// col_scale (optional float32 [d]).  bias: optional, of the weight's type.  rows: optional gather list (then h is left as it
// is: write_h must be 0).  write_h: 1 stores the sum in h, 2 stores the normalised result in h.
IMP_API int imp_add_layernorm_ex(float* h, float h_mult, const void* branch, const float* col_scale, const void* w, const void* bias, void* out,
                                 const int* rows, int n_out_rows, int d, float eps, int act_dtype, int w_dtype, int write_h, void* stream) {
    if (n_out_rows == 0) return 0;
    IMP_CHECK_ARG(h && w && out && d > 0 && n_out_rows > 0 && write_h >= 0 && write_h <= 2, "imp_add_layernorm: bad argument");
    IMP_CHECK_ARG(!(rows && write_h), "imp_add_layernorm: a gather list and write_h exclude each other");
    IMP_CHECK_ARG(write_h != 1 || h_mult == 1.f || branch, "imp_add_layernorm: a scaled stream is stored with its branch only");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (act_dtype == IMP_F32)
        e = w_dtype == IMP_F32 ? launch_layernorm<float, float>(h, branch, col_scale, w, out, rows, n_out_rows, d, eps, write_h, h_mult, bias, s)
                               : launch_layernorm<float, __nv_bfloat16>(h, branch, col_scale, w, out, rows, n_out_rows, d, eps, write_h, h_mult, bias, s);
    else
        e = w_dtype == IMP_F32 ? launch_layernorm<__nv_bfloat16, float>(h, branch, col_scale, w, out, rows, n_out_rows, d, eps, write_h, h_mult, bias, s)
                               : launch_layernorm<__nv_bfloat16, __nv_bfloat16>(h, branch, col_scale, w, out, rows, n_out_rows, d, eps, write_h, h_mult, bias, s);
    if (e != cudaSuccess) {
        imp_set_error("imp_add_layernorm: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

IMP_API int imp_add_layernorm(float* h, const void* branch, const float* col_scale, const void* w, void* out, const int* rows,
                              int n_out_rows, int d, float eps, int act_dtype, int w_dtype, int write_h, void* stream) {
    return imp_add_layernorm_ex(h, 1.f, branch, col_scale, w, nullptr, out, rows, n_out_rows, d, eps, act_dtype, w_dtype, write_h ? 1 : 0, stream);
}

// x[r][c] *= s[c], the product made in 32-bit.
template <typename TA> __global__ void scale_columns_kernel(TA* __restrict__ x, int64_t stride, int n_cols, const float* __restrict__ s) {
    pdl_wait();
    pdl_launch_dependents();
    TA* row = x + (int64_t)blockIdx.x * stride;
    for (int i = threadIdx.x; i < n_cols; i += blockDim.x) row[i] = from_float<TA>(to_float(row[i]) * s[i]);
}

IMP_API int imp_scale_columns(void* x, int64_t stride, int n_rows, int n_cols, const float* s, int dtype, void* stream) {
    if (n_rows == 0 || n_cols == 0) return 0;
    IMP_CHECK_ARG(x && s && n_rows > 0 && n_cols > 0, "imp_scale_columns: bad argument");
    cudaError_t e = dtype == IMP_F32
                        ? imp_launch(scale_columns_kernel<float>, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, (float*)x, stride, n_cols, s)
                        : imp_launch(scale_columns_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream,
                                     (__nv_bfloat16*)x, stride, n_cols, s);
    if (e != cudaSuccess) {
        imp_set_error("imp_scale_columns: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// out[r] = [ h[r] + s (.) branch[r] ; x0[r] ] rounded to the activation type: the input of a map over the stream and
// a second stream side by side.  The sum is not stored: whoever runs the map overwrites h with its result.
template <typename TA>
__global__ void concat_streams_kernel(TA* __restrict__ out, const float* __restrict__ h, const TA* __restrict__ branch,
                                      const float* __restrict__ col_scale, const float* __restrict__ x0, int d) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t r = blockIdx.x;
    const float* hrow = h + r * d;
    const float* xrow = x0 + r * d;
    const TA* brow = branch ? branch + r * d : nullptr;
    TA* orow = out + r * 2 * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = hrow[i];
        if (brow) v = col_scale ? fmaf(col_scale[i], to_float(brow[i]), v) : v + to_float(brow[i]);
        orow[i] = from_float<TA>(v);
        orow[d + i] = from_float<TA>(xrow[i]);
    }
}

IMP_API int imp_concat_streams(void* out, const float* h, const void* branch, const float* col_scale, const float* x0, int n_rows,
                               int d, int act_dtype, void* stream) {
    if (n_rows == 0) return 0;
    IMP_CHECK_ARG(out && h && x0 && n_rows > 0 && d > 0, "imp_concat_streams: bad argument");
    cudaError_t e = act_dtype == IMP_F32
                        ? imp_launch(concat_streams_kernel<float>, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, (float*)out, h,
                                     (const float*)branch, col_scale, x0, d)
                        : imp_launch(concat_streams_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream,
                                     (__nv_bfloat16*)out, h, (const __nv_bfloat16*)branch, col_scale, x0, d);
    if (e != cudaSuccess) {
        imp_set_error("imp_concat_streams: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// A branch that is layer-normed before it joins the stream, and the stream's next norm, in one pass:
//   n  = (branch - mean(branch)) / sqrt(var(branch) + eps_b) * bw + bb        (the branch's own norm)
//   h  = h + n                                                                (stored when write_h)
//   y  = (h - mean(h)) / sqrt(var(h) + eps) * w + b                           (the next norm; left out when w is null)
// Without h the kernel is the branch's norm alone: out = n in the activation type.  One CTA per row; the branch row and the
// sum wait in shared memory as 32-bit values between the passes, so every sum's order depends on the width alone.
template <typename TA, typename TW>
__global__ void __launch_bounds__(LN_BLOCK) add_normed_layernorm_kernel(float* __restrict__ h, const TA* __restrict__ branch, const TW* __restrict__ bw,
                                                                        const TW* __restrict__ bb, float eps_b, const TW* __restrict__ w,
                                                                        const TW* __restrict__ bias, float eps, TA* __restrict__ out,
                                                                        const int* __restrict__ rows, int d, int write_h) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float ln_rows[];   // the branch row [d], then the sum [d]
    __shared__ float scratch[33];
    float* bs = ln_rows;
    float* hs = ln_rows + d;
    const int r = blockIdx.x;
    const int64_t src = rows ? rows[r] : r;
    const TA* brow = branch + src * d;
    float sum = 0.f;
    for (int i = threadIdx.x; i < d; i += LN_BLOCK) {
        const float v = to_float(brow[i]);
        bs[i] = v;
        sum += v;
    }
    const float mean_b = block_sum(sum, scratch) / (float)d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += LN_BLOCK) {
        const float c = bs[i] - mean_b;
        ss = fmaf(c, c, ss);
    }
    const float inv_b = rsqrtf(block_sum(ss, scratch) / (float)d + eps_b);
    TA* orow = out ? out + (int64_t)r * d : nullptr;
    if (!h) {
        for (int i = threadIdx.x; i < d; i += LN_BLOCK)
            orow[i] = from_float<TA>(fmaf((bs[i] - mean_b) * inv_b, to_float(bw[i]), bb ? to_float(bb[i]) : 0.f));
        return;
    }
    float* hrow = h + src * d;
    sum = 0.f;
    for (int i = threadIdx.x; i < d; i += LN_BLOCK) {
        const float v = hrow[i] + fmaf((bs[i] - mean_b) * inv_b, to_float(bw[i]), bb ? to_float(bb[i]) : 0.f);
        if (write_h) hrow[i] = v;
        hs[i] = v;
        sum += v;
    }
    if (!w) return;
    const float mean = block_sum(sum, scratch) / (float)d;
    ss = 0.f;
    for (int i = threadIdx.x; i < d; i += LN_BLOCK) {
        const float c = hs[i] - mean;
        ss = fmaf(c, c, ss);
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += LN_BLOCK)
        orow[i] = from_float<TA>(fmaf((hs[i] - mean) * inv, to_float(w[i]), bias ? to_float(bias[i]) : 0.f));
}

template <typename T> __device__ __forceinline__ float4 round_as(float4 v) { return v; }
template <> __device__ __forceinline__ float4 round_as<__nv_bfloat16>(float4 v) {
    const float2 a = __bfloat1622float2(__floats2bfloat162_rn(v.x, v.y)), b = __bfloat1622float2(__floats2bfloat162_rn(v.z, v.w));
    return make_float4(a.x, a.y, b.x, b.y);
}

// The same for rows whose width is a multiple of 4, up to 256 x NV x 4 columns: the branch row and the stream's row are read
// once with 16-byte loads and stay in registers between the passes.
template <typename TA, typename TW, int NV>
__global__ void __launch_bounds__(LN_BLOCK) add_normed_layernorm_vec_kernel(float* __restrict__ h, const TA* __restrict__ branch, const TW* __restrict__ bw,
                                                                            const TW* __restrict__ bb, float eps_b, const TW* __restrict__ w,
                                                                            const TW* __restrict__ bias, float eps, TA* __restrict__ out,
                                                                            const int* __restrict__ rows, int d, int write_h,
                                                                            const float* __restrict__ conv_w, int taps, float* __restrict__ conv_state,
                                                                            const int* __restrict__ seq_of_token, const int* __restrict__ slots) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int64_t src = rows ? rows[r] : r;
    const TA* brow = branch + src * d;
    float* hrow = h + src * d;
    float4 b[NV], v[NV];
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < NV; ++e) {
        const int i = (threadIdx.x + e * LN_BLOCK) * 4;
        b[e] = i < d ? Vec4<TA>::load(brow + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        v[e] = i < d ? Vec4<float>::load(hrow + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        sum += (b[e].x + b[e].y) + (b[e].z + b[e].w);
    }
    const float mean_b = block_sum(sum, scratch) / (float)d;
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < NV; ++e) {
        const int i = (threadIdx.x + e * LN_BLOCK) * 4;
        if (i < d) {
            const float a0 = b[e].x - mean_b, a1 = b[e].y - mean_b, a2 = b[e].z - mean_b, a3 = b[e].w - mean_b;
            ss += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
        }
    }
    const float inv_b = rsqrtf(block_sum(ss, scratch) / (float)d + eps_b);
    sum = 0.f;
#pragma unroll
    for (int e = 0; e < NV; ++e) {
        const int i = (threadIdx.x + e * LN_BLOCK) * 4;
        if (i < d) {
            const float4 ww = Vec4<TW>::load(bw + i);
            const float4 bv = bb ? Vec4<TW>::load(bb + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            v[e].x += fmaf((b[e].x - mean_b) * inv_b, ww.x, bv.x), v[e].y += fmaf((b[e].y - mean_b) * inv_b, ww.y, bv.y);
            v[e].z += fmaf((b[e].z - mean_b) * inv_b, ww.z, bv.z), v[e].w += fmaf((b[e].w - mean_b) * inv_b, ww.w, bv.w);
            if (write_h) Vec4<float>::store(hrow + i, v[e]);
            sum += (v[e].x + v[e].y) + (v[e].z + v[e].w);
        }
    }
    if (!w) return;
    const float mean = block_sum(sum, scratch) / (float)d;
    ss = 0.f;
#pragma unroll
    for (int e = 0; e < NV; ++e) {
        const int i = (threadIdx.x + e * LN_BLOCK) * 4;
        if (i < d) {
            const float a0 = v[e].x - mean, a1 = v[e].y - mean, a2 = v[e].z - mean, a3 = v[e].w - mean;
            ss += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
        }
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)d + eps);
    TA* orow = out + (int64_t)r * d;
#pragma unroll
    for (int e = 0; e < NV; ++e) {
        const int i = (threadIdx.x + e * LN_BLOCK) * 4;
        if (i < d) {
            const float4 ww = Vec4<TW>::load(w + i);
            const float4 bv = bias ? Vec4<TW>::load(bias + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 y = make_float4(fmaf((v[e].x - mean) * inv, ww.x, bv.x), fmaf((v[e].y - mean) * inv, ww.y, bv.y),
                                   fmaf((v[e].z - mean) * inv, ww.z, bv.z), fmaf((v[e].w - mean) * inv, ww.w, bv.w));
            if (conv_w) {
                // A step of single tokens: the short convolution that the reader of this row would run next (y + sum_j w[j] * input j
                // steps back, the inputs before this token in the request's state), and the state's shift.  The row is rounded to the
                // activation type first, as the kernel that reads stored rows sees it, and the sum runs in that kernel's order.
                y = round_as<TA>(y);
                float* st = conv_state + (int64_t)slots[seq_of_token[r]] * (taps - 1) * d + i;
                float4 acc = y;
                for (int j = 0; j + 1 < taps; ++j) {
                    const float4 cw = Vec4<float>::load(conv_w + (int64_t)j * d + i), sv = Vec4<float>::load(st + (int64_t)j * d);
                    acc.x = fmaf(cw.x, sv.x, acc.x), acc.y = fmaf(cw.y, sv.y, acc.y), acc.z = fmaf(cw.z, sv.z, acc.z), acc.w = fmaf(cw.w, sv.w, acc.w);
                    if (j > 0) Vec4<float>::store(st + (int64_t)(j - 1) * d, sv);      // this thread alone reads and writes these entries
                }
                const float4 cw = Vec4<float>::load(conv_w + (int64_t)(taps - 1) * d + i);
                acc.x = fmaf(cw.x, y.x, acc.x), acc.y = fmaf(cw.y, y.y, acc.y), acc.z = fmaf(cw.z, y.z, acc.z), acc.w = fmaf(cw.w, y.w, acc.w);
                if (taps > 1) Vec4<float>::store(st + (int64_t)(taps - 2) * d, y);
                y = acc;
            }
            Vec4<TA>::store(orow + i, y);
        }
    }
}

template <typename TA, typename TW>
static cudaError_t launch_normed_layernorm(float* h, const void* branch, const void* bw, const void* bb, float eps_b, const void* w, const void* bias,
                                           float eps, void* out, const int* rows, int n, int d, int write_h, cudaStream_t s,
                                           const float* conv_w = nullptr, int taps = 0, float* conv_state = nullptr, const int* seq_of_token = nullptr,
                                           const int* slots = nullptr) {
    const auto al = [](const void* p, size_t n) { return (uintptr_t)p % n == 0; };
    if (h && d % 4 == 0 && d <= LN_BLOCK * 4 * 8 && al(h, 16) && al(branch, 8) && al(out, 8) && al(bw, 16) && al(bb, 16) && al(w, 16) && al(bias, 16)) {
        const int nv = (d / 4 + LN_BLOCK - 1) / LN_BLOCK;
#define IMP_NLN(NV)                                                                                                                                     \
    imp_launch(add_normed_layernorm_vec_kernel<TA, TW, NV>, dim3(n), dim3(LN_BLOCK), 0, s, h, (const TA*)branch, (const TW*)bw, (const TW*)bb, eps_b, \
               (const TW*)w, (const TW*)bias, eps, (TA*)out, rows, d, write_h, conv_w, taps, conv_state, seq_of_token, slots)
        if (nv <= 1) return IMP_NLN(1);
        if (nv <= 2) return IMP_NLN(2);
        if (nv <= 4) return IMP_NLN(4);
        return IMP_NLN(8);
#undef IMP_NLN
    }
    if (conv_w) return cudaErrorNotSupported;     // only the form with rows in registers runs the convolution
    const size_t smem = (size_t)2 * d * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(add_normed_layernorm_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return imp_launch(add_normed_layernorm_kernel<TA, TW>, dim3(n), dim3(LN_BLOCK), smem, s, h, (const TA*)branch, (const TW*)bw, (const TW*)bb, eps_b,
                      (const TW*)w, (const TW*)bias, eps, (TA*)out, rows, d, write_h);
}

// h: [*, d] float32 stream or null (then out = the branch's norm alone); branch: dense [*, d] of the activation type with its
// own norm (bw, optional bb, eps_b); w, bias, eps: the norm of the sum, w null to only add; rows: optional gather list (then
// write_h must be 0).  All weights of one type.
IMP_API int imp_add_normed_layernorm(float* h, const void* branch, const void* bw, const void* bb, float eps_b, const void* w, const void* bias,
                                     float eps, void* out, const int* rows, int n_out_rows, int d, int act_dtype, int w_dtype, int write_h,
                                     void* stream) {
    if (n_out_rows == 0) return 0;
    IMP_CHECK_ARG(branch && bw && d > 0 && n_out_rows > 0 && (h || out) && (out || !w) && (h || !rows), "imp_add_normed_layernorm: bad argument");
    IMP_CHECK_ARG(!(rows && write_h), "imp_add_normed_layernorm: a gather list and write_h exclude each other");
    IMP_CHECK_ARG((size_t)2 * d * sizeof(float) <= 200 * 1024, "imp_add_normed_layernorm: rows of %d values do not fit", d);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (act_dtype == IMP_F32)
        e = w_dtype == IMP_F32 ? launch_normed_layernorm<float, float>(h, branch, bw, bb, eps_b, w, bias, eps, out, rows, n_out_rows, d, write_h, s)
                               : launch_normed_layernorm<float, __nv_bfloat16>(h, branch, bw, bb, eps_b, w, bias, eps, out, rows, n_out_rows, d, write_h, s);
    else
        e = w_dtype == IMP_F32 ? launch_normed_layernorm<__nv_bfloat16, float>(h, branch, bw, bb, eps_b, w, bias, eps, out, rows, n_out_rows, d, write_h, s)
                               : launch_normed_layernorm<__nv_bfloat16, __nv_bfloat16>(h, branch, bw, bb, eps_b, w, bias, eps, out, rows, n_out_rows, d, write_h, s);
    if (e != cudaSuccess) {
        imp_set_error("imp_add_normed_layernorm: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// imp_add_normed_layernorm for a step of single tokens (row r is sequence seq_of_token[r]'s only token) with the short
// convolution of the row's reader behind the second norm: out = y + sum_j conv_w[j] * (input j steps back), conv_w float32
// [taps, d], the earlier inputs in conv_state [slot][taps - 1][d] (float32), which is shifted by this row.  Returns
// IMP_ERR_UNSUPPORTED, having launched nothing, for widths and alignments that the form with rows in registers does not take.
IMP_API int imp_add_normed_layernorm_conv(float* h, const void* branch, const void* bw, const void* bb, float eps_b, const void* w, const void* bias,
                                          float eps, void* out, int n_rows, int d, int act_dtype, int w_dtype, const float* conv_w, int taps,
                                          float* conv_state, const int* seq_of_token, const int* slots, void* stream) {
    if (n_rows == 0) return 0;
    IMP_CHECK_ARG(h && branch && bw && w && out && d > 0 && conv_w && taps >= 1 && (taps == 1 || conv_state) && seq_of_token && slots,
                  "imp_add_normed_layernorm_conv: bad argument");
    // Up to 2,048 columns (two vectors a thread): there the saved launch wins (8 sequences at width 1024: 0.344 -> 0.329 ms a decode step of
    // four layers); at width 4096 the one CTA a token that also walks the state and the taps' weights lost (0.682 -> 0.713 ms) to the
    // separate kernel, which spreads a token over more CTAs.
    if ((uintptr_t)conv_w % 16 || (uintptr_t)conv_state % 16 || d % 4 || d > LN_BLOCK * 4 * 2) return IMP_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (act_dtype == IMP_F32)
        e = w_dtype == IMP_F32 ? launch_normed_layernorm<float, float>(h, branch, bw, bb, eps_b, w, bias, eps, out, nullptr, n_rows, d, 1, s, conv_w, taps, conv_state, seq_of_token, slots)
                               : launch_normed_layernorm<float, __nv_bfloat16>(h, branch, bw, bb, eps_b, w, bias, eps, out, nullptr, n_rows, d, 1, s, conv_w, taps, conv_state, seq_of_token, slots);
    else
        e = w_dtype == IMP_F32 ? launch_normed_layernorm<__nv_bfloat16, float>(h, branch, bw, bb, eps_b, w, bias, eps, out, nullptr, n_rows, d, 1, s, conv_w, taps, conv_state, seq_of_token, slots)
                               : launch_normed_layernorm<__nv_bfloat16, __nv_bfloat16>(h, branch, bw, bb, eps_b, w, bias, eps, out, nullptr, n_rows, d, 1, s, conv_w, taps, conv_state, seq_of_token, slots);
    if (e == cudaErrorNotSupported) return IMP_ERR_UNSUPPORTED;
    if (e != cudaSuccess) {
        imp_set_error("imp_add_normed_layernorm_conv: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}
