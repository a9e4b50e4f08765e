// Routing of a mixture of experts, and the sum of the chosen experts' outputs.
//
//   z[t, e]   = x[t] . Wr[e] + b[e]                       32-bit
//   chosen    = the `top` experts with the largest z (the lower index wins a tie)
//   weight    = softmax over the chosen logits only; or, with sigmoid scores s = sigmoid(z): weight = s * weight_scale
//   groups    = optionally the experts form n_groups equal groups of neighbours; a group's score is the sum of its two
//               largest scores, and only the experts of the `keep` best groups can be chosen
//   gate[t]   = sigmoid(x[t] . Wg)                         one number per token, for a shared expert (optional)
//   out[t]    = sum_k weight[t, k] * y[place(t, k)] + gate[t] * shared[t]
//
// The expert products run over a list of (token, choice) pairs sorted by expert (see grouped_gemm.cu); moe_sort makes
// that list on the device: seg [E + 1], the token of every list row, and the row of every pair.  Nothing comes back
// to the host, so the launches of a step depend on its sizes alone.
#include "common.cuh"

namespace {

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

constexpr int ROUTE_BLOCK = 256, ROUTE_MAX_E = 1024, ROUTE_MAX_TOP = 32;

// A CTA routes TPB tokens: their rows wait in shared memory as 32-bit values while each warp walks the router's rows (and
// the shared expert's mixing row), one row at a time against all TPB tokens, so a row of the router is read once per CTA.
// A token's sums are made the same way whatever TPB is: lane-strided partial sums of four-wide pieces, then a shuffle tree.
template <typename TA, int TPB>
__global__ void __launch_bounds__(ROUTE_BLOCK) moe_route_kernel(const TA* __restrict__ x, int64_t ldx, int n_tokens, int d,
                                                               const float* __restrict__ wr, const float* __restrict__ br, int E, int top,
                                                               const float* __restrict__ wg, int* __restrict__ idx, float* __restrict__ wts,
                                                               float* __restrict__ gate, int vec, int score_mode, int n_groups, int keep,
                                                               float weight_scale) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float sm[];   // x [TPB][d4], then z [TPB][E], then the groups' scores [TPB][n_groups]
    const int d4 = (d + 3) & ~3;
    float* xs = sm;
    float* z = sm + (size_t)TPB * d4;
    float* gsc = z + (size_t)TPB * E;
    const int t0 = blockIdx.x * TPB, nt = min(TPB, n_tokens - t0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int e = tid; e < TPB * d4; e += ROUTE_BLOCK) {
        const int tk = e / d4, i = e % d4;
        xs[e] = (tk < nt && i < d) ? to_float(x[(int64_t)(t0 + tk) * ldx + i]) : 0.f;
    }
    __syncthreads();
    for (int e = warp; e < E + (wg ? 1 : 0); e += ROUTE_BLOCK / 32) {
        const float* w = e < E ? wr + (int64_t)e * d : wg;
        float acc[TPB];
#pragma unroll
        for (int tk = 0; tk < TPB; ++tk) acc[tk] = 0.f;
        if (vec) {
#pragma unroll 4
            for (int i = lane * 4; i < d; i += 128) {
                const float4 wv = *reinterpret_cast<const float4*>(w + i);
#pragma unroll
                for (int tk = 0; tk < TPB; ++tk) {
                    const float4 xv = *reinterpret_cast<const float4*>(xs + tk * d4 + i);
                    acc[tk] = fmaf(xv.x, wv.x, acc[tk]);
                    acc[tk] = fmaf(xv.y, wv.y, acc[tk]);
                    acc[tk] = fmaf(xv.z, wv.z, acc[tk]);
                    acc[tk] = fmaf(xv.w, wv.w, acc[tk]);
                }
            }
        } else {
            for (int i = lane; i < d; i += 32) {
                const float wv = w[i];
#pragma unroll
                for (int tk = 0; tk < TPB; ++tk) acc[tk] = fmaf(xs[tk * d4 + i], wv, acc[tk]);
            }
        }
#pragma unroll
        for (int tk = 0; tk < TPB; ++tk) {
            const float sum = warp_sum(acc[tk]);
            if (lane == 0 && tk < nt) {
                if (e < E) {
                    const float logit = sum + (br ? br[e] : 0.f);
                    z[tk * E + e] = score_mode == 1 ? 1.f / (1.f + expf(-logit)) : logit;
                } else {
                    gate[t0 + tk] = 1.f / (1.f + expf(-sum));
                }
            }
        }
    }
    __syncthreads();
    // `top` rounds of arg-max over the logits that are left, a warp per token; the lower index wins a tie
    for (int tk = warp; tk < nt; tk += ROUTE_BLOCK / 32) {
        float* zt = z + tk * E;
        const int64_t t = t0 + tk;
        float chosen[ROUTE_MAX_TOP];
        if (n_groups > 0) {
            // a group's score: the sum of its two largest scores (of its one score where a group is one expert); then `keep`
            // rounds of arg-max over the groups, the lower index winning a tie; the experts of the other groups leave
            float* gt = gsc + tk * n_groups;
            const int per = E / n_groups;
            for (int g = lane; g < n_groups; g += 32) {
                float a = -INFINITY, b = -INFINITY;
                for (int e = g * per; e < (g + 1) * per; ++e) {
                    const float v = zt[e];
                    if (v > a) b = a, a = v;
                    else if (v > b) b = v;
                }
                gt[g] = per > 1 ? a + b : a;
            }
            __syncwarp();
            for (int k = 0; k < keep; ++k) {
                float best = -INFINITY;
                int at = 0x7fffffff;
                for (int g = lane; g < n_groups; g += 32) {
                    const float v = gt[g];
                    if (v > best) best = v, at = g;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                    const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                    if (ov > best || (ov == best && oa < at)) best = ov, at = oa;
                }
                if (lane == 0 && at < n_groups) gt[at] = -INFINITY;   // kept
                __syncwarp();
            }
            for (int e = lane; e < E; e += 32)
                if (gt[e / per] != -INFINITY) zt[e] = -INFINITY;
            __syncwarp();
        }
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                const float v = zt[e];
                if (v > best) best = v, at = e;     // ascending e: the first of equal values stays
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ov > best || (ov == best && oa < at)) best = ov, at = oa;
            }
            chosen[k] = best;
            if (lane == 0) {
                idx[t * top + k] = at;
                zt[at] = -INFINITY;
            }
            __syncwarp();
        }
        if (lane == 0 && score_mode == 1) {
            for (int k = 0; k < top; ++k) wts[t * top + k] = chosen[k] * weight_scale;   // the scores themselves, not renormalised
        } else if (lane == 0) {
            const float largest = chosen[0];   // the first chosen is the largest
            float sum = 0.f;
            for (int k = 0; k < top; ++k) {
                chosen[k] = expf(chosen[k] - largest);
                sum += chosen[k];
            }
            for (int k = 0; k < top; ++k) wts[t * top + k] = chosen[k] / sum;
        }
    }
}

// One CTA.  seg[e] .. seg[e + 1]: expert e's rows of the list; row_token[r]: the token of row r; pair_row[p]: the row of
// pair p = t * top + k.  Within an expert the rows follow the pair index, so the list is the same for the same routing.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ idx, int n_pairs, int top, int E, int* __restrict__ seg,
                                                        int* __restrict__ row_token, int* __restrict__ pair_row) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ int cnt[];   // [E + 1]
    const int tid = threadIdx.x;
    for (int e = tid; e <= E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = tid; p < n_pairs; p += blockDim.x) {
        const int e = idx[p];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            const int c = cnt[e];
            cnt[e] = run;
            seg[e] = run;
            run += c;
        }
        cnt[E] = run;
        seg[E] = run;
    }
    __syncthreads();
    // every expert's rows in pair order: a warp walks the pairs of one expert at a time
    const int lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
    for (int e = warp; e < E; e += n_warps) {
        int at = cnt[e];
        for (int p0 = 0; p0 < n_pairs; p0 += 32) {
            const int p = p0 + lane;
            const bool mine = p < n_pairs && idx[p] == e;
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int r = at + __popc(m & ((1u << lane) - 1u));
                row_token[r] = p / top;
                pair_row[p] = r;
            }
            at += __popc(m);
        }
    }
}

template <typename TA>
__global__ void moe_combine_kernel(TA* __restrict__ out, const TA* __restrict__ y, const int* __restrict__ pair_row, const float* __restrict__ wts,
                                   int top, const TA* __restrict__ shared, const float* __restrict__ gate, int d) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t t = blockIdx.x;
    const float gt = gate ? gate[t] : 1.f;
    if ((d & 3) == 0) {
        // four columns a thread (rows start on 8 or 16 bytes: dense [*, d] with d a multiple of 4)
        for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < top; ++k) {
                const float wk = wts[t * top + k];
                const float4 v = Vec4<TA>::load(y + (int64_t)pair_row[t * top + k] * d + i);
                acc.x = fmaf(wk, v.x, acc.x), acc.y = fmaf(wk, v.y, acc.y), acc.z = fmaf(wk, v.z, acc.z), acc.w = fmaf(wk, v.w, acc.w);
            }
            if (shared) {
                const float4 v = Vec4<TA>::load(shared + t * d + i);
                acc.x = fmaf(gt, v.x, acc.x), acc.y = fmaf(gt, v.y, acc.y), acc.z = fmaf(gt, v.z, acc.z), acc.w = fmaf(gt, v.w, acc.w);
            }
            Vec4<TA>::store(out + t * d + i, acc);
        }
        return;
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) acc = fmaf(wts[t * top + k], to_float(y[(int64_t)pair_row[t * top + k] * d + i]), acc);
        if (shared) acc = fmaf(gt, to_float(shared[t * d + i]), acc);
        out[t * d + i] = from_float<TA>(acc);
    }
}

// dst[r] = src[idx[r]]: rows of d values, 16 bytes a thread where the rows allow it.
template <typename TA>
__global__ void gather_rows_kernel(TA* __restrict__ dst, const TA* __restrict__ src, int64_t ld, const int* __restrict__ idx, int d, int vec) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t r = blockIdx.x;
    const TA* from = src + (int64_t)idx[r] * ld;
    TA* to = dst + r * d;
    if (vec) {
        constexpr int PER = 16 / (int)sizeof(TA);
        for (int i = threadIdx.x * PER; i < d; i += blockDim.x * PER) *reinterpret_cast<uint4*>(to + i) = *reinterpret_cast<const uint4*>(from + i);
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) to[i] = from[i];
    }
}

}  // namespace

IMP_API int imp_gather_rows(void* dst, const void* src, int64_t ld, const int* idx, int n_rows, int d, int dtype, void* stream) {
    if (n_rows == 0) return 0;
    IMP_CHECK_ARG(dst && src && idx && d > 0, "imp_gather_rows: bad argument");
    const int el = dtype == IMP_F32 ? 4 : 2;
    const int vec = ((int64_t)d * el % 16 == 0 && ld * el % 16 == 0 && (uintptr_t)dst % 16 == 0 && (uintptr_t)src % 16 == 0) ? 1 : 0;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = dtype == IMP_F32 ? imp_launch(gather_rows_kernel<float>, dim3(n_rows), dim3(128), 0, s, (float*)dst, (const float*)src, ld, idx, d, vec)
                                     : imp_launch(gather_rows_kernel<__nv_bfloat16>, dim3(n_rows), dim3(128), 0, s, (__nv_bfloat16*)dst,
                                                  (const __nv_bfloat16*)src, ld, idx, d, vec);
    if (e != cudaSuccess) {
        imp_set_error("imp_gather_rows: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

template <typename TA, int TPB>
static cudaError_t launch_route(const void* x, int64_t ldx, int n_tokens, int d, const float* wr, const float* br, int E, int top, const float* wg,
                                int* idx, float* wts, float* gate, int vec, int score_mode, int n_groups, int keep, float weight_scale, size_t smem,
                                cudaStream_t s) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(moe_route_kernel<TA, TPB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return imp_launch(moe_route_kernel<TA, TPB>, dim3((n_tokens + TPB - 1) / TPB), dim3(ROUTE_BLOCK), smem, s, (const TA*)x, ldx, n_tokens, d, wr, br,
                      E, top, wg, idx, wts, gate, vec, score_mode, n_groups, keep, weight_scale);
}

template <typename TA>
static cudaError_t route_by_size(const void* x, int64_t ldx, int n_tokens, int d, const float* wr, const float* br, int E, int top, const float* wg,
                                 int* idx, float* wts, float* gate, int vec, int score_mode, int n_groups, int keep, float weight_scale,
                                 cudaStream_t s) {
    // more tokens a CTA where there are many (a row of the router is read once per CTA), one where there are few (more CTAs)
    int tpb = n_tokens >= 1024 ? 8 : n_tokens >= 256 ? 4 : n_tokens >= 64 ? 2 : 1;
    const int d4 = (d + 3) & ~3;
    auto bytes = [&](int t) { return ((size_t)t * d4 + (size_t)t * E + (size_t)t * n_groups) * 4; };
    while (tpb > 1 && bytes(tpb) > 160 * 1024) tpb /= 2;
    if (bytes(tpb) > 200 * 1024) return cudaErrorInvalidValue;
    switch (tpb) {
        case 8: return launch_route<TA, 8>(x, ldx, n_tokens, d, wr, br, E, top, wg, idx, wts, gate, vec, score_mode, n_groups, keep, weight_scale, bytes(8), s);
        case 4: return launch_route<TA, 4>(x, ldx, n_tokens, d, wr, br, E, top, wg, idx, wts, gate, vec, score_mode, n_groups, keep, weight_scale, bytes(4), s);
        case 2: return launch_route<TA, 2>(x, ldx, n_tokens, d, wr, br, E, top, wg, idx, wts, gate, vec, score_mode, n_groups, keep, weight_scale, bytes(2), s);
        default: return launch_route<TA, 1>(x, ldx, n_tokens, d, wr, br, E, top, wg, idx, wts, gate, vec, score_mode, n_groups, keep, weight_scale, bytes(1), s);
    }
}

// x [T, d] (activation type, rows ldx apart); wr float32 [E, d], br float32 [E] or null; wg float32 [d] or null (then
// gate is not written).  idx int32 [T, top], wts float32 [T, top], gate float32 [T].
// score_mode 0: weights are the softmax over the chosen logits; 1: scores are sigmoid(z) and a weight is its score times
// weight_scale.  n_groups > 0: only experts of the `keep` best of n_groups equal groups of neighbours can be chosen.
IMP_API int imp_moe_route_ex(const void* x, int64_t ldx, int n_tokens, int d, const float* wr, const float* br, int E, int top, const float* wg,
                             int* idx, float* wts, float* gate, int score_mode, int n_groups, int keep, float weight_scale, int act_dtype,
                             void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(x && wr && idx && wts && d > 0 && (!wg || gate), "imp_moe_route: bad argument");
    IMP_CHECK_ARG(E > 0 && E <= ROUTE_MAX_E && top > 0 && top <= E && top <= ROUTE_MAX_TOP,
                  "imp_moe_route: %d experts (at most %d), %d chosen (at most %d and no more than there are)", E, ROUTE_MAX_E, top, ROUTE_MAX_TOP);
    IMP_CHECK_ARG((score_mode == 0 || score_mode == 1) && n_groups >= 0 && (n_groups == 0 || (E % n_groups == 0 && keep > 0 && keep <= n_groups &&
                                                                                             top <= keep * (E / n_groups))),
                  "imp_moe_route: %d groups over %d experts, %d kept, %d chosen", n_groups, E, keep, top);
    const int vec = (d % 4 == 0 && (uintptr_t)wr % 16 == 0 && (!wg || (uintptr_t)wg % 16 == 0)) ? 1 : 0;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = act_dtype == IMP_F32 ? route_by_size<float>(x, ldx, n_tokens, d, wr, br, E, top, wg, idx, wts, gate, vec, score_mode, n_groups, keep, weight_scale, s)
                                         : route_by_size<__nv_bfloat16>(x, ldx, n_tokens, d, wr, br, E, top, wg, idx, wts, gate, vec, score_mode, n_groups, keep, weight_scale, s);
    if (e != cudaSuccess) {
        imp_set_error("imp_moe_route: %s (rows of %d values, %d experts)", cudaGetErrorString(e), d, E);
        return (int)e;
    }
    return 0;
}

IMP_API int imp_moe_route(const void* x, int64_t ldx, int n_tokens, int d, const float* wr, const float* br, int E, int top, const float* wg,
                          int* idx, float* wts, float* gate, int act_dtype, void* stream) {
    return imp_moe_route_ex(x, ldx, n_tokens, d, wr, br, E, top, wg, idx, wts, gate, 0, 0, 0, 1.f, act_dtype, stream);
}

IMP_API int imp_moe_sort(const int* idx, int n_tokens, int top, int E, int* seg, int* row_token, int* pair_row, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(idx && seg && row_token && pair_row && top > 0 && E > 0 && E <= ROUTE_MAX_E, "imp_moe_sort: bad argument");
    cudaError_t e = imp_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)(E + 1) * 4, (cudaStream_t)stream, idx, n_tokens * top, top, E, seg,
                               row_token, pair_row);
    if (e != cudaSuccess) {
        imp_set_error("imp_moe_sort: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// out [T, d] = sum_k wts[t, k] * y[pair_row[t * top + k]] (+ gate[t] * shared[t]); y [T * top, d], all dense.
IMP_API int imp_moe_combine(void* out, const void* y, const int* pair_row, const float* wts, int n_tokens, int top, const void* shared,
                            const float* gate, int d, int act_dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(out && y && pair_row && wts && top > 0 && d > 0, "imp_moe_combine: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = act_dtype == IMP_F32 ? imp_launch(moe_combine_kernel<float>, dim3(n_tokens), dim3(256), 0, s, (float*)out, (const float*)y,
                                                      pair_row, wts, top, (const float*)shared, gate, d)
                                         : imp_launch(moe_combine_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, s, (__nv_bfloat16*)out,
                                                      (const __nv_bfloat16*)y, pair_row, wts, top, (const __nv_bfloat16*)shared, gate, d);
    if (e != cudaSuccess) {
        imp_set_error("imp_moe_combine: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}
