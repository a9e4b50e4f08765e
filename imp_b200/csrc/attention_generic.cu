// Paged attention for any batch: every query token attends to the cached keys
// of its own sequence at positions max(0, p-window+1) .. p, p being the token's
// own position (its key and value are already in the pages).
//
// This is the plain kernel of the family: one block per (token, query head),
// 32-bit scores, running max and sum, 32-bit accumulator, IEEE expf.  It is the
// kernel of the float32 path and the yardstick of the faster bfloat16 kernels.
// The order of every reduction depends only on the token's own position, so
// the result is the same whatever else is in the batch and however the prompt
// was cut.
//
// Math as in the reference's flash kernel (src/compute/attention.cu:158-216):
// s_ij = scale * q_i.k_j, masked when j > i or i - j >= window, softmax with a
// running max, o_i = sum_j p_ij v_j; query head h reads kv head h / (Hq/Hkv)
// (src/compute/attention_paged.cu:84-160).  Unlike the reference's prefill
// kernels, which see only the call's own K and V (src/graph/executor_forward.cu:
// 568-604), keys come from the pages, so a later portion of a prompt sees the
// earlier ones.
//
// Two optional additions for mixers that are not plain softmax attention (both in 32-bit, after
// the scale): `bias` adds bias[h][min(p - j, n_dist - 1)] to the score of key j, a table by
// distance and query head; `sink` adds exp(sink[h]) to the softmax denominator, a term without a
// key or a value.
#include "common.cuh"

constexpr int ATT_BLOCK = 128;
constexpr int ATT_MAX_DH = 1024;
constexpr int ATT_ACC = ATT_MAX_DH / ATT_BLOCK;   // output entries a thread accumulates: tid, tid + 128, ...

template <typename TA>
__global__ void paged_attention_generic_kernel(
    TA* __restrict__ out, int64_t out_stride, const TA* __restrict__ q, int64_t q_stride,
    const TA* __restrict__ k_cache, const TA* __restrict__ v_cache,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ seq_of_token,
    const int* __restrict__ positions, int n_seqs, int Hq, int Hkv, int Dh, int page_size, int num_pages,
    float scale, int window, const float* __restrict__ bias, int n_dist, const float* __restrict__ sink, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float q_s[ATT_MAX_DH];
    __shared__ float p_s[ATT_BLOCK];
    __shared__ int64_t off_s[ATT_BLOCK];
    __shared__ float scratch[33];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int hk = h / (Hq / Hkv);
    const int seq = seq_of_token[t];
    const int pos = positions[t];
    TA* o = out + (int64_t)t * out_stride + (int64_t)h * Dh;
    if (seq < 0 || seq >= n_seqs || pos < 0 || pos / page_size >= bt_stride) {
        if (tid == 0) imp_report(status, seq < 0 || seq >= n_seqs ? IMP_BAD_SEQUENCE : IMP_BAD_POSITION);
        for (int d = tid; d < Dh; d += ATT_BLOCK) o[d] = from_float<TA>(0.f);
        return;
    }
    const TA* qp = q + (int64_t)t * q_stride + (int64_t)h * Dh;
    for (int d = tid; d < Dh; d += ATT_BLOCK) q_s[d] = to_float(qp[d]);
    __syncthreads();

    const int* bt = block_table + (int64_t)seq * bt_stride;
    const int first = imp_first_key(pos, window);
    const float* bias_h = bias ? bias + (int64_t)h * n_dist : nullptr;
    float m = -INFINITY, l = 0.f;
    float acc[ATT_ACC];            // dims tid + a * ATT_BLOCK
#pragma unroll
    for (int a = 0; a < ATT_ACC; ++a) acc[a] = 0.f;

    for (int j0 = first; j0 <= pos; j0 += ATT_BLOCK) {
        const int j = j0 + tid;
        float s = -INFINITY;
        int64_t off = -1;
        if (j <= pos) {
            const int page = bt[j / page_size];
            if (page < 0 || page >= num_pages) {
                imp_report(status, IMP_BAD_PAGE);
            } else {
                off = (((int64_t)page * Hkv + hk) * page_size + (j % page_size)) * Dh;
                const TA* kp = k_cache + off;
                // four interleaved partial sums (entries d, d + 1, d + 2, d + 3 of every group of four), added at the end:
                // shorter chains than one sum over the whole head, in an order the head size alone fixes
                float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
                int d = 0;
                for (; d + 3 < Dh; d += 4) {
                    d0 = fmaf(q_s[d], to_float(kp[d]), d0);
                    d1 = fmaf(q_s[d + 1], to_float(kp[d + 1]), d1);
                    d2 = fmaf(q_s[d + 2], to_float(kp[d + 2]), d2);
                    d3 = fmaf(q_s[d + 3], to_float(kp[d + 3]), d3);
                }
                for (; d < Dh; ++d) d0 = fmaf(q_s[d], to_float(kp[d]), d0);
                s = ((d0 + d1) + (d2 + d3)) * scale;
                if (bias_h) s += bias_h[min(pos - j, n_dist - 1)];
            }
        }
        const float m_new = fmaxf(m, block_max(s, scratch));
        const float p = (off >= 0) ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        p_s[tid] = p;
        off_s[tid] = off;
        const float psum = block_sum(p, scratch);  // contains the barrier that publishes p_s/off_s
        l = l * corr + psum;
        m = m_new;
        const int n_here = min(ATT_BLOCK, pos - j0 + 1);
#pragma unroll
        for (int a = 0; a < ATT_ACC; ++a) {
            const int dim = tid + a * ATT_BLOCK;
            if (dim < Dh) {
                // the chunk's 128 keys are summed on their own and then added to the running sum
                float part = 0.f;
                for (int i = 0; i < n_here; ++i)
                    if (off_s[i] >= 0) part = fmaf(p_s[i], to_float(v_cache[off_s[i] + dim]), part);
                acc[a] = fmaf(acc[a], corr, part);
            }
        }
        __syncthreads();  // p_s/off_s are rewritten by the next chunk
    }
    if (sink) {
        // one more term of the denominator: exp(sink) against the running maximum
        const float sk = sink[h];
        const float m_new = fmaxf(m, sk);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + expf(sk - m_new);
#pragma unroll
        for (int a = 0; a < ATT_ACC; ++a) acc[a] *= corr;
    }
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int a = 0; a < ATT_ACC; ++a)
        if (tid + a * ATT_BLOCK < Dh) o[tid + a * ATT_BLOCK] = from_float<TA>(acc[a] * inv_l);
}

// out: [n_tokens, out_stride] (head h at column h*Dh); q likewise with q_stride.
// k_cache, v_cache: [num_pages, Hkv, page_size, Dh] of one layer.
static int launch_generic(
    void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
    const int* block_table, int bt_stride, const int* seq_of_token, const int* positions, int n_tokens,
    int n_seqs, int Hq, int Hkv, int Dh, int page_size, int num_pages, float scale, int window, const float* bias,
    int n_dist, const float* sink, int dtype, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(out && q && k_cache && v_cache && block_table && seq_of_token && positions,
                  "imp_paged_attention_generic: null pointer");
    IMP_CHECK_ARG(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "imp_paged_attention_generic: %d query heads are not a multiple of %d kv heads", Hq, Hkv);
    IMP_CHECK_ARG(Dh > 0 && Dh <= ATT_MAX_DH, "imp_paged_attention_generic: head_dim %d outside (0, %d]", Dh, ATT_MAX_DH);
    IMP_CHECK_ARG(page_size > 0 && num_pages > 0, "imp_paged_attention_generic: bad cache geometry");
    IMP_CHECK_ARG(Hq <= 65535, "imp_paged_attention_generic: more than 65535 query heads");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, Hq);
    if (dtype == IMP_F32)
        paged_attention_generic_kernel<float><<<grid, ATT_BLOCK, 0, s>>>(
            (float*)out, out_stride, (const float*)q, q_stride, (const float*)k_cache, (const float*)v_cache,
            block_table, bt_stride, seq_of_token, positions, n_seqs, Hq, Hkv, Dh, page_size, num_pages, scale,
            window, bias, n_dist, sink, status);
    else
        paged_attention_generic_kernel<__nv_bfloat16><<<grid, ATT_BLOCK, 0, s>>>(
            (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache,
            (const __nv_bfloat16*)v_cache, block_table, bt_stride, seq_of_token, positions, n_seqs, Hq, Hkv, Dh,
            page_size, num_pages, scale, window, bias, n_dist, sink, status);
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_paged_attention_generic(
    void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
    const int* block_table, int bt_stride, const int* seq_of_token, const int* positions, int n_tokens,
    int n_seqs, int Hq, int Hkv, int Dh, int page_size, int num_pages, float scale, int window, int dtype,
    int* status, void* stream) {
    return launch_generic(out, out_stride, q, q_stride, k_cache, v_cache, block_table, bt_stride, seq_of_token, positions,
                          n_tokens, n_seqs, Hq, Hkv, Dh, page_size, num_pages, scale, window, nullptr, 0, nullptr, dtype,
                          status, stream);
}

// The same with a score bias by distance, bias [Hq, n_dist] (float32; null = none), and a sink per
// query head, sink [Hq] (float32; null = none).
IMP_API int imp_paged_attention_generic_bias(
    void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
    const int* block_table, int bt_stride, const int* seq_of_token, const int* positions, int n_tokens,
    int n_seqs, int Hq, int Hkv, int Dh, int page_size, int num_pages, float scale, int window, const float* bias,
    int n_dist, const float* sink, int dtype, int* status, void* stream) {
    IMP_CHECK_ARG(!bias || n_dist > 0, "imp_paged_attention_generic_bias: a bias table needs at least one distance");
    return launch_generic(out, out_stride, q, q_stride, k_cache, v_cache, block_table, bt_stride, seq_of_token, positions,
                          n_tokens, n_seqs, Hq, Hkv, Dh, page_size, num_pages, scale, window, bias, n_dist, sink, dtype,
                          status, stream);
}
