// Part kinds: layer norm, latent attention, the wkv recurrence, routed experts with a shared expert, a pre-norm block
// whose branches carry a learned factor per channel, and a block that re-makes the stream from itself and the
// embedding's output.  Every size and constant is a parameter; no kind knows which model it is in.
#include <cmath>

#include "kernels.h"
#include "ops.hpp"
#include "parts.hpp"

namespace imp {

namespace {

int64_t need_int(const Json& p, const char* key, const char* part) {
    const Json* v = p.find(key);
    if (!v || !v->is_number()) fail(IMP_ERROR_INVALID_MODEL, std::string(part) + ": parameter '" + key + "' is missing");
    return v->as_int();
}
double need_double(const Json& p, const char* key, const char* part) {
    const Json* v = p.find(key);
    if (!v || !v->is_number()) fail(IMP_ERROR_INVALID_MODEL, std::string(part) + ": parameter '" + key + "' is missing");
    return v->as_double();
}

// A branch whose unsummed parts, if any, have been added up; a factor per column stays with it.
Branch parts_summed(Runtime& rt, const Branch& b) {
    if (!b.split()) return b;
    Branch plain = b;
    plain.col_scale = nullptr;
    plain.own_norm = BranchNorm{};
    Branch out = Branch::of(summed(rt, plain));
    out.col_scale = b.col_scale;
    out.own_norm = b.own_norm;
    return out;
}

// -------------------------------------------------------------------------------------------- layer norm
// y = (x - mean) / sqrt(var + eps) * w (+ b) over the last axis, the variance being the mean of the squared deviations; a
// weight and, with `bias`, a bias.  Statistics in 32-bit.  It can store its result as the stream (post-norm blocks).
// params: size, eps, bias (default false).
struct LayerNorm : Norm {
    Tensor weight, bias{};
    float eps;
    explicit LayerNorm(BuildArgs& a) : weight(a.tensor("weight")), eps((float)a.params.get_double("eps", 1e-5)) {
        if (a.params.get_bool("bias", false)) {
            bias = a.tensor("bias");
            if (bias.dtype != weight.dtype || numel(bias) != numel(weight)) fail(IMP_ERROR_INVALID_MODEL, "layernorm: weight and bias must agree in type and size");
        }
    }
    bool takes_column_scale() const override { return true; }
    bool takes_normed_branch() const override { return true; }
    bool as_branch_norm(BranchNorm* out) const override {
        out->weight = weight.data;
        out->bias = bias.data;
        out->eps = eps;
        out->dtype = weight.dtype;
        return true;
    }
    bool stores_stream() const override { return true; }
    // A branch with a norm of its own that this kernel family cannot apply while adding (another weight type, or factors per
    // column as well) gets it applied first.
    Branch plain_or_normed(Runtime& rt, const Branch& branch) const {
        Branch b = parts_summed(rt, branch);
        if (b.own_norm.weight && (b.col_scale || b.own_norm.dtype != weight.dtype)) b = Branch::of(summed(rt, b));
        return b;
    }
    Tensor add_norm_store(Step& st, Tensor h, float h_mult, const Branch& branch) override {
        Runtime& rt = *st.rt;
        const int d = (int)cols(h);
        Tensor out = rt.empty(rows(h), d);
        if (h.dtype != F32 || !contiguous(h) || numel(weight) != d) fail(IMP_ERROR_INVALID_ARG, "layernorm: the stream must be dense float32 [T, d], the weight [d]");
        Branch b = parts_summed(rt, branch);
        if (b.own_norm.weight) b = Branch::of(summed(rt, b));
        if (!b.empty() && (rows(b.t) != rows(h) || cols(b.t) != d || b.t.dtype != out.dtype || !contiguous(b.t)))
            fail(IMP_ERROR_INVALID_ARG, "layernorm: the branch must be dense, of the stream's shape and the output's type");
        ++rt.launches;
        check_launch(imp_add_layernorm_ex((float*)h.data, h_mult, b.empty() ? nullptr : b.t.data, b.col_scale, weight.data, bias.data, out.data, nullptr,
                                          (int)rows(h), d, eps, out.dtype, weight.dtype, 2, rt.stream),
                     "add_layernorm");
        return out;
    }
    Tensor add_norm(Step& st, Tensor h, const Branch& branch, const int32_t* rows_idx, int n_rows) override {
        Runtime& rt = *st.rt;
        const int64_t n = rows_idx ? n_rows : rows(h);
        const int d = (int)cols(h);
        Tensor out = rt.empty(n, d, -1, /*step=*/rows_idx != nullptr);
        if (h.dtype != F32 || !contiguous(h) || numel(weight) != d) fail(IMP_ERROR_INVALID_ARG, "layernorm: the stream must be dense float32 [T, d], the weight [d]");
        const Branch b = plain_or_normed(rt, branch);
        if (!b.empty() && (rows(b.t) != rows(h) || cols(b.t) != d || b.t.dtype != out.dtype || !contiguous(b.t)))
            fail(IMP_ERROR_INVALID_ARG, "layernorm: the branch must be dense, of the stream's shape and the output's type");
        ++rt.launches;
        if (b.own_norm.weight && st.row_op && !rows_idx) {
            // ... and the per-row operation of the rows' reader behind it, where the kernel's form takes it
            RowOp& op = *st.row_op;
            const int rc = imp_add_normed_layernorm_conv((float*)h.data, b.t.data, b.own_norm.weight, b.own_norm.bias, b.own_norm.eps, weight.data, bias.data,
                                                         eps, out.data, (int)n, d, out.dtype, weight.dtype, op.conv_w, op.taps, op.conv_state,
                                                         st.view.seq_of_token, st.view.state_slots, rt.stream);
            if (rc == 0) {
                op.taken = true;
                return out;
            }
            if (rc != -2) check_launch(rc, "add_normed_layernorm_conv");   // -2: the kernel declined (width or alignment); the unfused launches follow
        }
        if (b.own_norm.weight) {
            // the branch's own norm, the sum and this norm in one pass
            check_launch(imp_add_normed_layernorm((float*)h.data, b.t.data, b.own_norm.weight, b.own_norm.bias, b.own_norm.eps, weight.data, bias.data, eps,
                                                  out.data, rows_idx, (int)n, d, out.dtype, weight.dtype, rows_idx ? 0 : 1, rt.stream),
                         "add_normed_layernorm");
            return out;
        }
        check_launch(imp_add_layernorm_ex((float*)h.data, 1.f, b.empty() ? nullptr : b.t.data, b.col_scale, weight.data, bias.data, out.data, rows_idx,
                                          (int)n, d, eps, out.dtype, weight.dtype, rows_idx ? 0 : 1, rt.stream),
                     "add_layernorm");
        return out;
    }
};

// ------------------------------------------------------------------------------------- latent attention
// Causal softmax attention whose keys and values are expanded from a small latent per token:
//   c_q = rms(W_dq x) * n_q;  q = W_uq c_q, per head [D plain | R rotated]
//   W_dkv x = [ latent (C) | rotated key part (R) ];  c = rms(latent) * n_kv;  the key part is one for all heads
//   per head: k_plain = W_uk c, v = W_uv c;  score = scale * (q_plain . k_plain + rot(q_rot) . rot(k_rot))
//   out = W_o [heads' softmax-weighted values]
// Only c and the rotated key part are cached: one vector [C + R] per token, keys only.  The products with W_uk and W_uv
// are moved to the query side and the output side: q_lat = W_uk^T q_plain lives in the latent space, attention runs as
// one shared "kv head" of size C + R over the cache (the pages serve as keys and as values; the last R entries of its
// output are not used), and W_uv maps each head's latent-space result to its values.  Per token the cache holds
// C + R numbers whatever the number of heads.
//
// params: hidden_size, num_heads, head_dim (plain), rot_dim, value_dim, kv_rank, q_rank, scale, norm_eps, rot_base,
//         rot_dims (entries of the rotated part that are rotated: even, at most rot_dim), max_positions.
struct LatentAttention : Mixer {
    int H, D, R, Dv, C, Q, rot_dims;
    float eps;
    AttentionGeometry g;
    Tensor w_down, w_uq, w_ukT, w_uv, w_o, n_q, n_kv;
    Position* position = nullptr;

    struct Sizes {
        int64_t d, H, D, R, Dv, C, Q;
    };
    static Sizes sizes(const Json& p) {
        const char* me = "latent_attention";
        Sizes s{need_int(p, "hidden_size", me), need_int(p, "num_heads", me), need_int(p, "head_dim", me), need_int(p, "rot_dim", me),
                need_int(p, "value_dim", me), need_int(p, "kv_rank", me), need_int(p, "q_rank", me)};
        if (s.H <= 0 || s.D <= 0 || s.R <= 0 || s.Dv <= 0 || s.C <= 0 || s.Q <= 0) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": every size must be positive");
        if (s.C + s.R > 1024)
            fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": kv_rank + rot_dim = " + std::to_string(s.C + s.R) + " exceeds the attention kernels' 1024 (tensor cores up to 256)");
        return s;
    }
    static TensorSpecs specs(const Json& p) {
        const Sizes z = sizes(p);
        TensorSpecs s;
        s.emplace_back("q_down", TensorSpec{{z.Q, z.d}});
        s.emplace_back("q_norm", TensorSpec{{z.Q}, "norm", "one_plus_normal"});
        s.emplace_back("q_up", TensorSpec{{z.H * (z.D + z.R), z.Q}});
        s.emplace_back("kv_down", TensorSpec{{z.C + z.R, z.d}});
        s.emplace_back("kv_norm", TensorSpec{{z.C}, "norm", "one_plus_normal"});
        s.emplace_back("k_up", TensorSpec{{z.H * z.D, z.C}});
        s.emplace_back("v_up", TensorSpec{{z.H * z.Dv, z.C}});
        s.emplace_back("o_proj", TensorSpec{{z.d, z.H * z.Dv}});
        return s;
    }
    static CacheSpec cache(const Json& p) {
        const Sizes z = sizes(p);
        CacheSpec s = CacheSpec::paged(1, (int)(z.C + z.R), 0);
        s.keys_only = true;
        return s;
    }

    explicit LatentAttention(BuildArgs& a) {
        const char* me = "latent_attention";
        const Sizes z = sizes(a.params);
        H = (int)z.H, D = (int)z.D, R = (int)z.R, Dv = (int)z.Dv, C = (int)z.C, Q = (int)z.Q;
        rot_dims = (int)a.params.get_int("rot_dims", R);
        if (rot_dims < 2 || rot_dims % 2 || rot_dims > R)
            fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": rot_dims " + std::to_string(rot_dims) + " must be even and within rot_dim " + std::to_string(R));
        eps = (float)a.params.get_double("norm_eps", 1e-6);
        g.hq = H, g.hkv = 1, g.dh = C + R, g.window = 0;
        g.scale = (float)need_double(a.params, "scale", me);
        Runtime& rt = *a.rt;
        // one product for both down-projections; its rows are padded to a multiple of 8
        std::vector<Tensor> in = {a.tensor("q_down"), a.tensor("kv_down")};
        const int64_t n = z.Q + z.C + z.R, pad = (8 - n % 8) % 8;
        Tensor zeros{};
        if (pad) {
            zeros = a.store->alloc(in[0].dtype, {pad, z.d});
            IMP_CUDA(cudaMemsetAsync(zeros.data, 0, (size_t)numel(zeros) * elem_size(zeros.dtype), rt.stream));
            in.push_back(zeros);
        }
        w_down = cat_rows(rt, *a.store, in);
        w_uq = a.tensor("q_up");
        w_uv = a.tensor("v_up");
        w_o = a.tensor("o_proj");
        // W_uk [H][D, C] -> [H][C, D]: the latent-space query is a product with W_uk's transpose
        const Tensor uk = a.tensor("k_up");
        w_ukT = a.store->alloc(uk.dtype, {z.H * z.C, z.D});
        check_launch(imp_transpose_groups(w_ukT.data, uk.data, H, D, C, uk.dtype == F32 ? 0 : 1, rt.stream), "transpose_groups");
        n_q = to_float32(rt, *a.store, a.tensor("q_norm"));
        n_kv = to_float32(rt, *a.store, a.tensor("kv_norm"));
        Json pos = Json::object(), pp = Json::object();
        pos["kind"] = "rotary";
        pp["head_dim"] = (int64_t)R;
        pp["rotary_dim"] = (int64_t)rot_dims;
        pp["theta"] = need_double(a.params, "rot_base", me);
        pp["max_positions"] = need_int(a.params, "max_positions", me);
        pos["params"] = pp;
        position = part_cast<Position>(a.factory->shared("position", pos), "a position encoding");
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        if (pad) a.store->release(zeros.data);
        for (const char* nme : {"q_down", "kv_down", "k_up", "q_norm", "kv_norm"}) a.drop(nme);
    }

    std::vector<TilingSpec> tilings() const override { return attention_tilings(); }

    Branch forward(Step& st, Tensor x, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!cache || !cache->paged()) fail(IMP_ERROR_INTERNAL, "latent_attention runs against a paged cache");
        const int64_t T = rows(x);
        const ImpCacheView& cv = cache->view;
        Position::Rotary rot{};
        if (!position->rotary(&rot)) fail(IMP_ERROR_INTERNAL, "latent_attention needs rotary tables");
        const int dt = rt.dtype == F32 ? 0 : 1;
        Tensor proj = rt.empty(T, rows(w_down));
        linear(rt, proj, x, w_down);
        Tensor cq = rt.empty(T, Q);
        ++rt.launches;
        check_launch(imp_latent_prepare(proj.data, proj.stride0, (int)T, Q, C, R, (const float*)n_q.data, (const float*)n_kv.data, eps, cq.data,
                                        cq.stride0, rot.cos, rot.sin, rot.rot_dim, rot.max_pos, st.view.positions, st.view.seq_of_token,
                                        cv.block_table, cv.bt_stride, st.B(), cv.writes ? cv.k_pages : nullptr, cv.page_size, cv.num_pages, dt,
                                        rt.status, rt.stream),
                     "latent_prepare");
        Tensor q = rt.empty(T, (int64_t)H * (D + R));
        linear(rt, q, cq, w_uq);
        const int64_t L = C + R;
        Tensor q_lat = rt.empty(T, H * L);
        rt.launches += 2;
        check_launch(imp_grouped_gemm(q_lat.data, q_lat.stride0, L, q.data, q.stride0, D + R, nullptr, w_ukT.data, nullptr, (int64_t)C * D, D, nullptr,
                                      (int)T, C, D, H, 0, dt, rt.stream),
                     "grouped_gemm (latent query)");
        check_launch(imp_latent_query_rope(q.data, q.stride0, (int)T, H, D, R, q_lat.data, q_lat.stride0, C, rot.cos, rot.sin, rot.rot_dim,
                                           rot.max_pos, st.view.positions, dt, rt.status, rt.stream),
                     "latent_query_rope");
        Tensor attn = rt.empty(T, H * L);
        paged_attention(st, attn, q_lat, g, *cache, tiling_ids);
        Tensor o = rt.empty(T, (int64_t)H * Dv);
        ++rt.launches;
        check_launch(imp_grouped_gemm(o.data, o.stride0, Dv, attn.data, attn.stride0, L, nullptr, w_uv.data, nullptr, (int64_t)Dv * C, C, nullptr,
                                      (int)T, Dv, C, H, 0, dt, rt.stream),
                     "grouped_gemm (values)");
        return linear(rt, rt.empty(T, rows(w_o)), o, w_o, defer_out);
    }
};

// -------------------------------------------------------------------------------------------------- wkv
// A linear recurrence with a matrix state per head (see csrc/wkv.cu for the formulas): each of r, k, v, the gate and the
// decay reads the input mixed with the previous token's, x + (x_prev - x) * mu_s; r, k, v = W_s mix_s; gate =
// silu(W_g mix_g); decay = exp(-exp(W_2 tanh(W_1 mix_w) + w0)) per head and key channel; the read-out adds a bonus u for
// the current token; each head's result is divided by its root mean square, times a weight, times the gate; then W_o.
// State per request: S (H heads of D x D; 32-bit in the bfloat16 path, 64-bit in the float32 path, whose read-out would
// otherwise lose five digits where a head's sum nearly cancels) and the last input row (float32), zero at the start.
//
// params: hidden_size, num_heads, head_dim, norm_eps, decay_rank (0 or absent: the rows of the checkpoint's W_1).
struct Wkv : Mixer {
    int H, D;
    float eps;
    Tensor w_r, w_k, w_v, w_g, w_1, w_2, w_o, mu, w0, u, out_norm;   // the last four float32

    static TensorSpecs specs(const Json& p) {
        const char* me = "wkv";
        const int64_t d = need_int(p, "hidden_size", me), H = need_int(p, "num_heads", me), D = need_int(p, "head_dim", me),
                      rank = p.get_int("decay_rank", 0);
        if (H <= 0 || D <= 0 || D > imp_wkv_max_head_dim())
            fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": head_dim must lie in (0, " + std::to_string(imp_wkv_max_head_dim()) + "] and num_heads be positive");
        TensorSpecs s;
        for (const char* n : {"mu_r", "mu_k", "mu_v", "mu_g", "mu_w"}) s.emplace_back(n, TensorSpec{{d}, "vector", "normal"});
        for (const char* n : {"r_proj", "k_proj", "v_proj", "g_proj"}) s.emplace_back(n, TensorSpec{{H * D, d}});
        s.emplace_back("decay_down", TensorSpec{{rank > 0 ? rank : -1, d}});
        s.emplace_back("decay_up", TensorSpec{{H * D, rank > 0 ? rank : -1}});
        s.emplace_back("decay_bias", TensorSpec{{H * D}, "vector", "normal"});
        s.emplace_back("bonus", TensorSpec{{H, D}, "vector", "normal"});
        s.emplace_back("out_norm", TensorSpec{{H * D}, "norm", "one_plus_normal"});
        s.emplace_back("o_proj", TensorSpec{{d, H * D}});
        return s;
    }
    static CacheSpec cache(const Json& p) {
        const char* me = "wkv";
        const int64_t d = need_int(p, "hidden_size", me), H = need_int(p, "num_heads", me), D = need_int(p, "head_dim", me);
        CacheSpec s;
        s.kind = CacheSpec::State;
        // room for S as 64-bit words: the float32 path carries the state in 64-bit (see csrc/wkv.cu), bfloat16 uses half of it
        s.states.push_back(StateTensorSpec{"S", {H, D, 2 * D}, F32});
        s.states.push_back(StateTensorSpec{"prev", {d}, F32});
        return s;
    }

    explicit Wkv(BuildArgs& a) {
        H = (int)need_int(a.params, "num_heads", "wkv");
        D = (int)need_int(a.params, "head_dim", "wkv");
        eps = (float)a.params.get_double("norm_eps", 1e-6);
        Runtime& rt = *a.rt;
        w_r = a.tensor("r_proj"), w_k = a.tensor("k_proj"), w_v = a.tensor("v_proj"), w_g = a.tensor("g_proj");
        w_1 = a.tensor("decay_down"), w_2 = a.tensor("decay_up"), w_o = a.tensor("o_proj");
        if (rows(w_1) != cols(w_2)) fail(IMP_ERROR_INVALID_MODEL, "wkv: the two decay matrices do not share their inner size");
        std::vector<Tensor> mus;
        for (const char* n : {"mu_r", "mu_k", "mu_v", "mu_g", "mu_w"}) {
            Tensor t = a.tensor(n);
            mus.push_back(tensor2d(t.data, t.dtype, 1, numel(t)));
        }
        Tensor m = cat_rows(rt, *a.store, mus);
        mu = to_float32(rt, *a.store, m);
        w0 = to_float32(rt, *a.store, a.tensor("decay_bias"));
        u = to_float32(rt, *a.store, a.tensor("bonus"));
        out_norm = to_float32(rt, *a.store, a.tensor("out_norm"));
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        a.store->release(m.data);
        for (const char* n : {"mu_r", "mu_k", "mu_v", "mu_g", "mu_w", "decay_bias", "bonus", "out_norm"}) a.drop(n);
    }

    Branch forward(Step& st, Tensor x, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!cache || cache->view.kind != 2 || cache->view.n_states < 2) fail(IMP_ERROR_INTERNAL, "wkv runs against a state cache");
        const int64_t T = rows(x), d = cols(x), HD = (int64_t)H * D;
        const int dt = rt.dtype == F32 ? 0 : 1;
        float* S = (float*)cache->view.states[0].data;
        float* prev = (float*)cache->view.states[1].data;
        Tensor mixes = rt.empty(5 * T, d);
        const bool single = st.decode_only();
        rt.launches += single ? 1 : 2;
        check_launch(imp_wkv_mix(x.data, x.stride0, (const float*)mu.data, prev, st.view.seq_of_token, st.view.q_start, st.view.state_slots, (int)T,
                                 st.B(), (int)d, mixes.data, single ? 1 : 0, dt, rt.status, rt.stream),
                     "wkv_mix");
        auto mix = [&](int s) { return tensor2d((char*)mixes.data + (size_t)s * (size_t)(T * d) * elem_size(mixes.dtype), mixes.dtype, T, d); };
        Tensor r = rt.empty(T, HD), k = rt.empty(T, HD), v = rt.empty(T, HD), gt = rt.empty(T, HD);
        linear(rt, r, mix(0), w_r);
        linear(rt, k, mix(1), w_k);
        linear(rt, v, mix(2), w_v);
        linear(rt, gt, mix(3), w_g);
        Tensor low = rt.empty(T, rows(w_1));
        linear(rt, low, mix(4), w_1);
        Tensor dlog = rt.empty(T, HD, F32);
        float* o = rt.arena->take<float>((size_t)(T * HD));
        Tensor y = rt.empty(T, HD);
        rt.launches += 3;
        check_launch(imp_tanh_inplace(low.data, numel(low), dt, rt.stream), "tanh");
        linear(rt, dlog, low, w_2);
        // an ordinary dependent launch (see csrc/wkv.cu)
        check_launch(imp_wkv_scan(r.data, k.data, v.data, HD, (const float*)dlog.data, (const float*)w0.data, (const float*)u.data, S, o, st.view.q_start,
                                  st.view.state_slots, st.B(), H, D, dt, rt.stream),
                     "wkv_scan");
        check_launch(imp_wkv_output(y.data, o, gt.data, gt.stride0, (const float*)out_norm.data, eps, (int)T, H, D, dt, rt.stream), "wkv_output");
        return linear(rt, rt.empty(T, rows(w_o)), y, w_o, defer_out);
    }
};

// --------------------------------------------------------------------------------------- routed experts
// A mixture of gated feed-forward experts: router logits z = W_r x + b in 32-bit; the `top_k` experts with the largest
// logits are chosen, weighted by the softmax over the chosen logits; expert e is W_down_e (silu(W_gate_e x) * (W_up_e x)).
// Optionally a shared expert of the same form runs for every token and is added times sigmoid(w_sg . x).
// The experts' matrices are stacked at load; a step sorts its (token, choice) pairs by expert on the device and runs two
// products over the sorted list (csrc/grouped_gemm.cu), so its launches do not depend on the routing.
//
// Options: the router without a bias (`router_bias`: false); sigmoid scores, a chosen expert weighing its score times
// `weight_scale`, not renormalised (`scores`: "sigmoid"; default "softmax" as above); experts in `num_groups` equal groups of
// neighbours of which the `keep_groups` best (by the sum of a group's two largest scores) can be chosen from; a shared expert
// that is added as it is (`shared_gate`: false).
//
// params: hidden_size, num_experts, top_k, expert_size, shared_size (0: no shared expert), router_bias, scores, weight_scale,
//         num_groups, keep_groups, shared_gate.
struct RoutedExperts : FeedForward {
    int64_t d, E, top, F, Fs;
    bool has_bias = true, has_sgate = true;
    int score_mode = 0, n_groups = 0, keep_groups = 0;
    float weight_scale = 1.f;
    Tensor w_gate, w_up, w_down;       // [E * F, d], [E * F, d], [E * d, F]; or w_gate [E * 2F, d], gate and up rows alternating in runs of 8
    bool interleaved = false;
    Tensor router, router_bias, sg;    // float32
    Tensor s_gu, s_down;               // the shared expert
    bool s_interleaved = false;

    static TensorSpecs specs(const Json& p) {
        const char* me = "routed_experts";
        const int64_t d = need_int(p, "hidden_size", me), E = need_int(p, "num_experts", me), top = need_int(p, "top_k", me),
                      F = need_int(p, "expert_size", me), Fs = p.get_int("shared_size", 0);
        if (E <= 0 || top <= 0 || top > E || F <= 0 || Fs < 0) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": 0 < top_k <= num_experts and positive sizes");
        TensorSpecs s;
        s.emplace_back("router", TensorSpec{{E, d}});
        if (p.get_bool("router_bias", true)) s.emplace_back("router_bias", TensorSpec{{E}, "vector", "normal"});
        const int64_t ng = p.get_int("num_groups", 0), keep = p.get_int("keep_groups", 0);
        if (ng < 0 || (ng > 0 && (E % ng || keep <= 0 || keep > ng || top > keep * (E / ng))))
            fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": " + std::to_string(ng) + " groups must divide the " + std::to_string(E) + " experts, and the " +
                                              std::to_string(keep) + " kept groups must hold the " + std::to_string(top) + " chosen experts");
        const std::string sc = p.get_string("scores", "softmax");
        if (sc != "softmax" && sc != "sigmoid") fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": unknown scores '" + sc + "' (known: softmax, sigmoid)");
        for (int64_t e = 0; e < E; ++e) {
            const std::string n = std::to_string(e);
            s.emplace_back("gate_" + n, TensorSpec{{F, d}});
            s.emplace_back("up_" + n, TensorSpec{{F, d}});
            s.emplace_back("down_" + n, TensorSpec{{d, F}});
        }
        if (Fs > 0) {
            s.emplace_back("shared_gate", TensorSpec{{Fs, d}});
            s.emplace_back("shared_up", TensorSpec{{Fs, d}});
            s.emplace_back("shared_down", TensorSpec{{d, Fs}});
            if (p.get_bool("shared_gate", true)) s.emplace_back("shared_mix", TensorSpec{{1, d}});
        }
        return s;
    }

    explicit RoutedExperts(BuildArgs& a) {
        const char* me = "routed_experts";
        d = need_int(a.params, "hidden_size", me), E = need_int(a.params, "num_experts", me), top = need_int(a.params, "top_k", me);
        F = need_int(a.params, "expert_size", me), Fs = a.params.get_int("shared_size", 0);
        has_bias = a.params.get_bool("router_bias", true);
        has_sgate = a.params.get_bool("shared_gate", true);
        score_mode = a.params.get_string("scores", "softmax") == "sigmoid" ? 1 : 0;
        weight_scale = (float)a.params.get_double("weight_scale", 1.0);
        n_groups = (int)a.params.get_int("num_groups", 0);
        keep_groups = (int)a.params.get_int("keep_groups", 0);
        Runtime& rt = *a.rt;
        std::vector<Tensor> gs, us, ds;
        for (int64_t e = 0; e < E; ++e) {
            const std::string n = std::to_string(e);
            gs.push_back(a.tensor("gate_" + n));
            us.push_back(a.tensor("up_" + n));
            ds.push_back(a.tensor("down_" + n));
        }
        // bfloat16 and F a multiple of 8: every expert's gate and up rows alternate in runs of 8, the layout of the fused
        // gate-up product, so that an expert with many rows can go to that product (see forward)
        interleaved = F % SWIGLU_INTERLEAVE == 0 && gs[0].dtype == BF16 && us[0].dtype == BF16;
        if (interleaved) {
            std::vector<Tensor> both;
            for (int64_t e = 0; e < E; ++e) both.push_back(interleave_gate_up(rt, *a.store, gs[(size_t)e], us[(size_t)e]));
            w_gate = cat_rows(rt, *a.store, both);
            IMP_CUDA(cudaStreamSynchronize(rt.stream));
            for (const Tensor& t : both) a.store->release(t.data);
        } else {
            w_gate = cat_rows(rt, *a.store, gs);
            w_up = cat_rows(rt, *a.store, us);
        }
        w_down = cat_rows(rt, *a.store, ds);
        router = to_float32(rt, *a.store, a.tensor("router"));
        if (has_bias) router_bias = to_float32(rt, *a.store, a.tensor("router_bias"));
        if (Fs > 0) {
            Tensor gate = a.tensor("shared_gate"), up = a.tensor("shared_up");
            s_interleaved = Fs % SWIGLU_INTERLEAVE == 0 && gate.dtype == up.dtype;
            s_gu = s_interleaved ? interleave_gate_up(rt, *a.store, gate, up) : cat_rows(rt, *a.store, {gate, up});
            s_down = a.tensor("shared_down");
            if (has_sgate) sg = to_float32(rt, *a.store, a.tensor("shared_mix"));
        }
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        for (int64_t e = 0; e < E; ++e) {
            const std::string n = std::to_string(e);
            a.drop("gate_" + n);
            a.drop("up_" + n);
            a.drop("down_" + n);
        }
        a.drop("router");
        if (has_bias) a.drop("router_bias");
        if (Fs > 0) {
            for (const char* n : {"shared_gate", "shared_up"}) a.drop(n);
            if (has_sgate) a.drop("shared_mix");
        }
    }

    Branch forward(Step& st, Tensor x) override {
        Runtime& rt = *st.rt;
        const int64_t T = rows(x), P = T * top;
        const int dt = rt.dtype == F32 ? 0 : 1;
        int* idx = rt.arena->take<int>((size_t)P);
        float* wts = rt.arena->take<float>((size_t)P);
        float* gate = rt.arena->take<float>((size_t)T);
        int* seg = rt.arena->take<int>((size_t)E + 1);
        int* row_token = rt.arena->take<int>((size_t)P);
        int* pair_row = rt.arena->take<int>((size_t)P);
        rt.launches += 5;
        const bool gated = Fs > 0 && has_sgate;
        check_launch(imp_moe_route_ex(x.data, x.stride0, (int)T, (int)d, (const float*)router.data, has_bias ? (const float*)router_bias.data : nullptr, (int)E,
                                      (int)top, gated ? (const float*)sg.data : nullptr, idx, wts, gate, score_mode, n_groups, keep_groups, weight_scale, dt,
                                      rt.stream),
                     "moe_route");
        check_launch(imp_moe_sort(idx, (int)T, (int)top, (int)E, seg, row_token, pair_row, rt.stream), "moe_sort");
        Tensor act = rt.empty(P, F);
        Tensor y = rt.empty(P, d);
        // Portions of prompts with much work an expert (rows x F x d of 2^31 and more on average): the list's offsets come to
        // the host, and every expert's rows go to the tensor-memory products as a dense matrix (the wait costs one round
        // trip a layer; 2,048 tokens on 16 experts of 4096 x 4096: 1.2 against 2.0 ms a layer; with experts of 1024 x 1024
        // the products' fixed cost loses: 5.9 against 4.0 ms for four layers).  All other steps, and every step that may
        // be captured into a graph, run the two products over groups, whose launches do not depend on the routing.
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        IMP_CUDA(cudaStreamIsCapturing(rt.stream, &capturing));
        static const double dense_work = [] { const std::string e = env_string("IMP_B200_MOE_DENSE_WORK", ""); return e.empty() ? 2147483648.0 : std::atof(e.c_str()); }();
        if (interleaved && !st.decode_only() && capturing == cudaStreamCaptureStatusNone && dense_work > 0 &&
            (double)P / (double)E * (double)F * (double)d >= dense_work) {
            std::vector<int> hseg((size_t)E + 1);
            Tensor xs = rt.empty(P, d);
            check_launch(imp_gather_rows(xs.data, x.data, x.stride0, row_token, (int)P, (int)d, dt, rt.stream), "gather_rows");
            IMP_CUDA(cudaMemcpyAsync(hseg.data(), seg, hseg.size() * 4, cudaMemcpyDeviceToHost, rt.stream));
            IMP_CUDA(cudaStreamSynchronize(rt.stream));
            const size_t el = elem_size(rt.dtype);
            for (int64_t e = 0; e < E; ++e) {
                const int64_t a0 = hseg[(size_t)e], n = hseg[(size_t)e + 1] - a0;
                if (n <= 0) continue;
                Tensor xe = tensor2d((char*)xs.data + (size_t)(a0 * d) * el, rt.dtype, n, d);
                Tensor ae = tensor2d((char*)act.data + (size_t)(a0 * F) * el, rt.dtype, n, F);
                Tensor ye = tensor2d((char*)y.data + (size_t)(a0 * d) * el, rt.dtype, n, d);
                Tensor wgu = tensor2d((char*)w_gate.data + (size_t)(e * 2 * F * d) * el, w_gate.dtype, 2 * F, d);
                Tensor wd = tensor2d((char*)w_down.data + (size_t)(e * d * F) * el, w_down.dtype, d, F);
                linear_swiglu(rt, ae, xe, wgu);
                linear(rt, ye, ae, wd);
            }
        } else {
            check_launch(imp_grouped_gemm(act.data, F, 0, x.data, x.stride0, 0, row_token, w_gate.data, interleaved ? nullptr : w_up.data,
                                          (interleaved ? 2 : 1) * F * d, d, seg, (int)P, (int)F, (int)d, (int)E, interleaved ? 2 : 1, dt, rt.stream),
                         "grouped_gemm (experts, gate and up)");
            check_launch(imp_grouped_gemm(y.data, d, 0, act.data, F, 0, nullptr, w_down.data, nullptr, d * F, F, seg, (int)P, (int)d, (int)F, (int)E, 0,
                                          dt, rt.stream),
                         "grouped_gemm (experts, down)");
        }
        Tensor shared{};
        if (Fs > 0) {
            Tensor sa = rt.empty(T, Fs);
            if (s_interleaved) {
                linear_swiglu(rt, sa, x, s_gu);
            } else {
                Tensor gu = rt.empty(T, 2 * Fs);
                linear(rt, gu, x, s_gu);
                swiglu(rt, sa, gu, 0);
            }
            shared = rt.empty(T, d);
            linear(rt, shared, sa, s_down);
        }
        Tensor out = rt.empty(T, d);
        check_launch(imp_moe_combine(out.data, y.data, pair_row, wts, (int)T, (int)top, Fs > 0 ? shared.data : nullptr, gated ? gate : nullptr, (int)d,
                                     dt, rt.stream),
                     "moe_combine");
        return Branch::of(out);
    }
};

// ------------------------------------------------------------------------- pre-norm block with scaled branches
// h += m * s1 (.) mixer(norm1(h));  h += m * s2 (.) ffn(norm2(h)): a constant m and a learned factor per channel for each
// branch.  The factors ride with the branch (Branch::col_scale) and are multiplied in, in 32-bit, by the norm that adds
// the branch into the stream; where the next normaliser cannot do that the branch is scaled before it is handed on.
// Slots: mixer_norm, mixer, and with has_ffn (default true) ffn_norm, feed_forward.  Tensors: mixer_scale [d] and with
// has_ffn ffn_scale [d].  params: hidden_size, residual_mult (default 1), has_ffn.
struct ScaledPreNormBlock : Block {
    Mixer* mixer_;
    FeedForward* ffn = nullptr;
    Norm *norm1, *norm2 = nullptr;
    Tensor s1, s2;   // float32, times residual_mult
    explicit ScaledPreNormBlock(BuildArgs& a) : mixer_(part_cast<Mixer>(a.part("mixer"), "a mixer")), norm1(part_cast<Norm>(a.part("mixer_norm"), "a norm")) {
        const float m = (float)a.params.get_double("residual_mult", 1.0);
        Runtime& rt = *a.rt;
        auto scaled = [&](const char* name) {
            Tensor f = to_float32(rt, *a.store, a.tensor(name));
            check_launch(imp_scaled_sum(f.data, f.data, m, nullptr, 0.f, nullptr, 0.f, 1, (int)numel(f), F32, rt.stream), "scaled_sum");
            return f;
        };
        s1 = scaled("mixer_scale");
        if (a.params.get_bool("has_ffn", true)) {
            ffn = part_cast<FeedForward>(a.part("feed_forward"), "a feed-forward");
            norm2 = part_cast<Norm>(a.part("ffn_norm"), "a norm");
            s2 = scaled("ffn_scale");
        }
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        a.drop("mixer_scale");
        if (ffn) a.drop("ffn_scale");
    }
    static std::vector<Slot> slots(const Json& p) {
        std::vector<Slot> s = {{"mixer_norm", "norm"}, {"mixer", "mixer"}};
        if (p.get_bool("has_ffn", true)) {
            s.push_back({"ffn_norm", "norm"});
            s.push_back({"feed_forward", "feed_forward"});
        }
        return s;
    }
    static TensorSpecs specs(const Json& p) {
        const int64_t d = need_int(p, "hidden_size", "scaled_prenorm");
        TensorSpecs s;
        s.emplace_back("mixer_scale", TensorSpec{{d}, "norm", "one_plus_normal"});
        if (p.get_bool("has_ffn", true)) s.emplace_back("ffn_scale", TensorSpec{{d}, "norm", "one_plus_normal"});
        return s;
    }
    bool takes_split_sum() const override { return norm1->takes_split_sum(); }
    bool takes_column_scale() const override { return norm1->takes_column_scale(); }
    Mixer* mixer() const override { return mixer_; }
    std::vector<Part*> parts() const override {
        std::vector<Part*> p = {norm1, mixer_};
        if (ffn) {
            p.push_back(norm2);
            p.push_back(ffn);
        }
        return p;
    }
    bool graph_safe() const override {
        for (Part* p : parts())
            if (!p->graph_safe()) return false;
        return true;
    }
    // The branch with its factors: riding along if the one who adds it multiplies them in, applied now otherwise.
    Branch with_scale(Step& st, Branch b, const Tensor& s, bool consumer_takes) const {
        b.col_scale = (const float*)s.data;
        if (consumer_takes) return b;
        return Branch::of(summed(st, b));
    }
    Branch forward(Step& st, Tensor h, const Branch& pending, LayerCache* cache) override {
        Tensor x = norm1->add_norm(st, h, pending);
        mixer_->defer_out = false;
        Branch a = with_scale(st, mixer_->forward(st, x, cache), s1, ffn ? norm2->takes_column_scale() : scale_pending);
        stage(st, "mixer", a);
        if (!ffn) return a;
        x = norm2->add_norm(st, h, a);
        ffn->defer_out = false;
        Branch f = with_scale(st, ffn->forward(st, x), s2, scale_pending);
        stage(st, "feed_forward", f);
        return f;
    }
};

// ------------------------------------------------------------------------------ the stream re-made from two
// h <- W [h ; x0]: one linear map over the stream and the embedding's output side by side, W [d, 2d] with the stream's
// columns first.  What the block before left pending is added first.  No parts; one tensor, `weight`.
// params: hidden_size.
struct StreamReinjectBlock : Block {
    Tensor weight;
    explicit StreamReinjectBlock(BuildArgs& a) : weight(a.tensor("weight")) {}
    static std::vector<Slot> slots(const Json&) { return {}; }
    static TensorSpecs specs(const Json& p) {
        const int64_t d = need_int(p, "hidden_size", "stream_reinject");
        TensorSpecs s;
        s.emplace_back("weight", TensorSpec{{d, 2 * d}});
        return s;
    }
    bool takes_column_scale() const override { return true; }
    bool wants_embedding() const override { return true; }
    std::vector<Part*> parts() const override { return {}; }
    Branch forward(Step& st, Tensor h, const Branch& pending, LayerCache*) override {
        Runtime& rt = *st.rt;
        if (!st.embedding_out.data) fail(IMP_ERROR_INTERNAL, "stream_reinject: the step kept no copy of the embedding's output");
        const int64_t T = rows(h), d = cols(h);
        const Branch b = parts_summed(rt, pending);
        Tensor both = rt.empty(T, 2 * d);
        ++rt.launches;
        check_launch(imp_concat_streams(both.data, (const float*)h.data, b.empty() ? nullptr : b.t.data, b.col_scale, (const float*)st.embedding_out.data,
                                        (int)T, (int)d, rt.dtype == F32 ? 0 : 1, rt.stream),
                     "concat_streams");
        linear(rt, h, both, weight);   // the stream is float32: the product's sums go there unrounded
        stage(st, "reinject", h);
        return Branch();
    }
};

template <typename T> PartClass class_of(TensorSpecs (*specs)(const Json&)) {
    PartClass c;
    if (specs) c.tensor_specs = specs;
    c.create = [](BuildArgs& a) -> Part* { return new T(a); };
    return c;
}

}  // namespace

void register_routed_parts() {
    PartClass norm = class_of<LayerNorm>(nullptr);
    norm.tensor_specs = [](const Json& p) {
        TensorSpecs s;
        s.emplace_back("weight", TensorSpec{{need_int(p, "size", "layernorm")}, "norm", "one_plus_normal"});
        if (p.get_bool("bias", false)) s.emplace_back("bias", TensorSpec{{need_int(p, "size", "layernorm")}, "vector", "normal"});
        return s;
    };
    register_part_class("norm", "layernorm", norm, true);
    PartClass la = class_of<LatentAttention>(&LatentAttention::specs);
    la.cache_spec = &LatentAttention::cache;
    register_part_class("mixer", "latent_attention", la, true);
    PartClass wkv = class_of<Wkv>(&Wkv::specs);
    wkv.cache_spec = &Wkv::cache;
    register_part_class("mixer", "wkv", wkv, true);
    register_part_class("feed_forward", "routed_experts", class_of<RoutedExperts>(&RoutedExperts::specs), true);
    PartClass block = class_of<ScaledPreNormBlock>(&ScaledPreNormBlock::specs);
    block.part_slots = &ScaledPreNormBlock::slots;
    register_part_class("block", "scaled_prenorm", block, true);
    PartClass inject = class_of<StreamReinjectBlock>(&StreamReinjectBlock::specs);
    inject.part_slots = &StreamReinjectBlock::slots;
    register_part_class("block", "stream_reinject", inject, true);
}

}  // namespace imp
