// Part kinds: a block with a norm before and after each sublayer, a short causal convolution added to what a sublayer
// reads, differential softmax attention (two score maps per head over the same values), and a feed-forward whose
// activation is a normalised polynomial.  Every size and constant is a parameter; no kind knows which model it is in.
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

Tensor upload_f32(Runtime& rt, WeightStore& store, const std::vector<float>& v) {
    Tensor t = store.alloc(F32, {(int64_t)v.size()});
    IMP_CUDA(cudaMemcpyAsync(t.data, v.data(), v.size() * 4, cudaMemcpyHostToDevice, rt.stream));
    IMP_CUDA(cudaStreamSynchronize(rt.stream));
    return t;
}

std::vector<float> download_f32(Runtime& rt, WeightStore& store, const Tensor& t) {
    Tensor f = to_float32(rt, store, t);
    std::vector<float> v((size_t)numel(f));
    IMP_CUDA(cudaMemcpyAsync(v.data(), f.data, v.size() * 4, cudaMemcpyDeviceToHost, rt.stream));
    IMP_CUDA(cudaStreamSynchronize(rt.stream));
    store.release(f.data);
    return v;
}

// Rows r0 .. r0 + n of a dense matrix.
Tensor row_slice(const Tensor& t, int64_t r0, int64_t n) {
    return tensor2d((char*)t.data + (size_t)(r0 * t.stride0) * elem_size(t.dtype), t.dtype, n, cols(t), t.stride0);
}

// ------------------------------------------------------------------------------- convolution on a sublayer's input
// out = x + conv(x): a causal convolution over time on each channel, conv(x)_t = sum_j w[:, j] x_(t - taps + 1 + j), zeros
// before a request's start.  It stands in a mixer slot because it owns state: a request's last taps - 1 inputs (float32).
// params: hidden_size, taps.  Tensor: weight [hidden_size, taps].
struct ResidualConv : Mixer {
    int C, taps;
    Tensor w;   // float32, tap by tap: [taps, hidden_size]
    static TensorSpecs specs(const Json& p) {
        TensorSpecs s;
        s.emplace_back("weight", TensorSpec{{need_int(p, "hidden_size", "residual_conv"), need_int(p, "taps", "residual_conv")}, "vector", "normal"});
        return s;
    }
    static CacheSpec cache(const Json& p) {
        const int64_t C = need_int(p, "hidden_size", "residual_conv"), taps = need_int(p, "taps", "residual_conv");
        if (C <= 0 || taps < 1 || taps > 64) fail(IMP_ERROR_INVALID_MODEL, "residual_conv: taps must lie in [1, 64] and hidden_size be positive");
        CacheSpec s;
        s.kind = CacheSpec::State;
        s.states.push_back(StateTensorSpec{"inputs", {std::max<int64_t>(taps - 1, 1), C}, F32});
        return s;
    }
    explicit ResidualConv(BuildArgs& a) {
        C = (int)need_int(a.params, "hidden_size", "residual_conv");
        taps = (int)need_int(a.params, "taps", "residual_conv");
        const std::vector<float> by_channel = download_f32(*a.rt, *a.store, a.tensor("weight"));
        std::vector<float> by_tap((size_t)C * taps);
        for (int c = 0; c < C; ++c)
            for (int j = 0; j < taps; ++j) by_tap[(size_t)j * C + c] = by_channel[(size_t)c * taps + j];
        w = upload_f32(*a.rt, *a.store, by_tap);
        a.drop("weight");
    }
    // A step of single tokens: the whole part is one operation per row, which the norm before it may run in its own kernel.
    bool as_row_op(Step& st, LayerCache* cache, RowOp* out) override {
        if (!st.decode_only() || !cache || cache->view.kind != 2 || cache->view.n_states < 1) return false;
        out->conv_w = (const float*)w.data;
        out->taps = taps;
        out->width = C;
        out->conv_state = (float*)cache->view.states[0].data;
        out->taken = false;
        return true;
    }
    Branch forward(Step& st, Tensor x, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!cache || cache->view.kind != 2 || cache->view.n_states < 1) fail(IMP_ERROR_INTERNAL, "residual_conv runs against a state cache");
        if (cols(x) != C) fail(IMP_ERROR_INVALID_ARG, "residual_conv: the input's width is not hidden_size");
        const int64_t T = rows(x);
        Tensor out = rt.empty(T, C);
        float* state = (float*)cache->view.states[0].data;
        const bool single = st.decode_only();
        ++rt.launches;
        check_launch(imp_add_conv(out.data, x.data, x.stride0, (const float*)w.data, taps, state, st.view.seq_of_token, st.view.q_start, st.view.state_slots,
                                  (int)T, st.B(), C, single ? 1 : 0, rt.dtype, rt.status, rt.stream),
                     "add_conv");
        if (!single && taps > 1) {
            ++rt.launches;
            check_launch(imp_gdr_conv_state(x.data, x.stride0, state, taps, C, st.view.q_start, st.view.state_slots, st.B(), rt.dtype, rt.stream), "gdr_conv_state");
        }
        return Branch::of(out);
    }
};

// --------------------------------------------------------------------------------------- differential attention
// Grouped-query softmax attention in which every head holds two score maps over the same values:
//   q [H heads x 2 maps x D], k [G heads x 2 maps x D], v [G heads x Dv] = W x, laid out head by head as [map 1, map 2];
//   optionally the first rot_dims entries of every map of q and k are rotated (pairs of neighbours 2i, 2i + 1 or halves
//   i, i + rot_dims/2; angle pos * f_i, f_i = rot_base^(-2i/rot_dims), optionally with long wavelengths slowed down: f kept
//   where 2 pi / f < original / high, f / factor where 2 pi / f > original / low, blended linearly in between);
//   a_m = softmax(scale q_m . k_m over the keys a query sees: all earlier ones, or the last `window`) v for m = 1, 2;
//   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init (four learned vectors of D, one number for the layer);
//   o = a_1 - lambda a_2;  y = o / rms(o) per head * (1 - lambda_init);  out = W_o y.
// The paged attention kernels run it as 2H query heads over 2G key heads: the query rows are ordered (group, map, head
// in group) at load, so that a map's heads share that map's key head, and each of a group's two key heads caches a copy
// of the group's values.  The cache's head size is the larger of D and Dv, rounded up to a multiple of 16.
// params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim (default head_dim), scale (default head_dim^-1/2),
//         lambda_init, norm_eps, window (0: all), rot_dims (0: none), rot_base, rot_pairing ("neighbours" | "halves"),
//         rot_scaling {factor, low, high, original} (optional).
struct DifferentialAttention : Mixer {
    AttentionGeometry g;   // 2H query heads, 2G key heads, over the cache's head size
    int H, G, D, Dv, rot, pairing;
    float eps, lambda_init;
    Tensor w_in, w_o, inv_freq, lambda;

    struct Sizes {
        int64_t d, H, G, D, Dv, Dc;
    };
    static Sizes sizes(const Json& p) {
        const char* me = "differential_attention";
        Sizes s{need_int(p, "hidden_size", me), need_int(p, "num_heads", me), need_int(p, "num_kv_heads", me), need_int(p, "head_dim", me), 0, 0};
        s.Dv = p.get_int("value_dim", s.D);
        if (s.G <= 0 || s.H <= 0 || s.H % s.G) fail(IMP_ERROR_INVALID_MODEL, std::to_string(s.H) + " query heads are not a multiple of " + std::to_string(s.G) + " kv heads");
        if (s.D <= 0 || s.Dv <= 0 || std::max(s.D, s.Dv) > 512) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": head_dim and value_dim must lie in (0, 512]");
        s.Dc = (std::max(s.D, s.Dv) + 15) / 16 * 16;
        return s;
    }
    static TensorSpecs specs(const Json& p) {
        const Sizes z = sizes(p);
        TensorSpecs s;
        s.emplace_back("q_proj", TensorSpec{{z.H * 2 * z.D, z.d}});
        s.emplace_back("k_proj", TensorSpec{{z.G * 2 * z.D, z.d}});
        s.emplace_back("v_proj", TensorSpec{{z.G * z.Dv, z.d}});
        for (const char* n : {"lambda_q1", "lambda_k1", "lambda_q2", "lambda_k2"}) s.emplace_back(n, TensorSpec{{z.D}, "vector", "normal"});
        s.emplace_back("o_proj", TensorSpec{{z.d, z.H * z.Dv}});
        return s;
    }
    static CacheSpec cache(const Json& p) {
        const Sizes z = sizes(p);
        return CacheSpec::paged((int)(2 * z.G), (int)z.Dc, (int)p.get_int("window", 0));
    }
    // f_i for i < rot/2, with the optional slowing of long wavelengths; computed in double, stored in 32-bit.
    static std::vector<float> frequencies(const Json& p, int rot) {
        const char* me = "differential_attention";
        const double base = p.get_double("rot_base", 10000.0);
        const Json* sc = p.find("rot_scaling");
        const bool scaled = sc && sc->is_object();
        double factor = 1, low = 1, high = 1, original = 1;
        if (scaled) {
            factor = need_double(*sc, "factor", me), low = need_double(*sc, "low", me), high = need_double(*sc, "high", me);
            original = need_double(*sc, "original", me);
            if (!(factor > 0) || !(high > low) || !(low > 0) || !(original > 0))
                fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": rot_scaling needs factor > 0, 0 < low < high and original > 0");
        }
        std::vector<float> f((size_t)rot / 2);
        const double two_pi = 6.283185307179586476925286766559;
        for (int i = 0; i < rot / 2; ++i) {
            double v = std::pow(base, -2.0 * i / rot);
            if (scaled) {
                const double wave = two_pi / v;
                if (wave > original / low) {
                    v /= factor;
                } else if (!(wave < original / high)) {
                    const double s = (original / wave - low) / (high - low);
                    v = (1.0 - s) * v / factor + s * v;
                }
            }
            f[(size_t)i] = (float)v;
        }
        return f;
    }
    explicit DifferentialAttention(BuildArgs& a) {
        const char* me = "differential_attention";
        const Json& p = a.params;
        const Sizes z = sizes(p);
        H = (int)z.H, G = (int)z.G, D = (int)z.D, Dv = (int)z.Dv;
        g.hq = 2 * H, g.hkv = 2 * G, g.dh = (int)z.Dc;
        g.window = (int)p.get_int("window", 0);
        if (g.window < 0) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": 'window' must not be negative");
        const double scale = p.get_double("scale", 0.0);
        g.scale = scale > 0 ? (float)scale : (float)(1.0 / std::sqrt((double)D));
        eps = (float)p.get_double("norm_eps", 1e-6);
        lambda_init = (float)need_double(p, "lambda_init", me);
        rot = (int)p.get_int("rot_dims", 0);
        if (rot < 0 || rot % 2 || rot > D) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": rot_dims " + std::to_string(rot) + " must be even and within head_dim " + std::to_string(D));
        const std::string pr = p.get_string("rot_pairing", "neighbours");
        if (pr != "neighbours" && pr != "halves") fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": unknown rot_pairing '" + pr + "' (known: neighbours, halves)");
        pairing = pr == "neighbours" ? 1 : 0;
        Runtime& rt = *a.rt;
        // query rows in the order (group, map, head in group)
        const Tensor wq = a.tensor("q_proj");
        const int R = H / G;
        std::vector<Tensor> in;
        for (int gi = 0; gi < G; ++gi)
            for (int m = 0; m < 2; ++m)
                for (int j = 0; j < R; ++j) in.push_back(row_slice(wq, ((int64_t)(gi * R + j) * 2 + m) * D, D));
        in.push_back(a.tensor("k_proj"));
        in.push_back(a.tensor("v_proj"));
        const int64_t n = (int64_t)(2 * H + 2 * G) * D + (int64_t)G * Dv, pad = (8 - n % 8) % 8;
        Tensor zeros{};
        if (pad) {
            zeros = a.store->alloc(wq.dtype, {pad, z.d});
            IMP_CUDA(cudaMemsetAsync(zeros.data, 0, (size_t)numel(zeros) * elem_size(zeros.dtype), rt.stream));
            in.push_back(zeros);
        }
        w_in = cat_rows(rt, *a.store, in);
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        if (pad) a.store->release(zeros.data);
        w_o = a.tensor("o_proj");
        if (rot > 0) inv_freq = upload_f32(rt, *a.store, frequencies(p, rot));
        // lambda, one number, in 32-bit
        const std::vector<float> q1 = download_f32(rt, *a.store, a.tensor("lambda_q1")), k1 = download_f32(rt, *a.store, a.tensor("lambda_k1")),
                                 q2 = download_f32(rt, *a.store, a.tensor("lambda_q2")), k2 = download_f32(rt, *a.store, a.tensor("lambda_k2"));
        float d1 = 0.f, d2 = 0.f;
        for (int i = 0; i < D; ++i) {
            d1 += q1[(size_t)i] * k1[(size_t)i];
            d2 += q2[(size_t)i] * k2[(size_t)i];
        }
        lambda = upload_f32(rt, *a.store, {std::exp(d1) - std::exp(d2) + lambda_init});
        for (const char* nm : {"q_proj", "k_proj", "v_proj", "lambda_q1", "lambda_k1", "lambda_q2", "lambda_k2"}) a.drop(nm);
    }
    std::vector<TilingSpec> tilings() const override { return attention_tilings(); }

    Branch forward(Step& st, Tensor x, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!cache || !cache->paged()) fail(IMP_ERROR_INTERNAL, "differential_attention runs against a paged cache");
        const int64_t T = rows(x);
        const ImpCacheView& cv = cache->view;
        Tensor proj = rt.empty(T, rows(w_in));
        linear(rt, proj, x, w_in);
        Tensor q = rt.empty(T, (int64_t)g.hq * g.dh);
        rt.launches += 2;
        check_launch(imp_qkv_prepare_ex(proj.data, proj.stride0, (int)T, g.hq, g.hkv, D, Dv, g.dh, nullptr, nullptr, eps, 0,
                                        rot > 0 ? (const float*)inv_freq.data : nullptr, rot, pairing, 2, nullptr, st.view.positions, st.view.seq_of_token,
                                        cv.block_table, cv.bt_stride, st.B(), q.data, q.stride0, cv.writes ? cv.k_pages : nullptr,
                                        cv.writes ? cv.v_pages : nullptr, cv.page_size, cv.num_pages, rt.dtype, rt.status, rt.stream),
                     "qkv_prepare");
        Tensor attn = rt.empty(T, (int64_t)g.hq * g.dh);
        paged_attention(st, attn, q, g, *cache, tiling_ids, nullptr);
        Tensor y = rt.empty(T, (int64_t)H * Dv);
        check_launch(imp_diff_combine(y.data, attn.data, attn.stride0, (int)T, G, H / G, g.dh, Dv, (const float*)lambda.data, eps, 1.f - lambda_init, rt.dtype,
                                      rt.stream),
                     "diff_combine");
        return linear(rt, rt.empty(T, rows(w_o)), y, w_o, defer_out);
    }
};

// ---------------------------------------------------------------------------------- polynomial feed-forward
// out = W_down act(W_up x), act(z) = a z / rms(z) + b z^2 / rms(z^2) + c z^3 / rms(z^3) + e with powers taken element by
// element, rms over a token's intermediate_size values (eps inside the root), and (a, b, c, e) the tensor `coef`.
// params: hidden_size, intermediate_size, norm_eps.
struct PolyNormMLP : FeedForward {
    int64_t f;
    float eps;
    Tensor w_up, w_down, coef;   // coef float32 [4]
    static TensorSpecs specs(const Json& p) {
        const int64_t d = need_int(p, "hidden_size", "polynorm_mlp"), f = need_int(p, "intermediate_size", "polynorm_mlp");
        TensorSpecs s;
        s.emplace_back("up_proj", TensorSpec{{f, d}});
        s.emplace_back("down_proj", TensorSpec{{d, f}});
        s.emplace_back("coef", TensorSpec{{4}, "vector", "normal"});
        return s;
    }
    explicit PolyNormMLP(BuildArgs& a) {
        f = need_int(a.params, "intermediate_size", "polynorm_mlp");
        eps = (float)a.params.get_double("norm_eps", 1e-6);
        w_up = a.tensor("up_proj");
        w_down = a.tensor("down_proj");
        coef = to_float32(*a.rt, *a.store, a.tensor("coef"));
        IMP_CUDA(cudaStreamSynchronize(a.rt->stream));
        a.drop("coef");
    }
    Branch forward(Step& st, Tensor x) override {
        Runtime& rt = *st.rt;
        const int64_t T = rows(x);
        Tensor z = rt.empty(T, f);
        linear(rt, z, x, w_up);
        Tensor hid = rt.empty(T, f);
        ++rt.launches;
        check_launch(imp_polynorm(hid.data, z.data, z.stride0, (int)T, (int)f, (const float*)coef.data, eps, rt.dtype, rt.stream), "polynorm");
        return linear(rt, rt.empty(T, rows(w_down)), hid, w_down, defer_out);
    }
};

// ------------------------------------------------------------------------- norms before and after each sublayer
// h += post1(mixer(c1(norm1(h))));  h += post2(ffn(c2(norm2(h)))): a norm before and a norm after each sublayer, and with
// `input_conv` a part c = x + conv(x) on what each sublayer reads (a mixer-category part that owns its state, such as
// residual_conv).  The norm after a sublayer rides with the branch (Branch::own_norm) to whoever adds the branch into the
// stream, who normalises it in the same pass; where the consumer cannot do that it is applied before the branch is handed on.
// Slots: mixer_norm, (mixer_conv,) mixer, mixer_post_norm, and with has_ffn (default true) ffn_norm, (ffn_conv,)
// feed_forward, ffn_post_norm.  params: has_ffn, input_conv (default false).
struct SandwichBlock : Block {
    Mixer *mixer_, *conv1 = nullptr, *conv2 = nullptr;
    FeedForward* ffn = nullptr;
    Norm *norm1, *post1, *norm2 = nullptr, *post2 = nullptr;
    BranchNorm own1{}, own2{};
    explicit SandwichBlock(BuildArgs& a)
        : mixer_(part_cast<Mixer>(a.part("mixer"), "a mixer")), norm1(part_cast<Norm>(a.part("mixer_norm"), "a norm")),
          post1(part_cast<Norm>(a.part("mixer_post_norm"), "a norm")) {
        const bool conv = a.params.get_bool("input_conv", false);
        if (conv) conv1 = part_cast<Mixer>(a.part("mixer_conv"), "a mixer-category part");
        if (a.params.get_bool("has_ffn", true)) {
            ffn = part_cast<FeedForward>(a.part("feed_forward"), "a feed-forward");
            norm2 = part_cast<Norm>(a.part("ffn_norm"), "a norm");
            post2 = part_cast<Norm>(a.part("ffn_post_norm"), "a norm");
            if (conv) conv2 = part_cast<Mixer>(a.part("ffn_conv"), "a mixer-category part");
        }
        if (!post1->as_branch_norm(&own1) || (post2 && !post2->as_branch_norm(&own2)))
            fail(IMP_ERROR_INVALID_MODEL, "sandwich: the norms after the sublayers must be able to ride with a branch (layernorm)");
    }
    static std::vector<Slot> slots(const Json& p) {
        const bool conv = p.get_bool("input_conv", false);
        std::vector<Slot> s = {{"mixer_norm", "norm"}};
        if (conv) s.push_back({"mixer_conv", "mixer"});
        s.push_back({"mixer", "mixer"});
        s.push_back({"mixer_post_norm", "norm"});
        if (p.get_bool("has_ffn", true)) {
            s.push_back({"ffn_norm", "norm"});
            if (conv) s.push_back({"ffn_conv", "mixer"});
            s.push_back({"feed_forward", "feed_forward"});
            s.push_back({"ffn_post_norm", "norm"});
        }
        return s;
    }
    bool takes_split_sum() const override { return norm1->takes_split_sum(); }
    bool takes_column_scale() const override { return norm1->takes_column_scale(); }
    bool takes_normed_branch() const override { return norm1->takes_normed_branch(); }
    Mixer* mixer() const override { return mixer_; }
    std::vector<Mixer*> mixers() const override {   // in the order of the mixer-category slots
        std::vector<Mixer*> m;
        if (conv1) m.push_back(conv1);
        m.push_back(mixer_);
        if (conv2) m.push_back(conv2);
        return m;
    }
    std::vector<Part*> parts() const override {
        std::vector<Part*> p = {norm1};
        if (conv1) p.push_back(conv1);
        p.push_back(mixer_);
        p.push_back(post1);
        if (ffn) {
            p.push_back(norm2);
            if (conv2) p.push_back(conv2);
            p.push_back(ffn);
            p.push_back(post2);
        }
        return p;
    }
    bool graph_safe() const override {
        for (Part* p : parts())
            if (!p->graph_safe()) return false;
        return true;
    }
    // The branch with the norm that follows its sublayer: riding along if the one who adds it normalises it, applied now otherwise.
    Branch with_norm(Step& st, const Branch& b, const BranchNorm& own, bool consumer_takes) const {
        Branch out = Branch::of(summed(st, b));
        out.own_norm = own;
        if (consumer_takes) return out;
        return Branch::of(summed(st, out));
    }
    // What a sublayer reads: the norm of the stream (the branch added on the way), then the part in front of the sublayer.  Where
    // that part is one operation per row in this step, the norm is offered it and the part runs only if the norm declined.
    Tensor normed_input(Step& st, Norm* norm, Tensor h, const Branch& branch, Mixer* conv, LayerCache* c_conv) const {
        RowOp op;
        const bool offered = conv && conv->as_row_op(st, c_conv, &op) && cols(h) == op.width;
        st.row_op = offered ? &op : nullptr;
        Tensor x = norm->add_norm(st, h, branch);
        st.row_op = nullptr;
        if (conv && !(offered && op.taken)) x = summed(st, conv->forward(st, x, c_conv));
        return x;
    }
    Branch forward(Step& st, Tensor h, const Branch& pending, LayerCache* cache) override {
        // caches in slot order: (conv1,) mixer, (conv2); a block whose only mixer has no cache gets a null pointer
        LayerCache* c_conv1 = conv1 ? &cache[0] : nullptr;
        LayerCache* c_mixer = conv1 ? &cache[1] : cache;
        LayerCache* c_conv2 = conv2 ? &cache[2] : nullptr;
        if (c_mixer && !c_mixer->view.kind) c_mixer = nullptr;
        Tensor x = normed_input(st, norm1, h, pending, conv1, c_conv1);
        mixer_->defer_out = false;
        Branch a = with_norm(st, mixer_->forward(st, x, c_mixer), own1, ffn ? norm2->takes_normed_branch() : norm_pending);
        stage(st, "mixer", a);
        if (!ffn) return a;
        x = normed_input(st, norm2, h, a, conv2, c_conv2);
        ffn->defer_out = false;
        Branch f = with_norm(st, ffn->forward(st, x), own2, norm_pending);
        stage(st, "feed_forward", f);
        return f;
    }
};

template <typename T> PartClass class_of(TensorSpecs (*specs)(const Json&)) {
    PartClass c;
    if (specs) c.tensor_specs = specs;
    c.create = [](BuildArgs& a) -> Part* { return new T(a); };
    return c;
}

}  // namespace

void register_sandwich_parts() {
    PartClass conv = class_of<ResidualConv>(&ResidualConv::specs);
    conv.cache_spec = &ResidualConv::cache;
    register_part_class("mixer", "residual_conv", conv, true);
    PartClass at = class_of<DifferentialAttention>(&DifferentialAttention::specs);
    at.cache_spec = &DifferentialAttention::cache;
    register_part_class("mixer", "differential_attention", at, true);
    register_part_class("feed_forward", "polynorm_mlp", class_of<PolyNormMLP>(&PolyNormMLP::specs), true);
    PartClass block = class_of<SandwichBlock>(nullptr);
    block.part_slots = &SandwichBlock::slots;
    register_part_class("block", "sandwich", block, true);
}

}  // namespace imp
