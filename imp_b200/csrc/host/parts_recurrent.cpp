// Part kinds: three recurrent mixers over the general scan of csrc/delta_rule.cu (retention, the generalised delta
// rule, the delta rule with a decay per key channel), softmax attention whose heads are normalised, rotated in part,
// scaled, masked by chunks and gated, and a post-norm block (the normalised sum is the stream) that holds one mixer
// or two side by side.  Every size and constant is a parameter; no kind knows which model it is in.
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

// Matrices stacked along the output dimension, the rows padded with zeros to a multiple of 8 (what the products'
// tensor maps take).
Tensor cat_rows_padded(Runtime& rt, WeightStore& store, std::vector<Tensor> in) {
    int64_t n = 0;
    for (const Tensor& t : in) n += rows(t);
    const int64_t pad = (8 - n % 8) % 8;
    Tensor zeros{};
    if (pad) {
        zeros = store.alloc(in[0].dtype, {pad, cols(in[0])});
        IMP_CUDA(cudaMemsetAsync(zeros.data, 0, (size_t)numel(zeros) * elem_size(zeros.dtype), rt.stream));
        in.push_back(zeros);
    }
    Tensor out = cat_rows(rt, store, in);
    IMP_CUDA(cudaStreamSynchronize(rt.stream));
    if (pad) store.release(zeros.data);
    return out;
}

Tensor upload_f32(Runtime& rt, WeightStore& store, const std::vector<float>& v) {
    Tensor t = store.alloc(F32, {(int64_t)v.size()});
    IMP_CUDA(cudaMemcpyAsync(t.data, v.data(), v.size() * 4, cudaMemcpyHostToDevice, rt.stream));
    IMP_CUDA(cudaStreamSynchronize(rt.stream));
    return t;
}

// The vectors of one step for imp_lsr_scan, from the layer's workspace.
struct ScanBuffers {
    float *q, *kw, *w = nullptr, *p = nullptr, *z = nullptr, *v, *scal, *o;
    ScanBuffers(Runtime& rt, int64_t T, int64_t H, int64_t D, int64_t Dv, bool decay, bool low_rank) {
        q = rt.arena->take<float>((size_t)(T * H * D));
        kw = rt.arena->take<float>((size_t)(T * H * D));
        if (decay) w = rt.arena->take<float>((size_t)(T * H * D));
        if (low_rank) {
            p = rt.arena->take<float>((size_t)(T * H * D));
            z = rt.arena->take<float>((size_t)(T * H * D));
        }
        v = rt.arena->take<float>((size_t)(T * H * Dv));
        scal = rt.arena->take<float>((size_t)(T * H * 2));
        o = rt.arena->take<float>((size_t)(T * H * Dv));
    }
};

CacheSpec scan_state(int64_t H, int64_t D, int64_t Dv) {
    CacheSpec s;
    s.kind = CacheSpec::State;
    // S in the scan kernel's own layout (whole lanes and column blocks; see csrc/delta_rule.cu)
    s.states.push_back(StateTensorSpec{"S", {imp_gdr_state_floats((int)H, (int)D, (int)Dv)}, F32});
    return s;
}

// ------------------------------------------------------------------------------------------- retention
// Linear attention with a fixed decay per head and neither softmax nor denominator:
//   q, k [H heads of D], v [H heads of Dv] = W x; k times key_scale;  S <- decay_h S + k v^T;  o = S^T q
//   y = o / rms(o) per head (no weight) * silu(W_g x);  out = W_o y.
// Options: an activation on q, k and v (`qkv_act`: "none" | "silu"); the gate's activation (`gate_act`: "silu" | "sigmoid"); the
// read-out normalised per head or over all heads together (`norm_over`: "head" | "row"); a weight on the normalised
// read-out (`out_norm`: a tensor [H * Dv]).
// State per request: S (H heads of D x Dv, float32), zero at the start.
// params: hidden_size, num_heads, key_dim, value_dim, decay (a number per head), key_scale (default key_dim^-1/2), norm_eps,
//         qkv_act, gate_act, norm_over, out_norm.
struct Retention : Mixer {
    int H, D, Dv;
    float eps, k_scale;
    int qkv_act = 0, gate_act = 0;
    bool norm_row = false;
    Tensor w_in, w_o, decay, out_norm{};   // out_norm float32

    struct Sizes {
        int64_t d, H, D, Dv;
    };
    static Sizes sizes(const Json& p) {
        const char* me = "retention";
        Sizes s{need_int(p, "hidden_size", me), need_int(p, "num_heads", me), need_int(p, "key_dim", me), need_int(p, "value_dim", me)};
        if (s.H <= 0 || s.D <= 0 || s.D > 256 || s.Dv <= 0) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": key_dim must lie in (0, 256], heads and value_dim be positive");
        return s;
    }
    static TensorSpecs specs(const Json& p) {
        const Sizes z = sizes(p);
        TensorSpecs s;
        s.emplace_back("q_proj", TensorSpec{{z.H * z.D, z.d}});
        s.emplace_back("k_proj", TensorSpec{{z.H * z.D, z.d}});
        s.emplace_back("v_proj", TensorSpec{{z.H * z.Dv, z.d}});
        s.emplace_back("gate_proj", TensorSpec{{z.H * z.Dv, z.d}});
        if (p.get_bool("out_norm", false)) s.emplace_back("out_norm", TensorSpec{{z.H * z.Dv}, "norm", "one_plus_normal"});
        s.emplace_back("o_proj", TensorSpec{{z.d, z.H * z.Dv}});
        return s;
    }
    static CacheSpec cache(const Json& p) {
        const Sizes z = sizes(p);
        return scan_state(z.H, z.D, z.Dv);
    }
    static int one_of(const Json& p, const char* key, const char* first, const char* second) {
        const std::string v = p.get_string(key, first);
        if (v != first && v != second) fail(IMP_ERROR_INVALID_MODEL, std::string("retention: '") + key + "' is '" + v + "' (known: " + first + ", " + second + ")");
        return v == second ? 1 : 0;
    }
    explicit Retention(BuildArgs& a) {
        const char* me = "retention";
        const Sizes z = sizes(a.params);
        H = (int)z.H, D = (int)z.D, Dv = (int)z.Dv;
        eps = (float)a.params.get_double("norm_eps", 1e-6);
        k_scale = (float)a.params.get_double("key_scale", 1.0 / std::sqrt((double)D));
        const Json* dj = a.params.find("decay");
        if (!dj || !dj->is_array() || (int64_t)dj->size() != z.H) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": 'decay' must list a number per head");
        std::vector<float> dec;
        for (const Json& e : dj->items()) {
            if (!e.is_number()) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": 'decay' must list numbers");
            dec.push_back((float)e.as_double());
        }
        qkv_act = one_of(a.params, "qkv_act", "none", "silu");
        gate_act = one_of(a.params, "gate_act", "silu", "sigmoid");
        norm_row = one_of(a.params, "norm_over", "head", "row") == 1;
        Runtime& rt = *a.rt;
        decay = upload_f32(rt, *a.store, dec);
        w_in = cat_rows_padded(rt, *a.store, {a.tensor("q_proj"), a.tensor("k_proj"), a.tensor("v_proj"), a.tensor("gate_proj")});
        w_o = a.tensor("o_proj");
        if (a.params.get_bool("out_norm", false)) {
            out_norm = to_float32(rt, *a.store, a.tensor("out_norm"));
            IMP_CUDA(cudaStreamSynchronize(rt.stream));
            a.drop("out_norm");
        }
        for (const char* n : {"q_proj", "k_proj", "v_proj", "gate_proj"}) a.drop(n);
    }
    Branch forward(Step& st, Tensor x, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!cache || cache->view.kind != 2 || cache->view.n_states < 1) fail(IMP_ERROR_INTERNAL, "retention runs against a state cache");
        const int64_t T = rows(x);
        Tensor proj = rt.empty(T, rows(w_in));
        linear(rt, proj, x, w_in);
        ScanBuffers b(rt, T, H, D, Dv, false, false);
        rt.launches += 3;
        check_launch(imp_retention_prepare_ex(proj.data, proj.stride0, (int)T, H, D, Dv, k_scale, qkv_act, b.q, b.kw, b.v, b.scal, rt.dtype, rt.stream),
                     "retention_prepare");
        check_launch(imp_lsr_scan(0, b.kw, b.q, nullptr, nullptr, nullptr, b.v, b.scal, (const float*)decay.data, (float*)cache->view.states[0].data, b.o,
                                  st.view.q_start, st.view.state_slots, st.B(), D, H, Dv, rt.stream),
                     "lsr_scan");
        Tensor y = rt.empty(T, (int64_t)H * Dv);
        const Tensor gate = col_slice(proj, (int64_t)2 * H * D + (int64_t)H * Dv, (int64_t)H * Dv);
        const float* wn = out_norm.data ? (const float*)out_norm.data : nullptr;
        if (norm_row)
            check_launch(imp_lsr_output_row(y.data, b.o, gate.data, gate.stride0, wn, gate_act, eps, (int)T, H * Dv, rt.dtype, rt.stream), "lsr_output_row");
        else
            check_launch(imp_gdr_output_ex(y.data, b.o, gate.data, gate.stride0, wn, wn ? Dv : 0, gate_act, eps, (int)T, H, Dv, rt.dtype, rt.stream), "gdr_output");
        return linear(rt, rt.empty(T, rows(w_o)), y, w_o, defer_out);
    }
};

// ------------------------------------------------------------------------------------ generalised delta rule
// r, k, v [H heads of D] = W x;  decay w = exp(-decay_scale * sigmoid(W_2 tanh(W_1 x) + w0)) and removal rate
// a = sigmoid(W_a x + b_a), both per head and key channel;  u = k / sqrt(sum k^2 + unit_eps) per head;
//   S <- diag(w) S - (a u) (u^T S) + k v^T  (both terms read the old state);  o = S^T r
//   y = o / rms(o) per head * w_norm [H * D] * sigmoid(W_g x);  out = W_o y.
// State per request: S (H heads of D x D, float32), zero at the start.
// params: hidden_size, num_heads, head_dim, norm_eps, decay_scale (default exp(-1/2)), unit_eps (default 1e-6),
//         decay_rank (0 or absent: the rows of the checkpoint's W_1).
struct GeneralDelta : Mixer {
    int H, D, rank;
    float eps, decay_scale, unit_eps;
    Tensor w_in, w_2, w_o, w0, a_bias, out_norm;   // the last three float32

    static TensorSpecs specs(const Json& p) {
        const char* me = "general_delta";
        const int64_t d = need_int(p, "hidden_size", me), H = need_int(p, "num_heads", me), D = need_int(p, "head_dim", me),
                      rank = p.get_int("decay_rank", 0);
        if (H <= 0 || D <= 0 || D > 256) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": head_dim must lie in (0, 256] and num_heads be positive");
        TensorSpecs s;
        for (const char* n : {"r_proj", "k_proj", "v_proj", "gate_proj", "a_proj"}) s.emplace_back(n, TensorSpec{{H * D, d}});
        s.emplace_back("a_bias", TensorSpec{{H * D}, "vector", "normal"});
        s.emplace_back("decay_down", TensorSpec{{rank > 0 ? rank : -1, d}});
        s.emplace_back("decay_up", TensorSpec{{H * D, rank > 0 ? rank : -1}});
        s.emplace_back("decay_bias", TensorSpec{{H * D}, "vector", "normal"});
        s.emplace_back("out_norm", TensorSpec{{H * D}, "norm", "one_plus_normal"});
        s.emplace_back("o_proj", TensorSpec{{d, H * D}});
        return s;
    }
    static CacheSpec cache(const Json& p) {
        const char* me = "general_delta";
        const int64_t H = need_int(p, "num_heads", me), D = need_int(p, "head_dim", me);
        return scan_state(H, D, D);
    }
    explicit GeneralDelta(BuildArgs& a) {
        const char* me = "general_delta";
        H = (int)need_int(a.params, "num_heads", me);
        D = (int)need_int(a.params, "head_dim", me);
        eps = (float)a.params.get_double("norm_eps", 1e-6);
        decay_scale = (float)a.params.get_double("decay_scale", std::exp(-0.5));
        unit_eps = (float)a.params.get_double("unit_eps", 1e-6);
        Runtime& rt = *a.rt;
        const Tensor w_1 = a.tensor("decay_down");
        w_2 = a.tensor("decay_up");
        rank = (int)rows(w_1);
        if (rows(w_1) != cols(w_2)) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": the two decay matrices do not share their inner size");
        w_in = cat_rows_padded(rt, *a.store, {a.tensor("r_proj"), a.tensor("k_proj"), a.tensor("v_proj"), a.tensor("gate_proj"), a.tensor("a_proj"), w_1});
        w_o = a.tensor("o_proj");
        w0 = to_float32(rt, *a.store, a.tensor("decay_bias"));
        a_bias = to_float32(rt, *a.store, a.tensor("a_bias"));
        out_norm = to_float32(rt, *a.store, a.tensor("out_norm"));
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        for (const char* n : {"r_proj", "k_proj", "v_proj", "gate_proj", "a_proj", "decay_down", "decay_bias", "a_bias", "out_norm"}) a.drop(n);
    }
    Branch forward(Step& st, Tensor x, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!cache || cache->view.kind != 2 || cache->view.n_states < 1) fail(IMP_ERROR_INTERNAL, "general_delta runs against a state cache");
        const int64_t T = rows(x), HD = (int64_t)H * D;
        Tensor proj = rt.empty(T, rows(w_in));
        linear(rt, proj, x, w_in);
        Tensor low = rt.empty(T, rank);
        rt.launches += 4;
        check_launch(imp_act_rows(low.data, col_slice(proj, 5 * HD, rank).data, proj.stride0, (int)T, rank, 1, rt.dtype, rt.stream), "act_rows");
        Tensor dlog = rt.empty(T, HD, F32);
        linear(rt, dlog, low, w_2);
        ScanBuffers b(rt, T, H, D, D, true, true);
        check_launch(imp_gdelta_prepare(proj.data, proj.stride0, (const float*)dlog.data, (const float*)w0.data, (const float*)a_bias.data, decay_scale,
                                        unit_eps, (int)T, H, D, b.q, b.kw, b.w, b.p, b.z, b.v, b.scal, rt.dtype, rt.stream),
                     "gdelta_prepare");
        check_launch(imp_lsr_scan(2, b.kw, b.q, b.w, b.p, b.z, b.v, b.scal, nullptr, (float*)cache->view.states[0].data, b.o, st.view.q_start,
                                  st.view.state_slots, st.B(), D, H, D, rt.stream),
                     "lsr_scan");
        Tensor y = rt.empty(T, HD);
        const Tensor gate = col_slice(proj, 3 * HD, HD);
        check_launch(imp_gdr_output_ex(y.data, b.o, gate.data, gate.stride0, (const float*)out_norm.data, D, 1, eps, (int)T, H, D, rt.dtype, rt.stream),
                     "gdr_output");
        return linear(rt, rt.empty(T, rows(w_o)), y, w_o, defer_out);
    }
};

// ------------------------------------------------------------------- delta rule with a decay per key channel
// q, k [G heads of D], v [H heads of Dv] = silu(conv(W x)) with a causal convolution of `conv_taps` taps per channel; q, k
// unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times D^(-1/2); head h reads q/k head h / (H / G);
//   beta = sigmoid(W_b x);  g = exp(-exp(A_log[h]) * softplus(W_a2 (W_a1 x) + dt_bias)) per head and key channel
//   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   y = o / rms(o) per head * w_norm [Dv] * sigmoid(W_g2 (W_g1 x));  out = W_o y.
// State per request: S (H heads of D x Dv) and the convolution's last conv_taps - 1 inputs, both float32.
// params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, conv_taps, norm_eps, unit_eps (default 1e-6),
//         decay_rank, gate_rank (0 or absent: the rows of the checkpoint's W_a1 / W_g1).
struct ChannelDeltaRule : Mixer {
    int H, G, D, Dv, taps, ra, rg;
    float eps, unit_eps;
    Tensor w_in, w_a2, w_g2, w_o, conv_w, a_log, dt_bias, out_norm;   // the last four float32

    struct Sizes {
        int64_t d, H, G, D, Dv, taps;
        int64_t channels() const { return 2 * G * D + H * Dv; }
    };
    static Sizes sizes(const Json& p) {
        const char* me = "channel_delta_rule";
        Sizes s{need_int(p, "hidden_size", me), need_int(p, "num_heads", me), need_int(p, "num_kv_heads", me), need_int(p, "key_dim", me),
                need_int(p, "value_dim", me), need_int(p, "conv_taps", me)};
        if (s.G <= 0 || s.H <= 0 || s.H % s.G) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": " + std::to_string(s.H) + " heads over " + std::to_string(s.G) + " key heads");
        if (s.D <= 0 || s.D > 256 || s.Dv <= 0) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": key_dim must lie in (0, 256] and value_dim be positive");
        if (s.taps < 1 || s.taps > 64) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": conv_taps must lie in [1, 64]");
        return s;
    }
    static TensorSpecs specs(const Json& p) {
        const Sizes z = sizes(p);
        const int64_t ra = p.get_int("decay_rank", 0), rg = p.get_int("gate_rank", 0);
        TensorSpecs s;
        s.emplace_back("q_proj", TensorSpec{{z.G * z.D, z.d}});
        s.emplace_back("q_conv", TensorSpec{{z.G * z.D, z.taps}, "vector", "normal"});
        s.emplace_back("k_proj", TensorSpec{{z.G * z.D, z.d}});
        s.emplace_back("k_conv", TensorSpec{{z.G * z.D, z.taps}, "vector", "normal"});
        s.emplace_back("v_proj", TensorSpec{{z.H * z.Dv, z.d}});
        s.emplace_back("v_conv", TensorSpec{{z.H * z.Dv, z.taps}, "vector", "normal"});
        s.emplace_back("beta_proj", TensorSpec{{z.H, z.d}});
        s.emplace_back("a_log", TensorSpec{{z.H}, "vector", "normal"});
        s.emplace_back("out_norm", TensorSpec{{z.Dv}, "norm", "one_plus_normal"});
        s.emplace_back("decay_down", TensorSpec{{ra > 0 ? ra : -1, z.d}});
        s.emplace_back("decay_up", TensorSpec{{z.H * z.D, ra > 0 ? ra : -1}});
        s.emplace_back("dt_bias", TensorSpec{{z.H * z.D}, "vector", "normal"});
        s.emplace_back("gate_down", TensorSpec{{rg > 0 ? rg : -1, z.d}});
        s.emplace_back("gate_up", TensorSpec{{z.H * z.Dv, rg > 0 ? rg : -1}});
        s.emplace_back("o_proj", TensorSpec{{z.d, z.H * z.Dv}});
        return s;
    }
    static CacheSpec cache(const Json& p) {
        const Sizes z = sizes(p);
        CacheSpec s = scan_state(z.H, z.D, z.Dv);
        s.states.push_back(StateTensorSpec{"conv", {std::max<int64_t>(z.taps - 1, 1), z.channels()}, F32});
        return s;
    }
    explicit ChannelDeltaRule(BuildArgs& a) {
        const char* me = "channel_delta_rule";
        const Sizes z = sizes(a.params);
        H = (int)z.H, G = (int)z.G, D = (int)z.D, Dv = (int)z.Dv, taps = (int)z.taps;
        eps = (float)a.params.get_double("norm_eps", 1e-6);
        unit_eps = (float)a.params.get_double("unit_eps", 1e-6);
        Runtime& rt = *a.rt;
        const Tensor a1 = a.tensor("decay_down"), g1 = a.tensor("gate_down");
        w_a2 = a.tensor("decay_up");
        w_g2 = a.tensor("gate_up");
        ra = (int)rows(a1), rg = (int)rows(g1);
        if (rows(a1) != cols(w_a2) || rows(g1) != cols(w_g2)) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": a pair of low-rank matrices does not share its inner size");
        // columns of the input product: q | k | v | beta | decay (low) | gate (low); each low-rank block starts on a multiple of 8
        // columns, so that the second product's input rows stay aligned
        std::vector<Tensor> in = {a.tensor("q_proj"), a.tensor("k_proj"), a.tensor("v_proj"), a.tensor("beta_proj")};
        col_a = z.channels() + z.H;
        std::vector<Tensor> pads;
        auto pad_to8 = [&](int64_t& at) {
            const int64_t pad = (8 - at % 8) % 8;
            if (pad) {
                Tensor zeros = a.store->alloc(in[0].dtype, {pad, z.d});
                IMP_CUDA(cudaMemsetAsync(zeros.data, 0, (size_t)numel(zeros) * elem_size(zeros.dtype), rt.stream));
                in.push_back(zeros);
                pads.push_back(zeros);
                at += pad;
            }
        };
        pad_to8(col_a);
        in.push_back(a1);
        col_g = col_a + ra;
        pad_to8(col_g);
        in.push_back(g1);
        w_in = cat_rows_padded(rt, *a.store, in);
        for (const Tensor& t : pads) a.store->release(t.data);
        w_o = a.tensor("o_proj");
        Tensor cw = cat_rows(rt, *a.store, {a.tensor("q_conv"), a.tensor("k_conv"), a.tensor("v_conv")});
        conv_w = to_float32(rt, *a.store, cw);
        a_log = to_float32(rt, *a.store, a.tensor("a_log"));
        dt_bias = to_float32(rt, *a.store, a.tensor("dt_bias"));
        out_norm = to_float32(rt, *a.store, a.tensor("out_norm"));
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        a.store->release(cw.data);
        for (const char* n : {"q_proj", "k_proj", "v_proj", "beta_proj", "decay_down", "gate_down", "q_conv", "k_conv", "v_conv", "a_log", "dt_bias", "out_norm"})
            a.drop(n);
    }
    int64_t col_a = 0, col_g = 0;

    Branch forward(Step& st, Tensor x, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!cache || cache->view.kind != 2 || cache->view.n_states < 2) fail(IMP_ERROR_INTERNAL, "channel_delta_rule runs against a state cache");
        const int64_t T = rows(x);
        const int C = 2 * G * D + H * Dv;
        Tensor proj = rt.empty(T, rows(w_in));
        linear(rt, proj, x, w_in);
        // the low-rank inputs as dense rows, then their second products: the decay's pre-activation in 32-bit, the gate's as activations
        Tensor low_a = rt.empty(T, ra), low_g = rt.empty(T, rg);
        rt.launches += 6;
        check_launch(imp_act_rows(low_a.data, col_slice(proj, col_a, ra).data, proj.stride0, (int)T, ra, 0, rt.dtype, rt.stream), "act_rows");
        check_launch(imp_act_rows(low_g.data, col_slice(proj, col_g, rg).data, proj.stride0, (int)T, rg, 0, rt.dtype, rt.stream), "act_rows");
        Tensor dpre = rt.empty(T, (int64_t)H * D, F32);
        linear(rt, dpre, low_a, w_a2);
        Tensor gate = rt.empty(T, (int64_t)H * Dv);
        linear(rt, gate, low_g, w_g2);
        ScanBuffers b(rt, T, H, D, Dv, true, false);
        float* S = (float*)cache->view.states[0].data;
        float* conv_state = (float*)cache->view.states[1].data;
        check_launch(imp_gdrc_prepare(proj.data, proj.stride0, (const float*)conv_w.data, taps, conv_state, st.view.seq_of_token, st.view.q_start,
                                      st.view.state_slots, (int)T, st.B(), G, D, H, Dv, (const float*)dpre.data, (const float*)a_log.data,
                                      (const float*)dt_bias.data, unit_eps, b.q, b.kw, b.w, b.v, b.scal, rt.dtype, rt.status, rt.stream),
                     "gdrc_prepare");
        check_launch(imp_gdr_conv_state(proj.data, proj.stride0, conv_state, taps, C, st.view.q_start, st.view.state_slots, st.B(), rt.dtype, rt.stream),
                     "gdr_conv_state");
        check_launch(imp_lsr_scan(1, b.kw, b.q, b.w, nullptr, nullptr, b.v, b.scal, nullptr, S, b.o, st.view.q_start, st.view.state_slots, st.B(), D, H, Dv,
                                  rt.stream),
                     "lsr_scan");
        Tensor y = rt.empty(T, (int64_t)H * Dv);
        check_launch(imp_gdr_output_ex(y.data, b.o, gate.data, gate.stride0, (const float*)out_norm.data, 0, 1, eps, (int)T, H, Dv, rt.dtype, rt.stream),
                     "gdr_output");
        return linear(rt, rt.empty(T, rows(w_o)), y, w_o, defer_out);
    }
};

// ------------------------------------------------------------------------------- attention with gated heads
// Grouped-query softmax attention over the paged cache with, each optional:
//   an RMS norm per head on q and k (one weight [head_dim] each, shared by the heads), before the rotation;
//   a rotation of the first rot_dims entries of every q and k head (pairs i, i + rot_dims/2, angle pos * rot_base^(-2i/rot_dims));
//   values divided by their root mean square per head before they are cached (value_norm);
//   a factor per query head on the scores (head_temp, tensor [heads]);
//   a mask by chunks: a query sees the earlier keys of its own chunk of `chunk` positions, counted from position 0;
//   a sink of score 0 without a value (sink: 1 joins the softmax denominator);
//   a gate per head, sigmoid(W_g x)_h, on the head's output (head_gate).
// Keys have head_dim entries and values value_dim; the cache's head size is the larger of the two, rounded up to a multiple
// of 16, and the rest of a cached row is zero.
// params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim (default head_dim), scale (default head_dim^-1/2), norm_eps,
//         qk_norm, value_norm, rot_dims (0: none), rot_base, head_temp, chunk (0: none), window (0: all), sink, head_gate.
struct GatedHeadAttention : Mixer {
    AttentionGeometry g;     // over the cache's head size
    int D, Dv, rot, chunk;
    bool qk_norm, v_norm, has_temp, has_gate, sink;
    float eps;
    Tensor w_in, w_o, q_norm, k_norm, inv_freq, temp, sink0, sink0_l2;

    struct Sizes {
        int64_t d, H, G, D, Dv, Dc;
    };
    static Sizes sizes(const Json& p) {
        const char* me = "gated_head_attention";
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
        s.emplace_back("q_proj", TensorSpec{{z.H * z.D, z.d}});
        s.emplace_back("k_proj", TensorSpec{{z.G * z.D, z.d}});
        s.emplace_back("v_proj", TensorSpec{{z.G * z.Dv, z.d}});
        if (p.get_bool("qk_norm", false)) {
            s.emplace_back("q_norm", TensorSpec{{z.D}, "norm", "one_plus_normal"});
            s.emplace_back("k_norm", TensorSpec{{z.D}, "norm", "one_plus_normal"});
        }
        if (p.get_bool("head_temp", false)) s.emplace_back("head_temp", TensorSpec{{z.H}, "norm", "one_plus_normal"});
        if (p.get_bool("head_gate", false)) s.emplace_back("gate_proj", TensorSpec{{z.H, z.d}});
        s.emplace_back("o_proj", TensorSpec{{z.d, z.H * z.Dv}});
        return s;
    }
    static CacheSpec cache(const Json& p) {
        const Sizes z = sizes(p);
        return CacheSpec::paged((int)z.G, (int)z.Dc, (int)p.get_int("window", 0));
    }
    explicit GatedHeadAttention(BuildArgs& a) {
        const char* me = "gated_head_attention";
        const Json& p = a.params;
        const Sizes z = sizes(p);
        D = (int)z.D, Dv = (int)z.Dv;
        g.hq = (int)z.H, g.hkv = (int)z.G, g.dh = (int)z.Dc;
        chunk = (int)p.get_int("chunk", 0);
        const int window = (int)p.get_int("window", 0);
        if (chunk < 0 || window < 0 || (chunk > 0 && window > 0)) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": 'chunk' and 'window' are non-negative and exclude each other");
        g.window = chunk > 0 ? -chunk : window;   // a negative window is a chunk size (imp_first_key in csrc/common.cuh)
        const double scale = p.get_double("scale", 0.0);
        g.scale = scale > 0 ? (float)scale : (float)(1.0 / std::sqrt((double)D));
        eps = (float)p.get_double("norm_eps", 1e-6);
        qk_norm = p.get_bool("qk_norm", false);
        v_norm = p.get_bool("value_norm", false);
        has_temp = p.get_bool("head_temp", false);
        has_gate = p.get_bool("head_gate", false);
        sink = p.get_bool("sink", false);
        rot = (int)p.get_int("rot_dims", 0);
        if (rot < 0 || rot % 2 || rot > D) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": rot_dims " + std::to_string(rot) + " must be even and within head_dim " + std::to_string(D));
        Runtime& rt = *a.rt;
        std::vector<Tensor> in = {a.tensor("q_proj"), a.tensor("k_proj"), a.tensor("v_proj")};
        if (has_gate) in.push_back(a.tensor("gate_proj"));
        w_in = cat_rows_padded(rt, *a.store, in);
        w_o = a.tensor("o_proj");
        if (qk_norm) {
            q_norm = to_float32(rt, *a.store, a.tensor("q_norm"));
            k_norm = to_float32(rt, *a.store, a.tensor("k_norm"));
        }
        if (has_temp) temp = to_float32(rt, *a.store, a.tensor("head_temp"));
        if (rot > 0) {
            const double base = p.get_double("rot_base", 10000.0);
            std::vector<float> f((size_t)rot / 2);
            for (int i = 0; i < rot / 2; ++i) f[(size_t)i] = (float)std::pow(base, -2.0 * i / rot);
            inv_freq = upload_f32(rt, *a.store, f);
        }
        if (sink) {
            sink0 = upload_f32(rt, *a.store, std::vector<float>((size_t)g.hq, 0.f));
            sink0_l2 = sink0;   // zero in natural and in base-2 units
        }
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        for (const char* n : {"q_proj", "k_proj", "v_proj"}) a.drop(n);
        if (has_gate) a.drop("gate_proj");
        if (qk_norm) {
            a.drop("q_norm");
            a.drop("k_norm");
        }
        if (has_temp) a.drop("head_temp");
    }
    std::vector<TilingSpec> tilings() const override { return attention_tilings(); }

    Branch forward(Step& st, Tensor x, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!cache || !cache->paged()) fail(IMP_ERROR_INTERNAL, "gated_head_attention runs against a paged cache");
        const int64_t T = rows(x);
        const ImpCacheView& cv = cache->view;
        Tensor proj = rt.empty(T, rows(w_in));
        linear(rt, proj, x, w_in);
        Tensor q = rt.empty(T, (int64_t)g.hq * g.dh);
        ++rt.launches;
        check_launch(imp_qkv_prepare(proj.data, proj.stride0, (int)T, g.hq, g.hkv, D, Dv, g.dh, qk_norm ? (const float*)q_norm.data : nullptr,
                                     qk_norm ? (const float*)k_norm.data : nullptr, eps, v_norm ? 1 : 0, rot > 0 ? (const float*)inv_freq.data : nullptr,
                                     rot, has_temp ? (const float*)temp.data : nullptr, st.view.positions, st.view.seq_of_token, cv.block_table,
                                     cv.bt_stride, st.B(), q.data, q.stride0, cv.writes ? cv.k_pages : nullptr, cv.writes ? cv.v_pages : nullptr,
                                     cv.page_size, cv.num_pages, rt.dtype, rt.status, rt.stream),
                     "qkv_prepare");
        Tensor attn = rt.empty(T, (int64_t)g.hq * g.dh);
        AttentionExtras ex;
        if (sink) {
            ex.sink = (const float*)sink0.data;
            ex.sink_l2 = (const float*)sink0_l2.data;
        }
        paged_attention(st, attn, q, g, *cache, tiling_ids, sink ? &ex : nullptr);
        if (has_gate) {
            ++rt.launches;
            const Tensor gt = col_slice(proj, (int64_t)(g.hq + g.hkv) * D + (int64_t)g.hkv * Dv, g.hq);
            check_launch(imp_head_gate(attn.data, attn.stride0, gt.data, gt.stride0, (int)T, g.hq, g.dh, rt.dtype, rt.stream), "head_gate");
        }
        Tensor y = attn;
        if (g.dh != Dv) {
            // the heads' values without the cache's padding, as dense rows for the output product
            y = rt.empty(T, (int64_t)g.hq * Dv);
            ++rt.launches;
            check_launch(imp_gather_head_cols(y.data, attn.data, (int)T, g.hq, g.dh, Dv, rt.dtype, rt.stream), "gather_head_cols");
        }
        return linear(rt, rt.empty(T, rows(w_o)), y, w_o, defer_out);
    }
};

// ----------------------------------------------------------------------------------------- post-norm block
// x <- norm1(m x + s1 (.) mixer(x));  then, if the layer has a feed-forward, x <- norm2(m x + s2 (.) ffn(x)): the
// normalised sum is the stream, the sublayers read the stream itself, m is a constant and s1, s2 learned factors per
// channel.  With `pair`, two mixers run side by side on the same input and the mixer's result is
// (rms(left) * w_left + rms(right) * w_right) / 2, each output normalised over the width with a weight of its own.
// Slots: mixer_norm, mixer (or left and right with `pair`), and with has_ffn (default true) ffn_norm, feed_forward.
// The norms must be able to store their result as the stream (layernorm).  Tensors: mixer_scale [d], with has_ffn
// ffn_scale [d], with pair left_out [d] and right_out [d].  params: hidden_size, residual_mult (default 1), has_ffn,
// pair, pair_eps.
struct PostNormBlock : Block {
    Mixer *left = nullptr, *right = nullptr;
    FeedForward* ffn = nullptr;
    Norm *norm1, *norm2 = nullptr;
    Tensor s1, s2, w_left, w_right;   // float32
    float mult, pair_eps;
    bool pair;
    explicit PostNormBlock(BuildArgs& a) : norm1(part_cast<Norm>(a.part("mixer_norm"), "a norm")) {
        mult = (float)a.params.get_double("residual_mult", 1.0);
        pair = a.params.get_bool("pair", false);
        pair_eps = (float)a.params.get_double("pair_eps", 1e-6);
        Runtime& rt = *a.rt;
        if (pair) {
            left = part_cast<Mixer>(a.part("left"), "a mixer");
            right = part_cast<Mixer>(a.part("right"), "a mixer");
            w_left = to_float32(rt, *a.store, a.tensor("left_out"));
            w_right = to_float32(rt, *a.store, a.tensor("right_out"));
        } else {
            left = part_cast<Mixer>(a.part("mixer"), "a mixer");
        }
        s1 = to_float32(rt, *a.store, a.tensor("mixer_scale"));
        if (a.params.get_bool("has_ffn", true)) {
            ffn = part_cast<FeedForward>(a.part("feed_forward"), "a feed-forward");
            norm2 = part_cast<Norm>(a.part("ffn_norm"), "a norm");
            s2 = to_float32(rt, *a.store, a.tensor("ffn_scale"));
        }
        if (!norm1->stores_stream() || (norm2 && !norm2->stores_stream()))
            fail(IMP_ERROR_INVALID_MODEL, "postnorm: its norms must be able to store their result as the stream (layernorm)");
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        a.drop("mixer_scale");
        if (ffn) a.drop("ffn_scale");
        if (pair) {
            a.drop("left_out");
            a.drop("right_out");
        }
    }
    static std::vector<Slot> slots(const Json& p) {
        std::vector<Slot> s = {{"mixer_norm", "norm"}};
        if (p.get_bool("pair", false)) {
            s.push_back({"left", "mixer"});
            s.push_back({"right", "mixer"});
        } else {
            s.push_back({"mixer", "mixer"});
        }
        if (p.get_bool("has_ffn", true)) {
            s.push_back({"ffn_norm", "norm"});
            s.push_back({"feed_forward", "feed_forward"});
        }
        return s;
    }
    static TensorSpecs specs(const Json& p) {
        const int64_t d = need_int(p, "hidden_size", "postnorm");
        TensorSpecs s;
        s.emplace_back("mixer_scale", TensorSpec{{d}, "norm", "one_plus_normal"});
        if (p.get_bool("has_ffn", true)) s.emplace_back("ffn_scale", TensorSpec{{d}, "norm", "one_plus_normal"});
        if (p.get_bool("pair", false)) {
            s.emplace_back("left_out", TensorSpec{{d}, "norm", "one_plus_normal"});
            s.emplace_back("right_out", TensorSpec{{d}, "norm", "one_plus_normal"});
        }
        return s;
    }
    Mixer* mixer() const override { return left; }
    std::vector<Mixer*> mixers() const override { return pair ? std::vector<Mixer*>{left, right} : std::vector<Mixer*>{left}; }
    std::vector<Part*> parts() const override {
        std::vector<Part*> p = {norm1, left};
        if (pair) p.push_back(right);
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
    Branch forward(Step& st, Tensor h, const Branch& pending, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!pending.empty()) fail(IMP_ERROR_UNSUPPORTED, "postnorm: the block before it left a branch pending; a post-norm block follows the embedding or another post-norm block");
        // the sublayers read the stream itself: its copy in the activation type, left by the norm that made the stream or made now
        Tensor x = st.stream_copy;
        if (!x.data || rows(x) != rows(h)) {
            x = rt.empty(rows(h), cols(h));
            cast(rt, x, h);
        }
        Tensor m;
        if (pair) {
            if (!cache) fail(IMP_ERROR_INTERNAL, "postnorm: a pair of mixers needs both caches");
            left->defer_out = right->defer_out = false;
            Tensor a = summed(st, left->forward(st, x, cache[0].view.kind ? &cache[0] : nullptr));
            Tensor b = summed(st, right->forward(st, x, cache[1].view.kind ? &cache[1] : nullptr));
            m = rt.empty(rows(a), cols(a));
            ++rt.launches;
            check_launch(imp_rms_pair_mean(m.data, a.data, (const float*)w_left.data, 0.5f, b.data, (const float*)w_right.data, 0.5f, (int)rows(a),
                                           (int)cols(a), pair_eps, m.dtype, rt.stream),
                         "rms_pair_mean");
        } else {
            left->defer_out = false;
            m = summed(st, left->forward(st, x, cache));
        }
        stage(st, "mixer", m);
        Branch bm = Branch::of(m);
        bm.col_scale = (const float*)s1.data;
        x = norm1->add_norm_store(st, h, mult, bm);
        if (ffn) {
            ffn->defer_out = false;
            Branch bf = Branch::of(summed(st, ffn->forward(st, x)));
            stage(st, "feed_forward", bf);
            bf.col_scale = (const float*)s2.data;
            x = norm2->add_norm_store(st, h, mult, bf);
        }
        st.stream_copy = x;
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

void register_recurrent_parts() {
    PartClass ret = class_of<Retention>(&Retention::specs);
    ret.cache_spec = &Retention::cache;
    register_part_class("mixer", "retention", ret, true);
    PartClass gd = class_of<GeneralDelta>(&GeneralDelta::specs);
    gd.cache_spec = &GeneralDelta::cache;
    register_part_class("mixer", "general_delta", gd, true);
    PartClass cd = class_of<ChannelDeltaRule>(&ChannelDeltaRule::specs);
    cd.cache_spec = &ChannelDeltaRule::cache;
    register_part_class("mixer", "channel_delta_rule", cd, true);
    PartClass at = class_of<GatedHeadAttention>(&GatedHeadAttention::specs);
    at.cache_spec = &GatedHeadAttention::cache;
    register_part_class("mixer", "gated_head_attention", at, true);
    PartClass block = class_of<PostNormBlock>(&PostNormBlock::specs);
    block.part_slots = &PostNormBlock::slots;
    register_part_class("block", "postnorm", block, true);
}

}  // namespace imp
