// TEST INFRASTRUCTURE — CPU oracle for the RWKV-7 forward step.  Not part of the product: only the
// test-suite, the smoke check and the benchmark's CPU-baseline leg may load this library.
//
// A restatement, in plain C++ fp32, of the reference's CPU path `src/model.rs` (Rust), function by
// function and in the same operation order.  The reference itself is Rust and cannot be compiled
// here (no cargo/rustc), so this file is pinned against the reference only through the known-answer
// vectors of its own unit tests: int8 unpack (src/model.rs:839-861), constant-group rebuild
// (:863-876), the int8 precision bound (:878-918), the argmax tie rule and the sampler's degenerate
// cases (src/backend_cuda.rs:9276-9396).  The full forward pass has no golden vector in the
// reference (its published logits need a checkpoint that is not available): for that part PARITY IS
// UNPINNED against the reference binary; it is cross-checked against an independent numpy
// restatement (oracle/rwkv7_numpy.py) instead.
//
// Floating-point contract: every product and sum is a separate IEEE fp32 operation in the order the
// Rust code performs them (compile with -ffp-contract=off, no fast-math).  `matvec` keeps the
// reference's [in,out] weight layout and its "skip x[i]==0" rule; threads split the OUTPUT index
// range only, so each y[j] sees the same sequence of additions whatever the thread count.
// One deliberate difference: the reference recomputes LN0 over the whole embedding table on every
// `forward` call (src/model.rs:385-392); here the same LN0 arithmetic is applied to the requested
// row only, which yields the identical bits.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../rwkv-rsv_b200/csrc/safetensors.hpp"

namespace {

constexpr float LN_EPS = 1.0e-5f;   // src/model.rs:6
constexpr float GN_EPS = 64.0e-5f;  // src/model.rs:7
constexpr float L2_EPS = 1.0e-12f;  // src/model.rs:8

thread_local std::string g_err;

using Vec = std::vector<float>;

// ---- src/model.rs:208-217 tensor_to_f32 ----
Vec tensor_to_f32(const rsv::StTensor& t) {
    Vec out((size_t)t.numel());
    if (t.dtype == "F32") {
        memcpy(out.data(), t.data, out.size() * 4);
    } else if (t.dtype == "F16") {
        const uint16_t* h = (const uint16_t*)t.data;
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < (int64_t)out.size(); ++i) out[(size_t)i] = rsv::half_bits_to_float(h[i]);
    } else {
        throw std::runtime_error("unsupported dtype: " + t.dtype);
    }
    return out;
}

// ---- src/model.rs:220-228 transpose: [rows, cols] -> [cols, rows] ----
Vec transpose(const Vec& d, size_t rows, size_t cols) {
    Vec out(d.size());
    constexpr size_t B = 32;
#pragma omp parallel for schedule(static)
    for (int64_t rb = 0; rb < (int64_t)((rows + B - 1) / B); ++rb)
        for (size_t cb = 0; cb < cols; cb += B)
            for (size_t r = (size_t)rb * B; r < std::min(rows, ((size_t)rb + 1) * B); ++r)
                for (size_t c = cb; c < std::min(cols, cb + B); ++c) out[c * rows + r] = d[r * cols + c];
    return out;
}

// ---- src/model.rs:234-252 dequant_int8 ----
void dequant_int8(const uint32_t* idx, const uint32_t* sz, size_t m, size_t k, float* w) {
    const size_t kg = k / 128;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)m; ++r) {
        for (size_t g = 0; g < kg; ++g) {
            uint32_t szv = sz[(size_t)r * kg + g];
            float scale = rsv::half_bits_to_float((uint16_t)(szv & 0xFFFFu));
            float zero = rsv::half_bits_to_float((uint16_t)(szv >> 16));
            for (size_t j = 0; j < 128; ++j) {
                size_t ki = g * 128 + j;
                uint32_t pack = idx[(size_t)r * (k / 4) + ki / 4];
                float q = (float)((pack >> ((ki % 4) * 8)) & 0xFFu);
                w[(size_t)r * k + ki] = scale * q + zero;
            }
        }
    }
}

// ---- src/model.rs:256-273 linear_to_f32: plain key wins, else int8 pair ----
Vec linear_to_f32(const rsv::SafeTensorsFile& st, const std::string& key, size_t m, size_t k) {
    if (st.has(key)) {
        Vec v = tensor_to_f32(st.get(key));
        if (v.size() != m * k) throw std::runtime_error(key + ": shape mismatch");
        return v;
    }
    const auto& it = st.get(key + ".int8_idx");
    const auto& zt = st.get(key + ".int8_sz");
    if (it.nbytes != m * k) throw std::runtime_error(key + ".int8_idx shape mismatch");
    if (zt.nbytes != m * k / 128 * 4) throw std::runtime_error(key + ".int8_sz shape mismatch");
    Vec w(m * k);
    dequant_int8((const uint32_t*)it.data, (const uint32_t*)zt.data, m, k, w.data());
    return w;
}

// ---- src/model.rs:625-635 ----
void layer_norm(const float* x, const float* w, const float* b, size_t n, float eps, float* out) {
    float sum = 0.f;
    for (size_t i = 0; i < n; ++i) sum += x[i];
    float mean = sum / (float)n;
    float sq = 0.f;
    for (size_t i = 0; i < n; ++i) {
        float d = x[i] - mean;
        sq += d * d;
    }
    float var = sq / (float)n + eps;
    float inv_std = 1.0f / std::sqrt(var);
    for (size_t i = 0; i < n; ++i) out[i] = (x[i] - mean) * inv_std * w[i] + b[i];
}

// ---- src/model.rs:654-660 ----
inline void lerp(const float* x, const float* y, const float* w, size_t n, float* out) {
    for (size_t i = 0; i < n; ++i) out[i] = x[i] + w[i] * (y[i] - x[i]);
}
inline float sigmoidf_(float v) { return 1.0f / (1.0f + std::exp(-v)); }  // src/model.rs:662-664

// ---- src/model.rs:700-713 matvec: y = x @ W, W [in,out] row-major, skip zero inputs ----
void matvec(const float* x, const float* w, size_t inp, size_t out, float* y) {
#pragma omp parallel
    {
#ifdef _OPENMP
        int nt = omp_get_num_threads(), t = omp_get_thread_num();
#else
        int nt = 1, t = 0;
#endif
        // split the output range in 16-float aligned slices
        size_t blocks = (out + 15) / 16;
        size_t b0 = blocks * (size_t)t / (size_t)nt, b1 = blocks * (size_t)(t + 1) / (size_t)nt;
        size_t j0 = std::min(out, b0 * 16), j1 = std::min(out, b1 * 16);
        if (j1 > j0) {
            for (size_t j = j0; j < j1; ++j) y[j] = 0.f;
            for (size_t i = 0; i < inp; ++i) {
                float xi = x[i];
                if (xi == 0.0f) continue;
                const float* row = w + i * out;
                for (size_t j = j0; j < j1; ++j) y[j] += xi * row[j];
            }
        }
    }
}

struct Config {
    size_t n_layer, n_embd, vocab, head_size, n_head, ffn_hidden, w_mid, a_mid, v_mid, g_mid;
};

struct Layer {  // src/model.rs:145-187
    Vec ln1_w, ln1_b, x_r, x_w, x_k, x_v, x_a, x_g, w0, a0, v0;
    Vec w1, w2, a1, a2, v1, v2, g1, g2;  // [in,out]
    Vec r_k, k_k, k_a;
    Vec receptance_w, key_w, value_w, output_w;  // [in,out]
    Vec ln_x_w, ln_x_b, ln2_w, ln2_b, ffn_x_k, ffn_key_w, ffn_value_w;
};

struct LayerState {  // src/model.rs:191-205
    Vec tmix_x, tmix_rnn, cmix_x;
};

struct Model {
    Config cfg;
    Vec emb_weight, ln0_w, ln0_b, ln_out_w, ln_out_b, head_weight;  // head [C,vocab]
    std::vector<Layer> layers;
};

struct State {
    std::vector<LayerState> layers;
    Vec v_first;  // last token's layer-0 v (carried only so the exported layout matches State::back)
};

size_t max_layer(const rsv::SafeTensorsFile& st) {  // src/model.rs:520-532
    size_t mx = 0;
    for (auto& kv : st.tensors()) {
        const std::string& k = kv.first;
        if (k.rfind("blocks.", 0) == 0) {
            size_t p = k.find('.', 7);
            if (p != std::string::npos) {
                try {
                    mx = std::max(mx, (size_t)std::stoul(k.substr(7, p - 7)));
                } catch (...) {
                }
            }
        }
    }
    return mx;
}

Layer load_layer(const rsv::SafeTensorsFile& st, size_t idx, const Config& cfg) {  // src/model.rs:534-620
    const size_t c = cfg.n_embd;
    const std::string pre = "blocks." + std::to_string(idx) + ".";
    auto p = [&](const std::string& name) { return tensor_to_f32(st.get(pre + name)); };
    auto lin_t = [&](const std::string& name, size_t out_dim, size_t in_dim) {
        Vec raw = linear_to_f32(st, pre + name + ".weight", out_dim, in_dim);
        return transpose(raw, out_dim, in_dim);
    };
    auto p_lr = [&](const std::string& name, size_t in_dim, size_t out_dim) {  // src/model.rs:564-581
        const auto& t = st.get(pre + "att." + name);
        if (t.shape.size() != 2) throw std::runtime_error(pre + "att." + name + ": expected 2-D");
        Vec data = tensor_to_f32(t);
        if ((size_t)t.shape[0] == in_dim && (size_t)t.shape[1] == out_dim) return data;
        if ((size_t)t.shape[0] == out_dim && (size_t)t.shape[1] == in_dim) return transpose(data, out_dim, in_dim);
        throw std::runtime_error(pre + "att." + name + ": unexpected shape");
    };
    Layer l;
    l.ln1_w = p("ln1.weight");
    l.ln1_b = p("ln1.bias");
    l.x_r = p("att.x_r");
    l.x_w = p("att.x_w");
    l.x_k = p("att.x_k");
    l.x_v = p("att.x_v");
    l.x_a = p("att.x_a");
    l.x_g = p("att.x_g");
    l.w0 = p("att.w0");
    l.a0 = p("att.a0");
    l.v0 = p("att.v0");
    l.w1 = p_lr("w1", c, cfg.w_mid);
    l.w2 = p_lr("w2", cfg.w_mid, c);
    l.a1 = p_lr("a1", c, cfg.a_mid);
    l.a2 = p_lr("a2", cfg.a_mid, c);
    l.v1 = p_lr("v1", c, cfg.v_mid);
    l.v2 = p_lr("v2", cfg.v_mid, c);
    l.g1 = p_lr("g1", c, cfg.g_mid);
    l.g2 = p_lr("g2", cfg.g_mid, c);
    l.r_k = p("att.r_k");
    l.k_k = p("att.k_k");
    l.k_a = p("att.k_a");
    l.receptance_w = lin_t("att.receptance", c, c);
    l.key_w = lin_t("att.key", c, c);
    l.value_w = lin_t("att.value", c, c);
    l.output_w = lin_t("att.output", c, c);
    l.ln_x_w = p("att.ln_x.weight");
    l.ln_x_b = p("att.ln_x.bias");
    l.ln2_w = p("ln2.weight");
    l.ln2_b = p("ln2.bias");
    l.ffn_x_k = p("ffn.x_k");
    l.ffn_key_w = lin_t("ffn.key", cfg.ffn_hidden, c);
    l.ffn_value_w = lin_t("ffn.value", c, cfg.ffn_hidden);
    return l;
}

std::unique_ptr<Model> load_model(const std::string& path) {  // src/model.rs:276-346
    rsv::SafeTensorsFile st(path);
    auto m = std::make_unique<Model>();
    Config& c = m->cfg;
    c.n_layer = 1 + max_layer(st);
    const auto& emb = st.get("emb.weight");
    c.vocab = (size_t)emb.shape.at(0);
    c.n_embd = (size_t)emb.shape.at(1);
    const auto& rk = st.get("blocks.0.att.r_k");
    c.n_head = (size_t)rk.shape.at(0);
    c.head_size = (size_t)rk.shape.at(1);
    auto mid_of = [&](const char* k) {
        const auto& t = st.get(k);
        return (size_t)t.shape.at(0) == c.n_embd ? (size_t)t.shape.at(1) : (size_t)t.shape.at(0);
    };
    c.w_mid = mid_of("blocks.0.att.w1");
    c.a_mid = mid_of("blocks.0.att.a1");
    c.v_mid = mid_of("blocks.0.att.v1");
    c.g_mid = mid_of("blocks.0.att.g1");
    c.ffn_hidden = st.has("blocks.0.ffn.key.weight") ? (size_t)st.get("blocks.0.ffn.key.weight").shape.at(0)
                                                     : (size_t)st.get("blocks.0.ffn.key.weight.int8_idx").shape.at(0);
    m->emb_weight = tensor_to_f32(emb);
    m->ln0_w = tensor_to_f32(st.get("blocks.0.ln0.weight"));
    m->ln0_b = tensor_to_f32(st.get("blocks.0.ln0.bias"));
    m->ln_out_w = tensor_to_f32(st.get("ln_out.weight"));
    m->ln_out_b = tensor_to_f32(st.get("ln_out.bias"));
    m->head_weight = transpose(linear_to_f32(st, "head.weight", c.vocab, c.n_embd), c.vocab, c.n_embd);
    for (size_t i = 0; i < c.n_layer; ++i) m->layers.push_back(load_layer(st, i, c));
    return m;
}

State init_state(const Model& m) {  // src/model.rs:365-371
    State s;
    const Config& c = m.cfg;
    s.layers.resize(c.n_layer);
    for (auto& l : s.layers) {
        l.tmix_x.assign(c.n_embd, 0.f);
        l.tmix_rnn.assign(c.n_head * c.head_size * c.head_size, 0.f);
        l.cmix_x.assign(c.n_embd, 0.f);
    }
    s.v_first.assign(c.n_embd, 0.f);
    return s;
}

// ---- src/model.rs:374-517 forward, one token ----
void forward_token(const Model& M, State& st, uint32_t token, float* logits, float* hidden = nullptr) {
    const Config& cf = M.cfg;
    const size_t c = cf.n_embd, h = cf.n_head, n = cf.head_size;
    const size_t wm = cf.w_mid, am = cf.a_mid, vm = cf.v_mid, gm = cf.g_mid, fh = cf.ffn_hidden;
    if (token >= cf.vocab) throw std::runtime_error("token id out of range");
    Vec x(c);
    layer_norm(&M.emb_weight[(size_t)token * c], M.ln0_w.data(), M.ln0_b.data(), c, LN_EPS, x.data());
    Vec v_first;
    bool have_v_first = false;
    Vec ln1(c), xr(c), xw(c), xk(c), xv(c), xa(c), xg(c), r(c), k(c), v(c), w(c), a(c), kk(c), k_mod(c), kk_l2(c), b_vec(c), y(c), g(c), y_g(c),
        y_out(c), ln2(c), xb(c), r2(fh), v2(c), full(c);
    Vec mid(std::max(std::max(wm, am), std::max(vm, gm)));
    for (size_t i = 0; i < cf.n_layer; ++i) {
        const Layer& L = M.layers[i];
        LayerState& S = st.layers[i];
        // ===== time mixing =====
        layer_norm(x.data(), L.ln1_w.data(), L.ln1_b.data(), c, LN_EPS, ln1.data());
        Vec prev = S.tmix_x;
        S.tmix_x = ln1;
        lerp(ln1.data(), prev.data(), L.x_r.data(), c, xr.data());
        lerp(ln1.data(), prev.data(), L.x_w.data(), c, xw.data());
        lerp(ln1.data(), prev.data(), L.x_k.data(), c, xk.data());
        lerp(ln1.data(), prev.data(), L.x_v.data(), c, xv.data());
        lerp(ln1.data(), prev.data(), L.x_a.data(), c, xa.data());
        lerp(ln1.data(), prev.data(), L.x_g.data(), c, xg.data());
        matvec(xr.data(), L.receptance_w.data(), c, c, r.data());
        matvec(xk.data(), L.key_w.data(), c, c, k.data());
        matvec(xv.data(), L.value_w.data(), c, c, v.data());
        if (!have_v_first) {
            v_first = v;
            have_v_first = true;
        } else {
            matvec(xv.data(), L.v1.data(), c, vm, mid.data());
            matvec(mid.data(), L.v2.data(), vm, c, full.data());
            for (size_t j = 0; j < c; ++j) {
                float gate = sigmoidf_(full[j] + L.v0[j]);
                v[j] = v[j] + gate * (v_first[j] - v[j]);
            }
        }
        // w = exp(-sigmoid(w0 + tanh(xw@w1)@w2) / sqrt(e))
        matvec(xw.data(), L.w1.data(), c, wm, mid.data());
        for (size_t j = 0; j < wm; ++j) mid[j] = std::tanh(mid[j]);
        matvec(mid.data(), L.w2.data(), wm, c, full.data());
        const float wscale = -1.0f / std::sqrt(2.71828182845904523536f);  // -1/sqrt(f32 E)
        for (size_t j = 0; j < c; ++j) w[j] = std::exp(sigmoidf_(full[j] + L.w0[j]) * wscale);
        // a = sigmoid(a0 + xa@a1@a2)
        matvec(xa.data(), L.a1.data(), c, am, mid.data());
        matvec(mid.data(), L.a2.data(), am, c, full.data());
        for (size_t j = 0; j < c; ++j) a[j] = sigmoidf_(full[j] + L.a0[j]);
        for (size_t j = 0; j < c; ++j) kk[j] = k[j] * L.k_k[j];
        for (size_t j = 0; j < c; ++j) {
            float ka = k[j] * a[j];
            k_mod[j] = k[j] + L.k_a[j] * (ka - k[j]);
        }
        // src/model.rs:716-727 l2_norm_groups
        for (size_t hi = 0; hi < h; ++hi) {
            float ss = 0.f;
            for (size_t j = 0; j < n; ++j) ss += kk[hi * n + j] * kk[hi * n + j];
            float norm = std::max(std::sqrt(ss), L2_EPS);
            float inv = 1.0f / norm;
            for (size_t j = 0; j < n; ++j) kk_l2[hi * n + j] = kk[hi * n + j] * inv;
        }
        for (size_t j = 0; j < c; ++j) b_vec[j] = kk_l2[j] * (-a[j]);
        // src/model.rs:732-766 dplr_update, :769-782 dplr_matvec
        for (size_t hi = 0; hi < h; ++hi) {
            float* s = &S.tmix_rnn[hi * n * n];
            const float *wh = &w[hi * n], *kh = &k_mod[hi * n], *vh = &v[hi * n], *ah = &kk_l2[hi * n], *bh = &b_vec[hi * n], *rh = &r[hi * n];
            std::vector<float> sa(n, 0.f);
            for (size_t ii = 0; ii < n; ++ii)
                for (size_t j = 0; j < n; ++j) sa[ii] += s[ii * n + j] * ah[j];
            for (size_t ii = 0; ii < n; ++ii)
                for (size_t j = 0; j < n; ++j) s[ii * n + j] = s[ii * n + j] * wh[j] + sa[ii] * bh[j] + vh[ii] * kh[j];
            for (size_t ii = 0; ii < n; ++ii) {
                float acc = 0.f;
                for (size_t j = 0; j < n; ++j) acc += s[ii * n + j] * rh[j];
                y[hi * n + ii] = acc;
            }
        }
        // src/model.rs:785-797 group_norm, :801-826 sum_rk_rk
        for (size_t hi = 0; hi < h; ++hi) {
            float* grp = &y[hi * n];
            float sum = 0.f;
            for (size_t j = 0; j < n; ++j) sum += grp[j];
            float mean = sum / (float)n;
            float sq = 0.f;
            for (size_t j = 0; j < n; ++j) sq += (grp[j] - mean) * (grp[j] - mean);
            float var = sq / (float)n + GN_EPS;
            float inv_std = 1.0f / std::sqrt(var);
            float srk = 0.f;
            for (size_t j = 0; j < n; ++j) srk += r[hi * n + j] * k_mod[hi * n + j] * L.r_k[hi * n + j];
            for (size_t j = 0; j < n; ++j) {
                float gn = (grp[j] - mean) * inv_std * L.ln_x_w[hi * n + j] + L.ln_x_b[hi * n + j];
                grp[j] = gn + srk * v[hi * n + j];
            }
        }
        // g = sigmoid(xg@g1)@g2
        matvec(xg.data(), L.g1.data(), c, gm, mid.data());
        for (size_t j = 0; j < gm; ++j) mid[j] = sigmoidf_(mid[j]);
        matvec(mid.data(), L.g2.data(), gm, c, g.data());
        for (size_t j = 0; j < c; ++j) y_g[j] = y[j] * g[j];
        matvec(y_g.data(), L.output_w.data(), c, c, y_out.data());
        for (size_t j = 0; j < c; ++j) x[j] = x[j] + y_out[j];
        // ===== channel mixing =====
        layer_norm(x.data(), L.ln2_w.data(), L.ln2_b.data(), c, LN_EPS, ln2.data());
        Vec prev_c = S.cmix_x;
        S.cmix_x = ln2;
        lerp(ln2.data(), prev_c.data(), L.ffn_x_k.data(), c, xb.data());
        matvec(xb.data(), L.ffn_key_w.data(), c, fh, r2.data());
        for (size_t j = 0; j < fh; ++j) {
            float m = std::max(r2[j], 0.0f);
            r2[j] = m * m;
        }
        matvec(r2.data(), L.ffn_value_w.data(), fh, c, v2.data());
        for (size_t j = 0; j < c; ++j) x[j] = x[j] + v2[j];
    }
    st.v_first = v_first;
    if (hidden) memcpy(hidden, x.data(), c * 4);  // the last layer's residual stream, before ln_out
    if (logits) {
        Vec xn(c);
        layer_norm(x.data(), M.ln_out_w.data(), M.ln_out_b.data(), c, LN_EPS, xn.data());
        matvec(xn.data(), M.head_weight.data(), c, cf.vocab, logits);
    }
}

// ---- sampler: src/backend_cuda.rs:3690-4009.  No CPU sampler exists in the reference; this follows
// the kernel's general ("fallback") path step by step, including the order of its block reductions
// (112 strided partial sums, fold 64+48, then a power-of-two tree).  The kernel's 1<=top_k<=50 fast
// path accumulates top-p and the draw from the SMALLEST kept probability, against the documented
// intent (src/gpu_model.rs:3889); that branch is deliberately not restated: every top_k takes the
// general path here. ----
inline float u01(uint32_t s) {  // src/backend_cuda.rs:3691-3698
    s += 0x9E3779B9u;
    uint32_t z = s;
    z = (z ^ (z >> 16)) * 0x85EBCA6Bu;
    z = (z ^ (z >> 13)) * 0xC2B2AE35u;
    z ^= z >> 16;
    return (float)z / 4294967296.0f;
}
constexpr int BS = 112;
float block_sum(const float* t, int n) {
    float s[BS];
    for (int tid = 0; tid < BS; ++tid) {
        float a = 0.f;
        for (int i = tid; i < n; i += BS) a += t[i];
        s[tid] = a;
    }
    for (int tid = 64; tid < BS; ++tid) s[tid - 64] += s[tid];
    for (int step = 32; step > 0; step >>= 1)
        for (int tid = 0; tid < step; ++tid) s[tid] += s[tid + step];
    return s[0];
}
// arg-max over unmasked entries; ties -> smaller index (src/backend_cuda.rs:3842-3858)
int masked_argmax(const float* t, const std::vector<uint8_t>& mask, int n, float* val) {
    float lm = -1e30f;
    int li = 0;
    for (int i = 0; i < n; ++i)
        if (!mask[(size_t)i] && t[i] > lm) {
            lm = t[i];
            li = i;
        }
    *val = lm;
    return li;
}
uint32_t sample(const float* logits, int n, const float* sp, const uint32_t* hist) {
    auto bits = [](float f) {
        uint32_t u;
        memcpy(&u, &f, 4);
        return u;
    };
    const float temperature = sp[0];
    const uint32_t top_k = bits(sp[1]);
    const float top_p = sp[2];
    const uint32_t seed = bits(sp[3]);
    const float rep = sp[4], freq = sp[5], pres = sp[6];
    const uint32_t hist_len = bits(sp[7]);
    const bool do_topk = top_k > 0u && top_k < (uint32_t)n;
    Vec temp(logits, logits + n);
    if (hist_len > 0u && (rep != 1.0f || freq != 0.0f || pres != 0.0f)) {
        std::vector<uint32_t> counter((size_t)n, 0u);
        for (uint32_t hh = 0; hh < hist_len; ++hh) counter[hist[hh]] += 1u;
        for (int i = 0; i < n; ++i) {
            uint32_t cnt = counter[(size_t)i];
            float l = temp[(size_t)i];
            if (cnt > 0u) {
                if (rep != 1.0f) l = l > 0.0f ? l / rep : l * rep;
                if (pres != 0.0f) l -= pres;
            }
            if (freq != 0.0f) l -= freq * (float)cnt;
            temp[(size_t)i] = l;
        }
    }
    float invT = 1.0f / temperature;
    if (!(temperature > 0.0f)) invT = 1.0f;
    for (int i = 0; i < n; ++i) temp[(size_t)i] *= invT;
    std::vector<uint8_t> mask((size_t)n, 0);
    if (do_topk) {
        float thr = -1e30f;
        for (uint32_t round = 0; round < top_k; ++round) {
            float v;
            int li = masked_argmax(temp.data(), mask, n, &v);
            thr = v;
            mask[(size_t)li] = 1;
        }
        for (int i = 0; i < n; ++i)
            if (temp[(size_t)i] < thr) temp[(size_t)i] = -1e30f;
    }
    float m = -1e30f;
    for (int i = 0; i < n; ++i) m = std::max(m, temp[(size_t)i]);
    for (int i = 0; i < n; ++i) temp[(size_t)i] = std::exp(temp[(size_t)i] - m);
    float total = block_sum(temp.data(), n);
    if (total > 0.0f)
        for (int i = 0; i < n; ++i) temp[(size_t)i] /= total;
    if (top_p > 0.0f && top_p < 1.0f) {
        std::fill(mask.begin(), mask.end(), 0);
        float cutoff = 0.0f, cum = 0.0f;
        for (int cnt = 0; cnt < 512 && cum < top_p; ++cnt) {
            float v;
            int li = masked_argmax(temp.data(), mask, n, &v);
            mask[(size_t)li] = 1;
            cum += v;
            cutoff = v;
        }
        for (int i = 0; i < n; ++i)
            if (temp[(size_t)i] < cutoff) temp[(size_t)i] = 0.0f;
    }
    float tot2 = block_sum(temp.data(), n);
    float u = u01(seed) * tot2;
    float acc = 0.0f;
    int chosen = n - 1;
    for (int i = 0; i < n; ++i) {
        acc += temp[(size_t)i];
        if (acc > u) {
            chosen = i;
            break;
        }
    }
    return (uint32_t)chosen;
}

}  // namespace

extern "C" {

const char* orc_last_error(void) { return g_err.c_str(); }

void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void* orc_model_load(const char* path) {
    try {
        return load_model(path).release();
    } catch (const std::exception& e) {
        g_err = e.what();
        return nullptr;
    }
}
void orc_model_free(void* m) { delete (Model*)m; }
// out: n_layer, n_embd, vocab, head_size, n_head, ffn_hidden, w_mid, a_mid, v_mid, g_mid
void orc_model_info(void* m, int64_t* out) {
    const Config& c = ((Model*)m)->cfg;
    size_t v[10] = {c.n_layer, c.n_embd, c.vocab, c.head_size, c.n_head, c.ffn_hidden, c.w_mid, c.a_mid, c.v_mid, c.g_mid};
    for (int i = 0; i < 10; ++i) out[i] = (int64_t)v[i];
}
void* orc_state_new(void* m) { return new State(init_state(*(Model*)m)); }
void orc_state_free(void* s) { delete (State*)s; }
void orc_state_reset(void* m, void* s) { *(State*)s = init_state(*(Model*)m); }
// Same flat layout as the reference's State::back (src/gpu_model.rs:3972-3990):
// per layer tmix_x[C] | tmix_rnn[H*N*N] | cmix_x[C], then v_first[C].
int64_t orc_state_len(void* m) {
    const Config& c = ((Model*)m)->cfg;
    return (int64_t)(c.n_layer * (2 * c.n_embd + c.n_head * c.head_size * c.head_size) + c.n_embd);
}
void orc_state_export(void* s_, float* out) {
    State* s = (State*)s_;
    for (auto& l : s->layers) {
        out = std::copy(l.tmix_x.begin(), l.tmix_x.end(), out);
        out = std::copy(l.tmix_rnn.begin(), l.tmix_rnn.end(), out);
        out = std::copy(l.cmix_x.begin(), l.cmix_x.end(), out);
    }
    std::copy(s->v_first.begin(), s->v_first.end(), out);
}
void orc_state_import(void* s_, const float* in) {
    State* s = (State*)s_;
    for (auto& l : s->layers) {
        std::copy(in, in + l.tmix_x.size(), l.tmix_x.begin());
        in += l.tmix_x.size();
        std::copy(in, in + l.tmix_rnn.size(), l.tmix_rnn.begin());
        in += l.tmix_rnn.size();
        std::copy(in, in + l.cmix_x.size(), l.cmix_x.begin());
        in += l.cmix_x.size();
    }
    std::copy(in, in + s->v_first.size(), s->v_first.begin());
}
// Model::forward (src/model.rs:374-517): runs every token, returns the last token's logits in
// `logits_last` [V]; if `logits_all` is non-null it also receives every position's logits [n,V].
int orc_forward(void* m, void* s, const uint32_t* tokens, int64_t n, float* logits_last, float* logits_all) {
    try {
        const Model& M = *(Model*)m;
        const size_t V = M.cfg.vocab;
        Vec tmp(V);
        for (int64_t t = 0; t < n; ++t) {
            bool want = logits_all || (t == n - 1 && logits_last);
            float* dst = logits_all ? logits_all + (size_t)t * V : tmp.data();
            forward_token(M, *(State*)s, tokens[t], want ? dst : nullptr);
            if (t == n - 1 && logits_last) memcpy(logits_last, dst, V * 4);
        }
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}
void orc_dequant_int8(const uint32_t* idx, const uint32_t* sz, int64_t m, int64_t k, float* out) { dequant_int8(idx, sz, (size_t)m, (size_t)k, out); }
// The WKV-7 step of one layer on its own, for one session over T tokens: the same statements, in the same order, as the time-mixing
// block of forward() above - v lerp (src/model.rs:418-434), kk / k~ / b (:445-460), l2_norm_groups (:716-727), dplr_update (:732-766),
// dplr_matvec (:769-782), group_norm (:785-797), sum_rk_rk (:801-826), gate.  Rows are [T, H*64]; vgate / vfirst may be null
// (first layer); state [H, 64, 64] is updated in place; y [T, H*64].
int orc_wkv7(int64_t H, int64_t T, const float* r, const float* k, const float* v_in, const float* w, const float* a, const float* g, const float* vgate,
             const float* vfirst, const float* k_k, const float* k_a, const float* r_k, const float* lnx_w, const float* lnx_b, float* state, float* y_out) {
    const size_t n = 64, h = (size_t)H, c = h * n;
    std::vector<float> v(c), kk(c), k_mod(c), kk_l2(c), b_vec(c), y(c), sa(n);
    for (int64_t t = 0; t < T; ++t) {
        const float *rt = r + t * c, *kt = k + t * c, *wt = w + t * c, *at = a + t * c, *gt = g + t * c;
        for (size_t j = 0; j < c; ++j) {
            const float vj = v_in[t * c + j];
            v[j] = vgate ? vj + vgate[t * c + j] * (vfirst[t * c + j] - vj) : vj;
        }
        for (size_t j = 0; j < c; ++j) kk[j] = kt[j] * k_k[j];
        for (size_t j = 0; j < c; ++j) {
            float ka = kt[j] * at[j];
            k_mod[j] = kt[j] + k_a[j] * (ka - kt[j]);
        }
        for (size_t hi = 0; hi < h; ++hi) {
            float ss = 0.f;
            for (size_t j = 0; j < n; ++j) ss += kk[hi * n + j] * kk[hi * n + j];
            float norm = std::max(std::sqrt(ss), L2_EPS);
            float inv = 1.0f / norm;
            for (size_t j = 0; j < n; ++j) kk_l2[hi * n + j] = kk[hi * n + j] * inv;
        }
        for (size_t j = 0; j < c; ++j) b_vec[j] = kk_l2[j] * (-at[j]);
        for (size_t hi = 0; hi < h; ++hi) {
            float* s = state + hi * n * n;
            const float *wh = &wt[hi * n], *kh = &k_mod[hi * n], *vh = &v[hi * n], *ah = &kk_l2[hi * n], *bh = &b_vec[hi * n], *rh = &rt[hi * n];
            std::fill(sa.begin(), sa.end(), 0.f);
            for (size_t ii = 0; ii < n; ++ii)
                for (size_t j = 0; j < n; ++j) sa[ii] += s[ii * n + j] * ah[j];
            for (size_t ii = 0; ii < n; ++ii)
                for (size_t j = 0; j < n; ++j) s[ii * n + j] = s[ii * n + j] * wh[j] + sa[ii] * bh[j] + vh[ii] * kh[j];
            for (size_t ii = 0; ii < n; ++ii) {
                float acc = 0.f;
                for (size_t j = 0; j < n; ++j) acc += s[ii * n + j] * rh[j];
                y[hi * n + ii] = acc;
            }
        }
        for (size_t hi = 0; hi < h; ++hi) {
            float* grp = &y[hi * n];
            float sum = 0.f;
            for (size_t j = 0; j < n; ++j) sum += grp[j];
            float mean = sum / (float)n;
            float sq = 0.f;
            for (size_t j = 0; j < n; ++j) sq += (grp[j] - mean) * (grp[j] - mean);
            float var = sq / (float)n + GN_EPS;
            float inv_std = 1.0f / std::sqrt(var);
            float srk = 0.f;
            for (size_t j = 0; j < n; ++j) srk += rt[hi * n + j] * k_mod[hi * n + j] * r_k[hi * n + j];
            for (size_t j = 0; j < n; ++j) {
                float gn = (grp[j] - mean) * inv_std * lnx_w[hi * n + j] + lnx_b[hi * n + j];
                grp[j] = gn + srk * v[hi * n + j];
            }
        }
        for (size_t j = 0; j < c; ++j) y_out[t * c + j] = y[j] * gt[j];
    }
    return 0;
}

// Mean over a prompt's tokens of the last layer's residual stream x (before ln_out), from a zero state: the router feature of
// forward_seq_batch_mean_hidden (src/gpu_model.rs:1013-1036), accumulated token by token like rwkv_segmean
// (src/backend_cuda.rs:4412-4431: acc += x[t] in token order, then acc / len).  out [n_embd].
int orc_mean_hidden(void* m, void* s, const uint32_t* tokens, int64_t n, float* out) {
    try {
        const Model& M = *(Model*)m;
        const size_t c = M.cfg.n_embd;
        Vec hid(c), acc(c, 0.f);
        for (int64_t t = 0; t < n; ++t) {
            forward_token(M, *(State*)s, tokens[t], nullptr, hid.data());
            for (size_t j = 0; j < c; ++j) acc[j] += hid[j];
        }
        for (size_t j = 0; j < c; ++j) out[j] = acc[j] / (float)n;
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}
// arg-max with ties -> smaller index (src/backend_cuda.rs:3640-3680)
uint32_t orc_argmax(const float* logits, int64_t n) {
    float lm = -1e30f;
    int64_t li = 0;
    for (int64_t i = 0; i < n; ++i)
        if (logits[i] > lm) {
            lm = logits[i];
            li = i;
        }
    return (uint32_t)li;
}
uint32_t orc_sample(const float* logits, int64_t n, const float* sampler8, const uint32_t* hist) { return sample(logits, (int)n, sampler8, hist); }
float orc_u01(uint32_t s) { return u01(s); }

}  // extern "C"
