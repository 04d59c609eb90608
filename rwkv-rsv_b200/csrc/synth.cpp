// Seeded synthetic RWKV-7 (x070) checkpoint writer.
//
// Emits a safetensors file with exactly the tensor names, shapes and dtypes the reference loaders
// read (src/model.rs:276-346, 534-620; src/gpu_model.rs:401-546, 3258-3568): hyper-parameters are
// carried only by the shapes.  Values follow the benchmark configurations: all matrices N(0, 0.02)
// stored as fp16; att.w0 ~ U(-6,-1); norm weights 1+N(0,0.02), norm biases N(0,0.02); token-shift
// mixes and att.k_a ~ U(0,1); att.k_k ~ U(0.5,1.5); att.a0, att.v0, att.r_k ~ N(0,0.02).
//
// int8 variants use the reference's container (tools/quantize_any4.py:241-300, decoded by
// src/model.rs:234-252): `{key}.int8_idx` U8 [M,K] and `{key}.int8_sz` U32 [M,K/128] holding
// fp16(scale) in the low half and fp16(zero) in the high half, w = scale*q + zero.
//   quant=1: symmetric per-output-row absmax.  s = fp16(absmax/127), q_s8 = clip(rint(w/s),-127,127),
//            stored as q_u8 = q_s8+128 with zero = fp16(-128*s) replicated over the row's groups, so
//            the container's fp32 dequant scale*q_u8+zero equals s*q_s8 exactly.
//   quant=2: the reference quantizer's own rule: per (row, group of 128) zero=min, scale=(max-min)/255,
//            q = clip(rint((w-zero)/scale),0,255), constant group -> scale 0.
// Every value is a pure function of (seed, tensor name, element index), so generation is
// order-independent and parallel.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "safetensors.hpp"
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

thread_local std::string g_err;

inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
inline uint64_t fnv1a(const std::string& s) {
    uint64_t h = 0xcbf29ce484222325ull;
    for (unsigned char c : s) {
        h ^= c;
        h *= 0x100000001b3ull;
    }
    return h;
}

struct Stream {
    uint64_t key;
    Stream(uint64_t seed, const std::string& name) : key(splitmix64(seed ^ (fnv1a(name) * 0x9E3779B97F4A7C15ull))) {}
    inline uint64_t bits(uint64_t idx) const { return splitmix64(key + idx * 0xD1342543DE82EF95ull); }
    // uniform in (0,1), 53-bit
    inline double uniform(uint64_t idx) const { return ((double)(bits(idx) >> 11) + 0.5) * (1.0 / 9007199254740992.0); }
    // standard normal; elements 2j and 2j+1 share one Box-Muller pair
    inline double normal(uint64_t idx) const {
        uint64_t j = idx >> 1;
        uint64_t z = bits(j);
        double u1 = ((double)(z >> 32) + 0.5) * (1.0 / 4294967296.0);
        double u2 = ((double)(z & 0xFFFFFFFFull) + 0.5) * (1.0 / 4294967296.0);
        double r = std::sqrt(-2.0 * std::log(u1));
        double a = 6.283185307179586476925286766559 * u2;
        return (idx & 1) ? r * std::sin(a) : r * std::cos(a);
    }
};

enum Dist { NORMAL, UNIFORM };
struct Spec {
    Dist dist;
    double a, b;  // NORMAL: mean a, std b.  UNIFORM: [a, b)
};

struct Entry {
    std::string name, dtype;
    std::vector<int64_t> shape;
    std::vector<uint8_t> bytes;
};

void fill_f16(std::vector<uint16_t>& out, const Stream& st, const Spec& sp, int64_t n) {
    out.resize((size_t)n);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        double v = sp.dist == NORMAL ? sp.a + sp.b * st.normal((uint64_t)i) : sp.a + (sp.b - sp.a) * st.uniform((uint64_t)i);
        out[(size_t)i] = rsv::float_to_half_bits((float)v);
    }
}

// Two-pass writer: pass 0 only records (name, dtype, shape, size) so that the header can be written
// first; pass 1 streams the tensor bytes straight behind it.
struct Writer {
    FILE* f = nullptr;
    int pass = 0;
    std::vector<Entry> entries;
    std::vector<std::pair<uint64_t, uint64_t>> offs;
    uint64_t cur = 0;

    bool dry() const { return pass == 0; }
    bool add(const std::string& name, const std::string& dtype, std::vector<int64_t> shape, const void* data, size_t nbytes) {
        if (pass == 0) {
            Entry e;
            e.name = name;
            e.dtype = dtype;
            e.shape = std::move(shape);
            entries.push_back(std::move(e));
            offs.emplace_back(cur, cur + nbytes);
            cur += nbytes;
            return true;
        }
        return fwrite(data, 1, nbytes, f) == nbytes;
    }
    bool begin_data(const std::string& path, const std::string& meta_json) {
        std::string h = "{\"__metadata__\":" + meta_json;
        for (size_t i = 0; i < entries.size(); ++i) {
            h += ",\"" + entries[i].name + "\":{\"dtype\":\"" + entries[i].dtype + "\",\"shape\":[";
            for (size_t d = 0; d < entries[i].shape.size(); ++d) {
                if (d) h += ",";
                h += std::to_string(entries[i].shape[d]);
            }
            h += "],\"data_offsets\":[" + std::to_string(offs[i].first) + "," + std::to_string(offs[i].second) + "]}";
        }
        h += "}";
        while (h.size() % 8) h += ' ';
        f = fopen(path.c_str(), "wb");
        if (!f) return false;
        uint64_t hl = h.size();
        pass = 1;
        return fwrite(&hl, 8, 1, f) == 1 && fwrite(h.data(), 1, h.size(), f) == h.size();
    }
    bool finish() {
        bool ok = f && fclose(f) == 0;
        f = nullptr;
        return ok;
    }
};

// Quantise an fp16 [M,K] matrix into the reference container.
void quantize(const std::vector<uint16_t>& w16, int64_t M, int64_t K, int mode, std::vector<uint8_t>& idx, std::vector<uint32_t>& sz) {
    const int64_t KG = K / 128;
    idx.resize((size_t)(M * K));
    sz.resize((size_t)(M * KG));
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        const uint16_t* row = &w16[(size_t)(m * K)];
        if (mode == 1) {
            float amax = 0.f;
            for (int64_t k = 0; k < K; ++k) amax = std::max(amax, std::fabs(rsv::half_bits_to_float(row[k])));
            uint16_t s16 = rsv::float_to_half_bits(amax / 127.0f);
            float s = rsv::half_bits_to_float(s16);
            uint16_t z16 = rsv::float_to_half_bits(-128.0f * s);
            for (int64_t k = 0; k < K; ++k) {
                float q = s > 0.f ? std::nearbyintf(rsv::half_bits_to_float(row[k]) / s) : 0.f;  // round half to even
                q = std::min(127.f, std::max(-127.f, q));
                idx[(size_t)(m * K + k)] = (uint8_t)((int)q + 128);
            }
            for (int64_t g = 0; g < KG; ++g) sz[(size_t)(m * KG + g)] = ((uint32_t)z16 << 16) | s16;
        } else {
            for (int64_t g = 0; g < KG; ++g) {
                float mn = INFINITY, mx = -INFINITY;
                for (int j = 0; j < 128; ++j) {
                    float v = rsv::half_bits_to_float(row[g * 128 + j]);
                    mn = std::min(mn, v);
                    mx = std::max(mx, v);
                }
                float span = mx - mn;
                bool constant = span == 0.f;
                float scale = (constant ? 1.0f : span) / 255.0f;
                float safe = constant ? 1.0f : scale;
                for (int j = 0; j < 128; ++j) {
                    float v = rsv::half_bits_to_float(row[g * 128 + j]);
                    float q = std::nearbyintf((v - mn) / safe);
                    q = std::min(255.f, std::max(0.f, q));
                    idx[(size_t)(m * K + g * 128 + j)] = (uint8_t)q;
                }
                uint16_t s16 = rsv::float_to_half_bits(constant ? 0.f : scale);
                uint16_t z16 = rsv::float_to_half_bits(mn);
                sz[(size_t)(m * KG + g)] = ((uint32_t)z16 << 16) | s16;
            }
        }
    }
}

}  // namespace

extern "C" {

typedef struct {
    int32_t n_layer, n_embd, n_head, head_size, ffn_hidden, vocab;
    int32_t w_mid, a_mid, v_mid, g_mid;
} rsv_synth_shape;

// flags: bit0 = store low-rank pairs transposed ([mid,C] / [C,mid]); bit1 = quantise head.weight too.
int rsv_synth_write(const char* path, const rsv_synth_shape* s, uint64_t seed, int quant, int flags) {
    try {
        if (!path || !s) throw std::runtime_error("null argument");
        const int64_t L = s->n_layer, C = s->n_embd, H = s->n_head, N = s->head_size, F = s->ffn_hidden, V = s->vocab;
        if (L < 1 || C < 1 || H < 1 || N < 1 || F < 1 || V < 1 || H * N != C) throw std::runtime_error("bad shape (need n_head*head_size == n_embd)");
        if (quant < 0 || quant > 2) throw std::runtime_error("quant must be 0 (fp16), 1 (int8 symmetric per row) or 2 (int8 per group)");
        if (quant && (C % 128 || F % 128)) throw std::runtime_error("int8 needs n_embd and ffn_hidden to be multiples of 128");
        const bool lr_t = flags & 1, q_head = (flags & 2) && quant;
        Writer w;
        std::vector<uint16_t> buf;
        std::vector<uint8_t> idx;
        std::vector<uint32_t> sz;
        bool ok = true;
        auto emit = [&](const std::string& name, std::vector<int64_t> shape, Spec sp) {
            int64_t n = 1;
            for (auto d : shape) n *= d;
            if (!w.dry()) fill_f16(buf, Stream(seed, name), sp, n);
            ok = ok && w.add(name, "F16", shape, buf.data(), (size_t)n * 2);
        };
        auto emit_linear = [&](const std::string& name, int64_t M, int64_t K, bool q) {
            if (!w.dry()) fill_f16(buf, Stream(seed, name), Spec{NORMAL, 0.0, 0.02}, M * K);
            if (!q) {
                ok = ok && w.add(name, "F16", {M, K}, buf.data(), (size_t)(M * K) * 2);
            } else {
                if (!w.dry()) quantize(buf, M, K, quant, idx, sz);
                ok = ok && w.add(name + ".int8_idx", "U8", {M, K}, idx.data(), (size_t)(M * K));
                ok = ok && w.add(name + ".int8_sz", "U32", {M, K / 128}, sz.data(), (size_t)(M * (K / 128)) * 4);
            }
        };
        const Spec G{NORMAL, 0.0, 0.02}, G1{NORMAL, 1.0, 0.02}, U01{UNIFORM, 0.0, 1.0};
        auto emit_all = [&]() {
            emit("emb.weight", {V, C}, G);
            emit("blocks.0.ln0.weight", {C}, G1);
            emit("blocks.0.ln0.bias", {C}, G);
            for (int64_t i = 0; i < L && ok; ++i) {
                const std::string p = "blocks." + std::to_string(i) + ".";
                emit(p + "ln1.weight", {C}, G1);
                emit(p + "ln1.bias", {C}, G);
                emit(p + "ln2.weight", {C}, G1);
                emit(p + "ln2.bias", {C}, G);
                for (const char* x : {"x_r", "x_w", "x_k", "x_v", "x_a", "x_g"}) emit(p + "att." + x, {1, 1, C}, U01);
                emit(p + "att.w0", {1, 1, C}, Spec{UNIFORM, -6.0, -1.0});
                emit(p + "att.a0", {1, 1, C}, G);
                emit(p + "att.v0", {1, 1, C}, G);
                const int64_t mids[4] = {s->w_mid, s->a_mid, s->v_mid, s->g_mid};
                const char* lr[4] = {"w", "a", "v", "g"};
                for (int j = 0; j < 4; ++j) {
                    // the stream is indexed in file order, so the two storage orientations are different
                    // (equally valid) random matrices, not transposes of one another
                    if (!lr_t) {
                        emit(p + "att." + lr[j] + "1", {C, mids[j]}, G);
                        emit(p + "att." + lr[j] + "2", {mids[j], C}, G);
                    } else {
                        emit(p + "att." + lr[j] + "1", {mids[j], C}, G);
                        emit(p + "att." + lr[j] + "2", {C, mids[j]}, G);
                    }
                }
                emit(p + "att.r_k", {H, N}, G);
                emit(p + "att.k_k", {1, 1, C}, Spec{UNIFORM, 0.5, 1.5});
                emit(p + "att.k_a", {1, 1, C}, U01);
                emit(p + "att.ln_x.weight", {C}, G1);
                emit(p + "att.ln_x.bias", {C}, G);
                emit_linear(p + "att.receptance.weight", C, C, quant != 0);
                emit_linear(p + "att.key.weight", C, C, quant != 0);
                emit_linear(p + "att.value.weight", C, C, quant != 0);
                emit_linear(p + "att.output.weight", C, C, quant != 0);
                emit(p + "ffn.x_k", {1, 1, C}, U01);
                emit_linear(p + "ffn.key.weight", F, C, quant != 0);
                emit_linear(p + "ffn.value.weight", C, F, quant != 0);
            }
            emit("ln_out.weight", {C}, G1);
            emit("ln_out.bias", {C}, G);
            emit_linear("head.weight", V, C, q_head);
        };
        emit_all();  // pass 0: sizes only
        std::string meta = "{\"generator\":\"rsv_synth_write\",\"seed\":\"" + std::to_string(seed) + "\",\"quant\":\"" + std::to_string(quant) +
                           "\",\"flags\":\"" + std::to_string(flags) + "\"}";
        if (!w.begin_data(path, meta)) throw std::runtime_error(std::string("cannot create ") + path);
        emit_all();  // pass 1: data
        bool closed = w.finish();
        if (!ok || !closed) throw std::runtime_error("short write (disk full?)");
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

const char* rsv_synth_last_error(void) { return g_err.c_str(); }

// Number of OpenMP threads the generator uses (launchers such as torchrun export OMP_NUM_THREADS=1).
void rsv_synth_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

}  // extern "C"
