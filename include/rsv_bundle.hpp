// C++ mirror of the reference's library API over the C ABI in rsv_b200.h (header-only).
//
// Same names, argument meaning and error behaviour as the Rust types in src/gpu_model.rs:
//   ModelBuilder (:3685-3703)  Bundle (:3708-3843)  State (:3920-4105)  SamplerParams (:3883-3913)
//   ModelInfo (:75-99)  RnnInput / RnnOption (:3846-3876)  SelfloopTicket (:204-212)
// Where the Rust API returns `R<T> = Result<T, Box<dyn Error>>`, these throw rsv::Error carrying the same
// kind of message string.  One host thread per Bundle, as in the reference (`&mut self` everywhere).
#pragma once
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "rsv_b200.h"

namespace rsv {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};
inline void check(int rc) {
    if (rc != 0) throw Error(rsv_last_error());
}

enum class ModelVersion { V7 };
struct ModelInfo {
    ModelVersion version = ModelVersion::V7;
    size_t num_layer = 0, num_emb = 0, num_hidden = 0, num_vocab = 0, num_head = 0, head_size = 0, ffn_hidden = 0;
    size_t w_mid = 0, a_mid = 0, v_mid = 0, g_mid = 0;
};

struct SamplerParams : rsv_sampler_params {
    SamplerParams() : rsv_sampler_params{1.0f, 0u, 1.0f, 0u, 1.0f, 0.0f, 0.0f} {}  // impl Default, :3901-3912
};

enum class RnnOption { Last, Full };
struct RnnInput {
    std::vector<uint32_t> tokens;
    size_t chunk_size = 0;
    RnnOption option = RnnOption::Last;
    RnnInput(std::vector<uint32_t> t, size_t cs) : tokens(std::move(t)), chunk_size(cs) {}
};

class GpuModel;

class State {
public:
    State(State&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
    State& operator=(State&& o) noexcept {
        std::swap(h_, o.h_);
        return *this;
    }
    ~State() {
        if (h_) rsv_state_free(h_);
    }
    size_t batch() const { return (size_t)rsv_state_batch(h_); }
    std::vector<float> back() const {
        std::vector<float> out((size_t)rsv_state_len(h_));
        check(rsv_state_back(h_, out.data(), (int64_t)out.size()));
        return out;
    }
    void load(const std::vector<float>& data) const { check(rsv_state_load(h_, data.data(), (int64_t)data.size())); }
    std::vector<float> slot_back(size_t slot) const {
        std::vector<float> out((size_t)rsv_state_len(h_) / batch());
        check(rsv_state_slot_back(h_, (int64_t)slot, out.data(), (int64_t)out.size()));
        return out;
    }
    void slot_load(size_t slot, const std::vector<float>& data) const { check(rsv_state_slot_load(h_, (int64_t)slot, data.data(), (int64_t)data.size())); }
    // state files: the f32 array of back() as raw bytes (examples/state_persist.rs:38-47)
    void save(const std::string& path) const { check(rsv_state_save(h_, path.c_str())); }
    void restore(const std::string& path) const { check(rsv_state_restore(h_, path.c_str())); }
    void slot_save(size_t slot, const std::string& path) const { check(rsv_state_slot_save(h_, (int64_t)slot, path.c_str())); }
    void slot_restore(size_t slot, const std::string& path) const { check(rsv_state_slot_restore(h_, (int64_t)slot, path.c_str())); }
    // session migration: slot src_slot of src -> slot `slot` here, device to device (slot_back + slot_load without the host)
    void slot_copy_from(size_t slot, const State& src, size_t src_slot) const { check(rsv_state_slot_copy(h_, (int64_t)slot, src.h_, (int64_t)src_slot)); }
    void reset() const { check(rsv_state_reset(h_)); }
    rsv_state* handle() const { return h_; }

private:
    friend class GpuModel;
    explicit State(rsv_state* h) : h_(h) {}
    rsv_state* h_ = nullptr;
};

// In-flight self-loop: everything is queued on the GPU at submit, one synchronisation at collect.
struct SelfloopTicket {
    rsv_ticket* h = nullptr;
    size_t batch = 0, n = 0;
};

class GpuModel {
public:
    static GpuModel from_safetensors(const std::string& path, int device = 0) {
        rsv_model* h = nullptr;
        check(rsv_model_load(path.c_str(), device, &h));
        return GpuModel(h);
    }
    GpuModel(GpuModel&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
    ~GpuModel() {
        if (h_) rsv_model_free(h_);
    }
    ModelInfo info() const {
        rsv_model_info c{};
        check(rsv_model_info_get(h_, &c));
        ModelInfo i;
        i.num_layer = (size_t)c.num_layer;
        i.num_emb = (size_t)c.num_emb;
        i.num_hidden = (size_t)c.num_hidden;
        i.num_vocab = (size_t)c.num_vocab;
        i.num_head = (size_t)c.num_head;
        i.head_size = (size_t)c.head_size;
        i.ffn_hidden = (size_t)c.ffn_hidden;
        i.w_mid = (size_t)c.w_mid;
        i.a_mid = (size_t)c.a_mid;
        i.v_mid = (size_t)c.v_mid;
        i.g_mid = (size_t)c.g_mid;
        return i;
    }
    State create_state() { return create_batch_state(1); }
    State create_batch_state(size_t batch) {
        rsv_state* s = nullptr;
        check(rsv_state_new(h_, (int64_t)batch, &s));
        return State(s);
    }
    // forward_seq_batch (:1001-1011): returns each slot's last token (the decode seed)
    std::vector<uint32_t> forward_seq_batch(State& st, const std::vector<std::vector<uint32_t>>& tokens_batch) {
        if (tokens_batch.empty()) throw Error("forward_seq_batch: empty batch");
        size_t t_pad = 1;
        for (auto& t : tokens_batch) t_pad = std::max(t_pad, t.size());
        std::vector<uint32_t> flat(tokens_batch.size() * t_pad, 0u), lens(tokens_batch.size()), seeds(tokens_batch.size());
        for (size_t b = 0; b < tokens_batch.size(); ++b) {
            std::copy(tokens_batch[b].begin(), tokens_batch[b].end(), flat.begin() + b * t_pad);
            lens[b] = (uint32_t)tokens_batch[b].size();
        }
        check(rsv_prefill_batch(h_, st.handle(), flat.data(), lens.data(), (int64_t)tokens_batch.size(), (int64_t)t_pad, seeds.data()));
        return seeds;
    }
    // forward_seq_batch_mean_hidden (:1013-1036): resets the state, prefills, returns per slot the token mean of the last layer's
    // residual stream; pad_to (0: none) fixes the row pitch of the token matrix
    std::vector<std::vector<float>> forward_seq_batch_mean_hidden(State& st, const std::vector<std::vector<uint32_t>>& tokens_batch, size_t pad_to = 0) {
        if (tokens_batch.empty()) throw Error("forward_seq_batch: empty batch");
        size_t t_pad = std::max<size_t>(1, pad_to);
        for (auto& t : tokens_batch) t_pad = std::max(t_pad, t.size());
        std::vector<uint32_t> flat(tokens_batch.size() * t_pad, 0u), lens(tokens_batch.size());
        for (size_t b = 0; b < tokens_batch.size(); ++b) {
            std::copy(tokens_batch[b].begin(), tokens_batch[b].end(), flat.begin() + b * t_pad);
            lens[b] = (uint32_t)tokens_batch[b].size();
        }
        const size_t c = (size_t)info().num_emb;
        std::vector<float> mean(tokens_batch.size() * c);
        check(rsv_prefill_batch_mean_hidden(h_, st.handle(), flat.data(), lens.data(), (int64_t)tokens_batch.size(), (int64_t)t_pad, mean.data()));
        std::vector<std::vector<float>> out(tokens_batch.size());
        for (size_t b = 0; b < out.size(); ++b) out[b].assign(mean.begin() + b * c, mean.begin() + (b + 1) * c);
        return out;
    }
    // submit_sample_selfloop_batch (:1639-1781); sp == nullptr -> arg-max
    SelfloopTicket submit_sample_selfloop_batch(State& st, const std::vector<uint32_t>& seeds, size_t n, const SamplerParams* sp) {
        SelfloopTicket t;
        t.batch = seeds.size();
        t.n = n;
        check(rsv_sample_selfloop_submit(h_, st.handle(), seeds.data(), (int64_t)seeds.size(), (int64_t)n, sp, &t.h));
        return t;
    }
    // collect_sample_selfloop_batch (:1784-1802)
    std::vector<std::vector<uint32_t>> collect_sample_selfloop_batch(SelfloopTicket t) {
        std::vector<uint32_t> flat(t.batch * t.n);
        check(rsv_sample_selfloop_collect(t.h, flat.data(), (int64_t)flat.size()));
        std::vector<std::vector<uint32_t>> out(t.batch);
        for (size_t b = 0; b < t.batch; ++b) out[b].assign(flat.begin() + b * t.n, flat.begin() + (b + 1) * t.n);
        return out;
    }
    void clear_kernel_prof() { check(rsv_prof_clear(h_)); }
    std::string dump_kernel_prof() {
        std::string buf(1 << 16, '\0');
        check(rsv_prof_dump(h_, buf.data(), (int64_t)buf.size()));
        buf.resize(buf.find('\0'));
        return buf;
    }
    rsv_model* handle() const { return h_; }

private:
    explicit GpuModel(rsv_model* h) : h_(h) {}
    rsv_model* h_ = nullptr;
};

class Bundle {
public:
    GpuModel model;
    State state;

    explicit Bundle(GpuModel m) : model(std::move(m)), state(model.create_state()) {}
    ModelInfo info() const { return model.info(); }
    std::vector<float> infer_tokens(const std::vector<uint32_t>& tokens) {
        std::vector<float> out(info().num_vocab);
        check(rsv_infer_tokens(model.handle(), state.handle(), tokens.data(), (int64_t)tokens.size(), out.data()));
        return out;
    }
    std::vector<float> infer_seq(const std::vector<uint32_t>& tokens) {
        std::vector<float> out(info().num_vocab);
        check(rsv_infer_seq(model.handle(), state.handle(), tokens.data(), (int64_t)tokens.size(), out.data()));
        return out;
    }
    std::vector<float> infer(const RnnInput& in) {
        const size_t V = info().num_vocab;
        if (in.option == RnnOption::Full) {
            std::vector<float> out(in.tokens.size() * V);
            check(rsv_infer_full(model.handle(), state.handle(), in.tokens.data(), (int64_t)in.tokens.size(), out.data()));
            return out;
        }
        std::vector<float> out(V);
        check(rsv_infer_chunked(model.handle(), state.handle(), in.tokens.data(), (int64_t)in.tokens.size(),
                                (int64_t)std::max<size_t>(in.chunk_size, 1), out.data()));
        return out;
    }
    std::vector<float> infer_chunked(const std::vector<uint32_t>& tokens, size_t chunk_size) { return infer(RnnInput(tokens, chunk_size)); }
    uint32_t infer_argmax(const std::vector<uint32_t>& tokens) {
        uint32_t t = 0;
        check(rsv_infer_argmax(model.handle(), state.handle(), tokens.data(), (int64_t)tokens.size(), &t));
        return t;
    }
    std::vector<uint32_t> infer_argmax_selfloop(uint32_t seed, size_t n) {
        std::vector<uint32_t> out(n);
        check(rsv_infer_argmax_selfloop(model.handle(), state.handle(), seed, (int64_t)n, out.data()));
        return out;
    }
    uint32_t infer_sample(const std::vector<uint32_t>& tokens, const SamplerParams& sp, const std::vector<uint32_t>& history) {
        uint32_t t = 0;
        check(rsv_infer_sample(model.handle(), state.handle(), tokens.data(), (int64_t)tokens.size(), &sp, history.empty() ? nullptr : history.data(),
                               (int64_t)history.size(), &t));
        return t;
    }
    std::vector<uint32_t> infer_sample_selfloop(uint32_t seed, size_t n, const SamplerParams& sp) {
        std::vector<uint32_t> out(n);
        check(rsv_infer_sample_selfloop(model.handle(), state.handle(), seed, (int64_t)n, &sp, out.data()));
        return out;
    }
    std::vector<float> state_back() const { return state.back(); }
    void state_load(const std::vector<float>& data) const { state.load(data); }
    void reset() { state.reset(); }
    void clear_kernel_prof() { model.clear_kernel_prof(); }
    std::string dump_kernel_prof() { return model.dump_kernel_prof(); }
};

class ModelBuilder {
public:
    explicit ModelBuilder(std::string path, int device = 0) : path_(std::move(path)), device_(device) {}
    Bundle build() { return Bundle(GpuModel::from_safetensors(path_, device_)); }

private:
    std::string path_;
    int device_;
};

}  // namespace rsv
