// extern "C" surface declared in include/rsv_b200.h: argument validation, step planning and the
// host<->device copies around the engine.  No exception crosses this boundary.
#include <algorithm>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "engine.hpp"
#include "rsv_b200.h"

using namespace rsv;

struct rsv_model {
    std::unique_ptr<Model> m;
};
struct rsv_state {
    State s;
};
struct rsv_ticket {
    Ticket t;
};

namespace {

thread_local std::string g_err;

template <class F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const CudaError& e) {
        g_err = e.what();
        return 2;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    } catch (...) {
        g_err = "unknown error";
        return 3;
    }
}

void need(bool cond, const char* msg) {
    if (!cond) throw std::runtime_error(msg);
}

void check_tokens(const Model& m, const uint32_t* tokens, int64_t n) {
    for (int64_t i = 0; i < n; ++i)
        if (tokens[i] >= (uint32_t)m.cfg.vocab)
            throw std::runtime_error("token id " + std::to_string(tokens[i]) + " at position " + std::to_string(i) + " is >= vocab " + std::to_string(m.cfg.vocab));
}

// B decode rows: row b belongs to slot b.
StepPlan decode_plan(int B, bool want_logits) {
    StepPlan p;
    p.rows.resize(B);
    p.segs.resize(B);
    for (int b = 0; b < B; ++b) {
        p.rows[b] = RowMeta{b, 0, 1, b};
        p.segs[b] = SegMeta{b, 1, b, 0};
        if (want_logits) p.out_rows.push_back(b);
    }
    p.multi_row_segments = false;
    return p;
}

// One chunk of T consecutive tokens of the session in `slot`.
StepPlan chunk_plan(int slot, int T, int out_mode /*0 none, 1 last, 2 all*/) {
    StepPlan p;
    p.rows.resize(T);
    for (int r = 0; r < T; ++r) p.rows[r] = RowMeta{slot, r > 0 ? 1 : 0, r == T - 1 ? 1 : 0, 0};
    p.segs.push_back(SegMeta{0, T, slot, 0});
    if (out_mode == 1) p.out_rows.push_back(T - 1);
    if (out_mode == 2)
        for (int r = 0; r < T; ++r) p.out_rows.push_back(r);
    p.multi_row_segments = T > 1;
    return p;
}

void ensure_tok_list(Model& m, size_t n) {
    if (n > m.ws.tok_list_cap) {
        RSV_CUDA(cudaStreamSynchronize(m.stream));
        if (m.ws.tok_list) cudaFree(m.ws.tok_list);
        m.ws.tok_list = nullptr;
        m.ws.tok_list_cap = 0;
        size_t cap = std::max<size_t>(n, 1024);
        RSV_CUDA(cudaMalloc(&m.ws.tok_list, cap * sizeof(uint32_t)));
        m.ws.tok_list_cap = cap;
    }
}

// token-by-token decode of `tokens` on slot 0; logits of the last token stay in ws.logits[0,:]
void decode_tokens(Model& m, State& st, const uint32_t* tokens, int64_t n) {
    need(st.model == &m, "state belongs to a different model");
    need(st.cap == 1, "this call needs a single-session state (batch == 1)");
    need(n >= 1 && n <= 0x7fffffff, "empty token list (the count must be between 1 and 2^31 - 1)");
    check_tokens(m, tokens, n);
    RSV_CUDA(cudaSetDevice(m.device));
    if (!m.prof_on && m.persistent_available(1)) {
        m.ensure_workspace(1, 1, 1);
        ensure_tok_list(m, (size_t)n);
        RSV_CUDA(cudaMemcpyAsync(m.ws.tok_list, tokens, (size_t)n * sizeof(uint32_t), cudaMemcpyHostToDevice, m.stream));
        const int slot0 = 0;
        m.run_persistent(st, 1, &slot0, (int)n, true, false, nullptr, nullptr, 0);  // all n tokens in one launch, head on the last
        return;
    }
    StepPlan with_head = decode_plan(1, true), no_head = decode_plan(1, false);
    m.upload_plan(with_head);
    ensure_tok_list(m, (size_t)n);
    RSV_CUDA(cudaMemcpyAsync(m.ws.tok_list, tokens, (size_t)n * sizeof(uint32_t), cudaMemcpyHostToDevice, m.stream));
    RSV_CUDA(cudaMemsetAsync(m.ws.tok_pos, 0, sizeof(int), m.stream));
    for (int64_t i = 0; i < n; ++i) m.forward_rows(st, i == n - 1 ? with_head : no_head, true);
}

constexpr int kMaxChunk = 512;  // rows per packed step on the chunk path

// chunked prefill of one session; out_mode 1: logits of the very last token in ws.logits[0,:];
// out_mode 2: every position, copied to `all_out` chunk by chunk
void prefill_tokens(Model& m, State& st, const uint32_t* tokens, int64_t n, int64_t chunk, int out_mode, float* all_out) {
    need(st.model == &m, "state belongs to a different model");
    need(st.cap == 1, "this call needs a single-session state (batch == 1)");
    need(n >= 1, "empty token list");
    check_tokens(m, tokens, n);
    RSV_CUDA(cudaSetDevice(m.device));
    const int64_t cs = std::max<int64_t>(1, std::min<int64_t>(chunk <= 0 ? kMaxChunk : chunk, out_mode == 2 ? 128 : kMaxChunk));
    const size_t V = m.cfg.vocab;
    for (int64_t off = 0; off < n; off += cs) {
        const int T = (int)std::min<int64_t>(cs, n - off);
        const bool last = off + T >= n;
        StepPlan p = chunk_plan(0, T, out_mode == 2 ? 2 : (last && out_mode == 1 ? 1 : 0));
        m.upload_plan(p);
        RSV_CUDA(cudaMemcpyAsync(m.ws.tokens, tokens + off, (size_t)T * sizeof(uint32_t), cudaMemcpyHostToDevice, m.stream));
        m.forward_rows(st, p, false);
        if (out_mode == 2) {
            RSV_CUDA(cudaMemcpyAsync(all_out + (size_t)off * V, m.ws.logits, (size_t)T * V * sizeof(float), cudaMemcpyDeviceToHost, m.stream));
            RSV_CUDA(cudaStreamSynchronize(m.stream));
        }
    }
}

void fetch_logits(Model& m, float* logits_out) {
    RSV_CUDA(cudaMemcpyAsync(logits_out, m.ws.logits, (size_t)m.cfg.vocab * sizeof(float), cudaMemcpyDeviceToHost, m.stream));
    m.check_status();  // synchronises
}

void pack_sampler_row(float* row, const rsv_sampler_params& sp, uint32_t seed, uint32_t hist_len) {
    row[0] = sp.temperature;
    memcpy(&row[1], &sp.top_k, 4);
    row[2] = sp.top_p;
    memcpy(&row[3], &seed, 4);
    row[4] = sp.repetition_penalty;
    row[5] = sp.frequency_penalty;
    row[6] = sp.presence_penalty;
    memcpy(&row[7], &hist_len, 4);
}

std::unique_ptr<rsv_ticket> selfloop_submit(Model& m, State& st, const uint32_t* seeds, int64_t batch, int64_t n, const rsv_sampler_params* sp) {
    need(st.model == &m, "state belongs to a different model");
    need(batch >= 1 && n >= 1 && batch <= 0x7fffffff && n <= 0x7fffffff, "batch and n must be between 1 and 2^31 - 1");
    need(st.cap == batch, "state batch differs from the number of seeds");  // src/gpu_model.rs:1649-1657
    check_tokens(m, seeds, batch);
    RSV_CUDA(cudaSetDevice(m.device));
    const int B = (int)batch;
    StepPlan p = decode_plan(B, true);
    m.upload_plan(p);
    auto tk = std::make_unique<rsv_ticket>();
    Ticket& t = tk->t;
    t.model = &m;
    t.batch = batch;
    t.n = n;
    RSV_CUDA(cudaMalloc(&t.seq, (size_t)batch * n * sizeof(uint32_t)));
    RSV_CUDA(cudaMalloc(&t.cnt, (size_t)batch * sizeof(int)));
    RSV_CUDA(cudaMemsetAsync(t.seq, 0, (size_t)batch * n * sizeof(uint32_t), m.stream));
    RSV_CUDA(cudaMemsetAsync(t.cnt, 0, (size_t)batch * sizeof(int), m.stream));
    RSV_CUDA(cudaMemcpyAsync(m.ws.tokens, seeds, (size_t)batch * sizeof(uint32_t), cudaMemcpyHostToDevice, m.stream));
    if (sp) {
        // round r of slot b draws with seed seeds[b] + r and penalises the r tokens generated so far
        // (src/gpu_model.rs:1738-1756); the kernel adds r itself from the slot's token counter.
        std::vector<float> rows((size_t)batch * 8);
        for (int64_t b = 0; b < batch; ++b) pack_sampler_row(&rows[(size_t)b * 8], *sp, seeds[b], 0);
        RSV_CUDA(cudaMalloc(&t.sampler, rows.size() * sizeof(float)));
        RSV_CUDA(cudaMemcpyAsync(t.sampler, rows.data(), rows.size() * sizeof(float), cudaMemcpyHostToDevice, m.stream));
        RSV_CUDA(cudaStreamSynchronize(m.stream));  // `rows` is a stack-lifetime pageable buffer
    }
    auto one_round = [&] {
        m.forward_rows(st, p, false);
        if (sp)
            engine_sample(m, m.ws.logits, B, t.sampler, t.seq, (int)n, t.cnt, m.ws.tokens, t.seq, t.cnt, (int)n);
        else
            engine_argmax(m, m.ws.logits, B, m.ws.tokens, t.seq, t.cnt, (int)n);
    };
    if (!m.prof_on && B <= 4 && m.persistent_available(B)) {
        // up to 4 sessions: the persistent kernel runs whole steps (and, for arg-max, the whole self-loop) in one launch
        int slots[4] = {0, 1, 2, 3};
        if (!sp) {
            m.run_persistent(st, B, slots, (int)n, false, true, t.seq, t.cnt, (int)n);
        } else {
            for (int64_t round = 0; round < n; ++round) {
                m.run_persistent(st, B, slots, 1, false, false, nullptr, nullptr, 0);
                engine_sample(m, m.ws.logits, B, t.sampler, t.seq, (int)n, t.cnt, m.ws.tokens, t.seq, t.cnt, (int)n);
            }
        }
        return tk;
    }
    // Round 0 runs eagerly (it also sizes every work buffer); the remaining rounds replay one captured CUDA graph
    // of the step, as the reference replays its captured self-loop step (src/gpu_model.rs:1847-1859).  Per-kernel
    // profiling needs event pairs between launches, so it keeps the eager path.
    one_round();
    if (n > 1) {
        if (m.prof_on || !m.use_graphs) {
            for (int64_t round = 1; round < n; ++round) one_round();
        } else {
            cudaGraph_t graph = nullptr;
            cudaGraphExec_t exec = nullptr;
            RSV_CUDA(cudaStreamBeginCapture(m.stream, cudaStreamCaptureModeThreadLocal));
            const long launches_before = m.launches;
            try {
                one_round();
            } catch (...) {
                cudaStreamEndCapture(m.stream, &graph);
                if (graph) cudaGraphDestroy(graph);
                throw;
            }
            RSV_CUDA(cudaStreamEndCapture(m.stream, &graph));
            const long per_round = m.launches - launches_before;
            cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
            if (e != cudaSuccess) {
                cudaGraphDestroy(graph);
                throw CudaError(std::string("cudaGraphInstantiate failed: ") + cudaGetErrorString(e));
            }
            m.launches = launches_before;  // the capture itself launched nothing
            for (int64_t round = 1; round < n; ++round) {
                e = cudaGraphLaunch(exec, m.stream);
                if (e != cudaSuccess) break;
                m.launches += per_round;
            }
            t.graph = graph;
            t.graph_exec = exec;
            if (e != cudaSuccess) throw CudaError(std::string("cudaGraphLaunch failed: ") + cudaGetErrorString(e));
        }
    }
    return tk;
}

void selfloop_collect(rsv_ticket* tk, uint32_t* out, int64_t len) {
    // a wrong length leaves the ticket (and its queued results) with the caller, who may call again
    need(len == tk->t.batch * tk->t.n, "output length must be batch * n");
    std::unique_ptr<rsv_ticket> own(tk);
    Ticket& t = tk->t;
    Model& m = *t.model;
    RSV_CUDA(cudaSetDevice(m.device));
    RSV_CUDA(cudaMemcpyAsync(out, t.seq, (size_t)len * sizeof(uint32_t), cudaMemcpyDeviceToHost, m.stream));
    m.check_status();
}

}  // namespace

namespace rsv {
void set_last_error(const std::string& msg) { g_err = msg; }
}  // namespace rsv

extern "C" {

const char* rsv_last_error(void) { return g_err.c_str(); }

int rsv_model_load(const char* path, int device, rsv_model** out) {
    return guarded([&] {
        need(path && out, "null argument");
        auto h = std::make_unique<rsv_model>();
        h->m = Model::load(path, device);
        *out = h.release();
    });
}
void rsv_model_free(rsv_model* m) { delete m; }
int rsv_model_info_get(const rsv_model* m, rsv_model_info* o) {
    return guarded([&] {
        need(m && o, "null argument");
        const Config& c = m->m->cfg;
        o->version = 7;
        o->num_layer = c.n_layer;
        o->num_emb = c.n_embd;
        o->num_hidden = c.n_embd;
        o->num_vocab = c.vocab;
        o->num_head = c.n_head;
        o->head_size = c.head_size;
        o->ffn_hidden = c.ffn_hidden;
        o->w_mid = c.w_mid;
        o->a_mid = c.a_mid;
        o->v_mid = c.v_mid;
        o->g_mid = c.g_mid;
    });
}
int64_t rsv_model_weight_bytes(const rsv_model* m) { return m ? (int64_t)m->m->weight_bytes : 0; }

int rsv_state_new(rsv_model* mh, int64_t batch, rsv_state** out) {
    return guarded([&] {
        need(mh && out, "null argument");
        Model& m = *mh->m;
        const int64_t cap = std::max<int64_t>(batch, 1);  // State::new_batched clamps to >= 1 (src/gpu_model.rs:3950)
        RSV_CUDA(cudaSetDevice(m.device));
        auto h = std::make_unique<rsv_state>();
        State& s = h->s;
        s.model = &m;
        s.cap = cap;
        const Config& c = m.cfg;
        const size_t nx = (size_t)c.n_layer * cap * c.n_embd, ns = (size_t)c.n_layer * cap * c.n_head * kHeadSize * kHeadSize, nv = (size_t)cap * c.n_embd;
        RSV_CUDA(cudaMalloc(&s.tmix_x, nx * 4));
        RSV_CUDA(cudaMalloc(&s.cmix_x, nx * 4));
        RSV_CUDA(cudaMalloc(&s.wkv, ns * 4));
        RSV_CUDA(cudaMalloc(&s.v_first, nv * 4));
        RSV_CUDA(cudaMemsetAsync(s.tmix_x, 0, nx * 4, m.stream));
        RSV_CUDA(cudaMemsetAsync(s.cmix_x, 0, nx * 4, m.stream));
        RSV_CUDA(cudaMemsetAsync(s.wkv, 0, ns * 4, m.stream));
        RSV_CUDA(cudaMemsetAsync(s.v_first, 0, nv * 4, m.stream));
        RSV_CUDA(cudaStreamSynchronize(m.stream));
        *out = h.release();
    });
}
void rsv_state_free(rsv_state* s) { delete s; }
int64_t rsv_state_batch(const rsv_state* s) { return s ? s->s.cap : 0; }
int64_t rsv_state_len(const rsv_state* s) { return s ? (int64_t)(s->s.cap * (int64_t)s->s.model->cfg.state_floats_per_slot()) : 0; }

// Copies slots [slot0, slot0+nslot) between the device arrays and the host layout of State::back.
static void state_copy(State& s, int64_t slot0, int64_t nslot, float* host, bool to_host) {
    Model& m = *s.model;
    const Config& c = m.cfg;
    RSV_CUDA(cudaSetDevice(m.device));
    const size_t C = c.n_embd, HNN = (size_t)c.n_head * kHeadSize * kHeadSize, per = c.state_floats_per_slot();
    const size_t per_layer = 2 * C + HNN;
    auto cp = [&](float* dev_base, size_t dev_row_floats, size_t host_off, size_t width_floats) {
        // nslot rows of `width_floats`: device pitch = row size, host pitch = one whole slot
        float* d = dev_base + (size_t)slot0 * dev_row_floats;
        float* h = host + host_off;
        if (to_host)
            RSV_CUDA(cudaMemcpy2DAsync(h, per * 4, d, dev_row_floats * 4, width_floats * 4, (size_t)nslot, cudaMemcpyDeviceToHost, m.stream));
        else
            RSV_CUDA(cudaMemcpy2DAsync(d, dev_row_floats * 4, h, per * 4, width_floats * 4, (size_t)nslot, cudaMemcpyHostToDevice, m.stream));
    };
    for (int l = 0; l < c.n_layer; ++l) {
        cp(s.tmix_x + (size_t)l * s.cap * C, C, (size_t)l * per_layer, C);
        cp(s.wkv + (size_t)l * s.cap * HNN, HNN, (size_t)l * per_layer + C, HNN);
        cp(s.cmix_x + (size_t)l * s.cap * C, C, (size_t)l * per_layer + C + HNN, C);
    }
    cp(s.v_first, C, (size_t)c.n_layer * per_layer, C);
    RSV_CUDA(cudaStreamSynchronize(m.stream));
}

int rsv_state_back(rsv_state* s, float* out, int64_t len) {
    return guarded([&] {
        need(s && out, "null argument");
        need(len == rsv_state_len(s), "state_back: buffer length does not match the state size");
        state_copy(s->s, 0, s->s.cap, out, true);
    });
}
int rsv_state_load(rsv_state* s, const float* data, int64_t len) {
    return guarded([&] {
        need(s && data, "null argument");
        need(len == rsv_state_len(s), "State::load length mismatch");  // src/gpu_model.rs:4001-4005
        state_copy(s->s, 0, s->s.cap, const_cast<float*>(data), false);
    });
}
int rsv_state_slot_back(rsv_state* s, int64_t slot, float* out, int64_t len) {
    return guarded([&] {
        need(s && out, "null argument");
        need(slot >= 0 && slot < s->s.cap, "slot_back: slot >= batch");  // src/gpu_model.rs:4046-4048
        need(len == (int64_t)s->s.model->cfg.state_floats_per_slot(), "slot_back: buffer length does not match one slot");
        state_copy(s->s, slot, 1, out, true);
    });
}
int rsv_state_slot_load(rsv_state* s, int64_t slot, const float* data, int64_t len) {
    return guarded([&] {
        need(s && data, "null argument");
        need(slot >= 0 && slot < s->s.cap, "slot_load: slot >= batch");
        need(len == (int64_t)s->s.model->cfg.state_floats_per_slot(), "State::slot_load length mismatch");
        state_copy(s->s, slot, 1, const_cast<float*>(data), false);
    });
}
// ---- state files and slot migration -------------------------------------------------------------------
// A state file is the f32 array of State::back as raw little-endian bytes with no header: the bytes the reference's
// examples/state_persist.rs:38-47 writes and reads back.  The size of the file is the only check there is.
static std::vector<float> read_state_file(const char* path, size_t floats) {
    FILE* f = fopen(path, "rb");
    if (!f) throw std::runtime_error(std::string("cannot open state file ") + path);
    std::vector<float> buf(floats);
    const size_t got = fread(buf.data(), 4, floats, f);
    char extra;
    const bool more = got == floats && fread(&extra, 1, 1, f) == 1;
    fclose(f);
    if (got != floats || more)
        throw std::runtime_error(std::string("state file ") + path + " does not hold exactly " + std::to_string(floats) + " f32 (State::load length mismatch)");
    return buf;
}
static void write_state_file(const char* path, const std::vector<float>& buf) {
    // written under a temporary name and renamed, so that a reader never sees half a state
    const std::string tmp = std::string(path) + ".part";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) throw std::runtime_error(std::string("cannot create state file ") + path);
    const size_t put = fwrite(buf.data(), 4, buf.size(), f);
    const bool ok = fclose(f) == 0 && put == buf.size();
    if (!ok || rename(tmp.c_str(), path) != 0) {
        remove(tmp.c_str());
        throw std::runtime_error(std::string("cannot write state file ") + path);
    }
}
int rsv_state_save(rsv_state* s, const char* path) {
    return guarded([&] {
        need(s && path, "null argument");
        std::vector<float> buf((size_t)rsv_state_len(s));
        state_copy(s->s, 0, s->s.cap, buf.data(), true);
        write_state_file(path, buf);
    });
}
int rsv_state_restore(rsv_state* s, const char* path) {
    return guarded([&] {
        need(s && path, "null argument");
        std::vector<float> buf = read_state_file(path, (size_t)rsv_state_len(s));  // the state is untouched when the file is refused
        state_copy(s->s, 0, s->s.cap, buf.data(), false);
    });
}
int rsv_state_slot_save(rsv_state* s, int64_t slot, const char* path) {
    return guarded([&] {
        need(s && path, "null argument");
        need(slot >= 0 && slot < s->s.cap, "slot_back: slot >= batch");
        std::vector<float> buf(s->s.model->cfg.state_floats_per_slot());
        state_copy(s->s, slot, 1, buf.data(), true);
        write_state_file(path, buf);
    });
}
int rsv_state_slot_restore(rsv_state* s, int64_t slot, const char* path) {
    return guarded([&] {
        need(s && path, "null argument");
        need(slot >= 0 && slot < s->s.cap, "slot_load: slot >= batch");
        std::vector<float> buf = read_state_file(path, s->s.model->cfg.state_floats_per_slot());
        state_copy(s->s, slot, 1, buf.data(), false);
    });
}
// Moves one session: slot `src_slot` of `src` -> slot `dst_slot` of `dst`, device to device (the two states may belong to
// different model handles on the same GPU or on two GPUs; the shapes must agree).  3 L + 1 copies, no host staging of ours:
// cudaMemcpyPeerAsync goes over NVLink when the driver allows peer access and through the host otherwise.
int rsv_state_slot_copy(rsv_state* dst, int64_t dst_slot, rsv_state* src, int64_t src_slot) {
    return guarded([&] {
        need(dst && src, "null argument");
        State &D = dst->s, &S = src->s;
        const Config &cd = D.model->cfg, &cs = S.model->cfg;
        need(dst_slot >= 0 && dst_slot < D.cap, "slot_load: slot >= batch");
        need(src_slot >= 0 && src_slot < S.cap, "slot_back: slot >= batch");
        need(cd.n_layer == cs.n_layer && cd.n_embd == cs.n_embd && cd.n_head == cs.n_head, "slot copy: the two states belong to models of different shapes");
        if (&D == &S && dst_slot == src_slot) return;
        const size_t C = cs.n_embd, HNN = (size_t)cs.n_head * kHeadSize * kHeadSize;
        const int dd = D.model->device, sd = S.model->device;
        // what the source's stream has queued (the session's last step) must be complete before the copy reads it; the copy
        // runs on the destination's stream, behind whatever that GPU still does with the slot
        RSV_CUDA(cudaSetDevice(sd));
        RSV_CUDA(cudaStreamSynchronize(S.model->stream));
        RSV_CUDA(cudaSetDevice(dd));
        cudaStream_t st = D.model->stream;
        auto cp = [&](float* dbase, const float* sbase, size_t width, int l) {
            float* d = dbase + ((size_t)l * D.cap + (size_t)dst_slot) * width;
            const float* q = sbase + ((size_t)l * S.cap + (size_t)src_slot) * width;
            if (dd == sd)
                RSV_CUDA(cudaMemcpyAsync(d, q, width * 4, cudaMemcpyDeviceToDevice, st));
            else
                RSV_CUDA(cudaMemcpyPeerAsync(d, dd, q, sd, width * 4, st));
        };
        for (int l = 0; l < cs.n_layer; ++l) {
            cp(D.tmix_x, S.tmix_x, C, l);
            cp(D.wkv, S.wkv, HNN, l);
            cp(D.cmix_x, S.cmix_x, C, l);
        }
        cp(D.v_first, S.v_first, C, 0);
        RSV_CUDA(cudaStreamSynchronize(st));
    });
}

int rsv_state_reset(rsv_state* sh) {
    return guarded([&] {
        need(sh, "null argument");
        State& s = sh->s;
        Model& m = *s.model;
        const Config& c = m.cfg;
        RSV_CUDA(cudaSetDevice(m.device));
        const size_t nx = (size_t)c.n_layer * s.cap * c.n_embd, ns = (size_t)c.n_layer * s.cap * c.n_head * kHeadSize * kHeadSize;
        RSV_CUDA(cudaMemsetAsync(s.tmix_x, 0, nx * 4, m.stream));
        RSV_CUDA(cudaMemsetAsync(s.cmix_x, 0, nx * 4, m.stream));
        RSV_CUDA(cudaMemsetAsync(s.wkv, 0, ns * 4, m.stream));
        RSV_CUDA(cudaMemsetAsync(s.v_first, 0, (size_t)s.cap * c.n_embd * 4, m.stream));
        RSV_CUDA(cudaStreamSynchronize(m.stream));
    });
}

int rsv_infer_tokens(rsv_model* m, rsv_state* s, const uint32_t* tokens, int64_t n, float* logits_out) {
    return guarded([&] {
        need(m && s && tokens && logits_out, "null argument");
        decode_tokens(*m->m, s->s, tokens, n);
        fetch_logits(*m->m, logits_out);
    });
}
int rsv_infer_seq(rsv_model* m, rsv_state* s, const uint32_t* tokens, int64_t n, float* logits_out) {
    return guarded([&] {
        need(m && s && tokens && logits_out, "null argument");
        prefill_tokens(*m->m, s->s, tokens, n, 0, 1, nullptr);
        fetch_logits(*m->m, logits_out);
    });
}
int rsv_infer_chunked(rsv_model* m, rsv_state* s, const uint32_t* tokens, int64_t n, int64_t chunk_size, float* logits_out) {
    return guarded([&] {
        need(m && s && tokens && logits_out, "null argument");
        prefill_tokens(*m->m, s->s, tokens, n, std::max<int64_t>(chunk_size, 1), 1, nullptr);  // chunk_size.max(1), src/gpu_model.rs:3775
        fetch_logits(*m->m, logits_out);
    });
}
int rsv_infer_full(rsv_model* m, rsv_state* s, const uint32_t* tokens, int64_t n, float* logits_out) {
    return guarded([&] {
        need(m && s && tokens && logits_out, "null argument");
        prefill_tokens(*m->m, s->s, tokens, n, 0, 2, logits_out);
        m->m->check_status();
    });
}
int rsv_infer_argmax(rsv_model* mh, rsv_state* s, const uint32_t* tokens, int64_t n, uint32_t* token_out) {
    return guarded([&] {
        need(mh && s && tokens && token_out, "null argument");
        Model& m = *mh->m;
        decode_tokens(m, s->s, tokens, n);
        engine_argmax(m, m.ws.logits, 1, m.ws.tokens, nullptr, nullptr, 0);
        RSV_CUDA(cudaMemcpyAsync(token_out, m.ws.tokens, sizeof(uint32_t), cudaMemcpyDeviceToHost, m.stream));
        m.check_status();
    });
}
int rsv_infer_argmax_selfloop(rsv_model* m, rsv_state* s, uint32_t seed, int64_t n, uint32_t* out) {
    return guarded([&] {
        need(m && s && out, "null argument");
        need(s->s.cap == 1, "this call needs a single-session state (batch == 1)");
        auto t = selfloop_submit(*m->m, s->s, &seed, 1, n, nullptr);
        selfloop_collect(t.release(), out, n);
    });
}
int rsv_infer_sample(rsv_model* mh, rsv_state* s, const uint32_t* tokens, int64_t n, const rsv_sampler_params* sp, const uint32_t* history,
                     int64_t nh, uint32_t* token_out) {
    return guarded([&] {
        need(mh && s && tokens && sp && token_out, "null argument");
        need(nh >= 0 && nh <= 0x7fffffff, "history length must be between 0 and 2^31 - 1");
        need(nh == 0 || history, "history is null but nh > 0");
        Model& m = *mh->m;
        decode_tokens(m, s->s, tokens, n);
        float row[8];
        pack_sampler_row(row, *sp, sp->seed, (uint32_t)nh);
        float* d_row = nullptr;
        uint32_t* d_hist = nullptr;
        RSV_CUDA(cudaMalloc(&d_row, sizeof(row)));
        if (nh) RSV_CUDA(cudaMalloc(&d_hist, (size_t)nh * sizeof(uint32_t)));
        int rc = guarded([&] {
            RSV_CUDA(cudaMemcpyAsync(d_row, row, sizeof(row), cudaMemcpyHostToDevice, m.stream));
            if (nh) RSV_CUDA(cudaMemcpyAsync(d_hist, history, (size_t)nh * sizeof(uint32_t), cudaMemcpyHostToDevice, m.stream));
            engine_sample(m, m.ws.logits, 1, d_row, d_hist, (int)nh, nullptr, m.ws.tokens, nullptr, nullptr, 0);
            RSV_CUDA(cudaMemcpyAsync(token_out, m.ws.tokens, sizeof(uint32_t), cudaMemcpyDeviceToHost, m.stream));
            m.check_status();
        });
        cudaFree(d_row);
        if (d_hist) cudaFree(d_hist);
        if (rc) throw std::runtime_error(g_err);
    });
}
int rsv_infer_sample_selfloop(rsv_model* m, rsv_state* s, uint32_t seed, int64_t n, const rsv_sampler_params* sp, uint32_t* out) {
    return guarded([&] {
        need(m && s && sp && out, "null argument");
        need(s->s.cap == 1, "this call needs a single-session state (batch == 1)");
        auto t = selfloop_submit(*m->m, s->s, &seed, 1, n, sp);
        selfloop_collect(t.release(), out, n);
    });
}

// forward_seq_batch_core (src/gpu_model.rs:914-997) over packed steps; with `mean_out` also the per-slot mean of the last layer's
// residual stream (forward_seq_batch_mean_hidden, :1013-1036).
static void prefill_batch(Model& m, State& st, const uint32_t* flat, const uint32_t* lens, int64_t batch, int64_t t_pad, uint32_t* seeds_out, float* mean_out) {
    need(batch >= 1 && batch <= 0x7fffffff, "forward_seq_batch: empty batch");      // src/gpu_model.rs:921-923
    need(t_pad >= 1 && t_pad <= 0x7fffffff, "forward_seq_batch: t_pad must be >= 1");
    need(st.cap == batch, "forward_seq_batch: state batch differs from the prompts");  // :924-931
    std::vector<int64_t> len(batch), done(batch, 0);
    for (int64_t b = 0; b < batch; ++b) {
        len[b] = std::min<int64_t>(std::max<int64_t>(lens[b], 1), t_pad);  // lens clamp, :947-950
        check_tokens(m, flat + b * t_pad, len[b]);
        if (seeds_out) seeds_out[b] = flat[b * t_pad + len[b] - 1];
    }
    RSV_CUDA(cudaSetDevice(m.device));
    const size_t C = m.cfg.n_embd;
    float* acc = nullptr;
    struct Free {
        float*& p;
        ~Free() {
            if (p) cudaFree(p);
        }
    } guard{acc};
    if (mean_out) {
        RSV_CUDA(cudaMalloc(&acc, (size_t)batch * C * 4));
        RSV_CUDA(cudaMemsetAsync(acc, 0, (size_t)batch * C * 4, m.stream));
    }
    // pack chunks of several sessions into steps of at most kMaxChunk rows
    std::vector<uint32_t> toks;
    for (;;) {
        StepPlan p;
        toks.clear();
        for (int64_t b = 0; b < batch && (int)p.rows.size() < kMaxChunk; ++b) {
            const int64_t rem = len[b] - done[b];
            if (rem <= 0) continue;
            const int T = (int)std::min<int64_t>(rem, kMaxChunk - (int64_t)p.rows.size());
            const int start = (int)p.rows.size(), seg = (int)p.segs.size();
            for (int r = 0; r < T; ++r) {
                p.rows.push_back(RowMeta{(int)b, r > 0 ? 1 : 0, r == T - 1 ? 1 : 0, seg});
                toks.push_back(flat[b * t_pad + done[b] + r]);
            }
            p.segs.push_back(SegMeta{start, T, (int)b, 0});
            if (T > 1) p.multi_row_segments = true;
            done[b] += T;
        }
        if (p.rows.empty()) break;
        m.upload_plan(p);
        RSV_CUDA(cudaMemcpyAsync(m.ws.tokens, toks.data(), toks.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, m.stream));
        m.forward_rows(st, p, false);
        if (mean_out) engine_segment_sums(m, (int)p.segs.size(), acc);
        RSV_CUDA(cudaStreamSynchronize(m.stream));  // `toks` is reused by the next step
    }
    m.check_status();
    if (mean_out) {
        RSV_CUDA(cudaMemcpy(mean_out, acc, (size_t)batch * C * 4, cudaMemcpyDeviceToHost));
        for (int64_t b = 0; b < batch; ++b)
            for (size_t c = 0; c < C; ++c) mean_out[b * C + c] = mean_out[b * C + c] / (float)len[b];  // acc / (float)len, src/backend_cuda.rs:4429
    }
}
int rsv_prefill_batch(rsv_model* mh, rsv_state* sh, const uint32_t* flat, const uint32_t* lens, int64_t batch, int64_t t_pad, uint32_t* seeds_out) {
    return guarded([&] {
        need(mh && sh && flat && lens && seeds_out, "null argument");
        need(sh->s.model == mh->m.get(), "state belongs to a different model");
        prefill_batch(*mh->m, sh->s, flat, lens, batch, t_pad, seeds_out, nullptr);
    });
}
int rsv_prefill_batch_mean_hidden(rsv_model* mh, rsv_state* sh, const uint32_t* flat, const uint32_t* lens, int64_t batch, int64_t t_pad, float* mean_out) {
    return guarded([&] {
        need(mh && sh && flat && lens && mean_out, "null argument");
        need(sh->s.model == mh->m.get(), "state belongs to a different model");
        need(rsv_state_reset(sh) == 0, "state reset failed");  // the feature starts from a zero state (src/gpu_model.rs:1024)
        prefill_batch(*mh->m, sh->s, flat, lens, batch, t_pad, nullptr, mean_out);
    });
}

int rsv_sample_selfloop_submit(rsv_model* m, rsv_state* s, const uint32_t* seeds, int64_t batch, int64_t n, const rsv_sampler_params* sp,
                               rsv_ticket** out) {
    return guarded([&] {
        need(m && s && seeds && out, "null argument");
        *out = selfloop_submit(*m->m, s->s, seeds, batch, n, sp).release();
    });
}
int rsv_sample_selfloop_collect(rsv_ticket* t, uint32_t* out, int64_t len) {
    return guarded([&] {
        need(t && out, "null argument");
        selfloop_collect(t, out, len);
    });
}

int rsv_prof_enable(rsv_model* m, int on) {
    return guarded([&] {
        need(m, "null argument");
        RSV_CUDA(cudaStreamSynchronize(m->m->stream));
        m->m->prof_on = on != 0;
    });
}
int rsv_prof_clear(rsv_model* m) {
    return guarded([&] {
        need(m, "null argument");
        m->m->prof.clear();
        m->m->launches = 0;
    });
}
int rsv_prof_dump(rsv_model* m, char* buf, int64_t cap) {
    return guarded([&] {
        need(m && buf && cap > 0, "null argument");
        std::string s = "{";
        bool first = true;
        for (auto& kv : m->m->prof) {
            if (!first) s += ",";
            first = false;
            char tmp[256];
            snprintf(tmp, sizeof(tmp), "\"%s\":{\"launches\":%ld,\"ms\":%.6f}", kv.first.c_str(), kv.second.launches, kv.second.ms);
            s += tmp;
        }
        s += "}";
        const size_t n = std::min<size_t>(s.size(), (size_t)cap - 1);
        memcpy(buf, s.data(), n);
        buf[n] = 0;
    });
}
int64_t rsv_launch_count(const rsv_model* m) { return m ? m->m->launches : 0; }
int rsv_timer_start(rsv_model* m) {
    return guarded([&] {
        need(m, "null argument");
        RSV_CUDA(cudaSetDevice(m->m->device));
        RSV_CUDA(cudaEventRecord(m->m->tev[0], m->m->stream));
    });
}
int rsv_timer_stop(rsv_model* m, float* ms_out) {
    return guarded([&] {
        need(m && ms_out, "null argument");
        RSV_CUDA(cudaEventRecord(m->m->tev[1], m->m->stream));
        RSV_CUDA(cudaEventSynchronize(m->m->tev[1]));
        RSV_CUDA(cudaEventElapsedTime(ms_out, m->m->tev[0], m->m->tev[1]));
    });
}
int rsv_synchronize(rsv_model* m) {
    return guarded([&] {
        need(m, "null argument");
        RSV_CUDA(cudaStreamSynchronize(m->m->stream));
    });
}

// ---- operator-level entry points ----------------------------------------------------------------
namespace {
struct DevBuf {
    void* p = nullptr;
    explicit DevBuf(size_t bytes) { RSV_CUDA(cudaMalloc(&p, std::max<size_t>(bytes, 16))); }
    ~DevBuf() {
        if (p) cudaFree(p);
    }
    DevBuf(const DevBuf&) = delete;
};
void select_device(int device) {
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0) throw CudaError(std::string("no CUDA device available (") + cudaGetErrorString(e) + "): this library has no CPU fallback");
    need(device >= 0 && device < ndev, "device index out of range");
    RSV_CUDA(cudaSetDevice(device));
}
}  // namespace

int rsv_op_dequant_int8(int device, const uint8_t* idx, const uint32_t* sz, int64_t M, int64_t K, float* out) {
    return guarded([&] {
        need(idx && sz && out, "null argument");
        need(M >= 1 && K >= 128 && K % 128 == 0, "dequant_int8: K must be a positive multiple of 128");
        select_device(device);
        DevBuf di((size_t)M * K), dz((size_t)M * (K / 128) * 4), dout((size_t)M * K * 4);
        RSV_CUDA(cudaMemcpy(di.p, idx, (size_t)M * K, cudaMemcpyHostToDevice));
        RSV_CUDA(cudaMemcpy(dz.p, sz, (size_t)M * (K / 128) * 4, cudaMemcpyHostToDevice));
        engine_dequant_int8(nullptr, (const uint8_t*)di.p, (const uint32_t*)dz.p, (size_t)M, (size_t)K, (float*)dout.p);
        RSV_CUDA(cudaMemcpy(out, dout.p, (size_t)M * K * 4, cudaMemcpyDeviceToHost));
    });
}
int rsv_quantize_int8(int device, const float* w, int64_t M, int64_t K, uint8_t* idx_out, uint32_t* sz_out) {
    return guarded([&] {
        need(w && idx_out && sz_out, "null argument");
        need(M >= 1 && K >= 128 && K % 128 == 0, "quantize_int8: K must be a positive multiple of 128");  // assert K % group == 0, tools/quantize_any4.py:253
        need(M <= 0x7fffffff && K <= 0x7fffffff, "quantize_int8: matrix too large");
        select_device(device);
        DevBuf dw((size_t)M * K * 4), di((size_t)M * K), dz((size_t)M * (K / 128) * 4);
        RSV_CUDA(cudaMemcpy(dw.p, w, (size_t)M * K * 4, cudaMemcpyHostToDevice));
        engine_quantize_int8(nullptr, (const float*)dw.p, (size_t)M, (size_t)K, (uint8_t*)di.p, (uint32_t*)dz.p);
        RSV_CUDA(cudaMemcpy(idx_out, di.p, (size_t)M * K, cudaMemcpyDeviceToHost));
        RSV_CUDA(cudaMemcpy(sz_out, dz.p, (size_t)M * (K / 128) * 4, cudaMemcpyDeviceToHost));
    });
}
int rsv_op_linear(int device, int path, int wtype, const void* w, const uint32_t* sz, int64_t M, int64_t K, const float* x, int64_t R, float* y) {
    return guarded([&] {
        need(w && x && y, "null argument");
        need(wtype == W_F16 || (wtype == W_INT8 && sz), "op_linear: wtype must be 0 (fp16) or 1 (int8, with sz)");
        need(path == 0 || path == 1, "op_linear: path must be 0 (SIMT) or 1 (tensor core)");
        need(M >= 1 && K >= 1 && R >= 1 && M <= 0x7fffffff && K <= 0x7fffffff && R <= 0x7fffffff, "op_linear: M, K and R must be between 1 and 2^31 - 1");
        select_device(device);
        auto m = Model::create_bare(device);
        engine_op_linear(*m, path, wtype, w, sz, (int)M, (int)K, x, (int)R, y);
    });
}
int rsv_op_wkv7(int device, int variant, int64_t nseg, int64_t T, int64_t H, const float* r, const float* k, const float* v, const float* w, const float* a,
                const float* g, const float* vgate, const float* vfirst, const float* k_k, const float* k_a, const float* r_k, const float* lnx_w,
                const float* lnx_b, float* state, float* y) {
    return guarded([&] {
        need(r && k && v && w && a && g && k_k && k_a && r_k && lnx_w && lnx_b && state && y, "null argument");
        need((vgate == nullptr) == (vfirst == nullptr), "wkv7: vgate and vfirst come together");
        need(nseg >= 1 && T >= 1 && H >= 1, "wkv7: empty input");
        need(nseg * T * H * 64 <= 0x7fffffffLL && nseg * H * 64 <= 0x7fffffffLL && nseg <= 65535, "wkv7: input too large");
        select_device(device);
        const float* in[8] = {r, k, v, w, a, g, vgate, vfirst};
        const float* par[5] = {k_k, k_a, r_k, lnx_w, lnx_b};
        engine_op_wkv7(device, variant, (int)nseg, (int)T, (int)H, in, par, state, y);
    });
}
int rsv_op_argmax(int device, const float* logits, int64_t rows, int64_t V, uint32_t* out) {
    return guarded([&] {
        need(logits && out, "null argument");
        need(rows >= 1 && V >= 1, "argmax: empty input");
        select_device(device);
        DevBuf dl((size_t)rows * V * 4), dout((size_t)rows * 4);
        RSV_CUDA(cudaMemcpy(dl.p, logits, (size_t)rows * V * 4, cudaMemcpyHostToDevice));
        engine_argmax_raw(nullptr, (const float*)dl.p, (int)rows, (int)V, (uint32_t*)dout.p);
        RSV_CUDA(cudaMemcpy(out, dout.p, (size_t)rows * 4, cudaMemcpyDeviceToHost));
    });
}
int rsv_op_sample(int device, const float* logits, int64_t rows, int64_t V, const float* sampler8, const uint32_t* hist, int64_t hist_stride,
                  uint32_t* out) {
    return guarded([&] {
        need(logits && sampler8 && out, "null argument");
        need(rows >= 1 && V >= 1, "sample: empty input");
        need(hist_stride == 0 || hist, "history is null but hist_stride > 0");
        for (int64_t r = 0; r < rows; ++r) {
            uint32_t hl;
            memcpy(&hl, &sampler8[r * 8 + 7], 4);
            need((int64_t)hl <= hist_stride, "sample: hist_len exceeds hist_stride");
        }
        select_device(device);
        DevBuf dl((size_t)rows * V * 4), ds((size_t)rows * 32), dh((size_t)rows * hist_stride * 4), dt((size_t)rows * V * 4), dc((size_t)rows * V * 4),
            dout((size_t)rows * 4);
        RSV_CUDA(cudaMemcpy(dl.p, logits, (size_t)rows * V * 4, cudaMemcpyHostToDevice));
        RSV_CUDA(cudaMemcpy(ds.p, sampler8, (size_t)rows * 32, cudaMemcpyHostToDevice));
        if (hist_stride) RSV_CUDA(cudaMemcpy(dh.p, hist, (size_t)rows * hist_stride * 4, cudaMemcpyHostToDevice));
        engine_sample_raw(nullptr, (const float*)dl.p, (int)rows, (int)V, (const float*)ds.p, hist_stride ? (const uint32_t*)dh.p : nullptr,
                          (int)hist_stride, (float*)dt.p, (uint32_t*)dc.p, (uint32_t*)dout.p);
        RSV_CUDA(cudaMemcpy(out, dout.p, (size_t)rows * 4, cudaMemcpyDeviceToHost));
    });
}

}  // extern "C"
