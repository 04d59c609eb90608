// Continuous-batching scheduler: sessions arrive at any time, every step packs one ragged batch of rows —
// one decode row per generating session plus chunks of the prompts still being prefilled — and runs it through
// the packed forward step.  The reference has only static batching (all slots start and stop together,
// prompts padded to a common length; src/gpu_model.rs:868-1803, examples/batch_summarize.rs:270-370); this
// replaces that batch scheduling.  Results per session are those of the single-session API:
//   prompt consumed by chunked prefill; token r is drawn from the logits of the previous token with RNG seed
//   `sp.seed + r` and the r tokens generated so far as penalty history (arg-max when no sampler is given).
// The host only plans: which rows, which slots, which sampler rows.  Tokens of generating sessions never
// leave the GPU (a gather kernel feeds them back), steps are queued without host synchronisation, and the
// host reads a session's tokens once, when it has finished.
#include <algorithm>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "engine.hpp"
#include "rsv_b200.h"

using namespace rsv;

namespace rsv {
void set_last_error(const std::string& msg);
}
struct rsv_model {
    std::unique_ptr<Model> m;
};

namespace {

struct Request {
    int64_t id = 0;
    std::vector<uint32_t> prompt;
    int64_t max_new = 0;
    bool sample = false;
    rsv_sampler_params sp{};
    // progress
    int slot = -1;
    int64_t fed = 0;        // prompt tokens already given to the model
    int64_t generated = 0;  // tokens whose sampling has been queued
    bool done = false;
    std::vector<uint32_t> out;
};

}  // namespace

struct rsv_sched {
    Model* m = nullptr;
    State st;
    int max_slots = 0, chunk = 0, max_rows = 0, seq_cap = 0;
    // device-side per-slot arrays
    uint32_t* slot_tok = nullptr;  // last generated token
    uint32_t* slot_seq = nullptr;  // [max_slots, seq_cap] generated tokens
    int* slot_cnt = nullptr;       // tokens generated so far (= sampling round)
    float* slot_sampler = nullptr; // [max_slots, 8]
    uint32_t* host_tok_dev = nullptr;  // [max_rows] prompt tokens / 0xFFFFFFFF of the step being queued
    int* out_slot_dev = nullptr;       // [max_rows] slot of every logits row of the step
    static constexpr int kRing = 4;
    void* pinned = nullptr;            // ring of staging areas for the arrays above and new sampler rows
    size_t pinned_area = 0;
    cudaEvent_t pin_ev[kRing] = {nullptr, nullptr, nullptr, nullptr};
    int pin_next = 0;
    uint32_t* pinned_out = nullptr;    // [max_slots, seq_cap] finished sessions' tokens land here (async copy + event)
    std::vector<cudaEvent_t> out_ev;   // per slot
    std::vector<int64_t> retiring;     // per slot: session whose tokens are on their way to pinned_out (0 = none)
    std::deque<int64_t> waiting;
    std::map<int64_t, Request> reqs;
    std::vector<int> free_slots;
    std::vector<int64_t> slot_owner;
    std::deque<int64_t> finished;
    int64_t next_id = 1;
    int64_t steps = 0, rows_total = 0;

    ~rsv_sched() {
        if (m) cudaSetDevice(m->device);
        for (void* p : {(void*)slot_tok, (void*)slot_seq, (void*)slot_cnt, (void*)slot_sampler, (void*)host_tok_dev, (void*)out_slot_dev})
            if (p) cudaFree(p);
        if (pinned) cudaFreeHost(pinned);
        if (pinned_out) cudaFreeHost(pinned_out);
        for (auto e : pin_ev)
            if (e) cudaEventDestroy(e);
        for (auto e : out_ev)
            if (e) cudaEventDestroy(e);
    }
};

namespace {

template <class F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const CudaError& e) {
        set_last_error(e.what());
        return 2;
    } catch (const std::exception& e) {
        set_last_error(e.what());
        return 1;
    } catch (...) {
        set_last_error("unknown error");
        return 3;
    }
}
void need(bool c, const char* msg) {
    if (!c) throw std::runtime_error(msg);
}

void zero_slot(rsv_sched& S, int slot) {
    Model& m = *S.m;
    const Config& c = m.cfg;
    const size_t C = c.n_embd, HNN = (size_t)c.n_head * kHeadSize * kHeadSize;
    // one strided memset per state array: n_layer rows, one slot wide
    RSV_CUDA(cudaMemset2DAsync(S.st.tmix_x + (size_t)slot * C, (size_t)S.st.cap * C * 4, 0, C * 4, c.n_layer, m.stream));
    RSV_CUDA(cudaMemset2DAsync(S.st.cmix_x + (size_t)slot * C, (size_t)S.st.cap * C * 4, 0, C * 4, c.n_layer, m.stream));
    RSV_CUDA(cudaMemset2DAsync(S.st.wkv + (size_t)slot * HNN, (size_t)S.st.cap * HNN * 4, 0, HNN * 4, c.n_layer, m.stream));
    RSV_CUDA(cudaMemsetAsync(S.st.v_first + (size_t)slot * C, 0, C * 4, m.stream));
    RSV_CUDA(cudaMemsetAsync(S.slot_cnt + slot, 0, sizeof(int), m.stream));
}

void pack_row(float* row, const rsv_sampler_params& sp) {
    row[0] = sp.temperature;
    memcpy(&row[1], &sp.top_k, 4);
    row[2] = sp.top_p;
    memcpy(&row[3], &sp.seed, 4);
    row[4] = sp.repetition_penalty;
    row[5] = sp.frequency_penalty;
    row[6] = sp.presence_penalty;
    row[7] = 0.f;
}

// A session whose last token has been queued: copy its tokens out asynchronously and free the slot at once
// (stream order keeps the copy ahead of whatever reuses the slot).
void retire(rsv_sched& S, Request& r) {
    Model& m = *S.m;
    const int slot = r.slot;
    RSV_CUDA(cudaMemcpyAsync(S.pinned_out + (size_t)slot * S.seq_cap, S.slot_seq + (size_t)slot * S.seq_cap, (size_t)r.max_new * sizeof(uint32_t),
                             cudaMemcpyDeviceToHost, m.stream));
    RSV_CUDA(cudaEventRecord(S.out_ev[slot], m.stream));
    S.retiring[slot] = r.id;
    S.free_slots.push_back(slot);
    S.slot_owner[slot] = 0;
}
// Moves the tokens of retired sessions whose copy has completed into their request; `wait_slot` >= 0 blocks for that slot.
void harvest(rsv_sched& S, int wait_slot) {
    for (int s = 0; s < S.max_slots; ++s) {
        if (!S.retiring[s]) continue;
        cudaError_t q = (s == wait_slot) ? cudaEventSynchronize(S.out_ev[s]) : cudaEventQuery(S.out_ev[s]);
        if (q == cudaErrorNotReady) continue;
        if (q != cudaSuccess) throw CudaError(std::string("scheduler: waiting for a finished session failed: ") + cudaGetErrorString(q));
        Request& r = S.reqs.at(S.retiring[s]);
        r.out.assign(S.pinned_out + (size_t)s * S.seq_cap, S.pinned_out + (size_t)s * S.seq_cap + r.max_new);
        r.slot = -1;
        r.done = true;
        S.finished.push_back(r.id);
        S.retiring[s] = 0;
    }
}

}  // namespace

extern "C" {

int rsv_sched_new(rsv_model* mh, int64_t max_slots, int64_t chunk, int64_t max_rows, int64_t max_new_cap, rsv_sched** out) {
    return guarded([&] {
        need(mh && out, "null argument");
        need(max_slots >= 1 && chunk >= 1 && max_rows >= max_slots && max_new_cap >= 1, "sched_new: need max_slots >= 1, chunk >= 1, max_rows >= max_slots, max_new_cap >= 1");
        Model& m = *mh->m;
        RSV_CUDA(cudaSetDevice(m.device));
        auto S = std::make_unique<rsv_sched>();
        S->m = &m;
        S->max_slots = (int)max_slots;
        S->chunk = (int)chunk;
        S->max_rows = (int)max_rows;
        S->seq_cap = (int)max_new_cap;
        State& st = S->st;
        st.model = &m;
        st.cap = max_slots;
        const Config& c = m.cfg;
        const size_t nx = (size_t)c.n_layer * max_slots * c.n_embd, ns = (size_t)c.n_layer * max_slots * c.n_head * kHeadSize * kHeadSize;
        RSV_CUDA(cudaMalloc(&st.tmix_x, nx * 4));
        RSV_CUDA(cudaMalloc(&st.cmix_x, nx * 4));
        RSV_CUDA(cudaMalloc(&st.wkv, ns * 4));
        RSV_CUDA(cudaMalloc(&st.v_first, (size_t)max_slots * c.n_embd * 4));
        RSV_CUDA(cudaMalloc(&S->slot_tok, (size_t)max_slots * 4));
        RSV_CUDA(cudaMalloc(&S->slot_seq, (size_t)max_slots * max_new_cap * 4));
        RSV_CUDA(cudaMalloc(&S->slot_cnt, (size_t)max_slots * 4));
        RSV_CUDA(cudaMalloc(&S->slot_sampler, (size_t)max_slots * 32));
        RSV_CUDA(cudaMalloc(&S->host_tok_dev, (size_t)max_rows * 4));
        RSV_CUDA(cudaMalloc(&S->out_slot_dev, (size_t)max_rows * 4));
        S->pinned_area = (size_t)max_rows * 8 + (size_t)max_slots * 32;
        RSV_CUDA(cudaMallocHost(&S->pinned, S->pinned_area * rsv_sched::kRing));
        for (auto& e : S->pin_ev) RSV_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        RSV_CUDA(cudaMallocHost(&S->pinned_out, (size_t)max_slots * max_new_cap * 4));
        S->out_ev.resize((size_t)max_slots, nullptr);
        for (auto& e : S->out_ev) RSV_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        S->retiring.assign((size_t)max_slots, 0);
        m.ensure_workspace((int)max_rows, (int)max_slots, (int)max_slots);  // the largest step, so that no step reallocates
        RSV_CUDA(cudaMemsetAsync(S->slot_tok, 0, (size_t)max_slots * 4, m.stream));
        RSV_CUDA(cudaMemsetAsync(S->slot_cnt, 0, (size_t)max_slots * 4, m.stream));
        RSV_CUDA(cudaStreamSynchronize(m.stream));
        S->slot_owner.assign((size_t)max_slots, 0);
        for (int s = (int)max_slots - 1; s >= 0; --s) S->free_slots.push_back(s);
        *out = S.release();
    });
}
void rsv_sched_free(rsv_sched* s) { delete s; }

int rsv_sched_submit(rsv_sched* S, const uint32_t* prompt, int64_t n_prompt, int64_t max_new, const rsv_sampler_params* sp, int64_t* id_out) {
    return guarded([&] {
        need(S && prompt && id_out, "null argument");
        need(n_prompt >= 1, "sched_submit: empty prompt");
        need(max_new >= 1 && max_new <= S->seq_cap, "sched_submit: max_new must be in [1, max_new_cap]");
        for (int64_t i = 0; i < n_prompt; ++i)
            if (prompt[i] >= (uint32_t)S->m->cfg.vocab) throw std::runtime_error("sched_submit: token id " + std::to_string(prompt[i]) + " is >= vocab");
        Request r;
        r.id = S->next_id++;
        r.prompt.assign(prompt, prompt + n_prompt);
        r.max_new = max_new;
        r.sample = sp != nullptr;
        if (sp) r.sp = *sp;
        *id_out = r.id;
        S->waiting.push_back(r.id);
        S->reqs.emplace(r.id, std::move(r));
    });
}

// Queues one packed step.  rows_out = rows in the step (0: nothing to do), active_out = sessions holding a slot after it.
int rsv_sched_step(rsv_sched* Sp, int64_t* rows_out, int64_t* active_out) {
    return guarded([&] {
        need(Sp, "null argument");
        rsv_sched& S = *Sp;
        Model& m = *S.m;
        RSV_CUDA(cudaSetDevice(m.device));
        // admission: a free slot per waiting request, state zeroed on the stream
        std::vector<std::pair<int, const rsv_sampler_params*>> new_rows;
        while (!S.waiting.empty() && !S.free_slots.empty()) {
            Request& r = S.reqs.at(S.waiting.front());
            S.waiting.pop_front();
            r.slot = S.free_slots.back();
            S.free_slots.pop_back();
            if (S.retiring[r.slot]) harvest(S, r.slot);  // the slot's previous tokens must have left its pinned area
            S.slot_owner[r.slot] = r.id;
            zero_slot(S, r.slot);
            if (!r.sample) {  // arg-max as a sampler row: keep only the largest logit
                r.sp = rsv_sampler_params{1.0f, 1u, 1.0f, 0u, 1.0f, 0.0f, 0.0f};
            }
            new_rows.emplace_back(r.slot, &r.sp);
        }
        // plan: decode rows first (one per generating session), then prompt chunks while rows remain
        StepPlan p;
        std::vector<uint32_t> host_tok;
        std::vector<int> out_slot;
        std::vector<int64_t> sampled_ids;
        bool any_sample = false;
        auto add_segment = [&](Request& r, int T, const uint32_t* toks, bool wants_logits) {
            const int start = (int)p.rows.size(), seg = (int)p.segs.size();
            for (int i = 0; i < T; ++i) {
                p.rows.push_back(RowMeta{r.slot, i > 0 ? 1 : 0, i == T - 1 ? 1 : 0, seg});
                host_tok.push_back(toks ? toks[i] : 0xFFFFFFFFu);
            }
            p.segs.push_back(SegMeta{start, T, r.slot, 0});
            if (T > 1) p.multi_row_segments = true;
            if (wants_logits) {
                p.out_rows.push_back(start + T - 1);
                out_slot.push_back(r.slot);
                sampled_ids.push_back(r.id);
                if (r.sample) any_sample = true;
            }
        };
        for (int s = 0; s < S.max_slots; ++s) {
            if (!S.slot_owner[s]) continue;
            Request& r = S.reqs.at(S.slot_owner[s]);
            if (r.fed == (int64_t)r.prompt.size() && r.generated < r.max_new) add_segment(r, 1, nullptr, true);
        }
        for (int s = 0; s < S.max_slots && (int)p.rows.size() < S.max_rows; ++s) {
            if (!S.slot_owner[s]) continue;
            Request& r = S.reqs.at(S.slot_owner[s]);
            const int64_t rem = (int64_t)r.prompt.size() - r.fed;
            if (rem <= 0) continue;
            const int T = (int)std::min<int64_t>({rem, (int64_t)S.chunk, (int64_t)S.max_rows - (int64_t)p.rows.size()});
            if (T <= 0) break;
            add_segment(r, T, r.prompt.data() + r.fed, r.fed + T == (int64_t)r.prompt.size());
            r.fed += T;
        }
        const int R = (int)p.rows.size(), O = (int)p.out_rows.size();
        if (rows_out) *rows_out = R;
        if (R > 0) {
            m.upload_plan(p);
            const int area = S.pin_next;
            S.pin_next = (S.pin_next + 1) % rsv_sched::kRing;
            RSV_CUDA(cudaEventSynchronize(S.pin_ev[area]));  // copies queued from this area kRing steps ago have long completed
            char* pin = (char*)S.pinned + (size_t)area * S.pinned_area;
            memcpy(pin, host_tok.data(), (size_t)R * 4);
            RSV_CUDA(cudaMemcpyAsync(S.host_tok_dev, pin, (size_t)R * 4, cudaMemcpyHostToDevice, m.stream));
            if (O) {
                memcpy(pin + (size_t)S.max_rows * 4, out_slot.data(), (size_t)O * 4);
                RSV_CUDA(cudaMemcpyAsync(S.out_slot_dev, pin + (size_t)S.max_rows * 4, (size_t)O * 4, cudaMemcpyHostToDevice, m.stream));
            }
            float* srows = (float*)(pin + (size_t)S.max_rows * 8);
            for (size_t i = 0; i < new_rows.size(); ++i) {
                pack_row(srows + i * 8, *new_rows[i].second);
                RSV_CUDA(cudaMemcpyAsync(S.slot_sampler + (size_t)new_rows[i].first * 8, srows + i * 8, 32, cudaMemcpyHostToDevice, m.stream));
            }
            RSV_CUDA(cudaEventRecord(S.pin_ev[area], m.stream));
            engine_merge_tokens(m, S.host_tok_dev, S.slot_tok, R);
            if (R == O && R <= 4 && !p.multi_row_segments && !m.prof_on && m.persistent_available(R)) {
                // a few decoding sessions and nothing else (the tail of a workload): one launch of the persistent decode kernel
                int slots[4] = {0, 0, 0, 0};
                for (int i = 0; i < R; ++i) slots[i] = p.rows[i].slot;
                m.run_persistent(S.st, R, slots, 1, false, false, nullptr, nullptr, 0);
            } else {
                m.forward_rows(S.st, p, false);
            }
            if (O) {
                // a step whose sessions all asked for arg-max uses the arg-max kernel (ties -> smaller id); any other step
                // goes through the sampler, where arg-max sessions carry a top_k = 1 row
                if (!any_sample)
                    engine_argmax(m, m.ws.logits, O, S.slot_tok, S.slot_seq, S.slot_cnt, S.seq_cap, S.out_slot_dev);
                else
                    engine_sample(m, m.ws.logits, O, S.slot_sampler, S.slot_seq, S.seq_cap, S.slot_cnt, S.slot_tok, S.slot_seq, S.slot_cnt, S.seq_cap,
                                  S.out_slot_dev);
            }
            for (int64_t id : sampled_ids) {
                Request& r = S.reqs.at(id);
                r.generated += 1;
            }
            S.steps += 1;
            S.rows_total += R;
        }
        // sessions whose last token has just been queued are complete
        for (int s = 0; s < S.max_slots; ++s) {
            if (!S.slot_owner[s]) continue;
            Request& r = S.reqs.at(S.slot_owner[s]);
            if (r.generated >= r.max_new) retire(S, r);
        }
        harvest(S, -1);
        if (active_out) {
            int64_t a = 0;
            for (int s = 0; s < S.max_slots; ++s) a += S.slot_owner[s] != 0;
            for (int s = 0; s < S.max_slots; ++s) a += S.retiring[s] != 0;
            *active_out = a + (int64_t)S.waiting.size();
        }
    });
}

// Ids of sessions that finished since the last poll.
int rsv_sched_poll(rsv_sched* S, int64_t* ids, int64_t cap, int64_t* n_out) {
    return guarded([&] {
        need(S && ids && n_out, "null argument");
        harvest(*S, -1);
        int64_t n = 0;
        while (n < cap && !S->finished.empty()) {
            ids[n++] = S->finished.front();
            S->finished.pop_front();
        }
        *n_out = n;
    });
}

// Generated tokens of a finished session (and forgets the session).
int rsv_sched_result(rsv_sched* S, int64_t id, uint32_t* out, int64_t cap, int64_t* n_out) {
    return guarded([&] {
        need(S && out && n_out, "null argument");
        auto it = S->reqs.find(id);
        need(it != S->reqs.end(), "sched_result: unknown session id");
        need(it->second.done, "sched_result: session has not finished");
        need((int64_t)it->second.out.size() <= cap, "sched_result: output buffer too small");
        std::copy(it->second.out.begin(), it->second.out.end(), out);
        *n_out = (int64_t)it->second.out.size();
        S->reqs.erase(it);
    });
}

// Blocks until everything queued so far has run; reports device-side errors (bad token ids, timeouts).
int rsv_sched_sync(rsv_sched* S) {
    return guarded([&] {
        need(S, "null argument");
        S->m->check_status();
        harvest(*S, -1);
    });
}

int rsv_sched_stats(rsv_sched* S, int64_t* steps, int64_t* rows) {
    return guarded([&] {
        need(S && steps && rows, "null argument");
        *steps = S->steps;
        *rows = S->rows_total;
    });
}

}  // extern "C"
