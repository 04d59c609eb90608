// Host-side engine: weights in HBM, session state, work buffers and the forward step over packed rows.
// Replaces, for the batched RWKV-7 forward step, the reference's GpuModel dispatch graph
// (src/gpu_model.rs:401-546, 868-1803, 1968-2543, 2911-3568) and its CudaBackend
// (src/backend_cuda.rs).  One host thread drives one Model; all work goes to the model's stream.
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>

#include <cuda.h>

#include "common.cuh"

namespace rsv {

struct Config {
    int n_layer = 0, n_embd = 0, vocab = 0, head_size = 0, n_head = 0, ffn_hidden = 0;
    int w_mid = 0, a_mid = 0, v_mid = 0, g_mid = 0;
    int mids() const { return w_mid + a_mid + v_mid + g_mid; }
    size_t state_floats_per_slot() const {
        return (size_t)n_layer * (2 * (size_t)n_embd + (size_t)n_head * head_size * head_size) + (size_t)n_embd;
    }
};

// One weight matrix in HBM, row-major [M,K] = [out,in] exactly as stored in the checkpoint.
struct LinearW {
    int M = 0, K = 0, wtype = W_F16;
    void* w = nullptr;         // fp16 [M,K] or u8 [M,K]
    uint32_t* sz = nullptr;    // int8: [M,K/128] (fp16 scale | fp16 zero << 16), the reference container
    size_t bytes() const { return wtype == W_INT8 ? (size_t)M * K + (size_t)M * (K / 128) * 4 : (size_t)M * K * 2; }
    // tensor-core path (tcgen05): A operand = the same bytes (or a zero-padded copy when M % 128 or the K pitch
    // does not fit), one (scale, zero) pair per output row for int8, and the TMA descriptor of the A operand
    bool tc_ok = false;
    int Mpad = 0, Kpad = 0;
    void* w_tc = nullptr;
    float *wscale = nullptr, *wzero = nullptr;
    CUtensorMap amap;
};

struct LayerW {
    float *ln1_w, *ln1_b, *ln2_w, *ln2_b, *lnx_w, *lnx_b;
    float *x_r, *x_w, *x_k, *x_v, *x_a, *x_g, *ffn_x_k;
    float *w0, *a0, *v0, *r_k, *k_k, *k_a;
    LinearW Wr, Wk, Wv, Wo, Wfk, Wfv;
    LinearW w1, a1, v1, g1;  // rank-space projections, stored [mid, C] fp16
    LinearW w2, a2, v2, g2;  // back-projections, stored [C, mid] fp16
};

struct Workspace {
    int rows = 0, outs = 0, segs = 0;  // capacities
    const float *final_x = nullptr, *final_delta = nullptr;  // after forward_rows: the last layer's residual stream of row i is final_x[i] + final_delta[i]
    float *x = nullptr, *x2 = nullptr, *delta = nullptr, *xmix = nullptr, *r = nullptr, *k = nullptr, *v = nullptr, *w = nullptr, *a = nullptr, *g = nullptr;
    float *yg = nullptr, *xb = nullptr, *mid = nullptr, *h = nullptr, *vfirst = nullptr, *xn = nullptr, *logits = nullptr, *staging = nullptr;
    // tensor-core linear path: B operands, per-row scales, fixed-point sums, split-K partials (grown on demand)
    uint8_t* tc_b = nullptr;
    size_t tc_b_bytes = 0;
    float* tc_xscale = nullptr;
    long long* tc_tsum = nullptr;
    size_t tc_rows = 0;
    void* tc_partials = nullptr;
    int* tc_cnt = nullptr;
    size_t tc_partials_bytes = 0;
    float* samp_temp = nullptr;      // [outs, V] sampler work area
    uint32_t* samp_cnt = nullptr;    // [outs, V] penalty histogram
    uint32_t* tokens = nullptr;    // [rows] input token of every row (device-resident between self-loop rounds)
    uint32_t* tok_list = nullptr;  // token cursor mode: [tok_list_cap]
    size_t tok_list_cap = 0;
    RowMeta* row_meta = nullptr;
    SegMeta* seg_meta = nullptr;
    int* out_rows = nullptr;
    int* status = nullptr;   // bit 0: token id out of range
    int* tok_pos = nullptr;  // cursor into tok_list
};

// Device-side tables and scratch of the persistent decode kernel (built on first use).
struct PersistentCtx {
    bool tried = false, ok = false;
    std::string why;            // reason when the model cannot take the persistent path
    void* d_layers = nullptr;   // DpLayer[L]
    void* d_maps = nullptr;     // CUtensorMap[]
    float *x = nullptr, *yg = nullptr, *vfirst = nullptr, *cand_val = nullptr;
    int* cand_idx = nullptr;
    unsigned* grid_bar = nullptr;
    long long* dbg = nullptr;  // builds with -DRSV_DP_DEBUG: phase time stamps of the persistent kernel
    void* region_data[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    void* region_meta[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    int* region_cnt[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    size_t region_cnt_bytes[5] = {0, 0, 0, 0, 0};
    float *rkv = nullptr, *mid = nullptr, *hbuf = nullptr;
    int region_pmax[5] = {1, 1, 1, 1, 1};
    int grid = 0, nstages = 0, btiles = 0;
    size_t smem = 0;
    std::vector<char> params_template;  // DpParams with everything but the per-call fields
    const float *bound_tmix = nullptr, *bound_wkv = nullptr, *bound_cmix = nullptr;  // state whose pointers the device layer table holds
    int64_t bound_cap = -1;                                                           // and its slot capacity (the per-layer strides)
};

// Device-side tables and scratch of the batch-1 weight-streaming decode kernel (built on first use).
struct StreamCtx {
    bool tried = false, ok = false;
    std::string why;           // reason when the model cannot take this path
    void* d_layers = nullptr;  // DsLayer[L]
    void *wstream = nullptr, *hstream = nullptr;  // second copy of the weights in the order the kernel consumes them
    long long wslot = 0, hslot = 0;
    float *x = nullptr, *yg = nullptr, *vfirst = nullptr, *rkv = nullptr, *mid = nullptr, *hbuf = nullptr, *cand_val = nullptr;
    int* cand_idx = nullptr;
    unsigned* grid_bar = nullptr;
    long long* dbg = nullptr;
    int grid = 0, kl = 0, ring_bytes = 0, vec_floats = 0;
    size_t smem = 0;
    std::vector<char> params_template;  // DsParams with everything but the per-call fields
};

struct KernelProf {
    double ms = 0;
    long launches = 0;
};

struct Model;

// Session state: per layer tmix_x[cap,C], wkv[cap,H,N,N], cmix_x[cap,C], plus v_first[cap,C]
// (src/gpu_model.rs:194-199, 3915-3963).  fp32 on the device, so back/load round-trips bit-exactly.
struct State {
    Model* model = nullptr;
    int64_t cap = 0;
    float *tmix_x = nullptr, *wkv = nullptr, *cmix_x = nullptr, *v_first = nullptr;
    CUtensorMap wkv_map;      // all layers' WKV states as one 2-D tensor [layers x slots x heads x 64][64] fp32 (TMA boxes of 64 rows x 32 columns)
    bool wkv_map_ok = false;  // encoded on first use
    ~State();
};

// A packed step: R rows grouped into segments (one per session present in the step).
struct StepPlan {
    std::vector<RowMeta> rows;
    std::vector<SegMeta> segs;
    std::vector<int> out_rows;  // rows whose logits are wanted (may be empty)
    bool multi_row_segments = false;
};

enum class PostOp { None, Argmax };

struct Model {
    int device = 0;
    cudaStream_t stream = nullptr;
    Config cfg;
    __half* emb = nullptr;
    float *ln0_w = nullptr, *ln0_b = nullptr, *ln_out_w = nullptr, *ln_out_b = nullptr;
    LinearW head;
    std::vector<LayerW> layers;
    std::vector<void*> allocs;  // every weight allocation, freed in the destructor
    size_t weight_bytes = 0;
    Workspace ws;
    // pinned staging for per-step metadata: a ring of kPinRing areas, each guarded by an event, so that queuing a step
    // never waits for the previous one
    static constexpr int kPinRing = 4;
    void* pinned = nullptr;
    size_t pinned_bytes = 0;  // bytes per ring area
    cudaEvent_t pin_ev[kPinRing] = {nullptr, nullptr, nullptr, nullptr};
    int pin_next = 0;
    // profiling (clear_kernel_prof / dump_kernel_prof of the reference, src/gpu_model.rs:561-570)
    bool prof_on = false;
    std::map<std::string, KernelProf> prof;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr, tev[2] = {nullptr, nullptr};
    long launches = 0;  // kernels launched since the counter was last cleared
    int num_sms = 148;
    bool use_pdl = true;     // launch the per-layer kernels of the batched path as programmatic dependents (RSV_NO_PDL=1 disables)
    bool use_graphs = true;  // replay self-loop rounds from a captured CUDA graph (RSV_NO_GRAPH=1 disables)
    int tc_min_rows = 5;  // packed steps with at least this many rows use the tensor-core linear path

    bool use_persistent = true;  // batch <= 4 decode goes through the persistent kernel (RSV_NO_PERSISTENT=1 disables)
    PersistentCtx pctx;
    bool use_stream = true;  // one session: the row-owner weight-streaming kernel (RSV_NO_STREAM=1 falls back to the tensor-core persistent kernel)
    StreamCtx sctx;
    bool stream_available();
    void run_stream(State& st, int slot, int n_tokens, bool tok_from_list, bool argmax_feed, uint32_t* seq_dev, int* seq_cnt_dev, int seq_cap);
    // Persistent decode: n_tokens steps for nb <= 4 sessions (slots[b] of `st`) in one cooperative launch.
    // Returns false (with pctx.why set) when this model cannot take that path.
    bool persistent_available(int nb);
    void run_persistent(State& st, int nb, const int* slots, int n_tokens, bool tok_from_list, bool argmax_feed, uint32_t* seq_dev, int* seq_cnt_dev,
                        int seq_cap);

    static std::unique_ptr<Model> create_bare(int device);  // stream + events only (operator-level entry points)

    static std::unique_ptr<Model> load(const std::string& path, int device);
    ~Model();

    void ensure_workspace(int rows, int outs, int segs);
    void upload_plan(const StepPlan& plan);
    // Runs one packed step.  Input tokens are read from ws.tokens[r] (or ws.tok_list[*tok_pos * R + r] when
    // `use_cursor`).  With out_rows non-empty, logits land in ws.logits[o, V] in out_rows order.
    void forward_rows(State& st, const StepPlan& plan, bool use_cursor);
    void check_status();
};

// Device-side products of a queued self-loop (SelfloopTicket, src/gpu_model.rs:204-212).
struct Ticket {
    Model* model = nullptr;
    int64_t batch = 0, n = 0;
    uint32_t* seq = nullptr;   // [batch, n] generated tokens
    int* cnt = nullptr;        // [batch] tokens generated so far per slot
    float* sampler = nullptr;  // [batch, 8] sampler rows (null for arg-max)
    cudaGraph_t graph = nullptr;  // captured step, alive until the queued replays have been collected
    cudaGraphExec_t graph_exec = nullptr;
    ~Ticket();
};

// launch wrappers defined next to the kernels
// `row_map_dev` (optional): logits row r belongs to entry row_map[r] of the per-session arrays
void engine_argmax(Model& m, const float* logits_dev, int rows, uint32_t* next_tok_dev, uint32_t* seq_dev, int* seq_cnt_dev, int seq_cap,
                   const int* row_map_dev = nullptr);
void engine_sample(Model& m, const float* logits_dev, int rows, const float* sampler8_dev, const uint32_t* hist_dev, int hist_stride,
                   const int* round_cnt_dev, uint32_t* next_tok_dev, uint32_t* seq_dev, int* seq_cnt_dev, int seq_cap, const int* row_map_dev = nullptr);
// ws.tokens[r] = host_tok[r], or slot_tok[slot of row r] where host_tok[r] == 0xFFFFFFFF (rows as last uploaded with upload_plan)
void engine_merge_tokens(Model& m, const uint32_t* host_tok_dev, const uint32_t* slot_tok_dev, int R);
void engine_argmax_raw(cudaStream_t stream, const float* logits_dev, int rows, int V, uint32_t* out_dev);
void engine_sample_raw(cudaStream_t stream, const float* logits_dev, int rows, int V, const float* sampler8_dev, const uint32_t* hist_dev,
                       int hist_stride, float* temp_dev, uint32_t* counter_dev, uint32_t* out_dev);
// Operator-level linear layer on host data: y[R,M] = x[R,K] . W[M,K]^T.  path 0 = SIMT kernel, 1 = tcgen05 kernel.
void engine_op_linear(Model& m, int path, int wtype, const void* w_host, const uint32_t* sz_host, int M, int K, const float* x_host, int R,
                      float* y_host);
// Operator-level WKV-7 step of one layer on host data: nseg sessions x T tokens, rows session-major.  in[] = r, k, v, w (decay), a, g,
// vgate, vfirst ([nseg T, H 64] each; the last two null for the first layer); par[] = k_k, k_a, r_k, lnx_w, lnx_b ([H 64]);
// state [nseg, H, 64, 64] is updated in place; y = (GroupNorm(S r) + (r . k~ r_k) v) g.  variant: 0 automatic, 1-4 one kernel each.
void engine_op_wkv7(int device, int variant, int nseg, int T, int H, const float* const in[8], const float* const par[5], float* state_host, float* y_host);
// acc[slot of segment][c] += sum over the segment's rows, in row order, of the last layer's residual stream left by forward_rows
void engine_segment_sums(Model& m, int n_segments, float* acc_dev);
void engine_quantize_int8(cudaStream_t stream, const float* w_dev, size_t M, size_t K, uint8_t* idx_dev, uint32_t* sz_dev);
void engine_dequant_int8(cudaStream_t stream, const uint8_t* idx_dev, const uint32_t* sz_dev, size_t M, size_t K, float* out_dev);

}  // namespace rsv
