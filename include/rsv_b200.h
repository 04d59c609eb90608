/* C ABI of the B200-native RWKV-7 forward step.
 *
 * This is the drop-in boundary for the reference's library API (`ModelBuilder` / `Bundle` / `State` /
 * `SamplerParams`, src/gpu_model.rs) — the functions a Rust `Bundle` shim would bind through
 * `extern "C"`.  Each entry point names the reference method it replaces.
 *
 * Conventions
 *   - every function returns 0 on success and a non-zero code on failure; `rsv_last_error()` then
 *     returns a thread-local message (the reference returns `Result<_, Box<dyn Error>>` strings,
 *     src/runtime.rs:18, src/backend_cuda.rs:23-30);
 *   - all buffers are caller-allocated host memory with explicit element counts; a length that does
 *     not match is an error (as State::load, src/gpu_model.rs:4001-4005);
 *   - one host thread per model handle; all GPU work is issued on the handle's own stream;
 *   - there is no CPU fallback: loading fails when no sm_100 device is present.
 */
#ifndef RSV_B200_H
#define RSV_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rsv_model rsv_model;   /* GpuModel: weights in HBM + work buffers (src/gpu_model.rs:401) */
typedef struct rsv_state rsv_state;   /* State (src/gpu_model.rs:3920) */
typedef struct rsv_ticket rsv_ticket; /* SelfloopTicket (src/gpu_model.rs:204-212) */

/* ModelInfo (src/gpu_model.rs:75-99).  version: 7 = ModelVersion::V7. */
typedef struct {
    int32_t version;
    int64_t num_layer, num_emb, num_hidden, num_vocab, num_head, head_size, ffn_hidden;
    int64_t w_mid, a_mid, v_mid, g_mid;
} rsv_model_info;

/* SamplerParams (src/gpu_model.rs:3883-3913).  Defaults: 1.0, 0, 1.0, 0, 1.0, 0.0, 0.0. */
typedef struct {
    float temperature;
    uint32_t top_k;
    float top_p;
    uint32_t seed;
    float repetition_penalty;
    float frequency_penalty;
    float presence_penalty;
} rsv_sampler_params;

const char* rsv_last_error(void);

/* ---- model ----------------------------------------------------------------------------------- */
/* ModelBuilder::new(path).build() / GpuModel::from_safetensors (src/gpu_model.rs:3691-3703, 401-546).
 * fp16 / int8 routing is per tensor, on the presence of `{key}.int8_idx`. */
int rsv_model_load(const char* path, int device, rsv_model** out);
void rsv_model_free(rsv_model* m);
/* Bundle::info (src/gpu_model.rs:3723). */
int rsv_model_info_get(const rsv_model* m, rsv_model_info* out);
/* Bytes of weights resident in HBM (for roofline accounting). */
int64_t rsv_model_weight_bytes(const rsv_model* m);

/* ---- state ----------------------------------------------------------------------------------- */
/* GpuModel::create_state / create_batch_state (src/gpu_model.rs:584, 871): zero-initialised. */
int rsv_state_new(rsv_model* m, int64_t batch, rsv_state** out);
void rsv_state_free(rsv_state* s);
/* State::batch (src/gpu_model.rs:3966). */
int64_t rsv_state_batch(const rsv_state* s);
/* Number of f32 in the whole state: batch * (L*(2C + H*N*N) + C). */
int64_t rsv_state_len(const rsv_state* s);
/* State::back / Bundle::state_back (src/gpu_model.rs:3972-3990, 3749): per slot, per layer
 * tmix_x[C] | tmix_rnn[H][N][N] | cmix_x[C], then v_first[C]; slots concatenated. */
int rsv_state_back(rsv_state* s, float* out, int64_t len);
/* State::load / Bundle::state_load (src/gpu_model.rs:3993-4035, 3754). */
int rsv_state_load(rsv_state* s, const float* data, int64_t len);
/* State::slot_back / slot_load (src/gpu_model.rs:4038-4095, 884-905). */
int rsv_state_slot_back(rsv_state* s, int64_t slot, float* out, int64_t len);
int rsv_state_slot_load(rsv_state* s, int64_t slot, const float* data, int64_t len);
/* State files: the f32 array of State::back as raw little-endian bytes, no header - the file the reference's
 * examples/state_persist.rs:38-47 writes with std::fs::write(bytemuck::cast_slice(&state)) and reads back into
 * Bundle::state_load.  save writes to "<path>.part" and renames; restore refuses a file whose size is not exactly
 * rsv_state_len (one slot's length for the slot variants) f32 and leaves the state untouched in that case. */
int rsv_state_save(rsv_state* s, const char* path);
int rsv_state_restore(rsv_state* s, const char* path);
int rsv_state_slot_save(rsv_state* s, int64_t slot, const char* path);
int rsv_state_slot_restore(rsv_state* s, int64_t slot, const char* path);
/* Session migration: slot src_slot of src -> slot dst_slot of dst, device to device, bit for bit (State::slot_back on one
 * state followed by State::slot_load on the other, src/gpu_model.rs:4038-4095, without the host round trip).  The states may
 * belong to different model handles, on one GPU or two; the model shapes must agree. */
int rsv_state_slot_copy(rsv_state* dst, int64_t dst_slot, rsv_state* src, int64_t src_slot);
/* State::reset / Bundle::reset (src/gpu_model.rs:4098-4104, 3759). */
int rsv_state_reset(rsv_state* s);

/* ---- single-session inference (state must have batch == 1) ----------------------------------- */
/* Bundle::infer_tokens (src/gpu_model.rs:3729): token-by-token decode path; logits_out[V] of the last token. */
int rsv_infer_tokens(rsv_model* m, rsv_state* s, const uint32_t* tokens, int64_t n, float* logits_out);
/* Bundle::infer_seq (src/gpu_model.rs:3734): all tokens advance through each layer together. */
int rsv_infer_seq(rsv_model* m, rsv_state* s, const uint32_t* tokens, int64_t n, float* logits_out);
/* Bundle::infer with RnnOption::Last / infer_chunked (src/gpu_model.rs:3774-3805). */
int rsv_infer_chunked(rsv_model* m, rsv_state* s, const uint32_t* tokens, int64_t n, int64_t chunk_size, float* logits_out);
/* Bundle::infer with RnnOption::Full (src/gpu_model.rs:3786-3793): logits_out[n*V], one row per position. */
int rsv_infer_full(rsv_model* m, rsv_state* s, const uint32_t* tokens, int64_t n, float* logits_out);
/* Bundle::infer_argmax (src/gpu_model.rs:3809): arg-max of the last token's logits, ties to the smaller id. */
int rsv_infer_argmax(rsv_model* m, rsv_state* s, const uint32_t* tokens, int64_t n, uint32_t* token_out);
/* Bundle::infer_argmax_selfloop (src/gpu_model.rs:3818): `seed` is the first INPUT token; out[n]. */
int rsv_infer_argmax_selfloop(rsv_model* m, rsv_state* s, uint32_t seed, int64_t n, uint32_t* out);
/* Bundle::infer_sample (src/gpu_model.rs:3826): history[nh] feeds the penalties. */
int rsv_infer_sample(rsv_model* m, rsv_state* s, const uint32_t* tokens, int64_t n, const rsv_sampler_params* sp, const uint32_t* history,
                     int64_t nh, uint32_t* token_out);
/* Bundle::infer_sample_selfloop (src/gpu_model.rs:3834): RNG seed of round r is `seed + r`, history = the r tokens
 * generated so far (src/gpu_model.rs:790-810). */
int rsv_infer_sample_selfloop(rsv_model* m, rsv_state* s, uint32_t seed, int64_t n, const rsv_sampler_params* sp, uint32_t* out);

/* ---- batched sessions (state batch == number of slots) --------------------------------------- */
/* GpuModel::forward_seq_batch (src/gpu_model.rs:1001-1011): slot b consumes flat[b*t_pad .. b*t_pad+lens[b]).
 * Ragged: only real tokens become rows (the reference pads to t_pad).  seeds_out[b] = last token of slot b. */
int rsv_prefill_batch(rsv_model* m, rsv_state* s, const uint32_t* flat, const uint32_t* lens, int64_t batch, int64_t t_pad, uint32_t* seeds_out);
/* GpuModel::forward_seq_batch_mean_hidden (src/gpu_model.rs:1013-1036) with rwkv_segmean (src/backend_cuda.rs:4412-4431): the
 * state is reset, the prompts are prefilled as above, and mean_out[batch * n_embd] receives per slot the mean over its lens[b]
 * tokens of the last layer's residual stream (before ln_out), accumulated in token order - the router feature. */
int rsv_prefill_batch_mean_hidden(rsv_model* m, rsv_state* s, const uint32_t* flat, const uint32_t* lens, int64_t batch, int64_t t_pad, float* mean_out);
/* GpuModel::submit_sample_selfloop(_batch) (src/gpu_model.rs:732-852, 1639-1781): queues n rounds for `batch`
 * slots without a host round-trip; seeds[b] is slot b's first input token and the base of its RNG seed.
 * sp == NULL selects arg-max instead of sampling. */
int rsv_sample_selfloop_submit(rsv_model* m, rsv_state* s, const uint32_t* seeds, int64_t batch, int64_t n, const rsv_sampler_params* sp,
                               rsv_ticket** out);
/* GpuModel::collect_sample_selfloop(_batch) (src/gpu_model.rs:856-866, 1784-1802): waits, copies out[batch*n]
 * (slot-major) and frees the ticket. */
int rsv_sample_selfloop_collect(rsv_ticket* t, uint32_t* out, int64_t len);

/* ---- continuous batching ----------------------------------------------------------------------
 * No counterpart in the reference, whose batching is static (fixed batch, prompts padded to a common length, all slots
 * decode the same number of steps; src/gpu_model.rs:868-1803, examples/batch_summarize.rs:270-370).  Sessions are submitted
 * at any time; each rsv_sched_step packs one ragged step — a decode row per generating session plus prompt chunks of at most
 * `chunk` tokens — and queues it on the model's stream without waiting for it.  Per session the result equals the
 * single-session API: the prompt is prefilled, then token r is sampled from the previous token's logits with RNG seed
 * sp->seed + r and the r tokens generated so far as penalty history (sp == NULL: arg-max). */
typedef struct rsv_sched rsv_sched;
/* max_slots: concurrent sessions (state slots); chunk: prompt tokens of one session per step; max_rows: rows per step
 * (>= max_slots); max_new_cap: upper bound on max_new of any session.  The model's step workspace is sized for max_rows rows
 * here, so that no step allocates. */
int rsv_sched_new(rsv_model* m, int64_t max_slots, int64_t chunk, int64_t max_rows, int64_t max_new_cap, rsv_sched** out);
void rsv_sched_free(rsv_sched* s);
int rsv_sched_submit(rsv_sched* s, const uint32_t* prompt, int64_t n_prompt, int64_t max_new, const rsv_sampler_params* sp, int64_t* id_out);
/* Queues one step.  rows_out: rows packed into it (0 = nothing to do); active_out: sessions not yet finished. */
int rsv_sched_step(rsv_sched* s, int64_t* rows_out, int64_t* active_out);
/* Ids of sessions whose tokens have reached the host since the last poll (never blocks). */
int rsv_sched_poll(rsv_sched* s, int64_t* ids, int64_t cap, int64_t* n_out);
/* Generated tokens of a finished session; the session is forgotten afterwards. */
int rsv_sched_result(rsv_sched* s, int64_t id, uint32_t* out, int64_t cap, int64_t* n_out);
/* Waits for everything queued so far and reports device-side errors. */
int rsv_sched_sync(rsv_sched* s);
int rsv_sched_stats(rsv_sched* s, int64_t* steps_out, int64_t* rows_out);

/* ---- profiling / timing ----------------------------------------------------------------------- */
/* Bundle::clear_kernel_prof / dump_kernel_prof (src/gpu_model.rs:3739-3746).  While enabled every kernel is
 * bracketed by a CUDA event pair on the model's stream (this serialises the stream: diagnostics only). */
int rsv_prof_enable(rsv_model* m, int on);
int rsv_prof_clear(rsv_model* m);
/* Writes a JSON object {"kernel": {"launches": n, "ms": t}, ...} into buf (NUL-terminated, truncated to cap). */
int rsv_prof_dump(rsv_model* m, char* buf, int64_t cap);
/* Kernels launched through this handle since the last rsv_prof_clear. */
int64_t rsv_launch_count(const rsv_model* m);
/* CUDA-event stopwatch on the model's stream: start, ..., stop -> elapsed device time in ms. */
int rsv_timer_start(rsv_model* m);
int rsv_timer_stop(rsv_model* m, float* ms_out);
int rsv_synchronize(rsv_model* m);

/* ---- operator-level entry points (host buffers in and out; used for kernel parity tests) ------ */
/* int8 container decode, w = scale*q + zero in fp32 (dequant_int8, src/model.rs:234-252): out[M*K]. */
int rsv_op_dequant_int8(int device, const uint8_t* idx, const uint32_t* sz, int64_t M, int64_t K, float* out);
/* The reference's offline int8 quantiser for one matrix (quantize_int8_matrix, tools/quantize_any4.py:241-300): w[M*K] f32 ->
 * idx_out u8 [M,K] and sz_out u32 [M,K/128] (scale fp16 | zero fp16 << 16), per group of 128: zero = min, scale = (max - min) /
 * 255, q = clip(round-half-even((w - zero) / scale), 0, 255); a constant group gets scale 0.  Bit for bit what the numpy tool
 * writes, so a checkpoint quantised here loads in the reference and the other way round. */
int rsv_quantize_int8(int device, const float* w, int64_t M, int64_t K, uint8_t* idx_out, uint32_t* sz_out);
/* One linear layer on its own: y[R*M] = x[R*K] . W[M,K]^T with W either fp16 (wtype 0, sz NULL) or the int8 container
 * (wtype 1: w = u8 [M,K], sz = u32 [M,K/128]).  path 0 = SIMT weight-streaming kernel, 1 = tcgen05 tensor-core kernel.
 * Stands in for the reference's per-kernel GEMV/GEMM unit tests (gemv_f16, gemv_variant, gemm; src/backend_cuda.rs:7440-7480,
 * 8880-9066, 9607-9675). */
int rsv_op_linear(int device, int path, int wtype, const void* w, const uint32_t* sz, int64_t M, int64_t K, const float* x, int64_t R, float* y);
/* The WKV-7 step of one layer on its own, nseg sessions x T tokens (rows session-major, [nseg*T, H*64] f32 each):
 *   kk = normalize(k * k_k) per head, k~ = k + k_a (k a - k), v' = v + vgate (vfirst - v) (vgate, vfirst NULL: v' = v),
 *   S <- S diag(w) + (S kk)(-kk a)^T + v' k~^T, y = (GroupNorm_head(S r; lnx_w, lnx_b, eps 64e-5) + (sum r k~ r_k) v') g
 * with w the decay (already exp(-e^-0.5 sigmoid(.))), a already sigmoid, S[h][i][j] i = value row, j = key column; state
 * [nseg, H, 64, 64] in and out.  The CPU path's l2_norm_groups / dplr_update / dplr_matvec / group_norm / sum_rk_rk
 * (src/model.rs:716-826) and the kernels fuse_ka_dplr_norm and rwkv_dplr_seq + rwkv_fuse_ka + rwkv_sum_rk_rk
 * (src/backend_cuda.rs:2620-2764, 4231-4309, 4507-4575; their unit tests :8549-8669).  variant picks the kernel:
 * 0 as the forward step would, 1 token kernel, 2 row-per-lane kernel with TMA-staged states, 3 / 4 sequence kernel with a
 * head over two CTAs / in one CTA. */
int rsv_op_wkv7(int device, int variant, int64_t nseg, int64_t T, int64_t H, const float* r, const float* k, const float* v, const float* w, const float* a,
                const float* g, const float* vgate, const float* vfirst, const float* k_k, const float* k_a, const float* r_k, const float* lnx_w,
                const float* lnx_b, float* state, float* y);
/* arg-max per row of logits[rows*V], ties to the smaller index (rwkv_argmax, src/backend_cuda.rs:3640-3680). */
int rsv_op_argmax(int device, const float* logits, int64_t rows, int64_t V, uint32_t* out);
/* The sampling kernel on its own (rwkv_sample(_batch), src/backend_cuda.rs:3690-4009, 2069-2387):
 * sampler8[rows*8] rows are [temperature, bits(top_k), top_p, bits(seed), rep, freq, pres, bits(hist_len)],
 * hist[rows*hist_stride] holds each row's history. */
int rsv_op_sample(int device, const float* logits, int64_t rows, int64_t V, const float* sampler8, const uint32_t* hist, int64_t hist_stride,
                  uint32_t* out);

/* Sampling for callers that cannot allocate device memory.  It has no counterpart in the reference.
 * Same kernel and semantics as rsv_op_sample, but every pointer is a DEVICE pointer supplied by the caller
 * (logits_dev[rows*V], sampler8_dev[rows*8], hist_dev[rows*hist_stride] or NULL, out_dev[rows]), the launch goes
 * to `stream` (a cudaStream_t, NULL = default stream) and returns without synchronising, and the kernel's work
 * area is a fixed pair of static device arrays inside the library: no cudaMalloc / cudaFree happens here.
 *   - limit: rows * V <= 1,048,576 elements (8 MiB of static device memory per GPU, held until exit); larger
 *     requests are rejected with an error, not truncated;
 *   - the first call on each device looks up the arrays' device addresses; make that call before any stream
 *     capture begins;
 *   - all calls share the one work area: calls whose kernels can overlap on the GPU (different streams) race;
 *     serialise them.  The work area needs no clearing between calls (the kernel rewrites what it reads);
 *   - each row's hist_len (word 7 of its sampler row) must not exceed hist_stride; this cannot be checked here
 *     because the rows live in device memory. */
int rsv_op_sample_static(int device, void* stream, const float* logits_dev, int64_t rows, int64_t V, const float* sampler8_dev,
                         const uint32_t* hist_dev, int64_t hist_stride, uint32_t* out_dev);

#ifdef __cplusplus
}
#endif
#endif /* RSV_B200_H */
