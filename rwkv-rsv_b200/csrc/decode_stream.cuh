// Batch-1 decode as a row-owner weight-streaming matrix-vector product inside one persistent launch.
//
// One cooperative launch runs n tokens x L layers x (head, arg-max) for ONE session: the launch stands in for the
// reference's captured-graph decode step (forward_token / forward_layer / selfloop_step, src/gpu_model.rs:1879-2392)
// and its weight-streaming GEMVs (gemv_variant, gemv_int8_rkv_stage1, gemv_f16; src/backend_cuda.rs:3229-3373,
// 2949-3152, 1421-1498), which read 4 rows per block with the dequantisation fused into the load.
//
// Decomposition.  CTA c (one per SM) owns output rows [c M / G, (c+1) M / G) of every matrix for the WHOLE K: no
// partial sums ever cross a CTA, so a phase is  activation vector -> dot products -> plain stores -> grid barrier.
//   warp 0      producer.  Walks the fixed sequence of weight rows this CTA will ever need - token after token, layer
//               after layer, phase after phase - and streams them with bulk asynchronous copies (cp.async.bulk, one
//               per row, issued by the lanes in parallel) into a byte-granular ring in shared memory; a chunk = one
//               tile of up to 16 rows x one piece (1280 bytes; 2560 for the head) of K, one mbarrier per chunk.  It never waits on a
//               grid barrier, only on ring space, so HBM keeps streaming while the other warps synchronise:
//               barriers cost latency, not bandwidth.
//   warps 1-16  consumers.  Per phase they build the activation vector in shared memory (LayerNorm, token shift,
//               fixed-point digits), laid out as the B fragments of the warp-level matrix instruction.  Then every
//               chunk belongs to ONE warp (chunk i of a phase to warp i mod 16, so the pieces of a long row are
//               multiplied by different warps at once), which multiplies it out of the ring (ldmatrix -> mma.sync,
//               the reduction over K happens inside the instruction): no shuffles in the loop, nothing to wait for
//               but the chunk itself.  The warp that finishes a tile's last piece adds the pieces' partial sums in
//               piece order and stores the outputs.  A row in the ring is padded by 16 bytes so that the rows of a
//               tile fall into different banks.
// Arithmetic.  int8 matrices: the u8 codes q are multiplied as they are (m16n8k32, u8 x s8 -> s32) with the four
// signed base-256 digits of the fixed-point activation t = rint(x / e 2^30), e = 2^ceil(log2 max|x|) (the digits are
// the bytes of (t + 0x808080) ^ 0x808080); the four int32 sums recombine to Q = sum_k q_k t_k exactly (int64), and
// with the container's per-row (scale s, zero z)  y = e 2^-30 (s Q + z T), T = sum_k t_k: no accumulation rounding,
// no dependence on the schedule.  fp16 matrices (head, rank projections, fp16 checkpoints): m16n8k16 f16 x f16 ->
// f32 with x / e split into hi + lo halves (two operand columns).  These are 8-column problems that stream weights at
// HBM speed; the tensor pipe is nearly idle, which is why the warp-level instruction is the right size here and the
// tcgen05 kernels take over once several rows make the product a dense contraction.
// Phases per layer, one grid barrier after each (bounded spin):
//   1  LN1 + token shift -> r, k, v and the four rank projections (tanh / sigmoid applied)
//   2  one CTA per head: rank back-projections (their rows arrive through the ring too), decay / a / v-gate / g,
//      WKV-7 state update in place, GroupNorm, bonus, gate
//   3  att.output, x += ...      4  LN2 + shift -> relu(ffn.key)^2      5  ffn.value, x += ...
// then ln_out + head -> logits, arg-max across CTAs, next token.
// All waits are bounded; on expiry bit 5 of the status word is set (and the word after it says which wait), every role drains its copies in flight and exits.
#pragma once
#include <cstddef>

#include "kernels.cuh"
#include "tc_linear.cuh"

namespace rsv {

constexpr int kDsConsumerWarps = 16;
constexpr int kDsConsumers = kDsConsumerWarps * 32;  // 512
constexpr int kDsThreads = kDsConsumers + 32;        // + producer warp
constexpr int kDsBars = 16;                          // chunks in flight (mbarrier pairs)
constexpr int kDsTileRows = 16;                      // rows of a tile (the m dimension of the matrix instruction)
constexpr int kDsPad = 16;                           // bytes between the rows of a tile in the ring, beyond the piece
constexpr int kDsMaxPiece = 2560;                    // bytes of K per piece (the head's rows)
constexpr int kDsLayerPiece = 1280;                  // bytes of K per piece of the layers' matrices (measured at the 3B shape: 640 -> 1.74, 1280 -> 1.55, 2560 -> 1.66 ms per token)
constexpr int kDsMaxTiles = 64;                      // tiles of one phase per CTA
constexpr int kDsPartBytes = 8 * 1024;               // per-piece partial sums of the tiles of one phase
constexpr int kDsMaxRows = 512;                      // rows of one phase per CTA whose (scale, zero) are staged
constexpr int kDsMaxSlice = 32;                      // channels of the residual stream per CTA
constexpr int kDsP = 30;                             // fixed-point bits of the activation digits
constexpr uint32_t kDsBarSpin = 1u << 22;

// What a finished dot product becomes.
enum DsOut : int { DSO_R = 0, DSO_K, DSO_V, DSO_MID_TANH, DSO_MID, DSO_MID_SIG, DSO_XADD, DSO_H, DSO_LOGITS };

// One matrix of a phase.
struct DsEntry {
    const char* base;     // fp16 [M,K] or u8 [M,K], row-major
    const float* wscale;  // int8: [M] per-row scale and zero of the container
    const float* wzero;
    const float* mix;     // rank projections: the token-shift mix vector of their input; null otherwise
    const uint32_t* sz;   // int8 with one (scale, zero) per row and group of 128 (is_i8 == 2): the container's [M, K/128] words, fp16 scale | fp16 zero << 16
    int M;                // output rows (0: the entry does not exist in this layer)
    int row_stride;       // bytes between rows
    int piece_bytes;      // bytes of K per piece (a multiple of 128, <= kDsMaxPiece)
    int npieces;          // pieces per row
    int is_i8;            // 0: fp16; 1: int8, one (scale, zero) per row (wscale, wzero); 2: int8, one per row and group of 128 (sz)
    int xvec;             // which vector of the phase's operand area the rows are multiplied with
    int out;              // DsOut
    int out_off;          // offset inside the rank-space vector for DSO_MID*
    int cta0, ncta;       // the rows are split over the ncta CTAs cta0, cta0 + 1, ... (mod G)
};
enum { DSE_W1 = 0, DSE_A1, DSE_G1, DSE_V1, DSE_WR, DSE_WK, DSE_WV, DSE_WO, DSE_WFK, DSE_WFV, DSE_COUNT };
struct DsLayer {
    DsEntry e[DSE_COUNT];
    const __half *w2, *a2, *v2, *g2;  // back-projections [C, mid] fp16
    const float *ln1_w, *ln1_b, *ln2_w, *ln2_b, *lnx_w, *lnx_b;
    const float *x_r, *x_k, *x_v, *ffn_x_k;
    const float *w0, *a0, *v0, *r_k, *k_k, *k_a;
};
struct DsParams {
    const DsLayer* layers;
    DsEntry head;
    const __half* emb;
    const float *ln0_w, *ln0_b, *lno_w, *lno_b;
    int L, C, H, F, V, wm, am, vm, gm;
    int slot;
    long long lay_x, lay_s;        // floats between consecutive layers of the shift states / the WKV states
    float *tmix_x, *wkv, *cmix_x;  // state bases (layer 0, slot 0)
    float* state_vfirst;           // [cap][C]
    float *x, *yg, *vfirst;        // [C]
    float* rkv;                    // [3][C]
    float* mid;                    // [wm+am+vm+gm]
    float* hbuf;                   // [F]
    uint32_t* tokens;              // [1] current input token (read at start, written after arg-max)
    const uint32_t* tok_list;      // [n_tokens], used when tok_from_list
    uint32_t* seq;
    int* seq_cnt;
    int seq_cap;
    float* logits;  // [V]
    float* cand_val;
    int* cand_idx;  // [G]
    unsigned* grid_bar;
    int* status;
    int n_tokens, tok_from_list, argmax_feed;
    const char* wstream;      // the layers' weights in consumption order: region (layer l, CTA c) at (l G + c) wslot
    long long wslot;
    const char* hstream;      // the head's rows in consumption order: region of CTA c at c hslot
    long long hslot;
    int ring_bytes;  // shared-memory ring
    int head_early;  // 1: a head's first chunk (w2, a2 rows) is released before the other two are awaited (ring too small for all three)
    int vec_floats;  // operand area, in 4-byte elements: max(4 C, F)
    long long* dbg;  // optional time stamps (built with -DRSV_DS_DEBUG only)
};

// ---- small helpers ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void ds_consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kDsConsumers) : "memory"); }
__device__ __forceinline__ uint32_t ds_lds32(uint32_t saddr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}
__device__ __forceinline__ uint4 ds_lds128(uint32_t saddr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
    return v;
}
// four 8 x 16-byte matrices, row addresses from lanes 8 i .. 8 i + 7: lane (g, t) gets bytes 4 t .. 4 t + 3 of row g of each
__device__ __forceinline__ uint4 ds_ldmatrix4(uint32_t saddr) {
    uint4 v;
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
    return v;
}
// D += A (16 x 32 u8, row-major: sixteen weight rows) x B (32 x 8 s8, column-major: the activation digits, one per column)
__device__ __forceinline__ void ds_mma_i8(int (&c)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}
// D += A (16 x 16 f16: sixteen weight rows) x B (16 x 8 f16: hi and lo halves of the activations), fp32 accumulation
__device__ __forceinline__ void ds_mma_f16(float (&c)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint64_t ds_evict_first_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// Bulk asynchronous copy global -> shared memory of this CTA (16-byte aligned addresses, size a multiple of 16), completion
// counted in bytes on `bar`.  Weights are read once per token: they are marked evict-first in L2 so that the small arrays and
// the recurrent state every phase re-reads stay resident.
__device__ __forceinline__ void ds_bulk_load(uint32_t dst_saddr, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst_saddr), "l"(src),
                 "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
// Wait that ignores the abort flag (used to drain copies in flight before leaving); still bounded.
__device__ __forceinline__ void ds_mbar_drain(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 20); ++i)
        if (mbar_try_wait(bar, parity)) return;
}
#ifdef RSV_DS_DEBUG
__device__ __forceinline__ long long ds_now0() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#endif
__device__ __forceinline__ float ds_pow2(int n) { return __int_as_float((n + 127) << 23); }
__device__ __forceinline__ int ds_ceil_log2(float a) {
    const int bits = __float_as_int(a);
    return ((bits >> 23) & 0xFF) - 127 + ((bits & 0x7FFFFF) ? 1 : 0);
}
// exponent e of the power-of-two scale of a vector whose largest magnitude is `amax`
__device__ __forceinline__ int ds_exponent(float amax) {
    int ex = 0;
    if (amax >= 1.0e-30f && amax < 3.0e38f) ex = ds_ceil_log2(amax);
    return max(-90, min(90, ex));
}
// first row of the share of virtual CTA index vc when M rows are split over n CTAs
__host__ __device__ inline int ds_row_begin(int vc, int M, int n) { return (int)(((long long)vc * M) / n); }
// the rows [r0, r0 + n) of entry E that CTA `cta` of G owns (n = 0: none)
__host__ __device__ inline void ds_rows_of(const DsEntry& E, int cta, int G, int& r0, int& n) {
    r0 = n = 0;
    if (E.M <= 0 || E.ncta <= 0) return;
    const int vc = ((cta - E.cta0) % G + G) % G;
    if (vc >= E.ncta) return;
    r0 = ds_row_begin(vc, E.M, E.ncta);
    n = ds_row_begin(vc + 1, E.M, E.ncta) - r0;
}
// bytes a chunk of nr rows of entry E holds in the ring
__host__ __device__ inline int ds_chunk_bytes(const DsEntry& E, int nr) { return nr * (E.piece_bytes + kDsPad); }
// the CTA that runs head h of layer l (H <= G: heads spread with a stride, rotated per layer so that the extra bytes of a
// head's back-projection rows do not always land on the same SMs); -1 when CTA `cta` has no head in that layer
__host__ __device__ inline int ds_head_of_cta(int cta, int l, int H, int G) {
    const int stride = G / H;
    const int d = ((cta - (l * 37) % G) % G + G) % G;
    if (d % stride) return -1;
    const int h = d / stride;
    return h < H ? h : -1;
}
// two fp16 packed in a 32-bit register -> two floats (no address of a local is taken, so nothing goes through local memory)
__device__ __forceinline__ float2 ds_half2_bits_to_float2(uint32_t u) {
    float2 f;
    asm("{\n\t.reg .f16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.f32.f16 %0, lo;\n\tcvt.f32.f16 %1, hi;\n\t}" : "=f"(f.x), "=f"(f.y) : "r"(u));
    return f;
}
// exact sum of a 64-bit value over the warp whose magnitude is below 2^40 per lane (two 32-bit reductions)
__device__ __forceinline__ long long ds_warp_sum_ll(long long v) {
    const unsigned lo = __reduce_add_sync(0xffffffffu, (unsigned)(v & 0xFFFF));
    const int hi = __reduce_add_sync(0xffffffffu, (int)(v >> 16));
    return (long long)hi * 65536 + (long long)lo;
}

// A chunk of weight rows: one tile (up to 16 rows of a matrix) x one piece of K.  The chunks a CTA consumes are the same in
// every layer (its row ranges do not change), so they are tabulated once per launch; the weights themselves are stored a
// second time in exactly this order (rows padded by 16 bytes, chunk after chunk), so that a chunk is ONE bulk copy.
struct alignas(16) DsChunk {
    int cb;            // bytes of the chunk, in the stream and in the ring: nr * stride
    int nr_steps;      // rows (<= 16) | 64-byte column steps (pairs of k steps) of the piece << 16
    int piece_np;      // which piece of the rows' K | pieces per row << 16
    uint32_t baddr;    // shared-memory address of the activation fragments of this piece (lane offset not included)
    int part_tile;     // byte offset of the tile's partial sums | arrival counter of the tile << 16
    int e_flags_row0;  // matrix DSE_* (DSE_COUNT: the head) | flags << 8 (1: int8, 2: absent in layer 0) | first row of the tile (from the CTA's first row) << 16
    int stage_off;     // first staged (scale, zero) of the matrix
    int stride;        // bytes between the rows of the chunk: piece + 16
};
// What the producer tells the consumer about the chunk on a barrier pair: where it landed in the ring.  Chunk j of the launch
// always uses barrier pair j mod 16 and, when it carries weight rows, belongs to consumer warp j mod 16; which table entry it
// is follows from its position in the phase, so the consumer reads the entry itself (two 16-byte loads) and the producer's work
// per chunk is a reservation, this word, and one bulk copy.
struct DsDesc {
    int ring_off;  // byte offset of the chunk in the ring
};
static_assert(sizeof(DsChunk) == 32, "a table entry is read as two 16-byte words");
constexpr int kDsMaxGroups = 128;  // groups of 128 in the longest reduction (K <= 16384)
constexpr int kDsMaxChunks = 256;  // table entries per CTA: the chunks of a layer plus the head's
enum { DSP_P1 = 0, DSP_P3, DSP_P4, DSP_P5, DSP_HEAD, DSP_COUNT };
// The CTA's static plan (built once per launch).
struct DsPlan {
    int er0[DSE_COUNT + 1], en[DSE_COUNT + 1];  // rows [er0, er0 + en) of every matrix (DSE_*; last: the head) this CTA owns: the same in all layers
    int rank_entry;                             // the rank projection whose rows this CTA owns (-1: none)
    int ph0[DSP_COUNT], phn[DSP_COUNT];         // the phases' ranges in ctab
    int phn_l0;                                 // chunks of phase 1 in layer 0 (no v-gate projection there)
    DsChunk ctab[kDsMaxChunks];
};

// ---- shared-memory layout: [ring][operand area: vec_floats x 4 bytes][DsShared][rank-space vector] ----------------
struct DsShared {
    uint64_t full[kDsBars], empty[kDsBars];
    int alloc[kDsBars];  // producer only: bytes (with wrap waste) a chunk in flight holds
    int abort_flag;
    float tg[4][kDsMaxGroups];  // per operand vector: the fixed-point sum of every group of 128 elements (as float; for per-group int8 rows)
    int abort_where;  // which wait gave up first (1 rows: full, 2 producer: empty, 3 grid barrier, 4 heads: full) | detail << 4
    uint32_t tok;
    float red_a[16], red_b[16], red_c[4 * 16];
    int red_i[16];
    long long tsw[4][16];  // per consumer warp: exact sum of the fixed-point values of operand vector v
    int ex[4];             // exponent of the power-of-two scale of operand vector v
    float xs_own[kDsMaxSlice];  // this CTA's slice of the residual stream
    float ts_own[kDsMaxSlice];  // pending time-mix shift state of the slice
    float cs_own[kDsMaxSlice];  // pending channel-mix shift state of the slice
    float ws[kDsMaxRows], wz[kDsMaxRows];  // (scale, zero) of the rows this CTA owns in the current phase
    alignas(16) float hv[10 * 64];                     // the 64-vectors of a head
    float best_val[kDsConsumers];          // per consumer thread: arg-max of the head rows it finished
    int best_idx[kDsConsumers];
    DsPlan plan;
    DsDesc desc[kDsBars];                  // what the chunk on barrier b is (written by the producer before it arms the barrier)
    int tile_cnt[kDsMaxTiles];             // pieces of a tile finished so far (zero between phases)
    long long part[kDsPartBytes / 8];      // per-piece partial sums: int64 (int8 matrices) or fp32 (fp16 matrices), 16 rows each
    DsLayer layer[2];                      // table of the current / next layer
};

// Operand area.  Vector v of a phase (`len` elements) occupies 4 len bytes at byte offset 4 v len, stored as the B fragments
// the consumer lanes load with one 16-byte read per two k steps:
//   int8 matrices (k step = 32 elements): index [k / 64][digit 0..3][t = (k % 16) / 4][word (k % 64) / 16], the word holding
//     the digit of the four consecutive k in its bytes; lane (g, t) of a warp reads the 16 bytes at ((k/64) 4 + g) 4 + t.
//   fp16 matrices (k step = 16 elements): index [k / 32][0 = hi, 1 = lo][t = (k % 8) / 2][word (k % 32) / 8], the word holding
//     the halves of k, k + 1.
// Writes the vectors (getval(v, i) = the i-th of a thread's NGR groups of four consecutive elements of vector v) in that form; the scale exponent
// goes to S->ex[v], for int8 the exact fixed-point sum to S->tsw[v].
template <int NV, int NGR, class GetVal>
__device__ __forceinline__ void ds_emit(DsShared* S, float* vec, int len, const bool (&i8)[NV], GetVal getval, int wtid, bool group_sums = false, long long* dbg = nullptr) {
    const int wwarp = wtid >> 5, lane = wtid & 31, len4 = len >> 2;
    float am[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        am[v] = 0.f;
#pragma unroll
        for (int gi = 0; gi < NGR; ++gi)
            if (wtid + kDsConsumers * gi < len4) {
                const float4 x = getval(v, gi);
                am[v] = fmaxf(am[v], fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) am[v] = fmaxf(am[v], __shfl_xor_sync(0xffffffffu, am[v], o));
        if (lane == 0) S->red_c[v * 16 + wwarp] = am[v];
    }
#ifdef RSV_DS_DEBUG
    if (dbg && wtid == 0) dbg[0] = ds_now0();
#endif
    ds_consumer_sync();
#ifdef RSV_DS_DEBUG
    if (dbg && wtid == 0) dbg[1] = ds_now0();
#endif
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        float a = S->red_c[v * 16 + (lane & 15)];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        const int ex = ds_exponent(a);
        if (wtid == 0) S->ex[v] = ex;
        uint32_t* vb = reinterpret_cast<uint32_t*>(vec + (size_t)v * len);
        if (i8[v]) {
            const float mult = ds_pow2(kDsP - ex);  // |x| <= 2^ex, so |t| <= 2^30; a NaN converts to 0
            long long ts = 0;
#pragma unroll
            for (int gi = 0; gi < NGR; ++gi) {
                const int g4 = wtid + kDsConsumers * gi;
                if (g4 < len4) {
                    const float4 x = getval(v, gi);
                    const float f[4] = {x.x * mult, x.y * mult, x.z * mult, x.w * mult};
                    uint32_t u[4];
                    long long t4 = 0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int t = __float2int_rn(f[j]);
                        t4 += t;
                        u[j] = ((uint32_t)t + 0x00808080u) ^ 0x00808080u;  // bytes = signed base-256 digits of t
                    }
                    ts += t4;
                    if (group_sums) {
                        // a warp's 32 groups of four are one group of 128 elements: its sum, for rows with a (scale, zero) per group
                        // (uniform branch: len4 is a multiple of 32, so a warp is inside the vector as a whole or not at all)
                        const long long tgrp = ds_warp_sum_ll(t4);
                        if (lane == 0) S->tg[v][g4 >> 5] = (float)tgrp;
                    }
                    // 4 x 4 byte transpose: word d = digit d of the four elements
                    const uint32_t lo01 = __byte_perm(u[0], u[1], 0x5140), hi01 = __byte_perm(u[0], u[1], 0x7362);
                    const uint32_t lo23 = __byte_perm(u[2], u[3], 0x5140), hi23 = __byte_perm(u[2], u[3], 0x7362);
                    uint32_t* dst = vb + ((size_t)(g4 >> 4) * 16 + (g4 & 3)) * 4 + ((g4 >> 2) & 3);
                    dst[0] = __byte_perm(lo01, lo23, 0x5410);
                    dst[16] = __byte_perm(lo01, lo23, 0x7632);
                    dst[32] = __byte_perm(hi01, hi23, 0x5410);
                    dst[48] = __byte_perm(hi01, hi23, 0x7632);
                }
            }
            ts = ds_warp_sum_ll(ts);
            if (lane == 0) S->tsw[v][wwarp] = ts;
        } else {
            const float mult = ds_pow2(-ex);
#pragma unroll
            for (int gi = 0; gi < NGR; ++gi) {
                const int g4 = wtid + kDsConsumers * gi;
                if (g4 < len4) {
                    const float4 x = getval(v, gi);
                    const float f[4] = {x.x * mult, x.y * mult, x.z * mult, x.w * mult};
                    __half hi[4], lo[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float q = fminf(fmaxf(f[j], -1.0f), 1.0f);
                        if (!(q == q)) q = 0.f;
                        hi[j] = __float2half_rn(q);
                        lo[j] = __float2half_rn(q - __half2float(hi[j]));
                    }
                    uint32_t* dst = vb + ((size_t)(g4 >> 3) * 8 + (g4 & 1) * 2) * 4 + ((g4 & 7) >> 1);
                    const __half2 h01 = __halves2half2(hi[0], hi[1]), h23 = __halves2half2(hi[2], hi[3]);
                    const __half2 l01 = __halves2half2(lo[0], lo[1]), l23 = __halves2half2(lo[2], lo[3]);
                    dst[0] = *reinterpret_cast<const uint32_t*>(&h01);   // row hi, t
                    dst[4] = *reinterpret_cast<const uint32_t*>(&h23);   // row hi, t + 1
                    dst[16] = *reinterpret_cast<const uint32_t*>(&l01);  // row lo, t
                    dst[20] = *reinterpret_cast<const uint32_t*>(&l23);  // row lo, t + 1
                }
            }
        }
    }
#ifdef RSV_DS_DEBUG
    if (dbg && wtid == 0) dbg[2] = ds_now0();
#endif
    ds_consumer_sync();
}

// What the consumer warps need to turn a row's sums into an output (passed by value: nothing of it lives in local memory).
struct DsPhaseCtx {
    uint32_t vec_s;  // shared-memory address of the operand area
    int k0;          // table index of the phase's first chunk
#ifdef RSV_DS_DEBUG
    long long* dbg;  // non-null: this call adds warp 0's time waiting for chunks to dbg[0] and its time multiplying to dbg[1]
#endif
};
#ifdef RSV_DS_DEBUG
#ifndef RSV_DS_DEBUG_WARPS
#define RSV_DS_DEBUG_WARPS 20  // which phase's per-warp stamps are recorded: 20 phase 1, 24 phase 3, 28 phase 4, 32 phase 5
#endif
__device__ __forceinline__ long long ds_now() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#endif

__device__ __forceinline__ void ds_store(const DsParams& P, DsShared* S, const DsEntry& E, int m, int rl, float y) {
    switch (E.out) {
        case DSO_R:
        case DSO_K:
        case DSO_V: P.rkv[(size_t)E.out * P.C + m] = y; break;
        case DSO_MID_TANH: P.mid[E.out_off + m] = tanhf(y); break;
        case DSO_MID: P.mid[E.out_off + m] = y; break;
        case DSO_MID_SIG: P.mid[E.out_off + m] = 1.0f / (1.0f + expf(-y)); break;
        case DSO_XADD: {
            const float nx = S->xs_own[rl] + y;
            S->xs_own[rl] = nx;
            P.x[m] = nx;
            break;
        }
        case DSO_H: {
            const float a = fmaxf(y, 0.f);
            P.hbuf[m] = a * a;
            break;
        }
        default: {
            P.logits[m] = y;
            // running arg-max of the head rows this lane finished (ties: smaller index); one slot per consumer thread
            const int sl = (int)threadIdx.x - 32;
            if (y > S->best_val[sl] || (y == S->best_val[sl] && m < S->best_idx[sl])) {
                S->best_val[sl] = y;
                S->best_idx[sl] = m;
            }
            break;
        }
    }
}

// Builds the CTA's plan: row ranges (the one place where the rows are divided), then the chunk table phase by phase
// (matrix after matrix, tile after tile, piece after piece).  `ents` = a layer's matrices (one with a v-gate projection),
// vec_s = shared-memory address of the operand area (0 where the table is only used to lay out the weight stream).
// Executed by one thread.  Returns false when the table would overflow.
__host__ __device__ inline bool ds_build_plan(DsPlan& pl, const DsEntry* ents, const DsEntry& head, int cta, int G, uint32_t vec_s) {
    for (int e = 0; e <= DSE_COUNT; ++e) {
        int r0, n;
        ds_rows_of(e == DSE_COUNT ? head : ents[e], cta, G, r0, n);
        pl.er0[e] = r0;
        pl.en[e] = n;
    }
    pl.rank_entry = -1;
    for (int e = DSE_W1; e <= DSE_V1; ++e)
        if (pl.en[e] > 0 && pl.rank_entry < 0) pl.rank_entry = e;
    const int first[DSP_COUNT] = {DSE_W1, DSE_WO, DSE_WFK, DSE_WFV, DSE_COUNT}, last[DSP_COUNT] = {DSE_WV, DSE_WO, DSE_WFK, DSE_WFV, DSE_COUNT};
    int k = 0;
    bool fits = true;
    pl.phn_l0 = 0;
    for (int ph = 0; ph < DSP_COUNT; ++ph) {
        pl.ph0[ph] = k;
        int tile = 0, part = 0, stage = 0;
        for (int e = first[ph]; e <= last[ph]; ++e) {
            const DsEntry& E = e == DSE_COUNT ? head : ents[e];
            const int n = pl.en[e];
            if (n <= 0) continue;
            const bool i8 = E.is_i8 != 0, pg = E.is_i8 == 2;
            const int steps = E.piece_bytes >> 6, klen = (i8 ? E.piece_bytes : (E.piece_bytes >> 1)) * E.npieces, bstep = (i8 ? 4 : 2) * 64, slot = (i8 && !pg) ? 8 : 4;
            // rows with a (scale, zero) per group of 128 carry them behind the rows: [group of the piece][16 rows] words
            const int sz_bytes = pg ? (E.piece_bytes >> 7) * kDsTileRows * 4 : 0;
            for (int row0 = 0; row0 < n; row0 += kDsTileRows) {
                const int nr = n - row0 < kDsTileRows ? n - row0 : kDsTileRows;
                for (int p = 0; p < E.npieces; ++p) {
                    if (k >= kDsMaxChunks) {
                        fits = false;
                        continue;
                    }
                    DsChunk& c = pl.ctab[k++];
                    c.stride = E.piece_bytes + kDsPad;
                    c.cb = nr * c.stride + sz_bytes;
                    c.nr_steps = nr | (steps << 16);
                    c.piece_np = p | (E.npieces << 16);
                    c.baddr = vec_s + (uint32_t)E.xvec * (uint32_t)klen * 4u + (uint32_t)p * (uint32_t)steps * (uint32_t)bstep;
                    c.part_tile = part | (tile << 16);
                    c.e_flags_row0 = e | ((i8 ? 1 : 0) << 8) | ((e == DSE_V1 ? 2 : 0) << 8) | ((pg ? 4 : 0) << 8) | (row0 << 16);
                    c.stage_off = stage;
                    if (ph == DSP_P1 && e != DSE_V1) ++pl.phn_l0;
                }
                ++tile;
                part += E.npieces * kDsTileRows * slot;
            }
            if (i8 && !pg) stage += n;
        }
        pl.phn[ph] = k - pl.ph0[ph];
    }
    return fits;
}

// The multiply loop of a chunk whose rows carry a (scale, zero) per group of 128 weights (a function of its own so that its
// registers do not weigh on the other formats' loop): per group two 64-byte steps into fresh integer accumulators, then the
// four digit sums weighted by their powers of 256 in fp32 (exact), times the group's scale, plus zero x the group's activation
// sum.  Returns this lane's contributions to rows g and g + 8 (lanes t = 0, 1 hold two digits each; t = 0 also the zero terms).
__device__ __noinline__ float2 ds_multiply_grouped(uint32_t aaddr, uint32_t baddr, int bstep, bool bcol_ok, int ngp, uint32_t sz_s, const float* tgp, int t) {
    const float w_lo = t < 2 ? (t == 0 ? 1.0f : 65536.0f) : 0.f, w_hi = w_lo * 256.0f;
    float acc0 = 0.f, acc1 = 0.f;
    for (int gi = 0; gi < ngp; ++gi) {
        int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const uint4 a0 = ds_ldmatrix4(aaddr), a1 = ds_ldmatrix4(aaddr + 32);
            uint4 b = make_uint4(0, 0, 0, 0);
            if (bcol_ok) b = ds_lds128(baddr);
            ds_mma_i8(c0, a0, b.x, b.y);
            ds_mma_i8(c1, a1, b.z, b.w);
            aaddr += 64;
            baddr += bstep;
        }
        const uint32_t za = ds_lds32(sz_s + (uint32_t)gi * 64u), zb = ds_lds32(sz_s + (uint32_t)gi * 64u + 32u);
        const float2 fa = ds_half2_bits_to_float2(za), fb = ds_half2_bits_to_float2(zb);  // (scale, zero) of rows g and g + 8
        const float qa = fmaf((float)(c0[1] + c1[1]), w_hi, (float)(c0[0] + c1[0]) * w_lo);
        const float qb = fmaf((float)(c0[3] + c1[3]), w_hi, (float)(c0[2] + c1[2]) * w_lo);
        acc0 = fmaf(fa.x, qa, acc0);
        acc1 = fmaf(fb.x, qb, acc1);
        if (t == 0) {
            const float tgv = tgp[gi];
            acc0 = fmaf(fa.y, tgv, acc0);
            acc1 = fmaf(fb.y, tgv, acc1);
        }
    }
    return make_float2(acc0, acc1);
}

// The weight rows of one phase: its chunks are J, J + 1, ..., J + n - 1 of the launch (matrix after matrix, tile after tile
// of 16 rows, piece after piece of <= 1280 bytes of K: the producer's order), and chunk j belongs to consumer warp j mod 16,
// so the pieces of a long row are multiplied by different warps at the same time.  A warp leaves the partial sums of its
// piece in shared memory and counts its arrival on the tile; the warp that arrives last adds the pieces in piece order (exact
// for int8, fixed order for fp16) and stores the outputs.  `tab`: the layer's matrices (indexed by DSE_*).  Returns false after a timeout.
__device__ __noinline__ bool ds_consume(const DsParams& P, DsShared* S, const DsEntry* tab, uint32_t ring_s, uint32_t J, int n, DsPhaseCtx pc, int wwarp, int lane) {
    const int g = lane >> 2, t = lane & 3;
    for (uint32_t j = J + ((wwarp - J) & (kDsConsumerWarps - 1)); (int)(j - J) < n; j += kDsConsumerWarps) {
#ifdef RSV_DS_DEBUG
        const long long tw0 = ds_now();
#endif
        const bool got = mbar_wait(&S->full[wwarp], (j / kDsBars) & 1u, (volatile int*)&S->abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
            if (lane == 0) atomicCAS(&S->abort_where, 0, 1 | (int)((j - J) << 4));
            return false;
        }
#ifdef RSV_DS_DEBUG
        const long long tw1 = ds_now();
#endif
        // the chunk's table entry (the j-th chunk of the phase) and, from the producer, where in the ring it landed
        const DsChunk* ce = &S->plan.ctab[pc.k0 + (int)(j - J)];
        const uint4 d0 = make_uint4((uint32_t)S->desc[wwarp].ring_off, 0u, 0u, 0u), c0w = reinterpret_cast<const uint4*>(ce)[0], c1w = reinterpret_cast<const uint4*>(ce)[1];
        const uint4 d1 = make_uint4(0u, c0w.y, c0w.z, c0w.w), d2 = c1w;
        const int ring_off = (int)d0.x, nr = (int)(d1.y & 0xFFFFu), steps = (int)(d1.y >> 16), piece = (int)(d1.z & 0xFFFFu), np = (int)(d1.z >> 16);
        const int part_off = (int)(d2.x & 0xFFFFu), tile_idx = (int)(d2.x >> 16), e = (int)(d2.y & 0xFFu), row0 = (int)(d2.y >> 16), stage_off = (int)d2.z,
                  stride = (int)d2.w;
        const bool i8 = (d2.y >> 8) & 1u;
        const DsEntry& E = e == DSE_COUNT ? P.head : tab[e];  // only the warp that finishes the tile looks at it
        // B fragments of this lane: 16 bytes per two k steps at [k-step pair][operand row g][t]; columns beyond the operand's rows are zero
        const int brows = i8 ? 4 : 2, bstep = brows * 64;
        const bool bcol_ok = g < brows;
        uint32_t baddr = d1.w + (uint32_t)(g * 4 + t) * 16u;
        // ldmatrix row addresses: lanes 0-7 rows 0-7, 8-15 rows 8-15 (bytes 0-15 of a 32-byte k step), lanes 16-31 the same rows, bytes 16-31
        const int arow = min((lane & 7) + ((lane >> 3) & 1) * 8, nr - 1);
        uint32_t aaddr = ring_s + (uint32_t)ring_off + (uint32_t)arow * (uint32_t)stride + (uint32_t)(lane >> 4) * 16u;
        const bool pg = (d2.y >> 10) & 1u;
        const int slot = (i8 && !pg) ? 8 : 4;
        char* part = reinterpret_cast<char*>(S->part) + part_off + piece * kDsTileRows * slot;
        if (pg) {
            // int8 rows with a (scale, zero) per group of 128: the integer sums of a group (two 64-byte steps) are weighted by the
            // digits' powers of 256 in fp32 (exact: |sum| < 2^23, power-of-two weights), multiplied by the group's scale and
            // accumulated in fp32 together with zero x (sum of the group's activations).
            const uint32_t sz_s = ring_s + (uint32_t)ring_off + (uint32_t)(nr * stride) + (uint32_t)g * 4u;  // [group][16 rows] words behind the rows
            const float2 acc = ds_multiply_grouped(aaddr, baddr, bstep, bcol_ok, steps >> 1, sz_s, S->tg[E.xvec] + piece * (steps >> 1), t);
            float acc0 = acc.x, acc1 = acc.y;
            acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
            if (t == 0) {
                reinterpret_cast<float*>(part)[g] = acc0;
                reinterpret_cast<float*>(part)[g + 8] = acc1;
            }
        } else if (i8) {
            int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};
            // operands of the next step are loaded before this step's products are issued (the loop is a chain of shared-memory
            // latency + MMA latency otherwise)
            uint4 a0 = ds_ldmatrix4(aaddr), a1 = ds_ldmatrix4(aaddr + 32);
            uint4 b = make_uint4(0, 0, 0, 0);
            if (bcol_ok) b = ds_lds128(baddr);
#pragma unroll 2
            for (int s2 = 1; s2 < steps; ++s2) {
                aaddr += 64;
                baddr += bstep;
                const uint4 n0 = ds_ldmatrix4(aaddr), n1 = ds_ldmatrix4(aaddr + 32);
                uint4 nb = make_uint4(0, 0, 0, 0);
                if (bcol_ok) nb = ds_lds128(baddr);
                ds_mma_i8(c0, a0, b.x, b.y);
                ds_mma_i8(c1, a1, b.z, b.w);
                a0 = n0;
                a1 = n1;
                b = nb;
            }
            ds_mma_i8(c0, a0, b.x, b.y);
            ds_mma_i8(c1, a1, b.z, b.w);
            // accumulator (rows g, g + 8; columns 2 t, 2 t + 1) = weight rows x digits 2 t, 2 t + 1 (t < 2); digit d weighs 256^d
            const int lo = t < 2 ? 16 * t : 0;
            long long va = t < 2 ? (((long long)(c0[0] + c1[0]) << lo) + ((long long)(c0[1] + c1[1]) << (lo + 8))) : 0;
            long long vb = t < 2 ? (((long long)(c0[2] + c1[2]) << lo) + ((long long)(c0[3] + c1[3]) << (lo + 8))) : 0;
            va += __shfl_xor_sync(0xffffffffu, va, 1);
            vb += __shfl_xor_sync(0xffffffffu, vb, 1);
            if (t == 0) {
                reinterpret_cast<long long*>(part)[g] = va;
                reinterpret_cast<long long*>(part)[g + 8] = vb;
            }
        } else {
            float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
            uint4 a0 = ds_ldmatrix4(aaddr), a1 = ds_ldmatrix4(aaddr + 32);
            uint4 b = make_uint4(0, 0, 0, 0);
            if (bcol_ok) b = ds_lds128(baddr);
#pragma unroll 2
            for (int s2 = 1; s2 < steps; ++s2) {
                aaddr += 64;
                baddr += bstep;
                const uint4 n0 = ds_ldmatrix4(aaddr), n1 = ds_ldmatrix4(aaddr + 32);
                uint4 nb = make_uint4(0, 0, 0, 0);
                if (bcol_ok) nb = ds_lds128(baddr);
                ds_mma_f16(c0, a0, b.x, b.y);
                ds_mma_f16(c1, a1, b.z, b.w);
                a0 = n0;
                a1 = n1;
                b = nb;
            }
            ds_mma_f16(c0, a0, b.x, b.y);
            ds_mma_f16(c1, a1, b.z, b.w);
            if (t == 0) {  // columns 0, 1 = hi, lo
                reinterpret_cast<float*>(part)[g] = (c0[0] + c1[0]) + (c0[1] + c1[1]);
                reinterpret_cast<float*>(part)[g + 8] = (c0[2] + c1[2]) + (c0[3] + c1[3]);
            }
        }
        __syncwarp();
        int old = 0;
        if (lane == 0) {
            mbar_arrive(&S->empty[wwarp]);
            __threadfence_block();
            old = atomicAdd(&S->tile_cnt[tile_idx], 1);
        }
        old = __shfl_sync(0xffffffffu, old, 0);
#ifdef RSV_DS_DEBUG
        if (pc.dbg && lane == 0 && wwarp == 0) {
            pc.dbg[0] += tw1 - tw0;
            pc.dbg[1] += ds_now() - tw1;
            pc.dbg[2] += 1;
        }
        if (pc.dbg && pc.dbg == P.dbg + RSV_DS_DEBUG_WARPS && lane == 0) {  // phase 1: per warp, the times of its last chunk
            P.dbg[64 + wwarp * 4 + 0] = tw0;
            P.dbg[64 + wwarp * 4 + 1] = tw1;
            P.dbg[64 + wwarp * 4 + 2] = ds_now();
        }
#endif
        if (old == np - 1) {
            // last piece of the tile: lane r adds the pieces of row r in piece order and stores the output
            __threadfence_block();
            const int rl = row0 + lane;
            long long T = 0;
            if (i8 && !pg) {  // exact sum of the operand's fixed-point values: 16 per-warp sums, one per lane, then a shuffle tree
                T = S->tsw[E.xvec][lane & 15];
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) T += __shfl_xor_sync(0xffffffffu, T, o);
            }
            if (lane < nr) {
                const char* pt = reinterpret_cast<const char*>(S->part) + part_off;
                const int r0 = S->plan.er0[e];
                if (i8 && !pg) {
                    long long Q = 0;
                    for (int q = 0; q < np; ++q) Q += reinterpret_cast<const volatile long long*>(pt + q * kDsTileRows * 8)[lane];
                    const double ws = S->ws[stage_off + rl], wz = S->wz[stage_off + rl];
                    ds_store(P, S, E, r0 + rl, rl, (float)((double)ds_pow2(S->ex[E.xvec] - kDsP) * (ws * (double)Q + wz * (double)T)));
                } else {
                    float y = 0.f;
                    for (int q = 0; q < np; ++q) y += reinterpret_cast<const volatile float*>(pt + q * kDsTileRows * 4)[lane];
                    ds_store(P, S, E, r0 + rl, rl, y * ds_pow2(S->ex[E.xvec] - (pg ? kDsP : 0)));
                }
            }
            if (lane == 0) S->tile_cnt[tile_idx] = 0;
#ifdef RSV_DS_DEBUG
            if (pc.dbg && pc.dbg == P.dbg + RSV_DS_DEBUG_WARPS && lane == 0) P.dbg[64 + wwarp * 4 + 3] = ds_now();
#endif
        }
    }
    return true;
}

#ifdef RSV_DS_DEBUG
// time stamps of CTA 0 at phase boundaries of token 1, layer 1
#define DS_STAMP(id)                                                                  \
    do {                                                                              \
        if (P.dbg && cta == 0 && wtid == 0 && t == 1 && l == 1) P.dbg[id] = ds_now(); \
    } while (0)
#define DS_STAMP_ALL(k)                                                                       \
    do {                                                                                      \
        if (P.dbg && wtid == 0 && t == 1 && l == 1) P.dbg[256 + cta * 16 + (k)] = ds_now0(); \
    } while (0)
#define DS_PSTAMP(id)                                                                 \
    do {                                                                              \
        if (P.dbg && cta == 0 && lane == 0 && t == 1 && l == 1) P.dbg[id] = ds_now(); \
    } while (0)
#else
#define DS_PSTAMP(id) \
    do {              \
    } while (0)
#define DS_STAMP(id) \
    do {             \
    } while (0)
#define DS_STAMP_ALL(k) \
    do {                \
    } while (0)
#endif

// Sum over the 512 consumer threads through a 16-entry array: one barrier per call.  Calls that follow each other must use
// different arrays (a thread may enter the next call while another still reads this one's array).
__device__ __forceinline__ float ds_block_sum(float v, float* arr, int wwarp, int lane) {
    v = warp_sum(v);
    if (lane == 0) arr[wwarp] = v;
    ds_consumer_sync();
    float s = arr[lane & 15];  // one read per lane, then a fixed shuffle tree over the 16 warp sums
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    return s;
}
// LayerNorm statistics (two passes, as the CPU path) of a C-vector spread over the consumer threads (NGR groups of four each)
template <int NGR>
__device__ __forceinline__ void ds_ln_stats(DsShared* S, int C, const float4 (&xv)[NGR], int wtid, float& mean, float& inv) {
    const int wwarp = wtid >> 5, lane = wtid & 31;
    float s = 0.f;
#pragma unroll
    for (int gi = 0; gi < NGR; ++gi)
        if (wtid + kDsConsumers * gi < C / 4) s += (xv[gi].x + xv[gi].y) + (xv[gi].z + xv[gi].w);
    mean = ds_block_sum(s, S->red_a, wwarp, lane) / (float)C;
    float q = 0.f;
#pragma unroll
    for (int gi = 0; gi < NGR; ++gi)
        if (wtid + kDsConsumers * gi < C / 4) {
            const float a = xv[gi].x - mean, b = xv[gi].y - mean, c = xv[gi].z - mean, d = xv[gi].w - mean;
            q += (a * a + b * b) + (c * c + d * d);
        }
    inv = 1.0f / sqrtf(ds_block_sum(q, S->red_b, wwarp, lane) / (float)C + kLnEps);
}
__device__ __forceinline__ float4 ds_ln_apply(float4 x, float mean, float inv, float4 w, float4 b) {
    return make_float4((x.x - mean) * inv * w.x + b.x, (x.y - mean) * inv * w.y + b.y, (x.z - mean) * inv * w.z + b.z, (x.w - mean) * inv * w.w + b.w);
}
__device__ __forceinline__ float4 ds_mix4(float4 cur, float4 m, float4 del) {
    return make_float4(cur.x + m.x * del.x, cur.y + m.y * del.y, cur.z + m.z * del.z, cur.w + m.w * del.w);
}
__device__ __forceinline__ float4 ds_ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 ds_ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

// CMAX: the largest n_embd the instantiation handles (it sizes the per-thread register arrays of the activation vectors)
template <int CMAX>
__global__ void __launch_bounds__(kDsThreads, 1) decode_stream_kernel(const __grid_constant__ DsParams P) {
    constexpr int NG = (CMAX / 4 + kDsConsumers - 1) / kDsConsumers;  // groups of four channels per consumer thread
    constexpr int NG5 = (CMAX + kDsConsumers - 1) / kDsConsumers;     // groups of four of the F = 4 C hidden values per thread
    extern __shared__ __align__(1024) uint8_t ds_smem_raw[];
    uint8_t* ring = (uint8_t*)(((uintptr_t)ds_smem_raw + 127) & ~(uintptr_t)127);
    float* vec = reinterpret_cast<float*>(ring + P.ring_bytes);
    DsShared* S = reinterpret_cast<DsShared*>(vec + P.vec_floats);  // 16-byte aligned: ring and operand area are multiples of 16 bytes
    float* sc_mid = reinterpret_cast<float*>(S + 1);
    volatile int* abort_flag = (volatile int*)&S->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x, cta = blockIdx.x;
    const int R = P.ring_bytes, C = P.C;
    const int nmid = P.wm + P.am + P.vm + P.gm;
    // bytes of the three chunks that carry a head's rank back-projection rows
    const int hbA = 64 * (P.wm + P.am) * 2, hbC = 32 * P.gm * 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDsBars; ++s) {
            mbar_init(&S->full[s], 1);
            mbar_init(&S->empty[s], 1);
        }
        S->abort_flag = 0;
        S->abort_where = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < kDsMaxTiles; i += kDsThreads) S->tile_cnt[i] = 0;
    if (threadIdx.x == 0) {
        // layer 1's table when there is one: layer 0 has no v-gate projection, otherwise all layers split alike
        if (!ds_build_plan(S->plan, P.layers[P.L > 1 ? 1 : 0].e, P.head, cta, G, smem_u32(vec))) {
            atomicOr(P.status, 8);
            S->abort_flag = 1;
        }
    }
    __syncthreads();

    if (warp == 0) {
        // =========================== producer ===========================
        const uint64_t pol = ds_evict_first_policy();
        const uint32_t ring_s = smem_u32(ring);
        int head = 0, used = 0;
        uint32_t j = 0, tail = 0;
        bool ok = true;
        // Reserves `bytes` in the ring for chunk j (waiting for the oldest chunks to be released); the chunk starts at `head - bytes`.
        auto reserve = [&](int bytes) -> bool {
            const bool wrap = head + bytes > R;  // the chunk does not fit behind the last one: it goes to the start of the ring
            const int waste = wrap ? R - head : 0;
            while (used + waste + bytes > R || j - tail >= (uint32_t)kDsBars) {
                const bool w = mbar_wait(&S->empty[tail % kDsBars], (tail / kDsBars) & 1u, abort_flag);
                if (!__all_sync(0xffffffffu, w)) {
                    if (lane == 0) atomicCAS(&S->abort_where, 0, 2 | (int)(j << 4));
                    return false;
                }
                used -= S->alloc[tail % kDsBars];
                ++tail;
            }
            if (wrap) head = 0;
            if (lane == 0) S->alloc[j % kDsBars] = waste + bytes;
            used += waste + bytes;
            head += bytes;
            return true;
        };
        // The weights lie in the stream in the order they are consumed: every chunk is one bulk copy from a running pointer.
        const char* src = nullptr;
        // table entry k: lane 0 publishes the ring offset, arms the barrier (a release: the offset is visible to whoever sees the
        // barrier complete) and issues the copy
        auto put_chunk = [&](int k) -> bool {
            const int cb = S->plan.ctab[k].cb;
            if (!reserve(cb)) return false;
            if (lane == 0) {
                S->desc[j % kDsBars].ring_off = head - cb;
                mbar_expect_tx(&S->full[j % kDsBars], (uint32_t)cb);
                ds_bulk_load(ring_s + (uint32_t)(head - cb), src, (uint32_t)cb, &S->full[j % kDsBars], pol);
            }
            src += cb;
            ++j;
            return true;
        };
        // a chunk that is not weight rows (a head's back-projection rows): only the offset is published
        auto put_raw = [&](int bytes) -> bool {
            if (!reserve(bytes)) return false;
            if (lane == 0) {
                S->desc[j % kDsBars].ring_off = head - bytes;
                mbar_expect_tx(&S->full[j % kDsBars], (uint32_t)bytes);
                ds_bulk_load(ring_s + (uint32_t)(head - bytes), src, (uint32_t)bytes, &S->full[j % kDsBars], pol);
            }
            src += bytes;
            ++j;
            return true;
        };
        auto put_phase = [&](int ph, bool layer0) -> bool {
            const int k0 = S->plan.ph0[ph], k1 = k0 + S->plan.phn[ph];
            for (int k = k0; k < k1; ++k) {
                if (layer0 && ((S->plan.ctab[k].e_flags_row0 >> 8) & 2)) continue;  // the v-gate projection does not exist in layer 0
                if (!put_chunk(k)) return false;
            }
            return true;
        };
        for (int t = 0; t < P.n_tokens && ok; ++t) {
            const bool do_head = P.argmax_feed || t == P.n_tokens - 1;
            for (int l = 0; l < P.L && ok; ++l) {
                src = P.wstream + ((size_t)l * G + cta) * (size_t)P.wslot;
                DS_PSTAMP(40);
                if (!(ok = put_phase(DSP_P1, l == 0))) break;
                DS_PSTAMP(41);
                if (ds_head_of_cta(cta, l, P.H, G) >= 0) {
                    // chunk A: w2, a2 rows of the head; chunk B: v2 rows (layers > 0) and the first 32 g2 rows; chunk C: the other 32
                    const int vb = l > 0 ? 64 * P.vm * 2 : 0;
                    if (!(ok = put_raw(hbA))) break;
                    DS_PSTAMP(42);
                    if (!(ok = put_raw(vb + hbC) && put_raw(hbC))) break;
                    DS_PSTAMP(43);
                }
                ok = put_phase(DSP_P3, false);
                DS_PSTAMP(44);
                ok = ok && put_phase(DSP_P4, false) && put_phase(DSP_P5, false);
                DS_PSTAMP(45);
            }
            if (ok && do_head) {
                src = P.hstream + (size_t)cta * (size_t)P.hslot;
                ok = put_phase(DSP_HEAD, false);
            }
        }
        // copies still in flight must land before the CTA may exit (only after an abort: otherwise every chunk was consumed)
        if (!ok)
            for (; tail < j; ++tail) ds_mbar_drain(&S->full[tail % kDsBars], (tail / kDsBars) & 1u);
    } else {
        // =========================== consumers ===========================
        const int wtid = threadIdx.x - 32, wwarp = wtid >> 5;
        const uint32_t ring_s = smem_u32(ring);
        uint32_t J = 0;  // chunks of this CTA consumed so far (the producer numbers them the same way)
        DsPhaseCtx pc{};
        pc.vec_s = smem_u32(vec);
        unsigned bar_target = 0;
        bool ok = true, pending = false;
        const int r0o = S->plan.er0[DSE_WO], nown = S->plan.en[DSE_WO];  // this CTA's slice of the channels = its rows of att.output / ffn.value
        uint32_t lt = 0;  // layers run so far: the table of the current layer sits in S->layer[lt & 1]

        auto stage_layer = [&](int l, uint32_t slot) {
            static_assert(sizeof(DsLayer) % 4 == 0, "DsLayer is copied word by word");
            const uint32_t* src = reinterpret_cast<const uint32_t*>(P.layers + l);
            uint32_t* dst = reinterpret_cast<uint32_t*>(&S->layer[slot & 1]);
            for (int i = wtid; i < (int)(sizeof(DsLayer) / 4); i += kDsConsumers) dst[i] = __ldg(src + i);
        };
        // Grid barrier in two halves: arrive as soon as this CTA's outputs are stored, wait just before the first load of
        // another CTA's outputs; what lies between (parameter staging of the next phase) overlaps the other CTAs' tails.
        // The counter only ever grows, so a CTA must have seen barrier n complete before it arrives on barrier n + 1
        // (otherwise its second arrival could stand in for a CTA that has not reached barrier n yet).
        auto bar_wait = [&]() -> bool {
            if (!pending) return *abort_flag == 0;
            pending = false;
            if (wtid == 0) {
                bool got = false;
                for (uint32_t i = 0; i < kDsBarSpin; ++i) {
                    unsigned v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(P.grid_bar) : "memory");
                    if ((int)(v - bar_target) >= 0) {
                        got = true;
                        break;
                    }
                    if ((i & 255u) == 255u && *abort_flag) break;
                }
                if (!got) {
                    atomicCAS(&S->abort_where, 0, 3 | (int)(bar_target << 4));
                    *abort_flag = 1;
                }
            }
            ds_consumer_sync();
            return *abort_flag == 0;
        };
        auto bar_arrive = [&]() {
            bar_wait();
            ds_consumer_sync();
            if (wtid == 0) {
                // one release operation instead of a fence and a relaxed atomic (the bar.sync above ordered the other warps' stores
                // before this thread)
                asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(P.grid_bar) : "memory");
            }
            bar_target += (unsigned)G;
            pending = true;
        };
        // (scale, zero) of the int8 rows this CTA owns in the coming phase -> shared memory (weights: no dependency on a barrier)
        auto stage_scales = [&](const DsEntry* ents, int e0, int cnt) {
            int off = 0;
            for (int i = 0; i < cnt; ++i) {
                const DsEntry& E = ents[i];
                const int r0 = S->plan.er0[e0 + i], n = E.M > 0 ? S->plan.en[e0 + i] : 0;
                if (E.is_i8 != 1 || n <= 0) continue;
                for (int q = wtid; q < n && off + q < kDsMaxRows; q += kDsConsumers) {
                    S->ws[off + q] = __ldg(E.wscale + r0 + q);
                    S->wz[off + q] = __ldg(E.wzero + r0 + q);
                }
                off += n;
            }
        };

        for (int t = 0; t < P.n_tokens && ok; ++t) {
            const bool do_head = P.argmax_feed || t == P.n_tokens - 1;
            if (wtid == 0) {
                uint32_t tk = (P.argmax_feed && t > 0) ? S->tok : (P.tok_from_list ? P.tok_list[t] : P.tokens[0]);
                if (tk >= (uint32_t)P.V) {
                    atomicOr(P.status, 1);
                    tk = 0;
                }
                S->tok = tk;
            }
            if (t == 0) stage_layer(0, 0);
            ds_consumer_sync();
            const uint32_t tok = S->tok;

            for (int l = 0; l < P.L && ok; ++l, ++lt) {
                const DsLayer& Ly = S->layer[lt & 1];
                float* tm_l = P.tmix_x + (size_t)l * P.lay_x + (size_t)P.slot * C;
                float* cm_l = P.cmix_x + (size_t)l * P.lay_x + (size_t)P.slot * C;
                float* wkv_l = P.wkv + (size_t)l * P.lay_s + (size_t)P.slot * P.H * 4096;
                DS_STAMP(0);
                DS_STAMP_ALL(0);
                // ================= phase 1: LN1 + token shift -> r, k, v, rank projections =================
                {
                    // this CTA's two operand vectors: the shifted input of its big matrix (receptance, key and value rows lie on
                    // disjoint thirds of the CTAs) and that of its rank projection (disjoint groups as well)
                    const int re = S->plan.rank_entry;
                    const int be = S->plan.en[DSE_WR] > 0 ? DSE_WR : S->plan.en[DSE_WK] > 0 ? DSE_WK : DSE_WV;
                    const float* bmix = Ly.e[be].mix;
                    const float* rmix = re >= 0 ? Ly.e[re].mix : bmix;
                    stage_scales(&Ly.e[DSE_W1], DSE_W1, 7);
                    if (!(ok = bar_wait())) break;
                    DS_STAMP(10);
                    DS_STAMP_ALL(10);
                    float4 xv[NG], lw[NG], lb[NG], pv[NG];
#pragma unroll
                    for (int gi = 0; gi < NG; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                        if (l > 0) xv[gi] = ds_ldcg4(P.x + k);
                        pv[gi] = ds_ldcg4(tm_l + k);
                        lw[gi] = ds_ldg4(Ly.ln1_w + k);
                        lb[gi] = ds_ldg4(Ly.ln1_b + k);
                    }
                    if (l == 0) {
                        // x = LN0(embedding row): every CTA builds the whole vector itself
                        const __half* erow = P.emb + (size_t)tok * C;
                        float4 w0v[NG], b0v[NG];
#pragma unroll
                        for (int gi = 0; gi < NG; ++gi) {
                            const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                            const uint2 raw = __ldg(reinterpret_cast<const uint2*>(erow + k));
                            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                            xv[gi] = make_float4(a.x, a.y, b.x, b.y);
                            w0v[gi] = ds_ldg4(P.ln0_w + k);
                            b0v[gi] = ds_ldg4(P.ln0_b + k);
                        }
                        float m0, i0;
                        ds_ln_stats<NG>(S, C, xv, wtid, m0, i0);
#pragma unroll
                        for (int gi = 0; gi < NG; ++gi) xv[gi] = ds_ln_apply(xv[gi], m0, i0, w0v[gi], b0v[gi]);
                    }
                    DS_STAMP(15);
                    // the two mix vectors are requested before the statistics: their latency hides behind the two block-wide sums
                    float4 mx0[NG], mx1[NG];
#pragma unroll
                    for (int gi = 0; gi < NG; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                        mx0[gi] = ds_ldg4(bmix + k);
                        mx1[gi] = ds_ldg4(rmix + k);
                    }
                    float mean, inv;
                    ds_ln_stats<NG>(S, C, xv, wtid, mean, inv);
                    DS_STAMP(16);
                    float4 val[2][NG];
#pragma unroll
                    for (int gi = 0; gi < NG; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                        const float4 m0 = mx0[gi], m1 = mx1[gi];
                        const float4 cur = ds_ln_apply(xv[gi], mean, inv, lw[gi], lb[gi]);
                        const float4 del = make_float4(pv[gi].x - cur.x, pv[gi].y - cur.y, pv[gi].z - cur.z, pv[gi].w - cur.w);
                        if (g4 < C / 4) {
                            const float xe[4] = {xv[gi].x, xv[gi].y, xv[gi].z, xv[gi].w}, ce[4] = {cur.x, cur.y, cur.z, cur.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int o = 4 * g4 + e - r0o;
                                if (o >= 0 && o < nown) {
                                    S->xs_own[o] = xe[e];
                                    S->ts_own[o] = ce[e];  // LN1(x): the new time-mix shift state, stored after barrier 2
                                }
                            }
                        }
                        val[0][gi] = ds_mix4(cur, m0, del);
                        val[1][gi] = ds_mix4(cur, m1, del);
                    }
                    DS_STAMP(17);
                    const bool i8[2] = {Ly.e[be].is_i8 != 0, false};
#ifdef RSV_DS_DEBUG
                    ds_emit<2, NG>(S, vec, C, i8, [&](int v, int gi) { return val[v][gi]; }, wtid, Ly.e[be].is_i8 == 2, (P.dbg && cta == 0 && t == 1 && l == 1) ? P.dbg + 52 : nullptr);
#else
                    ds_emit<2, NG>(S, vec, C, i8, [&](int v, int gi) { return val[v][gi]; }, wtid, Ly.e[be].is_i8 == 2);
#endif
                }
                DS_STAMP(1);
                DS_STAMP_ALL(1);
#ifdef RSV_DS_DEBUG
                pc.dbg = (P.dbg && cta == 0 && t == 1 && l == 1) ? P.dbg + 20 : nullptr;
#endif
                {
                    const int nc = l == 0 ? S->plan.phn_l0 : S->plan.phn[DSP_P1];
                    pc.k0 = S->plan.ph0[DSP_P1] + (S->plan.phn[DSP_P1] - nc);  // layer 0: the v-gate projection's chunks (first in the list of a CTA that has them) are skipped
                    if (!(ok = ds_consume(P, S, Ly.e, ring_s, J, nc, pc, wwarp, lane))) break;
                    J += (uint32_t)nc;
                }
                DS_STAMP(2);
                DS_STAMP_ALL(2);
                bar_arrive();

                // ================= phase 2: one CTA per head =================
                {
                    const int h = ds_head_of_cta(cta, l, P.H, G);
                    if (h >= 0) {
                        // state: 8 threads per row, 8 columns each; back-projections: threads 0-255 (4 per channel) do decay, a and the
                        // v gate, threads 256-511 the (longer) output gate
                        const int rrow = wtid >> 3, oct = wtid & 7, ch = h * 64 + rrow;
                        const int drow = (wtid & 255) >> 2, quad = wtid & 3, dch = h * 64 + drow;
                        const bool upper = wtid >= 256;
                        float* srow = wkv_l + ((size_t)h * 64 + rrow) * 64 + oct * 8;
                        const float p_w0 = __ldg(Ly.w0 + dch), p_a0 = __ldg(Ly.a0 + dch), p_kk = __ldg(Ly.k_k + dch), p_ka = __ldg(Ly.k_a + dch), p_rk = __ldg(Ly.r_k + dch);
                        const float p_v0 = l > 0 ? __ldg(Ly.v0 + dch) : 0.f;
                        const float p_gw = __ldg(Ly.lnx_w + ch), p_gb = __ldg(Ly.lnx_b + ch);
                        if (!(ok = bar_wait())) break;
                        DS_STAMP(11);
                        const float p_vf = l > 0 ? __ldcg(P.vfirst + dch) : 0.f;
                        // rank-space vectors and r, k, v of this head -> shared memory
                        for (int q = wtid; q < nmid + 3 * 64; q += kDsConsumers) {
                            const int qq = q - nmid;
                            const float v2 = q < nmid ? __ldcg(P.mid + q) : __ldcg(P.rkv + (size_t)(qq >> 6) * C + h * 64 + (qq & 63));
                            if (q < nmid)
                                sc_mid[q] = v2;
                            else
                                S->hv[qq] = v2;
                        }
                        ds_consumer_sync();
                        DS_STAMP(18);
                        // a row of a back-projection matrix times its rank-space vector: four threads split the rank dimension in contiguous quarters
                        auto dot_q = [&](const __half* W, int mid, const float* v) {
                            float a0 = 0.f, a1 = 0.f;
                            const int ql = mid >> 2;
                            if ((mid & 3) == 0 && (ql & 7) == 0) {
                                // 8 weights (one 16-byte read) against 8 vector elements (two 16-byte reads) per step, two accumulation chains
                                const __half* wrow = W + quad * ql;
                                const float* vv = v + quad * ql;
                                for (int q = 0; q < ql; q += 8) {
                                    const uint4 pk = *reinterpret_cast<const uint4*>(wrow + q);
                                    const float4 x0 = *reinterpret_cast<const float4*>(vv + q), x1 = *reinterpret_cast<const float4*>(vv + q + 4);
                                    const float2 f0 = ds_half2_bits_to_float2(pk.x), f1 = ds_half2_bits_to_float2(pk.y), f2 = ds_half2_bits_to_float2(pk.z),
                                                 f3 = ds_half2_bits_to_float2(pk.w);
                                    a0 = fmaf(f0.x, x0.x, a0);
                                    a1 = fmaf(f0.y, x0.y, a1);
                                    a0 = fmaf(f1.x, x0.z, a0);
                                    a1 = fmaf(f1.y, x0.w, a1);
                                    a0 = fmaf(f2.x, x1.x, a0);
                                    a1 = fmaf(f2.y, x1.y, a1);
                                    a0 = fmaf(f3.x, x1.z, a0);
                                    a1 = fmaf(f3.y, x1.w, a1);
                                }
                            } else {
                                for (int q = quad; q < mid; q += 4) a0 = fmaf(__half2float(W[q]), v[q], a0);
                            }
                            float a = a0 + a1;
                            a += __shfl_xor_sync(0xffffffffu, a, 1);
                            return a + __shfl_xor_sync(0xffffffffu, a, 2);
                        };
                        const int vb = l > 0 ? 64 * P.vm * 2 : 0;
                        // the three chunks of the head's back-projection rows: J, J + 1, J + 2
                        const uint32_t iA = J, iB = J + 1, iC = J + 2;
                        J += 3;
                        auto wait_chunk = [&](uint32_t idx) {
                            const bool w = mbar_wait(&S->full[idx % kDsBars], (idx / kDsBars) & 1u, abort_flag);
                            if (!w) atomicCAS(&S->abort_where, 0, 4 | (int)(idx << 4));
                            return __all_sync(0xffffffffu, w);
                        };
                        if (!wait_chunk(iA)) {
                            ok = false;
                            break;
                        }
                        DS_STAMP(55);
                        const uint8_t* cA = ring + S->desc[iA % kDsBars].ring_off;
                        float dw = 0.f, da = 0.f, dv = 0.f, dg = 0.f;
                        if (!upper) {
                            const __half* w2s = reinterpret_cast<const __half*>(cA);
                            dw = dot_q(w2s + (size_t)drow * P.wm, P.wm, sc_mid);
                            da = dot_q(w2s + (size_t)64 * P.wm + (size_t)drow * P.am, P.am, sc_mid + P.wm);
                        }
                        DS_STAMP(57);
                        if (P.head_early && !upper) {
                            // the ring cannot hold all three chunks: the first goes back as soon as the 8 warps that read it are done
                            asm volatile("bar.sync 2, 256;" ::: "memory");
                            if (wtid == 0) mbar_arrive(&S->empty[iA % kDsBars]);
                        }
                        if (!wait_chunk(iB) || !wait_chunk(iC)) {
                            ok = false;
                            break;
                        }
                        DS_STAMP(56);
                        const uint8_t* cB = ring + S->desc[iB % kDsBars].ring_off;
                        const uint8_t* cC = ring + S->desc[iC % kDsBars].ring_off;
                        if (upper) {
                            const __half* g2row = drow < 32 ? reinterpret_cast<const __half*>(cB + vb) + (size_t)drow * P.gm : reinterpret_cast<const __half*>(cC) + (size_t)(drow - 32) * P.gm;
                            dg = dot_q(g2row, P.gm, sc_mid + P.wm + P.am + P.vm);
                        } else if (l > 0) {
                            dv = dot_q(reinterpret_cast<const __half*>(cB) + (size_t)drow * P.vm, P.vm, sc_mid + P.wm + P.am);
                        }
                        // this thread's eight state elements: requested only now, so that they do not occupy registers during the dot products
                        // (the epilogue below and the block-wide sums cover most of their latency)
                        const float4 s4a = ds_ldcg4(srow), s4b = ds_ldcg4(srow + 4);
                        // per-channel quantities of the head -> shared memory; ||kk||^2 and the bonus sum over the 64 channels
                        float ssp = 0.f, srp = 0.f;
                        if (quad == 0) {
                            if (upper) {
                                S->hv[8 * 64 + drow] = dg;
                            } else {
                                const float wdec = expf((1.0f / (1.0f + expf(-(dw + p_w0)))) * kDecayScale);
                                const float aa = 1.0f / (1.0f + expf(-(da + p_a0)));
                                const float rr = S->hv[drow], kk0 = S->hv[64 + drow];
                                float vv0 = S->hv[128 + drow];
                                if (l == 0) {
                                    P.vfirst[dch] = vv0;
                                    P.state_vfirst[(size_t)P.slot * C + dch] = vv0;
                                } else {
                                    const float gate = 1.0f / (1.0f + expf(-(dv + p_v0)));
                                    vv0 = vv0 + gate * (p_vf - vv0);
                                }
                                const float kkj = kk0 * p_kk;
                                const float kt = kk0 + p_ka * (kk0 * aa - kk0);
                                S->hv[3 * 64 + drow] = wdec;
                                S->hv[4 * 64 + drow] = kkj;
                                S->hv[5 * 64 + drow] = aa;
                                S->hv[6 * 64 + drow] = kt;
                                S->hv[7 * 64 + drow] = vv0;
                                ssp = kkj * kkj;
                                srp = rr * kt * p_rk;
                            }
                        }
                        ssp = warp_sum(ssp);
                        srp = warp_sum(srp);
                        if (lane == 0) {
                            S->red_a[wwarp] = ssp;
                            S->red_b[wwarp] = srp;
                        }
                        DS_STAMP(19);
                        ds_consumer_sync();  // also: every warp is done with the three chunks
                        if (wtid == 0) {
                            if (!P.head_early) mbar_arrive(&S->empty[iA % kDsBars]);
                            mbar_arrive(&S->empty[iB % kDsBars]);
                            mbar_arrive(&S->empty[iC % kDsBars]);
                        }
                        float ss = 0.f, srk = 0.f;
#pragma unroll
                        for (int w = 0; w < 8; w += 4) {
                            ss += (S->red_a[w] + S->red_a[w + 1]) + (S->red_a[w + 2] + S->red_a[w + 3]);
                            srk += (S->red_b[w] + S->red_b[w + 1]) + (S->red_b[w + 2] + S->red_b[w + 3]);
                        }
                        const float invn = 1.0f / fmaxf(sqrtf(ss), kL2Eps);
                        const float vv_row = S->hv[7 * 64 + rrow];
                        float St[8] = {s4a.x, s4a.y, s4a.z, s4a.w, s4b.x, s4b.y, s4b.z, s4b.w};
                        // this thread's eight columns of the head's vectors (16-byte reads)
                        auto ld8 = [&](int arr, float (&o)[8]) {
                            const float4 lo = *reinterpret_cast<const float4*>(&S->hv[arr * 64 + oct * 8]), hi = *reinterpret_cast<const float4*>(&S->hv[arr * 64 + oct * 8 + 4]);
                            o[0] = lo.x, o[1] = lo.y, o[2] = lo.z, o[3] = lo.w, o[4] = hi.x, o[5] = hi.y, o[6] = hi.z, o[7] = hi.w;
                        };
                        float kkh[8], wv[8], av[8], ktv[8], rv[8], sa = 0.f;
                        ld8(4, kkh);
                        ld8(3, wv);
                        ld8(5, av);
                        ld8(6, ktv);
                        ld8(0, rv);
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            kkh[q] *= invn;
                            sa = fmaf(St[q], kkh[q], sa);
                        }
                        sa += __shfl_xor_sync(0xffffffffu, sa, 1);
                        sa += __shfl_xor_sync(0xffffffffu, sa, 2);
                        sa += __shfl_xor_sync(0xffffffffu, sa, 4);
                        float y = 0.f;
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const float bq = kkh[q] * (-av[q]);
                            St[q] = fmaf(St[q], wv[q], fmaf(sa, bq, vv_row * ktv[q]));
                            y = fmaf(St[q], rv[q], y);
                        }
                        y += __shfl_xor_sync(0xffffffffu, y, 1);
                        y += __shfl_xor_sync(0xffffffffu, y, 2);
                        y += __shfl_xor_sync(0xffffffffu, y, 4);
                        *reinterpret_cast<float4*>(srow) = make_float4(St[0], St[1], St[2], St[3]);
                        *reinterpret_cast<float4*>(srow + 4) = make_float4(St[4], St[5], St[6], St[7]);
                        DS_STAMP(50);
                        const float gmean = ds_block_sum(oct == 0 ? y : 0.f, S->red_c, wwarp, lane) / 64.0f;
                        const float d = y - gmean;
                        const float var = ds_block_sum(oct == 0 ? d * d : 0.f, S->red_c + 16, wwarp, lane) / 64.0f + kGnEps;
                        if (oct == 0) P.yg[ch] = (d * (1.0f / sqrtf(var)) * p_gw + p_gb + srk * vv_row) * S->hv[8 * 64 + rrow];
                    }
                }
                DS_STAMP(3);
                DS_STAMP_ALL(3);
                bar_arrive();

                // ================= phase 3: att.output, x += =================
                {
                    stage_scales(&Ly.e[DSE_WO], DSE_WO, 1);
                    if (!(ok = bar_wait())) break;
                    DS_STAMP(12);
                    DS_STAMP_ALL(12);
                    if (wtid < nown) tm_l[r0o + wtid] = S->ts_own[wtid];  // new time-mix shift state (every reader of the old one is past barrier 1)
                    float4 yv[NG];
#pragma unroll
                    for (int gi = 0; gi < NG; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                        yv[gi] = ds_ldcg4(P.yg + k);
                    }
                    const bool i8[1] = {Ly.e[DSE_WO].is_i8 != 0};
                    ds_emit<1, NG>(S, vec, C, i8, [&](int, int gi) { return yv[gi]; }, wtid, Ly.e[DSE_WO].is_i8 == 2);
                    DS_STAMP(4);
                    DS_STAMP_ALL(4);
#ifdef RSV_DS_DEBUG
                pc.dbg = (P.dbg && cta == 0 && t == 1 && l == 1) ? P.dbg + 24 : nullptr;
#endif
                    pc.k0 = S->plan.ph0[DSP_P3];
                    if (!(ok = ds_consume(P, S, Ly.e, ring_s, J, S->plan.phn[DSP_P3], pc, wwarp, lane))) break;
                    J += (uint32_t)S->plan.phn[DSP_P3];
                }
                DS_STAMP(5);
                DS_STAMP_ALL(5);
                bar_arrive();

                // ================= phase 4: LN2 + shift -> relu(ffn.key)^2 =================
                {
                    stage_scales(&Ly.e[DSE_WFK], DSE_WFK, 1);
                    const int lnext = l + 1 < P.L ? l + 1 : 0;
                    stage_layer(lnext, lt + 1);  // the table of the layer that runs next (the first one again after the last)
                    if (!(ok = bar_wait())) break;
                    DS_STAMP(13);
                    DS_STAMP_ALL(13);
                    float4 lw[NG], lb[NG], pv[NG], mx[NG], xv[NG];
#pragma unroll
                    for (int gi = 0; gi < NG; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                        xv[gi] = ds_ldcg4(P.x + k);
                        pv[gi] = ds_ldcg4(cm_l + k);
                        lw[gi] = ds_ldg4(Ly.ln2_w + k);
                        lb[gi] = ds_ldg4(Ly.ln2_b + k);
                        mx[gi] = ds_ldg4(Ly.ffn_x_k + k);
                    }
                    float mean, inv;
                    ds_ln_stats<NG>(S, C, xv, wtid, mean, inv);
                    float4 val[NG];
#pragma unroll
                    for (int gi = 0; gi < NG; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi;
                        const float4 cur = ds_ln_apply(xv[gi], mean, inv, lw[gi], lb[gi]);
                        const float4 del = make_float4(pv[gi].x - cur.x, pv[gi].y - cur.y, pv[gi].z - cur.z, pv[gi].w - cur.w);
                        val[gi] = ds_mix4(cur, mx[gi], del);
                        if (g4 < C / 4) {
                            const float ce[4] = {cur.x, cur.y, cur.z, cur.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int o = 4 * g4 + e - r0o;
                                if (o >= 0 && o < nown) S->cs_own[o] = ce[e];  // new channel-mix shift state, stored after the next barrier
                            }
                        }
                    }
                    const bool i8[1] = {Ly.e[DSE_WFK].is_i8 != 0};
                    ds_emit<1, NG>(S, vec, C, i8, [&](int, int gi) { return val[gi]; }, wtid, Ly.e[DSE_WFK].is_i8 == 2);
                    DS_STAMP(6);
                    DS_STAMP_ALL(6);
#ifdef RSV_DS_DEBUG
                pc.dbg = (P.dbg && cta == 0 && t == 1 && l == 1) ? P.dbg + 28 : nullptr;
#endif
                    pc.k0 = S->plan.ph0[DSP_P4];
                    if (!(ok = ds_consume(P, S, Ly.e, ring_s, J, S->plan.phn[DSP_P4], pc, wwarp, lane))) break;
                    J += (uint32_t)S->plan.phn[DSP_P4];
                }
                DS_STAMP(7);
                DS_STAMP_ALL(7);
                bar_arrive();

                // ================= phase 5: ffn.value (K = F = 4 C), x += =================
                {
                    stage_scales(&Ly.e[DSE_WFV], DSE_WFV, 1);
                    if (!(ok = bar_wait())) break;
                    DS_STAMP(14);
                    DS_STAMP_ALL(14);
                    if (wtid < nown) cm_l[r0o + wtid] = S->cs_own[wtid];
                    float4 hv4[NG5];
#pragma unroll
                    for (int gi = 0; gi < NG5; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi, k = g4 < C ? 4 * g4 : 0;
                        hv4[gi] = ds_ldcg4(P.hbuf + k);
                    }
                    const bool i8[1] = {Ly.e[DSE_WFV].is_i8 != 0};
                    ds_emit<1, NG5>(S, vec, 4 * C, i8, [&](int, int gi) { return hv4[gi]; }, wtid, Ly.e[DSE_WFV].is_i8 == 2);
                    DS_STAMP(8);
                    DS_STAMP_ALL(8);
#ifdef RSV_DS_DEBUG
                pc.dbg = (P.dbg && cta == 0 && t == 1 && l == 1) ? P.dbg + 32 : nullptr;
#endif
                    pc.k0 = S->plan.ph0[DSP_P5];
                    if (!(ok = ds_consume(P, S, Ly.e, ring_s, J, S->plan.phn[DSP_P5], pc, wwarp, lane))) break;
                    J += (uint32_t)S->plan.phn[DSP_P5];
                }
                DS_STAMP(9);
                DS_STAMP_ALL(9);
                bar_arrive();
            }
            if (!ok) break;

            // ================= ln_out + head -> logits, arg-max =================
            if (do_head) {
                stage_scales(&P.head, DSE_COUNT, 1);
                if (!(ok = bar_wait())) break;
                float4 lw[NG], lb[NG], xv[NG];
#pragma unroll
                for (int gi = 0; gi < NG; ++gi) {
                    const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                    xv[gi] = ds_ldcg4(P.x + k);
                    lw[gi] = ds_ldg4(P.lno_w + k);
                    lb[gi] = ds_ldg4(P.lno_b + k);
                }
                float mean, inv;
                ds_ln_stats<NG>(S, C, xv, wtid, mean, inv);
                float4 val[NG];
#pragma unroll
                for (int gi = 0; gi < NG; ++gi) val[gi] = ds_ln_apply(xv[gi], mean, inv, lw[gi], lb[gi]);
                const bool i8[1] = {P.head.is_i8 != 0};
                ds_emit<1, NG>(S, vec, C, i8, [&](int, int gi) { return val[gi]; }, wtid, P.head.is_i8 == 2);
                S->best_val[wtid] = -1e30f;
                S->best_idx[wtid] = 0x7fffffff;
                __syncwarp();
#ifdef RSV_DS_DEBUG
                pc.dbg = nullptr;
#endif
                pc.k0 = S->plan.ph0[DSP_HEAD];
                if (!(ok = ds_consume(P, S, nullptr, ring_s, J, S->plan.phn[DSP_HEAD], pc, wwarp, lane))) break;
                J += (uint32_t)S->plan.phn[DSP_HEAD];
                if (P.argmax_feed) {
                    // arg-max: lanes -> warp -> CTA -> grid; ties go to the smaller index
                    __syncwarp();
                    float bv = S->best_val[wtid];
                    int bi = S->best_idx[wtid];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                        if (ov > bv || (ov == bv && oi < bi)) {
                            bv = ov;
                            bi = oi;
                        }
                    }
                    if (lane == 0) {
                        S->red_a[wwarp] = bv;
                        S->red_i[wwarp] = bi;
                    }
                    ds_consumer_sync();
                    if (wtid == 0) {
                        for (int w = 1; w < kDsConsumerWarps; ++w) {
                            const float ov = S->red_a[w];
                            const int oi = S->red_i[w];
                            if (ov > bv || (ov == bv && oi < bi)) {
                                bv = ov;
                                bi = oi;
                            }
                        }
                        P.cand_val[cta] = bv;
                        P.cand_idx[cta] = bi;
                    }
                    bar_arrive();
                    if (!(ok = bar_wait())) break;
                    // every CTA reduces the candidates itself: no further barrier before the next token
                    if (wwarp == 0) {
                        bv = -1e30f;
                        bi = 0x7fffffff;
                        for (int c = lane; c < G; c += 32) {
                            const float ov = __ldcg(P.cand_val + c);
                            const int oi = __ldcg(P.cand_idx + c);
                            if (ov > bv || (ov == bv && oi < bi)) {
                                bv = ov;
                                bi = oi;
                            }
                        }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
                            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                            if (ov > bv || (ov == bv && oi < bi)) {
                                bv = ov;
                                bi = oi;
                            }
                        }
                        if (lane == 0) {
                            if (bi == 0x7fffffff) bi = 0;
                            S->tok = (uint32_t)bi;
                            if (cta == 0) {
                                P.tokens[0] = (uint32_t)bi;
                                if (P.seq) {
                                    const int cnt = P.seq_cnt[0];
                                    if (cnt < P.seq_cap) P.seq[cnt] = (uint32_t)bi;
                                    P.seq_cnt[0] = cnt + 1;
                                }
                            }
                        }
                    }
                    ds_consumer_sync();
                }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) {
        atomicOr(P.status, 32);
        // where: a CTA that gave up on its own chunks or ring outranks the CTAs that gave up on the grid barrier because of it
        if (S->abort_where) atomicMax(P.status + 1, (((S->abort_where & 15) == 3 ? 1 : 2) << 28) | (cta << 20) | (S->abort_where & 0xFFFFF));
    }
}

// Writes the second copy of the weights: for every layer and every CTA of the decode kernel, the CTA's chunks in the order it
// consumes them (rows padded to `stride`, the head's rows in a region of their own).  Launched once per model with the decode
// kernel's grid size; CTA c lays out the region of decode CTA c.
__global__ void __launch_bounds__(256) ds_retile_kernel(const __grid_constant__ DsParams P, char* wstream, long long wslot, char* hstream, long long hslot) {
    __shared__ DsPlan pl;
    const int G = gridDim.x, cta = blockIdx.x;
    if (threadIdx.x == 0) ds_build_plan(pl, P.layers[P.L > 1 ? 1 : 0].e, P.head, cta, G, 0u);
    __syncthreads();
    auto copy_chunk = [&](const DsEntry& E, const DsChunk& c, char* dst) {
        const int nr = c.nr_steps & 0xFFFF, piece = c.piece_np & 0xFFFF, e = c.e_flags_row0 & 0xFF, row0 = c.e_flags_row0 >> 16, per_row = c.stride >> 4;
        const char* src = E.base + (size_t)(pl.er0[e] + row0) * (size_t)E.row_stride + (size_t)piece * E.piece_bytes;
        for (int i = threadIdx.x; i < nr * per_row; i += blockDim.x) {
            const int row = i / per_row, col = (i % per_row) * 16;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (col < E.piece_bytes) v = *reinterpret_cast<const uint4*>(src + (size_t)row * E.row_stride + col);
            *reinterpret_cast<uint4*>(dst + (size_t)row * c.stride + col) = v;
        }
        if ((c.e_flags_row0 >> 8) & 4) {  // the rows' (scale, zero) words of this piece's groups: [group][16 rows], zero for rows past nr
            const int ngp = E.piece_bytes >> 7, kgroups = E.row_stride >> 7;
            uint32_t* zd = reinterpret_cast<uint32_t*>(dst + (size_t)nr * c.stride);
            for (int i = threadIdx.x; i < ngp * kDsTileRows; i += blockDim.x) {
                const int gi = i / kDsTileRows, row = i % kDsTileRows;
                zd[i] = row < nr ? E.sz[(size_t)(pl.er0[e] + row0 + row) * kgroups + (size_t)piece * ngp + gi] : 0u;
            }
        }
    };
    auto copy_raw = [&](const void* src, int bytes, char* dst) {
        for (int i = threadIdx.x * 16; i < bytes; i += blockDim.x * 16) *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>((const char*)src + i);
    };
    for (int l = 0; l < P.L; ++l) {
        const DsLayer& Ly = P.layers[l];
        char* dst = wstream + ((size_t)l * G + cta) * (size_t)wslot;
        for (int ph = DSP_P1; ph <= DSP_P5; ++ph) {
            for (int k = pl.ph0[ph]; k < pl.ph0[ph] + pl.phn[ph]; ++k) {
                const DsChunk& c = pl.ctab[k];
                if (l == 0 && ((c.e_flags_row0 >> 8) & 2)) continue;
                copy_chunk(Ly.e[c.e_flags_row0 & 0xFF], c, dst);
                dst += c.cb;
            }
            if (ph == DSP_P1) {
                const int h = ds_head_of_cta(cta, l, P.H, G);
                if (h >= 0) {  // the head's back-projection rows: w2, a2 | v2 (layers > 0), first 32 g2 rows | the other 32 g2 rows
                    copy_raw(Ly.w2 + (size_t)h * 64 * P.wm, 64 * P.wm * 2, dst);
                    dst += 64 * P.wm * 2;
                    copy_raw(Ly.a2 + (size_t)h * 64 * P.am, 64 * P.am * 2, dst);
                    dst += 64 * P.am * 2;
                    if (l > 0) {
                        copy_raw(Ly.v2 + (size_t)h * 64 * P.vm, 64 * P.vm * 2, dst);
                        dst += 64 * P.vm * 2;
                    }
                    copy_raw(Ly.g2 + (size_t)h * 64 * P.gm, 64 * P.gm * 2, dst);
                    dst += 64 * P.gm * 2;
                }
            }
        }
    }
    char* dst = hstream + (size_t)cta * (size_t)hslot;
    for (int k = pl.ph0[DSP_HEAD]; k < pl.ph0[DSP_HEAD] + pl.phn[DSP_HEAD]; ++k) {
        copy_chunk(P.head, pl.ctab[k], dst);
        dst += pl.ctab[k].cb;
    }
}

}  // namespace rsv
