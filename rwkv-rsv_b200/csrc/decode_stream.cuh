// Batch-1 decode as a row-owner weight-streaming GEMV inside one persistent launch.
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
//               per row, issued by the lanes in parallel) into a byte-granular ring in shared memory, a chunk (up to
//               16 rows of one matrix) per mbarrier.  It never waits on a grid barrier, only on ring space, so HBM
//               keeps streaming while the other warps synchronise: barriers cost latency, not bandwidth.
//   warps 1-8   consumers.  Per phase they build the activation vector in shared memory (LayerNorm, token shift,
//               fixed-point digits), then every warp takes rows of the chunk: a lane keeps its K slice of the
//               activation in REGISTERS for the whole matrix, reads 16-byte pieces of the row from the ring, and the
//               warp reduces once per row.
// Arithmetic.  int8 matrices: the u8 codes q are multiplied as they are (dp4a, u8 x s8) with D = 4 signed base-128
// digits of the fixed-point activation t = rint(x / e 2^27), e = 2^ceil(log2 max|x|); the four int32 sums recombine
// to Q = sum_k q_k t_k exactly (int64), and with the container's per-row (scale s, zero z)
// y = e 2^-27 (s Q + z T), T = sum_k t_k: the same numbers the tensor-core kernels produce, with no accumulation
// rounding and no dependence on the schedule.  fp16 matrices (head, rank projections, fp16 checkpoints): fp32 FMA
// on the converted halves, lane partial sums in a fixed order, then a shuffle tree.
// Phases per layer, one grid barrier after each (bounded spin):
//   1  LN1 + token shift -> r, k, v and the four rank projections (tanh / sigmoid applied)
//   2  one CTA per head: rank back-projections (their rows arrive through the ring too), decay / a / v-gate / g,
//      WKV-7 state update in place, GroupNorm, bonus, gate
//   3  att.output, x += ...      4  LN2 + shift -> relu(ffn.key)^2      5  ffn.value (K = F in pieces of C), x += ...
// then ln_out + head -> logits, arg-max across CTAs, next token.
// All waits are bounded; on expiry bit 2 of the status word is set, every role drains its copies in flight and exits.
#pragma once
#include "tc_linear.cuh"

namespace rsv {

constexpr int kDsConsumerWarps = 8;
constexpr int kDsConsumers = kDsConsumerWarps * 32;  // 256
constexpr int kDsThreads = kDsConsumers + 32;        // + producer warp
constexpr int kDsBars = 8;                           // chunks in flight (mbarrier pairs)
constexpr int kDsChunkBytes = 40 * 1024;             // target size of a chunk of rows
constexpr int kDsMaxRows = 512;                      // rows of one matrix per CTA whose (scale, zero) are staged per phase
constexpr int kDsMaxSlice = 32;                      // channels of the residual stream per CTA
constexpr int kDsP = 27;                             // fixed-point bits of the activation digits (4 digits of 7 bits)
constexpr uint32_t kDsBarSpin = 1u << 22;

// What a finished dot product becomes.
enum DsOut : int { DSO_R = 0, DSO_K, DSO_V, DSO_MID_TANH, DSO_MID, DSO_MID_SIG, DSO_XADD, DSO_H, DSO_LOGITS };

// One matrix of a phase.
struct DsEntry {
    const char* base;     // fp16 [M,K] or u8 [M,K], row-major
    const float* wscale;  // int8: [M] per-row scale and zero of the container
    const float* wzero;
    const float* mix;     // rank projections: the token-shift mix vector of their input; null otherwise
    int M;                // output rows (0: the entry does not exist in this layer)
    int row_bytes;        // bytes of one piece of a row: C (int8) or 2 C (fp16)
    int row_stride;       // bytes between rows
    int npieces;          // K / C
    int is_i8;
    int xvec;             // which vector of the phase's operand area the rows are multiplied with
    int out;              // DsOut
    int out_off;          // offset inside the rank-space vector for DSO_MID*
    int rot;              // the CTA with index c owns the row range of virtual index (c + rot) mod G
    int pad;
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
    long long lay_x, lay_s;                // floats between consecutive layers of the shift states / the WKV states
    float *tmix_x, *wkv, *cmix_x;          // state bases (layer 0, slot 0)
    float* state_vfirst;                   // [cap][C]
    float *x, *yg, *vfirst;                // [C]
    float* rkv;                            // [3][C]
    float* mid;                            // [wm+am+vm+gm]
    float* hbuf;                           // [F]
    uint32_t* tokens;                      // [1] current input token (read at start, written after arg-max)
    const uint32_t* tok_list;              // [n_tokens], used when tok_from_list
    uint32_t* seq;
    int* seq_cnt;
    int seq_cap;
    float* logits;  // [V]
    float* cand_val;
    int* cand_idx;  // [G]
    unsigned* grid_bar;
    int* status;
    int n_tokens, tok_from_list, argmax_feed;
    int ring_bytes;    // shared-memory ring
    int vec_floats;    // operand area, in 4-byte elements: max(5 C, F)
    long long* dbg;    // optional time stamps (built with -DRSV_DS_DEBUG only)
};

// ---- small helpers ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void ds_consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kDsConsumers) : "memory"); }
__device__ __forceinline__ int ds_dp4a_us(uint32_t a_u8x4, uint32_t b_s8x4, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_s8x4), "r"(c));
    return d;
}
__device__ __forceinline__ uint4 ds_lds128(uint32_t saddr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
    return v;
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
// rows of an M-row matrix owned by virtual CTA index vc of G
__device__ __forceinline__ int ds_row_begin(int vc, int M, int G) { return (int)(((long long)vc * M) / G); }
// rows per chunk: about kDsChunkBytes, a multiple of the consumer warp count (two rows per warp) when rows are short
__host__ __device__ inline int ds_rows_per_chunk(int row_bytes) {
    const int fit = kDsChunkBytes / row_bytes;
    return fit >= 16 ? 16 : (fit >= 8 ? 8 : (fit >= 4 ? 4 : (fit >= 2 ? 2 : 1)));
}
// the CTA that runs head h of layer l (H <= G: heads spread with a stride, rotated per layer so that the extra bytes of a
// head's back-projection rows do not always land on the same SMs); -1 when CTA `cta` has no head in that layer
__host__ __device__ inline int ds_head_of_cta(int cta, int l, int H, int G) {
    if (H > G) return -2;  // several heads per CTA: h = cta, cta + G, ...
    const int stride = G / H;
    const int d = ((cta - (l * 37) % G) % G + G) % G;
    if (d % stride) return -1;
    const int h = d / stride;
    return h < H ? h : -1;
}

// Four activations -> their base-128 digits, packed for dp4a: word d holds digit d (0 = most significant) of the four
// consecutive k.  Adds the four fixed-point values to `tsum`.
__device__ __forceinline__ uint4 ds_digits4(float4 v, float mult, long long& tsum) {
    const float lim = (float)(1 << kDsP);
    float f[4] = {v.x * mult, v.y * mult, v.z * mult, v.w * mult};
    uint32_t w0 = 0, w1 = 0, w2 = 0, w3 = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float q = fminf(fmaxf(f[j], -lim), lim);
        int t = (q == q) ? __float2int_rn(q) : 0;
        tsum += t;
        const int d3 = ((t + 64) & 127) - 64;
        t = (t - d3) >> 7;
        const int d2 = ((t + 64) & 127) - 64;
        t = (t - d2) >> 7;
        const int d1 = ((t + 64) & 127) - 64;
        t = (t - d1) >> 7;
        w0 |= (uint32_t)(t & 0xFF) << (8 * j);
        w1 |= (uint32_t)(d1 & 0xFF) << (8 * j);
        w2 |= (uint32_t)(d2 & 0xFF) << (8 * j);
        w3 |= (uint32_t)(d3 & 0xFF) << (8 * j);
    }
    return make_uint4(w0, w1, w2, w3);
}
// exact sum of a 64-bit value over the warp whose magnitude is below 2^40 per lane (two 32-bit reductions)
__device__ __forceinline__ long long ds_warp_sum_ll(long long v) {
    const unsigned lo = __reduce_add_sync(0xffffffffu, (unsigned)(v & 0xFFFF));
    const int hi = __reduce_add_sync(0xffffffffu, (int)(v >> 16));
    return (long long)hi * 65536 + (long long)lo;
}

// ---- shared-memory layout: [ring][operand area: vec_floats x 4 bytes][DsShared][rank-space vector] ----------------
struct DsShared {
    uint64_t full[kDsBars], empty[kDsBars];
    int alloc[kDsBars];  // producer only: bytes (with wrap waste) a chunk in flight holds
    int abort_flag;
    uint32_t tok;
    float red_a[8], red_b[8], red_c[3 * 8];
    int red_i[8];
    long long tsw[3][8];  // per consumer warp: exact sum of the fixed-point values of operand vector v
    int ex[4];            // exponent of the power-of-two scale of operand vector v
    float stats[2];
    float xs_own[kDsMaxSlice];   // this CTA's slice of the residual stream
    float cs_own[kDsMaxSlice];   // pending channel-mix shift state of the slice
    long long qacc[kDsMaxSlice]; // per-row sums over the pieces of a long row (int8: exact; fp16: facc)
    float facc[kDsMaxSlice];
    float ws[kDsMaxRows], wz[kDsMaxRows];  // (scale, zero) of the rows this CTA owns in the current phase
    float hv[8 * 64];                      // the 64-vectors of a head
    DsLayer layer[2];                      // table of the current / next layer
};

// consumer-side view of the ring: every consumer warp walks the same chunk sequence as the producer
struct DsCons {
    uint32_t ring_s;
    int R, head;
    int cur;     // byte offset of the chunk the last wait returned
    uint32_t j;  // chunks waited for so far
};
// Waits for the next chunk (of `bytes` bytes); its offset in the ring is left in cs.cur and its index (for the release) is
// returned; -1 after a timeout / abort.
__device__ __forceinline__ int ds_chunk_wait(DsCons& cs, DsShared* S, int bytes) {
    if (cs.head + bytes > cs.R) cs.head = 0;  // same placement rule as the producer
    cs.cur = cs.head;
    cs.head += bytes;
    const uint32_t idx = cs.j++;
    const bool ok = mbar_wait(&S->full[idx % kDsBars], (idx / kDsBars) & 1u, (volatile int*)&S->abort_flag);
    return __all_sync(0xffffffffu, ok) ? (int)(idx % kDsBars) : -1;
}
__device__ __forceinline__ void ds_chunk_release(DsShared* S, int bar_idx, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(&S->empty[bar_idx]);
}

// dot product of one int8 row piece (in the ring) with the lane's digits: four int32 partial sums, one per digit
template <int KL>
__device__ __forceinline__ void ds_dot_i8(uint32_t row_s, int lane, const uint32_t (&xr)[KL], int (&a)[4]) {
    constexpr int NCH = KL / 16;
    uint4 w[NCH];
#pragma unroll
    for (int i = 0; i < NCH; ++i) w[i] = ds_lds128(row_s + (uint32_t)(lane + 32 * i) * 16u);
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const uint32_t ww[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
            for (int d = 0; d < 4; ++d) a[d] = ds_dp4a_us(ww[g], xr[(i * 4 + g) * 4 + d], a[d]);
    }
}
// dot product of one fp16 row piece with the lane's fp32 activations (four chains, fixed order)
template <int KL>
__device__ __forceinline__ float ds_dot_f16(uint32_t row_s, int lane, const uint32_t (&xr)[KL]) {
    constexpr int NCH = KL / 8;
    float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const uint4 w = ds_lds128(row_s + (uint32_t)(lane + 32 * i) * 16u);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&ww[e]));
            a[e] = fmaf(f.x, __uint_as_float(xr[i * 8 + 2 * e]), a[e]);
            a[e] = fmaf(f.y, __uint_as_float(xr[i * 8 + 2 * e + 1]), a[e]);
        }
    }
    return (a[0] + a[1]) + (a[2] + a[3]);
}

// What the consumer warps need to turn a row's sums into an output.
struct DsPhaseCtx {
    uint32_t vec_s;     // shared-memory address of the operand area
    int stage_off;      // first staged (scale, zero) of the current entry
    float best_val;     // running arg-max of the head rows this warp finished (lane 0)
    int best_idx;
};

__device__ __forceinline__ void ds_store(const DsParams& P, DsShared* S, const DsEntry& E, int m, int rl, float y, DsPhaseCtx& pc) {
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
        default:
            P.logits[m] = y;
            if (y > pc.best_val || (y == pc.best_val && m < pc.best_idx)) {
                pc.best_val = y;
                pc.best_idx = m;
            }
            break;
    }
}

// One matrix of a phase: the rows [r0, r0 + n) this CTA owns, piece after piece, chunk after chunk.  Row i (counted from r0)
// belongs to consumer warp i mod 8.  Returns false after a timeout.
template <int KL>
__device__ __noinline__ bool ds_run_entry(const DsParams& P, DsShared* S, DsCons& cs, const DsEntry& E, int r0, int n, DsPhaseCtx& pc, int wwarp, int lane) {
    constexpr int C = KL * 32;
    const int rpc = ds_rows_per_chunk(E.row_bytes);
    const bool i8 = E.is_i8 != 0;
    const bool mine = n > wwarp;
    float xs = 0.f;
    long long T = 0;
    if (i8) {
        xs = ds_pow2(S->ex[E.xvec] - kDsP);
#pragma unroll
        for (int w = 0; w < 8; ++w) T += S->tsw[E.xvec][w];
    }
    for (int p = 0; p < E.npieces; ++p) {
        // ---- the lane's K slice of the activation, in registers for all rows of this piece ----
        uint32_t xr[KL];
        if (mine) {
            if (E.mix) {
                // rank projections: cur + mix (prev - cur), built from the LayerNorm output and the shift difference in the operand area
                const uint32_t cur_s = pc.vec_s + 3u * C * 4u, del_s = pc.vec_s + 4u * C * 4u;
#pragma unroll
                for (int i = 0; i < KL / 8; ++i) {
                    const int k0 = (lane + 32 * i) * 8;
                    const float4 m0 = __ldg(reinterpret_cast<const float4*>(E.mix + k0)), m1 = __ldg(reinterpret_cast<const float4*>(E.mix + k0 + 4));
                    const uint4 c0 = ds_lds128(cur_s + k0 * 4), c1 = ds_lds128(cur_s + k0 * 4 + 16);
                    const uint4 d0 = ds_lds128(del_s + k0 * 4), d1 = ds_lds128(del_s + k0 * 4 + 16);
                    const float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
                    const uint32_t cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                    const uint32_t dd[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
                    for (int e = 0; e < 8; ++e) xr[i * 8 + e] = __float_as_uint(__uint_as_float(cc[e]) + mm[e] * __uint_as_float(dd[e]));
                }
            } else if (i8) {
                // digits: uint4 (g, c) of the vector holds the four digit words of k = 16 c + 4 g .. + 3, stored at index g * (len / 16) + c
                const int len16 = (E.npieces * C) / 16;
                const uint32_t base = pc.vec_s + (uint32_t)E.xvec * C * 4u;
#pragma unroll
                for (int i = 0; i < KL / 16; ++i)
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const uint4 d = ds_lds128(base + (uint32_t)(g * len16 + p * (C / 16) + lane + 32 * i) * 16u);
                        xr[(i * 4 + g) * 4 + 0] = d.x;
                        xr[(i * 4 + g) * 4 + 1] = d.y;
                        xr[(i * 4 + g) * 4 + 2] = d.z;
                        xr[(i * 4 + g) * 4 + 3] = d.w;
                    }
            } else {
                const uint32_t base = pc.vec_s + ((uint32_t)E.xvec * C + (uint32_t)p * C) * 4u;
#pragma unroll
                for (int i = 0; i < KL / 8; ++i) {
                    const uint4 a = ds_lds128(base + (uint32_t)(lane + 32 * i) * 32u), b = ds_lds128(base + (uint32_t)(lane + 32 * i) * 32u + 16u);
                    xr[i * 8 + 0] = a.x;
                    xr[i * 8 + 1] = a.y;
                    xr[i * 8 + 2] = a.z;
                    xr[i * 8 + 3] = a.w;
                    xr[i * 8 + 4] = b.x;
                    xr[i * 8 + 5] = b.y;
                    xr[i * 8 + 6] = b.z;
                    xr[i * 8 + 7] = b.w;
                }
            }
        }
        const bool first = p == 0, last = p == E.npieces - 1;
        for (int c0 = 0; c0 < n; c0 += rpc) {
            const int nr = min(rpc, n - c0);
            const int bar_idx = ds_chunk_wait(cs, S, nr * E.row_bytes);
            if (bar_idx < 0) return false;
            const uint32_t ch = cs.ring_s + (uint32_t)cs.cur;
            const int ia = c0 + ((wwarp - c0) & 7), ib = ia + 8;
            const bool has_a = ia < c0 + nr, has_b = ib < c0 + nr;
            if (has_a) {
                const uint32_t ra = ch + (uint32_t)(ia - c0) * E.row_bytes, rb = ch + (uint32_t)(ib - c0) * E.row_bytes;
                if (i8) {
                    int qa[4] = {0, 0, 0, 0}, qb[4] = {0, 0, 0, 0};
                    ds_dot_i8<KL>(ra, lane, xr, qa);
                    if (has_b) ds_dot_i8<KL>(rb, lane, xr, qb);
#pragma unroll
                    for (int d = 0; d < 4; ++d) {
                        qa[d] = __reduce_add_sync(0xffffffffu, qa[d]);
                        qb[d] = __reduce_add_sync(0xffffffffu, qb[d]);
                    }
                    if (lane < 2 && (lane == 0 || has_b)) {
                        // lane 0 finishes row a, lane 1 row b
                        const int q0 = lane ? qb[0] : qa[0], q1 = lane ? qb[1] : qa[1], q2 = lane ? qb[2] : qa[2], q3 = lane ? qb[3] : qa[3];
                        const int rl = lane ? ib : ia;
                        long long Q = (((long long)q0 * 128 + q1) * 128 + q2) * 128 + q3;
                        if (!first) Q += S->qacc[rl];
                        if (!last) {
                            S->qacc[rl] = Q;
                        } else {
                            const double ws = S->ws[pc.stage_off + rl], wz = S->wz[pc.stage_off + rl];
                            ds_store(P, S, E, r0 + rl, rl, (float)((double)xs * (ws * (double)Q + wz * (double)T)), pc);
                        }
                    }
                } else {
                    float ya = ds_dot_f16<KL>(ra, lane, xr), yb = has_b ? ds_dot_f16<KL>(rb, lane, xr) : 0.f;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        ya += __shfl_xor_sync(0xffffffffu, ya, o);
                        yb += __shfl_xor_sync(0xffffffffu, yb, o);
                    }
                    if (lane == 0) {
                        // both rows by lane 0: the arg-max of the head rows is kept in its registers
                        for (int s = 0; s < (has_b ? 2 : 1); ++s) {
                            const int rl = s ? ib : ia;
                            float y = s ? yb : ya;
                            if (!first) y += S->facc[rl];
                            if (!last)
                                S->facc[rl] = y;
                            else
                                ds_store(P, S, E, r0 + rl, rl, y, pc);
                        }
                    }
                }
            }
            ds_chunk_release(S, bar_idx, lane);
        }
    }
    return true;
}

#ifdef RSV_DS_DEBUG
__device__ __forceinline__ long long ds_now() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// time stamps of CTA 0 at phase boundaries of token 1, layer 1
#define DS_STAMP(id)                                                                  \
    do {                                                                              \
        if (P.dbg && cta == 0 && wtid == 0 && t == 1 && l == 1) P.dbg[id] = ds_now(); \
    } while (0)
#else
#define DS_STAMP(id) \
    do {             \
    } while (0)
#endif

// Sum / maximum over the 256 consumer threads through an 8-entry array: one barrier per call.  Calls that follow each other
// must use different arrays (a thread may enter the next call while another still reads this one's array).
__device__ __forceinline__ float ds_block_sum(float v, float* arr, int wwarp, int lane) {
    v = warp_sum(v);
    if (lane == 0) arr[wwarp] = v;
    ds_consumer_sync();
    return ((arr[0] + arr[1]) + (arr[2] + arr[3])) + ((arr[4] + arr[5]) + (arr[6] + arr[7]));
}

// The activation vectors of a phase -> the operand area.  Vector v (LEN elements, NGR groups of four per thread) becomes
// base-128 digits in dp4a order when its matrix is int8 (uint4 (g, c) at index g * (LEN / 16) + c holds the digit words of
// k = 16 c + 4 g .. + 3), plain fp32 otherwise; the scale exponent goes to S->ex[v], the exact fixed-point sum to S->tsw[v].
template <int NV, int NGR>
__device__ __forceinline__ void ds_emit(DsShared* S, float* vec, int len, const bool (&i8)[NV], const float4 (&val)[NV][NGR], int wtid) {
    const int wwarp = wtid >> 5, lane = wtid & 31, len4 = len >> 2;
    float am[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        am[v] = 0.f;
#pragma unroll
        for (int gi = 0; gi < NGR; ++gi)
            if (wtid + kDsConsumers * gi < len4)
                am[v] = fmaxf(am[v], fmaxf(fmaxf(fabsf(val[v][gi].x), fabsf(val[v][gi].y)), fmaxf(fabsf(val[v][gi].z), fabsf(val[v][gi].w))));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) am[v] = fmaxf(am[v], __shfl_xor_sync(0xffffffffu, am[v], o));
        if (lane == 0) S->red_c[v * 8 + wwarp] = am[v];
    }
    ds_consumer_sync();
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) a = fmaxf(a, S->red_c[v * 8 + w]);
        const int ex = ds_exponent(a);
        const float mult = ds_pow2(kDsP - ex);
        if (wtid == 0) S->ex[v] = ex;
        long long ts = 0;
        float* vbase = vec + (size_t)v * len;
#pragma unroll
        for (int gi = 0; gi < NGR; ++gi) {
            const int g4 = wtid + kDsConsumers * gi;
            if (g4 < len4) {
                if (i8[v]) {
                    const uint4 d = ds_digits4(val[v][gi], mult, ts);
                    reinterpret_cast<uint4*>(vbase)[(g4 & 3) * (len >> 4) + (g4 >> 2)] = d;
                } else {
                    reinterpret_cast<float4*>(vbase)[g4] = val[v][gi];
                }
            }
        }
        ts = ds_warp_sum_ll(ts);
        if (lane == 0) S->tsw[v][wwarp] = ts;
    }
    ds_consumer_sync();
}

// LayerNorm statistics (two passes, as the CPU path) of a C-vector spread over the consumer threads (NGR groups of four each)
template <int C, int NGR>
__device__ __forceinline__ void ds_ln_stats(DsShared* S, const float4 (&xv)[NGR], int wtid, float& mean, float& inv) {
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

template <int KL>
__global__ void __launch_bounds__(kDsThreads, 1) decode_stream_kernel(const __grid_constant__ DsParams P) {
    constexpr int C = KL * 32;
    constexpr int NG = (C / 4 + kDsConsumers - 1) / kDsConsumers;  // groups of four channels per consumer thread
    extern __shared__ __align__(1024) uint8_t ds_smem_raw[];
    uint8_t* ring = (uint8_t*)(((uintptr_t)ds_smem_raw + 127) & ~(uintptr_t)127);
    float* vec = reinterpret_cast<float*>(ring + P.ring_bytes);
    DsShared* S = reinterpret_cast<DsShared*>(vec + P.vec_floats);
    float* sc_mid = reinterpret_cast<float*>(S + 1);
    volatile int* abort_flag = (volatile int*)&S->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x, cta = blockIdx.x;
    const int R = P.ring_bytes;
    const int nmid = P.wm + P.am + P.vm + P.gm;
    // bytes of the three chunks that carry a head's rank back-projection rows
    const int hbA = 64 * (P.wm + P.am) * 2, hbC = 32 * P.gm * 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDsBars; ++s) {
            mbar_init(&S->full[s], 1);
            mbar_init(&S->empty[s], kDsConsumerWarps);
        }
        S->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == 0) {
        // =========================== producer ===========================
        const uint64_t pol = ds_evict_first_policy();
        const uint32_t ring_s = smem_u32(ring);
        int head = 0, used = 0;
        uint32_t j = 0, tail = 0;
        bool ok = true;
        // Reserves `bytes` in the ring for chunk j (waiting for the oldest chunks to be released), arms its barrier, and
        // leaves its offset in `head - bytes`.
        auto reserve = [&](int bytes) -> bool {
            const int waste = (head + bytes > R) ? R - head : 0;
            while (used + waste + bytes > R || j - tail >= (uint32_t)kDsBars) {
                const bool w = mbar_wait(&S->empty[tail % kDsBars], (tail / kDsBars) & 1u, abort_flag);
                if (!__all_sync(0xffffffffu, w)) return false;
                used -= S->alloc[tail % kDsBars];
                ++tail;
            }
            if (waste) head = 0;
            __syncwarp();
            if (lane == 0) {
                S->alloc[j % kDsBars] = waste + bytes;
                mbar_expect_tx(&S->full[j % kDsBars], (uint32_t)bytes);
            }
            __syncwarp();
            used += waste + bytes;
            head += bytes;
            return true;
        };
        auto put_entry = [&](const DsEntry& E) -> bool {
            if (E.M <= 0) return true;
            const int vc = (cta + E.rot) % G;
            const int r0 = ds_row_begin(vc, E.M, G), n = ds_row_begin(vc + 1, E.M, G) - r0;
            if (n <= 0) return true;
            const int rpc = ds_rows_per_chunk(E.row_bytes);
            for (int p = 0; p < E.npieces; ++p)
                for (int c0 = 0; c0 < n; c0 += rpc) {
                    const int nr = min(rpc, n - c0), bytes = nr * E.row_bytes;
                    if (!reserve(bytes)) return false;
                    if (lane < nr)
                        ds_bulk_load(ring_s + (uint32_t)(head - bytes + lane * E.row_bytes),
                                     E.base + (size_t)(r0 + c0 + lane) * (size_t)E.row_stride + (size_t)p * E.row_bytes, (uint32_t)E.row_bytes,
                                     &S->full[j % kDsBars], pol);
                    ++j;
                }
            return true;
        };
        for (int t = 0; t < P.n_tokens && ok; ++t) {
            const bool do_head = P.argmax_feed || t == P.n_tokens - 1;
            for (int l = 0; l < P.L && ok; ++l) {
                const DsLayer* Lg = P.layers + l;
                for (int e = DSE_W1; e <= DSE_WV && ok; ++e) ok = put_entry(Lg->e[e]);
                if (!ok) break;
                const int h = ds_head_of_cta(cta, l, P.H, G);
                if (h >= 0) {
                    // chunk A: w2, a2 rows of the head; chunk B: v2 rows (layers > 0) and the first 32 g2 rows; chunk C: the other 32
                    const int vb = l > 0 ? 64 * P.vm * 2 : 0;
                    if (!(ok = reserve(hbA))) break;
                    if (lane == 0) ds_bulk_load(ring_s + (uint32_t)(head - hbA), Lg->w2 + (size_t)h * 64 * P.wm, 64u * P.wm * 2u, &S->full[j % kDsBars], pol);
                    if (lane == 1)
                        ds_bulk_load(ring_s + (uint32_t)(head - hbA + 64 * P.wm * 2), Lg->a2 + (size_t)h * 64 * P.am, 64u * P.am * 2u, &S->full[j % kDsBars], pol);
                    ++j;
                    if (!(ok = reserve(vb + hbC))) break;
                    if (lane == 0 && vb) ds_bulk_load(ring_s + (uint32_t)(head - vb - hbC), Lg->v2 + (size_t)h * 64 * P.vm, (uint32_t)vb, &S->full[j % kDsBars], pol);
                    if (lane == 1) ds_bulk_load(ring_s + (uint32_t)(head - hbC), Lg->g2 + (size_t)h * 64 * P.gm, (uint32_t)hbC, &S->full[j % kDsBars], pol);
                    ++j;
                    if (!(ok = reserve(hbC))) break;
                    if (lane == 0) ds_bulk_load(ring_s + (uint32_t)(head - hbC), Lg->g2 + ((size_t)h * 64 + 32) * P.gm, (uint32_t)hbC, &S->full[j % kDsBars], pol);
                    ++j;
                }
                for (int e = DSE_WO; e <= DSE_WFV && ok; ++e) ok = put_entry(Lg->e[e]);
            }
            if (ok && do_head) ok = put_entry(P.head);
        }
        // copies still in flight must land before the CTA may exit (only after an abort: otherwise every chunk was consumed)
        if (!ok)
            for (; tail < j; ++tail) ds_mbar_drain(&S->full[tail % kDsBars], (tail / kDsBars) & 1u);
    } else {
        // =========================== consumers ===========================
        const int wtid = threadIdx.x - 32, wwarp = wtid >> 5;
        DsCons cs{smem_u32(ring), R, 0, 0, 0u};
        DsPhaseCtx pc{smem_u32(vec), 0, -1e30f, 0x7fffffff};
        unsigned bar_target = 0;
        bool ok = true, pending = false;
        const int r0o = ds_row_begin(cta, C, G), nown = ds_row_begin(cta + 1, C, G) - r0o;  // this CTA's slice of the channels
        uint32_t lt = 0;  // layers run so far: the table of the current layer sits in S->layer[lt & 1]

        auto stage_layer = [&](int l, uint32_t slot) {
            static_assert(sizeof(DsLayer) % 4 == 0, "DsLayer is copied word by word");
            const uint32_t* src = reinterpret_cast<const uint32_t*>(P.layers + l);
            uint32_t* dst = reinterpret_cast<uint32_t*>(&S->layer[slot & 1]);
            for (int i = wtid; i < (int)(sizeof(DsLayer) / 4); i += kDsConsumers) dst[i] = __ldg(src + i);
        };
        // Grid barrier in two halves: arrive as soon as this CTA's outputs are stored, wait just before the first load of
        // another CTA's outputs; what lies between (parameter loads of the next phase) overlaps the other CTAs' tails.
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
                if (!got) *abort_flag = 1;
            }
            ds_consumer_sync();
            return *abort_flag == 0;
        };
        auto bar_arrive = [&]() {
            bar_wait();
            ds_consumer_sync();
            if (wtid == 0) {
                fence_acq_rel_gpu();
                atomicAdd(P.grid_bar, 1u);
            }
            bar_target += (unsigned)G;
            pending = true;
        };
        auto rows_of = [&](const DsEntry& E, int& r0, int& n) {
            r0 = n = 0;
            if (E.M <= 0) return;
            const int vc = (cta + E.rot) % G;
            r0 = ds_row_begin(vc, E.M, G);
            n = ds_row_begin(vc + 1, E.M, G) - r0;
        };
        // (scale, zero) of the int8 rows this CTA owns in the coming phase -> shared memory (weights: no dependency on a barrier)
        auto stage_scales = [&](const DsEntry* ents, int cnt) {
            int off = 0;
            for (int i = 0; i < cnt; ++i) {
                const DsEntry& E = ents[i];
                int r0, n;
                rows_of(E, r0, n);
                if (!E.is_i8 || n <= 0) continue;
                for (int q = wtid; q < n && off + q < kDsMaxRows; q += kDsConsumers) {
                    S->ws[off + q] = __ldg(E.wscale + r0 + q);
                    S->wz[off + q] = __ldg(E.wzero + r0 + q);
                }
                off += n;
            }
        };
        auto run_entries = [&](const DsEntry* ents, int cnt) -> bool {
            int off = 0;
            for (int i = 0; i < cnt; ++i) {
                const DsEntry& E = ents[i];
                int r0, n;
                rows_of(E, r0, n);
                if (n <= 0) continue;
                pc.stage_off = off;
                if (!ds_run_entry<KL>(P, S, cs, E, r0, n, pc, wwarp, lane)) return false;
                if (E.is_i8) off += n;
            }
            return true;
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
                // ================= phase 1: LN1 + token shift -> r, k, v, rank projections =================
                {
                    float4 lw[NG], lb[NG], pv[NG], mr[NG], mk[NG], mv[NG], xv[NG];
#pragma unroll
                    for (int gi = 0; gi < NG; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                        lw[gi] = ds_ldg4(Ly.ln1_w + k);
                        lb[gi] = ds_ldg4(Ly.ln1_b + k);
                        mr[gi] = ds_ldg4(Ly.x_r + k);
                        mk[gi] = ds_ldg4(Ly.x_k + k);
                        mv[gi] = ds_ldg4(Ly.x_v + k);
                        pv[gi] = ds_ldcg4(tm_l + k);
                    }
                    stage_scales(&Ly.e[DSE_W1], 7);
                    if (!(ok = bar_wait())) break;
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
                        ds_ln_stats<C, NG>(S, xv, wtid, m0, i0);
#pragma unroll
                        for (int gi = 0; gi < NG; ++gi) xv[gi] = ds_ln_apply(xv[gi], m0, i0, w0v[gi], b0v[gi]);
                    } else {
#pragma unroll
                        for (int gi = 0; gi < NG; ++gi) {
                            const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                            xv[gi] = ds_ldcg4(P.x + k);
                        }
                    }
                    float mean, inv;
                    ds_ln_stats<C, NG>(S, xv, wtid, mean, inv);
                    float4 val[3][NG];
#pragma unroll
                    for (int gi = 0; gi < NG; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi;
                        const float4 cur = ds_ln_apply(xv[gi], mean, inv, lw[gi], lb[gi]);
                        const float4 del = make_float4(pv[gi].x - cur.x, pv[gi].y - cur.y, pv[gi].z - cur.z, pv[gi].w - cur.w);
                        val[0][gi] = ds_mix4(cur, mr[gi], del);
                        val[1][gi] = ds_mix4(cur, mk[gi], del);
                        val[2][gi] = ds_mix4(cur, mv[gi], del);
                        if (g4 < C / 4) {
                            reinterpret_cast<float4*>(vec + 3 * C)[g4] = cur;  // LN1(x): the new shift state and the rank projections' input
                            reinterpret_cast<float4*>(vec + 4 * C)[g4] = del;
                            const float xe[4] = {xv[gi].x, xv[gi].y, xv[gi].z, xv[gi].w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int o = 4 * g4 + e - r0o;
                                if (o >= 0 && o < nown) S->xs_own[o] = xe[e];
                            }
                        }
                    }
                    const bool i8[3] = {Ly.e[DSE_WR].is_i8 != 0, Ly.e[DSE_WK].is_i8 != 0, Ly.e[DSE_WV].is_i8 != 0};
                    ds_emit<3, NG>(S, vec, C, i8, val, wtid);
                }
                DS_STAMP(1);
                if (!(ok = run_entries(&Ly.e[DSE_W1], 7))) break;
                DS_STAMP(2);
                bar_arrive();

                // ================= phase 2: one CTA per head =================
                {
                    const int h = ds_head_of_cta(cta, l, P.H, G);
                    if (h >= 0) {
                        const int rrow = wtid >> 2, quad = wtid & 3, ch = h * 64 + rrow;  // 4 threads per channel / state row
                        float* srow = wkv_l + ((size_t)h * 64 + rrow) * 64 + quad * 16;
                        float4 s4[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) s4[q] = ds_ldcg4(srow + 4 * q);
                        const float p_w0 = __ldg(Ly.w0 + ch), p_a0 = __ldg(Ly.a0 + ch), p_kk = __ldg(Ly.k_k + ch), p_ka = __ldg(Ly.k_a + ch), p_rk = __ldg(Ly.r_k + ch);
                        const float p_gw = __ldg(Ly.lnx_w + ch), p_gb = __ldg(Ly.lnx_b + ch);
                        const float p_v0 = l > 0 ? __ldg(Ly.v0 + ch) : 0.f;
                        if (!(ok = bar_wait())) break;
                        const float p_vf = l > 0 ? __ldcg(P.vfirst + ch) : 0.f;
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
                        // back-projections: the four threads of a channel split the rank dimension in contiguous quarters
                        auto dot_q = [&](const __half* W, int mid, const float* v) {
                            float a = 0.f;
                            const int ql = mid >> 2;
                            if ((mid & 3) == 0 && (ql & 7) == 0) {
                                const __half* wrow = W + quad * ql;
                                const float* vv = v + quad * ql;
                                for (int q = 0; q < ql; q += 8) {
                                    const uint4 pk = *reinterpret_cast<const uint4*>(wrow + q);
                                    const __half2* h2 = reinterpret_cast<const __half2*>(&pk);
#pragma unroll
                                    for (int e = 0; e < 4; ++e) {
                                        const float2 f = __half22float2(h2[e]);
                                        a = fmaf(f.x, vv[q + 2 * e], a);
                                        a = fmaf(f.y, vv[q + 2 * e + 1], a);
                                    }
                                }
                            } else {
                                for (int q = quad; q < mid; q += 4) a = fmaf(__half2float(W[q]), v[q], a);
                            }
                            a += __shfl_xor_sync(0xffffffffu, a, 1);
                            return a + __shfl_xor_sync(0xffffffffu, a, 2);
                        };
                        const int vb = l > 0 ? 64 * P.vm * 2 : 0;
                        const int bA = ds_chunk_wait(cs, S, hbA);
                        if (bA < 0) {
                            ok = false;
                            break;
                        }
                        const __half* w2s = reinterpret_cast<const __half*>(ring + cs.cur);
                        const float dw = dot_q(w2s + (size_t)rrow * P.wm, P.wm, sc_mid);
                        const float da = dot_q(w2s + (size_t)64 * P.wm + (size_t)rrow * P.am, P.am, sc_mid + P.wm);
                        ds_chunk_release(S, bA, lane);
                        const int bB = ds_chunk_wait(cs, S, vb + hbC);
                        const uint8_t* cB = ring + cs.cur;
                        const int bC = bB < 0 ? -1 : ds_chunk_wait(cs, S, hbC);
                        const uint8_t* cC = ring + cs.cur;
                        if (bB < 0 || bC < 0) {
                            ok = false;
                            break;
                        }
                        const __half* g2row = rrow < 32 ? reinterpret_cast<const __half*>(cB + vb) + (size_t)rrow * P.gm : reinterpret_cast<const __half*>(cC) + (size_t)(rrow - 32) * P.gm;
                        const float dg = dot_q(g2row, P.gm, sc_mid + P.wm + P.am + P.vm);
                        const float dv = l > 0 ? dot_q(reinterpret_cast<const __half*>(cB) + (size_t)rrow * P.vm, P.vm, sc_mid + P.wm + P.am) : 0.f;
                        ds_chunk_release(S, bB, lane);
                        ds_chunk_release(S, bC, lane);
                        const float wdec = expf((1.0f / (1.0f + expf(-(dw + p_w0)))) * kDecayScale);
                        const float aa = 1.0f / (1.0f + expf(-(da + p_a0)));
                        const float rr = S->hv[rrow], kk0 = S->hv[64 + rrow];
                        float vv0 = S->hv[128 + rrow];
                        if (l == 0) {
                            if (quad == 0) {
                                P.vfirst[ch] = vv0;
                                P.state_vfirst[(size_t)P.slot * C + ch] = vv0;
                            }
                        } else {
                            const float gate = 1.0f / (1.0f + expf(-(dv + p_v0)));
                            vv0 = vv0 + gate * (p_vf - vv0);
                        }
                        const float kkj = kk0 * p_kk;
                        const float kt = kk0 + p_ka * (kk0 * aa - kk0);
                        // ||kk||^2 and the bonus sum over the head's 64 channels in one round
                        float ss = warp_sum(quad == 0 ? kkj * kkj : 0.f), srk = warp_sum(quad == 0 ? rr * kt * p_rk : 0.f);
                        if (lane == 0) {
                            S->red_a[wwarp] = ss;
                            S->red_b[wwarp] = srk;
                        }
                        ds_consumer_sync();
                        ss = ((S->red_a[0] + S->red_a[1]) + (S->red_a[2] + S->red_a[3])) + ((S->red_a[4] + S->red_a[5]) + (S->red_a[6] + S->red_a[7]));
                        srk = ((S->red_b[0] + S->red_b[1]) + (S->red_b[2] + S->red_b[3])) + ((S->red_b[4] + S->red_b[5]) + (S->red_b[6] + S->red_b[7]));
                        const float kkh = kkj * (1.0f / fmaxf(sqrtf(ss), kL2Eps));
                        if (quad == 0) {
                            S->hv[3 * 64 + rrow] = wdec;
                            S->hv[4 * 64 + rrow] = rr;
                            S->hv[5 * 64 + rrow] = kkh;
                            S->hv[6 * 64 + rrow] = kkh * (-aa);
                            S->hv[7 * 64 + rrow] = kt;
                        }
                        ds_consumer_sync();
                        float St[16];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            St[4 * q] = s4[q].x;
                            St[4 * q + 1] = s4[q].y;
                            St[4 * q + 2] = s4[q].z;
                            St[4 * q + 3] = s4[q].w;
                        }
                        const float *s_w = S->hv + 3 * 64 + quad * 16, *s_r = S->hv + 4 * 64 + quad * 16, *s_kk = S->hv + 5 * 64 + quad * 16,
                                    *s_b = S->hv + 6 * 64 + quad * 16, *s_kt = S->hv + 7 * 64 + quad * 16;
                        float sa = 0.f;
#pragma unroll
                        for (int q = 0; q < 16; ++q) sa = fmaf(St[q], s_kk[q], sa);
                        sa += __shfl_xor_sync(0xffffffffu, sa, 1);
                        sa += __shfl_xor_sync(0xffffffffu, sa, 2);
                        float y = 0.f;
#pragma unroll
                        for (int q = 0; q < 16; ++q) {
                            St[q] = fmaf(St[q], s_w[q], fmaf(sa, s_b[q], vv0 * s_kt[q]));
                            y = fmaf(St[q], s_r[q], y);
                        }
                        y += __shfl_xor_sync(0xffffffffu, y, 1);
                        y += __shfl_xor_sync(0xffffffffu, y, 2);
#pragma unroll
                        for (int q = 0; q < 4; ++q) *reinterpret_cast<float4*>(srow + 4 * q) = make_float4(St[4 * q], St[4 * q + 1], St[4 * q + 2], St[4 * q + 3]);
                        const float gmean = ds_block_sum(quad == 0 ? y : 0.f, S->red_c, wwarp, lane) / 64.0f;
                        const float d = y - gmean;
                        const float var = ds_block_sum(quad == 0 ? d * d : 0.f, S->red_c + 8, wwarp, lane) / 64.0f + kGnEps;
                        if (quad == 0) P.yg[ch] = (d * (1.0f / sqrtf(var)) * p_gw + p_gb + srk * vv0) * dg;
                    }
                }
                DS_STAMP(3);
                bar_arrive();

                // ================= phase 3: att.output, x += =================
                {
                    stage_scales(&Ly.e[DSE_WO], 1);
                    if (!(ok = bar_wait())) break;
                    if (wtid < nown) tm_l[r0o + wtid] = vec[3 * C + r0o + wtid];  // new time-mix shift state (every reader of the old one is past barrier 1)
                    float4 yv[1][NG];
#pragma unroll
                    for (int gi = 0; gi < NG; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                        yv[0][gi] = ds_ldcg4(P.yg + k);
                    }
                    const bool i8[1] = {Ly.e[DSE_WO].is_i8 != 0};
                    ds_emit<1, NG>(S, vec, C, i8, yv, wtid);
                    DS_STAMP(4);
                    if (!(ok = run_entries(&Ly.e[DSE_WO], 1))) break;
                }
                DS_STAMP(5);
                bar_arrive();

                // ================= phase 4: LN2 + shift -> relu(ffn.key)^2 =================
                {
                    float4 lw[NG], lb[NG], pv[NG], mx[NG], xv[NG];
#pragma unroll
                    for (int gi = 0; gi < NG; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                        lw[gi] = ds_ldg4(Ly.ln2_w + k);
                        lb[gi] = ds_ldg4(Ly.ln2_b + k);
                        mx[gi] = ds_ldg4(Ly.ffn_x_k + k);
                        pv[gi] = ds_ldcg4(cm_l + k);
                    }
                    stage_scales(&Ly.e[DSE_WFK], 1);
                    const int lnext = l + 1 < P.L ? l + 1 : 0;
                    stage_layer(lnext, lt + 1);  // the table of the layer that runs next (the first one again after the last)
                    if (!(ok = bar_wait())) break;
#pragma unroll
                    for (int gi = 0; gi < NG; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                        xv[gi] = ds_ldcg4(P.x + k);
                    }
                    float mean, inv;
                    ds_ln_stats<C, NG>(S, xv, wtid, mean, inv);
                    float4 val[1][NG];
#pragma unroll
                    for (int gi = 0; gi < NG; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi;
                        const float4 cur = ds_ln_apply(xv[gi], mean, inv, lw[gi], lb[gi]);
                        const float4 del = make_float4(pv[gi].x - cur.x, pv[gi].y - cur.y, pv[gi].z - cur.z, pv[gi].w - cur.w);
                        val[0][gi] = ds_mix4(cur, mx[gi], del);
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
                    ds_emit<1, NG>(S, vec, C, i8, val, wtid);
                    DS_STAMP(6);
                    if (!(ok = run_entries(&Ly.e[DSE_WFK], 1))) break;
                }
                DS_STAMP(7);
                bar_arrive();

                // ================= phase 5: ffn.value (K = F = 4 C), x += =================
                {
                    constexpr int NG5 = (C + kDsConsumers - 1) / kDsConsumers;  // groups of four of the F = 4 C hidden values per thread
                    stage_scales(&Ly.e[DSE_WFV], 1);
                    if (!(ok = bar_wait())) break;
                    if (wtid < nown) cm_l[r0o + wtid] = S->cs_own[wtid];
                    float4 hv4[1][NG5];
#pragma unroll
                    for (int gi = 0; gi < NG5; ++gi) {
                        const int g4 = wtid + kDsConsumers * gi, k = g4 < C ? 4 * g4 : 0;
                        hv4[0][gi] = ds_ldcg4(P.hbuf + k);
                    }
                    const bool i8[1] = {Ly.e[DSE_WFV].is_i8 != 0};
                    ds_emit<1, NG5>(S, vec, 4 * C, i8, hv4, wtid);
                    DS_STAMP(8);
                    if (!(ok = run_entries(&Ly.e[DSE_WFV], 1))) break;
                }
                DS_STAMP(9);
                bar_arrive();
            }
            if (!ok) break;

            // ================= ln_out + head -> logits, arg-max =================
            if (do_head) {
                float4 lw[NG], lb[NG], xv[NG];
#pragma unroll
                for (int gi = 0; gi < NG; ++gi) {
                    const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                    lw[gi] = ds_ldg4(P.lno_w + k);
                    lb[gi] = ds_ldg4(P.lno_b + k);
                }
                stage_scales(&P.head, 1);
                if (!(ok = bar_wait())) break;
#pragma unroll
                for (int gi = 0; gi < NG; ++gi) {
                    const int g4 = wtid + kDsConsumers * gi, k = g4 < C / 4 ? 4 * g4 : 0;
                    xv[gi] = ds_ldcg4(P.x + k);
                }
                float mean, inv;
                ds_ln_stats<C, NG>(S, xv, wtid, mean, inv);
                float4 val[1][NG];
#pragma unroll
                for (int gi = 0; gi < NG; ++gi) val[0][gi] = ds_ln_apply(xv[gi], mean, inv, lw[gi], lb[gi]);
                const bool i8[1] = {P.head.is_i8 != 0};
                ds_emit<1, NG>(S, vec, C, i8, val, wtid);
                pc.best_val = -1e30f;
                pc.best_idx = 0x7fffffff;
                if (!(ok = run_entries(&P.head, 1))) break;
                if (P.argmax_feed) {
                    // arg-max: lanes -> warp -> CTA -> grid; ties go to the smaller index
                    float bv = pc.best_val;
                    int bi = pc.best_idx;
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
    if (threadIdx.x == 0 && *abort_flag) atomicOr(P.status, 4);
}

}  // namespace rsv
