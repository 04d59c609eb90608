// Persistent decode kernel: one cooperative launch runs n tokens x L layers x (head, arg-max) for up to 4
// sessions, so a whole self-loop is a single kernel.  It stands in for the reference's captured-graph decode
// step (forward_token / forward_layer / selfloop_step, src/gpu_model.rs:1879-2392) whose 8 kernels per layer
// are latency-bound at batch 1.
//
// Structure.  One CTA per SM, 320 threads:
//   warp 0   TMA producer.  Walks the fixed sequence of weight tiles (16 KB = 128 rows x 128 bytes) this CTA will
//            ever need — token after token, layer after layer, phase after phase — and keeps a shared-memory ring
//            full.  It never waits on a grid barrier, only on free ring slots, so HBM keeps streaming while the
//            other warps synchronise: the barriers cost latency, not bandwidth.
//   warp 1   MMA issuer.  tcgen05.mma (kind::i8 on the u8 codes / kind::f16) of each weight tile against the
//            activation operand tiles the workers left in shared memory; accumulators in TMEM (N = 16 columns:
//            4 sessions x 4 base-128 digits, or 4 x (hi, lo) halves).
//   warps 2-9  workers.  Per phase: build the activation operand tiles (LayerNorm, token shift, fixed-point
//            digits), drain finished accumulators to global partial sums, do the per-head WKV-7 work, take part
//            in the grid barriers.
// Work split: every GEMV phase is cut into units (128-row tile x 128-byte K block); CTA c owns the contiguous
// unit range [c*U/G, (c+1)*U/G), so each SM streams the same number of weight bytes.  The unit lists of the six
// phase shapes are tabulated in shared memory once per launch.  A run (the units of one tile inside one CTA)
// leaves an exact int32 (or fp32) partial [16 columns][128 rows] plus its own fixed-point scale.  Every worker
// warp owns a fixed (32-row, 8-column) sub-block of a tile and counts its arrival on it with one atomic; the warp
// that arrives last adds the sub-block's partials in slot order, applies the phase's epilogue and stores plain
// fp32 outputs, so consumers never see partial sums.  Integer partials make the split exact, and every
// floating-point sum has a fixed order: results are deterministic and independent of timing.
// Phases per layer (one grid barrier after each):
//   1  LN1 + token shift -> r,k,v (int8) and the four rank projections (fp16; tanh / sigmoid applied)
//   2  per (session, head): rank back-projections, decay/a/v/g, WKV-7 state update in place, GroupNorm, gate
//   3  att.output, x += ...        4  LN2 + shift -> relu(ffn.key)^2        5  ffn.value, x += ...
// then ln_out + head (fp16) -> logits, arg-max across CTAs, next token.
// All spin-waits are bounded; on expiry bit 2 of the status word is set and every role drains and exits.
#pragma once
#include "tc_linear.cuh"

namespace rsv {

constexpr int kDpThreads = 320;
constexpr int kDpWorkers = 256;
constexpr int kDpWarps = kDpWorkers / 32;
constexpr int kDpMaxNB = 4;
constexpr int kDpN = 16;
constexpr int kDpATile = 128 * 128;
constexpr int kDpBTile = kDpN * 128;
constexpr int kDpDigits = 4;
constexpr int kDpP = 7 * kDpDigits - 1;
constexpr uint32_t kDpBarSpin = 1u << 22;
constexpr int kDpMaxRuns = 8;    // runs (tiles touched) per CTA and phase
constexpr int kDpMaxShares = 4;  // problems touched per CTA and phase
constexpr int kDpMaxSlice = 64;  // channels of the residual stream per CTA (ceil(C / grid))

struct DpMat {
    int map, M, mtiles, kblocks, is_i8, K;
    const float* wscale;
    const float* wzero;
};
enum { DM_WR = 0, DM_WK, DM_WV, DM_WO, DM_WFK, DM_WFV, DM_W1, DM_A1, DM_V1, DM_G1, DM_HEAD };
struct DpLayer {
    DpMat mat[10];                    // indexed by DM_*
    const __half *w2, *a2, *v2, *g2;  // [C, mid] fp16
    const float *ln1_w, *ln1_b, *ln2_w, *ln2_b, *lnx_w, *lnx_b;
    const float *x_r, *x_w, *x_k, *x_v, *x_a, *x_g, *ffn_x_k;
    const float *w0, *a0, *v0, *r_k, *k_k, *k_a;
    float *tmix_x, *wkv, *cmix_x;
};
struct DpRunMeta {
    float xscale[kDpMaxNB];
    long long tsum[kDpMaxNB];
};
struct DpRegion {
    uint32_t* data;   // [tile][pmax][16][128]
    DpRunMeta* meta;  // [tile][pmax][worker warp]: every warp leaves its own copy, ordered with its own arrival
    int* cnt;         // [tile][worker warp] arrivals on a sub-block; zero between phases
    int pmax;
    int pad;
};
// phase variants: the schedule shapes that occur in a launch
enum { DV_P1A = 0 /*layer 0: no v1*/, DV_P1B, DV_P3, DV_P4, DV_P5, DV_HEAD, DV_COUNT };
enum { DR_P1 = 0, DR_P3, DR_P4, DR_P5, DR_HEAD };  // partial-sum regions
struct DpParams {
    const CUtensorMap* maps;  // [10*L + 1]: layer l, matrix DM_x -> 10*l + x; head -> 10*L
    const DpLayer* layers;
    DpMat head;
    const __half* emb;
    const float *ln0_w, *ln0_b, *lno_w, *lno_b;
    int L, C, H, F, V, wm, am, vm, gm;
    int nb;
    int slot[kDpMaxNB];
    float *x, *yg, *vfirst;  // [4][C]
    float* rkv;              // [4][3][C] r, k, v of the current layer
    float* mid;              // [4][wm+am+vm+gm] rank-space vectors (tanh / sigmoid applied)
    float* hbuf;             // [4][F] relu(ffn.key)^2
    float* state_vfirst;     // [cap][C]
    DpRegion reg[5];
    uint32_t* tokens;          // [4] current input token of every session (read at start, written after arg-max)
    const uint32_t* tok_list;  // [n_tokens][nb], used when tok_from_list
    uint32_t* seq;
    int* seq_cnt;
    int seq_cap;
    float* logits;  // [4][V]
    float* cand_val;
    int* cand_idx;  // [G][4]
    unsigned* grid_bar;
    int* status;
    int n_tokens;
    int tok_from_list;  // 1: step t reads tok_list[t*nb + b]; 0: step 0 reads tokens[b]
    int argmax_feed;    // 1: head + arg-max every step, the result is the next step's input (self-loop); 0: head on the last step only
    int nstages, btiles, max_units;  // max_units: capacity of the per-CTA unit table (all variants together)
    long long* dbg;                  // optional [64] time stamps (ns) of CTA 0 at phase boundaries of token 1, layer 1
};

// ---- per-CTA schedule tables (shared memory) ----
struct DpUnit {
    uint16_t kb, mt;
    uint8_t prob, btile, flags, pad;  // flags: 1 = first unit of its run, 2 = last unit of its run, 4 = int8 problem
};
struct DpRun {
    uint16_t tile;  // tile index inside the region
    uint16_t u0;    // first unit (index into the variant's unit list)
    uint8_t nu, slot, prob, ns;  // ns: number of CTAs (partial slots) that share the tile
};
struct DpShare {  // the K blocks of one problem this CTA feeds: operand tiles base .. base+ntile-1
    uint8_t prob, ntile, kb0, base;
};
struct DpVar {
    int nprob, U, ge, region;
    int nunits, nruns, nshares, unit0;  // unit0: offset of this variant's units in the unit table
    int p_mat[7], p_mtiles[7], p_kblocks[7], p_i8[7], p_unit0[7], p_tile0[7], p_K[7];
    DpRun run[kDpMaxRuns];
    DpShare share[kDpMaxShares];
};

// Phase time stamps (token 1, layer 1) for tuning: compiled in only with -DRSV_DP_DEBUG, together with the host code that
// allocates and prints them; otherwise the macros expand to nothing.
#ifdef RSV_DP_DEBUG
__device__ __forceinline__ long long dp_now() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define DP_STAMP_ALL(k)                                                                                 \
    do {                                                                                                \
        if (P.dbg && wtid == 0 && t == 1 && l == 1 && v == DV_P3) P.dbg[64 + cta * 8 + (k)] = dp_now(); \
    } while (0)
#define DP_STAMP(id)                                                                  \
    do {                                                                              \
        if (P.dbg && cta == 0 && wtid == 0 && t == 1 && l == 1) P.dbg[id] = dp_now(); \
    } while (0)
#define DP_DBG(...) __VA_ARGS__
#else
#define DP_STAMP_ALL(k) \
    do {                \
    } while (0)
#define DP_STAMP(id) \
    do {             \
    } while (0)
#define DP_DBG(...)
#endif

// Number of CTAs that take part in a phase of `n` problems with `unit0[i]` = first unit of problem i and U units in all.
// Normally min(G, U).  A CTA whose range straddles two problems has to build two sets of activation operands one after the
// other and everybody waits for it at the barrier; so when a slightly smaller count (>= 85 % of G) gives every CTA the same
// number of units q with every problem boundary on a multiple of q, that count is used: no CTA straddles.
__host__ __device__ inline int dp_choose_ge(const int* unit0, int n, int U, int G) {
    const int ge = G < U ? G : U;
    if (n <= 1 || U <= G) return ge;
    for (int q = (U + G - 1) / G; (U / q) * 100 >= G * 85; ++q) {
        if (U % q) continue;
        bool aligned = true;
        for (int i = 1; i < n; ++i) aligned = aligned && (unit0[i] % q == 0);
        if (aligned) return U / q;
    }
    return ge;
}
__device__ __forceinline__ int dp_cta_begin(int c, int U, int ge) { return (int)(((unsigned)c * (unsigned)U) / (unsigned)ge); }
__device__ __forceinline__ int dp_cta_of(int u, int U, int ge) { return (int)((((unsigned)u + 1u) * (unsigned)ge - 1u) / (unsigned)U); }

// 2^n as a float for -126 <= n <= 127 (exponent field only)
__device__ __forceinline__ float dp_pow2(int n) { return __int_as_float((n + 127) << 23); }
// smallest e with 2^e >= a for a normal positive float a (exponent field, +1 unless a is a power of two)
__device__ __forceinline__ int dp_ceil_log2(float a) {
    const int bits = __float_as_int(a);
    return ((bits >> 23) & 0xFF) - 127 + ((bits & 0x7FFFFF) ? 1 : 0);
}

// The CTAs of the grid share the work of pulling a small array into L2 ahead of its use (one 128-byte line per request).
__device__ __forceinline__ void dp_prefetch_l2(const void* base, size_t bytes, int cta, int G, int tid, int nthreads) {
    if (!base) return;
    const size_t lines = (bytes + 127) / 128;
    for (size_t i = (size_t)cta + (size_t)G * tid; i < lines; i += (size_t)G * nthreads)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(base) + i * 128));
}
__device__ __forceinline__ void dp_prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

__device__ __forceinline__ void dp_worker_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kDpWorkers) : "memory"); }

// Sum over the 256 worker threads; every worker gets the result.  `red` holds 8 floats.
__device__ __forceinline__ float dp_worker_sum(float v, float* red, int wtid) {
    v = warp_sum(v);
    dp_worker_sync();
    if ((wtid & 31) == 0) red[wtid >> 5] = v;
    dp_worker_sync();
    return ((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]));
}

// Grid-wide barrier among the workers of all CTAs (bounded spin).  Returns false after a timeout / abort.
__device__ __forceinline__ bool dp_grid_barrier(unsigned* bar, unsigned& target, int G, volatile int* abort_flag, int wtid) {
    dp_worker_sync();
    if (wtid == 0) {
        fence_acq_rel_gpu();
        atomicAdd(bar, 1u);
        const unsigned want = target + (unsigned)G;
        bool ok = false;
        for (uint32_t i = 0; i < kDpBarSpin; ++i) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar) : "memory");
            if (v >= want) {
                ok = true;
                break;
            }
            if ((i & 255u) == 255u && *abort_flag) break;
        }
        if (!ok) *abort_flag = 1;
    }
    target += (unsigned)G;
    dp_worker_sync();
    return *abort_flag == 0;
}

// Swizzled byte address of (column n, byte kbyte) inside a 16 x 128-byte K-major operand tile (128-byte swizzle:
// the 16-byte chunk index is XORed with the row index modulo 8; 8-row groups are 1024 bytes apart).
__device__ __forceinline__ int dp_b_offset(int n, int kbyte) { return (n >> 3) * 1024 + (n & 7) * 128 + ((((kbyte >> 4) ^ (n & 7)) & 7) << 4) + (kbyte & 15); }

struct DpStats {
    float mean, inv;
};

// Epilogue of one finished output (row m of problem `pi`, session b) of phase variant v.
__device__ __forceinline__ void dp_store_output(const DpParams& P, int v, int mat_id, int m, int b, float val) {
    switch (v) {
        case DV_P1A:
        case DV_P1B: {
            const int nmid = P.wm + P.am + P.vm + P.gm;
            if (mat_id <= DM_WV) {
                P.rkv[((size_t)b * 3 + mat_id) * P.C + m] = val;
            } else if (mat_id == DM_W1) {
                P.mid[(size_t)b * nmid + m] = tanhf(val);
            } else if (mat_id == DM_A1) {
                P.mid[(size_t)b * nmid + P.wm + m] = val;
            } else if (mat_id == DM_V1) {
                P.mid[(size_t)b * nmid + P.wm + P.am + m] = val;
            } else {
                P.mid[(size_t)b * nmid + P.wm + P.am + P.vm + m] = 1.0f / (1.0f + expf(-val));
            }
            break;
        }
        case DV_P4: {
            const float a = fmaxf(val, 0.f);
            P.hbuf[(size_t)b * P.F + m] = a * a;
            break;
        }
        default: P.logits[(size_t)b * P.V + m] = val; break;
    }
}

// Sum of one output row's int8-path partials over the tile's slots, in slot order.  The loads of BATCH slots are in flight
// together.  TWO: the column half holds two sessions.
template <bool TWO, int BATCH>
__device__ __forceinline__ void dp_sum_slots_i8(const uint32_t* d0, const DpRunMeta* mp, int ns, int b0, double ws, double wz, double& acc0, double& acc1) {
    for (int s0 = 0; s0 < ns; s0 += BATCH) {
        int i[BATCH][TWO ? 8 : 4];
        float xs[BATCH][TWO ? 2 : 1];
        long long ts[BATCH][TWO ? 2 : 1];
        // slot indices past the last one are clamped: every load is unconditional, so all of them are in flight together
#pragma unroll
        for (int k = 0; k < BATCH; ++k) {
            const int sk = min(s0 + k, ns - 1);
            const uint32_t* d = d0 + (size_t)sk * (kDpN * 128);
            const DpRunMeta* ms = mp + (size_t)sk * kDpWarps;
#pragma unroll
            for (int j = 0; j < (TWO ? 8 : 4); ++j) i[k][j] = (int)__ldcg(d + j * 128);
#pragma unroll
            for (int e = 0; e < (TWO ? 2 : 1); ++e) {
                xs[k][e] = __ldcg(&ms->xscale[b0 + e]);
                ts[k][e] = __ldcg(&ms->tsum[b0 + e]);
            }
        }
#pragma unroll
        for (int k = 0; k < BATCH; ++k) {
            if (s0 + k < ns) {
                const long long Q0 = (((long long)i[k][0] * 128 + i[k][1]) * 128 + i[k][2]) * 128 + i[k][3];
                acc0 += (double)xs[k][0] * (ws * (double)Q0 + wz * (double)ts[k][0]);
                if (TWO) {
                    const long long Q1 = (((long long)i[k][TWO ? 4 : 0] * 128 + i[k][TWO ? 5 : 1]) * 128 + i[k][TWO ? 6 : 2]) * 128 + i[k][TWO ? 7 : 3];
                    acc1 += (double)xs[k][TWO ? 1 : 0] * (ws * (double)Q1 + wz * (double)ts[k][TWO ? 1 : 0]);
                }
            }
        }
    }
}

// The warp in charge of sub-block (tile, q4, chalf) adds the partials of the tile's `ns` slots in slot order and stores the
// outputs of its 32 rows.  int8 tiles: column half `chalf` holds sessions 2 chalf, 2 chalf + 1 (4 digits each); fp16 tiles:
// half 0 holds all four sessions as (hi, lo) pairs.  Loads of data written by other CTAs bypass L1.
__device__ __noinline__ void dp_finish_subblock(const DpParams& P, const DpRegion& R, int v, int mat_id, const DpMat& mat, bool i8, int tile, int mt, int ns,
                                                int q4, int chalf, int wwarp, int lane, int NB) {
    const int ml = q4 * 32 + lane, m = mt * 128 + ml;
    const bool mok = m < mat.M;
    const size_t t = (size_t)tile * R.pmax;
    const uint32_t* d0 = R.data + t * (size_t)(kDpN * 128) + (size_t)(chalf * 8) * 128 + ml;
    const DpRunMeta* mp = R.meta + t * kDpWarps + wwarp;
    const bool to_x = v == DV_P3 || v == DV_P5;  // the result is added to the residual stream: its old value is requested first
    if (i8) {
        double acc0 = 0.0, acc1 = 0.0;
        const int b0 = chalf * 2;
        const bool two = b0 + 1 < NB;
        const float x0 = (to_x && mok) ? __ldcg(P.x + (size_t)b0 * P.C + m) : 0.f;
        const float x1 = (to_x && mok && two) ? __ldcg(P.x + (size_t)(b0 + 1) * P.C + m) : 0.f;
        const double ws = mok ? mat.wscale[m] : 0.f, wz = mok ? mat.wzero[m] : 0.f;
        if (two)
            dp_sum_slots_i8<true, 4>(d0, mp, ns, b0, ws, wz, acc0, acc1);
        else
            dp_sum_slots_i8<false, 8>(d0, mp, ns, b0, ws, wz, acc0, acc1);
        if (mok) {
            if (to_x) {
                P.x[(size_t)b0 * P.C + m] = x0 + (float)acc0;  // exactly one warp of the grid finishes a given output
                if (two) P.x[(size_t)(b0 + 1) * P.C + m] = x1 + (float)acc1;
            } else {
                dp_store_output(P, v, mat_id, m, b0, (float)acc0);
                if (two) dp_store_output(P, v, mat_id, m, b0 + 1, (float)acc1);
            }
        }
    } else {
        double acc[kDpMaxNB] = {0.0, 0.0, 0.0, 0.0};
        float xo[kDpMaxNB];
#pragma unroll
        for (int b = 0; b < kDpMaxNB; ++b) xo[b] = (to_x && mok && b < NB) ? __ldcg(P.x + (size_t)b * P.C + m) : 0.f;
        for (int s0 = 0; s0 < ns; s0 += 4) {  // four slots' loads in flight (clamped indices, unconditional loads); sums in slot order
            float hi[4][kDpMaxNB], lo[4][kDpMaxNB], xs[4][kDpMaxNB];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int sk = min(s0 + k, ns - 1);
                const uint32_t* d = d0 + (size_t)sk * (kDpN * 128);
                const DpRunMeta* ms = mp + (size_t)sk * kDpWarps;
#pragma unroll
                for (int b = 0; b < kDpMaxNB; ++b) {
                    const int bb = min(b, NB - 1);
                    hi[k][b] = __uint_as_float(__ldcg(d + (2 * bb) * 128));
                    lo[k][b] = __uint_as_float(__ldcg(d + (2 * bb + 1) * 128));
                    xs[k][b] = __ldcg(&ms->xscale[bb]);
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (s0 + k < ns) {
#pragma unroll
                    for (int b = 0; b < kDpMaxNB; ++b) acc[b] += (double)xs[k][b] * (double)(hi[k][b] + lo[k][b]);
                }
        }
        if (mok) {
#pragma unroll
            for (int b = 0; b < kDpMaxNB; ++b)
                if (b < NB) {
                    if (to_x)
                        P.x[(size_t)b * P.C + m] = xo[b] + (float)acc[b];
                    else
                        dp_store_output(P, v, mat_id, m, b, (float)acc[b]);
                }
        }
    }
}

// Builds the schedule of one phase variant for this CTA.  Executed by one thread.
__device__ void dp_build_variant(const DpParams& P, int v, int cta, int G, DpVar& V, DpUnit* units, int& unit_cursor, int* status) {
    const DpMat* lm = P.layers[0].mat;
    int mats[7], n = 0;
    switch (v) {
        case DV_P1A:
        case DV_P1B:
            mats[0] = DM_WR;
            mats[1] = DM_WK;
            mats[2] = DM_WV;
            mats[3] = DM_W1;
            mats[4] = DM_A1;
            mats[5] = DM_G1;
            n = 6;
            if (v == DV_P1B) mats[n++] = DM_V1;
            V.region = DR_P1;
            break;
        case DV_P3:
            mats[0] = DM_WO;
            n = 1;
            V.region = DR_P3;
            break;
        case DV_P4:
            mats[0] = DM_WFK;
            n = 1;
            V.region = DR_P4;
            break;
        case DV_P5:
            mats[0] = DM_WFV;
            n = 1;
            V.region = DR_P5;
            break;
        default:
            mats[0] = DM_HEAD;
            n = 1;
            V.region = DR_HEAD;
            break;
    }
    V.nprob = n;
    int U = 0, T = 0;
    for (int i = 0; i < n; ++i) {
        const DpMat& mt = mats[i] == DM_HEAD ? P.head : lm[mats[i]];
        V.p_mat[i] = mats[i];
        V.p_mtiles[i] = mt.mtiles;
        V.p_kblocks[i] = mt.kblocks;
        V.p_i8[i] = mt.is_i8;
        V.p_K[i] = mt.K;
        V.p_unit0[i] = U;
        V.p_tile0[i] = T;
        U += mt.mtiles * mt.kblocks;
        T += mt.mtiles;
    }
    V.U = U;
    V.ge = dp_choose_ge(V.p_unit0, n, U, G);  // only the first ge CTAs take part: the CTAs sharing a tile are consecutive
    V.unit0 = unit_cursor;
    V.nunits = V.nruns = V.nshares = 0;
    if (cta >= V.ge) return;
    const int ub = dp_cta_begin(cta, U, V.ge), ue = dp_cta_begin(cta + 1, U, V.ge);
    int base = 0;
    for (int i = 0; i < n; ++i) {  // operand shares
        const int lo = max(ub, V.p_unit0[i]), hi = min(ue, V.p_unit0[i] + V.p_mtiles[i] * V.p_kblocks[i]);
        if (hi <= lo) continue;
        const int nt = min(hi - lo, V.p_kblocks[i]);
        if (V.nshares < kDpMaxShares)
            V.share[V.nshares] = DpShare{(uint8_t)i, (uint8_t)nt, (uint8_t)((lo - V.p_unit0[i]) % V.p_kblocks[i]), (uint8_t)base};
        else
            atomicOr(status, 8);
        ++V.nshares;
        base += nt;
    }
    if (base > P.btiles || (ue - ub) + unit_cursor > P.max_units) {
        atomicOr(status, 8);  // tables too small for this shape (the host sizes them with the same formulas)
        V.nshares = 0;
        return;
    }
    int prev_tile = -1;
    for (int u = ub; u < ue; ++u) {
        int pi = 0;
        while (pi + 1 < n && u >= V.p_unit0[pi + 1]) ++pi;
        const int local = u - V.p_unit0[pi], kb = local % V.p_kblocks[pi], mt = local / V.p_kblocks[pi];
        const int tile = V.p_tile0[pi] + mt;
        int bt = 0, b2 = 0;  // operand tile of this unit
        for (int i = 0; i < n; ++i) {
            const int lo = max(ub, V.p_unit0[i]), hi = min(ue, V.p_unit0[i] + V.p_mtiles[i] * V.p_kblocks[i]);
            if (hi <= lo) continue;
            const int cnt = hi - lo;
            if (i == pi) {
                bt = b2 + (cnt >= V.p_kblocks[i] ? kb : u - lo);
                break;
            }
            b2 += min(cnt, V.p_kblocks[i]);
        }
        DpUnit& e = units[unit_cursor + V.nunits];
        e.kb = (uint16_t)kb;
        e.mt = (uint16_t)mt;
        e.prob = (uint8_t)pi;
        e.btile = (uint8_t)bt;
        e.flags = V.p_i8[pi] ? 4 : 0;
        e.pad = 0;
        if (tile != prev_tile) {
            e.flags |= 1;
            if (V.nunits > 0) units[unit_cursor + V.nunits - 1].flags |= 2;
            const int tile_first = u - kb;
            DpRun r;
            r.tile = (uint16_t)tile;
            r.u0 = (uint16_t)V.nunits;
            r.nu = 0;
            r.slot = (uint8_t)((u == tile_first) ? 0 : (cta - dp_cta_of(tile_first, U, V.ge)));
            r.prob = (uint8_t)pi;
            r.ns = (uint8_t)(dp_cta_of(tile_first + V.p_kblocks[pi] - 1, U, V.ge) - dp_cta_of(tile_first, U, V.ge) + 1);
            if (V.nruns < kDpMaxRuns)
                V.run[V.nruns] = r;
            else
                atomicOr(status, 8);
            ++V.nruns;
            prev_tile = tile;
        }
        if (V.nruns <= kDpMaxRuns) V.run[V.nruns - 1].nu++;
        ++V.nunits;
    }
    if (V.nunits > 0) units[unit_cursor + V.nunits - 1].flags |= 2;
    unit_cursor += V.nunits;
}

__global__ void __launch_bounds__(kDpThreads, 1) decode_persistent_kernel(const __grid_constant__ DpParams P) {
    extern __shared__ __align__(1024) uint8_t dp_smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)dp_smem_raw + 1023) & ~(uintptr_t)1023);
    const int NS = P.nstages;
    uint8_t* ring = smem;
    uint8_t* btile = ring + (size_t)NS * kDpATile;
    uint64_t* full = reinterpret_cast<uint64_t*>(btile + (size_t)P.btiles * kDpBTile);
    uint64_t* empty = full + NS;
    uint64_t* acc_full = empty + NS;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* b_ready = acc_empty + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(b_ready + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* red = reinterpret_cast<float*>(tmem_slot + 4);                              // [16]
    DpStats* st_ln = reinterpret_cast<DpStats*>(red + 16);                             // [4] stats of the current LN input
    DpStats* st_emb = st_ln + kDpMaxNB;                                                // [4] LN0 stats of the embedding rows
    float* sc_scale = reinterpret_cast<float*>(st_emb + kDpMaxNB);                     // [4 shares][4] operand scale
    int* sc_ex = reinterpret_cast<int*>(sc_scale + 16);                                // [4 shares][4] operand exponent
    float* sc_amax = reinterpret_cast<float*>(sc_ex + 16);                             // [8 warps][4]
    long long* sc_tsum = reinterpret_cast<long long*>(sc_amax + kDpWarps * 4);         // [btiles][4]
    float* sc_mid = reinterpret_cast<float*>(sc_tsum + (size_t)P.btiles * kDpMaxNB);   // [wm+am+vm+gm]
    float* sc_hv = sc_mid + (P.wm + P.am + P.vm + P.gm);                               // 8 x 64
    uint32_t* sc_tok = reinterpret_cast<uint32_t*>(sc_hv + 8 * 64);                    // [4]
    float* sc_shift = reinterpret_cast<float*>(sc_tok + 4);                            // [4][slice] pending channel-mix shift state
    DpLayer* sc_layer = reinterpret_cast<DpLayer*>(sc_shift + kDpMaxNB * kDpMaxSlice); // [2] table of the current / next layer
    DpVar* vars = reinterpret_cast<DpVar*>(sc_layer + 2);                              // [DV_COUNT]
    DpUnit* units = reinterpret_cast<DpUnit*>(vars + DV_COUNT);                        // [max_units]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x, cta = blockIdx.x;
    const int C = P.C, NB = P.nb;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], kDpWarps);
        }
        mbar_init(b_ready, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        int cursor = 0;
        for (int v = 0; v < DV_COUNT; ++v) dp_build_variant(P, v, cta, G, vars[v], units, cursor, P.status);
    }
    // zero the operand tiles once: columns of absent sessions stay zero for the whole launch
    for (int i = threadIdx.x; i < P.btiles * kDpBTile / 16; i += kDpThreads) reinterpret_cast<uint4*>(btile)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 1) {
        tmem_alloc(tmem_slot, 128);  // 2 run buffers x 4 accumulator chains x 16 columns
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // =========================== TMA producer ===========================
        // Lane 0 issues the weight tiles.  Before each phase's tiles all 32 lanes pull the small arrays of that phase
        // (LayerNorm / mix vectors, rank back-projection matrices, per-row scales, recurrent state) into L2, every CTA
        // its share of the lines: they are not part of the TMA stream, and the producer runs about one phase ahead of
        // the workers, so their dependent loads find the data in L2 instead of HBM.
        auto pf = [&](const void* p, size_t bytes) { dp_prefetch_l2(p, bytes, cta, G, lane, 32); };
        const size_t cb = (size_t)C * 4;
        uint32_t it = 0;
        bool ok = true;
        for (int t = 0; t < P.n_tokens && ok; ++t) {
            const bool do_head = P.argmax_feed || t == P.n_tokens - 1;
            for (int l = 0; l <= P.L && ok; ++l) {
                if (l == P.L && !do_head) break;
                for (int phs = 0; phs < (l == P.L ? 1 : 4) && ok; ++phs) {
                    const int v = l == P.L ? DV_HEAD : (phs == 0 ? (l == 0 ? DV_P1A : DV_P1B) : DV_P3 + phs - 1);
                    const DpVar& V = vars[v];
                    if (v == DV_HEAD) {
                        pf(P.lno_w, cb);
                        pf(P.lno_b, cb);
                    } else {
                        const DpLayer* Ln = &P.layers[l];
                        if (v == DV_P1A || v == DV_P1B) {
                            for (const float* p : {Ln->ln1_w, Ln->ln1_b, Ln->x_r, Ln->x_w, Ln->x_k, Ln->x_v, Ln->x_a, Ln->x_g}) pf(p, cb);
                            for (int mi : {DM_WR, DM_WK, DM_WV})
                                if (Ln->mat[mi].is_i8) {
                                    pf(Ln->mat[mi].wscale, cb);
                                    pf(Ln->mat[mi].wzero, cb);
                                }
                            for (int b = 0; b < NB; ++b) pf(Ln->tmix_x + (size_t)P.slot[b] * C, cb);
                        } else if (v == DV_P3) {  // the heads phase runs before phase 3
                            if (l + 1 < P.L) pf(P.layers + (l + 1), sizeof(DpLayer));  // the table the workers stage during phase 4
                            pf(Ln->w2, (size_t)C * P.wm * 2);
                            pf(Ln->a2, (size_t)C * P.am * 2);
                            pf(Ln->v2, (size_t)C * P.vm * 2);
                            pf(Ln->g2, (size_t)C * P.gm * 2);
                            for (const float* p : {Ln->w0, Ln->a0, Ln->v0, Ln->k_k, Ln->k_a, Ln->r_k, Ln->lnx_w, Ln->lnx_b}) pf(p, cb);
                            if (Ln->mat[DM_WO].is_i8) {
                                pf(Ln->mat[DM_WO].wscale, cb);
                                pf(Ln->mat[DM_WO].wzero, cb);
                            }
                            for (int b = 0; b < NB; ++b) pf(Ln->wkv + (size_t)P.slot[b] * P.H * 64 * 64, (size_t)P.H * 64 * 64 * 4);
                        } else if (v == DV_P4) {
                            for (const float* p : {Ln->ln2_w, Ln->ln2_b, Ln->ffn_x_k}) pf(p, cb);
                            for (int b = 0; b < NB; ++b) pf(Ln->cmix_x + (size_t)P.slot[b] * C, cb);
                            if (Ln->mat[DM_WFK].is_i8) {
                                pf(Ln->mat[DM_WFK].wscale, (size_t)P.F * 4);
                                pf(Ln->mat[DM_WFK].wzero, (size_t)P.F * 4);
                            }
                            if (Ln->mat[DM_WFV].is_i8) {
                                pf(Ln->mat[DM_WFV].wscale, cb);
                                pf(Ln->mat[DM_WFV].wzero, cb);
                            }
                        }
                    }
                    if (lane == 0) {
                        const DpUnit* un = units + V.unit0;
                        DP_DBG(const bool dbg_here = P.dbg && cta == 0 && t == 1 && l == 1 && v == DV_P4; if (dbg_here) P.dbg[55] = dp_now();)
                        for (int i = 0; i < V.nunits; ++i, ++it) {
                            const DpUnit e = un[i];
                            const int map = V.p_mat[e.prob] == DM_HEAD ? P.L * 10 : l * 10 + V.p_mat[e.prob];
                            const int s = it % NS;
                            if (!mbar_wait(&empty[s], ((it / NS) & 1u) ^ 1u, abort_flag)) {
                                ok = false;
                                break;
                            }
                            mbar_expect_tx(&full[s], kDpATile);
                            tma_load_2d(&P.maps[map], &full[s], ring + (size_t)s * kDpATile, (int)e.kb * ((e.flags & 4) ? 128 : 64), (int)e.mt * 128);
                        }
                        DP_DBG(if (dbg_here) P.dbg[56] = dp_now();)
                    }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;  // keeps the lanes in step with the tile issue
                }
            }
        }
    } else if (warp == 1) {
        // =========================== MMA issuer ===========================
        // The whole warp runs this loop convergently and one elected lane issues (see tc_mma_elect): operands stay warp-uniform,
        // ring slot and parity are counters instead of divisions.  Per 16 KB tile: one barrier wait, four MMAs, one commit.
        {
            uint32_t slot_i = 0, slot_par = 0, run = 0, phase_seq = 0;
            bool ok = true;
            const uint32_t idesc_i8 = tc_idesc(true, kDpN), idesc_f16 = tc_idesc(false, kDpN);
            const uint32_t ring_addr = smem_u32(ring), btile_addr = smem_u32(btile);
            for (int t = 0; t < P.n_tokens && ok; ++t) {
                const bool do_head = P.argmax_feed || t == P.n_tokens - 1;
                for (int l = 0; l <= P.L && ok; ++l) {
                    if (l == P.L && !do_head) break;
                    for (int phs = 0; phs < (l == P.L ? 1 : 4) && ok; ++phs) {
                        const int v = l == P.L ? DV_HEAD : (phs == 0 ? (l == 0 ? DV_P1A : DV_P1B) : DV_P3 + phs - 1);
                        const DpVar& V = vars[v];
                        const DpUnit* un = units + V.unit0;
                        const int nunits = V.nunits;
                        ok = __all_sync(0xffffffffu, mbar_wait(b_ready, phase_seq & 1u, abort_flag));
                        ++phase_seq;
                        if (!ok) break;
                        tc_fence_after();
                        DP_DBG(const bool dbg_here = P.dbg && cta == 0 && t == 1 && l == 1 && v == DV_P4; if (dbg_here && lane == 0) P.dbg[50] = dp_now();)
                        for (int i = 0; i < nunits; ++i) {
                            const DpUnit e = un[i];
                            if (e.flags & 1) {
                                ok = __all_sync(0xffffffffu, mbar_wait(&acc_empty[run & 1], (((run >> 1) & 1u) ^ 1u), abort_flag));
                                if (!ok) break;
                                tc_fence_after();
                            }
                            ok = __all_sync(0xffffffffu, mbar_wait(&full[slot_i], slot_par, abort_flag));
                            if (!ok) break;
                            tc_fence_after();
                            const uint64_t adesc = tc_smem_desc(ring_addr + slot_i * (uint32_t)kDpATile);
                            const uint64_t bdesc = tc_smem_desc(btile_addr + (uint32_t)e.btile * (uint32_t)kDpBTile);
                            // The four 32-byte K sub-blocks of a tile accumulate into four separate accumulators (summed when the run
                            // is drained), so no MMA waits for the previous one's result.
                            const uint32_t d_tmem = tmem_base + (run & 1) * (4 * kDpN);
                            const uint32_t acc0 = (e.flags & 1) ? 0u : 1u;
                            if (e.flags & 4) {
#pragma unroll
                                for (int k4 = 0; k4 < 4; ++k4)
                                    tc_mma_elect<true>(d_tmem + k4 * kDpN, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc_i8, acc0);
                            } else {
#pragma unroll
                                for (int k4 = 0; k4 < 4; ++k4)
                                    tc_mma_elect<false>(d_tmem + k4 * kDpN, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc_f16, acc0);
                            }
                            tc_commit_elect(&empty[slot_i]);
                            if (e.flags & 2) {
                                tc_commit_elect(&acc_full[run & 1]);
                                ++run;
                            }
                            if (++slot_i == (uint32_t)NS) {
                                slot_i = 0;
                                slot_par ^= 1u;
                            }
                        }
                        DP_DBG(if (dbg_here && lane == 0) {
                            P.dbg[51] = dp_now();
                            P.dbg[52] = 0;
                            P.dbg[53] = nunits;
                        })
                    }
                }
            }
        }
    } else {
        // =========================== workers ===========================
        const int wtid = threadIdx.x - 64;  // 0..255
        const int wwarp = wtid >> 5;
        const int q4 = warp & 3;       // TMEM lane quarter of this warp
        const int chalf = wwarp >> 2;  // which half of the 16 accumulator columns this warp drains
        unsigned bar_target = 0;
        uint32_t run = 0;
        bool ok = true;
        const int c0 = (int)(((long long)cta * C) / G), c1 = (int)(((long long)(cta + 1) * C) / G);  // this CTA's slice of the channels
        const int nmid = P.wm + P.am + P.vm + P.gm;
        // The layer table (pointers, matrix shapes) is read through shared memory: a pointer fetched from global memory in front of
        // every dependent load would add an L2 / HBM round trip to each step of the chain.
        auto stage_layer = [&](int l) {
            static_assert(sizeof(DpLayer) % 4 == 0, "DpLayer is copied word by word");
            const uint32_t* src = reinterpret_cast<const uint32_t*>(&P.layers[l]);
            uint32_t* dst = reinterpret_cast<uint32_t*>(&sc_layer[l & 1]);
            for (int i = wtid; i < (int)(sizeof(DpLayer) / 4); i += kDpWorkers) dst[i] = src[i];
        };

        for (int t = 0; t < P.n_tokens && ok; ++t) {
            const bool do_head = P.argmax_feed || t == P.n_tokens - 1;
            // ---- tokens of this step and LN0 statistics of their embedding rows ----
            if (wtid < NB) {
                uint32_t tok;
                if (P.argmax_feed && t > 0)
                    tok = sc_tok[wtid];
                else
                    tok = P.tok_from_list ? P.tok_list[(size_t)t * NB + wtid] : P.tokens[wtid];
                if (tok >= (uint32_t)P.V) {
                    atomicOr(P.status, 1);
                    tok = 0;
                }
                sc_tok[wtid] = tok;
            }
            stage_layer(0);
            dp_worker_sync();
            for (int b = 0; b < NB; ++b) {
                const __half* row = P.emb + (size_t)sc_tok[b] * C;
                float ev[16], s = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int k = wtid + i * kDpWorkers;
                    ev[i] = k < C ? __half2float(row[k]) : 0.f;
                    s += ev[i];
                }
                const float mean = dp_worker_sum(s, red, wtid) / (float)C;
                float qv = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float d = ev[i] - mean;
                    if (wtid + i * kDpWorkers < C) qv += d * d;
                }
                const float inv = 1.0f / sqrtf(dp_worker_sum(qv, red, wtid) / (float)C + kLnEps);
                if (wtid == 0) st_emb[b] = DpStats{mean, inv};
            }
            dp_worker_sync();
            // x slice of this CTA (the residual stream lives in global memory from here on)
            for (int i = wtid; i < NB * (c1 - c0); i += kDpWorkers) {
                const int b = i / (c1 - c0), m = c0 + i % (c1 - c0);
                P.x[(size_t)b * C + m] = (__half2float(P.emb[(size_t)sc_tok[b] * C + m]) - st_emb[b].mean) * st_emb[b].inv * P.ln0_w[m] + P.ln0_b[m];
            }

            for (int l = 0; l <= P.L && ok; ++l) {
                if (l == P.L && !do_head) break;
                const int nph = l == P.L ? 1 : 4;
                for (int phs = 0; phs < nph && ok; ++phs) {
                    const int v = l == P.L ? DV_HEAD : (phs == 0 ? (l == 0 ? DV_P1A : DV_P1B) : DV_P3 + phs - 1);
                    const DpVar& V = vars[v];
                    const DpLayer* Ly = l < P.L ? &sc_layer[l & 1] : nullptr;
                    const bool x_from_emb = (v == DV_P1A);  // x has not crossed a barrier yet: rebuild it from the embedding
                    DP_STAMP(phs * 10 + 0);

                    // ---------- phase 2 (heads) runs between P1 and P3 ----------
                    if (v == DV_P3) {
                        // new time-mix shift state = LN1(x) on this CTA's slice (all readers of the old state are past barrier 1)
                        for (int i = wtid; i < NB * (c1 - c0); i += kDpWorkers) {
                            const int b = i / (c1 - c0), m = c0 + i % (c1 - c0);
                            Ly->tmix_x[(size_t)P.slot[b] * C + m] = (P.x[(size_t)b * C + m] - st_ln[b].mean) * st_ln[b].inv * Ly->ln1_w[m] + Ly->ln1_b[m];
                        }
                        for (int item = cta; item < NB * P.H; item += G) {
                            const int b = item / P.H, h = item % P.H;
                            const int ch = h * 64 + (wtid >> 2), quad = wtid & 3;  // 4 threads per channel / state row
                            // state row (wtid>>2), columns [16*quad, 16*quad+16): requested first, used last
                            float* srow = Ly->wkv + (((size_t)P.slot[b] * P.H + h) * 64 + (wtid >> 2)) * 64 + quad * 16;
                            float4 s4[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) s4[j] = *reinterpret_cast<const float4*>(srow + 4 * j);
                            // this thread's quarter rows of the back-projection matrices -> L1, per-channel parameters -> registers
                            dp_prefetch_l1(Ly->w2 + (size_t)ch * P.wm + quad * (P.wm >> 2));
                            dp_prefetch_l1(Ly->a2 + (size_t)ch * P.am + quad * (P.am >> 2));
                            dp_prefetch_l1(Ly->g2 + (size_t)ch * P.gm + quad * (P.gm >> 2));
                            if ((P.gm >> 2) > 64) dp_prefetch_l1(Ly->g2 + (size_t)ch * P.gm + quad * (P.gm >> 2) + 64);
                            if (l > 0) dp_prefetch_l1(Ly->v2 + (size_t)ch * P.vm + quad * (P.vm >> 2));
                            const float p_w0 = Ly->w0[ch], p_a0 = Ly->a0[ch], p_kk = Ly->k_k[ch], p_ka = Ly->k_a[ch], p_rk = Ly->r_k[ch];
                            const float p_gw = Ly->lnx_w[ch], p_gb = Ly->lnx_b[ch];
                            const float p_v0 = l > 0 ? Ly->v0[ch] : 0.f, p_vf = l > 0 ? P.vfirst[(size_t)b * C + ch] : 0.f;
                            dp_worker_sync();  // the previous item is done with the scratch vectors
                            // rank-space vectors of session b and r, k, v of this head (all loads issued before the first store)
                            {
                                constexpr int kGather = 4;  // nmid + 192 <= 4 * 256
                                float gv[kGather];
#pragma unroll
                                for (int i = 0; i < kGather; ++i) {
                                    const int j = min(wtid + i * kDpWorkers, nmid + 3 * 64 - 1);
                                    const int jj = j - nmid;
                                    gv[i] = j < nmid ? P.mid[(size_t)b * nmid + j] : P.rkv[((size_t)b * 3 + (jj >> 6)) * C + h * 64 + (jj & 63)];
                                }
#pragma unroll
                                for (int i = 0; i < kGather; ++i) {
                                    const int j = wtid + i * kDpWorkers;
                                    if (j < nmid)
                                        sc_mid[j] = gv[i];
                                    else if (j < nmid + 3 * 64)
                                        sc_hv[j - nmid] = gv[i];
                                }
                                for (int j = wtid + kGather * kDpWorkers; j < nmid + 3 * 64; j += kDpWorkers) {  // larger rank spaces
                                    const int jj = j - nmid;
                                    const float t2 = j < nmid ? P.mid[(size_t)b * nmid + j] : P.rkv[((size_t)b * 3 + (jj >> 6)) * C + h * 64 + (jj & 63)];
                                    if (j < nmid)
                                        sc_mid[j] = t2;
                                    else
                                        sc_hv[jj] = t2;
                                }
                            }
                            dp_worker_sync();
                            // back-projections: the four threads of a channel split the rank dimension in contiguous quarters
                            auto dot_q = [&](const __half* W, int mid, const float* vec) {
                                float a = 0.f;
                                const int ql = mid >> 2;
                                if ((mid & 3) == 0 && (ql & 7) == 0) {
                                    const __half* wrow = W + (size_t)ch * mid + quad * ql;
                                    const float* vv = vec + quad * ql;
                                    for (int j = 0; j < ql; j += 8) {
                                        const uint4 pk = *reinterpret_cast<const uint4*>(wrow + j);
                                        const __half2* h2 = reinterpret_cast<const __half2*>(&pk);
#pragma unroll
                                        for (int e = 0; e < 4; ++e) {
                                            const float2 f = __half22float2(h2[e]);
                                            a = fmaf(f.x, vv[j + 2 * e], a);
                                            a = fmaf(f.y, vv[j + 2 * e + 1], a);
                                        }
                                    }
                                } else {
                                    for (int j = quad; j < mid; j += 4) a = fmaf(__half2float(W[(size_t)ch * mid + j]), vec[j], a);
                                }
                                a += __shfl_xor_sync(0xffffffffu, a, 1);
                                return a + __shfl_xor_sync(0xffffffffu, a, 2);
                            };
                            const float dw = dot_q(Ly->w2, P.wm, sc_mid);
                            const float da = dot_q(Ly->a2, P.am, sc_mid + P.wm);
                            const float dg = dot_q(Ly->g2, P.gm, sc_mid + P.wm + P.am + P.vm);
                            const float wdec = expf((1.0f / (1.0f + expf(-(dw + p_w0)))) * kDecayScale);
                            const float aa = 1.0f / (1.0f + expf(-(da + p_a0)));
                            const float rr = sc_hv[(wtid >> 2)], kk0 = sc_hv[64 + (wtid >> 2)];
                            float vv0 = sc_hv[128 + (wtid >> 2)];
                            if (l == 0) {
                                if (quad == 0) {
                                    P.vfirst[(size_t)b * C + ch] = vv0;
                                    P.state_vfirst[(size_t)P.slot[b] * C + ch] = vv0;
                                }
                            } else {
                                const float dv = dot_q(Ly->v2, P.vm, sc_mid + P.wm + P.am);
                                const float gate = 1.0f / (1.0f + expf(-(dv + p_v0)));
                                vv0 = vv0 + gate * (p_vf - vv0);
                            }
                            const float kkj = kk0 * p_kk;
                            const float ss = dp_worker_sum(quad == 0 ? kkj * kkj : 0.f, red, wtid);
                            const float kkh = kkj * (1.0f / fmaxf(sqrtf(ss), kL2Eps));
                            const float kt = kk0 + p_ka * (kk0 * aa - kk0);
                            if (quad == 0) {
                                const int i = wtid >> 2;
                                sc_hv[3 * 64 + i] = wdec;
                                sc_hv[4 * 64 + i] = rr;
                                sc_hv[5 * 64 + i] = kkh;
                                sc_hv[6 * 64 + i] = kkh * (-aa);
                                sc_hv[7 * 64 + i] = kt;
                            }
                            dp_worker_sync();
                            float S[16];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                S[4 * j] = s4[j].x;
                                S[4 * j + 1] = s4[j].y;
                                S[4 * j + 2] = s4[j].z;
                                S[4 * j + 3] = s4[j].w;
                            }
                            const float *s_w = sc_hv + 3 * 64 + quad * 16, *s_r = sc_hv + 4 * 64 + quad * 16, *s_kk = sc_hv + 5 * 64 + quad * 16,
                                        *s_b = sc_hv + 6 * 64 + quad * 16, *s_kt = sc_hv + 7 * 64 + quad * 16;
                            float sa = 0.f;
#pragma unroll
                            for (int j = 0; j < 16; ++j) sa = fmaf(S[j], s_kk[j], sa);
                            sa += __shfl_xor_sync(0xffffffffu, sa, 1);
                            sa += __shfl_xor_sync(0xffffffffu, sa, 2);
                            float y = 0.f;
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                S[j] = fmaf(S[j], s_w[j], fmaf(sa, s_b[j], vv0 * s_kt[j]));
                                y = fmaf(S[j], s_r[j], y);
                            }
                            y += __shfl_xor_sync(0xffffffffu, y, 1);
                            y += __shfl_xor_sync(0xffffffffu, y, 2);
#pragma unroll
                            for (int j = 0; j < 4; ++j) *reinterpret_cast<float4*>(srow + 4 * j) = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
                            const float mean = dp_worker_sum(quad == 0 ? y : 0.f, red, wtid) / 64.0f;
                            const float d = y - mean;
                            const float var = dp_worker_sum(quad == 0 ? d * d : 0.f, red, wtid) / 64.0f + kGnEps;
                            const float srk = dp_worker_sum(quad == 0 ? rr * kt * p_rk : 0.f, red, wtid);
                            if (quad == 0) P.yg[(size_t)b * C + ch] = (d * (1.0f / sqrtf(var)) * p_gw + p_gb + srk * vv0) * dg;
                        }
                        DP_STAMP(40);
                        ok = dp_grid_barrier(P.grid_bar, bar_target, G, abort_flag, wtid);
                        if (!ok) break;
                        DP_STAMP(41);
                    }

                    // ---------- LayerNorm statistics of the phase input (full rows, every CTA) ----------
                    if (v == DV_P1A || v == DV_P1B || v == DV_P4 || v == DV_HEAD) {
                        for (int b = 0; b < NB; ++b) {
                            const __half* erow = P.emb + (size_t)sc_tok[b] * C;
                            const DpStats se = st_emb[b];
                            // C <= 16 * 256: each worker keeps its elements in registers between the two passes
                            float xv[16];
                            float s = 0.f;
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const int k = wtid + i * kDpWorkers;
                                xv[i] = 0.f;
                                if (k < C) xv[i] = x_from_emb ? ((__half2float(erow[k]) - se.mean) * se.inv * P.ln0_w[k] + P.ln0_b[k]) : P.x[(size_t)b * C + k];
                                s += xv[i];
                            }
                            const float mean = dp_worker_sum(s, red, wtid) / (float)C;
                            float qv = 0.f;
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const float dd = xv[i] - mean;
                                if (wtid + i * kDpWorkers < C) qv += dd * dd;
                            }
                            const float inv = 1.0f / sqrtf(dp_worker_sum(qv, red, wtid) / (float)C + kLnEps);
                            if (wtid == 0) st_ln[b] = DpStats{mean, inv};
                        }
                        dp_worker_sync();
                    }
                    if (v == DV_P4 && l + 1 < P.L) stage_layer(l + 1);
                    if (v == DV_P4) {
                        // new channel-mix shift state = LN2(x) on this CTA's slice: computed now, while x is stable, stored in
                        // phase 5 when every reader of the old state is past the barrier (phase 5 itself updates x)
                        for (int i = wtid; i < NB * (c1 - c0); i += kDpWorkers) {
                            const int b = i / (c1 - c0), m = c0 + i % (c1 - c0);
                            sc_shift[i] = (P.x[(size_t)b * C + m] - st_ln[b].mean) * st_ln[b].inv * Ly->ln2_w[m] + Ly->ln2_b[m];
                        }
                    }
                    if (v == DV_P5) {
                        for (int i = wtid; i < NB * (c1 - c0); i += kDpWorkers) {
                            const int b = i / (c1 - c0), m = c0 + i % (c1 - c0);
                            Ly->cmix_x[(size_t)P.slot[b] * C + m] = sc_shift[i];
                        }
                    }
                    DP_STAMP(phs * 10 + 1);

                    // ---------- operand tiles of this CTA's units ----------
                    {
                        const float *lw = nullptr, *lb = nullptr, *shift = nullptr;
                        if (v == DV_P1A || v == DV_P1B) {
                            lw = Ly->ln1_w;
                            lb = Ly->ln1_b;
                            shift = Ly->tmix_x;
                        } else if (v == DV_P4) {
                            lw = Ly->ln2_w;
                            lb = Ly->ln2_b;
                            shift = Ly->cmix_x;
                        } else if (v == DV_HEAD) {
                            lw = P.lno_w;
                            lb = P.lno_b;
                        }
                        // The value of element k of the phase input is computed without a branch: every load has a valid (if unused)
                        // address and the phase kind only selects among the results, so that the loads of all of a thread's elements are
                        // in flight together instead of one element per memory round trip.
                        const bool has_ln = !(v == DV_P3 || v == DV_P5), has_mix = has_ln && v != DV_HEAD;
                        const float* src = v == DV_P3 ? P.yg : (v == DV_P5 ? P.hbuf : P.x);
                        const int sstride = v == DV_P5 ? P.F : C;
                        const float* lwp = has_ln ? lw : P.ln0_w;
                        const float* lbp = has_ln ? lb : P.ln0_b;
                        const float* shiftp = has_mix ? shift : P.ln0_w;
                        auto mixptr = [&](int pi) -> const float* {  // mix vector of a problem of phase 1 / 4
                            if (!has_mix) return P.ln0_w;
                            if (v == DV_P4) return Ly->ffn_x_k;
                            switch (V.p_mat[pi]) {
                                case DM_WR: return Ly->x_r;
                                case DM_WK: return Ly->x_k;
                                case DM_WV: return Ly->x_v;
                                case DM_W1: return Ly->x_w;
                                case DM_A1: return Ly->x_a;
                                case DM_G1: return Ly->x_g;
                                default: return Ly->x_v;  // DM_V1
                            }
                        };
                        auto input = [&](const float* mixp, int b, int k) -> float {
                            const int kl = has_ln ? k : 0;
                            const float xs = src[(size_t)b * sstride + k];
                            const float xe = (__half2float(P.emb[(size_t)sc_tok[b] * C + kl]) - st_emb[b].mean) * st_emb[b].inv * P.ln0_w[kl] + P.ln0_b[kl];
                            const float xv = x_from_emb ? xe : xs;
                            const float cur = (xv - st_ln[b].mean) * st_ln[b].inv * lwp[kl] + lbp[kl];
                            const float prev = shiftp[(has_mix ? (size_t)P.slot[b] * C : (size_t)0) + kl];
                            const float mixed = cur + mixp[kl] * (prev - cur);
                            return has_mix ? mixed : (has_ln ? cur : xs);
                        };
                        // quantise one element into its operand tile and add it to the tile's exact fixed-point sum
                        auto emit = [&](bool i8, uint8_t* tile, int tile_idx, int sh, int b, int e, float val) {
                            if (i8) {
                                float vq = val * dp_pow2(kDpP - sc_ex[sh * 4 + b]);
                                vq = fminf(fmaxf(vq, -(float)(1 << kDpP)), (float)(1 << kDpP));
                                int tq = (vq == vq) ? __float2int_rn(vq) : 0;
                                const int t_full = tq;
#pragma unroll
                                for (int j = kDpDigits - 1; j > 0; --j) {
                                    const int dj = ((tq + 64) & 127) - 64;
                                    tile[dp_b_offset(b * kDpDigits + j, e)] = (uint8_t)(int8_t)dj;
                                    tq = (tq - dj) >> 7;
                                }
                                tile[dp_b_offset(b * kDpDigits, e)] = (uint8_t)(int8_t)tq;
                                // the 32 lanes of a warp work on the same tile: one shared-memory add per warp.  |t| <= 2^27, so the warp sum is
                                // taken exactly with two 32-bit warp reductions (low 16 bits unsigned, the rest signed)
                                const unsigned lo_sum = __reduce_add_sync(0xffffffffu, (unsigned)(t_full & 0xFFFF));
                                const int hi_sum = __reduce_add_sync(0xffffffffu, t_full >> 16);
                                const long long ts = (long long)hi_sum * 65536 + (long long)lo_sum;
                                if (lane == 0) atomicAdd(reinterpret_cast<unsigned long long*>(&sc_tsum[(size_t)tile_idx * kDpMaxNB + b]), (unsigned long long)ts);
                            } else {
                                float vq = val * dp_pow2(-sc_ex[sh * 4 + b]);
                                vq = fminf(fmaxf(vq, -1.0f), 1.0f);
                                if (!(vq == vq)) vq = 0.f;
                                const __half hi16 = __float2half_rn(vq);
                                const __half lo16 = __float2half_rn(vq - __half2float(hi16));
                                *reinterpret_cast<__half*>(tile + dp_b_offset(b * 2, e * 2)) = hi16;
                                *reinterpret_cast<__half*>(tile + dp_b_offset(b * 2 + 1, e * 2)) = lo16;
                            }
                        };
                        // reduce the per-thread magnitudes to the power-of-two scale of (share, session); all workers call this
                        auto set_scale = [&](bool i8, int sh, int b, float am) {
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
                            if (lane == 0) sc_amax[wwarp] = am;
                            dp_worker_sync();
                            if (wtid == 0) {
                                float a = 0.f;
                                for (int w = 0; w < kDpWarps; ++w) a = fmaxf(a, sc_amax[w]);
                                int ex = 0;
                                if (a >= 1.0e-30f && a < 3.0e38f) ex = dp_ceil_log2(a);
                                ex = max(-90, min(90, ex));
                                sc_ex[sh * 4 + b] = ex;
                                sc_scale[sh * 4 + b] = i8 ? dp_pow2(ex - kDpP) : dp_pow2(ex);
                            }
                            dp_worker_sync();
                        };
                        constexpr int kMaxItems = 6;  // register-resident (tile, element) items per worker
                        const int nshare = min(V.nshares, kDpMaxShares);
                        int tiles_total = 0;
                        for (int sh = 0; sh < nshare; ++sh) tiles_total += V.share[sh].ntile;
                        for (int i = wtid; i < tiles_total * kDpMaxNB; i += kDpWorkers) sc_tsum[i] = 0;  // made visible by the syncs in set_scale
                        // loops over shares and sessions stay rolled: this code runs once per phase, so its size (instruction
                        // fetch) matters more than its issue rate
#pragma unroll 1
                        for (int sh = 0; sh < nshare; ++sh) {
                            const DpShare S = V.share[sh];
                            const int pi = S.prob;
                            const float* mixp = mixptr(pi);
                            const bool i8 = V.p_i8[pi] != 0;
                            const int epb = i8 ? 128 : 64, kbs = V.p_kblocks[pi], K = V.p_K[pi];
                            const int grp = kDpWorkers / epb;  // tiles handled side by side
                            const int sub = wtid / epb, e = wtid % epb;
#pragma unroll 1
                            for (int b = 0; b < NB; ++b) {
                                float am = 0.f;
                                if (S.ntile <= grp * kMaxItems) {
                                    // everything fits in registers: load once, reduce the magnitude, quantise
                                    float val[kMaxItems];
                                    if (v == DV_P4) DP_STAMP(63);
                                    // the loads are unconditional (clamped index) so that all of them are in flight before the first use
                                    int kk[kMaxItems];
#pragma unroll
                                    for (int it = 0; it < kMaxItems; ++it) {
                                        const int tl = it * grp + sub, tlc = min(tl, (int)S.ntile - 1);
                                        const int kb = S.ntile == kbs ? tlc : (S.kb0 + tlc) % kbs;
                                        const int k = kb * epb + e;
                                        kk[it] = (tl >= S.ntile || k >= K) ? -1 : k;
                                    }
                                    if (has_ln) {
#pragma unroll
                                        for (int it = 0; it < kMaxItems; ++it) val[it] = input(mixp, b, max(kk[it], 0));
                                    } else {  // att.output, ffn.value: the input vector as it is
#pragma unroll
                                        for (int it = 0; it < kMaxItems; ++it) val[it] = src[(size_t)b * sstride + max(kk[it], 0)];
                                    }
#pragma unroll
                                    for (int it = 0; it < kMaxItems; ++it)
                                        if (kk[it] < 0) val[it] = 0.f;
#pragma unroll
                                    for (int it = 0; it < kMaxItems; ++it) am = fmaxf(am, fabsf(val[it]));
                                    if (v == DV_P4) DP_STAMP(60);
                                    set_scale(i8, sh, b, am);
                                    if (v == DV_P4) DP_STAMP(61);
#pragma unroll
                                    for (int it = 0; it < kMaxItems; ++it) {
                                        const int tl = it * grp + sub;
                                        if (tl < S.ntile) emit(i8, btile + (size_t)(S.base + tl) * kDpBTile, S.base + tl, sh, b, e, val[it]);
                                    }
                                    if (v == DV_P4) DP_STAMP(62);
                                } else {
                                    // many tiles (the head): one pass for the magnitude, a second one that recomputes and quantises
#pragma unroll 1
                                    for (int tl = sub; tl < S.ntile; tl += grp) {
                                        const int kb = S.ntile == kbs ? tl : (S.kb0 + tl) % kbs;
                                        const int k = kb * epb + e;
                                        if (k < K) am = fmaxf(am, fabsf(input(mixp, b, k)));
                                    }
                                    set_scale(i8, sh, b, am);
#pragma unroll 1
                                    for (int tl = sub; tl < S.ntile; tl += grp) {
                                        const int kb = S.ntile == kbs ? tl : (S.kb0 + tl) % kbs;
                                        const int k = kb * epb + e;
                                        emit(i8, btile + (size_t)(S.base + tl) * kDpBTile, S.base + tl, sh, b, e, k < K ? input(mixp, b, k) : 0.f);
                                    }
                                }
                            }
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    dp_worker_sync();
                    DP_STAMP_ALL(0);
                    if (wtid == 0) mbar_arrive(b_ready);
                    DP_STAMP(phs * 10 + 2);

                    // ---------- drain the runs of this CTA ----------
                    {
                        const DpRegion& Rg = P.reg[V.region];
                        const int nruns = min(V.nruns, kDpMaxRuns);
                        int ndone = 0;
                        // pass 1: every run's accumulator -> partial sums and scale in global memory
                        for (int ri = 0; ri < nruns; ++ri) {
                            const DpRun r = V.run[ri];
                            const size_t tidx = (size_t)r.tile * Rg.pmax + r.slot;
                            const bool got = mbar_wait_parked(&acc_full[run & 1], (run >> 1) & 1u, abort_flag);
                            if (!__all_sync(0xffffffffu, got)) break;  // the abort flag is set; decided for all workers below
                            tc_fence_after();
                            uint32_t vv[8], v2[8];
                            const uint32_t tbase = tmem_base + ((uint32_t)(q4 * 32) << 16) + (run & 1) * (4 * kDpN) + chalf * 8;
                            const bool r_i8 = V.p_i8[r.prob] != 0;
#pragma unroll
                            for (int k4 = 0; k4 < 4; ++k4) {  // add the four accumulator chains (exact for int32; fixed order for fp32)
                                asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                             : "=r"(v2[0]), "=r"(v2[1]), "=r"(v2[2]), "=r"(v2[3]), "=r"(v2[4]), "=r"(v2[5]), "=r"(v2[6]), "=r"(v2[7])
                                             : "r"(tbase + k4 * kDpN));
                                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    if (k4 == 0)
                                        vv[j] = v2[j];
                                    else if (r_i8)
                                        vv[j] = (uint32_t)((int)vv[j] + (int)v2[j]);
                                    else
                                        vv[j] = __float_as_uint(__uint_as_float(vv[j]) + __uint_as_float(v2[j]));
                                }
                            }
                            // sessions live in the first 4 NB (int8) or 2 NB (fp16) columns: a warp whose column half holds none skips
                            if (chalf * 8 < (r_i8 ? 4 : 2) * NB) {
                                uint32_t* dst = Rg.data + tidx * (size_t)(kDpN * 128) + (size_t)(chalf * 8) * 128 + q4 * 32 + lane;
#pragma unroll
                                for (int j = 0; j < 8; ++j) dst[(size_t)j * 128] = vv[j];
                                if (lane < NB) {
                                    // scale of this CTA's operand for the problem, exact sum of the run's fixed-point values
                                    const DpUnit* un = units + V.unit0 + r.u0;
                                    long long ts = 0;
                                    for (int uu = 0; uu < r.nu; ++uu) ts += sc_tsum[(size_t)un[uu].btile * kDpMaxNB + lane];
                                    int sh = 0;
                                    while (sh + 1 < V.nshares && V.share[sh].prob != r.prob) ++sh;
                                    DpRunMeta* mp = Rg.meta + tidx * kDpWarps + wwarp;
                                    mp->xscale[lane] = sc_scale[sh * 4 + lane];
                                    mp->tsum[lane] = ts;
                                }
                            }
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&acc_empty[run & 1]);
                            ++run;
                            ++ndone;
                        }
                        // arrivals: one reduction per run and warp after a single fence
                        DP_STAMP_ALL(1);
                        __syncwarp();
                        if (lane == 0) {
                            fence_acq_rel_gpu();  // the warp's partials and scales are visible device-wide before the arrivals are counted
                            for (int ri = 0; ri < ndone; ++ri) {
                                const DpRun r = V.run[ri];
                                if (chalf * 8 < (V.p_i8[r.prob] ? 4 : 2) * NB) atomicAdd(&Rg.cnt[(size_t)r.tile * kDpWarps + wwarp], 1);
                            }
                        }
                        DP_STAMP_ALL(2);
                        // pass 2: sub-block w of a tile is finished by the CTA whose slot is (w + tile) mod ns, so the finishing work of
                        // a tile is spread over its sharers and no warp finishes two sub-blocks of one tile.  That warp waits (bounded)
                        // until all ns arrivals are counted.
                        for (int ri = 0; ri < ndone; ++ri) {
                            const DpRun r = V.run[ri];
                            const bool r_i8 = V.p_i8[r.prob] != 0;
                            if (!(chalf * 8 < (r_i8 ? 4 : 2) * NB) || (wwarp + (int)r.tile) % (int)r.ns != (int)r.slot) continue;
                            int* cnt = &Rg.cnt[(size_t)r.tile * kDpWarps + wwarp];
                            int seen = 0;
                            if (lane == 0) {
                                for (uint32_t i = 0; i < kDpBarSpin; ++i) {
                                    int c;
                                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(c) : "l"(cnt) : "memory");
                                    if (c >= (int)r.ns) {
                                        seen = 1;
                                        break;
                                    }
                                    if ((i & 255u) == 255u && *abort_flag) break;
                                }
                                if (seen)
                                    *cnt = 0;  // all arrivals counted: ready for the next use
                                else
                                    *abort_flag = 1;
                            }
                            seen = __shfl_sync(0xffffffffu, seen, 0);
                            if (!seen) break;
                            const int mat_id = V.p_mat[r.prob];
                            const DpUnit u0 = units[V.unit0 + r.u0];
                            dp_finish_subblock(P, Rg, v, mat_id, mat_id == DM_HEAD ? P.head : Ly->mat[mat_id], r_i8, r.tile, u0.mt, r.ns, q4, chalf, wwarp, lane, NB);
                        }
                    }
                    DP_STAMP(phs * 10 + 3);
                    DP_STAMP_ALL(3);
                    // every worker reaches the barrier below whether or not its warp left the loop early;
                    // dp_grid_barrier returns the shared abort state, so the decision to stop is the same for all
                    ok = dp_grid_barrier(P.grid_bar, bar_target, G, abort_flag, wtid);
                    if (!ok) break;
                    DP_STAMP(phs * 10 + 4);
                    DP_STAMP_ALL(4);

                    // ---------- logits, arg-max ----------
                    if (v == DV_HEAD) {
                        const int v0 = (int)(((long long)cta * P.V) / G), v1 = (int)(((long long)(cta + 1) * P.V) / G);
                        for (int b = 0; b < NB; ++b) {
                            float bv = -1e30f;
                            int bi = 0x7fffffff;
                            for (int vv = v0 + wtid; vv < v1; vv += kDpWorkers) {
                                const float lg = P.logits[(size_t)b * P.V + vv];
                                if (lg > bv) {
                                    bv = lg;
                                    bi = vv;
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
                            dp_worker_sync();
                            if (lane == 0) {
                                red[wwarp] = bv;
                                reinterpret_cast<int*>(red)[8 + wwarp] = bi;
                            }
                            dp_worker_sync();
                            if (wtid == 0) {
                                for (int w2 = 1; w2 < kDpWarps; ++w2) {
                                    const float ov = red[w2];
                                    const int oi = reinterpret_cast<int*>(red)[8 + w2];
                                    if (ov > bv || (ov == bv && oi < bi)) {
                                        bv = ov;
                                        bi = oi;
                                    }
                                }
                                P.cand_val[cta * kDpMaxNB + b] = bv;
                                P.cand_idx[cta * kDpMaxNB + b] = bi;
                            }
                        }
                        ok = dp_grid_barrier(P.grid_bar, bar_target, G, abort_flag, wtid);
                        if (!ok) break;
                        if (P.argmax_feed) {
                            // every CTA reduces the candidates itself: no further barrier before the next token
                            if (wtid < NB) {
                                float bv = -1e30f;
                                int bi = 0x7fffffff;
                                for (int c = 0; c < G; ++c) {
                                    const float ov = P.cand_val[c * kDpMaxNB + wtid];
                                    const int oi = P.cand_idx[c * kDpMaxNB + wtid];
                                    if (ov > bv || (ov == bv && oi < bi)) {
                                        bv = ov;
                                        bi = oi;
                                    }
                                }
                                if (bi == 0x7fffffff) bi = 0;
                                sc_tok[wtid] = (uint32_t)bi;
                                if (cta == 0) {
                                    P.tokens[wtid] = (uint32_t)bi;
                                    if (P.seq) {
                                        const int cnt = P.seq_cnt[wtid];
                                        if (cnt < P.seq_cap) P.seq[(size_t)wtid * P.seq_cap + cnt] = (uint32_t)bi;
                                        P.seq_cnt[wtid] = cnt + 1;
                                    }
                                }
                            }
                            dp_worker_sync();
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(P.status, 4);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 128);
    }
}

}  // namespace rsv
