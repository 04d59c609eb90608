// Persistent decode kernel: one cooperative launch runs n tokens x L layers x (head, arg-max) for up to 4
// sessions, so a whole self-loop is a single kernel.  It stands in for the reference's captured-graph decode
// step (forward_token / forward_layer / selfloop_step, src/gpu_model.rs:1879-2392) whose 8 kernels per layer
// are latency-bound at batch 1.
//
// Structure.  One CTA per SM, 192 threads:
//   warp 0   TMA producer.  Walks the fixed sequence of weight tiles (16 KB = 128 rows x 128 bytes) this CTA will
//            ever need — token after token, layer after layer, phase after phase — and keeps a shared-memory ring
//            full.  It never waits on a grid barrier, only on free ring slots, so HBM keeps streaming while the
//            other warps synchronise: the barriers cost latency, not bandwidth.
//   warp 1   MMA issuer.  tcgen05.mma (kind::i8 on the u8 codes / kind::f16) of each weight tile against the
//            activation operand tiles the workers left in shared memory; accumulators in TMEM (N = 16 columns:
//            4 sessions x 4 base-128 digits, or 4 x (hi, lo) halves).
//   warps 2-5  workers.  Per phase: build the activation operand tiles (LayerNorm, token shift, fixed-point
//            digits), drain finished accumulators to global partial sums, do the per-head WKV-7 work, take part
//            in the grid barriers.
// Work split: every GEMV phase is cut into units (128-row tile x 128-byte K block); CTA c owns the contiguous
// unit range [c*U/G, (c+1)*U/G), so each SM streams the same number of weight bytes.  A run (the units of one
// tile inside one CTA) leaves an exact int32 (or fp32) partial [16 columns][128 rows] plus its own fixed-point
// scale; consumers add a tile's partials in slot order.  Integer partials make the split exact, and every
// floating-point sum has a fixed order: results are deterministic and independent of timing.
// Phases per layer (grid barrier after each; a/b = finish the residual stream on disjoint slices, then share it):
//   1  LN1 + token shift -> r,k,v (int8) and the four rank projections (fp16)
//   2  per (session, head): rank back-projections, decay/a/v/g, WKV-7 state update in place, GroupNorm, gate
//   3  att.output           3b  x += ...        4  LN2 + shift -> ffn.key        5  relu^2 -> ffn.value   5b  x += ...
// then ln_out + head (fp16) -> logits, arg-max across CTAs, next token.
// All spin-waits are bounded; on expiry bit 2 of the status word is set and every role drains and exits.
#pragma once
#include "tc_linear.cuh"

namespace rsv {

constexpr int kDpThreads = 192;
constexpr int kDpWorkers = 128;
constexpr int kDpMaxNB = 4;
constexpr int kDpN = 16;
constexpr int kDpATile = 128 * 128;
constexpr int kDpBTile = kDpN * 128;
constexpr int kDpDigits = 4;
constexpr int kDpP = 7 * kDpDigits - 1;
constexpr uint32_t kDpBarSpin = 1u << 22;

struct DpMat {
    int map, M, mtiles, kblocks, is_i8, K;
    const float* wscale;
    const float* wzero;
};
struct DpLayer {
    DpMat Wr, Wk, Wv, Wo, Wfk, Wfv, w1, a1, v1, g1;
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
    DpRunMeta* meta;  // [tile][pmax]
    int pmax;
    int pad;
};
enum { DP_P1 = 0, DP_P3 = 1, DP_P4 = 2, DP_P5 = 3, DP_HEAD = 4 };
struct DpParams {
    const CUtensorMap* maps;
    const DpLayer* layers;
    DpMat head;
    const __half* emb;
    const float *ln0_w, *ln0_b, *lno_w, *lno_b;
    int L, C, H, F, V, wm, am, vm, gm;
    int nb;
    int slot[kDpMaxNB];
    float *x, *yg, *vfirst;  // [4][C]
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
    int nstages, btiles;
};

struct DpProb {
    DpMat mat;
    int unit0, tile0, in_kind;
    const float* mix;
};
struct DpPhase {
    DpProb p[7];
    int nprob, U, region;
};
enum { DP_IN_LNMIX = 0, DP_IN_VEC = 1, DP_IN_H = 2, DP_IN_LNOUT = 3 };

__device__ __forceinline__ void dp_add_prob(DpPhase& ph, const DpMat& m, int in_kind, const float* mix) {
    DpProb& q = ph.p[ph.nprob];
    q.mat = m;
    q.unit0 = ph.U;
    q.tile0 = ph.nprob ? ph.p[ph.nprob - 1].tile0 + ph.p[ph.nprob - 1].mat.mtiles : 0;
    q.in_kind = in_kind;
    q.mix = mix;
    ph.U += m.mtiles * m.kblocks;
    ++ph.nprob;
}
__device__ __forceinline__ void dp_build_phase(const DpParams& P, int layer, int phase, DpPhase& ph) {
    ph.nprob = 0;
    ph.U = 0;
    ph.region = phase;
    if (phase == DP_HEAD) {
        dp_add_prob(ph, P.head, DP_IN_LNOUT, nullptr);
        return;
    }
    const DpLayer& Ly = P.layers[layer];
    switch (phase) {
        case DP_P1:
            dp_add_prob(ph, Ly.Wr, DP_IN_LNMIX, Ly.x_r);
            dp_add_prob(ph, Ly.Wk, DP_IN_LNMIX, Ly.x_k);
            dp_add_prob(ph, Ly.Wv, DP_IN_LNMIX, Ly.x_v);
            dp_add_prob(ph, Ly.w1, DP_IN_LNMIX, Ly.x_w);
            dp_add_prob(ph, Ly.a1, DP_IN_LNMIX, Ly.x_a);
            dp_add_prob(ph, Ly.g1, DP_IN_LNMIX, Ly.x_g);
            if (layer > 0) dp_add_prob(ph, Ly.v1, DP_IN_LNMIX, Ly.x_v);
            break;
        case DP_P3: dp_add_prob(ph, Ly.Wo, DP_IN_VEC, nullptr); break;
        case DP_P4: dp_add_prob(ph, Ly.Wfk, DP_IN_LNMIX, Ly.ffn_x_k); break;
        case DP_P5: dp_add_prob(ph, Ly.Wfv, DP_IN_H, nullptr); break;
    }
}
__device__ __forceinline__ int dp_prob_of(const DpPhase& ph, int u) {
    int p = 0;
    while (p + 1 < ph.nprob && u >= ph.p[p + 1].unit0) ++p;
    return p;
}
// Shared-memory operand tile of unit u inside this CTA's range [ub, ue): problems whose share of the range spans a
// whole K sweep keep one tile per K block; shorter shares keep one tile per unit.
__device__ __forceinline__ int dp_btile_of(const DpPhase& ph, int ub, int ue, int u) {
    int base = 0;
    for (int p = 0; p < ph.nprob; ++p) {
        const DpProb& q = ph.p[p];
        const int lo = max(ub, q.unit0), hi = min(ue, q.unit0 + q.mat.mtiles * q.mat.kblocks);
        if (hi <= lo) continue;
        const int cnt = hi - lo;
        if (u >= lo && u < hi) return base + (cnt >= q.mat.kblocks ? (u - q.unit0) % q.mat.kblocks : u - lo);
        base += min(cnt, q.mat.kblocks);
    }
    return 0;
}

// Unit range of CTA `cta` in a phase.  Only the first min(G, U) CTAs take part, so that every participating CTA owns at
// least one unit and the CTAs sharing a tile are consecutive (the partial-slot numbering relies on it).
__device__ __forceinline__ void dp_range(const DpPhase& ph, int cta, int G, int& ub, int& ue) {
    const int ge = min(G, ph.U);
    ub = cta < ge ? tc_cta_begin(cta, ph.U, ge) : 0;
    ue = cta < ge ? tc_cta_begin(cta + 1, ph.U, ge) : 0;
}

__device__ __forceinline__ void dp_worker_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kDpWorkers) : "memory"); }

// Sum over the 128 worker threads; every worker gets the result.  `red` holds 4 floats.
__device__ __forceinline__ float dp_worker_sum(float v, float* red, int wtid) {
    v = warp_sum(v);
    dp_worker_sync();
    if ((wtid & 31) == 0) red[wtid >> 5] = v;
    dp_worker_sync();
    return (red[0] + red[1]) + (red[2] + red[3]);
}
__device__ __forceinline__ float dp_worker_max(float v, float* red, int wtid) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    dp_worker_sync();
    if ((wtid & 31) == 0) red[wtid >> 5] = v;
    dp_worker_sync();
    return fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
}

// Grid-wide barrier among the workers of all CTAs (bounded spin).  Returns false after a timeout / abort.
__device__ __forceinline__ bool dp_grid_barrier(unsigned* bar, unsigned& target, int G, volatile int* abort_flag, int wtid) {
    dp_worker_sync();
    if (wtid == 0) {
        __threadfence();
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
        __threadfence();
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

// value of output m of problem `pi` of a finished phase for session b: partials added in slot order
__device__ __forceinline__ float dp_finalize(const DpParams& P, const DpPhase& ph, int pi, int m, int b, int G) {
    const DpProb& q = ph.p[pi];
    const DpRegion& R = P.reg[ph.region];
    const int mt = m >> 7, ml = m & 127;
    const int tile_first = q.unit0 + mt * q.mat.kblocks;
    const int ge = min(G, ph.U);
    const int c_lo = tc_cta_of_unit(tile_first, ph.U, ge), c_hi = tc_cta_of_unit(tile_first + q.mat.kblocks - 1, ph.U, ge);
    const size_t t = (size_t)(q.tile0 + mt) * R.pmax;
    double acc = 0.0;
    if (q.mat.is_i8) {
        const double ws = q.mat.wscale[m], wz = q.mat.wzero[m];
        for (int s = 0; s <= c_hi - c_lo; ++s) {
            const uint32_t* d = R.data + (t + s) * (size_t)(kDpN * 128) + (size_t)(b * kDpDigits) * 128 + ml;
            long long Q = (int)d[0];
            Q = Q * 128 + (int)d[128];
            Q = Q * 128 + (int)d[256];
            Q = Q * 128 + (int)d[384];
            const DpRunMeta& mm = R.meta[t + s];
            acc += (double)mm.xscale[b] * (ws * (double)Q + wz * (double)mm.tsum[b]);
        }
    } else {
        for (int s = 0; s <= c_hi - c_lo; ++s) {
            const uint32_t* d = R.data + (t + s) * (size_t)(kDpN * 128) + (size_t)(b * 2) * 128 + ml;
            acc += (double)R.meta[t + s].xscale[b] * (double)(__uint_as_float(d[0]) + __uint_as_float(d[128]));
        }
    }
    return (float)acc;
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
    // worker scratch
    float* red = reinterpret_cast<float*>(tmem_slot + 4);                                  // [8]
    DpStats* st_ln = reinterpret_cast<DpStats*>(red + 8);                                   // [4] stats of the current LN input
    DpStats* st_emb = st_ln + kDpMaxNB;                                                     // [4] LN0 stats of the embedding rows
    float* sc_scale = reinterpret_cast<float*>(st_emb + kDpMaxNB);                          // [7][4] operand scale per (problem, session)
    long long* sc_tsum = reinterpret_cast<long long*>(sc_scale + 32);                       // [btiles][4]
    float* sc_mid = reinterpret_cast<float*>(sc_tsum + (size_t)P.btiles * kDpMaxNB);        // [wm+am+vm+gm]
    float* sc_hv = sc_mid + (P.wm + P.am + P.vm + P.gm);                                    // r,k,v,w,a(5x64) + kk,b,kt (3x64)
    uint32_t* sc_tok = reinterpret_cast<uint32_t*>(sc_hv + 8 * 64);                          // [4]

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
            mbar_init(&acc_empty[b], 4);
        }
        mbar_init(b_ready, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // zero the operand tiles once: columns of absent sessions stay zero for the whole launch
    for (int i = threadIdx.x; i < P.btiles * kDpBTile / 16; i += kDpThreads) reinterpret_cast<uint4*>(btile)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 1) {
        tmem_alloc(tmem_slot, 32);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // =========================== TMA producer ===========================
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = 0; t < P.n_tokens && ok; ++t) {
                const bool do_head = P.argmax_feed || t == P.n_tokens - 1;
                for (int l = 0; l <= P.L && ok; ++l) {
                    if (l == P.L && !do_head) break;
                    for (int phs = 0; phs < (l == P.L ? 1 : 4) && ok; ++phs) {
                        DpPhase ph;
                        dp_build_phase(P, l, l == P.L ? DP_HEAD : phs, ph);
                        int ub, ue;
                        dp_range(ph, cta, G, ub, ue);
                        for (int u = ub; u < ue; ++u, ++it) {
                            const int pi = dp_prob_of(ph, u);
                            const DpProb& q = ph.p[pi];
                            const int local = u - q.unit0, kb = local % q.mat.kblocks, mt = local / q.mat.kblocks;
                            const int s = it % NS;
                            if (!mbar_wait(&empty[s], ((it / NS) & 1u) ^ 1u, abort_flag)) {
                                ok = false;
                                break;
                            }
                            mbar_expect_tx(&full[s], kDpATile);
                            tma_load_2d(&P.maps[q.mat.map], &full[s], ring + (size_t)s * kDpATile, kb * (q.mat.is_i8 ? 128 : 64), mt * 128);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // =========================== MMA issuer ===========================
        if (lane == 0) {
            uint32_t it = 0, run = 0, phase_seq = 0;
            bool ok = true;
            for (int t = 0; t < P.n_tokens && ok; ++t) {
                const bool do_head = P.argmax_feed || t == P.n_tokens - 1;
                for (int l = 0; l <= P.L && ok; ++l) {
                    if (l == P.L && !do_head) break;
                    for (int phs = 0; phs < (l == P.L ? 1 : 4) && ok; ++phs) {
                        DpPhase ph;
                        dp_build_phase(P, l, l == P.L ? DP_HEAD : phs, ph);
                        int ub, ue;
                        dp_range(ph, cta, G, ub, ue);
                        ok = mbar_wait(b_ready, phase_seq & 1u, abort_flag);
                        ++phase_seq;
                        if (!ok) break;
                        tc_fence_after();
                        int prev_tile = -1;
                        for (int u = ub; u < ue; ++u, ++it) {
                            const int pi = dp_prob_of(ph, u);
                            const DpProb& q = ph.p[pi];
                            const int local = u - q.unit0, mt = local / q.mat.kblocks;
                            const int tile = q.tile0 + mt;
                            const bool first = tile != prev_tile;
                            if (first) {
                                if (prev_tile >= 0) {
                                    tc_commit(&acc_full[run & 1]);
                                    ++run;
                                }
                                ok = mbar_wait(&acc_empty[run & 1], (((run >> 1) & 1u) ^ 1u), abort_flag);
                                if (!ok) break;
                                tc_fence_after();
                                prev_tile = tile;
                            }
                            const int s = it % NS;
                            ok = mbar_wait(&full[s], (it / NS) & 1u, abort_flag);
                            if (!ok) break;
                            tc_fence_after();
                            const uint64_t adesc = tc_smem_desc(smem_u32(ring + (size_t)s * kDpATile));
                            const uint64_t bdesc = tc_smem_desc(smem_u32(btile + (size_t)dp_btile_of(ph, ub, ue, u) * kDpBTile));
                            const uint32_t d_tmem = tmem_base + (run & 1) * kDpN;
                            if (q.mat.is_i8) {
                                const uint32_t idesc = tc_idesc(true, kDpN);
#pragma unroll
                                for (int k4 = 0; k4 < 4; ++k4) tc_mma<true>(d_tmem, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc, (first && k4 == 0) ? 0u : 1u);
                            } else {
                                const uint32_t idesc = tc_idesc(false, kDpN);
#pragma unroll
                                for (int k4 = 0; k4 < 4; ++k4) tc_mma<false>(d_tmem, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc, (first && k4 == 0) ? 0u : 1u);
                            }
                            tc_commit(&empty[s]);
                        }
                        if (ok && prev_tile >= 0) {
                            tc_commit(&acc_full[run & 1]);
                            ++run;
                        }
                    }
                }
            }
        }
    } else {
        // =========================== workers ===========================
        const int wtid = threadIdx.x - 64;  // 0..127
        const int q4 = warp & 3;            // TMEM lane quarter of this warp
        unsigned bar_target = 0;
        uint32_t run = 0;
        bool ok = true;
        const int c0 = (int)(((long long)cta * C) / G), c1 = (int)(((long long)(cta + 1) * C) / G);  // this CTA's slice of the channels

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
            dp_worker_sync();
            for (int b = 0; b < NB; ++b) {
                const __half* row = P.emb + (size_t)sc_tok[b] * C;
                float s = 0.f;
                for (int k = wtid; k < C; k += kDpWorkers) s += __half2float(row[k]);
                const float mean = dp_worker_sum(s, red, wtid) / (float)C;
                float qv = 0.f;
                for (int k = wtid; k < C; k += kDpWorkers) {
                    const float d = __half2float(row[k]) - mean;
                    qv += d * d;
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
                    const int phase = l == P.L ? DP_HEAD : phs;
                    DpPhase ph;
                    dp_build_phase(P, l, phase, ph);
                    int ub, ue;
                        dp_range(ph, cta, G, ub, ue);
                    const DpLayer* Ly = l < P.L ? &P.layers[l] : nullptr;
                    const bool x_from_emb = (l == 0 && phase == DP_P1);  // x has not crossed a barrier yet: rebuild it from the embedding

                    // ---------- phase 2 (heads) runs between P1 and P3 ----------
                    if (phase == DP_P3) {
                        DpPhase p1;
                        dp_build_phase(P, l, DP_P1, p1);
                        // new time-mix shift state = LN1(x) on this CTA's slice (all readers of the old state are past barrier 1)
                        for (int i = wtid; i < NB * (c1 - c0); i += kDpWorkers) {
                            const int b = i / (c1 - c0), m = c0 + i % (c1 - c0);
                            Ly->tmix_x[(size_t)P.slot[b] * C + m] = (P.x[(size_t)b * C + m] - st_ln[b].mean) * st_ln[b].inv * Ly->ln1_w[m] + Ly->ln1_b[m];
                        }
                        const int nmid = P.wm + P.am + P.vm + P.gm;
                        for (int item = cta; item < NB * P.H; item += G) {
                            const int b = item / P.H, h = item % P.H;
                            dp_worker_sync();
                            // rank-space vectors of session b: tanh / sigmoid applied here
                            for (int j = wtid; j < nmid; j += kDpWorkers) {
                                int pi, jj;
                                if (j < P.wm) {
                                    pi = 3;
                                    jj = j;
                                } else if (j < P.wm + P.am) {
                                    pi = 4;
                                    jj = j - P.wm;
                                } else if (j < P.wm + P.am + P.vm) {
                                    pi = 6;
                                    jj = j - P.wm - P.am;
                                } else {
                                    pi = 5;
                                    jj = j - P.wm - P.am - P.vm;
                                }
                                float v = 0.f;
                                if (pi != 6 || l > 0) v = dp_finalize(P, p1, pi, jj, b, G);
                                if (pi == 3) v = tanhf(v);
                                if (pi == 5) v = 1.0f / (1.0f + expf(-v));
                                sc_mid[j] = v;
                            }
                            // r, k, v of this head
                            for (int j = wtid; j < 3 * 64; j += kDpWorkers) sc_hv[j] = dp_finalize(P, p1, j / 64, h * 64 + (j & 63), b, G);
                            dp_worker_sync();
                            const int ch = h * 64 + (wtid >> 1), half = wtid & 1;
                            // back-projections: each thread pair splits the rank dimension in two contiguous halves
                            auto dot_half = [&](const __half* W, int mid, const float* vec) {
                                const int hl = mid >> 1;
                                const __half* wrow = W + (size_t)ch * mid + half * hl;
                                const float* vv = vec + half * hl;
                                float a = 0.f;
                                if ((hl & 7) == 0) {
                                    for (int j = 0; j < hl; j += 8) {
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
                                    for (int j = 0; j < hl; ++j) a = fmaf(__half2float(wrow[j]), vv[j], a);
                                }
                                if ((mid & 1) && half == 1) a = fmaf(__half2float(W[(size_t)ch * mid + mid - 1]), vec[mid - 1], a);
                                return a + __shfl_xor_sync(0xffffffffu, a, 1);
                            };
                            const float dw = dot_half(Ly->w2, P.wm, sc_mid);
                            const float da = dot_half(Ly->a2, P.am, sc_mid + P.wm);
                            const float dg = dot_half(Ly->g2, P.gm, sc_mid + P.wm + P.am + P.vm);
                            const float wdec = expf((1.0f / (1.0f + expf(-(dw + Ly->w0[ch])))) * kDecayScale);
                            const float aa = 1.0f / (1.0f + expf(-(da + Ly->a0[ch])));
                            const float rr = sc_hv[(wtid >> 1)], kk0 = sc_hv[64 + (wtid >> 1)];
                            float vv0 = sc_hv[128 + (wtid >> 1)];
                            if (l == 0) {
                                if (half == 0) {
                                    P.vfirst[(size_t)b * C + ch] = vv0;
                                    P.state_vfirst[(size_t)P.slot[b] * C + ch] = vv0;
                                }
                            } else {
                                const float dv = dot_half(Ly->v2, P.vm, sc_mid + P.wm + P.am);
                                const float gate = 1.0f / (1.0f + expf(-(dv + Ly->v0[ch])));
                                vv0 = vv0 + gate * (P.vfirst[(size_t)b * C + ch] - vv0);
                            }
                            const float kkj = kk0 * Ly->k_k[ch];
                            const float ss = dp_worker_sum(half == 0 ? kkj * kkj : 0.f, red, wtid);
                            const float kkh = kkj * (1.0f / fmaxf(sqrtf(ss), kL2Eps));
                            const float kt = kk0 + Ly->k_a[ch] * (kk0 * aa - kk0);
                            if (half == 0) {
                                const int i = wtid >> 1;
                                sc_hv[3 * 64 + i] = wdec;
                                sc_hv[4 * 64 + i] = rr;
                                sc_hv[5 * 64 + i] = kkh;
                                sc_hv[6 * 64 + i] = kkh * (-aa);
                                sc_hv[7 * 64 + i] = kt;
                            }
                            dp_worker_sync();
                            // state row (wtid>>1), columns [32*half, 32*half+32)
                            float* srow = Ly->wkv + (((size_t)P.slot[b] * P.H + h) * 64 + (wtid >> 1)) * 64 + half * 32;
                            float S[32];
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 v4 = *reinterpret_cast<const float4*>(srow + j);
                                S[j] = v4.x;
                                S[j + 1] = v4.y;
                                S[j + 2] = v4.z;
                                S[j + 3] = v4.w;
                            }
                            const float *s_w = sc_hv + 3 * 64 + half * 32, *s_r = sc_hv + 4 * 64 + half * 32, *s_kk = sc_hv + 5 * 64 + half * 32,
                                        *s_b = sc_hv + 6 * 64 + half * 32, *s_kt = sc_hv + 7 * 64 + half * 32;
                            float sa = 0.f;
#pragma unroll
                            for (int j = 0; j < 32; ++j) sa = fmaf(S[j], s_kk[j], sa);
                            sa += __shfl_xor_sync(0xffffffffu, sa, 1);
                            float y = 0.f;
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                S[j] = fmaf(S[j], s_w[j], fmaf(sa, s_b[j], vv0 * s_kt[j]));
                                y = fmaf(S[j], s_r[j], y);
                            }
                            y += __shfl_xor_sync(0xffffffffu, y, 1);
#pragma unroll
                            for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(srow + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
                            const float mean = dp_worker_sum(half == 0 ? y : 0.f, red, wtid) / 64.0f;
                            const float d = y - mean;
                            const float var = dp_worker_sum(half == 0 ? d * d : 0.f, red, wtid) / 64.0f + kGnEps;
                            const float srk = dp_worker_sum(half == 0 ? rr * kt * Ly->r_k[ch] : 0.f, red, wtid);
                            if (half == 0) P.yg[(size_t)b * C + ch] = (d * (1.0f / sqrtf(var)) * Ly->lnx_w[ch] + Ly->lnx_b[ch] + srk * vv0) * dg;
                        }
                        ok = dp_grid_barrier(P.grid_bar, bar_target, G, abort_flag, wtid);
                        if (!ok) break;
                    }

                    // ---------- LayerNorm statistics of the phase input (full rows, every CTA) ----------
                    if (phase == DP_P1 || phase == DP_P4 || phase == DP_HEAD) {
                        for (int b = 0; b < NB; ++b) {
                            const __half* erow = P.emb + (size_t)sc_tok[b] * C;
                            const DpStats se = st_emb[b];
                            auto xval = [&](int k) {
                                return x_from_emb ? ((__half2float(erow[k]) - se.mean) * se.inv * P.ln0_w[k] + P.ln0_b[k]) : P.x[(size_t)b * C + k];
                            };
                            float s = 0.f;
                            for (int k = wtid; k < C; k += kDpWorkers) s += xval(k);
                            const float mean = dp_worker_sum(s, red, wtid) / (float)C;
                            float qv = 0.f;
                            for (int k = wtid; k < C; k += kDpWorkers) {
                                const float dd = xval(k) - mean;
                                qv += dd * dd;
                            }
                            const float inv = 1.0f / sqrtf(dp_worker_sum(qv, red, wtid) / (float)C + kLnEps);
                            if (wtid == 0) st_ln[b] = DpStats{mean, inv};
                        }
                        dp_worker_sync();
                    }
                    if (phase == DP_P5) {
                        // new channel-mix shift state = LN2(x) on this CTA's slice (readers of the old state are past barrier 4)
                        for (int i = wtid; i < NB * (c1 - c0); i += kDpWorkers) {
                            const int b = i / (c1 - c0), m = c0 + i % (c1 - c0);
                            Ly->cmix_x[(size_t)P.slot[b] * C + m] = (P.x[(size_t)b * C + m] - st_ln[b].mean) * st_ln[b].inv * Ly->ln2_w[m] + Ly->ln2_b[m];
                        }
                    }

                    // ---------- operand tiles of this CTA's units ----------
                    DpPhase p4;  // producer of h
                    if (phase == DP_P5) dp_build_phase(P, l, DP_P4, p4);
                    const float *lw = nullptr, *lb = nullptr, *shift = nullptr;
                    if (phase == DP_P1) {
                        lw = Ly->ln1_w;
                        lb = Ly->ln1_b;
                        shift = Ly->tmix_x;
                    } else if (phase == DP_P4) {
                        lw = Ly->ln2_w;
                        lb = Ly->ln2_b;
                        shift = Ly->cmix_x;
                    } else if (phase == DP_HEAD) {
                        lw = P.lno_w;
                        lb = P.lno_b;
                    }
                    auto input = [&](const DpProb& q, int b, int k) -> float {
                        switch (q.in_kind) {
                            case DP_IN_LNMIX: {
                                const float xv = x_from_emb ? ((__half2float(P.emb[(size_t)sc_tok[b] * C + k]) - st_emb[b].mean) * st_emb[b].inv * P.ln0_w[k] + P.ln0_b[k])
                                                            : P.x[(size_t)b * C + k];
                                const float cur = (xv - st_ln[b].mean) * st_ln[b].inv * lw[k] + lb[k];
                                const float prev = shift[(size_t)P.slot[b] * C + k];
                                return cur + q.mix[k] * (prev - cur);
                            }
                            case DP_IN_VEC: return P.yg[(size_t)b * C + k];
                            case DP_IN_H: {
                                const float a = fmaxf(dp_finalize(P, p4, 0, k, b, G), 0.f);
                                return a * a;
                            }
                            default: return (P.x[(size_t)b * C + k] - st_ln[b].mean) * st_ln[b].inv * lw[k] + lb[k];
                        }
                    };
                    {
                        int base = 0;
                        for (int pi = 0; pi < ph.nprob; ++pi) {
                            const DpProb& q = ph.p[pi];
                            const int lo = max(ub, q.unit0), hi = min(ue, q.unit0 + q.mat.mtiles * q.mat.kblocks);
                            if (hi <= lo) continue;
                            const int ntile = min(hi - lo, q.mat.kblocks);
                            const int kb0 = (lo - q.unit0) % q.mat.kblocks;  // K block of local tile 0 (all K blocks when ntile == kblocks)
                            const int epb = q.mat.is_i8 ? 128 : 64;          // elements per K block
                            const bool act = wtid < epb;
                            // pass 1: largest magnitude over everything this CTA feeds into this problem
                            float am[kDpMaxNB] = {0.f, 0.f, 0.f, 0.f};
                            for (int tl = 0; tl < ntile; ++tl) {
                                const int kb = ntile == q.mat.kblocks ? tl : (kb0 + tl) % q.mat.kblocks;
                                const int k = kb * epb + wtid;
                                if (act && k < q.mat.K)
                                    for (int b = 0; b < NB; ++b) am[b] = fmaxf(am[b], fabsf(input(q, b, k)));
                            }
                            int ex[kDpMaxNB];
                            for (int b = 0; b < NB; ++b) {
                                const float a = dp_worker_max(am[b], red, wtid);
                                int e = 0;
                                if (a > 0.f && a < 3.0e38f) {
                                    (void)frexpf(a, &e);
                                    if (a == ldexpf(0.5f, e)) e -= 1;
                                }
                                ex[b] = max(-100, min(100, e));
                                if (wtid == 0) sc_scale[pi * kDpMaxNB + b] = q.mat.is_i8 ? ldexpf(1.0f, ex[b] - kDpP) : ldexpf(1.0f, ex[b]);
                            }
                            // pass 2: digits (int8) or hi/lo halves (fp16) into the swizzled tiles
                            for (int tl = 0; tl < ntile; ++tl) {
                                const int kb = ntile == q.mat.kblocks ? tl : (kb0 + tl) % q.mat.kblocks;
                                const int k = kb * epb + wtid;
                                uint8_t* tile = btile + (size_t)(base + tl) * kDpBTile;
                                for (int b = 0; b < NB; ++b) {
                                    float v = (act && k < q.mat.K) ? input(q, b, k) : 0.f;
                                    long long tsum = 0;
                                    if (q.mat.is_i8) {
                                        v *= ldexpf(1.0f, kDpP - ex[b]);
                                        v = fminf(fmaxf(v, -(float)(1 << kDpP)), (float)(1 << kDpP));
                                        int tq = (v == v) ? __float2int_rn(v) : 0;
                                        tsum = tq;
                                        if (act) {
#pragma unroll
                                            for (int j = kDpDigits - 1; j > 0; --j) {
                                                const int dj = ((tq + 64) & 127) - 64;
                                                tile[dp_b_offset(b * kDpDigits + j, wtid)] = (uint8_t)(int8_t)dj;
                                                tq = (tq - dj) >> 7;
                                            }
                                            tile[dp_b_offset(b * kDpDigits, wtid)] = (uint8_t)(int8_t)tq;
                                        }
                                        // exact integer sum of this tile's fixed-point values
#pragma unroll
                                        for (int o = 16; o > 0; o >>= 1) tsum += __shfl_xor_sync(0xffffffffu, tsum, o);
                                        dp_worker_sync();
                                        if ((wtid & 31) == 0) reinterpret_cast<long long*>(red)[wtid >> 5] = tsum;
                                        dp_worker_sync();
                                        if (wtid == 0) {
                                            const long long* r4 = reinterpret_cast<const long long*>(red);
                                            sc_tsum[(size_t)(base + tl) * kDpMaxNB + b] = r4[0] + r4[1] + r4[2] + r4[3];
                                        }
                                    } else if (act) {
                                        v *= ldexpf(1.0f, -ex[b]);
                                        v = fminf(fmaxf(v, -1.0f), 1.0f);
                                        if (!(v == v)) v = 0.f;
                                        const __half hi16 = __float2half_rn(v);
                                        const __half lo16 = __float2half_rn(v - __half2float(hi16));
                                        *reinterpret_cast<__half*>(tile + dp_b_offset(b * 2, wtid * 2)) = hi16;
                                        *reinterpret_cast<__half*>(tile + dp_b_offset(b * 2 + 1, wtid * 2)) = lo16;
                                    }
                                }
                            }
                            base += ntile;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    dp_worker_sync();
                    if (wtid == 0) mbar_arrive(b_ready);

                    // ---------- drain the runs of this CTA ----------
                    {
                        const DpRegion& Rg = P.reg[ph.region];
                        int u = ub;
                        while (u < ue) {
                            const int pi = dp_prob_of(ph, u);
                            const DpProb& q = ph.p[pi];
                            const int local = u - q.unit0, kb = local % q.mat.kblocks, mt = local / q.mat.kblocks;
                            const int tile_first = u - kb;
                            const int run_end = min(ue, tile_first + q.mat.kblocks);
                            const int slot = (u == tile_first) ? 0 : (cta - tc_cta_of_unit(tile_first, ph.U, min(G, ph.U)));
                            const size_t tidx = (size_t)(q.tile0 + mt) * Rg.pmax + slot;
                            const bool got = mbar_wait(&acc_full[run & 1], (run >> 1) & 1u, abort_flag);
                            if (!__all_sync(0xffffffffu, got)) break;  // the abort flag is set; decided for all workers below
                            tc_fence_after();
                            uint32_t v[16];
                            tmem_ld16(tmem_base + ((uint32_t)(q4 * 32) << 16) + (run & 1) * kDpN, v);
                            uint32_t* dst = Rg.data + tidx * (size_t)(kDpN * 128) + q4 * 32 + lane;
#pragma unroll
                            for (int j = 0; j < 16; ++j) dst[(size_t)j * 128] = v[j];
                            if (wtid < NB) {
                                // scale of this CTA's operand for the problem, exact sum of the run's fixed-point values
                                long long ts = 0;
                                for (int uu = u; uu < run_end; ++uu) ts += sc_tsum[(size_t)dp_btile_of(ph, ub, ue, uu) * kDpMaxNB + wtid];
                                Rg.meta[tidx].xscale[wtid] = sc_scale[pi * kDpMaxNB + wtid];
                                Rg.meta[tidx].tsum[wtid] = ts;
                            }
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&acc_empty[run & 1]);
                            ++run;
                            u = run_end;
                        }
                    }
                    // every worker reaches the barrier below whether or not its warp left the loop early;
                    // dp_grid_barrier returns the shared abort state, so the decision to stop is the same for all
                    ok = dp_grid_barrier(P.grid_bar, bar_target, G, abort_flag, wtid);
                    if (!ok) break;

                    // ---------- residual stream: x += result, on disjoint slices, then a second barrier ----------
                    if (phase == DP_P3 || phase == DP_P5) {
                        for (int i = wtid; i < NB * (c1 - c0); i += kDpWorkers) {
                            const int b = i / (c1 - c0), m = c0 + i % (c1 - c0);
                            P.x[(size_t)b * C + m] += dp_finalize(P, ph, 0, m, b, G);
                        }
                        ok = dp_grid_barrier(P.grid_bar, bar_target, G, abort_flag, wtid);
                        if (!ok) break;
                    }
                    // ---------- logits, arg-max ----------
                    if (phase == DP_HEAD) {
                        const int v0 = (int)(((long long)cta * P.V) / G), v1 = (int)(((long long)(cta + 1) * P.V) / G);
                        for (int b = 0; b < NB; ++b) {
                            float bv = -1e30f;
                            int bi = 0x7fffffff;
                            for (int vv = v0 + wtid; vv < v1; vv += kDpWorkers) {
                                const float lg = dp_finalize(P, ph, 0, vv, b, G);
                                P.logits[(size_t)b * P.V + vv] = lg;
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
                            if ((wtid & 31) == 0) {
                                red[wtid >> 5] = bv;
                                reinterpret_cast<int*>(red)[4 + (wtid >> 5)] = bi;
                            }
                            dp_worker_sync();
                            if (wtid == 0) {
                                for (int w2 = 1; w2 < 4; ++w2) {
                                    const float ov = red[w2];
                                    const int oi = reinterpret_cast<int*>(red)[4 + w2];
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
        tmem_dealloc(tmem_base, 32);
    }
}

}  // namespace rsv
