// WKV-7 state update for steps with multi-token segments (prefill chunks).  Same arithmetic as wkv7_kernel
// (src/model.rs:436-471; rwkv_fuse_ka, rwkv_dplr_seq(_batch), GroupNorm and rwkv_sum_rk_rk of src/backend_cuda.rs).
// Inside a segment the recurrence is sequential in the tokens, so the time of a chunk is (tokens) x (time of one token in the
// warp that owns a state row).  The kernel therefore splits the work by role:
//   * preparation warps read the token's inputs from global memory (several tokens ahead) and build the six vectors the
//     recurrence needs (normalised kk, w, b = -kk a, k~, r, and the value v after its lerp) into a ring of token slots in
//     shared memory; they alternate tokens, so a slot has one writer;
//   * state warps (sixteen rows each; eight lanes share four rows, eight state columns of each per lane) only wait for the
//     slot, read the vectors and run the two row-times-vector products and the update: nothing but state-dependent work is
//     in their chain, and every vector element read from shared memory serves four rows;
//   * slots are handed over in groups of four tokens with mbarriers (full: one arrival per token by its writer; empty: one
//     arrival per state warp), so the state warps do not wait for one another;
//   * GroupNorm, the bonus term and the gate need y but do not feed the state: the loop leaves the raw y in the output buffer and
//     wkv7_finish_kernel applies them, one warp per (row, head) over the whole GPU.
// Every mbarrier wait is bounded; on expiry bit 16 of the status word is set and the CTA's roles stop.
#pragma once
#include "kernels.cuh"
#include "tc_linear.cuh"

namespace rsv {

constexpr int kWsStateWarps = 4;  // 16 state rows each
constexpr int kWsPrepWarps = 6;
constexpr int kWsWarps = kWsStateWarps + kWsPrepWarps;
constexpr int kWsThreads = 32 * kWsWarps;
constexpr int kWsGroup = 4;   // tokens handed over per barrier phase
constexpr int kWsDepth = 12;  // token slots in the ring
constexpr int kWsGroups = kWsDepth / kWsGroup;
static_assert(kWsDepth % kWsGroup == 0 && kWsGroup <= kWsPrepWarps, "a group's tokens are written by different preparation warps");
constexpr int kWsVecs = 6;   // kk, w, b, k~, r, v
static_assert(kWsDepth % kWsPrepWarps == 0, "a ring slot must always be written by the same preparation warp");

// The inputs of one token as a preparation warp holds them: channels `lane` and `lane + 32` of the head.  Loading does no
// arithmetic, so that the loads of a later token can be in flight while an earlier one is processed.
struct WsIn {
    float k0, k1, a0, a1, r0, r1, w0, w1, v0, v1, vg0, vg1, vf0, vf1;
};
__device__ __forceinline__ WsIn ws_load(const float* r, const float* k, const float* v, const float* vgate, const float* vfirst, const float* w,
                                        const float* a, size_t hb, int lane) {
    WsIn x;
    x.k0 = k[hb + lane];
    x.k1 = k[hb + lane + 32];
    x.a0 = a[hb + lane];
    x.a1 = a[hb + lane + 32];
    x.r0 = r[hb + lane];
    x.r1 = r[hb + lane + 32];
    x.w0 = w[hb + lane];
    x.w1 = w[hb + lane + 32];
    x.v0 = v[hb + lane];
    x.v1 = v[hb + lane + 32];
    x.vg0 = vgate ? vgate[hb + lane] : 0.f;
    x.vg1 = vgate ? vgate[hb + lane + 32] : 0.f;
    x.vf0 = vgate ? vfirst[hb + lane] : 0.f;
    x.vf1 = vgate ? vfirst[hb + lane + 32] : 0.f;
    return x;
}

// A lane's eight columns of one of the ring's vectors.
__device__ __forceinline__ void ws_vec8(float (&d)[8], const float* vec, int sub) {
    const float4 lo = *reinterpret_cast<const float4*>(vec + 4 * sub), hi = *reinterpret_cast<const float4*>(vec + 32 + 4 * sub);
    d[0] = lo.x, d[1] = lo.y, d[2] = lo.z, d[3] = lo.w;
    d[4] = hi.x, d[5] = hi.y, d[6] = hi.z, d[7] = hi.w;
}

// RPL consecutive floats (the rows of a lane) from / to 4 RPL-byte aligned memory.
template <int RPL>
__device__ __forceinline__ void ws_rows_load(float (&d)[RPL], const float* p) {
    static_assert(RPL == 2 || RPL == 4, "rows per lane");
    if constexpr (RPL == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        d[0] = t.x, d[1] = t.y, d[2] = t.z, d[3] = t.w;
    } else {
        const float2 t = *reinterpret_cast<const float2*>(p);
        d[0] = t.x, d[1] = t.y;
    }
}
template <int RPL>
__device__ __forceinline__ void ws_rows_store(float* p, const float (&d)[RPL]) {
    if constexpr (RPL == 4)
        *reinterpret_cast<float4*>(p) = make_float4(d[0], d[1], d[2], d[3]);
    else
        *reinterpret_cast<float2*>(p) = make_float2(d[0], d[1]);
}

// Grid (heads x 4 / RPL, segments): RPL = 4 state rows per lane puts a head in one CTA; RPL = 2 splits it over two CTAs (each
// prepares the vectors itself), which halves the arithmetic in a state warp's per-token chain - used when the step has few
// (head, segment) pairs, i.e. a prefill chunk of one or a few sessions.  `vgate` (layers > 0): v <- v + vgate * (vfirst - v), the lerp of src/model.rs:424-430.
template <int RPL>
__global__ void __launch_bounds__(kWsThreads, 2) wkv7_seq_kernel(const SegMeta* __restrict__ segs, const float* __restrict__ r, const float* __restrict__ k,
                                                                 const float* __restrict__ v, const float* __restrict__ vgate,
                                                                 const float* __restrict__ vfirst, const float* __restrict__ w, const float* __restrict__ a,
                                                                 const float* __restrict__ g, const float* __restrict__ k_k, const float* __restrict__ k_a,
                                                                 const float* __restrict__ r_k, const float* __restrict__ lnx_w,
                                                                 const float* __restrict__ lnx_b, float* __restrict__ state, float* __restrict__ v_first_state,
                                                                 float* yg, int H, int C, int* status) {
    constexpr int N = kHeadSize;
    __shared__ __align__(16) float ring[kWsDepth][kWsVecs][N];
    __shared__ __align__(8) uint64_t full[kWsGroups], empty[kWsGroups];
    __shared__ int s_abort;
    constexpr int kParts = 4 / RPL;  // CTAs per head
    const int h = blockIdx.x / kParts, part = blockIdx.x % kParts, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // state warps: a group of eight lanes owns four rows; lane `sub` of the group holds columns 4 sub .. 4 sub + 3 and
    // 32 + 4 sub .. 32 + 4 sub + 3 of them (a group's 16-byte reads of a vector are contiguous: no bank conflicts), so a vector
    // element read from shared memory is used for four rows.  Shared-memory bandwidth, not arithmetic, bounds this loop: with
    // one row per lane the eight warps of a head read 80 KB of vectors per token.
    const int sub = lane & 7, row0 = (part * kWsStateWarps + (warp & (kWsStateWarps - 1))) * 4 * RPL + (lane >> 3) * RPL;
    if (tid == 0) {
        for (int s = 0; s < kWsGroups; ++s) {
            mbar_init(&full[s], kWsGroup);
            mbar_init(&empty[s], kWsStateWarps);
        }
        s_abort = 0;
    }
    pdl_launch_dependents();
    const SegMeta sg = segs[blockIdx.y];  // plan data and state: written before the step's first kernel (see wkv7_kernel)
    const bool state_warp = warp < kWsStateWarps;
    float* sbase = state + (((size_t)sg.slot * H + h) * N + row0) * N + 4 * sub;
    float S[RPL][8];
    if (state_warp) {
#pragma unroll
        for (int rr = 0; rr < RPL; ++rr) {
            const float4 lo = *reinterpret_cast<const float4*>(sbase + rr * N), hi = *reinterpret_cast<const float4*>(sbase + rr * N + 32);
            S[rr][0] = lo.x, S[rr][1] = lo.y, S[rr][2] = lo.z, S[rr][3] = lo.w;
            S[rr][4] = hi.x, S[rr][5] = hi.y, S[rr][6] = hi.z, S[rr][7] = hi.w;
        }
    }
    __syncthreads();  // barriers initialised
    pdl_wait();
    r = pdl_fresh(r);
    k = pdl_fresh(k);
    v = pdl_fresh(v);
    vgate = pdl_fresh(vgate);
    vfirst = pdl_fresh(vfirst);
    w = pdl_fresh(w);
    a = pdl_fresh(a);
    g = pdl_fresh(g);
    const bool has_gate = vgate != nullptr;
    const int hc = h * N;
    const size_t hb0 = (size_t)sg.start * C + hc;
    if (!state_warp) {
        // ---- preparation: tokens p, p + P, p + 2P, ... ----
        const int p = warp - kWsStateWarps;
        const float kkc0 = k_k[hc + lane], kkc1 = k_k[hc + lane + 32], kac0 = k_a[hc + lane], kac1 = k_a[hc + lane + 32];
        const int last = sg.len - 1;
        // The warp's next token is requested before the current one is processed; a token's memory round trip is covered by
        // the number of preparation warps, not by deeper register pipelines (a rotated register waits for its load).
        WsIn c0 = ws_load(r, k, v, vgate, vfirst, w, a, hb0 + (size_t)min(p, last) * C, lane);
        // the last group is filled up with repeats of the last token, so that its barrier completes
        const int len_pad = (sg.len + kWsGroup - 1) / kWsGroup * kWsGroup;
        for (int t = p; t < len_pad; t += kWsPrepWarps) {
            const WsIn c1 = ws_load(r, k, v, vgate, vfirst, w, a, hb0 + (size_t)min(t + kWsPrepWarps, last) * C, lane);
            const int slot = t % kWsDepth, grp = slot / kWsGroup, use = t / kWsDepth;
            const float kk0 = c0.k0 * kkc0, kk1 = c0.k1 * kkc1;
            const float ss = warp_sum(kk0 * kk0 + kk1 * kk1);
            const float inv = 1.0f / fmaxf(sqrtf(ss), kL2Eps);
            const float kh0 = kk0 * inv, kh1 = kk1 * inv;
            const float v0 = has_gate ? c0.v0 + c0.vg0 * (c0.vf0 - c0.v0) : c0.v0;
            const float v1 = has_gate ? c0.v1 + c0.vg1 * (c0.vf1 - c0.v1) : c0.v1;
            if (use > 0 && !mbar_wait(&empty[grp], (uint32_t)(use - 1) & 1u, &s_abort)) {
                if (lane == 0) atomicOr(status, 16);
                break;
            }
            float(*b)[N] = ring[slot];
            b[0][lane] = kh0;
            b[0][lane + 32] = kh1;
            b[1][lane] = c0.w0;
            b[1][lane + 32] = c0.w1;
            b[2][lane] = kh0 * (-c0.a0);
            b[2][lane + 32] = kh1 * (-c0.a1);
            b[3][lane] = c0.k0 + kac0 * (c0.k0 * c0.a0 - c0.k0);
            b[3][lane + 32] = c0.k1 + kac1 * (c0.k1 * c0.a1 - c0.k1);
            b[4][lane] = c0.r0;
            b[4][lane + 32] = c0.r1;
            b[5][lane] = v0;
            b[5][lane + 32] = v1;
            __syncwarp();  // the warp's stores are ordered before lane 0's arrival (release)
            if (lane == 0) mbar_arrive(&full[grp]);
            if (v_first_state && t == last && part == 0) {
                v_first_state[(size_t)sg.slot * C + hc + lane] = v0;
                v_first_state[(size_t)sg.slot * C + hc + lane + 32] = v1;
            }
            c0 = c1;
        }
    } else {
        // ---- state rows: wait for a group of tokens, apply them, release the group ----
        // One wait and one arrival per group: a successful wait still costs its latency and keeps the compiler from moving the
        // next token's shared-memory reads above it.
        float yp[RPL] = {};  // the previous token's partial row sums of y
        bool gave_up = false;
        auto token = [&](int t, int slot) {
            const float(*sv)[N] = ring[slot];
            float vec[8];
            ws_vec8(vec, sv[0], sub);  // kk
            float vj[RPL];
            ws_rows_load<RPL>(vj, &sv[5][row0]);
            float sa[RPL];
#pragma unroll
            for (int rr = 0; rr < RPL; ++rr) {
                const float lo = fmaf(S[rr][3], vec[3], fmaf(S[rr][2], vec[2], fmaf(S[rr][1], vec[1], S[rr][0] * vec[0])));
                const float hi = fmaf(S[rr][7], vec[7], fmaf(S[rr][6], vec[6], fmaf(S[rr][5], vec[5], S[rr][4] * vec[4])));
                sa[rr] = lo + hi;
            }
            // one reduction tree for this token's sa and the previous token's y: only sa is in the recurrence, and y(t - 1)
            // would otherwise add a second three-level shuffle latency to every token
#pragma unroll
            for (int m = 1; m < 8; m <<= 1) {
#pragma unroll
                for (int rr = 0; rr < RPL; ++rr) {
                    sa[rr] += __shfl_xor_sync(0xffffffffu, sa[rr], m);
                    yp[rr] += __shfl_xor_sync(0xffffffffu, yp[rr], m);
                }
            }
            if (sub == 0 && t > 0) ws_rows_store<RPL>(&yg[hb0 + (size_t)(t - 1) * C + row0], yp);  // raw; finished by wkv7_finish_kernel
            float wv[8], bv[8], tv[8];
            ws_vec8(wv, sv[1], sub);
            ws_vec8(bv, sv[2], sub);
            ws_vec8(tv, sv[3], sub);
            ws_vec8(vec, sv[4], sub);  // r
#pragma unroll
            for (int rr = 0; rr < RPL; ++rr) {
#pragma unroll
                for (int c = 0; c < 8; ++c) S[rr][c] = fmaf(S[rr][c], wv[c], fmaf(sa[rr], bv[c], vj[rr] * tv[c]));
                const float lo = fmaf(S[rr][3], vec[3], fmaf(S[rr][2], vec[2], fmaf(S[rr][1], vec[1], S[rr][0] * vec[0])));
                const float hi = fmaf(S[rr][7], vec[7], fmaf(S[rr][6], vec[6], fmaf(S[rr][5], vec[5], S[rr][4] * vec[4])));
                yp[rr] = lo + hi;
            }
        };
        for (int t0 = 0; t0 < sg.len; t0 += kWsGroup) {
            const int slot0 = t0 % kWsDepth, grp = slot0 / kWsGroup, use = t0 / kWsDepth;
            if (!mbar_wait(&full[grp], (uint32_t)use & 1u, &s_abort)) {
                if (lane == 0) atomicOr(status, 16);
                gave_up = true;
                break;
            }
            if (t0 + kWsGroup <= sg.len) {
#pragma unroll
                for (int j = 0; j < kWsGroup; ++j) token(t0 + j, slot0 + j);
            } else {
                for (int j = 0; t0 + j < sg.len; ++j) token(t0 + j, slot0 + j);
            }
            __syncwarp();  // every lane has read the group
            if (lane == 0) mbar_arrive(&empty[grp]);
        }
        if (!gave_up) {  // the last token's y
#pragma unroll
            for (int m = 1; m < 8; m <<= 1) {
#pragma unroll
                for (int rr = 0; rr < RPL; ++rr) yp[rr] += __shfl_xor_sync(0xffffffffu, yp[rr], m);
            }
            if (sub == 0) ws_rows_store<RPL>(&yg[hb0 + (size_t)(sg.len - 1) * C + row0], yp);
        }
#pragma unroll
        for (int rr = 0; rr < RPL; ++rr) {
            *reinterpret_cast<float4*>(sbase + rr * N) = make_float4(S[rr][0], S[rr][1], S[rr][2], S[rr][3]);
            *reinterpret_cast<float4*>(sbase + rr * N + 32) = make_float4(S[rr][4], S[rr][5], S[rr][6], S[rr][7]);
        }
    }
}

// GroupNorm over a head's 64 outputs (two-pass, like the CPU path), the bonus term (r . k~ r_k) v and the gate, on the raw y that
// wkv7_seq_kernel left in `yg`: one warp per (row, head), lane l holds channels l and l + 32.  These need y but do not feed the
// state, so they are kept out of the sequential loop and spread over the whole GPU here.
constexpr int kWsFinishThreads = 256;
__global__ void __launch_bounds__(kWsFinishThreads) wkv7_finish_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                                                                       const float* __restrict__ vgate, const float* __restrict__ vfirst,
                                                                       const float* __restrict__ a, const float* __restrict__ g, const float* __restrict__ k_a,
                                                                       const float* __restrict__ r_k, const float* __restrict__ lnx_w,
                                                                       const float* __restrict__ lnx_b, float* yg, int R, int H, int C) {
    constexpr int N = kHeadSize;
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * (kWsFinishThreads / 32) + (threadIdx.x >> 5);
    pdl_launch_dependents();
    if (item >= R * H) return;
    const int row = item / H, h = item - row * H, hc = h * N;
    const float kac0 = k_a[hc + lane], kac1 = k_a[hc + lane + 32], rkc0 = r_k[hc + lane], rkc1 = r_k[hc + lane + 32];
    const float gw0 = lnx_w[hc + lane], gw1 = lnx_w[hc + lane + 32], gb0 = lnx_b[hc + lane], gb1 = lnx_b[hc + lane + 32];
    pdl_wait();
    r = pdl_fresh(r);
    k = pdl_fresh(k);
    v = pdl_fresh(v);
    vgate = pdl_fresh(vgate);
    vfirst = pdl_fresh(vfirst);
    a = pdl_fresh(a);
    g = pdl_fresh(g);
    yg = pdl_fresh(yg);
    const size_t hb = (size_t)row * C + hc;
    const float y0 = yg[hb + lane], y1 = yg[hb + lane + 32];
    const float k0 = k[hb + lane], k1 = k[hb + lane + 32], a0 = a[hb + lane], a1 = a[hb + lane + 32];
    const float r0 = r[hb + lane], r1 = r[hb + lane + 32];
    float v0 = v[hb + lane], v1 = v[hb + lane + 32];
    const float g0 = g[hb + lane], g1 = g[hb + lane + 32];
    if (vgate != nullptr) {
        v0 = v0 + vgate[hb + lane] * (vfirst[hb + lane] - v0);
        v1 = v1 + vgate[hb + lane + 32] * (vfirst[hb + lane + 32] - v1);
    }
    const float mean = warp_sum(y0 + y1) / (float)N;
    const float d0 = y0 - mean, d1 = y1 - mean;
    const float var = warp_sum(d0 * d0 + d1 * d1) / (float)N + kGnEps;
    const float inv_std = 1.0f / sqrtf(var);
    const float kt0 = k0 + kac0 * (k0 * a0 - k0), kt1 = k1 + kac1 * (k1 * a1 - k1);
    const float srk = warp_sum(r0 * kt0 * rkc0 + r1 * kt1 * rkc1);
    yg[hb + lane] = (d0 * inv_std * gw0 + gb0 + srk * v0) * g0;
    yg[hb + lane + 32] = (d1 * inv_std * gw1 + gb1 + srk * v1) * g1;
}

}  // namespace rsv
