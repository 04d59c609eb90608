// WKV-7 state update for many (session, head) pairs, one state row per lane.  Same arithmetic as wkv7_kernel
// (src/model.rs:436-471; rwkv_fuse_ka, rwkv_dplr_seq(_batch), GroupNorm and rwkv_sum_rk_rk of src/backend_cuda.rs), laid out for
// a batch whose recurrent state (32 KB of traffic per pair) dominates the step:
//   * a warp pair owns a head: lane l of warp half hf holds state row l + 32 hf, all 64 columns, in registers, so the two
//     row-times-vector products of the recurrence need no shuffles at all;
//   * everything an item needs arrives through one mbarrier, requested as soon as the previous item's copy is in registers: the 16 KB state as two TMA boxes (64 rows x 128
//     bytes, SWIZZLE_128B: a lane reads its 128-byte row segment chunk by chunk without bank conflicts), the first token's
//     eight input vectors and the head's five parameter vectors as 256-byte bulk copies.  No load of an iteration depends on
//     another load: with the memory system loaded a dependent global load costs microseconds per item;
//   * the updated rows leave through a staging tile and TMA stores;
//   * six warp pairs per CTA walk their own item streams (a head's chain of reductions and barriers is long and a thread holds
//     64 state registers, so the pairs are what hides latency: 96 KB of state reads in flight per SM); they share nothing but
//     the CTA's shared memory budget, and synchronise pairwise with named barriers (GroupNorm statistics over the 64 rows).
// Every mbarrier wait is bounded; on expiry bit 16 of the status word is set and the pair stops.
#pragma once
#include "kernels.cuh"
#include "tc_linear.cuh"

namespace rsv {

constexpr int kWrPairs = 6;
constexpr int kWrThreads = 64 * kWrPairs;
constexpr int kWrStages = 1;               // load stages per pair (plus one staging tile for the stores)
constexpr int kWrTileFloats = 64 * 32;     // one TMA box: 64 rows x 32 columns
constexpr int kWrStateBytes = 2 * kWrTileFloats * 4;
constexpr int kWrVecs = 13;                // r k v w a g vgate vfirst | k_k k_a r_k lnx_w lnx_b, 64 floats each
constexpr int kWrStageBytes = kWrStateBytes + 4096;  // state + vectors, 1 KB aligned
constexpr int kWrPairBytes = kWrStages * kWrStageBytes + kWrStateBytes;
constexpr size_t kWrSmemBytes = 1024 /*alignment*/ + (size_t)kWrPairs * kWrPairBytes + (size_t)kWrPairs * 5 * 64 * 4 + 512;

__device__ __forceinline__ void wr_pair_sync(int pair) { asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory"); }
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_load_256(void* dst, const void* src, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 256, [%2];" ::"r"(smem_u32(dst)), "l"(src), "r"(smem_u32(bar))
                 : "memory");
}

// `smap`: all layers' states as one 2-D tensor [rows = layers x slots x heads x 64][64 columns] fp32, box 32 columns x 64 rows;
// `row0`: first row of this layer.
__global__ void __launch_bounds__(kWrThreads, 1) wkv7_rows_kernel(const __grid_constant__ CUtensorMap smap, long long row0, const SegMeta* __restrict__ segs,
                                                                  int n_items, const float* __restrict__ r, const float* __restrict__ k,
                                                                  const float* __restrict__ v, const float* __restrict__ vgate,
                                                                  const float* __restrict__ vfirst, const float* __restrict__ w, const float* __restrict__ a,
                                                                  const float* __restrict__ g, const float* __restrict__ k_k, const float* __restrict__ k_a,
                                                                  const float* __restrict__ r_k, const float* __restrict__ lnx_w,
                                                                  const float* __restrict__ lnx_b, float* __restrict__ v_first_state, float* __restrict__ yg,
                                                                  int H, int C, int* status) {
    constexpr int N = kHeadSize;
    extern __shared__ __align__(1024) uint8_t wr_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)wr_raw + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, pair = warp >> 1, hf = warp & 1, rr = lane + 32 * hf;
    uint8_t* my = base + (size_t)pair * kWrPairBytes;                                   // [stage][state | vectors], then the store tile
    float* out_tile = reinterpret_cast<float*>(my + kWrStages * kWrStageBytes);
    float* svec = reinterpret_cast<float*>(base + (size_t)kWrPairs * kWrPairBytes);    // [pair][5][64]
    float* red = svec + (size_t)kWrPairs * 5 * N;                              // [pair][2 halves][2]
    uint64_t* full = reinterpret_cast<uint64_t*>(red + kWrPairs * 4);                   // [pair][stage]
    volatile int* s_abort = reinterpret_cast<volatile int*>(full + kWrPairs * kWrStages) + pair;  // one flag per warp pair
    const bool leader = hf == 0 && lane == 0;
    const int first = (int)blockIdx.x * kWrPairs + pair, stride = (int)gridDim.x * kWrPairs;
    const int my_items = n_items > first ? (n_items - 1 - first) / stride + 1 : 0;
    if (tid == 0) {
        for (int i = 0; i < kWrPairs * kWrStages; ++i) mbar_init(&full[i], 1);
        for (int i = 0; i < kWrPairs; ++i) (s_abort - pair)[i] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();  // the input vectors come from the predecessor kernels
    r = pdl_fresh(r);
    k = pdl_fresh(k);
    v = pdl_fresh(v);
    vgate = pdl_fresh(vgate);
    vfirst = pdl_fresh(vfirst);
    w = pdl_fresh(w);
    a = pdl_fresh(a);
    g = pdl_fresh(g);
    const int nvec = vgate ? kWrVecs : kWrVecs - 2;
    // segment descriptors run three items ahead in registers: the leader's copy addresses must not wait for a load of their own
    auto meta_of = [&](int n) { return n < my_items ? segs[(first + n * stride) / H] : SegMeta{0, 0, 0, 0}; };
    auto issue_load = [&](int n, const SegMeta& sg) {  // the pair's leader only
        const int st = n % kWrStages, item = first + n * stride, h = item % H;
        const int y = (int)(row0 + ((long long)sg.slot * H + h) * N);
        uint64_t* bar = &full[pair * kWrStages + st];
        uint8_t* dst = my + (size_t)st * kWrStageBytes;
        float* vdst = reinterpret_cast<float*>(dst + kWrStateBytes);
        mbar_expect_tx(bar, (uint32_t)(kWrStateBytes + nvec * 256));
        tma_load_2d(&smap, bar, dst, 0, y);
        tma_load_2d(&smap, bar, dst + kWrTileFloats * 4, 32, y);
        const size_t hb = (size_t)sg.start * C + (size_t)h * N;
        const float* in[8] = {r, k, v, w, a, g, vgate, vfirst};
        for (int i = 0; i < (vgate ? 8 : 6); ++i) bulk_load_256(vdst + i * N, in[i] + hb, bar);
        const float* pr[5] = {k_k, k_a, r_k, lnx_w, lnx_b};
        for (int i = 0; i < 5; ++i) bulk_load_256(vdst + (8 + i) * N, pr[i] + (size_t)h * N, bar);
    };
    SegMeta sg0 = meta_of(0), sg1 = meta_of(1), sg2 = meta_of(2);
    if (leader) {
        if (my_items > 0) issue_load(0, sg0);
        if (kWrStages > 1 && my_items > 1) issue_load(1, sg1);
    }
    float* sv = svec + (size_t)pair * 5 * N;  // both warps of the pair write the same five vectors (identical values) and read them back
    float* pred = red + pair * 4;
    for (int n = 0; n < my_items; ++n) {
        const int item = first + n * stride, h = item % H, st = n % kWrStages;
        const SegMeta sg = sg0;
        const SegMeta sg3 = meta_of(n + 3);
        const int hc = h * N;
        if (!mbar_wait(&full[pair * kWrStages + st], (uint32_t)(n / kWrStages) & 1u, s_abort)) atomicOr(status, 16);
        wr_pair_sync(pair);
        if (*s_abort) break;  // same decision for both warps of the pair: only they set the pair's flag, and only before this barrier
        const float* tl = reinterpret_cast<const float*>(my + (size_t)st * kWrStageBytes) + rr * 32;
        const float* vs = reinterpret_cast<const float*>(my + (size_t)st * kWrStageBytes + kWrStateBytes);
        float S[N];
#pragma unroll
        for (int X = 0; X < 2; ++X)
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float4 t4 = *reinterpret_cast<const float4*>(tl + X * kWrTileFloats + ((c ^ (rr & 7)) << 2));
                S[X * 32 + c * 4] = t4.x;
                S[X * 32 + c * 4 + 1] = t4.y;
                S[X * 32 + c * 4 + 2] = t4.z;
                S[X * 32 + c * 4 + 3] = t4.w;
            }
        WkvIn cur;
        cur.r0 = vs[0 * N + lane];
        cur.r1 = vs[0 * N + lane + 32];
        cur.k0 = vs[1 * N + lane];
        cur.k1 = vs[1 * N + lane + 32];
        cur.v = vs[2 * N + rr];
        cur.w0 = vs[3 * N + lane];
        cur.w1 = vs[3 * N + lane + 32];
        cur.a0 = vs[4 * N + lane];
        cur.a1 = vs[4 * N + lane + 32];
        cur.g = vs[5 * N + rr];
        cur.vg = vgate ? vs[6 * N + rr] : 0.f;
        cur.vf = vgate ? vs[7 * N + rr] : 0.f;
        const float kkc0 = vs[8 * N + lane], kkc1 = vs[8 * N + lane + 32], kac0 = vs[9 * N + lane], kac1 = vs[9 * N + lane + 32];
        const float rkc0 = vs[10 * N + lane], rkc1 = vs[10 * N + lane + 32], gw = vs[11 * N + rr], gb = vs[12 * N + rr];
        // the stage is free once both warps hold its contents: the data of item n + 2 may land in it
        wr_pair_sync(pair);
        if (leader && n + kWrStages < my_items) issue_load(n + kWrStages, kWrStages == 1 ? sg1 : sg2);
        for (int t = 0; t < sg.len; ++t) {
            const size_t hb = (size_t)(sg.start + t) * C + hc;
            WkvIn nx = cur;
            if (t + 1 < sg.len) nx = wkv_load_inputs(r, k, v, vgate, vfirst, w, a, g, hb + C, lane, rr);  // the next token's inputs, one token ahead
            const float vj = wkv_value(cur, vgate != nullptr);
            const float kk0 = cur.k0 * kkc0, kk1 = cur.k1 * kkc1;
            const float ss = warp_sum(kk0 * kk0 + kk1 * kk1);
            const float inv = 1.0f / fmaxf(sqrtf(ss), kL2Eps);
            const float kh0 = kk0 * inv, kh1 = kk1 * inv;
            const float kt0 = cur.k0 + kac0 * (cur.k0 * cur.a0 - cur.k0), kt1 = cur.k1 + kac1 * (cur.k1 * cur.a1 - cur.k1);
            const float srk = warp_sum(cur.r0 * kt0 * rkc0 + cur.r1 * kt1 * rkc1);
            wr_pair_sync(pair);  // the previous token's readers (both warps) are done with sv
            sv[0 * N + lane] = kh0;
            sv[0 * N + lane + 32] = kh1;
            sv[1 * N + lane] = cur.w0;
            sv[1 * N + lane + 32] = cur.w1;
            sv[2 * N + lane] = kh0 * (-cur.a0);
            sv[2 * N + lane + 32] = kh1 * (-cur.a1);
            sv[3 * N + lane] = kt0;
            sv[3 * N + lane + 32] = kt1;
            sv[4 * N + lane] = cur.r0;
            sv[4 * N + lane + 32] = cur.r1;
            wr_pair_sync(pair);
            float sa0 = 0.f, sa1 = 0.f, sa2 = 0.f, sa3 = 0.f;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const float4 kk4 = *reinterpret_cast<const float4*>(sv + 4 * c);  // the same address for every lane: a broadcast
                sa0 = fmaf(S[4 * c], kk4.x, sa0);
                sa1 = fmaf(S[4 * c + 1], kk4.y, sa1);
                sa2 = fmaf(S[4 * c + 2], kk4.z, sa2);
                sa3 = fmaf(S[4 * c + 3], kk4.w, sa3);
            }
            const float sa = (sa0 + sa1) + (sa2 + sa3);
            float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const float4 w4 = *reinterpret_cast<const float4*>(sv + 1 * N + 4 * c);
                const float4 b4 = *reinterpret_cast<const float4*>(sv + 2 * N + 4 * c);
                const float4 t4 = *reinterpret_cast<const float4*>(sv + 3 * N + 4 * c);
                const float4 r4 = *reinterpret_cast<const float4*>(sv + 4 * N + 4 * c);
                S[4 * c] = fmaf(S[4 * c], w4.x, fmaf(sa, b4.x, vj * t4.x));
                S[4 * c + 1] = fmaf(S[4 * c + 1], w4.y, fmaf(sa, b4.y, vj * t4.y));
                S[4 * c + 2] = fmaf(S[4 * c + 2], w4.z, fmaf(sa, b4.z, vj * t4.z));
                S[4 * c + 3] = fmaf(S[4 * c + 3], w4.w, fmaf(sa, b4.w, vj * t4.w));
                y0 = fmaf(S[4 * c], r4.x, y0);
                y1 = fmaf(S[4 * c + 1], r4.y, y1);
                y2 = fmaf(S[4 * c + 2], r4.z, y2);
                y3 = fmaf(S[4 * c + 3], r4.w, y3);
            }
            const float y = (y0 + y1) + (y2 + y3);
            // GroupNorm over the head's 64 outputs (two-pass, like the CPU path): one value per lane, two warps
            const float ys = warp_sum(y);
            if (lane == 0) pred[hf * 2] = ys;
            wr_pair_sync(pair);
            const float mean = (pred[0] + pred[2]) / (float)N;
            const float d = y - mean;
            const float qs = warp_sum(d * d);
            if (lane == 0) pred[hf * 2 + 1] = qs;
            wr_pair_sync(pair);
            const float var = (pred[1] + pred[3]) / (float)N + kGnEps;
            const float inv_std = 1.0f / sqrtf(var);
            yg[hb + rr] = (d * inv_std * gw + gb + srk * vj) * cur.g;
            if (v_first_state && t == sg.len - 1) v_first_state[(size_t)sg.slot * C + hc + rr] = vj;
            cur = nx;
        }
        // updated rows -> staging tile (free once the previous item's stores have read it) -> TMA stores
        if (leader) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        wr_pair_sync(pair);
        {
            float* ot = out_tile + rr * 32;
#pragma unroll
            for (int X = 0; X < 2; ++X)
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<float4*>(ot + X * kWrTileFloats + ((c ^ (rr & 7)) << 2)) =
                        make_float4(S[X * 32 + c * 4], S[X * 32 + c * 4 + 1], S[X * 32 + c * 4 + 2], S[X * 32 + c * 4 + 3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the rows are read by the TMA stores below
        wr_pair_sync(pair);
        if (leader) {
            const int y = (int)(row0 + ((long long)sg.slot * H + h) * N);
            tma_store_2d(&smap, out_tile, 0, y);
            tma_store_2d(&smap, out_tile + kWrTileFloats, 32, y);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        sg0 = sg1;
        sg1 = sg2;
        sg2 = sg3;
    }
    if (leader) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every state has left shared memory before the CTA ends
}

}  // namespace rsv
