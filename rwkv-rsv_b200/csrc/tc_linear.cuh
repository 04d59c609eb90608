// Weight-streaming linear layers on the 5th-generation tensor cores (sm_100a): TMA -> shared memory ->
// tcgen05.mma -> TMEM.  Replaces, for many rows at once, the reference's dequant-to-scratch + cuBLAS GEMM +
// separate epilogue pass (rwkv_dequant_int8, cublasGemmEx, rwkv_gemm_epilogue; src/backend_cuda.rs:4195-4227,
// 1254-1368, 4613-4633) and its register-tiled batched GEMVs (gemv_variant_mb, gemv_int8_rkv_stage1_batch;
// :3381-3554, :1665-1910).
//
// Arithmetic.  The weights are never converted: the u8 codes q of the int8 container are the A operand of
// `tcgen05.mma.kind::i8` exactly as they sit in HBM (row-major [M,K], K contiguous).  An activation row x is
// turned once into D signed base-128 digits of a fixed-point value t = rint(x / e * 2^P), e = 2^ceil(log2 max|x|),
// P = 7D-1, which form D columns of the B operand (int8, [N,K], K contiguous).  The tensor core returns the exact
// int32 sums I_j = sum_k q_k d_jk; Q = sum_j 128^(D-1-j) I_j = sum_k q_k t_k exactly (int64), and with the per-row
// (scale s_m, zero z_m) of the container  y = e 2^-P (s_m Q + z_m T),  T = sum_k t_k, which is
// sum_k (s_m q_k + z_m) x_k up to the 2^-P fixed-point step of x — no accumulation rounding at all, and any
// split of K across CTAs sums exactly, so results do not depend on the schedule.  This needs one (scale, zero)
// per output row; checkpoints whose groups of 128 differ within a row take the SIMT kernel instead.
// fp16 weights use `kind::f16` with x/e split into hi + lo halves (two B columns), fp32 accumulation in TMEM.
//
// Work decomposition.  A unit is one (128-row M tile, N tile, 128-byte K block) = 16 KB of weights.  Units are
// ordered problem -> M tile -> N tile -> K block and cut into equal contiguous ranges, one per CTA (persistent,
// one CTA per SM), so every SM streams the same number of bytes whatever the matrix shape.  Each maximal run of
// units inside one tile accumulates in TMEM.  A run that covers its tile's whole K range is scaled and stored by the
// fused epilogue directly.  A tile that a CTA boundary cuts is written as int32/fp32 partials [slot][n][m]; every
// epilogue warp owns a fixed (lane quarter, column chunk class) sub-block of a tile, counts its arrival on that
// sub-block with one atomic, and the warp that arrives last adds the sub-block's partials in slot order (exact for
// int32, fixed order for fp32) and runs the epilogue - no second kernel and no barrier inside the CTA.
//
// Roles per CTA (576 threads): warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM owner), warps 2-17 = epilogue
// (four warps per TMEM lane quarter, interleaved 16-column chunks).
// Every wait on an mbarrier is bounded; on expiry the kernel raises bit 1 of the status word and drains.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace rsv {

constexpr int kTcEpiWarps = 16;
constexpr int kTcThreads = 64 + 32 * kTcEpiWarps;  // warp 0 TMA, warp 1 MMA, then the epilogue warps
constexpr int kTcTileM = 128;
constexpr int kTcKBlockBytes = 128;
constexpr int kTcMaxProblems = 8;
constexpr uint32_t kTcSpinLimit = 1u << 26;  // ~ seconds; far beyond any legitimate wait

struct TcProb {
    int M;        // output rows (weights rows)
    int kblocks;  // K in 128-byte blocks
    int ncols;    // valid B columns (= R * D)
    int n_tiles;  // ceil(ncols / nt)
    int unit0;    // first unit of this problem
    int tile0;    // first (M tile, N tile) index of this problem in the partial buffer
    int R, D;     // activation rows; B columns per row (int8: digits, fp16: 2 = hi/lo)
    // epilogue
    const float* wscale;    // int8: [M] per-row scale and zero of the container
    const float* wzero;
    const float* xscale;    // [R]
    const long long* tsum;  // int8: [R]
    float* y;
    float* y2;
    const float* bias;
    const float* aux;
    int ldy, ldaux, epi, pad;
};
constexpr int kTcMaxSplit = 320;  // a CTA boundary can cut at most one tile: < number of CTAs
struct alignas(64) TcLaunch {
    CUtensorMap amap[kTcMaxProblems];
    CUtensorMap bmap[kTcMaxProblems];
    TcProb p[kTcMaxProblems];
    int nprob, total_units, nt, is_i8, pmax, nstages, grid, nsplit;
    int snap;  // 1: CTA c owns the units [split_unit[c], split_unit[c + 1]), whole tiles only (no tile is cut; nsplit = 0)
    void* partials;  // [cut tile][pmax][nt][128] int32 or fp32
    int* tile_cnt;   // [cut tile][epilogue warp] arrival counters, zero between launches
    int* status;
    int split_unit[kTcMaxSplit];  // first unit of every tile that is cut by a CTA boundary (snap: the CTAs' first units)
};

// ---- PTX wrappers -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and leaves `*abort_flag` set) when the limit is hit or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kTcSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// The same for warps that expect to wait long (epilogue / worker warps waiting for an accumulator): the try_wait carries a
// suspend-time hint, so the warp is parked by the hardware instead of re-issuing the instruction back to back and competing
// with the single MMA-issuing thread of its scheduler for issue slots.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_parked(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < (kTcSpinLimit >> 6); ++i) {
        if (mbar_try_wait_parked(bar, parity, 20000u)) return true;
        if ((i & 15u) == 15u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, uint64_t* bar, void* dst, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
                 "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
                 : "memory");
}
// Release / acquire fence at device scope (lighter than the sequentially consistent fence of __threadfence()).  Used as
// "stores; __syncwarp(); lane 0: fence, atomic" on the producing side and "lane 0: atomic, fence; __syncwarp(); loads that
// bypass L1" on the consuming side.
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
template <bool I8>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (I8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
// The same two instructions for a warp that runs its issue loop convergently: every lane computes the (identical) operands,
// one elected lane issues.  Measured on this part with 64 back-to-back 128 x 16 x 32-byte MMAs: 38 cycles per MMA this way,
// 56 from a single active lane with straight-line code, about 150 from a single lane inside a loop with integer divisions -
// with one lane active the compiler cannot keep descriptors in uniform registers.
template <bool I8>
__device__ __forceinline__ void tc_mma_elect(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (I8) {
        asm volatile(
            "{\n\t.reg .pred p, q;\n\telect.sync _|q, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "@q tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p, q;\n\telect.sync _|q, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
__device__ __forceinline__ void tc_commit_elect(uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
          "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, stored with the 128-byte swizzle
// the TMA applies: 8-row groups are 1024 bytes apart (SBO), layout type 2, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address, 16-byte units
    d |= (uint64_t)1 << 16;                    // leading byte offset (unused with swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                    // version
    d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D format (1 = f32, 2 = s32) bits [4,6); A format [7,10); B format [10,13);
// A/B K-major (bits 15,16 = 0); N>>3 at [17,23); M>>4 at [24,29).
__device__ __forceinline__ uint32_t tc_idesc(bool i8, int n) {
    uint32_t d = i8 ? ((2u << 4) | (0u << 7) | (1u << 10)) : ((1u << 4) | (0u << 7) | (0u << 10));  // i8: A u8, B s8; f16: A,B f16
    d |= (uint32_t)(n >> 3) << 17;
    d |= (uint32_t)(kTcTileM >> 4) << 24;
    return d;
}

struct TcUnit {
    int p, mt, nt, kb, tile;  // problem, M tile, N tile, K block, global tile index
};
__device__ __forceinline__ TcUnit tc_decode(const TcLaunch& L, int u) {
    int p = 0;
    while (p + 1 < L.nprob && u >= L.p[p + 1].unit0) ++p;
    const TcProb& P = L.p[p];
    const int local = u - P.unit0;
    TcUnit r;
    r.p = p;
    r.kb = local % P.kblocks;
    const int t = local / P.kblocks;
    r.nt = t % P.n_tiles;
    r.mt = t / P.n_tiles;
    r.tile = P.tile0 + t;
    return r;
}
// Walks consecutive units without divisions (the decode above costs two integer divisions per unit).
struct TcWalk {
    int p, mt, nt, kb, kblocks, n_tiles, prob_end;
    __device__ __forceinline__ void start(const TcLaunch& L, int u) {
        const TcUnit un = tc_decode(L, u);
        p = un.p;
        mt = un.mt;
        nt = un.nt;
        kb = un.kb;
        kblocks = L.p[p].kblocks;
        n_tiles = L.p[p].n_tiles;
        prob_end = p + 1 < L.nprob ? L.p[p + 1].unit0 : L.total_units;
    }
    // moves from unit u to u + 1
    __device__ __forceinline__ void next(const TcLaunch& L, int u) {
        if (++kb < kblocks) return;
        kb = 0;
        if (u + 1 == prob_end && p + 1 < L.nprob) {
            ++p;
            mt = nt = 0;
            kblocks = L.p[p].kblocks;
            n_tiles = L.p[p].n_tiles;
            prob_end = p + 1 < L.nprob ? L.p[p + 1].unit0 : L.total_units;
        } else if (++nt == n_tiles) {
            nt = 0;
            ++mt;
        }
    }
};
// CTA c owns units [c*U/G, (c+1)*U/G).  Partial slot of a run = how many CTA boundaries lie inside the tile before it.
__host__ __device__ __forceinline__ int tc_cta_begin(int c, int U, int G) { return (int)(((long long)c * U) / G); }
__host__ __device__ __forceinline__ int tc_cta_of_unit(int u, int U, int G) { return (int)((((long long)u + 1) * G - 1) / U); }

// Fused epilogue for NR activation rows (r0 .. r0+NR-1) of one output m.  Loads that the epilogue needs (the
// old y for += and v-lerp, aux) are issued together before any of them is used, so a thread keeps NR (or 2 NR)
// independent requests in flight instead of one.
__device__ __forceinline__ bool tc_epi_reads_y(int epi) { return epi == EPI_ADD || epi == EPI_VLERP; }
template <int NR>
__device__ __forceinline__ void tc_epilogue_rows(const TcProb& P, int r0, int m, float bias, const float (&acc)[NR]) {
    float yold[NR], aux[NR];
    const bool ry = tc_epi_reads_y(P.epi), ra = P.epi == EPI_VLERP;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        yold[i] = 0.f;
        aux[i] = 0.f;
        if (r0 + i < P.R) {
            if (ry) yold[i] = P.y[(size_t)(r0 + i) * P.ldy + m];
            if (ra) aux[i] = P.aux[(size_t)(r0 + i) * P.ldaux + m];
        }
    }
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        if (r0 + i >= P.R) continue;
        const float a = acc[i];
        float out;
        switch (P.epi) {
            case EPI_ADD: out = yold[i] + a; break;
            case EPI_RELU2: {
                const float t = fmaxf(a, 0.f);
                out = t * t;
                break;
            }
            case EPI_TANH: out = tanhf(a); break;
            case EPI_SIGMOID: out = 1.0f / (1.0f + expf(-a)); break;
            case EPI_DECAY: out = expf((1.0f / (1.0f + expf(-(a + bias)))) * kDecayScale); break;
            case EPI_SIGMOID_BIAS: out = 1.0f / (1.0f + expf(-(a + bias))); break;
            case EPI_VLERP: {
                const float gate = 1.0f / (1.0f + expf(-(a + bias)));
                out = yold[i] + gate * (aux[i] - yold[i]);
                break;
            }
            default: out = a; break;  // EPI_STORE
        }
        P.y[(size_t)(r0 + i) * P.ldy + m] = out;
        if (P.epi == EPI_STORE && P.y2) P.y2[(size_t)(r0 + i) * P.ldy + m] = out;
    }
}
// 16 accumulator columns -> outputs.  int8: 4 activation rows x 4 digits; fp16: 8 rows x (hi, lo).
template <bool I8>
__device__ __forceinline__ void tc_finish16(const TcProb& P, int n0, int m, float ws, float wz, float bias, const long long (&Q)[4],
                                            const float (&fsum)[8]) {
    if constexpr (I8) {
        float acc[4];
        const int r0 = n0 >> 2;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = min(r0 + i, P.R - 1);
            acc[i] = (float)((double)P.xscale[r] * ((double)ws * (double)Q[i] + (double)wz * (double)P.tsum[r]));
        }
        tc_epilogue_rows<4>(P, r0, m, bias, acc);
    } else {
        float acc[8];
        const int r0 = n0 >> 1;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = P.xscale[min(r0 + i, P.R - 1)] * fsum[i];
        tc_epilogue_rows<8>(P, r0, m, bias, acc);
    }
}

template <bool I8>
__global__ void __launch_bounds__(kTcThreads, 1) tc_linear_kernel(const __grid_constant__ TcLaunch L) {
    extern __shared__ __align__(1024) uint8_t tc_smem_raw[];
    // carve: stages (1024-aligned), then barriers
    uint8_t* smem = (uint8_t*)(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    const int NT = L.nt, NS = L.nstages;
    const uint32_t a_bytes = kTcTileM * kTcKBlockBytes, b_bytes = (uint32_t)NT * kTcKBlockBytes, stage_bytes = a_bytes + b_bytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)NS * stage_bytes);
    uint64_t* empty = full + NS;
    uint64_t* acc_full = empty + NS;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x, U = L.total_units;
    const int u_begin = L.snap ? L.split_unit[blockIdx.x] : tc_cta_begin(blockIdx.x, U, G);
    const int u_end = L.snap ? L.split_unit[blockIdx.x + 1] : tc_cta_begin(blockIdx.x + 1, U, G);
    const uint32_t tmem_cols = (2 * NT <= 32) ? 32u : (uint32_t)(2 * NT);  // NT is a power of two >= 16

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], kTcEpiWarps);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        // The weight tiles of the first ring pass do not depend on the predecessor kernel: they are requested before the
        // dependency wait, so HBM streams while the predecessor (operand preparation) is still running.  The activation tiles
        // follow after the wait, on the same barrier.
        if (lane == 0 && u_begin < u_end) {
            const int npre = min(NS, u_end - u_begin);
            TcWalk w;
            w.start(L, u_begin);
            for (int j = 0; j < npre; ++j) {
                uint8_t* a_dst = smem + (size_t)j * stage_bytes;
                mbar_expect_tx(&full[j], stage_bytes);
                tma_load_2d(&L.amap[w.p], &full[j], a_dst, w.kb * (I8 ? 128 : 64), w.mt * kTcTileM);
                w.next(L, u_begin + j);
            }
            pdl_wait();
            w.start(L, u_begin);
            for (int j = 0; j < npre; ++j) {
                uint8_t* b_dst = smem + (size_t)j * stage_bytes + a_bytes;
                tma_load_2d(&L.bmap[w.p], &full[j], b_dst, w.kb * (I8 ? 128 : 64), w.nt * NT);
                w.next(L, u_begin + j);
            }
            // w now stands on unit u_begin + npre
            int s = npre == NS ? 0 : npre;
            uint32_t par = npre == NS ? 0u : 1u;  // parity to wait for on empty[s]: a fresh barrier passes a wait on parity 1
            for (int u = u_begin + npre; u < u_end; ++u) {
                if (!mbar_wait(&empty[s], par, abort_flag)) break;
                uint8_t* a_dst = smem + (size_t)s * stage_bytes;
                uint8_t* b_dst = a_dst + a_bytes;
                mbar_expect_tx(&full[s], stage_bytes);
                const int kelem = w.kb * (I8 ? 128 : 64);
                tma_load_2d(&L.amap[w.p], &full[s], a_dst, kelem, w.mt * kTcTileM);
                tma_load_2d(&L.bmap[w.p], &full[s], b_dst, kelem, w.nt * NT);
                w.next(L, u);
                if (++s == NS) {
                    s = 0;
                    par ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // The warp runs this loop convergently; one elected lane issues (see tc_mma_elect).
        if (u_begin < u_end) {
            const uint32_t idesc = tc_idesc(I8, NT);
            const uint32_t smem_addr = smem_u32(smem);
            uint32_t run = 0, s = 0, par = 0;
            bool ok = true, started = false;
            TcWalk w;
            w.start(L, u_begin);
            for (int u = u_begin; u < u_end; ++u) {
                const bool first = w.kb == 0 || u == u_begin;
                if (first) {
                    if (started) {
                        tc_commit_elect(&acc_full[run & 1]);  // previous run complete -> epilogue
                        ++run;
                    }
                    // accumulator buffer (run & 1) must have been drained (its use number is run >> 1)
                    ok = __all_sync(0xffffffffu, mbar_wait(&acc_empty[run & 1], (((run >> 1) & 1u) ^ 1u), abort_flag));
                    if (!ok) break;
                    tc_fence_after();
                    started = true;
                }
                ok = __all_sync(0xffffffffu, mbar_wait(&full[s], par, abort_flag));
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_addr + s * stage_bytes;
                const uint64_t adesc = tc_smem_desc(a_addr), bdesc = tc_smem_desc(a_addr + a_bytes);
                const uint32_t d_tmem = tmem_base + (run & 1) * NT;
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4)  // 4 x 32 bytes of K per 128-byte block; +2 = 32 bytes in 16-byte units
                    tc_mma_elect<I8>(d_tmem, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc, (first && k4 == 0) ? 0u : 1u);
                tc_commit_elect(&empty[s]);  // stage may be refilled once these MMAs have read it
                w.next(L, u);
                if (++s == (uint32_t)NS) {
                    s = 0;
                    par ^= 1u;
                }
            }
            if (ok && started) tc_commit_elect(&acc_full[run & 1]);
        }
    } else {
        // ---------------- epilogue: TMEM -> outputs, or -> partial buffer for tiles cut by a CTA boundary ----------------
        pdl_wait();  // scales, sums, outputs and partial buffers are shared with the predecessor
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        const int ew = warp - 2, cidx = ew >> 2;  // which of the warps of this lane quarter
        constexpr int kChunkStep = 16 * (kTcEpiWarps / 4);
        uint32_t run = 0;
        int u = u_begin;
        while (u < u_end) {
            const TcUnit un = tc_decode(L, u);
            const TcProb& P = L.p[un.p];
            // the run = units of this tile inside [u_begin, u_end)
            const int tile_first = u - un.kb;                       // unit index of the tile's K block 0
            const int run_end = min(u_end, tile_first + P.kblocks);  // exclusive
            const int slot = (u == tile_first) ? 0 : (blockIdx.x - tc_cta_of_unit(tile_first, U, G));
            const bool got = mbar_wait_parked(&acc_full[run & 1], (run >> 1) & 1u, abort_flag);
            if (!__all_sync(0xffffffffu, got)) break;
            tc_fence_after();
            const int ncols = min(NT, P.ncols - un.nt * NT);
            const int row = q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (run & 1) * NT;
            const bool whole = (u == tile_first) && (run_end == tile_first + P.kblocks);
            const int m = un.mt * kTcTileM + row;
            const bool mok = m < P.M;
            // 16 accumulator columns of output row m, complete in K -> scale, epilogue, store
            auto finish_chunk = [&](int c0, const uint32_t(&v)[16], float ws, float wz, float bias) {
                long long Q[4];
                float fs[8];
                if (I8) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        long long t = (int)v[4 * i];
                        t = t * 128 + (int)v[4 * i + 1];
                        t = t * 128 + (int)v[4 * i + 2];
                        Q[i] = t * 128 + (int)v[4 * i + 3];
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) fs[i] = __uint_as_float(v[2 * i]) + __uint_as_float(v[2 * i + 1]);
                }
                tc_finish16<I8>(P, un.nt * NT + c0, m, ws, wz, bias, Q, fs);
            };
            float ws = 0.f, wz = 0.f, bias = 0.f;
            if (mok) {
                if (I8) {
                    ws = P.wscale[m];
                    wz = P.wzero[m];
                }
                if (P.bias) bias = P.bias[m];
            }
            if (whole) {
                for (int c0 = cidx * 16; c0 < ncols; c0 += kChunkStep) {
                    uint32_t v[16];
                    tmem_ld16(taddr + c0, v);
                    if (mok) finish_chunk(c0, v, ws, wz, bias);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[run & 1]);
            } else {
                int lo = 0, hi = L.nsplit - 1;  // ordinal of this tile among the cut tiles (sorted by first unit)
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (L.split_unit[mid] < tile_first) lo = mid + 1; else hi = mid;
                }
                const size_t slot_stride = (size_t)NT * kTcTileM;
                uint32_t* tile_base = reinterpret_cast<uint32_t*>(L.partials) + (size_t)lo * L.pmax * slot_stride;
                // partial layout of a slot: uint4 index (chunk * 4 + j4) * 128 + row holds columns 16 chunk + 4 j4 .. + 3 of that row
                uint4* dst = reinterpret_cast<uint4*>(tile_base + (size_t)slot * slot_stride);
                for (int c0 = cidx * 16; c0 < ncols; c0 += kChunkStep) {
                    uint32_t v[16];
                    tmem_ld16(taddr + c0, v);
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) dst[(size_t)((c0 >> 4) * 4 + j4) * kTcTileM + row] = make_uint4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
                }
                tc_fence_before();
                __syncwarp();
                int old = 0;
                if (lane == 0) {
                    mbar_arrive(&acc_empty[run & 1]);  // the accumulator may be reused while the tile is finished
                    fence_acq_rel_gpu();               // the warp's partials are visible device-wide before the arrival is counted
                    old = atomicAdd(&L.tile_cnt[lo * kTcEpiWarps + ew], 1);
                    fence_acq_rel_gpu();
                }
                old = __shfl_sync(0xffffffffu, old, 0);
                const int nslots = tc_cta_of_unit(tile_first + P.kblocks - 1, U, G) - tc_cta_of_unit(tile_first, U, G) + 1;
                if (old == nslots - 1) {
                    // last arrival on this sub-block: every slot is complete
                    if (lane == 0) L.tile_cnt[lo * kTcEpiWarps + ew] = 0;  // ready for the next launch
                    auto accumulate = [&](uint32_t(&v)[16], const uint4(&t)[4]) {
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4) {
                            const uint32_t e[4] = {t[j4].x, t[j4].y, t[j4].z, t[j4].w};
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                v[4 * j4 + i] = I8 ? (uint32_t)((int)v[4 * j4 + i] + (int)e[i]) : __float_as_uint(__uint_as_float(v[4 * j4 + i]) + __uint_as_float(e[i]));
                        }
                    };
                    for (int c0 = cidx * 16; c0 < ncols; c0 += kChunkStep) {
                        uint32_t v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0u;
                        const uint4* src = reinterpret_cast<const uint4*>(tile_base) + (size_t)((c0 >> 4) * 4) * kTcTileM + row;
                        for (int sl = 0; sl < nslots; sl += 2) {  // two slots' loads in flight; added in slot order
                            const bool two = sl + 1 < nslots;
                            uint4 ta[4], tb[4];
#pragma unroll
                            for (int j4 = 0; j4 < 4; ++j4) ta[j4] = __ldcg(src + (size_t)sl * (slot_stride / 4) + (size_t)j4 * kTcTileM);
#pragma unroll
                            for (int j4 = 0; j4 < 4; ++j4)
                                tb[j4] = two ? __ldcg(src + (size_t)(sl + 1) * (slot_stride / 4) + (size_t)j4 * kTcTileM) : make_uint4(0u, 0u, 0u, 0u);
                            accumulate(v, ta);
                            if (two) accumulate(v, tb);
                        }
                        if (mok) finish_chunk(c0, v, ws, wz, bias);
                    }
                }
            }
            ++run;
            u = run_end;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(L.status, 2);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

// ------------------------------------------------------------------------------------------------
// Operand preparation: one CTA per activation row.
//   int8 path : t = rint(x / e * 2^P); D balanced base-128 digits -> B[(r*D + j), k] (s8); xscale[r] = e*2^-P;
//               tsum[r] = sum_k t_k
//   fp16 path : hi = fp16(x/e), lo = fp16(x/e - hi) -> B[2r, k], B[2r+1, k]; xscale[r] = e
// ------------------------------------------------------------------------------------------------
constexpr int kPrepThreads = 256;       // block size when there are enough rows to fill the GPU
constexpr int kPrepThreadsWide = 1024;  // few rows: one large block per row keeps the row's latency chain short
constexpr int kPrepCache = 10;          // elements per thread kept in registers between the two passes
struct TcPrepRegion {
    const float* x;
    void* B;
    float* xscale;
    long long* tsum;
    int ldx, K, Kpad, is_i8;
};
constexpr int kTcMaxRegions = 12;  // activation operands prepared by one launch (int8 and fp16 groups together)
struct TcPrepLaunch {
    TcPrepRegion r[kTcMaxRegions];
};
// smallest ex with 2^ex >= amax (0 for an all-zero or non-finite row; non-finite input is clamped by the callers)
__device__ __forceinline__ int tc_scale_exp(float amax) {
    int ex = 0;
    if (amax > 0.f && amax < 3.0e38f) {
        (void)frexpf(amax, &ex);                // amax = f * 2^ex, f in [0.5, 1)
        if (amax == ldexpf(0.5f, ex)) ex -= 1;   // exactly a power of two
    }
    return max(-100, min(100, ex));
}
__device__ __forceinline__ float tc_block_max(float amax, float* redf) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) redf[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = redf[0];
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) amax = fmaxf(amax, redf[i]);
    return amax;
}
// The first kPrepCache elements of a thread stay in registers (loaded with clamped indices so that all loads are in flight
// together); longer rows re-read the rest.
__device__ __forceinline__ float tc_prep_load(const float* xr, int K, float (&xv)[kPrepCache]) {
    const int nt = blockDim.x;
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < kPrepCache; ++c) {
        const int k = threadIdx.x + c * nt;
        const float t = xr[min(k, K - 1)];
        xv[c] = k < K ? t : 0.f;
        amax = fmaxf(amax, fabsf(xv[c]));
    }
    for (int k = threadIdx.x + kPrepCache * nt; k < K; k += nt) amax = fmaxf(amax, fabsf(xr[k]));
    return amax;
}
// grid (rows, regions): every activation operand of a layer stage - the int8 group's digits and the fp16 group's hi / lo
// halves - is prepared by one kernel
template <int D>
__global__ void __launch_bounds__(kPrepThreadsWide) tc_prepare_kernel(const __grid_constant__ TcPrepLaunch L) {
    __shared__ float redf[32];
    __shared__ long long redl[32];
    constexpr int P = 7 * D - 1;
    pdl_launch_dependents();
    pdl_wait();
    const TcPrepRegion& G = L.r[blockIdx.y];
    const int r = blockIdx.x, K = G.K, Kpad = G.Kpad, nt = blockDim.x;
    const float* xr = G.x + (size_t)r * G.ldx;
    float xv[kPrepCache];
    const int ex = tc_scale_exp(tc_block_max(tc_prep_load(xr, K, xv), redf));
    if (G.is_i8) {
        int8_t* B = reinterpret_cast<int8_t*>(G.B);
        const float inv = ldexpf(1.0f, P - ex);  // 2^P / e, exact
        long long ts = 0;
        auto digits = [&](int k, float x) {
            float v = x * inv;
            v = fminf(fmaxf(v, -(float)(1 << P)), (float)(1 << P));
            int t = __float2int_rn(v);
            if (!(v == v)) t = 0;  // NaN
            ts += t;
            int8_t d[D];
#pragma unroll
            for (int j = D - 1; j > 0; --j) {
                const int dj = ((t + 64) & 127) - 64;
                d[j] = (int8_t)dj;
                t = (t - dj) >> 7;
            }
            d[0] = (int8_t)t;
#pragma unroll
            for (int j = 0; j < D; ++j) B[((size_t)r * D + j) * Kpad + k] = d[j];
        };
#pragma unroll
        for (int c = 0; c < kPrepCache; ++c) {
            const int k = threadIdx.x + c * nt;
            if (k < K) digits(k, xv[c]);
        }
        for (int k = threadIdx.x + kPrepCache * nt; k < K; k += nt) digits(k, xr[k]);
        for (int k = K + threadIdx.x; k < Kpad; k += nt)
#pragma unroll
            for (int j = 0; j < D; ++j) B[((size_t)r * D + j) * Kpad + k] = 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ts += __shfl_xor_sync(0xffffffffu, ts, o);
        if ((threadIdx.x & 31) == 0) redl[threadIdx.x >> 5] = ts;
        __syncthreads();
        if (threadIdx.x == 0) {
            long long t = 0;
            for (int i = 0; i < (nt >> 5); ++i) t += redl[i];
            G.tsum[r] = t;
            G.xscale[r] = ldexpf(1.0f, ex - P);
        }
    } else {
        __half* B = reinterpret_cast<__half*>(G.B);
        const float inv = ldexpf(1.0f, -ex);
        auto split = [&](int k, float x) {
            float v = x * inv;
            v = fminf(fmaxf(v, -1.0f), 1.0f);
            if (!(v == v)) v = 0.f;
            const __half hi = __float2half_rn(v);
            const __half lo = __float2half_rn(v - __half2float(hi));
            B[((size_t)r * 2) * Kpad + k] = hi;
            B[((size_t)r * 2 + 1) * Kpad + k] = lo;
        };
#pragma unroll
        for (int c = 0; c < kPrepCache; ++c) {
            const int k = threadIdx.x + c * nt;
            if (k < K) split(k, xv[c]);
        }
        for (int k = threadIdx.x + kPrepCache * nt; k < K; k += nt) split(k, xr[k]);
        for (int k = K + threadIdx.x; k < Kpad; k += nt) {
            B[((size_t)r * 2) * Kpad + k] = __float2half_rn(0.f);
            B[((size_t)r * 2 + 1) * Kpad + k] = __float2half_rn(0.f);
        }
        if (threadIdx.x == 0) G.xscale[r] = ldexpf(1.0f, ex);
    }
}

}  // namespace rsv
