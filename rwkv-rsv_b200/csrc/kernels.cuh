// SIMT kernels of the RWKV-7 forward step (sm_100a).  fp16 / int8 appear only as weight storage:
// activations, state and every accumulation are fp32, reductions run in a fixed order (no atomics),
// so results are deterministic run to run.  Each kernel names the reference kernels it stands in for
// (all of them NVRTC strings in src/backend_cuda.rs) and the CPU-path lines that define its math.
#pragma once
#include "common.cuh"

namespace rsv {

// ------------------------------------------------------------------------------------------------
// small device helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over a whole CTA of NW warps; every thread returns the same value, summed in a fixed order.
template <int NW>
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();  // red[] may still be read from a previous call
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < NW; ++i) t += red[i];
    return t;
}

__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + expf(-v)); }

// streaming 16-byte load: weights are touched once per step, keep them out of L1
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// byte i of `word` as an exact float: build 2^23 + b in the mantissa, subtract 2^23
template <int I>
__device__ __forceinline__ float byte_to_float(uint32_t word) {
    return __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540u + I)) - 8388608.0f;
}

// ------------------------------------------------------------------------------------------------
// LayerNorm of one row held in global memory, two-pass variance exactly as src/model.rs:625-635:
// mean = sum/n ; var = sum((x-mean)^2)/n + eps ; out = (x-mean)/sqrt(var)*w + b.
// Returns (mean, inv_std) to every thread of the CTA.
// ------------------------------------------------------------------------------------------------
template <int NT>
__device__ __forceinline__ void row_stats(const float* __restrict__ x, int C, float eps, float* red, float& mean, float& inv_std) {
    float s = 0.f;
    for (int i = threadIdx.x; i < C; i += NT) s += x[i];
    mean = block_sum<NT / 32>(s, red) / (float)C;
    float q = 0.f;
    for (int i = threadIdx.x; i < C; i += NT) {
        float d = x[i] - mean;
        q += d * d;
    }
    float var = block_sum<NT / 32>(q, red) / (float)C + eps;
    inv_std = 1.0f / sqrtf(var);
}

// x[r] = LN0(emb[token[r]]).  Stands in for the reference's load-time emb_ln table plus
// rwkv_gather_row(s)_f16 (src/gpu_model.rs:450-460, src/backend_cuda.rs:4028-4041, 1644-1658); the
// CPU path applies the same LN0 in fp32 (src/model.rs:385-397).  Token ids are validated on the
// device: an id >= vocab sets bit 0 of *status and row 0 of the table is used instead, so a bad id
// can never index outside the table.
constexpr int kRowThreads = 256;
__global__ void __launch_bounds__(kRowThreads) embed_ln0_kernel(const __half* __restrict__ emb, const float* __restrict__ w,
                                                                const float* __restrict__ b, const uint32_t* __restrict__ tokens,
                                                                const int* __restrict__ tok_pos, int R, int C, int V, float* __restrict__ x,
                                                                int* __restrict__ status) {
    __shared__ float red[kRowThreads / 32];
    const int r = blockIdx.x;
    uint32_t tok = tokens[(tok_pos ? (size_t)(*tok_pos) * R : 0) + r];
    if (tok >= (uint32_t)V) {
        if (threadIdx.x == 0) atomicOr(status, 1);
        tok = 0;
    }
    const __half* row = emb + (size_t)tok * C;
    float s = 0.f;
    for (int i = threadIdx.x; i < C; i += kRowThreads) s += __half2float(row[i]);
    float mean = block_sum<kRowThreads / 32>(s, red) / (float)C;
    float q = 0.f;
    for (int i = threadIdx.x; i < C; i += kRowThreads) {
        float d = __half2float(row[i]) - mean;
        q += d * d;
    }
    float inv_std = 1.0f / sqrtf(block_sum<kRowThreads / 32>(q, red) / (float)C + kLnEps);
    for (int i = threadIdx.x; i < C; i += kRowThreads) x[(size_t)r * C + i] = (__half2float(row[i]) - mean) * inv_std * w[i] + b[i];
}

// Advances the device-side token cursor used by the token-by-token decode path.
__global__ void advance_cursor_kernel(int* pos) { *pos += 1; }

// LayerNorm + token shift.  NMIX=6: ln1 and the six time-mix lerps; NMIX=1: ln2 and the channel-mix
// lerp.  Stands in for norm_lerp6(_batch), cmix_norm_lerp(_batch), rwkv_seq_shift(_batch) and
// rwkv_copy_token(_batch) (src/backend_cuda.rs:2412-2549, 1505-1640, 4313-4406); math per
// src/model.rs:402-411, 487-490: out_m = cur + mix_m * (prev - cur), state <- cur.
// The residual add of the preceding linear layer is folded in: when `delta` is given the row's input is
// x_in + delta (src/model.rs:484, 495) and that sum is written to x_out, a different buffer, because
// row r also needs row r-1's sum while another CTA produces it.
// `prev` is the LayerNorm of row r-1 when that row is the session's previous token (recomputed here
// with the same code, hence the same bits) and the slot's shift state otherwise.  When a step holds
// multi-row segments the new shift state goes to `staging` (one row per segment) and is committed by
// commit_shift_kernel afterwards, because the segment's first row still has to read the old state.
struct MixPtrs {
    const float* m[6];
};
template <int NT>
__device__ __forceinline__ void row_stats2(const float* __restrict__ x, const float* __restrict__ d, int C, float eps, float* red, float& mean,
                                           float& inv_std) {
    float s = 0.f;
    for (int i = threadIdx.x; i < C; i += NT) s += d ? x[i] + d[i] : x[i];
    mean = block_sum<NT / 32>(s, red) / (float)C;
    float q = 0.f;
    for (int i = threadIdx.x; i < C; i += NT) {
        const float t = (d ? x[i] + d[i] : x[i]) - mean;
        q += t * t;
    }
    const float var = block_sum<NT / 32>(q, red) / (float)C + eps;
    inv_std = 1.0f / sqrtf(var);
}
template <int NMIX>
__global__ void __launch_bounds__(kRowThreads) ln_shift_kernel(const float* __restrict__ x_in, const float* __restrict__ delta, float* __restrict__ x_out,
                                                               const float* __restrict__ lw, const float* __restrict__ lb, MixPtrs mix,
                                                               const RowMeta* __restrict__ rows, int R, int C, float* __restrict__ shift_state,
                                                               float* __restrict__ staging, float* __restrict__ out) {
    __shared__ float red[kRowThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    x_in = pdl_fresh(x_in);
    delta = pdl_fresh(delta);
    shift_state = pdl_fresh(shift_state);
    const int r = blockIdx.x;
    const RowMeta rm = rows[r];
    const float* xr = x_in + (size_t)r * C;
    const float* dr = delta ? delta + (size_t)r * C : nullptr;
    float mean, inv_std, pmean = 0.f, pinv = 0.f;
    row_stats2<kRowThreads>(xr, dr, C, kLnEps, red, mean, inv_std);
    if (rm.has_prev) row_stats2<kRowThreads>(xr - C, dr ? dr - C : nullptr, C, kLnEps, red, pmean, pinv);
    // gridDim.y CTAs share a row: each has the full-row statistics and writes the channels [c_lo, c_hi)
    const int c_lo = (int)(((long long)blockIdx.y * C) / gridDim.y), c_hi = (int)(((long long)(blockIdx.y + 1) * C) / gridDim.y);
    for (int i = c_lo + threadIdx.x; i < c_hi; i += kRowThreads) {
        const float wi = lw[i], bi = lb[i];
        const float xv = dr ? xr[i] + dr[i] : xr[i];
        if (dr) x_out[(size_t)r * C + i] = xv;
        const float cur = (xv - mean) * inv_std * wi + bi;
        float prev;
        if (rm.has_prev) {
            const float xp = dr ? xr[i - C] + dr[i - C] : xr[i - C];
            prev = (xp - pmean) * pinv * wi + bi;
        } else {
            prev = shift_state[(size_t)rm.slot * C + i];
        }
#pragma unroll
        for (int m = 0; m < NMIX; ++m) out[((size_t)m * R + r) * C + i] = cur + mix.m[m][i] * (prev - cur);
        if (rm.is_last) {
            if (staging)
                staging[(size_t)rm.seg * C + i] = cur;
            else
                shift_state[(size_t)rm.slot * C + i] = cur;
        }
    }
}
__global__ void commit_shift_kernel(const float* __restrict__ staging, const SegMeta* __restrict__ segs, int C, float* __restrict__ shift_state) {
    pdl_launch_dependents();
    pdl_wait();
    staging = pdl_fresh(staging);
    const SegMeta sg = segs[blockIdx.x];
    for (int i = threadIdx.x; i < C; i += blockDim.x) shift_state[(size_t)sg.slot * C + i] = staging[(size_t)blockIdx.x * C + i];
}

// Plain LayerNorm of selected rows (ln_out before the head; src/model.rs:507, rwkv_norm at
// src/backend_cuda.rs:2555-2610).  out[o] = LN(x[out_rows[o]] (+ delta[out_rows[o]])).
__global__ void __launch_bounds__(kRowThreads) ln_rows_kernel(const float* __restrict__ x, const float* __restrict__ delta, const float* __restrict__ lw,
                                                              const float* __restrict__ lb, const int* __restrict__ out_rows, int C,
                                                              float* __restrict__ out) {
    __shared__ float red[kRowThreads / 32];
    const size_t row = (size_t)out_rows[blockIdx.x];
    const float* xr = x + row * C;
    const float* dr = delta ? delta + row * C : nullptr;
    float mean, inv_std;
    row_stats2<kRowThreads>(xr, dr, C, kLnEps, red, mean, inv_std);
    for (int i = threadIdx.x; i < C; i += kRowThreads)
        out[(size_t)blockIdx.x * C + i] = ((dr ? xr[i] + dr[i] : xr[i]) - mean) * inv_std * lw[i] + lb[i];
}

// ------------------------------------------------------------------------------------------------
// Weight-streaming linear layer, SIMT form: y[r, m] = epi( sum_k W[m,k] * x[r,k] ).
// Stands in for gemv_f16, gemv_variant(_mb), gemv_(int8_)rkv_stage1(_batch), gemv_lowrank_chain4(_batch),
// rwkv_dequant_int8 + GEMM + rwkv_gemm_epilogue (src/backend_cuda.rs:1421-1498, 1665-1986, 2772-3554,
// 4195-4227, 4580-4633).  Differences by design: fp32 accumulation (the reference accumulates in half2),
// the int8 dequant w = scale*q + zero (src/model.rs:234-252) is applied per group of 128 in factored
// form  sum_g [ scale_g * sum_{k in g} q_k x_k  +  zero_g * sum_{k in g} x_k ],  and one warp owns an
// output element so its reduction order is fixed.
// A launch runs up to 8 independent problems (r/k/v plus the four rank-space projections of a layer
// go out together).  Every weight byte is read once per tile of RT rows.
// ------------------------------------------------------------------------------------------------
constexpr int kLinWarps = 8;
constexpr int kLinWR = 2;  // output rows a warp carries at a time
struct LinProb {
    const void* w;       // fp16 [M,K] or u8 [M,K]
    const uint32_t* sz;  // int8 only: [M, K/128] words, fp16 scale (low half) | fp16 zero (high half)
    const float* x;      // [R, ldx]
    float* y;            // [R, ldy]
    float* y2;           // optional second copy of the output (EPI_STORE only)
    const float* bias;   // [M]     (EPI_DECAY, EPI_SIGMOID_BIAS, EPI_VLERP)
    const float* aux;    // [R, ldaux] (EPI_VLERP)
    int M, K, ldx, ldy, ldaux, wtype, epi;
    int rows_per_blk;  // output rows per CTA, multiple of kLinWarps*kLinWR
    int blk0;          // first blockIdx.x of this problem
};
struct LinGroup {
    LinProb p[8];
    int n;
};

__device__ __forceinline__ void lin_epilogue(const LinProb& P, int r, int m, float acc) {
    float* yp = P.y + (size_t)r * P.ldy + m;
    switch (P.epi) {
        case EPI_STORE:
            *yp = acc;
            if (P.y2) P.y2[(size_t)r * P.ldy + m] = acc;
            break;
        case EPI_ADD: *yp += acc; break;
        case EPI_RELU2: {
            float t = fmaxf(acc, 0.f);
            *yp = t * t;
            break;
        }
        case EPI_TANH: *yp = tanhf(acc); break;
        case EPI_SIGMOID: *yp = sigmoidf_(acc); break;
        case EPI_DECAY: *yp = expf(sigmoidf_(acc + P.bias[m]) * kDecayScale); break;
        case EPI_SIGMOID_BIAS: *yp = sigmoidf_(acc + P.bias[m]); break;
        case EPI_VLERP: {
            float v = *yp;
            float gate = sigmoidf_(acc + P.bias[m]);
            *yp = v + gate * (P.aux[(size_t)r * P.ldaux + m] - v);
            break;
        }
    }
}

// x tile in shared memory: element k of row rr lives in float4 slot [(rr*JPC + j) * nchunk + c] with
// c = k / CH (the chunk one lane consumes per step), j = (k % CH) / 4.  Consecutive lanes read
// consecutive float4 slots, so the reads are bank-conflict free.
template <int RT>
__global__ void __launch_bounds__(kLinWarps * 32) linear_rows_kernel(const __grid_constant__ LinGroup g, int R) {
    extern __shared__ float4 smem4[];
    int pi = 0;
    while (pi + 1 < g.n && (int)blockIdx.x >= g.p[pi + 1].blk0) ++pi;
    const LinProb& P = g.p[pi];
    const int K = P.K, M = P.M;
    const bool i8 = P.wtype == W_INT8;
    const int CH = i8 ? 16 : 8, JPC = CH / 4;
    const int nchunk = K / CH;
    const int r0 = blockIdx.y * RT;
    float4* xs = smem4;                                        // [RT][JPC][nchunk]
    float* xsum = reinterpret_cast<float*>(xs + RT * (K / 4));  // [RT][nchunk] (int8 only)

    const int k4 = K / 4;
    for (int idx = threadIdx.x; idx < RT * k4; idx += kLinWarps * 32) {
        const int rr = idx / k4, f = idx - rr * k4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r0 + rr < R) v = *reinterpret_cast<const float4*>(P.x + (size_t)(r0 + rr) * P.ldx + (size_t)f * 4);
        xs[(rr * JPC + (f % JPC)) * nchunk + f / JPC] = v;
    }
    __syncthreads();
    if (i8) {
        for (int idx = threadIdx.x; idx < RT * nchunk; idx += kLinWarps * 32) {
            const int rr = idx / nchunk, c = idx - rr * nchunk;
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float4 v = xs[(rr * 4 + j) * nchunk + c];
                s += (v.x + v.y) + (v.z + v.w);
            }
            xsum[idx] = s;
        }
        __syncthreads();
    }

    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int mblk = ((int)blockIdx.x - P.blk0) * P.rows_per_blk;
    const int mend = min(M, mblk + P.rows_per_blk);
    for (int m0 = mblk + wid * kLinWR; m0 < mend; m0 += kLinWarps * kLinWR) {
        float acc[kLinWR][RT];
#pragma unroll
        for (int a = 0; a < kLinWR; ++a)
#pragma unroll
            for (int rr = 0; rr < RT; ++rr) acc[a][rr] = 0.f;
        const bool has1 = m0 + 1 < mend;
        if (i8) {
            const int KG = K / 128;
            const uint8_t* w0 = reinterpret_cast<const uint8_t*>(P.w) + (size_t)m0 * K;
            const uint8_t* w1 = w0 + (has1 ? K : 0);
            const uint32_t* s0 = P.sz + (size_t)m0 * KG;
            const uint32_t* s1 = s0 + (has1 ? KG : 0);
            for (int c = lane; c < nchunk; c += 32) {
                const uint4 wa = ld_stream(reinterpret_cast<const uint4*>(w0) + c);
                const uint4 wb = ld_stream(reinterpret_cast<const uint4*>(w1) + c);
                const uint32_t za = __ldg(s0 + (c >> 3)), zb = __ldg(s1 + (c >> 3));
                float qa[16], qb[16];
                {
                    const uint32_t wv[4] = {wa.x, wa.y, wa.z, wa.w};
                    const uint32_t uv[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        qa[4 * j + 0] = byte_to_float<0>(wv[j]);
                        qa[4 * j + 1] = byte_to_float<1>(wv[j]);
                        qa[4 * j + 2] = byte_to_float<2>(wv[j]);
                        qa[4 * j + 3] = byte_to_float<3>(wv[j]);
                        qb[4 * j + 0] = byte_to_float<0>(uv[j]);
                        qb[4 * j + 1] = byte_to_float<1>(uv[j]);
                        qb[4 * j + 2] = byte_to_float<2>(uv[j]);
                        qb[4 * j + 3] = byte_to_float<3>(uv[j]);
                    }
                }
                const float sa = __half2float(__ushort_as_half((unsigned short)(za & 0xFFFFu)));
                const float oa = __half2float(__ushort_as_half((unsigned short)(za >> 16)));
                const float sb = __half2float(__ushort_as_half((unsigned short)(zb & 0xFFFFu)));
                const float ob = __half2float(__ushort_as_half((unsigned short)(zb >> 16)));
#pragma unroll
                for (int rr = 0; rr < RT; ++rr) {
                    float pa = 0.f, pb = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 xv = xs[(rr * 4 + j) * nchunk + c];
                        pa = fmaf(qa[4 * j + 0], xv.x, pa);
                        pa = fmaf(qa[4 * j + 1], xv.y, pa);
                        pa = fmaf(qa[4 * j + 2], xv.z, pa);
                        pa = fmaf(qa[4 * j + 3], xv.w, pa);
                        pb = fmaf(qb[4 * j + 0], xv.x, pb);
                        pb = fmaf(qb[4 * j + 1], xv.y, pb);
                        pb = fmaf(qb[4 * j + 2], xv.z, pb);
                        pb = fmaf(qb[4 * j + 3], xv.w, pb);
                    }
                    const float xsm = xsum[rr * nchunk + c];
                    acc[0][rr] += sa * pa + oa * xsm;
                    acc[1][rr] += sb * pb + ob * xsm;
                }
            }
        } else {
            const __half* w0 = reinterpret_cast<const __half*>(P.w) + (size_t)m0 * K;
            const __half* w1 = w0 + (has1 ? K : 0);
            for (int c = lane; c < nchunk; c += 32) {
                const uint4 wa = ld_stream(reinterpret_cast<const uint4*>(w0) + c);
                const uint4 wb = ld_stream(reinterpret_cast<const uint4*>(w1) + c);
                float qa[8], qb[8];
                {
                    const uint32_t wv[4] = {wa.x, wa.y, wa.z, wa.w};
                    const uint32_t uv[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&wv[j]));
                        const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&uv[j]));
                        qa[2 * j] = fa.x;
                        qa[2 * j + 1] = fa.y;
                        qb[2 * j] = fb.x;
                        qb[2 * j + 1] = fb.y;
                    }
                }
#pragma unroll
                for (int rr = 0; rr < RT; ++rr) {
                    float pa = acc[0][rr], pb = acc[1][rr];
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const float4 xv = xs[(rr * 2 + j) * nchunk + c];
                        pa = fmaf(qa[4 * j + 0], xv.x, pa);
                        pa = fmaf(qa[4 * j + 1], xv.y, pa);
                        pa = fmaf(qa[4 * j + 2], xv.z, pa);
                        pa = fmaf(qa[4 * j + 3], xv.w, pa);
                        pb = fmaf(qb[4 * j + 0], xv.x, pb);
                        pb = fmaf(qb[4 * j + 1], xv.y, pb);
                        pb = fmaf(qb[4 * j + 2], xv.z, pb);
                        pb = fmaf(qb[4 * j + 3], xv.w, pb);
                    }
                    acc[0][rr] = pa;
                    acc[1][rr] = pb;
                }
            }
        }
#pragma unroll
        for (int a = 0; a < kLinWR; ++a)
#pragma unroll
            for (int rr = 0; rr < RT; ++rr) {
                const float v = warp_sum(acc[a][rr]);
                if (lane == 0 && (a == 0 || has1) && r0 + rr < R) lin_epilogue(P, r0 + rr, m0 + a, v);
            }
    }
}

// ------------------------------------------------------------------------------------------------
// WKV-7: per (segment, head) the 64x64 fp32 state is loaded once, advanced over the segment's rows
// in order and written back in place through the slot table.  Stands in for fuse_ka_dplr_norm,
// rwkv_fuse_ka, rwkv_dplr_seq(_batch), rwkv_norm (GroupNorm) and rwkv_sum_rk_rk
// (src/backend_cuda.rs:2620-2764, 4231-4309, 4436-4575).  Math per src/model.rs:445-480, 716-826:
//   kk = k*k_k ; kk^ = kk / max(|kk|_2, 1e-12)   (true L2 norm; the reference's fused decode kernel
//        divides by sqrt(2*sum kk^2), src/backend_cuda.rs:2671-2680 — not reproduced)
//   k~ = k + k_a*(k*a - k) ; b = -kk^*a
//   sa[i] = sum_j S[i][j] kk^[j] ; S[i][j] = S[i][j] w[j] + sa[i] b[j] + v[i] k~[j] ; y[i] = sum_j S[i][j] r[j]
//   out = (GroupNorm(y; eps 64e-5) + (sum_j r[j] k~[j] r_k[j]) * v) * g
// Four threads share state row i (16 columns each, in registers); their partial sums are combined with shuffles.
// ------------------------------------------------------------------------------------------------
constexpr int kWkvThreads = 256;
// One CTA per (head, segment); warp w owns state rows 8w .. 8w+7, four lanes per row.  Lane quad q of a row holds
// columns 16 jj + 4 q + c (jj, c = 0..3), so one float4 instruction of a warp covers eight full 64-byte runs.
// The per-token vectors over the column index (normalised kk, decay w, b = -kk a, k~, r) and the two scalars that
// depend on the inputs only (|kk|^2 and the bonus dot product) are computed by every warp for itself with warp
// shuffles; only the GroupNorm statistics of y cross warps (two block barriers per token).  All global loads of a
// token are issued before the first use, so a CTA waits for memory once per token.
// The per-token inputs of one lane (two of the 64 channels, and the row's v, g and v-lerp operands), shared with the row-per-lane
// kernel for large batches (wkv_rows.cuh).  Loading does no arithmetic, so that a token's inputs can be requested one token
// ahead of their use: inside a multi-token segment (prefill) the recurrence is sequential and a memory round trip per token
// would be its whole cost.
struct WkvIn {
    float k0, k1, a0, a1, r0, r1, w0, w1, v, g, vg, vf;
};
__device__ __forceinline__ WkvIn wkv_load_inputs(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                                                 const float* __restrict__ vgate, const float* __restrict__ vfirst, const float* __restrict__ w,
                                                 const float* __restrict__ a, const float* __restrict__ g, size_t hb, int lane, int i) {
    WkvIn x;
    x.k0 = k[hb + lane];
    x.k1 = k[hb + lane + 32];
    x.a0 = a[hb + lane];
    x.a1 = a[hb + lane + 32];
    x.r0 = r[hb + lane];
    x.r1 = r[hb + lane + 32];
    x.w0 = w[hb + lane];
    x.w1 = w[hb + lane + 32];
    x.v = v[hb + i];
    x.g = g[hb + i];
    x.vg = vgate ? vgate[hb + i] : 0.f;
    x.vf = vgate ? vfirst[hb + i] : 0.f;
    return x;
}
// v of the token: layers > 0 lerp towards the first layer's v (src/model.rs:424-430)
__device__ __forceinline__ float wkv_value(const WkvIn& x, bool has_gate) { return has_gate ? x.v + x.vg * (x.vf - x.v) : x.v; }

// `vgate` (layers > 0): v <- v + vgate * (vfirst - v), the lerp of src/model.rs:424-430 (the gate itself,
// sigmoid(v0 + (xv v1) v2), comes from the rank back-projection).
__global__ void __launch_bounds__(kWkvThreads, 4) wkv7_kernel(const SegMeta* __restrict__ segs, const float* __restrict__ r, const float* __restrict__ k,
                                                              const float* __restrict__ v, const float* __restrict__ vgate,
                                                              const float* __restrict__ vfirst, const float* __restrict__ w, const float* __restrict__ a,
                                                              const float* __restrict__ g, const float* __restrict__ k_k, const float* __restrict__ k_a,
                                                              const float* __restrict__ r_k, const float* __restrict__ lnx_w, const float* __restrict__ lnx_b,
                                                              float* __restrict__ state, float* __restrict__ v_first_state, float* __restrict__ yg, int H,
                                                              int C) {
    constexpr int N = kHeadSize;
    __shared__ __align__(16) float s_vec[kWkvThreads / 32][5][N];  // per warp: kk, w, b, k~, r
    __shared__ float red_a[kWkvThreads / 32], red_b[kWkvThreads / 32];
    const int h = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, i = tid >> 2, quad = tid & 3;
    pdl_launch_dependents();
    // The segment table and this layer's state were last written before the step's first kernel (plan upload, the previous
    // step's launch of this kernel): they may be read before the predecessor in the stream has finished.
    const SegMeta sg = segs[blockIdx.y];
    float* srow = state + (((size_t)sg.slot * H + h) * N + i) * N + quad * 4;
    float S[16];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
        const float4 t = *reinterpret_cast<const float4*>(srow + 16 * jj);
        S[4 * jj] = t.x;
        S[4 * jj + 1] = t.y;
        S[4 * jj + 2] = t.z;
        S[4 * jj + 3] = t.w;
    }
    pdl_wait();
    r = pdl_fresh(r);
    k = pdl_fresh(k);
    v = pdl_fresh(v);
    vgate = pdl_fresh(vgate);
    vfirst = pdl_fresh(vfirst);
    w = pdl_fresh(w);
    a = pdl_fresh(a);
    g = pdl_fresh(g);
    const int hc = h * N;
    const float kkc0 = k_k[hc + lane], kkc1 = k_k[hc + lane + 32], kac0 = k_a[hc + lane], kac1 = k_a[hc + lane + 32];
    const float rkc0 = r_k[hc + lane], rkc1 = r_k[hc + lane + 32];
    const float gw = lnx_w[hc + i], gb = lnx_b[hc + i];
    float(*sv)[N] = s_vec[warp];
    WkvIn nxt = wkv_load_inputs(r, k, v, vgate, vfirst, w, a, g, (size_t)sg.start * C + hc, lane, i);
    for (int t = 0; t < sg.len; ++t) {
        const size_t hb = (size_t)(sg.start + t) * C + hc;
        const WkvIn cur = nxt;
        if (t + 1 < sg.len) nxt = wkv_load_inputs(r, k, v, vgate, vfirst, w, a, g, hb + C, lane, i);  // the next token's inputs, one token ahead
        const float k0 = cur.k0, k1 = cur.k1, a0 = cur.a0, a1 = cur.a1, r0 = cur.r0, r1 = cur.r1, w0 = cur.w0, w1 = cur.w1;
        const float vj = wkv_value(cur, vgate != nullptr);
        const float gj = cur.g;
        const float kk0 = k0 * kkc0, kk1 = k1 * kkc1;
        const float ss = warp_sum(kk0 * kk0 + kk1 * kk1);
        const float inv = 1.0f / fmaxf(sqrtf(ss), kL2Eps);
        const float kh0 = kk0 * inv, kh1 = kk1 * inv;
        const float kt0 = k0 + kac0 * (k0 * a0 - k0), kt1 = k1 + kac1 * (k1 * a1 - k1);
        const float srk = warp_sum(r0 * kt0 * rkc0 + r1 * kt1 * rkc1);
        __syncwarp();  // the previous token's readers are done with sv
        sv[0][lane] = kh0;
        sv[0][lane + 32] = kh1;
        sv[1][lane] = w0;
        sv[1][lane + 32] = w1;
        sv[2][lane] = kh0 * (-a0);
        sv[2][lane + 32] = kh1 * (-a1);
        sv[3][lane] = kt0;
        sv[3][lane + 32] = kt1;
        sv[4][lane] = r0;
        sv[4][lane + 32] = r1;
        __syncwarp();
        float sa = 0.f;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const float4 kk4 = *reinterpret_cast<const float4*>(&sv[0][16 * jj + 4 * quad]);
            sa = fmaf(S[4 * jj], kk4.x, sa);
            sa = fmaf(S[4 * jj + 1], kk4.y, sa);
            sa = fmaf(S[4 * jj + 2], kk4.z, sa);
            sa = fmaf(S[4 * jj + 3], kk4.w, sa);
        }
        sa += __shfl_xor_sync(0xffffffffu, sa, 1);
        sa += __shfl_xor_sync(0xffffffffu, sa, 2);
        float y = 0.f;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int c0 = 16 * jj + 4 * quad;
            const float4 w4 = *reinterpret_cast<const float4*>(&sv[1][c0]);
            const float4 b4 = *reinterpret_cast<const float4*>(&sv[2][c0]);
            const float4 t4 = *reinterpret_cast<const float4*>(&sv[3][c0]);
            const float4 r4 = *reinterpret_cast<const float4*>(&sv[4][c0]);
            S[4 * jj] = fmaf(S[4 * jj], w4.x, fmaf(sa, b4.x, vj * t4.x));
            S[4 * jj + 1] = fmaf(S[4 * jj + 1], w4.y, fmaf(sa, b4.y, vj * t4.y));
            S[4 * jj + 2] = fmaf(S[4 * jj + 2], w4.z, fmaf(sa, b4.z, vj * t4.z));
            S[4 * jj + 3] = fmaf(S[4 * jj + 3], w4.w, fmaf(sa, b4.w, vj * t4.w));
            y = fmaf(S[4 * jj], r4.x, y);
            y = fmaf(S[4 * jj + 1], r4.y, y);
            y = fmaf(S[4 * jj + 2], r4.z, y);
            y = fmaf(S[4 * jj + 3], r4.w, y);
        }
        y += __shfl_xor_sync(0xffffffffu, y, 1);
        y += __shfl_xor_sync(0xffffffffu, y, 2);
        // GroupNorm over the head's 64 outputs (two-pass, like the CPU path)
        const float ys = warp_sum(quad == 0 ? y : 0.f);
        if (lane == 0) red_a[warp] = ys;
        __syncthreads();
        const float mean = (((red_a[0] + red_a[1]) + (red_a[2] + red_a[3])) + ((red_a[4] + red_a[5]) + (red_a[6] + red_a[7]))) / (float)N;
        const float d = y - mean;
        const float qs = warp_sum(quad == 0 ? d * d : 0.f);
        if (lane == 0) red_b[warp] = qs;
        __syncthreads();
        const float var = (((red_b[0] + red_b[1]) + (red_b[2] + red_b[3])) + ((red_b[4] + red_b[5]) + (red_b[6] + red_b[7]))) / (float)N + kGnEps;
        const float inv_std = 1.0f / sqrtf(var);
        if (quad == 0) {
            yg[hb + i] = (d * inv_std * gw + gb + srk * vj) * gj;
            if (v_first_state && t == sg.len - 1) v_first_state[(size_t)sg.slot * C + hc + i] = vj;
        }
    }
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) *reinterpret_cast<float4*>(srow + 16 * jj) = make_float4(S[4 * jj], S[4 * jj + 1], S[4 * jj + 2], S[4 * jj + 3]);
}

// ------------------------------------------------------------------------------------------------
// arg-max over each logits row, ties -> smaller index (rwkv_argmax, src/backend_cuda.rs:3640-3680).
// Writes the token to next_tok[row] (the next step's input) and appends it to the row's sequence
// buffer (rwkv_record_token(s), src/backend_cuda.rs:4014-4023, 2392-2403).
// ------------------------------------------------------------------------------------------------
constexpr int kArgmaxThreads = 1024;
__device__ __forceinline__ void argmax_combine(float& bv, int& bi, float ov, int oi) {
    if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
    }
}
// `row_map` (optional) sends logits row r to entry row_map[r] of next_tok / seq / seq_cnt (the continuous-batching
// scheduler keeps those per slot, while the logits rows are packed per step).
__global__ void __launch_bounds__(kArgmaxThreads) argmax_rows_kernel(const float* __restrict__ logits, int V, uint32_t* __restrict__ next_tok,
                                                                     uint32_t* __restrict__ seq, int* __restrict__ seq_cnt, int seq_cap,
                                                                     const int* __restrict__ row_map) {
    __shared__ float sv[kArgmaxThreads / 32];
    __shared__ int si[kArgmaxThreads / 32];
    const int row = blockIdx.x;
    const float* lg = logits + (size_t)row * V;
    float bv = -1e30f;
    int bi = 0;
    for (int i = threadIdx.x; i < V; i += kArgmaxThreads) {
        const float x = lg[i];
        if (x > bv) {
            bv = x;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_combine(bv, bi, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = bv;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i2 = 1; i2 < kArgmaxThreads / 32; ++i2) argmax_combine(bv, bi, sv[i2], si[i2]);
        const int dst = row_map ? row_map[row] : row;
        next_tok[dst] = (uint32_t)bi;
        if (seq) {
            const int c = seq_cnt[dst];
            if (c < seq_cap) seq[(size_t)dst * seq_cap + c] = (uint32_t)bi;
            seq_cnt[dst] = c + 1;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Sampling: penalties -> temperature -> top-k -> softmax -> top-p -> draw, one CTA per logits row.
// Specification = the general path of rwkv_sample(_batch) (src/backend_cuda.rs:3741-3769, 3835-3908,
// 3923-3957, 3980-4006): top-k keeps everything >= the K-th largest value; top-p picks probabilities
// from the largest down (at most 512 picks) until the running sum reaches top_p and keeps everything
// >= the last pick; the draw is u = u01(seed) * sum(kept) and the first index, in vocabulary order,
// whose running sum exceeds u.  The reference's 1<=top_k<=50 fast path accumulates top-p and the
// draw from the smallest kept probability (:3913-3922, :3962-3978), against its documented intent;
// that variant is not reproduced — every top_k takes the path above.
// Here the K-th largest value comes from a 4-pass radix select instead of K arg-max sweeps, the 512
// picks from a radix select plus a 512-element bitonic sort, and the vocabulary-order walk from a
// block prefix sum; sums are fp32 but grouped differently from the reference's 112-thread tree, so
// a draw can differ from it only when u falls within rounding distance of a CDF step.
// Per-row history for the penalties is seq[row*seq_cap .. +round) — the reference's batched kernel
// reads slot b's history at b*hist_len instead of b*n (src/backend_cuda.rs:2124 vs :2400); that
// indexing slip is not reproduced.
// ------------------------------------------------------------------------------------------------
constexpr int kSampleThreads = 1024;
constexpr int kTopPMaxPicks = 512;

__device__ __forceinline__ float u01(uint32_t s) {  // src/backend_cuda.rs:3691-3698
    s += 0x9E3779B9u;
    uint32_t z = s;
    z = (z ^ (z >> 16)) * 0x85EBCA6Bu;
    z = (z ^ (z >> 13)) * 0xC2B2AE35u;
    z ^= z >> 16;
    return (float)z / 4294967296.0f;
}
__device__ __forceinline__ uint32_t float_key(float f) {  // order-preserving float -> uint
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}
// Key of the K-th largest (1-based) of vals[0..n), values below `floor_thr` read as -1e30.
__device__ uint32_t kth_largest_key(const float* vals, int n, int K, float floor_thr, uint32_t* hist, uint32_t* sh) {
    uint32_t prefix = 0, mask = 0;
    int krem = K;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += kSampleThreads) hist[i] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += kSampleThreads) {
            float v = vals[i];
            if (v < floor_thr) v = -1e30f;
            const uint32_t key = float_key(v);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int b = 255, cum = 0;
            for (; b > 0; --b) {
                if (cum + (int)hist[b] >= krem) break;
                cum += (int)hist[b];
            }
            sh[0] = (uint32_t)b;
            sh[1] = (uint32_t)(krem - cum);
        }
        __syncthreads();
        prefix |= sh[0] << shift;
        mask |= 255u << shift;
        krem = (int)sh[1];
        __syncthreads();
    }
    return prefix;
}

__global__ void __launch_bounds__(kSampleThreads) sample_rows_kernel(const float* __restrict__ logits, int V, const float* __restrict__ sampler8,
                                                                     const uint32_t* __restrict__ hist, int hist_stride,
                                                                     const int* __restrict__ round_cnt, float* __restrict__ temp_all,
                                                                     uint32_t* __restrict__ counter_all, uint32_t* __restrict__ next_tok,
                                                                     uint32_t* __restrict__ seq, int* __restrict__ seq_cnt, int seq_cap,
                                                                     const int* __restrict__ row_map) {
    __shared__ float red[kSampleThreads / 32];
    __shared__ uint32_t s_hist[256];
    __shared__ uint32_t s_sh[2];
    __shared__ float s_list[kTopPMaxPicks];
    __shared__ int s_count;
    __shared__ float s_cut;
    __shared__ int s_chosen;
    const int row = blockIdx.x, tid = threadIdx.x;
    const int ent = row_map ? row_map[row] : row;  // entry of the per-session arrays (sampler rows, history, counters, tokens)
    const float* lg = logits + (size_t)row * V;
    float* temp = temp_all + (size_t)row * V;
    const float* sp = sampler8 + (size_t)ent * 8;
    const float temperature = sp[0];
    const uint32_t top_k = __float_as_uint(sp[1]);
    const float top_p = sp[2];
    uint32_t seed = __float_as_uint(sp[3]);
    const float rep = sp[4], freq = sp[5], pres = sp[6];
    uint32_t hist_len = __float_as_uint(sp[7]);
    if (round_cnt) {  // self-loop: round r uses seed+r and the r tokens generated so far
        const uint32_t round = (uint32_t)round_cnt[ent];
        seed += round;
        hist_len = min(round, (uint32_t)hist_stride);
    }
    const uint32_t* hrow = hist ? hist + (size_t)ent * hist_stride : nullptr;
    const bool penal = hist_len > 0u && hrow && (rep != 1.0f || freq != 0.0f || pres != 0.0f);
    if (penal) {
        uint32_t* counter = counter_all + (size_t)row * V;
        for (int i = tid; i < V; i += kSampleThreads) counter[i] = 0u;
        __syncthreads();
        for (int h = tid; h < (int)hist_len; h += kSampleThreads) {
            const uint32_t t = hrow[h];
            if (t < (uint32_t)V) atomicAdd(&counter[t], 1u);
        }
        __syncthreads();
    }
    float invT = 1.0f / temperature;
    if (!(temperature > 0.0f)) invT = 1.0f;
    float lm = -1e30f;
    for (int i = tid; i < V; i += kSampleThreads) {
        float l = lg[i];
        if (penal) {
            const uint32_t cnt = counter_all[(size_t)row * V + i];
            if (cnt > 0u) {
                if (rep != 1.0f) l = l > 0.0f ? l / rep : l * rep;
                if (pres != 0.0f) l -= pres;
            }
            if (freq != 0.0f) l -= freq * (float)cnt;
        }
        l *= invT;
        temp[i] = l;
        lm = fmaxf(lm, l);
    }
    // block max
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lm = fmaxf(lm, __shfl_xor_sync(0xffffffffu, lm, o));
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = lm;
    __syncthreads();
    float mx = red[0];
#pragma unroll
    for (int i = 1; i < kSampleThreads / 32; ++i) mx = fmaxf(mx, red[i]);
    __syncthreads();

    float thr = -3.0e38f;
    if (top_k > 0u && top_k < (uint32_t)V) thr = key_float(kth_largest_key(temp, V, (int)top_k, -3.0e38f, s_hist, s_sh));

    float ps = 0.f;
    for (int i = tid; i < V; i += kSampleThreads) {
        float l = temp[i];
        if (l < thr) l = -1e30f;
        const float e = expf(l - mx);
        temp[i] = e;
        ps += e;
    }
    const float total = block_sum<kSampleThreads / 32>(ps, red);
    if (total > 0.0f)
        for (int i = tid; i < V; i += kSampleThreads) temp[i] = temp[i] / total;
    __syncthreads();

    float cutoff = 0.0f;
    if (top_p > 0.0f && top_p < 1.0f) {
        const int L = min(kTopPMaxPicks, V);
        const uint32_t tkey = kth_largest_key(temp, V, L, -3.0e38f, s_hist, s_sh);
        const float tval = key_float(tkey);
        if (tid == 0) s_count = 0;
        for (int i = tid; i < kTopPMaxPicks; i += kSampleThreads) s_list[i] = -1.0f;
        __syncthreads();
        for (int i = tid; i < V; i += kSampleThreads) {
            const float p = temp[i];
            if (p > tval) {
                const int pos = atomicAdd(&s_count, 1);
                if (pos < kTopPMaxPicks) s_list[pos] = p;
            }
        }
        __syncthreads();
        const int ngreater = min(s_count, L);
        for (int i = ngreater + tid; i < L; i += kSampleThreads) s_list[i] = tval;  // ties with the L-th largest
        __syncthreads();
        for (int kk = 2; kk <= kTopPMaxPicks; kk <<= 1)  // bitonic sort, descending
            for (int j = kk >> 1; j > 0; j >>= 1) {
                for (int idx = tid; idx < kTopPMaxPicks; idx += kSampleThreads) {
                    const int ixj = idx ^ j;
                    if (ixj > idx) {
                        const float a0 = s_list[idx], a1 = s_list[ixj];
                        const bool desc = (idx & kk) == 0;
                        if (desc ? (a0 < a1) : (a0 > a1)) {
                            s_list[idx] = a1;
                            s_list[ixj] = a0;
                        }
                    }
                }
                __syncthreads();
            }
        if (tid == 0) {
            float cum = 0.0f, cut = 0.0f;
            for (int c = 0; c < L && cum < top_p; ++c) {
                cum += s_list[c];
                cut = s_list[c];
            }
            s_cut = cut;
        }
        __syncthreads();
        cutoff = s_cut;
    }

    // draw: thread t owns the contiguous index range [t*per, (t+1)*per)
    const int per = (V + kSampleThreads - 1) / kSampleThreads;
    const int i0 = min(V, tid * per), i1 = min(V, i0 + per);
    float csum = 0.f;
    for (int i = i0; i < i1; ++i) {
        const float p = temp[i];
        csum += (p < cutoff) ? 0.0f : p;
    }
    // inclusive scan of csum over the CTA
    float incl = csum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if ((tid & 31) >= o) incl += t;
    }
    __syncthreads();
    if ((tid & 31) == 31) red[tid >> 5] = incl;
    if (tid == 0) s_chosen = V - 1;
    __syncthreads();
    float wbase = 0.f, total2 = 0.f;
#pragma unroll
    for (int i = 0; i < kSampleThreads / 32; ++i) {
        if (i < (tid >> 5)) wbase += red[i];
        total2 += red[i];
    }
    const float u = u01(seed) * total2;
    float acc = wbase + incl - csum;  // exclusive prefix of this thread's range
    for (int i = i0; i < i1; ++i) {
        const float p = temp[i];
        acc += (p < cutoff) ? 0.0f : p;
        if (acc > u) {
            atomicMin(&s_chosen, i);
            break;
        }
    }
    __syncthreads();
    if (tid == 0) {
        const uint32_t tok = (uint32_t)s_chosen;
        next_tok[ent] = tok;
        if (seq) {
            const int c = seq_cnt[ent];
            if (c < seq_cap) seq[(size_t)ent * seq_cap + c] = tok;
            seq_cnt[ent] = c + 1;
        }
    }
}

// Continuous batching: the input token of row r is either a prompt token supplied by the host or, for a decode
// row (host value 0xFFFFFFFF), the token last generated for the row's session, which never left the GPU.
// Per-session sum of the last layer's residual stream over a step's rows (the accumulation of rwkv_segmean,
// src/backend_cuda.rs:4412-4431: acc += x[t] in token order; the caller divides by the prompt length at the end).  A prompt
// longer than a step continues the same accumulator in the next step, so the order of the additions is the token order.
// Grid (segments, ceil(C / 256)).
__global__ void segment_sums_kernel(const float* __restrict__ x, const float* __restrict__ delta, const SegMeta* __restrict__ segs, int C, float* __restrict__ acc) {
    const SegMeta sg = segs[blockIdx.x];
    const int c = blockIdx.y * 256 + threadIdx.x;
    if (c >= C) return;
    float a = acc[(size_t)sg.slot * C + c];
    for (int t = 0; t < sg.len; ++t) {
        const size_t i = (size_t)(sg.start + t) * C + c;
        a += delta ? x[i] + delta[i] : x[i];
    }
    acc[(size_t)sg.slot * C + c] = a;
}

__global__ void merge_tokens_kernel(const uint32_t* __restrict__ host_tok, const RowMeta* __restrict__ rows, const uint32_t* __restrict__ slot_tok, int R,
                                    uint32_t* __restrict__ tokens) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < R) tokens[r] = host_tok[r] == 0xFFFFFFFFu ? slot_tok[rows[r].slot] : host_tok[r];
}

// Bit-exact int8 container decode to fp32: w = scale*q + zero evaluated in fp32 with separate
// multiply and add, as src/model.rs:234-252 does (rwkv_dequant_int8, src/backend_cuda.rs:4195-4227,
// writes fp16 instead).  Used for the dequant parity check, not on the forward path.
__global__ void dequant_int8_kernel(const uint8_t* __restrict__ idx, const uint32_t* __restrict__ sz, size_t M, size_t K, float* __restrict__ out) {
    const size_t n = M * K;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t m = i / K, kk = i - m * K;
        const uint32_t word = sz[m * (K / 128) + kk / 128];
        const float scale = __half2float(__ushort_as_half((unsigned short)(word & 0xFFFFu)));
        const float zero = __half2float(__ushort_as_half((unsigned short)(word >> 16)));
        out[i] = __fadd_rn(__fmul_rn(scale, (float)idx[i]), zero);
    }
}

// Per-group asymmetric int8 quantiser of the reference's offline tool (quantize_int8_matrix, tools/quantize_any4.py:241-300), group
// = 128 weights of a row: zero = min, scale = (max - min) / 255 (a constant group: scale 0, every q = 0),
// q = clip(rint((w - zero) / scale), 0, 255) with the quotient an IEEE fp32 division and ties to even, as numpy evaluates it; the
// container stores scale and zero as fp16 (round to nearest even), packed zero << 16 | scale.  One warp per group: four weights
// per lane, min and max by shuffles.  Grid-stride over the M * K / 128 groups.
__global__ void quantize_int8_kernel(const float* __restrict__ w, size_t groups, uint8_t* __restrict__ idx, uint32_t* __restrict__ sz) {
    const int lane = threadIdx.x & 31;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t g = warp; g < groups; g += nwarps) {
        const float4 x = reinterpret_cast<const float4*>(w + g * 128)[lane];
        float mn = fminf(fminf(x.x, x.y), fminf(x.z, x.w)), mx = fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        const float span = __fsub_rn(mx, mn);
        const bool flat = span == 0.0f;
        const float scale = __fdiv_rn(flat ? 1.0f : span, 255.0f);
        const float in[4] = {x.x, x.y, x.z, x.w};
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float q = fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(in[j], mn), scale)), 0.0f), 255.0f);
            packed |= (uint32_t)q << (8 * j);
        }
        reinterpret_cast<uint32_t*>(idx + g * 128)[lane] = packed;
        if (lane == 0)
            sz[g] = ((uint32_t)__half_as_ushort(__float2half_rn(mn)) << 16) | (uint32_t)__half_as_ushort(__float2half_rn(flat ? 0.0f : scale));
    }
}

}  // namespace rsv
