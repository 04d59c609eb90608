// Engine implementation: checkpoint loading, HBM layout, work buffers, the packed forward step.
#include "engine.hpp"

#include <algorithm>
#include <cstring>
#include <mutex>

#include "kernels.cuh"
#include "safetensors.hpp"
#include "tc_linear.cuh"
#include "decode_persistent.cuh"
#include "decode_stream_layout.hpp"
#include "wkv_rows.cuh"
#include "wkv_seq.cuh"

namespace rsv {

// ------------------------------------------------------------------------------------------------
// launch bookkeeping: every kernel goes through LAUNCH so that it is counted and, when profiling is
// on, timed with a CUDA event pair on the model's stream (PROF_CUDA_KERNEL in the reference,
// src/backend_cuda.rs:412-460).
// ------------------------------------------------------------------------------------------------
struct LaunchScope {
    Model& m;
    const char* name;
    LaunchScope(Model& m_, const char* n) : m(m_), name(n) {
        if (m.prof_on) cudaEventRecord(m.ev0, m.stream);
    }
    ~LaunchScope() {
        ++m.launches;
        if (m.prof_on) {
            cudaEventRecord(m.ev1, m.stream);
            cudaEventSynchronize(m.ev1);
            float ms = 0.f;
            cudaEventElapsedTime(&ms, m.ev0, m.ev1);
            auto& p = m.prof[name];
            p.ms += ms;
            p.launches += 1;
        }
    }
};
#define LAUNCH(model, name) if (LaunchScope _ls{model, name}; true)

// Launch with the programmatic-stream-serialization attribute: the kernel may be scheduled while its predecessor in the
// stream is still running and synchronises with it through pdl_wait().  Only kernels that call pdl_wait() before they
// touch anything an earlier kernel of the step produces are launched this way.
template <typename... KArgs, typename... Args>
static void launch_pdl(Model& m, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = m.stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = m.use_pdl ? 1 : 0;
    RSV_CUDA(cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...));
}

static void check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) throw CudaError(std::string("kernel launch failed (") + what + "): " + cudaGetErrorString(e));
}

// ------------------------------------------------------------------------------------------------
// loading
// ------------------------------------------------------------------------------------------------
namespace {

std::vector<float> to_f32(const StTensor& t) {
    std::vector<float> out((size_t)t.numel());
    if (t.dtype == "F32") {
        if (t.nbytes != out.size() * 4) throw std::runtime_error("tensor byte size mismatch");
        memcpy(out.data(), t.data, t.nbytes);
    } else if (t.dtype == "F16") {
        if (t.nbytes != out.size() * 2) throw std::runtime_error("tensor byte size mismatch");
        const uint16_t* h = (const uint16_t*)t.data;
        for (size_t i = 0; i < out.size(); ++i) out[i] = half_bits_to_float(h[i]);
    } else {
        throw std::runtime_error("unsupported dtype " + t.dtype + " (need F16 or F32)");  // src/model.rs:208-217
    }
    return out;
}

std::vector<uint16_t> to_f16_bits(const StTensor& t) {
    std::vector<uint16_t> out((size_t)t.numel());
    if (t.dtype == "F16") {
        memcpy(out.data(), t.data, out.size() * 2);
    } else if (t.dtype == "F32") {
        const float* f = (const float*)t.data;
        for (size_t i = 0; i < out.size(); ++i) out[i] = float_to_half_bits(f[i]);
    } else {
        throw std::runtime_error("unsupported dtype " + t.dtype + " (need F16 or F32)");
    }
    return out;
}


// cuTensorMapEncodeTiled is fetched through the runtime so that the library does not link libcuda directly.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        RSV_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        if (!p || q != cudaDriverEntryPointSuccess) throw CudaError("cuTensorMapEncodeTiled is not available in this driver");
        fn = (EncodeTiledFn)p;
    }
    return fn;
}
// 2-D K-major operand [rows, kelems]: box = 128 bytes of K x box_rows rows, 128-byte swizzle.
void encode_kmajor_map(CUtensorMap* map, bool i8, void* base, size_t rows, size_t kelems, int box_rows) {
    const size_t es = i8 ? 1 : 2;
    cuuint64_t dims[2] = {(cuuint64_t)kelems, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(kelems * es)};
    cuuint32_t box[2] = {(cuuint32_t)(kTcKBlockBytes / es), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_tiled_fn()(map, i8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw CudaError("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
}
// All layers' WKV states of a State as one row-major fp32 tensor [rows][64]; box = 32 columns x 64 rows with the 128-byte swizzle.
void encode_state_map(CUtensorMap* map, float* base, size_t rows) {
    cuuint64_t dims[2] = {64, (cuuint64_t)rows};
    cuuint64_t strides[1] = {64 * sizeof(float)};
    cuuint32_t box[2] = {32, 64};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw CudaError("cuTensorMapEncodeTiled (state) failed with code " + std::to_string((int)r));
}
inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Loader {
    Model& m;
    const SafeTensorsFile* st;

    void* dev_alloc(size_t bytes) {
        void* p = nullptr;
        RSV_CUDA(cudaMalloc(&p, std::max<size_t>(bytes, 16)));
        m.allocs.push_back(p);
        m.weight_bytes += bytes;
        return p;
    }
    void* upload(const void* src, size_t bytes) {
        void* p = dev_alloc(bytes);
        RSV_CUDA(cudaMemcpy(p, src, bytes, cudaMemcpyHostToDevice));
        return p;
    }
    float* vec(const std::string& key, size_t expect) {
        std::vector<float> v = to_f32(st->get(key));
        if (v.size() != expect) throw std::runtime_error(key + ": expected " + std::to_string(expect) + " elements, file has " + std::to_string(v.size()));
        return (float*)upload(v.data(), v.size() * 4);
    }
    // [out,in] matrix: int8 pair if `{key}.int8_idx` exists (as src/gpu_model.rs:3438-3441), else fp16.
    LinearW linear(const std::string& key, int M, int K) {
        LinearW L;
        L.M = M;
        L.K = K;
        if (st->has(key + ".int8_idx")) {
            const StTensor& it = st->get(key + ".int8_idx");
            const StTensor& zt = st->get(key + ".int8_sz");
            if (K % 128) throw std::runtime_error(key + ": int8 needs K % 128 == 0");
            if (it.dtype != "U8" || it.nbytes != (size_t)M * K) throw std::runtime_error(key + ".int8_idx: expected U8 [" + std::to_string(M) + "," + std::to_string(K) + "]");
            if (zt.dtype != "U32" || zt.nbytes != (size_t)M * (K / 128) * 4) throw std::runtime_error(key + ".int8_sz: expected U32 [M, K/128]");
            L.wtype = W_INT8;
            L.w = upload(it.data, it.nbytes);
            L.sz = (uint32_t*)upload(zt.data, zt.nbytes);
            prepare_tc_i8(L, (const uint32_t*)zt.data);
        } else {
            const StTensor& t = st->get(key);
            if (t.numel() != (int64_t)M * K) throw std::runtime_error(key + ": shape mismatch");
            if (K % 8) throw std::runtime_error(key + ": fp16 needs K % 8 == 0");
            L.wtype = W_F16;
            if (t.dtype == "F16") {
                L.w = upload(t.data, t.nbytes);
                prepare_tc_f16(L, (const uint16_t*)t.data);
            } else {
                auto h = to_f16_bits(t);
                L.w = upload(h.data(), h.size() * 2);
                prepare_tc_f16(L, h.data());
            }
        }
        return L;
    }
    // int8: the tensor-core path needs one (scale, zero) per output row (all groups of a row equal) and
    // M, K multiples of 128; other files keep tc_ok = false and run on the SIMT kernel.
    void prepare_tc_i8(LinearW& L, const uint32_t* sz_host) {
        const int KG = L.K / 128;
        if (L.M % kTcTileM || L.K % kTcKBlockBytes) return;
        std::vector<float> sc(L.M), zr(L.M);
        for (int m = 0; m < L.M; ++m) {
            const uint32_t w0 = sz_host[(size_t)m * KG];
            for (int g = 1; g < KG; ++g)
                if (sz_host[(size_t)m * KG + g] != w0) return;
            sc[m] = half_bits_to_float((uint16_t)(w0 & 0xFFFFu));
            zr[m] = half_bits_to_float((uint16_t)(w0 >> 16));
        }
        L.wscale = (float*)upload(sc.data(), sc.size() * 4);
        L.wzero = (float*)upload(zr.data(), zr.size() * 4);
        L.Mpad = L.M;
        L.Kpad = L.K;
        L.w_tc = L.w;
        encode_kmajor_map(&L.amap, true, L.w_tc, L.Mpad, L.Kpad, kTcTileM);
        L.tc_ok = true;
    }
    // fp16: zero-pad to [Mpad = ceil128(M), Kpad = ceil64(K)] when the shape needs it (only small matrices do).
    void prepare_tc_f16(LinearW& L, const uint16_t* w_host) {
        L.Mpad = (int)round_up(L.M, kTcTileM);
        L.Kpad = (int)round_up(L.K, 64);
        if (L.Mpad == L.M && L.Kpad == L.K) {
            L.w_tc = L.w;
        } else {
            std::vector<uint16_t> pad((size_t)L.Mpad * L.Kpad, 0);
            for (int m = 0; m < L.M; ++m) memcpy(&pad[(size_t)m * L.Kpad], &w_host[(size_t)m * L.K], (size_t)L.K * 2);
            L.w_tc = upload(pad.data(), pad.size() * 2);
        }
        encode_kmajor_map(&L.amap, false, L.w_tc, L.Mpad, L.Kpad, kTcTileM);
        L.tc_ok = true;
    }
    // Low-rank pair member.  The file holds either [in,out] or [out,in] (src/model.rs:564-581 accepts
    // both, first match wins when in == out); HBM always holds [out,in] fp16.
    LinearW lowrank(const std::string& key, int in_dim, int out_dim) {
        const StTensor& t = st->get(key);
        if (t.shape.size() != 2) throw std::runtime_error(key + ": expected a 2-D tensor");
        std::vector<uint16_t> h = to_f16_bits(t);
        std::vector<uint16_t> oi((size_t)in_dim * out_dim);
        if (t.shape[0] == in_dim && t.shape[1] == out_dim) {
            for (int i = 0; i < in_dim; ++i)
                for (int o = 0; o < out_dim; ++o) oi[(size_t)o * in_dim + i] = h[(size_t)i * out_dim + o];
        } else if (t.shape[0] == out_dim && t.shape[1] == in_dim) {
            oi = h;
        } else {
            throw std::runtime_error(key + ": unexpected shape, want [" + std::to_string(in_dim) + "," + std::to_string(out_dim) + "] or its transpose");
        }
        if (in_dim % 8) throw std::runtime_error(key + ": inner dimension must be a multiple of 8");
        LinearW L;
        L.M = out_dim;
        L.K = in_dim;
        L.wtype = W_F16;
        L.w = upload(oi.data(), oi.size() * 2);
        prepare_tc_f16(L, oi.data());
        return L;
    }
};

}  // namespace

std::unique_ptr<Model> Model::load(const std::string& path, int device) {
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0)
        throw CudaError(std::string("no CUDA device available (") + cudaGetErrorString(e) + "): this library has no CPU fallback");
    if (device < 0 || device >= ndev) throw std::runtime_error("device index out of range");
    RSV_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    RSV_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) throw std::runtime_error("this library is built for sm_100a (B200) only; device is sm_" + std::to_string(prop.major) + std::to_string(prop.minor));

    SafeTensorsFile st(path);
    auto m = std::make_unique<Model>();
    m->device = device;
    Config& c = m->cfg;
    // hyper-parameters come from tensor shapes only (src/gpu_model.rs:406-444)
    int max_layer = -1;
    for (auto& kv : st.tensors()) {
        const std::string& k = kv.first;
        if (k.rfind("blocks.", 0) == 0) {
            size_t p = k.find('.', 7);
            if (p != std::string::npos) {
                bool digits = p > 7;
                for (size_t i = 7; i < p; ++i) digits = digits && k[i] >= '0' && k[i] <= '9';
                if (digits) max_layer = std::max(max_layer, std::stoi(k.substr(7, p - 7)));
            }
        }
    }
    if (max_layer < 0) throw std::runtime_error("no blocks.* tensors in checkpoint");
    c.n_layer = max_layer + 1;
    const StTensor& emb = st.get("emb.weight");
    if (emb.shape.size() != 2) throw std::runtime_error("emb.weight must be 2-D");
    c.vocab = (int)emb.shape[0];
    c.n_embd = (int)emb.shape[1];
    const StTensor& rk = st.get("blocks.0.att.r_k");
    if (rk.shape.size() != 2) throw std::runtime_error("blocks.0.att.r_k must be [H,N]");
    c.n_head = (int)rk.shape[0];
    c.head_size = (int)rk.shape[1];
    auto mid_of = [&](const char* k) {
        const StTensor& t = st.get(k);
        if (t.shape.size() != 2) throw std::runtime_error(std::string(k) + " must be 2-D");
        return (int)(t.shape[0] == c.n_embd ? t.shape[1] : t.shape[0]);
    };
    c.w_mid = mid_of("blocks.0.att.w1");
    c.a_mid = mid_of("blocks.0.att.a1");
    c.v_mid = mid_of("blocks.0.att.v1");
    c.g_mid = mid_of("blocks.0.att.g1");
    c.ffn_hidden = (int)(st.has("blocks.0.ffn.key.weight") ? st.get("blocks.0.ffn.key.weight").shape.at(0)
                                                            : st.get("blocks.0.ffn.key.weight.int8_idx").shape.at(0));
    if (c.head_size != kHeadSize) throw std::runtime_error("head_size must be 64");
    if (c.n_head * c.head_size != c.n_embd) throw std::runtime_error("n_head * head_size != n_embd");
    if (c.n_embd % 8 || c.ffn_hidden % 8) throw std::runtime_error("n_embd and ffn_hidden must be multiples of 8");

    m->num_sms = prop.multiProcessorCount;
    if (const char* e = getenv("RSV_NO_PERSISTENT"))
        if (*e && *e != '0') m->use_persistent = false;
    if (const char* e = getenv("RSV_NO_STREAM"))
        if (*e && *e != '0') m->use_stream = false;
    if (const char* e = getenv("RSV_NO_GRAPH"))
        if (*e && *e != '0') m->use_graphs = false;
    if (const char* e = getenv("RSV_NO_PDL"))
        if (*e && *e != '0') m->use_pdl = false;
    RSV_CUDA(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
    RSV_CUDA(cudaEventCreate(&m->ev0));
    RSV_CUDA(cudaEventCreate(&m->ev1));
    RSV_CUDA(cudaEventCreate(&m->tev[0]));
    RSV_CUDA(cudaEventCreate(&m->tev[1]));

    Loader ld{*m, &st};
    const int C = c.n_embd, F = c.ffn_hidden;
    {
        auto h = to_f16_bits(emb);
        m->emb = (__half*)ld.upload(h.data(), h.size() * 2);
    }
    m->ln0_w = ld.vec("blocks.0.ln0.weight", C);
    m->ln0_b = ld.vec("blocks.0.ln0.bias", C);
    m->ln_out_w = ld.vec("ln_out.weight", C);
    m->ln_out_b = ld.vec("ln_out.bias", C);
    m->head = ld.linear("head.weight", c.vocab, C);
    m->layers.resize(c.n_layer);
    for (int i = 0; i < c.n_layer; ++i) {
        const std::string p = "blocks." + std::to_string(i) + ".";
        LayerW& L = m->layers[i];
        L.ln1_w = ld.vec(p + "ln1.weight", C);
        L.ln1_b = ld.vec(p + "ln1.bias", C);
        L.ln2_w = ld.vec(p + "ln2.weight", C);
        L.ln2_b = ld.vec(p + "ln2.bias", C);
        L.lnx_w = ld.vec(p + "att.ln_x.weight", C);
        L.lnx_b = ld.vec(p + "att.ln_x.bias", C);
        L.x_r = ld.vec(p + "att.x_r", C);
        L.x_w = ld.vec(p + "att.x_w", C);
        L.x_k = ld.vec(p + "att.x_k", C);
        L.x_v = ld.vec(p + "att.x_v", C);
        L.x_a = ld.vec(p + "att.x_a", C);
        L.x_g = ld.vec(p + "att.x_g", C);
        L.ffn_x_k = ld.vec(p + "ffn.x_k", C);
        L.w0 = ld.vec(p + "att.w0", C);
        L.a0 = ld.vec(p + "att.a0", C);
        L.v0 = ld.vec(p + "att.v0", C);
        L.r_k = ld.vec(p + "att.r_k", C);
        L.k_k = ld.vec(p + "att.k_k", C);
        L.k_a = ld.vec(p + "att.k_a", C);
        L.Wr = ld.linear(p + "att.receptance.weight", C, C);
        L.Wk = ld.linear(p + "att.key.weight", C, C);
        L.Wv = ld.linear(p + "att.value.weight", C, C);
        L.Wo = ld.linear(p + "att.output.weight", C, C);
        L.Wfk = ld.linear(p + "ffn.key.weight", F, C);
        L.Wfv = ld.linear(p + "ffn.value.weight", C, F);
        L.w1 = ld.lowrank(p + "att.w1", C, c.w_mid);
        L.w2 = ld.lowrank(p + "att.w2", c.w_mid, C);
        L.a1 = ld.lowrank(p + "att.a1", C, c.a_mid);
        L.a2 = ld.lowrank(p + "att.a2", c.a_mid, C);
        L.v1 = ld.lowrank(p + "att.v1", C, c.v_mid);
        L.v2 = ld.lowrank(p + "att.v2", c.v_mid, C);
        L.g1 = ld.lowrank(p + "att.g1", C, c.g_mid);
        L.g2 = ld.lowrank(p + "att.g2", c.g_mid, C);
    }
    m->pinned_bytes = 1 << 18;
    RSV_CUDA(cudaMallocHost(&m->pinned, m->pinned_bytes * Model::kPinRing));
    for (int i = 0; i < Model::kPinRing; ++i) RSV_CUDA(cudaEventCreateWithFlags(&m->pin_ev[i], cudaEventDisableTiming));
    RSV_CUDA(cudaMalloc(&m->ws.status, 2 * sizeof(int)));
    RSV_CUDA(cudaMalloc(&m->ws.tok_pos, sizeof(int)));
    RSV_CUDA(cudaMemsetAsync(m->ws.status, 0, 2 * sizeof(int), m->stream));
    RSV_CUDA(cudaMemsetAsync(m->ws.tok_pos, 0, sizeof(int), m->stream));
    return m;
}

std::unique_ptr<Model> Model::create_bare(int device) {
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0)
        throw CudaError(std::string("no CUDA device available (") + cudaGetErrorString(e) + "): this library has no CPU fallback");
    if (device < 0 || device >= ndev) throw std::runtime_error("device index out of range");
    RSV_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    RSV_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) throw std::runtime_error("this library is built for sm_100a (B200) only");
    auto m = std::make_unique<Model>();
    m->device = device;
    m->num_sms = prop.multiProcessorCount;
    RSV_CUDA(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
    RSV_CUDA(cudaEventCreate(&m->ev0));
    RSV_CUDA(cudaEventCreate(&m->ev1));
    RSV_CUDA(cudaEventCreate(&m->tev[0]));
    RSV_CUDA(cudaEventCreate(&m->tev[1]));
    RSV_CUDA(cudaMalloc(&m->ws.status, 2 * sizeof(int)));
    RSV_CUDA(cudaMemsetAsync(m->ws.status, 0, 2 * sizeof(int), m->stream));
    return m;
}

static void free_workspace(Workspace& w) {
    void* ptrs[] = {w.x, w.x2, w.delta, w.xmix, w.r, w.k, w.v, w.w, w.a, w.g, w.yg, w.xb, w.mid, w.h, w.vfirst, w.xn, w.logits, w.staging, w.tokens, w.row_meta, w.seg_meta, w.out_rows, w.samp_temp, w.samp_cnt};
    for (void* p : ptrs)
        if (p) cudaFree(p);
    int* status = w.status;
    int* pos = w.tok_pos;
    Workspace keep = w;
    w = Workspace{};
    w.status = status;
    w.tok_pos = pos;
    w.tok_list = keep.tok_list;
    w.tok_list_cap = keep.tok_list_cap;
    w.tc_b = keep.tc_b;
    w.tc_b_bytes = keep.tc_b_bytes;
    w.tc_xscale = keep.tc_xscale;
    w.tc_tsum = keep.tc_tsum;
    w.tc_rows = keep.tc_rows;
    w.tc_partials = keep.tc_partials;
    w.tc_cnt = keep.tc_cnt;
    w.tc_partials_bytes = keep.tc_partials_bytes;
}

Model::~Model() {
    cudaSetDevice(device);
    if (stream) cudaStreamSynchronize(stream);
    free_workspace(ws);
    if (ws.status) cudaFree(ws.status);
    if (ws.tok_pos) cudaFree(ws.tok_pos);
    if (ws.tok_list) cudaFree(ws.tok_list);
    for (void* p : allocs) cudaFree(p);
    for (void* p : {(void*)ws.tc_b, (void*)ws.tc_xscale, (void*)ws.tc_tsum, ws.tc_partials, (void*)ws.tc_cnt})
        if (p) cudaFree(p);
    for (void* p : {pctx.d_layers, pctx.d_maps, (void*)pctx.x, (void*)pctx.yg, (void*)pctx.vfirst, (void*)pctx.cand_val, (void*)pctx.cand_idx, (void*)pctx.rkv, (void*)pctx.mid, (void*)pctx.hbuf,
                    (void*)pctx.grid_bar})
        if (p) cudaFree(p);
    for (void* p : {sctx.d_layers, sctx.wstream, sctx.hstream, (void*)sctx.x, (void*)sctx.yg, (void*)sctx.vfirst, (void*)sctx.rkv, (void*)sctx.mid, (void*)sctx.hbuf, (void*)sctx.cand_val,
                    (void*)sctx.cand_idx, (void*)sctx.grid_bar, (void*)sctx.dbg})
        if (p) cudaFree(p);
    for (int i = 0; i < 5; ++i) {
        if (pctx.region_data[i]) cudaFree(pctx.region_data[i]);
        if (pctx.region_meta[i]) cudaFree(pctx.region_meta[i]);
        if (pctx.region_cnt[i]) cudaFree(pctx.region_cnt[i]);
    }
    if (pinned) cudaFreeHost(pinned);
    for (int i = 0; i < kPinRing; ++i)
        if (pin_ev[i]) cudaEventDestroy(pin_ev[i]);
    if (ev0) cudaEventDestroy(ev0);
    if (ev1) cudaEventDestroy(ev1);
    if (tev[0]) cudaEventDestroy(tev[0]);
    if (tev[1]) cudaEventDestroy(tev[1]);
    if (stream) cudaStreamDestroy(stream);
}

State::~State() {
    if (model) {
        cudaSetDevice(model->device);
        // the persistent kernel's device layer table may point into this state: a later state that cudaMalloc places at the
        // same addresses (with another batch, hence other per-layer strides) must not be taken for it
        if (model->pctx.bound_tmix == tmix_x) {
            model->pctx.bound_tmix = model->pctx.bound_wkv = model->pctx.bound_cmix = nullptr;
            model->pctx.bound_cap = -1;
        }
    }
    for (float* p : {tmix_x, wkv, cmix_x, v_first})
        if (p) cudaFree(p);
}

void Model::ensure_workspace(int rows, int outs, int segs) {
    if (rows <= ws.rows && outs <= ws.outs && segs <= ws.segs) return;
    RSV_CUDA(cudaStreamSynchronize(stream));
    // Growing frees and reallocates every array (each a device synchronisation), so a dimension that grows a second time gets
    // a quarter of slack: a server whose step size creeps up reallocates a few times, not at every new maximum.
    auto grow = [](int want, int have) { return want <= have ? have : (have > 1 ? want + want / 4 : want); };
    rows = grow(rows, ws.rows);
    outs = grow(outs, ws.outs);
    segs = grow(segs, ws.segs);
    free_workspace(ws);
    const size_t C = cfg.n_embd, F = cfg.ffn_hidden, V = cfg.vocab, R = rows;
    auto fa = [&](float*& p, size_t n) { RSV_CUDA(cudaMalloc(&p, std::max<size_t>(n, 4) * sizeof(float))); };
    fa(ws.x, R * C);
    fa(ws.x2, R * C);
    fa(ws.delta, R * C);
    fa(ws.xmix, 6 * R * C);
    fa(ws.r, R * C);
    fa(ws.k, R * C);
    fa(ws.v, R * C);
    fa(ws.w, R * C);
    fa(ws.a, R * C);
    fa(ws.g, R * C);
    fa(ws.yg, R * C);
    fa(ws.xb, R * C);
    fa(ws.mid, R * (size_t)cfg.mids());
    fa(ws.h, R * F);
    fa(ws.vfirst, R * C);
    fa(ws.xn, (size_t)outs * C);
    fa(ws.logits, (size_t)outs * V);
    fa(ws.staging, (size_t)segs * C);
    fa(ws.samp_temp, (size_t)outs * V);
    RSV_CUDA(cudaMalloc(&ws.samp_cnt, std::max<size_t>((size_t)outs * V, 4) * sizeof(uint32_t)));
    RSV_CUDA(cudaMalloc(&ws.tokens, R * sizeof(uint32_t)));
    RSV_CUDA(cudaMemsetAsync(ws.tokens, 0, R * sizeof(uint32_t), stream));
    RSV_CUDA(cudaMalloc(&ws.row_meta, R * sizeof(RowMeta)));
    RSV_CUDA(cudaMalloc(&ws.seg_meta, (size_t)segs * sizeof(SegMeta)));
    RSV_CUDA(cudaMalloc(&ws.out_rows, (size_t)std::max(outs, 1) * sizeof(int)));
    ws.rows = rows;
    ws.outs = outs;
    ws.segs = segs;
    const size_t need = R * sizeof(RowMeta) + (size_t)segs * sizeof(SegMeta) + (size_t)outs * sizeof(int) + R * sizeof(uint32_t) + 256;
    if (need > pinned_bytes) {
        cudaFreeHost(pinned);
        pinned = nullptr;
        pinned_bytes = need * 2;
        RSV_CUDA(cudaMallocHost(&pinned, pinned_bytes * kPinRing));
    }
}

void Model::upload_plan(const StepPlan& plan) {
    const int R = (int)plan.rows.size(), S = (int)plan.segs.size(), O = (int)plan.out_rows.size();
    ensure_workspace(R, std::max(O, 1), S);
    // next area of the staging ring; its previous copies (kPinRing uploads ago) must have completed
    const int slot = pin_next;
    pin_next = (pin_next + 1) % kPinRing;
    if (pin_ev[slot]) RSV_CUDA(cudaEventSynchronize(pin_ev[slot]));
    char* p = (char*)pinned + (size_t)slot * pinned_bytes;
    memcpy(p, plan.rows.data(), R * sizeof(RowMeta));
    RSV_CUDA(cudaMemcpyAsync(ws.row_meta, p, R * sizeof(RowMeta), cudaMemcpyHostToDevice, stream));
    p += R * sizeof(RowMeta);
    memcpy(p, plan.segs.data(), S * sizeof(SegMeta));
    RSV_CUDA(cudaMemcpyAsync(ws.seg_meta, p, S * sizeof(SegMeta), cudaMemcpyHostToDevice, stream));
    p += S * sizeof(SegMeta);
    if (O) {
        memcpy(p, plan.out_rows.data(), O * sizeof(int));
        RSV_CUDA(cudaMemcpyAsync(ws.out_rows, p, O * sizeof(int), cudaMemcpyHostToDevice, stream));
    }
    if (pin_ev[slot]) RSV_CUDA(cudaEventRecord(pin_ev[slot], stream));
}

// ------------------------------------------------------------------------------------------------
// linear launch helper
// ------------------------------------------------------------------------------------------------
namespace {

struct LinReq {
    const LinearW* W;
    const float* x;
    int ldx;
    float* y;
    int ldy;
    int epi;
    const float* bias = nullptr;
    const float* aux = nullptr;
    int ldaux = 0;
    float* y2 = nullptr;
};

template <int RT>
void launch_linear_rt(Model& m, const LinGroup& g, int nblk, int R, size_t smem) {
    static bool configured[8] = {false};
    int dev = m.device & 7;
    if (!configured[dev]) {
        RSV_CUDA(cudaFuncSetAttribute(linear_rows_kernel<RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured[dev] = true;
    }
    dim3 grid(nblk, (R + RT - 1) / RT);
    linear_rows_kernel<RT><<<grid, kLinWarps * 32, smem, m.stream>>>(g, R);
    check_launch("linear_rows");
}

void run_linear_simt(Model& m, const char* name, const LinReq* reqs, int n, int R) {
    LinGroup g;
    memset(&g, 0, sizeof(g));
    g.n = n;
    int total_rows = 0, kmax = 0;
    bool any_i8 = false;
    for (int i = 0; i < n; ++i) {
        total_rows += reqs[i].W->M;
        kmax = std::max(kmax, reqs[i].W->K);
        any_i8 = any_i8 || reqs[i].W->wtype == W_INT8;
    }
    // rows per CTA: aim for a few waves over 148 SMs, but amortise the x staging
    const int unit = kLinWarps * kLinWR;
    int rpb = (total_rows / (148 * 4)) / unit * unit;
    rpb = std::min(std::max(rpb, unit), 8 * unit);
    int blk = 0;
    for (int i = 0; i < n; ++i) {
        const LinReq& q = reqs[i];
        LinProb& P = g.p[i];
        P.w = q.W->w;
        P.sz = q.W->sz;
        P.x = q.x;
        P.y = q.y;
        P.y2 = q.y2;
        P.bias = q.bias;
        P.aux = q.aux;
        P.M = q.W->M;
        P.K = q.W->K;
        P.ldx = q.ldx;
        P.ldy = q.ldy;
        P.ldaux = q.ldaux;
        P.wtype = q.W->wtype;
        P.epi = q.epi;
        P.rows_per_blk = rpb;
        P.blk0 = blk;
        blk += (P.M + rpb - 1) / rpb;
    }
    auto smem_for = [&](int rt) { return (size_t)rt * kmax * 4 + (any_i8 ? (size_t)rt * (kmax / 16) * 4 : 0); };
    int rt = R >= 4 ? 4 : (R >= 2 ? 2 : 1);
    while (rt > 1 && smem_for(rt) > 200 * 1024) rt >>= 1;
    if (smem_for(rt) > 200 * 1024) throw std::runtime_error("linear: inner dimension too large for the shared-memory tile");
    LAUNCH(m, name) {
        if (rt == 4)
            launch_linear_rt<4>(m, g, blk, R, smem_for(4));
        else if (rt == 2)
            launch_linear_rt<2>(m, g, blk, R, smem_for(2));
        else
            launch_linear_rt<1>(m, g, blk, R, smem_for(1));
    }
}


// ---- tensor-core path ---------------------------------------------------------------------------
void ensure_tc_buffers(Model& m, size_t b_bytes, size_t rows, size_t partial_bytes) {
    Workspace& w = m.ws;
    if (!w.tc_cnt) {
        RSV_CUDA(cudaMalloc(&w.tc_cnt, (size_t)kTcMaxSplit * kTcEpiWarps * sizeof(int)));
        RSV_CUDA(cudaMemsetAsync(w.tc_cnt, 0, (size_t)kTcMaxSplit * kTcEpiWarps * sizeof(int), m.stream));
    }
    if (b_bytes <= w.tc_b_bytes && rows <= w.tc_rows && partial_bytes <= w.tc_partials_bytes) return;
    RSV_CUDA(cudaStreamSynchronize(m.stream));
    if (b_bytes > w.tc_b_bytes) {
        if (w.tc_b) cudaFree(w.tc_b);
        w.tc_b = nullptr;
        w.tc_b_bytes = 0;
        const size_t nb = b_bytes + b_bytes / 4;
        RSV_CUDA(cudaMalloc(&w.tc_b, nb));
        RSV_CUDA(cudaMemsetAsync(w.tc_b, 0, nb, m.stream));
        w.tc_b_bytes = nb;
    }
    if (rows > w.tc_rows) {
        if (w.tc_xscale) cudaFree(w.tc_xscale);
        if (w.tc_tsum) cudaFree(w.tc_tsum);
        w.tc_xscale = nullptr;
        w.tc_tsum = nullptr;
        w.tc_rows = 0;
        const size_t nr = rows + rows / 4;
        RSV_CUDA(cudaMalloc(&w.tc_xscale, nr * sizeof(float)));
        RSV_CUDA(cudaMalloc(&w.tc_tsum, nr * sizeof(long long)));
        w.tc_rows = nr;
    }
    if (partial_bytes > w.tc_partials_bytes) {
        if (w.tc_partials) cudaFree(w.tc_partials);
        w.tc_partials = nullptr;
        w.tc_partials_bytes = 0;
        const size_t np = partial_bytes + partial_bytes / 4;
        RSV_CUDA(cudaMalloc(&w.tc_partials, np));
        w.tc_partials_bytes = np;
    }
}

constexpr int kTcDigits = 4;  // base-128 digits of the fixed-point activations (P = 27 bits)

// One launch group of the tensor-core path: all requests share the weight kind (int8 or fp16).  A stage of a layer has up to
// two groups; their activation operands are prepared by one launch, then each group's GEMM is launched.
struct TcRegion {
    const float* x;
    int ldx, K, Kpad;
    size_t off;  // bytes from the group's base in the operand buffer
    int row0;    // first scale / sum row of the region inside the group
};
struct TcGroup {
    bool i8 = false;
    int n = 0, R = 0, D = 0, ncols = 0, NT = 0, ncols_pad = 0, rows = 0, U = 0, G = 0;
    LinReq reqs[kTcMaxProblems];
    std::vector<TcRegion> regions;
    int region_of[kTcMaxProblems];
    size_t b_bytes = 0, b_base = 0, partial_bytes = 0;
    int row_base = 0;
    TcLaunch L;
};

void tc_plan_group(Model& m, TcGroup& g) {
    const bool i8 = g.i8;
    const int n = g.n, R = g.R;
    g.D = i8 ? kTcDigits : 2;
    g.ncols = R * g.D;
    g.NT = 16;
    while (g.NT < g.ncols && g.NT < 256) g.NT <<= 1;
    g.ncols_pad = (int)round_up(g.ncols, g.NT);
    const size_t es = i8 ? 1 : 2;
    // B operand regions (requests that read the same activations share one)
    for (int i = 0; i < n; ++i) {
        const LinearW& W = *g.reqs[i].W;
        int found = -1;
        for (size_t j = 0; j < g.regions.size(); ++j)
            if (g.regions[j].x == g.reqs[i].x && g.regions[j].K == W.K && g.regions[j].Kpad == W.Kpad && g.regions[j].ldx == g.reqs[i].ldx) found = (int)j;
        if (found < 0) {
            g.regions.push_back(TcRegion{g.reqs[i].x, g.reqs[i].ldx, W.K, W.Kpad, g.b_bytes, g.rows});
            found = (int)g.regions.size() - 1;
            g.b_bytes += round_up((size_t)g.ncols_pad * W.Kpad * es, 1024);
            g.rows += R;
        }
        g.region_of[i] = found;
    }
    // units, tiles, CTA count
    TcLaunch& L = g.L;
    memset(&L, 0, sizeof(L));
    int U = 0, T = 0;
    const int n_tiles = g.ncols_pad / g.NT;
    for (int i = 0; i < n; ++i) {
        const LinearW& W = *g.reqs[i].W;
        TcProb& P = L.p[i];
        P.M = W.M;
        P.kblocks = (int)((size_t)W.Kpad * es / kTcKBlockBytes);
        P.ncols = g.ncols;
        P.n_tiles = n_tiles;
        P.unit0 = U;
        P.tile0 = T;
        const int mtiles = W.Mpad / kTcTileM;
        U += mtiles * n_tiles * P.kblocks;
        T += mtiles * n_tiles;
        L.amap[i] = W.amap;
    }
    // CTA count.  A tile cut between CTAs costs a partial-sum round trip through global memory and a serial sum over its
    // pieces, which at few rows outweighs the idle SMs: a CTA gets about a K = 2560 int8 tile's worth of K blocks (20), and the
    // piece length divides the shortest tile of the group, so that cuts fall on tile boundaries or split a tile evenly
    // (3B shape, 64 rows: 7.4 -> 5.7 ms per step against one unit range per SM).
    int kb_min = L.p[0].kblocks;
    for (int i = 1; i < n; ++i) kb_min = std::min(kb_min, L.p[i].kblocks);
    int upc = kb_min;
    while (upc > 30 && upc % 2 == 0) upc /= 2;  // K = 10240 tiles (80 K blocks) in four pieces: measured best of 1, 2, 4, 8
    int G = std::min(m.num_sms, std::max(1, U / upc));
    // Short reductions (the rank back-projections: 1-5 K blocks per tile), where a cut tile's partial-sum round trip is longer
    // than the tile itself, and launches with at least a tile per SM (many rows): CTAs get whole tiles, balanced by their K
    // blocks, and no tile is cut (256 rows: 10.9 -> 10.4 ms per step; 512-row prefill chunks 2 % faster).
    int kb_max = 0;
    for (int i = 0; i < n; ++i) kb_max = std::max(kb_max, L.p[i].kblocks);
    const bool snap = (kb_max <= 8 || T >= m.num_sms) && std::min(m.num_sms, T) + 1 <= kTcMaxSplit;
    if (snap) {
        G = std::min(m.num_sms, T);
        std::vector<int> tk;
        tk.reserve((size_t)T);
        for (int i = 0; i < n; ++i)
            for (int t = (i + 1 < n ? L.p[i + 1].tile0 : T) - L.p[i].tile0; t > 0; --t) tk.push_back(L.p[i].kblocks);
        int ti = 0, u = 0;
        for (int c = 0; c < G; ++c) {
            L.split_unit[c] = u;
            const int left = G - c;  // CTAs still to be served, this one included: each gets at least one tile
            const double target = (double)(U - u) / left;
            int taken = 0;
            while (ti < T && T - ti > left - 1) {
                if (taken > 0 && taken + 0.5 * tk[ti] > target) break;
                taken += tk[ti++];
            }
            u += taken;
        }
        if (u != U || ti != T) throw std::runtime_error("tc_linear: tile assignment does not cover the launch");
        L.split_unit[G] = U;
        L.snap = 1;
    }
    // tiles cut by a CTA boundary keep partial sums; the epilogue warp that arrives last on a sub-block finishes it
    int pmax = 1, nsplit = 0;
    for (int c = 1; c < G && !snap; ++c) {
        const int bnd = tc_cta_begin(c, U, G);
        int pi = 0;
        while (pi + 1 < n && bnd >= L.p[pi + 1].unit0) ++pi;
        const TcProb& P = L.p[pi];
        const int local = bnd - P.unit0;
        if (local % P.kblocks == 0) continue;  // boundary falls between tiles
        const int tile_first = bnd - local % P.kblocks;
        if (nsplit > 0 && L.split_unit[nsplit - 1] == tile_first) {
            // same tile cut again
        } else {
            if (nsplit >= kTcMaxSplit) throw std::runtime_error("tc_linear: too many split tiles");
            L.split_unit[nsplit++] = tile_first;
        }
        pmax = std::max(pmax, tc_cta_of_unit(tile_first + P.kblocks - 1, U, G) - tc_cta_of_unit(tile_first, U, G) + 1);
    }
    g.partial_bytes = (size_t)nsplit * pmax * g.NT * kTcTileM * 4;
    g.U = U;
    g.G = G;
    L.nprob = n;
    L.total_units = U;
    L.nt = g.NT;
    L.is_i8 = i8;
    L.pmax = pmax;
    L.grid = G;
    L.nsplit = nsplit;
}

void tc_launch_group(Model& m, const char* name, TcGroup& g) {
    Workspace& w = m.ws;
    TcLaunch& L = g.L;
    for (int i = 0; i < g.n; ++i) {
        const TcRegion& rg = g.regions[g.region_of[i]];
        const LinReq& q = g.reqs[i];
        encode_kmajor_map(&L.bmap[i], g.i8, w.tc_b + g.b_base + rg.off, g.ncols_pad, rg.Kpad, g.NT);
        TcProb& P = L.p[i];
        P.R = g.R;
        P.D = g.D;
        P.wscale = q.W->wscale;
        P.wzero = q.W->wzero;
        P.xscale = w.tc_xscale + g.row_base + rg.row0;
        P.tsum = w.tc_tsum + g.row_base + rg.row0;
        P.y = q.y;
        P.y2 = q.y2;
        P.bias = q.bias;
        P.aux = q.aux;
        P.ldy = q.ldy;
        P.ldaux = q.ldaux;
        P.epi = q.epi;
    }
    const size_t stage_bytes = (size_t)kTcTileM * kTcKBlockBytes + (size_t)g.NT * kTcKBlockBytes;
    L.nstages = (int)std::min<size_t>(8, (200 * 1024) / stage_bytes);
    L.partials = w.tc_partials;
    L.tile_cnt = w.tc_cnt;
    L.status = w.status;
    const size_t smem = (size_t)L.nstages * stage_bytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
    static bool configured[16] = {false};
    if (!configured[m.device & 15]) {
        RSV_CUDA(cudaFuncSetAttribute(tc_linear_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        RSV_CUDA(cudaFuncSetAttribute(tc_linear_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        configured[m.device & 15] = true;
    }
    LAUNCH(m, name) {
        if (g.i8)
            launch_pdl(m, tc_linear_kernel<true>, dim3(g.G), dim3(kTcThreads), smem, L);
        else
            launch_pdl(m, tc_linear_kernel<false>, dim3(g.G), dim3(kTcThreads), smem, L);
        check_launch("tc_linear");
    }
}

void run_linear_tc(Model& m, const char* name, const LinReq* reqs, int n, int R) {
    TcGroup ga, gb;
    ga.i8 = true;
    gb.i8 = false;
    ga.R = gb.R = R;
    for (int i = 0; i < n; ++i) {
        TcGroup& g = reqs[i].W->wtype == W_INT8 ? ga : gb;
        if (g.n >= kTcMaxProblems) throw std::runtime_error("tc_linear: too many problems in one group");
        g.reqs[g.n++] = reqs[i];
    }
    if (ga.n) tc_plan_group(m, ga);
    if (gb.n) tc_plan_group(m, gb);
    gb.b_base = ga.b_bytes;  // the fp16 group's operands follow the int8 group's
    gb.row_base = ga.rows;
    if (ga.regions.size() + gb.regions.size() > (size_t)kTcMaxRegions) throw std::runtime_error("tc_linear: too many operand regions");
    ensure_tc_buffers(m, ga.b_bytes + gb.b_bytes, (size_t)(ga.rows + gb.rows), std::max(ga.partial_bytes, gb.partial_bytes));
    Workspace& w = m.ws;
    // operand preparation: one launch for every activation operand of the stage
    {
        TcPrepLaunch PL;
        memset(&PL, 0, sizeof(PL));
        int nr = 0;
        for (TcGroup* g : {&ga, &gb})
            for (const TcRegion& rg : g->regions)
                PL.r[nr++] = TcPrepRegion{rg.x, w.tc_b + g->b_base + rg.off, w.tc_xscale + g->row_base + rg.row0, w.tc_tsum + g->row_base + rg.row0,
                                          rg.ldx, rg.K, rg.Kpad, g->i8 ? 1 : 0};
        LAUNCH(m, "tc_prepare") {
            const dim3 grid(R, (unsigned)nr);
            const dim3 block((size_t)R * nr < 2 * (size_t)m.num_sms ? kPrepThreadsWide : kPrepThreads);
            launch_pdl(m, tc_prepare_kernel<kTcDigits>, grid, block, 0, PL);
            check_launch("tc_prepare");
        }
    }
    std::string nm = std::string(name) + "_tc";
    if (ga.n) tc_launch_group(m, nm.c_str(), ga);
    if (gb.n) tc_launch_group(m, nm.c_str(), gb);
}

void run_linear(Model& m, const char* name, const LinReq* reqs, int n, int R) {
    bool tc = R >= m.tc_min_rows;
    for (int i = 0; i < n; ++i) tc = tc && reqs[i].W->tc_ok;
    if (!tc) return run_linear_simt(m, name, reqs, n, R);
    run_linear_tc(m, name, reqs, n, R);
}
}  // namespace

// ------------------------------------------------------------------------------------------------
// the packed forward step (one token per row), Appendix-style data flow of src/model.rs:396-516
// ------------------------------------------------------------------------------------------------
void Model::forward_rows(State& st, const StepPlan& plan, bool use_cursor) {
    const int R = (int)plan.rows.size(), S = (int)plan.segs.size(), O = (int)plan.out_rows.size();
    const int C = cfg.n_embd, H = cfg.n_head, F = cfg.ffn_hidden, V = cfg.vocab, MIDS = cfg.mids();
    if (R == 0) return;
    RSV_CUDA(cudaSetDevice(device));
    const size_t RC = (size_t)R * C;
    float* xm[6];
    for (int i = 0; i < 6; ++i) xm[i] = ws.xmix + i * RC;  // order: r, w, k, v, a, g
    float* staging = plan.multi_row_segments ? ws.staging : nullptr;

    LAUNCH(*this, "embed_ln0") {
        embed_ln0_kernel<<<R, kRowThreads, 0, stream>>>(emb, ln0_w, ln0_b, use_cursor ? ws.tok_list : ws.tokens, use_cursor ? ws.tok_pos : nullptr, R, C, V,
                                                        ws.x, ws.status);
        check_launch("embed_ln0");
    }
    // The residual stream ping-pongs between two buffers: each LayerNorm kernel folds in the pending residual of the
    // linear layer before it (x_cur + pending -> x_alt) so that no linear epilogue has to read-modify-write x.
    float *x_cur = ws.x, *x_alt = ws.x2;
    const float* pending = nullptr;
    // few rows: several CTAs share a row of the LayerNorm + shift kernels (each recomputes the row statistics, then handles a
    // slice of the channels), so that the step's latency does not hang on R single CTAs
    // (a thread's channels are handled one after the other, each a dependent round of loads: five CTAs per row keep that to two rounds)
    const int ln_split = std::max(R <= 512 ? 5 : 1, std::min(10, (2 * num_sms) / std::max(R, 1)));
    const size_t lay_x = (size_t)st.cap * C, lay_s = (size_t)st.cap * H * kHeadSize * kHeadSize;
    for (int l = 0; l < cfg.n_layer; ++l) {
        const LayerW& L = layers[l];
        float* tmix_x = st.tmix_x + l * lay_x;
        float* cmix_x = st.cmix_x + l * lay_x;
        float* wkv = st.wkv + l * lay_s;
        LAUNCH(*this, "ln_shift6") {
            MixPtrs mp{{L.x_r, L.x_w, L.x_k, L.x_v, L.x_a, L.x_g}};
            launch_pdl(*this, ln_shift_kernel<6>, dim3(R, ln_split), dim3(kRowThreads), 0, x_cur, pending, x_alt, L.ln1_w, L.ln1_b, mp, ws.row_meta, R, C, tmix_x, staging, ws.xmix);
            check_launch("ln_shift6");
        }
        if (pending) {
            std::swap(x_cur, x_alt);
            pending = nullptr;
        }
        if (staging) LAUNCH(*this, "commit_shift") {
                launch_pdl(*this, commit_shift_kernel, dim3(S), dim3(256), 0, staging, ws.seg_meta, C, tmix_x);
                check_launch("commit_shift");
            }
        float* vgate = l == 0 ? nullptr : ws.xb;  // xb is free until ln_shift1
        {
            // r, k, v and the four rank-space projections in one launch
            float* mw = ws.mid;
            float* ma = mw + cfg.w_mid;
            float* mv = ma + cfg.a_mid;
            float* mg = mv + cfg.v_mid;
            LinReq q[7] = {
                {&L.Wr, xm[0], C, ws.r, C, EPI_STORE},
                {&L.Wk, xm[2], C, ws.k, C, EPI_STORE},
                {&L.Wv, xm[3], C, ws.v, C, EPI_STORE, nullptr, nullptr, 0, l == 0 ? ws.vfirst : nullptr},
                {&L.w1, xm[1], C, mw, MIDS, EPI_TANH},
                {&L.a1, xm[4], C, ma, MIDS, EPI_STORE},
                {&L.g1, xm[5], C, mg, MIDS, EPI_SIGMOID},
                {&L.v1, xm[3], C, mv, MIDS, EPI_STORE},
            };
            run_linear(*this, "linear_rkv_rank", q, l == 0 ? 6 : 7, R);
            // back-projections: decay w, a, gate g and (layers > 0) the v-lerp gate; all plain stores
            LinReq q2[4] = {
                {&L.w2, mw, MIDS, ws.w, C, EPI_DECAY, L.w0},
                {&L.a2, ma, MIDS, ws.a, C, EPI_SIGMOID_BIAS, L.a0},
                {&L.g2, mg, MIDS, ws.g, C, EPI_STORE},
                {&L.v2, mv, MIDS, vgate, C, EPI_SIGMOID_BIAS, L.v0},
            };
            run_linear(*this, "linear_rank_back", q2, l == 0 ? 3 : 4, R);
        }
        LAUNCH(*this, "wkv7") {
            const int n_items = H * S;
            if (plan.multi_row_segments) {
                // prefill chunks: vectors built by preparation warps, only state-dependent work in the per-token chain (wkv_seq.cuh)
// few (head, segment) pairs: a head over two CTAs
                if (H * S <= num_sms) {
                    launch_pdl(*this, wkv7_seq_kernel<2>, dim3(2 * H, S), dim3(kWsThreads), 0, ws.seg_meta, ws.r, ws.k, ws.v, vgate, ws.vfirst, ws.w, ws.a, ws.g,
                               L.k_k, L.k_a, L.r_k, L.lnx_w, L.lnx_b, wkv, l == 0 ? st.v_first : nullptr, ws.yg, H, C, ws.status);
                } else {
                    launch_pdl(*this, wkv7_seq_kernel<4>, dim3(H, S), dim3(kWsThreads), 0, ws.seg_meta, ws.r, ws.k, ws.v, vgate, ws.vfirst, ws.w, ws.a, ws.g,
                               L.k_k, L.k_a, L.r_k, L.lnx_w, L.lnx_b, wkv, l == 0 ? st.v_first : nullptr, ws.yg, H, C, ws.status);
                }
                launch_pdl(*this, wkv7_finish_kernel, dim3((R * H + kWsFinishThreads / 32 - 1) / (kWsFinishThreads / 32)), dim3(kWsFinishThreads), 0, ws.r, ws.k,
                           ws.v, vgate, ws.vfirst, ws.a, ws.g, L.k_a, L.r_k, L.lnx_w, L.lnx_b, ws.yg, R, H, C);
            } else if (n_items >= 4 * num_sms) {
                // many (session, head) pairs: one state row per lane, states staged by TMA (wkv_rows.cuh)
                const size_t rows_total = (size_t)cfg.n_layer * st.cap * H * kHeadSize;
                if (rows_total >= (1ull << 31)) throw std::runtime_error("state too large for the 32-bit row coordinate of its tensor map");
                if (!st.wkv_map_ok) {
                    encode_state_map(&st.wkv_map, st.wkv, rows_total);
                    st.wkv_map_ok = true;
                }
                static bool configured[16] = {false};
                if (!configured[device & 15]) {
                    RSV_CUDA(cudaFuncSetAttribute(wkv7_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kWrSmemBytes));
                    configured[device & 15] = true;
                }
                if (C % 64) throw std::runtime_error("n_embd must be a multiple of 64");
                const int ctas = std::min((n_items + kWrPairs - 1) / kWrPairs, num_sms);
                launch_pdl(*this, wkv7_rows_kernel, dim3(ctas), dim3(kWrThreads), kWrSmemBytes, st.wkv_map, (long long)l * st.cap * H * kHeadSize, ws.seg_meta,
                           n_items, ws.r, ws.k, ws.v, vgate, ws.vfirst, ws.w, ws.a, ws.g, L.k_k, L.k_a, L.r_k, L.lnx_w, L.lnx_b,
                           l == 0 ? st.v_first : nullptr, ws.yg, H, C, ws.status);
            } else {
                launch_pdl(*this, wkv7_kernel, dim3(H, S), dim3(kWkvThreads), 0, ws.seg_meta, ws.r, ws.k, ws.v, vgate, ws.vfirst, ws.w, ws.a, ws.g, L.k_k, L.k_a,
                           L.r_k, L.lnx_w, L.lnx_b, wkv, l == 0 ? st.v_first : nullptr, ws.yg, H, C);
            }
            check_launch("wkv7");
        }
        {
            LinReq q = {&L.Wo, ws.yg, C, ws.delta, C, EPI_STORE};
            run_linear(*this, "linear_att_out", &q, 1, R);
            pending = ws.delta;
        }
        LAUNCH(*this, "ln_shift1") {
            MixPtrs mp{{L.ffn_x_k, nullptr, nullptr, nullptr, nullptr, nullptr}};
            launch_pdl(*this, ln_shift_kernel<1>, dim3(R, ln_split), dim3(kRowThreads), 0, x_cur, pending, x_alt, L.ln2_w, L.ln2_b, mp, ws.row_meta, R, C, cmix_x, staging, ws.xb);
            check_launch("ln_shift1");
        }
        std::swap(x_cur, x_alt);
        pending = nullptr;
        if (staging) LAUNCH(*this, "commit_shift") {
                launch_pdl(*this, commit_shift_kernel, dim3(S), dim3(256), 0, staging, ws.seg_meta, C, cmix_x);
                check_launch("commit_shift");
            }
        {
            LinReq q = {&L.Wfk, ws.xb, C, ws.h, F, EPI_RELU2};
            run_linear(*this, "linear_ffn_key", &q, 1, R);
            LinReq q2 = {&L.Wfv, ws.h, F, ws.delta, C, EPI_STORE};
            run_linear(*this, "linear_ffn_value", &q2, 1, R);
            pending = ws.delta;
        }
    }
    ws.final_x = x_cur;
    ws.final_delta = pending;
    if (O) {
        LAUNCH(*this, "ln_out") {
            ln_rows_kernel<<<O, kRowThreads, 0, stream>>>(x_cur, pending, ln_out_w, ln_out_b, ws.out_rows, C, ws.xn);
            check_launch("ln_out");
        }
        LinReq q = {&head, ws.xn, C, ws.logits, V, EPI_STORE};
        run_linear(*this, "linear_head", &q, 1, O);
    }
    if (use_cursor) LAUNCH(*this, "advance_cursor") {
            advance_cursor_kernel<<<1, 1, 0, stream>>>(ws.tok_pos);
            check_launch("advance_cursor");
        }
}


// ------------------------------------------------------------------------------------------------
// persistent decode kernel: host side
// ------------------------------------------------------------------------------------------------
namespace {

DpMat make_dpmat(const LinearW& W, int map_index) {
    DpMat d;
    d.map = map_index;
    d.M = W.M;
    d.mtiles = W.Mpad / kTcTileM;
    d.is_i8 = W.wtype == W_INT8;
    d.kblocks = (int)((size_t)W.Kpad * (d.is_i8 ? 1 : 2) / kTcKBlockBytes);
    d.K = W.K;
    d.wscale = W.wscale;
    d.wzero = W.wzero;
    return d;
}
struct HostProb {
    int mtiles, kblocks;
};
// largest number of CTAs that share one tile, and per CTA the largest numbers of operand tiles, units, runs and
// problem shares, for one phase shape (the device builds its tables with the same formulas)
struct PhaseShape {
    int pmax = 1, btiles = 0, tiles = 0, units = 0, runs = 0, shares = 0;
};
PhaseShape phase_shape(const std::vector<HostProb>& probs, int G) {
    PhaseShape ps;
    int U = 0;
    std::vector<int> unit0;
    for (auto& q : probs) {
        unit0.push_back(U);
        U += q.mtiles * q.kblocks;
    }
    G = dp_choose_ge(unit0.data(), (int)unit0.size(), U, G);  // CTAs that take part in the phase (same rule as on the device)
    int u0 = 0;
    for (auto& q : probs) {
        for (int t = 0; t < q.mtiles; ++t) {
            const int first = u0 + t * q.kblocks;
            ps.pmax = std::max(ps.pmax, tc_cta_of_unit(first + q.kblocks - 1, U, G) - tc_cta_of_unit(first, U, G) + 1);
        }
        u0 += q.mtiles * q.kblocks;
        ps.tiles += q.mtiles;
    }
    for (int c = 0; c < G; ++c) {
        const int ub = tc_cta_begin(c, U, G), ue = tc_cta_begin(c + 1, U, G);
        int need = 0, p0 = 0, runs = 0, shares = 0;
        for (auto& q : probs) {
            const int lo = std::max(ub, p0), hi = std::min(ue, p0 + q.mtiles * q.kblocks);
            if (hi > lo) {
                need += std::min(hi - lo, q.kblocks);
                ++shares;
                runs += (hi - 1 - p0) / q.kblocks - (lo - p0) / q.kblocks + 1;
            }
            p0 += q.mtiles * q.kblocks;
        }
        ps.btiles = std::max(ps.btiles, need);
        ps.units = std::max(ps.units, ue - ub);
        ps.runs = std::max(ps.runs, runs);
        ps.shares = std::max(ps.shares, shares);
    }
    return ps;
}

}  // namespace

bool Model::persistent_available(int nb) {
    if (!use_persistent || nb < 1 || nb > kDpMaxNB) return false;
    if (nb == 1 && stream_available()) return true;  // one session: the weight-streaming kernel
    PersistentCtx& pc = pctx;
    if (pc.tried) return pc.ok;
    pc.tried = true;
    auto fail = [&](const std::string& why) {
        pc.why = why;
        pc.ok = false;
        return false;
    };
    RSV_CUDA(cudaSetDevice(device));
    int coop = 0;
    RSV_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device));
    if (!coop) return fail("device does not support cooperative launches");
    if (!head.tc_ok) return fail("head matrix cannot take the tensor-core path");
    for (const LayerW& L : layers)
        for (const LinearW* W : {&L.Wr, &L.Wk, &L.Wv, &L.Wo, &L.Wfk, &L.Wfv, &L.w1, &L.a1, &L.v1, &L.g1})
            if (!W->tc_ok) return fail("a weight matrix cannot take the tensor-core path (int8 files need one scale/zero per output row)");
    const int L = cfg.n_layer, C = cfg.n_embd;
    // tensor maps and per-layer tables
    std::vector<CUtensorMap> maps;
    std::vector<DpLayer> dl(L);
    auto add = [&](const LinearW& W) {
        maps.push_back(W.amap);
        return make_dpmat(W, (int)maps.size() - 1);
    };
    for (int l = 0; l < L; ++l) {
        const LayerW& Lw = layers[l];
        DpLayer& d = dl[l];
        memset(&d, 0, sizeof(d));
        d.mat[DM_WR] = add(Lw.Wr);
        d.mat[DM_WK] = add(Lw.Wk);
        d.mat[DM_WV] = add(Lw.Wv);
        d.mat[DM_WO] = add(Lw.Wo);
        d.mat[DM_WFK] = add(Lw.Wfk);
        d.mat[DM_WFV] = add(Lw.Wfv);
        d.mat[DM_W1] = add(Lw.w1);
        d.mat[DM_A1] = add(Lw.a1);
        d.mat[DM_V1] = add(Lw.v1);
        d.mat[DM_G1] = add(Lw.g1);
        d.w2 = (const __half*)Lw.w2.w;
        d.a2 = (const __half*)Lw.a2.w;
        d.v2 = (const __half*)Lw.v2.w;
        d.g2 = (const __half*)Lw.g2.w;
        d.ln1_w = Lw.ln1_w;
        d.ln1_b = Lw.ln1_b;
        d.ln2_w = Lw.ln2_w;
        d.ln2_b = Lw.ln2_b;
        d.lnx_w = Lw.lnx_w;
        d.lnx_b = Lw.lnx_b;
        d.x_r = Lw.x_r;
        d.x_w = Lw.x_w;
        d.x_k = Lw.x_k;
        d.x_v = Lw.x_v;
        d.x_a = Lw.x_a;
        d.x_g = Lw.x_g;
        d.ffn_x_k = Lw.ffn_x_k;
        d.w0 = Lw.w0;
        d.a0 = Lw.a0;
        d.v0 = Lw.v0;
        d.r_k = Lw.r_k;
        d.k_k = Lw.k_k;
        d.k_a = Lw.k_a;
    }
    DpParams P;
    memset(&P, 0, sizeof(P));
    P.head = add(head);
    const int G = num_sms;
    // phase shapes (layer 0 has no v1 problem; all layers share the matrix shapes)
    auto hp = [&](const DpMat& d) { return HostProb{d.mtiles, d.kblocks}; };
    const DpLayer& d0 = dl[0];
    std::vector<HostProb> p1a = {hp(d0.mat[DM_WR]), hp(d0.mat[DM_WK]), hp(d0.mat[DM_WV]), hp(d0.mat[DM_W1]), hp(d0.mat[DM_A1]), hp(d0.mat[DM_G1])};
    std::vector<HostProb> p1b = p1a;
    p1b.push_back(hp(d0.mat[DM_V1]));
    int pmax[5], tiles[5], btiles = 0, max_units = 8, max_runs = 0, max_shares = 0;
    {
        const PhaseShape a = phase_shape(p1a, G), b = phase_shape(p1b, G);
        pmax[0] = std::max(a.pmax, b.pmax);
        tiles[0] = b.tiles;
        btiles = std::max(a.btiles, b.btiles);
        max_units += a.units + b.units;
        max_runs = std::max(a.runs, b.runs);
        max_shares = std::max(a.shares, b.shares);
    }
    const DpMat* single[4] = {&d0.mat[DM_WO], &d0.mat[DM_WFK], &d0.mat[DM_WFV], &P.head};
    for (int i = 0; i < 4; ++i) {
        const PhaseShape a = phase_shape({hp(*single[i])}, G);
        pmax[i + 1] = a.pmax;
        tiles[i + 1] = a.tiles;
        btiles = std::max(btiles, a.btiles);
        max_units += a.units;
        max_runs = std::max(max_runs, a.runs);
        max_shares = std::max(max_shares, a.shares);
    }
    if (max_runs > kDpMaxRuns || max_shares > kDpMaxShares) return fail("schedule tables of the persistent kernel are too small for this shape");
    if (btiles > 255) return fail("too many operand tiles per CTA for this shape");
    if (C > 16 * kDpWorkers) return fail("n_embd too large for the persistent kernel's register-resident LayerNorm");
    if ((C + G - 1) / G + 1 > kDpMaxSlice) return fail("n_embd too large for the persistent kernel's per-CTA slice of the residual stream");
    // shared memory: ring + operand tiles + barriers + worker scratch
    const size_t fixed = (size_t)btiles * kDpBTile + 1024 /*alignment*/ + 2048 /*barriers, small scratch*/ + (size_t)btiles * kDpMaxNB * 8 +
                         (size_t)cfg.mids() * 4 + 8 * 64 * 4 + (size_t)kDpMaxNB * kDpMaxSlice * 4 + 2 * sizeof(DpLayer) + DV_COUNT * sizeof(DpVar) + (size_t)max_units * sizeof(DpUnit);
    const size_t budget = 227 * 1024;
    if (fixed + 3 * (size_t)kDpATile > budget) return fail("operand tiles do not fit in shared memory for this shape");
    const int nstages = (int)std::min<size_t>(10, (budget - fixed) / kDpATile);
    pc.smem = fixed + (size_t)nstages * kDpATile;
    pc.grid = G;
    pc.nstages = nstages;
    pc.btiles = btiles;
    RSV_CUDA(cudaFuncSetAttribute(decode_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pc.smem));
    int per_sm = 0;
    RSV_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_persistent_kernel, kDpThreads, pc.smem));
    if (per_sm < 1) return fail("persistent kernel does not fit on an SM");
    // device tables and scratch
    RSV_CUDA(cudaMalloc(&pc.d_layers, dl.size() * sizeof(DpLayer)));
    RSV_CUDA(cudaMalloc(&pc.d_maps, maps.size() * sizeof(CUtensorMap)));
    RSV_CUDA(cudaMemcpy(pc.d_maps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice));
    RSV_CUDA(cudaMalloc(&pc.x, (size_t)kDpMaxNB * C * 4));
    RSV_CUDA(cudaMalloc(&pc.yg, (size_t)kDpMaxNB * C * 4));
    RSV_CUDA(cudaMalloc(&pc.vfirst, (size_t)kDpMaxNB * C * 4));
    RSV_CUDA(cudaMalloc(&pc.rkv, (size_t)kDpMaxNB * 3 * C * 4));
    RSV_CUDA(cudaMalloc(&pc.mid, (size_t)kDpMaxNB * cfg.mids() * 4));
    RSV_CUDA(cudaMalloc(&pc.hbuf, (size_t)kDpMaxNB * cfg.ffn_hidden * 4));
    RSV_CUDA(cudaMemsetAsync(pc.mid, 0, (size_t)kDpMaxNB * cfg.mids() * 4, stream));
    RSV_CUDA(cudaMalloc(&pc.cand_val, (size_t)G * kDpMaxNB * 4));
    RSV_CUDA(cudaMalloc(&pc.cand_idx, (size_t)G * kDpMaxNB * 4));
    RSV_CUDA(cudaMalloc(&pc.grid_bar, 4));
#ifdef RSV_DP_DEBUG
    RSV_CUDA(cudaMalloc(&pc.dbg, (64 + 8 * 1024) * sizeof(long long)));
    RSV_CUDA(cudaMemsetAsync(pc.dbg, 0, (64 + 8 * 1024) * sizeof(long long), stream));
#endif
    RSV_CUDA(cudaMemsetAsync(pc.vfirst, 0, (size_t)kDpMaxNB * C * 4, stream));
    for (int i = 0; i < 5; ++i) {
        const size_t runs = (size_t)tiles[i] * pmax[i];
        RSV_CUDA(cudaMalloc(&pc.region_data[i], runs * kDpN * 128 * 4));
        RSV_CUDA(cudaMalloc(&pc.region_meta[i], runs * kDpWarps * sizeof(DpRunMeta)));
        RSV_CUDA(cudaMalloc(&pc.region_cnt[i], (size_t)tiles[i] * kDpWarps * sizeof(int)));
        pc.region_cnt_bytes[i] = (size_t)tiles[i] * kDpWarps * sizeof(int);
        RSV_CUDA(cudaMemsetAsync(pc.region_data[i], 0, runs * kDpN * 128 * 4, stream));
        RSV_CUDA(cudaMemsetAsync(pc.region_meta[i], 0, runs * kDpWarps * sizeof(DpRunMeta), stream));
        RSV_CUDA(cudaMemsetAsync(pc.region_cnt[i], 0, (size_t)tiles[i] * kDpWarps * sizeof(int), stream));
        pc.region_pmax[i] = pmax[i];
    }
    // layer tables need the state pointers of the call: only the state-independent part is stored here
    pc.params_template.resize(sizeof(DpParams) + dl.size() * sizeof(DpLayer));
    P.maps = (const CUtensorMap*)pc.d_maps;
    P.layers = (const DpLayer*)pc.d_layers;
    P.emb = emb;
    P.ln0_w = ln0_w;
    P.ln0_b = ln0_b;
    P.lno_w = ln_out_w;
    P.lno_b = ln_out_b;
    P.L = L;
    P.C = C;
    P.H = cfg.n_head;
    P.F = cfg.ffn_hidden;
    P.V = cfg.vocab;
    P.wm = cfg.w_mid;
    P.am = cfg.a_mid;
    P.vm = cfg.v_mid;
    P.gm = cfg.g_mid;
    P.x = pc.x;
    P.yg = pc.yg;
    P.vfirst = pc.vfirst;
    P.rkv = pc.rkv;
    P.mid = pc.mid;
    P.hbuf = pc.hbuf;
    for (int i = 0; i < 5; ++i) {
        P.reg[i].data = (uint32_t*)pc.region_data[i];
        P.reg[i].meta = (DpRunMeta*)pc.region_meta[i];
        P.reg[i].cnt = pc.region_cnt[i];
        P.reg[i].pmax = pmax[i];
    }
    P.dbg = pc.dbg;
    P.cand_val = pc.cand_val;
    P.cand_idx = pc.cand_idx;
    P.grid_bar = pc.grid_bar;
    P.status = ws.status;
    P.nstages = nstages;
    P.btiles = btiles;
    P.max_units = max_units;
    memcpy(pc.params_template.data(), &P, sizeof(P));
    memcpy(pc.params_template.data() + sizeof(P), dl.data(), dl.size() * sizeof(DpLayer));
    pc.ok = true;
    return true;
}

void Model::run_persistent(State& st, int nb, const int* slots, int n_tokens, bool tok_from_list, bool argmax_feed, uint32_t* seq_dev, int* seq_cnt_dev,
                           int seq_cap) {
    if (nb == 1 && stream_available()) return run_stream(st, slots[0], n_tokens, tok_from_list, argmax_feed, seq_dev, seq_cnt_dev, seq_cap);
    if (!persistent_available(nb)) throw std::runtime_error("persistent decode path unavailable: " + pctx.why);
    PersistentCtx& pc = pctx;
    RSV_CUDA(cudaSetDevice(device));
    const int L = cfg.n_layer, C = cfg.n_embd, H = cfg.n_head;
    ensure_workspace(std::max(nb, 1), std::max(nb, 1), std::max(nb, 1));
    DpParams P;
    memcpy(&P, pc.params_template.data(), sizeof(P));
    // the device layer table carries the state pointers: rewrite it only when another state is used
    if (pc.bound_tmix != st.tmix_x || pc.bound_wkv != st.wkv || pc.bound_cmix != st.cmix_x || pc.bound_cap != st.cap) {
        std::vector<DpLayer> dl(L);
        memcpy(dl.data(), pc.params_template.data() + sizeof(P), dl.size() * sizeof(DpLayer));
        const size_t lay_x = (size_t)st.cap * C, lay_s = (size_t)st.cap * H * kHeadSize * kHeadSize;
        for (int l = 0; l < L; ++l) {
            dl[l].tmix_x = st.tmix_x + l * lay_x;
            dl[l].cmix_x = st.cmix_x + l * lay_x;
            dl[l].wkv = st.wkv + l * lay_s;
        }
        RSV_CUDA(cudaStreamSynchronize(stream));  // earlier launches may still read the table
        RSV_CUDA(cudaMemcpyAsync(pc.d_layers, dl.data(), dl.size() * sizeof(DpLayer), cudaMemcpyHostToDevice, stream));
        RSV_CUDA(cudaStreamSynchronize(stream));  // `dl` is a local pageable buffer
        pc.bound_tmix = st.tmix_x;
        pc.bound_wkv = st.wkv;
        pc.bound_cmix = st.cmix_x;
        pc.bound_cap = st.cap;
    }
    P.nb = nb;
    for (int b = 0; b < kDpMaxNB; ++b) P.slot[b] = b < nb ? slots[b] : 0;
    P.state_vfirst = st.v_first;
    P.tokens = ws.tokens;
    P.tok_list = ws.tok_list;
    P.seq = seq_dev;
    P.seq_cnt = seq_cnt_dev;
    P.seq_cap = seq_cap;
    P.logits = ws.logits;
    P.status = ws.status;
    P.n_tokens = n_tokens;
    P.tok_from_list = tok_from_list ? 1 : 0;
    P.argmax_feed = argmax_feed ? 1 : 0;
    RSV_CUDA(cudaMemsetAsync(pc.grid_bar, 0, 4, stream));
    void* args[] = {&P};
    LAUNCH(*this, "decode_persistent") {
        RSV_CUDA(cudaLaunchCooperativeKernel((const void*)decode_persistent_kernel, dim3(pc.grid), dim3(kDpThreads), args, pc.smem, stream));
    }
#ifdef RSV_DP_DEBUG
    if (pc.dbg && n_tokens >= 2) {
        std::vector<long long> hv(64 + 8 * 1024);
        long long* h = hv.data();
        RSV_CUDA(cudaStreamSynchronize(stream));
        RSV_CUDA(cudaMemcpy(h, pc.dbg, hv.size() * sizeof(long long), cudaMemcpyDeviceToHost));
        const char* names[7] = {"phase start", "stats done", "operands done", "runs drained", "barrier done", "x slice done", "barrier b done"};
        long long t0 = h[0];
        fprintf(stderr, "[persistent kernel, CTA 0, token 1, layer 1] times in us since P1 start\n");
        for (int ph = 0; ph < 4; ++ph) {
            if (ph == 1) fprintf(stderr, "  heads done %.2f, barrier 2 done %.2f\n", (h[40] - t0) / 1e3, (h[41] - t0) / 1e3);
            for (int i = 0; i < 7; ++i)
                if (h[ph * 10 + i]) fprintf(stderr, "  phase %d %-14s %.2f\n", ph, names[i], (h[ph * 10 + i] - t0) / 1e3);
        }
        {
            const char* nm[5] = {"operands done", "partials stored", "arrivals returned", "finishing done", "barrier left"};
            const long long p3 = h[10];  // CTA 0, phase 3 start
            for (int k = 0; k < 5; ++k) {
                long long mn = 1LL << 62, mx = 0, sum = 0;
                int amx = -1, n = 0;
                for (int c = 0; c < pc.grid && c < 1024; ++c) {
                    const long long v = h[64 + c * 8 + k];
                    if (!v) continue;
                    ++n;
                    sum += v - p3;
                    if (v < mn) mn = v;
                    if (v > mx) {
                        mx = v;
                        amx = c;
                    }
                }
                if (n) fprintf(stderr, "  att.output phase, all CTAs: %-18s min %.2f avg %.2f max %.2f (CTA %d) [us since CTA 0 entered the phase]\n", nm[k], (mn - p3) / 1e3, sum / 1e3 / n, (mx - p3) / 1e3, amx);
            }
        }
        fprintf(stderr, "  ffn.key operands: loads start %.2f, values loaded %.2f, scale set %.2f, digits written %.2f\n", (h[63] - t0) / 1e3, (h[60] - t0) / 1e3, (h[61] - t0) / 1e3, (h[62] - t0) / 1e3);
        fprintf(stderr, "  ffn.key phase: producer issued its %lld tiles from %.2f to %.2f; MMA thread started %.2f, last issue %.2f, waited %.2f us for tiles/accumulators\n",
                h[53], (h[55] - t0) / 1e3, (h[56] - t0) / 1e3, (h[50] - t0) / 1e3, (h[51] - t0) / 1e3, h[52] / 1e3);
    }
#endif
}

// ------------------------------------------------------------------------------------------------
// batch-1 weight-streaming decode kernel: host side
// ------------------------------------------------------------------------------------------------
namespace {

template <int CMAX>
void launch_stream(const DsParams& P, int grid, size_t smem, cudaStream_t stream, bool configure_only) {
    if (configure_only) {
        RSV_CUDA(cudaFuncSetAttribute(decode_stream_kernel<CMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        int per_sm = 0;
        RSV_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stream_kernel<CMAX>, kDsThreads, smem));
        if (per_sm < 1) throw std::runtime_error("weight-streaming decode kernel does not fit on an SM");
        return;
    }
    void* args[] = {(void*)&P};
    RSV_CUDA(cudaLaunchCooperativeKernel((const void*)decode_stream_kernel<CMAX>, dim3(grid), dim3(kDsThreads), args, smem, stream));
}
void dispatch_stream(int cmax, const DsParams& P, int grid, size_t smem, cudaStream_t stream, bool configure_only) {
    switch (cmax) {
        case 512: return launch_stream<512>(P, grid, smem, stream, configure_only);
        case 1024: return launch_stream<1024>(P, grid, smem, stream, configure_only);
        case 2048: return launch_stream<2048>(P, grid, smem, stream, configure_only);
        case 2560: return launch_stream<2560>(P, grid, smem, stream, configure_only);
        case 4096: return launch_stream<4096>(P, grid, smem, stream, configure_only);
        default: throw std::runtime_error("weight-streaming decode kernel: unsupported n_embd");
    }
}

}  // namespace

bool Model::stream_available() {
    if (!use_persistent || !use_stream) return false;
    StreamCtx& sc = sctx;
    if (sc.tried) return sc.ok;
    sc.tried = true;
    auto fail = [&](const std::string& why) {
        sc.why = why;
        sc.ok = false;
        if (const char* e = getenv("RSV_VERBOSE"))
            if (*e && *e != '0') fprintf(stderr, "[rsv] weight-streaming decode kernel not used: %s\n", why.c_str());
        return false;
    };
    RSV_CUDA(cudaSetDevice(device));
    int coop = 0;
    RSV_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device));
    if (!coop) return fail("device does not support cooperative launches");
    const int L = cfg.n_layer, C = cfg.n_embd, F = cfg.ffn_hidden, V = cfg.vocab, H = cfg.n_head, G = num_sms;
    // int8 matrices: one (scale, zero) per output row, or the reference container's one per row and group of 128 weights
    auto format_of = [](const LinearW& W) { return W.wtype != W_INT8 ? 0 : (W.wscale && W.wzero) ? 1 : W.sz ? 2 : -1; };
    if (format_of(head) < 0) return fail("int8 head without scales");
    const int fmt = layers.empty() ? 0 : format_of(layers[0].Wr);
    for (const LayerW& Lw : layers)
        for (const LinearW* W : {&Lw.Wr, &Lw.Wk, &Lw.Wv, &Lw.Wo, &Lw.Wfk, &Lw.Wfv})
            if (format_of(*W) != fmt || fmt < 0) return fail("the big matrices of the layers differ in their weight format, or an int8 matrix has no scales");
    // the layout (row ownership, chunks, shared memory, every capacity of the kernel's tables) is pure arithmetic on the shape
    const DsShape shp{L, C, F, V, H, cfg.w_mid, cfg.a_mid, cfg.v_mid, cfg.g_mid, fmt, format_of(head)};
    DsLayout lay;
    {
        std::string why;
        if (!ds_layout(shp, G, lay, why)) return fail(why);
    }
    const int cmax = lay.cmax, vec_floats = lay.vec_floats, ring_bytes = lay.ring_bytes;
    const bool head_early = lay.head_early;
    sc.kl = cmax;
    sc.grid = G;
    sc.ring_bytes = ring_bytes;
    sc.vec_floats = vec_floats;
    sc.smem = lay.smem;
    DsParams P;
    memset(&P, 0, sizeof(P));
    try {
        dispatch_stream(cmax, P, G, sc.smem, stream, true);
    } catch (const std::exception& e) {
        return fail(e.what());
    }
    // per-layer tables: sizes and CTA groups from the layout, pointers from the checkpoint
    auto bind = [&](DsEntry& e, const LinearW& W, const float* mix) -> bool {
        if (e.M != 0 && (W.M != e.M || (e.is_i8 ? W.K : 2 * W.K) != e.row_stride)) return false;
        e.base = (const char*)W.w;
        e.wscale = W.wscale;
        e.wzero = W.wzero;
        e.sz = W.sz;
        e.mix = mix;
        return true;
    };
    std::vector<DsLayer> dl((size_t)L);
    for (int l = 0; l < L; ++l) {
        const LayerW& Lw = layers[l];
        DsLayer& d = dl[l];
        memset(&d, 0, sizeof(d));
        ds_layer_entries(shp, G, l > 0, d.e);
        if (!(bind(d.e[DSE_W1], Lw.w1, Lw.x_w) && bind(d.e[DSE_A1], Lw.a1, Lw.x_a) && bind(d.e[DSE_G1], Lw.g1, Lw.x_g) && bind(d.e[DSE_V1], Lw.v1, Lw.x_v) &&
              bind(d.e[DSE_WR], Lw.Wr, Lw.x_r) && bind(d.e[DSE_WK], Lw.Wk, Lw.x_k) && bind(d.e[DSE_WV], Lw.Wv, Lw.x_v) && bind(d.e[DSE_WO], Lw.Wo, nullptr) &&
              bind(d.e[DSE_WFK], Lw.Wfk, nullptr) && bind(d.e[DSE_WFV], Lw.Wfv, nullptr)))
            return fail("a matrix of the checkpoint does not have the model's shape");
        for (const LinearW* W : {&Lw.w1, &Lw.a1, &Lw.g1, &Lw.v1})
            if (W->wtype != W_F16) return fail("rank projections must be fp16 [mid, n_embd]");
        d.w2 = (const __half*)Lw.w2.w;
        d.a2 = (const __half*)Lw.a2.w;
        d.v2 = (const __half*)Lw.v2.w;
        d.g2 = (const __half*)Lw.g2.w;
        d.ln1_w = Lw.ln1_w;
        d.ln1_b = Lw.ln1_b;
        d.ln2_w = Lw.ln2_w;
        d.ln2_b = Lw.ln2_b;
        d.lnx_w = Lw.lnx_w;
        d.lnx_b = Lw.lnx_b;
        d.x_r = Lw.x_r;
        d.x_k = Lw.x_k;
        d.x_v = Lw.x_v;
        d.ffn_x_k = Lw.ffn_x_k;
        d.w0 = Lw.w0;
        d.a0 = Lw.a0;
        d.v0 = Lw.v0;
        d.r_k = Lw.r_k;
        d.k_k = Lw.k_k;
        d.k_a = Lw.k_a;
    }
    RSV_CUDA(cudaMalloc(&sc.d_layers, dl.size() * sizeof(DsLayer)));
    RSV_CUDA(cudaMemcpy(sc.d_layers, dl.data(), dl.size() * sizeof(DsLayer), cudaMemcpyHostToDevice));
    {
        // second copy of the weights in the order the kernel consumes them (a chunk = one bulk copy): region sizes = the largest CTA's
        const long long wslot = lay.wslot, hslot = lay.hslot;
        DsEntry head_e = ds_head_entry(shp, G);
        if (!bind(head_e, head, nullptr)) return fail("the head of the checkpoint does not have the model's shape");
        sc.wslot = wslot;
        sc.hslot = hslot;
        RSV_CUDA(cudaMalloc(&sc.wstream, (size_t)wslot * G * L));
        RSV_CUDA(cudaMalloc(&sc.hstream, (size_t)hslot * G));
        DsParams Q;
        memset(&Q, 0, sizeof(Q));
        Q.layers = (const DsLayer*)sc.d_layers;
        Q.head = head_e;
        Q.L = L;
        Q.H = H;
        Q.wm = cfg.w_mid;
        Q.am = cfg.a_mid;
        Q.vm = cfg.v_mid;
        Q.gm = cfg.g_mid;
        ds_retile_kernel<<<G, 256, 0, stream>>>(Q, (char*)sc.wstream, wslot, (char*)sc.hstream, hslot);
        check_launch("ds_retile");
        RSV_CUDA(cudaStreamSynchronize(stream));
        if (const char* e = getenv("RSV_VERBOSE"))
            if (*e && *e != '0')
                fprintf(stderr, "[rsv] weight-streaming decode kernel: %.2f GB second copy of the weights in consumption order (%lld bytes per layer and SM); ring %d bytes%s\n",
                        ((double)wslot * G * L + (double)hslot * G) / 1e9, wslot, ring_bytes, head_early ? ", a head's first chunk released early" : "");
    }
    RSV_CUDA(cudaMalloc(&sc.x, (size_t)C * 4));
    RSV_CUDA(cudaMalloc(&sc.yg, (size_t)C * 4));
    RSV_CUDA(cudaMalloc(&sc.vfirst, (size_t)C * 4));
    RSV_CUDA(cudaMalloc(&sc.rkv, (size_t)3 * C * 4));
    RSV_CUDA(cudaMalloc(&sc.mid, (size_t)std::max(cfg.mids(), 1) * 4));
    RSV_CUDA(cudaMalloc(&sc.hbuf, (size_t)F * 4));
    RSV_CUDA(cudaMalloc(&sc.cand_val, (size_t)G * 4));
    RSV_CUDA(cudaMalloc(&sc.cand_idx, (size_t)G * 4));
    RSV_CUDA(cudaMalloc(&sc.grid_bar, 4));
    RSV_CUDA(cudaMemsetAsync(sc.mid, 0, (size_t)std::max(cfg.mids(), 1) * 4, stream));
    RSV_CUDA(cudaMemsetAsync(sc.vfirst, 0, (size_t)C * 4, stream));
#ifdef RSV_DS_DEBUG
    RSV_CUDA(cudaMalloc(&sc.dbg, (256 + 16 * 256) * sizeof(long long)));
    RSV_CUDA(cudaMemsetAsync(sc.dbg, 0, (256 + 16 * 256) * sizeof(long long), stream));
#endif
    P.layers = (const DsLayer*)sc.d_layers;
    P.head = ds_head_entry(shp, G);
    bind(P.head, head, nullptr);
    P.emb = emb;
    P.ln0_w = ln0_w;
    P.ln0_b = ln0_b;
    P.lno_w = ln_out_w;
    P.lno_b = ln_out_b;
    P.L = L;
    P.C = C;
    P.H = H;
    P.F = F;
    P.V = V;
    P.wm = cfg.w_mid;
    P.am = cfg.a_mid;
    P.vm = cfg.v_mid;
    P.gm = cfg.g_mid;
    P.x = sc.x;
    P.yg = sc.yg;
    P.vfirst = sc.vfirst;
    P.rkv = sc.rkv;
    P.mid = sc.mid;
    P.hbuf = sc.hbuf;
    P.cand_val = sc.cand_val;
    P.cand_idx = sc.cand_idx;
    P.grid_bar = sc.grid_bar;
    P.wstream = (const char*)sc.wstream;
    P.wslot = sc.wslot;
    P.hstream = (const char*)sc.hstream;
    P.hslot = sc.hslot;
    P.ring_bytes = ring_bytes;
    P.head_early = head_early ? 1 : 0;
    P.vec_floats = vec_floats;
    P.dbg = sc.dbg;
    sc.params_template.resize(sizeof(DsParams));
    memcpy(sc.params_template.data(), &P, sizeof(P));
    sc.ok = true;
    return true;
}

void Model::run_stream(State& st, int slot, int n_tokens, bool tok_from_list, bool argmax_feed, uint32_t* seq_dev, int* seq_cnt_dev, int seq_cap) {
    if (!stream_available()) throw std::runtime_error("weight-streaming decode path unavailable: " + sctx.why);
    StreamCtx& sc = sctx;
    RSV_CUDA(cudaSetDevice(device));
    if (slot < 0 || slot >= st.cap) throw std::runtime_error("state slot out of range");
    ensure_workspace(1, 1, 1);
    DsParams P;
    memcpy(&P, sc.params_template.data(), sizeof(P));
    P.slot = slot;
    P.lay_x = (long long)st.cap * cfg.n_embd;
    P.lay_s = (long long)st.cap * cfg.n_head * kHeadSize * kHeadSize;
    P.tmix_x = st.tmix_x;
    P.wkv = st.wkv;
    P.cmix_x = st.cmix_x;
    P.state_vfirst = st.v_first;
    P.tokens = ws.tokens;
    P.tok_list = ws.tok_list;
    P.seq = seq_dev;
    P.seq_cnt = seq_cnt_dev;
    P.seq_cap = seq_cap;
    P.logits = ws.logits;
    P.status = ws.status;
    P.n_tokens = n_tokens;
    P.tok_from_list = tok_from_list ? 1 : 0;
    P.argmax_feed = argmax_feed ? 1 : 0;
    RSV_CUDA(cudaMemsetAsync(sc.grid_bar, 0, 4, stream));
    LAUNCH(*this, "decode_stream") { dispatch_stream(sc.kl, P, sc.grid, sc.smem, stream, false); }
#ifdef RSV_DS_DEBUG
    if (sc.dbg && n_tokens >= 2) {
        static long long h[256 + 16 * 256];
        RSV_CUDA(cudaStreamSynchronize(stream));
        RSV_CUDA(cudaMemcpy(h, sc.dbg, sizeof(h), cudaMemcpyDeviceToHost));
        const int order[15] = {0, 10, 1, 2, 11, 3, 12, 4, 5, 13, 6, 7, 14, 8, 9};
        const char* names[15] = {"layer start", "P1 operands", "P1 rows done", "heads done", "P3 operands", "P3 rows done", "P4 operands", "P4 rows done", "P5 operands", "P5 rows done",
                                 "barrier 5 passed", "barrier 1 passed", "barrier 2 passed", "barrier 3 passed", "barrier 4 passed"};
        fprintf(stderr, "[decode_stream_kernel, CTA 0, token 1, layer 1] us since the layer started\n");
        for (int i = 0; i < 15; ++i) fprintf(stderr, "  %-18s %.2f\n", names[order[i]], (h[order[i]] - h[0]) / 1e3);
        fprintf(stderr, "  P1 prologue: loads issued %.2f, statistics done %.2f, shift / slice done %.2f\n", (h[15] - h[0]) / 1e3, (h[16] - h[0]) / 1e3, (h[17] - h[0]) / 1e3);
        fprintf(stderr, "  producer, first chunks of the launch (ring empty), us between issues:");
        for (int i = 1; i < 8; ++i) fprintf(stderr, " %.2f", (h[200 + i] - h[200 + i - 1]) / 1e3);
        fprintf(stderr, "\n");
        fprintf(stderr, "  P1 operands: magnitudes %.2f, barrier %.2f, digits written %.2f\n", (h[52] - h[0]) / 1e3, (h[53] - h[0]) / 1e3, (h[54] - h[0]) / 1e3);
        fprintf(stderr, "  heads: vectors gathered %.2f, first chunk there %.2f, its dot products done %.2f, all three there %.2f, dot products done %.2f, state updated %.2f\n", (h[18] - h[0]) / 1e3,
                (h[55] - h[0]) / 1e3, (h[57] - h[0]) / 1e3, (h[56] - h[0]) / 1e3, (h[19] - h[0]) / 1e3, (h[50] - h[0]) / 1e3);
        const char* ph[4] = {"P1", "P3", "P4", "P5"};
        for (int i = 0; i < 4; ++i)
            fprintf(stderr, "  %s rows, consumer warp 0: %lld chunks, %.2f us waiting for them, %.2f us multiplying\n", ph[i], h[20 + 4 * i + 2], h[20 + 4 * i] / 1e3, h[20 + 4 * i + 1] / 1e3);
        fprintf(stderr, "  producer: P1 rows issued %.2f .. %.2f, head chunk A issued %.2f, C issued %.2f, att.out issued %.2f, ffn.value issued %.2f\n", (h[40] - h[0]) / 1e3,
                (h[41] - h[0]) / 1e3, (h[42] - h[0]) / 1e3, (h[43] - h[0]) / 1e3, (h[44] - h[0]) / 1e3, (h[45] - h[0]) / 1e3);
        for (int w = 0; w < 16; ++w)
            fprintf(stderr, "  P1 warp %2d: last chunk wait %.2f .. %.2f, multiplied %.2f, tile finished %.2f\n", w, (h[64 + 4 * w] - h[0]) / 1e3, (h[65 + 4 * w] - h[0]) / 1e3,
                    (h[66 + 4 * w] - h[0]) / 1e3, h[67 + 4 * w] ? (h[67 + 4 * w] - h[0]) / 1e3 : 0.0);
        {
            const int ord[15] = {0, 10, 1, 2, 3, 12, 4, 5, 13, 6, 7, 14, 8, 9, -1};
            const char* nm[15] = {"layer start", "P1 operands", "P1 rows done", "heads done", "P3 operands", "P3 rows done", "P4 operands", "P4 rows done", "P5 operands", "P5 rows done",
                                  "barrier 5 passed", "", "barrier 2 passed", "barrier 3 passed", "barrier 4 passed"};
            fprintf(stderr, "  all CTAs (us since CTA 0's layer start): min / mean / max (CTA)\n");
            for (int i = 0; ord[i] >= 0; ++i) {
                const int k = ord[i];
                long long mn = 1LL << 62, mx = 0, sum = 0;
                int amx = -1, n = 0;
                for (int c = 0; c < sc.grid && c < 256; ++c) {
                    const long long v = h[256 + c * 16 + k];
                    if (!v) continue;
                    ++n;
                    sum += v - h[0];
                    mn = std::min(mn, v);
                    if (v > mx) {
                        mx = v;
                        amx = c;
                    }
                }
                if (n) fprintf(stderr, "    %-18s %7.2f %7.2f %7.2f (%d)\n", nm[k], (mn - h[0]) / 1e3, sum / 1e3 / n, (mx - h[0]) / 1e3, amx);
            }
        }
        RSV_CUDA(cudaMemsetAsync(sc.dbg, 0, (256 + 16 * 256) * sizeof(long long), stream));
    }
#endif
}

void Model::check_status() {
    int sw[2] = {0, 0};  // status bits; where the weight-streaming decode kernel gave up
    RSV_CUDA(cudaMemcpyAsync(sw, ws.status, 2 * sizeof(int), cudaMemcpyDeviceToHost, stream));
    RSV_CUDA(cudaStreamSynchronize(stream));
    const int s = sw[0];
    if (s) {
        RSV_CUDA(cudaMemsetAsync(ws.status, 0, 2 * sizeof(int), stream));
        if (s & (2 | 4 | 32)) {
            // a kernel that gave up on a wait may have left arrival counters non-zero: the next launch must start from zero
            if (ws.tc_cnt) RSV_CUDA(cudaMemsetAsync(ws.tc_cnt, 0, (size_t)kTcMaxSplit * kTcEpiWarps * sizeof(int), stream));
            for (int i = 0; i < 5; ++i)
                if (pctx.region_cnt[i]) RSV_CUDA(cudaMemsetAsync(pctx.region_cnt[i], 0, pctx.region_cnt_bytes[i], stream));
        }
        if (s & 32) {
            static const char* const site[5] = {"a wait", "a chunk of weight rows", "room in the ring", "a grid barrier", "a chunk of a head's rows"};
            const int k = sw[1] & 15;
            throw std::runtime_error(std::string("weight-streaming decode kernel gave up waiting for ") + site[k >= 1 && k <= 4 ? k : 0] + " (device status bit 5; CTA " +
                                     std::to_string((sw[1] >> 20) & 255) + ", index " + std::to_string((sw[1] >> 4) & 0xFFFF) + ")");
        }
        if (s & 16) throw std::runtime_error("WKV kernel gave up waiting for a staged state (device status bit 4)");
        if (s & 8) throw std::runtime_error("persistent decode kernel: schedule tables too small for this shape (device status bit 3)");
        if (s & 4) throw std::runtime_error("persistent decode kernel gave up waiting on a barrier (device status bit 2)");
        if (s & 2) throw std::runtime_error("tensor-core kernel gave up waiting on a barrier (device status bit 1)");
        if (s & 1) throw std::runtime_error("token id out of range (>= vocab); the embedding row 0 was used instead");
        throw std::runtime_error("device status word = " + std::to_string(s));
    }
}

// ------------------------------------------------------------------------------------------------
// helpers used by the C ABI
// ------------------------------------------------------------------------------------------------
void engine_argmax(Model& m, const float* logits_dev, int rows, uint32_t* next_tok_dev, uint32_t* seq_dev, int* seq_cnt_dev, int seq_cap,
                   const int* row_map_dev) {
    LAUNCH(m, "argmax") {
        argmax_rows_kernel<<<rows, kArgmaxThreads, 0, m.stream>>>(logits_dev, m.cfg.vocab, next_tok_dev, seq_dev, seq_cnt_dev, seq_cap, row_map_dev);
        check_launch("argmax");
    }
}

void engine_sample(Model& m, const float* logits_dev, int rows, const float* sampler8_dev, const uint32_t* hist_dev, int hist_stride,
                   const int* round_cnt_dev, uint32_t* next_tok_dev, uint32_t* seq_dev, int* seq_cnt_dev, int seq_cap, const int* row_map_dev) {
    if (rows > m.ws.outs) throw std::runtime_error("engine_sample: more rows than the work area holds");
    LAUNCH(m, "sample") {
        sample_rows_kernel<<<rows, kSampleThreads, 0, m.stream>>>(logits_dev, m.cfg.vocab, sampler8_dev, hist_dev, hist_stride, round_cnt_dev, m.ws.samp_temp,
                                                                  m.ws.samp_cnt, next_tok_dev, seq_dev, seq_cnt_dev, seq_cap, row_map_dev);
        check_launch("sample");
    }
}

void engine_sample_raw(cudaStream_t stream, const float* logits_dev, int rows, int V, const float* sampler8_dev, const uint32_t* hist_dev,
                       int hist_stride, float* temp_dev, uint32_t* counter_dev, uint32_t* out_dev) {
    sample_rows_kernel<<<rows, kSampleThreads, 0, stream>>>(logits_dev, V, sampler8_dev, hist_dev, hist_stride, nullptr, temp_dev, counter_dev, out_dev,
                                                            nullptr, nullptr, 0, nullptr);
    check_launch("sample");
}

Ticket::~Ticket() {
    if (model) {
        cudaSetDevice(model->device);
        if (graph_exec || graph) cudaStreamSynchronize(model->stream);
    }
    if (graph_exec) cudaGraphExecDestroy(graph_exec);
    if (graph) cudaGraphDestroy(graph);
    if (seq) cudaFree(seq);
    if (cnt) cudaFree(cnt);
    if (sampler) cudaFree(sampler);
}

void engine_merge_tokens(Model& m, const uint32_t* host_tok_dev, const uint32_t* slot_tok_dev, int R) {
    LAUNCH(m, "merge_tokens") {
        merge_tokens_kernel<<<(R + 255) / 256, 256, 0, m.stream>>>(host_tok_dev, m.ws.row_meta, slot_tok_dev, R, m.ws.tokens);
        check_launch("merge_tokens");
    }
}

void engine_argmax_raw(cudaStream_t stream, const float* logits_dev, int rows, int V, uint32_t* out_dev) {
    argmax_rows_kernel<<<rows, kArgmaxThreads, 0, stream>>>(logits_dev, V, out_dev, nullptr, nullptr, 0, nullptr);
    check_launch("argmax");
}

void engine_dequant_int8(cudaStream_t stream, const uint8_t* idx_dev, const uint32_t* sz_dev, size_t M, size_t K, float* out_dev) {
    dequant_int8_kernel<<<148 * 8, 256, 0, stream>>>(idx_dev, sz_dev, M, K, out_dev);
    check_launch("dequant_int8");
}


void engine_quantize_int8(cudaStream_t stream, const float* w_dev, size_t M, size_t K, uint8_t* idx_dev, uint32_t* sz_dev) {
    const size_t groups = M * (K / 128);
    const int blocks = (int)std::min<size_t>((groups + 7) / 8, 148 * 16);
    quantize_int8_kernel<<<blocks, 256, 0, stream>>>(w_dev, groups, idx_dev, sz_dev);
    check_launch("quantize_int8");
}

void engine_segment_sums(Model& m, int n_segments, float* acc_dev) {
    if (!m.ws.final_x) throw std::runtime_error("segment sums: no step has run");
    LAUNCH(m, "segment_sums") {
        segment_sums_kernel<<<dim3(n_segments, (m.cfg.n_embd + 255) / 256), 256, 0, m.stream>>>(m.ws.final_x, m.ws.final_delta, m.ws.seg_meta, m.cfg.n_embd, acc_dev);
        check_launch("segment_sums");
    }
}

// Operator-level WKV-7 step on host data (see the declaration).  The four kernels are launched as forward_rows launches them.
void engine_op_wkv7(int device, int variant, int nseg, int T, int H, const float* const in[8], const float* const par[5], float* state_host, float* y_host) {
    RSV_CUDA(cudaSetDevice(device));
    const int C = H * kHeadSize, R = nseg * T;
    const size_t row_bytes = (size_t)R * C * 4, st_floats = (size_t)nseg * H * kHeadSize * kHeadSize;
    struct Buf {
        void* p = nullptr;
        ~Buf() {
            if (p) cudaFree(p);
        }
    };
    Buf din[8], dpar[5], dstate, dy, dseg, dstatus;
    for (int i = 0; i < 8; ++i)
        if (in[i]) {
            RSV_CUDA(cudaMalloc(&din[i].p, row_bytes));
            RSV_CUDA(cudaMemcpy(din[i].p, in[i], row_bytes, cudaMemcpyHostToDevice));
        }
    for (int i = 0; i < 5; ++i) {
        RSV_CUDA(cudaMalloc(&dpar[i].p, (size_t)C * 4));
        RSV_CUDA(cudaMemcpy(dpar[i].p, par[i], (size_t)C * 4, cudaMemcpyHostToDevice));
    }
    RSV_CUDA(cudaMalloc(&dstate.p, st_floats * 4));
    RSV_CUDA(cudaMemcpy(dstate.p, state_host, st_floats * 4, cudaMemcpyHostToDevice));
    RSV_CUDA(cudaMalloc(&dy.p, row_bytes));
    RSV_CUDA(cudaMemset(dy.p, 0, row_bytes));
    std::vector<SegMeta> segs((size_t)nseg);
    for (int s2 = 0; s2 < nseg; ++s2) segs[s2] = SegMeta{s2 * T, T, s2, 0};
    RSV_CUDA(cudaMalloc(&dseg.p, segs.size() * sizeof(SegMeta)));
    RSV_CUDA(cudaMemcpy(dseg.p, segs.data(), segs.size() * sizeof(SegMeta), cudaMemcpyHostToDevice));
    RSV_CUDA(cudaMalloc(&dstatus.p, 8));
    RSV_CUDA(cudaMemset(dstatus.p, 0, 8));
    const float *r = (const float*)din[0].p, *k = (const float*)din[1].p, *v = (const float*)din[2].p, *w = (const float*)din[3].p, *a = (const float*)din[4].p,
                *g = (const float*)din[5].p, *vgate = (const float*)din[6].p, *vfirst = (const float*)din[7].p;
    const float *k_k = (const float*)dpar[0].p, *k_a = (const float*)dpar[1].p, *r_k = (const float*)dpar[2].p, *lnx_w = (const float*)dpar[3].p,
                *lnx_b = (const float*)dpar[4].p;
    float *state = (float*)dstate.p, *yg = (float*)dy.p;
    int* status = (int*)dstatus.p;
    const SegMeta* sm = (const SegMeta*)dseg.p;
    cudaDeviceProp prop;
    RSV_CUDA(cudaGetDeviceProperties(&prop, device));
    const int sms = prop.multiProcessorCount, n_items = H * nseg;
    if (variant == 0) variant = T > 1 ? (n_items <= sms ? 3 : 4) : (n_items >= 4 * sms ? 2 : 1);
    if (variant == 1) {
        wkv7_kernel<<<dim3(H, nseg), kWkvThreads>>>(sm, r, k, v, vgate, vfirst, w, a, g, k_k, k_a, r_k, lnx_w, lnx_b, state, nullptr, yg, H, C);
    } else if (variant == 2) {
        CUtensorMap map;
        encode_state_map(&map, state, (size_t)nseg * H * kHeadSize);
        RSV_CUDA(cudaFuncSetAttribute(wkv7_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kWrSmemBytes));
        const int ctas = std::min((n_items + kWrPairs - 1) / kWrPairs, sms);
        wkv7_rows_kernel<<<ctas, kWrThreads, kWrSmemBytes>>>(map, 0LL, sm, n_items, r, k, v, vgate, vfirst, w, a, g, k_k, k_a, r_k, lnx_w, lnx_b, nullptr, yg, H, C, status);
    } else if (variant == 3 || variant == 4) {
        if (variant == 3)
            wkv7_seq_kernel<2><<<dim3(2 * H, nseg), kWsThreads>>>(sm, r, k, v, vgate, vfirst, w, a, g, k_k, k_a, r_k, lnx_w, lnx_b, state, nullptr, yg, H, C, status);
        else
            wkv7_seq_kernel<4><<<dim3(H, nseg), kWsThreads>>>(sm, r, k, v, vgate, vfirst, w, a, g, k_k, k_a, r_k, lnx_w, lnx_b, state, nullptr, yg, H, C, status);
        check_launch("wkv7_seq");
        wkv7_finish_kernel<<<(R * H + kWsFinishThreads / 32 - 1) / (kWsFinishThreads / 32), kWsFinishThreads>>>(r, k, v, vgate, vfirst, a, g, k_a, r_k, lnx_w, lnx_b, yg,
                                                                                                              R, H, C);
    } else {
        throw std::runtime_error("wkv7: variant must be 0 (automatic), 1 (token kernel), 2 (row-per-lane kernel), 3 or 4 (sequence kernel, head over two CTAs / one CTA)");
    }
    check_launch("wkv7");
    RSV_CUDA(cudaDeviceSynchronize());
    int st = 0;
    RSV_CUDA(cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost));
    if (st) throw std::runtime_error("WKV kernel gave up waiting for a staged state (device status " + std::to_string(st) + ")");
    RSV_CUDA(cudaMemcpy(state_host, state, st_floats * 4, cudaMemcpyDeviceToHost));
    RSV_CUDA(cudaMemcpy(y_host, yg, row_bytes, cudaMemcpyDeviceToHost));
}

void engine_op_linear(Model& m, int path, int wtype, const void* w_host, const uint32_t* sz_host, int M, int K, const float* x_host, int R,
                      float* y_host) {
    RSV_CUDA(cudaSetDevice(m.device));
    if (M < 1 || K < 8 || R < 1) throw std::runtime_error("op_linear: empty problem");
    if (wtype == W_INT8 ? (K % 128 != 0) : (K % 8 != 0)) throw std::runtime_error("op_linear: K must be a multiple of 128 (int8) or 8 (fp16)");
    Loader ld{m, nullptr};
    LinearW W;
    W.M = M;
    W.K = K;
    W.wtype = wtype;
    const size_t first_alloc = m.allocs.size();
    float *dx = nullptr, *dy = nullptr;
    try {
        if (wtype == W_INT8) {
            W.w = ld.upload(w_host, (size_t)M * K);
            W.sz = (uint32_t*)ld.upload(sz_host, (size_t)M * (K / 128) * 4);
            ld.prepare_tc_i8(W, sz_host);
        } else {
            W.w = ld.upload(w_host, (size_t)M * K * 2);
            ld.prepare_tc_f16(W, (const uint16_t*)w_host);
        }
        if (path == 1 && !W.tc_ok) throw std::runtime_error("op_linear: this matrix cannot take the tensor-core path (needs one scale/zero per row, M and K multiples of 128)");
        RSV_CUDA(cudaMalloc(&dx, (size_t)R * K * 4));
        RSV_CUDA(cudaMalloc(&dy, (size_t)R * M * 4));
        RSV_CUDA(cudaMemcpyAsync(dx, x_host, (size_t)R * K * 4, cudaMemcpyHostToDevice, m.stream));
        LinReq q = {&W, dx, K, dy, M, EPI_STORE};
        if (path == 1) {
            run_linear_tc(m, "op_linear", &q, 1, R);
        } else {
            run_linear_simt(m, "op_linear_simt", &q, 1, R);
        }
        RSV_CUDA(cudaMemcpyAsync(y_host, dy, (size_t)R * M * 4, cudaMemcpyDeviceToHost, m.stream));
        m.check_status();
    } catch (...) {
        cudaStreamSynchronize(m.stream);
        if (dx) cudaFree(dx);
        if (dy) cudaFree(dy);
        while (m.allocs.size() > first_alloc) {
            cudaFree(m.allocs.back());
            m.allocs.pop_back();
        }
        throw;
    }
    cudaFree(dx);
    cudaFree(dy);
    while (m.allocs.size() > first_alloc) {
        cudaFree(m.allocs.back());
        m.allocs.pop_back();
    }
}

// ------------------------------------------------------------------------------------------------
// Sampling without any allocation.  Some callers must not allocate device memory at the moment they
// sample: code running inside a memory-pool or arena discipline that forbids cudaMalloc on the hot
// path, latency-critical serving loops (cudaMalloc/cudaFree synchronise the device), and plugins that
// are handed device buffers by a host framework and may not own allocations of their own.  For them
// the sampler's work area lives in two file-scope device arrays that every GPU loading this library
// holds until the process exits: 2 x 4 MiB (kStaticSampleMaxElems floats + as many u32).
// ------------------------------------------------------------------------------------------------
constexpr size_t kStaticSampleMaxElems = size_t(1) << 20;  // rows * V <= 1,048,576 (e.g. 16 rows of a 65536 vocabulary)
static __device__ __align__(256) float g_static_sample_temp[kStaticSampleMaxElems];
static __device__ __align__(256) uint32_t g_static_sample_cnt[kStaticSampleMaxElems];

namespace {
struct StaticScratch {
    float* temp = nullptr;
    uint32_t* cnt = nullptr;
};
constexpr int kMaxDevices = 64;
StaticScratch g_static_scratch[kMaxDevices];
std::once_flag g_static_once[kMaxDevices];
}  // namespace

void set_last_error(const std::string& msg);  // defined with the C ABI

}  // namespace rsv

// The sampling kernel with its work area in static device memory; device pointers in, device pointer out.
// See include/rsv_b200.h for the contract.
extern "C" int rsv_op_sample_static(int device, void* stream, const float* logits_dev, int64_t rows, int64_t V, const float* sampler8_dev,
                                    const uint32_t* hist_dev, int64_t hist_stride, uint32_t* out_dev) {
    using namespace rsv;
    try {
        if (!logits_dev || !sampler8_dev || !out_dev) throw std::runtime_error("sample_static: null argument");
        if (rows < 1 || V < 1) throw std::runtime_error("sample_static: empty input");
        if (hist_stride < 0 || (hist_stride > 0 && !hist_dev)) throw std::runtime_error("sample_static: history is null but hist_stride > 0");
        if (hist_stride > 0x7fffffffLL || rows > 0x7fffffffLL || V > 0x7fffffffLL) throw std::runtime_error("sample_static: rows, V and hist_stride must fit in 31 bits");
        if ((uint64_t)rows * (uint64_t)V > kStaticSampleMaxElems)
            throw std::runtime_error("sample_static: rows * V = " + std::to_string((uint64_t)rows * (uint64_t)V) + " exceeds the static work area of " +
                                     std::to_string(kStaticSampleMaxElems) + " elements; use rsv_op_sample or fewer rows per call");
        if (device < 0 || device >= kMaxDevices) throw std::runtime_error("sample_static: device index out of range");
        RSV_CUDA(cudaSetDevice(device));
        StaticScratch& sc = g_static_scratch[device];
        // first call on this device: resolve the device addresses of the static arrays (in host code their names are only
        // handles, not device pointers).  Once per device, also when several host threads make their first call together.
        std::call_once(g_static_once[device], [&] {
            float* t = nullptr;
            uint32_t* c = nullptr;
            if (cudaGetSymbolAddress((void**)&t, g_static_sample_temp) == cudaSuccess && cudaGetSymbolAddress((void**)&c, g_static_sample_cnt) == cudaSuccess) {
                sc.cnt = c;
                sc.temp = t;
            }
        });
        if (!sc.temp || !sc.cnt) throw CudaError("sample_static: cudaGetSymbolAddress failed for the static work area");
        sample_rows_kernel<<<(unsigned)rows, kSampleThreads, 0, (cudaStream_t)stream>>>(logits_dev, (int)V, sampler8_dev, hist_stride ? hist_dev : nullptr,
                                                                                        (int)hist_stride, nullptr, sc.temp, sc.cnt, out_dev, nullptr,
                                                                                        nullptr, 0, nullptr);
        check_launch("sample_static");
        return 0;
    } catch (const CudaError& e) {
        set_last_error(e.what());
        return 2;
    } catch (const std::exception& e) {
        set_last_error(e.what());
        return 1;
    }
}
