// Shared definitions for the sm_100a RWKV-7 forward-step library.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>

namespace rsv {

// Numerical constants of the reference's CPU path (src/model.rs:6-8, :438).
constexpr float kLnEps = 1.0e-5f;
constexpr float kGnEps = 64.0e-5f;
constexpr float kL2Eps = 1.0e-12f;
constexpr float kDecayScale = -0.60653065971263342f;  // -1/sqrt(e)
constexpr int kHeadSize = 64;                         // the only head size RWKV-7 checkpoints use

struct CudaError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

#define RSV_CUDA(expr)                                                                                              \
    do {                                                                                                            \
        cudaError_t _e = (expr);                                                                                    \
        if (_e != cudaSuccess)                                                                                      \
            throw ::rsv::CudaError(std::string(#expr) + " failed: " + cudaGetErrorString(_e) + " (" __FILE__ ":" + \
                                   std::to_string(__LINE__) + ")");                                                 \
    } while (0)

enum WType : int { W_F16 = 0, W_INT8 = 1 };

// Epilogues of the weight-streaming linear kernel.  `acc` is the fp32 dot product for (row r, output m).
enum Epi : int {
    EPI_STORE = 0,         // y = acc
    EPI_ADD = 1,           // y += acc                                   (residual)
    EPI_RELU2 = 2,         // y = max(acc,0)^2                           (ffn.key)
    EPI_TANH = 3,          // y = tanh(acc)                              (decay adapter, rank space)
    EPI_SIGMOID = 4,       // y = sigmoid(acc)                           (gate adapter, rank space)
    EPI_DECAY = 5,         // y = exp(-sigmoid(acc + bias[m]) / sqrt(e)) (w)
    EPI_SIGMOID_BIAS = 6,  // y = sigmoid(acc + bias[m])                 (a)
    EPI_VLERP = 7,         // y = y + sigmoid(acc + bias[m]) * (aux[r,m] - y)   (v <- lerp(v, v_first, gate))
};

// Row r of a packed step: which session slot it belongs to and how it chains to its neighbours.
struct RowMeta {
    int slot;      // state slot of the session this row belongs to
    int has_prev;  // 1: row r-1 is the previous token of the same session; 0: previous token lives in the slot state
    int is_last;   // 1: last row of its session in this step -> writes the shift state
    int seg;       // index of the row's segment
};
// A segment = consecutive rows of one session (1 row for decode, up to the chunk length for prefill).
struct SegMeta {
    int start, len, slot, pad;
};

// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization attribute may start
// while its predecessor in the stream still runs; pdl_wait() blocks until that predecessor has completed and its
// memory is visible, pdl_launch_dependents() allows the successor to be scheduled.  Both are no-ops for a normal
// launch.  Rule used here: a kernel reads or writes nothing but its parameters and the model's weights (and state that
// only an earlier step wrote) before pdl_wait().
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// A pointer to data the predecessor produces, as seen after pdl_wait().  `const __restrict__` parameters promise the compiler
// that nobody writes the data while the kernel runs, so it may move their loads above the wait; passing the pointer through
// this (empty) asm after the wait makes every later load depend on it.
template <typename T>
__device__ __forceinline__ T* pdl_fresh(T* p) {
    asm volatile("" : "+l"(p)::"memory");
    return p;
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace rsv
