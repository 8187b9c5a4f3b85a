// Host-side plumbing shared by the translation units of libslideformer_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "sf_kernels.cuh"
#include "slideformer_b200.h"

namespace sf {

// Records `msg` as the calling thread's last error and returns `code`.
int fail(int code, const std::string& msg);
// cudaGetLastError() after a launch; counts the launch when it succeeded.
int check_launch(const char* what);

struct DevInfo {
    int sms = 0;
};
int device_info(DevInfo* out);

struct Tuning {
    int variant = 1;      // 0: 128-bit default caching, 1: 128-bit streaming hints, 2: 256-bit
    int ctas_per_sm = 0;  // 0: one tile per CTA (measured best: the hardware CTA scheduler keeps
                          // loads and stores of different CTAs interleaved); k > 0: persistent
                          // grid of SMs * k CTAs walking the tiles
    int push_vec = 8;     // elements per thread of the fused pull+push kernel: 4 or 8
    int push_world = 1;   // 1: kernels specialised for world 2 / 4 / 8; 0: runtime world only
    uint64_t host_piece = 8u << 20;  // elements per copy / launch piece of the host-streaming pipeline
    int nvls_groups = 1;  // 8-element groups per thread of the NVLS kernel: 1, 2 or 4 (measured equal: 0.90 ms at 8 GPUs)
};
extern Tuning g_tune;

inline bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

inline int grid_for(uint64_t ntiles, int sms, int ctas_per_sm)
{
    uint64_t cap = ctas_per_sm > 0 ? (uint64_t)sms * (uint64_t)ctas_per_sm : (uint64_t)0x7fffffff;
    uint64_t g = ntiles < cap ? ntiles : cap;
    return (int)(g < 1 ? 1 : g);
}

// A vector kernel leaves [nvec, n) to scalar code; beyond this many elements the launchers use
// the grid-wide scalar kernel instead (a reference call leaves at most 15).
constexpr uint64_t kMaxVectorRemainder = 64;

#define SF_CUDA(call)                                                                           \
    do {                                                                                        \
        cudaError_t e_ = (call);                                                                \
        if (e_ != cudaSuccess)                                                                  \
            return ::sf::fail(SF_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)); \
    } while (0)

// What one launch needs besides the arrays.
struct StepCtx {
    sfk::K c;
    int mode;            // sfk::MODE_*
    bool ex;             // gradient multiplier and / or statistics requested
    SfGradStats* stats;  // device pointer or NULL
};
int make_ctx(const SfAdamScalars* s, StepCtx* out);

// Peer-memory launchers (sf_adam_dp.cu).  Arguments are validated by the callers.
int launch_sharded(const StepCtx& x, float* p, const void* const* peer_g, int world, int g_dtype, float* m,
                   float* v, uint16_t* out, uint64_t n, uint64_t vec_n, bool a16, cudaStream_t st);
int launch_push(const StepCtx& x, float* p, const void* const* peer_g, uint16_t* const* peer_out, int world,
                int g_dtype, float* m, float* v, uint64_t n, uint64_t vec_n, bool a16, cudaStream_t st);
int launch_push_multi(const sfk::SegTable& table, int total_ctas, int mode, bool ex, SfGradStats* stats, int g_dtype,
                      cudaStream_t st);
int launch_nvls(const StepCtx& x, float* p, const void* mc_g, uint16_t* mc_out, const void* const* peer_g,
                uint16_t* const* peer_out, int world, float* m, float* v, uint64_t n, uint64_t vec_n,
                cudaStream_t st);
int launch_copy16(void* dst, const void* src, uint64_t n16, cudaStream_t st);
int launch_mean(const void* const* peer_g, int world, int g_dtype, float* mean, uint64_t n, bool a16,
                cudaStream_t st);

}  // namespace sf
