// Fused LayerAdam step for B200 (sm_100a): kernels and the C ABI declared in
// include/slideformer_b200.h.
//
// One pass over a layer's flat vectors: read fp32 p, m, v and the bf16 (or fp32) gradient,
// apply the Adam / AdamW update in registers with single-rounded IEEE binary32 operations in
// the order of the reference's AVX-512 loop (optimizer/layer_adam/csrc/cpu_adam.h:158-193),
// write p, m, v back and emit the round-to-nearest-even bf16 copy of the new p.  28 bytes
// move per parameter (14 read, 14 written) and nothing is reused, so the kernel is bound by
// HBM bandwidth; there is no GEMM-shaped work here and the tensor cores are not involved.
//
// Bit parity rules followed everywhere below:
//   * only __fmul_rn / __fmaf_rn / __fadd_rn / __fsqrt_rn / __fdiv_rn, never a plain * or +
//     on floats, so the compiler can neither fuse nor reorder; no fast-math flags;
//   * elements at or above vec_n use the contraction the reference's compiled scalar tail
//     uses (cpu_adam_impl.cpp:46-66): m = fma(m, b1, g*(1-b1)), v = fma(v, b2, (g*g)*(1-b2));
//   * bf16 output: RNE on the upper 16 bits, every NaN becomes 0x7FC0 (simd.h:56-86).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>
#include <cmath>
#include <cstring>
#include <mutex>
#include <string>
#include <type_traits>
#include <unordered_map>

#include "slideformer_b200.h"

namespace {

// ------------------------------------------------------------------------------------------
// error plumbing
// ------------------------------------------------------------------------------------------
thread_local std::string t_err;
std::atomic<uint64_t> g_launches{0};

int fail(int code, const std::string& msg)
{
    t_err = msg;
    return code;
}

#define SF_CUDA(call)                                                                       \
    do {                                                                                    \
        cudaError_t e_ = (call);                                                            \
        if (e_ != cudaSuccess)                                                              \
            return fail(SF_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_));   \
    } while (0)

// ------------------------------------------------------------------------------------------
// host scalar state machine (cpu_adam.h:24-106)
// ------------------------------------------------------------------------------------------
struct HostAdam {
    float alpha, betta1, betta2, eps, weight_decay;
    float betta1_t, betta2_t;
    uint64_t step;
    float bc1, bc2;
    bool adamw;
};

std::mutex g_mu;
std::unordered_map<int, HostAdam> g_opts;

// cpu_adam.h:57-76.  The pow() there takes (float, size_t): both promote to double and the
// result narrows to float on assignment.
void increment_step(HostAdam& o, uint64_t step, float beta1, float beta2)
{
    if (beta1 != o.betta1 || beta2 != o.betta2) {
        o.step = step;
        o.betta1 = beta1;
        o.betta2 = beta2;
        o.betta1_t = (float)std::pow((double)o.betta1, (double)step);
        o.betta2_t = (float)std::pow((double)o.betta2, (double)step);
    } else {
        o.step++;
        if (o.step != step) {
            o.betta1_t = (float)std::pow((double)o.betta1, (double)step);
            o.betta2_t = (float)std::pow((double)o.betta2, (double)step);
            o.step = step;
        } else {
            o.betta1_t = o.betta1_t * o.betta1;
            o.betta2_t = o.betta2_t * o.betta2;
        }
    }
}

// cpu_adam.h:77-89, then the constants of cpu_adam.h:131-148.
void update_state(HostAdam& o, float lr, float eps, float wd, int bias_correction, SfAdamScalars* s)
{
    o.alpha = lr;
    o.eps = eps;
    o.weight_decay = wd;
    o.bc1 = 1.0f;
    o.bc2 = 1.0f;
    if (bias_correction == 1) {
        o.bc1 = 1 - o.betta1_t;
        o.bc2 = 1 / sqrtf(1 - o.betta2_t);
    }
    s->beta1 = o.betta1;
    s->beta2 = o.betta2;
    s->omb1 = 1 - o.betta1;
    s->omb2 = 1 - o.betta2;
    s->bc2 = o.bc2;
    s->eps = o.eps;
    s->step_size = -1 * o.alpha / o.bc1;
    s->w_decay = -1 * o.alpha * o.weight_decay;
    s->weight_decay = o.weight_decay;
    s->adamw_mode = o.adamw ? 1 : 0;
}

// ------------------------------------------------------------------------------------------
// device arithmetic
// ------------------------------------------------------------------------------------------
enum { MODE_NODECAY = 0, MODE_ADAMW = 1, MODE_L2 = 2 };

struct K {  // kernel-side constants
    float b1, b2, omb1, omb2, bc2, eps, step_size, w_decay, wd;
};

template <int MODE>
__device__ __forceinline__ void adam_body(const K& c, float& p, float g, float& m, float& v)
{
    if (MODE == MODE_L2) g = __fmaf_rn(p, c.wd, g);
    m = __fmul_rn(m, c.b1);
    m = __fmaf_rn(g, c.omb1, m);
    v = __fmul_rn(v, c.b2);
    float g2 = __fmul_rn(g, g);
    v = __fmaf_rn(g2, c.omb2, v);
    float d = __fsqrt_rn(v);
    d = __fmaf_rn(d, c.bc2, c.eps);
    float u = __fdiv_rn(m, d);
    if (MODE == MODE_ADAMW) p = __fmaf_rn(p, c.w_decay, p);
    p = __fmaf_rn(u, c.step_size, p);
}

template <int MODE>
__device__ __forceinline__ void adam_tail(const K& c, float& p, float g, float& m, float& v)
{
    if (MODE == MODE_L2) g = __fmaf_rn(p, c.wd, g);
    float t1 = __fmul_rn(g, c.omb1);
    m = __fmaf_rn(m, c.b1, t1);
    float g2 = __fmul_rn(g, g);
    float t2 = __fmul_rn(g2, c.omb2);
    v = __fmaf_rn(v, c.b2, t2);
    float d = __fsqrt_rn(v);
    d = __fmaf_rn(d, c.bc2, c.eps);
    float u = __fdiv_rn(m, d);
    if (MODE == MODE_ADAMW) p = __fmaf_rn(c.w_decay, p, p);
    p = __fmaf_rn(u, c.step_size, p);
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }

__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f)
{
    uint32_t u = __float_as_uint(f);
    uint32_t r = (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
    return ((u & 0x7fffffffu) > 0x7f800000u) ? 0x7fc0u : r;
}

// two floats -> packed bf16x2 (lo in the low half).  cvt.rn.bf16x2.f32 rounds to nearest
// even like the integer formula; only NaN differs (0x7FFF), so NaN lanes are patched.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    if (lo != lo) r = (r & 0xffff0000u) | 0x7fc0u;
    if (hi != hi) r = (r & 0x0000ffffu) | 0x7fc00000u;
    return r;
}

// ---- global memory access flavours -------------------------------------------------------
// HINT 0: default caching.  HINT 1: streaming (evict-first) on every access; nothing in this
// kernel is read twice.
template <int HINT>
__device__ __forceinline__ float4 ld4(const float* a)
{
    if (HINT == 1) return __ldcs(reinterpret_cast<const float4*>(a));
    return *reinterpret_cast<const float4*>(a);
}
template <int HINT>
__device__ __forceinline__ uint2 ld2u(const void* a)
{
    if (HINT == 1) return __ldcs(reinterpret_cast<const uint2*>(a));
    return *reinterpret_cast<const uint2*>(a);
}
template <int HINT>
__device__ __forceinline__ void st4(float* a, float4 x)
{
    if (HINT == 1) __stcs(reinterpret_cast<float4*>(a), x);
    else *reinterpret_cast<float4*>(a) = x;
}
template <int HINT>
__device__ __forceinline__ void st2u(void* a, uint2 x)
{
    if (HINT == 1) __stcs(reinterpret_cast<uint2*>(a), x);
    else *reinterpret_cast<uint2*>(a) = x;
}

struct f8 {
    float x[8];
};
// 256-bit global accesses (sm_100+).
__device__ __forceinline__ f8 ld8(const float* a)
{
    f8 r;
    asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.x[0]), "=f"(r.x[1]), "=f"(r.x[2]), "=f"(r.x[3]), "=f"(r.x[4]),
                   "=f"(r.x[5]), "=f"(r.x[6]), "=f"(r.x[7])
                 : "l"(a));
    return r;
}
__device__ __forceinline__ void st8(float* a, const f8& r)
{
    asm volatile("st.global.v8.f32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};" ::"f"(r.x[0]), "f"(r.x[1]),
                 "f"(r.x[2]), "f"(r.x[3]), "f"(r.x[4]), "f"(r.x[5]), "f"(r.x[6]), "f"(r.x[7]),
                 "l"(a)
                 : "memory");
}

// Gradient sources.  `load4` returns 4 consecutive gradients as floats.
struct GradBf16 {
    static constexpr bool kPeer = false;
    const uint16_t* g;
    template <int HINT>
    __device__ __forceinline__ void load4(uint64_t i, float (&o)[4]) const
    {
        uint2 r = ld2u<HINT>(g + i);
        o[0] = bf16_bits_to_f32(r.x & 0xffffu);
        o[1] = bf16_bits_to_f32(r.x >> 16);
        o[2] = bf16_bits_to_f32(r.y & 0xffffu);
        o[3] = bf16_bits_to_f32(r.y >> 16);
    }
    __device__ __forceinline__ float load1(uint64_t i) const { return bf16_bits_to_f32(g[i]); }
};
struct GradF32 {
    static constexpr bool kPeer = false;
    const float* g;
    template <int HINT>
    __device__ __forceinline__ void load4(uint64_t i, float (&o)[4]) const
    {
        float4 r = ld4<HINT>(g + i);
        o[0] = r.x; o[1] = r.y; o[2] = r.z; o[3] = r.w;
    }
    __device__ __forceinline__ float load1(uint64_t i) const { return g[i]; }
};

#define SF_MAX_WORLD 16
// Rank-ordered fp32 mean over peer-mapped gradients (shared_data_parallel.py:130-133):
// zero accumulator, add rank 0..world-1, true division by world.
template <typename ELT>
struct GradPeers {
    static constexpr bool kPeer = true;
    const ELT* g[SF_MAX_WORLD];
    int world;
    float fworld;
    template <int HINT>
    __device__ __forceinline__ void load4(uint64_t i, float (&o)[4]) const
    {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int r = 0; r < world; r++) {
            float t[4];
            if (sizeof(ELT) == 2) {
                uint2 q = ld2u<HINT>(g[r] + i);
                t[0] = bf16_bits_to_f32(q.x & 0xffffu);
                t[1] = bf16_bits_to_f32(q.x >> 16);
                t[2] = bf16_bits_to_f32(q.y & 0xffffu);
                t[3] = bf16_bits_to_f32(q.y >> 16);
            } else {
                float4 q = ld4<HINT>(reinterpret_cast<const float*>(g[r]) + i);
                t[0] = q.x; t[1] = q.y; t[2] = q.z; t[3] = q.w;
            }
#pragma unroll
            for (int k = 0; k < 4; k++) acc[k] = __fadd_rn(acc[k], t[k]);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) o[k] = __fdiv_rn(acc[k], fworld);
    }
    __device__ __forceinline__ float load1(uint64_t i) const
    {
        float acc = 0.f;
        for (int r = 0; r < world; r++) {
            float t;
            if (sizeof(ELT) == 2) t = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(g[r])[i]);
            else t = reinterpret_cast<const float*>(g[r])[i];
            acc = __fadd_rn(acc, t);
        }
        return __fdiv_rn(acc, fworld);
    }
};

// ------------------------------------------------------------------------------------------
// kernels
// ------------------------------------------------------------------------------------------

// Elements outside the vector range, one per thread-iteration.  Also the whole-array path
// for buffers that are not 16-byte aligned.
template <typename GS, int MODE, bool OUT>
__device__ __forceinline__ void scalar_range(const K& c, float* p, const GS& gs, float* m, float* v,
                                             uint16_t* out, uint64_t lo, uint64_t hi, uint64_t vec_n,
                                             uint64_t tid, uint64_t nthreads)
{
    for (uint64_t i = lo + tid; i < hi; i += nthreads) {
        float pp = p[i], mm = m[i], vv = v[i];
        float g = gs.load1(i);
        if (i < vec_n) adam_body<MODE>(c, pp, g, mm, vv);
        else adam_tail<MODE>(c, pp, g, mm, vv);
        p[i] = pp; m[i] = mm; v[i] = vv;
        if (OUT) out[i] = (uint16_t)f32_to_bf16_bits(pp);
    }
}

template <typename GS, int MODE, bool OUT>
__global__ void __launch_bounds__(256)
adam_scalar_kernel(K c, float* p, GS gs, float* m, float* v, uint16_t* out, uint64_t n, uint64_t vec_n)
{
    scalar_range<GS, MODE, OUT>(c, p, gs, m, v, out, 0, n, vec_n,
                                (uint64_t)blockIdx.x * blockDim.x + threadIdx.x,
                                (uint64_t)gridDim.x * blockDim.x);
}

// 128-bit kernel.  A CTA walks tiles of THREADS*4*U elements; inside a tile, sub-iteration u
// of thread t covers the 4 elements at tile + (u*THREADS + t)*4, so every load and store
// instruction of a warp touches one contiguous, fully used 512-byte (fp32) or 256-byte (bf16)
// span.  All U loads of p, m, v, g are issued before the arithmetic to keep
// U * 56 bytes per thread in flight.
//   nvec    = elements handled here, a multiple of 4, all below vec_n (body arithmetic)
//   [nvec, n) is finished by the last CTA with scalar accesses.
template <typename GS, int MODE, bool OUT, int HINT, int U, int THREADS, int MINB = 1>
__global__ void __launch_bounds__(THREADS, MINB)
adam_vec4_kernel(K c, float* __restrict__ p, GS gs, float* __restrict__ m, float* __restrict__ v,
                 uint16_t* __restrict__ out, uint64_t nvec, uint64_t n, uint64_t vec_n)
{
    constexpr uint64_t TILE = (uint64_t)THREADS * 4 * U;
    const uint64_t ntiles = (nvec + TILE - 1) / TILE;
    for (uint64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const uint64_t base = tile * TILE + (uint64_t)threadIdx.x * 4;
        float4 P[U], M[U], V[U];
        float G[U][4];
        bool ok[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint64_t i = base + (uint64_t)u * THREADS * 4;
            ok[u] = i < nvec;
            if (ok[u]) {
                P[u] = ld4<HINT>(p + i);
                M[u] = ld4<HINT>(m + i);
                V[u] = ld4<HINT>(v + i);
                gs.template load4<HINT>(i, G[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint64_t i = base + (uint64_t)u * THREADS * 4;
            if (ok[u]) {
                adam_body<MODE>(c, P[u].x, G[u][0], M[u].x, V[u].x);
                adam_body<MODE>(c, P[u].y, G[u][1], M[u].y, V[u].y);
                adam_body<MODE>(c, P[u].z, G[u][2], M[u].z, V[u].z);
                adam_body<MODE>(c, P[u].w, G[u][3], M[u].w, V[u].w);
                st4<HINT>(p + i, P[u]);
                st4<HINT>(m + i, M[u]);
                st4<HINT>(v + i, V[u]);
                if (OUT) {
                    uint2 o;
                    o.x = pack_bf16x2(P[u].x, P[u].y);
                    o.y = pack_bf16x2(P[u].z, P[u].w);
                    st2u<HINT>(out + i, o);
                }
            }
        }
    }
    if (blockIdx.x == gridDim.x - 1)
        scalar_range<GS, MODE, OUT>(c, p, gs, m, v, out, nvec, n, vec_n, threadIdx.x, THREADS);
}

// 256-bit kernel (bf16 or fp32 gradient in local memory only): thread t of a tile owns 8
// consecutive elements, p / m / v move as one 32-byte access each, the bf16 gradient and the
// bf16 output as one 16-byte access each.
template <bool G_BF16, int MODE, bool OUT, int U, int THREADS>
__global__ void __launch_bounds__(THREADS)
adam_vec8_kernel(K c, float* __restrict__ p, const void* __restrict__ gptr, float* __restrict__ m,
                 float* __restrict__ v, uint16_t* __restrict__ out, uint64_t nvec, uint64_t n,
                 uint64_t vec_n)
{
    constexpr uint64_t TILE = (uint64_t)THREADS * 8 * U;
    const uint64_t ntiles = (nvec + TILE - 1) / TILE;
    for (uint64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const uint64_t base = tile * TILE + (uint64_t)threadIdx.x * 8;
        f8 P[U], M[U], V[U], G[U];
        bool ok[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint64_t i = base + (uint64_t)u * THREADS * 8;
            ok[u] = i < nvec;
            if (ok[u]) {
                P[u] = ld8(p + i);
                M[u] = ld8(m + i);
                V[u] = ld8(v + i);
                if (G_BF16) {
                    uint4 r = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(gptr) + i);
                    G[u].x[0] = bf16_bits_to_f32(r.x & 0xffffu); G[u].x[1] = bf16_bits_to_f32(r.x >> 16);
                    G[u].x[2] = bf16_bits_to_f32(r.y & 0xffffu); G[u].x[3] = bf16_bits_to_f32(r.y >> 16);
                    G[u].x[4] = bf16_bits_to_f32(r.z & 0xffffu); G[u].x[5] = bf16_bits_to_f32(r.z >> 16);
                    G[u].x[6] = bf16_bits_to_f32(r.w & 0xffffu); G[u].x[7] = bf16_bits_to_f32(r.w >> 16);
                } else {
                    G[u] = ld8(reinterpret_cast<const float*>(gptr) + i);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint64_t i = base + (uint64_t)u * THREADS * 8;
            if (ok[u]) {
#pragma unroll
                for (int k = 0; k < 8; k++)
                    adam_body<MODE>(c, P[u].x[k], G[u].x[k], M[u].x[k], V[u].x[k]);
                st8(p + i, P[u]);
                st8(m + i, M[u]);
                st8(v + i, V[u]);
                if (OUT) {
                    uint4 o;
                    o.x = pack_bf16x2(P[u].x[0], P[u].x[1]);
                    o.y = pack_bf16x2(P[u].x[2], P[u].x[3]);
                    o.z = pack_bf16x2(P[u].x[4], P[u].x[5]);
                    o.w = pack_bf16x2(P[u].x[6], P[u].x[7]);
                    *reinterpret_cast<uint4*>(out + i) = o;
                }
            }
        }
    }
    if (blockIdx.x == gridDim.x - 1) {
        if (G_BF16) {
            GradBf16 gs{reinterpret_cast<const uint16_t*>(gptr)};
            scalar_range<GradBf16, MODE, OUT>(c, p, gs, m, v, out, nvec, n, vec_n, threadIdx.x, THREADS);
        } else {
            GradF32 gs{reinterpret_cast<const float*>(gptr)};
            scalar_range<GradF32, MODE, OUT>(c, p, gs, m, v, out, nvec, n, vec_n, threadIdx.x, THREADS);
        }
    }
}

// Fused data-parallel step: gradient mean pulled from every rank, Adam on the owned slice, and
// the bf16 result PUSHED into every rank's copy of the layer, all in one kernel.  The bf16
// stores go to `world` destinations (local and peer-mapped); with NVLink full duplex the pushes
// (egress) overlap the gradient pulls (ingress), and no separate all-gather pass is needed.
struct PushDst {
    uint16_t* out[SF_MAX_WORLD];
    int world;
};

template <typename GS, int MODE, int U, int THREADS, int MINB = 1>
__global__ void __launch_bounds__(THREADS, MINB)
adam_vec4_push_kernel(K c, float* __restrict__ p, GS gs, float* __restrict__ m, float* __restrict__ v,
                      PushDst dst, uint64_t nvec, uint64_t n, uint64_t vec_n)
{
    constexpr uint64_t TILE = (uint64_t)THREADS * 4 * U;
    const uint64_t ntiles = (nvec + TILE - 1) / TILE;
    for (uint64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const uint64_t base = tile * TILE + (uint64_t)threadIdx.x * 4;
        float4 P[U], M[U], V[U];
        float G[U][4];
        bool ok[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint64_t i = base + (uint64_t)u * THREADS * 4;
            ok[u] = i < nvec;
            if (ok[u]) {
                gs.template load4<1>(i, G[u]);   // the long-latency peer reads go first
                P[u] = ld4<1>(p + i);
                M[u] = ld4<1>(m + i);
                V[u] = ld4<1>(v + i);
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint64_t i = base + (uint64_t)u * THREADS * 4;
            if (ok[u]) {
                adam_body<MODE>(c, P[u].x, G[u][0], M[u].x, V[u].x);
                adam_body<MODE>(c, P[u].y, G[u][1], M[u].y, V[u].y);
                adam_body<MODE>(c, P[u].z, G[u][2], M[u].z, V[u].z);
                adam_body<MODE>(c, P[u].w, G[u][3], M[u].w, V[u].w);
                st4<1>(p + i, P[u]);
                st4<1>(m + i, M[u]);
                st4<1>(v + i, V[u]);
                uint2 o;
                o.x = pack_bf16x2(P[u].x, P[u].y);
                o.y = pack_bf16x2(P[u].z, P[u].w);
                for (int r = 0; r < dst.world; r++) *reinterpret_cast<uint2*>(dst.out[r] + i) = o;
            }
        }
    }
    if (blockIdx.x == gridDim.x - 1) {
        for (uint64_t i = nvec + threadIdx.x; i < n; i += THREADS) {
            float pp = p[i], mm = m[i], vv = v[i];
            float g = gs.load1(i);
            if (i < vec_n) adam_body<MODE>(c, pp, g, mm, vv);
            else adam_tail<MODE>(c, pp, g, mm, vv);
            p[i] = pp; m[i] = mm; v[i] = vv;
            const uint16_t o = (uint16_t)f32_to_bf16_bits(pp);
            for (int r = 0; r < dst.world; r++) dst.out[r][i] = o;
        }
    }
}

// fp32 rank-ordered mean of the peers' gradients, 4 elements per thread-iteration.
template <typename GS>
__global__ void __launch_bounds__(256)
dp_mean_kernel(GS gs, float* __restrict__ mean, uint64_t nvec, uint64_t n)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x * 4;
    for (uint64_t i = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < nvec; i += stride) {
        float o[4];
        gs.template load4<1>(i, o);
        __stcs(reinterpret_cast<float4*>(mean + i), make_float4(o[0], o[1], o[2], o[3]));
    }
    if (blockIdx.x == gridDim.x - 1)
        for (uint64_t i = nvec + threadIdx.x; i < n; i += blockDim.x) mean[i] = gs.load1(i);
}

// ------------------------------------------------------------------------------------------
// launch plumbing
// ------------------------------------------------------------------------------------------
struct Tuning {
    int variant = 1;      // 0: 128-bit default caching, 1: 128-bit streaming hints, 2: 256-bit
    int ctas_per_sm = 0;  // 0: one tile per CTA (measured best: the hardware CTA scheduler keeps
                          // loads and stores of different CTAs interleaved); k > 0: persistent
                          // grid of SMs * k CTAs walking the tiles
};
Tuning g_tune;

struct DevInfo {
    int sms = 0;
};
std::mutex g_dev_mu;
std::unordered_map<int, DevInfo> g_dev;

int device_info(DevInfo* out)
{
    int dev = 0;
    SF_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_dev_mu);
    auto it = g_dev.find(dev);
    if (it == g_dev.end()) {
        DevInfo d;
        SF_CUDA(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev));
        it = g_dev.emplace(dev, d).first;
    }
    *out = it->second;
    return SF_OK;
}

inline bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

K make_k(const SfAdamScalars* s, int* mode)
{
    K c{s->beta1, s->beta2, s->omb1, s->omb2, s->bc2, s->eps, s->step_size, s->w_decay, s->weight_decay};
    // cpu_adam.h:171 and :186: decay only when _weight_decay > 0.
    *mode = (s->weight_decay > 0) ? (s->adamw_mode ? MODE_ADAMW : MODE_L2) : MODE_NODECAY;
    return c;
}

template <typename F>
int dispatch_mode_out(int mode, bool has_out, F&& f)
{
    // f<MODE, OUT>() via integral constants
    switch (mode * 2 + (has_out ? 1 : 0)) {
        case 0: return f(std::integral_constant<int, 0>{}, std::false_type{});
        case 1: return f(std::integral_constant<int, 0>{}, std::true_type{});
        case 2: return f(std::integral_constant<int, 1>{}, std::false_type{});
        case 3: return f(std::integral_constant<int, 1>{}, std::true_type{});
        case 4: return f(std::integral_constant<int, 2>{}, std::false_type{});
        default: return f(std::integral_constant<int, 2>{}, std::true_type{});
    }
}

int grid_for(uint64_t ntiles, int sms, int ctas_per_sm)
{
    uint64_t cap = ctas_per_sm > 0 ? (uint64_t)sms * (uint64_t)ctas_per_sm : (uint64_t)0x7fffffff;
    uint64_t g = ntiles < cap ? ntiles : cap;
    return (int)(g < 1 ? 1 : g);
}

int check_launch(const char* what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(SF_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return SF_OK;
}

// Launch the 128-bit kernel for any gradient source.
template <typename GS>
int launch_vec4(const K& c, int mode, float* p, const GS& gs, float* m, float* v, uint16_t* out,
                uint64_t n, uint64_t vec_n, cudaStream_t st, int hint)
{
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    const uint64_t nvec = (vec_n < n ? vec_n : n) & ~(uint64_t)3;
    const int cps = g_tune.ctas_per_sm;
    return dispatch_mode_out(mode, out != nullptr, [&](auto MODE, auto OUT) -> int {
        constexpr int M = decltype(MODE)::value;
        constexpr bool O = decltype(OUT)::value;
        // Local gradients: two 4-element groups per thread at half occupancy is the fastest HBM
        // shape.  Peer-mapped gradients: one group per thread at full occupancy (32 registers)
        // hides the NVLink read latency (measured with the push kernel, which shares the shape).
        constexpr bool PEER = GS::kPeer;
        constexpr int U = PEER ? 1 : 2, T = 256, MINB = PEER ? 8 : 1;
        uint64_t ntiles = (nvec + (uint64_t)T * 4 * U - 1) / ((uint64_t)T * 4 * U);
        int grid = grid_for(ntiles, di.sms, cps);
        if (hint)
            adam_vec4_kernel<GS, M, O, 1, U, T, MINB><<<grid, T, 0, st>>>(c, p, gs, m, v, out, nvec, n, vec_n);
        else
            adam_vec4_kernel<GS, M, O, 0, U, T, MINB><<<grid, T, 0, st>>>(c, p, gs, m, v, out, nvec, n, vec_n);
        return check_launch("adam_vec4_kernel");
    });
}

template <typename GS>
int launch_scalar(const K& c, int mode, float* p, const GS& gs, float* m, float* v, uint16_t* out,
                  uint64_t n, uint64_t vec_n, cudaStream_t st)
{
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    uint64_t blocks = (n + 255) / 256;
    int grid = grid_for(blocks, di.sms, 8);
    return dispatch_mode_out(mode, out != nullptr, [&](auto MODE, auto OUT) -> int {
        constexpr int M = decltype(MODE)::value;
        constexpr bool O = decltype(OUT)::value;
        adam_scalar_kernel<GS, M, O><<<grid, 256, 0, st>>>(c, p, gs, m, v, out, n, vec_n);
        return check_launch("adam_scalar_kernel");
    });
}

template <bool G_BF16>
int launch_vec8(const K& c, int mode, float* p, const void* g, float* m, float* v, uint16_t* out,
                uint64_t n, uint64_t vec_n, cudaStream_t st)
{
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    const uint64_t nvec = (vec_n < n ? vec_n : n) & ~(uint64_t)7;
    const int cps = g_tune.ctas_per_sm;
    return dispatch_mode_out(mode, out != nullptr, [&](auto MODE, auto OUT) -> int {
        constexpr int M = decltype(MODE)::value;
        constexpr bool O = decltype(OUT)::value;
        constexpr int U = 1, T = 256;
        uint64_t ntiles = (nvec + (uint64_t)T * 8 * U - 1) / ((uint64_t)T * 8 * U);
        int grid = grid_for(ntiles, di.sms, cps);
        adam_vec8_kernel<G_BF16, M, O, U, T><<<grid, T, 0, st>>>(c, p, g, m, v, out, nvec, n, vec_n);
        return check_launch("adam_vec8_kernel");
    });
}

int step_impl(const SfAdamScalars* s, float* p, const void* g, int g_dtype, float* m, float* v,
              uint16_t* out, uint64_t n, uint64_t vec_n, cudaStream_t st)
{
    if (!s) return fail(SF_ERR_NULL, "scalars pointer is NULL");
    if (g_dtype != SF_GRAD_BF16 && g_dtype != SF_GRAD_F32)
        return fail(SF_ERR_DTYPE, "gradient dtype code " + std::to_string(g_dtype) + " is not supported (0 = bf16, 1 = fp32)");
    if (n == 0) return SF_OK;
    if (!p || !g || !m || !v) return fail(SF_ERR_NULL, "p, g, m and v must be non-NULL when n > 0");
    if (n > ((uint64_t)1 << 40)) return fail(SF_ERR_SIZE, "n exceeds 2^40 elements");
    if (!aligned(p, 4) || !aligned(m, 4) || !aligned(v, 4) || !aligned(g, g_dtype == SF_GRAD_BF16 ? 2 : 4) ||
        !aligned(out, 2))
        return fail(SF_ERR_ALIGN, "a buffer is not aligned to its element size");
    if (vec_n > n) vec_n = n;
    int mode;
    K c = make_k(s, &mode);
    const bool a16 = aligned(p, 16) && aligned(m, 16) && aligned(v, 16) && aligned(g, 16) && aligned(out, 16);
    const bool a32 = a16 && aligned(p, 32) && aligned(m, 32) && aligned(v, 32);
    if (!a16 || n < 4) {
        if (g_dtype == SF_GRAD_BF16)
            return launch_scalar(c, mode, p, GradBf16{(const uint16_t*)g}, m, v, out, n, vec_n, st);
        return launch_scalar(c, mode, p, GradF32{(const float*)g}, m, v, out, n, vec_n, st);
    }
    const int variant = g_tune.variant;
    if (variant == 2 && a32 && (g_dtype == SF_GRAD_BF16 || aligned(g, 32))) {
        if (g_dtype == SF_GRAD_BF16) return launch_vec8<true>(c, mode, p, g, m, v, out, n, vec_n, st);
        return launch_vec8<false>(c, mode, p, g, m, v, out, n, vec_n, st);
    }
    const int hint = variant == 0 ? 0 : 1;
    if (g_dtype == SF_GRAD_BF16)
        return launch_vec4(c, mode, p, GradBf16{(const uint16_t*)g}, m, v, out, n, vec_n, st, hint);
    return launch_vec4(c, mode, p, GradF32{(const float*)g}, m, v, out, n, vec_n, st, hint);
}

// ---- host-streaming resources: three side streams and per-slot events, one set per device ---
struct HostPipe {
    cudaStream_t s_in = nullptr, s_k = nullptr, s_out = nullptr;
    cudaEvent_t ev_start = nullptr, ev_in[2] = {nullptr, nullptr}, ev_k[2] = {nullptr, nullptr},
                ev_out[2] = {nullptr, nullptr}, ev_done = nullptr;
    bool ready = false;
};
std::mutex g_pipe_mu;
std::unordered_map<int, HostPipe> g_pipes;

int get_pipe(HostPipe** out)
{
    int dev = 0;
    SF_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_pipe_mu);
    HostPipe& hp = g_pipes[dev];
    if (!hp.ready) {
        SF_CUDA(cudaStreamCreateWithFlags(&hp.s_in, cudaStreamNonBlocking));
        SF_CUDA(cudaStreamCreateWithFlags(&hp.s_k, cudaStreamNonBlocking));
        SF_CUDA(cudaStreamCreateWithFlags(&hp.s_out, cudaStreamNonBlocking));
        SF_CUDA(cudaEventCreateWithFlags(&hp.ev_start, cudaEventDisableTiming));
        SF_CUDA(cudaEventCreateWithFlags(&hp.ev_done, cudaEventDisableTiming));
        for (int i = 0; i < 2; i++) {
            SF_CUDA(cudaEventCreateWithFlags(&hp.ev_in[i], cudaEventDisableTiming));
            SF_CUDA(cudaEventCreateWithFlags(&hp.ev_k[i], cudaEventDisableTiming));
            SF_CUDA(cudaEventCreateWithFlags(&hp.ev_out[i], cudaEventDisableTiming));
        }
        hp.ready = true;
    }
    *out = &hp;
    return SF_OK;
}

size_t round256(size_t x) { return (x + 255) & ~(size_t)255; }

// ---- scratch for the entry point that must not allocate ------------------------------------
// Reserved in the library image itself: every GPU that loads the library carries these 16 MiB
// until the process exits.  The name below is only a handle on the host; the device address
// comes from cudaGetSymbolAddress, once per device, with that device current.
constexpr uint64_t kStaticMeanMaxElems = SF_STATIC_SCRATCH_MAX_ELEMS;  // 4 Mi fp32 values = 16 MiB
static __device__ __align__(256) float g_static_mean[kStaticMeanMaxElems];

std::mutex g_static_mu;
std::unordered_map<int, float*> g_static_addr;  // device ordinal -> device address of g_static_mean

int static_mean_address(float** out)
{
    int dev = 0;
    SF_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_static_mu);
    auto it = g_static_addr.find(dev);
    if (it == g_static_addr.end()) {
        float* ptr = nullptr;
        SF_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_mean));
        if (!ptr) return fail(SF_ERR_CUDA, "cudaGetSymbolAddress returned a NULL address for the static scratch");
        it = g_static_addr.emplace(dev, ptr).first;
    }
    *out = it->second;
    return SF_OK;
}

}  // namespace

// ==========================================================================================
// C ABI
// ==========================================================================================
extern "C" {

int sf_adam_create(int id, float lr, float beta1, float beta2, float eps, float weight_decay,
                   int adamw_mode, int should_log)
{
    HostAdam o{};
    o.alpha = lr;
    o.betta1 = beta1;
    o.betta2 = beta2;
    o.eps = eps;
    o.weight_decay = weight_decay;
    o.betta1_t = 1.0f;
    o.betta2_t = 1.0f;
    o.step = 0;
    o.bc1 = 1.0f;
    o.bc2 = 1.0f;
    o.adamw = adamw_mode != 0;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        g_opts[id] = o;
    }
    if (should_log) {
        printf("Adam Optimizer #%d is created with sm_100a fused-kernel arithmetic capability.\n", id);
        printf("Config: alpha=%f, betas=(%f, %f), weight_decay=%f, adam_w=%d\n", lr, beta1, beta2,
               weight_decay, (int)(adamw_mode != 0));
    }
    return SF_OK;
}

int sf_adam_destroy(int id)
{
    std::lock_guard<std::mutex> lk(g_mu);
    g_opts.erase(id);
    return SF_OK;
}

int sf_adam_scalars(int id, uint64_t step, float lr, float beta1, float beta2, float eps,
                    float weight_decay, int bias_correction, SfAdamScalars* out)
{
    if (!out) return fail(SF_ERR_NULL, "out is NULL");
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_opts.find(id);
    if (it == g_opts.end()) return fail(SF_ERR_UNKNOWN_ID, "optimizer id " + std::to_string(id) + " was not created");
    increment_step(it->second, step, beta1, beta2);
    update_state(it->second, lr, eps, weight_decay, bias_correction, out);
    return SF_OK;
}

int sf_adam_step(const SfAdamScalars* s, float* p, const void* g, int g_dtype, float* m, float* v,
                 uint16_t* p_bf16, uint64_t n, uint64_t vec_n, void* stream)
{
    return step_impl(s, p, g, g_dtype, m, v, p_bf16, n, vec_n, (cudaStream_t)stream);
}

int sf_adam_update(int id, uint64_t step, float lr, float beta1, float beta2, float eps,
                   float weight_decay, int bias_correction, float* p, const void* g, int g_dtype,
                   float* m, float* v, uint16_t* p_bf16, uint64_t n, void* stream)
{
    // Validate what can be validated before the state machine moves, so a rejected call
    // leaves the optimizer where it was.
    if (g_dtype != SF_GRAD_BF16 && g_dtype != SF_GRAD_F32)
        return fail(SF_ERR_DTYPE, "gradient dtype code " + std::to_string(g_dtype) + " is not supported (0 = bf16, 1 = fp32)");
    if (n > 0 && (!p || !g || !m || !v)) return fail(SF_ERR_NULL, "p, g, m and v must be non-NULL when n > 0");
    SfAdamScalars s;
    if (int rc = sf_adam_scalars(id, step, lr, beta1, beta2, eps, weight_decay, bias_correction, &s)) return rc;
    return step_impl(&s, p, g, g_dtype, m, v, p_bf16, n, n & ~(uint64_t)15, (cudaStream_t)stream);
}

int sf_adam_step_sharded(const SfAdamScalars* s, float* p, const void* const* peer_g, int world,
                         int g_dtype, float* m, float* v, uint16_t* p_bf16, uint64_t n,
                         uint64_t vec_n, void* stream)
{
    if (!s) return fail(SF_ERR_NULL, "scalars pointer is NULL");
    if (g_dtype != SF_GRAD_BF16 && g_dtype != SF_GRAD_F32)
        return fail(SF_ERR_DTYPE, "gradient dtype code " + std::to_string(g_dtype) + " is not supported (0 = bf16, 1 = fp32)");
    if (world < 1 || world > SF_MAX_WORLD)
        return fail(SF_ERR_ARG, "world must be in [1, " + std::to_string(SF_MAX_WORLD) + "]");
    if (n == 0) return SF_OK;
    if (!p || !peer_g || !m || !v) return fail(SF_ERR_NULL, "p, peer_g, m and v must be non-NULL when n > 0");
    if (n > ((uint64_t)1 << 40)) return fail(SF_ERR_SIZE, "n exceeds 2^40 elements");
    if (vec_n > n) vec_n = n;
    bool a16 = aligned(p, 16) && aligned(m, 16) && aligned(v, 16) && aligned(p_bf16, 16);
    for (int r = 0; r < world; r++) {
        if (!peer_g[r]) return fail(SF_ERR_NULL, "peer_g[" + std::to_string(r) + "] is NULL");
        a16 = a16 && aligned(peer_g[r], 16);
        if (!aligned(peer_g[r], g_dtype == SF_GRAD_BF16 ? 2 : 4))
            return fail(SF_ERR_ALIGN, "a peer gradient is not aligned to its element size");
    }
    int mode;
    K c = make_k(s, &mode);
    cudaStream_t st = (cudaStream_t)stream;
    if (g_dtype == SF_GRAD_BF16) {
        GradPeers<uint16_t> gs;
        for (int r = 0; r < SF_MAX_WORLD; r++) gs.g[r] = (const uint16_t*)peer_g[r < world ? r : 0];
        gs.world = world;
        gs.fworld = (float)world;
        if (!a16 || n < 4) return launch_scalar(c, mode, p, gs, m, v, p_bf16, n, vec_n, st);
        return launch_vec4(c, mode, p, gs, m, v, p_bf16, n, vec_n, st, 1);
    }
    GradPeers<float> gs;
    for (int r = 0; r < SF_MAX_WORLD; r++) gs.g[r] = (const float*)peer_g[r < world ? r : 0];
    gs.world = world;
    gs.fworld = (float)world;
    if (!a16 || n < 4) return launch_scalar(c, mode, p, gs, m, v, p_bf16, n, vec_n, st);
    return launch_vec4(c, mode, p, gs, m, v, p_bf16, n, vec_n, st, 1);
}

int sf_adam_step_sharded_push(const SfAdamScalars* s, float* p, const void* const* peer_g,
                               uint16_t* const* peer_out, int world, int g_dtype, float* m, float* v,
                               uint64_t n, uint64_t vec_n, void* stream)
{
    if (!s) return fail(SF_ERR_NULL, "scalars pointer is NULL");
    if (g_dtype != SF_GRAD_BF16 && g_dtype != SF_GRAD_F32)
        return fail(SF_ERR_DTYPE, "gradient dtype code " + std::to_string(g_dtype) + " is not supported (0 = bf16, 1 = fp32)");
    if (world < 1 || world > SF_MAX_WORLD)
        return fail(SF_ERR_ARG, "world must be in [1, " + std::to_string(SF_MAX_WORLD) + "]");
    if (n == 0) return SF_OK;
    if (!p || !peer_g || !peer_out || !m || !v)
        return fail(SF_ERR_NULL, "p, peer_g, peer_out, m and v must be non-NULL when n > 0");
    if (n > ((uint64_t)1 << 40)) return fail(SF_ERR_SIZE, "n exceeds 2^40 elements");
    if (vec_n > n) vec_n = n;
    bool a16 = aligned(p, 16) && aligned(m, 16) && aligned(v, 16);
    PushDst dst;
    dst.world = world;
    for (int r = 0; r < SF_MAX_WORLD; r++) dst.out[r] = nullptr;
    for (int r = 0; r < world; r++) {
        if (!peer_g[r] || !peer_out[r]) return fail(SF_ERR_NULL, "peer_g / peer_out entry " + std::to_string(r) + " is NULL");
        if (!aligned(peer_g[r], g_dtype == SF_GRAD_BF16 ? 2 : 4) || !aligned(peer_out[r], 2))
            return fail(SF_ERR_ALIGN, "a peer buffer is not aligned to its element size");
        a16 = a16 && aligned(peer_g[r], 16) && aligned(peer_out[r], 16);
        dst.out[r] = peer_out[r];
    }
    int mode;
    K c = make_k(s, &mode);
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const uint64_t nvec = a16 ? ((vec_n < n ? vec_n : n) & ~(uint64_t)3) : 0;
    // Launch shape measured on two NVLink-connected B200s: one 4-element group per thread and
    // full occupancy (256 threads x 8 CTAs per SM, 32 registers) hides the peer-read latency best
    // (0.65 ms for a 109 M-element slice against 1.44 ms for the single-GPU shape U=2 at half
    // occupancy).  At 0.65 ms each GPU receives 436 MB (its pulls plus the peer's pushes) and sends
    // as much: about 675 GB/s per direction, close to the 770 GB/s a peer copy reaches, so the
    // kernel is NVLink-bound; 8-element-per-thread variants with 128-bit peer accesses measured
    // the same.
    constexpr int U = 1, T = 256, MINB = 8;
    const uint64_t ntiles = (nvec + (uint64_t)T * 4 * U - 1) / ((uint64_t)T * 4 * U);
    const int grid = grid_for(ntiles, di.sms, 0);
    auto launch = [&](auto gs) -> int {
        using GS = decltype(gs);
        if (mode == MODE_NODECAY)
            adam_vec4_push_kernel<GS, MODE_NODECAY, U, T, MINB><<<grid, T, 0, st>>>(c, p, gs, m, v, dst, nvec, n, vec_n);
        else if (mode == MODE_ADAMW)
            adam_vec4_push_kernel<GS, MODE_ADAMW, U, T, MINB><<<grid, T, 0, st>>>(c, p, gs, m, v, dst, nvec, n, vec_n);
        else
            adam_vec4_push_kernel<GS, MODE_L2, U, T, MINB><<<grid, T, 0, st>>>(c, p, gs, m, v, dst, nvec, n, vec_n);
        return check_launch("adam_vec4_push_kernel");
    };
    if (g_dtype == SF_GRAD_BF16) {
        GradPeers<uint16_t> gs;
        for (int r = 0; r < SF_MAX_WORLD; r++) gs.g[r] = (const uint16_t*)peer_g[r < world ? r : 0];
        gs.world = world;
        gs.fworld = (float)world;
        return launch(gs);
    }
    GradPeers<float> gs;
    for (int r = 0; r < SF_MAX_WORLD; r++) gs.g[r] = (const float*)peer_g[r < world ? r : 0];
    gs.world = world;
    gs.fworld = (float)world;
    return launch(gs);
}

int sf_dp_mean(const void* const* peer_g, int world, int g_dtype, float* mean, uint64_t n, void* stream)
{
    if (g_dtype != SF_GRAD_BF16 && g_dtype != SF_GRAD_F32)
        return fail(SF_ERR_DTYPE, "gradient dtype code " + std::to_string(g_dtype) + " is not supported (0 = bf16, 1 = fp32)");
    if (world < 1 || world > SF_MAX_WORLD)
        return fail(SF_ERR_ARG, "world must be in [1, " + std::to_string(SF_MAX_WORLD) + "]");
    if (n == 0) return SF_OK;
    if (!peer_g || !mean) return fail(SF_ERR_NULL, "peer_g and mean must be non-NULL when n > 0");
    bool a16 = aligned(mean, 16);
    for (int r = 0; r < world; r++) {
        if (!peer_g[r]) return fail(SF_ERR_NULL, "peer_g[" + std::to_string(r) + "] is NULL");
        a16 = a16 && aligned(peer_g[r], 16);
    }
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    const uint64_t nvec = a16 ? (n & ~(uint64_t)3) : 0;
    int grid = grid_for((n + 1023) / 1024, di.sms, 8);
    cudaStream_t st = (cudaStream_t)stream;
    if (g_dtype == SF_GRAD_BF16) {
        GradPeers<uint16_t> gs;
        for (int r = 0; r < SF_MAX_WORLD; r++) gs.g[r] = (const uint16_t*)peer_g[r < world ? r : 0];
        gs.world = world;
        gs.fworld = (float)world;
        dp_mean_kernel<<<grid, 256, 0, st>>>(gs, mean, nvec, n);
    } else {
        GradPeers<float> gs;
        for (int r = 0; r < SF_MAX_WORLD; r++) gs.g[r] = (const float*)peer_g[r < world ? r : 0];
        gs.world = world;
        gs.fworld = (float)world;
        dp_mean_kernel<<<grid, 256, 0, st>>>(gs, mean, nvec, n);
    }
    return check_launch("dp_mean_kernel");
}

int sf_adam_update_dp_static(int id, uint64_t step, float lr, float beta1, float beta2, float eps,
                             float weight_decay, int bias_correction, float* p,
                             const void* const* peer_g, int world, int g_dtype, float* m, float* v,
                             uint16_t* p_bf16, uint64_t n, void* stream)
{
    if (n > kStaticMeanMaxElems)
        return fail(SF_ERR_SIZE, "n = " + std::to_string(n) + " exceeds the built-in scratch of " +
                                     std::to_string(kStaticMeanMaxElems) +
                                     " elements; split the call or use sf_dp_mean + sf_adam_update with your own buffer");
    if (n > 0 && (!p || !m || !v)) return fail(SF_ERR_NULL, "p, m and v must be non-NULL when n > 0");
    float* mean = nullptr;
    if (int rc = static_mean_address(&mean)) return rc;
    // mean[0, n) is fully rewritten by the first kernel before the second reads it, so nothing
    // left over from an earlier call is ever consumed and nothing needs clearing.
    if (int rc = sf_dp_mean(peer_g, world, g_dtype, mean, n, stream)) return rc;
    return sf_adam_update(id, step, lr, beta1, beta2, eps, weight_decay, bias_correction, p, mean,
                          SF_GRAD_F32, m, v, p_bf16, n, stream);
}

size_t sf_adam_host_scratch_bytes(uint64_t chunk_elems, int g_dtype, int g_on_host)
{
    size_t per_slot = 3 * round256((size_t)chunk_elems * 4);
    if (g_on_host) per_slot += round256((size_t)chunk_elems * (g_dtype == SF_GRAD_BF16 ? 2 : 4));
    return 2 * per_slot;
}

int sf_adam_update_host(int id, uint64_t step, float lr, float beta1, float beta2, float eps,
                        float weight_decay, int bias_correction, float* p_host, const void* g,
                        int g_dtype, int g_on_host, float* m_host, float* v_host,
                        uint16_t* p_bf16_dev, uint64_t n, uint64_t chunk_elems, int per_chunk_scalars,
                        void* scratch, size_t scratch_bytes, void* stream)
{
    if (g_dtype != SF_GRAD_BF16 && g_dtype != SF_GRAD_F32)
        return fail(SF_ERR_DTYPE, "gradient dtype code " + std::to_string(g_dtype) + " is not supported (0 = bf16, 1 = fp32)");
    if (chunk_elems == 0 || (chunk_elems & 15)) return fail(SF_ERR_ARG, "chunk_elems must be a positive multiple of 16");
    if (n > 0 && (!p_host || !g || !m_host || !v_host || !scratch))
        return fail(SF_ERR_NULL, "p_host, g, m_host, v_host and scratch must be non-NULL when n > 0");
    if (!aligned(scratch, 256)) return fail(SF_ERR_ALIGN, "scratch must be 256-byte aligned");
    if (n > 0 && scratch_bytes < sf_adam_host_scratch_bytes(chunk_elems, g_dtype, g_on_host))
        return fail(SF_ERR_SIZE, "scratch is smaller than sf_adam_host_scratch_bytes()");
    if (!aligned(p_host, 16) || !aligned(m_host, 16) || !aligned(v_host, 16) || !aligned(g, 16) ||
        !aligned(p_bf16_dev, 16))
        return fail(SF_ERR_ALIGN, "host-streaming buffers must be 16-byte aligned");
    SfAdamScalars s;
    if (int rc = sf_adam_scalars(id, step, lr, beta1, beta2, eps, weight_decay, bias_correction, &s)) return rc;
    if (n == 0) return SF_OK;

    HostPipe* hp;
    if (int rc = get_pipe(&hp)) return rc;
    cudaStream_t user = (cudaStream_t)stream;
    const size_t gsz = g_dtype == SF_GRAD_BF16 ? 2 : 4;
    const size_t arr = round256((size_t)chunk_elems * 4);
    const size_t garr = g_on_host ? round256((size_t)chunk_elems * gsz) : 0;
    const size_t slot_bytes = 3 * arr + garr;
    char* base = (char*)scratch;

    SF_CUDA(cudaEventRecord(hp->ev_start, user));
    SF_CUDA(cudaStreamWaitEvent(hp->s_in, hp->ev_start, 0));
    SF_CUDA(cudaStreamWaitEvent(hp->s_k, hp->ev_start, 0));
    SF_CUDA(cudaStreamWaitEvent(hp->s_out, hp->ev_start, 0));

    const uint64_t nchunks = (n + chunk_elems - 1) / chunk_elems;
    for (uint64_t k = 0; k < nchunks; k++) {
        const int slot = (int)(k & 1);
        const uint64_t lo = k * chunk_elems;
        const uint64_t len = (lo + chunk_elems <= n) ? chunk_elems : n - lo;
        float* dp = (float*)(base + slot * slot_bytes);
        float* dm = (float*)(base + slot * slot_bytes + arr);
        float* dv = (float*)(base + slot * slot_bytes + 2 * arr);
        void* dg = g_on_host ? (void*)(base + slot * slot_bytes + 3 * arr) : (void*)((const char*)g + lo * gsz);
        // the slot is free once the device->host copies of its previous user are done (chunk
        // k-2 of this call, or a chunk of an earlier call; waiting on a never-recorded event
        // is a no-op)
        SF_CUDA(cudaStreamWaitEvent(hp->s_in, hp->ev_out[slot], 0));
        SF_CUDA(cudaMemcpyAsync(dp, p_host + lo, len * 4, cudaMemcpyHostToDevice, hp->s_in));
        SF_CUDA(cudaMemcpyAsync(dm, m_host + lo, len * 4, cudaMemcpyHostToDevice, hp->s_in));
        SF_CUDA(cudaMemcpyAsync(dv, v_host + lo, len * 4, cudaMemcpyHostToDevice, hp->s_in));
        if (g_on_host)
            SF_CUDA(cudaMemcpyAsync(dg, (const char*)g + lo * gsz, len * gsz, cudaMemcpyHostToDevice, hp->s_in));
        SF_CUDA(cudaEventRecord(hp->ev_in[slot], hp->s_in));

        SF_CUDA(cudaStreamWaitEvent(hp->s_k, hp->ev_in[slot], 0));
        if (k > 0 && per_chunk_scalars)
            if (int rc = sf_adam_scalars(id, step, lr, beta1, beta2, eps, weight_decay, bias_correction, &s)) return rc;
        if (int rc = step_impl(&s, dp, dg, g_dtype, dm, dv, p_bf16_dev ? p_bf16_dev + lo : nullptr, len,
                               len & ~(uint64_t)15, hp->s_k))
            return rc;
        SF_CUDA(cudaEventRecord(hp->ev_k[slot], hp->s_k));

        SF_CUDA(cudaStreamWaitEvent(hp->s_out, hp->ev_k[slot], 0));
        SF_CUDA(cudaMemcpyAsync(p_host + lo, dp, len * 4, cudaMemcpyDeviceToHost, hp->s_out));
        SF_CUDA(cudaMemcpyAsync(m_host + lo, dm, len * 4, cudaMemcpyDeviceToHost, hp->s_out));
        SF_CUDA(cudaMemcpyAsync(v_host + lo, dv, len * 4, cudaMemcpyDeviceToHost, hp->s_out));
        SF_CUDA(cudaEventRecord(hp->ev_out[slot], hp->s_out));
    }
    // s_out is ordered after the last kernel; make the caller's stream wait for everything.
    SF_CUDA(cudaEventRecord(hp->ev_done, hp->s_out));
    SF_CUDA(cudaStreamWaitEvent(user, hp->ev_done, 0));
    return SF_OK;
}

const char* sf_last_error(void) { return t_err.c_str(); }
int sf_abi_version(void) { return SF_ABI_VERSION; }
uint64_t sf_launch_count(void) { return g_launches.load(); }

int sf_set_tuning(int variant, int ctas_per_sm)
{
    if (variant > 2) return fail(SF_ERR_ARG, "variant must be 0 (128-bit, default caching), 1 (128-bit, streaming) or 2 (256-bit)");
    if (variant >= 0) g_tune.variant = variant;
    if (ctas_per_sm >= 0) g_tune.ctas_per_sm = ctas_per_sm;
    return SF_OK;
}

int sf_dev_alloc(size_t bytes, void** dev_ptr_out)
{
    if (!dev_ptr_out) return fail(SF_ERR_NULL, "dev_ptr_out is NULL");
    *dev_ptr_out = nullptr;
    if (bytes == 0) return SF_OK;
    SF_CUDA(cudaMalloc(dev_ptr_out, bytes));
    return SF_OK;
}

int sf_dev_free(void* dev_ptr)
{
    if (!dev_ptr) return SF_OK;
    SF_CUDA(cudaFree(dev_ptr));
    return SF_OK;
}

int sf_ipc_export(void* dev_ptr, void* handle_out)
{
    static_assert(sizeof(cudaIpcMemHandle_t) == SF_IPC_HANDLE_BYTES, "IPC handle size");
    if (!dev_ptr || !handle_out) return fail(SF_ERR_NULL, "dev_ptr and handle_out must be non-NULL");
    cudaIpcMemHandle_t h;
    SF_CUDA(cudaIpcGetMemHandle(&h, dev_ptr));
    std::memcpy(handle_out, &h, sizeof(h));
    return SF_OK;
}

int sf_ipc_open(const void* handle, void** dev_ptr_out)
{
    if (!handle || !dev_ptr_out) return fail(SF_ERR_NULL, "handle and dev_ptr_out must be non-NULL");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    SF_CUDA(cudaIpcOpenMemHandle(dev_ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
    return SF_OK;
}

int sf_ipc_close(void* dev_ptr)
{
    if (!dev_ptr) return SF_OK;
    SF_CUDA(cudaIpcCloseMemHandle(dev_ptr));
    return SF_OK;
}

}  // extern "C"
