// Device code of the fused LayerAdam step for B200 (sm_100a), shared by the translation units
// that launch it.
//
// One pass over a layer's flat vectors: read fp32 p, m, v and the bf16 (or fp32) gradient,
// apply the Adam / AdamW update in registers with single-rounded IEEE binary32 operations in
// the order of the reference's AVX-512 loop (optimizer/layer_adam/csrc/cpu_adam.h:158-193),
// write p, m, v back and emit the round-to-nearest-even bf16 copy of the new p.  28 bytes
// move per parameter (14 read, 14 written) and nothing is reused, so the kernels are bound by
// HBM bandwidth (by NVLink when the gradients or the bf16 outputs live on other GPUs); there is
// no GEMM-shaped work here and the tensor cores are not involved.
//
// Bit parity rules followed everywhere below:
//   * only __fmul_rn / __fmaf_rn / __fadd_rn / __fsqrt_rn / __fdiv_rn, never a plain * or +
//     on floats, so the compiler can neither fuse nor reorder; no fast-math flags;
//   * elements at or above vec_n use the contraction the reference's compiled scalar tail
//     uses (cpu_adam_impl.cpp:46-66): m = fma(m, b1, g*(1-b1)), v = fma(v, b2, (g*g)*(1-b2));
//   * bf16 output: RNE on the upper 16 bits, every NaN becomes 0x7FC0 (simd.h:56-86).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "slideformer_b200.h"

#define SF_MAX_WORLD 16

namespace sfk {

enum { MODE_NODECAY = 0, MODE_ADAMW = 1, MODE_L2 = 2 };

struct K {  // kernel-side constants
    float b1, b2, omb1, omb2, bc2, eps, step_size, w_decay, wd, gscale;
};

// ------------------------------------------------------------------------------------------
// arithmetic
// ------------------------------------------------------------------------------------------
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

// ------------------------------------------------------------------------------------------
// gradient-side additions: statistics of the incoming gradient and a multiplier on it.
// Everything here compiles away when EX is false, which is the reference's element loop.
// ------------------------------------------------------------------------------------------
struct StatAcc {
    float ss;
    uint32_t bad;
};

template <bool EX>
__device__ __forceinline__ float grad_pre(const K& c, float g, StatAcc& a)
{
    if (EX) {
        a.ss = __fmaf_rn(g, g, a.ss);
        a.bad |= ((__float_as_uint(g) & 0x7f800000u) == 0x7f800000u) ? 1u : 0u;
        g = __fmul_rn(g, c.gscale);
    }
    return g;
}

// Block reduction, then one atomic per CTA on one of SF_STATS_LANES partial sums.
template <int THREADS>
__device__ __forceinline__ void stat_flush(const StatAcc& a, SfGradStats* stats)
{
    if (stats == nullptr) return;  // uniform across the grid
    __shared__ float s_ss[THREADS / 32];
    __shared__ uint32_t s_bad[THREADS / 32];
    float ss = a.ss;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const uint32_t bad = __reduce_or_sync(0xffffffffu, a.bad);
    const int w = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) {
        s_ss[w] = ss;
        s_bad[w] = bad;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        uint32_t b = 0;
#pragma unroll
        for (int k = 0; k < THREADS / 32; k++) {
            t += s_ss[k];
            b |= s_bad[k];
        }
        atomicAdd(&stats->sumsq[blockIdx.x % SF_STATS_LANES], t);
        if (b) atomicOr(&stats->nonfinite, 1u);
    }
}

// ------------------------------------------------------------------------------------------
// global memory access flavours
// ------------------------------------------------------------------------------------------
// HINT 0: default caching.  HINT 1: streaming (evict-first) on every access; nothing in these
// kernels is read twice.
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

__device__ __forceinline__ void unpack4(uint2 r, float (&o)[4])
{
    o[0] = bf16_bits_to_f32(r.x & 0xffffu);
    o[1] = bf16_bits_to_f32(r.x >> 16);
    o[2] = bf16_bits_to_f32(r.y & 0xffffu);
    o[3] = bf16_bits_to_f32(r.y >> 16);
}

// ------------------------------------------------------------------------------------------
// gradient sources.  `load4` returns 4 consecutive gradients as floats.
// ------------------------------------------------------------------------------------------
struct GradBf16 {
    static constexpr bool kPeer = false;
    const uint16_t* g;
    template <int HINT>
    __device__ __forceinline__ void load4(uint64_t i, float (&o)[4]) const
    {
        unpack4(ld2u<HINT>(g + i), o);
    }
    __device__ __forceinline__ float load1(uint64_t i) const { return bf16_bits_to_f32(g[i]); }
};
// fp16 gradients (the <float, Half, float> triple of cpu_adam_impl.cpp:189): widened exactly.
__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }
struct GradF16 {
    static constexpr bool kPeer = false;
    const uint16_t* g;
    template <int HINT>
    __device__ __forceinline__ void load4(uint64_t i, float (&o)[4]) const
    {
        uint2 r = ld2u<HINT>(g + i);
        o[0] = f16_bits_to_f32(r.x & 0xffffu);
        o[1] = f16_bits_to_f32(r.x >> 16);
        o[2] = f16_bits_to_f32(r.y & 0xffffu);
        o[3] = f16_bits_to_f32(r.y >> 16);
    }
    __device__ __forceinline__ float load1(uint64_t i) const { return f16_bits_to_f32(g[i]); }
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

// Rank-ordered fp32 mean over peer-mapped gradients (multi_gpu/shared_data_parallel.py:130-133):
// zero accumulator, add rank 0..world-1, true division by world.
// W > 0: the world size is a compile-time constant, so every peer load of a thread is issued
// before the first add (W independent long-latency NVLink reads in flight per thread).
// W == 0: any world up to SF_MAX_WORLD, loads issued four at a time.
template <typename ELT, int W>
struct GradPeers {
    static constexpr bool kPeer = true;
    static constexpr int CAP = W > 0 ? W : SF_MAX_WORLD;
    const ELT* g[CAP];
    int world;
    float fworld;

    template <int HINT>
    __device__ __forceinline__ void load4(uint64_t i, float (&o)[4]) const
    {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (W > 0) {
            if (sizeof(ELT) == 2) {
                uint2 q[CAP];
#pragma unroll
                for (int r = 0; r < W; r++) q[r] = ld2u<HINT>(g[r] + i);
#pragma unroll
                for (int r = 0; r < W; r++) {
                    float t[4];
                    unpack4(q[r], t);
#pragma unroll
                    for (int k = 0; k < 4; k++) acc[k] = __fadd_rn(acc[k], t[k]);
                }
            } else {
                float4 q[CAP];
#pragma unroll
                for (int r = 0; r < W; r++) q[r] = ld4<HINT>(reinterpret_cast<const float*>(g[r]) + i);
#pragma unroll
                for (int r = 0; r < W; r++) {
                    acc[0] = __fadd_rn(acc[0], q[r].x);
                    acc[1] = __fadd_rn(acc[1], q[r].y);
                    acc[2] = __fadd_rn(acc[2], q[r].z);
                    acc[3] = __fadd_rn(acc[3], q[r].w);
                }
            }
        } else {
#pragma unroll 4
            for (int r = 0; r < world; r++) {
                float t[4];
                if (sizeof(ELT) == 2) {
                    unpack4(ld2u<HINT>(g[r] + i), t);
                } else {
                    float4 q = ld4<HINT>(reinterpret_cast<const float*>(g[r]) + i);
                    t[0] = q.x; t[1] = q.y; t[2] = q.z; t[3] = q.w;
                }
#pragma unroll
                for (int k = 0; k < 4; k++) acc[k] = __fadd_rn(acc[k], t[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; k++) o[k] = __fdiv_rn(acc[k], fworld);
    }

    // 8 consecutive bf16 gradients per peer as one 16-byte load (bf16 only).
    __device__ __forceinline__ void load8(uint64_t i, float (&o)[8]) const
    {
        static_assert(W > 0, "load8 needs a compile-time world");
        uint4 q[CAP];
#pragma unroll
        for (int r = 0; r < W; r++) q[r] = __ldcs(reinterpret_cast<const uint4*>(g[r] + i));
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < W; r++) {
            float t[8];
            t[0] = bf16_bits_to_f32(q[r].x & 0xffffu); t[1] = bf16_bits_to_f32(q[r].x >> 16);
            t[2] = bf16_bits_to_f32(q[r].y & 0xffffu); t[3] = bf16_bits_to_f32(q[r].y >> 16);
            t[4] = bf16_bits_to_f32(q[r].z & 0xffffu); t[5] = bf16_bits_to_f32(q[r].z >> 16);
            t[6] = bf16_bits_to_f32(q[r].w & 0xffffu); t[7] = bf16_bits_to_f32(q[r].w >> 16);
#pragma unroll
            for (int k = 0; k < 8; k++) acc[k] = __fadd_rn(acc[k], t[k]);
        }
#pragma unroll
        for (int k = 0; k < 8; k++) o[k] = __fdiv_rn(acc[k], fworld);
    }

    __device__ __forceinline__ float load1(uint64_t i) const
    {
        float acc = 0.f;
        const int n = W > 0 ? W : world;
        for (int r = 0; r < n; r++) {
            float t;
            if (sizeof(ELT) == 2) t = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(g[r])[i]);
            else t = reinterpret_cast<const float*>(g[r])[i];
            acc = __fadd_rn(acc, t);
        }
        return __fdiv_rn(acc, fworld);
    }
};

// Resident CTAs per SM (of 256 threads) the peer kernels are compiled for.  Holding W peer loads
// in flight per thread needs registers: 32 per thread (8 CTAs) is enough up to two peers, four
// peers get 40 (6 CTAs), eight get 48 (5 CTAs).
template <int W>
constexpr int peer_min_ctas()
{
    return W == 8 ? 5 : (W == 4 ? 6 : 8);
}

// ------------------------------------------------------------------------------------------
// bf16 output sinks
// ------------------------------------------------------------------------------------------
struct OutNone {
    __device__ __forceinline__ void store1(uint64_t, uint16_t) const {}
};
struct OutLocal {
    uint16_t* o;
    __device__ __forceinline__ void store1(uint64_t i, uint16_t x) const { o[i] = x; }
};
// Every rank's copy of the layer (local and peer-mapped): the parameter all-gather done as
// stores from the kernel that computed the values.
template <int W>
struct OutPush {
    static constexpr int CAP = W > 0 ? W : SF_MAX_WORLD;
    uint16_t* o[CAP];
    int world;
    __device__ __forceinline__ int count() const { return W > 0 ? W : world; }
    __device__ __forceinline__ void store1(uint64_t i, uint16_t x) const
    {
        for (int r = 0; r < count(); r++) o[r][i] = x;
    }
    __device__ __forceinline__ void store4(uint64_t i, uint2 x) const
    {
        if (W > 0) {
#pragma unroll
            for (int r = 0; r < W; r++) *reinterpret_cast<uint2*>(o[r] + i) = x;
        } else {
            for (int r = 0; r < world; r++) *reinterpret_cast<uint2*>(o[r] + i) = x;
        }
    }
    __device__ __forceinline__ void store8(uint64_t i, uint4 x) const
    {
#pragma unroll
        for (int r = 0; r < CAP; r++)
            if (r < count()) *reinterpret_cast<uint4*>(o[r] + i) = x;
    }
};

// ------------------------------------------------------------------------------------------
// kernels
// ------------------------------------------------------------------------------------------

// One element per thread-iteration over [lo, hi): the remainder of a vector kernel, and the
// whole-array path for buffers that are not 16-byte aligned.  Body arithmetic below vec_n,
// tail arithmetic from there on.
template <typename GS, int MODE, typename SINK, bool EX>
__device__ __forceinline__ void scalar_range(const K& c, float* p, const GS& gs, float* m, float* v,
                                             const SINK& sink, uint64_t lo, uint64_t hi, uint64_t vec_n,
                                             uint64_t tid, uint64_t nthreads, StatAcc& acc)
{
    for (uint64_t i = lo + tid; i < hi; i += nthreads) {
        float pp = p[i], mm = m[i], vv = v[i];
        float g = grad_pre<EX>(c, gs.load1(i), acc);
        if (i < vec_n) adam_body<MODE>(c, pp, g, mm, vv);
        else adam_tail<MODE>(c, pp, g, mm, vv);
        p[i] = pp; m[i] = mm; v[i] = vv;
        sink.store1(i, (uint16_t)f32_to_bf16_bits(pp));
    }
}

template <typename GS, int MODE, typename SINK, bool EX>
__global__ void __launch_bounds__(256)
adam_scalar_kernel(K c, float* p, GS gs, float* m, float* v, SINK sink, uint64_t n, uint64_t vec_n,
                   SfGradStats* stats)
{
    StatAcc acc{0.f, 0u};
    scalar_range<GS, MODE, SINK, EX>(c, p, gs, m, v, sink, 0, n, vec_n,
                                     (uint64_t)blockIdx.x * blockDim.x + threadIdx.x,
                                     (uint64_t)gridDim.x * blockDim.x, acc);
    if (EX) stat_flush<256>(acc, stats);
}

// 128-bit kernel.  A CTA walks tiles of THREADS*4*U elements; inside a tile, sub-iteration u
// of thread t covers the 4 elements at tile + (u*THREADS + t)*4, so every load and store
// instruction of a warp touches one contiguous, fully used 512-byte (fp32) or 256-byte (bf16)
// span.  All U loads of p, m, v, g are issued before the arithmetic to keep
// U * 56 bytes per thread in flight.
//   nvec    = elements handled here, a multiple of 4, all below vec_n (body arithmetic)
//   [nvec, n) is finished by the last CTA with scalar accesses (at most 18 elements: the
//   launcher sends anything longer to the scalar kernel).
template <typename GS, int MODE, bool OUT, int HINT, int U, int THREADS, int MINB, bool EX>
__global__ void __launch_bounds__(THREADS, MINB)
adam_vec4_kernel(K c, float* __restrict__ p, GS gs, float* __restrict__ m, float* __restrict__ v,
                 uint16_t* __restrict__ out, uint64_t nvec, uint64_t n, uint64_t vec_n, SfGradStats* stats)
{
    constexpr uint64_t TILE = (uint64_t)THREADS * 4 * U;
    const uint64_t ntiles = (nvec + TILE - 1) / TILE;
    StatAcc acc{0.f, 0u};
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
                if (GS::kPeer) gs.template load4<HINT>(i, G[u]);   // the long-latency peer reads go first
                P[u] = ld4<HINT>(p + i);
                M[u] = ld4<HINT>(m + i);
                V[u] = ld4<HINT>(v + i);
                if (!GS::kPeer) gs.template load4<HINT>(i, G[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint64_t i = base + (uint64_t)u * THREADS * 4;
            if (ok[u]) {
                if (EX) {
#pragma unroll
                    for (int k = 0; k < 4; k++) G[u][k] = grad_pre<EX>(c, G[u][k], acc);
                }
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
    if (blockIdx.x == gridDim.x - 1) {
        if (OUT) scalar_range<GS, MODE, OutLocal, EX>(c, p, gs, m, v, OutLocal{out}, nvec, n, vec_n, threadIdx.x, THREADS, acc);
        else scalar_range<GS, MODE, OutNone, EX>(c, p, gs, m, v, OutNone{}, nvec, n, vec_n, threadIdx.x, THREADS, acc);
    }
    if (EX) stat_flush<THREADS>(acc, stats);
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
        StatAcc acc{0.f, 0u};
        if (G_BF16) {
            GradBf16 gs{reinterpret_cast<const uint16_t*>(gptr)};
            if (OUT) scalar_range<GradBf16, MODE, OutLocal, false>(c, p, gs, m, v, OutLocal{out}, nvec, n, vec_n, threadIdx.x, THREADS, acc);
            else scalar_range<GradBf16, MODE, OutNone, false>(c, p, gs, m, v, OutNone{}, nvec, n, vec_n, threadIdx.x, THREADS, acc);
        } else {
            GradF32 gs{reinterpret_cast<const float*>(gptr)};
            if (OUT) scalar_range<GradF32, MODE, OutLocal, false>(c, p, gs, m, v, OutLocal{out}, nvec, n, vec_n, threadIdx.x, THREADS, acc);
            else scalar_range<GradF32, MODE, OutNone, false>(c, p, gs, m, v, OutNone{}, nvec, n, vec_n, threadIdx.x, THREADS, acc);
        }
    }
}

// Fused data-parallel step: the gradient mean is PULLED from every rank, Adam runs on the owned
// slice, and the bf16 result is PUSHED into every rank's copy of the layer, all in one kernel.
// With NVLink full duplex the pushes (egress) overlap the pulls (ingress), and no separate
// reduce-scatter or all-gather pass exists.  One tile of 256 * VEC elements per CTA:
//   VEC 4: 8-byte peer loads and pushes, 16-byte p/m/v accesses, 8 CTAs per SM;
//   VEC 8: 16-byte peer loads and pushes, 32-byte p/m/v accesses (bf16 gradients only).
// Elements [nvec, n) are spread over the whole grid one at a time.
template <typename ELT, int W, int MODE, int VEC, bool EX>
__global__ void __launch_bounds__(256, VEC == 4 ? peer_min_ctas<W>() : 3)
adam_push_kernel(K c, float* __restrict__ p, GradPeers<ELT, W> gs, float* __restrict__ m,
                 float* __restrict__ v, OutPush<W> dst, uint64_t nvec, uint64_t n, uint64_t vec_n,
                 SfGradStats* stats)
{
    StatAcc acc{0.f, 0u};
    const uint64_t i = ((uint64_t)blockIdx.x * 256 + threadIdx.x) * VEC;
    if (i < nvec) {
        if (VEC == 4) {
            float G[4];
            gs.template load4<1>(i, G);
            float4 P = ld4<1>(p + i), M = ld4<1>(m + i), V = ld4<1>(v + i);
            if (EX) {
#pragma unroll
                for (int k = 0; k < 4; k++) G[k] = grad_pre<EX>(c, G[k], acc);
            }
            adam_body<MODE>(c, P.x, G[0], M.x, V.x);
            adam_body<MODE>(c, P.y, G[1], M.y, V.y);
            adam_body<MODE>(c, P.z, G[2], M.z, V.z);
            adam_body<MODE>(c, P.w, G[3], M.w, V.w);
            st4<1>(p + i, P);
            st4<1>(m + i, M);
            st4<1>(v + i, V);
            uint2 o;
            o.x = pack_bf16x2(P.x, P.y);
            o.y = pack_bf16x2(P.z, P.w);
            dst.store4(i, o);
        } else {
            float G[8];
            if constexpr (VEC == 8 && W > 0 && sizeof(ELT) == 2) gs.load8(i, G);
            f8 P = ld8(p + i), M = ld8(m + i), V = ld8(v + i);
#pragma unroll
            for (int k = 0; k < 8; k++) {
                float g = EX ? grad_pre<EX>(c, G[k], acc) : G[k];
                adam_body<MODE>(c, P.x[k], g, M.x[k], V.x[k]);
            }
            st8(p + i, P);
            st8(m + i, M);
            st8(v + i, V);
            uint4 o;
            o.x = pack_bf16x2(P.x[0], P.x[1]);
            o.y = pack_bf16x2(P.x[2], P.x[3]);
            o.z = pack_bf16x2(P.x[4], P.x[5]);
            o.w = pack_bf16x2(P.x[6], P.x[7]);
            dst.store8(i, o);
        }
    }
    scalar_range<GradPeers<ELT, W>, MODE, OutPush<W>, EX>(c, p, gs, m, v, dst, nvec, n, vec_n,
                                                          (uint64_t)blockIdx.x * 256 + threadIdx.x,
                                                          (uint64_t)gridDim.x * 256, acc);
    if (EX) stat_flush<256>(acc, stats);
}

// Many small slices in ONE launch of the pull + push step: a model made of small units (GPT-2
// small: 14 units of 2 to 39 M parameters) otherwise pays one launch and two cross-rank stream
// barriers per unit.  Every segment carries the constants of its own reference call (the host
// state machine still advances once per call), its own arrays and its own peer pointers; a
// CTA finds its segment from the table in the kernel parameters.  4 elements per thread.
#define SF_MULTI_MAX_SEGMENTS 32
#define SF_MULTI_MAX_WORLD 8
struct SegDev {
    K c;
    float* p;
    float* m;
    float* v;
    const void* g[SF_MULTI_MAX_WORLD];
    uint16_t* o[SF_MULTI_MAX_WORLD];
    uint64_t nvec, n, vec_n;
    uint32_t first_cta, num_ctas;
};
struct SegTable {
    int nseg, world;
    float fworld;
    SegDev seg[SF_MULTI_MAX_SEGMENTS];
};

template <typename ELT>
__device__ __forceinline__ void seg_load4(const SegDev& d, int world, float fworld, uint64_t i, float (&o)[4])
{
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int r = 0; r < world; r++) {
        float t[4];
        if (sizeof(ELT) == 2) {
            unpack4(ld2u<1>(reinterpret_cast<const uint16_t*>(d.g[r]) + i), t);
        } else {
            float4 q = ld4<1>(reinterpret_cast<const float*>(d.g[r]) + i);
            t[0] = q.x; t[1] = q.y; t[2] = q.z; t[3] = q.w;
        }
#pragma unroll
        for (int k = 0; k < 4; k++) acc[k] = __fadd_rn(acc[k], t[k]);
    }
#pragma unroll
    for (int k = 0; k < 4; k++) o[k] = __fdiv_rn(acc[k], fworld);
}

template <typename ELT>
__device__ __forceinline__ float seg_load1(const SegDev& d, int world, float fworld, uint64_t i)
{
    float acc = 0.f;
    for (int r = 0; r < world; r++) {
        float t;
        if (sizeof(ELT) == 2) t = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(d.g[r])[i]);
        else t = reinterpret_cast<const float*>(d.g[r])[i];
        acc = __fadd_rn(acc, t);
    }
    return __fdiv_rn(acc, fworld);
}

template <typename ELT, int MODE, bool EX>
__global__ void __launch_bounds__(256, 5)
adam_push_multi_kernel(const __grid_constant__ SegTable t, SfGradStats* stats)
{
    int s = 0;
    while (s + 1 < t.nseg && blockIdx.x >= t.seg[s + 1].first_cta) s++;
    const SegDev& d = t.seg[s];
    const uint64_t cta = blockIdx.x - d.first_cta;
    StatAcc acc{0.f, 0u};
    const uint64_t i = (cta * 256 + threadIdx.x) * 4;
    if (i < d.nvec) {
        float G[4];
        seg_load4<ELT>(d, t.world, t.fworld, i, G);
        float4 P = ld4<1>(d.p + i), M = ld4<1>(d.m + i), V = ld4<1>(d.v + i);
        if (EX) {
#pragma unroll
            for (int k = 0; k < 4; k++) G[k] = grad_pre<EX>(d.c, G[k], acc);
        }
        adam_body<MODE>(d.c, P.x, G[0], M.x, V.x);
        adam_body<MODE>(d.c, P.y, G[1], M.y, V.y);
        adam_body<MODE>(d.c, P.z, G[2], M.z, V.z);
        adam_body<MODE>(d.c, P.w, G[3], M.w, V.w);
        st4<1>(d.p + i, P);
        st4<1>(d.m + i, M);
        st4<1>(d.v + i, V);
        uint2 o;
        o.x = pack_bf16x2(P.x, P.y);
        o.y = pack_bf16x2(P.z, P.w);
        for (int r = 0; r < t.world; r++) *reinterpret_cast<uint2*>(d.o[r] + i) = o;
    }
    for (uint64_t j = d.nvec + cta * 256 + threadIdx.x; j < d.n; j += (uint64_t)d.num_ctas * 256) {
        float pp = d.p[j], mm = d.m[j], vv = d.v[j];
        float g = grad_pre<EX>(d.c, seg_load1<ELT>(d, t.world, t.fworld, j), acc);
        if (j < d.vec_n) adam_body<MODE>(d.c, pp, g, mm, vv);
        else adam_tail<MODE>(d.c, pp, g, mm, vv);
        d.p[j] = pp; d.m[j] = mm; d.v[j] = vv;
        const uint16_t ob = (uint16_t)f32_to_bf16_bits(pp);
        for (int r = 0; r < t.world; r++) d.o[r][j] = ob;
    }
    if (EX) stat_flush<256>(acc, stats);
}

// The same step with the exchange done by the NVSwitch (NVLS): `mc_g` and `mc_out` are MULTICAST
// addresses that alias the same offset of every rank's gradient buffer / bf16 layer buffer.
//   multimem.ld_reduce  one 16-byte request returns the sum of all ranks' 8 bf16 gradients, added
//                       inside the switch in fp32 and rounded once to bf16; only the reduced
//                       16 bytes cross this GPU's ingress links instead of (world - 1) * 16;
//   multimem.st         one 16-byte store is replicated by the switch into every rank's bf16
//                       layer; it crosses this GPU's egress links once instead of world - 1 times.
// The sum's order inside the switch is not specified and it is rounded to bf16 before the
// division by world, so the gradient mean differs from the reference's fp32 rank-order mean by
// up to half a bf16 ulp of the sum: this kernel is NOT bit-exact and is offered beside the exact
// adam_push_kernel, never in its place.  Elements [nvec, n) take the exact peer path.
// The kernel waits on nothing; the caller orders it between two cross-rank stream barriers.
template <int MODE, bool EX, int U>
__global__ void __launch_bounds__(256, U == 1 ? 4 : (U == 2 ? 3 : 2))
adam_nvls_kernel(K c, float* __restrict__ p, const uint16_t* mc_g, float* __restrict__ m,
                 float* __restrict__ v, uint16_t* mc_out, GradPeers<uint16_t, 0> gs, OutPush<0> dst,
                 uint64_t nvec, uint64_t n, uint64_t vec_n, SfGradStats* stats)
{
    StatAcc acc{0.f, 0u};
    // U groups of 8 elements per thread, a tile of 2048 * U elements per CTA; all U in-switch
    // reductions of a thread are requested before the first result is used
    const uint64_t base = (uint64_t)blockIdx.x * (2048 * U) + (uint64_t)threadIdx.x * 8;
    uint4 Q[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
        const uint64_t i = base + (uint64_t)u * 2048;
        ok[u] = i < nvec;
        if (ok[u])
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                         : "=r"(Q[u].x), "=r"(Q[u].y), "=r"(Q[u].z), "=r"(Q[u].w)
                         : "l"(mc_g + i)
                         : "memory");
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
        const uint64_t i = base + (uint64_t)u * 2048;
        if (!ok[u]) continue;
        const uint4 q = Q[u];
        f8 P = ld8(p + i), M = ld8(m + i), V = ld8(v + i);
        float G[8];
        G[0] = bf16_bits_to_f32(q.x & 0xffffu); G[1] = bf16_bits_to_f32(q.x >> 16);
        G[2] = bf16_bits_to_f32(q.y & 0xffffu); G[3] = bf16_bits_to_f32(q.y >> 16);
        G[4] = bf16_bits_to_f32(q.z & 0xffffu); G[5] = bf16_bits_to_f32(q.z >> 16);
        G[6] = bf16_bits_to_f32(q.w & 0xffffu); G[7] = bf16_bits_to_f32(q.w >> 16);
#pragma unroll
        for (int k = 0; k < 8; k++) {
            float g = __fdiv_rn(G[k], gs.fworld);
            if (EX) g = grad_pre<EX>(c, g, acc);
            adam_body<MODE>(c, P.x[k], g, M.x[k], V.x[k]);
        }
        st8(p + i, P);
        st8(m + i, M);
        st8(v + i, V);
        uint4 o;
        o.x = pack_bf16x2(P.x[0], P.x[1]);
        o.y = pack_bf16x2(P.x[2], P.x[3]);
        o.z = pack_bf16x2(P.x[4], P.x[5]);
        o.w = pack_bf16x2(P.x[6], P.x[7]);
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_out + i), "r"(o.x),
                     "r"(o.y), "r"(o.z), "r"(o.w)
                     : "memory");
    }
    scalar_range<GradPeers<uint16_t, 0>, MODE, OutPush<0>, EX>(c, p, gs, m, v, dst, nvec, n, vec_n,
                                                               (uint64_t)blockIdx.x * 256 + threadIdx.x,
                                                               (uint64_t)gridDim.x * 256, acc);
    if (EX) stat_flush<256>(acc, stats);
}

// fp32 rank-ordered mean of the peers' gradients, 4 elements per thread-iteration; elements
// [nvec, n) one at a time, spread over the grid.
template <typename GS>
__global__ void __launch_bounds__(256)
dp_mean_kernel(GS gs, float* __restrict__ mean, uint64_t nvec, uint64_t n)
{
    const uint64_t gtid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthreads = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = gtid * 4; i < nvec; i += nthreads * 4) {
        float o[4];
        gs.template load4<1>(i, o);
        __stcs(reinterpret_cast<float4*>(mean + i), make_float4(o[0], o[1], o[2], o[3]));
    }
    for (uint64_t i = nvec + gtid; i < n; i += nthreads) mean[i] = gs.load1(i);
}

// Plain copy with 16-byte accesses (any 16-byte aligned pointers, local or peer-mapped): the
// yardstick the data-parallel kernels' link traffic is compared with.
static __global__ void __launch_bounds__(256)
copy16_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, uint64_t n16)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) dst[i] = src[i];
}

}  // namespace sfk
