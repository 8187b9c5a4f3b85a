// Launchers of the kernels that read gradients from (and store bf16 weights to) other GPUs:
// the data-parallel flavours of the fused LayerAdam step.  The kernels use ordinary loads and
// stores on peer-mapped pointers; none of them waits on another GPU, and no TMA multicast is
// involved.
#include <type_traits>

#include "sf_internal.h"

namespace sf {

using namespace sfk;

namespace {

template <typename ELT, int W>
GradPeers<ELT, W> make_peers(const void* const* peer_g, int world)
{
    GradPeers<ELT, W> gs;
    for (int r = 0; r < GradPeers<ELT, W>::CAP; r++) gs.g[r] = (const ELT*)peer_g[r < world ? r : 0];
    gs.world = world;
    gs.fworld = (float)world;
    return gs;
}

template <int W>
OutPush<W> make_dst(uint16_t* const* peer_out, int world)
{
    OutPush<W> d;
    for (int r = 0; r < OutPush<W>::CAP; r++) d.o[r] = peer_out[r < world ? r : 0];
    d.world = world;
    return d;
}

// f(integral_constant<int, MODE>, bool_constant<EX>)
template <typename F>
int dispatch_mode_ex(int mode, bool ex, F&& f)
{
    switch (mode * 2 + (ex ? 1 : 0)) {
        case 0: return f(std::integral_constant<int, 0>{}, std::false_type{});
        case 1: return f(std::integral_constant<int, 0>{}, std::true_type{});
        case 2: return f(std::integral_constant<int, 1>{}, std::false_type{});
        case 3: return f(std::integral_constant<int, 1>{}, std::true_type{});
        case 4: return f(std::integral_constant<int, 2>{}, std::false_type{});
        default: return f(std::integral_constant<int, 2>{}, std::true_type{});
    }
}

// ---- pull only: bf16 written to local memory (or nowhere) ----------------------------------
template <int W, typename GS>
int sharded_vec4(const StepCtx& x, float* p, const GS& gs, float* m, float* v, uint16_t* out, uint64_t n,
                 uint64_t vec_n, cudaStream_t st)
{
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    const uint64_t nvec = (vec_n < n ? vec_n : n) & ~(uint64_t)3;
    // One 4-element group per thread at full occupancy (256 threads x 8 CTAs per SM, 32-40
    // registers) hides the NVLink read latency; the single-GPU shape (two groups, half
    // occupancy) took 2.2x longer on two NVLink-connected B200s.
    constexpr int U = 1, T = 256, MINB = peer_min_ctas<W>();
    const uint64_t ntiles = (nvec + (uint64_t)T * 4 * U - 1) / ((uint64_t)T * 4 * U);
    const int grid = grid_for(ntiles, di.sms, g_tune.ctas_per_sm);
    return dispatch_mode_ex(x.mode, x.ex, [&](auto MODE, auto EX) -> int {
        constexpr int M = decltype(MODE)::value;
        constexpr bool E = decltype(EX)::value;
        if (out)
            adam_vec4_kernel<GS, M, true, 1, U, T, MINB, E><<<grid, T, 0, st>>>(x.c, p, gs, m, v, out, nvec, n, vec_n, x.stats);
        else
            adam_vec4_kernel<GS, M, false, 1, U, T, MINB, E><<<grid, T, 0, st>>>(x.c, p, gs, m, v, out, nvec, n, vec_n, x.stats);
        return check_launch("adam_vec4_kernel (peer gradients)");
    });
}

template <typename GS>
int sharded_scalar(const StepCtx& x, float* p, const GS& gs, float* m, float* v, uint16_t* out, uint64_t n,
                   uint64_t vec_n, cudaStream_t st)
{
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    const int grid = grid_for((n + 255) / 256, di.sms, 8);
    return dispatch_mode_ex(x.mode, x.ex, [&](auto MODE, auto EX) -> int {
        constexpr int M = decltype(MODE)::value;
        constexpr bool E = decltype(EX)::value;
        if (out)
            adam_scalar_kernel<GS, M, OutLocal, E><<<grid, 256, 0, st>>>(x.c, p, gs, m, v, OutLocal{out}, n, vec_n, x.stats);
        else
            adam_scalar_kernel<GS, M, OutNone, E><<<grid, 256, 0, st>>>(x.c, p, gs, m, v, OutNone{}, n, vec_n, x.stats);
        return check_launch("adam_scalar_kernel (peer gradients)");
    });
}

template <typename ELT, int W>
int sharded_any(const StepCtx& x, float* p, const void* const* peer_g, int world, float* m, float* v,
                uint16_t* out, uint64_t n, uint64_t vec_n, bool vec, cudaStream_t st)
{
    auto gs = make_peers<ELT, W>(peer_g, world);
    if (vec) return sharded_vec4<W>(x, p, gs, m, v, out, n, vec_n, st);
    return sharded_scalar(x, p, gs, m, v, out, n, vec_n, st);
}

// ---- pull + push ------------------------------------------------------------------------------
template <typename ELT, int W, int VEC>
int push_any(const StepCtx& x, float* p, const void* const* peer_g, uint16_t* const* peer_out, int world,
             float* m, float* v, uint64_t n, uint64_t vec_n, bool a16, cudaStream_t st)
{
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    auto gs = make_peers<ELT, W>(peer_g, world);
    auto dst = make_dst<W>(peer_out, world);
    const uint64_t body = vec_n < n ? vec_n : n;
    const uint64_t nvec = a16 ? (body & ~(uint64_t)(VEC - 1)) : 0;
    const uint64_t tile = (uint64_t)256 * VEC;
    // the grid covers the vector part one tile per CTA and is at least wide enough to spread a
    // long scalar remainder (misaligned buffers, or a call whose vec_n is far below n)
    uint64_t ctas = (nvec + tile - 1) / tile;
    const uint64_t rem_ctas = (n - nvec + 255) / 256;
    const uint64_t rem_cap = (uint64_t)di.sms * 8;
    if (ctas < (rem_ctas < rem_cap ? rem_ctas : rem_cap)) ctas = rem_ctas < rem_cap ? rem_ctas : rem_cap;
    const int grid = grid_for(ctas, di.sms, 0);
    return dispatch_mode_ex(x.mode, x.ex, [&](auto MODE, auto EX) -> int {
        constexpr int M = decltype(MODE)::value;
        constexpr bool E = decltype(EX)::value;
        adam_push_kernel<ELT, W, M, VEC, E><<<grid, 256, 0, st>>>(x.c, p, gs, m, v, dst, nvec, n, vec_n, x.stats);
        return check_launch("adam_push_kernel");
    });
}

}  // namespace

int launch_sharded(const StepCtx& x, float* p, const void* const* peer_g, int world, int g_dtype, float* m,
                   float* v, uint16_t* out, uint64_t n, uint64_t vec_n, bool a16, cudaStream_t st)
{
    const uint64_t body = vec_n < n ? vec_n : n;
    const bool vec = a16 && n >= 4 && n - (body & ~(uint64_t)3) <= kMaxVectorRemainder;
    if (g_dtype == SF_GRAD_BF16) {
        if (g_tune.push_world) {
            if (world == 2) return sharded_any<uint16_t, 2>(x, p, peer_g, world, m, v, out, n, vec_n, vec, st);
            if (world == 4) return sharded_any<uint16_t, 4>(x, p, peer_g, world, m, v, out, n, vec_n, vec, st);
            if (world == 8) return sharded_any<uint16_t, 8>(x, p, peer_g, world, m, v, out, n, vec_n, vec, st);
        }
        return sharded_any<uint16_t, 0>(x, p, peer_g, world, m, v, out, n, vec_n, vec, st);
    }
    return sharded_any<float, 0>(x, p, peer_g, world, m, v, out, n, vec_n, vec, st);
}

int launch_push(const StepCtx& x, float* p, const void* const* peer_g, uint16_t* const* peer_out, int world,
                int g_dtype, float* m, float* v, uint64_t n, uint64_t vec_n, bool a16, cudaStream_t st)
{
    if (g_dtype == SF_GRAD_BF16) {
        if (g_tune.push_world && (world == 2 || world == 4 || world == 8)) {
            // 32-byte p / m / v accesses need 32-byte aligned slices; the 16-byte peer accesses are
            // aligned whenever the 8-byte ones are and the element index is a multiple of 8.
            const bool a32 = a16 && aligned(p, 32) && aligned(m, 32) && aligned(v, 32);
            if (g_tune.push_vec == 8 && a32) {
                if (world == 2) return push_any<uint16_t, 2, 8>(x, p, peer_g, peer_out, world, m, v, n, vec_n, true, st);
                if (world == 4) return push_any<uint16_t, 4, 8>(x, p, peer_g, peer_out, world, m, v, n, vec_n, true, st);
                return push_any<uint16_t, 8, 8>(x, p, peer_g, peer_out, world, m, v, n, vec_n, true, st);
            }
            if (world == 2) return push_any<uint16_t, 2, 4>(x, p, peer_g, peer_out, world, m, v, n, vec_n, a16, st);
            if (world == 4) return push_any<uint16_t, 4, 4>(x, p, peer_g, peer_out, world, m, v, n, vec_n, a16, st);
            return push_any<uint16_t, 8, 4>(x, p, peer_g, peer_out, world, m, v, n, vec_n, a16, st);
        }
        return push_any<uint16_t, 0, 4>(x, p, peer_g, peer_out, world, m, v, n, vec_n, a16, st);
    }
    return push_any<float, 0, 4>(x, p, peer_g, peer_out, world, m, v, n, vec_n, a16, st);
}

int launch_push_multi(const SegTable& table, int total_ctas, int mode, bool ex, SfGradStats* stats, int g_dtype,
                      cudaStream_t st)
{
    return dispatch_mode_ex(mode, ex, [&](auto MODE, auto EX) -> int {
        constexpr int M = decltype(MODE)::value;
        constexpr bool E = decltype(EX)::value;
        if (g_dtype == SF_GRAD_BF16)
            adam_push_multi_kernel<uint16_t, M, E><<<total_ctas, 256, 0, st>>>(table, stats);
        else
            adam_push_multi_kernel<float, M, E><<<total_ctas, 256, 0, st>>>(table, stats);
        return check_launch("adam_push_multi_kernel");
    });
}

int launch_nvls(const StepCtx& x, float* p, const void* mc_g, uint16_t* mc_out, const void* const* peer_g,
                uint16_t* const* peer_out, int world, float* m, float* v, uint64_t n, uint64_t vec_n,
                cudaStream_t st)
{
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    auto gs = make_peers<uint16_t, 0>(peer_g, world);
    auto dst = make_dst<0>(peer_out, world);
    const uint64_t body = vec_n < n ? vec_n : n;
    const uint64_t nvec = body & ~(uint64_t)7;
    const int U = g_tune.nvls_groups;
    const uint64_t tile = (uint64_t)2048 * U;
    uint64_t ctas = (nvec + tile - 1) / tile;
    const uint64_t rem_ctas = (n - nvec + 255) / 256;
    const uint64_t rem_cap = (uint64_t)di.sms * 8;
    if (ctas < (rem_ctas < rem_cap ? rem_ctas : rem_cap)) ctas = rem_ctas < rem_cap ? rem_ctas : rem_cap;
    const int grid = grid_for(ctas, di.sms, 0);
    return dispatch_mode_ex(x.mode, x.ex, [&](auto MODE, auto EX) -> int {
        constexpr int M = decltype(MODE)::value;
        constexpr bool E = decltype(EX)::value;
        if (U == 1)
            adam_nvls_kernel<M, E, 1><<<grid, 256, 0, st>>>(x.c, p, (const uint16_t*)mc_g, m, v, mc_out, gs, dst, nvec, n, vec_n, x.stats);
        else if (U == 2)
            adam_nvls_kernel<M, E, 2><<<grid, 256, 0, st>>>(x.c, p, (const uint16_t*)mc_g, m, v, mc_out, gs, dst, nvec, n, vec_n, x.stats);
        else
            adam_nvls_kernel<M, E, 4><<<grid, 256, 0, st>>>(x.c, p, (const uint16_t*)mc_g, m, v, mc_out, gs, dst, nvec, n, vec_n, x.stats);
        return check_launch("adam_nvls_kernel");
    });
}

int launch_copy16(void* dst, const void* src, uint64_t n16, cudaStream_t st)
{
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    const int grid = grid_for((n16 + 255) / 256, di.sms, 8);
    copy16_kernel<<<grid, 256, 0, st>>>((uint4*)dst, (const uint4*)src, n16);
    return check_launch("copy16_kernel");
}

int launch_mean(const void* const* peer_g, int world, int g_dtype, float* mean, uint64_t n, bool a16,
                cudaStream_t st)
{
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    const uint64_t nvec = a16 ? (n & ~(uint64_t)3) : 0;
    const uint64_t work = nvec ? (n + 1023) / 1024 : (n + 255) / 256;
    const int grid = grid_for(work, di.sms, 8);
    if (g_dtype == SF_GRAD_BF16) {
        auto gs = make_peers<uint16_t, 0>(peer_g, world);
        dp_mean_kernel<<<grid, 256, 0, st>>>(gs, mean, nvec, n);
    } else {
        auto gs = make_peers<float, 0>(peer_g, world);
        dp_mean_kernel<<<grid, 256, 0, st>>>(gs, mean, nvec, n);
    }
    return check_launch("dp_mean_kernel");
}

}  // namespace sf
