// The C ABI declared in include/slideformer_b200.h: host scalar state machine, argument
// checks, launches of the single-GPU kernels and the host-streaming pipeline.  The device code
// lives in sf_kernels.cuh, the peer-memory launchers in sf_adam_dp.cu.
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

#include "sf_internal.h"
#include "slideformer_b200.h"

namespace sf {

thread_local std::string t_err;
std::atomic<uint64_t> g_launches{0};
Tuning g_tune;

int fail(int code, const std::string& msg)
{
    t_err = msg;
    return code;
}

int check_launch(const char* what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(SF_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return SF_OK;
}

namespace {
std::mutex g_dev_mu;
std::unordered_map<int, DevInfo> g_dev;
}  // namespace

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

int make_ctx(const SfAdamScalars* s, StepCtx* out)
{
    out->c = sfk::K{s->beta1, s->beta2, s->omb1, s->omb2, s->bc2, s->eps, s->step_size, s->w_decay,
                    s->weight_decay, s->grad_scale};
    // cpu_adam.h:171 and :186: decay only when _weight_decay > 0.
    out->mode = (s->weight_decay > 0) ? (s->adamw_mode ? sfk::MODE_ADAMW : sfk::MODE_L2) : sfk::MODE_NODECAY;
    out->stats = s->grad_stats;
    out->ex = s->grad_stats != nullptr || s->grad_scale != 1.0f;
    return SF_OK;
}

}  // namespace sf

using namespace sf;
using namespace sfk;

namespace {

// ------------------------------------------------------------------------------------------
// host scalar state machine (cpu_adam.h:24-106)
// ------------------------------------------------------------------------------------------
struct HostAdam {
    float alpha, betta1, betta2, eps, weight_decay;
    float betta1_t, betta2_t;
    uint64_t step;
    float bc1, bc2;
    bool adamw;
    float grad_scale;          // gradient-side additions copied into every SfAdamScalars
    SfGradStats* grad_stats;
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
    s->grad_scale = o.grad_scale;
    s->grad_stats = o.grad_stats;
}

// ------------------------------------------------------------------------------------------
// launch plumbing (single-GPU kernels)
// ------------------------------------------------------------------------------------------
// f(integral_constant<int, MODE>, bool_constant<OUT>, bool_constant<EX>)
template <typename F>
int dispatch(int mode, bool has_out, bool ex, F&& f)
{
    auto with_ex = [&](auto MODE, auto OUT) -> int {
        if (ex) return f(MODE, OUT, std::true_type{});
        return f(MODE, OUT, std::false_type{});
    };
    switch (mode * 2 + (has_out ? 1 : 0)) {
        case 0: return with_ex(std::integral_constant<int, 0>{}, std::false_type{});
        case 1: return with_ex(std::integral_constant<int, 0>{}, std::true_type{});
        case 2: return with_ex(std::integral_constant<int, 1>{}, std::false_type{});
        case 3: return with_ex(std::integral_constant<int, 1>{}, std::true_type{});
        case 4: return with_ex(std::integral_constant<int, 2>{}, std::false_type{});
        default: return with_ex(std::integral_constant<int, 2>{}, std::true_type{});
    }
}

// The 128-bit kernel on local gradients: two 4-element groups per thread, one 2048-element tile
// per CTA, the fastest HBM shape measured.
template <typename GS>
int launch_vec4(const StepCtx& x, float* p, const GS& gs, float* m, float* v, uint16_t* out,
                uint64_t n, uint64_t vec_n, cudaStream_t st, int hint)
{
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    const uint64_t nvec = (vec_n < n ? vec_n : n) & ~(uint64_t)3;
    const int cps = g_tune.ctas_per_sm;
    return dispatch(x.mode, out != nullptr, x.ex, [&](auto MODE, auto OUT, auto EX) -> int {
        constexpr int M = decltype(MODE)::value;
        constexpr bool O = decltype(OUT)::value;
        constexpr bool E = decltype(EX)::value;
        constexpr int U = 2, T = 256, MINB = 1;
        uint64_t ntiles = (nvec + (uint64_t)T * 4 * U - 1) / ((uint64_t)T * 4 * U);
        int grid = grid_for(ntiles, di.sms, cps);
        if (hint)
            adam_vec4_kernel<GS, M, O, 1, U, T, MINB, E><<<grid, T, 0, st>>>(x.c, p, gs, m, v, out, nvec, n, vec_n, x.stats);
        else
            adam_vec4_kernel<GS, M, O, 0, U, T, MINB, E><<<grid, T, 0, st>>>(x.c, p, gs, m, v, out, nvec, n, vec_n, x.stats);
        return check_launch("adam_vec4_kernel");
    });
}

template <typename GS>
int launch_scalar(const StepCtx& x, float* p, const GS& gs, float* m, float* v, uint16_t* out,
                  uint64_t n, uint64_t vec_n, cudaStream_t st)
{
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    uint64_t blocks = (n + 255) / 256;
    int grid = grid_for(blocks, di.sms, 8);
    return dispatch(x.mode, out != nullptr, x.ex, [&](auto MODE, auto OUT, auto EX) -> int {
        constexpr int M = decltype(MODE)::value;
        constexpr bool E = decltype(EX)::value;
        if (decltype(OUT)::value)
            adam_scalar_kernel<GS, M, OutLocal, E><<<grid, 256, 0, st>>>(x.c, p, gs, m, v, OutLocal{out}, n, vec_n, x.stats);
        else
            adam_scalar_kernel<GS, M, OutNone, E><<<grid, 256, 0, st>>>(x.c, p, gs, m, v, OutNone{}, n, vec_n, x.stats);
        return check_launch("adam_scalar_kernel");
    });
}

template <bool G_BF16>
int launch_vec8(const StepCtx& x, float* p, const void* g, float* m, float* v, uint16_t* out,
                uint64_t n, uint64_t vec_n, cudaStream_t st)
{
    DevInfo di;
    if (int rc = device_info(&di)) return rc;
    const uint64_t nvec = (vec_n < n ? vec_n : n) & ~(uint64_t)7;
    const int cps = g_tune.ctas_per_sm;
    return dispatch(x.mode, out != nullptr, false, [&](auto MODE, auto OUT, auto) -> int {
        constexpr int M = decltype(MODE)::value;
        constexpr bool O = decltype(OUT)::value;
        constexpr int U = 1, T = 256;
        uint64_t ntiles = (nvec + (uint64_t)T * 8 * U - 1) / ((uint64_t)T * 8 * U);
        int grid = grid_for(ntiles, di.sms, cps);
        adam_vec8_kernel<G_BF16, M, O, U, T><<<grid, T, 0, st>>>(x.c, p, g, m, v, out, nvec, n, vec_n);
        return check_launch("adam_vec8_kernel");
    });
}

// Gradient dtypes of the single-GPU and host-streaming entry points.
inline bool local_dtype_ok(int g_dtype) { return g_dtype == SF_GRAD_BF16 || g_dtype == SF_GRAD_F32 || g_dtype == SF_GRAD_F16; }
inline size_t grad_elem_size(int g_dtype) { return g_dtype == SF_GRAD_F32 ? 4 : 2; }
int bad_local_dtype(int g_dtype)
{
    return fail(SF_ERR_DTYPE, "gradient dtype code " + std::to_string(g_dtype) + " is not supported (0 = bf16, 1 = fp32, 2 = fp16)");
}

int step_impl(const SfAdamScalars* s, float* p, const void* g, int g_dtype, float* m, float* v,
              uint16_t* out, uint64_t n, uint64_t vec_n, cudaStream_t st)
{
    if (!s) return fail(SF_ERR_NULL, "scalars pointer is NULL");
    if (!local_dtype_ok(g_dtype)) return bad_local_dtype(g_dtype);
    if (n == 0) return SF_OK;
    if (!p || !g || !m || !v) return fail(SF_ERR_NULL, "p, g, m and v must be non-NULL when n > 0");
    if (n > ((uint64_t)1 << 40)) return fail(SF_ERR_SIZE, "n exceeds 2^40 elements");
    if (!aligned(p, 4) || !aligned(m, 4) || !aligned(v, 4) || !aligned(g, grad_elem_size(g_dtype)) ||
        !aligned(out, 2))
        return fail(SF_ERR_ALIGN, "a buffer is not aligned to its element size");
    if (vec_n > n) vec_n = n;
    StepCtx x;
    make_ctx(s, &x);
    const bool a16 = aligned(p, 16) && aligned(m, 16) && aligned(v, 16) && aligned(g, 16) && aligned(out, 16);
    const bool a32 = a16 && aligned(p, 32) && aligned(m, 32) && aligned(v, 32);
    // misaligned buffers, tiny arrays, or a call whose tail arithmetic starts far below n
    if (!a16 || n < 4 || n - (vec_n & ~(uint64_t)3) > kMaxVectorRemainder) {
        if (g_dtype == SF_GRAD_BF16)
            return launch_scalar(x, p, GradBf16{(const uint16_t*)g}, m, v, out, n, vec_n, st);
        if (g_dtype == SF_GRAD_F16)
            return launch_scalar(x, p, GradF16{(const uint16_t*)g}, m, v, out, n, vec_n, st);
        return launch_scalar(x, p, GradF32{(const float*)g}, m, v, out, n, vec_n, st);
    }
    const int variant = g_tune.variant;
    if (variant == 2 && !x.ex && a32 && g_dtype != SF_GRAD_F16 && (g_dtype == SF_GRAD_BF16 || aligned(g, 32))) {
        if (g_dtype == SF_GRAD_BF16) return launch_vec8<true>(x, p, g, m, v, out, n, vec_n, st);
        return launch_vec8<false>(x, p, g, m, v, out, n, vec_n, st);
    }
    const int hint = variant == 0 ? 0 : 1;
    if (g_dtype == SF_GRAD_BF16)
        return launch_vec4(x, p, GradBf16{(const uint16_t*)g}, m, v, out, n, vec_n, st, hint);
    if (g_dtype == SF_GRAD_F16)
        return launch_vec4(x, p, GradF16{(const uint16_t*)g}, m, v, out, n, vec_n, st, hint);
    return launch_vec4(x, p, GradF32{(const float*)g}, m, v, out, n, vec_n, st, hint);
}

// ---- host-streaming resources: three side streams and per-slot events, one set per device ---
constexpr int kHostSlots = 8;
struct HostPipe {
    cudaStream_t s_in = nullptr, s_k = nullptr, s_out = nullptr;
    cudaEvent_t ev_start = nullptr, ev_in[kHostSlots] = {}, ev_k[kHostSlots] = {}, ev_out[kHostSlots] = {},
                ev_done = nullptr;
    uint64_t next_slot = 0;   // slots are handed out round-robin across calls
    const void* last_base = nullptr;   // scratch layout of the previous call: slot events only
    size_t last_slot_bytes = 0;        // guard a slot's memory while the layout stays the same
    int last_nslots = 0;
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
        for (int i = 0; i < kHostSlots; i++) {
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
    o.grad_scale = 1.0f;
    o.grad_stats = nullptr;
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

int sf_adam_set_grad_hooks(int id, float grad_scale, SfGradStats* grad_stats_dev)
{
    if (!(grad_scale == grad_scale) || std::isinf(grad_scale))
        return fail(SF_ERR_ARG, "grad_scale must be finite");
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_opts.find(id);
    if (it == g_opts.end()) return fail(SF_ERR_UNKNOWN_ID, "optimizer id " + std::to_string(id) + " was not created");
    it->second.grad_scale = grad_scale;
    it->second.grad_stats = grad_stats_dev;
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
    if (!local_dtype_ok(g_dtype)) return bad_local_dtype(g_dtype);
    if (n > 0 && (!p || !g || !m || !v)) return fail(SF_ERR_NULL, "p, g, m and v must be non-NULL when n > 0");
    SfAdamScalars s;
    if (int rc = sf_adam_scalars(id, step, lr, beta1, beta2, eps, weight_decay, bias_correction, &s)) return rc;
    return step_impl(&s, p, g, g_dtype, m, v, p_bf16, n, n & ~(uint64_t)15, (cudaStream_t)stream);
}

// Shared argument checks of the peer-gradient entry points.  *a16 says whether every buffer
// allows 16-byte accesses.
static int check_peers(const SfAdamScalars* s, const void* p, const void* const* peer_g, uint16_t* const* peer_out,
                       bool need_out, int world, int g_dtype, const void* m, const void* v, const void* local_out,
                       uint64_t n, bool* a16)
{
    if (!s) return fail(SF_ERR_NULL, "scalars pointer is NULL");
    if (g_dtype != SF_GRAD_BF16 && g_dtype != SF_GRAD_F32)
        return fail(SF_ERR_DTYPE, "gradient dtype code " + std::to_string(g_dtype) + " is not supported (0 = bf16, 1 = fp32)");
    if (world < 1 || world > SF_MAX_WORLD)
        return fail(SF_ERR_ARG, "world must be in [1, " + std::to_string(SF_MAX_WORLD) + "]");
    if (n == 0) return SF_OK;
    if (!p || !peer_g || !m || !v || (need_out && !peer_out))
        return fail(SF_ERR_NULL, need_out ? "p, peer_g, peer_out, m and v must be non-NULL when n > 0"
                                          : "p, peer_g, m and v must be non-NULL when n > 0");
    if (n > ((uint64_t)1 << 40)) return fail(SF_ERR_SIZE, "n exceeds 2^40 elements");
    if (!aligned(p, 4) || !aligned(m, 4) || !aligned(v, 4) || !aligned(local_out, 2))
        return fail(SF_ERR_ALIGN, "a buffer is not aligned to its element size");
    bool a = aligned(p, 16) && aligned(m, 16) && aligned(v, 16) && aligned(local_out, 16);
    for (int r = 0; r < world; r++) {
        if (!peer_g[r] || (need_out && !peer_out[r]))
            return fail(SF_ERR_NULL, "peer_g / peer_out entry " + std::to_string(r) + " is NULL");
        if (!aligned(peer_g[r], g_dtype == SF_GRAD_BF16 ? 2 : 4) || (need_out && !aligned(peer_out[r], 2)))
            return fail(SF_ERR_ALIGN, "a peer buffer is not aligned to its element size");
        a = a && aligned(peer_g[r], 16) && (!need_out || aligned(peer_out[r], 16));
    }
    *a16 = a;
    return SF_OK;
}

int sf_adam_step_sharded(const SfAdamScalars* s, float* p, const void* const* peer_g, int world,
                         int g_dtype, float* m, float* v, uint16_t* p_bf16, uint64_t n,
                         uint64_t vec_n, void* stream)
{
    bool a16 = false;
    if (int rc = check_peers(s, p, peer_g, nullptr, false, world, g_dtype, m, v, p_bf16, n, &a16)) return rc;
    if (n == 0) return SF_OK;
    if (vec_n > n) vec_n = n;
    StepCtx x;
    make_ctx(s, &x);
    return launch_sharded(x, p, peer_g, world, g_dtype, m, v, p_bf16, n, vec_n, a16, (cudaStream_t)stream);
}

int sf_adam_step_sharded_push(const SfAdamScalars* s, float* p, const void* const* peer_g,
                               uint16_t* const* peer_out, int world, int g_dtype, float* m, float* v,
                               uint64_t n, uint64_t vec_n, void* stream)
{
    bool a16 = false;
    if (int rc = check_peers(s, p, peer_g, peer_out, true, world, g_dtype, m, v, nullptr, n, &a16)) return rc;
    if (n == 0) return SF_OK;
    if (vec_n > n) vec_n = n;
    StepCtx x;
    make_ctx(s, &x);
    return launch_push(x, p, peer_g, peer_out, world, g_dtype, m, v, n, vec_n, a16, (cudaStream_t)stream);
}

int sf_adam_step_sharded_push_multi(const SfPushSegment* segs, int nseg, int world, int g_dtype, void* stream)
{
    if (g_dtype != SF_GRAD_BF16 && g_dtype != SF_GRAD_F32)
        return fail(SF_ERR_DTYPE, "gradient dtype code " + std::to_string(g_dtype) + " is not supported (0 = bf16, 1 = fp32)");
    if (world < 1 || world > SF_MULTI_MAX_WORLD)
        return fail(SF_ERR_ARG, "world must be in [1, " + std::to_string(SF_MULTI_MAX_WORLD) + "] for the multi-segment launch");
    if (nseg < 0 || nseg > SF_MULTI_MAX_SEGMENTS)
        return fail(SF_ERR_ARG, "nseg must be in [0, " + std::to_string(SF_MULTI_MAX_SEGMENTS) + "]");
    if (nseg == 0) return SF_OK;
    if (!segs) return fail(SF_ERR_NULL, "segs is NULL");
    SegTable table;
    table.nseg = 0;
    table.world = world;
    table.fworld = (float)world;
    int mode = -1;
    bool ex = false;
    SfGradStats* stats = nullptr;
    uint64_t ctas = 0;
    for (int k = 0; k < nseg; k++) {
        const SfPushSegment& sg = segs[k];
        bool a16 = false;
        if (int rc = check_peers(&sg.s, sg.p, sg.peer_g, sg.peer_out, true, world, g_dtype, sg.m, sg.v, nullptr, sg.n, &a16))
            return rc;
        if (sg.n == 0) continue;
        StepCtx x;
        make_ctx(&sg.s, &x);
        if (mode < 0) {
            mode = x.mode;
            ex = x.ex;
            stats = x.stats;
        } else if (mode != x.mode || ex != x.ex || stats != x.stats) {
            return fail(SF_ERR_ARG, "all segments of one launch must share the decay mode and the gradient hooks");
        }
        SegDev& d = table.seg[table.nseg++];
        d.c = x.c;
        d.p = sg.p;
        d.m = sg.m;
        d.v = sg.v;
        for (int r = 0; r < SF_MULTI_MAX_WORLD; r++) {
            d.g[r] = sg.peer_g[r < world ? r : 0];
            d.o[r] = sg.peer_out[r < world ? r : 0];
        }
        d.n = sg.n;
        d.vec_n = sg.vec_n < sg.n ? sg.vec_n : sg.n;
        d.nvec = a16 ? (d.vec_n & ~(uint64_t)3) : 0;
        uint64_t c = (d.nvec + 1023) / 1024;
        const uint64_t rem = (d.n - d.nvec + 255) / 256;
        if (c < (rem < 1024 ? rem : 1024)) c = rem < 1024 ? rem : 1024;
        if (c < 1) c = 1;
        d.first_cta = (uint32_t)ctas;
        d.num_ctas = (uint32_t)c;
        ctas += c;
        if (ctas > 0x7fffffffull) return fail(SF_ERR_SIZE, "too many elements for one multi-segment launch");
    }
    if (table.nseg == 0) return SF_OK;
    return launch_push_multi(table, (int)ctas, mode, ex, stats, g_dtype, (cudaStream_t)stream);
}

int sf_adam_step_sharded_nvls(const SfAdamScalars* s, float* p, const void* mc_g, uint16_t* mc_out,
                               const void* const* peer_g, uint16_t* const* peer_out, int world, float* m,
                               float* v, uint64_t n, uint64_t vec_n, void* stream)
{
    bool a16 = false;
    if (int rc = check_peers(s, p, peer_g, peer_out, true, world, SF_GRAD_BF16, m, v, nullptr, n, &a16)) return rc;
    if (n == 0) return SF_OK;
    if (!mc_g || !mc_out) return fail(SF_ERR_NULL, "the multicast addresses must be non-NULL");
    if (!a16 || !aligned(mc_g, 16) || !aligned(mc_out, 16) || !aligned(p, 32) || !aligned(m, 32) || !aligned(v, 32))
        return fail(SF_ERR_ALIGN, "the multicast path needs 16-byte aligned gradient / bf16 addresses and 32-byte "
                                  "aligned p, m, v; use sf_adam_step_sharded_push for other layouts");
    if (vec_n > n) vec_n = n;
    StepCtx x;
    make_ctx(s, &x);
    return launch_nvls(x, p, mc_g, mc_out, peer_g, peer_out, world, m, v, n, vec_n, (cudaStream_t)stream);
}

int sf_dp_mean(const void* const* peer_g, int world, int g_dtype, float* mean, uint64_t n, void* stream)
{
    if (g_dtype != SF_GRAD_BF16 && g_dtype != SF_GRAD_F32)
        return fail(SF_ERR_DTYPE, "gradient dtype code " + std::to_string(g_dtype) + " is not supported (0 = bf16, 1 = fp32)");
    if (world < 1 || world > SF_MAX_WORLD)
        return fail(SF_ERR_ARG, "world must be in [1, " + std::to_string(SF_MAX_WORLD) + "]");
    if (n == 0) return SF_OK;
    if (!peer_g || !mean) return fail(SF_ERR_NULL, "peer_g and mean must be non-NULL when n > 0");
    if (!aligned(mean, 4)) return fail(SF_ERR_ALIGN, "mean is not aligned to its element size");
    bool a16 = aligned(mean, 16);
    for (int r = 0; r < world; r++) {
        if (!peer_g[r]) return fail(SF_ERR_NULL, "peer_g[" + std::to_string(r) + "] is NULL");
        if (!aligned(peer_g[r], g_dtype == SF_GRAD_BF16 ? 2 : 4))
            return fail(SF_ERR_ALIGN, "a peer gradient is not aligned to its element size");
        a16 = a16 && aligned(peer_g[r], 16);
    }
    return launch_mean(peer_g, world, g_dtype, mean, n, a16, (cudaStream_t)stream);
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
    if (g_on_host) per_slot += round256((size_t)chunk_elems * (g_dtype == SF_GRAD_F32 ? 4 : 2));
    return 2 * per_slot;
}

int sf_adam_update_host(int id, uint64_t step, float lr, float beta1, float beta2, float eps,
                        float weight_decay, int bias_correction, float* p_host, const void* g,
                        int g_dtype, int g_on_host, float* m_host, float* v_host,
                        uint16_t* p_bf16_dev, uint64_t n, uint64_t chunk_elems, int per_chunk_scalars,
                        void* scratch, size_t scratch_bytes, void* stream)
{
    if (!local_dtype_ok(g_dtype)) return bad_local_dtype(g_dtype);
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
    const size_t gsz = grad_elem_size(g_dtype);
    // A chunk is one reference call; inside it the copies and launches move in PIECES of at most
    // g_tune.host_piece elements through up to eight scratch slots, so that a call's first upload
    // and last download (the only copies nothing of the same call overlaps) stay short and the
    // tail of one call overlaps the head of the next one issued from another stream.
    uint64_t piece = g_tune.host_piece < chunk_elems ? g_tune.host_piece : chunk_elems;
    piece = piece < 16 ? 16 : (piece & ~(uint64_t)15);
    const size_t arr = round256((size_t)piece * 4);
    const size_t garr = g_on_host ? round256((size_t)piece * gsz) : 0;
    const size_t slot_bytes = 3 * arr + garr;
    int nslots = (int)(scratch_bytes / slot_bytes);
    nslots = nslots > kHostSlots ? kHostSlots : nslots;
    if (nslots < 2) return fail(SF_ERR_SIZE, "scratch is too small for two pipeline slots");
    char* base = (char*)scratch;

    SF_CUDA(cudaEventRecord(hp->ev_start, user));
    SF_CUDA(cudaStreamWaitEvent(hp->s_in, hp->ev_start, 0));
    SF_CUDA(cudaStreamWaitEvent(hp->s_k, hp->ev_start, 0));
    SF_CUDA(cudaStreamWaitEvent(hp->s_out, hp->ev_start, 0));
    if (hp->last_base != scratch || hp->last_slot_bytes != slot_bytes || hp->last_nslots != nslots) {
        // another scratch buffer or slot layout than last time: let every copy of the earlier
        // calls finish before this call's slots are written
        SF_CUDA(cudaStreamWaitEvent(hp->s_in, hp->ev_done, 0));
        hp->last_base = scratch;
        hp->last_slot_bytes = slot_bytes;
        hp->last_nslots = nslots;
    }

    const uint64_t nchunks = (n + chunk_elems - 1) / chunk_elems;
    for (uint64_t k = 0; k < nchunks; k++) {
        const uint64_t c_lo = k * chunk_elems;
        const uint64_t c_hi = (c_lo + chunk_elems <= n) ? c_lo + chunk_elems : n;
        if (k > 0 && per_chunk_scalars)
            if (int rc = sf_adam_scalars(id, step, lr, beta1, beta2, eps, weight_decay, bias_correction, &s)) return rc;
        for (uint64_t lo = c_lo; lo < c_hi; lo += piece) {
            const uint64_t len = (lo + piece <= c_hi) ? piece : c_hi - lo;
            const int slot = (int)(hp->next_slot++ % (uint64_t)nslots);
            float* dp = (float*)(base + slot * slot_bytes);
            float* dm = (float*)(base + slot * slot_bytes + arr);
            float* dv = (float*)(base + slot * slot_bytes + 2 * arr);
            void* dg = g_on_host ? (void*)(base + slot * slot_bytes + 3 * arr) : (void*)((const char*)g + lo * gsz);
            // the slot is free once the device->host copies of its previous user are done (an
            // earlier piece of this call or of an earlier call; waiting on a never-recorded event
            // is a no-op)
            SF_CUDA(cudaStreamWaitEvent(hp->s_in, hp->ev_out[slot], 0));
            SF_CUDA(cudaMemcpyAsync(dp, p_host + lo, len * 4, cudaMemcpyHostToDevice, hp->s_in));
            SF_CUDA(cudaMemcpyAsync(dm, m_host + lo, len * 4, cudaMemcpyHostToDevice, hp->s_in));
            SF_CUDA(cudaMemcpyAsync(dv, v_host + lo, len * 4, cudaMemcpyHostToDevice, hp->s_in));
            if (g_on_host)
                SF_CUDA(cudaMemcpyAsync(dg, (const char*)g + lo * gsz, len * gsz, cudaMemcpyHostToDevice, hp->s_in));
            SF_CUDA(cudaEventRecord(hp->ev_in[slot], hp->s_in));

            SF_CUDA(cudaStreamWaitEvent(hp->s_k, hp->ev_in[slot], 0));
            // piece boundaries are multiples of 16, so only the last piece of a chunk can hold the
            // chunk's scalar tail: the same split as one launch over the whole chunk
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
    }
    // s_out is ordered after the last kernel; make the caller's stream wait for everything.
    SF_CUDA(cudaEventRecord(hp->ev_done, hp->s_out));
    SF_CUDA(cudaStreamWaitEvent(user, hp->ev_done, 0));
    return SF_OK;
}

const char* sf_last_error(void) { return t_err.c_str(); }
int sf_abi_version(void) { return SF_ABI_VERSION; }
uint64_t sf_launch_count(void) { return g_launches.load(); }

int sf_copy_bytes(void* dst, const void* src, size_t bytes, void* stream)
{
    if (bytes == 0) return SF_OK;
    if (!dst || !src) return fail(SF_ERR_NULL, "dst and src must be non-NULL");
    if (!aligned(dst, 16) || !aligned(src, 16) || (bytes & 15))
        return fail(SF_ERR_ALIGN, "dst, src and bytes must be multiples of 16");
    return launch_copy16(dst, src, bytes / 16, (cudaStream_t)stream);
}

int sf_set_host_piece(uint64_t piece_elems)
{
    if (piece_elems < 16 || (piece_elems & 15)) return fail(SF_ERR_ARG, "piece_elems must be a positive multiple of 16");
    g_tune.host_piece = piece_elems;
    return SF_OK;
}

int sf_set_nvls_tuning(int groups_per_thread)
{
    if (groups_per_thread != 1 && groups_per_thread != 2 && groups_per_thread != 4)
        return fail(SF_ERR_ARG, "groups_per_thread must be 1, 2 or 4");
    g_tune.nvls_groups = groups_per_thread;
    return SF_OK;
}

int sf_set_push_tuning(int vec, int specialise_world)
{
    if (vec >= 0 && vec != 4 && vec != 8) return fail(SF_ERR_ARG, "vec must be 4 or 8 (or negative to keep the setting)");
    if (vec >= 0) g_tune.push_vec = vec;
    if (specialise_world >= 0) g_tune.push_world = specialise_world ? 1 : 0;
    return SF_OK;
}

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
