/*
 * C ABI of the B200 LayerAdam library (libslideformer_b200.so).
 *
 * The library replaces the CPU Adam extension of the reference project on its per-layer
 * optimizer path.  The reference binds three functions through pybind11
 * (optimizer/layer_adam/csrc/cpu_adam.cpp:8-13: create_adam, adam_update, destroy_adam) that
 * take torch CPU tensors.  The entry points below take plain pointers and sizes instead, so
 * any host language can bind them; the element buffers are DEVICE pointers (HBM) unless an
 * entry point says otherwise.  bf16 values are raw uint16_t bit patterns.
 *
 * Conventions
 *   - every function returns an SfStatus (0 = success); sf_last_error() gives the message of
 *     the calling thread's last failure.  No C++ exception crosses this boundary.
 *   - kernels are launched asynchronously on the CUDA stream the caller passes (a
 *     cudaStream_t cast to void*; NULL = the legacy default stream).  The caller owns all
 *     buffers and the library retains none of them after the work on the stream completes.
 *   - there is no CPU implementation behind these calls: without a CUDA device they fail
 *     with SF_ERR_CUDA.
 */
#ifndef SLIDEFORMER_B200_H
#define SLIDEFORMER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SF_ABI_VERSION 2

typedef enum SfStatus {
    SF_OK = 0,
    SF_ERR_NULL = 1,       /* a required pointer is NULL                                  */
    SF_ERR_ALIGN = 2,      /* a pointer or size breaks an alignment rule the call states   */
    SF_ERR_SIZE = 3,       /* n overflows, or a range / scratch size is inconsistent       */
    SF_ERR_UNKNOWN_ID = 4, /* optimizer id was never created (the reference dereferences
                              a null pointer here, cpu_adam_impl.cpp:239-240)             */
    SF_ERR_CUDA = 5,       /* a CUDA runtime call failed; message holds cudaGetErrorString */
    SF_ERR_DTYPE = 6,      /* unsupported gradient dtype code (reference: runtime_error,
                              cpu_adam_impl.cpp:255-261)                                  */
    SF_ERR_ARG = 7         /* any other invalid argument (world size, chunk size, ...)     */
} SfStatus;

/* Gradient element type.  Parameters, exp_avg and exp_avg_sq are always fp32: the triples
 * <float, BFloat16, float>, <float, float, float> and <float, Half, float> of
 * cpu_adam_impl.cpp:187-189, which are the ones a caller with fp32 master weights can reach
 * (the reference's other six have 16-bit parameters).  fp16 gradients are accepted by the
 * single-GPU and host-streaming entry points; the data-parallel exchange takes bf16 or fp32. */
typedef enum SfGradDtype { SF_GRAD_BF16 = 0, SF_GRAD_F32 = 1, SF_GRAD_F16 = 2 } SfGradDtype;

/* Gradient statistics gathered by the same pass that applies the update, so that a loss-health
 * check (the reference tests isfinite(loss), multi_gpu/scripts/main_dp.py:102-105) or a
 * gradient-norm figure costs no extra trip through HBM.  Lives in DEVICE memory, owned and
 * zeroed by the caller; launches accumulate with atomics (one per CTA and lane), so sumsq is
 * reproducible to rounding only.  In the data-parallel entry points g is the fp32 mean of the
 * ranks' gradients and each rank accumulates the slice it owns. */
#define SF_STATS_LANES 32
typedef struct SfGradStats {
    float sumsq[SF_STATS_LANES]; /* the sum of all lanes is sum(g*g) over the elements seen */
    uint32_t nonfinite;          /* != 0 once any gradient element was Inf or NaN           */
    uint32_t reserved[31];
} SfGradStats;

/* The per-call constants of the element loop, all binary32, computed on the host exactly as
 * Adam_Optimizer::Step_AVX derives them (cpu_adam.h:124-150). */
typedef struct SfAdamScalars {
    float beta1;        /* _betta1                                  */
    float beta2;        /* _betta2                                  */
    float omb1;         /* 1 - _betta1                              */
    float omb2;         /* 1 - _betta2                              */
    float bc2;          /* _bias_correction2 = 1 / sqrt(1 - beta2^t) */
    float eps;          /* _eps                                     */
    float step_size;    /* -1 * _alpha / _bias_correction1          */
    float w_decay;      /* -1 * _alpha * _weight_decay (AdamW)      */
    float weight_decay; /* _weight_decay (L2 mode adds wd*p to g)   */
    int32_t adamw_mode; /* 1 = decoupled decay, 0 = L2              */
    /* Gradient-side additions (no counterpart in the reference's kernel; its training
     * scripts do this work in separate passes).  With grad_scale == 1 and grad_stats == NULL
     * the element loop is the reference's, bit for bit. */
    float grad_scale;   /* g is multiplied by this (one rounded fp32 product) before the
                           update; 1.0f = the gradient as it is                          */
    SfGradStats* grad_stats; /* DEVICE pointer or NULL: the launch adds its share of
                           sum(g*g) and its non-finite flag there (g before grad_scale)   */
} SfAdamScalars;


/* ---- optimizer objects: the scalar state machine --------------------------------------- */

/* Replaces create_adam_optimizer (cpu_adam_impl.cpp:91-129).  Creates or overwrites the
 * scalar block `id` (beta^t running products start at 1, step at 0). */
int sf_adam_create(int id, float lr, float beta1, float beta2, float eps, float weight_decay,
                   int adamw_mode, int should_log);

/* Replaces destroy_adam_optimizer (cpu_adam_impl.cpp:272-277).  Unknown ids are ignored. */
int sf_adam_destroy(int id);

/* Advances optimizer `id` exactly like the first half of ds_adam_step
 * (cpu_adam_impl.cpp:239-242: IncrementStep then update_state, cpu_adam.h:57-89) and
 * writes the constants one element loop uses.  Host only; needs no GPU.  One call of this
 * function corresponds to ONE reference adam_update call: the reference advances its state
 * machine on every call, and whether beta^t comes from the running float product or from
 * pow() depends on the call history. */
int sf_adam_scalars(int id, uint64_t step, float lr, float beta1, float beta2, float eps,
                    float weight_decay, int bias_correction, SfAdamScalars* out);

/* Sets the gradient-side additions that every later sf_adam_scalars(id, ...) copies into its
 * output (and therefore every sf_adam_update* call of this id applies): the multiplier and the
 * device statistics block.  Defaults after sf_adam_create: 1.0f and NULL.  Typical use: the
 * training loop computes grad_scale for the next step from the norm the last step measured
 * (a delayed global-norm clip: a layer-wise optimizer updates layer k before layer k-1 has a
 * gradient, so the current step's global norm does not exist yet) or uses it to undo a loss
 * scale. */
int sf_adam_set_grad_hooks(int id, float grad_scale, SfGradStats* grad_stats_dev);

/* ---- the fused step, HBM-resident ------------------------------------------------------ */

/* Replaces ds_adam_step / adam_update (cpu_adam_impl.cpp:220-270) for device buffers:
 * sf_adam_scalars(id, ...) followed by sf_adam_step(...) with vec_n = n rounded down to 16.
 *   p, m, v   fp32[n], updated in place
 *   g         bf16[n], fp32[n] or fp16[n] according to g_dtype, read only
 *   p_bf16    optional bf16[n] output: round-to-nearest-even copy of the UPDATED p, NaN ->
 *             0x7FC0.  Replaces the reference's separate CPU cast, transformer_layer.py:296-305.
 * Any n >= 0 and any natural element alignment is accepted.  The 128-bit vector kernel runs
 * when p, m, v, g and p_bf16 are all 16-byte aligned, otherwise a scalar kernel runs. */
int sf_adam_update(int id, uint64_t step, float lr, float beta1, float beta2, float eps,
                   float weight_decay, int bias_correction, float* p, const void* g,
                   int g_dtype, float* m, float* v, uint16_t* p_bf16, uint64_t n, void* stream);

/* The element loop alone, with explicit constants (Step_AVX, cpu_adam.h:108-197, plus the
 * Step_1 tail, cpu_adam_impl.cpp:41-68).  Elements [0, vec_n) use the vector body's
 * operation order, elements [vec_n, n) the tail's; a caller that updates a slice of what
 * the reference would process in one call passes the slice-relative position of that call's
 * (n_ref rounded down to 16) boundary, clamped to [0, n]. */
int sf_adam_step(const SfAdamScalars* s, float* p, const void* g, int g_dtype, float* m,
                 float* v, uint16_t* p_bf16, uint64_t n, uint64_t vec_n, void* stream);

/* ---- the fused step with the data-parallel gradient mean folded in ---------------------- */

/* Replaces SharedDataParallel.reduce_chunk's rank-0 arithmetic
 * (multi_gpu/shared_data_parallel.py:130-136) for the slice this rank owns: for each element
 * the kernel loads the `world` per-rank gradients through peer-mapped pointers, adds them to
 * a zero fp32 accumulator in rank order 0..world-1, divides by world, and applies the step.
 *   peer_g[r]  device pointer (local or peer-mapped) to rank r's gradient for THIS slice, n
 *              elements of g_dtype; 1 <= world <= 16
 * The caller must order this launch after every rank has finished writing its gradient and
 * must keep the gradients unchanged until the launch completes (the kernel itself never
 * waits on another GPU).  The vector kernel runs when all pointers are 16-byte aligned; a
 * grid-wide scalar kernel handles any other alignment. */
int sf_adam_step_sharded(const SfAdamScalars* s, float* p, const void* const* peer_g, int world,
                         int g_dtype, float* m, float* v, uint16_t* p_bf16, uint64_t n,
                         uint64_t vec_n, void* stream);

/* sf_adam_step_sharded with the parameter all-gather folded in as well: the bf16 copy of the
 * updated slice is stored into EVERY rank's bf16 layer buffer (peer_out[r] = device pointer,
 * local or peer-mapped, to rank r's buffer at this slice; world entries) from the same kernel
 * that pulls the gradients, so the pushes (NVLink egress) overlap the pulls (ingress) and the
 * reference's "publish the weights to all ranks" step (one shared fp32 mapping read by every
 * rank, multi_gpu/shared_data_parallel.py:92-105) needs no separate collective.  The caller
 * orders the launch after all ranks wrote their gradients and must place a cross-rank stream
 * barrier after it before any rank reads the bf16 buffers.  The kernel never waits on a peer.
 * The order of peer_out does not matter to the result; the order of peer_g is the order of the
 * fp32 sum.  Buffers that are not 16-byte aligned are handled one element at a time, spread
 * over the whole grid. */
int sf_adam_step_sharded_push(const SfAdamScalars* s, float* p, const void* const* peer_g,
                               uint16_t* const* peer_out, int world, int g_dtype, float* m, float* v,
                               uint64_t n, uint64_t vec_n, void* stream);

/* Up to SF_MAX_SEGMENTS calls of sf_adam_step_sharded_push in ONE kernel launch, for models made
 * of many small units (the reference makes one adam_update per unit and chunk,
 * multi_gpu/transformer_layer.py:417-458; a launch and two cross-rank barriers per unit cost more
 * than the update itself when a unit has a few million parameters).  Each segment keeps the
 * constants of its own reference call, so the caller still calls sf_adam_scalars once per
 * segment, in the reference's order, and the results are bit-identical to separate launches.
 * world <= 8; segments with n == 0 are skipped; all segments must share the decay mode and the
 * gradient hooks.  peer_g / peer_out: `world` pointers each, as in sf_adam_step_sharded_push. */
#define SF_MAX_SEGMENTS 32
typedef struct SfPushSegment {
    SfAdamScalars s;
    float* p;
    float* m;
    float* v;
    const void* const* peer_g;
    uint16_t* const* peer_out;
    uint64_t n;
    uint64_t vec_n;
} SfPushSegment;
int sf_adam_step_sharded_push_multi(const SfPushSegment* segs, int nseg, int world, int g_dtype, void* stream);

/* No counterpart in the reference: sf_adam_step_sharded_push with the exchange done inside the
 * NVSwitch (NVLS).  mc_g / mc_out are MULTICAST device addresses (cuMulticast* objects bound to
 * the same offset of every rank's bf16 gradient buffer / bf16 layer buffer) at this slice;
 * peer_g / peer_out are the ordinary per-rank addresses of the same slice as in
 * sf_adam_step_sharded_push.  For elements below the last multiple of 8 under vec_n the kernel
 * issues one multimem.ld_reduce (the switch adds the ranks' bf16 gradients in fp32 and returns
 * the sum rounded to bf16) and one multimem.st (the switch replicates the bf16 weights to every
 * rank); the few remaining elements take the exact peer path.  Per launch a GPU then receives
 * n * 2 * (world - 1) / world bytes of pushed weights plus n * 2 / world bytes of reduced gradients
 * instead of twice the former, and sends about as much.
 *
 * NOT bit-exact: the switch's summation order is unspecified and its result is rounded to bf16
 * before the division by world, so the mean differs from the reference's fp32 rank-order mean
 * (multi_gpu/shared_data_parallel.py:130-133) by up to half a bf16 ulp of the sum, which is the
 * accuracy of an NCCL bf16 reduce-scatter.  bf16 gradients only; gradient / bf16 addresses 16-byte
 * and p, m, v 32-byte aligned.  Ordering rules as for sf_adam_step_sharded_push. */
int sf_adam_step_sharded_nvls(const SfAdamScalars* s, float* p, const void* mc_g, uint16_t* mc_out,
                               const void* const* peer_g, uint16_t* const* peer_out, int world, float* m,
                               float* v, uint64_t n, uint64_t vec_n, void* stream);

/* The gradient mean alone, for callers that keep the reference's update(params, mean, m, v)
 * callback (shared_data_parallel.py:130-135): mean[i] = (0 + g_0[i] + ... + g_{world-1}[i]) / world
 * in fp32, rank order.  mean is a local fp32[n] device buffer. */
int sf_dp_mean(const void* const* peer_g, int world, int g_dtype, float* mean, uint64_t n, void* stream);

/* No counterpart in the reference.  Same result as sf_dp_mean into a caller buffer followed by
 * sf_adam_update on that fp32 mean, but the mean is staged in memory that is part of the
 * library image, so the call performs no device allocation of any kind.
 *
 * Who needs this: code that runs once the training step is in steady state, typically the
 * per-chunk gradient reduction on the optimizer thread in the middle of backward.  By then the
 * HBM budget is fully handed out (fp32 state, the layer window, activations), so a cudaMalloc
 * can fail, and even when it succeeds it stalls the device that the main thread is feeding
 * with kernels.  Such callers cannot allocate a staging buffer, and may not own one.
 *
 * Limit: n <= SF_STATIC_SCRATCH_MAX_ELEMS (4 Mi elements, a 16 MiB fp32 array that every GPU
 * using the library holds until the process exits); larger n is rejected with SF_ERR_SIZE
 * before anything runs -- split the range into several calls.
 *
 * The first call on each device looks up the array's device address (with that device
 * current) and remembers it; make that first call before starting any stream capture.
 * All calls on a device share the one array and it keeps whatever the last call left there.
 * Nothing has to be cleared between calls because each call rewrites mean[0, n) before reading
 * it, but two calls that can run at the same time on the GPU (different streams, no ordering)
 * race on it: keep calls on one device ordered.  Other arguments as for sf_dp_mean and
 * sf_adam_update. */
#define SF_STATIC_SCRATCH_MAX_ELEMS (4u << 20)
int sf_adam_update_dp_static(int id, uint64_t step, float lr, float beta1, float beta2, float eps,
                             float weight_decay, int bias_correction, float* p,
                             const void* const* peer_g, int world, int g_dtype, float* m, float* v,
                             uint16_t* p_bf16, uint64_t n, void* stream);

/* ---- the fused step for host-resident state -------------------------------------------- */

/* For optimizer state that does not fit in HBM: p, m, v live in PINNED host memory (the
 * reference keeps them in pageable/pinned CPU tensors, transformer_layer.py:192-196 and
 * layer_adam.py:163-173).  The call cuts [0, n) into chunks of chunk_elems, and for each
 * chunk copies p, m, v host->device into one of two scratch slots, runs the kernel, and
 * copies p, m, v device->host, with the three phases of neighbouring chunks overlapped on
 * three internal side streams ordered by CUDA events.
 *   g            gradient; g_on_host != 0 means pinned host memory (copied per chunk),
 *                otherwise a device pointer
 *   p_bf16_dev   optional DEVICE bf16[n] output (the window buffer the next forward reads)
 *   scratch      device memory of at least sf_adam_host_scratch_bytes(chunk_elems, g_dtype,
 *                g_on_host) bytes, 256-byte aligned, owned by the caller
 *   stream       the work is ordered after everything already on `stream`, and `stream`
 *                waits for the last device->host copy before later work runs
 * chunk_elems must be a multiple of 16 (so every chunk but the last stays on the vector
 * body, like the reference's 32 Mi-element chunks, transformer_layer.py:26-27).  The scalar
 * state machine advances once (one reference call per chunk would take the pow() branch
 * from the second chunk on; pass per_chunk_scalars != 0 to reproduce that).  Inside a chunk the
 * data moves in smaller pieces (sf_set_host_piece) through the scratch slots.  All calls that
 * target one device share one set of internal streams and events: issue them from one thread
 * at a time.  Two calls issued back to back from DIFFERENT streams overlap: the second one's
 * uploads start while the first one's downloads drain. */
size_t sf_adam_host_scratch_bytes(uint64_t chunk_elems, int g_dtype, int g_on_host);
int sf_adam_update_host(int id, uint64_t step, float lr, float beta1, float beta2, float eps,
                        float weight_decay, int bias_correction, float* p_host,
                        const void* g, int g_dtype, int g_on_host, float* m_host, float* v_host,
                        uint16_t* p_bf16_dev, uint64_t n, uint64_t chunk_elems,
                        int per_chunk_scalars, void* scratch, size_t scratch_bytes, void* stream);

/* ---- plumbing -------------------------------------------------------------------------- */

/* Message of the calling thread's most recent failing call ("" if none). */
const char* sf_last_error(void);

/* SF_ABI_VERSION the library was built with. */
int sf_abi_version(void);

/* Number of kernels this library has launched in the calling process (all threads). */
uint64_t sf_launch_count(void);

/* Access pattern and grid size of the vector kernel.  variant: 0 = 128-bit accesses with
 * default caching, 1 = 128-bit accesses with streaming (evict-first) hints, 2 = 256-bit
 * accesses.  ctas_per_sm: 0 = one 2048-element tile per CTA; k > 0 = persistent grid of SM
 * count * k CTAs of 256 threads walking the tiles.  A negative value keeps the current
 * setting.  Intended for benchmarking; the defaults (1, 0) are the measured best.  Not thread
 * safe. */
int sf_set_tuning(int variant, int ctas_per_sm);

/* Shape of the fused pull + push kernel (sf_adam_step_sharded_push).  vec: elements per thread,
 * 4 (8-byte peer accesses) or 8 (16-byte peer accesses, bf16 gradients).  specialise_world:
 * non-zero = use the kernels compiled for a world of 2, 4 or 8, in which every peer load of a
 * thread is issued before the first add; 0 = always the runtime-world kernel.  Negative values
 * keep the current setting; the defaults are (8, 1).  For benchmarking; not thread safe. */
int sf_set_push_tuning(int vec, int specialise_world);

/* Elements per piece of the host-streaming pipeline (sf_adam_update_host): a chunk is cut into
 * pieces of at most this many elements that move through up to eight scratch slots.  A multiple
 * of 16; default 8 Mi.  Results do not depend on it.  Not thread safe. */
int sf_set_host_piece(uint64_t piece_elems);

/* 8-element groups per thread of the NVLS kernel (sf_adam_step_sharded_nvls): 1, 2 or 4
 * in-switch reductions in flight per thread.  For benchmarking; not thread safe. */
int sf_set_nvls_tuning(int groups_per_thread);

/* A plain copy kernel (16-byte loads and stores; dst, src and bytes multiples of 16) on device
 * pointers that may be local or peer-mapped.  It exists so that the NVLink traffic of the
 * data-parallel kernels can be compared with what a bare copy reaches between the same GPUs,
 * in one direction or with every GPU sending and receiving at once. */
int sf_copy_bytes(void* dst, const void* src, size_t bytes, void* stream);

/* cudaIpc plumbing for the sharded path: export a handle for a cudaMalloc'ed base pointer
 * and map a peer's handle into this process.  handle is SF_IPC_HANDLE_BYTES bytes. */
#define SF_IPC_HANDLE_BYTES 64
/* Plain cudaMalloc / cudaFree on the current device, for buffers that must be the base of an
 * allocation so that an IPC handle can be exported for them. */
int sf_dev_alloc(size_t bytes, void** dev_ptr_out);
int sf_dev_free(void* dev_ptr);
int sf_ipc_export(void* dev_ptr, void* handle_out);
int sf_ipc_open(const void* handle, void** dev_ptr_out);
int sf_ipc_close(void* dev_ptr);

#ifdef __cplusplus
}
#endif
#endif /* SLIDEFORMER_B200_H */
