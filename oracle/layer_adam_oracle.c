/*
 * CPU restatement of the reference LayerAdam step.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker for the CUDA path: only the test suite, the smoke check and the
 * benchmark's CPU-baseline leg may build, load or call it.  Nothing in the shipped package
 * links or imports it, and it is never the thing that is measured as the product.
 *
 * Parity status: PINNED.  The functions below are checked bit-for-bit against the compiled
 * reference kernel (optimizer/layer_adam/csrc, built from its own sources by
 * oracle/build_ref.py) and against the golden vectors under tests/golden/ that were
 * generated from that compiled reference.
 *
 * Every arithmetic step is a single-rounded IEEE binary32 operation.  The file must be
 * compiled with -ffp-contract=off so that the compiler neither fuses nor splits any of the
 * explicit mul / fma operations written here.
 *
 * Reference files followed (paths inside the reference project):
 *   optimizer/layer_adam/csrc/cpu_adam.h:24-106       Adam_Optimizer scalars, IncrementStep, update_state
 *   optimizer/layer_adam/csrc/cpu_adam.h:108-197      Step_AVX, the 16-lane vector body
 *   optimizer/layer_adam/csrc/cpu_adam_impl.cpp:23-70 Step_1 scalar tail for n mod 16
 *   optimizer/layer_adam/csrc/simd.h:47-86            bf16 load (shift) and store (RNE, NaN -> 0x7FC0)
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define ORACLE_LANES 16 /* SIMD_WIDTH of the AVX-512 build, simd.h:46 */

typedef struct {
    /* cpu_adam.h:91-105 */
    float alpha, betta1, betta2, eps, weight_decay;
    float betta1_t, betta2_t;
    uint64_t step;
    float bias_correction1, bias_correction2;
    int adamw_mode;
} oracle_adam_t;

/* The per-call constants Step_AVX derives from the scalar block, cpu_adam.h:124-150. */
typedef struct {
    float betta1, betta2, omb1, omb2, bc2, eps, step_size, w_decay, weight_decay;
    int adamw_mode;
} oracle_consts_t;

/* cpu_adam.h:26-41 */
void oracle_adam_init(oracle_adam_t* o, float alpha, float betta1, float betta2, float eps,
                      float weight_decay, int adamw_mode)
{
    memset(o, 0, sizeof(*o));
    o->alpha = alpha;
    o->betta1 = betta1;
    o->betta2 = betta2;
    o->eps = eps;
    o->weight_decay = weight_decay;
    o->betta1_t = 1.0f;
    o->betta2_t = 1.0f;
    o->step = 0;
    o->adamw_mode = adamw_mode;
}

/* cpu_adam.h:57-76.  std::pow(float, size_t) promotes both arguments to double and the
 * result is narrowed to float on assignment. */
void oracle_increment_step(oracle_adam_t* o, uint64_t step, float beta1, float beta2)
{
    if (beta1 != o->betta1 || beta2 != o->betta2) {
        o->step = step;
        o->betta1 = beta1;
        o->betta2 = beta2;
        o->betta1_t = (float)pow((double)o->betta1, (double)step);
        o->betta2_t = (float)pow((double)o->betta2, (double)step);
    } else {
        o->step++;
        if (o->step != step) {
            o->betta1_t = (float)pow((double)o->betta1, (double)step);
            o->betta2_t = (float)pow((double)o->betta2, (double)step);
            o->step = step;
        } else {
            o->betta1_t = o->betta1_t * o->betta1;
            o->betta2_t = o->betta2_t * o->betta2;
        }
    }
}

/* cpu_adam.h:77-89.  The sqrt resolves to the float overload: 1 - betta2_t is a float. */
void oracle_update_state(oracle_adam_t* o, float lr, float epsilon, float weight_decay,
                         int bias_correction)
{
    o->alpha = lr;
    o->eps = epsilon;
    o->weight_decay = weight_decay;
    o->bias_correction1 = 1.0f;
    o->bias_correction2 = 1.0f;
    if (bias_correction == 1) {
        o->bias_correction1 = 1 - o->betta1_t;
        o->bias_correction2 = 1 / sqrtf(1 - o->betta2_t);
    }
}

/* cpu_adam.h:131-148 and cpu_adam_impl.cpp:35-39 (same expressions in both places). */
void oracle_consts(const oracle_adam_t* o, oracle_consts_t* c)
{
    c->betta1 = o->betta1;
    c->betta2 = o->betta2;
    c->omb1 = 1 - o->betta1;
    c->omb2 = 1 - o->betta2;
    c->bc2 = o->bias_correction2;
    c->eps = o->eps;
    c->step_size = -1 * o->alpha / o->bias_correction1;
    c->w_decay = -1 * o->alpha * o->weight_decay;
    c->weight_decay = o->weight_decay;
    c->adamw_mode = o->adamw_mode;
}

/* simd.h:47-54: a bf16 becomes the upper half of a binary32, exactly. */
static inline float bf16_to_f32(uint16_t h)
{
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* IEEE binary16 -> binary32, exact (the reference widens with _mm512_cvtph_ps, simd.h; its
 * scalar tail converts through c10::Half).  Subnormals, infinities and NaN payloads included. */
static inline float f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* simd.h:56-86 and c10::BFloat16 round_to_nearest_even: RNE on the upper 16 bits,
 * every NaN becomes 0x7FC0. */
static inline uint16_t f32_to_bf16_rne(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
    uint32_t bias = ((u >> 16) & 1u) + 0x7fffu;
    return (uint16_t)((u + bias) >> 16);
}

/* One element with the vector-body operation order, cpu_adam.h:158-193. */
static inline void body_elem(const oracle_consts_t* c, float* p, float g, float* m, float* v)
{
    float param = *p, mom = *m, var = *v;
    if (c->weight_decay > 0 && !c->adamw_mode) g = fmaf(param, c->weight_decay, g);
    mom = mom * c->betta1;
    mom = fmaf(g, c->omb1, mom);
    var = var * c->betta2;
    g = g * g;
    var = fmaf(g, c->omb2, var);
    g = sqrtf(var);
    g = fmaf(g, c->bc2, c->eps);
    g = mom / g;
    if (c->weight_decay > 0 && c->adamw_mode) param = fmaf(param, c->w_decay, param);
    param = fmaf(g, c->step_size, param);
    *p = param;
    *m = mom;
    *v = var;
}

/* One element of the n mod 16 tail, cpu_adam_impl.cpp:46-66.  The source writes separate
 * multiplies and adds; the reference's build (g++ -O3 with FMA, default contraction) fuses
 * the SECOND product of each moment update into the add, i.e. m = fma(m, b1, g*(1-b1)) and
 * v = fma(v, b2, (g*g)*(1-b2)), which rounds differently from the vector body. */
static inline void tail_elem(const oracle_consts_t* c, float* p, float g, float* m, float* v)
{
    float param = *p, mom = *m, var = *v;
    if (c->weight_decay > 0 && !c->adamw_mode) g = fmaf(param, c->weight_decay, g);
    float t1 = g * c->omb1;
    mom = fmaf(mom, c->betta1, t1);
    g = g * g;
    float t2 = g * c->omb2;
    var = fmaf(var, c->betta2, t2);
    g = sqrtf(var);
    g = fmaf(g, c->bc2, c->eps);
    g = mom / g;
    if (c->weight_decay > 0 && c->adamw_mode) param = fmaf(c->w_decay, param, param);
    param = fmaf(g, c->step_size, param);
    *p = param;
    *m = mom;
    *v = var;
}

/* Step_8 -> Step_4 -> Step_1 (cpu_adam_impl.cpp:23-148) peel 128-, 64- and 16-element
 * blocks with identical per-lane arithmetic, so the split collapses to: elements below
 * n rounded down to 16 use the body, the rest use the tail.
 * vec_n lets a caller who processes a slice of a longer reference call say where that
 * call's tail begins; pass (n & ~15) for a whole call. */
void oracle_step_f32_bf16(const oracle_consts_t* c, float* p, const uint16_t* g, float* m,
                          float* v, uint16_t* p_bf16, size_t n, size_t vec_n)
{
    if (vec_n > n) vec_n = n;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < vec_n; i++) {
        body_elem(c, p + i, bf16_to_f32(g[i]), m + i, v + i);
        if (p_bf16) p_bf16[i] = f32_to_bf16_rne(p[i]);
    }
    for (size_t i = vec_n; i < n; i++) {
        tail_elem(c, p + i, bf16_to_f32(g[i]), m + i, v + i);
        if (p_bf16) p_bf16[i] = f32_to_bf16_rne(p[i]);
    }
}

void oracle_step_f32_f32(const oracle_consts_t* c, float* p, const float* g, float* m,
                         float* v, uint16_t* p_bf16, size_t n, size_t vec_n)
{
    if (vec_n > n) vec_n = n;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < vec_n; i++) {
        body_elem(c, p + i, g[i], m + i, v + i);
        if (p_bf16) p_bf16[i] = f32_to_bf16_rne(p[i]);
    }
    for (size_t i = vec_n; i < n; i++) {
        tail_elem(c, p + i, g[i], m + i, v + i);
        if (p_bf16) p_bf16[i] = f32_to_bf16_rne(p[i]);
    }
}

/* <float, Half, float>, cpu_adam_impl.cpp:189. */
void oracle_step_f32_f16(const oracle_consts_t* c, float* p, const uint16_t* g, float* m,
                         float* v, uint16_t* p_bf16, size_t n, size_t vec_n)
{
    if (vec_n > n) vec_n = n;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < vec_n; i++) {
        body_elem(c, p + i, f16_to_f32(g[i]), m + i, v + i);
        if (p_bf16) p_bf16[i] = f32_to_bf16_rne(p[i]);
    }
    for (size_t i = vec_n; i < n; i++) {
        tail_elem(c, p + i, f16_to_f32(g[i]), m + i, v + i);
        if (p_bf16) p_bf16[i] = f32_to_bf16_rne(p[i]);
    }
}

/* The separate fp32 -> bf16 staging cast of the reference, transformer_layer.py:296-305
 * (torch copy_ from float32 to bfloat16 on the CPU). */
void oracle_f32_to_bf16(const float* src, uint16_t* dst, size_t n)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) dst[i] = f32_to_bf16_rne(src[i]);
}

/* Rank-ordered fp32 mean of per-rank gradient rows, multi_gpu/shared_data_parallel.py:130-133:
 * a zero fp32 accumulator, add_ of peer 0..world-1 in order, then a true division. */
void oracle_mean_bf16(const uint16_t* rows, size_t row_stride, int world, float* mean, size_t n)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        float acc = 0.0f;
        for (int r = 0; r < world; r++) acc = acc + bf16_to_f32(rows[(size_t)r * row_stride + i]);
        mean[i] = acc / (float)world;
    }
}

void oracle_mean_f32(const float* rows, size_t row_stride, int world, float* mean, size_t n)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        float acc = 0.0f;
        for (int r = 0; r < world; r++) acc = acc + rows[(size_t)r * row_stride + i];
        mean[i] = acc / (float)world;
    }
}

size_t oracle_sizeof_adam(void) { return sizeof(oracle_adam_t); }
size_t oracle_sizeof_consts(void) { return sizeof(oracle_consts_t); }
