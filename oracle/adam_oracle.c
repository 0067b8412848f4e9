/* TEST INFRASTRUCTURE — CPU restatement of the reference's per-chunk optimizer
 * step.  This file is the parity checker for the CUDA path.  Only tests, the
 * smoke check and the CPU-baseline leg of the benchmark may build or call it;
 * no product code path links or loads it.
 *
 * Parity status: PINNED.  The functions below are checked bit-for-bit against
 * the reference's own AVX build (compiled unmodified into oracle/_ref, see
 * oracle/build.py) and against golden vectors generated from that build
 * (tests/golden/).
 *
 * Reference files restated (paths inside the PatrickStar project):
 *   patrickstar/ops/csrc/adam/cpu_adam.cpp:33-185   Adam_Optimizer::Step, SIMD body
 *   patrickstar/ops/csrc/adam/cpu_adam.cpp:187-377  Step_4   (same arithmetic, unrolled 4x)
 *   patrickstar/ops/csrc/adam/cpu_adam.cpp:419-698  Step_8   (same arithmetic, unrolled 8x)
 *   patrickstar/ops/csrc/includes/cpu_adam.h:143-175 IncrementStep / update_state
 *   patrickstar/ops/csrc/adam/cpu_adam.cpp:700-742  ds_adam_step (call order)
 *   patrickstar/ops/chunk_io_buff.py:85-128         fp32 master -> fp16 param chunk cast
 *   patrickstar/fp16/loss_scaler.py:133-155         inf/nan test on a gradient
 *   patrickstar/core/client.py:831-838              reduce-scatter SUM then payload /= world_size in fp16
 *
 * Every arithmetic step is one correctly rounded IEEE binary32 operation, the
 * same one a lane of the reference's AVX instructions performs: SIMD_MUL ->
 * a*b, SIMD_FMA -> fmaf, SIMD_DIV -> a/b, SIMD_SQRT -> sqrtf.  The file is
 * compiled with -ffp-contract=off so the compiler fuses nothing on its own.
 *
 * Deliberate difference: the reference sends the last (n mod SIMD_WIDTH)
 * elements of a tensor through a scalar loop (cpu_adam.cpp:146-184) whose
 * multiply-adds the compiler may or may not fuse, so its result depends on the
 * compiler and on the SIMD width of the build.  Here every element, tail
 * included, follows the SIMD body's operation order.  For n a multiple of 16
 * (every tensor of the benchmark configurations) there is no tail.
 */
#include <immintrin.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    float alpha, betta1, betta2, eps, weight_decay;
    float betta1_t, betta2_t;
    size_t step;
    float bias_correction1, bias_correction2;
    int adamw_mode;
} ps_oracle_adam;

static inline float h2f(uint16_t h) { return _cvtsh_ss(h); }
static inline uint16_t f2h(float f) { return _cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT); }

/* cpu_adam.h:93-112 — constructor defaults; betta^t starts at 1, step at 0. */
ps_oracle_adam* ps_oracle_adam_create(float alpha, float betta1, float betta2, float eps,
                                      float weight_decay, int adamw_mode)
{
    ps_oracle_adam* o = (ps_oracle_adam*)calloc(1, sizeof(ps_oracle_adam));
    o->alpha = alpha;
    o->betta1 = betta1;
    o->betta2 = betta2;
    o->eps = eps;
    o->weight_decay = weight_decay;
    o->betta1_t = 1.0f;
    o->betta2_t = 1.0f;
    o->step = 0;
    o->adamw_mode = adamw_mode;
    return o;
}

void ps_oracle_adam_destroy(ps_oracle_adam* o) { free(o); }

/* cpu_adam.h:143-162 — betta^t is either float(pow(double(betta), step)) or the
 * running float product, depending on the call history. */
void ps_oracle_adam_increment_step(ps_oracle_adam* o, size_t step, float beta1, float beta2)
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
            o->betta1_t *= o->betta1;
            o->betta2_t *= o->betta2;
        }
    }
}

/* cpu_adam.h:163-175 */
void ps_oracle_adam_update_state(ps_oracle_adam* o, float lr, float epsilon, float weight_decay,
                                 int bias_correction)
{
    o->alpha = lr;
    o->eps = epsilon;
    o->weight_decay = weight_decay;
    o->bias_correction1 = 1.0f;
    o->bias_correction2 = 1.0f;
    if (bias_correction == 1) {
        o->bias_correction1 = 1 - o->betta1_t;
        /* float sqrt and float division: verified against the reference build for
         * steps 1..399 (a double sqrt differs on a quarter of the steps) */
        o->bias_correction2 = 1 / sqrtf(1 - o->betta2_t);
    }
}

/* out[0..3] = betta1_t, betta2_t, bias_correction1, bias_correction2 */
void ps_oracle_adam_get_state(const ps_oracle_adam* o, float* out, uint64_t* step)
{
    out[0] = o->betta1_t;
    out[1] = o->betta2_t;
    out[2] = o->bias_correction1;
    out[3] = o->bias_correction2;
    *step = (uint64_t)o->step;
}

/* cpu_adam.cpp:33-144 — one element in the SIMD body's operation order. */
static inline void adam_element(float g, float* pp, float* pm, float* pv, float loss_scale,
                                float betta1, float betta2, float betta1_minus1,
                                float betta2_minus1, float bias2_sqrt, float eps, float step_size,
                                float weight_decay, float w_decay, int adamw_mode)
{
    if (loss_scale > 0) g = g / loss_scale;
    float m = *pm, v = *pv, p = *pp;
    if (weight_decay > 0 && !adamw_mode) g = fmaf(p, weight_decay, g);
    m = m * betta1;
    m = fmaf(g, betta1_minus1, m);
    v = v * betta2;
    g = g * g;
    v = fmaf(g, betta2_minus1, v);
    g = sqrtf(v);
    g = fmaf(g, bias2_sqrt, eps);
    g = m / g;
    if (weight_decay > 0 && adamw_mode) p = fmaf(p, w_decay, p);
    p = fmaf(g, step_size, p);
    *pp = p;
    *pm = m;
    *pv = v;
}

/* Adam_Optimizer::Step_8 with the object's current state.  grads is fp16 bits
 * (g_is_half) or fp32. */
void ps_oracle_adam_step(const ps_oracle_adam* o, float* params, const void* grads, float* exp_avg,
                         float* exp_avg_sq, size_t n, int g_is_half, float loss_scale)
{
    /* cpu_adam.cpp:42-46: derived scalars, each one float operation */
    const float betta1_minus1 = 1 - o->betta1;
    const float betta2_minus1 = 1 - o->betta2;
    const float step_size = -1 * o->alpha / o->bias_correction1;
    const float w_decay = -1 * o->alpha * o->weight_decay;
    const uint16_t* g16 = (const uint16_t*)grads;
    const float* g32 = (const float*)grads;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        float g = g_is_half ? h2f(g16[i]) : g32[i];
        adam_element(g, params + i, exp_avg + i, exp_avg_sq + i, loss_scale, o->betta1, o->betta2,
                     betta1_minus1, betta2_minus1, o->bias_correction2, o->eps, step_size,
                     o->weight_decay, w_decay, o->adamw_mode);
    }
}

/* ds_adam_step (cpu_adam.cpp:700-742): IncrementStep, update_state, Step_8. */
int ps_oracle_adam_update(ps_oracle_adam* o, size_t step, float lr, float beta1, float beta2,
                          float epsilon, float weight_decay, int bias_correction, float* params,
                          const void* grads, float* exp_avg, float* exp_avg_sq, size_t n,
                          int g_is_half, float loss_scale)
{
    ps_oracle_adam_increment_step(o, step, beta1, beta2);
    ps_oracle_adam_update_state(o, lr, epsilon, weight_decay, bias_correction);
    ps_oracle_adam_step(o, params, grads, exp_avg, exp_avg_sq, n, g_is_half, loss_scale);
    return 0;
}

/* chunk_io_buff.py:85-128 — fp16 param chunk := cast(fp32 master chunk), round
 * to nearest even (torch's float->half copy). */
void ps_oracle_cast_fp32_to_fp16(const float* src, uint16_t* dst, size_t n)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) dst[i] = f2h(src[i]);
}

/* loss_scaler.py:133-155 — the reference sums the gradient in fp32 and tests
 * the sum for +-inf / nan.  A sum of at most 2^26 finite halves cannot leave
 * the fp32 range, and one inf or nan element always makes the sum inf or nan,
 * so the test is "any element has all exponent bits set". */
int ps_oracle_has_inf_or_nan_f16(const uint16_t* g, size_t n)
{
    int found = 0;
#pragma omp parallel for schedule(static) reduction(| : found)
    for (size_t i = 0; i < n; i++) found |= ((g[i] & 0x7c00u) == 0x7c00u);
    return found;
}

/* client.py:838 — after the SUM reduce-scatter the local fp16 chunk is divided
 * by world_size in fp16: torch computes half(float(h) / float(world)). */
void ps_oracle_div_world_f16(uint16_t* g, size_t n, int world_size)
{
    /* `payload /= world_size` on a CUDA fp16 tensor with a Python scalar: torch
     * multiplies by the fp32 reciprocal of the scalar (its division kernel takes
     * that route for a scalar divisor) and rounds the fp32 product to fp16.  For
     * a power-of-two world size this is the true quotient. */
    const float inv = 1.0f / (float)world_size;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) g[i] = f2h(h2f(g[i]) * inv);
}

/* fp16 SUM of `world` buffers the way a reduction with fp32 accumulation and a
 * single final rounding does it; used as the tolerance anchor for the
 * collective, not as a bit-exact model of NCCL's summation order. */
void ps_oracle_sum_f16(const uint16_t* const* bufs, int world, uint16_t* out, size_t n)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        float acc = 0.f;
        for (int r = 0; r < world; r++) acc += h2f(bufs[r][i]);
        out[i] = f2h(acc);
    }
}
