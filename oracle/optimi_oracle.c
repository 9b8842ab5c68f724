/* CPU oracle for the optimizer-step hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, what the reference's foreach path
 * computes on a CUDA device: optimi/adam.py:399-453, lion.py:341-380, sgd.py:375-421,
 * stableadamw.py:475-544, adan.py:472-546, radam.py:420-479, ranger.py:476-561, one ATen op per
 * primitive, each op's fp32 result rounded to the storage type (see oracle_ops.inc).  It exists so
 * the CUDA kernels can be checked element by element on hosts without the reference installed.
 * Only the tests, the smoke check and the benchmark's cpu-baseline leg load it; the product
 * library never does.
 *
 * Pinned against: golden outputs of the unmodified reference run on a B200 (tests/golden/cuda.npz,
 * bit-exact except StableAdamW's reduction order) and on a CPU in float32 (tests/golden/cpu_f32.npz,
 * 1e-6 relative).  Single-op probes on the same B200 fixed the fp32 formula of every op.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -mfma -mf16c -fopenmp -shared -fPIC).
 * -ffp-contract=off matters: every fused multiply-add below is an explicit fmaf(), nothing else
 * may be contracted.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_F32 0
#define ORACLE_BF16 1
#define ORACLE_F16 2

/* Host-computed scalars (Python doubles in the reference, narrowed to fp32 op by op) and flags. */
typedef struct {
  double lr, beta1_comp, beta2, beta2_hat, beta2_comp, beta3_hat, beta3_comp;
  double weight_decay, eps, max_lr, momentum, rect, alpha;
  int decouple_wd, decouple_lr, kahan, update, dampening, adam_wd, lookahead, single_param_lookahead;
} oracle_scalars;

#ifdef _OPENMP
#define PARFOR _Pragma("omp parallel for schedule(static)")
#define PARSUM _Pragma("omp parallel for schedule(static) reduction(+ : acc)")
#else
#define PARFOR
#define PARSUM
#endif

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff; /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);                    /* round to nearest even */
  return (uint16_t)(u >> 16);
}
static inline float f16_to_f32(uint16_t h) {
  _Float16 x;
  memcpy(&x, &h, 2);
  return (float)x;
}
static inline uint16_t f32_to_f16(float f) {
  _Float16 x = (_Float16)f; /* round to nearest even */
  uint16_t h;
  memcpy(&h, &x, 2);
  return h;
}

#define T float
#define SFX f32
#define LD(x) (x)
#define ST(x) (x)
#include "oracle_ops.inc"
#undef T
#undef SFX
#undef LD
#undef ST

#define T uint16_t
#define SFX bf16
#define LD(x) bf16_to_f32(x)
#define ST(x) f32_to_bf16(x)
#include "oracle_ops.inc"
#undef SFX
#undef LD
#undef ST

#define SFX f16
#define LD(x) f16_to_f32(x)
#define ST(x) f32_to_f16(x)
#include "oracle_ops.inc"
#undef T
#undef SFX
#undef LD
#undef ST

#define DISPATCH(call_f32, call_bf16, call_f16) \
  switch (dtype) {                              \
    case ORACLE_F32: call_f32; return 0;        \
    case ORACLE_BF16: call_bf16; return 0;      \
    case ORACLE_F16: call_f16; return 0;        \
    default: return -1;                         \
  }

int oracle_adam(void *p, void *g, void *m, void *v, void *k, int64_t n, int dtype, const oracle_scalars *s) {
  DISPATCH(step_adam_f32(p, g, m, v, k, n, s), step_adam_bf16(p, g, m, v, k, n, s), step_adam_f16(p, g, m, v, k, n, s))
}

int oracle_lion(void *p, void *g, void *m, void *k, int64_t n, int dtype, const oracle_scalars *s) {
  DISPATCH(step_lion_f32(p, g, m, k, n, s), step_lion_bf16(p, g, m, k, n, s), step_lion_f16(p, g, m, k, n, s))
}

int oracle_sgd(void *p, void *g, void *m, void *k, int64_t n, int dtype, const oracle_scalars *s) {
  DISPATCH(step_sgd_f32(p, g, m, k, n, s), step_sgd_bf16(p, g, m, k, n, s), step_sgd_f16(p, g, m, k, n, s))
}

/* eps_sq_bits: the storage-type bit pattern of eps^2 (float bits for f32, 16-bit pattern otherwise) */
int oracle_stableadamw(void *p, void *g, void *m, void *v, void *k, int64_t n, int dtype, uint32_t eps_sq_bits,
                       const oracle_scalars *s) {
  float e32;
  memcpy(&e32, &eps_sq_bits, 4);
  DISPATCH(step_stableadamw_f32(p, g, m, v, k, n, e32, s),
           step_stableadamw_bf16(p, g, m, v, k, n, (uint16_t)eps_sq_bits, s),
           step_stableadamw_f16(p, g, m, v, k, n, (uint16_t)eps_sq_bits, s))
}

int oracle_adan(void *p, void *g, void *m, void *d, void *q, void *pg, void *k, int64_t n, int dtype,
                const oracle_scalars *s) {
  DISPATCH(step_adan_f32(p, g, m, d, q, pg, k, n, s), step_adan_bf16(p, g, m, d, q, pg, k, n, s),
           step_adan_f16(p, g, m, d, q, pg, k, n, s))
}

/* la == NULL: RAdam; la != NULL: Ranger */
int oracle_radam_ranger(void *p, void *g, void *m, void *v, void *la, void *k, int64_t n, int dtype,
                        const oracle_scalars *s) {
  DISPATCH(step_radam_ranger_f32(p, g, m, v, la, k, n, s), step_radam_ranger_bf16(p, g, m, v, la, k, n, s),
           step_radam_ranger_f16(p, g, m, v, la, k, n, s))
}

int oracle_sizeof_scalars(void) { return (int)sizeof(oracle_scalars); }
