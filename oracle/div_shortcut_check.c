/* Test infrastructure (not part of the product): exhaustive host check of the division shortcut the 16-bit
 * step kernels use in place of the IEEE division (div16 in optimi_b200/csrc/mta_common.cuh).
 *
 *   q0 = a*y;  r = fma(-b, q0, a);  q = fma(r, y, q0)      with y an approximate reciprocal of b
 *   guard: |a| >= 2^-60 and q is not a NaN; a zero numerator is answered by q0
 *
 * Claim: whenever the guard passes, q is the correctly rounded fp32 quotient a/b for a, b with significands of
 * at most 8 bits (bfloat16) or 11 bits (float16).  The reciprocal is taken as the correctly rounded 1/b moved by
 * -2..+2 units in the last place, which covers an approximation good to one unit.
 *
 *   div_shortcut_check bf16 [stride]   a in 2^-60..2^127, b in 2^-126..2^65, all 128 x 128 significand pairs
 *   div_shortcut_check f16  [stride]   a, b over float16's whole range (subnormals included), 1024 x 1024 pairs
 * `stride` > 1 visits every stride-th significand of each operand (a quicker run).  Exit status 0 = no wrong result.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static float as_float(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }
static uint32_t as_bits(float x) { uint32_t v; memcpy(&v, &x, 4); return v; }

int main(int argc, char** argv) {
  const int half = argc > 1 && !strcmp(argv[1], "f16");
  const int stride = argc > 2 ? atoi(argv[2]) : 1;
  const int bits = half ? 11 : 8;
  const int s0 = 1 << (bits - 1), s1 = 1 << bits;
  const int ea0 = half ? -24 : -60, ea1 = half ? 15 : 127;
  const int eb0 = half ? -24 : -126, eb1 = half ? 8 : 65;
  long wrong = 0, total = 0, turned_away = 0;
#pragma omp parallel for reduction(+ : wrong, total, turned_away) schedule(dynamic) collapse(2)
  for (int ea = ea0; ea <= ea1; ea++)
    for (int eb = eb0; eb <= eb1; eb++)
      for (int sa = s0; sa < s1; sa += stride)
        for (int sb = s0; sb < s1; sb += stride) {
          const float a = ldexpf((float)sa / (float)s0, ea), b = ldexpf((float)sb / (float)s0, eb);
          /* the double quotient of two values of <= 11 bits rounds correctly to fp32 (53 >= 2*24 + 2) */
          const float want = (float)((double)a / (double)b);
          const float y_exact = (float)(1.0 / (double)b);
          for (int p = -2; p <= 2; p++) {
            const float y = as_float(as_bits(y_exact) + p);
            const float q0 = a * y, r = fmaf(-b, q0, a), q = fmaf(r, y, q0);
            total++;
            if (!(fabsf(a) >= 0x1p-60f) || q != q) { turned_away++; continue; }
            if (as_bits(q) != as_bits(want)) wrong++;
          }
        }
  /* zero numerators: q0 = (+-0)*y must be the IEEE quotient, sign included, for every finite positive b */
  for (int eb = eb0; eb <= eb1; eb++)
    for (int sign = 0; sign < 2; sign++) {
      const float a = sign ? -0.0f : 0.0f, b = ldexpf(1.25f, eb), y = (float)(1.0 / (double)b);
      total++;
      if (as_bits(a * y) != as_bits(a / b)) wrong++;
    }
  printf("%s: %ld wrong, %ld turned away by the guard, of %ld\n", half ? "f16" : "bf16", wrong, turned_away, total);
  return wrong != 0;
}
