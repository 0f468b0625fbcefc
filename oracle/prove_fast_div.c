/*
 * Exhaustive check of the three-instruction division used by the CUDA kernels.
 * TEST INFRASTRUCTURE ONLY (never linked into the shipped library).
 *
 * Claim:  for a 16-bit float input x (bf16: 8 significant bits, fp16: 11) and
 * any fp32 scale s, with r = RN(1/s),
 *     q0 = RN(x * r);  ne = RN(fma(q0, s, -x));  q = RN(fma(-ne, r, q0))
 * equals RN(x / s) bit for bit whenever nothing under- or overflows.
 * Scaling x or s by a power of two scales every intermediate by a power of
 * two, so it is enough to try every significand pair once:
 * 2^23 scale significands x (2^7 bf16 | 2^10 fp16) input significands.
 * fp16 subnormal inputs have fewer significant bits and are covered by the
 * same significand set after normalisation.
 *
 * usage: prove_fast_div [stride]   (stride>1 subsamples the scale significands)
 * exit status 0 and "mismatches 0" means the claim holds on the tried set.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static inline float u2f(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint32_t f2u(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

int main(int argc, char** argv) {
  const uint32_t stride = argc > 1 ? (uint32_t)strtoul(argv[1], 0, 10) : 1u;
  unsigned long long bad = 0, tried = 0;
#pragma omp parallel for schedule(dynamic, 4096) reduction(+ : bad, tried)
  for (uint32_t sm = 0; sm < (1u << 23); sm += stride) {
    const float s = u2f(0x3F800000u | sm); /* 1.0 <= s < 2.0 */
    const float r = 1.0f / s;              /* correctly rounded reciprocal */
    /* 10 significand bits cover fp16; the bf16 set (7 bits) is the subset with the low 3 bits clear */
    for (uint32_t xm = 0; xm < (1u << 10); ++xm) {
      const float x = u2f(0x3F800000u | (xm << 13));
      const float q0 = x * r;
      const float ne = fmaf(q0, s, -x); /* negated residual, as in the kernel */
      const float q = fmaf(-ne, r, q0);
      const float ref = x / s;
      ++tried;
      if (f2u(q) != f2u(ref)) {
        ++bad;
        if (bad < 5) fprintf(stderr, "x=%a s=%a fast=%a exact=%a\n", x, s, q, ref);
      }
    }
  }
  /* signed zeros: the quotient of a zero keeps the sign rule of IEEE division (s > 0) */
  {
    volatile float zs[2] = {0.0f, -0.0f}; /* volatile: evaluate at run time, not in the compiler */
    volatile float ss[3] = {1.0f, 0.37f, 448.0f};
    for (int i = 0; i < 2; ++i)
      for (int j = 0; j < 3; ++j) {
        const float x = zs[i], s = ss[j], r = 1.0f / s;
        const float q0 = x * r;
        /* volatile: gcc otherwise rewrites -fma(a,b,c) as fma(-a,b,-c), which is the
         * same number except for the sign of an exact zero -- the very thing tested here */
        volatile float ne = fmaf(q0, s, -x);
        const float q = fmaf(-ne, r, q0);
        ++tried;
        if (f2u(q) != f2u(x / s)) {
          ++bad;
          fprintf(stderr, "zero case x=%a s=%a fast=%a exact=%a\n", x, s, q, x / s);
        }
      }
  }
  printf("tried %llu mismatches %llu\n", tried, bad);
  return bad != 0;
}
