/* Host check of the division step used by the Normalize / row-norm kernels (div_exact in
 * shadow_b200/csrc/math.cuh): q0 = x*rcp, r = fma(-d, q0, x), q = fma(r, rcp, q0) with rcp the
 * correctly rounded reciprocal of d, for |x| and d in [2^-60, 2^60].  Compares with the IEEE quotient
 * on `n` pseudo-random pairs, a quarter of them with significands next to a power of two (the
 * worst cases for a one-step correction).  Prints the number of mismatches. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static float as_float(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint64_t state = 88172645463325252ull;
static uint64_t next(void) { state ^= state << 13; state ^= state >> 7; state ^= state << 17; return state; }

int main(int argc, char** argv) {
  long n = argc > 1 ? atol(argv[1]) : 10000000L, bad = 0;
  for (long i = 0; i < n; ++i) {
    uint64_t r = next();
    uint32_t mx = (uint32_t)r & 0x7fffff, md = (uint32_t)(r >> 23) & 0x7fffff;
    int mode = (int)((r >> 46) & 7);
    if (mode == 0) mx &= 0xff;
    if (mode == 1) md = 0x7fffff - (md & 0xff);
    if (mode == 2) md &= 0xff;
    if (mode == 3) mx = 0x7fffff - (mx & 0xff);
    uint32_t ex = 127 - 60 + (uint32_t)((r >> 49) % 121), ed = 127 - 60 + (uint32_t)((r >> 56) % 121);
    float x = as_float((ex << 23) | mx), d = as_float((ed << 23) | md);
    if (r & (1ull << 63)) x = -x;
    float rcp = 1.0f / d;                       /* correctly rounded, like __frcp_rn */
    float q0 = x * rcp;
    float res = fmaf(-d, q0, x);
    float q = fmaf(res, rcp, q0);
    if (q != x / d) ++bad;
  }
  printf("%ld\n", bad);
  return 0;
}
