// Philox4x32-10 (Salmon et al., 2011) and a normal draw that gives the same bits on the host.
//
// The sampler takes its uniform draws from it (one counter per sampled token) and random-weights
// mode its normals (one counter per four elements). The normal is Box-Muller in double precision
// built from +, *, / and sqrt only, each rounded to nearest on its own (no fused multiply-add, no
// library logarithm or cosine), so the host statement of the same steps in numpy
// (weights/random_init.py) produces the very same doubles and, after rounding, the same stored
// values.
#pragma once
#include <stdint.h>

struct Philox4 { unsigned w[4]; };

__host__ __device__ __forceinline__ Philox4 philox4x32_10(unsigned c0, unsigned c1, unsigned c2, unsigned c3,
                                                            unsigned k0, unsigned k1) {
  const unsigned M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  unsigned c[4] = {c0, c1, c2, c3};
#pragma unroll
  for (int r = 0; r < 10; r++) {
    unsigned long long p0 = (unsigned long long)M0 * c[0], p1 = (unsigned long long)M1 * c[2];
    unsigned n0 = (unsigned)(p1 >> 32) ^ c[1] ^ k0, n1 = (unsigned)p1, n2 = (unsigned)(p0 >> 32) ^ c[3] ^ k1, n3 = (unsigned)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += W0; k1 += W1;
  }
  Philox4 out;
  out.w[0] = c[0]; out.w[1] = c[1]; out.w[2] = c[2]; out.w[3] = c[3];
  return out;
}

#ifdef __CUDACC__
// ln(u) for 0 < u < 1: u = m 2^e with m in [sqrt(1/2), sqrt(2)); ln m = 2 atanh(s), s = (m-1)/(m+1),
// as the odd series up to s^19 (|s| < 0.1716: the first dropped term is below 3e-17 of the sum).
__device__ __forceinline__ double exact_log(double u) {
  int e;
  double m = frexp(u, &e);                         // m in [0.5, 1), exact
  if (m < 0.70710678118654752440) { m = __dmul_rn(m, 2.0); e -= 1; }
  double s = __ddiv_rn(__dadd_rn(m, -1.0), __dadd_rn(m, 1.0));
  double s2 = __dmul_rn(s, s);
  double p = 1.0 / 19.0;
#pragma unroll
  for (int k = 17; k >= 1; k -= 2) p = __dadd_rn(__dmul_rn(p, s2), __ddiv_rn(1.0, (double)k));
  double lnm = __dmul_rn(__dmul_rn(2.0, s), p);
  return __dadd_rn(__dmul_rn((double)e, 0.693147180559945309417), lnm);
}

// cos and sin of 2 pi t for t = b / 2^32: the quarter turn is exact, the rest y in [0, pi/4] goes
// through the Taylor series up to y^16 / y^15 (the first dropped terms are below 1e-16).
__device__ __forceinline__ void exact_sincos_turn(unsigned b, double* c_out, double* s_out) {
  unsigned q = b >> 30;                            // quarter
  unsigned r = b & 0x3FFFFFFFu;                    // position inside the quarter, / 2^30
  bool swap = r > 0x20000000u;                     // past the middle: mirror, swap sine and cosine
  unsigned rr = swap ? 0x40000000u - r : r;
  double y = __dmul_rn((double)rr * (1.0 / 1073741824.0), 1.57079632679489661923);   // rr/2^30 is exact
  double y2 = __dmul_rn(y, y);
  double ps = -1.0 / 1307674368000.0;              // -1/15!
  ps = __dadd_rn(__dmul_rn(ps, y2), 1.0 / 6227020800.0);
  ps = __dadd_rn(__dmul_rn(ps, y2), -1.0 / 39916800.0);
  ps = __dadd_rn(__dmul_rn(ps, y2), 1.0 / 362880.0);
  ps = __dadd_rn(__dmul_rn(ps, y2), -1.0 / 5040.0);
  ps = __dadd_rn(__dmul_rn(ps, y2), 1.0 / 120.0);
  ps = __dadd_rn(__dmul_rn(ps, y2), -1.0 / 6.0);
  ps = __dadd_rn(__dmul_rn(ps, y2), 1.0);
  double sn = __dmul_rn(ps, y);
  double pc = 1.0 / 20922789888000.0;              // 1/16!
  pc = __dadd_rn(__dmul_rn(pc, y2), -1.0 / 87178291200.0);
  pc = __dadd_rn(__dmul_rn(pc, y2), 1.0 / 479001600.0);
  pc = __dadd_rn(__dmul_rn(pc, y2), -1.0 / 3628800.0);
  pc = __dadd_rn(__dmul_rn(pc, y2), 1.0 / 40320.0);
  pc = __dadd_rn(__dmul_rn(pc, y2), -1.0 / 720.0);
  pc = __dadd_rn(__dmul_rn(pc, y2), 1.0 / 24.0);
  pc = __dadd_rn(__dmul_rn(pc, y2), -0.5);
  double cs = __dadd_rn(__dmul_rn(pc, y2), 1.0);
  double c1 = swap ? sn : cs, s1 = swap ? cs : sn;  // of the angle inside the quarter
  double c, s;
  switch (q) {
    case 0: c = c1; s = s1; break;
    case 1: c = -s1; s = c1; break;
    case 2: c = -c1; s = -s1; break;
    default: c = s1; s = -c1; break;
  }
  *c_out = c;
  *s_out = s;
}

// Two standard normals from two 32-bit words: r = sqrt(-2 ln u1), u1 = (a + 1/2) / 2^32 in (0,1);
// z0 = r cos(2 pi u2), z1 = r sin(2 pi u2), u2 = b / 2^32.
__device__ __forceinline__ void exact_normal_pair(unsigned a, unsigned b, double* z0, double* z1) {
  double u1 = __dmul_rn(__dadd_rn((double)a, 0.5), 1.0 / 4294967296.0);
  double r = __dsqrt_rn(__dmul_rn(-2.0, exact_log(u1)));
  double c, s;
  exact_sincos_turn(b, &c, &s);
  *z0 = __dmul_rn(r, c);
  *z1 = __dmul_rn(r, s);
}
#endif
