/*
 * eb_synth.h -- the definition of the synthetic tensors this library can fill
 * buffers with (random-init weights, seeded K/V, seeded activations).
 *
 * A tensor element is a pure function of (seed, stream, index).  The same
 * inline code compiles for the host and for sm_100a, and uses only operations
 * that IEEE-754 rounds identically everywhere (integer mixing, +, *, fused
 * multiply-add written out explicitly, /, sqrt).  No libm transcendental is
 * called, so a host program and a CUDA kernel that evaluate the same
 * (seed, stream, index) get the same bits.  Host translation units that include
 * this header must be compiled with -ffp-contract=off (device code uses the
 * _rn intrinsics, which the compiler never contracts).
 *
 * The reference project (eidola-ai/eidola) has no counterpart: it never holds a
 * weight or a KV cache.  It delegates inference to a `llama-server` child process
 * (crates/eidola-app-core/src/local_models.rs:1612-1626) or to a remote provider
 * (crates/eidola-server/src/backend.rs:421-433).
 */
#ifndef EB_SYNTH_H_
#define EB_SYNTH_H_

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define EB_HD __host__ __device__ __forceinline__
#else
#include <math.h>
#define EB_HD static inline
#endif

#if defined(__CUDA_ARCH__)
#define EB_FMUL(a, b) __fmul_rn((a), (b))
#define EB_FADD(a, b) __fadd_rn((a), (b))
#define EB_FSUB(a, b) __fsub_rn((a), (b))
#define EB_FFMA(a, b, c) __fmaf_rn((a), (b), (c))
#define EB_FDIV(a, b) __fdiv_rn((a), (b))
#define EB_FSQRT(a) __fsqrt_rn((a))
#else
#define EB_FMUL(a, b) ((a) * (b))
#define EB_FADD(a, b) ((a) + (b))
#define EB_FSUB(a, b) ((a) - (b))
#define EB_FFMA(a, b, c) fmaf((a), (b), (c))
#define EB_FDIV(a, b) ((a) / (b))
#define EB_FSQRT(a) sqrtf((a))
#endif

EB_HD uint32_t eb_f2u(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
#endif
}
EB_HD float eb_u2f(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f;
  memcpy(&f, &u, 4);
  return f;
#endif
}

/* 64-bit finaliser (splitmix64 constants) over a (seed, stream, index) triple. */
EB_HD uint64_t eb_mix64(uint64_t z) {
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z;
}
EB_HD uint64_t eb_hash(uint64_t seed, uint64_t stream, uint64_t idx) {
  uint64_t z = eb_mix64(seed + 0x9E3779B97F4A7C15ull);
  z = eb_mix64(z ^ (stream * 0xD1B54A32D192ED03ull + 0x8CB92BA72F3D8DD7ull));
  z = eb_mix64(z ^ (idx * 0x9E3779B97F4A7C15ull + 0x2545F4914F6CDD1Dull));
  return z;
}

/* 24 random bits -> (0,1), exactly representable in fp32. */
EB_HD float eb_unit24(uint32_t bits24) {
  return EB_FMUL((float)(2 * bits24 + 1), 2.98023223876953125e-8f); /* (2b+1)/2^25 */
}

/* ln(u) for u in (0,1): exponent split + atanh series, |err| ~ 1e-7 relative. */
EB_HD float eb_logf_exact(float u) {
  uint32_t b = eb_f2u(u);
  int e = (int)(b >> 23) - 127;
  float m = eb_u2f((b & 0x007FFFFFu) | 0x3F800000u);
  if (m > 1.41421356f) {
    m = EB_FMUL(m, 0.5f);
    e += 1;
  }
  float s = EB_FDIV(EB_FSUB(m, 1.0f), EB_FADD(m, 1.0f));
  float s2 = EB_FMUL(s, s);
  float p = 0.11111111f;
  p = EB_FFMA(p, s2, 0.14285714f);
  p = EB_FFMA(p, s2, 0.2f);
  p = EB_FFMA(p, s2, 0.33333333f);
  p = EB_FMUL(p, s2);
  float two_s = EB_FADD(s, s);
  float lm = EB_FFMA(two_s, p, two_s);
  return EB_FFMA((float)e, 0.69314718f, lm);
}

/* cos(2*pi*u) for u in (0,1): exact quadrant reduction + degree-8/9 polynomials. */
EB_HD float eb_cos2pi_exact(float u) {
  float t = EB_FMUL(u, 4.0f);
  int q = (int)EB_FADD(t, 0.5f); /* truncation of a positive number = floor */
  float f = EB_FSUB(t, (float)q);
  float a = EB_FMUL(f, 1.57079633f);
  float a2 = EB_FMUL(a, a);
  float c = 2.48015873e-5f;
  c = EB_FFMA(c, a2, -1.38888889e-3f);
  c = EB_FFMA(c, a2, 4.16666667e-2f);
  c = EB_FFMA(c, a2, -0.5f);
  c = EB_FFMA(c, a2, 1.0f);
  float s = 2.75573192e-6f;
  s = EB_FFMA(s, a2, -1.98412698e-4f);
  s = EB_FFMA(s, a2, 8.33333333e-3f);
  s = EB_FFMA(s, a2, -1.66666667e-1f);
  s = EB_FMUL(s, a2);
  s = EB_FFMA(s, a, a);
  switch (q & 3) {
    case 0: return c;
    case 1: return -s;
    case 2: return -c;
    default: return s;
  }
}

/* Standard normal (Box-Muller, cosine branch). */
EB_HD float eb_normal(uint64_t seed, uint64_t stream, uint64_t idx) {
  uint64_t h = eb_hash(seed, stream, idx);
  float u1 = eb_unit24((uint32_t)(h >> 40));
  float u2 = eb_unit24((uint32_t)(h >> 8) & 0x00FFFFFFu);
  float r = EB_FSQRT(EB_FMUL(-2.0f, eb_logf_exact(u1)));
  return EB_FMUL(r, eb_cos2pi_exact(u2));
}

/* Uniform in [lo, hi). */
EB_HD float eb_uniform(uint64_t seed, uint64_t stream, uint64_t idx, float lo, float hi) {
  uint64_t h = eb_hash(seed, stream, idx);
  float u = eb_unit24((uint32_t)(h >> 40));
  return EB_FFMA(u, EB_FSUB(hi, lo), lo);
}

/* ---- number formats ---------------------------------------------------- */

/* fp32 -> bf16 bits, round to nearest even; NaN stays NaN. */
EB_HD uint16_t eb_bf16_from_f32(float f) {
  uint32_t u = eb_f2u(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
EB_HD float eb_bf16_to_f32(uint16_t h) { return eb_u2f(((uint32_t)h) << 16); }

/*
 * fp32 -> e4m3 (1-4-3, bias 7, max finite 448, no infinities), round to nearest
 * even, saturating to +-448; NaN -> 0x7F.  Matches cvt.rn.satfinite.e4m3x2.f32.
 */
EB_HD uint8_t eb_f32_to_e4m3(float f) {
  uint32_t u = eb_f2u(f);
  uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return (uint8_t)(sign | 0x7Fu);
  if (a >= 0x43E80000u) return (uint8_t)(sign | 0x7Eu); /* >= 464 rounds past 448: saturate */
  if (a < 0x3C800000u) {                                /* < 2^-6: subnormal grid of 2^-9 */
    float q = EB_FMUL(eb_u2f(a), 512.0f);
    /* round to nearest even without libm: add and subtract 2^23 */
    float r = EB_FSUB(EB_FADD(q, 8388608.0f), 8388608.0f);
    return (uint8_t)(sign | (uint8_t)(int)r);
  }
  uint32_t r = a + 0x7FFFFu + ((a >> 20) & 1u);
  uint32_t e = (r >> 23) - 127u + 7u;
  uint32_t m = (r >> 20) & 7u;
  uint32_t code = (e << 3) | m;
  if (code > 0x7Eu) code = 0x7Eu;
  return (uint8_t)(sign | code);
}
EB_HD float eb_e4m3_to_f32(uint8_t c) {
  uint32_t s = ((uint32_t)(c & 0x80u)) << 24;
  uint32_t e = (c >> 3) & 0xFu;
  uint32_t m = c & 7u;
  if (e == 0xFu && m == 7u) return eb_u2f(s | 0x7FC00000u);
  float v;
  if (e == 0) {
    v = EB_FMUL((float)m, 0.001953125f); /* m * 2^-9 */
  } else {
    v = eb_u2f(((e + 120u) << 23) | (m << 20));
  }
  return eb_u2f(eb_f2u(v) | s);
}

#endif /* EB_SYNTH_H_ */
