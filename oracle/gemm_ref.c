/*
 * Plain-C restatement of the GEMM hot path.  TEST INFRASTRUCTURE ONLY: built into
 * oracle/libgemm_ref.so and loaded by tests/ (and the CPU-baseline leg of
 * bench.py); the product never links or calls it.
 *
 * Semantics follow the reference's kernel definition:
 *   - out = [bias +] a @ bt^T, a[M,K], bt[N,K] row-major, bmm per batch
 *     (ayla/gemm_jit.py:267-307);
 *   - bias joins the accumulator before rounding (ayla/gemm_jit.py:280-283);
 *   - one round-to-nearest-even from the wide accumulator to the 16-bit output
 *     (ayla/passes/lower_to_ptx_template.py:134-149);
 *   - silu(g) * u on the accumulators before that rounding
 *     (ayla/passes/lower_to_ptx_template.py:296-315, :62-81).
 * Products of two 16-bit floats are exact in fp32/fp64; the accumulator here is
 * fp64, so the only rounding is the final one.  The reference's own oracle
 * (PyTorch fp32 matmul) differs from this by fp32 summation error, i.e. by at
 * most a flip of the final rounding on a small fraction of elements.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else { /* subnormal: normalise */
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while ((man & 0x400u) == 0);
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static uint16_t f64_to_f16_rne(double d) {
  /* Round a double to binary16, ties to even, via exact scaling. */
  if (isnan(d)) return 0x7e00u;
  uint16_t sign = (uint16_t)(signbit(d) ? 0x8000u : 0);
  double a = fabs(d);
  if (a >= 65520.0) return (uint16_t)(sign | 0x7c00u); /* overflow to inf */
  if (a < 5.9604644775390625e-8 / 2) return sign;      /* below half the smallest subnormal */
  int e;
  (void)frexp(a, &e); /* a = f * 2^e, f in [0.5,1) */
  int exp = e - 1;    /* a in [2^exp, 2^(exp+1)) */
  if (exp < -14) exp = -14;
  double scaled = ldexp(a, 10 - exp); /* integer part = mantissa incl. hidden bit */
  double r = nearbyint(scaled);       /* default rounding mode: ties to even */
  uint32_t m = (uint32_t)r;
  uint32_t bits;
  if (exp == -14 && m < 1024u) {
    bits = m; /* subnormal */
  } else {
    if (m == 2048u) {
      m = 1024u;
      ++exp;
    }
    bits = ((uint32_t)(exp + 15) << 10) | (m - 1024u);
  }
  return (uint16_t)(sign | bits);
}

static float load16(const uint16_t* p, int64_t i, int is_bf16) {
  return is_bf16 ? bf16_to_f32(p[i]) : f16_to_f32(p[i]);
}

static uint16_t store16(double v, int is_bf16) {
  if (is_bf16) {
    /* double -> float is itself a rounding; do RNE to bf16 directly on the double
       by going through a float only when that is exact enough: emulate with a
       sticky bit so the two-step rounding cannot double-round. */
    float f = (float)v;
    double back = (double)f;
    if (back != v) {
      uint32_t u;
      memcpy(&u, &f, 4);
      /* make the float's last bit odd if it was inexact (round-to-odd), which
         preserves the final RNE decision at 8 bits of mantissa */
      if ((u & 1u) == 0) {
        if ((fabs(back) > fabs(v))) u -= 1u; else u += 1u;
      }
      memcpy(&f, &u, 4);
    }
    return f32_to_bf16_rne(f);
  }
  return f64_to_f16_rne(v);
}

/* out[b][m][n] = bias[n] + sum_k a[b][m][k] * bt[b][n][k]; bias may be NULL. */
void gemm_ref(const uint16_t* bias, const uint16_t* a, const uint16_t* bt, uint16_t* out,
              int64_t batch, int64_t m, int64_t n, int64_t k, int is_bf16) {
  for (int64_t b = 0; b < batch; ++b) {
    const uint16_t* ab = a + b * m * k;
    const uint16_t* bb = bt + b * n * k;
    uint16_t* ob = out + b * m * n;
    for (int64_t i = 0; i < m; ++i) {
      for (int64_t j = 0; j < n; ++j) {
        double acc = bias ? (double)load16(bias, j, is_bf16) : 0.0;
        for (int64_t p = 0; p < k; ++p) {
          acc += (double)load16(ab, i * k + p, is_bf16) * (double)load16(bb, j * k + p, is_bf16);
        }
        ob[i * n + j] = store16(acc, is_bf16);
      }
    }
  }
}

/* out[m][n] = silu(x @ wg^T) * (x @ wu^T) */
void swiglu_ref(const uint16_t* x, const uint16_t* wg, const uint16_t* wu, uint16_t* out, int64_t m,
                int64_t n, int64_t k, int is_bf16) {
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      double g = 0.0, u = 0.0;
      for (int64_t p = 0; p < k; ++p) {
        const double xv = (double)load16(x, i * k + p, is_bf16);
        g += xv * (double)load16(wg, j * k + p, is_bf16);
        u += xv * (double)load16(wu, j * k + p, is_bf16);
      }
      out[i * n + j] = store16(g / (1.0 + exp(-g)) * u, is_bf16);
    }
  }
}
