/* CPU oracle in plain C for the zentorch quantized-linear hot path.  TEST INFRASTRUCTURE ONLY:
 * it is linked by the tests, the smoke entry and the CPU-baseline leg of the benchmark, never by
 * the shipped library.
 *
 * The reference's arithmetic lives in AMD ZenDNN (tag zendnn-2026-WW29), which is absent from the
 * reference tree, so this file restates the algorithm from the reference's wrapper code and from the
 * formulas its tests use as ground truth.  Each function names the reference lines it follows.
 * Loops over output rows are OpenMP-parallel so that the same code doubles as a timed CPU baseline.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even, NaN kept quiet (matches torch's float -> bfloat16 cast) */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* [N,K] int8 -> [N,K/8] int32, value i of each run of eight at bits [4i,4i+4).
 * src/cpu/cpp/WOQ_Linear.cpp:294-357. Returns 0, or 1 when K is not a positive multiple of 8. */
int zt_oracle_woq_repack_weight(const int8_t *w, int64_t n, int64_t k, int32_t *out) {
  if (k < 8 || k % 8 != 0) return 1;
  const int64_t k8 = k / 8;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r) {
    for (int64_t c = 0; c < k8; ++c) {
      uint32_t word = 0;
      for (int i = 0; i < 8; ++i) word |= ((uint32_t)(w[r * k + c * 8 + i] & 0x0F)) << (4 * i);
      out[r * k8 + c] = (int32_t)word;
    }
  }
  return 0;
}

/* PyTorch CPU int4pack ([N,K/2] uint8, 64-row blocks) -> [N,K] int8 in 0..15.
 * src/cpu/cpp/WOQ_Linear.cpp:361-428. Returns 1 when N is not a multiple of 64. */
int zt_oracle_unpack_int4pack(const uint8_t *packed, int64_t n, int64_t k_half, int8_t *out) {
  if (n % 64 != 0) return 1;
  const int64_t k = 2 * k_half, nb = n / 64;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < nb; ++b) {
    const uint8_t *src = packed + b * k * 32;
    int8_t *dst = out + b * 64 * k;
    for (int64_t c = 0; c < k; ++c) {
      for (int d = 0; d < 16; ++d) {
        const uint8_t p02 = src[c * 32 + d], p13 = src[c * 32 + 16 + d];
        dst[(d + 0) * k + c] = (int8_t)(p02 & 0x0F);
        dst[(d + 32) * k + c] = (int8_t)(p02 >> 4);
        dst[(d + 16) * k + c] = (int8_t)(p13 & 0x0F);
        dst[(d + 48) * k + c] = (int8_t)(p13 >> 4);
      }
    }
  }
  return 0;
}

static inline float post_op(float y, int id, float operand) {
  switch (id) { /* ids: src/cpu/cpp/Utils.hpp:56-72 */
    case 1: return y > 0.f ? y : 0.f;
    case 2: { /* gelu, tanh approximation */
      const float c = 0.7978845608028654f, y3 = y * y * y;
      return 0.5f * y * (1.f + tanhf(c * (y + 0.044715f * y3)));
    }
    case 3: return 0.5f * y * (1.f + erff(y * 0.7071067811865476f));
    case 4: return y / (1.f + expf(-y));
    case 5: return 1.f / (1.f + expf(-y));
    case 6: return tanhf(y);
    case 7: return y * operand;
    case 8: return y + operand;
    default: return y;
  }
}

/* Y = X . dq(Wq) + b, post-ops, cast.  x: bf16 bits [M,K]; wq: N-major words (word n*(K/8)+k/8);
 * scales / zeros fp32 [G,N]; zeros NULL => signed nibbles (dq = q*s), else dq = (q-8)*s + z.
 * round_dq != 0 rounds dq to bf16 before the product, as the reference test oracle does
 * (test/unittests/op_tests/test_woq_linear.py:123-131).  post buffers are bf16 bits [M,N].
 * src/cpu/cpp/WOQ_Linear.cpp:14-176 (operand layout :138-146). y_f32 (optional) gets the value
 * before the final cast, y_bf16 (optional) the cast result. */
int zt_oracle_woq_linear(const uint16_t *x, int64_t m, int64_t k, const int32_t *wq, int64_t n,
                         const float *scales, const float *zeros, int64_t groups, const float *bias,
                         int n_post, const int *post_ids, const uint16_t *const *post_bufs, int round_dq,
                         float *y_f32, uint16_t *y_bf16) {
  if (k % 8 != 0 || groups <= 0 || k % groups != 0) return 1;
  const int64_t gs = k / groups, k8 = k / 8;
#pragma omp parallel
  {
    float *dq = (float *)malloc(sizeof(float) * (size_t)k);
#pragma omp for schedule(static)
    for (int64_t c = 0; c < n; ++c) {
      for (int64_t kk = 0; kk < k; ++kk) {
        const uint32_t word = (uint32_t)wq[c * k8 + kk / 8];
        int q = (int)((word >> (4 * (kk % 8))) & 0xF);
        const float s = scales[(kk / gs) * n + c];
        float v;
        if (zeros) {
          v = ((float)q - 8.0f) * s + zeros[(kk / gs) * n + c];
        } else {
          if (q >= 8) q -= 16;
          v = (float)q * s;
        }
        dq[kk] = round_dq ? bf16_to_f32(f32_to_bf16(v)) : v;
      }
      for (int64_t r = 0; r < m; ++r) {
        double acc = 0.0;
        for (int64_t kk = 0; kk < k; ++kk) acc += (double)bf16_to_f32(x[r * k + kk]) * (double)dq[kk];
        float y = (float)acc;
        if (bias) y += bias[c];
        int b = 0;
        for (int p = 0; p < n_post; ++p) {
          float operand = 0.f;
          if (post_ids[p] == 7 || post_ids[p] == 8) operand = bf16_to_f32(post_bufs[b++][r * n + c]);
          y = post_op(y, post_ids[p], operand);
        }
        if (y_f32) y_f32[r * n + c] = y;
        if (y_bf16) y_bf16[r * n + c] = f32_to_bf16(y);
      }
    }
    free(dq);
  }
  return 0;
}

/* Per-row symmetric s8 quantisation: s = max(absmax,1e-12)/127, q = clamp(rint(x/s),-128,127).
 * test/unittests/op_tests/test_dynamic_qlinear.py:32-36. x is fp32 (bf16 inputs are widened by the
 * caller); the current rounding mode must be the default round-to-nearest-even. */
void zt_oracle_dynamic_quantize_s8(const float *x, int64_t m, int64_t k, int8_t *q, float *scale) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
    float amax = 0.f;
    for (int64_t c = 0; c < k; ++c) {
      const float a = fabsf(x[r * k + c]);
      if (a > amax) amax = a;
    }
    if (amax < 1e-12f) amax = 1e-12f;
    const float s = amax / 127.0f;
    scale[r] = s;
    for (int64_t c = 0; c < k; ++c) {
      float v = nearbyintf(x[r * k + c] / s);
      if (v < -128.f) v = -128.f;
      if (v > 127.f) v = 127.f;
      q[r * k + c] = (int8_t)v;
    }
  }
}

/* Per-row affine u8 quantisation (extension; scheme of test/unittests/quant_utils.py:13-83 applied
 * per token): lo=min(x,0), hi=max(x,0), s=max(hi-lo,1e-12)/255, zp=clamp(rint(-lo/s),0,255),
 * q=clamp(rint(x/s)+zp,0,255). */
void zt_oracle_dynamic_quantize_u8(const float *x, int64_t m, int64_t k, uint8_t *q, float *scale, int32_t *zp) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
    float lo = 0.f, hi = 0.f;
    for (int64_t c = 0; c < k; ++c) {
      const float v = x[r * k + c];
      if (v < lo) lo = v;
      if (v > hi) hi = v;
    }
    float range = hi - lo;
    if (range < 1e-12f) range = 1e-12f;
    const float s = range / 255.0f;
    float z = nearbyintf(-lo / s);
    if (z < 0.f) z = 0.f;
    if (z > 255.f) z = 255.f;
    scale[r] = s;
    zp[r] = (int32_t)z;
    for (int64_t c = 0; c < k; ++c) {
      float v = nearbyintf(x[r * k + c] / s) + z;
      if (v < 0.f) v = 0.f;
      if (v > 255.f) v = 255.f;
      q[r * k + c] = (uint8_t)v;
    }
  }
}

/* acc[m,n] = sum_k q[m,k] * w[n,k], exact int32 (test/unittests/op_tests/test_group_matmul.py:394-409).
 * q_is_u8 selects unsigned activations. */
void zt_oracle_int8_gemm(const void *q, int q_is_u8, const int8_t *w, int64_t m, int64_t n, int64_t k, int32_t *acc) {
  const int8_t *qs = (const int8_t *)q;
  const uint8_t *qu = (const uint8_t *)q;
#pragma omp parallel for schedule(static)
  for (int64_t c = 0; c < n; ++c) {
    for (int64_t r = 0; r < m; ++r) {
      int32_t a = 0;
      if (q_is_u8)
        for (int64_t kk = 0; kk < k; ++kk) a += (int32_t)qu[r * k + kk] * (int32_t)w[c * k + kk];
      else
        for (int64_t kk = 0; kk < k; ++kk) a += (int32_t)qs[r * k + kk] * (int32_t)w[c * k + kk];
      acc[r * n + c] = a;
    }
  }
}

/* y = acc * (s_m * w_n) + b_n (fp32), optional single unary post-op, returned as fp32.
 * src/cpu/cpp/DynamicQLinear.cpp:74-135; formula test_dynamic_qlinear.py:83-92.
 * zp / wsum non-NULL apply the u8 zero-point correction acc - zp_m * sum_k w[n,k]. */
void zt_oracle_qlinear_epilogue(const int32_t *acc, int64_t m, int64_t n, const float *src_scale,
                                const float *w_scale, const float *bias, const int32_t *zp,
                                const int32_t *wsum, int post_id, float *y) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
    for (int64_t c = 0; c < n; ++c) {
      int64_t a = acc[r * n + c];
      if (zp && wsum) a -= (int64_t)zp[r] * (int64_t)wsum[c];
      float v = (float)a * (src_scale[r] * w_scale[c]);
      if (bias) v += bias[c];
      y[r * n + c] = post_op(v, post_id, 0.f);
    }
  }
}

/* ---- static-quantisation qlinear (src/cpu/cpp/QLinear.cpp:66-366; float restatement the reference's tests
 * compare with: test/unittests/quant_utils.py:13-83) ---------------------------------------------------- */

/* q = clamp(rint(x * (1 / s)) + zp): unsigned 8 bit when is_u8 (zero point given), else signed with zp = 0. */
void zt_oracle_static_quantize(const float *x, int64_t numel, float scale, int32_t zp, int is_u8, void *q) {
  const float inv = 1.0f / scale;
  const float lo = is_u8 ? 0.f : -128.f, hi = is_u8 ? 255.f : 127.f;
  for (int64_t i = 0; i < numel; ++i) {
    float r = nearbyintf(x[i] * inv) + (is_u8 ? (float)zp : 0.f);
    r = r < lo ? lo : (r > hi ? hi : r);
    if (is_u8)
      ((uint8_t *)q)[i] = (uint8_t)(int)r;
    else
      ((int8_t *)q)[i] = (int8_t)(int)r;
  }
}

/* v = post( acc' * (s_x * s_w[n]) + bias[n] ) with acc' = acc - zp_x * sum_k w[n,k]; then, when out_scale > 0,
 * the requantised value clamp(rint(v * (1 / s_o)) + zp_o) in [0, 255] (out_is_u8) or [-128, 127], returned as
 * float; else v itself.  w_scale has one element (w_per_tensor) or n.  post_id is one unary id or 0;
 * mul / add (either may be NULL) are [m, n] operands applied as v * mul + add after it. */
void zt_oracle_static_qlinear_epilogue(const int32_t *acc, int64_t m, int64_t n, float x_scale, int32_t x_zp,
                                       const int32_t *wsum, const float *w_scale, int w_per_tensor,
                                       const float *bias, int post_id, const float *mul, const float *add,
                                       float out_scale, int32_t out_zp, int out_is_u8, float *y) {
  const float inv_o = out_scale > 0.f ? 1.0f / out_scale : 0.f;
  const float lo = out_is_u8 ? 0.f : -128.f, hi = out_is_u8 ? 255.f : 127.f;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
    for (int64_t c = 0; c < n; ++c) {
      int64_t a = acc[r * n + c];
      if (wsum) a -= (int64_t)x_zp * (int64_t)wsum[c];
      float v = (float)a * (x_scale * w_scale[w_per_tensor ? 0 : c]);
      if (bias) v += bias[c];
      v = post_op(v, post_id, 0.f);
      if (mul) v *= mul[r * n + c];
      if (add) v += add[r * n + c];
      if (out_scale > 0.f) {
        v = nearbyintf(v * inv_o) + (float)out_zp;
        v = v < lo ? lo : (v > hi ? hi : v);
      }
      y[r * n + c] = v;
    }
  }
}
