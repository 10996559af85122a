/*
 * C restatement (OpenMP) of the element-wise part of the float8_experimental hot path.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE: used by the tests (cross-checked against the
 * numpy oracle and the reference's recorded outputs) and by the CPU-baseline arm of the
 * benchmark, where it stands in for PyTorch's vectorised CPU kernels so that the timed
 * CPU path is not dominated by numpy overhead.  Build: oracle/Makefile -> oracle/_build/.
 *
 * Each function cites the reference file:line it follows (paths inside
 * pytorch-labs/float8_experimental).  Rounding points restate PyTorch eager semantics:
 * bf16/fp16 element-wise ops compute in fp32 and round to the tensor dtype after every op.
 *
 * dtype codes: 0 = bf16, 1 = fp16, 2 = fp32 (bf16/fp16 as uint16 bit patterns);
 * fp8 kinds:   0 = e4m3fn (max 448), 1 = e5m2 (max 57344); fp8 values are uint8 patterns.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }
static inline float f16_to_f32(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }

/* fp32 -> bf16 (RNE) -> fp32 */
static inline float round_bf16(float v) {
  uint32_t u = f32_bits(v);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return bits_f32(0x7FC00000u);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return bits_f32(u & 0xFFFF0000u);
}
static inline float round_f16(float v) { return (float)(_Float16)v; }
static inline float round_to(float v, int dtype) {
  return dtype == 0 ? round_bf16(v) : dtype == 1 ? round_f16(v) : v;
}
static inline float load_hp(const void* x, int dtype, int64_t i) {
  if (dtype == 0) return bf16_to_f32(((const uint16_t*)x)[i]);
  if (dtype == 1) return f16_to_f32(((const uint16_t*)x)[i]);
  return ((const float*)x)[i];
}
static inline float fp8_max(int kind) { return kind == 0 ? 448.0f : 57344.0f; }

/* fp32 -> fp8 bits: saturate to the finite range, round to nearest even (subnormals
 * included); NaN -> 0x7F; -0 -> 0x80.  clamp + `x.to(float8_dtype)` at
 * float8_experimental/float8_utils.py:135-137.  Normal results are rounded with integer
 * arithmetic on the fp32 bit pattern (add half an ulp of the target, ties to even, carry
 * propagates into the exponent); subnormal results with one fp32 addition of 2^(e_min -
 * mbits + 23), whose own round-to-nearest-even leaves the target mantissa in the low bits. */
static inline uint8_t encode_fp8(float v, int kind) {
  const int mbits = kind == 0 ? 3 : 2, bias = kind == 0 ? 7 : 15;
  uint32_t u = f32_bits(v);
  const uint8_t sign = (uint8_t)((u >> 31) << 7);
  u &= 0x7FFFFFFFu;
  if (u > 0x7F800000u) return 0x7F;
  const uint32_t top = f32_bits(fp8_max(kind));
  if (u > top) u = top;
  const uint32_t min_normal = (uint32_t)(127 + 1 - bias) << 23;
  if (u < min_normal) {
    const float magic = bits_f32((uint32_t)(127 + 1 - bias - mbits + 23) << 23);
    const float f = bits_f32(u) + magic;
    return (uint8_t)(sign | (uint8_t)(f32_bits(f) - f32_bits(magic)));
  }
  const int shift = 23 - mbits;
  u += ((1u << (shift - 1)) - 1u) + ((u >> shift) & 1u);
  const uint32_t e = (u >> 23) - 127u + (uint32_t)bias;
  const uint32_t m = (u >> shift) & ((1u << mbits) - 1u);
  return (uint8_t)(sign | (e << mbits) | m);
}

static inline float decode_fp8(uint8_t b, int kind) {
  const int ebits = kind == 0 ? 4 : 5, mbits = kind == 0 ? 3 : 2, bias = kind == 0 ? 7 : 15;
  const int e = (b >> mbits) & ((1 << ebits) - 1), m = b & ((1 << mbits) - 1);
  float v;
  if (kind == 0 && e == 15 && m == 7) v = NAN;
  else if (kind == 1 && e == 31) v = m ? NAN : INFINITY;
  else if (e == 0) v = ldexpf((float)m / (float)(1 << mbits), 1 - bias);
  else v = ldexpf(1.0f + (float)m / (float)(1 << mbits), e - bias);
  return (b & 0x80) ? -v : v;
}

/* torch.max(torch.abs(x)): float8_experimental/float8_utils.py:102-104.  NaN propagates. */
float f8o_amax(const void* x, int dtype, int64_t n) {
  float best = 0.0f;
  int has_nan = 0;
#pragma omp parallel for reduction(max : best) reduction(| : has_nan) schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float a = fabsf(load_hp(x, dtype, i));
    if (a != a) has_nan = 1;
    else if (a > best) best = a;
  }
  return has_nan ? NAN : best;
}

/* amax_to_scale: float8_experimental/float8_utils.py:35-57 (reciprocal, then multiply,
 * each rounded to the dtype the amax is held in; fp16 clamp keyed on orig_dtype). */
float f8o_amax_to_scale(float amax, int kind, int amax_dtype, int orig_dtype) {
  const float eps = round_to(1e-12f, amax_dtype);
  const float c = (amax != amax) ? amax : (amax > eps ? amax : eps);
  const float r = round_to(1.0f / c, amax_dtype);
  float s = round_to(r * fp8_max(kind), amax_dtype);
  if (orig_dtype == 1 && s == s && s > 65504.0f) s = 65504.0f;
  return s;
}

/* to_fp8_saturated(tensor * scale): float8_experimental/float8_tensor.py:158-159 and
 * float8_utils.py:123-139.  product_dtype: where x*scale is rounded before the clamp. */
void f8o_cast(const void* x, int dtype, int64_t n, float scale, int kind, int product_dtype, uint8_t* out) {
  const float top = fp8_max(kind);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float p = round_to(load_hp(x, dtype, i) * scale, product_dtype);
    if (p == p) p = p > top ? top : (p < -top ? -top : p);
    out[i] = encode_fp8(p, kind);
  }
}

/* m.float() / s : float8_experimental/float8_aten_api.py:24-25 */
void f8o_dequant_f32(const uint8_t* in, int kind, int64_t n, float scale, float* out) {
  float lut[256];
  for (int b = 0; b < 256; ++b) lut[b] = decode_fp8((uint8_t)b, kind) / scale;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = lut[in[i]];
}

/* fp32 -> bf16/fp16 storage (the `.to(dtype3)` at float8_aten_api.py:28) */
void f8o_round_store(const float* in, int64_t n, int dtype, void* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    if (dtype == 0) {
      ((uint16_t*)out)[i] = (uint16_t)(f32_bits(round_bf16(in[i])) >> 16);
    } else if (dtype == 1) {
      _Float16 h = (_Float16)in[i];
      memcpy((uint16_t*)out + i, &h, 2);
    } else {
      ((float*)out)[i] = in[i];
    }
  }
}
