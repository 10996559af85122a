// RMSNorm fused into the dynamic fp8 cast of its output (the producer of a Float8Linear
// input).  Unfused, the norm reads x and writes y (2 + 2 bytes per element) and the cast then
// reads y twice and writes fp8 (2 + 2 + 1): 9 bytes per element.  Here pass A reads x and
// produces the per-row 1/rms and the amax of y without writing y, pass B reads x again and
// writes fp8: 5 bytes per element, and y never exists in memory.
//
// Arithmetic (T = dtype of x and of the weight), every step one IEEE operation so that a
// CPU restatement gives the same bits:
//   ss_t   = per-thread sum of fl(x*x) in fp32, thread t owning the 8-element chunks
//            c with (c mod 256) == t, in increasing order
//   total  = butterfly sum over the 32 lanes of each warp, then over the 8 warp sums
//   rstd   = fl(1 / fl(sqrt(fl(fl(total / cols) + eps))))
//   y      = RN_T(float(RN_T(fl(x * rstd))) * float(w))
// which is RMSNorm.forward of float8_experimental/benchmarks/profile_linear_float8.py:69-74
// with the reduction order fixed.  The cast of y is the dynamic cast of cast.cu
// (float8_experimental/float8_scaling_utils.py:33-62).
#include "common.cuh"

namespace f8b200 {
namespace {

constexpr int kNormThreads = 256;

template <int HP>
__device__ __forceinline__ float load_hp(const void* base, int64_t i) {
  if constexpr (HP == F8B200_BF16) {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
  } else if constexpr (HP == F8B200_FP16) {
    return __half2float(reinterpret_cast<const __half*>(base)[i]);
  } else {
    return reinterpret_cast<const float*>(base)[i];
  }
}

// Widens the eight 16-bit values of a 16-byte word.
template <int HP>
__device__ __forceinline__ void widen8(const uint4& q, float (&v)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (HP == F8B200_BF16) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    } else {
      v[2 * i] = __half2float(__ushort_as_half((unsigned short)(w[i] & 0xFFFFu)));
      v[2 * i + 1] = __half2float(__ushort_as_half((unsigned short)(w[i] >> 16)));
    }
  }
}

// Loads chunk `c` (elements 8c .. 8c+7) of a row; `n` of them exist.
template <int HP, bool VEC>
__device__ __forceinline__ void load_chunk(const char* row, int64_t c, int n, float (&v)[8]) {
  if constexpr (VEC) {
    widen8<HP>(__ldg(reinterpret_cast<const uint4*>(row) + c), v);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = j < n ? load_hp<HP>(row, c * 8 + j) : 0.0f;
  }
}

// Sum over the CTA in a fixed order: xor butterfly inside each warp, then over the warp sums.
__device__ __forceinline__ float block_sum_fixed(float v, float* smem) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
  if (lane == 0) smem[w] = v;
  __syncthreads();
  float t = lane < (kNormThreads / 32) ? smem[lane] : 0.0f;
#pragma unroll
  for (int off = (kNormThreads / 64); off > 0; off >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xFFFFFFFFu, t, off));
  t = __shfl_sync(0xFFFFFFFFu, t, 0);
  __syncthreads();  // smem is reused by the next row
  return t;
}

template <int HP>
__device__ __forceinline__ float norm_value(float x, float rstd, float w) {
  const float o = round_hp<HP>(__fmul_rn(x, rstd));
  return round_hp<HP>(__fmul_rn(o, w));
}

__device__ __forceinline__ uint32_t abs_bits(float y) { return __float_as_uint(y) & 0x7FFFFFFFu; }

// Pass A: rstd per row and the amax of y over the whole tensor.
template <int HP, bool VEC>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_amax_kernel(const char* __restrict__ x, int64_t ld_bytes, int64_t rows, int64_t cols,
                    const char* __restrict__ weight, float eps, float* __restrict__ rstd_out,
                    uint32_t* __restrict__ amax_bits) {
  __shared__ float red[kNormThreads / 32];
  __shared__ uint32_t redu[kNormThreads / 32];
  const int64_t chunks = (cols + 7) / 8;
  uint32_t amax = 0;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const char* row = x + r * ld_bytes;
    float ss = 0.0f;
    for (int64_t c = threadIdx.x; c < chunks; c += kNormThreads) {
      float v[8];
      const int n = (int)min((int64_t)8, cols - c * 8);
      load_chunk<HP, VEC>(row, c, n, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = __fadd_rn(ss, __fmul_rn(v[j], v[j]));
    }
    const float total = block_sum_fixed(ss, red);
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)cols), eps)));
    if (threadIdx.x == 0) rstd_out[r] = rstd;
    // second sweep over the row (16 KB for 8192 bf16 columns: served from L1/L2)
    for (int64_t c = threadIdx.x; c < chunks; c += kNormThreads) {
      float v[8], w[8];
      const int n = (int)min((int64_t)8, cols - c * 8);
      load_chunk<HP, VEC>(row, c, n, v);
      load_chunk<HP, VEC>(weight, c, n, w);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < n) amax = max(amax, abs_bits(norm_value<HP>(v[j], rstd, w[j])));
    }
  }
  amax = warp_max_u32(amax);
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  if (lane == 0) redu[wp] = amax;
  __syncthreads();
  if (wp == 0) {
    amax = lane < (kNormThreads / 32) ? redu[lane] : 0u;
    amax = warp_max_u32(amax);
    if (lane == 0 && amax > *reinterpret_cast<volatile uint32_t*>(amax_bits)) atomicMax(amax_bits, amax);
  }
}

// Pass B: y again from x, rstd and the weight; scale from the amax; saturating RNE cast.
template <int HP, int KIND, bool VEC>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_cast_kernel(const char* __restrict__ x, int64_t ld_bytes, int64_t rows, int64_t cols,
                    const char* __restrict__ weight, const float* __restrict__ rstd_in,
                    const float* __restrict__ amax_in, float* __restrict__ scale_out, uint8_t* __restrict__ out,
                    int64_t ld_out) {
  const float scale = amax_to_scale_dev(__ldg(amax_in), fp8_max_of(KIND), HP, HP == F8B200_FP16);
  if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out != nullptr) *scale_out = scale;
  const int64_t chunks = (cols + 7) / 8;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const char* row = x + r * ld_bytes;
    const float rstd = __ldg(rstd_in + r);
    uint8_t* orow = out + r * ld_out;
    for (int64_t c = threadIdx.x; c < chunks; c += kNormThreads) {
      float v[8], w[8], q[8];
      const int n = (int)min((int64_t)8, cols - c * 8);
      load_chunk<HP, VEC>(row, c, n, v);
      load_chunk<HP, VEC>(weight, c, n, w);
#pragma unroll
      for (int j = 0; j < 8; ++j) q[j] = __fmul_rn(norm_value<HP>(v[j], rstd, w[j]), scale);
      // the product with a 0-dim scale is rounded to T before the clamp (fp32 input: no rounding)
      const uint32_t lo = cast4<HP, KIND>(q[0], q[1], q[2], q[3], HP != F8B200_FP32);
      const uint32_t hi = cast4<HP, KIND>(q[4], q[5], q[6], q[7], HP != F8B200_FP32);
      if (VEC && n == 8) {
        *reinterpret_cast<uint2*>(orow + c * 8) = make_uint2(lo, hi);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < n) orow[c * 8 + j] = (uint8_t)(((j < 4 ? lo : hi) >> (8 * (j & 3))) & 0xFFu);
      }
    }
  }
}

// ---- fast path: 16-bit dtypes, rows of at most CH * 2048 elements held in registers --------
// Same arithmetic as above with fewer instructions: x*x is exact in fp32 for 16-bit inputs, so
// fma(x, x, ss) equals fl(ss + fl(x*x)); RN_T of two products is one packed convert; the product of
// two T values rounded to T is one packed multiply (the exact product fits fp32), which covers both
// "* w" and "* scale" (the scale is derived in T arithmetic, hence representable in T).
template <int HP>
__device__ __forceinline__ uint32_t pack_round2(float a, float b) {
  if constexpr (HP == F8B200_BF16) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&p);
  } else {
    const __half2 p = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&p);
  }
}
template <int HP>
__device__ __forceinline__ uint32_t mul2(uint32_t a2, uint32_t b2) {
  if constexpr (HP == F8B200_BF16) {
    const __nv_bfloat162 p = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a2),
                                     *reinterpret_cast<const __nv_bfloat162*>(&b2));
    return *reinterpret_cast<const uint32_t*>(&p);
  } else {
    const __half2 p = __hmul2(*reinterpret_cast<const __half2*>(&a2), *reinterpret_cast<const __half2*>(&b2));
    return *reinterpret_cast<const uint32_t*>(&p);
  }
}
template <int HP>
__device__ __forceinline__ void unpack_pair(uint32_t x2, float& a, float& b) {
  if constexpr (HP == F8B200_BF16) {
    a = __uint_as_float(x2 << 16);
    b = __uint_as_float(x2 & 0xFFFF0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&x2));
    a = f.x;
    b = f.y;
  }
}
// y (two packed T values) of two packed x values
template <int HP>
__device__ __forceinline__ uint32_t norm_pair(uint32_t x2, float rstd, uint32_t w2) {
  float a, b;
  unpack_pair<HP>(x2, a, b);
  return mul2<HP>(pack_round2<HP>(__fmul_rn(a, rstd), __fmul_rn(b, rstd)), w2);
}
template <int HP>
__device__ __forceinline__ float sumsq_word(uint32_t x2, float ss) {
  float a, b;
  unpack_pair<HP>(x2, a, b);
  return fmaf(b, b, fmaf(a, a, ss));
}
template <int HP, int KIND>
__device__ __forceinline__ uint32_t pair_to_fp8(uint32_t y2, uint32_t s2) {
  const uint32_t p = mul2<HP>(y2, s2);
  if constexpr (HP == F8B200_BF16) {
    return cvt_pair_raw<KIND>(__uint_as_float(p << 16), __uint_as_float(p & 0xFFFF0000u));
  } else {
    const __nv_fp8_interpretation_t interp = (KIND == F8B200_E4M3) ? __NV_E4M3 : __NV_E5M2;
    __half2_raw r;
    r.x = (unsigned short)(p & 0xFFFFu);
    r.y = (unsigned short)(p >> 16);
    return __nv_cvt_halfraw2_to_fp8x2(r, __NV_SATFINITE, interp);
  }
}

template <int HP, int CH>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_amax_fast_kernel(const char* __restrict__ x, int64_t ld_bytes, int64_t rows, int64_t cols,
                         const char* __restrict__ weight, float eps, float* __restrict__ rstd_out,
                         uint32_t* __restrict__ amax_bits) {
  __shared__ float red[kNormThreads / 32];
  __shared__ uint32_t redu[kNormThreads / 32];
  const int chunks = (int)(cols / 8);
  uint4 wq[CH];
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    wq[i] = c < chunks ? __ldg(reinterpret_cast<const uint4*>(weight) + c) : make_uint4(0u, 0u, 0u, 0u);
  }
  uint32_t amax2 = 0;  // packed unsigned max over |y| bit patterns
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint4* row = reinterpret_cast<const uint4*>(x + r * ld_bytes);
    uint4 q[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      q[i] = c < chunks ? __ldcs(row + c) : make_uint4(0u, 0u, 0u, 0u);
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      ss = sumsq_word<HP>(q[i].x, ss);
      ss = sumsq_word<HP>(q[i].y, ss);
      ss = sumsq_word<HP>(q[i].z, ss);
      ss = sumsq_word<HP>(q[i].w, ss);
    }
    const float total = block_sum_fixed(ss, red);
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)cols), eps)));
    if (threadIdx.x == 0) rstd_out[r] = rstd;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      amax2 = __vmaxu2(amax2, norm_pair<HP>(q[i].x, rstd, wq[i].x) & 0x7FFF7FFFu);
      amax2 = __vmaxu2(amax2, norm_pair<HP>(q[i].y, rstd, wq[i].y) & 0x7FFF7FFFu);
      amax2 = __vmaxu2(amax2, norm_pair<HP>(q[i].z, rstd, wq[i].z) & 0x7FFF7FFFu);
      amax2 = __vmaxu2(amax2, norm_pair<HP>(q[i].w, rstd, wq[i].w) & 0x7FFF7FFFu);
    }
  }
  // widen the larger 16-bit pattern to fp32 bits (order-preserving for |y|, NaN stays NaN)
  const uint32_t h = max(amax2 & 0xFFFFu, amax2 >> 16);
  uint32_t amax = HP == F8B200_BF16 ? (h << 16) : __float_as_uint(__half2float(__ushort_as_half((unsigned short)h)));
  amax = warp_max_u32(amax);
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  if (lane == 0) redu[wp] = amax;
  __syncthreads();
  if (wp == 0) {
    amax = lane < (kNormThreads / 32) ? redu[lane] : 0u;
    amax = warp_max_u32(amax);
    if (lane == 0 && amax > *reinterpret_cast<volatile uint32_t*>(amax_bits)) atomicMax(amax_bits, amax);
  }
}

template <int HP, int KIND, int CH>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_cast_fast_kernel(const char* __restrict__ x, int64_t ld_bytes, int64_t rows, int64_t cols,
                         const char* __restrict__ weight, const float* __restrict__ rstd_in,
                         const float* __restrict__ amax_in, float* __restrict__ scale_out,
                         uint8_t* __restrict__ out, int64_t ld_out) {
  const float scale = amax_to_scale_dev(__ldg(amax_in), fp8_max_of(KIND), HP, HP == F8B200_FP16);
  if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out != nullptr) *scale_out = scale;
  const uint32_t s2 = pack_round2<HP>(scale, scale);  // exact: the scale is a value of T
  const int chunks = (int)(cols / 8);
  uint4 wq[CH];
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    wq[i] = c < chunks ? __ldg(reinterpret_cast<const uint4*>(weight) + c) : make_uint4(0u, 0u, 0u, 0u);
  }
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint4* row = reinterpret_cast<const uint4*>(x + r * ld_bytes);
    const float rstd = __ldg(rstd_in + r);
    uint2* orow = reinterpret_cast<uint2*>(out + r * ld_out);
    uint4 q[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      q[i] = c < chunks ? __ldcs(row + c) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      if (c < chunks) {
        const uint32_t lo = pair_to_fp8<HP, KIND>(norm_pair<HP>(q[i].x, rstd, wq[i].x), s2) |
                            (pair_to_fp8<HP, KIND>(norm_pair<HP>(q[i].y, rstd, wq[i].y), s2) << 16);
        const uint32_t hi = pair_to_fp8<HP, KIND>(norm_pair<HP>(q[i].z, rstd, wq[i].z), s2) |
                            (pair_to_fp8<HP, KIND>(norm_pair<HP>(q[i].w, rstd, wq[i].w), s2) << 16);
        orow[c] = make_uint2(lo, hi);
      }
    }
  }
}

int norm_grid(int64_t rows) {
  const int64_t cap = (int64_t)sm_count() * 8;
  return (int)(rows < cap ? rows : cap);
}

}  // namespace
}  // namespace f8b200

using namespace f8b200;

extern "C" int f8b200_rmsnorm_amax(const void* x, int hp_dtype, int64_t rows, int64_t cols, int64_t ld_x,
                                   const void* weight, float eps, float* rstd_out, float* amax_out, void* stream) {
  if (x == nullptr || weight == nullptr || rstd_out == nullptr || amax_out == nullptr) return F8B200_ERR_BAD_ARG;
  if (hp_dtype < 0 || hp_dtype > 2 || rows <= 0 || cols <= 0 || ld_x < cols) return F8B200_ERR_BAD_ARG;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int es = hp_size_of(hp_dtype);
  const bool vec = es == 2 && cols % 8 == 0 && ld_x % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(weight) % 16 == 0;
  cudaError_t e = cudaMemsetAsync(amax_out, 0, sizeof(float), st);
  if (e != cudaSuccess) return record_cuda_error(e);
  const char* xp = static_cast<const char*>(x);
  const char* wp = static_cast<const char*>(weight);
  uint32_t* ab = reinterpret_cast<uint32_t*>(amax_out);
  const int grid = norm_grid(rows);
  if (vec && cols <= 4 * 2048) {
    const int64_t ldb = ld_x * es;
#define F8_FAST_A(HP, CH) \
  rmsnorm_amax_fast_kernel<HP, CH><<<grid, kNormThreads, 0, st>>>(xp, ldb, rows, cols, wp, eps, rstd_out, ab)
#define F8_FAST_A_CH(HP)                        \
  do {                                          \
    if (cols <= 2048) F8_FAST_A(HP, 1);         \
    else if (cols <= 4096) F8_FAST_A(HP, 2);    \
    else F8_FAST_A(HP, 4);                      \
  } while (0)
    if (hp_dtype == F8B200_BF16) F8_FAST_A_CH(F8B200_BF16); else F8_FAST_A_CH(F8B200_FP16);
#undef F8_FAST_A_CH
#undef F8_FAST_A
    return check_launch();
  }
#define F8_LAUNCH_A(HP, VEC) \
  rmsnorm_amax_kernel<HP, VEC><<<grid, kNormThreads, 0, st>>>(xp, ld_x * es, rows, cols, wp, eps, rstd_out, ab)
  if (hp_dtype == F8B200_BF16) {
    if (vec) F8_LAUNCH_A(F8B200_BF16, true); else F8_LAUNCH_A(F8B200_BF16, false);
  } else if (hp_dtype == F8B200_FP16) {
    if (vec) F8_LAUNCH_A(F8B200_FP16, true); else F8_LAUNCH_A(F8B200_FP16, false);
  } else {
    F8_LAUNCH_A(F8B200_FP32, false);
  }
#undef F8_LAUNCH_A
  return check_launch();
}

extern "C" int f8b200_rmsnorm_cast(const void* x, int hp_dtype, int64_t rows, int64_t cols, int64_t ld_x,
                                   const void* weight, const float* rstd, const float* amax, int fp8_kind,
                                   float* scale_out, void* out, int64_t ld_out, void* stream) {
  if (x == nullptr || weight == nullptr || rstd == nullptr || amax == nullptr || out == nullptr) return F8B200_ERR_BAD_ARG;
  if (hp_dtype < 0 || hp_dtype > 2 || fp8_kind < 0 || fp8_kind > 1) return F8B200_ERR_BAD_ARG;
  if (rows <= 0 || cols <= 0 || ld_x < cols || ld_out < cols) return F8B200_ERR_BAD_ARG;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int es = hp_size_of(hp_dtype);
  const bool vec = es == 2 && cols % 8 == 0 && ld_x % 8 == 0 && ld_out % 8 == 0 &&
                   reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(weight) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 8 == 0;
  const char* xp = static_cast<const char*>(x);
  const char* wp = static_cast<const char*>(weight);
  uint8_t* op = static_cast<uint8_t*>(out);
  const int grid = norm_grid(rows);
  if (vec && cols <= 4 * 2048) {
    const int64_t ldb = ld_x * es;
#define F8_FAST_B(HP, KIND, CH)                                                                                   \
  rmsnorm_cast_fast_kernel<HP, KIND, CH><<<grid, kNormThreads, 0, st>>>(xp, ldb, rows, cols, wp, rstd, amax, \
                                                                         scale_out, op, ld_out)
#define F8_FAST_B_CH(HP, KIND)                      \
  do {                                              \
    if (cols <= 2048) F8_FAST_B(HP, KIND, 1);       \
    else if (cols <= 4096) F8_FAST_B(HP, KIND, 2);  \
    else F8_FAST_B(HP, KIND, 4);                    \
  } while (0)
    if (hp_dtype == F8B200_BF16) {
      if (fp8_kind == F8B200_E4M3) F8_FAST_B_CH(F8B200_BF16, F8B200_E4M3); else F8_FAST_B_CH(F8B200_BF16, F8B200_E5M2);
    } else {
      if (fp8_kind == F8B200_E4M3) F8_FAST_B_CH(F8B200_FP16, F8B200_E4M3); else F8_FAST_B_CH(F8B200_FP16, F8B200_E5M2);
    }
#undef F8_FAST_B_CH
#undef F8_FAST_B
    return check_launch();
  }
#define F8_LAUNCH_B(HP, KIND, VEC)                                                                                 \
  rmsnorm_cast_kernel<HP, KIND, VEC><<<grid, kNormThreads, 0, st>>>(xp, ld_x * es, rows, cols, wp, rstd, amax, \
                                                                     scale_out, op, ld_out)
#define F8_DISPATCH_B(HP, VEC)                                     \
  do {                                                             \
    if (fp8_kind == F8B200_E4M3) F8_LAUNCH_B(HP, F8B200_E4M3, VEC); \
    else F8_LAUNCH_B(HP, F8B200_E5M2, VEC);                         \
  } while (0)
  if (hp_dtype == F8B200_BF16) {
    if (vec) F8_DISPATCH_B(F8B200_BF16, true); else F8_DISPATCH_B(F8B200_BF16, false);
  } else if (hp_dtype == F8B200_FP16) {
    if (vec) F8_DISPATCH_B(F8B200_FP16, true); else F8_DISPATCH_B(F8B200_FP16, false);
  } else {
    F8_DISPATCH_B(F8B200_FP32, false);
  }
#undef F8_DISPATCH_B
#undef F8_LAUNCH_B
  return check_launch();
}

// ===========================================================================
// SwiGLU gate fused into the dynamic fp8 cast of its output: y = RN_T(RN_T(silu(a)) * b),
// silu(a) = a / (1 + exp(-a)) in fp32, which is `F.silu(self.w1(x)) * self.w3(x)` of
// float8_experimental/benchmarks/profile_linear_float8.py:117-118, the producer of the input of
// the w2 linear.  Unfused: silu 2 + 2, multiply 2 + 2 + 2, cast 2 + 2 + 1 = 17 bytes per element.
// Here pass A reads a and b for the amax of y (4) and pass B either reads them again and writes fp8
// (4 + 1; y is never written) or, when pass A was also asked to write y (4 + 2), is the plain cast of
// y (2 + 1): 9 bytes per element both ways.  exp and an IEEE division per element make the gate
// issue-bound rather than memory-bound, so evaluating it once (the second form) is the faster one.
// ===========================================================================
namespace f8b200 {
namespace {

__device__ __forceinline__ float silu_f32(float a) { return __fdiv_rn(a, __fadd_rn(1.0f, expf(-a))); }

// Opt-in approximate gate (the `_approx` entry points): sigmoid from ex2.approx and rcp.approx (about 2^-21
// relative error in fp32 instead of correctly rounded division and a 1-ulp exp), then the same roundings to T.
// The error is far below half an ulp of a 16-bit T, so silu(a) rounds to the same T value except where the
// exact result lies within ~2^-12 of an ulp of a rounding boundary; there it is the neighbouring T value.
__device__ __forceinline__ float sigmoid_approx(float a) { return __fdividef(1.0f, 1.0f + __expf(-a)); }

template <int HP, bool APPROX = false>
__device__ __forceinline__ uint32_t swiglu_pair(uint32_t a2, uint32_t b2) {
  float a0, a1;
  unpack_pair<HP>(a2, a0, a1);
  if constexpr (APPROX) return mul2<HP>(pack_round2<HP>(a0 * sigmoid_approx(a0), a1 * sigmoid_approx(a1)), b2);
  return mul2<HP>(pack_round2<HP>(silu_f32(a0), silu_f32(a1)), b2);
}

template <int HP>
__device__ __forceinline__ float swiglu_value(float a, float b) {
  return round_hp<HP>(__fmul_rn(round_hp<HP>(silu_f32(a)), b));
}

constexpr int kGluThreads = 256;

// 16-bit dtypes, 8 elements per thread and step; rows x cols with separate row pitches for a and b
// (the two halves of one fused w1|w3 output are the usual case).
template <int HP, bool WRITE_Y, bool APPROX = false>
__global__ void __launch_bounds__(kGluThreads)
swiglu_amax_fast_kernel(const char* __restrict__ a, const char* __restrict__ b, int64_t lda_bytes, int64_t ldb_bytes,
                        int64_t rows, int64_t chunks_per_row, uint32_t* __restrict__ amax_bits,
                        char* __restrict__ y_out, int64_t ldy_bytes) {
  __shared__ uint32_t redu[kGluThreads / 32];
  const int64_t total = rows * chunks_per_row;
  uint32_t amax2 = 0;
  for (int64_t i = (int64_t)blockIdx.x * kGluThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kGluThreads) {
    const int64_t r = i / chunks_per_row, c = i - r * chunks_per_row;
    const uint4 qa = __ldcs(reinterpret_cast<const uint4*>(a + r * lda_bytes) + c);
    const uint4 qb = __ldcs(reinterpret_cast<const uint4*>(b + r * ldb_bytes) + c);
    uint4 y;
    y.x = swiglu_pair<HP, APPROX>(qa.x, qb.x);
    y.y = swiglu_pair<HP, APPROX>(qa.y, qb.y);
    y.z = swiglu_pair<HP, APPROX>(qa.z, qb.z);
    y.w = swiglu_pair<HP, APPROX>(qa.w, qb.w);
    amax2 = __vmaxu2(amax2, y.x & 0x7FFF7FFFu);
    amax2 = __vmaxu2(amax2, y.y & 0x7FFF7FFFu);
    amax2 = __vmaxu2(amax2, y.z & 0x7FFF7FFFu);
    amax2 = __vmaxu2(amax2, y.w & 0x7FFF7FFFu);
    if constexpr (WRITE_Y) reinterpret_cast<uint4*>(y_out + r * ldy_bytes)[c] = y;
  }
  const uint32_t h = max(amax2 & 0xFFFFu, amax2 >> 16);
  uint32_t amax = HP == F8B200_BF16 ? (h << 16) : __float_as_uint(__half2float(__ushort_as_half((unsigned short)h)));
  amax = warp_max_u32(amax);
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  if (lane == 0) redu[wp] = amax;
  __syncthreads();
  if (wp == 0) {
    amax = lane < (kGluThreads / 32) ? redu[lane] : 0u;
    amax = warp_max_u32(amax);
    if (lane == 0 && amax > *reinterpret_cast<volatile uint32_t*>(amax_bits)) atomicMax(amax_bits, amax);
  }
}

template <int HP, int KIND>
__global__ void __launch_bounds__(kGluThreads)
swiglu_cast_fast_kernel(const char* __restrict__ a, const char* __restrict__ b, int64_t lda_bytes, int64_t ldb_bytes,
                        int64_t rows, int64_t chunks_per_row, const float* __restrict__ amax_in,
                        float* __restrict__ scale_out, uint8_t* __restrict__ out, int64_t ld_out) {
  const float scale = amax_to_scale_dev(__ldg(amax_in), fp8_max_of(KIND), HP, HP == F8B200_FP16);
  if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out != nullptr) *scale_out = scale;
  const uint32_t s2 = pack_round2<HP>(scale, scale);
  const int64_t total = rows * chunks_per_row;
  for (int64_t i = (int64_t)blockIdx.x * kGluThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kGluThreads) {
    const int64_t r = i / chunks_per_row, c = i - r * chunks_per_row;
    const uint4 qa = __ldcs(reinterpret_cast<const uint4*>(a + r * lda_bytes) + c);
    const uint4 qb = __ldcs(reinterpret_cast<const uint4*>(b + r * ldb_bytes) + c);
    const uint32_t lo = pair_to_fp8<HP, KIND>(swiglu_pair<HP>(qa.x, qb.x), s2) |
                        (pair_to_fp8<HP, KIND>(swiglu_pair<HP>(qa.y, qb.y), s2) << 16);
    const uint32_t hi = pair_to_fp8<HP, KIND>(swiglu_pair<HP>(qa.z, qb.z), s2) |
                        (pair_to_fp8<HP, KIND>(swiglu_pair<HP>(qa.w, qb.w), s2) << 16);
    reinterpret_cast<uint2*>(out + r * ld_out)[c] = make_uint2(lo, hi);
  }
}

// Any dtype, shape and alignment: one element per thread and step.
template <int HP>
__device__ __forceinline__ void store_hp(void* base, int64_t i, float v) {
  if constexpr (HP == F8B200_BF16) {
    reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(v);
  } else if constexpr (HP == F8B200_FP16) {
    reinterpret_cast<__half*>(base)[i] = __float2half_rn(v);
  } else {
    reinterpret_cast<float*>(base)[i] = v;
  }
}

template <int HP>
__global__ void __launch_bounds__(kGluThreads)
swiglu_amax_generic_kernel(const char* __restrict__ a, const char* __restrict__ b, int64_t lda, int64_t ldb,
                           int64_t rows, int64_t cols, uint32_t* __restrict__ amax_bits, char* __restrict__ y_out,
                           int64_t ldy) {
  __shared__ uint32_t redu[kGluThreads / 32];
  const int64_t total = rows * cols;
  uint32_t amax = 0;
  for (int64_t i = (int64_t)blockIdx.x * kGluThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kGluThreads) {
    const int64_t r = i / cols, c = i - r * cols;
    const float y = swiglu_value<HP>(load_hp<HP>(a, r * lda + c), load_hp<HP>(b, r * ldb + c));
    amax = max(amax, abs_bits(y));
    if (y_out != nullptr) store_hp<HP>(y_out, r * ldy + c, y);  // y is a value of T: the store is exact
  }
  amax = warp_max_u32(amax);
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  if (lane == 0) redu[wp] = amax;
  __syncthreads();
  if (wp == 0) {
    amax = lane < (kGluThreads / 32) ? redu[lane] : 0u;
    amax = warp_max_u32(amax);
    if (lane == 0 && amax > *reinterpret_cast<volatile uint32_t*>(amax_bits)) atomicMax(amax_bits, amax);
  }
}

template <int HP, int KIND>
__global__ void __launch_bounds__(kGluThreads)
swiglu_cast_generic_kernel(const char* __restrict__ a, const char* __restrict__ b, int64_t lda, int64_t ldb,
                           int64_t rows, int64_t cols, const float* __restrict__ amax_in,
                           float* __restrict__ scale_out, uint8_t* __restrict__ out, int64_t ld_out) {
  const float scale = amax_to_scale_dev(__ldg(amax_in), fp8_max_of(KIND), HP, HP == F8B200_FP16);
  if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out != nullptr) *scale_out = scale;
  const int64_t total = rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * kGluThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kGluThreads) {
    const int64_t r = i / cols, c = i - r * cols;
    const float q = __fmul_rn(swiglu_value<HP>(load_hp<HP>(a, r * lda + c), load_hp<HP>(b, r * ldb + c)), scale);
    out[r * ld_out + c] = (uint8_t)(cast4<HP, KIND>(q, 0.f, 0.f, 0.f, HP != F8B200_FP32) & 0xFFu);
  }
}

int glu_grid(int64_t work_items) {
  const int64_t need = (work_items + kGluThreads - 1) / kGluThreads;
  const int64_t cap = (int64_t)sm_count() * 8;
  return (int)(need < cap ? (need < 1 ? 1 : need) : cap);
}

bool glu_vec_ok(int hp_dtype, int64_t cols, int64_t lda, int64_t ldb, const void* a, const void* b) {
  return hp_size_of(hp_dtype) == 2 && cols % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0 &&
         reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0;
}

}  // namespace
}  // namespace f8b200

static int swiglu_amax_impl(const void* a, const void* b, int hp_dtype, int64_t rows, int64_t cols, int64_t ld_a,
                            int64_t ld_b, void* y_out, int64_t ld_y, float* amax_out, void* stream, bool approx) {
  using namespace f8b200;
  if (a == nullptr || b == nullptr || amax_out == nullptr) return F8B200_ERR_BAD_ARG;
  if (hp_dtype < 0 || hp_dtype > 2 || rows <= 0 || cols <= 0 || ld_a < cols || ld_b < cols) return F8B200_ERR_BAD_ARG;
  if (y_out != nullptr && ld_y < cols) return F8B200_ERR_BAD_ARG;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(amax_out, 0, sizeof(float), st);
  if (e != cudaSuccess) return record_cuda_error(e);
  const char* ap = static_cast<const char*>(a);
  const char* bp = static_cast<const char*>(b);
  char* yp = static_cast<char*>(y_out);
  uint32_t* ab = reinterpret_cast<uint32_t*>(amax_out);
  const bool y_vec = y_out == nullptr || (ld_y % 8 == 0 && reinterpret_cast<uintptr_t>(y_out) % 16 == 0);
  const bool vec = glu_vec_ok(hp_dtype, cols, ld_a, ld_b, a, b) && y_vec;
  if (approx && !vec) return F8B200_ERR_UNSUPPORTED;  // only the vectorised 16-bit kernels have the approximate gate
  if (vec) {
    const int64_t cpr = cols / 8;
    const int grid = glu_grid(rows * cpr);
#define F8_GLU_A(HP, WY, AX) \
  swiglu_amax_fast_kernel<HP, WY, AX><<<grid, kGluThreads, 0, st>>>(ap, bp, ld_a * 2, ld_b * 2, rows, cpr, ab, yp, ld_y * 2)
#define F8_GLU_A2(HP, WY) do { if (approx) F8_GLU_A(HP, WY, true); else F8_GLU_A(HP, WY, false); } while (0)
    if (hp_dtype == F8B200_BF16) {
      if (y_out != nullptr) F8_GLU_A2(F8B200_BF16, true); else F8_GLU_A2(F8B200_BF16, false);
    } else {
      if (y_out != nullptr) F8_GLU_A2(F8B200_FP16, true); else F8_GLU_A2(F8B200_FP16, false);
    }
#undef F8_GLU_A2
#undef F8_GLU_A
    return check_launch();
  }
  const int grid = glu_grid(rows * cols);
  if (hp_dtype == F8B200_BF16)
    swiglu_amax_generic_kernel<F8B200_BF16><<<grid, kGluThreads, 0, st>>>(ap, bp, ld_a, ld_b, rows, cols, ab, yp, ld_y);
  else if (hp_dtype == F8B200_FP16)
    swiglu_amax_generic_kernel<F8B200_FP16><<<grid, kGluThreads, 0, st>>>(ap, bp, ld_a, ld_b, rows, cols, ab, yp, ld_y);
  else
    swiglu_amax_generic_kernel<F8B200_FP32><<<grid, kGluThreads, 0, st>>>(ap, bp, ld_a, ld_b, rows, cols, ab, yp, ld_y);
  return check_launch();
}

extern "C" int f8b200_swiglu_amax(const void* a, const void* b, int hp_dtype, int64_t rows, int64_t cols, int64_t ld_a,
                                  int64_t ld_b, void* y_out, int64_t ld_y, float* amax_out, void* stream) {
  return swiglu_amax_impl(a, b, hp_dtype, rows, cols, ld_a, ld_b, y_out, ld_y, amax_out, stream, false);
}

extern "C" int f8b200_swiglu_amax_approx(const void* a, const void* b, int hp_dtype, int64_t rows, int64_t cols,
                                         int64_t ld_a, int64_t ld_b, void* y_out, int64_t ld_y, float* amax_out,
                                         void* stream) {
  return swiglu_amax_impl(a, b, hp_dtype, rows, cols, ld_a, ld_b, y_out, ld_y, amax_out, stream, true);
}

extern "C" int f8b200_swiglu_cast(const void* a, const void* b, int hp_dtype, int64_t rows, int64_t cols, int64_t ld_a,
                                  int64_t ld_b, const float* amax, int fp8_kind, float* scale_out, void* out,
                                  int64_t ld_out, void* stream) {
  if (a == nullptr || b == nullptr || amax == nullptr || out == nullptr) return F8B200_ERR_BAD_ARG;
  if (hp_dtype < 0 || hp_dtype > 2 || fp8_kind < 0 || fp8_kind > 1) return F8B200_ERR_BAD_ARG;
  if (rows <= 0 || cols <= 0 || ld_a < cols || ld_b < cols || ld_out < cols) return F8B200_ERR_BAD_ARG;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const char* ap = static_cast<const char*>(a);
  const char* bp = static_cast<const char*>(b);
  uint8_t* op = static_cast<uint8_t*>(out);
  if (glu_vec_ok(hp_dtype, cols, ld_a, ld_b, a, b) && ld_out % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0) {
    const int64_t cpr = cols / 8;
    const int grid = glu_grid(rows * cpr);
#define F8_GLU_FAST(HP, KIND)                                                                                    \
  swiglu_cast_fast_kernel<HP, KIND><<<grid, kGluThreads, 0, st>>>(ap, bp, ld_a * 2, ld_b * 2, rows, cpr, amax, \
                                                                   scale_out, op, ld_out)
    if (hp_dtype == F8B200_BF16) {
      if (fp8_kind == F8B200_E4M3) F8_GLU_FAST(F8B200_BF16, F8B200_E4M3); else F8_GLU_FAST(F8B200_BF16, F8B200_E5M2);
    } else {
      if (fp8_kind == F8B200_E4M3) F8_GLU_FAST(F8B200_FP16, F8B200_E4M3); else F8_GLU_FAST(F8B200_FP16, F8B200_E5M2);
    }
#undef F8_GLU_FAST
    return check_launch();
  }
  const int grid = glu_grid(rows * cols);
#define F8_GLU_GEN(HP, KIND)                                                                                  \
  swiglu_cast_generic_kernel<HP, KIND><<<grid, kGluThreads, 0, st>>>(ap, bp, ld_a, ld_b, rows, cols, amax, \
                                                                      scale_out, op, ld_out)
#define F8_GLU_GEN_K(HP)                                              \
  do {                                                                \
    if (fp8_kind == F8B200_E4M3) F8_GLU_GEN(HP, F8B200_E4M3);         \
    else F8_GLU_GEN(HP, F8B200_E5M2);                                 \
  } while (0)
  if (hp_dtype == F8B200_BF16) F8_GLU_GEN_K(F8B200_BF16);
  else if (hp_dtype == F8B200_FP16) F8_GLU_GEN_K(F8B200_FP16);
  else F8_GLU_GEN_K(F8B200_FP32);
#undef F8_GLU_GEN_K
#undef F8_GLU_GEN
  return check_launch();
}

// ===========================================================================
// Backward of the two fused producers (the casts are transparent to autograd, so these are the
// plain RMSNorm and SwiGLU backward formulas), one pass over the saved inputs each.
//
// RMSNorm:  n = x * rstd,  dn = RN_T(g * w),  c = mean(dn * n) over the row,
//           dx = RN_T(rstd * (dn - n * c)),   dw[col] = sum over rows of g * RN_T(n)
//           (the gradient of `output * weight` and of `_norm` in
//           float8_experimental/benchmarks/profile_linear_float8.py:69-74).  Reads x and g, writes
//           dx: 6 bytes per element; dw is accumulated per CTA in registers and written as
//           per-CTA partial sums that a second small kernel adds up.
// SwiGLU:   s = a * sig(a),  ds = RN_T(g * b),  da = RN_T(ds * sig * (1 + a * (1 - sig))),
//           db = RN_T(g * RN_T(s)).  Reads a, b, g, writes da, db: 10 bytes per element.
// ===========================================================================
namespace f8b200 {
namespace {

template <int HP, int CH>
__global__ void __launch_bounds__(kNormThreads, 2)
rmsnorm_bwd_kernel(const char* __restrict__ x, int64_t ldx_bytes, const char* __restrict__ g, int64_t ldg_bytes,
                   int64_t rows, int64_t cols, const char* __restrict__ weight, const float* __restrict__ rstd_in,
                   char* __restrict__ dx, int64_t lddx_bytes, float* __restrict__ dw_partial) {
  __shared__ float red[kNormThreads / 32];
  const int chunks = (int)(cols / 8);
  // The weight row (at most 16 KB) is re-read from L1 for every row instead of being held in registers:
  // with the packed rows of x and g (2 x CH x 4 registers) and the CH x 8 dw accumulators that keeps the
  // 8192-column instantiation inside the 128 registers two CTAs per SM allow (it used to spill).
  const uint4* wrow = reinterpret_cast<const uint4*>(weight);
  float dw[CH][8];
#pragma unroll
  for (int i = 0; i < CH; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[i][j] = 0.0f;
  }
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint4* xrow = reinterpret_cast<const uint4*>(x + r * ldx_bytes);
    const uint4* grow = reinterpret_cast<const uint4*>(g + r * ldg_bytes);
    const float rstd = __ldg(rstd_in + r);
    // the row of x and of g stays packed in registers; n and dn are recomputed in the second sweep
    uint4 qx[CH], qg[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      qx[i] = c < chunks ? __ldcs(xrow + c) : make_uint4(0u, 0u, 0u, 0u);
      qg[i] = c < chunks ? __ldcs(grow + c) : make_uint4(0u, 0u, 0u, 0u);
    }
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      float xv[8], gv[8], wv[8];
      widen8<HP>(qx[i], xv);
      widen8<HP>(qg[i], gv);
      widen8<HP>(c < chunks ? __ldg(wrow + c) : make_uint4(0u, 0u, 0u, 0u), wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float n = xv[j] * rstd;
        dot = fmaf(round_hp<HP>(gv[j] * wv[j]), n, dot);
        dw[i][j] = fmaf(gv[j], round_hp<HP>(n), dw[i][j]);
      }
    }
    const float cmean = block_sum_fixed(dot, red) / (float)cols;
    uint4* orow = reinterpret_cast<uint4*>(dx + r * lddx_bytes);
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      if (c < chunks) {
        float xv[8], gv[8], wv[8], o[8];
        widen8<HP>(qx[i], xv);
        widen8<HP>(qg[i], gv);
        widen8<HP>(__ldg(wrow + c), wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (round_hp<HP>(gv[j] * wv[j]) - xv[j] * rstd * cmean);
        orow[c] = make_uint4(pack_round2<HP>(o[0], o[1]), pack_round2<HP>(o[2], o[3]), pack_round2<HP>(o[4], o[5]),
                             pack_round2<HP>(o[6], o[7]));
      }
    }
  }
  float* mine = dw_partial + (int64_t)blockIdx.x * cols;
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    if (c < chunks) {
      reinterpret_cast<float4*>(mine + (int64_t)c * 8)[0] = make_float4(dw[i][0], dw[i][1], dw[i][2], dw[i][3]);
      reinterpret_cast<float4*>(mine + (int64_t)c * 8)[1] = make_float4(dw[i][4], dw[i][5], dw[i][6], dw[i][7]);
    }
  }
}

// dw[col] = sum of the per-CTA partial sums, rounded to T.  One CTA per 32 columns; its eight
// warps take every eighth partial row, shared memory adds the eight sums.
template <int HP>
__global__ void __launch_bounds__(256)
rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, int parts, int64_t cols, char* __restrict__ dw_out) {
  __shared__ float acc[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c = (int64_t)blockIdx.x * 32 + tx;
  float s = 0.0f;
  if (c < cols)
    for (int p = ty; p < parts; p += 8) s += partial[(int64_t)p * cols + c];
  acc[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < cols) {
    float t = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += acc[k][tx];
    store_hp<HP>(dw_out, c, t);
  }
}

template <int HP, bool APPROX = false>
__global__ void __launch_bounds__(kGluThreads)
swiglu_bwd_kernel(const char* __restrict__ a, const char* __restrict__ b, const char* __restrict__ g, int64_t lda_bytes,
                  int64_t ldb_bytes, int64_t ldg_bytes, int64_t rows, int64_t chunks_per_row, char* __restrict__ da,
                  char* __restrict__ db, int64_t ldo_bytes) {
  const int64_t total = rows * chunks_per_row;
  for (int64_t i = (int64_t)blockIdx.x * kGluThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kGluThreads) {
    const int64_t r = i / chunks_per_row, c = i - r * chunks_per_row;
    float av[8], bv[8], gv[8], dav[8], dbv[8];
    widen8<HP>(__ldcs(reinterpret_cast<const uint4*>(a + r * lda_bytes) + c), av);
    widen8<HP>(__ldcs(reinterpret_cast<const uint4*>(b + r * ldb_bytes) + c), bv);
    widen8<HP>(__ldcs(reinterpret_cast<const uint4*>(g + r * ldg_bytes) + c), gv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sig = APPROX ? sigmoid_approx(av[j]) : __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-av[j])));
      const float ds = round_hp<HP>(gv[j] * bv[j]);
      dav[j] = ds * (sig * (1.0f + av[j] * (1.0f - sig)));
      dbv[j] = gv[j] * round_hp<HP>(APPROX ? av[j] * sig : silu_f32(av[j]));
    }
    uint4 oa, ob;
    oa.x = pack_round2<HP>(dav[0], dav[1]); oa.y = pack_round2<HP>(dav[2], dav[3]);
    oa.z = pack_round2<HP>(dav[4], dav[5]); oa.w = pack_round2<HP>(dav[6], dav[7]);
    ob.x = pack_round2<HP>(dbv[0], dbv[1]); ob.y = pack_round2<HP>(dbv[2], dbv[3]);
    ob.z = pack_round2<HP>(dbv[4], dbv[5]); ob.w = pack_round2<HP>(dbv[6], dbv[7]);
    reinterpret_cast<uint4*>(da + r * ldo_bytes)[c] = oa;
    reinterpret_cast<uint4*>(db + r * ldo_bytes)[c] = ob;
  }
}

// Generic variants (any column count, fp32 as well as the 16-bit types, any row pitch): one CTA per
// row, the row is read twice (the second sweep hits L2), dw goes through the same per-CTA partial
// sums (each CTA owns one row of `dw_partial`, which it zeroes first).  Same formulas and roundings.
template <int HP>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_generic_kernel(const char* __restrict__ x, int64_t ldx, const char* __restrict__ g, int64_t ldg, int64_t rows,
                           int64_t cols, const char* __restrict__ weight, const float* __restrict__ rstd_in,
                           char* __restrict__ dx, int64_t lddx, float* __restrict__ dw_partial) {
  __shared__ float red[kNormThreads / 32];
  constexpr int ESZ = HP == F8B200_FP32 ? 4 : 2;
  float* mine = dw_partial + (int64_t)blockIdx.x * cols;
  for (int64_t c = threadIdx.x; c < cols; c += kNormThreads) mine[c] = 0.0f;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const char* xrow = x + r * ldx * ESZ;
    const char* grow = g + r * ldg * ESZ;
    const float rstd = __ldg(rstd_in + r);
    float dot = 0.0f;
    for (int64_t c = threadIdx.x; c < cols; c += kNormThreads) {  // each thread owns its columns: no race on `mine`
      const float xv = load_hp<HP>(xrow, c), gv = load_hp<HP>(grow, c), wv = load_hp<HP>(weight, c);
      const float n = xv * rstd;
      dot = fmaf(round_hp<HP>(gv * wv), n, dot);
      mine[c] = fmaf(gv, round_hp<HP>(n), mine[c]);
    }
    const float cmean = block_sum_fixed(dot, red) / (float)cols;
    char* orow = dx + r * lddx * ESZ;
    for (int64_t c = threadIdx.x; c < cols; c += kNormThreads) {
      const float xv = load_hp<HP>(xrow, c), gv = load_hp<HP>(grow, c), wv = load_hp<HP>(weight, c);
      store_hp<HP>(orow, c, rstd * (round_hp<HP>(gv * wv) - xv * rstd * cmean));
    }
  }
}

template <int HP>
__global__ void __launch_bounds__(kGluThreads)
swiglu_bwd_generic_kernel(const char* __restrict__ a, const char* __restrict__ b, const char* __restrict__ g, int64_t lda,
                          int64_t ldb, int64_t ldg, int64_t rows, int64_t cols, char* __restrict__ da,
                          char* __restrict__ db, int64_t ldo) {
  constexpr int ESZ = HP == F8B200_FP32 ? 4 : 2;
  const int64_t total = rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * kGluThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kGluThreads) {
    const int64_t r = i / cols, c = i - r * cols;
    const float av = load_hp<HP>(a + r * lda * ESZ, c), bv = load_hp<HP>(b + r * ldb * ESZ, c);
    const float gv = load_hp<HP>(g + r * ldg * ESZ, c);
    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-av)));
    const float ds = round_hp<HP>(gv * bv);
    store_hp<HP>(da + r * ldo * ESZ, c, ds * (sig * (1.0f + av * (1.0f - sig))));
    store_hp<HP>(db + r * ldo * ESZ, c, gv * round_hp<HP>(silu_f32(av)));
  }
}

}  // namespace
}  // namespace f8b200

// The fast kernels cover 16-bit dtypes, cols a multiple of 8 (RMSNorm: at most 8192) and 16-byte
// aligned rows; every other shape or dtype runs on the generic kernels above.  `workspace` holds the
// per-CTA partial sums of dw: f8b200_rmsnorm_bwd_workspace_bytes(cols) bytes of device memory, fp32.
static int norm_bwd_grid(int64_t rows) {
  const int64_t cap = (int64_t)sm_count() * 2;  // two CTAs of the backward kernel fit an SM
  return (int)(rows < cap ? rows : cap);
}

extern "C" int64_t f8b200_rmsnorm_bwd_workspace_bytes(int64_t cols) {
  return (int64_t)sm_count() * 2 * cols * (int64_t)sizeof(float);
}

extern "C" int f8b200_rmsnorm_bwd(const void* x, const void* grad_y, int hp_dtype, int64_t rows, int64_t cols,
                                  int64_t ld_x, int64_t ld_g, const void* weight, const float* rstd, void* dx,
                                  int64_t ld_dx, void* dweight, void* workspace, int64_t workspace_bytes,
                                  void* stream) {
  if (x == nullptr || grad_y == nullptr || weight == nullptr || rstd == nullptr || dx == nullptr ||
      dweight == nullptr || workspace == nullptr)
    return F8B200_ERR_BAD_ARG;
  if (rows <= 0 || cols <= 0 || ld_x < cols || ld_g < cols || ld_dx < cols) return F8B200_ERR_BAD_ARG;
  if (hp_dtype < 0 || hp_dtype > 2) return F8B200_ERR_BAD_ARG;
  auto al16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool fast = hp_dtype != F8B200_FP32 && cols % 8 == 0 && cols <= 8192 && ld_x % 8 == 0 && ld_g % 8 == 0 &&
                    ld_dx % 8 == 0 && al16(x) && al16(grad_y) && al16(weight) && al16(dx) && al16(workspace);
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  const int grid = norm_bwd_grid(rows);
  if (workspace_bytes < (int64_t)grid * cols * (int64_t)sizeof(float)) return F8B200_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const char* xp = static_cast<const char*>(x);
  const char* gp = static_cast<const char*>(grad_y);
  const char* wp = static_cast<const char*>(weight);
  char* dxp = static_cast<char*>(dx);
  float* part = static_cast<float*>(workspace);
  const unsigned blocks = (unsigned)((cols + 31) / 32);
  if (!fast) {
#define F8_RMS_BWD_GEN(HP)                                                                                         \
  do {                                                                                                             \
    rmsnorm_bwd_generic_kernel<HP><<<grid, kNormThreads, 0, st>>>(xp, ld_x, gp, ld_g, rows, cols, wp, rstd, dxp,   \
                                                                  ld_dx, part);                                    \
    rc = check_launch();                                                                                           \
    if (rc != F8B200_OK) return rc;                                                                                \
    rmsnorm_dw_reduce_kernel<HP><<<blocks, 256, 0, st>>>(part, grid, cols, static_cast<char*>(dweight));           \
  } while (0)
    if (hp_dtype == F8B200_BF16) F8_RMS_BWD_GEN(F8B200_BF16);
    else if (hp_dtype == F8B200_FP16) F8_RMS_BWD_GEN(F8B200_FP16);
    else F8_RMS_BWD_GEN(F8B200_FP32);
#undef F8_RMS_BWD_GEN
    return check_launch();
  }
#define F8_RMS_BWD(HP, CH)                                                                                        \
  rmsnorm_bwd_kernel<HP, CH><<<grid, kNormThreads, 0, st>>>(xp, ld_x * 2, gp, ld_g * 2, rows, cols, wp, rstd, dxp, \
                                                            ld_dx * 2, part)
#define F8_RMS_BWD_CH(HP)                    \
  do {                                       \
    if (cols <= 2048) F8_RMS_BWD(HP, 1);     \
    else if (cols <= 4096) F8_RMS_BWD(HP, 2); \
    else F8_RMS_BWD(HP, 4);                  \
  } while (0)
  if (hp_dtype == F8B200_BF16) F8_RMS_BWD_CH(F8B200_BF16); else F8_RMS_BWD_CH(F8B200_FP16);
#undef F8_RMS_BWD_CH
#undef F8_RMS_BWD
  rc = check_launch();
  if (rc != F8B200_OK) return rc;
  if (hp_dtype == F8B200_BF16)
    rmsnorm_dw_reduce_kernel<F8B200_BF16><<<blocks, 256, 0, st>>>(part, grid, cols, static_cast<char*>(dweight));
  else
    rmsnorm_dw_reduce_kernel<F8B200_FP16><<<blocks, 256, 0, st>>>(part, grid, cols, static_cast<char*>(dweight));
  return check_launch();
}

static int swiglu_bwd_impl(const void* a, const void* b, const void* grad_y, int hp_dtype, int64_t rows, int64_t cols,
                           int64_t ld_a, int64_t ld_b, int64_t ld_g, void* da, void* db, int64_t ld_out, void* stream,
                           bool approx) {
  using namespace f8b200;
  if (a == nullptr || b == nullptr || grad_y == nullptr || da == nullptr || db == nullptr) return F8B200_ERR_BAD_ARG;
  if (rows <= 0 || cols <= 0 || ld_a < cols || ld_b < cols || ld_g < cols || ld_out < cols) return F8B200_ERR_BAD_ARG;
  if (hp_dtype < 0 || hp_dtype > 2) return F8B200_ERR_BAD_ARG;
  auto al16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool fast = hp_dtype != F8B200_FP32 && cols % 8 == 0 && ld_a % 8 == 0 && ld_b % 8 == 0 && ld_g % 8 == 0 &&
                    ld_out % 8 == 0 && al16(a) && al16(b) && al16(grad_y) && al16(da) && al16(db);
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (approx && !fast) return F8B200_ERR_UNSUPPORTED;  // only the vectorised 16-bit kernel has the approximate gate
  if (!fast) {
    const int ggrid = glu_grid(rows * cols);
#define F8_GLU_BWD_GEN(HP)                                                                                             \
  swiglu_bwd_generic_kernel<HP><<<ggrid, kGluThreads, 0, st>>>(                                                        \
      static_cast<const char*>(a), static_cast<const char*>(b), static_cast<const char*>(grad_y), ld_a, ld_b, ld_g, rows, \
      cols, static_cast<char*>(da), static_cast<char*>(db), ld_out)
    if (hp_dtype == F8B200_BF16) F8_GLU_BWD_GEN(F8B200_BF16);
    else if (hp_dtype == F8B200_FP16) F8_GLU_BWD_GEN(F8B200_FP16);
    else F8_GLU_BWD_GEN(F8B200_FP32);
#undef F8_GLU_BWD_GEN
    return check_launch();
  }
  const int64_t cpr = cols / 8;
  const int grid = glu_grid(rows * cpr);
#define F8_GLU_BWD(HP, AX)                                                                                             \
  swiglu_bwd_kernel<HP, AX><<<grid, kGluThreads, 0, st>>>(                                                             \
      static_cast<const char*>(a), static_cast<const char*>(b), static_cast<const char*>(grad_y), ld_a * 2, ld_b * 2, \
      ld_g * 2, rows, cpr, static_cast<char*>(da), static_cast<char*>(db), ld_out * 2)
  if (hp_dtype == F8B200_BF16) {
    if (approx) F8_GLU_BWD(F8B200_BF16, true); else F8_GLU_BWD(F8B200_BF16, false);
  } else {
    if (approx) F8_GLU_BWD(F8B200_FP16, true); else F8_GLU_BWD(F8B200_FP16, false);
  }
#undef F8_GLU_BWD
  return check_launch();
}

extern "C" int f8b200_swiglu_bwd(const void* a, const void* b, const void* grad_y, int hp_dtype, int64_t rows,
                                 int64_t cols, int64_t ld_a, int64_t ld_b, int64_t ld_g, void* da, void* db,
                                 int64_t ld_out, void* stream) {
  return swiglu_bwd_impl(a, b, grad_y, hp_dtype, rows, cols, ld_a, ld_b, ld_g, da, db, ld_out, stream, false);
}

extern "C" int f8b200_swiglu_bwd_approx(const void* a, const void* b, const void* grad_y, int hp_dtype, int64_t rows,
                                        int64_t cols, int64_t ld_a, int64_t ld_b, int64_t ld_g, void* da, void* db,
                                        int64_t ld_out, void* stream) {
  return swiglu_bwd_impl(a, b, grad_y, hp_dtype, rows, cols, ld_a, ld_b, ld_g, da, db, ld_out, stream, true);
}
