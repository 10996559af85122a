// Shared device/host helpers for the sm_100a float8 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/f8b200.h"

namespace f8b200 {

constexpr float kE4M3Max = 448.0f;
constexpr float kE5M2Max = 57344.0f;
constexpr float kFp16Max = 65504.0f;
constexpr float kEps = 1e-12f;  // float8_experimental/float8_utils.py:19

// Remembers the last CUDA error text for f8b200_last_cuda_error().
int record_cuda_error(cudaError_t e);
int sm_count();  // SM count of the current device

// One-time set-up that has to run once on EVERY device of the process (function attributes such as
// the dynamic shared-memory opt-in are per device).  run() calls `fn` the first time the current
// device asks and remembers only a success: a failed attempt is tried again by the next call.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
  unsigned char done[kMaxDevices] = {};
  int value[kMaxDevices] = {};  // a number the set-up computed for the device (e.g. an occupancy)
  template <typename Fn>
  cudaError_t run(Fn&& fn, int* value_out = nullptr);
};
int current_device_slot();                 // index of the current device, -1 when unknown / beyond kMaxDevices
void per_device_lock();
void per_device_unlock();
template <typename Fn>
cudaError_t PerDeviceOnce::run(Fn&& fn, int* value_out) {
  const int dev = current_device_slot();
  if (dev < 0) return cudaErrorInvalidDevice;
  per_device_lock();
  cudaError_t e = cudaSuccess;
  if (!done[dev]) {
    int v = 0;
    e = fn(&v);
    if (e == cudaSuccess) {
      value[dev] = v;
      done[dev] = 1;
    }
  }
  if (value_out != nullptr) *value_out = value[dev];
  per_device_unlock();
  return e;
}
inline int check_launch() { return record_cuda_error(cudaGetLastError()); }

__host__ __device__ inline float fp8_max_of(int kind) { return kind == F8B200_E4M3 ? kE4M3Max : kE5M2Max; }
__host__ __device__ inline int hp_size_of(int dt) { return dt == F8B200_FP32 ? 4 : 2; }

// Rounds an fp32 value to the high-precision dtype and widens it back.
template <int HP>
__device__ __forceinline__ float round_hp(float v) {
  if constexpr (HP == F8B200_BF16) {
    return __bfloat162float(__float2bfloat16_rn(v));
  } else if constexpr (HP == F8B200_FP16) {
    return __half2float(__float2half_rn(v));
  } else {
    return v;
  }
}

__device__ __forceinline__ float round_hp_rt(float v, int hp) {
  if (hp == F8B200_BF16) return round_hp<F8B200_BF16>(v);
  if (hp == F8B200_FP16) return round_hp<F8B200_FP16>(v);
  return v;
}

// scale = RN_T( RN_T(1 / max(amax, RN_T(eps))) * fp8_max ), fp16 clamp on request.
// Reciprocal-then-multiply with a rounding after every step is what
// `finfo.max / clamp(amax, EPS)` evaluates to in PyTorch eager mode.
__device__ __forceinline__ float amax_to_scale_dev(float amax, float fp8_max, int amax_dtype,
                                                   bool clamp_fp16) {
  const float eps_t = round_hp_rt(kEps, amax_dtype);
  const float c = (amax != amax) ? amax : fmaxf(amax, eps_t);
  const float r = round_hp_rt(__fdiv_rn(1.0f, c), amax_dtype);
  float s = round_hp_rt(__fmul_rn(r, fp8_max), amax_dtype);
  if (clamp_fp16 && s == s) s = fminf(s, kFp16Max);
  return s;
}

// Two fp32 values -> two fp8 bytes (low byte = a).  cvt.rn.satfinite clamps to the
// finite range and rounds to nearest even, subnormals included; NaN is forced to 0x7F.
template <int KIND>
__device__ __forceinline__ uint32_t cvt_pair(float a, float b) {
  const __nv_fp8_interpretation_t interp = (KIND == F8B200_E4M3) ? __NV_E4M3 : __NV_E5M2;
  uint32_t r = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, interp);
  if (a != a) r = (r & 0xFF00u) | 0x7Fu;
  if (b != b) r = (r & 0x00FFu) | 0x7F00u;
  return r;
}

// Same rounding as round_hp, but bf16 goes through integer arithmetic (add half an
// ulp, ties to even, truncate) instead of the conversion pipe.  NaN inputs may come out
// as arbitrary values: callers test the UNROUNDED value for NaN.
template <int HP>
__device__ __forceinline__ float round_hp_fast(float v) {
  if constexpr (HP == F8B200_BF16) {
    uint32_t u = __float_as_uint(v);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return __uint_as_float(u & 0xFFFF0000u);
  } else {
    return round_hp<HP>(v);
  }
}

// cvt_pair without the NaN fix-up.
template <int KIND>
__device__ __forceinline__ uint32_t cvt_pair_raw(float a, float b) {
  const __nv_fp8_interpretation_t interp = (KIND == F8B200_E4M3) ? __NV_E4M3 : __NV_E5M2;
  return __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, interp);
}

// Four products -> four fp8 bytes (byte i = element i): optional rounding to the
// high-precision dtype, saturating RNE conversion, NaN forced to 0x7F.
template <int HP, int KIND>
__device__ __forceinline__ uint32_t cast4(float q0, float q1, float q2, float q3, bool round_to_hp) {
  float p0 = q0, p1 = q1, p2 = q2, p3 = q3;
  if (round_to_hp) {
    p0 = round_hp_fast<HP>(q0); p1 = round_hp_fast<HP>(q1); p2 = round_hp_fast<HP>(q2); p3 = round_hp_fast<HP>(q3);
  }
  uint32_t w = cvt_pair_raw<KIND>(p0, p1) | (cvt_pair_raw<KIND>(p2, p3) << 16);
  if ((q0 != q0) | (q1 != q1) | (q2 != q2) | (q3 != q3)) {
    if (q0 != q0) w = (w & 0xFFFFFF00u) | 0x0000007Fu;
    if (q1 != q1) w = (w & 0xFFFF00FFu) | 0x00007F00u;
    if (q2 != q2) w = (w & 0xFF00FFFFu) | 0x007F0000u;
    if (q3 != q3) w = (w & 0x00FFFFFFu) | 0x7F000000u;
  }
  return w;
}

__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) {
  return __reduce_max_sync(0xFFFFFFFFu, v);
}

}  // namespace f8b200
