// Second half of the reduce-scatter that starts in the GEMM epilogue (f8b200_gemm_fp8_scatter_rows):
// every rank has stored its partial product of this rank's rows into one slot of this rank's buffer;
// this kernel adds the slots up.  out[i] = RN_T(sum over s of slot_s[i]), accumulated in fp32 in
// slot order, so the result does not depend on timing.  HBM-bound: (n_slots + 1) x numel elements.
#include "common.cuh"

namespace f8b200 {
namespace {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }

// One thread handles 16 bytes of every slot at a time.
template <typename T>
__global__ void __launch_bounds__(256) sum_slots_kernel(const T* __restrict__ slots, int n_slots, int64_t slot_stride,
                                                        int64_t numel, T* __restrict__ out) {
  constexpr int V = 16 / (int)sizeof(T);
  const int64_t nvec = numel / V;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; ++e) acc[e] = 0.f;
    for (int s = 0; s < n_slots; ++s) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(slots + (int64_t)s * slot_stride) + i);
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] += to_f32<T>(v[e]);
    }
    uint4 packed;
    T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
    for (int e = 0; e < V; ++e) o[e] = from_f32<T>(acc[e]);
    reinterpret_cast<uint4*>(out)[i] = packed;
  }
  // tail (numel not a multiple of the vector width)
  for (int64_t i = nvec * V + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += stride) {
    float acc = 0.f;
    for (int s = 0; s < n_slots; ++s) acc += to_f32<T>(slots[(int64_t)s * slot_stride + i]);
    out[i] = from_f32<T>(acc);
  }
}

template <typename T>
int launch_sum(const void* slots, int n_slots, int64_t slot_stride, int64_t numel, void* out, cudaStream_t st) {
  constexpr int V = 16 / (int)sizeof(T);
  int64_t blocks = (numel / V + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  sum_slots_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const T*>(slots), n_slots, slot_stride, numel,
                                                          static_cast<T*>(out));
  return check_launch();
}

}  // namespace
}  // namespace f8b200

using namespace f8b200;

extern "C" int f8b200_sum_slots(const void* slots, int n_slots, int64_t slot_stride, int hp_dtype, int64_t numel,
                                void* out, void* stream) {
  if (slots == nullptr || out == nullptr || n_slots < 1 || numel < 0 || slot_stride < numel) return F8B200_ERR_BAD_ARG;
  if (hp_dtype < 0 || hp_dtype > 2) return F8B200_ERR_BAD_ARG;
  if (numel == 0) return F8B200_OK;
  const int esz = hp_size_of(hp_dtype);
  if (reinterpret_cast<uintptr_t>(slots) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0 ||
      (slot_stride * esz) % 16 != 0)
    return F8B200_ERR_ALIGNMENT;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (hp_dtype == F8B200_BF16) return launch_sum<__nv_bfloat16>(slots, n_slots, slot_stride, numel, out, st);
  if (hp_dtype == F8B200_FP16) return launch_sum<__half>(slots, n_slots, slot_stride, numel, out, st);
  return launch_sum<float>(slots, n_slots, slot_stride, numel, out, st);
}
