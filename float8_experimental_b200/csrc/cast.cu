// Per-tensor scaling kernels: amax reduction, scale derivation, saturating RNE cast
// to e4m3fn / e5m2 with the transposed copy emitted from the same read, the fp8
// transpose, and the batched delayed-scaling bookkeeping.  All of them are bound by
// HBM bandwidth (or by launch latency for the bookkeeping), so the design rules are:
// 128-bit / 64-bit coalesced global accesses, enough loads in flight per thread to
// cover HBM latency, one atomic per CTA, and no re-read of the source.
#include <type_traits>

#include "common.cuh"

namespace f8b200 {

// ---------------------------------------------------------------------------
// amax
// ---------------------------------------------------------------------------
// |x| bit patterns order like unsigned integers for non-NaN values and every NaN
// pattern is larger than inf, so an unsigned max both finds the amax and propagates
// NaN.  2-byte types are reduced two at a time with a packed unsigned max.
template <int HP>
struct AbsMax {
  uint32_t m = 0;
  __device__ __forceinline__ void add_word(uint32_t w) {
    if constexpr (HP == F8B200_FP32) {
      m = max(m, w & 0x7FFFFFFFu);
    } else {
      m = __vmaxu2(m, w & 0x7FFF7FFFu);
    }
  }
  __device__ __forceinline__ void add_half(uint16_t h) { m = __vmaxu2(m, (uint32_t)(h & 0x7FFFu)); }
  // fp32 bit pattern of the running amax
  __device__ __forceinline__ uint32_t f32_bits() const {
    if constexpr (HP == F8B200_FP32) {
      return m;
    } else {
      const uint32_t h = max(m & 0xFFFFu, m >> 16);
      if constexpr (HP == F8B200_BF16) {
        return h << 16;
      } else {
        return __float_as_uint(__half2float(__ushort_as_half((unsigned short)h)));
      }
    }
  }
};

// CTA-wide max of `v`, then at most one atomic on the global word.
__device__ __forceinline__ void block_atomic_max(uint32_t v, uint32_t* out, uint32_t* smem) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_max_u32(v);
  if (lane == 0) smem[w] = v;
  __syncthreads();
  if (w == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    v = lane < nw ? smem[lane] : 0u;
    v = warp_max_u32(v);
    if (lane == 0 && v > *reinterpret_cast<volatile uint32_t*>(out)) atomicMax(out, v);
  }
}

template <int HP>
__device__ __forceinline__ uint32_t amax_flat_body(const char* base, int64_t n, int64_t gtid,
                                                   int64_t gstride) {
  constexpr int ES = (HP == F8B200_FP32) ? 4 : 2;
  constexpr int EPV = 16 / ES;
  AbsMax<HP> acc;
  // scalar head up to the first 16-byte boundary, vector body, scalar tail
  const uintptr_t addr = reinterpret_cast<uintptr_t>(base);
  int64_t head = (int64_t)(((16 - (addr & 15)) & 15) / ES);
  if (head > n) head = n;
  const int64_t nvec = (n - head) / EPV;
  const int64_t tail0 = head + nvec * EPV;
  if (gtid < head + (n - tail0)) {
    const int64_t i = gtid < head ? gtid : tail0 + (gtid - head);
    if constexpr (ES == 4) {
      acc.add_word(reinterpret_cast<const uint32_t*>(base)[i]);
    } else {
      acc.add_half(reinterpret_cast<const uint16_t*>(base)[i]);
    }
  }
  const uint4* v = reinterpret_cast<const uint4*>(base + head * ES);
  int64_t i = gtid;
  // eight independent 16-byte loads in flight per thread
  for (; i + 7 * gstride < nvec; i += 8 * gstride) {
    uint4 a[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) a[u] = v[i + u * gstride];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      acc.add_word(a[u].x); acc.add_word(a[u].y); acc.add_word(a[u].z); acc.add_word(a[u].w);
    }
  }
  for (; i < nvec; i += gstride) {
    const uint4 a = v[i];
    acc.add_word(a.x); acc.add_word(a.y); acc.add_word(a.z); acc.add_word(a.w);
  }
  return acc.f32_bits();
}

template <int HP>
__global__ void __launch_bounds__(512) amax_flat_kernel(const void* x, int64_t n, uint32_t* out) {
  __shared__ uint32_t smem[16];
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t gstride = (int64_t)gridDim.x * blockDim.x;
  const uint32_t m = amax_flat_body<HP>(static_cast<const char*>(x), n, gtid, gstride);
  block_atomic_max(m, out, smem);
}

constexpr int kMultiMax = 128;  // tensors per launch (2 KB of kernel parameters)
struct MultiAmaxArgs {
  const void* ptr[kMultiMax];
  int64_t numel[kMultiMax];
};

template <int HP>
__global__ void __launch_bounds__(512) multi_amax_kernel(const MultiAmaxArgs args, uint32_t* out) {
  __shared__ uint32_t smem[16];
  const int t = blockIdx.y;
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t gstride = (int64_t)gridDim.x * blockDim.x;
  const int64_t n = args.numel[t];
  uint32_t m = 0;
  if (n > 0) m = amax_flat_body<HP>(static_cast<const char*>(args.ptr[t]), n, gtid, gstride);
  block_atomic_max(m, out + t, smem);
}

__global__ void amax_to_scale_kernel(const float* amax, int64_t n, float fp8_max, int amax_dtype,
                                     int clamp_fp16, float* scale) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) scale[i] = amax_to_scale_dev(amax[i], fp8_max, amax_dtype, clamp_fp16 != 0);
}

// ---------------------------------------------------------------------------
// cast (+ transposed copy, + amax of the same read)
// ---------------------------------------------------------------------------
struct CastParams {
  const void* x;
  int64_t rows, cols, ld_x;
  const float* scale_in;
  float* scale_out;
  int scale_src;
  int product_fp32;
  uint8_t* out;
  int64_t ld_out;
  uint8_t* out_t;
  int64_t ld_out_t;
  uint32_t* amax_out;
  int reverse;
  int64_t tiles_c, ntiles;
  // further destinations of the row-major bytes (same row pitch): the gathered buffers of peer GPUs
  uint8_t* out_more[F8B200_CAST_MAX_EXTRA];
  int n_more;
};

template <int HP>
__device__ __forceinline__ float load_scale(const CastParams& p, float fp8_max) {
  if (p.scale_src == 1) {
    const float s = amax_to_scale_dev(*p.scale_in, fp8_max, HP, HP == F8B200_FP16);
    if (p.scale_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *p.scale_out = s;
    return s;
  }
  return *p.scale_in;
}

// A 128x128 byte tile held as 16 row-words per thread (warp w owns rows 16w..16w+15,
// lane owns columns 4*lane..4*lane+3) is transposed with byte permutes into one
// 16-byte vector per owned column, staged through shared memory with an XOR swizzle
// (conflict-free for both the 16-byte writes and the 16-byte reads) and written out
// as 128-byte contiguous row segments of the transposed matrix.
__device__ __forceinline__ void store_transposed_tile(const uint32_t (&rw)[16], uint4* smem_t,
                                                      uint8_t* out_t, int64_t ld_out_t,
                                                      int64_t tile_row0, int64_t tile_col0,
                                                      int64_t rows, int64_t cols) {
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  uint32_t cw[4][4];  // [column j][row group k]
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t a = rw[4 * k], b = rw[4 * k + 1], c = rw[4 * k + 2], d = rw[4 * k + 3];
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140);
    const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362);
    cw[0][k] = __byte_perm(t0, t1, 0x5410);
    cw[1][k] = __byte_perm(t0, t1, 0x7632);
    cw[2][k] = __byte_perm(t2, t3, 0x5410);
    cw[3][k] = __byte_perm(t2, t3, 0x7632);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = 4 * lane + j;
    smem_t[c * 8 + (w ^ (lane & 7))] = make_uint4(cw[j][0], cw[j][1], cw[j][2], cw[j][3]);
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int idx = it * 256 + tid;
    const int c = idx >> 3, chunk = idx & 7;
    const uint4 val = smem_t[c * 8 + (chunk ^ ((c >> 2) & 7))];
    const int64_t gc = tile_col0 + c;
    const int64_t gr = tile_row0 + chunk * 16;
    if (gc < cols && gr < rows) {
      uint8_t* dst = out_t + gc * ld_out_t + gr;
      if (gr + 16 <= rows) {
        *reinterpret_cast<uint4*>(dst) = val;
      } else {
        const uint32_t wv[4] = {val.x, val.y, val.z, val.w};
        for (int b = 0; b < 16 && gr + b < rows; ++b) dst[b] = (uint8_t)(wv[b >> 2] >> (8 * (b & 3)));
      }
    }
  }
}

template <int HP, int KIND>
__global__ void __launch_bounds__(256, 3) cast_tile_kernel(const CastParams p) {
  __shared__ uint4 smem_t[128 * 8];
  __shared__ uint32_t smem_max[8];
  constexpr int ES = (HP == F8B200_FP32) ? 4 : 2;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int64_t t = p.reverse ? (p.ntiles - 1 - (int64_t)blockIdx.x) : (int64_t)blockIdx.x;
  const int64_t tile_row0 = (t / p.tiles_c) * 128, tile_col0 = (t % p.tiles_c) * 128;
  const int64_t row0 = tile_row0 + w * 16, col = tile_col0 + lane * 4;
  const bool col_ok = col < p.cols;
  const float s = load_scale<HP>(p, (KIND == F8B200_E4M3) ? kE4M3Max : kE5M2Max);
  const char* xb = static_cast<const char*>(p.x);
  const bool round_to_hp = (ES == 2) && !p.product_fp32;

  uint32_t rw[16];
  AbsMax<HP> acc;
  if constexpr (ES == 2) {
    uint2 v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int64_t r = row0 + i;
      v[i] = make_uint2(0u, 0u);
      if (col_ok && r < p.rows) v[i] = __ldcs(reinterpret_cast<const uint2*>(xb + (r * p.ld_x + col) * ES));
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      acc.add_word(v[i].x);
      acc.add_word(v[i].y);
      float f0, f1, f2, f3;
      if constexpr (HP == F8B200_BF16) {
        f0 = __uint_as_float(v[i].x << 16);
        f1 = __uint_as_float(v[i].x & 0xFFFF0000u);
        f2 = __uint_as_float(v[i].y << 16);
        f3 = __uint_as_float(v[i].y & 0xFFFF0000u);
      } else {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v[i].x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v[i].y));
        f0 = a.x; f1 = a.y; f2 = b.x; f3 = b.y;
      }
      rw[i] = cast4<HP, KIND>(__fmul_rn(f0, s), __fmul_rn(f1, s), __fmul_rn(f2, s), __fmul_rn(f3, s), round_to_hp);
    }
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint4 v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int64_t r = row0 + h * 8 + i;
        v[i] = make_uint4(0u, 0u, 0u, 0u);
        if (col_ok && r < p.rows) v[i] = __ldcs(reinterpret_cast<const uint4*>(xb + (r * p.ld_x + col) * ES));
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        acc.add_word(v[i].x); acc.add_word(v[i].y); acc.add_word(v[i].z); acc.add_word(v[i].w);
        rw[h * 8 + i] = cast4<HP, KIND>(__fmul_rn(__uint_as_float(v[i].x), s), __fmul_rn(__uint_as_float(v[i].y), s),
                                        __fmul_rn(__uint_as_float(v[i].z), s), __fmul_rn(__uint_as_float(v[i].w), s),
                                        false);
      }
    }
  }

  if (p.out != nullptr && col_ok) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int64_t r = row0 + i;
      if (r < p.rows) *reinterpret_cast<uint32_t*>(p.out + r * p.ld_out + col) = rw[i];
    }
  }
  for (int d = 0; d < p.n_more && col_ok; ++d) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int64_t r = row0 + i;
      if (r < p.rows) *reinterpret_cast<uint32_t*>(p.out_more[d] + r * p.ld_out + col) = rw[i];
    }
  }
  if (p.out_t != nullptr) {
    store_transposed_tile(rw, smem_t, p.out_t, p.ld_out_t, tile_row0, tile_col0, p.rows, p.cols);
  }
  if (p.amax_out != nullptr) block_atomic_max(acc.f32_bits(), p.amax_out, smem_max);
}

// ---------------------------------------------------------------------------
// Main cast kernel: 128x128 tile per CTA, 8 rows x 8 columns per thread.
//   loads   16 bytes per row (two for fp32 input): a half-warp reads 256 contiguous bytes
//   stores  8 fp8 bytes per row: a half-warp writes 128 contiguous bytes
//   transposed copy: 8x8 byte transpose in registers (byte permutes), 8-byte columns
//           staged through 16 KB of shared memory with an XOR swizzle (conflict free in
//           both directions), written as 128-byte contiguous segments
// When the product x*scale is to be rounded to the input dtype and the scale itself is
// representable in that dtype (always true for a scale derived from the amax in that
// dtype) the product is taken with packed half-precision multiplies: the exact product
// of two 8-bit (bf16) or 11-bit (fp16) significands fits fp32, so
// RN_T(RN_fp32(x*s)) == RN_T(x*s), which is what HMUL2 returns.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void transpose4x4(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t& c0,
                                             uint32_t& c1, uint32_t& c2, uint32_t& c3) {
  const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140);
  const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362);
  c0 = __byte_perm(t0, t1, 0x5410);
  c1 = __byte_perm(t0, t1, 0x7632);
  c2 = __byte_perm(t2, t3, 0x5410);
  c3 = __byte_perm(t2, t3, 0x7632);
}

// lo[i] / hi[i]: fp8 bytes of columns 0..3 / 4..7 of row i (8 rows per thread).
__device__ __forceinline__ void store_transposed_tile8(const uint32_t (&lo)[8], const uint32_t (&hi)[8], uint2* smem_t,
                                                       uint8_t* out_t, int64_t ld_out_t, int64_t tile_row0,
                                                       int64_t tile_col0, int64_t rows, int64_t cols) {
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int cg = lane & 15, rg = w * 2 + (lane >> 4);
  uint32_t c[8][2];
  transpose4x4(lo[0], lo[1], lo[2], lo[3], c[0][0], c[1][0], c[2][0], c[3][0]);
  transpose4x4(lo[4], lo[5], lo[6], lo[7], c[0][1], c[1][1], c[2][1], c[3][1]);
  transpose4x4(hi[0], hi[1], hi[2], hi[3], c[4][0], c[5][0], c[6][0], c[7][0]);
  transpose4x4(hi[4], hi[5], hi[6], hi[7], c[4][1], c[5][1], c[6][1], c[7][1]);
#pragma unroll
  for (int j = 0; j < 8; ++j) smem_t[(cg * 8 + j) * 16 + (rg ^ cg)] = make_uint2(c[j][0], c[j][1]);
  __syncthreads();
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int idx = it * 256 + tid;
    const int col = idx >> 4, chunk = idx & 15;
    const uint2 val = smem_t[col * 16 + (chunk ^ ((col >> 3) & 15))];
    const int64_t gc = tile_col0 + col, gr = tile_row0 + chunk * 8;
    if (gc < cols && gr < rows) {
      uint8_t* dst = out_t + gc * ld_out_t + gr;
      if (gr + 8 <= rows) {
        *reinterpret_cast<uint2*>(dst) = val;
      } else {
        for (int b = 0; b < 8 && gr + b < rows; ++b)
          dst[b] = (uint8_t)((b < 4 ? val.x : val.y) >> (8 * (b & 3)));
      }
    }
  }
}

template <int KIND>
__device__ __forceinline__ uint32_t cvt_f16x2(uint32_t h2) {
  const __nv_fp8_interpretation_t interp = (KIND == F8B200_E4M3) ? __NV_E4M3 : __NV_E5M2;
  __half2_raw r;
  r.x = (unsigned short)(h2 & 0xFFFFu);
  r.y = (unsigned short)(h2 >> 16);
  return __nv_cvt_halfraw2_to_fp8x2(r, __NV_SATFINITE, interp);
}

// Two packed high-precision elements times the packed scale -> two fp8 bytes.
template <int HP, int KIND>
__device__ __forceinline__ uint32_t packed_mul_cvt(uint32_t x2, uint32_t s2) {
  if constexpr (HP == F8B200_BF16) {
    const __nv_bfloat162 p = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&x2),
                                     *reinterpret_cast<const __nv_bfloat162*>(&s2));
    const uint32_t u = *reinterpret_cast<const uint32_t*>(&p);
    return cvt_pair_raw<KIND>(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
  } else {
    const __half2 p = __hmul2(*reinterpret_cast<const __half2*>(&x2), *reinterpret_cast<const __half2*>(&s2));
    return cvt_f16x2<KIND>(*reinterpret_cast<const uint32_t*>(&p));
  }
}

template <int HP>
__device__ __forceinline__ void unpack2(uint32_t x2, float& a, float& b) {
  if constexpr (HP == F8B200_BF16) {
    a = __uint_as_float(x2 << 16);
    b = __uint_as_float(x2 & 0xFFFF0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&x2));
    a = f.x;
    b = f.y;
  }
}

template <int HP, int KIND, bool WANT_AMAX>
__global__ void __launch_bounds__(256, 2) cast_tile8_kernel(const CastParams p) {
  __shared__ uint2 smem_t[128 * 16];
  __shared__ uint32_t smem_max[8];
  constexpr int ES = (HP == F8B200_FP32) ? 4 : 2;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int cg = lane & 15, rg = w * 2 + (lane >> 4);
  const int64_t t = p.reverse ? (p.ntiles - 1 - (int64_t)blockIdx.x) : (int64_t)blockIdx.x;
  const int64_t tile_row0 = (t / p.tiles_c) * 128, tile_col0 = (t % p.tiles_c) * 128;
  const int64_t r0 = tile_row0 + rg * 8, c0 = tile_col0 + cg * 8;
  const bool col_ok = c0 < p.cols;  // cols is a multiple of 8 on this path
  int nrows = 0;
  if (col_ok && r0 < p.rows) nrows = (p.rows - r0) >= 8 ? 8 : (int)(p.rows - r0);
  const float s = load_scale<HP>(p, (KIND == F8B200_E4M3) ? kE4M3Max : kE5M2Max);
  const char* src = static_cast<const char*>(p.x) + (r0 * p.ld_x + c0) * ES;
  const int64_t row_bytes = p.ld_x * ES;

  uint32_t lo[8], hi[8];
  AbsMax<HP> acc;
  if constexpr (ES == 2) {
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] = make_uint4(0u, 0u, 0u, 0u);
      if (i < nrows) v[i] = __ldcs(reinterpret_cast<const uint4*>(src + i * row_bytes));
    }
    if constexpr (WANT_AMAX) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        acc.add_word(v[i].x); acc.add_word(v[i].y); acc.add_word(v[i].z); acc.add_word(v[i].w);
      }
    }
    // packed multiply only when it is bit-identical to the fp32 route (see above)
    const bool packed = !p.product_fp32 && round_hp<HP>(s) == s;
    if (packed) {
      uint32_t s2;
      if constexpr (HP == F8B200_BF16) {
        const __nv_bfloat162 sb = __float2bfloat162_rn(s);
        s2 = *reinterpret_cast<const uint32_t*>(&sb);
      } else {
        const __half2 sh = __float2half2_rn(s);
        s2 = *reinterpret_cast<const uint32_t*>(&sh);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        lo[i] = packed_mul_cvt<HP, KIND>(v[i].x, s2) | (packed_mul_cvt<HP, KIND>(v[i].y, s2) << 16);
        hi[i] = packed_mul_cvt<HP, KIND>(v[i].z, s2) | (packed_mul_cvt<HP, KIND>(v[i].w, s2) << 16);
      }
    } else {
      const bool round_to_hp = !p.product_fp32;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float f0, f1, f2, f3;
        unpack2<HP>(v[i].x, f0, f1);
        unpack2<HP>(v[i].y, f2, f3);
        lo[i] = cast4<HP, KIND>(__fmul_rn(f0, s), __fmul_rn(f1, s), __fmul_rn(f2, s), __fmul_rn(f3, s), round_to_hp);
        unpack2<HP>(v[i].z, f0, f1);
        unpack2<HP>(v[i].w, f2, f3);
        hi[i] = cast4<HP, KIND>(__fmul_rn(f0, s), __fmul_rn(f1, s), __fmul_rn(f2, s), __fmul_rn(f3, s), round_to_hp);
      }
    }
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint4 va[4], vb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        va[i] = make_uint4(0u, 0u, 0u, 0u);
        vb[i] = make_uint4(0u, 0u, 0u, 0u);
        if (h * 4 + i < nrows) {
          va[i] = __ldcs(reinterpret_cast<const uint4*>(src + (h * 4 + i) * row_bytes));
          vb[i] = __ldcs(reinterpret_cast<const uint4*>(src + (h * 4 + i) * row_bytes + 16));
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if constexpr (WANT_AMAX) {
          acc.add_word(va[i].x); acc.add_word(va[i].y); acc.add_word(va[i].z); acc.add_word(va[i].w);
          acc.add_word(vb[i].x); acc.add_word(vb[i].y); acc.add_word(vb[i].z); acc.add_word(vb[i].w);
        }
        lo[h * 4 + i] = cast4<HP, KIND>(__fmul_rn(__uint_as_float(va[i].x), s), __fmul_rn(__uint_as_float(va[i].y), s),
                                        __fmul_rn(__uint_as_float(va[i].z), s), __fmul_rn(__uint_as_float(va[i].w), s),
                                        false);
        hi[h * 4 + i] = cast4<HP, KIND>(__fmul_rn(__uint_as_float(vb[i].x), s), __fmul_rn(__uint_as_float(vb[i].y), s),
                                        __fmul_rn(__uint_as_float(vb[i].z), s), __fmul_rn(__uint_as_float(vb[i].w), s),
                                        false);
      }
    }
  }

  if (p.out != nullptr) {
    uint8_t* dst = p.out + r0 * p.ld_out + c0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < nrows) *reinterpret_cast<uint2*>(dst + i * p.ld_out) = make_uint2(lo[i], hi[i]);
  }
  for (int d = 0; d < p.n_more; ++d) {  // the same bytes into every peer's gathered buffer
    uint8_t* dst = p.out_more[d] + r0 * p.ld_out + c0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < nrows) *reinterpret_cast<uint2*>(dst + i * p.ld_out) = make_uint2(lo[i], hi[i]);
  }
  if (p.out_t != nullptr) {
    store_transposed_tile8(lo, hi, smem_t, p.out_t, p.ld_out_t, tile_row0, tile_col0, p.rows, p.cols);
  }
  if constexpr (WANT_AMAX) block_atomic_max(acc.f32_bits(), p.amax_out, smem_max);
}

// Any shape, stride or alignment: one element per thread.  Used only when the tiled
// kernel's alignment requirements do not hold.
template <int HP, int KIND>
__global__ void __launch_bounds__(256) cast_generic_kernel(const CastParams p) {
  __shared__ uint32_t smem_max[8];
  const float s = load_scale<HP>(p, (KIND == F8B200_E4M3) ? kE4M3Max : kE5M2Max);
  const int64_t n = p.rows * p.cols;
  AbsMax<HP> acc;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / p.cols, c = i % p.cols;
    float f;
    if constexpr (HP == F8B200_FP32) {
      const uint32_t u = static_cast<const uint32_t*>(p.x)[r * p.ld_x + c];
      acc.add_word(u);
      f = __uint_as_float(u);
    } else {
      const uint16_t u = static_cast<const uint16_t*>(p.x)[r * p.ld_x + c];
      acc.add_half(u);
      f = (HP == F8B200_BF16) ? __uint_as_float((uint32_t)u << 16) : __half2float(__ushort_as_half(u));
    }
    float pr = __fmul_rn(f, s);
    if (!p.product_fp32) pr = round_hp<HP>(pr);
    const uint8_t b = (uint8_t)(cvt_pair<KIND>(pr, 0.0f) & 0xFFu);
    if (p.out != nullptr) p.out[r * p.ld_out + c] = b;
    for (int d = 0; d < p.n_more; ++d) p.out_more[d][r * p.ld_out + c] = b;
    if (p.out_t != nullptr) p.out_t[c * p.ld_out_t + r] = b;
  }
  if (p.amax_out != nullptr) block_atomic_max(acc.f32_bits(), p.amax_out, smem_max);
}

// ---------------------------------------------------------------------------
// multi-tensor cast: n contiguous tensors, one scale each, one launch
// ---------------------------------------------------------------------------
constexpr int kMultiCastMax = 96;  // tensors per launch (kernel parameters stay below 4 KB)
struct MultiCastArgs {
  const void* x[kMultiCastMax];
  uint8_t* out[kMultiCastMax];
  int64_t numel[kMultiCastMax];
  const float* scales;  // scales[first + t] belongs to tensor t of this launch
  int first;
  int product_fp32;
};

// blockIdx.y picks the tensor, blockIdx.x strides over its 16-byte input vectors.  Same arithmetic as
// the tiled cast: product in fp32, rounded to the tensor's dtype unless product_fp32, saturating RNE.
template <int HP, int KIND>
__global__ void __launch_bounds__(256) multi_cast_kernel(const MultiCastArgs a) {
  constexpr int ES = (HP == F8B200_FP32) ? 4 : 2;
  constexpr int V = 16 / ES;
  const int t = blockIdx.y;
  const int64_t n = a.numel[t];
  const float s = a.scales[a.first + t];
  const bool round_to_hp = !a.product_fp32;
  const char* src = static_cast<const char*>(a.x[t]);
  uint8_t* dst = a.out[t];
  const bool vec = (reinterpret_cast<uintptr_t>(src) % 16 == 0) && (reinterpret_cast<uintptr_t>(dst) % (V / 4 * 4) == 0);
  const int64_t nvec = vec ? n / V : 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const uint4 v = __ldcs(reinterpret_cast<const uint4*>(src) + i);
    if constexpr (ES == 2) {
      float f0, f1, f2, f3;
      unpack2<HP>(v.x, f0, f1);
      unpack2<HP>(v.y, f2, f3);
      const uint32_t lo = cast4<HP, KIND>(__fmul_rn(f0, s), __fmul_rn(f1, s), __fmul_rn(f2, s), __fmul_rn(f3, s), round_to_hp);
      unpack2<HP>(v.z, f0, f1);
      unpack2<HP>(v.w, f2, f3);
      const uint32_t hi = cast4<HP, KIND>(__fmul_rn(f0, s), __fmul_rn(f1, s), __fmul_rn(f2, s), __fmul_rn(f3, s), round_to_hp);
      reinterpret_cast<uint2*>(dst)[i] = make_uint2(lo, hi);
    } else {
      reinterpret_cast<uint32_t*>(dst)[i] =
          cast4<HP, KIND>(__fmul_rn(__uint_as_float(v.x), s), __fmul_rn(__uint_as_float(v.y), s),
                          __fmul_rn(__uint_as_float(v.z), s), __fmul_rn(__uint_as_float(v.w), s), false);
    }
  }
  for (int64_t i = nvec * V + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float f;
    if constexpr (HP == F8B200_FP32) f = static_cast<const float*>(a.x[t])[i];
    else if constexpr (HP == F8B200_BF16) f = __uint_as_float((uint32_t)static_cast<const uint16_t*>(a.x[t])[i] << 16);
    else f = __half2float(__ushort_as_half(static_cast<const uint16_t*>(a.x[t])[i]));
    float pr = __fmul_rn(f, s);
    if (round_to_hp) pr = round_hp<HP>(pr);
    dst[i] = (uint8_t)(cvt_pair<KIND>(pr, 0.0f) & 0xFFu);
  }
}

// ---------------------------------------------------------------------------
// fp8 transpose
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) transpose_u8_tile_kernel(const uint8_t* in, int64_t rows, int64_t cols,
                                                                int64_t ld_in, uint8_t* out, int64_t ld_out,
                                                                int64_t tiles_c) {
  __shared__ uint4 smem_t[128 * 8];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int64_t t = blockIdx.x;
  const int64_t tile_row0 = (t / tiles_c) * 128, tile_col0 = (t % tiles_c) * 128;
  const int64_t row0 = tile_row0 + w * 16, col = tile_col0 + lane * 4;
  uint32_t rw[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int64_t r = row0 + i;
    rw[i] = 0u;
    if (col < cols && r < rows) rw[i] = __ldcs(reinterpret_cast<const uint32_t*>(in + r * ld_in + col));
  }
  store_transposed_tile(rw, smem_t, out, ld_out, tile_row0, tile_col0, rows, cols);
}

__global__ void __launch_bounds__(256) transpose_u8_tile8_kernel(const uint8_t* in, int64_t rows, int64_t cols,
                                                                 int64_t ld_in, uint8_t* out, int64_t ld_out,
                                                                 int64_t tiles_c) {
  __shared__ uint2 smem_t[128 * 16];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int cg = lane & 15, rg = w * 2 + (lane >> 4);
  const int64_t t = blockIdx.x;
  const int64_t tile_row0 = (t / tiles_c) * 128, tile_col0 = (t % tiles_c) * 128;
  const int64_t r0 = tile_row0 + rg * 8, c0 = tile_col0 + cg * 8;
  uint32_t lo[8], hi[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint2 v = make_uint2(0u, 0u);
    if (c0 < cols && r0 + i < rows) v = __ldcs(reinterpret_cast<const uint2*>(in + (r0 + i) * ld_in + c0));
    lo[i] = v.x;
    hi[i] = v.y;
  }
  store_transposed_tile8(lo, hi, smem_t, out, ld_out, tile_row0, tile_col0, rows, cols);
}

__global__ void transpose_u8_generic_kernel(const uint8_t* in, int64_t rows, int64_t cols, int64_t ld_in,
                                            uint8_t* out, int64_t ld_out) {
  const int64_t n = rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, c = i % cols;
    out[c * ld_out + r] = in[r * ld_in + c];
  }
}

// ---------------------------------------------------------------------------
// delayed-scaling bookkeeping
// ---------------------------------------------------------------------------
// General form: one thread per (layer, tensor) row walks the history.
__global__ void delayed_sync_serial_kernel(const float* amax, const float* hist, int64_t ld_hist, int64_t rows,
                                           int hist_len, int64_t n_e4m3, int clamp_fp16, float* scale_out,
                                           float* hist_out, int64_t ld_hist_out) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const float cur = amax[r];
  const float* h = hist + r * ld_hist;
  float m = cur;
  bool has_nan = cur != cur;
  float prev = cur;  // value moving into slot i
  for (int i = 0; i < hist_len; ++i) {
    const float old = h[i];
    if (i < hist_len - 1) {  // old h[i] survives the roll (lands in slot i+1)
      has_nan |= (old != old);
      m = fmaxf(m, old);
    }
    if (hist_out != nullptr) hist_out[r * ld_hist_out + i] = prev;
    prev = old;
  }
  if (has_nan) m = __uint_as_float(0x7FC00000u);
  const float fmax8 = r < n_e4m3 ? kE4M3Max : kE5M2Max;
  scale_out[r] = amax_to_scale_dev(m, fmax8, F8B200_FP32, clamp_fp16 != 0);
}

// hist_len <= 16 (the default recipe): 16 lanes per row, one parallel load of the whole
// history, roll by shuffle, max by butterfly.  All reads of a row happen before any write,
// so hist_out may alias hist.
__global__ void __launch_bounds__(128) delayed_sync_kernel(const float* amax, const float* hist, int64_t ld_hist,
                                                           int64_t rows, int hist_len, int64_t n_e4m3,
                                                           int clamp_fp16, float* scale_out, float* hist_out,
                                                           int64_t ld_hist_out) {
  const int sub = threadIdx.x & 15;
  const int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
  const bool live = r < rows;
  const bool has_entry = live && sub < hist_len;
  const float cur = live ? amax[r] : 0.0f;
  const float old = has_entry ? hist[r * ld_hist + sub] : 0.0f;
  float prev = __shfl_up_sync(0xFFFFFFFFu, old, 1, 16);  // entry sub-1 of the same row
  if (sub == 0) prev = cur;
  // entries 0..H-2 survive the roll; the current amax joins them
  float m = (has_entry && sub < hist_len - 1) ? old : 0.0f;
  bool has_nan = (m != m) || (cur != cur);
  m = fmaxf(m, cur);
  const unsigned nanbits = __ballot_sync(0xFFFFFFFFu, has_nan);
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
  __syncwarp();
  if (has_entry && hist_out != nullptr) hist_out[r * ld_hist_out + sub] = prev;
  if (live && sub == 0) {
    if (nanbits & (0xFFFFu << (threadIdx.x & 16))) m = __uint_as_float(0x7FC00000u);
    const float fmax8 = r < n_e4m3 ? kE4M3Max : kE5M2Max;
    scale_out[r] = amax_to_scale_dev(m, fmax8, F8B200_FP32, clamp_fp16 != 0);
  }
}

// ---------------------------------------------------------------------------
// host entry points
// ---------------------------------------------------------------------------
static inline bool aligned_to(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

template <typename F>
static int dispatch_hp(int hp, F&& f) {
  switch (hp) {
    case F8B200_BF16: return f(std::integral_constant<int, F8B200_BF16>{});
    case F8B200_FP16: return f(std::integral_constant<int, F8B200_FP16>{});
    case F8B200_FP32: return f(std::integral_constant<int, F8B200_FP32>{});
    default: return F8B200_ERR_BAD_ARG;
  }
}

}  // namespace f8b200

using namespace f8b200;

extern "C" int f8b200_amax(const void* x, int hp_dtype, int64_t numel, float* amax_out, void* stream) {
  if (x == nullptr || amax_out == nullptr || numel <= 0) return F8B200_ERR_BAD_ARG;
  if (hp_dtype < 0 || hp_dtype > 2) return F8B200_ERR_BAD_ARG;
  if (!aligned_to(x, hp_size_of(hp_dtype)) || !aligned_to(amax_out, 4)) return F8B200_ERR_ALIGNMENT;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = record_cuda_error(cudaMemsetAsync(amax_out, 0, sizeof(float), st));
  if (rc != F8B200_OK) return rc;
  const int64_t nvec = numel / (16 / hp_size_of(hp_dtype));
  int64_t blocks = (nvec + 512 * 8 - 1) / (512 * 8);
  const int64_t cap = (int64_t)sm_count() * 3;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return dispatch_hp(hp_dtype, [&](auto hp) {
    amax_flat_kernel<decltype(hp)::value><<<(unsigned)blocks, 512, 0, st>>>(x, numel, reinterpret_cast<uint32_t*>(amax_out));
    return check_launch();
  });
}

extern "C" int f8b200_multi_amax(const void* const* ptrs, const int64_t* numels, int n, int hp_dtype,
                                 float* amax_out, void* stream) {
  if (n < 0 || (n > 0 && (ptrs == nullptr || numels == nullptr || amax_out == nullptr))) return F8B200_ERR_BAD_ARG;
  if (hp_dtype < 0 || hp_dtype > 2) return F8B200_ERR_BAD_ARG;
  if (n == 0) return F8B200_OK;
  for (int i = 0; i < n; ++i) {
    if (numels[i] < 0 || (numels[i] > 0 && ptrs[i] == nullptr)) return F8B200_ERR_BAD_ARG;
    if (numels[i] > 0 && !aligned_to(ptrs[i], hp_size_of(hp_dtype))) return F8B200_ERR_ALIGNMENT;
  }
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = record_cuda_error(cudaMemsetAsync(amax_out, 0, sizeof(float) * (size_t)n, st));
  if (rc != F8B200_OK) return rc;
  for (int base = 0; base < n; base += kMultiMax) {
    const int cnt = (n - base < kMultiMax) ? (n - base) : kMultiMax;
    MultiAmaxArgs args;
    int64_t biggest = 0;
    for (int i = 0; i < kMultiMax; ++i) {
      args.ptr[i] = i < cnt ? ptrs[base + i] : nullptr;
      args.numel[i] = i < cnt ? numels[base + i] : 0;
      if (args.numel[i] > biggest) biggest = args.numel[i];
    }
    // enough CTAs per tensor to keep every SM busy even when only a few tensors are large
    int64_t bx = (biggest / (16 / hp_size_of(hp_dtype)) + 512 * 4 - 1) / (512 * 4);
    int64_t cap = ((int64_t)sm_count() * 8 + cnt - 1) / cnt;
    if (cap < 1) cap = 1;
    if (bx > cap) bx = cap;
    if (bx < 1) bx = 1;
    dim3 grid((unsigned)bx, (unsigned)cnt);
    rc = dispatch_hp(hp_dtype, [&](auto hp) {
      multi_amax_kernel<decltype(hp)::value><<<grid, 512, 0, st>>>(args, reinterpret_cast<uint32_t*>(amax_out) + base);
      return check_launch();
    });
    if (rc != F8B200_OK) return rc;
  }
  return F8B200_OK;
}

extern "C" int f8b200_amax_to_scale(const float* amax, int64_t n, int fp8_kind, int amax_dtype, int orig_dtype,
                                    float* scale_out, void* stream) {
  if (n < 0 || (n > 0 && (amax == nullptr || scale_out == nullptr))) return F8B200_ERR_BAD_ARG;
  if (fp8_kind < 0 || fp8_kind > 1 || amax_dtype < 0 || amax_dtype > 2 || orig_dtype < 0 || orig_dtype > 2)
    return F8B200_ERR_BAD_ARG;
  if (n == 0) return F8B200_OK;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  amax_to_scale_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      amax, n, fp8_max_of(fp8_kind), amax_dtype, orig_dtype == F8B200_FP16 ? 1 : 0, scale_out);
  return check_launch();
}

static int cast_impl(const void* x, int hp_dtype, int64_t rows, int64_t cols, int64_t ld_x, int scale_src,
                     const float* scale_in, float* scale_out, int product_fp32, int fp8_kind, void* out, int64_t ld_out,
                     void* out_t, int64_t ld_out_t, float* amax_out, int reverse, void* const* more_outs, int n_more,
                     void* stream) {
  if (rows < 0 || cols < 0 || hp_dtype < 0 || hp_dtype > 2 || fp8_kind < 0 || fp8_kind > 1) return F8B200_ERR_BAD_ARG;
  if (n_more < 0 || n_more > F8B200_CAST_MAX_EXTRA || (n_more > 0 && (more_outs == nullptr || ld_out < cols)))
    return F8B200_ERR_BAD_ARG;
  for (int d = 0; d < n_more; ++d)
    if (more_outs[d] == nullptr) return F8B200_ERR_BAD_ARG;
  if (scale_src < 0 || scale_src > 1 || scale_in == nullptr) return F8B200_ERR_BAD_ARG;
  if (ld_x < cols || (out != nullptr && ld_out < cols) || (out_t != nullptr && ld_out_t < rows)) return F8B200_ERR_BAD_ARG;
  if (rows > 0 && cols > 0 && x == nullptr) return F8B200_ERR_BAD_ARG;
  const int es = hp_size_of(hp_dtype);
  if (!aligned_to(x, es) || !aligned_to(scale_in, 4) || !aligned_to(scale_out, 4) || !aligned_to(amax_out, 4))
    return F8B200_ERR_ALIGNMENT;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (amax_out != nullptr) {
    rc = record_cuda_error(cudaMemsetAsync(amax_out, 0, sizeof(float), st));
    if (rc != F8B200_OK) return rc;
  }
  CastParams p;
  p.x = x; p.rows = rows; p.cols = cols; p.ld_x = ld_x;
  p.scale_in = scale_in; p.scale_out = scale_out; p.scale_src = scale_src; p.product_fp32 = product_fp32;
  p.out = static_cast<uint8_t*>(out); p.ld_out = ld_out;
  p.out_t = static_cast<uint8_t*>(out_t); p.ld_out_t = ld_out_t;
  p.amax_out = reinterpret_cast<uint32_t*>(amax_out); p.reverse = reverse;
  p.n_more = n_more;
  bool more4 = ld_out % 4 == 0, more8 = ld_out % 8 == 0;
  for (int d = 0; d < F8B200_CAST_MAX_EXTRA; ++d) {
    p.out_more[d] = d < n_more ? static_cast<uint8_t*>(more_outs[d]) : nullptr;
    if (d < n_more) {
      more4 = more4 && aligned_to(more_outs[d], 4);
      more8 = more8 && aligned_to(more_outs[d], 8);
    }
  }
  p.tiles_c = (cols + 127) / 128;
  p.ntiles = p.tiles_c * ((rows + 127) / 128);
  const bool empty = rows == 0 || cols == 0;
  if (empty) {
    // nothing to cast; the scale of a dynamic cast is still defined by the amax word
    p.ntiles = 0;
  }
  const bool fast = cols % 4 == 0 && ld_x % 4 == 0 && aligned_to(x, 4 * es) &&
                    (out == nullptr || (ld_out % 4 == 0 && aligned_to(out, 4))) &&
                    (out_t == nullptr || (ld_out_t % 16 == 0 && aligned_to(out_t, 16))) && (n_more == 0 || more4);
  const bool fast8 = cols % 8 == 0 && (ld_x * es) % 16 == 0 && aligned_to(x, 16) &&
                     (out == nullptr || (ld_out % 8 == 0 && aligned_to(out, 8))) &&
                     (out_t == nullptr || (ld_out_t % 8 == 0 && aligned_to(out_t, 8))) && (n_more == 0 || more8);
  return dispatch_hp(hp_dtype, [&](auto hp) {
    constexpr int HP = decltype(hp)::value;
    if (empty) {
      if (scale_src == 1 && scale_out != nullptr) {
        amax_to_scale_kernel<<<1, 32, 0, st>>>(scale_in, 1, fp8_max_of(fp8_kind), HP, HP == F8B200_FP16, scale_out);
        return check_launch();
      }
      return (int)F8B200_OK;
    }
    if (fast8) {
      if (p.ntiles > 0x7FFFFFFFLL) return (int)F8B200_ERR_UNSUPPORTED;
      const unsigned g = (unsigned)p.ntiles;
      if (fp8_kind == F8B200_E4M3) {
        if (amax_out != nullptr) cast_tile8_kernel<HP, F8B200_E4M3, true><<<g, 256, 0, st>>>(p);
        else cast_tile8_kernel<HP, F8B200_E4M3, false><<<g, 256, 0, st>>>(p);
      } else {
        if (amax_out != nullptr) cast_tile8_kernel<HP, F8B200_E5M2, true><<<g, 256, 0, st>>>(p);
        else cast_tile8_kernel<HP, F8B200_E5M2, false><<<g, 256, 0, st>>>(p);
      }
    } else if (fast) {
      if (p.ntiles > 0x7FFFFFFFLL) return (int)F8B200_ERR_UNSUPPORTED;
      if (fp8_kind == F8B200_E4M3) cast_tile_kernel<HP, F8B200_E4M3><<<(unsigned)p.ntiles, 256, 0, st>>>(p);
      else cast_tile_kernel<HP, F8B200_E5M2><<<(unsigned)p.ntiles, 256, 0, st>>>(p);
    } else {
      int64_t blocks = (rows * cols + 255) / 256;
      const int64_t cap = (int64_t)sm_count() * 16;
      if (blocks > cap) blocks = cap;
      if (fp8_kind == F8B200_E4M3) cast_generic_kernel<HP, F8B200_E4M3><<<(unsigned)blocks, 256, 0, st>>>(p);
      else cast_generic_kernel<HP, F8B200_E5M2><<<(unsigned)blocks, 256, 0, st>>>(p);
    }
    return check_launch();
  });
}

extern "C" int f8b200_cast(const void* x, int hp_dtype, int64_t rows, int64_t cols, int64_t ld_x, int scale_src,
                           const float* scale_in, float* scale_out, int product_fp32, int fp8_kind, void* out,
                           int64_t ld_out, void* out_t, int64_t ld_out_t, float* amax_out, int reverse,
                           void* stream) {
  return cast_impl(x, hp_dtype, rows, cols, ld_x, scale_src, scale_in, scale_out, product_fp32, fp8_kind, out, ld_out,
                   out_t, ld_out_t, amax_out, reverse, nullptr, 0, stream);
}

extern "C" int f8b200_multi_cast(const void* const* xs, const int64_t* numels, int n, int hp_dtype, const float* scales,
                                 int product_fp32, int fp8_kind, void* const* outs, void* stream) {
  if (n < 0 || hp_dtype < 0 || hp_dtype > 2 || fp8_kind < 0 || fp8_kind > 1) return F8B200_ERR_BAD_ARG;
  if (n == 0) return F8B200_OK;
  if (xs == nullptr || numels == nullptr || outs == nullptr || scales == nullptr) return F8B200_ERR_BAD_ARG;
  const int es = hp_size_of(hp_dtype);
  int64_t largest = 0;
  for (int i = 0; i < n; ++i) {
    if (numels[i] < 0 || (numels[i] > 0 && (xs[i] == nullptr || outs[i] == nullptr))) return F8B200_ERR_BAD_ARG;
    if (!aligned_to(xs[i], es)) return F8B200_ERR_ALIGNMENT;
    if (numels[i] > largest) largest = numels[i];
  }
  if (!aligned_to(scales, 4)) return F8B200_ERR_ALIGNMENT;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int first = 0; first < n; first += kMultiCastMax) {
    const int cnt = (n - first) < kMultiCastMax ? (n - first) : kMultiCastMax;
    MultiCastArgs a = {};
    int64_t big = 0;
    for (int t = 0; t < cnt; ++t) {
      a.x[t] = xs[first + t];
      a.out[t] = static_cast<uint8_t*>(outs[first + t]);
      a.numel[t] = numels[first + t];
      if (a.numel[t] > big) big = a.numel[t];
    }
    a.scales = scales;
    a.first = first;
    a.product_fp32 = product_fp32;
    // enough CTAs for the largest tensor of the launch, capped so that the grid stays a few waves
    int64_t bx = (big / (16 / es) + 255) / 256;
    const int64_t cap = ((int64_t)sm_count() * 8 + cnt - 1) / cnt;
    if (bx > cap) bx = cap;
    if (bx < 1) bx = 1;
    const dim3 grid((unsigned)bx, (unsigned)cnt);
    rc = dispatch_hp(hp_dtype, [&](auto hp) {
      constexpr int HP = decltype(hp)::value;
      if (fp8_kind == F8B200_E4M3) multi_cast_kernel<HP, F8B200_E4M3><<<grid, 256, 0, st>>>(a);
      else multi_cast_kernel<HP, F8B200_E5M2><<<grid, 256, 0, st>>>(a);
      return check_launch();
    });
    if (rc != F8B200_OK) return rc;
  }
  return F8B200_OK;
}

extern "C" int f8b200_cast_dynamic(const void* x, int hp_dtype, int64_t rows, int64_t cols, int fp8_kind, float* amax_out,
                                   float* scale_out, void* out, void* stream) {
  if (amax_out == nullptr || out == nullptr || rows <= 0 || cols <= 0) return F8B200_ERR_BAD_ARG;
  int rc = f8b200_amax(x, hp_dtype, rows * cols, amax_out, stream);
  if (rc != F8B200_OK) return rc;
  return cast_impl(x, hp_dtype, rows, cols, cols, 1, amax_out, scale_out, 0, fp8_kind, out, cols, nullptr, 0, nullptr, 1,
                   nullptr, 0, stream);
}

extern "C" int f8b200_cast_scatter(const void* x, int hp_dtype, int64_t rows, int64_t cols, int64_t ld_x, int scale_src,
                                   const float* scale_in, float* scale_out, int product_fp32, int fp8_kind,
                                   void* const* outs, int n_outs, int64_t ld_out, void* stream) {
  if (outs == nullptr || n_outs < 1 || n_outs > F8B200_CAST_MAX_EXTRA + 1) return F8B200_ERR_BAD_ARG;
  return cast_impl(x, hp_dtype, rows, cols, ld_x, scale_src, scale_in, scale_out, product_fp32, fp8_kind, outs[0],
                   ld_out, nullptr, 0, nullptr, 0, outs + 1, n_outs - 1, stream);
}

extern "C" int f8b200_transpose_u8(const void* in, int64_t rows, int64_t cols, int64_t ld_in, void* out,
                                   int64_t ld_out, void* stream) {
  if (rows < 0 || cols < 0 || ld_in < cols || ld_out < rows) return F8B200_ERR_BAD_ARG;
  if (rows == 0 || cols == 0) return F8B200_OK;
  if (in == nullptr || out == nullptr) return F8B200_ERR_BAD_ARG;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool fast = cols % 4 == 0 && ld_in % 4 == 0 && aligned_to(in, 4) && ld_out % 16 == 0 && aligned_to(out, 16);
  const bool fast8 = cols % 8 == 0 && ld_in % 8 == 0 && aligned_to(in, 8) && ld_out % 8 == 0 && aligned_to(out, 8);
  if (fast8) {
    const int64_t tiles_c = (cols + 127) / 128;
    const int64_t ntiles = tiles_c * ((rows + 127) / 128);
    if (ntiles > 0x7FFFFFFFLL) return F8B200_ERR_UNSUPPORTED;
    transpose_u8_tile8_kernel<<<(unsigned)ntiles, 256, 0, st>>>(static_cast<const uint8_t*>(in), rows, cols, ld_in,
                                                                static_cast<uint8_t*>(out), ld_out, tiles_c);
  } else if (fast) {
    const int64_t tiles_c = (cols + 127) / 128;
    const int64_t ntiles = tiles_c * ((rows + 127) / 128);
    if (ntiles > 0x7FFFFFFFLL) return F8B200_ERR_UNSUPPORTED;
    transpose_u8_tile_kernel<<<(unsigned)ntiles, 256, 0, st>>>(static_cast<const uint8_t*>(in), rows, cols, ld_in,
                                                               static_cast<uint8_t*>(out), ld_out, tiles_c);
  } else {
    int64_t blocks = (rows * cols + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    transpose_u8_generic_kernel<<<(unsigned)blocks, 256, 0, st>>>(static_cast<const uint8_t*>(in), rows, cols, ld_in,
                                                                  static_cast<uint8_t*>(out), ld_out);
  }
  return check_launch();
}

extern "C" int f8b200_delayed_sync(const float* amax, const float* hist, int64_t ld_hist, int64_t rows, int hist_len,
                                   int64_t n_e4m3, int orig_dtype, float* scale_out, float* hist_out,
                                   int64_t ld_hist_out, void* stream) {
  if (rows < 0 || hist_len < 1 || n_e4m3 < 0 || orig_dtype < 0 || orig_dtype > 2) return F8B200_ERR_BAD_ARG;
  if (rows == 0) return F8B200_OK;
  if (amax == nullptr || hist == nullptr || scale_out == nullptr || ld_hist < hist_len) return F8B200_ERR_BAD_ARG;
  if (hist_out != nullptr && ld_hist_out < hist_len) return F8B200_ERR_BAD_ARG;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int clamp = orig_dtype == F8B200_FP16 ? 1 : 0;
  if (hist_len <= 16) {
    const unsigned blocks = (unsigned)((rows * 16 + 127) / 128);
    delayed_sync_kernel<<<blocks, 128, 0, st>>>(amax, hist, ld_hist, rows, hist_len, n_e4m3, clamp, scale_out,
                                                hist_out, ld_hist_out);
  } else {
    const unsigned blocks = (unsigned)((rows + 127) / 128);
    delayed_sync_serial_kernel<<<blocks, 128, 0, st>>>(amax, hist, ld_hist, rows, hist_len, n_e4m3, clamp,
                                                       scale_out, hist_out, ld_hist_out);
  }
  return check_launch();
}
