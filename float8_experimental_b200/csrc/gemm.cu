// Scaled fp8 GEMM for sm_100a:  out[M,N] = (A[M,K] . B[N,K]^T) / (sa * sb) (+ bias).
//
// Four persistent, warp-specialised kernels share the device code of this file:
//   pair-wide kernel (namespace pairwide, the default for large products with K >= 8192) two CTAs per
//                 512x256 tile, two tcgen05.mma.cta_group::2 per k-step, one 256x256 accumulator per CTA
//                 drained by halves;
//   pair kernel   (namespace pair, the default for short K, for products whose 512x256 tiles would fill
//                 the last wave badly and for at most 256 rows: see gemm_mode) two CTAs per 256x256 tile,
//                 tcgen05.mma.cta_group::2, accumulators double buffered in tensor memory;
//   wide kernel   (namespace wide) one CTA per 256x256 tile, two M128 N256 MMAs per k-step, the
//                 accumulator fills tensor memory;
//   one-CTA kernel (below) one CTA per 128x256 tile; kept as the simplest reference of the scheme.
// Each operand is fp8 bytes, K-major (storage [rows, K]) or MN-major (storage [K, rows]).
// Tiles are walked in L2-friendly bands, with a fixed stride per CTA or claimed from a counter
// (dynamic tile scheduling, see TileRing).  Warp roles, in every kernel:
//   warp 0      TMA producer: cp.async.bulk.tensor 128-byte-swizzled boxes of A and B into a
//               shared-memory ring, mbarrier complete_tx.
//   warp 1      MMA issuer: one thread issues tcgen05.mma.kind::f8f6f4 (K = 32 per instruction)
//               from shared-memory descriptors into fp32 accumulators in tensor memory;
//               tcgen05.commit releases ring slots and publishes finished accumulators.
//   warps 2..   epilogue: tcgen05.ld the accumulator, multiply by 1/(sa*sb), add bias,
//               convert to the output dtype and store through swizzled staging boxes and
//               TMA stores (or per-thread stores when the output is not 16-byte aligned).
// Every mbarrier wait is bounded by a cycle budget; on expiry the kernel raises a flag
// in a device error word, all roles leave their loops, tensor memory is released and
// the kernel returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace f8b200 {

__device__ uint32_t g_device_error = 0;

namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;  // bytes == fp8 elements; one 128-byte swizzle span
constexpr int UMMA_K = 32;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;
constexpr int B_BYTES = BN * BK;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr long long WAIT_BUDGET_CYCLES = 2000000000LL;  // about one second

struct __align__(8) Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 4 * 2 * 32 * 128 /* epilogue staging */ + 1024 /* alignment slack */ +
                           (int)sizeof(Barriers);

// ---- PTX wrappers ---------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same probe with a suspend-time hint: the hardware may keep the thread suspended for up to about
// `hint_ns` while the phase is incomplete and wakes it when the phase completes, so a long wait costs a few
// probes instead of a polling loop.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
constexpr uint32_t WAIT_BY_HINT = 0x80000000u;  // flag in a `backoff_ns` argument: the rest is a suspend-time hint

// Bounded wait.  Returns false when the budget ran out or another role already gave up.
// `backoff_ns` > 0 puts the polling thread to sleep between probes: waits that are long
// and off the critical path (ring slots coming free, a whole tile being accumulated)
// should not burn issue slots and power that the tensor pipe could use.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Barriers* bars, uint32_t who,
                                          uint32_t backoff_ns = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 0; it < 0x7FFFFFFFu; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (backoff_ns != 0u) __nanosleep(backoff_ns);
    if ((it & 63u) == 63u) {
      if (bars->abort_flag != 0u) return false;
      if (clock64() - t0 > WAIT_BUDGET_CYCLES) break;
    }
  }
  bars->abort_flag = 1u;
  atomicOr(&g_device_error, who);
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// L2 eviction-priority policies for the bulk tensor copies (0 = normal, 1 = evict first, 2 = evict last).
// Kind 0 returns 0, which the load wrappers below take as "issue the copy WITHOUT a cache-hint operand".
// That matters: operand loads that carry an explicit policy, even the evict-normal one, are not merged by
// the L2 request coalescer, while plain loads of the same 128-byte lines by several SMs at about the same
// time are served by one L2 lookup (ncu: lrc__average_xbar2gpc_sectors_op_read.ratio 1.00 with the hint,
// 1.15-1.29 without; L2 lookups of the wo forward GEMM 6.56 -> 5.11 GB, die-to-die L2 traffic 1.29 -> 0.74
// GB, and 1.5 % less time over the twelve GEMMs of the LLaMa-2-70B step).
__device__ __forceinline__ uint64_t l2_policy(int kind) {
  uint64_t p = 0;
  if (kind == 1) asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  else if (kind == 2) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar,
                                                 uint64_t policy) {
  if (policy == 0) {  // default L2 policy: no hint operand (see l2_policy)
    tma_load_2d(smem_dst, map, x, y, bar);
    return;
  }
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], "
      "[%4], %5;" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tc_mma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tc_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128
// bytes with the 128-byte swizzle (what the TMA box load produces): 8-row groups are
// 1024 bytes apart (stride byte offset), the leading byte offset is unused for
// swizzled K-major layouts (encoded 1), descriptor version 1 (sm_100), layout type 2.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// The same for an MN-major operand tile: the TMA box is [K rows] x [128 bytes of M (or N)], so one
// 128-byte row holds 128 consecutive M/N positions of one k and eight k rows make one 1024-byte
// swizzle atom.  Stride byte offset = distance between groups of eight k rows (1024), leading byte
// offset = distance between blocks of 128 M/N positions (`mn_block_bytes`, one box).  One MMA
// (K = 32) spans four atoms; the next one starts 32 rows = 4096 bytes further on.
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t smem_addr, uint32_t mn_block_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((mn_block_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Operand layouts travel in bits 24 (A) and 25 (B) of the packed `raster` word: 0 = K-major
// (storage [rows, K], K contiguous), 1 = MN-major (storage [K, rows], rows contiguous).
constexpr int LAYOUT_A_MN_BIT = 24;
constexpr int LAYOUT_B_MN_BIT = 25;
constexpr int EPI_ALL_POLL_BIT = 29;  // pair kernels: every epilogue warp polls the accumulator barrier itself (the earlier scheme)
constexpr int WAIT_SLEEP_BIT = 28;  // 512x256 pair kernel: waits sleep between probes (or spin) instead of passing a suspend-time hint
// Encoded-address step between consecutive K = 32 MMAs inside one 128-wide k-block.
__device__ __forceinline__ uint64_t desc_k_step(bool mn_major) {
  return mn_major ? (uint64_t)((UMMA_K * 128) >> 4) : (uint64_t)(UMMA_K >> 4);
}

// Instruction descriptor for kind::f8f6f4: fp32 accumulate, A/B formats
// (0 = e4m3, 1 = e5m2), both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(int a_kind, int b_kind) {
  return (1u << 4) | ((uint32_t)a_kind << 7) | ((uint32_t)b_kind << 10) | ((uint32_t)(BN >> 3) << 17) |
         ((uint32_t)(BM >> 4) << 24);
}

struct TileCoord {
  int m, n;
};
// Tile order for L2 reuse.  Tiles are visited in bands of `group` tiles along one
// dimension (M when along_n == 0), fastest inside the band, then along the other
// dimension.  The CTAs running at the same time then share one operand panel
// (group x K bytes, sized on the host to stay in L2) while the other operand streams by.
// `raster` packs group (low 16 bits) and along_n (bit 16).
__device__ __forceinline__ TileCoord tile_coord(int64_t idx, int tiles_m, int tiles_n, int raster) {
  const int group = raster & 0xFFFF;
  const bool along_n = (raster >> 16) & 1;
  const int t_band = along_n ? tiles_n : tiles_m;   // dimension cut into bands
  const int t_other = along_n ? tiles_m : tiles_n;
  const int64_t per_group = (int64_t)group * t_other;
  const int g = (int)(idx / per_group);
  const int first = g * group;
  const int gsz = min(group, t_band - first);
  const int64_t in_g = idx - (int64_t)g * per_group;
  const int a = first + (int)(in_g % gsz);
  const int b = (int)(in_g / gsz);
  TileCoord c;
  c.m = along_n ? b : a;
  c.n = along_n ? a : b;
  return c;
}

// ---- dynamic tile scheduling ---------------------------------------------------
// With a scheduling word (`sched`, one uint32 in global memory that the host zeroes before the
// launch) the persistent CTAs do not walk a fixed stride of tiles: a CTA (or CTA pair) starts on the
// tile of its own index and then claims tiles num_units + atomicAdd(sched, 1).  A CTA that gets its SM
// late, because a kernel on another stream (a collective) held it, then simply does fewer tiles, where
// the fixed stride would make the whole GEMM wait for it.  The TMA producer thread claims the next
// tile a few k-blocks before the end of the current one and publishes it to the other roles through
// a small ring in shared memory: ring.tile[j % RING] holds the (j+1)-th tile of this CTA, or -1 when
// there is none, and ring.full[j % RING] completes once per publication.  The ring needs no "empty"
// barrier, because the producer cannot lap its readers: it publishes entry j right after issuing the
// last loads of its j-th tile, and it could issue those only after the MMA thread had consumed a
// k-block at most `stages` (<= 6) k-blocks, hence at most 6 tiles, earlier.  The MMA thread starts a
// tile only after the epilogue warps have drained the tile two (one, in the wide kernel) before it,
// and every role reads entry i straight after its work on tile i.  So when entry j is written every
// reader has read entry j - 9 or later, and RING = 16 entries are never overwritten unread.
constexpr int RING = 16;
struct TileRing {
  uint64_t full[RING];
  int32_t tile[RING];
};

template <typename OutT>
__device__ __forceinline__ void store_chunk(OutT* dst, const float (&v)[32], int ncols, bool vec_ok) {
  if constexpr (sizeof(OutT) == 2) {
    if (vec_ok && ncols == 32) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          OutT lo = static_cast<OutT>(v[q * 8 + 2 * e]), hi = static_cast<OutT>(v[q * 8 + 2 * e + 1]);
          w[e] = (uint32_t)(*reinterpret_cast<unsigned short*>(&lo)) |
                 ((uint32_t)(*reinterpret_cast<unsigned short*>(&hi)) << 16);
        }
        *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      return;
    }
  } else {
    if (vec_ok && ncols == 32) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<float4*>(dst + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
      return;
    }
  }
  for (int e = 0; e < 32; ++e)
    if (e < ncols) dst[e] = static_cast<OutT>(v[e]);
}

// ---- epilogue: accumulator -> scaled output ---------------------------------
// Each epilogue warp owns 32 accumulator rows.  Preferred path: the warp converts 32
// columns at a time, writes them into a 128-byte-swizzled staging box in shared memory
// (32 rows x 128 bytes) and one lane hands the box to a TMA store, so the output leaves
// the SM as full 128-byte lines and rows/columns beyond M/N are clipped by the tensor
// map.  Two boxes per warp alternate so conversion overlaps the stores.  The direct path
// (16-byte stores per thread) is used when the output does not meet TMA alignment.
constexpr int EPI_BOX_BYTES = 32 * 128;
constexpr int EPI_STAGING_BYTES = 4 /*warps*/ * 2 /*boxes*/ * EPI_BOX_BYTES;

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* map, const void* smem_src, int x, int y,
                                                  uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Row scatter of the output (used by the GEMM whose epilogue is the first half of a reduce-scatter):
// output row i belongs to block i / rows_per_block; blocks go round-robin to the n destinations, so
// row i lands in destination (block % n) at row (block / n) * rows_per_block + i % rows_per_block.
// The destinations may be buffers of other GPUs mapped into this process (plain stores over NVLink).
constexpr int MAX_SCATTER = 16;
struct RowScatter {
  void* base[MAX_SCATTER];
  int n;
  int rows_per_block;
};
struct NoScatter {};

template <typename OutT>
__device__ __forceinline__ OutT* scatter_row_ptr(const RowScatter& sc, int row, int64_t ldo) {
  const int blk = row / sc.rows_per_block;
  const int within = row - blk * sc.rows_per_block;
  const int owner = blk % sc.n;
  return static_cast<OutT*>(sc.base[owner]) + ((int64_t)(blk / sc.n) * sc.rows_per_block + within) * ldo;
}

template <typename OutT>
struct EpilogueArgs {
  const OutT* bias;
  OutT* out;
  int64_t ldo;
  int m, n;
  int out_vec_ok;
  int use_tma;
  const CUtensorMap* tma_out;
  uint8_t* staging;  // this warp's two boxes, 1024-byte aligned
  float inv;
  int store_evict_first;  // the output is not read again by this kernel: do not let it displace operands in L2
  const RowScatter* scatter;  // rows go to several destinations (per-thread and warp-written store paths); null = `out`
};

// Drains `ncol_total` accumulator columns starting at TMEM address `taddr` for the 32
// rows row0..row0+31 (lane = row).  `boxes` counts the TMA boxes this warp has issued so
// far (selects the staging box and tells how many stores may still be reading it).
template <typename OutT>
__device__ __forceinline__ void drain_accumulator(const EpilogueArgs<OutT>& e, uint32_t taddr, int row0, int col0,
                                                  int ncol_total, uint32_t& boxes) {
  constexpr int COLS_PER_BOX = 128 / (int)sizeof(OutT);  // 64 (16-bit) or 32 (fp32)
  constexpr int CHUNKS_PER_BOX = COLS_PER_BOX / 32;      // tcgen05.ld chunks of 32 columns
  const int lane = threadIdx.x & 31;
  const int row = row0 + lane;
#pragma unroll 1
  for (int c = 0; c < ncol_total / 32; ++c) {
    uint32_t r[32];
    tc_ld_32x32b_x32(taddr + (uint32_t)(c * 32), r);
    tc_wait_ld();
    const int col = col0 + c * 32;
    int ncols = e.n - col;
    if (ncols > 32) ncols = 32;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * e.inv;
    if (e.bias != nullptr && ncols > 0) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ncols) v[i] += static_cast<float>(e.bias[col + i]);
    }
    if (!e.use_tma) {
      if (row < e.m && ncols > 0) store_chunk<OutT>(e.out + (int64_t)row * e.ldo + col, v, ncols, e.out_vec_ok != 0);
      continue;
    }
    const int sub = c % CHUNKS_PER_BOX;  // which 32-column part of the box
    // boxes that start beyond the matrix are skipped altogether (uniform over the warp);
    // partial ones are clipped by the tensor map
    if (col - sub * 32 >= e.n || row0 >= e.m) continue;
    uint8_t* box = e.staging + (boxes & 1u) * EPI_BOX_BYTES;
    if (sub == 0 && boxes >= 2u) {
      // the store issued two boxes ago (same staging box) must have finished reading it
      if (lane == 0) bulk_wait_read<1>();
      __syncwarp();
    }
    // row `lane` of the box is 128 bytes = eight 16-byte chunks; chunk j lives at j ^ (lane & 7)
    uint8_t* rowp = box + lane * 128;
    if constexpr (sizeof(OutT) == 2) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t w[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          OutT lo = static_cast<OutT>(v[q * 8 + 2 * h]), hi = static_cast<OutT>(v[q * 8 + 2 * h + 1]);
          w[h] = (uint32_t)(*reinterpret_cast<unsigned short*>(&lo)) |
                 ((uint32_t)(*reinterpret_cast<unsigned short*>(&hi)) << 16);
        }
        const int j = sub * 4 + q;
        *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        *reinterpret_cast<float4*>(rowp + ((q ^ (lane & 7)) << 4)) =
            make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
      }
    }
    if (sub == CHUNKS_PER_BOX - 1) {
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (e.store_evict_first) tma_store_2d_hint(e.tma_out, box, col - sub * 32, row0, l2_policy(1));
        else tma_store_2d(e.tma_out, box, col - sub * 32, row0);
        bulk_commit();
      }
      ++boxes;
    }
  }
}

template <typename OutT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                const __grid_constant__ CUtensorMap tma_out, const float* __restrict__ scale_a,
                const float* __restrict__ scale_b, const OutT* __restrict__ bias, OutT* __restrict__ out, int64_t ldo,
                int m, int n, int k, uint32_t idesc, int out_vec_ok, int use_tma_store, int raster) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = tiles + STAGES * STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(staging + EPI_STAGING_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (m + BM - 1) / BM, tiles_n = (n + BN - 1) / BN;
  const int64_t num_tiles = (int64_t)tiles_m * tiles_n;
  const int num_kb = (k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 4);
    }
    bars->abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_b)) : "memory");
      // raster bit 16: bands run along N (B is the resident panel, A streams), else along M.
      // hint bits: 21 = streaming operand evict-first, 22 = panel operand evict-last.
      const bool panel_is_b = (raster >> 16) & 1;
      const int pol_panel = ((raster >> 22) & 1) ? 2 : 0, pol_stream = ((raster >> 21) & 1) ? 1 : 0;
      const uint64_t pol_a = l2_policy(panel_is_b ? pol_stream : pol_panel);
      const uint64_t pol_b = l2_policy(panel_is_b ? pol_panel : pol_stream);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n, raster);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1u, bars, 1u, 64u)) { ok = false; break; }
          uint8_t* sa = tiles + stage * STAGE_BYTES;
          mbar_expect_tx(&bars->full[stage], STAGE_BYTES);
          tma_load_2d_hint(sa, &tma_a, kb * BK, tc.m * BM, &bars->full[stage], pol_a);
          tma_load_2d_hint(sa + A_BYTES, &tma_b, kb * BK, tc.n * BN, &bars->full[stage], pol_b);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // let bulk copies already in flight land before the CTA's shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int64_t local = 0;
      for (int64_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x, ++local) {
        const int acc = (int)(local & 1);
        const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1u, bars, 2u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, bars, 4u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * STAGE_BYTES);
          const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(a_addr + A_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // advancing 32 bytes along K inside the swizzle span = +2 in the 16-byte address field
            tc_mma_f8(tmem_d, da + (uint64_t)(kk * (UMMA_K >> 4)), db + (uint64_t)(kk * (UMMA_K >> 4)), idesc,
                      (kb | kk) != 0 ? 1u : 0u);
          }
          tc_commit(&bars->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc_commit(&bars->tmem_full[acc]);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
    float inv = 0.f;
    {
      const float sa = __ldg(scale_a), sb = __ldg(scale_b);
      inv = __fmul_rn(__fdiv_rn(1.0f, sa), __fdiv_rn(1.0f, sb));
    }
    const EpilogueArgs<OutT> ea{bias, out, ldo, m, n, out_vec_ok, use_tma_store, &tma_out,
                                staging + (warp - 2) * 2 * EPI_BOX_BYTES, inv, (raster >> 20) & 1};
    uint32_t boxes = 0;
    bool ok = true;
    int64_t local = 0;
    for (int64_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x, ++local) {
      const TileCoord tc = tile_coord(t, tiles_m, tiles_n, raster);
      const int acc = (int)(local & 1);
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      // one lane polls, the rest of the warp sleeps at the shuffle
      int got = 1;
      if (lane == 0) got = mbar_wait(&bars->tmem_full[acc], acc_phase, bars, 8u, 256u) ? 1 : 0;
      if (__shfl_sync(0xFFFFFFFFu, got, 0) == 0) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
      drain_accumulator<OutT>(ea, taddr, tc.m * BM + quarter * 32, tc.n * BN, BN, boxes);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
    }
    if (use_tma_store && lane == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// ===========================================================================
// Wide one-CTA variant: one CTA per 256x256 output tile, no cluster.  Each k-step issues
// two M128 N256 K32 MMAs that share the B operand in this CTA's own shared memory; the
// two 128-row halves accumulate in TMEM columns 0..255 and 256..511 (all of TMEM, so the
// accumulator is not double buffered: the epilogue of a tile is exposed, but it is split
// over two groups of four warps, one per half).  Per flop this moves as many bytes from
// L2 as the two-CTA kernel and none between SMs.
// ===========================================================================
namespace wide {

constexpr int WBM = 256;
constexpr int WBN = 256;
constexpr int WSTAGES = 3;
constexpr int WA_BYTES = WBM * BK;  // 32 KB: rows 0..127 then 128..255
constexpr int WB_BYTES = WBN * BK;  // 32 KB
constexpr int WSTAGE_BYTES = WA_BYTES + WB_BYTES;
constexpr int WTHREADS = 320;  // TMA warp, MMA warp, 2 x 4 epilogue warps

struct __align__(8) WideBarriers {
  uint64_t full[WSTAGES];
  uint64_t empty[WSTAGES];
  uint64_t tmem_full;
  uint64_t tmem_empty;
  TileRing ring;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

// 3 x 64 KB stages + 8 warps x 1 box x 4 KB would fit two boxes only with 2 stages; one box
// per warp is enough here because a warp's stores are waited for before the box is reused.
constexpr int WSMEM_BYTES = WSTAGES * WSTAGE_BYTES + 8 * EPI_BOX_BYTES + 1024 + (int)sizeof(WideBarriers);

__device__ __forceinline__ bool wide_wait(uint64_t* bar, uint32_t parity, WideBarriers* bars, uint32_t who,
                                          uint32_t backoff_ns = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 0; it < 0x7FFFFFFFu; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (backoff_ns != 0u) __nanosleep(backoff_ns);
    if ((it & 63u) == 63u) {
      if (bars->abort_flag != 0u) return false;
      if (clock64() - t0 > WAIT_BUDGET_CYCLES) break;
    }
  }
  bars->abort_flag = 1u;
  atomicOr(&g_device_error, who | 0x200u);
  return false;
}

__host__ __device__ constexpr uint32_t make_idesc_wide(int a_kind, int b_kind, int a_mn = 0, int b_mn = 0) {
  return (1u << 4) | ((uint32_t)a_kind << 7) | ((uint32_t)b_kind << 10) | ((uint32_t)a_mn << 15) |
         ((uint32_t)b_mn << 16) | ((uint32_t)(WBN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// Like drain_accumulator, with ONE staging box per warp (the previous store of this warp
// has to finish reading the box before it is refilled).
template <typename OutT>
__device__ __forceinline__ void drain_accumulator_1box(const EpilogueArgs<OutT>& e, uint32_t taddr, int row0, int col0,
                                                       int ncol_total, uint32_t& boxes) {
  constexpr int COLS_PER_BOX = 128 / (int)sizeof(OutT);
  constexpr int CHUNKS_PER_BOX = COLS_PER_BOX / 32;
  const int lane = threadIdx.x & 31;
  const int row = row0 + lane;
#pragma unroll 1
  for (int c = 0; c < ncol_total / 32; ++c) {
    uint32_t r[32];
    tc_ld_32x32b_x32(taddr + (uint32_t)(c * 32), r);
    tc_wait_ld();
    const int col = col0 + c * 32;
    int ncols = e.n - col;
    if (ncols > 32) ncols = 32;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * e.inv;
    if (e.bias != nullptr && ncols > 0) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ncols) v[i] += static_cast<float>(e.bias[col + i]);
    }
    if (!e.use_tma) {
      if (row < e.m && ncols > 0) {
        OutT* dst = e.scatter != nullptr ? scatter_row_ptr<OutT>(*e.scatter, row, e.ldo) : e.out + (int64_t)row * e.ldo;
        store_chunk<OutT>(dst + col, v, ncols, e.out_vec_ok != 0);
      }
      continue;
    }
    const int sub = c % CHUNKS_PER_BOX;
    if (col - sub * 32 >= e.n || row0 >= e.m) continue;
    uint8_t* box = e.staging;
    if (sub == 0 && boxes >= 1u) {
      if (lane == 0) bulk_wait_read<0>();
      __syncwarp();
    }
    uint8_t* rowp = box + lane * 128;
    if constexpr (sizeof(OutT) == 2) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t w[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          OutT lo = static_cast<OutT>(v[q * 8 + 2 * h]), hi = static_cast<OutT>(v[q * 8 + 2 * h + 1]);
          w[h] = (uint32_t)(*reinterpret_cast<unsigned short*>(&lo)) |
                 ((uint32_t)(*reinterpret_cast<unsigned short*>(&hi)) << 16);
        }
        const int j = sub * 4 + q;
        *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        *reinterpret_cast<float4*>(rowp + ((q ^ (lane & 7)) << 4)) =
            make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
      }
    }
    if (sub == CHUNKS_PER_BOX - 1) {
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (e.store_evict_first) tma_store_2d_hint(e.tma_out, box, col - sub * 32, row0, l2_policy(1));
        else tma_store_2d(e.tma_out, box, col - sub * 32, row0);
        bulk_commit();
      }
      ++boxes;
    }
  }
}

// 16-bit outputs: the warp's 4 KB of staging holds TWO boxes of 32 rows x 64 bytes (64-byte swizzle),
// one per 32-column chunk, which alternate: the store of chunk c is in flight while chunk c+1 is
// converted, and only the store issued two chunks ago has to have finished reading its box.  With a
// single 128-byte box the warp stalled on every second chunk for its own store, and in these
// kernels nothing hides the epilogue (the accumulator fills all of TMEM).
// One 32-column chunk of the half-box epilogue: scale, bias, convert, stage in this warp's next box and
// hand the box to a TMA store.
template <typename OutT>
__device__ __forceinline__ void halfbox_emit(const EpilogueArgs<OutT>& e, const uint32_t (&r)[32], int row0, int col,
                                             uint32_t& boxes) {
  const int lane = threadIdx.x & 31;
  int ncols = e.n - col;
  if (ncols > 32) ncols = 32;
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * e.inv;
  if (e.bias != nullptr) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < ncols) v[i] += static_cast<float>(e.bias[col + i]);
  }
  uint8_t* box = e.staging + (boxes & 1u) * (EPI_BOX_BYTES / 2);
  if (boxes >= 2u) {
    if (lane == 0) bulk_wait_read<1>();
    __syncwarp();
  }
  // row `lane` of the box is 64 bytes = four 16-byte chunks; chunk j lives at j ^ ((lane >> 1) & 3)
  uint8_t* rowp = box + lane * 64;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t w[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      OutT lo = static_cast<OutT>(v[q * 8 + 2 * h]), hi = static_cast<OutT>(v[q * 8 + 2 * h + 1]);
      w[h] = (uint32_t)(*reinterpret_cast<unsigned short*>(&lo)) |
             ((uint32_t)(*reinterpret_cast<unsigned short*>(&hi)) << 16);
    }
    *reinterpret_cast<uint4*>(rowp + ((q ^ ((lane >> 1) & 3)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  fence_async_smem();
  __syncwarp();
  if (lane == 0) {
    if (e.store_evict_first) tma_store_2d_hint(e.tma_out, box, col, row0, l2_policy(1));
    else tma_store_2d(e.tma_out, box, col, row0);
    bulk_commit();
  }
  ++boxes;
}

// 16-bit outputs: the warp's 4 KB of staging holds TWO boxes of 32 rows x 64 bytes (64-byte swizzle),
// one per 32-column chunk, which alternate: the store of chunk c is in flight while chunk c+1 is
// converted, and only the store issued two chunks ago has to have finished reading its box.  The
// tensor-memory loads are software pipelined as well: the load of chunk c+1 is issued before chunk c is
// converted (two register sets in turn), because in these kernels nothing else hides the epilogue
// (the accumulator fills all of tensor memory).
template <typename OutT>
__device__ __forceinline__ void drain_accumulator_halfbox(const EpilogueArgs<OutT>& e, uint32_t taddr, int row0,
                                                          int col0, int ncol_total, uint32_t& boxes) {
  static_assert(sizeof(OutT) == 2, "half boxes are for 16-bit outputs");
  if (row0 >= e.m) return;  // uniform over the warp
  int nch = ncol_total / 32;
  const int avail = (e.n - col0 + 31) / 32;  // chunks that start inside the matrix
  if (avail < nch) nch = avail;
  if (nch <= 0) return;
  uint32_t ra[32], rb[32];
  tc_ld_32x32b_x32(taddr, ra);
#pragma unroll 1
  for (int c = 0; c < nch; c += 2) {
    tc_wait_ld();
    if (c + 1 < nch) tc_ld_32x32b_x32(taddr + (uint32_t)((c + 1) * 32), rb);
    halfbox_emit<OutT>(e, ra, row0, col0 + c * 32, boxes);
    if (c + 1 < nch) {
      tc_wait_ld();
      if (c + 2 < nch) tc_ld_32x32b_x32(taddr + (uint32_t)((c + 2) * 32), ra);
      halfbox_emit<OutT>(e, rb, row0, col0 + (c + 1) * 32, boxes);
    }
  }
}

// Coalesced store path without TMA (`use_tma` == 2): every round covers one 128-byte line per row (64
// columns of a 16-bit output, 32 of fp32).  Each lane converts its row's part and stages it in the warp's
// own 32 x 128-byte box (16-byte pieces XOR-swizzled by row, conflict-free both ways); after a warp
// barrier the warp writes the box out four rows per instruction, eight lanes per row, so every store
// instruction fills whole 128-byte lines.  The tensor-memory load of the next round is issued before the
// write-out of the current one.  This path exists because a TMA store issued while the producer is
// prefetching the next tile queues behind up to 190 KB of operand loads in the same TMA unit: measured,
// a 2 KB box took ~1100 cycles from hand-over to "box may be reused", 4500 cycles per accumulator half.
template <typename OutT>
__device__ __forceinline__ void drain_accumulator_coalesced(const EpilogueArgs<OutT>& e, uint32_t taddr, int row0,
                                                            int col0, int ncol_total) {
  constexpr int ESZ = (int)sizeof(OutT);
  constexpr int CPR = 128 / ESZ;  // columns per round
  constexpr int CH = CPR / 32;    // 32-column tensor-memory chunks per round
  constexpr int PIECE = 16 / ESZ; // columns per 16-byte piece
  const int lane = threadIdx.x & 31;
  if (row0 >= e.m || col0 >= e.n) return;  // uniform over the warp
  uint8_t* box = e.staging;
  uint32_t r[CH][32];
#pragma unroll
  for (int ch = 0; ch < CH; ++ch) tc_ld_32x32b_x32(taddr + (uint32_t)(ch * 32), r[ch]);
#pragma unroll 1
  for (int c0 = 0; c0 < ncol_total; c0 += CPR) {
    const int col = col0 + c0;
    tc_wait_ld();
    uint8_t* rowp = box + lane * 128;
#pragma unroll
    for (int ch = 0; ch < CH; ++ch) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[ch][i]) * e.inv;
      if (e.bias != nullptr) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (col + ch * 32 + i < e.n) v[i] += static_cast<float>(e.bias[col + ch * 32 + i]);
      }
      if constexpr (ESZ == 2) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t w[4];
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            OutT lo = static_cast<OutT>(v[q * 8 + 2 * h]), hi = static_cast<OutT>(v[q * 8 + 2 * h + 1]);
            w[h] = (uint32_t)(*reinterpret_cast<unsigned short*>(&lo)) |
                   ((uint32_t)(*reinterpret_cast<unsigned short*>(&hi)) << 16);
          }
          const int j = ch * 4 + q;
          *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<float4*>(rowp + ((q ^ (lane & 7)) << 4)) =
              make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
      }
    }
    const bool more = c0 + CPR < ncol_total && col + CPR < e.n;
    if (more) {
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) tc_ld_32x32b_x32(taddr + (uint32_t)(c0 + CPR + ch * 32), r[ch]);
    }
    __syncwarp();
    const int p = lane & 7;
    const int gcol = col + p * PIECE;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = i * 4 + (lane >> 3);
      const uint4 val = *reinterpret_cast<const uint4*>(box + rr * 128 + ((p ^ (rr & 7)) << 4));
      const int grow = row0 + rr;
      if (grow < e.m && gcol < e.n) {
        OutT* dst = (e.scatter != nullptr ? scatter_row_ptr<OutT>(*e.scatter, grow, e.ldo) : e.out + (int64_t)grow * e.ldo) + gcol;
        if (gcol + PIECE <= e.n) {
          __stcs(reinterpret_cast<uint4*>(dst), val);
        } else {
          const OutT* src = reinterpret_cast<const OutT*>(&val);
          for (int k2 = 0; k2 < PIECE && gcol + k2 < e.n; ++k2) dst[k2] = src[k2];
        }
      }
    }
    __syncwarp();  // the box is refilled in the next round
    if (!more) break;
  }
}

// Epilogue of the kernels whose accumulator fills TMEM: half boxes for 16-bit outputs when the TMA
// store path is on (`use_tma` then means the output map was encoded with half boxes).
template <typename OutT>
__device__ __forceinline__ void drain_wide(const EpilogueArgs<OutT>& e, uint32_t taddr, int row0, int col0,
                                           int ncol_total, uint32_t& boxes) {
  if (e.use_tma == 2) {
    drain_accumulator_coalesced<OutT>(e, taddr, row0, col0, ncol_total);
    return;
  }
  if constexpr (sizeof(OutT) == 2) {
    if (e.use_tma) {
      drain_accumulator_halfbox<OutT>(e, taddr, row0, col0, ncol_total, boxes);
      return;
    }
  }
  drain_accumulator_1box<OutT>(e, taddr, row0, col0, ncol_total, boxes);
}

template <typename OutT>
__global__ void __launch_bounds__(WTHREADS, 1)
gemm_fp8_wide_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                     const __grid_constant__ CUtensorMap tma_out, const float* __restrict__ scale_a,
                     const float* __restrict__ scale_b, const OutT* __restrict__ bias, OutT* __restrict__ out,
                     int64_t ldo, int m, int n, int k, uint32_t idesc, int out_vec_ok, int use_tma_store, int raster,
                     uint32_t* sched) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = tiles + WSTAGES * WSTAGE_BYTES;
  WideBarriers* bars = reinterpret_cast<WideBarriers*>(staging + 8 * EPI_BOX_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (m + WBM - 1) / WBM, tiles_n = (n + WBN - 1) / WBN;
  const int64_t num_tiles = (int64_t)tiles_m * tiles_n;
  const int num_kb = (k + BK - 1) / BK;
  const bool a_mn = (raster >> LAYOUT_A_MN_BIT) & 1, b_mn = (raster >> LAYOUT_B_MN_BIT) & 1;
  const uint64_t step_a = desc_k_step(a_mn), step_b = desc_k_step(b_mn);

  if (threadIdx.x == 0) {
    for (int s = 0; s < WSTAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->tmem_full, 1);
    mbar_init(&bars->tmem_empty, 8);
    for (int r = 0; r < RING; ++r) mbar_init(&bars->ring.full[r], 1);
    bars->abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_b)) : "memory");
      const uint64_t pol = l2_policy(0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int claim_kb = num_kb > 4 ? num_kb - 4 : 0;
      uint32_t published = 0;
      int64_t t = blockIdx.x;
      while (ok && t < num_tiles) {
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n, raster);
        int64_t next = t + gridDim.x;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (sched != nullptr && kb == claim_kb) next = (int64_t)gridDim.x + (int64_t)atomicAdd(sched, 1u);
          if (!wide_wait(&bars->empty[stage], phase ^ 1u, bars, 1u, 64u)) { ok = false; break; }
          uint8_t* sa = tiles + stage * WSTAGE_BYTES;
          mbar_expect_tx(&bars->full[stage], WSTAGE_BYTES);
          if (!a_mn) {
            tma_load_2d_hint(sa, &tma_a, kb * BK, tc.m * WBM, &bars->full[stage], pol);  // one box of 256 rows
          } else {  // two boxes of [128 k rows] x [128 M positions]
            tma_load_2d_hint(sa, &tma_a, tc.m * WBM, kb * BK, &bars->full[stage], pol);
            tma_load_2d_hint(sa + 128 * BK, &tma_a, tc.m * WBM + 128, kb * BK, &bars->full[stage], pol);
          }
          if (!b_mn) {
            tma_load_2d_hint(sa + WA_BYTES, &tma_b, kb * BK, tc.n * WBN, &bars->full[stage], pol);
          } else {
            tma_load_2d_hint(sa + WA_BYTES, &tma_b, tc.n * WBN, kb * BK, &bars->full[stage], pol);
            tma_load_2d_hint(sa + WA_BYTES + 128 * BK, &tma_b, tc.n * WBN + 128, kb * BK, &bars->full[stage], pol);
          }
          if (++stage == WSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (sched != nullptr) {
          const uint32_t slot = published & (RING - 1);
          bars->ring.tile[slot] = next < num_tiles ? (int32_t)next : -1;
          mbar_arrive(&bars->ring.full[slot]);  // release: the entry is visible to whoever sees the phase
          ++published;
        }
        t = next;
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int64_t local = 0;
      int64_t t = blockIdx.x;
      for (; ok && t < num_tiles; ++local) {
        if (!wide_wait(&bars->tmem_empty, (uint32_t)(local & 1) ^ 1u, bars, 2u)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wide_wait(&bars->full[stage], phase, bars, 4u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * WSTAGE_BYTES);
          const uint64_t da0 = a_mn ? make_smem_desc_mn(a_addr, 128 * BK) : make_smem_desc(a_addr);
          const uint64_t da1 = a_mn ? make_smem_desc_mn(a_addr + 128 * BK, 128 * BK) : make_smem_desc(a_addr + 128 * BK);
          const uint64_t db = b_mn ? make_smem_desc_mn(a_addr + WA_BYTES, 128 * BK) : make_smem_desc(a_addr + WA_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t off_a = (uint64_t)kk * step_a, off_b = (uint64_t)kk * step_b;
            const uint32_t accum = (kb | kk) != 0 ? 1u : 0u;
            tc_mma_f8(tmem_base, da0 + off_a, db + off_b, idesc, accum);
            tc_mma_f8(tmem_base + 256u, da1 + off_a, db + off_b, idesc, accum);
          }
          tc_commit(&bars->empty[stage]);
          if (++stage == WSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(&bars->tmem_full);
        if (sched != nullptr) {
          const uint32_t slot = (uint32_t)local & (RING - 1);
          if (!wide_wait(&bars->ring.full[slot], (uint32_t)(local >> 4) & 1u, bars, 16u)) { ok = false; break; }
          const int32_t v = *reinterpret_cast<volatile int32_t*>(&bars->ring.tile[slot]);
          t = v < 0 ? num_tiles : (int64_t)v;
        } else {
          t += gridDim.x;
        }
      }
    }
  } else {
    // warps 2..5 drain rows 0..127 (TMEM columns 0..255), warps 6..9 rows 128..255 (columns 256..511)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    float inv = 0.f;
    {
      const float sa = __ldg(scale_a), sb = __ldg(scale_b);
      inv = __fmul_rn(__fdiv_rn(1.0f, sa), __fdiv_rn(1.0f, sb));
    }
    const EpilogueArgs<OutT> ea{bias, out, ldo, m, n, out_vec_ok, use_tma_store, &tma_out,
                                staging + (warp - 2) * EPI_BOX_BYTES, inv, (raster >> 20) & 1};
    uint32_t boxes = 0;
    bool ok = true;
    int64_t local = 0;
    int64_t t = blockIdx.x;
    for (; ok && t < num_tiles; ++local) {
      const TileCoord tc = tile_coord(t, tiles_m, tiles_n, raster);
      int got = 1;
      if (lane == 0) got = wide_wait(&bars->tmem_full, (uint32_t)(local & 1), bars, 8u, 256u) ? 1 : 0;
      if (__shfl_sync(0xFFFFFFFFu, got, 0) == 0) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 256);
      drain_wide<OutT>(ea, taddr, tc.m * WBM + half * 128 + quarter * 32, tc.n * WBN, WBN, boxes);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty);
      if (sched != nullptr) {
        int v = -2;  // -2: gave up waiting
        if (lane == 0) {
          const uint32_t slot = (uint32_t)local & (RING - 1);
          if (wide_wait(&bars->ring.full[slot], (uint32_t)(local >> 4) & 1u, bars, 32u, 64u))
            v = *reinterpret_cast<volatile int32_t*>(&bars->ring.tile[slot]);
        }
        v = __shfl_sync(0xFFFFFFFFu, v, 0);
        if (v == -2) { ok = false; break; }
        t = v < 0 ? num_tiles : (int64_t)v;
      } else {
        t += gridDim.x;
      }
    }
    if (use_tma_store == 1 && lane == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

}  // namespace wide

// ===========================================================================
// Two-CTA variant: a cluster of two CTAs (two SMs) works on one 256x256 output tile
// with tcgen05.mma.cta_group::2 (instruction shape M256 N256 K32).  CTA r of the pair
// loads rows [128r, 128r+128) of the A tile and rows [128r, 128r+128) of the B tile, so
// each SM stages 32 KB per k-block instead of 48 KB and the tensor core of each SM reads
// half of B from its partner's shared memory.  Only the pair's leader (rank 0) issues
// MMAs.  Cross-CTA signalling:
//   full[s]        lives in the leader; both CTAs' TMA loads complete_tx on it
//   empty[s]       one per CTA; released by a multicast tcgen05.commit from the leader
//   tmem_full[a]   one per CTA; same multicast commit when a tile's MMAs are done
//   tmem_empty[a]  lives in the leader; 8 arrivals (4 epilogue warps of each CTA)
// No TMA load here uses cluster multicast: every CTA fetches its own boxes.
// ===========================================================================
namespace pair {

constexpr int PBM = 256;  // rows of the pair tile (128 per CTA)
constexpr int PBN = 256;  // columns of the pair tile (each CTA stages 128 of B's rows)
constexpr int PSTAGES = 6;
constexpr int PA_BYTES = 128 * BK;
constexpr int PB_BYTES = 128 * BK;
constexpr int PSTAGE_BYTES = PA_BYTES + PB_BYTES;

struct __align__(8) PairBarriers {
  uint64_t full[PSTAGES];
  uint64_t empty[PSTAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  TileRing ring;  // written in both CTAs by the leader's producer thread
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

constexpr int PSMEM_BYTES = PSTAGES * PSTAGE_BYTES + EPI_STAGING_BYTES + 1024 + (int)sizeof(PairBarriers);

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t cta_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Arrive that publishes this thread's earlier stores (also those to the partner's shared memory) to a
// waiter in the partner CTA.
__device__ __forceinline__ void mbar_arrive_release_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_acquire_cluster_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_acquire_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// The same load without an L2 cache-hint operand (default L2 policy).
__device__ __forceinline__ void tma_load_2d_pair_plain(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                       uint32_t mbar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(mbar_cluster_addr)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t mbar_cluster_addr, uint64_t policy) {
  if (policy == 0) {  // default L2 policy: no hint operand (see l2_policy)
    tma_load_2d_pair_plain(smem_dst, map, x, y, mbar_cluster_addr);
    return;
  }
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(mbar_cluster_addr), "l"(policy)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once all
// MMAs issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__host__ __device__ constexpr uint32_t make_idesc_pair(int a_kind, int b_kind, int a_mn = 0, int b_mn = 0) {
  return (1u << 4) | ((uint32_t)a_kind << 7) | ((uint32_t)b_kind << 10) | ((uint32_t)a_mn << 15) |
         ((uint32_t)b_mn << 16) | ((uint32_t)(PBN >> 3) << 17) | ((uint32_t)(PBM >> 4) << 24);
}

// Bounded wait that also raises the partner's abort flag when it gives up.
template <bool CLUSTER_ACQUIRE = false, typename Bars = PairBarriers>
__device__ __forceinline__ bool pair_wait(uint64_t* bar, uint32_t parity, Bars* bars, uint32_t peer_rank,
                                          uint32_t who, uint32_t backoff_ns = 0) {
  const bool by_hint = (backoff_ns & WAIT_BY_HINT) != 0u;
  const uint32_t hint = backoff_ns & ~WAIT_BY_HINT;
  auto probe = [&]() {
    if (by_hint) return CLUSTER_ACQUIRE ? mbar_try_wait_acquire_cluster_hint(bar, parity, hint) : mbar_try_wait_hint(bar, parity, hint);
    return CLUSTER_ACQUIRE ? mbar_try_wait_acquire_cluster(bar, parity) : mbar_try_wait(bar, parity);
  };
  if (probe()) return true;
  const long long t0 = clock64();
  for (uint32_t it = 0; it < 0x7FFFFFFFu; ++it) {
    if (probe()) return true;
    if (backoff_ns != 0u && !by_hint) __nanosleep(backoff_ns);
    if ((it & 63u) == 63u) {
      if (bars->abort_flag != 0u) return false;
      if (clock64() - t0 > WAIT_BUDGET_CYCLES) break;
    }
  }
  bars->abort_flag = 1u;
  st_cluster_u32(mapa_u32(smem_u32(const_cast<uint32_t*>(&bars->abort_flag)), peer_rank), 1u);
  atomicOr(&g_device_error, who | 0x100u);
  return false;
}

// Entry `j` of this CTA's tile ring (the (j+1)-th tile of the pair): -1 = no more tiles, -2 = gave up.
template <typename Bars>
__device__ __forceinline__ int32_t pair_ring_read(Bars* bars, uint32_t j, uint32_t peer_rank, uint32_t who,
                                                  uint32_t backoff_ns) {
  const uint32_t slot = j & (RING - 1);
  if (!pair_wait<true>(&bars->ring.full[slot], (j >> 4) & 1u, bars, peer_rank, who, backoff_ns)) return -2;
  return *reinterpret_cast<volatile int32_t*>(&bars->ring.tile[slot]);
}

template <typename OutT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                     const __grid_constant__ CUtensorMap tma_out, const float* __restrict__ scale_a,
                     const float* __restrict__ scale_b, const OutT* __restrict__ bias, OutT* __restrict__ out,
                     int64_t ldo, int m, int n, int k, uint32_t idesc, int out_vec_ok, int use_tma_store, int raster,
                     uint32_t* sched) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = tiles + PSTAGES * PSTAGE_BYTES;
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(staging + EPI_STAGING_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t peer = rank ^ 1u;
  const bool leader = rank == 0;
  const int tiles_m = (m + PBM - 1) / PBM, tiles_n = (n + PBN - 1) / PBN;
  const int64_t num_tiles = (int64_t)tiles_m * tiles_n;
  const int num_kb = (k + BK - 1) / BK;
  const int64_t cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const bool a_mn = (raster >> LAYOUT_A_MN_BIT) & 1, b_mn = (raster >> LAYOUT_B_MN_BIT) & 1;
  const bool one_poller = ((raster >> EPI_ALL_POLL_BIT) & 1) == 0;
  const uint64_t step_a = desc_k_step(a_mn), step_b = desc_k_step(b_mn);

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 8);
    }
    for (int r = 0; r < RING; ++r) mbar_init(&bars->ring.full[r], 1);
    bars->abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA) ----------------
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_b)) : "memory");
      // raster bit 16: bands run along N (B is the resident panel, A streams), else along M.
      // hint bits: 21 = streaming operand evict-first, 22 = panel operand evict-last.
      const bool panel_is_b = (raster >> 16) & 1;
      const int pol_panel = ((raster >> 22) & 1) ? 2 : 0, pol_stream = ((raster >> 21) & 1) ? 1 : 0;
      const uint64_t pol_a = l2_policy(panel_is_b ? pol_stream : pol_panel);
      const uint64_t pol_b = l2_policy(panel_is_b ? pol_panel : pol_stream);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int claim_kb = num_kb > 4 ? num_kb - 4 : 0;
      uint32_t entry = 0;  // ring entries published (leader) or read (partner) so far
      int64_t t = cluster_id;
      while (ok && t < num_tiles) {
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n, raster);
        const int row_a = tc.m * PBM + (int)rank * 128;
        const int row_b = tc.n * PBN + (int)rank * 128;
        int64_t next = t + num_clusters;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (sched != nullptr && leader && kb == claim_kb) next = num_clusters + (int64_t)atomicAdd(sched, 1u);
          if (!pair_wait(&bars->empty[stage], phase ^ 1u, bars, peer, 1u, 64u)) { ok = false; break; }
          uint8_t* sa = tiles + stage * PSTAGE_BYTES;
          if (leader) mbar_expect_tx(&bars->full[stage], 2 * PSTAGE_BYTES);
          const uint32_t full_in_leader = mapa_u32(smem_u32(&bars->full[stage]), 0u);
          // K-major box: x = k offset, y = row; MN-major box: x = row (contiguous), y = k offset
          tma_load_2d_pair(sa, &tma_a, a_mn ? row_a : kb * BK, a_mn ? kb * BK : row_a, full_in_leader, pol_a);
          tma_load_2d_pair(sa + PA_BYTES, &tma_b, b_mn ? row_b : kb * BK, b_mn ? kb * BK : row_b, full_in_leader,
                           pol_b);
          if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (sched != nullptr) {
          if (leader) {
            const uint32_t slot = entry & (RING - 1);
            const int32_t v = next < num_tiles ? (int32_t)next : -1;
            bars->ring.tile[slot] = v;
            mbar_arrive(&bars->ring.full[slot]);
            st_cluster_u32(mapa_u32(smem_u32(&bars->ring.tile[slot]), 1u), (uint32_t)v);
            mbar_arrive_release_cluster(mapa_u32(smem_u32(&bars->ring.full[slot]), 1u));
          } else {
            const int32_t v = pair_ring_read(bars, entry, peer, 64u, 32u);
            if (v == -2) { ok = false; break; }
            next = v < 0 ? num_tiles : (int64_t)v;
          }
          ++entry;
        }
        t = next;
      }
      // tail: every release the leader multicast to this CTA's empty barriers has landed
      for (int s = 0; ok && s < PSTAGES; ++s) {
        if (!pair_wait(&bars->empty[stage], phase ^ 1u, bars, peer, 1u, 64u)) { ok = false; break; }
        if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int64_t local = 0;
      int64_t t = cluster_id;
      for (; ok && t < num_tiles; ++local) {
        const int acc = (int)(local & 1);
        const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
        if (!pair_wait(&bars->tmem_empty[acc], acc_phase ^ 1u, bars, peer, 2u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * PBN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!pair_wait(&bars->full[stage], phase, bars, peer, 4u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * PSTAGE_BYTES);
          const uint64_t da = a_mn ? make_smem_desc_mn(a_addr, PA_BYTES) : make_smem_desc(a_addr);
          const uint64_t db = b_mn ? make_smem_desc_mn(a_addr + PA_BYTES, PB_BYTES) : make_smem_desc(a_addr + PA_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            tc_mma_f8_pair(tmem_d, da + (uint64_t)kk * step_a, db + (uint64_t)kk * step_b, idesc,
                           (kb | kk) != 0 ? 1u : 0u);
          }
          tc_commit_pair(&bars->empty[stage]);
          if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit_pair(&bars->tmem_full[acc]);
        if (sched != nullptr) {
          const int32_t v = pair_ring_read(bars, (uint32_t)local, peer, 16u, 0u);
          if (v == -2) { ok = false; break; }
          t = v < 0 ? num_tiles : (int64_t)v;
        } else {
          t += num_clusters;
        }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
    const int quarter = warp & 3;
    float inv = 0.f;
    {
      const float sa = __ldg(scale_a), sb = __ldg(scale_b);
      inv = __fmul_rn(__fdiv_rn(1.0f, sa), __fdiv_rn(1.0f, sb));
    }
    const EpilogueArgs<OutT> ea{bias, out, ldo, m, n, out_vec_ok, use_tma_store, &tma_out,
                                staging + (warp - 2) * 2 * EPI_BOX_BYTES, inv, (raster >> 20) & 1};
    uint32_t boxes = 0;
    bool ok = true;
    int64_t local = 0;
    int64_t t = cluster_id;
    for (; ok && t < num_tiles; ++local) {
      const TileCoord tc = tile_coord(t, tiles_m, tiles_n, raster);
      const int acc = (int)(local & 1);
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      int got = 1;
      if (!one_poller || warp == 2) {
        if (lane == 0) got = pair_wait(&bars->tmem_full[acc], acc_phase, bars, peer, 8u, 256u) ? 1 : 0;
        got = __shfl_sync(0xFFFFFFFFu, got, 0);
      }
      if (one_poller) {  // one warp polls, the other three wait in named barrier 1 (see the 512x256 kernel): -0.6 to -0.9 %
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (lane == 0) {
          (void)mbar_try_wait(&bars->tmem_full[acc], acc_phase);
          got = bars->abort_flag != 0u ? 0 : 1;
        }
        got = __shfl_sync(0xFFFFFFFFu, got, 0);
      }
      if (got == 0) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * PBN);
      drain_accumulator<OutT>(ea, taddr, tc.m * PBM + (int)rank * 128 + quarter * 32, tc.n * PBN, PBN, boxes);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bars->tmem_empty[acc]), 0u));
      if (sched != nullptr) {
        int v = 0;
        if (lane == 0) v = pair_ring_read(bars, (uint32_t)local, peer, 32u, 64u);
        v = __shfl_sync(0xFFFFFFFFu, v, 0);
        if (v == -2) {
          if (one_poller) asm volatile("bar.arrive 1, 128;" ::: "memory");
          ok = false;
          break;
        }
        t = v < 0 ? num_tiles : (int64_t)v;
      } else {
        t += num_clusters;
      }
    }
    if (use_tma_store && lane == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still touch its barriers or TMEM
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

}  // namespace pair


// ===========================================================================
// Two-CTA variant with a 256x256 accumulator per CTA: a cluster of two CTAs works on one 512x256
// output tile.  CTA r stages rows [256r, 256r+256) of the A tile and rows [128r, 128r+128) of the B
// tile, and every k-step issues TWO tcgen05.mma.cta_group::2 (M256 N256 K32): MMA h multiplies
// the h-th 128-row block of both CTAs' A stages with the pair's B and accumulates into tensor-memory
// columns [256h, 256h+256) of both CTAs.  Per k-block a CTA pulls 48 KB through L2 for 256x256 of
// output where the kernels above pull 64 KB (32 KB for 128x256), i.e. 25 % fewer operand bytes
// per flop, and 4 stages of 48 KB buffer as many k-steps of tensor work as 6 stages did there.
// The price: the accumulators fill all 512 tensor-memory columns, so they cannot be double buffered.
// The epilogue is instead overlapped by halves: all eight epilogue warps drain columns 0..255 first
// and release them (tmem_empty[0]), then columns 256..511 (tmem_empty[1]); the MMA thread starts the
// next tile's h = 0 MMAs for the first k-blocks (as many as there are stages) as soon as the first
// half is free, catches up with h = 1 on the same stages when the second half is free, and only then
// releases those stages.  The end of a tile mirrors that: on the last k-blocks (as many as there are
// stages) the h = 0 MMAs are issued first and half 0 is handed to the epilogue (tmem_full[0]) while the
// h = 1 MMAs on the same stages still run (tmem_full[1] follows).  Accumulation order per output element
// is unchanged (k ascending), so the result is bit-identical to the other kernels.
//   full[s]        lives in the leader; both CTAs' TMA loads complete_tx on it (96 KB per stage)
//   empty[s]       one per CTA; released by a multicast tcgen05.commit from the leader
//   tmem_full[h]   per CTA; same multicast commit when the MMAs of a tile into accumulator half h are done
//   tmem_empty[h]  live in the leader; 16 arrivals each (8 epilogue warps of each CTA)
// No TMA load here uses cluster multicast.
// ===========================================================================
namespace pairwide {

using namespace pair;

constexpr int QBM = 512;  // rows of the pair tile (256 per CTA)
constexpr int QBN = 256;  // columns of the pair tile (each CTA stages 128 of B's rows)
constexpr int QSTAGES = 4;
constexpr int QA_BYTES = 256 * BK;  // rows 0..127 then 128..255 of this CTA's half of the A tile
constexpr int QB_BYTES = 128 * BK;
constexpr int QSTAGE_BYTES = QA_BYTES + QB_BYTES;
constexpr int QTHREADS = 320;  // TMA warp, MMA warp, 8 epilogue warps
constexpr int SPLIT_DRAIN_BIT = 26;  // bit of the packed `raster` word: overlap the epilogue by halves
constexpr int SPLIT_TAIL_BIT = 27;   // and finish accumulator half 0 ahead of half 1 at the end of a tile

struct __align__(8) QBarriers {
  uint64_t full[QSTAGES];
  uint64_t empty[QSTAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  TileRing ring;  // written in both CTAs by the leader's producer thread
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

constexpr int QSMEM_BYTES = QSTAGES * QSTAGE_BYTES + 8 * EPI_BOX_BYTES + 1024 + (int)sizeof(QBarriers);

template <typename OutT, bool SCATTER = false>
__global__ void __launch_bounds__(QTHREADS, 1)
gemm_fp8_pairwide_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                         const __grid_constant__ CUtensorMap tma_out, const float* __restrict__ scale_a,
                         const float* __restrict__ scale_b, const OutT* __restrict__ bias, OutT* __restrict__ out,
                         int64_t ldo, int m, int n, int k, uint32_t idesc, int out_vec_ok, int use_tma_store,
                         int raster, uint32_t* sched,
                         const __grid_constant__ std::conditional_t<SCATTER, RowScatter, NoScatter> scatter) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = tiles + QSTAGES * QSTAGE_BYTES;
  QBarriers* bars = reinterpret_cast<QBarriers*>(staging + 8 * EPI_BOX_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t peer = rank ^ 1u;
  const bool leader = rank == 0;
  const int tiles_m = (m + QBM - 1) / QBM, tiles_n = (n + QBN - 1) / QBN;
  const int64_t num_tiles = (int64_t)tiles_m * tiles_n;
  const int num_kb = (k + BK - 1) / BK;
  const int64_t cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const bool a_mn = (raster >> LAYOUT_A_MN_BIT) & 1, b_mn = (raster >> LAYOUT_B_MN_BIT) & 1;
  const bool split_drain = (raster >> SPLIT_DRAIN_BIT) & 1;
  const bool split_tail = (raster >> SPLIT_TAIL_BIT) & 1;
  // Waits pass a suspend-time hint to mbarrier.try_wait (the hardware parks the thread and wakes it when the
  // phase completes) instead of sleeping between probes or spinning: 12-17 % fewer executed instructions and
  // 0.4-0.5 % less time over the twelve GEMMs of the 70B step.  F8B200_GEMM_WAIT=sleep restores the loops.
  // (The 256x256 pair kernel keeps the loops: with hints its twelve LLaMa-3-8B products took 2.85-2.88 ms
  // against 2.80 ms.)
  const bool hw_wait = ((raster >> WAIT_SLEEP_BIT) & 1) == 0;
  const bool one_poller = ((raster >> EPI_ALL_POLL_BIT) & 1) == 0;
  auto bo = [&](uint32_t ns) { return hw_wait ? (WAIT_BY_HINT | (ns == 0u ? 2000u : ns * 32u)) : ns; };
  const uint64_t step_a = desc_k_step(a_mn), step_b = desc_k_step(b_mn);

  if (threadIdx.x == 0) {
    for (int s = 0; s < QSTAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->tmem_full[0], 1);
    mbar_init(&bars->tmem_full[1], 1);
    mbar_init(&bars->tmem_empty[0], 16);
    mbar_init(&bars->tmem_empty[1], 16);
    for (int r = 0; r < RING; ++r) mbar_init(&bars->ring.full[r], 1);
    bars->abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA) ----------------
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_b)) : "memory");
      auto load = [&](void* dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
        tma_load_2d_pair_plain(dst, map, x, y, bar);  // no cache-hint operand: see l2_policy
      };
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int claim_kb = num_kb > 4 ? num_kb - 4 : 0;
      uint32_t entry = 0;  // ring entries published (leader) or read (partner) so far
      int64_t t = cluster_id;
      while (ok && t < num_tiles) {
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n, raster);
        const int row_a = tc.m * QBM + (int)rank * 256;
        const int row_b = tc.n * QBN + (int)rank * 128;
        int64_t next = t + num_clusters;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (sched != nullptr && leader && kb == claim_kb) next = num_clusters + (int64_t)atomicAdd(sched, 1u);
          if (!pair_wait(&bars->empty[stage], phase ^ 1u, bars, peer, 1u, bo(64u))) { ok = false; break; }
          uint8_t* sa = tiles + stage * QSTAGE_BYTES;
          if (leader) mbar_expect_tx(&bars->full[stage], 2 * QSTAGE_BYTES);
          const uint32_t full_in_leader = mapa_u32(smem_u32(&bars->full[stage]), 0u);
          if (!a_mn) {  // one box of 256 rows x 128 bytes of K
            load(sa, &tma_a, kb * BK, row_a, full_in_leader);
          } else {  // two boxes of [128 k rows] x [128 M positions]
            load(sa, &tma_a, row_a, kb * BK, full_in_leader);
            load(sa + 128 * BK, &tma_a, row_a + 128, kb * BK, full_in_leader);
          }
          load(sa + QA_BYTES, &tma_b, b_mn ? row_b : kb * BK, b_mn ? kb * BK : row_b, full_in_leader);
          if (++stage == QSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (sched != nullptr) {
          if (leader) {
            const uint32_t slot = entry & (RING - 1);
            const int32_t v = next < num_tiles ? (int32_t)next : -1;
            bars->ring.tile[slot] = v;
            mbar_arrive(&bars->ring.full[slot]);
            st_cluster_u32(mapa_u32(smem_u32(&bars->ring.tile[slot]), 1u), (uint32_t)v);
            mbar_arrive_release_cluster(mapa_u32(smem_u32(&bars->ring.full[slot]), 1u));
          } else {
            const int32_t v = pair_ring_read(bars, entry, peer, 64u, bo(32u));
            if (v == -2) { ok = false; break; }
            next = v < 0 ? num_tiles : (int64_t)v;
          }
          ++entry;
        }
        t = next;
      }
      // tail: every release the leader multicast to this CTA's empty barriers has landed
      for (int s = 0; ok && s < QSTAGES; ++s) {
        if (!pair_wait(&bars->empty[stage], phase ^ 1u, bars, peer, 1u, bo(64u))) { ok = false; break; }
        if (++stage == QSTAGES) { stage = 0; phase ^= 1u; }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int64_t local = 0;
      int64_t t = cluster_id;
      // the four K = 32 MMAs of one k-block into accumulator half h
      auto issue_half = [&](int st, int kb, int h) {
        const uint32_t a_addr = smem_u32(tiles + st * QSTAGE_BYTES);
        const uint32_t ah = a_addr + (uint32_t)h * 128u * BK;
        const uint64_t da = a_mn ? make_smem_desc_mn(ah, 128 * BK) : make_smem_desc(ah);
        const uint64_t db = b_mn ? make_smem_desc_mn(a_addr + QA_BYTES, QB_BYTES) : make_smem_desc(a_addr + QA_BYTES);
        const uint32_t tmem_d = tmem_base + (uint32_t)(h * 256);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk)
          tc_mma_f8_pair(tmem_d, da + (uint64_t)kk * step_a, db + (uint64_t)kk * step_b, idesc, (kb | kk) != 0 ? 1u : 0u);
      };
      for (; ok && t < num_tiles; ++local) {
        const uint32_t free_parity = (uint32_t)(local & 1) ^ 1u;
        if (!pair_wait(&bars->tmem_empty[0], free_parity, bars, peer, 2u, bo(0u))) { ok = false; break; }
        tc_fence_after();
        // head of the tile on accumulator half 0 alone, while the epilogue still drains half 1
        const int head = split_drain ? (num_kb < QSTAGES ? num_kb : QSTAGES) : 0;
        {
          int st = stage;
          uint32_t ph = phase;
          for (int kb = 0; kb < head; ++kb) {
            if (!pair_wait(&bars->full[st], ph, bars, peer, 4u, bo(0u))) { ok = false; break; }
            tc_fence_after();
            issue_half(st, kb, 0);
            if (++st == QSTAGES) { st = 0; ph ^= 1u; }
          }
        }
        if (!ok) break;
        if (!pair_wait(&bars->tmem_empty[1], free_parity, bars, peer, 2u, bo(0u))) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < head; ++kb) {  // these stages are known to be full
          issue_half(stage, kb, 1);
          tc_commit_pair(&bars->empty[stage]);
          if (++stage == QSTAGES) { stage = 0; phase ^= 1u; }
        }
        // tail of the tile: half 0 finishes its last k-blocks first and is handed to the epilogue while
        // half 1 still runs them
        int tail = split_tail ? (num_kb - head < QSTAGES ? num_kb - head : QSTAGES) : 0;
        if (tail < 0) tail = 0;
        for (int kb = head; kb < num_kb - tail; ++kb) {
          if (!pair_wait(&bars->full[stage], phase, bars, peer, 4u, bo(0u))) { ok = false; break; }
          tc_fence_after();
          issue_half(stage, kb, 0);
          issue_half(stage, kb, 1);
          tc_commit_pair(&bars->empty[stage]);
          if (++stage == QSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        {
          int st = stage;
          uint32_t ph = phase;
          for (int kb = num_kb - tail; kb < num_kb; ++kb) {
            if (!pair_wait(&bars->full[st], ph, bars, peer, 4u, bo(0u))) { ok = false; break; }
            tc_fence_after();
            issue_half(st, kb, 0);
            if (++st == QSTAGES) { st = 0; ph ^= 1u; }
          }
        }
        if (!ok) break;
        tc_commit_pair(&bars->tmem_full[0]);
        for (int kb = num_kb - tail; kb < num_kb; ++kb) {  // these stages are known to be full
          issue_half(stage, kb, 1);
          tc_commit_pair(&bars->empty[stage]);
          if (++stage == QSTAGES) { stage = 0; phase ^= 1u; }
        }
        tc_commit_pair(&bars->tmem_full[1]);
        if (sched != nullptr) {
          const int32_t v = pair_ring_read(bars, (uint32_t)local, peer, 16u, bo(0u));
          if (v == -2) { ok = false; break; }
          t = v < 0 ? num_tiles : (int64_t)v;
        } else {
          t += num_clusters;
        }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9 of both CTAs) ----------------
    // Warp w drains lanes [32q, 32q+32), q = w & 3, and the column block p = (w - 2) >> 2 (128 of the
    // 256 columns) of accumulator half 0 (rows 0..127 of this CTA), then of half 1 (rows 128..255).
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;
    float inv = 0.f;
    {
      const float sa = __ldg(scale_a), sb = __ldg(scale_b);
      inv = __fmul_rn(__fdiv_rn(1.0f, sa), __fdiv_rn(1.0f, sb));
    }
    const RowScatter* sc = nullptr;
    if constexpr (SCATTER) sc = &scatter;
    const EpilogueArgs<OutT> ea{bias, out, ldo, m, n, out_vec_ok, use_tma_store, &tma_out,
                                staging + (warp - 2) * EPI_BOX_BYTES, inv, (raster >> 20) & 1, sc};
    uint32_t boxes = 0;
    bool ok = true;
    int64_t local = 0;
    int64_t t = cluster_id;
    for (; ok && t < num_tiles; ++local) {
      const TileCoord tc = tile_coord(t, tiles_m, tiles_n, raster);
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        int got = 1;
        if (!one_poller || warp == 2) {
          if (lane == 0) got = pair_wait(&bars->tmem_full[h], (uint32_t)(local & 1), bars, peer, 8u, bo(256u)) ? 1 : 0;
          got = __shfl_sync(0xFFFFFFFFu, got, 0);
        }
        if (one_poller) {
          // One warp waits for the accumulator half; the other seven sit in a hardware barrier (named barrier 1,
          // the eight epilogue warps), which costs no instructions while they wait and wakes them at once:
          // 27-37 % fewer executed instructions per GEMM and 0.3-0.5 % less time than eight polling warps
          // (F8B200_GEMM_EPIWAIT=all).  Every warp arrives at the barrier exactly once per accumulator half; a
          // warp that leaves the loop early (its tile-ring read gave up) arrives without waiting, below, and
          // the abort flag read after the barrier sends the others after it.
          asm volatile("bar.sync 1, 256;" ::: "memory");
          if (lane == 0) {
            (void)mbar_try_wait(&bars->tmem_full[h], (uint32_t)(local & 1));  // this warp's own acquire of the phase
            got = bars->abort_flag != 0u ? 0 : 1;
          }
          got = __shfl_sync(0xFFFFFFFFu, got, 0);
        }
        if (got == 0) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(h * 256 + part * 128);
        wide::drain_wide<OutT>(ea, taddr, tc.m * QBM + (int)rank * 256 + h * 128 + quarter * 32, tc.n * QBN + part * 128,
                               128, boxes);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bars->tmem_empty[h]), 0u));
      }
      if (!ok) break;
      if (sched != nullptr) {
        int v = 0;
        if (lane == 0) v = pair_ring_read(bars, (uint32_t)local, peer, 32u, bo(64u));
        v = __shfl_sync(0xFFFFFFFFu, v, 0);
        if (v == -2) {
          if (one_poller) asm volatile("bar.arrive 1, 256;" ::: "memory");
          ok = false;
          break;
        }
        t = v < 0 ? num_tiles : (int64_t)v;
      } else {
        t += num_clusters;
      }
    }
    if (use_tma_store == 1 && lane == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still touch its barriers or TMEM
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

}  // namespace pairwide

// ---- host side --------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }
  });
  return fn;
}

// MN-major operand: 2-D byte tensor [k, rows] with row stride ld (rows contiguous),
// box = [128 k rows] x [128 bytes of rows], 128B swizzle.
static int encode_operand_map_mn(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t ld);

// L2 promotion of the operand maps: how much L2 fetches from HBM around a requested 128-byte row piece.
// 256 bytes (the next k-block of the same row comes along) is the default; F8B200_GEMM_L2PROMO=0/64/128/256.
static CUtensorMapL2promotion operand_l2_promotion() {
  const char* e = getenv("F8B200_GEMM_L2PROMO");
  if (e == nullptr || e[0] == 0) return CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  const int v = atoi(e);
  return v == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE : v == 64 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
       : v == 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
}

// 2-D byte tensor [rows, k] with row stride ld, box = [box_rows, 128 bytes], 128B swizzle.
static int encode_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t ld, int box_rows) {
  auto fn = get_encode_fn();
  if (fn == nullptr) return F8B200_ERR_DRIVER;
  const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)ld};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, operand_l2_promotion(),
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? F8B200_OK : F8B200_ERR_DRIVER;
}

static int encode_operand_map_mn(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t ld) {
  auto fn = get_encode_fn();
  if (fn == nullptr) return F8B200_ERR_DRIVER;
  const cuuint64_t gdim[2] = {(cuuint64_t)rows, (cuuint64_t)k};
  const cuuint64_t gstride[1] = {(cuuint64_t)ld};
  const cuuint32_t box[2] = {128u, (cuuint32_t)BK};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, operand_l2_promotion(),
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? F8B200_OK : F8B200_ERR_DRIVER;
}

// Output tensor map for the TMA-store epilogue: boxes of 32 rows x 128 bytes, 128B swizzle.
// `half_boxes` (16-bit outputs only): boxes of 32 rows x 64 bytes with the 64-byte swizzle, the unit
// the wide kernels' epilogue stages (two of them alternate per warp).
static int encode_output_map(CUtensorMap* map, void* base, int64_t m, int64_t n, int64_t ldo, int out_dtype,
                             bool half_boxes = false) {
  auto fn = get_encode_fn();
  if (fn == nullptr) return F8B200_ERR_DRIVER;
  const int esz = out_dtype == F8B200_FP32 ? 4 : 2;
  half_boxes = half_boxes && esz == 2;
  const CUtensorMapDataType dt = out_dtype == F8B200_FP32   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : out_dtype == F8B200_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                            : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const cuuint64_t gdim[2] = {(cuuint64_t)n, (cuuint64_t)m};
  const cuuint64_t gstride[1] = {(cuuint64_t)(ldo * esz)};
  const cuuint32_t box[2] = {(cuuint32_t)((half_boxes ? 64 : 128) / esz), 32u};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, dt, 2, base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        half_boxes ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? F8B200_OK : F8B200_ERR_DRIVER;
}

// Picks the band direction and width (see tile_coord): the band's operand panel
// (width x tile x K bytes) should stay in L2 while the other operand is re-read once per
// band; choose the direction with the smaller total HBM traffic.
static int choose_raster(int64_t m, int64_t n, int64_t k, int tile_m, int tile_n) {
  int64_t panel_bytes = 32ll << 20;
  if (const char* e = getenv("F8B200_GEMM_PANEL_MB")) {
    const long v = atol(e);
    if (v > 0) panel_bytes = (int64_t)v << 20;
  }
  int64_t min_band = 8;
  if (const char* e = getenv("F8B200_GEMM_MINBAND")) {
    const long v = atol(e);
    if (v > 0) min_band = v;
  }
  const int64_t tiles_m = (m + tile_m - 1) / tile_m, tiles_n = (n + tile_n - 1) / tile_n;
  auto width = [&](int tile, int64_t tiles) {
    int64_t g = panel_bytes / ((int64_t)tile * (k > 0 ? k : 1));
    if (g < min_band) g = min_band;  // very long K: the panel cannot stay resident anyway, keep the band wide
    if (g > tiles) g = tiles;
    if (g > 0xFFFF) g = 0xFFFF;
    return g < 1 ? (int64_t)1 : g;
  };
  const int64_t gm = width(tile_m, tiles_m), gn = width(tile_n, tiles_n);
  const double a_bytes = (double)m * k, b_bytes = (double)n * k;
  const double cost_m = a_bytes + b_bytes * (double)((tiles_m + gm - 1) / gm);
  const double cost_n = b_bytes + a_bytes * (double)((tiles_n + gn - 1) / gn);
  // L2 hints (bit 0: output stores evict-first, bit 1: streaming operand evict-first,
  // bit 2: panel operand evict-last); F8B200_GEMM_L2HINT overrides the default.  An operand without a
  // hint bit is loaded with no cache-hint operand at all (see l2_policy: that is what lets the L2 request
  // coalescer merge its loads), so the default asks for none.
  int hints = 1;
  if (const char* e = getenv("F8B200_GEMM_L2HINT")) hints = atoi(e) & 7;
  return (cost_n < cost_m ? (int)(gn | (1 << 16)) : (int)gm) | (hints << 20);
}

// Dynamic tile scheduling is used when the caller gave a scheduling word, there is more than one
// tile per CTA (or pair) to hand out, and tile indices fit the ring's int32 entries.
// F8B200_GEMM_SCHED=static switches it off (read at every call).
static uint32_t* usable_sched(uint32_t* sched, int64_t tiles, int units) {
  if (sched == nullptr || tiles <= units || tiles + units >= 0x7FFFFFFFLL) return nullptr;
  const char* e = getenv("F8B200_GEMM_SCHED");
  if (e != nullptr && e[0] == 's') return nullptr;
  return sched;
}

// SMs left free for kernels that run beside the GEMM on other streams (collectives): the persistent
// GEMMs otherwise hold every SM until they end, which serialises a concurrent all-gather or
// reduce-scatter behind them.  F8B200_GEMM_SM_MARGIN, read at every call; default 0.
static int sm_margin() {
  const char* e = getenv("F8B200_GEMM_SM_MARGIN");
  if (e == nullptr || e[0] == 0) return 0;
  const int v = atoi(e);
  return v < 0 ? 0 : v;
}
static int persistent_ctas() {
  const int g = sm_count() - sm_margin();
  return g < 2 ? 2 : g;
}

template <typename OutT>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, int use_tma, const float* sa,
                  const float* sb, const void* bias, void* out, int64_t ldo, int m, int n, int k, uint32_t idesc,
                  int vec_ok, cudaStream_t st) {
  static PerDeviceOnce setup;  // the shared-memory opt-in is a per-device attribute
  const cudaError_t attr_err = setup.run([](int*) {
    return cudaFuncSetAttribute(gemm_fp8_kernel<OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  });
  if (attr_err != cudaSuccess) return record_cuda_error(attr_err);
  const int64_t tiles = (int64_t)((m + BM - 1) / BM) * ((n + BN - 1) / BN);
  int grid = persistent_ctas();
  if (tiles < grid) grid = (int)tiles;
  gemm_fp8_kernel<OutT><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ma, mb, mo, sa, sb, static_cast<const OutT*>(bias),
                                                                static_cast<OutT*>(out), ldo, m, n, k, idesc, vec_ok,
                                                                use_tma, choose_raster(m, n, k, BM, BN));
  return check_launch();
}

// F8B200_GEMM_EPIWAIT=all (read at every call): every epilogue warp of the pair kernels polls for its accumulator
static int epi_wait_bits() {
  const char* e = getenv("F8B200_GEMM_EPIWAIT");
  return (e != nullptr && e[0] == 'a') ? (1 << EPI_ALL_POLL_BIT) : 0;
}
// F8B200_GEMM_WAIT=sleep (read at every call): the 512x256 pair kernel's waits sleep between probes
static int wait_bits() {
  const char* e = getenv("F8B200_GEMM_WAIT");
  return (e != nullptr && e[0] == 's') ? (1 << WAIT_SLEEP_BIT) : 0;
}

template <typename OutT>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, int use_tma,
                       const float* sa, const float* sb, const void* bias, void* out, int64_t ldo, int m, int n, int k,
                       uint32_t idesc, int vec_ok, int layouts, uint32_t* sched, cudaStream_t st) {
  static PerDeviceOnce setup;  // shared-memory opt-in and cluster occupancy, once per device
  int max_clusters = 0;
  auto kernel = pair::gemm_fp8_pair_kernel<OutT>;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = pair::PSMEM_BYTES;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t attr_err = setup.run(
      [&](int* clusters_out) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::PSMEM_BYTES);
        if (e == cudaSuccess) {
          cfg.gridDim = dim3(2 * (sm_count() / 2));
          e = cudaOccupancyMaxActiveClusters(clusters_out, kernel, &cfg);
        }
        return e;
      },
      &max_clusters);
  if (attr_err != cudaSuccess) return record_cuda_error(attr_err);
  if (max_clusters < 1) return F8B200_ERR_UNSUPPORTED;
  const int64_t tiles = (int64_t)((m + pair::PBM - 1) / pair::PBM) * ((n + pair::PBN - 1) / pair::PBN);
  int clusters = max_clusters;
  if (persistent_ctas() / 2 < clusters) clusters = persistent_ctas() / 2;
  if (tiles < clusters) clusters = (int)tiles;
  cfg.gridDim = dim3(2 * clusters);
  const OutT* bias_t = static_cast<const OutT*>(bias);
  OutT* out_t = static_cast<OutT*>(out);
  sched = usable_sched(sched, tiles, clusters);
  if (sched != nullptr) {
    const cudaError_t e = cudaMemsetAsync(sched, 0, sizeof(uint32_t), st);
    if (e != cudaSuccess) return record_cuda_error(e);
  }
  return record_cuda_error(
      cudaLaunchKernelEx(&cfg, kernel, ma, mb, mo, sa, sb, bias_t, out_t, ldo, m, n, k, idesc, vec_ok, use_tma,
                         choose_raster(m, n, k, pair::PBM, pair::PBN) | layouts | epi_wait_bits(), sched));
}

template <typename OutT>
static int launch_wide(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, int use_tma,
                       const float* sa, const float* sb, const void* bias, void* out, int64_t ldo, int m, int n, int k,
                       uint32_t idesc, int vec_ok, int layouts, uint32_t* sched, cudaStream_t st) {
  static PerDeviceOnce setup;
  const cudaError_t attr_err = setup.run([](int*) {
    return cudaFuncSetAttribute(wide::gemm_fp8_wide_kernel<OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                wide::WSMEM_BYTES);
  });
  if (attr_err != cudaSuccess) return record_cuda_error(attr_err);
  const int64_t tiles = (int64_t)((m + wide::WBM - 1) / wide::WBM) * ((n + wide::WBN - 1) / wide::WBN);
  int grid = persistent_ctas();
  if (tiles < grid) grid = (int)tiles;
  sched = usable_sched(sched, tiles, grid);
  if (sched != nullptr) {
    const cudaError_t e = cudaMemsetAsync(sched, 0, sizeof(uint32_t), st);
    if (e != cudaSuccess) return record_cuda_error(e);
  }
  wide::gemm_fp8_wide_kernel<OutT><<<grid, wide::WTHREADS, wide::WSMEM_BYTES, st>>>(
      ma, mb, mo, sa, sb, static_cast<const OutT*>(bias), static_cast<OutT*>(out), ldo, m, n, k, idesc, vec_ok,
      use_tma, choose_raster(m, n, k, wide::WBM, wide::WBN) | layouts, sched);
  return check_launch();
}

template <typename OutT, bool SCATTER = false>
static int launch_pairwide(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, int use_tma,
                           const float* sa, const float* sb, const void* bias, void* out, int64_t ldo, int m, int n,
                           int k, uint32_t idesc, int vec_ok, int layouts, uint32_t* sched, cudaStream_t st,
                           const std::conditional_t<SCATTER, RowScatter, NoScatter>& scatter = {}) {
  static PerDeviceOnce setup;  // shared-memory opt-in and cluster occupancy, once per device
  int max_clusters = 0;
  auto kernel = pairwide::gemm_fp8_pairwide_kernel<OutT, SCATTER>;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(pairwide::QTHREADS);
  cfg.dynamicSmemBytes = pairwide::QSMEM_BYTES;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t attr_err = setup.run(
      [&](int* clusters_out) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pairwide::QSMEM_BYTES);
        if (e == cudaSuccess) {
          cfg.gridDim = dim3(2 * (sm_count() / 2));
          e = cudaOccupancyMaxActiveClusters(clusters_out, kernel, &cfg);
        }
        return e;
      },
      &max_clusters);
  if (attr_err != cudaSuccess) return record_cuda_error(attr_err);
  if (max_clusters < 1) return F8B200_ERR_UNSUPPORTED;
  const int64_t tiles = (int64_t)((m + pairwide::QBM - 1) / pairwide::QBM) * ((n + pairwide::QBN - 1) / pairwide::QBN);
  int clusters = max_clusters;
  if (persistent_ctas() / 2 < clusters) clusters = persistent_ctas() / 2;
  if (tiles < clusters) clusters = (int)tiles;
  cfg.gridDim = dim3(2 * clusters);
  const OutT* bias_t = static_cast<const OutT*>(bias);
  OutT* out_t = static_cast<OutT*>(out);
  sched = usable_sched(sched, tiles, clusters);
  if (sched != nullptr) {
    const cudaError_t e = cudaMemsetAsync(sched, 0, sizeof(uint32_t), st);
    if (e != cudaSuccess) return record_cuda_error(e);
  }
  // F8B200_GEMM_SPLIT_DRAIN=0 makes the MMA thread wait for the whole accumulator (read at every call)
  // ("head": only the start of the next tile overlaps the drain, not the end of the current one)
  int split = (1 << pairwide::SPLIT_DRAIN_BIT) | (1 << pairwide::SPLIT_TAIL_BIT);
  if (const char* e = getenv("F8B200_GEMM_SPLIT_DRAIN")) {
    if (e[0] == '0') split = 0;
    if (e[0] == 'h') split = 1 << pairwide::SPLIT_DRAIN_BIT;
  }
  split |= wait_bits();
  split |= epi_wait_bits();
  return record_cuda_error(
      cudaLaunchKernelEx(&cfg, kernel, ma, mb, mo, sa, sb, bias_t, out_t, ldo, m, n, k, idesc, vec_ok, use_tma,
                         choose_raster(m, n, k, pairwide::QBM, pairwide::QBN) | layouts | split, sched, scatter));
}

// Kernel choice: 0 = one CTA per 128x256 tile, 1 = CTA pairs on 256x256 tiles (cta_group::2, two accumulators),
// 2 = one CTA per 256x256 tile, 3 = CTA pairs on 512x256 tiles (cta_group::2, one 256x256 accumulator per CTA).
// Kernel 3 moves 25 % fewer operand bytes from L2 per flop than the others (48 KB per k-block for 256x256 of
// output against 64 KB), which on a power-capped part is worth more than the fully hidden epilogue of kernel 1:
// sustained over the twelve GEMMs of the LLaMa-2-70B step (M = 16384, K >= 8192) it measured 33.6 ms against
// 35.1 ms for kernel 1, ahead or level on every shape.  Kernel 1 is the better one where kernel 3's price shows:
// (a) its accumulator drain is only partly overlapped (about 2500 cycles per tile stay exposed, which is 7 %
// of a K = 4096 tile), and (b) its tiles are twice as large, so a product of a few hundred tiles fills the
// last wave worse (256 tiles on 74 pairs: 4 waves for the work of 3.46).  The rule below scores both kernels,
// score = (tiles / (waves x pairs)) x (share of a tile's time that is MMA work, with kernel 1's larger operand
// traffic as a penalty that grows with K), and takes kernel 1 only when it scores 4 % better, which keeps
// kernel 3 on every product of the 70B step.  Measured on the LLaMa-3-8B products (M = 8192; K, N in 1024 /
// 4096 / 14336) the rule's choices are 2-4 % faster than kernel 3 alone (and 1.5x on the 1024 x 4096 x 8192
// weight gradient, whose 32 large tiles leave most pairs idle).  With at most 256 rows a 512-row tile would be
// half empty: kernel 1.
// F8B200_GEMM_MODE ("1cta" / "2cta" / "wide" / "pw") forces one kernel; F8B200_GEMM_WIDE_K=<k> restores an earlier
// rule (kernel 1 below that K, kernel 2 above).  Both are read at every call so that tests can exercise every
// kernel in one process.
static int gemm_mode(int64_t m, int64_t n, int64_t k) {
  const char* e = getenv("F8B200_GEMM_MODE");
  if (e != nullptr && e[0] == '1') return 0;
  if (e != nullptr && e[0] == '2') return 1;
  if (e != nullptr && e[0] == 'w') return 2;
  if (e != nullptr && e[0] == 'p') return 3;
  const char* t = getenv("F8B200_GEMM_WIDE_K");
  if (t != nullptr && t[0] != 0) return k >= atoll(t) ? 2 : 1;
  if (m <= 256) return 1;
  const double pairs = (double)(persistent_ctas() / 2 > 0 ? persistent_ctas() / 2 : 1);
  auto fill = [&](int64_t tile_m) {  // share of the pair-waves' capacity that the product's tiles use
    const double tiles = (double)((m + tile_m - 1) / tile_m) * (double)((n + 255) / 256);
    const double waves = (double)(int64_t)((tiles + pairs - 1) / pairs);
    return tiles / (waves * pairs);
  };
  const double kb = (double)((k + 127) / 128);
  const double busy_wide = kb * 1024.0 / (kb * 1024.0 + 2500.0);
  double busy_pair = 0.963;
  if (k > 8192) busy_pair -= 0.02 * log2((double)k / 8192.0);
  return fill(256) * busy_pair > 1.04 * fill(512) * busy_wide ? 1 : 3;
}

}  // namespace gemm
}  // namespace f8b200

using namespace f8b200;

template <typename Fn>
static int dispatch_out_dtype(int out_dtype, Fn&& fn) {
  switch (out_dtype) {
    case F8B200_BF16: return fn(static_cast<__nv_bfloat16*>(nullptr));
    case F8B200_FP16: return fn(static_cast<__half*>(nullptr));
    default: return fn(static_cast<float*>(nullptr));
  }
}

// Argument checks shared by the entry points.  *empty is set when there is nothing to compute
// (m == 0 or n == 0): the caller returns F8B200_OK without launching.
static int gemm_fp8_validate(const void* a, int a_kind, int a_layout, int64_t lda, const void* b, int b_kind,
                             int b_layout, int64_t ldb, const float* scale_a, const float* scale_b, const void* bias,
                             int out_dtype, const void* out, int64_t ldo, int64_t m, int64_t n, int64_t k, bool* empty) {
  *empty = false;
  if (m < 0 || n < 0 || k < 0) return F8B200_ERR_BAD_ARG;
  if (a_kind < 0 || a_kind > 1 || b_kind < 0 || b_kind > 1 || out_dtype < 0 || out_dtype > 2) return F8B200_ERR_BAD_ARG;
  if (a_layout < 0 || a_layout > 1 || b_layout < 0 || b_layout > 1) return F8B200_ERR_BAD_ARG;
  if (m == 0 || n == 0) {
    *empty = true;
    return F8B200_OK;
  }
  if (a == nullptr || b == nullptr || out == nullptr || scale_a == nullptr || scale_b == nullptr) return F8B200_ERR_BAD_ARG;
  if (k == 0) return F8B200_ERR_UNSUPPORTED;
  if (lda < (a_layout ? m : k) || ldb < (b_layout ? n : k) || ldo < n) return F8B200_ERR_BAD_ARG;
  if (m > 0x7FFFFFFFLL || n > 0x7FFFFFFFLL || k > 0x7FFFFFFFLL) return F8B200_ERR_UNSUPPORTED;
  if (lda % 16 != 0 || ldb % 16 != 0 || reinterpret_cast<uintptr_t>(a) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(b) % 16 != 0)
    return F8B200_ERR_ALIGNMENT;
  const int osz = out_dtype == F8B200_FP32 ? 4 : 2;
  if (reinterpret_cast<uintptr_t>(out) % osz != 0 || (bias != nullptr && reinterpret_cast<uintptr_t>(bias) % osz != 0))
    return F8B200_ERR_ALIGNMENT;
  return f8b200_device_check();
}

// a_layout / b_layout: F8B200_K_MAJOR = storage [rows, K] with K contiguous (ld >= K);
// F8B200_MN_MAJOR = storage [K, rows] with rows contiguous (ld >= rows).
static int gemm_fp8_impl(const void* a, int a_kind, int a_layout, int64_t lda, const void* b, int b_kind, int b_layout,
                         int64_t ldb, const float* scale_a, const float* scale_b, const void* bias, int out_dtype,
                         void* out, int64_t ldo, int64_t m, int64_t n, int64_t k, uint32_t* sched, void* stream) {
  bool empty = false;
  int rc = gemm_fp8_validate(a, a_kind, a_layout, lda, b, b_kind, b_layout, ldb, scale_a, scale_b, bias, out_dtype, out,
                             ldo, m, n, k, &empty);
  if (rc != F8B200_OK || empty) return rc;
  const int osz = out_dtype == F8B200_FP32 ? 4 : 2;

  const int vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && ((ldo * osz) % 16 == 0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap ma, mb, mo;
  // TMA-store epilogue needs a 16-byte aligned base and row pitch; F8B200_GEMM_STORE=direct forces the
  // per-thread store path (used by the tests to cover both)
  // Store path of the epilogue.  F8B200_GEMM_STORE = tma (TMA stores through staging boxes; needs a
  // 16-byte aligned base and row pitch; the default when the output qualifies), direct (per-thread
  // stores), smem (kernels whose accumulator fills tensor memory only: whole 128-byte lines per row
  // written by the warps after staging in shared memory; same alignment needs).  The smem path drains
  // an accumulator half in fewer cycles than the TMA path, whose stores queue behind the producer's
  // operand loads in the TMA unit, but under the power limit it measured 2 % slower on every product
  // of the LLaMa-2-70B step (34.45 against 33.79 ms): the extra load / store instructions of 256
  // threads cost more clock than the shorter drain gains.  Read at every call (tests cover every path).
  int use_tma = vec_ok;
  int store_mode_full_tmem = vec_ok;
  {
    const char* e = getenv("F8B200_GEMM_STORE");
    if (e != nullptr && e[0] == 'd') use_tma = 0, store_mode_full_tmem = 0;
    if (e != nullptr && e[0] == 's') store_mode_full_tmem = vec_ok ? 2 : 0;
  }
  auto encode_output = [&](bool half_boxes) {
    if (!use_tma) {
      memset(&mo, 0, sizeof(mo));
      return (int)F8B200_OK;
    }
    return gemm::encode_output_map(&mo, out, m, n, ldo, out_dtype, half_boxes);
  };
  const int layouts = (a_layout << gemm::LAYOUT_A_MN_BIT) | (b_layout << gemm::LAYOUT_B_MN_BIT);
  // operand maps: K-major boxes are [box_rows] x [128 bytes of K]; MN-major boxes are always
  // [128 k rows] x [128 bytes of M or N]
  auto encode_operands = [&](int box_rows, int box_rows_b = 0) {
    int r = a_layout ? gemm::encode_operand_map_mn(&ma, a, m, k, lda) : gemm::encode_operand_map(&ma, a, m, k, lda, box_rows);
    if (r != F8B200_OK) return r;
    return b_layout ? gemm::encode_operand_map_mn(&mb, b, n, k, ldb)
                    : gemm::encode_operand_map(&mb, b, n, k, ldb, box_rows_b > 0 ? box_rows_b : box_rows);
  };
  int mode = gemm::gemm_mode(m, n, k);
  if (mode == 3) {
    // CTA pairs on 512x256 tiles: each CTA fetches a 256-row box of A and a 128-row box of B
    rc = encode_operands(256, 128);
    if (rc == F8B200_OK) rc = store_mode_full_tmem == 1 ? encode_output(true) : (memset(&mo, 0, sizeof(mo)), (int)F8B200_OK);
    if (rc != F8B200_OK) return rc;
    const uint32_t idq = gemm::pair::make_idesc_pair(a_kind, b_kind, a_layout, b_layout);
    rc = dispatch_out_dtype(out_dtype, [&](auto* tag) {
      using OutT = std::remove_pointer_t<decltype(tag)>;
      return gemm::launch_pairwide<OutT>(ma, mb, mo, store_mode_full_tmem, scale_a, scale_b, bias, out, ldo, (int)m, (int)n, (int)k,
                                         idq, vec_ok, layouts, sched, st);
    });
    if (rc != F8B200_ERR_UNSUPPORTED) return rc;
    mode = 2;  // no room for a two-CTA cluster on this device
  }
  if (mode == 1) {
    // each CTA of a pair fetches 128-row boxes of both operands
    rc = encode_operands(128);
    if (rc == F8B200_OK) rc = encode_output(false);
    if (rc != F8B200_OK) return rc;
    const uint32_t idesc2 = gemm::pair::make_idesc_pair(a_kind, b_kind, a_layout, b_layout);
    rc = dispatch_out_dtype(out_dtype, [&](auto* tag) {
      using OutT = std::remove_pointer_t<decltype(tag)>;
      return gemm::launch_pair<OutT>(ma, mb, mo, use_tma, scale_a, scale_b, bias, out, ldo, (int)m, (int)n, (int)k,
                                     idesc2, vec_ok, layouts, sched, st);
    });
    if (rc != F8B200_ERR_UNSUPPORTED) return rc;
    mode = 2;  // no room for a two-CTA cluster on this device: the wide kernel needs none
  }
  if (mode == 2) {
    rc = encode_operands(256);
    if (rc == F8B200_OK) rc = store_mode_full_tmem == 1 ? encode_output(true) : (memset(&mo, 0, sizeof(mo)), (int)F8B200_OK);
    if (rc != F8B200_OK) return rc;
    const uint32_t idw = gemm::wide::make_idesc_wide(a_kind, b_kind, a_layout, b_layout);
    return dispatch_out_dtype(out_dtype, [&](auto* tag) {
      using OutT = std::remove_pointer_t<decltype(tag)>;
      return gemm::launch_wide<OutT>(ma, mb, mo, store_mode_full_tmem, scale_a, scale_b, bias, out, ldo, (int)m, (int)n, (int)k, idw,
                                     vec_ok, layouts, sched, st);
    });
  }
  // one CTA per 128x256 tile (F8B200_GEMM_MODE=1cta): K-major operands, fixed tile stride
  if (a_layout != 0 || b_layout != 0) return F8B200_ERR_UNSUPPORTED;
  rc = encode_output(false);
  if (rc != F8B200_OK) return rc;
  rc = gemm::encode_operand_map(&ma, a, m, k, lda, gemm::BM);
  if (rc != F8B200_OK) return rc;
  rc = gemm::encode_operand_map(&mb, b, n, k, ldb, gemm::BN);
  if (rc != F8B200_OK) return rc;
  const uint32_t idesc = gemm::make_idesc(a_kind, b_kind);
  return dispatch_out_dtype(out_dtype, [&](auto* tag) {
    using OutT = std::remove_pointer_t<decltype(tag)>;
    return gemm::launch<OutT>(ma, mb, mo, use_tma, scale_a, scale_b, bias, out, ldo, (int)m, (int)n, (int)k, idesc,
                              vec_ok, st);
  });
}

extern "C" int f8b200_gemm_fp8(const void* a, int a_kind, int64_t lda, const void* b, int b_kind, int64_t ldb,
                               const float* scale_a, const float* scale_b, const void* bias, int out_dtype, void* out,
                               int64_t ldo, int64_t m, int64_t n, int64_t k, int use_fast_accum, void* stream) {
  (void)use_fast_accum;  // tcgen05 accumulates in fp32 tensor memory either way
  return gemm_fp8_impl(a, a_kind, F8B200_K_MAJOR, lda, b, b_kind, F8B200_K_MAJOR, ldb, scale_a, scale_b, bias, out_dtype,
                       out, ldo, m, n, k, nullptr, stream);
}

extern "C" int f8b200_gemm_fp8_ws(const void* a, int a_kind, int a_layout, int64_t lda, const void* b, int b_kind,
                                  int b_layout, int64_t ldb, const float* scale_a, const float* scale_b,
                                  const void* bias, int out_dtype, void* out, int64_t ldo, int64_t m, int64_t n,
                                  int64_t k, int use_fast_accum, void* workspace, int64_t workspace_bytes,
                                  void* stream) {
  (void)use_fast_accum;
  if (workspace == nullptr || workspace_bytes < F8B200_GEMM_WORKSPACE_BYTES) return F8B200_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(workspace) % 16 != 0) return F8B200_ERR_ALIGNMENT;
  return gemm_fp8_impl(a, a_kind, a_layout, lda, b, b_kind, b_layout, ldb, scale_a, scale_b, bias, out_dtype, out, ldo,
                       m, n, k, static_cast<uint32_t*>(workspace), stream);
}

// ---- scheduling words in static device memory ----------------------------------
// f8b200_gemm_fp8_static_scratch needs no workspace from the caller: its scheduling words live in a
// file-scope device array, one 256-byte slot per stream that has called it on this device.
namespace {
constexpr int kStaticSlots = F8B200_STATIC_SCRATCH_BYTES / F8B200_GEMM_WORKSPACE_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[F8B200_STATIC_SCRATCH_BYTES];

struct StaticScratch {
  unsigned char* base = nullptr;  // address of g_static_scratch on this device; null until a lookup succeeds
  std::mutex mu;
  cudaStream_t owner[kStaticSlots];
  int used = 0;
};
static StaticScratch g_static[kMaxDevices];
}  // namespace

extern "C" int f8b200_gemm_fp8_static_scratch(const void* a, int a_kind, int64_t lda, const void* b, int b_kind,
                                              int64_t ldb, const float* scale_a, const float* scale_b,
                                              const void* bias, int out_dtype, void* out, int64_t ldo, int64_t m,
                                              int64_t n, int64_t k, int use_fast_accum, void* stream) {
  (void)use_fast_accum;
  // the argument checks come first: a refused or empty call neither looks the array up nor takes a slot
  bool empty = false;
  int rc = gemm_fp8_validate(a, a_kind, F8B200_K_MAJOR, lda, b, b_kind, F8B200_K_MAJOR, ldb, scale_a, scale_b, bias,
                             out_dtype, out, ldo, m, n, k, &empty);
  if (rc != F8B200_OK || empty) return rc;
  const int dev = current_device_slot();
  if (dev < 0) return F8B200_ERR_UNSUPPORTED;
  StaticScratch& sc = g_static[dev];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int slot = -1;
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(sc.mu);
    // set-up, once per device: the symbol's address (the call that must not fall inside a stream
    // capture).  Only a successful lookup is kept; after a failure the next call tries again.
    if (sc.base == nullptr) {
      void* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess) return record_cuda_error(e);
      sc.base = static_cast<unsigned char*>(p);
    }
    base = sc.base;
    for (int i = 0; i < sc.used; ++i)
      if (sc.owner[i] == st) slot = i;
    if (slot < 0) {
      // one more stream needs one more slot: beyond the array's size the request is refused
      if ((int64_t)(sc.used + 1) * F8B200_GEMM_WORKSPACE_BYTES > (int64_t)F8B200_STATIC_SCRATCH_BYTES)
        return F8B200_ERR_UNSUPPORTED;
      slot = sc.used++;
      sc.owner[slot] = st;
    }
  }
  return gemm_fp8_impl(a, a_kind, F8B200_K_MAJOR, lda, b, b_kind, F8B200_K_MAJOR, ldb, scale_a, scale_b, bias, out_dtype,
                       out, ldo, m, n, k, reinterpret_cast<uint32_t*>(base + (size_t)slot * F8B200_GEMM_WORKSPACE_BYTES),
                       stream);
}

extern "C" int f8b200_read_device_error(uint32_t* flags_out) {
  if (flags_out == nullptr) return F8B200_ERR_BAD_ARG;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  uint32_t v = 0;
  rc = record_cuda_error(cudaMemcpyFromSymbol(&v, g_device_error, sizeof(v)));
  if (rc != F8B200_OK) return rc;
  const uint32_t zero = 0;
  rc = record_cuda_error(cudaMemcpyToSymbol(g_device_error, &zero, sizeof(zero)));
  *flags_out = v;
  return rc;
}

extern "C" int f8b200_gemm_fp8_scatter_rows(const void* a, int a_kind, int a_layout, int64_t lda, const void* b,
                                            int b_kind, int b_layout, int64_t ldb, const float* scale_a,
                                            const float* scale_b, const void* bias, int out_dtype, void* const* outs,
                                            int n_outs, int64_t rows_per_block, int64_t ldo, int64_t m, int64_t n,
                                            int64_t k, void* workspace, int64_t workspace_bytes, void* stream) {
  if (outs == nullptr || n_outs < 1 || n_outs > gemm::MAX_SCATTER || rows_per_block < 1) return F8B200_ERR_BAD_ARG;
  for (int i = 0; i < n_outs; ++i)
    if (outs[i] == nullptr) return F8B200_ERR_BAD_ARG;
  if (m % (rows_per_block * n_outs) != 0 || rows_per_block > 0x7FFFFFFFLL) return F8B200_ERR_BAD_ARG;
  if (workspace != nullptr && (workspace_bytes < F8B200_GEMM_WORKSPACE_BYTES || reinterpret_cast<uintptr_t>(workspace) % 16 != 0))
    return F8B200_ERR_BAD_ARG;
  bool empty = false;
  int rc = gemm_fp8_validate(a, a_kind, a_layout, lda, b, b_kind, b_layout, ldb, scale_a, scale_b, bias, out_dtype, outs[0],
                             ldo, m, n, k, &empty);
  if (rc != F8B200_OK || empty) return rc;
  const int osz = out_dtype == F8B200_FP32 ? 4 : 2;
  int vec_ok = (ldo * osz) % 16 == 0;
  gemm::RowScatter sc = {};
  sc.n = n_outs;
  sc.rows_per_block = (int)rows_per_block;
  for (int i = 0; i < n_outs; ++i) {
    sc.base[i] = outs[i];
    if (reinterpret_cast<uintptr_t>(outs[i]) % osz != 0) return F8B200_ERR_ALIGNMENT;
    if (reinterpret_cast<uintptr_t>(outs[i]) % 16 != 0) vec_ok = 0;
  }
  CUtensorMap ma, mb, mo;
  memset(&mo, 0, sizeof(mo));  // the scattered output is written by the epilogue warps themselves, not by TMA
  // Store path: whole 128-byte lines per row, written by the warp after staging in shared memory (eight
  // lanes per line), when rows are 16-byte aligned; a store that crosses NVLink is one packet per 32-byte
  // sector a thread touches, and the per-thread path (each lane 16 bytes of its own row) sends four times
  // as many.  F8B200_GEMM_SCATTER_STORE=direct restores the per-thread path (read at every call).
  int store_mode = vec_ok ? 2 : 0;
  if (const char* e = getenv("F8B200_GEMM_SCATTER_STORE"))
    if (e[0] == 'd') store_mode = 0;
  rc = a_layout ? gemm::encode_operand_map_mn(&ma, a, m, k, lda) : gemm::encode_operand_map(&ma, a, m, k, lda, 256);
  if (rc != F8B200_OK) return rc;
  rc = b_layout ? gemm::encode_operand_map_mn(&mb, b, n, k, ldb) : gemm::encode_operand_map(&mb, b, n, k, ldb, 128);
  if (rc != F8B200_OK) return rc;
  const int layouts = (a_layout << gemm::LAYOUT_A_MN_BIT) | (b_layout << gemm::LAYOUT_B_MN_BIT);
  const uint32_t idq = gemm::pair::make_idesc_pair(a_kind, b_kind, a_layout, b_layout);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dispatch_out_dtype(out_dtype, [&](auto* tag) {
    using OutT = std::remove_pointer_t<decltype(tag)>;
    return gemm::launch_pairwide<OutT, true>(ma, mb, mo, store_mode, scale_a, scale_b, bias, outs[0], ldo, (int)m, (int)n, (int)k,
                                             idq, vec_ok, layouts, static_cast<uint32_t*>(workspace), st, sc);
  });
}

extern "C" int f8b200_gemm_kernel_choice(int64_t m, int64_t n, int64_t k) {
  return gemm::gemm_mode(m, n, k);
}

extern "C" int f8b200_check_device_error(void) {
  uint32_t flags = 0;
  const int rc = f8b200_read_device_error(&flags);
  if (rc != F8B200_OK) return rc;
  return flags != 0 ? F8B200_ERR_TIMEOUT : F8B200_OK;
}
