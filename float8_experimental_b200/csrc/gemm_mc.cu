// Single-GPU variant of the wide fp8 GEMM that shares operand tiles inside a thread-block cluster
// with TMA multicast.  It is built into a library of its own (libf8b200_mc.so) from this file and
// is used only when that library is present: runs on two or more GPUs leave both out and fall
// back to the kernels of gemm.cu, which this file includes for the shared device code.
//
// ONLY jobs that use ONE GPU may call into this library.  A multicast load must never be given a
// tensor map that covers another GPU's memory, so the entry point refuses (F8B200_ERR_UNSUPPORTED,
// nothing launched) any operand or output that is not plain device memory OWNED BY THE CURRENT
// DEVICE: a peer pointer, an IPC or symmetric-memory mapping, managed or host memory.  The library
// is built with hidden visibility and exports only its two f8b200_mc_* symbols: the copies of
// gemm.cu's functions, error word and static scratch array it carries are private to it and never
// interpose the ones of libf8b200.so.
//
// A cluster of CM x CN CTAs computes a (CM*256) x (CN*256) block of the output, one 256x256 tile
// per CTA (two M128 N256 K32 MMAs per k-step, accumulators in all 512 TMEM columns, as in the
// wide kernel).  The CN CTAs of one block row need the same 256 rows of A: each fetches 256/CN of
// them and multicasts its box to all of them; likewise the CM CTAs of one block column share B.
// Per tile and k-block a CTA then pulls 32/CN + 32/CM KB through L2 instead of 64 KB, which on a
// power-capped part is worth clock (a measured -25 % of that traffic gave +4.8 % throughput).
//
// Synchronisation.  full[s] (per CTA) expects the whole 64 KB stage: the CTA's own boxes plus the
// boxes its neighbours multicast into it, all of which complete_tx on the barrier at the same
// offset in every destination CTA.  A box may be multicast into stage s of a neighbour only after
// that neighbour's MMAs have finished reading the stage's previous contents, so empty[s] counts
// one arrival per CTA that shares an operand with this one (itself included) and every MMA thread
// releases a stage with a tcgen05.commit multicast to exactly those CTAs.  Tiles are claimed per
// cluster by CTA 0 and published to all CTAs of the cluster through their tile rings.
#include "gemm.cu"

namespace f8b200 {
namespace gemm {
namespace mc {

using namespace wide;

__device__ __forceinline__ void tma_load_2d_mcast(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar,
                                                  uint16_t cta_mask, uint64_t policy) {
  if (policy == 0) {  // default L2 policy: no hint operand (see l2_policy in gemm.cu)
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.multicast::cluster "
        "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)), "h"(cta_mask)
        : "memory");
    return;
  }
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.multicast::cluster.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5, %6;" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)), "h"(cta_mask), "l"(policy)
      : "memory");
}
// Arrives on the barrier at this offset in every CTA of `cta_mask` once all MMAs issued so far by
// this thread have completed.
__device__ __forceinline__ void tc_commit_mcast(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}

// Bounded wait; on giving up it raises the abort flag of every CTA of the cluster.
template <bool CLUSTER_ACQUIRE = false>
__device__ __forceinline__ bool mc_wait(uint64_t* bar, uint32_t parity, WideBarriers* bars, int cluster_size,
                                        uint32_t who, uint32_t backoff_ns = 0) {
  auto probe = [&]() {
    return CLUSTER_ACQUIRE ? pair::mbar_try_wait_acquire_cluster(bar, parity) : mbar_try_wait(bar, parity);
  };
  if (probe()) return true;
  const long long t0 = clock64();
  for (uint32_t it = 0; it < 0x7FFFFFFFu; ++it) {
    if (probe()) return true;
    if (backoff_ns != 0u) __nanosleep(backoff_ns);
    if ((it & 63u) == 63u) {
      if (bars->abort_flag != 0u) return false;
      if (clock64() - t0 > WAIT_BUDGET_CYCLES) break;
    }
  }
  for (int r = 0; r < cluster_size; ++r)
    pair::st_cluster_u32(pair::mapa_u32(smem_u32(const_cast<uint32_t*>(&bars->abort_flag)), (uint32_t)r), 1u);
  atomicOr(&g_device_error, who | 0x400u);
  return false;
}

__device__ __forceinline__ int32_t mc_ring_read(WideBarriers* bars, uint32_t j, int cluster_size, uint32_t who,
                                                uint32_t backoff_ns) {
  const uint32_t slot = j & (RING - 1);
  if (!mc_wait<true>(&bars->ring.full[slot], (j >> 4) & 1u, bars, cluster_size, who, backoff_ns)) return -2;
  return *reinterpret_cast<volatile int32_t*>(&bars->ring.tile[slot]);
}

// CM, CN: cluster extent along M and N in tiles (2x1 or 2x2).
template <typename OutT, int CM, int CN>
__global__ void __launch_bounds__(WTHREADS, 1)
gemm_fp8_mc_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                   const __grid_constant__ CUtensorMap tma_out, const float* __restrict__ scale_a,
                   const float* __restrict__ scale_b, const OutT* __restrict__ bias, OutT* __restrict__ out, int64_t ldo,
                   int m, int n, int k, uint32_t idesc, int out_vec_ok, int use_tma_store, int raster,
                   uint32_t* sched) {
  constexpr int CS = CM * CN;
  constexpr int A_ROWS = WBM / CN;  // rows of A this CTA fetches (and multicasts when CN > 1)
  constexpr int B_ROWS = WBN / CM;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = tiles + WSTAGES * WSTAGE_BYTES;
  WideBarriers* bars = reinterpret_cast<WideBarriers*>(staging + 8 * EPI_BOX_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)pair::cluster_ctarank();
  const int rm = rank % CM, rn = rank / CM;
  // CTAs that need the A rows I fetch: same rm, every rn.  For B: same rn, every rm.
  uint16_t mask_a = 0, mask_b = 0;
#pragma unroll
  for (int j = 0; j < CN; ++j) mask_a |= (uint16_t)(1u << (rm + CM * j));
#pragma unroll
  for (int i = 0; i < CM; ++i) mask_b |= (uint16_t)(1u << (i + CM * rn));
  const uint16_t mask_share = mask_a | mask_b;  // everybody who writes into my stages, me included
  constexpr uint32_t SHARERS = 1 + (CM - 1) + (CN - 1);

  const int stiles_m = (m + CM * WBM - 1) / (CM * WBM), stiles_n = (n + CN * WBN - 1) / (CN * WBN);
  const int64_t num_tiles = (int64_t)stiles_m * stiles_n;  // cluster-sized blocks of tiles
  const int num_kb = (k + BK - 1) / BK;
  const int64_t cluster_id = blockIdx.x / CS, num_clusters = gridDim.x / CS;
  const bool a_mn = (raster >> LAYOUT_A_MN_BIT) & 1, b_mn = (raster >> LAYOUT_B_MN_BIT) & 1;
  const uint64_t step_a = desc_k_step(a_mn), step_b = desc_k_step(b_mn);

  if (threadIdx.x == 0) {
    for (int s = 0; s < WSTAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], SHARERS);
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
  pair::cluster_sync_all();  // every CTA's barriers exist before a neighbour signals them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_b)) : "memory");
      const uint64_t pol = l2_policy(0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int claim_kb = num_kb > 4 ? num_kb - 4 : 0;
      uint32_t entry = 0;
      int64_t t = cluster_id;
      while (ok && t < num_tiles) {
        const TileCoord tc = tile_coord(t, stiles_m, stiles_n, raster);
        const int row_a = (tc.m * CM + rm) * WBM + rn * A_ROWS;  // my share of my tile row's A
        const int row_b = (tc.n * CN + rn) * WBN + rm * B_ROWS;  // my share of my tile column's B
        int64_t next = t + num_clusters;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (sched != nullptr && rank == 0 && kb == claim_kb) next = num_clusters + (int64_t)atomicAdd(sched, 1u);
          if (!mc_wait(&bars->empty[stage], phase ^ 1u, bars, CS, 1u, 64u)) { ok = false; break; }
          uint8_t* sa = tiles + stage * WSTAGE_BYTES + rn * A_ROWS * BK;
          uint8_t* sb = tiles + stage * WSTAGE_BYTES + WA_BYTES + rm * B_ROWS * BK;
          mbar_expect_tx(&bars->full[stage], WSTAGE_BYTES);
          // K-major box: x = k offset, y = row, [rows] x [128 B of k]; MN-major boxes hold 128 rows
          // each ([128 k] x [128 B of rows]), so a share of 256 rows takes two of them
          if (!a_mn) {
            if (CN > 1) tma_load_2d_mcast(sa, &tma_a, kb * BK, row_a, &bars->full[stage], mask_a, pol);
            else tma_load_2d_hint(sa, &tma_a, kb * BK, row_a, &bars->full[stage], pol);
          } else {
#pragma unroll
            for (int h = 0; h < A_ROWS / 128; ++h) {
              if (CN > 1) tma_load_2d_mcast(sa + h * 128 * BK, &tma_a, row_a + h * 128, kb * BK, &bars->full[stage], mask_a, pol);
              else tma_load_2d_hint(sa + h * 128 * BK, &tma_a, row_a + h * 128, kb * BK, &bars->full[stage], pol);
            }
          }
          if (!b_mn) {
            tma_load_2d_mcast(sb, &tma_b, kb * BK, row_b, &bars->full[stage], mask_b, pol);
          } else {
#pragma unroll
            for (int h = 0; h < B_ROWS / 128; ++h)
              tma_load_2d_mcast(sb + h * 128 * BK, &tma_b, row_b + h * 128, kb * BK, &bars->full[stage], mask_b, pol);
          }
          if (++stage == WSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (sched != nullptr) {
          if (rank == 0) {
            const uint32_t slot = entry & (RING - 1);
            const int32_t v = next < num_tiles ? (int32_t)next : -1;
            bars->ring.tile[slot] = v;
            mbar_arrive(&bars->ring.full[slot]);
#pragma unroll
            for (int r = 1; r < CS; ++r) {
              pair::st_cluster_u32(pair::mapa_u32(smem_u32(&bars->ring.tile[slot]), (uint32_t)r), (uint32_t)v);
              pair::mbar_arrive_release_cluster(pair::mapa_u32(smem_u32(&bars->ring.full[slot]), (uint32_t)r));
            }
          } else {
            const int32_t v = mc_ring_read(bars, entry, CS, 64u, 32u);
            if (v == -2) { ok = false; break; }
            next = v < 0 ? num_tiles : (int64_t)v;
          }
          ++entry;
        }
        t = next;
      }
      // tail: every release the neighbours multicast to this CTA's empty barriers has landed
      for (int s = 0; ok && s < WSTAGES; ++s) {
        if (!mc_wait(&bars->empty[stage], phase ^ 1u, bars, CS, 1u, 64u)) { ok = false; break; }
        if (++stage == WSTAGES) { stage = 0; phase ^= 1u; }
      }
      if (!ok) {
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
      int64_t t = cluster_id;
      for (; ok && t < num_tiles; ++local) {
        if (!mc_wait(&bars->tmem_empty, (uint32_t)(local & 1) ^ 1u, bars, CS, 2u)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mc_wait(&bars->full[stage], phase, bars, CS, 4u)) { ok = false; break; }
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
          tc_commit_mcast(&bars->empty[stage], mask_share);
          if (++stage == WSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(&bars->tmem_full);
        if (sched != nullptr) {
          const int32_t v = mc_ring_read(bars, (uint32_t)local, CS, 16u, 0u);
          if (v == -2) { ok = false; break; }
          t = v < 0 ? num_tiles : (int64_t)v;
        } else {
          t += num_clusters;
        }
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 rows 0..127, warps 6..9 rows 128..255 ----------------
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
    int64_t t = cluster_id;
    for (; ok && t < num_tiles; ++local) {
      const TileCoord tc = tile_coord(t, stiles_m, stiles_n, raster);
      const int tile_m = tc.m * CM + rm, tile_n = tc.n * CN + rn;
      int got = 1;
      if (lane == 0) got = mc_wait(&bars->tmem_full, (uint32_t)(local & 1), bars, CS, 8u, 256u) ? 1 : 0;
      if (__shfl_sync(0xFFFFFFFFu, got, 0) == 0) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 256);
      drain_wide<OutT>(ea, taddr, tile_m * WBM + half * 128 + quarter * 32, tile_n * WBN, WBN, boxes);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty);
      if (sched != nullptr) {
        int v = 0;
        if (lane == 0) v = mc_ring_read(bars, (uint32_t)local, CS, 32u, 64u);
        v = __shfl_sync(0xFFFFFFFFu, v, 0);
        if (v == -2) { ok = false; break; }
        t = v < 0 ? num_tiles : (int64_t)v;
      } else {
        t += num_clusters;
      }
    }
    if (use_tma_store && lane == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  pair::cluster_sync_all();  // nobody leaves while a neighbour may still write its stages or barriers
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

template <typename OutT, int CM, int CN>
static int launch_mc(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, int use_tma, const float* sa,
                     const float* sb, const void* bias, void* out, int64_t ldo, int m, int n, int k, uint32_t idesc,
                     int vec_ok, int layouts, uint32_t* sched, cudaStream_t st) {
  constexpr int CS = CM * CN;
  static PerDeviceOnce setup;
  int max_clusters = 0;
  auto kernel = gemm_fp8_mc_kernel<OutT, CM, CN>;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(WTHREADS);
  cfg.dynamicSmemBytes = WSMEM_BYTES;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t attr_err = setup.run(
      [&](int* clusters_out) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WSMEM_BYTES);
        if (e == cudaSuccess) {
          cfg.gridDim = dim3(CS * (sm_count() / CS));
          e = cudaOccupancyMaxActiveClusters(clusters_out, kernel, &cfg);
        }
        return e;
      },
      &max_clusters);
  if (attr_err != cudaSuccess) return record_cuda_error(attr_err);
  if (max_clusters < 1) return F8B200_ERR_UNSUPPORTED;
  const int64_t tiles = (int64_t)((m + CM * WBM - 1) / (CM * WBM)) * ((n + CN * WBN - 1) / (CN * WBN));
  int clusters = max_clusters;
  if (tiles < clusters) clusters = (int)tiles;
  cfg.gridDim = dim3(CS * clusters);
  sched = usable_sched(sched, tiles, clusters);
  if (sched != nullptr) {
    const cudaError_t e = cudaMemsetAsync(sched, 0, sizeof(uint32_t), st);
    if (e != cudaSuccess) return record_cuda_error(e);
  }
  const OutT* bias_t = static_cast<const OutT*>(bias);
  OutT* out_t = static_cast<OutT*>(out);
  return record_cuda_error(cudaLaunchKernelEx(&cfg, kernel, ma, mb, mo, sa, sb, bias_t, out_t, ldo, m, n, k, idesc,
                                              vec_ok, use_tma, choose_raster(m, n, k, CM * WBM, CN * WBN) | layouts,
                                              sched));
}

// ===========================================================================
// CTA pairs with multicast: a cluster of FOUR CTAs = two cta_group::2 pairs that work on two
// 256x256 tiles with the same N range (adjacent in M).  Both pairs need the same 256 rows of B,
// 128 per CTA as in the pair kernel; the CTAs with the same position in their pairs split those
// 128 rows and multicast their 64-row box to each other, so a CTA pulls 16 + 8 KB per k-block
// through L2 instead of 32 KB and the epilogue stays hidden behind the next tile's MMAs (two
// accumulators in TMEM), which the wide multicast kernel above cannot offer.
//
// full[s] lives in each pair's leader and expects the 64 KB both CTAs of the pair receive per stage,
// as in the pair kernel.  The loads are the cta_group::2 forms, whose mbarrier operand may name the
// partner CTA: the address of the local full[s] with the pair bit (bit 24 of a shared-window
// address) cleared designates the even CTA of the pair, and for a multicast load it does so in
// every destination's pair, so a B box multicast to the same position of the other pair completes
// on that pair's leader.  empty[s] counts two arrivals, one tcgen05.commit from each pair's leader,
// multicast to all four CTAs: a B box may only be overwritten once both pairs have consumed the stage.
// ===========================================================================
namespace pairmc {

using namespace pair;

struct __align__(8) PairMcBarriers {
  uint64_t full[PSTAGES];  // used in the pair leaders
  uint64_t empty[PSTAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  TileRing ring;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

constexpr uint32_t PAIR_BIT_MASK = 0xFEFFFFFFu;  // clears the bit that tells the two CTAs of a pair apart

// cta_group::2 loads: `leader_bar` is the local barrier address with the pair bit cleared.
__device__ __forceinline__ void tma_load_2d_pair_local(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                       uint32_t leader_bar, uint64_t policy) {
  if (policy == 0) {
    tma_load_2d_pair_plain(smem_dst, map, x, y, leader_bar);
    return;
  }
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(leader_bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair_mcast(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                       uint32_t leader_bar, uint16_t cta_mask, uint64_t policy) {
  if (policy == 0) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.multicast::cluster"
        " [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(leader_bar), "h"(cta_mask)
        : "memory");
    return;
  }
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.multicast::cluster"
      ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5, %6;" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(leader_bar), "h"(cta_mask), "l"(policy)
      : "memory");
}

constexpr int PMC_SMEM_BYTES = PSTAGES * PSTAGE_BYTES + EPI_STAGING_BYTES + 1024 + (int)sizeof(PairMcBarriers);
constexpr int PMC_CLUSTER = 4;

template <bool CLUSTER_ACQUIRE = false>
__device__ __forceinline__ bool pmc_wait(uint64_t* bar, uint32_t parity, PairMcBarriers* bars, uint32_t who,
                                         uint32_t backoff_ns = 0) {
  auto probe = [&]() { return CLUSTER_ACQUIRE ? mbar_try_wait_acquire_cluster(bar, parity) : mbar_try_wait(bar, parity); };
  if (probe()) return true;
  const long long t0 = clock64();
  for (uint32_t it = 0; it < 0x7FFFFFFFu; ++it) {
    if (probe()) return true;
    if (backoff_ns != 0u) __nanosleep(backoff_ns);
    if ((it & 63u) == 63u) {
      if (bars->abort_flag != 0u) return false;
      if (clock64() - t0 > WAIT_BUDGET_CYCLES) break;
    }
  }
  for (int r = 0; r < PMC_CLUSTER; ++r)
    st_cluster_u32(mapa_u32(smem_u32(const_cast<uint32_t*>(&bars->abort_flag)), (uint32_t)r), 1u);
  atomicOr(&g_device_error, who | 0x800u);
  return false;
}

__device__ __forceinline__ int32_t pmc_ring_read(PairMcBarriers* bars, uint32_t j, uint32_t who, uint32_t backoff_ns) {
  const uint32_t slot = j & (RING - 1);
  if (!pmc_wait<true>(&bars->ring.full[slot], (j >> 4) & 1u, bars, who, backoff_ns)) return -2;
  return *reinterpret_cast<volatile int32_t*>(&bars->ring.tile[slot]);
}

__device__ __forceinline__ void tc_commit_pair_mask(uint64_t* bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}

// K-major operands only.
template <typename OutT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_pairmc_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                       const __grid_constant__ CUtensorMap tma_out, const float* __restrict__ scale_a,
                       const float* __restrict__ scale_b, const OutT* __restrict__ bias, OutT* __restrict__ out,
                       int64_t ldo, int m, int n, int k, uint32_t idesc, int out_vec_ok, int use_tma_store, int raster,
                       uint32_t* sched) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = tiles + PSTAGES * PSTAGE_BYTES;
  PairMcBarriers* bars = reinterpret_cast<PairMcBarriers*>(staging + EPI_STAGING_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0..3
  const uint32_t pr = rank >> 1, r = rank & 1u;  // pair in the cluster, position in the pair
  const bool leader = r == 0;
  const uint32_t my_leader = rank & ~1u;
  const uint16_t pair_mask = (uint16_t)(3u << (2 * pr));
  const uint16_t b_mask = (uint16_t)((1u << r) | (1u << (r + 2)));  // same position in both pairs
  const int stiles_m = (m + 2 * PBM - 1) / (2 * PBM), tiles_n = (n + PBN - 1) / PBN;
  const int64_t num_tiles = (int64_t)stiles_m * tiles_n;  // blocks of two tiles
  const int num_kb = (k + BK - 1) / BK;
  const int64_t cluster_id = blockIdx.x / PMC_CLUSTER, num_clusters = gridDim.x / PMC_CLUSTER;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 2);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 8);
    }
    for (int q = 0; q < RING; ++q) mbar_init(&bars->ring.full[q], 1);
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
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer (every CTA) ----------------
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_b)) : "memory");
      const uint64_t pol = l2_policy(0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int claim_kb = num_kb > 4 ? num_kb - 4 : 0;
      uint32_t entry = 0;
      int64_t t = cluster_id;
      while (ok && t < num_tiles) {
        const TileCoord tc = tile_coord(t, stiles_m, tiles_n, raster);
        const int row_a = (tc.m * 2 + (int)pr) * PBM + (int)r * 128;      // my 128 rows of my pair's A tile
        const int row_b = tc.n * PBN + (int)r * 128 + (int)pr * 64;       // my 64 of the 128 B rows CTAs r need
        int64_t next = t + num_clusters;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (sched != nullptr && rank == 0 && kb == claim_kb) next = num_clusters + (int64_t)atomicAdd(sched, 1u);
          if (!pmc_wait(&bars->empty[stage], phase ^ 1u, bars, 1u, 64u)) { ok = false; break; }
          uint8_t* sa = tiles + stage * PSTAGE_BYTES;
          if (leader) mbar_expect_tx(&bars->full[stage], 2 * PSTAGE_BYTES);
          const uint32_t leader_bar = smem_u32(&bars->full[stage]) & PAIR_BIT_MASK;
          tma_load_2d_pair_local(sa, &tma_a, kb * BK, row_a, leader_bar, pol);
          tma_load_2d_pair_mcast(sa + PA_BYTES + pr * 64 * BK, &tma_b, kb * BK, row_b, leader_bar, b_mask, pol);
          if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (sched != nullptr) {
          if (rank == 0) {
            const uint32_t slot = entry & (RING - 1);
            const int32_t v = next < num_tiles ? (int32_t)next : -1;
            bars->ring.tile[slot] = v;
            mbar_arrive(&bars->ring.full[slot]);
#pragma unroll
            for (int q = 1; q < PMC_CLUSTER; ++q) {
              st_cluster_u32(mapa_u32(smem_u32(&bars->ring.tile[slot]), (uint32_t)q), (uint32_t)v);
              mbar_arrive_release_cluster(mapa_u32(smem_u32(&bars->ring.full[slot]), (uint32_t)q));
            }
          } else {
            const int32_t v = pmc_ring_read(bars, entry, 64u, 32u);
            if (v == -2) { ok = false; break; }
            next = v < 0 ? num_tiles : (int64_t)v;
          }
          ++entry;
        }
        t = next;
      }
      for (int s = 0; ok && s < PSTAGES; ++s) {
        if (!pmc_wait(&bars->empty[stage], phase ^ 1u, bars, 1u, 64u)) { ok = false; break; }
        if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------- MMA issuer (pair leaders) ----------------
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int64_t local = 0;
      int64_t t = cluster_id;
      for (; ok && t < num_tiles; ++local) {
        const int acc = (int)(local & 1);
        const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
        if (!pmc_wait(&bars->tmem_empty[acc], acc_phase ^ 1u, bars, 2u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * PBN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!pmc_wait(&bars->full[stage], phase, bars, 4u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * PSTAGE_BYTES);
          const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(a_addr + PA_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            tc_mma_f8_pair(tmem_d, da + (uint64_t)(kk * (UMMA_K >> 4)), db + (uint64_t)(kk * (UMMA_K >> 4)), idesc,
                           (kb | kk) != 0 ? 1u : 0u);
          }
          tc_commit_pair_mask(&bars->empty[stage], (uint16_t)0xF);
          if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit_pair_mask(&bars->tmem_full[acc], pair_mask);
        if (sched != nullptr) {
          const int32_t v = pmc_ring_read(bars, (uint32_t)local, 16u, 0u);
          if (v == -2) { ok = false; break; }
          t = v < 0 ? num_tiles : (int64_t)v;
        } else {
          t += num_clusters;
        }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5 of every CTA) ----------------
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
      const TileCoord tc = tile_coord(t, stiles_m, tiles_n, raster);
      const int acc = (int)(local & 1);
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      int got = 1;
      if (lane == 0) got = pmc_wait(&bars->tmem_full[acc], acc_phase, bars, 8u, 256u) ? 1 : 0;
      if (__shfl_sync(0xFFFFFFFFu, got, 0) == 0) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * PBN);
      drain_accumulator<OutT>(ea, taddr, (tc.m * 2 + (int)pr) * PBM + (int)r * 128 + quarter * 32, tc.n * PBN, PBN, boxes);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bars->tmem_empty[acc]), my_leader));
      if (sched != nullptr) {
        int v = 0;
        if (lane == 0) v = pmc_ring_read(bars, (uint32_t)local, 32u, 64u);
        v = __shfl_sync(0xFFFFFFFFu, v, 0);
        if (v == -2) { ok = false; break; }
        t = v < 0 ? num_tiles : (int64_t)v;
      } else {
        t += num_clusters;
      }
    }
    if (use_tma_store && lane == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

template <typename OutT>
static int launch_pairmc(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, int use_tma,
                         const float* sa, const float* sb, const void* bias, void* out, int64_t ldo, int m, int n, int k,
                         uint32_t idesc, int vec_ok, uint32_t* sched, cudaStream_t st) {
  static PerDeviceOnce setup;
  int max_clusters = 0;
  auto kernel = gemm_fp8_pairmc_kernel<OutT>;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PMC_CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = PMC_SMEM_BYTES;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t attr_err = setup.run(
      [&](int* clusters_out) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PMC_SMEM_BYTES);
        if (e == cudaSuccess) {
          cfg.gridDim = dim3(PMC_CLUSTER * (sm_count() / PMC_CLUSTER));
          e = cudaOccupancyMaxActiveClusters(clusters_out, kernel, &cfg);
        }
        return e;
      },
      &max_clusters);
  if (attr_err != cudaSuccess) return record_cuda_error(attr_err);
  if (max_clusters < 1) return F8B200_ERR_UNSUPPORTED;
  const int64_t tiles = (int64_t)((m + 2 * PBM - 1) / (2 * PBM)) * ((n + PBN - 1) / PBN);
  int clusters = max_clusters;
  if (tiles < clusters) clusters = (int)tiles;
  cfg.gridDim = dim3(PMC_CLUSTER * clusters);
  sched = usable_sched(sched, tiles, clusters);
  if (sched != nullptr) {
    const cudaError_t e = cudaMemsetAsync(sched, 0, sizeof(uint32_t), st);
    if (e != cudaSuccess) return record_cuda_error(e);
  }
  const OutT* bias_t = static_cast<const OutT*>(bias);
  OutT* out_t = static_cast<OutT*>(out);
  return record_cuda_error(cudaLaunchKernelEx(&cfg, kernel, ma, mb, mo, sa, sb, bias_t, out_t, ldo, m, n, k, idesc,
                                              vec_ok, use_tma, choose_raster(m, n, k, 2 * PBM, PBN), sched));
}

}  // namespace pairmc
}  // namespace mc
}  // namespace gemm
}  // namespace f8b200

#define F8B200_MC_EXPORT extern "C" __attribute__((visibility("default")))

// True when `p` is ordinary device memory allocated on the current device.
static bool owned_by_current_device(const void* p) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  return attr.type == cudaMemoryTypeDevice && attr.device == dev;
}

// Same contract as f8b200_gemm_fp8_ws plus the cluster shape (cluster_m x cluster_n tiles: 2x1 or
// 2x2).  F8B200_ERR_UNSUPPORTED when such clusters cannot be scheduled on the device, or when an
// operand / the output is not this device's own memory (see the head of this file).
F8B200_MC_EXPORT int f8b200_mc_gemm_fp8(const void* a, int a_kind, int a_layout, int64_t lda, const void* b, int b_kind,
                                  int b_layout, int64_t ldb, const float* scale_a, const float* scale_b,
                                  const void* bias, int out_dtype, void* out, int64_t ldo, int64_t m, int64_t n,
                                  int64_t k, int cluster_m, int cluster_n, void* workspace, int64_t workspace_bytes,
                                  void* stream) {
  if (m < 0 || n < 0 || k < 0) return F8B200_ERR_BAD_ARG;
  if (a_kind < 0 || a_kind > 1 || b_kind < 0 || b_kind > 1 || out_dtype < 0 || out_dtype > 2) return F8B200_ERR_BAD_ARG;
  if (a_layout < 0 || a_layout > 1 || b_layout < 0 || b_layout > 1) return F8B200_ERR_BAD_ARG;
  const bool pairs = cluster_m == 4 && cluster_n == 1;  // two CTA pairs sharing B (K-major operands only)
  if (!((cluster_m == 2 && cluster_n == 1) || (cluster_m == 2 && cluster_n == 2) || pairs)) return F8B200_ERR_BAD_ARG;
  if (pairs && (a_layout != 0 || b_layout != 0)) return F8B200_ERR_UNSUPPORTED;
  if (m == 0 || n == 0) return F8B200_OK;
  if (a == nullptr || b == nullptr || out == nullptr || scale_a == nullptr || scale_b == nullptr) return F8B200_ERR_BAD_ARG;
  if (k == 0) return F8B200_ERR_UNSUPPORTED;
  if (lda < (a_layout ? m : k) || ldb < (b_layout ? n : k) || ldo < n) return F8B200_ERR_BAD_ARG;
  if (m > 0x7FFFFFFFLL || n > 0x7FFFFFFFLL || k > 0x7FFFFFFFLL) return F8B200_ERR_UNSUPPORTED;
  if (lda % 16 != 0 || ldb % 16 != 0 || reinterpret_cast<uintptr_t>(a) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(b) % 16 != 0)
    return F8B200_ERR_ALIGNMENT;
  if (workspace != nullptr && (workspace_bytes < F8B200_GEMM_WORKSPACE_BYTES || reinterpret_cast<uintptr_t>(workspace) % 16 != 0))
    return F8B200_ERR_BAD_ARG;
  const int osz = out_dtype == F8B200_FP32 ? 4 : 2;
  if (reinterpret_cast<uintptr_t>(out) % osz != 0 || (bias != nullptr && reinterpret_cast<uintptr_t>(bias) % osz != 0))
    return F8B200_ERR_ALIGNMENT;
  int rc = f8b200_device_check();
  if (rc != F8B200_OK) return rc;
  // the tensor maps given to multicast loads may cover this GPU's own memory only
  if (!owned_by_current_device(a) || !owned_by_current_device(b) || !owned_by_current_device(out))
    return F8B200_ERR_UNSUPPORTED;
  const int vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && ((ldo * osz) % 16 == 0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap ma, mb, mo;
  int use_tma = vec_ok;
  {
    const char* e = getenv("F8B200_GEMM_STORE");
    if (e != nullptr && e[0] == 'd') use_tma = 0;
  }
  if (use_tma) {
    rc = gemm::encode_output_map(&mo, out, m, n, ldo, out_dtype, !pairs);
    if (rc != F8B200_OK) return rc;
  } else {
    memset(&mo, 0, sizeof(mo));
  }
  if (pairs) {
    // A: 128-row boxes (one per CTA); B: 64-row boxes (each CTA fetches a quarter of the tile's rows)
    rc = gemm::encode_operand_map(&ma, a, m, k, lda, 128);
    if (rc != F8B200_OK) return rc;
    rc = gemm::encode_operand_map(&mb, b, n, k, ldb, 64);
    if (rc != F8B200_OK) return rc;
    const uint32_t idp = gemm::pair::make_idesc_pair(a_kind, b_kind);
    uint32_t* sched_p = static_cast<uint32_t*>(workspace);
    return dispatch_out_dtype(out_dtype, [&](auto* tag) {
      using OutT = std::remove_pointer_t<decltype(tag)>;
      return gemm::mc::pairmc::launch_pairmc<OutT>(ma, mb, mo, use_tma, scale_a, scale_b, bias, out, ldo, (int)m, (int)n,
                                                   (int)k, idp, vec_ok, sched_p, st);
    });
  }
  // K-major boxes hold the rows one CTA fetches per k-block: 256 / cluster_n of A, 256 / cluster_m of B
  rc = a_layout ? gemm::encode_operand_map_mn(&ma, a, m, k, lda)
                : gemm::encode_operand_map(&ma, a, m, k, lda, gemm::wide::WBM / cluster_n);
  if (rc != F8B200_OK) return rc;
  rc = b_layout ? gemm::encode_operand_map_mn(&mb, b, n, k, ldb)
                : gemm::encode_operand_map(&mb, b, n, k, ldb, gemm::wide::WBN / cluster_m);
  if (rc != F8B200_OK) return rc;
  const int layouts = (a_layout << gemm::LAYOUT_A_MN_BIT) | (b_layout << gemm::LAYOUT_B_MN_BIT);
  const uint32_t idw = gemm::wide::make_idesc_wide(a_kind, b_kind, a_layout, b_layout);
  uint32_t* sched = static_cast<uint32_t*>(workspace);
  return dispatch_out_dtype(out_dtype, [&](auto* tag) {
    using OutT = std::remove_pointer_t<decltype(tag)>;
    if (cluster_n == 1)
      return gemm::mc::launch_mc<OutT, 2, 1>(ma, mb, mo, use_tma, scale_a, scale_b, bias, out, ldo, (int)m, (int)n, (int)k,
                                             idw, vec_ok, layouts, sched, st);
    return gemm::mc::launch_mc<OutT, 2, 2>(ma, mb, mo, use_tma, scale_a, scale_b, bias, out, ldo, (int)m, (int)n, (int)k,
                                           idw, vec_ok, layouts, sched, st);
  });
}

// The device error word of THIS library's kernels (a bounded wait that gave up).
F8B200_MC_EXPORT int f8b200_mc_read_device_error(uint32_t* flags_out) { return f8b200_read_device_error(flags_out); }
