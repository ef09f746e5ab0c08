// Two-CTA variant of the batched tcgen05 GEMM: a cluster of two CTAs (one SM pair)
// computes one 256 x 256 tile with tcgen05.mma.cta_group::2.  Each CTA loads its own
// 128 rows of A and only HALF of B (128 of the tile's 256 columns), so shared-memory
// fill traffic per FLOP drops by a third against the one-CTA kernel and a stage shrinks
// from 48 KB to 32 KB: six stages fit where four did.
//
// Roles per CTA: warp 0 = TMA producer for this CTA's operands; warp 1 = in the leader
// CTA (cluster rank 0) the MMA issuer (idle in the other CTA); warps 2-9 = epilogue of this
// CTA's 128 accumulator rows (the epilogue code is shared with the one-CTA kernel).  Every
// TMA load is a per-CTA load into the CTA's own shared memory (no multicast); both CTAs' loads
// of a stage complete on ONE barrier, in the leader, which the .cta_group::2 form of the copy
// permits; only the leader's producer announces the pair's byte count on it.  The other
// cluster-wide operations are the epilogues' mbarrier arrives on the leader's barriers, the
// tcgen05.commit that arrives in both CTAs and the two cluster barriers that bracket the
// kernel.  Arrives on a peer's barrier use the default (CTA-scope) semantics: a
// `.release.cluster` arrive once per stage cost about 0.5 us each and held the whole
// pipeline to a third of its rate.
//
// Measured on a B200 against the one-CTA kernel (same call, alternating runs): the Gram iteration
// of 18 blocks of 3584 x 4096 takes 13.6-14.4 ms instead of 15.7-16.8, the whole Llama-3-8B-shaped
// optimizer step 97.5-100.5 ms instead of 100.0-103.1.  It is the default; DIONW_GEMM_CTA_PAIRS=0
// selects the one-CTA kernel.
//
// Every spin-wait is bounded, as in the one-CTA kernel.
#pragma once

#include "gemm_sm100.cuh"

namespace dionw {
namespace gemm2 {

using gemm::Params;
using gemm::Tile;

constexpr int kPairM = 256;                        // rows of a pair's tile
constexpr int kBM = 128;                           // rows per CTA
constexpr int kBN = 256;
constexpr int kBK = 64;
constexpr int kHalfN = 128;                        // columns of B each CTA loads
constexpr int kStages = 6;
constexpr int kThreads = 320;
constexpr int kEpilogueThreads = 256;
constexpr uint32_t kABytes = kBM * kBK * 2;        // 16 KB
constexpr uint32_t kBBytes = kHalfN * kBK * 2;     // 16 KB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kPanelBytes = 64 * kBK * 2;
constexpr size_t kSmemBytes = size_t(kStages) * kStageBytes + 1024 + 256 + gemm::kMirrorBytes;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of the same shared-memory object in another CTA of the cluster.
__device__ __forceinline__ uint32_t peer_address(const void* local, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(gemm::smem_u32(local)), "r"(rank));
  return out;
}

__device__ __forceinline__ void remote_arrive(uint32_t cluster_address) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}

// Arrive with release semantics at cluster scope: what this thread wrote before (its own or the
// peer's shared memory) is visible to a thread of either CTA that then observes the phase with an
// acquire at cluster scope.  Used once per tile (the tile hand-out), never per stage.
__device__ __forceinline__ void remote_arrive_release(uint32_t cluster_address) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}

__device__ __forceinline__ void remote_store_s32(uint32_t cluster_address, int value) {
  asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(cluster_address), "r"(value) : "memory");
}

__device__ __forceinline__ bool mbar_try_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(gemm::smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait with the acquire at cluster scope (see gemm::mbar_wait for the protocol).
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                  uint64_t limit_ns) {
  uint32_t spins = 0;
  uint64_t start = 0;
  while (!mbar_try_cluster(bar, parity)) {
    if ((++spins & 1023u) == 0) {
      if (*abort_flag != 0) return false;
      const uint64_t now = gemm::global_ns();
      if (start == 0) start = now;
      else if (now - start > limit_ns) {
        *abort_flag = 1;
        if (status != nullptr) atomicExch(status, gemm::kWaitCode);
        return false;
      }
    }
  }
  return true;
}

// TMA load into this CTA's shared memory whose completion is signalled on a barrier of the
// pair's leader CTA (the .cta_group::2 form allows the barrier to be the peer's).
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint32_t leader_bar, int c0,
                                                 int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(gemm::smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc2(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gemm::smem_u32(slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc2(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}

__device__ __forceinline__ void umma2_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on the barrier at this offset in BOTH CTAs once the pair's MMAs issued so far have completed.
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          gemm::smem_u32(bar)),
      "h"(mask)
      : "memory");
}

// Instruction descriptor: fp32 accumulate, A K-major, M = 256 (128 rows in each CTA), N = 256.
template <typename T, bool kBMajorMN>
__device__ __forceinline__ uint32_t make_idesc2() {
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  uint32_t d = 0;
  d |= 1u << 4;
  d |= fmt << 7;
  d |= fmt << 10;
  d |= (kBMajorMN ? 1u : 0u) << 16;
  d |= uint32_t(kBN >> 3) << 17;
  d |= uint32_t(kPairM >> 4) << 24;
  return d;
}

// Pair tiles are 256 x 256.  General: groups of 4 tile rows sweep the columns.
__device__ __forceinline__ Tile general_tile(int t, const Params& p) {
  Tile tile;
  tile.batch = t / p.tiles_per_batch;
  int r = t - tile.batch * p.tiles_per_batch;
  const int group_rows = 4;
  const int per_group = group_rows * p.tiles_n;
  const int g = r / per_group;
  const int first = g * group_rows;
  const int rows_here = min(group_rows, p.tiles_m - first);
  r -= g * per_group;
  tile.tm = first + r % rows_here;
  tile.tn = r / rows_here;
  return tile;
}

// Symmetric: tile row i needs tile columns 0..i; i(i+1)/2 tiles precede row i.  (Walking the
// triangle in groups of four tile rows swept by columns, as the general schedule does, was measured
// and dropped: 18 blocks of 3584^2, K = 3584, 664 / 707 / 801 / 804 us against 646 / 733 / 776 / 740 us
// for A A^T plain / with Cin / with two outputs / with B != A -- no better on balance.)
__device__ __forceinline__ Tile sym_tile(int t, const Params& p) {
  Tile tile;
  tile.batch = t / p.tiles_per_batch;
  const int r = t - tile.batch * p.tiles_per_batch;
  int i = int((sqrtf(8.0f * float(r) + 1.0f) - 1.0f) * 0.5f);
  while (i * (i + 1) / 2 > r) --i;
  while ((i + 1) * (i + 2) / 2 <= r) ++i;
  tile.tm = i;
  tile.tn = r - i * (i + 1) / 2;
  return tile;
}

// ----------------------------------------------------------------------------
// tile hand-out
// ----------------------------------------------------------------------------
// A pair takes its tiles either in a fixed stride (tile = pair, pair + pairs, ...: no shared state)
// or from a counter in global memory, one atomicAdd per tile (Params::tile_counter non-null).  The
// second form is for products that run beside other kernels (NCCL's, another stream's): a pair whose
// CTAs become resident late, or not before the others are done, simply takes fewer tiles, where the
// fixed stride makes the whole product wait for it.
//
// The leader CTA's producer thread draws the index and publishes it to every consumer of the pair
// through a ring of kTileSlots entries kept in BOTH CTAs' shared memory: it writes the entry (its own
// copy and, through the cluster's shared-memory window, the peer's), then arrives with release at
// cluster scope on the slot's `tile_full` barrier of each CTA.  Consumers -- the leader's MMA thread,
// the peer's producer thread and the eight epilogue warps of each CTA, 18 in all -- wait on their own
// CTA's `tile_full` (acquire at cluster scope), read the entry and arrive on the LEADER's `tile_empty`
// barrier of the slot; the producer reuses a slot after all 18 have done so.  -1 ends the pair's work.
// When a pair has drawn its -1 it adds one to a second counter; the pair that brings that to the number
// of pairs knows that nobody will draw again and clears both counters for the next launch on the stream.
constexpr int kTileSlots = 4;
constexpr uint32_t kTileConsumers = 2 * (1 + kEpilogueThreads / 32);

// ----------------------------------------------------------------------------
// the kernel (launched as clusters of two CTAs)
// ----------------------------------------------------------------------------
template <typename InT, typename OutT, bool kBMajorMN, bool kSym>
__global__ void __launch_bounds__(kThreads, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  using namespace gemm;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + size_t(kStages) * kStageBytes);  // leader's: both CTAs' stage landed
  uint64_t* empty_bar = full_bar + kStages;   // both: the pair's MMAs on this stage completed
  uint64_t* acc_full = empty_bar + kStages;   // [2] both: accumulator complete
  uint64_t* acc_empty = acc_full + 2;         // [2] leader only: both CTAs' epilogues drained it
  uint64_t* tile_full = acc_empty + 2;        // [kTileSlots] both: the slot's tile index is written
  uint64_t* tile_empty = tile_full + kTileSlots;  // [kTileSlots] leader only: every consumer has read the slot
  int* tile_ring = reinterpret_cast<int*>(tile_empty + kTileSlots);  // [kTileSlots]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tile_ring + kTileSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint16_t* mirror_stage = reinterpret_cast<uint16_t*>(smem + size_t(kStages) * kStageBytes + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();       // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;
  const int total_tiles = p.tiles_per_batch * p.batches;
  const int k_blocks = (p.kdim + kBK - 1) / kBK;
  const bool dynamic = p.tile_counter != nullptr;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);   // the leader's producer arrives once with the pair's byte count
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * kEpilogueThreads);
    }
    for (int s = 0; s < kTileSlots; ++s) {
      mbar_init(&tile_full[s], 1);
      mbar_init(&tile_empty[s], kTileConsumers);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc2(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  cluster_sync();   // both CTAs' barriers exist before anyone arrives on a peer's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  gemm::griddep_wait();     // set-up above overlaps the tail of the previous product; global memory from here on
  gemm::griddep_launch();

  // The n-th tile of this pair for a consumer: its index, -1 when the pair is done, -2 when the wait
  // gave up.  Called by ONE thread per consumer (the single-thread roles themselves, lane 0 of an
  // epilogue warp), which also reports the slot as read.
  const uint32_t leader_tile_empty = peer_address(&tile_empty[0], 0);
  auto take_tile = [&](uint32_t n) -> int {
    if (!dynamic) {
      const long long t = (long long)pair + (long long)n * pairs;
      return t < total_tiles ? int(t) : -1;
    }
    const uint32_t slot = n % kTileSlots;
    if (!mbar_wait_cluster(&tile_full[slot], (n / kTileSlots) & 1u, abort_flag, p.status, p.wait_ns)) return -2;
    const int t = tile_ring[slot];
    remote_arrive_release(leader_tile_empty + slot * uint32_t(sizeof(uint64_t)));
    return t;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      // The draw for tile n + 1 is issued before the loads of tile n: its latency hides behind them.
      int drawn = (dynamic && rank == 0) ? atomicAdd(p.tile_counter, 1) : 0;
      for (uint32_t n = 0; ok; ++n) {
        int t;
        if (dynamic && rank == 0) {
          // publish the tile drawn last to the pair
          const uint32_t slot = n % kTileSlots;
          if (!mbar_wait_cluster(&tile_empty[slot], ((n / kTileSlots) & 1u) ^ 1u, abort_flag, p.status, p.wait_ns)) break;
          t = drawn < total_tiles ? drawn : -1;
          if (t >= 0) drawn = atomicAdd(p.tile_counter, 1);
          tile_ring[slot] = t;
          remote_store_s32(peer_address(&tile_ring[slot], 1), t);
          remote_arrive_release(peer_address(&tile_full[slot], 0));
          remote_arrive_release(peer_address(&tile_full[slot], 1));
          if (t < 0) {
            // nobody of this pair draws again; the last pair to get here clears the counters
            if (atomicAdd(p.tile_counter + 1, 1) == pairs - 1) {
              p.tile_counter[0] = 0;
              p.tile_counter[1] = 0;
              __threadfence();
            }
          }
        } else {
          t = take_tile(n);
        }
        if (t < 0) break;
        const Tile tile = kSym ? gemm2::sym_tile(t, p) : gemm2::general_tile(t, p);
        const int m0 = tile.tm * kPairM + int(rank) * kBM;
        const int n0 = tile.tn * kBN + int(rank) * kHalfN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1u;
          if (!mbar_wait(&empty_bar[s], phase ^ 1u, abort_flag, p.status, p.wait_ns)) { ok = false; break; }
          uint8_t* a_dst = smem + size_t(s) * kStageBytes;
          uint8_t* b_dst = a_dst + kABytes;
          const uint32_t leader_full = peer_address(&full_bar[s], 0);
          // The peer's bytes may land before the leader has announced them: the phase still
          // cannot complete before the leader's arrive, and the peer cannot run a phase ahead
          // because its empty barrier is released by the MMAs that consumed this one.
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * kStageBytes);
          tma_load_3d_pair(a_dst, &map_a, leader_full, kb * kBK, m0, tile.batch);
          if constexpr (kBMajorMN) {
#pragma unroll
            for (int panel = 0; panel < kHalfN / 64; ++panel)
              tma_load_3d_pair(b_dst + panel * kPanelBytes, &map_b, leader_full, n0 + panel * 64, kb * kBK, tile.batch);
          } else {
            tma_load_3d_pair(b_dst, &map_b, leader_full, kb * kBK, n0, tile.batch);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank != 0) {
      // the second CTA's MMA warp has nothing to issue
    } else if (lane == 0) {
      // ------------------------------------------------------------ MMA issuer (leader)
      const uint32_t idesc = make_idesc2<InT, kBMajorMN>();
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t local = 0; ok; ++local) {
        if (take_tile(local) < 0) break;
        const uint32_t acc = local & 1u;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, p.wait_ns)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * uint32_t(kBN);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1u;
          if (!mbar_wait(&full_bar[s], phase, abort_flag, p.status, p.wait_ns)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + size_t(s) * kStageBytes);
          const uint32_t b_addr = a_addr + kABytes;
          const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024);
          const uint64_t b_desc = kBMajorMN ? make_smem_desc(b_addr, kPanelBytes, 1024)
                                            : make_smem_desc(b_addr, 16, 1024);
#pragma unroll
          for (int j = 0; j < kBK / kUmmaK; ++j) {
            const uint64_t a_step = uint64_t((j * kUmmaK * 2) >> 4);
            const uint64_t b_step = kBMajorMN ? uint64_t((j * kUmmaK * 128) >> 4) : a_step;
            umma2_f16(tmem_d, a_desc + a_step, b_desc + b_step, idesc, (kb > 0 || j > 0) ? 1u : 0u);
          }
          umma2_commit_both(&empty_bar[s]);
        }
        if (ok) umma2_commit_both(&acc_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int ew = warp - 2;
    const int sub = warp & 3;
    const int first_chunk = (ew >> 2) * (kBN / 64);
    uint16_t* stage = mirror_stage + ew * 32 * kMirrorPitch;
    const uint32_t leader_empty[2] = {peer_address(&acc_empty[0], 0), peer_address(&acc_empty[1], 0)};
    bool ok = true;
    for (uint32_t local = 0; ok; ++local) {
      int t = 0;
      if (lane == 0) t = take_tile(local);   // one lane waits, reads and reports; the warp follows it
      t = __shfl_sync(0xffffffffu, t, 0);
      if (t < 0) break;
      const Tile tile = kSym ? gemm2::sym_tile(t, p) : gemm2::general_tile(t, p);
      const uint32_t acc = local & 1u;
      const uint32_t acc_phase = (local >> 1) & 1u;
      if (p.job != nullptr) {
        // The accumulator of this tile is still being summed: take rows of the streaming job
        // meanwhile, at most `per_wait` of them, one at a time, looking at the barrier in between.
        const int limit = p.job->per_wait;
        for (int taken = 0; taken < limit; ++taken) {
          long long row = -1;
          if (lane == 0 && !mbar_try(&acc_full[acc], acc_phase)) row = atomicAdd(&p.job->cursor, 1);
          row = __shfl_sync(0xffffffffu, row, 0);
          if (row < 0 || row >= p.job->total_rows) break;
          decay_job_row(p.job, row, lane);
        }
      }
      if (!epilogue_tile<InT, OutT, kSym>(p, tile.batch, tile.tm * kPairM + int(rank) * kBM, tile.tn * kBN,
                                          tmem_base + acc * uint32_t(kBN), &acc_full[acc], acc_phase, abort_flag,
                                          stage, sub, lane, first_chunk)) {
        ok = false;
        break;
      }
      tc_fence_before();
      remote_arrive(leader_empty[acc]);
    }
  }

  // ------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag != 0 && threadIdx.x == 0) {
    const uint64_t start = global_ns();
    while (global_ns() - start < 200000ull) {
    }
  }
  cluster_sync();   // the peer may still be reading this CTA's shared memory through the pair's MMAs
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc2(tmem_base, kTmemCols);
  }
}

}  // namespace gemm2
}  // namespace dionw
