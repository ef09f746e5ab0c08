// Batched tcgen05 GEMM for sm_100a: TMA-fed shared-memory ring, accumulators in
// TMEM, a persistent tile loop with three warp roles (TMA producer, MMA issuer,
// eight epilogue warps).  Two tile schedules: every tile of a general product,
// or only the tiles on and below the diagonal of a symmetric product, whose
// strictly-lower 128x128 sub-blocks are also stored transposed.
//
// Tile 128 x 256 x 64 (one tcgen05.mma is 128 x 256 x 16), cta_group::1,
// 4-stage ring (48 KB per stage), two 256-column accumulators so the epilogue
// of tile t overlaps the main loop of tile t+1.  No cluster multicast anywhere.
//
// Every spin-wait is bounded; when one runs out the kernel stores a code in the
// device status word and leaves through the common teardown (TMEM is freed).
#pragma once

#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "decay_job.cuh"

namespace dionw {
namespace gemm {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;
constexpr int kStages = 4;
constexpr int kUmmaK = 16;
constexpr int kThreads = 320;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-9: epilogue
constexpr int kEpilogueThreads = 256;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kABytes = kBM * kBK * 2;        // 16 KB
constexpr uint32_t kBBytes = kBN * kBK * 2;        // 32 KB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kPanelBytes = 64 * kBK * 2;     // one 64-column panel of an MN-major B stage
constexpr int kMirrorPitch = 34;                   // halves per staged row: 17 words, conflict-free both ways
constexpr uint32_t kMirrorBytes = 8 * 32 * kMirrorPitch * 2;  // one 32 x 32 staging tile per epilogue warp
constexpr size_t kSmemBytes =
    size_t(kStages) * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + kMirrorBytes;

constexpr int kWaitCode = 0x7001;
constexpr uint64_t kWaitLimitNs = 2000000000ull;   // default limit of a bounded wait: two seconds

struct Params {
  // epilogue operands (element pointers; strides in elements)
  const void* cin;       // nullable
  void* out;
  void* out2;            // nullable: out + diag on the diagonal (symmetric schedule only)
  int64_t ldc, ldo;
  int64_t cin_batch, out_batch;
  float alpha, beta, diag;
  // problem
  int m, n, kdim;        // output m x n, reduction length kdim
  int batches;
  int tiles_m, tiles_n, tiles_per_batch;
  int mirror_diagonal;   // symmetric schedule with B != A: also mirror inside the diagonal sub-blocks
  float* rowsq;          // nullable, general products only: [batches, m, rowsq_parts] partial row sums of out^2
  int rowsq_parts;       // = 2 * tiles_n: one partial per 128 columns, written once each, summed by the reader
  int* tile_counter;     // two-CTA kernel: {next tile, pairs done} in global memory, or null for a fixed stride
  DecayJob* job;         // two-CTA kernel: streaming job the epilogue warps work on while they wait, or null
  int* status;           // device status word (may be null: the code is then not recorded)
  uint64_t wait_ns;      // limit of every bounded wait, in nanoseconds of %globaltimer
};

// ----------------------------------------------------------------------------
// PTX wrappers
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Programmatic dependent launch: the host launches every product with the stream-serialization
// attribute, so the CTAs of the next product may become resident, and run their set-up, as soon as
// CTAs of this one exit.  Nothing of global memory is read or written before griddep_wait()
// returns, which it does once the previous kernel of the stream has completed and its writes are
// visible; griddep_launch() then allows the kernel after this one to start the same way.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait: gives up after `limit_ns` (two seconds unless the launch says otherwise), flags
// the failure in the device status word and tells the rest of the CTA to stop through `abort_flag`.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, uint64_t limit_ns = kWaitLimitNs) {
  uint32_t spins = 0;
  uint64_t start = 0;   // the timer is first read after 1024 failed tries: a wait that ends soon never pays for it
  while (!mbar_try(bar, parity)) {
    if ((++spins & 1023u) == 0) {
      if (*abort_flag != 0) return false;
      const uint64_t now = global_ns();
      if (start == 0) start = now;
      else if (now - start > limit_ns) {
        *abort_flag = 1;
        if (status != nullptr) atomicExch(status, kWaitCode);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (Blackwell).
//   K-major operand  (rows of 64 elements = 128 B): SBO = 1024 B between 8-row groups, LBO unused (1).
//   MN-major operand (64-element panels, one 128 B row per k): LBO = bytes between
//   panels, SBO = 1024 B between 8-k groups.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((addr >> 4) & 0x3FFFu);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= uint64_t(1) << 46;  // descriptor version
  d |= uint64_t(2) << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16: fp32 accumulate, A K-major, M = 128, N = 256.
template <typename T, bool kBMajorMN>
__device__ __forceinline__ uint32_t make_idesc() {
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  uint32_t d = 0;
  d |= 1u << 4;                       // D format f32
  d |= fmt << 7;                      // A format
  d |= fmt << 10;                     // B format
  d |= (kBMajorMN ? 1u : 0u) << 16;   // B major
  d |= uint32_t(kBN >> 3) << 17;      // N
  d |= uint32_t(kBM >> 4) << 24;      // M
  return d;
}

// ----------------------------------------------------------------------------
// tile schedules
// ----------------------------------------------------------------------------
struct Tile {
  int batch, tm, tn;
};

// General product: groups of 8 tile rows sweep the tile columns, so that one
// wave of CTAs reuses a band of A and the whole of B from L2.
__device__ __forceinline__ Tile general_tile(int t, const Params& p) {
  Tile tile;
  tile.batch = t / p.tiles_per_batch;
  int r = t - tile.batch * p.tiles_per_batch;
  const int group_rows = 8;
  const int per_group = group_rows * p.tiles_n;
  const int g = r / per_group;
  const int first = g * group_rows;
  const int rows_here = min(group_rows, p.tiles_m - first);
  r -= g * per_group;
  tile.tm = first + r % rows_here;
  tile.tn = r / rows_here;
  return tile;
}

// Symmetric product: tile row i (128 rows) needs tile columns 0..i/2 (256
// columns each).  Rows 2q and 2q+1 hold q+1 tiles each, q(q+1) tiles precede them.
__device__ __forceinline__ int sym_tiles(int tiles_m) {
  const int q = tiles_m / 2;
  return q * (q + 1) + ((tiles_m & 1) ? q + 1 : 0);
}

__device__ __forceinline__ Tile sym_tile(int t, const Params& p) {
  Tile tile;
  tile.batch = t / p.tiles_per_batch;
  const int r = t - tile.batch * p.tiles_per_batch;
  int q = int((sqrtf(4.0f * float(r) + 1.0f) - 1.0f) * 0.5f);
  while (q * (q + 1) > r) --q;
  while ((q + 1) * (q + 2) <= r) ++q;
  const int rem = r - q * (q + 1);
  if (rem <= q) {
    tile.tm = 2 * q;
    tile.tn = rem;
  } else {
    tile.tm = 2 * q + 1;
    tile.tn = rem - (q + 1);
  }
  return tile;
}

template <typename OutT>
__device__ __forceinline__ OutT from_float(float v);
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ----------------------------------------------------------------------------
// epilogue of one accumulator: 128 rows (m_base ..) x 256 columns (n_base ..) of batch
// ``batch``, read from TMEM at ``tmem_acc`` by the warp that owns sub-partition ``sub``;
// this warp handles chunks first_chunk .. first_chunk+3 of the eight 32-column chunks.
// Returns false when the bounded wait for the accumulator ran out.
// ----------------------------------------------------------------------------
template <typename InT, typename OutT, bool kSym>
__device__ __forceinline__ bool epilogue_tile(const Params& p, int batch, int m_base, int n_base, uint32_t tmem_acc,
                                              uint64_t* acc_full_bar, uint32_t acc_phase, volatile int* abort_flag,
                                              uint16_t* stage, int sub, int lane, int first_chunk) {
  const InT* cin = reinterpret_cast<const InT*>(p.cin);
  OutT* out = reinterpret_cast<OutT*>(p.out);
  OutT* out2 = reinterpret_cast<OutT*>(p.out2);
  const int row_in_tile = sub * 32 + lane;
  const int row = m_base + row_in_tile;
  const int row0 = m_base + sub * 32;
  const bool row_ok = row < p.m;
  const InT* cin_row = cin ? cin + size_t(batch) * p.cin_batch + size_t(row) * p.ldc : nullptr;
  OutT* out_b = out + size_t(batch) * p.out_batch;
  OutT* out2_b = out2 ? out2 + size_t(batch) * p.out_batch : nullptr;
  // Class of the 32 x 32 piece at (row0, col0) under the symmetric schedule:
  // 0 stored as it is; 1 strictly below the diagonal: stored and stored transposed;
  // 2 strictly above: skipped (its mirror image writes it); 3 on the diagonal of a
  // product with B != A: lower triangle stored and mirrored element by element.
  auto class_of = [&](int col0) -> int {
    if constexpr (!kSym) return 0;
    if (col0 + 32 <= row0) return 1;
    if (col0 >= row0 + 32) return 2;
    return p.mirror_diagonal != 0 ? 3 : 0;
  };
  // Pieces wholly inside the matrix move between global memory and registers in
  // "piece order": lane l holds 8 consecutive elements of row 8*it + l/4 at column
  // 8*(l%4), it = 0..3, so one instruction touches 8 rows x 64 contiguous bytes.  The
  // accumulator arrives in "row order" (lane = row); a 32 x 34 staging tile in shared
  // memory converts between the two.
  const bool aligned = (p.ldo & 7) == 0 && (reinterpret_cast<uintptr_t>(out_b) & 15u) == 0 &&
                       (out2_b == nullptr || (reinterpret_cast<uintptr_t>(out2_b) & 15u) == 0) &&
                       (cin == nullptr || ((p.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(cin) & 15u) == 0 &&
                                           (p.cin_batch & 7) == 0));
  const bool rows_inside = row0 + 32 <= p.m;
  const int piece_row = lane >> 2, piece_col = (lane & 3) * 8;
  auto fast_piece = [&](int col0, int cls) { return aligned && rows_inside && col0 + 32 <= p.n && cls != 3; };
  // The epilogue is a chain of dependent latencies; the Cin piece of the next chunk is
  // requested before the current chunk is worked on.  (Requesting all four chunks of a
  // tile up front was measured slower: 48 more live registers for no shorter chain.)
  uint4 ahead[4];
  auto prefetch = [&](int chunk) {
    const int col0 = n_base + chunk * 32;
    const int cls = class_of(col0);
    if (cin == nullptr || cls == 2 || !fast_piece(col0, cls)) return;
    const InT* base = cin + size_t(batch) * p.cin_batch + size_t(row0 + piece_row) * p.ldc + col0 + piece_col;
#pragma unroll
    for (int it = 0; it < 4; ++it) ahead[it] = *reinterpret_cast<const uint4*>(base + size_t(8 * it) * p.ldc);
  };
  prefetch(first_chunk);   // does not depend on the accumulator: overlaps the wait below
  if (!mbar_wait(acc_full_bar, acc_phase, abort_flag, p.status, p.wait_ns)) return false;
  tc_fence_after();
  uint32_t* my_row = reinterpret_cast<uint32_t*>(stage + lane * kMirrorPitch);
  // Sum of the squares of this row's rounded results over the warp's 128 columns, for NorMuon:
  // the value is in registers here, so the row statistics need no second pass over the output.
  // One partial per (row, 128 columns), added left to right: the order is fixed.
  const bool want_sq = !kSym && p.rowsq != nullptr;
  float sq = 0.0f;
#pragma unroll 1
  for (int chunk = first_chunk; chunk < first_chunk + kBN / 64; ++chunk) {
    const int col0 = n_base + chunk * 32;
    const int cls = class_of(col0);
    uint4 now[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) now[j] = ahead[j];
    if (chunk + 1 < first_chunk + kBN / 64) prefetch(chunk + 1);
    if (col0 >= p.n) break;       // uniform over the warp
    if (cls == 2) continue;       // uniform over the warp
    uint32_t v[32];
    const uint32_t taddr = tmem_acc + (uint32_t(sub * 32) << 16) + uint32_t(chunk * 32);
    tmem_load32(taddr, v);
    if (fast_piece(col0, cls)) {
      __align__(16) OutT r[32];
      if (cin != nullptr) {
        // Cin: piece order -> staging tile -> row order
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          uint32_t* dst = reinterpret_cast<uint32_t*>(stage + (8 * it + piece_row) * kMirrorPitch + piece_col);
          dst[0] = now[it].x; dst[1] = now[it].y; dst[2] = now[it].z; dst[3] = now[it].w;
        }
        __syncwarp();
        __align__(16) InT c[32];
        uint32_t* cw = reinterpret_cast<uint32_t*>(c);
#pragma unroll
        for (int j = 0; j < 16; ++j) cw[j] = my_row[j];
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          r[j] = from_float<OutT>(fmaf(p.beta, to_float<InT>(c[j]), p.alpha * __uint_as_float(v[j])));
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = from_float<OutT>(p.alpha * __uint_as_float(v[j]));
      }
      if (want_sq) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float f = to_float<OutT>(r[j]);
          sq = fmaf(f, f, sq);
        }
      }
      // result: row order -> staging tile
      const uint32_t* words = reinterpret_cast<const uint32_t*>(r);
#pragma unroll
      for (int j = 0; j < 16; ++j) my_row[j] = words[j];
      __syncwarp();
      // stored as it is, in piece order
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int lr = 8 * it + piece_row;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(stage + lr * kMirrorPitch + piece_col);
        uint4 piece = make_uint4(src[0], src[1], src[2], src[3]);
        const size_t at = size_t(row0 + lr) * p.ldo + col0 + piece_col;
        *reinterpret_cast<uint4*>(out_b + at) = piece;
        if constexpr (kSym) {
          if (out2_b != nullptr) {
            const int d = row0 + lr - (col0 + piece_col);  // position of the diagonal inside the 8 elements
            if (d >= 0 && d < 8) {
              OutT* e = reinterpret_cast<OutT*>(&piece);
              e[d] = from_float<OutT>(to_float<OutT>(e[d]) + p.diag);
            }
            *reinterpret_cast<uint4*>(out2_b + at) = piece;
          }
        }
      }
      if constexpr (kSym) {
        if (cls == 1) {
          // stored transposed: gather columns of the staging tile
          const int seg = lane & 3;
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int cc = (lane >> 2) + 8 * it;  // source column = destination row
            __align__(16) uint16_t gathered[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) gathered[q] = stage[(seg * 8 + q) * kMirrorPitch + cc];
            const size_t at = size_t(col0 + cc) * p.ldo + row0 + seg * 8;
            *reinterpret_cast<uint4*>(out_b + at) = *reinterpret_cast<const uint4*>(gathered);
            if (out2_b != nullptr)
              *reinterpret_cast<uint4*>(out2_b + at) = *reinterpret_cast<const uint4*>(gathered);
          }
        }
      }
      __syncwarp();
      continue;
    }
    // ---- pieces at the matrix edge, unaligned operands, symmetrised diagonal pieces: one row per lane
    if (!row_ok) continue;
    __align__(16) OutT r[32];
    __align__(16) OutT r2[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float x = p.alpha * __uint_as_float(v[j]);
      if (cin_row != nullptr && col0 + j < p.n) x = fmaf(p.beta, to_float<InT>(cin_row[col0 + j]), x);
      r[j] = from_float<OutT>(x);
      if (want_sq && col0 + j < p.n) {
        const float f = to_float<OutT>(r[j]);
        sq = fmaf(f, f, sq);
      }
      if constexpr (kSym) r2[j] = (row == col0 + j) ? from_float<OutT>(to_float<OutT>(r[j]) + p.diag) : r[j];
    }
    OutT* dst = out_b + size_t(row) * p.ldo + col0;
    if (cls == 3) {
      // A B^T with B != A is symmetric only up to rounding: keep the lower triangle of
      // the diagonal piece and mirror it, so that the stored matrix is exactly symmetric.
      for (int j = 0; j < 32; ++j) {
        const int col = col0 + j;
        if (col > row || col >= p.n) continue;
        dst[j] = r[j];
        if (out2_b != nullptr) out2_b[size_t(row) * p.ldo + col] = r2[j];
        if (col < row) {
          out_b[size_t(col) * p.ldo + row] = r[j];
          if (out2_b != nullptr) out2_b[size_t(col) * p.ldo + row] = r[j];
        }
      }
      continue;
    }
    for (int j = 0; j < 32; ++j) {
      if (col0 + j >= p.n) break;
      dst[j] = r[j];
      if constexpr (kSym) {
        if (out2_b != nullptr) out2_b[size_t(row) * p.ldo + col0 + j] = r2[j];
        if (cls == 1) {
          out_b[size_t(col0 + j) * p.ldo + row] = r[j];
          if (out2_b != nullptr) out2_b[size_t(col0 + j) * p.ldo + row] = r[j];
        }
      }
    }
  }
  if (want_sq && row_ok) {
    const int part = 2 * (n_base / kBN) + first_chunk / (kBN / 64);
    p.rowsq[(size_t(batch) * p.m + row) * p.rowsq_parts + part] = sq;
  }
  return true;
}

// ----------------------------------------------------------------------------
// the kernel
// ----------------------------------------------------------------------------
template <typename InT, typename OutT, bool kBMajorMN, bool kSym>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + size_t(kStages) * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_full = empty_bar + kStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint16_t* mirror_stage = reinterpret_cast<uint16_t*>(smem + size_t(kStages) * kStageBytes + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.tiles_per_batch * p.batches;
  const int k_blocks = (p.kdim + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], kEpilogueThreads);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  griddep_wait();
  griddep_launch();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const Tile tile = kSym ? sym_tile(t, p) : general_tile(t, p);
        const int m0 = tile.tm * kBM, n0 = tile.tn * kBN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1u;
          if (!mbar_wait(&empty_bar[s], phase ^ 1u, abort_flag, p.status, p.wait_ns)) { ok = false; break; }
          uint8_t* a_dst = smem + size_t(s) * kStageBytes;
          uint8_t* b_dst = a_dst + kABytes;
          mbar_expect_tx(&full_bar[s], kStageBytes);
          tma_load_3d(a_dst, &map_a, &full_bar[s], kb * kBK, m0, tile.batch);
          if constexpr (kBMajorMN) {
#pragma unroll
            for (int panel = 0; panel < kBN / 64; ++panel)
              tma_load_3d(b_dst + panel * kPanelBytes, &map_b, &full_bar[s], n0 + panel * 64, kb * kBK, tile.batch);
          } else {
            tma_load_3d(b_dst, &map_b, &full_bar[s], kb * kBK, n0, tile.batch);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc<InT, kBMajorMN>();
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
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
            // K-major: 16 elements = 32 B further along each 128 B row.
            // MN-major: 16 k-rows of 128 B further.
            const uint64_t a_step = uint64_t((j * kUmmaK * 2) >> 4);
            const uint64_t b_step = kBMajorMN ? uint64_t((j * kUmmaK * 128) >> 4) : a_step;
            umma_f16(tmem_d, a_desc + a_step, b_desc + b_step, idesc, (kb > 0 || j > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&acc_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    // Eight warps: two per TMEM sub-partition (a warp may only read the 32 lanes
    // 32 * (warp % 4) ...), each taking four of the tile's eight 32-column chunks.
    const int ew = warp - 2;                  // 0..7
    const int sub = warp & 3;                 // TMEM lanes 32*sub .. 32*sub+31
    const int first_chunk = (ew >> 2) * (kBN / 64);
    uint16_t* stage = mirror_stage + ew * 32 * kMirrorPitch;
    uint32_t local = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
      const Tile tile = kSym ? sym_tile(t, p) : general_tile(t, p);
      const uint32_t acc = local & 1u;
      const uint32_t acc_phase = (local >> 1) & 1u;
      if (!epilogue_tile<InT, OutT, kSym>(p, tile.batch, tile.tm * kBM, tile.tn * kBN, tmem_base + acc * uint32_t(kBN),
                                          &acc_full[acc], acc_phase, abort_flag, stage, sub, lane, first_chunk)) {
        ok = false;
        break;
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
    }
  }

  // ------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag != 0 && threadIdx.x == 0) {
    // Give copies that may still be in flight time to land before the CTA's
    // shared memory is released.
    const uint64_t start = global_ns();
    while (global_ns() - start < 200000ull) {
    }
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace gemm
}  // namespace dionw
