// HBM-bound passes over bucketed momentum: accumulate + row scores, row
// selection, error-feedback decay + pack to the Newton-Schulz operand.
//
// Every byte these kernels touch is used once per step, so their loads and stores carry
// the streaming (evict-first) hint: they run next to the tensor-core products on another
// stream and must not push the products' operands out of L2.
//
// Row kernels give one warp to one row.  The row is walked in chunks of 1024
// elements; lane t of the warp owns the float4 slots t, t+32, ..., t+224 of a
// chunk, i.e. the "score lanes" 4(t+32q)+i of the documented 1024-lane order,
// so the fold below reproduces that order exactly: lanes are combined by
// halving (512, 256, 128 inside a thread; 64..4 by shuffles; 2, 1 inside
// thread 0).
#include "common.cuh"

namespace dionw {
namespace {

constexpr int kTable = 64;
constexpr int kWarpsPerBlock = 8;

struct RowTable {
  const void* ptr[kTable];
  long long row_end[kTable];  // exclusive prefix of rows, relative to the launch
  int n;
};

__device__ __forceinline__ int find_tensor(const RowTable& tab, long long row) {
  int lo = 0, hi = tab.n - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (row < tab.row_end[mid]) hi = mid; else lo = mid + 1;
  }
  return lo;
}

template <typename G>
__device__ __forceinline__ void load4(const G* p, bool vec, long long e, long long cols, float (&out)[4]);

template <>
__device__ __forceinline__ void load4<float>(const float* p, bool vec, long long e, long long cols, float (&out)[4]) {
  if (vec) {
    const float4 v = __ldcs(reinterpret_cast<const float4*>(p + e));
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = (e + i < cols) ? p[e + i] : 0.0f;
  }
}
template <>
__device__ __forceinline__ void load4<__half>(const __half* p, bool vec, long long e, long long cols, float (&out)[4]) {
  if (vec) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p + e);
    const __half2 a = *reinterpret_cast<const __half2*>(&raw.x);
    const __half2 b = *reinterpret_cast<const __half2*>(&raw.y);
    out[0] = __low2float(a); out[1] = __high2float(a); out[2] = __low2float(b); out[3] = __high2float(b);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = (e + i < cols) ? __half2float(p[e + i]) : 0.0f;
  }
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, bool vec, long long e, long long cols,
                                                      float (&out)[4]) {
  if (vec) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p + e);
    out[0] = __uint_as_float(raw.x << 16); out[1] = __uint_as_float(raw.x & 0xFFFF0000u);
    out[2] = __uint_as_float(raw.y << 16); out[3] = __uint_as_float(raw.y & 0xFFFF0000u);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = (e + i < cols) ? __bfloat162float(p[e + i]) : 0.0f;
  }
}

__device__ __forceinline__ void load4f(const float* p, bool vec, long long e, long long cols, float (&out)[4]) {
  if (vec) {
    const float4 v = __ldcs(reinterpret_cast<const float4*>(p + e));
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = (e + i < cols) ? p[e + i] : 0.0f;
  }
}

__device__ __forceinline__ void store4f(float* p, bool vec, long long e, long long cols, const float (&v)[4]) {
  if (vec) {
    __stcs(reinterpret_cast<float4*>(p + e), make_float4(v[0], v[1], v[2], v[3]));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (e + i < cols) p[e + i] = v[i];
  }
}

// Folds the 8 x 4 per-thread lane accumulators of a warp into one value, in
// the documented order.  The result is valid in lane 0.
__device__ __forceinline__ float fold_lanes(float (&acc)[8][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[0][i] = __fadd_rn(acc[0][i], acc[4][i]);
    acc[1][i] = __fadd_rn(acc[1][i], acc[5][i]);
    acc[2][i] = __fadd_rn(acc[2][i], acc[6][i]);
    acc[3][i] = __fadd_rn(acc[3][i], acc[7][i]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[0][i] = __fadd_rn(acc[0][i], acc[2][i]);
    acc[1][i] = __fadd_rn(acc[1][i], acc[3][i]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[0][i] = __fadd_rn(acc[0][i], acc[1][i]);
#pragma unroll
  for (int delta = 16; delta >= 1; delta >>= 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[0][i] = __fadd_rn(acc[0][i], __shfl_down_sync(0xffffffffu, acc[0][i], delta));
  }
  const float a = __fadd_rn(acc[0][0], acc[0][2]);
  const float b = __fadd_rn(acc[0][1], acc[0][3]);
  return __fadd_rn(a, b);
}

// M += G; scores = sum |M|; sumsq = sum M^2 per row.
template <typename G>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
accumulate_row_l1_kernel(const RowTable tab, float* __restrict__ momentum, float* __restrict__ scores,
                         float* __restrict__ sumsq, long long cols, long long total_rows, bool vec) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= total_rows) return;
  const int t = find_tensor(tab, row);
  const long long first = t == 0 ? 0 : tab.row_end[t - 1];
  const G* g = reinterpret_cast<const G*>(tab.ptr[t]) + (row - first) * cols;
  float* m = momentum + row * cols;
  float l1[8][4], sq[8][4];
#pragma unroll
  for (int q = 0; q < 8; ++q)
#pragma unroll
    for (int i = 0; i < 4; ++i) l1[q][i] = sq[q][i] = 0.0f;
  for (long long base = 0; base < cols; base += 1024) {
    float gv[8][4], mv[8][4];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const long long e = base + 4 * (lane + 32 * q);
      if (e < cols) {
        load4<G>(g, vec, e, cols, gv[q]);
        load4f(m, vec, e, cols, mv[q]);
      }
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const long long e = base + 4 * (lane + 32 * q);
      if (e < cols) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float v = __fadd_rn(mv[q][i], gv[q][i]);
          mv[q][i] = v;
          // Elements past the row end were loaded as zero and add nothing.
          l1[q][i] = __fadd_rn(l1[q][i], fabsf(v));
          sq[q][i] = __fadd_rn(sq[q][i], __fmul_rn(v, v));
        }
        store4f(m, vec, e, cols, mv[q]);
      }
    }
  }
  const float s1 = fold_lanes(l1);
  const float s2 = fold_lanes(sq);
  if (lane == 0) {
    scores[row] = s1;
    sumsq[row] = s2;
  }
}

// m = M + G; M = decay m; u = m or G + decay m; sumsq = sum u^2 per row.
template <typename G>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
accumulate_copy_decay_kernel(const RowTable tab, float* __restrict__ momentum, float* __restrict__ u,
                             float* __restrict__ sumsq, long long cols, long long total_rows, float decay,
                             bool nesterov, bool vec) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= total_rows) return;
  const int t = find_tensor(tab, row);
  const long long first = t == 0 ? 0 : tab.row_end[t - 1];
  const G* g = reinterpret_cast<const G*>(tab.ptr[t]) + (row - first) * cols;
  float* m = momentum + row * cols;
  float* out = u + row * cols;
  float sq[8][4];
#pragma unroll
  for (int q = 0; q < 8; ++q)
#pragma unroll
    for (int i = 0; i < 4; ++i) sq[q][i] = 0.0f;
  for (long long base = 0; base < cols; base += 1024) {
    float gv[8][4], mv[8][4];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const long long e = base + 4 * (lane + 32 * q);
      if (e < cols) {
        load4<G>(g, vec, e, cols, gv[q]);
        load4f(m, vec, e, cols, mv[q]);
      }
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const long long e = base + 4 * (lane + 32 * q);
      if (e < cols) {
        float uv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float sum = __fadd_rn(mv[q][i], gv[q][i]);
          const float decayed = __fmul_rn(sum, decay);
          mv[q][i] = decayed;
          uv[i] = nesterov ? __fadd_rn(gv[q][i], decayed) : sum;
          sq[q][i] = __fadd_rn(sq[q][i], __fmul_rn(uv[i], uv[i]));
        }
        store4f(m, vec, e, cols, mv[q]);
        store4f(out, vec, e, cols, uv);
      }
    }
  }
  const float s2 = fold_lanes(sq);
  if (lane == 0) sumsq[row] = s2;
}

// ---------------------------------------------------------------------------
// row selection
// ---------------------------------------------------------------------------
constexpr int kSelectThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t bits = __float_as_uint(v);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

// One CTA per block: radix-select the k-th largest score, then list the chosen
// rows in ascending order (rows equal to the threshold are taken lowest first).
__global__ void __launch_bounds__(kSelectThreads)
select_rows_kernel(const float* __restrict__ scores, const float* __restrict__ sumsq, int rows, int k,
                   int32_t* __restrict__ index, int32_t* __restrict__ rowmap, float* __restrict__ frob) {
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_remaining;
  __shared__ uint32_t warp_totals[32];
  __shared__ float partial[kSelectThreads];
  const int tid = threadIdx.x;
  const long long b = blockIdx.x;
  const float* sc = scores + b * rows;
  const float* ss = sumsq + b * rows;

  const int warp = tid >> 5, lane = tid & 31;
  uint32_t prefix = 0, mask = 0, remaining = uint32_t(k);
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    // Scores of one block share sign and exponent, so in the first passes nearly every key
    // falls into one bin: the lanes of a warp that hit the same bin add once, together.
    for (int start = 0; start < rows; start += kSelectThreads) {
      const int r = start + tid;
      uint32_t bin = 256;   // not a candidate (or past the end)
      if (r < rows) {
        const uint32_t key = order_key(sc[r]);
        if ((key & mask) == prefix) bin = (key >> shift) & 255u;
      }
      const uint32_t peers = __match_any_sync(0xffffffffu, bin);
      if (bin < 256 && lane == __ffs(peers) - 1) atomicAdd(&hist[bin], uint32_t(__popc(peers)));
    }
    __syncthreads();
    // The highest bin whose count, added to the counts above it, reaches `remaining`: lane l of
    // warp 0 holds bins 8l..8l+7, a suffix sum over the lanes finds the lane, which finds the bin.
    if (warp == 0) {
      uint32_t cnt[8], own = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        cnt[i] = hist[lane * 8 + i];
        own += cnt[i];
      }
      uint32_t incl = own;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t v = __shfl_down_sync(0xffffffffu, incl, d);
        if (lane + d < 32) incl += v;
      }
      uint32_t above = incl - own;   // candidates in the bins of higher lanes
      if (above < remaining && remaining <= incl) {
        int found = 0;
        bool open = true;
#pragma unroll
        for (int i = 7; i > 0; --i) {
          if (open && above + cnt[i] >= remaining) {
            found = i;
            open = false;
          }
          if (open) above += cnt[i];
        }
        s_prefix = prefix | (uint32_t(lane * 8 + found) << shift);
        s_remaining = remaining - above;
      }
    }
    __syncthreads();
    prefix = s_prefix;
    remaining = s_remaining;
    mask |= 255u << shift;
    __syncthreads();
  }
  const uint32_t threshold = prefix;     // key of the k-th largest score
  const uint32_t take_equal = remaining; // rows equal to it that are still needed

  uint32_t base_gt = 0, base_eq = 0;
  float local = 0.0f;
  for (int start = 0; start < rows; start += kSelectThreads) {
    const int r = start + tid;
    uint32_t key = 0;
    bool gt = false, eq = false;
    if (r < rows) {
      key = order_key(sc[r]);
      gt = key > threshold;
      eq = key == threshold;
    }
    const uint32_t gt_ballot = __ballot_sync(0xffffffffu, gt);
    const uint32_t eq_ballot = __ballot_sync(0xffffffffu, eq);
    const uint32_t below = (1u << lane) - 1u;
    uint32_t gt_before = __popc(gt_ballot & below);
    uint32_t eq_before = __popc(eq_ballot & below);
    if (lane == 0) warp_totals[warp] = (__popc(gt_ballot) << 16) | __popc(eq_ballot);
    __syncthreads();
    uint32_t gt_total = 0, eq_total = 0;
    for (int w = 0; w < 32; ++w) {
      const uint32_t packed = warp_totals[w];
      if (w < warp) {
        gt_before += packed >> 16;
        eq_before += packed & 0xFFFFu;
      }
      gt_total += packed >> 16;
      eq_total += packed & 0xFFFFu;
    }
    if (r < rows) {
      const uint32_t eq_rank = base_eq + eq_before;
      const bool chosen = gt || (eq && eq_rank < take_equal);
      int32_t pos = -1;
      if (chosen) {
        const uint32_t eq_taken_before = eq_rank < take_equal ? eq_rank : take_equal;
        pos = int32_t(base_gt + gt_before + eq_taken_before);
        index[b * k + pos] = r;
        local = __fadd_rn(local, ss[r]);
      }
      rowmap[b * rows + r] = pos;
    }
    base_gt += gt_total;
    base_eq += eq_total;
    __syncthreads();
  }
  partial[tid] = local;
  __syncthreads();
  for (int width = kSelectThreads / 2; width >= 1; width >>= 1) {
    if (tid < width) partial[tid] = __fadd_rn(partial[tid], partial[tid + width]);
    __syncthreads();
  }
  if (tid == 0) frob[b] = sqrtf(partial[0]);
}

__global__ void __launch_bounds__(kSelectThreads)
block_norms_kernel(const float* __restrict__ sumsq, int rows, float* __restrict__ frob) {
  __shared__ float partial[kSelectThreads];
  const int tid = threadIdx.x;
  const float* ss = sumsq + (long long)blockIdx.x * rows;
  float local = 0.0f;
  for (int r = tid; r < rows; r += kSelectThreads) local = __fadd_rn(local, ss[r]);
  partial[tid] = local;
  __syncthreads();
  for (int width = kSelectThreads / 2; width >= 1; width >>= 1) {
    if (tid < width) partial[tid] = __fadd_rn(partial[tid], partial[tid + width]);
    __syncthreads();
  }
  if (tid == 0) frob[blockIdx.x] = sqrtf(partial[0]);
}

// ---------------------------------------------------------------------------
// decay + pack
// ---------------------------------------------------------------------------
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <bool kBf16>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
pack_rows_kernel(float* __restrict__ src, const int32_t* __restrict__ index, const float* __restrict__ frob,
                 long long rows, long long k, long long cols, long long total, float decay, bool decay_rows,
                 float eps, float norm_scale, uint16_t* __restrict__ x, long long ldx, bool vec) {
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (item >= total) return;
  const long long b = item / k;
  const long long source_row = index ? (long long)index[item] : (item - b * k);
  float* m = src + (b * rows + source_row) * cols;
  uint16_t* dst = x + item * ldx;
  float denom;
  if (kBf16) {
    // The bf16 iterations normalise in bf16: norm, scaled norm and sum are each rounded.
    denom = bf16_round(bf16_round(bf16_round(frob[b]) * norm_scale) + eps);
  } else {
    denom = __fadd_rn(frob[b], eps);
  }
  // Four 16-byte loads per lane are requested before the first is used: a warp keeps 2 KB of
  // the row in flight, which is what the stream needs to approach the memory rate.
  constexpr int kUnroll = 4;
  for (long long e0 = 4LL * lane; e0 < cols; e0 += 128 * kUnroll) {
    float v[kUnroll][4];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long e = e0 + 128LL * u;
      if (e < cols) load4f(m, vec, e, cols, v[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long e = e0 + 128LL * u;
      if (e >= cols) break;
      uint16_t h[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (kBf16) {
          const __nv_bfloat16 r = __float2bfloat16_rn(__fdiv_rn(bf16_round(v[u][i]), denom));
          h[i] = *reinterpret_cast<const uint16_t*>(&r);
        } else {
          const __half r = __float2half_rn(__fdiv_rn(v[u][i], denom));
          h[i] = *reinterpret_cast<const uint16_t*>(&r);
        }
      }
      if (vec) {
        uint2 packed;
        packed.x = uint32_t(h[0]) | (uint32_t(h[1]) << 16);
        packed.y = uint32_t(h[2]) | (uint32_t(h[3]) << 16);
        __stcs(reinterpret_cast<uint2*>(dst + e), packed);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (e + i < cols) dst[e + i] = h[i];
      }
      if (decay_rows) {
#pragma unroll
        for (int i = 0; i < 4; ++i) v[u][i] = __fmul_rn(v[u][i], decay);
        store4f(m, vec, e, cols, v[u]);
      }
    }
  }
  // Zero the padding columns so that they add nothing to any product.
  for (long long e = cols + lane; e < ldx; e += 32) dst[e] = 0;
}

__global__ void transpose_2byte_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, long long rows,
                                       long long cols, long long ld_in, long long ld_out) {
  __shared__ uint16_t tile[64][66];
  const long long b = blockIdx.z;
  const uint16_t* src = in + b * rows * ld_in;
  uint16_t* dst = out + b * cols * ld_out;
  const long long r0 = (long long)blockIdx.y * 64, c0 = (long long)blockIdx.x * 64;
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const long long r = r0 + i;
    for (int j = threadIdx.x; j < 64; j += blockDim.x) {
      const long long c = c0 + j;
      tile[i][j] = (r < rows && c < cols) ? src[r * ld_in + c] : uint16_t(0);
    }
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const long long c = c0 + i;
    for (int j = threadIdx.x; j < 64; j += blockDim.x) {
      const long long r = r0 + j;
      if (c < cols && r < rows) dst[c * ld_out + r] = tile[j][i];
    }
  }
  // padding columns of the output rows
  if (blockIdx.y == 0) {
    for (int i = threadIdx.y; i < 64; i += blockDim.y) {
      const long long c = c0 + i;
      if (c < cols)
        for (long long p = rows + threadIdx.x; p < ld_out; p += blockDim.x) dst[c * ld_out + p] = 0;
    }
  }
}

template <typename Fn>
int for_each_table(const void* const* ptrs, const int64_t* rows_per_tensor, int n_tensors, Fn&& launch_one) {
  long long done_rows = 0;
  for (int start = 0; start < n_tensors; start += kTable) {
    RowTable tab;
    tab.n = (n_tensors - start < kTable) ? n_tensors - start : kTable;
    long long acc = 0;
    for (int i = 0; i < tab.n; ++i) {
      tab.ptr[i] = ptrs[start + i];
      acc += rows_per_tensor[start + i];
      tab.row_end[i] = acc;
    }
    const int st = launch_one(tab, done_rows, acc);
    if (st != DIONW_OK) return st;
    done_rows += acc;
  }
  return DIONW_OK;
}

bool table_vectorizable(const void* const* ptrs, int n, int64_t cols) {
  if (cols % 4 != 0) return false;
  for (int i = 0; i < n; ++i)
    if (!aligned16(ptrs[i])) return false;
  return true;
}

}  // namespace
}  // namespace dionw

using namespace dionw;

extern "C" int dionw_accumulate_row_l1_run(const void* const* grads, int grad_dtype, const int64_t* rows_per_tensor,
                                           int n_tensors, float* momentum, float* scores, float* sumsq, int64_t cols,
                                           void* stream_ptr) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  DIONW_REQUIRE(n_tensors > 0 && cols > 0, "accumulate_row_l1_run: empty run");
  DIONW_REQUIRE(grad_dtype >= DIONW_F32 && grad_dtype <= DIONW_BF16, "accumulate_row_l1_run: bad gradient dtype");
  const bool vec = table_vectorizable(grads, n_tensors, cols) && aligned16(momentum);
  return for_each_table(grads, rows_per_tensor, n_tensors, [&](const RowTable& tab, long long row0, long long nrows) {
    if (nrows == 0) return DIONW_OK;
    const unsigned grid = unsigned((nrows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    float* m = momentum + row0 * cols;
    if (grad_dtype == DIONW_F32)
      accumulate_row_l1_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(tab, m, scores + row0, sumsq + row0, cols, nrows, vec);
    else if (grad_dtype == DIONW_F16)
      accumulate_row_l1_kernel<__half><<<grid, kWarpsPerBlock * 32, 0, stream>>>(tab, m, scores + row0, sumsq + row0, cols, nrows, vec);
    else
      accumulate_row_l1_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, stream>>>(tab, m, scores + row0, sumsq + row0, cols, nrows, vec);
    return launch_status("accumulate_row_l1_kernel");
  });
}

extern "C" int dionw_accumulate_copy_decay_run(const void* const* grads, int grad_dtype,
                                               const int64_t* rows_per_tensor, int n_tensors, float* momentum,
                                               float* u, float* sumsq, int64_t cols, float decay, int nesterov,
                                               void* stream_ptr) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  DIONW_REQUIRE(n_tensors > 0 && cols > 0, "accumulate_copy_decay_run: empty run");
  DIONW_REQUIRE(grad_dtype >= DIONW_F32 && grad_dtype <= DIONW_BF16, "accumulate_copy_decay_run: bad gradient dtype");
  const bool vec = table_vectorizable(grads, n_tensors, cols) && aligned16(momentum) && aligned16(u);
  return for_each_table(grads, rows_per_tensor, n_tensors, [&](const RowTable& tab, long long row0, long long nrows) {
    if (nrows == 0) return DIONW_OK;
    const unsigned grid = unsigned((nrows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    float* m = momentum + row0 * cols;
    float* out = u + row0 * cols;
    const bool nest = nesterov != 0;
    if (grad_dtype == DIONW_F32)
      accumulate_copy_decay_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(tab, m, out, sumsq + row0, cols, nrows, decay, nest, vec);
    else if (grad_dtype == DIONW_F16)
      accumulate_copy_decay_kernel<__half><<<grid, kWarpsPerBlock * 32, 0, stream>>>(tab, m, out, sumsq + row0, cols, nrows, decay, nest, vec);
    else
      accumulate_copy_decay_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, stream>>>(tab, m, out, sumsq + row0, cols, nrows, decay, nest, vec);
    return launch_status("accumulate_copy_decay_kernel");
  });
}

extern "C" int dionw_select_rows(const float* scores, const float* sumsq, int64_t blocks, int64_t rows, int64_t k,
                                 int32_t* index, int32_t* rowmap, float* frob, void* stream_ptr) {
  DIONW_REQUIRE(blocks > 0 && rows > 0 && k > 0 && k <= rows, "select_rows: need 0 < k <= rows and blocks > 0");
  DIONW_REQUIRE(rows < (1LL << 30), "select_rows: too many rows");
  select_rows_kernel<<<unsigned(blocks), kSelectThreads, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      scores, sumsq, int(rows), int(k), index, rowmap, frob);
  return launch_status("select_rows_kernel");
}

extern "C" int dionw_block_norms(const float* sumsq, int64_t blocks, int64_t rows, float* frob, void* stream_ptr) {
  DIONW_REQUIRE(blocks > 0 && rows > 0, "block_norms: empty problem");
  block_norms_kernel<<<unsigned(blocks), kSelectThreads, 0, static_cast<cudaStream_t>(stream_ptr)>>>(sumsq, int(rows), frob);
  return launch_status("block_norms_kernel");
}

extern "C" int dionw_pack_rows(float* src, const int32_t* index, const float* frob, int64_t blocks, int64_t rows,
                               int64_t k, int64_t cols, float decay, int decay_rows, float eps, float norm_scale,
                               void* x, int x_dtype, int64_t ldx, void* stream_ptr) {
  DIONW_REQUIRE(blocks > 0 && rows > 0 && k > 0 && k <= rows && cols > 0, "pack_rows: empty problem");
  DIONW_REQUIRE(x_dtype == DIONW_F16 || x_dtype == DIONW_BF16, "pack_rows: x must be F16 or BF16");
  DIONW_REQUIRE(ldx >= cols, "pack_rows: ldx must be >= cols");
  const long long total = blocks * k;
  const bool vec = cols % 4 == 0 && ldx % 4 == 0 && aligned16(src) && aligned16(x);
  const unsigned grid = unsigned((total + kWarpsPerBlock - 1) / kWarpsPerBlock);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (x_dtype == DIONW_BF16)
    pack_rows_kernel<true><<<grid, kWarpsPerBlock * 32, 0, stream>>>(src, index, frob, rows, k, cols, total, decay,
                                                                      decay_rows != 0, eps, norm_scale,
                                                                      static_cast<uint16_t*>(x), ldx, vec);
  else
    pack_rows_kernel<false><<<grid, kWarpsPerBlock * 32, 0, stream>>>(src, index, frob, rows, k, cols, total, decay,
                                                                       decay_rows != 0, eps, norm_scale,
                                                                       static_cast<uint16_t*>(x), ldx, vec);
  return launch_status("pack_rows_kernel");
}

extern "C" int dionw_transpose_2byte(const void* in, void* out, int64_t blocks, int64_t rows, int64_t cols,
                                     int64_t ld_in, int64_t ld_out, void* stream_ptr) {
  DIONW_REQUIRE(blocks > 0 && rows > 0 && cols > 0, "transpose_2byte: empty problem");
  DIONW_REQUIRE(ld_in >= cols && ld_out >= rows, "transpose_2byte: leading dimensions too small");
  DIONW_REQUIRE(blocks <= 65535, "transpose_2byte: more than 65535 blocks in one call");
  const dim3 grid(unsigned((cols + 63) / 64), unsigned((rows + 63) / 64), unsigned(blocks));
  transpose_2byte_kernel<<<grid, dim3(32, 8), 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out), rows, cols, ld_in, ld_out);
  return launch_status("transpose_2byte_kernel");
}
