// NorMuon row statistics, the fused decay + update of the weights, fused
// AdamW and the EMA passes.  All HBM-bound streaming kernels.
#include <type_traits>

#include "common.cuh"
#include "decay_job.cuh"

namespace dionw {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kReduceThreads = 1024;

// ---------------------------------------------------------------------------
// NorMuon
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
row_sumsq_bf16_kernel(const uint16_t* __restrict__ o, long long total_rows, long long cols, long long ldo,
                      float* __restrict__ s, bool vec) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= total_rows) return;
  const uint16_t* src = o + row * ldo;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (vec) {
    for (long long e = 8LL * lane; e < cols; e += 256) {
      const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(src + e));
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xFFFF0000u);
        acc[2 * i] = fmaf(lo, lo, acc[2 * i]);
        acc[2 * i + 1] = fmaf(hi, hi, acc[2 * i + 1]);
      }
    }
  } else {
    for (long long e = lane; e < cols; e += 32) {
      const float v = __uint_as_float(uint32_t(src[e]) << 16);
      acc[0] = fmaf(v, v, acc[0]);
    }
  }
  float sum = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
#pragma unroll
  for (int delta = 16; delta >= 1; delta >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, delta);
  if (lane == 0) s[row] = sum;
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int tid = threadIdx.x;
  scratch[tid] = v;
  __syncthreads();
  for (int width = kReduceThreads / 2; width >= 1; width >>= 1) {
    if (tid < width) scratch[tid] += scratch[tid + width];
    __syncthreads();
  }
  const float total = scratch[0];
  __syncthreads();
  return total;
}

// One CTA per block: new row variances, row denominators, block scale.
__global__ void __launch_bounds__(kReduceThreads)
normuon_rows_kernel(const float* __restrict__ s, int parts, float* __restrict__ variance,
                    const int32_t* __restrict__ index, int rows, int k, float inv_count_cols, float weight, float eps,
                    float step_host, const float* __restrict__ step_device, bool normalize,
                    float* __restrict__ denom, float* __restrict__ scale) {
  __shared__ float scratch[kReduceThreads];
  const long long b = blockIdx.x;
  const int tid = threadIdx.x;
  const float step = step_device != nullptr ? *step_device : step_host;
  if (!normalize) {
    for (int r = tid; r < k; r += kReduceThreads) denom[b * k + r] = 1.0f;
    if (tid == 0) scale[b] = step;
    return;
  }
  float n0 = 0.0f, n1 = 0.0f;
  for (int r = tid; r < k; r += kReduceThreads) {
    const long long slot = b * rows + (index ? index[b * k + r] : r);
    // a row's sum of squares arrives whole (parts == 1) or as partials per 128 columns,
    // added here left to right
    const float* partial = s + (b * k + r) * parts;
    float sr = 0.0f;
    if ((parts & 3) == 0 && (reinterpret_cast<uintptr_t>(s) & 15u) == 0) {
      for (int j = 0; j < parts; j += 4) {   // same order, four partials per load
        const float4 q = __ldcs(reinterpret_cast<const float4*>(partial + j));
        sr = (((sr + q.x) + q.y) + q.z) + q.w;
      }
    } else {
      for (int j = 0; j < parts; ++j) sr += partial[j];
    }
    const float mean = sr * inv_count_cols;
    const float old = variance[slot];
    // torch.lerp: start + weight * (end - start) for weight < 0.5, else the mirrored form.
    const float v = weight < 0.5f ? fmaf(weight, mean - old, old) : mean - (mean - old) * (1.0f - weight);
    variance[slot] = v;
    const float d = sqrtf(v) + eps;
    denom[b * k + r] = d;
    n0 += sr;
    n1 += sr / (d * d);
  }
  const float total0 = block_sum(n0, scratch);
  const float total1 = block_sum(n1, scratch);
  if (tid == 0) {
    const float restore = sqrtf(total0) / fmaxf(sqrtf(total1), eps);
    scale[b] = restore * step;
  }
}

// ---------------------------------------------------------------------------
// weights: decay every row, add the update to the selected rows
// ---------------------------------------------------------------------------
// One launch updates up to kTable weight tensors.  Every tensor brings its own
// update rows, row map, row divisors and block scales (pointers at ITS first
// block), so tensors whose updates were computed by different ranks, and lie in
// different receive slots, share a launch.
constexpr int kTable = 64;
struct ApplyEntry {
  float* w;
  const uint16_t* o;        // bf16 [blocks of this tensor, k, ldo]
  const int32_t* rowmap;    // [blocks of this tensor, rows] or null: every row is updated
  const float* denom;       // [blocks of this tensor, k]
  const float* scale;       // [blocks of this tensor]
  long long row_end;        // rows of this and the earlier tensors of the launch
};
struct ApplyTable {
  ApplyEntry e[kTable];
  int n;
};

// The kernel only streams: what hides the memory latency is the number of rows in flight, so the
// register count is held down (32-bit indices inside a row, the update's scale folded once per row).
__global__ void __launch_bounds__(kWarpsPerBlock * 32, 6)
apply_run_kernel(const ApplyTable tab, long long total_rows, int ldo, int rows, int k, int cols, float decay_host,
                 const float* __restrict__ decay_device, bool has_decay, bool vec, const DecayJob* __restrict__ job) {
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;   // one row per warp; the launch chooses the CTA size
  const long long stride = (long long)gridDim.x * warps;
  // Rows below this were offered to the tensor-core kernels' streaming job: the unselected ones among
  // them are decayed already.
  long long decayed_below = 0;
  if (job != nullptr) {
    const long long handed_out = job->cursor;
    decayed_below = handed_out < total_rows ? handed_out : total_rows;
  }
  for (long long local = (long long)blockIdx.x * warps + (threadIdx.x >> 5); local < total_rows; local += stride) {
    int lo = 0, hi = tab.n - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (local < tab.e[mid].row_end) hi = mid; else lo = mid + 1;
    }
    const long long row = local - (lo == 0 ? 0 : tab.e[lo - 1].row_end);  // row within the tensor
    const int b = int(row / rows);
    const int32_t* rowmap = tab.e[lo].rowmap;
    const int pos = rowmap ? rowmap[row] : int(row - (long long)b * rows);
    if (pos < 0 && (!has_decay || local < decayed_below)) continue;
    float* __restrict__ w = tab.e[lo].w + row * cols;
    const float decay_factor = decay_device != nullptr ? __ldg(decay_device) : decay_host;
    if (pos < 0) {
      if (vec) {
        float4* w4 = reinterpret_cast<float4*>(w);
        const int n4 = cols >> 2;
#pragma unroll 4
        for (int i = lane; i < n4; i += 32) {
          float4 v = __ldcs(w4 + i);
          v.x = __fmul_rn(v.x, decay_factor); v.y = __fmul_rn(v.y, decay_factor);
          v.z = __fmul_rn(v.z, decay_factor); v.w = __fmul_rn(v.w, decay_factor);
          __stcs(w4 + i, v);
        }
      } else {
        for (int e = lane; e < cols; e += 32) w[e] = __fmul_rn(w[e], decay_factor);
      }
      continue;
    }
    const long long orow = (long long)b * k + pos;
    const uint16_t* __restrict__ src = tab.e[lo].o + orow * ldo;
    const float d = tab.e[lo].denom[orow];
    const float sc = tab.e[lo].scale[b];
    if (vec) {
      float4* w4 = reinterpret_cast<float4*>(w);
      const uint2* s2 = reinterpret_cast<const uint2*>(src);
      const int n4 = cols >> 2;
#pragma unroll 4
      for (int i = lane; i < n4; i += 32) {
        float4 v = __ldcs(w4 + i);
        const uint2 raw = __ldcs(s2 + i);
        float x[4] = {v.x, v.y, v.z, v.w};
        const float ov[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
                             __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u)};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (has_decay) x[j] = __fmul_rn(x[j], decay_factor);
          x[j] = __fadd_rn(x[j], __fmul_rn(__fdiv_rn(ov[j], d), sc));
        }
        __stcs(w4 + i, make_float4(x[0], x[1], x[2], x[3]));
      }
    } else {
      for (int e = lane; e < cols; e += 32) {
        float x = w[e];
        if (has_decay) x = __fmul_rn(x, decay_factor);
        const float ov = __uint_as_float(uint32_t(src[e]) << 16);
        w[e] = __fadd_rn(x, __fmul_rn(__fdiv_rn(ov, d), sc));
      }
    }
  }
}

// ---------------------------------------------------------------------------
// AdamW
// ---------------------------------------------------------------------------
constexpr int kAdamTable = 48;
constexpr int kAdamThreads = 256;
constexpr int kAdamChunk = kAdamThreads * 16;  // elements per CTA

struct AdamTable {
  float* p[kAdamTable];
  const float* g[kAdamTable];
  float* m[kAdamTable];
  float* v[kAdamTable];
  float* step[kAdamTable];
  long long numel[kAdamTable];
  unsigned block_end[kAdamTable];
  int n;
};

__global__ void adamw_bump_steps_kernel(const AdamTable tab) {
  const int i = threadIdx.x;
  if (i < tab.n) *tab.step[i] += 1.0f;
}

__device__ __forceinline__ void adamw_math(float& p, float g, float& m, float& v, float lr, float beta1, float beta2,
                                           float weight_decay, float eps, float step_size, float bc2_sqrt) {
  if (weight_decay != 0.0f) p -= lr * weight_decay * p;
  m = fmaf(beta1, m, fmaf(-beta1, g, g));
  const float gg = g * g;
  v = fmaf(beta2, v, fmaf(-beta2, gg, gg));
  const float denom = sqrtf(v) / bc2_sqrt + eps;
  p -= step_size * m / denom;
}

__global__ void __launch_bounds__(kAdamThreads)
adamw_multi_kernel(const AdamTable tab, float lr_host, float beta1, float beta2, float weight_decay_host, float eps,
                   const float* __restrict__ hyper_device) {
  // learning rate and weight decay come from device memory when the caller keeps them there
  const float lr = hyper_device != nullptr ? hyper_device[0] : lr_host;
  const float weight_decay = hyper_device != nullptr ? hyper_device[1] : weight_decay_host;
  int lo = 0, hi = tab.n - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (blockIdx.x < tab.block_end[mid]) hi = mid; else lo = mid + 1;
  }
  const unsigned first_block = lo == 0 ? 0u : tab.block_end[lo - 1];
  const long long base = (long long)(blockIdx.x - first_block) * kAdamChunk;
  const long long n = tab.numel[lo];
  float* __restrict__ p = tab.p[lo];
  const float* __restrict__ g = tab.g[lo];
  float* __restrict__ m = tab.m[lo];
  float* __restrict__ v = tab.v[lo];
  const float step = *tab.step[lo];
  const float bc1 = 1.0f - powf(beta1, step);
  const float bc2_sqrt = sqrtf(1.0f - powf(beta2, step));
  const float step_size = lr / bc1;
  const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                     reinterpret_cast<uintptr_t>(v)) & 15u) == 0;
  if (vec && base + kAdamChunk <= n) {
    float4 pv[4], gv[4], mv[4], vv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long e = base + 4LL * (threadIdx.x + j * kAdamThreads);
      pv[j] = __ldcs(reinterpret_cast<const float4*>(p + e));
      gv[j] = __ldcs(reinterpret_cast<const float4*>(g + e));
      mv[j] = __ldcs(reinterpret_cast<const float4*>(m + e));
      vv[j] = __ldcs(reinterpret_cast<const float4*>(v + e));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long e = base + 4LL * (threadIdx.x + j * kAdamThreads);
      adamw_math(pv[j].x, gv[j].x, mv[j].x, vv[j].x, lr, beta1, beta2, weight_decay, eps, step_size, bc2_sqrt);
      adamw_math(pv[j].y, gv[j].y, mv[j].y, vv[j].y, lr, beta1, beta2, weight_decay, eps, step_size, bc2_sqrt);
      adamw_math(pv[j].z, gv[j].z, mv[j].z, vv[j].z, lr, beta1, beta2, weight_decay, eps, step_size, bc2_sqrt);
      adamw_math(pv[j].w, gv[j].w, mv[j].w, vv[j].w, lr, beta1, beta2, weight_decay, eps, step_size, bc2_sqrt);
      __stcs(reinterpret_cast<float4*>(p + e), pv[j]);
      __stcs(reinterpret_cast<float4*>(m + e), mv[j]);
      __stcs(reinterpret_cast<float4*>(v + e), vv[j]);
    }
  } else {
    const long long end = base + kAdamChunk < n ? base + kAdamChunk : n;
    for (long long e = base + threadIdx.x; e < end; e += kAdamThreads) {
      float pe = p[e], me = m[e], ve = v[e];
      adamw_math(pe, g[e], me, ve, lr, beta1, beta2, weight_decay, eps, step_size, bc2_sqrt);
      p[e] = pe; m[e] = me; v[e] = ve;
    }
  }
}

// ---------------------------------------------------------------------------
// EMA
// ---------------------------------------------------------------------------
constexpr int kEmaTable = 96;
constexpr int kEmaThreads = 256;
constexpr int kEmaChunk = kEmaThreads * 16;

struct EmaTable {
  float* dst[kEmaTable];
  const void* src[kEmaTable];
  long long numel[kEmaTable];
  unsigned block_end[kEmaTable];
  int n;
};

enum class EmaOp { kCopy, kLerp };

__device__ __forceinline__ float lerp_step(float shadow, float source, float weight) {
  const float diff = source - shadow;
  return weight < 0.5f ? fmaf(weight, diff, shadow) : source - diff * (1.0f - weight);
}

template <typename S, EmaOp kOp>
__global__ void __launch_bounds__(kEmaThreads)
ema_multi_kernel(const EmaTable tab, float weight) {
  int lo = 0, hi = tab.n - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (blockIdx.x < tab.block_end[mid]) hi = mid; else lo = mid + 1;
  }
  const unsigned first_block = lo == 0 ? 0u : tab.block_end[lo - 1];
  const long long base = (long long)(blockIdx.x - first_block) * kEmaChunk;
  const long long n = tab.numel[lo];
  float* __restrict__ dst = tab.dst[lo];
  const S* __restrict__ src = reinterpret_cast<const S*>(tab.src[lo]);
  if (std::is_same<S, float>::value && base + kEmaChunk <= n &&
      ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0) {
    const float* fsrc = reinterpret_cast<const float*>(src);
    float4 sv[4], dv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long e = base + 4LL * (threadIdx.x + j * kEmaThreads);
      sv[j] = __ldcs(reinterpret_cast<const float4*>(fsrc + e));
      if (kOp == EmaOp::kLerp) dv[j] = __ldcs(reinterpret_cast<const float4*>(dst + e));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long e = base + 4LL * (threadIdx.x + j * kEmaThreads);
      if (kOp == EmaOp::kLerp) {
        dv[j].x = lerp_step(dv[j].x, sv[j].x, weight); dv[j].y = lerp_step(dv[j].y, sv[j].y, weight);
        dv[j].z = lerp_step(dv[j].z, sv[j].z, weight); dv[j].w = lerp_step(dv[j].w, sv[j].w, weight);
      } else {
        dv[j] = sv[j];
      }
      __stcs(reinterpret_cast<float4*>(dst + e), dv[j]);
    }
  } else {
    const long long end = base + kEmaChunk < n ? base + kEmaChunk : n;
    for (long long e = base + threadIdx.x; e < end; e += kEmaThreads) {
      const float s = to_float<S>(src[e]);
      dst[e] = kOp == EmaOp::kLerp ? lerp_step(dst[e], s, weight) : s;
    }
  }
}

template <typename Table, int kCap, int kChunk, typename Fill, typename Launch>
int chunked_tables(const int64_t* numels, int n_tensors, Fill&& fill, Launch&& launch_one) {
  int start = 0;
  while (start < n_tensors) {
    Table tab;
    int count = 0;
    unsigned long long blocks = 0;
    while (start + count < n_tensors && count < kCap) {
      const int64_t n = numels[start + count];
      const unsigned long long need = (unsigned long long)((n + kChunk - 1) / kChunk);
      if (blocks + need > 0x7FFFFFFFull) break;
      fill(tab, count, start + count);
      blocks += need;
      tab.numel[count] = n;
      tab.block_end[count] = unsigned(blocks);
      ++count;
    }
    if (count == 0) {
      set_error("a tensor of %lld elements is too large for one launch", (long long)numels[start]);
      return DIONW_ERR_UNSUPPORTED;
    }
    tab.n = count;
    if (blocks > 0) {
      const int st = launch_one(tab, unsigned(blocks));
      if (st != DIONW_OK) return st;
    }
    start += count;
  }
  return DIONW_OK;
}

}  // namespace
}  // namespace dionw

using namespace dionw;

// Step scalars kept in device memory: the values travel as kernel arguments (copied when the
// launch is made, so the host may change its own copy at once) and are stored by one small kernel.
constexpr int kScalarsPerLaunch = 512;
struct ScalarTable {
  float v[kScalarsPerLaunch];
};

__global__ void write_scalars_kernel(const ScalarTable tab, float* __restrict__ dst, int n) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = tab.v[i];
}

extern "C" int dionw_write_scalars(float* dst, const float* values, int64_t n, void* stream_ptr) {
  DIONW_REQUIRE(dst != nullptr && values != nullptr && n >= 0, "write_scalars: null table");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  for (int64_t start = 0; start < n; start += kScalarsPerLaunch) {
    ScalarTable tab;
    const int count = int(n - start < kScalarsPerLaunch ? n - start : kScalarsPerLaunch);
    for (int i = 0; i < count; ++i) tab.v[i] = values[start + i];
    write_scalars_kernel<<<1, 128, 0, stream>>>(tab, dst + start, count);
    const int st = launch_status("write_scalars_kernel");
    if (st != DIONW_OK) return st;
  }
  return DIONW_OK;
}

extern "C" int dionw_row_sumsq_bf16(const void* o, int64_t blocks, int64_t k, int64_t cols, int64_t ldo, float* s,
                                    void* stream_ptr) {
  DIONW_REQUIRE(blocks > 0 && k > 0 && cols > 0 && ldo >= cols, "row_sumsq_bf16: bad shape");
  const long long total = blocks * k;
  const bool vec = cols % 8 == 0 && ldo % 8 == 0 && aligned16(o);
  const unsigned grid = unsigned((total + kWarpsPerBlock - 1) / kWarpsPerBlock);
  row_sumsq_bf16_kernel<<<grid, kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const uint16_t*>(o), total, cols, ldo, s, vec);
  return launch_status("row_sumsq_bf16_kernel");
}

extern "C" int dionw_normuon_rows(const float* s, int64_t parts, float* variance, const int32_t* index, int64_t blocks,
                                  int64_t rows, int64_t k, int64_t cols, float weight, float eps, float step,
                                  const float* step_device, int normalize, float* denom, float* scale,
                                  void* stream_ptr) {
  DIONW_REQUIRE(blocks > 0 && rows > 0 && k > 0 && k <= rows && cols > 0 && parts >= 1 && parts <= 4096,
                "normuon_rows: bad shape");
  normuon_rows_kernel<<<unsigned(blocks), kReduceThreads, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      s, int(parts), variance, index, int(rows), int(k), 1.0f / float(cols), weight, eps, step, step_device,
      normalize != 0, denom, scale);
  return launch_status("normuon_rows_kernel");
}

extern "C" int dionw_apply_round(void* const* weights, const int64_t* rows_per_tensor, const void* const* o,
                                 const int32_t* const* rowmap, const float* const* denom, const float* const* scale,
                                 int n_tensors, int64_t ldo, int64_t rows, int64_t k, int64_t cols,
                                 float decay_factor, const float* decay_device, int has_decay, int cta_warps,
                                 const void* decay_job, void* stream_ptr) {
  DIONW_REQUIRE(n_tensors > 0 && rows > 0 && k > 0 && cols > 0, "apply_round: empty round");
  DIONW_REQUIRE(rows < (1ll << 31) && cols < (1ll << 31) && ldo < (1ll << 31), "apply_round: a block dimension exceeds 2^31");
  DIONW_REQUIRE(cta_warps >= 0 && cta_warps <= kWarpsPerBlock, "apply_round: cta_warps must be 0 (default) .. %d",
                kWarpsPerBlock);
  const int warps = cta_warps == 0 ? kWarpsPerBlock : cta_warps;
  DIONW_REQUIRE(weights && rows_per_tensor && o && denom && scale, "apply_round: null table");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  bool vec = cols % 4 == 0 && ldo % 4 == 0;
  for (int i = 0; i < n_tensors; ++i) vec = vec && aligned16(weights[i]) && (reinterpret_cast<uintptr_t>(o[i]) & 7u) == 0;
  DIONW_REQUIRE(decay_job == nullptr || n_tensors <= kTable,
                "apply_round: a decay job covers at most %d tensors, the round has %d", kTable, n_tensors);
  for (int start = 0; start < n_tensors; start += kTable) {
    ApplyTable tab;
    tab.n = (n_tensors - start < kTable) ? n_tensors - start : kTable;
    long long acc = 0;
    for (int i = 0; i < tab.n; ++i) {
      const int t = start + i;
      DIONW_REQUIRE(rows_per_tensor[t] >= 0 && rows_per_tensor[t] % rows == 0,
                    "apply_round: tensor %d has %lld rows, not a multiple of the block's %lld", t,
                    (long long)rows_per_tensor[t], (long long)rows);
      acc += rows_per_tensor[t];
      tab.e[i] = ApplyEntry{static_cast<float*>(weights[t]), static_cast<const uint16_t*>(o[t]),
                            rowmap ? rowmap[t] : nullptr, denom[t], scale[t], acc};
    }
    if (acc > 0) {
      long long grid = (acc + warps - 1) / warps;
      if (grid > 0x7FFFFFFFll) grid = 0x7FFFFFFFll;   // the kernel walks the rows with a stride
      apply_run_kernel<<<unsigned(grid), warps * 32, 0, stream>>>(tab, acc, int(ldo), int(rows), int(k), int(cols),
                                                                  decay_factor, decay_device, has_decay != 0, vec,
                                                                  static_cast<const DecayJob*>(decay_job));
      const int st = launch_status("apply_run_kernel");
      if (st != DIONW_OK) return st;
    }
  }
  return DIONW_OK;
}

extern "C" int dionw_apply_run(void* const* weights, const int64_t* rows_per_tensor, int n_tensors, const void* o,
                               int64_t ldo, const int32_t* rowmap, const float* denom, const float* scale,
                               int64_t rows, int64_t k, int64_t cols, float decay_factor, int has_decay,
                               void* stream_ptr) {
  DIONW_REQUIRE(n_tensors > 0 && n_tensors <= 1024 && rows > 0 && k > 0 && cols > 0 && rows_per_tensor != nullptr,
                "apply_run: empty run (or more than 1024 tensors)");
  // The tensors of a run lie one after the other in the run's buffers.
  const void* o_of[1024];
  const int32_t* map_of[1024];
  const float* denom_of[1024];
  const float* scale_of[1024];
  long long row = 0;
  for (int i = 0; i < n_tensors; ++i) {
    const long long block = row / rows;
    o_of[i] = static_cast<const uint16_t*>(o) + block * k * ldo;
    map_of[i] = rowmap ? rowmap + row : nullptr;
    denom_of[i] = denom + block * k;
    scale_of[i] = scale + block;
    row += rows_per_tensor[i];
  }
  return dionw_apply_round(weights, rows_per_tensor, o_of, rowmap ? map_of : nullptr, denom_of, scale_of, n_tensors,
                           ldo, rows, k, cols, decay_factor, nullptr, has_decay, 0, nullptr, stream_ptr);
}

// ---------------------------------------------------------------------------
// the decay job of a round (decay_job.cuh)
// ---------------------------------------------------------------------------
namespace dionw {
namespace {
struct JobInit {
  float* w[kJobTensors];
  const int32_t* rowmap[kJobTensors];
  long long row_end[kJobTensors];
};

__global__ void decay_job_begin_kernel(DecayJob* job, const JobInit init, int n, int rows, int cols, int vec,
                                       int per_wait, long long total_rows, float decay_host,
                                       const float* decay_device) {
  const int i = threadIdx.x;
  if (i < n) {
    job->w[i] = init.w[i];
    job->rowmap[i] = init.rowmap[i];
    job->row_end[i] = init.row_end[i];
  }
  if (i == 0) {
    job->n = n;
    job->rows = rows;
    job->cols = cols;
    job->vec = vec;
    job->per_wait = per_wait;
    job->cursor = 0;
    job->total_rows = total_rows;
    job->decay_host = decay_host;
    job->decay_device = decay_device;
  }
}
}  // namespace
}  // namespace dionw

extern "C" size_t dionw_decay_job_bytes(void) { return sizeof(dionw::DecayJob); }

extern "C" int dionw_decay_job_begin(void* job, void* const* weights, const int32_t* const* rowmap,
                                     const int64_t* rows_per_tensor, int n_tensors, int64_t rows, int64_t cols,
                                     float decay_factor, const float* decay_device, int rows_per_wait,
                                     void* stream_ptr) {
  DIONW_REQUIRE(job != nullptr && (reinterpret_cast<uintptr_t>(job) & 15u) == 0, "decay_job_begin: job must be 16-byte aligned device memory");
  DIONW_REQUIRE(n_tensors > 0 && n_tensors <= kJobTensors, "decay_job_begin: 1 .. %d tensors (got %d)", kJobTensors,
                n_tensors);
  DIONW_REQUIRE(weights && rowmap && rows_per_tensor && rows > 0 && cols > 0 && cols < (1ll << 31) && rows < (1ll << 31),
                "decay_job_begin: bad shape");
  DIONW_REQUIRE(rows_per_wait >= 0 && rows_per_wait <= 64, "decay_job_begin: rows_per_wait must be 0 .. 64");
  JobInit init;
  long long acc = 0;
  bool vec = cols % 4 == 0;
  for (int i = 0; i < n_tensors; ++i) {
    DIONW_REQUIRE(rowmap[i] != nullptr, "decay_job_begin: tensor %d has no row map (every row is selected: nothing to decay ahead)", i);
    DIONW_REQUIRE(rows_per_tensor[i] >= 0 && rows_per_tensor[i] % rows == 0, "decay_job_begin: tensor %d has %lld rows, not a multiple of %lld", i, (long long)rows_per_tensor[i], (long long)rows);
    acc += rows_per_tensor[i];
    init.w[i] = static_cast<float*>(weights[i]);
    init.rowmap[i] = rowmap[i];
    init.row_end[i] = acc;
    vec = vec && aligned16(weights[i]);
  }
  DIONW_REQUIRE(acc < (1ll << 30), "decay_job_begin: too many rows for one job");
  decay_job_begin_kernel<<<1, kJobTensors, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<DecayJob*>(job), init, n_tensors, int(rows), int(cols), vec ? 1 : 0, rows_per_wait, acc, decay_factor,
      decay_device);
  return launch_status("decay_job_begin_kernel");
}

extern "C" int dionw_adamw_multi(void* const* params, const void* const* grads, void* const* exp_avg,
                                 void* const* exp_avg_sq, void* const* steps, const int64_t* numels, int n_tensors,
                                 float lr, float beta1, float beta2, float weight_decay, float eps,
                                 const float* hyper_device, void* stream_ptr) {
  DIONW_REQUIRE(n_tensors >= 0, "adamw_multi: negative tensor count");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  return chunked_tables<AdamTable, kAdamTable, kAdamChunk>(
      numels, n_tensors,
      [&](AdamTable& tab, int slot, int i) {
        tab.p[slot] = static_cast<float*>(params[i]);
        tab.g[slot] = static_cast<const float*>(grads[i]);
        tab.m[slot] = static_cast<float*>(exp_avg[i]);
        tab.v[slot] = static_cast<float*>(exp_avg_sq[i]);
        tab.step[slot] = static_cast<float*>(steps[i]);
      },
      [&](const AdamTable& tab, unsigned blocks) {
        adamw_bump_steps_kernel<<<1, kAdamTable, 0, stream>>>(tab);
        int st = launch_status("adamw_bump_steps_kernel");
        if (st != DIONW_OK) return st;
        adamw_multi_kernel<<<blocks, kAdamThreads, 0, stream>>>(tab, lr, beta1, beta2, weight_decay, eps,
                                                                hyper_device);
        return launch_status("adamw_multi_kernel");
      });
}

template <EmaOp kOp>
static int ema_launch(const EmaTable& tab, unsigned blocks, int source_dtype, float weight, cudaStream_t stream) {
  if (source_dtype == DIONW_F32)
    ema_multi_kernel<float, kOp><<<blocks, kEmaThreads, 0, stream>>>(tab, weight);
  else if (source_dtype == DIONW_F16)
    ema_multi_kernel<__half, kOp><<<blocks, kEmaThreads, 0, stream>>>(tab, weight);
  else
    ema_multi_kernel<__nv_bfloat16, kOp><<<blocks, kEmaThreads, 0, stream>>>(tab, weight);
  return launch_status("ema_multi_kernel");
}

extern "C" int dionw_ema_multi(void* const* shadows, const void* const* sources, const int64_t* numels, int n_tensors,
                               int source_dtype, float weight, int first, void* stream_ptr) {
  DIONW_REQUIRE(n_tensors >= 0, "ema_multi: negative tensor count");
  DIONW_REQUIRE(source_dtype >= DIONW_F32 && source_dtype <= DIONW_BF16, "ema_multi: bad source dtype");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  return chunked_tables<EmaTable, kEmaTable, kEmaChunk>(
      numels, n_tensors,
      [&](EmaTable& tab, int slot, int i) {
        tab.dst[slot] = static_cast<float*>(shadows[i]);
        tab.src[slot] = sources[i];
      },
      [&](const EmaTable& tab, unsigned blocks) {
        return first ? ema_launch<EmaOp::kCopy>(tab, blocks, source_dtype, weight, stream)
                     : ema_launch<EmaOp::kLerp>(tab, blocks, source_dtype, weight, stream);
      });
}

extern "C" int dionw_ema_stage_pack(const void* const* sources, const int64_t* numels, const int64_t* offsets,
                                    int n_tensors, int source_dtype, float* staging, void* stream_ptr) {
  DIONW_REQUIRE(n_tensors >= 0, "ema_stage_pack: negative tensor count");
  DIONW_REQUIRE(source_dtype >= DIONW_F32 && source_dtype <= DIONW_BF16, "ema_stage_pack: bad source dtype");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  return chunked_tables<EmaTable, kEmaTable, kEmaChunk>(
      numels, n_tensors,
      [&](EmaTable& tab, int slot, int i) {
        tab.dst[slot] = staging + offsets[i];
        tab.src[slot] = sources[i];
      },
      [&](const EmaTable& tab, unsigned blocks) {
        return ema_launch<EmaOp::kCopy>(tab, blocks, source_dtype, 0.0f, stream);
      });
}
