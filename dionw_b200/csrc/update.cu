// NorMuon row statistics, the fused decay + update of the weights, fused
// AdamW and the EMA passes.  All HBM-bound streaming kernels.
#include <type_traits>

#include "common.cuh"

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
normuon_rows_kernel(const float* __restrict__ s, float* __restrict__ variance, const int32_t* __restrict__ index,
                    int rows, int k, float inv_count_cols, float weight, float eps, float step, bool normalize,
                    float* __restrict__ denom, float* __restrict__ scale) {
  __shared__ float scratch[kReduceThreads];
  const long long b = blockIdx.x;
  const int tid = threadIdx.x;
  if (!normalize) {
    for (int r = tid; r < k; r += kReduceThreads) denom[b * k + r] = 1.0f;
    if (tid == 0) scale[b] = step;
    return;
  }
  float n0 = 0.0f, n1 = 0.0f;
  for (int r = tid; r < k; r += kReduceThreads) {
    const long long slot = b * rows + (index ? index[b * k + r] : r);
    const float sr = s[b * k + r];
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
constexpr int kTable = 64;
struct WeightTable {
  void* ptr[kTable];
  long long row_end[kTable];
  int n;
};

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
apply_run_kernel(const WeightTable tab, long long first_row, long long total_rows, const uint16_t* __restrict__ o,
                 long long ldo, const int32_t* __restrict__ rowmap, const float* __restrict__ denom,
                 const float* __restrict__ scale, long long rows, long long k, long long cols, float decay_factor,
                 bool has_decay, bool vec) {
  const int lane = threadIdx.x & 31;
  const long long local = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (local >= total_rows) return;
  const long long row = first_row + local;  // row within the run
  const long long b = row / rows;
  const long long in_block = row - b * rows;
  const long long pos = rowmap ? (long long)rowmap[row] : in_block;
  if (pos < 0 && !has_decay) return;
  int lo = 0, hi = tab.n - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (local < tab.row_end[mid]) hi = mid; else lo = mid + 1;
  }
  const long long start = lo == 0 ? 0 : tab.row_end[lo - 1];
  float* w = reinterpret_cast<float*>(tab.ptr[lo]) + (local - start) * cols;
  if (pos < 0) {
    if (vec) {
#pragma unroll 4
      for (long long e = 4LL * lane; e < cols; e += 128) {
        float4 v = __ldcs(reinterpret_cast<const float4*>(w + e));
        v.x = __fmul_rn(v.x, decay_factor); v.y = __fmul_rn(v.y, decay_factor);
        v.z = __fmul_rn(v.z, decay_factor); v.w = __fmul_rn(v.w, decay_factor);
        __stcs(reinterpret_cast<float4*>(w + e), v);
      }
    } else {
      for (long long e = lane; e < cols; e += 32) w[e] = __fmul_rn(w[e], decay_factor);
    }
    return;
  }
  const uint16_t* src = o + (b * k + pos) * ldo;
  const float d = denom[b * k + pos];
  const float sc = scale[b];
  if (vec) {
#pragma unroll 4
    for (long long e = 4LL * lane; e < cols; e += 128) {
      float4 v = __ldcs(reinterpret_cast<const float4*>(w + e));
      const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(src + e));
      float x[4] = {v.x, v.y, v.z, v.w};
      const float ov[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
                           __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u)};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (has_decay) x[i] = __fmul_rn(x[i], decay_factor);
        x[i] = __fadd_rn(x[i], __fmul_rn(__fdiv_rn(ov[i], d), sc));
      }
      __stcs(reinterpret_cast<float4*>(w + e), make_float4(x[0], x[1], x[2], x[3]));
    }
  } else {
    for (long long e = lane; e < cols; e += 32) {
      float x = w[e];
      if (has_decay) x = __fmul_rn(x, decay_factor);
      const float ov = __uint_as_float(uint32_t(src[e]) << 16);
      w[e] = __fadd_rn(x, __fmul_rn(__fdiv_rn(ov, d), sc));
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
adamw_multi_kernel(const AdamTable tab, float lr, float beta1, float beta2, float weight_decay, float eps) {
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

extern "C" int dionw_normuon_rows(const float* s, float* variance, const int32_t* index, int64_t blocks, int64_t rows,
                                  int64_t k, int64_t cols, float weight, float eps, float step, int normalize,
                                  float* denom, float* scale, void* stream_ptr) {
  DIONW_REQUIRE(blocks > 0 && rows > 0 && k > 0 && k <= rows && cols > 0, "normuon_rows: bad shape");
  normuon_rows_kernel<<<unsigned(blocks), kReduceThreads, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      s, variance, index, int(rows), int(k), 1.0f / float(cols), weight, eps, step, normalize != 0, denom, scale);
  return launch_status("normuon_rows_kernel");
}

extern "C" int dionw_apply_run(void* const* weights, const int64_t* rows_per_tensor, int n_tensors, const void* o,
                               int64_t ldo, const int32_t* rowmap, const float* denom, const float* scale,
                               int64_t rows, int64_t k, int64_t cols, float decay_factor, int has_decay,
                               void* stream_ptr) {
  DIONW_REQUIRE(n_tensors > 0 && rows > 0 && k > 0 && cols > 0, "apply_run: empty run");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  bool vec = cols % 4 == 0 && ldo % 4 == 0 && aligned16(o);
  for (int i = 0; i < n_tensors; ++i) vec = vec && aligned16(weights[i]);
  long long done = 0;
  for (int start = 0; start < n_tensors; start += kTable) {
    WeightTable tab;
    tab.n = (n_tensors - start < kTable) ? n_tensors - start : kTable;
    long long acc = 0;
    for (int i = 0; i < tab.n; ++i) {
      tab.ptr[i] = weights[start + i];
      acc += rows_per_tensor[start + i];
      tab.row_end[i] = acc;
    }
    if (acc > 0) {
      const unsigned grid = unsigned((acc + kWarpsPerBlock - 1) / kWarpsPerBlock);
      apply_run_kernel<<<grid, kWarpsPerBlock * 32, 0, stream>>>(tab, done, acc, static_cast<const uint16_t*>(o), ldo,
                                                                 rowmap, denom, scale, rows, k, cols, decay_factor,
                                                                 has_decay != 0, vec);
      const int st = launch_status("apply_run_kernel");
      if (st != DIONW_OK) return st;
    }
    done += acc;
  }
  return DIONW_OK;
}

extern "C" int dionw_adamw_multi(void* const* params, const void* const* grads, void* const* exp_avg,
                                 void* const* exp_avg_sq, void* const* steps, const int64_t* numels, int n_tensors,
                                 float lr, float beta1, float beta2, float weight_decay, float eps,
                                 void* stream_ptr) {
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
        adamw_multi_kernel<<<blocks, kAdamThreads, 0, stream>>>(tab, lr, beta1, beta2, weight_decay, eps);
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
