// A streaming job that the tensor-core kernels work on while their epilogue warps wait.
//
// The sharded step spends 8 B per weight element on every rank on the decoupled weight decay of
// rows that were NOT selected (three quarters of them): `w *= 1 - lr * wd`, HBM-bound, dependent on
// nothing but the row maps, which exist before the first Newton-Schulz product of the round.  A
// separate kernel cannot run beside the persistent products (their CTAs hold 54 K of an SM's 64 K
// registers), but the products' own eight epilogue warps wait about 15 us of every 24 us tile.  So a
// job describes the rows of a round's weights; an epilogue warp that finds its accumulator not ready
// draws a row from the job's cursor (one atomicAdd), decays it if the row map says it is unselected,
// and looks at its barrier again.  The weight update kernel that follows reads the cursor and leaves
// the rows below it alone unless they are selected.  Same multiplication on the same values, once per
// element: the results are bit-identical to the update kernel doing all of it.
#pragma once

#include <cstdint>

namespace dionw {

constexpr int kJobTensors = 64;

struct DecayJob {
  int n;                       // tensors
  int rows;                    // rows per block (the row map is [blocks, rows] per tensor)
  int cols;                    // fp32 elements per row
  int vec;                     // rows may be walked in float4
  int per_wait;                // rows one warp may take per tile it waits for
  int cursor;                  // next row to hand out (atomic); rows below min(cursor, total_rows) are done
  long long total_rows;
  float decay_host;
  const float* decay_device;   // overrides decay_host when non-null
  float* w[kJobTensors];
  const int32_t* rowmap[kJobTensors];
  long long row_end[kJobTensors];   // rows of this and the earlier tensors
};

// Decays row `row` of the job if it is not selected.  Called by all 32 lanes of a warp.
__device__ __forceinline__ void decay_job_row(const DecayJob* job, long long row, int lane) {
  int lo = 0, hi = job->n - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (row < job->row_end[mid]) hi = mid; else lo = mid + 1;
  }
  const long long local = row - (lo == 0 ? 0 : job->row_end[lo - 1]);
  if (job->rowmap[lo][local] >= 0) return;   // a selected row: the update kernel decays it and adds its update
  const float factor = job->decay_device != nullptr ? __ldg(job->decay_device) : job->decay_host;
  float* __restrict__ w = job->w[lo] + local * job->cols;
  if (job->vec) {
    float4* w4 = reinterpret_cast<float4*>(w);
    const int n4 = job->cols >> 2;
#pragma unroll 4
    for (int i = lane; i < n4; i += 32) {
      float4 v = __ldcs(w4 + i);
      v.x = __fmul_rn(v.x, factor); v.y = __fmul_rn(v.y, factor);
      v.z = __fmul_rn(v.z, factor); v.w = __fmul_rn(v.w, factor);
      __stcs(w4 + i, v);
    }
  } else {
    for (int e = lane; e < job->cols; e += 32) w[e] = __fmul_rn(w[e], factor);
  }
}

}  // namespace dionw
