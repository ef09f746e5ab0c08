// Error text, version, the device status word, and the host worker of the CPU EMA.
#include <atomic>
#include <condition_variable>
#include <cstdarg>
#include <cstring>
#include <mutex>
#include <new>
#include <thread>
#include <vector>

#include "common.cuh"

namespace dionw {
namespace {
thread_local char g_error[512] = "";
std::atomic<long long> g_launches{0};
__device__ int g_device_status = 0;
}  // namespace

void set_error(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void reset_tile_counters();   // gemm.cu

int* device_status_word() {
  static thread_local int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_device_status) == cudaSuccess) cached[dev] = static_cast<int*>(ptr);
  }
  return cached[dev];
}

}  // namespace dionw

extern "C" void dionw_last_error(char* buffer, size_t size) {
  if (buffer == nullptr || size == 0) return;
  strncpy(buffer, dionw::g_error, size - 1);
  buffer[size - 1] = '\0';
}

extern "C" const char* dionw_version(void) { return "dionw_b200 0.1.0 (sm_100a)"; }

extern "C" int64_t dionw_launch_count(void) { return dionw::g_launches.load(std::memory_order_relaxed); }

extern "C" int dionw_device_status(int* status) {
  using namespace dionw;
  DIONW_REQUIRE(status != nullptr, "device_status: null output");
  DIONW_CUDA(cudaDeviceSynchronize());
  int value = 0;
  DIONW_CUDA(cudaMemcpyFromSymbol(&value, g_device_status, sizeof(int)));
  if (value != 0) {
    const int zero = 0;
    DIONW_CUDA(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
  }
  *status = value;
  return DIONW_OK;
}

extern "C" int dionw_check_device(void) {
  int value = 0;
  const int st = dionw_device_status(&value);
  if (st != DIONW_OK) return st;
  if (value != 0) {
    dionw::reset_tile_counters();
    dionw::set_error(
        "a bounded wait inside a kernel ran out (device status 0x%x): the results of the work queued since the "
        "last check are not to be trusted",
        value);
    return DIONW_ERR_DEVICE_WAIT;
  }
  return DIONW_OK;
}

// ---------------------------------------------------------------------------
// CPU EMA worker
// ---------------------------------------------------------------------------
struct dionw_cpu_ema_job {
  std::vector<float*> shadows;
  std::vector<const float*> staged;
  std::vector<int64_t> numels;
  std::vector<uint8_t> first;
  float weight = 0.0f;
  cudaEvent_t event = nullptr;
  int threads = 1;
  std::mutex mutex;
  std::condition_variable cv;
  bool copy_ready = false;
  bool update_done = false;
  int failure = 0;
  char failure_text[256] = "";
  std::thread worker;
};

namespace {

// The two forms of the difference-form lerp (src/dionw/ema/_update.py:17-70 there; torch's
// lerp picks them by |weight| < 0.5).  The small-weight form is one fused multiply-add per
// element; without an FMA instruction in the compile target that is a libm call per element
// (2.3 ns each, measured: 160 ms for 567 M elements on 8 threads), so on x86-64 the same loops
// are also compiled for AVX2 + FMA and chosen at run time.  Both builds give the same bits:
// the fused multiply-add is exactly rounded either way, and the large-weight form is compiled
// with floating-point contraction off.
inline void lerp_small_body(float* __restrict__ shadow, const float* __restrict__ staged, int64_t n, float weight) {
  for (int64_t i = 0; i < n; ++i) shadow[i] = __builtin_fmaf(weight, staged[i] - shadow[i], shadow[i]);
}

inline void lerp_large_body(float* __restrict__ shadow, const float* __restrict__ staged, int64_t n, float keep) {
  for (int64_t i = 0; i < n; ++i) shadow[i] = staged[i] - (staged[i] - shadow[i]) * keep;
}

#if defined(__x86_64__) && defined(__GNUC__)
__attribute__((target("avx2,fma"))) void lerp_small_fma(float* __restrict__ shadow, const float* __restrict__ staged,
                                                        int64_t n, float weight) {
  for (int64_t i = 0; i < n; ++i) shadow[i] = __builtin_fmaf(weight, staged[i] - shadow[i], shadow[i]);
}

__attribute__((target("avx2,fma"))) void lerp_large_fma(float* __restrict__ shadow, const float* __restrict__ staged,
                                                        int64_t n, float keep) {
  for (int64_t i = 0; i < n; ++i) shadow[i] = staged[i] - (staged[i] - shadow[i]) * keep;
}

bool host_has_fma() {
  static const bool has = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
  return has;
}
#else
bool host_has_fma() { return false; }
void lerp_small_fma(float*, const float*, int64_t, float) {}
void lerp_large_fma(float*, const float*, int64_t, float) {}
#endif

void lerp_range(float* shadow, const float* staged, int64_t begin, int64_t end, float weight, bool first) {
  if (first) {
    std::memcpy(shadow + begin, staged + begin, size_t(end - begin) * sizeof(float));
    return;
  }
  const int64_t n = end - begin;
  const bool fast = host_has_fma();
  if (weight < 0.5f) {
    if (fast) lerp_small_fma(shadow + begin, staged + begin, n, weight);
    else lerp_small_body(shadow + begin, staged + begin, n, weight);
  } else {
    const float keep = 1.0f - weight;
    if (fast) lerp_large_fma(shadow + begin, staged + begin, n, keep);
    else lerp_large_body(shadow + begin, staged + begin, n, keep);
  }
}

void run_job(dionw_cpu_ema_job* job) {
  int failure = 0;
  if (job->event != nullptr) {
    const cudaError_t err = cudaEventSynchronize(job->event);
    if (err != cudaSuccess) {
      failure = DIONW_ERR_CUDA;
      snprintf(job->failure_text, sizeof(job->failure_text), "CPU EMA worker: waiting for the staged copy failed: %s",
               cudaGetErrorString(err));
    }
  }
  {
    std::lock_guard<std::mutex> lock(job->mutex);
    job->copy_ready = true;
    job->failure = failure;
  }
  job->cv.notify_all();
  if (failure == 0) {
    // A segment without a buffer is refused here, on the worker, so that the failure travels
    // the same way a failed wait does: stored, both waits released, re-raised by the waiter.
    for (size_t i = 0; i < job->numels.size(); ++i) {
      if (job->numels[i] < 0 || (job->numels[i] > 0 && (job->shadows[i] == nullptr || job->staged[i] == nullptr))) {
        failure = DIONW_ERR_WORKER;
        snprintf(job->failure_text, sizeof(job->failure_text),
                 "CPU EMA worker: segment %zu of %zu has no shadow or no staged buffer", i, job->numels.size());
        break;
      }
    }
  }
  if (failure == 0) {
    // Split the flat element space of all segments evenly over the helper threads.
    int64_t total = 0;
    for (int64_t n : job->numels) total += n;
    const int workers = job->threads < 1 ? 1 : job->threads;
    auto body = [job, total, workers](int w) {
      const int64_t lo = total * w / workers, hi = total * (w + 1) / workers;
      int64_t offset = 0;
      for (size_t i = 0; i < job->numels.size(); ++i) {
        const int64_t n = job->numels[i];
        const int64_t begin = lo > offset ? lo - offset : 0;
        const int64_t end = hi - offset < n ? hi - offset : n;
        if (begin < end) lerp_range(job->shadows[i], job->staged[i], begin, end, job->weight, job->first[i] != 0);
        offset += n;
        if (offset >= hi) break;
      }
    };
    // The pool lives outside the try block: if a helper thread cannot be started, the ones
    // already running are joined below instead of being destroyed while joinable (which would
    // terminate the process), and the update is reported as failed.
    std::vector<std::thread> pool;
    int started = 1;
    try {
      pool.reserve(size_t(workers));
      for (; started < workers; ++started) pool.emplace_back(body, started);
    } catch (const std::exception& e) {
      failure = DIONW_ERR_WORKER;
      snprintf(job->failure_text, sizeof(job->failure_text), "CPU EMA worker could not start a helper thread: %s",
               e.what());
    }
    body(0);
    for (auto& t : pool) t.join();
  }
  {
    std::lock_guard<std::mutex> lock(job->mutex);
    job->update_done = true;
    if (failure != 0) job->failure = failure;
  }
  job->cv.notify_all();
}

int job_result(dionw_cpu_ema_job* job) {
  if (job->failure != 0) {
    dionw::set_error("%s", job->failure_text);
    return job->failure;
  }
  return DIONW_OK;
}

}  // namespace

extern "C" dionw_cpu_ema_job* dionw_cpu_ema_job_start(float* const* shadows, const float* const* staged,
                                                      const int64_t* numels, const uint8_t* first, int n,
                                                      float weight, void* cuda_event, int threads) {
  if (n <= 0 || shadows == nullptr || staged == nullptr || numels == nullptr || first == nullptr) {
    dionw::set_error("cpu_ema_job_start: needs at least one segment");
    return nullptr;
  }
  dionw_cpu_ema_job* job = new (std::nothrow) dionw_cpu_ema_job();
  if (job == nullptr) {
    dionw::set_error("cpu_ema_job_start: out of host memory");
    return nullptr;
  }
  job->shadows.assign(shadows, shadows + n);
  job->staged.assign(staged, staged + n);
  job->numels.assign(numels, numels + n);
  job->first.assign(first, first + n);
  job->weight = weight;
  job->event = static_cast<cudaEvent_t>(cuda_event);
  job->threads = threads;
  try {
    job->worker = std::thread(run_job, job);
  } catch (const std::exception& e) {   // thread creation failed: no exception crosses the C boundary
    dionw::set_error("cpu_ema_job_start: the worker thread could not be started: %s", e.what());
    delete job;
    return nullptr;
  }
  return job;
}

extern "C" int dionw_cpu_ema_job_wait_copy(dionw_cpu_ema_job* job) {
  if (job == nullptr) return DIONW_ERR_ARGUMENT;
  std::unique_lock<std::mutex> lock(job->mutex);
  job->cv.wait(lock, [job] { return job->copy_ready; });
  return job_result(job);
}

extern "C" int dionw_cpu_ema_job_wait_update(dionw_cpu_ema_job* job) {
  if (job == nullptr) return DIONW_ERR_ARGUMENT;
  {
    std::unique_lock<std::mutex> lock(job->mutex);
    job->cv.wait(lock, [job] { return job->update_done; });
  }
  if (job->worker.joinable()) job->worker.join();
  return job_result(job);
}

extern "C" int dionw_cpu_ema_job_done(dionw_cpu_ema_job* job) {
  if (job == nullptr) return 1;
  std::lock_guard<std::mutex> lock(job->mutex);
  return job->update_done ? 1 : 0;
}

extern "C" void dionw_cpu_ema_job_destroy(dionw_cpu_ema_job* job) {
  if (job == nullptr) return;
  if (job->worker.joinable()) job->worker.join();
  delete job;
}
