// Host side of the tcgen05 GEMMs: tensor maps, launches, and the Newton-Schulz
// product schedules built from them.
#include <atomic>
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

#include "gemm2_sm100.cuh"

namespace dionw {
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so that the library itself
// links against the CUDA runtime only and still loads on a machine without a GPU.
EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
        res == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(ptr);
    }
  });
  return fn;
}

// 3-D map over a batch of row-major 2-byte matrices: (inner, rows, batch).
int make_map(CUtensorMap* map, const void* base, int dtype, int64_t inner, int64_t rows, int64_t batches,
             int64_t ld, int64_t batch_stride, uint32_t box_inner, uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return DIONW_ERR_CUDA;
  }
  DIONW_REQUIRE(aligned16(base), "matrix base address must be 16-byte aligned");
  DIONW_REQUIRE(ld % 8 == 0 && batch_stride % 8 == 0,
                "leading dimension (%lld) and batch stride (%lld) must be multiples of 8 elements",
                (long long)ld, (long long)batch_stride);
  cuuint64_t dims[3] = {cuuint64_t(inner), cuuint64_t(rows), cuuint64_t(batches)};
  cuuint64_t strides[2] = {cuuint64_t(ld) * 2, cuuint64_t(batch_stride) * 2};
  if (batches == 1) strides[1] = cuuint64_t(ld) * 2 * cuuint64_t(rows);
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t elem[3] = {1, 1, 1};
  const CUtensorMapDataType type = dtype == DIONW_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult res = fn(map, type, 3, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (inner=%lld rows=%lld batches=%lld ld=%lld)", int(res),
              (long long)inner, (long long)rows, (long long)batches, (long long)ld);
    return DIONW_ERR_CUDA;
  }
  return DIONW_OK;
}

constexpr int kMaxDevices = 64;

// Ordinal of the current device, clamped into the per-device tables.
int current_device() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) device = 0;
  return device;
}

// Products are launched with programmatic stream serialization (the kernels wait with
// griddepcontrol.wait before they touch global memory), unless DIONW_GEMM_PDL=0.  Measured on the
// Llama-3-8B-shaped step: 95.1-96.2 ms with it, 98.3-99.0 ms without (about 290 product launches per step).
bool use_dependent_launch() {
  static const bool on = [] {
    const char* v = std::getenv("DIONW_GEMM_PDL");
    return v == nullptr || v[0] != '0';
  }();
  return on;
}

template <typename InT, typename OutT, bool kBMajorMN, bool kSym>
int launch(const CUtensorMap& map_a, const CUtensorMap& map_b, const gemm::Params& p, cudaStream_t stream) {
  auto kernel = gemm::gemm_kernel<InT, OutT, kBMajorMN, kSym>;
  static std::atomic<bool> configured[kMaxDevices];   // the attribute is per device
  const int device = current_device();
  if (!configured[device].load(std::memory_order_acquire)) {
    DIONW_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm::kSmemBytes)));
    configured[device].store(true, std::memory_order_release);
  }
  const int total = p.tiles_per_batch * p.batches;
  if (total == 0) return DIONW_OK;
  const int grid = total < sm_count() ? total : sm_count();
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(unsigned(grid));
  config.blockDim = dim3(gemm::kThreads);
  config.dynamicSmemBytes = gemm::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = use_dependent_launch() ? 1 : 0;
  count_launch();
  return check_cuda(cudaLaunchKernelEx(&config, kernel, map_a, map_b, p), "gemm_kernel launch");
}

// ---- tile counters of the two-CTA kernel's dynamic hand-out ------------------------------------
// One {next tile, pairs done} pair per (device, stream) that has launched a product with the dynamic
// hand-out: launches of one stream run one after the other and each leaves its counters at zero,
// launches of different streams may overlap and must not share.  The counters live in the library's
// device image (zero at load); their address on a device is looked up once.
constexpr int kCounterSlots = 1024;
__device__ int g_tile_counters[kCounterSlots][2];

std::mutex g_counter_mutex;
std::map<std::pair<int, cudaStream_t>, int> g_counter_slot;   // guarded by g_counter_mutex
int g_counter_next[kMaxDevices];                              // guarded by g_counter_mutex
int* g_counter_base[kMaxDevices];                             // guarded by g_counter_mutex

// Process-wide switch (dionw_gemm_dynamic_tiles): off by default.  A product launched with it on
// draws its tiles from a counter; see gemm2_sm100.cuh.
std::atomic<int> g_dynamic_tiles{-1};

bool use_dynamic_tiles() {
  int mode = g_dynamic_tiles.load(std::memory_order_relaxed);
  if (mode < 0) {
    const char* v = std::getenv("DIONW_GEMM_DYNAMIC_TILES");
    mode = (v != nullptr && v[0] == '1') ? 1 : 0;
    g_dynamic_tiles.store(mode, std::memory_order_relaxed);
  }
  return mode != 0;
}

// The counters of `stream` on the current device, or null when they cannot be had (the product then
// takes its tiles in the fixed stride).
int* tile_counters(cudaStream_t stream) {
  const int device = current_device();
  std::lock_guard<std::mutex> lock(g_counter_mutex);
  if (g_counter_base[device] == nullptr) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_tile_counters) != cudaSuccess) return nullptr;
    g_counter_base[device] = static_cast<int*>(address);
  }
  const auto key = std::make_pair(device, stream);
  auto found = g_counter_slot.find(key);
  if (found == g_counter_slot.end()) {
    if (g_counter_next[device] >= kCounterSlots) return nullptr;
    found = g_counter_slot.emplace(key, g_counter_next[device]++).first;
  }
  return g_counter_base[device] + 2 * found->second;
}

// The streaming job (decay_job.cuh) that products launched by this thread carry, or null.
thread_local DecayJob* t_side_job = nullptr;

// Two-CTA tiles (clusters of two CTAs) unless the environment says DIONW_GEMM_CTA_PAIRS=0,
// which selects the one-CTA kernel.
bool use_cta_pairs() {
  static const bool on = [] {
    const char* v = std::getenv("DIONW_GEMM_CTA_PAIRS");
    return v == nullptr || v[0] != '0';
  }();
  return on;
}

template <typename InT, typename OutT, bool kBMajorMN, bool kSym>
int launch2(const CUtensorMap& map_a, const CUtensorMap& map_b, gemm::Params p, cudaStream_t stream) {
  auto kernel = gemm2::gemm2_kernel<InT, OutT, kBMajorMN, kSym>;
  static std::atomic<bool> configured[kMaxDevices];   // the attribute is per device
  const int device = current_device();
  if (!configured[device].load(std::memory_order_acquire)) {
    DIONW_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm2::kSmemBytes)));
    configured[device].store(true, std::memory_order_release);
  }
  // Pair tiles are 256 x 256.
  p.tiles_m = (p.m + gemm2::kPairM - 1) / gemm2::kPairM;
  p.tiles_n = (p.n + gemm2::kBN - 1) / gemm2::kBN;
  p.tiles_per_batch = kSym ? p.tiles_m * (p.tiles_m + 1) / 2 : p.tiles_m * p.tiles_n;
  const int total = p.tiles_per_batch * p.batches;
  if (total == 0) return DIONW_OK;
  const int pairs_max = sm_count() / 2;
  const int pairs = total < pairs_max ? total : pairs_max;
  // Tiles from a counter only where a pair takes more than one: a one-wave product gains nothing
  // from it and would pay the hand-out's latency on its critical path.
  p.tile_counter = (use_dynamic_tiles() && total > pairs) ? tile_counters(stream) : nullptr;
  // The streaming job rides on products whose main loop is long enough to hide a row behind it.
  p.job = (p.kdim >= 24 * gemm2::kBK) ? t_side_job : nullptr;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(unsigned(2 * pairs));
  config.blockDim = dim3(gemm2::kThreads);
  config.dynamicSmemBytes = gemm2::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = 2;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = use_dependent_launch() ? 2 : 1;
  count_launch();
  return check_cuda(cudaLaunchKernelEx(&config, kernel, map_a, map_b, p), "gemm2_kernel launch");
}

// The one-CTA kernel, or the two-CTA kernel when it is switched on.  The tensor map of B is
// built by the caller for the variant in use (their B boxes differ).
template <typename InT, typename OutT, bool kBMajorMN, bool kSym>
int launch_any(const CUtensorMap& map_a, const CUtensorMap& map_b, const gemm::Params& p, cudaStream_t stream) {
  if (use_cta_pairs()) return launch2<InT, OutT, kBMajorMN, kSym>(map_a, map_b, p, stream);
  return launch<InT, OutT, kBMajorMN, kSym>(map_a, map_b, p, stream);
}

int host_sym_tiles(int tiles_m) {
  const int q = tiles_m / 2;
  return q * (q + 1) + ((tiles_m & 1) ? q + 1 : 0);
}

}  // namespace

// C = alpha A B^T + beta Cin for a product known to be symmetric (B = A, or A and B symmetric
// matrices that commute): lower tiles + mirror, optional second output with diag added.
// b == nullptr means B = A.
int symmetric_product(const void* a, const void* b, int64_t blocks, int64_t m, int64_t kdim, int64_t lda,
                      int64_t a_batch, int64_t ldb, int64_t b_batch, const void* cin, int64_t ldc, int64_t cin_batch, float alpha, float beta, void* out,
                      int64_t ldo, int64_t out_batch, void* out2, float diag, int dtype, cudaStream_t stream) {
  DIONW_REQUIRE(dtype == DIONW_F16 || dtype == DIONW_BF16, "symmetric_product: dtype must be F16 or BF16");
  DIONW_REQUIRE(blocks > 0 && m > 0 && kdim > 0, "symmetric_product: empty problem");
  CUtensorMap map_a, map_b;
  int st = make_map(&map_a, a, dtype, kdim, m, blocks, lda, a_batch, gemm::kBK, gemm::kBM);
  if (st != DIONW_OK) return st;
  const bool same = b == nullptr || b == a;
  if (b == nullptr) {
    b = a;
    ldb = lda;
    b_batch = a_batch;
  }
  st = make_map(&map_b, b, dtype, kdim, m, blocks, ldb, b_batch, gemm::kBK,
                use_cta_pairs() ? gemm2::kHalfN : gemm::kBN);
  if (st != DIONW_OK) return st;
  gemm::Params p{};
  p.cin = cin;
  p.out = out;
  p.out2 = out2;
  p.ldc = ldc;
  p.ldo = ldo;
  p.cin_batch = cin_batch;
  p.out_batch = out_batch;
  p.alpha = alpha;
  p.beta = beta;
  p.diag = diag;
  p.m = int(m);
  p.n = int(m);
  p.kdim = int(kdim);
  p.batches = int(blocks);
  p.tiles_m = int((m + gemm::kBM - 1) / gemm::kBM);
  p.tiles_n = int((m + gemm::kBN - 1) / gemm::kBN);
  p.tiles_per_batch = host_sym_tiles(p.tiles_m);
  p.mirror_diagonal = same ? 0 : 1;
  p.status = device_status_word();
  p.wait_ns = gemm::kWaitLimitNs;
  if (dtype == DIONW_F16) return launch_any<__half, __half, false, true>(map_a, map_b, p, stream);
  return launch_any<__nv_bfloat16, __nv_bfloat16, false, true>(map_a, map_b, p, stream);
}

// C = A B + beta Cin.
int batched_gemm(const void* a, int64_t lda, int64_t a_batch, const void* b, int64_t ldb, int64_t b_batch,
                 bool b_is_nk, const void* cin, int64_t ldc, int64_t cin_batch, float beta, void* out, int64_t ldo,
                 int64_t out_batch, int64_t blocks, int64_t m, int64_t n, int64_t kdim, int in_dtype, int out_dtype,
                 float* rowsq, cudaStream_t stream) {
  DIONW_REQUIRE(in_dtype == DIONW_F16 || in_dtype == DIONW_BF16, "batched_gemm: input dtype must be F16 or BF16");
  DIONW_REQUIRE(out_dtype == DIONW_F16 || out_dtype == DIONW_BF16, "batched_gemm: output dtype must be F16 or BF16");
  DIONW_REQUIRE(blocks > 0 && m > 0 && n > 0 && kdim > 0, "batched_gemm: empty problem");
  CUtensorMap map_a, map_b;
  int st = make_map(&map_a, a, in_dtype, kdim, m, blocks, lda, a_batch, gemm::kBK, gemm::kBM);
  if (st != DIONW_OK) return st;
  if (b_is_nk) {
    st = make_map(&map_b, b, in_dtype, kdim, n, blocks, ldb, b_batch, gemm::kBK,
                  use_cta_pairs() ? gemm2::kHalfN : gemm::kBN);
  } else {
    st = make_map(&map_b, b, in_dtype, n, kdim, blocks, ldb, b_batch, 64, gemm::kBK);
  }
  if (st != DIONW_OK) return st;
  gemm::Params p{};
  p.cin = cin;
  p.out = out;
  p.out2 = nullptr;
  p.ldc = ldc;
  p.ldo = ldo;
  p.cin_batch = cin_batch;
  p.out_batch = out_batch;
  p.alpha = 1.0f;
  p.beta = beta;
  p.diag = 0.0f;
  p.m = int(m);
  p.n = int(n);
  p.kdim = int(kdim);
  p.batches = int(blocks);
  p.tiles_m = int((m + gemm::kBM - 1) / gemm::kBM);
  p.tiles_n = int((n + gemm::kBN - 1) / gemm::kBN);
  p.tiles_per_batch = p.tiles_m * p.tiles_n;
  p.rowsq = rowsq;
  p.rowsq_parts = 2 * p.tiles_n;   // both kernels' tiles are 256 columns wide
  p.status = device_status_word();
  p.wait_ns = gemm::kWaitLimitNs;
  const bool f16 = in_dtype == DIONW_F16;
  const bool out_same = out_dtype == in_dtype;
  if (b_is_nk) {
    if (f16 && out_same) return launch_any<__half, __half, false, false>(map_a, map_b, p, stream);
    if (f16) return launch_any<__half, __nv_bfloat16, false, false>(map_a, map_b, p, stream);
    if (out_same) return launch_any<__nv_bfloat16, __nv_bfloat16, false, false>(map_a, map_b, p, stream);
  } else {
    if (f16 && out_same) return launch_any<__half, __half, true, false>(map_a, map_b, p, stream);
    if (f16) return launch_any<__half, __nv_bfloat16, true, false>(map_a, map_b, p, stream);
    if (out_same) return launch_any<__nv_bfloat16, __nv_bfloat16, true, false>(map_a, map_b, p, stream);
  }
  set_error("batched_gemm: bf16 inputs with an fp16 output are not supported");
  return DIONW_ERR_UNSUPPORTED;
}

}  // namespace dionw

extern "C" int dionw_symmetric_product(const void* a, const void* b, int64_t blocks, int64_t m, int64_t kdim,
                                       int64_t lda, int64_t ldb, const void* cin, int64_t ldc, float alpha,
                                       float beta, void* out, int64_t ldo, void* out2, float diag, int dtype,
                                       void* stream) {
  return dionw::symmetric_product(a, b, blocks, m, kdim, lda, m * lda, ldb, m * ldb, cin, ldc, m * ldc, alpha, beta,
                                  out, ldo, m * ldo, out2, diag, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int dionw_batched_gemm(const void* a, int64_t lda, const void* b, int64_t ldb, int b_is_nk,
                                  const void* cin, int64_t ldc, float beta, void* out, int64_t ldo, int64_t blocks,
                                  int64_t m, int64_t n, int64_t kdim, int in_dtype, int out_dtype, void* stream) {
  const int64_t b_rows = b_is_nk ? n : kdim;
  return dionw::batched_gemm(a, lda, m * lda, b, ldb, b_rows * ldb, b_is_nk != 0, cin, ldc, m * ldc, beta, out, ldo,
                             m * ldo, blocks, m, n, kdim, in_dtype, out_dtype, nullptr,
                             static_cast<cudaStream_t>(stream));
}

namespace dionw {
// After a wait that ran out a product may have left its tile counters in any state: put them back to
// zero on the current device (called by dionw_check_device when it reports a failure).
void reset_tile_counters() {
  void* address = nullptr;
  if (cudaGetSymbolAddress(&address, g_tile_counters) == cudaSuccess)
    cudaMemset(address, 0, sizeof(int) * 2 * kCounterSlots);
}
}  // namespace dionw

extern "C" void dionw_gemm_side_job(void* job) { dionw::t_side_job = static_cast<dionw::DecayJob*>(job); }

extern "C" int dionw_gemm_dynamic_tiles(int on) {
  const int before = dionw::use_dynamic_tiles() ? 1 : 0;
  if (on >= 0) dionw::g_dynamic_tiles.store(on != 0 ? 1 : 0, std::memory_order_relaxed);
  return before;
}

// ---------------------------------------------------------------------------
// Self-test of the bounded wait.  One CTA of one warp initialises an mbarrier on
// which nothing ever arrives (no TMA, no TMEM, no other CTA) and waits on it with
// the products' own mbar_wait and a limit of `limit_ns`.  The wait runs out, the
// kernel stores the wait code in the device status word and returns normally: the
// context stays usable and the host reads the code with dionw_check_device().
// ---------------------------------------------------------------------------
namespace dionw {
namespace {

__global__ void __launch_bounds__(32)
wait_selftest_kernel(int* status, uint64_t limit_ns, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    gemm::mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const bool ok = gemm::mbar_wait(&bar, 0u, &abort_flag, status, limit_ns);
    if (gave_up != nullptr) *gave_up = ok ? 0 : 1;
  }
}

}  // namespace
}  // namespace dionw

extern "C" int dionw_selftest_wait_timeout(int64_t limit_us, int* gave_up, void* stream) {
  using namespace dionw;
  DIONW_REQUIRE(limit_us > 0 && limit_us <= 100000, "selftest_wait_timeout: the limit must be 1 .. 100000 us (got %lld)",
                (long long)limit_us);
  wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(device_status_word(),
                                                                        uint64_t(limit_us) * 1000ull, gave_up);
  return launch_status("wait_selftest_kernel");
}
