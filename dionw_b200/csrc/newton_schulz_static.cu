// dionw_newton_schulz_static: the Newton-Schulz iteration for callers that
// cannot hand over scratch memory.
//
// Who that is.  dionw_newton_schulz wants a workspace from its caller, and the
// callers this library was written for get one from torch's caching allocator.
// Some callers have no allocator to ask: a C or C++ host that binds this ABI
// without torch; a serving or real-time loop whose memory budget was fixed at
// start-up and whose rules forbid cudaMalloc afterwards; a process in which a
// framework's pool already owns nearly all device memory, so a raw cudaMalloc
// of a few hundred megabytes would simply fail; a hot loop that must not stall,
// where cudaMalloc and cudaFree are out because both synchronise the device.
// For them the scratch lives below, inside the library image, and this entry
// point allocates nothing at all.
//
// The price is a fixed ceiling: kStaticScratchBytes per GPU, part of the library's
// device image.  The CUDA runtime loads that image on a GPU when the library is first
// used there (with lazy module loading, the default, as late as the first call of this
// entry point), and it then stays until the process exits.  So the first call on a
// device can fail with DIONW_ERR_CUDA in a process whose pools already hold nearly all
// of that GPU's memory: make it during set-up, before the pools are filled.  Problems
// that need more scratch than the ceiling are refused.
#include <atomic>

#include "common.cuh"

namespace dionw {
namespace {

// 64 MiB: enough for, e.g., 2 blocks of 1024 x 4096, 8 blocks of 512 x 2048 or
// 1 block of 1536 x 4096 (dionw_newton_schulz_workspace_bytes gives the need).
constexpr size_t kStaticScratchBytes = DIONW_STATIC_SCRATCH_BYTES;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch per device ordinal.  The symbol's name is
// only a host-side handle: the address a kernel can use has to be asked for,
// with the device in question current.
std::atomic<void*> g_scratch_address[64];   // zero-initialised; threads may race to fill a slot with the same value

int scratch_for_current_device(void** out) {
  int device = 0;
  DIONW_CUDA(cudaGetDevice(&device));
  DIONW_REQUIRE(device >= 0 && device < 64, "newton_schulz_static: device ordinal %d is out of range", device);
  void* address = g_scratch_address[device].load(std::memory_order_acquire);
  if (address == nullptr) {
    DIONW_CUDA(cudaGetSymbolAddress(&address, g_static_scratch));
    g_scratch_address[device].store(address, std::memory_order_release);
  }
  *out = address;
  return DIONW_OK;
}

}  // namespace
}  // namespace dionw

extern "C" int dionw_newton_schulz_static(void* x, void* out, int64_t blocks, int64_t m, int64_t n, int64_t ldx,
                                          int kind, void* stream) {
  using namespace dionw;
  const size_t need = dionw_newton_schulz_workspace_bytes(blocks, m, n, kind);
  if (need == 0) {
    set_error("newton_schulz_static: needs blocks > 0, m > 0, n > 0");
    return DIONW_ERR_ARGUMENT;
  }
  // The ceiling is stated for operands stored with the smallest legal leading dimension, which is
  // what dionw_newton_schulz_workspace_bytes assumes: a wider ldx would make the iteration's second
  // operand, which has the same layout, larger than that figure.
  if (ldx != (n + 7) / 8 * 8) {
    set_error(
        "newton_schulz_static: ldx must be n rounded up to a multiple of 8 (%lld for n = %lld), got %lld: the built-in "
        "scratch is sized for that layout; use dionw_newton_schulz with a workspace of your own for padded operands",
        (long long)((n + 7) / 8 * 8), (long long)n, (long long)ldx);
    return DIONW_ERR_ARGUMENT;
  }
  if (need > kStaticScratchBytes) {
    set_error(
        "newton_schulz_static: %lld blocks of %lld x %lld need %zu bytes of scratch, the built-in scratch holds %zu; "
        "use dionw_newton_schulz with a workspace of your own, or fewer blocks per call",
        (long long)blocks, (long long)m, (long long)n, need, kStaticScratchBytes);
    return DIONW_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  const int status = scratch_for_current_device(&scratch);
  if (status != DIONW_OK) return status;
  // Nothing in the scratch has to start at zero: every product of the schedule
  // writes the whole of its output before a later product reads it, so what the
  // previous call left behind is never looked at.
  return dionw_newton_schulz(x, out, blocks, m, n, ldx, kind, scratch, kStaticScratchBytes, nullptr, stream);
}
