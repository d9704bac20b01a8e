// k2j_exclusive_scan_u32_noalloc: the device-wide exclusive scan for callers that must not allocate.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a profiler's buffer-completed
// or teardown callback while the CUDA context is being torn down or the allocator lock is held, in a
// process whose memory pool is fully owned by a framework's caching allocator, or between the capture
// boundaries of code that forbids allocation.  The regular entry point (k2j_exclusive_scan_u32) takes
// its block-sum scratch from the context's grow-only workspace, which may call cudaMalloc.  This
// variant keeps the scratch in a fixed array that is part of the library image instead: every GPU that
// loads libk2j.so holds kNoAllocScratchBytes (about 64 KiB) of device memory for it until the process
// exits, and no call here allocates or frees anything, on the host side of CUDA or through any library.
//
// Limits and rules for callers:
//   * at most K2J_NOALLOC_SCAN_MAX elements per call; larger inputs are rejected, not truncated;
//   * the first call on a device resolves the scratch address (cudaGetSymbolAddress with that device
//     current) and should therefore happen before any stream capture begins on that device;
//   * all calls on a device share the one scratch array: two calls whose kernels may overlap on the GPU
//     (different streams without ordering) race on it and give wrong offsets.  Order them.
//   * nothing in the scratch has to start at zero: each call overwrites every block sum it later reads,
//     so leftovers of the previous call are harmless;
//   * under CUDA's default lazy module loading the driver sets up this file's kernels and the scratch array when
//     they are first used, and that set-up allocates: make one call with n >= 1 on each device (or run with
//     CUDA_MODULE_LOADING=EAGER) before entering a region that must not allocate;
//   * the scratch address is looked up once per device and kept: do not use the entry point across a
//     cudaDeviceReset of that device;
//   * the caller's current device is the same after the call as before it.
#include "../../include/k2j.h"

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace {

constexpr int kThreads = 256;
constexpr int kItems = 8;
constexpr int kTile = kThreads * kItems;                                    // 2048 elements per block
constexpr unsigned long long kMaxElems = K2J_NOALLOC_SCAN_MAX;              // 16 Mi elements
constexpr unsigned int kMaxBlocks = (unsigned int)((kMaxElems + kTile - 1) / kTile);  // 8192 block sums
constexpr size_t kNoAllocScratchBytes = (size_t)(kMaxBlocks + 32) * sizeof(unsigned long long);

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress; it is not a
// device address and must never be passed to a kernel directly.
static __device__ __align__(256) unsigned long long g_noalloc_scratch[kMaxBlocks + 32];
static_assert(sizeof(g_noalloc_scratch) == kNoAllocScratchBytes && kNoAllocScratchBytes <= 80 * 1024, "the scratch is meant to stay modest");

constexpr int kMaxDevices = 64;
unsigned long long* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

__device__ __forceinline__ unsigned long long block_scan(unsigned long long v, unsigned long long* total) {
  __shared__ unsigned long long s_warp[kThreads / 32];
  const unsigned lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  unsigned long long x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= (unsigned)o) x += y;
  }
  __syncthreads();
  if (lane == 31) s_warp[w] = x;
  __syncthreads();
  unsigned long long base = 0, tot = 0;
#pragma unroll
  for (int i = 0; i < kThreads / 32; i++) { if ((unsigned)i < w) base += s_warp[i]; tot += s_warp[i]; }
  *total = tot;
  return base + x - v;
}

__global__ void __launch_bounds__(kThreads) k_na_reduce(const uint32_t* in, unsigned long long n, unsigned long long* sums) {
  const unsigned long long base = (unsigned long long)blockIdx.x * kTile;
  unsigned long long s = 0;
#pragma unroll
  for (int k = 0; k < kItems; k++) {
    const unsigned long long i = base + (unsigned long long)k * kThreads + threadIdx.x;
    if (i < n) s += in[i];
  }
  unsigned long long tot;
  block_scan(s, &tot);
  if (threadIdx.x == 0) sums[blockIdx.x] = tot;
}
__global__ void __launch_bounds__(kThreads) k_na_sums(unsigned long long* sums, unsigned int nb, unsigned long long* total) {
  unsigned long long carry = 0;
  for (unsigned int b0 = 0; b0 < nb; b0 += kThreads) {
    const unsigned int i = b0 + threadIdx.x;
    const unsigned long long v = i < nb ? sums[i] : 0;
    unsigned long long tot;
    const unsigned long long ex = block_scan(v, &tot);
    if (i < nb) sums[i] = carry + ex;
    carry += tot;
    __syncthreads();
  }
  if (threadIdx.x == 0) *total = carry;
}
__global__ void __launch_bounds__(kThreads) k_na_apply(const uint32_t* in, unsigned long long n, const unsigned long long* sums,
                                                       unsigned long long* out) {
  const unsigned long long base = (unsigned long long)blockIdx.x * kTile + (unsigned long long)threadIdx.x * kItems;
  uint32_t v[kItems];
  unsigned long long s = 0;
#pragma unroll
  for (int k = 0; k < kItems; k++) { const unsigned long long i = base + k; v[k] = i < n ? in[i] : 0; s += v[k]; }
  unsigned long long tot;
  unsigned long long ex = block_scan(s, &tot) + sums[blockIdx.x];
#pragma unroll
  for (int k = 0; k < kItems; k++) { const unsigned long long i = base + k; if (i < n) out[i] = ex; ex += v[k]; }
}

}  // namespace

extern "C" k2j_status k2j_exclusive_scan_u32_noalloc(int device, void* stream, const uint32_t* sizes, uint64_t n,
                                                     uint64_t* offsets, uint64_t* total) {
  if (device < 0 || device >= kMaxDevices) return K2J_ERR_INVALID_ARGUMENT;
  if (!total || (n && (!sizes || !offsets))) return K2J_ERR_INVALID_ARGUMENT;
  if (n > kMaxElems) return K2J_ERR_INVALID_ARGUMENT;  // beyond the fixed scratch: refuse, never truncate
  int previous = -1;
  if (cudaGetDevice(&previous) != cudaSuccess) { cudaGetLastError(); previous = -1; }
  if (cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return K2J_ERR_CUDA; }
  struct Restore {  // the caller's current device is put back on every way out
    int dev;
    ~Restore() { if (dev >= 0) cudaSetDevice(dev); }
  } restore{previous != device ? previous : -1};
  unsigned long long* scratch;
  {
    std::lock_guard<std::mutex> guard(g_setup_mutex);
    if (!g_scratch_ptr[device]) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) { cudaGetLastError(); return K2J_ERR_CUDA; }
      g_scratch_ptr[device] = static_cast<unsigned long long*>(p);
    }
    scratch = g_scratch_ptr[device];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned int nb = n ? (unsigned int)((n + kTile - 1) / kTile) : 1u;
  unsigned long long* d_total = reinterpret_cast<unsigned long long*>(total);
  k_na_reduce<<<nb, kThreads, 0, s>>>(sizes, n, scratch);
  k_na_sums<<<1, kThreads, 0, s>>>(scratch, nb, d_total);
  if (n) k_na_apply<<<nb, kThreads, 0, s>>>(sizes, n, scratch, reinterpret_cast<unsigned long long*>(offsets));
  if (cudaGetLastError() != cudaSuccess) return K2J_ERR_CUDA;
  return K2J_OK;
}
