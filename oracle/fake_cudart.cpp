// TEST INFRASTRUCTURE — stand-ins for the six CUDA runtime calls the reference library makes, so
// that the reference sees the SAME device properties on every machine (they are an input of the
// path: "blocks per SM", "warps per SM" and the occupancy block depend on them; reference:
// libkineto/src/DeviceProperties.cpp:48-75 createDeviceProps, :161-222).  The values come from the
// DEVPROPS section of the synthetic trace, set through k2j_fake_set_device_props().  This mirrors the
// reference's own test technique of replacing the hardware-facing layer
// (libkineto/test/CuptiActivityProfilerTest.cpp:320-346).  Also pins getpid() and the realtime
// clock so the pid column and ChromeTraceBaseTime (libkineto/src/output_json.h:265-279) are
// reproducible inputs instead of properties of the run.
#include <cuda_runtime_api.h>
#include <sys/syscall.h>
#include <time.h>
#include <unistd.h>
#include <cstring>
#include <vector>

static std::vector<cudaDeviceProp> g_props;
static int g_fake_pid = 0;
static long long g_fake_now_ns = 0;

extern "C" void k2j_fake_set_device_count(int n) { g_props.assign(n, cudaDeviceProp{}); }
extern "C" cudaDeviceProp* k2j_fake_device_prop(int i) { return &g_props[i]; }
extern "C" void k2j_fake_set_pid(int pid) { g_fake_pid = pid; }
extern "C" void k2j_fake_set_now_ns(long long ns) { g_fake_now_ns = ns; }

extern "C" pid_t getpid(void) {
  return g_fake_pid ? g_fake_pid : (pid_t)syscall(SYS_getpid);
}
extern "C" int clock_gettime(clockid_t clk, struct timespec* ts) {
  if (clk == CLOCK_REALTIME && g_fake_now_ns) {
    ts->tv_sec = g_fake_now_ns / 1000000000LL;
    ts->tv_nsec = g_fake_now_ns % 1000000000LL;
    return 0;
  }
  return (int)syscall(SYS_clock_gettime, clk, ts);
}

#ifndef K2J_REAL_CUDART  // the shim driver runs on a real GPU and keeps the real runtime
extern "C" cudaError_t cudaGetDeviceCount(int* count) {
  *count = (int)g_props.size();
  return cudaSuccess;
}
extern "C" cudaError_t cudaGetDeviceProperties_v2(cudaDeviceProp* prop, int device) {
  if (device < 0 || device >= (int)g_props.size()) return cudaErrorInvalidDevice;
  *prop = g_props[device];
  return cudaSuccess;
}
extern "C" cudaError_t cudaRuntimeGetVersion(int* v) { *v = CUDART_VERSION; return cudaSuccess; }
extern "C" cudaError_t cudaDriverGetVersion(int* v) { *v = CUDART_VERSION; return cudaSuccess; }
extern "C" cudaError_t cudaDeviceSynchronize(void) { return cudaSuccess; }
extern "C" const char* cudaGetErrorString(cudaError_t) { return "fake cudart"; }
#endif
