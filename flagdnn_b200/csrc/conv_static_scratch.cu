// fdnn_conv2d_fwd_static_scratch: the forward call for callers that may not
// allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc once they are running: an
// inference server that sized its arena at start-up and hands out nothing
// afterwards, a plug-in that lives inside another framework's memory budget,
// or a process that shares the GPU under a fixed per-process quota.  For them
// the scratch the repacking kernels need (the NHWC / TF32-split copy of x that
// fdnn_conv2d_fwd expects in `workspace`) lives in a fixed array inside the
// library image.  Every GPU that loads the library carries that array until
// the process exits, which is why it is kept modest.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/flagdnn_b200.h"

namespace {

// File-scope scratch.  In host code this name is only a handle for the runtime;
// the device address is obtained with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[FDNN_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_lookup_mutex;
void* g_scratch_ptr[kMaxDevices];  // set once the lookup on that device has succeeded

thread_local char g_msg[512];

int pass_through(int status) {
  // keep the promise of fdnn_static_scratch_last_error for failures of the calls this one is built on
  if (status != FDNN_OK) snprintf(g_msg, sizeof g_msg, "%s", fdnn_last_error());
  return status;
}

}  // namespace

extern "C" {

int64_t fdnn_static_scratch_bytes(void) { return FDNN_STATIC_SCRATCH_BYTES; }

const char* fdnn_static_scratch_last_error(void) { return g_msg; }

int fdnn_conv2d_fwd_static_scratch(const fdnn_conv_desc* desc, const void* x, const void* w,
                                   const void* w_packed, const void* bias, const void* scale,
                                   int activation, void* y, void* stream) {
  g_msg[0] = 0;
  fdnn_conv_plan plan;
  // Plan exactly as fdnn_conv2d_fwd will (a packed filter, when given, is used).
  int st = fdnn_conv2d_query(desc, x, w_packed != nullptr ? reinterpret_cast<const void*>(1) : w, y, &plan);
  if (st != FDNN_OK) return pass_through(st);
  if (plan.workspace_bytes > FDNN_STATIC_SCRATCH_BYTES) {
    snprintf(g_msg, sizeof g_msg,
             "this problem needs %lld bytes of scratch; the built-in scratch holds %lld "
             "(use fdnn_conv2d_fwd with a caller-provided workspace)",
             (long long)plan.workspace_bytes, (long long)FDNN_STATIC_SCRATCH_BYTES);
    return FDNN_WORKSPACE_TOO_SMALL;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    snprintf(g_msg, sizeof g_msg, "cannot identify the current device");
    return FDNN_CUDA_ERROR;
  }
  // Set-up, once per device, with that device current: translate the symbol
  // into the address the kernels can use.  Only a successful lookup is kept: a
  // first call that fails (made during a stream capture, say) is retried by the
  // next call instead of failing that device for good.
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_lookup_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess || p == nullptr) {
        cudaGetLastError();
        snprintf(g_msg, sizeof g_msg, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        return FDNN_CUDA_ERROR;
      }
      g_scratch_ptr[dev] = p;
    }
    scratch = g_scratch_ptr[dev];
  }
  // The relayout kernels overwrite every byte of the region they use (channel
  // padding included), so nothing in the array has to be cleared between calls.
  return pass_through(fdnn_conv2d_fwd(desc, x, w, w_packed, bias, scale, activation, y, scratch,
                                      FDNN_STATIC_SCRATCH_BYTES, stream));
}

}  // extern "C"
