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
std::once_flag g_once[kMaxDevices];
void* g_scratch_ptr[kMaxDevices];
cudaError_t g_scratch_err[kMaxDevices];

thread_local char g_msg[256];

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
  if (st != FDNN_OK) return st;
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
  // into the address the kernels can use.
  std::call_once(g_once[dev], [dev]() {
    void* p = nullptr;
    g_scratch_err[dev] = cudaGetSymbolAddress(&p, g_static_scratch);
    g_scratch_ptr[dev] = (g_scratch_err[dev] == cudaSuccess) ? p : nullptr;
  });
  if (g_scratch_err[dev] != cudaSuccess || g_scratch_ptr[dev] == nullptr) {
    cudaGetLastError();
    snprintf(g_msg, sizeof g_msg, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(g_scratch_err[dev]));
    return FDNN_CUDA_ERROR;
  }
  // The relayout kernels overwrite every byte of the region they use (channel
  // padding included), so nothing in the array has to be cleared between calls.
  return fdnn_conv2d_fwd(desc, x, w, w_packed, bias, scale, activation, y, g_scratch_ptr[dev],
                         FDNN_STATIC_SCRATCH_BYTES, stream);
}

}  // extern "C"
