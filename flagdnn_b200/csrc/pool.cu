// Pooling next to the convolution path: max_pool2d (the layer after a ResNet
// stem) and adaptive_avg_pool2d (the one before its classifier).  Both are
// HBM-bound maps with a small window, so the kernels are about access order,
// not arithmetic: a thread's linear index walks y in y's own memory order
// (channel fastest for channels-last, width fastest for NCHW), and dense
// channels-last 16-bit tensors move 8 channels (16 bytes) per thread.
//
// Semantics follow torch.nn.functional.max_pool2d / adaptive_avg_pool2d, which
// the reference's operators are tested against
// (src/flag_dnn/ops/max_pool2d.py:174-243, tests/test_max_pool2d.py:49-58;
// src/flag_dnn/ops/adaptive_avg_pool2d.py:456-480): -inf padding, NaN wins a
// maximum, indices are ih * W + iw of the first maximum in scan order; an
// adaptive window is [floor(o * L / O), ceil((o + 1) * L / O)), summed in fp32
// (fp64 for doubles) and divided by its size.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "conv_convert.cuh"
#include "conv_internal.h"

namespace fdnn {
namespace {

template <typename T>
struct Acc {
  using type = float;
};
template <>
struct Acc<double> {
  using type = double;
};

template <typename T>
__device__ __forceinline__ typename Acc<T>::type up(T v) {
  if constexpr (sizeof(T) == 2) return to_f32<T>(v);
  else return v;
}
template <typename T>
__device__ __forceinline__ T down(typename Acc<T>::type v) {
  if constexpr (sizeof(T) == 2) return from_f32<T>(v);
  else return static_cast<T>(v);
}

// linear index -> (n, c, oh, ow) in y's memory order.  I is unsigned 32-bit whenever the output has fewer
// than 2^31 elements: four 64-bit divisions per element are what such a kernel would otherwise spend
// its time on.
template <typename I>
__device__ __forceinline__ void unravel(I i, const PoolParams& p, bool c_fastest, int& n, int& c, int& oh,
                                        int& ow) {
  if (c_fastest) {
    c = int(i % I(p.C)); i /= I(p.C);
    ow = int(i % I(p.OW)); i /= I(p.OW);
    oh = int(i % I(p.OH)); n = int(i / I(p.OH));
  } else {
    ow = int(i % I(p.OW)); i /= I(p.OW);
    oh = int(i % I(p.OH)); i /= I(p.OH);
    c = int(i % I(p.C)); n = int(i / I(p.C));
  }
}

template <typename T, typename I>
__global__ void max_pool2d_kernel(const PoolParams p) {
  using A = typename Acc<T>::type;
  const T* x = static_cast<const T*>(p.x);
  T* y = static_cast<T*>(p.y);
  const bool c_fastest = p.y_s[1] == 1 && p.C > 1;
  const long long total = (long long)p.N * p.C * p.OH * p.OW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int n, c, oh, ow;
    unravel<I>(I(i), p, c_fastest, n, c, oh, ow);
    const T* xc = x + n * p.x_s[0] + c * p.x_s[1];
    A best = -INFINITY;
    long long best_at = -1;
    for (int r = 0; r < p.kh; ++r) {
      const int ih = oh * p.sh - p.ph + r * p.dh;
      if (ih < 0 || ih >= p.H) continue;
      for (int s = 0; s < p.kw; ++s) {
        const int iw = ow * p.sw - p.pw + s * p.dw;
        if (iw < 0 || iw >= p.W) continue;
        const A v = up<T>(xc[ih * p.x_s[2] + iw * p.x_s[3]]);
        const long long pos = (long long)ih * p.W + iw;
        if (best_at < 0) best_at = pos;  // the window's first element, as torch starts
        if (v > best || v != v) {
          best = v;
          best_at = pos;
        }
      }
    }
    const long long at = n * p.y_s[0] + c * p.y_s[1] + oh * p.y_s[2] + ow * p.y_s[3];
    y[at] = down<T>(best);
    if (p.idx != nullptr) p.idx[at] = best_at;
  }
}

// Dense channels-last 16-bit tensors, C % 8 == 0, no indices: 8 channels per thread.
template <typename T, typename I>
__global__ void max_pool2d_nhwc8_kernel(const PoolParams p) {
  const int c8 = p.C / 8;
  const long long total = (long long)p.N * p.OH * p.OW * c8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    I t = I(i);
    const int cv = int(t % I(c8)); t /= I(c8);
    const int ow = int(t % I(p.OW)); t /= I(p.OW);
    const int oh = int(t % I(p.OH));
    const int n = int(t / I(p.OH));
    const T* xc = static_cast<const T*>(p.x) + n * p.x_s[0] + cv * 8;
    float best[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) best[j] = -INFINITY;
    for (int r = 0; r < p.kh; ++r) {
      const int ih = oh * p.sh - p.ph + r * p.dh;
      if (ih < 0 || ih >= p.H) continue;
      for (int s = 0; s < p.kw; ++s) {
        const int iw = ow * p.sw - p.pw + s * p.dw;
        if (iw < 0 || iw >= p.W) continue;
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(xc + ih * p.x_s[2] + iw * p.x_s[3]));
        const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float v = to_f32<T>(e[j]);
          if (v > best[j] || v != v) best[j] = v;
        }
      }
    }
    uint4 out;
    out.x = pack2(from_f32<T>(best[0]), from_f32<T>(best[1]));
    out.y = pack2(from_f32<T>(best[2]), from_f32<T>(best[3]));
    out.z = pack2(from_f32<T>(best[4]), from_f32<T>(best[5]));
    out.w = pack2(from_f32<T>(best[6]), from_f32<T>(best[7]));
    T* yc = static_cast<T*>(p.y) + n * p.y_s[0] + oh * p.y_s[2] + ow * p.y_s[3] + cv * 8;
    *reinterpret_cast<uint4*>(yc) = out;
  }
}

__device__ __forceinline__ int win_start(int o, int in, int out) { return int(((long long)o * in) / out); }
__device__ __forceinline__ int win_end(int o, int in, int out) { return int(((long long)(o + 1) * in + out - 1) / out); }

template <typename T, typename I>
__global__ void adaptive_avg_pool2d_kernel(const PoolParams p) {
  using A = typename Acc<T>::type;
  const T* x = static_cast<const T*>(p.x);
  T* y = static_cast<T*>(p.y);
  const bool c_fastest = p.y_s[1] == 1 && p.C > 1;
  const long long total = (long long)p.N * p.C * p.OH * p.OW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int n, c, oh, ow;
    unravel<I>(I(i), p, c_fastest, n, c, oh, ow);
    const int h0 = win_start(oh, p.H, p.OH), h1 = win_end(oh, p.H, p.OH);
    const int w0 = win_start(ow, p.W, p.OW), w1 = win_end(ow, p.W, p.OW);
    const T* xc = x + n * p.x_s[0] + c * p.x_s[1];
    A sum = 0;
    for (int ih = h0; ih < h1; ++ih)
      for (int iw = w0; iw < w1; ++iw) sum += up<T>(xc[ih * p.x_s[2] + iw * p.x_s[3]]);
    y[n * p.y_s[0] + c * p.y_s[1] + oh * p.y_s[2] + ow * p.y_s[3]] = down<T>(sum / A((h1 - h0) * (w1 - w0)));
  }
}

template <typename T, typename I>
__global__ void adaptive_avg_pool2d_nhwc8_kernel(const PoolParams p) {
  const int c8 = p.C / 8;
  const long long total = (long long)p.N * p.OH * p.OW * c8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    I t = I(i);
    const int cv = int(t % I(c8)); t /= I(c8);
    const int ow = int(t % I(p.OW)); t /= I(p.OW);
    const int oh = int(t % I(p.OH));
    const int n = int(t / I(p.OH));
    const int h0 = win_start(oh, p.H, p.OH), h1 = win_end(oh, p.H, p.OH);
    const int w0 = win_start(ow, p.W, p.OW), w1 = win_end(ow, p.W, p.OW);
    const T* xc = static_cast<const T*>(p.x) + n * p.x_s[0] + cv * 8;
    float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int ih = h0; ih < h1; ++ih)
      for (int iw = w0; iw < w1; ++iw) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(xc + ih * p.x_s[2] + iw * p.x_s[3]));
        const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[j] += to_f32<T>(e[j]);
      }
    const float inv = float((h1 - h0) * (w1 - w0));
    uint4 out;
    out.x = pack2(from_f32<T>(sum[0] / inv), from_f32<T>(sum[1] / inv));
    out.y = pack2(from_f32<T>(sum[2] / inv), from_f32<T>(sum[3] / inv));
    out.z = pack2(from_f32<T>(sum[4] / inv), from_f32<T>(sum[5] / inv));
    out.w = pack2(from_f32<T>(sum[6] / inv), from_f32<T>(sum[7] / inv));
    T* yc = static_cast<T*>(p.y) + n * p.y_s[0] + oh * p.y_s[2] + ow * p.y_s[3] + cv * 8;
    *reinterpret_cast<uint4*>(yc) = out;
  }
}

bool nhwc8_ok(const PoolParams& p, int es) {
  auto a16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  if (es != 2 || p.C % 8 != 0 || p.idx != nullptr) return false;
  if (p.x_s[1] != 1 || p.y_s[1] != 1 || !a16(p.x) || !a16(p.y)) return false;
  for (int i : {0, 2, 3})
    if (p.x_s[i] % 8 != 0 || p.y_s[i] % 8 != 0) return false;
  return true;
}

int grid_for(long long work) {
  long long blocks = (work + 255) / 256;
  if (blocks > 148LL * 256) blocks = 148LL * 256;
  return int(blocks < 1 ? 1 : blocks);
}

}  // namespace

#define FDNN_POOL_GO(KERNEL, T)                                            \
  do {                                                                    \
    if (small) KERNEL<T, uint32_t><<<g, 256, 0, stream>>>(p);             \
    else KERNEL<T, unsigned long long><<<g, 256, 0, stream>>>(p);         \
  } while (0)

cudaError_t launch_max_pool2d(int dtype, const PoolParams& p, cudaStream_t stream) {
  const long long total = (long long)p.N * p.C * p.OH * p.OW;
  if (total == 0) return cudaSuccess;
  const bool small = total < (1ll << 31);
  const int es = dtype == FDNN_F64 ? 8 : (dtype == FDNN_F32 ? 4 : 2);
  if (nhwc8_ok(p, es)) {
    const int g = grid_for(total / 8);
    if (dtype == FDNN_F16) FDNN_POOL_GO(max_pool2d_nhwc8_kernel, __half);
    else FDNN_POOL_GO(max_pool2d_nhwc8_kernel, __nv_bfloat16);
    return cudaGetLastError();
  }
  const int g = grid_for(total);
  switch (dtype) {
    case FDNN_F16: FDNN_POOL_GO(max_pool2d_kernel, __half); break;
    case FDNN_BF16: FDNN_POOL_GO(max_pool2d_kernel, __nv_bfloat16); break;
    case FDNN_F32: FDNN_POOL_GO(max_pool2d_kernel, float); break;
    case FDNN_F64: FDNN_POOL_GO(max_pool2d_kernel, double); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_adaptive_avg_pool2d(int dtype, const PoolParams& p, cudaStream_t stream) {
  const long long total = (long long)p.N * p.C * p.OH * p.OW;
  if (total == 0) return cudaSuccess;
  const bool small = total < (1ll << 31);
  const int es = dtype == FDNN_F64 ? 8 : (dtype == FDNN_F32 ? 4 : 2);
  if (nhwc8_ok(p, es)) {
    const int g = grid_for(total / 8);
    if (dtype == FDNN_F16) FDNN_POOL_GO(adaptive_avg_pool2d_nhwc8_kernel, __half);
    else FDNN_POOL_GO(adaptive_avg_pool2d_nhwc8_kernel, __nv_bfloat16);
    return cudaGetLastError();
  }
  const int g = grid_for(total);
  switch (dtype) {
    case FDNN_F16: FDNN_POOL_GO(adaptive_avg_pool2d_kernel, __half); break;
    case FDNN_BF16: FDNN_POOL_GO(adaptive_avg_pool2d_kernel, __nv_bfloat16); break;
    case FDNN_F32: FDNN_POOL_GO(adaptive_avg_pool2d_kernel, float); break;
    case FDNN_F64: FDNN_POOL_GO(adaptive_avg_pool2d_kernel, double); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}
#undef FDNN_POOL_GO

}  // namespace fdnn
