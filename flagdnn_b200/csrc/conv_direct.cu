// Direct convolution on CUDA cores: one thread per output element, any dtype
// (f16 / bf16 / f32 accumulate in fp32, f64 in fp64), any groups, dilation and
// element strides.  It serves the parts of conv2d's surface the tensor-core
// kernel does not take: grouped and depthwise convolutions, fp64, geometry
// outside the TMA im2col limits, and problems too small to fill the machine
// (the reference covers these with its depthwise and fp64 kernels,
// src/flag_dnn/ops/conv2d.py:2613-2800, 3276-3460).  Index arithmetic follows
// src/flag_dnn/graph/kernels/fused_conv.py:249-299.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "conv_internal.h"

namespace fdnn {
namespace {

template <typename T> struct Acc { using type = float; };
template <> struct Acc<double> { using type = double; };

template <typename T, typename A> __device__ __forceinline__ A ld(const T* p) { return static_cast<A>(*p); }
template <> __device__ __forceinline__ float ld<__half, float>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ld<__nv_bfloat16, float>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T, typename A> __device__ __forceinline__ T cvt(A v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ __half cvt<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256)
conv_direct_kernel(const DirectParams p, const bool k_fastest) {
  using A = typename Acc<T>::type;
  const long long total = (long long)p.N * p.K * p.OH * p.OW;
  const T* x = static_cast<const T*>(p.x);
  const T* w = static_cast<const T*>(p.w);
  const T* bias = static_cast<const T*>(p.bias);
  const T* scale = static_cast<const T*>(p.scale);
  T* y = static_cast<T*>(p.y);
  const int cg = p.C / p.groups;
  const int kg = p.K / p.groups;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    int n, k, oh, ow;
    long long t = idx;
    if (k_fastest) {  // channels-last output: neighbouring threads write neighbouring channels
      k = int(t % p.K); t /= p.K;
      ow = int(t % p.OW); t /= p.OW;
      oh = int(t % p.OH); t /= p.OH;
      n = int(t);
    } else {
      ow = int(t % p.OW); t /= p.OW;
      oh = int(t % p.OH); t /= p.OH;
      k = int(t % p.K); t /= p.K;
      n = int(t);
    }
    const int g = k / kg;
    A acc = A(0);
    const T* xg = x + n * p.x_s[0] + (long long)(g * cg) * p.x_s[1];
    const T* wk = w + k * p.w_s[0];
    for (int r = 0; r < p.R; ++r) {
      const int ih = oh * p.stride_h + r * p.dil_h - p.pad_top;
      if (ih < 0 || ih >= p.H) continue;
      for (int s = 0; s < p.S; ++s) {
        const int iw = ow * p.stride_w + s * p.dil_w - p.pad_left;
        if (iw < 0 || iw >= p.W) continue;
        const T* xp = xg + ih * p.x_s[2] + iw * p.x_s[3];
        const T* wp = wk + r * p.w_s[2] + s * p.w_s[3];
        for (int c = 0; c < cg; ++c) {
          acc += ld<T, A>(xp + c * p.x_s[1]) * ld<T, A>(wp + c * p.w_s[1]);
        }
      }
    }
    if (scale != nullptr) acc *= ld<T, A>(scale + k);
    if (bias != nullptr) acc += ld<T, A>(bias + k);
    const long long y_idx = n * p.y_s[0] + k * p.y_s[1] + oh * p.y_s[2] + ow * p.y_s[3];
    if (p.residual != nullptr) acc += ld<T, A>(static_cast<const T*>(p.residual) + y_idx);
    if (p.act == FDNN_ACT_RELU) {
      acc = (acc < A(0)) ? A(0) : acc;  // keeps NaN, like torch.relu
    } else if (p.act == FDNN_ACT_GELU) {
      acc = A(0.5) * acc * (A(1) + erf(acc * A(0.70710678118654752440)));
    } else if (p.act == FDNN_ACT_GELU_TANH) {
      const A u = A(0.79788456080286535588) * (acc + A(0.044715) * acc * acc * acc);
      acc = A(0.5) * acc * (A(1) + tanh(u));
    }
    y[y_idx] = cvt<T, A>(acc);
  }
}

template <typename T>
cudaError_t go(const DirectParams& p, cudaStream_t stream) {
  const long long total = (long long)p.N * p.K * p.OH * p.OW;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 64) blocks = 148LL * 64;
  if (blocks < 1) blocks = 1;
  const bool k_fastest = p.y_s[1] == 1 && p.K > 1;
  conv_direct_kernel<T><<<int(blocks), 256, 0, stream>>>(p, k_fastest);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_direct(int dtype, const DirectParams& p, cudaStream_t stream) {
  switch (dtype) {
    case FDNN_F16: return go<__half>(p, stream);
    case FDNN_BF16: return go<__nv_bfloat16>(p, stream);
    case FDNN_F32: return go<float>(p, stream);
    case FDNN_F64: return go<double>(p, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace fdnn
