// Depthwise convolution (groups == C == K, one filter per channel) on CUDA cores.
//
// A depthwise layer does 2*R*S flops per output element against two bytes read and two written: it is
// bound by memory traffic, not arithmetic, so the job is to touch x and y once each with wide, coalesced
// accesses and to keep the R*S taps out of global memory.  Two kernels, chosen by layout (the reference
// has one Triton kernel per layout as well: src/flag_dnn/ops/conv2d.py:2613-2800 for NCHW,
// src/flag_dnn/ops/conv2d.py:3089-3190 for channels-last):
//
//   channels-last  one thread owns 16 bytes of channels (8 x 16-bit or 4 x fp32) of four (two in the run-time
//                  variant) neighbouring output pixels of a row; every input pixel it needs is one 16-byte
//                  load that serves all of them; the filter sits in shared memory as fp32 [R*S][C];
//   NCHW           one block owns one (image, channel) plane: its taps sit in registers (shared memory in the
//                  run-time variant), its threads walk the plane's output pixels four (two) at a time along
//                  W, and the plane's input stays in L1.
// 3x3 and 5x5 filters at stride 1 and 2 without dilation have fully unrolled instantiations of both.
//
// Arithmetic as everywhere in this library: fp32 accumulate (fp64 is left to the direct kernel), scale,
// bias and residual in fp32, activation, one rounding.  Index arithmetic follows
// src/flag_dnn/graph/kernels/fused_conv.py:249-299.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "conv_convert.cuh"
#include "conv_epilogue.cuh"
#include "conv_internal.h"

namespace fdnn {
namespace {

constexpr int kDwThreads = 256;
constexpr int kDwMaxSmemFloats = 12288;  // 48 KB of taps at most

template <typename T>
__device__ __forceinline__ void unpack_vec(const uint4& q, float (&v)[16 / sizeof(T)]) {
  if constexpr (std::is_same<T, float>::value) {
    v[0] = __uint_as_float(q.x); v[1] = __uint_as_float(q.y); v[2] = __uint_as_float(q.z); v[3] = __uint_as_float(q.w);
  } else {
    unpack2<T>(q.x, v[0], v[1]);
    unpack2<T>(q.y, v[2], v[3]);
    unpack2<T>(q.z, v[4], v[5]);
    unpack2<T>(q.w, v[6], v[7]);
  }
}

template <typename T>
__device__ __forceinline__ uint4 pack_vec(const float (&v)[16 / sizeof(T)]) {
  uint4 q;
  if constexpr (std::is_same<T, float>::value) {
    q.x = __float_as_uint(v[0]); q.y = __float_as_uint(v[1]); q.z = __float_as_uint(v[2]); q.w = __float_as_uint(v[3]);
  } else {
    q.x = round_pack2<T>(v[0], v[1]);
    q.y = round_pack2<T>(v[2], v[3]);
    q.z = round_pack2<T>(v[4], v[5]);
    q.w = round_pack2<T>(v[6], v[7]);
  }
  return q;
}

// ------------------------------------------------------------------ channels-last
// KR, KS, KSTRIDE: filter size and (equal) strides known at compile time, dilation 1 — every loop unrolls and
// the tap a column serves for each output is resolved by the compiler; 0, 0, 0 takes everything from `p`.
template <typename T, int KR, int KS, int KSTRIDE>
__global__ void __launch_bounds__(kDwThreads)
depthwise_cl_kernel(const DirectParams p) {
  constexpr int V = 16 / int(sizeof(T));  // channels per thread
  constexpr int PW = KR != 0 ? 4 : 2;     // output pixels per thread, along W
  constexpr bool kStatic = KR != 0;
  extern __shared__ float s_w[];          // [R*S][C]
  const T* w = static_cast<const T*>(p.w);
  const int R = kStatic ? KR : p.R, S = kStatic ? KS : p.S;
  const int stride_h = kStatic ? KSTRIDE : p.stride_h, stride_w = kStatic ? KSTRIDE : p.stride_w;
  const int dil_h = kStatic ? 1 : p.dil_h, dil_w = kStatic ? 1 : p.dil_w;
  const int taps = R * S;
  for (int i = threadIdx.x; i < taps * p.C; i += blockDim.x) {
    const int tap = i / p.C, c = i - tap * p.C;
    const int r = tap / S, s = tap - r * S;
    s_w[i] = to_f32<T>(w[c * p.w_s[0] + r * p.w_s[2] + s * p.w_s[3]]);
  }
  __syncthreads();
  const T* x = static_cast<const T*>(p.x);
  const T* bias = static_cast<const T*>(p.bias);
  const T* scale = static_cast<const T*>(p.scale);
  const T* res = static_cast<const T*>(p.residual);
  T* y = static_cast<T*>(p.y);
  const int cv = p.C / V;
  const int owg = (p.OW + PW - 1) / PW;
  const long long items = (long long)p.N * p.OH * owg * cv;
  constexpr int kSpanStatic = (PW - 1) * KSTRIDE + KS;           // input columns the PW outputs touch
  const int span = kStatic ? kSpanStatic : (PW - 1) * stride_w + (S - 1) * dil_w + 1;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < items;
       idx += (long long)gridDim.x * blockDim.x) {
    long long t = idx;
    const int c0 = int(t % cv) * V; t /= cv;
    const int ow0 = int(t % owg) * PW; t /= owg;
    const int oh = int(t % p.OH); t /= p.OH;
    const int n = int(t);
    float acc[PW][V];
#pragma unroll
    for (int q = 0; q < PW; ++q)
#pragma unroll
      for (int v = 0; v < V; ++v) acc[q][v] = 0.0f;
    const int iw0 = ow0 * stride_w - p.pad_left;
    const T* img = x + n * p.x_s[0] + c0;
    if constexpr (kStatic) {
#pragma unroll
      for (int r = 0; r < KR; ++r) {
        const int ih = oh * KSTRIDE + r - p.pad_top;
        if (ih < 0 || ih >= p.H) continue;
        const T* row = img + ih * p.x_s[2];
#pragma unroll
        for (int j = 0; j < kSpanStatic; ++j) {
          const int iw = iw0 + j;
          float xv[V];
          uint4 raw = make_uint4(0u, 0u, 0u, 0u);
          if (iw >= 0 && iw < p.W) raw = __ldg(reinterpret_cast<const uint4*>(row + iw * p.x_s[3]));
          unpack_vec<T>(raw, xv);
#pragma unroll
          for (int q = 0; q < PW; ++q) {
            const int s = j - q * KSTRIDE;   // a constant once the loops are unrolled
            if (s >= 0 && s < KS) {
              const float* wt = s_w + (r * KS + s) * p.C + c0;
#pragma unroll
              for (int v = 0; v < V; ++v) acc[q][v] = fmaf(xv[v], wt[v], acc[q][v]);
            }
          }
        }
      }
    } else {
      for (int r = 0; r < R; ++r) {
        const int ih = oh * stride_h + r * dil_h - p.pad_top;
        if (ih < 0 || ih >= p.H) continue;
        const T* row = img + ih * p.x_s[2];
        for (int j = 0; j < span; ++j) {
          const int iw = iw0 + j;
          if (iw < 0 || iw >= p.W) continue;
          float xv[V];
          unpack_vec<T>(__ldg(reinterpret_cast<const uint4*>(row + iw * p.x_s[3])), xv);
#pragma unroll
          for (int q = 0; q < PW; ++q) {
            const int d = j - q * stride_w;          // = s * dil_w for the tap this column is for output q
            if (d < 0 || d % dil_w != 0) continue;
            const int s = d / dil_w;
            if (s >= S) continue;
            const float* wt = s_w + (r * S + s) * p.C + c0;
#pragma unroll
            for (int v = 0; v < V; ++v) acc[q][v] = fmaf(xv[v], wt[v], acc[q][v]);
          }
        }
      }
    }
#pragma unroll
    for (int q = 0; q < PW; ++q) {
      const int ow = ow0 + q;
      if (ow >= p.OW) continue;
      const long long y_idx = n * p.y_s[0] + oh * p.y_s[2] + ow * p.y_s[3] + c0;
      float rv[V];
      if (res != nullptr) unpack_vec<T>(__ldg(reinterpret_cast<const uint4*>(res + y_idx)), rv);
#pragma unroll
      for (int v = 0; v < V; ++v) {
        float a = acc[q][v];
        if (scale != nullptr) a *= to_f32<T>(scale[c0 + v]);
        if (bias != nullptr) a += to_f32<T>(bias[c0 + v]);
        if (res != nullptr) a += rv[v];
        acc[q][v] = apply_activation(a, p.act);
      }
      *reinterpret_cast<uint4*>(y + y_idx) = pack_vec<T>(acc[q]);
    }
  }
}

// --------------------------------------------------------------------------- NCHW
template <typename T, int KR, int KS, int KSTRIDE>
__global__ void __launch_bounds__(kDwThreads)
depthwise_plane_kernel(const DirectParams p) {
  constexpr bool kStatic = KR != 0;
  constexpr int PW = kStatic ? 4 : 2;
  extern __shared__ float s_w[];  // [R*S] taps of this block's channel
  const int plane = blockIdx.x;   // n * C + c
  const int n = plane / p.C, c = plane - n * p.C;
  const T* w = static_cast<const T*>(p.w) + c * p.w_s[0];
  const int R = kStatic ? KR : p.R, S = kStatic ? KS : p.S;
  const int stride_h = kStatic ? KSTRIDE : p.stride_h, stride_w = kStatic ? KSTRIDE : p.stride_w;
  const int dil_h = kStatic ? 1 : p.dil_h, dil_w = kStatic ? 1 : p.dil_w;
  const int taps = R * S;
  for (int i = threadIdx.x; i < taps; i += blockDim.x) {
    const int r = i / S, s = i - r * S;
    s_w[i] = to_f32<T>(w[r * p.w_s[2] + s * p.w_s[3]]);
  }
  __syncthreads();
  float wt[kStatic ? KR * KS : 1];
  if constexpr (kStatic) {
#pragma unroll
    for (int i = 0; i < KR * KS; ++i) wt[i] = s_w[i];   // the taps live in registers: every index below is static
  }
  const T* x = static_cast<const T*>(p.x) + n * p.x_s[0] + c * p.x_s[1];
  T* y = static_cast<T*>(p.y) + n * p.y_s[0] + c * p.y_s[1];
  const T* res = p.residual != nullptr ? static_cast<const T*>(p.residual) + n * p.y_s[0] + c * p.y_s[1] : nullptr;
  const float sc = p.scale != nullptr ? to_f32<T>(static_cast<const T*>(p.scale)[c]) : 1.0f;
  const float bi = p.bias != nullptr ? to_f32<T>(static_cast<const T*>(p.bias)[c]) : 0.0f;
  const int owg = (p.OW + PW - 1) / PW;
  const int items = p.OH * owg;
  constexpr int kSpanStatic = (PW - 1) * KSTRIDE + KS;
  const int span = kStatic ? kSpanStatic : (PW - 1) * stride_w + (S - 1) * dil_w + 1;
  for (int idx = threadIdx.x; idx < items; idx += blockDim.x) {
    const int oh = idx / owg;
    const int ow0 = (idx - oh * owg) * PW;
    float acc[PW];
#pragma unroll
    for (int q = 0; q < PW; ++q) acc[q] = 0.0f;
    const int iw0 = ow0 * stride_w - p.pad_left;
    if constexpr (kStatic) {
#pragma unroll
      for (int r = 0; r < KR; ++r) {
        const int ih = oh * KSTRIDE + r - p.pad_top;
        if (ih < 0 || ih >= p.H) continue;
        const T* row = x + ih * p.x_s[2];
#pragma unroll
        for (int j = 0; j < kSpanStatic; ++j) {
          const int iw = iw0 + j;
          const float xv = (iw >= 0 && iw < p.W) ? to_f32<T>(row[iw * p.x_s[3]]) : 0.0f;
#pragma unroll
          for (int q = 0; q < PW; ++q) {
            const int s = j - q * KSTRIDE;
            if (s >= 0 && s < KS) acc[q] = fmaf(xv, wt[r * KS + s], acc[q]);
          }
        }
      }
    } else {
      for (int r = 0; r < R; ++r) {
        const int ih = oh * stride_h + r * dil_h - p.pad_top;
        if (ih < 0 || ih >= p.H) continue;
        const T* row = x + ih * p.x_s[2];
        for (int j = 0; j < span; ++j) {
          const int iw = iw0 + j;
          if (iw < 0 || iw >= p.W) continue;
          const float xv = to_f32<T>(row[iw * p.x_s[3]]);
#pragma unroll
          for (int q = 0; q < PW; ++q) {
            const int d = j - q * stride_w;
            if (d < 0 || d % dil_w != 0) continue;
            const int s = d / dil_w;
            if (s < S) acc[q] = fmaf(xv, s_w[r * S + s], acc[q]);
          }
        }
      }
    }
#pragma unroll
    for (int q = 0; q < PW; ++q) {
      const int ow = ow0 + q;
      if (ow >= p.OW) continue;
      const long long y_idx = oh * p.y_s[2] + ow * p.y_s[3];
      float a = fmaf(acc[q], sc, bi);
      if (res != nullptr) a += to_f32<T>(res[y_idx]);
      y[y_idx] = from_f32<T>(apply_activation(a, p.act));
    }
  }
}

template <typename T, int KR, int KS, int KSTRIDE>
cudaError_t go_static(const DirectParams& p, bool channels_last, cudaStream_t stream) {
  if (channels_last) {
    constexpr int V = 16 / int(sizeof(T));
    constexpr int PW = KR != 0 ? 4 : 2;
    const long long items = (long long)p.N * p.OH * ((p.OW + PW - 1) / PW) * (p.C / V);
    long long blocks = (items + kDwThreads - 1) / kDwThreads;
    if (blocks > 148LL * 32) blocks = 148LL * 32;
    if (blocks < 1) blocks = 1;
    depthwise_cl_kernel<T, KR, KS, KSTRIDE>
        <<<int(blocks), kDwThreads, size_t(p.R) * p.S * p.C * sizeof(float), stream>>>(p);
  } else {
    depthwise_plane_kernel<T, KR, KS, KSTRIDE><<<p.N * p.C, kDwThreads, size_t(p.R) * p.S * sizeof(float), stream>>>(p);
  }
  return cudaGetLastError();
}

template <typename T>
cudaError_t go(const DirectParams& p, bool channels_last, cudaStream_t stream) {
  // the common filters get fully unrolled kernels; everything else (dilation, unequal strides, other sizes)
  // the run-time one
  if (p.dil_h == 1 && p.dil_w == 1 && p.stride_h == p.stride_w && p.R == p.S) {
    if (p.R == 3 && p.stride_w == 1) return go_static<T, 3, 3, 1>(p, channels_last, stream);
    if (p.R == 3 && p.stride_w == 2) return go_static<T, 3, 3, 2>(p, channels_last, stream);
    if (p.R == 5 && p.stride_w == 1) return go_static<T, 5, 5, 1>(p, channels_last, stream);
    if (p.R == 5 && p.stride_w == 2) return go_static<T, 5, 5, 2>(p, channels_last, stream);
  }
  return go_static<T, 0, 0, 0>(p, channels_last, stream);
}

}  // namespace

// 0: not a case for these kernels (the caller uses the direct kernel); 1: channels-last kernel; 2: plane kernel.
int depthwise_kind(int dtype, const DirectParams& p) {
  if (p.groups != p.C || p.K != p.C || p.C < 1) return 0;
  if (dtype != FDNN_F16 && dtype != FDNN_BF16 && dtype != FDNN_F32) return 0;
  if ((long long)p.N * p.C <= 0 || p.OH <= 0 || p.OW <= 0) return 0;
  const int es = dtype == FDNN_F32 ? 4 : 2;
  const int v = 16 / es;
  const bool aligned = ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.y) |
                         reinterpret_cast<uintptr_t>(p.residual)) & 15u) == 0;
  auto mult = [v](long long extent, long long stride) { return extent <= 1 || stride % v == 0; };
  const bool cl = p.C % v == 0 && (p.C == 1 || (p.x_s[1] == 1 && p.y_s[1] == 1)) && aligned &&
                  mult(p.N, p.x_s[0]) && mult(p.H, p.x_s[2]) && mult(p.W, p.x_s[3]) && mult(p.N, p.y_s[0]) &&
                  mult(p.OH, p.y_s[2]) && mult(p.OW, p.y_s[3]) && (long long)p.R * p.S * p.C <= kDwMaxSmemFloats &&
                  p.C > 1;
  if (cl) return 1;
  if ((long long)p.N * p.C < 2147483647LL && p.R * p.S <= kDwMaxSmemFloats) return 2;
  return 0;
}

cudaError_t launch_depthwise(int dtype, const DirectParams& p, int kind, cudaStream_t stream) {
  switch (dtype) {
    case FDNN_F16: return go<__half>(p, kind == 1, stream);
    case FDNN_BF16: return go<__nv_bfloat16>(p, kind == 1, stream);
    case FDNN_F32: return go<float>(p, kind == 1, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace fdnn
