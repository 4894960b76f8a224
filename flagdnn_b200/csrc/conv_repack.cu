// Relayout kernels feeding the implicit-GEMM path.
//
// The tensor-core kernel reads activations as NHWC with 16-byte aligned pixel
// rows and filters as [K, R, S, C] with the same channel padding.  Tensors that
// already look like that are consumed in place; everything else (NCHW inputs,
// channel counts that are not a multiple of 16 bytes, fp32 tensors that must be
// split into TF32 halves) passes through one of these kernels first.  The
// filter relayout is the counterpart of the reference's one-time weight packers
// (src/flag_dnn/ops/conv2d.py:193-276).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "conv_internal.h"

namespace fdnn {
namespace {

// fp32 -> (hi, lo) with hi = x rounded to TF32 and lo = (x - hi) rounded to
// TF32; hi + lo carries about 21 mantissa bits of x.
__device__ __forceinline__ void split_tf32(float v, float& hi, float& lo) {
  uint32_t h, l;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
  hi = __uint_as_float(h);
  const float rem = v - hi;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rem));
  lo = __uint_as_float(l);
}

template <typename T>
__device__ __forceinline__ void put(T* dst, long long plane, long long i, T v) {
  if constexpr (std::is_same<T, float>::value) {
    float hi, lo;
    split_tf32(v, hi, lo);
    dst[i] = hi;
    dst[plane + i] = lo;
  } else {
    dst[i] = v;
  }
}

// Generic gather: one thread per destination element, channel fastest.
template <typename T>
__global__ void __launch_bounds__(256)
repack_x_generic(const T* __restrict__ x, long long sn, long long sc, long long sh, long long sw,
                 int N, int C, int H, int W, int c_pad, T* __restrict__ dst, long long plane) {
  const long long total = (long long)N * H * W * c_pad;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i;
    const int c = int(t % c_pad); t /= c_pad;
    const int w = int(t % W); t /= W;
    const int h = int(t % H); t /= H;
    const int n = int(t);
    const T v = (c < C) ? x[n * sn + c * sc + h * sh + w * sw] : T(0.0f);
    put<T>(dst, plane, i, v);
  }
}

// W-contiguous sources (NCHW): 32 channels x 32 columns go through shared
// memory so both the reads (along W) and the writes (along C) are coalesced.
template <typename T>
__global__ void __launch_bounds__(256)
repack_x_wfast(const T* __restrict__ x, long long sn, long long sc, long long sh, int N, int C,
               int H, int W, int c_pad, T* __restrict__ dst, long long plane) {
  __shared__ T tile[32][33];
  const int w_tiles = (W + 31) / 32;
  const int c_tiles = (c_pad + 31) / 32;
  const long long total = (long long)N * H * w_tiles * c_tiles;
  const int tx = threadIdx.x & 31;
  const int ty = threadIdx.x >> 5;  // 0..7
  for (long long b = blockIdx.x; b < total; b += gridDim.x) {
    long long t = b;
    const int ct = int(t % c_tiles); t /= c_tiles;
    const int wt = int(t % w_tiles); t /= w_tiles;
    const int h = int(t % H); t /= H;
    const int n = int(t);
    const int w0 = wt * 32, c0 = ct * 32;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = c0 + ty + j * 8;
      const int w = w0 + tx;
      tile[ty + j * 8][tx] = (c < C && w < W) ? x[n * sn + c * sc + h * sh + w] : T(0.0f);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int w = w0 + ty + j * 8;
      const int c = c0 + tx;
      if (w < W && c < c_pad) {
        const long long o = (((long long)n * H + h) * W + w) * c_pad + c;
        put<T>(dst, plane, o, tile[tx][ty + j * 8]);
      }
    }
    __syncthreads();
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
pack_w_kernel(const T* __restrict__ w, long long sk, long long sc, long long sr, long long ss, int K,
              int C, int R, int S, int c_pad, T* __restrict__ dst, long long plane) {
  const long long total = (long long)K * R * S * c_pad;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i;
    const int c = int(t % c_pad); t /= c_pad;
    const int s = int(t % S); t /= S;
    const int r = int(t % R); t /= R;
    const int k = int(t);
    const T v = (c < C) ? w[k * sk + c * sc + r * sr + s * ss] : T(0.0f);
    put<T>(dst, plane, i, v);
  }
}

int grid_for(long long work_items, int per_block) {
  long long blocks = (work_items + per_block - 1) / per_block;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  if (blocks < 1) blocks = 1;
  return int(blocks);
}

template <typename T>
cudaError_t repack_x_t(const void* x, const long long s[4], int N, int C, int H, int W, int c_pad,
                       void* dst, long long plane, cudaStream_t stream) {
  if (s[3] == 1 && s[1] != 1) {
    const long long tiles = (long long)N * H * ((W + 31) / 32) * ((c_pad + 31) / 32);
    repack_x_wfast<T><<<grid_for(tiles, 1), 256, 0, stream>>>(
        static_cast<const T*>(x), s[0], s[1], s[2], N, C, H, W, c_pad, static_cast<T*>(dst), plane);
  } else {
    const long long total = (long long)N * H * W * c_pad;
    repack_x_generic<T><<<grid_for(total, 256), 256, 0, stream>>>(
        static_cast<const T*>(x), s[0], s[1], s[2], s[3], N, C, H, W, c_pad, static_cast<T*>(dst),
        plane);
  }
  return cudaGetLastError();
}

template <typename T>
cudaError_t pack_w_t(const void* w, const long long s[4], int K, int C, int R, int S, int c_pad,
                     void* dst, long long plane, cudaStream_t stream) {
  const long long total = (long long)K * R * S * c_pad;
  pack_w_kernel<T><<<grid_for(total, 256), 256, 0, stream>>>(
      static_cast<const T*>(w), s[0], s[1], s[2], s[3], K, C, R, S, c_pad, static_cast<T*>(dst), plane);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_repack_x(int dtype, const void* x, const long long x_s[4], int N, int C, int H,
                            int W, int c_pad, void* dst, long long plane_elems,
                            cudaStream_t stream) {
  switch (dtype) {
    case FDNN_F16: return repack_x_t<__half>(x, x_s, N, C, H, W, c_pad, dst, plane_elems, stream);
    case FDNN_BF16: return repack_x_t<__nv_bfloat16>(x, x_s, N, C, H, W, c_pad, dst, plane_elems, stream);
    case FDNN_F32: return repack_x_t<float>(x, x_s, N, C, H, W, c_pad, dst, plane_elems, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_pack_w(int dtype, const void* w, const long long w_s[4], int K, int C, int R,
                          int S, int c_pad, void* dst, long long plane_elems, cudaStream_t stream) {
  switch (dtype) {
    case FDNN_F16: return pack_w_t<__half>(w, w_s, K, C, R, S, c_pad, dst, plane_elems, stream);
    case FDNN_BF16: return pack_w_t<__nv_bfloat16>(w, w_s, K, C, R, S, c_pad, dst, plane_elems, stream);
    case FDNN_F32: return pack_w_t<float>(w, w_s, K, C, R, S, c_pad, dst, plane_elems, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace fdnn
