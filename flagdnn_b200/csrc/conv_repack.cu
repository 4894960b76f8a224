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

// Low-channel input relayout: one thread per stored pixel (4 channels = 8 bytes).
template <typename T>
__global__ void __launch_bounds__(256)
repack_x_lowc_kernel(const T* __restrict__ x, long long sn, long long sc, long long sh, long long sw,
                     int N, int C, int H, int W, int pad_left, int w_pad, T* __restrict__ dst) {
  const long long total = (long long)N * H * w_pad;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i;
    const int j = int(t % w_pad); t /= w_pad;
    const int h = int(t % H); t /= H;
    const int n = int(t);
    const int w = j - pad_left;
    T v[4] = {T(0.0f), T(0.0f), T(0.0f), T(0.0f)};
    if (w >= 0 && w < W) {
      const T* src = x + n * sn + h * sh + w * sw;
      for (int c = 0; c < C; ++c) v[c] = src[c * sc];
    }
    uint2 packed;
    packed.x = uint32_t(*reinterpret_cast<uint16_t*>(&v[0])) | (uint32_t(*reinterpret_cast<uint16_t*>(&v[1])) << 16);
    packed.y = uint32_t(*reinterpret_cast<uint16_t*>(&v[2])) | (uint32_t(*reinterpret_cast<uint16_t*>(&v[3])) << 16);
    reinterpret_cast<uint2*>(dst)[i] = packed;
  }
}

// Fast path of the low-channel relayout for a dense 3-channel NHWC source with
// 16-byte aligned rows and W % 8 == 0: one thread turns 8 pixels (48 bytes, three
// aligned 16-byte loads) into 8 four-channel pixels (64 bytes, four aligned stores).
__global__ void __launch_bounds__(256)
repack_x_lowc_c3_kernel(const uint16_t* __restrict__ x, long long sn, long long sh, int N, int H, int W,
                        int pad_left, int w_pad, uint16_t* __restrict__ dst) {
  const int w8s = W / 8;
  const long long total = (long long)N * H * w8s;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i;
    const int w8 = int(t % w8s); t /= w8s;
    const int h = int(t % H); t /= H;
    const int n = int(t);
    const uint4* src = reinterpret_cast<const uint4*>(x + n * sn + h * sh + w8 * 24);
    uint32_t in[12];
    const uint4 a = src[0], b = src[1], c = src[2];
    in[0] = a.x; in[1] = a.y; in[2] = a.z; in[3] = a.w;
    in[4] = b.x; in[5] = b.y; in[6] = b.z; in[7] = b.w;
    in[8] = c.x; in[9] = c.y; in[10] = c.z; in[11] = c.w;
    auto get16 = [&in](int e) -> uint32_t { return (in[e >> 1] >> (16 * (e & 1))) & 0xffffu; };
    uint16_t* row = dst + (((long long)n * H + h) * w_pad) * 4;
    uint4* out = reinterpret_cast<uint4*>(row + (long long)(pad_left + 8 * w8) * 4);
#pragma unroll
    for (int q = 0; q < 4; ++q) {  // two pixels per 16-byte store
      const int p0 = 2 * q, p1 = 2 * q + 1;
      uint4 v;
      v.x = get16(3 * p0) | (get16(3 * p0 + 1) << 16);
      v.y = get16(3 * p0 + 2);
      v.z = get16(3 * p1) | (get16(3 * p1 + 1) << 16);
      v.w = get16(3 * p1 + 2);
      out[q] = v;
    }
    if (w8 == 0) {
      for (int j = 0; j < pad_left; ++j) reinterpret_cast<uint2*>(row)[j] = make_uint2(0u, 0u);
    }
    if (w8 == w8s - 1) {
      for (int j = pad_left + W; j < w_pad; ++j) reinterpret_cast<uint2*>(row)[j] = make_uint2(0u, 0u);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
pack_w_lowc_kernel(const T* __restrict__ w, long long sk, long long sc, long long sr, long long ss, int K,
                   int C, int R, int S, int stride_w, int chans, int shift_elems, T* __restrict__ dst) {
  const long long total = 4LL * K * R * 64;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i;
    const int e = int(t % 64); t /= 64;
    const int r = int(t % R); t /= R;
    const int row = int(t);          // q * K + k
    const int q = row / K, k = row - q * K;
    // element = shift_elems + chans * (stride_w * q + tap) + channel
    const int rel = e - shift_elems - chans * stride_w * q;
    const int s = rel >= 0 ? rel / chans : -1;
    const int c = rel >= 0 ? rel - s * chans : 0;
    T v = T(0.0f);
    if (rel >= 0 && c < C && s < S) v = w[k * sk + c * sc + r * sr + s * ss];
    dst[i] = v;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
pack_w_grouped_kernel(const T* __restrict__ w, long long sk, long long sc, long long sr, long long ss, int K,
                      int C, int R, int S, int stride_w, int q, int c_pad, T* __restrict__ dst) {
  const int sv = S + (q - 1) * stride_w;
  const long long total = (long long)q * K * R * sv * c_pad;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i;
    const int c = int(t % c_pad); t /= c_pad;
    const int j = int(t % sv); t /= sv;
    const int r = int(t % R); t /= R;
    const int row = int(t);          // g * K + k
    const int g = row / K, k = row - g * K;
    const int s = j - g * stride_w;
    T v = T(0.0f);
    if (c < C && s >= 0 && s < S) v = w[k * sk + c * sc + r * sr + s * ss];
    dst[i] = v;
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

cudaError_t launch_repack_x_lowc(int dtype, const void* x, const long long x_s[4], int N, int C, int H,
                                 int W, int pad_left, int w_pad, void* dst, cudaStream_t stream) {
  const bool fast = (dtype == FDNN_F16 || dtype == FDNN_BF16) && C == 3 && x_s[1] == 1 && x_s[3] == 3 &&
                    W % 8 == 0 && pad_left % 2 == 0 && x_s[2] % 8 == 0 && (N <= 1 || x_s[0] % 8 == 0) &&
                    (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  if (fast) {
    const long long items = (long long)N * H * (W / 8);
    repack_x_lowc_c3_kernel<<<grid_for(items, 256), 256, 0, stream>>>(
        static_cast<const uint16_t*>(x), x_s[0], x_s[2], N, H, W, pad_left, w_pad, static_cast<uint16_t*>(dst));
    return cudaGetLastError();
  }
  const long long total = (long long)N * H * w_pad;
  const int grid = grid_for(total, 256);
  if (dtype == FDNN_F16) {
    repack_x_lowc_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(x), x_s[0], x_s[1], x_s[2],
                                                           x_s[3], N, C, H, W, pad_left, w_pad,
                                                           static_cast<__half*>(dst));
  } else if (dtype == FDNN_BF16) {
    repack_x_lowc_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), x_s[0], x_s[1], x_s[2], x_s[3], N, C, H, W, pad_left, w_pad,
        static_cast<__nv_bfloat16*>(dst));
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_pack_w_lowc(int dtype, const void* w, const long long w_s[4], int K, int C, int R,
                               int S, int stride_w, int chans, int shift_elems, void* dst, cudaStream_t stream) {
  const long long total = 4LL * K * R * 64;
  const int grid = grid_for(total, 256);
  if (dtype == FDNN_F16) {
    pack_w_lowc_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(w), w_s[0], w_s[1], w_s[2],
                                                         w_s[3], K, C, R, S, stride_w, chans, shift_elems, static_cast<__half*>(dst));
  } else if (dtype == FDNN_BF16) {
    pack_w_lowc_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(w), w_s[0], w_s[1], w_s[2], w_s[3], K, C, R, S, stride_w, chans, shift_elems,
        static_cast<__nv_bfloat16*>(dst));
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_pack_w_grouped(int dtype, const void* w, const long long w_s[4], int K, int C, int R,
                                  int S, int stride_w, int q, int c_pad, void* dst, cudaStream_t stream) {
  const long long total = (long long)q * K * R * (S + (q - 1) * stride_w) * c_pad;
  const int grid = grid_for(total, 256);
  if (dtype == FDNN_F16) {
    pack_w_grouped_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(w), w_s[0], w_s[1],
                                                            w_s[2], w_s[3], K, C, R, S, stride_w, q, c_pad,
                                                            static_cast<__half*>(dst));
  } else if (dtype == FDNN_BF16) {
    pack_w_grouped_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(w), w_s[0], w_s[1], w_s[2], w_s[3], K, C, R, S, stride_w, q, c_pad,
        static_cast<__nv_bfloat16*>(dst));
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

// A grouped filter [K][C/G][R][S] (any strides) written as the dense channels-last filter [K][R][S][C] of the
// same convolution: filter k keeps its group's C/G channels at their place among the C input channels and is zero
// everywhere else (a block-diagonal GEMM operand).
template <typename T>
__global__ void densify_w_kernel(const T* __restrict__ w, long long s0, long long s1, long long s2, long long s3, int K,
                                 int C, int R, int S, int groups, T* __restrict__ dense) {
  const long long total = (long long)K * R * S * C;
  const int cg = C / groups, kg = K / groups;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i;
    const int c = int(t % C); t /= C;
    const int s = int(t % S); t /= S;
    const int r = int(t % R); t /= R;
    const int k = int(t);
    const int local = c - (k / kg) * cg;
    T v = static_cast<T>(0.0f);
    if (local >= 0 && local < cg) v = w[k * s0 + local * s1 + r * s2 + s * s3];
    dense[i] = v;
  }
}

template <typename T>
cudaError_t densify_w_t(const void* w, const long long w_s[4], int K, int C, int R, int S, int groups, void* dense,
                        cudaStream_t stream) {
  const long long total = (long long)K * R * S * C;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  if (blocks < 1) blocks = 1;
  densify_w_kernel<T><<<int(blocks), 256, 0, stream>>>(static_cast<const T*>(w), w_s[0], w_s[1], w_s[2], w_s[3], K, C, R,
                                                       S, groups, static_cast<T*>(dense));
  return cudaGetLastError();
}

cudaError_t launch_densify_w(int dtype, const void* w, const long long w_s[4], int K, int C, int R, int S, int groups,
                             void* dense, cudaStream_t stream) {
  switch (dtype) {
    case FDNN_F16: return densify_w_t<__half>(w, w_s, K, C, R, S, groups, dense, stream);
    case FDNN_BF16: return densify_w_t<__nv_bfloat16>(w, w_s, K, C, R, S, groups, dense, stream);
    case FDNN_F32: return densify_w_t<float>(w, w_s, K, C, R, S, groups, dense, stream);
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
