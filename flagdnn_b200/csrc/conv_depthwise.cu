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

#include <atomic>
#include <type_traits>

#include "conv_convert.cuh"
#include "conv_epilogue.cuh"
#include "conv_internal.h"

namespace fdnn {
namespace {

constexpr int kDwThreads = 256;
constexpr int kDwMaxSmemFloats = 12288;  // 48 KB of taps at most
constexpr int kDwRounds = 6;              // units a resident thread group should get at least (load balance)

// SM count of the current device, looked up once per device ordinal.
inline int sm_count_dw() {
  static std::atomic<int> cached[64];
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  v = cached[dev].load(std::memory_order_relaxed);
  if (v > 0) return v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v < 1) return 148;
  cached[dev].store(v, std::memory_order_relaxed);
  return v;
}

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
// How a launch divides the work: a block is `tcx` channel vectors wide and `tpy` units deep; a unit is PW
// neighbouring output columns of `band_rows` consecutive output rows of one image, walked top to bottom by one
// thread per channel vector (so two of a 3x3 window's three input rows are still in L1 from the row before).
struct DwTiling {
  int tcx, tpy;        // blockDim.x = tcx * tpy
  int owg;             // column groups per output row
  int bands;           // row bands per image
  int band_rows;
  unsigned units;      // N * bands * owg
};

// VB bytes of neighbouring channels as 32-bit words.
template <int VB>
struct Words {
  uint32_t w[VB / 4];
};
template <int VB>
__device__ __forceinline__ Words<VB> load_words(const void* ptr) {
  Words<VB> r;
  if constexpr (VB == 16) {
    const uint4 q = __ldg(static_cast<const uint4*>(ptr));
    r.w[0] = q.x; r.w[1] = q.y; r.w[2] = q.z; r.w[3] = q.w;
  } else if constexpr (VB == 8) {
    const uint2 q = __ldg(static_cast<const uint2*>(ptr));
    r.w[0] = q.x; r.w[1] = q.y;
  } else {
    r.w[0] = __ldg(static_cast<const uint32_t*>(ptr));
  }
  return r;
}
template <int VB>
__device__ __forceinline__ void store_words_streaming(void* ptr, const Words<VB>& r) {
  if constexpr (VB == 16) {
    __stcs(static_cast<uint4*>(ptr), make_uint4(r.w[0], r.w[1], r.w[2], r.w[3]));
  } else if constexpr (VB == 8) {
    __stcs(static_cast<uint2*>(ptr), make_uint2(r.w[0], r.w[1]));
  } else {
    __stcs(static_cast<uint32_t*>(ptr), r.w[0]);
  }
}
// Two fp32 values of neighbouring channels in one 64-bit register, the operand form of fma.rn.f32x2 (two
// independent, correctly rounded fp32 FMAs per instruction).  They are kept as 64-bit integers so that the
// compiler carries each pair through branches and loops as one value instead of splitting and re-joining it.
using F2 = unsigned long long;
__device__ __forceinline__ F2 f2_make(uint32_t lo_bits, uint32_t hi_bits) {
  F2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo_bits), "r"(hi_bits));
  return d;
}
__device__ __forceinline__ void f2_split(F2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ F2 f2_fma(F2 a, F2 b, F2 c) {
  F2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
// The words as fp32 pairs of neighbouring channels (one pair per word for 16-bit types, per two words for fp32).
template <typename T, int VB>
__device__ __forceinline__ void words_to_pairs(const Words<VB>& r, F2 (&v)[VB / (2 * sizeof(T))]) {
#pragma unroll
  for (int h = 0; h < int(VB / (2 * sizeof(T))); ++h) {
    if constexpr (std::is_same<T, float>::value) {
      v[h] = f2_make(r.w[2 * h], r.w[2 * h + 1]);
    } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      v[h] = f2_make(r.w[h] << 16, r.w[h] & 0xffff0000u);
    } else {
      float lo, hi;
      unpack2<T>(r.w[h], lo, hi);
      v[h] = f2_make(__float_as_uint(lo), __float_as_uint(hi));
    }
  }
}

// Shared memory of one block: fp32 pairs of neighbouring channels, [R*S + 2][V/2][tcx] — the taps of channels
// cbase .. cbase + cspan, then their scale (1 when the call has none), then their bias (0 when none).  Thread tc
// owns channels tc*V .. tc*V+V-1; with the thread index innermost the 32 lanes of a warp read 32 consecutive
// 8-byte words, two wavefronts per load (rows of V floats per thread cost eight).
template <typename T>
__device__ __forceinline__ void fill_filter_rows(float* s_w, const DirectParams& p, int R, int S, int V, int tcx,
                                                 int cbase, int cspan) {
  const T* w = static_cast<const T*>(p.w);
  const T* bias = static_cast<const T*>(p.bias);
  const T* scale = static_cast<const T*>(p.scale);
  const int taps = R * S, h2 = V / 2;
  for (int i = threadIdx.x; i < (taps + 2) * cspan; i += blockDim.x) {
    const int tap = i / cspan, c = i - tap * cspan;
    float v;
    if (tap < taps) {
      const int r = tap / S, s = tap - r * S;
      v = to_f32<T>(w[(cbase + c) * p.w_s[0] + r * p.w_s[2] + s * p.w_s[3]]);
    } else if (tap == taps) {
      v = scale != nullptr ? to_f32<T>(scale[cbase + c]) : 1.0f;
    } else {
      v = bias != nullptr ? to_f32<T>(bias[cbase + c]) : 0.0f;
    }
    const int tc = c / V, e = c - tc * V;
    s_w[((tap * h2 + (e >> 1)) * tcx + tc) * 2 + (e & 1)] = v;
  }
}

// One output pixel's VB bytes of channels: scale and bias, residual, activation, one rounding, streaming store.
template <typename T, int VB>
__device__ __forceinline__ void emit_pixel(const F2 (&acc)[VB / (2 * sizeof(T))], const F2* s_scale, const F2* s_bias,
                                           int pair_stride, const T* res, T* y, int act) {
  constexpr int H2 = VB / (2 * int(sizeof(T)));
  constexpr int V = 2 * H2;
  float v[V];
#pragma unroll
  for (int h = 0; h < H2; ++h)
    f2_split(f2_fma(acc[h], s_scale[h * pair_stride], s_bias[h * pair_stride]), v[2 * h], v[2 * h + 1]);
  if (res != nullptr) {
    const Words<VB> rw = load_words<VB>(res);
#pragma unroll
    for (int h = 0; h < H2; ++h) {
      float lo, hi;
      if constexpr (std::is_same<T, float>::value) {
        lo = __uint_as_float(rw.w[2 * h]); hi = __uint_as_float(rw.w[2 * h + 1]);
      } else {
        unpack2<T>(rw.w[h], lo, hi);
      }
      v[2 * h] += lo; v[2 * h + 1] += hi;
    }
  }
  Words<VB> out;
  if constexpr (std::is_same<T, float>::value) {
#pragma unroll
    for (int e = 0; e < V; ++e) out.w[e] = __float_as_uint(act ? apply_activation(v[e], act) : v[e]);
  } else if (act == 1) {   // ReLU folded into the rounding conversion, as in the tensor-core epilogue
#pragma unroll
    for (int h = 0; h < H2; ++h) out.w[h] = round_pack2_relu<T>(v[2 * h], v[2 * h + 1]);
  } else {
    if (act) {
#pragma unroll
      for (int e = 0; e < V; ++e) v[e] = apply_activation(v[e], act);
    }
#pragma unroll
    for (int h = 0; h < H2; ++h) out.w[h] = round_pack2<T>(v[2 * h], v[2 * h + 1]);
  }
  store_words_streaming<VB>(y, out);
}

// KR, KS, KSTRIDE: filter size and (equal) strides known at compile time, dilation 1 — every loop unrolls and
// the tap a column serves for each output is resolved by the compiler; 0, 0, 0 takes everything from `p`.
// VB: bytes of channels a thread owns (16, or 8 where more resident warps pay more than wider accesses).
// Shared memory holds the R*S taps, the scale and the bias of the block's channels as fp32 pairs (fill_filter_rows).
// All arithmetic is on pairs of neighbouring channels (fma.rn.f32x2: two independent, correctly rounded fp32
// FMAs per instruction).
template <typename T, int KR, int KS, int KSTRIDE, int VB>
__global__ void __launch_bounds__(kDwThreads, (KR == 5 && KSTRIDE == 2) ? 1 : 2)
depthwise_cl_kernel(const DirectParams p, const DwTiling g) {
  constexpr int V = VB / int(sizeof(T));  // channels per thread
  constexpr int H2 = V / 2;               // pairs of channels
  constexpr bool kStatic = KR != 0;
  constexpr int PW = kStatic ? 4 : 2;     // output pixels per thread, along W
  extern __shared__ __align__(16) float s_w[];   // [R*S + 2][tcx * V]
  const int R = kStatic ? KR : p.R, S = kStatic ? KS : p.S;
  const int stride_h = kStatic ? KSTRIDE : p.stride_h, stride_w = kStatic ? KSTRIDE : p.stride_w;
  const int dil_h = kStatic ? 1 : p.dil_h, dil_w = kStatic ? 1 : p.dil_w;
  const int taps = R * S;
  const int pitch = g.tcx * V;
  const int cbase = blockIdx.y * pitch;
  const int cspan = min(pitch, p.C - cbase);
  fill_filter_rows<T>(s_w, p, R, S, V, g.tcx, cbase, cspan);
  __syncthreads();
  const int tc = threadIdx.x % g.tcx, tp = threadIdx.x / g.tcx;
  if (tc * V >= cspan) return;
  const int c0 = cbase + tc * V;
  const F2* s_mine = reinterpret_cast<const F2*>(s_w) + tc;   // pair h of tap t: s_mine[(t * H2 + h) * tcx]
  const int tcx = g.tcx;
  const int act = p.act;
  constexpr int kSpanStatic = (PW - 1) * KSTRIDE + KS;           // input columns the PW outputs touch
  const int span = kStatic ? kSpanStatic : (PW - 1) * stride_w + (S - 1) * dil_w + 1;

  // the grid is sized to the resident blocks of the device: a block fills its shared memory once and walks units
  for (unsigned unit = blockIdx.x * unsigned(g.tpy) + unsigned(tp); unit < g.units; unit += gridDim.x * unsigned(g.tpy)) {
  const int colg = int(unit % unsigned(g.owg));
  const unsigned rest = unit / unsigned(g.owg);
  const int band = int(rest % unsigned(g.bands));
  const int n = int(rest / unsigned(g.bands));
  const int ow0 = colg * PW;
  const int oh_begin = band * g.band_rows;
  const int oh_end = min(p.OH, oh_begin + g.band_rows);
  const int iw0 = ow0 * stride_w - p.pad_left;

  const T* img = static_cast<const T*>(p.x) + n * p.x_s[0] + c0;
  const T* res = p.residual != nullptr ? static_cast<const T*>(p.residual) + n * p.y_s[0] + c0 : nullptr;
  T* yimg = static_cast<T*>(p.y) + n * p.y_s[0] + c0;
  unsigned col_ok = 0;                                           // bit j: column iw0 + j lies inside the image
  if constexpr (kStatic) {
#pragma unroll
    for (int j = 0; j < kSpanStatic; ++j) col_ok |= (iw0 + j >= 0 && iw0 + j < p.W) ? (1u << j) : 0u;
  }

  for (int oh = oh_begin; oh < oh_end; ++oh) {
    F2 acc[PW][H2];
#pragma unroll
    for (int q = 0; q < PW; ++q)
#pragma unroll
      for (int h = 0; h < H2; ++h) acc[q][h] = 0ull;
    if constexpr (kStatic) {
      // no branch around the arithmetic: a row or column outside the image loads zeros instead
#pragma unroll
      for (int r = 0; r < KR; ++r) {
        const int ih = oh * KSTRIDE + r - p.pad_top;
        const bool row_ok = ih >= 0 && ih < p.H;
        const T* row = img + (row_ok ? ih : 0) * p.x_s[2] + iw0 * p.x_s[3];
        Words<VB> raw[kSpanStatic];
        if (row_ok && col_ok == (1u << kSpanStatic) - 1u) {   // all but the units on the image's border
#pragma unroll
          for (int j = 0; j < kSpanStatic; ++j) raw[j] = load_words<VB>(row + j * p.x_s[3]);
        } else {
#pragma unroll
          for (int j = 0; j < kSpanStatic; ++j) {
#pragma unroll
            for (int i = 0; i < VB / 4; ++i) raw[j].w[i] = 0u;
            if (row_ok && (col_ok & (1u << j))) raw[j] = load_words<VB>(row + j * p.x_s[3]);
          }
        }
#pragma unroll
        for (int j = 0; j < kSpanStatic; ++j) {
          F2 xv[H2];
          words_to_pairs<T, VB>(raw[j], xv);
#pragma unroll
          for (int q = 0; q < PW; ++q) {
            const int s = j - q * KSTRIDE;   // a constant once the loops are unrolled
            if (s >= 0 && s < KS) {
              const F2* tap = s_mine + (r * KS + s) * H2 * tcx;
#pragma unroll
              for (int h = 0; h < H2; ++h) acc[q][h] = f2_fma(xv[h], tap[h * tcx], acc[q][h]);
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
          F2 xv[H2];
          words_to_pairs<T, VB>(load_words<VB>(row + iw * p.x_s[3]), xv);
#pragma unroll
          for (int q = 0; q < PW; ++q) {
            const int d = j - q * stride_w;          // = s * dil_w for the tap this column is for output q
            if (d < 0 || d % dil_w != 0) continue;
            const int s = d / dil_w;
            if (s >= S) continue;
            const F2* tap = s_mine + (r * S + s) * H2 * tcx;
#pragma unroll
            for (int h = 0; h < H2; ++h) acc[q][h] = f2_fma(xv[h], tap[h * tcx], acc[q][h]);
          }
        }
      }
    }
#pragma unroll
    for (int q = 0; q < PW; ++q) {
      const int ow = ow0 + q;
      if (ow >= p.OW) continue;
      const long long y_idx = oh * p.y_s[2] + ow * p.y_s[3];
      emit_pixel<T, VB>(acc[q], s_mine + taps * H2 * tcx, s_mine + (taps + 1) * H2 * tcx, tcx,
                        res != nullptr ? res + y_idx : nullptr, yimg + y_idx, act);
    }
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

// ------------------------------------------------- NCHW, rows read as 16- or 8-byte vectors
// W-contiguous planes whose rows start on VB-byte boundaries, "same" padding (pad_left == KS / 2), no dilation:
// a thread owns V = VB / sizeof(T) neighbouring outputs of a row.  The input columns they need are KSTRIDE
// aligned vectors plus KS / 2 single columns on the left and KS - KS / 2 - KSTRIDE on the right (L1 hits: they
// are the neighbouring threads' vectors).  A unit is one such column group over `band_rows` output rows of one
// plane; its thread keeps the plane's taps, scale and bias in registers.
struct DwRowTiling {
  int owg, bands, band_rows;
  long long units;     // N * C * bands * owg
};

template <typename T, int VB>
__device__ __forceinline__ void words_to_floats(const Words<VB>& r, float (&v)[VB / sizeof(T)]) {
  if constexpr (std::is_same<T, float>::value) {
#pragma unroll
    for (int i = 0; i < VB / 4; ++i) v[i] = __uint_as_float(r.w[i]);
  } else {
#pragma unroll
    for (int i = 0; i < VB / 4; ++i) unpack2<T>(r.w[i], v[2 * i], v[2 * i + 1]);
  }
}

template <typename T, int KR, int KS, int KSTRIDE, int VB>
__global__ void __launch_bounds__(kDwThreads)
depthwise_rowvec_kernel(const DirectParams p, const DwRowTiling g) {
  constexpr int V = VB / int(sizeof(T));
  constexpr int PAD = KS / 2;
  constexpr int kSpan = (V - 1) * KSTRIDE + KS;
  constexpr int kRight0 = PAD + KSTRIDE * V;          // first column index right of the vectors
  const long long unit = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (unit >= g.units) return;
  const int colg = int(unit % g.owg);
  long long rest = unit / g.owg;
  const int band = int(rest % g.bands);
  rest /= g.bands;
  const int c = int(rest % p.C);
  const int n = int(rest / p.C);
  const int ow0 = colg * V;
  const int col0 = ow0 * KSTRIDE;                     // column of the first vector: a multiple of V
  const int oh_begin = band * g.band_rows;
  const int oh_end = min(p.OH, oh_begin + g.band_rows);

  const T* w = static_cast<const T*>(p.w) + c * p.w_s[0];
  float wt[KR * KS];
#pragma unroll
  for (int r = 0; r < KR; ++r)
#pragma unroll
    for (int s2 = 0; s2 < KS; ++s2) wt[r * KS + s2] = to_f32<T>(__ldg(w + r * p.w_s[2] + s2 * p.w_s[3]));
  const float sc = p.scale != nullptr ? to_f32<T>(static_cast<const T*>(p.scale)[c]) : 1.0f;
  const float bi = p.bias != nullptr ? to_f32<T>(static_cast<const T*>(p.bias)[c]) : 0.0f;
  const T* x = static_cast<const T*>(p.x) + n * p.x_s[0] + c * p.x_s[1];
  T* y = static_cast<T*>(p.y) + n * p.y_s[0] + c * p.y_s[1];
  const T* res = p.residual != nullptr ? static_cast<const T*>(p.residual) + n * p.y_s[0] + c * p.y_s[1] : nullptr;
  const int act = p.act;
  const bool full_store = ow0 + V <= p.OW;

  for (int oh = oh_begin; oh < oh_end; ++oh) {
    float acc[V];
#pragma unroll
    for (int q = 0; q < V; ++q) acc[q] = 0.0f;
#pragma unroll
    for (int r = 0; r < KR; ++r) {
      const int ih = oh * KSTRIDE + r - p.pad_top;
      if (ih < 0 || ih >= p.H) continue;
      const T* row = x + ih * p.x_s[2];
      float xin[kSpan];
#pragma unroll
      for (int j = 0; j < PAD; ++j) {
        const int iw = col0 - PAD + j;
        xin[j] = (iw >= 0 && iw < p.W) ? to_f32<T>(__ldg(row + iw)) : 0.0f;
      }
#pragma unroll
      for (int t = 0; t < KSTRIDE; ++t) {
        const int col = col0 + t * V;
        if (col + V <= p.W) {
          float xv[V];
          words_to_floats<T, VB>(load_words<VB>(row + col), xv);
#pragma unroll
          for (int e = 0; e < V; ++e)
            if (PAD + t * V + e < kSpan) xin[PAD + t * V + e] = xv[e];
        } else {
#pragma unroll
          for (int e = 0; e < V; ++e)
            if (PAD + t * V + e < kSpan) xin[PAD + t * V + e] = (col + e < p.W) ? to_f32<T>(__ldg(row + col + e)) : 0.0f;
        }
      }
#pragma unroll
      for (int j = kRight0; j < kSpan; ++j) {
        const int iw = col0 - PAD + j;
        xin[j] = (iw < p.W) ? to_f32<T>(__ldg(row + iw)) : 0.0f;
      }
#pragma unroll
      for (int q = 0; q < V; ++q)
#pragma unroll
        for (int s2 = 0; s2 < KS; ++s2) acc[q] = fmaf(xin[q * KSTRIDE + s2], wt[r * KS + s2], acc[q]);
    }
    const long long y_idx = oh * p.y_s[2] + ow0;
#pragma unroll
    for (int q = 0; q < V; ++q) acc[q] = fmaf(acc[q], sc, bi);
    if (full_store) {
      if (res != nullptr) {
        float rv[V];
        words_to_floats<T, VB>(load_words<VB>(res + y_idx), rv);
#pragma unroll
        for (int q = 0; q < V; ++q) acc[q] += rv[q];
      }
      Words<VB> out;
      if constexpr (std::is_same<T, float>::value) {
#pragma unroll
        for (int q = 0; q < V; ++q) out.w[q] = __float_as_uint(act ? apply_activation(acc[q], act) : acc[q]);
      } else if (act == 1) {
#pragma unroll
        for (int q = 0; q < V / 2; ++q) out.w[q] = round_pack2_relu<T>(acc[2 * q], acc[2 * q + 1]);
      } else {
        if (act) {
#pragma unroll
          for (int q = 0; q < V; ++q) acc[q] = apply_activation(acc[q], act);
        }
#pragma unroll
        for (int q = 0; q < V / 2; ++q) out.w[q] = round_pack2<T>(acc[2 * q], acc[2 * q + 1]);
      }
      store_words_streaming<VB>(y + y_idx, out);
    } else {
#pragma unroll
      for (int q = 0; q < V; ++q) {
        if (ow0 + q >= p.OW) continue;
        float a = acc[q];
        if (res != nullptr) a += to_f32<T>(res[y_idx + q]);
        y[y_idx + q] = from_f32<T>(apply_activation(a, act));
      }
    }
  }
}

template <typename T, int KR, int KS, int KSTRIDE, int VB>
cudaError_t launch_rowvec(const DirectParams& p, cudaStream_t stream) {
  constexpr int V = VB / int(sizeof(T));
  DwRowTiling g;
  g.owg = (p.OW + V - 1) / V;
  g.band_rows = 8;
  while (g.band_rows > 1 &&
         (long long)p.N * p.C * ((p.OH + g.band_rows - 1) / g.band_rows) * g.owg < 148LL * 8 * kDwThreads)
    g.band_rows /= 2;
  g.bands = (p.OH + g.band_rows - 1) / g.band_rows;
  g.units = (long long)p.N * p.C * g.bands * g.owg;
  const long long blocks = (g.units + kDwThreads - 1) / kDwThreads;
  depthwise_rowvec_kernel<T, KR, KS, KSTRIDE, VB><<<unsigned(blocks), kDwThreads, 0, stream>>>(p, g);
  return cudaGetLastError();
}

// Launch of a channels-last kernel: V channels per thread, PW output columns per unit, at most `band_max` rows.
// The grid is the blocks the device keeps resident (asked of the runtime once per kernel and shared-memory
// size), so that a block fills its shared memory once and then walks units.
template <typename Kernel>
cudaError_t launch_cl(Kernel kernel, const DirectParams& p, int V, int PW, int band_max, cudaStream_t stream) {
  DwTiling g;
  const int cv = p.C / V;
  g.tcx = cv < kDwThreads ? cv : kDwThreads;
  const int fit = kDwMaxSmemFloats / ((p.R * p.S + 2) * V);   // channel vectors whose rows fit shared memory
  if (g.tcx > fit) g.tcx = fit;
  g.tpy = kDwThreads / g.tcx;
  g.owg = (p.OW + PW - 1) / PW;
  const size_t smem = size_t(p.R * p.S + 2) * g.tcx * V * sizeof(float);
  static std::atomic<long long> cached{0};   // smem << 8 | blocks per SM (one per instantiation, i.e. per kernel)
  long long c = cached.load(std::memory_order_relaxed);
  if ((c >> 8) != (long long)smem || (c & 255) == 0) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, g.tcx * g.tpy, smem) != cudaSuccess ||
        per_sm < 1)
      per_sm = 1;
    c = ((long long)smem << 8) | (per_sm & 255);
    cached.store(c, std::memory_order_relaxed);
  }
  const int chunks = (cv + g.tcx - 1) / g.tcx;
  const long long resident = (long long)sm_count_dw() * (c & 255);
  const long long groups = resident / chunks > 0 ? resident / chunks * g.tpy : g.tpy;   // units in flight
  // rows per unit: `band_max` while every resident thread group still gets kDwRounds units, fewer otherwise
  g.band_rows = band_max;
  while (g.band_rows > 1 &&
         (long long)p.N * ((p.OH + g.band_rows - 1) / g.band_rows) * g.owg < kDwRounds * groups)
    g.band_rows = (g.band_rows + 1) / 2;
  g.bands = (p.OH + g.band_rows - 1) / g.band_rows;
  g.units = unsigned((long long)p.N * g.bands * g.owg);
  long long gx = (g.units + g.tpy - 1) / g.tpy;
  if (gx > groups / g.tpy) gx = groups / g.tpy;
  if (gx < 1) gx = 1;
  kernel<<<dim3(unsigned(gx), chunks), g.tcx * g.tpy, smem, stream>>>(p, g);
  return cudaGetLastError();
}

template <typename T, int KR, int KS, int KSTRIDE>
cudaError_t go_static(const DirectParams& p, int kind, cudaStream_t stream) {
  const bool channels_last = kind == 1;
  if constexpr (KR != 0) {
    if (kind == 3) return launch_rowvec<T, KR, KS, KSTRIDE, 16>(p, stream);
    if (kind == 4) return launch_rowvec<T, KR, KS, KSTRIDE, 8>(p, stream);
    if constexpr (sizeof(T) == 2) {
      if (kind == 5) return launch_rowvec<T, KR, KS, KSTRIDE, 4>(p, stream);
    }
  }
  if (channels_last) {
    constexpr int VB = 16;
    return launch_cl(depthwise_cl_kernel<T, KR, KS, KSTRIDE, VB>, p, VB / int(sizeof(T)), KR != 0 ? 4 : 2, 8, stream);
  } else {
    depthwise_plane_kernel<T, KR, KS, KSTRIDE><<<p.N * p.C, kDwThreads, size_t(p.R) * p.S * sizeof(float), stream>>>(p);
  }
  return cudaGetLastError();
}

template <typename T>
cudaError_t go(const DirectParams& p, int channels_last, cudaStream_t stream) {   // the kind, passed through
  // the common filters get fully unrolled kernels; everything else (dilation, unequal strides, other sizes)
  // the run-time one
  if (p.dil_h == 1 && p.dil_w == 1 && p.stride_h == p.stride_w && p.R == p.S) {
    if (p.R == 3 && p.stride_w == 1) return go_static<T, 3, 3, 1>(p, channels_last, stream);
    if (p.R == 3 && p.stride_w == 2) return go_static<T, 3, 3, 2>(p, channels_last, stream);
    if (p.R == 5 && p.stride_w == 1) return go_static<T, 5, 5, 1>(p, channels_last, stream);
    if (p.R == 5 && p.stride_w == 2) return go_static<T, 5, 5, 2>(p, channels_last, stream);
  }
  return go_static<T, 0, 0, 0>(p, channels_last >= 3 ? 2 : channels_last, stream);
}

}  // namespace

// 0: not a case for these kernels (the caller uses the direct kernel); 1: channels-last kernel; 2: plane kernel;
// 3 / 4 / 5: row-vector kernel (NCHW) on 16- / 8- / 4-byte vectors.
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
                  mult(p.OH, p.y_s[2]) && mult(p.OW, p.y_s[3]) && (long long)(p.R * p.S + 2) * v <= kDwMaxSmemFloats &&
                  p.C > 1 && (long long)p.N * p.OH * p.OW < 2147483647LL && p.C / v < 65536LL * 8;
  if (cl) return 1;
  // W-contiguous planes with vector-aligned rows and "same" padding of an unrolled filter: the row-vector kernel
  // on the widest vectors the rows are aligned for (16 bytes; 8 for rows of 28 16-bit values; 4 for rows of 14)
  const bool unrolled = p.dil_h == 1 && p.dil_w == 1 && p.stride_h == p.stride_w && p.R == p.S &&
                        (p.R == 3 || p.R == 5) && (p.stride_w == 1 || p.stride_w == 2);
  if (unrolled && p.pad_left == p.S / 2 && p.x_s[3] == 1 && p.y_s[3] == 1) {
    for (int vb = 16; vb >= 4; vb /= 2) {
      const int vv = vb / es;
      if (vv < 2) break;
      const bool al = ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.y) |
                        reinterpret_cast<uintptr_t>(p.residual)) & uintptr_t(vb - 1)) == 0;
      auto m = [vv](long long extent, long long stride) { return extent <= 1 || stride % vv == 0; };
      if (al && m(p.N, p.x_s[0]) && m(p.C, p.x_s[1]) && m(p.H, p.x_s[2]) && m(p.N, p.y_s[0]) && m(p.C, p.y_s[1]) &&
          m(p.OH, p.y_s[2]) && p.W >= vv && (long long)p.N * p.C * p.OH * ((p.OW + vv - 1) / vv) < 2147483647LL * 128)
        return vb == 16 ? 3 : (vb == 8 ? 4 : 5);
    }
  }
  if ((long long)p.N * p.C < 2147483647LL && p.R * p.S <= kDwMaxSmemFloats) return 2;
  return 0;
}

cudaError_t launch_depthwise(int dtype, const DirectParams& p, int kind, cudaStream_t stream) {
  switch (dtype) {
    case FDNN_F16: return go<__half>(p, kind, stream);
    case FDNN_BF16: return go<__nv_bfloat16>(p, kind, stream);
    case FDNN_F32: return go<float>(p, kind, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace fdnn
