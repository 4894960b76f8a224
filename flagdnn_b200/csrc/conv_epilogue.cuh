// Epilogue shared by the implicit-GEMM kernels when y is dense NHWC: one warp
// drains its 32 accumulator rows from tensor memory, applies per-channel scale,
// bias and the activation in fp32, rounds once, stages 32 rows x 128 bytes in shared
// memory and hands each box to a TMA store.  The arithmetic is that of the
// reference's fused kernel (src/flag_dnn/graph/kernels/fused_conv.py:297-310),
// plus an optional residual tensor added in fp32 before the activation.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "sm100_ptx.cuh"
#include "stream_k.cuh"

namespace fdnn {

// max(a, 0) that returns NaN for NaN, like torch.relu (plain max would return 0).
__device__ __forceinline__ float relu_keep_nan(float a) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(0.0f));
  return r;
}

// Two fp32 values -> max(., 0) -> one rounding -> a packed 16-bit pair, in one conversion instruction
// (cvt.rn.relu): saves the two separate maximum instructions per pair in a drain loop that is bound by
// instruction issue on short-reduction layers.  NaN stays NaN (the canonical one), like torch.relu.
template <typename T>
__device__ __forceinline__ uint32_t round_pack2_relu(float a, float b);
template <>
__device__ __forceinline__ uint32_t round_pack2_relu<__half>(float a, float b) {
  uint32_t r;
  asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));  // first source operand lands in the high half
  return r;
}
template <>
__device__ __forceinline__ uint32_t round_pack2_relu<__nv_bfloat16>(float a, float b) {
  uint32_t r;
  asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}

// Epilogue activation by its FDNN_ACT_* code: none, ReLU, GELU (erf form, torch's default) or GELU's tanh
// approximation (torch's approximate="tanh").  All keep NaN.
__device__ __forceinline__ float apply_activation(float v, int act) {
  if (act == 1) return relu_keep_nan(v);
  if (act == 2) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
  if (act == 3) {
    const float u = 0.79788456080286536f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(u));
  }
  return v;
}

template <typename T>
__device__ __forceinline__ uint32_t round_pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t round_pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t round_pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Two packed 16-bit values -> fp32 (identity for fp32 words is handled by the caller).
template <typename T>
__device__ __forceinline__ void unpack2(uint32_t w, float& a, float& b);
template <>
__device__ __forceinline__ void unpack2<__half>(uint32_t w, float& a, float& b) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
  a = f.x;
  b = f.y;
}
template <>
__device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t w, float& a, float& b) {
  a = __uint_as_float(w << 16);
  b = __uint_as_float(w & 0xffff0000u);
}
template <>
__device__ __forceinline__ void unpack2<float>(uint32_t w, float& a, float& b) {
  a = __uint_as_float(w);
  b = 0.0f;
}

// How an epilogue warp gets its residual values: the TMA unit copies the 32-row x 128-byte box of the residual
// tensor (seen exactly like y, same swizzle) straight into the staging buffer the outputs will leave from; the
// lane then reads its own row, adds, and writes the finished row back in place.  With two staging buffers the
// box of the next column group is on its way while this one is computed.
struct ResidualFetch {
  const CUtensorMap* tm;          // nullptr: no residual for this warp's rows
  uint64_t* bars;                 // this warp's mbarriers, one per staging buffer
  uint32_t* phases;               // bit b: the parity bars[b] completes next
  volatile uint32_t* abort_flag;  // bounded waits, as everywhere in the kernels
  uint32_t* status_word;
  long long wait_limit;
};

// t_row     tensor-memory address of this warp's lane quarter, first column of the tile
// n0        first GEMM column of the tile; kout: number of valid GEMM columns overall
// s_scale / s_bias  this warp's fp32 copies for columns n0 .. n0+BN-1
// my_out    this warp's NBUF 4 KB staging buffers (1024-byte aligned; two are used in rotation so
//           that a box can still be leaving through the TMA unit while the next one is staged;
//           with one, the other warp of the lane quarter fills that gap)
// tm_full / tm_tail  output maps with a 32-row box and a box of the tile's ragged last rows
// st_row, st_img     y coordinates (row, image) of the warp's first row; st_rows: valid rows (<= 0: none)
// store_seq          running count of this warp's staged boxes (selects the staging buffer)
// use_scale          false when the launch has no per-channel scale (s_scale then holds ones and is not read)
// RES                a residual tensor (same layout as y) is added before the activation
// rf                 how the residual box reaches the staging buffer (see ResidualFetch; the producer asked for
//                    the tile's residual values to be brought into L2 a main loop earlier)
// sk_slot0 / sk_count / sk_slot_stride / sk_row / sk_pc0
//                    reduction splitting: the accumulator holds only the tile's last reduction steps; add the
//                    fp32 partial sums of sk_count other CTAs first (slots sk_slot0, sk_slot0 - sk_slot_stride,
//                    ... in that order; this lane's row sk_row, this warp's first 16-byte piece sk_pc0)
template <typename T, int BN, bool RES = false, int NBUF = 2>
__device__ __forceinline__ void epilogue_store_tile(uint32_t t_row, int n0, int kout, int act,
                                                    const float* s_scale, const float* s_bias,
                                                    uint8_t* my_out, int lane, const CUtensorMap* tm_full,
                                                    const CUtensorMap* tm_tail, int st_row, int st_img,
                                                    int st_rows, uint32_t& store_seq,
                                                    const ResidualFetch* rf = nullptr, bool use_scale = true,
                                                    const float* sk_slot0 = nullptr, int sk_count = 0,
                                                    long long sk_slot_stride = 0, int sk_row = 0, int sk_pc0 = 0) {
  constexpr int kPerStore = 128 / int(sizeof(T));  // channels per staged row: 64 (16-bit) or 32 (fp32)
  constexpr int kLoads = kPerStore / 32;
  int groups = (kout - n0 + kPerStore - 1) / kPerStore;
  if (groups > BN / kPerStore) groups = BN / kPerStore;
  if (groups <= 0) return;
  uint32_t raw[kLoads][32];
#pragma unroll
  for (int l = 0; l < kLoads; ++l) tmem_ld_32x32b_x32(t_row + l * 32, raw[l]);
#pragma unroll 1
  for (int g = 0; g < groups; ++g) {
    uint8_t* buf = my_out + (NBUF == 2 ? (store_seq & 1u) * (32 * 128) : 0u);  // alternates across groups AND tiles
    ++store_seq;
    if constexpr (RES) {
      const bool have = rf != nullptr && rf->tm != nullptr && st_rows > 0;   // uniform across the warp
      const uint32_t b = NBUF == 2 ? ((store_seq - 1u) & 1u) : 0u;
      if (lane == 0) {
        bulk_wait_group_read0();   // every staged box has left: both buffers may be written
        if (have) {
          if (g == 0 || NBUF == 1) {
            mbar_arrive_expect_tx(&rf->bars[b], 32 * 128);
            tma_load_3d(buf, rf->tm, &rf->bars[b], n0 + g * kPerStore, st_row, st_img);
          }
          if (NBUF == 2 && g + 1 < groups) {
            mbar_arrive_expect_tx(&rf->bars[b ^ 1u], 32 * 128);
            tma_load_3d(my_out + (b ^ 1u) * (32 * 128), rf->tm, &rf->bars[b ^ 1u], n0 + (g + 1) * kPerStore, st_row,
                        st_img);
          }
        }
      }
      __syncwarp();
      if (have) {
        mbar_wait_bounded(&rf->bars[b], (*rf->phases >> b) & 1u, rf->abort_flag, rf->status_word,
                          kIncidentResidualWait, rf->wait_limit);
        *rf->phases ^= 1u << b;
      }
    }
    tmem_ld_wait();
    for (int c = 0; c < sk_count; ++c) {  // uniform across the launch's owner tiles; zero otherwise
      const float* slot = sk_slot0 - c * sk_slot_stride;
#pragma unroll
      for (int l = 0; l < kLoads; ++l) {
        float4 part[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) part[j] = sk_load_piece(slot, sk_pc0 + g * (kPerStore / 4) + l * 8 + j, sk_row);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          raw[l][4 * j + 0] = __float_as_uint(__uint_as_float(raw[l][4 * j + 0]) + part[j].x);
          raw[l][4 * j + 1] = __float_as_uint(__uint_as_float(raw[l][4 * j + 1]) + part[j].y);
          raw[l][4 * j + 2] = __float_as_uint(__uint_as_float(raw[l][4 * j + 2]) + part[j].z);
          raw[l][4 * j + 3] = __float_as_uint(__uint_as_float(raw[l][4 * j + 3]) + part[j].w);
        }
      }
    }
    uint32_t row[32];  // the 128 bytes this lane contributes
#pragma unroll
    for (int l = 0; l < kLoads; ++l) {
      const float4* sc4 = reinterpret_cast<const float4*>(s_scale + g * kPerStore + l * 32);
      const float4* bi4 = reinterpret_cast<const float4*>(s_bias + g * kPerStore + l * 32);
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4) {
        // without a per-channel scale the multiplier is 1 and its shared-memory read is skipped (uniform
        // branch): -13 % on a 64 -> 256 1x1 layer; packing scale and bias into one word per column instead
        // saves the same reads but pays them back in unpacking instructions
        const float4 sc = use_scale ? sc4[j4] : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        const float4 bi = bi4[j4];
        float v0 = fmaf(__uint_as_float(raw[l][4 * j4 + 0]), sc.x, bi.x);
        float v1 = fmaf(__uint_as_float(raw[l][4 * j4 + 1]), sc.y, bi.y);
        float v2 = fmaf(__uint_as_float(raw[l][4 * j4 + 2]), sc.z, bi.z);
        float v3 = fmaf(__uint_as_float(raw[l][4 * j4 + 3]), sc.w, bi.w);
        if constexpr (RES) {
          if constexpr (std::is_same<T, float>::value) {
            const uint4 mine = *reinterpret_cast<const uint4*>(buf + lane * 128 + ((j4 ^ (lane & 7)) << 4));
            v0 += __uint_as_float(mine.x);
            v1 += __uint_as_float(mine.y);
            v2 += __uint_as_float(mine.z);
            v3 += __uint_as_float(mine.w);
          } else {
            // 16-byte piece l*4 + j4/2 of the row holds the eight values of two passes of this loop
            const uint2 mine = *reinterpret_cast<const uint2*>(
                buf + lane * 128 + (((l * 4 + (j4 >> 1)) ^ (lane & 7)) << 4) + ((j4 & 1) << 3));
            float r0, r1, r2, r3;
            unpack2<T>(mine.x, r0, r1);
            unpack2<T>(mine.y, r2, r3);
            v0 += r0;
            v1 += r1;
            v2 += r2;
            v3 += r3;
          }
        }
        if constexpr (std::is_same<T, float>::value) {
          if (act) {  // uniform across the launch
            v0 = apply_activation(v0, act);
            v1 = apply_activation(v1, act);
            v2 = apply_activation(v2, act);
            v3 = apply_activation(v3, act);
          }
          row[4 * j4 + 0] = __float_as_uint(v0);
          row[4 * j4 + 1] = __float_as_uint(v1);
          row[4 * j4 + 2] = __float_as_uint(v2);
          row[4 * j4 + 3] = __float_as_uint(v3);
        } else if (act == 1) {  // ReLU folded into the rounding conversion
          row[l * 16 + 2 * j4 + 0] = round_pack2_relu<T>(v0, v1);
          row[l * 16 + 2 * j4 + 1] = round_pack2_relu<T>(v2, v3);
        } else {
          if (act) {
            v0 = apply_activation(v0, act);
            v1 = apply_activation(v1, act);
            v2 = apply_activation(v2, act);
            v3 = apply_activation(v3, act);
          }
          row[l * 16 + 2 * j4 + 0] = round_pack2<T>(v0, v1);
          row[l * 16 + 2 * j4 + 1] = round_pack2<T>(v2, v3);
        }
      }
    }
    // the accumulator columns of the next group travel while this one is stored
    if (g + 1 < groups) {
#pragma unroll
      for (int l = 0; l < kLoads; ++l) tmem_ld_32x32b_x32(t_row + (g + 1) * kPerStore + l * 32, raw[l]);
    }
    if constexpr (!RES) {
      if (lane == 0) {
        // the box staged NBUF groups ago has left this buffer
        if constexpr (NBUF == 2) bulk_wait_group_read1(); else bulk_wait_group_read0();
      }
    }
    __syncwarp();
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      // 128-byte swizzle: the 16-byte pieces of neighbouring rows land in different banks
      *reinterpret_cast<uint4*>(buf + lane * 128 + ((q ^ (lane & 7)) << 4)) =
          make_uint4(row[4 * q], row[4 * q + 1], row[4 * q + 2], row[4 * q + 3]);
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      // committed even when empty so that "all but the latest group" always means the other buffer
      if (st_rows > 0) tma_store_3d(st_rows >= 32 ? tm_full : tm_tail, buf, n0 + g * kPerStore, st_row, st_img);
      bulk_commit_group();
    }
  }
}

// Contributor side of reduction splitting: this warp's 32 rows x WC raw fp32 accumulator columns go to the
// CTA's slot (piece pc0 onwards, row `row`) instead of through the epilogue.
template <int WC>
__device__ __forceinline__ void epilogue_dump_partial(uint32_t t_row, float* slot, int pc0, int row) {
  uint32_t raw[2][32];
  tmem_ld_32x32b_x32(t_row, raw[0]);
#pragma unroll
  for (int c = 0; c < WC / 32; ++c) {
    tmem_ld_wait();
    if (c + 1 < WC / 32) tmem_ld_32x32b_x32(t_row + (c + 1) * 32, raw[(c + 1) & 1]);
#pragma unroll
    for (int j = 0; j < 8; ++j) sk_store_piece(slot, pc0 + c * 8 + j, row, &raw[c & 1][4 * j]);
  }
}

}  // namespace fdnn
