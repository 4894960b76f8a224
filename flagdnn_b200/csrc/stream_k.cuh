// Reduction splitting across CTA pairs ("stream-K") for the implicit-GEMM kernel on pairs.
//
// With whole tiles per pair, T tiles on P pairs take ceil(T / P) rounds: 196 tiles of the 3x3 256-channel
// layer on 74 pairs are 2.65 rounds of work done in 3.  Here the pairs share the linear space of
// (tile, reduction step) instead: pair p owns steps [bound(p), bound(p+1)) of T * K and walks them from
// the top down.  A tile cut by a boundary is computed in pieces:
//   * the pair whose range ENDS inside the tile holds its first reduction steps.  That piece is the first
//     thing the pair computes; its epilogue warps write the raw fp32 accumulators to the pair's slot in
//     global memory and raise one flag per warp ("contributor");
//   * the pair whose range STARTS inside the tile holds its last steps and reaches them last.  Its epilogue
//     warps wait for the flags of the pairs below it, add their slots in a fixed order (p-1, p-2, ...) to the
//     accumulator and run the ordinary epilogue ("owner").
// Every wait therefore targets work that a lower-numbered pair does first, without waiting for anything, so
// pairs that are resident never wait for pairs that are not (CTAs start in index order), and the wait is
// bounded like every other one.  Results do not depend on timing: the assignment and the order of the
// additions are functions of the problem and the grid alone.
#pragma once
#include <stdint.h>

namespace fdnn {

// First linear step of pair p's range (p in [0, P]); L = T * K steps in all.
__device__ __forceinline__ long long sk_bound(int p, long long L, int P, int K, int min_frag) {
  if (p <= 0) return 0;
  if (p >= P) return L;
  const long long raw = L * p / P;
  long long t = raw / K;
  int rem = int(raw - t * K);
  if (rem < min_frag) {
    rem = 0;
  } else if (rem > K - min_frag) {
    rem = 0;
    ++t;
  }
  return t * K + rem;
}

// The sequence of (tile, first step, end step) a pair computes; identical in every role of both CTAs.
struct TileWalk {
  int K;           // reduction steps per tile
  int tile, kb, ke;
  // whole-tile mode
  int next_tile, stride, total;
  // split mode
  bool split;
  long long lo, hi;
};

__device__ __forceinline__ void walk_init(TileWalk& w, bool split, int pair_id, int num_pairs, int total_tiles,
                                          int k_iters, int min_frag) {
  w.K = k_iters;
  w.split = split;
  w.next_tile = pair_id;
  w.stride = num_pairs;
  w.total = total_tiles;
  w.lo = w.hi = 0;
  if (split) {
    const long long L = (long long)total_tiles * k_iters;
    w.lo = sk_bound(pair_id, L, num_pairs, k_iters, min_frag);
    w.hi = sk_bound(pair_id + 1, L, num_pairs, k_iters, min_frag);
  }
}

__device__ __forceinline__ bool walk_next(TileWalk& w) {
  if (!w.split) {
    if (w.next_tile >= w.total) return false;
    w.tile = w.next_tile;
    w.next_tile += w.stride;
    w.kb = 0;
    w.ke = w.K;
    return true;
  }
  if (w.hi <= w.lo) return false;
  const long long t = (w.hi - 1) / w.K;
  const long long base = t * w.K;
  const long long b = w.lo > base ? w.lo : base;
  w.tile = int(t);
  w.kb = int(b - base);
  w.ke = int(w.hi - base);
  w.hi = b;
  return true;
}

// Slot layout of one CTA (128 rows x 256 fp32 columns): 16-byte piece pc (four columns) of row r sits at
// float4 index pc * 128 + r, so that the 32 lanes of a warp (32 consecutive rows) write 512 contiguous bytes.
constexpr int kSkSlotFloats = 128 * 256;
constexpr int kSkFlagsPerCta = 8;

__device__ __forceinline__ void sk_store_piece(float* slot, int pc, int row, const uint32_t* v) {
  float4 q = make_float4(__uint_as_float(v[0]), __uint_as_float(v[1]), __uint_as_float(v[2]), __uint_as_float(v[3]));
  __stcg(reinterpret_cast<float4*>(slot) + pc * 128 + row, q);
}
__device__ __forceinline__ float4 sk_load_piece(const float* slot, int pc, int row) {
  return __ldcg(reinterpret_cast<const float4*>(slot) + pc * 128 + row);  // L2: another SM wrote it
}

__device__ __forceinline__ void sk_flag_release(uint32_t* flag, uint32_t value) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}
__device__ __forceinline__ uint32_t sk_flag_acquire(const uint32_t* flag) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
  return v;
}

}  // namespace fdnn
