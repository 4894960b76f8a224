// Implicit-GEMM convolution forward for sm_100a.
//
//   y[m, k] = act( scale[k] * sum_{r,s,c} x[n, oh*sh + r*dh - pt, ow*sw + s*dw - pl, c] * w[k, r, s, c] + bias[k] )
//
// with m = (n, oh, ow) flattened.  One persistent CTA per SM walks 128-row
// output tiles.  Three roles, one pipeline:
//   warp 0      TMA producer: per (r, s, channel block) one im2col-mode copy of
//               128 pixels x 128 bytes of activations (padding arrives as the
//               copy's zero fill) into a ring of shared-memory stages guarded
//               by full/empty mbarriers;
//               and one tiled copy of the filter slice (optionally issued by a
//               second producer warp, FDNN_PRODUCERS=2);
//   warp 1      MMA issuer: tcgen05.mma from shared-memory descriptors into one
//               of two fp32 accumulators in tensor memory; tcgen05.commit frees
//               the stage and, after the last reduction step, publishes the
//               accumulator;
//   warps 4..11 epilogue: tcgen05.ld of the finished accumulator, per-channel
//               scale, bias, ReLU, one rounding to the output type, store —
//               while the issuer already fills the other accumulator.  Two
//               warps share each tensor-memory lane quarter and take half of
//               the tile's columns each: a short-reduction layer (1x1, few
//               input channels) is bound by how fast tiles drain, and one warp
//               per quarter leaves its chain of load, convert, stage and store
//               latencies exposed.
// fp32 tensors run the same loop on TF32-split operands (high and low halves
// staged side by side): lo*hi + hi*lo + hi*hi per reduction step.
//
// The arithmetic restated here is that of the reference's fused kernel
// (src/flag_dnn/graph/kernels/fused_conv.py:249-310): fp32 accumulate, bias
// added in fp32, max(., 0), single cast at the store.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "conv_convert.cuh"
#include "conv_epilogue.cuh"
#include "conv_internal.h"
#include "sm100_ptx.cuh"

namespace fdnn {

namespace {

constexpr int kBM = 128;            // output rows per tile (= tcgen05 M, = TMEM lanes)
constexpr int kRowBytes = 128;      // one swizzled shared-memory row
#ifndef FDNN_EPI_WARPS
#define FDNN_EPI_WARPS 8
#endif
constexpr int kEpiWarps = FDNN_EPI_WARPS;  // 8: two per tensor-memory lane quarter (4: one)
#ifndef FDNN_PRODUCERS
#define FDNN_PRODUCERS 1
#endif
// 2: activation and filter copies come from different warps.  Measured on B200: no faster on any layer
// shape (a reduction step is bound by shared-memory bandwidth, operand reads of the MMAs plus the copies'
// fills, not by the issuing thread), so one producer is the default.
constexpr int kProducers = FDNN_PRODUCERS;
constexpr int kFilterProducerWarp = 2;  // in the first warp group, beside the producer and the issuer
// Warp group 0 holds the producer, the issuer (and the optional filter producer); the epilogue warps are
// whole warp groups after it, so that group 0 can hand most of its registers to them: the kernel starts
// with 168 registers per thread (64 K / 384), group 0 keeps kRegsLean and each epilogue thread gets
// kRegsEpilogue — the epilogue holds two 32-column accumulator slices, a finished row and, with a
// residual, a 32 x 128-byte box in flight, which does not fit in 168 without spilling.
constexpr int kFirstEpiWarp = 4;
constexpr int kThreads = 32 * (kFirstEpiWarp + kEpiWarps);
constexpr int kRegsLean = 104;
constexpr int kRegsEpilogue = kEpiWarps == 8 ? 200 : 232;  // 128 * 104 + 256 * 200 = 384 * 168
// the warp groups re-divide the launch allocation (168 registers x 384 threads); more than that and the
// epilogue groups' setmaxnreg.inc would wait forever
static_assert(128 * kRegsLean + 32 * kEpiWarps * kRegsEpilogue <= kThreads * (65536 / kThreads / 8 * 8),
              "register reallocation exceeds the launch allocation");

template <typename T, int BN>
struct TileCfg {
  static constexpr bool kSplit = std::is_same<T, float>::value;
  static constexpr int kKB = kRowBytes / int(sizeof(T));  // reduction elements per stage
  static constexpr int kUK = 32 / int(sizeof(T));         // reduction elements per MMA
  static constexpr int kABytes = kBM * kRowBytes;
  static constexpr int kBBytes = BN * kRowBytes;
  static constexpr int kStageBytes = (kSplit ? 2 : 1) * (kABytes + kBBytes);
  static constexpr int kTmemCols = 2 * BN;  // two accumulators; 128, 256 or 512
  // per-warp output staging (32 rows x 128 bytes, swizzled, for the TMA store),
  // per-warp scale and bias staging, then barriers and bookkeeping words
  static constexpr int kOutCols = kRowBytes / int(sizeof(T));  // output channels per TMA store
  // a tile's columns are split between the two warps of a lane quarter when each half is two stores
  // or more (narrower tiles keep one warp per quarter and spend the shared memory on pipeline stages)
  static constexpr int kColSplit = (kEpiWarps == 8 && BN / kOutCols >= 4) ? 2 : 1;
  static constexpr int kWarpCols = BN / kColSplit;             // columns one epilogue warp drains
  static constexpr int kActiveEpiWarps = 4 * kColSplit;
  static constexpr int kOutBytes = kActiveEpiWarps * 2 * 32 * kRowBytes;  // two 4 KB buffers per warp
  static constexpr int kEpiBytes = kActiveEpiWarps * 2 * kWarpCols * int(sizeof(float));
  // operand ring: what is left of the 227 KB; 3 x 48 KB for the widest 16-bit tile
  static constexpr int kMaxStages = 16;
  static constexpr int kRingBudget = 227 * 1024 - kOutBytes - kEpiBytes - (2 * kMaxStages + 8) * 8 - 1024;
  static constexpr int kStages = kRingBudget / kStageBytes < kMaxStages ? kRingBudget / kStageBytes : kMaxStages;
  static constexpr int kBarBytes = (2 * kStages + 4 + 1 + 1 + 16) * 8 + 16;   // ring, accumulators, drain, slot words, residual boxes
  static constexpr int kSmemBytes = kStages * kStageBytes + kOutBytes + kEpiBytes + kBarBytes + 1024;
  static_assert(kStages >= 2, "pipeline needs at least two stages");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

// 32 finished values of one output pixel -> 32 consecutive channels of y.
template <typename T>
__device__ __forceinline__ void store32_contig(T* dst, const float (&v)[32]) {
  if constexpr (std::is_same<T, float>::value) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 q = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      reinterpret_cast<float4*>(dst)[i] = q;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 q;
      q.x = pack2(from_f32<T>(v[8 * i + 0]), from_f32<T>(v[8 * i + 1]));
      q.y = pack2(from_f32<T>(v[8 * i + 2]), from_f32<T>(v[8 * i + 3]));
      q.z = pack2(from_f32<T>(v[8 * i + 4]), from_f32<T>(v[8 * i + 5]));
      q.w = pack2(from_f32<T>(v[8 * i + 6]), from_f32<T>(v[8 * i + 7]));
      reinterpret_cast<uint4*>(dst)[i] = q;
    }
  }
}

template <typename T, int BN, bool RES>
__global__ void __launch_bounds__(kThreads, 1)
conv_igemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
                  const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmB2,
                  const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmR,
                  const __grid_constant__ CUtensorMap tmRbox, const IgemmParams p) {
  using Cfg = TileCfg<T, BN>;
  constexpr int kStages = Cfg::kStages;
  constexpr uint32_t kFmt = std::is_same<T, __half>::value ? 0u : (std::is_same<T, __nv_bfloat16>::value ? 1u : 2u);
  constexpr uint32_t kIdesc = make_idesc(kFmt, kBM, BN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint8_t* out_stage = smem + kStages * Cfg::kStageBytes;  // 1024-byte aligned: stages are multiples of 1 KB
  float* epi_stage = reinterpret_cast<float*>(out_stage + Cfg::kOutBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + Cfg::kOutBytes + Cfg::kEpiBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tmem_full = bars + 2 * kStages;       // [2]
  uint64_t* tmem_empty = bars + 2 * kStages + 2;  // [2]
  uint64_t* drain_bar = bars + 2 * kStages + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 5);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint64_t* res_bar = bars + 2 * kStages + 6;     // [8 epilogue warps][2 staging buffers]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  griddep_launch_dependents();  // all CTAs of this grid are resident: the next launch may queue behind them
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], kProducers);
      mbar_init(&empty_bar[i], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_full[1], 1);
    mbar_init(&tmem_empty[0], Cfg::kActiveEpiWarps * 32);
    mbar_init(&tmem_empty[1], Cfg::kActiveEpiWarps * 32);
    mbar_init(drain_bar, 1);
    if constexpr (RES) {
      for (int i = 0; i < 16; ++i) mbar_init(&res_bar[i], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (p.tma_store) tma_prefetch_desc(&tmY);
    if constexpr (Cfg::kSplit) {
      tma_prefetch_desc(&tmA2);
      tma_prefetch_desc(&tmB2);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  griddep_wait();  // from here on global memory is consumed: the launch before this one must be complete

  const int total_tiles = p.m_tiles * p.n_tiles;
  const int k_iters = p.R * p.S * p.c_blocks;
  const int ohw = p.OH * p.OW;

  // One elected thread issues copies; with two producers the activation and the filter copies of a
  // stage come from different warps and each credits its own bytes to the stage's "full" barrier.
  auto produce = [&](const bool do_a, const bool do_b, const bool record) {
    uint32_t it = 0;
    bool alive = true;
    long long prof_wait = 0, prof_issue = 0, prof_t0 = p.prof ? clock64() : 0;
    for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x) {
      const int m_tile = tile / p.n_tiles;
      const int n_tile = tile - m_tile * p.n_tiles;
      int img, w_base, h_base;
      if (p.lowc) {
        img = m_tile / p.tiles_per_image;
        const int ti = m_tile - img * p.tiles_per_image;
        w_base = 0;
        h_base = ti * p.ohs * p.stride_h - p.pad_top;
      } else {
        const int m0 = m_tile * kBM;
        img = m0 / ohw;
        const int rem = m0 - img * ohw;
        const int oh0 = rem / p.OW;
        const int ow0 = rem - oh0 * p.OW;
        w_base = ow0 * p.stride_w - p.pad_left;
        h_base = oh0 * p.stride_h - p.pad_top;
      }
      if constexpr (RES) {
        // the epilogue of this tile will read its 128 x BN residual values a whole main loop from now:
        // ask for them to be brought into L2 so that its loads are short and HBM reads are requested early
        if (do_a && p.residual != nullptr && p.tma_store && !p.lowc) tma_prefetch_l2_3d(&tmR, n_tile * BN, m_tile * kBM, 0);
      }
      const uint32_t a_tx = (Cfg::kSplit ? 2u : 1u) * (p.lowc ? uint32_t(p.a_tx_bytes) : uint32_t(Cfg::kABytes));
      const uint32_t b_tx = (Cfg::kSplit ? 2u : 1u) * uint32_t(Cfg::kBBytes);
      const uint32_t my_tx = (do_a ? a_tx : 0u) + (do_b ? b_tx : 0u);
      for (int r = 0; r < p.R && alive; ++r) {
        for (int s = 0; s < p.S && alive; ++s) {
          const uint16_t off_w = static_cast<uint16_t>(s * p.dil_w);
          const uint16_t off_h = static_cast<uint16_t>(r * p.dil_h);
          const int tap = r * p.S + s;
          for (int cb = 0; cb < p.c_blocks; ++cb, ++it) {
            const uint32_t stage = it % kStages;
            const uint32_t phase = (it / kStages) & 1u;
            const long long pt0 = p.prof ? clock64() : 0;
            if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, p.status,
                                   kIncidentProducerWait, p.wait_limit)) {
              alive = false;
              break;
            }
            const long long pt1 = p.prof ? clock64() : 0;
            prof_wait += pt1 - pt0;
            uint8_t* st = stage_base + stage * Cfg::kStageBytes;
            mbar_arrive_expect_tx(&full_bar[stage], my_tx);
            const int c0 = cb * Cfg::kKB;
            if (do_a) {
              if (p.lowc) {
                // window copy: (64 elements, all quads of a row, `ohs` rows at the conv stride, image)
                tma_load_4d(st, &tmA, &full_bar[stage], 0, 0, h_base + r * p.dil_h, img);
              } else {
                tma_load_im2col_4d(st, &tmA, &full_bar[stage], c0, w_base, h_base, img, off_w, off_h);
              }
              if constexpr (Cfg::kSplit) {
                tma_load_im2col_4d(st + Cfg::kABytes, &tmA2, &full_bar[stage], c0, w_base, h_base,
                                   img, off_w, off_h);
              }
            }
            if (do_b) {
              if constexpr (Cfg::kSplit) {
                tma_load_3d(st + 2 * Cfg::kABytes, &tmB, &full_bar[stage], c0, tap, n_tile * BN);
                tma_load_3d(st + 2 * Cfg::kABytes + Cfg::kBBytes, &tmB2, &full_bar[stage], c0, tap,
                            n_tile * BN);
              } else {
                tma_load_3d(st + Cfg::kABytes, &tmB, &full_bar[stage], c0, tap, n_tile * BN);
              }
            }
            if (p.prof) prof_issue += clock64() - pt1;
          }
        }
      }
    }
    if (record && p.prof && blockIdx.x == 0) {
      p.prof[0] = prof_wait; p.prof[1] = prof_issue; p.prof[2] = clock64() - prof_t0; p.prof[3] = it;
    }
    if (!alive || *abort_flag) {
      // Teardown after an incident: let the copies already issued land before
      // the CTA gives its shared memory back.
      const uint32_t first = it > uint32_t(kStages) ? it - kStages : 0u;
      for (uint32_t j = first; j < it; ++j) {
        volatile uint32_t never = 0;
        mbar_wait_bounded(&full_bar[j % kStages], (j / kStages) & 1u, &never, p.status,
                          kIncidentDrainWait, kWaitLimitCycles / 16);
      }
    }
  };

  if (warp < kFirstEpiWarp) {
#ifndef FDNN_NO_REG_REALLOC
  warpgroup_reg_dec<kRegsLean>();
#endif
  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0 && !p.skip_copies) produce(true, kProducers == 1, true);
  } else if (kProducers == 2 && warp == kFilterProducerWarp) {
    // ---------------------------------------------- producer of the filter copies
    if (lane == 0 && !p.skip_copies) produce(false, true, false);
  } else if (warp == 1) {
    // -------------------------------------------------------------- issuer
    if (lane == 0) {
      uint32_t it = 0;
      uint32_t tcount = 0;
      bool alive = true;
      long long prof_wfull = 0, prof_wtmem = 0, prof_t0 = p.prof ? clock64() : 0;
      for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x, ++tcount) {
        const uint32_t buf = tcount & 1u;
        const uint32_t bphase = (tcount >> 1) & 1u;
        const long long mt0 = p.prof ? clock64() : 0;
        if (!mbar_wait_bounded(&tmem_empty[buf], bphase ^ 1u, abort_flag, p.status,
                               kIncidentMmaWaitTmem, p.wait_limit)) {
          alive = false;
          break;
        }
        if (p.prof) prof_wtmem += clock64() - mt0;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        // the reduction loop holds the wait, the MMAs and the commit and nothing else: the issuing thread is on
        // the critical path of every step (cycle counters are compiled into a second copy of the loop)
        auto reduce = [&](auto prof_tag) {
          constexpr bool kProf = decltype(prof_tag)::value;
          for (int kit = 0; kit < k_iters; ++kit, ++it) {
            const uint32_t stage = it % kStages;
            const uint32_t phase = (it / kStages) & 1u;
            long long mt1 = 0;
            if constexpr (kProf) mt1 = clock64();
            if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, p.status,
                                   kIncidentMmaWaitFull, p.wait_limit)) {
              alive = false;
              break;
            }
            if constexpr (kProf) prof_wfull += clock64() - mt1;
            tc_fence_after();
            const uint32_t st = smem_u32(stage_base + stage * Cfg::kStageBytes);
#pragma unroll
            for (int k = 0; k < Cfg::kKB / Cfg::kUK; ++k) {
              const uint32_t acc = (kit > 0 || k > 0) ? 1u : 0u;
              if constexpr (Cfg::kSplit) {
                const uint64_t a_hi = make_sw128_kmajor_desc(st + k * 32);
                const uint64_t a_lo = make_sw128_kmajor_desc(st + Cfg::kABytes + k * 32);
                const uint64_t b_hi = make_sw128_kmajor_desc(st + 2 * Cfg::kABytes + k * 32);
                const uint64_t b_lo =
                    make_sw128_kmajor_desc(st + 2 * Cfg::kABytes + Cfg::kBBytes + k * 32);
                mma_tf32(d_tmem, a_lo, b_hi, kIdesc, acc);
                mma_tf32(d_tmem, a_hi, b_lo, kIdesc, 1u);
                mma_tf32(d_tmem, a_hi, b_hi, kIdesc, 1u);
              } else {
                const uint64_t a = make_sw128_kmajor_desc(st + k * 32);
                const uint64_t b = make_sw128_kmajor_desc(st + Cfg::kABytes + k * 32);
                mma_f16(d_tmem, a, b, kIdesc, acc);
              }
            }
            tc_commit(&empty_bar[stage]);
          }
        };
        if (p.prof == nullptr) reduce(std::false_type{}); else reduce(std::true_type{});
        if (alive) tc_commit(&tmem_full[buf]);
      }
      if (p.prof && blockIdx.x == 0) {
        p.prof[4] = prof_wfull; p.prof[5] = prof_wtmem; p.prof[6] = clock64() - prof_t0; p.prof[7] = tcount;
      }
      if (!alive || *abort_flag) {
        // Make sure no MMA is still writing tensor memory before it is freed.
        volatile uint32_t never = 0;
        tc_commit(drain_bar);
        mbar_wait_bounded(drain_bar, 0u, &never, p.status, kIncidentDrainWait, kWaitLimitCycles / 16);
      }
    }
  }
  } else {
#ifndef FDNN_NO_REG_REALLOC
  warpgroup_reg_inc<kRegsEpilogue>();
#endif
  if (warp - kFirstEpiWarp < Cfg::kActiveEpiWarps) {
    // ------------------------------------------------------------ epilogue
    constexpr int WC = Cfg::kWarpCols;
    const int ew = warp & 3;           // tensor-memory lane quarter this warp may read
    const int chalf = (warp - kFirstEpiWarp) >> 2;  // which share of the tile's columns it drains
    float* s_scale = epi_stage + (warp - kFirstEpiWarp) * 2 * WC;
    float* s_bias = s_scale + WC;
    const T* g_bias = static_cast<const T*>(p.bias);
    const T* g_scale = static_cast<const T*>(p.scale);
    T* y = static_cast<T*>(p.y);
    const T* g_res = (RES && !p.lowc) ? static_cast<const T*>(p.residual) : nullptr;
    uint32_t tcount = 0;
    uint32_t store_seq = 0;
    uint32_t res_phases = 0;
    ResidualFetch rf;
    rf.tm = (g_res != nullptr && p.tma_store) ? &tmRbox : nullptr;
    rf.bars = res_bar + (warp - kFirstEpiWarp) * 2;
    rf.phases = &res_phases;
    rf.abort_flag = abort_flag;
    rf.status_word = p.status;
    rf.wait_limit = p.wait_limit;
    int staged_n_tile = -1;
    long long prof_ewait = 0, prof_t0 = p.prof ? clock64() : 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++tcount) {
      const int m_tile = tile / p.n_tiles;
      const int n_tile = tile - m_tile * p.n_tiles;
      const int n0 = n_tile * BN + chalf * WC;  // first column this warp owns
      const uint32_t buf = tcount & 1u;
      const uint32_t bphase = (tcount >> 1) & 1u;

      if (n_tile != staged_n_tile) {
        __syncwarp();
        for (int j = lane; j < WC; j += 32) {
          const int col = n0 + j;
          s_scale[j] = (g_scale != nullptr && col < p.Kout) ? to_f32<T>(g_scale[col % p.k_real]) : 1.0f;
          s_bias[j] = (g_bias != nullptr && col < p.Kout) ? to_f32<T>(g_bias[col % p.k_real]) : 0.0f;
        }
        __syncwarp();
        staged_n_tile = n_tile;
      }

      const int m = m_tile * kBM + ew * 32 + lane;
      const bool row_ok = m < p.M;
      long long y_off = 0;
      if (row_ok) {
        const int img = m / ohw;
        const int rem = m - img * ohw;
        const int oh = rem / p.OW;
        const int ow = rem - oh * p.OW;
        y_off = img * p.y_sn + oh * p.y_sh + ow * p.y_sw;
      }
      const long long et0 = p.prof ? clock64() : 0;
      bool ok = mbar_wait_bounded(&tmem_full[buf], bphase, abort_flag, p.status, kIncidentEpilogueWait, p.wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (p.prof) prof_ewait += clock64() - et0;
      if (!ok) break;
      tc_fence_after();

      const uint32_t t_row = tmem_base + (uint32_t(ew * 32) << 16) + buf * BN + chalf * WC;
      // Where this warp's 32 rows go in y seen as (channel, row, image): the whole
      // output is one "image" outside low-channel mode.
      int st_row, st_img, st_rows;
      if (p.lowc) {
        st_img = m_tile / p.tiles_per_image;
        st_row = (m_tile - st_img * p.tiles_per_image) * p.rows_per_tile + ew * 32;
        st_rows = p.rows_per_tile - ew * 32;
      } else {
        st_img = 0;
        st_row = m_tile * kBM + ew * 32;
        st_rows = 32;
      }
      if (p.tma_store) {
        // a tile's last warp may own fewer than 32 valid rows: tmA2 then holds a second
        // output map whose box is exactly that short (low-channel mode, 16-bit only)
        epilogue_store_tile<T, WC, RES>(t_row, n0, p.Kout, p.act, s_scale, s_bias,
                                   out_stage + (warp - kFirstEpiWarp) * 2 * 32 * kRowBytes, lane, &tmY, &tmA2, st_row,
                                   st_img, st_rows, store_seq, &rf, g_scale != nullptr);
      } else {
#pragma unroll 1
      for (int chunk = 0; chunk < WC / 32; ++chunk) {
        const int col0 = n0 + chunk * 32;
        if (col0 >= p.Kout) break;  // uniform across the warp
        uint32_t raw[32];
        tmem_ld_32x32b_x32(t_row + chunk * 32, raw);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float a = __uint_as_float(raw[j]);
          a = fmaf(a, s_scale[chunk * 32 + j], s_bias[chunk * 32 + j]);
          if (RES && g_res != nullptr && row_ok && col0 + j < p.Kout)
            a += to_f32<T>(g_res[y_off + (long long)(col0 + j) * p.y_sk]);
          if (p.act) a = apply_activation(a, p.act);
          v[j] = a;
        }
        if (row_ok && p.out_f32) {
          // 16-bit operands, float32 result: the finished values are stored as they are
          float* yf = static_cast<float*>(p.y);
          if (p.vec_store && col0 + 32 <= p.Kout) {
            store32_contig<float>(yf + y_off + col0, v);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col0 + j < p.Kout) yf[y_off + (long long)(col0 + j) * p.y_sk] = v[j];
            }
          }
        } else if (row_ok) {
          if (p.vec_store && col0 + 32 <= p.Kout) {
            store32_contig<T>(y + y_off + col0, v);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col0 + j < p.Kout) y[y_off + (long long)(col0 + j) * p.y_sk] = from_f32<T>(v[j]);
            }
          }
        }
      }
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[buf]);
    }
    if (p.tma_store && lane == 0) bulk_wait_group0();  // stores must be done before the CTA retires
    if (p.prof && blockIdx.x == 0 && threadIdx.x == 32 * kFirstEpiWarp) {  // first epilogue warp
      p.prof[8] = prof_ewait; p.prof[9] = clock64() - prof_t0;
    }
  }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <typename T, int BN>
cudaError_t launch_one(const CUtensorMap& tmA, const CUtensorMap& tmA2, const CUtensorMap& tmB,
                       const CUtensorMap& tmB2, const CUtensorMap& tmY, const CUtensorMap& tmR, const CUtensorMap& tmRbox,
                       const IgemmParams& p,
                       int grid, cudaStream_t stream) {
  using Cfg = TileCfg<T, BN>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // set-up may overlap the previous launch's tail
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = launch_overlap_enabled() ? 1 : 0;
  if (p.residual != nullptr)
    return cudaLaunchKernelEx(&cfg, conv_igemm_kernel<T, BN, true>, tmA, tmA2, tmB, tmB2, tmY, tmR, tmRbox, p);
  return cudaLaunchKernelEx(&cfg, conv_igemm_kernel<T, BN, false>, tmA, tmA2, tmB, tmB2, tmY, tmR, tmRbox, p);
}

template <typename T, int BN>
cudaError_t prepare_one() {
  using Cfg = TileCfg<T, BN>;
  cudaError_t e = cudaFuncSetAttribute(conv_igemm_kernel<T, BN, false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(conv_igemm_kernel<T, BN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              Cfg::kSmemBytes);
}

}  // namespace

cudaError_t igemm_prepare_device() {
  cudaError_t e;
#define FDNN_PREP(T, BN)                 \
  e = prepare_one<T, BN>();              \
  if (e != cudaSuccess) return e;
  FDNN_PREP(__half, 64) FDNN_PREP(__half, 128) FDNN_PREP(__half, 256)
  FDNN_PREP(__nv_bfloat16, 64) FDNN_PREP(__nv_bfloat16, 128) FDNN_PREP(__nv_bfloat16, 256)
  FDNN_PREP(float, 64) FDNN_PREP(float, 128)
#undef FDNN_PREP
  return cudaSuccess;
}

int igemm_smem_bytes(int dtype, int tile_n) {
  if (dtype == FDNN_F32) return tile_n == 64 ? TileCfg<float, 64>::kSmemBytes : TileCfg<float, 128>::kSmemBytes;
  if (tile_n == 64) return TileCfg<__half, 64>::kSmemBytes;
  if (tile_n == 128) return TileCfg<__half, 128>::kSmemBytes;
  return TileCfg<__half, 256>::kSmemBytes;
}

int igemm_threads() { return kThreads; }

int igemm_stages(int dtype, int tile_n) {
  if (dtype == FDNN_F32) return tile_n == 64 ? TileCfg<float, 64>::kStages : TileCfg<float, 128>::kStages;
  if (tile_n == 64) return TileCfg<__half, 64>::kStages;
  if (tile_n == 128) return TileCfg<__half, 128>::kStages;
  return TileCfg<__half, 256>::kStages;
}

cudaError_t launch_igemm(int dtype, int tile_n, const CUtensorMap& tmA, const CUtensorMap& tmA2,
                         const CUtensorMap& tmB, const CUtensorMap& tmB2, const CUtensorMap& tmY,
                         const CUtensorMap& tmR, const CUtensorMap& tmRbox, const IgemmParams& p, int grid,
                         cudaStream_t stream) {
#define FDNN_GO(T, BN) return launch_one<T, BN>(tmA, tmA2, tmB, tmB2, tmY, tmR, tmRbox, p, grid, stream);
  if (dtype == FDNN_F16) {
    if (tile_n == 64) FDNN_GO(__half, 64)
    if (tile_n == 128) FDNN_GO(__half, 128)
    if (tile_n == 256) FDNN_GO(__half, 256)
  } else if (dtype == FDNN_BF16) {
    if (tile_n == 64) FDNN_GO(__nv_bfloat16, 64)
    if (tile_n == 128) FDNN_GO(__nv_bfloat16, 128)
    if (tile_n == 256) FDNN_GO(__nv_bfloat16, 256)
  } else if (dtype == FDNN_F32) {
    if (tile_n == 64) FDNN_GO(float, 64)
    if (tile_n == 128) FDNN_GO(float, 128)
  }
#undef FDNN_GO
  return cudaErrorInvalidValue;
}

}  // namespace fdnn
