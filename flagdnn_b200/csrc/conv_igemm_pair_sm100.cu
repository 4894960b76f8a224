// Implicit-GEMM convolution forward on CTA pairs (tcgen05 cta_group::2).
//
// Same arithmetic and GEMM view as conv_igemm_sm100.cu; what changes is who
// holds what.  Two CTAs of a cluster share one 256-row x 256-channel output
// tile: each CTA copies its own 128 activation rows and its own 128 filter rows
// (half of the tile's output channels), and the leader CTA issues MMAs of shape
// 256 x 256 x 16 that read both CTAs' shared memory and accumulate into both
// CTAs' tensor memory (128 rows each).  Per SM that is 32 KB of operands per
// reduction step instead of 48 KB, which is what the single-CTA kernel is short
// of on compute-bound layers.  Nothing is broadcast: every copy is issued by,
// and lands in, the CTA that uses it.
//
//   warp 0 (each CTA)  producer: waits for its own "stage empty" barrier, copies
//                      A (im2col mode) and its half of B, crediting the bytes to
//                      the LEADER's "stage full" barrier
//   warp 1 (leader)    issuer: waits "stage full", issues the pair MMAs, commits
//                      to both CTAs' "stage empty" barriers, and after the last
//                      step to both CTAs' "accumulator full" barriers
//   warps 4..11 (each) epilogue on the CTA's own 128 rows (two warps per tensor-
//                      memory lane quarter, half of the columns each), then an
//                      arrive on the leader's "accumulator empty" barrier
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "conv_convert.cuh"
#include "conv_epilogue.cuh"
#include "conv_internal.h"
#include "sm100_ptx.cuh"
#include "stream_k.cuh"

namespace fdnn {
namespace {

constexpr int kRows = 128;           // output rows per CTA (pair tile: 256)
constexpr int kPairN = 256;          // output channels per pair tile
constexpr int kHalfN = 128;          // filter rows staged per CTA
constexpr int kRowB = 128;           // bytes per swizzled shared-memory row
constexpr int kKB = 64;              // 16-bit reduction elements per stage
constexpr int kABytes = kRows * kRowB;
constexpr int kBBytes = kHalfN * kRowB;
constexpr int kStageBytes = kABytes + kBBytes;      // 32 KB per CTA per stage
constexpr int kStages = 5;                           // streaming mode: 5 x 32 KB
constexpr int kRingBytes = 184 * 1024;               // operand region (stages, or resident filter + A stages)
constexpr int kMaxStages = 8;                        // barrier slots
constexpr int kMaxResidentSteps = 7;                 // resident filter: at most 7 x 16 KB per CTA
#ifndef FDNN_CONV_BATCH
#define FDNN_CONV_BATCH 4
#endif
constexpr int kConvBatch = FDNN_CONV_BATCH;          // 16-byte pieces a converter thread keeps in flight (fused 3-channel mode)
#ifndef FDNN_PAIR_EPI_WARPS
#define FDNN_PAIR_EPI_WARPS 8
#endif
constexpr int kEpiWarpsPair = FDNN_PAIR_EPI_WARPS;   // 8: two per tensor-memory lane quarter, half the columns each
constexpr int kColSplitPair = kEpiWarpsPair / 4;
constexpr int kWarpCols = kPairN / kColSplitPair;
constexpr int kOutBufs = kEpiWarpsPair == 8 ? 1 : 2; // TMA-store staging buffers per warp (32 KB in all either way)
constexpr int kFirstEpiWarpPair = 4;                 // warp group 0: producer, issuer, two idle warps
constexpr int kThreadsPair = 32 * (kFirstEpiWarpPair + kEpiWarpsPair);
// warp group 0 hands registers to the epilogue warp groups (see conv_igemm_sm100.cu)
#ifndef FDNN_PAIR_REGS_LEAN
#define FDNN_PAIR_REGS_LEAN 128
#endif
#ifndef FDNN_PAIR_REGS_EPI
#define FDNN_PAIR_REGS_EPI 184
#endif
constexpr int kRegsLeanPair = FDNN_PAIR_REGS_LEAN;
constexpr int kRegsEpiloguePair = kEpiWarpsPair == 8 ? FDNN_PAIR_REGS_EPI : 224;
// The warp groups can only re-divide what the launch allocated: 168 registers per thread (64 K registers / 384
// threads, rounded down to a multiple of 8).  A split that adds up to more than that makes the epilogue groups'
// setmaxnreg.inc wait forever for registers that never come, even if it is within the 64 K of the register file.
static_assert(128 * kRegsLeanPair + 32 * kEpiWarpsPair * kRegsEpiloguePair <= kThreadsPair * (65536 / kThreadsPair / 8 * 8),
              "register reallocation exceeds the launch allocation");
constexpr int kOutBytes = kEpiWarpsPair * kOutBufs * 32 * kRowB;
constexpr int kEpiBytes = kEpiWarpsPair * 2 * kWarpCols * int(sizeof(float));
constexpr int kBarBytes = (2 * kMaxStages + 11 + 1 + kEpiWarpsPair) * 8 + 16;   // ... slot words, one residual-box barrier per epilogue warp
constexpr int kSmemPair = kRingBytes + kOutBytes + kEpiBytes + kBarBytes + 1024;
static_assert(kStages * kStageBytes <= kRingBytes, "streaming ring must fit");
constexpr uint32_t kTmemColsPair = 512;              // two 256-column accumulators
static_assert(kSmemPair <= 227 * 1024, "shared memory budget");

template <typename T, bool RES>
__global__ void __launch_bounds__(kThreadsPair, 1)
conv_igemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmY2,
                       const __grid_constant__ CUtensorMap tmR, const __grid_constant__ CUtensorMap tmRbox,
                       const IgemmParams p) {
  constexpr uint32_t kFmt = std::is_same<T, __half>::value ? 0u : 1u;
  constexpr uint32_t kIdesc = make_idesc(kFmt, 2 * kRows, kPairN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // Operand region.  Streaming mode: a ring of (A, B-half) stages.  Resident mode
  // (small reductions, one channel tile): this CTA's half of the whole filter is
  // copied once and stays; the ring then holds activation tiles only.
  const int k_iters = p.R * p.S * p.c_blocks;
  const bool b_resident = p.b_resident != 0;
  uint8_t* b_res = smem;
  // fused 3-channel mode: an image of a scratch slot (the tile's input rows, shifted and zero-padded) is put
  // together here by bulk copies and leaves for global memory in one piece
  const int conv_bytes = p.fused3 ? (p.slot_elems * 2 + 1023) / 1024 * 1024 : 0;
  uint8_t* conv_stage = smem + (b_resident ? k_iters * kBBytes : 0);
  uint8_t* stage_base = conv_stage + conv_bytes;
  const int stage_stride = b_resident ? kABytes : kStageBytes;
  int n_stages = b_resident ? (kRingBytes - k_iters * kBBytes - conv_bytes) / kABytes : kStages;
  if (n_stages > kMaxStages) n_stages = kMaxStages;
  uint8_t* out_stage = smem + kRingBytes;
  float* epi_stage = reinterpret_cast<float*>(out_stage + kOutBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + kOutBytes + kEpiBytes);
  uint64_t* full_bar = bars;                          // used in the leader only
  uint64_t* empty_bar = bars + kMaxStages;            // each CTA's own
  uint64_t* tmem_full = bars + 2 * kMaxStages;        // [2], each CTA's own
  uint64_t* tmem_empty = bars + 2 * kMaxStages + 2;   // [2], used in the leader only
  uint64_t* drain_bar = bars + 2 * kMaxStages + 4;
  uint64_t* bres_bar = bars + 2 * kMaxStages + 5;     // resident filter has landed (leader only)
  uint64_t* raw_full = bars + 2 * kMaxStages + 6;     // [2] fused 3-channel mode: a scratch slot holds a tile's input rows
  uint64_t* raw_empty = bars + 2 * kMaxStages + 8;    // [2] ... and every window copy of the tile that used it has landed
  uint64_t* conv_in = bars + 2 * kMaxStages + 10;     // the input rows of a tile have landed in conv_stage
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 11);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint64_t* res_bar = bars + 2 * kMaxStages + 12;     // [epilogue warps] a residual box has landed in the staging buffer

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();         // 0 = leader
  const uint32_t peer = rank ^ 1u;

  griddep_launch_dependents();  // all CTAs of this grid are resident: the next launch may queue behind them
  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(&full_bar[i], 1);                  // the leader producer's arrive.expect_tx
      mbar_init(&empty_bar[i], 1);                 // one commit from the leader's issuer
    }
    mbar_init(bres_bar, 1);
    mbar_init(&raw_full[0], p.x_unaligned ? 2 : 1);   // converter warps that arrive per tile
    mbar_init(&raw_full[1], p.x_unaligned ? 2 : 1);
    mbar_init(conv_in, 1);
    mbar_init(&raw_empty[0], 1);                   // the leader's issuer
    mbar_init(&raw_empty[1], 1);
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_full[1], 1);
    mbar_init(&tmem_empty[0], 2 * kEpiWarpsPair * 32);  // epilogue threads of both CTAs
    mbar_init(&tmem_empty[1], 2 * kEpiWarpsPair * 32);
    mbar_init(drain_bar, 1);
    if constexpr (RES) {
      for (int i = 0; i < kEpiWarpsPair; ++i) mbar_init(&res_bar[i], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmY);
    if (p.lowc) tma_prefetch_desc(&tmY2);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemColsPair);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  griddep_wait();      // from here on global memory is consumed: the launch before this one must be complete
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_tiles = (p.Kout + kPairN - 1) / kPairN;
  const int m_pairs = (p.m_tiles + 1) / 2;
  const int total_tiles = m_pairs * n_tiles;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int ohw = p.OH * p.OW;
  const bool split = p.stream_k != 0;  // reduction splitting across pairs (stream_k.cuh)

  if (warp < kFirstEpiWarpPair) {
#ifndef FDNN_NO_REG_REALLOC
  warpgroup_reg_dec<kRegsLeanPair>();
#endif
  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0 && !p.skip_copies) {
      uint32_t stage = 0, phase = 0;
      bool alive = true;
      long long prof_wait = 0, prof_issue = 0, prof_iters = 0, prof_t0 = p.prof ? clock64() : 0;
      const uint32_t full0 = map_to_cta(smem_u32(&full_bar[0]), 0);  // the leader's barriers
      if (b_resident && pair_id < total_tiles) {
        // this CTA's 128 filter rows for every reduction step, once (n_tiles == 1 in this mode)
        const uint32_t bres = map_to_cta(smem_u32(bres_bar), 0);
        if (rank == 0) mbar_arrive_expect_tx(bres_bar, uint32_t(2 * k_iters * kBBytes));
        int kit = 0;
        for (int r = 0; r < p.R; ++r)
          for (int s = 0; s < p.S; ++s)
            for (int cb = 0; cb < p.c_blocks; ++cb, ++kit)
              tma_load_3d_pair(b_res + kit * kBBytes, &tmB, bres, cb * kKB, r * p.S + s, int(rank) * kHalfN);
      }
      TileWalk walk;
      walk_init(walk, split, pair_id, num_pairs, total_tiles, k_iters, p.sk_min_frag);
      uint32_t tiles_done = 0;
      while (alive && walk_next(walk)) {
        const int tile = walk.tile;
        const int m_pair = tile / n_tiles;
        const int n_tile = tile - m_pair * n_tiles;
        const int m_tile = 2 * m_pair + int(rank);  // this CTA's 128-row tile (may lie past the end)
        int img, w_base, h_base;
        if (p.lowc) {
          img = m_tile / p.tiles_per_image;
          const int ti = m_tile - img * p.tiles_per_image;
          w_base = 0;
          h_base = ti * p.ohs * p.stride_h - p.pad_top;
        } else {
          const int m0 = m_tile * kRows;
          img = m0 / ohw;
          const int rem = m0 - img * ohw;
          const int oh0 = rem / p.OW;
          const int ow0 = rem - oh0 * p.OW;
          w_base = ow0 * p.stride_w - p.pad_left;
          h_base = oh0 * p.stride_h - p.pad_top;
        }
        if constexpr (RES) {
          // this CTA's 128 x 256 residual values of the tile, asked into L2 a whole main loop before the
          // epilogue reads them (only the pair that finishes the tile reads them)
          if (p.residual != nullptr && !p.lowc && walk.ke == k_iters)
            tma_prefetch_l2_3d(&tmR, n_tile * kPairN, m_tile * kRows, 0);
        }
        const uint32_t a_tx = p.lowc ? uint32_t(p.a_tx_bytes) : uint32_t(kABytes);
        const uint32_t pair_tx = 2 * (a_tx + (b_resident ? 0u : uint32_t(kBBytes)));
        const int b_row0 = n_tile * kPairN + int(rank) * kHalfN;
        if (p.fused3) {
          // the converter warps have written this tile's input rows into slot (tiles_done & 1)
          const uint32_t b_ = tiles_done & 1u;
          if (!mbar_wait_bounded(&raw_full[b_], (tiles_done >> 1) & 1u, abort_flag, p.status, kIncidentProducerWait,
                                 p.wait_limit)) {
            alive = false;
            break;
          }
          img = int(blockIdx.x) * 2 + int(b_);     // the slot is the window map's outermost coordinate
          h_base = 0;
        }
        ++tiles_done;
        // reduction step kit = (r * S + s) * c_blocks + cb
        int tap = walk.kb / p.c_blocks;
        int cb = walk.kb - tap * p.c_blocks;
        int r = tap / p.S;
        int s_ = tap - r * p.S;
        auto copy_steps = [&](auto prof_tag) {
          constexpr bool kProf = decltype(prof_tag)::value;
          for (int kit = walk.kb; kit < walk.ke; ++kit) {
            long long pt0 = 0, pt1 = 0;
            if constexpr (kProf) pt0 = clock64();
            if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, p.status,
                                   kIncidentProducerWait, p.wait_limit)) {
              alive = false;
              break;
            }
            if constexpr (kProf) {
              pt1 = clock64();
              prof_wait += pt1 - pt0;
              ++prof_iters;
            }
            uint8_t* st = stage_base + stage * stage_stride;
            if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], pair_tx);
            const uint32_t bar = full0 + stage * 8;
            const int c0 = cb * kKB;
            if (p.lowc) {
              tma_load_4d_pair(st, &tmA, bar, 0, 0, h_base + r * p.dil_h, img);
            } else {
              tma_load_im2col_4d_pair(st, &tmA, bar, c0, w_base, h_base, img, static_cast<uint16_t>(s_ * p.dil_w),
                                      static_cast<uint16_t>(r * p.dil_h));
            }
            if (!b_resident) tma_load_3d_pair(st + kABytes, &tmB, bar, c0, r * p.S + s_, b_row0);
            if constexpr (kProf) prof_issue += clock64() - pt1;
            if (++stage == uint32_t(n_stages)) {
              stage = 0;
              phase ^= 1u;
            }
            if (++cb == p.c_blocks) {
              cb = 0;
              if (++s_ == p.S) {
                s_ = 0;
                ++r;
              }
            }
          }
        };
        if (p.prof == nullptr) copy_steps(std::false_type{}); else copy_steps(std::true_type{});
      }
      if (p.prof && blockIdx.x == 0) {
        p.prof[0] = prof_wait; p.prof[1] = prof_issue; p.prof[2] = clock64() - prof_t0; p.prof[3] = prof_iters;
      }
      if (!alive || *abort_flag) {
        // After an incident: give copies already issued time to land.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------- issuer (leader only)
    if (rank == 0 && lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t tcount = 0;
      bool alive = true;
      long long prof_wfull = 0, prof_wtmem = 0, prof_t0 = p.prof ? clock64() : 0;
      if (b_resident && pair_id < total_tiles) {
        alive = mbar_wait_bounded(bres_bar, 0u, abort_flag, p.status, kIncidentMmaWaitFull, p.wait_limit);
      }
      const uint32_t empty_own = smem_u32(&empty_bar[0]);
      const uint32_t empty_peer = map_to_cta(empty_own, 1);
      const uint32_t tfull_own = smem_u32(&tmem_full[0]);
      const uint32_t tfull_peer = map_to_cta(tfull_own, 1);
      const uint32_t raw_empty_peer = map_to_cta(smem_u32(&raw_empty[0]), 1);
      const int k16 = p.k16_per_step;  // 16-element reduction slices per step that hold data (4, or 3)
      TileWalk walk;
      walk_init(walk, split, pair_id, num_pairs, total_tiles, k_iters, p.sk_min_frag);
      for (; alive && walk_next(walk); ++tcount) {
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
        const uint32_t d_tmem = tmem_base + buf * kPairN;
        // The reduction loop is the hot path of every layer and is sensitive to anything beside the wait, the
        // MMAs and the commits (a conditional barrier arrive in it cost 17 % on the 3x3 256-channel layer):
        // it exists once with four MMAs per step and once with a runtime count for the 3-channel mode.
        auto reduce = [&](auto four_tag, auto prof_tag) {
          constexpr bool kFour = decltype(four_tag)::value;
          constexpr bool kProf = decltype(prof_tag)::value;
          for (int kit = walk.kb; kit < walk.ke; ++kit) {
            long long mt1 = 0;
            if constexpr (kProf) mt1 = clock64();
            if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, p.status, kIncidentMmaWaitFull, p.wait_limit)) {
              alive = false;
              break;
            }
            if constexpr (kProf) prof_wfull += clock64() - mt1;
            tc_fence_after();
            const uint32_t st = smem_u32(stage_base + stage * stage_stride);
            const uint32_t bt = b_resident ? smem_u32(b_res + kit * kBBytes) : st + kABytes;
            if constexpr (kFour) {
#pragma unroll
              for (int k = 0; k < kKB / 16; ++k) {
                const uint64_t a = make_sw128_kmajor_desc(st + k * 32);
                const uint64_t b = make_sw128_kmajor_desc(bt + k * 32);
                mma_f16_pair(d_tmem, a, b, kIdesc, (kit > walk.kb || k > 0) ? 1u : 0u);
              }
            } else {
              for (int k = 0; k < k16; ++k) {
                const uint64_t a = make_sw128_kmajor_desc(st + k * 32);
                const uint64_t b = make_sw128_kmajor_desc(bt + k * 32);
                mma_f16_pair(d_tmem, a, b, kIdesc, (kit > walk.kb || k > 0) ? 1u : 0u);
              }
            }
            tc_commit_pair(empty_own + stage * 8);
            tc_commit_pair(empty_peer + stage * 8);
            if (++stage == uint32_t(n_stages)) {
              stage = 0;
              phase ^= 1u;
            }
          }
        };
        if (k16 != kKB / 16) {
          reduce(std::false_type{}, std::false_type{});
        } else if (p.prof == nullptr) {
          reduce(std::true_type{}, std::false_type{});
        } else {
          reduce(std::true_type{}, std::true_type{});   // cycle counters of the role (development aid)
        }
        if (alive) {
          tc_commit_pair(tfull_own + buf * 8);
          tc_commit_pair(tfull_peer + buf * 8);
          if (p.fused3) {
            // every window copy of this tile has landed in both CTAs (all of its "stage full" barriers were
            // passed above): their converters may reuse the scratch slot
            mbar_arrive(&raw_empty[tcount & 1u]);
            mbar_arrive_cluster(raw_empty_peer + (tcount & 1u) * 8);
          }
        }
      }
      if (p.prof && blockIdx.x == 0) {
        p.prof[4] = prof_wfull; p.prof[5] = prof_wtmem; p.prof[6] = clock64() - prof_t0; p.prof[7] = tcount;
      }
      if (!alive || *abort_flag) {
        volatile uint32_t never = 0;
        tc_commit_pair(smem_u32(drain_bar));
        mbar_wait_bounded(drain_bar, 0u, &never, p.status, kIncidentDrainWait, kWaitLimitCycles / 16);
      }
    }
  }
  else if (p.fused3 && !p.skip_copies && !p.x_unaligned) {
    // ---------------------------------------------- converter (warp 2), fused 3-channel mode
    // A tile reads raw_rows input rows of its image.  The image of a scratch slot is assembled in conv_stage:
    // row hr = lead_chunks zero pieces (the left padding, rounded so that windows start on 16 bytes), the input
    // row, zeros to the end; rows above or below the image are all zeros.  Input rows arrive by bulk copies
    // (nothing passes through registers), the finished image leaves by one bulk copy to the CTA's slot in
    // global memory, where it stays in L2 for the window copies of the producer.
    if (warp == 2) {
      const int row_bytes = p.row_chunks * 16;
      const int lead_bytes = p.lead_chunks * 16;
      int data_bytes = p.x_row_chunks * 16;
      if (data_bytes > row_bytes - lead_bytes) data_bytes = row_bytes - lead_bytes;
      const int slot_bytes = p.slot_elems * 2;
      for (int i = lane * 16; i < conv_bytes; i += 32 * 16)
        *reinterpret_cast<uint4*>(conv_stage + i) = make_uint4(0u, 0u, 0u, 0u);   // the padding stays zero for good
      fence_proxy_async_smem();
      __syncwarp();
      const uint8_t* xb = static_cast<const uint8_t*>(p.x3);
      uint32_t use = 0, in_phase = 0;
      TileWalk walk;
      walk_init(walk, false, pair_id, num_pairs, total_tiles, k_iters, 0);
      while (walk_next(walk)) {
        const int m_tile = 2 * (walk.tile / n_tiles) + int(rank);
        const int img = m_tile / p.tiles_per_image;
        const int ti = m_tile - img * p.tiles_per_image;
        const int h0 = ti * p.ohs * p.stride_h - p.pad_top;
        const bool img_ok = m_tile < p.m_tiles;   // the pair's second tile may lie past the last image
        const uint32_t b_ = use & 1u;
        // rows outside the image: zeros over whatever an earlier tile left there
        int rows_in = 0;
        for (int hr = 0; hr < p.raw_rows; ++hr) {
          const int h = h0 + hr;
          if (img_ok && h >= 0 && h < p.x_h) {
            ++rows_in;
          } else {
            for (int i = lane * 16; i < data_bytes; i += 32 * 16)
              *reinterpret_cast<uint4*>(conv_stage + hr * row_bytes + lead_bytes + i) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        bool ok = true;
        if (lane == 0) {
          if (rows_in > 0) {
            mbar_arrive_expect_tx(conv_in, uint32_t(rows_in) * uint32_t(data_bytes));
            for (int hr = 0; hr < p.raw_rows; ++hr) {
              const int h = h0 + hr;
              if (h >= 0 && h < p.x_h)
                bulk_load_1d(conv_stage + hr * row_bytes + lead_bytes,
                             xb + ((long long)img * p.x_h + h) * (p.x_row_chunks * 16), uint32_t(data_bytes), conv_in);
            }
          }
          // the slot in global memory is free once every window copy of the tile that used it has landed
          ok = mbar_wait_bounded(&raw_empty[b_], ((use >> 1) & 1u) ^ 1u, abort_flag, p.status, kIncidentProducerWait,
                                 p.wait_limit);
          if (rows_in > 0) {
            ok = mbar_wait_bounded(conv_in, in_phase, abort_flag, p.status, kIncidentProducerWait, p.wait_limit) && ok;
            in_phase ^= 1u;
          }
          if (ok) {
            bulk_store_1d(static_cast<uint8_t*>(p.scratch3) + (long long)(int(blockIdx.x) * 2 + int(b_)) * slot_bytes,
                          conv_stage, uint32_t(slot_bytes));
            bulk_commit_group();
            bulk_wait_group0();   // written, and conv_stage may be filled again
            mbar_arrive(&raw_full[b_]);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        ++use;
      }
    }
  }
  else if (p.fused3 && !p.skip_copies) {
    // ---------------------------------------------- converters (warps 2 and 3), fused 3-channel mode, input not
    // 16-byte aligned: the same slot image written piece by piece from registers
    // A tile reads raw_rows input rows of its image.  Each goes into the CTA's scratch slot as row_chunks
    // 16-byte pieces: lead_chunks zero pieces (the left padding, rounded so that windows start on 16 bytes),
    // the row's x_row_chunks pieces, zeros to the end; rows above or below the image are all zeros.
    const int t = (warp - 2) * 32 + lane;
    const int per_tile = p.raw_rows * p.row_chunks;
    const uint4* x16 = static_cast<const uint4*>(p.x3);
    const uint16_t* x2 = static_cast<const uint16_t*>(p.x3);
    uint32_t use = 0;
    bool alive = true;
    TileWalk walk;
    walk_init(walk, false, pair_id, num_pairs, total_tiles, k_iters, 0);
    while (alive && walk_next(walk)) {
      const int m_tile = 2 * (walk.tile / n_tiles) + int(rank);
      const int img = m_tile / p.tiles_per_image;
      const int ti = m_tile - img * p.tiles_per_image;
      const int h0 = ti * p.ohs * p.stride_h - p.pad_top;
      const uint32_t b_ = use & 1u;
      bool ok = mbar_wait_bounded(&raw_empty[b_], ((use >> 1) & 1u) ^ 1u, abort_flag, p.status, kIncidentProducerWait,
                                  p.wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.scratch3) +
                                            (long long)(int(blockIdx.x) * 2 + int(b_)) * p.slot_elems);
      const bool img_ok = m_tile < p.m_tiles;   // the pair's second tile may lie past the last image
      for (int base = t; base < per_tile; base += 64 * kConvBatch) {
        uint4 v[kConvBatch];
#pragma unroll
        for (int u = 0; u < kConvBatch; ++u) {
          const int idx = base + u * 64;
          v[u] = make_uint4(0u, 0u, 0u, 0u);
          if (idx < per_tile) {
            const int hr = idx / p.row_chunks;
            const int j = idx - hr * p.row_chunks - p.lead_chunks;
            const int h = h0 + hr;
            if (img_ok && h >= 0 && h < p.x_h && j >= 0 && j < p.x_row_chunks) {
              const long long piece = ((long long)img * p.x_h + h) * p.x_row_chunks + j;
              if (!p.x_unaligned) {
                v[u] = __ldg(x16 + piece);
              } else {
                const uint16_t* e = x2 + piece * 8;
                v[u].x = e[0] | (uint32_t(e[1]) << 16);
                v[u].y = e[2] | (uint32_t(e[3]) << 16);
                v[u].z = e[4] | (uint32_t(e[5]) << 16);
                v[u].w = e[6] | (uint32_t(e[7]) << 16);
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kConvBatch; ++u) {
          const int idx = base + u * 64;
          if (idx < per_tile) dst[idx] = v[u];
        }
      }
      __threadfence();
      fence_proxy_async_all();   // the window copies (async proxy) read what these threads wrote
      __syncwarp();
      if (lane == 0) mbar_arrive(&raw_full[b_]);
      ++use;
    }
  }
  } else {
#ifndef FDNN_NO_REG_REALLOC
  warpgroup_reg_inc<kRegsEpiloguePair>();
#endif
  {
    // ------------------------------------------------------------ epilogue
    const int ew = warp & 3;
    const int chalf = (warp - kFirstEpiWarpPair) >> 2;  // which share of the tile's columns this warp drains
    float* s_scale = epi_stage + (warp - kFirstEpiWarpPair) * 2 * kWarpCols;
    float* s_bias = s_scale + kWarpCols;
    const T* g_bias = static_cast<const T*>(p.bias);
    const T* g_scale = static_cast<const T*>(p.scale);
    const T* g_res = (RES && !p.lowc) ? static_cast<const T*>(p.residual) : nullptr;
    uint8_t* my_out = out_stage + (warp - kFirstEpiWarpPair) * kOutBufs * 32 * kRowB;
    const uint32_t tempty_leader = map_to_cta(smem_u32(&tmem_empty[0]), 0);
    uint32_t tcount = 0;
    uint32_t store_seq = 0;
    uint32_t res_phases = 0;
    ResidualFetch rf;
    rf.tm = g_res != nullptr ? &tmRbox : nullptr;
    rf.bars = res_bar + (warp - kFirstEpiWarpPair);
    rf.phases = &res_phases;
    rf.abort_flag = abort_flag;
    rf.status_word = p.status;
    rf.wait_limit = p.wait_limit;
    int staged_n_tile = -1;
    long long prof_ewait = 0, prof_t0 = p.prof ? clock64() : 0;
    TileWalk walk;
    walk_init(walk, split, pair_id, num_pairs, total_tiles, k_iters, p.sk_min_frag);
    const int my_warp = warp - kFirstEpiWarpPair;
    const int sk_row = ew * 32 + lane;                   // this lane's row in the CTA's slot
    const int sk_pc0 = chalf * (kWarpCols / 4);          // this warp's first 16-byte piece of a slot row
    for (; walk_next(walk); ++tcount) {
      const int tile = walk.tile;
      const int m_pair = tile / n_tiles;
      const int n_tile = tile - m_pair * n_tiles;
      const int n0 = n_tile * kPairN + chalf * kWarpCols;  // first column this warp owns
      const uint32_t buf = tcount & 1u;
      const uint32_t bphase = (tcount >> 1) & 1u;
      const bool finishes = walk.ke == k_iters;            // this pair computes the tile's last reduction steps
      if (finishes && n_tile != staged_n_tile) {
        __syncwarp();
        for (int j = lane; j < kWarpCols; j += 32) {
          const int col = n0 + j;
          s_scale[j] = (g_scale != nullptr && col < p.Kout) ? to_f32<T>(g_scale[col % p.k_real]) : 1.0f;
          s_bias[j] = (g_bias != nullptr && col < p.Kout) ? to_f32<T>(g_bias[col % p.k_real]) : 0.0f;
        }
        __syncwarp();
        staged_n_tile = n_tile;
      }
      const int m_tile = 2 * m_pair + int(rank);
      const long long et0 = p.prof ? clock64() : 0;
      bool ok = mbar_wait_bounded(&tmem_full[buf], bphase, abort_flag, p.status, kIncidentEpilogueWait, p.wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (p.prof) prof_ewait += clock64() - et0;
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(ew * 32) << 16) + buf * kPairN + chalf * kWarpCols;
      if (!finishes) {
        // contributor: the tile's first reduction steps; the raw sums go to this CTA's slot
        float* slot = p.sk_slots + (long long)blockIdx.x * kSkSlotFloats;
        epilogue_dump_partial<kWarpCols>(t_row, slot, sk_pc0, sk_row);
        __threadfence();
        __syncwarp();
        if (lane == 0) sk_flag_release(p.sk_flags + blockIdx.x * kSkFlagsPerCta + my_warp, 1u);
        tc_fence_before();
        mbar_arrive_cluster(tempty_leader + buf * 8);
        continue;
      }
      int sk_count = 0;
      if (walk.kb > 0) {
        // owner of a split tile: pairs pair_id-1, pair_id-2, ... hold its earlier steps, each as the first
        // thing it computed; wait for this warp's counterpart in each of them
        const long long L = (long long)total_tiles * k_iters;
        const long long tile_base = (long long)tile * k_iters;
        for (int q = pair_id - 1; q >= 0 && ok; --q) {
          ++sk_count;
          const uint32_t* flag = p.sk_flags + (2 * q + int(rank)) * kSkFlagsPerCta + my_warp;
          if (lane == 0) {
            const long long t0 = clock64();
            uint32_t spins = 0;
            while (sk_flag_acquire(flag) == 0u) {
              if ((++spins & 0x3f) == 0 && (*abort_flag || clock64() - t0 > p.wait_limit)) {
                atomicCAS(p.status, 0u, uint32_t(kIncidentPartialWait));
                *abort_flag = 1;
                ok = false;
                break;
              }
            }
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (sk_bound(q, L, num_pairs, k_iters, p.sk_min_frag) <= tile_base) break;  // q reaches the tile's first step
        }
        if (!ok) break;
      }
      int st_row, st_img, st_rows;
      if (p.lowc) {
        st_img = m_tile / p.tiles_per_image;
        st_row = (m_tile - st_img * p.tiles_per_image) * p.rows_per_tile + ew * 32;
        st_rows = p.rows_per_tile - ew * 32;
      } else {
        st_img = 0;
        st_row = m_tile * kRows + ew * 32;
        st_rows = 32;
      }
      const float* sk_slot0 = sk_count > 0 ? p.sk_slots + (long long)(2 * (pair_id - 1) + int(rank)) * kSkSlotFloats : nullptr;
      epilogue_store_tile<T, kWarpCols, RES, kOutBufs>(t_row, n0, p.Kout, p.act, s_scale, s_bias, my_out, lane, &tmY, &tmY2,
                                     st_row, st_img, st_rows, store_seq, &rf, g_scale != nullptr,
                                     sk_slot0, sk_count, 2LL * kSkSlotFloats, sk_row, sk_pc0);
      if (sk_count > 0) {
        // the slots are read: lower the flags for the next launch
        __syncwarp();
        if (lane == 0)
          for (int c = 0; c < sk_count; ++c)
            p.sk_flags[(2 * (pair_id - 1 - c) + int(rank)) * kSkFlagsPerCta + my_warp] = 0u;
      }
      tc_fence_before();
      mbar_arrive_cluster(tempty_leader + buf * 8);
    }
    if (lane == 0) bulk_wait_group0();
    if (p.prof && blockIdx.x == 0 && threadIdx.x == 32 * kFirstEpiWarpPair) {  // first epilogue warp of the first leader
      p.prof[8] = prof_ewait; p.prof[9] = clock64() - prof_t0;
    }
  }
  }

  // Neither CTA may retire while its partner can still signal its barriers or
  // the leader's MMAs can still read its shared memory.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemColsPair);
  }
}

template <typename T>
cudaError_t launch_pair_t(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY,
                          const CUtensorMap& tmY2, const CUtensorMap& tmR, const CUtensorMap& tmRbox, const IgemmParams& p,
                          int grid,
                          cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kThreadsPair, 1, 1);
  cfg.dynamicSmemBytes = kSmemPair;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // set-up may overlap the previous launch's tail
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = launch_overlap_enabled() ? 2 : 1;
  if (p.residual != nullptr) return cudaLaunchKernelEx(&cfg, conv_igemm_pair_kernel<T, true>, tmA, tmB, tmY, tmY2, tmR, tmRbox, p);
  return cudaLaunchKernelEx(&cfg, conv_igemm_pair_kernel<T, false>, tmA, tmB, tmY, tmY2, tmR, tmRbox, p);
}

}  // namespace

cudaError_t igemm_pair_prepare_device() {
  cudaError_t e = cudaFuncSetAttribute(conv_igemm_pair_kernel<__half, false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemPair);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(conv_igemm_pair_kernel<__half, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemPair);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(conv_igemm_pair_kernel<__nv_bfloat16, false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemPair);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(conv_igemm_pair_kernel<__nv_bfloat16, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemPair);
  return e;
}

int igemm_pair_smem_bytes() { return kSmemPair; }
int igemm_pair_stages() { return kStages; }
int igemm_pair_threads() { return kThreadsPair; }
int igemm_pair_max_resident_steps() { return kMaxResidentSteps; }

cudaError_t launch_igemm_pair(int dtype, const CUtensorMap& tmA, const CUtensorMap& tmB,
                              const CUtensorMap& tmY, const CUtensorMap& tmY2, const CUtensorMap& tmR,
                              const CUtensorMap& tmRbox,
                              const IgemmParams& p, int grid, cudaStream_t stream) {
  if (dtype == FDNN_F16) return launch_pair_t<__half>(tmA, tmB, tmY, tmY2, tmR, tmRbox, p, grid, stream);
  if (dtype == FDNN_BF16) return launch_pair_t<__nv_bfloat16>(tmA, tmB, tmY, tmY2, tmR, tmRbox, p, grid, stream);
  return cudaErrorInvalidValue;
}

}  // namespace fdnn
