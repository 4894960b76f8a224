// Internal declarations shared by the C-ABI front end (conv_api.cu) and the
// kernel translation units.  Nothing here is exported.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flagdnn_b200.h"

namespace fdnn {

// Per-device incident word written by bounded waits (see sm100_ptx.cuh).
uint32_t* device_status_word();  // device address for the current device, or nullptr on error

// Geometry handed to the implicit-GEMM kernel.  GEMM view: rows m = (n, oh, ow)
// flattened, columns = output channels, reduction = (r, s, c) with c innermost.
struct IgemmParams {
  int M;                 // N * OH * OW
  int Kout;              // output channels
  int OH, OW;
  int stride_h, stride_w, pad_top, pad_left, dil_h, dil_w;
  int R, S;
  int c_blocks;          // ceil(Cpad / channels per 128-byte row)
  int m_tiles, n_tiles;
  long long y_sn, y_sk, y_sh, y_sw;  // element strides of y
  long long y_row;       // dense NHWC y (tma_store): elements between consecutive output pixels
  const void* bias;      // [Kout] in the tensor dtype, or nullptr
  const void* scale;     // [Kout] in the tensor dtype, or nullptr
  void* y;
  const void* residual;  // tensor with y's dtype and strides added before the activation, or nullptr
  int act;               // FDNN_ACT_* applied after scale, bias and residual
  int vec_store;         // 1: y is channel-contiguous and 16-byte aligned per pixel
  int tma_store;         // 1: y is dense NHWC; the epilogue writes it through the tmY tensor map
  int out_f32;           // 1: y is float32 although the operands are 16-bit (per-thread store path only)
  // Low-channel mode (C <= 4): one GEMM row is a quad of 4 output pixels of one
  // image row, its reduction operand a 16-pixel window of the repacked input;
  // a tile is `ohs` output rows x OW/4 quads and never crosses an image.
  int lowc;              // 1: low-channel mode
  int rows_per_tile;     // valid GEMM rows per tile (128 outside low-channel mode)
  int tiles_per_image;   // low-channel mode: ceil(OH / ohs)
  int ohs;               // low-channel mode: output rows per tile
  int a_tx_bytes;        // bytes one activation copy delivers (rows_per_tile * 128 in low-channel mode)
  int b_resident;        // pair kernel: the filter half stays in shared memory for the whole launch
  // Low-channel mode on a dense 3-channel NHWC input (the stem), pair kernel only: no relayout pass.  Two warps
  // of each CTA copy the tile's input rows, shifted to a 16-byte boundary and zero-padded left and right,
  // into a per-CTA scratch slot in global memory (it stays in L2); the window copies then read that slot.
  int fused3;            // 1: this mode
  const void* x3;        // the input tensor (element type = tensor dtype)
  void* scratch3;        // 2 slots per CTA of slot_elems elements each
  int x_h;               // input height
  int x_row_chunks;      // 16-byte pieces per input row (W * 3 / 8)
  int x_unaligned;       // 1: x is not 16-byte aligned (pieces are read element by element)
  int raw_rows;          // input rows a tile reads: (ohs - 1) * stride_h + (R - 1) * dil_h + 1
  int row_chunks;        // 16-byte pieces per scratch row
  int lead_chunks;       // zero pieces stored before an input row's first piece
  int slot_elems;        // elements per scratch slot
  int k16_per_step;      // MMAs (16 reduction elements each) per reduction step: 4, or 3 in this mode
  int k_real;            // length of bias / scale (GEMM column j uses entry j % k_real)
  uint32_t* status;
  long long* prof;       // optional: 16 cycle counters written by CTA 0 (nullptr = off)
  // Reduction splitting on CTA pairs ("stream-K"): the pairs share the linear space (tile, reduction step)
  // evenly instead of whole tiles; a tile cut by a range boundary is finished by the pair that holds its last
  // reduction steps, which adds the fp32 partial sums the others left in sk_slots (see stream_k.cuh).
  int stream_k;          // 1: split as above (pair kernel only), 0: whole tiles, round-robin
  int sk_min_frag;       // range boundaries closer than this many reduction steps to a tile edge snap to it
  float* sk_slots;       // one 128 x 256 fp32 slot per CTA
  uint32_t* sk_flags;    // 8 words per CTA (one per epilogue warp), zero between launches
  long long wait_limit;  // SM clocks after which a wait on a barrier gives up (see fdnn_debug_set_wait_limit)
  int skip_copies;       // test aid: the copy-issuing role does nothing, so the first wait for data runs out
};

// Whether the tensor-core kernels are launched with programmatic stream serialization (their set-up
// overlaps the tail of the launch before them on the stream).  On unless the environment variable
// FLAGDNN_B200_LAUNCH_OVERLAP is "0" when the library makes its first launch.
bool launch_overlap_enabled();

// Default for IgemmParams::wait_limit: about two seconds of SM clocks.
long long default_wait_limit_cycles();

// Launchers (defined in conv_igemm_sm100.cu).  `dtype` is FDNN_F16/BF16/F32.
// tmA2 / tmB2 are the low-half operands of the split-TF32 path (ignored for
// 16-bit types); tmY is the output map used when p.tma_store is set; tmR covers the residual tensor
// with one tile-sized box (L2 prefetch; read only when p.residual is set and y is dense NHWC), tmRbox covers it
// exactly as tmY covers y (32-row x 128-byte boxes the epilogue warps copy into their staging buffers).  Returns a
// cudaError_t from the launch.
cudaError_t launch_igemm(int dtype, int tile_n, const CUtensorMap& tmA, const CUtensorMap& tmA2,
                         const CUtensorMap& tmB, const CUtensorMap& tmB2, const CUtensorMap& tmY,
                         const CUtensorMap& tmR, const CUtensorMap& tmRbox, const IgemmParams& p, int grid,
                         cudaStream_t stream);
// Dynamic shared memory and pipeline depth of a tile configuration.
int igemm_smem_bytes(int dtype, int tile_n);
int igemm_stages(int dtype, int tile_n);
int igemm_threads();       // threads per CTA of the single-CTA kernel
// One-time opt-in to large dynamic shared memory for every instantiation.
cudaError_t igemm_prepare_device();

// CTA-pair variant (conv_igemm_pair_sm100.cu): 16-bit types, 256 x 256 pair
// tiles, TMA-store epilogue only (p.tma_store must be set).  `grid` must be even.
cudaError_t launch_igemm_pair(int dtype, const CUtensorMap& tmA, const CUtensorMap& tmB,
                              const CUtensorMap& tmY, const CUtensorMap& tmY2, const CUtensorMap& tmR,
                              const CUtensorMap& tmRbox, const IgemmParams& p, int grid, cudaStream_t stream);
cudaError_t igemm_pair_prepare_device();
int igemm_pair_smem_bytes();
int igemm_pair_stages();
int igemm_pair_threads();
int igemm_pair_max_resident_steps();  // reductions this short (and one channel tile) keep the filter resident

// Direct convolution on CUDA cores (conv_direct.cu): any dtype, groups, strides.
struct DirectParams {
  int N, C, H, W, K, R, S, OH, OW;
  int stride_h, stride_w, pad_top, pad_left, dil_h, dil_w, groups;
  long long x_s[4], w_s[4], y_s[4];
  const void* x;
  const void* w;
  const void* bias;
  const void* scale;
  const void* residual;  // same dtype and strides as y, or nullptr
  void* y;
  int act;  // FDNN_ACT_*
};
cudaError_t launch_direct(int dtype, const DirectParams& p, cudaStream_t stream);
// Depthwise layers (groups == C == K) in f16 / bf16 / f32 (conv_depthwise.cu): `depthwise_kind` answers 0 when
// the problem is not one of its cases (the direct kernel then runs), 1 for the channels-last kernel (16 bytes
// of channels per thread), 2 for the kernel that gives every (image, channel) plane a block, 3 / 4 / 5 for the
// NCHW kernel that reads rows as 16- / 8- / 4-byte vectors.
int depthwise_kind(int dtype, const DirectParams& p);
cudaError_t launch_depthwise(int dtype, const DirectParams& p, int kind, cudaStream_t stream);

// Pooling (pool.cu): element strides of x and y in (n, c, h, w) order; idx (max pooling only) may be null.
struct PoolParams {
  int N, C, H, W, OH, OW;
  int kh, kw, sh, sw, ph, pw, dh, dw;
  long long x_s[4], y_s[4];
  const void* x;
  void* y;
  long long* idx;
};
cudaError_t launch_max_pool2d(int dtype, const PoolParams& p, cudaStream_t stream);
cudaError_t launch_adaptive_avg_pool2d(int dtype, const PoolParams& p, cudaStream_t stream);

// Relayout kernels (conv_repack.cu).
// x[N,C,H,W] (any strides) -> dense NHWC with C padded to c_pad (zeros).  For
// f32 two planes are written: TF32-rounded high halves at dst, the rounded
// remainders at dst + plane_elems.
cudaError_t launch_repack_x(int dtype, const void* x, const long long x_s[4], int N, int C, int H,
                            int W, int c_pad, void* dst, long long plane_elems,
                            cudaStream_t stream);
// Low-channel relayouts (C <= 4, 16-bit types):
// x -> [N][H][w_pad][4]: `pad_left` zero pixels, the image row, zeros up to w_pad; channel 4 is zero.
cudaError_t launch_repack_x_lowc(int dtype, const void* x, const long long x_s[4], int N, int C, int H,
                                 int W, int pad_left, int w_pad, void* dst, cudaStream_t stream);
// w -> [4*K][R][64]: row (q, k) holds filter k shifted to the q-th output pixel of a quad: with `chans`
// stored channels per pixel (4, or 3 for the fused 3-channel mode), element
// shift_elems + chans * (stride_w * q + t) + c of tap row r is w[k][c][r][t]; everything else is zero.
// `shift_elems` = elements stored before the quad's first input pixel.
cudaError_t launch_pack_w_lowc(int dtype, const void* w, const long long w_s[4], int K, int C, int R,
                               int S, int stride_w, int chans, int shift_elems, void* dst, cudaStream_t stream);
// Pixel-grouped filter: w -> [q*K][R][S + (q-1)*stride_w][c_pad]; row (g, k) holds filter k
// shifted by g*stride_w taps (zero where the g-th pixel of the group does not reach).
cudaError_t launch_pack_w_grouped(int dtype, const void* w, const long long w_s[4], int K, int C, int R,
                                  int S, int stride_w, int q, int c_pad, void* dst, cudaStream_t stream);
// w[K,C,R,S] (any strides) -> dense [K,R,S,c_pad]; f32 split like x.
// A grouped filter as the dense channels-last [K][R][S][C] filter of the same convolution (zeros outside each
// filter's own group of input channels).
cudaError_t launch_densify_w(int dtype, const void* w, const long long w_s[4], int K, int C, int R, int S, int groups,
                             void* dense, cudaStream_t stream);
cudaError_t launch_pack_w(int dtype, const void* w, const long long w_s[4], int K, int C, int R,
                          int S, int c_pad, void* dst, long long plane_elems, cudaStream_t stream);

}  // namespace fdnn
