/*
 * flagdnn_b200 — C ABI of the B200 (sm_100a) convolution forward path.
 *
 * This is the boundary a FlagDNN maintainer binds to replace the Triton
 * launches of the conv2d hot path.  Plain pointers and sizes only: no torch,
 * no C++ types.  Every entry point returns an fdnn_status code; nothing
 * aborts, traps or throws.  All device pointers are caller-owned; the library
 * allocates no device memory (fdnn_conv2d_query tells the caller how much
 * workspace and packed-filter storage to provide).
 *
 * Tensor conventions follow the reference: logical shapes are always
 * x[N,C,H,W], w[K,C/groups,R,S], bias[K], y[N,K,OH,OW]; the physical layout
 * (NCHW, NHWC/channels_last, or any strided view) is carried by element
 * strides in that logical order, as torch reports them.
 */
#ifndef FLAGDNN_B200_H_
#define FLAGDNN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FDNN_ABI_VERSION 2

/* Status codes.  The Python shim maps BAD_PARAM / CUDA_ERROR / DEVICE_TIMEOUT /
 * WORKSPACE_TOO_SMALL to RuntimeError and NOT_SUPPORTED / ARCH_MISMATCH to
 * NotImplementedError, the two exception types the reference raises
 * (src/flag_dnn/ops/conv2d.py:99-135, 3592-3595;
 *  src/flag_dnn/graph/kernels/fused_conv.py:73-90). */
typedef enum fdnn_status {
  FDNN_OK = 0,
  FDNN_BAD_PARAM = 1,
  FDNN_NOT_SUPPORTED = 2,
  FDNN_ARCH_MISMATCH = 3,
  FDNN_WORKSPACE_TOO_SMALL = 4,
  FDNN_CUDA_ERROR = 5,
  FDNN_DEVICE_TIMEOUT = 6
} fdnn_status;

/* dtype ids, same numbering as _dtype_id in src/flag_dnn/ops/conv2d.py:138-147 */
#define FDNN_F16 0
#define FDNN_BF16 1
#define FDNN_F32 2
#define FDNN_F64 3

/* algorithm selector */
#define FDNN_ALGO_AUTO 0
#define FDNN_ALGO_DIRECT 1 /* CUDA-core direct convolution (any dtype, groups) */
#define FDNN_ALGO_IGEMM 2  /* tcgen05 implicit GEMM, one CTA per tile (f16/bf16, f32 via 3xTF32) */
#define FDNN_ALGO_IGEMM_PAIR 3 /* tcgen05 implicit GEMM on CTA pairs (f16/bf16, dense NHWC y) */
/* OR-ed into fdnn_conv_desc.algo: the plan may split reductions across CTA pairs (see FDNN_STREAMK_FLAG_BYTES).
 * Off by default: measured on B200, the layers it applies to are bound by L2 -> SM operand traffic, which the
 * split does not change, and it came out 1-3 % slower than whole tiles on the 3x3 256-channel layer. */
#define FDNN_ALGO_FLAG_STREAM_K 0x100
/* OR-ed into fdnn_conv_desc.algo: x, w, bias and scale are f16 / bf16 as desc->dtype says, but y is float32
 * (y_strides in float elements): the fp32 accumulators are stored after scale, bias and activation without the
 * rounding to 16 bits.  What the reference's mm offers as out_dtype=float32 (src/flag_dnn/ops/mm.py:336).
 * Tensor-core path on one CTA per tile only; no residual. */
#define FDNN_ALGO_FLAG_OUT_F32 0x200
/* OR-ed into fdnn_conv_desc.algo, for tuning runs: fix the width of the single-CTA kernel's tiles to 64 / 128 /
 * 256 output channels instead of the planner's choice (fp32 tiles stop at 128), and keep the planner from
 * grouping output pixels of narrow layers.  The reference fixes its launch configurations per shape from a
 * tuned table (src/flag_dnn/utils/libentry.py:499-579, tune_configs.yaml:1326-1466); here the planner decides,
 * `python -m flagdnn_b200.tune` measures every alternative beside its choice through these flags. */
#define FDNN_ALGO_FLAG_TILE_N_64 0x400
#define FDNN_ALGO_FLAG_TILE_N_128 0x800
#define FDNN_ALGO_FLAG_TILE_N_256 0xC00
#define FDNN_ALGO_FLAG_TILE_N_MASK 0xC00
#define FDNN_ALGO_FLAG_NO_PIXEL_GROUP 0x1000

/* epilogue activation */
#define FDNN_ACT_NONE 0
#define FDNN_ACT_RELU 1
#define FDNN_ACT_GELU 2      /* 0.5 x (1 + erf(x / sqrt 2)), torch's default */
#define FDNN_ACT_GELU_TANH 3 /* torch's approximate="tanh" form */

/* Problem descriptor.  Replaces the argument list the reference passes to its
 * Triton launches (src/flag_dnn/graph/kernels/fused_conv.py:151-191,
 * src/flag_dnn/ops/conv2d.py:3826-3865). */
typedef struct fdnn_conv_desc {
  int32_t dtype;                /* FDNN_F16 .. FDNN_F64; x, w, bias, scale, y share it */
  int32_t n, c, h, w;           /* input  x[N,C,H,W] */
  int32_t k, r, s;              /* filter w[K,C/groups,R,S] */
  int32_t stride_h, stride_w;
  int32_t pad_top, pad_bottom, pad_left, pad_right;
  int32_t dil_h, dil_w;
  int32_t groups;
  int32_t algo;                 /* FDNN_ALGO_* */
  int64_t x_strides[4];         /* element strides of x in (n,c,h,w) order */
  int64_t w_strides[4];         /* element strides of w in (k,c,r,s) order */
  int64_t y_strides[4];         /* element strides of y in (n,k,oh,ow) order */
} fdnn_conv_desc;

/* What fdnn_conv2d_query decides for a descriptor. */
typedef struct fdnn_conv_plan {
  int32_t algo;                 /* FDNN_ALGO_DIRECT, FDNN_ALGO_IGEMM or FDNN_ALGO_IGEMM_PAIR */
  int32_t oh, ow;               /* output size, rule of src/flag_dnn/ops/conv2d.py:52-62 */
  int32_t tile_m, tile_n, tile_k, stages; /* igemm tile; 0 for direct */
  int32_t x_repacked;           /* 1: x is first rewritten into the workspace as NHWC, C padded */
  int32_t w_packed;             /* 1: fwd needs a packed filter from fdnn_conv2d_pack_weight */
  int32_t c_padded;             /* channel count the igemm kernel iterates over */
  int32_t grid, block;          /* launch shape of the main kernel */
  int32_t launches;             /* kernels one fwd call launches (main + repack; per-group launches of a
                                   grouped layer all counted) */
  int32_t low_channel;          /* 1: C <= 4 path (pixel quads as GEMM rows, 16-pixel input windows) */
  int32_t pixel_group;          /* > 1: that many neighbouring output pixels form one GEMM row (narrow layers) */
  int32_t stream_k;             /* 1: given streamk_bytes of scratch, fdnn_conv2d_fwd_ex splits reductions over the CTA pairs */
  int64_t workspace_bytes;      /* scratch fwd needs (0 when x is consumed in place) */
  int64_t streamk_bytes;        /* size of that optional scratch (0: the plan does not split) */
  int64_t packed_weight_bytes;  /* size of the packed filter (0 when w is consumed in place); for a grouped
                                   layer the dense block-diagonal filter plus its packed form, or one
                                   packed filter per group back to back */
  int64_t smem_bytes;           /* dynamic shared memory of the main kernel */
  double flops;                 /* 2*N*OH*OW*K*(C/groups)*R*S, benchmark/test_conv2d_perf.py:139-148 */
  double bytes;                 /* x + w + bias + y once each, benchmark/base.py:661-668 */
} fdnn_conv_plan;

/* Reduction splitting ("stream-K", plan.stream_k): when the tiles of a layer do not fill a whole number of
 * rounds of the GPU's CTA pairs (196 tiles on 74 pairs: 2.65 rounds of work in 3), the pairs share the
 * (tile, reduction step) space evenly and exchange fp32 partial sums of the tiles cut in between through
 * plan.streamk_bytes of scratch.  It is optional and explicit: only fdnn_conv2d_fwd_ex takes that scratch;
 * without it (and through every other entry point) the same kernel runs whole tiles.  The first
 * FDNN_STREAMK_FLAG_BYTES of the scratch are flags: they must be zero when the scratch is first used, and
 * every launch leaves them zero, so one scratch buffer serves any number of launches as long as they do not
 * overlap on the GPU (one buffer per stream).  A launch that ended in FDNN_DEVICE_TIMEOUT may leave flags
 * raised: zero them again.  Results do not depend on timing, but a tile's fp32 additions are grouped by the
 * split, so the last bit of an output can differ from the unsplit schedule's. */
#define FDNN_STREAMK_FLAG_BYTES 8192

/* Library/ABI version (FDNN_ABI_VERSION of the built library). */
int fdnn_abi_version(void);

/* Human-readable text for a status code; never NULL. */
const char* fdnn_status_string(int status);

/* Detail text of the last non-OK status returned on the calling thread. */
const char* fdnn_last_error(void);

/* Validates `desc` (same rules and order as _check_conv2d_inputs,
 * src/flag_dnn/ops/conv2d.py:90-135) and fills `plan`.  Needs no GPU except to
 * read the current device's SM count for the grid size (148 assumed if no
 * device is visible).  `x`, `w`, `y` may be NULL; when given, their alignment
 * decides whether the tensors can be consumed in place by TMA. */
int fdnn_conv2d_query(const fdnn_conv_desc* desc, const void* x, const void* w,
                      const void* y, fdnn_conv_plan* plan);

/* One-time filter relayout, the counterpart of the reference's packers
 * (src/flag_dnn/ops/conv2d.py:193-276): w[K,C/g,R,S] (any strides) ->
 * [K,R,S,Cpad] with zero padding (for f32 a second copy holds the low TF32
 * halves), or the low-channel / pixel-grouped layout when the plan for `desc`
 * says plan.low_channel / plan.pixel_group.  `y` is the output pointer the
 * forward call will write (NULL: a 16-byte aligned one); only its alignment is
 * read, because it takes part in choosing the plan and with it the layout.
 * `packed` must hold plan.packed_weight_bytes.  Asynchronous on `stream` (a
 * cudaStream_t passed as void*).  The library remembers, per `packed` address,
 * which layout it wrote; fdnn_conv2d_fwd answers FDNN_BAD_PARAM when handed a
 * buffer whose remembered layout is not the one its own plan reads. */
int fdnn_conv2d_pack_weight(const fdnn_conv_desc* desc, const void* w, const void* y,
                            void* packed, int64_t packed_bytes, void* stream);

/* y = act( conv(x, w) * scale[k] + bias[k] ), fp32 accumulate, one rounding to
 * the output dtype.  Replaces conv2d()'s Triton launches
 * (src/flag_dnn/ops/conv2d.py:3575-4449) and fused_conv2d_bias_relu()
 * (src/flag_dnn/graph/kernels/fused_conv.py:62-193).
 *   w_packed : from fdnn_conv2d_pack_weight when plan.w_packed, else NULL
 *   bias     : [K] or NULL;  scale : [K] or NULL (BN-folded per-channel scale)
 *   workspace: >= plan.workspace_bytes, 256-byte aligned (may be NULL if 0)
 * Asynchronous on `stream`; performs no allocation and no host sync, so it
 * can be captured into a CUDA graph.  The device current at the call must be
 * the one that owns the pointers. */
int fdnn_conv2d_fwd(const fdnn_conv_desc* desc, const void* x, const void* w,
                    const void* w_packed, const void* bias, const void* scale,
                    int activation, void* y, void* workspace,
                    int64_t workspace_bytes, void* stream);

/* y = act( conv(x, w) * scale[k] + bias[k] + residual ): fdnn_conv2d_fwd with a
 * residual tensor added in fp32 before the activation and the single rounding
 * (a ResNet block's third convolution, its shortcut add and the ReLU in one
 * pass; the reference runs them as separate nodes, src/flag_dnn/ops/binary.py:380
 * after src/flag_dnn/ops/conv2d.py:3575).  `residual` has y's dtype, shape and
 * strides (desc->y_strides), the same address alignment modulo 16 bytes, and
 * must not overlap y; NULL makes this fdnn_conv2d_fwd.  The low-channel path
 * (plan.low_channel) answers FDNN_NOT_SUPPORTED when a residual is given. */
int fdnn_conv2d_fwd_residual(const fdnn_conv_desc* desc, const void* x,
                             const void* w, const void* w_packed,
                             const void* bias, const void* scale,
                             const void* residual, int activation, void* y,
                             void* workspace, int64_t workspace_bytes,
                             void* stream);

/* fdnn_conv2d_fwd_residual plus the optional scratch for reduction splitting (see FDNN_STREAMK_FLAG_BYTES):
 * `streamk_scratch` of at least plan.streamk_bytes, 256-byte aligned, flags zero; NULL runs whole tiles.
 * No counterpart in the reference, whose Triton kernels assign whole tiles
 * (src/flag_dnn/graph/kernels/fused_conv.py:145-149). */
int fdnn_conv2d_fwd_ex(const fdnn_conv_desc* desc, const void* x, const void* w,
                       const void* w_packed, const void* bias, const void* scale,
                       const void* residual, int activation, void* y,
                       void* workspace, int64_t workspace_bytes,
                       void* streamk_scratch, int64_t streamk_bytes, void* stream);

/* Host-buffer convenience: same as fdnn_conv2d_fwd but x, w, bias, scale and y
 * are HOST pointers (dense, described by the strides in `desc`); copies in,
 * runs and copies y back on `stream`, using the caller-provided device arena
 * `dev_arena` of `arena_bytes` (see fdnn_conv2d_host_arena_bytes).
 * Synchronises `stream` before returning. */
int fdnn_conv2d_fwd_host(const fdnn_conv_desc* desc, const void* x_host,
                         const void* w_host, const void* bias_host,
                         const void* scale_host, int activation, void* y_host,
                         void* dev_arena, int64_t arena_bytes, void* stream);

/* Device bytes fdnn_conv2d_fwd_host needs for `desc`. */
int fdnn_conv2d_host_arena_bytes(const fdnn_conv_desc* desc, int64_t* bytes);

/* Pooling next to the path (the layers either side of a ResNet's convolutions).
 * Strides are element strides in (n, c, h, w) order; NCHW and channels-last
 * both work, dense channels-last f16/bf16 with c % 8 == 0 moves 16 bytes per
 * thread.  `oh` / `ow` are the output sizes the caller computed (for max
 * pooling with the ceil_mode rule of src/flag_dnn/ops/max_pool2d.py:201-230). */
typedef struct fdnn_pool_desc {
  int32_t dtype; /* FDNN_F16 / BF16 / F32 / F64 */
  int32_t n, c, h, w, oh, ow;
  int32_t kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w; /* max pooling only */
  int64_t x_strides[4];
  int64_t y_strides[4];
} fdnn_pool_desc;

/* Replaces the Triton launches of max_pool2d (src/flag_dnn/ops/max_pool2d.py:174-330).
 * -inf padding, NaN wins; `indices` (int64, y's strides, ih * W + iw) may be NULL. */
int fdnn_max_pool2d_fwd(const fdnn_pool_desc* desc, const void* x, void* y,
                        int64_t* indices, void* stream);

/* Replaces the Triton launches of adaptive_avg_pool2d
 * (src/flag_dnn/ops/adaptive_avg_pool2d.py:456-640): window
 * [floor(o*L/O), ceil((o+1)*L/O)), fp32 (fp64) accumulate. */
int fdnn_adaptive_avg_pool2d_fwd(const fdnn_pool_desc* desc, const void* x,
                                 void* y, void* stream);

/* Every wait inside the kernels is bounded; a wait that runs out records a
 * code in a per-device status word and the kernel returns early.  This call
 * synchronises the current device, returns the word in *word (0 = no
 * incident) and clears it.  Returns FDNN_DEVICE_TIMEOUT if it was non-zero. */
int fdnn_device_status(uint32_t* word);

/* Forward call for callers that cannot allocate device memory (no counterpart
 * in the reference).  Identical to fdnn_conv2d_fwd except that the scratch for
 * the relayout of x is a fixed array of FDNN_STATIC_SCRATCH_BYTES inside the
 * library image instead of a caller-provided workspace.  It exists for hosts
 * that fixed their device-memory budget at start-up and may not call
 * cudaMalloc afterwards (serving processes with a pre-sized arena, plug-ins
 * running inside another framework's memory pool, processes under a per-job
 * memory quota).  It calls no cudaMalloc, cudaFree or allocating library
 * routine.
 *   - Problems whose plan.workspace_bytes exceeds FDNN_STATIC_SCRATCH_BYTES are
 *     refused with FDNN_WORKSPACE_TOO_SMALL (text in
 *     fdnn_static_scratch_last_error); use fdnn_conv2d_fwd for those.
 *   - The first call on each device looks up the array's device address; make
 *     that first call before starting any stream capture on that device.
 *   - Every call on a device shares the one array, which keeps whatever the
 *     last call left in it.  Calls that may overlap on the GPU (different
 *     streams, or graphs replayed concurrently) race on it: serialise them.
 *   - x, w, w_packed, bias, scale and y are passed exactly as for
 *     fdnn_conv2d_fwd; a packed filter, where the plan asks for one, is still
 *     the caller's buffer. */
#define FDNN_STATIC_SCRATCH_BYTES (16 * 1024 * 1024)
int fdnn_conv2d_fwd_static_scratch(const fdnn_conv_desc* desc, const void* x, const void* w,
                                   const void* w_packed, const void* bias, const void* scale,
                                   int activation, void* y, void* stream);
/* Capacity of the built-in scratch (FDNN_STATIC_SCRATCH_BYTES of the built library). */
int64_t fdnn_static_scratch_bytes(void);
/* Detail text of the last failure of fdnn_conv2d_fwd_static_scratch on this thread. */
const char* fdnn_static_scratch_last_error(void);

/* Development aid: when given a device buffer of 16 int64, the implicit-GEMM
 * kernel's first CTA writes per-role cycle counters into it on every launch
 * (producer: [0] stage-wait, [1] copy-issue, [2] total, [3] reduction steps;
 * issuer: [4] data-wait, [5] accumulator-wait, [6] total, [7] tiles;
 * epilogue: [8] accumulator-wait, [9] total).  NULL switches it off (default).
 * The setting belongs to the device that is current when this is called. */
int fdnn_debug_set_profile_buffer(void* device_buffer_16_int64);

/* Test aid for the bounded waits: launches made after this call give up a wait
 * after `wait_limit_cycles` SM clocks (0 restores the default of about two
 * seconds); with `skip_copies` non-zero the kernels' copy-issuing role does
 * nothing, so that the first wait for data runs out.  The kernel then records
 * its incident code, returns normally and fdnn_device_status reports
 * FDNN_DEVICE_TIMEOUT once.  Process-wide; not for production use. */
int fdnn_debug_set_wait_limit(int64_t wait_limit_cycles, int skip_copies);

/* Encoded tensor maps are remembered per calling thread, keyed by every
 * argument of the encode call, so a layer run again on the same buffers does
 * not go back to the driver (the reference keeps its tuned launch
 * configurations per shape in a similar table, src/flag_dnn/utils/libentry.py:499-579).
 * This reports, process-wide since load, how many maps were taken from the
 * table (`reused`) and how many had to be encoded (`encoded`); either may be NULL. */
int fdnn_debug_tensor_map_counters(int64_t* reused, int64_t* encoded);

#ifdef __cplusplus
}
#endif
#endif /* FLAGDNN_B200_H_ */
