/*
 * itexb200.h - C-ABI of libitexb200, the B200 (sm_100a) implementation of the
 * quantized-inference hot path of intel/intel-extension-for-tensorflow (ITEX).
 *
 * Three layers, all plain C (no exceptions cross this boundary, every function
 * returns an itexb_status_t unless noted, caller owns every pointer it passes):
 *
 *   1. Device runtime   itexb_rt_*      - what ITEX's StreamExecutor callbacks do
 *   2. Kernel launches  itexb_quantize / itexb_dequantize / itexb_gemm / itexb_conv2d /
 *                       itexb_fp8_*     - raw device pointers + POD descriptors
 *   3. Op layer         itexb_op_*      - ITEX's op names, attrs, input/output order,
 *                       HostMemory conventions and error behaviour; this is what a
 *                       TensorFlow PluggableDevice shim binds its create/compute/delete
 *                       callbacks to.
 *
 * Citations name files of the reference project by their path inside it.
 */
#ifndef ITEXB200_H_
#define ITEXB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ITEXB_API __attribute__((visibility("default")))

/* Status codes carry TensorFlow's TF_Code values so a shim can forward them to
 * TF_SetStatus unchanged (the reference reports errors through
 * OP_REQUIRES -> TF_OpKernelContext_Failure, itex/core/utils/op_kernel.cc:511-532). */
typedef enum itexb_status {
  ITEXB_OK = 0,
  ITEXB_INVALID_ARGUMENT = 3,
  ITEXB_NOT_FOUND = 5,
  ITEXB_RESOURCE_EXHAUSTED = 8,
  ITEXB_FAILED_PRECONDITION = 9,
  ITEXB_ABORTED = 10,
  ITEXB_UNIMPLEMENTED = 12,
  ITEXB_INTERNAL = 13
} itexb_status_t;

/* Element types, numbered like TensorFlow's DataType enum (the attr values T, T1,
 * Toutput, Tbias, dtype ... arrive as these numbers).  FP8 has no TF number on this
 * path: the reference carries e4m3/e5m2 bytes in DT_INT8 tensors and names the
 * format in a string attr (itex/core/ops/fp8_ops.cc:22-61). */
typedef enum itexb_dtype {
  ITEXB_DT_INVALID = 0,
  ITEXB_DT_FLOAT = 1,
  ITEXB_DT_INT32 = 3,
  ITEXB_DT_UINT8 = 4,
  ITEXB_DT_INT8 = 6,
  ITEXB_DT_INT64 = 9,
  ITEXB_DT_QINT8 = 11,
  ITEXB_DT_QUINT8 = 12,
  ITEXB_DT_QINT32 = 13,
  ITEXB_DT_BFLOAT16 = 14,
  ITEXB_DT_HALF = 19,
  ITEXB_DT_FP8_E4M3 = 101,
  ITEXB_DT_FP8_E5M2 = 102
} itexb_dtype_t;

/* Thread-local text of the last non-OK status returned on the calling thread. */
ITEXB_API const char* itexb_last_error(void);
ITEXB_API const char* itexb_version(void);
/* Number of kernel launches this library has issued (all threads) since load. */
ITEXB_API uint64_t itexb_launch_count(void);

/* ------------------------------------------------------------------------- */
/* 1. Device runtime.  Replaces the StreamExecutor callback table the reference
 *    fills in itex/core/devices/gpu/gpu_device_plugin.cc:26-376 (listed at
 *    itex/core/wrapper/itex_gpu_wrapper.cc:190-228): device memory through the
 *    plugin's own caching allocator, pinned host memory, streams, events,
 *    async/sync copies, memset, host callbacks.  itexb_stream_t is a cudaStream_t
 *    (NULL = the legacy default stream); itexb_event_t is a cudaEvent_t.          */
/* ------------------------------------------------------------------------- */
typedef void* itexb_stream_t;
typedef void* itexb_event_t;

typedef struct itexb_allocator_stats {
  int64_t num_allocs;       /* calls served */
  int64_t bytes_in_use;     /* handed out and not yet freed */
  int64_t peak_bytes_in_use;
  int64_t bytes_reserved;   /* held from the driver (in use + cached) */
  int64_t largest_alloc_size;
  int64_t bytes_limit;      /* 0 = no limit (env ITEXB_LIMIT_MEMORY_MB, like ITEX_LIMIT_MEMORY_SIZE_IN_MB) */
} itexb_allocator_stats_t;

ITEXB_API int itexb_rt_device_count(int* count);
ITEXB_API int itexb_rt_set_device(int ordinal);
ITEXB_API int itexb_rt_device_memory_usage(int ordinal, int64_t* free_bytes, int64_t* total_bytes);
ITEXB_API int itexb_rt_allocate(int ordinal, size_t bytes, void** ptr);      /* 256-byte aligned */
/* The block goes back to the free lists at once and may be handed out again by the next allocate: the caller must
 * know that all device work that reads or writes it has finished (the contract of StreamExecutor's deallocate,
 * itex/core/devices/gpu/gpu_device_plugin.cc:80-92, where TensorFlow orders frees itself). */
ITEXB_API int itexb_rt_deallocate(int ordinal, void* ptr);
/* Stream-ordered free: the block is reused only after the work queued on `stream` so far has finished (an event is
 * recorded; allocate checks it).  What the op layer uses for its own per-instance buffers. */
ITEXB_API int itexb_rt_deallocate_after(int ordinal, void* ptr, itexb_stream_t stream);
ITEXB_API int itexb_rt_host_allocate(size_t bytes, void** ptr);              /* pinned */
ITEXB_API int itexb_rt_host_deallocate(void* ptr);
ITEXB_API int itexb_rt_allocator_stats(int ordinal, itexb_allocator_stats_t* stats);
ITEXB_API int itexb_rt_trim(int ordinal);                                    /* return cached blocks to the driver */
ITEXB_API int itexb_rt_create_stream(int ordinal, itexb_stream_t* stream);
ITEXB_API int itexb_rt_destroy_stream(itexb_stream_t stream);
ITEXB_API int itexb_rt_stream_dependency(itexb_stream_t dependent, itexb_stream_t other);
ITEXB_API int itexb_rt_stream_device(itexb_stream_t stream, int* ordinal);     /* the device a stream belongs to (NULL stream: the current device) */
ITEXB_API int itexb_rt_stream_status(itexb_stream_t stream);                 /* OK, or INTERNAL when the stream is in error */
ITEXB_API int itexb_rt_create_event(itexb_event_t* event);
ITEXB_API int itexb_rt_destroy_event(itexb_event_t event);
ITEXB_API int itexb_rt_record_event(itexb_stream_t stream, itexb_event_t event);
ITEXB_API int itexb_rt_wait_for_event(itexb_stream_t stream, itexb_event_t event);
ITEXB_API int itexb_rt_event_status(itexb_event_t event, int* complete);
ITEXB_API int itexb_rt_event_elapsed_ms(itexb_event_t start, itexb_event_t stop, float* ms);
ITEXB_API int itexb_rt_memcpy_h2d(void* dst_dev, const void* src_host, size_t bytes, itexb_stream_t stream);
ITEXB_API int itexb_rt_memcpy_d2h(void* dst_host, const void* src_dev, size_t bytes, itexb_stream_t stream);
ITEXB_API int itexb_rt_memcpy_d2d(void* dst_dev, const void* src_dev, size_t bytes, itexb_stream_t stream);
ITEXB_API int itexb_rt_sync_memcpy_h2d(void* dst_dev, const void* src_host, size_t bytes);
ITEXB_API int itexb_rt_sync_memcpy_d2h(void* dst_host, const void* src_dev, size_t bytes);
ITEXB_API int itexb_rt_sync_memcpy_d2d(void* dst_dev, const void* src_dev, size_t bytes);
ITEXB_API int itexb_rt_mem_zero(void* dev, size_t bytes, itexb_stream_t stream);
ITEXB_API int itexb_rt_memset(void* dev, uint8_t value, size_t bytes, itexb_stream_t stream);
ITEXB_API int itexb_rt_memset32(void* dev, uint32_t pattern, size_t bytes, itexb_stream_t stream);
ITEXB_API int itexb_rt_block_host_until_done(itexb_stream_t stream);
ITEXB_API int itexb_rt_block_host_for_event(itexb_event_t event);
ITEXB_API int itexb_rt_synchronize_all_activity(int ordinal);
ITEXB_API int itexb_rt_host_callback(itexb_stream_t stream, void (*fn)(void* arg), void* arg);

/* Peer memory for multi-GPU jobs with one process per GPU (no counterpart in the reference's callback table).
 * itexb_rt_ipc_export: a 64-byte handle of a block obtained from itexb_rt_allocate, to be sent to the other processes
 * of the node by any host channel.  itexb_rt_ipc_open (with the opening process's own device current): maps the block
 * into this process and enables peer access; the pointer may be stored to (and loaded from) by this process's
 * kernels over NVLink.  itexb_rt_ipc_close unmaps it.  The exporting process must keep the block allocated while
 * any other process has it open. */
#define ITEXB_IPC_HANDLE_BYTES 64
ITEXB_API int itexb_rt_ipc_export(void* dev_ptr, unsigned char handle[ITEXB_IPC_HANDLE_BYTES]);
ITEXB_API int itexb_rt_ipc_open(const unsigned char handle[ITEXB_IPC_HANDLE_BYTES], void** dev_ptr);
ITEXB_API int itexb_rt_ipc_close(void* dev_ptr);
/* Completion flags of the fused all-gather.  Each GPU owns an int32 array `flags[world]` in memory its peers have
 * opened.  The value written and waited for is  value + *value_ptr  (value_ptr optional): a step counter kept in
 * device memory and advanced by itexb_peer_advance lets a CUDA graph that holds a whole step be replayed, its kernel
 * arguments unchanged, with a new value every time.
 * itexb_peer_signal (on the stream that carried the GEMM): after everything queued before it on `stream` has finished
 * and been made visible system-wide, stores the value into flag_ptrs[i] for i in [0, n) - normally slot [my_rank] of
 * every GPU's array.  itexb_peer_wait: one small kernel that polls local_flags[0 .. n) until each is >= the value
 * (values only grow); the wait is bounded (about a second, or half the "gemm_wait_limit_cycles" hook) and on expiry
 * writes 5 into *status_word (optional) and returns, so a peer that never signals costs a status, not a hang.
 * itexb_peer_advance: *counter += 1 on the stream. */
ITEXB_API int itexb_peer_signal(int32_t* const* flag_ptrs, int32_t n, int32_t value, const int32_t* value_ptr, itexb_stream_t stream);
ITEXB_API int itexb_peer_wait(const int32_t* local_flags, int32_t n, int32_t value, const int32_t* value_ptr, int32_t* status_word,
                              itexb_stream_t stream);
ITEXB_API int itexb_peer_advance(int32_t* counter, itexb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* 2. Kernel launches (device pointers; asynchronous on `stream`).            */
/* ------------------------------------------------------------------------- */

/* How the affine quantize kernel combines its per-slice constants. */
typedef enum itexb_quant_kind {
  ITEXB_QUANT_SCALED = 0,          /* q = sat(rne(x*s))                     SCALED      */
  ITEXB_QUANT_MIN_FIRST_LEGACY = 1,/* q = sat(rne(x*s + shift*s))           legacy MIN_FIRST, shift = -min */
  ITEXB_QUANT_MIN_FIRST_CLASSIC = 2/* q = sat(rne(x*s + zp))                classic asymmetric */
} itexb_quant_kind_t;

/* Replaces the dnnl::reorder / dnnl::binary the reference executes in
 * QuantizeV2Op::Compute (itex/core/kernels/common/quantize_op.h:256-314,394).
 * x: FLOAT | BFLOAT16 | HALF, q: QINT8 | QUINT8, n elements.  The tensor is viewed
 * as [outer, nslice, inner]; slice of element i is (i / inner) % nslice.  With
 * nslice == 1 and scale == NULL the host scalars are used.  `shift` carries the
 * second constant of kinds 1 and 2 (NULL -> shift_host).                       */
ITEXB_API int itexb_quantize(const void* x, int x_dtype, void* q, int q_dtype, int64_t n,
                             int64_t inner, int64_t nslice, int kind,
                             const float* scale, const float* shift,
                             float scale_host, float shift_host, itexb_stream_t stream);

/* Replaces the dnnl::reorder of DequantizeOp::Compute
 * (itex/core/kernels/common/dequantize_op.h:143-169): y = ydtype((float(q) - zp) * s). */
ITEXB_API int itexb_dequantize(const void* q, int q_dtype, void* y, int y_dtype, int64_t n,
                               int64_t inner, int64_t nslice, const float* scale, const float* zp,
                               float scale_host, float zp_host, itexb_stream_t stream);

/* min and max of a FLOAT|BFLOAT16 tensor into minmax[0], minmax[1] (device), for graphs
 * that derive a dynamic range on the device.  minmax must be initialised by
 * itexb_minmax_init first (+inf, -inf).  No counterpart kernel in the reference: there
 * the range arrives as a HostMemory input (itex/core/kernels/gpu/quantize_op.cc:25-31). */
ITEXB_API int itexb_minmax_init(float* minmax, itexb_stream_t stream);
ITEXB_API int itexb_minmax(const void* x, int x_dtype, int64_t n, float* minmax, itexb_stream_t stream);
/* QuantizeV2 SCALED whose range is read on the device from minmax[0..1] (already
 * adjusted like AdjustInputMinMaxRange + GetScaleAndZeropointAndAlignMinMax would);
 * writes the scale it used and the aligned range to out3 = {scale, out_min, out_max}. */
ITEXB_API int itexb_quantize_dynamic(const void* x, int x_dtype, void* q, int q_dtype, int64_t n,
                                     const float* minmax, float ensure_minimum_range, float* out3,
                                     itexb_stream_t stream);

/* itexb_quantize_dynamic that also writes the consuming matmul's per-output-channel scales (what
 * itexb_matmul_scales_dynamic computes: scales[j] for j < n_scales from weight_range[j]), saving a launch. */
ITEXB_API int itexb_quantize_dynamic_scales(const void* x, int x_dtype, void* q, int q_dtype, int64_t n,
                                            const float* minmax, float ensure_minimum_range, float* out3,
                                            const float* weight_range, int32_t n_scales, float* scales,
                                            itexb_stream_t stream);

/* Per-output-channel scale of the fused matmul ops, computed on the device from a device-resident
 * activation range: scales[j] = (max(|out_min|,|out_max|) * weight_range[j]) / (max_int8(a_dtype) * 127),
 * range3 = the {scale, out_min, out_max} itexb_quantize_dynamic wrote, weight_range[j] =
 * max(|min_b[j]|, |max_b[j]|).  The formula of QuantizedFusedMatMulOp::ExtendInt8PostOps
 * (itex/core/kernels/common/quantized_matmul_common.h:1627-1650); there it runs on the host after a
 * blocking copy of the range (HostDataCache, kernels/common/host_data_cache.h:36-97). */
ITEXB_API int itexb_matmul_scales_dynamic(const float* range3, const float* weight_range, int32_t n, int a_dtype,
                                          float* scales, itexb_stream_t stream);

/* Weight pre-pack: [k,n] row-major (the TF layout of `b`) -> [n,k_pad] row-major with k
 * padded by zeros to a multiple of 16, the K-major layout the MMA kernel stages with TMA.
 * Plays the role of the cached weight reorder of
 * itex/core/kernels/common/quantized_matmul_common.h:241-275.  1-byte elements.        */
ITEXB_API int itexb_pack_weights_kn(const void* b_kn, void* b_nk, int64_t k, int64_t n, int64_t k_pad,
                                    itexb_stream_t stream);
/* The same for `batch` matrices: matrix i is read at b_kn + i*src_stride and written at b_nk + i*dst_stride
 * (bytes).  Used where a batched matmul receives its right operand as [.., k, n]
 * (adj_y = false, itex/core/kernels/common/batch_matmul_op.h:112-121).  batch <= 65535. */
ITEXB_API int itexb_pack_weights_kn_batched(const void* b_kn, void* b_nk, int64_t k, int64_t n, int64_t k_pad, int64_t batch,
                                            int64_t src_stride, int64_t dst_stride, itexb_stream_t stream);
/* Column sums of an int8 [k,n] weight (MIN_FIRST compensation,
 * quantized_matmul_common.h:569-574). */
ITEXB_API int itexb_colsum_s8(const int8_t* b_kn, int32_t* colsum, int64_t k, int64_t n, itexb_stream_t stream);

/* What the GEMM / conv epilogue does with an accumulator acc[m][n]:
 *   f = float(acc) * scale[n or 0]     (scale == NULL and scale_count == 0: no multiply)
 *   f = f + bias[n]                    (bias != NULL)
 *   f = f + sum_scale * float(summand[m][n])   (summand != NULL)
 *   f = max(f, 0)                      (relu)
 *   f = activation(f) * post_scale     (activation != ITEXB_ACT_NONE; post_scale 0 means 1)
 *   f = float(mid_dtype(f))            (mid_dtype != 0)
 *   out = convert(f): QUINT8/QINT8/QINT32 saturate then round-to-nearest-even;
 *         FLOAT/BFLOAT16/HALF plain conversion; FP8_E4M3 saturating RNE of f*out_scale[0]
 *         with amax[0] = max(amax[0], max|f|).
 * Separate fp32 multiply and add (no FMA), the order oneDNN's int8 primitives use for
 * "scale on DNNL_ARG_WEIGHTS, bias after" (itex/core/utils/onednn/onednn_post_op_util.cc:283-295).
 * raw_acc = 1 with out_dtype QINT32 stores the exact int32 accumulator instead.        */
/* Element-wise post-ops of the fused matmul ops, named after the oneDNN algorithms the reference maps
 * them to (itex/core/utils/onednn/onednn_post_op_util.cc:22-71): relu with negative slope act_alpha
 * (Relu: 0, LeakyRelu), clip to [act_alpha, act_beta] (Relu6), gelu_erf, gelu_tanh, logistic, tanh,
 * elu(act_alpha), swish(act_alpha), linear act_alpha*f + act_beta. */
typedef enum itexb_activation {
  ITEXB_ACT_NONE = 0,
  ITEXB_ACT_RELU = 1,
  ITEXB_ACT_CLIP = 2,
  ITEXB_ACT_GELU_ERF = 3,
  ITEXB_ACT_GELU_TANH = 4,
  ITEXB_ACT_SIGMOID = 5,
  ITEXB_ACT_TANH = 6,
  ITEXB_ACT_ELU = 7,
  ITEXB_ACT_SWISH = 8,
  ITEXB_ACT_LINEAR = 9
} itexb_activation_t;

typedef struct itexb_epilogue {
  const float* scale;      /* device, scale_count entries */
  int32_t scale_count;     /* 0, 1 or n */
  const float* alpha_a;    /* optional device scalars: scale used is alpha_a[0]*alpha_b[0] */
  const float* alpha_b;    /*   (FP8: a_scale_inv[i], b_scale_inv[j]); overrides `scale` */
  const float* bias;       /* device fp32 [n] or NULL */
  const void* summand;     /* device [m][n] or NULL */
  int32_t summand_dtype;   /* QUINT8 | QINT8 | FLOAT | BFLOAT16 | HALF */
  int64_t ld_summand;      /* elements */
  float sum_scale;
  int32_t relu;
  int32_t raw_acc;
  const float* out_scale;  /* FP8 output only: device scalar c_scale */
  float* amax;             /* FP8 output only: device scalar, atomically maxed */
  int32_t mid_dtype;       /* 0, or BFLOAT16 | HALF: round f to that type before the final
                              conversion (FP8 output of a matmul whose sum type is 16-bit) */
  int32_t activation;      /* itexb_activation_t, applied after summand and relu */
  float act_alpha, act_beta;
  float post_scale;        /* multiplies the activation's result; 0 is read as 1 */
} itexb_epilogue_t;

/* out[m][n] = epilogue( sum_k a[m][k] * b[n][k] ).
 * Replaces dnnl::inner_product_forward (quantized_matmul_common.h:223-226,92) and, for
 * FP8, the dequantize + dnnl::matmul (+ quantize) chain of
 * itex/core/kernels/gpu/fp8/fp8_matmul_gpu.h:34-162.
 * a: [m,k] row-major, lda elements (multiple of 16, base 16-byte aligned);
 * b: packed [n,k] row-major, ldb likewise.  a_dtype QUINT8|QINT8 with b_dtype QINT8
 * (int32 accumulation, exact), or both FP8_E4M3|FP8_E5M2 (fp32 accumulation).
 * status_word: optional device int32 that the kernel sets non-zero if one of its
 * bounded waits expired (0 stays 0 on success).                                        */
typedef struct itexb_gemm_params {
  int32_t m, n, k;
  int32_t a_dtype, b_dtype, out_dtype;
  const void* a; int64_t lda;
  const void* b; int64_t ldb;
  void* out;     int64_t ldo;
  itexb_epilogue_t ep;
  int32_t* status_word;
  /* Batched form (0 or 1 = a single GEMM): `batch` independent products with the same m, n, k and epilogue;
   * batch i reads a + i*stride_a, b + i*stride_b (elements = bytes; positive multiples of 16) and
   * writes out + i*stride_out elements (a multiple of ldo, at least m*ldo).  A summand follows out's layout.
   * Replaces the batched dnnl::matmul of BatchMatMulOp (itex/core/kernels/common/batch_matmul_op.h). */
  int32_t batch;
  int64_t stride_a, stride_b, stride_out;
  /* Fused all-gather by peer stores (column-parallel linears: each GPU computes [m, n] = its column shard and every
   * GPU needs all shards).  With num_peers > 0 every finished output tile is written not only to `out` but also,
   * by two copying warps of the kernel with ordinary 16-byte global stores (whole 512-byte rows per instruction), to
   * the same offsets of peer_out[0 .. num_peers) - device pointers into OTHER GPUs' memory (itexb_rt_ipc_open) laid
   * out exactly like `out` (same ldo) - while the tensor cores work on the next tiles.  Nothing is ever loaded from a peer.  Needs 16-byte aligned output rows (n * element size a multiple
   * of 16) and a single GEMM (batch <= 1); at most ITEXB_MAX_PEERS.  Completion is signalled separately
   * (itexb_peer_signal after the GEMM on the same stream, itexb_peer_wait on the receiving side).  No counterpart in
   * the reference, whose only collective call site is an all-reduce (itex/core/kernels/gpu/collective_ops.h:338-430). */
  int32_t num_peers;
  void* const* peer_out;   /* host array of num_peers device pointers */
} itexb_gemm_params_t;
#define ITEXB_MAX_PEERS 7
ITEXB_API int itexb_gemm(const itexb_gemm_params_t* p, itexb_stream_t stream);

/* Test hooks of the GEMM / convolution kernels' failure path; process-wide, read at every launch.  They have no
 * counterpart in the reference.  Keys:
 *   "gemm_wait_limit_cycles"  clock cycles the MMA issuer's wait on a pipeline stage may take before the kernel gives up
 *                             (the waits behind it - a producer's on a stage's release, the epilogue's on a whole
 *                             accumulator - get twice that); 0 restores the default of 4e9 (about 2 s);
 *   "gemm_skip_kblock"        the TMA producer of every CTA leaves out this k-block of its first tile - a barrier that
 *                             nothing completes, made on the host's request, so that a test can watch a wait run out
 *                             (status word 2, the MMA issuer's role), the kernel return and the next launch work; -1: off;
 *   "gemm_cta_pair"           1: plain GEMMs with 256-column tiles and an even number of tile rows run as pairs of CTAs
 *                             (a cluster of two per 256 x 256 tile, each CTA loading half of the B tile); 0: never;
 *                             -1: the launch decides (the default).  Results are bit-identical either way.
 * Unknown keys give ITEXB_NOT_FOUND. */
ITEXB_API int itexb_debug_set(const char* key, int64_t value);

/* NHWC x (packed) HWIO convolution as an implicit GEMM with the same epilogue.
 * Replaces dnnl::convolution_forward (itex/core/kernels/common/conv_ops.h:953-957,801).
 * x: [n,h,w,c] QUINT8|QINT8; filter packed by itexb_pack_filter_hwio to [co][k_pad],
 * k_pad = kh*kw*c_pad rounded up to 16; out: [n,oh,ow,co].  Padding is zero fill; pad_top/pad_left as
 * computed by GetWindowedOutputSizeVerboseV2 (itex/core/utils/common_shape_fns.cc:42-81).
 * c_pad is the channel pitch of one filter tap in the packed filter; itexb_conv2d_filter_c_pad
 * returns the value to use for a geometry (it reads n,h,w,c,kh,kw,strides,dilations,padding,oh,ow):
 * when the input can be read by TMA im2col loads (c a multiple of 16, strides up to 8, padding up to
 * 128) c rounded up to 32, 64 or a multiple of 128 (one filter tap is then one k-block of the GEMM),
 * otherwise c.  c_pad == c is always accepted. */
typedef struct itexb_conv_params {
  int32_t n, h, w, c;
  int32_t kh, kw, co;
  int32_t stride_h, stride_w, dil_h, dil_w;
  int32_t pad_top, pad_left;
  int32_t oh, ow;
  int32_t c_pad;           /* channels per tap in the packed filter: itexb_conv2d_filter_c_pad(), or c */
  int32_t x_dtype, out_dtype;
  const void* x;
  const void* filter_packed;
  void* out;
  itexb_epilogue_t ep;     /* scale_count 0, 1 or co; summand laid out like out */
  int32_t* status_word;
  void* workspace;         /* device scratch of itexb_conv2d_workspace_bytes() or NULL if 0 */
} itexb_conv_params_t;
ITEXB_API int itexb_pack_filter_hwio(const void* f_hwio, void* f_packed, int32_t kh, int32_t kw, int32_t c,
                                     int32_t co, int32_t c_pad, itexb_stream_t stream);
ITEXB_API int32_t itexb_conv2d_filter_c_pad(const itexb_conv_params_t* p);
ITEXB_API size_t itexb_conv2d_workspace_bytes(const itexb_conv_params_t* p);
ITEXB_API int itexb_conv2d(const itexb_conv_params_t* p, itexb_stream_t stream);

/* itexb_conv2d for callers that cannot allocate: same arguments, results and checks, but
 * p->workspace is ignored and the patch matrix goes into an array built into the library's
 * device image.  It exists for hosts that may not call cudaMalloc when the convolution is
 * due - a plugin inside another framework's memory arena, code between the begin and end of
 * a stream capture, an allocation-free serving loop.  It has no counterpart in the
 * reference (whose kernels take scratch from the framework's allocator).
 *   - Limit: convolutions whose itexb_conv2d_workspace_bytes() exceeds
 *     ITEXB_STATIC_SCRATCH_BYTES (16 MiB, held by every GPU that loads the library until the
 *     process exits) are refused with ITEXB_RESOURCE_EXHAUSTED.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call before any
 *     stream capture begins.
 *   - All calls share the one array, which keeps the previous call's contents (each call
 *     overwrites every byte it uses, padding zeros included).  Two calls whose kernels can
 *     overlap on the GPU - different streams, or different host threads - race on it:
 *     serialise them.                                                                       */
#define ITEXB_STATIC_SCRATCH_BYTES (16u << 20)
ITEXB_API int itexb_conv2d_static_scratch(const itexb_conv_params_t* p, itexb_stream_t stream);

/* y = transpose(x, perm): y.dims[d] = x.dims[perm[d]], elements of elem_size bytes (1: qint8 / quint8, 2, 4: qint32).
 * The data movement of the reference's QuantizedTransposeOp (itex/core/kernels/common/transpose_op.h:197-236 over its
 * TransposeOp); the range tensors pass through in the op layer.                                                        */
#define ITEXB_TRANSPOSE_MAX_RANK 8
typedef struct itexb_transpose_params {
  const void* x;
  void* y;
  int32_t rank;
  int32_t elem_size;
  int64_t dims[ITEXB_TRANSPOSE_MAX_RANK];   /* of x */
  int32_t perm[ITEXB_TRANSPOSE_MAX_RANK];
} itexb_transpose_params_t;
ITEXB_API int itexb_transpose(const itexb_transpose_params_t* p, itexb_stream_t stream);
/* `outer` dense rows of `width` bytes at src -> rows of `dpitch` bytes at dst, starting at byte `col` of each: one input of
 * a concatenation along an inner axis (the dnnl::concat of itex/core/kernels/common/quantized_concat_op.cc:196-231).  */
ITEXB_API int itexb_copy_rows(const void* src, void* dst, int64_t outer, int64_t width, int64_t dpitch, int64_t col, itexb_stream_t stream);

/* NHWC 8-bit pooling: max, or average over the window cells that lie inside the image
 * (rne(float(sum)/float(count)), saturated).  Replaces the dnnl::pooling_forward behind the
 * reference's quantized pooling kernels (itex/core/kernels/cpu/maxpooling_op.cc:43-52,
 * cpu/avgpooling_op.cc:50-58 over kernels/common/pooling_ops_common.h).                      */
typedef struct itexb_pool_params {
  int32_t n, h, w, c;
  int32_t kh, kw, stride_h, stride_w, pad_top, pad_left, oh, ow;
  int32_t dtype;           /* QUINT8 | QINT8 */
  int32_t is_avg;          /* 0 max, 1 average (padding excluded) */
  const void* x;
  void* out;
} itexb_pool_params_t;
ITEXB_API int itexb_pool2d(const itexb_pool_params_t* p, itexb_stream_t stream);

/* FP8 pointwise ops.  Replace the SYCL PointWiseKernel launched by
 * functor::Fp8Quantize / Fp8Dequantize (itex/core/kernels/gpu/fp8/fp8_quantize_gpu.h:36-72,
 * vectorized_pointwise.h:27-88).  scale / scale_inv / amax point at the meta element
 * (base + fp8_meta_index).  y = fp8(float(x)*scale[0]) saturating RNE; amax[0] is
 * atomically raised to max|x|.                                                          */
ITEXB_API int itexb_fp8_quantize(const void* x, int x_dtype, void* y, int fp8_dtype, int64_t n,
                                 const float* scale, float* amax, itexb_stream_t stream);
ITEXB_API int itexb_fp8_dequantize(const void* x, int fp8_dtype, void* y, int y_dtype, int64_t n,
                                   const float* scale_inv, itexb_stream_t stream);
/* y = fp8(gelu(x) * scale[0]), amax[0] raised to max|gelu(x)|; gelu(v) = v*(0.5 + 0.5*tanh(v*(0.79788456 + 0.03567741*v*v))).
 * Replaces functor::Fp8Gelu (itex/core/kernels/gpu/fp8/fp8_gelu_gpu.h:29-58). */
ITEXB_API int itexb_fp8_gelu(const void* x, int x_dtype, void* y, int fp8_dtype, int64_t n, const float* scale,
                             float* amax, itexb_stream_t stream);
/* The delayed-scaling state of one layer (amax_history [history_len, n], scale [n], scale_inv [n], device fp32) to and
 * from one self-describing host blob of itexb_fp8_meta_blob_bytes(history_len, n) bytes: what a checkpoint holds for a
 * layer.  In the reference the state is three non-trainable tf.Variables per direction
 * (itex/python/transformer/base.py:60-93) that TensorFlow's own checkpointing saves.  Both calls are ordered after the
 * work queued on `stream` and return when the copy is complete; load refuses a blob of another shape. */
ITEXB_API size_t itexb_fp8_meta_blob_bytes(int32_t history_len, int32_t n);
ITEXB_API int itexb_fp8_meta_save(const float* amax_history, const float* scale, const float* scale_inv, int32_t history_len, int32_t n,
                                  void* blob, size_t blob_bytes, itexb_stream_t stream);
ITEXB_API int itexb_fp8_meta_load(float* amax_history, float* scale, float* scale_inv, int32_t history_len, int32_t n, const void* blob,
                                  size_t blob_bytes, itexb_stream_t stream);
/* The FP8 cast of a gradient fused with its bias gradient, optionally through the derivative of GELU:
 *   t = grad (gelu_inp == NULL)  or  t = dgelu(gelu_inp) * grad;   out = fp8(t * scale[0]) [rows, cols];
 *   dbias[cols] = sum over rows of t (fp32 sums, stored in `dtype`);   amax[0] raised to max|t| (amax may be NULL).
 * grad, gelu_inp and dbias share `dtype` (FLOAT | BFLOAT16 | HALF).  workspace: device scratch of
 * itexb_fp8_quantize_dbias_workspace_bytes(rows, cols) bytes (per-block partial sums, added in a fixed order).
 * Replaces functor::Fp8QuantizeDbiasFused / Fp8QuantizeDbiasDgeluFused
 * (itex/core/kernels/gpu/fp8/fp8_quantize_fusion_gpu.h:33-300). */
ITEXB_API size_t itexb_fp8_quantize_dbias_workspace_bytes(int64_t rows, int64_t cols);
ITEXB_API int itexb_fp8_quantize_dbias(const void* grad, const void* gelu_inp, int dtype, void* out, int fp8_dtype, void* dbias,
                                       int64_t rows, int64_t cols, const float* scale, float* amax, void* workspace,
                                       itexb_stream_t stream);
/* Layer normalisation over the columns of x [rows, cols] with an FP8 (z_dtype FP8_E4M3|FP8_E5M2: z = fp8(v * z_scale[0]),
 * z_amax[0] raised to max|v|) or real-valued (FLOAT|BFLOAT16|HALF, z_scale / z_amax unused) output;
 * v = gamma * (x - mu) * rsigma + beta, mu[rows] and rsigma[rows] = rsqrt(var + epsilon) are returned.
 * Replaces functor::Fp8LayerNormFwd (itex/core/kernels/gpu/fp8/fp8_layernorm_gpu.h:108-257). */
ITEXB_API int itexb_fp8_layernorm(const void* x, int x_dtype, const void* gamma, const void* beta, int w_dtype, void* z,
                                  int z_dtype, float* mu, float* rsigma, int64_t rows, int64_t cols, float epsilon,
                                  const float* z_scale, float* z_amax, itexb_stream_t stream);
/* Delayed-scaling update of itex/python/fp8/autocast.py:44-121 for `n` meta slots on the
 * device: amax = max over the `history_len` rows (algo 0 "max") or row 0 (algo 1
 * "most_recent"); scale from amax; roll rows by -1 and zero row 0; scale_inv = 1/scale. */
ITEXB_API int itexb_fp8_amax_and_scale_update(float* amax_history, float* scale, float* scale_inv,
                                              int32_t history_len, int32_t n, float fp8_max, float margin,
                                              int32_t algo, itexb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* 3. Op layer.  One kernel object per graph node, created from the node's op name
 *    and attrs, computed many times, possibly from several threads (each instance
 *    serialises itself like the reference's mu_compute_,
 *    quantized_matmul_common.h:62, conv_ops.h:786).  Mirrors the three callbacks
 *    the reference registers with TF_NewKernelBuilder (itex/core/utils/op_kernel.h:710-714,
 *    op_kernel.cc:887-918).                                                             */
/* ------------------------------------------------------------------------- */
#define ITEXB_MAX_DIMS 8

typedef struct itexb_tensor {
  int32_t dtype;                 /* itexb_dtype_t */
  int32_t rank;
  int64_t dims[ITEXB_MAX_DIMS];
  void* data;                    /* device memory, or host memory for HostMemory args */
  int32_t on_host;               /* 1: `data` is host memory */
  int32_t reserved;
} itexb_tensor_t;

typedef enum itexb_attr_type {
  ITEXB_ATTR_INT = 0, ITEXB_ATTR_FLOAT = 1, ITEXB_ATTR_BOOL = 2, ITEXB_ATTR_STRING = 3,
  ITEXB_ATTR_TYPE = 4, ITEXB_ATTR_INT_LIST = 5, ITEXB_ATTR_STRING_LIST = 6
} itexb_attr_type_t;

typedef struct itexb_attr {
  const char* name;
  int32_t type;                  /* itexb_attr_type_t */
  int64_t i;                     /* INT, BOOL, TYPE (itexb_dtype_t) */
  float f;                       /* FLOAT */
  const char* s;                 /* STRING */
  const int64_t* list_i;         /* INT_LIST */
  const char* const* list_s;     /* STRING_LIST */
  int32_t list_len;
} itexb_attr_t;

typedef struct itexb_op itexb_op_t;

/* The op's view of one Compute call: what TF_GetInput / TF_AllocateOutput /
 * TF_AllocateTemp / TF_GetStream give the reference's kernels
 * (itex/core/utils/op_kernel.cc:117,338,441; op_kernel.h:404-407).
 * allocate_output must set out->data for a tensor whose dtype/rank/dims/on_host the
 * op has filled in; allocate_temp memory only needs to live until the work the op has
 * enqueued on `stream` has run (the default context frees it stream-ordered).        */
typedef struct itexb_op_context {
  void* user;
  int32_t num_inputs;
  const itexb_tensor_t* inputs;
  int32_t device_ordinal;
  itexb_stream_t stream;
  int (*allocate_output)(void* user, int index, itexb_tensor_t* out);
  int (*allocate_temp)(void* user, size_t bytes, int on_host, void** ptr);
} itexb_op_context_t;

/* Names of the ops this library implements, NULL-terminated. */
ITEXB_API const char* const* itexb_op_list(void);
/* Input names and which inputs/outputs are HostMemory for an op (the lists of
 * itex/core/kernels/gpu/quantize_op.cc:25-46, gpu/quantized_matmul.cc:53-102,
 * gpu/quantized_conv_ops.cc:72-140).  Bit i of the masks = argument i.  The fused matmul ops
 * (_QuantizedFusedMatMul*, _QuantizedMatMul) take list-typed arguments whose length depends on
 * fused_ops: they report -1 counts and an input mask of 0, and every range tensor
 * (min_*, max_*) must be in host memory - the HostMemoryList arguments of
 * gpu/quantized_matmul.cc:137-182.                                                  */
ITEXB_API int itexb_op_signature(const char* op_name, int* num_inputs, int* num_outputs,
                                 uint32_t* host_input_mask, uint32_t* host_output_mask);
/* The op definition a TensorFlow plugin has to register for `op_name` before its kernels can be found: the strings are
 * the arguments of TF_OpDefinitionBuilderAddInput / AddOutput / AddAttr ("a: T1", "T1: quantizedtype",
 * "transpose_a: bool = false" ...), as the reference registers them (itex/core/ops/nn_ops.cc:1070-1127,1601-1772,
 * 3339-3600,4136-4325,4513-4760; itex/core/ops/fp8_ops.cc:22-61,124-143,192-226).  defined_by_plugin = 0 means the name
 * is an op TensorFlow defines itself (QuantizeV2, QuantizedConv2DWithBias..., _QuantizedMatMul ...) or one the reference
 * registers kernels for without a definition of its own: only kernels are registered for it.  For such a name the
 * strings are those of the twin op the reference defines with the same argument list (_ITEXQuantizeV2 for QuantizeV2
 * ...): the argument names serve TF_KernelBuilder_HostMemory, and an attr is read only if the node has it.
 * The pointers are to static storage. */
typedef struct itexb_op_def {
  const char* name;
  int32_t defined_by_plugin;
  int32_t num_inputs;
  const char* const* inputs;
  int32_t num_outputs;
  const char* const* outputs;
  int32_t num_attrs;
  const char* const* attrs;
} itexb_op_def_t;
ITEXB_API int itexb_op_def(const char* op_name, itexb_op_def_t* def);
ITEXB_API int itexb_op_create(const char* op_name, const itexb_attr_t* attrs, int num_attrs, itexb_op_t** op);
/* Compute enqueues on ctx->stream and returns without waiting (kernel_compute of itex/core/utils/op_kernel.h:859-917);
 * one Compute at a time per instance (mu_compute_, quantized_matmul_common.h:62), and the launches of one instance are
 * expected on one stream per device (calls from another stream are ordered behind the instance's cached uploads).
 * Errors a kernel can only report after it ran - a bounded device wait that expired - are kept in a per-instance
 * device status word and surface as ITEXB_ABORTED from the instance's NEXT itexb_op_compute (which then does not
 * run), from a Compute under ITEXB_SYNC_EXEC / ITEXB_VERBOSE (same call), or from itexb_op_check. */
ITEXB_API int itexb_op_compute(itexb_op_t* op, itexb_op_context_t* ctx);
/* Status of the launches this instance has made so far: ITEXB_OK, or ITEXB_ABORTED with the kernel role that gave up.
 * wait != 0 blocks until the work queued by the last Compute has finished; wait == 0 only looks at what has landed. */
ITEXB_API int itexb_op_check(itexb_op_t* op, int wait);
/* Frees the instance and its device buffers (stream-ordered behind its last launches).  A pending kernel error that
 * nobody collected is written to stderr. */
ITEXB_API void itexb_op_delete(itexb_op_t* op);

/* Graph-side routing (what a TF_InitGraph optimizer needs, free of TensorFlow types): should this stock-TensorFlow
 * INT8 node be replaced by one of this library's `_ITEX*` ops, and with which extra attrs?  Restates the reference's
 * rename table (itex/core/graph/native_layout/native_layout.cc:113-199), its predicate RewriteQuantize
 * (itex/core/graph/utils/layout_utils.cc:315-354: MIN_COMBINED never; MIN_FIRST Dequantize not on the GPU; SCALED only
 * with HALF_TO_EVEN) and its attr copiers (layout_utils.cc:471-542: data_format = "NHWC" and Tbias for the convolutions,
 * Tbias for the matmuls, dtype and classic_asymmetric_algorithm for QuantizeV2).  new_op == NULL: leave the node as it
 * is.  Otherwise the new node takes all attrs of the old one plus added[0 .. num_added) (an added attr replaces one of
 * the same name).  A node that lacks an attr the rule must read (mode; out_type; Toutput) is an INVALID_ARGUMENT. */
typedef struct itexb_rewrite_query {
  const char* op;
  const itexb_attr_t* attrs;
  int32_t num_attrs;
  int32_t on_gpu;                        /* the node is placed on this plugin's device */
  int32_t all_consumers_are_dequantize;  /* QuantizeV2: every consumer of output 0 is a Dequantize node */
} itexb_rewrite_query_t;
typedef struct itexb_rewrite_result {
  const char* new_op;
  int32_t num_added;
  itexb_attr_t added[4];
} itexb_rewrite_result_t;
ITEXB_API int itexb_rewrite_node(const itexb_rewrite_query_t* q, itexb_rewrite_result_t* r);
/* The table itself: rule `index` renames *from to *to; NOT_FOUND past the end. */
ITEXB_API int itexb_rewrite_rule(int index, const char** from, const char** to);

/* A ready-made context over the runtime above: outputs and temps come from
 * itexb_rt_allocate / itexb_rt_host_allocate.  Outputs stay valid until
 * itexb_simple_context_reset or _destroy.                                           */
typedef struct itexb_simple_context itexb_simple_context_t;
ITEXB_API int itexb_simple_context_create(int device_ordinal, itexb_stream_t stream, itexb_simple_context_t** c);
ITEXB_API itexb_op_context_t* itexb_simple_context_begin(itexb_simple_context_t* c, const itexb_tensor_t* inputs,
                                                         int num_inputs);
ITEXB_API int itexb_simple_context_num_outputs(itexb_simple_context_t* c);
ITEXB_API const itexb_tensor_t* itexb_simple_context_output(itexb_simple_context_t* c, int index);
ITEXB_API int itexb_simple_context_reset(itexb_simple_context_t* c);
ITEXB_API void itexb_simple_context_destroy(itexb_simple_context_t* c);

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* ITEXB200_H_ */
