/*
 * ctb200 -- C ABI of the B200 (sm_100a) tensor codec that stands in for the torch-CPU
 * codec path of compressed-tensors.
 *
 * Conventions shared by every entry point
 *   - plain C: raw device pointers, explicit sizes, dtype codes, a CUDA stream handle
 *     (`void *stream` is a cudaStream_t; NULL = the legacy default stream);
 *   - returns a ctb_status (0 = ok); never throws, never traps, never synchronises the
 *     host and, unless a function says otherwise, never allocates;
 *   - inputs are read-only, outputs are fully overwritten, buffers must not overlap;
 *   - tensors are dense row-major; leading dimensions are flattened so that every
 *     operand is a [rows, cols] matrix;
 *   - ctb_last_error_string() returns a thread-local description of the last failure.
 *
 * Citations name the reference function each entry point replaces, by path inside the
 * reference project (src/compressed_tensors/...):line.
 */
#ifndef CTB200_H
#define CTB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ctb_status {
    CTB_OK = 0,
    CTB_EINVAL_SHAPE = 1,  /* sizes that the reference rejects too (ValueError there) */
    CTB_EINVAL_DTYPE = 2,
    CTB_EINVAL_ALIGN = 3,
    CTB_EINVAL_NULL = 4,
    CTB_ETIMEOUT = 5,      /* a bounded device-side wait gave up */
    CTB_ECUDA = 6,         /* a CUDA runtime call failed; see ctb_last_error_string() */
    CTB_EUNSUPPORTED = 7   /* valid in the reference, not built here (NotImplementedError) */
} ctb_status;

typedef enum ctb_dtype {
    CTB_BF16 = 0,
    CTB_F16 = 1,
    CTB_F32 = 2,
    CTB_F64 = 3,
    CTB_I8 = 4,
    CTB_E4M3 = 5, /* float8_e4m3fn */
    CTB_U8 = 6,
    CTB_I32 = 7,
    CTB_I64 = 8
} ctb_dtype;

typedef enum ctb_qtype { CTB_QINT = 0, CTB_QFLOAT = 1 } ctb_qtype;

/* Third value of the `precision` argument of the rotation entry points (besides CTB_F64 and CTB_F32):
 * run the block-128 rotation on the tensor cores (tcgen05, bf16 operands, fp32 accumulators in TMEM).
 * Needs n = 128, bf16, forward, and tensors that are whole tiles of 128 x 128 elements. */
#define CTB_ROT_TENSOR 100

/* What a quantize / dequantize call stores or loads on the quantized side. */
typedef enum ctb_codec {
    CTB_CODE_DTYPE = 0,  /* one element per value in `q_dtype` (a float dtype, I8 or E4M3) */
    CTB_CODE_PACK32 = 1, /* int codes packed 32/num_bits per int32 word (pack_to_int32 layout) */
    CTB_CODE_FP4X2 = 2   /* e2m1 codes, two per byte, even column in the low nibble */
} ctb_codec;

/*
 * Geometry of one quantization problem.  The qparam (scale / zero point) that applies to
 * element (r, c) is  (r / row_group) * scale_row_stride + c / col_group, or, when a g_idx
 * column map is given,  (r / row_group) * scale_row_stride + g_idx[c].
 *   TENSOR:  col_group = cols, scale_row_stride = 0, row_group = 1
 *   CHANNEL / TOKEN: col_group = cols, scale_row_stride = 1
 *   GROUP / TENSOR_GROUP: col_group = group_size, scale_row_stride = cols / group_size
 *   BLOCK [bh, bw]: row_group = bh, col_group = bw, scale_row_stride = cols / bw
 */
typedef struct ctb_qdesc {
    int64_t rows, cols;
    int64_t col_group, row_group, scale_row_stride;
    int32_t qtype;     /* ctb_qtype */
    int32_t num_bits;  /* int: 1..8, float: 8 (e4m3) or 4 (e2m1) */
    int32_t x_dtype;   /* dtype of the dense side (input of quantize, output of dequantize) */
    int32_t scale_dtype;
    int32_t zp_dtype;  /* I8 or E4M3; ignored when zero_point is NULL */
    int32_t q_dtype;   /* dtype of the quantized side when codec == CTB_CODE_DTYPE */
    int32_t codec;     /* ctb_codec */
    int32_t reserved;
} ctb_qdesc;

const char *ctb_version(void);
const char *ctb_last_error_string(void);
/* Number of kernels this library has launched in the calling process (all threads). */
int64_t ctb_launch_count(void);

/* ---- quantize / dequantize / fake_quantize ------------------------------------------
 * quantization/lifecycle/forward.py:45-81 quantize, :455-487 _quantize and
 * quantization/quant_args.py:384-408 round_to_quantized_type:
 *   q = round(clamp(x / scale' + zero_point, qmin, qmax)),  scale' = scale or scale / global_scale,
 * every intermediate rounded to the dtype torch's promotion rules give it.
 * With codec PACK32 the codes go straight into pack_to_int32 words
 * (compressors/quantized_compressors/pack_quantized.py:88-145 compress_weight, :186-246);
 * with codec FP4X2 into pack_fp4_to_uint8 bytes
 * (compressors/quantized_compressors/fp4_quantized.py:84-106, :135-178).
 * g_idx (int32 [cols]) and global_scale (fp32 [1], device) may be NULL. */
int ctb_quantize(const ctb_qdesc *desc, const void *x, const void *scale, const void *zero_point,
                 const int32_t *g_idx, const float *global_scale, void *out, void *stream);

/* forward.py:85-153 dequantize, :491-514 _dequantize:  x = (q - zero_point) * scale'.
 * `q` is read through desc->codec (PACK32 = unpack_from_int32 fused in front,
 * pack_quantized.py:147-183; FP4X2 = unpack_fp4_from_uint8, fp4_quantized.py:108-123, :187-221);
 * the result is written in desc->x_dtype.  zero_point is always one int8/e4m3 per qparam. */
int ctb_dequantize(const ctb_qdesc *desc, const void *q, const void *scale, const void *zero_point,
                   const int32_t *g_idx, const float *global_scale, void *out, void *stream);

/* forward.py:157-189 fake_quantize: quantize then dequantize without leaving registers.
 * Input dtype desc->x_dtype, output dtype desc->q_dtype (a float dtype). */
int ctb_fake_quantize(const ctb_qdesc *desc, const void *x, const void *scale, const void *zero_point,
                      const int32_t *g_idx, const float *global_scale, void *out, void *stream);

/* ---- quantization parameters ----------------------------------------------------------
 * quantization/utils/helpers.py:149-205 compute_dynamic_scales_and_zp (the amin/amax part):
 * min and max over every [row_group x col_group] tile of x, written in x's dtype as
 * [rows/row_group, cols/col_group].  A tile that spans several thread blocks is combined
 * through `workspace` (device memory, ctb_minmax_workspace_bytes() bytes, contents ignored). */
int64_t ctb_minmax_workspace_bytes(int64_t rows, int64_t cols, int64_t row_group, int64_t col_group);
int ctb_minmax(const void *x, int32_t x_dtype, int64_t rows, int64_t cols, int64_t row_group,
               int64_t col_group, void *out_min, void *out_max, void *workspace, void *stream);

/* helpers.py:67-146 calculate_qparams over n (min, max) pairs of dtype `dtype`.
 * Scale is written in `dtype`, or in e4m3 for fp4 with a global scale (:103-120);
 * zero point in zp_dtype (I8 for int types, E4M3 for float types). */
int ctb_calculate_qparams(const void *min_vals, const void *max_vals, int32_t dtype, int64_t n,
                          int32_t qtype, int32_t num_bits, int32_t symmetric,
                          const float *global_scale, void *out_scale, void *out_zero_point,
                          int32_t zp_dtype, void *stream);

/* helpers.py:414-434 generate_gparam: 448*6 / max(|min|, |max|) computed in `dtype`, stored as fp32[1]. */
int ctb_generate_gparam(const void *min_val, const void *max_val, int32_t dtype, float *out,
                        void *stream);

/* quantization/utils/mxfp4_utils.py:43-72 round_to_power_2 (bf16 in, bf16 out), :75-97 generate_mxfp4_scales
 * (bf16 in, uint8 exponent out) and :25-40 convert_mxfp4_exp_scale (uint8 exponent in, bf16 / f16 / f32 out). */
int ctb_mxfp4_round_pow2(const void *x_bf16, int64_t n, void *out_bf16, void *stream);
int ctb_mxfp4_generate_scales(const void *x_bf16, int64_t n, uint8_t *out_exponent, void *stream);
int ctb_mxfp4_convert_scales(const uint8_t *exponent, int64_t n, int32_t out_dtype, void *out, void *stream);

/* ---- stand-alone packing ---------------------------------------------------------------
 * pack_quantized.py:186-246 pack_to_int32.  value is int8 [rows, cols] addressed with element
 * strides (row_stride, col_stride) so that packed_dim=0 is the same call on the transposed view;
 * out is int32 [rows, ceil(cols / (32/num_bits))] contiguous.  Pad fields are zero. */
int ctb_pack_int32(const int8_t *value, int64_t rows, int64_t cols, int64_t row_stride,
                   int64_t col_stride, int32_t num_bits, int32_t *out, void *stream);
/* pack_quantized.py:249-309 unpack_from_int32.  words int32 [rows, ceil(cols/pf)] addressed with
 * element strides; out int8 [rows, cols] contiguous. */
int ctb_unpack_int32(const int32_t *words, int64_t rows, int64_t cols, int64_t row_stride,
                     int64_t col_stride, int32_t num_bits, int8_t *out, void *stream);
/* fp4_quantized.py:135-178 pack_fp4_to_uint8: x [m, n] of `dtype` holding e2m1 grid values
 * -> uint8 [m, n/2]; odd n is CTB_EINVAL_SHAPE. */
int ctb_pack_fp4(const void *x, int32_t dtype, int64_t m, int64_t n, uint8_t *out, void *stream);
/* fp4_quantized.py:187-221 unpack_fp4_from_uint8 -> [m, n] of out_dtype. */
int ctb_unpack_fp4(const uint8_t *packed, int64_t m, int64_t n, void *out, int32_t out_dtype,
                   void *stream);
/* utils/helpers.py:302-313 pack_bitmasks: bool/uint8 [rows, cols] -> uint8 [rows, ceil(cols/8)],
 * column 8k+j in bit j of byte k. */
int ctb_pack_bitmasks(const uint8_t *bytemask, int64_t rows, int64_t cols, uint8_t *out, void *stream);
/* utils/helpers.py:316-339 unpack_bitmasks -> uint8 0/1 [rows, cols]. */
int ctb_unpack_bitmasks(const uint8_t *packed, int64_t rows, int64_t cols, uint8_t *out, void *stream);

/* ---- sparse codecs ---------------------------------------------------------------------
 * compressors/sparse_compressors/sparse_24_bitmask.py:227-260 get_24_bytemasks: keep-mask of the
 * two largest magnitudes in every run of 4 consecutive elements (flat view), ties resolved as
 * torch.topk does on CPU.  dtype: BF16 / F16 / F32 / I8 / E4M3 (ranked through its int8 view). */
int ctb_sparse24_mask(const void *x, int32_t dtype, int64_t numel, uint8_t *out_bytemask, void *stream);
/* sparse_24_bitmask.py:162-203 sparse24_bitmask_compress for cols % 8 == 0:
 * values [rows, cols/2] (same dtype as x) and bitmask uint8 [rows, ceil(cols/8)] in one pass. */
int ctb_sparse24_compress(const void *x, int32_t dtype, int64_t rows, int64_t cols, void *out_values,
                          uint8_t *out_bitmask, void *stream);
/* A stacked float-quantized + sparse-24-bitmask weight in one pass: per-channel static FP8 quantization
 * (compressors/quantized_compressors/naive_quantized.py:124-140 compress_weight ->
 * quantization/lifecycle/forward.py:462-489 _quantize to float8_e4m3fn) followed by
 * sparse_24_bitmask.py:162-203 on the e4m3 result, which is never written to memory.
 * x bf16 [rows, cols], cols % 8 == 0; scale bf16 [rows] (one per output channel); zero_point [rows] of
 * zp_dtype or NULL (the reference adds it before rounding, so even an all-zero one turns -0.0 into +0.0).
 * out_values e4m3 [rows, cols/2], out_bitmask uint8 [rows, cols/8]: bit-identical to ctb_quantize followed
 * by ctb_sparse24_compress. */
int ctb_quantize_fp8_sparse24(const void *x, const void *scale, const void *zero_point, int32_t zp_dtype,
                              int64_t rows, int64_t cols, void *out_values, uint8_t *out_bitmask, void *stream);
/* The inverse walk in one pass (model_compressor.py:580-611: sparse_24_bitmask.py:206-224 decompress, then
 * naive_quantized.py:113-140 decompress_weight -> forward.py:504-512 dequantize): kept e4m3 values [nvalues]
 * (rows*cols/2 for a two-per-four bitmask) + bitmask [rows, cols/8] + bf16 scale [rows] -> bf16 [rows, cols].
 * Any bitmask gives the result of ctb_sparse24_decompress followed by ctb_dequantize (a bitmask that is not
 * two-per-four takes the generic codec).  workspace: ctb_sparse24_dequantize_workspace_bytes. */
int64_t ctb_sparse24_dequantize_workspace_bytes(int64_t rows, int64_t cols);
int ctb_sparse24_decompress_dequantize_fp8(const void *values, int64_t nvalues, const uint8_t *bitmask, const void *scale,
                                           int64_t rows, int64_t cols, void *out, void *workspace, void *stream);
/* compressors/sparse_compressors/sparse_bitmask.py:131-149 bitmask_compress.
 * out_values needs room for rows*cols elements; the first *out_nnz (device int64) are valid,
 * row-major.  out_row_offsets is int64 [rows] (exclusive prefix of per-row counts).
 * Elements equal to zero (+0.0 and -0.0) are dropped; NaN is kept. */
/* `workspace`: ctb_bitmask_workspace_bytes(rows, cols) bytes of device scratch (contents ignored); with it the
 * codec runs as two kernels over flat 512-element tiles, one per warp and step (kept counts of every warp's
 * contiguous range of tiles, then the compaction with a running offset); NULL selects the row-by-row
 * count / scan / scatter path. */
int64_t ctb_bitmask_workspace_bytes(int64_t rows, int64_t cols);
/* ctb_bitmask_force_two_kernels(0) lets ctb_bitmask_compress, given a `workspace`, run tensors of up to 16384 tiles of
 * 8192 elements on a device with cooperative launches as ONE kernel that reads x from HBM once (bulk copies into shared
 * memory, per-tile counts exchanged through the workspace, every wait bounded; if a wait gives up, *out_nnz reads -1 and
 * the outputs are undefined).  The default (1) is the count + compaction pair of kernels, which is faster while the
 * tensor fits the L2 cache, and it is what a stream that is being captured into a CUDA graph always gets (the single
 * kernel tells its per-tile counts from stale scratch by a ticket chosen per launch call, which a replay would repeat).
 * Process-wide switch; no counterpart in the reference. */
void ctb_bitmask_force_two_kernels(int32_t on);
int ctb_bitmask_compress(const void *x, int32_t dtype, int64_t rows, int64_t cols, void *out_values,
                         uint8_t *out_bitmask, int64_t *out_row_offsets, int64_t *out_nnz,
                         void *workspace, void *stream);
/* The same compaction with the keep-mask given explicitly (uint8 0/1 [rows, cols]): the reference's
 * `tensor[bytemasks]` + pack_bitmasks (sparse_24_bitmask.py:192-203) for shapes the fused 2:4 kernel
 * does not take (cols % 8 != 0). */
int ctb_masked_compress(const void *x, const uint8_t *bytemask, int32_t dtype, int64_t rows, int64_t cols,
                        void *out_values, uint8_t *out_bitmask, int64_t *out_row_offsets,
                        int64_t *out_nnz, void *stream);
/* sparse_bitmask.py:152-169 bitmask_decompress and sparse_24_bitmask.py:206-224
 * sparse24_bitmask_decompress: zeros, then values scattered row-major to the set bits.
 * `workspace` is device scratch of ctb_bitmask_workspace_bytes(rows, cols) bytes (start offsets are rebuilt
 * from the bitmask; the reference does not consult row_offsets either). */
int ctb_bitmask_decompress(const void *values, const uint8_t *bitmask, int32_t dtype, int64_t rows,
                           int64_t cols, void *out, void *workspace, void *stream);

/* sparse_24_bitmask.py:206-224 sparse24_bitmask_decompress.  Same result as ctb_bitmask_decompress for any
 * bitmask.  `nvalues` is the number of elements `values` holds.  When it is at least rows * cols / 2 and the bitmask
 * keeps exactly two of every four columns (what the 2:4 compressor writes) a scan-free kernel does the work and the
 * generic kernels return at once; a shorter `values` is never read past its end: it takes the generic kernels
 * directly.  workspace: ctb_bitmask_workspace_bytes(). */
int ctb_sparse24_decompress(const void *values, int64_t nvalues, const uint8_t *bitmask, int32_t dtype,
                            int64_t rows, int64_t cols, void *out, void *workspace, void *stream);

/* No counterpart in the reference.  Same result as ctb_bitmask_decompress, for callers that cannot
 * allocate device memory where they decompress (a server whose memory went to a fixed arena at
 * start-up, a load hook running while something else owns the allocator): the per-row offsets live
 * in a 512 KiB array inside the library instead of caller scratch, which every GPU that loads the
 * library keeps until the process exits.  Limits and rules:
 *   - rows <= 65536, otherwise CTB_EINVAL_SHAPE;
 *   - calls no cudaMalloc / cudaFree and no allocating library routine;
 *   - the first call on each device looks the array's device address up (with that device
 *     current); make that first call before any stream capture;
 *   - all calls on a device share the array, so two calls that overlap on the GPU (different
 *     streams) race: keep calls of this entry point ordered on one stream or separate them with
 *     events. */
int ctb_bitmask_decompress_static(const void *values, const uint8_t *bitmask, int32_t dtype, int64_t rows,
                                  int64_t cols, void *out, void *stream);

/* ---- Hadamard rotation -------------------------------------------------------------------
 * transform/factory/hadamard.py:104-121 HadamardTransform.forward with
 * transform/utils/matrix.py:65-134 apply_transform_weight for torch.nn.Linear weights:
 *   side 0 (weight_input):  out = W @ Wh^T per n-column block,
 *   side 1 (weight_output): out = Wh^T @ W per n-row block,
 * Wh = diag(signs) @ H_n (Sylvester; signs int8 +-1 [n] or NULL = all +1; transform/utils/
 * hadamard.py:33-89), transposed when `inverse`; result / sqrt(n) cast to the dtype of W.
 * precision: CTB_F64 accumulates like the reference's offline path; CTB_F32 is the fast mode.
 * normalize = 0 leaves out the division by sqrt(n) (apply_transform_weight on its own, matrix.py:65).
 * n is a power of two: 8 .. 8192 for side 0 (16-byte aligned buffers), up to 8192 for side 1; a head_dim-sized
 * block (128) or a whole hidden dimension (4096, 8192).  Other sizes return CTB_EUNSUPPORTED. */
int ctb_hadamard(const void *x, int32_t dtype, int64_t rows, int64_t cols, int32_t n,
                 const int8_t *signs, int32_t inverse, int32_t side, int32_t precision,
                 int32_t normalize, void *out, void *stream);

/* ---- Marlin-24 packing (compressors/sparse_quantized_compressors/marlin_24.py:124-273) --------------------
 * utils/semi_structured_conversions.py:79-209 sparse_semi_structured_from_dense_cutlass for a 16-bit dense dtype:
 * dense [rows, cols] (f16 / bf16 values, or int8 codes standing for the 16-bit tensor of the same integers) ->
 * out_sparse [rows, cols/2] (same element type) and out_meta int16 [rows, cols/16] in CUTLASS's reordered layout. */
int ctb_cutlass24_compress(const void *dense, int32_t dtype, int64_t rows, int64_t cols, void *out_sparse,
                           int16_t *out_meta, void *stream);
/* utils/semi_structured_conversions.py:216-308 sparse_semi_structured_to_dense_cutlass (int16 meta): the inverse,
 * sparse [rows, cols_sparse] + reordered meta [rows, cols_sparse/8] -> dense [rows, 2 * cols_sparse]. */
int ctb_cutlass24_decompress(const void *sparse, const int16_t *meta, int32_t dtype, int64_t rows, int64_t cols_sparse,
                             void *out_dense, void *stream);
/* marlin_24.py:208-249 marlin_permute_weights + pack_weight_24 (including the transpose and the shift to unsigned
 * of :186-193): sparse int8 codes [size_n, size_k] -> int32 [size_k/16, size_n*16/(32/num_bits)]. */
int ctb_marlin24_pack_weight(const int8_t *sparse, int64_t size_n, int64_t size_k, int32_t num_bits, int32_t *out,
                             void *stream);
/* marlin_24.py:252-273 pack_scales_24 (including the transpose of :188): 16-bit scales [size_n, groups] ->
 * [groups, size_n]; `grouped` != 0 selects the group permutation (group size below size_k). */
int ctb_marlin24_pack_scales(const void *scale, int64_t size_n, int64_t groups, int32_t grouped, void *out,
                             void *stream);

/* ---- fused calibrate + quantize + pack (single pass over the dense tensor) -------------------
 * Symmetric min-max calibration (helpers.py:67-146 with the group's own amin/amax) followed by
 * ctb_quantize with the scales it produced.  out_scale is written in desc->scale_dtype, which
 * must equal desc->x_dtype; zero points are all zero and not written.
 * With n > 0 the weight_input Hadamard rotation of ctb_hadamard (side 0) is applied in front,
 * rounding to x_dtype in between exactly as the two separate calls would.
 * codec CTB_CODE_DTYPE with q_dtype CTB_BF16 selects dynamic fake quantization (forward.py:415-452 forward_quantize
 * with args.dynamic, per token / channel): the output is ctb_fake_quantize with the row's own symmetric qparams;
 * built for whole rows (col_group == cols) of up to 8192 int8 / fp8-quantized elements. */
int ctb_absmax_quantize(const ctb_qdesc *desc, const void *x, const float *global_scale,
                        void *out_scale, void *out, int32_t hadamard_n, const int8_t *signs,
                        int32_t precision, void *stream);

/* ---- whole-shard batches ------------------------------------------------------------------------
 * The reference walks a state dict one tensor at a time (compressors/quantized_compressors/base.py:91,
 * model_compressors/model_compressor.py:469, :558).  These entry points take the whole list and run it
 * as ONE grid, so small tensors cost neither a launch nor a kernel tail each.  Results are identical to
 * the per-tensor calls.  All tensors: bf16, cols % 128 == 0, symmetric int4, group_size 128. */
typedef struct ctb_tensor_ref {
    const void *in;  /* compress: dense bf16 weight;        decompress: packed int32 words      */
    void *out;       /* compress: packed int32 words;       decompress: dense bf16 weight       */
    void *scale;     /* bf16 [rows, cols/128]: written by compress, read by decompress           */
    int64_t rows, cols; /* of the dense weight */
} ctb_tensor_ref;

/* ctb_absmax_quantize(hadamard_n = 128, group 128, PACK32) for every tensor of the table. */
/* device_status (int32 the device can write: device memory, or page-locked host memory, which the host can then
 * read without a copy; may be NULL) receives CTB_ETIMEOUT if a bounded wait inside the tensor-core kernel gives up;
 * it is left untouched otherwise. */
int ctb_rotate_quantize_int4_batch(const ctb_tensor_ref *tensors, int32_t count, const int8_t *signs,
                                   int32_t precision, int32_t *device_status, void *stream);
/* The CTB_ROT_TENSOR form of the call above with the bound of its device-side waits given by the caller
 * (spin_cycles, in SM clocks; the default is about a second) and, for skip_tile >= 0, with the copy of that one
 * tile left out, so that the wait for it runs out: the kernel then drains what it has in flight, frees its
 * tensor memory, returns, and *device_status reads CTB_ETIMEOUT.  This is how the error path is exercised
 * without a fault; the outputs of such a call are undefined.  No counterpart in the reference. */
int ctb_rotate_quantize_int4_batch_bounded(const ctb_tensor_ref *tensors, int32_t count, const int8_t *signs,
                                           int32_t *device_status, int64_t spin_cycles, int32_t skip_tile,
                                           void *stream);
/* ctb_quantize(codec PACK32, num_bits 4, group 128, bf16 scale GIVEN in t.scale, no zero point) for every tensor:
 * the compress walk of a model that was calibrated beforehand (quantized_compressors/base.py:91-122 calling
 * pack_quantized.py:88-145 per weight).  t.in = dense bf16 weight, t.out = int32 words, t.scale is read. */
int ctb_quantize_pack_int4_batch(const ctb_tensor_ref *tensors, int32_t count, void *stream);
/* ctb_dequantize(codec PACK32, num_bits 4, group 128, bf16 scale, no zero point) for every tensor. */
int ctb_unpack_dequantize_int4_batch(const ctb_tensor_ref *tensors, int32_t count, void *stream);

/* Whole-shard FP8: ctb_quantize(q_dtype E4M3, CHANNEL strategy, static bf16 scale, one per row) for every tensor of
 * the table: the compress walk of a calibrated FP8 model (quantized_compressors/base.py:91-122 calling
 * naive_quantized.py:74-110 per weight).  t.in = dense bf16 weight [rows, cols], cols % 8 == 0, t.out = e4m3
 * [rows, cols], t.scale = bf16 [rows] (read).  zero_points: NULL, or `count` device pointers ([rows] of zp_dtype each,
 * NULL entries allowed) for modules that carry a zero point (the reference adds it before rounding). */
int ctb_quantize_fp8_channel_batch(const ctb_tensor_ref *tensors, int32_t count, const void *const *zero_points,
                                   int32_t zp_dtype, void *stream);
/* ctb_dequantize(E4M3 codes, CHANNEL strategy, bf16 scale, no zero point) for every tensor (base.py:190-237 calling
 * naive_quantized.py:113-140).  t.in = e4m3 [rows, cols], t.out = bf16 [rows, cols], t.scale = bf16 [rows]. */
int ctb_dequantize_fp8_channel_batch(const ctb_tensor_ref *tensors, int32_t count, void *stream);

/* Whole-shard NVFP4: ctb_quantize(codec FP4X2, num_bits 4, group 16, e4m3 scales, fp32 global scale) for every tensor
 * of the table (quantized_compressors/base.py:91-122 calling fp4_quantized.py:84-105 per weight).  t.in = dense bf16
 * weight [rows, cols], cols % 16 == 0, t.out = uint8 [rows, cols/2], t.scale = e4m3 [rows, cols/16] (read).
 * global_scales: `count` device pointers to fp32 [1].  zero_points: NULL, or `count` device pointers
 * ([rows, cols/16] of zp_dtype each, NULL entries allowed). */
int ctb_quantize_fp4_g16_batch(const ctb_tensor_ref *tensors, int32_t count, const void *const *global_scales,
                               const void *const *zero_points, int32_t zp_dtype, void *stream);
/* ctb_dequantize(codec FP4X2, group 16, e4m3 scales, fp32 global scale, no zero point) for every tensor
 * (base.py:190-237 calling fp4_quantized.py:108-132).  t.in = uint8 [rows, cols/2], t.out = bf16 [rows, cols]. */
int ctb_dequantize_fp4_g16_batch(const ctb_tensor_ref *tensors, int32_t count, const void *const *global_scales,
                                 void *stream);

/* ---- staging memory of the host <-> device pipeline ------------------------------------------------------
 * The reference keeps a state dict in ordinary host memory and never leaves the CPU
 * (compressors/quantized_compressors/base.py:74, :125 compression_device="cpu").  Here host-resident tensors are
 * streamed through the GPU, which needs page-locked buffers on the host side; these two calls allocate and free
 * them (cudaHostAlloc, portable) so that the caller can pool them.  No counterpart in the reference. */
int ctb_pinned_alloc(int64_t nbytes, void **out);
int ctb_pinned_free(void *ptr);

#ifdef __cplusplus
}
#endif
#endif /* CTB200_H */
