/*
 * nnq.h -- C ABI of libnnq_b200: block-quantized weight x activation products on
 * NVIDIA B200 (sm_100a), behind the seams the alabsystems/nn reference exposes for
 * this path. Each entry point names the reference interface it replaces (paths are
 * relative to the reference repository root). A Rust shim implementing
 * `GpuBackend::matmul` / `quantized_linear` binds exactly these symbols.
 *
 * Conventions
 *   - Plain C types only. Device pointers are CUDA device addresses; `stream` is a
 *     cudaStream_t passed as void* (NULL = the legacy default stream).
 *   - Every call returns an nnq_status. Nothing throws, aborts or traps the device;
 *     nnq_last_error(ctx) gives the message of the last failing call on that context.
 *   - Weights are [N, K] = [out_features, in_features], row-major, quantization blocks
 *     running along K and never crossing a row, exactly as the reference stores them
 *     (crates/nn-core/src/dyn_tensor/quantized_matmul.rs:198-203).
 *   - The library owns nnq_weight objects (a device copy, possibly re-tiled for the
 *     kernels; the byte count is preserved). The caller owns activation / output
 *     buffers and the stream.
 *   - A context is bound to one device. Calls on one context from several host threads
 *     must be serialised by the caller; distinct contexts are independent.
 */
#ifndef NNQ_H
#define NNQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define NNQ_API __attribute__((visibility("default")))
#else
#define NNQ_API
#endif

#define NNQ_VERSION_MAJOR 0
#define NNQ_VERSION_MINOR 1

typedef struct nnq_ctx nnq_ctx;
typedef struct nnq_weight nnq_weight;
typedef struct nnq_moe nnq_moe;
typedef struct nnq_comm nnq_comm;

/* Status codes. The first group mirrors QuantizedMatmulError
 * (crates/nn-core/src/dyn_tensor/quantized_matmul.rs:30-76) and the storage
 * validation errors of QuantizedStorage::new
 * (crates/nn-core/src/dyn_tensor/quantized.rs:118-139); the second group mirrors
 * BackendErrorKind (crates/nn-core/src/error.rs:48-93). */
typedef enum nnq_status {
    NNQ_OK = 0,
    NNQ_ERR_INVALID_ARG = 1,      /* null pointer, negative size, unknown enum value      */
    NNQ_ERR_NOT_QUANTIZED = 2,    /* QuantizedMatmulError::NotQuantized                    */
    NNQ_ERR_WRONG_QUANT_TYPE = 3, /* QuantizedMatmulError::WrongQuantType                  */
    NNQ_ERR_SHAPE_MISMATCH = 4,   /* QuantizedMatmulError::ShapeMismatch (input K != W K)  */
    NNQ_ERR_WEIGHT_RANK = 5,      /* QuantizedMatmulError::WeightRank                      */
    NNQ_ERR_BIAS_MISMATCH = 6,    /* QuantizedMatmulError::BiasMismatch                    */
    NNQ_ERR_INVALID_SHAPE = 7,    /* TensorError::InvalidShape: elements % block != 0      */
    NNQ_ERR_DATA_LENGTH = 8,      /* TensorError::DataLengthMismatch: bytes != blocks*size */
    NNQ_ERR_RANK_MISMATCH = 9,    /* TensorError::RankMismatch: input rank < 2             */
    NNQ_ERR_UNSUPPORTED = 10,     /* TensorError::Unsupported                              */
    NNQ_ERR_VALUE_OUT_OF_RANGE = 11, /* TensorError::ValueOutOfRange: non-finite encoder input */
    NNQ_ERR_OUT_OF_MEMORY = 20,   /* BackendErrorKind::OutOfMemory                         */
    NNQ_ERR_DISPATCH_FAILED = 21, /* BackendErrorKind::DispatchFailed (launch / CUDA error)*/
    NNQ_ERR_TIMEOUT = 22,         /* BackendErrorKind::Timeout (a bounded device wait ran out) */
    NNQ_ERR_NO_DEVICE = 23,       /* no CUDA device / not an sm_100 device                 */
    NNQ_ERR_OTHER = 24            /* BackendErrorKind::Other                               */
} nnq_status;

/* Weight formats. Q4_0/Q4_1/Q8_0 are nn-core's QuantType
 * (crates/nn-core/src/dyn_tensor/quantized.rs:28-56); Q4_K/Q6_K are the nn-gguf block
 * layouts (crates/nn-gguf/src/dequant.rs:335-398,415-459); Q4_K_GGML is nn-core's
 * BlockQ4K decode of the same 144-byte block
 * (crates/nn-core/src/layers/quantized/linear.rs:63-92); the MXFP4 variants are
 * nn-core's Mxfp4Block (mxfp4.rs:73-78), the [N,K/2]+[N,K/32] buffers of the
 * reference's GPU kernel contract (crates/nn-metal/src/mxfp4_gemm_msl.rs:47-61) and
 * nn-gptoss's Mxfp4Tensor (crates/nn-gptoss/src/quantize.rs:55-62). */
typedef enum nnq_format {
    NNQ_Q4_0 = 0,
    NNQ_Q4_1 = 1,
    NNQ_Q8_0 = 2,
    NNQ_Q4_K = 3,
    NNQ_Q4_K_GGML = 4,
    NNQ_Q6_K = 5,
    NNQ_MXFP4_CORE = 6,
    NNQ_MXFP4_SPLIT = 7,
    NNQ_MXFP4_GPTOSS = 8,
    /* the other nn-gguf block decoders (crates/nn-gguf/src/dequant.rs:241-316,476-684): dequantization
     * and nnq_linear on the row kernel / tensor path; no tiled layout, not accepted by nnq_moe_create */
    NNQ_Q5_0 = 9,
    NNQ_Q5_1 = 10,
    NNQ_Q2_K = 11,
    NNQ_Q3_K = 12,
    NNQ_Q5_K = 13,
    /* unquantized weights behind the same entry points: f32 / bf16 [N, K] row-major, handled as
     * "blocks" of 32 consecutive values (K a multiple of 32). The dense branch of Linear::forward
     * (crates/nn-core/src/layers/core_layers.rs:118-143) and the unquantized experts of
     * GptOssMoeBlock::forward / fused_moe_forward (crates/nn-gptoss/src/layers.rs:254,
     * crates/nn-gptoss/src/moe_dispatch.rs:50). */
    NNQ_F32_DENSE = 14,
    NNQ_BF16_DENSE = 15,
    NNQ_FORMAT_COUNT = 16
} nnq_format;

typedef enum nnq_dtype { NNQ_F32 = 0, NNQ_BF16 = 1 } nnq_dtype;

/* Kernel selection for nnq_linear. AUTO picks per shape from measured crossovers: M = 1 the
 * streaming skinny kernel (Q4_K), M > 16 (M >= 5 with bf16 activations) the tensor-core tile
 * pipeline (K a multiple of 64; weights and activations rounded to bf16),
 * otherwise the portable row kernel. The other values force one
 * path (tests and measurements use them). */
typedef enum nnq_path {
    NNQ_PATH_AUTO = 0,
    NNQ_PATH_GENERIC = 1, /* portable dequant-fused row kernel on the raw block layout */
    NNQ_PATH_SKINNY = 2,  /* M <= 16: tiled layout, mma-based streaming kernel           */
    NNQ_PATH_TENSOR = 3   /* M >= 128: TMA + tcgen05/TMEM tile pipeline                  */
} nnq_path;

/* ---- library / context ---------------------------------------------------------- */

/* Library version as major*1000 + minor. */
NNQ_API int nnq_version(void);

/* Human-readable name of a status code (static string). */
NNQ_API const char *nnq_status_str(nnq_status s);

/* Block geometry of a format: weights per block, bytes per block in the main buffer,
 * bytes per block in the separate scale buffer (non-zero only for the split MXFP4
 * layouts). Replaces GgufDType::{block_size,type_size}
 * (crates/nn-gguf/src/dequant.rs:84-114) and QuantType::{block_size,block_bytes}
 * (crates/nn-core/src/dyn_tensor/quantized.rs:58-76). */
NNQ_API nnq_status nnq_format_geometry(nnq_format fmt, int *block_elems, int *block_bytes,
                               int *scale_bytes);

/* Create / destroy a context on CUDA device `device`. Replaces
 * init_cuda_runtime(device_ordinal) (crates/nn-cuda/src/dyn_tensor_cuda.rs:117) and
 * the backend registration of crates/nn-core/src/dyn_tensor/gpu.rs:156-162. */
NNQ_API nnq_status nnq_init(int device, nnq_ctx **out);
NNQ_API void nnq_destroy(nnq_ctx *ctx);

/* Message of the last failing call on this context ("" if none). */
NNQ_API const char *nnq_last_error(const nnq_ctx *ctx);

/* Force a kernel path for subsequent nnq_linear calls on this context. */
NNQ_API nnq_status nnq_set_path(nnq_ctx *ctx, nnq_path path);

/* Reads and clears the device-side status word that kernels set when a bounded wait
 * runs out or an internal check fails. Synchronises `stream`. NNQ_OK when clear. */
NNQ_API nnq_status nnq_device_status(nnq_ctx *ctx, void *stream);

/* ---- weights --------------------------------------------------------------------- */

/* Wrap raw quantized blocks of an [N, K] weight. `data` (and `scales` for the split
 * MXFP4 layouts, else NULL/0) may be host or device memory; the bytes are copied.
 * Validation follows QuantizedStorage::new: N*K must be a multiple of the block size
 * (NNQ_ERR_INVALID_SHAPE), K must be a multiple of it too so that blocks do not cross
 * rows, and nbytes must equal blocks * block_bytes (NNQ_ERR_DATA_LENGTH).
 * Replaces DynTensor::from_quantized (crates/nn-core/src/dyn_tensor/quantized.rs:270)
 * plus GpuBackend::to_gpu (crates/nn-core/src/dyn_tensor/gpu.rs:46-139). */
NNQ_API nnq_status nnq_weight_create(nnq_ctx *ctx, nnq_format fmt, const void *data, size_t nbytes,
                             const void *scales, size_t scales_nbytes, int64_t n, int64_t k,
                             nnq_weight **out);

/* Tensor-parallel shard of an [N, K] weight given as raw bytes (host or device).
 * axis 0 (column-parallel): rows [rank*N/world, (rank+1)*N/world).
 * axis 1 (row-parallel): whole units [rank*U/world, (rank+1)*U/world) of every row, gathered
 * into a contiguous [N, K_rank] weight; a unit is 256 weights when K is a multiple of 256 (every
 * shard then keeps a tiled layout), else one block. The shards may differ by one unit (K = 25600
 * over 8 ranks: 13 or 12 super-blocks); nnq_weight_info gives a shard's K. Rows (axis 0) must
 * split evenly, else NNQ_ERR_INVALID_SHAPE. No counterpart in the reference, which runs on one
 * device. */
NNQ_API nnq_status nnq_weight_create_shard(nnq_ctx *ctx, nnq_format fmt, const void *data, size_t nbytes,
                                   const void *scales, size_t scales_nbytes, int64_t n,
                                   int64_t k, int axis, int rank, int world, nnq_weight **out);

NNQ_API void nnq_weight_destroy(nnq_weight *w);

/* Shape, format and stored byte counts of a weight (any out pointer may be NULL). */
NNQ_API nnq_status nnq_weight_info(const nnq_weight *w, nnq_format *fmt, int64_t *n, int64_t *k,
                           size_t *nbytes, size_t *scales_nbytes);

/* ---- quantization (f32 -> blocks) --------------------------------------------------- */

/* Encode `num_elements` f32 values resident on the device into blocks, byte-identical to the
 * reference's CPU encoders; the last block is padded with zeros as the reference pads it.
 *   NNQ_Q4_K_GGML    BlockQ4K::quantize behind QLinear::from_linear
 *                    (crates/nn-core/src/layers/quantized/linear.rs:95-162,195-254,309-343)
 *   NNQ_MXFP4_CORE   quantize_tensor / quantize_block
 *                    (crates/nn-core/src/layers/quantized/mxfp4.rs:183-207,307-329)
 *   NNQ_MXFP4_GPTOSS Mxfp4Tensor::quantize (crates/nn-gptoss/src/quantize.rs:122-153);
 *                    `scales_dev` receives one byte per block
 * Other formats: NNQ_ERR_UNSUPPORTED (the reference has no encoder for them).
 * `dst_dev` must be 16-byte aligned and hold blocks * block bytes (nnq_format_geometry);
 * *blocks (optional) receives the block count. A non-finite input is
 * NNQ_ERR_VALUE_OUT_OF_RANGE where the reference returns ValueOutOfRange (the nn-gptoss
 * encoder encodes it as zero instead). The call waits for the stream: encoding is a
 * load-time step. */
NNQ_API nnq_status nnq_quantize(nnq_ctx *ctx, nnq_format fmt, const float *src_dev, int64_t num_elements,
                                void *dst_dev, size_t dst_nbytes, void *scales_dev, size_t scales_nbytes,
                                int64_t *blocks, void *stream);

/* ---- INT8 per-channel weights (W8A16) ------------------------------------------------ */

/* Buffers follow the reference's GPU kernel contract (crates/nn-metal/src/int8_gemm_msl.rs:35-52):
 * W uint8 [N, K] read as signed bytes, scale f32 [N], zero_point int32 [N];
 * w = (f32(q) - f32(zero_point)) * scale. All pointers are device pointers.
 *
 * nnq_int8_quantize_per_channel: quantize_per_channel + compute_channel_params
 * (crates/nn-core/src/layers/quantized/int8.rs:82-137,187-221); mode 0 = Int8Mode::Symmetric,
 * 1 = Asymmetric; byte-identical outputs; a non-finite weight is NNQ_ERR_VALUE_OUT_OF_RANGE.
 * Waits for the stream (a load-time step).
 * nnq_int8_dequantize_per_channel: dequantize_per_channel (int8.rs:146-185), bit-identical.
 * nnq_int8_linear: Int8Linear::forward (int8_linear.rs:175-213) without materialising the f32
 * weight: y[M, N] = x[M, K] . w^T (+ bias), f32 accumulation. Four tokens share one pass
 * over the weights; larger M repeats the pass. */
NNQ_API nnq_status nnq_int8_quantize_per_channel(nnq_ctx *ctx, const float *w_dev, int64_t n, int64_t k, int mode,
                                                 void *q_dev, float *scale_dev, int32_t *zp_dev, void *stream);
NNQ_API nnq_status nnq_int8_dequantize_per_channel(nnq_ctx *ctx, const void *q_dev, const float *scale_dev,
                                                   const int32_t *zp_dev, int64_t n, int64_t k, float *dst_dev,
                                                   void *stream);
NNQ_API nnq_status nnq_int8_linear(nnq_ctx *ctx, const void *q_dev, const float *scale_dev, const int32_t *zp_dev,
                                   int64_t n, int64_t k, const void *x_dev, nnq_dtype x_dt, int64_t m,
                                   const float *bias_dev, void *y_dev, nnq_dtype y_dt, void *stream);

/* ---- INT4 / INT8 weights with per-group scales; GPTQ / AWQ packed weights ---------- */

/* The reference's QuantizedTensor (crates/nn-core/src/layers/quantized/weight_quant.rs:153-165):
 * codes for a weight [N, K], int8 one per byte, int4 two per byte over the flat index (even
 * index in the low nibble, two's complement); scale f32 and zero_point int32 per group of
 * `group_size` consecutive weights of a row, [N * K / group_size] each; w = (f32(code) -
 * f32(zp)) * scale. All pointers are device pointers.
 *
 * nnq_group_quantize: quantize_per_group + compute_group_params (weight_quant.rs:232-365).
 * bits 4 or 8; symmetric != 0: scale = max|w| / 7 (127), zero point 0; else scale = (max - min) /
 * 15 (255), zero point = round(qmin - min / scale). q_dev receives N*K bytes (int8) or
 * (N*K + 1) / 2 (int4). group_size 0 and a non-finite weight: NNQ_ERR_VALUE_OUT_OF_RANGE;
 * group_size not dividing K: NNQ_ERR_SHAPE_MISMATCH. Same codes, scales and zero points as the
 * reference, bit for bit. Waits for the stream (a load-time step).
 * nnq_group_dequantize: dequantize (weight_quant.rs:381-412) to f32 [N, K], bit-identical. */
NNQ_API nnq_status nnq_group_quantize(nnq_ctx *ctx, const float *w_dev, int64_t n, int64_t k, int bits, int64_t group_size,
                                      int symmetric, void *q_dev, float *scale_dev, int32_t *zp_dev, void *stream);
NNQ_API nnq_status nnq_group_dequantize(nnq_ctx *ctx, const void *q_dev, const float *scale_dev, const int32_t *zp_dev,
                                        int64_t n, int64_t k, int bits, int64_t group_size, float *dst_dev, void *stream);

/* A group-quantized weight resident on the device, in one layout for both sources: codes row-major
 * [N, K], scale and zero point f32 [N, groups]. The inputs are copied (per-group form) or repacked
 * (GPTQ / AWQ); the caller's buffers are not referenced afterwards. Creation waits for the stream
 * and reserves the context's bf16 scratch for the large-batch product (load-time steps).
 *
 * nnq_gq_create_per_group: from the fields of a QuantizedTensor (above).
 * nnq_gq_create_gptq: load_gptq_linear / load_awq_linear (gptq_loader.rs:329-351,
 * awq_loader.rs:74-96): qweight u32 [K / 8, N] (bits [4i+3 : 4i] of a word = the i-th of eight
 * consecutive in-features), scales f32 [groups, N], qzeros u32 [groups, N / 8] (eight consecutive
 * out-features per word), group = in-feature / group_size, w[n][k] = (q - zero) * scale. groups must
 * equal ceil(K / group_size) (NNQ_ERR_DATA_LENGTH); K and N multiples of 8 (NNQ_ERR_SHAPE_MISMATCH).
 * The reference decodes to f32 at load and multiplies dense; here the 4-bit codes stay packed. */
typedef struct nnq_gq_weight nnq_gq_weight;
NNQ_API nnq_status nnq_gq_create_per_group(nnq_ctx *ctx, const void *q_dev, const float *scale_dev, const int32_t *zp_dev,
                                           int64_t n, int64_t k, int bits, int64_t group_size, void *stream,
                                           nnq_gq_weight **out);
NNQ_API nnq_status nnq_gq_create_gptq(nnq_ctx *ctx, const uint32_t *qweight_dev, const float *scales_dev,
                                      const uint32_t *qzeros_dev, int64_t n, int64_t k, int64_t groups, int64_t group_size,
                                      void *stream, nnq_gq_weight **out);
/* Any out pointer may be NULL. *streaming: 1 when one-token products run the 16-byte streaming
 * kernel (K % 32 == 0, group_size % 8 == 0, |zero point| < 4e6), 0 for the element-wise kernel. */
NNQ_API nnq_status nnq_gq_info(const nnq_gq_weight *w, int64_t *n, int64_t *k, int *bits, int64_t *group_size,
                               int64_t *groups, int *streaming);
/* f32 [N, K], bit-identical to dequantize (weight_quant.rs:381-412) / to the weight of
 * load_gptq_linear (dequantize_gptq then transpose, gptq_loader.rs:139-187,342). */
NNQ_API nnq_status nnq_gq_dequantize(nnq_gq_weight *w, float *dst_dev, void *stream);
/* quantized_matmul (weight_quant.rs:451-473) and GptqLinear::forward (gptq_loader.rs:283-311):
 * y[M, N] = x[M, K] . w^T (+ bias), f32 accumulation. M <= 16: codes streamed once per four
 * tokens (f32 bar); larger M with K % 64 == 0: one decode to bf16, then the tensor-core product
 * (bf16 bar, as the other formats). Allocates nothing and does not synchronise. */
NNQ_API nnq_status nnq_gq_linear(nnq_gq_weight *w, const void *x_dev, nnq_dtype x_dt, int64_t m, const float *bias_dev,
                                 void *y_dev, nnq_dtype y_dt, void *stream);
NNQ_API void nnq_gq_destroy(nnq_gq_weight *w);

/* unpack_gptq_qweight (gptq_loader.rs:69-91; unpack_awq_qweight, awq_loader.rs:54-56, is the same
 * function): u32 [rows, cols] -> f32 [8 * rows, cols], values 0..15.
 * unpack_gptq_qzeros (gptq_loader.rs:101-123): u32 [groups, cols] -> f32 [groups, 8 * cols].
 * dequantize_gptq (gptq_loader.rs:139-187): q, dst f32 [K, N]; scales, zeros f32 [groups, N];
 * dst[i][j] = (q[i][j] - zeros[i / group_size][j]) * scales[i / group_size][j]; groups must equal
 * ceil(K / group_size) (NNQ_ERR_DATA_LENGTH). */
NNQ_API nnq_status nnq_gptq_unpack_qweight(nnq_ctx *ctx, const uint32_t *packed_dev, int64_t rows, int64_t cols,
                                           float *dst_dev, void *stream);
NNQ_API nnq_status nnq_gptq_unpack_qzeros(nnq_ctx *ctx, const uint32_t *packed_dev, int64_t groups, int64_t cols,
                                          float *dst_dev, void *stream);
NNQ_API nnq_status nnq_gptq_dequantize(nnq_ctx *ctx, const float *q_dev, const float *scales_dev, const float *zeros_dev,
                                       int64_t k, int64_t n, int64_t groups, int64_t group_size, float *dst_dev,
                                       void *stream);

/* ---- dequantization (bit-exact gate) ---------------------------------------------- */

/* Dequantize a weight to f32 [N, K] on the device. Bit-identical to the reference's
 * CPU decoders. Replaces DynTensor::dequantize
 * (crates/nn-core/src/dyn_tensor/quantized.rs:285-294) and QLinear::dequantize
 * (crates/nn-core/src/layers/quantized/linear.rs:345-353). */
NNQ_API nnq_status nnq_dequantize(nnq_ctx *ctx, const nnq_weight *w, float *dst_dev, void *stream);

/* Dequantize raw blocks resident on the device: `num_elements` values from `nbytes`
 * bytes; as in the reference a short buffer decodes only the whole blocks present.
 * *decoded (optional) receives the number of values written. Replaces
 * dequantize_q8_0 / dequantize_q4_k / dequantize_q6_k and the dtype dispatch of
 * GgufFile::read_tensor_f32 (crates/nn-gguf/src/dequant.rs:123-139,178-196,335-398,
 * 415-459; crates/nn-gguf/src/reader.rs:253-284), Mxfp4 dequantize_tensor
 * (crates/nn-core/src/layers/quantized/mxfp4.rs:335-348) and Mxfp4Tensor::dequantize
 * (crates/nn-gptoss/src/quantize.rs:167-188). */
NNQ_API nnq_status nnq_dequantize_raw(nnq_ctx *ctx, nnq_format fmt, const void *src_dev, size_t nbytes,
                              const void *scales_dev, size_t scales_nbytes, int64_t num_elements,
                              float *dst_dev, int64_t *decoded, void *stream);

/* ---- the product ------------------------------------------------------------------ */

/* y[M, N] = x[M, K] * W^T (+ bias[N]); x and y on the device, contiguous, row-major;
 * x_dt / y_dt in {F32, BF16}; accumulation in f32. M = product of all leading
 * dimensions of the reference's [.., M, K] input. bias may be NULL.
 * Replaces quantized_matmul_q4_0 / quantized_matmul_q8_0 / quantized_linear
 * (crates/nn-core/src/dyn_tensor/quantized_matmul.rs:296,335,367), QLinear::forward
 * (crates/nn-core/src/layers/quantized/linear.rs:366-399), the quantized branch of
 * DynTensor::matmul (crates/nn-core/src/dyn_tensor/ops/mod.rs:284-297) with
 * GpuBackend::matmul (crates/nn-core/src/dyn_tensor/gpu.rs:76), and the MXFP4 linear
 * kernel contract (crates/nn-metal/src/compiled_model_kernel_spec_mxfp4.rs:76-104). */
NNQ_API nnq_status nnq_linear(nnq_ctx *ctx, const nnq_weight *w, const void *x_dev, nnq_dtype x_dt,
                      int64_t m, const float *bias_dev, void *y_dev, nnq_dtype y_dt,
                      void *stream);

/* Same product with HOST activations and outputs: copies x (and bias) in, runs
 * nnq_linear, copies y out and synchronises. This is the shape of the reference's own
 * call, whose DynTensors live in host memory (quantized_linear(&input, &weight, bias)).
 * Staging buffers are owned by the context and grow on demand. */
NNQ_API nnq_status nnq_linear_host(nnq_ctx *ctx, const nnq_weight *w, const void *x_host, nnq_dtype x_dt,
                           int64_t m, const float *bias_host, void *y_host, nnq_dtype y_dt);

/* Several products in one call: for i in [0, count): y[i] = x[i] * W[i]^T (+ bias[i]),
 * every x[i] with the same M and dtype. Pointer arrays live in host memory. Used for
 * the q/k/v and gate/up groups of a decoder layer and for per-expert products.
 * Replaces the consecutive Linear::forward calls of
 * crates/nn-qwen3/src/layers.rs:40-47,94-167. */
NNQ_API nnq_status nnq_linear_batch(nnq_ctx *ctx, int count, const nnq_weight *const *w,
                            const void *const *x_dev, nnq_dtype x_dt, int64_t m,
                            const float *const *bias_dev, void *const *y_dev, nnq_dtype y_dt,
                            void *stream);

/* nnq_linear_batch with host-resident tensors: the activations (each distinct pointer once), the
 * biases and the outputs go through the context's pinned staging buffers with one copy in each
 * direction and one synchronisation for the whole batch (count <= 16). Products that pass the same
 * x_host pointer share their device copy and, on the skinny path, one launch: the q / k / v or
 * gate / up projections of a layer called as the reference's consecutive Linear::forward calls on
 * one input (crates/nn-qwen3/src/layers.rs:40-47,94-110). */
NNQ_API nnq_status nnq_linear_batch_host(nnq_ctx *ctx, int count, const nnq_weight *const *w,
                                         const void *const *x_host, nnq_dtype x_dt, int64_t m,
                                         const float *const *bias_host, void *const *y_host, nnq_dtype y_dt);

/* ---- compiled product plan ---------------------------------------------------------- */

/* A recorded sequence of M = 1 products (one token) run as ONE kernel launch: the counterpart, for
 * this path, of the reference's compiled dispatch plan, which is built once from a trace and then
 * replayed step by step (CompiledModel, crates/nn-metal/src/compiled_model.rs:232,305-311;
 * run_steps, crates/nn-metal/src/compiled_model_execute.rs:124). The products are added in the
 * order a decoder layer issues them (crates/nn-qwen3/src/layers.rs:40-47,94-167): a group is up to
 * 4 products that share their activations (q / k / v, gate / up), each group is one
 * nnq_linear_batch call's worth of work. nnq_plan_run gives the same results as those calls made
 * one after another on a stream: by default every group sees everything the groups before it
 * wrote. With NNQ_PLAN_ANALYZE_DEPS a group only waits for the latest earlier group whose
 * buffers overlap its own (its input was written, or its output was read or written, there).
 * The persistent kernel keeps streaming weights while a group waits for its activations, so a
 * plan runs faster than the separate launches (no ramp and tail per product).
 *   - weights: Q4_K / Q4_K_GGML with K a multiple of 256; activations x_dt, outputs y_dt as in
 *     nnq_linear; every pointer is fixed at nnq_plan_add time (CUDA-graph style): the caller
 *     updates the contents of the buffers, not their addresses;
 *   - nnq_plan_finalize allocates the plan's device tables (never later: nnq_plan_run allocates
 *     nothing and does not synchronise, so it may be captured in a CUDA graph);
 *   - a bounded device wait that runs out ends the launch and nnq_device_status reports
 *     NNQ_ERR_TIMEOUT; call nnq_plan_reset before the plan is run again;
 *   - one plan must not run twice at the same time (its counters are shared). */
typedef struct nnq_plan nnq_plan;
#define NNQ_PLAN_ANALYZE_DEPS 1
NNQ_API nnq_status nnq_plan_create(nnq_ctx *ctx, nnq_dtype x_dt, nnq_dtype y_dt, int flags, nnq_plan **out);
NNQ_API nnq_status nnq_plan_add(nnq_plan *p, int count, const nnq_weight *const *w, const void *x_dev,
                                const float *const *bias_dev, void *const *y_dev);
/* A row-parallel product whose partial outputs are summed over the ranks of `comm` inside the
 * kernel (see nnq_comm_linear): every rank adds the same group at the same place of its plan.
 * No counterpart in the reference (single device). */
NNQ_API nnq_status nnq_plan_add_reduced(nnq_plan *p, nnq_comm *comm, const nnq_weight *w, const void *x_dev,
                                        const float *bias_dev, void *y_dev);
NNQ_API nnq_status nnq_plan_finalize(nnq_plan *p);
NNQ_API nnq_status nnq_plan_run(nnq_plan *p, void *stream);
NNQ_API nnq_status nnq_plan_reset(nnq_plan *p, void *stream);
/* Bound of a dependency wait in polls of the group counter (default 2^21, about a second). */
NNQ_API nnq_status nnq_plan_set_spin_limit(nnq_plan *p, unsigned polls);
/* Groups recorded; after nnq_plan_finalize also the grid (CTAs), the copy-ring depth per warp, the
 * shared memory per CTA and the bytes of device tables the plan holds. Any pointer may be NULL. */
NNQ_API nnq_status nnq_plan_info(const nnq_plan *p, int *groups, int *ctas, int *stages, size_t *smem_bytes,
                                 size_t *table_bytes);
/* The group whose completion group `group` waits for (-1: none), after nnq_plan_finalize. */
NNQ_API nnq_status nnq_plan_dependency(const nnq_plan *p, int group, int *dep);
/* How a group of row_tiles x k_tiles tiles is split over `ctas` CTAs: the largest number of tiles
 * any CTA gets and the largest number of CTAs any row tile is spread over. Host arithmetic only. */
NNQ_API nnq_status nnq_plan_geometry(int row_tiles, int k_tiles, int ctas, int *max_tiles_per_cta, int *max_parts);
NNQ_API void nnq_plan_destroy(nnq_plan *p);

/* ---- mixture-of-experts block ------------------------------------------------------ */

/* Storage of the expert weight tensors.
 * NNQ_MOE_KN_GPTOSS: gate_up is [E, hidden, 2*inter] and down is [E, inter, hidden], i.e. each
 *   expert's matrix is stored [K, N] (x * W), quantized as one flat nn-gptoss Mxfp4Tensor, so the
 *   32-value blocks run along N (crates/nn-gptoss/src/quantized_model.rs:69-80). fmt must be
 *   NNQ_MXFP4_GPTOSS.
 * NNQ_MOE_NK: gate_up is [E, 2*inter, hidden] and down is [E, hidden, inter], each expert an
 *   [N, K] weight in any nnq_format with blocks along K (the [N,K/2]+[N,K/32] MXFP4 contract of
 *   crates/nn-metal/src/mxfp4_gemm_msl.rs:47-61 when fmt = NNQ_MXFP4_SPLIT). */
typedef enum nnq_moe_layout { NNQ_MOE_KN_GPTOSS = 0, NNQ_MOE_NK = 1 } nnq_moe_layout;

/* Build the MoE block of one decoder layer. All tensors may be host or device memory and are
 * copied. router_w [E, hidden] and router_b [E] are f32; gate_up_bias [E, 2*inter] and down_bias
 * [E, hidden] are f32; the first `inter` outputs of gate_up are the gate, the rest the up
 * projection. Replaces QuantizedDecoderLayer::load for the MoE part
 * (crates/nn-gptoss/src/quantized_model.rs:44-97). */
NNQ_API nnq_status nnq_moe_create(nnq_ctx *ctx, int n_experts, int hidden, int inter, int top_k,
                                  float swiglu_limit, const float *router_w, const float *router_b,
                                  nnq_moe_layout layout, nnq_format fmt, const void *gate_up,
                                  size_t gate_up_bytes, const void *gate_up_scales,
                                  size_t gate_up_scales_bytes, const float *gate_up_bias,
                                  const void *down, size_t down_bytes, const void *down_scales,
                                  size_t down_scales_bytes, const float *down_bias, nnq_moe **out);
/* Expert-parallel shard of the same block: this device holds experts [expert_begin,
 * expert_begin + expert_count) only (the expert tensors and biases passed cover just those),
 * the router covers all n_experts. nnq_moe_forward on a shard adds up the contributions of the
 * local experts; with activations replicated on every rank, the sum of the shards' outputs over
 * the ranks (an all-reduce) is the full block's output. The reference is single-device and has
 * no counterpart. */
NNQ_API nnq_status nnq_moe_create_shard(nnq_ctx *ctx, int n_experts, int expert_begin, int expert_count,
                                        int hidden, int inter, int top_k, float swiglu_limit,
                                        const float *router_w, const float *router_b, nnq_moe_layout layout,
                                        nnq_format fmt, const void *gate_up, size_t gate_up_bytes,
                                        const void *gate_up_scales, size_t gate_up_scales_bytes,
                                        const float *gate_up_bias, const void *down, size_t down_bytes,
                                        const void *down_scales, size_t down_scales_bytes,
                                        const float *down_bias, nnq_moe **out);
NNQ_API void nnq_moe_destroy(nnq_moe *m);

/* y[T, hidden] (f32) = MoE(x[T, hidden]): router linear, softmax over all experts, top-k,
 * renormalisation, per-expert x*W_gu+b, clamp(silu(gate), +-limit)*up, *W_d+b, and the
 * routing-weighted sum per token with the experts taken in index order. Routing stays on the
 * device. Replaces QuantizedDecoderLayer::{expert_forward,moe_forward}
 * (crates/nn-gptoss/src/quantized_model.rs:99-194), GptOssMoeBlock::forward
 * (crates/nn-gptoss/src/layers.rs:254) and fused_moe_forward (crates/nn-gptoss/src/moe_dispatch.rs:50). */
NNQ_API nnq_status nnq_moe_forward(nnq_ctx *ctx, const nnq_moe *m, const void *x_dev, nnq_dtype x_dt,
                                   int64_t tokens, float *y_dev, void *stream);

/* Routing only: expert indices [T, top_k] (descending probability) and renormalised weights
 * [T, top_k]. Replaces the softmax / topk / renormalise prefix of moe_forward
 * (crates/nn-gptoss/src/quantized_model.rs:136-144; crates/nn-core/src/dyn_tensor/ops/topk.rs:100-139). */
NNQ_API nnq_status nnq_moe_route(nnq_ctx *ctx, const nnq_moe *m, const void *x_dev, nnq_dtype x_dt,
                                 int64_t tokens, int32_t *idx_dev, float *weights_dev, void *stream);

/* Expert parallelism with token dispatch (tokens sharded over the ranks, every rank holding
 * n_experts / world experts; no counterpart in the reference, which runs on one device). The
 * library provides the device-side pieces, the exchange of the rows between the ranks is the
 * caller's all-to-all (NCCL):
 *   nnq_moe_route          expert indices / weights of the local tokens (router replicated);
 *   nnq_moe_gather_rows    out[i, :] = x[index[i], :] -- the token permute: rows sorted by
 *                          destination expert before they are sent;
 *   nnq_moe_forward_routed the expert MLPs over rows whose routing the caller supplies: idx_dev /
 *                          weights_dev are [rows, slots] (global expert indices; a row whose expert
 *                          is not held by this block contributes nothing): on the owner of the
 *                          experts, slots = 1 and weight 1 give each received row its expert's output
 *                          (quantized_model.rs:152-189, gather :183 and expert_forward);
 *   nnq_moe_combine_rows   y[t, :] = sum over the token's slots, in expert-index order, of
 *                          weights[t, s] * rows[pos[t, s], :] -- the weighted scatter-add of
 *                          quantized_model.rs:186-188 over the rows that came back (pos < 0: skipped). */
NNQ_API nnq_status nnq_moe_forward_routed(nnq_ctx *ctx, const nnq_moe *m, const void *x_dev, nnq_dtype x_dt, int64_t rows,
                                          int slots, const int32_t *idx_dev, const float *weights_dev, float *y_dev,
                                          void *stream);
NNQ_API nnq_status nnq_moe_gather_rows(nnq_ctx *ctx, const void *x_dev, nnq_dtype dt, const int32_t *index_dev, int64_t count,
                                       int64_t width, void *out_dev, void *stream);
NNQ_API nnq_status nnq_moe_combine_rows(nnq_ctx *ctx, const float *rows_dev, const int32_t *idx_dev, const float *weights_dev,
                                        const int32_t *pos_dev, int64_t tokens, int hidden, int top_k, float *y_dev,
                                        void *stream);

/* Same computation as nnq_moe_forward for callers that cannot allocate device memory: an
 * inference server that has handed the whole device to its own memory pool (a library-side
 * cudaMalloc would fail there), or a latency-critical loop that must not take the device-wide
 * synchronisation cudaMalloc / cudaFree imply. It has no counterpart in the reference. The
 * routing tables and intermediate activations live in a fixed 8 MiB area inside the library's
 * device image (held by every GPU that loads the library until the process exits) instead of the
 * context's growable scratch buffer, and the call performs no allocation of any kind.
 * Limits and rules:
 *   - tokens * top_k * ((2*inter + hidden) * s + inter) * 4 bytes (plus small tables) must fit the
 *     8 MiB area, with s = 1 whenever the expert weights have a tiled layout (both layouts at
 *     gpt-oss-20b's hidden = inter = 2880: 182 routed rows, 45 tokens at top-4) and s = 4 only for
 *     an [E,K,N] block whose shape has none (partial sums per K slice); larger calls are rejected
 *     with NNQ_ERR_UNSUPPORTED and a message naming both sizes;
 *   - the first call on a device looks up the area's address (cudaGetSymbolAddress); make that
 *     first call before any stream capture;
 *   - all calls on a device share the area: two calls whose kernels overlap on the GPU (different
 *     streams, or different contexts on one device) race. Calls on one stream are safe. Nothing
 *     in the area needs clearing between calls. */
NNQ_API nnq_status nnq_moe_forward_static(nnq_ctx *ctx, const nnq_moe *m, const void *x_dev, nnq_dtype x_dt,
                                          int64_t tokens, float *y_dev, void *stream);

/* ---- tensor-parallel exchange ------------------------------------------------------ */

/* One-shot all-reduce (sum) of small vectors between the ranks of one NVLink box, one process
 * per GPU: the partial outputs of row-parallel projections (o_proj, down_proj). The reference
 * is single-device and has no counterpart. Set-up: every rank creates a communicator, publishes
 * its 64-byte handle (nnq_comm_get_handle), gathers all ranks' handles in rank order by any
 * host-side means and opens them (nnq_comm_open_peers). world <= 8; max_bytes bounds one message.
 * nnq_comm_all_reduce sums `count` elements of `buf_dev` in place over all ranks (rank order,
 * identical bits everywhere), is a single kernel without host synchronisation (graph-capturable),
 * and must be called the same number of times, in the same order, by every rank. A peer that
 * never arrives makes the bounded device wait run out: nnq_device_status then reports
 * NNQ_ERR_TIMEOUT and the buffer contents are undefined. A rank whose wait ran out has still
 * advanced its sequence number while the late peer has not, so after a timeout the ranks no longer
 * agree on it: destroy the communicators of all ranks and create new ones (there is no in-place
 * resynchronisation). Messages of 32 KB and more use several CTAs; smaller ones a single CTA. */
NNQ_API nnq_status nnq_comm_create(nnq_ctx *ctx, int rank, int world, size_t max_bytes, nnq_comm **out);
NNQ_API nnq_status nnq_comm_get_handle(nnq_comm *c, void *handle64);
NNQ_API nnq_status nnq_comm_open_peers(nnq_comm *c, const void *handles);
NNQ_API nnq_status nnq_comm_all_reduce(nnq_comm *c, void *buf_dev, nnq_dtype dt, int64_t count, void *stream);
/* Bound of every device-side wait of kernels that use this communicator, in polls of a flag
 * (default 2^22, a few seconds). Synchronises the device. After a wait has run out
 * (NNQ_ERR_TIMEOUT from nnq_device_status) this rank's sequence numbers are out of step with its
 * peers': destroy the communicators of all ranks and build new ones. Mirrors the Timeout kind of
 * the reference's backend errors (crates/nn-core/src/error.rs:48-93). */
NNQ_API nnq_status nnq_comm_set_spin_limit(nnq_comm *c, unsigned polls);
/* Single-process set-up (one process driving several GPUs with peer access enabled, or several
 * communicators on one device): instead of exchanging IPC handles, pass every rank's buffer
 * (nnq_comm_local_buffer of that rank's communicator) as a device pointer valid in this process;
 * peer_dev_ptrs has `world` entries, the entry of this rank is ignored. */
NNQ_API nnq_status nnq_comm_local_buffer(nnq_comm *c, void **dev_ptr);
NNQ_API nnq_status nnq_comm_open_local_peers(nnq_comm *c, void *const *peer_dev_ptrs);
/* Row-parallel product and its all-reduce in one call: y = sum over ranks of (x_r * W_r^T) + bias,
 * the same y on every rank (pass the same bias everywhere; it is added once). For M = 1 on a tiled
 * Q4_K shard (and max_bytes >= 8 * N) this is ONE kernel: the warp that finishes a row tile sends
 * its partial sums to the peers as 8-byte (value, sequence number) stores over peer memory, waits
 * (bounded) for theirs and writes the finished rows, so the exchange overlaps the rest of the
 * product. Otherwise it is nnq_linear followed by nnq_comm_all_reduce. M * N * 4 must fit the
 * communicator's max_bytes. No counterpart in the reference (single device). */
NNQ_API nnq_status nnq_comm_linear(nnq_comm *c, const nnq_weight *w, const void *x_dev, nnq_dtype x_dt, int64_t m,
                                   const float *bias_dev, void *y_dev, nnq_dtype y_dt, void *stream);
NNQ_API void nnq_comm_destroy(nnq_comm *c);

/* ------------------------------------------------------------------------------------------
 * One decode step of a Qwen3-shaped decoder around the quantized products (batch 1, greedy).
 * Replaces, for the decode loop, Qwen3DecoderLayer::forward / Qwen3Attention::forward / Qwen3MLP::forward
 * (crates/nn-qwen3/src/layers.rs:40-47,94-167,205-226), RmsNorm (crates/nn-core/src/layers/rms_norm.rs:87-100),
 * RotaryEmbedding tables and the half-split rotation (layers/attention/rope.rs:78-106,
 * rope_half_split.rs:98-134), sdpa (attention/sdpa.rs:59-71), KvCacheLayer::append
 * (layers/generation/kv_cache.rs:132) and the greedy argmax of the generation loop
 * (generation/autoregressive_sampling.rs:14-21: of equal maxima the last wins).
 * The current token and position live on the device and are advanced by the step itself, so the
 * launches of nnq_decoder_step may be captured in a CUDA graph once and replayed per token.
 * head_dim must be 128; activations between the kernels are f32, the inputs of the products are
 * converted to act_dtype (NNQ_F32 keeps the reference's arithmetic, NNQ_BF16 is faster).
 * The weights, the embedding table ([vocab, hidden] bf16, device) and the vocabulary projection
 * stay owned by the caller and must outlive the decoder. */
typedef struct nnq_decoder nnq_decoder;
typedef struct nnq_decoder_config {
    int32_t hidden, n_heads, n_kv_heads, head_dim, ffn, n_layers, vocab, max_seq;
    float rms_eps;
    double rope_theta;
    int32_t act_dtype;   /* nnq_dtype */
    int32_t tp_rank, tp_world;   /* tensor parallelism over key/value heads and the FFN width; 0 of 1 = none */
} nnq_decoder_config;
NNQ_API nnq_status nnq_decoder_create(nnq_ctx *ctx, const nnq_decoder_config *cfg, nnq_decoder **out);
/* norm weights: f32, host or device pointers (copied) */
NNQ_API nnq_status nnq_decoder_set_layer(nnq_decoder *d, int layer, const nnq_weight *q, const nnq_weight *k,
                                         const nnq_weight *v, const nnq_weight *o, const nnq_weight *gate,
                                         const nnq_weight *up, const nnq_weight *down, const float *in_norm,
                                         const float *post_norm, const float *q_norm, const float *k_norm);
NNQ_API nnq_status nnq_decoder_set_head(nnq_decoder *d, const void *embed_bf16_dev, const float *final_norm,
                                        const nnq_weight *lm_head);
/* The caches hold max_seq positions and do not grow (the reference's KvCacheLayer::append doubles
 * its buffer instead, crates/nn-core/src/layers/generation/kv_cache.rs:132): the step that would
 * consume position max_seq is refused with NNQ_ERR_UNSUPPORTED by nnq_decoder_step, and, when a
 * captured graph is replayed past the end, by nnq_device_status (the step then changes no state).
 * Tensor-parallel decoder (tp_world > 1): set_layer takes this rank's shards (q / k / v / gate / up
 * split by rows: heads [rank * n_heads / world, ...), FFN rows likewise; o / down split along K in
 * the same ranges), norms, embedding and the vocabulary projection are replicated, and the o and
 * down products are exchanged through `comm` (nnq_comm_linear; max_bytes >= 8 * hidden). All ranks
 * hold identical hidden states and produce the same token. The vocabulary projection is either
 * replicated ([vocab, hidden] on every rank) or vocabulary-parallel: set_head takes this rank's
 * rows [rank * vocab / world, (rank + 1) * vocab / world) (nnq_weight_create_shard, axis 0), each
 * rank forms the logits of its rows only (at their global offsets in the logits buffer) and the
 * ranks agree on the greedy token by exchanging (value, index) through `comm`
 * (max_bytes >= 8 * hidden + 16), keeping the reference's rule that the last of equal maxima wins. */
NNQ_API nnq_status nnq_decoder_set_comm(nnq_decoder *d, nnq_comm *comm);
/* next input token and the position it is written at (synchronises the stream) */
NNQ_API nnq_status nnq_decoder_reset(nnq_decoder *d, int token, int pos, void *stream);
/* one token: consumes (token, pos), appends to the caches, leaves the logits in the logits buffer,
 * stores the argmax as the next token and advances the position */
NNQ_API nnq_status nnq_decoder_step(nnq_decoder *d, void *stream);
/* Prompt pass: runs `count` prompt tokens (host array) through the decoder at positions
 * start_pos .. start_pos + count - 1 in blocks of up to 1024 rows -- the products on the M > 16 paths,
 * attention under the causal mask (every row sees the cache up to its own position:
 * crates/nn-qwen3/src/forward_common.rs:55-64,189-204, crates/nn-core/src/layers/attention/sdpa.rs:118-141)
 * -- fills the caches, leaves the logits of the last prompt token in the logits buffer, stores its
 * greedy successor as the next token and sets the position to start_pos + count, so that
 * nnq_decoder_step continues the sequence. No nnq_decoder_reset is needed before it. The first call
 * allocates the row buffers; the call synchronises the stream (not for graph capture). */
NNQ_API nnq_status nnq_decoder_prefill(nnq_decoder *d, const int32_t *tokens_host, int count, int start_pos, void *stream);
/* reads (next token, next position, steps taken) back; synchronises the stream */
NNQ_API nnq_status nnq_decoder_state(nnq_decoder *d, int *token, int *pos, int *steps, void *stream);
/* device buffers: key / value caches [layers, kv_heads, max_seq, head_dim] f32, logits [vocab] f32,
 * generated tokens [max_seq] (token produced at position p is stored at index p) */
NNQ_API nnq_status nnq_decoder_buffers(nnq_decoder *d, float **k_cache, float **v_cache, float **logits, int **tokens);
NNQ_API void nnq_decoder_destroy(nnq_decoder *d);

/* Number of kernels this library has launched on this context since creation. */
NNQ_API int64_t nnq_launch_count(const nnq_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* NNQ_H */
