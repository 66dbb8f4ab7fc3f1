/*
 * loom_b200.h -- C ABI of the B200 (sm_100a) implementation of Loom's BitNet
 * ternary-weight x int8-activation linear path.
 *
 * The library replaces the WGSL/wgpu column of Loom's kernel layer for this one path.
 * Each entry point names the reference interface it stands in for (paths relative to
 * the openfluke/loom project root).  Conventions follow Loom's accelerator-plugin ABI
 * (poly/accel/include/loom_accel.h:11-66): every call returns an int (0 = ok, negative
 * = error), the message is available from loom_b200_last_error(), and the library
 * never keeps a caller's host pointer after the call returns.
 *
 * There is no CPU fallback: a call that cannot run on the GPU returns an error.
 * Calls on one context must be serialised by the caller (like a WGPUContext, which
 * owns a single command encoder, poly/wgpu_kernels.go:245-260).  Work is asynchronous
 * on the context's stream; loom_b200_sync() (or any download) waits for it.
 *
 * Device buffers are plain device addresses (void*): a Go caller keeps them as
 * uintptr exactly where it keeps *wgpu.Buffer today.
 */
#ifndef LOOM_B200_H
#define LOOM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LOOM_B200_API_VERSION 1

/* error codes */
#define LOOM_B200_OK 0
#define LOOM_B200_ERR_INVALID (-1)     /* null pointer, bad shape, bad handle */
#define LOOM_B200_ERR_CUDA (-2)        /* a CUDA call failed; see last_error */
#define LOOM_B200_ERR_UNSUPPORTED (-3) /* shape or option outside what the kernels cover */
#define LOOM_B200_ERR_NO_DEVICE (-4)   /* no sm_100 device */
#define LOOM_B200_ERR_TIMEOUT (-5)     /* a bounded device-side wait ran out */
#define LOOM_B200_ERR_COMM (-6)        /* NCCL / multi-GPU set-up failed */

/* poly.ActivationType, poly/poly.go:86-98 */
#define LOOM_B200_ACT_RELU 0
#define LOOM_B200_ACT_SILU 1
#define LOOM_B200_ACT_GELU 2
#define LOOM_B200_ACT_TANH 3
#define LOOM_B200_ACT_SIGMOID 4
#define LOOM_B200_ACT_LEAKY_RELU 5
#define LOOM_B200_ACT_RELU2 6
#define LOOM_B200_ACT_LINEAR (-1)

typedef struct loom_b200_ctx loom_b200_ctx;       /* stands in for *poly.WGPUContext */
typedef struct loom_b200_graph loom_b200_graph;   /* a recorded command buffer (one frame) */
typedef struct loom_b200_weight loom_b200_weight; /* a packed ternary matrix resident in HBM:
                                                     WeightStore.GPUWeights[key] + GPUScaleValues[key],
                                                     poly/weights.go:14-24 */

/* ---- library / context ------------------------------------------------------------ */

/* loom_accel_api_version, poly/accel/include/loom_accel.h:22 */
int loom_b200_api_version(void);
/* number of CUDA devices of compute capability 10.x; 0 when there is none */
int loom_b200_device_count(void);
/* loom_accel_last_error, poly/accel/include/loom_accel.h:66.  ctx may be NULL (errors of
 * ctx_create).  The string stays valid until the next failing call on the same context. */
const char* loom_b200_last_error(const loom_b200_ctx* ctx);

/* Replaces WGPUContext creation (poly/wgpu_context_native.go) for this path.  `stream` is an
 * existing cudaStream_t to launch on, or NULL to let the context create its own. */
int loom_b200_ctx_create(int device, void* stream, loom_b200_ctx** out);
void loom_b200_ctx_destroy(loom_b200_ctx* ctx);
/* FlushFrame + wait, poly/wgpu_context_native.go:276 */
int loom_b200_sync(loom_b200_ctx* ctx);
/* BeginFrame ... FlushFrame (poly/wgpu_context_native.go:263-276, used once per forward by
 * ForwardTokenIDsWGPU, poly/wgpu_forward.go:99,564): the dispatches issued between begin and end are
 * recorded into a CUDA graph instead of running; graph_launch replays them with one submission.
 * Run the same dispatches once before graph_begin so that every scratch buffer already has its size;
 * allocation, upload, download and sync are refused while recording. */
int loom_b200_graph_begin(loom_b200_ctx* ctx);
int loom_b200_graph_end(loom_b200_ctx* ctx, loom_b200_graph** out);
int loom_b200_graph_launch(loom_b200_ctx* ctx, loom_b200_graph* graph);
void loom_b200_graph_free(loom_b200_ctx* ctx, loom_b200_graph* graph);
/* the cudaStream_t the context launches on */
void* loom_b200_ctx_stream(loom_b200_ctx* ctx);
/* Tuning knobs, the counterpart of the tileSize argument the WGSL dispatchers take
 * (poly/wgpu_kernels.go:416-427): "gemv_variant" 0 = integer-MMA inner loop, 1 = dp4a inner loop;
 * "gemv_ctas_per_sm" 1..8; "pdl" 0/1 = programmatic dependent launch.  Results never depend on them. */
int loom_b200_ctx_set_option(loom_b200_ctx* ctx, const char* key, int value);
/* number of kernels of this library launched on the context since creation */
uint64_t loom_b200_launch_count(const loom_b200_ctx* ctx);

/* ---- device buffers (GetActivationBuffer / CreatePersistentBuffer / ReadBuffer,
 *      poly/wgpu_context_native.go:313,438 and ReadBuffer) ---------------------------- */
int loom_b200_buffer_alloc(loom_b200_ctx* ctx, size_t bytes, void** dptr);
int loom_b200_buffer_free(loom_b200_ctx* ctx, void* dptr);
int loom_b200_buffer_upload(loom_b200_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int loom_b200_buffer_download(loom_b200_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);
int loom_b200_buffer_zero(loom_b200_ctx* ctx, void* dst_dev, size_t bytes);

/* ---- packed ternary weights ----------------------------------------------------------- */

/* VolumetricLayer.syncBitNetPackedMatrix, poly/bitnet_gpu.go:28-50: takes BitNetTernaryMatrix.Words
 * (row-major, 16 two-bit codes per u32, code = weight+1, poly/bitnet_cpu.go:16-43) and its Scale.
 * The words are copied during the call and re-tiled on the device for the kernels; results do not
 * depend on the internal layout.  row_words must be ceil(cols/16). */
int loom_b200_upload_ternary(loom_b200_ctx* ctx, const uint32_t* words, int rows, int cols, int row_words,
                             float scale, loom_b200_weight** out);
/* GetBitNetTernaryMatrix from an fp32 Master slab, poly/bitnet_cpu.go:345-354,934-977, done on the
 * device: per-matrix absmean scale, round(w/scale) clipped to [-1,1], the already-ternary rule.
 * master_dev points at rows*cols fp32 values in device memory. */
int loom_b200_pack_ternary_f32(loom_b200_ctx* ctx, const float* master_dev, int rows, int cols,
                               loom_b200_weight** out);
/* SetMicrosoftBitNetPackedMatrixBytes, poly/bitnet_cpu.go:1031-1052,1078-1098: host bytes of the
 * microsoft/bitnet-b1.58 offline layout ((rows/4)*cols bytes); scale as SetBitNetPackedScale. */
int loom_b200_upload_microsoft_u8(loom_b200_ctx* ctx, const uint8_t* packed, int rows, int cols, float scale,
                                  loom_b200_weight** out);
int loom_b200_weight_info(const loom_b200_weight* w, int* rows, int* cols, int* row_words, float* scale);
/* SetBitNetPackedScale, poly/bitnet_cpu.go:979-993 */
int loom_b200_weight_set_scale(loom_b200_weight* w, float scale);
/* reads the matrix back in the reference's word layout (rows*row_words u32) -- the round trip of
 * the re-tiling, and what entity_bitnet.go would serialise */
int loom_b200_weight_download_words(loom_b200_ctx* ctx, const loom_b200_weight* w, uint32_t* words_host);
void loom_b200_weight_free(loom_b200_ctx* ctx, loom_b200_weight* w);

/* ---- kernel dispatch (device buffers) --------------------------------------------------- */

/* WGPUContext.DispatchBitNetQuantizeActivation(batch, in, inputBuf, qPackedBuf, scaleBuf),
 * poly/wgpu_kernels.go:384-414; arithmetic of bitNetQuantizeActivationNumeric, poly/bitnet_cpu.go:45-106.
 * x [batch,in] fp32 -> q [batch,in] int8 (natural byte order = the reference's 4-per-u32 packing) and
 * amax [batch] fp32.  Unlike the WGSL kernel the second output is the absmax itself, not absmax/127:
 * the CPU path's float64 rescale needs it unrounded. */
int loom_b200_quantize_activation(loom_b200_ctx* ctx, int batch, int in, const float* x, int8_t* q, float* amax);
/* float64-input twin, bitNetQuantizeActivationFloat64, poly/bitnet_cpu.go:108-117 */
int loom_b200_quantize_activation_f64(loom_b200_ctx* ctx, int batch, int in, const double* x, int8_t* q,
                                      float* amax);

/* WGPUContext.DispatchDenseBitNetTernaryQuantized(batch, in, out, qPacked, scale, weight, bias, output,
 * weightScale, activation, tileSize), poly/wgpu_kernels.go:416-475; arithmetic of
 * bitNetTernaryMatVecQuantized + the Dense epilogue, poly/bitnet_cpu.go:536-546, poly/dense.go:94-98:
 *   out[b,r] = Activate( float32( float64(acc[b,r]) * (float64(scale)*float64(amax[b])/127) + bias[r] ) )
 *              (+ residual[b,r], a float32 add, when residual != NULL)
 * q [batch,cols] int8, amax [batch], bias [rows] or NULL, residual [batch,rows] or NULL,
 * out [batch,rows] fp32.  acc_out [batch,rows] int32 (or NULL) receives the raw accumulators. */
int loom_b200_ternary_linear(loom_b200_ctx* ctx, const loom_b200_weight* w, int batch, const int8_t* q,
                             const float* amax, const float* bias, const float* residual, int activation,
                             float* out, int32_t* acc_out);

/* WGPUContext.DispatchBitNetGateProduct(batch, hidden, act, gate, up, out), poly/wgpu_kernels.go:477-507;
 * arithmetic of swigluGateProduct in float64, poly/swiglu.go:37-46 */
int loom_b200_gate_product(loom_b200_ctx* ctx, int batch, int hidden, int activation, const float* gate,
                           const float* up, float* out);

/* WGPUContext.DispatchRMSNorm used as the BitNet inner norm (poly/wgpu_forward.go:258-266,383-389);
 * arithmetic of bitNetRMSNormTensorRowWeighted, poly/bitnet_cpu.go:893-913.  In place on x [batch,n];
 * weight [weight_len] or NULL; eps <= 0 means 1e-5. */
int loom_b200_inner_rmsnorm(loom_b200_ctx* ctx, int batch, int n, float* x, const float* weight, int weight_len,
                            double eps);

#ifdef __cplusplus
}
#endif
#endif
