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
/* FlushFrame + wait, poly/wgpu_context_native.go:276.  Also reports a bounded device-side wait that ran out since the
 * last sync (LOOM_B200_ERR_TIMEOUT; the results of the calls in between are invalid) and clears that condition. */
int loom_b200_sync(loom_b200_ctx* ctx);
/* Tensor-pipe micro-peak (no counterpart in the reference): one CTA per SM issues iters x 4 tcgen05.mma kind::i8
 * instructions of M = 128, N = 256, K = 32 on operands resident in shared memory and reports dense int8 TOP/s.  The
 * denominator for the GEMM's tensor roofline on the GPU at hand. */
int loom_b200_selftest_i8_peak(loom_b200_ctx* ctx, int iters, double* tops_out);
/* Failure-detection self-test (no counterpart in the reference): launches one thread that polls a flag nothing ever
 * sets, gives up after `polls` reads and raises the context's device status word, exactly as the bounded waits inside
 * the kernels do (tile copies, the GEMM pipeline, tensor-parallel peers).  Returns LOOM_B200_ERR_TIMEOUT through the
 * same path loom_b200_sync uses, clears the word, and leaves the context usable.  Nothing faults, traps or hangs. */
int loom_b200_selftest_wait_timeout(loom_b200_ctx* ctx, unsigned int polls);

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
 * "gemv_ctas_per_sm" 1..8; "gemv_partition" 0 = choose, 1 = stream-K over tiles with the int32 fix-up,
 * 2 = whole strips per CTA; "pdl" 0/1 = programmatic dependent launch; "tp_graph" 0/1 = record the
 * tensor-parallel decode step, collectives included, as a graph; "gemm_tile" 0 / 128 / 256 = tokens per CTA of the
 * token-block GEMM (0 = choose); "gemm_splitk" 0/1 = let several CTAs share the K range of an output tile;
 * "fold_rope" 0/1 = one-token decoder steps apply RoPE inside the attention kernel (one launch less per block);
 * "decode_splits" 0..32 = position splits of the one-token attention, read by loom_b200_decoder_create (0 = choose); "tp_peer" 0/1 = use the peer mailboxes when attached;
 * "attn_stream" 0/1 = a pass of several sequences runs its attention as one streaming CTA per (sequence, KV head) (1, default) or as
 * clusters / the split kernel (0);
 * "gemv_lean" 0/1 = one-token launches with a fused prologue use GEMV instantiations compiled without the stream-K, general-prologue
 * and phase-trace code (1, default: +7 % decode tok/s) or the full kernels (0);
 * "tp_fused" 0/1 = row-parallel projections under the peer mailboxes as statistics kernel + GEMV + finalize kernel (0), or with the
 * exchange of the partial sums in the GEMV's epilogue (1, default);
 * "prefill_gemm" 0/1 = prompts of 32 or more tokens
 * run their projections as token-block GEMMs on the tensor cores (1) or eight tokens at a time through the GEMV (0).  "gemm_cache" 0/1 = the token-block GEMM reads pre-expanded int8 codes (one byte per weight, built per
 * matrix the first time it meets the GEMM, four times its packed bytes; the device twin of ensureBitNetCodes,
 * poly/bitnet_cpu.go:700-729) and fuses the SwiGLU gate product into the gate/up GEMM (1), or expands the 2-bit tiles
 * inside the kernel (0); "head_stream" 0/1 = the fp32 LM head streams
 * its rows through shared memory with bulk copies and folds the greedy step (argmax, position, next embedding row) into
 * its tail (1), or runs as a warp-per-row kernel followed by separate launches (0; read when the embeddings are set);
 * "attn_cluster" 0/1 = one-token decoder steps run their attention
 * as one thread-block cluster per KV head that combines its position slices through distributed shared memory (1) or as
 * independent (head, slice) CTAs with a last-arriver combine (0).  Results never depend on them beyond the order of
 * float64 additions. */
int loom_b200_ctx_set_option(loom_b200_ctx* ctx, const char* key, int value);
/* Phase trace, the counterpart of WGPUContext.TimeCommands (poly/wgpu_context_native.go:553) and of the
 * per-layer timing ForwardTokenIDsWGPU emits (poly/wgpu_forward.go:121-127).  With option "trace" = 1 every
 * GEMV / RoPE / attention / LM-head launch (also inside a recorded frame) gets a row of eight 64-bit slots, in
 * launch order modulo 1024, and its first CTA writes the GPU global timer (ns): 0 start, 1 weights requested,
 * 2 upstream data ready, 3 activations staged (attention: scores done), 4 dot products done, 5 end.  Unused
 * slots stay 0.  trace_read copies the first `rows` rows; trace_label names the kernel of a row. */
int loom_b200_trace_read(loom_b200_ctx* ctx, uint64_t* host, int rows);
const char* loom_b200_trace_label(const loom_b200_ctx* ctx, int row);
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
/* A BITNET_TERNARY blob of an .entity checkpoint as encodeEntityBitNetTernaryBlob writes it
 * (poly/entity_bitnet.go:38-88): 24-byte little-endian header {rows, cols, offset, float32 scale bits, rowWords,
 * nWords} followed by nWords packed words.  Validated like decodeEntityBitNetTernaryBlob (short or truncated
 * blobs are errors; rowWords 0 means ceil(cols/16)).  *offset_out (may be NULL) receives the slab offset the
 * reference keys the matrix by (10000 + offset, poly/bitnet_cpu.go:286-292). */
int loom_b200_upload_entity_blob(loom_b200_ctx* ctx, const uint8_t* blob, size_t len, int* offset_out,
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

/* The batched (prompt) form of DispatchBitNetQuantizeActivation + DispatchDenseBitNetTernaryQuantized
 * (poly/wgpu_forward.go:167-180, poly/wgpu_kernels.go:384-475) as one tensor-core GEMM: x [tokens, cols] fp32 on the
 * device is quantized per token (absmax int8, poly/bitnet_cpu.go:45-106) and multiplied with the packed ternary
 * matrix on tcgen05 (kind::i8, int32 accumulators in tensor memory); the epilogue is the one of
 * loom_b200_ternary_linear.  out [tokens, rows] fp32 and/or acc_out [tokens, rows] int32; amax_out [tokens] or NULL.
 * Same bits as the per-token path. */
int loom_b200_ternary_gemm(loom_b200_ctx* ctx, const loom_b200_weight* w, int tokens, const float* x, const float* bias,
                           const float* residual, int activation, float* out, int32_t* acc_out, float* amax_out);

/* No counterpart in the reference.  The same computation as loom_b200_ternary_linear (without the raw
 * accumulator output) for hosts that must not allocate device memory while they run inference: an embedder
 * with a fixed, already-spent device-memory budget, a frame loop that promised "no allocation after load", or
 * code running where the CUDA allocator may not be entered.  The regular entry point may grow its fix-up
 * scratch with cudaMalloc when a larger shape first arrives; this one keeps that scratch in a fixed
 * 1.02 MiB array inside the library image (held by every GPU that loads the library until the process exits)
 * and calls no cudaMalloc, cudaFree or allocating routine.
 *   Limits: rows <= 65,536 and 16*ceil(rows/16)*tokens_per_pass <= 262,144, where tokens_per_pass is
 *   min(batch, 8) for inputs of up to about 19,000 columns and fewer beyond (5 at 28,672 columns: the same
 *   rule as loom_b200_ternary_linear); beyond them the call fails with LOOM_B200_ERR_UNSUPPORTED and a message
 *   naming loom_b200_ternary_linear.  A bounded device-side wait that runs out inside this call is reported
 *   by loom_b200_sync like one inside the regular call (the context's own status word is used).
 *   The first call on a device looks the array's address up (cudaGetSymbolAddress); make that call before
 *   starting any stream capture.  Every call clears the part of the array it is about to use.  The array is
 *   shared by all contexts of the process: two calls whose GPU work overlaps in time (different streams or
 *   contexts on the same device) race on it -- run them one after the other. */
int loom_b200_ternary_linear_no_alloc(loom_b200_ctx* ctx, const loom_b200_weight* w, int batch, const int8_t* q,
                                      const float* amax, const float* bias, const float* residual, int activation,
                                      float* out);

/* WGPUContext.DispatchBitNetGateProduct(batch, hidden, act, gate, up, out), poly/wgpu_kernels.go:477-507;
 * arithmetic of swigluGateProduct in float64, poly/swiglu.go:37-46 */
int loom_b200_gate_product(loom_b200_ctx* ctx, int batch, int hidden, int activation, const float* gate,
                           const float* up, float* out);

/* WGPUContext.DispatchRMSNorm used as the BitNet inner norm (poly/wgpu_forward.go:258-266,383-389);
 * arithmetic of bitNetRMSNormTensorRowWeighted, poly/bitnet_cpu.go:893-913.  In place on x [batch,n];
 * weight [weight_len] or NULL; eps <= 0 means 1e-5. */
int loom_b200_inner_rmsnorm(loom_b200_ctx* ctx, int batch, int n, float* x, const float* weight, int weight_len,
                            double eps);

/* ---- layer forwards (host buffers) --------------------------------------------------------
 * The packed-ternary layer paths of poly, with host tensors in and out like the cabi exports
 * LoomDenseForwardPackedTernaryCPU / LoomSwiGLUForwardPackedTernaryCPU / LoomMHAForwardPackedTernaryCPU
 * (welvet/cabi/engine_ext.go:267-331).  Host-to-device and device-to-host copies happen inside the call. */

/* DenseForwardPackedTernaryCPU, poly/dense.go:66-101: in [batch,cols] -> pre, post [batch,rows]
 * (either may be NULL).  No bias. */
int loom_b200_dense_forward(loom_b200_ctx* ctx, const loom_b200_weight* w, int activation, const float* in_host,
                            int batch, float* pre_host, float* post_host);

/* SwiGLUForwardPackedTernaryCPU, poly/swiglu.go:270-322: in [seq,hidden] -> pre [seq,inter] (the gate
 * product after the always-on inner RMSNorm) and post [seq,hidden].  Bias and inner-norm vectors are host
 * pointers or NULL; rms_eps <= 0 means 1e-5 (layer.RMSNormEps unset). */
int loom_b200_swiglu_forward(loom_b200_ctx* ctx, const loom_b200_weight* gate, const loom_b200_weight* up,
                             const loom_b200_weight* down, const float* bias_gate, const float* bias_up,
                             const float* bias_down, const float* inner_norm_w, int inner_norm_len, double rms_eps,
                             int activation, const float* in_host, int seq, float* pre_host, float* post_host);

/* The MHA VolumetricLayer with its ring KV cache (fields read by MHAForwardPackedTernaryCPU,
 * poly/mha.go:204-371).  Weights are borrowed and must outlive the layer; host vectors are copied.
 * max_seq_len 0 means 512, rope_theta <= 0 means 10000, rms_eps as layer.RMSNormEps. */
typedef struct loom_b200_mha loom_b200_mha;
int loom_b200_mha_create(loom_b200_ctx* ctx, int d_model, int num_heads, int num_kv_heads, int head_dim,
                         int max_seq_len, double rope_theta, double rms_eps, const loom_b200_weight* wq,
                         const loom_b200_weight* wk, const loom_b200_weight* wv, const loom_b200_weight* wo,
                         const float* bq, const float* bk, const float* bv, const float* bo, const float* q_norm_w,
                         int q_norm_len, const float* k_norm_w, int k_norm_len, const float* inner_norm_w,
                         int inner_norm_len, loom_b200_mha** out);
void loom_b200_mha_destroy(loom_b200_mha* layer);
/* Transformer.Reset for this layer: KVOffset = 0, poly/transformer.go:119-127 */
int loom_b200_mha_reset(loom_b200_mha* layer);
int loom_b200_mha_kv_offset(const loom_b200_mha* layer);
/* MHAForwardPackedTernaryCPU: in [batch,seq,d_model] -> pre (normalised attention rows) and post
 * [batch,seq,d_model].  The ring restarts unless batch == seq == 1 and it already holds positions
 * (mhaPrepareKVForForward, poly/mha_layout.go:62-70).  Positions beyond max_seq_len are refused. */
int loom_b200_mha_forward(loom_b200_mha* layer, const float* in_host, int batch, int seq, float* pre_host,
                          float* post_host);
/* copies the KV ring [max_seq_len, kv_heads*head_dim] to the host (either pointer may be NULL) */
int loom_b200_mha_download_cache(loom_b200_mha* layer, float* k_host, float* v_host);

/* ---- decoder --------------------------------------------------------------------------------
 * The ternary decoder stack InitHFDecoderBlocks wires (poly/hf_decoder.go:20-68) driven the way
 * Transformer.Generate drives ForwardTokenIDsWGPU (poly/transformer.go:341-485, poly/wgpu_forward.go:31). */
typedef struct loom_b200_decoder loom_b200_decoder;

/* HFDecoderDims (poly/hf_decoder.go:4-16) + vocabulary + MaxSeqLen.  rms_eps is applied like
 * SetRMSNormEps (block norms, MHA layers, final norm; poly/transformer.go:162-175). */
typedef struct loom_b200_decoder_dims {
    int num_layers, hidden, num_heads, num_kv_heads, head_dim, intermediate, vocab;
    double rms_eps, rope_theta;
    int activation;  /* SwiGLU activation: LOOM_B200_ACT_SILU or LOOM_B200_ACT_RELU2 */
    int max_seq_len; /* <= 0 means 2048 */
} loom_b200_decoder_dims;

/* GenMetrics, poly/transformer.go:323-338 (the timing fields) */
typedef struct loom_b200_gen_metrics {
    double prefill_seconds;        /* host clock around the prompt forward */
    double decode_seconds;         /* host clock around the decode loop, tokens copied back */
    double decode_device_seconds;  /* CUDA events around the decode loop */
    int prefill_tokens, generated_tokens;
    double launches_per_token;     /* kernels of this library inside one decode step */
} loom_b200_gen_metrics;

int loom_b200_decoder_create(loom_b200_ctx* ctx, const loom_b200_decoder_dims* dims, loom_b200_decoder** out);
void loom_b200_decoder_destroy(loom_b200_decoder* dec);
/* One decoder block = layers 4b..4b+3.  Gains are host vectors [hidden] or NULL (= 1).  w7 = the packed
 * projections in slab order q, k, v, o, gate, up, down (borrowed; syncBitNetPackedMHA / ...SwiGLU,
 * poly/bitnet_gpu.go:56-115).  Inner-norm vectors (attn_sub_norm / ffn_sub_norm) are host or NULL. */
int loom_b200_decoder_set_block(loom_b200_decoder* dec, int block, const float* norm1_gain, const float* norm2_gain,
                                const loom_b200_weight* const* w7, const float* attn_inner_norm, int attn_inner_len,
                                const float* ffn_inner_norm, int ffn_inner_len);
/* Tied fp32 embedding / LM head [vocab,hidden] in device memory (borrowed) and the final norm gain (host). */
int loom_b200_decoder_set_embeddings(loom_b200_decoder* dec, const float* emb_dev, const float* final_gain);
/* Untied LM head as a packed ternary matrix [vocab, hidden] (borrowed): with an untied head and exact dtypes the
 * reference runs the head itself through the packed-ternary matvec (usePackedTernaryLMHead / applyPackedTernaryLMHead,
 * poly/transformer.go:721-755): logits = float32(packed matvec of the quantized, final-normalised row).  Call it after
 * set_embeddings (which still provides the embedding table); NULL goes back to the tied fp32 head. */
int loom_b200_decoder_set_lm_head_ternary(loom_b200_decoder* dec, const loom_b200_weight* head);
/* Transformer.Reset */
int loom_b200_decoder_reset(loom_b200_decoder* dec);
int loom_b200_decoder_kv_offset(const loom_b200_decoder* dec);
/* ForwardTokenIDsWGPU(tokens, nil, true, true), poly/wgpu_forward.go:31: runs the stack over n token ids and
 * returns the logits of the last one ([vocab], may be NULL to skip the readback).  n > 1 restarts the KV
 * rings (a prompt); n == 1 continues them. */
int loom_b200_decoder_forward(loom_b200_decoder* dec, const int32_t* tokens, int n, float* logits_host);
/* the last token's hidden row after the final RMSNorm [hidden] */
int loom_b200_decoder_last_hidden(loom_b200_decoder* dec, float* hidden_host);
/* Continues the greedy loop for `steps` more tokens from the logits of the last forward, entirely on the
 * device and without waiting for it (call loom_b200_sync to wait).  The body of Generate's loop,
 * poly/transformer.go:434-485. */
int loom_b200_decoder_continue(loom_b200_decoder* dec, int steps);
/* ---- independent sequences on one decoder ---------------------------------------------------------------
 * The reference shares ONE KV ring across a batch: MHAForwardPackedTernaryCPU walks batch*seq rows as consecutive positions
 * of one sequence (poly/mha.go:258-270, poly/mha_layout.go:62-70), so "batch 16" there means sixteen positions, not
 * sixteen sequences.  Serving several sequences at once is therefore an extension, defined by its oracle: the result
 * for every sequence is that of a decoder of its own fed the same tokens.  `batch` KV rings per block share the
 * weights; a decode step carries up to eight sequences per pass over every packed matrix (the M dimension of the
 * GEMV) and several hidden rows per pass over the LM head.  One GPU, or a tensor-parallel group with the peer
 * mailboxes attached and a vocabulary that divides by the group (the sharded head's tail then exchanges the ranks'
 * (maximum, index) pairs).
 *
 * set_batch comes before the first set_block.  select(seq) picks the sequence the single-sequence calls act on
 * (decoder_forward for its prompt, kv_offset, reset, upload/download_cache, last_hidden, read_tokens ...).  step_batch
 * forwards one token per sequence (tokens [batch], or NULL to continue greedily from every sequence's last logits) and
 * returns the logits [batch, vocab] (or NULL to skip the read-back); continue_batch runs `steps` greedy steps for all
 * sequences on the device without waiting; read_tokens_batch returns the last n tokens every sequence fed to a forward,
 * [batch, n].  Every sequence needs a prompt behind it before the first batch call. */
int loom_b200_decoder_set_batch(loom_b200_decoder* dec, int batch);
int loom_b200_decoder_batch(const loom_b200_decoder* dec);
int loom_b200_decoder_select(loom_b200_decoder* dec, int seq);
int loom_b200_decoder_step_batch(loom_b200_decoder* dec, const int32_t* tokens, float* logits_host);
int loom_b200_decoder_continue_batch(loom_b200_decoder* dec, int steps);
int loom_b200_decoder_read_tokens_batch(loom_b200_decoder* dec, int32_t* tokens_host, int n);
/* Cuts the sequence back to its first kv_offset positions (0 < kv_offset <= the current offset), like assigning
 * layer.KVOffset on every MHA layer: the next one-token forward writes position kv_offset.  Ring rows beyond stay
 * until they are overwritten. */
int loom_b200_decoder_set_kv_offset(loom_b200_decoder* dec, int kv_offset);
/* Kernels of this library one greedy decode step launches (argmax included); 1 before the first step was recorded. */
int loom_b200_decoder_step_launches(const loom_b200_decoder* dec);
/* Measurement aid, the counterpart of timing the BitNet dispatches alone (WGPUContext.TimeCommands around
 * DispatchDenseBitNetTernaryQuantized, poly/wgpu_context_native.go:553): enqueues the ternary projections of ONE
 * one-token decode step exactly as the step runs them -- QKV, O, gate+up, down of every block with their fused
 * normalise/quantize prologues and epilogues, on the step's own buffers -- without attention, embedding, head or
 * position update.  May be recorded between graph_begin and graph_end.  The newest K/V ring row and the residual
 * scratch are overwritten; the next real step rewrites both. */
int loom_b200_decoder_linears_frame(loom_b200_decoder* dec);
/* The last n tokens the device-resident greedy loop (decoder_continue / decoder_generate) fed to a forward, oldest
 * first; waits for the device.  n must not exceed the number of such tokens since the last reset. */
int loom_b200_decoder_read_tokens(loom_b200_decoder* dec, int32_t* tokens_host, int n);
/* copies block's KV ring [max_seq_len, kv_heads*head_dim] to the host (layer.KVCacheK / KVCacheV) */
int loom_b200_decoder_download_cache(loom_b200_decoder* dec, int block, float* k_host, float* v_host);
/* The inverse: installs positions 0..kv_offset-1 of block's KV ring from host rows [kv_offset, kv_heads*head_dim]
 * (position-major like layer.KVCacheK / KVCacheV, poly/mha.go:262-270) and, like assigning layer.KVOffset, makes
 * kv_offset the position of the next token for the whole decoder: restoring a saved sequence.  Call it for every
 * block with the same kv_offset before the next one-token forward. */
int loom_b200_decoder_upload_cache(loom_b200_decoder* dec, int block, int kv_offset, const float* k_host, const float* v_host);
/* The residual stream after the last block, before the final norm, for the tokens of the last forward call's last
 * pass (the x that forwardOnCPUNormal returns, poly/transformer_forward.go:236-253): up to max_rows rows of
 * [hidden] floats; *rows_out = rows written.  A prompt of up to 1024 tokens that took the token-block path is one
 * pass; the eight-tokens-per-pass path leaves its last pass. */
int loom_b200_decoder_last_residual(loom_b200_decoder* dec, float* rows_host, int max_rows, int* rows_out);
/* Transformer.Generate with deterministic (greedy) sampling: prefill the prompt, then max_new times
 * {first-maximum token, forward it}.  The loop runs on the device; tokens come back once at the end. */
int loom_b200_decoder_generate(loom_b200_decoder* dec, const int32_t* prompt, int n_prompt, int max_new,
                               int32_t* out_tokens, loom_b200_gen_metrics* metrics);

/* ---- tensor parallelism over the GPUs of one box --------------------------------------------------
 * The reference has no multi-device path (its only sharding notion is the per-layer tile size,
 * poly/wgpu_context.go).  The split used here is the one the integer arithmetic allows without changing a bit
 * of the result: Q/K/V/gate/up hold a contiguous slice of their ROWS (heads, intermediate units), O/down the
 * matching slice of their COLUMNS; the partial int32 accumulators of O/down are summed across ranks (exact),
 * after the ranks have agreed on the per-token sum of squares (float64) and absmax (float32) of the sharded
 * vector.  One process per GPU; each process owns one context.  NCCL is loaded at run time (libnccl.so.2).
 *
 * A weight slice must carry the scale of the WHOLE matrix (absmean over all rows and columns,
 * NewBitNetPackedMatrixFromFloat32, poly/bitnet_cpu.go:97-131): ternarize first, slice the codes after. */

/* Fills id128 (128 bytes) with a fresh NCCL unique id; rank 0 calls it and hands the bytes to every rank. */
int loom_b200_tp_unique_id(uint8_t* id128);
/* Joins the group (collective: every rank calls it with the same id).  world == 1 is accepted and a no-op. */
int loom_b200_tp_init(loom_b200_ctx* ctx, int rank, int world, const uint8_t* id128);
/* Optional, after tp_init: exchange through peer memory instead of NCCL for the row-parallel projections.  Every
 * rank calls tp_peer_handle (allocates its 8.4 MB mailbox, returns a 64-byte CUDA IPC handle), the host gathers the
 * handles of all ranks in rank order (world x 64 bytes, any transport), and every rank calls tp_attach_peers.  The
 * three per-projection exchanges (sum of squares, absmax, int32 accumulators) then travel as 8-byte {value,
 * sequence} stores straight into the receivers' mailboxes over NVLink, inside the library's own kernels; polls are
 * bounded (status word 5, LOOM_B200_ERR_TIMEOUT semantics) so a missing rank cannot hang a GPU.  Option "tp_peer" 0
 * switches back to NCCL.  With the mailboxes the vocabulary-sharded LM head also keeps the greedy step in its tail: the
 * ranks exchange the (maximum, index) pairs of their slices, and the full row of logits is gathered (NCCL) only by calls
 * that return logits to the host -- which every rank must then make alike. */
int loom_b200_tp_peer_handle(loom_b200_ctx* ctx, uint8_t* handle64);
int loom_b200_tp_attach_peers(loom_b200_ctx* ctx, const uint8_t* handles);
/* Leaves the group (also done by loom_b200_ctx_destroy). */
void loom_b200_tp_finalize(loom_b200_ctx* ctx);
int loom_b200_tp_rank(const loom_b200_ctx* ctx);
int loom_b200_tp_world(const loom_b200_ctx* ctx);
/* In-place sum of n int32 values across the group, ordered on the context's stream. */
int loom_b200_tp_allreduce_i32(loom_b200_ctx* ctx, int32_t* buf, size_t n);
/* Row-sharded ternary linear on device buffers: x_local [batch, w->cols] holds this rank's slice of a vector of
 * cols_global entries; the always-on inner RMSNorm (bitNetRMSNormTensorRowWeighted, poly/bitnet_cpu.go:893-913)
 * runs over the whole vector, inner_w_local is this rank's slice of its weight (or NULL).  out [batch, w->rows]
 * = float(sum over ranks of acc * outputScale + bias) + residual, the same bits on every rank and the same bits
 * as the unsharded loom_b200_ternary_linear after loom_b200_inner_rmsnorm.  bias and residual may be NULL;
 * residual may alias out.  batch <= 8. */
int loom_b200_tp_rowsharded_linear(loom_b200_ctx* ctx, const loom_b200_weight* w, int batch, const float* x_local,
                                   int cols_global, const float* inner_w_local, int inner_w_len, double eps,
                                   const float* bias, const float* residual, float* out);
/* With a group of more than one rank on the context, loom_b200_decoder_create takes the UNSHARDED dimensions
 * and builds rank tp_rank's part: num_heads, num_kv_heads and intermediate must be multiples of the world
 * size; loom_b200_decoder_set_block then expects the slices q [heads/W*hd, hidden], k/v [kv_heads/W*hd, hidden],
 * o [hidden, heads/W*hd], gate/up [inter/W, hidden], down [hidden, inter/W] and the matching slices of the
 * inner-norm vectors; embeddings stay whole on every rank, the LM head is computed in vocabulary slices and
 * gathered when vocab is a multiple of the world size.  Every rank makes the same calls with the same tokens
 * and ends with the same logits and tokens. */

#ifdef __cplusplus
}
#endif
#endif
