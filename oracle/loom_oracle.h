/*
 * loom_oracle.h -- CPU restatement of Loom's BitNet ternary x int8 linear path.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker for the CUDA path: it is
 * loaded by the test-suite, by the smoke check and by the benchmark's CPU-baseline
 * leg, and by nothing that ships.  The product library never links or calls it.
 *
 * Every function restates, in plain C++ with IEEE double/float arithmetic and no
 * FMA contraction, the arithmetic of the reference's Go CPU path.  The reference
 * file:line each one follows is given beside its declaration (paths are relative
 * to the openfluke/loom project root).
 *
 * Parity pin: the reference is Go and cannot be compiled where this is built, so
 * the pins are the known-answer tests in the reference's own test files (absmean
 * quantizer, Microsoft offline layout decode, tail columns, dequantised-dense
 * tolerance, SIMD-vs-scalar exact equality), replayed by tests/test_oracle_kat.py.
 */
#ifndef LOOM_ORACLE_H
#define LOOM_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* poly.ActivationType values, poly/poly.go:86-98 */
#define ORC_ACT_RELU 0
#define ORC_ACT_SILU 1
#define ORC_ACT_GELU 2
#define ORC_ACT_TANH 3
#define ORC_ACT_SIGMOID 4
#define ORC_ACT_LEAKY_RELU 5
#define ORC_ACT_RELU2 6
#define ORC_ACT_LINEAR (-1)

/* ---- scalar pieces --------------------------------------------------------- */

/* bitNetTernaryScale, poly/bitnet_cpu.go:119-132 */
float orc_ternary_scale(const float* w, size_t n);
/* bitNetQuantValue, poly/bitnet_cpu.go:134-146; returns -1, 0 or +1 */
int orc_quant_value(float v, float scale);
/* RowWords = ceil(cols/16), poly/bitnet_cpu.go:928 */
int orc_row_words(int cols);
/* packFloat32AsBitNetTernaryMatrix, poly/bitnet_cpu.go:934-962 (+ packTernaryRowsToU32 :964-977).
 * words must hold rows*orc_row_words(cols) zero-initialised or not (it is cleared). Returns 0 on success. */
int orc_pack_f32(const float* w, int rows, int cols, uint32_t* words, float* scale_out);
/* whole-store absmean ternarizer: MorphBitNetTernary, poly/bitnet_cpu.go:151-166. q receives -1/0/+1. */
float orc_morph_ternary(const float* w, size_t n, int8_t* q);
/* packNativeTernaryToBitNetMatrix, poly/bitnet_cpu.go:918-932: q holds -1/0/+1 */
int orc_pack_native(const int8_t* q, int rows, int cols, uint32_t* words);
/* packMicrosoftOfflineBitNetRowsToU32FromBytes, poly/bitnet_cpu.go:1078-1098 */
int orc_pack_microsoft_u8(const uint8_t* packed, int rows, int cols, uint32_t* words);
/* packMicrosoftOfflineBitNetRowsToU32FromFloatU8Slots, poly/bitnet_cpu.go:1056-1076 */
int orc_pack_microsoft_f32slots(const float* packed, int rows, int cols, uint32_t* words);

/* bitNetQuantizeActivationNumeric, poly/bitnet_cpu.go:45-57,73-83,97-106. Returns amax. */
float orc_quantize_f32(const float* x, int n, int8_t* q);
/* bitNetQuantizeActivationFloat64, poly/bitnet_cpu.go:59-71,85-95,108-117 */
float orc_quantize_f64(const double* x, int n, int8_t* q);

/* int32 accumulators of bitNetTernaryMatVecInt8Scalar, poly/bitnet_cpu.go:752-776,810-854 */
void orc_matvec_i32(const uint32_t* words, int rows, int cols, const int8_t* xq, int32_t* acc);
/* scalar twin of simd.BitNetTernaryCodeRowDot, poly/simd/bitnet_ternary.go:18-24 */
int32_t orc_code_row_dot_scalar(const uint8_t* codes, const int8_t* acts, int nbytes);
/* AVX2 twin, poly/simd/bitnet_ternary_amd64.s:7-39 (falls back to scalar without AVX2) */
int32_t orc_code_row_dot_avx2(const uint8_t* codes, const int8_t* acts, int nbytes);
int orc_has_avx2(void);

/* swigluGateProduct, poly/swiglu.go:37-46 */
double orc_gate_product(double g, double u, int activation);
/* Activate[float32], poly/poly.go:167-200 */
float orc_activate_f32(float v, int activation);
/* bitNetRMSNormTensorRowWeighted, poly/bitnet_cpu.go:893-913 (in place) */
void orc_inner_rmsnorm_f32(float* data, int n, const float* weight, int weight_len, double eps);
/* bitNetRMSNormFloat64Weighted, poly/bitnet_cpu.go:868-887 (in place) */
void orc_inner_rmsnorm_f64(double* data, int n, const float* weight, int weight_len, double eps);
/* RMSNormForwardPolymorphic, poly/norm.go:102-138: rows x n; rms_out (rows) may be NULL */
void orc_block_rmsnorm(const float* in, int rows, int n, const float* gain, double eps, float* out, float* rms_out);

/* ---- packed matrix object ---------------------------------------------------- */

typedef struct orc_matrix orc_matrix; /* BitNetTernaryMatrix, poly/bitnet_cpu.go:16-43 */

orc_matrix* orc_matrix_from_words(const uint32_t* words, int rows, int cols, float scale);
orc_matrix* orc_matrix_from_f32(const float* w, int rows, int cols); /* GetBitNetTernaryMatrix from Master, :345-354 */
void orc_matrix_free(orc_matrix* m);
int orc_matrix_rows(const orc_matrix* m);
int orc_matrix_cols(const orc_matrix* m);
int orc_matrix_row_words(const orc_matrix* m);
float orc_matrix_scale(const orc_matrix* m);
void orc_matrix_set_scale(orc_matrix* m, float scale); /* SetBitNetPackedScale, :979-993 */
const uint32_t* orc_matrix_words(const orc_matrix* m);

/* bitNetTernaryMatVecQuantized, poly/bitnet_cpu.go:536-566 (+ :733-776 variants, :780-808 row fan-out).
 * simd: 0 = scalar word decode, 1 = byte-code AVX2 MAD path.  threads: the GOMAXPROCS stand-in. */
int orc_matrix_matvec(orc_matrix* m, const int8_t* xq, float amax, double* out, int simd, int threads);

/* ---- layers -------------------------------------------------------------------- */

/* DenseForwardPackedTernaryCPU, poly/dense.go:66-101.  in [batch,K]; pre/post [batch,N]. */
int orc_dense_forward(orc_matrix* w, int activation, const float* in, int batch, float* pre, float* post,
                      int simd, int threads);

/* SwiGLUForwardPackedTernaryCPU, poly/swiglu.go:270-322.  in [seq,H]; pre [seq,I] (normalised gate
 * product); post [seq,H].  Biases may be NULL (zero).  Optional taps (may be NULL): q_in [seq,H] int8,
 * amax_in [seq], raw_prod [seq,I] (gate product before the inner norm), q_pre [seq,I], amax_pre [seq]. */
int orc_swiglu_forward(orc_matrix* gate, orc_matrix* up, orc_matrix* down, const float* bias_gate,
                       const float* bias_up, const float* bias_down, const float* inner_w, int inner_w_len,
                       double rms_eps, int activation, const float* in, int seq, float* pre, float* post,
                       int8_t* q_in, float* amax_in, float* raw_prod, int8_t* q_pre, float* amax_pre, int simd,
                       int threads);

typedef struct orc_mha orc_mha; /* the MHA VolumetricLayer with its ring KV cache */

/* fields of VolumetricLayer used by MHAForwardPackedTernaryCPU, poly/mha.go:204-371.
 * Matrices are borrowed (not freed by orc_mha_free).  Bias / norm pointers are copied; NULL = absent. */
orc_mha* orc_mha_create(int d_model, int num_heads, int num_kv_heads, int head_dim, int max_seq_len,
                        double rope_theta, double rms_eps, orc_matrix* wq, orc_matrix* wk, orc_matrix* wv,
                        orc_matrix* wo, const float* bq, const float* bk, const float* bv, const float* bo,
                        const float* q_norm_w, int q_norm_len, const float* k_norm_w, int k_norm_len,
                        const float* inner_w, int inner_w_len);
void orc_mha_free(orc_mha* l);
void orc_mha_reset(orc_mha* l); /* Transformer.Reset: KVOffset = 0, poly/transformer.go:119-127 */
int orc_mha_kv_offset(const orc_mha* l);
/* installs a KV ring state (layer.KVCacheK/V + KVOffset) so that a decode step can be timed or checked at a
 * given context length without replaying the prompt; k, v are [max_seq_len, kvDim] */
int orc_mha_set_state(orc_mha* l, int kv_offset, const float* k, const float* v);
const float* orc_mha_cache_k(const orc_mha* l); /* [max_seq_len, kvDim] */
const float* orc_mha_cache_v(const orc_mha* l);
/* in [batch,seq,dModel].  pre (normalised attention rows) and post [batch,seq,dModel].  Optional taps:
 * q_f64 [batch*seq,qDim] after q-norm and RoPE; attn_f64 [batch*seq,qDim] before the inner norm.
 * attn_threads > 1 splits (token,head) pairs across threads; each pair's arithmetic is unchanged. */
int orc_mha_forward(orc_mha* l, const float* in, int batch, int seq, float* pre, float* post, double* q_f64,
                    double* attn_f64, int simd, int threads, int attn_threads);

/* ---- decoder (InitHFDecoderBlocks + Transformer) -------------------------------------- */

typedef struct orc_decoder orc_decoder;

/* HFDecoderDims, poly/hf_decoder.go:4-16; rms_eps applied like SetRMSNormEps (poly/transformer.go:162-175):
 * block norms, MHA layers and the final norm; the SwiGLU inner norm keeps its 1e-5 default. */
orc_decoder* orc_decoder_create(int num_layers, int hidden, int num_heads, int num_kv_heads, int head_dim,
                                int intermediate, int vocab, double rms_eps, double rope_theta, int activation,
                                int max_seq_len);
void orc_decoder_free(orc_decoder* d);
/* Block weights: fp32 masters of each projection are ternarised per matrix exactly as
 * PrepareDecoderBlockBitNetTernaryCPU does (poly/bitnet_cpu.go:376-394, 437-487).  Gains may be NULL (1.0). */
int orc_decoder_set_block(orc_decoder* d, int block, const float* norm1_gain, const float* wq, const float* wk,
                          const float* wv, const float* wo, const float* norm2_gain, const float* w_gate,
                          const float* w_up, const float* w_down);
/* same, from already packed words + scales (order q,k,v,o,gate,up,down) */
int orc_decoder_set_block_packed(orc_decoder* d, int block, const float* norm1_gain, const float* norm2_gain,
                                 const uint32_t* const* words7, const float* scales7);
/* tied fp32 embedding / LM head [vocab,hidden] (borrowed pointer: must outlive the decoder) and final gain */
int orc_decoder_set_embeddings(orc_decoder* d, const float* emb, const float* final_gain);
void orc_decoder_reset(orc_decoder* d);
/* Untied LM head as a packed ternary matrix [vocab, hidden] (usePackedTernaryLMHead / applyPackedTernaryLMHead,
 * poly/transformer.go:721-755): the logits are float32(packed matvec of the quantized normalised row).  Borrowed pointer;
 * NULL goes back to the tied fp32 head. */
int orc_decoder_set_lm_head_ternary(orc_decoder* d, orc_matrix* head);
/* orc_mha_set_state on one block */
int orc_decoder_set_kv(orc_decoder* d, int block, int kv_offset, const float* k, const float* v);
/* forwardOnCPUNormal over n tokens (poly/transformer_forward.go:220-253) then ApplyLMHead on the last row
 * (poly/transformer.go:635-719).  hidden_out [n,hidden] and logits_out [vocab] may be NULL. */
int orc_decoder_forward(orc_decoder* d, const int32_t* tokens, int n, float* hidden_out, float* logits_out,
                        int simd, int threads, int attn_threads);
/* the same forward; block_out (may be NULL) receives the residual stream after every block, [layers][n][hidden]:
 * the x that forwardOnCPUNormal hands from block to block (poly/transformer_forward.go:236-251) */
int orc_decoder_forward_taps(orc_decoder* d, const int32_t* tokens, int n, float* hidden_out, float* logits_out,
                             float* block_out, int simd, int threads, int attn_threads);
/* Generate's greedy loop (poly/transformer.go:341-485, poly/sampling.go:44-55): prefill the prompt, then
 * max_new tokens.  out_tokens [max_new].  decode_seconds (may be NULL) = wall time of the decode loop. */
int orc_decoder_generate(orc_decoder* d, const int32_t* prompt, int n_prompt, int max_new, int32_t* out_tokens,
                         double* prefill_seconds, double* decode_seconds, int simd, int threads,
                         int attn_threads);
/* first index of the maximum, poly/sampling.go:45-55 */
int orc_argmax(const float* logits, int n);
/* applyFP32LMHeadRows, poly/transformer.go:659-719 */
void orc_lm_head(const float* hidden, const float* head, int vocab, int hidden_size, float* logits, int threads);

#ifdef __cplusplus
}
#endif
#endif
