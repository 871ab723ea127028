/*
 * tpx_b200 — C ABI of the B200 (sm_100a) implementation of the LLM-inference hot path of
 * libxsmm/tpp-pytorch-extension: weight-only quantized linear (MXFP4 / int8 weights, bf16
 * activations, fused bias / GeLU / SiLU / mul / residual epilogues), RMSNorm, RoPE + KV-cache
 * write and attention over the blocked KV cache.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in _host;
 *   - bf16 tensors are passed as uint16_t bit patterns, row-major, contiguous;
 *   - every call enqueues work on `stream` (a cudaStream_t passed as void*) and returns without
 *     synchronising; nothing allocates device memory: scratch is passed in by the caller;
 *   - return value 0 = success; otherwise a TPX_ERR_* code, with text from tpx_last_error().
 *     The reference aborts the process on its own argument checks (TPP_ASSERT -> exit(1),
 *     src/csrc/utils.h:34-41); this library reports instead.
 *
 * Each declaration cites the reference interface it replaces (paths relative to the reference
 * repository root).
 */
#ifndef TPX_B200_H
#define TPX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  TPX_OK = 0,
  TPX_ERR_ARG = 1,      /* bad shape / pointer / alignment                         */
  TPX_ERR_UNSUPPORTED = 2,
  TPX_ERR_CUDA = 3,     /* a CUDA runtime call failed; see tpx_last_error()        */
  TPX_ERR_SCRATCH = 4   /* scratch buffer too small                                */
};

/* activation selector of the fused epilogue (post-ops of src/csrc/fused_gemm.h:1343-1410) */
enum { TPX_ACT_NONE = 0, TPX_ACT_GELU = 1, TPX_ACT_SILU = 2, TPX_ACT_RELU = 3 };

/* weight kinds (dispatch of src/csrc/fused_gemm.h:1509-1597) */
enum { TPX_W_MXFP4 = 1, TPX_W_INT8 = 2 };

int tpx_version(void);
const char* tpx_last_error(void);
/* number of SMs of the current device (used by callers to size scratch) */
int tpx_sm_count(void);
/* The kernel-selection switches (TPX_TC_WHOLE, TPX_TC_WIDE, TPX_TC_F4, TPX_TC_CLUSTER, TPX_TC_PF, TPX_ATTN_SPLITS) are
 * read from the environment once, at first use; this call reads them again. None of them changes a result; they exist
 * so that tests can run every kernel family. No counterpart in the reference.                                     */
void tpx_reload_options(void);
/* Number of kernels of the linear / norm / rope / attention path this library has launched so far in this process
 * (host-side tally, for benchmarks that report their launch count). No counterpart in the reference.          */
unsigned long long tpx_launch_count(void);

/* out256[b] = the two fp16 values (low half = low nibble) that the GPU's own E2M1 decoder makes of byte b: the element
 * table of the MXFP4 codes (src/csrc/qtypes.cpp:42-57) as this hardware implements it. 256 words of device memory. */
int tpx_e2m1_pair_table(uint32_t* out256, void* stream);

/* ---------------------------------------------------------------- quantize / remap
 * Replaces _C._qtype.remap_and_quantize_mxfp4 (src/csrc/qtypes.cpp:783-864, pybind :1086).
 * in:  blocked bf16 weight [K1][C1][C2][K2][C3] as BlockedParameter.block() lays it out
 *      (src/tpp_pytorch_extension/utils/blocked_layout.py:268-292), C3 = 2.
 * out: codes  uint8 [K1*K2/32][C1][C2][32]   (two E2M1 codes per byte, low nibble = even lane)
 *      scales uint8 [K1*K2/32][C1][C2*2/32][32]  (UE8M0)
 * i.e. the storage of the reference's quantized tensor, bit for bit.                       */
int tpx_remap_and_quantize_mxfp4(const uint16_t* blocked, int64_t K1, int64_t C1, int64_t C2, int64_t K2,
                                 int64_t C3, uint8_t* codes, uint8_t* scales, void* stream);

/* Replaces _C._qtype.remap_and_quantize_qint8 (src/csrc/qtypes.cpp:866-932, pybind :1087).
 * block_size plays the role of the QINT8_BLOCK_SIZE environment variable (:28), and is
 * adjusted as the reference does when it does not divide K (:878-889: the largest power of two
 * from 4096 down to 64 below the request that divides K, else the blocked tensor's own C2*C3);
 * the block size actually used, B, is returned through *block_size_used. block_size must be a
 * positive multiple of 4. scales_capacity is the number of floats `scales` can hold; the call
 * refuses (TPX_ERR_ARG) when B needs more than that.
 * out: q int8 [K1][C/B][B/4][K2][4], scales fp32 [K1][C/B][1][K2].                         */
int tpx_remap_and_quantize_qint8(const uint16_t* blocked, int64_t K1, int64_t C1, int64_t C2, int64_t K2,
                                 int64_t C3, int64_t block_size, int8_t* q, float* scales,
                                 int64_t scales_capacity, int64_t* block_size_used, void* stream);

/* Replaces Tensor.dequantize() on the two quantized carriers
 * (PerBlockMxFPQuantizer::dequantize src/csrc/qtypes.cpp:438-445, PerBlockAffineQuantizer
 * :521-560): fp32 output in the same blocked 5-D shape as the quantizer input.            */
int tpx_dequantize_mxfp4(const uint8_t* codes, const uint8_t* scales, int64_t K1, int64_t C1, int64_t C2,
                         int64_t K2, float* out, void* stream);
int tpx_dequantize_qint8(const int8_t* q, const float* scales, int64_t K1, int64_t C1, int64_t C2,
                         int64_t K2, float* out, void* stream);

/* ---------------------------------------------------------------- device repack
 * The reference keeps one blocked layout and, for prefill, a second copy with merged blocks
 * (wt_tensor_for_first_token, src/csrc/llm/fused_llm_infer.cpp:365-420). Here the interchange
 * tensors above are re-laid once into the streaming layout the kernels read:
 *   MXFP4 tiles  [N/16][Kp/128] of 1088 bytes: codes [2][32 lanes][16 B], then scales [16 rows][4]
 *                (scales_bytes is 0: they ride inside the tiles; pk_scales may be NULL)
 *   int8  values [N/16][K/64][2][32 lanes][16 B],  scales fp32 [N/16][K/B][16 rows]
 * (Kp = K rounded up to 128; the padding holds zero codes).
 * tpx_packed_bytes returns the byte sizes of the two outputs.                              */
int tpx_packed_bytes(int kind, int64_t N, int64_t K, int64_t block_size, size_t* codes_bytes,
                     size_t* scales_bytes);
int tpx_repack_mxfp4(const uint8_t* codes, const uint8_t* scales, int64_t N, int64_t K, uint8_t* pk_codes,
                     uint8_t* pk_scales, void* stream);
int tpx_repack_qint8(const int8_t* q, const float* scales, int64_t N, int64_t K, int64_t block_size,
                     uint8_t* pk_codes, float* pk_scales, void* stream);
/* ---------------------------------------------------------------- quantized linear
 * Replaces GemmCaller / fc_plain with a post-op (src/csrc/fused_gemm.h:1509-1650) and
 * torch.ops.tpp_llm.fc_plain (src/csrc/llm/fused_llm_infer.cpp:1514-1566):
 *     y[M][N] = epilogue( x[M][K] . dequant(W)[N][K]^T + bias[N] )
 *     epilogue(v) = act(v) * mul_in[M][N] (MulPostOp) + res[M][N] * res_scale (AddScalePostOp)
 * With pk_codes2 != NULL the call computes the gate/up pair of the SwiGLU MLP in one pass
 * (the reference issues SiluPostOp then MulPostOp, fused_llm_infer.cpp:1271-1272):
 *     y = act(x.W^T) * (x.W2^T)
 * NULL for bias / mul_in / res / pk_codes2 means "absent" (the reference's empty tensor).
 * fp32 accumulation, one bf16 rounding at the store.
 * scratch: tpx_qlinear_scratch_bytes(...) bytes, 256-byte aligned. Its first 64 KiB (arrival counters,
 * and an error word at byte 65532 that a kernel sets if a bounded wait inside it gave up) must be
 * zero-filled once by the caller before first use; the kernels leave the counters zeroed. Calls that
 * share a scratch buffer must not overlap on the device.                                    */
size_t tpx_qlinear_scratch_bytes(int kind, int64_t M, int64_t N, int64_t K, int64_t block_size, int dual);
int tpx_qlinear(int kind, const uint8_t* pk_codes, const void* pk_scales, const uint8_t* pk_codes2,
                const void* pk_scales2, int64_t block_size, const uint16_t* x, int64_t M, int64_t N,
                int64_t K, const uint16_t* bias, int act, const uint16_t* mul_in, const uint16_t* res,
                float res_scale, uint16_t* y, void* scratch, size_t scratch_bytes, void* stream);

/* ---------------------------------------------------------------- MXFP4 linear on the tcgen05 tensor cores
 * Same contract as tpx_qlinear for MXFP4 weights (it replaces the same reference interfaces), with the
 * weight in the layout the tensor-core path reads (TN = ceil(N/128); KS = ceil(K/128) rounded up to a
 * multiple of 4 for one weight, of 2 for a gate/up pair; padding holds zero codes):
 *   one weight : wq [TN][KS][128 rows][64 bytes]      sfa [TN][KS][512]
 *   gate/up    : wq [TN][KS][2][128 rows][64 bytes]   sfa [TN][KS][2][512]
 * wq holds packed E2M1 codes, low nibble = even k, unpacked by TMA; byte (r%32)*16 + (r/32)*4 + j of a
 * 512-byte scale block is the UE8M0 scale of row r of the tile for the j-th 32-wide block of the k step.
 * Both are built by tpx_repack_mxfp4_tc from the interchange tensors of tpx_remap_and_quantize_mxfp4
 * (codes2/scales2 NULL = one weight). With pair != 0 the linear computes y = act(x.Wg^T) * (x.Wu^T).
 * Activations are split on the device into two E4M3 terms with a shared power-of-two block scale
 * (exact for bf16 inputs within 2^-10 of their block maximum). The scratch buffer holds those terms and the
 * partial tiles; its first 64 KiB must be zero before first use, as for tpx_qlinear. x and y may also be
 * pinned (page-locked, device-addressable) host memory: the kernels then read x and write y across the bus.   */
int tpx_tc_packed_bytes(int64_t N, int64_t K, int pair, size_t* wq_bytes, size_t* sfa_bytes);
int tpx_repack_mxfp4_tc(const uint8_t* codes, const uint8_t* scales, const uint8_t* codes2, const uint8_t* scales2,
                        int64_t N, int64_t K, uint8_t* wq, uint8_t* sfa, void* stream);
size_t tpx_qlinear_mxfp4_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int pair);
int tpx_qlinear_mxfp4_tc(const uint8_t* wq, const uint8_t* sfa, int pair, const uint16_t* x, int64_t M, int64_t N,
                         int64_t K, const uint16_t* bias, int act, const uint16_t* mul_in, const uint16_t* res,
                         float res_scale, uint16_t* y, void* scratch, size_t scratch_bytes, void* stream);

/* RMSNorm followed by the linear, the pair the reference's decoder block runs before q/k/v and before gate/up
 * (llama_rms_norm then the fused loop nests, src/csrc/llm/fused_llm_infer.cpp:1204-1272): x is normalised
 * (y = bf16(x * rsqrt(mean(x^2) + eps) * gamma), gamma bf16 or fp32) on its way into the activation split, so the
 * normalised tensor never goes to memory. Rows of up to 8192 elements; otherwise as tpx_qlinear_mxfp4_tc.     */
int tpx_rmsnorm_qlinear_mxfp4_tc(const uint8_t* wq, const uint8_t* sfa, int pair, const uint16_t* x, const void* gamma,
                                 int gamma_is_f32, float eps, int64_t M, int64_t N, int64_t K, const uint16_t* bias, int act,
                                 const uint16_t* mul_in, const uint16_t* res, float res_scale, uint16_t* y, void* scratch,
                                 size_t scratch_bytes, void* stream);

/* The same linear for callers that cannot allocate device memory where they call it (all free memory already
 * handed to a cache pool, a fixed budget inside another framework, a thread that must stay off the allocator's
 * locks). It has no counterpart in the reference. Its scratch is an 8 MiB array built into the library
 * (tpx_qlinear_mxfp4_tc_static_max_bytes). Where the kernel family the planner would pick needs more scratch than
 * that, the call runs the family with the smallest scratch instead; a shape that fits neither is refused with
 * TPX_ERR_SCRATCH. The call allocates nothing. The first call on each device looks up the
 * array's device address and should therefore come before any stream capture. All calls on one GPU share the
 * array: two of them in flight at once (different streams) corrupt each other; serialise them.
 * A kernel that gave up on one of its bounded waits leaves a non-zero code in a word of the array; the word stays set
 * across later calls until tpx_qlinear_mxfp4_tc_static_status copies it to *status_host and clears it (that call
 * waits for `stream`). 0 = every call since the last read completed normally.                                  */
size_t tpx_qlinear_mxfp4_tc_static_max_bytes(void);
int tpx_qlinear_mxfp4_tc_static_status(void* stream, unsigned* status_host);
int tpx_qlinear_mxfp4_tc_static(const uint8_t* wq, const uint8_t* sfa, int pair, const uint16_t* x, int64_t M,
                                int64_t N, int64_t K, const uint16_t* bias, int act, const uint16_t* mul_in,
                                const uint16_t* res, float res_scale, uint16_t* y, void* stream);

/* ---------------------------------------------------------------- bf16-weight linear on the tcgen05 tensor cores
 * Replaces fc_plain on an unquantized bf16 weight (TppBlockedLinearW<bf16>, src/csrc/fused_gemm.h:784-1073, reached from
 * torch.ops.tpp_llm.fc_plain, src/csrc/llm/fused_llm_infer.cpp:1514-1566): on the decoder path this is the lm_head, which
 * the reference leaves in bf16 unless it is asked to quantize it (examples/llm/run_generation.py:277-282).
 *     y[M][N] = epilogue(x[M][K] . w[N][K]^T + bias[N]),   epilogue as for tpx_qlinear
 * w is the plain row-major weight (nn.Linear.weight), not re-laid out; K a multiple of 8; any M and N. fp32
 * accumulation, one bf16 rounding at the store. The scratch (tpx_linear_bf16_tc_scratch_bytes, 64 KiB, zero before
 * first use, 256-byte aligned) only carries the error word of the bounded waits at byte 65532.                    */
size_t tpx_linear_bf16_tc_scratch_bytes(int64_t M, int64_t N, int64_t K);
int tpx_linear_bf16_tc(const uint16_t* w, const uint16_t* x, int64_t M, int64_t N, int64_t K, const uint16_t* bias, int act,
                       const uint16_t* mul_in, const uint16_t* res, float res_scale, uint16_t* y, void* scratch,
                       size_t scratch_bytes, void* stream);

/* ---------------------------------------------------------------- int8 linear on the tcgen05 tensor cores
 * Any number of tokens (tiles of 16, 32, 64 or 128 tokens x 128 features) with the reference's own int8 arithmetic
 * (TppBlockedQInt8LinearW, src/csrc/fused_gemm.h:1075-1341):
 * the activations are quantised on the fly to int8 with one scale per (token, K block) (:1249), each K block is an
 * int8 x int8 -> int32 product and y accumulates tmp * s_x * s_w (:1197-1204); the running sum stays in fp32 where
 * the reference rounds it to bf16 after every block. wq is the plain int8 weight [ceil(N/128)*128][ceil(K/128)*128]
 * (zero padding) and swT its scales [K/block][ceil(N/128)*128], both built by tpx_repack_qint8_tc from the
 * interchange tensors of tpx_remap_and_quantize_qint8. Block sizes 64, 128, 256, 512. Post-ops as tpx_qlinear. The
 * scratch holds the quantised activations; its first 64 KiB as for tpx_qlinear. reuse_act != 0 skips the quantisation
 * and reads what the previous call on the same scratch left there (same x, same K and block size: the second linear
 * of a gate/up pair). gamma != NULL applies an RMSNorm (gamma bf16 or fp32, eps) to x before the quantisation, in the
 * same kernel (rows of up to 8192 values, blocks of up to 256).                                                    */
int tpx_tc_packed_bytes_qint8(int64_t N, int64_t K, int64_t block_size, size_t* wq_bytes, size_t* sw_bytes);
int tpx_repack_qint8_tc(const int8_t* q, const float* scales, int64_t N, int64_t K, int64_t block_size, int8_t* wq,
                        float* swT, void* stream);
/* The packed int8 weight of tpx_repack_qint8_tc as a plain bf16 matrix w[N][K] = bf16(q * s): what the host feeds
 * tpx_linear_bf16_tc for more than 128 tokens, where the per-block drain of the int8 kernel costs more than its MMAs
 * (weight-only arithmetic with bf16 activations: the reference's QINT8_EMU mode, src/csrc/qtypes.cpp:27, :928-930).     */
int tpx_unpack_qint8_tc_bf16(const int8_t* wq, const float* swT, int64_t N, int64_t K, int64_t block_size, uint16_t* w_bf16,
                             void* stream);
size_t tpx_qlinear_qint8_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int64_t block_size);
int tpx_qlinear_qint8_tc(const int8_t* wq, const float* swT, const uint16_t* x, const void* gamma, int gamma_is_f32,
                         float eps, int64_t M, int64_t N, int64_t K, int64_t block_size, int reuse_act, const uint16_t* bias, int act, const uint16_t* mul_in,
                         const uint16_t* res, float res_scale, uint16_t* y, void* scratch, size_t scratch_bytes, void* stream);

/* ---------------------------------------------------------------- decoder-layer pieces
 * RMSNorm: y = x * rsqrt(mean(x^2) + eps) * gamma, fp32 statistics. Replaces llama_rms_norm
 * (src/csrc/llm/fused_llm_infer.cpp:336-363; RMSNormFwdTPP::ref src/csrc/xsmm_functors.h:4628-4654).
 * gamma is bf16 or, with gamma_is_f32 != 0, fp32 (the reference accepts either, :346-357).             */
int tpx_rmsnorm(const uint16_t* x, const void* gamma, int gamma_is_f32, float eps, int64_t rows, int64_t D,
                uint16_t* y, void* stream);

/* LayerNorm: y = (x - mean) * rsqrt(var + eps) * gamma + beta, fp32 statistics, variance around the mean. Replaces
 * lyr_norm (src/csrc/llm/fused_llm_infer.cpp:256-306; LayerNormFwdTPP src/csrc/xsmm_functors.h:4720), the norm of the
 * OPT and GPT-J decoder blocks. gamma and beta are both bf16 or, with params_are_f32 != 0, both fp32.           */
int tpx_layernorm(const uint16_t* x, const void* gamma, const void* beta, int params_are_f32, float eps, int64_t rows,
                  int64_t D, uint16_t* y, void* stream);

/* Greedy sampling: out[r] = index of the largest of x[r][0..n), the first among equals, NaN above every number, as
 * torch.argmax(-1) of the head's logits returns it (the reference drives HF generate with --greedy,
 * examples/llm/run_generation.py:337-339). x bf16 [rows][n], out int64 [rows].                          */
int tpx_argmax_bf16(const uint16_t* x, int64_t rows, int64_t n, int64_t* out, void* stream);

/* RoPE + KV-cache append in one pass. Replaces apply_rotary_pos_emb_llama on q and k
 * (src/csrc/llm/fused_llm_infer.cpp:206-253), the q/k/v views and the q permute of self_mha (:563-584) and
 * TppCache::update -> LayerCache::update (src/csrc/llm/attn.h:197-221, KVLayout_BNSH src/csrc/llm/attn.cpp:389-463).
 *   qkv   [B*S][(Nq + 2*Nkv)*H] bf16: output of the fused q/k/v linear (q heads, k heads, v heads)
 *   ep    [2][MP][HR] fp32 (0 = cos, 1 = sin), pos int64 [Bpos][S] with Bpos 1 or B
 *   q_out [B][Nkv][S][Nq/Nkv][H] rotated queries
 *   kc,vc [capacity/32][B][Nkv][32][H] cache tensors; the S new tokens land at offset .. offset+S-1
 * The caller owns the cache tensors and their growth (the reference grows by offset + S + KV_CACHE_INC_SIZE,
 * attn.h:171-177); this call refuses a write beyond `capacity` tokens. With dev_len != NULL the offset is read
 * on the device from *dev_len instead of the `offset` argument (a decode step recorded once in a CUDA graph and
 * replayed keeps its lengths in device memory); writes beyond `capacity` are then dropped by the kernel.     */
int tpx_rope_kv_update(const uint16_t* qkv, const float* ep, const int64_t* pos, int64_t B, int64_t S, int64_t Nq,
                       int64_t Nkv, int64_t H, int64_t MP, int64_t HR, int64_t Bpos, int64_t offset, int64_t capacity,
                       const int32_t* dev_len, uint16_t* q_out, uint16_t* kc, uint16_t* vc, void* stream);

/* The same for GPT-J (apply_rotary_pos_emb_gptj, src/csrc/llm/fused_llm_infer.cpp:150-204): the first HR values of every q
 * and k head rotate in adjacent pairs (2i, 2i+1) with ep [MP][HR] fp32 (HR/2 sines, then HR/2 cosines), the rest of the head
 * passes through; q permute and cache append as tpx_rope_kv_update. The cache is given as tensors (kc, vc) or, when
 * k_pages != NULL, as page tables.                                                                                */
int tpx_rope_kv_update_gptj(const uint16_t* qkv, const float* ep, const int64_t* pos, int64_t B, int64_t S, int64_t Nq, int64_t Nkv,
                            int64_t H, int64_t MP, int64_t HR, int64_t Bpos, int64_t offset, int64_t capacity, const int32_t* dev_len,
                            uint16_t* q_out, uint16_t* kc, uint16_t* vc, const uint64_t* k_pages, const uint64_t* v_pages, void* stream);

/* Attention over the blocked cache. Replaces attn<T> (src/csrc/llm/attn.cpp:780-955):
 *   out = softmax(q.k^T / sqrt(H) + am[b][key], causal: key <= key_len - Sq + query) . v
 * q/out [B][Nkv][Sq][R][H] (GQA group folded into the row dimension, attn.cpp:793-795), am additive bf16 mask
 * [B][Spad] or NULL (0 keep, finfo.min drop; attn.h:310-322). Scores and the output are accumulated in fp32 on
 * the tensor cores (bf16 operands: the probabilities are rounded to bf16 before they meet the values, as a bf16
 * batch-reduce GEMM would), softmax in fp32, one bf16 rounding of the output. With a long cache and few (batch,
 * head) pairs the key range is split over CTAs (flash-decoding); the split that finishes last merges them. The
 * scratch holds arrival counters and the un-normalised partials: it must be 16-byte aligned and zero-filled once
 * before first use (the kernel leaves the counters zero); calls sharing it must not overlap. out_bsnrh != 0
 * writes out as [B][Sq][Nkv][R][H], i.e. already as the [B*Sq][Nq*H] rows of the output projection (the
 * reference permutes and copies, src/csrc/llm/fused_llm_infer.cpp:581). With dev_len != NULL the number of keys
 * is *dev_len + Sq, read on the device; `key_len` is then only the planning maximum (cache capacity).         */
size_t tpx_attention_scratch_bytes(int64_t B, int64_t Nkv, int64_t Sq, int64_t R, int64_t H, int64_t key_len);
int tpx_attention(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, const uint16_t* am, int64_t B, int64_t Nkv,
                  int64_t Sq, int64_t R, int64_t H, int64_t key_len, int64_t Spad, int causal, int out_bsnrh,
                  const int32_t* dev_len, uint16_t* out, void* scratch, size_t scratch_bytes, void* stream);

/* Paged form of the two calls above. The cache of one layer is a sequence of 32-token pages, each a separate
 * [B][Nkv][32][H] slab (what one index of the reference's leading cache dimension holds, src/csrc/llm/attn.h:144-153);
 * k_pages / v_pages are DEVICE arrays of the pages' device addresses, entry i for tokens 32i .. 32i+31. A cache grows by
 * appending pages, where the reference allocates a larger tensor and copies (src/csrc/llm/attn.h:162-178); nothing
 * already cached moves. Everything else as tpx_rope_kv_update / tpx_attention (`capacity` = 32 x the number of pages).
 * Prompts on a paged cache run on the mma.sync attention kernel (the TMA kernel needs one contiguous tensor).      */
int tpx_rope_kv_update_paged(const uint16_t* qkv, const float* ep, const int64_t* pos, int64_t B, int64_t S, int64_t Nq,
                             int64_t Nkv, int64_t H, int64_t MP, int64_t HR, int64_t Bpos, int64_t offset, int64_t capacity,
                             const int32_t* dev_len, uint16_t* q_out, const uint64_t* k_pages, const uint64_t* v_pages, void* stream);
int tpx_attention_paged(const uint16_t* q, const uint64_t* k_pages, const uint64_t* v_pages, const uint16_t* am, int64_t B, int64_t Nkv,
                        int64_t Sq, int64_t R, int64_t H, int64_t key_len, int64_t Spad, int causal, int out_bsnrh,
                        const int32_t* dev_len, uint16_t* out, void* scratch, size_t scratch_bytes, void* stream);

/* The prefill kernel behind tpx_attention (64 query rows or more per (batch, kv head): tcgen05 tensor cores, K/V tiles by
 * TMA; cache slots past key_len must hold finite values, as a zero-initialised or cropped cache does) has no scratch to
 * report through: a bounded wait that gave up leaves a code in a word inside the library. This call copies that word
 * to *status_host and clears it (it waits for `stream`). 0 = every call since the last read completed normally.
 * No counterpart in the reference.                                                                              */
int tpx_attention_tc_status(void* stream, unsigned* status_host);

/* ---------------------------------------------------------------- 8-bit floating-point weights
 * The reference stores a linear's weight as bfloat8 (E5M2) or hfloat8 (E4M3) when asked to (--weight-dtype bfloat8 /
 * hfloat8: src/tpp_pytorch_extension/llm/llm_common.py:519-522 casts the blocked weight) and multiplies through
 * TppBlockedLinearW<Tin, bfloat8 / hfloat8, Tout> (src/csrc/fused_gemm.h:1558-1565): bf16 activations, the weight
 * converted up, fp32 accumulation, the same post-ops. Here the bytes go to the tensor cores as they are
 * (tcgen05.mma kind::mxf8f6f4 with the weight as an E4M3 / E5M2 operand and unit block scales) against the two-term
 * E4M3 split of the activations that the MXFP4 path uses. tpx_repack_fp8_tc tiles a plain [N][K] byte matrix (w2 != NULL:
 * a gate/up pair) into wq [TN][KS][(2)][128 rows][128 bytes] + sfa (constant scale blocks), sizes from
 * tpx_fp8_tc_packed_bytes; tpx_qlinear_fp8_tc has the contract of tpx_qlinear_mxfp4_tc plus the weight format and an
 * optional RMSNorm of x (gamma NULL: none). N % 32 == 0, K % 64 == 0.                                              */
enum { TPX_FP8_E4M3 = 1, TPX_FP8_E5M2 = 2 };
int tpx_fp8_tc_packed_bytes(int64_t N, int64_t K, int pair, size_t* wq_bytes, size_t* sfa_bytes);
int tpx_repack_fp8_tc(const uint8_t* w, const uint8_t* w2, int64_t N, int64_t K, uint8_t* wq, uint8_t* sfa, void* stream);
size_t tpx_qlinear_fp8_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int pair);
int tpx_qlinear_fp8_tc(const uint8_t* wq, const uint8_t* sfa, int fmt, int pair, const uint16_t* x, const void* gamma,
                       int gamma_is_f32, float eps, int64_t M, int64_t N, int64_t K, const uint16_t* bias, int act,
                       const uint16_t* mul_in, const uint16_t* res, float res_scale, uint16_t* y, void* scratch,
                       size_t scratch_bytes, void* stream);

/* ---------------------------------------------------------------- a decoder layer in two calls
 * LlamaDecoderLayer::_forward / Qwen2DecoderLayer::_forward (src/csrc/llm/fused_llm_infer.cpp:1195-1286, :1440-1510) on
 * MXFP4 weights, as two sequences of the entry points above issued from C: tpx_llama_layer_attention = RMSNorm + fused
 * q/k/v (+ bias), rotary embedding + cache append, attention, o_proj + residual -> io->so; tpx_llama_layer_mlp = RMSNorm +
 * gate/up with SiLU * up, down_proj + residual -> io->out. The reference all-reduces after each half under tensor
 * parallelism (:1263-1277): the caller does so between and after the calls. TpxLlamaLayer holds what is fixed per layer
 * (packed weights from tpx_repack_mxfp4_tc, the gate/up pair packed together), TpxLlamaLayerIO what changes per call;
 * every buffer is the caller's: qkv [T][(Nq+2Nkv)H], q [B][Nkv][S][Nq/Nkv][H], ctx [T][Nq*H], so/out [T][D],
 * inter [T][FF] with T = B*S; scratch sized for the largest of the four linears (tpx_qlinear_mxfp4_tc_scratch_bytes),
 * attn_scratch by tpx_attention_scratch_bytes; the cache as kc/vc or, when k_pages != NULL, as page tables.       */
typedef struct {
  int64_t D, Nq, Nkv, H, FF, MP, HR;
  float eps, res_scale;
  int gamma_is_f32;
  const void *gamma1, *gamma2;
  const uint16_t* bias_qkv; /* NULL: none */
  const float* ep;          /* [2][MP][HR] */
  const uint8_t *wqkv, *sfa_qkv, *wo, *sfa_o, *wgu, *sfa_gu, *wd, *sfa_d;
} TpxLlamaLayer;
typedef struct {
  int64_t B, S, Bpos, Spad, offset, capacity;
  const uint16_t* x;
  const int64_t* pos;
  const uint16_t* mask;     /* additive [B][Spad] or NULL */
  const int32_t* dev_len;   /* NULL, or the cached length on the device (CUDA-graph decoding) */
  uint16_t *kc, *vc;
  const uint64_t *k_pages, *v_pages;
  uint16_t *qkv, *q, *ctx, *so, *inter, *out;
  void* scratch;
  size_t scratch_bytes;
  void* attn_scratch;
  size_t attn_scratch_bytes;
  void* handoff;            /* NULL, or a zero-initialised buffer (1024-byte aligned) of handoff_bytes that only these calls */
  size_t handoff_bytes;     /* write: at most 64 tokens pass from gate/up to down through it (2 * 64 * FF + FF * 4 bytes suffice) */
} TpxLlamaLayerIO;
int tpx_llama_layer_attention(const TpxLlamaLayer* layer, const TpxLlamaLayerIO* io, void* stream);
int tpx_llama_layer_mlp(const TpxLlamaLayer* layer, const TpxLlamaLayerIO* io, void* stream);

/* ---------------------------------------------------------------- tensor-parallel all-reduce over peer memory
 * Replaces tpp_llm.allreduce (src/csrc/llm/fused_llm_infer.cpp:101-119) for the small bf16 tensors a decoder layer
 * reduces after its row-parallel linears (:1263-1277); the reference's own latency-oriented path is its shared-memory
 * all-reduce (src/csrc/shm_coll.cpp). In-place SUM of data[n] (n a multiple of 8, at most buf_elems / 2) over `world`
 * ranks (2..8) of one NVLink domain, fp32 accumulation in rank order (every rank gets the same bits), one kernel per
 * rank and call. The caller provides, per rank r, an exchange buffer of buf_elems bf16 (buf_ptrs_host[r]) and a flag
 * array of tpx_allreduce_flag_bytes() bytes (flag_ptrs_host[r]), all of them addressable from every rank (peer or
 * symmetric memory) and zero before first use; `state` is 16 bytes of this rank's own device memory, zero before first
 * use: word 0 counts the calls, word 2 receives 1 + the rank of a peer that did not arrive within the bounded wait
 * (the kernel then finishes with a wrong sum instead of hanging). buf_ptrs_host / flag_ptrs_host are HOST arrays of
 * `world` device addresses. Every rank must make the same sequence of calls with the same n.                      */
size_t tpx_allreduce_flag_bytes(void);
int tpx_allreduce_bf16(uint16_t* data, int64_t n, int rank, int world, const uint64_t* buf_ptrs_host,
                       const uint64_t* flag_ptrs_host, void* state, int64_t buf_elems, void* stream);

/* TppCache::align_and_invert_mask (src/csrc/llm/attn.h:310-322): [B][S] bf16 0/1 mask -> [B][Spad] additive
 * mask (1 -> 0, 0 -> min_bits, padding -> min_bits), Spad a multiple of 32.                                  */
int tpx_align_and_invert_mask(const uint16_t* mask, int64_t B, int64_t S, int64_t Spad, uint16_t min_bits,
                              uint16_t* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TPX_B200_H */
