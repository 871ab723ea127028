/*
 * CPU oracle for the quantized-linear + attention hot path of
 * libxsmm/tpp-pytorch-extension (src/csrc/llm, src/csrc/fused_gemm.h, src/csrc/qtypes.*).
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is a plain-C restatement of the reference's CPU
 * algorithm, used only as the checker in tests, in the smoke test and as the timed CPU
 * baseline of the benchmark. The product (the CUDA library) never links or calls it.
 *
 * Parity status: the reference holds no golden vectors or tests for this path, and its GEMM
 * inner kernels live in libxsmm, which is not vendored. The element quantiser below is pinned
 * against the reference's own src/csrc/mxfp_quant.h compiled from where it lies (oracle/_ref,
 * see ref_shim.cpp); the loops, layouts and the GEMM/attention math are restated from the cited
 * lines and are otherwise "parity unpinned".
 *
 * Every function cites the reference file:line it follows (paths relative to the reference root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------------------------------------------------------------- bf16 helpers */

static inline float bf16_to_f32(uint16_t h) {
  union { uint32_t u; float f; } v;
  v.u = ((uint32_t)h) << 16;
  return v.f;
}

/* round-to-nearest-even fp32 -> bf16, the conversion at::BFloat16 performs */
static inline uint16_t f32_to_bf16(float f) {
  union { uint32_t u; float f; } v;
  v.f = f;
  if ((v.u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((v.u >> 16) | 0x40); /* NaN */
  uint32_t lsb = (v.u >> 16) & 1u;
  v.u += 0x7fffu + lsb;
  return (uint16_t)(v.u >> 16);
}

static inline uint32_t f32_bits(float f) {
  union { uint32_t u; float f; } v;
  v.f = f;
  return v.u;
}
static inline float bits_f32(uint32_t u) {
  union { uint32_t u; float f; } v;
  v.u = u;
  return v.f;
}

/* Launchers export OMP_NUM_THREADS=1 to the ranks they start; a timed run asks for the host's cores explicitly. */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ---------------------------------------------------------------- MXFP4 element math
 * Shared scale of one 32-element block from its absmax
 * (src/csrc/qtypes.cpp:69-76 -> src/csrc/mxfp_quant.h:127-161):
 *   e  = biased fp32 exponent of absmax;  flush the whole block when e == 0
 *   se = (e == 255) ? 255 : e - 2          (E2M1 has emax = 2)
 *   clamp: se-127 > 127 -> 255 ; se-127 < -127 -> 0
 *   scale_fp = 2^(se-127), built with the top mantissa bit set when se is 0 or 255
 *   stored byte = biased exponent of scale_fp = se                                  */
uint8_t orc_mx_scale_byte(float absmax, int* flush_block, float* scale_fp) {
  int e = (int)((f32_bits(absmax) & 0x7f800000u) >> 23);
  if (flush_block) *flush_block = (e == 0);
  int se = (e != 255) ? e - 2 : e;
  int ub = se - 127;
  if (ub > 127) se = 255;
  if (ub < -127) se = 0;
  uint32_t mant = (se == 0 || se == 255) ? 0x400000u : 0u;
  if (scale_fp) *scale_fp = bits_f32(((uint32_t)se << 23) | mant);
  return (uint8_t)se;
}

/* One element to its E2M1 code (src/csrc/qtypes.cpp:87-135 with
 * quantize_elemwise(bits=3, exp_bits=2, max_norm=6, rd_even, saturate, denorms) of
 * src/csrc/mxfp_quant.h:240-300): x = w / scale_fp, round to nearest even onto
 * {0, .5, 1, 1.5, 2, 3, 4, 6}, saturate at 6, keep the sign (a negative that rounds to zero
 * stays code 8 only if the rounded value compares equal to -0.0 first, which 0.0 == -0.0 makes
 * code 0: the chain tests `== 0.0` before `== -0.0`).
 * Restated with integer arithmetic on the fp32 bit pattern of x.                        */
uint8_t orc_e2m1_code(float x) {
  uint32_t u = f32_bits(x);
  uint32_t sign = u >> 31;
  int be = (int)((u >> 23) & 0xff);
  uint32_t tm = u & 0x7fffffu;
  /* target format: bias 1, 2 significand bits including the hidden one */
  int nbe = be - 127 + 1;
  int exp_diff = nbe <= 0 ? 1 - nbe : 0;
  /* |x| < 0.125 (and every fp32 subnormal): the shifted significand is 0 before and after the
   * rounding increment, so the reference returns 0.0 whatever its tie/even flags say */
  if (exp_diff >= 3) return 0;
  int is_sub = (be == 0);
  uint32_t m = is_sub ? tm : (tm | 0x800000u);
  int sig = is_sub ? 23 : 24;
  int tbits = exp_diff + (sig - 2);
  /* the reference examines the truncated bits on the un-shifted significand */
  int tie = ((m & ((1u << (tbits - 1)) - 1u)) == 0);
  int even = (tbits < 32) ? ((m & (1u << tbits)) == 0) : 1;
  m >>= exp_diff;
  m >>= (sig - 2 - 1);
  if (!(tie && even)) m += 1;
  m >>= 1;
  if (m == 0) return 0; /* +-0 -> code 0 (see above) */
  /* rebuild the value the reference compares against its table */
  uint32_t full = m << (sig - 2 + exp_diff);
  int overflow = full >= (1u << sig);
  if (overflow && !is_sub) full >>= 1;
  full &= 0x7fffffu;
  int obe = overflow ? be + 1 : be;
  float mag = bits_f32(((uint32_t)obe << 23) | full);
  if (mag > 6.0f || obe >= 255) mag = 6.0f; /* saturate_normals (also catches inf/nan input) */
  uint8_t code;
  if (mag == 0.5f) code = 1;
  else if (mag == 1.0f) code = 2;
  else if (mag == 1.5f) code = 3;
  else if (mag == 2.0f) code = 4;
  else if (mag == 3.0f) code = 5;
  else if (mag == 4.0f) code = 6;
  else if (mag == 6.0f) code = 7;
  else code = 0; /* not reachable for finite inputs; the reference leaves qval = 0 */
  return (uint8_t)(code | (sign << 3));
}

static const float kE2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

/* lut[code] * 2^(byte-127), byte 0 -> 0.0 (src/csrc/qtypes.cpp:147-150,
 * get_fp_scale src/csrc/mxfp_quant.h:78-83) */
float orc_mxfp4_dequant_elem(uint8_t code, uint8_t scale_byte) {
  return kE2M1[code & 15] * bits_f32(((uint32_t)scale_byte) << 23);
}

/* ---------------------------------------------------------------- block quantisers
 * Loop structure of PerBlockQuantizer::quantize_symetric (src/csrc/qtypes.h:133-193).
 * The input is viewed as in[pre][bs][post][vnni]; one scale per (pre, post).
 * For 4-bit outputs two codes share a byte, low nibble = even vnni lane (:166-178).   */
void orc_quantize_mxfp4_blocks(const uint16_t* in_bf16, long pre, long bs, long post, long vnni,
                               uint8_t* codes /* [pre][bs][post][vnni/2] */,
                               uint8_t* scales /* [pre][post] */) {
#pragma omp parallel for collapse(2)
  for (long i = 0; i < pre; i++) {
    for (long j = 0; j < post; j++) {
      const uint16_t* base = in_bf16 + (i * bs * post + j) * vnni;
      float mx = fabsf(bf16_to_f32(base[0]));
      for (long k = 0; k < bs; k++)
        for (long v = 0; v < vnni; v++) {
          float a = fabsf(bf16_to_f32(base[k * post * vnni + v]));
          mx = a > mx ? a : mx; /* std::max(max, val): NaN in val is dropped */
        }
      int flush;
      float scale_fp;
      scales[i * post + j] = orc_mx_scale_byte(mx, &flush, &scale_fp);
      for (long k = 0; k < bs; k++)
        for (long v1 = 0; v1 < vnni / 2; v1++) {
          unsigned packed = 0;
          for (int v2 = 0; v2 < 2; v2++) {
            float w = bf16_to_f32(base[k * post * vnni + v1 * 2 + v2]);
            float x = flush ? 0.0f : w / scale_fp;
            packed |= ((unsigned)orc_e2m1_code(x) & 0xF) << (4 * v2);
          }
          codes[((i * bs + k) * post + j) * (vnni / 2) + v1] = (uint8_t)packed;
        }
    }
  }
}

/* Int8SymQuant (src/csrc/qtypes.cpp:153-197): scale = max/127.0 (double divide, stored as
 * fp32), iscale = 1.0f/scale or 0, q = clamp(nearbyintf(w * iscale), -127, 127).       */
void orc_quantize_int8_blocks(const uint16_t* in_bf16, long pre, long bs, long post, long vnni,
                              int8_t* q /* [pre][bs][post][vnni] */, float* scales /* [pre][post] */) {
#pragma omp parallel for collapse(2)
  for (long i = 0; i < pre; i++) {
    for (long j = 0; j < post; j++) {
      const uint16_t* base = in_bf16 + (i * bs * post + j) * vnni;
      float mx = fabsf(bf16_to_f32(base[0]));
      for (long k = 0; k < bs; k++)
        for (long v = 0; v < vnni; v++) {
          float a = fabsf(bf16_to_f32(base[k * post * vnni + v]));
          mx = a > mx ? a : mx;
        }
      float scale = (float)((double)mx / 127.0);
      float iscale = (scale != 0) ? (1.0f / scale) : 0;
      scales[i * post + j] = scale;
      for (long k = 0; k < bs; k++)
        for (long v = 0; v < vnni; v++) {
          volatile float prod = bf16_to_f32(base[k * post * vnni + v]) * iscale;
          int qi = (int)nearbyintf(prod);
          qi = qi < -127 ? -127 : (qi > 127 ? 127 : qi);
          q[((i * bs + k) * post + j) * vnni + v] = (int8_t)qi;
        }
    }
  }
}

/* Same quantiser for fp32 activations with one block = `bs` consecutive elements of a row
 * (TppBlockedQInt8LinearW quantises its input with quantize_int8sym(X, block, -1, false),
 * src/csrc/fused_gemm.h:1249). X is bf16 in the reference's LLM path.                   */
void orc_quantize_act_int8(const uint16_t* x_bf16, long rows, long K, long bs, int8_t* q, float* scales) {
  orc_quantize_int8_blocks(x_bf16, rows * (K / bs), bs, 1, 1, q, scales);
}

/* dequantize_symetric (src/csrc/qtypes.h:195-242) */
void orc_dequantize_mxfp4_blocks(const uint8_t* codes, const uint8_t* scales, long pre, long bs,
                                 long post, long vnni, float* out /* [pre][bs][post][vnni] */) {
#pragma omp parallel for collapse(2)
  for (long i = 0; i < pre; i++)
    for (long j = 0; j < post; j++) {
      uint8_t s = scales[i * post + j];
      for (long k = 0; k < bs; k++)
        for (long v1 = 0; v1 < vnni / 2; v1++) {
          unsigned p = codes[((i * bs + k) * post + j) * (vnni / 2) + v1];
          for (int v2 = 0; v2 < 2; v2++)
            out[((i * bs + k) * post + j) * vnni + v1 * 2 + v2] =
                orc_mxfp4_dequant_elem((p >> (4 * v2)) & 0xF, s);
        }
    }
}

void orc_dequantize_int8_blocks(const int8_t* q, const float* scales, long pre, long bs, long post,
                                long vnni, float* out) {
#pragma omp parallel for collapse(2)
  for (long i = 0; i < pre; i++)
    for (long j = 0; j < post; j++) {
      float s = scales[i * post + j];
      for (long k = 0; k < bs; k++)
        for (long v = 0; v < vnni; v++) {
          long idx = ((i * bs + k) * post + j) * vnni + v;
          out[idx] = (float)q[idx] * s; /* src/csrc/qtypes.cpp:193-196 */
        }
    }
}

/* ---------------------------------------------------------------- epilogues
 * Activation codes shared with the CUDA library (include/tpx_b200.h).               */
enum { ORC_ACT_NONE = 0, ORC_ACT_GELU = 1, ORC_ACT_SILU = 2, ORC_ACT_RELU = 3 };

static inline float orc_act(float v, int act) {
  switch (act) {
    case ORC_ACT_GELU: /* erf form, GeluFwdTPP::ref src/csrc/xsmm_functors.h:2794-2799 */
      return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    case ORC_ACT_SILU: /* x * sigmoid(x), SiLUFwdTPP::ref src/csrc/xsmm_functors.h:3286-3296 */
      return v / (1.0f + expf(-v));
    case ORC_ACT_RELU:
      return v > 0.0f ? v : 0.0f;
    default:
      return v;
  }
}

/* Weight-only quantized linear, fp32 accumulation, one bf16 rounding of the result:
 *   y = epilogue( x . Wd^T + bias )            (TppBlockedLinearW, src/csrc/fused_gemm.h:829-954)
 * Wd is the dequantized weight in plain [N][K] fp32 (the caller un-blocks it).
 * Epilogue order follows the post-op callbacks (src/csrc/fused_gemm.h:1343-1488):
 *   act -> * mul_in (MulPostOp) -> + res*res_scale (AddScalePostOp, ScaleAddTPP::ref
 *   src/csrc/xsmm_functors.h:1862-1869).
 * ref_rounding != 0 reproduces the reference's extra bf16 stores (GEMM result stored to bf16
 * before the post-op runs in place on it).                                             */
void orc_qlinear_f32w(const uint16_t* x_bf16, const float* wd, const uint16_t* bias_bf16,
                      const uint16_t* mul_in_bf16, const uint16_t* res_bf16, float res_scale, int act,
                      int ref_rounding, long M, long N, long K, uint16_t* y_bf16) {
#pragma omp parallel for collapse(2) schedule(static)
  for (long m = 0; m < M; m++) {
    for (long n = 0; n < N; n++) {
      const uint16_t* xr = x_bf16 + m * K;
      const float* wr = wd + n * K;
      float acc = 0.0f;
      for (long k = 0; k < K; k++) acc += bf16_to_f32(xr[k]) * wr[k];
      if (bias_bf16) acc += bf16_to_f32(bias_bf16[n]);
      if (ref_rounding) acc = bf16_to_f32(f32_to_bf16(acc));
      float v = orc_act(acc, act);
      if (ref_rounding && act != ORC_ACT_NONE) v = bf16_to_f32(f32_to_bf16(v));
      if (mul_in_bf16) {
        v = v * bf16_to_f32(mul_in_bf16[m * N + n]);
        if (ref_rounding) v = bf16_to_f32(f32_to_bf16(v));
      }
      if (res_bf16) v = v + bf16_to_f32(res_bf16[m * N + n]) * res_scale;
      y_bf16[m * N + n] = f32_to_bf16(v);
    }
  }
}

/* Fused gate/up pair: y = silu(x.Wg^T) * (x.Wu^T). The reference issues two GEMMs,
 * SiluPostOp then MulPostOp (src/csrc/llm/fused_llm_infer.cpp:1271-1272).              */
void orc_gate_up_f32w(const uint16_t* x_bf16, const float* wg, const float* wu, int act, int ref_rounding,
                      long M, long N, long K, uint16_t* y_bf16) {
#pragma omp parallel for collapse(2) schedule(static)
  for (long m = 0; m < M; m++) {
    for (long n = 0; n < N; n++) {
      const uint16_t* xr = x_bf16 + m * K;
      float ag = 0.0f, au = 0.0f;
      for (long k = 0; k < K; k++) {
        float xv = bf16_to_f32(xr[k]);
        ag += xv * wg[n * K + k];
        au += xv * wu[n * K + k];
      }
      if (ref_rounding) {
        ag = bf16_to_f32(f32_to_bf16(ag));
        au = bf16_to_f32(f32_to_bf16(au));
      }
      float g = orc_act(ag, act);
      if (ref_rounding) g = bf16_to_f32(f32_to_bf16(g));
      y_bf16[m * N + n] = f32_to_bf16(g * au);
    }
  }
}

/* The same linear straight from packed MXFP4 in the reference layout, decoding as it goes
 * (this is what the timed CPU baseline runs: it streams 4-bit codes like the reference's
 * BRGEMM does instead of a pre-dequantised fp32 matrix).
 * codes [N/32][K/64][32][32] bytes, byte (k1,c1,r,k2) = W[32k1+k2][64c1+2r+{0,1}];
 * scales [N/32][K/64][2][32] (src/csrc/qtypes.cpp:783-864, src/csrc/fused_gemm.h:884-886). */
void orc_qlinear_mxfp4_packed(const uint16_t* x_bf16, const uint8_t* codes, const uint8_t* scales,
                              const uint8_t* codes2, const uint8_t* scales2, int act, long M, long N,
                              long K, uint16_t* y_bf16) {
  long C1 = K / 64;
  enum { MB = 32 };
  float* xf = (float*)malloc(sizeof(float) * (size_t)M * (size_t)K);
  for (long i = 0; i < M * K; i++) xf[i] = bf16_to_f32(x_bf16[i]);
#pragma omp parallel
  {
    float wt[64][32];                 /* one decoded [64 k][32 n] weight tile, scale applied */
    float acc[2][MB][32];
#pragma omp for schedule(dynamic, 1)
    for (long k1 = 0; k1 < N / 32; k1++) {
      for (long m0 = 0; m0 < M; m0 += MB) {
        long mb = M - m0 < MB ? M - m0 : MB;
        memset(acc, 0, sizeof(acc));
        for (int which = 0; which < (codes2 ? 2 : 1); which++) {
          const uint8_t* cd = which ? codes2 : codes;
          const uint8_t* sc = which ? scales2 : scales;
          for (long c1 = 0; c1 < C1; c1++) {
            const uint8_t* cb = cd + (k1 * C1 + c1) * 32 * 32;
            const uint8_t* sb = sc + (k1 * C1 + c1) * 2 * 32;
            for (int r = 0; r < 32; r++) {
              const uint8_t* sbr = sb + (r / 16) * 32;
              for (int k2 = 0; k2 < 32; k2++) {
                unsigned p = cb[r * 32 + k2];
                float s = bits_f32(((uint32_t)sbr[k2]) << 23);
                wt[2 * r][k2] = kE2M1[p & 15] * s;
                wt[2 * r + 1][k2] = kE2M1[p >> 4] * s;
              }
            }
            for (long m = 0; m < mb; m++) {
              const float* xr = xf + (m0 + m) * K + c1 * 64;
              float* a = acc[which][m];
              for (int kk = 0; kk < 64; kk++) {
                float xv = xr[kk];
                for (int k2 = 0; k2 < 32; k2++) a[k2] += xv * wt[kk][k2];
              }
            }
          }
        }
        for (long m = 0; m < mb; m++)
          for (int k2 = 0; k2 < 32; k2++) {
            float v = orc_act(acc[0][m][k2], act);
            if (codes2) v *= acc[1][m][k2];
            y_bf16[(m0 + m) * N + k1 * 32 + k2] = f32_to_bf16(v);
          }
      }
    }
  }
  free(xf);
}

/* Reference int8 path: dynamic per-(row, K-block) activation quantisation, int8 x int8 -> int32
 * per K-block, out += acc * s_x * s_w, with `out` held in bf16 between K-blocks
 * (src/csrc/fused_gemm.h:1158-1235, DequantTPP::ref src/csrc/xsmm_functors.h:998-1031).
 * wq plain [N][K] int8, ws [N][K/bs] fp32 (caller un-blocks).                            */
void orc_qlinear_int8_dynact(const int8_t* xq, const float* xs, const int8_t* wq, const float* ws,
                             const uint16_t* bias_bf16, int act, long M, long N, long K, long bs,
                             uint16_t* y_bf16) {
  long nb = K / bs;
#pragma omp parallel for collapse(2) schedule(static)
  for (long m = 0; m < M; m++)
    for (long n = 0; n < N; n++) {
      uint16_t out = bias_bf16 ? bias_bf16[n] : 0;
      for (long b = 0; b < nb; b++) {
        int32_t acc = 0;
        for (long k = 0; k < bs; k++) acc += (int32_t)xq[m * K + b * bs + k] * (int32_t)wq[n * K + b * bs + k];
        float v = bf16_to_f32(out) + (float)acc * xs[m * nb + b] * ws[n * nb + b];
        out = f32_to_bf16(v);
      }
      float v = orc_act(bf16_to_f32(out), act);
      y_bf16[m * N + n] = f32_to_bf16(v);
    }
}

/* ---------------------------------------------------------------- norm / rope
 * RMSNormFwdTPP::ref (src/csrc/xsmm_functors.h:4628-4654): fp32 stats, y = x * rsqrt(mean(x^2)+eps) * g */
void orc_rmsnorm(const uint16_t* x_bf16, const uint16_t* g_bf16, float eps, long rows, long D, uint16_t* y_bf16) {
#pragma omp parallel for
  for (long r = 0; r < rows; r++) {
    float ss = 0.0f;
    for (long d = 0; d < D; d++) {
      float v = bf16_to_f32(x_bf16[r * D + d]);
      ss += v * v;
    }
    float inv = 1.0f / sqrtf(ss / (float)D + eps);
    for (long d = 0; d < D; d++)
      y_bf16[r * D + d] = f32_to_bf16(bf16_to_f32(x_bf16[r * D + d]) * inv * bf16_to_f32(g_bf16[d]));
  }
}

/* apply_rotary_pos_emb_llama (src/csrc/llm/fused_llm_infer.cpp:206-253): in place on
 * x[B][S][N][H]; pairs (h, h+HR/2); table ep[2][MP][HR] fp32 (0 = cos, 1 = sin); positions
 * int64 [Bpos][S] with Bpos 1 or B; rows whose position >= MP are left untouched.        */
void orc_rope_llama(uint16_t* x_bf16, const float* ep, const int64_t* pos, long B, long S, long N, long H,
                    long MP, long HR, long Bpos) {
  long coff = HR / 2;
#pragma omp parallel for collapse(3)
  for (long b = 0; b < B; b++)
    for (long s = 0; s < S; s++)
      for (long n = 0; n < N; n++) {
        int64_t p = pos[(Bpos == 1 ? 0 : b) * S + s];
        if (p >= MP) continue;
        uint16_t* row = x_bf16 + ((b * S + s) * N + n) * H;
        for (long h2 = 0; h2 < HR / 2; h2++) {
          float in0 = bf16_to_f32(row[h2]), in1 = bf16_to_f32(row[coff + h2]);
          float c = ep[(0 * MP + p) * HR + h2], sn = ep[(1 * MP + p) * HR + h2];
          float o0 = in0 * c - in1 * sn;
          float o1 = in1 * c + in0 * sn;
          row[h2] = f32_to_bf16(o0);
          row[coff + h2] = f32_to_bf16(o1);
        }
      }
}

/* ---------------------------------------------------------------- attention
 * attn<T> (src/csrc/llm/attn.cpp:780-955) restated with fp32 softmax over the whole key range
 * (mathematically what the blockwise running-max loop computes; the reference additionally
 * stores un-normalised probabilities and the running output in bf16).
 *   q   [B][Nkv][Sq][R][H]  bf16          (GQA folded: R = Nq/Nkv, attn.cpp:793-795)
 *   kc,vc key/value cache [S1][B][Nkv][32][H] bf16, token t at (t/32, t%32) (attn.cpp:383-427)
 *   am  additive mask [B][Spad] in bf16 (0 keep, finfo.min drop; attn.h:310-322)
 *   key_len = tokens in the cache including the Sq new ones; offset = key_len - Sq;
 *   causal: key j visible to query i iff j <= offset + i (fill -1e9, attn.cpp:905-921).   */
void orc_attention(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, const uint16_t* am, long B,
                   long Nkv, long Sq, long R, long H, long key_len, long Spad, int causal,
                   uint16_t* out /* same shape as q */) {
  long offset = key_len - Sq;
  float inv_sqrt = 1.0f / sqrtf((float)H);
#pragma omp parallel
  {
    float* sc = (float*)malloc(sizeof(float) * (size_t)key_len);
    float* acc = (float*)malloc(sizeof(float) * (size_t)H);
#pragma omp for collapse(3) schedule(dynamic, 4)
    for (long b = 0; b < B; b++)
      for (long n = 0; n < Nkv; n++)
        for (long i = 0; i < Sq * R; i++) {
          long sq = i / R;
          const uint16_t* qr = q + (((b * Nkv + n) * Sq) * R + i) * H;
          long kend = causal ? (offset + sq + 1) : key_len;
          if (kend > key_len) kend = key_len;
          float mx = -INFINITY;
          for (long j = 0; j < kend; j++) {
            const uint16_t* kr = kc + ((((j / 32) * B + b) * Nkv + n) * 32 + (j % 32)) * H;
            float d = 0.0f;
            for (long h = 0; h < H; h++) d += bf16_to_f32(qr[h]) * bf16_to_f32(kr[h]);
            d = d * inv_sqrt + (am ? bf16_to_f32(am[b * Spad + j]) : 0.0f);
            sc[j] = d;
            mx = d > mx ? d : mx;
          }
          float sum = 0.0f;
          for (long h = 0; h < H; h++) acc[h] = 0.0f;
          for (long j = 0; j < kend; j++) {
            float p = expf(sc[j] - mx);
            sum += p;
            const uint16_t* vr = vc + ((((j / 32) * B + b) * Nkv + n) * 32 + (j % 32)) * H;
            for (long h = 0; h < H; h++) acc[h] += p * bf16_to_f32(vr[h]);
          }
          uint16_t* orow = out + (((b * Nkv + n) * Sq) * R + i) * H;
          for (long h = 0; h < H; h++) orow[h] = f32_to_bf16(acc[h] / sum);
        }
    free(sc);
    free(acc);
  }
}
