// Weight quantisers, dequantisers and the repack into the streaming layout.
//
// The quantisers reproduce, bit for bit, what the reference computes on the CPU
// (src/csrc/qtypes.cpp:36-197 element math, src/csrc/qtypes.h:133-242 block loops,
// src/csrc/qtypes.cpp:783-932 re-layout); they are one-off, bandwidth-trivial kernels: one thread
// owns one scale block.
#include "tpx_common.cuh"

namespace tpx {

// ---------------------------------------------------------------- MX element math (device)
// Shared scale of a block from its absmax (src/csrc/qtypes.cpp:69-76, src/csrc/mxfp_quant.h:127-161).
__device__ __forceinline__ uint8_t mx_scale_byte(float absmax, bool* flush, float* scale_fp) {
  int e = (int)((__float_as_uint(absmax) >> 23) & 0xff);
  *flush = (e == 0);
  int se = (e != 255) ? e - 2 : e;
  int ub = se - 127;
  if (ub > 127) se = 255;
  if (ub < -127) se = 0;
  uint32_t mant = (se == 0 || se == 255) ? 0x400000u : 0u;
  *scale_fp = __uint_as_float(((uint32_t)se << 23) | mant);
  return (uint8_t)se;
}

// Round-to-nearest-even of x onto the E2M1 grid with saturation at 6, as an E2M1 code
// (src/csrc/qtypes.cpp:87-135 over quantize_elemwise, src/csrc/mxfp_quant.h:240-300).
__device__ __forceinline__ uint32_t e2m1_code(float x) {
  uint32_t u = __float_as_uint(x);
  uint32_t sign = u >> 31;
  int be = (int)((u >> 23) & 0xff);
  uint32_t tm = u & 0x7fffffu;
  int nbe = be - 126;
  int exp_diff = nbe <= 0 ? 1 - nbe : 0;
  if (exp_diff >= 3) return 0;  // |x| < 0.125 rounds to +0 whatever its sign
  uint32_t m = tm | 0x800000u;  // be >= 124 here, never subnormal
  int tbits = exp_diff + 22;
  bool tie = (m & ((1u << (tbits - 1)) - 1u)) == 0;
  bool even = (m & (1u << tbits)) == 0;
  m >>= (exp_diff + 21);
  if (!(tie && even)) m += 1;
  m >>= 1;
  if (m == 0) return 0;
  uint32_t full = m << (22 + exp_diff);
  bool ovf = full >= (1u << 24);
  if (ovf) full >>= 1;
  full &= 0x7fffffu;
  int obe = ovf ? be + 1 : be;
  float mag = __uint_as_float(((uint32_t)obe << 23) | full);
  if (mag > 6.0f || obe >= 255) mag = 6.0f;
  // mag is one of .5 1 1.5 2 3 4 6: code = 2*(exp+1) + mantissa bit of the E2M1 encoding
  uint32_t mb = __float_as_uint(mag);
  int ex = (int)(mb >> 23) - 127;  // -1 .. 2
  uint32_t code = (ex < 0) ? 1u : (uint32_t)(2 * (ex + 1)) + ((mb >> 22) & 1u);
  return code | (sign << 3);
}

// ---------------------------------------------------------------- quantize MXFP4
// Thread = one (k1', c1, blk, k2') scale block of 32 elements: 16 consecutive c2 x 2 lanes.
__global__ void quantize_mxfp4_kernel(const uint16_t* __restrict__ in, int64_t K1, int64_t C1, int64_t C2,
                                      int64_t K2, uint8_t* __restrict__ codes, uint8_t* __restrict__ scales) {
  const int64_t K1o = K1 * K2 / 32;
  const int64_t nblk = C2 / 16;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = K1o * C1 * nblk * 32;
  if (idx >= total) return;
  int64_t k2o = idx % 32;
  int64_t blk = (idx / 32) % nblk;
  int64_t c1 = (idx / (32 * nblk)) % C1;
  int64_t k1o = idx / (32 * nblk * C1);
  // source coordinates of (k1o, k2o) in the blocked input (merge or split of K2, qtypes.cpp:799-812)
  int64_t k1, k2;
  if (K2 <= 32) {
    int64_t R = 32 / K2;
    k1 = k1o * R + k2o / K2;
    k2 = k2o % K2;
  } else {
    int64_t R = K2 / 32;
    k1 = k1o / R;
    k2 = (k1o % R) * 32 + k2o;
  }
  const uint32_t* src = reinterpret_cast<const uint32_t*>(in) + ((k1 * C1 + c1) * C2 + blk * 16) * K2 + k2;
  uint32_t w[16];
  float mx = 0.0f;
#pragma unroll
  for (int c = 0; c < 16; c++) {
    w[c] = src[(int64_t)c * K2];
    float a = fabsf(bf16_bits_to_f32((uint16_t)(w[c] & 0xffff)));
    float b = fabsf(bf16_bits_to_f32((uint16_t)(w[c] >> 16)));
    mx = a > mx ? a : mx;  // NaN operands are dropped, as std::max(max, val) does
    mx = b > mx ? b : mx;
  }
  bool flush;
  float scale_fp;
  uint8_t sb = mx_scale_byte(mx, &flush, &scale_fp);
  scales[((k1o * C1 + c1) * nblk + blk) * 32 + k2o] = sb;
  uint8_t* dst = codes + ((k1o * C1 + c1) * C2 + blk * 16) * 32 + k2o;
#pragma unroll
  for (int c = 0; c < 16; c++) {
    float a = bf16_bits_to_f32((uint16_t)(w[c] & 0xffff));
    float b = bf16_bits_to_f32((uint16_t)(w[c] >> 16));
    float xa = flush ? 0.0f : __fdiv_rn(a, scale_fp);
    float xb = flush ? 0.0f : __fdiv_rn(b, scale_fp);
    dst[(int64_t)c * 32] = (uint8_t)(e2m1_code(xa) | (e2m1_code(xb) << 4));
  }
}

// ---------------------------------------------------------------- quantize int8
// Thread = one (k1, c1n, k2) block of B consecutive input features of one output row.
__global__ void quantize_qint8_kernel(const uint16_t* __restrict__ in, int64_t K1, int64_t C1, int64_t C2,
                                      int64_t K2, int64_t C3, int64_t B, int8_t* __restrict__ q,
                                      float* __restrict__ scales) {
  const int64_t C = C1 * C2 * C3;
  const int64_t C1n = C / B;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= K1 * C1n * K2) return;
  int64_t k2 = idx % K2;
  int64_t c1n = (idx / K2) % C1n;
  int64_t k1 = idx / (K2 * C1n);
  const int64_t bc = C2 * C3;
  float mx = 0.0f;
  for (int64_t j = 0; j < B; j++) {
    int64_t k = c1n * B + j;
    int64_t off = (((k1 * C1 + k / bc) * C2 + (k % bc) / C3) * K2 + k2) * C3 + (k % C3);
    float a = fabsf(bf16_bits_to_f32(in[off]));
    mx = a > mx ? a : mx;
  }
  float scale = (float)((double)mx / 127.0);                     // Int8SymQuant ctor, qtypes.cpp:163-166
  float iscale = (scale != 0.0f) ? __fdiv_rn(1.0f, scale) : 0.0f;
  scales[(k1 * C1n + c1n) * K2 + k2] = scale;
  for (int64_t j = 0; j < B; j++) {
    int64_t k = c1n * B + j;
    int64_t off = (((k1 * C1 + k / bc) * C2 + (k % bc) / C3) * K2 + k2) * C3 + (k % C3);
    float v = __fmul_rn(bf16_bits_to_f32(in[off]), iscale);
    int qi = __float2int_rn(v);                                   // nearbyintf, ties to even
    qi = max(-127, min(127, qi));
    q[(((k1 * C1n + c1n) * (B / 4) + j / 4) * K2 + k2) * 4 + (j % 4)] = (int8_t)qi;
  }
}

// ---------------------------------------------------------------- dequantize (reference layouts)
__constant__ float kE2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

// codes [K1][C1][C2][K2], scales [K1][C1][C2/16][K2] -> out fp32 [K1][C1][C2][K2][2]
__global__ void dequantize_mxfp4_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                        int64_t total, int64_t C2, int64_t K2, float* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  int64_t k2 = idx % K2;
  int64_t c2 = (idx / K2) % C2;
  int64_t kc = idx / (K2 * C2);
  uint8_t p = codes[idx];
  uint8_t s = scales[(kc * (C2 / 16) + c2 / 16) * K2 + k2];
  float sf = __uint_as_float(((uint32_t)s) << 23);  // byte 0 -> 0.0, as get_fp_scale does
  out[idx * 2] = __fmul_rn(kE2M1[p & 15], sf);
  out[idx * 2 + 1] = __fmul_rn(kE2M1[p >> 4], sf);
}

// q [K1][C1][C2][K2][4], scales [K1][C1][1][K2]
__global__ void dequantize_qint8_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales,
                                        int64_t total, int64_t C2, int64_t K2, float* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  int64_t k2 = (idx / 4) % K2;
  int64_t kc = idx / (4 * K2 * C2);
  out[idx] = __fmul_rn((float)q[idx], scales[kc * K2 + k2]);
}

// ---------------------------------------------------------------- repack into the streaming layout
// MXFP4: one thread builds one 32-bit word = 8 codes of one row for one 32-wide scale block.
// Tile (nt, kt) occupies 1088 bytes at (nt*KT + kt)*1088: codes [h][lane][16 B], then scales [16 rows][4].
//   word (nt, kt, h, lane=4g+t, b): row n = 16nt + g + 8h; nibble j holds k = 128kt + 32b + 16(j/4) + 4t + (j%4)
// Source byte (k1,c1,r,k2) of the reference tensor holds W[32k1+k2][64c1+2r+{0,1}], low nibble first.
__global__ void repack_mxfp4_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                    int64_t N, int64_t K, int64_t KT, uint32_t* __restrict__ pk) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (N / 16) * KT * 256;
  if (idx >= total) return;
  int b = idx & 3;
  int lane = (idx >> 2) & 31;
  int h = (idx >> 7) & 1;
  int64_t tile = idx >> 8;
  int64_t kt = tile % KT, nt = tile / KT;
  int g = lane >> 2, t = lane & 3;
  int64_t n = nt * 16 + g + 8 * h;
  int64_t C1 = K / 64;
  uint32_t word = 0;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    int64_t k = kt * 128 + b * 32 + 16 * (j >> 2) + 4 * t + (j & 3);
    uint32_t c = 0;
    if (k < K) {
      uint8_t byte = codes[(((n / 32) * C1 + k / 64) * 32 + (k % 64) / 2) * 32 + (n % 32)];
      c = (k & 1) ? (byte >> 4) : (byte & 15);
    }
    word |= c << (4 * j);
  }
  // a tile is 1088 bytes: 1024 of codes, then the 64 scale bytes [row 0..15][b]
  pk[tile * 272 + (idx & 255)] = word;
  if (t == 0) {
    int64_t kb = kt * 4 + b;  // 32-wide block index along K
    uint8_t s = 0;
    if (kb * 32 < K) s = scales[(((n / 32) * C1 + kb / 2) * 2 + (kb & 1)) * 32 + (n % 32)];
    reinterpret_cast<uint8_t*>(pk)[tile * 1088 + 1024 + (g + 8 * h) * 4 + b] = s;
  }
}

// int8: word (nt, kt, h, lane, b): row n = 16nt + g + 8h; byte i holds k = 64kt + 16b + 4t + i.
// Source q [N/K2][K/B][B/4][K2][4]: byte (k1,c1,r,k2,v) = W[K2 k1 + k2][B c1 + 4r + v].
__global__ void repack_qint8_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales, int64_t N,
                                    int64_t K, int64_t B, int64_t K2, uint32_t* __restrict__ pk,
                                    float* __restrict__ pks) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t KT = K / 64;
  int64_t total = (N / 16) * KT * 256;
  if (idx < total) {
    int b = idx & 3;
    int lane = (idx >> 2) & 31;
    int h = (idx >> 7) & 1;
    int64_t tile = idx >> 8;
    int64_t kt = tile % KT, nt = tile / KT;
    int g = lane >> 2, t = lane & 3;
    int64_t n = nt * 16 + g + 8 * h;
    int64_t k = kt * 64 + 16 * b + 4 * t;  // 4 consecutive k share one source word
    int64_t off = ((((n / K2) * (K / B) + k / B) * (B / 4) + (k % B) / 4) * K2 + (n % K2)) * 4;
    pk[idx] = *reinterpret_cast<const uint32_t*>(q + off);
  }
  // scales: [N/16][K/B][16]
  int64_t nb = K / B;
  if (idx < N * nb) {
    int row = idx % 16;
    int64_t kb = (idx / 16) % nb;
    int64_t nt = idx / (16 * nb);
    int64_t n = nt * 16 + row;
    pks[idx] = scales[((n / K2) * nb + kb) * K2 + (n % K2)];
  }
}

}  // namespace tpx

using namespace tpx;

static inline unsigned blocks_for(int64_t total, int threads) { return (unsigned)((total + threads - 1) / threads); }

extern "C" int tpx_remap_and_quantize_mxfp4(const uint16_t* blocked, int64_t K1, int64_t C1, int64_t C2, int64_t K2,
                                            int64_t C3, uint8_t* codes, uint8_t* scales, void* stream) {
  TPX_REQUIRE(blocked && codes && scales, TPX_ERR_ARG, "remap_and_quantize_mxfp4: null pointer");
  TPX_REQUIRE(C3 == 2, TPX_ERR_UNSUPPORTED, "remap_and_quantize_mxfp4: expects the VNNI2 blocked layout (C3 == 2), got C3=%ld", (long)C3);
  TPX_REQUIRE(K1 > 0 && C1 > 0 && C2 > 0 && K2 > 0, TPX_ERR_ARG, "remap_and_quantize_mxfp4: empty shape");
  TPX_REQUIRE((K2 <= 32 && 32 % K2 == 0 && K1 % (32 / K2) == 0) || (K2 > 32 && K2 % 32 == 0), TPX_ERR_ARG,
              "Shape not compatible for MXFP4 (K1=%ld K2=%ld)", (long)K1, (long)K2);
  TPX_REQUIRE(C2 % 16 == 0, TPX_ERR_ARG, "Axis size must be multiple of block_size (C2=%ld)", (long)C2);
  int64_t total = (K1 * K2 / 32) * C1 * (C2 / 16) * 32;
  quantize_mxfp4_kernel<<<blocks_for(total, 128), 128, 0, (cudaStream_t)stream>>>(blocked, K1, C1, C2, K2, codes, scales);
  TPX_LAUNCH_OK();
  return TPX_OK;
}

extern "C" int tpx_remap_and_quantize_qint8(const uint16_t* blocked, int64_t K1, int64_t C1, int64_t C2, int64_t K2,
                                            int64_t C3, int64_t block_size, int8_t* q, float* scales,
                                            int64_t scales_capacity, int64_t* block_size_used, void* stream) {
  TPX_REQUIRE(blocked && q && scales, TPX_ERR_ARG, "remap_and_quantize_qint8: null pointer");
  TPX_REQUIRE(C3 == 1 || C3 == 2 || C3 == 4, TPX_ERR_ARG, "remap_and_quantize_qint8: C3 must be 1, 2 or 4");
  TPX_REQUIRE(K1 > 0 && C1 > 0 && C2 > 0 && K2 > 0, TPX_ERR_ARG, "remap_and_quantize_qint8: empty shape");
  TPX_REQUIRE(block_size >= 4 && block_size % 4 == 0, TPX_ERR_ARG, "remap_and_quantize_qint8: block size %ld must be a positive multiple of 4",
              (long)block_size);
  int64_t C = C1 * C2 * C3;
  int64_t B = block_size;
  if (C % B != 0) {  // src/csrc/qtypes.cpp:881-888; with no candidate the tensor keeps its own inner block C2*C3
    B = C2 * C3;
    for (int64_t QBS = 4096; QBS >= 64; QBS /= 2)
      if (block_size > QBS && C % QBS == 0) { B = QBS; break; }
  }
  TPX_REQUIRE(B > 0 && C % B == 0 && B % 4 == 0, TPX_ERR_ARG, "Shape not compatible for VNNI4 (C=%ld block=%ld)", (long)C, (long)B);
  if (block_size_used) *block_size_used = B;
  int64_t total = K1 * (C / B) * K2;
  TPX_REQUIRE(scales_capacity >= total, TPX_ERR_ARG, "remap_and_quantize_qint8: block size %ld needs %ld scales, the buffer holds %ld",
              (long)B, (long)total, (long)scales_capacity);
  quantize_qint8_kernel<<<blocks_for(total, 128), 128, 0, (cudaStream_t)stream>>>(blocked, K1, C1, C2, K2, C3, B, q, scales);
  TPX_LAUNCH_OK();
  return TPX_OK;
}

extern "C" int tpx_dequantize_mxfp4(const uint8_t* codes, const uint8_t* scales, int64_t K1, int64_t C1, int64_t C2,
                                    int64_t K2, float* out, void* stream) {
  TPX_REQUIRE(codes && scales && out, TPX_ERR_ARG, "dequantize_mxfp4: null pointer");
  TPX_REQUIRE(C2 % 16 == 0, TPX_ERR_ARG, "dequantize_mxfp4: C2 must be a multiple of 16");
  int64_t total = K1 * C1 * C2 * K2;
  dequantize_mxfp4_kernel<<<blocks_for(total, 256), 256, 0, (cudaStream_t)stream>>>(codes, scales, total, C2, K2, out);
  TPX_LAUNCH_OK();
  return TPX_OK;
}

extern "C" int tpx_dequantize_qint8(const int8_t* q, const float* scales, int64_t K1, int64_t C1, int64_t C2,
                                    int64_t K2, float* out, void* stream) {
  TPX_REQUIRE(q && scales && out, TPX_ERR_ARG, "dequantize_qint8: null pointer");
  int64_t total = K1 * C1 * C2 * K2 * 4;
  dequantize_qint8_kernel<<<blocks_for(total, 256), 256, 0, (cudaStream_t)stream>>>(q, scales, total, C2, K2, out);
  TPX_LAUNCH_OK();
  return TPX_OK;
}

extern "C" int tpx_packed_bytes(int kind, int64_t N, int64_t K, int64_t block_size, size_t* codes_bytes,
                                size_t* scales_bytes) {
  TPX_REQUIRE(N > 0 && K > 0 && N % 16 == 0, TPX_ERR_ARG, "packed_bytes: N must be a positive multiple of 16");
  if (kind == TPX_W_MXFP4) {
    TPX_REQUIRE(K % 64 == 0, TPX_ERR_ARG, "packed_bytes: MXFP4 needs K %% 64 == 0");
    int64_t KT = (K + 127) / 128;
    if (codes_bytes) *codes_bytes = (size_t)(N / 16) * KT * 1088;  // the scales ride inside the tiles
    if (scales_bytes) *scales_bytes = 0;
    return TPX_OK;
  }
  if (kind == TPX_W_INT8) {
    TPX_REQUIRE(K % 64 == 0 && block_size >= 64 && block_size % 64 == 0 && K % block_size == 0, TPX_ERR_ARG,
                "packed_bytes: int8 needs K %% 64 == 0 and a block size that is a multiple of 64 dividing K");
    if (codes_bytes) *codes_bytes = (size_t)N * K;
    if (scales_bytes) *scales_bytes = (size_t)N * (K / block_size) * sizeof(float);
    return TPX_OK;
  }
  set_error("packed_bytes: unknown weight kind %d", kind);
  return TPX_ERR_ARG;
}

extern "C" int tpx_repack_mxfp4(const uint8_t* codes, const uint8_t* scales, int64_t N, int64_t K, uint8_t* pk_codes,
                                uint8_t* pk_scales, void* stream) {
  (void)pk_scales;
  TPX_REQUIRE(codes && scales && pk_codes, TPX_ERR_ARG, "repack_mxfp4: null pointer");
  TPX_REQUIRE(N % 32 == 0 && K % 64 == 0, TPX_ERR_ARG, "repack_mxfp4: needs N %% 32 == 0 and K %% 64 == 0 (N=%ld K=%ld)", (long)N, (long)K);
  int64_t KT = (K + 127) / 128;
  int64_t total = (N / 16) * KT * 256;
  repack_mxfp4_kernel<<<blocks_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      codes, scales, N, K, KT, reinterpret_cast<uint32_t*>(pk_codes));
  TPX_LAUNCH_OK();
  return TPX_OK;
}

extern "C" int tpx_repack_qint8(const int8_t* q, const float* scales, int64_t N, int64_t K, int64_t block_size,
                                uint8_t* pk_codes, float* pk_scales, void* stream) {
  TPX_REQUIRE(q && scales && pk_codes && pk_scales, TPX_ERR_ARG, "repack_qint8: null pointer");
  TPX_REQUIRE(N % 16 == 0 && K % 64 == 0 && block_size % 64 == 0 && K % block_size == 0, TPX_ERR_ARG,
              "repack_qint8: needs N %% 16 == 0, K %% 64 == 0 and a block size that is a multiple of 64 dividing K");
  int64_t total = (N / 16) * (K / 64) * 256;
  repack_qint8_kernel<<<blocks_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      q, scales, N, K, block_size, 16, reinterpret_cast<uint32_t*>(pk_codes), pk_scales);
  TPX_LAUNCH_OK();
  return TPX_OK;
}
