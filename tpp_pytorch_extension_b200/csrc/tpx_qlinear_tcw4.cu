// MXFP4 weight-only linear for up to 64 tokens (decoding): weights on the wide (N) side of the MMA, both operands in
// packed 4-bit form (tcgen05 kind::mxf4), and for up to 8 tokens no separate activation kernel at all.
//
// Same contract and the same packed weights as tpx_qlinear_tc.cu (TppBlockedLinearW with the MXFP4 BRGEMM of the
// reference, src/csrc/fused_gemm.h:875-949; fc_plain / the gate-up pair of src/csrc/llm/fused_llm_infer.cpp:1204-1277).
//
// What bounds a decode linear on this GPU is the tensor pipe's fixed cost per instruction, not its arithmetic: a
// 128-row MMA costs ~100 cycles however few columns it has, and every 512-byte scale-factor copy costs about as much.
// So each instruction should consume as many weight bytes as possible:
//   B (256 rows) = 256 output features of packed E2M1 weights, as they lie in HBM: one MMA (K = 64) reads 8 KiB of them
//   A (128 rows) = the activation terms: a bf16 value x of a 32-wide block becomes the integer n = round(x / 2^s)
//                  (2^s chosen so that the block maximum lands in (877, 1755]: exact to 2^-11..2^-10 of the block maximum),
//                  and n + 2340 is written in base 8: n = sum_i (d_i - 4) * 8^i, digits d_i - 4 in [-4, 3], all of them
//                  E2M1 values; term i carries the block scale 2^(s + 3i). Integer arithmetic only, no conversion
//                  instructions. The four terms of a token are four ROWS of A inside one 32-lane quarter of tensor
//                  memory, so the epilogue adds them with two warp shuffles
//   D            = [token term][feature], 256 fp32 columns of tensor memory
// Token-count classes (TOKP):
//    8: up to 8 tokens, two per quarter. The activation terms of the CTA's whole K range are built by the CTA itself
//       (its four epilogue warps, idle until the end otherwise) straight into shared memory, optionally behind the RMSNorm
//       of the reference's decoder block (llama_rms_norm, src/csrc/llm/fused_llm_infer.cpp:336-363): no activation kernel
//       runs before the GEMM and no activation bytes travel through the pipeline stages. Where every CTA needs the whole
//       K range (whole tiles), the CTAs of a thread-block cluster share the work: each builds the terms of some k steps and
//       stores them into every member's shared memory (distributed shared memory).
//   32: up to 32 tokens, eight per quarter; terms come from split4w_kernel through TMA, per stage.
//   64: up to 64 tokens, sixteen per quarter; two A tiles (terms 0,1 and terms 2,3) accumulate into the same D.
// Work split: whole 256-feature tiles per CTA when the tile count suits the SM count, else one thread-block cluster per
// tile that cuts K and reduces over distributed shared memory. Other tile counts stay with the older kernels.
#include "tpx_tc_ptx.cuh"

namespace tpx {

constexpr int kW4MaxStages = 8;
constexpr int kW4ConvThreads = 384;  // TOKP 8: threads that build the activation terms (the four epilogue warps and eight more)

template <int TOKP>
struct W4Cfg {
  static constexpr bool RES = TOKP == 8;                    // activation terms resident in shared memory
  static constexpr int ATILES = TOKP == 64 ? 2 : 1;         // A operand tiles per k step
  static constexpr int LIVE = TOKP == 64 ? 16 : TOKP == 32 ? 8 : 2;  // tokens per 32-lane quarter
  static constexpr int UKS = TOKP == 64 ? 1 : 2;            // k steps (of 128) per pipeline stage
  static constexpr int A1 = ATILES * 128 * 64;              // activation terms per k step when they travel by TMA
  static constexpr int RES_A1 = 32 * 64;                    // resident terms per k step: 32 stored rows of 64 bytes
  static constexpr int B1 = 256 * 64;                       // packed weights per k step
  static constexpr int SFA1 = ATILES * 512;
  static constexpr int STAGE_RAW = UKS * (B1 + 1024 + (RES ? 0 : A1 + SFA1));
  static constexpr int STAGE_BYTES = (STAGE_RAW + 1023) / 1024 * 1024;
  static constexpr int SFC = 8 + 4 * ATILES;                // tensor-memory columns of one k step's scale factors in the ring
  static constexpr int RING_COL0 = 256;                     // D: [0, 256)
  static constexpr int MAX_RES_KSTEPS = 32;                 // 2.5 KiB of shared memory each
  static_assert(RING_COL0 + kW4MaxStages * UKS * SFC <= 512, "tensor memory");
};

struct W4Params {
  TcParams t;            // sfa = weight scale blocks, sfb = activation scale blocks (TOKP 32/64), epilogue fields, TN, KS (units per tile)
  const uint16_t* x;     // TOKP 8: the bf16 activations [M][K]
  const void* gamma;     // TOKP 8: optional RMSNorm weight (null: none)
  int gamma_f32;
  float eps;
  int tiles128, ksteps;  // 128-feature tiles and k steps of the packed weight
  int stages;            // pipeline stages that fit beside the resident terms
  int share;             // TOKP 8, whole tiles: CTAs per cluster that build the terms together (1: every CTA for itself)
};

// K-major operand of 64-byte rows, 64-byte swizzle, 8-row groups `sbo` bytes apart (512: plain; 128: groups overlap and
// group g starts at stored row 2g, so that only two rows per group need to exist in memory).
__device__ __forceinline__ uint64_t w4_desc64(uint32_t saddr, uint32_t sbo) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46) | (4ull << 61);
}

// Block scale exponent s of a 32-wide block from its maximum: max / 2^s in (877, 1755]. The four lanes of a block call
// this together (their eight-value maxima are combined with shuffles).
__device__ __forceinline__ int w4_block_exp(const float (&f)[8]) {
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(f[j]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  int sx = -120;
  if (amax > 0.0f && amax < INFINITY) {
    sx = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127 - 9;  // amax / 2^s in [512, 1024)
    sx = max(-119, min(110, sx));
    if (amax * __uint_as_float((uint32_t)(127 - (sx - 1)) << 23) <= 1755.0f) sx--;
  }
  return sx;
}

// Eight values of a block with scale exponent s -> four words of eight E2M1 codes (value j in nibble j): word i holds
// digit i of n + 2340 in base 8, n = round(x / 2^s) clamped to [-2340, 1755], as the E2M1 code of (digit - 4).
__device__ __forceinline__ void w4_digits(const float (&f)[8], int sx, uint32_t (&packed)[4]) {
  const float inv = __uint_as_float((uint32_t)(127 - sx) << 23);
#pragma unroll
  for (int i = 0; i < 4; i++) packed[i] = 0u;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const float t = fminf(fmaxf(f[j] * inv, -2340.0f), 1755.0f);
    // round to nearest even through the mantissa of t + 1.5 * 2^23
    const uint32_t m = (__float_as_uint(t + 12582912.0f) & 0x7fffffu) - 0x400000u + 2340u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t d = (m >> (3 * i)) & 7u;
      packed[i] |= ((0x5420ACDEu >> (4u * d)) & 15u) << (4 * j);  // codes of -4, -3, -2, -1, 0, 1, 2, 3
    }
  }
}

// Table behind the in-kernel activation split: entry m (= n + 2340, 0..4095) holds the E2M1 codes of the four base-8
// digits of m, each minus 4, one code per byte (term i in byte i). Filled once per device by w4_lut_init_kernel; the
// GEMM copies it into shared memory while it waits for its input.
static __device__ __align__(16) uint32_t g_w4_lut[4096];

__global__ void w4_lut_init_kernel() {
  const uint32_t m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= 4096) return;
  uint32_t e = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) e |= ((0x5420ACDEu >> (4u * ((m >> (3 * i)) & 7u))) & 15u) << (8 * i);
  g_w4_lut[m] = e;
}

// Eight values of a block with scale exponent s -> the same four words as w4_digits, through the table in shared memory.
__device__ __forceinline__ void w4_digits_lut(const float (&f)[8], int sx, const uint32_t* __restrict__ lut, uint32_t (&packed)[4]) {
  const float inv = __uint_as_float((uint32_t)(127 - sx) << 23);
  uint32_t E[8];
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const float t = fminf(fmaxf(f[j] * inv, -2340.0f), 1755.0f);
    const uint32_t m = (__float_as_uint(t + 12582912.0f) & 0x7fffffu) - 0x400000u + 2340u;
    E[j] = lut[m];
  }
  // byte i of P_a: the codes of term i for values 2a (low nibble) and 2a + 1; then a 4 x 4 byte transpose
  const uint32_t P0 = E[0] | (E[1] << 4), P1 = E[2] | (E[3] << 4), P2 = E[4] | (E[5] << 4), P3 = E[6] | (E[7] << 4);
  const uint32_t A = __byte_perm(P0, P1, 0x5140), B = __byte_perm(P2, P3, 0x5140);
  const uint32_t Cc = __byte_perm(P0, P1, 0x7362), D = __byte_perm(P2, P3, 0x7362);
  packed[0] = __byte_perm(A, B, 0x5410);
  packed[1] = __byte_perm(A, B, 0x7632);
  packed[2] = __byte_perm(Cc, D, 0x5410);
  packed[3] = __byte_perm(Cc, D, 0x7632);
}

// Bounded wait that also sees what other CTAs of the cluster stored before they arrived on the barrier.
__device__ __forceinline__ bool w4_wait_cluster(uint32_t bar, uint32_t parity) {
  for (unsigned spins = 0; spins < kTcSpinLimit; spins++) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    if (ok) return true;
    __nanosleep(200);  // a long wait beside working warps: leave them the issue slots and the memory pipeline
  }
  return false;
}
// Bounded wait for long waits beside working warps (the producer waiting for a free stage): polls with pauses.
__device__ __forceinline__ bool w4_wait_relaxed(uint32_t bar, uint32_t parity) {
  for (unsigned spins = 0; spins < kTcSpinLimit; spins++) {
    if (tc_mbar_try_wait(bar, parity)) return true;
    __nanosleep(100);
  }
  return false;
}
__device__ __forceinline__ void w4_st_cluster_b32(uint32_t caddr, uint32_t v) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(caddr), "r"(v) : "memory");
}
__device__ __forceinline__ void w4_st_cluster_b8(uint32_t caddr, uint32_t v) {
  asm volatile("st.shared::cluster.b8 [%0], %1;" ::"r"(caddr), "r"(v) : "memory");
}
__device__ __forceinline__ void w4_arrive_cluster(uint32_t cbar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cbar) : "memory");
}

// 16-byte global load that stays where it is written: a batch of these is issued before anything consumes them.
__device__ __forceinline__ uint4 w4_ld16(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr) : "memory");
  return v;
}

__device__ __forceinline__ void w4_unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; j++) {
    f[2 * j] = bf16_bits_to_f32((uint16_t)(w[j] & 0xffff));
    f[2 * j + 1] = bf16_bits_to_f32((uint16_t)(w[j] >> 16));
  }
}

// ---------------------------------------------------------------- activation split for 32 / 64 token tiles
//   terms [k step][A tile][128 rows][64 bytes], sfa [k step][A tile][512]
// MMA row of (token, term): TOKP 32: 32*(tok/8) + 8*term + tok%8; TOKP 64: tile term/2, row 32*(tok/16) + 16*(term%2) + tok%16.
// Scale byte of MMA row R, 32-wide block j of the k step: (R%32)*16 + (R/32)*4 + j. One thread per 8 elements.
__device__ __forceinline__ void w4_emit(float (&f)[8], bool store, int tok, int i, int TOKP, uint8_t* __restrict__ terms,
                                        uint8_t* __restrict__ sfa) {
  const int sx = w4_block_exp(f);
  uint32_t packed[4];
  w4_digits(f, sx, packed);
  if (!store) return;
  const int ks = i >> 4, chunk = i & 15, j = chunk >> 2;
  const int at = TOKP == 64 ? 2 : 1;
#pragma unroll
  for (int t = 0; t < 4; t++) {
    const int tile = TOKP == 64 ? t >> 1 : 0;
    const int R = TOKP == 64 ? 32 * (tok >> 4) + 16 * (t & 1) + (tok & 15) : 32 * (tok >> 3) + 8 * t + (tok & 7);
    *reinterpret_cast<uint32_t*>(terms + ((size_t)(ks * at + tile) * 128 + R) * 64 + chunk * 4) = packed[t];
    if ((chunk & 3) == 0) sfa[(size_t)(ks * at + tile) * 512 + (R % 32) * 16 + (R / 32) * 4 + j] = (uint8_t)(127 + sx + 3 * t);
  }
}

__global__ void __launch_bounds__(128) split4w_kernel(const uint16_t* __restrict__ x, int M, int K, int KS, int TOKP,
                                                      uint8_t* __restrict__ terms, uint8_t* __restrict__ sfa) {
  pdl_trigger();
  pdl_wait();
  const int nvp = KS * 16;  // 8-element vectors of a padded row
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool in = idx < (long long)TOKP * nvp;  // whole warps: every lane takes part in the shuffles
  const int tok = in ? (int)(idx / nvp) : 0, i = in ? (int)(idx % nvp) : 0;
  float f[8];
#pragma unroll
  for (int j = 0; j < 8; j++) f[j] = 0.0f;
  if (in && tok < M && i * 8 < K) w4_unpack8(*reinterpret_cast<const uint4*>(x + (size_t)tok * K + i * 8), f);
  w4_emit(f, in, tok, i, TOKP, terms, sfa);
}

// RMSNorm fused into the split: one CTA per token row of up to 8192 elements.
constexpr int kW4NormThreads = 256;
__global__ void __launch_bounds__(kW4NormThreads) rmsnorm_split4w_kernel(const uint16_t* __restrict__ x, const void* __restrict__ gamma,
                                                                         int gamma_f32, float eps, int M, int K, int KS, int TOKP,
                                                                         uint8_t* __restrict__ terms, uint8_t* __restrict__ sfa) {
  __shared__ float red[kW4NormThreads / 32];
  pdl_trigger();
  pdl_wait();
  const int tok = blockIdx.x;
  const bool live_row = tok < M;
  const int nv = K / 8, nvp = KS * 16;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)tok * K);
  float xv[4][8], gm[4][8];
  float ss = 0.0f;
#pragma unroll
  for (int q = 0; q < 4; q++) {
    const int i = threadIdx.x + q * kW4NormThreads;
    const bool have = live_row && i < nv;
    w4_unpack8(have ? xr[i] : make_uint4(0, 0, 0, 0), xv[q]);
    if (have && gamma_f32) {
      const float4 g0 = reinterpret_cast<const float4*>(gamma)[2 * i], g1 = reinterpret_cast<const float4*>(gamma)[2 * i + 1];
      gm[q][0] = g0.x; gm[q][1] = g0.y; gm[q][2] = g0.z; gm[q][3] = g0.w;
      gm[q][4] = g1.x; gm[q][5] = g1.y; gm[q][6] = g1.z; gm[q][7] = g1.w;
    } else if (have) {
      w4_unpack8(reinterpret_cast<const uint4*>(gamma)[i], gm[q]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) gm[q][j] = 0.0f;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) ss += xv[q][j] * xv[q][j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int w = 0; w < kW4NormThreads / 32; w++) tot += red[w];
  const float inv = rsqrtf(tot / (float)K + eps);
#pragma unroll
  for (int q = 0; q < 4; q++) {
    const int i = threadIdx.x + q * kW4NormThreads;
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; j++) f[j] = bf16_bits_to_f32(f32_to_bf16_bits(xv[q][j] * inv * gm[q][j]));
    w4_emit(f, i < nvp, tok, i < nvp ? i : 0, TOKP, terms, sfa);
  }
}

// ---------------------------------------------------------------- epilogue of 4 or 8 consecutive output features of one token
template <bool DUAL, int W>
__device__ __forceinline__ void w4_finish(const TcParams& p, int tok, int n, const float (&v)[W], const float (&u)[W]) {
  const size_t o = (size_t)tok * p.N + n;
  float x[W];
  __align__(16) uint16_t tb[W], tm[W], tr[W];
  if (p.bias) {
#pragma unroll
    for (int i = 0; i < W; i += 4) *reinterpret_cast<uint2*>(tb + i) = *reinterpret_cast<const uint2*>(p.bias + n + i);
  }
  if (p.mul_in) {
#pragma unroll
    for (int i = 0; i < W; i += 4) *reinterpret_cast<uint2*>(tm + i) = *reinterpret_cast<const uint2*>(p.mul_in + o + i);
  }
  if (p.res) {
#pragma unroll
    for (int i = 0; i < W; i += 4) *reinterpret_cast<uint2*>(tr + i) = *reinterpret_cast<const uint2*>(p.res + o + i);
  }
#pragma unroll
  for (int i = 0; i < W; i++) x[i] = v[i] + (p.bias ? bf16_bits_to_f32(tb[i]) : 0.0f);
  switch (p.act) {
    case TPX_ACT_GELU:
#pragma unroll
      for (int i = 0; i < W; i++) x[i] = 0.5f * x[i] * (1.0f + erff(x[i] * 0.70710678118654752f));
      break;
    case TPX_ACT_SILU:
#pragma unroll
      for (int i = 0; i < W; i++) x[i] = __fdividef(x[i], 1.0f + __expf(-x[i]));
      break;
    case TPX_ACT_RELU:
#pragma unroll
      for (int i = 0; i < W; i++) x[i] = fmaxf(x[i], 0.0f);
      break;
    default: break;
  }
  if (DUAL) {
#pragma unroll
    for (int i = 0; i < W; i++) x[i] *= u[i];
  }
  if (p.mul_in) {
#pragma unroll
    for (int i = 0; i < W; i++) x[i] *= bf16_bits_to_f32(tm[i]);
  }
  if (p.res) {
#pragma unroll
    for (int i = 0; i < W; i++) x[i] += bf16_bits_to_f32(tr[i]) * p.res_scale;
  }
  __align__(16) uint16_t out[W];
#pragma unroll
  for (int i = 0; i < W; i++) out[i] = f32_to_bf16_bits(x[i]);
#pragma unroll
  for (int i = 0; i < W; i += 4) *reinterpret_cast<uint2*>(p.y + o + i) = *reinterpret_cast<const uint2*>(out + i);
}

// ---------------------------------------------------------------- the GEMM kernel
template <int TOKP, bool DUAL>
__global__ void __launch_bounds__(TOKP == 8 ? 64 + kW4ConvThreads : kTcThreads, 1)
qlinear_tcw4_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, W4Params pp) {
  using C = W4Cfg<TOKP>;
  constexpr int UKS = C::UKS;
  const TcParams& p = pp.t;
  extern __shared__ unsigned char w4_smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[kW4MaxStages], bar_empty[kW4MaxStages];
  __shared__ __align__(8) unsigned long long bar_acc_full, bar_acc_empty, bar_a_ready, bar_lut;
  __shared__ uint32_t tmem_holder;
  __shared__ float inv_rms[8];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (tc_smem_u32(w4_smem_raw) + 1023u) & ~1023u;
  const int STAGES = pp.stages;
  if (threadIdx.x == 0) tc_stamp(p, 0);

  const long long G = gridDim.x;
  const long long T = p.TN;
  const int crank = p.cluster > 1 ? (int)tc_cluster_rank() : 0;
  const long long ctile = blockIdx.x / p.cluster;
  // whole tiles: CTA b owns tiles [b*T/G, (b+1)*T/G); cluster: member r of cluster t owns units [r*KS/c, (r+1)*KS/c) of tile t
  const long long u0 = p.cluster > 1 ? ctile * p.KS + (long long)crank * p.KS / p.cluster : ((long long)blockIdx.x * T / G) * p.KS;
  const long long u1 = p.cluster > 1 ? ctile * p.KS + ((long long)crank + 1) * p.KS / p.cluster : (((long long)blockIdx.x + 1) * T / G) * p.KS;
  const int nunits = (int)(u1 - u0);
  const int tile0 = (int)(u0 / p.KS), ks0 = (int)(u0 % p.KS);
  // resident terms: the k steps [res_k0, res_k0 + res_n) of every tile this CTA works on
  const int res_k0 = ks0 * UKS;
  const int res_n = (p.cluster > 1 ? nunits : p.KS) * UKS;
  const uint32_t res_a = smem_base;                                    // [res_n][32 rows][64 B]
  const uint32_t res_sf = smem_base + (uint32_t)res_n * C::RES_A1;     // [res_n][512]
  const uint32_t lut_s = (res_sf + (uint32_t)res_n * 512 + 15u) & ~15u;  // [4096] words: the split table
  const uint32_t stage0 = C::RES ? ((lut_s + 16384u + 1023u) & ~1023u) : smem_base;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kW4MaxStages; s++) {
      tc_mbar_init(tc_smem_u32(&bar_full[s]), 1);
      tc_mbar_init(tc_smem_u32(&bar_empty[s]), 1);
    }
    tc_mbar_init(tc_smem_u32(&bar_acc_full), 1);
    tc_mbar_init(tc_smem_u32(&bar_acc_empty), 4);
    tc_mbar_init(tc_smem_u32(&bar_a_ready), (uint32_t)kW4ConvThreads * (uint32_t)(pp.share > 1 ? pp.share : 1));
    tc_mbar_init(tc_smem_u32(&bar_lut), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(&tmem_holder)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_holder;
  if (C::RES && pp.share > 1) tc_cluster_sync();  // every member's barriers exist before anyone arrives on them from afar
  if (threadIdx.x == 0) tc_stamp(p, 1);
  pdl_trigger();

  // weight tiles (of 128 features) of feature tile t at k step ks: a pair is stored as [t][ks][gate, up], single
  // weights as [tile128][ks], so the two halves of a 256-feature tile are `ksteps` tiles apart
  auto wtile_a = [&](int t, int kstep) { return DUAL ? (t * pp.ksteps + kstep) * 2 : (2 * t * pp.ksteps + kstep); };
  auto wtile_b = [&](int t, int kstep) { return DUAL ? (t * pp.ksteps + kstep) * 2 + 1 : ((2 * t + 1) * pp.ksteps + kstep); };
  auto has_b = [&](int t) { return DUAL || 2 * t + 1 < pp.tiles128; };
  // stage layout: [A terms UKS*A1 (TOKP 32/64)][weights UKS*B1][activation scale blocks UKS*SFA1 (TOKP 32/64)][weight scale blocks UKS*1024]
  constexpr uint32_t OFF_B = C::RES ? 0 : UKS * C::A1;
  constexpr uint32_t OFF_SFA = OFF_B + UKS * C::B1;
  constexpr uint32_t OFF_SFW = OFF_SFA + (C::RES ? 0 : UKS * C::SFA1);

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      auto fetch_w = [&](int s, int t, int ks) {
        const uint32_t st = stage0 + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t bar = tc_smem_u32(&bar_full[s]);
        const bool second = has_b(t);
        tc_mbar_expect_tx(bar, (C::RES ? 0 : UKS * (C::A1 + C::SFA1)) + UKS * (second ? C::B1 + 1024 : C::B1 / 2 + 512));
#pragma unroll
        for (int kk = 0; kk < UKS; kk++) {
          const int ta = wtile_a(t, ks * UKS + kk), tb = wtile_b(t, ks * UKS + kk);
          if (DUAL) {
            tc_tma_2d(st + OFF_B + kk * C::B1, &tmW, 0, ta * 128, bar);  // 256 rows: gate tile and up tile are adjacent
            tc_bulk_g2s(st + OFF_SFW + kk * 1024, p.sfa + (size_t)ta * 512, 1024, bar);
          } else {
            tc_tma_2d(st + OFF_B + kk * C::B1, &tmW, 0, ta * 128, bar);
            tc_bulk_g2s(st + OFF_SFW + kk * 1024, p.sfa + (size_t)ta * 512, 512, bar);
            if (second) {
              tc_tma_2d(st + OFF_B + kk * C::B1 + C::B1 / 2, &tmW, 0, tb * 128, bar);
              tc_bulk_g2s(st + OFF_SFW + kk * 1024 + 512, p.sfa + (size_t)tb * 512, 512, bar);
            }
          }
        }
      };
      auto fetch_x = [&](int s, int ks) {  // TOKP 32/64: the stage's activation terms (256 rows of 64 bytes) and their scale blocks
        const uint32_t st = stage0 + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t bar = tc_smem_u32(&bar_full[s]);
        tc_tma_2d(st, &tmX, 0, ks * UKS * C::ATILES * 128, bar);
        tc_bulk_g2s(st + OFF_SFA, p.sfb + (size_t)ks * UKS * C::SFA1, UKS * C::SFA1, bar);
      };
      if (C::RES) {  // the split table: constant, fetched ahead of everything else
        tc_mbar_expect_tx(tc_smem_u32(&bar_lut), 16384);
        tc_bulk_g2s(lut_s, g_w4_lut, 16384, tc_smem_u32(&bar_lut));
      }
      const int early = nunits < STAGES ? nunits : STAGES;
      int ptile = tile0, pks = ks0;
      for (int pit = 0; pit < early; pit++) {  // weights do not depend on earlier grids: out before the dependency wait
        fetch_w(pit, ptile, pks);
        if (++pks == p.KS) { pks = 0; ptile++; }
      }
      if (!C::RES) pdl_wait();
      int tile = tile0, ks = ks0;
      for (int it = 0; it < nunits; it++) {
        const int s = it % STAGES;
        if (it >= STAGES) {
          if (!w4_wait_relaxed(tc_smem_u32(&bar_empty[s]), (uint32_t)((it / STAGES - 1) & 1))) { atomicExch(p.err, 2u); break; }
          fetch_w(s, tile, ks);
        }
        if (!C::RES) fetch_x(s, ks);
        if (++ks == p.KS) { ks = 0; tile++; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // kind::mxf4: A = B = E2M1 (1), both K-major, N = 256, UE8M0 scales, M = 128, K = 64
      const uint32_t idesc0 = (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
      bool ok = true;
      if (C::RES) {  // the epilogue warps (of this CTA, or of all members of its cluster) have built the terms
        ok = w4_wait_cluster(tc_smem_u32(&bar_a_ready), 0);
        if (!ok) atomicExch(p.err, 5u);
        asm volatile("fence.proxy.async;" ::: "memory");  // written with ordinary stores, read by the tensor core
        tc_fence_after();
      }
      int ks = ks0;
      uint32_t acc_phase = 0;
      bool fresh = true;
      for (int it = 0; ok && it < nunits; it++) {
        const int s = it % STAGES;
        const uint32_t ph = (uint32_t)((it / STAGES) & 1);
        if (fresh && it > 0) {
          if (!tc_wait(tc_smem_u32(&bar_acc_empty), acc_phase)) { atomicExch(p.err, 3u); break; }
          acc_phase ^= 1;
        }
        if (!tc_wait(tc_smem_u32(&bar_full[s]), ph)) { atomicExch(p.err, 4u); break; }
        if (it == 0) tc_stamp(p, 2);
        if (it == nunits - 1) tc_stamp(p, 3);
        tc_fence_after();
        const uint32_t st = stage0 + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t ring = tmem + C::RING_COL0 + (uint32_t)s * UKS * C::SFC;
        const bool part_end = (ks == p.KS - 1) || (it == nunits - 1);
#pragma unroll
        for (int kk = 0; kk < UKS; kk++) {
          const uint32_t sfw = ring + kk * C::SFC;  // 8 weight columns, then 4 per A tile
          tc_cp_sf(sfw, tc_sf_desc(st + OFF_SFW + kk * 1024));
          tc_cp_sf(sfw + 4, tc_sf_desc(st + OFF_SFW + kk * 1024 + 512));
          const int kl = (ks - ks0 * (p.cluster > 1 ? 1 : 0)) * UKS + kk;  // index of this k step among the resident ones
          if (C::RES) {
            tc_cp_sf(sfw + 8, tc_sf_desc(res_sf + (uint32_t)kl * 512));
          } else {
#pragma unroll
            for (int a = 0; a < C::ATILES; a++) tc_cp_sf(sfw + 8 + 4 * a, tc_sf_desc(st + OFF_SFA + (kk * C::ATILES + a) * 512));
          }
#pragma unroll
          for (int j = 0; j < 2; j++) {  // k 64*j .. 64*j+63 of the step: 32 bytes along the rows, scale bytes 2j and 2j+1
            const uint32_t sfid = (uint32_t)(2 * j);
            const uint32_t idesc = idesc0 | (sfid << 29) | (sfid << 4);
            const uint64_t bdesc = w4_desc64(st + OFF_B + kk * C::B1, 512) + (uint64_t)(2 * j);
#pragma unroll
            for (int a = 0; a < C::ATILES; a++) {
              const uint64_t adesc = (C::RES ? w4_desc64(res_a + (uint32_t)kl * C::RES_A1, 128)
                                             : w4_desc64(st + (kk * C::ATILES + a) * 128 * 64, 512)) + (uint64_t)(2 * j);
              const uint32_t sfa_t = sfw + 8 + 4 * a;
              tc_mma_f4(tmem, adesc, bdesc, idesc, sfa_t | (sfid << 30), sfw | (sfid << 30), (fresh && kk == 0 && j == 0 && a == 0) ? 0u : 1u);
            }
          }
        }
        tc_commit(tc_smem_u32(&bar_empty[s]));
        if (part_end) tc_commit(tc_smem_u32(&bar_acc_full));
        fresh = part_end;
        if (++ks == p.KS) ks = 0;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ warps 2..: (TOKP 8) build the terms; warps 2..5: the epilogue
    const int sub = warp & 3;  // tensor-memory lanes 32*sub .. 32*sub+31 belong to this warp
    pdl_wait();  // x, residual and multiplier inputs belong to earlier grids
    if (threadIdx.x == 64) tc_stamp(p, 7);
    if (C::RES) {
      // The split is a chain of dependent integer operations: one warp per scheduler would run it at a fraction of the
      // issue rate, so the kernel carries extra warps that do nothing else (kW4ConvThreads in all, with the epilogue warps).
      constexpr int NCV = kW4ConvThreads;
      const int ct = (int)threadIdx.x - 64;
      if (pp.gamma) {  // RMSNorm statistics over the whole rows (this CTA may only multiply a slice of K)
        for (int tok = warp - 2; tok < p.M; tok += NCV / 32) {
          const uint4* xr = reinterpret_cast<const uint4*>(pp.x + (size_t)tok * p.K);
          float ss = 0.0f;
          for (int i = lane; i < p.K / 8; i += 32) {
            float f[8];
            w4_unpack8(xr[i], f);
#pragma unroll
            for (int j = 0; j < 8; j++) ss += f[j] * f[j];
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          if (lane == 0) inv_rms[tok] = rsqrtf(ss / (float)p.K + pp.eps);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NCV) : "memory");
      }
      // Work items are (token, 8-element chunk) pairs; the four chunks of a 32-wide block sit in four neighbouring lanes.
      // With `share` members building together, member r takes the resident k steps r, r + share, ... and stores each
      // result into every member's shared memory.
      const int nshare = pp.share > 1 ? pp.share : 1;
      const int myrank = nshare > 1 ? (int)tc_cluster_rank() : 0;
      const int myks = (res_n - myrank + nshare - 1) / nshare;   // k steps this CTA builds
      const int nch = myks * 16;
      const int total = p.M * nch;
      constexpr int U = 4;  // items per thread and round: loads first, then the arithmetic of all, then the stores
      const uint32_t* lut = reinterpret_cast<const uint32_t*>(w4_smem_raw + (lut_s - tc_smem_u32(w4_smem_raw)));
      if (!tc_wait(tc_smem_u32(&bar_lut), 0) && lane == 0) atomicExch(p.err, 8u);
#pragma unroll 1
      for (int base = 0; base < total; base += NCV * U) {
        uint4 raw[U];
        int tokv[U], cv[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
          const int idx = base + u * NCV + ct;
          const bool in = idx < total;
          tokv[u] = in ? idx / nch : -1;
          cv[u] = in ? idx % nch : 0;
          raw[u] = make_uint4(0, 0, 0, 0);
          const int k = (res_k0 + myrank + (cv[u] >> 4) * nshare) * 128 + (cv[u] & 15) * 8;
          if (in && k < p.K) raw[u] = w4_ld16(pp.x + (size_t)tokv[u] * p.K + k);
        }
        uint32_t packed[U][4];
        int sxv[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
          const bool in = tokv[u] >= 0;
          float f[8];
          w4_unpack8(raw[u], f);
#ifdef TPX_DEBUG
          if (threadIdx.x == 64 && base == 0 && u == 0 && p.tl) { if (f[0] == 12345.678f) inv_rms[7] = 1.0f; tc_stamp(p, 1); }
#endif
          if (pp.gamma) {  // the normalised value rounded to bf16, as the separate kernel would store it
            const int k = (res_k0 + myrank + (cv[u] >> 4) * nshare) * 128 + (cv[u] & 15) * 8;
            float g[8];
#pragma unroll
            for (int j = 0; j < 8; j++) g[j] = 0.0f;
            if (in && k < p.K) {
              if (pp.gamma_f32) {
                const float4 g0 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(pp.gamma) + k);
                const float4 g1 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(pp.gamma) + k + 4);
                g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
              } else {
                w4_unpack8(*reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(pp.gamma) + k), g);
              }
            }
            const float inv = in ? inv_rms[tokv[u]] : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++) f[j] = bf16_bits_to_f32(f32_to_bf16_bits(f[j] * inv * g[j]));
          }
          sxv[u] = w4_block_exp(f);
          w4_digits_lut(f, sxv[u], lut, packed[u]);
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
          if (tokv[u] < 0) continue;
          const int kl = myrank + (cv[u] >> 4) * nshare, c16 = cv[u] & 15;
          const int q = tokv[u] >> 1, i2 = tokv[u] & 1;
#pragma unroll
          for (int t = 0; t < 4; t++) {
            const int row = 8 * q + 2 * t + i2;  // stored row; the MMA reads it as its row 32q + 8t + i2
            const uint32_t off = (uint32_t)kl * C::RES_A1 + (uint32_t)row * 64 + ((uint32_t)((c16 >> 2) ^ ((row >> 1) & 3)) << 4) + (uint32_t)(c16 & 3) * 4;
            const uint32_t sfo = (uint32_t)kl * 512 + (uint32_t)(8 * t + i2) * 16 + (uint32_t)q * 4 + (uint32_t)(c16 >> 2);
            if (nshare == 1) {
              asm volatile("st.shared.b32 [%0], %1;" ::"r"(res_a + off), "r"(packed[u][t]) : "memory");
              if ((c16 & 3) == 0) asm volatile("st.shared.b8 [%0], %1;" ::"r"(res_sf + sfo), "r"((uint32_t)(127 + sxv[u] + 3 * t)) : "memory");
            } else {
              for (int m = 0; m < nshare; m++) {
                w4_st_cluster_b32(tc_mapa(res_a + off, (uint32_t)m), packed[u][t]);
                if ((c16 & 3) == 0) w4_st_cluster_b8(tc_mapa(res_sf + sfo, (uint32_t)m), (uint32_t)(127 + sxv[u] + 3 * t));
              }
            }
          }
        }
      }
      asm volatile("fence.proxy.async;" ::: "memory");  // the tensor core reads these bytes through the async proxy
      if (nshare == 1) {
        tc_mbar_arrive(tc_smem_u32(&bar_a_ready));
      } else {
        for (int m = 0; m < nshare; m++) w4_arrive_cluster(tc_mapa(tc_smem_u32(&bar_a_ready), (uint32_t)m));
      }
      if (threadIdx.x == 64) tc_stamp(p, 4);
    }
    if (warp < 6) {  // ---------------------------------------------- epilogue
    const uint32_t lane_base = ((uint32_t)(sub * 32)) << 16;
    constexpr bool TWO = TOKP != 64;  // two shuffle rounds (four term lanes per token) or one (two)
    const int tok = TWO ? sub * C::LIVE + (lane & 7) : sub * 16 + (lane & 15);
    const bool lane_live = TWO ? (lane & 7) < C::LIVE : true;
    const int hi = lane >> 4, g = (lane >> 3) & 1;
    constexpr int W = TWO ? 4 : 8;  // output features a lane finishes per 16-column chunk
    int tile = tile0, ks = ks0;
    uint32_t acc_phase = 0;
    for (int it = 0; it < nunits; it++) {
      const bool part_end = (ks == p.KS - 1) || (it == nunits - 1);
      if (part_end) {
        if (!tc_wait(tc_smem_u32(&bar_acc_full), acc_phase)) {
          if (lane == 0) atomicExch(p.err, 6u);
          break;
        }
        acc_phase ^= 1;
        tc_fence_after();
        if (threadIdx.x == 64 && it == nunits - 1) tc_stamp(p, 5);
        constexpr int CHUNKS = DUAL ? 8 : 16;
#pragma unroll 1
        for (int c0 = 0; c0 < CHUNKS; c0 += 2) {  // two 16-column chunks per round trip to tensor memory
          uint32_t a[2][16], b[2][16];
#pragma unroll
          for (int q = 0; q < 2; q++) {
            tc_ld_x16(tmem + lane_base + (c0 + q) * 16, a[q]);
            if (DUAL) tc_ld_x16(tmem + lane_base + 128 + (c0 + q) * 16, b[q]);
          }
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int q = 0; q < 2; q++) {
            // the term lanes of a token exchange halves: after round one a lane holds 8 of the 16 columns summed over two
            // terms, after round two (TOKP 8/32) 4 columns summed over all four
            float v8[8], u8[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
              const float mine = __uint_as_float(hi ? a[q][i + 8] : a[q][i]);
              const float send = __uint_as_float(hi ? a[q][i] : a[q][i + 8]);
              v8[i] = mine + __shfl_xor_sync(0xffffffffu, send, 16);
              if (DUAL) {
                const float mine2 = __uint_as_float(hi ? b[q][i + 8] : b[q][i]);
                const float send2 = __uint_as_float(hi ? b[q][i] : b[q][i + 8]);
                u8[i] = mine2 + __shfl_xor_sync(0xffffffffu, send2, 16);
              } else {
                u8[i] = 0.0f;
              }
            }
            float v[W], u[W];
            int col;
            if (TWO) {
#pragma unroll
              for (int i = 0; i < 4; i++) {
                const float mine = g ? v8[i + 4] : v8[i];
                const float send = g ? v8[i] : v8[i + 4];
                v[i] = mine + __shfl_xor_sync(0xffffffffu, send, 8);
                if (DUAL) {
                  const float mine2 = g ? u8[i + 4] : u8[i];
                  const float send2 = g ? u8[i] : u8[i + 4];
                  u[i] = mine2 + __shfl_xor_sync(0xffffffffu, send2, 8);
                } else {
                  u[i] = 0.0f;
                }
              }
              col = (c0 + q) * 16 + hi * 8 + g * 4;
            } else {
#pragma unroll
              for (int i = 0; i < W; i++) { v[i] = v8[i]; u[i] = u8[i]; }
              col = (c0 + q) * 16 + hi * 8;
            }
            if (p.cluster == 1) {
              const int n = DUAL ? tile * 128 + col : tile * 256 + col;
              if (lane_live && tok < p.M && n < p.N) w4_finish<DUAL, W>(p, tok, n, v, u);
            } else if (lane_live) {  // partial of a cluster member: [token][256 columns] fp32 at the start of shared memory
              const uint32_t sp = smem_base + (uint32_t)((tok * 256 + col) * 4);
#pragma unroll
              for (int i = 0; i < W; i += 4) {
                tc_st_shared_f4(sp + i * 4, make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]));
                if (DUAL) tc_st_shared_f4(sp + 512 + i * 4, make_float4(u[i], u[i + 1], u[i + 2], u[i + 3]));
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) tc_mbar_arrive(tc_smem_u32(&bar_acc_empty));
      }
      if (++ks == p.KS) { ks = 0; tile++; }
    }
    }  // warps 2..5
  }
  if (threadIdx.x == 64) tc_stamp(p, 6);
  tc_fence_before();
  __syncthreads();
  if (p.cluster > 1) {
    // every member's partial is in its own shared memory; the (token, 8 features) groups of the tile go round the
    // members, each adds the members' parts in rank order (distributed shared memory reads) and finishes its groups.
    // Nobody leaves before all have finished reading.
    tc_cluster_sync();
    if (warp >= 2 && warp < 6) {
      constexpr int GROUPS = DUAL ? 16 : 32;  // groups of 8 output features per token
      const int et = (int)threadIdx.x - 64;
      const int live_tok = p.M < TOKP ? p.M : TOKP;
      for (int i = crank * 128 + et; i < live_tok * GROUPS; i += 128 * p.cluster) {
        const int tk = i / GROUPS, col = (i % GROUPS) * 8;
        const int n = DUAL ? (int)ctile * 128 + col : (int)ctile * 256 + col;
        if (n >= p.N) continue;
        float v[8], u[8];
#pragma unroll
        for (int q = 0; q < 8; q++) v[q] = u[q] = 0.0f;
        const uint32_t sp = smem_base + (uint32_t)((tk * 256 + col) * 4);
        tc_cluster_sum<2, 4>(sp, p.cluster, v);
        if (DUAL) tc_cluster_sum<2, 4>(sp + 512, p.cluster, u);
        w4_finish<DUAL, 8>(p, tk, n, v, u);
      }
    }
    tc_cluster_sync();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// ---------------------------------------------------------------- host side
struct W4Plan {
  int tokp, KS, KU, tiles128, TN, grid, cluster, res_n, stages;
  size_t smem, off_terms, off_sfa, total;
  bool ok;
};

static W4Plan w4_plan(int64_t M, int64_t N, int64_t K, bool pair) {
  W4Plan pl = {};
  pl.tokp = M <= 8 ? 8 : M <= 32 ? 32 : 64;
  const int uks = pl.tokp == 64 ? 1 : 2;
  pl.KS = tc_padded_ks(K, pair);
  pl.KU = pl.KS / uks;
  pl.tiles128 = (int)((N + 127) / 128);
  pl.TN = pair ? pl.tiles128 : (pl.tiles128 + 1) / 2;
  const long long T = pl.TN;
  const int sms = sm_count();
  const bool whole = (T * 10 >= (long long)sms * 7 && T <= sms) || T >= 8LL * sms;
  pl.cluster = 1;
  if (!whole) {
    if (T * 2 > sms || knobs().tc_cluster == 0) return pl;  // tile counts this kernel does not serve
    int c = (int)(sms / T);
    if (c > 8) c = 8;
    if (c > pl.KU) c = pl.KU;
    if (c < 2) return pl;
    pl.cluster = c;
  }
  pl.grid = pl.cluster > 1 ? (int)T * pl.cluster : (int)(T < sms ? T : sms);
  return pl;
}

// Shared memory and stage count for a given cluster size (the launch may have to take a smaller cluster than planned).
static void w4_size(W4Plan& pl, int cluster) {
  const int uks = pl.tokp == 64 ? 1 : 2;
  const int budget = 227 * 1024 - 2048;
  const int stage = pl.tokp == 8 ? W4Cfg<8>::STAGE_BYTES : pl.tokp == 32 ? W4Cfg<32>::STAGE_BYTES : W4Cfg<64>::STAGE_BYTES;
  pl.cluster = cluster;
  pl.res_n = (cluster > 1 ? (pl.KU + cluster - 1) / cluster : pl.KU) * uks;
  const int res = pl.tokp == 8 ? (pl.res_n * 2560 + 16384 + 16 + 1023) / 1024 * 1024 : 0;
  int st = (budget - res) / stage;
  if (st > kW4MaxStages) st = kW4MaxStages;
  pl.stages = st;
  pl.smem = (size_t)res + (size_t)st * stage + 1024;
  pl.ok = st >= 2 && (pl.tokp != 8 || pl.res_n <= W4Cfg<8>::MAX_RES_KSTEPS);
  if ((size_t)pl.tokp * 1024 > (size_t)res + (size_t)st * stage) pl.ok = false;  // a cluster member's partial tile must fit
}

static W4Plan w4_full_plan(int64_t M, int64_t N, int64_t K, bool pair) {
  W4Plan pl = w4_plan(M, N, K, pair);
  if (pl.grid == 0) return pl;
  w4_size(pl, pl.cluster);
  if (!pl.ok && pl.tokp == 8) {  // K range too long to keep resident: the 32-token class with the split kernel
    pl.tokp = 32;
    w4_size(pl, pl.cluster);
  }
  size_t o = kTcCounterBytes;
  auto bump = [&](size_t bytes) { size_t r = o; o += (bytes + 1023) & ~(size_t)1023; return r; };
  const int at = pl.tokp == 64 ? 2 : 1;
  pl.off_terms = bump(pl.tokp == 8 ? 0 : (size_t)pl.KS * at * 128 * 64);
  pl.off_sfa = bump(pl.tokp == 8 ? 0 : (size_t)pl.KS * at * 512);
  pl.total = o;
  return pl;
}

bool tcw4_serves(int64_t M, int64_t N, int64_t K, bool pair) {
  if (M < 1 || M > 64) return false;
  const W4Plan pl = w4_full_plan(M, N, K, pair);
  return pl.grid > 0 && pl.ok;
}

size_t tcw4_scratch_bytes(int64_t M, int64_t N, int64_t K, bool pair) { return w4_full_plan(M, N, K, pair).total; }

template <int TOKP, bool DUAL>
static int w4_launch(const CUtensorMap& w, const CUtensorMap& x, W4Params pp, W4Plan pl, cudaStream_t st) {
  static int opted[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int di = (dev >= 0 && dev < 16) ? dev : 0;
  if (opted[di] < (int)pl.smem) {
    TPX_CUDA_OK(cudaFuncSetAttribute(qlinear_tcw4_kernel<TOKP, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024));
    opted[di] = 227 * 1024 - 1024;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(TOKP == 8 ? 64 + kW4ConvThreads : kTcThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  int c = pl.cluster;
  if (c > 1) {
    // the largest cluster size, from the planned one down, of which one cluster per tile can be resident at once
    static int fits[16][9] = {};
    for (; c >= 2; c--) {
      W4Plan q = pl;
      w4_size(q, c);
      if (!q.ok || q.tokp != pl.tokp) continue;
      int& f = fits[di][c];
      if (f == 0) {
        attr[1].val.clusterDim.x = (unsigned)c;
        cfg.gridDim = dim3((unsigned)(pl.TN * c));
        cfg.dynamicSmemBytes = 227 * 1024 - 1024;
        cfg.numAttrs = 2;
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, qlinear_tcw4_kernel<TOKP, DUAL>, &cfg);
        if (e != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
        f = 1 + n;
      }
      if (f - 1 >= pl.TN) { pl = q; break; }
    }
    TPX_REQUIRE(c >= 2, TPX_ERR_UNSUPPORTED, "qlinear_mxfp4_tc (wide packed-fp4 kernel): no cluster size fits %d tiles on this device", pl.TN);
  }
  pp.t.cluster = c > 1 ? c : 1;
  pp.stages = pl.stages;
  pp.share = 1;
  int cdim = pp.t.cluster;
  if (TOKP == 8 && c <= 1 && pp.t.M >= 2) {
    // whole tiles: every CTA needs the terms of the whole K range; the members of a cluster build them together
    static int share_ok[16][9] = {};  // 0 unknown, 1 no, 2 yes
    for (int sh = 8; sh >= 2; sh--) {
      if (pl.grid % sh) continue;
      int& f = share_ok[di][sh];
      if (f == 0) {
        attr[1].val.clusterDim.x = (unsigned)sh;
        cfg.gridDim = dim3((unsigned)pl.grid);
        cfg.dynamicSmemBytes = 227 * 1024 - 1024;
        cfg.numAttrs = 2;
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, qlinear_tcw4_kernel<TOKP, DUAL>, &cfg);
        if (e != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
        f = n >= 1 ? 2 : 1;
      }
      if (f == 2) { pp.share = sh; cdim = sh; break; }
    }
  }
  attr[1].val.clusterDim.x = (unsigned)cdim;
  cfg.gridDim = dim3((unsigned)(c > 1 ? pl.TN * c : pl.grid));
  cfg.dynamicSmemBytes = pl.smem;
  cfg.numAttrs = cdim > 1 ? 2 : 1;
  count_launch();
  TPX_CUDA_OK(cudaLaunchKernelEx(&cfg, qlinear_tcw4_kernel<TOKP, DUAL>, w, x, pp));
  return TPX_OK;
}

int tcw4_run(const uint8_t* wq, const uint8_t* sfa, bool pair, const uint16_t* x, int64_t M, int64_t N, int64_t K, const TcParams& base,
             void* scratch, size_t scratch_bytes, cudaStream_t st, const TcNorm* norm) {
  W4Plan pl = w4_full_plan(M, N, K, pair);
  TPX_REQUIRE(pl.grid > 0 && pl.ok, TPX_ERR_UNSUPPORTED, "qlinear_mxfp4_tc (wide packed-fp4 kernel): shape M=%ld N=%ld K=%ld not served", (long)M,
              (long)N, (long)K);
  TPX_REQUIRE(scratch && scratch_bytes >= pl.total, TPX_ERR_SCRATCH, "qlinear_mxfp4_tc: scratch of %zu bytes needed, %zu given", pl.total,
              scratch_bytes);
  TPX_REQUIRE((((uintptr_t)base.y | (uintptr_t)base.bias | (uintptr_t)base.mul_in | (uintptr_t)base.res) & 15) == 0 && N % 8 == 0, TPX_ERR_ARG,
              "qlinear_mxfp4_tc: y, bias, mul_in and res must be 16-byte aligned");
  unsigned char* sc = reinterpret_cast<unsigned char*>(scratch);
  uint8_t *terms = sc + pl.off_terms, *sfx = sc + pl.off_sfa;
  const bool has_norm = norm && norm->gamma;
  if (pl.tokp != 8) {
    if (has_norm) {
      TPX_REQUIRE(pl.KS * 16 <= kW4NormThreads * 4, TPX_ERR_UNSUPPORTED, "fused RMSNorm: rows of more than %d elements are not supported (K=%ld)",
                  kW4NormThreads * 32, (long)K);
      TPX_REQUIRE((((uintptr_t)x | (uintptr_t)norm->gamma) & 15) == 0, TPX_ERR_ARG, "fused RMSNorm: x and gamma must be 16-byte aligned");
      TPX_CUDA_OK(launch_pdl(rmsnorm_split4w_kernel, dim3((unsigned)pl.tokp), dim3(kW4NormThreads), 0, st, x, norm->gamma, norm->gamma_f32,
                             norm->eps, (int)M, (int)K, pl.KS, pl.tokp, terms, sfx));
    } else {
      const long long threads = (long long)pl.tokp * pl.KS * 16;
      TPX_CUDA_OK(launch_pdl(split4w_kernel, dim3((unsigned)((threads + 127) / 128)), dim3(128), 0, st, x, (int)M, (int)K, pl.KS, pl.tokp, terms, sfx));
    }
  } else if (has_norm) {
    TPX_REQUIRE((((uintptr_t)x | (uintptr_t)norm->gamma) & 15) == 0, TPX_ERR_ARG, "fused RMSNorm: x and gamma must be 16-byte aligned");
  }
  if (pl.tokp == 8) {  // the split table of this device, once
    static bool lut_done[64] = {};
    int dev = 0;
    TPX_CUDA_OK(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !lut_done[dev]) {
      w4_lut_init_kernel<<<16, 256, 0, st>>>();
      TPX_LAUNCH_OK();
      lut_done[dev] = true;
    }
  }
  CUtensorMap mw, mx;
  const uint64_t wrows = (uint64_t)(pair ? pl.TN * 2 : pl.tiles128) * pl.KS * 128;
  int rc = tc_make_map64(&mw, wq, wrows, pair ? 256 : 128);
  if (rc) return rc;
  if (pl.tokp != 8) {
    rc = tc_make_map64(&mx, terms, (uint64_t)pl.KS * (pl.tokp == 64 ? 2 : 1) * 128, 256);
    if (rc) return rc;
  } else {
    mx = mw;  // unused by the resident class
  }
  W4Params pp = {};
  pp.t = base;
  pp.t.sfa = sfa; pp.t.sfa2 = nullptr; pp.t.sfb = sfx;
  pp.t.partial = nullptr;
  pp.t.counters = reinterpret_cast<unsigned*>(sc);
  pp.t.err = reinterpret_cast<unsigned*>(sc + kTcCounterBytes - 4);
  pp.t.M = (int)M; pp.t.N = (int)N; pp.t.K = (int)K; pp.t.KS = pl.KU; pp.t.TN = pl.TN; pp.t.TM = 1; pp.t.whole_tiles = 1;
  pp.x = x;
  pp.gamma = has_norm ? norm->gamma : nullptr;
  pp.gamma_f32 = has_norm ? norm->gamma_f32 : 0;
  pp.eps = has_norm ? norm->eps : 0.0f;
  pp.tiles128 = pl.tiles128;
  pp.ksteps = pl.KS;
  if (pair) {
    switch (pl.tokp) {
      case 8: return w4_launch<8, true>(mw, mx, pp, pl, st);
      case 32: return w4_launch<32, true>(mw, mx, pp, pl, st);
      default: return w4_launch<64, true>(mw, mx, pp, pl, st);
    }
  }
  switch (pl.tokp) {
    case 8: return w4_launch<8, false>(mw, mx, pp, pl, st);
    case 32: return w4_launch<32, false>(mw, mx, pp, pl, st);
    default: return w4_launch<64, false>(mw, mx, pp, pl, st);
  }
}

}  // namespace tpx
