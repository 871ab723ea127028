// MXFP4 weight-only linear on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// Replaces TppBlockedLinearW with the MXFP4 BRGEMM of the reference
// (src/csrc/fused_gemm.h:875-949; libxsmm flag INTERPRETE_A_AS_MXFP4_VNNI2, src/csrc/xsmm_functors.h:2646).
//
// The weight never passes through CUDA cores: TMA unpacks the 4-bit codes from HBM straight into the
// shared-memory operand layout, and tcgen05.mma kind::mxf8f6f4 multiplies E2M1 codes with their UE8M0
// block scales natively. The reference multiplies *bf16* activations, which this instruction cannot take,
// so each activation is split beforehand into two E4M3 terms that share one power-of-two scale per
// 32-wide block: x = (hi + lo) * 2^e. A bf16 value has 8 significant bits, hi and lo carry 4 each, so the
// split is exact for every element within 2^-10 of its block maximum (smaller ones keep an absolute error
// below 2^-18 of the block maximum). Two MMAs (hi, lo) accumulate into the same fp32 tile in tensor memory.
//
//   rows of W (output features) = M of the MMA (128 per tile), tokens = N (TOK per tile), K step 128
//   warp 0   : TMA producer (W tiles, activation terms, scale-factor blocks) into a ring of stages
//   warp 1   : allocates tensor memory, issues the MMAs, commits stages back to the producer
//   warps 2-5: copy the scale factors of each stage into tensor memory, then run the epilogue
//
// Work is the flat list of (output tile, k step) units cut into equal contiguous ranges, one CTA per SM:
// every SM streams the same number of weight bytes. A tile cut between CTAs is completed through fp32
// partial tiles in scratch (one slot per contributor, summed in a fixed order by the last to arrive).
#include <cuda.h>

#include "tpx_common.cuh"
#include <cuda_fp8.h>

namespace tpx {

constexpr unsigned kTcSpinLimit = 1u << 22;
constexpr int kTcThreads = 192;
constexpr size_t kTcCounterBytes = 64 * 1024;  // arrival counters (one per output tile) + error word at the end

struct TcParams {
  const uint8_t* sfa;   // [ceil(N/128)][KS][512] scale-factor blocks of W
  const uint8_t* sfa2;
  const uint8_t* sfb;   // [TM][KS][512] scale-factor blocks of the activation terms
  const uint16_t* bias;
  const uint16_t* mul_in;
  const uint16_t* res;
  float res_scale;
  uint16_t* y;
  float* partial;       // [grid][2 slots][NW][TOK][128]
  unsigned* counters;
  unsigned* err;
  int M, N, K;
  int KS;               // k steps of 128
  int TN, TM;           // output tiles along features / tokens
  int act;
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}
// Bounded wait: false when the barrier never flipped (the caller reports and leaves).
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity) {
  for (unsigned spins = 0; spins < kTcSpinLimit; spins++)
    if (tc_mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tc_tma_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                       uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "  tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p; }" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
__device__ __forceinline__ void tc_st_x4(uint32_t taddr, uint4 v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void tc_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// K-major operand tile, 128-byte rows, 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// ---------------------------------------------------------------- activation split
// x[M][K] bf16 -> hi, lo [Mpad][Kp] E4M3 and the UE8M0 scale blocks, one thread per (token, 32-wide block).
// Scale-factor block of (token tile tm, k step ks): byte (r%32)*16 + (r/32)*4 + j for row r of the tile and
// the j-th 32-wide block of the step. Padding rows and padding columns get zeros with scale 2^0.
__global__ void split_activations_kernel(const uint16_t* __restrict__ x, int M, int K, int Mpad, int Kp, int TOK,
                                         uint8_t* __restrict__ hi, uint8_t* __restrict__ lo, uint8_t* __restrict__ sfb) {
  const int nb = Kp / 32;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)Mpad * nb) return;
  const int kb = (int)(idx % nb);
  const int tok = (int)(idx / nb);
  float v[32];
  float amax = 0.0f;
  const bool live = tok < M && kb * 32 < K;
  if (live) {
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)tok * K + kb * 32);
#pragma unroll
    for (int q = 0; q < 4; q++) {
      uint4 w = src[q];
      uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        v[q * 8 + 2 * j] = bf16_bits_to_f32((uint16_t)(ww[j] & 0xffff));
        v[q * 8 + 2 * j + 1] = bf16_bits_to_f32((uint16_t)(ww[j] >> 16));
      }
    }
#pragma unroll
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(v[i]));
  } else {
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = 0.0f;
  }
  // block maximum to [128, 256): E4M3 holds up to 448
  int e = 0;
  if (amax > 0.0f && amax < INFINITY) e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127 - 7;
  e = max(-127, min(127, e));
  const float down = __uint_as_float((uint32_t)(127 - e) << 23);
  uint32_t ph[8], pl[8];
#pragma unroll
  for (int i = 0; i < 8; i++) {
    uint32_t h4 = 0, l4 = 0;
#pragma unroll
    for (int j = 0; j < 2; j++) {
      float a = v[4 * i + 2 * j] * down, b = v[4 * i + 2 * j + 1] * down;
      __nv_fp8x2_storage_t hs = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
      __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(hs, __NV_E4M3);
      float ra = a - __half2float(__ushort_as_half(hr.x)), rb = b - __half2float(__ushort_as_half(hr.y));
      __nv_fp8x2_storage_t ls = __nv_cvt_float2_to_fp8x2(make_float2(ra, rb), __NV_SATFINITE, __NV_E4M3);
      h4 |= (uint32_t)hs << (16 * j);
      l4 |= (uint32_t)ls << (16 * j);
    }
    ph[i] = h4;
    pl[i] = l4;
  }
  uint4* dh = reinterpret_cast<uint4*>(hi + (size_t)tok * Kp + kb * 32);
  uint4* dl = reinterpret_cast<uint4*>(lo + (size_t)tok * Kp + kb * 32);
  dh[0] = make_uint4(ph[0], ph[1], ph[2], ph[3]);
  dh[1] = make_uint4(ph[4], ph[5], ph[6], ph[7]);
  dl[0] = make_uint4(pl[0], pl[1], pl[2], pl[3]);
  dl[1] = make_uint4(pl[4], pl[5], pl[6], pl[7]);
  const int tm = tok / TOK, r = tok % TOK, ks = kb / 4, j = kb % 4;
  sfb[((size_t)tm * (Kp / 128) + ks) * 512 + (r % 32) * 16 + (r / 32) * 4 + j] = (uint8_t)(e + 127);
}

// ---------------------------------------------------------------- repack for the tensor-core path
// Interchange tensors of remap_and_quantize_mxfp4 -> row-major packed codes wq[N][K/2] (low nibble = even k)
// and scale-factor blocks sfa[ceil(N/128)][KS][512]. One thread per output byte of wq.
__global__ void repack_mxfp4_tc_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales, int64_t N,
                                       int64_t K, uint8_t* __restrict__ wq, uint8_t* __restrict__ sfa) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t C1 = K / 64;
  if (idx < N * (K / 2)) {
    int64_t n = idx / (K / 2), k = (idx % (K / 2)) * 2;
    // source byte (k1,c1,r,k2) = W[32k1+k2][64c1+2r+{0,1}]: already the (k, k+1) pair
    wq[idx] = codes[(((n / 32) * C1 + k / 64) * 32 + (k % 64) / 2) * 32 + (n % 32)];
  }
  const int64_t KS = (K + 127) / 128;
  const int64_t TN = (N + 127) / 128;
  if (idx < TN * KS * 512) {
    int64_t blk = idx / 512;
    int b = (int)(idx % 512);
    int r = (b / 16) + 32 * ((b % 16) / 4), j = b % 4;
    int64_t n = (blk / KS) * 128 + r, kb = (blk % KS) * 4 + j;
    uint8_t s = 0;
    if (n < N && kb * 32 < K) s = scales[(((n / 32) * C1 + kb / 2) * 2 + (kb & 1)) * 32 + (n % 32)];
    sfa[idx] = s;
  }
}

// ---------------------------------------------------------------- the GEMM kernel
template <int TOK, bool DUAL>
struct TcCfg {
  static constexpr int NW = DUAL ? 2 : 1;
  static constexpr int A_BYTES = 128 * 128;  // shared-memory footprint of an unpacked 128 x 128 fp4 tile
  static constexpr int A_TX = 128 * 64;      // bytes the copy accounts for (the packed data)
  static constexpr int B_BYTES = TOK * 128;
  static constexpr int SF_BYTES = 512;
  static constexpr int RAW = NW * A_BYTES + 2 * B_BYTES + (NW + 1) * SF_BYTES;
  static constexpr int STAGE_BYTES = (RAW + 1023) / 1024 * 1024;
  static constexpr int TX = NW * A_TX + 2 * B_BYTES + (NW + 1) * SF_BYTES;
  static constexpr int STAGES_RAW = (200 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SF_COLS = (NW + 1) * 4;  // tensor-memory columns of one stage's scale factors
  static constexpr int D_COLS = NW * TOK;
  static constexpr int COLS_RAW = D_COLS + STAGES * SF_COLS;
  static constexpr int TMEM_COLS = COLS_RAW <= 32 ? 32 : COLS_RAW <= 64 ? 64 : COLS_RAW <= 128 ? 128 : COLS_RAW <= 256 ? 256 : 512;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;  // + alignment slack
};

__device__ __forceinline__ void tc_finish(const TcParams& p, int tok, int n, float v, float v2, bool dual) {
  size_t o = (size_t)tok * p.N + n;
  if (p.bias) v += bf16_bits_to_f32(p.bias[n]);
  v = apply_act(v, p.act);
  if (dual) v *= v2;
  if (p.mul_in) v *= bf16_bits_to_f32(p.mul_in[o]);
  if (p.res) v += bf16_bits_to_f32(p.res[o]) * p.res_scale;
  p.y[o] = f32_to_bf16_bits(v);
}

template <int TOK, bool DUAL>
__global__ void __launch_bounds__(kTcThreads, 1)
qlinear_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmW2,
                  const __grid_constant__ CUtensorMap tmXh, const __grid_constant__ CUtensorMap tmXl, TcParams p) {
  using C = TcCfg<TOK, DUAL>;
  extern __shared__ unsigned char tc_smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[C::STAGES], bar_empty[C::STAGES], bar_sf[C::STAGES];
  __shared__ __align__(8) unsigned long long bar_acc_full, bar_acc_empty;
  __shared__ uint32_t tmem_holder;
  __shared__ unsigned last_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (tc_smem_u32(tc_smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_gen = tc_smem_raw + (smem_base - tc_smem_u32(tc_smem_raw));

  // this CTA's contiguous range of (tile, k step) units
  const long long U = (long long)p.TN * p.TM * p.KS;
  const long long G = gridDim.x;
  const long long u0 = (long long)blockIdx.x * U / G, u1 = ((long long)blockIdx.x + 1) * U / G;
  const int nunits = (int)(u1 - u0);
  const int tile0 = (int)(u0 / p.KS), ks0 = (int)(u0 % p.KS);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; s++) {
      tc_mbar_init(tc_smem_u32(&bar_full[s]), 1);
      tc_mbar_init(tc_smem_u32(&bar_empty[s]), 1);
      tc_mbar_init(tc_smem_u32(&bar_sf[s]), 4);
    }
    tc_mbar_init(tc_smem_u32(&bar_acc_full), 1);
    tc_mbar_init(tc_smem_u32(&bar_acc_empty), 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(&tmem_holder)),
                 "r"((uint32_t)C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_holder;
  const uint32_t sf_col0 = C::D_COLS;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int tile = tile0, ks = ks0;
      for (int it = 0; it < nunits; it++) {
        const int s = it % C::STAGES;
        if (it >= C::STAGES && !tc_wait(tc_smem_u32(&bar_empty[s]), (uint32_t)((it / C::STAGES - 1) & 1))) {
          atomicExch(p.err, 2u);
          break;
        }
        const int tn = tile / p.TM, tm = tile % p.TM;
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t bar = tc_smem_u32(&bar_full[s]);
        tc_mbar_expect_tx(bar, C::TX);
        tc_tma_2d(st, &tmW, ks * 128, tn * 128, bar);
        if (DUAL) tc_tma_2d(st + C::A_BYTES, &tmW2, ks * 128, tn * 128, bar);
        const uint32_t sb = st + C::NW * C::A_BYTES;
        tc_tma_2d(sb, &tmXh, ks * 128, tm * TOK, bar);
        tc_tma_2d(sb + C::B_BYTES, &tmXl, ks * 128, tm * TOK, bar);
        const uint32_t ssf = sb + 2 * C::B_BYTES;
        tc_bulk_g2s(ssf, p.sfa + ((size_t)tn * p.KS + ks) * 512, 512, bar);
        if (DUAL) tc_bulk_g2s(ssf + 512, p.sfa2 + ((size_t)tn * p.KS + ks) * 512, 512, bar);
        tc_bulk_g2s(ssf + C::NW * 512, p.sfb + ((size_t)tm * p.KS + ks) * 512, 512, bar);
        if (++ks == p.KS) { ks = 0; tile++; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: A = E2M1 (5), B = E4M3 (0), both K-major, N = TOK, UE8M0 scales, M = 128
      const uint32_t idesc0 = (5u << 7) | (0u << 10) | ((uint32_t)(TOK >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
      int ks = ks0;
      uint32_t acc_phase = 0;
      bool fresh = true;  // next MMA starts a new accumulation
      for (int it = 0; it < nunits; it++) {
        const int s = it % C::STAGES;
        const uint32_t ph = (uint32_t)((it / C::STAGES) & 1);
        if (fresh && it > 0) {  // the previous tile must have left tensor memory
          if (!tc_wait(tc_smem_u32(&bar_acc_empty), acc_phase)) { atomicExch(p.err, 3u); break; }
          acc_phase ^= 1;
        }
        if (!tc_wait(tc_smem_u32(&bar_full[s]), ph) || !tc_wait(tc_smem_u32(&bar_sf[s]), ph)) {
          atomicExch(p.err, 4u);
          break;
        }
        tc_fence_after();
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t sf_t = tmem + sf_col0 + (uint32_t)s * C::SF_COLS;
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const uint32_t idesc = idesc0 | ((uint32_t)j << 29) | ((uint32_t)j << 4);
#pragma unroll
          for (int term = 0; term < 2; term++) {
            const uint64_t bdesc = tc_smem_desc(st + C::NW * C::A_BYTES + term * C::B_BYTES) + (uint64_t)(2 * j);
#pragma unroll
            for (int d = 0; d < C::NW; d++) {
              const uint64_t adesc = tc_smem_desc(st + d * C::A_BYTES) + (uint64_t)(2 * j);
              const uint32_t acc = (fresh && j == 0 && term == 0) ? 0u : 1u;
              tc_mma(tmem + d * TOK, adesc, bdesc, idesc, (sf_t + d * 4) | ((uint32_t)j << 30),
                     (sf_t + C::NW * 4) | ((uint32_t)j << 30), acc);
            }
          }
        }
        fresh = false;
        tc_commit(tc_smem_u32(&bar_empty[s]));
        if (++ks == p.KS || it == nunits - 1) {
          tc_commit(tc_smem_u32(&bar_acc_full));
          ks = (ks == p.KS) ? 0 : ks;
          fresh = true;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ scale factors + epilogue (warps 2..5)
    const int sub = warp & 3;  // tensor-memory lanes 32*sub .. 32*sub+31 belong to this warp
    const uint32_t lane_base = ((uint32_t)(sub * 32)) << 16;
    int tile = tile0, ks = ks0;
    int part_first_ks = ks0;
    uint32_t acc_phase = 0;
    bool dead = false;
    for (int it = 0; it < nunits && !dead; it++) {
      const int s = it % C::STAGES;
      const uint32_t ph = (uint32_t)((it / C::STAGES) & 1);
      if (!tc_wait(tc_smem_u32(&bar_full[s]), ph)) {
        if (lane == 0) atomicExch(p.err, 5u);
        dead = true;
        break;
      }
      const unsigned char* ssf = smem_gen + (size_t)s * C::STAGE_BYTES + C::NW * C::A_BYTES + 2 * C::B_BYTES;
      const uint32_t sf_t = tmem + lane_base + sf_col0 + (uint32_t)s * C::SF_COLS;
#pragma unroll
      for (int q = 0; q < C::NW + 1; q++) tc_st_x4(sf_t + q * 4, reinterpret_cast<const uint4*>(ssf + q * 512)[lane]);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(tc_smem_u32(&bar_sf[s]));

      const bool part_end = (ks == p.KS - 1) || (it == nunits - 1);
      if (part_end) {
        if (!tc_wait(tc_smem_u32(&bar_acc_full), acc_phase)) {
          if (lane == 0) atomicExch(p.err, 6u);
          dead = true;
          break;
        }
        acc_phase ^= 1;
        tc_fence_after();
        const int tn = tile / p.TM, tm = tile % p.TM;
        const int row = sub * 32 + lane;
        const int n = tn * 128 + row;
        const int tok0 = tm * TOK;
        const bool whole = (part_first_ks == 0) && (ks == p.KS - 1);
        float* myslot = p.partial + (((size_t)blockIdx.x * 2 + (tile == tile0 ? 0 : 1)) * C::NW) * TOK * 128;
#pragma unroll 1
        for (int c0 = 0; c0 < TOK; c0 += 16) {
          uint32_t r0[16], r1[16];
          tc_ld_x16(tmem + lane_base + c0, r0);
          if (DUAL) tc_ld_x16(tmem + lane_base + TOK + c0, r1);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (whole) {
            if (n < p.N) {
#pragma unroll
              for (int j = 0; j < 16; j++)
                if (tok0 + c0 + j < p.M)
                  tc_finish(p, tok0 + c0 + j, n, __uint_as_float(r0[j]), DUAL ? __uint_as_float(r1[j]) : 0.0f, DUAL);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; j++) {
              __stcg(myslot + (size_t)(c0 + j) * 128 + row, __uint_as_float(r0[j]));
              if (DUAL) __stcg(myslot + (size_t)(TOK + c0 + j) * 128 + row, __uint_as_float(r1[j]));
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) tc_mbar_arrive(tc_smem_u32(&bar_acc_empty));  // tensor memory may be overwritten
        if (!whole) {
          // hand the partial tile in; the last contributor adds all of them in CTA order
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const long long ta = (long long)tile * p.KS, tb = ta + p.KS - 1;
          const int cfirst = (int)(((ta + 1) * G - 1) / U), clast = (int)(((tb + 1) * G - 1) / U);
          if (threadIdx.x == 64) {
            unsigned prev = atomicAdd(p.counters + tile, 1u);
            last_flag = (prev == (unsigned)(clast - cfirst)) ? 1u : 0u;
            if (last_flag) p.counters[tile] = 0;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (last_flag) {
            __threadfence();
            if (n < p.N) {
#pragma unroll 1
              for (int j = 0; j < TOK; j++) {
                if (tok0 + j >= p.M) break;
                float v = 0.0f, v2 = 0.0f;
                for (int c = cfirst; c <= clast; c++) {
                  const int ctile0 = (int)(((long long)c * U / G) / p.KS);
                  const float* slot = p.partial + (((size_t)c * 2 + (tile == ctile0 ? 0 : 1)) * C::NW) * TOK * 128;
                  v += __ldcg(slot + (size_t)j * 128 + row);
                  if (DUAL) v2 += __ldcg(slot + (size_t)(TOK + j) * 128 + row);
                }
                tc_finish(p, tok0 + j, n, v, v2, DUAL);
              }
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");  // last_flag is reused by the next tile
        }
      }
      if (++ks == p.KS) {
        ks = 0;
        tile++;
        part_first_ks = 0;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)C::TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &ptr, 12000, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D row-major tensor [rows][cols elements], box = 128 elements x box_rows, 128-byte swizzle.
static int make_map(CUtensorMap* m, CUtensorMapDataType dt, const void* base, uint64_t cols, uint64_t rows,
                    uint64_t row_stride_bytes, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  TPX_REQUIRE(fn, TPX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {row_stride_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, dt, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TPX_REQUIRE(r == CUDA_SUCCESS, TPX_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (cols=%llu rows=%llu stride=%llu)", (int)r,
              (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)row_stride_bytes);
  return TPX_OK;
}

struct TcPlan {
  int tok;      // tokens per tile
  int TN, TM, KS, Kp, Mpad, grid;
  size_t off_hi, off_lo, off_sfb, off_partial, total;
};

static TcPlan tc_plan(int64_t M, int64_t N, int64_t K, bool dual) {
  TcPlan pl;
  pl.tok = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  pl.KS = (int)((K + 127) / 128);
  pl.Kp = pl.KS * 128;
  pl.TN = (int)((N + 127) / 128);
  pl.TM = (int)((M + pl.tok - 1) / pl.tok);
  pl.Mpad = pl.TM * pl.tok;
  long long U = (long long)pl.TN * pl.TM * pl.KS;
  int sms = sm_count();
  pl.grid = (int)(U < sms ? U : sms);
  size_t o = kTcCounterBytes;
  auto bump = [&](size_t bytes) { size_t r = o; o += (bytes + 255) & ~(size_t)255; return r; };
  pl.off_hi = bump((size_t)pl.Mpad * pl.Kp);
  pl.off_lo = bump((size_t)pl.Mpad * pl.Kp);
  pl.off_sfb = bump((size_t)pl.TM * pl.KS * 512);
  pl.off_partial = bump((size_t)pl.grid * 2 * (dual ? 2 : 1) * pl.tok * 128 * sizeof(float));
  pl.total = o;
  return pl;
}

template <int TOK, bool DUAL>
static int tc_launch(const CUtensorMap& w, const CUtensorMap& w2, const CUtensorMap& xh, const CUtensorMap& xl,
                     const TcParams& p, int grid, cudaStream_t st) {
  using C = TcCfg<TOK, DUAL>;
  static bool opted[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || !opted[dev]) {
    TPX_CUDA_OK(cudaFuncSetAttribute(qlinear_tc_kernel<TOK, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    if (dev >= 0 && dev < 16) opted[dev] = true;
  }
  qlinear_tc_kernel<TOK, DUAL><<<grid, kTcThreads, C::SMEM, st>>>(w, w2, xh, xl, p);
  TPX_LAUNCH_OK();
  return TPX_OK;
}

}  // namespace tpx

using namespace tpx;

extern "C" int tpx_tc_packed_bytes(int64_t N, int64_t K, size_t* wq_bytes, size_t* sfa_bytes) {
  TPX_REQUIRE(N > 0 && K > 0 && N % 32 == 0 && K % 64 == 0, TPX_ERR_ARG, "tc_packed_bytes: needs N %% 32 == 0 and K %% 64 == 0");
  if (wq_bytes) *wq_bytes = (size_t)N * (K / 2);
  if (sfa_bytes) *sfa_bytes = (size_t)((N + 127) / 128) * ((K + 127) / 128) * 512;
  return TPX_OK;
}

extern "C" int tpx_repack_mxfp4_tc(const uint8_t* codes, const uint8_t* scales, int64_t N, int64_t K, uint8_t* wq,
                                   uint8_t* sfa, void* stream) {
  TPX_REQUIRE(codes && scales && wq && sfa, TPX_ERR_ARG, "repack_mxfp4_tc: null pointer");
  TPX_REQUIRE(N % 32 == 0 && K % 64 == 0, TPX_ERR_ARG, "repack_mxfp4_tc: needs N %% 32 == 0 and K %% 64 == 0");
  int64_t a = N * (K / 2), b = ((N + 127) / 128) * ((K + 127) / 128) * 512;
  int64_t total = a > b ? a : b;
  repack_mxfp4_tc_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(codes, scales, N, K, wq, sfa);
  TPX_LAUNCH_OK();
  return TPX_OK;
}

extern "C" size_t tpx_qlinear_mxfp4_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int dual) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return tc_plan(M, N, K, dual != 0).total;
}

extern "C" int tpx_qlinear_mxfp4_tc(const uint8_t* wq, const uint8_t* sfa, const uint8_t* wq2, const uint8_t* sfa2,
                                    const uint16_t* x, int64_t M, int64_t N, int64_t K, const uint16_t* bias, int act,
                                    const uint16_t* mul_in, const uint16_t* res, float res_scale, uint16_t* y,
                                    void* scratch, size_t scratch_bytes, void* stream) {
  TPX_REQUIRE(M >= 0 && N > 0 && K > 0, TPX_ERR_ARG, "qlinear_mxfp4_tc: bad shape");
  if (M == 0) return TPX_OK;
  TPX_REQUIRE(wq && sfa && x && y, TPX_ERR_ARG, "qlinear_mxfp4_tc: null pointer");
  TPX_REQUIRE((wq2 == nullptr) == (sfa2 == nullptr), TPX_ERR_ARG, "qlinear_mxfp4_tc: second weight needs codes and scales");
  TPX_REQUIRE(!(wq2 && mul_in), TPX_ERR_ARG, "qlinear_mxfp4_tc: gate/up pair and mul_in are exclusive");
  TPX_REQUIRE(N % 32 == 0 && K % 64 == 0, TPX_ERR_ARG, "qlinear_mxfp4_tc: needs N %% 32 == 0 and K %% 64 == 0");
  TPX_REQUIRE(act >= TPX_ACT_NONE && act <= TPX_ACT_RELU, TPX_ERR_ARG, "qlinear_mxfp4_tc: unknown activation %d", act);
  TPX_REQUIRE(((uintptr_t)wq & 31) == 0 && ((uintptr_t)wq2 & 31) == 0 && ((uintptr_t)sfa & 15) == 0 && ((uintptr_t)sfa2 & 15) == 0 &&
                  ((uintptr_t)x & 15) == 0 && ((uintptr_t)scratch & 255) == 0,
              TPX_ERR_ARG, "qlinear_mxfp4_tc: misaligned pointer");
  const bool dual = wq2 != nullptr;
  TcPlan pl = tc_plan(M, N, K, dual);
  TPX_REQUIRE((size_t)pl.TN * pl.TM * sizeof(unsigned) <= kTcCounterBytes - 16, TPX_ERR_UNSUPPORTED,
              "qlinear_mxfp4_tc: %d x %d output tiles exceed the counter region; split the batch", pl.TN, pl.TM);
  TPX_REQUIRE(scratch && scratch_bytes >= pl.total, TPX_ERR_SCRATCH, "qlinear_mxfp4_tc: scratch of %zu bytes needed, %zu given",
              pl.total, scratch_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  unsigned char* sc = reinterpret_cast<unsigned char*>(scratch);
  uint8_t *hi = sc + pl.off_hi, *lo = sc + pl.off_lo, *sfb = sc + pl.off_sfb;
  {
    long long threads = (long long)pl.Mpad * (pl.Kp / 32);
    split_activations_kernel<<<(unsigned)((threads + 127) / 128), 128, 0, st>>>(x, (int)M, (int)K, pl.Mpad, pl.Kp, pl.tok, hi, lo, sfb);
    TPX_LAUNCH_OK();
  }
  CUtensorMap mw, mw2, mxh, mxl;
  int rc = make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, wq, (uint64_t)K, (uint64_t)N, (uint64_t)K / 2, 128);
  if (rc) return rc;
  rc = make_map(&mw2, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, dual ? wq2 : wq, (uint64_t)K, (uint64_t)N, (uint64_t)K / 2, 128);
  if (rc) return rc;
  rc = make_map(&mxh, CU_TENSOR_MAP_DATA_TYPE_UINT8, hi, (uint64_t)pl.Kp, (uint64_t)pl.Mpad, (uint64_t)pl.Kp, (uint32_t)pl.tok);
  if (rc) return rc;
  rc = make_map(&mxl, CU_TENSOR_MAP_DATA_TYPE_UINT8, lo, (uint64_t)pl.Kp, (uint64_t)pl.Mpad, (uint64_t)pl.Kp, (uint32_t)pl.tok);
  if (rc) return rc;
  TcParams p;
  p.sfa = sfa; p.sfa2 = sfa2; p.sfb = sfb; p.bias = bias; p.mul_in = mul_in; p.res = res; p.res_scale = res_scale; p.y = y;
  p.partial = reinterpret_cast<float*>(sc + pl.off_partial);
  p.counters = reinterpret_cast<unsigned*>(sc);
  p.err = reinterpret_cast<unsigned*>(sc + kTcCounterBytes - 4);
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.KS = pl.KS; p.TN = pl.TN; p.TM = pl.TM; p.act = act;
  switch (pl.tok) {
    case 16: return dual ? tc_launch<16, true>(mw, mw2, mxh, mxl, p, pl.grid, st) : tc_launch<16, false>(mw, mw2, mxh, mxl, p, pl.grid, st);
    case 32: return dual ? tc_launch<32, true>(mw, mw2, mxh, mxl, p, pl.grid, st) : tc_launch<32, false>(mw, mw2, mxh, mxl, p, pl.grid, st);
    case 64: return dual ? tc_launch<64, true>(mw, mw2, mxh, mxl, p, pl.grid, st) : tc_launch<64, false>(mw, mw2, mxh, mxl, p, pl.grid, st);
    default: return dual ? tc_launch<128, true>(mw, mw2, mxh, mxl, p, pl.grid, st) : tc_launch<128, false>(mw, mw2, mxh, mxl, p, pl.grid, st);
  }
}
