// MXFP4 weight-only linear for many tokens on CTA pairs: tcgen05.mma.cta_group::2 (M = 256 over two SMs).
//
// Replaces the same reference functions as tpx_qlinear_tcp.cu (fc_plain / fc_gate_up / fc_add of
// src/csrc/llm/fused_llm_infer.cpp on MXFP4 weights, many tokens). A cluster of two CTAs computes two 128-feature weight
// tiles against one 128-token tile with ONE instruction stream: the MMA has M = 256 (rows 0-127 from the first CTA's
// shared memory into the first CTA's tensor memory, rows 128-255 likewise in the second) and N = 256 (the hi E4M3 terms
// of the 128 tokens, then the lo terms); each CTA holds only HALF of the B operand (the first CTA the hi rows, the
// second the lo rows) and the hardware reads both halves for both CTAs. Per CTA and k step that is 16 KB of unpacked
// weights + 16 KB of activation terms instead of 16 + 32 KB, so three stages of two k steps fit where the one-CTA
// kernels hold two, the N = 256 MMA runs at the full rate (128 cycles against 2 x 107 for two N = 128 MMAs), and a third
// less data crosses from L2 into shared memory.
//   * Copies: every CTA loads its own operands with cp.async.bulk.tensor ... .cta_group::2 (no multicast), all
//     completing on the FIRST CTA's mbarrier, which expects the bytes of both; scale factors travel as small tensor
//     copies for the same reason. Both CTAs load both activation scale blocks (each SM's tensor core needs the scales
//     of all 256 columns), each its own weight scale block; tcgen05.cp.cta_group::2 moves them into tensor memory.
//   * One thread of the first CTA issues every MMA; tcgen05.commit ... .multicast::cluster frees a stage in both CTAs
//     and announces a finished accumulator to both.
//   * One 256-column accumulator per CTA (hi and lo columns, added by the epilogue). The sixteen epilogue warps of
//     each CTA first pull their part of the accumulator into registers and hand tensor memory back (an arrival on the
//     first CTA's barrier, remote for the second CTA), then run bias / activation / gate / residual and the stores while
//     the next tile's MMAs proceed. A gate/up pair is two consecutive accumulations; the gate values wait in registers.
// Layouts of the packed weights, scale blocks and activation terms are those of tpx_qlinear_tc.cu (token tile 128).
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "tpx_tc_ptx.cuh"

namespace tpx {

// ROWS: one activation scale per token (rowscale_split_kernel): no activation scale blocks in the stages.
template <int UKS, bool ROWS>
struct Tcp2Cfg {
  static constexpr int A_BYTES = 128 * 128;             // an unpacked 128 x 128 fp4 tile in shared memory
  static constexpr int A_TX = 128 * 64;                 // what its copy accounts for (packed bytes)
  static constexpr int B_BYTES = 128 * 128;             // this CTA's half of B for one k step: 128 rows of one term
  static constexpr int SF_BYTES = ROWS ? 512 : 512 + 1024;  // per k step: own weight block (+ both activation blocks)
  static constexpr int RAW = UKS * (A_BYTES + B_BYTES + SF_BYTES);
  static constexpr int STAGE_BYTES = (RAW + 1023) / 1024 * 1024;
  static constexpr int TX_CTA = UKS * (A_TX + B_BYTES + SF_BYTES);  // bytes one CTA's copies deliver per stage
  static constexpr int BUDGET = 227 * 1024 - 2048;
  static constexpr int STAGES_RAW = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SF_COLS = UKS * (ROWS ? 4 : 12);  // per k step 4 (weights) + 8 (activations) columns
  static constexpr int D_COLS = 256;
  static constexpr int CONST_COLS = ROWS ? 8 : 0;       // activation scale factors 1.0 for all 256 columns, written once
  static constexpr int TMEM_COLS = 512;
  static constexpr int EPI_SPLIT = 4;                   // warps per 32-lane quarter of tensor memory, 32 tokens each
  static constexpr int THREADS = 96 + 128 * EPI_SPLIT;  // weight producer, MMA issuer, activation producer, epilogue warps
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;
  static_assert(STAGES >= 2, "at least two stages");
  static_assert(D_COLS + CONST_COLS + STAGES * SF_COLS <= 512, "tensor memory");
};

__device__ __forceinline__ void t2_tma_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar)
      : "memory");
}
__device__ __forceinline__ void t2_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                       uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "  tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p; }" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
__device__ __forceinline__ void t2_cp_sf(uint32_t taddr, uint64_t sdesc) {  // in both CTAs, each from its own shared memory
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void t2_commit_both(uint32_t bar) {  // arrives on the barrier at this offset in both CTAs
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ void t2_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ bool t2_wait_cluster(uint32_t bar, uint32_t parity) {  // arrivals come from both CTAs
  for (unsigned spins = 0; spins < kTcSpinLimit; spins++) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    if (ok) return true;
  }
  return false;
}

// Activation split with ONE power-of-two scale per token instead of one per 32 values: x / 2^e as a hi and a lo E4M3
// term, 2^e in `tok_scale` for the epilogue. The activation scale factors of the block-scaled MMA are then the constant
// 1.0, written to tensor memory once per kernel instead of copied per k step (two of the three scale-factor copies of a
// k step, each of which holds the tensor pipe for about 100 cycles). The row maximum lands in [128, 256) of E4M3's
// range (largest finite value 448, smallest subnormal 2^-9): values down to 2^-17 of the row maximum keep a non-zero hi
// term, so the two terms carry 8 significant bits wherever the value matters to a dot product with the row.
// One CTA per token row, the row in registers (VECS x 256 threads x 8 elements); optional RMSNorm first
// (llama_rms_norm, src/csrc/llm/fused_llm_infer.cpp:336-363, rounded to bf16 as the reference stores it).
// Term layout as split_activations_kernel with 128-token tiles: [tm][k step][hi 128 rows | lo 128 rows][128 B].
// Rows of up to 4096 elements run with 128 threads (more CTAs, hence more loads in flight, per SM: about 4 us less for
// 4096 x 4096), longer ones with 256.
constexpr int kRsThreads = 256;
template <int VECS, int THREADS>
__global__ void __launch_bounds__(THREADS) rowscale_split_kernel(const uint16_t* __restrict__ x, const void* __restrict__ gamma, int gamma_f32,
                                                                    float eps, int M, int K, int KS, uint8_t* __restrict__ terms,
                                                                    float* __restrict__ tok_scale) {
  __shared__ float red[THREADS / 32];
  pdl_trigger();
  pdl_wait();
  const int tok = blockIdx.x;
  const bool live_row = tok < M;
  const int nv = K / 8, nvp = KS * 16;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)tok * K);
  float f[VECS][8];
  float ss = 0.0f;
#pragma unroll
  for (int q = 0; q < VECS; q++) {
    const int i = threadIdx.x + q * THREADS;
    const bool have = live_row && i < nv;
    const uint4 v = have ? xr[i] : make_uint4(0, 0, 0, 0);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      f[q][2 * j] = bf16_bits_to_f32((uint16_t)(w[j] & 0xffff));
      f[q][2 * j + 1] = bf16_bits_to_f32((uint16_t)(w[j] >> 16));
      ss += f[q][2 * j] * f[q][2 * j] + f[q][2 * j + 1] * f[q][2 * j + 1];
    }
  }
  if (gamma) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; w++) tot += red[w];
    __syncthreads();
    const float inv = rsqrtf(tot / (float)K + eps);
#pragma unroll
    for (int q = 0; q < VECS; q++) {
      const int i = threadIdx.x + q * THREADS;
      if (!(live_row && i < nv)) continue;
      float g[8];
      if (gamma_f32) {
        const float4 g0 = reinterpret_cast<const float4*>(gamma)[2 * i], g1 = reinterpret_cast<const float4*>(gamma)[2 * i + 1];
        g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
      } else {
        const uint4 gv = reinterpret_cast<const uint4*>(gamma)[i];
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
          g[2 * j] = bf16_bits_to_f32((uint16_t)(gw[j] & 0xffff));
          g[2 * j + 1] = bf16_bits_to_f32((uint16_t)(gw[j] >> 16));
        }
      }
#pragma unroll
      for (int j = 0; j < 8; j++) f[q][j] = bf16_bits_to_f32(f32_to_bf16_bits(f[q][j] * inv * g[j]));
    }
  }
  float amax = 0.0f;
#pragma unroll
  for (int q = 0; q < VECS; q++) {
#pragma unroll
    for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(f[q][j]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
#pragma unroll
  for (int w = 0; w < THREADS / 32; w++) amax = fmaxf(amax, red[w]);
  int e = 0;
  if (amax > 0.0f && amax < INFINITY) e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127 - 7;
  e = max(-126, min(127, e));
  const float down = __uint_as_float((uint32_t)(127 - e) << 23);
  if (threadIdx.x == 0) tok_scale[tok] = __uint_as_float((uint32_t)(127 + e) << 23);
  const int tm = tok / 128, r = tok % 128;
#pragma unroll
  for (int q = 0; q < VECS; q++) {
    const int i = threadIdx.x + q * THREADS;  // vector index: 16 vectors per k step of 128
    if (i >= nvp) continue;
    uint32_t ph[2], pl[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; h2++) {
      uint32_t h4 = 0, l4 = 0;
#pragma unroll
      for (int j = 0; j < 2; j++) {
        const float a = f[q][4 * h2 + 2 * j] * down, b = f[q][4 * h2 + 2 * j + 1] * down;
        __nv_fp8x2_storage_t hs = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
        __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(hs, __NV_E4M3);
        const float ra = a - __half2float(__ushort_as_half(hr.x)), rb = b - __half2float(__ushort_as_half(hr.y));
        __nv_fp8x2_storage_t ls = __nv_cvt_float2_to_fp8x2(make_float2(ra, rb), __NV_SATFINITE, __NV_E4M3);
        h4 |= (uint32_t)hs << (16 * j);
        l4 |= (uint32_t)ls << (16 * j);
      }
      ph[h2] = h4;
      pl[h2] = l4;
    }
    const int ks = i >> 4, c = i & 15;  // k step and 8-byte column inside its 128-byte row
    const size_t step = (size_t)tm * KS + ks;
    *reinterpret_cast<uint2*>(terms + (step * 256 + r) * 128 + c * 8) = make_uint2(ph[0], ph[1]);
    *reinterpret_cast<uint2*>(terms + (step * 256 + 128 + r) * 128 + c * 8) = make_uint2(pl[0], pl[1]);
  }
}

// UKS k steps of 128 per pipeline stage; DUAL: gate/up pair. Launched as clusters of two CTAs; p.KS counts stages per
// accumulation; pairs of feature tiles x token tiles are cut evenly between the clusters.
template <int UKS, bool DUAL, bool ROWS>
__global__ void __launch_bounds__(Tcp2Cfg<UKS, ROWS>::THREADS, 1)
qlinear_tcp2_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                    const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB, TcParams p) {
  using C = Tcp2Cfg<UKS, ROWS>;
  constexpr int NWT = DUAL ? 2 : 1;  // accumulations per output tile
  extern __shared__ unsigned char tcp2_smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[C::STAGES], bar_empty[C::STAGES];
  __shared__ __align__(8) unsigned long long bar_acc_full, bar_acc_empty;
  __shared__ uint32_t tmem_holder;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (tc_smem_u32(tcp2_smem_raw) + 1023u) & ~1023u;
  const int crank = (int)tc_cluster_rank();  // 0: issues the MMAs and owns the barriers the copies complete on
  const long long TNP = (p.TN + 1) / 2;      // pairs of feature tiles
  const long long T = TNP * p.TM, G = gridDim.x / 2;
  const long long cid = blockIdx.x / 2;
  const int t0 = (int)(cid * T / G), t1 = (int)((cid + 1) * T / G);
  const int ntiles = t1 - t0;
  const int KU = p.KS;
  const int KSS = KU * UKS;
  const int nunits = ntiles * NWT * KU;

  if (threadIdx.x == 0) tc_stamp(p, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; s++) {
      tc_mbar_init(tc_smem_u32(&bar_full[s]), 1);
      tc_mbar_init(tc_smem_u32(&bar_empty[s]), 1);
    }
    tc_mbar_init(tc_smem_u32(&bar_acc_full), 1);
    tc_mbar_init(tc_smem_u32(&bar_acc_empty), 2 * 4 * C::EPI_SPLIT);  // the epilogue warps of both CTAs
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // the same warp of both CTAs: the allocation covers both SMs at the same address
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(&tmem_holder)),
                 "r"((uint32_t)C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_holder;
  if (ROWS && warp >= 3 && warp < 7) {  // one warp per 32-lane quarter: UE8M0 127 = 1.0 in every byte of the 8 columns
    const uint32_t t = tmem + (((uint32_t)((warp & 3) * 32)) << 16) + C::D_COLS;
    const uint4 ones = make_uint4(0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
    tc_st_x4(t, ones);
    tc_st_x4(t + 4, ones);
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_cluster_sync();  // the partner's barriers and tensor memory exist before anything is sent to them
  tc_fence_after();
  const uint32_t sf_col0 = C::D_COLS + C::CONST_COLS;
  if (threadIdx.x == 0) tc_stamp(p, 1);
  pdl_trigger();

  auto where = [&](int it, int& tn, int& tm, int& d, int& ku) {
    const int a = it / KU;
    ku = it - a * KU;
    const int tile = t0 + a / NWT;
    d = a % NWT;
    const int tnp = tile / p.TM;
    tm = tile - tnp * p.TM;
    tn = tnp * 2 + crank;
  };
  if (warp == 0) {
    // ------------------------------------------------------------ weight producer (one thread in each CTA)
    // Issuing a stage's copies takes one thread about as long as the stage's MMAs run, so the weights and the
    // activation terms have a producer thread each.
    if (lane == 0) {
      for (int it = 0; it < nunits; it++) {
        const int s = it % C::STAGES;
        int tn, tm, d, ku;
        where(it, tn, tm, d, ku);
        if (it >= C::STAGES) {
          if (!tc_wait(tc_smem_u32(&bar_empty[s]), (uint32_t)((it / C::STAGES - 1) & 1))) {
            atomicExch(p.err, 2u);
            break;
          }
        }
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t lbar = tc_mapa(tc_smem_u32(&bar_full[s]), 0u);  // the first CTA's barrier
        if (crank == 0) tc_mbar_expect_tx(tc_smem_u32(&bar_full[s]), 2u * (C::TX_CTA + (p.wfmt ? UKS * (128 * 128 - C::A_TX) : 0)));
        const uint32_t ssf = st + UKS * (C::A_BYTES + C::B_BYTES);
        const int ks0 = tn * KSS + ku * UKS;
        if (DUAL) {
#pragma unroll
          for (int kk = 0; kk < UKS; kk++) {
            const int wt = (ks0 + kk) * 2 + d;
            t2_tma_2d(st + kk * C::A_BYTES, &tmW, 0, wt * 128, lbar);
            t2_tma_2d(ssf + kk * 512, &tmSFA, 0, wt, lbar);
          }
        } else {
          t2_tma_2d(st, &tmW, 0, ks0 * 128, lbar);
          t2_tma_2d(ssf, &tmSFA, 0, ks0, lbar);
        }
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------ activation producer (one thread in each CTA)
    if (lane == 0) {
      pdl_wait();  // the activation terms belong to the split kernel until it has completed
      for (int it = 0; it < nunits; it++) {
        const int s = it % C::STAGES;
        int tn, tm, d, ku;
        where(it, tn, tm, d, ku);
        if (it >= C::STAGES) {
          if (!tc_wait(tc_smem_u32(&bar_empty[s]), (uint32_t)((it / C::STAGES - 1) & 1))) {
            atomicExch(p.err, 5u);
            break;
          }
        }
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t lbar = tc_mapa(tc_smem_u32(&bar_full[s]), 0u);
        const uint32_t sb = st + UKS * C::A_BYTES;
        const int xrow = (tm * KU + ku) * (UKS * 256) + crank * 128;
#pragma unroll
        for (int kk = 0; kk < UKS; kk++) t2_tma_2d(sb + kk * C::B_BYTES, &tmX, 0, xrow + kk * 256, lbar);
        if (!ROWS) t2_tma_2d(st + UKS * (C::A_BYTES + C::B_BYTES) + UKS * 512, &tmSFB, 0, (tm * KU + ku) * UKS * 2, lbar);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (first CTA only)
    if (lane == 0 && crank == 0) {
      // instruction descriptor: A = E2M1 (5), B = E4M3 (0), both K-major, N = 256, UE8M0 scales, M = 256 over the pair
      const uint32_t idesc0 = ((p.wfmt == 0 ? 5u : p.wfmt == 1 ? 0u : 1u) << 7) | (0u << 10) | ((uint32_t)(256 >> 3) << 17) | (1u << 23) | ((256u >> 4) << 24);
      for (int it = 0; it < nunits; it++) {
        const int s = it % C::STAGES;
        const uint32_t ph = (uint32_t)((it / C::STAGES) & 1);
        const int a = it / KU, ku = it - a * KU;
        if (ku == 0 && a >= 1) {  // both CTAs' epilogue warps have read the previous accumulator
          if (!t2_wait_cluster(tc_smem_u32(&bar_acc_empty), (uint32_t)((a - 1) & 1))) { atomicExch(p.err, 3u); break; }
        }
        if (!tc_wait(tc_smem_u32(&bar_full[s]), ph)) {
          atomicExch(p.err, 4u);
          break;
        }
        if (it == 0) tc_stamp(p, 2);
        if (it == nunits - 1) tc_stamp(p, 3);
        tc_fence_after();
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t sb = st + UKS * C::A_BYTES;
        const uint32_t ssf = st + UKS * (C::A_BYTES + C::B_BYTES);
        const uint32_t sf_t = tmem + sf_col0 + (uint32_t)s * C::SF_COLS;
        if (TPX_DBG(p) & 1) {
          // timing experiment without MMAs: release the stage and the accumulator in both CTAs by hand
          tc_mbar_arrive(tc_smem_u32(&bar_empty[s]));
          t2_arrive_cluster(tc_mapa(tc_smem_u32(&bar_empty[s]), 1u));
          if (ku == KU - 1) {
            tc_mbar_arrive(tc_smem_u32(&bar_acc_full));
            t2_arrive_cluster(tc_mapa(tc_smem_u32(&bar_acc_full), 1u));
          }
        } else {
#pragma unroll
          for (int kk = 0; kk < UKS; kk++) {
            t2_cp_sf(sf_t + kk * 4, tc_sf_desc(ssf + kk * 512));
            if (!ROWS) {
              t2_cp_sf(sf_t + UKS * 4 + kk * 8, tc_sf_desc(ssf + UKS * 512 + kk * 1024));
              t2_cp_sf(sf_t + UKS * 4 + kk * 8 + 4, tc_sf_desc(ssf + UKS * 512 + kk * 1024 + 512));
            }
          }
#pragma unroll
          for (int kk = 0; kk < UKS; kk++) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const uint32_t idesc = idesc0 | ((uint32_t)j << 29) | ((uint32_t)j << 4);
              const uint64_t adesc = tc_smem_desc(st + kk * C::A_BYTES) + (uint64_t)(2 * j);
              const uint64_t bdesc = tc_smem_desc(sb + kk * C::B_BYTES) + (uint64_t)(2 * j);
              const uint32_t acc = (ku == 0 && kk == 0 && j == 0) ? 0u : 1u;
              t2_mma(tmem, adesc, bdesc, idesc, (sf_t + kk * 4) | ((uint32_t)j << 30),
                     (ROWS ? tmem + C::D_COLS : sf_t + UKS * 4 + kk * 8) | ((uint32_t)j << 30), acc);
            }
          }
          t2_commit_both(tc_smem_u32(&bar_empty[s]));
          if (ku == KU - 1) t2_commit_both(tc_smem_u32(&bar_acc_full));
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 3 .. 18 of both CTAs)
    const int sub = warp & 3;  // tensor-memory lanes 32*sub .. 32*sub+31 belong to this warp
    const uint32_t lane_base = ((uint32_t)(sub * 32)) << 16;
    const int cpart = (warp - 3) >> 2;  // tokens cpart*32 .. cpart*32+31 of the tile
    const int row = sub * 32 + lane;
    const uint32_t lbar_empty = tc_mapa(tc_smem_u32(&bar_acc_empty), 0u);
    // the accumulator's 32 tokens of this thread into registers (hi + lo columns), then tensor memory is handed back
    auto pull = [&](float (&r)[32]) {
#pragma unroll
      for (int c = 0; c < 2; c++) {
        uint32_t h[16], l[16];
        tc_ld_x16(tmem + lane_base + (uint32_t)(cpart * 32 + c * 16), h);
        tc_ld_x16(tmem + lane_base + 128u + (uint32_t)(cpart * 32 + c * 16), l);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; j++) r[c * 16 + j] = __uint_as_float(h[j]) + __uint_as_float(l[j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) t2_arrive_cluster(lbar_empty);
    };
    pdl_wait();  // residual and gate inputs belong to earlier grids
    uint32_t acc_n = 0;  // accumulators seen so far
    for (int ti = 0; ti < ntiles; ti++) {
      const int tile = t0 + ti;
      const int tnp = tile / p.TM, tm = tile - tnp * p.TM;
      const int n = (tnp * 2 + crank) * 128 + row;
      const int tokb = tm * 128 + cpart * 32;
      const bool live = n < p.N;
      uint32_t resp[2][8], mulp[2][8];
#pragma unroll
      for (int c = 0; c < 2; c++) {
#pragma unroll
        for (int j = 0; j < 8; j++) resp[c][j] = mulp[c][j] = 0u;
      }
      if (live) {  // in flight while the tile's MMAs run
#pragma unroll
        for (int c = 0; c < 2; c++) {
          if (p.res) tc_preload16(p.res, p.M, p.N, tokb + c * 16, n, resp[c]);
          if (p.mul_in) tc_preload16(p.mul_in, p.M, p.N, tokb + c * 16, n, mulp[c]);
        }
      }
      float g[32], u[32];
      if (!tc_wait(tc_smem_u32(&bar_acc_full), acc_n & 1u)) {
        if (lane == 0) atomicExch(p.err, 6u);
        break;
      }
      acc_n++;
      tc_fence_after();
      pull(g);
      if (DUAL) {
        if (!tc_wait(tc_smem_u32(&bar_acc_full), acc_n & 1u)) {
          if (lane == 0) atomicExch(p.err, 7u);
          break;
        }
        acc_n++;
        tc_fence_after();
        if (threadIdx.x == 96 && ti == ntiles - 1) tc_stamp(p, 5);
        pull(u);
      } else {
        if (threadIdx.x == 96 && ti == ntiles - 1) tc_stamp(p, 5);
      }
#pragma unroll
      for (int c = 0; c < 2; c++) {
        float x[16], uf[16];
#pragma unroll
        for (int j = 0; j < 16; j++) {
          x[j] = g[c * 16 + j];
          uf[j] = DUAL ? u[c * 16 + j] : 0.0f;
        }
        if (live && tokb + c * 16 < p.M) tc_finish16_pre<DUAL>(p, tokb + c * 16, n, x, uf, resp[c], mulp[c], ROWS ? p.partial : nullptr);
      }
    }
  }
  if (threadIdx.x == 96) tc_stamp(p, 6);
  tc_fence_before();
  __syncthreads();
  tc_cluster_sync();  // nobody leaves, and tensor memory is not freed, while the partner may still use this CTA's memory
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)C::TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------- host side
struct Tcp2Plan {
  int TN, TM, KS, Mpad, uks, rows;  // rows: one activation scale per token (rows of up to 16384 elements)
  size_t off_terms, off_sfb, off_tscale, total;
};

static Tcp2Plan tcp2_plan(int64_t M, int64_t N, int64_t K, bool pair) {
  Tcp2Plan pl;
  pl.uks = knobs().tc_p_uks == 1 ? 1 : 2;
  pl.KS = tc_padded_ks(K, pair);
  pl.TN = (int)((N + 127) / 128);
  pl.TM = (int)((M + 127) / 128);
  pl.Mpad = pl.TM * 128;
  size_t o = kTcCounterBytes;
  auto bump = [&](size_t bytes) { size_t r = o; o += (bytes + 1023) & ~(size_t)1023; return r; };
  pl.off_terms = bump((size_t)pl.Mpad * pl.KS * 128 * 2);
  pl.off_sfb = bump((size_t)pl.TM * pl.KS * 2 * 512);
  pl.off_tscale = bump((size_t)pl.Mpad * sizeof(float));
  pl.rows = (knobs().tc_p_rows != 0 && pl.KS * 16 <= kRsThreads * 8) ? 1 : 0;
  pl.total = o;
  return pl;
}

// Served: more than 64 tokens when at least a quarter of the SMs get a tile, or K is short. Measured against the
// general kernel and the one-CTA many-token kernel over the linear shapes of a Llama-3-8B layer from 128 to 32768
// tokens it is the fastest everywhere except few tiles with a long K (4096 x 14336 at 128 / 256 tokens: 56 / 59 us
// against 40 / 54 us for the cluster split of K in the general kernel). TPX_TC_P2=0 never, TPX_TC_P2=1 for every M > 64.
bool tcp2_serves(int64_t M, int64_t N, int64_t K, bool pair) {
  (void)pair;
  const int k = knobs().tc_p2;
  if (k == 0 || M <= 64) return false;
  if (k > 0) return true;
  const long long TP = ((N + 255) / 256) * ((M + 127) / 128);
  return TP * 4 >= sm_count() || K <= 4096;
}

size_t tcp2_scratch_bytes(int64_t M, int64_t N, int64_t K, bool pair) { return tcp2_plan(M, N, K, pair).total; }

template <int UKS, bool DUAL, bool ROWS>
static int tcp2_launch(const CUtensorMap& w, const CUtensorMap& x, const CUtensorMap& sfa, const CUtensorMap& sfb, const TcParams& p,
                       long long pairs, cudaStream_t st) {
  using C = Tcp2Cfg<UKS, ROWS>;
  static bool opted[16] = {};
  static int resident[16] = {};  // clusters of two that fit the device at once
  int dev = 0;
  cudaGetDevice(&dev);
  const int di = (dev >= 0 && dev < 16) ? dev : 0;
  if (!opted[di]) {
    TPX_CUDA_OK(cudaFuncSetAttribute(qlinear_tcp2_kernel<UKS, DUAL, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    opted[di] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(C::THREADS);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  if (resident[di] == 0) {
    cfg.gridDim = dim3((unsigned)(2 * (sm_count() / 2)));
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, qlinear_tcp2_kernel<UKS, DUAL, ROWS>, &cfg);
    if (e != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
    resident[di] = n > 0 ? n : -1;
  }
  TPX_REQUIRE(resident[di] > 0, TPX_ERR_UNSUPPORTED, "qlinear_mxfp4_tc: no cluster of two CTAs fits this device");
  long long clusters = pairs < resident[di] ? pairs : resident[di];
  if (clusters > sm_count() / 2) clusters = sm_count() / 2;
  cfg.gridDim = dim3((unsigned)(2 * clusters));
  count_launch();
  TPX_CUDA_OK(cudaLaunchKernelEx(&cfg, qlinear_tcp2_kernel<UKS, DUAL, ROWS>, w, x, sfa, sfb, p));
  return TPX_OK;
}

int tcp2_run(const uint8_t* wq, const uint8_t* sfa, bool pair, const uint16_t* x, int64_t M, int64_t N, int64_t K, const TcParams& base,
             void* scratch, size_t scratch_bytes, cudaStream_t st, const TcNorm* norm) {
  const Tcp2Plan pl = tcp2_plan(M, N, K, pair);
  TPX_REQUIRE(scratch && scratch_bytes >= pl.total, TPX_ERR_SCRATCH, "qlinear_mxfp4_tc: scratch of %zu bytes needed, %zu given", pl.total,
              scratch_bytes);
  unsigned char* sc = reinterpret_cast<unsigned char*>(scratch);
  uint8_t *terms = sc + pl.off_terms, *sfb = sc + pl.off_sfb;
  float* tscale = reinterpret_cast<float*>(sc + pl.off_tscale);
  if (pl.rows) {
    TPX_REQUIRE(((uintptr_t)x & 15) == 0 && (!norm || !norm->gamma || ((uintptr_t)norm->gamma & 15) == 0), TPX_ERR_ARG,
                "qlinear_mxfp4_tc: x and gamma must be 16-byte aligned");
    const void* gamma = norm ? norm->gamma : nullptr;
    const int gf = norm ? norm->gamma_f32 : 0;
    const float eps = norm ? norm->eps : 0.0f;
    if (pl.KS * 16 <= 128 * 4)
      TPX_CUDA_OK(launch_pdl(rowscale_split_kernel<4, 128>, dim3((unsigned)pl.Mpad), dim3(128), 0, st, x, gamma, gf, eps, (int)M, (int)K, pl.KS,
                             terms, tscale));
    else if (pl.KS * 16 <= kRsThreads * 4)
      TPX_CUDA_OK(launch_pdl(rowscale_split_kernel<4, kRsThreads>, dim3((unsigned)pl.Mpad), dim3(kRsThreads), 0, st, x, gamma, gf, eps, (int)M,
                             (int)K, pl.KS, terms, tscale));
    else
      TPX_CUDA_OK(launch_pdl(rowscale_split_kernel<8, kRsThreads>, dim3((unsigned)pl.Mpad), dim3(kRsThreads), 0, st, x, gamma, gf, eps, (int)M,
                             (int)K, pl.KS, terms, tscale));
  } else {
    int rc0 = tc_launch_split(x, (int)M, (int)K, pl.Mpad, pl.KS, 128, pl.uks, 0, terms, sfb, st, norm);
    if (rc0) return rc0;
  }
  const int nwt = pair ? 2 : 1;
  CUtensorMap mw, mx, msfa, msfb;
  int rc = tc_make_map(&mw, base.wfmt ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, wq,
                       (uint64_t)pl.TN * pl.KS * nwt * 128, base.wfmt ? 128 : 64, pair ? 128u : (uint32_t)pl.uks * 128u);
  if (rc) return rc;
  rc = tc_make_map(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, terms, (uint64_t)pl.Mpad * pl.KS * 2, 128, 128);
  if (rc) return rc;
  rc = tc_make_map_sf(&msfa, sfa, (uint64_t)pl.TN * pl.KS * nwt, pair ? 1u : (uint32_t)pl.uks);
  if (rc) return rc;
  rc = tc_make_map_sf(&msfb, sfb, (uint64_t)pl.TM * pl.KS * 2, 2u * (uint32_t)pl.uks);
  if (rc) return rc;
  TcParams p = base;
  p.sfa = sfa; p.sfa2 = nullptr; p.sfb = sfb;
  p.partial = pl.rows ? tscale : nullptr;  // this kernel has no partial tiles: the field carries the per-token scales
  p.counters = reinterpret_cast<unsigned*>(sc);
  p.err = reinterpret_cast<unsigned*>(sc + kTcCounterBytes - 4);
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.KS = pl.KS / pl.uks; p.TN = pl.TN; p.TM = pl.TM;
  p.whole_tiles = 1; p.cluster = 2;
  const long long pairs = (long long)((pl.TN + 1) / 2) * pl.TM;
  if (pl.rows) {
    if (pl.uks == 2) return pair ? tcp2_launch<2, true, true>(mw, mx, msfa, msfb, p, pairs, st) : tcp2_launch<2, false, true>(mw, mx, msfa, msfb, p, pairs, st);
    return pair ? tcp2_launch<1, true, true>(mw, mx, msfa, msfb, p, pairs, st) : tcp2_launch<1, false, true>(mw, mx, msfa, msfb, p, pairs, st);
  }
  if (pl.uks == 2) return pair ? tcp2_launch<2, true, false>(mw, mx, msfa, msfb, p, pairs, st) : tcp2_launch<2, false, false>(mw, mx, msfa, msfb, p, pairs, st);
  return pair ? tcp2_launch<1, true, false>(mw, mx, msfa, msfb, p, pairs, st) : tcp2_launch<1, false, false>(mw, mx, msfa, msfb, p, pairs, st);
}

}  // namespace tpx
