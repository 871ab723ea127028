// MXFP4 weight-only linear for few tokens (M <= 64: decoding), tensor-core path with the WEIGHTS on the wide side.
//
// A tcgen05.mma of shape 128 x N x 32 reads its 128-row A slab from shared memory at a fixed pace whatever N is, so
// a kernel that puts 128 weight rows on the A side consumes at most one 2 KiB slab of packed weights per ~110
// cycles: about 30 bytes/ns per SM, well below an SM's share of HBM bandwidth. Here the roles are swapped:
//   A (128 rows)  = the activation terms of up to 64 tokens (hi and lo E4M3 terms are separate rows),
//   B (256 rows)  = 256 output features of packed E2M1 weights (a gate tile and its up tile, or two adjacent tiles),
//   D             = [token term][feature] in tensor memory, 256 fp32 columns.
// Every MMA then consumes 4 KiB of packed weights in about the time the other orientation needs for 2 KiB (a
// 128-row MMA costs ~97 cycles however narrow it is, ~128 at N = 256). A pipeline stage holds two k steps (32 KiB
// of packed weights) for up to 16 tokens, one k step otherwise.
//
// Replaces the same reference functions as tpx_qlinear_tc.cu (fc_plain / fc_gate_up of
// src/csrc/llm/fused_llm_infer.cpp on MXFP4 weights) for M <= 64; layouts of the packed weights are shared.
//
// Work split: stream-K over (feature tile, k step) with whole tiles when the tile count suits the SM count;
// partial tiles go to per-CTA slots and a second, programmatically launched kernel sums them in CTA order.
#include "tpx_tc_ptx.cuh"

namespace tpx {

template <int TOKP, int UKS>
struct TcwCfg {
  static constexpr int X1 = 2 * TOKP * 128;             // both terms of one k step (128 k values of TOKP tokens)
  static constexpr int B1 = 256 * 128;                  // 256 features x 128 k values, unpacked to 16-byte-aligned groups
  static constexpr int X_BYTES = UKS * X1;              // a stage holds UKS k steps
  static constexpr int B_BYTES = UKS * B1;
  static constexpr int B_TX = 256 * 64;                 // what the copy of one k step accounts for (packed bytes)
  static constexpr int SF_BYTES = UKS * (512 + 2 * 512);  // per k step: activation scale block, two weight scale blocks
  static constexpr int RAW = X_BYTES + B_BYTES + SF_BYTES;
  static constexpr int STAGE_BYTES = (RAW + 1023) / 1024 * 1024;
  static constexpr int BUDGET = 227 * 1024 - 2048;
  static constexpr int STAGES_RAW = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
  static constexpr int SF_COLS = 12 * UKS;              // per k step 4 (activations) + 8 (weights) columns
  static constexpr int D_COLS = 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int EPI_WARPS = TOKP == 16 ? 4 : TOKP / 16;  // 32-lane quarters of tensor memory that hold tokens
  // The epilogue is a chain of dependent scalar instructions per (token, column): one warp per quarter ran it at a
  // fraction of the issue rate (5 us of a 27 us gate/up launch at 64 tokens). Every quarter therefore has EPI_SPLIT
  // warps, each taking a contiguous share of the 16-column chunks.
  static constexpr int EPI_SPLIT = 4;
  static constexpr int THREADS = 64 + 128 * EPI_SPLIT;
  static constexpr int TOK_PER_WARP = TOKP == 16 ? 4 : 16;       // 16 tokens are spread four per quarter (row map 2)
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;
  static_assert(D_COLS + STAGES * SF_COLS <= 512, "tensor memory");
  static_assert((UKS - 1) * X1 + 128 * 128 <= X_BYTES + B_BYTES, "the A descriptor spans 128 rows inside the stage");
  static_assert(UKS * 2 * TOKP <= 256, "one copy request for the activation rows of a stage");
};

// Eight consecutive output features of one token: bias, activation, gate multiply, residual, one 16-byte store.
template <bool DUAL>
__device__ __forceinline__ void tcw_finish8(const TcParams& p, int tok, int n, const float (&v)[8], const float (&u)[8],
                                            float* stored = nullptr) {
  const size_t o = (size_t)tok * p.N + n;
  float x[8];
#pragma unroll
  for (int i = 0; i < 8; i++) x[i] = v[i];
  auto unpack = [](const uint4& q, float (&f)[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      f[2 * i] = bf16_bits_to_f32((uint16_t)(w[i] & 0xffff));
      f[2 * i + 1] = bf16_bits_to_f32((uint16_t)(w[i] >> 16));
    }
  };
  uint4 qb = make_uint4(0, 0, 0, 0), qm = qb, qr = qb;
  if (p.bias) qb = *reinterpret_cast<const uint4*>(p.bias + n);
  if (p.mul_in) qm = *reinterpret_cast<const uint4*>(p.mul_in + o);
  if (p.res) qr = *reinterpret_cast<const uint4*>(p.res + o);
  if (p.bias) {
    float f[8];
    unpack(qb, f);
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] += f[i];
  }
  switch (p.act) {
    case TPX_ACT_GELU:
#pragma unroll
      for (int i = 0; i < 8; i++) x[i] = 0.5f * x[i] * (1.0f + erff(x[i] * 0.70710678118654752f));
      break;
    case TPX_ACT_SILU:
#pragma unroll
      for (int i = 0; i < 8; i++) x[i] = __fdividef(x[i], 1.0f + __expf(-x[i]));
      break;
    case TPX_ACT_RELU:
#pragma unroll
      for (int i = 0; i < 8; i++) x[i] = fmaxf(x[i], 0.0f);
      break;
    default: break;
  }
  if (DUAL) {
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] *= u[i];
  }
  if (p.mul_in) {
    float f[8];
    unpack(qm, f);
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] *= f[i];
  }
  if (p.res) {
    float f[8];
    unpack(qr, f);
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] += f[i] * p.res_scale;
  }
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; i++) w[i] = (uint32_t)f32_to_bf16_bits(x[2 * i]) | ((uint32_t)f32_to_bf16_bits(x[2 * i + 1]) << 16);
  *reinterpret_cast<uint4*>(p.y + o) = make_uint4(w[0], w[1], w[2], w[3]);
  if (stored) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      stored[2 * i] = bf16_bits_to_f32((uint16_t)(w[i] & 0xffff));
      stored[2 * i + 1] = bf16_bits_to_f32((uint16_t)(w[i] >> 16));
    }
  }
}

// Hand-over of a finished 32-feature block to the next linear (TcEmit): lanes l and l ^ 16 hold one token's features
// [n0, n0 + 32) as st[q][i] = feature n0 + 16 q + 8 half + i. Called by every lane of the warp; `live` lanes store.
__device__ __forceinline__ void tcw_emit32(const TcEmit& E, int tok, int n0, int half, bool live, const float (&st)[2][8]) {
  float am = 0.0f;
#pragma unroll
  for (int q = 0; q < 2; q++)
#pragma unroll
    for (int i = 0; i < 8; i++) am = fmaxf(am, fabsf(st[q][i]));
  am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 16));
  const int e = tc_emit_exp(__float_as_uint(am));
  const float down = __uint_as_float((uint32_t)(127 - e) << 23);
  if (!live) return;
  const TcEmitAddr a = tc_emit_addr(E, tok, n0 >> 5);
#pragma unroll
  for (int q = 0; q < 2; q++) {
    uint32_t h[2] = {0, 0}, l[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint32_t hi, lo;
      tc_emit_cvt2(st[q][2 * i], st[q][2 * i + 1], down, hi, lo);
      h[i >> 1] |= hi << (16 * (i & 1));
      l[i >> 1] |= lo << (16 * (i & 1));
    }
    *reinterpret_cast<uint2*>(a.hi + q * 16 + half * 8) = make_uint2(h[0], h[1]);
    *reinterpret_cast<uint2*>(a.lo + q * 16 + half * 8) = make_uint2(l[0], l[1]);
  }
  if (half == 0) {
    *a.sh = (uint8_t)(e + 127);
    *a.sl = (uint8_t)(e + 127);
  }
}

// p.TN counts the 256-feature tiles here (a gate/up pair: 128 + 128), p.TM is 1, p.KS the k units (UKS k steps of
// 128 each) per tile, ksteps the k steps of a tile in the packed weight.
template <int TOKP, bool DUAL, int UKS>
__global__ void __launch_bounds__(TcwCfg<TOKP, UKS>::THREADS, 1)
qlinear_tcw_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, TcParams p, const uint8_t* wq,
                   int tiles128, int ksteps) {
  using C = TcwCfg<TOKP, UKS>;
  extern __shared__ unsigned char tcw_smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[C::STAGES], bar_empty[C::STAGES];
  __shared__ __align__(8) unsigned long long bar_acc_full, bar_acc_empty;
  __shared__ uint32_t tmem_holder;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (tc_smem_u32(tcw_smem_raw) + 1023u) & ~1023u;

  const long long U = (long long)p.TN * p.KS;
  const long long G = gridDim.x;
  const long long T = p.TN;
  // p.cluster > 1: the CTAs of a cluster share one tile and cut its k units evenly between them
  const int crank = p.cluster > 1 ? (int)tc_cluster_rank() : 0;
  const long long ctile = blockIdx.x / p.cluster;
  const long long u0 = p.cluster > 1 ? ctile * p.KS + (long long)crank * p.KS / p.cluster
                     : p.whole_tiles ? ((long long)blockIdx.x * T / G) * p.KS : (long long)blockIdx.x * U / G;
  const long long u1 = p.cluster > 1 ? ctile * p.KS + ((long long)crank + 1) * p.KS / p.cluster
                     : p.whole_tiles ? (((long long)blockIdx.x + 1) * T / G) * p.KS : ((long long)blockIdx.x + 1) * U / G;
  const int nunits = (int)(u1 - u0);
  const int tile0 = (int)(u0 / p.KS), ks0 = (int)(u0 % p.KS);

  if (threadIdx.x == 0) tc_stamp(p, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; s++) {
      tc_mbar_init(tc_smem_u32(&bar_full[s]), 1);
      tc_mbar_init(tc_smem_u32(&bar_empty[s]), 1);
    }
    tc_mbar_init(tc_smem_u32(&bar_acc_full), 1);
    tc_mbar_init(tc_smem_u32(&bar_acc_empty), C::EPI_WARPS * C::EPI_SPLIT);
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
  if (threadIdx.x == 0) tc_stamp(p, 1);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the fix-up kernel may get its CTAs ready

  // weight tiles (of 128 features) of feature tile t at k step ks: a pair is stored as [t][ks][gate, up], single
  // weights as [tile128][ks], so the two halves of a 256-feature tile are p.KS tiles apart
  auto wtile_a = [&](int t, int kstep) { return DUAL ? (t * ksteps + kstep) * 2 : (2 * t * ksteps + kstep); };
  auto wtile_b = [&](int t, int kstep) { return DUAL ? (t * ksteps + kstep) * 2 + 1 : ((2 * t + 1) * ksteps + kstep); };
  auto has_b = [&](int t) { return DUAL || 2 * t + 1 < tiles128; };

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      auto fetch_w = [&](int s, int t, int ks) {
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t bar = tc_smem_u32(&bar_full[s]);
        const uint32_t sb = st + C::X_BYTES, ssf = sb + C::B_BYTES + UKS * 512;
        const bool second = has_b(t);
        const int b_tx = p.wfmt ? 2 * C::B_TX : C::B_TX;  // 8-bit weights arrive byte for byte, packed 4-bit ones at half the footprint
        tc_mbar_expect_tx(bar, C::X_BYTES + UKS * 512 + UKS * (second ? b_tx + 1024 : b_tx / 2 + 512));
#pragma unroll
        for (int kk = 0; kk < UKS; kk++) {
          const int ta = wtile_a(t, ks * UKS + kk), tb = wtile_b(t, ks * UKS + kk);
          if (DUAL) {
            tc_tma_2d(sb + kk * C::B1, &tmW, 0, ta * 128, bar);  // 256 rows: gate tile and up tile are adjacent
            tc_bulk_g2s(ssf + kk * 1024, p.sfa + (size_t)ta * 512, 1024, bar);
          } else {
            tc_tma_2d(sb + kk * C::B1, &tmW, 0, ta * 128, bar);
            tc_bulk_g2s(ssf + kk * 1024, p.sfa + (size_t)ta * 512, 512, bar);
            if (second) {
              tc_tma_2d(sb + kk * C::B1 + C::B1 / 2, &tmW, 0, tb * 128, bar);
              tc_bulk_g2s(ssf + kk * 1024 + 512, p.sfa + (size_t)tb * 512, 512, bar);
            }
          }
        }
      };
      auto fetch_x = [&](int s, int ks) {
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t bar = tc_smem_u32(&bar_full[s]);
        tc_tma_2d(st, &tmX, 0, ks * UKS * 2 * TOKP, bar);
        tc_bulk_g2s(st + C::X_BYTES + C::B_BYTES, p.sfb + (size_t)ks * UKS * 512, UKS * 512, bar);
      };
      // Packed weights further ahead than the stages reach are prefetched into L2, so that the bytes in flight from
      // HBM are not limited by shared memory.
      auto prefetch_w = [&](int t, int ks) {
        if (DUAL) {
          tc_prefetch_bulk(wq + (size_t)wtile_a(t, ks * UKS) * 8192, UKS * 16384);  // the k steps of a pair tile are adjacent
        } else {
          tc_prefetch_bulk(wq + (size_t)wtile_a(t, ks * UKS) * 8192, UKS * 8192);
          if (has_b(t)) tc_prefetch_bulk(wq + (size_t)wtile_b(t, ks * UKS) * 8192, UKS * 8192);
        }
      };
      const int early = nunits < C::STAGES ? nunits : C::STAGES;
      int ptile = tile0, pks = ks0, pit = 0;
      for (; pit < early; pit++) {  // weights do not depend on the split kernel: out before the grid dependency wait
        fetch_w(pit, ptile, pks);
        if (++pks == p.KS) { pks = 0; ptile++; }
      }
      for (; pit < nunits && pit < early + p.pf; pit++) {
        prefetch_w(ptile, pks);
        if (++pks == p.KS) { pks = 0; ptile++; }
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      int tile = tile0, ks = ks0;
      for (int it = 0; it < nunits; it++) {
        const int s = it % C::STAGES;
        if (pit < nunits && pit < it + C::STAGES + p.pf) {
          prefetch_w(ptile, pks);
          pit++;
          if (++pks == p.KS) { pks = 0; ptile++; }
        }
        if (it >= C::STAGES) {
          if (!tc_wait(tc_smem_u32(&bar_empty[s]), (uint32_t)((it / C::STAGES - 1) & 1))) {
            atomicExch(p.err, 2u);
            break;
          }
          fetch_w(s, tile, ks);
        }
        fetch_x(s, ks);
        if (++ks == p.KS) { ks = 0; tile++; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // A = E4M3 (0), B = E2M1 (5), both K-major, N = 256, UE8M0 scales, M = 128
      const uint32_t idesc0 = (0u << 7) | ((p.wfmt == 0 ? 5u : p.wfmt == 1 ? 0u : 1u) << 10) | ((256u >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
      int ks = ks0;
      uint32_t acc_phase = 0;
      bool fresh = true;
      for (int it = 0; it < nunits; it++) {
        const int s = it % C::STAGES;
        const uint32_t ph = (uint32_t)((it / C::STAGES) & 1);
        if (fresh && it > 0) {
          if (!tc_wait(tc_smem_u32(&bar_acc_empty), acc_phase)) { atomicExch(p.err, 3u); break; }
          acc_phase ^= 1;
        }
        if (!tc_wait(tc_smem_u32(&bar_full[s]), ph)) { atomicExch(p.err, 4u); break; }
        if (it == 0) tc_stamp(p, 2);
        if (it == nunits - 1) tc_stamp(p, 3);
        tc_fence_after();
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t sb = st + C::X_BYTES;
        const uint32_t ssf = sb + C::B_BYTES;
        const uint32_t sf_t = tmem + C::D_COLS + (uint32_t)s * C::SF_COLS;
        const bool part_end = (ks == p.KS - 1) || (it == nunits - 1);
#pragma unroll
        for (int kk = 0; kk < UKS; kk++) {
          // shared memory: [activation blocks of the UKS k steps][weight blocks, two per k step]; tensor memory: per k
          // step 4 activation columns, then 8 weight columns
          const uint32_t sfk = sf_t + kk * 12;
          tc_cp_sf(sfk, tc_sf_desc(ssf + kk * 512));
          tc_cp_sf(sfk + 4, tc_sf_desc(ssf + UKS * 512 + kk * 1024));
          tc_cp_sf(sfk + 8, tc_sf_desc(ssf + UKS * 512 + kk * 1024 + 512));
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const uint32_t idesc = idesc0 | ((uint32_t)j << 29) | ((uint32_t)j << 4);
            // rows past the stored ones alias other rows or the weight area: unused lanes. 16 tokens: 8-row groups 256
            // bytes apart, so that MMA rows 32q + 16*term + t read the stored row 8q + 4*term + t
            const uint64_t adesc = (TOKP == 16 ? tc_smem_desc_sbo(st + kk * C::X1, 256) : tc_smem_desc(st + kk * C::X1)) + (uint64_t)(2 * j);
            const uint64_t bdesc = tc_smem_desc(sb + kk * C::B1) + (uint64_t)(2 * j);
            tc_mma(tmem, adesc, bdesc, idesc, sfk | ((uint32_t)j << 30), (sfk + 4) | ((uint32_t)j << 30),
                   (fresh && kk == 0 && j == 0) ? 0u : 1u);
          }
        }
        tc_commit(tc_smem_u32(&bar_empty[s]));
        if (part_end) tc_commit(tc_smem_u32(&bar_acc_full));
        fresh = part_end;
        if (++ks == p.KS) ks = 0;
      }
    }
    __syncwarp();
  } else if ((warp & 3) < C::EPI_WARPS) {
    // ------------------------------------------------------------ epilogue: quarter `sub` of tensor memory holds
    // tokens 16*sub .. 16*sub+15: hi terms in lanes 0-15, lo terms in lanes 16-31
    const int sub = warp & 3;
    const uint32_t lane_base = ((uint32_t)(sub * 32)) << 16;
    const int tok = sub * C::TOK_PER_WARP + (lane & 15);
    const bool lane_live = (lane & 15) < C::TOK_PER_WARP;  // lanes beyond hold rows that alias others
    const int half = lane >> 4;  // after the hi+lo sum both halves hold the same values: each finishes 8 of 16 features
    int tile = tile0, ks = ks0;
    int part_first_ks = ks0;
    uint32_t acc_phase = 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");  // scratch, residual and gate inputs belong to earlier grids
    for (int it = 0; it < nunits; it++) {
      const bool part_end = (ks == p.KS - 1) || (it == nunits - 1);
      if (part_end) {
        if (!tc_wait(tc_smem_u32(&bar_acc_full), acc_phase)) {
          if (lane == 0) atomicExch(p.err, 6u);
          break;
        }
        acc_phase ^= 1;
        tc_fence_after();
        if (threadIdx.x == 128 && it == nunits - 1) tc_stamp(p, 5);
        const bool whole = (part_first_ks == 0) && (ks == p.KS - 1);
        float* myslot = p.partial + (((size_t)blockIdx.x * 2 + (tile == tile0 ? 0 : 1)) * TOKP + tok) * 256;
        constexpr int CHUNKS = DUAL ? 8 : 16;
        constexpr int CPW = CHUNKS / C::EPI_SPLIT;  // chunks of this warp: [cpart * CPW, +CPW)
        const int cpart = (warp - 2) >> 2;
#pragma unroll 1
        for (int c0 = cpart * CPW; c0 < (cpart + 1) * CPW; c0 += 2) {  // two 16-column chunks per round trip to tensor memory
          uint32_t a[2][16], b[2][16];
#pragma unroll
          for (int q = 0; q < 2; q++) {
            tc_ld_x16(tmem + lane_base + (c0 + q) * 16, a[q]);
            if (DUAL) tc_ld_x16(tmem + lane_base + 128 + (c0 + q) * 16, b[q]);
          }
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          float st[2][8];  // the stored values of this round, for the hand-over to the next linear
#pragma unroll
          for (int q = 0; q < 2; q++)
#pragma unroll
            for (int i = 0; i < 8; i++) st[q][i] = 0.0f;
#pragma unroll
          for (int q = 0; q < 2; q++) {
            // lanes l and l ^ 16 hold the hi and lo sums of one token: each keeps 8 of the 16 columns and gets the
            // other term of those from its partner
            float v[8], u[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
              const float mine = __uint_as_float(half ? a[q][i + 8] : a[q][i]);
              const float send = __uint_as_float(half ? a[q][i] : a[q][i + 8]);
              v[i] = mine + __shfl_xor_sync(0xffffffffu, send, 16);
              if (DUAL) {
                const float mine2 = __uint_as_float(half ? b[q][i + 8] : b[q][i]);
                const float send2 = __uint_as_float(half ? b[q][i] : b[q][i + 8]);
                u[i] = mine2 + __shfl_xor_sync(0xffffffffu, send2, 16);
              } else {
                u[i] = 0.0f;
              }
            }
            const int col = (c0 + q) * 16 + half * 8;  // first of this thread's 8 accumulator columns
            if (whole) {
              const int n = DUAL ? tile * 128 + col : tile * 256 + col;
              if (lane_live && tok < p.M && n < p.N) tcw_finish8<DUAL>(p, tok, n, v, u, p.emit.terms ? st[q] : nullptr);
            } else if (p.cluster > 1) {  // partial of a cluster member: [token][256 columns] fp32 at the start of its stages
              if (lane_live) {
                const uint32_t sp = smem_base + (uint32_t)((tok * 256 + col) * 4);
                tc_st_shared_f4(sp, make_float4(v[0], v[1], v[2], v[3]));
                tc_st_shared_f4(sp + 16, make_float4(v[4], v[5], v[6], v[7]));
                if (DUAL) {
                  tc_st_shared_f4(sp + 512, make_float4(u[0], u[1], u[2], u[3]));
                  tc_st_shared_f4(sp + 528, make_float4(u[4], u[5], u[6], u[7]));
                }
              }
            } else if (lane_live) {
              __stcg(reinterpret_cast<float4*>(myslot + col), make_float4(v[0], v[1], v[2], v[3]));
              __stcg(reinterpret_cast<float4*>(myslot + col) + 1, make_float4(v[4], v[5], v[6], v[7]));
              if (DUAL) {
                __stcg(reinterpret_cast<float4*>(myslot + 128 + col), make_float4(u[0], u[1], u[2], u[3]));
                __stcg(reinterpret_cast<float4*>(myslot + 128 + col) + 1, make_float4(u[4], u[5], u[6], u[7]));
              }
            }
          }
          if (whole && p.emit.terms) {  // uniform over the warp
            const int n0 = (DUAL ? tile * 128 : tile * 256) + c0 * 16;
            tcw_emit32(p.emit, tok, n0, half, lane_live && tok < p.M && n0 < p.N, st);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) tc_mbar_arrive(tc_smem_u32(&bar_acc_empty));
      }
      if (++ks == p.KS) {
        ks = 0;
        tile++;
        part_first_ks = 0;
      }
    }
  }
  if (threadIdx.x == 128) tc_stamp(p, 6);
  tc_fence_before();
  __syncthreads();
  if (p.cluster > 1) {
    // every member's partial is in its own shared memory; the (token, 8 features) groups of the tile go round the
    // members, each adds the members' parts in rank order (distributed shared memory reads) and finishes its groups.
    // Nobody leaves before all have finished reading.
    tc_cluster_sync();
    if (threadIdx.x == 128) tc_stamp(p, 4);
    if (warp >= 2) {
      constexpr int GROUPS = DUAL ? 16 : 32;  // groups of 8 output features per token
      constexpr int NT = C::THREADS - 64;
      const int et = (int)threadIdx.x - 64;
      const int live_tok = p.M < TOKP ? p.M : TOKP;
      // items go round the members a warp's worth at a time, so that every member's shared memory port and store
      // path carry an equal share (handed out a CTA's worth at a time, 16 tokens left everything to the first member:
      // 128 KB through one SM's port, 4.3 us)
      for (int i = (((et >> 5) * p.cluster + crank) << 5) + (et & 31); i < live_tok * GROUPS; i += NT * p.cluster) {
        const int tk = i / GROUPS, col = (i % GROUPS) * 8;
        const int n = DUAL ? (int)ctile * 128 + col : (int)ctile * 256 + col;
        if (n >= p.N) continue;
        float v[8], u[8];
#pragma unroll
        for (int q = 0; q < 8; q++) v[q] = u[q] = 0.0f;
        const uint32_t sp = smem_base + (uint32_t)((tk * 256 + col) * 4);
        tc_cluster_sum<2, 4>(sp, p.cluster, v);
        if (DUAL) tc_cluster_sum<2, 4>(sp + 512, p.cluster, u);
        tcw_finish8<DUAL>(p, tk, n, v, u);
      }
    }
    tc_cluster_sync();
  }
  if (threadIdx.x == 128) tc_stamp(p, 7);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)C::TMEM_COLS) : "memory");
  }
}


// ---------------------------------------------------------------- fix-up of tiles cut between CTAs
// One thread per (token, 8 output features) of a tile; contributors are the consecutive CTAs cfirst..clast, CTA c
// keeps its part in slot 0 if the tile is the first it touched, else in slot 1. Fixed summation order.
template <bool DUAL>
__global__ void __launch_bounds__(128) tcw_fixup_kernel(TcParams p, int TOKP, int G) {
  constexpr int GROUPS = DUAL ? 16 : 32;
  pdl_trigger();
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int tile = blockIdx.x;
  const int idx = blockIdx.y * 128 + threadIdx.x;
  const int tok = idx / GROUPS, col = (idx % GROUPS) * 8;
  const long long U = (long long)p.TN * p.KS;
  const long long ta = (long long)tile * p.KS, tb = ta + p.KS - 1;
  const int cfirst = (int)(((ta + 1) * G - 1) / U), clast = (int)(((tb + 1) * G - 1) / U);
  if (cfirst == clast) return;  // one CTA had the whole tile and finished it itself
  const int n = DUAL ? tile * 128 + col : tile * 256 + col;
  if (tok >= p.M || tok >= TOKP || n >= p.N) return;
  float v[8], u[8];
#pragma unroll
  for (int i = 0; i < 8; i++) v[i] = u[i] = 0.0f;
#pragma unroll 1
  for (int cb = cfirst; cb <= clast; cb += 4) {  // four contributors' loads in flight at a time
    float4 t[4][DUAL ? 4 : 2];
#pragma unroll
    for (int cc = 0; cc < 4; cc++) {
      const int c = cb + cc;
      if (c <= clast) {
        const int ctile0 = (int)(((long long)c * U / G) / p.KS);
        const float* slot = p.partial + (((size_t)c * 2 + (tile == ctile0 ? 0 : 1)) * TOKP + tok) * 256 + col;
        t[cc][0] = __ldcg(reinterpret_cast<const float4*>(slot));
        t[cc][1] = __ldcg(reinterpret_cast<const float4*>(slot) + 1);
        if (DUAL) {
          t[cc][DUAL ? 2 : 0] = __ldcg(reinterpret_cast<const float4*>(slot + 128));
          t[cc][DUAL ? 3 : 1] = __ldcg(reinterpret_cast<const float4*>(slot + 128) + 1);
        }
      }
    }
#pragma unroll
    for (int cc = 0; cc < 4; cc++) {
      if (cb + cc <= clast) {
        v[0] += t[cc][0].x; v[1] += t[cc][0].y; v[2] += t[cc][0].z; v[3] += t[cc][0].w;
        v[4] += t[cc][1].x; v[5] += t[cc][1].y; v[6] += t[cc][1].z; v[7] += t[cc][1].w;
        if (DUAL) {
          u[0] += t[cc][DUAL ? 2 : 0].x; u[1] += t[cc][DUAL ? 2 : 0].y; u[2] += t[cc][DUAL ? 2 : 0].z; u[3] += t[cc][DUAL ? 2 : 0].w;
          u[4] += t[cc][DUAL ? 3 : 1].x; u[5] += t[cc][DUAL ? 3 : 1].y; u[6] += t[cc][DUAL ? 3 : 1].z; u[7] += t[cc][DUAL ? 3 : 1].w;
        }
      }
    }
  }
  tcw_finish8<DUAL>(p, tok, n, v, u);
}

// ---------------------------------------------------------------- host side
struct TcwPlan {
  int tokp, uks, KS, KU, tiles128, TN, grid, whole, cluster;  // KS k steps, KU = KS / uks pipeline units per tile
  size_t off_terms, off_sfb, off_partial, total;
};

static TcwPlan tcw_plan(int64_t M, int64_t N, int64_t K, bool pair) {
  TcwPlan pl;
  pl.tokp = M <= 16 ? 16 : M <= 32 ? 32 : 64;
  pl.KS = tc_padded_ks(K, pair);
  pl.uks = pl.tokp == 16 ? 2 : 1;  // two k steps per stage while three such stages fit in shared memory
  pl.KU = pl.KS / pl.uks;
  pl.tiles128 = (int)((N + 127) / 128);
  pl.TN = pair ? pl.tiles128 : (pl.tiles128 + 1) / 2;
  const long long U = (long long)pl.TN * pl.KU, T = pl.TN;
  const int sms = sm_count();
  // whole tiles when their count suits the SM count (no fix-up pass), else the (tile, k step) units are cut evenly
  pl.whole = (T * 10 >= (long long)sms * 7 && T <= sms) || T >= 8LL * sms;
  if (knobs().tc_whole >= 0) pl.whole = knobs().tc_whole;
  pl.grid = pl.whole ? (int)(T < sms ? T : sms) : (int)(U < sms ? U : sms);
  // few tiles: a cluster of CTAs per tile cuts K and reduces over distributed shared memory (no fix-up pass)
  pl.cluster = 1;
  if (!pl.whole && T * 2 <= sms) {
    int c = (int)(sms / T);
    if (c > 8) c = 8;
    if (c > pl.KU) c = pl.KU;
    if (c > 1) pl.cluster = c;
  }
  if (knobs().tc_cluster == 0) pl.cluster = 1;
  size_t o = kTcCounterBytes;
  auto bump = [&](size_t bytes) { size_t r = o; o += (bytes + 1023) & ~(size_t)1023; return r; };
  pl.off_terms = bump((size_t)pl.KS * 2 * pl.tokp * 128);
  pl.off_sfb = bump((size_t)pl.KS * 512);
  pl.off_partial = bump((size_t)pl.grid * 2 * pl.tokp * 256 * sizeof(float));
  pl.total = o;
  return pl;
}

size_t tcw_scratch_bytes(int64_t M, int64_t N, int64_t K, bool pair) { return tcw_plan(M, N, K, pair).total; }

template <int TOKP, bool DUAL, int UKS>
static int tcw_launch(const CUtensorMap& w, const CUtensorMap& x, const TcParams& p, const uint8_t* wq, int tiles128, int ksteps,
                      int grid, cudaStream_t st) {
  using C = TcwCfg<TOKP, UKS>;
  static bool opted[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || !opted[dev]) {
    TPX_CUDA_OK(cudaFuncSetAttribute(qlinear_tcw_kernel<TOKP, DUAL, UKS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    if (dev >= 0 && dev < 16) opted[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(C::THREADS);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (p.cluster > 1) {
    // one cluster per tile, all of them resident at once, or not at all (then the tiles are cut stream-K fashion)
    cudaLaunchConfig_t cc = cfg;
    cc.gridDim = dim3((unsigned)(p.TN * p.cluster));
    cudaLaunchAttribute a2[2];
    a2[0] = attr[0];
    a2[1].id = cudaLaunchAttributeClusterDimension;
    a2[1].val.clusterDim.x = (unsigned)p.cluster;
    a2[1].val.clusterDim.y = 1;
    a2[1].val.clusterDim.z = 1;
    cc.attrs = a2;
    cc.numAttrs = 2;
    // the largest cluster size, from the planned one down, of which one cluster per tile can be resident at once
    static int fits[16][9] = {};  // 0 unknown, else 1 + the number of clusters of this size that can be resident
    int c = p.cluster;
    for (; c >= 2; c--) {
      int& f = fits[(dev >= 0 && dev < 16) ? dev : 0][c];
      if (f == 0) {
        a2[1].val.clusterDim.x = (unsigned)c;
        cc.gridDim = dim3((unsigned)(p.TN * c));
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, qlinear_tcw_kernel<TOKP, DUAL, UKS>, &cc);
        if (e != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
        f = 1 + n;
      }
      if (f - 1 >= p.TN) break;
    }
    if (c >= 2) {
      TcParams q = p;
      q.cluster = c;
      a2[1].val.clusterDim.x = (unsigned)c;
      cc.gridDim = dim3((unsigned)(p.TN * c));
      count_launch();
      TPX_CUDA_OK(cudaLaunchKernelEx(&cc, qlinear_tcw_kernel<TOKP, DUAL, UKS>, w, x, q, wq, tiles128, ksteps));
      return TPX_OK;
    }
    TcParams q = p;
    q.cluster = 1;
    return tcw_launch<TOKP, DUAL, UKS>(w, x, q, wq, tiles128, ksteps, grid, st);
  }
  count_launch();
  TPX_CUDA_OK(cudaLaunchKernelEx(&cfg, qlinear_tcw_kernel<TOKP, DUAL, UKS>, w, x, p, wq, tiles128, ksteps));
  if (!p.whole_tiles && grid > 1) {
    constexpr int GROUPS = DUAL ? 16 : 32;
    cudaLaunchConfig_t c2 = {};
    c2.gridDim = dim3((unsigned)p.TN, (unsigned)(TOKP * GROUPS / 128));
    c2.blockDim = dim3(128);
    c2.stream = st;
    c2.attrs = attr;
    c2.numAttrs = 1;
    count_launch();
  TPX_CUDA_OK(cudaLaunchKernelEx(&c2, tcw_fixup_kernel<DUAL>, p, (int)TOKP, grid));
  }
  return TPX_OK;
}

int tcw_run(const uint8_t* wq, const uint8_t* sfa, bool pair, const uint16_t* x, int64_t M, int64_t N, int64_t K, const TcParams& base,
            void* scratch, size_t scratch_bytes, cudaStream_t st, const TcNorm* norm) {
  TcwPlan pl = tcw_plan(M, N, K, pair);
  TPX_REQUIRE(scratch && scratch_bytes >= pl.total, TPX_ERR_SCRATCH, "qlinear_mxfp4_tc: scratch of %zu bytes needed, %zu given", pl.total,
              scratch_bytes);
  TPX_REQUIRE((((uintptr_t)base.y | (uintptr_t)base.bias | (uintptr_t)base.mul_in | (uintptr_t)base.res) & 15) == 0, TPX_ERR_ARG,
              "qlinear_mxfp4_tc: y, bias, mul_in and res must be 16-byte aligned");
  unsigned char* sc = reinterpret_cast<unsigned char*>(scratch);
  uint8_t *terms = sc + pl.off_terms, *sfb = sc + pl.off_sfb;
  int rc;
  if (norm && norm->pre) {  // the previous linear's epilogue wrote the terms
    const TcEmit& e = *norm->pre;
    TPX_REQUIRE(!norm->gamma && e.TOK == pl.tokp && e.UKS == 1 && e.KS == pl.KS && e.rowmap == (pl.tokp == 16 ? 2 : 1), TPX_ERR_ARG,
                "qlinear_mxfp4_tc: handed-over activation terms do not fit this launch");
    terms = e.terms;
    sfb = e.sfb;
  } else {
    rc = tc_launch_split(x, (int)M, (int)K, pl.tokp, pl.KS, pl.tokp, 1, pl.tokp == 16 ? 2 : 1, terms, sfb, st, norm);
    if (rc) return rc;
  }
  CUtensorMap mw, mx;
  const uint64_t wrows = (uint64_t)(pair ? pl.TN * 2 : pl.tiles128) * pl.KS * 128;
  rc = tc_make_map(&mw, base.wfmt ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, wq, wrows, base.wfmt ? 128 : 64,
                   pair ? 256 : 128);
  if (rc) return rc;
  rc = tc_make_map(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, terms, (uint64_t)pl.KS * 2 * pl.tokp, 128, (uint32_t)(pl.uks * 2 * pl.tokp));
  if (rc) return rc;
  TcParams p = base;
  p.sfa = sfa; p.sfa2 = nullptr; p.sfb = sfb;
  p.partial = reinterpret_cast<float*>(sc + pl.off_partial);
  p.counters = reinterpret_cast<unsigned*>(sc);
  p.err = reinterpret_cast<unsigned*>(sc + kTcCounterBytes - 4);
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.KS = pl.KU; p.TN = pl.TN; p.TM = 1; p.whole_tiles = pl.whole; p.cluster = pl.cluster;
  if (!pl.whole) p.emit.terms = nullptr;  // only the whole-tile epilogue hands its output over
  tc_note_emitted(p.emit.terms != nullptr);
  if (pair) {
    switch (pl.tokp) {
      case 16: return tcw_launch<16, true, 2>(mw, mx, p, wq, pl.tiles128, pl.KS, pl.grid, st);
      case 32: return tcw_launch<32, true, 1>(mw, mx, p, wq, pl.tiles128, pl.KS, pl.grid, st);
      default: return tcw_launch<64, true, 1>(mw, mx, p, wq, pl.tiles128, pl.KS, pl.grid, st);
    }
  }
  switch (pl.tokp) {
    case 16: return tcw_launch<16, false, 2>(mw, mx, p, wq, pl.tiles128, pl.KS, pl.grid, st);
    case 32: return tcw_launch<32, false, 1>(mw, mx, p, wq, pl.tiles128, pl.KS, pl.grid, st);
    default: return tcw_launch<64, false, 1>(mw, mx, p, wq, pl.tiles128, pl.KS, pl.grid, st);
  }
}

// Split layout of this kernel as the consumer of a hand-over (one weight, K a whole number of 128-wide k steps).
bool tcw_handoff_layout(int64_t M, int64_t N, int64_t K, TcEmit* E, size_t* terms_bytes, size_t* sfb_bytes) {
  if (M < 1 || M > 64 || K % 128) return false;
  const TcwPlan pl = tcw_plan(M, N, K, false);
  if ((int64_t)pl.KS * 128 != K) return false;
  E->TOK = pl.tokp; E->UKS = 1; E->KS = pl.KS; E->rowmap = pl.tokp == 16 ? 2 : 1;
  *terms_bytes = (size_t)pl.KS * 2 * pl.tokp * 128;
  *sfb_bytes = (size_t)pl.KS * 512;
  return true;
}

}  // namespace tpx
