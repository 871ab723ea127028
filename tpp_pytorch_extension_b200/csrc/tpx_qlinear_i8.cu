// int8 linear on the tcgen05 tensor cores, with the reference's own arithmetic, for any number of tokens.
//
// Replaces TppBlockedQInt8LinearW (src/csrc/fused_gemm.h:1075-1341): activations are quantised on the fly to int8 with
// one scale per (token, K block) (quantize_int8sym, :1249), every K block is an int8 x int8 -> int32 product
// (:1134-1137, :1197-1198) and the output accumulates tmp * s_x[token, block] * s_w[block, feature]
// (DequantTPP, :1200-1204). Here:
//   quantize_act_i8_kernel   x bf16 [M][K] -> xq int8 [TOKP][Kp] (padding tokens zero), sx fp32 [K/B][TOKP]
//   qlinear_i8_kernel<TOK>   A = 128 weight rows (int8, TMA, 128-byte swizzle), B = TOK tokens, tcgen05.mma kind::i8,
//                            one int32 accumulator per K block in tensor memory (a ring of them); the four epilogue
//                            warps pull each finished block, scale it and add it to fp32 registers
// Difference to the reference, inside the parity tolerance: the running output is kept in fp32, where the reference
// rounds it to bf16 after every K block.
//
// Work split: one output tile (128 features x TOK tokens, TOK = 16, 32, 64 or, for more than 64 tokens, 128) per CTA;
// when tiles are few, a thread-block cluster per tile cuts K between its CTAs, which add their parts over distributed
// shared memory.
#include "tpx_tc_ptx.cuh"

namespace tpx {

constexpr int kI8MaxStages = 8;

struct I8Params {
  TcParams t;          // epilogue fields (bias, act, mul_in, res, res_scale, y, M, N, err, cluster)
  const float* swT;    // [K/B][Np] weight scales, feature-contiguous
  const float* sx;     // [K/B][TOKP] activation scales
  int ksteps;          // k steps of 128 (K padded)
  int bsteps;          // k32 steps per scale block (B / 32)
  int Np;              // features padded to 128
  int nblk;            // scale blocks of the real K (the k padding of the last step has none)
  int tilesN;          // feature tiles; CTA (or cluster) t works on feature tile t % tilesN, token tile t / tilesN
  int Mp;              // tokens padded to whole token tiles: row stride of sx
};

__device__ __forceinline__ void i8_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "  tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One thread per (token row of the padded tile, K block): scale = max|x| / 127 in double as the reference does
// (src/csrc/qtypes.cpp:153-197), q = clamp(rint(x / scale)).
__global__ void quantize_act_i8_kernel(const uint16_t* __restrict__ x, int M, int K, int Kp, int B, int TOKP, int8_t* __restrict__ xq,
                                       float* __restrict__ sx) {
  pdl_trigger();
  pdl_wait();
  const int nb = K / B;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= TOKP * nb) return;
  const int tok = idx / nb, blk = idx % nb;
  int8_t* dst = xq + (size_t)tok * Kp + (size_t)blk * B;
  if (tok >= M) {
    for (int i = 0; i < B; i += 16) *reinterpret_cast<uint4*>(dst + i) = make_uint4(0, 0, 0, 0);
    sx[(size_t)blk * TOKP + tok] = 0.0f;
    return;
  }
  const uint16_t* src = x + (size_t)tok * K + (size_t)blk * B;
  float amax = 0.0f;
  for (int i = 0; i < B; i += 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(src + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      amax = fmaxf(amax, fabsf(bf16_bits_to_f32((uint16_t)(w[j] & 0xffff))));
      amax = fmaxf(amax, fabsf(bf16_bits_to_f32((uint16_t)(w[j] >> 16))));
    }
  }
  const float scale = (float)((double)amax / 127.0);
  const float iscale = scale != 0.0f ? 1.0f / scale : 0.0f;
  for (int i = 0; i < B; i += 16) {
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; q++) {
      uint32_t word = 0;
#pragma unroll
      for (int e = 0; e < 4; e++) {
        float f = nearbyintf(bf16_bits_to_f32(src[i + 4 * q + e]) * iscale);
        f = fminf(fmaxf(f, -127.0f), 127.0f);
        word |= ((uint32_t)(uint8_t)(int8_t)(int)f) << (8 * e);
      }
      o[q] = word;
    }
    *reinterpret_cast<uint4*>(dst + i) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  sx[(size_t)blk * TOKP + tok] = scale;
}

// The same quantisation with one CTA per token row, vectorised, for blocks of up to 256 values, optionally behind an
// RMSNorm of the row (y = bf16(x * rsqrt(mean(x^2) + eps) * gamma), llama_rms_norm of the reference, rows of up to
// 8192 values then): eight consecutive values per thread, the B/8 threads of a block reduce its maximum with shuffles.
constexpr int kQaThreads = 256;
__global__ void __launch_bounds__(kQaThreads) quantize_act_i8_row_kernel(const uint16_t* __restrict__ x, const void* __restrict__ gamma,
                                                                         int gamma_f32, float eps, int M, int K, int Kp, int B, int TOKP,
                                                                         int8_t* __restrict__ xq, float* __restrict__ sx) {
  __shared__ float red[kQaThreads / 32];
  pdl_trigger();
  pdl_wait();
  const int tok = blockIdx.x;
  const int nv = K / 8;
  const int lanes = B / 8;  // threads per scale block: 8, 16 or 32
  const bool live = tok < M;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)tok * K);
  float inv = 1.0f;
  if (gamma && live) {
    float ss = 0.0f;
    for (int i = threadIdx.x; i < nv; i += kQaThreads) {
      const uint4 v = xr[i];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float a = bf16_bits_to_f32((uint16_t)(w[j] & 0xffff)), b = bf16_bits_to_f32((uint16_t)(w[j] >> 16));
        ss += a * a + b * b;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < kQaThreads / 32; w++) tot += red[w];
    inv = rsqrtf(tot / (float)K + eps);
  }
  for (int i0 = 0; i0 < nv; i0 += kQaThreads) {
    const int i = i0 + threadIdx.x;
    const bool in = i < nv;
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; j++) f[j] = 0.0f;
    if (in && live) {
      const uint4 v = xr[i];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        f[2 * j] = bf16_bits_to_f32((uint16_t)(w[j] & 0xffff));
        f[2 * j + 1] = bf16_bits_to_f32((uint16_t)(w[j] >> 16));
      }
      if (gamma) {
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
        for (int j = 0; j < 8; j++) f[j] = bf16_bits_to_f32(f32_to_bf16_bits(f[j] * inv * g[j]));
      }
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(f[j]));
    for (int o = 1; o < lanes; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = (float)((double)amax / 127.0);
    const float iscale = scale != 0.0f ? 1.0f / scale : 0.0f;
    uint32_t o2[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      uint32_t word = 0;
#pragma unroll
      for (int e = 0; e < 4; e++) {
        float q = nearbyintf(f[4 * h + e] * iscale);
        q = fminf(fmaxf(q, -127.0f), 127.0f);
        word |= ((uint32_t)(uint8_t)(int8_t)(int)q) << (8 * e);
      }
      o2[h] = word;
    }
    if (in) {
      *reinterpret_cast<uint2*>(xq + (size_t)tok * Kp + (size_t)i * 8) = make_uint2(o2[0], o2[1]);
      if ((i % lanes) == 0) sx[(size_t)(i / lanes) * TOKP + tok] = live ? scale : 0.0f;
    }
  }
}

// Interchange tensors of remap_and_quantize_qint8 (q [N/16][K/B][B/4][16][4], scales [N/16][K/B][16]) -> plain int8
// weight [Np][Kp] (zero padding) and feature-contiguous scales [K/B][Np].
__global__ void repack_qint8_tc_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales, int64_t N, int64_t K, int64_t B,
                                       int64_t Np, int64_t Kp, int8_t* __restrict__ wq, float* __restrict__ swT) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < Np * (Kp / 4)) {
    const int64_t n = idx / (Kp / 4), k = (idx % (Kp / 4)) * 4;
    uint32_t w = 0;
    if (n < N && k < K) w = *reinterpret_cast<const uint32_t*>(q + ((((n / 16) * (K / B) + k / B) * (B / 4) + (k % B) / 4) * 16 + (n % 16)) * 4);
    *reinterpret_cast<uint32_t*>(wq + n * Kp + k) = w;
  }
  const int64_t nb = K / B;
  if (idx < nb * Np) {
    const int64_t blk = idx / Np, n = idx % Np;
    swT[idx] = n < N ? scales[((n / 16) * nb + blk) * 16 + (n % 16)] : 0.0f;
  }
}

template <int TOK>
struct I8Cfg {
  static constexpr int A_BYTES = 128 * 128;   // 128 features x 128 k values
  static constexpr int B_BYTES = TOK * 128;   // TOK tokens x 128 k values
  static constexpr int STAGE_BYTES = (A_BYTES + B_BYTES + 1023) / 1024 * 1024;
  static constexpr int STAGES_FIT = (227 * 1024 - 3072) / STAGE_BYTES;   // as many stages as shared memory holds: the bytes in
  static constexpr int STAGES = STAGES_FIT > kI8MaxStages ? kI8MaxStages : STAGES_FIT;  // flight bound the stream, not the MMAs
  static constexpr int GROUP = TOK >= 128 ? 2 : 4;  // accumulators per group; a group (up to GROUP K blocks, 256 k values or one
                                                    // larger block) is handed to the epilogue per barrier round trip
  static constexpr int NBUF = 512 / TOK > 16 ? 16 : 512 / TOK;  // int32 accumulators (one per K block) in tensor memory
  // Draining a K block (tensor memory -> int32 -> * s_x * s_w -> fp32 sum) is a chain of dependent scalar instructions;
  // with one warp per 32-row quarter it, not the MMAs, bounds the kernel as soon as there are many tokens. Every quarter
  // has EPI_SPLIT warps, each owning TW = TOK / EPI_SPLIT tokens (columns) of the tile.
  static constexpr int EPI_SPLIT = TOK >= 64 ? 4 : TOK / 16;
  static constexpr int TW = TOK / EPI_SPLIT;
  static constexpr int THREADS = 64 + 128 * EPI_SPLIT;
  static constexpr int NGRP = NBUF / GROUP;
  static constexpr int TMEM_COLS = NBUF * TOK < 32 ? 32 : NBUF * TOK;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;
  static_assert(NBUF * TOK <= 512, "tensor memory");
  static_assert(128 * TOK * 4 <= STAGES * STAGE_BYTES, "the partial tile of a cluster member fits in the stages");
};

template <int TOK>
__global__ void __launch_bounds__(I8Cfg<TOK>::THREADS, 1)
qlinear_i8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, I8Params p) {
  using C = I8Cfg<TOK>;
  extern __shared__ unsigned char i8_smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[C::STAGES], bar_empty[C::STAGES];
  __shared__ __align__(8) unsigned long long d_full[C::NGRP], d_free[C::NGRP];
  __shared__ uint32_t tmem_holder;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (tc_smem_u32(i8_smem_raw) + 1023u) & ~1023u;
  const int csize = p.t.cluster;
  const int crank = csize > 1 ? (int)tc_cluster_rank() : 0;
  const int tile = (int)(blockIdx.x / csize) % p.tilesN;  // feature tile
  const int tm = (int)(blockIdx.x / csize) / p.tilesN;    // token tile
  // K range of this CTA in k steps, aligned to whole scale blocks
  const int align = p.bsteps > 4 ? p.bsteps / 4 : 1;  // k steps per scale block when a block spans several
  const int groups = p.ksteps / align;
  const int ks0 = (int)((long long)crank * groups / csize) * align, ks1 = (int)((long long)(crank + 1) * groups / csize) * align;
  const int nsteps = ks1 - ks0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; s++) {
      tc_mbar_init(tc_smem_u32(&bar_full[s]), 1);
      tc_mbar_init(tc_smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < C::NGRP; b++) {
      tc_mbar_init(tc_smem_u32(&d_full[b]), 1);
      tc_mbar_init(tc_smem_u32(&d_free[b]), 4 * C::EPI_SPLIT);
    }
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
  pdl_trigger();

  constexpr int TW = C::TW;
  float acc[TW];  // this thread's tokens of its feature row
#pragma unroll
  for (int i = 0; i < TW; i++) acc[i] = 0.0f;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      auto fetch_w = [&](int s, int ks) {
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        tc_mbar_expect_tx(tc_smem_u32(&bar_full[s]), C::A_BYTES + C::B_BYTES);
        tc_tma_2d(st, &tmW, ks * 128, tile * 128, tc_smem_u32(&bar_full[s]));
      };
      const int early = nsteps < C::STAGES ? nsteps : C::STAGES;
      for (int it = 0; it < early; it++) fetch_w(it, ks0 + it);  // weights do not depend on the quantisation kernel
      pdl_wait();
      for (int it = 0; it < nsteps; it++) {
        const int s = it % C::STAGES;
        if (it >= C::STAGES) {
          if (!tc_wait(tc_smem_u32(&bar_empty[s]), (uint32_t)((it / C::STAGES - 1) & 1))) { atomicExch(p.t.err, 2u); break; }
          fetch_w(s, ks0 + it);
        }
        tc_tma_2d(smem_base + (uint32_t)s * C::STAGE_BYTES + C::A_BYTES, &tmX, (ks0 + it) * 128, tm * TOK, tc_smem_u32(&bar_full[s]));
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // kind::i8: D = S32 (2), A = B = S8 (1), both K-major, N = TOK, M = 128
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TOK >> 3) << 17) | ((128u >> 4) << 24);
      int buf = 0, inblk = 0;  // accumulator in use, k32 steps already in the current scale block
      uint32_t free_phase = 0;  // bit g: parity to wait for on d_free[g]
      unsigned used = 0;        // bit g: group g has been handed out before
      const int nblocks = nsteps * 4 / p.bsteps;
      const int gsize = p.bsteps >= 8 ? 1 : (8 / p.bsteps < C::GROUP ? 8 / p.bsteps : C::GROUP);  // blocks per group: 256 k values, or one larger block
      int done_blocks = 0;
      for (int it = 0; it < nsteps; it++) {
        const int s = it % C::STAGES;
        if (!tc_wait(tc_smem_u32(&bar_full[s]), (uint32_t)((it / C::STAGES) & 1))) { atomicExch(p.t.err, 4u); break; }
        tc_fence_after();
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        bool dead = false;
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int grp = buf / C::GROUP;
          if (inblk == 0 && buf % C::GROUP == 0 && ((used >> grp) & 1u)) {  // a recycled group: the epilogue must have read it
            if (!tc_wait(tc_smem_u32(&d_free[grp]), (free_phase >> grp) & 1u)) { atomicExch(p.t.err, 3u); dead = true; break; }
            free_phase ^= 1u << grp;
            tc_fence_after();
          }
          i8_mma(tmem + buf * TOK, tc_smem_desc(st) + (uint64_t)(2 * j), tc_smem_desc(st + C::A_BYTES) + (uint64_t)(2 * j), idesc,
                 inblk == 0 ? 0u : 1u);
          if (++inblk == p.bsteps) {  // block complete
            inblk = 0;
            done_blocks++;
            if (buf % C::GROUP + 1 == gsize || done_blocks == nblocks) {
              // group complete: hand its accumulators to the epilogue. This one commit also tells that the stages the
              // group read are free again (the epilogue passes that on to the producer), so stages need none of their own.
              tc_commit(tc_smem_u32(&d_full[grp]));
              used |= 1u << grp;
              buf = (grp + 1) * C::GROUP % C::NBUF;
            } else {
              buf++;
            }
          }
        }
        if (dead) break;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue: thread = feature row of the tile
    const int sub = warp & 3;
    const uint32_t lane_base = ((uint32_t)(sub * 32)) << 16;
    const int row = sub * 32 + lane;
    const int n = tile * 128 + row;
    pdl_wait();
    const int nblocks = nsteps * 4 / p.bsteps;
    const int blk0 = ks0 * 4 / p.bsteps;
    uint32_t full_phase = 0;
    constexpr bool kPrefetchSx = TW * C::GROUP <= 128;  // activation scales of a whole group in registers
    const int cpart = (warp - 2) >> 2;                   // this warp's tokens: [cpart * TW, +TW) of the tile
    const int gsize = p.bsteps >= 8 ? 1 : (8 / p.bsteps < C::GROUP ? 8 / p.bsteps : C::GROUP);
    const float* sx_tile = p.sx + (size_t)tm * TOK + (size_t)cpart * TW;  // this warp's columns of sx [K/B][Mp]
    int b = 0, buf = 0;
    bool dead = false;
    while (b < nblocks && !dead) {
      const int grp = buf / C::GROUP;
      const int cnt = nblocks - b < gsize ? nblocks - b : gsize;
      // scales of the group's blocks are fetched before the wait (a block of pure k padding has none: zeros)
      float sw[C::GROUP];
      float sxg[kPrefetchSx ? C::GROUP : 1][kPrefetchSx ? TW : 1];
#pragma unroll
      for (int q = 0; q < C::GROUP; q++) {
        const int blk = blk0 + b + q;
        const bool real = q < cnt && blk < p.nblk;
        sw[q] = real ? p.swT[(size_t)blk * p.Np + n] : 0.0f;
        if (kPrefetchSx) {
          const float4* sxp = reinterpret_cast<const float4*>(sx_tile + (size_t)(real ? blk : 0) * p.Mp);
#pragma unroll
          for (int i = 0; i < TW / 4; i++) {
            const float4 v = sxp[i];
            sxg[q][4 * i] = v.x; sxg[q][4 * i + 1] = v.y; sxg[q][4 * i + 2] = v.z; sxg[q][4 * i + 3] = v.w;
          }
        }
      }
      if (!tc_wait(tc_smem_u32(&d_full[grp]), (full_phase >> grp) & 1u)) {
        if (lane == 0) atomicExch(p.t.err, 6u);
        dead = true;
        break;
      }
      full_phase ^= 1u << grp;
      tc_fence_after();
      if (sub == 0 && lane == 0 && cpart == 0) {  // the MMAs of this group are complete: the stages they read may be refilled
        const int it_lo = b * p.bsteps / 4, it_hi = (b + cnt) * p.bsteps / 4;
        for (int it = it_lo; it < it_hi; it++) tc_mbar_arrive(tc_smem_u32(&bar_empty[it % C::STAGES]));
      }
#pragma unroll
      for (int q = 0; q < C::GROUP; q++) {
        if (q < cnt) {
          const int blk = blk0 + b + q;
          const float4* sxp = reinterpret_cast<const float4*>(sx_tile + (size_t)(blk < p.nblk ? blk : 0) * p.Mp);
#pragma unroll
          for (int c0 = 0; c0 < TW; c0 += 16) {
            float sxc[16];
            if (!kPrefetchSx) {  // many tokens: the scales of 16 tokens at a time (they sit in L1 after the first warp's read)
#pragma unroll
              for (int i = 0; i < 4; i++) {
                const float4 v = sxp[c0 / 4 + i];
                sxc[4 * i] = v.x; sxc[4 * i + 1] = v.y; sxc[4 * i + 2] = v.z; sxc[4 * i + 3] = v.w;
              }
            }
            uint32_t d[16];
            tc_ld_x16(tmem + lane_base + (buf + q) * TOK + cpart * TW + c0, d);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 16; i++) acc[c0 + i] += (float)(int)d[i] * (kPrefetchSx ? sxg[q][c0 + i] : sxc[i]) * sw[q];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(tc_smem_u32(&d_free[grp]));
      b += cnt;
      buf = (grp + 1) * C::GROUP % C::NBUF;
    }
    if (csize == 1) {
#pragma unroll
      for (int c0 = 0; c0 < TW; c0 += 16) {
        float v[16], v2[16];
#pragma unroll
        for (int i = 0; i < 16; i++) { v[i] = acc[c0 + i]; v2[i] = 0.0f; }
        const int tok0 = tm * TOK + cpart * TW + c0;
        if (n < p.t.N && tok0 < p.t.M) tc_finish16<false>(p.t, tok0, n, v, v2);
      }
    } else {
      const uint32_t sp = smem_base + (uint32_t)((row * TOK + cpart * TW) * 4);
#pragma unroll
      for (int c0 = 0; c0 < TW; c0 += 4) tc_st_shared_f4(sp + c0 * 4, make_float4(acc[c0], acc[c0 + 1], acc[c0 + 2], acc[c0 + 3]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (csize > 1) {
    // every member's partial tile is in its own shared memory; 16-token chunks go round the members, each adds the
    // parts in rank order over distributed shared memory and finishes its chunks. Nobody leaves before all have read.
    tc_cluster_sync();
    if (warp >= 2 && warp < 6) {
      const int row = (warp & 3) * 32 + lane;
      const int n = tile * 128 + row;
#pragma unroll 1
      for (int c0 = crank * 16; c0 < TOK; c0 += 16 * csize) {
        float v[16], v2[16];
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = v2[i] = 0.0f;
        const uint32_t sp = smem_base + (uint32_t)((row * TOK + c0) * 4);
        tc_cluster_sum<4, 2>(sp, csize, v);
        if (n < p.t.N && tm * TOK + c0 < p.t.M) tc_finish16<false>(p.t, tm * TOK + c0, n, v, v2);
      }
    }
    tc_cluster_sync();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)C::TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------- host side
struct I8Plan {
  int tokp, ksteps, tiles, cluster, TM;  // tiles = feature tiles x token tiles
  int64_t Kp, Np, Mp;
  size_t off_xq, off_sx, total;
};

static I8Plan i8_plan(int64_t M, int64_t N, int64_t K, int64_t B) {
  I8Plan pl;
  pl.tokp = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  pl.TM = (int)((M + pl.tokp - 1) / pl.tokp);
  pl.Mp = (int64_t)pl.TM * pl.tokp;
  pl.Kp = (K + 127) / 128 * 128;
  pl.Np = (N + 127) / 128 * 128;
  pl.ksteps = (int)(pl.Kp / 128);
  pl.tiles = (int)(pl.Np / 128) * pl.TM;
  const int sms = sm_count();
  const int groups = (int)(B > 128 ? pl.ksteps / (B / 128) : pl.ksteps);  // units a cluster can cut K into
  int c = pl.tiles > 0 ? sms / pl.tiles : 1;
  if (c > 8) c = 8;
  if (c > groups) c = groups;
  pl.cluster = c < 1 ? 1 : c;
  size_t o = kTcCounterBytes;
  auto bump = [&](size_t bytes) { size_t r = o; o += (bytes + 1023) & ~(size_t)1023; return r; };
  pl.off_xq = bump((size_t)pl.Mp * pl.Kp);
  pl.off_sx = bump((size_t)(K / B) * pl.Mp * sizeof(float));
  pl.total = o;
  return pl;
}

template <int TOK>
static int i8_launch(const CUtensorMap& w, const CUtensorMap& x, I8Params p, int tiles, cudaStream_t st) {
  using C = I8Cfg<TOK>;
  static bool opted[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || !opted[dev]) {
    TPX_CUDA_OK(cudaFuncSetAttribute(qlinear_i8_kernel<TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    if (dev >= 0 && dev < 16) opted[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(C::THREADS);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  // the largest cluster size, from the planned one down, of which one cluster per tile can be resident at once
  static int fits[16][9] = {};
  int c = p.t.cluster;
  for (; c >= 2; c--) {
    int& f = fits[(dev >= 0 && dev < 16) ? dev : 0][c];
    if (f == 0) {
      attr[1].val.clusterDim.x = (unsigned)c;
      cfg.gridDim = dim3((unsigned)(tiles * c));
      cfg.numAttrs = 2;
      int n = 0;
      cudaError_t e = cudaOccupancyMaxActiveClusters(&n, qlinear_i8_kernel<TOK>, &cfg);
      if (e != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
      f = 1 + n;
    }
    if (f - 1 >= tiles) break;
  }
  if (c < 2) c = 1;
  p.t.cluster = c;
  attr[1].val.clusterDim.x = (unsigned)c;
  cfg.gridDim = dim3((unsigned)(tiles * c));
  cfg.numAttrs = c > 1 ? 2 : 1;
  count_launch();
  TPX_CUDA_OK(cudaLaunchKernelEx(&cfg, qlinear_i8_kernel<TOK>, w, x, p));
  return TPX_OK;
}

static int make_map_u8(CUtensorMap* m, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
  typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                         const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Fn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &ptr, 12000, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<Fn>(ptr);
  }
  TPX_REQUIRE(fn, TPX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {row_bytes, rows};
  cuuint64_t gstr[1] = {row_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TPX_REQUIRE(r == CUDA_SUCCESS, TPX_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (rows=%llu row_bytes=%llu box_rows=%u)", (int)r,
              (unsigned long long)rows, (unsigned long long)row_bytes, box_rows);
  return TPX_OK;
}

}  // namespace tpx

using namespace tpx;

extern "C" int tpx_tc_packed_bytes_qint8(int64_t N, int64_t K, int64_t block_size, size_t* wq_bytes, size_t* sw_bytes) {
  TPX_REQUIRE(N > 0 && K > 0 && N % 16 == 0 && block_size % 64 == 0 && K % block_size == 0, TPX_ERR_ARG,
              "tc_packed_bytes_qint8: needs N %% 16 == 0 and a block size that is a multiple of 64 dividing K");
  const int64_t Np = (N + 127) / 128 * 128, Kp = (K + 127) / 128 * 128;
  if (wq_bytes) *wq_bytes = (size_t)Np * Kp;
  if (sw_bytes) *sw_bytes = (size_t)(K / block_size) * Np * sizeof(float);
  return TPX_OK;
}

extern "C" int tpx_repack_qint8_tc(const int8_t* q, const float* scales, int64_t N, int64_t K, int64_t block_size, int8_t* wq, float* swT,
                                   void* stream) {
  TPX_REQUIRE(q && scales && wq && swT, TPX_ERR_ARG, "repack_qint8_tc: null pointer");
  TPX_REQUIRE(N % 16 == 0 && block_size % 64 == 0 && K % block_size == 0, TPX_ERR_ARG,
              "repack_qint8_tc: needs N %% 16 == 0 and a block size that is a multiple of 64 dividing K");
  const int64_t Np = (N + 127) / 128 * 128, Kp = (K + 127) / 128 * 128;
  const int64_t total = Np * (Kp / 4) > (K / block_size) * Np ? Np * (Kp / 4) : (K / block_size) * Np;
  repack_qint8_tc_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(q, scales, N, K, block_size, Np, Kp, wq, swT);
  TPX_LAUNCH_OK();
  return TPX_OK;
}

extern "C" size_t tpx_qlinear_qint8_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int64_t block_size) {
  if (M <= 0 || N <= 0 || K <= 0 || block_size <= 0) return 0;
  return i8_plan(M, N, K, block_size).total;
}

extern "C" int tpx_qlinear_qint8_tc(const int8_t* wq, const float* swT, const uint16_t* x, const void* gamma, int gamma_is_f32, float eps,
                                    int64_t M, int64_t N, int64_t K, int64_t block_size, int reuse_act, const uint16_t* bias, int act, const uint16_t* mul_in,
                                    const uint16_t* res, float res_scale, uint16_t* y, void* scratch, size_t scratch_bytes, void* stream) {
  TPX_REQUIRE(M >= 0 && N > 0 && K > 0, TPX_ERR_ARG, "qlinear_qint8_tc: bad shape");
  if (M == 0) return TPX_OK;
  TPX_REQUIRE(M <= (1 << 20), TPX_ERR_UNSUPPORTED, "qlinear_qint8_tc: at most 2^20 tokens per call (M=%ld)", (long)M);
  TPX_REQUIRE(wq && swT && x && y, TPX_ERR_ARG, "qlinear_qint8_tc: null pointer");
  TPX_REQUIRE(block_size == 64 || block_size == 128 || block_size == 256 || block_size == 512, TPX_ERR_UNSUPPORTED,
              "qlinear_qint8_tc: block size %ld not supported (64, 128, 256, 512)", (long)block_size);
  TPX_REQUIRE(N % 16 == 0 && K % block_size == 0, TPX_ERR_ARG, "qlinear_qint8_tc: needs N %% 16 == 0 and K %% block_size == 0");
  TPX_REQUIRE(act >= TPX_ACT_NONE && act <= TPX_ACT_RELU, TPX_ERR_ARG, "qlinear_qint8_tc: unknown activation %d", act);
  TPX_REQUIRE((((uintptr_t)wq | (uintptr_t)x | (uintptr_t)swT) & 15) == 0 && ((uintptr_t)scratch & 255) == 0, TPX_ERR_ARG,
              "qlinear_qint8_tc: misaligned pointer");
  I8Plan pl = i8_plan(M, N, K, block_size);
  TPX_REQUIRE(pl.Kp % block_size == 0, TPX_ERR_UNSUPPORTED, "qlinear_qint8_tc: K rounded up to 128 must stay a multiple of the block size");
  TPX_REQUIRE(scratch && scratch_bytes >= pl.total, TPX_ERR_SCRATCH, "qlinear_qint8_tc: scratch of %zu bytes needed, %zu given", pl.total,
              scratch_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  unsigned char* sc = reinterpret_cast<unsigned char*>(scratch);
  int8_t* xq = reinterpret_cast<int8_t*>(sc + pl.off_xq);
  float* sx = reinterpret_cast<float*>(sc + pl.off_sx);
  if (!reuse_act && pl.Kp != K) TPX_CUDA_OK(cudaMemsetAsync(xq, 0, (size_t)pl.Mp * pl.Kp, st));  // the k padding reads as zero
  TPX_REQUIRE(!gamma || (K <= 8192 && block_size <= 256 && ((uintptr_t)gamma & 15) == 0), TPX_ERR_UNSUPPORTED,
              "qlinear_qint8_tc: the fused RMSNorm takes rows of up to 8192 values, blocks of up to 256 and a 16-byte aligned gamma");
  if (!reuse_act && block_size <= 256) {
    TPX_CUDA_OK(launch_pdl(quantize_act_i8_row_kernel, dim3((unsigned)pl.Mp), dim3(kQaThreads), 0, st, x, gamma, gamma_is_f32, eps, (int)M,
                           (int)K, (int)pl.Kp, (int)block_size, (int)pl.Mp, xq, sx));
  } else if (!reuse_act) {
    const long long threads = (long long)pl.Mp * (K / block_size);
    TPX_CUDA_OK(launch_pdl(quantize_act_i8_kernel, dim3((unsigned)((threads + 127) / 128)), dim3(128), 0, st, x, (int)M, (int)K, (int)pl.Kp,
                           (int)block_size, (int)pl.Mp, xq, sx));
  }
  CUtensorMap mw, mx;
  int rc = make_map_u8(&mw, wq, (uint64_t)pl.Np, (uint64_t)pl.Kp, 128);
  if (rc) return rc;
  rc = make_map_u8(&mx, xq, (uint64_t)pl.Mp, (uint64_t)pl.Kp, (uint32_t)pl.tokp);
  if (rc) return rc;
  I8Params p = {};
  p.t.bias = bias; p.t.mul_in = mul_in; p.t.res = res; p.t.res_scale = res_scale; p.t.y = y; p.t.act = act;
  p.t.M = (int)M; p.t.N = (int)N; p.t.K = (int)K; p.t.cluster = pl.cluster;
  p.t.err = reinterpret_cast<unsigned*>(sc + kTcCounterBytes - 4);
  p.swT = swT; p.sx = sx; p.ksteps = pl.ksteps; p.bsteps = (int)(block_size / 32); p.Np = (int)pl.Np; p.nblk = (int)(K / block_size);
  p.tilesN = (int)(pl.Np / 128); p.Mp = (int)pl.Mp;
  switch (pl.tokp) {
    case 16: return i8_launch<16>(mw, mx, p, pl.tiles, st);
    case 32: return i8_launch<32>(mw, mx, p, pl.tiles, st);
    case 64: return i8_launch<64>(mw, mx, p, pl.tiles, st);
    default: return i8_launch<128>(mw, mx, p, pl.tiles, st);
  }
}


// ---------------------------------------------------------------- int8 weight -> bf16 matrix (many tokens)
// With many tokens the per-K-block drain of the int8 kernel (one pass over the accumulator per 64 to 512 k) costs more
// than the MMAs it serves (253 TOP/s at block 64), while the bf16 tensor-core kernel runs the same shapes at 1000-1170
// TFLOP/s: for more than 128 tokens the host unpacks the weight to bf16 (w = q * s, rounded once) into a transient
// buffer and runs tpx_linear_bf16_tc on it, i.e. weight-only arithmetic with bf16 activations (the reference's QINT8_EMU
// mode, src/csrc/qtypes.cpp:27, :928-930). One thread per 16 consecutive k of one output row.
namespace tpx {
__global__ void unpack_qint8_bf16_kernel(const int8_t* __restrict__ wq, const float* __restrict__ swT, long long N, long long K, long long Kp,
                                         long long Np, int block, uint16_t* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long per_row = K / 16;
  if (idx >= N * per_row) return;
  const long long n = idx / per_row, k = (idx % per_row) * 16;
  const uint4 q = *reinterpret_cast<const uint4*>(wq + n * Kp + k);
  const float s = swT[(k / block) * Np + n];  // block sizes are multiples of 16: one scale for the sixteen values
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  uint32_t o[8];
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const int a = (int)(int8_t)((w[j >> 1] >> (16 * (j & 1))) & 0xff), b = (int)(int8_t)((w[j >> 1] >> (16 * (j & 1) + 8)) & 0xff);
    o[j] = (uint32_t)f32_to_bf16_bits((float)a * s) | ((uint32_t)f32_to_bf16_bits((float)b * s) << 16);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + n * K + k);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}
}  // namespace tpx

extern "C" int tpx_unpack_qint8_tc_bf16(const int8_t* wq, const float* swT, int64_t N, int64_t K, int64_t block_size, uint16_t* w_bf16,
                                        void* stream) {
  TPX_REQUIRE(wq && swT && w_bf16, TPX_ERR_ARG, "unpack_qint8_tc_bf16: null pointer");
  TPX_REQUIRE(N > 0 && K > 0 && K % 16 == 0 && block_size >= 16 && block_size % 16 == 0 && K % block_size == 0, TPX_ERR_ARG,
              "unpack_qint8_tc_bf16: bad shape (N=%ld K=%ld block=%ld)", (long)N, (long)K, (long)block_size);
  TPX_REQUIRE((((uintptr_t)wq | (uintptr_t)w_bf16) & 15) == 0, TPX_ERR_ARG, "unpack_qint8_tc_bf16: misaligned pointer");
  const long long Kp = (K + 127) / 128 * 128, Np = (N + 127) / 128 * 128;
  const long long total = N * (K / 16);
  TPX_CUDA_OK(tpx::launch_pdl(tpx::unpack_qint8_bf16_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, wq, swT,
                              (long long)N, (long long)K, Kp, Np, (int)block_size, w_bf16));
  return TPX_OK;
}
