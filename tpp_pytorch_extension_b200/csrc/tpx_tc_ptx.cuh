// Inline PTX wrappers and shared parameter block of the tensor-core (tcgen05 + TMA) linear kernels.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdlib.h>

#include "tpx_common.cuh"

namespace tpx {

constexpr unsigned kTcSpinLimit = 1u << 22;
constexpr int kTcThreads = 192;
constexpr size_t kTcCounterBytes = 64 * 1024;  // arrival counters (one per output tile) + error word at the end

// Where the epilogue of one linear puts its output as the activation terms of the linear that consumes it (the layout
// split_activations_kernel would produce from the bf16 output): the consumer then starts without a split kernel of its
// own. TOK, UKS, KS and rowmap are the consumer's split parameters. terms == nullptr: nothing is emitted.
struct TcEmit {
  uint8_t* terms;
  uint8_t* sfb;
  int TOK, UKS, KS, rowmap;
};

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
  int KS;               // k units (of UKS k steps of 128) per tile
  int TN, TM;           // output tiles along features / tokens
  int act;
  int whole_tiles;      // 1: every CTA owns whole output tiles (no partial tiles, no fix-up)
  unsigned long long* tl;  // optional per-CTA timeline (8 globaltimer stamps each), null in normal use
  int cluster;          // CTAs per thread-block cluster that share one output tile along K (1: none)
  int pf;               // units prefetched into L2 ahead of the shared-memory stages
  TcEmit emit;          // optional hand-over of the output to the next linear (decode-shaped gate/up launches)
  int wfmt;             // weight operand of the 128-row kernel: 0 = packed E2M1 (unpacked by the copy), 1 = E4M3 bytes, 2 = E5M2 bytes
  int dbg;              // timing-experiment knobs, honoured only by a -DTPX_DEBUG build (results are then wrong): 1 = skip MMAs,
                        // 2 = skip weight copies, 128 = skip activation copies; packed-fp4 kernel: 16 = skip scale-factor
                        // copies, 32 = MMA thread issues them
};

// The default build compiles the experiment knobs and the timeline stamps out: TPX_DBG(p) is the constant 0 there.
#ifdef TPX_DEBUG
#define TPX_DBG(p) ((p).dbg)
__device__ __forceinline__ void tc_stamp(const TcParams& p, int slot) {
  if (p.tl) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.tl[(size_t)blockIdx.x * 8 + slot] = t;
  }
}
#else
#define TPX_DBG(p) 0
__device__ __forceinline__ void tc_stamp(const TcParams&, int) {}
#endif

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
// thread-block cluster helpers (split-K partners reduce through distributed shared memory)
__device__ __forceinline__ uint32_t tc_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void tc_cluster_sync() {  // every thread of every CTA of the cluster
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t tc_mapa(uint32_t saddr, uint32_t rank) {  // the same offset in CTA `rank` of the cluster
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 tc_ld_cluster_f4(uint32_t caddr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(caddr) : "memory");
  return v;
}
// acc[4 * NV] += the NV consecutive float4 at shared-memory offset saddr of every cluster member, members in rank order
// (the sum every thread computes is the same whatever the batching). The loads of BATCH members are issued together
// and added afterwards: issued one member at a time with the adds in between, every member cost a full round trip over
// the cluster's shared-memory network (a cluster of 8: 3 us for the down projection at one token, 5.7 us at 16).
template <int NV, int BATCH>
__device__ __forceinline__ void tc_cluster_sum(uint32_t saddr, int cluster, float (&acc)[4 * NV]) {
#pragma unroll
  for (int m0 = 0; m0 < 8; m0 += BATCH) {
    if (m0 < cluster) {
      float4 t[BATCH][NV];
#pragma unroll
      for (int j = 0; j < BATCH; j++) {
        if (m0 + j < cluster) {
          const uint32_t rp = tc_mapa(saddr, (uint32_t)(m0 + j));
#pragma unroll
          for (int q = 0; q < NV; q++) t[j][q] = tc_ld_cluster_f4(rp + q * 16);
        }
      }
#pragma unroll
      for (int j = 0; j < BATCH; j++) {
        if (m0 + j < cluster) {
#pragma unroll
          for (int q = 0; q < NV; q++) {
            acc[4 * q] += t[j][q].x; acc[4 * q + 1] += t[j][q].y; acc[4 * q + 2] += t[j][q].z; acc[4 * q + 3] += t[j][q].w;
          }
        }
      }
    }
  }
}
__device__ __forceinline__ void tc_st_shared_f4(uint32_t saddr, float4 v) {
  asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(saddr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// L2 prefetches: no shared memory is tied up while the data travels from HBM
__device__ __forceinline__ void tc_prefetch_2d(const CUtensorMap* map, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_prefetch_bulk(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
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
// Both operands packed E2M1 (two codes per byte in shared memory), K = 64 per instruction, one UE8M0 scale per 32 k:
// the instruction reads two consecutive scale bytes per row, selected by scale-factor id 0 or 2.
__device__ __forceinline__ void tc_mma_f4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                          uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "  tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p; }" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
// 32 rows x 16 bytes, rows 16 bytes apart, no swizzle: 8-row core matrices 128 bytes apart.
__device__ __forceinline__ uint64_t tc_sf_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) | (1ull << 46);
}
// shared -> tensor memory: 32 lanes x 128 bits, replicated to the four 32-lane quarters
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
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

// K-major operand tile of 64-byte rows (128 packed 4-bit codes), 64-byte swizzle: 8-row groups are 512 bytes apart.
__device__ __forceinline__ uint64_t tc_smem_desc64(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(512 >> 4) << 32) | (1ull << 46) | (4ull << 61);
}

// The same tile read with its 8-row groups `sbo` bytes apart instead of 1024: consecutive groups then overlap in
// memory (group g starts at row g * sbo / 128). Swizzling acts on address bits, so rows written by a plain swizzled
// copy are read back consistently.
__device__ __forceinline__ uint64_t tc_smem_desc_sbo(uint32_t saddr, uint32_t sbo) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Epilogue of 16 consecutive tokens of one output feature n: bias, activation, gate multiply, residual, bf16 store.
// ---- hand-over of an output to the next linear as activation terms (TcEmit)
// Address of the first byte of 32-block kb of token tok in the hi and the lo term, and of its two scale bytes.
struct TcEmitAddr {
  uint8_t *hi, *lo, *sh, *sl;
};
__device__ __forceinline__ TcEmitAddr tc_emit_addr(const TcEmit& E, int tok, int kb) {
  const int tm = tok / E.TOK, r = tok % E.TOK, ks = kb >> 2, j = kb & 3;
  const size_t step = (size_t)tm * E.KS + ks;
  int rh, rl, gh, gl;
  size_t blk_off;
  if (E.rowmap == 1) {
    rh = gh = 32 * (r / 16) + (r % 16);
    rl = gl = rh + 16;
    blk_off = step * 512;
  } else if (E.rowmap == 2) {
    rh = 8 * (r / 4) + (r % 4);
    rl = rh + 4;
    gh = 32 * (r / 4) + (r % 4);
    gl = gh + 16;
    blk_off = step * 512;
  } else {
    rh = gh = r;
    rl = gl = E.TOK + r;
    blk_off = step * (size_t)((2 * E.TOK + 127) / 128) * 512;
  }
  TcEmitAddr a;
  a.hi = E.terms + (step * 2 * E.TOK + rh) * 128 + j * 32;
  a.lo = E.terms + (step * 2 * E.TOK + rl) * 128 + j * 32;
  uint8_t* blk = E.sfb + blk_off;
  a.sh = blk + (gh / 128) * 512 + (gh % 32) * 16 + ((gh % 128) / 32) * 4 + j;
  a.sl = blk + (gl / 128) * 512 + (gl % 32) * 16 + ((gl % 128) / 32) * 4 + j;
  return a;
}
// Block exponent of the split (block maximum to [128, 256): E4M3 holds up to 448) from the maximum's bit pattern.
__device__ __forceinline__ int tc_emit_exp(uint32_t amax_bits) {
  int e = 0;
  if (amax_bits > 0u && amax_bits < 0x7f800000u) e = (int)((amax_bits >> 23) & 0xff) - 127 - 7;
  return max(-127, min(127, e));
}
// Two values -> their hi and lo E4M3 bytes (low byte = first value), scaled by `down` = 2^-e.
__device__ __forceinline__ void tc_emit_cvt2(float a, float b, float down, uint32_t& hi, uint32_t& lo) {
  a *= down;
  b *= down;
  __nv_fp8x2_storage_t hs = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(hs, __NV_E4M3);
  float ra = a - __half2float(__ushort_as_half(hr.x)), rb = b - __half2float(__ushort_as_half(hr.y));
  __nv_fp8x2_storage_t ls = __nv_cvt_float2_to_fp8x2(make_float2(ra, rb), __NV_SATFINITE, __NV_E4M3);
  hi = (uint32_t)hs;
  lo = (uint32_t)ls;
}
// A warp whose lane l holds output feature n0 + l (n0 a multiple of 32) of 16 consecutive tokens: one 32-block per
// token. xr: the outputs as stored (rounded to bf16). Called by all 32 lanes.
__device__ __forceinline__ void tc_emit16_lanes(const TcEmit& E, int tok0, int live, int n, const float (&xr)[16]) {
  const int lane = n & 31, kb = n >> 5;
#pragma unroll
  for (int j = 0; j < 16; j++) {
    if (j < live) {
      const uint32_t amax = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(xr[j])));
      const int e = tc_emit_exp(amax);
      const float down = __uint_as_float((uint32_t)(127 - e) << 23);
      uint32_t hi, lo;
      tc_emit_cvt2(xr[j], 0.0f, down, hi, lo);
      const TcEmitAddr a = tc_emit_addr(E, tok0 + j, kb);
      a.hi[lane] = (uint8_t)hi;
      a.lo[lane] = (uint8_t)lo;
      if (lane == 0) {
        *a.sh = (uint8_t)(e + 127);
        *a.sl = (uint8_t)(e + 127);
      }
    }
  }
}

// Straight-line code over the 16 tokens (loads first, then arithmetic, then stores) so that the tokens' dependent
// chains overlap; only the loads and stores are predicated on the token being inside M.
template <bool DUAL>
__device__ __forceinline__ void tc_finish16(const TcParams& p, int tok0, int n, const float (&v)[16], const float (&v2)[16],
                                            float* stored = nullptr) {
  const int live = p.M - tok0;  // tokens tok0 .. tok0+live-1 exist
  const size_t o0 = (size_t)tok0 * p.N + n;
  const float b = p.bias ? bf16_bits_to_f32(p.bias[n]) : 0.0f;
  float x[16];
#pragma unroll
  for (int j = 0; j < 16; j++) x[j] = v[j] + b;
  switch (p.act) {
    case TPX_ACT_GELU:
#pragma unroll
      for (int j = 0; j < 16; j++) x[j] = 0.5f * x[j] * (1.0f + erff(x[j] * 0.70710678118654752f));
      break;
    case TPX_ACT_SILU:
#pragma unroll
      for (int j = 0; j < 16; j++) x[j] = __fdividef(x[j], 1.0f + __expf(-x[j]));
      break;
    case TPX_ACT_RELU:
#pragma unroll
      for (int j = 0; j < 16; j++) x[j] = fmaxf(x[j], 0.0f);
      break;
    default: break;
  }
  if (DUAL) {
#pragma unroll
    for (int j = 0; j < 16; j++) x[j] *= v2[j];
  }
  if (p.mul_in) {
    uint16_t t[16];
#pragma unroll
    for (int j = 0; j < 16; j++) t[j] = j < live ? p.mul_in[o0 + (size_t)j * p.N] : (uint16_t)0;
#pragma unroll
    for (int j = 0; j < 16; j++) x[j] *= bf16_bits_to_f32(t[j]);
  }
  if (p.res) {
    uint16_t t[16];
#pragma unroll
    for (int j = 0; j < 16; j++) t[j] = j < live ? p.res[o0 + (size_t)j * p.N] : (uint16_t)0;
#pragma unroll
    for (int j = 0; j < 16; j++) x[j] += bf16_bits_to_f32(t[j]) * p.res_scale;
  }
#pragma unroll
  for (int j = 0; j < 16; j++) {
    const uint16_t bits = f32_to_bf16_bits(x[j]);
    if (j < live) p.y[o0 + (size_t)j * p.N] = bits;
    if (stored) stored[j] = bf16_bits_to_f32(bits);
  }
}

// Epilogue of the many-token kernels: 16 consecutive tokens of output feature n from the accumulator values x (gate/up
// pair: u holds the up values), with the residual / gate-input values loaded beforehand (tc_preload16, while the MMAs ran):
// bias, activation, gate multiply, residual, bf16 stores; residual / gate inputs arrive packed two per register.
template <bool DUAL>
__device__ __forceinline__ void tc_finish16_pre(const TcParams& p, int tok0, int n, float (&x)[16], float (&u)[16],
                                            const uint32_t (&resp)[8], const uint32_t (&mulp)[8], const float* __restrict__ tok_scale) {
  const int live = p.M - tok0;
  const size_t o0 = (size_t)tok0 * p.N + n;
  if (tok_scale) {  // the activations were split as x / 2^e per token: give the 2^e back (the array is padded to whole tiles)
    const float4* sp = reinterpret_cast<const float4*>(tok_scale + tok0);
    const float4 s0 = __ldg(sp), s1 = __ldg(sp + 1), s2 = __ldg(sp + 2), s3 = __ldg(sp + 3);
    const float sc[16] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w, s2.x, s2.y, s2.z, s2.w, s3.x, s3.y, s3.z, s3.w};
#pragma unroll
    for (int j = 0; j < 16; j++) {
      x[j] *= sc[j];
      if (DUAL) u[j] *= sc[j];
    }
  }
  if (p.bias) {
    const float b = bf16_bits_to_f32(p.bias[n]);
#pragma unroll
    for (int j = 0; j < 16; j++) x[j] += b;
  }
  switch (p.act) {
    case TPX_ACT_GELU:
#pragma unroll
      for (int j = 0; j < 16; j++) x[j] = 0.5f * x[j] * (1.0f + erff(x[j] * 0.70710678118654752f));
      break;
    case TPX_ACT_SILU:
#pragma unroll
      for (int j = 0; j < 16; j++) x[j] = __fdividef(x[j], 1.0f + __expf(-x[j]));
      break;
    case TPX_ACT_RELU:
#pragma unroll
      for (int j = 0; j < 16; j++) x[j] = fmaxf(x[j], 0.0f);
      break;
    default: break;
  }
  if (DUAL) {
#pragma unroll
    for (int j = 0; j < 16; j++) x[j] *= u[j];
  }
  if (p.mul_in) {
#pragma unroll
    for (int j = 0; j < 16; j++) x[j] *= bf16_bits_to_f32((uint16_t)(mulp[j >> 1] >> (16 * (j & 1))));
  }
  if (p.res) {
#pragma unroll
    for (int j = 0; j < 16; j++) x[j] += bf16_bits_to_f32((uint16_t)(resp[j >> 1] >> (16 * (j & 1)))) * p.res_scale;
  }
#pragma unroll
  for (int j = 0; j < 16; j++)
    if (j < live) p.y[o0 + (size_t)j * p.N] = f32_to_bf16_bits(x[j]);
}

__device__ __forceinline__ void tc_preload16(const uint16_t* __restrict__ src, int M, int N, int tok0, int n, uint32_t (&pk)[8]) {
  const int live = M - tok0;
  const uint16_t* s = src + (size_t)tok0 * N + n;
  uint16_t t[16];
#pragma unroll
  for (int j = 0; j < 16; j++) t[j] = j < live ? __ldg(s + (size_t)j * N) : (uint16_t)0;
#pragma unroll
  for (int j = 0; j < 8; j++) pk[j] = (uint32_t)t[2 * j] | ((uint32_t)t[2 * j + 1] << 16);
}

// host helpers shared by the tensor-core linears
int tc_make_map(CUtensorMap* m, CUtensorMapDataType dt, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows);
int tc_make_map64(CUtensorMap* m, const void* base, uint64_t rows, uint32_t box_rows);
int tc_make_map_sf(CUtensorMap* m, const void* base, uint64_t rows, uint32_t box_rows);
int tc_padded_ks(int64_t K, bool pair);
struct TcNorm {  // optional RMSNorm applied to x on its way into the split (null gamma: none)
  const void* gamma;
  int gamma_f32;
  float eps;
  const TcEmit* pre = nullptr;  // the activation terms are already there (the previous linear's epilogue wrote them): no split
};
// Hand-over between two decode-shaped linears (at most 64 tokens), used by the layer calls. tc_handoff_plan fills E
// with the split layout of the consumer y[M][N] = x[M][K] (one weight) inside buf, or leaves E->terms null when
// that consumer's kernel takes another layout or K is padded. tc_set_emit: the next tpx_*_qlinear_mxfp4_tc call of this
// host thread also writes its output as those terms if its kernel can (tc_emitted() tells); tc_set_pre: the next call
// reads its activation from them instead of splitting x.
int tc_handoff_plan(int64_t M, int64_t N, int64_t K, void* buf, size_t bytes, TcEmit* E);
void tc_set_emit(const TcEmit& E);
void tc_set_pre(const TcEmit& E);
bool tc_emitted();
void tc_note_emitted(bool v);
bool tcw_handoff_layout(int64_t M, int64_t N, int64_t K, TcEmit* E, size_t* terms_bytes, size_t* sfb_bytes);
int tc_launch_split(const uint16_t* x, int M, int K, int Mpad, int KS, int TOK, int UKS, int rowmap, uint8_t* terms, uint8_t* sfb,
                    cudaStream_t st, const TcNorm* norm = nullptr);
int tc_launch_fixup(bool dual, const TcParams& p, int TOK, int grid, cudaStream_t st);
// packed-fp4 variant for up to 32 tokens (activations as four E2M1 terms): tpx_qlinear_tc4.cu
size_t tc4_scratch_bytes(int64_t M, int64_t N, int64_t K, bool pair);
int tc4_run(const uint8_t* wq, const uint8_t* sfa, bool pair, const uint16_t* x, int64_t M, int64_t N, int64_t K, const TcParams& base,
            void* scratch, size_t scratch_bytes, cudaStream_t st, const TcNorm* norm = nullptr);
// decode-shaped variant (tokens on the M side of the MMA): tpx_qlinear_tcw.cu
size_t tcw_scratch_bytes(int64_t M, int64_t N, int64_t K, bool pair);
int tcw_run(const uint8_t* wq, const uint8_t* sfa, bool pair, const uint16_t* x, int64_t M, int64_t N, int64_t K, const TcParams& base,
            void* scratch, size_t scratch_bytes, cudaStream_t st, const TcNorm* norm = nullptr);
// weights on the N side, packed-fp4 operands, up to 64 tokens (up to 8 without an activation kernel): tpx_qlinear_tcw4.cu
bool tcw4_serves(int64_t M, int64_t N, int64_t K, bool pair);
size_t tcw4_scratch_bytes(int64_t M, int64_t N, int64_t K, bool pair);
int tcw4_run(const uint8_t* wq, const uint8_t* sfa, bool pair, const uint16_t* x, int64_t M, int64_t N, int64_t K, const TcParams& base,
             void* scratch, size_t scratch_bytes, cudaStream_t st, const TcNorm* norm = nullptr);
// many tokens, whole tiles of 128 x 128, three accumulators (the epilogue overlaps the next tile): tpx_qlinear_tcp.cu
bool tcp_serves(int64_t M, int64_t N, int64_t K, bool pair);
size_t tcp_scratch_bytes(int64_t M, int64_t N, int64_t K, bool pair);
int tcp_run(const uint8_t* wq, const uint8_t* sfa, bool pair, const uint16_t* x, int64_t M, int64_t N, int64_t K, const TcParams& base,
            void* scratch, size_t scratch_bytes, cudaStream_t st, const TcNorm* norm = nullptr);
// the same on CTA pairs (tcgen05.mma.cta_group::2, each CTA holds half of the activation operand): tpx_qlinear_tcp2.cu
bool tcp2_serves(int64_t M, int64_t N, int64_t K, bool pair);
size_t tcp2_scratch_bytes(int64_t M, int64_t N, int64_t K, bool pair);
int tcp2_run(const uint8_t* wq, const uint8_t* sfa, bool pair, const uint16_t* x, int64_t M, int64_t N, int64_t K, const TcParams& base,
             void* scratch, size_t scratch_bytes, cudaStream_t st, const TcNorm* norm = nullptr);
}  // namespace tpx
