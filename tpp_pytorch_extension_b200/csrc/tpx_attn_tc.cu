// Prefill attention on the 5th-generation tensor cores: tcgen05.mma with accumulators in tensor memory, K/V tiles by TMA.
//
// Replaces attn<T> of the reference (src/csrc/llm/attn.cpp:780-955) for many query rows per (batch, kv head): the
// flash-attention loop of the reference (scores of a key chunk, running max and sum, rescaled output; VarSoftMaxFwdTPP,
// SoftMaxFixUpTPP, SoftMaxFlashScaleTPP of src/csrc/xsmm_functors.h:4123-4566) with both contractions on tcgen05:
//   S = Q.K^T   A = 128 query rows (K-major, H along k), B = 128 keys (K-major), D = 128 fp32 columns of tensor memory
//   T = P.V     A = P in tensor memory (bf16, written by the softmax warps), B = 128 keys x H values read MN-major
//               (the cache keeps H contiguous), D = H fp32 columns
// One CTA owns 128 consecutive query rows ((query position, group member) pairs) of one (batch, kv head) and walks the
// keys in tiles of 128 = four 32-token cache blocks, fetched by one 4-D TMA request per operand half.
//   warp 0   : TMA producer (Q once, then K and V tiles into two stages)
//   warp 1   : allocates tensor memory, issues the MMAs: S of tile j+1 is issued before P.V of tile j, so the tensor
//              core computes the next scores while the softmax warps work on the current ones
//   warps 2-17: softmax and output, four warps per 32-row quarter of tensor memory (a thread holds 32 keys and H/4 output
//              columns of one row): masks, running max / sum (the quarter's warps exchange their maxima through shared
//              memory), P = exp(S - max) as bf16 into tensor memory, and the output accumulation o = o * alpha + T in
//              registers (the tile product is not accumulated in tensor memory, so no rescaling pass over it is
//              needed). Sixteen warps because this part is a chain of dependent scalar instructions: with one warp per
//              scheduler it ran at a fraction of the issue rate.
// Scores and T are double / single buffered in tensor memory: S0, S1 (128 columns each), P0, P1 (64 each), T (H).
#include "tpx_attn.cuh"
#include "tpx_tc_ptx.cuh"

namespace tpx {

static __device__ unsigned g_attn_tc_err;  // set when a bounded wait gave up; read and cleared by tpx_attention_tc_status

template <int H>
struct AtCfg {
  static constexpr int HALVES = H / 64;                 // 64-element (128-byte) slabs along the head dimension
  static constexpr int HALF_BYTES = 128 * 128;          // 128 rows x 128 bytes
  static constexpr int Q_BYTES = HALVES * HALF_BYTES;
  static constexpr int KV_BYTES = HALVES * HALF_BYTES;  // one tile of keys, or of values
  static constexpr int STAGE_BYTES = 2 * KV_BYTES;
  static constexpr int STAGES = 2;
  static constexpr size_t SMEM = Q_BYTES + STAGES * STAGE_BYTES + 1024;
  static constexpr uint32_t COL_S = 0, COL_P = 256, COL_T = 384;
  static_assert(COL_T + H <= 512, "tensor memory");
};

__device__ __forceinline__ void at_tma_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
// A from shared memory (descriptor) or from tensor memory (address)
__device__ __forceinline__ void at_mma_ss(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0;\n  tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d), "l"(adesc),
               "l"(bdesc), "r"(idesc), "r"(acc)
               : "memory");
}
__device__ __forceinline__ void at_mma_ts(uint32_t d, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0;\n  tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }" ::"r"(d), "r"(a_tmem),
               "l"(bdesc), "r"(idesc), "r"(acc)
               : "memory");
}
// MN-major operand (the contiguous dimension is the MMA's N, here the head dimension), 128-byte swizzle: rows of 128 bytes
// are consecutive k (keys), 8-key groups 1024 bytes apart, the next 64 values of the head dimension `lbo` bytes further.
__device__ __forceinline__ uint64_t at_desc_mn(uint32_t saddr, uint32_t lbo) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void at_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void at_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr), "r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
      "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ float at_ex2(float x) {  // 2^x on the special-function unit; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t at_pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int kAtThreads = 64 + 512;  // producer warp, MMA warp, sixteen softmax warps

template <int H>
__global__ void __launch_bounds__(kAtThreads, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
               AttnParams p) {
  using C = AtCfg<H>;
  extern __shared__ unsigned char at_smem_raw[];
  __shared__ __align__(8) unsigned long long q_full, kv_full[2], kv_empty[2], s_full[2], p_full[2], o_full, o_free;
  __shared__ uint32_t tmem_holder;
  __shared__ float xmax[2][4][128];  // per tile parity: the four key ranges' maxima of every row (then once the row sums)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (tc_smem_u32(at_smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = smem_base, kv_s = smem_base + C::Q_BYTES;

  const int bn = blockIdx.x;
  const int chunk = (int)gridDim.y - 1 - (int)blockIdx.y;  // the chunks with the most keys (causal) start first
  const int b = bn / p.Nkv;
  const int rows_total = p.Sq * p.R;
  const int row0 = chunk * 128;

  if (threadIdx.x == 0) {
    tc_mbar_init(tc_smem_u32(&q_full), 1);
    for (int s = 0; s < 2; s++) {
      tc_mbar_init(tc_smem_u32(&kv_full[s]), 1);
      tc_mbar_init(tc_smem_u32(&kv_empty[s]), 1);
      tc_mbar_init(tc_smem_u32(&s_full[s]), 1);
      tc_mbar_init(tc_smem_u32(&p_full[s]), kAtThreads - 64);
    }
    tc_mbar_init(tc_smem_u32(&o_full), 1);
    tc_mbar_init(tc_smem_u32(&o_free), kAtThreads - 64);
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
  pdl_trigger();
  pdl_wait();  // q and the cache were written by earlier grids

  const int key_len = p.dev_len ? *p.dev_len + p.Sq : p.key_len;
  const int offset = key_len - p.Sq;
  const int cta_last_row = min(rows_total, row0 + 128) - 1;
  const int kmax = p.causal ? min(key_len, offset + cta_last_row / p.R + 1) : key_len;
  const int ntiles = (kmax + 127) / 128;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      tc_mbar_expect_tx(tc_smem_u32(&q_full), C::Q_BYTES);
#pragma unroll
      for (int h = 0; h < C::HALVES; h++) tc_tma_2d(q_s + h * C::HALF_BYTES, &tmQ, h * 64, bn * rows_total + row0, tc_smem_u32(&q_full));
      for (int j = 0; j < ntiles; j++) {
        const int s = j & 1;
        if (j >= 2 && !tc_wait(tc_smem_u32(&kv_empty[s]), (uint32_t)(((j >> 1) - 1) & 1))) { atomicExch(&g_attn_tc_err, 2u); break; }
        const uint32_t st = kv_s + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t bar = tc_smem_u32(&kv_full[s]);
        tc_mbar_expect_tx(bar, C::STAGE_BYTES);
#pragma unroll
        for (int h = 0; h < C::HALVES; h++) {  // 64 values x 32 slots x 1 (batch, head) x 4 cache blocks = 128 keys x 128 bytes
          at_tma_4d(st + h * C::HALF_BYTES, &tmK, h * 64, 0, bn, j * 4, bar);
          at_tma_4d(st + C::KV_BYTES + h * C::HALF_BYTES, &tmV, h * 64, 0, bn, j * 4, bar);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
      const uint32_t idesc_t = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(H >> 3) << 17) | ((128u >> 4) << 24);
      bool ok = tc_wait(tc_smem_u32(&q_full), 0);
      if (!ok) atomicExch(&g_attn_tc_err, 3u);
      auto issue_s = [&](int j) -> bool {  // S_j = Q.K_j^T into score buffer j & 1
        const int s = j & 1;
        if (!tc_wait(tc_smem_u32(&kv_full[s]), (uint32_t)((j >> 1) & 1))) { atomicExch(&g_attn_tc_err, 4u); return false; }
        tc_fence_after();
        const uint32_t ks = kv_s + (uint32_t)s * C::STAGE_BYTES;
#pragma unroll
        for (int kk = 0; kk < H / 16; kk++) {
          const uint32_t koff = (uint32_t)(kk >> 2) * C::HALF_BYTES + (uint32_t)(kk & 3) * 32;
          at_mma_ss(tmem + C::COL_S + s * 128, tc_smem_desc(q_s + koff), tc_smem_desc(ks + koff), idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(tc_smem_u32(&s_full[s]));
        return true;
      };
      if (ok && ntiles > 0) ok = issue_s(0);
      for (int j = 0; ok && j < ntiles; j++) {
        const int s = j & 1;
        if (j + 1 < ntiles && !issue_s(j + 1)) break;
        if (!tc_wait(tc_smem_u32(&p_full[s]), (uint32_t)((j >> 1) & 1))) { atomicExch(&g_attn_tc_err, 5u); break; }
        if (j > 0 && !tc_wait(tc_smem_u32(&o_free), (uint32_t)((j - 1) & 1))) { atomicExch(&g_attn_tc_err, 6u); break; }
        tc_fence_after();
        const uint32_t vs = kv_s + (uint32_t)s * C::STAGE_BYTES + C::KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < 8; kk++)  // 16 keys per MMA: 8 columns of packed bf16 probabilities, two 8-key groups of values
          at_mma_ts(tmem + C::COL_T, tmem + C::COL_P + s * 64 + kk * 8, at_desc_mn(vs + kk * 2048, C::HALF_BYTES), idesc_t, kk > 0 ? 1u : 0u);
        tc_commit(tc_smem_u32(&o_full));
        tc_commit(tc_smem_u32(&kv_empty[s]));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ softmax and output: sixteen warps, four per 32-row quarter
    // of tensor memory; the four warps of a quarter share its rows: warp `part` takes keys [32*part, +32) of every tile
    // and columns [HP*part, +HP) of the output. A thread therefore holds 32 scores and HP output values of one row.
    constexpr int HP = H / 4;
    const int sub = warp & 3, part = (warp - 2) >> 2;
    const uint32_t lane_base = ((uint32_t)(sub * 32)) << 16;
    const int rl = sub * 32 + lane;  // row within the CTA's 128
    const int row = row0 + rl;
    const bool row_live = row < rows_total;
    const int sq = row_live ? row / p.R : 0;
    const int klim = row_live ? (p.causal ? min(key_len, offset + sq + 1) : key_len) : 0;  // keys [0, klim) are visible
    const uint16_t* am = p.am ? p.am + (int64_t)b * p.Spad : nullptr;
    const float sc2 = p.scale * 1.4426950408889634f;  // scores in units of log2(e): exp(x) = exp2(x * log2 e)
    float o[HP];
#pragma unroll
    for (int i = 0; i < HP; i++) o[i] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f, alpha_prev = 1.0f;
    bool dead = false;

    auto accumulate = [&](int t, float alpha) {  // o = o * alpha + T_t (this warp's columns)
      if (!tc_wait(tc_smem_u32(&o_full), (uint32_t)(t & 1))) { atomicExch(&g_attn_tc_err, 7u); dead = true; return; }
      tc_fence_after();
      uint32_t v[HP];
      if (HP == 32) {
        at_ld_x32(tmem + lane_base + C::COL_T + part * HP, reinterpret_cast<uint32_t(&)[32]>(v));
      } else {
        tc_ld_x16(tmem + lane_base + C::COL_T + part * HP, reinterpret_cast<uint32_t(&)[16]>(v));
      }
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int i = 0; i < HP; i++) o[i] = fmaf(o[i], alpha, __uint_as_float(v[i]));
      tc_fence_before();
      tc_mbar_arrive(tc_smem_u32(&o_free));
    };

    for (int j = 0; j < ntiles && !dead; j++) {
      const int s = j & 1;
      if (!tc_wait(tc_smem_u32(&s_full[s]), (uint32_t)((j >> 1) & 1))) { atomicExch(&g_attn_tc_err, 8u); dead = true; break; }
      tc_fence_after();
      const int k0 = j * 128 + part * 32;  // this thread's 32 keys
      uint32_t v[32];
      at_ld_x32(tmem + lane_base + C::COL_S + s * 128 + part * 32, v);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      float x[32];
      if (!am && k0 + 32 <= klim) {  // every key visible, no mask
#pragma unroll
        for (int i = 0; i < 32; i++) x[i] = __uint_as_float(v[i]) * sc2;
      } else {
#pragma unroll
        for (int i = 0; i < 32; i++) {
          const int key = k0 + i;
          // the mask's "drop" value is the most negative finite bf16: it must stay finite after the change of units, so
          // that a row whose visible keys are all dropped still averages them, as the reference's softmax does
          const float madd = (am && key < p.Spad) ? fmaxf(bf16_bits_to_f32(am[key]) * 1.4426950408889634f, -3.0e38f) : 0.0f;
          x[i] = key < klim ? fmaf(__uint_as_float(v[i]), sc2, madd) : -INFINITY;
        }
      }
      float t4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 32; i++) t4[i & 3] = fmaxf(t4[i & 3], x[i]);
      xmax[s][part][rl] = fmaxf(fmaxf(t4[0], t4[1]), fmaxf(t4[2], t4[3]));
      asm volatile("bar.sync %0, 128;" ::"r"(1 + sub) : "memory");  // the four warps of this quarter
      const float tmax = fmaxf(fmaxf(xmax[s][0][rl], xmax[s][1][rl]), fmaxf(xmax[s][2][rl], xmax[s][3][rl]));
      const float m_new = fmaxf(m_run, tmax);
      const float alpha = (m_new == -INFINITY) ? 1.0f : at_ex2(m_run - m_new);
      const float mref = (m_new == -INFINITY) ? 0.0f : m_new;
      float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float e0 = at_ex2(x[i] - mref), e1 = at_ex2(x[i + 1] - mref);  // exp2(-inf) = 0 for hidden keys
        l4[(i >> 1) & 3] += e0 + e1;
        w[i >> 1] = at_pack_bf16x2(e0, e1);
      }
      at_st_x16(tmem + lane_base + C::COL_P + s * 64 + part * 16, w);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      tc_mbar_arrive(tc_smem_u32(&p_full[s]));
      l_run = l_run * alpha + ((l4[0] + l4[1]) + (l4[2] + l4[3]));
      m_run = m_new;
      if (j > 0) accumulate(j - 1, alpha_prev);  // the previous tile's product, while the tensor core works on this tile's
      alpha_prev = alpha;
    }
    if (!dead && ntiles > 0) accumulate(ntiles - 1, alpha_prev);
    // the row sums of the four key ranges
    xmax[0][part][rl] = l_run;
    asm volatile("bar.sync %0, 128;" ::"r"(1 + sub) : "memory");
    const float l_tot = (xmax[0][0][rl] + xmax[0][1][rl]) + (xmax[0][2][rl] + xmax[0][3][rl]);
    if (row_live && !dead) {
      const float inv = 1.0f / l_tot;
      uint16_t* dst = p.out + attn_out_index(p, bn, row, H) + part * HP;
#pragma unroll
      for (int i = 0; i < HP; i += 8) {
        uint32_t wv[4];
#pragma unroll
        for (int u = 0; u < 4; u++) wv[u] = at_pack_bf16x2(o[i + 2 * u] * inv, o[i + 2 * u + 1] * inv);
        *reinterpret_cast<uint4*>(dst + i) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*AtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static AtEncodeFn at_encode_fn() {
  static AtEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &ptr, 12000, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<AtEncodeFn>(ptr);
  }
  return fn;
}

bool attn_tc_serves(int64_t rows, int64_t H) { return rows >= 64 && (H == 64 || H == 128) && knobs().attn_tc != 0; }

template <int H>
static int at_launch(const AttnParams& p, cudaStream_t st) {
  using C = AtCfg<H>;
  AtEncodeFn fn = at_encode_fn();
  TPX_REQUIRE(fn, TPX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const uint64_t rows_total = (uint64_t)p.Sq * p.R, bn = (uint64_t)p.B * p.Nkv;
  const uint64_t s1 = ((uint64_t)p.key_len + 31) / 32;  // cache blocks that may hold keys; tiles beyond read as zeros
  CUtensorMap mq, mk, mv;
  {
    cuuint64_t gdim[2] = {(cuuint64_t)H, bn * rows_total};
    cuuint64_t gstr[1] = {(cuuint64_t)H * 2};
    cuuint32_t box[2] = {64, 128};
    cuuint32_t es[2] = {1, 1};
    CUresult r = fn(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(p.q), gdim, gstr, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TPX_REQUIRE(r == CUDA_SUCCESS, TPX_ERR_CUDA, "attention: cuTensorMapEncodeTiled (queries) failed with %d", (int)r);
  }
  for (int which = 0; which < 2; which++) {
    cuuint64_t gdim[4] = {(cuuint64_t)H, 32, bn, s1};
    cuuint64_t gstr[3] = {(cuuint64_t)H * 2, (cuuint64_t)32 * H * 2, bn * 32 * H * 2};
    cuuint32_t box[4] = {64, 32, 1, 4};
    cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult r = fn(which ? &mv : &mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<uint16_t*>(which ? p.vc : p.kc), gdim, gstr, box, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TPX_REQUIRE(r == CUDA_SUCCESS, TPX_ERR_CUDA, "attention: cuTensorMapEncodeTiled (cache) failed with %d", (int)r);
  }
  static bool opted[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || !opted[dev]) {
    TPX_CUDA_OK(cudaFuncSetAttribute(attn_tc_kernel<H>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    if (dev >= 0 && dev < 16) opted[dev] = true;
  }
  const unsigned chunks = (unsigned)((rows_total + 127) / 128);
  TPX_REQUIRE(chunks <= 65535, TPX_ERR_UNSUPPORTED, "attention: too many query rows in one call");
  TPX_CUDA_OK(launch_pdl(attn_tc_kernel<H>, dim3((unsigned)bn, chunks), dim3(kAtThreads), C::SMEM, st, mq, mk, mv, p));
  return TPX_OK;
}

int attn_tc_launch(const AttnParams& p, cudaStream_t st) {
  TPX_REQUIRE((((uintptr_t)p.q | (uintptr_t)p.kc | (uintptr_t)p.vc | (uintptr_t)p.out) & 15) == 0, TPX_ERR_ARG,
              "attention: q, the cache and out must be 16-byte aligned");
  return p.H == 128 ? at_launch<128>(p, st) : at_launch<64>(p, st);
}

}  // namespace tpx

using namespace tpx;

extern "C" int tpx_attention_tc_status(void* stream, unsigned* status_host) {
  TPX_REQUIRE(status_host, TPX_ERR_ARG, "attention_tc_status: null pointer");
  static void* ptrs[64] = {};
  int dev = 0;
  TPX_CUDA_OK(cudaGetDevice(&dev));
  TPX_REQUIRE(dev >= 0 && dev < 64, TPX_ERR_UNSUPPORTED, "attention_tc_status: device index %d out of range", dev);
  if (!ptrs[dev]) TPX_CUDA_OK(cudaGetSymbolAddress(&ptrs[dev], g_attn_tc_err));
  TPX_CUDA_OK(cudaMemcpyAsync(status_host, ptrs[dev], 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  TPX_CUDA_OK(cudaMemsetAsync(ptrs[dev], 0, 4, (cudaStream_t)stream));
  TPX_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
  return TPX_OK;
}
