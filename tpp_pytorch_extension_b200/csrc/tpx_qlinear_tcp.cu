// MXFP4 weight-only linear for many tokens (prefill), tcgen05 + TMA, with the epilogue hidden behind the next tile.
//
// Replaces the same reference functions as tpx_qlinear_tc.cu (fc_plain / fc_gate_up / fc_add of
// src/csrc/llm/fused_llm_infer.cpp on MXFP4 weights) where every CTA owns whole output tiles of 128 features x 128
// tokens. The general kernel keeps one accumulator per CTA, so its MMAs stop while the epilogue drains a tile: measured
// per tile at 8192 tokens (K = 4096) 17.6 us of MMAs, 0.9 us of drain and 3.9 us of epilogue, 15.8 us when the epilogue
// also reads a residual. Here
//   * both activation terms accumulate into the SAME 128 columns of tensor memory (two N = 128 MMAs per k slice, the
//     hi and the lo term, each with its own scale block) instead of 128 + 128 columns that the epilogue adds, so an
//     accumulator is 128 columns and three of them fit beside the scale factors: the MMAs of the next tile run while
//     sixteen epilogue warps drain the previous one;
//   * a gate/up pair is two consecutive accumulations (gate tile, then up tile, over the same activation tile) whose
//     accumulators the epilogue reads together; with three accumulators the next gate tile starts meanwhile;
//   * residual and gate-input values of a tile are loaded into registers BEFORE the epilogue warps wait for the
//     accumulator, i.e. during the tile's MMAs.
// Layouts of the packed weights, their scale blocks, the activation terms and their scale blocks are those of
// tpx_qlinear_tc.cu (token tile 128).
#include "tpx_tc_ptx.cuh"

namespace tpx {

template <int UKS>
struct TcpCfg {
  static constexpr int TOK = 128;
  static constexpr int A_BYTES = 128 * 128;             // an unpacked 128 x 128 fp4 tile in shared memory
  static constexpr int A_TX = 128 * 64;                 // what its copy accounts for (packed bytes)
  static constexpr int B_BYTES = TOK * 128;             // one term of one k step
  static constexpr int X_ROWS = UKS * 2 * TOK;          // per k step: 128 hi rows, then 128 lo rows
  static constexpr int SF_BLOCKS = UKS * 3;             // weight blocks first (one per k step), then hi/lo activation blocks
  static constexpr int RAW = UKS * A_BYTES + X_ROWS * 128 + SF_BLOCKS * 512;
  static constexpr int STAGE_BYTES = (RAW + 1023) / 1024 * 1024;
  static constexpr int TX = UKS * A_TX + X_ROWS * 128 + SF_BLOCKS * 512;
  static constexpr int BUDGET = 227 * 1024 - 2048;
  static constexpr int STAGES_RAW = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
  static constexpr int SF_COLS = SF_BLOCKS * 4;
  static constexpr int NBUF = 3;                        // accumulators of 128 columns
  static constexpr int D_COLS = 128;
  static constexpr int TMEM_COLS = 512;
  static constexpr int EPI_SPLIT = 4;                   // warps per 32-lane quarter of tensor memory, 32 tokens each
  static constexpr int THREADS = 64 + 128 * EPI_SPLIT;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;
  static_assert(STAGES >= 2, "at least two stages");
  static_assert(NBUF * D_COLS + STAGES * SF_COLS <= 512, "tensor memory");
};

// UKS k steps of 128 per pipeline stage; DUAL: gate/up pair (weights interleaved per k step: gate tile, up tile).
// p.KS counts stages per accumulation; p.TN x p.TM tiles of 128 features x 128 tokens, cut evenly between the CTAs.
template <int UKS, bool DUAL>
__global__ void __launch_bounds__(TcpCfg<UKS>::THREADS, 1)
qlinear_tcp_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, TcParams p) {
  using C = TcpCfg<UKS>;
  constexpr int NWT = DUAL ? 2 : 1;  // accumulations per output tile
  extern __shared__ unsigned char tcp_smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[C::STAGES], bar_empty[C::STAGES];
  __shared__ __align__(8) unsigned long long bar_acc_full[C::NBUF], bar_acc_empty[C::NBUF];
  __shared__ uint32_t tmem_holder;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (tc_smem_u32(tcp_smem_raw) + 1023u) & ~1023u;
  const long long T = (long long)p.TN * p.TM, G = gridDim.x;
  const int t0 = (int)((long long)blockIdx.x * T / G), t1 = (int)(((long long)blockIdx.x + 1) * T / G);
  const int ntiles = t1 - t0;
  const int KU = p.KS;               // stages per accumulation
  const int KSS = KU * UKS;          // k steps per accumulation
  const int nunits = ntiles * NWT * KU;

  if (threadIdx.x == 0) tc_stamp(p, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; s++) {
      tc_mbar_init(tc_smem_u32(&bar_full[s]), 1);
      tc_mbar_init(tc_smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < C::NBUF; b++) {
      tc_mbar_init(tc_smem_u32(&bar_acc_full[b]), 1);
      tc_mbar_init(tc_smem_u32(&bar_acc_empty[b]), 4 * C::EPI_SPLIT);
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
  const uint32_t sf_col0 = C::NBUF * C::D_COLS;
  if (threadIdx.x == 0) tc_stamp(p, 1);
  pdl_trigger();

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      auto fetch_w = [&](int s, int tn, int d, int ku) {  // weights and their scale blocks: independent of earlier kernels
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t bar = tc_smem_u32(&bar_full[s]);
        const uint32_t ssf = st + UKS * C::A_BYTES + C::X_ROWS * 128;
        tc_mbar_expect_tx(bar, C::TX);
        const int ks0 = tn * KSS + ku * UKS;  // first k step of the stage in the weight's [tile][k step] order
        if (DUAL) {
#pragma unroll
          for (int kk = 0; kk < UKS; kk++) {
            const int wt = (ks0 + kk) * 2 + d;
            tc_tma_2d(st + kk * C::A_BYTES, &tmW, 0, wt * 128, bar);
            tc_bulk_g2s(ssf + kk * 512, p.sfa + (size_t)wt * 512, 512, bar);
          }
        } else {
          tc_tma_2d(st, &tmW, 0, ks0 * 128, bar);
          tc_bulk_g2s(ssf, p.sfa + (size_t)ks0 * 512, UKS * 512, bar);
        }
      };
      auto fetch_x = [&](int s, int tm, int ku) {  // activation terms and their scale blocks
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t bar = tc_smem_u32(&bar_full[s]);
        const uint32_t sb = st + UKS * C::A_BYTES;
        const int xrow = (tm * KU + ku) * C::X_ROWS;
#pragma unroll
        for (int r = 0; r < UKS; r++) tc_tma_2d(sb + r * 256 * 128, &tmX, 0, xrow + r * 256, bar);
        tc_bulk_g2s(sb + C::X_ROWS * 128 + UKS * 512, p.sfb + ((size_t)tm * KU + ku) * UKS * 1024, UKS * 1024, bar);
      };
      auto where = [&](int it, int& tn, int& tm, int& d, int& ku) {
        const int a = it / KU;
        ku = it - a * KU;
        const int tile = t0 + a / NWT;
        d = a % NWT;
        tn = tile / p.TM;
        tm = tile - tn * p.TM;
      };
      const int early = nunits < C::STAGES ? nunits : C::STAGES;
      for (int it = 0; it < early; it++) {
        int tn, tm, d, ku;
        where(it, tn, tm, d, ku);
        fetch_w(it, tn, d, ku);
      }
      pdl_wait();  // the activation terms belong to the split kernel until it has completed
      for (int it = 0; it < nunits; it++) {
        const int s = it % C::STAGES;
        int tn, tm, d, ku;
        where(it, tn, tm, d, ku);
        if (it >= C::STAGES) {
          if (!tc_wait(tc_smem_u32(&bar_empty[s]), (uint32_t)((it / C::STAGES - 1) & 1))) {
            atomicExch(p.err, 2u);
            break;
          }
          fetch_w(s, tn, d, ku);
        }
        fetch_x(s, tm, ku);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: A = E2M1 (5), B = E4M3 (0), both K-major, N = 128, UE8M0 scales, M = 128
      const uint32_t idesc0 = (5u << 7) | (0u << 10) | ((uint32_t)(128 >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
      for (int it = 0; it < nunits; it++) {
        const int s = it % C::STAGES;
        const uint32_t ph = (uint32_t)((it / C::STAGES) & 1);
        const int a = it / KU, ku = it - a * KU;
        const int slot = a % C::NBUF;
        if (ku == 0 && a >= C::NBUF) {  // the accumulator's previous tile must have been read
          if (!tc_wait(tc_smem_u32(&bar_acc_empty[slot]), (uint32_t)((a / C::NBUF - 1) & 1))) { atomicExch(p.err, 3u); break; }
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
        const uint32_t ssf = sb + C::X_ROWS * 128;
        const uint32_t sf_t = tmem + sf_col0 + (uint32_t)s * C::SF_COLS;
        const uint32_t dacc = tmem + (uint32_t)slot * C::D_COLS;
        if (TPX_DBG(p) & 1) {
          tc_mbar_arrive(tc_smem_u32(&bar_empty[s]));
          if (ku == KU - 1) tc_mbar_arrive(tc_smem_u32(&bar_acc_full[slot]));
        } else {
#pragma unroll
          for (int q = 0; q < C::SF_BLOCKS; q++) tc_cp_sf(sf_t + q * 4, tc_sf_desc(ssf + q * 512));
#pragma unroll
          for (int kk = 0; kk < UKS; kk++) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const uint32_t idesc = idesc0 | ((uint32_t)j << 29) | ((uint32_t)j << 4);
              const uint64_t adesc = tc_smem_desc(st + kk * C::A_BYTES) + (uint64_t)(2 * j);
#pragma unroll
              for (int t = 0; t < 2; t++) {  // hi term, then lo term, into the same columns
                const uint64_t bdesc = tc_smem_desc(sb + (kk * 2 + t) * C::B_BYTES) + (uint64_t)(2 * j);
                const uint32_t acc = (ku == 0 && kk == 0 && j == 0 && t == 0) ? 0u : 1u;
                tc_mma(dacc, adesc, bdesc, idesc, (sf_t + kk * 4) | ((uint32_t)j << 30),
                       (sf_t + (UKS + kk * 2 + t) * 4) | ((uint32_t)j << 30), acc);
              }
            }
          }
          tc_commit(tc_smem_u32(&bar_empty[s]));
          if (ku == KU - 1) tc_commit(tc_smem_u32(&bar_acc_full[slot]));
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2 .. 2 + 4*EPI_SPLIT - 1)
    const int sub = warp & 3;  // tensor-memory lanes 32*sub .. 32*sub+31 belong to this warp
    const uint32_t lane_base = ((uint32_t)(sub * 32)) << 16;
    const int cpart = (warp - 2) >> 2;  // tokens cpart*32 .. cpart*32+31 of the tile
    const int row = sub * 32 + lane;
    pdl_wait();  // residual and gate inputs belong to earlier grids
    for (int ti = 0; ti < ntiles; ti++) {
      const int tile = t0 + ti;
      const int tn = tile / p.TM, tm = tile - tn * p.TM;
      const int n = tn * 128 + row;
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
      const int a0 = ti * NWT;
      const int slot0 = a0 % C::NBUF, slot1 = (a0 + 1) % C::NBUF;
      bool ok = tc_wait(tc_smem_u32(&bar_acc_full[slot0]), (uint32_t)((a0 / C::NBUF) & 1));
      if (DUAL && ok) ok = tc_wait(tc_smem_u32(&bar_acc_full[slot1]), (uint32_t)(((a0 + 1) / C::NBUF) & 1));
      if (!ok) {
        if (lane == 0) atomicExch(p.err, 6u);
        break;
      }
      tc_fence_after();
      if (threadIdx.x == 64 && ti == ntiles - 1) tc_stamp(p, 5);
#pragma unroll
      for (int c = 0; c < 2; c++) {
        const int c0 = cpart * 32 + c * 16;
        uint32_t g[16], u[16];
        tc_ld_x16(tmem + lane_base + (uint32_t)slot0 * C::D_COLS + c0, g);
        if (DUAL) tc_ld_x16(tmem + lane_base + (uint32_t)slot1 * C::D_COLS + c0, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float x[16], uf[16];
#pragma unroll
        for (int j = 0; j < 16; j++) {
          x[j] = __uint_as_float(g[j]);
          uf[j] = DUAL ? __uint_as_float(u[j]) : 0.0f;
        }
        if (live && tm * 128 + c0 < p.M) tc_finish16_pre<DUAL>(p, tm * 128 + c0, n, x, uf, resp[c], mulp[c], nullptr);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {  // the accumulators may be overwritten
        tc_mbar_arrive(tc_smem_u32(&bar_acc_empty[slot0]));
        if (DUAL) tc_mbar_arrive(tc_smem_u32(&bar_acc_empty[slot1]));
      }
    }
  }
  if (threadIdx.x == 64) tc_stamp(p, 6);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)C::TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------- host side
struct TcpPlan {
  int TN, TM, KS, Mpad, grid, uks;
  size_t off_terms, off_sfb, total;
};

static TcpPlan tcp_plan(int64_t M, int64_t N, int64_t K, bool pair) {
  TcpPlan pl;
  pl.uks = knobs().tc_p_uks == 1 ? 1 : 2;  // two k steps per stage: fewer, larger copy requests (8192 tokens, K = 4096: 921 against 808 TFLOP/s)
  pl.KS = tc_padded_ks(K, pair);  // a multiple of 2
  pl.TN = (int)((N + 127) / 128);
  pl.TM = (int)((M + 127) / 128);
  pl.Mpad = pl.TM * 128;
  const long long T = (long long)pl.TN * pl.TM;
  const int sms = sm_count();
  pl.grid = (int)(T < sms ? T : sms);
  size_t o = kTcCounterBytes;
  auto bump = [&](size_t bytes) { size_t r = o; o += (bytes + 1023) & ~(size_t)1023; return r; };
  pl.off_terms = bump((size_t)pl.Mpad * pl.KS * 128 * 2);
  pl.off_sfb = bump((size_t)pl.TM * pl.KS * 2 * 512);
  pl.total = o;
  return pl;
}

// Whole tiles only. Measured against the general kernel (which balances by cutting tiles between CTAs, with a fix-up
// pass or a cluster reduction): faster or equal from 128 to 32768 tokens at every shape of a Llama-3-8B layer except
// where fewer than a quarter of the SMs get a tile and K is long (128 tokens, 4096 x 14336: 70 against 40 us with the
// cluster split of K). TPX_TC_P=0 never, TPX_TC_P=1 for every M > 64.
bool tcp_serves(int64_t M, int64_t N, int64_t K, bool pair) {
  (void)pair;
  const int k = knobs().tc_p;
  if (k == 0 || M <= 64) return false;
  if (k > 0) return true;
  const long long T = ((N + 127) / 128) * ((M + 127) / 128);
  return T * 2 >= sm_count() || (T * 4 >= sm_count() && K <= 4096);
}

size_t tcp_scratch_bytes(int64_t M, int64_t N, int64_t K, bool pair) { return tcp_plan(M, N, K, pair).total; }

template <int UKS, bool DUAL>
static int tcp_launch(const CUtensorMap& w, const CUtensorMap& x, const TcParams& p, int grid, cudaStream_t st) {
  using C = TcpCfg<UKS>;
  static bool opted[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || !opted[dev]) {
    TPX_CUDA_OK(cudaFuncSetAttribute(qlinear_tcp_kernel<UKS, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    if (dev >= 0 && dev < 16) opted[dev] = true;
  }
  TPX_CUDA_OK(launch_pdl(qlinear_tcp_kernel<UKS, DUAL>, dim3((unsigned)grid), dim3(C::THREADS), C::SMEM, st, w, x, p));
  return TPX_OK;
}

int tcp_run(const uint8_t* wq, const uint8_t* sfa, bool pair, const uint16_t* x, int64_t M, int64_t N, int64_t K, const TcParams& base,
            void* scratch, size_t scratch_bytes, cudaStream_t st, const TcNorm* norm) {
  const TcpPlan pl = tcp_plan(M, N, K, pair);
  TPX_REQUIRE(scratch && scratch_bytes >= pl.total, TPX_ERR_SCRATCH, "qlinear_mxfp4_tc: scratch of %zu bytes needed, %zu given", pl.total,
              scratch_bytes);
  unsigned char* sc = reinterpret_cast<unsigned char*>(scratch);
  uint8_t *terms = sc + pl.off_terms, *sfb = sc + pl.off_sfb;
  {
    int rc0 = tc_launch_split(x, (int)M, (int)K, pl.Mpad, pl.KS, 128, pl.uks, 0, terms, sfb, st, norm);
    if (rc0) return rc0;
  }
  CUtensorMap mw, mx;
  int rc = tc_make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, wq, (uint64_t)pl.TN * pl.KS * (pair ? 2 : 1) * 128, 64,
                       pair ? 128u : (uint32_t)pl.uks * 128u);
  if (rc) return rc;
  rc = tc_make_map(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, terms, (uint64_t)pl.Mpad * pl.KS * 2, 128, 256);
  if (rc) return rc;
  TcParams p = base;
  p.sfa = sfa; p.sfa2 = nullptr; p.sfb = sfb;
  p.partial = nullptr;
  p.counters = reinterpret_cast<unsigned*>(sc);
  p.err = reinterpret_cast<unsigned*>(sc + kTcCounterBytes - 4);
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.KS = pl.KS / pl.uks; p.TN = pl.TN; p.TM = pl.TM;
  p.whole_tiles = 1; p.cluster = 1;
  if (pl.uks == 2) return pair ? tcp_launch<2, true>(mw, mx, p, pl.grid, st) : tcp_launch<2, false>(mw, mx, p, pl.grid, st);
  return pair ? tcp_launch<1, true>(mw, mx, p, pl.grid, st) : tcp_launch<1, false>(mw, mx, p, pl.grid, st);
}

}  // namespace tpx
