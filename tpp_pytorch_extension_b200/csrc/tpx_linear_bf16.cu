// bf16-weight linear on the 5th-generation tensor cores (tcgen05 kind::f16, sm_100a).
//
// Replaces TppBlockedLinearW<bf16> (src/csrc/fused_gemm.h:784-1073), the GEMM behind torch.ops.tpp_llm.fc_plain for
// unquantized weights; on the decoder path that is the lm_head (src/csrc/llm/fused_llm_infer.cpp:1514-1566), which the
// reference keeps in bf16 unless --quantize-lm-head is given.
//
//     y[M][N] = epilogue(x[M][K] . W[N][K]^T + bias[N])
//
// Neither operand is re-laid out: TMA reads 128-row x 64-column boxes of the plain row-major W and TOK-row boxes of x
// straight into the 128-byte-swizzled K-major operand layout; rows and columns beyond the matrices read as zero.
//
//   rows of W (output features) = M of the MMA (128 per tile), tokens = N (TOK per tile), 64 k values per k step
//   warp 0   : TMA producer into a ring of stages
//   warp 1   : allocates tensor memory, issues the MMAs (K = 16 each), commits stages back to the producer
//   warps 2-5: epilogue (tensor memory -> registers -> bias / activation / multiply / residual -> y)
//
// One CTA per SM walks a contiguous range of output tiles (the token tiles of one feature tile are neighbours, so a
// weight tile fetched for the first of them is found in L2 by the others). Two accumulators in tensor memory: the
// epilogue of a tile runs under the MMAs of the next. At decode sizes the kernel is a plain stream of W at HBM rate.
#include "tpx_tc_ptx.cuh"

namespace tpx {

struct BfParams {
  TcParams t;   // epilogue fields (bias, act, mul_in, res, res_scale, y, M, N, err)
  int ksteps;   // k steps of 64 (K rounded up)
  int TN, TM;   // feature tiles, token tiles
};

template <int TOK>
struct BfCfg {
  static constexpr int UK = TOK <= 64 ? 2 : 1;           // k steps per pipeline stage
  static constexpr int A_BYTES = 128 * 128;              // 128 features x 64 bf16
  static constexpr int B_BYTES = TOK * 128;              // TOK tokens x 64 bf16
  static constexpr int STAGE_BYTES = UK * (A_BYTES + B_BYTES);
  static constexpr int STAGES_FIT = (227 * 1024 - 3072) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 10 ? 10 : STAGES_FIT;
  static constexpr int COLS_RAW = 2 * TOK;               // two accumulators
  static constexpr int TMEM_COLS = COLS_RAW <= 32 ? 32 : COLS_RAW <= 64 ? 64 : COLS_RAW <= 128 ? 128 : COLS_RAW <= 256 ? 256 : 512;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;
  static_assert(STAGES >= 3, "at least three stages");
  static_assert(COLS_RAW <= 512, "tensor memory");
};

__device__ __forceinline__ void bf_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "  tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int TOK>
__global__ void __launch_bounds__(kTcThreads, 1)
linear_bf16_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, BfParams p) {
  using C = BfCfg<TOK>;
  extern __shared__ unsigned char bf_smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[C::STAGES], bar_empty[C::STAGES];
  __shared__ __align__(8) unsigned long long acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_holder;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (tc_smem_u32(bf_smem_raw) + 1023u) & ~1023u;
  const long long T = (long long)p.TN * p.TM;
  const int tile0 = (int)((long long)blockIdx.x * T / gridDim.x), tile1 = (int)(((long long)blockIdx.x + 1) * T / gridDim.x);
  const int nstages = (p.ksteps + C::UK - 1) / C::UK;  // pipeline stages per tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; s++) {
      tc_mbar_init(tc_smem_u32(&bar_full[s]), 1);
      tc_mbar_init(tc_smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; b++) {
      tc_mbar_init(tc_smem_u32(&acc_full[b]), 1);
      tc_mbar_init(tc_smem_u32(&acc_empty[b]), 4);
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

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      pdl_wait();  // x (and, in a chain of launches, nothing else) comes from earlier grids
      long long it = 0;
      bool dead = false;
      for (int tile = tile0; tile < tile1 && !dead; tile++) {
        const int tn = tile / p.TM, tm = tile % p.TM;
        for (int g = 0; g < nstages; g++, it++) {
          const int s = (int)(it % C::STAGES);
          if (it >= C::STAGES && !tc_wait(tc_smem_u32(&bar_empty[s]), (uint32_t)((it / C::STAGES - 1) & 1))) {
            atomicExch(p.t.err, 2u);
            dead = true;
            break;
          }
          const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
          const uint32_t bar = tc_smem_u32(&bar_full[s]);
          tc_mbar_expect_tx(bar, C::STAGE_BYTES);
#pragma unroll
          for (int u = 0; u < C::UK; u++) {  // a k step beyond K reads as zeros
            const int kc = (g * C::UK + u) * 64;
            tc_tma_2d(st + u * C::A_BYTES, &tmW, kc, tn * 128, bar);
            tc_tma_2d(st + C::UK * C::A_BYTES + u * C::B_BYTES, &tmX, kc, tm * TOK, bar);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // kind::f16: D = F32 (1), A = B = BF16 (1), both K-major, N = TOK, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TOK >> 3) << 17) | ((128u >> 4) << 24);
      long long it = 0;
      uint32_t empty_phase = 0;  // bit b: parity to wait for on acc_empty[b]
      bool dead = false;
      for (int tile = tile0; tile < tile1 && !dead; tile++) {
        const int buf = (tile - tile0) & 1;
        if (tile - tile0 >= 2) {  // the epilogue must have drained this accumulator
          if (!tc_wait(tc_smem_u32(&acc_empty[buf]), (empty_phase >> buf) & 1u)) { atomicExch(p.t.err, 3u); break; }
          empty_phase ^= 1u << buf;
          tc_fence_after();
        }
        for (int g = 0; g < nstages; g++, it++) {
          const int s = (int)(it % C::STAGES);
          if (!tc_wait(tc_smem_u32(&bar_full[s]), (uint32_t)((it / C::STAGES) & 1))) { atomicExch(p.t.err, 4u); dead = true; break; }
          tc_fence_after();
          const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
#pragma unroll
          for (int u = 0; u < C::UK; u++) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
              bf_mma(tmem + buf * TOK, tc_smem_desc(st + u * C::A_BYTES) + (uint64_t)(2 * j),
                     tc_smem_desc(st + C::UK * C::A_BYTES + u * C::B_BYTES) + (uint64_t)(2 * j), idesc, (g == 0 && u == 0 && j == 0) ? 0u : 1u);
            }
          }
          tc_commit(tc_smem_u32(&bar_empty[s]));
        }
        if (!dead) tc_commit(tc_smem_u32(&acc_full[buf]));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int sub = warp & 3;  // tensor-memory lanes 32*sub .. 32*sub+31 belong to this warp
    const uint32_t lane_base = ((uint32_t)(sub * 32)) << 16;
    uint32_t full_phase = 0;
    pdl_wait();  // residual and multiplier inputs belong to earlier grids
    for (int tile = tile0; tile < tile1; tile++) {
      const int buf = (tile - tile0) & 1;
      if (!tc_wait(tc_smem_u32(&acc_full[buf]), (full_phase >> buf) & 1u)) {
        if (lane == 0) atomicExch(p.t.err, 6u);
        break;
      }
      full_phase ^= 1u << buf;
      tc_fence_after();
      const int tn = tile / p.TM, tm = tile % p.TM;
      const int n = tn * 128 + sub * 32 + lane;
      const int tok0 = tm * TOK;
#pragma unroll 1
      for (int c0 = 0; c0 < TOK; c0 += 16) {
        uint32_t a[16];
        float v[16], v2[16];
        tc_ld_x16(tmem + lane_base + buf * TOK + c0, a);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; j++) { v[j] = __uint_as_float(a[j]); v2[j] = 0.0f; }
        if (n < p.t.N && tok0 + c0 < p.t.M) tc_finish16<false>(p.t, tok0 + c0, n, v, v2);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(tc_smem_u32(&acc_empty[buf]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)C::TMEM_COLS) : "memory");
  }
}

// 2-D bf16 tensor [rows][cols] (row stride cols * 2 bytes), box = 64 columns x box_rows, 128-byte swizzle.
static int bf_make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
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
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TPX_REQUIRE(r == CUDA_SUCCESS, TPX_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (rows=%llu cols=%llu box_rows=%u)", (int)r,
              (unsigned long long)rows, (unsigned long long)cols, box_rows);
  return TPX_OK;
}

template <int TOK>
static int bf_launch(const CUtensorMap& w, const CUtensorMap& x, const BfParams& p, cudaStream_t st) {
  using C = BfCfg<TOK>;
  static bool opted[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || !opted[dev]) {
    TPX_CUDA_OK(cudaFuncSetAttribute(linear_bf16_kernel<TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    if (dev >= 0 && dev < 16) opted[dev] = true;
  }
  const long long T = (long long)p.TN * p.TM;
  const int sms = sm_count();
  TPX_CUDA_OK(launch_pdl(linear_bf16_kernel<TOK>, dim3((unsigned)(T < sms ? T : sms)), dim3(kTcThreads), C::SMEM, st, w, x, p));
  return TPX_OK;
}

}  // namespace tpx

using namespace tpx;

extern "C" size_t tpx_linear_bf16_tc_scratch_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return kTcCounterBytes;
}

extern "C" int tpx_linear_bf16_tc(const uint16_t* w, const uint16_t* x, int64_t M, int64_t N, int64_t K, const uint16_t* bias, int act,
                                  const uint16_t* mul_in, const uint16_t* res, float res_scale, uint16_t* y, void* scratch,
                                  size_t scratch_bytes, void* stream) {
  TPX_REQUIRE(M >= 0 && N > 0 && K > 0, TPX_ERR_ARG, "linear_bf16_tc: bad shape");
  if (M == 0) return TPX_OK;
  TPX_REQUIRE(w && x && y, TPX_ERR_ARG, "linear_bf16_tc: null pointer");
  TPX_REQUIRE(K % 8 == 0, TPX_ERR_ARG, "linear_bf16_tc: K must be a multiple of 8 (rows of whole 16-byte units), got %ld", (long)K);
  TPX_REQUIRE(M < (1 << 24) && N < (1 << 24) && K < (1 << 24), TPX_ERR_ARG, "linear_bf16_tc: shape too large");
  TPX_REQUIRE(act >= TPX_ACT_NONE && act <= TPX_ACT_RELU, TPX_ERR_ARG, "linear_bf16_tc: unknown activation %d", act);
  TPX_REQUIRE((((uintptr_t)w | (uintptr_t)x) & 15) == 0 && ((uintptr_t)scratch & 255) == 0, TPX_ERR_ARG, "linear_bf16_tc: misaligned pointer");
  TPX_REQUIRE(scratch && scratch_bytes >= kTcCounterBytes, TPX_ERR_SCRATCH, "linear_bf16_tc: scratch of %zu bytes needed, %zu given",
              kTcCounterBytes, scratch_bytes);
  const int tok = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  BfParams p = {};
  p.t.bias = bias; p.t.mul_in = mul_in; p.t.res = res; p.t.res_scale = res_scale; p.t.y = y; p.t.act = act;
  p.t.M = (int)M; p.t.N = (int)N; p.t.K = (int)K;
  p.t.err = reinterpret_cast<unsigned*>(reinterpret_cast<unsigned char*>(scratch) + kTcCounterBytes - 4);
  p.ksteps = (int)((K + 63) / 64);
  p.TN = (int)((N + 127) / 128);
  p.TM = (int)((M + tok - 1) / tok);
  CUtensorMap mw, mx;
  int rc = bf_make_map(&mw, w, (uint64_t)N, (uint64_t)K, 128);
  if (rc) return rc;
  rc = bf_make_map(&mx, x, (uint64_t)M, (uint64_t)K, (uint32_t)tok);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  switch (tok) {
    case 16: return bf_launch<16>(mw, mx, p, st);
    case 32: return bf_launch<32>(mw, mx, p, st);
    case 64: return bf_launch<64>(mw, mx, p, st);
    case 128: return bf_launch<128>(mw, mx, p, st);
    default: return bf_launch<256>(mw, mx, p, st);
  }
}
