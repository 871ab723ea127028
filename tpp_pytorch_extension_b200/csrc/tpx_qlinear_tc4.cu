// MXFP4 weight-only linear for up to 32 tokens with both MMA operands in packed 4-bit form (tcgen05 kind::mxf4).
//
// Same contract and the same packed weights as tpx_qlinear_tc.cu (TppBlockedLinearW with the MXFP4 BRGEMM of the
// reference, src/csrc/fused_gemm.h:875-949). The difference is how the bf16 activations reach the tensor core.
// kind::mxf8f6f4 reads 4-bit codes only from 8-bit containers, so every packed weight byte occupies two bytes of
// shared memory and an MMA covers K = 32. kind::mxf4 reads the packed bytes as they lie in HBM (half the shared
// memory per weight, twice the stages) and covers K = 64 per instruction, but both operands must then be E2M1.
// A bf16 activation therefore becomes FOUR E2M1 terms, each with its own power-of-two block scale:
//     x = 2^e * (q1 + q2 / 4 + q3 / 32 + q4 / 256) + r,   |r| <= 2^(e-9),   2^e * 6 >= max |x| of the 32-wide block
// (q1 = round(x / 2^e) leaves a residual of at most 1, q2 = round(4 * residual) one of at most 1/2, and so on: the
// residuals are exact in fp32, so the only error is the last one: below 2^-10.5 of the block maximum). The terms are
// 4 * TOK columns of one MMA; UE8M0 scale bytes e, e-2, e-5, e-8 give each column group its weight; the epilogue adds
// the four column groups of the fp32 tile.
//
//   rows of W = M of the MMA (128 per tile), tokens = N (4 * TOK columns), k step 128 = two MMAs
//   warp 0: TMA producer, warp 1: MMA issue, warps 2-5: epilogue (as in tpx_qlinear_tc.cu), warp 6: scale-factor copies
#include "tpx_tc_ptx.cuh"

namespace tpx {

// ---------------------------------------------------------------- activation split into four E2M1 terms
//   terms [TM][KU][UKS][4 terms][TOK rows][64 bytes]   (one k step of one term = a TOK x 64-byte operand tile,
//         low nibble = even k)
//   sfb   [TM][KU][UKS][512]   scale bytes of the 4*TOK MMA columns (column t*TOK + r for term t of token r):
//         byte (c%32)*16 + (c/32)*4 + j for column c and 32-wide block j of the k step
// One thread owns 8 consecutive elements; the four threads of a 32-wide block share the scale.
__device__ __forceinline__ void split4_emit(const float (&f)[8], bool store, int tok, int i, int KS, int TOK, int UKS,
                                            uint8_t* __restrict__ terms, uint8_t* __restrict__ sfb) {
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(f[j]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  // 2^e: the block maximum lands in (3, 6]
  int e = -119;
  if (amax > 0.0f && amax < INFINITY) {
    e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127 - 2;  // amax / 2^e in [4, 8)
    e = max(-119, min(125, e));
    if (amax * __uint_as_float((uint32_t)(127 - e) << 23) > 6.0f) e++;
  }
  const float down = __uint_as_float((uint32_t)(127 - e) << 23);
  float r[8];
#pragma unroll
  for (int j = 0; j < 8; j++) r[j] = f[j] * down;
  uint32_t packed[4];
#pragma unroll
  for (int t = 0; t < 4; t++) {
    // eight values -> eight E2M1 codes (element 0 in the lowest nibble), round to nearest, and back to see what they hold
    uint32_t w, h0, h1, h2, h3;
    asm("{ .reg .b8 b0, b1, b2, b3;\n"
        "  cvt.rn.satfinite.e2m1x2.f32 b0, %6, %5;\n"
        "  cvt.rn.satfinite.e2m1x2.f32 b1, %8, %7;\n"
        "  cvt.rn.satfinite.e2m1x2.f32 b2, %10, %9;\n"
        "  cvt.rn.satfinite.e2m1x2.f32 b3, %12, %11;\n"
        "  mov.b32 %0, {b0, b1, b2, b3};\n"
        "  cvt.rn.f16x2.e2m1x2 %1, b0;\n"
        "  cvt.rn.f16x2.e2m1x2 %2, b1;\n"
        "  cvt.rn.f16x2.e2m1x2 %3, b2;\n"
        "  cvt.rn.f16x2.e2m1x2 %4, b3; }"
        : "=r"(w), "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3)
        : "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]));
    packed[t] = w;
    if (t < 3) {  // the residual, exact in fp32, scaled into the next term's range
      const uint32_t h[4] = {h0, h1, h2, h3};
      const float up = t == 0 ? 4.0f : 8.0f;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float2 q = __half22float2(*reinterpret_cast<const __half2*>(&h[j]));
        r[2 * j] = (r[2 * j] - q.x) * up;
        r[2 * j + 1] = (r[2 * j + 1] - q.y) * up;
      }
    }
  }
  if (!store) return;
  const int tm = tok / TOK, row = tok % TOK;
  const int ks = i >> 4, chunk = i & 15, j = chunk >> 2;
  const int KU = KS / UKS;
  const size_t step = ((size_t)tm * KU + ks / UKS) * UKS + ks % UKS;  // k step in fetch order
#pragma unroll
  for (int t = 0; t < 4; t++)
    *reinterpret_cast<uint32_t*>(terms + ((step * 4 + t) * TOK + row) * 64 + chunk * 4) = packed[t];
  if ((chunk & 3) == 0) {
    uint8_t* blk = sfb + step * 512;
    const int shift[4] = {0, 2, 5, 8};
#pragma unroll
    for (int t = 0; t < 4; t++) {
      const int c = t * TOK + row;
      blk[(c % 32) * 16 + (c / 32) * 4 + j] = (uint8_t)(e + 127 - shift[t]);
    }
  }
}

// x[M][K] bf16 -> terms, any K: one thread per 8 elements of the padded [Mpad][KS*128] matrix.
__global__ void __launch_bounds__(128) split4_kernel(const uint16_t* __restrict__ x, int M, int K, int Mpad, int KS, int TOK, int UKS,
                                                     uint8_t* __restrict__ terms, uint8_t* __restrict__ sfb) {
  pdl_trigger();
  pdl_wait();
  const int nvp = KS * 16;  // 8-element vectors of a padded row
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool in = idx < (long long)Mpad * nvp;  // the grid is a whole number of warps: every lane takes part in the shuffles
  const int tok = in ? (int)(idx / nvp) : 0, i = in ? (int)(idx % nvp) : 0;
  float f[8];
#pragma unroll
  for (int j = 0; j < 8; j++) f[j] = 0.0f;
  if (in && tok < M && i * 8 < K) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)tok * K + i * 8);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      f[2 * j] = bf16_bits_to_f32((uint16_t)(w[j] & 0xffff));
      f[2 * j + 1] = bf16_bits_to_f32((uint16_t)(w[j] >> 16));
    }
  }
  split4_emit(f, in, tok, i, KS, TOK, UKS, terms, sfb);
}

// RMSNorm fused into the split (llama_rms_norm, src/csrc/llm/fused_llm_infer.cpp:336-363): one CTA per token row of
// up to 8192 elements, the row kept in registers; the normalised value is rounded to bf16 before it is split, as the
// separate kernel would store it.
constexpr int kN4Threads = 256;
constexpr int kN4Vecs = 4;
__global__ void __launch_bounds__(kN4Threads) rmsnorm_split4_kernel(const uint16_t* __restrict__ x, const void* __restrict__ gamma,
                                                                    int gamma_f32, float eps, int M, int K, int KS, int TOK, int UKS,
                                                                    uint8_t* __restrict__ terms, uint8_t* __restrict__ sfb) {
  __shared__ float red[kN4Threads / 32];
  pdl_trigger();
  pdl_wait();
  const int tok = blockIdx.x;
  const bool live_row = tok < M;
  const int nv = K / 8, nvp = KS * 16;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)tok * K);
  float xv[kN4Vecs][8], gm[kN4Vecs][8];
  float ss = 0.0f;
#pragma unroll
  for (int q = 0; q < kN4Vecs; q++) {
    const int i = threadIdx.x + q * kN4Threads;
    const bool have = live_row && i < nv;
    const uint4 v = have ? xr[i] : make_uint4(0, 0, 0, 0);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      xv[q][2 * j] = bf16_bits_to_f32((uint16_t)(w[j] & 0xffff));
      xv[q][2 * j + 1] = bf16_bits_to_f32((uint16_t)(w[j] >> 16));
    }
    if (have && gamma_f32) {
      const float4 g0 = reinterpret_cast<const float4*>(gamma)[2 * i], g1 = reinterpret_cast<const float4*>(gamma)[2 * i + 1];
      gm[q][0] = g0.x; gm[q][1] = g0.y; gm[q][2] = g0.z; gm[q][3] = g0.w;
      gm[q][4] = g1.x; gm[q][5] = g1.y; gm[q][6] = g1.z; gm[q][7] = g1.w;
    } else if (have) {
      const uint4 gv = reinterpret_cast<const uint4*>(gamma)[i];
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        gm[q][2 * j] = bf16_bits_to_f32((uint16_t)(gw[j] & 0xffff));
        gm[q][2 * j + 1] = bf16_bits_to_f32((uint16_t)(gw[j] >> 16));
      }
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
  for (int w = 0; w < kN4Threads / 32; w++) tot += red[w];
  const float inv = rsqrtf(tot / (float)K + eps);
#pragma unroll
  for (int q = 0; q < kN4Vecs; q++) {
    const int i = threadIdx.x + q * kN4Threads;
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; j++) f[j] = bf16_bits_to_f32(f32_to_bf16_bits(xv[q][j] * inv * gm[q][j]));
    split4_emit(f, i < nvp, tok, i < nvp ? i : 0, KS, TOK, UKS, terms, sfb);
  }
}

static int tc4_launch_split(const uint16_t* x, int M, int K, int Mpad, int KS, int TOK, int UKS, uint8_t* terms, uint8_t* sfb,
                            cudaStream_t st, const TcNorm* norm) {
  if (norm && norm->gamma) {
    TPX_REQUIRE(KS * 16 <= kN4Threads * kN4Vecs, TPX_ERR_UNSUPPORTED, "fused RMSNorm: rows of more than %d elements are not supported (K=%d)",
                kN4Threads * kN4Vecs * 8, K);
    TPX_REQUIRE((((uintptr_t)x | (uintptr_t)norm->gamma) & 15) == 0, TPX_ERR_ARG, "fused RMSNorm: x and gamma must be 16-byte aligned");
    TPX_CUDA_OK(launch_pdl(rmsnorm_split4_kernel, dim3((unsigned)Mpad), dim3(kN4Threads), 0, st, x, norm->gamma, norm->gamma_f32, norm->eps,
                           M, K, KS, TOK, UKS, terms, sfb));
    return TPX_OK;
  }
  const long long threads = (long long)Mpad * KS * 16;
  TPX_CUDA_OK(launch_pdl(split4_kernel, dim3((unsigned)((threads + 127) / 128)), dim3(128), 0, st, x, M, K, Mpad, KS, TOK, UKS, terms, sfb));
  return TPX_OK;
}

// ---------------------------------------------------------------- the GEMM kernel
// TOK tokens per tile (16 or 32), DUAL = gate/up pair, UKS = k steps (of 128) per pipeline unit.
// OCC = CTAs meant to share an SM: with 2, a CTA keeps to half of the shared memory and at most 256 columns of tensor
// memory, so that the CTAs of the NEXT launch become resident (programmatic dependent launch) while this one still
// streams: their prologue and their first weight stages then overlap this launch's stream instead of following it.
template <int TOK, bool DUAL, int UKS, int OCC = 1>
struct Tc4Cfg {
  static constexpr int NW = DUAL ? 2 : 1;
  static constexpr int A_BYTES = 128 * 64;             // a packed 128 x 128 tile, in shared memory as in HBM
  static constexpr int A_TILES = UKS * NW;             // tiles per unit, fetched 2 at a time (256 rows, 16 KiB)
  static constexpr int B_BYTES = TOK * 64;             // one term of one k step
  static constexpr int X_ROWS = UKS * 4 * TOK;         // rows of 64 bytes of the four terms of the unit
  static constexpr int X_BOX = X_ROWS > 256 ? 256 : X_ROWS;
  static constexpr int NCOL = 4 * TOK;                 // MMA N: term 1 columns, term 2 columns, ...
  // weight blocks first, then one activation block per k step (packing the two k steps' 64 columns of a 16-token unit
  // into one block saves a copy per unit but measured slower end to end: 2.94 against 2.84 ms/token, Llama-3-8B batch 1)
  static constexpr int SF_BLOCKS = UKS * (NW + 1);
  static constexpr int RAW = A_TILES * A_BYTES + X_ROWS * 64 + SF_BLOCKS * 512;
  static constexpr int STAGE_BYTES = (RAW + 1023) / 1024 * 1024;
  static constexpr int TX = RAW;
  static constexpr int BUDGET = OCC == 2 ? 112 * 1024 - 1024 : 227 * 1024 - 2048;
  static constexpr int STAGES_RAW = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SF_COLS = SF_BLOCKS * 4;        // tensor-memory columns of one stage's scale factors
  static constexpr int D_COLS = NW * NCOL;
  static constexpr int COLS_RAW = D_COLS + STAGES * SF_COLS;
  static constexpr int TMEM_COLS = COLS_RAW <= 32 ? 32 : COLS_RAW <= 64 ? 64 : COLS_RAW <= 128 ? 128 : COLS_RAW <= 256 ? 256 : 512;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;  // + alignment slack
  static constexpr int W_BOX = 2;                      // weight tiles per copy request
  static_assert(NCOL <= 128, "one activation scale block per k step");
  static_assert(A_TILES % W_BOX == 0, "weight tiles are fetched two at a time");
  static_assert(X_ROWS % X_BOX == 0, "activation rows are fetched in whole boxes");
  static_assert(STAGES >= 2, "at least two stages");
  static_assert(COLS_RAW <= 512, "tensor memory");
  static_assert(OCC == 1 || COLS_RAW <= 256, "two CTAs per SM share the 512 columns");
  static_assert(STAGES * STAGE_BYTES >= NW * 128 * TOK * 4, "the stages hold a cluster member's partial tile");
};

constexpr int kTc4Threads = 224;  // + warp 6: scale-factor copies, issued apart from the MMAs

template <int TOK, bool DUAL, int UKS, int OCC = 1>
__global__ void __launch_bounds__(kTc4Threads, OCC)
qlinear_tc4_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, TcParams p) {
  using C = Tc4Cfg<TOK, DUAL, UKS, OCC>;
  extern __shared__ unsigned char tc4_smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[C::STAGES], bar_empty[C::STAGES], bar_sf[C::STAGES];
  __shared__ __align__(8) unsigned long long bar_acc_full, bar_acc_empty;
  __shared__ uint32_t tmem_holder;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (tc_smem_u32(tc4_smem_raw) + 1023u) & ~1023u;

  // this CTA's contiguous range of (tile, k unit) units; p.KS counts k units
  const long long U = (long long)p.TN * p.TM * p.KS;
  const long long G = gridDim.x;
  const long long T = (long long)p.TN * p.TM;
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
      tc_mbar_init(tc_smem_u32(&bar_sf[s]), 1);
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
  if (threadIdx.x == 0) tc_stamp(p, 1);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      auto fetch_w = [&](int s, int tn, int ks) {  // weight tiles and their scale blocks: independent of the split kernel
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t bar = tc_smem_u32(&bar_full[s]);
        tc_mbar_expect_tx(bar, C::TX);
        const int wtile = (tn * p.KS + ks) * C::A_TILES;  // first weight tile of the unit
#pragma unroll
        for (int r = 0; r < C::A_TILES / C::W_BOX; r++) tc_tma_2d(st + r * C::W_BOX * C::A_BYTES, &tmW, 0, (wtile + C::W_BOX * r) * 128, bar);
        tc_bulk_g2s(st + C::A_TILES * C::A_BYTES + C::X_ROWS * 64, p.sfa + (size_t)wtile * 512, C::A_TILES * 512, bar);
      };
      auto fetch_x = [&](int s, int tm, int ks) {  // activation terms and their scale blocks
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t bar = tc_smem_u32(&bar_full[s]);
        const uint32_t sb = st + C::A_TILES * C::A_BYTES;
        const int xrow = (tm * p.KS + ks) * C::X_ROWS;
#pragma unroll
        for (int r = 0; r < C::X_ROWS / C::X_BOX; r++) tc_tma_2d(sb + r * C::X_BOX * 64, &tmX, 0, xrow + r * C::X_BOX, bar);
        tc_bulk_g2s(sb + C::X_ROWS * 64 + C::A_TILES * 512, p.sfb + ((size_t)tm * p.KS + ks) * UKS * 512, UKS * 512, bar);
      };
      auto prefetch_w = [&](int tn, int ks) {  // into L2, ahead of the stages
        const int wtile = (tn * p.KS + ks) * C::A_TILES;
#pragma unroll
        for (int r = 0; r < C::A_TILES / C::W_BOX; r++) tc_prefetch_2d(&tmW, 0, (wtile + C::W_BOX * r) * 128);
        tc_prefetch_bulk(p.sfa + (size_t)wtile * 512, C::A_TILES * 512);
      };
      // the first stages' weights go out before this grid is allowed to see the split kernel's output
      const int early = nunits < C::STAGES ? nunits : C::STAGES;
      int ptile = tile0, pks = ks0, pit = 0;  // prefetch cursor
      for (; pit < early; pit++) {
        fetch_w(pit, ptile / p.TM, pks);
        if (++pks == p.KS) { pks = 0; ptile++; }
      }
      for (; pit < nunits && pit < early + p.pf; pit++) {
        prefetch_w(ptile / p.TM, pks);
        if (++pks == p.KS) { pks = 0; ptile++; }
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      tc_stamp(p, 4);
      int tile = tile0, ks = ks0;
      for (int it = 0; it < nunits; it++) {
        const int s = it % C::STAGES;
        const int tn = tile / p.TM, tm = tile % p.TM;
        if (pit < nunits && pit < it + C::STAGES + p.pf) {
          prefetch_w(ptile / p.TM, pks);
          pit++;
          if (++pks == p.KS) { pks = 0; ptile++; }
        }
        if (it >= C::STAGES) {
          if (!tc_wait(tc_smem_u32(&bar_empty[s]), (uint32_t)((it / C::STAGES - 1) & 1))) {
            atomicExch(p.err, 2u);
            break;
          }
          fetch_w(s, tn, ks);
        }
        fetch_x(s, tm, ks);
        if (++ks == p.KS) { ks = 0; tile++; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: A = B = E2M1 (1 in this kind), both K-major, N = 4*TOK, UE8M0 scales, M = 128, K = 64
      const uint32_t idesc0 = (1u << 7) | (1u << 10) | ((uint32_t)(C::NCOL >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
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
        if (!tc_wait(tc_smem_u32(&bar_full[s]), ph)) {
          atomicExch(p.err, 4u);
          break;
        }
        if (it == 0) tc_stamp(p, 2);
        if (it == nunits - 1) tc_stamp(p, 3);
        tc_fence_after();
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t sf_t = tmem + sf_col0 + (uint32_t)s * C::SF_COLS;
        const uint32_t sb = st + C::A_TILES * C::A_BYTES;
        const uint32_t ssf = sb + C::X_ROWS * 64;
        const bool part_end = (ks == p.KS - 1) || (it == nunits - 1);
        if (TPX_DBG(p) & 32) {  // timing experiment: copies issued by this thread, in order with its MMAs
#pragma unroll
          for (int q = 0; q < C::SF_BLOCKS; q++) tc_cp_sf(sf_t + q * 4, tc_sf_desc(ssf + q * 512));
        } else if (!(TPX_DBG(p) & 16)) {
          if (!tc_wait(tc_smem_u32(&bar_sf[s]), ph)) { atomicExch(p.err, 5u); break; }
          tc_fence_after();
        }
#pragma unroll
        for (int kk = 0; kk < UKS; kk++) {
          if (TPX_DBG(p) & 1) break;
#pragma unroll
          for (int j = 0; j < 2; j++) {  // k 64*j .. 64*j+63 of the step: 32 bytes along the row, scale bytes 2j and 2j+1
            const uint32_t sfid = (uint32_t)(2 * j);
            const uint32_t idesc = idesc0 | (sfid << 29) | (sfid << 4);
            const uint64_t bdesc = tc_smem_desc64(sb + kk * 4 * C::B_BYTES) + (uint64_t)(2 * j);
#pragma unroll
            for (int d = 0; d < C::NW; d++) {
              const uint64_t adesc = tc_smem_desc64(st + (kk * C::NW + d) * C::A_BYTES) + (uint64_t)(2 * j);
              const uint32_t acc = (fresh && kk == 0 && j == 0) ? 0u : 1u;
              tc_mma_f4(tmem + d * C::NCOL, adesc, bdesc, idesc, (sf_t + (kk * C::NW + d) * 4) | (sfid << 30),
                        (sf_t + (C::A_TILES + kk) * 4) | (sfid << 30), acc);
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
  } else if (warp == 6) {
    // ------------------------------------------------------------ scale-factor copies (shared -> tensor memory)
    // Issued by their own thread so that they are not queued in order between the MMAs; a stage's tensor-memory
    // columns are free again once its shared memory has been refilled (the refill waits for the stage's MMAs).
    if (lane == 0 && !(TPX_DBG(p) & 48)) {
      for (int it = 0; it < nunits; it++) {
        const int s = it % C::STAGES;
        const uint32_t ph = (uint32_t)((it / C::STAGES) & 1);
        if (!tc_wait(tc_smem_u32(&bar_full[s]), ph)) { atomicExch(p.err, 7u); break; }
        tc_fence_after();
        const uint32_t ssf = smem_base + (uint32_t)s * C::STAGE_BYTES + C::A_TILES * C::A_BYTES + C::X_ROWS * 64;
        const uint32_t sf_t = tmem + sf_col0 + (uint32_t)s * C::SF_COLS;
#pragma unroll
        for (int q = 0; q < C::SF_BLOCKS; q++) tc_cp_sf(sf_t + q * 4, tc_sf_desc(ssf + q * 512));
        tc_commit(tc_smem_u32(&bar_sf[s]));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int sub = warp & 3;  // tensor-memory lanes 32*sub .. 32*sub+31 belong to this warp
    const uint32_t lane_base = ((uint32_t)(sub * 32)) << 16;
    int tile = tile0, ks = ks0;
    int part_first_ks = ks0;
    uint32_t acc_phase = 0;
    bool dead = false;
    asm volatile("griddepcontrol.wait;" ::: "memory");  // scratch, residual and gate inputs belong to earlier grids
    for (int it = 0; it < nunits && !dead; it++) {
      const bool part_end = (ks == p.KS - 1) || (it == nunits - 1);
      if (part_end) {
        if (!tc_wait(tc_smem_u32(&bar_acc_full), acc_phase)) {
          if (lane == 0) atomicExch(p.err, 6u);
          dead = true;
          break;
        }
        acc_phase ^= 1;
        tc_fence_after();
        if (threadIdx.x == 64 && it == nunits - 1) tc_stamp(p, 5);
        const int tn = tile / p.TM, tm = tile % p.TM;
        const int row = sub * 32 + lane;
        const int n = tn * 128 + row;
        const int tok0 = tm * TOK;
        const bool whole = (part_first_ks == 0) && (ks == p.KS - 1);
        // partial tiles live as [slot][weight][128 rows][TOK] fp32: a thread owns one row, TOK consecutive floats
        float* myslot = p.partial + (((size_t)blockIdx.x * 2 + (tile == tile0 ? 0 : 1)) * C::NW) * TOK * 128 + (size_t)row * TOK;
#pragma unroll 1
        for (int c0 = 0; c0 < TOK; c0 += 16) {
          float r0[16], r1[16];
          {  // the four terms' column groups
            uint32_t a[4][16], b[4][16];
#pragma unroll
            for (int t = 0; t < 4; t++) {
              tc_ld_x16(tmem + lane_base + t * TOK + c0, a[t]);
              if (DUAL) tc_ld_x16(tmem + lane_base + C::NCOL + t * TOK + c0, b[t]);
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 16; j++) {
              r0[j] = (__uint_as_float(a[0][j]) + __uint_as_float(a[1][j])) + (__uint_as_float(a[2][j]) + __uint_as_float(a[3][j]));
              r1[j] = DUAL ? (__uint_as_float(b[0][j]) + __uint_as_float(b[1][j])) + (__uint_as_float(b[2][j]) + __uint_as_float(b[3][j])) : 0.0f;
            }
          }
          if (whole) {
            if (n < p.N && tok0 + c0 < p.M) {  // uniform over the warp (N is a multiple of 32)
              float st[16];
              tc_finish16<DUAL>(p, tok0 + c0, n, r0, r1, p.emit.terms ? st : nullptr);
              if (p.emit.terms) tc_emit16_lanes(p.emit, tok0 + c0, p.M - tok0 - c0, n, st);
            }
          } else if (p.cluster > 1) {  // partial of a cluster member: [weight][128 rows][TOK] fp32 at the start of its stages
            const uint32_t sp = smem_base + (uint32_t)((row * TOK + c0) * 4);
#pragma unroll
            for (int q = 0; q < 4; q++) {
              tc_st_shared_f4(sp + q * 16, make_float4(r0[4 * q], r0[4 * q + 1], r0[4 * q + 2], r0[4 * q + 3]));
              if (DUAL)
                tc_st_shared_f4(sp + 128 * TOK * 4 + q * 16, make_float4(r1[4 * q], r1[4 * q + 1], r1[4 * q + 2], r1[4 * q + 3]));
            }
          } else {
#pragma unroll
            for (int q = 0; q < 4; q++) {
              __stcg(reinterpret_cast<float4*>(myslot + c0) + q, make_float4(r0[4 * q], r0[4 * q + 1], r0[4 * q + 2], r0[4 * q + 3]));
              if (DUAL)
                __stcg(reinterpret_cast<float4*>(myslot + (size_t)TOK * 128 + c0) + q,
                       make_float4(r1[4 * q], r1[4 * q + 1], r1[4 * q + 2], r1[4 * q + 3]));
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) tc_mbar_arrive(tc_smem_u32(&bar_acc_empty));  // tensor memory may be overwritten
      }
      if (++ks == p.KS) {
        ks = 0;
        tile++;
        part_first_ks = 0;
      }
    }
  }
  if (threadIdx.x == 64) tc_stamp(p, 6);
  tc_fence_before();
  __syncthreads();
  if (p.cluster > 1) {
    // every member's partial is in its own shared memory; each member takes some 16-token chunks of the tile, adds
    // the members' parts in rank order (distributed shared memory reads) and runs the epilogue on them. Nobody
    // leaves before all have finished reading.
    tc_cluster_sync();
    if (warp >= 2) {
      const int sub = warp & 3;
      const int row = sub * 32 + lane;
      const int tn = (int)(ctile / p.TM), tm = (int)(ctile % p.TM);
      const int n = tn * 128 + row, tok0 = tm * TOK;
#pragma unroll 1
      for (int c0 = crank * 16; c0 < TOK; c0 += 16 * p.cluster) {
        float v[16], v2[16];
#pragma unroll
        for (int j = 0; j < 16; j++) v[j] = v2[j] = 0.0f;
        const uint32_t sp = smem_base + (uint32_t)((row * TOK + c0) * 4);
        tc_cluster_sum<4, (OCC == 2 ? 2 : 4)>(sp, p.cluster, v);
        if (DUAL) tc_cluster_sum<4, (OCC == 2 ? 2 : 4)>(sp + 128 * TOK * 4, p.cluster, v2);
        if (n < p.N && tok0 + c0 < p.M) tc_finish16<DUAL>(p, tok0 + c0, n, v, v2);
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
struct Tc4Plan {
  int tok, uks, occ;
  int TN, TM, KS, KU, Mpad, grid, xbox, whole_tiles, cluster;
  size_t off_terms, off_sfb, off_partial, total;
};

// Work split as in the 8-bit-container kernel: whole tiles when tiles are about as many as SMs (or many per SM), a
// cluster per tile cutting K when tiles are few, otherwise (tile, k unit) ranges with a fix-up pass.
static Tc4Plan tc4_plan(int64_t M, int64_t N, int64_t K, bool pair) {
  Tc4Plan pl;
  pl.tok = M <= 16 ? 16 : 32;
  pl.occ = (knobs().tc4_occ == 2 && (pl.tok == 16 || !pair)) ? 2 : 1;
  pl.uks = (pl.occ == 2 && pair) ? 1 : 2;
  pl.KS = tc_padded_ks(K, pair);
  pl.KU = pl.KS / pl.uks;
  pl.TN = (int)((N + 127) / 128);
  pl.TM = (int)((M + pl.tok - 1) / pl.tok);
  pl.Mpad = pl.TM * pl.tok;
  const int xrows = pl.uks * 4 * pl.tok;
  pl.xbox = xrows > 256 ? 256 : xrows;
  const long long U = (long long)pl.TN * pl.TM * pl.KU;
  const long long T = (long long)pl.TN * pl.TM;
  const int sms = sm_count();
  pl.whole_tiles = (T * 10 >= (long long)sms * 7 && T <= sms) || T >= 8LL * sms;
  if (knobs().tc_whole >= 0) pl.whole_tiles = knobs().tc_whole;
  pl.grid = pl.whole_tiles ? (int)(T < sms ? T : sms) : (int)(U < sms ? U : sms);
  pl.cluster = 1;
  if (!pl.whole_tiles && T * 2 <= sms) {
    int c = (int)(sms / T);
    if (c > 8) c = 8;
    if (c > pl.KU) c = pl.KU;
    if (c > 1) pl.cluster = c;
  }
  if (knobs().tc_cluster == 0) pl.cluster = 1;
  size_t o = kTcCounterBytes;
  auto bump = [&](size_t bytes) { size_t r = o; o += (bytes + 1023) & ~(size_t)1023; return r; };
  pl.off_terms = bump((size_t)pl.Mpad * pl.KS * 4 * 64);
  pl.off_sfb = bump((size_t)pl.TM * pl.KS * 512);
  pl.off_partial = bump((size_t)pl.grid * 2 * (pair ? 2 : 1) * pl.tok * 128 * sizeof(float));
  pl.total = o;
  return pl;
}

template <int TOK, bool DUAL, int UKS, int OCC = 1>
static int tc4_launch(const CUtensorMap& w, const CUtensorMap& x, const TcParams& p, int grid, cudaStream_t st) {
  using C = Tc4Cfg<TOK, DUAL, UKS, OCC>;
  static bool opted[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || !opted[dev]) {
    TPX_CUDA_OK(cudaFuncSetAttribute(qlinear_tc4_kernel<TOK, DUAL, UKS, OCC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    if (dev >= 0 && dev < 16) opted[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kTc4Threads);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (p.cluster > 1) {
    // one cluster per tile, all of them resident at once; the largest cluster size that fits is used
    const int tiles = p.TN * p.TM;
    static int fits[16][9] = {};  // 0 unknown, else 1 + the number of clusters of this size that can be resident
    for (int c = p.cluster; c > 1; c--) {
      cudaLaunchConfig_t cc = cfg;
      cc.gridDim = dim3((unsigned)(tiles * c));
      attr[1].id = cudaLaunchAttributeClusterDimension;
      attr[1].val.clusterDim.x = (unsigned)c;
      attr[1].val.clusterDim.y = 1;
      attr[1].val.clusterDim.z = 1;
      cc.numAttrs = 2;
      int& f = fits[(dev >= 0 && dev < 16) ? dev : 0][c];
      if (f == 0) {
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, qlinear_tc4_kernel<TOK, DUAL, UKS, OCC>, &cc);
        if (e != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
        f = 1 + n;
      }
      if (f - 1 >= tiles) {
        TcParams q = p;
        q.cluster = c;
        count_launch();
        TPX_CUDA_OK(cudaLaunchKernelEx(&cc, qlinear_tc4_kernel<TOK, DUAL, UKS, OCC>, w, x, q));
        return TPX_OK;
      }
    }
    TcParams q = p;
    q.cluster = 1;
    return tc4_launch<TOK, DUAL, UKS, OCC>(w, x, q, grid, st);
  }
  count_launch();
  TPX_CUDA_OK(cudaLaunchKernelEx(&cfg, qlinear_tc4_kernel<TOK, DUAL, UKS, OCC>, w, x, p));
  if (!p.whole_tiles && grid > 1) return tc_launch_fixup(DUAL, p, TOK, grid, st);  // tiles cut between CTAs
  return TPX_OK;
}

size_t tc4_scratch_bytes(int64_t M, int64_t N, int64_t K, bool pair) { return tc4_plan(M, N, K, pair).total; }

int tc4_run(const uint8_t* wq, const uint8_t* sfa, bool pair, const uint16_t* x, int64_t M, int64_t N, int64_t K, const TcParams& base,
            void* scratch, size_t scratch_bytes, cudaStream_t st, const TcNorm* norm) {
  TPX_REQUIRE(M >= 1 && M <= 32, TPX_ERR_UNSUPPORTED, "qlinear_mxfp4_tc (packed-fp4 kernel): 1..32 tokens, got %ld", (long)M);
  const Tc4Plan pl = tc4_plan(M, N, K, pair);
  TPX_REQUIRE(scratch && scratch_bytes >= pl.total, TPX_ERR_SCRATCH, "qlinear_mxfp4_tc: scratch of %zu bytes needed, %zu given", pl.total,
              scratch_bytes);
  unsigned char* sc = reinterpret_cast<unsigned char*>(scratch);
  uint8_t *terms = sc + pl.off_terms, *sfb = sc + pl.off_sfb;
  int rc = tc4_launch_split(x, (int)M, (int)K, pl.Mpad, pl.KS, pl.tok, pl.uks, terms, sfb, st, norm);
  if (rc) return rc;
  CUtensorMap mw, mx;
  // weight: 64-byte rows of 128 packed codes, 256 rows (two tiles) per request; activation terms: 64-byte rows
  rc = tc_make_map64(&mw, wq, (uint64_t)pl.TN * pl.KS * (pair ? 2 : 1) * 128, 256);
  if (rc) return rc;
  rc = tc_make_map64(&mx, terms, (uint64_t)pl.Mpad * pl.KS * 4, (uint32_t)pl.xbox);
  if (rc) return rc;
  TcParams p = base;
  p.sfa = sfa; p.sfa2 = nullptr; p.sfb = sfb;
  p.partial = reinterpret_cast<float*>(sc + pl.off_partial);
  p.counters = reinterpret_cast<unsigned*>(sc);
  p.err = reinterpret_cast<unsigned*>(sc + kTcCounterBytes - 4);
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.KS = pl.KU; p.TN = pl.TN; p.TM = pl.TM;
  p.whole_tiles = pl.whole_tiles; p.cluster = pl.cluster;
  if (!pl.whole_tiles) p.emit.terms = nullptr;  // only the whole-tile epilogue hands its output over
  tc_note_emitted(p.emit.terms != nullptr);
  if (pl.occ == 2) {
    if (pair) return tc4_launch<16, true, 1, 2>(mw, mx, p, pl.grid, st);
    if (pl.tok == 16) return tc4_launch<16, false, 2, 2>(mw, mx, p, pl.grid, st);
    return tc4_launch<32, false, 2, 2>(mw, mx, p, pl.grid, st);
  }
  if (pair) {
    if (pl.tok == 16) return tc4_launch<16, true, 2>(mw, mx, p, pl.grid, st);
    return tc4_launch<32, true, 2>(mw, mx, p, pl.grid, st);
  }
  if (pl.tok == 16) return tc4_launch<16, false, 2>(mw, mx, p, pl.grid, st);
  return tc4_launch<32, false, 2>(mw, mx, p, pl.grid, st);
}

}  // namespace tpx
