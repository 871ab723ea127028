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
// below 2^-18 of the block maximum). The two terms sit side by side as 2*TOK columns of one MMA, so the
// weight tile is read from shared memory once; the epilogue adds the two halves of the fp32 tile.
//
//   rows of W (output features) = M of the MMA (128 per tile), tokens = N (TOK per tile), K step 128
//   warp 0   : TMA producer (W tiles, activation terms, scale-factor blocks) into a ring of stages
//   warp 1   : allocates tensor memory; per stage copies the scale-factor blocks from shared to tensor
//              memory (tcgen05.cp, which runs in order with the MMAs of the same thread), issues the
//              MMAs and commits the stage back to the producer
//   warps 2-5: epilogue (tensor memory -> registers -> bias / activation / gate / residual -> y)
//
// The TMA unit of an SM retires roughly one copy request per 0.12 us whatever its size, so a stage is
// fetched with few, large requests: 16 KiB of packed weight per request (a gate/up pair of tiles, or two
// k steps of one weight), both activation terms of all k steps of the unit in one request, and one request
// each for the weight and activation scale-factor blocks.
//
// Work is the flat list of (output tile, k unit) units cut into equal contiguous ranges, one CTA per SM:
// every SM streams the same number of weight bytes. A tile cut between CTAs leaves fp32 partial tiles in scratch
// (one slot per contributor); a small second kernel, launched as a programmatic dependent so that its launch
// latency hides behind the GEMM, adds them in CTA order and runs the epilogue. Doing this inside the GEMM (last
// arriver per tile) cost a store -> atomic -> load chain at loaded-memory latency (~2 us per hop).
#include "tpx_tc_ptx.cuh"
#include <cuda_fp8.h>

namespace tpx {

// ---------------------------------------------------------------- activation split
// x[M][K] bf16 -> two E4M3 terms and the UE8M0 scale blocks, one thread per (token, 32-wide block), written
// in the order the GEMM fetches them:
//   terms [TM][KU][UKS][2 terms][TOK rows][128 bytes]     (one k step of one term = a TOK x 128 operand tile)
//   sfb   [TM][KU][UKS][ceil(2*TOK/128)][512]   scale blocks over the 2*TOK MMA columns (hi columns, then lo
//         columns with the same scales): byte (c%32)*16 + ((c%128)/32)*4 + j of block c/128 for column c
// Padding rows and padding columns get zeros with scale 2^0.
// rowmap 2 (16 tokens on the M side, four per 32-lane quarter of tensor memory so that four warps share the
// epilogue): 32 rows per k step in memory, token r at row 8*(r/4) + r%4 (hi) and 4 further (lo); the MMA reads them
// through a descriptor whose 8-row groups are 256 bytes apart, as its rows 32*(r/4) + r%4 and 16 further.
// rowmap 1 (tokens on the M side of the MMA, one token tile): a k step holds 2*TOK rows with the hi row of token r
// at 32*(r/16) + r%16 and its lo row 16 further, so that both terms of a token sit in the same 32-lane quarter of
// tensor memory; one scale block of 128 rows per k step.
__global__ void split_activations_kernel(const uint16_t* __restrict__ x, int M, int K, int Mpad, int KS, int TOK, int UKS,
                                         int rowmap, uint8_t* __restrict__ terms, uint8_t* __restrict__ sfb) {
  // let the GEMM that consumes these terms start its prologue and weight prefetch now; it waits for this
  // grid to finish (griddepcontrol.wait) before it touches the terms
  pdl_trigger();
  pdl_wait();  // x and the scratch belong to earlier grids until they have completed
  const int nb = KS * 4;
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
  const int tm = tok / TOK, r = tok % TOK, ks = kb / 4, j = kb % 4;
  const int KU = KS / UKS, ku = ks / UKS, kk = ks % UKS;
  const size_t step = ((size_t)tm * KU + ku) * UKS + kk;  // k step in fetch order
  if (rowmap >= 1) {
    // rows in memory (rh, rl) and rows as the MMA numbers them (gh, gl: the scale bytes are indexed by those)
    int rh, rl, gh, gl;
    if (rowmap == 1) {
      rh = gh = 32 * (r / 16) + (r % 16);
      rl = gl = rh + 16;
    } else {
      rh = 8 * (r / 4) + (r % 4);
      rl = rh + 4;
      gh = 32 * (r / 4) + (r % 4);
      gl = gh + 16;
    }
    uint4* dh = reinterpret_cast<uint4*>(terms + (step * 2 * TOK + rh) * 128 + j * 32);
    uint4* dl = reinterpret_cast<uint4*>(terms + (step * 2 * TOK + rl) * 128 + j * 32);
    dh[0] = make_uint4(ph[0], ph[1], ph[2], ph[3]);
    dh[1] = make_uint4(ph[4], ph[5], ph[6], ph[7]);
    dl[0] = make_uint4(pl[0], pl[1], pl[2], pl[3]);
    dl[1] = make_uint4(pl[4], pl[5], pl[6], pl[7]);
    uint8_t* blk = sfb + step * 512;
    blk[(gh % 32) * 16 + (gh / 32) * 4 + j] = (uint8_t)(e + 127);
    blk[(gl % 32) * 16 + (gl / 32) * 4 + j] = (uint8_t)(e + 127);
    return;
  }
  uint4* dh = reinterpret_cast<uint4*>(terms + ((step * 2 + 0) * TOK + r) * 128 + j * 32);
  uint4* dl = reinterpret_cast<uint4*>(terms + ((step * 2 + 1) * TOK + r) * 128 + j * 32);
  dh[0] = make_uint4(ph[0], ph[1], ph[2], ph[3]);
  dh[1] = make_uint4(ph[4], ph[5], ph[6], ph[7]);
  dl[0] = make_uint4(pl[0], pl[1], pl[2], pl[3]);
  dl[1] = make_uint4(pl[4], pl[5], pl[6], pl[7]);
  // the hi columns are MMA columns r, the lo columns TOK + r: both carry this scale
  const int per = (2 * TOK + 127) / 128;
  uint8_t* blk = sfb + step * per * 512;
  const int r2 = TOK + r;
  blk[(r / 128) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + j] = (uint8_t)(e + 127);
  blk[(r2 / 128) * 512 + (r2 % 32) * 16 + ((r2 % 128) / 32) * 4 + j] = (uint8_t)(e + 127);
}

// RMSNorm fused into the split: one CTA per token row (rows up to 8192 elements), the row kept in registers.
// y = bf16(x * rsqrt(mean(x^2) + eps) * gamma) is what llama_rms_norm (src/csrc/llm/fused_llm_infer.cpp:336-363)
// hands to the next linear; it is split here without a trip through memory. Same output layouts as above.
constexpr int kNsThreads = 256;
constexpr int kNsVecs = 4;
__global__ void __launch_bounds__(kNsThreads) rmsnorm_split_kernel(const uint16_t* __restrict__ x, const void* __restrict__ gamma,
                                                                   int gamma_f32, float eps, int M, int K, int KS, int TOK, int UKS,
                                                                   int rowmap, uint8_t* __restrict__ terms, uint8_t* __restrict__ sfb) {
  __shared__ float red[kNsThreads / 32];
  pdl_trigger();
  pdl_wait();
  const int tok = blockIdx.x;
  const bool live_row = tok < M;
  const int nv = K / 8, nvp = KS * 16;  // 8-element vectors of the row, and of the row padded to whole k steps
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)tok * K);
  uint4 v[kNsVecs];
  float gm[kNsVecs][8];  // gamma is fetched together with the row, not after the reduction
  float ss = 0.0f;
#pragma unroll
  for (int q = 0; q < kNsVecs; q++) {
    const int i = threadIdx.x + q * kNsThreads;
    const bool have = live_row && i < nv;
    v[q] = have ? xr[i] : make_uint4(0, 0, 0, 0);
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
  }
#pragma unroll
  for (int q = 0; q < kNsVecs; q++) {
    const uint32_t w[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float a = bf16_bits_to_f32((uint16_t)(w[j] & 0xffff)), b = bf16_bits_to_f32((uint16_t)(w[j] >> 16));
      ss += a * a + b * b;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int w = 0; w < kNsThreads / 32; w++) tot += red[w];
  const float inv = rsqrtf(tot / (float)K + eps);

  const int tm = tok / TOK, r = tok % TOK, KU = KS / UKS;
#pragma unroll
  for (int q = 0; q < kNsVecs; q++) {
    const int i = threadIdx.x + q * kNsThreads;  // vector index: four consecutive threads hold one block of 32
    const bool in = i < nvp;
    float f[8];
    {
      const uint32_t w[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
#pragma unroll
      for (int j = 0; j < 4; j++) {  // the normalised value rounded to bf16, as the separate kernel stores it
        f[2 * j] = bf16_bits_to_f32(f32_to_bf16_bits(bf16_bits_to_f32((uint16_t)(w[j] & 0xffff)) * inv * gm[q][2 * j]));
        f[2 * j + 1] = bf16_bits_to_f32(f32_to_bf16_bits(bf16_bits_to_f32((uint16_t)(w[j] >> 16)) * inv * gm[q][2 * j + 1]));
      }
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(f[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    int e = 0;
    if (amax > 0.0f && amax < INFINITY) e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127 - 7;
    e = max(-127, min(127, e));
    const float down = __uint_as_float((uint32_t)(127 - e) << 23);
    uint32_t ph[2], pl[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; h2++) {
      uint32_t h4 = 0, l4 = 0;
#pragma unroll
      for (int j = 0; j < 2; j++) {
        float a = f[4 * h2 + 2 * j] * down, b = f[4 * h2 + 2 * j + 1] * down;
        __nv_fp8x2_storage_t hs = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
        __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(hs, __NV_E4M3);
        float ra = a - __half2float(__ushort_as_half(hr.x)), rb = b - __half2float(__ushort_as_half(hr.y));
        __nv_fp8x2_storage_t ls = __nv_cvt_float2_to_fp8x2(make_float2(ra, rb), __NV_SATFINITE, __NV_E4M3);
        h4 |= (uint32_t)hs << (16 * j);
        l4 |= (uint32_t)ls << (16 * j);
      }
      ph[h2] = h4;
      pl[h2] = l4;
    }
    if (!in) continue;
    const int kb = i >> 2, part = i & 3, ks = kb >> 2, j = kb & 3;
    const size_t step = ((size_t)tm * KU + ks / UKS) * UKS + ks % UKS;
    int rh, rl, gh, gl;  // rows of the hi and lo term in memory, and as the MMA numbers them (scale bytes)
    size_t blk_off;
    if (rowmap == 1) {
      rh = gh = 32 * (r / 16) + (r % 16);
      rl = gl = rh + 16;
      blk_off = step * 512;
    } else if (rowmap == 2) {
      rh = 8 * (r / 4) + (r % 4);
      rl = rh + 4;
      gh = 32 * (r / 4) + (r % 4);
      gl = gh + 16;
      blk_off = step * 512;
    } else {
      rh = gh = r;
      rl = gl = TOK + r;
      blk_off = step * (size_t)((2 * TOK + 127) / 128) * 512;
    }
    *reinterpret_cast<uint2*>(terms + (step * 2 * TOK + rh) * 128 + j * 32 + part * 8) = make_uint2(ph[0], ph[1]);
    *reinterpret_cast<uint2*>(terms + (step * 2 * TOK + rl) * 128 + j * 32 + part * 8) = make_uint2(pl[0], pl[1]);
    if (part == 0) {
      uint8_t* blk = sfb + blk_off;
      blk[(gh / 128) * 512 + (gh % 32) * 16 + ((gh % 128) / 32) * 4 + j] = (uint8_t)(e + 127);
      blk[(gl / 128) * 512 + (gl % 32) * 16 + ((gl % 128) / 32) * 4 + j] = (uint8_t)(e + 127);
    }
  }
}

// ---------------------------------------------------------------- repack for the tensor-core path
// Interchange tensors of remap_and_quantize_mxfp4 -> tiled packed codes and scale-factor blocks.
//   one weight : wq [TN][KS][128 rows][64 bytes]          sfa [TN][KS][512]          KS padded to a multiple of 4
//   gate/up    : wq [TN][KS][2][128 rows][64 bytes]       sfa [TN][KS][2][512]       KS padded to a multiple of 2
// (low nibble = even k; rows beyond N and columns beyond K hold zero codes and zero scale bytes). A copy
// request of 256 such 64-byte rows is 16 KiB of consecutive addresses. One thread per output byte of wq.
__global__ void repack_mxfp4_tc_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                       const uint8_t* __restrict__ codes2, const uint8_t* __restrict__ scales2, int64_t N,
                                       int64_t K, int64_t KS, uint8_t* __restrict__ wq, uint8_t* __restrict__ sfa) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t C1 = K / 64;
  const int64_t TN = (N + 127) / 128;
  const int NW = codes2 ? 2 : 1;
  if (idx < TN * KS * NW * 8192) {
    int64_t tile = idx / 8192;  // (tn*KS + ks)*NW + d
    int d = (int)(tile % NW);
    int64_t tk = tile / NW;
    int r = (int)((idx % 8192) / 64), kb = (int)(idx % 64);
    int64_t n = (tk / KS) * 128 + r, k = (tk % KS) * 128 + 2 * kb;
    const uint8_t* src = d ? codes2 : codes;
    // source byte (k1,c1,r,k2) = W[32k1+k2][64c1+2r+{0,1}]: already the (k, k+1) pair
    wq[idx] = (n < N && k < K) ? src[(((n / 32) * C1 + k / 64) * 32 + (k % 64) / 2) * 32 + (n % 32)] : (uint8_t)0;
  }
  if (idx < TN * KS * NW * 512) {
    int64_t blk = idx / 512;  // (tn*KS + ks)*NW + d
    int d = (int)(blk % NW);
    int64_t tk = blk / NW;
    int b = (int)(idx % 512);
    int r = (b / 16) + 32 * ((b % 16) / 4), j = b % 4;
    int64_t n = (tk / KS) * 128 + r, kbk = (tk % KS) * 4 + j;
    const uint8_t* src = d ? scales2 : scales;
    uint8_t sv = 0;
    if (n < N && kbk * 32 < K) sv = src[(((n / 32) * C1 + kbk / 2) * 2 + (kbk & 1)) * 32 + (n % 32)];
    sfa[idx] = sv;
  }
}

// 8-bit floating-point weights (E4M3 or E5M2 bytes, plain [N][K]) -> the same tiling with 128-byte rows:
//   one weight : wq [TN][KS][128 rows][128 bytes]     gate/up : wq [TN][KS][2][128 rows][128 bytes]
// and scale blocks of the constant 1.0 (these formats carry no scales). One thread per 16 bytes of wq.
__global__ void repack_fp8_tc_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ w2, int64_t N, int64_t K, int64_t KS,
                                     uint8_t* __restrict__ wq, uint8_t* __restrict__ sfa) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t TN = (N + 127) / 128;
  const int NW = w2 ? 2 : 1;
  if (idx < TN * KS * NW * 1024) {
    int64_t tile = idx / 1024;  // (tn*KS + ks)*NW + d
    int d = (int)(tile % NW);
    int64_t tk = tile / NW;
    int r = (int)((idx % 1024) / 8), c = (int)(idx % 8);
    int64_t n = (tk / KS) * 128 + r, k = (tk % KS) * 128 + 16 * c;
    const uint8_t* src = d ? w2 : w;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (n < N && k < K) v = *reinterpret_cast<const uint4*>(src + n * K + k);  // K is a multiple of 16
    reinterpret_cast<uint4*>(wq)[idx] = v;
  }
  if (idx < TN * KS * NW * 32) reinterpret_cast<uint4*>(sfa)[idx] = make_uint4(0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
}

// ---------------------------------------------------------------- the GEMM kernel
// TOK tokens per tile, DUAL = gate/up pair, UKS = k steps (of 128) per pipeline unit.
template <int TOK, bool DUAL, int UKS>
struct TcCfg {
  static constexpr int NW = DUAL ? 2 : 1;
  static constexpr int A_BYTES = 128 * 128;            // shared-memory footprint of an unpacked 128 x 128 fp4 tile
  static constexpr int A_TX = 128 * 64;                // bytes the copy accounts for (the packed data)
  static constexpr int A_TILES = UKS * NW;             // tiles per unit, fetched 2 at a time (256 rows, 16 KiB)
  static constexpr int B_BYTES = TOK * 128;            // one term of one k step
  static constexpr int X_ROWS = UKS * 2 * TOK;         // rows of 128 bytes of both terms of the unit
  static constexpr int X_BOX = X_ROWS > 256 ? 256 : X_ROWS;
  static constexpr int NCOL = 2 * TOK;                 // MMA N: hi columns then lo columns
  static constexpr int SFB_PER = (NCOL + 127) / 128;   // activation scale blocks per k step
  static constexpr int SF_BLOCKS = UKS * (NW + SFB_PER);  // weight blocks first, then activation blocks
  static constexpr int RAW = A_TILES * A_BYTES + X_ROWS * 128 + SF_BLOCKS * 512;
  static constexpr int STAGE_BYTES = (RAW + 1023) / 1024 * 1024;
  static constexpr int TX = A_TILES * A_TX + X_ROWS * 128 + SF_BLOCKS * 512;
  static constexpr int BUDGET = 227 * 1024 - 2048;
  static constexpr int STAGES_RAW = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
  static constexpr int SF_COLS = SF_BLOCKS * 4;        // tensor-memory columns of one stage's scale factors
  static constexpr int D_COLS = NW * NCOL;
  static constexpr int COLS_RAW = D_COLS + STAGES * SF_COLS;
  static constexpr int TMEM_COLS = COLS_RAW <= 32 ? 32 : COLS_RAW <= 64 ? 64 : COLS_RAW <= 128 ? 128 : COLS_RAW <= 256 ? 256 : 512;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;  // + alignment slack
  static constexpr int W_BOX = A_TILES >= 2 ? 2 : 1;     // weight tiles per copy request (256 or 128 rows)
  // The epilogue is a chain of dependent scalar instructions per output value; one warp per 32-row quarter of tensor
  // memory runs it at a fraction of the issue rate, and the tile's MMAs wait for it. With 32 tokens or more every quarter
  // has two warps, each taking half of the 16-token chunks.
  static constexpr int EPI_SPLIT = TOK >= 32 ? 2 : 1;
  static constexpr int THREADS = 64 + 128 * EPI_SPLIT;
  static_assert(A_TILES % W_BOX == 0, "weight tiles are fetched W_BOX at a time");
  static_assert(STAGES >= 2, "at least two stages");
  static_assert(COLS_RAW <= 512, "tensor memory");
};

template <int TOK, bool DUAL, int UKS>
__global__ void __launch_bounds__(TcCfg<TOK, DUAL, UKS>::THREADS, 1)
qlinear_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, TcParams p) {
  using C = TcCfg<TOK, DUAL, UKS>;
  extern __shared__ unsigned char tc_smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[C::STAGES], bar_empty[C::STAGES];
  __shared__ __align__(8) unsigned long long bar_acc_full, bar_acc_empty;
  __shared__ uint32_t tmem_holder;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (tc_smem_u32(tc_smem_raw) + 1023u) & ~1023u;

  // this CTA's contiguous range of (tile, k unit) units; p.KS counts k units here
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
    }
    tc_mbar_init(tc_smem_u32(&bar_acc_full), 1);
    tc_mbar_init(tc_smem_u32(&bar_acc_empty), 4 * C::EPI_SPLIT);
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
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the fix-up kernel may get its CTAs ready

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      auto fetch_w = [&](int s, int tn, int ks) {  // weight tiles and their scale blocks: independent of the split kernel
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t bar = tc_smem_u32(&bar_full[s]);
        // 8-bit weights arrive byte for byte; packed 4-bit ones are accounted with their packed size
        const int w_tx = C::A_TILES * (p.wfmt ? C::A_BYTES : C::A_TX);
        tc_mbar_expect_tx(bar, ((TPX_DBG(p) & 2) ? C::TX - C::A_TILES * C::A_TX : C::TX - C::A_TILES * C::A_TX + w_tx) - ((TPX_DBG(p) & 128) ? C::X_ROWS * 128 + UKS * C::SFB_PER * 512 : 0));
        const int wtile = (tn * p.KS + ks) * C::A_TILES;  // first weight tile of the unit
        if (!(TPX_DBG(p) & 2)) {
#pragma unroll
          for (int r = 0; r < C::A_TILES / C::W_BOX; r++) tc_tma_2d(st + r * C::W_BOX * C::A_BYTES, &tmW, 0, (wtile + C::W_BOX * r) * 128, bar);
        }
        tc_bulk_g2s(st + C::A_TILES * C::A_BYTES + C::X_ROWS * 128, p.sfa + (size_t)wtile * 512, C::A_TILES * 512, bar);
      };
      auto fetch_x = [&](int s, int tm, int ks) {  // activation terms and their scale blocks
        const uint32_t st = smem_base + (uint32_t)s * C::STAGE_BYTES;
        const uint32_t bar = tc_smem_u32(&bar_full[s]);
        const uint32_t sb = st + C::A_TILES * C::A_BYTES;
        const int xrow = (tm * p.KS + ks) * C::X_ROWS;
#pragma unroll
        for (int r = 0; r < C::X_ROWS / C::X_BOX; r++) tc_tma_2d(sb + r * C::X_BOX * 128, &tmX, 0, xrow + r * C::X_BOX, bar);
        tc_bulk_g2s(sb + C::X_ROWS * 128 + C::A_TILES * 512, p.sfb + ((size_t)tm * p.KS + ks) * UKS * C::SFB_PER * 512,
                    UKS * C::SFB_PER * 512, bar);
      };
      // Units further ahead than the shared-memory stages reach are prefetched into L2: the bytes in flight from
      // HBM are then not limited by shared memory, and the stage copies find their data at L2 latency.
      auto prefetch_w = [&](int tn, int ks) {
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
        if (!(TPX_DBG(p) & 128)) fetch_x(s, tm, ks);
        if (++ks == p.KS) { ks = 0; tile++; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: A = E2M1 (5), B = E4M3 (0), both K-major, N = TOK, UE8M0 scales, M = 128
      const uint32_t idesc0 = ((p.wfmt == 0 ? 5u : p.wfmt == 1 ? 0u : 1u) << 7) | (0u << 10) | ((uint32_t)(C::NCOL >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
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
        const uint32_t ssf = sb + C::X_ROWS * 128;
        const bool part_end = (ks == p.KS - 1) || (it == nunits - 1);
        if (TPX_DBG(p) & 1) {
          tc_mbar_arrive(tc_smem_u32(&bar_empty[s]));
          if (part_end) tc_mbar_arrive(tc_smem_u32(&bar_acc_full));
        } else {
#pragma unroll
          for (int q = 0; q < C::SF_BLOCKS; q++) tc_cp_sf(sf_t + q * 4, tc_sf_desc(ssf + q * 512));
#pragma unroll
          for (int kk = 0; kk < UKS; kk++) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const uint32_t idesc = idesc0 | ((uint32_t)j << 29) | ((uint32_t)j << 4);
              const uint64_t bdesc = tc_smem_desc(sb + kk * 2 * C::B_BYTES) + (uint64_t)(2 * j);
#pragma unroll
              for (int d = 0; d < C::NW; d++) {
                const uint64_t adesc = tc_smem_desc(st + (kk * C::NW + d) * C::A_BYTES) + (uint64_t)(2 * j);
                const uint32_t acc = (fresh && kk == 0 && j == 0) ? 0u : 1u;
                tc_mma(tmem + d * C::NCOL, adesc, bdesc, idesc, (sf_t + (kk * C::NW + d) * 4) | ((uint32_t)j << 30),
                       (sf_t + (C::A_TILES + kk * C::SFB_PER) * 4) | ((uint32_t)j << 30), acc);
              }
            }
          }
          tc_commit(tc_smem_u32(&bar_empty[s]));
          if (part_end) tc_commit(tc_smem_u32(&bar_acc_full));
        }
        fresh = part_end;
        if (++ks == p.KS) ks = 0;
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
        constexpr int TPW = TOK / C::EPI_SPLIT;  // tokens of this warp: [cpart * TPW, +TPW)
        const int cpart = (warp - 2) >> 2;
#pragma unroll 1
        for (int c0 = cpart * TPW; c0 < (cpart + 1) * TPW; c0 += 16) {
          float r0[16], r1[16];
          {  // hi columns + lo columns
            uint32_t a0[16], t0[16], a1[16], t1[16];
            tc_ld_x16(tmem + lane_base + c0, a0);
            tc_ld_x16(tmem + lane_base + TOK + c0, t0);
            if (DUAL) {
              tc_ld_x16(tmem + lane_base + C::NCOL + c0, a1);
              tc_ld_x16(tmem + lane_base + C::NCOL + TOK + c0, t1);
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 16; j++) {
              r0[j] = __uint_as_float(a0[j]) + __uint_as_float(t0[j]);
              r1[j] = DUAL ? __uint_as_float(a1[j]) + __uint_as_float(t1[j]) : 0.0f;
            }
          }
          if (whole) {
            if (n < p.N && tok0 + c0 < p.M) tc_finish16<DUAL>(p, tok0 + c0, n, r0, r1);
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
    if (warp >= 2 && warp < 6) {  // 16-token chunks of the tile go round the members
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
        tc_cluster_sum<4, 4>(sp, p.cluster, v);
        if (DUAL) tc_cluster_sum<4, 4>(sp + 128 * TOK * 4, p.cluster, v2);
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

// ---------------------------------------------------------------- fix-up of tiles cut between CTAs
// One CTA of 128 threads (= the 128 rows of a tile) per (tile, 16-token chunk). Contributors of a tile are the
// consecutive GEMM CTAs cfirst..clast; CTA c keeps its part of the tile in slot 0 if the tile is the first it
// touched, else in slot 1. Summation order is fixed (CTA order), so results do not depend on timing.
template <bool DUAL>
__global__ void __launch_bounds__(128) tc_fixup_kernel(TcParams p, int TOK, int G) {
  constexpr int NW = DUAL ? 2 : 1;
  pdl_trigger();
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int tile = blockIdx.x, c0 = blockIdx.y * 16, row = threadIdx.x;
  const long long U = (long long)p.TN * p.TM * p.KS;
  const long long ta = (long long)tile * p.KS, tb = ta + p.KS - 1;
  const int cfirst = (int)(((ta + 1) * G - 1) / U), clast = (int)(((tb + 1) * G - 1) / U);
  if (cfirst == clast) return;  // one CTA had the whole tile and finished it itself
  const int tn = tile / p.TM, tm = tile % p.TM;
  const int n = tn * 128 + row, tok0 = tm * TOK;
  if (n >= p.N || tok0 + c0 >= p.M) return;
  float v[16], v2[16];
#pragma unroll
  for (int j = 0; j < 16; j++) v[j] = v2[j] = 0.0f;
#pragma unroll 1
  for (int cb = cfirst; cb <= clast; cb += 4) {  // four contributors' loads in flight at a time
    uint4 t[4][NW][4];
#pragma unroll
    for (int cc = 0; cc < 4; cc++) {
      const int c = cb + cc;
      if (c <= clast) {
        const int ctile0 = (int)(((long long)c * U / G) / p.KS);
        const float* slot = p.partial + (((size_t)c * 2 + (tile == ctile0 ? 0 : 1)) * NW) * TOK * 128 + (size_t)row * TOK + c0;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          t[cc][0][q] = __ldcg(reinterpret_cast<const uint4*>(slot) + q);
          if (DUAL) t[cc][NW - 1][q] = __ldcg(reinterpret_cast<const uint4*>(slot + (size_t)TOK * 128) + q);
        }
      }
    }
#pragma unroll
    for (int cc = 0; cc < 4; cc++) {
      if (cb + cc <= clast) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
          v[4 * q] += __uint_as_float(t[cc][0][q].x); v[4 * q + 1] += __uint_as_float(t[cc][0][q].y);
          v[4 * q + 2] += __uint_as_float(t[cc][0][q].z); v[4 * q + 3] += __uint_as_float(t[cc][0][q].w);
          if (DUAL) {
            v2[4 * q] += __uint_as_float(t[cc][NW - 1][q].x); v2[4 * q + 1] += __uint_as_float(t[cc][NW - 1][q].y);
            v2[4 * q + 2] += __uint_as_float(t[cc][NW - 1][q].z); v2[4 * q + 3] += __uint_as_float(t[cc][NW - 1][q].w);
          }
        }
      }
    }
  }
  tc_finish16<DUAL>(p, tok0 + c0, n, v, v2);
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

// A tensor map is a pure function of its arguments, and a decoder calls the same few dozen (weight, shape) pairs
// over and over: encoded maps are kept in a small per-thread, direct-mapped table keyed by those arguments.
struct MapKey {
  const void* base;
  uint64_t rows, row_bytes;
  uint32_t box_rows;
  int dt, kind;  // kind 0: 128-element rows, 128-byte swizzle; 1: 64-byte rows, 64-byte swizzle; 2: 512-byte rows, no swizzle
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && row_bytes == o.row_bytes && box_rows == o.box_rows && dt == o.dt && kind == o.kind;
  }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kMapSlots = 256;
static MapSlot* map_slot(const MapKey& k) {
  static thread_local MapSlot table[kMapSlots] = {};
  uint64_t h = (uint64_t)(uintptr_t)k.base * 0x9E3779B97F4A7C15ull ^ (k.rows * 0xC2B2AE3D27D4EB4Full) ^ ((uint64_t)k.box_rows << 7) ^ ((uint64_t)k.dt << 3) ^
               (uint64_t)k.kind ^ (k.row_bytes << 17);
  return &table[(h >> 32) % kMapSlots];
}

// 2-D tensor of `rows` rows of 128 elements (row_bytes apart), box = 128 elements x box_rows, 128-byte swizzle.
int tc_make_map(CUtensorMap* m, CUtensorMapDataType dt, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
  const MapKey key = {base, rows, row_bytes, box_rows, (int)dt, 0};
  MapSlot* slot = map_slot(key);
  if (slot->used && slot->key == key) {
    *m = slot->map;
    return TPX_OK;
  }
  EncodeTiledFn fn = encode_fn();
  TPX_REQUIRE(fn, TPX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {128, rows};
  cuuint64_t gstr[1] = {row_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, dt, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TPX_REQUIRE(r == CUDA_SUCCESS, TPX_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (rows=%llu row_bytes=%llu box_rows=%u)", (int)r,
              (unsigned long long)rows, (unsigned long long)row_bytes, box_rows);
  slot->key = key; slot->map = *m; slot->used = true;
  return TPX_OK;
}

// 2-D byte tensor of `rows` rows of 64 bytes, box = 64 bytes x box_rows, 64-byte swizzle (packed 4-bit operands).
int tc_make_map64(CUtensorMap* m, const void* base, uint64_t rows, uint32_t box_rows) {
  const MapKey key = {base, rows, 64, box_rows, (int)CU_TENSOR_MAP_DATA_TYPE_UINT8, 1};
  MapSlot* slot = map_slot(key);
  if (slot->used && slot->key == key) {
    *m = slot->map;
    return TPX_OK;
  }
  EncodeTiledFn fn = encode_fn();
  TPX_REQUIRE(fn, TPX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {64, rows};
  cuuint64_t gstr[1] = {64};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TPX_REQUIRE(r == CUDA_SUCCESS, TPX_ERR_CUDA, "cuTensorMapEncodeTiled (64-byte rows) failed with %d (rows=%llu box_rows=%u)", (int)r,
              (unsigned long long)rows, box_rows);
  slot->key = key; slot->map = *m; slot->used = true;
  return TPX_OK;
}

// 2-D tensor of 512-byte scale blocks (128 32-bit words per row), no swizzle: rows land back to back in shared memory.
int tc_make_map_sf(CUtensorMap* m, const void* base, uint64_t rows, uint32_t box_rows) {
  const MapKey key = {base, rows, 512, box_rows, (int)CU_TENSOR_MAP_DATA_TYPE_UINT32, 2};
  MapSlot* slot = map_slot(key);
  if (slot->used && slot->key == key) {
    *m = slot->map;
    return TPX_OK;
  }
  EncodeTiledFn fn = encode_fn();
  TPX_REQUIRE(fn, TPX_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {128, rows};
  cuuint64_t gstr[1] = {512};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TPX_REQUIRE(r == CUDA_SUCCESS, TPX_ERR_CUDA, "cuTensorMapEncodeTiled (scale blocks) failed with %d (rows=%llu box_rows=%u)", (int)r,
              (unsigned long long)rows, box_rows);
  slot->key = key; slot->map = *m; slot->used = true;
  return TPX_OK;
}

int tc_padded_ks(int64_t K, bool pair) {
  int ks = (int)((K + 127) / 128);
  int m = pair ? 2 : 4;
  return (ks + m - 1) / m * m;
}

int tc_launch_split(const uint16_t* x, int M, int K, int Mpad, int KS, int TOK, int UKS, int rowmap, uint8_t* terms, uint8_t* sfb,
                    cudaStream_t st, const TcNorm* norm) {
  if (norm && norm->gamma) {
    TPX_REQUIRE(KS * 16 <= kNsThreads * kNsVecs, TPX_ERR_UNSUPPORTED, "fused RMSNorm: rows of more than %d elements are not supported (K=%d)",
                kNsThreads * kNsVecs * 8, K);
    TPX_REQUIRE((((uintptr_t)x | (uintptr_t)norm->gamma) & 15) == 0, TPX_ERR_ARG, "fused RMSNorm: x and gamma must be 16-byte aligned");
    TPX_CUDA_OK(launch_pdl(rmsnorm_split_kernel, dim3((unsigned)Mpad), dim3(kNsThreads), 0, st, x, norm->gamma, norm->gamma_f32, norm->eps, M, K,
                           KS, TOK, UKS, rowmap, terms, sfb));
    return TPX_OK;
  }
  long long threads = (long long)Mpad * KS * 4;
  TPX_CUDA_OK(launch_pdl(split_activations_kernel, dim3((unsigned)((threads + 127) / 128)), dim3(128), 0, st, x, M, K, Mpad, KS, TOK, UKS,
                         rowmap, terms, sfb));
  return TPX_OK;
}

struct TcPlan {
  int tok, uks;     // tokens per tile, k steps per unit
  int TN, TM, KS, KU, Mpad, grid, xbox, whole_tiles, cluster;
  size_t off_terms, off_sfb, off_partial, total;
};

static TcPlan tc_plan(int64_t M, int64_t N, int64_t K, bool pair, bool allow_cluster = true) {
  TcPlan pl;
  pl.tok = M <= 16 ? 16 : M <= 32 ? 32 : (M <= 64 || pair) ? 64 : 128;  // a pair needs 4*tok columns of tensor memory
  pl.uks = pair ? 2 : (pl.tok <= 32 ? 4 : 2);
  pl.KS = tc_padded_ks(K, pair);
  pl.KU = pl.KS / pl.uks;
  pl.TN = (int)((N + 127) / 128);
  pl.TM = (int)((M + pl.tok - 1) / pl.tok);
  pl.Mpad = pl.TM * pl.tok;
  int xrows = pl.uks * 2 * pl.tok;
  pl.xbox = xrows > 256 ? 256 : xrows;
  long long U = (long long)pl.TN * pl.TM * pl.KU;
  long long T = (long long)pl.TN * pl.TM;
  int sms = sm_count();
  // Cutting tiles between CTAs balances the weight stream exactly but costs a fix-up pass through scratch at
  // loaded-memory latency; with nearly as many tiles as SMs, or many tiles per SM, whole tiles are cheaper.
  pl.whole_tiles = (T * 10 >= (long long)sms * 7 && T <= sms) || T >= 8LL * sms;
  if (knobs().tc_whole >= 0) pl.whole_tiles = knobs().tc_whole;
  pl.grid = pl.whole_tiles ? (int)(T < sms ? T : sms) : (int)(U < sms ? U : sms);
  // Few tiles: a cluster of c CTAs per tile cuts K between them and reduces through distributed shared memory,
  // which takes the fix-up pass (a second kernel behind a round trip through L2) off the critical path.
  pl.cluster = 1;
  if (allow_cluster && !pl.whole_tiles && T * 2 <= sms) {  // (down projection, M = 128: 39.9 us against 47.5 us with the fix-up pass)
    int c = (int)(sms / T);
    if (c > 8) c = 8;
    if (c > pl.KU) c = pl.KU;
    if (c > 1) pl.cluster = c;
  }
  size_t o = kTcCounterBytes;
  auto bump = [&](size_t bytes) { size_t r = o; o += (bytes + 1023) & ~(size_t)1023; return r; };
  pl.off_terms = bump((size_t)pl.Mpad * pl.KS * 128 * 2);
  pl.off_sfb = bump((size_t)pl.TM * pl.KS * ((2 * pl.tok + 127) / 128) * 512);
  pl.off_partial = bump((size_t)pl.grid * 2 * (pair ? 2 : 1) * pl.tok * 128 * sizeof(float));
  pl.total = o;
  return pl;
}

template <int TOK, bool DUAL, int UKS>
static int tc_launch(const CUtensorMap& w, const CUtensorMap& x, const TcParams& p, int grid, cudaStream_t st) {
  using C = TcCfg<TOK, DUAL, UKS>;
  static bool opted[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || !opted[dev]) {
    TPX_CUDA_OK(cudaFuncSetAttribute(qlinear_tc_kernel<TOK, DUAL, UKS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    if (dev >= 0 && dev < 16) opted[dev] = true;
  }
  // programmatic dependent launch: the prologue and the first weight fetches overlap the split kernel
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
    const int tiles = p.TN * p.TM;
    cudaLaunchConfig_t cc = cfg;
    cc.gridDim = dim3((unsigned)(tiles * p.cluster));
    cudaLaunchAttribute a2[2];
    a2[0] = attr[0];
    a2[1].id = cudaLaunchAttributeClusterDimension;
    a2[1].val.clusterDim.x = (unsigned)p.cluster;
    a2[1].val.clusterDim.y = 1;
    a2[1].val.clusterDim.z = 1;
    cc.attrs = a2;
    cc.numAttrs = 2;
    // the largest cluster size, from the planned one down, of which one cluster per tile can be resident at once
    // (48 clusters of 3 do not fit 148 SMs in GPCs of 16 to 18, 48 of 2 do)
    static int fits[16][9] = {};  // 0 unknown, else 1 + the number of clusters of this size that can be resident
    int c = p.cluster;
    for (; c >= 2; c--) {
      int& f = fits[(dev >= 0 && dev < 16) ? dev : 0][c];
      if (f == 0) {
        a2[1].val.clusterDim.x = (unsigned)c;
        cc.gridDim = dim3((unsigned)(tiles * c));
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, qlinear_tc_kernel<TOK, DUAL, UKS>, &cc);
        if (e != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
        f = 1 + n;
      }
      if (f - 1 >= tiles) break;
    }
    if (c >= 2) {
      TcParams q = p;
      q.cluster = c;
      a2[1].val.clusterDim.x = (unsigned)c;
      cc.gridDim = dim3((unsigned)(tiles * c));
      count_launch();
      TPX_CUDA_OK(cudaLaunchKernelEx(&cc, qlinear_tc_kernel<TOK, DUAL, UKS>, w, x, q));
      return TPX_OK;
    }
    TcParams q = p;
    q.cluster = 1;
    return tc_launch<TOK, DUAL, UKS>(w, x, q, grid, st);
  }
  count_launch();
  TPX_CUDA_OK(cudaLaunchKernelEx(&cfg, qlinear_tc_kernel<TOK, DUAL, UKS>, w, x, p));
  if (!p.whole_tiles && grid > 1) {  // tiles cut between CTAs are completed by the fix-up kernel
    cudaLaunchConfig_t c2 = {};
    c2.gridDim = dim3((unsigned)(p.TN * p.TM), (unsigned)(TOK / 16));
    c2.blockDim = dim3(128);
    c2.stream = st;
    c2.attrs = attr;
    c2.numAttrs = 1;
    count_launch();
  TPX_CUDA_OK(cudaLaunchKernelEx(&c2, tc_fixup_kernel<DUAL>, p, (int)TOK, grid));
  }
  return TPX_OK;
}

int tc_launch_fixup(bool dual, const TcParams& p, int TOK, int grid, cudaStream_t st) {
  cudaLaunchConfig_t c2 = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  c2.gridDim = dim3((unsigned)(p.TN * p.TM), (unsigned)(TOK / 16));
  c2.blockDim = dim3(128);
  c2.stream = st;
  c2.attrs = attr;
  c2.numAttrs = 1;
  count_launch();
  if (dual) TPX_CUDA_OK(cudaLaunchKernelEx(&c2, tc_fixup_kernel<true>, p, TOK, grid));
  else TPX_CUDA_OK(cudaLaunchKernelEx(&c2, tc_fixup_kernel<false>, p, TOK, grid));
  return TPX_OK;
}

}  // namespace tpx

using namespace tpx;

static unsigned long long* g_tc_timeline = nullptr;

#ifdef TPX_DEBUG
// Debug aid (only in a -DTPX_DEBUG build): when set, every CTA of the next tensor-core GEMMs writes 8 globaltimer
// stamps to `buf`.
extern "C" void tpx_debug_tc_timeline(void* buf) { g_tc_timeline = reinterpret_cast<unsigned long long*>(buf); }
#endif

extern "C" int tpx_tc_packed_bytes(int64_t N, int64_t K, int pair, size_t* wq_bytes, size_t* sfa_bytes) {
  TPX_REQUIRE(N > 0 && K > 0 && N % 32 == 0 && K % 64 == 0, TPX_ERR_ARG, "tc_packed_bytes: needs N %% 32 == 0 and K %% 64 == 0");
  size_t tiles = (size_t)((N + 127) / 128) * tc_padded_ks(K, pair != 0) * (pair ? 2 : 1);
  if (wq_bytes) *wq_bytes = tiles * 8192;
  if (sfa_bytes) *sfa_bytes = tiles * 512;
  return TPX_OK;
}

extern "C" int tpx_repack_mxfp4_tc(const uint8_t* codes, const uint8_t* scales, const uint8_t* codes2, const uint8_t* scales2,
                                   int64_t N, int64_t K, uint8_t* wq, uint8_t* sfa, void* stream) {
  TPX_REQUIRE(codes && scales && wq && sfa, TPX_ERR_ARG, "repack_mxfp4_tc: null pointer");
  TPX_REQUIRE((codes2 == nullptr) == (scales2 == nullptr), TPX_ERR_ARG, "repack_mxfp4_tc: the second weight needs codes and scales");
  TPX_REQUIRE(N % 32 == 0 && K % 64 == 0, TPX_ERR_ARG, "repack_mxfp4_tc: needs N %% 32 == 0 and K %% 64 == 0");
  const bool pair = codes2 != nullptr;
  int64_t KS = tc_padded_ks(K, pair);
  int64_t total = ((N + 127) / 128) * KS * (pair ? 2 : 1) * 8192;
  repack_mxfp4_tc_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(codes, scales, codes2, scales2, N, K, KS, wq, sfa);
  TPX_LAUNCH_OK();
  return TPX_OK;
}

// Kernel choice for up to 64 tokens. The kernel with the weights on the wide (N) side of the MMA spends fewer
// tensor-pipe cycles per weight byte (one 128x256x32 MMA per 4 KiB instead of two 128x32x32 per 2 KiB each); the rule
// below follows a sweep of both kernels over the linear shapes of Llama-3-8B, Llama-2-7B and Llama-2-70B (2 and 8
// tensor-parallel ranks) at 1 to 64 tokens, launches back to back. TPX_TC_WIDE=1 forces the wide kernel for every
// M <= 64, TPX_TC_WIDE=0 disables it.
static bool tc_wide(int64_t M, int64_t N, int64_t K, bool pair) {
  if (M > 64) return false;
  if (knobs().tc_wide >= 0) return knobs().tc_wide != 0;
  (void)K;
  const int sms = sm_count();
  auto whole = [&](long long T) { return (T * 10 >= (long long)sms * 7 && T <= sms) || T >= 8LL * sms; };
  const long long T0 = (N + 127) / 128;                        // tiles of the 128-row kernel (a pair: pair tiles)
  const long long T1 = pair ? (N + 127) / 128 : (N + 255) / 256;  // tiles of the wide kernel
  if (whole(T1)) return true;  // every CTA owns whole tiles
  // A pair has the same tiles in both kernels; the wide one measured faster or equal at every token count (Llama-2-7B
  // gate/up, 86 tiles, 64 tokens: 28.5 against 41.2 us; 28 tiles of K = 8192: 24.8 against 28.8 us).
  if (pair) return true;
  if (whole(T0)) return false;
  // The 128-row kernel would cut tiles between CTAs and add a fix-up pass; the wide kernel has half as many tiles and
  // can usually split K inside clusters (q/k/v of 12288 features, 64 tokens: 20.2 against 27.2 us).
  if (T0 * 2 > sms) return true;
  // Both split K inside clusters. Up to 16 tokens the wide kernel: launched back to back the 128-row kernel measured
  // faster at 16 tokens (4096 x 14336: 17.6 against 19.5 us) but a whole Llama-3-8B decode step at batch 16 slower (4.13
  // against 3.96 ms), so the choice follows the model-level measurement. Beyond 16 tokens the 128-row kernel has the
  // shorter epilogue (4096 x 4096 at 64 tokens: 16.4 against 19.2 us).
  return M <= 16;
}

// Kernel family for a call: 0 = weights on the 128-row side (all M), 1 = weights on the N side (M <= 64),
// 2 = packed-fp4 operands (M <= 32). Default where every CTA owns whole tiles (the gate/up pair of a decode step:
// 20.0 against 24.3 us at M = 8, 23.2 against 26.2 us at M = 32, launches back to back; Llama-3-8B decodes at 2.81
// against 2.94 ms/token). Not where tiles are cut between CTAs with a fix-up pass: single launches measured faster up
// to 16 tokens (gate/up pair of 11008 features: 22.2 against 24.3 us at M = 8) but a whole model slower (Llama-2-7B,
// its q/k/v and gate/up linears on this family: 2.76 against 2.66 ms/token). Not where few tiles cut K inside a
// cluster either (down projection: 19.4 against 18.7 us at M = 8). TPX_TC_F4=1 selects it for every M <= 32,
// TPX_TC_F4=0 never.
constexpr int kW4AutoMaxTokens = 0;  // token counts up to which family 3 is chosen without being asked for
static int tc_kind(int64_t M, int64_t N, int64_t K, bool pair) {
  // 3 = weights on the N side with packed-fp4 operands (tpx_qlinear_tcw4.cu): the default up to 32 tokens wherever its
  // work split applies (whole tiles or a cluster per tile), unless a test forces another family; TPX_TC_W4=1 selects it
  // for every shape it serves (up to 64 tokens), TPX_TC_W4=0 never.
  {
    const int w4 = knobs().tc_w4;
    const bool other_forced = knobs().tc_f4 >= 0 || knobs().tc_wide >= 0;
    if (w4 != 0 && (w4 > 0 || (!other_forced && M <= kW4AutoMaxTokens)) && tcw4_serves(M, N, K, pair)) return 3;
  }
  if (M <= 32) {
    const int forced = knobs().tc_f4;
    const long long T = (N + 127) / 128;  // one token tile up to 32 tokens
    const int sms = sm_count();
    const bool whole = (T * 10 >= (long long)sms * 7 && T <= sms) || T >= 8LL * sms;
    if (forced >= 0 ? forced != 0 : whole) return 2;
  }
  if (tcp2_serves(M, N, K, pair)) return 5;  // many tokens on CTA pairs
  if (tcp_serves(M, N, K, pair)) return 4;  // many tokens in whole tiles: the kernel with overlapped epilogue
  return tc_wide(M, N, K, pair) ? 1 : 0;
}

static size_t tc_scratch_need(int64_t M, int64_t N, int64_t K, bool pair, int kind) {
  return kind == 5 ? tcp2_scratch_bytes(M, N, K, pair) : kind == 4 ? tcp_scratch_bytes(M, N, K, pair) : kind == 3 ? tcw4_scratch_bytes(M, N, K, pair) : kind == 2 ? tc4_scratch_bytes(M, N, K, pair) : kind == 1 ? tcw_scratch_bytes(M, N, K, pair)
                   : tc_plan(M, N, K, pair).total;
}

extern "C" size_t tpx_qlinear_mxfp4_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int pair) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return tc_scratch_need(M, N, K, pair != 0, tc_kind(M, N, K, pair != 0));
}

// ---- hand-over between two decode-shaped linears (see TcEmit)
static thread_local TcEmit g_emit_next = {}, g_pre_next = {};
static thread_local bool g_emitted = false;
namespace tpx {
void tc_set_emit(const TcEmit& E) { g_emit_next = E; }
void tc_set_pre(const TcEmit& E) { g_pre_next = E; }
bool tc_emitted() { return g_emitted; }
void tc_note_emitted(bool v) { g_emitted = v; }
}  // namespace tpx

static int tc_run(const uint8_t* wq, const uint8_t* sfa, int pair, const uint16_t* x, int64_t M, int64_t N, int64_t K,
                  const uint16_t* bias, int act, const uint16_t* mul_in, const uint16_t* res, float res_scale, uint16_t* y,
                  void* scratch, size_t scratch_bytes, void* stream, int kind, const TcNorm* norm = nullptr, int wfmt = 0) {
  TPX_REQUIRE(M >= 0 && N > 0 && K > 0, TPX_ERR_ARG, "qlinear_mxfp4_tc: bad shape");
  TPX_REQUIRE(wfmt == 0 || kind == 0 || kind == 1 || kind == 5, TPX_ERR_ARG, "qlinear_tc: 8-bit weights run on the kernels with 8-bit operand containers only");
  if (M == 0) return TPX_OK;
  TPX_REQUIRE(wq && sfa && x && y, TPX_ERR_ARG, "qlinear_mxfp4_tc: null pointer");
  TPX_REQUIRE(!(pair && mul_in), TPX_ERR_ARG, "qlinear_mxfp4_tc: gate/up pair and mul_in are exclusive");
  TPX_REQUIRE(N % 32 == 0 && K % 64 == 0, TPX_ERR_ARG, "qlinear_mxfp4_tc: needs N %% 32 == 0 and K %% 64 == 0");
  TPX_REQUIRE(act >= TPX_ACT_NONE && act <= TPX_ACT_RELU, TPX_ERR_ARG, "qlinear_mxfp4_tc: unknown activation %d", act);
  TPX_REQUIRE(((uintptr_t)wq & 31) == 0 && ((uintptr_t)sfa & 15) == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)scratch & 255) == 0,
              TPX_ERR_ARG, "qlinear_mxfp4_tc: misaligned pointer");
  const bool dual = pair != 0;
  // a hand-over announced for this call (consumed whatever happens)
  const TcEmit emit = g_emit_next, pre = g_pre_next;
  g_emit_next = {};
  g_pre_next = {};
  g_emitted = false;
  TcNorm with_pre = {};
  if (pre.terms) {
    TPX_REQUIRE((kind == 0 || kind == 1) && !(norm && norm->gamma) && !dual, TPX_ERR_ARG, "qlinear_mxfp4_tc: this launch cannot take handed-over terms");
    with_pre.pre = &pre;
    norm = &with_pre;
  }
  if (kind == 5) {
    TcParams b = {};
    b.bias = bias; b.mul_in = mul_in; b.res = res; b.res_scale = res_scale; b.y = y; b.act = act; b.tl = g_tc_timeline;
    b.dbg = knobs().dbg;
    b.wfmt = wfmt;
    return tcp2_run(wq, sfa, dual, x, M, N, K, b, scratch, scratch_bytes, (cudaStream_t)stream, norm);
  }
  if (kind == 4) {
    TcParams b = {};
    b.bias = bias; b.mul_in = mul_in; b.res = res; b.res_scale = res_scale; b.y = y; b.act = act; b.tl = g_tc_timeline;
    b.dbg = knobs().dbg;
    return tcp_run(wq, sfa, dual, x, M, N, K, b, scratch, scratch_bytes, (cudaStream_t)stream, norm);
  }
  if (kind == 3) {
    TcParams b = {};
    b.bias = bias; b.mul_in = mul_in; b.res = res; b.res_scale = res_scale; b.y = y; b.act = act; b.tl = g_tc_timeline;
    return tcw4_run(wq, sfa, dual, x, M, N, K, b, scratch, scratch_bytes, (cudaStream_t)stream, norm);
  }
  if (kind == 2) {
    TcParams b = {};
    b.bias = bias; b.mul_in = mul_in; b.res = res; b.res_scale = res_scale; b.y = y; b.act = act; b.tl = g_tc_timeline;
    b.dbg = knobs().dbg;
    // no L2 prefetch ahead of the stages: this kernel's stages already hold 160-210 KB of packed weights per SM, and
    // prefetches issued at the start delay the first stage (gate/up, M = 8: 26.5 us without, 29.2 us with 8 units ahead)
    b.pf = knobs().tc_pf;
    b.emit = emit;
    return tc4_run(wq, sfa, dual, x, M, N, K, b, scratch, scratch_bytes, (cudaStream_t)stream, norm);
  }
  if (kind == 1) {
    TcParams b = {};
    b.bias = bias; b.mul_in = mul_in; b.res = res; b.res_scale = res_scale; b.y = y; b.act = act; b.tl = g_tc_timeline;
    b.dbg = knobs().dbg;
    // L2 prefetch ahead of the stages is off: with launches back to back it delays the first stage more than it helps
    // later ones (gate/up, M = 8: 23.4 us without, 25.3 us with 8 units ahead)
    b.pf = wfmt ? 0 : knobs().tc_pf;
    b.emit = emit;
    b.wfmt = wfmt;
    return tcw_run(wq, sfa, dual, x, M, N, K, b, scratch, scratch_bytes, (cudaStream_t)stream, norm);
  }
  TcPlan pl = tc_plan(M, N, K, dual);
  TPX_REQUIRE(scratch && scratch_bytes >= pl.total, TPX_ERR_SCRATCH, "qlinear_mxfp4_tc: scratch of %zu bytes needed, %zu given",
              pl.total, scratch_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  unsigned char* sc = reinterpret_cast<unsigned char*>(scratch);
  uint8_t *terms = sc + pl.off_terms, *sfb = sc + pl.off_sfb;
  if (norm && norm->pre) {  // the previous linear's epilogue wrote the terms
    const TcEmit& e = *norm->pre;
    TPX_REQUIRE(e.TOK == pl.tok && e.UKS == pl.uks && e.KS == pl.KS && e.rowmap == 0, TPX_ERR_ARG,
                "qlinear_mxfp4_tc: handed-over activation terms do not fit this launch");
    terms = e.terms;
    sfb = e.sfb;
  } else {
    int rc0 = tc_launch_split(x, (int)M, (int)K, pl.Mpad, pl.KS, pl.tok, pl.uks, 0, terms, sfb, st, norm);
    if (rc0) return rc0;
  }
  CUtensorMap mw, mx;
  // weight: 64-byte rows of 128 codes, 256 rows (two tiles) per request; activation terms: 128-byte rows
  int rc;
  rc = tc_make_map(&mw, wfmt ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, wq, (uint64_t)pl.TN * pl.KS * (dual ? 2 : 1) * 128,
                   wfmt ? 128 : 64, (dual ? 2 : 1) * pl.uks >= 2 ? 256 : 128);
  if (rc) return rc;
  rc = tc_make_map(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, terms, (uint64_t)pl.Mpad * pl.KS * 2, 128, (uint32_t)pl.xbox);
  if (rc) return rc;
  TcParams p;
  p.sfa = sfa; p.sfa2 = nullptr; p.sfb = sfb; p.bias = bias; p.mul_in = mul_in; p.res = res; p.res_scale = res_scale; p.y = y;
  p.partial = reinterpret_cast<float*>(sc + pl.off_partial);
  p.counters = reinterpret_cast<unsigned*>(sc);
  p.err = reinterpret_cast<unsigned*>(sc + kTcCounterBytes - 4);
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.KS = pl.KU; p.TN = pl.TN; p.TM = pl.TM; p.act = act; p.whole_tiles = pl.whole_tiles; p.cluster = pl.cluster; p.tl = g_tc_timeline;
  p.dbg = knobs().dbg;
  p.wfmt = wfmt;
  p.emit = {};
  p.pf = knobs().tc_pf;  // off by default, see above (prefill shapes: 842 against 838 TFLOP/s)
  if (knobs().tc_cluster == 0) p.cluster = 1;
  if (dual) {
    switch (pl.tok) {
      case 16: return tc_launch<16, true, 2>(mw, mx, p, pl.grid, st);
      case 32: return tc_launch<32, true, 2>(mw, mx, p, pl.grid, st);
      default: return tc_launch<64, true, 2>(mw, mx, p, pl.grid, st);
    }
  }
  switch (pl.tok) {
    case 16: return tc_launch<16, false, 4>(mw, mx, p, pl.grid, st);
    case 32: return tc_launch<32, false, 4>(mw, mx, p, pl.grid, st);
    case 64: return tc_launch<64, false, 2>(mw, mx, p, pl.grid, st);
    default: return tc_launch<128, false, 2>(mw, mx, p, pl.grid, st);
  }
}

namespace tpx {
int tc_handoff_plan(int64_t M, int64_t N, int64_t K, void* buf, size_t bytes, TcEmit* E) {
  *E = {};
  if (!buf || M < 1 || M > 64 || K % 128) return TPX_OK;
  const int kind = tc_kind(M, N, K, false);
  TcEmit e = {};
  size_t tb = 0, sb = 0;
  if (kind == 1) {
    if (!tcw_handoff_layout(M, N, K, &e, &tb, &sb)) return TPX_OK;
  } else if (kind == 0) {
    const TcPlan pl = tc_plan(M, N, K, false);
    if ((int64_t)pl.KS * 128 != K) return TPX_OK;
    e.TOK = pl.tok; e.UKS = pl.uks; e.KS = pl.KS; e.rowmap = 0;
    tb = (size_t)pl.Mpad * pl.KS * 256;
    sb = (size_t)pl.TM * pl.KS * ((2 * pl.tok + 127) / 128) * 512;
  } else {
    return TPX_OK;
  }
  tb = (tb + 1023) & ~(size_t)1023;
  if (tb + sb > bytes || ((uintptr_t)buf & 1023)) return TPX_OK;
  e.terms = reinterpret_cast<uint8_t*>(buf);
  e.sfb = e.terms + tb;
  *E = e;
  return TPX_OK;
}
}  // namespace tpx

extern "C" int tpx_qlinear_mxfp4_tc(const uint8_t* wq, const uint8_t* sfa, int pair, const uint16_t* x, int64_t M, int64_t N,
                                    int64_t K, const uint16_t* bias, int act, const uint16_t* mul_in, const uint16_t* res,
                                    float res_scale, uint16_t* y, void* scratch, size_t scratch_bytes, void* stream) {
  return tc_run(wq, sfa, pair, x, M, N, K, bias, act, mul_in, res, res_scale, y, scratch, scratch_bytes, stream, tc_kind(M, N, K, pair != 0));
}

// ---------------------------------------------------------------- 8-bit floating-point weights (E4M3 / E5M2, no scales)
extern "C" int tpx_fp8_tc_packed_bytes(int64_t N, int64_t K, int pair, size_t* wq_bytes, size_t* sfa_bytes) {
  TPX_REQUIRE(N > 0 && K > 0 && N % 32 == 0 && K % 64 == 0, TPX_ERR_ARG, "fp8_tc_packed_bytes: needs N %% 32 == 0 and K %% 64 == 0");
  size_t tiles = (size_t)((N + 127) / 128) * tc_padded_ks(K, pair != 0) * (pair ? 2 : 1);
  if (wq_bytes) *wq_bytes = tiles * 16384;
  if (sfa_bytes) *sfa_bytes = tiles * 512;
  return TPX_OK;
}

extern "C" int tpx_repack_fp8_tc(const uint8_t* w, const uint8_t* w2, int64_t N, int64_t K, uint8_t* wq, uint8_t* sfa, void* stream) {
  TPX_REQUIRE(w && wq && sfa, TPX_ERR_ARG, "repack_fp8_tc: null pointer");
  TPX_REQUIRE(N % 32 == 0 && K % 64 == 0, TPX_ERR_ARG, "repack_fp8_tc: needs N %% 32 == 0 and K %% 64 == 0");
  TPX_REQUIRE((((uintptr_t)w | (uintptr_t)w2 | (uintptr_t)wq | (uintptr_t)sfa) & 15) == 0, TPX_ERR_ARG, "repack_fp8_tc: misaligned pointer");
  const bool pair = w2 != nullptr;
  int64_t KS = tc_padded_ks(K, pair);
  int64_t total = ((N + 127) / 128) * KS * (pair ? 2 : 1) * 1024;
  repack_fp8_tc_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(w, w2, N, K, KS, wq, sfa);
  TPX_LAUNCH_OK();
  return TPX_OK;
}

// Kernel for 8-bit weights: the choice made for MXFP4 at this shape, among the kernels whose weight operand sits in
// 8-bit containers (the packed-fp4 kernels become the wide kernel, the one-CTA many-token kernel the 128-row one).
static int fp8_kind(int64_t M, int64_t N, int64_t K, bool pair) {
  const int k = tc_kind(M, N, K, pair);
  if (k == 2 || k == 3) return 1;
  if (k == 4) return 0;
  return k;
}

extern "C" size_t tpx_qlinear_fp8_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int pair) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return tc_scratch_need(M, N, K, pair != 0, fp8_kind(M, N, K, pair != 0));
}

extern "C" int tpx_qlinear_fp8_tc(const uint8_t* wq, const uint8_t* sfa, int fmt, int pair, const uint16_t* x, const void* gamma,
                                  int gamma_is_f32, float eps, int64_t M, int64_t N, int64_t K, const uint16_t* bias, int act,
                                  const uint16_t* mul_in, const uint16_t* res, float res_scale, uint16_t* y, void* scratch,
                                  size_t scratch_bytes, void* stream) {
  TPX_REQUIRE(fmt == TPX_FP8_E4M3 || fmt == TPX_FP8_E5M2, TPX_ERR_ARG, "qlinear_fp8_tc: unknown weight format %d", fmt);
  TcNorm nm = {gamma, gamma_is_f32, eps};
  return tc_run(wq, sfa, pair, x, M, N, K, bias, act, mul_in, res, res_scale, y, scratch, scratch_bytes, stream, fp8_kind(M, N, K, pair != 0),
                gamma ? &nm : nullptr, fmt);
}

extern "C" int tpx_rmsnorm_qlinear_mxfp4_tc(const uint8_t* wq, const uint8_t* sfa, int pair, const uint16_t* x, const void* gamma,
                                            int gamma_is_f32, float eps, int64_t M, int64_t N, int64_t K, const uint16_t* bias, int act,
                                            const uint16_t* mul_in, const uint16_t* res, float res_scale, uint16_t* y, void* scratch,
                                            size_t scratch_bytes, void* stream) {
  TPX_REQUIRE(gamma, TPX_ERR_ARG, "rmsnorm_qlinear_mxfp4_tc: null gamma");
  TcNorm nm = {gamma, gamma_is_f32, eps};
  return tc_run(wq, sfa, pair, x, M, N, K, bias, act, mul_in, res, res_scale, y, scratch, scratch_bytes, stream, tc_kind(M, N, K, pair != 0), &nm);
}

// ---------------------------------------------------------------- variant that allocates nothing
// Some callers may not allocate device memory at the point where they run a linear: a serving loop that has
// handed all free memory to its KV-cache pool, a plugin running inside another framework's memory budget, or a
// host thread that must not take the allocator's locks. For them the scratch of the tensor-core linear lives in
// this file-scope device array instead of a caller-provided buffer. Every GPU that loads the library holds these
// 8 MiB until the process exits.
static constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_tc_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle: the device address comes from cudaGetSymbolAddress, once per
// device, with that device current.
static int static_scratch_ptr(void** out) {
  static void* ptrs[64] = {};
  int dev = 0;
  TPX_CUDA_OK(cudaGetDevice(&dev));
  TPX_REQUIRE(dev >= 0 && dev < 64, TPX_ERR_UNSUPPORTED, "qlinear_mxfp4_tc_static: device index %d out of range", dev);
  if (!ptrs[dev]) {
    void* p = nullptr;
    TPX_CUDA_OK(cudaGetSymbolAddress(&p, g_tc_static_scratch));
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return TPX_OK;
}

extern "C" size_t tpx_qlinear_mxfp4_tc_static_max_bytes(void) { return kStaticScratchBytes; }

// The bounded waits inside the kernels report through a word of the scratch; with the built-in array the caller has no
// pointer to it, so this call copies it out (and clears it). It waits for `stream`: use it at a point where a
// synchronisation is acceptable (after a step, not between the launches of one).
extern "C" int tpx_qlinear_mxfp4_tc_static_status(void* stream, unsigned* status_host) {
  TPX_REQUIRE(status_host, TPX_ERR_ARG, "qlinear_mxfp4_tc_static_status: null pointer");
  void* sc = nullptr;
  int rc = static_scratch_ptr(&sc);
  if (rc) return rc;
  unsigned char* word = reinterpret_cast<unsigned char*>(sc) + kTcCounterBytes - 4;
  TPX_CUDA_OK(cudaMemcpyAsync(status_host, word, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  TPX_CUDA_OK(cudaMemsetAsync(word, 0, 4, (cudaStream_t)stream));
  TPX_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
  return TPX_OK;
}

extern "C" int tpx_qlinear_mxfp4_tc_static(const uint8_t* wq, const uint8_t* sfa, int pair, const uint16_t* x, int64_t M,
                                           int64_t N, int64_t K, const uint16_t* bias, int act, const uint16_t* mul_in,
                                           const uint16_t* res, float res_scale, uint16_t* y, void* stream) {
  TPX_REQUIRE(M >= 0 && N > 0 && K > 0, TPX_ERR_ARG, "qlinear_mxfp4_tc_static: bad shape");
  if (M == 0) return TPX_OK;
  // the planner's kernel family if its scratch fits the array, else the family with the smallest scratch (the
  // 128-row-side kernel); only when that does not fit either is the shape refused
  int wide = tc_kind(M, N, K, pair != 0);
  if (wide && tc_scratch_need(M, N, K, pair != 0, wide) > kStaticScratchBytes) wide = 0;
  const size_t need = tc_scratch_need(M, N, K, pair != 0, wide);
  TPX_REQUIRE(need <= kStaticScratchBytes, TPX_ERR_SCRATCH,
              "qlinear_mxfp4_tc_static: M=%ld N=%ld K=%ld needs %zu bytes of scratch, the built-in array holds %zu; "
              "use tpx_qlinear_mxfp4_tc with a caller-provided buffer",
              (long)M, (long)N, (long)K, need, kStaticScratchBytes);
  void* sc = nullptr;
  int rc = static_scratch_ptr(&sc);
  if (rc) return rc;
  // the array keeps whatever the previous call left: the arrival counters must start at zero. The error word at the
  // end of the counter block is left alone: it stays set until tpx_qlinear_mxfp4_tc_static_status reads it.
  TPX_CUDA_OK(cudaMemsetAsync(sc, 0, kTcCounterBytes - 4, (cudaStream_t)stream));
  return tc_run(wq, sfa, pair, x, M, N, K, bias, act, mul_in, res, res_scale, y, sc, kStaticScratchBytes, stream, wide);
}
