// Weight-streaming quantized linear for small token counts (decode): y = epilogue(x . dequant(W)^T).
//
// Replaces TppBlockedLinearW / TppBlockedQInt8LinearW of the reference
// (src/csrc/fused_gemm.h:784-1073, :1075-1341) for the bandwidth-bound regime. The weight matrix is
// read exactly once per 32 tokens, as 128-bit loads of fully contiguous 512-byte warp rows, and is
// the M dimension of mma.sync.m16n8k16 (rows of W = "m", tokens = "n"): each warp owns 16 output
// features and streams along K. 4-bit codes are expanded to f16 with cvt.e2m1x2 (exact), the block
// scale (a power of two) multiplies the fp32 block sum after the MMAs, so every product is exact.
// Activations are staged once per CTA in shared memory as f16 after an exact power-of-two
// pre-scale that keeps them in f16 range.
//
// Work split: grid.x CTAs stride over groups of 8 row tiles (one per warp), grid.y splits K.
// With a K split the partial sums go to fp32 scratch and the last-arriving warp of each row tile
// (a counter per tile) adds them in a fixed order and runs the epilogue.
#include "tpx_common.cuh"

namespace tpx {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kPrefetch = 4;  // weight tiles in flight per warp

struct StreamParams {
  const uint4* w;       // packed codes, tile-major
  const void* s;        // packed scales
  const uint4* w2;      // second weight (gate/up pair) or null
  const void* s2;
  const uint16_t* x;    // [M][K] bf16
  const uint16_t* bias; // [N] or null
  const uint16_t* mul_in;
  const uint16_t* res;
  float res_scale;
  uint16_t* y;          // [M][N]
  float* partial;       // [ksplit][2][Mpad][N] fp32 (ksplit > 1)
  unsigned* counters;   // [N/16]
  int M, N, K;          // K = logical K
  int KT;               // k tiles in the packed tensor
  int ksplit;           // grid.y
  int kt_per_split;     // tiles per split (last split may be shorter)
  int m0, mcount;       // token window of this launch
  int act;
  int sblocks_per_tile; // int8: tiles (64 k) per scale block
};

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// two E2M1 codes (one byte) -> f16x2, low nibble in the low half
__device__ __forceinline__ uint32_t cvt_e2m1x2(uint32_t byte) {
  uint32_t r;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(r) : "r"(byte));
  return r;
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Stage the activation window [mcount tokens] x [k range] into shared memory as f16, scaled by
// 2^-p so that the largest magnitude lies in [2^14, 2^15). Returns 2^p through *unscale.
// Layout: row = token (padded to NT*8 rows of zeros), row stride = kslice*2 + 32 bytes, which
// makes the 8-byte fragment reads of a half-warp hit 32 distinct banks.
template <int NT>
__device__ __forceinline__ void stage_x(const StreamParams& p, int k_begin, int kslice, unsigned char* smem,
                                        float* red, float* unscale) {
  const int rows = NT * 8;
  const int stride = kslice * 2 + 32;
  float mx = 0.0f;
  const int vec_per_row = kslice / 8;
  for (int i = threadIdx.x; i < rows * vec_per_row; i += kThreads) {
    int r = i / vec_per_row, c = i % vec_per_row;
    int k = k_begin + c * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < p.mcount && k < p.K) v = *reinterpret_cast<const uint4*>(p.x + (size_t)(p.m0 + r) * p.K + k);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      mx = fmaxf(mx, fabsf(bf16_bits_to_f32((uint16_t)(w[j] & 0xffff))));
      mx = fmaxf(mx, fabsf(bf16_bits_to_f32((uint16_t)(w[j] >> 16))));
    }
    *reinterpret_cast<uint4*>(smem + r * stride + c * 16) = v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int w = 1; w < kWarps; w++) mx = fmaxf(mx, red[w]);
  int e = (int)((__float_as_uint(mx) >> 23) & 0xff) - 127;
  int pw = (mx == 0.0f || e > 127) ? 0 : e - 14;
  pw = max(pw, -100);
  float down = __uint_as_float((uint32_t)(127 - pw) << 23);  // 2^-p
  *unscale = __uint_as_float((uint32_t)(127 + pw) << 23);    // 2^p
  for (int i = threadIdx.x; i < rows * vec_per_row; i += kThreads) {
    int r = i / vec_per_row, c = i % vec_per_row;
    uint4* ptr = reinterpret_cast<uint4*>(smem + r * stride + c * 16);
    uint4 v = *ptr;
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float lo = bf16_bits_to_f32((uint16_t)(w[j] & 0xffff)) * down;
      float hi = bf16_bits_to_f32((uint16_t)(w[j] >> 16)) * down;
      __half2 h = __floats2half2_rn(lo, hi);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    *ptr = make_uint4(w[0], w[1], w[2], w[3]);
  }
  __syncthreads();
}

// Epilogue for one output element (src/csrc/fused_gemm.h:1343-1458): bias, activation, gate multiply, residual.
__device__ __forceinline__ void finish(const StreamParams& p, int tok, int row, float v, float v2, bool dual) {
  if (tok >= p.mcount || row >= p.N) return;
  size_t o = (size_t)(p.m0 + tok) * p.N + row;
  if (p.bias) v += bf16_bits_to_f32(p.bias[row]);
  v = apply_act(v, p.act);
  if (dual) v *= v2;
  if (p.mul_in) v *= bf16_bits_to_f32(p.mul_in[o]);
  if (p.res) v += bf16_bits_to_f32(p.res[o]) * p.res_scale;
  p.y[o] = f32_to_bf16_bits(v);
}

// acc element i of n-tile j of a thread (g, t): row = g + 8*(i>>1), token = 8j + 2t + (i&1)
template <int NT, bool DUAL>
__device__ __forceinline__ void reduce_and_finish(const StreamParams& p, int nt, int lane, float (&tot)[DUAL ? 2 : 1][NT][4]) {
  const int g = lane >> 2, t = lane & 3;
  const int Mpad = NT * 8;
  if (p.ksplit == 1) {
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int i = 0; i < 4; i++)
        finish(p, 8 * j + 2 * t + (i & 1), nt * 16 + g + 8 * (i >> 1), tot[0][j][i], DUAL ? tot[DUAL ? 1 : 0][j][i] : 0.0f, DUAL);
    return;
  }
  const int ks = blockIdx.y;
  const size_t plane = (size_t)Mpad * p.N;
#pragma unroll
  for (int d = 0; d < (DUAL ? 2 : 1); d++)
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int tok = 8 * j + 2 * t + (i & 1), row = nt * 16 + g + 8 * (i >> 1);
        __stcg(p.partial + ((size_t)(ks * 2 + d)) * plane + (size_t)tok * p.N + row, tot[d][j][i]);
      }
  __threadfence();
  __syncwarp();
  unsigned prev = 0;
  if (lane == 0) prev = atomicAdd(p.counters + nt, 1u);
  prev = __shfl_sync(0xffffffffu, prev, 0);
  if (prev != (unsigned)(p.ksplit - 1)) return;
  __threadfence();
#pragma unroll
  for (int j = 0; j < NT; j++)
#pragma unroll
    for (int i = 0; i < 4; i++) {
      int tok = 8 * j + 2 * t + (i & 1), row = nt * 16 + g + 8 * (i >> 1);
      float v = 0.0f, v2 = 0.0f;
      for (int s = 0; s < p.ksplit; s++) {  // fixed order: the result does not depend on arrival order
        v += __ldcg(p.partial + ((size_t)(s * 2)) * plane + (size_t)tok * p.N + row);
        if (DUAL) v2 += __ldcg(p.partial + ((size_t)(s * 2 + 1)) * plane + (size_t)tok * p.N + row);
      }
      finish(p, tok, row, v, v2, DUAL);
    }
  if (lane == 0) p.counters[nt] = 0;  // leave the counter ready for the next launch
}

// ---------------------------------------------------------------- MXFP4
template <int NT, bool DUAL>
__global__ void __launch_bounds__(kThreads) qlinear_stream_mxfp4(StreamParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float red[kWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kt0 = blockIdx.y * p.kt_per_split;
  const int kt1 = min(p.KT, kt0 + p.kt_per_split);
  const int kslice = p.kt_per_split * 128;
  const int stride = kslice * 2 + 32;
  float unscale;
  stage_x<NT>(p, kt0 * 128, kslice, smem, red, &unscale);

  const int ntiles = p.N / 16;
  for (int nt = blockIdx.x * kWarps + warp; nt < ntiles; nt += gridDim.x * kWarps) {
    float tot[DUAL ? 2 : 1][NT][4];
#pragma unroll
    for (int d = 0; d < (DUAL ? 2 : 1); d++)
#pragma unroll
      for (int j = 0; j < NT; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) tot[d][j][i] = 0.0f;

    const uint4* wbase[2] = {p.w + (size_t)nt * p.KT * 64 + lane, DUAL ? p.w2 + (size_t)nt * p.KT * 64 + lane : nullptr};
    const uint32_t* sbase[2] = {reinterpret_cast<const uint32_t*>(p.s) + (size_t)nt * p.KT * 16,
                                DUAL ? reinterpret_cast<const uint32_t*>(p.s2) + (size_t)nt * p.KT * 16 : nullptr};
    // register ring of weight tiles: [slot][weight][half]
    uint4 buf[kPrefetch][DUAL ? 2 : 1][2];
    uint32_t sc[kPrefetch][DUAL ? 2 : 1][2];
#pragma unroll
    for (int s = 0; s < kPrefetch; s++) {
      int kt = kt0 + s;
      if (kt < kt1) {
#pragma unroll
        for (int d = 0; d < (DUAL ? 2 : 1); d++) {
          buf[s][d][0] = ldg_stream(wbase[d] + (size_t)kt * 64);
          buf[s][d][1] = ldg_stream(wbase[d] + (size_t)kt * 64 + 32);
          sc[s][d][0] = __ldg(sbase[d] + (size_t)kt * 16 + g);
          sc[s][d][1] = __ldg(sbase[d] + (size_t)kt * 16 + g + 8);
        }
      }
    }
    for (int ktb = kt0; ktb < kt1; ktb += kPrefetch) {
#pragma unroll
      for (int s = 0; s < kPrefetch; s++) {
        const int kt = ktb + s;
        if (kt < kt1) {
          uint4 cur[DUAL ? 2 : 1][2];
          uint32_t csc[DUAL ? 2 : 1][2];
#pragma unroll
          for (int d = 0; d < (DUAL ? 2 : 1); d++) {
            cur[d][0] = buf[s][d][0];
            cur[d][1] = buf[s][d][1];
            csc[d][0] = sc[s][d][0];
            csc[d][1] = sc[s][d][1];
          }
          const int ktn = kt + kPrefetch;
          if (ktn < kt1) {
#pragma unroll
            for (int d = 0; d < (DUAL ? 2 : 1); d++) {
              buf[s][d][0] = ldg_stream(wbase[d] + (size_t)ktn * 64);
              buf[s][d][1] = ldg_stream(wbase[d] + (size_t)ktn * 64 + 32);
              sc[s][d][0] = __ldg(sbase[d] + (size_t)ktn * 16 + g);
              sc[s][d][1] = __ldg(sbase[d] + (size_t)ktn * 16 + g + 8);
            }
          }
          const unsigned char* xrow = smem + g * stride + ((kt - kt0) * 128 + 4 * t) * 2;
#pragma unroll
          for (int b = 0; b < 4; b++) {
            // B fragments of this 32-wide block for every token tile: [hh][j]
            uint2 xb[2][NT];
#pragma unroll
            for (int hh = 0; hh < 2; hh++)
#pragma unroll
              for (int j = 0; j < NT; j++)
                xb[hh][j] = *reinterpret_cast<const uint2*>(xrow + j * 8 * stride + (32 * b + 16 * hh) * 2);
#pragma unroll
            for (int d = 0; d < (DUAL ? 2 : 1); d++) {
              const uint32_t wa = b == 0 ? cur[d][0].x : b == 1 ? cur[d][0].y : b == 2 ? cur[d][0].z : cur[d][0].w;
              const uint32_t wc = b == 0 ? cur[d][1].x : b == 1 ? cur[d][1].y : b == 2 ? cur[d][1].z : cur[d][1].w;
              float blk[NT][4];
#pragma unroll
              for (int j = 0; j < NT; j++)
#pragma unroll
                for (int i = 0; i < 4; i++) blk[j][i] = 0.0f;
#pragma unroll
              for (int hh = 0; hh < 2; hh++) {
                uint32_t a0 = cvt_e2m1x2((wa >> (16 * hh)) & 0xff);
                uint32_t a2 = cvt_e2m1x2((wa >> (16 * hh + 8)) & 0xff);
                uint32_t a1 = cvt_e2m1x2((wc >> (16 * hh)) & 0xff);
                uint32_t a3 = cvt_e2m1x2((wc >> (16 * hh + 8)) & 0xff);
#pragma unroll
                for (int j = 0; j < NT; j++) mma_f16(blk[j], a0, a1, a2, a3, xb[hh][j].x, xb[hh][j].y);
              }
              const float s0 = __uint_as_float(((csc[d][0] >> (8 * b)) & 0xffu) << 23);
              const float s1 = __uint_as_float(((csc[d][1] >> (8 * b)) & 0xffu) << 23);
#pragma unroll
              for (int j = 0; j < NT; j++) {
                tot[d][j][0] = fmaf(s0, blk[j][0], tot[d][j][0]);
                tot[d][j][1] = fmaf(s0, blk[j][1], tot[d][j][1]);
                tot[d][j][2] = fmaf(s1, blk[j][2], tot[d][j][2]);
                tot[d][j][3] = fmaf(s1, blk[j][3], tot[d][j][3]);
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int d = 0; d < (DUAL ? 2 : 1); d++)
#pragma unroll
      for (int j = 0; j < NT; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) tot[d][j][i] *= unscale;
    reduce_and_finish<NT, DUAL>(p, nt, lane, tot);
  }
}

// ---------------------------------------------------------------- int8
// Tile = 16 rows x 64 k. Bytes become f16 through the 1024+u magic number (exact for -128..127).
__device__ __forceinline__ void s8x4_to_f16x2x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;  // biased to 0..255
  uint32_t l, h;
  asm("prmt.b32 %0, %1, %2, 0x5140;" : "=r"(l) : "r"(u), "r"(0x64646464u));
  asm("prmt.b32 %0, %1, %2, 0x7362;" : "=r"(h) : "r"(u), "r"(0x64646464u));
  const uint32_t magic = 0x64806480u;  // 1024 + 128
  asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(l), "r"(magic));
  asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(h), "r"(magic));
}

template <int NT, bool DUAL>
__global__ void __launch_bounds__(kThreads) qlinear_stream_int8(StreamParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float red[kWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kt0 = blockIdx.y * p.kt_per_split;
  const int kt1 = min(p.KT, kt0 + p.kt_per_split);
  const int kslice = p.kt_per_split * 64;
  const int stride = kslice * 2 + 32;
  float unscale;
  stage_x<NT>(p, kt0 * 64, kslice, smem, red, &unscale);
  const int nsb = p.KT / p.sblocks_per_tile;  // scale blocks along K

  const int ntiles = p.N / 16;
  for (int nt = blockIdx.x * kWarps + warp; nt < ntiles; nt += gridDim.x * kWarps) {
    float tot[DUAL ? 2 : 1][NT][4];
    float blk[DUAL ? 2 : 1][NT][4];
#pragma unroll
    for (int d = 0; d < (DUAL ? 2 : 1); d++)
#pragma unroll
      for (int j = 0; j < NT; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) tot[d][j][i] = blk[d][j][i] = 0.0f;
    const uint4* wbase[2] = {p.w + (size_t)nt * p.KT * 64 + lane, DUAL ? p.w2 + (size_t)nt * p.KT * 64 + lane : nullptr};
    const float* sbase[2] = {reinterpret_cast<const float*>(p.s) + (size_t)nt * nsb * 16,
                             DUAL ? reinterpret_cast<const float*>(p.s2) + (size_t)nt * nsb * 16 : nullptr};
    uint4 buf[kPrefetch][DUAL ? 2 : 1][2];
#pragma unroll
    for (int s = 0; s < kPrefetch; s++) {
      int kt = kt0 + s;
      if (kt < kt1) {
#pragma unroll
        for (int d = 0; d < (DUAL ? 2 : 1); d++) {
          buf[s][d][0] = ldg_stream(wbase[d] + (size_t)kt * 64);
          buf[s][d][1] = ldg_stream(wbase[d] + (size_t)kt * 64 + 32);
        }
      }
    }
    for (int ktb = kt0; ktb < kt1; ktb += kPrefetch) {
#pragma unroll
      for (int s = 0; s < kPrefetch; s++) {
        const int kt = ktb + s;
        if (kt < kt1) {
          uint4 cur[DUAL ? 2 : 1][2];
#pragma unroll
          for (int d = 0; d < (DUAL ? 2 : 1); d++) {
            cur[d][0] = buf[s][d][0];
            cur[d][1] = buf[s][d][1];
          }
          const int ktn = kt + kPrefetch;
          if (ktn < kt1) {
#pragma unroll
            for (int d = 0; d < (DUAL ? 2 : 1); d++) {
              buf[s][d][0] = ldg_stream(wbase[d] + (size_t)ktn * 64);
              buf[s][d][1] = ldg_stream(wbase[d] + (size_t)ktn * 64 + 32);
            }
          }
          const unsigned char* xrow = smem + g * stride + ((kt - kt0) * 64 + 4 * t) * 2;
#pragma unroll
          for (int b = 0; b < 4; b++) {
            uint2 xb[NT];
#pragma unroll
            for (int j = 0; j < NT; j++) xb[j] = *reinterpret_cast<const uint2*>(xrow + j * 8 * stride + 16 * b * 2);
#pragma unroll
            for (int d = 0; d < (DUAL ? 2 : 1); d++) {
              const uint32_t wa = b == 0 ? cur[d][0].x : b == 1 ? cur[d][0].y : b == 2 ? cur[d][0].z : cur[d][0].w;
              const uint32_t wc = b == 0 ? cur[d][1].x : b == 1 ? cur[d][1].y : b == 2 ? cur[d][1].z : cur[d][1].w;
              uint32_t a0, a1, a2, a3;
              s8x4_to_f16x2x2(wa, a0, a2);
              s8x4_to_f16x2x2(wc, a1, a3);
#pragma unroll
              for (int j = 0; j < NT; j++) mma_f16(blk[d][j], a0, a1, a2, a3, xb[j].x, xb[j].y);
            }
          }
          if ((kt + 1) % p.sblocks_per_tile == 0) {  // end of a scale block: fold it in
            const int sb = kt / p.sblocks_per_tile;
#pragma unroll
            for (int d = 0; d < (DUAL ? 2 : 1); d++) {
              const float s0 = __ldg(sbase[d] + (size_t)sb * 16 + g);
              const float s1 = __ldg(sbase[d] + (size_t)sb * 16 + g + 8);
#pragma unroll
              for (int j = 0; j < NT; j++) {
                tot[d][j][0] = fmaf(s0, blk[d][j][0], tot[d][j][0]);
                tot[d][j][1] = fmaf(s0, blk[d][j][1], tot[d][j][1]);
                tot[d][j][2] = fmaf(s1, blk[d][j][2], tot[d][j][2]);
                tot[d][j][3] = fmaf(s1, blk[d][j][3], tot[d][j][3]);
                blk[d][j][0] = blk[d][j][1] = blk[d][j][2] = blk[d][j][3] = 0.0f;
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int d = 0; d < (DUAL ? 2 : 1); d++)
#pragma unroll
      for (int j = 0; j < NT; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) tot[d][j][i] *= unscale;
    reduce_and_finish<NT, DUAL>(p, nt, lane, tot);
  }
}

// ---------------------------------------------------------------- host side
constexpr int kMaxSmem = 200 * 1024;

struct Plan {
  int nt;          // token tiles of 8 per pass (1, 2 or 4)
  int ksplit;
  int kt_per_split;
  int grid_x;
  size_t smem;
};

static Plan make_plan(int kind, int64_t M, int64_t N, int KT, int sblocks_per_tile) {
  Plan pl;
  const int ktile = (kind == TPX_W_MXFP4) ? 128 : 64;
  int mpass = (int)(M < 32 ? M : 32);
  pl.nt = mpass <= 8 ? 1 : mpass <= 16 ? 2 : 4;
  const int rows = pl.nt * 8;
  const int sms = sm_count();
  const int ntiles = (int)(N / 16);
  const int groups = (ntiles + kWarps - 1) / kWarps;
  // unit in which K may be split: whole scale blocks
  const int unit = (kind == TPX_W_INT8) ? sblocks_per_tile : 1;
  const int units = KT / unit;
  // smallest split whose activation slice fits shared memory, then more splits while the grid is
  // short of two CTAs per SM
  int ksplit = 1;
  auto smem_for = [&](int split) {
    int per = ((units + split - 1) / split) * unit;
    return (size_t)rows * ((size_t)per * ktile * 2 + 32);
  };
  while (smem_for(ksplit) > (size_t)kMaxSmem && ksplit < units) ksplit++;
  while (ksplit < units && ksplit < 16 && (int64_t)groups * ksplit < 2 * sms) ksplit++;
  pl.kt_per_split = ((units + ksplit - 1) / ksplit) * unit;
  pl.ksplit = (KT + pl.kt_per_split - 1) / pl.kt_per_split;
  pl.smem = (size_t)rows * ((size_t)pl.kt_per_split * ktile * 2 + 32);
  int ctas_per_sm = (int)(kMaxSmem / (pl.smem + 1024));
  ctas_per_sm = ctas_per_sm < 1 ? 1 : (ctas_per_sm > 3 ? 3 : ctas_per_sm);
  int want = sms * ctas_per_sm / pl.ksplit;
  if (want < 1) want = 1;
  pl.grid_x = groups < want ? groups : want;
  return pl;
}

}  // namespace tpx

using namespace tpx;

extern "C" size_t tpx_qlinear_scratch_bytes(int kind, int64_t M, int64_t N, int64_t K, int dual) {
  (void)kind; (void)M; (void)K; (void)dual;
  // partial sums: up to 16 K-splits x 2 weights x 32 tokens x N fp32, then one counter per 16 rows
  size_t partial = (size_t)16 * 2 * 32 * (size_t)N * sizeof(float);
  size_t counters = ((size_t)(N / 16) * sizeof(unsigned) + 255) & ~(size_t)255;
  return partial + counters;
}

template <int NT, bool DUAL>
static int launch_stream(int kind, const StreamParams& p, const Plan& pl, cudaStream_t st) {
  dim3 grid(pl.grid_x, pl.ksplit);
  if (kind == TPX_W_MXFP4) {
    TPX_CUDA_OK(cudaFuncSetAttribute(qlinear_stream_mxfp4<NT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    qlinear_stream_mxfp4<NT, DUAL><<<grid, kThreads, pl.smem, st>>>(p);
  } else {
    TPX_CUDA_OK(cudaFuncSetAttribute(qlinear_stream_int8<NT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    qlinear_stream_int8<NT, DUAL><<<grid, kThreads, pl.smem, st>>>(p);
  }
  TPX_LAUNCH_OK();
  return TPX_OK;
}

namespace tpx {
int qlinear_stream(int kind, const uint8_t* pk_codes, const void* pk_scales, const uint8_t* pk_codes2,
                   const void* pk_scales2, int64_t block_size, const uint16_t* x, int64_t M, int64_t N, int64_t K,
                   const uint16_t* bias, int act, const uint16_t* mul_in, const uint16_t* res, float res_scale,
                   uint16_t* y, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  const bool dual = pk_codes2 != nullptr;
  const int ktile = (kind == TPX_W_MXFP4) ? 128 : 64;
  const int KT = (int)((K + ktile - 1) / ktile);
  const int spt = (kind == TPX_W_INT8) ? (int)(block_size / 64) : 1;
  Plan pl = make_plan(kind, M, N, KT, spt);
  size_t need = tpx_qlinear_scratch_bytes(kind, M, N, K, dual);
  TPX_REQUIRE(pl.ksplit <= 16, TPX_ERR_UNSUPPORTED, "qlinear: K=%ld needs more than 16 K-splits", (long)K);
  if (pl.ksplit > 1) TPX_REQUIRE(scratch && scratch_bytes >= need, TPX_ERR_SCRATCH, "qlinear: scratch of %zu bytes needed, %zu given", need, scratch_bytes);
  StreamParams p;
  p.w = reinterpret_cast<const uint4*>(pk_codes);
  p.s = pk_scales;
  p.w2 = reinterpret_cast<const uint4*>(pk_codes2);
  p.s2 = pk_scales2;
  p.x = x; p.bias = bias; p.mul_in = mul_in; p.res = res; p.res_scale = res_scale; p.y = y;
  p.partial = reinterpret_cast<float*>(scratch);
  p.counters = scratch ? reinterpret_cast<unsigned*>(reinterpret_cast<unsigned char*>(scratch) + (size_t)16 * 2 * 32 * (size_t)N * sizeof(float)) : nullptr;
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.KT = KT;
  p.ksplit = pl.ksplit; p.kt_per_split = pl.kt_per_split; p.act = act; p.sblocks_per_tile = spt;
  const int mpass = pl.nt * 8;
  for (int64_t m0 = 0; m0 < M; m0 += mpass) {
    p.m0 = (int)m0;
    p.mcount = (int)((M - m0) < mpass ? (M - m0) : mpass);
    int rc;
    if (pl.nt == 1) rc = dual ? launch_stream<1, true>(kind, p, pl, st) : launch_stream<1, false>(kind, p, pl, st);
    else if (pl.nt == 2) rc = dual ? launch_stream<2, true>(kind, p, pl, st) : launch_stream<2, false>(kind, p, pl, st);
    else rc = dual ? launch_stream<4, true>(kind, p, pl, st) : launch_stream<4, false>(kind, p, pl, st);
    if (rc != TPX_OK) return rc;
  }
  return TPX_OK;
}
}  // namespace tpx
