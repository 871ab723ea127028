// Weight-streaming quantized linear for small token counts (decode): y = epilogue(x . dequant(W)^T).
//
// Replaces TppBlockedLinearW / TppBlockedQInt8LinearW of the reference
// (src/csrc/fused_gemm.h:784-1073, :1075-1341) in the bandwidth-bound regime (up to 32 tokens per
// pass). The packed weight is a sequence of self-contained tiles (16 output rows x 128 k for MXFP4
// with the 64 scale bytes appended, 16 x 64 k for int8), ordered [row tile][k tile], so any run of
// tiles of one row tile is one contiguous byte range.
//
//   * Work is a flat list of tiles per K slice, cut into equal contiguous ranges, one per warp
//     (stream-K): every warp of the grid streams the same number of bytes (+-1 tile).
//   * Each warp owns a ring of shared-memory stages filled by 1-D bulk async copies
//     (cp.async.bulk ... mbarrier::complete_tx) issued by its lane 0, so many KB per warp are in
//     flight without holding them in registers.
//   * W is the M operand of mma.sync.m16n8k16 (rows of W = "m", tokens = "n"). 4-bit codes become f16
//     with cvt.e2m1x2 (exact), int8 through the 1024+u magic number (exact); the block scale
//     multiplies the fp32 block sum after the MMAs, so every product is exact.
//   * Activations of the CTA's K slice are staged once in shared memory as f16 after an exact
//     power-of-two pre-scale that keeps them in f16 range.
//   * A row tile whose K range was cut between warps is completed through fp32 partial sums in
//     scratch: each contributor has its own slot, the last to arrive (a counter per row tile) adds the
//     slots in a fixed order and runs the epilogue, so results do not depend on timing.
#include "tpx_common.cuh"

namespace tpx {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 6;
constexpr int kTileMx = 1088;  // 1024 B of codes + 64 B of scales
constexpr int kTileI8 = 1024;
constexpr unsigned kSpinLimit = 1u << 26;  // bounded wait on a copy that never lands

struct StreamParams {
  const unsigned char* w;   // packed tiles
  const unsigned char* w2;  // second weight (gate/up pair) or null
  const float* s;           // int8 scales [N/16][K/B][16]
  const float* s2;
  const uint16_t* x;        // [M][K] bf16
  const uint16_t* bias;     // [N] or null
  const uint16_t* mul_in;
  const uint16_t* res;
  float res_scale;
  uint16_t* y;              // [M][N]
  float* partial;           // [slot][2][mpad][N] fp32
  unsigned* counters;       // [N/16]
  unsigned* err;            // set to 1 if a bounded wait gave up
  int M, N, K;
  int KT;                   // k tiles in the packed tensor
  int ksplit;               // grid.y
  int kt_per_split;         // k tiles per slice (the last slice may be shorter)
  int m0, mcount;           // token window of this launch
  int act;
  int tiles_per_sblock;     // int8: k tiles per scale block
  int max_slots;            // scratch slots per (row tile, slice)
};

// ---------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// two E2M1 codes (one byte) -> f16x2, low nibble in the low half
__device__ __forceinline__ uint32_t cvt_e2m1x2(uint32_t byte) {
  uint32_t r;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(r) : "r"(byte));
  return r;
}

__device__ __forceinline__ void s8x4_to_f16x2x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;  // biased to 0..255
  uint32_t l, h;
  asm("prmt.b32 %0, %1, %2, 0x5140;" : "=r"(l) : "r"(u), "r"(0x64646464u));
  asm("prmt.b32 %0, %1, %2, 0x7362;" : "=r"(h) : "r"(u), "r"(0x64646464u));
  const uint32_t magic = 0x64806480u;  // 1024 + 128
  asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(l), "r"(magic));
  asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(h), "r"(magic));
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------- activation staging
// The token window [mcount] x [k range] goes to shared memory as f16 scaled by 2^-p so that the
// largest magnitude lies in [2^14, 2^15). Rows beyond mcount are zero. Row stride = kslice*2 + 32
// bytes, which makes the 8-byte fragment reads of a half-warp hit 32 distinct banks.
template <int NT>
__device__ __forceinline__ float stage_x(const StreamParams& p, int k_begin, int kslice, unsigned char* xs, float* red) {
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
    *reinterpret_cast<uint4*>(xs + r * stride + c * 16) = v;
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
  const float down = __uint_as_float((uint32_t)(127 - pw) << 23);  // 2^-p
  for (int i = threadIdx.x; i < rows * vec_per_row; i += kThreads) {
    int r = i / vec_per_row, c = i % vec_per_row;
    uint4* ptr = reinterpret_cast<uint4*>(xs + r * stride + c * 16);
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
  return __uint_as_float((uint32_t)(127 + pw) << 23);  // 2^p
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

// Ownership of the flat tile list of one slice: warp gw of W owns units [gw*U/W, (gw+1)*U/W).
__device__ __forceinline__ long long owner_of(long long u, long long U, long long W) { return ((u + 1) * W - 1) / U; }

// One warp hands in its sum over its part of row tile nt. acc element i of token tile j of thread
// (g, t): row = g + 8*(i>>1), token = 8j + 2t + (i&1).
template <int NT, bool DUAL>
__device__ __forceinline__ void flush_rowtile(const StreamParams& p, int nt, int lane, int ks, int Lk, long long gw,
                                              long long U, long long W, bool whole, float (&tot)[DUAL ? 2 : 1][NT][4]) {
  const int g = lane >> 2, t = lane & 3;
  if (whole && p.ksplit == 1) {  // this warp saw the row tile's entire K range: no exchange needed
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int i = 0; i < 4; i++)
        finish(p, 8 * j + 2 * t + (i & 1), nt * 16 + g + 8 * (i >> 1), tot[0][j][i], DUAL ? tot[DUAL ? 1 : 0][j][i] : 0.0f, DUAL);
    return;
  }
  const int mpad = NT * 8;
  const size_t plane = (size_t)mpad * p.N;
  const long long first = owner_of((long long)nt * Lk, U, W);
  const int slot = ks * p.max_slots + (int)(gw - first);
#pragma unroll
  for (int d = 0; d < (DUAL ? 2 : 1); d++)
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int tok = 8 * j + 2 * t + (i & 1), row = nt * 16 + g + 8 * (i >> 1);
        if (tok < p.mcount) __stcg(p.partial + ((size_t)(slot * 2 + d)) * plane + (size_t)tok * p.N + row, tot[d][j][i]);
      }
  // contributors of this row tile over all slices (each slice is cut the same way)
  unsigned expected = 0;
  for (int s = 0; s < p.ksplit; s++) {
    int Ls = min(p.kt_per_split, p.KT - s * p.kt_per_split);
    long long Us = (long long)(p.N / 16) * Ls;
    expected += (unsigned)(owner_of((long long)(nt + 1) * Ls - 1, Us, W) - owner_of((long long)nt * Ls, Us, W) + 1);
  }
  __threadfence();
  __syncwarp();
  unsigned prev = 0;
  if (lane == 0) prev = atomicAdd(p.counters + nt, 1u);
  prev = __shfl_sync(0xffffffffu, prev, 0);
  if (prev != expected - 1) return;
  __threadfence();
  float v[NT][4], v2[NT][4];
#pragma unroll
  for (int j = 0; j < NT; j++)
#pragma unroll
    for (int i = 0; i < 4; i++) v[j][i] = v2[j][i] = 0.0f;
  for (int s = 0; s < p.ksplit; s++) {  // fixed order: slices, then contributors within a slice
    int Ls = min(p.kt_per_split, p.KT - s * p.kt_per_split);
    long long Us = (long long)(p.N / 16) * Ls;
    int cnt = (int)(owner_of((long long)(nt + 1) * Ls - 1, Us, W) - owner_of((long long)nt * Ls, Us, W) + 1);
    for (int c = 0; c < cnt; c++) {
      const float* base = p.partial + ((size_t)((s * p.max_slots + c) * 2)) * plane;
      float a[NT][4], b[NT][4];
#pragma unroll
      for (int j = 0; j < NT; j++)  // all of this contributor's loads are issued before any is used
#pragma unroll
        for (int i = 0; i < 4; i++) {
          int tok = 8 * j + 2 * t + (i & 1), row = nt * 16 + g + 8 * (i >> 1);
          a[j][i] = tok < p.mcount ? __ldcg(base + (size_t)tok * p.N + row) : 0.0f;
          b[j][i] = (DUAL && tok < p.mcount) ? __ldcg(base + plane + (size_t)tok * p.N + row) : 0.0f;
        }
#pragma unroll
      for (int j = 0; j < NT; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
          v[j][i] += a[j][i];
          v2[j][i] += b[j][i];
        }
    }
  }
#pragma unroll
  for (int j = 0; j < NT; j++)
#pragma unroll
    for (int i = 0; i < 4; i++)
      finish(p, 8 * j + 2 * t + (i & 1), nt * 16 + g + 8 * (i >> 1), v[j][i], v2[j][i], DUAL);
  if (lane == 0) p.counters[nt] = 0;  // leave the counter ready for the next launch
}

// ---------------------------------------------------------------- the kernel
// KIND: TPX_W_MXFP4 or TPX_W_INT8. NT: token tiles of 8. DUAL: gate/up pair.
template <int KIND, int NT, bool DUAL>
__global__ void __launch_bounds__(kThreads) qlinear_stream(StreamParams p) {
  constexpr int TILEB = (KIND == TPX_W_MXFP4) ? kTileMx : kTileI8;
  constexpr int KTILE = (KIND == TPX_W_MXFP4) ? 128 : 64;
  constexpr int STAGEB = (DUAL ? 2 : 1) * TILEB;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float red[kWarps];
  __shared__ __align__(8) unsigned long long bars[kWarps][kStages];

  pdl_trigger();
  pdl_wait();  // x, the residual and the scratch belong to earlier grids until they have completed
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int ks = blockIdx.y;
  const int kt_base = ks * p.kt_per_split;
  const int Lk = min(p.kt_per_split, p.KT - kt_base);
  const int T = p.N / 16;
  const long long U = (long long)T * Lk;
  const long long W = (long long)gridDim.x * kWarps;
  const long long gw = (long long)blockIdx.x * kWarps + warp;
  const long long u0 = gw * U / W, u1 = (gw + 1) * U / W;

  unsigned char* ring = smem + (size_t)warp * kStages * STAGEB;
  unsigned char* xs = smem + (size_t)kWarps * kStages * STAGEB;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kStages; s++) mbar_init(smem_u32(&bars[warp][s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();

  auto issue = [&](int stage, int nt, int kl) {  // lane 0 only
    const size_t off = ((size_t)nt * p.KT + kt_base + kl) * TILEB;
    const uint32_t bar = smem_u32(&bars[warp][stage]);
    const uint32_t dst = smem_u32(ring + (size_t)stage * STAGEB);
    mbar_expect_tx(bar, STAGEB);
    bulk_g2s(dst, p.w + off, TILEB, bar);
    if (DUAL) bulk_g2s(dst + TILEB, p.w2 + off, TILEB, bar);
  };
  const int nunits = (int)(u1 - u0);
  // (row tile, k tile) of the next unit to be fetched, advanced without divisions
  int f_nt = (nunits > 0) ? (int)(u0 / Lk) : 0, f_kl = (nunits > 0) ? (int)(u0 % Lk) : 0, fetched = 0;
  if (lane == 0) {
    for (; fetched < kStages && fetched < nunits; fetched++) {
      issue(fetched, f_nt, f_kl);
      if (++f_kl == Lk) { f_kl = 0; f_nt++; }
    }
  }

  const int kslice = p.kt_per_split * KTILE;
  const int stride = kslice * 2 + 32;
  const float unscale = stage_x<NT>(p, kt_base * KTILE, kslice, xs, red);

  float tot[DUAL ? 2 : 1][NT][4];
  float blk[DUAL ? 2 : 1][NT][4];  // int8: running sum of the current scale block
#pragma unroll
  for (int d = 0; d < (DUAL ? 2 : 1); d++)
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int i = 0; i < 4; i++) tot[d][j][i] = blk[d][j][i] = 0.0f;

  int cur_nt = (nunits > 0) ? (int)(u0 / Lk) : -1;
  int first_kl = (nunits > 0) ? (int)(u0 % Lk) : 0;
  bool dead = false;
  int nt = cur_nt, kl = first_kl - 1, stage = -1;
  uint32_t parity = 0;

  for (int it = 0; it < nunits && !dead; it++) {
    if (++kl == Lk) { kl = 0; nt++; }
    if (++stage == kStages) { stage = 0; parity ^= (it != 0); }
    if (nt != cur_nt) {
#pragma unroll
      for (int d = 0; d < (DUAL ? 2 : 1); d++)
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
          for (int i = 0; i < 4; i++) tot[d][j][i] *= unscale;
      flush_rowtile<NT, DUAL>(p, cur_nt, lane, ks, Lk, gw, U, W, first_kl == 0, tot);
#pragma unroll
      for (int d = 0; d < (DUAL ? 2 : 1); d++)
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
          for (int i = 0; i < 4; i++) tot[d][j][i] = 0.0f;
      cur_nt = nt;
      first_kl = 0;
    }
    const uint32_t bar = smem_u32(&bars[warp][stage]);
    unsigned spins = 0;
    while (!mbar_try_wait(bar, parity)) {
      if (++spins > kSpinLimit) {  // the copy never landed: report and leave instead of hanging
        if (lane == 0) atomicExch(p.err, 1u);
        dead = true;
        break;
      }
    }
    if (dead) break;
    const unsigned char* st = ring + (size_t)stage * STAGEB;
    uint4 cur[DUAL ? 2 : 1][2];
    uint32_t csc[DUAL ? 2 : 1][2];
#pragma unroll
    for (int d = 0; d < (DUAL ? 2 : 1); d++) {
      const uint4* tp = reinterpret_cast<const uint4*>(st + d * TILEB);
      cur[d][0] = tp[lane];
      cur[d][1] = tp[32 + lane];
      if (KIND == TPX_W_MXFP4) {
        const uint32_t* sp = reinterpret_cast<const uint32_t*>(st + d * TILEB + 1024);
        csc[d][0] = sp[g];
        csc[d][1] = sp[g + 8];
      }
    }

    const unsigned char* xrow = xs + g * stride + (kl * KTILE + 4 * t) * 2;
    if (KIND == TPX_W_MXFP4) {
#pragma unroll
      for (int b = 0; b < 4; b++) {
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
          float bs[NT][4];
#pragma unroll
          for (int j = 0; j < NT; j++)
#pragma unroll
            for (int i = 0; i < 4; i++) bs[j][i] = 0.0f;
#pragma unroll
          for (int hh = 0; hh < 2; hh++) {
            uint32_t a0 = cvt_e2m1x2((wa >> (16 * hh)) & 0xff);
            uint32_t a2 = cvt_e2m1x2((wa >> (16 * hh + 8)) & 0xff);
            uint32_t a1 = cvt_e2m1x2((wc >> (16 * hh)) & 0xff);
            uint32_t a3 = cvt_e2m1x2((wc >> (16 * hh + 8)) & 0xff);
#pragma unroll
            for (int j = 0; j < NT; j++) mma_f16(bs[j], a0, a1, a2, a3, xb[hh][j].x, xb[hh][j].y);
          }
          const float s0 = __uint_as_float(((csc[d][0] >> (8 * b)) & 0xffu) << 23);
          const float s1 = __uint_as_float(((csc[d][1] >> (8 * b)) & 0xffu) << 23);
#pragma unroll
          for (int j = 0; j < NT; j++) {
            tot[d][j][0] = fmaf(s0, bs[j][0], tot[d][j][0]);
            tot[d][j][1] = fmaf(s0, bs[j][1], tot[d][j][1]);
            tot[d][j][2] = fmaf(s1, bs[j][2], tot[d][j][2]);
            tot[d][j][3] = fmaf(s1, bs[j][3], tot[d][j][3]);
          }
        }
      }
    } else {
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
      // fold the running sum in at the end of a scale block, or when this warp's part of the row tile ends
      const int kt = kt_base + kl;
      const bool last_of_part = (it + 1 == nunits) || (kl + 1 == Lk);
      if ((kt + 1) % p.tiles_per_sblock == 0 || last_of_part) {
        const int sb = kt / p.tiles_per_sblock;
        const int nsb = p.KT / p.tiles_per_sblock;
#pragma unroll
        for (int d = 0; d < (DUAL ? 2 : 1); d++) {
          const float* sp = (d ? p.s2 : p.s) + ((size_t)nt * nsb + sb) * 16;
          const float s0 = __ldg(sp + g), s1 = __ldg(sp + g + 8);
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
    // the stage's contents have been consumed by every lane (their values fed the MMAs): refill it
    __syncwarp();
    if (lane == 0 && fetched < nunits) {
      issue(stage, f_nt, f_kl);
      fetched++;
      if (++f_kl == Lk) { f_kl = 0; f_nt++; }
    }
  }
  if (cur_nt >= 0 && !dead) {
#pragma unroll
    for (int d = 0; d < (DUAL ? 2 : 1); d++)
#pragma unroll
      for (int j = 0; j < NT; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) tot[d][j][i] *= unscale;
    const bool whole = first_kl == 0 && kl == Lk - 1;
    flush_rowtile<NT, DUAL>(p, cur_nt, lane, ks, Lk, gw, U, W, whole, tot);
  }
}

// ---------------------------------------------------------------- host side
constexpr int kMaxSmem = 220 * 1024;
constexpr int kMaxSplit = 16;
// Scratch layout: [0, 64 KiB) one arrival counter per 16-row tile, always at the same place so that a
// buffer reused across shapes keeps them zero; its last word is the error flag. The partial sums follow.
static constexpr size_t kCounterBytes = 64 * 1024;

struct Plan {
  int nt;            // token tiles of 8 per pass (1, 2 or 4)
  int ksplit;
  int kt_per_split;
  int grid_x;
  int max_slots;
  size_t smem;
  size_t scratch;
};

static Plan make_plan(int kind, int64_t M, int64_t N, int64_t K, int64_t block_size, bool dual) {
  Plan pl;
  const int ktile = (kind == TPX_W_MXFP4) ? 128 : 64;
  const int tileb = (kind == TPX_W_MXFP4) ? kTileMx : kTileI8;
  const int KT = (int)((K + ktile - 1) / ktile);
  const int unit = (kind == TPX_W_INT8) ? (int)(block_size / 64) : 1;  // K may only be cut at scale-block ends
  const int units = KT / unit;
  int mpass = (int)(M < 32 ? M : 32);
  pl.nt = mpass <= 8 ? 1 : mpass <= 16 ? 2 : 4;
  const int rows = pl.nt * 8;
  const size_t ring = (size_t)kWarps * kStages * (dual ? 2 : 1) * tileb;
  const int sms = sm_count();
  const int T = (int)(N / 16);
  auto xbytes = [&](int split) {
    int per = ((units + split - 1) / split) * unit;
    return (size_t)rows * ((size_t)per * ktile * 2 + 32);
  };
  int ksplit = 1;
  while (ring + xbytes(ksplit) > (size_t)kMaxSmem && ksplit < units) ksplit++;
  pl.kt_per_split = ((units + ksplit - 1) / ksplit) * unit;
  pl.ksplit = (KT + pl.kt_per_split - 1) / pl.kt_per_split;
  pl.smem = ring + (size_t)rows * ((size_t)pl.kt_per_split * ktile * 2 + 32);
  // one CTA per SM over all slices, the same number of CTAs for every slice; never more warps than
  // tiles in the shortest slice
  int gx = sms / pl.ksplit;
  if (gx < 1) gx = 1;
  const int last_len = KT - (pl.ksplit - 1) * pl.kt_per_split;
  const long long min_units = (long long)T * last_len;
  while (gx > 1 && (long long)gx * kWarps > min_units) gx--;
  pl.grid_x = gx;
  // contributors per (row tile, slice): a row tile of L tiles cut into ranges of >= floor(U/W) tiles
  const long long Wt = (long long)gx * kWarps;
  const long long per = min_units / Wt;  // shortest range over all slices
  long long slots = (per > 0 ? (pl.kt_per_split + per - 1) / per : pl.kt_per_split) + 1;
  if (slots > pl.kt_per_split) slots = pl.kt_per_split;
  if (slots < 1) slots = 1;
  pl.max_slots = (int)slots;
  pl.scratch = kCounterBytes + (size_t)pl.ksplit * pl.max_slots * 2 * rows * (size_t)N * sizeof(float);
  return pl;
}

template <int KIND, int NT, bool DUAL>
static int launch_one(const StreamParams& p, const Plan& pl, cudaStream_t st) {
  static bool opted[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || !opted[dev]) {
    TPX_CUDA_OK(cudaFuncSetAttribute(qlinear_stream<KIND, NT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem));
    if (dev >= 0 && dev < 16) opted[dev] = true;
  }
  TPX_CUDA_OK(launch_pdl(qlinear_stream<KIND, NT, DUAL>, dim3(pl.grid_x, pl.ksplit), dim3(kThreads), (size_t)pl.smem, st, p));
  return TPX_OK;
}

template <int KIND>
static int launch_kind(const StreamParams& p, const Plan& pl, bool dual, cudaStream_t st) {
  if (pl.nt == 1) return dual ? launch_one<KIND, 1, true>(p, pl, st) : launch_one<KIND, 1, false>(p, pl, st);
  if (pl.nt == 2) return dual ? launch_one<KIND, 2, true>(p, pl, st) : launch_one<KIND, 2, false>(p, pl, st);
  return dual ? launch_one<KIND, 4, true>(p, pl, st) : launch_one<KIND, 4, false>(p, pl, st);
}

size_t qlinear_stream_scratch_bytes(int kind, int64_t M, int64_t N, int64_t K, int64_t block_size, bool dual) {
  return make_plan(kind, M, N, K, block_size, dual).scratch;
}

int qlinear_stream_launch(int kind, const uint8_t* pk_codes, const void* pk_scales, const uint8_t* pk_codes2,
                          const void* pk_scales2, int64_t block_size, const uint16_t* x, int64_t M, int64_t N, int64_t K,
                          const uint16_t* bias, int act, const uint16_t* mul_in, const uint16_t* res, float res_scale,
                          uint16_t* y, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  const bool dual = pk_codes2 != nullptr;
  Plan pl = make_plan(kind, M, N, K, block_size, dual);
  TPX_REQUIRE(pl.ksplit <= kMaxSplit, TPX_ERR_UNSUPPORTED, "qlinear: K=%ld needs more than %d K slices", (long)K, kMaxSplit);
  TPX_REQUIRE((size_t)(N / 16) * sizeof(unsigned) <= kCounterBytes - 16, TPX_ERR_UNSUPPORTED, "qlinear: N=%ld exceeds the counter region", (long)N);
  TPX_REQUIRE(scratch && scratch_bytes >= pl.scratch, TPX_ERR_SCRATCH, "qlinear: scratch of %zu bytes needed, %zu given", pl.scratch, scratch_bytes);
  StreamParams p;
  p.w = pk_codes; p.w2 = pk_codes2;
  p.s = reinterpret_cast<const float*>(pk_scales); p.s2 = reinterpret_cast<const float*>(pk_scales2);
  p.x = x; p.bias = bias; p.mul_in = mul_in; p.res = res; p.res_scale = res_scale; p.y = y;
  p.counters = reinterpret_cast<unsigned*>(scratch);
  p.err = reinterpret_cast<unsigned*>(reinterpret_cast<unsigned char*>(scratch) + kCounterBytes - 4);
  p.partial = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(scratch) + kCounterBytes);
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.KT = (int)((K + ((kind == TPX_W_MXFP4) ? 127 : 63)) / ((kind == TPX_W_MXFP4) ? 128 : 64));
  p.ksplit = pl.ksplit; p.kt_per_split = pl.kt_per_split; p.act = act;
  p.tiles_per_sblock = (kind == TPX_W_INT8) ? (int)(block_size / 64) : 1;
  p.max_slots = pl.max_slots;
  const int mpass = pl.nt * 8;
  for (int64_t m0 = 0; m0 < M; m0 += mpass) {
    p.m0 = (int)m0;
    p.mcount = (int)((M - m0) < mpass ? (M - m0) : mpass);
    int rc = (kind == TPX_W_MXFP4) ? launch_kind<TPX_W_MXFP4>(p, pl, dual, st) : launch_kind<TPX_W_INT8>(p, pl, dual, st);
    if (rc != TPX_OK) return rc;
  }
  return TPX_OK;
}

}  // namespace tpx
