// RMSNorm, RoPE + KV-cache write, and attention over the blocked KV cache.
//
// Replaces, on the decoder-layer path of the reference:
//   llama_rms_norm / RMSNormFwdTPP           src/csrc/llm/fused_llm_infer.cpp:336-363, src/csrc/xsmm_functors.h:4628-4654
//   apply_rotary_pos_emb_llama               src/csrc/llm/fused_llm_infer.cpp:206-253
//   LayerCache::update / KVLayout_BNSH       src/csrc/llm/attn.h:197-221, src/csrc/llm/attn.cpp:389-463
//   attn<T>                                  src/csrc/llm/attn.cpp:780-955
//
// The KV cache keeps the reference's layout [S1][B][Nkv][32][H] (token t at block t/32, slot t%32): a block of
// 32 tokens of one (batch, kv head) is 32*H contiguous elements, which is what the attention kernel streams.
#include "tpx_attn.cuh"

namespace tpx {

// ---------------------------------------------------------------- RMSNorm: one warp per row
__global__ void rmsnorm_kernel(const uint16_t* __restrict__ x, const void* __restrict__ gamma, int gamma_f32, float eps,
                               int64_t rows, int D, uint16_t* __restrict__ y) {
  pdl_trigger();
  pdl_wait();
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
  float ss = 0.0f;
  for (int i = lane; i < D / 8; i += 32) {
    uint4 v = xr[i];
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float a = bf16_bits_to_f32((uint16_t)(w[j] & 0xffff)), b = bf16_bits_to_f32((uint16_t)(w[j] >> 16));
      ss += a * a + b * b;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = rsqrtf(ss / (float)D + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + row * D);
  for (int i = lane; i < D / 8; i += 32) {
    uint4 v = xr[i];
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float g0, g1;
      if (gamma_f32) {
        g0 = reinterpret_cast<const float*>(gamma)[i * 8 + 2 * j];
        g1 = reinterpret_cast<const float*>(gamma)[i * 8 + 2 * j + 1];
      } else {
        g0 = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(gamma)[i * 8 + 2 * j]);
        g1 = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(gamma)[i * 8 + 2 * j + 1]);
      }
      float a = bf16_bits_to_f32((uint16_t)(w[j] & 0xffff)) * inv * g0;
      float b = bf16_bits_to_f32((uint16_t)(w[j] >> 16)) * inv * g1;
      o[j] = (uint32_t)f32_to_bf16_bits(a) | ((uint32_t)f32_to_bf16_bits(b) << 16);
    }
    yr[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---------------------------------------------------------------- LayerNorm: one warp per row
// y = (x - mean) * rsqrt(var + eps) * gamma + beta with fp32 statistics (lyr_norm / LayerNormFwdTPP,
// src/csrc/llm/fused_llm_infer.cpp:256-306): the norm of the OPT and GPT-J blocks. The variance is taken around the
// mean in a second pass over the row (it comes from L1), not as E[x^2] - mean^2.
__device__ __forceinline__ float ln_param(const void* p, int f32, int i) {
  return f32 ? reinterpret_cast<const float*>(p)[i] : bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(p)[i]);
}
__global__ void layernorm_kernel(const uint16_t* __restrict__ x, const void* __restrict__ gamma, const void* __restrict__ beta,
                                 int params_f32, float eps, int64_t rows, int D, uint16_t* __restrict__ y) {
  pdl_trigger();
  pdl_wait();
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
  float s = 0.0f;
  for (int i = lane; i < D / 8; i += 32) {
    const uint4 v = xr[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) s += bf16_bits_to_f32((uint16_t)(w[j] & 0xffff)) + bf16_bits_to_f32((uint16_t)(w[j] >> 16));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float mean = s / (float)D;
  float ss = 0.0f;
  for (int i = lane; i < D / 8; i += 32) {
    const uint4 v = xr[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float a = bf16_bits_to_f32((uint16_t)(w[j] & 0xffff)) - mean, b = bf16_bits_to_f32((uint16_t)(w[j] >> 16)) - mean;
      ss += a * a + b * b;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = rsqrtf(ss / (float)D + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + row * D);
  for (int i = lane; i < D / 8; i += 32) {
    const uint4 v = xr[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float a = (bf16_bits_to_f32((uint16_t)(w[j] & 0xffff)) - mean) * inv * ln_param(gamma, params_f32, i * 8 + 2 * j) +
                      ln_param(beta, params_f32, i * 8 + 2 * j);
      const float b = (bf16_bits_to_f32((uint16_t)(w[j] >> 16)) - mean) * inv * ln_param(gamma, params_f32, i * 8 + 2 * j + 1) +
                      ln_param(beta, params_f32, i * 8 + 2 * j + 1);
      o[j] = (uint32_t)f32_to_bf16_bits(a) | ((uint32_t)f32_to_bf16_bits(b) << 16);
    }
    yr[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Few rows (decoding): one CTA of 256 threads per row, the row kept in registers between the two passes.
constexpr int kNormThreads = 256;
constexpr int kNormVecs = 4;  // uint4 vectors per thread held in registers: rows up to 256 * 4 * 8 = 8192 elements
__global__ void __launch_bounds__(kNormThreads) rmsnorm_row_kernel(const uint16_t* __restrict__ x, const void* __restrict__ gamma,
                                                                   int gamma_f32, float eps, int D, uint16_t* __restrict__ y) {
  __shared__ float red[kNormThreads / 32];
  pdl_trigger();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int nv = D / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
  uint4 v[kNormVecs];
  float ss = 0.0f;
#pragma unroll
  for (int q = 0; q < kNormVecs; q++) {
    const int i = threadIdx.x + q * kNormThreads;
    v[q] = i < nv ? xr[i] : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int q = 0; q < kNormVecs; q++) {
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
  for (int w = 0; w < kNormThreads / 32; w++) tot += red[w];
  const float inv = rsqrtf(tot / (float)D + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + row * D);
#pragma unroll
  for (int q = 0; q < kNormVecs; q++) {
    const int i = threadIdx.x + q * kNormThreads;
    if (i >= nv) continue;
    const uint32_t w[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
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
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float a = bf16_bits_to_f32((uint16_t)(w[j] & 0xffff)) * inv * g[2 * j];
      float b = bf16_bits_to_f32((uint16_t)(w[j] >> 16)) * inv * g[2 * j + 1];
      o[j] = (uint32_t)f32_to_bf16_bits(a) | ((uint32_t)f32_to_bf16_bits(b) << 16);
    }
    yr[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---------------------------------------------------------------- RoPE + KV-cache write
// qkv: [B*S][(Nq + 2*Nkv)*H] bf16, the output of the fused q/k/v linear (q heads, then k heads, then v heads).
// q is rotated and written as q_out[B][Nkv][S][R][H] (R = Nq/Nkv, the layout the reference hands to attention,
// src/csrc/llm/fused_llm_infer.cpp:563-584); k is rotated and stored, v stored, at cache tokens offset .. offset+S-1.
// One thread per (token, head, pair of rotary lanes).
__global__ void rope_kv_kernel(const uint16_t* __restrict__ qkv, const float* __restrict__ ep, const int64_t* __restrict__ pos,
                               int B, int S, int Nq, int Nkv, int H, int MP, int HR, int Bpos, int64_t offset_arg,
                               const int* __restrict__ dev_len, int64_t capacity, uint16_t* __restrict__ q_out, uint16_t* __restrict__ kc, uint16_t* __restrict__ vc,
                               const uint64_t* __restrict__ kpages, const uint64_t* __restrict__ vpages) {
  pdl_trigger();
  pdl_wait();
  const int heads = Nq + 2 * Nkv;
  const int half = H / 2;
  const int64_t offset = dev_len ? (int64_t)*dev_len : offset_arg;  // tokens already cached
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)B * S * heads * half) return;
  const int h2 = (int)(idx % half);
  const int hd = (int)((idx / half) % heads);
  const int s = (int)((idx / ((int64_t)half * heads)) % S);
  const int b = (int)(idx / ((int64_t)half * heads * S));
  const uint16_t* src = qkv + ((int64_t)(b * S + s) * heads + hd) * H;
  uint16_t o0 = src[h2], o1 = src[h2 + half];
  if (hd < Nq + Nkv) {  // q and k heads rotate: pair (h2, h2 + H/2)
    const int64_t p = pos[(int64_t)(Bpos == 1 ? 0 : b) * S + s];
    if (p < MP) {  // positions beyond the table are left untouched, as in the reference
      const float x0 = bf16_bits_to_f32(o0), x1 = bf16_bits_to_f32(o1);
      const float c = ep[(0 * (int64_t)MP + p) * HR + h2], sn = ep[(1 * (int64_t)MP + p) * HR + h2];
      o0 = f32_to_bf16_bits(x0 * c - x1 * sn);
      o1 = f32_to_bf16_bits(x1 * c + x0 * sn);
    }
  }
  uint16_t* dst;
  if (hd < Nq) {
    const int R = Nq / Nkv, n = hd / R, r = hd % R;
    dst = q_out + ((((int64_t)b * Nkv + n) * S + s) * R + r) * H;
  } else {
    const bool is_k = hd < Nq + Nkv;
    const int n = is_k ? hd - Nq : hd - Nq - Nkv;
    const int64_t t = offset + s;
    if (t >= capacity) return;  // never write beyond the cache (the host checks this when it knows the offset)
    if (kpages) {  // paged cache: block t / 32 lives wherever its page was allocated
      dst = reinterpret_cast<uint16_t*>((is_k ? kpages : vpages)[t / 32]) + (((int64_t)b * Nkv + n) * 32 + (t % 32)) * H;
    } else {
      dst = (is_k ? kc : vc) + ((((t / 32) * B + b) * Nkv + n) * 32 + (t % 32)) * H;
    }
  }
  dst[h2] = o0;
  dst[h2 + half] = o1;
}

// The same with one thread per (token, head, eight pairs of rotary lanes): 16-byte loads and stores. For head sizes
// that are a multiple of 16 and 16-byte aligned tensors; the arithmetic is the scalar kernel's, lane for lane.
__global__ void rope_kv_v8_kernel(const uint16_t* __restrict__ qkv, const float* __restrict__ ep, const int64_t* __restrict__ pos,
                                  int B, int S, int Nq, int Nkv, int H, int MP, int HR, int Bpos, int64_t offset_arg,
                                  const int* __restrict__ dev_len, int64_t capacity, uint16_t* __restrict__ q_out, uint16_t* __restrict__ kc,
                                  uint16_t* __restrict__ vc, const uint64_t* __restrict__ kpages, const uint64_t* __restrict__ vpages) {
  pdl_trigger();
  pdl_wait();
  const int heads = Nq + 2 * Nkv;
  const int half = H / 2, groups = half / 8;
  const int64_t offset = dev_len ? (int64_t)*dev_len : offset_arg;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)B * S * heads * groups) return;
  const int h2 = (int)(idx % groups) * 8;
  const int hd = (int)((idx / groups) % heads);
  const int s = (int)((idx / ((int64_t)groups * heads)) % S);
  const int b = (int)(idx / ((int64_t)groups * heads * S));
  const uint16_t* src = qkv + ((int64_t)(b * S + s) * heads + hd) * H;
  uint4 lo = *reinterpret_cast<const uint4*>(src + h2), hi = *reinterpret_cast<const uint4*>(src + h2 + half);
  if (hd < Nq + Nkv) {
    const int64_t p = pos[(int64_t)(Bpos == 1 ? 0 : b) * S + s];
    if (p < MP) {
      const float* cs = ep + (0 * (int64_t)MP + p) * HR + h2;
      const float* sp = ep + (1 * (int64_t)MP + p) * HR + h2;
      const float4 c0 = *reinterpret_cast<const float4*>(cs), c1 = *reinterpret_cast<const float4*>(cs + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
      const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        uint32_t nl = 0, nh = 0;
#pragma unroll
        for (int e = 0; e < 2; e++) {
          const float x0 = bf16_bits_to_f32((uint16_t)(lw[j] >> (16 * e))), x1 = bf16_bits_to_f32((uint16_t)(hw[j] >> (16 * e)));
          const float c = cv[2 * j + e], sn = sv[2 * j + e];
          nl |= (uint32_t)f32_to_bf16_bits(x0 * c - x1 * sn) << (16 * e);
          nh |= (uint32_t)f32_to_bf16_bits(x1 * c + x0 * sn) << (16 * e);
        }
        lw[j] = nl;
        hw[j] = nh;
      }
      lo = make_uint4(lw[0], lw[1], lw[2], lw[3]);
      hi = make_uint4(hw[0], hw[1], hw[2], hw[3]);
    }
  }
  uint16_t* dst;
  if (hd < Nq) {
    const int R = Nq / Nkv, n = hd / R, r = hd % R;
    dst = q_out + ((((int64_t)b * Nkv + n) * S + s) * R + r) * H;
  } else {
    const bool is_k = hd < Nq + Nkv;
    const int n = is_k ? hd - Nq : hd - Nq - Nkv;
    const int64_t t = offset + s;
    if (t >= capacity) return;
    if (kpages) {
      dst = reinterpret_cast<uint16_t*>((is_k ? kpages : vpages)[t / 32]) + (((int64_t)b * Nkv + n) * 32 + (t % 32)) * H;
    } else {
      dst = (is_k ? kc : vc) + ((((t / 32) * B + b) * Nkv + n) * 32 + (t % 32)) * H;
    }
  }
  *reinterpret_cast<uint4*>(dst + h2) = lo;
  *reinterpret_cast<uint4*>(dst + h2 + half) = hi;
}

// GPT-J's rotary embedding (apply_rotary_pos_emb_gptj, src/csrc/llm/fused_llm_infer.cpp:150-204) with the same q permute
// and cache append: the first HR values of a head rotate in ADJACENT pairs (2i, 2i+1), the table is [MP][HR] with the
// HR/2 sines first, then the cosines; the rest of the head passes through. One thread per (token, head, adjacent pair).
__global__ void rope_kv_gptj_kernel(const uint16_t* __restrict__ qkv, const float* __restrict__ ep, const int64_t* __restrict__ pos,
                                    int B, int S, int Nq, int Nkv, int H, int MP, int HR, int Bpos, int64_t offset_arg,
                                    const int* __restrict__ dev_len, int64_t capacity, uint16_t* __restrict__ q_out, uint16_t* __restrict__ kc,
                                    uint16_t* __restrict__ vc, const uint64_t* __restrict__ kpages, const uint64_t* __restrict__ vpages) {
  pdl_trigger();
  pdl_wait();
  const int heads = Nq + 2 * Nkv;
  const int half = H / 2;
  const int64_t offset = dev_len ? (int64_t)*dev_len : offset_arg;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)B * S * heads * half) return;
  const int h2 = (int)(idx % half);
  const int hd = (int)((idx / half) % heads);
  const int s = (int)((idx / ((int64_t)half * heads)) % S);
  const int b = (int)(idx / ((int64_t)half * heads * S));
  const uint16_t* src = qkv + ((int64_t)(b * S + s) * heads + hd) * H;
  const uint32_t in = *reinterpret_cast<const uint32_t*>(src + 2 * h2);
  uint16_t o0 = (uint16_t)(in & 0xffff), o1 = (uint16_t)(in >> 16);
  if (hd < Nq + Nkv && 2 * h2 < HR) {
    const int64_t p = pos[(int64_t)(Bpos == 1 ? 0 : b) * S + s];
    if (p < MP) {
      const float x0 = bf16_bits_to_f32(o0), x1 = bf16_bits_to_f32(o1);
      const float sn = ep[p * HR + h2], c = ep[p * HR + HR / 2 + h2];
      // every product rounded on its own (no fused multiply-add): the same value on every compiler and in the oracle
      o0 = f32_to_bf16_bits(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn)));
      o1 = f32_to_bf16_bits(__fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, sn)));
    }
  }
  uint16_t* dst;
  if (hd < Nq) {
    const int R = Nq / Nkv, n = hd / R, r = hd % R;
    dst = q_out + ((((int64_t)b * Nkv + n) * S + s) * R + r) * H;
  } else {
    const bool is_k = hd < Nq + Nkv;
    const int n = is_k ? hd - Nq : hd - Nq - Nkv;
    const int64_t t = offset + s;
    if (t >= capacity) return;
    if (kpages) {
      dst = reinterpret_cast<uint16_t*>((is_k ? kpages : vpages)[t / 32]) + (((int64_t)b * Nkv + n) * 32 + (t % 32)) * H;
    } else {
      dst = (is_k ? kc : vc) + ((((t / 32) * B + b) * Nkv + n) * 32 + (t % 32)) * H;
    }
  }
  *reinterpret_cast<uint32_t*>(dst + 2 * h2) = (uint32_t)o0 | ((uint32_t)o1 << 16);
}

// ---------------------------------------------------------------- attention
// Query rows are consecutive (query position, group member) pairs of one (batch, kv head). Each warp keeps a
// running (max, sum, fp32 output) for 16 rows over the KV blocks it visits. With more than one KV split a CTA
// writes an un-normalised partial (max, sum, output); the split that arrives last merges them (flash-decoding).

// ---- tensor-core attention (mma.sync m16n8k16, bf16 in, fp32 accumulate), flash-attention style
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // size 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// MODE 0 (prefill): a CTA owns 64 consecutive query rows (16 per warp) of one (batch, kv head); its four warps
//   share every KV block, copied once into shared memory (two stages, cp.async).
// MODE 1 (decoding, at most 16 query rows): all kDecWarps warps work on the same 16 rows and take every kDecWarps-th KV block of
//   the CTA's split, each with its own two stages; the warps' (max, sum, output) are merged through shared memory,
//   and with more than one KV split the CTA writes an un-normalised partial that the last-arriving split merges.
// Rows of a KV block are kept 16 bytes apart from a power-of-two pitch so that ldmatrix is conflict-free.
template <int H, int MODE>
__global__ void __launch_bounds__((MODE == 0 ? kAttnWarps : kDecWarps) * 32) attn_mma_kernel(AttnParams p) {
  constexpr int WARPS = MODE == 0 ? kAttnWarps : kDecWarps;
  constexpr int PB = H * 2 + 16;        // bytes per key row in shared memory
  constexpr int TILE = 32 * PB;         // one block of keys or of values
  constexpr int STAGE = 2 * TILE;       // keys, then values
  constexpr int NT = H / 8;             // output n-tiles
  constexpr int KK = H / 16;            // k steps of Q.K^T
  constexpr int GROUP = MODE == 0 ? WARPS * 32 : 32;  // threads that share a KV stream
  extern __shared__ __align__(16) unsigned char attn_smem[];
  __shared__ float red_m[WARPS][kAttnRows], red_l[WARPS][kAttnRows];

  pdl_trigger();
  pdl_wait();
  const int bn = blockIdx.x, chunk = blockIdx.y, split = blockIdx.z;
  const int b = bn / p.Nkv, n = bn % p.Nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int rows_total = p.Sq * p.R;
  const int cta_row0 = chunk * (MODE == 0 ? 64 : 16);
  const int row0 = cta_row0 + (MODE == 0 ? warp * 16 : 0);  // first of this warp's 16 rows
  const int key_len = p.dev_len ? *p.dev_len + p.Sq : p.key_len;
  const int offset = key_len - p.Sq;

  // keys this CTA can see at all (last row's causal limit), cut into the CTA's KV split
  const int cta_last_row = min(rows_total, cta_row0 + (MODE == 0 ? 64 : 16)) - 1;
  const int kmax = p.causal ? min(key_len, offset + cta_last_row / p.R + 1) : key_len;
  const int nblocks = (kmax + 31) / 32;
  const int per_split = (nblocks + p.splits - 1) / p.splits;
  const int blk0 = split * per_split, blk1 = min(nblocks, blk0 + per_split);
  // keys this warp's rows can see
  const int warp_last_row = min(rows_total - 1, row0 + 15);
  const int warp_kmax = (row0 < rows_total) ? (p.causal ? min(key_len, offset + warp_last_row / p.R + 1) : key_len) : 0;

  // query fragments (A operand), straight from global memory
  uint32_t qf[KK][4];
  {
    const uint16_t* qbase = p.q + (int64_t)bn * rows_total * H;
    const int ra = row0 + g, rb = row0 + g + 8;
#pragma unroll
    for (int kk = 0; kk < KK; kk++) {
      const int c = kk * 16 + 2 * t;
      qf[kk][0] = ra < rows_total ? *reinterpret_cast<const uint32_t*>(qbase + (int64_t)ra * H + c) : 0u;
      qf[kk][1] = rb < rows_total ? *reinterpret_cast<const uint32_t*>(qbase + (int64_t)rb * H + c) : 0u;
      qf[kk][2] = ra < rows_total ? *reinterpret_cast<const uint32_t*>(qbase + (int64_t)ra * H + c + 8) : 0u;
      qf[kk][3] = rb < rows_total ? *reinterpret_cast<const uint32_t*>(qbase + (int64_t)rb * H + c + 8) : 0u;
    }
  }
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};  // rows g and g + 8; l is this thread's share

  constexpr int NST = 2;  // stages per KV stream (a third stage per warp measured no faster, also with 16 blocks per warp: 102.5 against 103.5 us at batch 64 x 4096 tokens; a warp's own arithmetic per block bounds decoding)
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(attn_smem) + (MODE == 0 ? 0u : (uint32_t)warp * (uint32_t)NST * STAGE);
  const int gtid = MODE == 0 ? threadIdx.x : lane;
  // A copying thread keeps its chunk column and walks down the rows: thread j of the group copies chunk j % CPR of
  // rows j / CPR, + GROUP / CPR, ...; per copy that is one add on each side.
  constexpr int CPR = H / 8;            // 16-byte chunks per row
  constexpr int RSTEP = GROUP / CPR;    // rows between a thread's consecutive copies
  static_assert(GROUP % CPR == 0 && 32 % RSTEP == 0, "copy pattern");
  const int cp_r0 = gtid / CPR, cp_c = gtid % CPR;
  const uint32_t cp_dst0 = sbase + (uint32_t)(cp_r0 * PB + cp_c * 16);
  const int64_t cp_src0 = (((int64_t)b * p.Nkv + n) * 32 + cp_r0) * H + cp_c * 8;
  const int64_t blk_stride = (int64_t)p.B * p.Nkv * 32 * H;
  // mask values can be read two at a time when every row of the mask starts on a 4-byte boundary
  const bool am_pairs = p.am && (p.Spad & 1) == 0 && (reinterpret_cast<uintptr_t>(p.am) & 3) == 0;
  auto load_block = [&](int blk, int stage) {
    const uint32_t dst = cp_dst0 + (uint32_t)stage * STAGE;
    const uint16_t* ks = (p.kpages ? reinterpret_cast<const uint16_t*>(p.kpages[blk]) : p.kc + (int64_t)blk * blk_stride) + cp_src0;
    const uint16_t* vs = (p.vpages ? reinterpret_cast<const uint16_t*>(p.vpages[blk]) : p.vc + (int64_t)blk * blk_stride) + cp_src0;
    const int live = key_len - blk * 32 - cp_r0;  // rows r0 + k*RSTEP with k*RSTEP < live hold cached tokens
#pragma unroll
    for (int k = 0; k < 32 / RSTEP; k++) {
      const bool valid = k * RSTEP < live;  // slots past the cached length may hold anything: zero-filled
      cp_async_16(dst + k * RSTEP * PB, ks + k * RSTEP * H, valid);
      cp_async_16(dst + TILE + k * RSTEP * PB, vs + k * RSTEP * H, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto group_sync = [&]() {
    if (MODE == 0) __syncthreads(); else __syncwarp();
  };

  const int first = MODE == 0 ? blk0 : blk0 + warp, step = MODE == 0 ? 1 : WARPS;
  // every round commits exactly one copy group (an empty one when the stream has run out), so "all but the NST-1
  // newest groups are complete" always means "this round's block has landed"
#pragma unroll
  for (int s0 = 0; s0 < NST - 1; s0++) {
    if (first + s0 * step < blk1) load_block(first + s0 * step, s0);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  int it = 0;
  for (int blk = first; blk < blk1; blk += step, it++) {
    const int stage = it % NST;
    if (blk + (NST - 1) * step < blk1) load_block(blk + (NST - 1) * step, (it + NST - 1) % NST);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    if (NST == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
    else asm volatile("cp.async.wait_group 2;" ::: "memory");
    group_sync();
    if (blk * 32 < warp_kmax) {
      const uint32_t sk = sbase + (uint32_t)stage * STAGE, sv = sk + TILE;
      // ---- S = Q.K^T for 32 keys: four n-tiles of 8 keys
      float sc[4][4];
#pragma unroll
      for (int i = 0; i < 4; i++) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < KK; kk += 2) {
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
          uint32_t kf[4];  // keys nt*8..+7: h [kk*16, +8), [kk*16+8, +16), [(kk+1)*16, +8), [(kk+1)*16+8, +16)
          ldmatrix_x4(kf, sk + (nt * 8 + (lane & 7)) * PB + (kk * 16 + (lane >> 3) * 8) * 2);
          mma_bf16_16816(sc[nt], qf[kk], kf[0], kf[1]);
          mma_bf16_16816(sc[nt], qf[kk + 1], kf[2], kf[3]);
        }
      }
      // ---- scale, masks, running max
      float bm[2] = {-INFINITY, -INFINITY};
      const int sq_a = (row0 + g) / p.R, sq_b = (row0 + g + 8) / p.R;
      const int kbase = blk * 32 + 2 * t;  // this thread's keys: kbase + 8*nt + {0, 1}
      // a block wholly inside the cached length, the causal limit of every row of the warp and the mask needs no per-key tests
      const bool plain = blk * 32 + 31 < key_len && (!p.causal || blk * 32 + 31 <= offset + row0 / p.R) && (!p.am || (blk * 32 + 31 < p.Spad && am_pairs));
      if (plain) {
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
          float m0 = 0.0f, m1 = 0.0f;
          if (p.am) {  // two consecutive bf16 mask values in one load (kbase is even)
            const uint32_t mw = *reinterpret_cast<const uint32_t*>(p.am + (int64_t)b * p.Spad + kbase + 8 * nt);
            m0 = bf16_bits_to_f32((uint16_t)(mw & 0xffff));
            m1 = bf16_bits_to_f32((uint16_t)(mw >> 16));
          }
          sc[nt][0] = fmaf(sc[nt][0], p.scale, m0);
          sc[nt][1] = fmaf(sc[nt][1], p.scale, m1);
          sc[nt][2] = fmaf(sc[nt][2], p.scale, m0);
          sc[nt][3] = fmaf(sc[nt][3], p.scale, m1);
          bm[0] = fmaxf(bm[0], fmaxf(sc[nt][0], sc[nt][1]));
          bm[1] = fmaxf(bm[1], fmaxf(sc[nt][2], sc[nt][3]));
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const int key = kbase + nt * 8 + e;
            const float madd = (p.am && key < p.Spad) ? bf16_bits_to_f32(p.am[(int64_t)b * p.Spad + key]) : 0.0f;
            const bool in = key < key_len;
            const bool va = in && (!p.causal || key <= offset + sq_a);
            const bool vb = in && (!p.causal || key <= offset + sq_b);
            sc[nt][e] = va ? fmaf(sc[nt][e], p.scale, madd) : -INFINITY;
            sc[nt][2 + e] = vb ? fmaf(sc[nt][2 + e], p.scale, madd) : -INFINITY;
            bm[0] = fmaxf(bm[0], sc[nt][e]);
            bm[1] = fmaxf(bm[1], sc[nt][2 + e]);
          }
        }
      }
      float alpha[2];
#pragma unroll
      for (int h = 0; h < 2; h++) {
        bm[h] = fmaxf(bm[h], __shfl_xor_sync(0xffffffffu, bm[h], 1));
        bm[h] = fmaxf(bm[h], __shfl_xor_sync(0xffffffffu, bm[h], 2));
        const float mn = fmaxf(m_run[h], bm[h]);
        alpha[h] = (mn == -INFINITY) ? 1.0f : __expf(m_run[h] - mn);
        m_run[h] = mn;
        l_run[h] *= alpha[h];
      }
      // ---- P = exp(S - max), packed to bf16 A fragments; row sums
      uint32_t pf[2][4];
#pragma unroll
      for (int nt = 0; nt < 4; nt++) {
        float e0 = (m_run[0] == -INFINITY) ? 0.0f : __expf(sc[nt][0] - m_run[0]);
        float e1 = (m_run[0] == -INFINITY) ? 0.0f : __expf(sc[nt][1] - m_run[0]);
        float e2 = (m_run[1] == -INFINITY) ? 0.0f : __expf(sc[nt][2] - m_run[1]);
        float e3 = (m_run[1] == -INFINITY) ? 0.0f : __expf(sc[nt][3] - m_run[1]);
        l_run[0] += e0 + e1;
        l_run[1] += e2 + e3;
        pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(e0, e1);
        pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(e2, e3);
      }
      // ---- O = O * alpha + P.V
#pragma unroll
      for (int i = 0; i < NT; i++) {
        o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
        o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
      }
#pragma unroll
      for (int j = 0; j < 2; j++) {
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
          uint32_t vf[4];  // keys j*16..+7 and +8..+15 for h tiles nt and nt+1
          ldmatrix_x4_trans(vf, sv + (j * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * PB + ((nt + (lane >> 4)) * 8) * 2);
          mma_bf16_16816(o[nt], pf[j], vf[0], vf[1]);
          mma_bf16_16816(o[nt + 1], pf[j], vf[2], vf[3]);
        }
      }
    }
    group_sync();  // the stage is rewritten by the copy issued at the top of the next round
  }

  // row sums over the four threads of a row
#pragma unroll
  for (int h = 0; h < 2; h++) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }

  if (MODE == 0) {
    // every warp finishes its own rows (no KV split in this mode)
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int row = row0 + g + 8 * h;
      if (row >= rows_total) continue;
      const float inv = 1.0f / l_run[h];
      uint16_t* dst = p.out + attn_out_index(p, bn, row, H);
#pragma unroll
      for (int i = 0; i < NT; i++)
        *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) = pack_bf16x2(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
    }
    return;
  }

  // MODE 1: merge the warps through shared memory (the KV stages are free now)
  __syncthreads();
  float* red_o = reinterpret_cast<float*>(attn_smem);  // [warp][16][H]
  if (t == 0) {
    red_m[warp][g] = m_run[0]; red_m[warp][g + 8] = m_run[1];
    red_l[warp][g] = l_run[0]; red_l[warp][g + 8] = l_run[1];
  }
#pragma unroll
  for (int i = 0; i < NT; i++) {
    float* ra = red_o + ((size_t)warp * kAttnRows + g) * H + i * 8 + 2 * t;
    float* rb = red_o + ((size_t)warp * kAttnRows + g + 8) * H + i * 8 + 2 * t;
    ra[0] = o[i][0]; ra[1] = o[i][1];
    rb[0] = o[i][2]; rb[1] = o[i][3];
  }
  __syncthreads();
  const int rows = min(kAttnRows, rows_total - cta_row0);
  for (int i = threadIdx.x; i < rows * H; i += blockDim.x) {
    const int r = i / H, h = i % H;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; w++) mm = fmaxf(mm, red_m[w][r]);
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < WARPS; w++) {
      const float f = (red_m[w][r] == -INFINITY) ? 0.0f : __expf(red_m[w][r] - mm);
      ll += red_l[w][r] * f;
      oo += red_o[((size_t)w * kAttnRows + r) * H + h] * f;
    }
    if (p.splits == 1) {
      p.out[attn_out_index(p, bn, cta_row0 + r, H) + h] = f32_to_bf16_bits(oo / ll);
    } else {
      float* dst = p.part + ((((int64_t)bn * p.chunks + chunk) * p.splits + split) * kAttnRows + r) * (H + 2);
      __stcg(dst + h, oo);
      if (h == 0) { __stcg(dst + H, mm); __stcg(dst + H + 1, ll); }
    }
  }
  if (p.splits == 1) return;
  // The split that arrives last merges all of them (no second kernel behind a grid boundary).
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(&p.counters[bn * p.chunks + chunk], 1u);
    is_last = prev == (unsigned)p.splits - 1;
    if (is_last) p.counters[bn * p.chunks + chunk] = 0;  // ready for the next call
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < rows * H; i += blockDim.x) {
    const int r = i / H, h = i % H;
    const float* base = p.part + (((int64_t)bn * p.chunks + chunk) * p.splits * kAttnRows + r) * (H + 2);
    float mm = -INFINITY;
    for (int s2 = 0; s2 < p.splits; s2++) mm = fmaxf(mm, __ldcg(base + (int64_t)s2 * kAttnRows * (H + 2) + H));
    float ll = 0.0f, oo = 0.0f;
    for (int s2 = 0; s2 < p.splits; s2++) {
      const float* ps = base + (int64_t)s2 * kAttnRows * (H + 2);
      const float pm = __ldcg(ps + H);
      const float f = (pm == -INFINITY) ? 0.0f : __expf(pm - mm);
      ll += __ldcg(ps + H + 1) * f;
      oo += __ldcg(ps + h) * f;
    }
    p.out[attn_out_index(p, bn, cta_row0 + r, H) + h] = f32_to_bf16_bits(oo / ll);
  }
}

// ---------------------------------------------------------------- mask helper
// TppCache::align_and_invert_mask (src/csrc/llm/attn.h:310-322): [B][S] of 0/1 -> [B][Spad] additive, padding masked.
__global__ void invert_mask_kernel(const uint16_t* __restrict__ mask, int B, int S, int Spad, uint16_t minval,
                                   uint16_t* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)B * Spad) return;
  int s = (int)(idx % Spad), b = (int)(idx / Spad);
  uint16_t v = minval;
  if (s < S && bf16_bits_to_f32(mask[(int64_t)b * S + s]) > 0.0f) v = 0;
  out[idx] = v;
}

// ---------------------------------------------------------------- greedy sampling
// Index of the largest value of every row of x[rows][n] (bf16), the first one among equals and NaN above everything, as
// torch.argmax over the last dimension returns it. One CTA per row: the head's logits of a decode step are a few
// rows of ~10^5 values, read once with 16-byte loads.
constexpr int kArgmaxThreads = 1024;
__device__ __forceinline__ bool argmax_better(float v, long long i, float bv, long long bi) {
  const bool vn = v != v, bn = bv != bv;
  if (vn != bn) return vn;
  if (!vn && v != bv) return v > bv;
  return i < bi;
}
__global__ void __launch_bounds__(kArgmaxThreads) argmax_rows_kernel(const uint16_t* __restrict__ x, long long n, long long* __restrict__ out) {
  __shared__ float sv[kArgmaxThreads / 32];
  __shared__ long long si[kArgmaxThreads / 32];
  pdl_trigger();
  pdl_wait();
  const uint16_t* row = x + (size_t)blockIdx.x * n;
  float bv = -INFINITY;
  long long bi = 0x7fffffffffffffffLL;
  // the row starts on an 8-element boundary when both the base and n allow 16-byte loads
  const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
  const long long nv = vec ? n / 8 : 0;
#pragma unroll 4
  for (long long i = threadIdx.x; i < nv; i += kArgmaxThreads) {
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(row) + i);
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float a = bf16_bits_to_f32((uint16_t)(ww[j] & 0xffff)), b = bf16_bits_to_f32((uint16_t)(ww[j] >> 16));
      if (argmax_better(a, i * 8 + 2 * j, bv, bi)) { bv = a; bi = i * 8 + 2 * j; }
      if (argmax_better(b, i * 8 + 2 * j + 1, bv, bi)) { bv = b; bi = i * 8 + 2 * j + 1; }
    }
  }
  for (long long i = nv * 8 + threadIdx.x; i < n; i += kArgmaxThreads) {
    const float a = bf16_bits_to_f32(row[i]);
    if (argmax_better(a, i, bv, bi)) { bv = a; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (argmax_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    bv = sv[threadIdx.x]; bi = si[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (argmax_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = bi;
  }
}

}  // namespace tpx

using namespace tpx;

extern "C" int tpx_argmax_bf16(const uint16_t* x, int64_t rows, int64_t n, int64_t* out, void* stream) {
  TPX_REQUIRE(rows >= 0 && n > 0, TPX_ERR_ARG, "argmax: bad shape");
  if (rows == 0) return TPX_OK;
  TPX_REQUIRE(x && out, TPX_ERR_ARG, "argmax: null pointer");
  TPX_CUDA_OK(launch_pdl(argmax_rows_kernel, dim3((unsigned)rows), dim3(kArgmaxThreads), 0, (cudaStream_t)stream, x, (long long)n,
                         reinterpret_cast<long long*>(out)));
  return TPX_OK;
}

extern "C" int tpx_rmsnorm(const uint16_t* x, const void* gamma, int gamma_is_f32, float eps, int64_t rows, int64_t D,
                           uint16_t* y, void* stream) {
  TPX_REQUIRE(rows >= 0 && D > 0 && D % 8 == 0, TPX_ERR_ARG, "rmsnorm: D must be a positive multiple of 8 (D=%ld)", (long)D);
  if (rows == 0) return TPX_OK;  // an empty tensor has no storage: nothing to check, nothing to do
  TPX_REQUIRE(x && gamma && y, TPX_ERR_ARG, "rmsnorm: null pointer");
  const bool aligned = (((uintptr_t)x | (uintptr_t)y | (uintptr_t)gamma) & 15) == 0;
  if (rows <= 2048 && D <= kNormThreads * kNormVecs * 8 && aligned)
    TPX_CUDA_OK(launch_pdl(rmsnorm_row_kernel, dim3((unsigned)rows), dim3(kNormThreads), 0, (cudaStream_t)stream, x, gamma, gamma_is_f32,
                           eps, (int)D, y));
  else
    TPX_CUDA_OK(launch_pdl(rmsnorm_kernel, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, (cudaStream_t)stream, x, gamma, gamma_is_f32, eps,
                           rows, (int)D, y));
  return TPX_OK;
}

extern "C" int tpx_layernorm(const uint16_t* x, const void* gamma, const void* beta, int params_are_f32, float eps, int64_t rows,
                             int64_t D, uint16_t* y, void* stream) {
  TPX_REQUIRE(rows >= 0 && D > 0 && D % 8 == 0, TPX_ERR_ARG, "layernorm: D must be a positive multiple of 8 (D=%ld)", (long)D);
  if (rows == 0) return TPX_OK;
  TPX_REQUIRE(x && gamma && beta && y, TPX_ERR_ARG, "layernorm: null pointer");
  TPX_REQUIRE((((uintptr_t)x | (uintptr_t)y) & 15) == 0, TPX_ERR_ARG, "layernorm: x and y must be 16-byte aligned");
  TPX_CUDA_OK(launch_pdl(layernorm_kernel, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, (cudaStream_t)stream, x, gamma, beta,
                         params_are_f32, eps, rows, (int)D, y));
  return TPX_OK;
}

static int rope_kv_update_impl(const uint16_t* qkv, const float* ep, const int64_t* pos, int64_t B, int64_t S, int64_t Nq,
                               int64_t Nkv, int64_t H, int64_t MP, int64_t HR, int64_t Bpos, int64_t offset,
                               int64_t capacity, const int32_t* dev_len, uint16_t* q_out, uint16_t* kc, uint16_t* vc,
                               const uint64_t* kpages, const uint64_t* vpages, void* stream) {
  if (S == 0 && B > 0) return TPX_OK;  // nothing to rotate or append
  TPX_REQUIRE(qkv && ep && pos && q_out && ((kc && vc) || (kpages && vpages)), TPX_ERR_ARG, "rope_kv_update: null pointer");
  TPX_REQUIRE(B > 0 && S >= 0 && Nq > 0 && Nkv > 0 && Nq % Nkv == 0 && H % 2 == 0, TPX_ERR_ARG,
              "rope_kv_update: bad shape");
  TPX_REQUIRE(HR == H, TPX_ERR_UNSUPPORTED, "rope_kv_update: rotary width %ld != head dim %ld (partial rotary is not built)", (long)HR, (long)H);
  TPX_REQUIRE(Bpos == 1 || Bpos == B, TPX_ERR_ARG, "position_ids shape not compatible");
  if (!dev_len)
    TPX_REQUIRE(offset >= 0 && offset + S <= capacity, TPX_ERR_ARG, "rope_kv_update: cache capacity %ld is short of %ld tokens",
                (long)capacity, (long)(offset + S));
  if (S == 0) return TPX_OK;
  const bool aligned = (((uintptr_t)qkv | (uintptr_t)ep | (uintptr_t)q_out | (uintptr_t)kc | (uintptr_t)vc) & 15) == 0;
  if (H % 16 == 0 && aligned) {  // pages are whole [B][Nkv][32][H] slabs of an aligned allocation
    int64_t total8 = B * S * (Nq + 2 * Nkv) * (H / 16);
    TPX_CUDA_OK(launch_pdl(rope_kv_v8_kernel, dim3((unsigned)((total8 + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, qkv, ep, pos, (int)B,
                           (int)S, (int)Nq, (int)Nkv, (int)H, (int)MP, (int)HR, (int)Bpos, offset, dev_len, capacity, q_out, kc, vc, kpages, vpages));
    return TPX_OK;
  }
  int64_t total = B * S * (Nq + 2 * Nkv) * (H / 2);
  TPX_CUDA_OK(launch_pdl(rope_kv_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, qkv, ep, pos, (int)B,
                         (int)S, (int)Nq, (int)Nkv, (int)H, (int)MP, (int)HR, (int)Bpos, offset, dev_len, capacity, q_out, kc, vc, kpages, vpages));
  return TPX_OK;
}

extern "C" int tpx_rope_kv_update_gptj(const uint16_t* qkv, const float* ep, const int64_t* pos, int64_t B, int64_t S, int64_t Nq,
                                       int64_t Nkv, int64_t H, int64_t MP, int64_t HR, int64_t Bpos, int64_t offset, int64_t capacity,
                                       const int32_t* dev_len, uint16_t* q_out, uint16_t* kc, uint16_t* vc, const uint64_t* k_pages,
                                       const uint64_t* v_pages, void* stream) {
  if (S == 0 && B > 0) return TPX_OK;
  TPX_REQUIRE(qkv && ep && pos && q_out && ((kc && vc) || (k_pages && v_pages)), TPX_ERR_ARG, "rope_kv_update_gptj: null pointer");
  TPX_REQUIRE(B > 0 && S >= 0 && Nq > 0 && Nkv > 0 && Nq % Nkv == 0 && H % 2 == 0 && HR % 2 == 0 && HR >= 0 && HR <= H, TPX_ERR_ARG,
              "rope_kv_update_gptj: bad shape");
  TPX_REQUIRE(Bpos == 1 || Bpos == B, TPX_ERR_ARG, "position_ids shape not compatible");
  if (!dev_len)
    TPX_REQUIRE(offset >= 0 && offset + S <= capacity, TPX_ERR_ARG, "rope_kv_update_gptj: cache capacity %ld is short of %ld tokens",
                (long)capacity, (long)(offset + S));
  if (S == 0) return TPX_OK;
  const int64_t total = B * S * (Nq + 2 * Nkv) * (H / 2);
  TPX_CUDA_OK(launch_pdl(rope_kv_gptj_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, qkv, ep, pos, (int)B,
                         (int)S, (int)Nq, (int)Nkv, (int)H, (int)MP, (int)HR, (int)Bpos, offset, dev_len, capacity, q_out, kc, vc, k_pages,
                         v_pages));
  return TPX_OK;
}

extern "C" int tpx_rope_kv_update(const uint16_t* qkv, const float* ep, const int64_t* pos, int64_t B, int64_t S, int64_t Nq,
                                  int64_t Nkv, int64_t H, int64_t MP, int64_t HR, int64_t Bpos, int64_t offset,
                                  int64_t capacity, const int32_t* dev_len, uint16_t* q_out, uint16_t* kc, uint16_t* vc, void* stream) {
  return rope_kv_update_impl(qkv, ep, pos, B, S, Nq, Nkv, H, MP, HR, Bpos, offset, capacity, dev_len, q_out, kc, vc, nullptr, nullptr, stream);
}

extern "C" int tpx_rope_kv_update_paged(const uint16_t* qkv, const float* ep, const int64_t* pos, int64_t B, int64_t S, int64_t Nq,
                                        int64_t Nkv, int64_t H, int64_t MP, int64_t HR, int64_t Bpos, int64_t offset,
                                        int64_t capacity, const int32_t* dev_len, uint16_t* q_out, const uint64_t* k_pages,
                                        const uint64_t* v_pages, void* stream) {
  return rope_kv_update_impl(qkv, ep, pos, B, S, Nq, Nkv, H, MP, HR, Bpos, offset, capacity, dev_len, q_out, nullptr, nullptr, k_pages, v_pages, stream);
}

// More than 16 query rows: 64 rows per CTA, no KV split. Up to 16 rows (decoding): one CTA row tile and the KV range
// cut into the number of splits that minimises waves x (blocks per warp + fixed cost per CTA). One CTA is resident per
// SM (its copy stages take most of the shared memory), so a grid a little over a multiple of the SM count pays for a
// whole extra wave; the fixed cost (first copy's latency, query load, merge) is worth about two blocks, three when
// partials go through global memory. TPX_ATTN_SPLITS overrides the choice.
static int attn_plan(int64_t B, int64_t Nkv, int64_t Sq, int64_t R, int64_t H, int64_t key_len, int* chunks, int* splits) {
  const int64_t rows = Sq * R;
  if (rows > kAttnRows || H > 128) {  // head size 256 (GPT-J): the four warps of a CTA share one KV stream at every row count
    *chunks = (int)((rows + 63) / 64);
    *splits = 1;
    return 0;
  }
  *chunks = 1;
  const int64_t ctas = B * Nkv;
  const int nblocks = (int)((key_len + 31) / 32);
  const int sms = sm_count();
  const int forced = knobs().attn_splits;
  int best = 1;
  if (forced > 0) {
    best = forced < 64 ? forced : 64;
    while (best > 1 && nblocks / best < 1) best--;
  } else {
    double best_cost = 1e30;
    for (int s = 1; s <= 64; s++) {
      if (s > 1 && nblocks / s < kDecWarps) break;  // every warp of every split keeps a block
      const int64_t waves = (ctas * s + sms - 1) / sms;
      const int per_warp = ((nblocks + s - 1) / s + kDecWarps - 1) / kDecWarps;
      const double cost = (double)waves * (per_warp + (s > 1 ? 3 : 2));
      if (cost < best_cost * 0.97) { best_cost = cost; best = s; }  // ties go to fewer splits
    }
  }
  *splits = best;
  return 0;
}

template <int H, int MODE>
static int attn_launch(const AttnParams& p, dim3 grid, cudaStream_t st) {
  constexpr int STAGE = 2 * 32 * (H * 2 + 16);
  constexpr int WARPS = MODE == 0 ? kAttnWarps : kDecWarps;
  constexpr size_t smem = MODE == 0 ? 2 * STAGE : (size_t)WARPS * 2 * STAGE;  // two stages per stream, as in the kernel
  static_assert(MODE == 0 || smem >= (size_t)WARPS * kAttnRows * H * sizeof(float), "merge area");
  static_assert(smem <= 227 * 1024, "shared memory");
  static bool opted[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || !opted[dev]) {
    TPX_CUDA_OK(cudaFuncSetAttribute(attn_mma_kernel<H, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev >= 0 && dev < 16) opted[dev] = true;
  }
  TPX_CUDA_OK(launch_pdl(attn_mma_kernel<H, MODE>, grid, dim3(WARPS * 32), smem, st, p));
  return TPX_OK;
}

static size_t attn_counter_bytes(int64_t B, int64_t Nkv, int chunks) {
  return ((size_t)B * Nkv * chunks * sizeof(unsigned) + 255) & ~(size_t)255;
}

extern "C" size_t tpx_attention_scratch_bytes(int64_t B, int64_t Nkv, int64_t Sq, int64_t R, int64_t H, int64_t key_len) {
  int chunks, splits;
  attn_plan(B, Nkv, Sq, R, H, key_len, &chunks, &splits);
  if (splits == 1) return 0;
  return attn_counter_bytes(B, Nkv, chunks) + (size_t)B * Nkv * chunks * splits * kAttnRows * (H + 2) * sizeof(float);
}

static int attention_impl(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, const uint64_t* kpages, const uint64_t* vpages,
                          const uint16_t* am, int64_t B, int64_t Nkv, int64_t Sq, int64_t R, int64_t H, int64_t key_len, int64_t Spad, int causal,
                          int out_bsnrh, const int32_t* dev_len, uint16_t* out, void* scratch, size_t scratch_bytes, void* stream) {
  if (Sq == 0 && B > 0 && Nkv > 0 && R > 0) return TPX_OK;  // no queries
  TPX_REQUIRE(q && ((kc && vc) || (kpages && vpages)) && out, TPX_ERR_ARG, "attention: null pointer");
  TPX_REQUIRE(B > 0 && Nkv > 0 && Sq >= 0 && R > 0 && key_len >= Sq, TPX_ERR_ARG, "attention: bad shape");
  TPX_REQUIRE(H == 64 || H == 128 || H == 256, TPX_ERR_UNSUPPORTED, "attention: head dim %ld not supported (64, 128 or 256)", (long)H);
  TPX_REQUIRE(!am || Spad >= key_len, TPX_ERR_ARG, "attention: mask of %ld keys is shorter than the cache (%ld)", (long)Spad, (long)key_len);
  if (Sq == 0) return TPX_OK;
  AttnParams p;
  p.q = q; p.kc = kc; p.vc = vc; p.kpages = kpages; p.vpages = vpages; p.am = am; p.out = out; p.part = nullptr; p.counters = nullptr;
  p.B = (int)B; p.Nkv = (int)Nkv; p.Sq = (int)Sq; p.R = (int)R; p.H = (int)H;
  p.key_len = (int)key_len; p.Spad = (int)Spad; p.causal = causal; p.out_bsnrh = out_bsnrh; p.dev_len = dev_len;
  attn_plan(B, Nkv, Sq, R, H, key_len, &p.chunks, &p.splits);
  p.scale = 1.0f / sqrtf((float)H);
  if (p.splits > 1) {
    size_t need = tpx_attention_scratch_bytes(B, Nkv, Sq, R, H, key_len);
    TPX_REQUIRE(scratch && scratch_bytes >= need, TPX_ERR_SCRATCH, "attention: scratch of %zu bytes needed, %zu given", need, scratch_bytes);
    TPX_REQUIRE(((uintptr_t)scratch & 15) == 0, TPX_ERR_ARG, "attention: scratch must be 16-byte aligned");
    p.counters = reinterpret_cast<unsigned*>(scratch);
    p.part = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(scratch) + attn_counter_bytes(B, Nkv, p.chunks));
  }
  if (!kpages && attn_tc_serves(Sq * R, H)) return attn_tc_launch(p, (cudaStream_t)stream);  // prefill on a contiguous cache: tcgen05 + TMA kernel
  dim3 grid((unsigned)(B * Nkv), (unsigned)p.chunks, (unsigned)p.splits);
  TPX_REQUIRE(p.chunks <= 65535, TPX_ERR_UNSUPPORTED, "attention: too many query rows in one call");
  cudaStream_t st = (cudaStream_t)stream;
  const bool decode = Sq * R <= kAttnRows;
  int rc;
  if (H == 256) rc = attn_launch<256, 0>(p, grid, st);  // 66 KB of KV stages per stream: one stream per CTA
  else if (H == 128) rc = decode ? attn_launch<128, 1>(p, grid, st) : attn_launch<128, 0>(p, grid, st);
  else rc = decode ? attn_launch<64, 1>(p, grid, st) : attn_launch<64, 0>(p, grid, st);
  if (rc) return rc;
  return TPX_OK;
}

extern "C" int tpx_attention(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, const uint16_t* am, int64_t B,
                             int64_t Nkv, int64_t Sq, int64_t R, int64_t H, int64_t key_len, int64_t Spad, int causal,
                             int out_bsnrh, const int32_t* dev_len, uint16_t* out, void* scratch, size_t scratch_bytes, void* stream) {
  return attention_impl(q, kc, vc, nullptr, nullptr, am, B, Nkv, Sq, R, H, key_len, Spad, causal, out_bsnrh, dev_len, out, scratch, scratch_bytes, stream);
}

extern "C" int tpx_attention_paged(const uint16_t* q, const uint64_t* k_pages, const uint64_t* v_pages, const uint16_t* am, int64_t B,
                                   int64_t Nkv, int64_t Sq, int64_t R, int64_t H, int64_t key_len, int64_t Spad, int causal,
                                   int out_bsnrh, const int32_t* dev_len, uint16_t* out, void* scratch, size_t scratch_bytes, void* stream) {
  return attention_impl(q, nullptr, nullptr, k_pages, v_pages, am, B, Nkv, Sq, R, H, key_len, Spad, causal, out_bsnrh, dev_len, out, scratch,
                        scratch_bytes, stream);
}

extern "C" int tpx_align_and_invert_mask(const uint16_t* mask, int64_t B, int64_t S, int64_t Spad, uint16_t min_bits,
                                         uint16_t* out, void* stream) {
  TPX_REQUIRE(mask && out, TPX_ERR_ARG, "align_and_invert_mask: null pointer");
  TPX_REQUIRE(Spad >= S && Spad % 32 == 0, TPX_ERR_ARG, "align_and_invert_mask: padded length must be a multiple of 32 >= S");
  int64_t total = B * Spad;
  if (total == 0) return TPX_OK;
  invert_mask_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(mask, (int)B, (int)S, (int)Spad, min_bits, out);
  TPX_LAUNCH_OK();
  return TPX_OK;
}
