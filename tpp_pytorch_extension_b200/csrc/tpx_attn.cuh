// Parameter block shared by the attention kernels (tpx_attn.cu: mma.sync kernel for decoding and short prompts;
// tpx_attn_tc.cu: tcgen05 + TMA kernel for prefill).
#pragma once
#include "tpx_common.cuh"

namespace tpx {

constexpr int kAttnWarps = 4;
// Warps of a decoding CTA (MODE 1): each keeps its own two stages of K and V blocks (17 KB each at head size 128) and
// takes every sixth block of the CTA's split. A warp is bound by its own chain per block (wait, 64 mma.sync, softmax), so
// more warps per SM stream more: six, the most that shared memory holds, against four measured 95 against 103 us at
// batch 64 x 4096 tokens (5.6 TB/s of KV bytes), 28.0 against 29.4 us at batch 16 x 2048.
constexpr int kDecWarps = 6;
constexpr int kAttnRows = 16;

struct AttnParams {
  const uint16_t* q;    // [B][Nkv][Sq][R][H]
  const uint16_t* kc;   // [S1][B][Nkv][32][H]
  const uint16_t* vc;
  const uint64_t* kpages;  // paged cache: device addresses of the 32-token pages [B][Nkv][32][H], one per block (null: kc / vc are
  const uint64_t* vpages;  // one contiguous tensor)
  const uint16_t* am;   // [B][Spad] additive mask or null
  uint16_t* out;        // same shape as q
  float* part;          // [B*Nkv][chunks][splits][16][H + 2]
  unsigned* counters;   // [B*Nkv][chunks] arrivals of the KV splits; zero between calls
  int B, Nkv, Sq, R, H;
  int key_len, Spad, causal;
  int chunks, splits;
  const int* dev_len;   // when set: keys cached before this call; key_len = *dev_len + Sq (key_len above is then the planning maximum)
  int out_bsnrh;        // 0: out laid out like q; 1: out[B][Sq][Nkv][R][H] (rows of the following linear)
  float scale;
};

__device__ __forceinline__ int64_t attn_out_index(const AttnParams& p, int bn, int row, int H) {
  if (!p.out_bsnrh) return ((int64_t)bn * p.Sq * p.R + row) * H;
  const int b = bn / p.Nkv, n = bn % p.Nkv, sq = row / p.R, r = row % p.R;
  return ((((int64_t)b * p.Sq + sq) * p.Nkv + n) * p.R + r) * H;
}


// prefill on the 5th-generation tensor cores (tpx_attn_tc.cu); returns TPX_ERR_UNSUPPORTED when the tensor maps cannot be made
bool attn_tc_serves(int64_t rows, int64_t H);
int attn_tc_launch(const AttnParams& p, cudaStream_t st);

}  // namespace tpx
