// One call per half of a Llama / Qwen2 decoder layer on MXFP4 weights: the sequence of launches of
// LlamaDecoderLayer::_forward (src/csrc/llm/fused_llm_infer.cpp:1195-1286) issued from C, so that a host language
// with an expensive foreign-call path (Python: 15-25 us per call) pays it twice per layer instead of once per kernel.
// The two halves meet where the reference all-reduces under tensor parallelism (:1263-1277): the caller runs its
// collective between them and after the second. Every step is one of the library's own entry points; nothing is
// allocated, all buffers come from the caller.
#include "tpx_common.cuh"
#include "tpx_tc_ptx.cuh"
#include "../../include/tpx_b200.h"

extern "C" int tpx_llama_layer_attention(const TpxLlamaLayer* L, const TpxLlamaLayerIO* io, void* stream) {
  TPX_REQUIRE(L && io, TPX_ERR_ARG, "llama_layer: null argument");
  TPX_REQUIRE(io->x && io->qkv && io->q && io->ctx && io->so, TPX_ERR_ARG, "llama_layer: null activation buffer");
  const int64_t T = io->B * io->S, D = L->D, H = L->H;
  const int64_t nqkv = (L->Nq + 2 * L->Nkv) * H;
  // llama_rms_norm + fused q/k/v (+ bias): the normalised tensor never goes to memory
  int rc = tpx_rmsnorm_qlinear_mxfp4_tc(L->wqkv, L->sfa_qkv, 0, io->x, L->gamma1, L->gamma_is_f32, L->eps, T, nqkv, D, L->bias_qkv,
                                        TPX_ACT_NONE, nullptr, nullptr, 0.0f, io->qkv, io->scratch, io->scratch_bytes, stream);
  if (rc) return rc;
  // rotary embedding, q permute, cache append
  if (io->k_pages)
    rc = tpx_rope_kv_update_paged(io->qkv, L->ep, io->pos, io->B, io->S, L->Nq, L->Nkv, H, L->MP, L->HR, io->Bpos, io->offset, io->capacity,
                                  io->dev_len, io->q, io->k_pages, io->v_pages, stream);
  else
    rc = tpx_rope_kv_update(io->qkv, L->ep, io->pos, io->B, io->S, L->Nq, L->Nkv, H, L->MP, L->HR, io->Bpos, io->offset, io->capacity,
                            io->dev_len, io->q, io->kc, io->vc, stream);
  if (rc) return rc;
  const int64_t key_len = io->dev_len ? io->capacity : io->offset + io->S;
  if (io->k_pages)
    rc = tpx_attention_paged(io->q, io->k_pages, io->v_pages, io->mask, io->B, L->Nkv, io->S, L->Nq / L->Nkv, H, key_len, io->Spad, 1, 1,
                             io->dev_len, io->ctx, io->attn_scratch, io->attn_scratch_bytes, stream);
  else
    rc = tpx_attention(io->q, io->kc, io->vc, io->mask, io->B, L->Nkv, io->S, L->Nq / L->Nkv, H, key_len, io->Spad, 1, 1, io->dev_len,
                       io->ctx, io->attn_scratch, io->attn_scratch_bytes, stream);
  if (rc) return rc;
  // o_proj with the residual pre-scaled by 1 / world
  return tpx_qlinear_mxfp4_tc(L->wo, L->sfa_o, 0, io->ctx, T, D, L->Nq * H, nullptr, TPX_ACT_NONE, nullptr, io->x, L->res_scale, io->so,
                              io->scratch, io->scratch_bytes, stream);
}

extern "C" int tpx_llama_layer_mlp(const TpxLlamaLayer* L, const TpxLlamaLayerIO* io, void* stream) {
  TPX_REQUIRE(L && io, TPX_ERR_ARG, "llama_layer: null argument");
  TPX_REQUIRE(io->so && io->inter && io->out, TPX_ERR_ARG, "llama_layer: null activation buffer");
  const int64_t T = io->B * io->S, D = L->D;
  // With 33 to 64 tokens the gate/up kernel's epilogue also writes its output as the activation terms the down
  // projection reads (io->handoff), when both kernels chosen for these shapes can: one kernel fewer in the chain
  // (Llama-3-8B shape, 1024 cached tokens: 4.53 against 4.63 ms per step at batch 33, 5.20 against 5.30 at batch 48,
  // 5.86 against 5.96 at batch 64). With fewer tokens it loses: the split kernel it
  // saves is short and ran while the down projection's CTAs fetched their first weights, and the packed-fp4 kernel's
  // four epilogue warps pay for the conversion on the critical path (batch 16: 4.52 against 4.06 ms; batch 1: 2.9
  // against 2.76). TPX_HANDOFF_MIN_TOKENS moves the lower bound.
  tpx::TcEmit E = {};
  if (T >= tpx::knobs().handoff_min && T <= 64 && io->handoff) {
    int rc0 = tpx::tc_handoff_plan(T, D, L->FF, io->handoff, io->handoff_bytes, &E);
    if (rc0) return rc0;
    if (E.terms) tpx::tc_set_emit(E);
  }
  // post-attention norm + gate/up pair with SiLU * up
  int rc = tpx_rmsnorm_qlinear_mxfp4_tc(L->wgu, L->sfa_gu, 1, io->so, L->gamma2, L->gamma_is_f32, L->eps, T, L->FF, D, nullptr, TPX_ACT_SILU,
                                        nullptr, nullptr, 0.0f, io->inter, io->scratch, io->scratch_bytes, stream);
  if (rc) return rc;
  // down_proj with the residual
  if (E.terms && tpx::tc_emitted()) tpx::tc_set_pre(E);
  return tpx_qlinear_mxfp4_tc(L->wd, L->sfa_d, 0, io->inter, T, D, L->FF, nullptr, TPX_ACT_NONE, nullptr, io->so, L->res_scale, io->out,
                              io->scratch, io->scratch_bytes, stream);
}
