"""Beam search over the fused runner (LlamaRunner.beam_search): the KV cache rows are reordered every step
(TppCache.reorder_cache). Checks: one beam equals greedy decoding; the scores returned for several beams equal the
log-probabilities of the returned sequences recomputed from scratch without a cache (a wrong cache reordering would
break this); beams come best first and are distinct."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _runner(cuda):
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    shape = FL.LlamaShape(2, 256, 4, 2, 512, 320, max_position_embeddings=128)
    return FL.build_random_llama(shape, "mxfp4", cuda, std=0.08)


def test_one_beam_is_greedy(cuda):
    r = _runner(cuda)
    ids = torch.randint(2, 300, (3, 11), generator=torch.Generator().manual_seed(0)).to(cuda)
    want = r.generate(ids, 6, use_graph=False)
    seqs, _ = r.beam_search(ids, 6, num_beams=1)
    assert torch.equal(seqs[:, 0], want)


@pytest.mark.parametrize("beams", [2, 4])
def test_scores_match_recomputed_log_probabilities(cuda, beams):
    r = _runner(cuda)
    B, P, NEW = 2, 9, 5
    ids = torch.randint(2, 300, (B, P), generator=torch.Generator().manual_seed(1)).to(cuda)
    seqs, scores = r.beam_search(ids, NEW, num_beams=beams)
    assert seqs.shape == (B, beams, P + NEW) and scores.shape == (B, beams)
    assert bool((scores[:, :-1] >= scores[:, 1:]).all())
    for b in range(B):
        assert len({tuple(s.tolist()) for s in seqs[b]}) == beams
        assert bool((seqs[b, :, :P] == ids[b]).all())
    r.only_last_logit = False
    try:
        flat = seqs.reshape(B * beams, P + NEW)
        logits, _ = r.forward(flat)  # no cache: every hypothesis from scratch
    finally:
        r.only_last_logit = True
    logp = torch.log_softmax(logits.float(), dim=-1)
    tok_lp = logp[:, P - 1:-1].gather(-1, flat[:, P:].unsqueeze(-1)).squeeze(-1).sum(-1).view(B, beams)
    # bf16 logits computed in a different batch composition: a few hundredths per token at most
    assert float((tok_lp - scores).abs().max()) <= 0.05 * NEW
