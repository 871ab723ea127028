"""Greedy generation benchmark on a random-weight Llama: the counterpart of the reference's examples/llm/run_generation.py
(its flags --weight-dtype, --input-tokens, --max-new-tokens, --batch-size, --num-iter, --num-warmup keep their meaning;
examples/llm/run_generation.py:36-131).  There is no checkpoint or tokenizer here: weights are seeded random values of the
named architecture and the prompt is random token ids, so only the timing is meaningful.

    python -m tpp_pytorch_extension_b200.examples.run_generation --model llama3-8b --weight-dtype mxfp4 \
        --batch-size 1 --input-tokens 1024 --max-new-tokens 128

Prints one JSON line: first-token (prefill) latency, per-token decode latency and decode tokens/s.
Under torchrun every rank holds its shard of each layer (tensor parallel) and rank 0 prints.
"""
import argparse
import json
import os
import time

import torch

from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
from tpp_pytorch_extension_b200._C import _fused_llm_infer as fused_llm_cpp

from tpp_pytorch_extension_b200.llm import fused_gptj_infer as FG
from tpp_pytorch_extension_b200.llm import fused_opt_infer as FO

MODELS = {"llama2-7b": FL.LLAMA2_7B, "llama3-8b": FL.LLAMA3_8B, "llama2-70b": FL.LLAMA2_70B,
          "opt-6.7b": FO.OPTShape(32, 4096, 32, 16384, 50272), "opt-30b": FO.OPTShape(48, 7168, 56, 28672, 50272),
          "gptj-6b": FG.GPTJShape(28, 4096, 16, 16384, 50400, 64)}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b", choices=sorted(MODELS))
    ap.add_argument("--weight-dtype", default="mxfp4", choices=["mxfp4", "qint8", "qint2", "bfloat16", "bfloat8", "hfloat8"])
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--input-tokens", type=int, default=1024)
    ap.add_argument("--max-new-tokens", type=int, default=128)
    ap.add_argument("--num-iter", type=int, default=3)
    ap.add_argument("--num-warmup", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0, help="keep only this many decoder layers (0 = all)")
    ap.add_argument("--no-graph", action="store_true", help="decode eagerly instead of replaying a CUDA graph")
    ap.add_argument("--quantize-lm-head", action="store_true", help="quantize the lm_head like the decoder linears (bf16 otherwise)")
    ap.add_argument("--save-sharded-model", action="store_true", help="write this rank's quantized, packed shard to ./sharded_model/r<rank>_<size>/model.pt")
    ap.add_argument("--load-sharded-model", action="store_true", help="read the shard written by --save-sharded-model instead of building the model")
    a = ap.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        fused_llm_cpp.set_pg(dist.group.WORLD)
    shape = MODELS[a.model]
    if a.layers:
        import dataclasses
        shape = dataclasses.replace(shape, num_hidden_layers=a.layers)
    wd = {"bfloat16": "bf16"}.get(a.weight_dtype, a.weight_dtype)
    from tpp_pytorch_extension_b200.llm import llm_common
    if a.load_sharded_model:
        model = llm_common.load_sharded_model()
    elif isinstance(shape, FO.OPTShape):
        model = FO.build_random_opt(shape, wd, "cuda")
    elif isinstance(shape, FG.GPTJShape):
        model = FG.build_random_gptj(shape, wd, "cuda")
    else:
        model = FL.build_random_llama(shape, wd, "cuda", max_positions=a.input_tokens + a.max_new_tokens + 8,
                                      quantize_lm_head=a.quantize_lm_head and wd != "bf16")
    if a.save_sharded_model:
        llm_common.save_sharded_model(model)
    g = torch.Generator(device="cpu").manual_seed(1234)
    ids = torch.randint(0, shape.vocab_size, (a.batch_size, a.input_tokens), generator=g).cuda()

    def run(new):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = model.generate(ids, new, use_graph=not a.no_graph)
        torch.cuda.synchronize()
        return time.perf_counter() - t0, out

    first, total = [], []
    for it in range(a.num_warmup + a.num_iter):
        t1, _ = run(1)
        tn, out = run(a.max_new_tokens)
        if it >= a.num_warmup:
            first.append(t1)
            total.append(tn)
    t1 = sorted(first)[len(first) // 2]
    tn = sorted(total)[len(total) // 2]
    steps = max(a.max_new_tokens - 1, 1)
    per_tok = (tn - t1) / steps
    if rank == 0:
        print(json.dumps({
            "model": a.model, "weight_dtype": a.weight_dtype, "tp": world, "layers": shape.num_hidden_layers,
            "batch_size": a.batch_size, "input_tokens": a.input_tokens, "max_new_tokens": a.max_new_tokens,
            "graph": not a.no_graph, "first_token_ms": round(t1 * 1e3, 3), "next_token_ms": round(per_tok * 1e3, 4),
            "decode_tokens_per_s": round(a.batch_size / per_tok, 1),
            "prefill_tokens_per_s": round(a.batch_size * a.input_tokens / t1, 1), "data": "synthetic"}))
    if world > 1:
        import gc
        import torch.distributed as dist
        # a CUDA graph that recorded NCCL collectives must be gone before its communicator is destroyed
        model.last_graph = None
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
