"""CPU tests of the tensor-parallel host logic with two gloo ranks: the sharding rule, and that the sharded decoder
layer (column-parallel q/k/v/gate/up, row-parallel o/down, residual pre-scaled by 1/world, all-reduce after each
row-parallel linear) reproduces the single-rank result. The arithmetic is the CPU oracle's; what is under test is the
host-side partitioning in tpp_pytorch_extension_b200.llm."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
        from tpp_pytorch_extension_b200.llm import llm_common as LC
        assert LC.get_rank() == rank and LC.get_size() == world
        rng = np.random.default_rng(11)  # every rank draws the same full weights
        D, Nq, Nkv, H, FF, B, S = 128, 4, 2, 32, 192, 2, 6
        shapes = {"q": (Nq * H, D), "k": (Nkv * H, D), "v": (Nkv * H, D), "o": (D, Nq * H), "gate": (FF, D), "up": (FF, D), "down": (D, FF)}
        W = {k: (rng.standard_normal(s) * 0.05).astype(np.float32) for k, s in shapes.items()}
        W["ln1"] = O.f32_to_bf16(np.ones(D, np.float32))
        W["ln2"] = O.f32_to_bf16(np.ones(D, np.float32))
        hs = O.randn_bf16(rng, (B, S, D))
        ep = O.rope_table(32, H, 1e4)
        pos = np.arange(S, dtype=np.int64)[None]
        mask = O.align_and_invert_mask(np.ones((B, S)))
        full = O.llama_layer(hs, mask, pos, W, O.KVCache(), 0, Nq, Nkv, H, 1e-5, ep)
        # shard exactly as make_layer does
        grp = H * (Nq // Nkv)
        plan = {"q": (0, grp), "k": (0, H), "v": (0, H), "o": (1, grp), "gate": (0, 64), "up": (0, 64), "down": (1, 64)}
        Ws = {k: FL._shard(torch.from_numpy(W[k]), d, b).numpy() for k, (d, b) in plan.items()}
        Ws["ln1"], Ws["ln2"] = W["ln1"], W["ln2"]

        def allreduce(bits):  # fp32 sum of the bf16 payloads, rounded once (what NCCL's bf16 all-reduce approximates)
            t = torch.from_numpy(O.bf16_to_f32(bits).copy())
            dist.all_reduce(t)
            return O.f32_to_bf16(t.numpy())

        nq_l = Ws["q"].shape[0] // H
        nkv_l = Ws["k"].shape[0] // H
        out = O.llama_layer(hs, mask, pos, Ws, O.KVCache(), 0, nq_l, nkv_l, H, 1e-5, ep, world=world, allreduce=allreduce)
        err = O.rel_err(out, full)
        # ShardLinear on a real nn.Linear, uneven split: 3 blocks of 64 over 2 ranks -> 64 / 128
        lin = torch.nn.Linear(16, 192, bias=True)
        LC.ShardLinear(lin, 0, rank, world, 64)
        ok_uneven = lin.split_sizes == [64, 128] and lin.weight.shape[0] == lin.split_sizes[rank] and lin.bias.shape[0] == lin.split_sizes[rank]
        lin2 = torch.nn.Linear(192, 8, bias=True)
        b0 = lin2.bias.data.clone()
        LC.ShardLinear(lin2, 1, rank, world, 64)
        ok_row = lin2.weight.shape[1] == [64, 128][rank] and torch.allclose(lin2.bias.data, b0 / world)
        # fc_plain with parallel_dim 0 (column-parallel, uneven all-gather of the outputs) and 1 (row-parallel, the
        # input split by split_sizes, all-reduce): fc_plain_wrap of the reference, src/csrc/llm/fused_llm_infer.cpp:1514-1566.
        # The single-rank linear underneath is replaced by a CPU one: what is under test is the host logic around it.
        from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
        F.set_pg(dist.group.WORLD)
        g = torch.Generator().manual_seed(5)
        wfull = torch.randn(192, 128, generator=g)
        bfull = torch.randn(192, generator=g)
        xin = torch.randn(3, 128, generator=g)
        real_fc = F.fc_plain
        F.fc_plain = lambda x, w, b=None, parallel_dim=-1, split_sizes=(): torch.nn.functional.linear(x, w, b)
        try:
            split0 = [64, 128]  # 3 blocks of 64 over 2 ranks
            lo = sum(split0[:rank])
            y0 = LC.fc_plain_parallel(xin, wfull[lo:lo + split0[rank]], bfull[lo:lo + split0[rank]], 0, split0)
            ok_gather = torch.allclose(y0, torch.nn.functional.linear(xin, wfull, bfull), atol=1e-5)
            split1 = [64, 64]
            w1 = torch.randn(16, 128, generator=g)
            b1 = torch.randn(16, generator=g)
            y1 = LC.fc_plain_parallel(xin, w1[:, 64 * rank:64 * rank + 64].contiguous(), b1 / world, 1, split1)
            ok_reduce = torch.allclose(y1, torch.nn.functional.linear(xin, w1, b1), atol=1e-4)
        finally:
            F.fc_plain = real_fc
        q.put((rank, err, bool(ok_uneven), bool(ok_row and ok_gather and ok_reduce), None))
        dist.destroy_process_group()
    except Exception as e:  # surface the failure in the parent instead of hanging it
        q.put((rank, None, False, False, repr(e)))


def test_shard_offsets_rule():
    from tpp_pytorch_extension_b200.llm.llm_common import shard_offsets
    assert shard_offsets(4096, 8, 128) == [0, 512, 1024, 1536, 2048, 2560, 3072, 3584, 4096]
    assert shard_offsets(11008, 8, 64) == [0, 1344, 2752, 4096, 5504, 6848, 8256, 9600, 11008]  # uneven: 21/22 blocks
    assert shard_offsets(192, 2, 64) == [0, 64, 192]
    with pytest.raises(AssertionError):
        shard_offsets(100, 2, 64)


def test_two_rank_decoder_layer_matches_single_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, err, ok_uneven, ok_row, exc in res:
        assert exc is None, exc
        assert ok_uneven and ok_row
        assert err <= 2e-2, (rank, err)
