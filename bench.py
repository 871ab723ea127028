#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

Workload (the MXFP4 sweep configuration of the benchmark): MXFP4 weight-only linears of the Llama-3-8B MLP shape,
W_gate/W_up [14336, 4096] and W_down [4096, 14336], bf16 activations X [M, 4096] for
M in {1, 8, 64, 512, 4096}. One *step* is one pass of the sweep: for every M, the fused
gate/up pair with the SiLU*mul epilogue, then the down projection. The K timed steps are issued shape by shape
(K gate/up launches of M = 1, K down launches of M = 1, K gate/up launches of M = 8, ...) with CUDA events only where the
shape changes: consecutive launches then overlap prologue and tail through programmatic dependent launch as the
kernels of a decode step do (every kernel waits for its predecessor before touching memory); an event recorded
between two launches forbids that overlap and adds about 6 us to each.

Headline `value`: quantized-GEMM HBM GB/s over the decode-shaped part of the sweep (M <= 64):
algorithmic bytes (packed codes + scales + activations in + out) / device time. The prefill part
(M >= 512) is reported as TFLOP/s under `prefill`. Weights rotate over several distinct packed
copies (together larger than L2) so that no launch finds its weights in L2.

`python bench.py --impl reference` times the CPU restatement of the reference's path (the
reference's own libxsmm build is not possible here) on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

D_MODEL, D_FF = 4096, 14336
SWEEP = [1, 8, 64, 512, 4096]
DECODE_MAX_M = 64
# dram__bytes_read.sum + dram__bytes_write.sum of one gate/up launch of the tensor-core kernels, from the ncu captures
# summarised under profiles/ (bytes); None where no capture exists
NCU_TRAFFIC = {1: 63.02e6, 8: 63.02e6, 64: 63.82e6}  # M=1 runs the M=8 kernel instantiation on the same weight bytes
N_COPIES = 6  # distinct packed weight sets: 6 x 93.6 MB = 561 MB >> 126 MB of L2


def _lib_launch_count():
    """The library's own tally of the kernels it has launched (tpx_launch_count)."""
    from tpp_pytorch_extension_b200 import _lib
    fn = _lib.lib().tpx_launch_count
    return lambda: int(fn())


def packed_bytes(N, K):
    return N * K // 2 + N * K // 32


def op_bytes(M, pair):
    """Algorithmic bytes of one launch (weights once, activations in, result out)."""
    if pair:  # gate/up: two weights, X in, H out
        return 2 * packed_bytes(D_FF, D_MODEL) + M * D_MODEL * 2 + M * D_FF * 2
    return packed_bytes(D_MODEL, D_FF) + M * D_FF * 2 + M * D_MODEL * 2


def op_flops(M, pair):
    return (4 if pair else 2) * M * D_FF * D_MODEL


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- CPU arm
def host_threads():
    """The cores this process may use (launchers set OMP_NUM_THREADS=1 for their ranks; the CPU arm undoes that)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_arm(seconds_target=12.0):
    """Times the CPU restatement on a bounded sample: the gate/up pair at every decode-shaped token count of the sweep
    (M = 1, 8, 64) over a slice of 1024 output features (of 14336), on all host threads. GB/s of algorithmic bytes."""
    import numpy as np
    from oracle import oracle as O
    O.lib().orc_set_num_threads(host_threads())
    rng = np.random.default_rng(0)
    Ns = 1024
    wg = O.randn_bf16(rng, (Ns, D_MODEL), 0.02)
    wu = O.randn_bf16(rng, (Ns, D_MODEL), 0.02)
    cg, sg = O.remap_and_quantize_mxfp4(wg)
    cu, su = O.remap_and_quantize_mxfp4(wu)
    threads = O.lib().orc_num_threads()
    total_b, total_t = 0.0, 0.0
    per_m = {}
    ms = [M for M in SWEEP if M <= DECODE_MAX_M]
    for M in ms:
        x = O.randn_bf16(rng, (M, D_MODEL))
        O.qlinear_mxfp4_packed(x, cg, sg, cu, su, act=O.ACT_SILU)  # warm-up
        reps, t0 = 0, time.perf_counter()
        while True:
            O.qlinear_mxfp4_packed(x, cg, sg, cu, su, act=O.ACT_SILU)
            reps += 1
            dt = time.perf_counter() - t0
            if dt > seconds_target / len(ms) or reps >= 200:
                break
        b = reps * (2 * packed_bytes(Ns, D_MODEL) + M * D_MODEL * 2 + M * Ns * 2)
        per_m[M] = b / dt / 1e9
        total_b += b
        total_t += dt
    return {"value": total_b / total_t / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"gate/up pair, M in {tuple(ms)}, a slice of {Ns} of the {D_FF} output features, K = {D_MODEL}, plain-C port "
                      f"(not the reference's libxsmm kernels); "
                      f"per-M GB/s {', '.join(f'M={m}: {v:.2f}' for m, v in per_m.items())}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    vals = []
    for _ in range(max(1, args.warmup) - 1 + 1):
        pass
    per_step = max(2.0, min(20.0, 60.0 / max(1, args.steps)))
    for _ in range(args.steps):
        vals.append(cpu_arm(per_step))
    dt = time.perf_counter() - t0
    v = sum(x["value"] for x in vals) / len(vals)
    cb = dict(vals[-1])
    cb["value"] = v
    line = {"impl": "reference", "metric": "qgemm_hbm_gbs", "value": v, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3 / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x mxfp4 -> fp32 acc",
            "data": "synthetic", "config": workload_config(), "cpu_baseline": cb,
            "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "CPU restatement of the reference path (oracle/tpx_oracle.c): the reference's libxsmm build is not available"}
    print(json.dumps(line))


def workload_config():
    return {"workload": "config 2: MXFP4 weight-only linear sweep, Llama-3-8B MLP shape "
                        "(gate/up [14336x4096] pair with SiLU*mul, down [4096x14336]), M in {1,8,64,512,4096}",
            "metric_scope": f"HBM GB/s over M <= {DECODE_MAX_M}; prefill TFLOP/s over M >= 512 reported under 'prefill'",
            "l2": f"weights rotate over {N_COPIES} distinct packed copies (561 MB > 126 MB L2)",
            "order": "K steps issued shape by shape, events at shape boundaries (launches back to back); the M <= 64 shapes and the M >= 512 shapes in separate timed blocks",
            "parallelism": "replicas (one independent sweep per GPU)"}


# --------------------------------------------------------------------------- GPU arm
def spot_rows(N):
    """Eight runs of 32 consecutive output features spread over [0, N), first and last rows included."""
    import torch
    starts = sorted({int(round(g * (N - 32) / 7 / 32)) * 32 for g in range(8)})
    return torch.cat([torch.arange(s, s + 32) for s in starts])


def parity_spot_check(wset, w_cpu, xs_host, dev):
    """The timed ops once more at M = 8 on the seed-0 weight set, compared with the CPU oracle on 256 sampled output
    features (the oracle quantizes those rows itself): max |y - ref| / max |ref|, bound 2e-2."""
    import numpy as np
    import torch
    from oracle import oracle as O
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F

    def bits(t):
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)

    wg, wu, wd = wset
    x = xs_host[8] if 8 in xs_host else torch.randn(8, D_MODEL, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16)
    h = F.fc_gate_up(x.to(dev), wg, wu)
    y = F.fc_plain(h, wd)
    torch.cuda.synchronize()
    deq = [O.mxfp4_dequant_plain(*O.remap_and_quantize_mxfp4(bits(w))) for w in w_cpu]
    e1 = O.rel_err(bits(h)[:, spot_rows(D_FF).numpy()], O.gate_up(bits(x), deq[0], deq[1]))
    e2 = O.rel_err(bits(y)[:, spot_rows(D_MODEL).numpy()], O.qlinear(bits(h), deq[2]))
    return {"gate_up_rel_err": e1, "down_rel_err": e2, "bound": 2e-2, "ok": bool(e1 <= 2e-2 and e2 <= 2e-2),
            "scope": "M = 8, 256 sampled output features of each op, against the CPU oracle"}


def model_bytes_per_step(shape, batch, context, world, lm_head_bf16=True, wbytes=0.53125):
    """Algorithmic bytes ONE GPU reads per decode step: its shard of the MXFP4 decoder weights (0.53125 B per weight),
    of the bf16 lm_head and of the KV cache (keys and values of `context` tokens per sequence)."""
    D, H = shape.hidden_size, shape.head_dim
    per_layer = (shape.num_attention_heads + 2 * shape.num_key_value_heads) * H * D + D * shape.num_attention_heads * H \
        + 3 * shape.intermediate_size * D
    w = shape.num_hidden_layers * per_layer * wbytes  # MXFP4: 4-bit code + 1/32 scale byte; int8, blocks of 64: 1 + 4/64
    lm = shape.vocab_size * D * (2 if lm_head_bf16 else 0.53125)
    kv = shape.num_hidden_layers * 2 * context * batch * shape.num_key_value_heads * H * 2
    return (w + lm + kv) / world


def model_decode_leg(name, shape, batch, context, steps, dev, world, rank, real_prefill, weight_dtype="mxfp4"):
    """Greedy decode of `steps` tokens per sequence on a random-weight MXFP4 model of the named shape, tensor parallel
    over the `world` ranks (all-reduce after o_proj, down_proj and lm_head), the step replayed as a CUDA graph. The
    context is either prefilled for real (timed) or stands in as a random KV cache of the same shape."""
    import torch
    import torch.distributed as dist
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    t0 = time.perf_counter()
    torch.cuda.empty_cache()
    if weight_dtype == "qint8":
        os.environ["QINT8_BLOCK_SIZE"] = "64"  # the configuration's K-block size (the reference's switch of the same name)
    runner = FL.build_random_llama(shape, weight_dtype, dev, max_positions=context + steps + 16)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    g = torch.Generator(device="cpu").manual_seed(1234)
    out = {"model": name, "layers": shape.num_hidden_layers, "batch": batch, "context": context, "tensor_parallel": world,
           "build_s": round(build_s, 1)}
    mask = torch.ones((batch, context), dtype=torch.int64, device=dev)
    if real_prefill:
        ids = torch.randint(0, shape.vocab_size, (batch, context), generator=g).to(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        runner.forward(ids[:, :64])  # warm-up of the prefill kernels on a short prompt
        torch.cuda.synchronize()
        a.record()
        logits, cache = runner.forward(ids, mask)
        b.record()
        torch.cuda.synchronize()
        pre_ms = a.elapsed_time(b)
        out["prefill_ms"] = round(pre_ms, 2)
        out["prefill_tok_s"] = round(batch * context / (pre_ms * 1e-3), 1)
        tok = logits[:, -1].argmax(-1, keepdim=True)
        out["context_source"] = "prefilled in this run (timed)"
    else:
        cache = runner.synthetic_cache(batch, context, steps + 16)
        tok = torch.randint(0, shape.vocab_size, (batch, 1), generator=g).to(dev)
        out["context_source"] = "random KV cache of the prefilled shape (a decode step's cost does not depend on the values)"
    timing = {}
    sampler = ClockSampler(dev.index)  # the leg's own clock record: a decode right behind a long prefill starts power-capped
    sampler.start()
    runner.decode(tok, cache, mask, steps + 1, use_graph=True, timing=timing)
    torch.cuda.synchronize()
    out["clocks"] = sampler.stop()
    ms = timing["events"][0].elapsed_time(timing["events"][1]) / max(1, timing["steps"])
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    bps = model_bytes_per_step(shape, batch, context + steps // 2, world, wbytes=0.53125 if weight_dtype == "mxfp4" else 1.0625)
    pk = peaks()
    out.update({"ms_per_step": round(ms, 4), "decode_tok_s": round(batch / (ms * 1e-3), 1), "timed_steps": timing["steps"],
                "graph": runner.last_graph is not None,
                "bytes_per_step_per_gpu": int(bps), "hbm_gbs_per_gpu": round(bps / (ms * 1e-3) / 1e9, 1),
                "hbm_frac_of_peak": round(bps / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)})
    if world > 1:  # the all-reduces of one step, timed alone (they cannot carry events inside the replayed graph)
        D = shape.hidden_size
        bufs = [torch.zeros((batch, D), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        lg = torch.zeros((batch, shape.vocab_size), dtype=torch.bfloat16, device=dev)
        n = 2 * shape.num_hidden_layers
        for _ in range(3):
            dist.all_reduce(bufs[0])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):
            dist.all_reduce(bufs[i & 1])
        dist.all_reduce(lg)
        b.record()
        torch.cuda.synchronize()
        ar = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
        dist.all_reduce(ar, op=dist.ReduceOp.MAX)
        out["allreduce"] = {"calls_per_step": n + 1, "payload_bytes": batch * D * 2, "ms_back_to_back": round(float(ar.item()), 4),
                            "share_of_step": round(float(ar.item()) / ms, 3),
                            "note": "NCCL all-reduces of one step issued back to back outside the graph; inside the step they sit between dependent kernels"}
    del runner, cache
    torch.cuda.empty_cache()
    return out


def tp_consistency_check(dev, world):
    """Two layers of the tensor-parallel configuration's shape, same seeded weights: logits of the sharded model (this
    run's ranks) against the unsharded model built on the same GPU. max |a - b| / max |b|."""
    import dataclasses
    import torch
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    from tpp_pytorch_extension_b200.llm import llm_common as LC
    shape = dataclasses.replace(FL.LLAMA2_70B, num_hidden_layers=2)
    ids = torch.randint(0, shape.vocab_size, (4, 96), generator=torch.Generator().manual_seed(7)).to(dev)
    sharded = FL.build_random_llama(shape, "mxfp4", dev, max_positions=256)
    l_tp, _ = sharded.forward(ids)
    del sharded
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    LC.tensor_parallel_enabled = False
    pg = F._pg
    try:
        single = FL.build_random_llama(shape, "mxfp4", dev, max_positions=256)
        F.set_pg(None)  # the layers ask the op module for the group size
        l_1, _ = single.forward(ids)
        del single
    finally:
        LC.tensor_parallel_enabled = True
        F.set_pg(pg)
    a, b = l_tp[:, -1].float(), l_1[:, -1].float()
    err = float((a - b).abs().max() / b.abs().max())
    torch.cuda.empty_cache()
    return {"layers": 2, "tokens": "4 x 96", "max_rel_diff_vs_unsharded": err, "same_argmax": bool((a.argmax(-1) == b.argmax(-1)).all()),
            "ranks": world}


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from tpp_pytorch_extension_b200 import _lib
    from tpp_pytorch_extension_b200._C import _fused_llm_infer as F
    from tpp_pytorch_extension_b200._C import _qtype

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.lib()  # fails loudly when the CUDA library is missing

    def block(w):  # BlockedParameter.block() with bk=16, bc=64, VNNI2
        N, K = w.shape
        return w.view(N // 16, 16, K // 64, 32, 2).permute(0, 2, 3, 1, 4).contiguous()

    g = torch.Generator(device="cpu").manual_seed(0)
    sets = []
    w_cpu = []  # 256 sampled rows of each weight of the first set, for the oracle spot check
    for c in range(N_COPIES):
        ws = []
        for (N, K) in ((D_FF, D_MODEL), (D_FF, D_MODEL), (D_MODEL, D_FF)):
            if c == 0:  # seed-0 CPU weights for the first set, device RNG for the L2-rotation copies
                w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
                w_cpu.append(w[spot_rows(N)].clone())
                w = w.to(dev)
            else:
                w = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
            ws.append(_qtype.remap_and_quantize_mxfp4(block(w)))
            del w
        ws[0].prepare(drop_interchange=True, pair_with=ws[1])
        ws[2].prepare(drop_interchange=True)
        sets.append(ws)
    xs_host = {M: torch.randn(M, D_MODEL, generator=g).to(torch.bfloat16).pin_memory() for M in SWEEP}
    xs = {M: xs_host[M].to(dev) for M in SWEEP}
    ys_host = {M: torch.empty(M, D_MODEL, dtype=torch.bfloat16).pin_memory() for M in SWEEP}
    torch.cuda.synchronize()

    launch_count = _lib_launch_count()
    per_op_launches = {}  # (M, op) -> kernels the library launched for one call

    counter = [0]

    def sweep(host=False):
        """One step in interleaved order (warm-up and the end-to-end pass): gate/up then down, for every token count."""
        for mi, M in enumerate(SWEEP):
            wg, wu, wd = sets[counter[0] % N_COPIES]
            counter[0] += 1
            x = xs_host[M] if host else xs[M]
            c0 = launch_count()
            h = F.fc_gate_up(x, wg, wu)
            c1 = launch_count()
            y = F.fc_plain(h, wd, out=ys_host[M] if host else None)
            per_op_launches[(M, "gate_up")], per_op_launches[(M, "down")] = c1 - c0, launch_count() - c1
            hs[M] = h

    def run_shape(M, pair, n, ev):
        """n launches of one shape back to back, weights rotating over the copies, one event pair around them: the
        launches overlap their prologues with the previous launch's tail (programmatic dependent launch) exactly as
        the kernels of a decode step do; an event between two launches would forbid that."""
        ev[0].record()
        for _ in range(n):
            wg, wu, wd = sets[counter[0] % N_COPIES]
            counter[0] += 1
            if pair:
                F.fc_gate_up(xs[M], wg, wu)
            else:
                F.fc_plain(hs[M], wd)
        ev[1].record()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    hs = {}  # input of the down projection per token count: the gate/up output of the last warm-up step
    for _ in range(max(args.warmup, 3)):
        sweep()
    # ---- device-resident timing: the K steps are issued shape by shape (K launches of each), events at shape boundaries.
    # Two timed blocks, each repeated (`rounds`) until its share of min_seconds of device time has been measured and
    # each under its own clock record: first the decode-shaped launches (M <= 64, the headline HBM figure), then the
    # many-token ones. Timed in one block, the 25 ms of power-capped tensor-core work per round set the SM clock the
    # 3 ms of decode launches that follow it run at, which no decode loop would see; every figure is the mean over the
    # rounds of its block.
    def timed_block(idx, min_ms):
        sampler = ClockSampler(local)
        barrier()
        sampler.start()
        seg = np.zeros((len(SWEEP), 2))
        total_ms, rounds, launches = 0.0, 0, 0
        while True:
            evs = [[[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(2)] for _ in SWEEP]
            t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            # Hold the stream busy while the host enqueues the first launches, so that the events measure device
            # time of back-to-back launches and not the host's launch rate (the end-to-end figure below keeps it).
            torch.cuda._sleep(int(5e6))
            launches_before = launch_count()
            t_start.record()
            for mi in idx:
                run_shape(SWEEP[mi], True, args.steps, evs[mi][0])
                run_shape(SWEEP[mi], False, args.steps, evs[mi][1])
            t_end.record()
            launches += launch_count() - launches_before
            torch.cuda.synchronize()
            total_ms += t_start.elapsed_time(t_end)
            for mi in idx:
                for o in range(2):
                    seg[mi, o] += evs[mi][o][0].elapsed_time(evs[mi][o][1]) / args.steps  # ms per launch
            rounds += 1
            flag = torch.tensor([1.0 if (total_ms >= min_ms or rounds >= 2000) else 0.0], device=dev)
            if world > 1:
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)  # every rank runs the same number of rounds
            if flag.item() > 0:
                break
        barrier()
        return seg / rounds, total_ms / rounds, launches // rounds, rounds, sampler.stop()

    dec = [i for i, M in enumerate(SWEEP) if M <= DECODE_MAX_M]
    pre = [i for i, M in enumerate(SWEEP) if M > DECODE_MAX_M]
    seg = np.zeros((len(SWEEP), 2))
    total_ms, timed_launches, rounds, clocks, pre_clocks, pre_rounds = 0.0, 0, 0, None, None, 0
    if dec:
        seg_d, ms_d, n_d, rounds, clocks = timed_block(dec, args.min_seconds * 1e3 * (0.5 if pre else 1.0))
        seg += seg_d
        total_ms += ms_d
        timed_launches += n_d
    if pre:
        seg_p, ms_p, n_p, pre_rounds, pre_clocks = timed_block(pre, args.min_seconds * 1e3 * (0.5 if dec else 1.0))
        seg += seg_p
        total_ms += ms_p
        timed_launches += n_p
    if clocks is None:
        clocks, rounds = pre_clocks, pre_rounds
    _lib.assert_no_kernel_error()  # a kernel that gave up on a bounded wait finishes early: such a run is not a measurement
    # ---- end to end: host buffers in, host buffers out, through the public ops
    for _ in range(2):
        sweep(host=True)
    barrier()
    # K steps over the decode shapes (the ones `value` is computed from), one event pair around all of them: the host
    # issues every launch inside the timed region (no kernel holds the stream back for it), so the figure is the
    # smaller of what the host path and the device sustain; repeated like the device-timed block.
    cur = torch.cuda.current_stream()
    e2e_total, e2e_rounds = 0.0, 0
    while True:
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ea.record(cur)
        for s in range(args.steps):
            for mi in dec:
                M = SWEEP[mi]
                wg, wu, wd = sets[counter[0] % N_COPIES]
                counter[0] += 1
                # the public ops take the pinned host buffers themselves: the activation-split kernel reads X across
                # the bus, the down projection's epilogue writes Y to host memory (no separate copies in the stream)
                F.fc_plain(F.fc_gate_up(xs_host[M], wg, wu), wd, out=ys_host[M])
        eb.record(cur)
        barrier()
        e2e_total += ea.elapsed_time(eb) / args.steps
        e2e_rounds += 1
        flag = torch.tensor([1.0 if (e2e_total * args.steps >= args.min_seconds * 250.0 or e2e_rounds >= 500) else 0.0], device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if flag.item() > 0 or not dec:
            break
    e2e_step_ms = e2e_total / e2e_rounds
    _lib.assert_no_kernel_error()
    parity = parity_spot_check(sets[0], w_cpu, xs_host, dev) if rank == 0 else None

    dec_bytes = sum(op_bytes(SWEEP[i], True) + op_bytes(SWEEP[i], False) for i in dec)
    dec_ms = float(sum(seg[i].sum() for i in dec))
    pre_flops = sum(op_flops(SWEEP[i], True) + op_flops(SWEEP[i], False) for i in pre)
    pre_ms = float(sum(seg[i].sum() for i in pre))
    stats = torch.tensor([total_ms, dec_ms, pre_ms, e2e_step_ms], device=dev, dtype=torch.float64)
    per_rank = [stats.clone() for _ in range(world)]
    if world > 1:
        dist.all_gather(per_rank, stats)
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    per_rank_dec_ms = [round(float(t[1]), 5) for t in per_rank]
    per_rank_e2e_ms = [round(float(t[3]), 5) for t in per_rank]
    total_ms, dec_ms, pre_ms, e2e_dec_ms = [float(v) for v in stats.cpu()]
    pk = peaks()
    value = world * dec_bytes / (dec_ms * 1e-3) / 1e9
    e2e_value = world * dec_bytes / (e2e_dec_ms * 1e-3) / 1e9
    # dominant decode kernel: the gate/up pair launch with the largest time share among M <= 64
    dom = max(dec, key=lambda i: seg[i, 0])
    dom_gbs = op_bytes(SWEEP[dom], True) / (seg[dom, 0] * 1e-3) / 1e9
    kernels = []
    for i, M in enumerate(SWEEP):
        for j, pair in enumerate((True, False)):
            ms = float(seg[i, j])
            kernels.append({"M": M, "op": "gate_up" if pair else "down", "ms": round(ms, 5),
                            "gbs": round(op_bytes(M, pair) / (ms * 1e-3) / 1e9, 1),
                            "tflops": round(op_flops(M, pair) / (ms * 1e-3) / 1e12, 2),
                            "launches": per_op_launches.get((M, "gate_up" if pair else "down"))})
    dom_share = float(seg[dom, 0] / max(1e-9, sum(seg[i].sum() for i in dec)))
    if rank == 0:
        line = {
            "metric": "qgemm_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x mxfp4 -> fp32 acc", "data": "synthetic",
            "config": workload_config(),
            "prefill": {"tflops": world * pre_flops / (pre_ms * 1e-3) / 1e12 if pre_ms > 0 else None, "unit": "TFLOP/s",
                        "frac_of_bf16_peak": pre_flops / (pre_ms * 1e-3) / 1e12 / pk["bf16_tflops"] if pre_ms > 0 else None,
                        # the prefill kernel issues kind::mxf8f6f4 MMAs, which run at the 8-bit rate (twice the bf16 rate)
                        "frac_of_issued_kind_peak": pre_flops / (pre_ms * 1e-3) / 1e12 / (2 * pk["bf16_tflops"]) if pre_ms > 0 else None,
                        "issued_kind_peak": "2 x the bf16 cuBLAS burst figure (no 8-bit GEMM peak is measured on this pool)",
                        "peak_src": pk["src"], "clocks": pre_clocks, "rounds": pre_rounds},
            "roofline": {"bound": "hbm",
                         "kernel": f"MXFP4 gate/up pair GEMM, M={SWEEP[dom]} (tcgen05: qlinear_tc4_kernel, kind::mxf4, for M <= 32; "
                                   f"qlinear_tcw_kernel, kind::mxf8f6f4, for M <= 64; qlinear_tcp2_kernel, cta_group::2, beyond)"
                                   if F.mxfp4_path() == "tc" else f"qlinear_stream gate/up pair, M={SWEEP[dom]}",
                         "achieved": dom_gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": dom_gbs / pk["hbm_gbs"],
                         "peak_src": pk["src"], "traffic": NCU_TRAFFIC.get(SWEEP[dom]),
                         "traffic_src": "ncu capture summarised under profiles/, not measured in this run",
                         "duration": "CUDA events around K back-to-back launches of the op (activation-split kernel + GEMM kernel each), divided by K"},
            "kernels": kernels,
            "e2e": {"value": e2e_value, "unit": "GB/s",
                    "h2d_bytes_per_step": sum(SWEEP[i] * D_MODEL * 2 for i in dec),
                    "d2h_bytes_per_step": sum(SWEEP[i] * D_MODEL * 2 for i in dec), "rounds": e2e_rounds,
                    "scope": "the decode-shaped launches (M <= 64) through the public ops with pinned HOST X in and pinned host Y out: the "
                             "kernels read X from and write Y to host memory directly (every byte crosses the bus inside the timed "
                             "region); K steps inside one event pair, the host issuing every launch inside it"},
            "gpu_launches": int(timed_launches),
            "timed": {"rounds": rounds, "prefill_rounds": pre_rounds,
                      "note": "decode-shaped and many-token launches are timed in separate blocks of K steps, each repeated until its "
                              "half of min_seconds of device time and each with its own clock record ('clocks' = decode block, "
                              "'prefill.clocks'); figures are means over a block's rounds; ms_per_step adds the two"},
            "per_rank": {"decode_ms": per_rank_dec_ms, "e2e_decode_ms": per_rank_e2e_ms},
            "kernel_errors": 0, "parity_check": parity,
            "clocks": clocks,
        }
        if world == 1:
            line["cpu_baseline"] = cpu_arm()
    # ---- model-level decode legs (outside the timed region of the headline metric)
    del sets
    torch.cuda.empty_cache()
    legs = {}
    want = [v for v in args.legs.split(",") if v]
    from tpp_pytorch_extension_b200.llm import fused_llama_infer as FL
    import dataclasses
    if "cfg3" in want and world == 1:
        legs["config3_llama2_7b_int8"] = model_decode_leg("Llama-2-7B shape, int8 (K blocks of 64)", FL.LLAMA2_7B, 1, 1024, 128, dev, 1, 0, True,
                                                          weight_dtype="qint8")
    if "cfg4" in want and world == 1:
        legs["config4_llama3_8b_mxfp4"] = model_decode_leg("Llama-3-8B shape, MXFP4", FL.LLAMA3_8B, 16, 2048, args.model_steps, dev, 1, 0, True)
    if "cfg5" in want:
        shape = FL.LLAMA2_70B if not args.cfg5_layers else dataclasses.replace(FL.LLAMA2_70B, num_hidden_layers=args.cfg5_layers)
        if world > 1:
            legs["config5_tp_consistency"] = tp_consistency_check(dev, world)
        legs["config5_llama2_70b_mxfp4_tp"] = model_decode_leg("Llama-2-70B shape, MXFP4, tensor parallel", shape, 64, 4096, args.model_steps, dev,
                                                               world, rank, False)
    if rank == 0:
        line["decode_models"] = legs
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ms", default="", help="comma-separated subset of the token counts to run (for profiler captures)")
    ap.add_argument("--legs", default="cfg3,cfg4,cfg5", help="model-level decode legs to run after the op sweep: cfg3 (Llama-2-7B shape, int8, one GPU), cfg4 (Llama-3-8B shape, one GPU), "
                    "cfg5 (Llama-2-70B shape, tensor parallel over --gpus ranks); empty for none")
    ap.add_argument("--model-steps", type=int, default=48, help="decode steps timed in each model-level leg")
    ap.add_argument("--cfg5-layers", type=int, default=0, help="decoder layers of the 70B-shape leg (0 = all 80)")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="repeat the K timed steps until this much device time was measured")
    args = ap.parse_args()
    if args.ms:
        global SWEEP
        SWEEP = [int(v) for v in args.ms.split(",")]
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
