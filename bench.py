#!/usr/bin/env python
"""Contract benchmark: decode tokens/s (+ p50 TTFT) of the paged-KV attention path.

Workload (BASELINE.json configs[1]): Qwen3-0.6B (random-init, bf16), 256 sequences x 1024-token
prompts, kvcache_block_size 16, CUDA-graph decode, one engine per GPU.  A "step" is one decode
step of the whole batch (one pass of the hot path: 28 x [K8 epilogue, paged decode attention,
fused norms/activation] + cuBLAS GEMMs + sampling).

  value      device-timed decode throughput: K graph replays with the step's inputs resident in HBM
  e2e        the same K steps through the public API (LLM.step): per step one H2D of the packed
             step metadata from pinned memory and one D2H of the sampled ids, scheduler included
  roofline   the dominant kernel (paged_decode_kernel) timed alone over all 28 layers' caches
             (28 GiB streamed per pass, far beyond L2), launched the way the step launches it (the
             runner's grid; two half-batch launches per layer when the step runs as two micro-batches,
             with the one-launch-per-layer figure beside it), algorithmic KV bytes / event time
  cpu_baseline  the reference's CPU path (oracle port of models/qwen3.py + torch-native
             attention) on the host cores, bounded sample of the same decode step

N > 1 (torchrun): independent data-parallel replicas, no data-path collective ("weak" scaling) --
the headline line -- plus a `tp` object: Qwen3-32B (BASELINE configs[3]) decode at the same batch /
context tensor-parallel over all N GPUs (fused NVLink all-reduce + residual add + RMSNorm), with
the all-reduce form and its latency, and the same workload at TP=1 (rank 0) for the speed-up.
`--tp` instead makes the tensor-parallel engine the whole line ("strong" scaling).
`--impl reference` times only the CPU reference arm.
`--hybrid` leaves the contract workload aside: the Zegopel hybrid decoder beside the dense decoder of the same width
(prefill and decode throughput through the engine) and the rooflines of its kernels beside their like kernels;
`--hybrid --design nirelix` does the same for the Nirelix decoder beside the Zegopel decoder of the same width, and
`--hybrid --design fitevik` for the Fitevik decoder beside the Nirelix decoder of the same width, and
`--hybrid --design nurilorn` for the Nurilorn decoder beside the Zegopel decoder of the same width.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "nano-vllm-ascend_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

METRIC = "decode_tokens_per_s"
UNIT = "tokens/s"


def moe_expert_roofline(runner, B, peak_gbs):
    """Sparse-MoE models: the expert GEMMs (csrc/moe.cu) are the other HBM stream of a decode step.
    Timed alone with CUDA events over every layer's own expert weights (>= 1 GB per layer, cold in L2);
    algorithmic bytes per layer = experts hit x 3 x hidden x moe_intermediate x 2 B."""
    from nanovllm import ops
    from nanovllm.layers.moe import SparseMoeBlock
    blocks = [m for m in runner.model.modules() if isinstance(m, SparseMoeBlock)]
    blk = blocks[0]
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(B, blk.hidden_size, device="cuda", generator=g).to(runner.dtype)
    scores = torch.rand(B, blk.num_experts, device="cuda", generator=g)
    ids = scores.topk(blk.top_k, dim=1).indices.to(torch.int32).contiguous()
    w = torch.full((B, blk.top_k), 1.0 / blk.top_k, device="cuda").to(runner.dtype)
    plan = ops.moe_align(ids, blk.expert_begin, blk.num_local)
    hit = int((plan.offsets[1:] > plan.offsets[:-1]).sum())

    def one_pass():
        for b in blocks:
            ops.moe_experts(x, b.w13, b.w2, ids, w, plan)
    for _ in range(2):
        one_pass()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 4
    e0.record()
    for _ in range(reps):
        one_pass()
    e1.record()
    torch.cuda.synchronize()
    per_layer_s = e0.elapsed_time(e1) / 1e3 / (reps * len(blocks))
    nbytes = hit * 3 * blk.hidden_size * blk.inter * x.element_size()
    achieved = nbytes / per_layer_s / 1e9
    return {"bound": "hbm", "kernel": "moe_gemm_kernel<gate_up> + <down> + moe_combine_kernel",
            "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs,
            "algorithmic_bytes_per_launch": nbytes, "us_per_layer": per_layer_s * 1e6,
            "experts_hit": hit, "local_experts": blk.num_local, "layers": len(blocks)}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--model", default="qwen3-0.6b")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--tp", action="store_true", help="tensor-parallel over --gpus instead of replicas")
    ap.add_argument("--tp-model", default="qwen3-32b",
                    help="model of the `tp` object a multi-GPU replica run adds (BASELINE configs[3])")
    ap.add_argument("--no-tp-block", action="store_true", help="multi-GPU replica run without the `tp` object")
    ap.add_argument("--tp-timeout", type=float, default=420.0, help="seconds before the `tp` object is abandoned")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--mem-util", type=float, default=0.7, help="gpu_memory_utilization of the engine")
    ap.add_argument("--cpu-sample-seqs", type=int, default=32)
    ap.add_argument("--hybrid", action="store_true",
                    help="instead of the contract workload: prefill and decode throughput of the Zegopel hybrid "
                         "decoder beside the dense decoder of the same width and depth, and its kernels' rooflines")
    ap.add_argument("--hybrid-pairs", default=None,
                    help="model:model,... (default zegopel-1k:qwen3-0.6b,zegopel-2k:llama-3.2-1b; with --design "
                         "nirelix: nirelix-1k:zegopel-1k,nirelix-2k:zegopel-2k; with --design fitevik: "
                         "fitevik-1k:nirelix-1k,fitevik-2k:nirelix-2k; with --design nurilorn: "
                         "nurilorn-1k:zegopel-1k,nurilorn-2k:zegopel-2k)")
    ap.add_argument("--design", default="zegopel", choices=["zegopel", "nirelix", "fitevik", "nurilorn"],
                    help="with --hybrid: whose presets and kernel table are measured")
    ap.add_argument("--kv-cache-dtype", default="auto", choices=["auto", "fp8"],
                    help="fp8: e4m3 KV cache (an extra line; the contract line is the default bf16 cache)")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    except (OSError, ValueError, KeyError, TypeError):
        return 6650.0, "fallback (B200_PROFILING.md)"


def tensor_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured burst cuBLAS bf16 (MEASURED_PEAKS.json)"
    except (OSError, ValueError, KeyError, TypeError):
        return 1590.0, "fallback (B200_PROFILING.md)"


def prefill_roofline():
    """The tensor-bound kernel of the path (prefill_umma_kernel) timed alone with CUDA events on the
    shapes BASELINE names: configs[1]'s prefill batch (16 x 1024 tokens, Qwen3-0.6B heads) and configs[2]
    (Llama-3.2-1B, 8192-token prompt: whole, and the prefix-cache-hit form -- 256 new tokens against
    7936 cached ones read through block tables). Flops = 4 * H * D * sum over rows of visible keys
    (causal); inputs rotate over copies totalling > L2."""
    from nanovllm import ops
    peak, src = tensor_peak()
    g = torch.Generator(device="cuda").manual_seed(0)
    bf = torch.bfloat16

    def timed(fns, iters=24):
        for f in fns:
            f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fns[i % len(fns)]()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3 / iters

    def packed(nseq, L, H, G, D, copies):
        T = nseq * L
        cu = torch.arange(0, T + 1, L, dtype=torch.int32, device="cuda")
        out = torch.empty(T, H * D, dtype=bf, device="cuda")
        fns = []
        for _ in range(copies):
            qkv = torch.randn(T, (H + 2 * G) * D, device="cuda", generator=g).to(bf)
            q = qkv[:, :H * D].unflatten(1, (H, D))
            k = qkv[:, H * D:(H + G) * D].unflatten(1, (G, D))
            v = qkv[:, (H + G) * D:].unflatten(1, (G, D))
            fns.append(lambda q=q, k=k, v=v: ops.prefill_varlen_attn(q, k, v, cu, cu, L, L, D ** -0.5, G, out=out))
        sec = timed(fns)
        flops = 2 * L * L * H * D * nseq
        return {"shape": f"{nseq} x {L} tokens, H={H} Hkv={G} D={D}, packed, causal", "us": sec * 1e6,
                "tflops": flops / sec / 1e12, "frac": flops / sec / 1e12 / peak}

    def prefix_hit(qlen, klen, H, G, D, bs, copies):
        nblk = (klen + bs - 1) // bs
        cu_q = torch.tensor([0, qlen], dtype=torch.int32, device="cuda")
        cu_k = torch.tensor([0, klen], dtype=torch.int32, device="cuda")
        out = torch.empty(qlen, H * D, dtype=bf, device="cuda")
        q = torch.randn(qlen, H, D, device="cuda", generator=g).to(bf)
        fns = []
        for _ in range(copies):
            kc = torch.randn(nblk + 1, bs, G * D, device="cuda", generator=g).to(bf)
            vc = torch.randn(nblk + 1, bs, G * D, device="cuda", generator=g).to(bf)
            bt = torch.randperm(nblk, device="cuda", generator=g).to(torch.int32).view(1, -1).contiguous()
            fns.append(lambda kc=kc, vc=vc, bt=bt: ops.prefill_varlen_attn(
                q, kc, vc, cu_q, cu_k, qlen, klen, D ** -0.5, G, block_tables=bt, out=out))
        sec = timed(fns)
        flops = 4 * H * D * (qlen * (klen - qlen) + qlen * qlen / 2)
        return {"shape": f"q {qlen} / k {klen} tokens, H={H} Hkv={G} D={D}, paged block {bs} (prefix-cache hit)",
                "us": sec * 1e6, "tflops": flops / sec / 1e12, "frac": flops / sec / 1e12 / peak}

    main = packed(16, 1024, 16, 8, 128, 2)
    shapes = [main, packed(4, 4096, 16, 8, 128, 2), packed(1, 8192, 32, 8, 64, 4),
              prefix_hit(256, 8192, 32, 8, 64, 16, 16)]
    return {"bound": "tensor", "kernel": "prefill_umma_kernel", "achieved": main["tflops"], "peak": peak,
            "unit": "TFLOP/s", "frac": main["frac"], "peak_source": src, "traffic": None,
            "shapes": shapes}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms during the timed regions. The process
    is started early (its NVML start-up takes driver locks for a few hundred ms: started right before
    the timed region it randomly stalled the first prefill step by 100-400 ms and with it every TTFT);
    only rows that arrive after begin() are counted."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index, self.t_begin = [], None, index, 0.0

    def begin(self):
        self.t_begin = time.perf_counter()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, r in self.rows:
            if t < self.t_begin:
                continue
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # under load = samples within 85% of the hottest power draw is unknowable here; use median
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ CPU reference arm
def cpu_reference_step(n_seqs, ctx, block_size, steps, warmup, threads=None):
    """The reference's CPU path (oracle port: eager layers + torch-native attention, bf16) on a
    bounded sample: one full-model decode step for `n_seqs` of the workload's sequences at the
    workload's context length. Returns (tokens/s, seconds per step)."""
    from oracle import model_ref as M
    if threads:
        torch.set_num_threads(threads)
    cfg = M.ModelCfg.qwen3_0_6b()
    w = M.seeded_weights(cfg, seed=0)
    nblk_per = (ctx + 1 + block_size - 1) // block_size
    nb = n_seqs * nblk_per + 1
    g = torch.Generator().manual_seed(0)
    kv = (0.5 * torch.randn(2, cfg.num_layers, nb, block_size, cfg.num_kv_heads, cfg.head_dim,
                            generator=g)).to(cfg.dtype)
    tables = [list(range(i * nblk_per, (i + 1) * nblk_per)) for i in range(n_seqs)]
    lens = [ctx] * n_seqs
    ids = torch.randint(0, 10000, (n_seqs,), generator=g)
    times = []
    with torch.inference_mode():
        for i in range(warmup + steps):
            pos, meta = M.decode_meta(lens, tables, block_size)
            t0 = time.perf_counter()
            logits = M.forward(w, cfg, ids, pos, meta, kv, block_size, attn_mode="reference")
            ids = logits.float().argmax(-1)
            dt = time.perf_counter() - t0
            if i >= warmup:
                times.append(dt)
    sec = sum(times) / len(times)
    return n_seqs / sec, sec


def reference_cpu_step(n_seqs, ctx, block_size, steps, warmup, in_process):
    """The CPU arm. With the reference archive present (oracle/_ref/, packed by oracle/stage_ref.py at
    build time) the reference's OWN modules run: models/qwen3.py + layers/attention_torch_native.py on
    all host cores (kind "reference"); otherwise the oracle port of the same graph (kind "port").
    The reference registers a stub package named `nanovllm`, which is also the product's package name:
    the GPU arm therefore runs it in a child process."""
    from oracle import ref_runtime
    cores = os.cpu_count() or 1
    if ref_runtime.reference_dir() is None:
        tps, sec = cpu_reference_step(n_seqs, ctx, block_size, steps, warmup, cores)
        return tps, sec, "port", torch.get_num_threads()
    if in_process:
        tps, sec = ref_runtime.reference_decode_step(n_seqs, ctx, block_size, steps, warmup, cores)
        return tps, sec, "reference", torch.get_num_threads()
    r = subprocess.run([sys.executable, "-m", "oracle.ref_runtime", "--seqs", str(n_seqs), "--ctx", str(ctx),
                        "--block-size", str(block_size), "--steps", str(steps), "--warmup", str(warmup)],
                       cwd=ROOT, capture_output=True, text=True, timeout=1200)
    try:
        if r.returncode != 0:
            raise RuntimeError(r.stderr[-2000:])
        d = json.loads(r.stdout.strip().splitlines()[-1])
        return d["tokens_per_s"], d["s_per_step"], "reference", d["threads"]
    except (RuntimeError, ValueError, KeyError, IndexError) as e:
        # the reference's modules could not be run here: say so and time the oracle port instead
        print(f"bench.py: reference CPU arm failed ({type(e).__name__}: {str(e)[-300:]}); "
              f"timing the oracle port", file=sys.stderr)
        tps, sec = cpu_reference_step(n_seqs, ctx, block_size, steps, warmup, cores)
        return tps, sec, "port", torch.get_num_threads()


def cpu_sample_text(kind, n_seqs, batch, ctx, steps, sec):
    what = ("the reference's own models/qwen3.py + attention_torch_native.py (oracle/_ref archive)"
            if kind == "reference" else
            "oracle port of the reference CPU path (no reference archive on this box)")
    return (f"batch {n_seqs} (of the workload's {batch} sequences), one full 28-layer decode step at "
            f"ctx={ctx}, {steps} timed steps of {sec:.2f} s each; {what}")


def run_reference_arm(args, rank):
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    # bounded sample: as many of the workload's sequences as keep the whole run near a minute
    # (about 0.07 s per sequence-step on 8 host cores)
    n_seqs = max(1, min(32, args.batch, int(600 / (steps + warmup))))
    args.cpu_sample_seqs = n_seqs
    tps, sec, kind, cores = reference_cpu_step(n_seqs, args.ctx, args.block_size, steps, warmup, True)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(workload_config(args, 1), cpu_sample_batch=n_seqs),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": cpu_sample_text(kind, n_seqs, args.batch, args.ctx, steps, sec)},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config(args, world):
    par = "replicas" if not args.tp else f"tp{world}"
    return {"workload": f"{args.model} decode, batch {args.batch}/GPU, ctx {args.ctx}, "
                        f"kvcache_block_size {args.block_size}, CUDA-graph decode (BASELINE configs[1])",
            "global_batch": args.batch * (1 if args.tp else world), "seq_len": args.ctx,
            "parallelism": f"{par}x{world}" if world > 1 else "single",
            "l2": "inputs exceed L2 (>= 28 GiB of KV streamed per step)",
            **({} if args.kv_cache_dtype == "auto" else {"kv_cache_dtype": "fp8_e4m3"})}


# ------------------------------------------------------------------ the GPU arm
def dbg(rank, *a):
    if os.environ.get("B200_BENCH_DEBUG"):
        print(f"[bench rank{rank} {time.strftime('%X')}]", *a, file=sys.stderr, flush=True)


class Group:
    """The ranks a measurement spans: every torchrun rank (replicas, TP=N) or this rank alone (the
    TP=1 comparison run rank 0 makes while the others wait)."""

    def __init__(self, world):
        self.world = world

    def barrier(self):
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max(self, x):
        if self.world == 1:
            return x
        import torch.distributed as dist
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())


def decode_workload(llm, group, B, ctx, K, W, prompt_seed, rank):
    """The workload of BASELINE configs[1] on one engine: submit B prompts of `ctx` tokens at t = 0,
    prefill (TTFT), W warm-up decode steps, K decode steps through LLM.step() (e2e: pinned H2D of the
    step metadata + D2H of the sampled ids inside the timed region), then K replays of the captured
    step with its inputs resident (device). Times are CUDA events, max over the group's ranks."""
    from nanovllm import SamplingParams
    runner = llm.model_runner
    rnd = random.Random(prompt_seed)
    prompts = [[rnd.randint(0, 10000) for _ in range(ctx)] for _ in range(B)]
    sp = SamplingParams(temperature=0.6, ignore_eos=True, max_tokens=W + K + 8)
    group.barrier()
    t_submit = time.perf_counter()
    seqs = [llm.add_request(p, sp) for p in prompts]
    prefill_steps = 0
    step_ms = []
    while llm.scheduler.waiting:
        t_step = time.perf_counter()
        llm.step()
        step_ms.append((time.perf_counter() - t_step) * 1e3)
        prefill_steps += 1
    submit_ms = (t_step - t_submit) * 1e3 - sum(step_ms[:-1]) if step_ms else 0.0   # add_request x B
    ttfts = sorted((s.first_token_time - t_submit) * 1e3 for s in seqs)
    dbg(rank, 'prefill done')
    for _ in range(W):
        llm.step()
    group.barrier()
    h2d0, d2h0 = runner.h2d_bytes, runner.d2h_bytes
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    t0 = time.perf_counter()
    for _ in range(K):
        out, ntok = llm.step()
        assert ntok == -B, f"decode batch shrank to {-ntok}"
    e1.record()
    torch.cuda.synchronize()
    e2e_s = group.max(max(e0.elapsed_time(e1) / 1e3, time.perf_counter() - t0))
    dbg(rank, 'e2e done')
    graph, launches = runner.decode_graph(B)       # the graph run() replays at this batch / context
    for _ in range(W):
        graph.replay()
    group.barrier()
    e0.record()
    for _ in range(K):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    dev_s = group.max(e0.elapsed_time(e1) / 1e3)
    del graph
    dbg(rank, 'replay done')
    return {"e2e_s": e2e_s, "dev_s": dev_s, "ttfts": ttfts, "prefill_steps": prefill_steps,
            "prefill_step_ms": [round(t, 2) for t in step_ms], "submit_ms": round(submit_ms, 2),
            "h2d_per": (runner.h2d_bytes - h2d0) / K, "d2h_per": (runner.d2h_bytes - d2h0) / K,
            "launches": launches * K, "ctx_now": ctx + W + K,
            "two_micro_batches": runner.use_split(B, int(runner.h_ctx[:B].sum()))}


def attention_roofline(runner, group, B, K, tpw, fp8, peak, peak_src):
    """The dominant kernel alone: one launch per layer over that layer's own cache (all layers = tens
    of GB per pass, cold in L2), CUDA events on the launching stream."""
    from nanovllm import ops
    spec = runner.spec
    Hq, Hkv, D = spec.num_heads // tpw, max(1, spec.num_kv_heads // tpw), spec.head_dim
    q = torch.randn(B, Hq, D, device="cuda", dtype=runner.dtype)
    o = torch.empty(B, Hq * D, device="cuda", dtype=runner.dtype)
    ws = ops.decode_workspace(B, Hq, Hkv, D, q.device)
    L = spec.num_layers
    attn_fn = ops.paged_decode_attn_fp8 if fp8 else ops.paged_decode_attn

    # launched the way the step launches it: the runner's grid size, and -- when the step runs as two
    # micro-batches at this batch / context -- two launches of half the rows each
    ctas = runner._attn_ctas(B)
    split = runner._overlap_split(B) if runner.use_split(B, int(runner.h_ctx[:B].sum())) else 0
    parts = [(0, split), (split, B)] if split else [(0, B)]

    def attn_pass(pieces):
        for layer in range(L):
            for lo, hi in pieces:
                attn_fn(q[lo:hi], runner.kv_cache[0, layer], runner.kv_cache[1, layer],
                        runner.d_tables[lo:hi], runner.d_ctx[lo:hi], D ** -0.5, Hkv, out=o[lo:hi], workspace=ws,
                        num_ctas=ctas)

    def seconds_per_pass(pieces, reps):
        for _ in range(3):
            attn_pass(pieces)
        group.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            attn_pass(pieces)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3 / reps
    reps = max(4, min(K, 32))
    launch_s = seconds_per_pass(parts, reps) / (L * len(parts))
    ctx_sum = int(runner.d_ctx[:B].sum().item())
    whole = None
    if split:      # for comparison: the same rows as ONE launch per layer (what the one-batch graph does)
        whole_s = seconds_per_pass([(0, B)], max(4, reps // 2)) / L
        whole_bytes = ctx_sum * 2 * Hkv * D * runner.kv_cache.dtype.itemsize
        whole = {"rows_per_launch": B, "us_per_launch": whole_s * 1e6, "achieved": whole_bytes / whole_s / 1e9,
                 "frac": whole_bytes / whole_s / 1e9 / peak}
    nbytes = ctx_sum * 2 * Hkv * D * runner.kv_cache.dtype.itemsize / len(parts)   # algorithmic bytes / launch
    achieved = nbytes / launch_s / 1e9
    traffic = traffic_ctx = None
    tpath = os.path.join(ROOT, "profiles", "decode_attn_traffic.json")
    if os.path.exists(tpath) and not fp8 and tpw == 1:
        with open(tpath) as f:
            t = json.load(f)
        # the ncu capture was taken at its own context length: scale its bytes/token to this run's
        per_token = t["dram_bytes_per_launch"] / t["context_tokens_per_launch"]
        traffic, traffic_ctx = per_token * ctx_sum / len(parts), t["context_tokens_per_launch"] // B
    return {"bound": "hbm", "kernel": "paged_decode_fp8_kernel" if fp8 else "paged_decode_kernel",
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": traffic, "traffic_source": None if traffic is None else
            f"ncu dram__bytes_read+write per cached token at ctx {traffic_ctx} (profiles/"
            f"decode_attn_traffic.json) x this run's {ctx_sum} cached tokens per launch",
            "peak_source": peak_src, "algorithmic_bytes_per_launch": nbytes,
            "us_per_launch": launch_s * 1e6, "layers": L, "launches_per_layer": len(parts),
            "rows_per_launch": B // len(parts), "grid_ctas": ctas or None, "one_launch_per_layer": whole}


def release(llm):
    """Tear an engine down and give its memory back (the caller must hold no other reference to the
    runner): graphs, KV cache, weights, peer-memory regions."""
    import gc
    llm.exit()
    del llm
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()


def allreduce_microbench(runner, rows, reps=200):
    """The layer's collective alone: the fused all-reduce + residual add + RMSNorm kernel over NVLink
    (or NCCL all-reduce + the add-RMSNorm kernel when the fused path does not take the shape)."""
    import torch.distributed as dist
    from nanovllm import ops
    from nanovllm.comm import get_comm
    hidden = runner.spec.hidden_size
    comm = get_comm()
    res = torch.zeros(rows, hidden, dtype=runner.dtype, device="cuda")
    w = torch.ones(hidden, dtype=runner.dtype, device="cuda")
    out = torch.empty_like(res)
    form = comm.mode(rows, hidden, res.element_size()) if comm is not None else None

    def one():
        if form is not None:
            comm.partial_buffer(rows, hidden, runner.dtype)
            comm.allreduce_add_rmsnorm(out, res, w, 1e-6)
        else:
            dist.all_reduce(out)
            ops.add_rmsnorm_(out, res, w, 1e-6)
    for _ in range(10):
        one()
    torch.cuda.synchronize()
    dist.barrier()
    # inside a CUDA graph, like the decode step: device time per call, not the host's launch rate
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            one()
    graph.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    del graph
    return form or "nccl", e0.elapsed_time(e1) * 1e3 / reps


def tp_engine_measure(args, rank, world, K, W, peak, peak_src, kw):
    """One tensor-parallel engine over all `world` ranks: decode workload, all-reduce microbench,
    attention roofline. Returns the `tp` fields that do not need the TP=1 comparison."""
    from nanovllm import LLM
    B, ctx = args.batch, args.ctx
    llm = LLM(args.tp_model, tensor_parallel_size=world, **kw)
    runner = llm.model_runner
    r = decode_workload(llm, Group(world), B, ctx, K, W, 0, rank)
    form, ar_us = allreduce_microbench(runner, B)
    roof = attention_roofline(runner, Group(world), B, K, world, False, peak, peak_src)
    L, spec = runner.spec.num_layers, runner.spec
    weight_bytes = sum(p.numel() * p.element_size() for p in runner.model.parameters())
    step_bytes = weight_bytes + roof["algorithmic_bytes_per_launch"] * L
    out = {
        "tokens_per_s": B * K / r["dev_s"], "ms_per_step": r["dev_s"] / K * 1e3,
        "e2e_tokens_per_s": B * K / r["e2e_s"], "e2e_ms_per_step": r["e2e_s"] / K * 1e3,
        "ttft_p50_ms": r["ttfts"][len(r["ttfts"]) // 2], "gpu_launches_per_step": r["launches"] // K,
        "allreduce_form": form, "allreduce_us": ar_us, "allreduces_per_step": 2 * L,
        "allreduce_message_bytes": B * spec.hidden_size * 2,
        "sampling": "vocab-sharded keys + 8 B/row MAX all-reduce" if runner.sharded_sampling else
                    "logits gathered on rank 0",
        "attention_us_per_layer": roof["us_per_launch"], "attention_frac_of_hbm_peak": roof["frac"],
        "per_rank_bytes_per_step": step_bytes,
        "per_rank_hbm_floor_ms": step_bytes / (peak * 1e9) * 1e3,
    }
    del runner
    release(llm)
    return out


def tp_block(args, rank, world, K, W, peak, peak_src):
    """BASELINE configs[3]: Qwen3-32B decode, batch 256, ctx 1024, tensor-parallel over ALL `world`
    GPUs of this run, next to the same workload at TP=1 (rank 0 alone, the other ranks wait), so the
    driver's scaling record carries the north_star's "TP=8 >= 6x TP=1" figure."""
    import torch.distributed as dist
    from nanovllm import LLM
    B, ctx = args.batch, args.ctx
    kw = dict(kvcache_block_size=args.block_size, max_num_seqs=B, max_model_len=4096,
              max_num_batched_tokens=16384, distributed_launch="env", gpu_memory_utilization=0.88,
              graph_batch_sizes=(B,), seed=0)
    out = {"model": args.tp_model, "tp": world, "batch": B, "ctx": ctx}
    out.update(tp_engine_measure(args, rank, world, K, W, peak, peak_src, kw))
    dist.barrier()
    if rank == 0:
        llm = LLM(args.tp_model, tensor_parallel_size=1, **kw)
        r1 = decode_workload(llm, Group(1), B, ctx, K, W, 0, rank)
        out.update({"tp1_tokens_per_s": B * K / r1["dev_s"], "tp1_ms_per_step": r1["dev_s"] / K * 1e3,
                    "tp1_e2e_tokens_per_s": B * K / r1["e2e_s"]})
        out["speedup_vs_tp1"] = out["tokens_per_s"] / out["tp1_tokens_per_s"]
        out["e2e_speedup_vs_tp1"] = out["e2e_tokens_per_s"] / out["tp1_e2e_tokens_per_s"]
        release(llm)
    dist.barrier()
    return out


def _timed(fn, flush, reps=5):
    """Median CUDA-event time (s) of fn() with L2 flushed (a 256 MB write) before every launch."""
    out = []
    for i in range(reps + 2):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        if i >= 2:
            out.append(e0.elapsed_time(e1) / 1e3)
    return statistics.median(out)


def hybrid_kernel_table(width, head_dim, tokens, seqs, peak_gbs):
    """The row-wise and mixer kernels of the hybrid decoder alone, at the layer sizes of a `width`-wide model, as a
    prompt step (`seqs` x tokens/seqs) and as a decode step (`seqs` rows at that context), each beside the dense
    decoders' kernel that does the like job. frac = algorithmic bytes / time / measured copy bandwidth."""
    from nanovllm import ops
    dev, bf = "cuda", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g)
    H = width // head_dim
    G = max(1, H // 4)
    rows = []

    def add(name, step, fn, nbytes, like=None, like_fn=None, like_bytes=None, flops=None):
        t = _timed(fn, flush)
        row = {"kernel": name, "step": step, "us": round(t * 1e6, 1), "GB/s": round(nbytes / t / 1e9),
               "frac_of_measured_copy": round(nbytes / t / 1e9 / peak_gbs, 3)}
        if flops:
            row["TFLOP/s_fp32"] = round(flops / t / 1e12, 2)
        if like_fn is not None:
            tl = _timed(like_fn, flush)
            row["like"] = {"kernel": like, "us": round(tl * 1e6, 1),
                           "frac_of_measured_copy": round(like_bytes / tl / 1e9 / peak_gbs, 3)}
        rows.append(row)

    for step, T, spans_of in (("prompt", tokens, None), ("decode", seqs, None)):
        per = T // seqs if step == "prompt" else 1
        ctx = tokens // seqs
        if step == "prompt":
            cu = torch.arange(0, T + 1, per, dtype=torch.int32, device=dev)
            spans = ops.StepSpans(cu, cu, None, per)
        else:
            spans = ops.StepSpans(None, None, torch.full((T,), ctx, dtype=torch.int32, device=dev))
        slots = torch.arange(seqs, dtype=torch.int32, device=dev)
        # residual path
        y, res = rnd(T, width).to(bf), rnd(T, width)
        w1, w2 = rnd(width) * 0.1, rnd(width) * 0.1
        xb, rb, wb = rnd(T, width).to(bf), rnd(T, width).to(bf), rnd(width).to(bf)
        add("residual_add_norms", step, lambda: ops.residual_add_norms_(y, res, w1, w2, 1e-6), T * width * 12,
            "add_rmsnorm", lambda: ops.add_rmsnorm_(xb, rb, wb, 1e-6), T * width * 8)
        ff = 3 * width
        gu = rnd(T, 2 * ff).to(bf)
        add("act_and_mul(relu)", step, lambda: ops.act_and_mul(gu, "relu"), T * ff * 6,
            "silu_and_mul", lambda: ops.silu_and_mul(gu), T * ff * 6)
        # attention mixer epilogue: convolution, then unit norms + temperature + scatter
        nq, nk = H * head_dim, G * head_dim
        C = nq + 2 * nk
        proj = rnd(T, C + nq).to(bf)
        cw = rnd(C, 3)
        cstate = torch.zeros(seqs + 1, 2, C, dtype=bf, device=dev)
        add("causal_conv(q|k|v, 3 taps)", step,
            lambda: ops.causal_conv(proj[:, :C], cw, None, spans, cstate, slots), T * C * 4)
        qkv = rnd(T, C).to(bf)
        pos = torch.arange(T, device=dev) % max(per, 1) + (0 if step == "prompt" else ctx - 1)
        nb = (T + 15) // 16 + 1
        kc = torch.zeros(nb, 16, nk, dtype=bf, device=dev)
        vc = torch.zeros(nb, 16, nk, dtype=bf, device=dev)
        sl = torch.arange(T, dtype=torch.int32, device=dev)
        table = torch.cat([torch.cos(rnd(4096, head_dim // 2)), torch.sin(rnd(4096, head_dim // 2))], -1).contiguous()
        qw = torch.ones(head_dim, dtype=bf, device=dev)
        like_pos = pos.clamp(max=4095)
        add("unitnorm_temp_cache", step,
            lambda: ops.unitnorm_temp_cache(qkv, pos, 1e-6, 0.1, 1024, H, G, head_dim, head_dim, kc, vc, sl),
            T * (2 * (nq + nk) * 2 + nk * 2 + 2 * nk * 2),
            "qknorm_rope_cache", lambda: ops.qknorm_rope_cache(qkv, like_pos, table, qw, qw, 1e-6, kc, vc, sl, H, G, head_dim),
            T * (2 * (nq + nk) * 2 + nk * 2 + 2 * nk * 2))
        o32, gate = rnd(T, nq), rnd(T, 2 * nq).to(bf)
        nw = rnd(nq)
        add("gated_norm(norm, sigmoid gate)", step, lambda: ops.gated_norm(o32, gate[:, nq:], nw, 1e-6), T * nq * 8)
        # recurrences: lightning (H heads of head_dim x head_dim) and the selective form (2*width/64 heads, state 128)
        p4 = rnd(T, 4 * nq).to(bf)
        decay = torch.linspace(0.9, 0.999, H, device=dev)
        st = torch.zeros(seqs + 1, H, head_dim, head_dim, device=dev)
        rec_bytes = T * nq * (3 * 2 + 4) + (2 * seqs * H * head_dim * head_dim * 4 if step == "decode" else 0)
        add("linear_recurrence(constant decay)", step,
            lambda: ops.linear_recurrence(p4[:, :nq], p4[:, nq:2 * nq], p4[:, 2 * nq:3 * nq], spans, H, H, head_dim,
                                          head_dim, st, slots, decay=decay, act_silu=True),
            rec_bytes, flops=4.0 * T * H * head_dim * head_dim)
        Hm, dvm, N, Gm = 2 * width // 64, 64, 128, 8
        xbc = rnd(T, Hm * dvm + 2 * Gm * N).to(bf)
        dt = rnd(T, Hm).to(bf)
        stm = torch.zeros(seqs + 1, Hm, N, dvm, device=dev)
        par = [rnd(Hm) * 0.5, -torch.rand(Hm, device=dev, generator=g) * 2, torch.ones(Hm, device=dev)]
        inner = Hm * dvm
        add("linear_recurrence(selective)", step,
            lambda: ops.linear_recurrence(xbc[:, inner + Gm * N:], xbc[:, inner:inner + Gm * N], xbc[:, :inner], spans,
                                          Hm, Gm, N, dvm, stm, slots, dt=dt, dt_bias=par[0], a_log=par[1], d_skip=par[2]),
            T * (inner * 6 + 2 * Gm * N * 2) + (2 * seqs * Hm * N * dvm * 4 if step == "decode" else 0),
            flops=4.0 * T * Hm * N * dvm)
    return rows


def nirelix_kernel_table(width, head_dim, tokens, seqs, peak_gbs):
    """The kernels that the Nirelix decoder adds, alone, at the layer sizes of a `width`-wide model, as a prompt step
    (`seqs` x tokens/seqs) and as a decode step (`seqs` rows at that context), each beside the like kernel of the
    Zegopel decoder. frac = algorithmic bytes / time / measured copy bandwidth."""
    from nanovllm import ops
    dev, bf = "cuda", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g)
    H = width // head_dim
    G = max(1, H // 2)
    S = 4
    rows = []

    def add(name, step, fn, nbytes, like=None, like_fn=None, like_bytes=None, flops=None):
        t = _timed(fn, flush)
        row = {"kernel": name, "step": step, "us": round(t * 1e6, 1), "GB/s": round(nbytes / t / 1e9),
               "frac_of_measured_copy": round(nbytes / t / 1e9 / peak_gbs, 3)}
        if flops:
            row["TFLOP/s"] = round(flops / t / 1e12, 2)
        if like_fn is not None:
            tl = _timed(like_fn, flush)
            row["like"] = {"kernel": like, "us": round(tl * 1e6, 1),
                           "frac_of_measured_copy": round(like_bytes / tl / 1e9 / peak_gbs, 3)}
            row["times_as_far_from_roofline_as_like"] = round((like_bytes / tl) / (nbytes / t), 2)
        rows.append(row)

    for step, T in (("prompt", tokens), ("decode", seqs)):
        per = T // seqs if step == "prompt" else 1
        ctx = tokens // seqs
        if step == "prompt":
            cu = torch.arange(0, T + 1, per, dtype=torch.int32, device=dev)
            spans = ops.StepSpans(cu, cu, None, per)
        else:
            spans = ops.StepSpans(None, None, torch.full((T,), ctx, dtype=torch.int32, device=dev))
        slots = torch.arange(seqs, dtype=torch.int32, device=dev)
        pos = (torch.arange(T, device=dev) % max(per, 1) + (0 if step == "prompt" else ctx - 1)).contiguous()
        # residual path: S streams rewritten + read + layer norm, beside the one-stream add + two RMS norms
        X, y, res = rnd(T, S, width), rnd(T, width).to(bf), rnd(T, width)
        mix, ow, iw, w1, w2 = rnd(S, S), rnd(S), rnd(S), rnd(width), rnd(width)
        add("stream_mix_norm(4 streams)", step,
            lambda: ops.stream_mix_norm_(X, y, mix, ow, iw, w1, w2, 1e-6, bf), T * width * (S * 8 + 4),
            "residual_add_norms", lambda: ops.residual_add_norms_(y, res, w1, w2, 1e-6), T * width * 12)
        ff = 3 * width
        gu = rnd(T, 2 * ff).to(bf)
        add("glu_clamped", step, lambda: ops.glu_clamped(gu, 1.702, 7.0), T * ff * 6,
            "act_and_mul(relu)", lambda: ops.act_and_mul(gu, "relu"), T * ff * 6)
        # retention: rotary on q|k into fp32, then the constant-decay recurrence on fp32 q, k
        nq = H * head_dim
        p4 = rnd(T, 4 * nq).to(bf)
        qk_view = p4[:, :2 * nq].unflatten(1, (2 * H, head_dim))
        qkv_like = rnd(T, nq + 2 * G * head_dim).to(bf)
        nb = (T + 15) // 16 + 1
        kc = torch.zeros(nb, 16, G * head_dim, dtype=bf, device=dev)
        vc = torch.zeros(nb, 16, G * head_dim, dtype=bf, device=dev)
        sl = torch.arange(T, dtype=torch.int32, device=dev)
        add("rotary_heads(q|k -> fp32)", step,
            lambda: ops.rotary_heads(qk_view, pos, 2 * H, head_dim, head_dim, 1e6, False, out_f32=True, split=H,
                                     scale_hi=head_dim ** -0.5), T * 2 * nq * 6,
            "unitnorm_temp_cache", lambda: ops.unitnorm_temp_cache(qkv_like, pos, 1e-6, 0.1, 1024, H, G, head_dim,
                                                                   head_dim, kc, vc, sl),
            T * (2 * (nq + G * head_dim) * 2 + 3 * G * head_dim * 2))
        qk32 = rnd(T, 2 * nq)
        decay = torch.linspace(0.9, 0.999, H, device=dev)
        st = torch.zeros(seqs + 1, H, head_dim, head_dim, device=dev)
        state_bytes = 2 * seqs * H * head_dim * head_dim * 4 if step == "decode" else 0
        add("linear_recurrence(fp32 q, k; constant decay)", step,
            lambda: ops.linear_recurrence(qk32[:, :nq], qk32[:, nq:], p4[:, 2 * nq:3 * nq], spans, H, H, head_dim,
                                          head_dim, st, slots, decay=decay), T * nq * (2 * 4 + 2 + 4) + state_bytes,
            "linear_recurrence(bf16 q, k)", lambda: ops.linear_recurrence(p4[:, :nq], p4[:, nq:2 * nq], p4[:, 2 * nq:3 * nq],
                                                                         spans, H, H, head_dim, head_dim, st, slots,
                                                                         decay=decay, act_silu=True),
            T * nq * (3 * 2 + 4) + state_bytes, flops=4.0 * T * H * head_dim * head_dim)
        o32, gate = rnd(T, nq), rnd(T, nq).to(bf)
        ones = torch.ones(nq, device=dev)
        add("gated_norm(a norm per head, silu gate)", step,
            lambda: ops.gated_norm(o32, gate, ones, 1e-6, groups=H, gate_act="silu"), T * nq * 8,
            "gated_norm(one norm per row)", lambda: ops.gated_norm(o32, gate, ones, 1e-6), T * nq * 8)
        # delta rule: preparation, then the recurrence (like: the selective recurrence, which also decays per token)
        ngk = G * head_dim
        qkc = rnd(T, 2 * ngk + nq).to(bf)
        a_in, b_in = rnd(T, nq).to(bf), rnd(T, H).to(bf)
        dtb, alog = rnd(nq), -torch.rand(H, device=dev, generator=g) * 2 - 1
        add("delta_prep", step, lambda: ops.delta_prep(qkc[:, :2 * ngk], a_in, b_in, dtb, alog, H, G, head_dim, 1e-6,
                                                       head_dim ** -0.5), T * (2 * ngk * 6 + nq * 6 + H * 6))
        q32, dec, beta = ops.delta_prep(qkc[:, :2 * ngk], a_in, b_in, dtb, alog, H, G, head_dim, 1e-6, head_dim ** -0.5)
        Hm, dvm, N, Gm = 2 * width // 64, 64, 128, 8
        xbc = rnd(T, Hm * dvm + 2 * Gm * N).to(bf)
        dt = rnd(T, Hm).to(bf)
        stm = torch.zeros(seqs + 1, Hm, N, dvm, device=dev)
        par = [rnd(Hm) * 0.5, -torch.rand(Hm, device=dev, generator=g) * 2, torch.ones(Hm, device=dev)]
        inner = Hm * dvm
        add("delta_rule", step,
            lambda: ops.delta_rule(q32[:, :ngk], q32[:, ngk:], qkc[:, 2 * ngk:], dec, beta, spans, H, G, head_dim,
                                   head_dim, st, slots), T * (2 * ngk * 4 + nq * 4 + nq * 2 + nq * 4) + state_bytes,
            "linear_recurrence(selective)",
            lambda: ops.linear_recurrence(xbc[:, inner + Gm * N:], xbc[:, inner:inner + Gm * N], xbc[:, :inner], spans,
                                          Hm, Gm, N, dvm, stm, slots, dt=dt, dt_bias=par[0], a_log=par[1], d_skip=par[2]),
            T * (inner * 6 + 2 * Gm * N * 2) + (2 * seqs * Hm * N * dvm * 4 if step == "decode" else 0),
            flops=8.0 * T * H * head_dim * head_dim)
        # latent attention: latent rows + cache write, then attention over [latent | rotated key] rows in a window
        R, dr, Q, window = 4 * head_dim, head_dim // 2, 3 * width // 4, 512
        lat = rnd(T, Q + R + dr).to(bf)
        wq, wc = rnd(Q), rnd(R)
        nbl = seqs * (-(-ctx // 16)) + 1
        cache = (torch.randn(nbl, 16, R + dr, device=dev, generator=g) * 0.3).to(bf)
        tables = torch.arange(seqs * (-(-ctx // 16)), dtype=torch.int32, device=dev).view(seqs, -1)
        add("latent_kv_prep", step,
            lambda: ops.latent_kv_prep(lat[:, :Q], lat[:, Q:], wq, wc, pos, R, dr, dr, 1e4, True, 1e-6, cache, sl),
            T * ((Q + R + dr) * 2 + Q * 2 + 2 * (R + dr) * 2))
        qx = (rnd(T, H, R + dr) * 0.3).to(bf)
        keys = min(window, ctx)
        att_flops = 2.0 * T * H * (min(window, (per + 1) / 2) if step == "prompt" else keys) * (2 * R + dr)
        add("attn_generic(latent rows, window 512)", step,
            lambda: ops.attn_generic(qx, cache, None, spans, 0.07, 1, R, block_tables=tables, window=window),
            T * H * (R + dr + R) * 2 + seqs * min(ctx, keys + per) * (R + dr) * 2, flops=att_flops)
        # what 16-bit prompts and windowed decode steps run instead: library products around the masked softmax kernel
        from nanovllm.layers.seq_mixers import LatentAttention
        from nanovllm.utils.context import get_context, reset_context, set_context
        la = LatentAttention(H, head_dim, dr, head_dim, R, 0.07, window=window)
        la.k_cache = cache
        if step == "prompt":
            set_context(True, cu_seqlens_q=spans.cu_q, cu_seqlens_k=spans.cu_k, max_seqlen_q=per, max_seqlen_k=per,
                        block_tables=tables, block_size=16, host_spans=[(i * per, per, per) for i in range(seqs)])
            fn = lambda: la._prefill_by_products(qx, None, get_context(), True)
            band = sum(min(window, i + 1) for i in range(per)) * seqs          # visible (query, key) pairs
        else:
            set_context(False, context_lens=spans.ctx_lens, block_tables=tables, block_size=16)
            fn = lambda: la._decode_window_by_products(qx, get_context())
            band = T * keys
        add("latent attention by products (window 512)", step, fn,
            T * H * (R + dr + R) * 2 + seqs * min(ctx, keys + per) * (R + dr) * 2, flops=2.0 * band * H * (2 * R + dr))
        reset_context()
        # mixture of experts: router, then the expert kernels (like: the softmax router and the same expert kernels)
        E, top, ffe = 16, 2, width // 2
        x = rnd(T, width).to(bf)
        logits = rnd(T, E)
        corr = rnd(E) * 0.1
        add("moe_route_grouped", step, lambda: ops.moe_route_grouped(logits, corr, top, 4, 2, 1.5), T * (E * 4 + top * 8),
            "moe_route(softmax)", lambda: ops.moe_route(logits.to(bf), top), T * (E * 2 + top * 6))
        ids, wts = ops.moe_route_grouped(logits, corr, top, 4, 2, 1.5)
        plan = ops.moe_align(ids, 0, E)
        w13, w2e = (rnd(E, 2 * ffe, width) * 0.03).to(bf), (rnd(E, width, ffe) * 0.03).to(bf)
        wb = wts.to(bf)
        add("moe_experts_generic", step, lambda: ops.moe_experts_generic(x, w13, w2e, wts, plan),
            3 * E * ffe * width * 2 + T * width * 4,
            "moe_experts(tensor cores)", lambda: ops.moe_experts(x, w13, w2e, ids, wb, plan),
            3 * E * ffe * width * 2 + T * width * 4, flops=6.0 * T * top * ffe * width)
    return rows


def fitevik_kernel_table(width, head_dim, tokens, seqs, peak_gbs):
    """The kernels that the Fitevik decoder adds, alone, at the layer sizes of a `width`-wide model, as a prompt step
    (`seqs` x tokens/seqs) and as a decode step (`seqs` rows at that context), each beside the like kernel of the
    Nirelix (or Zegopel) decoder. frac = algorithmic bytes / time / measured copy bandwidth."""
    from nanovllm import ops
    dev, bf = "cuda", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g)
    H = width // head_dim
    G = max(1, H // 4)
    rows = []

    def add(name, step, fn, nbytes, like=None, like_fn=None, like_bytes=None, flops=None, like_flops=None):
        t = _timed(fn, flush)
        row = {"kernel": name, "step": step, "us": round(t * 1e6, 1), "GB/s": round(nbytes / t / 1e9),
               "frac_of_measured_copy": round(nbytes / t / 1e9 / peak_gbs, 3)}
        if flops:
            row["TFLOP/s"] = round(flops / t / 1e12, 2)
        if like_fn is not None:
            tl = _timed(like_fn, flush)
            row["like"] = {"kernel": like, "us": round(tl * 1e6, 1),
                           "frac_of_measured_copy": round(like_bytes / tl / 1e9 / peak_gbs, 3)}
            if like_flops:
                row["like"]["TFLOP/s"] = round(like_flops / tl / 1e12, 2)
            row["times_as_far_from_roofline_as_like"] = round((like_bytes / tl) / (nbytes / t), 2)
            if flops and like_flops:
                row["times_as_far_from_flop_roofline_as_like"] = round((like_flops / tl) / (flops / t), 2)
        rows.append(row)

    for step, T in (("prompt", tokens), ("decode", seqs)):
        per = T // seqs if step == "prompt" else 1
        ctx = tokens // seqs
        if step == "prompt":
            cu = torch.arange(0, T + 1, per, dtype=torch.int32, device=dev)
            spans = ops.StepSpans(cu, cu, None, per)
        else:
            spans = ops.StepSpans(None, None, torch.full((T,), ctx, dtype=torch.int32, device=dev))
        slots = torch.arange(seqs, dtype=torch.int32, device=dev)
        pos = (torch.arange(T, device=dev) % max(per, 1) + (0 if step == "prompt" else ctx - 1)).contiguous()
        # residual path: layer norm on the sublayer's output + add, beside the add + two RMS norms / the 1-stream form
        y, res, res2 = rnd(T, width).to(bf), rnd(T, width), rnd(T, width)
        w1, w2 = rnd(width), rnd(width)
        add("norm_residual(layer norm on the output)", step, lambda: ops.norm_residual_(res, y, w1, w2, 1e-5, bf),
            T * width * 12, "residual_add_norms", lambda: ops.residual_add_norms_(y, res2, w1, w2, 1e-6), T * width * 12)
        emb, ptab = rnd(32768, width).to(bf), rnd(8192, width).to(bf)
        ids = torch.randint(0, 32768, (T,), device=dev, generator=g)
        add("norm_residual(embedding + position, gathered)", step,
            lambda: ops.norm_residual_(res, emb, w1, w2, 1e-5, bf, accumulate=False, y_index=ids, y2=ptab, y2_index=pos),
            T * width * 10)
        ff = 3 * width
        up = rnd(T, 2 * ff).to(bf)
        up1 = up[:, :ff].contiguous()
        add("act_only(relu squared)", step, lambda: ops.act_only(up1, "relu2"), T * ff * 4,
            "act_and_mul(relu)", lambda: ops.act_and_mul(up, "relu"), T * ff * 6)
        # attention preparation: norms over the whole q and k projections + cache write
        nq, nk = H * head_dim, G * head_dim
        qkv = rnd(T, nq + 2 * nk).to(bf)
        qkv2 = qkv.clone()
        nb = (T + 15) // 16 + 1
        kc = torch.zeros(nb, 16, nk, dtype=bf, device=dev)
        vc = torch.zeros(nb, 16, nk, dtype=bf, device=dev)
        sl = torch.arange(T, dtype=torch.int32, device=dev)
        wq, wk = rnd(nq), rnd(nk)
        prep_bytes = T * (2 * (nq + nk) * 2 + 3 * nk * 2)
        add("rownorm_cache", step, lambda: ops.rownorm_cache(qkv, nq, nk, nk, wq, wk, 1e-5, kc, vc, sl), prep_bytes,
            "unitnorm_temp_cache", lambda: ops.unitnorm_temp_cache(qkv2, pos, 1e-6, 0.1, 1024, H, G, head_dim, head_dim,
                                                                   kc, vc, sl), prep_bytes)
        # the recurrence: gate and query in fp32, then the tied-gate form (like: delta_prep and the delta rule)
        p3 = rnd(T, 3 * nq).to(bf)
        gb, lower = rnd(nq), torch.rand(nq, device=dev, generator=g) * 0.9
        Gd = max(1, H // 2)
        ngk = Gd * head_dim
        qkc = rnd(T, 2 * ngk + nq).to(bf)
        a_in, b_in = rnd(T, nq).to(bf), rnd(T, H).to(bf)
        dtb, alog = rnd(nq), -torch.rand(H, device=dev, generator=g) * 2 - 1
        add("gate_prep", step, lambda: ops.gate_prep(p3[:, :nq], p3[:, nq:2 * nq], gb, lower), T * nq * (4 + 8),
            "delta_prep", lambda: ops.delta_prep(qkc[:, :2 * ngk], a_in, b_in, dtb, alog, H, Gd, head_dim, 1e-6,
                                                 head_dim ** -0.5), T * (2 * ngk * 6 + nq * 6 + H * 6))
        q32, f32 = ops.gate_prep(p3[:, :nq], p3[:, nq:2 * nq], gb, lower)
        dq32, dec, beta = ops.delta_prep(qkc[:, :2 * ngk], a_in, b_in, dtb, alog, H, Gd, head_dim, 1e-6, head_dim ** -0.5)
        st = torch.zeros(seqs + 1, H, head_dim, head_dim, device=dev)
        state_bytes = 2 * seqs * H * head_dim * head_dim * 4 if step == "decode" else 0
        add("linear_recurrence(tied forget gate per channel)", step,
            lambda: ops.linear_recurrence(q32, f32, p3[:, 2 * nq:], spans, H, H, head_dim, head_dim, st, slots,
                                          tied_gate=True), T * nq * (4 + 4 + 2 + 4) + state_bytes,
            "delta_rule", lambda: ops.delta_rule(dq32[:, :ngk], dq32[:, ngk:], qkc[:, 2 * ngk:], dec, beta, spans, H, Gd,
                                                 head_dim, head_dim, st, slots),
            T * (2 * ngk * 4 + nq * 4 + nq * 2 + nq * 4) + state_bytes,
            flops=4.0 * T * H * head_dim * head_dim, like_flops=8.0 * T * H * head_dim * head_dim)
        o32, gate = rnd(T, nq), rnd(T, nq).to(bf)
        ones = torch.ones(nq, device=dev)
        add("gated_norm(a norm per head, no gate)", step,
            lambda: ops.gated_norm(o32, None, ones, 1e-5, groups=H, dtype=bf), T * nq * 6,
            "gated_norm(a norm per head, silu gate)", lambda: ops.gated_norm(o32, gate, ones, 1e-6, groups=H, gate_act="silu"),
            T * nq * 8)
        # attention: heads mixed before the softmax, distance bias, sink, window 512 over paged keys and values
        window = 512
        nbl = seqs * (-(-ctx // 16)) + 1
        kcache = (torch.randn(nbl, 16, nk, device=dev, generator=g) * 0.3).to(bf)
        vcache = (torch.randn(nbl, 16, nk, device=dev, generator=g) * 0.3).to(bf)
        tables = torch.arange(seqs * (-(-ctx // 16)), dtype=torch.int32, device=dev).view(seqs, -1)
        qh = (rnd(T, H, head_dim) * 0.3).to(bf)
        talk = torch.eye(H, device=dev) + 0.1 * rnd(H, H)
        sink = rnd(H)
        slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device=dev)
        keys = min(window, ctx)
        band = sum(min(window, i + 1) for i in range(per)) * seqs if step == "prompt" else T * keys
        R, dr = 4 * head_dim, head_dim // 2
        lcache = (torch.randn(nbl, 16, R + dr, device=dev, generator=g) * 0.3).to(bf)
        qx = (rnd(T, H, R + dr) * 0.3).to(bf)
        from nanovllm.layers.seq_mixers import LatentAttention, MixedHeadAttention
        from nanovllm.utils.context import get_context, reset_context, set_context
        la = LatentAttention(H, head_dim, dr, head_dim, R, 0.07, window=window)
        la.k_cache = lcache
        mh = MixedHeadAttention(H, G, head_dim, head_dim, 0.3, window=window, slope_base=8.0).to(dev)
        mh.talk.data.copy_(talk)
        mh.sink.data.copy_(sink)
        mh.k_cache, mh.v_cache = kcache, vcache
        if step == "prompt":
            set_context(True, cu_seqlens_q=spans.cu_q, cu_seqlens_k=spans.cu_k, max_seqlen_q=per, max_seqlen_k=per,
                        block_tables=tables, block_size=16, host_spans=[(i * per, per, per) for i in range(seqs)])
            like_fn = lambda: la._prefill_by_products(qx, None, get_context(), True)
        else:
            set_context(False, context_lens=spans.ctx_lens, block_tables=tables, block_size=16)
            like_fn = lambda: la._decode_window_by_products(qx, get_context())
        att_bytes = T * 2 * nq * 2 + seqs * min(ctx, keys + per) * 2 * nk * 2
        lat_bytes = T * H * (R + dr + R) * 2 + seqs * min(ctx, keys + per) * (R + dr) * 2
        add("mixed-head attention as the model runs it (window 512)", step, lambda: mh(qh), att_bytes,
            "latent attention by products (window 512)", like_fn, lat_bytes,
            flops=4.0 * band * H * head_dim, like_flops=2.0 * band * H * (2 * R + dr))
        add("mixed_attn kernel alone (window 512)", step,
            lambda: ops.mixed_attn(qh, kcache, vcache, spans, 0.3, G, head_dim, block_tables=tables, window=window,
                                   slopes=slopes, talk=talk, sink=sink), att_bytes,
            "attn_generic(latent rows, window 512)",
            lambda: ops.attn_generic(qx, lcache, None, spans, 0.07, 1, R, block_tables=tables, window=window), lat_bytes,
            flops=4.0 * band * H * head_dim, like_flops=2.0 * band * H * (2 * R + dr))
        reset_context()
        # mixture of experts: router, then experts without a gate (like: the grouped sigmoid router, gated experts)
        E, top, ffe = 16, 2, width // 2
        x = rnd(T, width).to(bf)
        logits = rnd(T, E)
        corr = rnd(E) * 0.1
        add("moe_route_topk", step, lambda: ops.moe_route_topk(logits, corr, top), T * (E * 4 + top * 8),
            "moe_route_grouped", lambda: ops.moe_route_grouped(logits, corr, top, 4, 2, 1.5), T * (E * 4 + top * 8))
        from nanovllm.layers.moe import GroupedSigmoidMoe, TopkSoftmaxMoe
        with torch.device(dev):
            ours, theirs = TopkSoftmaxMoe(width, ffe, E, top).to(bf), GroupedSigmoidMoe(width, ffe, E, top, 4, 2, 1.5).to(bf)
        for m_ in (ours, theirs):
            for p_ in m_.parameters():
                p_.data.copy_((torch.randn(p_.shape, device=dev, generator=g) * 0.03).to(p_.dtype))
            m_.router.data = m_.router.data.float()
        ours.router_bias.data, theirs.correction.data = ours.router_bias.data.float(), theirs.correction.data.float()
        with torch.inference_mode():
            add("mixture of experts without a gate (router + experts)", step, lambda: ours(x),
                2 * E * ffe * width * 2 + T * width * 4,
                "mixture of gated experts (router + experts)", lambda: theirs(x), 3 * E * ffe * width * 2 + T * width * 4,
                flops=4.0 * T * top * ffe * width, like_flops=6.0 * T * top * ffe * width)
    return rows


def nurilorn_kernel_table(width, head_dim, tokens, seqs, peak_gbs):
    """The kernels that the Nurilorn decoder adds or extends, alone, at the layer sizes of a `width`-wide model, as a
    prompt step (`seqs` x tokens/seqs) and as a decode step (`seqs` rows at that context), each beside the like kernel of
    the Zegopel (or Nirelix) decoder. frac = algorithmic bytes / time / measured copy bandwidth."""
    from nanovllm import ops
    from nanovllm.layers.seq_mixers import BandScaledRotary
    dev, bf = "cuda", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g)
    H = width // head_dim
    G = max(1, H // 4)
    rows = []

    def add(name, step, fn, nbytes, like=None, like_fn=None, like_bytes=None, flops=None, like_flops=None):
        t = _timed(fn, flush)
        row = {"kernel": name, "step": step, "us": round(t * 1e6, 1), "GB/s": round(nbytes / t / 1e9),
               "frac_of_measured_copy": round(nbytes / t / 1e9 / peak_gbs, 3)}
        if flops:
            row["TFLOP/s"] = round(flops / t / 1e12, 2)
        if like_fn is not None:
            tl = _timed(like_fn, flush)
            row["like"] = {"kernel": like, "us": round(tl * 1e6, 1),
                           "frac_of_measured_copy": round(like_bytes / tl / 1e9 / peak_gbs, 3)}
            if like_flops:
                row["like"]["TFLOP/s"] = round(like_flops / tl / 1e12, 2)
            row["times_as_far_from_roofline_as_like"] = round((like_bytes / tl) / (nbytes / t), 2)
            if flops and like_flops:
                row["times_as_far_from_flop_roofline_as_like"] = round((like_flops / tl) / (flops / t), 2)
        rows.append(row)

    rot = BandScaledRotary(head_dim // 2, 1e6, True, {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0})
    for step, T in (("prompt", tokens), ("decode", seqs)):
        per = T // seqs if step == "prompt" else 1
        ctx = tokens // seqs
        if step == "prompt":
            cu = torch.arange(0, T + 1, per, dtype=torch.int32, device=dev)
            spans = ops.StepSpans(cu, cu, None, per)
        else:
            spans = ops.StepSpans(None, None, torch.full((T,), ctx, dtype=torch.int32, device=dev))
        # residual path: scaled branch + grouped norm (like: post-norm + add + pre-norm of the Zegopel decoder)
        y, res = rnd(T, width).to(bf), rnd(T, width)
        ls, w1, w2 = rnd(width), rnd(width) * 0.1, rnd(width) * 0.1
        add("residual_scale_groupnorm", step,
            lambda: ops.residual_scale_groupnorm_(res, y, ls, 0.5, w1, 1e-6, 4, bf), T * width * 12,
            "residual_add_norms", lambda: ops.residual_add_norms_(y, res, w1, w2, 1e-6), T * width * 12)
        emb = rnd(32768, width).to(bf)
        ids = torch.randint(0, 32768, (T,), device=dev, generator=g)
        add("residual_scale_groupnorm, embedding looked up", step,
            lambda: ops.residual_scale_groupnorm_(res, emb, None, 32.0, w1, 1e-6, 4, bf, accumulate=False, y_index=ids),
            T * width * 8)
        ff = 3 * width
        gu = rnd(T, 2 * ff).to(bf)
        add("glu_clamped", step, lambda: ops.glu_clamped(gu, 1.702, 7.0), T * ff * 6,
            "act_and_mul(relu)", lambda: ops.act_and_mul(gu, "relu"), T * ff * 6)
        # mixer preparation: rotation by the step's table + value blending + scatter (like: unit norms + temperature + scatter)
        nq, nk = H * head_dim, G * head_dim
        C = nq + 2 * nk
        qkv, other = rnd(T, C).to(bf), rnd(T, nk).to(bf)
        pos = torch.arange(T, device=dev) % max(per, 1) + (0 if step == "prompt" else ctx - 1)
        nb = (T + 15) // 16 + 1
        kc = torch.zeros(nb, 16, nk, dtype=bf, device=dev)
        vc = torch.zeros(nb, 16, nk, dtype=bf, device=dev)
        sl = torch.arange(T, dtype=torch.int32, device=dev)
        lam = torch.full((1,), 0.4, device=dev)
        freq = rot.freq.to(dev)
        tab = ops.rotary_table(pos, freq, rot.magnitude)
        prep_bytes = T * (2 * (nq + nk) * 2 + nk * 2 + 2 * nk * 2)
        add("rope_mix_cache", step,
            lambda: ops.rope_mix_cache(qkv, tab, H, G, head_dim, head_dim, rot.dims, True, other, lam, kc, vc, sl),
            prep_bytes + T * (nk * 2 * 2 + rot.dims * 4),
            "unitnorm_temp_cache",
            lambda: ops.unitnorm_temp_cache(qkv, pos, 1e-6, 0.1, 1024, H, G, head_dim, head_dim, kc, vc, sl), prep_bytes)
        add("rotary_table (once per step)", step, lambda: ops.rotary_table(pos, freq, rot.magnitude), T * (8 + rot.dims * 4))
        o, gl = rnd(T, nq).to(bf), rnd(T, H + 8).to(bf)
        gfull = rnd(T, 2 * nq).to(bf)
        add("head_gate", step, lambda: ops.head_gate_(o, gl[:, :H], H), T * nq * 4,
            "gated_norm(gate alone)", lambda: ops.gated_norm(o, gfull[:, nq:], None, 1e-6), T * nq * 6)
        # attention over a paged cache: the tensor-core kernels with a score cap and a sink (like: the same kernels plain,
        # as the Zegopel decoder runs them), and the generic kernel that fp32 models run
        bs = 64
        per_seq = -(-ctx // bs)
        nblk = seqs * per_seq
        kcache, vcache = rnd(nblk + 1, bs, nk).to(bf), rnd(nblk + 1, bs, nk).to(bf)
        tables = torch.randperm(nblk, device=dev, generator=g).to(torch.int32).view(seqs, per_seq)
        qh = (rnd(T, H, head_dim) * 0.5).to(bf)
        sink = torch.zeros(H, device=dev)
        scale, cap = head_dim ** -0.5, 30.0
        att_bytes = T * 2 * nq * 2 + seqs * ctx * 2 * nk * 2
        if step == "prompt":
            fl = 4.0 * seqs * (per * (per + 1) / 2) * H * head_dim
            fast = lambda **kw: ops.prefill_varlen_attn(qh, kcache, vcache, spans.cu_q, spans.cu_k, per, per, scale, G,
                                                        block_tables=tables, **kw)
            name = "prefill_varlen_attn (tcgen05)"
        else:
            fl = 4.0 * seqs * ctx * H * head_dim
            fast = lambda **kw: ops.paged_decode_attn(qh, kcache, vcache, tables, spans.ctx_lens, scale, G, **kw)
            name = "paged_decode_attn"
        add(name + ", score cap + sink", step, lambda: fast(softcap=cap, sink=sink), att_bytes,
            name + ", plain", lambda: fast(), att_bytes, flops=fl, like_flops=fl)
        add(name + ", sink alone", step, lambda: fast(sink=sink), att_bytes, flops=fl)
        gt = rnd(T, H).to(bf)
        add("attn_generic, score cap + sink + head gate", step,
            lambda: ops.attn_generic(qh, kcache, vcache, spans, scale, G, head_dim, block_tables=tables, softcap=cap,
                                     sink=sink, gate=gt), att_bytes,
            "attn_generic, plain",
            lambda: ops.attn_generic(qh, kcache, vcache, spans, scale, G, head_dim, block_tables=tables), att_bytes,
            flops=fl, like_flops=fl)
        # mixture of experts: the grouped softmax router and experts with the clamped unit (like: the grouped sigmoid
        # router and silu-gated experts of the Nirelix decoder)
        E, top, ffe = 16, 2, width // 2
        x = rnd(T, width).to(bf)
        logits = rnd(T, E)
        corr = rnd(E) * 0.1
        add("moe_route_grouped_softmax", step, lambda: ops.moe_route_grouped_softmax(logits, top, 4, 2),
            T * (E * 4 + top * 8), "moe_route_grouped", lambda: ops.moe_route_grouped(logits, corr, top, 4, 2, 1.5),
            T * (E * 4 + top * 8))
        from nanovllm.layers.moe import GroupedSigmoidMoe, GroupedSoftmaxMoe
        with torch.device(dev):
            ours = GroupedSoftmaxMoe(width, ffe, E, top, 4, 2, glu=(1.702, 7.0)).to(bf)
            theirs = GroupedSigmoidMoe(width, ffe, E, top, 4, 2, 1.5).to(bf)
        for m_ in (ours, theirs):
            for p_ in m_.parameters():
                p_.data.copy_((torch.randn(p_.shape, device=dev, generator=g) * 0.03).to(p_.dtype))
            m_.router.data = m_.router.data.float()
        theirs.correction.data = theirs.correction.data.float()
        moe_bytes = 3 * E * ffe * width * 2 + T * width * 4
        with torch.inference_mode():
            add("mixture of clamped-unit experts (router + experts)", step, lambda: ours(x), moe_bytes,
                "mixture of silu-gated experts (router + experts)", lambda: theirs(x), moe_bytes,
                flops=6.0 * T * top * ffe * width, like_flops=6.0 * T * top * ffe * width)
    return rows


def hybrid_compare(args):
    """--hybrid: the Zegopel presets beside the dense presets of the same width and depth, each through the engine
    (LLM.add_request / LLM.step; prompt steps, then CUDA-graph decode steps), plus the kernel table."""
    from nanovllm import LLM
    K, W, B, ctx = min(args.steps, 64), max(3, args.warmup), min(args.batch, 64), args.ctx
    peak, peak_src = peaks()
    clocks = ClockSampler(0)
    clocks.start()
    clocks.begin()
    out = {"metric": "hybrid_vs_dense_tokens_per_s", "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W,
           "dtype": "bf16", "data": "synthetic (random-init weights, random token ids)",
           "config": {"batch": B, "ctx": ctx, "block_size": args.block_size, "l2": "prompts and caches exceed L2; "
                      "kernel table: 256 MB flush before every timed launch"}, "models": [], "peak_source": peak_src}
    pairs = args.hybrid_pairs or {"nirelix": "nirelix-1k:zegopel-1k,nirelix-2k:zegopel-2k",
                                  "fitevik": "fitevik-1k:nirelix-1k,fitevik-2k:nirelix-2k",
                                  "nurilorn": "nurilorn-1k:zegopel-1k,nurilorn-2k:zegopel-2k"}.get(
        args.design, "zegopel-1k:qwen3-0.6b,zegopel-2k:llama-3.2-1b")
    out["design"] = args.design
    for pair in pairs.split(","):
        for name in pair.split(":"):
            llm = LLM(name, kvcache_block_size=args.block_size, max_num_seqs=B, max_model_len=max(4096, ctx + W + K + 16),
                      max_num_batched_tokens=16384, gpu_memory_utilization=args.mem_util, seed=0)
            decode_workload(llm, Group(1), B, ctx, 4, 3, 1, 0)      # untimed: first-call set-up of every kernel
            while not llm.is_finished():
                llm.step()
            r = decode_workload(llm, Group(1), B, ctx, K, W, 0, 0)
            n_params = sum(p.numel() for p in llm.model_runner.model.parameters())
            out["models"].append({"model": name, "parameters_M": round(n_params / 1e6),
                                  "prefill_tokens_per_s": round(B * ctx / (sum(r["prefill_step_ms"]) / 1e3)),
                                  "prefill_steps": r["prefill_steps"],
                                  "decode_tokens_per_s": round(B * K / r["dev_s"]),
                                  "decode_ms_per_step": round(r["dev_s"] / K * 1e3, 3),
                                  "e2e_decode_tokens_per_s": round(B * K / r["e2e_s"]),
                                  "gpu_launches_per_step": r["launches"] // K})
            release(llm)
            del llm
            torch.cuda.empty_cache()
    table = {"nirelix": nirelix_kernel_table, "fitevik": fitevik_kernel_table,
             "nurilorn": nurilorn_kernel_table}.get(args.design, hybrid_kernel_table)
    out["kernels"] = {"width_1024_head_128": table(1024, 128, 16384, 16, peak),
                      "width_2048_head_64": table(2048, 64, 16384, 16, peak)}
    out["clocks"] = clocks.stop()
    print(json.dumps(out))


def main():
    args = parse_args()
    if args.hybrid:
        hybrid_compare(args)
        return
    if os.environ.get("B200_BENCH_DEBUG"):
        import faulthandler
        faulthandler.dump_traceback_later(int(os.environ["B200_BENCH_DEBUG"]), exit=True)
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the b200 arm has no CPU fallback)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from nanovllm import LLM
    K, W, B, ctx = args.steps, max(3, args.warmup), args.batch, args.ctx
    max_len = ctx + W + K + 16
    clocks = ClockSampler(local)
    clocks.start()
    llm = LLM(args.model, kvcache_block_size=args.block_size, max_num_seqs=B,
              max_model_len=max(4096, max_len), max_num_batched_tokens=16384,
              tensor_parallel_size=world if args.tp else 1, distributed_launch="env",
              gpu_memory_utilization=args.mem_util, kv_cache_dtype=args.kv_cache_dtype, seed=0)
    runner = llm.model_runner
    spec = runner.spec
    group = Group(world)
    dbg(rank, 'engine built')
    group.barrier()
    clocks.begin()
    r = decode_workload(llm, group, B, ctx, K, W, rank if not args.tp else 0, rank)
    peak, peak_src = peaks()
    fp8 = args.kv_cache_dtype != "auto"
    hybrid = runner.kv_cache.dim() != 5      # per-layer caches of a hybrid decoder: no single KV stream to time alone
    roof = None if hybrid else attention_roofline(runner, group, B, K, world if args.tp else 1, fp8, peak, peak_src)
    dbg(rank, 'attn loop done')
    clk = clocks.stop()

    ttfts, dev_s, e2e_s = r["ttfts"], r["dev_s"], r["e2e_s"]
    prefill_s = ttfts[-1] / 1e3
    engines = 1 if args.tp else world
    value = engines * B * K / dev_s
    # KV-read roofline of the whole step at the measured peak (what `value` is bounded by)
    if roof is None:
        roof = {"note": "hybrid decoder: see `bench.py --hybrid` for its kernels' rooflines"}
    else:
        step_kv_bytes = roof["algorithmic_bytes_per_launch"] * roof["layers"] * roof["launches_per_layer"]
        roof["step_kv_roofline_tokens_per_s"] = B / (step_kv_bytes / (peak * 1e9))
        roof["step_frac_of_kv_roofline"] = (B * K / dev_s) / roof["step_kv_roofline_tokens_per_s"]
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_s / K * 1e3, "higher_is_better": True, "scaling": "weak" if not args.tp else "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random-init weights, random token ids)",
        "config": dict(workload_config(args, world), ctx_during_timing=[ctx + W, r["ctx_now"]],
                       decode_step="two micro-batches on two streams in one CUDA graph" if r["two_micro_batches"]
                       else "one batch"),
        "e2e": {"value": engines * B * K / e2e_s, "unit": UNIT, "h2d_bytes_per_step": r["h2d_per"],
                "d2h_bytes_per_step": r["d2h_per"], "ms_per_step": e2e_s / K * 1e3},
        "ttft_p50_ms": ttfts[len(ttfts) // 2], "ttft_max_ms": ttfts[-1], "prefill_steps": r["prefill_steps"],
        "prefill_step_ms": r["prefill_step_ms"], "submit_ms": r["submit_ms"],
        "prefill_tokens_per_s": engines * B * ctx / prefill_s,
        "gpu_launches": r["launches"],
        "roofline": roof,
        "clocks": clk,
    }
    if getattr(spec, "num_experts", 0):
        line["moe_roofline"] = moe_expert_roofline(runner, B, peak)
    dbg(rank, 'before exit')
    del runner
    release(llm)
    dbg(rank, 'after exit')
    if world == 1 and args.model == "qwen3-0.6b":
        try:
            line["prefill_roofline"] = prefill_roofline()
        except Exception as e:            # an extra object: its failure must not cost the contract line
            line["prefill_roofline"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    if world > 1 and not args.tp and not args.no_tp_block:
        # the replicas above say nothing about the collective design: the same run also measures the
        # tensor-parallel path (BASELINE configs[3]) over all `world` GPUs, with its TP=1 comparison
        def bail():                       # a hung collective must not cost the replica line
            line["tp"] = {"error": f"tensor-parallel block did not finish within {args.tp_timeout} s"}
            if rank == 0:
                print(json.dumps(line))
                sys.stdout.flush()
            os._exit(0)
        watchdog = threading.Timer(args.tp_timeout, bail)
        watchdog.daemon = True
        watchdog.start()
        try:
            line["tp"] = tp_block(args, rank, world, K, W, peak, peak_src)
        except Exception as e:            # symmetric failures only (OOM on every rank); reported, not hidden
            line["tp"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        watchdog.cancel()
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.model == "qwen3-0.6b":
        tps, sec, kind, cores = reference_cpu_step(args.cpu_sample_seqs, ctx, args.block_size, 3, 1, False)
        line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": cores, "kind": kind,
                                "sample": cpu_sample_text(kind, args.cpu_sample_seqs, B, ctx, 3, sec)}
        line["config"]["cpu_sample_batch"] = args.cpu_sample_seqs
    if rank == 0:
        print(json.dumps(line))
        sys.stdout.flush()
    if world > 1:
        # everything is measured and printed: a rank that failed inside the tp block must not turn the
        # orderly shutdown into a hang (destroy_process_group itself returns in < 1 s, see
        # profiles/r02_tp_teardown_probe.log)
        closer = threading.Timer(60.0, lambda: os._exit(0))
        closer.daemon = True
        closer.start()
        dist.barrier()
        dist.destroy_process_group()
        closer.cancel()


if __name__ == "__main__":
    main()
