"""-m gpu: the Fitevik decoder (HGRN2 recurrences whose forget gate also decides what is written; attention with a
whole-projection query/key norm, a distance bias, heads mixed before the softmax, a sink and a sliding window, whose
keys and values may be another layer's; a norm on every sublayer's output; plain and mixture feed-forwards with a
squared relu) against tests/fitevik_oracle.py, a plain float64 restatement.

Every test makes its own small configuration and random weights. Models run in true fp32 (the sharp comparison:
relative error of every row of logits below 2e-4) and in bf16 (the serving precision). The schedules are fed through
LLMEngine.step_given -- the scheduler's block manager, the runner's step and the model's kernels -- so what is
compared is the engine, not a forward function. Where random weights would hide a fault (a window's edge, a key far
back, a block border, a sink) the mechanism tests scale one query and key so that one score stands out.
"""
import json
import math
import os
import random

import pytest
import torch

import fitevik_oracle as O

pytestmark = pytest.mark.gpu
F64 = torch.float64


def hgrn2(heads, dim, vdim, mlp=None):
    return {"type": "hgrn2", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def attention(heads, kv, dim, vdim, window, scale, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mlp": mlp, "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config_a():
    """Odd sizes everywhere: 6 query heads over 2 key/value heads with key size 24 and value size 20, a window of 19
    tokens over blocks of 16, a borrower with ANOTHER window (33) and scale, a recurrence with key size 72 (two lanes
    per state column), value size 40 above key size 16, a borrower of a later lender with a window of 7, 6 experts of
    which 3 and 4 of which 1 are chosen, layers without feed-forward."""
    return {"architecture": "Fitevik", "vocab": 211, "width": 88, "norm": {"eps": 1e-5}, "logit_scale": 0.4,
            "max_positions": 400,
            "layers": [hgrn2(3, 20, 28, mlp=dense(72)),
                       attention(6, 2, 24, 20, 19, 0.3, mlp=moe(6, 3, 40)),
                       hgrn2(2, 72, 16),
                       attention(6, 2, 24, 20, 33, 0.2, kv_from=1, mlp=dense(56)),
                       attention(3, 3, 16, 40, 0, 0.25, mlp=moe(4, 1, 24)),
                       attention(3, 3, 16, 40, 7, 0.25, kv_from=4)]}


def config_b():
    """Values that are 1 or equal: one recurrent head, one key/value head, every expert chosen (no discrete choice:
    the strict bf16 comparison), no window entry on the lender, a window equal to the block size on its borrower, key
    size = value size, logit scale 1, width 128."""
    return {"architecture": "Fitevik", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "max_positions": 512,
            "layers": [attention(4, 1, 32, 32, 0, 0.18, mlp=dense(128)),
                       hgrn2(1, 64, 32, mlp=moe(2, 2, 64)),
                       attention(4, 1, 32, 32, 16, 0.18, kv_from=0),
                       hgrn2(4, 32, 48, mlp=dense(64))]}


def config_c():
    """Recurrences only: no layer holds keys or values, blocks only count tokens."""
    return {"architecture": "Fitevik", "vocab": 150, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
            "max_positions": 256,
            "layers": [hgrn2(2, 16, 16, mlp=dense(48)), hgrn2(4, 8, 24, mlp=moe(3, 2, 32))]}


CONFIGS = {"a": config_a, "b": config_b, "c": config_c}
STRICT_BF16 = {"a": False, "b": True, "c": False}
_MODELS = {}


def model_dir(tmp_path_factory, name):
    """(folder with config.json + model.safetensors, config, float64 tensors) of a named test model, made once."""
    if name not in _MODELS:
        from safetensors.torch import save_file
        cfg = CONFIGS[name]()
        tensors = O.random_model(cfg, seed=len(name) + ord(name[0]))
        d = tmp_path_factory.mktemp("fitevik_" + name)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(d, "model.safetensors"))
        _MODELS[name] = (str(d), cfg, O.as_f64(tensors))
    return _MODELS[name]


_ENGINES = {}


def engine(tmp_path_factory, name, dtype, eager=False, blocks=24, block_size=16):
    key = (name, dtype, eager, blocks, block_size)
    if key not in _ENGINES:
        from nanovllm.engine.llm_engine import LLMEngine
        path, cfg, tensors = model_dir(tmp_path_factory, name)
        _ENGINES[key] = LLMEngine(path, dtype=dtype, kvcache_block_size=block_size, num_kvcache_blocks=blocks + 1,
                                  max_num_seqs=4, max_model_len=blocks * block_size,
                                  max_num_batched_tokens=4 * blocks * block_size, return_logits=True,
                                  enforce_eager=eager, chunked_prefill=True)
    return _ENGINES[key], _MODELS[name][1], _MODELS[name][2]


def row_err(got, want):
    """Per row: root mean square of the difference (row means removed) over that of the reference."""
    d = got.to(F64).cpu() - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt()


def close(got, want, dtype, strict=True):
    e = row_err(got, want)
    if dtype == "float32":
        return bool((e < 2e-4).all())
    if strict:
        return float(e.pow(2).mean().sqrt()) < 3e-2 and float(e.max()) < 0.2
    # a model that chooses experts: bf16 rounding may flip a close choice for a token, so a few rows may differ
    return float(e.median()) < 3e-2 and float((e < 0.2).double().mean()) >= 0.9


def tokens_of(cfg, n, seed):
    g = random.Random(seed)
    return [g.randrange(cfg["vocab"]) for _ in range(n)]


def feed(eng, rid, toks, cuts):
    """One request alone, cut at `cuts`; returns logits of every position."""
    outs, lo = [], 0
    for hi in list(cuts) + [len(toks)]:
        if hi <= lo:
            continue
        outs.append(eng.step_given([(rid, toks[lo:hi], list(range(hi - lo)))], [rid] if hi == len(toks) else []))
        lo = hi
    return torch.cat(outs)


CASES = [("a", "float32"), ("a", "bfloat16"), ("b", "float32"), ("b", "bfloat16"), ("c", "float32")]


# ------------------------------------------------------------------ whole prompts, decoding, portions
@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompt_and_layers(tmp_path_factory, name, dtype):
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype)
    toks = tokens_of(cfg, 75, 1)
    want, layers = O.forward(cfg, tensors, toks, return_layers=True)
    model = eng.model_runner.model
    model.trace_layers = []
    try:
        got = feed(eng, "w", toks, [])
        seen = [x.cpu() for x in model.trace_layers]
    finally:
        model.trace_layers = None
    assert len(seen) == len(cfg["layers"])
    if dtype == "float32":
        for i, x in enumerate(seen):                  # the residual stream after every layer
            assert float((x.to(F64) - layers[i]).abs().max() / layers[i].abs().max()) < 2e-4, i
    assert close(got, want, dtype, STRICT_BF16[name])


@pytest.mark.parametrize("name,dtype", CASES[:4])
@pytest.mark.parametrize("eager", [False, True])
def test_prefill_then_token_by_token(tmp_path_factory, name, dtype, eager):
    """Most of a prompt in one step, the rest one token a step (CUDA-graph decode and eager decode): decoded
    positions cross block borders and leave every window behind; a one-token prompt starts from the first token."""
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype, eager)
    toks = tokens_of(cfg, 70, 2)
    want = O.forward(cfg, tensors, toks)
    for first in (1, 2, 29):
        got = feed(eng, "d", toks, range(first, len(toks)))
        assert close(got, want, dtype, STRICT_BF16[name]), first


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_every_size(tmp_path_factory, name, dtype):
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype)
    toks = tokens_of(cfg, 90, 3)
    want = O.forward(cfg, tensors, toks)
    for size in (2, 3, 7, 16, 19, 33):
        got = feed(eng, "p", toks, range(size, len(toks), size))
        assert close(got, want, dtype, STRICT_BF16[name]), size
    g = random.Random(5)
    cuts, at = [], 0
    while at < len(toks):
        at += g.choice([1, 1, 2, 2, 3, 5, 16, 21])
        cuts.append(at)
    got = feed(eng, "p", toks, [c for c in cuts if c < len(toks)])
    assert close(got, want, dtype, STRICT_BF16[name])


@pytest.mark.parametrize("name,dtype", CASES[:4])
def test_unequal_batches_and_reused_slots(tmp_path_factory, name, dtype):
    """Up to four live requests, portions of some beside single tokens of others, requests that sit out a step;
    every request ends at its own time and later ones take over its blocks and state slot (the pool has 12 blocks,
    the seven requests need 23); each must match its own run alone."""
    pool = 12
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype, blocks=pool)
    g = random.Random(7)
    lens = [37, 90, 5, 64, 51, 33, 18]
    reqs = {f"r{i}": tokens_of(cfg, n, 10 + i) for i, n in enumerate(lens)}
    want = {k: O.forward(cfg, tensors, v) for k, v in reqs.items()}
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    waiting, live = list(reqs), []
    bm = eng.scheduler.block_manager
    blocks_of = lambda k: -(-len(reqs[k]) // bm.block_size)
    slots, tables = {}, {}
    while waiting or live:
        while waiting and len(live) < 4 and sum(map(blocks_of, live)) + blocks_of(waiting[0]) <= pool:
            live.append(waiting.pop(0))
        entries, end = [], []
        for k in live:
            if at[k] > 0 and g.random() < 0.15:
                continue                                   # left out of this step, goes on later
            n = min(len(reqs[k]) - at[k], g.choice([1, 1, 1, 2, 3, 11, 24]))
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        if not entries:
            continue
        out = eng.step_given(entries, end)
        row = 0
        for k, t, w in entries:
            got[k].append(out[row:row + len(w)])
            row += len(w)
            if k in eng.scheduler.given:
                slots[k] = eng.scheduler.given[k].state_slot
                tables[k] = list(eng.scheduler.given[k].block_table)
        live = [k for k in live if k not in end]
    assert len(set(slots.values())) <= 4 < len(slots)                            # slots were used again
    assert sum(len(t) for t in tables.values()) > pool                           # and so were blocks
    assert len(bm.free_block_ids) == pool and len(bm.free_state_slots) == 4      # everything was given back
    for k in reqs:
        assert close(torch.cat(got[k]), want[k], dtype, STRICT_BF16[name]), \
            (k, float(row_err(torch.cat(got[k]), want[k]).max()))


def test_long_decoding(tmp_path_factory):
    """300 tokens one by one after a 3-token prompt in fp32: the states are carried 300 times, every window passes
    over decoded tokens only, attention reads 19 blocks through the table; the logits still match."""
    eng, cfg, tensors = engine(tmp_path_factory, "a", "float32", blocks=20)
    toks = tokens_of(cfg, 303, 4)
    want = O.forward(cfg, tensors, toks)
    got = feed(eng, "l", toks, range(3, len(toks)))
    assert float(row_err(got, want).max()) < 2e-4


def test_greedy_generation_through_the_scheduler(tmp_path_factory):
    """LLM.generate (waiting/running queues, prefill steps, graph decode steps, sampling) in fp32 against the
    oracle's greedy continuation, for three prompts of unequal length at once."""
    from nanovllm import LLM, SamplingParams
    path, cfg, tensors = model_dir(tmp_path_factory, "b")
    llm = LLM(path, dtype="float32", kvcache_block_size=16, num_kvcache_blocks=40, max_num_seqs=4, max_model_len=128,
              max_num_batched_tokens=512)
    prompts = [tokens_of(cfg, n, 20 + n) for n in (9, 30, 17)]
    outs = llm.generate(prompts, SamplingParams(temperature=1.0, max_tokens=10, ignore_eos=True, greedy=True),
                        use_tqdm=False)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o["token_ids"]:
            logits = O.forward(cfg, tensors, seq)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) > 1e-3 * float(logits.abs().max()):
                assert tok == int(logits.argmax()), (len(seq), tok)
            seq.append(tok)
    llm.exit()


# ------------------------------------------------------------------ mechanisms alone
def _dev(x, dtype=torch.float32):
    return x.to(dtype).cuda().contiguous()


def _spans(q_lens, k_lens):
    from nanovllm import ops
    cu = lambda v: torch.tensor([0] + list(torch.tensor(v).cumsum(0)), dtype=torch.int32).cuda()
    return ops.StepSpans(cu(q_lens), cu(k_lens), None, max(q_lens))


def _decode_spans(ctx_lens):
    from nanovllm import ops
    return ops.StepSpans(None, None, torch.tensor(ctx_lens, dtype=torch.int32).cuda())


@pytest.mark.parametrize("W,kind", [(37, "layer"), (96, "layer"), (64, "rms")])
def test_norm_on_the_output_then_residual(W, kind):
    """x += norm(y) with weight and bias (or the RMS form), and the gathered form x = norm(table1[i] + table2[j])."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(W)
    rows, eps = 9, 1e-5
    x0, y = torch.randn(rows, W, generator=g, dtype=F64), torch.randn(rows, W, generator=g, dtype=F64) * 3 + 0.5
    w, b = 1 + 0.2 * torch.randn(W, generator=g, dtype=F64), 0.3 * torch.randn(W, generator=g, dtype=F64)
    if kind == "layer":
        want = x0 + O.layer_norm(y, w, b, eps)
    else:
        want = x0 + O.rms_norm(y, 0.5 + w, eps)
    x = _dev(x0)
    h = ops.norm_residual_(x, _dev(y), _dev(w), _dev(b) if kind == "layer" else None, eps, torch.float32, kind=kind,
                           offset=0.5 if kind == "rms" else 0.0)
    assert float((x.cpu().to(F64) - want).abs().max()) < 1e-5
    assert torch.equal(h, x)
    xb = _dev(x0)
    hb = ops.norm_residual_(xb, _dev(y, torch.bfloat16), _dev(w), _dev(b) if kind == "layer" else None, eps,
                            torch.bfloat16, kind=kind, offset=0.5 if kind == "rms" else 0.0)
    assert xb.dtype == torch.float32 and torch.equal(hb, xb.to(torch.bfloat16))          # the stream itself stays fp32
    if kind == "layer":
        tab1, tab2 = torch.randn(20, W, generator=g, dtype=F64), torch.randn(11, W, generator=g, dtype=F64)
        i1 = torch.tensor([3, 19, 0, 7, 7, 12, 1, 5, 18])
        i2 = torch.tensor([0, 1, 10, 3, 4, 5, 6, 2, 9])
        out = torch.full((rows, W), float("nan"), device="cuda")
        ops.norm_residual_(out, _dev(tab1), _dev(w), _dev(b), eps, torch.float32, accumulate=False, y_index=i1.cuda(),
                           y2=_dev(tab2), y2_index=i2.cuda())
        assert float((out.cpu().to(F64) - O.layer_norm(tab1[i1] + tab2[i2], w, b, eps)).abs().max()) < 1e-5


@pytest.mark.parametrize("n", [13, 64, 4096])
def test_squared_relu(n):
    from nanovllm import ops
    x = torch.randn(7, n, generator=torch.Generator().manual_seed(n), dtype=F64)
    got = ops.act_only(_dev(x), "relu2")
    assert float((got.cpu().to(F64) - O.relu_squared(x)).abs().max()) < 1e-5
    gb = ops.act_only(_dev(x, torch.bfloat16), "relu2")
    assert float((gb.cpu().to(F64) - O.relu_squared(x.to(torch.bfloat16).to(F64))).abs().max()) < 0.1


def test_whole_projection_norms_and_cache_write():
    """q over all 5 x 24 columns at once and k over all 2 x 24 (NOT per head), the cache rows at flat slots and at
    (block, offset) pairs; a borrower's queries alone."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(3)
    T, nq, nk, nv, eps = 11, 120, 48, 40, 1e-5
    x = torch.randn(T, nq + nk + nv, generator=g, dtype=F64) * torch.linspace(0.2, 3, nq + nk + nv, dtype=F64)
    wq, wk = 1 + 0.3 * torch.randn(nq, generator=g, dtype=F64), 1 + 0.3 * torch.randn(nk, generator=g, dtype=F64)
    q_want, k_want = O.rms_norm(x[:, :nq], wq, eps), O.rms_norm(x[:, nq:nq + nk], wk, eps)
    per_head = O.rms_norm(x[:, :24], wq[:24], eps)
    assert float((per_head - q_want[:, :24]).abs().max()) > 1e-2          # the two readings differ on this input
    bs = 4
    for pairs in (False, True):
        kc, vc = torch.zeros(8, bs, nk, device="cuda"), torch.zeros(8, bs, nv, device="cuda")
        slot = torch.tensor([5, 9, 30, 2, 3, 17, 18, 19, 20, 0, 27])
        slots = torch.stack([slot // bs, slot % bs], 1).int().cuda().contiguous() if pairs else slot.int().cuda()
        buf = _dev(x)
        ops.rownorm_cache(buf, nq, nk, nv, _dev(wq), _dev(wk), eps, kc, vc, slots)
        assert float((buf[:, :nq].cpu().to(F64) - q_want).abs().max()) < 1e-5
        assert float((buf[:, nq:nq + nk].cpu().to(F64) - k_want).abs().max()) < 1e-5
        assert float((kc.view(-1, nk)[slot.cuda()].cpu().to(F64) - k_want).abs().max()) < 1e-5
        assert float((vc.view(-1, nv)[slot.cuda()].cpu().to(F64) - x[:, nq + nk:]).abs().max()) < 1e-6
        assert int((kc.view(-1, nk).abs().sum(1) > 0).sum()) == T                         # nothing else was written
    only_q = _dev(x[:, :nq])
    ops.rownorm_cache(only_q, nq, 0, 0, _dev(wq), None, eps)
    assert float((only_q.cpu().to(F64) - q_want).abs().max()) < 1e-5


def test_forget_gate_and_query():
    from nanovllm import ops
    g = torch.Generator().manual_seed(4)
    T, n = 6, 44
    p = torch.randn(T, 3 * n, generator=g, dtype=F64) * 3
    bias, lower = torch.randn(n, generator=g, dtype=F64), torch.rand(n, generator=g, dtype=F64)
    buf = _dev(p)
    q32, f32 = ops.gate_prep(buf[:, :n], buf[:, n:2 * n], _dev(bias), _dev(lower))
    f_want = lower + (1 - lower) * torch.sigmoid(p[:, n:2 * n] + bias)
    assert float((q32.cpu().to(F64) - O.silu(p[:, :n])).abs().max()) < 1e-5
    assert float((f32.cpu().to(F64) - f_want).abs().max()) < 1e-6
    assert bool((f32.cpu().to(F64) >= lower - 1e-6).all())
    bb = _dev(p, torch.bfloat16)
    qb, fb = ops.gate_prep(bb[:, :n], bb[:, n:2 * n], _dev(bias), _dev(lower))
    assert qb.dtype == torch.float32 and fb.dtype == torch.float32                        # the gate stays 32-bit


@pytest.mark.parametrize("H,d,dv", [(3, 20, 28), (2, 72, 16), (1, 130, 40), (2, 16, 130), (4, 64, 64)])
@pytest.mark.parametrize("vdtype", [torch.float32, torch.bfloat16])
def test_tied_gate_recurrence_in_portions(H, d, dv, vdtype):
    """S <- diag(f) S + (1 - f) v^T in one span, in portions down to single tokens with the state carried in a slot,
    beside another sequence, and in a slot that another sequence used before."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(H * 1000 + d)
    T = 41
    q = torch.randn(T, H, d, generator=g, dtype=F64)
    f = torch.rand(T, H, d, generator=g, dtype=F64) ** 0.3
    v = torch.randn(T, H, dv, generator=g, dtype=F64).to(vdtype).to(F64)
    want, S_end = O.hgrn2_states(q, f, v)
    qd, fd, vd = _dev(q.view(T, -1)), _dev(f.view(T, -1)), _dev(v.view(T, -1), vdtype)
    state = torch.full((3, H, d, dv), 7.0, device="cuda")                                 # slots hold leftovers
    got = ops.linear_recurrence(qd, fd, vd, _spans([T], [T]), H, H, d, dv, state, torch.tensor([1], dtype=torch.int32).cuda(),
                                tied_gate=True)
    assert float((got.cpu().to(F64).view(T, H, dv) - want).abs().max()) < 1e-4
    assert float((state[1].cpu().to(F64) - S_end).abs().max()) < 1e-4
    slots = torch.tensor([2, 0], dtype=torch.int32).cuda()
    outs, at = [], 0
    for n in (2, 1, 1, 16, 5, 1, 15):                                                     # a second sequence rides along
        other = 3 if at == 0 else 1
        qq = torch.cat([qd[at:at + n], qd[:other]])
        ff = torch.cat([fd[at:at + n], fd[:other]])
        vv = torch.cat([vd[at:at + n], vd[:other]])
        if n == 1 and other == 1:
            spans = _decode_spans([at + 1, 20])
        else:
            spans = _spans([n, other], [at + n, 20 if at else other])
        o = ops.linear_recurrence(qq, ff, vv, spans, H, H, d, dv, state, slots, tied_gate=True)
        outs.append(o[:n])
        at += n
    assert at == T
    assert float((torch.cat(outs).cpu().to(F64).view(T, H, dv) - want).abs().max()) < 1e-4


def test_tied_gate_far_token_survives_and_is_overwritten():
    """A gate of exactly 1 keeps a channel's state for hundreds of tokens; a gate of 0 replaces it at once."""
    from nanovllm import ops
    T, d, dv = 300, 8, 8
    f = torch.ones(T, 1, d, dtype=F64)
    f[0] = 0.0                                        # token 0 is written in full
    f[200, 0, :4] = 0.0                               # token 200 overwrites the first four channels
    v = torch.zeros(T, 1, dv, dtype=F64)
    v[0], v[200] = 1.0, -2.0
    q = torch.ones(T, 1, d, dtype=F64)
    want, _ = O.hgrn2_states(q, f, v)
    got = ops.linear_recurrence(_dev(q.view(T, -1)), _dev(f.view(T, -1)), _dev(v.view(T, -1)), _spans([T], [T]), 1, 1, d, dv,
                                tied_gate=True)
    assert float((got.cpu().to(F64).view(T, 1, dv) - want).abs().max()) < 1e-5
    assert float(got[199, 0]) == 8.0 and float(got[299, 0]) == 4.0 - 8.0


def _attn_case(n, H, G, d, dv, seed, dtype=torch.float32, star=None, gain=6.0):
    """Random q, k, v of one sequence; `star` = (query position, key position, head): that query's head and that key
    are made parallel and long, so that the key stands out wherever it is visible."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n, H, d, generator=g, dtype=F64)
    k = torch.randn(n, G, d, generator=g, dtype=F64)
    v = torch.randn(n, G, dv, generator=g, dtype=F64)
    if star is not None:
        i, j, h = star
        k[j, h // (H // G)] = gain * q[i, h] / q[i, h].norm()
        q[i, h] = gain * q[i, h] / q[i, h].norm()
        v[j, h // (H // G)] = 5.0
    rd = lambda x: x.to(dtype).to(F64)
    return rd(q), rd(k), rd(v)


def _paged(k, v, bs, order):
    """Caches whose blocks are in `order`; returns (k_cache, v_cache, block table [1, n])."""
    n, G, d = k.shape
    dv = v.shape[-1]
    nb = -(-n // bs)
    kc = torch.zeros(max(order) + 2, bs, G * d, dtype=k.dtype)
    vc = torch.zeros(max(order) + 2, bs, G * dv, dtype=v.dtype)
    for b in range(nb):
        rows = slice(b * bs, min(n, (b + 1) * bs))
        kc[order[b], :rows.stop - rows.start] = k[rows].reshape(-1, G * d)
        vc[order[b], :rows.stop - rows.start] = v[rows].reshape(-1, G * dv)
    return kc, vc, torch.tensor([order[:nb]], dtype=torch.int32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_window_edges_in_prompts_and_decoding(dtype):
    """A standout key exactly window - 1 back is seen, one token further it is not: in a whole prompt, in a portion
    that starts inside a block, and for a single decoded token; keys through a shuffled block table."""
    from nanovllm import ops
    H, G, d, dv, n, window, bs = 6, 2, 24, 20, 70, 19, 16
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    talk = torch.eye(H, dtype=F64) + 0.2 * torch.randn(H, H, generator=torch.Generator().manual_seed(1), dtype=F64)
    sink = torch.randn(H, generator=torch.Generator().manual_seed(2), dtype=F64)
    slopes = O.head_slopes(H)
    for back, seen in ((window - 1, True), (window, False)):
        i = 60
        q, k, v = _attn_case(n, H, G, d, dv, 5, dtype, star=(i, i - back, 2))
        want = O.mixed_head_attention(q, k, v, 0.3, window, talk, sink, slopes)
        assert (float(want[i, 2].mean()) > 2.0) == seen                                   # the star decides the output
        kw = dict(window=window, slopes=_dev(torch.tensor(slopes)), talk=_dev(talk), sink=_dev(sink))
        got = ops.mixed_attn(_dev(q, dtype), _dev(k, dtype), _dev(v, dtype), _spans([n], [n]), 0.3, G, dv, **kw)
        assert float((got.cpu().to(F64).view(n, H, dv) - want).abs().max()) < tol
        order = [5, 2, 7, 0, 3]
        kc, vc, table = _paged(k, v, bs, order)
        kc, vc, table = _dev(kc, dtype), _dev(vc, dtype), table.cuda()
        for lo in (53, 59):                                                              # a portion from inside a block
            part = ops.mixed_attn(_dev(q[lo:n], dtype), kc, vc, _spans([n - lo], [n]), 0.3, G, dv, block_tables=table, **kw)
            assert float((part.cpu().to(F64).view(n - lo, H, dv) - want[lo:]).abs().max()) < tol
        one = ops.mixed_attn(_dev(q[i:i + 1], dtype), kc, vc, _decode_spans([i + 1]), 0.3, G, dv, block_tables=table, **kw)
        assert float((one.cpu().to(F64).view(H, dv) - want[i]).abs().max()) < tol


def test_far_key_without_a_window_and_block_borders():
    """Without a window a standout key 500 tokens back is found, also when it is the last row of a block or the
    first row of the next; the first tokens of a sequence see only what exists."""
    from nanovllm import ops
    H, G, d, dv, n, bs = 3, 3, 16, 40, 530, 16
    slopes = None                                                                         # a bias would bury a far key
    for j in (15, 16, 0):
        q, k, v = _attn_case(n, H, G, d, dv, 6 + j, star=(520, j, 1), gain=9.0)
        want = O.mixed_head_attention(q[515:525], k, v, 0.25, 0, None, None, slopes, first_pos=515)
        assert float(want[5, 1].mean()) > 3.0
        kc, vc, table = _paged(k, v, bs, list(range(40))[::-1])
        got = ops.mixed_attn(_dev(q[515:525]), _dev(kc), _dev(vc), _spans([10], [525]), 0.25, G, dv,
                             block_tables=table.cuda())
        assert float((got.cpu().to(F64).view(10, H, dv) - want).abs().max()) < 1e-4
    q, k, v = _attn_case(5, H, G, d, dv, 9)
    want = O.mixed_head_attention(q, k, v, 0.25, 3, None, None, O.head_slopes(H))
    got = ops.mixed_attn(_dev(q), _dev(k), _dev(v), _spans([5], [5]), 0.25, G, dv, window=3,
                         slopes=_dev(torch.tensor(O.head_slopes(H))))
    assert float((got.cpu().to(F64).view(5, H, dv) - want).abs().max()) < 1e-5
    assert float((got[0].cpu().to(F64).view(H, dv) - v[0]).abs().max()) < 1e-5            # token 0 sees itself alone


def test_sink_mixing_and_bias_each_matter():
    """Each of the three additions changes the output, and each matches the oracle alone and together; a large sink
    takes nearly all the weight (the output shrinks towards zero), a very negative one changes nothing."""
    from nanovllm import ops
    H, G, d, dv, n = 4, 2, 32, 32, 45
    g = torch.Generator().manual_seed(11)
    q, k, v = _attn_case(n, H, G, d, dv, 10)
    talk = torch.randn(H, H, generator=g, dtype=F64)
    sink = torch.randn(H, generator=g, dtype=F64)
    slopes = O.head_slopes(H)
    plain = O.mixed_head_attention(q, k, v, 0.2, 0, None, None, None)
    run = lambda **kw: ops.mixed_attn(_dev(q), _dev(k), _dev(v), _spans([n], [n]), 0.2, G, dv, **kw).cpu().to(F64).view(n, H, dv)
    assert float((run() - plain).abs().max()) < 1e-5
    for t, s, b in ((talk, None, None), (None, sink, None), (None, None, slopes), (talk, sink, slopes)):
        want = O.mixed_head_attention(q, k, v, 0.2, 0, t, s, b)
        assert float((want - plain).abs().max()) > 1e-2
        got = run(talk=_dev(t) if t is not None else None, sink=_dev(s) if s is not None else None,
                  slopes=_dev(torch.tensor(b)) if b is not None else None)
        assert float((got - want).abs().max()) < 1e-5
    big = run(sink=_dev(torch.full((H,), 30.0, dtype=F64)))
    assert float(big.abs().max()) < 1e-6
    none = run(sink=_dev(torch.full((H,), -80.0, dtype=F64)))
    assert float((none - plain).abs().max()) < 1e-5


@pytest.mark.parametrize("H,G,d,dv", [(1, 1, 8, 8), (8, 8, 64, 64), (16, 4, 128, 128), (5, 5, 40, 136), (64, 8, 16, 16)])
def test_mixed_attention_sizes_and_batches(H, G, d, dv):
    """Head counts and sizes from one head to 64, value sizes up to 136; three sequences of unequal length in one
    launch, each equal to its own run, as prompt portions and as single tokens."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(H + d)
    talk = torch.eye(H, dtype=F64) + 0.1 * torch.randn(H, H, generator=g, dtype=F64)
    sink = torch.randn(H, generator=g, dtype=F64)
    slopes = O.head_slopes(H)
    lens, window, bs = [21, 3, 34], 12, 8
    cases = [_attn_case(n, H, G, d, dv, 20 + n) for n in lens]
    wants = [O.mixed_head_attention(q, k, v, 0.1, window, talk, sink, slopes) for q, k, v in cases]
    kw = dict(window=window, slopes=_dev(torch.tensor(slopes)), talk=_dev(talk), sink=_dev(sink))
    qs = torch.cat([c[0] for c in cases])
    ks = torch.cat([c[1] for c in cases])
    vs = torch.cat([c[2] for c in cases])
    got = ops.mixed_attn(_dev(qs), _dev(ks), _dev(vs), _spans(lens, lens), 0.1, G, dv, **kw).cpu().to(F64)
    want = torch.cat([w.view(-1, H * dv) for w in wants])
    assert float((got - want).abs().max()) < 1e-4
    # the same through one paged cache, the last token of every sequence as a single-token row
    nb = [-(-n // bs) for n in lens]
    kc = torch.zeros(sum(nb) + 1, bs, G * d, dtype=F64)
    vc = torch.zeros(sum(nb) + 1, bs, G * dv, dtype=F64)
    table = torch.full((3, max(nb)), -1, dtype=torch.int32)
    ids = list(range(sum(nb)))[::-1]
    for s, (q, k, v) in enumerate(cases):
        for b in range(nb[s]):
            blk = ids.pop()
            table[s, b] = blk
            rows = slice(b * bs, min(lens[s], (b + 1) * bs))
            kc[blk, :rows.stop - rows.start] = k[rows].reshape(-1, G * d)
            vc[blk, :rows.stop - rows.start] = v[rows].reshape(-1, G * dv)
    last = torch.stack([c[0][-1] for c in cases])
    one = ops.mixed_attn(_dev(last), _dev(kc), _dev(vc), _decode_spans(lens), 0.1, G, dv, block_tables=table.cuda(), **kw)
    want_last = torch.stack([w[-1].reshape(-1) for w in wants])
    assert float((one.cpu().to(F64) - want_last).abs().max()) < 1e-4


@pytest.mark.parametrize("E,top", [(6, 3), (4, 1), (2, 2), (64, 8), (130, 16)])
def test_topk_router_softmax_over_the_chosen(E, top):
    from nanovllm import ops
    g = torch.Generator().manual_seed(E)
    T, W = 50, 24
    u = torch.randn(T, W, generator=g, dtype=F64)
    wr, br = torch.randn(E, W, generator=g, dtype=F64), torch.randn(E, generator=g, dtype=F64) * 2
    idx, wt = O.route(u, wr, br, top)
    z = _dev(u @ wr.T)
    ids, w = ops.moe_route_topk(z, _dev(br), top)
    assert torch.equal(ids.cpu().long(), idx)                                             # the bias takes part in the choice
    assert float((w.cpu().to(F64) - wt).abs().max()) < 1e-5
    assert float((w.sum(1) - 1).abs().max()) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,ff,E,top,tokens", [(88, 40, 6, 3, 150), (128, 64, 4, 4, 33), (64, 24, 3, 1, 7),
                                               (256, 128, 8, 2, 700)])
def test_mixture_without_a_gate(W, ff, E, top, tokens, dtype):
    from nanovllm.layers.moe import TopkSoftmaxMoe
    g = torch.Generator().manual_seed(W + E)
    rd = lambda x: x.to(dtype).to(F64)
    u = rd(torch.randn(tokens, W, generator=g, dtype=F64))
    w = {"router": torch.randn(E, W, generator=g, dtype=F64) * 0.5, "router.b": torch.randn(E, generator=g, dtype=F64)}
    for e in range(E):
        w[f"e{e}.up"] = rd(torch.randn(ff, W, generator=g, dtype=F64) / math.sqrt(W))
        w[f"e{e}.down"] = rd(torch.randn(W, ff, generator=g, dtype=F64) / math.sqrt(ff))
    want = O.moe_ff(u, moe(E, top, ff), w)
    with torch.device("cuda"):
        m = TopkSoftmaxMoe(W, ff, E, top).to(dtype)
    m.router.data = _dev(w["router"])
    m.router_bias.data = _dev(w["router.b"])
    for e in range(E):
        m.w1.data[e] = _dev(w[f"e{e}.up"], dtype)
        m.w2.data[e] = _dev(w[f"e{e}.down"], dtype)
    with torch.inference_mode():
        got = m(_dev(u, dtype)).cpu().to(F64)
    rel = (got - want).norm(dim=1) / want.norm(dim=1)
    if dtype == torch.float32:
        assert float(rel.max()) < 1e-4
    else:
        assert float(rel.median()) < 2e-2 and float(rel.max()) < 0.1


@pytest.mark.parametrize("H,dv", [(3, 28), (2, 16), (4, 64), (1, 130)])
def test_norm_per_head_without_a_gate(H, dv):
    from nanovllm import ops
    g = torch.Generator().manual_seed(dv)
    y = torch.randn(13, H, dv, generator=g, dtype=F64) * 4
    w = 1 + 0.3 * torch.randn(dv, generator=g, dtype=F64)
    want = O.rms_norm(y, w, 1e-5).view(13, H * dv)
    got = ops.gated_norm(_dev(y.view(13, -1)), None, _dev(w.repeat(H)), 1e-5, groups=H, dtype=torch.float32)
    assert float((got.cpu().to(F64) - want).abs().max()) < 1e-5
    gb = ops.gated_norm(_dev(y.view(13, -1)), None, _dev(w.repeat(H)), 1e-5, groups=H, dtype=torch.bfloat16)
    assert gb.dtype == torch.bfloat16 and float((gb.cpu().to(F64) - want).abs().max()) < 0.05


def _mixed_module(H, G, d, dv, scale, window, seed):
    from nanovllm.layers.seq_mixers import MixedHeadAttention
    g = torch.Generator().manual_seed(seed)
    attn = MixedHeadAttention(H, G, d, dv, scale, window=window, slope_base=8.0).cuda()
    talk = torch.eye(H, dtype=F64) + 0.2 * torch.randn(H, H, generator=g, dtype=F64)
    sink = torch.randn(H, generator=g, dtype=F64)
    attn.talk.data.copy_(talk)
    attn.sink.data.copy_(sink)
    return attn, talk, sink


def test_prompts_on_library_products():
    """Prompt portions of a 16-bit model run as library products around the mixed softmax kernel: a 150-token portion
    that continues 60 cached tokens (three query chunks of 64, key ranges that start inside the window), a second whole
    sequence and a short portion beside them (which runs on the kernel), over a shuffled block table; a standout key
    at the window's edge of a query in the second chunk; grouped heads with a value size other than the key size."""
    from nanovllm.utils.context import get_context, reset_context, set_context
    dtype, window, H, G, d, dv, bs = torch.bfloat16, 19, 6, 2, 24, 20, 16
    lens, starts = [210, 100, 30], [60, 0, 21]                # tokens in all, tokens already cached
    star_q, star_h = 140, 4
    attn, talk, sink = _mixed_module(H, G, d, dv, 0.3, window, 1)
    attn.PRODUCT_CHUNK = 64
    cases = [_attn_case(n, H, G, d, dv, 30 + i, dtype, star=(star_q, star_q - window + 1, star_h) if i == 0 else None)
             for i, n in enumerate(lens)]
    wants = [O.mixed_head_attention(q[s:], k, v, 0.3, window, talk, sink, O.head_slopes(H), first_pos=s)
             for (q, k, v), s in zip(cases, starts)]
    assert float(wants[0][star_q - starts[0], star_h].mean()) > 2.0
    nb = sum(-(-n // bs) for n in lens)
    order = list(range(nb))
    random.Random(3).shuffle(order)
    attn.k_cache = torch.zeros(nb + 1, bs, G * d, dtype=dtype, device="cuda")
    attn.v_cache = torch.zeros(nb + 1, bs, G * dv, dtype=dtype, device="cuda")
    tables, at = [], 0
    for (q, k, v), n in zip(cases, lens):
        blocks = order[at:at + -(-n // bs)]
        at += len(blocks)
        tables.append(blocks + [-1] * (14 - len(blocks)))
        for j in range(n):
            attn.k_cache[blocks[j // bs], j % bs] = k[j].reshape(-1).to(dtype)
            attn.v_cache[blocks[j // bs], j % bs] = v[j].reshape(-1).to(dtype)
    q_lens = [n - s for n, s in zip(lens, starts)]
    cu_q = [0] + list(torch.tensor(q_lens).cumsum(0).tolist())
    cu_k = [0] + list(torch.tensor(lens).cumsum(0).tolist())
    dev_i32 = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    qx = torch.cat([c[0][s:] for c, s in zip(cases, starts)]).to(dtype).cuda()
    want = torch.cat([w.view(-1, H * dv) for w in wants])
    set_context(True, cu_seqlens_q=dev_i32(cu_q), cu_seqlens_k=dev_i32(cu_k), max_seqlen_q=max(q_lens),
                max_seqlen_k=max(lens), block_tables=dev_i32(tables), block_size=bs,
                host_spans=[(cu_q[i], q_lens[i], lens[i]) for i in range(3)])
    try:
        got = attn._prefill_by_products(qx, None, None, get_context(), True).cpu().to(F64)
        through = attn(qx).cpu().to(F64)                      # the module takes the same path by itself
        attn.force_generic = True
        plain = attn(qx).cpu().to(F64)
    finally:
        reset_context()
    assert float((got - want).abs().max()) < 3e-2 and torch.equal(got, through)
    assert float((plain - want).abs().max()) < 3e-2
    row = star_q - starts[0]
    assert float(got.view(-1, H, dv)[row, star_h].mean()) > 2.0 > float(got.view(-1, H, dv)[row + 1, star_h].mean())


@pytest.mark.parametrize("window", [19, 200])
def test_decode_rows_inside_a_window_on_library_products(window):
    """Decode steps of a 16-bit model gather each sequence's last `window` key and value rows: sequences shorter than
    the window, exactly at it, with a standout key just inside and just outside, and a padded row (0 keys) in one
    launch; a window wider than what a block table can hold (200 > 5 blocks of 16) gathers the table's capacity."""
    from nanovllm.utils.context import get_context, reset_context, set_context
    dtype, H, G, d, dv, bs, star = torch.bfloat16, 4, 2, 16, 24, 16, 37
    attn, talk, sink = _mixed_module(H, G, d, dv, 0.3, window, 2)
    q, k, v = _attn_case(80, H, G, d, dv, 40, dtype)
    at = [4, 18, 19, star + 18, star + 19, 79]                                      # positions of the decoded tokens
    for i in (star + 18, star + 19):                                                # both queries point at the star key
        q[i, 1] = 6.0 * k[star, 0] / k[star, 0].norm()
    k[star, 0] = 6.0 * k[star, 0] / k[star, 0].norm()
    v[star, 0] = 5.0
    q, k, v = (x.to(dtype).to(F64) for x in (q, k, v))
    want = O.mixed_head_attention(q, k, v, 0.3, window, talk, sink, O.head_slopes(H))
    table = [7, 2, 5, 0, 3]
    attn.k_cache = torch.zeros(9, bs, G * d, dtype=dtype, device="cuda")
    attn.v_cache = torch.zeros(9, bs, G * dv, dtype=dtype, device="cuda")
    for j in range(80):
        attn.k_cache[table[j // bs], j % bs] = k[j].reshape(-1).to(dtype)
        attn.v_cache[table[j // bs], j % bs] = v[j].reshape(-1).to(dtype)
    ctx_lens = [p + 1 for p in at] + [0]
    qx = torch.cat([q[at], torch.zeros(1, H, d, dtype=F64)]).to(dtype).cuda()
    tables = torch.tensor([table] * 6 + [[-1] * 5], dtype=torch.int32).cuda()
    set_context(False, context_lens=torch.tensor(ctx_lens, dtype=torch.int32).cuda(), block_tables=tables, block_size=bs)
    try:
        got = attn._decode_window_by_products(qx, get_context()).cpu().to(F64).view(-1, H, dv)
        through = attn(qx).cpu().to(F64).view(-1, H, dv)
        attn.force_generic = True
        plain = attn(qx).cpu().to(F64).view(-1, H, dv)
    finally:
        reset_context()
    assert float((got[:6] - want[at]).abs().max()) < 3e-2 and torch.equal(got, through)
    assert float((plain[:6] - want[at]).abs().max()) < 3e-2
    assert float(got[6].abs().max()) == 0.0
    if window == 19:
        assert float(got[3, 1].mean()) > 2.0 > float(got[4, 1].mean())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rows_by_slot_regrouped_per_head(dtype):
    """The gather that feeds the batched products: rows picked by slot (repeats, any order) land as [entries, G, keys,
    size]; from a cache and from a row-strided view of packed rows; sizes that rule out 16-byte copies take the fallback."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(7)
    for G, size, extra in ((2, 24, 40), (4, 64, 0), (3, 5, 3)):
        rows = 57
        wide = torch.randn(rows, extra + G * size, generator=g).to(dtype).cuda()
        src = wide[:, extra:].unflatten(1, (G, size))                       # a view whose rows are `extra` apart
        slots = torch.randint(0, rows, (3 * 11,), generator=g).cuda()
        got = ops.gather_rows_by_head(src, slots, 3, 11)
        want = src[slots].view(3, 11, G, size).permute(0, 2, 1, 3)
        assert got.shape == (3, G, 11, size) and torch.equal(got, want)
