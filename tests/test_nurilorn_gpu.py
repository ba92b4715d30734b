"""-m gpu: the Nurilorn decoder (attention behind short convolutions, rotary positions stretched band by band, values
blended with an earlier layer's, capped scores, a sink in the softmax denominator and a gate per head; branches scaled
per channel onto an fp32 residual with RMS norms in groups; dense and mixture feed-forwards with a clamped gated unit,
the mixture behind a softmax router with group-limited choice) against tests/nurilorn_oracle.py, a plain float64
restatement.

Every test makes its own small configuration and random weights. Models run in true fp32 (the sharp comparison:
relative error of every row of logits below 2e-4) and in bf16 (the serving precision). The schedules are fed through
LLMEngine.step_given -- the scheduler's block manager, the runner's step and the model's kernels -- so what is
compared is the engine, not a forward function. Where random weights would hide a fault (a key far back, a block
border, the sink, the first tokens) the mechanism tests scale one query and key so that one score stands out, or make
all scores tiny so that the sink's share of the denominator shows.
"""
import json
import math
import os
import random

import pytest
import torch

import nurilorn_oracle as O

pytestmark = pytest.mark.gpu
F64 = torch.float64


def rot(dims, base=10000.0, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def layer(heads, kv, dim, vdim, rt, conv=3, scale=0.2, softcap=8.0, v_mix=True, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "rot": rt, "scale": scale,
                      "softcap": softcap, "v_mix": v_mix}}


def dense(ff, limit=1.2):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, count=1, keep=1, limit=2.0):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def config_a():
    """Odd sizes everywhere: 6 query heads over 2 key/value heads with key size 24 and value size 20, 16 rotated columns
    stretched by 8 over a short original length, three norm groups of 32, five taps; the first layer does not blend (so
    the first blending layer is the second one) and has other head sizes; 6 experts in 3 groups of which 2 stay and 3
    experts are chosen, 4 experts of which 1; a layer without feed-forward."""
    r = rot(16, 5000.0, (8.0, 48, 6.0, 1.5))
    return {"architecture": "Nurilorn", "vocab": 211, "width": 96, "norm": {"eps": 1e-5, "groups": 3},
            "embedding": {"scale": 7.0}, "residual_mult": 0.6, "logit_scale": 0.4,
            "layers": [layer(3, 3, 16, 40, rot(8, 300.0), conv=2, v_mix=False, mlp=dense(72)),
                       layer(6, 2, 24, 20, r, conv=5, mlp=moe(6, 3, 40, 3, 2)),
                       layer(6, 2, 24, 20, r, conv=5, softcap=3.0),
                       layer(4, 2, 12, 20, rot(12, 5000.0), conv=3, scale=0.5, mlp=moe(4, 1, 24, 2, 2, limit=0.7)),
                       layer(6, 1, 24, 40, r, conv=4, v_mix=False, mlp=dense(56, limit=0.5))]}


def config_b():
    """Values that are 1 or equal: one key/value head, one norm group, one tap, every column rotated, no stretch, no
    cap, unit multipliers, every expert chosen from a single group (no discrete choice: the strict bf16 comparison),
    key size = value size."""
    r = rot(32, 10000.0)
    return {"architecture": "Nurilorn", "vocab": 320, "width": 128, "norm": {"eps": 1e-6, "groups": 1},
            "embedding": {"scale": 1.0}, "residual_mult": 1.0, "logit_scale": 1.0,
            "layers": [layer(4, 1, 32, 32, r, conv=1, softcap=0.0, scale=0.18, mlp=dense(128, limit=7.0)),
                       layer(4, 1, 32, 32, r, conv=1, softcap=0.0, scale=0.18, mlp=moe(2, 2, 64)),
                       layer(4, 1, 32, 32, r, conv=4, softcap=50.0, scale=0.18, mlp=dense(64))]}


def config_c():
    """The sizes that 16-bit models run on the tensor cores: six heads of 64 over two key/value heads, 48 of the
    columns rotated, experts of 128 behind a router of 8 in 2 groups of which one stays."""
    r = rot(48, 5e5, (2.5, 300, 16.0, 2.0))
    return {"architecture": "Nurilorn", "vocab": 410, "width": 384, "norm": {"eps": 1e-5, "groups": 3},
            "embedding": {"scale": 5.0}, "residual_mult": 0.7, "logit_scale": 0.8,
            "layers": [layer(6, 2, 64, 64, r, conv=3, scale=0.11, softcap=20.0, mlp=dense(192)),
                       layer(6, 2, 64, 64, r, conv=3, scale=0.11, softcap=20.0, mlp=moe(8, 2, 128, 2, 1))]}


def config_d():
    """Nothing is a multiple of 8: width 100 in five norm groups, five heads of 10 (6 rotated) with values of 6, 50- and
    18-wide feed-forwards, three experts of which one is chosen, 135 projection columns per token."""
    r = rot(6, 777.0, (3.0, 20, 4.0, 0.5))
    return {"architecture": "Nurilorn", "vocab": 97, "width": 100, "norm": {"eps": 1e-4, "groups": 5},
            "embedding": {"scale": 3.0}, "residual_mult": 0.8, "logit_scale": 1.5,
            "layers": [layer(5, 5, 10, 6, r, conv=3, scale=0.4, softcap=5.0, mlp=dense(50)),
                       layer(5, 5, 10, 6, r, conv=3, scale=0.4, softcap=5.0, mlp=moe(3, 1, 18))]}


CONFIGS = {"a": config_a, "b": config_b, "c": config_c, "d": config_d}
STRICT_BF16 = {"a": False, "b": True, "c": False, "d": False}
_MODELS = {}


def model_dir(tmp_path_factory, name):
    """(folder with config.json + model.safetensors, config, tensors) of a named test model, made once."""
    if name not in _MODELS:
        from safetensors.torch import save_file
        cfg = CONFIGS[name]()
        tensors = O.random_weights(cfg, seed=len(name) + ord(name[0]))
        d = tmp_path_factory.mktemp("nurilorn_" + name)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(d, "model.safetensors"))
        _MODELS[name] = (str(d), cfg, tensors)
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


CASES = [("a", "float32"), ("a", "bfloat16"), ("b", "float32"), ("b", "bfloat16"), ("c", "float32"), ("c", "bfloat16"),
         ("d", "float32"), ("d", "bfloat16")]


# ------------------------------------------------------------------ whole prompts, decoding, portions
@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompt_and_layers(tmp_path_factory, name, dtype):
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype)
    toks = tokens_of(cfg, 75, 1)
    layers = []
    want, _ = O.forward(cfg, tensors, toks, layers_out=layers)
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


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("eager", [False, True])
def test_prefill_then_token_by_token(tmp_path_factory, name, dtype, eager):
    """Most of a prompt in one step, the rest one token a step (CUDA-graph decode and eager decode): decoded positions
    cross block borders, the convolution tails and the blended values are carried token by token; a one-token prompt
    starts from the first token, where the sink is the only other entry of the softmax."""
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype, eager)
    toks = tokens_of(cfg, 70, 2)
    want, _ = O.forward(cfg, tensors, toks)
    for first in (1, 2, 29):
        got = feed(eng, "d", toks, range(first, len(toks)))
        assert close(got, want, dtype, STRICT_BF16[name]), first


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_every_size(tmp_path_factory, name, dtype):
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype)
    toks = tokens_of(cfg, 90, 3)
    want, _ = O.forward(cfg, tensors, toks)
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


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_and_reused_slots(tmp_path_factory, name, dtype):
    """Up to four live requests, portions of some beside single tokens of others, requests that sit out a step;
    every request ends at its own time and later ones take over its blocks and state slot (the pool has 12 blocks,
    the seven requests need 23); each must match its own run alone."""
    pool = 12
    eng, cfg, tensors = engine(tmp_path_factory, name, dtype, blocks=pool)
    g = random.Random(7)
    lens = [37, 90, 5, 64, 51, 33, 18]
    reqs = {f"r{i}": tokens_of(cfg, n, 10 + i) for i, n in enumerate(lens)}
    want = {k: O.forward(cfg, tensors, v)[0] for k, v in reqs.items()}
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
    """300 tokens one by one after a 3-token prompt in fp32: tails and blended values are carried 300 times, attention
    reads 19 blocks through the table, the rotation reaches positions far past the original length; the logits match."""
    eng, cfg, tensors = engine(tmp_path_factory, "a", "float32", blocks=20)
    toks = tokens_of(cfg, 303, 4)
    want, _ = O.forward(cfg, tensors, toks)
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
            logits = O.forward(cfg, tensors, seq)[0][-1]
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


@pytest.mark.parametrize("W,groups", [(37, 1), (96, 3), (64, 4), (90, 5), (512, 4), (2048, 8)])
def test_scaled_branch_and_grouped_norm(W, groups):
    """x += c * scale * y and the norm in groups, for widths that take the 16-byte form and widths that do not; the
    embedding lookup times a constant; a norm without a new branch."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(W)
    rows, eps, c = 9, 1e-5, 0.6
    x0, y = torch.randn(rows, W, generator=g, dtype=F64) * 2, torch.randn(rows, W, generator=g, dtype=F64) * 3 + 0.5
    x0[:, :W // groups] *= 30.0                                        # one group far louder than the others
    ls, w = 1 + 0.3 * torch.randn(W, generator=g, dtype=F64), 1 + 0.2 * torch.randn(W, generator=g, dtype=F64)
    want_x = x0 + c * (y * ls)
    want_h = O.grouped_rms_norm(want_x, w, groups, eps)
    x = _dev(x0)
    h = ops.residual_scale_groupnorm_(x, _dev(y), _dev(ls), c, _dev(w), eps, groups, torch.float32)
    assert float((x.cpu().to(F64) - want_x).abs().max()) < 1e-4
    assert float((h.cpu().to(F64) - want_h).abs().max()) < 1e-5
    if groups > 1:                                                     # one norm over the whole row is another result
        assert float((want_h - O.grouped_rms_norm(want_x, w, 1, eps)).abs().max()) > 0.1
    xb = _dev(x0)
    hb = ops.residual_scale_groupnorm_(xb, _dev(y, torch.bfloat16), _dev(ls), c, _dev(w), eps, groups, torch.bfloat16)
    assert xb.dtype == torch.float32 and hb.dtype == torch.bfloat16          # the stream itself stays fp32
    yb = y.to(torch.bfloat16).to(F64)
    assert float((xb.cpu().to(F64) - (x0 + c * (yb * ls))).abs().max()) < 1e-4
    # the scaled embedding: a table lookup, no earlier stream, then the norm
    table = torch.randn(20, W, generator=g, dtype=F64)
    idx = torch.tensor([3, 19, 0, 7, 7, 12, 1, 5, 18])
    out = torch.full((rows, W), float("nan"), device="cuda")
    h2 = ops.residual_scale_groupnorm_(out, _dev(table), None, 16.0, _dev(w), eps, groups, torch.float32,
                                       accumulate=False, y_index=idx.cuda())
    assert float((out.cpu().to(F64) - 16.0 * table[idx]).abs().max()) < 1e-5
    assert float((h2.cpu().to(F64) - O.grouped_rms_norm(16.0 * table[idx], w, groups, eps)).abs().max()) < 1e-5
    # the norm alone
    h3 = ops.residual_scale_groupnorm_(x, None, None, 1.0, _dev(w), eps, groups, torch.float32)
    assert torch.equal(h3, h)


@pytest.mark.parametrize("scaling", [None, (4.0, 64, 8.0, 1.0), (16.0, 1000, 40.0, 0.5), (2.0, 8, 1.0, 1.0)])
@pytest.mark.parametrize("dims,dim", [(8, 8), (16, 24), (6, 10), (64, 64)])
def test_band_scaled_rotation(scaling, dims, dim):
    """The frequency table against the restatement (ramp ends, a ramp of zero width, no stretch), the rotation of the
    first `dims` columns in neighbouring pairs at positions up to a million (fp64 angles), the columns that pass."""
    from nanovllm import ops
    from nanovllm.layers.seq_mixers import BandScaledRotary
    r = rot(dims, 1e4, scaling)
    f, mag = O.yarn_frequencies(r)
    br = BandScaledRotary(dims, 1e4, True, r.get("scaling"))
    assert float((br.freq - f).abs().max()) < 1e-15 and abs(br.magnitude - mag) < 1e-15
    H, G, dv, T = 3, 1, 8, 7                                           # dims 6 / dim 10 takes the scalar form, the others 16 bytes
    g = torch.Generator().manual_seed(dims)
    pos = torch.tensor([0, 1, 2, 63, 64, 4097, 1000003])
    qkv = torch.randn(T, H * dim + G * dim + G * dv, generator=g, dtype=F64)
    table = ops.rotary_table(pos.cuda(), br.freq.cuda(), br.magnitude)
    got = ops.rope_mix_cache(_dev(qkv), table, H, G, dim, dv, dims).cpu().to(F64)
    want_q = O.rotate(qkv[:, :H * dim].reshape(T, H, dim), pos, r)
    want_k = O.rotate(qkv[:, H * dim:(H + G) * dim].reshape(T, G, dim), pos, r)
    assert float((got[:, :H * dim].reshape(T, H, dim) - want_q).abs().max()) < 2e-6 * mag * 4
    assert float((got[:, H * dim:(H + G) * dim].reshape(T, G, dim) - want_k).abs().max()) < 2e-6 * mag * 4
    assert torch.equal(got[:, (H + G) * dim:], qkv[:, (H + G) * dim:].float().to(F64))       # values untouched
    if dims < dim:
        assert torch.equal(got[:, dims:dim], qkv[:, dims:dim].float().to(F64))               # columns that pass


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dv,skip", [(12, 5), (16, 8)])
def test_value_blending_and_cache_rows(dtype, dv, skip):
    """v <- (1 - lambda) v + lambda v_other in place, rotated k and blended v at their slots (flat, and (block, offset)
    pairs; a negative slot writes nothing); a layer that does not blend stores its values as they are. Value size 12
    behind an unaligned view takes the scalar form, 16 behind an aligned one the 16-byte form."""
    from nanovllm import ops
    H, G, d, T, bs = 4, 2, 16, 6, 4
    g = torch.Generator().manual_seed(1)
    qkv = torch.randn(T, (H + G) * d + G * dv, generator=g, dtype=F64).to(dtype)
    other = torch.randn(T, G * dv + skip, generator=g, dtype=F64).to(dtype)[:, skip:]          # a row-strided view
    lam = torch.tensor([0.3], dtype=torch.float32)
    pos = torch.arange(10, 10 + T)
    r = rot(8, 100.0)
    table = ops.rotary_table(pos.cuda(), O.yarn_frequencies(r)[0].cuda(), 1.0)
    slots = torch.tensor([5, 2, -1, 11, 0, 7], dtype=torch.int32)
    for paired in (False, True):
        kc = torch.zeros(3, bs, G * d, dtype=dtype, device="cuda")
        vc = torch.zeros(3, bs, G * dv, dtype=dtype, device="cuda")
        x = qkv.cuda().clone()
        sl = torch.stack([slots // bs, slots % bs], 1).contiguous() if paired else slots
        sl = sl.clone()
        if paired:
            sl[2] = torch.tensor([-1, 0])
        ops.rope_mix_cache(x, table, H, G, d, dv, 8, True, v_other=other.cuda(), lam=lam.cuda(), k_cache=kc, v_cache=vc,
                           slots=sl.cuda())
        want_v = ((1 - 0.3) * qkv[:, (H + G) * d:].to(F64) + 0.3 * other.to(F64))
        want_k = O.rotate(qkv[:, H * d:(H + G) * d].to(F64).reshape(T, G, d), pos, r).reshape(T, G * d)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert float((x[:, (H + G) * d:].cpu().to(F64) - want_v).abs().max()) < tol
        for t in range(T):
            s = int(slots[t])
            if s < 0:
                continue
            assert torch.equal(vc.view(-1, G * dv)[s], x[t, (H + G) * d:])                    # what is cached is the blend
            assert torch.equal(kc.view(-1, G * d)[s], x[t, H * d:(H + G) * d])
            assert float((kc.view(-1, G * d)[s].cpu().to(F64) - want_k[t]).abs().max()) < tol
        assert int((kc.view(-1, G * d).abs().sum(1) > 0).sum()) == 5                           # the negative slot wrote nothing
    vc = torch.zeros(3, bs, G * dv, dtype=dtype, device="cuda")
    kc = torch.zeros(3, bs, G * d, dtype=dtype, device="cuda")
    x = qkv.cuda().clone()
    ops.rope_mix_cache(x, table, H, G, d, dv, 8, True, k_cache=kc, v_cache=vc, slots=slots.cuda())
    assert torch.equal(x[:, (H + G) * d:], qkv[:, (H + G) * d:].cuda())
    assert torch.equal(vc.view(-1, G * dv)[5], qkv[0, (H + G) * d:].cuda())


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


def _attention_module(H, G, d, dv, scale, softcap, dtype, kc=None, vc=None):
    from nanovllm.layers.seq_mixers import VarSizeAttention
    m = VarSizeAttention(H, G, d, dv, scale, softcap=softcap, sink=0.0).cuda()
    if kc is not None:
        m.k_cache, m.v_cache = kc.to(dtype).cuda(), vc.to(dtype).cuda()
    return m


def _run_attention(m, q, k, v, dtype, q_lens=None, k_lens=None, ctx_lens=None, table=None, bs=16, gate=None):
    """The attention block as a layer calls it, under a step context made by hand."""
    from nanovllm.utils.context import reset_context, set_context
    dev = lambda x: x.to(dtype).cuda().contiguous()
    if ctx_lens is None:
        cu = lambda x: torch.tensor([0] + list(torch.tensor(x).cumsum(0)), dtype=torch.int32).cuda()
        spans, at = [], 0
        for ql, kl in zip(q_lens, k_lens):
            spans.append((at, ql, kl))
            at += ql
        set_context(True, cu(q_lens), cu(k_lens), max(q_lens), max(k_lens), block_tables=table, block_size=bs,
                    host_spans=spans)
    else:
        set_context(False, context_lens=torch.tensor(ctx_lens, dtype=torch.int32).cuda(), block_tables=table, block_size=bs)
    try:
        return m(dev(q), dev(k), dev(v), gate=None if gate is None else dev(gate)).cpu().to(F64)
    finally:
        reset_context()


SHAPES = [(6, 2, 24, 20), (5, 5, 48, 32), (4, 2, 64, 64), (8, 1, 128, 128), (3, 3, 16, 40)]


@pytest.mark.parametrize("H,G,d,dv", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_capped_attention_with_a_sink(H, G, d, dv, dtype):
    """Capped scores, the sink and the gate against the restatement: a whole prompt from this step's rows, the same
    prompt as three portions over a shuffled block table beside a second sequence, and its last tokens as decode rows
    beside a padded row."""
    n, bs, scale, cap = 83, 16, 0.35, 4.0
    q, k, v = _attn_case(n, H, G, d, dv, 3, dtype)
    gate = torch.randn(n, H, generator=torch.Generator().manual_seed(9), dtype=F64).to(dtype).to(F64)
    want = O.sink_attention(q, k, v, scale, cap) * torch.sigmoid(gate)[:, :, None]
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    m = _attention_module(H, G, d, dv, scale, cap, dtype)
    got = _run_attention(m, q, k, v, dtype, [n], [n], gate=gate)
    assert float((got.view(n, H, dv) - want).abs().max()) < tol
    # without the cap or without the sink the result is another one: the test would see either left out
    assert float((O.sink_attention(q, k, v, scale, 0.0) - O.sink_attention(q, k, v, scale, cap)).abs().max()) > 0.05
    order = [5, 0, 3, 1, 4, 2]
    kc, vc, table = _paged(k, v, bs, order)
    m = _attention_module(H, G, d, dv, scale, cap, dtype, kc, vc)
    table2 = torch.cat([table, table], 0).cuda()
    at = 0
    for ql in (21, 30, 32):                                            # portions start inside blocks; a neighbour rides along
        qq = torch.cat([q[at:at + ql], q[:5]])
        got = _run_attention(m, qq, qq[:, :G], v[:ql + 5], dtype, [ql, 5], [at + ql, 5], table=table2,
                             gate=torch.cat([gate[at:at + ql], gate[:5]]))
        assert float((got[:ql].view(ql, H, dv) - want[at:at + ql]).abs().max()) < tol, at
        assert float((got[ql:].view(5, H, dv) - want[:5]).abs().max()) < tol
        at += ql
    for pos in (0, 15, 16, 47, 82):                                    # decode rows: first token, block borders, the end
        table3 = torch.cat([table, table, table], 0).cuda()
        got = _run_attention(m, q[[pos, 0, 31]], k[[pos, 0, 31]], v[[pos, 0, 31]], dtype, ctx_lens=[pos + 1, 0, 32],
                             table=table3, gate=gate[[pos, 0, 31]])
        assert float((got[0].view(H, dv) - want[pos]).abs().max()) < tol, pos
        assert float((got[2].view(H, dv) - want[31]).abs().max()) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 24, 20), (4, 2, 64, 64)])
def test_far_key_at_block_borders(H, G, d, dv, dtype):
    """One key hundreds of tokens back, at a block's last and first row, takes the whole softmax of one query head: in
    a prompt, in a portion that continues a cached prefix, and for a decoded token."""
    n, bs, scale = 600, 16, 1.0
    for j in (15, 16, 0, 31):
        i = 599
        q, k, v = _attn_case(n, H, G, d, dv, 5 + j, dtype, star=(i, j, 1), gain=7.0)
        want = O.sink_attention(q[i:], k, v, scale, 60.0, first_pos=i)
        assert float(want[0, 1].min()) > 4.5                          # the far value (5.0) is what the head returns
        tol = 1e-4 if dtype == torch.float32 else 5e-2
        order = list(range(37, -1, -1))
        kc, vc, table = _paged(k, v, bs, order)
        m = _attention_module(H, G, d, dv, scale, 60.0, dtype, kc, vc)
        got = _run_attention(m, q[i:], k[i:], v[i:], dtype, ctx_lens=[n], table=table.cuda())
        assert float((got.view(1, H, dv) - want).abs().max()) < tol, j
        got = _run_attention(m, q[590:], k[590:], v[590:], dtype, [10], [n], table=table.cuda())
        assert float((got[9].view(H, dv) - want[0]).abs().max()) < tol, j
        m2 = _attention_module(H, G, d, dv, scale, 60.0, dtype)
        got = _run_attention(m2, q, k, v, dtype, [n], [n])
        assert float((got[i].view(H, dv) - want[0]).abs().max()) < tol, j


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sink_share_and_first_tokens(dtype):
    """All scores zero: token t returns the mean of its t + 1 values times (t + 1) / (t + 2), the sink's share is what
    is missing -- at the first token one half. A cap far below the scores flattens them to +-cap."""
    H, G, d, dv, n = 2, 1, 16, 8, 40
    q = torch.zeros(n, H, d, dtype=F64)
    k = torch.randn(n, G, d, generator=torch.Generator().manual_seed(2), dtype=F64)
    v = torch.randn(n, G, dv, generator=torch.Generator().manual_seed(3), dtype=F64).to(dtype).to(F64)
    m = _attention_module(H, G, d, dv, 1.0, 5.0, dtype)
    got = _run_attention(m, q, k, v, dtype, [n], [n]).view(n, H, dv)
    want = v[:, 0].cumsum(0) / torch.arange(2, n + 2, dtype=F64)[:, None]
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got[:, 0] - want).abs().max()) < tol and float((got[:, 1] - want).abs().max()) < tol
    assert float((got[0, 0] - 0.5 * v[0, 0]).abs().max()) < tol
    # scores of +-1000 under a cap of 2: the weights are e^2 and e^-2 against the sink's 1
    q = torch.ones(3, 1, 4, dtype=F64)
    k = torch.tensor([[1.0], [-1.0], [1.0]], dtype=F64)[:, :, None].expand(3, 1, 4) * 250.0
    v = torch.tensor([[1.0, 0.0, 0.0], [0.0, 1.0, 0.0], [0.0, 0.0, 1.0]], dtype=F64)[:, None, :]
    m = _attention_module(1, 1, 4, 3, 1.0, 2.0, dtype)
    got = _run_attention(m, q, k.contiguous(), v, dtype, [3], [3]).view(3, 3)
    e2, em2 = math.exp(2.0), math.exp(-2.0)
    want = torch.tensor([e2, em2, e2], dtype=F64) / (1 + 2 * e2 + em2)
    assert float((got[2] - want).abs().max()) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("E,count,keep,top", [(10, 5, 4, 3), (6, 3, 2, 3), (16, 4, 1, 2), (4, 1, 1, 4), (12, 12, 5, 5),
                                              (9, 3, 3, 2)])
def test_grouped_softmax_router(E, count, keep, top):
    """Softmax over all experts, a group's score is its largest entry, only the best groups stay in play, the chosen
    scores are normalised: against the restatement, and on a row where the sum of a group's two largest entries would
    keep another group than its maximum does."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(E + top)
    z = torch.randn(50, E, generator=g, dtype=F64) * 2
    ids, w = ops.moe_route_grouped_softmax(_dev(z), top, count, keep)
    want_ids, want_w = O.route(z.float().to(F64), top, count, keep)
    assert torch.equal(ids.cpu().long().sort(1).values, want_ids.sort(1).values)
    got = torch.zeros(50, E, dtype=F64).scatter_(1, ids.cpu().long(), w.cpu().to(F64))
    ref = torch.zeros(50, E, dtype=F64).scatter_(1, want_ids, want_w)
    assert float((got - ref).abs().max()) < 1e-6
    assert float((w.sum(1) - 1).abs().max()) < 1e-5
    if (E, count, keep, top) == (6, 3, 2, 3):
        # groups (0,1) (2,3) (4,5): the largest entries are e^3.0, e^2.9, e^2.5 (times a constant); the sum of two would
        # rank the last group (2 e^2.5) first and drop the second: with one group dropped by its maximum, experts 4 and
        # 5 must be out and expert 3 in
        row = torch.tensor([[3.0, -5.0, 2.9, -4.0, 2.5, 2.5]], dtype=F64)
        ids, _ = ops.moe_route_grouped_softmax(_dev(row), 3, 3, 2)
        assert sorted(ids[0].tolist()) == [0, 2, 3]


@pytest.mark.parametrize("dtype,T,hidden,inter,E,top", [(torch.float32, 19, 40, 24, 4, 2), (torch.float32, 7, 128, 64, 8, 3),
                                                        (torch.bfloat16, 33, 96, 40, 6, 3), (torch.bfloat16, 5, 128, 64, 8, 4),
                                                        (torch.bfloat16, 1024, 128, 64, 4, 2), (torch.bfloat16, 600, 256, 128, 2, 2)])
def test_experts_with_a_clamped_unit(dtype, T, hidden, inter, E, top):
    """The mixture layer (router, experts with g sigmoid(1.702 g) (u + 1) on clamped g and u, weighted sum) against the
    restatement: fp32 and bf16, sizes only the generic kernels take, and prompt-sized batches on the tensor cores. The
    limit is low enough to clamp many entries."""
    from nanovllm.layers.moe import GroupedSoftmaxMoe
    g = torch.Generator().manual_seed(T + hidden)
    limit = 0.8
    mlp = moe(E, top, inter, count=2, keep=2 if top > E // 2 else 1, limit=limit)
    w = {"p.router": torch.randn(E, hidden, generator=g) * 0.3}
    for e in range(E):
        w[f"p.e{e}.gate"] = torch.randn(inter, hidden, generator=g) * hidden ** -0.5 * 2
        w[f"p.e{e}.up"] = torch.randn(inter, hidden, generator=g) * hidden ** -0.5 * 2
        w[f"p.e{e}.down"] = torch.randn(hidden, inter, generator=g) * inter ** -0.5
    w = {k: v.to(dtype).to(F64) for k, v in w.items()}
    x = torch.randn(T, hidden, generator=g, dtype=F64).to(dtype).to(F64)
    torch.set_default_dtype(dtype)                                     # as the runner builds a model: the router stays fp32
    try:
        m = GroupedSoftmaxMoe(hidden, inter, E, top, 2, mlp["router"]["groups"]["keep"], glu=(1.702, limit))
    finally:
        torch.set_default_dtype(torch.float32)
    assert m.router.dtype == torch.float32 and m.w13.dtype == dtype
    m.router.data.copy_(w["p.router"])
    for e in range(E):
        m.w13.data[e, :inter].copy_(w[f"p.e{e}.gate"])
        m.w13.data[e, inter:].copy_(w[f"p.e{e}.up"])
        m.w2.data[e].copy_(w[f"p.e{e}.down"])
    m = m.cuda()
    got = m(x.to(dtype).cuda()).cpu().to(F64)
    rows = slice(0, min(T, 64))
    want = O.moe_ff(x[rows], w, "p.", mlp)
    if dtype == torch.float32:
        assert float((got[rows] - want).abs().max()) < 1e-4
    else:
        err = (got[rows] - want).abs().max(1).values / want.abs().max()
        assert float(err.median()) < 2e-2 and float((err < 5e-2).double().mean()) > 0.9       # a close choice may flip
    if T > 64:                                                         # the tensor-core form against the generic one
        m.fast = False
        slow = m(x.to(dtype).cuda()).cpu().to(F64)
        assert float((got - slow).abs().max() / slow.abs().max()) < 3e-2


def test_short_convolution_tails_per_projection():
    """Three projections' channels side by side with their own taps; a sequence continued over portions of 1 to 5 tokens
    reads the tail that the step before left in its slot."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(4)
    C, taps, T = 44, 4, 23
    u, w = torch.randn(T, C, generator=g, dtype=F64), torch.randn(C, taps, generator=g, dtype=F64)
    want, _ = O.short_conv(u, w)
    state = torch.full((3, taps - 1, C), 9.0, device="cuda")                     # slots hold leftovers
    slots = torch.tensor([1], dtype=torch.int32).cuda()
    outs, at = [], 0
    for n in (5, 1, 1, 2, 3, 1, 4, 1, 5):
        spans = _spans([n], [at + n]) if not (n == 1 and at > 0) else _decode_spans([at + 1])
        outs.append(ops.causal_conv(_dev(u[at:at + n]), _dev(w), None, spans, state, slots))
        at += n
    assert at == T
    assert float((torch.cat(outs).cpu().to(F64) - want).abs().max()) < 1e-5


@pytest.mark.parametrize("H,G,D", [(4, 2, 64), (8, 1, 128), (8, 8, 64)])
def test_cap_and_sink_on_the_tensor_core_kernels(H, G, D):
    """The tcgen05 prompt kernel and the paged decode kernel with a score cap and a sink against the generic kernel:
    a long prompt, a short portion over thousands of cached keys (the keys are split over CTAs and the sink must join
    once), and decode rows whose keys are split over CTAs beside short ones."""
    from nanovllm import ops
    g = torch.Generator().manual_seed(D + H)
    n, bs, scale, cap = 4100, 64, D ** -0.5 * 2.0, 3.0
    q = torch.randn(n, H, D, generator=g).bfloat16().cuda()
    k = torch.randn(n, G, D, generator=g).bfloat16().cuda()
    v = torch.randn(n, G, D, generator=g).bfloat16().cuda()
    sink = torch.tensor([0.0, 1.5, -2.0, 0.3] * (H // 4), dtype=torch.float32).cuda()
    nb = -(-n // bs)
    order = torch.randperm(nb, generator=g)
    kc = torch.zeros(nb + 1, bs, G * D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    pad = nb * bs - n
    kc[order.cuda()] = torch.nn.functional.pad(k.view(n, -1), (0, 0, 0, pad)).view(nb, bs, -1)
    vc[order.cuda()] = torch.nn.functional.pad(v.view(n, -1), (0, 0, 0, pad)).view(nb, bs, -1)
    table = order.to(torch.int32).cuda()[None, :].contiguous()
    cu = lambda *x: torch.tensor(x, dtype=torch.int32).cuda()
    ref = ops.attn_generic(q, k, v, ops.StepSpans(cu(0, n), cu(0, n), None, n), scale, G, D, softcap=cap, sink=sink).float()
    plain = ops.attn_generic(q[-8:], kc, vc, ops.StepSpans(cu(0, 8), cu(0, n), None, 8), scale, G, D, block_tables=table).float()
    assert float((plain - ref[-8:]).abs().max()) > 0.05               # cap and sink matter on this input
    got = ops.prefill_varlen_attn(q, k, v, cu(0, n), cu(0, n), n, n, scale, G, softcap=cap, sink=sink).float()
    assert float((got - ref).abs().max()) < 3e-2
    for ql in (128, 40):                                               # few queries, many keys: split along the keys
        got = ops.prefill_varlen_attn(q[n - ql:], kc, vc, cu(0, ql), cu(0, n), ql, n, scale, G, block_tables=table,
                                      softcap=cap, sink=sink).float()
        assert float((got - ref[n - ql:]).abs().max()) < 3e-2, ql
    rows = [n - 1, 16, 899, 0]
    tables = table.repeat(len(rows), 1).contiguous()
    ctx_lens = torch.tensor([r + 1 for r in rows], dtype=torch.int32).cuda()
    got = ops.paged_decode_attn(q[rows], kc, vc, tables, ctx_lens, scale, G, softcap=cap, sink=sink).float()
    assert float((got - ref[rows]).abs().max()) < 3e-2
