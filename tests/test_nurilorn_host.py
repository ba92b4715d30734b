"""CPU: the host side of the Nurilorn decoder -- registry and native configuration, presets, checkpoint tensors routed
onto fused projections and stacked experts, the band-scaled frequencies, configurations that are refused, and the
float64 oracle's own invariants (so that the GPU tests compare against something sound)."""
import json
import math

import pytest
import torch

import nurilorn_oracle as O
from test_nurilorn_gpu import config_a, config_b, config_c, config_d, layer, rot, tokens_of

F64 = torch.float64


def test_registry_native_config_and_presets(tmp_path):
    from nanovllm.config import Config, NativeConfig
    from nanovllm.models.models_map import model_dict
    from nanovllm.engine.model_runner import _resolve_dtype
    cfg = config_a()
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    c = Config(str(tmp_path), max_model_len=4096, max_num_batched_tokens=4096, dtype="float32")
    assert isinstance(c.hf_config, NativeConfig) and c.hf_config.architectures == ["Nurilorn"]
    cls = model_dict["Nurilorn"]
    assert cls.supports_fp32 and not cls.prefix_caching
    assert _resolve_dtype(c.hf_config, "float32", cls) == torch.float32
    p = Config("tiny-nurilorn").hf_config.to_dict()
    assert [l["mlp"] and l["mlp"]["kind"] for l in p["layers"]] == ["dense", "moe", None]
    big = Config("nurilorn-1k").hf_config.to_dict()
    assert len(big["layers"]) == 28 and big["width"] == 1024 and big["width"] % big["norm"]["groups"] == 0
    assert all(e["mixer"]["heads"] % e["mixer"]["kv_heads"] == 0 for e in big["layers"])


@pytest.mark.parametrize("make", [config_a, config_b, config_c, config_d])
def test_checkpoint_tensors_route_onto_the_model(tmp_path, make):
    """Every tensor of a checkpoint lands somewhere, every parameter is covered, the fused projection holds q, k, v and
    the gate rows in the order the mixer slices them, experts are stacked gate rows first."""
    from safetensors.torch import save_file
    from nanovllm.config import NativeConfig
    from nanovllm.layers.moe import GroupedSoftmaxMoe
    from nanovllm.models.models_map import model_dict
    from nanovllm.utils.loader import load_model
    cfg = make()
    tensors = O.random_weights(cfg, seed=3)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    model = model_dict["Nurilorn"](NativeConfig(cfg))
    for p in model.parameters():
        p.data.fill_(float("nan"))
    assert load_model(model, str(tmp_path)) == len(tensors)
    assert not any(torch.isnan(p).any() for p in model.parameters())
    assert model.lm_head.scale == cfg["logit_scale"] and model.mult == cfg["residual_mult"]
    assert model.embed_scale == cfg["embedding"]["scale"] and model.groups == cfg["norm"]["groups"]
    assert torch.equal(model.norm.weight, tensors["final.norm"].float())
    for i, entry in enumerate(cfg["layers"]):
        lay, mix, m = model.layers[i], model.layers[i].mix, entry["mixer"]
        t = lambda n: tensors[f"l{i}.{n}"].float()
        assert torch.equal(lay.norm1.weight, t("norm1")) and torch.equal(lay.ls1, t("ls1"))
        nq, nk, nv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
        w = mix.proj.weight.float()
        assert w.shape[0] == nq + nk + nv + m["heads"]
        assert torch.equal(w[:nq], t("mix.q")) and torch.equal(w[nq:nq + nk], t("mix.k"))
        assert torch.equal(w[nq + nk:nq + nk + nv], t("mix.v")) and torch.equal(w[nq + nk + nv:], t("mix.g"))
        cw = mix.conv.weight
        assert cw.shape == (nq + nk + nv, m["conv"]) and torch.equal(cw[nq:nq + nk], t("mix.k.conv"))
        assert torch.equal(cw[nq + nk:], t("mix.v.conv"))
        assert float(mix.vmix.data) == float(t("mix.vmix")) and mix.v_mix == m["v_mix"]
        assert mix.attn.softcap == m["softcap"] and mix.attn.scale == m["scale"] and mix.attn.sink.tolist() == [0.0] * m["heads"]
        assert mix.attn.cache_rows() == (nk, nv) and mix.conv.state_shapes() == (
            {"conv_state": ((m["conv"] - 1, nq + nk + nv), None)} if m["conv"] > 1 else {})
        assert torch.equal(mix.o_proj.weight.float(), t("mix.o"))
        mlp = entry["mlp"]
        if mlp is None:
            assert lay.mlp is None and not hasattr(lay, "norm2")
        elif mlp["kind"] == "dense":
            assert lay.mlp.limit == mlp["limit"] and torch.equal(lay.mlp.gate_up_proj.weight.float()[mlp["ff"]:], t("mlp.up"))
            assert torch.equal(lay.ls2, t("ls2"))
        else:
            assert isinstance(lay.mlp, GroupedSoftmaxMoe) and lay.mlp.router.dtype == torch.float32
            ff, r = mlp["expert"]["ff"], mlp["router"]
            assert (lay.mlp.top_k, lay.mlp.groups, lay.mlp.keep) == (r["top"], r["groups"]["count"], r["groups"]["keep"])
            assert lay.mlp.glu == (1.702, mlp["expert"]["limit"])
            e = r["experts"] - 1
            assert torch.equal(lay.mlp.w13.float()[e, :ff], t(f"mlp.e{e}.gate"))
            assert torch.equal(lay.mlp.w13.float()[e, ff:], t(f"mlp.e{e}.up"))
            assert torch.equal(lay.mlp.w2.float()[e], t(f"mlp.e{e}.down"))
    names = [n for n, _ in model.named_parameters()]
    assert len(names) == len(set(names))


def test_refused_configurations():
    from nanovllm.config import NativeConfig
    from nanovllm.models.models_map import model_dict
    cls = model_dict["Nurilorn"]
    cfg = config_b()
    cfg["layers"][0]["type"] = "recurrence"
    with pytest.raises(ValueError):
        cls(NativeConfig(cfg))
    cfg = config_b()
    cfg["layers"][1]["mlp"]["kind"] = "sparse"
    with pytest.raises(ValueError):
        cls(NativeConfig(cfg))
    cfg = config_b()
    cfg["norm"]["groups"] = 3                           # 128 columns do not split into three groups
    with pytest.raises(ValueError):
        cls(NativeConfig(cfg))


def test_band_scaled_frequencies():
    """Fast pairs keep their frequency, slow ones are divided by the factor, the ramp lies between; the magnitude grows
    with the logarithm of the factor; without a stretch nothing changes."""
    from nanovllm.layers.seq_mixers import BandScaledRotary
    plain = BandScaledRotary(48, 5e5, True, None)
    assert plain.magnitude == 1.0 and float(plain.freq[0]) == 1.0
    assert float(plain.freq[5]) == pytest.approx(5e5 ** (-10 / 48))
    sc = {"factor": 6.0, "original": 2048, "fast": 24.0, "slow": 2.0}
    br = BandScaledRotary(48, 5e5, True, sc)
    f, mag = O.yarn_frequencies({"dims": 48, "base": 5e5, "scaling": sc})
    assert torch.equal(br.freq, f) and br.magnitude == mag == pytest.approx(0.1 * math.log(6.0) + 1)
    ratio = br.freq / plain.freq
    assert float(ratio[0]) == 1.0 and float(ratio[-1]) == pytest.approx(1 / 6.0)
    assert bool((ratio[1:] <= ratio[:-1] + 1e-15).all())               # monotone from 1 down to 1 / factor
    # pairs 0..4 turn at least 24 times over the original length and keep their frequency, pairs from 10 on turn at
    # most twice and are divided by the factor, the ramp lies between
    assert int((ratio == 1.0).sum()) == 5 and int(((ratio - 1 / 6.0).abs() < 1e-15).sum()) == 14
    assert br.key != plain.key and BandScaledRotary(48, 5e5, True, dict(sc)).key == br.key


# ------------------------------------------------------------------ the oracle's own invariants
def test_oracle_continues_a_sequence():
    """A prompt in one piece equals the same prompt continued from handed-over state (tails, keys, blended values)."""
    cfg = config_a()
    tensors = O.random_weights(cfg, seed=3)
    toks = tokens_of(cfg, 21, 8)
    whole, _ = O.forward(cfg, tensors, toks)
    a, st = O.forward(cfg, tensors, toks[:9])
    b, st = O.forward(cfg, tensors, toks[9:10], states=st, first_pos=9)
    c, _ = O.forward(cfg, tensors, toks[10:], states=st, first_pos=10)
    assert float((torch.cat([a, b, c]) - whole).abs().max()) < 1e-9


def test_oracle_is_causal_and_blends_the_first_layers_values():
    cfg = config_a()
    tensors = O.random_weights(cfg, seed=4)
    toks = tokens_of(cfg, 17, 9)
    a, _ = O.forward(cfg, tensors, toks)
    other = list(toks)
    other[12] = (other[12] + 1) % cfg["vocab"]
    b, _ = O.forward(cfg, tensors, other)
    assert torch.equal(a[:12], b[:12]) and not torch.equal(a[12:], b[12:])
    # lambda = 0 in every blending layer equals a model that does not blend
    t0 = {k: (torch.zeros_like(v) if k.endswith("vmix") else v) for k, v in tensors.items()}
    plain = json.loads(json.dumps(cfg))
    for e in plain["layers"]:
        e["mixer"]["v_mix"] = False
    assert float((O.forward(cfg, t0, toks)[0] - O.forward(plain, t0, toks)[0]).abs().max()) < 1e-12
    assert float((O.forward(cfg, tensors, toks)[0] - O.forward(plain, tensors, toks)[0]).abs().max()) > 1e-3


def test_oracle_sink_cap_and_norm_groups():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, 2, 8, generator=g, dtype=F64) for _ in range(3))
    with_sink = O.sink_attention(q, k, v, 0.3, 0.0)
    # the sink only shrinks: the output is the plain softmax result times sum / (1 + sum)
    for t in (0, 5):
        s = (k[:t + 1, 0] @ q[t, 0]) * 0.3
        plain = torch.softmax(s, 0) @ v[:t + 1, 0]
        share = float(torch.exp(s).sum() / (1 + torch.exp(s).sum()))
        assert float((with_sink[t, 0] - share * plain).abs().max()) < 1e-12
    capped = O.sink_attention(q * 50, k, v, 1.0, 2.0)
    assert bool(torch.isfinite(capped).all())
    x, w = torch.randn(5, 12, generator=g, dtype=F64), torch.ones(12, dtype=F64)
    n = O.grouped_rms_norm(x, w, 3, 0.0)
    assert float((n.reshape(5, 3, 4).pow(2).mean(-1) - 1).abs().max()) < 1e-12
    u, cw = torch.randn(6, 3, generator=g, dtype=F64), torch.randn(3, 4, generator=g, dtype=F64)
    y, tail = O.short_conv(u, cw)
    assert float((y[0] - cw[:, 3] * u[0]).abs().max()) < 1e-15 and torch.equal(tail, u[3:])
    ids, wts = O.route(torch.tensor([[0.0, 1.0, 2.0, 3.0]], dtype=F64), 2, 2, 1)
    assert sorted(ids[0].tolist()) == [2, 3] and float(wts.sum()) == pytest.approx(1.0)
