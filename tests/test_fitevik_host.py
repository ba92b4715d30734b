"""CPU: the host side of the Fitevik decoder -- registry and native configuration (the learned position table bounds the
sequence length), presets, checkpoint tensors routed onto fused projections and stacked experts, borrowers of keys and
values wired to their lenders, and the float64 oracle's own invariants (so that the GPU tests compare against
something sound)."""
import json
import math

import pytest
import torch

import fitevik_oracle as O
from test_fitevik_gpu import attention, config_a, config_b, config_c, dense, hgrn2

F64 = torch.float64


def test_registry_native_config_and_presets(tmp_path):
    from nanovllm.config import Config, NativeConfig
    from nanovllm.models.models_map import model_dict
    from nanovllm.engine.model_runner import _resolve_dtype
    cfg = config_a()
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    c = Config(str(tmp_path), max_model_len=4096, max_num_batched_tokens=4096, dtype="float32")
    assert isinstance(c.hf_config, NativeConfig) and c.hf_config.architectures == ["Fitevik"]
    assert c.max_model_len == cfg["max_positions"]                # no sequence outgrows the position table
    assert model_dict["Fitevik"].supports_fp32 and not model_dict["Fitevik"].prefix_caching
    assert _resolve_dtype(c.hf_config, "float32", model_dict["Fitevik"]) == torch.float32
    p = Config("tiny-fitevik").hf_config.to_dict()
    assert [l["type"] for l in p["layers"]] == ["hgrn2", "hgrn2", "attention", "attention"]
    assert p["layers"][3]["mixer"]["kv_from"] == 2 and "kv_from" not in p["layers"][2]["mixer"]
    big = Config("fitevik-1k").hf_config.to_dict()
    assert len(big["layers"]) == 28 and big["width"] == 1024
    for i, e in enumerate(big["layers"]):                         # every borrower names an earlier lender
        j = e["mixer"].get("kv_from")
        if j is not None:
            assert j < i and big["layers"][j]["type"] == "attention" and "kv_from" not in big["layers"][j]["mixer"]


@pytest.mark.parametrize("make", [config_a, config_b, config_c])
def test_checkpoint_tensors_route_onto_the_model(tmp_path, make):
    """Every tensor of a checkpoint lands somewhere, every parameter is covered, fused projections hold the pieces in
    the order the mixers slice them, and a borrower has no key or value rows at all."""
    from safetensors.torch import save_file
    from nanovllm.config import NativeConfig
    from nanovllm.layers.moe import TopkSoftmaxMoe
    from nanovllm.models.models_map import model_dict
    from nanovllm.utils.loader import load_model
    cfg = make()
    tensors = O.random_model(cfg, seed=3)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    model = model_dict["Fitevik"](NativeConfig(cfg))
    for p in model.parameters():
        p.data.fill_(float("nan"))
    assert load_model(model, str(tmp_path)) == len(tensors)
    assert not any(torch.isnan(p).any() for p in model.parameters())
    assert model.lm_head.scale == cfg["logit_scale"] and model.positions.weight.shape[0] == cfg["max_positions"]
    assert torch.equal(model.positions.weight.float(), tensors["pos"].float())
    assert torch.equal(model.embed_norm.bias, tensors["embed.norm.b"].float())
    for i, entry in enumerate(cfg["layers"]):
        layer, mix, m = model.layers[i], model.layers[i].mix, entry["mixer"]
        t = lambda n: tensors[f"l{i}.{n}"].float()
        assert torch.equal(layer.norm1.weight, t("norm1")) and torch.equal(layer.norm1.bias, t("norm1.b"))
        w = mix.proj.weight.float()
        if entry["type"] == "hgrn2":
            n, nv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            assert torch.equal(w[:n], t("mix.q")) and torch.equal(w[n:2 * n], t("mix.f")) and torch.equal(w[2 * n:], t("mix.v"))
            assert w.shape[0] == 2 * n + nv and mix.rec.tied_gate
            assert torch.equal(mix.rec.lower, t("mix.lower")) and torch.equal(mix.rec.gate_bias, t("mix.f.b"))
            assert torch.equal(mix.norm.weight, t("mix.norm").repeat(m["heads"]))
        else:
            nq, nk = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
            assert torch.equal(w[:nq], t("mix.q")) and torch.equal(mix.q_norm, t("mix.q.norm"))
            assert torch.equal(mix.attn.talk, t("mix.talk")) and torch.equal(mix.attn.sink, t("mix.sink"))
            assert mix.attn.window == (m.get("mask") or {}).get("size", 0) and mix.attn.scale == m["scale"]
            assert mix.attn.slopes.tolist() == pytest.approx(O.head_slopes(m["heads"]))
            if "kv_from" in m:
                assert w.shape[0] == nq and mix.attn.kv_source is model.layers[m["kv_from"]].mix.attn
                assert mix.attn.cache_rows() == (0, 0) and not hasattr(mix, "k_norm")
            else:
                assert torch.equal(w[nq:nq + nk], t("mix.k")) and torch.equal(w[nq + nk:], t("mix.v"))
                assert mix.attn.kv_source is None and mix.attn.cache_rows() == (nk, m["kv_heads"] * m["vdim"])
        if isinstance(layer.mlp, TopkSoftmaxMoe):
            e = entry["mlp"]["router"]["experts"] - 1
            assert torch.equal(layer.mlp.w1.float()[e], t(f"mlp.e{e}.up")) and torch.equal(layer.mlp.w2.float()[0], t("mlp.e0.down"))
            assert layer.mlp.router.dtype == torch.float32 and torch.equal(layer.mlp.router_bias, t("mlp.router.b"))
            assert layer.mlp.top_k == entry["mlp"]["router"]["top"] and layer.mlp.act == "relu2"
        elif layer.mlp is not None:
            assert torch.equal(layer.mlp.up_proj.bias.float(), t("mlp.up.b")) and torch.equal(layer.mlp.down_proj.weight.float(), t("mlp.down"))
        else:
            assert not hasattr(layer, "norm2")
    # parameters are listed once although a borrower refers to its lender
    names = [n for n, _ in model.named_parameters()]
    assert len(names) == len(set(names)) and not any("kv_source" in n for n in names)


def test_borrowers_need_a_real_lender():
    from nanovllm.config import NativeConfig
    from nanovllm.models.models_map import model_dict
    base = {"architecture": "Fitevik", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "logit_scale": 1.0, "max_positions": 64}
    for layers in ([hgrn2(1, 8, 8), attention(2, 1, 8, 8, 0, 0.3, kv_from=0)],                      # not an attention layer
                   [attention(2, 1, 8, 8, 0, 0.3, kv_from=1), attention(2, 1, 8, 8, 0, 0.3)],       # not earlier
                   [attention(2, 1, 8, 8, 0, 0.3), attention(2, 1, 8, 8, 0, 0.3, kv_from=0),
                    attention(2, 1, 8, 8, 0, 0.3, kv_from=1)],                                      # a borrower lends nothing
                   [attention(2, 1, 8, 8, 0, 0.3), attention(2, 2, 8, 8, 0, 0.3, kv_from=0)]):      # other kv heads
        with pytest.raises(ValueError):
            model_dict["Fitevik"](NativeConfig(dict(base, layers=layers)))
    with pytest.raises(ValueError):
        model_dict["Fitevik"](NativeConfig(dict(base, layers=[{"type": "lightning", "mixer": {}, "mlp": None}])))
    with pytest.raises(ValueError):
        model_dict["Fitevik"](NativeConfig(dict(base, layers=[hgrn2(1, 8, 8, mlp={"kind": "gated", "ff": 8})])))


def test_random_init_is_finite_and_shares_the_head_norm():
    from nanovllm.config import Config
    from nanovllm.models.models_map import model_dict
    model = model_dict["Fitevik"](Config("tiny-fitevik").hf_config)
    model.random_init(1)
    rec = model.layers[0].mix
    assert torch.equal(rec.norm.weight[:rec.dv], rec.norm.weight[rec.dv:2 * rec.dv])
    assert float(rec.rec.lower.detach().min()) >= 0.0 and float(rec.rec.lower.detach().max()) < 1.0
    assert all(torch.isfinite(p).all() for p in model.parameters())


# ------------------------------------------------------------------ the oracle's own invariants
def test_oracle_is_causal_and_windows_cut():
    cfg = config_a()
    t = O.as_f64(O.random_model(cfg, 1))
    toks = list(range(40))
    full = O.forward(cfg, t, toks)
    assert torch.allclose(O.forward(cfg, t, toks[:25]), full[:25], atol=1e-9)
    m = dict(cfg["layers"][1]["mixer"])
    u = torch.randn(30, cfg["width"], generator=torch.Generator().manual_seed(2), dtype=F64)
    P = O.sub(t, "l1.mix.")
    base, _ = O.attention_mixer(u, m, P, 1e-5)
    u2 = u.clone()
    u2[3] += 1.0                                        # inside the window (19) of token 21, outside of token 22
    moved, _ = O.attention_mixer(u2, m, P, 1e-5)
    assert torch.allclose(moved[22:], base[22:], atol=1e-12) and not torch.allclose(moved[21], base[21], atol=1e-9)


def test_oracle_attention_pieces():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(6, 2, 4, generator=g, dtype=F64) for _ in range(3))
    plain = O.mixed_head_attention(q, k, v, 0.5, 0, None, None, None)
    w = torch.softmax(torch.einsum("ihd,jhd->hij", q, k)[:, 5] * 0.5, -1)                # the last query against all keys
    assert torch.allclose(plain[5], torch.einsum("hj,jhv->hv", w, v))
    # the sink only shrinks: the weights of the keys keep their ratios and sum to less than one
    sunk = O.mixed_head_attention(q, k, v, 0.5, 0, None, torch.tensor([0.0, 2.0], dtype=F64), None)
    ratio = sunk[5] / plain[5]
    assert torch.allclose(ratio[0], ratio[0, :1].expand(4)) and bool((ratio.abs() < 1).all())
    # an identity mix is no mix; swapping the rows of the mix swaps the heads' weights but not their values
    eye = O.mixed_head_attention(q, k, v, 0.5, 0, torch.eye(2, dtype=F64), None, None)
    assert torch.allclose(eye, plain)
    vv = v.clone()
    vv[:, 1] = vv[:, 0]
    a = O.mixed_head_attention(q, k, vv, 0.5, 0, None, None, None)
    b = O.mixed_head_attention(q, k, vv, 0.5, 0, torch.tensor([[0.0, 1.0], [1.0, 0.0]], dtype=F64), None, None)
    assert torch.allclose(a[:, 0], b[:, 1]) and torch.allclose(a[:, 1], b[:, 0])
    # the distance bias is the same for (i - j) as for -j alone when there is neither sink nor cap: softmax is shift
    # invariant per query; with a sink the two differ
    s = O.head_slopes(2)
    assert s == [2.0 ** -4, 2.0 ** -8]
    near = O.mixed_head_attention(q, k, v, 0.5, 0, None, None, [50.0, 50.0])
    assert torch.allclose(near, v[:, :, :], atol=1e-9)                                   # a steep bias leaves the token itself


def test_oracle_gate_and_router():
    lower = torch.tensor([0.0, 0.5, 0.9], dtype=F64)
    f = O.forget_gate(torch.zeros(1, 2, dtype=F64), torch.zeros(3, 2, dtype=F64), torch.tensor([-50.0, 0.0, 50.0], dtype=F64), lower)
    assert torch.allclose(f[0], torch.tensor([0.0, 0.75, 1.0], dtype=F64), atol=1e-12)
    # f = 1 keeps, f = 0 replaces; the read-out sees the current token's write
    q = torch.ones(2, 1, 2, dtype=F64)
    v = torch.tensor([[[3.0]], [[5.0]]], dtype=F64)
    o, S = O.hgrn2_states(q, torch.tensor([[[0.0, 0.0]], [[1.0, 0.0]]], dtype=F64), v)
    assert o[:, 0, 0].tolist() == [6.0, 8.0] and S[0, :, 0].tolist() == [3.0, 5.0]
    # a state handed over equals one run
    g = torch.Generator().manual_seed(1)
    q, f, v = torch.randn(9, 2, 3, generator=g, dtype=F64), torch.rand(9, 2, 3, generator=g, dtype=F64), torch.randn(9, 2, 4, generator=g, dtype=F64)
    whole, _ = O.hgrn2_states(q, f, v)
    first, S = O.hgrn2_states(q[:4], f[:4], v[:4])
    rest, _ = O.hgrn2_states(q[4:], f[4:], v[4:], S)
    assert torch.allclose(torch.cat([first, rest]), whole)
    idx, w = O.route(torch.eye(4, dtype=F64)[:1], torch.tensor([[1.0, 0, 0, 0], [3.0, 0, 0, 0], [2.0, 0, 0, 0]], dtype=F64),
                     torch.tensor([0.0, 0.0, 1.5], dtype=F64), 2)
    assert idx[0].tolist() == [2, 1]                                                     # the bias takes part in the choice
    assert torch.allclose(w[0], torch.softmax(torch.tensor([3.5, 3.0], dtype=F64), 0))
    assert math.isclose(float(O.relu_squared(torch.tensor(-2.0))), 0.0) and float(O.relu_squared(torch.tensor(3.0))) == 9.0
