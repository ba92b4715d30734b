"""Fitevik: a decoder whose layers are listed one by one in its configuration, on an fp32 residual stream with the
norm on each sublayer's OUTPUT -- the sublayers read the stream itself:

    x <- LN(embed[token] + pos[p]);   x <- x + LN(mixer(x));   x <- x + LN(ff(x));   logits = logit_scale * head LN(x)

(LN: layer norm with weight and bias; positions are a learned table, not scaled.) Each layer has one of two sequence
mixers and an optional feed-forward:

  hgrn2      linear attention in which the forget gate also decides what is written: q = silu(W_q h), v = W_v h,
             f = l + (1 - l) sigmoid(W_f h + b) per head and key channel with a learned lower bound l; per head
             S <- diag(f) S + (1 - f) v^T, o = S^T q (fp32 state, no key, no other scale); o / rms(o) per head times a
             weight shared by the heads; W_o
  attention  q, k, v projections; q and k divided by the root mean square of the WHOLE projection (all heads at once),
             times a plain weight; no rotation; score = scale q.k - slope_h (i - j) with slope_h = 2^(-8 (h + 1) / H);
             the heads' scores are mixed by a learned [H, H] matrix before the softmax; sliding window; a learned sink per
             head in the softmax denominator; W_o. A layer with "kv_from": j has no key/value projections and attends
             over layer j's cached keys and values with its own queries.
  dense ff   W_down relu(W_up h + b)^2 + b          moe   router logits in fp32 (with bias), the `top` largest chosen,
                                                          weights = softmax over the chosen; experts without biases

Launches per mixer sublayer: one GEMM in (every projection that reads the sublayer input fused), the mechanism's
preparation kernel (gate and query in fp32 / whole-row norms + cache write), the mixer kernel, the per-head norm
(hgrn2), one GEMM out, and ONE kernel for "norm the output, add it to the stream, hand the stream to the next
sublayer in the model dtype". What the design fixes is a constant here; every size and every constant that may differ
between models comes from the config.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from .. import ops
from ..layers.embed_head import ParallelLMHead, VocabParallelEmbedding
from ..layers.linear import MergedColumnParallelLinear, ReplicatedLinear, RowParallelLinear, tp_rank_size
from ..layers.moe import TopkSoftmaxMoe
from ..layers.seq_mixers import GatedNorm, LinearRecurrence, MixedHeadAttention, small_param
from ..utils.context import get_context

SLOPE_BASE = 8.0           # distance bias of head h: 2^(-8 (h + 1) / H) per position
FF_ACT = "relu2"           # the square of relu, dense and expert feed-forwards alike


@dataclass
class FitevikSpec:
    """What the runner asks of a model's spec."""
    vocab_size: int
    hidden_size: int
    num_layers: int
    rms_eps: float
    num_experts: int = 0
    tie_embeddings: bool = False


class AffineNorm(nn.Module):
    """Weight and bias of one layer norm; the arithmetic runs fused with the residual update."""

    def __init__(self, size: int):
        super().__init__()
        self.weight, self.bias = small_param(size, fill=1.0), small_param(size)


class Hgrn2Mixer(nn.Module):

    def __init__(self, width: int, m: dict, eps: float):
        super().__init__()
        H, d = m["heads"], m["dim"]
        dv = m.get("vdim", d)
        self.H, self.d, self.dv = H, d, dv
        self.sizes = [H * d, H * d, H * dv]                             # q | forget | v
        self.proj = MergedColumnParallelLinear(width, self.sizes)
        self.rec = LinearRecurrence(H, H, d, dv, tied_gate=True)
        self.norm = GatedNorm(H * dv, eps, groups=H, gate_first=False)
        self.norm.weight.weight_loader = lambda p, w: p.data.copy_(w.repeat(H))          # one [vdim] weight for all heads
        self.o_proj = RowParallelLinear(H * dv, width)

    def forward(self, positions, h):
        p = self.proj(h)
        nq, nf, _ = self.sizes
        o = self.rec(p[:, :nq], p[:, nq:nq + nf], p[:, nq + nf:])
        return self.o_proj(self.norm(o, None, dtype=h.dtype))


class TalkingAttentionMixer(nn.Module):

    def __init__(self, width: int, m: dict, eps: float, lender: "TalkingAttentionMixer | None" = None):
        super().__init__()
        H, d = m["heads"], m["dim"]
        G, dv = m.get("kv_heads", H), m.get("vdim", d)         # absent: one kv head per query head, values as wide as keys
        self.H, self.G, self.d, self.dv, self.eps = H, G, d, dv, eps
        self.borrows = lender is not None
        self.sizes = [H * d, 0, 0] if self.borrows else [H * d, G * d, G * dv]           # q | k | v
        self.proj = MergedColumnParallelLinear(width, [n for n in self.sizes if n])
        self.q_norm = small_param(H * d, fill=1.0)
        if not self.borrows:
            self.k_norm = small_param(G * d, fill=1.0)
        self.attn = MixedHeadAttention(H, G, d, dv, float(m.get("scale", d ** -0.5)),
                                       window=int((m.get("mask") or {}).get("size", 0) or 0),
                                       slope_base=SLOPE_BASE, kv_source=lender.attn if lender is not None else None)
        self.o_proj = RowParallelLinear(H * dv, width)

    def forward(self, positions, h):
        qkv = self.proj(h)
        nq, nk, nv = self.sizes
        attn = self.attn
        ctx = get_context()
        have_cache = attn.k_cache.numel() > 0 and ctx.slot_mapping is not None and not self.borrows
        ops.rownorm_cache(qkv, nq, nk, nv, self.q_norm, None if self.borrows else self.k_norm, self.eps,
                          attn.k_cache if have_cache else None, attn.v_cache if have_cache else None,
                          ctx.slot_mapping if have_cache else None)
        q = qkv[:, :nq].unflatten(1, (self.H, self.d))
        if self.borrows:
            return self.o_proj(attn(q))
        k = qkv[:, nq:nq + nk].unflatten(1, (self.G, self.d))
        v = qkv[:, nq + nk:].unflatten(1, (self.G, self.dv))
        return self.o_proj(attn(q, k, v))


class PlainFeedForward(nn.Module):
    """W_down act(W_up h + b) + b: no gate."""

    def __init__(self, width: int, ff: int, act: str = FF_ACT):
        super().__init__()
        self.act = act
        self.up_proj = ReplicatedLinear(width, ff, bias=True)
        self.down_proj = RowParallelLinear(ff, width, bias=True)

    def forward(self, h):
        return self.down_proj(ops.act_only(self.up_proj(h), self.act))


def build_feed_forward(width: int, mlp: dict) -> nn.Module:
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return PlainFeedForward(width, mlp["ff"])
    if kind == "moe":
        r = mlp["router"]
        return TopkSoftmaxMoe(width, mlp["expert"]["ff"], r["experts"], r["top"], act=FF_ACT)
    raise ValueError(f"unknown feed-forward kind {kind!r}")


class FitevikLayer(nn.Module):

    def __init__(self, width: int, entry: dict, eps: float, earlier: list):
        super().__init__()
        kind, m = entry["type"], entry["mixer"]
        if kind == "hgrn2":
            self.mix = Hgrn2Mixer(width, m, eps)
        elif kind == "attention":
            lender = None
            if m.get("kv_from") is not None:
                j = int(m["kv_from"])
                if not 0 <= j < len(earlier) or not isinstance(earlier[j].mix, TalkingAttentionMixer) or earlier[j].mix.borrows:
                    raise ValueError(f"kv_from: {j} must name an earlier attention layer with projections of its own")
                lender = earlier[j].mix
            self.mix = TalkingAttentionMixer(width, m, eps, lender)
        else:
            raise ValueError(f"unknown mixer {kind!r}")
        self.norm1 = AffineNorm(width)
        if entry.get("mlp"):
            self.mlp = build_feed_forward(width, entry["mlp"])
            self.norm2 = AffineNorm(width)
        else:
            self.mlp = None


class FitevikForCausalLM(nn.Module):
    supports_fp32 = True            # every kernel of this stack has a true 32-bit form
    prefix_caching = False          # recurrent state at a prefix's end is not kept, so cached blocks are no use
    split_decode = False

    def __init__(self, config):
        super().__init__()
        if tp_rank_size()[1] != 1:
            raise ValueError("Fitevik runs on one GPU per replica (no tensor-parallel sharding of its mixers)")
        c = config.to_dict() if hasattr(config, "to_dict") else dict(config)
        self.eps = float(c["norm"]["eps"])
        W = c["width"]
        n_exp = max([e["mlp"]["router"]["experts"] for e in c["layers"]
                     if e.get("mlp") and e["mlp"].get("kind") == "moe"] or [0])
        self.spec = FitevikSpec(c["vocab"], W, len(c["layers"]), self.eps, num_experts=n_exp)
        self.embed_tokens = VocabParallelEmbedding(c["vocab"], W)
        self.positions = VocabParallelEmbedding(int(c["max_positions"]), W)         # learned, added unscaled
        self.embed_norm = AffineNorm(W)
        layers: list[FitevikLayer] = []
        for entry in c["layers"]:
            layers.append(FitevikLayer(W, entry, self.eps, layers))
        self.layers = nn.ModuleList(layers)
        self.norm = AffineNorm(W)
        self.lm_head = ParallelLMHead(c["vocab"], W, scale=float(c.get("logit_scale", 1.0)))
        self.trace_layers = None                       # a list: the residual stream after every layer is appended

    # ------------------------------------------------------------------ forward
    def _sublayers(self):
        """(callable, output norm, closes a layer) in execution order."""
        out = []
        for layer in self.layers:
            out.append((layer.mix, layer.norm1, layer.mlp is None))
            if layer.mlp is not None:
                out.append((lambda pos, h, f=layer.mlp: f(h), layer.norm2, True))
        return out

    def forward(self, input_ids, positions):
        # index tensors that the layers share live for ONE pass: a context may see several passes (an eager pass, then
        # the capture of a CUDA graph), and what an earlier pass computed is neither current nor part of the graph
        get_context().scratch.clear()
        dtype = self.embed_tokens.weight.dtype
        T, W = input_ids.shape[0], self.spec.hidden_size
        x = torch.empty(T, W, dtype=torch.float32, device=input_ids.device)            # the residual stream
        n0 = self.embed_norm
        h = ops.norm_residual_(x, self.embed_tokens.weight, n0.weight, n0.bias, self.eps, dtype, accumulate=False,
                               y_index=input_ids, y2=self.positions.weight, y2_index=positions)
        for fn, norm, closes in self._sublayers():
            y = fn(positions, h).contiguous()
            h = ops.norm_residual_(x, y, norm.weight, norm.bias, self.eps, dtype)
            if closes and self.trace_layers is not None:
                self.trace_layers.append(x.clone())
        return ops.stream_mix_norm_(x.view(T, 1, W), None, None, None, None, self.norm.weight, self.norm.bias,
                                    self.eps, dtype)

    def compute_logits(self, hidden_states):
        return self.lm_head(hidden_states)

    # ------------------------------------------------------------------ weights
    def route_checkpoint_tensor(self, name: str):
        """Checkpoint tensor name -> (parameter name, shard id or None)."""
        top = {"embed": "embed_tokens.weight", "pos": "positions.weight", "head": "lm_head.weight",
               "embed.norm": "embed_norm.weight", "embed.norm.b": "embed_norm.bias",
               "final.norm": "norm.weight", "final.norm.b": "norm.bias"}
        if name in top:
            return top[name], None
        layer, _, rest = name.partition(".")
        i = int(layer[1:])
        base = f"layers.{i}."
        if rest in ("norm1", "norm2"):
            return base + rest + ".weight", None
        if rest in ("norm1.b", "norm2.b"):
            return base + rest[:5] + ".bias", None
        if rest.startswith("mlp."):
            key = rest[4:]
            if isinstance(self.layers[i].mlp, TopkSoftmaxMoe):
                if key == "router":
                    return base + "mlp.router", None
                if key == "router.b":
                    return base + "mlp.router_bias", None
                e, part = key.split(".")
                return base + "mlp." + {"up": "w1", "down": "w2"}[part], int(e[1:])
            return {"up": (base + "mlp.up_proj.weight", None), "up.b": (base + "mlp.up_proj.bias", None),
                    "down": (base + "mlp.down_proj.weight", None), "down.b": (base + "mlp.down_proj.bias", None)}[key]
        key = rest[4:]                                  # after "mix."
        mix = self.layers[i].mix
        if key == "o":
            return base + "mix.o_proj.weight", None
        if isinstance(mix, Hgrn2Mixer):
            return {"q": (base + "mix.proj.weight", 0), "f": (base + "mix.proj.weight", 1),
                    "v": (base + "mix.proj.weight", 2), "f.b": (base + "mix.rec.gate_bias", None),
                    "lower": (base + "mix.rec.lower", None), "norm": (base + "mix.norm.weight", None)}[key]
        return {"q": (base + "mix.proj.weight", 0), "k": (base + "mix.proj.weight", 1),
                "v": (base + "mix.proj.weight", 2), "q.norm": (base + "mix.q_norm", None),
                "k.norm": (base + "mix.k_norm", None), "talk": (base + "mix.attn.talk", None),
                "sink": (base + "mix.attn.sink", None)}[key]

    @torch.no_grad()
    def random_init(self, seed: int = 0, std: float | None = None) -> None:
        """Random weights for synthetic runs: matrices N(0, 1/fan_in), norm weights near one, biases small, head-mixing
        matrices near the identity, lower bounds of the forget gates spread over (0, 1)."""
        g = torch.Generator().manual_seed(seed)
        for name, p in sorted(self.named_parameters()):
            if name.endswith("attn.talk"):
                v = torch.eye(p.shape[0]) + 0.1 * torch.randn(p.shape, generator=g)
            elif name.endswith("rec.lower"):
                v = torch.rand(p.shape, generator=g) * 0.9
            elif name.endswith(".bias") or name.endswith("_bias") or name.endswith("attn.sink"):
                v = 0.1 * torch.randn(p.shape, generator=g)
            elif p.dim() == 1:
                v = 1 + 0.1 * torch.randn(p.shape, generator=g)
            elif name in ("embed_tokens.weight", "positions.weight"):
                v = torch.randn(p.shape, generator=g)
            else:
                v = torch.randn(p.shape, generator=g) * (std if std is not None else p.shape[-1] ** -0.5)
            p.data.copy_(v.to(p.dtype))
        for layer in self.layers:
            if isinstance(layer.mix, Hgrn2Mixer):
                layer.mix.norm.weight.data.copy_(layer.mix.norm.weight.data[:layer.mix.dv].repeat(layer.mix.H))
