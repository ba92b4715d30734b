"""Nirelix: a decoder whose layers are listed one by one in its configuration. The residual is kept in several
fp32 streams that every sublayer reads as a weighted sum and rewrites through a mixing matrix; each layer has one
of three sequence mixers and an optional feed-forward (dense with a clamped gated unit, or a mixture of experts
with a grouped sigmoid router), each behind a layer norm with weight and bias.

    u = sum_s read[s] x_s;  y = sublayer(LN(u));  x_t <- sum_s mix[s, t] x_s + write[t] y     (all streams at once)

  retention         q, k, v, g projections; rotary positions (pairs (i, i + dims/2)) on q and k, k times dim^-1/2;
                    per head S <- decay_h S + k v^T, o = S^T q (fp32 state); o / rms(o) per head, times silu(g); W_o
  channel_delta     q, k, v projections -> short causal convolution + silu; q, k unit vectors per head, q times
                    dim^-1/2; beta = sigmoid(W_b h); a decay per head and key channel from a low-rank projection,
                    exp(-exp(A) softplus(W_a2 W_a1 h + bias)); gated delta rule (fp32 state); o / rms(o) per head times
                    a weight shared by the heads, times sigmoid(W_g2 W_g1 h); W_o
  latent_attention  query through a normed latent; ONE cached row per token = [normed key/value latent | rotated
                    shared key part] (pairs (2i, 2i+1)); sliding-window softmax attention with the up-projections
                    absorbed into the query and the output; times sigmoid(W_g h); W_o

Launches per mixer sublayer: one GEMM in (every projection that reads the sublayer input fused), the mechanism's
preparation kernel (rotary / convolution + unit vectors and decays / latent norms + cache write), the mixer kernel,
the gate/norm kernel, one GEMM out, and ONE kernel for "rewrite the streams, read them for the next sublayer, layer
norm". What the design fixes is a constant here; every size and every constant that may differ between models
comes from the config.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from .. import ops
from ..layers.activation import ClampedGatedFeedForward
from ..layers.embed_head import ParallelLMHead, VocabParallelEmbedding
from ..layers.linear import MergedColumnParallelLinear, PaddedMergedLinear, ReplicatedLinear, RowParallelLinear, tp_rank_size
from ..layers.moe import GroupedSigmoidMoe
from ..layers.seq_mixers import (DeltaRule, GatedNorm, LatentAttention, LinearRecurrence, Rotary, ShortConv,
                                 StreamResidual, small_param)
from ..utils.context import get_context

UNIT_EPS = 1e-6            # inside the root of the delta rule's unit vectors
GLU_ALPHA = 1.702          # slope of the sigmoid in the dense feed-forward's gated unit


@dataclass
class NirelixSpec:
    """What the runner asks of a model's spec."""
    vocab_size: int
    hidden_size: int
    num_layers: int
    rms_eps: float
    num_experts: int = 0
    tie_embeddings: bool = False


class AffineNorm(nn.Module):
    """Weight and bias of one layer norm; the arithmetic runs fused with the stream update."""

    def __init__(self, size: int):
        super().__init__()
        self.weight, self.bias = small_param(size, fill=1.0), small_param(size)


class RetentionMixer(nn.Module):

    def __init__(self, width: int, m: dict, eps: float):
        super().__init__()
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        self.H, self.d, self.dv = H, d, dv
        self.sizes = [H * d, H * d, H * dv, H * dv]                     # q | k | v | gate
        self.proj = MergedColumnParallelLinear(width, self.sizes)
        self.rot = Rotary(m["rot"]["dims"], m["rot"]["base"], interleaved=False)
        self.rec = LinearRecurrence(H, H, d, dv, decay=m["decay"])
        self.norm = GatedNorm(H * dv, eps, groups=H, gate_first=False, gate_act="silu")     # weight stays at one
        self.o_proj = RowParallelLinear(H * dv, width)

    def forward(self, positions, h):
        p = self.proj(h)
        nq, nk, nv, _ = self.sizes
        T, H, d = p.shape[0], self.H, self.d
        # q and k heads are neighbours in the projection: one launch rotates both, k is scaled after the rotation
        qk = self.rot(p[:, :nq + nk].unflatten(1, (2 * H, d)), positions, out_f32=True, split=H, scale_lo=1.0,
                      scale_hi=d ** -0.5).view(T, 2 * H * d)
        o = self.rec(qk[:, :nq], qk[:, nq:], p[:, nq + nk:nq + nk + nv])
        return self.o_proj(self.norm(o, p[:, nq + nk + nv:]))


class ChannelDeltaMixer(nn.Module):

    def __init__(self, width: int, m: dict, eps: float, rank_a: int, rank_g: int):
        super().__init__()
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        self.H, self.G, self.d, self.dv = H, G, d, dv
        self.nqk = 2 * G * d
        self.proj = MergedColumnParallelLinear(width, [G * d, G * d, H * dv])           # q | k | v (convolved)
        # the small projections that read the same input: decay latent | gate latent | beta
        self.small = PaddedMergedLinear(width, [rank_a, rank_g, H])
        self.a_up = PaddedMergedLinear(rank_a, [H * d], pad_input=True)
        self.g_up = PaddedMergedLinear(rank_g, [H * dv], pad_input=True)
        self.conv = ShortConv([G * d, G * d, H * dv], m["conv"], act="silu")
        self.rule = DeltaRule(H, G, d, dv, unit_eps=UNIT_EPS)
        self.norm = GatedNorm(H * dv, eps, groups=H, gate_first=False, gate_act="sigmoid")
        self.norm.weight.weight_loader = lambda p, w: p.data.copy_(w.repeat(H))         # one [vdim] weight for all heads
        self.o_proj = RowParallelLinear(H * dv, width)

    def forward(self, positions, h):
        qkv = self.conv(self.proj(h))
        s = self.small(h)
        a = self.a_up.part(self.a_up(self.small.padded_part(s, 0)), 0)
        gate = self.g_up.part(self.g_up(self.small.padded_part(s, 1)), 0)
        o = self.rule(qkv[:, :self.nqk], qkv[:, self.nqk:], a, self.small.part(s, 2))
        return self.o_proj(self.norm(o, gate))


class LatentAttentionMixer(nn.Module):

    def __init__(self, width: int, m: dict, eps: float):
        super().__init__()
        H, d, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
        self.H, self.d, self.dr, self.dv, self.eps = H, d, dr, dv, eps
        self.q_rank, self.rank = m["q_rank"], m["kv_rank"]
        self.proj = PaddedMergedLinear(width, [self.q_rank, self.rank + dr, H * dv])     # dq | dkv | gate
        self.q_norm, self.kv_norm = small_param(self.q_rank, fill=1.0), small_param(self.rank, fill=1.0)
        self.q_up = ReplicatedLinear(self.q_rank, H * (d + dr))
        self.rot = Rotary(m["rot"]["dims"], m["rot"]["base"], interleaved=True)
        self.attn = LatentAttention(H, d, dr, dv, self.rank, m.get("scale", (d + dr) ** -0.5),
                                    window=(m.get("mask") or {}).get("size", 0))
        self.gate = GatedNorm(H * dv, eps, norm=False)
        self.o_proj = RowParallelLinear(H * dv, width)

    def forward(self, positions, h):
        p = self.proj(h)
        attn = self.attn
        ctx = get_context()
        have_cache = attn.k_cache.numel() > 0 and ctx.slot_mapping is not None
        cq, kc = ops.latent_kv_prep(self.proj.part(p, 0), self.proj.part(p, 1), self.q_norm, self.kv_norm,
                                    positions, self.rank, self.dr, self.rot.dims, self.rot.base, True, self.eps,
                                    cache=attn.k_cache if have_cache else None,
                                    slots=ctx.slot_mapping if have_cache else None)
        q = self.q_up(cq).unflatten(1, (self.H, self.d + self.dr))
        o = attn(q[:, :, :self.d], lambda out: self.rot(q[:, :, self.d:], positions, out=out), kc)
        return self.o_proj(self.gate(o, self.proj.part(p, 2)))


MIXERS = {"retention": RetentionMixer, "channel_delta": ChannelDeltaMixer, "latent_attention": LatentAttentionMixer}


def build_feed_forward(width: int, mlp: dict) -> nn.Module:
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return ClampedGatedFeedForward(width, mlp["ff"], mlp["limit"], GLU_ALPHA)
    if kind == "moe":
        r = mlp["router"]
        groups = r.get("groups") or {}
        return GroupedSigmoidMoe(width, mlp["expert"]["ff"], r["experts"], r["top"], groups.get("count", 1),
                                 groups.get("keep", 1), r.get("scale", 1.0))
    raise ValueError(f"unknown feed-forward kind {kind!r}")


class NirelixLayer(nn.Module):

    def __init__(self, width: int, entry: dict, eps: float, streams: int, ranks=None):
        super().__init__()
        if entry["type"] not in MIXERS:
            raise ValueError(f"unknown mixer {entry['type']!r}")
        extra = ranks if entry["type"] == "channel_delta" else ()
        self.mix = MIXERS[entry["type"]](width, entry["mixer"], eps, *extra)
        self.norm1, self.hc1 = AffineNorm(width), StreamResidual(streams)
        if entry.get("mlp"):
            self.mlp = build_feed_forward(width, entry["mlp"])
            self.norm2, self.hc2 = AffineNorm(width), StreamResidual(streams)
        else:
            self.mlp = None


class NirelixForCausalLM(nn.Module):
    supports_fp32 = True            # every kernel of this stack has a true 32-bit form
    reads_checkpoint_shapes = True  # inner sizes of the delta mixers' low-rank projections are the tensors' shapes
    prefix_caching = False          # recurrent state at a prefix's end is not kept, so cached blocks are no use
    split_decode = False

    def __init__(self, config):
        super().__init__()
        if tp_rank_size()[1] != 1:
            raise ValueError("Nirelix runs on one GPU per replica (no tensor-parallel sharding of its mixers)")
        c = config.to_dict() if hasattr(config, "to_dict") else dict(config)
        self.eps = float(c["norm"]["eps"])
        W = c["width"]
        self.streams = int(c.get("streams", 1))          # without the key: one stream with unit weights = a plain residual
        self.has_stream_weights = "streams" in c
        n_exp = max([e["mlp"]["router"]["experts"] for e in c["layers"]
                     if e.get("mlp") and e["mlp"].get("kind") == "moe"] or [0])
        self.spec = NirelixSpec(c["vocab"], W, len(c["layers"]), self.eps, num_experts=n_exp)
        self.embed_tokens = VocabParallelEmbedding(c["vocab"], W)
        shapes = getattr(config, "checkpoint_shapes", None) or {}
        self.layers = nn.ModuleList([NirelixLayer(W, entry, self.eps, self.streams, self._ranks(i, entry, shapes))
                                     for i, entry in enumerate(c["layers"])])
        self.norm = AffineNorm(W)
        self.lm_head = ParallelLMHead(c["vocab"], W)
        self.trace_layers = None                       # a list: the sum of the streams after every layer is appended

    # ------------------------------------------------------------------ forward
    def _sublayers(self):
        """(norm, stream weights, callable, closes a layer) in execution order."""
        out = []
        for layer in self.layers:
            out.append((layer.norm1, layer.hc1, layer.mix, layer.mlp is None))
            if layer.mlp is not None:
                out.append((layer.norm2, layer.hc2, lambda pos, h, f=layer.mlp: f(h), True))
        return out

    def forward(self, input_ids, positions):
        # index tensors that the layers share live for ONE pass: a context may see several passes (an eager pass, then
        # the capture of a CUDA graph), and what an earlier pass computed is neither current nor part of the graph
        get_context().scratch.clear()
        dtype = self.embed_tokens.weight.dtype
        x = self.embed_tokens(input_ids).float()
        T, W = x.shape
        X = x.unsqueeze(1).repeat(1, self.streams, 1)                      # [T, streams, W] fp32
        subs = self._sublayers()
        n0, hc0 = subs[0][0], subs[0][1]
        h = ops.stream_mix_norm_(X, None, None, None, hc0.read, n0.weight, n0.bias, self.eps, dtype)
        for i, (_, hc, fn, closes) in enumerate(subs):
            y = fn(positions, h).contiguous()
            last = i + 1 == len(subs)
            nxt_norm = self.norm if last else subs[i + 1][0]
            nxt_read = None if last else subs[i + 1][1].read               # the model's output is the plain sum
            h = ops.stream_mix_norm_(X, y, hc.mix, hc.write, nxt_read, nxt_norm.weight, nxt_norm.bias, self.eps, dtype)
            if closes and self.trace_layers is not None:
                self.trace_layers.append(X.sum(1))
        return h                                       # already through the final norm

    def compute_logits(self, hidden_states):
        return self.lm_head(hidden_states)

    # ------------------------------------------------------------------ weights
    @staticmethod
    def _ranks(i: int, entry: dict, shapes: dict):
        """Inner sizes of layer i's low-rank decay and gate projections: the checkpoint tensors' shapes; a
        configuration without a checkpoint (synthetic weights) may give "decay_rank" / "gate_rank"."""
        m = entry["mixer"]
        if f"l{i}.mix.a1" in shapes:
            return shapes[f"l{i}.mix.a1"][0], shapes[f"l{i}.mix.g1"][0]
        default = max(1, m.get("dim", 16) // 4)
        return int(m.get("decay_rank", default)), int(m.get("gate_rank", default))

    def route_checkpoint_tensor(self, name: str):
        """Checkpoint tensor name -> (parameter name, shard id or None)."""
        if name == "embed":
            return "embed_tokens.weight", None
        if name == "head":
            return "lm_head.weight", None
        if name in ("final.norm", "final.norm.b"):
            return "norm." + ("bias" if name.endswith(".b") else "weight"), None
        layer, _, rest = name.partition(".")
        i = int(layer[1:])
        base = f"layers.{i}."
        if rest in ("norm1", "norm2"):
            return base + rest + ".weight", None
        if rest in ("norm1.b", "norm2.b"):
            return base + rest[:5] + ".bias", None
        if rest.startswith("hc"):
            which, key = rest.split(".")
            return base + which + "." + {"in": "read", "out": "write", "mix": "mix"}[key], None
        if rest.startswith("mlp."):
            key = rest[4:]
            if isinstance(self.layers[i].mlp, GroupedSigmoidMoe):
                if key in ("router", "correction"):
                    return base + "mlp." + key, None
                e, part = key.split(".")
                e = int(e[1:])
                return {"gate": (base + "mlp.w13", (e, 0)), "up": (base + "mlp.w13", (e, 1)),
                        "down": (base + "mlp.w2", e)}[part]
            return {"gate": (base + "mlp.gate_up_proj.weight", 0), "up": (base + "mlp.gate_up_proj.weight", 1),
                    "down": (base + "mlp.down_proj.weight", None)}[key]
        key = rest[4:]                                  # after "mix."
        mix = self.layers[i].mix
        if key == "o":
            return base + "mix.o_proj.weight", None
        if isinstance(mix, RetentionMixer):
            return base + "mix.proj.weight", "qkvg".index(key)
        if isinstance(mix, ChannelDeltaMixer):
            if key in ("q", "k", "v"):
                return base + "mix.proj.weight", "qkv".index(key)
            if key in ("q.conv", "k.conv", "v.conv"):
                return base + "mix.conv.weight", "qkv".index(key[0])
            return {"a1": (base + "mix.small.weight", 0), "g1": (base + "mix.small.weight", 1),
                    "b": (base + "mix.small.weight", 2), "a2": (base + "mix.a_up.weight", 0),
                    "g2": (base + "mix.g_up.weight", 0), "A_log": (base + "mix.rule.A_log", None),
                    "dt_bias": (base + "mix.rule.dt_bias", None), "norm": (base + "mix.norm.weight", None)}[key]
        return {"dq": (base + "mix.proj.weight", 0), "dkv": (base + "mix.proj.weight", 1),
                "g": (base + "mix.proj.weight", 2), "dq.norm": (base + "mix.q_norm", None),
                "dkv.norm": (base + "mix.kv_norm", None), "uq": (base + "mix.q_up.weight", None),
                "uk": (base + "mix.attn.w_uk", None), "uv": (base + "mix.attn.w_uv", None)}[key]

    @torch.no_grad()
    def random_init(self, seed: int = 0, std: float | None = None) -> None:
        """Random weights for synthetic runs: matrices N(0, 1/fan_in), norm weights near one, biases small, stream
        weights near a plain residual, decay parameters in the range where the recurrences neither vanish nor blow up."""
        g = torch.Generator().manual_seed(seed)
        S = self.streams
        for name, p in sorted(self.named_parameters()):
            if name.endswith("A_log"):
                v = torch.rand(p.shape, generator=g) * 2 - 3
            elif name.endswith("dt_bias") or name.endswith("correction"):
                v = 0.5 * torch.randn(p.shape, generator=g)
            elif name.endswith("conv.weight"):
                v = 0.5 * torch.randn(p.shape, generator=g)
            elif name.endswith(".mix"):
                v = torch.eye(S) + 0.1 * torch.randn(p.shape, generator=g)
            elif name.endswith(".read") or name.endswith(".write"):
                v = 1.0 / S ** 0.5 + 0.1 * torch.randn(p.shape, generator=g)
            elif name.endswith(".bias"):
                v = 0.1 * torch.randn(p.shape, generator=g)
            elif p.dim() == 1:
                v = 1 + 0.1 * torch.randn(p.shape, generator=g)
            elif name == "embed_tokens.weight":
                v = torch.randn(p.shape, generator=g)
            else:
                v = torch.randn(p.shape, generator=g) * (std if std is not None else p.shape[-1] ** -0.5)
            p.data.copy_(v.to(p.dtype))
        for layer in self.layers:                      # padding of the fused small projections stays zero
            mix = layer.mix
            if isinstance(mix, ChannelDeltaMixer):
                for m in (mix.small, mix.a_up, mix.g_up):
                    m.zero_padding()
                mix.norm.weight.data.copy_(mix.norm.weight.data[:mix.dv].repeat(mix.H))
            elif isinstance(mix, LatentAttentionMixer):
                mix.proj.zero_padding()
            elif isinstance(mix, RetentionMixer):
                mix.norm.weight.data.fill_(1.0)
