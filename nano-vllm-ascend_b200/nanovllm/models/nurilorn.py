"""Nurilorn: a decoder whose layers are listed one by one in its configuration; every layer is a gated softmax
attention and an optional feed-forward (dense with a clamped gated unit, or a mixture of experts with a grouped
softmax router), on an fp32 residual stream with scaled branches and RMS norms taken in groups.

    x <- E[token] * embedding.scale
    x <- x + m * (ls1 . mixer(N1(x)));   x <- x + m * (ls2 . ff(N2(x)));   logits = logit_scale * head N(x)
    N(x): the row in `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps), times a weight

  attention   q, k, v projections without bias -> short causal convolution over time on every channel -> rotary
              positions on the first rot.dims columns of every q and k head (pairs (2i, 2i+1); frequencies stretched
              band by band, layers.seq_mixers.BandScaledRotary) -> in every layer that says v_mix but the first such
              one, v <- (1 - lambda) v + lambda v_first with v_first that first layer's values of the same token
              (the blended v is what the cache holds) -> scores scale q.k capped by c tanh(s / c), causal, softmax
              with one added to the denominator (a sink of logit 0 without a value) -> head h times sigmoid(W_g x)_h
              -> W_o

Launches per mixer sublayer: one GEMM in (q | k | v | gate logits fused), the convolution, ONE kernel for rotation +
value blending + K/V scatter, the attention kernel (the gate in its epilogue, or a small gate kernel after the tensor-core
kernels), one GEMM out, and ONE kernel for "scale the branch, add it to the stream, grouped norm for the next sublayer".
What the design fixes is a constant here; every size and every constant that may differ between models comes from
the config.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from .. import ops
from ..layers.activation import ClampedGatedFeedForward
from ..layers.embed_head import ParallelLMHead, VocabParallelEmbedding
from ..layers.linear import MergedColumnParallelLinear, RowParallelLinear, tp_rank_size
from ..layers.moe import GroupedSoftmaxMoe
from ..layers.seq_mixers import BandScaledRotary, ShortConv, VarSizeAttention, small_param
from ..utils.context import get_context

GLU_ALPHA = 1.702          # slope of the sigmoid in the feed-forwards' gated unit
SINK_LOGIT = 0.0           # the softmax denominator's extra entry: exp(0) = 1
FIRST_VALUES = "first mixed values"      # key of the per-pass scratch: the value rows later layers blend in


@dataclass
class NurilornSpec:
    """What the runner asks of a model's spec."""
    vocab_size: int
    hidden_size: int
    num_layers: int
    rms_eps: float
    num_experts: int = 0
    tie_embeddings: bool = False


class BranchNorm(nn.Module):
    """Weight of one grouped norm of the residual path; the arithmetic runs fused with the residual update."""

    def __init__(self, size: int):
        super().__init__()
        self.weight = small_param(size, fill=1.0)


class GatedCappedAttention(nn.Module):

    def __init__(self, width: int, m: dict):
        super().__init__()
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        self.H, self.G, self.d, self.dv = H, G, d, dv
        self.sizes = [H * d, G * d, G * dv, H]                          # q | k | v | gate logit per head
        self.proj = MergedColumnParallelLinear(width, self.sizes)
        taps = int(m.get("conv") or 0)
        self.conv = ShortConv(self.sizes[:3], taps) if taps else None
        rot = m.get("rot") or {"dims": 0, "base": 1.0}
        self.rot = BandScaledRotary(rot["dims"], rot["base"], interleaved=True, scaling=rot.get("scaling"))
        self.v_mix = bool(m.get("v_mix"))
        self.vmix = small_param(1)                                      # lambda; unused in the first blending layer
        self.attn = VarSizeAttention(H, G, d, dv, float(m["scale"]), softcap=float(m.get("softcap") or 0.0),
                                     sink=SINK_LOGIT)
        self.o_proj = RowParallelLinear(H * dv, width)

    def forward(self, positions, h):
        qkvg = self.proj(h)
        nq, nk, nv = self.sizes[:3]
        qkv = qkvg[:, :nq + nk + nv]
        qkv = self.conv(qkv) if self.conv is not None else qkv.contiguous()
        attn = self.attn
        ctx = get_context()
        v_first = ctx.scratch.get(FIRST_VALUES) if self.v_mix else None
        if v_first is not None and v_first.shape[1] != nv:
            raise ValueError("layers that blend values need the first such layer's kv head count and value size")
        have_cache = attn.k_cache.numel() > 0 and ctx.slot_mapping is not None
        ops.rope_mix_cache(qkv, self.rot.table(positions), self.H, self.G, self.d, self.dv, self.rot.dims,
                           self.rot.interleaved, v_other=v_first, lam=self.vmix if v_first is not None else None,
                           k_cache=attn.k_cache if have_cache else None, v_cache=attn.v_cache if have_cache else None,
                           slots=ctx.slot_mapping if have_cache else None)
        if self.v_mix and v_first is None:
            ctx.scratch[FIRST_VALUES] = qkv[:, nq + nk:]                # the first blending layer's own values
        q = qkv[:, :nq].unflatten(1, (self.H, self.d))
        k = qkv[:, nq:nq + nk].unflatten(1, (self.G, self.d))
        v = qkv[:, nq + nk:].unflatten(1, (self.G, self.dv))
        return self.o_proj(attn(q, k, v, gate=qkvg[:, nq + nk + nv:]))


MIXERS = {"attention": GatedCappedAttention}


def build_feed_forward(width: int, mlp: dict) -> nn.Module:
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return ClampedGatedFeedForward(width, mlp["ff"], mlp["limit"], GLU_ALPHA)
    if kind == "moe":
        r = mlp["router"]
        groups = r.get("groups") or {}
        return GroupedSoftmaxMoe(width, mlp["expert"]["ff"], r["experts"], r["top"], groups.get("count", 1),
                                 groups.get("keep", 1), glu=(GLU_ALPHA, float(mlp["expert"]["limit"])))
    raise ValueError(f"unknown feed-forward kind {kind!r}")


class NurilornLayer(nn.Module):

    def __init__(self, width: int, entry: dict):
        super().__init__()
        if entry["type"] not in MIXERS:
            raise ValueError(f"unknown mixer {entry['type']!r}")
        self.mix = MIXERS[entry["type"]](width, entry["mixer"])
        self.norm1, self.ls1 = BranchNorm(width), small_param(width, fill=1.0)
        if entry.get("mlp"):
            self.mlp = build_feed_forward(width, entry["mlp"])
            self.norm2, self.ls2 = BranchNorm(width), small_param(width, fill=1.0)
        else:
            self.mlp = None


class NurilornForCausalLM(nn.Module):
    supports_fp32 = True            # every kernel of this stack has a true 32-bit form
    prefix_caching = False          # the convolution tails at a prefix's end are not kept, so cached blocks are no use
    split_decode = False

    def __init__(self, config):
        super().__init__()
        if tp_rank_size()[1] != 1:
            raise ValueError("Nurilorn runs on one GPU per replica (no tensor-parallel sharding of its mixers)")
        c = config.to_dict() if hasattr(config, "to_dict") else dict(config)
        norm = c.get("norm") or {}
        self.eps, self.groups = float(norm.get("eps", 1e-6)), int(norm.get("groups", 1))
        self.mult = float(c.get("residual_mult", 1.0))
        self.embed_scale = float((c.get("embedding") or {}).get("scale", 1.0))
        W = c["width"]
        if W % self.groups:
            raise ValueError(f"width {W} does not split into {self.groups} norm groups")
        n_exp = max([e["mlp"]["router"]["experts"] for e in c["layers"]
                     if e.get("mlp") and e["mlp"].get("kind") == "moe"] or [0])
        self.spec = NurilornSpec(c["vocab"], W, len(c["layers"]), self.eps, num_experts=n_exp)
        self.embed_tokens = VocabParallelEmbedding(c["vocab"], W)
        self.layers = nn.ModuleList([NurilornLayer(W, entry) for entry in c["layers"]])
        self.norm = BranchNorm(W)
        self.lm_head = ParallelLMHead(c["vocab"], W, scale=float(c.get("logit_scale", 1.0)))
        self.trace_layers = None                       # a list: the residual stream after every layer is appended

    # ------------------------------------------------------------------ forward
    def _sublayers(self):
        """(norm, layer scale, callable, closes a layer) in execution order."""
        out = []
        for layer in self.layers:
            out.append((layer.norm1, layer.ls1, layer.mix, layer.mlp is None))
            if layer.mlp is not None:
                out.append((layer.norm2, layer.ls2, lambda pos, h, f=layer.mlp: f(h), True))
        return out

    def forward(self, input_ids, positions):
        # what the layers share lives for ONE pass: a context may see several passes (an eager pass, then the capture
        # of a CUDA graph), and what an earlier pass computed is neither current nor part of the graph
        get_context().scratch.clear()
        table = self.embed_tokens.weight
        dtype = table.dtype
        ids = input_ids.to(torch.int64).contiguous()
        x = torch.empty(ids.numel(), table.shape[1], dtype=torch.float32, device=table.device)
        subs = self._sublayers()
        norm = lambda w: dict(w=w, eps=self.eps, groups=self.groups, dtype=dtype)
        # the scaled embedding and the first norm in one launch
        h = ops.residual_scale_groupnorm_(x, table, None, self.embed_scale, accumulate=False, y_index=ids,
                                          **norm(subs[0][0].weight if subs else self.norm.weight))
        for i, (_, ls, fn, closes) in enumerate(subs):
            y = fn(positions, h).contiguous()
            nxt = subs[i + 1][0] if i + 1 < len(subs) else self.norm
            h = ops.residual_scale_groupnorm_(x, y, ls, self.mult, **norm(nxt.weight))
            if closes and self.trace_layers is not None:
                self.trace_layers.append(x.clone())
        return h                                       # already through the final norm

    def compute_logits(self, hidden_states):
        return self.lm_head(hidden_states)

    # ------------------------------------------------------------------ weights
    def route_checkpoint_tensor(self, name: str):
        """Checkpoint tensor name -> (parameter name, shard id or None)."""
        if name == "embed":
            return "embed_tokens.weight", None
        if name == "head":
            return "lm_head.weight", None
        if name == "final.norm":
            return "norm.weight", None
        layer, _, rest = name.partition(".")
        i = int(layer[1:])
        base = f"layers.{i}."
        if rest in ("norm1", "norm2"):
            return base + rest + ".weight", None
        if rest in ("ls1", "ls2"):
            return base + rest, None
        if rest.startswith("mlp."):
            key = rest[4:]
            if isinstance(self.layers[i].mlp, GroupedSoftmaxMoe):
                if key == "router":
                    return base + "mlp.router", None
                e, part = key.split(".")
                e = int(e[1:])
                return {"gate": (base + "mlp.w13", (e, 0)), "up": (base + "mlp.w13", (e, 1)),
                        "down": (base + "mlp.w2", e)}[part]
            return {"gate": (base + "mlp.gate_up_proj.weight", 0), "up": (base + "mlp.gate_up_proj.weight", 1),
                    "down": (base + "mlp.down_proj.weight", None)}[key]
        key = rest[4:]                                  # after "mix."
        if key == "o":
            return base + "mix.o_proj.weight", None
        if key == "vmix":
            return base + "mix.vmix", None
        head, _, tail = key.partition(".")
        shard = "qkvg".index(head)
        if tail == "":
            return base + "mix.proj.weight", shard
        if tail == "conv":
            return base + "mix.conv.weight", shard
        raise KeyError(name)

    @torch.no_grad()
    def random_init(self, seed: int = 0, std: float | None = None) -> None:
        """Random weights for synthetic runs: matrices N(0, 1/fan_in), norm weights and layer scales near one, taps
        of the order of one, blending weights inside (0.2, 0.8)."""
        g = torch.Generator().manual_seed(seed)
        for name, p in sorted(self.named_parameters()):
            if name.endswith("conv.weight"):
                v = 0.5 * torch.randn(p.shape, generator=g)
            elif name.endswith(".vmix"):
                v = 0.2 + 0.6 * torch.rand(p.shape, generator=g)
            elif p.dim() == 1:
                v = 1 + 0.1 * torch.randn(p.shape, generator=g)
            elif name == "embed_tokens.weight":
                v = torch.randn(p.shape, generator=g) / self.embed_scale
            else:
                v = torch.randn(p.shape, generator=g) * (std if std is not None else p.shape[-1] ** -0.5)
            p.data.copy_(v.to(p.dtype))
