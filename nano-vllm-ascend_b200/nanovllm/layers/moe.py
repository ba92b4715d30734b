"""Sparse mixture-of-experts MLP on the csrc/moe.cu kernels (reference: ``Qwen3MoeSparseMoeBlock``,
models/qwen3_moe.py:125-186, and its expert ``Qwen3MoeMLP`` :95-122).

Parameter names are the reference's -- ``gate.weight``, ``experts.N.gate_up_proj.weight`` (loaded
from ``gate_proj`` / ``up_proj`` through the packed-module mapping), ``experts.N.down_proj.weight``
-- but the storage is not: every rank keeps the experts it owns stacked in two tensors
(``w13 [n_local, 2*I, h]``, ``w2 [n_local, h, I]``) that the grouped kernels index by expert, and
the per-expert parameters are views into them, so checkpoints and the seeded initialiser fill the
stacks without knowing about them.

Parallel layout (differs from the reference on purpose): the reference shards every expert's
matrices across the tensor-parallel group and all-reduces once per expert inside a Python loop
(qwen3_moe.py:101-112,176-186). Here a rank owns ``E / tp`` experts WHOLE (expert parallelism over
the same group); tokens are already replicated on every rank, so dispatch is a local selection
and the combine is ONE sum all-reduce of the layer output -- the same collective a dense row-
parallel ``down_proj`` issues, fused with the following add+RMSNorm when it fits (comm.py).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from .. import ops
from .linear import ReplicatedLinear, tp_collectives, tp_rank_size


class _ExpertMatrix(nn.Module):
    """One expert matrix: ``weight`` is a view into the rank's stacked tensor."""

    def __init__(self, storage: torch.Tensor, output_sizes: list[int] | None):
        super().__init__()
        self.weight = nn.Parameter(storage, requires_grad=False)
        self.weight.weight_loader = self.weight_loader
        self.tp_dim, self.tp_size = None, 1            # never sharded: experts are placed, not cut
        if output_sizes is not None:
            self.output_sizes = output_sizes           # gate | up, routed by shard id like a merged linear

    def weight_loader(self, param, loaded_weight, loaded_shard_id: int | None = None):
        if loaded_shard_id is None:
            param.data.copy_(loaded_weight)
            return
        start = sum(self.output_sizes[:loaded_shard_id])
        param.data.narrow(0, start, self.output_sizes[loaded_shard_id]).copy_(loaded_weight)


class _Expert(nn.Module):

    def __init__(self, w13: torch.Tensor, w2: torch.Tensor, inter: int):
        super().__init__()
        self.gate_up_proj = _ExpertMatrix(w13, [inter, inter])
        self.down_proj = _ExpertMatrix(w2, None)


class SparseMoeBlock(nn.Module):

    def __init__(self, hidden_size: int, moe_intermediate_size: int, num_experts: int, top_k: int):
        super().__init__()
        self.ep_rank, self.ep_size = tp_rank_size()
        if num_experts % self.ep_size:
            raise ValueError(f"{num_experts} experts do not divide over {self.ep_size} ranks")
        if top_k > 8 or num_experts > 256:
            raise ValueError("moe kernels support top_k <= 8 and <= 256 experts")
        self.hidden_size, self.inter, self.num_experts, self.top_k = (
            hidden_size, moe_intermediate_size, num_experts, top_k)
        self.num_local = num_experts // self.ep_size
        self.expert_begin = self.ep_rank * self.num_local
        self.gate = ReplicatedLinear(hidden_size, num_experts, bias=False)
        self.register_buffer("w13", torch.empty(self.num_local, 2 * self.inter, hidden_size), persistent=False)
        self.register_buffer("w2", torch.empty(self.num_local, hidden_size, self.inter), persistent=False)
        # sparse ModuleDict keyed by the GLOBAL expert index, so parameter names match the checkpoint
        self.experts = nn.ModuleDict({
            str(self.expert_begin + i): _Expert(self.w13[i], self.w2[i], self.inter)
            for i in range(self.num_local)})
        self.defer_allreduce = False       # set by the decoder layer: the next op is an add+RMSNorm

    def nonlocal_param_shapes(self, prefix: str) -> dict[str, tuple[int, ...]]:
        """Names/shapes of the expert parameters other ranks hold (the seeded initialiser numbers
        parameters over the FULL name list so that every layout draws the same weights)."""
        out = {}
        for e in range(self.num_experts):
            if not self.expert_begin <= e < self.expert_begin + self.num_local:
                out[f"{prefix}experts.{e}.gate_up_proj.weight"] = (2 * self.inter, self.hidden_size)
                out[f"{prefix}experts.{e}.down_proj.weight"] = (self.hidden_size, self.inter)
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        tokens, hidden = x.shape
        router_logits = F.linear(x, self.gate.weight)
        topk_ids, topk_w = ops.moe_route(router_logits, self.top_k)
        plan = ops.moe_align(topk_ids, self.expert_begin, self.num_local)
        out = None
        if self.ep_size > 1 and self.defer_allreduce:
            from ..comm import get_comm
            comm = get_comm()
            if comm is not None and comm.fits(tokens, hidden, x.dtype.itemsize):
                out = comm.partial_buffer(tokens, hidden, x.dtype)   # RMSNorm completes the all-reduce
                return ops.moe_experts(x, self.w13, self.w2, topk_ids, topk_w, plan, out=out)
        y = ops.moe_experts(x, self.w13, self.w2, topk_ids, topk_w, plan)
        if self.ep_size > 1 and tp_collectives():
            dist.all_reduce(y)
        return y


class GroupedSigmoidMoe(nn.Module):
    """Mixture of experts with a sigmoid router: choice scores are sigmoid(z) plus a stored correction, experts form
    ``groups`` equal groups of neighbours of which only the ``keep`` best (by the sum of their two largest choice
    scores) stay in play, ``top_k`` experts are chosen and weighted by their sigmoid scores, normalised and scaled.
    The router runs in fp32 (ops.moe_route_grouped); experts are gate/up/down MLPs with silu, stacked in two tensors.
    16-bit models whose sizes fit the tensor-core kernels of csrc/moe.cu run the expert GEMMs there, everything else
    (fp32, other sizes) on the generic kernels of csrc/moe_generic.cu with fp32 routing weights."""

    def __init__(self, hidden_size: int, inter: int, num_experts: int, top_k: int, groups: int = 1, keep: int = 1,
                 scale: float = 1.0):
        super().__init__()
        if tp_rank_size()[1] != 1:
            raise ValueError("GroupedSigmoidMoe holds every expert on one GPU")
        self.hidden_size, self.inter, self.num_experts, self.top_k = hidden_size, inter, num_experts, top_k
        self.groups, self.keep, self.scale = groups, keep, scale
        self.router = nn.Parameter(torch.empty(num_experts, hidden_size, dtype=torch.float32))
        self.correction = nn.Parameter(torch.zeros(num_experts, dtype=torch.float32))
        self.w13 = nn.Parameter(torch.empty(num_experts, 2 * inter, hidden_size))
        self.w2 = nn.Parameter(torch.empty(num_experts, hidden_size, inter))
        self.w13.weight_loader = self._load_w13
        self.w2.weight_loader = lambda p, w, e: p.data[e].copy_(w)
        self.fast = True           # False: always the generic kernels

    def _load_w13(self, param, loaded, shard):
        e, part = shard                                                  # part 0: gate rows, 1: up rows
        param.data[e, part * self.inter:(part + 1) * self.inter].copy_(loaded)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = F.linear(x.float(), self.router)
        ids, w = ops.moe_route_grouped(logits, self.correction, self.top_k, self.groups, self.keep, self.scale)
        plan = ops.moe_align(ids, 0, self.num_experts)
        if (self.fast and x.dtype != torch.float32 and self.hidden_size % 128 == 0 and self.inter % 64 == 0
                and self.top_k <= 8 and self.num_experts <= 256):
            return ops.moe_experts(x, self.w13, self.w2, ids, w.to(x.dtype), plan)
        return ops.moe_experts_generic(x, self.w13, self.w2, w, plan)


class GroupedSoftmaxMoe(nn.Module):
    """Mixture of experts with a softmax router: s = softmax(z) over all experts in fp32, experts form ``groups`` equal
    groups of neighbours of which only the ``keep`` best (by their largest s) stay in play, ``top_k`` experts are chosen
    and weighted by s / (sum of the chosen s + 1e-20). Experts are gate/up/down MLPs without biases, stacked in two
    tensors; ``glu = (alpha, limit)`` selects the clamped unit g sigmoid(alpha g) (u + 1) with g = min(gate, limit),
    u = clamp(up, +-limit) in place of silu(g) u. 16-bit models whose sizes fit run the expert GEMMs on the tensor-core
    kernels (the grouped tcgen05 GEMM of csrc/moe_umma.cu for prompt-sized batches, the weight-streaming kernels of
    csrc/moe.cu below that); everything else (fp32, other sizes) on the generic kernels of csrc/moe_generic.cu with
    fp32 routing weights."""

    def __init__(self, hidden_size: int, inter: int, num_experts: int, top_k: int, groups: int = 1, keep: int = 1,
                 glu: tuple[float, float] | None = None):
        super().__init__()
        if tp_rank_size()[1] != 1:
            raise ValueError("GroupedSoftmaxMoe holds every expert on one GPU")
        self.hidden_size, self.inter, self.num_experts, self.top_k = hidden_size, inter, num_experts, top_k
        self.groups, self.keep, self.glu = groups, keep, glu
        self.router = nn.Parameter(torch.empty(num_experts, hidden_size, dtype=torch.float32))
        self.w13 = nn.Parameter(torch.empty(num_experts, 2 * inter, hidden_size))
        self.w2 = nn.Parameter(torch.empty(num_experts, hidden_size, inter))
        self.w13.weight_loader = self._load_w13
        self.w2.weight_loader = lambda p, w, e: p.data[e].copy_(w)
        self.fast = True           # False: always the generic kernels

    def _load_w13(self, param, loaded, shard):
        e, part = shard                                                  # part 0: gate rows, 1: up rows
        param.data[e, part * self.inter:(part + 1) * self.inter].copy_(loaded)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = F.linear(x.float(), self.router)
        ids, w = ops.moe_route_grouped_softmax(logits, self.top_k, self.groups, self.keep)
        plan = ops.moe_align(ids, 0, self.num_experts)
        if (self.fast and x.dtype != torch.float32 and self.hidden_size % 128 == 0 and self.inter % 64 == 0
                and self.top_k <= 8 and self.num_experts <= 256):
            if self.glu is None:
                return ops.moe_experts(x, self.w13, self.w2, ids, w.to(x.dtype), plan)
            return ops.moe_experts_glu_clamped(x, self.w13, self.w2, ids, w.to(x.dtype), plan, *self.glu)
        return ops.moe_experts_generic(x, self.w13, self.w2, w, plan, glu=self.glu)


class TopkSoftmaxMoe(nn.Module):
    """Mixture of experts whose router is a plain linear map with a bias, computed in fp32: the ``top_k`` experts with
    the largest logits are chosen and weighted by the softmax over the chosen logits only. Experts are feed-forwards
    WITHOUT a gate, W_down act(W_up h), no biases, stacked in two tensors (``w1`` [E, inter, hidden], ``w2`` [E, hidden,
    inter]). 16-bit models whose sizes fit the tensor-core kernels run the expert GEMMs on them (ops.moe_experts_ungated:
    the grouped tcgen05 GEMM for prompt-sized batches, the weight-streaming kernels below that), everything else (fp32,
    other sizes) on the generic kernels of csrc/moe_generic.cu with fp32 routing weights in an fp32 combine."""

    def __init__(self, hidden_size: int, inter: int, num_experts: int, top_k: int, act: str = "relu2"):
        super().__init__()
        if tp_rank_size()[1] != 1:
            raise ValueError("TopkSoftmaxMoe holds every expert on one GPU")
        self.hidden_size, self.inter, self.num_experts, self.top_k, self.act = hidden_size, inter, num_experts, top_k, act
        self.router = nn.Parameter(torch.empty(num_experts, hidden_size, dtype=torch.float32))
        self.router_bias = nn.Parameter(torch.zeros(num_experts, dtype=torch.float32))
        self.w1 = nn.Parameter(torch.empty(num_experts, inter, hidden_size))
        self.w2 = nn.Parameter(torch.empty(num_experts, hidden_size, inter))
        self.w1.weight_loader = lambda p, w, e: p.data[e].copy_(w)
        self.w2.weight_loader = lambda p, w, e: p.data[e].copy_(w)
        self.fast = True           # False: always the generic kernels

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = F.linear(x.float(), self.router)
        ids, w = ops.moe_route_topk(logits, self.router_bias, self.top_k)
        plan = ops.moe_align(ids, 0, self.num_experts)
        if (self.fast and x.dtype != torch.float32 and self.hidden_size % 128 == 0 and self.inter % 128 == 0
                and self.top_k <= 8 and self.num_experts <= 256):
            return ops.moe_experts_ungated(x, self.w1, self.w2, ids, w.to(x.dtype), plan, act=self.act)
        return ops.moe_experts_generic(x, self.w1, self.w2, w, plan, act=self.act)
