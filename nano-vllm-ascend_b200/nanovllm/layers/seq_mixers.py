"""Building blocks of hybrid decoders: a short causal convolution with a carried tail, linear recurrences
with an fp32 state (constant decay per head, the selective state-space form, a forget gate per key channel that also
decides what is written, or the gated delta rule with a decay per key channel), the gated norms that follow them,
rotary positions on part of a head (plain, or with frequencies stretched by a ramp between a fast and a slow band),
causal softmax attention whose key and value sizes may differ (optionally inside a sliding window, with capped scores,
a sink in the denominator and a gate per head), attention whose heads are mixed before the softmax (with a distance bias, a sink, and keys and
values that may be another layer's), attention over a cached latent, and the mixing weights of a residual that is
kept in several streams.

Every block reads the step's ``Context`` (which tokens belong to which sequence, their cache slots and
state slots) and runs on the kernels of ``csrc/seq_ops.cu`` / ``csrc/seq_mixers.cu``. Per-sequence state is
NOT owned by the blocks: a block declares what it needs per sequence (``state_shapes``), the runner
allocates one row per state slot and binds it, and the scheduler's block manager hands slots to sequences.
A span that starts at position 0 ignores what its slot held, so slots need no clearing when reused.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..utils.context import get_context

F32 = torch.float32


def small_param(*shape, fill: float = 0.0) -> nn.Parameter:
    """fp32 whatever the model dtype: norm weights, taps, decays and biases enter fp32 arithmetic."""
    return nn.Parameter(torch.full(shape, fill, dtype=F32))


def _spans_and_slots(module_state):
    ctx = get_context()
    spans = ops.StepSpans.of(ctx)
    bound = module_state is not None and module_state.numel() > 0 and ctx.state_slots is not None
    return ctx, spans, bound


class ShortConv(nn.Module):
    """y_t = act(b + sum_j w[:, j] * u_(t - taps + 1 + j)) per channel; ``conv_state`` keeps each sequence's
    last taps - 1 inputs. Channels may be the concatenation of several projections (``segments``), each loaded
    from its own checkpoint tensor."""

    def __init__(self, segments, taps: int, bias: bool = False, act: str | None = None):
        super().__init__()
        self.segments = list(segments)
        self.channels, self.taps, self.act = sum(self.segments), int(taps), act
        self.weight = small_param(self.channels, self.taps)
        self.weight.weight_loader = self._load_segment
        if bias:
            self.bias = small_param(self.channels)
            self.bias.weight_loader = self._load_segment
        else:
            self.register_parameter("bias", None)
        self.conv_state = None

    def _load_segment(self, param, loaded, shard_id: int = 0):
        start = sum(self.segments[:shard_id])
        param.data.narrow(0, start, loaded.shape[0]).copy_(loaded)

    def state_shapes(self):
        return {"conv_state": ((self.taps - 1, self.channels), None)} if self.taps > 1 else {}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ctx, spans, bound = _spans_and_slots(self.conv_state)
        return ops.causal_conv(x, self.weight, self.bias, spans, self.conv_state if bound else None,
                               ctx.state_slots if bound else None, self.act)


class LinearRecurrence(nn.Module):
    """o_t = S_t^T q_t with S_t = a_t S_(t-1) + k_t (b_t v_t)^T per head, S fp32 [kdim, vdim] in ``state``.
    ``decay`` (a list, one constant per head) selects the constant-decay form; ``tied_gate`` the form in which a forget
    gate per key channel also decides what is written, S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T with f = lower +
    (1 - lower) sigmoid(W_f h + gate_bias) and q = silu(W_q h) (``forward(q, f, v)`` takes the raw projections; gate and
    query are made fp32 by ops.gate_prep); otherwise the selective form with learned ``dt_bias``, ``A_log`` and ``D``
    (a_t = exp(-exp(A_log) softplus(dt_t + dt_bias)))."""

    def __init__(self, num_heads: int, groups: int, kdim: int, vdim: int, decay=None, act_silu: bool = False,
                 tied_gate: bool = False):
        super().__init__()
        self.num_heads, self.groups, self.kdim, self.vdim = num_heads, groups, kdim, vdim
        self.act_silu = act_silu
        self.tied_gate = bool(tied_gate)
        if tied_gate:
            assert decay is None and not act_silu, "the tied-gate form has neither a constant decay nor an activation flag"
            self.decay = None
            self.lower, self.gate_bias = small_param(groups * kdim), small_param(groups * kdim)
        elif decay is not None:
            self.register_buffer("decay", torch.tensor([float(d) for d in decay], dtype=F32), persistent=False)
            assert self.decay.numel() == num_heads, "one decay per head"
        else:
            self.decay = None
            self.dt_bias, self.A_log, self.D = small_param(num_heads), small_param(num_heads), small_param(num_heads)
        self.state = None

    def state_shapes(self):
        return {"state": ((self.num_heads, self.kdim, self.vdim), F32)}

    def forward(self, q, k, v, dt=None) -> torch.Tensor:
        """q and k may be fp32 beside 16-bit v (constant-decay form): rotated or normalised in 32-bit upstream."""
        ctx, spans, bound = _spans_and_slots(self.state)
        if self.tied_gate:
            q, k = ops.gate_prep(q, k, self.gate_bias, self.lower)
            kw = dict(tied_gate=True)
        elif self.decay is not None:
            kw = dict(decay=self.decay, act_silu=self.act_silu)
        else:
            kw = dict(dt=dt, dt_bias=self.dt_bias, a_log=self.A_log, d_skip=self.D)
        return ops.linear_recurrence(q, k, v, spans, self.num_heads, self.groups, self.kdim, self.vdim,
                                     self.state if bound else None, ctx.state_slots if bound else None, **kw)


class GatedNorm(nn.Module):
    """RMS norm over ``groups`` equal parts of the row times a plain weight, and a gate act(g): the gate is
    applied before the norm (``gate_first``) or after it. ``norm=False``: the gate alone."""

    def __init__(self, size: int, eps: float, groups: int = 1, gate_first: bool = False, gate_act: str = "sigmoid",
                 norm: bool = True):
        super().__init__()
        self.eps, self.groups, self.gate_first, self.gate_act = eps, groups, gate_first, gate_act
        if norm:
            self.weight = small_param(size, fill=1.0)
        else:
            self.register_parameter("weight", None)

    def forward(self, y: torch.Tensor, gate: torch.Tensor | None, dtype=None) -> torch.Tensor:
        """gate None: the grouped norm alone, written in ``dtype``."""
        return ops.gated_norm(y, gate, self.weight, self.eps, self.groups, self.gate_first, self.gate_act, dtype=dtype)


class VarSizeAttention(nn.Module):
    """Causal softmax attention with ``dim``-wide queries/keys and ``vdim``-wide values over paged caches
    ``k_cache`` [nb, bs, G*dim] / ``v_cache`` [nb, bs, G*vdim] (bound by the runner; K/V rows are written by the
    caller's fused epilogue). 16-bit models with dim == vdim in {64, 128} run on the tcgen05 prefill kernel and
    the paged decode kernel of the dense decoders; everything else (other sizes, fp32) on the generic kernel.
    ``softcap`` c > 0 turns every score s into c tanh(s / c); ``sink`` (a logit) adds exp(sink) to every softmax
    denominator, an entry without key or value; ``forward(..., gate)`` multiplies head h of token t by sigmoid(gate[t, h])."""

    def __init__(self, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float, window: int = 0,
                 softcap: float = 0.0, sink: float | None = None):
        super().__init__()
        self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.scale = num_heads, num_kv_heads, dim, vdim, scale
        self.window = int(window)                       # > 0: position i sees keys j with 0 <= i - j < window
        self.softcap = float(softcap or 0.0)
        if sink is not None:
            self.register_buffer("sink", torch.full((num_heads,), float(sink), dtype=F32), persistent=False)
        else:
            self.sink = None
        self.k_cache = torch.tensor([])
        self.v_cache = torch.tensor([])
        self.layer_id = -1
        self.force_generic = False

    def cache_rows(self) -> tuple[int, int]:
        return self.num_kv_heads * self.dim, self.num_kv_heads * self.vdim

    def _fast(self, q) -> bool:
        rep, G = self.num_heads // self.num_kv_heads, self.num_kv_heads
        return (not self.force_generic and not self.window
                and q.dtype in (torch.bfloat16, torch.float16) and self.dim == self.vdim
                and self.dim in (64, 128) and rep <= 8 and (G in (1, 2, 4) or G % 8 == 0))

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor | None = None) -> torch.Tensor:
        """q [T, H, dim]; k [T, G, dim], v [T, G, vdim]: this step's rows (used when no cache is bound); gate [T, H]
        logits of an output gate per head, or None."""
        ctx = get_context()
        paged = self.k_cache.numel() > 0 and ctx.block_tables is not None
        if self._fast(q) and (paged or ctx.is_prefill):
            out = None
            soft = dict(softcap=self.softcap, sink=self.sink)
            # a score cap or a sink: the tcgen05 kernel only, whose TMA maps want 16-byte row strides and blocks that
            # tile its 128-key steps
            tma_ok = not (self.softcap or self.sink is not None) or (
                q.stride(0) % 8 == 0 and (paged and (ctx.block_size % 128 == 0 or 128 % ctx.block_size == 0) or
                                          not paged and k.stride(0) % 8 == 0 and v.stride(0) % 8 == 0))
            if not ctx.is_prefill:
                out = ops.paged_decode_attn(q, self.k_cache, self.v_cache, ctx.block_tables, ctx.context_lens,
                                            self.scale, self.num_kv_heads, num_ctas=ctx.decode_attn_ctas, **soft)
            elif paged and ctx.block_size % 16 == 0 and tma_ok:
                out = ops.prefill_varlen_attn(q, self.k_cache, self.v_cache, ctx.cu_seqlens_q, ctx.cu_seqlens_k,
                                              ctx.max_seqlen_q, ctx.max_seqlen_k, self.scale, self.num_kv_heads,
                                              block_tables=ctx.block_tables, **soft)
            elif not paged and tma_ok:
                out = ops.prefill_varlen_attn(q, k, v, ctx.cu_seqlens_q, ctx.cu_seqlens_k, ctx.max_seqlen_q,
                                              ctx.max_seqlen_k, self.scale, self.num_kv_heads, **soft)
            if out is not None:
                out = out.view(q.shape[0], self.num_heads * self.vdim)
                return out if gate is None else ops.head_gate_(out, gate, self.num_heads)
        spans = ops.StepSpans.of(ctx)
        extras = dict(window=self.window, softcap=self.softcap, sink=self.sink, gate=gate)
        if paged:
            return ops.attn_generic(q, self.k_cache, self.v_cache, spans, self.scale, self.num_kv_heads, self.vdim,
                                    block_tables=ctx.block_tables, **extras)
        return ops.attn_generic(q, k, v, spans, self.scale, self.num_kv_heads, self.vdim, **extras)


class MixedHeadAttention(nn.Module):
    """Causal softmax attention whose heads are mixed BEFORE the softmax (``talk`` [H, H], s'_h = sum_g talk[h, g] s_g),
    with an optional linear distance bias per head (s_h(i, j) = scale q.k - slope_h (i - j); ``slope_base`` b gives
    slope_h = 2^(-b (h + 1) / H)), an optional learned ``sink`` per head that joins the softmax denominator without a
    key or value, and an optional sliding window. Keys/values live in paged caches ``k_cache`` [nb, bs, G*dim] /
    ``v_cache`` [nb, bs, G*vdim] written by the caller's fused epilogue -- or, with ``kv_source`` (another
    MixedHeadAttention of the same head counts), in THAT layer's caches: this layer then projects queries only and
    reads the other layer's keys (as cached, after their norm) and values through the same block tables."""

    def __init__(self, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float, window: int = 0,
                 slope_base: float | None = None, talk: bool = True, sink: bool = True, kv_source=None):
        super().__init__()
        self.num_heads, self.num_kv_heads, self.dim, self.vdim = num_heads, num_kv_heads, dim, vdim
        self.scale, self.window = float(scale), int(window)
        if slope_base is not None:
            slopes = [2.0 ** (-float(slope_base) * (h + 1) / num_heads) for h in range(num_heads)]
            self.register_buffer("slopes", torch.tensor(slopes, dtype=F32), persistent=False)
        else:
            self.slopes = None
        if talk:
            self.talk = nn.Parameter(torch.eye(num_heads, dtype=F32))
        else:
            self.register_parameter("talk", None)
        if sink:
            self.sink = small_param(num_heads)
        else:
            self.register_parameter("sink", None)
        if kv_source is not None and (kv_source.num_kv_heads, kv_source.dim, kv_source.vdim) != (num_kv_heads, dim, vdim):
            raise ValueError("a layer that borrows keys and values needs the lender's kv head count and sizes")
        object.__setattr__(self, "kv_source", kv_source)          # not a submodule: the lender owns its parameters
        self.k_cache = torch.tensor([])
        self.v_cache = torch.tensor([])
        self.layer_id = -1
        self.force_generic = False                  # True: always the kernel of csrc/mixed_attn.cu
        self.step_kv = None                         # this step's (k, v) rows, kept for a borrower when no cache is bound

    def cache_rows(self) -> tuple[int, int]:
        if self.kv_source is not None:
            return 0, 0                             # the runner binds the lender's caches
        return self.num_kv_heads * self.dim, self.num_kv_heads * self.vdim

    def forward(self, q: torch.Tensor, k: torch.Tensor | None = None, v: torch.Tensor | None = None) -> torch.Tensor:
        """q [T, H, dim]; k [T, G, dim], v [T, G, vdim]: this step's rows (None for a borrower)."""
        ctx = get_context()
        if self.kv_source is None:
            self.step_kv = (k, v)
        else:
            k, v = self.kv_source.step_kv
        spans = ops.StepSpans.of(ctx)
        paged = self.k_cache.numel() > 0 and ctx.block_tables is not None
        sixteen = q.dtype != torch.float32 and not self.force_generic and self.num_heads <= 64
        if (sixteen and ctx.is_prefill and ctx.host_spans is not None and ctx.max_seqlen_q >= self.PRODUCT_MIN_TOKENS):
            out = self._prefill_by_products(q, k, v, ctx, paged)
            if out is not None:
                return out
        elif (sixteen and not ctx.is_prefill and paged and self.window > 0 and
              min(self.window, ctx.block_tables.shape[1] * ctx.block_size) <= self.DECODE_WINDOW_MAX and
              self._fits(min(self.window, ctx.block_tables.shape[1] * ctx.block_size))):
            return self._decode_window_by_products(q, ctx)
        if paged:
            return ops.mixed_attn(q, self.k_cache, self.v_cache, spans, self.scale, self.num_kv_heads, self.vdim,
                                  block_tables=ctx.block_tables, **self._extras())
        return ops.mixed_attn(q, k, v, spans, self.scale, self.num_kv_heads, self.vdim, **self._extras())

    def _extras(self):
        return dict(window=self.window, slopes=self.slopes, talk=self.talk, sink=self.sink)

    def _fits(self, nk: int) -> bool:
        """The softmax kernel keeps a token's heads x visible keys block (and the mixing matrix) in shared memory."""
        H = self.num_heads
        ns = min(nk, self.window) if self.window else nk
        return (H * ns + H * max(4, 1 << (H - 1).bit_length())) * 4 <= ops.MIXED_SOFTMAX_SMEM

    DECODE_WINDOW_MAX = 4096      # decode steps gather a window of at most this many rows per sequence
    PRODUCT_BYTES = 512 << 20     # fp32 scores held at a time
    PRODUCT_MIN_TOKENS = 64       # longest portion of the step from which prompts run on library products
    PRODUCT_CHUNK = 256           # query tokens per product

    def _decode_window_by_products(self, q, ctx):
        """Decode steps inside a sliding window, 16-bit models: the last `window` cached key and value rows of every
        sequence are gathered into dense blocks (fixed shapes: capturable in a CUDA graph); one batched library product
        per kv head gives the raw scores of its query heads (fp32 out); the mixed softmax kernel applies scale, distance
        bias, head mixing, mask (rows before a sequence's start, padded graph rows) and sink; one batched product with
        the value rows. Without a window the kernel of csrc/mixed_attn.cu reads the cache through the block table."""
        B, H, d = q.shape
        G, dv, bs = self.num_kv_heads, self.vdim, ctx.block_size
        rep = H // G
        W = min(self.window, ctx.block_tables.shape[1] * bs)                 # no sequence holds more rows than its table
        slots = ctx.scratch.get(("window rows", W))                          # the same for every layer of the step
        if slots is None:
            pos = ctx.context_lens.long() - 1                                # -1 on padded rows
            j = (pos[:, None] - (W - 1) + torch.arange(W, device=q.device)).clamp(min=0)
            blocks = ctx.block_tables.gather(1, j // bs).clamp(min=0).long()
            slots = ctx.scratch[("window rows", W)] = (blocks * bs + j % bs).view(-1)
        # ONE gather per cache, straight into [B, G, W, size]: the batched products want a kv head's rows together
        krows = ops.gather_rows_by_head(self.k_cache.view(-1, G, d), slots, B, W).view(B * G, W, d)
        vrows = ops.gather_rows_by_head(self.v_cache.view(-1, G, dv), slots, B, W).view(B * G, W, dv)
        scores = torch.bmm(q.reshape(B * G, rep, d), krows.transpose(1, 2), out_dtype=torch.float32)   # [B * G, rep, W]
        p = ops.mixed_softmax(scores.view(B, G, 1, rep, W), self.scale, self.window, q.dtype, self.slopes, self.talk,
                              self.sink, ctx_lens=ctx.context_lens)
        return torch.bmm(p.view(B * G, rep, W), vrows).reshape(B, H * dv)

    def _prefill_by_products(self, q, k, v, ctx, paged):
        """Prompt portions of 16-bit models on the tensor cores, all chunks of the step at once: gather the chunks' query
        rows and key/value ranges; the raw scores of every kv head's query heads against its keys as one batched library
        product with fp32 output; the mixed softmax kernel (scale, distance bias, head mixing, mask, sink; fp32 in,
        16-bit probabilities out); one batched product with the values. Portions shorter than PRODUCT_MIN_TOKENS beside
        long ones run on the kernel of csrc/mixed_attn.cu; so does the whole step (None is returned) when a token's
        heads x keys block would not fit the softmax kernel's shared memory."""
        T, H, d = q.shape
        G, dv, CH = self.num_kv_heads, self.vdim, self.PRODUCT_CHUNK
        rep = H // G
        key = ("prompt plan", self.window, CH, self.PRODUCT_MIN_TOKENS, paged)
        plan = ctx.scratch.get(key)
        if plan is None:
            plan = ctx.scratch[key] = prompt_chunk_plan(ctx, paged, q.device, CH, self.window, self.PRODUCT_MIN_TOKENS)
        NC = plan["chunks"]
        if NC and not self._fits(plan["NK"]):
            return None
        out = torch.empty(T, H * dv, dtype=q.dtype, device=q.device)
        for s, q0, ql, kl in plan["short"]:
            sub = ops.StepSpans(torch.tensor([0, ql], dtype=torch.int32, device=q.device),
                                torch.tensor([0, kl], dtype=torch.int32, device=q.device), None, ql)
            if paged:
                out[q0:q0 + ql] = ops.mixed_attn(q[q0:q0 + ql], self.k_cache, self.v_cache, sub, self.scale, G, dv,
                                                 block_tables=ctx.block_tables[s:s + 1], **self._extras())
            else:
                out[q0:q0 + ql] = ops.mixed_attn(q[q0:q0 + ql], k[q0:q0 + ql], v[q0:q0 + ql], sub, self.scale, G, dv,
                                                 **self._extras())
        if NC == 0:
            return out
        NK = plan["NK"]
        flat_k = self.k_cache.view(-1, G, d) if paged else k
        flat_v = self.v_cache.view(-1, G, dv) if paged else v
        per = max(1, min(256, self.PRODUCT_BYTES // (CH * H * NK * 4)))      # chunks per launch: bounded score memory
        for g0 in range(0, NC, per):
            g1 = min(NC, g0 + per)
            n = g1 - g0
            kslots = plan["kslots"][g0 * NK:g1 * NK]     # ONE gather per tensor, straight into [chunks, G, NK, size]
            kk = ops.gather_rows_by_head(flat_k, kslots, n, NK).view(n * G, NK, d)
            vv = ops.gather_rows_by_head(flat_v, kslots, n, NK).view(n * G, NK, dv)
            run = plan["run"]
            qs = q[run + g0 * CH:run + g1 * CH] if run is not None else q[plan["qrows"][g0 * CH:g1 * CH]]
            qs = qs.reshape(n, CH, G, rep, d).permute(0, 2, 1, 3, 4).reshape(n * G, CH * rep, d)
            scores = torch.bmm(qs, kk.transpose(1, 2), out_dtype=torch.float32)                 # [n * G, CH * rep, NK]
            p = ops.mixed_softmax(scores.view(n, G, CH, rep, NK), self.scale, self.window, q.dtype, self.slopes,
                                  self.talk, self.sink, chunks=(plan["first"][g0:g1], plan["lo"][g0:g1]))
            o = torch.bmm(p.view(n * G, CH * rep, NK), vv)                                      # [n * G, CH * rep, dv]
            o = o.view(n, G, CH, rep, dv).permute(0, 2, 1, 3, 4).reshape(n * CH, H * dv)
            if run is not None:
                out[run + g0 * CH:run + g1 * CH] = o
            elif plan["full"]:
                out[plan["qrows"][g0 * CH:g1 * CH]] = o
            else:
                sel = (plan["src"] >= g0 * CH) & (plan["src"] < g1 * CH)
                out[plan["dst"][sel]] = o[plan["src"][sel] - g0 * CH]
        return out


class DeltaRule(nn.Module):
    """Gated delta rule with one decay per head and key channel, state S fp32 [kdim, vdim] per head in ``state``:
    S <- diag(g) S; w = beta (v - S^T k); S <- S + k w^T; o = S^T q, with g = exp(-exp(A_log_h) softplus(a + dt_bias)),
    beta = sigmoid(b), q and k divided by sqrt(sum x^2 + unit_eps) per head and q times ``q_scale``. Everything but the
    projected activations is fp32."""

    def __init__(self, num_heads: int, groups: int, kdim: int, vdim: int, unit_eps: float = 1e-6,
                 q_scale: float | None = None):
        super().__init__()
        self.num_heads, self.groups, self.kdim, self.vdim = num_heads, groups, kdim, vdim
        self.unit_eps = unit_eps
        self.q_scale = kdim ** -0.5 if q_scale is None else q_scale
        self.A_log, self.dt_bias = small_param(num_heads), small_param(num_heads * kdim)
        self.state = None

    def state_shapes(self):
        return {"state": ((self.num_heads, self.kdim, self.vdim), F32)}

    def forward(self, qk, v, a, b) -> torch.Tensor:
        """qk [T, 2*groups*kdim] (q heads, then k heads), v [T, H*vdim], a [T, H*kdim], b [T, H] -> fp32 [T, H*vdim]."""
        ctx, spans, bound = _spans_and_slots(self.state)
        qk32, g, beta = ops.delta_prep(qk, a, b, self.dt_bias, self.A_log, self.num_heads, self.groups, self.kdim,
                                       self.unit_eps, self.q_scale)
        n = self.groups * self.kdim
        return ops.delta_rule(qk32[:, :n], qk32[:, n:], v, g, beta, spans, self.num_heads, self.groups, self.kdim,
                              self.vdim, self.state if bound else None, ctx.state_slots if bound else None)


class Rotary:
    """Rotary positions on the first ``dims`` columns of a head: angle pos * base^(-2i/dims), pairs (2i, 2i+1)
    (``interleaved``) or (i, i + dims/2). Constants only; the kernel computes the angles in fp64."""

    def __init__(self, dims: int, base: float, interleaved: bool):
        self.dims, self.base, self.interleaved = int(dims), float(base), bool(interleaved)

    def __call__(self, x, positions, out=None, out_f32=False, split=0, scale_lo=1.0, scale_hi=1.0):
        """x [T, heads, width] view -> rotated (and scaled) copy, see ops.rotary_heads."""
        return ops.rotary_heads(x, positions, x.shape[1], x.shape[2], self.dims, self.base, self.interleaved, out=out,
                                out_f32=out_f32, split=split, scale_lo=scale_lo, scale_hi=scale_hi)


class BandScaledRotary:
    """Rotary positions whose frequencies are stretched band by band: f_i = base^(-2i/dims), i < dims/2; with
    n(t) = dims ln(original / (2 pi t)) / (2 ln base) (the pair index that makes t turns over the original length),
    lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    the frequency becomes f_i / factor * ramp_i + f_i (1 - ramp_i): pairs that turn fast keep their frequency, slow
    ones are divided by ``factor``, and cos and sin are multiplied by 0.1 ln(factor) + 1. Without ``scaling`` the
    frequencies are the plain ones. The step's (cos, sin) table is computed once per pass (fp64 angles) and shared by
    all layers with the same constants; the rotation itself runs fused with the layer's cache write
    (ops.rope_mix_cache)."""

    MAGNITUDE_SLOPE = 0.1

    def __init__(self, dims: int, base: float, interleaved: bool = True, scaling: dict | None = None):
        import math
        self.dims, self.base, self.interleaved = int(dims), float(base), bool(interleaved)
        half = self.dims // 2
        f = [self.base ** (-2.0 * i / self.dims) for i in range(half)]
        self.magnitude = 1.0
        if scaling:
            factor, original = float(scaling["factor"]), float(scaling["original"])
            turns_at = lambda t: self.dims * math.log(original / (2 * math.pi * t)) / (2 * math.log(self.base))
            lo = max(math.floor(turns_at(float(scaling["fast"]))), 0)
            hi = min(math.ceil(turns_at(float(scaling["slow"]))), self.dims - 1)
            ramp = [min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001))) for i in range(half)]
            f = [fi / factor * r + fi * (1 - r) for fi, r in zip(f, ramp)]
            self.magnitude = self.MAGNITUDE_SLOPE * math.log(factor) + 1.0
        self.freq = torch.tensor(f, dtype=torch.float64)
        self.key = ("rotary table", self.dims, self.interleaved, self.magnitude, tuple(f))

    def table(self, positions: torch.Tensor) -> torch.Tensor | None:
        """fp32 [T, dims/2, 2] for this pass's positions, from the context's per-pass scratch."""
        if self.dims == 0:
            return None
        ctx = get_context()
        t = ctx.scratch.get(self.key)
        if t is None or t.shape[0] != positions.numel():
            if self.freq.device != positions.device:
                self.freq = self.freq.to(positions.device)
            t = ctx.scratch[self.key] = ops.rotary_table(positions, self.freq, self.magnitude)
        return t


def prompt_chunk_plan(ctx, paged, device, chunk: int, window: int, min_tokens: int):
    """Index tensors of the step's prompt chunks, built once per pass and shared by the layers: every span of at
    least `min_tokens` tokens is cut into chunks of `chunk` query tokens; all chunks see a key range of
    the same length NK (a multiple of 128 that covers the widest visible range; what lies before a sequence's
    start or outside a row's window is hidden by the softmax kernel)."""
    import numpy as np
    CH, W, bs = chunk, window, ctx.block_size
    chunks, short = [], []                      # (sequence, first token row, tokens, first position)
    for s, (q0, ql, kl) in enumerate(ctx.host_spans):
        if ql < min_tokens:
            short.append((s, q0, ql, kl))
            continue
        for c0 in range(0, ql, CH):
            chunks.append((s, q0 + c0, min(CH, ql - c0), kl - ql + c0))
    plan = {"short": short, "chunks": len(chunks)}
    if not chunks:
        return plan
    seq = np.array([c[0] for c in chunks])
    row0 = np.array([c[1] for c in chunks])
    n = np.array([c[2] for c in chunks])
    pos0 = np.array([c[3] for c in chunks])
    hi = pos0 + n                                # keys of a chunk end at its last token
    vis_lo = np.maximum(0, pos0 - W + 1) if W else np.zeros_like(pos0)
    NK = int(-(-int((hi - vis_lo).max()) // 128) * 128)
    lo = hi - NK                                 # may be negative: those columns repeat row 0 and are hidden
    dev = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to(dt).to(device, non_blocking=True)
    tok = np.arange(CH)[None, :]
    qrows = row0[:, None] + np.minimum(tok, n[:, None] - 1)           # rows past a chunk's end repeat its last token
    kpos = np.maximum(lo[:, None] + np.arange(NK)[None, :], 0)
    kpos_d = dev(kpos, torch.int64)
    if paged:
        tables = ctx.block_tables[dev(seq, torch.int64)]               # [chunks, blocks]
        kslots = tables.gather(1, kpos_d // bs).long() * bs + kpos_d % bs
    else:                                        # no cache bound: a span's keys are this step's rows
        span_row0 = np.array([ctx.host_spans[c[0]][0] for c in chunks])
        kslots = kpos_d + dev(span_row0, torch.int64)[:, None]
    valid = tok < n[:, None]                     # [chunks, CH]
    flatq = qrows.reshape(-1)
    # chunks that are all full and follow each other in the packed batch need no gather of query rows
    plan["run"] = int(flatq[0]) if bool(valid.all()) and bool((np.diff(flatq) == 1).all()) else None
    plan.update(NK=NK, qrows=dev(qrows.reshape(-1), torch.int64), kslots=kslots.reshape(-1),
                first=dev(pos0, torch.int32), lo=dev(lo, torch.int32),
                src=dev(np.nonzero(valid.reshape(-1))[0], torch.int64), dst=dev(qrows[valid], torch.int64),
                full=bool(valid.all()))
    return plan


class LatentAttention(nn.Module):
    """Softmax attention whose keys and values are up-projections of ONE cached latent row per token:
    score_h(i, j) = scale (q_h^plain . W_uk,h c_j + q_h^rot . r_j), value_h(j) = W_uv,h c_j, with c the normed latent
    [rank] and r the rotated key part [rot] shared by all heads. Only [c | r] is cached (``k_cache`` [nb, bs,
    rank + rot]; there is no value cache). The up-projections are absorbed: the query is moved into latent space
    (q_h^plain W_uk,h, one batched product), attention runs as ONE kv head of key size rank + rot whose values are
    the first ``rank`` columns of the same rows, and W_uv,h is applied to the attended latent."""

    def __init__(self, num_heads: int, dim: int, rot: int, vdim: int, rank: int, scale: float, window: int = 0):
        super().__init__()
        self.num_heads, self.dim, self.rot, self.vdim, self.rank = num_heads, dim, rot, vdim, rank
        self.scale, self.window = float(scale), int(window)
        self.w_uk = nn.Parameter(torch.empty(num_heads, dim, rank))       # [h, d, r]: rows of W_uk per head
        self.w_uv = nn.Parameter(torch.empty(num_heads, vdim, rank))
        self.w_uk.weight_loader = self._load_heads
        self.w_uv.weight_loader = self._load_heads
        self.k_cache = torch.tensor([])
        self.v_cache = torch.tensor([])
        self.layer_id = -1
        self.force_generic = False

    @staticmethod
    def _load_heads(param, loaded):
        param.data.copy_(loaded.view(param.shape))

    def cache_rows(self) -> tuple[int, int]:
        return self.rank + self.rot, 0

    def forward(self, q_plain: torch.Tensor, q_rot_writer, kc: torch.Tensor) -> torch.Tensor:
        """q_plain [T, H, dim] (a view); q_rot_writer(out_view [T, H, rot]) fills the rotated query part; kc
        [T, rank + rot] this step's cache rows (used when no cache is bound). Returns [T, H * vdim]."""
        ctx = get_context()
        T, H, R = q_plain.shape[0], self.num_heads, self.rank
        qx = torch.empty(T, H, R + self.rot, dtype=q_plain.dtype, device=q_plain.device)
        qx[:, :, :R].copy_(torch.bmm(q_plain.transpose(0, 1), self.w_uk).transpose(0, 1))
        q_rot_writer(qx[:, :, R:])
        spans = ops.StepSpans.of(ctx)
        paged = self.k_cache.numel() > 0 and ctx.block_tables is not None
        if (ctx.is_prefill and ctx.host_spans is not None and qx.dtype != torch.float32 and not self.force_generic
                and ctx.max_seqlen_q >= self.PRODUCT_MIN_TOKENS):
            lat = self._prefill_by_products(qx, kc, ctx, paged)
        elif (not ctx.is_prefill and paged and self.window > 0 and not self.force_generic and
              min(self.window, ctx.block_tables.shape[1] * ctx.block_size) <= self.DECODE_WINDOW_MAX):
            lat = self._decode_window_by_products(qx, ctx)
        elif paged:
            lat = ops.attn_generic(qx, self.k_cache, None, spans, self.scale, 1, R, block_tables=ctx.block_tables,
                                   window=self.window)
        else:
            lat = ops.attn_generic(qx, kc.unsqueeze(1), None, spans, self.scale, 1, R, window=self.window)
        out = torch.bmm(lat.view(T, H, R).transpose(0, 1), self.w_uv.transpose(1, 2))      # [H, T, vdim]
        return out.transpose(0, 1).reshape(T, H * self.vdim)

    DECODE_WINDOW_MAX = 4096      # decode steps gather a window of at most this many rows per sequence

    def _decode_window_by_products(self, qx, ctx):
        """Decode steps inside a sliding window: every sequence sees at most `window` keys, so the step gathers the
        last `window` cached rows of every sequence into one dense block (fixed shapes: capturable in a CUDA graph),
        scores all heads against it with one batched library product (fp32 out), runs the masked softmax kernel
        (rows before a sequence's start and padded graph rows are hidden) and multiplies by the latent part of the same
        rows. Without a window the generic kernel reads the cache through the block table instead."""
        B, H, D = qx.shape
        R, bs = self.rank, ctx.block_size
        W = min(self.window, ctx.block_tables.shape[1] * bs)                 # no sequence holds more rows than its table
        slots = ctx.scratch.get(("window rows", W))                          # the same for every layer of the step
        if slots is None:
            pos = ctx.context_lens.long() - 1                                # -1 on padded rows
            j = (pos[:, None] - (W - 1) + torch.arange(W, device=qx.device)).clamp(min=0)
            blocks = ctx.block_tables.gather(1, j // bs).clamp(min=0).long()
            slots = ctx.scratch[("window rows", W)] = (blocks * bs + j % bs).view(-1)
        rows = self.k_cache.view(-1, D)[slots].view(B, W, D)
        if qx.dtype == torch.float32:
            scores = torch.bmm(qx, rows.transpose(1, 2))
        else:
            scores = torch.bmm(qx, rows.transpose(1, 2), out_dtype=torch.float32)
        p = ops.masked_softmax(scores.view(B * H, W), H, 0, 0, self.scale, self.window, qx.dtype,
                               ctx_lens=ctx.context_lens)
        return torch.bmm(p.view(B, H, W), rows[:, :, :R]).reshape(B, H * R)

    OWN_SCORE_PRODUCT = True      # scores on the tcgen05 GEMM of csrc/moe_umma.cu (False: torch.bmm with fp32 output)
    PRODUCT_BYTES = 512 << 20     # fp32 scores held at a time
    PRODUCT_MIN_TOKENS = 64       # longest portion of the step from which prompts run on library products
    PRODUCT_CHUNK = 512           # query tokens per product

    def _prompt_plan(self, ctx, paged, device):
        return prompt_chunk_plan(ctx, paged, device, self.PRODUCT_CHUNK, self.window, self.PRODUCT_MIN_TOKENS)

    def _prefill_by_products(self, qx, kc, ctx, paged):
        """Prompt portions of 16-bit models on the tensor cores, all chunks of the step at once: gather the chunks'
        query rows and key ranges; scores of ALL heads of a chunk against its key range as one group of a grouped
        product with fp32 output (the heads share the latent rows; the library's tcgen05 GEMM of csrc/moe_umma.cu, or
        torch.bmm with fp32 output); the masked softmax kernel (fp32 in, 16-bit probabilities out); one batched product
        with the latent part of the same rows. Portions shorter than PRODUCT_MIN_TOKENS beside long ones, and fp32
        models, run on attn_generic."""
        T, H, R = qx.shape[0], self.num_heads, self.rank
        D, CH = R + self.rot, self.PRODUCT_CHUNK
        key = ("prompt plan", self.window, CH, self.PRODUCT_MIN_TOKENS, paged)
        plan = ctx.scratch.get(key)
        if plan is None:
            plan = ctx.scratch[key] = self._prompt_plan(ctx, paged, qx.device)
        lat = torch.empty(T, H * R, dtype=qx.dtype, device=qx.device)
        for s, q0, ql, kl in plan["short"]:
            sub = ops.StepSpans(torch.tensor([0, ql], dtype=torch.int32, device=qx.device),
                                torch.tensor([0, kl], dtype=torch.int32, device=qx.device), None, ql)
            if paged:
                lat[q0:q0 + ql] = ops.attn_generic(qx[q0:q0 + ql], self.k_cache, None, sub, self.scale, 1, R,
                                                   block_tables=ctx.block_tables[s:s + 1], window=self.window)
            else:
                lat[q0:q0 + ql] = ops.attn_generic(qx[q0:q0 + ql], kc[q0:q0 + ql].unsqueeze(1), None, sub,
                                                   self.scale, 1, R, window=self.window)
        NC = plan["chunks"]
        if NC == 0:
            return lat
        NK = plan["NK"]
        # the tcgen05 GEMM multiplies 64 columns at a time; rows of other widths would have to be copied into padded
        # buffers (measured slower than the library's product at 288 columns), except where they are tiny
        own = self.OWN_SCORE_PRODUCT and (D % 64 == 0 or D < 64)
        Dp = -(-D // 64) * 64 if own else D
        flat = self.k_cache.view(-1, D) if paged else kc
        per = max(1, min(256, self.PRODUCT_BYTES // (CH * H * NK * 4)))      # chunks per launch: bounded score memory
        for g0 in range(0, NC, per):
            g1 = min(NC, g0 + per)
            G = g1 - g0
            rows = flat[plan["kslots"][g0 * NK:g1 * NK]]                           # [G * NK, D]
            run = plan["run"]
            q = (qx[run + g0 * CH:run + g1 * CH] if run is not None else qx[plan["qrows"][g0 * CH:g1 * CH]]).reshape(
                G * CH * H, D)
            if own:
                if Dp != D:
                    rows_p, q = torch.nn.functional.pad(rows, (0, Dp - D)), torch.nn.functional.pad(q, (0, Dp - D))
                else:
                    rows_p = rows
                offsets = torch.arange(0, (G + 1) * CH * H, CH * H, dtype=torch.int32, device=qx.device)
                scores = ops.scores_umma(q, rows_p.view(G, NK, Dp), offsets)       # [G * CH * H, NK] fp32
            else:
                scores = torch.bmm(q.view(G, CH * H, D), rows.view(G, NK, D).transpose(1, 2),
                                   out_dtype=torch.float32).view(G * CH * H, NK)
            p = ops.masked_softmax(scores, H, 0, 0, self.scale, self.window, qx.dtype,
                                   chunks=(plan["first"][g0:g1], plan["lo"][g0:g1], CH * H))
            out = torch.bmm(p.view(G, CH * H, NK), rows.view(G, NK, D)[:, :, :R].contiguous()).view(G * CH, H * R)
            if run is not None:
                lat[run + g0 * CH:run + g1 * CH] = out
            elif plan["full"]:
                lat[plan["qrows"][g0 * CH:g1 * CH]] = out
            else:
                sel = (plan["src"] >= g0 * CH) & (plan["src"] < g1 * CH)
                lat[plan["dst"][sel]] = out[plan["src"][sel] - g0 * CH]
        return lat


class StreamResidual(nn.Module):
    """Mixing weights of one sublayer of a residual kept in ``streams`` copies: the sublayer reads
    u = sum_s read[s] x_s and every stream becomes x_t <- sum_s mix[s, t] x_s + write[t] y. The arithmetic runs in
    ops.stream_mix_norm_, fused with the norm of the next sublayer."""

    def __init__(self, streams: int):
        super().__init__()
        self.read, self.write = small_param(streams, fill=1.0), small_param(streams, fill=1.0)
        self.mix = nn.Parameter(torch.eye(streams, dtype=F32))
