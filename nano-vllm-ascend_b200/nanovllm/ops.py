"""Tensor-level wrappers over the C ABI: torch owns memory and streams, CUDA does the work.

Each function validates what the C side cannot know (device, dtype, contiguity of the inner
dimensions), then passes raw pointers + the current stream. All of them enqueue only; they
are safe inside CUDA-graph capture.
"""
from __future__ import annotations

import os

import torch

from . import _C

_DT = {torch.bfloat16: _C.BF16, torch.float16: _C.F16}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"b200attn kernels take bf16/fp16 tensors, got {t.dtype}") from None


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "b200attn: the hot path runs on CUDA only (got a CPU tensor); there is no "
                "CPU fallback -- use oracle/ for CPU reference results")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def _cache_dims(cache: torch.Tensor, row_elems: int) -> tuple[int, int]:
    """(num_blocks, block_size) of a cache given as [nb, bs, Hkv*D] or [nb, bs, Hkv, D]."""
    if cache.dim() not in (3, 4) or not cache.is_contiguous():
        raise ValueError("KV cache must be a contiguous [nb, bs, Hkv*D] (or [nb, bs, Hkv, D]) tensor")
    if cache[0, 0].numel() != row_elems:
        raise ValueError(f"KV cache row has {cache[0, 0].numel()} elements, expected {row_elems}")
    return cache.shape[0], cache.shape[1]


def launch_count() -> int:
    return _C.load().b200_launch_count()


def reset_launch_count() -> None:
    _C.load().b200_reset_launch_count()


def reshape_and_cache(key, value, k_cache, v_cache, slot_mapping):
    """K1/K2. key/value [T, Hkv, D] (token-strided views allowed), slot_mapping [T] flat or
    [T, 2] (block, offset); int32."""
    _need_cuda(key, value, k_cache, v_cache, slot_mapping)
    T, Hkv, D = key.shape
    if value.shape != key.shape:
        raise ValueError("key/value shape mismatch")
    if key.stride(2) != 1 or key.stride(1) != D or value.stride(2) != 1 or value.stride(1) != D:
        raise ValueError("key/value must be contiguous in (heads, head_dim)")
    if slot_mapping.dtype != torch.int32 or not slot_mapping.is_contiguous():
        raise TypeError("slot_mapping must be a contiguous int32 tensor")
    nb, bs = _cache_dims(k_cache, Hkv * D)
    lib = _C.load()
    two_d = slot_mapping.dim() == 2
    if slot_mapping.shape[0] != T or (two_d and slot_mapping.shape[1] != 2):
        raise ValueError(f"slot_mapping shape {tuple(slot_mapping.shape)} does not match {T} tokens")
    fn = lib.b200_reshape_and_cache_2d if two_d else lib.b200_reshape_and_cache
    _C.check(fn(key.data_ptr(), value.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                slot_mapping.data_ptr(), T, Hkv, D, key.stride(0) if T > 1 else Hkv * D,
                value.stride(0) if T > 1 else Hkv * D, nb, bs, _dt(key), _stream()),
             "b200_reshape_and_cache")


def _is_fp8_cache(cache: torch.Tensor) -> bool:
    return cache.dtype in (torch.uint8, torch.float8_e4m3fn)


def reshape_and_cache_fp8(key, value, k_cache, v_cache, slot_mapping, k_scale=1.0, v_scale=1.0):
    """K1/K2 into an e4m3 cache (uint8 / float8_e4m3fn tensors [nb, bs, Hkv*D]):
    cache <- e4m3(x * (1/scale)), saturating. key/value [T, Hkv, D] bf16/fp16."""
    _need_cuda(key, value, k_cache, v_cache, slot_mapping)
    T, Hkv, D = key.shape
    if value.shape != key.shape:
        raise ValueError("key/value shape mismatch")
    if key.stride(2) != 1 or key.stride(1) != D or value.stride(2) != 1 or value.stride(1) != D:
        raise ValueError("key/value must be contiguous in (heads, head_dim)")
    if slot_mapping.dtype != torch.int32 or not slot_mapping.is_contiguous():
        raise TypeError("slot_mapping must be a contiguous int32 tensor")
    if not (_is_fp8_cache(k_cache) and _is_fp8_cache(v_cache)):
        raise TypeError("fp8 KV caches must be uint8 or float8_e4m3fn tensors")
    nb, bs = _cache_dims(k_cache, Hkv * D)
    two_d = slot_mapping.dim() == 2
    if slot_mapping.shape[0] != T or (two_d and slot_mapping.shape[1] != 2):
        raise ValueError(f"slot_mapping shape {tuple(slot_mapping.shape)} does not match {T} tokens")
    _C.check(_C.load().b200_reshape_and_cache_fp8(
        key.data_ptr(), value.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
        slot_mapping.data_ptr(), 1 if two_d else 0, T, Hkv, D,
        key.stride(0) if T > 1 else Hkv * D, value.stride(0) if T > 1 else Hkv * D, nb, bs,
        float(k_scale), float(v_scale), _dt(key), _stream()), "b200_reshape_and_cache_fp8")


_decode_ws: dict = {}


def decode_workspace(batch, num_heads, num_kv_heads, head_dim, device) -> torch.Tensor:
    need = _C.load().b200_paged_decode_attn_workspace_size(batch, num_heads, num_kv_heads, head_dim)
    if need == 0:
        raise _C.B200Error("b200_paged_decode_attn: unsupported head configuration "
                           f"(H={num_heads}, Hkv={num_kv_heads}, D={head_dim})")
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _decode_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=device)   # arrival counters start at 0
        _decode_ws[key] = ws
    return ws


def paged_decode_attn(q, k_cache, v_cache, block_tables, context_lens, scale, num_kv_heads,
                      out=None, workspace=None, num_ctas=0, softcap=0.0, sink=None):
    """K6. q [B, H, D] (token-strided view allowed) -> out [B, H*D]. softcap > 0: scores become softcap *
    tanh(score / softcap); sink fp32 [H]: exp(sink[h]) joins the softmax denominator (no key, no value)."""
    _need_cuda(q, k_cache, v_cache, block_tables, context_lens, sink)
    _f32(sink)
    B, H, D = q.shape
    if sink is not None and sink.numel() != H:
        raise ValueError("sink [H]")
    if q.stride(2) != 1 or q.stride(1) != D:
        raise ValueError("q must be contiguous in (heads, head_dim)")
    if block_tables.dtype != torch.int32 or context_lens.dtype != torch.int32:
        raise TypeError("block_tables/context_lens must be int32")
    if block_tables.dim() != 2 or block_tables.stride(1) != 1 or not context_lens.is_contiguous():
        raise ValueError("block_tables must be [B, max_blocks] row-major, context_lens contiguous")
    nb, bs = _cache_dims(k_cache, num_kv_heads * D)
    if out is None:
        out = torch.empty(B, H * D, dtype=q.dtype, device=q.device)
    if workspace is None:
        workspace = decode_workspace(B, H, num_kv_heads, D, q.device)
    _C.check(_C.load().b200_paged_decode_attn_capped(
        out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
        block_tables.data_ptr(), context_lens.data_ptr(), B, H, num_kv_heads, D,
        q.stride(0) if B > 1 else H * D, out.stride(0) if B > 1 else H * D, nb, bs,
        block_tables.stride(0), float(scale), float(softcap or 0.0), _ptr(sink), workspace.data_ptr(),
        workspace.numel(), int(num_ctas), _dt(q), _stream()), "b200_paged_decode_attn")
    return out


def paged_decode_attn_fp8(q, k_cache, v_cache, block_tables, context_lens, scale, num_kv_heads,
                          k_scale=1.0, v_scale=1.0, out=None, workspace=None, num_ctas=0):
    """K6 over an e4m3 cache. q [B, H, D] bf16/fp16 -> out [B, H*D] in q's dtype."""
    _need_cuda(q, k_cache, v_cache, block_tables, context_lens)
    B, H, D = q.shape
    if q.stride(2) != 1 or q.stride(1) != D:
        raise ValueError("q must be contiguous in (heads, head_dim)")
    if block_tables.dtype != torch.int32 or context_lens.dtype != torch.int32:
        raise TypeError("block_tables/context_lens must be int32")
    if block_tables.dim() != 2 or block_tables.stride(1) != 1 or not context_lens.is_contiguous():
        raise ValueError("block_tables must be [B, max_blocks] row-major, context_lens contiguous")
    if not (_is_fp8_cache(k_cache) and _is_fp8_cache(v_cache)):
        raise TypeError("fp8 KV caches must be uint8 or float8_e4m3fn tensors")
    nb, bs = _cache_dims(k_cache, num_kv_heads * D)
    if out is None:
        out = torch.empty(B, H * D, dtype=q.dtype, device=q.device)
    if workspace is None:
        workspace = decode_workspace(B, H, num_kv_heads, D, q.device)
    _C.check(_C.load().b200_paged_decode_attn_fp8(
        out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
        block_tables.data_ptr(), context_lens.data_ptr(), B, H, num_kv_heads, D,
        q.stride(0) if B > 1 else H * D, out.stride(0) if B > 1 else H * D, nb, bs,
        block_tables.stride(0), float(scale), float(k_scale), float(v_scale), workspace.data_ptr(),
        workspace.numel(), int(num_ctas), _dt(q), _stream()), "b200_paged_decode_attn_fp8")
    return out


def gather_dequant_fp8(k_cache, v_cache, block_tables, cu_seqlens_k, max_seqlen_k, num_kv_heads, head_dim,
                       k_scale=1.0, v_scale=1.0, dtype=torch.bfloat16, total_k=None):
    """Paged e4m3 caches -> packed [total_k, Hkv, D] K and V in `dtype` (prefix-hit / chunked prefill over
    an fp8 cache). total_k: number of packed rows (= cu_seqlens_k[-1]); when None it is bounded by
    num_seqs * max_seqlen_k so that no device value has to be read back."""
    _need_cuda(k_cache, v_cache, block_tables, cu_seqlens_k)
    if not (_is_fp8_cache(k_cache) and _is_fp8_cache(v_cache)):
        raise TypeError("fp8 KV caches must be uint8 or float8_e4m3fn tensors")
    if block_tables.dtype != torch.int32 or block_tables.stride(1) != 1 or cu_seqlens_k.dtype != torch.int32:
        raise TypeError("block_tables must be row-major int32, cu_seqlens_k int32")
    num_seqs = cu_seqlens_k.numel() - 1
    nb, bs = _cache_dims(k_cache, num_kv_heads * head_dim)
    rows = int(total_k) if total_k is not None else num_seqs * int(max_seqlen_k)
    # zeros, not empty: rows past the last sequence are inside the prefill kernel's TMA bounds, and a
    # masked key's probability 0 times a stale NaN pattern in V would poison the output row
    k = torch.zeros(rows, num_kv_heads, head_dim, dtype=dtype, device=k_cache.device)
    v = torch.zeros_like(k)
    _C.check(_C.load().b200_gather_dequant_fp8(
        k.data_ptr(), v.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
        cu_seqlens_k.data_ptr(), num_seqs, int(max_seqlen_k), block_tables.stride(0), nb, bs, num_kv_heads,
        head_dim, float(k_scale), float(v_scale), _dt(k), _stream()), "b200_gather_dequant_fp8")
    return k, v


_prefill_ws: dict = {}


def prefill_workspace(device, head_dim: int) -> torch.Tensor:
    """The split-KV workspace of the prefill kernel (b200_prefill_workspace_size bytes, a few MB),
    one per device and stream, allocated on first use -- outside CUDA-graph capture; prefill runs eagerly."""
    key = (device, head_dim, torch.cuda.current_stream(device).cuda_stream)   # concurrent launches must not share it
    ws = _prefill_ws.get(key)
    if ws is None:
        n = int(_C.load().b200_prefill_workspace_size(int(head_dim)))
        ws = _prefill_ws[key] = torch.empty(n, dtype=torch.uint8, device=device)
    return ws


def prefill_varlen_attn(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale,
                        num_kv_heads, block_tables=None, out=None, workspace="auto", softcap=0.0, sink=None):
    """K4/K5. q [Tq, H, D]; packed mode: k/v [Tk, Hkv, D]; paged mode (block_tables given):
    k/v are the caches [nb, bs, Hkv*D]. Returns out [Tq, H*D]. workspace: "auto" (the per-device
    split-KV workspace), None (never split the keys across CTAs) or a uint8 CUDA tensor. softcap, sink as in
    paged_decode_attn (the tcgen05 kernel only)."""
    _need_cuda(q, k, v, cu_seqlens_q, cu_seqlens_k, block_tables, sink)
    _f32(sink)
    Tq, H, D = q.shape
    if sink is not None and sink.numel() != H:
        raise ValueError("sink [H]")
    if q.stride(2) != 1 or q.stride(1) != D:
        raise ValueError("q must be contiguous in (heads, head_dim)")
    if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_k.dtype != torch.int32:
        raise TypeError("cu_seqlens must be int32")
    num_seqs = cu_seqlens_q.numel() - 1
    if out is None:
        out = torch.empty(Tq, H * D, dtype=q.dtype, device=q.device)
    if block_tables is not None:
        if block_tables.dtype != torch.int32 or block_tables.stride(1) != 1:
            raise TypeError("block_tables must be row-major int32")
        nb, bs = _cache_dims(k, num_kv_heads * D)
        ks = vs = num_kv_heads * D
        bt_ptr, bt_stride = block_tables.data_ptr(), block_tables.stride(0)
    else:
        if k.stride(2) != 1 or k.stride(1) != D or v.stride(2) != 1 or v.stride(1) != D:
            raise ValueError("k/v must be contiguous in (heads, head_dim)")
        nb = bs = 0
        ks = k.stride(0) if k.shape[0] > 1 else num_kv_heads * D
        vs = v.stride(0) if v.shape[0] > 1 else num_kv_heads * D
        bt_ptr, bt_stride = None, 0
    if isinstance(workspace, str):
        workspace = prefill_workspace(q.device, D)
    ws_ptr, ws_bytes = (None, 0) if workspace is None else (workspace.data_ptr(), workspace.numel())
    _C.check(_C.load().b200_prefill_varlen_attn_capped(
        out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), cu_seqlens_q.data_ptr(),
        cu_seqlens_k.data_ptr(), num_seqs, Tq, 0 if block_tables is not None else k.shape[0],
        int(max_seqlen_q), int(max_seqlen_k), H, num_kv_heads,
        D, q.stride(0) if Tq > 1 else H * D, ks, vs, out.stride(0) if Tq > 1 else H * D, bt_ptr,
        bt_stride, nb, bs, float(scale), float(softcap or 0.0), _ptr(sink), _dt(q), ws_ptr, ws_bytes, _stream()),
        "b200_prefill_varlen_attn")
    return out


def qknorm_rope_cache(qkv, positions, cos_sin_cache, q_norm_weight, k_norm_weight, eps,
                      k_cache, v_cache, slots, num_heads, num_kv_heads, head_dim):
    """K8, in place on qkv [T, (H+2Hkv)*D]. k_cache/v_cache/slots may be None (no cache bound)."""
    _need_cuda(qkv, positions, cos_sin_cache, q_norm_weight, k_norm_weight, k_cache, v_cache, slots)
    T = qkv.shape[0]
    if qkv.dim() != 2 or qkv.stride(1) != 1:
        raise ValueError("qkv must be [T, (H+2Hkv)*D] with unit inner stride")
    if positions.dtype != torch.int64 or not positions.is_contiguous():
        raise TypeError("positions must be contiguous int64")
    if cos_sin_cache.dtype != torch.float32 or not cos_sin_cache.is_contiguous():
        raise TypeError("cos_sin_cache must be contiguous fp32")
    if cos_sin_cache.shape[-1] != head_dim:
        raise ValueError("cos_sin_cache last dim must equal head_dim")
    have_cache = k_cache is not None and k_cache.numel() > 0
    nb = bs = 0
    if have_cache:
        nb, bs = _cache_dims(k_cache, num_kv_heads * head_dim)
        if slots.dtype != torch.int32 or not slots.is_contiguous():
            raise TypeError("slots must be contiguous int32")
    _C.check(_C.load().b200_qknorm_rope_cache(
        qkv.data_ptr(), positions.data_ptr(), cos_sin_cache.data_ptr(), _ptr(q_norm_weight),
        _ptr(k_norm_weight), float(eps), k_cache.data_ptr() if have_cache else None,
        v_cache.data_ptr() if have_cache else None, slots.data_ptr() if have_cache else None,
        1 if (have_cache and slots.dim() == 2) else 0, T, num_heads, num_kv_heads, head_dim,
        qkv.stride(0) if T > 1 else qkv.shape[1], cos_sin_cache.shape[0], nb, bs, _dt(qkv),
        _stream()), "b200_qknorm_rope_cache")
    return qkv


def rmsnorm(x, weight, eps, out=None):
    _need_cuda(x, weight)
    if not x.is_contiguous():
        raise ValueError("rmsnorm input must be contiguous")
    hidden = x.shape[-1]
    rows = x.numel() // hidden if hidden else 0
    if out is None:
        out = torch.empty_like(x)
    _C.check(_C.load().b200_rmsnorm(out.data_ptr(), x.data_ptr(), weight.data_ptr(), float(eps),
                                    rows, hidden, _dt(x), _stream()), "b200_rmsnorm")
    return out


def add_rmsnorm_(x, residual, weight, eps):
    """In place: residual <- x + residual; x <- RMSNorm(x + residual) * weight."""
    _need_cuda(x, residual, weight)
    if not (x.is_contiguous() and residual.is_contiguous()):
        raise ValueError("add_rmsnorm tensors must be contiguous")
    hidden = x.shape[-1]
    rows = x.numel() // hidden if hidden else 0
    _C.check(_C.load().b200_add_rmsnorm(x.data_ptr(), residual.data_ptr(), weight.data_ptr(),
                                        float(eps), rows, hidden, _dt(x), _stream()),
             "b200_add_rmsnorm")
    return x, residual


def silu_and_mul(x, out=None):
    _need_cuda(x)
    if not x.is_contiguous():
        raise ValueError("silu_and_mul input must be contiguous")
    inter = x.shape[-1] // 2
    rows = x.numel() // (2 * inter) if inter else 0
    if out is None:
        out = torch.empty(*x.shape[:-1], inter, dtype=x.dtype, device=x.device)
    _C.check(_C.load().b200_silu_and_mul(out.data_ptr(), x.data_ptr(), rows, inter, _dt(x),
                                         _stream()), "b200_silu_and_mul")
    return out


def sample(logits, temperatures=None, seed=0, step=0, out=None, step_offset=None):
    """argmax (temperatures=None or <= 0) or Gumbel-max sampling over [rows, vocab] bf16/fp16
    logits. step_offset: optional device int64 scalar added to `step` when the kernel runs."""
    _need_cuda(logits, temperatures, step_offset)
    rows, vocab = logits.shape
    if logits.stride(1) != 1:
        raise ValueError("logits must have unit inner stride")
    if temperatures is not None and (temperatures.dtype != torch.float32 or
                                     not temperatures.is_contiguous()):
        raise TypeError("temperatures must be contiguous fp32")
    if out is None:
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    _C.check(_C.load().b200_sample(out.data_ptr(), logits.data_ptr(), _ptr(temperatures), rows,
                                   vocab, logits.stride(0) if rows > 1 else vocab, int(seed),
                                   int(step), _ptr(step_offset), _dt(logits), _stream()),
             "b200_sample")
    return out


def sample_shard(logits, temperatures=None, seed=0, step=0, index_offset=0, out=None, step_offset=None):
    """Vocab-sharded sampling (tensor parallelism): packed (score, global index) keys of this rank's
    shard, to be MAX-all-reduced over the ranks; see include/b200attn.h::b200_sample_shard."""
    _need_cuda(logits, temperatures, step_offset)
    rows, vocab = logits.shape
    if logits.stride(1) != 1:
        raise ValueError("logits must have unit inner stride")
    if temperatures is not None and (temperatures.dtype != torch.float32 or
                                     not temperatures.is_contiguous()):
        raise TypeError("temperatures must be contiguous fp32")
    if out is None:
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    _C.check(_C.load().b200_sample_shard(out.data_ptr(), logits.data_ptr(), _ptr(temperatures), rows, vocab,
                                         logits.stride(0) if rows > 1 else vocab, int(index_offset),
                                         int(seed), int(step), _ptr(step_offset), _dt(logits), _stream()),
             "b200_sample_shard")
    return out


def decode_sample_keys(keys: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Token ids from (all-reduced) sample_shard keys: id = 0x7fffffff - (key & 0x7fffffff)."""
    ids = 0x7FFFFFFF - (keys & 0x7FFFFFFF)
    if out is None:
        return ids
    out.copy_(ids)
    return out


# ------------------------------------------------------------------ dense layers on the grouped tcgen05 kernel
_dense_offsets: dict = {}


def _dense_plan(rows: int, device) -> torch.Tensor:
    """offsets = {0, rows}: one group holding every row (csrc/moe_umma.cu serves an ordinary linear
    layer as a one-expert group). Cached per (rows, device) so that graph capture never allocates it."""
    key = (rows, device)
    t = _dense_offsets.get(key)
    if t is None:
        t = _dense_offsets[key] = torch.tensor([0, rows], dtype=torch.int32, device=device)
    return t


def gate_up_silu_umma(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """SiluAndMul(x @ w_gate_up.T) in ONE kernel: the gate|up GEMM of a dense MLP on the grouped tcgen05
    kernel (one group) with the activation as its TMEM epilogue. Not on the decode path: at M = 256
    it measured 41.87 k tok/s against 41.93 k for cuBLAS + silu_and_mul (no gain, r02).
    x [M, K] contiguous; w_gate_up [2*I, K] (gate rows, then up rows); K % 64 == 0, I % 64 == 0."""
    _need_cuda(x, w_gate_up)
    M, K = x.shape
    inter = w_gate_up.shape[0] // 2
    if not x.is_contiguous() or not w_gate_up.is_contiguous() or w_gate_up.shape[1] != K:
        raise ValueError("gate_up_silu_umma takes contiguous x [M, K] and w [2*I, K]")
    h = torch.empty(M, inter, dtype=x.dtype, device=x.device)
    _C.check(_C.load().b200_moe_gemm_gate_up_umma(h.data_ptr(), x.data_ptr(), w_gate_up.data_ptr(),
                                                  _dense_plan(M, x.device).data_ptr(), M, K, inter, 1,
                                                  _dt(x), _stream()), "b200_moe_gemm_gate_up_umma (dense)")
    return h


def linear_umma(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """x @ w.T on the same kernel (plain epilogue). x [M, K]; w [N, K]; K % 64 == 0, N % 128 == 0."""
    _need_cuda(x, w)
    M, K = x.shape
    N = w.shape[0]
    if not x.is_contiguous() or not w.is_contiguous() or w.shape[1] != K:
        raise ValueError("linear_umma takes contiguous x [M, K] and w [N, K]")
    if out is None:
        out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    elif out.shape != (M, N) or not out.is_contiguous() or out.dtype != x.dtype:
        raise ValueError("out must be a contiguous [M, N] tensor of x's dtype")
    _C.check(_C.load().b200_moe_gemm_down_umma(out.data_ptr(), x.data_ptr(), w.data_ptr(),
                                               _dense_plan(M, x.device).data_ptr(), None, None, M, K, N, 1,
                                               _dt(x), _stream()), "b200_moe_gemm_down_umma (dense)")
    return out


def scores_umma(x: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor | None = None) -> torch.Tensor:
    """Products with fp32 OUTPUT on the tcgen05 kernel (the accumulators are stored unrounded): attention scores of
    16-bit operands. x [M, K] @ w [N, K]^T, or grouped: w [G, N, K] and offsets int32 [G + 1], rows offsets[g] ..
    offsets[g+1] of x against w[g]. Contiguous; K % 64 == 0, N % 128 == 0, G <= 256. Returns fp32 [M, N]."""
    _need_cuda(x, w, offsets)
    M, K = x.shape
    G = w.shape[0] if w.dim() == 3 else 1
    N = w.shape[-2]
    if not x.is_contiguous() or not w.is_contiguous() or w.shape[-1] != K or x.dtype != w.dtype:
        raise ValueError("scores_umma takes contiguous x [M, K] and w [(G,) N, K] of one 16-bit dtype")
    if (offsets is None) != (w.dim() == 2) or (offsets is not None and (offsets.dtype != torch.int32 or
                                                                        offsets.numel() != G + 1)):
        raise ValueError("grouped form: w [G, N, K] with int32 offsets [G + 1]")
    out = torch.empty(M, N, dtype=torch.float32, device=x.device)
    off = offsets if offsets is not None else _dense_plan(M, x.device)
    _C.check(_C.load().b200_gemm_f32out_umma(out.data_ptr(), x.data_ptr(), w.data_ptr(), off.data_ptr(), M, K, N, G,
                                             _dt(x), _stream()), "b200_gemm_f32out_umma")
    return out


# ------------------------------------------------------------------ sparse MoE (csrc/moe.cu)
class MoePlan:
    """Device-side dispatch plan of one MoE layer call (b200_moe_align): fixed-capacity buffers,
    nothing is read back by the host."""
    __slots__ = ("offsets", "sorted_pair", "pos_of_pair", "counts", "num_local", "expert_begin", "top_k")

    def __init__(self, num_pairs: int, num_local: int, expert_begin: int, top_k: int, device):
        i32 = dict(dtype=torch.int32, device=device)
        self.offsets = torch.empty(num_local + 1, **i32)
        self.sorted_pair = torch.zeros(num_pairs, **i32)     # tail beyond offsets[-1] stays 0 (a valid pair index)
        self.pos_of_pair = torch.empty(num_pairs, **i32)
        self.counts = torch.empty(num_local, **i32)
        self.num_local, self.expert_begin, self.top_k = num_local, expert_begin, top_k


def moe_route(router_logits: torch.Tensor, top_k: int):
    """softmax (fp32) over all experts + top-k + renormalise (qwen3_moe.py:150-158).
    router_logits [T, E] bf16/fp16 -> (topk_ids int32 [T, k], topk_weights dtype [T, k])."""
    _need_cuda(router_logits)
    T, E = router_logits.shape
    if router_logits.stride(1) != 1:
        raise ValueError("router_logits must be contiguous along the expert dimension")
    ids = torch.empty(T, top_k, dtype=torch.int32, device=router_logits.device)
    w = torch.empty(T, top_k, dtype=router_logits.dtype, device=router_logits.device)
    _C.check(_C.load().b200_moe_route(ids.data_ptr(), w.data_ptr(), router_logits.data_ptr(), T, E, top_k,
                                      router_logits.stride(0) if T > 1 else E, _dt(router_logits),
                                      _stream()), "b200_moe_route")
    return ids, w


def moe_align(topk_ids: torch.Tensor, expert_begin: int, num_local: int) -> MoePlan:
    """Pairs (t, j) stably sorted by local expert; see include/b200attn.h."""
    _need_cuda(topk_ids)
    if topk_ids.dtype != torch.int32 or not topk_ids.is_contiguous():
        raise TypeError("topk_ids must be a contiguous int32 tensor")
    T, k = topk_ids.shape
    plan = MoePlan(T * k, num_local, expert_begin, k, topk_ids.device)
    _C.check(_C.load().b200_moe_align(plan.offsets.data_ptr(), plan.sorted_pair.data_ptr(),
                                      plan.pos_of_pair.data_ptr(), plan.counts.data_ptr(),
                                      topk_ids.data_ptr(), T * k, expert_begin, num_local, _stream()),
             "b200_moe_align")
    return plan


def moe_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_ids: torch.Tensor,
                topk_weights: torch.Tensor, plan: MoePlan, out: torch.Tensor | None = None) -> torch.Tensor:
    """The expert MLPs of the local experts and the per-token combine.
    x [T, hidden]; w13 [num_local, 2*inter, hidden]; w2 [num_local, hidden, inter].
    Returns out [T, hidden]: this rank's partial sum (the full result when it owns every expert)."""
    _need_cuda(x, w13, w2, topk_ids, topk_weights)
    T, hidden = x.shape
    n_local, two_i, h2 = w13.shape
    inter = two_i // 2
    if h2 != hidden or w2.shape != (n_local, hidden, inter) or n_local != plan.num_local:
        raise ValueError("expert weight shapes do not match")
    if not (w13.is_contiguous() and w2.is_contiguous() and topk_weights.is_contiguous()):
        raise ValueError("expert weights / routing weights must be contiguous")
    if x.stride(1) != 1 or x.dtype != w13.dtype or x.dtype != w2.dtype or x.dtype != topk_weights.dtype:
        raise ValueError("x must be row-major and share its dtype with the weights")
    k = plan.top_k
    pairs = T * k
    lib = _C.load()
    if _MOE_BIG_GEMM != "stream" and pairs >= _MOE_BIG_GEMM_ROWS * n_local:
        big = _moe_expert_gemms_umma if _MOE_BIG_GEMM == "umma" else _moe_expert_gemms_library
        y = big(x, w13, w2, topk_weights, plan)
        return _moe_combine(lib, y, topk_ids, plan, T, hidden, out, x)
    h = torch.empty(pairs, inter, dtype=x.dtype, device=x.device)
    y = torch.empty(pairs, hidden, dtype=x.dtype, device=x.device)
    _C.check(lib.b200_moe_gemm_gate_up(h.data_ptr(), x.data_ptr(), w13.data_ptr(), plan.offsets.data_ptr(),
                                       plan.sorted_pair.data_ptr(), hidden, inter, n_local, k,
                                       x.stride(0) if T > 1 else hidden, _dt(x), _stream()),
             "b200_moe_gemm_gate_up")
    _C.check(lib.b200_moe_gemm_down(y.data_ptr(), h.data_ptr(), w2.data_ptr(), plan.offsets.data_ptr(),
                                    plan.sorted_pair.data_ptr(), topk_weights.data_ptr(), inter, hidden,
                                    n_local, k, _dt(x), _stream()), "b200_moe_gemm_down")
    return _moe_combine(lib, y, topk_ids, plan, T, hidden, out, x)


# Prefill-sized batches (hundreds of rows per expert) are tensor-bound, not weight-streaming: from
# _MOE_BIG_GEMM_ROWS average rows per local expert on they go through the tcgen05 grouped GEMM of
# csrc/moe_umma.cu (measured on Qwen3-30B-A3B, 4096-token prefill layer: 721 us vs 1224 us for the
# weight-streaming kernel; whole-model prefill 99.9 k vs 51.8 k tok/s). Module attributes, not
# environment switches: "stream" forces the weight-streaming kernel for every size, "library" routes
# through torch._grouped_mm (comparator for tools/moe_diag.py and the tests).
_MOE_BIG_GEMM = "umma"
_MOE_BIG_GEMM_ROWS = 96


def _moe_expert_gemms_umma(x, w13, w2, topk_weights, plan: MoePlan) -> torch.Tensor:
    T, hidden = x.shape
    n_local, two_i, _ = w13.shape
    inter, k = two_i // 2, plan.top_k
    pairs = T * k
    lib = _C.load()
    xs = torch.empty(pairs, hidden, dtype=x.dtype, device=x.device)
    h = torch.empty(pairs, inter, dtype=x.dtype, device=x.device)
    y = torch.empty(pairs, hidden, dtype=x.dtype, device=x.device)
    _C.check(lib.b200_moe_gather_rows(xs.data_ptr(), x.data_ptr(), plan.offsets.data_ptr(),
                                      plan.sorted_pair.data_ptr(), pairs, n_local, k, hidden,
                                      x.stride(0) if T > 1 else hidden, _dt(x), _stream()),
             "b200_moe_gather_rows")
    _C.check(lib.b200_moe_gemm_gate_up_umma(h.data_ptr(), xs.data_ptr(), w13.data_ptr(),
                                            plan.offsets.data_ptr(), pairs, hidden, inter, n_local,
                                            _dt(x), _stream()), "b200_moe_gemm_gate_up_umma")
    _C.check(lib.b200_moe_gemm_down_umma(y.data_ptr(), h.data_ptr(), w2.data_ptr(), plan.offsets.data_ptr(),
                                         plan.sorted_pair.data_ptr(), topk_weights.data_ptr(), pairs, inter,
                                         hidden, n_local, _dt(x), _stream()), "b200_moe_gemm_down_umma")
    return y


def moe_experts_ungated(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_ids: torch.Tensor,
                        topk_weights: torch.Tensor, plan: MoePlan, act: str = "relu2") -> torch.Tensor:
    """Experts WITHOUT a gate on the tensor-core kernels, down(act(up x)) and the per-token combine, 16-bit models:
    x [T, hidden]; w1 [E, inter, hidden]; w2 [E, hidden, inter]; topk_weights [T, k] in x's dtype. Prompt-sized
    batches gather their rows and run both products on the grouped tcgen05 GEMM (the activation between them);
    smaller ones run on the weight-streaming kernels (the activation is the up product's epilogue).
    hidden % 128 == 0, inter % 128 == 0."""
    _need_cuda(x, w1, w2, topk_ids, topk_weights)
    T, hidden = x.shape
    E, inter, h2 = w1.shape
    if h2 != hidden or w2.shape != (E, hidden, inter) or E != plan.num_local:
        raise ValueError("expert weight shapes do not match")
    if not (w1.is_contiguous() and w2.is_contiguous() and topk_weights.is_contiguous()):
        raise ValueError("expert weights / routing weights must be contiguous")
    if x.stride(1) != 1 or x.dtype != w1.dtype or x.dtype != w2.dtype or x.dtype != topk_weights.dtype:
        raise ValueError("x must be row-major and share its dtype with the weights")
    k = plan.top_k
    pairs = T * k
    lib = _C.load()
    h = torch.empty(pairs, inter, dtype=x.dtype, device=x.device)
    y = torch.empty(pairs, hidden, dtype=x.dtype, device=x.device)
    if _MOE_BIG_GEMM != "stream" and pairs >= _MOE_BIG_GEMM_ROWS * E:
        xs = torch.empty(pairs, hidden, dtype=x.dtype, device=x.device)
        _C.check(lib.b200_moe_gather_rows(xs.data_ptr(), x.data_ptr(), plan.offsets.data_ptr(),
                                          plan.sorted_pair.data_ptr(), pairs, E, k, hidden,
                                          x.stride(0) if T > 1 else hidden, _dt(x), _stream()), "b200_moe_gather_rows")
        _C.check(lib.b200_moe_gemm_down_umma(h.data_ptr(), xs.data_ptr(), w1.data_ptr(), plan.offsets.data_ptr(), None,
                                             None, pairs, hidden, inter, E, _dt(x), _stream()),
                 "b200_moe_gemm_down_umma (up)")
        h = act_only(h, act)
        _C.check(lib.b200_moe_gemm_down_umma(y.data_ptr(), h.data_ptr(), w2.data_ptr(), plan.offsets.data_ptr(),
                                             plan.sorted_pair.data_ptr(), topk_weights.data_ptr(), pairs, inter,
                                             hidden, E, _dt(x), _stream()), "b200_moe_gemm_down_umma")
        return _moe_combine(lib, y, topk_ids, plan, T, hidden, None, x)
    _C.check(lib.b200_moe_gemm_up_act(h.data_ptr(), x.data_ptr(), w1.data_ptr(), plan.offsets.data_ptr(),
                                      plan.sorted_pair.data_ptr(), hidden, inter, E, k,
                                      x.stride(0) if T > 1 else hidden, _PLAIN_ACTS[act], _dt(x), _stream()),
             "b200_moe_gemm_up_act")
    _C.check(lib.b200_moe_gemm_down(y.data_ptr(), h.data_ptr(), w2.data_ptr(), plan.offsets.data_ptr(),
                                    plan.sorted_pair.data_ptr(), topk_weights.data_ptr(), inter, hidden, E, k,
                                    _dt(x), _stream()), "b200_moe_gemm_down")
    return _moe_combine(lib, y, topk_ids, plan, T, hidden, None, x)


def moe_experts_glu_clamped(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_ids: torch.Tensor,
                            topk_weights: torch.Tensor, plan: MoePlan, alpha: float, limit: float) -> torch.Tensor:
    """Gated experts whose unit is the clamped one of glu_clamped, 16-bit models on the tensor-core kernels. Prompt-sized
    batches run on the grouped tcgen05 GEMM: rows gathered by expert, gate and up rows of every expert as ONE product
    (w13 [E, 2*inter, hidden]), the unit, the down product with the routing weights in its epilogue; smaller ones on the
    weight-streaming kernels (the unit is the gate/up product's epilogue). Then the per-token combine. topk_weights
    [T, k] in x's dtype. hidden % 128 == 0, inter % 64 == 0."""
    _need_cuda(x, w13, w2, topk_ids, topk_weights)
    T, hidden = x.shape
    E, two_i, h2 = w13.shape
    inter = two_i // 2
    if h2 != hidden or w2.shape != (E, hidden, inter) or E != plan.num_local:
        raise ValueError("expert weight shapes do not match")
    if not (w13.is_contiguous() and w2.is_contiguous() and topk_weights.is_contiguous()):
        raise ValueError("expert weights / routing weights must be contiguous")
    if x.stride(1) != 1 or x.dtype != w13.dtype or x.dtype != w2.dtype or x.dtype != topk_weights.dtype:
        raise ValueError("x must be row-major and share its dtype with the weights")
    k = plan.top_k
    pairs = T * k
    lib = _C.load()
    y = torch.empty(pairs, hidden, dtype=x.dtype, device=x.device)
    if _MOE_BIG_GEMM == "stream" or pairs < _MOE_BIG_GEMM_ROWS * E:
        h = torch.empty(pairs, inter, dtype=x.dtype, device=x.device)
        _C.check(lib.b200_moe_gemm_gate_up_glu(h.data_ptr(), x.data_ptr(), w13.data_ptr(), plan.offsets.data_ptr(),
                                               plan.sorted_pair.data_ptr(), hidden, inter, E, k,
                                               x.stride(0) if T > 1 else hidden, float(alpha), float(limit), _dt(x),
                                               _stream()), "b200_moe_gemm_gate_up_glu")
        _C.check(lib.b200_moe_gemm_down(y.data_ptr(), h.data_ptr(), w2.data_ptr(), plan.offsets.data_ptr(),
                                        plan.sorted_pair.data_ptr(), topk_weights.data_ptr(), inter, hidden, E, k,
                                        _dt(x), _stream()), "b200_moe_gemm_down")
        return _moe_combine(lib, y, topk_ids, plan, T, hidden, None, x)
    xs = torch.empty(pairs, hidden, dtype=x.dtype, device=x.device)
    gu = torch.empty(pairs, two_i, dtype=x.dtype, device=x.device)
    _C.check(lib.b200_moe_gather_rows(xs.data_ptr(), x.data_ptr(), plan.offsets.data_ptr(), plan.sorted_pair.data_ptr(),
                                      pairs, E, k, hidden, x.stride(0) if T > 1 else hidden, _dt(x), _stream()),
             "b200_moe_gather_rows")
    _C.check(lib.b200_moe_gemm_down_umma(gu.data_ptr(), xs.data_ptr(), w13.data_ptr(), plan.offsets.data_ptr(), None,
                                         None, pairs, hidden, two_i, E, _dt(x), _stream()),
             "b200_moe_gemm_down_umma (gate | up)")
    h = glu_clamped(gu, alpha, limit)
    _C.check(lib.b200_moe_gemm_down_umma(y.data_ptr(), h.data_ptr(), w2.data_ptr(), plan.offsets.data_ptr(),
                                         plan.sorted_pair.data_ptr(), topk_weights.data_ptr(), pairs, inter, hidden, E,
                                         _dt(x), _stream()), "b200_moe_gemm_down_umma")
    return _moe_combine(lib, y, topk_ids, plan, T, hidden, None, x)


def _moe_expert_gemms_library(x, w13, w2, topk_weights, plan: MoePlan) -> torch.Tensor:
    k = plan.top_k
    pair = plan.sorted_pair.long()                    # tail entries are 0: harmless rows, never combined
    xs = x.index_select(0, pair // k)                 # [pairs, hidden] in expert order
    offs = plan.offsets[1:]
    gu = torch._grouped_mm(xs, w13.transpose(1, 2), offs=offs)
    h = silu_and_mul(gu)
    y = torch._grouped_mm(h, w2.transpose(1, 2), offs=offs)
    return y * topk_weights.reshape(-1)[pair].unsqueeze(1)      # dtype multiply, as qwen3_moe.py:180-182


def _moe_combine(lib, y, topk_ids, plan: MoePlan, T, hidden, out, x):
    k = plan.top_k
    if out is None:
        out = torch.empty(T, hidden, dtype=x.dtype, device=x.device)
    elif out.shape != (T, hidden) or out.dtype != x.dtype or out.stride(1) != 1:
        raise ValueError("out must be a row-major [T, hidden] tensor of x's dtype")
    _C.check(lib.b200_moe_combine(out.data_ptr(), y.data_ptr(), topk_ids.data_ptr(),
                                  plan.pos_of_pair.data_ptr(), T, k, hidden,
                                  out.stride(0) if T > 1 else hidden, _dt(x), _stream()),
             "b200_moe_combine")
    return out


# ---------------------------------------------------------------------------------------------------
# Sequence-mixer kernels of the hybrid decoders (csrc/seq_ops.cu, csrc/seq_mixers.cu). They take bf16,
# fp16 and fp32 activations; small parameters (norm weights, convolution taps, decays) are fp32 tensors.
_DT3 = {torch.bfloat16: _C.BF16, torch.float16: _C.F16, torch.float32: _C.F32}


def _dt3(t: torch.Tensor) -> int:
    try:
        return _DT3[t.dtype]
    except KeyError:
        raise TypeError(f"sequence-mixer kernels take bf16/fp16/fp32 tensors, got {t.dtype}") from None


def _f32(*tensors) -> None:
    for t in tensors:
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or not t.is_cuda):
            raise TypeError("small parameters of the sequence-mixer kernels are contiguous fp32 CUDA tensors")


class StepSpans:
    """Which tokens of the step belong to which sequence, as the kernels take it: packed spans
    (``cu_q``/``cu_k``, any mix of prompt portions and single tokens) or one token per row
    (``ctx_lens``; 0 = a padded graph row). Built from the runner's step context, or directly in tests."""
    __slots__ = ("cu_q", "cu_k", "ctx_lens", "num_seqs", "max_q")

    def __init__(self, cu_q=None, cu_k=None, ctx_lens=None, max_q=1):
        if (cu_q is None) == (ctx_lens is None):
            raise ValueError("give either cu_q/cu_k (packed spans) or ctx_lens (one token per row)")
        for t in (cu_q, cu_k, ctx_lens):
            if t is not None and (t.dtype != torch.int32 or not t.is_contiguous() or not t.is_cuda):
                raise TypeError("span tensors are contiguous int32 CUDA tensors")
        self.cu_q, self.cu_k, self.ctx_lens = cu_q, cu_k, ctx_lens
        self.num_seqs = (cu_q.numel() - 1) if cu_q is not None else ctx_lens.numel()
        self.max_q = int(max_q) if cu_q is not None else 1

    @classmethod
    def of(cls, context) -> "StepSpans":
        if context.is_prefill:
            return cls(context.cu_seqlens_q, context.cu_seqlens_k, None, context.max_seqlen_q)
        return cls(None, None, context.context_lens)

    def ptrs(self):
        return _ptr(self.cu_q), _ptr(self.cu_k), _ptr(self.ctx_lens)


def residual_rmsnorm(residual, weight, eps, dtype, offset=1.0):
    """h = residual * rsqrt(mean(residual^2) + eps) * (offset + weight); residual fp32 [rows, hidden] -> h in `dtype`."""
    _need_cuda(residual, weight)
    _f32(residual, weight)
    rows, hidden = residual.shape
    out = torch.empty(rows, hidden, dtype=dtype, device=residual.device)
    _C.check(_C.load().b200_residual_rmsnorm(out.data_ptr(), residual.data_ptr(), weight.data_ptr(), float(offset),
                                             float(eps), rows, hidden, _dt3(out), _stream()),
             "b200_residual_rmsnorm")
    return out


def residual_add_norms_(y, residual, w_post, w_pre, eps, offset=1.0):
    """residual += norm(y; w_post) in place (fp32); returns h = norm(residual; w_pre) in y's dtype, or None when
    w_pre is None. Both norms are x * rsqrt(mean x^2 + eps) * (offset + w)."""
    _need_cuda(y, residual, w_post, w_pre)
    _f32(residual, w_post, w_pre)
    if not y.is_contiguous() or y.shape != residual.shape:
        raise ValueError("y must be contiguous and shaped like the residual")
    rows, hidden = residual.shape
    h = torch.empty_like(y) if w_pre is not None else None
    _C.check(_C.load().b200_residual_add_norms(_ptr(h), residual.data_ptr(), y.data_ptr(), w_post.data_ptr(),
                                               _ptr(w_pre), float(offset), float(eps), rows, hidden, _dt3(y),
                                               _stream()), "b200_residual_add_norms")
    return h


def causal_conv(x, weight, bias, spans: StepSpans, state=None, state_slots=None, act=None):
    """Depth-wise causal convolution over time. x [T, C] (row-strided view allowed), weight fp32 [C, taps] (last
    column = current token), bias fp32 [C] or None, act None | "silu". state [slots, taps-1, C] in x's dtype holds
    each sequence's last taps-1 inputs between steps (read unless the span starts at position 0, then rewritten)."""
    _need_cuda(x, weight, bias, state, state_slots)
    _f32(weight, bias)
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be [T, C] with unit inner stride")
    T, C = x.shape
    taps = weight.shape[1]
    if weight.shape[0] != C:
        raise ValueError("one row of taps per channel")
    if state is not None:
        if state.dtype != x.dtype or not state.is_contiguous() or tuple(state.shape[1:]) != (taps - 1, C):
            raise ValueError(f"conv state must be a contiguous [slots, {taps - 1}, {C}] tensor of x's dtype")
        if state_slots is None or state_slots.dtype != torch.int32:
            raise TypeError("state_slots must be int32")
    out = torch.empty(T, C, dtype=x.dtype, device=x.device)
    cu_q, cu_k, ctx = spans.ptrs()
    _C.check(_C.load().b200_causal_conv(out.data_ptr(), C, x.data_ptr(), x.stride(0) if T > 1 else C,
                                        weight.data_ptr(), _ptr(bias), 1 if act == "silu" else 0, _ptr(state),
                                        _ptr(state_slots), cu_q, cu_k, ctx, spans.num_seqs, spans.max_q, C, taps,
                                        _dt3(x), _stream()), "b200_causal_conv")
    return out


def unitnorm_temp_cache(qkv, positions, eps, temp_coef, temp_every, num_heads, num_kv_heads, dim, vdim,
                        k_cache=None, v_cache=None, slots=None):
    """In place on qkv [T, H*dim | G*dim | G*vdim]: every q and k head is divided by its root mean square, q is
    then scaled by 1 + coef * ln(floor((pos + 1) / every) + 1); k and v rows are stored at `slots` of the paged
    caches [nb, bs, G*dim] / [nb, bs, G*vdim] when those are given."""
    _need_cuda(qkv, positions, k_cache, v_cache, slots)
    T = qkv.shape[0]
    if qkv.dim() != 2 or qkv.stride(1) != 1 or qkv.shape[1] != num_heads * dim + num_kv_heads * (dim + vdim):
        raise ValueError("qkv must be [T, H*dim + G*dim + G*vdim] with unit inner stride")
    if positions.dtype != torch.int64 or not positions.is_contiguous():
        raise TypeError("positions must be contiguous int64")
    have = k_cache is not None and k_cache.numel() > 0
    bs = 0
    if have:
        _, bs = _cache_dims(k_cache, num_kv_heads * dim)
        _cache_dims(v_cache, num_kv_heads * vdim)
        if slots.dtype != torch.int32 or not slots.is_contiguous():
            raise TypeError("slots must be contiguous int32")
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
            raise TypeError("caches must have the activations' dtype")
    _C.check(_C.load().b200_unitnorm_temp_cache(
        qkv.data_ptr(), qkv.stride(0) if T > 1 else qkv.shape[1], positions.data_ptr(), float(eps),
        float(temp_coef), int(temp_every), k_cache.data_ptr() if have else None,
        v_cache.data_ptr() if have else None, slots.data_ptr() if have else None,
        1 if (have and slots.dim() == 2) else 0, bs, T, num_heads, num_kv_heads, dim, vdim, _dt3(qkv), _stream()),
        "b200_unitnorm_temp_cache")
    return qkv


def gated_norm(y, gate, weight, eps, groups=1, gate_first=False, gate_act="sigmoid", dtype=None):
    """y [rows, n] (fp32 or gate's dtype), gate [rows, n] (row-strided view allowed) -> [rows, n] in gate's dtype.
    weight fp32 [n]: RMS norm over each of `groups` equal parts, before (gate_first=False) or after the gate;
    weight None: the gate alone. gate None (with a weight): the grouped norm alone, output in `dtype`."""
    _need_cuda(y, gate, weight)
    _f32(weight)
    rows, n = y.shape
    if gate is None:
        if weight is None or dtype is None:
            raise ValueError("without a gate: give the norm weight and the output dtype")
        gate_act = "none"
    elif gate.shape != y.shape or gate.stride(1) != 1:
        raise ValueError("gate [rows, n] with unit inner stride")
    else:
        dtype = gate.dtype
    if not y.is_contiguous():
        raise ValueError("y contiguous [rows, n]")
    if y.dtype not in (torch.float32, dtype):
        raise TypeError("y must be fp32 or of the gate's dtype")
    out = torch.empty(rows, n, dtype=dtype, device=y.device)
    _C.check(_C.load().b200_gated_norm(out.data_ptr(), y.data_ptr(), 1 if y.dtype == torch.float32 else 0,
                                       _ptr(gate), (gate.stride(0) if rows > 1 else n) if gate is not None else n,
                                       _ptr(weight), float(eps), rows, n, int(groups), 1 if gate_first else 0,
                                       {"sigmoid": 0, "silu": 1, "none": 2}[gate_act], _DT3[dtype], _stream()),
             "b200_gated_norm")
    return out


_ACTS = {"silu": 0, "relu": 1, "gelu_tanh": 2}


def act_and_mul(x, act="silu"):
    """x [rows, 2*inter] = (gate | up) -> act(gate) * up, act in silu | relu | gelu_tanh."""
    _need_cuda(x)
    if not x.is_contiguous() or x.dim() != 2:
        raise ValueError("act_and_mul input must be a contiguous matrix")
    rows, inter = x.shape[0], x.shape[1] // 2
    out = torch.empty(rows, inter, dtype=x.dtype, device=x.device)
    _C.check(_C.load().b200_act_and_mul(out.data_ptr(), x.data_ptr(), rows, inter, _ACTS[act], _dt3(x), _stream()),
             "b200_act_and_mul")
    return out


_PLAIN_ACTS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "relu2": 3}


def act_only(x, act="relu2"):
    """act(x) elementwise for a feed-forward without a gate: silu | relu | gelu_tanh | relu2 (the square of relu)."""
    _need_cuda(x)
    if not x.is_contiguous():
        raise ValueError("act_only input must be contiguous")
    out = torch.empty_like(x)
    _C.check(_C.load().b200_act_only(out.data_ptr(), x.data_ptr(), x.numel(), _PLAIN_ACTS[act], _dt3(x), _stream()),
             "b200_act_only")
    return out


def norm_residual_(residual, y, w, b, eps, dtype, kind="layer", offset=0.0, accumulate=True, y_index=None, y2=None,
                   y2_index=None, want_h=True):
    """A norm on a sublayer's OUTPUT, then the residual: residual (fp32 [rows, hidden], in place) <- (residual if
    accumulate else 0) + norm(y [+ y2]); returns the new residual in `dtype` (the next sublayer reads the stream
    itself). kind "layer": (u - mean) / sqrt(var + eps) * w + b; "rms": u / sqrt(mean u^2 + eps) * (offset + w).
    y_index / y2_index (int64 [rows]): rows of y / y2 are gathered by index (clamped to the table) -- token embedding
    plus learned position plus norm in one launch."""
    _need_cuda(residual, y, w, b, y_index, y2, y2_index)
    _f32(residual, w, b)
    rows, hidden = residual.shape
    for t, idx in ((y, y_index), (y2, y2_index)):
        if t is None:
            continue
        if not t.is_contiguous() or t.shape[-1] != hidden or t.dtype != dtype or (idx is None and t.shape[0] != rows):
            raise ValueError("y / y2: contiguous [rows or table, hidden] of the model dtype")
        if idx is not None and (idx.dtype != torch.int64 or not idx.is_contiguous() or idx.numel() != rows):
            raise TypeError("row indices are contiguous int64 [rows]")
    h = torch.empty(rows, hidden, dtype=dtype, device=residual.device) if want_h else None
    _C.check(_C.load().b200_norm_residual(_ptr(h), residual.data_ptr(), y.data_ptr(), _ptr(y_index), y.shape[0],
                                          _ptr(y2), _ptr(y2_index), y2.shape[0] if y2 is not None else 0,
                                          w.data_ptr(), _ptr(b), float(eps), float(offset),
                                          {"layer": 0, "rms": 1}[kind], 1 if accumulate else 0, rows, hidden,
                                          _DT3[dtype], _stream()), "b200_norm_residual")
    return h


def rownorm_cache(x, nq, nk, nv, wq, wk, eps, k_cache=None, v_cache=None, slots=None):
    """In place on x [T, nq + nk + nv] (unit inner stride): the nq query columns and the nk key columns are each
    divided by the root mean square of ALL their columns (every head at once) and multiplied by the plain weights wq,
    wk; k and v rows are stored at `slots` of the paged caches [nb, bs, nk] / [nb, bs, nv] when given. nk = nv = 0: a
    layer that projects queries only."""
    _need_cuda(x, wq, wk, k_cache, v_cache, slots)
    _f32(wq, wk)
    T = x.shape[0]
    if x.dim() != 2 or x.stride(1) != 1 or x.shape[1] != nq + nk + nv or wq.numel() != nq or (nk and wk.numel() != nk):
        raise ValueError("x must be [T, nq + nk + nv] with unit inner stride; one weight per q / k column")
    have = k_cache is not None and k_cache.numel() > 0 and nk > 0
    bs = 0
    if have:
        _, bs = _cache_dims(k_cache, nk)
        _cache_dims(v_cache, nv)
        if slots.dtype != torch.int32 or not slots.is_contiguous():
            raise TypeError("slots must be contiguous int32")
        if k_cache.dtype != x.dtype or v_cache.dtype != x.dtype:
            raise TypeError("caches must have the activations' dtype")
    _C.check(_C.load().b200_rownorm_cache(x.data_ptr(), x.stride(0) if T > 1 else x.shape[1], wq.data_ptr(), _ptr(wk),
                                          float(eps), k_cache.data_ptr() if have else None,
                                          v_cache.data_ptr() if have else None, slots.data_ptr() if have else None,
                                          1 if (have and slots.dim() == 2) else 0, bs, T, nq, nk, nv, _dt3(x),
                                          _stream()), "b200_rownorm_cache")
    return x


def gate_prep(q, f, bias, lower):
    """q, f [T, n] (row-strided views) -> (silu(q), lower + (1 - lower) * sigmoid(f + bias)), both fp32 [T, n]: the
    query and the lower-bounded forget gate of a gated linear recurrence; bias, lower fp32 [n] or None (0)."""
    _need_cuda(q, f, bias, lower)
    _f32(bias, lower)
    T, n = q.shape
    if f.shape != q.shape or q.stride(1) != 1 or f.stride(1) != 1 or q.dtype != f.dtype:
        raise ValueError("q, f [T, n] with unit inner stride, one dtype")
    q32 = torch.empty(T, n, dtype=torch.float32, device=q.device)
    f32 = torch.empty(T, n, dtype=torch.float32, device=q.device)
    stride = lambda t: t.stride(0) if T > 1 else n
    _C.check(_C.load().b200_gate_prep(q32.data_ptr(), f32.data_ptr(), q.data_ptr(), stride(q), f.data_ptr(), stride(f),
                                      _ptr(bias), _ptr(lower), T, n, _dt3(q), _stream()), "b200_gate_prep")
    return q32, f32


def mixed_attn(q, k, v, spans: StepSpans, scale, num_kv_heads, vdim, block_tables=None, window=0, slopes=None,
               talk=None, sink=None):
    """Causal softmax attention whose heads are mixed BEFORE the softmax. Shapes, paging, spans and the window as in
    attn_generic. slopes fp32 [H]: s_h(i, j) = scale q.k - slopes[h] (i - j); talk fp32 [H, H]: s'_h = sum_g
    talk[h, g] s_g; sink fp32 [H]: exp(sink[h]) joins the softmax denominator (no key, no value). Each may be None."""
    _need_cuda(q, k, v, block_tables, slopes, talk, sink)
    _f32(slopes, talk, sink)
    T, H, dim = q.shape
    if q.stride(2) != 1 or q.stride(1) != dim:
        raise ValueError("q must be contiguous in (heads, dim)")
    G = num_kv_heads
    if (talk is not None and talk.shape != (H, H)) or any(t is not None and t.numel() != H for t in (slopes, sink)):
        raise ValueError("talk [H, H]; slopes, sink [H]")
    if block_tables is not None:
        if block_tables.dtype != torch.int32 or block_tables.stride(1) != 1:
            raise TypeError("block_tables must be row-major int32")
        _, bs = _cache_dims(k, G * dim)
        _cache_dims(v, G * vdim)
        ks, vs, bt_ptr, bt_stride = G * dim, G * vdim, block_tables.data_ptr(), block_tables.stride(0)
    else:
        if k.stride(2) != 1 or k.stride(1) != dim or v.stride(2) != 1 or v.stride(1) != vdim:
            raise ValueError("k/v must be contiguous in (heads, dim)")
        bs, bt_ptr, bt_stride = 0, None, 0
        ks = k.stride(0) if k.shape[0] > 1 else G * dim
        vs = v.stride(0) if v.shape[0] > 1 else G * vdim
    out = torch.empty(T, H * vdim, dtype=q.dtype, device=q.device)
    cu_q, cu_k, ctx = spans.ptrs()
    _C.check(_C.load().b200_mixed_attn(out.data_ptr(), q.data_ptr(), q.stride(0) if T > 1 else H * dim, k.data_ptr(),
                                       ks, v.data_ptr(), vs, bt_ptr, bt_stride, bs, cu_q, cu_k, ctx, spans.num_seqs,
                                       spans.max_q, H, G, dim, vdim, float(scale), int(window), _ptr(slopes),
                                       _ptr(talk), _ptr(sink), _dt3(q), _stream()), "b200_mixed_attn")
    return out


def attn_generic(q, k, v, spans: StepSpans, scale, num_kv_heads, vdim, block_tables=None, window=0, softcap=0.0,
                 sink=None, gate=None):
    """Causal softmax attention for any head sizes and dtypes. q [T, H, dim]; packed mode: k [Tk, G, dim],
    v [Tk, G, vdim] (token-strided views allowed) in the order of spans.cu_k; paged mode (block_tables given):
    k, v are the caches [nb, bs, G*dim], [nb, bs, G*vdim]. Returns [T, H*vdim]. window > 0: position i sees the
    keys j with 0 <= i - j < window. v None: the values are the first vdim columns of the key rows. softcap > 0:
    scores become softcap * tanh(score / softcap). sink fp32 [H]: exp(sink[h]) joins the softmax denominator (no key,
    no value). gate [T, H] (q's dtype, row-strided view allowed): head h of token t is multiplied by sigmoid(gate[t, h])."""
    _need_cuda(q, k, v, block_tables, sink, gate)
    _f32(sink)
    T, H, dim = q.shape
    if sink is not None and sink.numel() != H:
        raise ValueError("sink [H]")
    if gate is not None and (gate.shape != (T, H) or gate.stride(1) != 1 or gate.dtype != q.dtype):
        raise ValueError("gate [T, H] of q's dtype with unit inner stride")
    if q.stride(2) != 1 or q.stride(1) != dim:
        raise ValueError("q must be contiguous in (heads, dim)")
    G = num_kv_heads
    if block_tables is not None:
        if block_tables.dtype != torch.int32 or block_tables.stride(1) != 1:
            raise TypeError("block_tables must be row-major int32")
        _, bs = _cache_dims(k, G * dim)
        if v is not None:
            _cache_dims(v, G * vdim)
        ks, vs, bt_ptr, bt_stride = G * dim, G * vdim, block_tables.data_ptr(), block_tables.stride(0)
    else:
        if k.stride(2) != 1 or k.stride(1) != dim or (v is not None and (v.stride(2) != 1 or v.stride(1) != vdim)):
            raise ValueError("k/v must be contiguous in (heads, dim)")
        bs, bt_ptr, bt_stride = 0, None, 0
        ks = k.stride(0) if k.shape[0] > 1 else G * dim
        vs = (v.stride(0) if v.shape[0] > 1 else G * vdim) if v is not None else 0
    if v is None and (G != 1 and vdim != dim or vdim > dim):
        raise ValueError("values inside the key rows: one kv head with vdim <= dim, or vdim == dim")
    out = torch.empty(T, H * vdim, dtype=q.dtype, device=q.device)
    cu_q, cu_k, ctx = spans.ptrs()
    _C.check(_C.load().b200_attn_generic(out.data_ptr(), q.data_ptr(), q.stride(0) if T > 1 else H * dim,
                                         k.data_ptr(), ks, _ptr(v), vs, bt_ptr, bt_stride, bs, cu_q, cu_k, ctx,
                                         spans.num_seqs, spans.max_q, H, G, dim, vdim, float(scale), int(window),
                                         float(softcap), _ptr(sink), _ptr(gate),
                                         (gate.stride(0) if T > 1 else H) if gate is not None else 0, _dt3(q),
                                         _stream()), "b200_attn_generic")
    return out


def linear_recurrence(q, k, v, spans: StepSpans, num_heads, groups, kdim, vdim, state=None, state_slots=None,
                      decay=None, act_silu=False, dt=None, dt_bias=None, a_log=None, d_skip=None, tied_gate=False):
    """Per head S_t = a_t S_(t-1) + k_t (b_t v_t)^T, o_t = S_t^T q_t, S fp32 [kdim, vdim] carried in
    state[slot] ([slots, H, kdim, vdim] fp32) between steps. q, k [T, groups*kdim] (head h reads group
    h // (H / groups)), v [T, H*vdim]; row-strided views allowed. Returns fp32 [T, H*vdim].
      decay given (fp32 [H]): a_t = decay_h, b_t = 1; act_silu applies silu to q, k, v as they are read.
      dt given ([T, H]):      step = softplus(dt + dt_bias_h), a_t = exp(-exp(a_log_h) * step), b_t = step, and
                              o_t += d_skip_h * v_t.
      tied_gate:              k holds a forget gate f per key channel (fp32, like q) that also decides what is written:
                              S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T."""
    _need_cuda(q, k, v, state, state_slots, decay, dt, dt_bias, a_log, d_skip)
    _f32(decay, dt_bias, a_log, d_skip, state)
    T = q.shape[0]
    qk_f32 = q.dtype == torch.float32 and v.dtype != torch.float32     # q, k rotated or normalised in fp32 upstream
    for t, n in ((q, groups * kdim), (k, groups * kdim), (v, num_heads * vdim)):
        if t.dim() != 2 or t.shape[1] != n or t.stride(1) != 1 or (t.dtype != q.dtype and not (qk_f32 and t is v)):
            raise ValueError("q, k [T, groups*kdim] and v [T, H*vdim] with unit inner stride, one dtype")
    if tied_gate and (q.dtype != torch.float32 or decay is not None or dt is not None or act_silu):
        raise ValueError("tied-gate form: fp32 q and gate, no decay, dt or activation")
    if qk_f32 and not tied_gate and (decay is None or act_silu):
        raise ValueError("fp32 q/k beside 16-bit v: constant-decay or tied-gate form without activation only")
    if state is not None and tuple(state.shape[1:]) != (num_heads, kdim, vdim):
        raise ValueError(f"state must be [slots, {num_heads}, {kdim}, {vdim}]")
    if state is not None and (state_slots is None or state_slots.dtype != torch.int32):
        raise TypeError("state_slots must be int32")
    mode = 2 if tied_gate else 0 if decay is not None else 1
    if mode == 1 and (dt is None or dt.shape != (T, num_heads) or dt.stride(1) != 1 or dt.dtype != q.dtype):
        raise ValueError("dt must be [T, H] of q's dtype")
    out = torch.empty(T, num_heads * vdim, dtype=torch.float32, device=q.device)
    cu_q, cu_k, ctx = spans.ptrs()
    stride = lambda t: t.stride(0) if T > 1 else t.shape[1]
    _C.check(_C.load().b200_linear_recurrence(
        out.data_ptr(), q.data_ptr(), stride(q), k.data_ptr(), stride(k), v.data_ptr(), stride(v), _ptr(state),
        _ptr(state_slots), cu_q, cu_k, ctx, spans.num_seqs, spans.max_q, num_heads, groups, kdim, vdim, mode,
        1 if act_silu else 0, _ptr(decay), _ptr(dt), stride(dt) if dt is not None else 0, _ptr(dt_bias),
        _ptr(a_log), _ptr(d_skip), 1 if qk_f32 else 0, _dt3(v), _stream()), "b200_linear_recurrence")
    return out


# ---------------------------------------------------------------------------------------------------
# Multi-stream residuals, rotary positions, delta rule, latent attention, clamped gated unit (csrc/stream_ops.cu,
# csrc/delta_rule.cu) and the generic mixture-of-experts kernels (csrc/moe_generic.cu).
def stream_mix_norm_(x, y, mix, out_w, in_w, w, b, eps, dtype, kind="layer", offset=0.0, sum_out=False):
    """x fp32 [rows, S, hidden] (in place). With y [rows, hidden]: every stream t becomes sum_s mix[s, t] x_s +
    out_w[t] y. Then u = sum_t in_w[t] x_t (in_w None: the plain sum) and h = norm(u) in `dtype` when w is given:
    kind "layer" (u - mean) / sqrt(var + eps) * w + b, kind "rms" u / sqrt(mean u^2 + eps) * (offset + w).
    Returns h (or None), and u as fp32 too when sum_out."""
    _need_cuda(x, y, mix, out_w, in_w, w, b)
    _f32(x, mix, out_w, in_w, w, b)
    rows, S, hidden = x.shape
    if y is not None and (not y.is_contiguous() or y.shape != (rows, hidden) or y.dtype != dtype):
        raise ValueError("y must be a contiguous [rows, hidden] tensor of the model dtype")
    h = torch.empty(rows, hidden, dtype=dtype, device=x.device) if w is not None else None
    u = torch.empty(rows, hidden, dtype=torch.float32, device=x.device) if sum_out else None
    _C.check(_C.load().b200_stream_mix_norm(_ptr(h), x.data_ptr(), _ptr(y), _ptr(mix), _ptr(out_w), _ptr(in_w),
                                            _ptr(w), _ptr(b), _ptr(u), float(eps), float(offset),
                                            {"layer": 0, "rms": 1}[kind], rows, S, hidden, _DT3[dtype], _stream()),
             "b200_stream_mix_norm")
    return (h, u) if sum_out else h


def rotary_heads(x, positions, heads, width, dims, base, interleaved, out=None, out_f32=False, split=0,
                 scale_lo=1.0, scale_hi=1.0):
    """x [T, heads, width] (a strided view: unit inner stride, any head and token strides). The first `dims` columns
    of every head are rotated by pos * base^(-2i/dims) in pairs (2i, 2i+1) (interleaved) or (i, i + dims/2); heads
    below `split` are then multiplied by scale_lo, the others by scale_hi. out: a view of the same shape (fp32 when
    out_f32, else x's dtype); by default a new contiguous tensor."""
    _need_cuda(x, positions, out)
    T = x.shape[0]
    if x.dim() != 3 or x.shape[1:] != (heads, width) or x.stride(2) != 1:
        raise ValueError("x must be [T, heads, width] with unit inner stride")
    if positions.dtype != torch.int64 or not positions.is_contiguous():
        raise TypeError("positions must be contiguous int64")
    if out is None:
        out = torch.empty(T, heads, width, dtype=torch.float32 if out_f32 else x.dtype, device=x.device)
    if out.shape != x.shape or out.stride(2) != 1 or out.dtype != (torch.float32 if out_f32 else x.dtype):
        raise ValueError("out must be shaped like x, unit inner stride, fp32 or x's dtype")
    _C.check(_C.load().b200_rotary_heads(out.data_ptr(), out.stride(0) if T > 1 else 0, out.stride(1),
                                         1 if out_f32 else 0, x.data_ptr(), x.stride(0) if T > 1 else 0, x.stride(1),
                                         positions.data_ptr(), T, heads, width, int(dims), float(base),
                                         1 if interleaved else 0, int(split), float(scale_lo), float(scale_hi),
                                         _dt3(x), _stream()), "b200_rotary_heads")
    return out


def delta_prep(qk, a, b, dt_bias, a_log, num_heads, groups, dim, unit_eps, q_scale):
    """qk [T, 2*groups*dim] (q heads then k heads), a [T, H*dim], b [T, H] (row-strided views allowed) ->
    (qk fp32 unit vectors with q scaled, decay fp32 [T, H*dim], beta fp32 [T, H])."""
    _need_cuda(qk, a, b, dt_bias, a_log)
    _f32(dt_bias, a_log)
    T = qk.shape[0]
    if qk.shape[1] != 2 * groups * dim or a.shape != (T, num_heads * dim) or b.shape != (T, num_heads):
        raise ValueError("delta_prep shapes")
    if qk.stride(1) != 1 or a.stride(1) != 1 or b.stride(1) != 1 or a.dtype != qk.dtype or b.dtype != qk.dtype:
        raise ValueError("delta_prep inputs: unit inner stride, one dtype")
    dev = qk.device
    qk32 = torch.empty(T, 2 * groups * dim, dtype=torch.float32, device=dev)
    decay = torch.empty(T, num_heads * dim, dtype=torch.float32, device=dev)
    beta = torch.empty(T, num_heads, dtype=torch.float32, device=dev)
    stride = lambda t: t.stride(0) if T > 1 else t.shape[1]
    _C.check(_C.load().b200_delta_prep(qk32.data_ptr(), decay.data_ptr(), beta.data_ptr(), qk.data_ptr(), stride(qk),
                                       a.data_ptr(), stride(a), b.data_ptr(), stride(b), dt_bias.data_ptr(),
                                       a_log.data_ptr(), T, num_heads, groups, dim, float(unit_eps), float(q_scale),
                                       _dt3(qk), _stream()), "b200_delta_prep")
    return qk32, decay, beta


def delta_rule(q, k, v, g, beta, spans: StepSpans, num_heads, groups, kdim, vdim, state=None, state_slots=None):
    """Gated delta rule per head (S fp32 [kdim, vdim], carried in state[slot]): S <- diag(g) S; w = beta (v - S^T k);
    S <- S + k w^T; o = S^T q. q, k fp32 [T, groups*kdim] (row-strided views allowed), g fp32 [T, H*kdim], beta fp32
    [T, H], v [T, H*vdim] in the model dtype. Returns fp32 [T, H*vdim]."""
    _need_cuda(q, k, v, g, beta, state, state_slots)
    _f32(g, beta, state)
    T = q.shape[0]
    for t, n in ((q, groups * kdim), (k, groups * kdim)):
        if t.dtype != torch.float32 or t.shape != (T, n) or t.stride(1) != 1:
            raise ValueError("q, k fp32 [T, groups*kdim] with unit inner stride")
    if v.shape != (T, num_heads * vdim) or v.stride(1) != 1 or g.shape != (T, num_heads * kdim) or \
            beta.shape != (T, num_heads):
        raise ValueError("delta_rule shapes")
    if state is not None and tuple(state.shape[1:]) != (num_heads, kdim, vdim):
        raise ValueError(f"state must be [slots, {num_heads}, {kdim}, {vdim}]")
    if state is not None and (state_slots is None or state_slots.dtype != torch.int32):
        raise TypeError("state_slots must be int32")
    out = torch.empty(T, num_heads * vdim, dtype=torch.float32, device=q.device)
    cu_q, cu_k, ctx = spans.ptrs()
    stride = lambda t: t.stride(0) if T > 1 else t.shape[1]
    _C.check(_C.load().b200_delta_rule(out.data_ptr(), q.data_ptr(), stride(q), k.data_ptr(), stride(k), v.data_ptr(),
                                       stride(v), g.data_ptr(), beta.data_ptr(), _ptr(state), _ptr(state_slots),
                                       cu_q, cu_k, ctx, spans.num_seqs, num_heads, groups, kdim, vdim, _dt3(v),
                                       _stream()), "b200_delta_rule")
    return out


def latent_kv_prep(dq, dkv, wq, wc, positions, rank, rot, dims, base, interleaved, eps, cache=None, slots=None):
    """dq [T, q_rank], dkv [T, rank + rot] (row-strided views) -> (cq [T, q_rank] = rms(dq) * wq, kc [T, rank + rot] =
    [rms(dkv[:, :rank]) * wc | rotary(dkv[:, rank:])]); kc rows are also stored at `slots` of the paged cache
    [nb, bs, rank + rot] when given."""
    _need_cuda(dq, dkv, wq, wc, positions, cache, slots)
    _f32(wq, wc)
    T, q_rank = dq.shape
    if dkv.shape != (T, rank + rot) or dq.stride(1) != 1 or dkv.stride(1) != 1 or dq.dtype != dkv.dtype:
        raise ValueError("latent_kv_prep shapes")
    if positions.dtype != torch.int64 or not positions.is_contiguous():
        raise TypeError("positions must be contiguous int64")
    have = cache is not None and cache.numel() > 0 and slots is not None
    bs = 0
    if have:
        _, bs = _cache_dims(cache, rank + rot)
        if slots.dtype != torch.int32 or not slots.is_contiguous() or cache.dtype != dq.dtype:
            raise TypeError("slots contiguous int32; cache of the activations' dtype")
    cq = torch.empty(T, q_rank, dtype=dq.dtype, device=dq.device)
    kc = torch.empty(T, rank + rot, dtype=dq.dtype, device=dq.device)
    stride = lambda t: t.stride(0) if T > 1 else t.shape[1]
    _C.check(_C.load().b200_latent_kv_prep(cq.data_ptr(), kc.data_ptr(), cache.data_ptr() if have else None,
                                           slots.data_ptr() if have else None,
                                           1 if (have and slots.dim() == 2) else 0, bs, dq.data_ptr(), stride(dq),
                                           dkv.data_ptr(), stride(dkv), wq.data_ptr(), wc.data_ptr(),
                                           positions.data_ptr(), T, q_rank, rank, rot, int(dims), float(base),
                                           1 if interleaved else 0, float(eps), _dt3(dq), _stream()),
             "b200_latent_kv_prep")
    return cq, kc


def masked_softmax(scores, heads, first_pos, key_lo, scale, window, dtype, ctx_lens=None, chunks=None):
    """scores fp32 [rows, nk] of `heads` query heads per token -> softmax(scale * scores) over the visible keys in
    `dtype`, hidden keys 0. Without ctx_lens / chunks the rows are consecutive tokens of one sequence (row r at position
    first_pos + r // heads, column j the key at position key_lo + j); with ctx_lens (int32 per sequence) row r is the
    one token of sequence r // heads at position ctx_lens - 1 and column j the key at position pos - nk + 1 + j; with
    chunks = (first int32 [C], lo int32 [C], rows_per_chunk) chunk c holds consecutive tokens from position first[c]
    on against keys from position lo[c] on. A key is visible iff it exists, is not ahead of the token and lies inside
    the window (0: no window)."""
    _need_cuda(scores, ctx_lens)
    if scores.dtype != torch.float32 or not scores.is_contiguous() or scores.dim() != 2:
        raise TypeError("scores are a contiguous fp32 matrix")
    if ctx_lens is not None and (ctx_lens.dtype != torch.int32 or not ctx_lens.is_contiguous()):
        raise TypeError("ctx_lens must be contiguous int32")
    rows, nk = scores.shape
    cf = cl = None
    per = 0
    if chunks is not None:
        cf, cl, per = chunks
        _need_cuda(cf, cl)
        if cf.dtype != torch.int32 or cl.dtype != torch.int32 or cf.numel() * per != rows or cl.numel() != cf.numel():
            raise TypeError("chunks: int32 first / lo per chunk, rows_per_chunk * chunks == rows")
    p = torch.empty(rows, nk, dtype=dtype, device=scores.device)
    _C.check(_C.load().b200_masked_softmax(p.data_ptr(), scores.data_ptr(), rows, nk, int(heads), int(first_pos),
                                           int(key_lo), int(window), float(scale), _ptr(ctx_lens), _ptr(cf), _ptr(cl),
                                           int(per), _DT3[dtype], _stream()), "b200_masked_softmax")
    return p


def gather_rows_by_head(src, slots, entries, nk):
    """src [rows, G, size] (a cache viewed per head, or a row-strided view of packed rows); slots int64 [entries * nk] ->
    [entries, G, nk, size] with out[n, g, j] = src[slots[n * nk + j], g]: rows picked by slot and regrouped per kv head,
    the operand layout of a batched product per head. 16-byte copies where head size and row stride allow them, else
    torch indexing."""
    _need_cuda(src, slots)
    rows, G, size = src.shape
    if slots.dtype != torch.int64 or not slots.is_contiguous() or slots.numel() != entries * nk:
        raise TypeError("slots are contiguous int64 [entries * nk]")
    item = src.element_size()
    if (src.stride(2) != 1 or src.stride(1) != size or (size * item) % 16 or (src.stride(0) * item) % 16 or
            src.data_ptr() % 16):
        return src[slots].view(entries, nk, G, size).permute(0, 2, 1, 3).contiguous()
    out = torch.empty(entries, G, nk, size, dtype=src.dtype, device=src.device)
    _C.check(_C.load().b200_gather_rows_by_head(out.data_ptr(), src.data_ptr(), src.stride(0) * item, slots.data_ptr(),
                                                entries, nk, G, size * item, _stream()), "b200_gather_rows_by_head")
    return out


MIXED_SOFTMAX_SMEM = 200 * 1024      # a token's heads x visible keys block (+ the mixing matrix) lives in shared memory


def mixed_softmax(scores, scale, window, dtype, slopes=None, talk=None, sink=None, ctx_lens=None, chunks=None):
    """scores fp32 [entries, G, C, rep, nk] (raw dot products; entry = a chunk of a prompt or a sequence of a decode step,
    C tokens per entry, head g * rep + r) -> probabilities of the same shape in `dtype` for heads that are mixed before the
    softmax: x_h = scale s_h - slopes[h] (pos - key), x'_h = sum_g talk[h, g] x_g, softmax over the visible keys with
    exp(sink[h]) in the denominator. chunks = (first int32 [entries], lo int32 [entries]): token c of entry b sits at
    position first[b] + c, column j is the key at position lo[b] + j; ctx_lens int32 [entries] (C == 1): the token sits at
    ctx_lens - 1 and the columns are the last nk positions. Visibility as in masked_softmax."""
    _need_cuda(scores, slopes, talk, sink, ctx_lens)
    _f32(slopes, talk, sink)
    if scores.dtype != torch.float32 or not scores.is_contiguous() or scores.dim() != 5:
        raise TypeError("scores are a contiguous fp32 [entries, G, C, rep, nk] tensor")
    B, G, C, rep, nk = scores.shape
    cf = cl = None
    if chunks is not None:
        cf, cl = chunks
        _need_cuda(cf, cl)
        if cf.dtype != torch.int32 or cl.dtype != torch.int32 or cf.numel() != B or cl.numel() != B:
            raise TypeError("chunks: int32 first / lo per entry")
    elif ctx_lens is None or ctx_lens.dtype != torch.int32 or not ctx_lens.is_contiguous() or ctx_lens.numel() != B or C != 1:
        raise TypeError("give chunks, or contiguous int32 ctx_lens [entries] with one token per entry")
    p = torch.empty(scores.shape, dtype=dtype, device=scores.device)
    _C.check(_C.load().b200_mixed_softmax(p.data_ptr(), scores.data_ptr(), B, C, G, rep, nk, float(scale), int(window),
                                          _ptr(slopes), _ptr(talk), _ptr(sink), _ptr(ctx_lens), _ptr(cf), _ptr(cl),
                                          _DT3[dtype], _stream()), "b200_mixed_softmax")
    return p


def glu_clamped(x, alpha, limit):
    """x [rows, 2*inter] = (gate | up) -> g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, +-limit)."""
    _need_cuda(x)
    if not x.is_contiguous() or x.dim() != 2:
        raise ValueError("glu_clamped input must be a contiguous matrix")
    rows, inter = x.shape[0], x.shape[1] // 2
    out = torch.empty(rows, inter, dtype=x.dtype, device=x.device)
    _C.check(_C.load().b200_glu_clamped(out.data_ptr(), x.data_ptr(), rows, inter, float(alpha), float(limit),
                                        _dt3(x), _stream()), "b200_glu_clamped")
    return out


def moe_route_grouped(router_logits, bias, top_k, groups=1, keep=1, scale=1.0):
    """Sigmoid router with a selection bias and group-limited choice. router_logits fp32 [T, E]; bias fp32 [E] or
    None -> (topk_ids int32 [T, k], topk_weights fp32 [T, k])."""
    _need_cuda(router_logits, bias)
    _f32(bias)
    if router_logits.dtype != torch.float32 or router_logits.stride(1) != 1:
        raise TypeError("router logits are fp32 with unit inner stride")
    T, E = router_logits.shape
    ids = torch.empty(T, top_k, dtype=torch.int32, device=router_logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=router_logits.device)
    _C.check(_C.load().b200_moe_route_grouped(ids.data_ptr(), w.data_ptr(), router_logits.data_ptr(),
                                              router_logits.stride(0) if T > 1 else E, _ptr(bias), T, E, int(top_k),
                                              int(groups), int(keep), float(scale), _stream()),
             "b200_moe_route_grouped")
    return ids, w


def moe_route_grouped_softmax(router_logits, top_k, groups=1, keep=1, scale=1.0):
    """Softmax router with group-limited choice. router_logits fp32 [T, E]: s = softmax over all experts; a group of
    neighbours scores its largest s, only the `keep` best of the `groups` groups stay in play; the top_k s are taken
    (ties to the lower index) -> (topk_ids int32 [T, k], topk_weights fp32 [T, k] = s / (sum s + 1e-20) * scale)."""
    _need_cuda(router_logits)
    if router_logits.dtype != torch.float32 or router_logits.stride(1) != 1:
        raise TypeError("router logits are fp32 with unit inner stride")
    T, E = router_logits.shape
    ids = torch.empty(T, top_k, dtype=torch.int32, device=router_logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=router_logits.device)
    _C.check(_C.load().b200_moe_route_grouped_softmax(ids.data_ptr(), w.data_ptr(), router_logits.data_ptr(),
                                                      router_logits.stride(0) if T > 1 else E, T, E, int(top_k),
                                                      int(groups), int(keep), float(scale), _stream()),
             "b200_moe_route_grouped_softmax")
    return ids, w


def moe_route_topk(router_logits, bias, top_k):
    """The top_k largest of router_logits + bias (fp32 [T, E]; bias fp32 [E] or None), weighted by the softmax over
    the chosen logits only -> (topk_ids int32 [T, k], topk_weights fp32 [T, k]). Ties go to the lower index."""
    _need_cuda(router_logits, bias)
    _f32(bias)
    if router_logits.dtype != torch.float32 or router_logits.stride(1) != 1:
        raise TypeError("router logits are fp32 with unit inner stride")
    T, E = router_logits.shape
    ids = torch.empty(T, top_k, dtype=torch.int32, device=router_logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=router_logits.device)
    _C.check(_C.load().b200_moe_route_topk(ids.data_ptr(), w.data_ptr(), router_logits.data_ptr(),
                                           router_logits.stride(0) if T > 1 else E, _ptr(bias), T, E, int(top_k),
                                           _stream()), "b200_moe_route_topk")
    return ids, w


def moe_experts_generic(x, w13, w2, topk_weights, plan: MoePlan, act=None, glu=None) -> torch.Tensor:
    """Expert MLPs and the weighted combine for any sizes and dtypes (fp32 included): x [T, hidden]; w2 [E, hidden,
    inter]; topk_weights fp32 [T, k]. act None: gated experts down(silu(gate x) * up x) with w13 [E, 2*inter, hidden]
    (glu = (alpha, limit): the clamped unit g sigmoid(alpha g) (u + 1) of glu_clamped in place of silu(g) u);
    act "silu" | "relu" | "gelu_tanh" | "relu2": experts without a gate, down(act(up x)) with w13 [E, inter, hidden]."""
    _need_cuda(x, w13, w2, topk_weights)
    _f32(topk_weights)
    T, hidden = x.shape
    E, two_i, _ = w13.shape
    inter, k = (two_i // 2 if act is None else two_i), plan.top_k
    if w13.shape != (E, two_i, hidden) or w2.shape != (E, hidden, inter) or E != plan.num_local:
        raise ValueError("expert weight shapes do not match")
    if not (w13.is_contiguous() and w2.is_contiguous()) or x.stride(1) != 1 or x.dtype != w13.dtype or x.dtype != w2.dtype:
        raise ValueError("contiguous expert weights of x's dtype; x row-major")
    pairs = T * k
    lib = _C.load()
    h = torch.empty(pairs, inter, dtype=x.dtype, device=x.device)
    y = torch.empty(pairs, hidden, dtype=torch.float32, device=x.device)
    out = torch.empty(T, hidden, dtype=x.dtype, device=x.device)
    _C.check(lib.b200_moe_gemm_generic(h.data_ptr(), x.data_ptr(), x.stride(0) if T > 1 else hidden, w13.data_ptr(),
                                       plan.offsets.data_ptr(), plan.sorted_pair.data_ptr(), pairs, hidden, inter, E,
                                       k, 1 if act is None else 2 + _PLAIN_ACTS[act], float(glu[0]) if glu else 0.0,
                                       float(glu[1]) if glu else 0.0, _dt3(x), _stream()),
             "b200_moe_gemm_generic (up)")
    _C.check(lib.b200_moe_gemm_generic(y.data_ptr(), h.data_ptr(), inter, w2.data_ptr(), plan.offsets.data_ptr(),
                                       plan.sorted_pair.data_ptr(), pairs, inter, hidden, E, k, 0, 0.0, 0.0, _dt3(x),
                                       _stream()), "b200_moe_gemm_generic (down)")
    _C.check(lib.b200_moe_combine_weighted(out.data_ptr(), y.data_ptr(), topk_weights.data_ptr(),
                                           plan.pos_of_pair.data_ptr(), T, k, hidden, _dt3(x), _stream()),
             "b200_moe_combine_weighted")
    return out


# ---------------------------------------------------------------------------------------------------
# Scaled residual with a grouped norm, rotary positions from a frequency table fused with value blending and the K/V
# scatter, and the per-head output gate (csrc/seq_ops.cu).
def residual_scale_groupnorm_(residual, y, scale, c, w, eps, groups, dtype, offset=0.0, accumulate=True, y_index=None):
    """residual (fp32 [rows, hidden], in place) <- (residual if accumulate else 0) + c * scale * y, with scale fp32
    [hidden] or None and y [rows, hidden] in `dtype` (or, with y_index int64 [rows], a table whose rows are looked up:
    the scaled token embedding); y None leaves the residual as it is. Returns h = the residual's RMS norm over each of
    `groups` equal consecutive parts times (offset + w) in `dtype`, or None when w is None."""
    _need_cuda(residual, y, scale, w, y_index)
    _f32(residual, scale, w)
    rows, hidden = residual.shape
    if y is not None:
        if not y.is_contiguous() or y.shape[-1] != hidden or y.dtype != dtype or (y_index is None and y.shape[0] != rows):
            raise ValueError("y: contiguous [rows or table, hidden] of the model dtype")
        if y_index is not None and (y_index.dtype != torch.int64 or not y_index.is_contiguous() or y_index.numel() != rows):
            raise TypeError("row indices are contiguous int64 [rows]")
    if hidden % groups:
        raise ValueError("the row does not split into equal groups")
    h = torch.empty(rows, hidden, dtype=dtype, device=residual.device) if w is not None else None
    _C.check(_C.load().b200_residual_scale_groupnorm(_ptr(h), residual.data_ptr(), _ptr(y), _ptr(y_index),
                                                     y.shape[0] if y is not None else 0, _ptr(scale), float(c),
                                                     1 if accumulate else 0, _ptr(w), float(offset), float(eps), rows,
                                                     hidden, int(groups), _DT3[dtype], _stream()),
             "b200_residual_scale_groupnorm")
    return h


def rotary_table(positions, freq, magnitude=1.0):
    """positions int64 [T], freq fp64 [half] -> fp32 [T, half, 2] = (cos, sin)(position * freq) * magnitude, angles fp64."""
    _need_cuda(positions, freq)
    if positions.dtype != torch.int64 or not positions.is_contiguous():
        raise TypeError("positions must be contiguous int64")
    if freq.dtype != torch.float64 or not freq.is_contiguous():
        raise TypeError("frequencies are a contiguous fp64 vector")
    T, half = positions.numel(), freq.numel()
    table = torch.empty(T, half, 2, dtype=torch.float32, device=positions.device)
    _C.check(_C.load().b200_rotary_table(table.data_ptr(), positions.data_ptr(), freq.data_ptr(), float(magnitude), T,
                                         half, _stream()), "b200_rotary_table")
    return table


def rope_mix_cache(qkv, table, num_heads, num_kv_heads, dim, vdim, dims, interleaved=True, v_other=None, lam=None,
                   k_cache=None, v_cache=None, slots=None):
    """In place on qkv [T, H*dim | G*dim | G*vdim]: the first `dims` columns of every q and k head are rotated by
    table [T, dims/2, 2] (rotary_table) in pairs (2i, 2i+1) (interleaved) or (i, i + dims/2); with v_other [T, G*vdim]
    (row-strided view allowed) and lam (fp32 scalar tensor) every value row becomes (1 - lam) v + lam v_other; k and v
    rows are stored at `slots` of the paged caches [nb, bs, G*dim] / [nb, bs, G*vdim] when those are given."""
    _need_cuda(qkv, table, v_other, lam, k_cache, v_cache, slots)
    _f32(lam)
    T = qkv.shape[0]
    if qkv.dim() != 2 or qkv.stride(1) != 1 or qkv.shape[1] != num_heads * dim + num_kv_heads * (dim + vdim):
        raise ValueError("qkv must be [T, H*dim + G*dim + G*vdim] with unit inner stride")
    if dims and (table is None or table.dtype != torch.float32 or not table.is_contiguous() or
                 table.shape != (T, dims // 2, 2)):
        raise ValueError("table: contiguous fp32 [T, dims/2, 2]")
    if v_other is not None and (v_other.shape != (T, num_kv_heads * vdim) or v_other.stride(1) != 1 or
                                v_other.dtype != qkv.dtype or lam is None or lam.numel() != 1):
        raise ValueError("v_other [T, G*vdim] of qkv's dtype with unit inner stride, and a scalar lam")
    have = k_cache is not None and k_cache.numel() > 0
    bs = 0
    if have:
        _, bs = _cache_dims(k_cache, num_kv_heads * dim)
        _cache_dims(v_cache, num_kv_heads * vdim)
        if slots.dtype != torch.int32 or not slots.is_contiguous():
            raise TypeError("slots must be contiguous int32")
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
            raise TypeError("caches must have the activations' dtype")
    _C.check(_C.load().b200_rope_mix_cache(
        qkv.data_ptr(), qkv.stride(0) if T > 1 else qkv.shape[1], _ptr(table), int(dims), 1 if interleaved else 0,
        _ptr(v_other), (v_other.stride(0) if T > 1 else v_other.shape[1]) if v_other is not None else 0, _ptr(lam),
        k_cache.data_ptr() if have else None, v_cache.data_ptr() if have else None, slots.data_ptr() if have else None,
        1 if (have and slots.dim() == 2) else 0, bs, T, num_heads, num_kv_heads, dim, vdim, _dt3(qkv), _stream()),
        "b200_rope_mix_cache")
    return qkv


def head_gate_(x, gate, num_heads):
    """x [T, H*vdim] (contiguous, in place) times sigmoid(gate [T, H]) per head; gate may be a row-strided view."""
    _need_cuda(x, gate)
    T, n = x.shape
    if not x.is_contiguous() or n % num_heads or gate.shape != (T, num_heads) or gate.stride(1) != 1 or gate.dtype != x.dtype:
        raise ValueError("x contiguous [T, H*vdim]; gate [T, H] of x's dtype with unit inner stride")
    _C.check(_C.load().b200_head_gate(x.data_ptr(), x.data_ptr(), gate.data_ptr(), gate.stride(0) if T > 1 else num_heads,
                                      T, num_heads, n // num_heads, _dt3(x), _stream()), "b200_head_gate")
    return x
