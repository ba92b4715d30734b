"""Plain, slow restatement of the Fitevik decoder for the tests: one function per mechanism, token by token where
the mechanism is a recurrence, query by query where it is attention, float64 on the CPU. It shares no code with the
package.

Notation: ``u`` is a sublayer's input [T, width]; weights are stored [out, in] and applied as ``u @ W.T``.
A model is (config dict, {tensor name: float64 tensor}) with the checkpoint's names (``l<i>.mix.q`` ...).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- small pieces
def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = (x - mu).pow(2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def silu(x):
    return x * torch.sigmoid(x)


def relu_squared(x):
    return torch.clamp(x, min=0.0) ** 2


def head_slopes(H):
    return [2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]


# ----------------------------------------------------------------------------- the two mixers
def forget_gate(u, w_f, b_f, lower):
    """f = l + (1 - l) sigmoid(W_f u + b): never below the learned lower bound l."""
    return lower + (1.0 - lower) * torch.sigmoid(u @ w_f.T + b_f)


def hgrn2_states(q, f, v, S0=None):
    """q, f [T, H, d], v [T, H, dv]. Per head S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t.
    Returns (o [T, H, dv], the last state [H, d, dv])."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=q.dtype) if S0 is None else S0.clone()
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        for h in range(H):
            S[h] = f[t, h][:, None] * S[h] + (1.0 - f[t, h])[:, None] * v[t, h][None, :]
            out[t, h] = S[h].T @ q[t, h]
    return out, S


def hgrn2_mixer(u, m, w, eps):
    """w: the mixer's tensors by their short names (q, f, f.b, lower, v, norm, o)."""
    T = u.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(u @ w["q"].T).view(T, H, d)
    v = (u @ w["v"].T).view(T, H, dv)
    f = forget_gate(u, w["f"], w["f.b"], w["lower"]).view(T, H, d)
    o, _ = hgrn2_states(q, f, v)
    o = rms_norm(o, w["norm"], eps)                       # per head, one weight for all heads
    return o.reshape(T, H * dv) @ w["o"].T


def mixed_head_attention(q, k, v, scale, window, talk, sink, slopes, first_pos=0):
    """q [Tq, H, d] at positions first_pos .. ; k [Tk, G, d], v [Tk, G, dv] at positions 0 .. Tk - 1. Query by query,
    key by key: scores of all heads, minus the distance bias, mixed over the heads, then a softmax per head whose
    denominator also holds exp(sink_h)."""
    Tq, H, _ = q.shape
    G, dv = k.shape[1], v.shape[-1]
    rep = H // G
    out = torch.zeros(Tq, H, dv, dtype=q.dtype)
    for t in range(Tq):
        i = first_pos + t
        lo = max(0, i - window + 1) if window else 0
        keys = list(range(lo, i + 1))
        s = torch.zeros(H, len(keys), dtype=q.dtype)
        for h in range(H):
            for n, j in enumerate(keys):
                s[h, n] = float(q[t, h] @ k[j, h // rep]) * scale - (slopes[h] * (i - j) if slopes is not None else 0.0)
        if talk is not None:
            s = talk @ s
        for h in range(H):
            top = max(float(s[h].max()), float(sink[h]) if sink is not None else -math.inf)
            e = torch.exp(s[h] - top)
            den = e.sum() + (math.exp(float(sink[h]) - top) if sink is not None else 0.0)
            p = e / den
            for n, j in enumerate(keys):
                out[t, h] += p[n] * v[j, h // rep]
    return out


def attention_mixer(u, m, w, eps, kv=None):
    """w: q, q.norm, talk, sink, o and -- unless the layer borrows -- k, k.norm, v. kv: a lender's (k, v).
    Returns (output, (k, v)) so that a later layer can borrow them."""
    T = u.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(u @ w["q"].T, w["q.norm"], eps).view(T, H, d)         # over the whole projection, before the split
    if kv is None:
        k = rms_norm(u @ w["k"].T, w["k.norm"], eps).view(T, G, d)
        v = (u @ w["v"].T).view(T, G, dv)
    else:
        k, v = kv
    window = (m.get("mask") or {}).get("size", 0)
    o = mixed_head_attention(q, k, v, m["scale"], window, w["talk"], w["sink"], head_slopes(H))
    return o.reshape(T, H * dv) @ w["o"].T, (k, v)


# ----------------------------------------------------------------------------- feed-forwards
def dense_ff(u, w):
    return relu_squared(u @ w["up"].T + w["up.b"]) @ w["down"].T + w["down.b"]


def route(u, w_router, b_router, top):
    """(chosen experts [T, top], their weights [T, top]): the largest logits, softmax over the chosen only."""
    z = u @ w_router.T + b_router
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe_ff(u, mlp, w):
    idx, wt = route(u, w["router"], w["router.b"], mlp["router"]["top"])
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for c in range(idx.shape[1]):
            e = int(idx[t, c])
            out[t] += wt[t, c] * (relu_squared(u[t] @ w[f"e{e}.up"].T) @ w[f"e{e}.down"].T)
    return out


# ----------------------------------------------------------------------------- the model
def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and the residual stream after every layer)."""
    eps = cfg["norm"]["eps"]
    toks = torch.as_tensor(tokens, dtype=torch.long)
    T = toks.numel()
    x = tensors["embed"][toks] + tensors["pos"][:T]
    x = layer_norm(x, tensors["embed.norm"], tensors["embed.norm.b"], eps)
    lent, layers = {}, []
    for i, entry in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = entry["mixer"]
        if entry["type"] == "hgrn2":
            y = hgrn2_mixer(x, m, sub(tensors, p + "mix."), eps)
        else:
            src = m.get("kv_from")
            y, kv = attention_mixer(x, m, sub(tensors, p + "mix."), eps, lent[src] if src is not None else None)
            if src is None:
                lent[i] = kv
        x = x + layer_norm(y, tensors[p + "norm1"], tensors[p + "norm1.b"], eps)
        mlp = entry.get("mlp")
        if mlp:
            w = sub(tensors, p + "mlp.")
            y = dense_ff(x, w) if mlp["kind"] == "dense" else moe_ff(x, mlp, w)
            x = x + layer_norm(y, tensors[p + "norm2"], tensors[p + "norm2.b"], eps)
        layers.append(x.clone())
    x = layer_norm(x, tensors["final.norm"], tensors["final.norm.b"], eps)
    logits = (x @ tensors["head"].T) * cfg.get("logit_scale", 1.0)
    return (logits, layers) if return_layers else logits


# ----------------------------------------------------------------------------- random models
def random_model(cfg, seed=0):
    """{name: bf16 tensor} with the checkpoint's names: every value is a bf16 number, so that engines of either
    precision load exactly what the oracle computes with."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    t = {}

    def mat(name, out, inp, gain=1.0):
        t[name] = torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)

    def vec(name, n, mean=0.0, std=0.1):
        t[name] = mean + std * torch.randn(n, generator=g)

    def norm(name, n):
        vec(name, n, 1.0)
        vec(name + ".b", n)

    t["embed"] = torch.randn(cfg["vocab"], W, generator=g)
    t["pos"] = 0.5 * torch.randn(cfg["max_positions"], W, generator=g)
    norm("embed.norm", W)
    for i, entry in enumerate(cfg["layers"]):
        p, m = f"l{i}.", entry["mixer"]
        norm(p + "norm1", W)
        if entry["type"] == "hgrn2":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            mat(p + "mix.q", H * d, W)
            mat(p + "mix.f", H * d, W, 2.0)
            vec(p + "mix.f.b", H * d, 0.5, 1.0)
            t[p + "mix.lower"] = torch.rand(H * d, generator=g) * 0.95
            mat(p + "mix.v", H * dv, W)
            vec(p + "mix.norm", dv, 1.0)
            mat(p + "mix.o", W, H * dv)
        else:
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mat(p + "mix.q", H * d, W)
            vec(p + "mix.q.norm", H * d, 1.0)
            if m.get("kv_from") is None:
                mat(p + "mix.k", G * d, W)
                vec(p + "mix.k.norm", G * d, 1.0)
                mat(p + "mix.v", G * dv, W)
            t[p + "mix.talk"] = torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)
            vec(p + "mix.sink", H, 0.0, 1.0)
            mat(p + "mix.o", W, H * dv)
        mlp = entry.get("mlp")
        if mlp:
            norm(p + "norm2", W)
            if mlp["kind"] == "dense":
                mat(p + "mlp.up", mlp["ff"], W)
                vec(p + "mlp.up.b", mlp["ff"])
                mat(p + "mlp.down", W, mlp["ff"])
                vec(p + "mlp.down.b", W)
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                mat(p + "mlp.router", E, W, 2.0)
                vec(p + "mlp.router.b", E, 0.0, 0.5)
                for e in range(E):
                    mat(p + f"mlp.e{e}.up", ff, W)
                    mat(p + f"mlp.e{e}.down", W, ff)
    norm("final.norm", W)
    mat("head", cfg["vocab"], W)
    return {k: v.to(torch.bfloat16) for k, v in t.items()}


def as_f64(tensors):
    return {k: v.to(F64) for k, v in tensors.items()}
