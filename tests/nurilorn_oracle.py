"""A plain, slow restatement of the Nurilorn decoder in float64, one function per mechanism, for the tests.

It shares no code with the package: every function works on whole sequences held in torch tensors on the CPU,
query by query where a mask is involved. Weights come as a dict {checkpoint tensor name: tensor}; the configuration is
the dict of config.json.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def grouped_rms_norm(x, w, groups: int, eps: float):
    """x [..., n] split into `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps); times w."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(shape) * w


def short_conv(u, w, tail=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros (or `tail`, the taps-1 inputs before u)
    ahead of the sequence. Returns (y, the last taps-1 inputs)."""
    taps = w.shape[1]
    T, C = u.shape
    if tail is None:
        tail = torch.zeros(taps - 1, C, dtype=u.dtype)
    full = torch.cat([tail, u], 0)
    y = torch.zeros(T, C, dtype=u.dtype)
    for j in range(taps):
        y += full[j:j + T] * w[:, j]
    return y, full[full.shape[0] - (taps - 1):]


def yarn_frequencies(rot: dict):
    """(frequencies [dims/2], magnitude) of rotary positions with the frequency-dependent stretch."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = torch.tensor([min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001))) for i in range(half)], dtype=F64)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot: dict):
    """x [T, heads, dim]: pairs (2i, 2i+1) of the first rot.dims columns turned by position * frequency_i."""
    f, mag = yarn_frequencies(rot)
    dims = int(rot["dims"])
    a = positions.to(F64)[:, None] * f[None, :]                     # [T, dims/2]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def sink_attention(q, k, v, scale: float, softcap: float, first_pos: int = 0):
    """q [Tq, H, d]; k [Tk, G, d], v [Tk, G, dv] hold the keys of positions 0..Tk-1; query t sits at first_pos + t.
    Capped scores, causal mask, softmax with one added to the denominator."""
    Tq, H, d = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(Tq, H, v.shape[2], dtype=q.dtype)
    for t in range(Tq):
        n = first_pos + t + 1
        for h in range(H):
            g = h // rep
            s = (k[:n, g] @ q[t, h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            m = max(float(s.max()), 0.0)
            e = torch.exp(s - m)
            p = e / (math.exp(-m) + e.sum())
            out[t, h] = p @ v[:n, g]
    return out


def clamped_unit(g, u, limit: float, alpha: float = 1.702):
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, -limit, limit)
    return g * torch.sigmoid(alpha * g) * (u + 1)


def dense_ff(h, w, prefix: str, limit: float):
    y = clamped_unit(h @ w[prefix + "gate"].T, h @ w[prefix + "up"].T, limit)
    return y @ w[prefix + "down"].T


def route(z, top: int, groups: int, keep: int):
    """z [T, E] router logits -> (ids [T, top], weights [T, top]): softmax over all experts; a group's score is its
    largest score; only experts of the `keep` best groups can be chosen."""
    T, E = z.shape
    s = torch.softmax(z, -1)
    gs = s.reshape(T, groups, E // groups).max(-1).values
    best = gs.topk(keep, -1).indices
    allowed = torch.zeros(T, groups, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    masked = torch.where(allowed[:, :, None].expand(T, groups, E // groups).reshape(T, E), s, torch.full_like(s, -1.0))
    ids = masked.topk(top, -1).indices
    wts = s.gather(1, ids)
    return ids, wts / (wts.sum(-1, keepdim=True) + 1e-20)


def moe_ff(h, w, prefix: str, mlp: dict):
    r = mlp["router"]
    g = r.get("groups") or {"count": 1, "keep": 1}
    ids, wts = route(h @ w[prefix + "router"].T, r["top"], g["count"], g["keep"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out[t] += wts[t, j] * dense_ff(h[t:t + 1], w, f"{prefix}e{e}.", mlp["expert"]["limit"])[0]
    return out


def attention_mixer(h, w, prefix: str, m: dict, positions, v_first=None, lam=None, state=None):
    """One attention mixer over a whole sequence (state None) or a continuation: state = dict(tails, k, v) of what the
    earlier tokens left. Returns (output [T, width], this layer's unmixed... see below, new state).
    The second result is the value rows BEFORE mixing (what a later layer mixes in when this is the first)."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    tails = state["tails"] if state else {}
    new_tails = {}
    proj = {}
    for name in "qkv":
        u = h @ w[prefix + name].T
        proj[name], new_tails[name] = short_conv(u, w[prefix + name + ".conv"], tails.get(name))
    q = rotate(proj["q"].reshape(T, H, d), positions, m["rot"])
    k = rotate(proj["k"].reshape(T, G, d), positions, m["rot"])
    v_own = proj["v"].reshape(T, G, dv)
    v = v_own if v_first is None else (1 - lam) * v_own + lam * v_first
    if state:
        k_all, v_all = torch.cat([state["k"], k], 0), torch.cat([state["v"], v], 0)
    else:
        k_all, v_all = k, v
    o = sink_attention(q, k_all, v_all, float(m["scale"]), float(m.get("softcap", 0.0)), first_pos=int(positions[0]))
    gate = torch.sigmoid(h @ w[prefix + "g"].T)                          # [T, H]
    o = (o * gate[:, :, None]).reshape(T, H * dv)
    return o @ w[prefix + "o"].T, v_own, {"tails": new_tails, "k": k_all, "v": v_all}


def forward(cfg: dict, weights: dict, tokens, states=None, first_pos: int = 0, layers_out=None):
    """Logits [T, vocab] (float64) for `tokens` at positions first_pos..; `states` (a list, one dict per layer, from an
    earlier call) continues a sequence. Returns (logits, states). layers_out: a list that receives the residual stream
    after every layer."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups", 1))
    mult = float(cfg.get("residual_mult", 1.0))
    x = w["embed"][torch.as_tensor(tokens)] * float(cfg["embedding"]["scale"])
    T = x.shape[0]
    positions = torch.arange(first_pos, first_pos + T)
    new_states = []
    v_first = None
    for i, entry in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = entry["mixer"]
        h = grouped_rms_norm(x, w[p + "norm1"], groups, eps)
        mixes = bool(m.get("v_mix")) and v_first is not None
        y, v_own, st = attention_mixer(h, w, p + "mix.", m, positions, v_first if mixes else None,
                                       w[p + "mix.vmix"] if mixes else None, states[i] if states else None)
        if m.get("v_mix") and v_first is None:
            v_first = v_own
        new_states.append(st)
        x = x + mult * (y * w[p + "ls1"])
        mlp = entry.get("mlp")
        if mlp:
            h = grouped_rms_norm(x, w[p + "norm2"], groups, eps)
            y = dense_ff(h, w, p + "mlp.", mlp["limit"]) if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp)
            x = x + mult * (y * w[p + "ls2"])
        if layers_out is not None:
            layers_out.append(x.clone())
    h = grouped_rms_norm(x, w["final.norm"], groups, eps)
    return h @ w["head"].T * float(cfg.get("logit_scale", 1.0)), new_states


def random_weights(cfg: dict, seed: int = 0, dtype=torch.bfloat16) -> dict:
    """Random weights for a configuration, rounded to `dtype` (the values every implementation then starts from)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    out = {}

    def mat(o, i, std=None):
        return torch.randn(o, i, generator=g) * (std if std is not None else i ** -0.5)

    out["embed"] = torch.randn(cfg["vocab"], W, generator=g) * 0.1
    out["head"] = mat(cfg["vocab"], W)
    out["final.norm"] = 1 + 0.1 * torch.randn(W, generator=g)
    for i, entry in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = entry["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        for n in ("norm1", "norm2", "ls1", "ls2"):
            out[p + n] = 1 + 0.1 * torch.randn(W, generator=g)
        for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
            out[p + "mix." + n] = mat(rows, W)
            out[p + f"mix.{n}.conv"] = torch.randn(rows, m["conv"], generator=g) * 0.5
        out[p + "mix.vmix"] = torch.rand((), generator=g) * 0.6 + 0.2
        out[p + "mix.g"] = mat(H, W)
        out[p + "mix.o"] = mat(W, H * dv)
        mlp = entry.get("mlp")
        if not mlp:
            del out[p + "norm2"], out[p + "ls2"]
        elif mlp["kind"] == "dense":
            out[p + "mlp.gate"], out[p + "mlp.up"] = mat(mlp["ff"], W), mat(mlp["ff"], W)
            out[p + "mlp.down"] = mat(W, mlp["ff"])
        else:
            ff = mlp["expert"]["ff"]
            out[p + "mlp.router"] = mat(mlp["router"]["experts"], W, std=4.0 * W ** -0.5)
            for e in range(mlp["router"]["experts"]):
                out[p + f"mlp.e{e}.gate"], out[p + f"mlp.e{e}.up"] = mat(ff, W), mat(ff, W)
                out[p + f"mlp.e{e}.down"] = mat(W, ff)
    return {k: v.to(dtype) for k, v in out.items()}
