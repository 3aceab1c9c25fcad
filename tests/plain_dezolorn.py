"""A plain, slow statement of the Dezolorn decoder: whole sequences, no cache, float64 by default,
one function per mechanism.  It shares no code with the package; the tests compare the engine with it.

`cfg` is the model's config.json as a dict, `w` maps tensor names to tensors.
"""

from __future__ import annotations

import math

import torch


def layer_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * gain with the population variance, no bias."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * gain


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def rotary_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """Per-pair frequencies f_i and the factor on cos and sin.  With a `scaling` block (YaRN): the pairs
    that turn often keep f_i, those that turn rarely get f_i / factor, a linear ramp between them."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns: float) -> float:
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict, layout: str) -> torch.Tensor:
    """x [T, heads, dim]; the first rot.dims dimensions of each head turn, the rest pass.
    layout "interleaved": pairs (2i, 2i+1); "half": pairs (i, i + dims/2)."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    a = positions.to(torch.float64)[:, None] * f[None, :]
    cos, sin = (torch.cos(a) * mag)[:, None, :].to(x.dtype), (torch.sin(a) * mag)[:, None, :].to(x.dtype)
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., : dims // 2], x[..., dims // 2: dims]
        out[..., : dims // 2] = u * cos - v * sin
        out[..., dims // 2: dims] = v * cos + u * sin
    return out


def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    return j <= i and (i - j < size or j < keep_first)


def visible_mask(T: int, size: int, keep_first: int) -> torch.Tensor:
    """[T, T] of `visible(i, j)`."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def attention_mixer(h: torch.Tensor, m: dict, w: dict, p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    q = rms_unit(q, eps) * w[p + "q.norm"]
    k = rms_unit(k, eps) * w[p + "k.norm"]
    pos = torch.arange(T)
    q = rotate(q.view(T, H, D), pos, m["rot"], "interleaved")
    k = rotate(k.view(T, G, D), pos, m["rot"], "interleaved")
    v = v.view(T, G, V)
    size, keep = int(m["mask"]["size"]), int(m["mask"]["keep_first"])
    out = torch.zeros(T, H, V, dtype=h.dtype)
    mask = visible_mask(T, size, keep)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~mask, float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * V) @ w[p + "o"].T


def retention_mixer(h: torch.Tensor, m: dict, w: dict, p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = rotate((h @ w[p + "q"].T).view(T, H, D), pos, m["rot"], "half")
    k = rotate((h @ w[p + "k"].T).view(T, H, D), pos, m["rot"], "half") * D ** -0.5
    v = (h @ w[p + "v"].T).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = float(m["decay"][hd]) * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    out = rms_unit(out, eps).reshape(T, H * V)
    return (out * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def short_convolution(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, n]: y[t, c] = sum_j taps[c, j] * x[t - (n - 1) + j, c], zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    xp = torch.cat([torch.zeros(n - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + xp[j: j + T] * taps[:, j]
    return y


def delta_mixer(h: torch.Tensor, m: dict, w: dict, p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(short_convolution(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, D)
    k = silu(short_convolution(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, D)
    v = silu(short_convolution(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    g = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        kv = hd // (H // G)
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = g[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, hd] = S.T @ q[t, kv]
    out = rms_unit(out, eps) * w[p + "norm"]
    return (out.reshape(T, H * V) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def dense_feed_forward(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


MIXERS = {"attention": attention_mixer, "retention": retention_mixer, "delta": delta_mixer}


def layer_schedule(cfg: dict) -> list[tuple[int, bool]]:
    """(layer, whether the embedding output is added before it) in the order of execution."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(start)]
    for t in range(times if stop > start else 0):
        runs += [(i, t > 0 and i == start) for i in range(start, stop)]
    runs += [(i, False) for i in range(max(stop, start), n)]
    return runs


def forward(cfg: dict, w: dict, tokens: list[int], dtype=torch.float64, trace: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; `trace` collects the stream after every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    x0 = w["embed"][torch.tensor(tokens)]
    x = x0.clone()
    for i, add_input in layer_schedule(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        if add_input:
            x = x + x0
        x = x + MIXERS[layer["type"]](layer_norm(x, w[p + "norm1"], eps), layer["mixer"], w, p + "mix.", eps)
        if layer.get("mlp") is not None:
            x = x + dense_feed_forward(layer_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        if trace is not None:
            trace.append(x.clone())
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T * float(cfg["logit_scale"])
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(logits / cap) if cap > 0 else logits
