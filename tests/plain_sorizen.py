"""A plain, slow statement of the Sorizen decoder: whole sequences, no cache, float64, one function per mechanism.

It shares no code with the package: the configuration is the config.json dictionary and the weights a dictionary
of checkpoint names to tensors.  Everything is written the long way round (keys and values decompressed per head
from the latent, one softmax row per query) so that it checks the engine's absorbed, paged form.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def yarn_frequencies(rot: dict):
    """Frequencies of the rotated pairs and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F), 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, rot: dict):
    """x [T, ..., n]: the pair (2i, 2i+1) of the first rot.dims features turns by positions * f_i; the rest pass."""
    if not rot or x.shape[-1] == 0:
        return x
    dims = int(rot["dims"])
    if dims < x.shape[-1]:
        return torch.cat([rotate_interleaved(x[..., :dims], positions, rot), x[..., dims:]], dim=-1)
    f, mag = yarn_frequencies(rot)
    ang = positions.to(F)[:, None] * f[None, :]                  # [T, dims/2]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    cos, sin = torch.cos(ang) * mag, torch.sin(ang) * mag
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * cos - v * sin
    out[..., 1::2] = v * cos + u * sin
    return out


def latent_attention(h, w: dict, m: dict, eps: float, kind: str):
    """h [T, width] of one sequence; `w`: the mixer's tensors by their short names; `m`: the layer's "mixer" block."""
    T = h.shape[0]
    H, d, r, dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = torch.arange(T)
    q = (h @ w["q"].T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_interleaved(q[..., d:], pos, m.get("rot"))
    dkv = h @ w["dkv"].T
    c = rms_norm(dkv[:, :R], w["dkv.norm"], eps)
    k_rot = rotate_interleaved(dkv[:, R:], pos, m.get("rot"))           # [T, r], shared by the heads
    k_plain = (c @ w["uk"].T).view(T, H, d)
    v = (c @ w["uv"].T).view(T, H, dv)
    window = int(m["mask"]["size"]) if m.get("mask") else T + 1
    out = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        s = (q_plain[:, hh] @ k_plain[:, hh].T + q_rot[:, hh] @ k_rot.T) * float(m["scale"])   # [query, key]
        i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
        seen = (i - j >= 0) & (i - j < window)
        s = s.masked_fill(~seen, -math.inf)
        top = s.max(-1, keepdim=True).values
        if kind == "latent_attention":
            top = torch.maximum(top, w["sink"][hh].expand_as(top))
            e = torch.exp(s - top)
            p = e / (e.sum(-1, keepdim=True) + torch.exp(w["sink"][hh] - top))
        else:
            e = torch.exp(s - top)
            p = e / e.sum(-1, keepdim=True)
        out[:, hh] = p @ v[:, hh]
    if kind == "latent_attention_2":
        out = out * torch.sigmoid(h @ w["g"].T)[:, :, None]
    return out.reshape(T, H * dv) @ w["o"].T


def route(h, w_router, r: dict):
    """Chosen experts [T, top] and their weights [T, top]."""
    E, top = int(r["experts"]), int(r["top"])
    s = torch.sigmoid(h @ w_router.T)                               # [T, E]
    g = r.get("groups")
    allowed = torch.ones_like(s, dtype=torch.bool)
    if g:
        count, keep = int(g["count"]), int(g["keep"])
        per = E // count
        grouped = s.view(-1, count, per)
        gscore = grouped.topk(min(2, per), dim=-1).values.sum(-1)  # [T, count]
        best = gscore.topk(keep, dim=-1).indices
        gmask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, best, True)
        allowed = gmask[:, :, None].expand(-1, -1, per).reshape(-1, E)
    chosen = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    ws = s.gather(1, chosen)
    ws = ws / (ws.sum(-1, keepdim=True) + 1e-20) * float(r["scale"])
    return chosen, ws


def feed_forward(h, w: dict, mlp: dict):
    if mlp["kind"] == "dense":
        return gelu_erf(h @ w["up"].T) @ w["down"].T
    chosen, ws = route(h, w["router"], mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), ws[t].tolist()):
            x = h[t]
            out[t] += a * ((silu(w[f"e{e}.gate"] @ x) * (w[f"e{e}.up"] @ x)) @ w[f"e{e}.down"].T)
    return out


def _sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v.to(F) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and, on request, the stream after every layer run: the sum of the streams)."""
    eps = float(cfg["norm"]["eps"])
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = tensors["embed"].to(F)[tok] * float(cfg["embedding"]["scale"])
    S = cfg.get("streams")
    streams = [x.clone() for _ in range(int(S))] if S else None
    after = []
    for i, layer in enumerate(cfg["layers"]):
        j = layer.get("weights_of", i)
        p = f"l{j}."
        t = _sub(tensors, p)
        subs = [(1, lambda u: latent_attention(u, _sub(tensors, p + "mix."), layer["mixer"], eps, layer["type"]))]
        if layer.get("mlp") is not None:
            subs.append((2, lambda u: feed_forward(u, _sub(tensors, p + "mlp."), layer["mlp"])))
        for qn, fn in subs:
            nw, nb = t[f"norm{qn}"], t[f"norm{qn}.b"]
            if streams is None:
                x = x + fn(layer_norm(x, nw, nb, eps))
                continue
            a, o, mix = t[f"hc{qn}.in"], t[f"hc{qn}.out"], t[f"hc{qn}.mix"]
            u = sum(a[s] * streams[s] for s in range(len(streams)))
            y = fn(layer_norm(u, nw, nb, eps))
            streams = [sum(mix[s, tt] * streams[s] for s in range(len(streams))) + o[tt] * y for tt in range(len(streams))]
        after.append(sum(streams) if streams is not None else x.clone())
    x = sum(streams) if streams is not None else x
    x = layer_norm(x, tensors["final.norm"].to(F), tensors["final.norm.b"].to(F), eps)
    logits = x @ tensors["head"].to(F).T
    return (logits, torch.stack(after)) if return_layers else logits
