"""Plain, slow restatement of the Guvusun decoder (test infrastructure only; shares no code with the product path).

One function per mechanism, float64 torch on the CPU, whole sequences only (a sequence is processed from position 0).  The product
(paged latent cache, state slots, ragged steps, CUDA kernels) is compared against this.

Guvusun in short: token embedding plus a hashed bigram embedding, normed; layers of the form "norm AFTER the sum" (x <- norm(a x +
sublayer(x))); the mixer is multi-head attention over a low-rank latent (only the latent and one shared rotated key part are kept per
token), with a per-head sink in the softmax denominator and a per-head sigmoid gate on the output; the feed-forward is a mixture of
experts with group-limited top-k routing, a selection-only correction term and parameter-free identity experts; after the feed-forward
a small per-layer, per-token embedding is gated by the stream and added back through a norm.

Notation: T tokens, D width, H heads, dn / dr unrotated / rotated query-key sizes, dv value size, R latent size, E experts that have
weights, I identity experts, N = E + I router outputs.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def bigram_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """row of the bigram table for every token: a hash of (previous, current); the first token of a sequence takes the extra last row"""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return rows


def embed(tokens: List[int], table: torch.Tensor, bigram: Optional[torch.Tensor], norm_w: torch.Tensor, bg: Optional[dict], eps: float) -> torch.Tensor:
    x = table.to(F)[torch.tensor(tokens, dtype=torch.long)]
    if bg:
        rows = torch.tensor(bigram_rows(tokens, int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"])), dtype=torch.long)
        x = x + bigram.to(F)[rows]
    return rms(x, eps) * norm_w.to(F)


def rotary_angles(T: int, dims: int, base: float, scaling: Optional[dict]):
    """cos / sin [T, dims/2] with YaRN: frequencies below the ramp are divided by the factor, both tables carry the magnitude term."""
    half = dims // 2
    i = torch.arange(half, dtype=F)
    f = float(base) ** (-2.0 * i / dims)
    mag = 1.0
    if scaling:
        fac, orig = float(scaling["factor"]), float(scaling["original"])
        where = lambda turns: dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(where(float(scaling["fast"]))), 0)
        hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / fac * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(fac) + 1.0
    ang = torch.arange(T, dtype=F)[:, None] * f[None, :]
    return torch.cos(ang) * mag, torch.sin(ang) * mag


def rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, ..., dims]; element i pairs with i + dims/2"""
    half = x.shape[-1] // 2
    u, v = x[..., :half], x[..., half:]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = cos.reshape(shape), sin.reshape(shape)
    return torch.cat([u * c - v * s, v * c + u * s], -1)


def latent_kv(h: torch.Tensor, w_dkv: torch.Tensor, w_norm: torch.Tensor, R: int, dr: int, rot: dict, eps: float):
    """-> (latent [T, R] normed, shared rotated key part [T, dr] after rotation)"""
    T = h.shape[0]
    z = h @ w_dkv.to(F).T
    c = rms(z[:, :R], eps) * w_norm.to(F)
    cos, sin = rotary_angles(T, dr, float(rot["base"]), rot.get("scaling"))
    return c, rotate_half(z[:, R:R + dr], cos, sin)


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, shared=None):
    """h [T, D] -> ([T, D], (latent, rotated key)).  ``shared`` = the (latent, rotated key) of another layer to attend over instead of
    this layer's own."""
    T = h.shape[0]
    H, dn, dr, dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    rot = m["rot"]
    g = lambda n: w[n].to(F)
    q = (h @ g("q").T).reshape(T, H, dn + dr)
    cos, sin = rotary_angles(T, dr, float(rot["base"]), rot.get("scaling"))
    qn, qr = q[..., :dn], rotate_half(q[..., dn:], cos, sin)
    c, kr = shared if shared is not None else latent_kv(h, w["dkv"], w["dkv.norm"], R, dr, rot, eps)
    kn = (c @ g("uk").T).reshape(T, H, dn)
    v = (c @ g("uv").T).reshape(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * float(m["scale"])
    s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)), float("-inf"))
    sink = g("sink")[:, None, None] if "sink" in w else torch.full((H, 1, 1), float("-inf"), dtype=F)
    mx = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - mx)
    p = e / (e.sum(-1, keepdim=True) + torch.exp(sink - mx))      # the sink adds to the denominator and to nothing else
    o = torch.einsum("hij,jhd->ihd", p, v)
    if "g" in w:
        o = o * torch.sigmoid(h @ g("g").T)[..., None]          # one gate per token and head
    o = o.reshape(T, H * dv)
    return o @ g("o").T, (c, kr)


def route(h: torch.Tensor, w_router: torch.Tensor, correction: torch.Tensor, r: dict):
    """-> (ids [T, top], weights [T, top]).  Selection uses softmax + correction, restricted to the ``keep`` groups with the best
    single member; weights use the plain softmax of the chosen, normalised, times the scale."""
    n_all, top = w_router.shape[0], int(r["top"])
    s = torch.softmax(h @ w_router.to(F).T, -1)
    pick = s if correction is None else s + correction.to(F)
    groups = r.get("groups")
    if groups:
        cnt, keep = int(groups["count"]), int(groups["keep"])
        per = n_all // cnt
        best = pick.reshape(-1, cnt, per).max(-1).values
        kept = torch.topk(best, keep, -1).indices
        allow = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        pick = pick.masked_fill(~allow[:, :, None].expand(-1, -1, per).reshape(-1, n_all), float("-inf"))
    ids = torch.topk(pick, top, -1).indices
    ws = torch.gather(s, 1, ids)
    return ids, ws / (ws.sum(-1, keepdim=True) + 1e-20) * float(r["scale"])


def moe(h: torch.Tensor, w: Dict[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    r = cfg["router"]
    n_all, n_id = int(r["experts"]) + int(r.get("identity", 0)), int(r.get("identity", 0))
    # "experts" counts the experts that have weights; the identity experts are the last router outputs
    if w["router"].shape[0] != n_all:
        raise ValueError("router rows != experts + identity")
    ids, ws = route(h, w["router"], w.get("correction"), r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), ws[t]):
            if e >= n_all - n_id:
                out[t] += a * h[t]
            else:
                g = lambda n: w[f"e{e}.{n}"].to(F)
                out[t] += a * (g("down") @ (silu(g("gate") @ h[t]) * (g("up") @ h[t])))
    return out


def token_side(x: torch.Tensor, tokens: List[int], side_embed: torch.Tensor, layer: int, dim: int, w: Dict[str, torch.Tensor], eps: float):
    e = side_embed.to(F)[torch.tensor(tokens, dtype=torch.long), layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w["gate"].to(F).T) * e) @ w["proj"].to(F).T
    return x + rms(y, eps) * w["norm"].to(F)


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], hidden: Optional[list] = None) -> torch.Tensor:
    """-> logits [T, vocab]; ``hidden`` collects the stream after every layer"""
    eps, alpha = float(cfg["norm"]["eps"]), float(cfg["postln_alpha"])
    sub = lambda pre: {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}
    bg = (cfg.get("embedding") or {}).get("bigram")
    x = embed(tokens, w["embed"], w.get("bigram"), w["embed.norm"], bg, eps)
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        if L["type"] != "latent_attention":
            raise ValueError(L["type"])
        src = L["mixer"].get("kv_from")
        y, kept[i] = latent_attention(x, sub(p + "mix."), L["mixer"], eps, shared=None if src is None else kept[int(src)])
        x = rms(alpha * x + y, eps) * w[p + "norm1"].to(F)
        if L.get("mlp"):
            x = rms(alpha * x + moe(x, sub(p + "mlp."), L["mlp"]), eps) * w[p + "norm2"].to(F)
        elif p + "norm2" in w:
            x = rms(alpha * x, eps) * w[p + "norm2"].to(F)
        if cfg.get("token_side"):
            x = token_side(x, tokens, w["side.embed"], i, int(cfg["token_side"]["dim"]), sub(p + "side."), eps)
        if hidden is not None:
            hidden.append(x.clone())
    return (rms(x, eps) * w["final.norm"].to(F)) @ w["head"].to(F).T


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(forward(cfg, w, ids)[-1]))
        out.append(t); ids.append(t)
    return out
