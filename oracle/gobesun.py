"""Plain, slow restatement of the Gobesun decoder (test infrastructure only; shares no code with the product path).

One function per mechanism, float64 torch on the CPU, whole sequences only: a sequence is processed from position 0 with
empty state, token by token where the mechanism is a recurrence.  The product (paged cache, state slots, batched steps,
CUDA kernels) is compared against this.

Notation: T tokens, D model width, H query / value heads, G key heads, dk key size, dv value size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_zero_centred(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def short_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """Causal depthwise convolution over time.  x [T, C], taps [C, K]; column K-1 multiplies the current token, column
    K-1-d the token d steps back; tokens before the start count as zero."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for d in range(K):
        if d < T:
            y[d:] += x[:T - d] * taps[:, K - 1 - d]
    return y


def unit(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def delta_recurrence(q, k, v, beta, decay):
    """Gated delta rule.  q, k [T, H, dk]; v [T, H, dv]; beta, decay [T, H].  Per head, with S [dk, dv] starting at zero:
    S <- decay_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=F)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = S * decay[t][:, None, None]
        pred = torch.einsum("hkv,hk->hv", S, k[t])
        u = beta[t][:, None] * (v[t] - pred)
        S = S + torch.einsum("hk,hv->hkv", k[t], u)
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def delta_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """h [T, D] -> [T, D]; W holds the mixer's tensors by their short names ('q', 'q.conv', ...)."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(short_conv(h @ W["q"].T, W["q.conv"])).view(T, G, dk)
    k = silu(short_conv(h @ W["k"].T, W["k.conv"])).view(T, G, dk)
    v = silu(short_conv(h @ W["v"].T, W["v.conv"])).view(T, H, dv)
    q = unit(q) * dk ** -0.5
    k = unit(k)
    rep = H // G
    q = q.repeat_interleave(rep, dim=1)
    k = k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ W["b"].T)
    decay = torch.exp(-torch.exp(W["A_log"]) * torch.nn.functional.softplus(h @ W["a"].T + W["dt_bias"]))
    o = delta_recurrence(q, k, v, beta, decay)
    o = rms(o, eps) * W["norm"]
    gate = silu(h @ W["g"].T).view(T, H, dv)
    return (o * gate).reshape(T, H * dv) @ W["o"].T


def rotary_angles(rot: dict, positions: torch.Tensor):
    """cos, sin [T, dims/2] including the YaRN frequency blend and magnitude factor."""
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    i = torch.arange(half, dtype=F)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        def corr(turns):
            return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(corr(sc["fast"])), 0)
        hi = min(math.ceil(corr(sc["slow"])), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(sc["factor"]) + 1.0
    ang = positions.to(F)[:, None] * f[None, :]
    return torch.cos(ang) * mag, torch.sin(ang) * mag


def rotate(x: torch.Tensor, cos, sin, dims: int) -> torch.Tensor:
    """x [T, heads, d]: the first `dims` entries of every head are rotated, entry i paired with entry i + dims/2."""
    half = dims // 2
    a, b, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)


def visible(i: int, j: int, mask: Optional[dict]) -> bool:
    """may the query at position i look at the key at position j?"""
    if j > i:
        return False
    if mask and "size" in mask:
        return i // mask["size"] == j // mask["size"]
    return True


def masked_attention(q, k, v, scale: float, mask: Optional[dict], pos) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] of one sequence whose rows sit at positions pos [T] -> [T, H, dv]."""
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[-1]
    rep = H // G
    allowed = torch.tensor([[visible(int(pos[a]), int(pos[b]), mask) for b in range(T)] for a in range(T)])
    out = torch.zeros(T, H, dv, dtype=F)
    for hd in range(H):
        s = (q[:, hd] @ k[:, hd // rep].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, hd // rep]
    return out


def attention_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], m: dict, eps: float, positions=None) -> torch.Tensor:
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(T) if positions is None else positions
    q = rms(h @ W["q"].T, eps) * W["q.norm"]
    k = rms(h @ W["k"].T, eps) * W["k.norm"]
    v = (h @ W["v"].T).view(T, G, dv)
    q, k = q.view(T, H, dk), k.view(T, G, dk)
    rot = m.get("rot")
    if rot:
        cos, sin = rotary_angles(rot, pos)
        q, k = rotate(q, cos, sin, rot["dims"]), rotate(k, cos, sin, rot["dims"])
    out = masked_attention(q, k, v, m["scale"], m.get("mask"), pos)
    return out.reshape(T, H * dv) @ W["o"].T


def dense_mlp(h, W):
    return (gelu_tanh(h @ W["gate"].T) * (h @ W["up"].T)) @ W["down"].T


def layer_order(cfg: dict) -> List[int]:
    """Indices of the layers in the order they run, the looped span repeated."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens, trace: Optional[list] = None) -> torch.Tensor:
    """tokens: T ids of ONE sequence from position 0 -> logits [T, vocab] (float64).  `trace`, if a list, receives the residual
    stream after every layer run."""
    W = {k: v.to(F) for k, v in weights.items() if v.is_floating_point()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    for li in layer_order(cfg):
        L = cfg["layers"][li]
        p = f"l{li}."
        mix = {k[len(p) + 4:]: v for k, v in W.items() if k.startswith(p + "mix.")}
        hin = norm_zero_centred(x, W[p + "norm1"], eps)
        y = delta_mixer(hin, mix, L["mixer"], eps) if L["type"] == "delta" else attention_mixer(hin, mix, L["mixer"], eps)
        x = x + norm_zero_centred(y, W[p + "norm1b"], eps)
        if L.get("mlp"):
            mlp = {k[len(p) + 4:]: v for k, v in W.items() if k.startswith(p + "mlp.")}
            x = x + norm_zero_centred(dense_mlp(norm_zero_centred(x, W[p + "norm2"], eps), mlp), W[p + "norm2b"], eps)
        if trace is not None:
            trace.append(x.clone())
    return norm_zero_centred(x, W["final.norm"], eps) @ W["head"].T


def greedy(cfg, weights, prompt, steps: int) -> List[int]:
    """Greedy continuation by re-running the whole sequence (slow, on purpose)."""
    ids = list(prompt)
    for _ in range(steps):
        ids.append(int(forward(cfg, weights, ids)[-1].argmax()))
    return ids[len(prompt):]
