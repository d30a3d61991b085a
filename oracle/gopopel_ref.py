"""Slow reference of the Gopopel family in float64 on the CPU, one function per mechanism.

Test infrastructure only: nothing under agentic-traffic-testing_b200/ imports it, and it imports nothing from there.
Every function works on a whole sequence at once ([n, ...] tensors, position = row index) and is written as the
defining sums over all pairs of positions (no pages, no carried cache, no tiling, no absorbed products).

Notation: n tokens, model width W; `lin(u, M)` = u M^T for a matrix M [out, in]. `cfg` is the parsed config.json of a
model, `wt` maps tensor names to float64 tensors.

The family: x = E[token] * s_emb; every layer computes u = dyt(x) once and adds mixer(u) + ffn(u) to x (the two
sublayers run side by side on the same normalised input); logits = head . dyt(x). Two mixers: softmax attention under
a sliding window with a per-head linear distance penalty, per-head unit-rms q/k, a learned sink logit in the
denominator and value blending with the first blending layer's values; and latent attention (queries and keys/values
through low-rank bottlenecks, a rotated key part shared by all heads, sigmoid output gate).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def lin(u: torch.Tensor, m: torch.Tensor) -> torch.Tensor:
    return u @ m.T


def dyt(x: torch.Tensor, alpha: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Element-wise squashing norm: w * tanh(alpha x) + b. No statistics of the row are taken."""
    return torch.tanh(alpha * x) * w + b


def unit_rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x scaled to unit root-mean-square over the last axis (eps under the root), times the weight as it is stored."""
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * w


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) ** 2


def head_slopes(heads: int) -> torch.Tensor:
    """Penalty per unit of distance of head h (0-based): 2^(-8 (h + 1) / heads)."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=F64)


def window_mask(n: int, size: int) -> torch.Tensor:
    """[n, n] bool: query i sees key j iff 0 <= i - j < size."""
    i = torch.arange(n)
    d = i[:, None] - i[None, :]
    return (d >= 0) & (d < size)


def rotate_pairs(x: torch.Tensor, dims: int, base: float, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [n, ..., D]: the first `dims` entries of the last axis, taken as adjacent pairs (2i, 2i+1), are turned by the
    angle p * base^(-2i/dims) at position p (row index unless given); the rest pass through."""
    n = x.shape[0]
    p = (torch.arange(n) if positions is None else positions).to(F64)
    i = torch.arange(dims // 2, dtype=F64)
    ang = p[:, None] * torch.pow(torch.tensor(base, dtype=F64), -2.0 * i / dims)[None, :]       # [n, dims/2]
    shape = [n] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = ang.cos().view(shape), ang.sin().view(shape)
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, visible: torch.Tensor,
                      slopes: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [n, H, D], k [n, G, D], v [n, G, V], visible [n, n] bool. Head h reads key/value head h // (H / G).
    a[h, i, j] = scale (q_i . k_j) - slopes[h] (i - j); weights = exp(a) / (sum over visible j of exp(a) + exp(sinks[h]))
    (the sink term has no value row); out [n, H, V]."""
    n, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    a = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if slopes is not None:
        i = torch.arange(n, dtype=F64)
        a = a - slopes[:, None, None] * (i[:, None] - i[None, :])[None]
    a = a.masked_fill(~visible[None], -math.inf)
    m = a.max(dim=-1, keepdim=True).values
    if sinks is not None:
        m = torch.maximum(m, sinks.to(F64)[:, None, None])
    e = torch.exp(a - m)
    den = e.sum(dim=-1, keepdim=True)
    if sinks is not None:
        den = den + torch.exp(sinks.to(F64)[:, None, None] - m)
    return torch.einsum("hij,jhv->ihv", e / den, vv)


def window_attention_mixer(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], p: str, eps: float,
                           shared: dict) -> torch.Tensor:
    """The 'attention' mixer. `shared` carries the first blending layer's values across layers of one forward pass."""
    n = u.shape[0]
    H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = unit_rms(lin(u, wt[p + "q"]).view(n, H, D), wt[p + "q.norm"], eps)
    k = unit_rms(lin(u, wt[p + "k"]).view(n, G, D), wt[p + "k.norm"], eps)
    v = lin(u, wt[p + "v"]).view(n, G, V)
    if c.get("v_mix"):
        if "v_first" not in shared:
            shared["v_first"] = v
        else:
            lam = wt[p + "vmix"]
            v = (1.0 - lam) * v + lam * shared["v_first"]
    o = softmax_attention(q, k, v, float(c["scale"]), window_mask(n, int(c["mask"]["size"])), head_slopes(H),
                          wt[p + "sink"])
    return lin(o.reshape(n, H * V), wt[p + "o"])


def latent_attention_mixer(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """The 'latent_attention' mixer, with keys and values of every head written out in full."""
    n = u.shape[0]
    H, D, R, V, C = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    rot = c["rot"]
    cq = unit_rms(lin(u, wt[p + "dq"]), wt[p + "dq.norm"], eps)
    q = lin(cq, wt[p + "uq"]).view(n, H, D + R)
    q_flat, q_rot = q[..., :D], rotate_pairs(q[..., D:].contiguous(), int(rot["dims"]), float(rot["base"]))
    dkv = lin(u, wt[p + "dkv"])
    lat = unit_rms(dkv[:, :C], wt[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(dkv[:, C:].contiguous().view(n, 1, R), int(rot["dims"]), float(rot["base"]))
    k_flat = lin(lat, wt[p + "uk"]).view(n, H, D)
    v = lin(lat, wt[p + "uv"]).view(n, H, V)
    qq = torch.cat([q_flat, q_rot], dim=-1)
    kk = torch.cat([k_flat, k_rot.expand(n, H, R)], dim=-1)
    o = softmax_attention(qq, kk, v, float(c["scale"]), window_mask(n, int(c["mask"]["size"])))
    o = o.reshape(n, H * V) * torch.sigmoid(lin(u, wt[p + "g"]))
    return lin(o, wt[p + "o"])


def dense_ffn(u: torch.Tensor, wt: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return lin(relu_squared(lin(u, wt[p + "up"])), wt[p + "down"])


def forward(cfg: dict, wt: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence; `residuals` (a list) receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = wt["embed"][torch.tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    shared: dict = {}
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        u = dyt(x, wt[p + "norm1.alpha"], wt[p + "norm1"], wt[p + "norm1.b"])
        if l["type"] == "attention":
            y = window_attention_mixer(u, l["mixer"], wt, p + "mix.", eps, shared)
        elif l["type"] == "latent_attention":
            y = latent_attention_mixer(u, l["mixer"], wt, p + "mix.", eps)
        else:
            raise ValueError(l["type"])
        if l.get("mlp") is not None:
            y = y + dense_ffn(u, wt, p + "mlp.")
        x = x + y
        if residuals is not None:
            residuals.append(x.clone())
    u = dyt(x, wt["final.norm.alpha"], wt["final.norm"], wt["final.norm.b"])
    return lin(u, wt["head"])


# ---- checkpoints for the tests ---------------------------------------------------------------------------------------


def checkpoint_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
    W, out = int(cfg["width"]), {}
    out["embed"] = (int(cfg["vocab"]), W)

    def norm(name: str) -> None:
        out[name], out[name + ".b"], out[name + ".alpha"] = (W,), (W,), ()

    for i, l in enumerate(cfg["layers"]):
        p, c = f"l{i}.", l["mixer"]
        norm(p + "norm1")
        m = p + "mix."
        if l["type"] == "attention":
            H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
            out[m + "q"], out[m + "k"], out[m + "v"] = (H * D, W), (G * D, W), (G * V, W)
            out[m + "q.norm"], out[m + "k.norm"] = (D,), (D,)
            if c.get("v_mix"):
                out[m + "vmix"] = ()
            out[m + "sink"], out[m + "o"] = (H,), (W, H * V)
        else:
            H, D, R, V, C, Q = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"], c["q_rank"]
            out[m + "dq"], out[m + "dq.norm"], out[m + "uq"] = (Q, W), (Q,), (H * (D + R), Q)
            out[m + "dkv"], out[m + "dkv.norm"] = (C + R, W), (C,)
            out[m + "uk"], out[m + "uv"] = (H * D, C), (H * V, C)
            out[m + "g"], out[m + "o"] = (H * V, W), (W, H * V)
        if l.get("mlp") is not None:
            F = l["mlp"]["ff"]
            out[p + "mlp.up"], out[p + "mlp.down"] = (F, W), (W, F)
    norm("final.norm")
    out["head"] = (int(cfg["vocab"]), W)
    return out


def random_checkpoint(cfg: dict, seed: int, round_bf16: bool = True) -> Dict[str, torch.Tensor]:
    """Seeded float64 tensors (values representable in bf16 when round_bf16, so that a bf16 engine loads them exactly)."""
    g = torch.Generator().manual_seed(seed)
    wt = {}
    for name, sh in checkpoint_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if len(sh) == 2:
            t = torch.randn(sh, generator=g, dtype=F64) * (sh[1] ** -0.5)
            if name == "embed":
                t = t * 0.3
        elif leaf == "alpha":
            t = 0.3 + 0.4 * torch.rand((), generator=g, dtype=F64)
        elif leaf == "b":
            t = 0.05 * torch.randn(sh, generator=g, dtype=F64)
        elif leaf == "vmix":
            t = 0.2 + 0.5 * torch.rand((), generator=g, dtype=F64)
        elif leaf == "sink":
            t = torch.randn(sh, generator=g, dtype=F64)
        else:   # norm weights
            t = 1.0 + 0.1 * torch.randn(sh, generator=g, dtype=F64)
        wt[name] = t.to(torch.bfloat16).to(F64) if round_bf16 else t
    return wt
