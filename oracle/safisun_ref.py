"""Slow reference of the Safisun family in float64 on the CPU, one function per mechanism.

Test infrastructure only: nothing under agentic-traffic-testing_b200/ imports it, and it imports nothing from there.
Every function works on a whole sequence at once ([n, ...] tensors, position = row index) and is written as the
defining sums, not as the kernels compute them (no chunking, no carried state, no pages).

Notation: n tokens, model width W; for a mixer input u [n, W] and a matrix M [out, in], `lin(u, M)` = u M^T.
`cfg` is the parsed config.json of a model, `wt` maps tensor names to tensors.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def lin(u: torch.Tensor, m: torch.Tensor) -> torch.Tensor:
    return u @ m.T


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x scaled to unit root-mean-square over the last axis; eps sits under the root."""
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def swish(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def decayed_linear_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, lam: torch.Tensor) -> torch.Tensor:
    """o[t, h] = sum_{j <= t} lam_h^(t-j) (q[t,h] . k[j,h]) v[j,h]  for q, k [n, H, D], v [n, H, V], lam [H]:
    the closed form of S_t = lam S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    n = q.shape[0]
    t = torch.arange(n)
    gap = (t[:, None] - t[None, :]).clamp(min=0).to(F64)
    causal = (t[:, None] >= t[None, :]).to(F64)
    w = torch.pow(lam.to(F64)[:, None, None], gap[None]) * causal[None]         # [H, n, n]
    a = torch.einsum("thd,jhd->htj", q, k) * w
    return torch.einsum("htj,jhv->thv", a, v)


def lightning_mixer(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    n = u.shape[0]
    H, D, V = c["heads"], c["dim"], c["vdim"]
    q = swish(lin(u, wt[p + "q"])).view(n, H, D)
    k = swish(lin(u, wt[p + "k"])).view(n, H, D)
    v = swish(lin(u, wt[p + "v"])).view(n, H, V)
    o = decayed_linear_attention(q, k, v, torch.tensor(c["decay"], dtype=F64)).reshape(n, H * V)
    o = unit_rms(o, eps) * wt[p + "norm"] * torch.sigmoid(lin(u, wt[p + "g"]))
    return lin(o, wt[p + "o"])


def causal_taps(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y[t, c] = bias[c] + sum_j taps[c, K-1-j] x[t-j, c], x before the start being zero (taps [C, K], last = current)."""
    n, K = x.shape[0], taps.shape[1]
    y = bias.expand(n, -1).clone()
    for j in range(K):
        shifted = torch.zeros_like(x)
        if j < n:
            shifted[j:] = x[:n - j]
        y = y + shifted * taps[:, K - 1 - j]
    return y


def selective_scan(x: torch.Tensor, b: torch.Tensor, c: torch.Tensor, dt: torch.Tensor, rate: torch.Tensor,
                   skip: torch.Tensor) -> torch.Tensor:
    """x [n, H, P], b / c [n, H, N] (already expanded from groups), dt [n, H], rate [H] = exp(A_log), skip [H].
    With L[t] = sum_{i <= t} rate dt[i]:  y[t] = sum_{j <= t} exp(-(L[t] - L[j])) dt[j] (c[t] . b[j]) x[j] + skip x[t]."""
    n = x.shape[0]
    L = torch.cumsum(rate[None, :] * dt, dim=0)                                  # [n, H]
    t = torch.arange(n)
    causal = (t[:, None] >= t[None, :])
    diff = (L[:, None, :] - L[None, :, :]).permute(2, 0, 1)                      # [H, t, j]
    w = torch.where(causal[None], torch.exp(-diff.clamp(min=0)), torch.zeros((), dtype=F64))
    a = torch.einsum("thn,jhn->htj", c, b) * w * dt.T[:, None, :]
    return torch.einsum("htj,jhp->thp", a, x) + skip[None, :, None] * x


def mamba2_mixer(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    n = u.shape[0]
    H, P, N, G, R = c["heads"], c["vdim"], c["state"], c["groups"], c["norm_groups"]
    inner = H * P
    z, xbc, dt = torch.split(lin(u, wt[p + "in"]), [inner, inner + 2 * G * N, H], dim=-1)
    xbc = swish(causal_taps(xbc, wt[p + "conv"], wt[p + "conv.b"]))
    x, b, cc = torch.split(xbc, [inner, G * N, G * N], dim=-1)
    rep = H // G
    b = b.view(n, G, N).repeat_interleave(rep, dim=1)
    cc = cc.view(n, G, N).repeat_interleave(rep, dim=1)
    dt = torch.log1p(torch.exp(dt + wt[p + "dt_bias"]))
    y = selective_scan(x.view(n, H, P), b, cc, dt, torch.exp(wt[p + "A_log"]), wt[p + "D"]).reshape(n, inner)
    y = y * swish(z)
    y = unit_rms(y.view(n, R, inner // R), eps).reshape(n, inner) * wt[p + "norm"]
    return lin(y, wt[p + "o"])


def rotate_pairs(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [n, heads, D]: dimensions (2i, 2i+1), i < dims/2, of the row at position p turn by p * base^(-2i/dims)."""
    if not dims:
        return x
    n = x.shape[0]
    i = torch.arange(dims // 2, dtype=F64)
    ang = torch.arange(n, dtype=F64)[:, None] * base ** (-2.0 * i / dims)        # [n, dims/2]
    cs, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = even * cs - odd * sn
    out[..., 1:dims:2] = odd * cs + even * sn
    return out


def sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, cap: Optional[float],
                   size: Optional[int]) -> torch.Tensor:
    """q, k [n, H, D], v [n, H, V] (row = position). score = scale q.k, squashed to cap tanh(score / cap); row t sees
    j <= t inside its own block of `size` positions (all j <= t without size); weights exp(s_j) / (1 + sum exp(s_j))."""
    n = q.shape[0]
    s = torch.einsum("thd,jhd->htj", q, k) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    t = torch.arange(n)
    seen = t[:, None] >= t[None, :]
    if size:
        seen = seen & ((t[:, None] // size) == (t[None, :] // size))
    e = torch.exp(s) * seen[None].to(F64)
    prob = e / (1.0 + e.sum(dim=-1, keepdim=True))           # the extra 1: a sink of score 0 that carries no value
    return torch.einsum("htj,jhv->thv", prob, v)


def local_attention(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    n = u.shape[0]
    H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = unit_rms(lin(u, wt[p + "q"]) + wt[p + "q.b"], eps) * wt[p + "q.norm"]
    k = unit_rms(lin(u, wt[p + "k"]) + wt[p + "k.b"], eps) * wt[p + "k.norm"]
    v = (lin(u, wt[p + "v"]) + wt[p + "v.b"]).view(n, G, V)
    rot = c.get("rot") or {}
    q = rotate_pairs(q.view(n, H, D), int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
    k = rotate_pairs(k.view(n, G, D), int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    o = sink_attention(q, k, v, c["scale"], c.get("softcap"), (c.get("mask") or {}).get("size"))
    o = o * torch.sigmoid(lin(u, wt[p + "g"]))[:, :, None]
    return lin(o.reshape(n, H * V), wt[p + "o"])


def parallel_mixer(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    return (c["left_scale"] * local_attention(u, c["left"], wt, p + "left.", eps) +
            c["right_scale"] * lightning_mixer(u, c["right"], wt, p + "right.", eps))


def gated_ffn(u: torch.Tensor, wt: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return lin(swish(lin(u, wt[p + "gate"])) * lin(u, wt[p + "up"]), wt[p + "down"])


MIXERS = {"lightning": lightning_mixer, "mamba2": mamba2_mixer, "parallel": parallel_mixer}


def layer_order(cfg: dict) -> List[Tuple[int, Optional[int]]]:
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, None) for i in range(n)]
    head = [(i, None) for i in range(lp["start"])]
    body = [(i, t) for t in range(lp["times"]) for i in range(lp["start"], lp["stop"])]
    return head + body + [(i, None) for i in range(lp["stop"], n)]


def forward(cfg: dict, wt: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence. `residuals`, if a list, receives the stream after every layer run."""
    wt = {k: v.to(F64) for k, v in wt.items()}
    eps = cfg["norm"]["eps"]
    x0 = wt["embed"][torch.tensor(tokens, dtype=torch.long)]
    x = x0
    for i, t in layer_order(cfg):
        spec, p = cfg["layers"][i], f"l{i}."
        if t is not None and i == cfg["loop"]["start"]:
            x = lin(torch.cat([x, x0], dim=-1), wt["loop.in"]) + wt["loop.step"][t]
        m = MIXERS[spec["type"]](unit_rms(x, eps) * wt[p + "norm1"], spec["mixer"], wt, p + "mix.", eps)
        x = x + unit_rms(m, eps) * wt[p + "norm1b"]
        if spec.get("mlp") is not None:
            f = gated_ffn(unit_rms(x, eps) * wt[p + "norm2"], wt, p + "mlp.")
            x = x + unit_rms(f, eps) * wt[p + "norm2b"]
        if residuals is not None:
            residuals.append(x.clone())
    return lin(unit_rms(x, eps) * wt["final.norm"], wt["head"])


# ---- random checkpoints for tests ---------------------------------------------------------------------------------


def checkpoint_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
    W, V = cfg["width"], cfg["vocab"]
    sh: Dict[str, Tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    if cfg.get("loop"):
        sh["loop.in"], sh["loop.step"] = (W, 2 * W), (cfg["loop"]["times"], W)

    def linear_attention(p: str, c: dict) -> None:
        hd, hv = c["heads"] * c["dim"], c["heads"] * c["vdim"]
        sh.update({p + "q": (hd, W), p + "k": (hd, W), p + "v": (hv, W), p + "g": (hv, W), p + "o": (W, hv),
                   p + "norm": (hv,)})

    for i, spec in enumerate(cfg["layers"]):
        p, c = f"l{i}.", spec["mixer"]
        sh[p + "norm1"] = sh[p + "norm1b"] = (W,)
        if spec["type"] == "lightning":
            linear_attention(p + "mix.", c)
        elif spec["type"] == "mamba2":
            inner, gn, H = c["heads"] * c["vdim"], c["groups"] * c["state"], c["heads"]
            sh.update({p + "mix.in": (2 * inner + 2 * gn + H, W), p + "mix.conv": (inner + 2 * gn, c["conv"]),
                       p + "mix.conv.b": (inner + 2 * gn,), p + "mix.dt_bias": (H,), p + "mix.A_log": (H,),
                       p + "mix.D": (H,), p + "mix.norm": (inner,), p + "mix.o": (W, inner)})
        else:
            a, q = c["left"], p + "mix.left."
            hd, gd, gv, hv = a["heads"] * a["dim"], a["kv_heads"] * a["dim"], a["kv_heads"] * a["vdim"], a["heads"] * a["vdim"]
            sh.update({q + "q": (hd, W), q + "q.b": (hd,), q + "k": (gd, W), q + "k.b": (gd,), q + "v": (gv, W),
                       q + "v.b": (gv,), q + "q.norm": (hd,), q + "k.norm": (gd,), q + "g": (a["heads"], W),
                       q + "o": (W, hv)})
            linear_attention(p + "mix.right.", c["right"])
        if spec.get("mlp") is not None:
            F = spec["mlp"]["ff"]
            sh[p + "norm2"] = sh[p + "norm2b"] = (W,)
            sh.update({p + "mlp.gate": (F, W), p + "mlp.up": (F, W), p + "mlp.down": (W, F)})
    return sh


def random_checkpoint(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Seeded weights, every value exactly representable in bfloat16 (so both element types see the same model)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in sorted(checkpoint_shapes(cfg).items()):
        leaf = name.rsplit(".", 1)[-1]
        if name == "loop.step" or leaf == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif leaf == "conv":
            t = 0.5 * torch.randn(shape, generator=g)
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) * (1.5 / math.sqrt(shape[1]))
        elif leaf == "A_log":
            t = torch.log(0.2 + 2.0 * torch.rand(shape, generator=g))
        elif leaf == "dt_bias":
            t = -1.0 + torch.randn(shape, generator=g)
        elif leaf == "D":
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        else:   # norm weights
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
