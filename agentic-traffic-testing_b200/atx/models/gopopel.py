"""Gopopel: a decoder-only family whose layers are listed one by one in config.json, every layer PARALLEL:

    u = tanh(alpha x) * w + b              (a norm without row statistics; one per layer, both sublayers read it)
    x <- x + mixer(u) + ffn(u)             (ffn optional: W_down relu(W_up u)^2)

The stream starts as embed[token] * embedding.scale; logits = head . norm(x) with the same kind of norm. The mixers:

  attention         softmax attention with grouped key/value heads: q and k of every head are divided by their root mean
                    square and multiplied by one weight vector shared by the heads; no rotation; the score
                    scale (q . k) loses slope_h (i - j), slope_h = 2^(-8 (h + 1) / heads); a query sees itself and the
                    mask.size - 1 positions before it; the softmax denominator also holds exp(sink_h), a learned number
                    per head without a value; in layers with `v_mix` (all but the first of them) the values become
                    (1 - lam) v + lam v_first, v_first being the first such layer's values of the same token, and the
                    blended values are what the pages keep.
  latent_attention  queries through a bottleneck (W_dq, RMS norm, W_uq), laid out per head as [dim plain | rot_dim
                    rotated]; keys and values from a second bottleneck: the first kv_rank outputs of W_dkv, RMS-normed,
                    are the latent c, the last rot_dim are one rotated key part shared by all heads; per head
                    k = [W_uk c | rotated part], v = W_uv c; sliding window; plain softmax; the concatenated heads are
                    multiplied by sigmoid(W_g u) before the output projection. Rotation turns adjacent pairs (2i, 2i+1)
                    of the first rot.dims elements by position * base^(-2i / dims).

Latent attention runs in its absorbed form: the pages hold only [c | rotated key part] per token (one "key head" of
kv_rank + rot_dim elements whose first kv_rank elements double as the value), the query of head h becomes
[W_uk,h^T q_plain | q_rotated], and W_uv,h is applied to the attention output of the head. Prompt portions and decoded
tokens take the same path, so a position's result does not depend on how the prompt was cut.

fp32 whatever the element type: the residual stream (the GEMMs of the output and down projections add into it), norms,
softmax, rotation, the value blend. Projections run in the element type (bf16 on the tcgen05 GEMM, or fp32 on the FMA
pipe) with fp32 accumulation.

The program below only issues kernels; scheduling, pages, staging, sampling and the step loop are the runner's and the
engine's (atx/runner.py, atx/engine.py)."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch

from .. import _cabi
from .common import _Linear, rotation_table

# ---- configuration --------------------------------------------------------------------------------------------------


@dataclass
class Config:
    name: str = "gopopel"
    vocab_size: int = 0
    width: int = 0
    eps: float = 1e-6
    embed_scale: float = 1.0
    layers: List[dict] = field(default_factory=list)   # {"type", "mixer", "mlp"} as in config.json
    eos_token_ids: tuple = ()
    bos_token_id: int = 0
    max_position_embeddings: int = 131072    # the design sets no limit; this bounds the server's default max_model_len
    architecture = "Gopopel"
    recurrent = False     # nothing but pages is carried from step to step

    @classmethod
    def from_json(cls, d: dict, name: str = "gopopel") -> "Config":
        cfg = cls(name=name, vocab_size=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]),
                  embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)), layers=[dict(l) for l in d["layers"]])
        cfg.validate()
        return cfg

    def validate(self) -> None:
        vshape = None
        for i, l in enumerate(self.layers):
            c = l["mixer"] = dict(l["mixer"])
            if l["type"] == "attention":
                c.setdefault("kv_heads", c["heads"])      # keys a configuration may leave out where the meaning is plain
                c.setdefault("vdim", c["dim"])
                if c["heads"] % c["kv_heads"]:
                    raise ValueError(f"layer {i}: {c['heads']} heads over {c['kv_heads']} key/value heads")
                if c.get("v_mix"):
                    sh = (c["kv_heads"], c["vdim"])
                    if vshape is not None and sh != vshape:
                        raise ValueError(f"layer {i}: value blending needs the value shape {vshape} of the first such layer")
                    vshape = sh
            elif l["type"] == "latent_attention":
                c["rot"] = dict(c.get("rot") or {})
                c["rot"].setdefault("dims", c["rot_dim"])  # the rotated part turns as a whole unless told otherwise
                c["rot"].setdefault("base", 10000.0)
                c.setdefault("vdim", c["dim"])
                rd = int(c["rot"]["dims"])
                if rd % 2 or rd > c["rot_dim"]:
                    raise ValueError(f"layer {i}: rot.dims={rd} must be even and at most rot_dim={c['rot_dim']}")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            if int((c.get("mask") or {}).get("size", 0)) < 0:
                raise ValueError(f"layer {i}: negative window")
            if l.get("mlp") is not None and l["mlp"].get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {l['mlp'].get('kind')!r}")

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def first_mix_layer(self) -> Optional[int]:
        for i, l in enumerate(self.layers):
            if l["type"] == "attention" and l["mixer"].get("v_mix"):
                return i
        return None

    def tensor_shapes(self) -> Dict[str, Tuple[int, ...]]:
        """Name -> shape of every tensor of a checkpoint of this configuration."""
        W, out = self.width, {}
        out["embed"] = (self.vocab_size, W)

        def norm(name: str) -> None:
            out[name], out[name + ".b"], out[name + ".alpha"] = (W,), (W,), ()

        for i, l in enumerate(self.layers):
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
        out["head"] = (self.vocab_size, W)
        return out

    # ---- bytes, for the benchmarks' rooflines -------------------------------------------------------------------
    def weight_bytes_per_decode_step(self, elem: int = 2) -> int:
        sh = self.tensor_shapes()
        return elem * sum(math.prod(v) for k, v in sh.items() if k != "embed")

    def kv_bytes_per_token(self, elem: int = 2) -> int:
        n = 0
        for l in self.layers:
            c = l["mixer"]
            if l["type"] == "attention":
                n += c["kv_heads"] * (c["dim"] + c["vdim"]) * elem
            else:
                n += (c["kv_rank"] + c["rot_dim"]) * elem
        return n


    def decode_kv_bytes(self, ctx: int, elem: int = 2) -> int:
        """Page bytes one decoded token at context length ctx reads: every layer at most its window."""
        n = 0
        for l in self.layers:
            c = l["mixer"]
            keys = min(ctx, int((c.get("mask") or {}).get("size", 0) or ctx))
            row = c["kv_heads"] * (c["dim"] + c["vdim"]) if l["type"] == "attention" else c["kv_rank"] + c["rot_dim"]
            n += keys * row * elem
        return n


def named_shape(name: str) -> Optional[Config]:
    """`random:gopopel-<size>`: shapes whose layers resemble a real model's, for benchmarks (no checkpoint exists).
    `gopopel-8b` / `gopopel-1b` have the width, feed-forward size, vocabulary and depth of the Llama 8B / 1B shapes;
    layers alternate latent attention and windowed attention (the second with value blending), each with a feed-forward."""
    key = name.lower()
    shapes = {"gopopel-8b": (4096, 14336, 16, 128256), "gopopel-1b": (2048, 8192, 8, 128256),
              "gopopel-tiny": (256, 512, 1, 1024)}     # width, feed-forward, repeats of the 2-layer pattern, vocabulary
    if key not in shapes:
        return None
    W, F, groups, vocab = shapes[key]
    hd = 128 if W >= 4096 else 64
    heads = W // hd
    ffn = {"ff": F, "kind": "dense"}
    lat = {"type": "latent_attention", "mlp": ffn,
           "mixer": {"dim": hd, "heads": heads, "kv_rank": 128, "q_rank": W * 3 // 8, "rot_dim": 64,
                     "rot": {"base": 10000.0, "dims": 64}, "mask": {"size": 4096}, "scale": (hd + 64) ** -0.5,
                     "vdim": hd}}
    att = {"type": "attention", "mlp": ffn,
           "mixer": {"dim": hd, "heads": heads, "kv_heads": max(1, heads // 4), "mask": {"size": 2048},
                     "scale": hd ** -0.5, "v_mix": True, "vdim": hd}}
    cfg = Config(name=key, vocab_size=vocab, width=W, eps=1e-6, embed_scale=1.0,
                 layers=[json.loads(json.dumps(l)) for l in [lat, att] * groups])
    cfg.validate()
    return cfg


# ---- weights ----------------------------------------------------------------------------------------------------------


class _Norm:
    def __init__(self, alpha: float, w: torch.Tensor, b: torch.Tensor) -> None:
        self.alpha, self.w, self.b = alpha, w, b


class _Layer:
    """Device tensors of one layer in the layout the kernels read (projections that share an input are stacked)."""

    def __init__(self) -> None:
        self.kind = ""
        self.norm: Optional[_Norm] = None
        self.w_in = self.w_o = None          # every projection of the mixer's input, stacked; output projection
        self.q_norm = self.k_norm = None     # attention: per-head norm weights [dim]
        self.sinks = self.slopes = None      # attention: fp32 [heads]
        self.vmix = 0.0
        self.dq_norm = self.dkv_norm = None  # latent attention
        self.w_uq = None                     # [heads * (dim + rot_dim), q_rank]
        self.w_ukt = None                    # [heads * kv_rank, dim]: W_uk of every head, transposed (absorbed into the query)
        self.w_uv = None                     # [heads * vdim, kv_rank]
        self.w_up = self.w_down = None


def distance_slopes(heads: int) -> List[float]:
    """Penalty per unit of distance for head h = 0 .. heads - 1: 2^(-8 (h + 1) / heads)."""
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


class Weights:
    def __init__(self, cfg: Config, device: torch.device, dtype: torch.dtype):
        self.cfg, self.device, self.dtype = cfg, device, dtype
        self.embed = self.head = None
        self.final_norm: Optional[_Norm] = None
        self.layers: List[_Layer] = []
        self.tp_size, self.tp_rank = 1, 0

    def nbytes(self) -> int:
        ts = [self.embed, self.head, self.final_norm.w, self.final_norm.b]
        for l in self.layers:
            ts += [v for v in vars(l).values() if isinstance(v, torch.Tensor)] + [l.norm.w, l.norm.b]
        return sum(t.numel() * t.element_size() for t in ts if isinstance(t, torch.Tensor))

    @classmethod
    def from_dir(cls, cfg: Config, path: Path, device: torch.device, dtype: torch.dtype) -> "Weights":
        from ..weights import _SafetensorsSource

        return cls._from_source(cfg, _SafetensorsSource(Path(path)), device, dtype)

    @classmethod
    def from_state_dict(cls, cfg: Config, sd: Dict[str, torch.Tensor], device: torch.device,
                        dtype: torch.dtype = torch.bfloat16) -> "Weights":
        from ..weights import _DictSource

        return cls._from_source(cfg, _DictSource(sd), device, dtype)

    @classmethod
    def random(cls, cfg: Config, seed: int, device: torch.device, dtype: torch.dtype = torch.bfloat16) -> "Weights":
        """Seeded random tensors generated on the device, one at a time."""
        g = torch.Generator(device=device).manual_seed(1000 * seed + 11)
        shapes = cfg.tensor_shapes()

        class _Gen:
            def has(self, name):
                return name in shapes

            def shape(self, name):
                return shapes[name]

            def full(self, name):
                sh = shapes[name]
                leaf = name.rsplit(".", 1)[-1]
                if len(sh) == 2:
                    return torch.randn(sh, generator=g, device=device) * (sh[1] ** -0.5)
                if leaf == "alpha":
                    return 0.3 + 0.4 * torch.rand(sh, generator=g, device=device)
                if leaf == "b":
                    return 0.05 * torch.randn(sh, generator=g, device=device)
                if leaf == "vmix":
                    return 0.2 + 0.5 * torch.rand(sh, generator=g, device=device)
                if leaf == "sink":
                    return torch.randn(sh, generator=g, device=device)
                return 1.0 + 0.1 * torch.randn(sh, generator=g, device=device)

        return cls._from_source(cfg, _Gen(), device, dtype)

    @classmethod
    def _from_source(cls, cfg: Config, src, device: torch.device, dtype: torch.dtype) -> "Weights":
        w = cls(cfg, device, dtype)
        want = cfg.tensor_shapes()

        def get(name: str) -> torch.Tensor:
            if not src.has(name):
                raise KeyError(f"checkpoint has no tensor {name!r}")
            t = src.full(name)
            if tuple(t.shape) != tuple(want[name]):
                raise ValueError(f"{name}: shape {tuple(t.shape)}, configuration says {tuple(want[name])}")
            return t

        def dev(t: torch.Tensor) -> torch.Tensor:
            return t.to(device=device, dtype=dtype).contiguous()

        def f32(t) -> torch.Tensor:
            return torch.as_tensor(t, dtype=torch.float32).to(device).contiguous()

        def norm(name: str) -> _Norm:
            return _Norm(float(get(name + ".alpha").float()), dev(get(name)), dev(get(name + ".b")))

        w.embed, w.head, w.final_norm = dev(get("embed")), dev(get("head")), norm("final.norm")
        first_mix = cfg.first_mix_layer()
        for i, spec in enumerate(cfg.layers):
            p, c, l = f"l{i}.", spec["mixer"], _Layer()
            l.kind = spec["type"]
            l.norm = norm(p + "norm1")
            m = p + "mix."
            if l.kind == "attention":
                l.w_in = dev(torch.cat([get(m + "q"), get(m + "k"), get(m + "v")], 0))
                l.q_norm, l.k_norm = dev(get(m + "q.norm")), dev(get(m + "k.norm"))
                l.sinks, l.slopes = f32(get(m + "sink").float()), f32(distance_slopes(c["heads"]))
                if c.get("v_mix") and i != first_mix:
                    l.vmix = float(get(m + "vmix").float())
                l.w_o = dev(get(m + "o"))
            else:
                H, D, C = c["heads"], c["dim"], c["kv_rank"]
                l.w_in = dev(torch.cat([get(m + "dq"), get(m + "dkv"), get(m + "g")], 0))
                l.dq_norm, l.dkv_norm = dev(get(m + "dq.norm")), dev(get(m + "dkv.norm"))
                l.w_uq = dev(get(m + "uq"))
                l.w_ukt = dev(get(m + "uk").reshape(H, D, C).transpose(1, 2).reshape(H * C, D))
                l.w_uv, l.w_o = dev(get(m + "uv")), dev(get(m + "o"))
            if spec.get("mlp") is not None:
                l.w_up, l.w_down = dev(get(p + "mlp.up")), dev(get(p + "mlp.down"))
            w.layers.append(l)
        return w


# ---- the layer program ------------------------------------------------------------------------------------------------


def _pad4(n: int) -> int:
    return (n + 3) // 4 * 4


class Program:
    needs_seq_view = True     # the attention kernels read the step row by row: sequence of a row, one block table
    graph_safe = True         # a padded row (no page slot, no sequence) is skipped by every kernel that writes pages

    def __init__(self, r) -> None:
        self.r = r
        cfg: Config = r.m
        w: Weights = r.w
        e = r.e
        self.cfg, self.w = cfg, w
        if e.tp_size != 1:
            raise ValueError("Gopopel runs on one GPU per replica")
        xt = w.dtype
        self.dt = _cabi.DT_F32 if xt == torch.float32 else _cabi.DT_BF16
        self.xt, self.esz = xt, (4 if xt == torch.float32 else 2)
        dev, T, lib = r.dev, r.Tmax, r.lib
        W = cfg.width
        f32 = torch.float32
        # widest intermediates of any layer
        n_in = n_q2 = n_up = n_qb = n_lat = n_mix = n_cq = n_v = 1
        for spec in cfg.layers:
            c = spec["mixer"]
            if spec["type"] == "attention":
                H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
                n_in, n_qb, n_mix = max(n_in, H * D + G * D + G * V), max(n_qb, H * D), max(n_mix, H * V)
                if c.get("v_mix"):
                    n_v = max(n_v, G * V)
            else:
                H, D, R, V, C, Q = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"], c["q_rank"]
                n_in, n_q2 = max(n_in, Q + C + R + H * V), max(n_q2, H * (D + R))
                n_qb, n_lat, n_mix, n_cq = max(n_qb, H * (C + R)), max(n_lat, H * C), max(n_mix, H * V), max(n_cq, Q)
            if spec.get("mlp") is not None:
                n_up = max(n_up, spec["mlp"]["ff"])
        self.n_in, self.n_q2, self.n_up = n_in, n_q2, n_up
        self.h = torch.zeros(T, W, dtype=f32, device=dev)                      # residual stream
        # fp32 GEMM outputs of a layer, back to back so that one pass clears them when split-K accumulates into them:
        # [mixer input projections | expanded queries (latent attention) | feed-forward up projection]
        self.scratch = torch.zeros(T * (_pad4(n_in) + _pad4(n_q2) + _pad4(n_up)) + 16, dtype=f32, device=dev)
        self.vfirst = torch.zeros(T * n_v, dtype=f32, device=dev)              # values of the first blending layer
        self.xn = torch.zeros(T, W, dtype=xt, device=dev)
        self.cq_flat = torch.zeros(T * n_cq, dtype=xt, device=dev)
        self.q_flat = torch.zeros(T * n_qb, dtype=xt, device=dev)
        self.lat_flat = torch.zeros(T * n_lat, dtype=xt, device=dev)
        self.mix_flat = torch.zeros(T * n_mix, dtype=xt, device=dev)
        self.act_flat = torch.zeros(T * n_up, dtype=xt, device=dev)
        self.xl = torch.zeros(r.Rmax, W, dtype=xt, device=dev)
        self._views: Dict[Tuple[int, int], torch.Tensor] = {}

        def view(flat: torch.Tensor, k: int) -> torch.Tensor:
            key = (flat.data_ptr(), k)
            if key not in self._views:
                self._views[key] = flat[:T * k].view(T, k)
            return self._views[key]

        # ---- linears (TMA descriptors are per (weight, input buffer) pair) -------------------------------------------
        self.lin: List[dict] = []
        for spec, l in zip(cfg.layers, w.layers):
            d = {"in": _Linear(lib, l.w_in, self.xn, self.dt),
                 "o": _Linear(lib, l.w_o, view(self.mix_flat, l.w_o.shape[1]), self.dt)}
            if l.w_uq is not None:
                d["uq"] = _Linear(lib, l.w_uq, view(self.cq_flat, l.w_uq.shape[1]), self.dt)
            if l.w_up is not None:
                d["up"] = _Linear(lib, l.w_up, self.xn, self.dt)
                d["down"] = _Linear(lib, l.w_down, view(self.act_flat, l.w_down.shape[1]), self.dt)
            self.lin.append(d)
        self.lin_head = _Linear(lib, w.head, self.xl, self.dt)

        # ---- pages: one set per layer --------------------------------------------------------------------------------
        bs = r.bs
        page_bytes = cfg.kv_bytes_per_token(self.esz) * bs
        if e.num_gpu_blocks is not None:
            nb = int(e.num_gpu_blocks)
        else:
            free, total = torch.cuda.mem_get_info(dev)
            budget = int(total * e.gpu_memory_utilization) - (total - free) - (512 << 20)
            nb = min(budget // page_bytes, r.MB * r.Smax)
            if nb < r.MB:
                raise RuntimeError(f"KV budget holds {nb} blocks; one sequence of max_model_len needs {r.MB}")
        r.num_blocks = nb
        r.block_bytes = page_bytes
        self.kv: List[Tuple[torch.Tensor, Optional[torch.Tensor]]] = []
        self.rot: Dict[Tuple[float, int], torch.Tensor] = {}
        for spec in cfg.layers:
            c = spec["mixer"]
            if spec["type"] == "attention":
                self.kv.append((torch.zeros(nb, c["kv_heads"], bs, c["dim"], dtype=xt, device=dev),
                                torch.zeros(nb, c["kv_heads"], bs, c["vdim"], dtype=xt, device=dev)))
            else:
                # one row per token: [latent | rotated key part]; the latent is read again as the value
                self.kv.append((torch.zeros(nb, 1, bs, c["kv_rank"] + c["rot_dim"], dtype=xt, device=dev), None))
                rot = c.get("rot") or {}
                key = (float(rot.get("base", 10000.0)), int(rot.get("dims", 0)))
                if key[1] and key not in self.rot:
                    self.rot[key] = rotation_table(key[0], key[1], e.max_model_len, dev)
        self.first_mix = cfg.first_mix_layer()
        # second stream for the feed-forward of decode-sized steps (see forward)
        self.overlap_ffn = True
        self.side = torch.cuda.Stream(device=dev)
        self.ev_fork, self.ev_join = torch.cuda.Event(), torch.cuda.Event()
        # scratch of the decode attention's key slices: [tokens, heads, slices, value width + 2] fp32
        self.max_splits = 32
        self.sms = torch.cuda.get_device_properties(dev).multi_processor_count
        h_max = max(spec["mixer"]["heads"] for spec in cfg.layers)
        self.split_ws = torch.zeros(max(2, r.Smax * h_max * self.max_splits * (128 + 2)), dtype=f32, device=dev)

    # ------------------------------------------------------------------------------------------------------------------
    def _attend(self, q: int, kc: int, vc: int, k_row: int, v_row: int, out: int, ldo: int, T: int, n_dec: int, n_pf: int,
                H: int, G: int, D: int, Vd: int, scale: float, window: int, slopes, sinks, fl: int, st: int) -> int:
        """Attention of the step's rows over their sequences' pages: prompt portions on the tensor cores where the
        element type and the sizes have such a kernel; single decoded tokens (and every row otherwise) on the kernel
        that gives a warp to each (row, head). Returns the launch count."""
        r, lib, ck, dp, dt = self.r, self.r.lib, self.r._ck, self.r._dp, self.dt
        sink = 1 if sinks is not None else 0
        tc = n_pf > 0 and lib.atx_attn_window_prefill_supported(D, Vd, k_row, v_row, dt)
        rows = n_dec if tc else T
        n = 0
        if rows and rows == n_dec and lib.atx_attn_window_decode_supported(H, G, D, Vd, k_row, v_row, dt):
            # decoded tokens: the heads of a key/value group as the rows of a tensor-core tile, the keys cut into slices
            # (as many as fill the GPU about three times, by the longest span a query of this layer can see: a fixed number per
            # layer and batch size, so a captured graph stays valid)
            keys = min(window or r.e.max_model_len, r.e.max_model_len)
            splits = max(1, min((keys + 63) // 64, self.max_splits, -(-3 * self.sms // (rows * G))))
            ws = self.split_ws
            ck(lib.atx_attn_window_decode(q, kc, vc, k_row, v_row, dp["seq_bt"], r.MB, dp["tok_seq"], dp["pos"], None, 0, out,
                                          ldo, ws.data_ptr(), ws.numel() * 4, splits, rows, H, G, D, Vd, r.bs, scale, 0.0, 0,
                                          window, slopes, sinks, sink, 1.0, dt, fl, st))
            n += 2 if splits > 1 else 1
        elif rows:
            ck(lib.atx_attn_window(q, kc, vc, k_row, v_row, dp["seq_bt"], r.MB, dp["tok_seq"], dp["pos"], None, 0, out, ldo,
                                   rows, H, G, D, Vd, r.bs, scale, 0.0, 0, window, slopes, sinks, sink, 1.0, dt, fl, st))
            n += 1
        if tc:
            ck(lib.atx_attn_window_prefill(q, kc, vc, k_row, v_row, dp["seq_bt"] + 4 * n_dec * r.MB, r.MB,
                                           dp["seq_start"] + 4 * n_dec, dp["seq_count"] + 4 * n_dec,
                                           dp["seq_pos0"] + 4 * n_dec, n_pf, T - n_dec, None, 0, out, ldo, H, G, D, Vd, r.bs,
                                           scale, 0.0, 0, window, slopes, sinks, sink, 1.0, dt, fl, st))
            n += 1
        return n

    def forward(self, T: int, n_dec: int, n_pf: int, n_rows: int) -> int:
        """Issue every kernel of one step on the current stream; returns the launch count. The step's first n_dec
        sequences are single decoded tokens (rows 0 .. n_dec-1), the next n_pf are prompt portions."""
        r, cfg, w = self.r, self.cfg, self.w
        lib, ck, dp, fl, dt = r.lib, r._ck, r._dp, r.flags, self.dt
        st = torch.cuda.current_stream().cuda_stream
        W, V, eps, bs = cfg.width, cfg.vocab_size, cfg.eps, r.bs
        h, xn = self.h.data_ptr(), self.xn.data_ptr()
        esz = self.esz
        ADD = _cabi.GEMM_ADD_F32
        n = 0
        ck(lib.atx_embed_rows_scaled(dp["ids"], w.embed.data_ptr(), h, T, W, V, cfg.embed_scale, dt, fl, st))
        n += 1
        probe = r.layer_probe
        seg, segs = _cabi.HeadSeg, _cabi.head_segs
        ROWS, PAGES = _cabi.HEAD_DST_ROWS, _cabi.HEAD_DST_PAGES
        qb, mix = self.q_flat.data_ptr(), self.mix_flat.data_ptr()
        for li, (spec, l, lin) in enumerate(zip(cfg.layers, w.layers, self.lin)):
            c = spec["mixer"]
            ld = l.w_in.shape[0]
            # this layer's fp32 GEMM outputs in the scratch buffer
            proj = self.scratch.data_ptr()
            q2 = proj + 4 * _pad4(T * ld)
            n_q2 = lin["uq"].N if "uq" in lin else 0
            up = q2 + 4 * _pad4(T * n_q2)
            n_ff = lin["up"].N if "up" in lin else 0
            fused_act = "up" in lin and lin["up"].plan is not None     # squared ReLU in the GEMM's epilogue (tcgen05 path)
            n_up = 0 if fused_act else n_ff
            acc = lin["in"].accumulates(T)        # decode-sized steps: the split-K GEMMs add into cleared buffers
            zero_bytes = 0
            if acc:
                zero_bytes = (up + 4 * T * n_up - proj + 15) // 16 * 16
            nm = l.norm
            ck(lib.atx_tanh_norm(h, None, nm.alpha, nm.w.data_ptr(), nm.b.data_ptr(), xn, T, W, proj if acc else None,
                                 zero_bytes, dt, fl, st))
            # Decode-sized steps: the feed-forward does not wait for the mixer (both read xn, both ADD into the stream with
            # red.add), so its two weight-streaming GEMMs run on a second stream beside the mixer's chain of short,
            # latency-bound kernels; the streams join before the next layer's norm. Inside a captured graph these are two
            # branches of the layer.
            side = None
            if fused_act and T <= 64 and self.overlap_ffn and lin["o"].plan is not None and lin["down"].plan is not None:
                side = self.side
                self.ev_fork.record(torch.cuda.current_stream())
                side.wait_event(self.ev_fork)
                ss = side.cuda_stream
                lin["up"].run(self.act_flat.data_ptr(), n_ff, T, fl, ss, mode=_cabi.GEMM_RELU2_BF16)
                lin["down"].run(h, W, T, fl, ss, mode=ADD)
                self.ev_join.record(side)
                n += 2
            lin["in"].run(proj, ld, T, fl, st, zeroed=acc)
            n += 2
            window = int((c.get("mask") or {}).get("size", 0) or 0)
            K_o = l.w_o.shape[1]
            kc, vc = self.kv[li]
            if l.kind == "attention":
                H, G, D, Vd = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
                mixing = bool(c.get("v_mix"))
                first = mixing and li == self.first_mix
                vf = self.vfirst.data_ptr()
                sg = segs(seg(src_off=0, src_stride=D, heads=H, width=D, norm_dims=D, norm_w=l.q_norm.data_ptr(),
                              dst_kind=ROWS, dst=qb, dst_ld=H * D, dst_off=0, dst_stride=D),
                          seg(src_off=H * D, src_stride=D, heads=G, width=D, norm_dims=D, norm_w=l.k_norm.data_ptr(),
                              dst_kind=PAGES, dst=kc.data_ptr(), dst_off=0, dst_stride=D),
                          seg(src_off=H * D + G * D, src_stride=Vd, heads=G, width=Vd,
                              save=vf if first else None, mix_src=vf if (mixing and not first) else None, mix=l.vmix,
                              dst_kind=PAGES, dst=vc.data_ptr(), dst_off=0, dst_stride=Vd))
                ck(lib.atx_head_prepare(proj, ld, sg, 3, dp["pos"], dp["slots"], T, bs, eps, dt, fl, st))
                n += 1 + self._attend(qb, kc.data_ptr(), vc.data_ptr(), D, Vd, mix, K_o, T, n_dec, n_pf, H, G, D, Vd,
                                      float(c["scale"]), window, l.slopes.data_ptr(), l.sinks.data_ptr(), fl, st)
            else:
                H, D, R, Vd, C, Q = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"], c["q_rank"]
                rot = c.get("rot") or {}
                rd = int(rot.get("dims", 0))
                table = self.rot[(float(rot.get("base", 10000.0)), rd)].data_ptr() if rd else None
                cq, lat = self.cq_flat.data_ptr(), self.lat_flat.data_ptr()
                # the two bottlenecks: normed query latent -> rows; [normed latent | rotated key part] -> the token's page row
                sg = segs(seg(src_off=0, src_stride=Q, heads=1, width=Q, norm_dims=Q, norm_w=l.dq_norm.data_ptr(),
                              dst_kind=ROWS, dst=cq, dst_ld=Q, dst_off=0, dst_stride=Q),
                          seg(src_off=Q, src_stride=C + R, heads=1, width=C + R, norm_dims=C,
                              norm_w=l.dkv_norm.data_ptr(), rot_off=C, rot_dims=rd, rot=table,
                              dst_kind=PAGES, dst=kc.data_ptr(), dst_off=0, dst_stride=C + R))
                ck(lib.atx_head_prepare(proj, ld, sg, 2, dp["pos"], dp["slots"], T, bs, eps, dt, fl, st))
                lin["uq"].run(q2, n_q2, T, fl, st, zeroed=acc)
                # queries in the latent's coordinates: [W_uk,h^T q_plain | rotated q part] per head
                sg = segs(seg(src_off=D, src_stride=D + R, heads=H, width=R, rot_off=0, rot_dims=rd, rot=table,
                              dst_kind=ROWS, dst=qb, dst_ld=H * (C + R), dst_off=C, dst_stride=C + R))
                ck(lib.atx_head_prepare(q2, n_q2, sg, 1, dp["pos"], dp["slots"], T, bs, eps, dt, fl, st))
                ck(lib.atx_head_gemm(q2, 1, n_q2, 0, D + R, l.w_ukt.data_ptr(), D, None, 0, qb, H * (C + R), 0, C + R, T, H,
                                     C, D, dt, fl, st))
                n += self._attend(qb, kc.data_ptr(), kc.data_ptr(), C + R, C + R, lat, H * C, T, n_dec, n_pf, H, 1, C + R, C,
                                  float(c["scale"]), window, None, None, fl, st)
                # values of the head from its attention output over latents, times the output gate
                ck(lib.atx_head_gemm(lat, 0, H * C, 0, C, l.w_uv.data_ptr(), C, proj + 4 * (Q + C + R), ld, mix, K_o, 0, Vd,
                                     T, H, Vd, C, dt, fl, st))
                n += 5
            lin["o"].run(h, W, T, fl, st, mode=ADD)
            n += 1
            if side is not None:
                torch.cuda.current_stream().wait_event(self.ev_join)
            elif "up" in lin:
                act = self.act_flat.data_ptr()
                if fused_act:
                    lin["up"].run(act, n_ff, T, fl, st, mode=_cabi.GEMM_RELU2_BF16)
                else:
                    lin["up"].run(up, n_ff, T, fl, st, zeroed=acc)
                    ck(lib.atx_unary_act(up, n_ff, act, n_ff, T, n_ff, _cabi.ACT_RELU2, dt, fl, st))
                    n += 1
                lin["down"].run(h, W, T, fl, st, mode=ADD)
                n += 2
            if probe is not None:
                probe.append(self.h[:T].clone())
        if n_rows:
            nm = w.final_norm
            ck(lib.atx_tanh_norm(h, dp["rows"], nm.alpha, nm.w.data_ptr(), nm.b.data_ptr(), self.xl.data_ptr(), n_rows, W,
                                 None, 0, dt, fl, st))
            self.lin_head.run(r.logits.data_ptr(), V, n_rows, fl, st)
            ck(lib.atx_sample(r.logits.data_ptr(), V, dp["temps"], dp["top_p"], dp["seeds"], dp["steps"],
                              r.out_ids.data_ptr(), n_rows, V, fl, st))
            n += 3
        return n
