"""Safisun: a decoder-only family whose layers are listed one by one in config.json.

Each layer has one sequence mixer and, optionally, a gated feed-forward; every sublayer sits between two RMS norms
(`x += norm_b(f(norm_a(x)))`). The mixers:

  lightning  linear attention with a fixed decay per head: S <- decay_h S + k v^T, o = S^T q, q/k/v through silu; the
             heads together are RMS-normed, gated by sigmoid(W_g h) and projected.
  mamba2     selective state-space scan: in-projection [z | x | B | C | dt], short causal convolution + silu over
             x, B, C, dt = softplus(dt + bias), S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x, gate silu(z)
             BEFORE an RMS norm in equal groups, projection.
  parallel   two mixers on the same input, summed with fixed scales: softmax attention (grouped KV heads, biases,
             RMS norm over the whole q and whole k projection, rotation of adjacent pairs on the first `rot.dims`
             dimensions, tanh score cap, block-local causal mask, +1 in the softmax denominator, a sigmoid gate per
             head) beside a lightning mixer.

A block of consecutive layers may run several times with the same weights (`loop`); every pass has caches and states of
its own and starts with x <- W_in [x ; x0] + step[pass], x0 being the embedding output.

What is computed in fp32 whatever the element type: the residual stream, all norms, softmax, the recurrent states and
everything entering a recurrence but the projections (decays, step sizes, gates), the convolution. Projections run in
the element type (bf16 on the tcgen05 GEMM, or fp32 on the FMA pipe) with fp32 accumulation.

The program below only issues kernels; scheduling, pages, state slots, staging, sampling and the step loop are the
runner's and the engine's (atx/runner.py, atx/engine.py)."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch

from .. import _cabi
from .common import _Linear, _use_tc, rotation_table  # noqa: F401  (shared by every layer-list family)

# ---- configuration --------------------------------------------------------------------------------------------------


@dataclass
class Config:
    name: str = "safisun"
    vocab_size: int = 0
    width: int = 0
    eps: float = 1e-5
    layers: List[dict] = field(default_factory=list)   # {"type", "mixer", "mlp"} as in config.json
    loop: Optional[dict] = None                        # {"start", "stop", "times"}
    eos_token_ids: tuple = ()
    bos_token_id: int = 0
    max_position_embeddings: int = 131072    # the design sets no limit; this bounds the server's default max_model_len
    architecture = "Safisun"
    recurrent = True      # sequences own a state slot; cached prefixes cannot be re-attached (the state is not kept)

    @classmethod
    def from_json(cls, d: dict, name: str = "safisun") -> "Config":
        loop = d.get("loop") or None
        cfg = cls(name=name, vocab_size=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]),
                  layers=[dict(l) for l in d["layers"]], loop=dict(loop) if loop else None)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for i, l in enumerate(self.layers):
            if l["type"] not in ("lightning", "mamba2", "parallel"):
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            if l.get("mlp") is not None and l["mlp"].get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {l['mlp'].get('kind')!r}")
        if self.loop:
            a, b, n = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not (0 <= a < b <= len(self.layers) and n >= 1):
                raise ValueError(f"bad loop {self.loop}")

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.runs())

    def runs(self) -> List[Tuple[int, Optional[int]]]:
        """(layer index, pass number or None) in execution order; a looped layer appears once per pass."""
        n = len(self.layers)
        if not self.loop:
            return [(i, None) for i in range(n)]
        a, b, t = self.loop["start"], self.loop["stop"], self.loop["times"]
        return ([(i, None) for i in range(a)] + [(i, p) for p in range(t) for i in range(a, b)] +
                [(i, None) for i in range(b, n)])

    def tensor_shapes(self) -> Dict[str, Tuple[int, ...]]:
        """Name -> shape of every tensor of a checkpoint of this configuration."""
        W, out = self.width, {}
        out["embed"] = (self.vocab_size, W)
        if self.loop:
            out["loop.in"] = (W, 2 * W)
            out["loop.step"] = (self.loop["times"], W)

        def lightning(p: str, c: dict) -> None:
            H, D, V = c["heads"], c["dim"], c["vdim"]
            out[p + "q"], out[p + "k"] = (H * D, W), (H * D, W)
            out[p + "v"], out[p + "g"] = (H * V, W), (H * V, W)
            out[p + "o"], out[p + "norm"] = (W, H * V), (H * V,)

        for i, l in enumerate(self.layers):
            p, c = f"l{i}.", l["mixer"]
            out[p + "norm1"], out[p + "norm1b"] = (W,), (W,)
            if l["type"] == "lightning":
                lightning(p + "mix.", c)
            elif l["type"] == "mamba2":
                H, P, N, G, K = c["heads"], c["vdim"], c["state"], c["groups"], c["conv"]
                inner, ch = H * P, H * P + 2 * G * N
                out[p + "mix.in"] = (2 * inner + 2 * G * N + H, W)
                out[p + "mix.conv"], out[p + "mix.conv.b"] = (ch, K), (ch,)
                out[p + "mix.dt_bias"], out[p + "mix.A_log"], out[p + "mix.D"] = (H,), (H,), (H,)
                out[p + "mix.norm"], out[p + "mix.o"] = (inner,), (W, inner)
            else:
                a = c["left"]
                H, G, D, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
                q = p + "mix.left."
                out[q + "q"], out[q + "q.b"] = (H * D, W), (H * D,)
                out[q + "k"], out[q + "k.b"] = (G * D, W), (G * D,)
                out[q + "v"], out[q + "v.b"] = (G * V, W), (G * V,)
                out[q + "q.norm"], out[q + "k.norm"] = (H * D,), (G * D,)
                out[q + "g"], out[q + "o"] = (H, W), (W, H * V)
                lightning(p + "mix.right.", c["right"])
            if l.get("mlp") is not None:
                F = l["mlp"]["ff"]
                out[p + "norm2"], out[p + "norm2b"] = (W,), (W,)
                out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = (F, W), (F, W), (W, F)
        out["final.norm"], out["head"] = (W,), (self.vocab_size, W)
        return out

    # ---- bytes, for the benchmarks' rooflines -------------------------------------------------------------------
    def weight_bytes_per_decode_step(self, elem: int = 2) -> int:
        sh = self.tensor_shapes()
        per_layer = {}
        for k, v in sh.items():
            if k.startswith("l") and k[1].isdigit():
                i = int(k[1:k.index(".")])
                per_layer[i] = per_layer.get(i, 0) + math.prod(v)
        total = sum(per_layer[i] for i, _ in self.runs())
        if self.loop:
            total += math.prod(sh["loop.in"]) * self.loop["times"]
        return elem * (total + math.prod(sh["head"]))

    def kv_bytes_per_token(self, elem: int = 2) -> int:
        n = 0
        for i, _ in self.runs():
            l = self.layers[i]
            if l["type"] == "parallel":
                a = l["mixer"]["left"]
                n += a["kv_heads"] * (a["dim"] + a["vdim"]) * elem
        return n

    def state_bytes_per_sequence(self) -> int:
        n = 0
        for i, _ in self.runs():
            l, c = self.layers[i], self.layers[i]["mixer"]
            if l["type"] == "lightning":
                n += c["heads"] * c["dim"] * c["vdim"] * 4
            elif l["type"] == "mamba2":
                n += c["heads"] * c["state"] * c["vdim"] * 4
                n += (c["conv"] - 1) * (c["heads"] * c["vdim"] + 2 * c["groups"] * c["state"]) * 4
            else:
                r = c["right"]
                n += r["heads"] * r["dim"] * r["vdim"] * 4
        return n


def _geometric_decays(heads: int) -> List[float]:
    lo, hi = math.log(1.0 - math.exp(-0.5)), math.log(1.0 - 0.999)
    return [1.0 - math.exp(lo + (hi - lo) * i / max(1, heads - 1)) for i in range(heads)]


def named_shape(name: str) -> Optional[Config]:
    """`random:safisun-<size>`: shapes whose layers resemble a real model's, for benchmarks (no checkpoint exists).
    `safisun-8b` / `safisun-1b` have the width, feed-forward size, head size, vocabulary and depth of the Llama 8B / 1B
    shapes: layers in the pattern mamba2, mamba2, parallel, lightning, each with a feed-forward."""
    key = name.lower()
    shapes = {"safisun-8b": (4096, 14336, 8, 128256), "safisun-1b": (2048, 8192, 4, 128256),
              "safisun-tiny": (256, 512, 1, 1024)}     # width, feed-forward, repeats of the 4-layer pattern, vocabulary
    if key not in shapes:
        return None
    W, F, groups, vocab = shapes[key]
    hd = 128 if W >= 4096 else 64
    heads = W // hd
    ffn = {"ff": F, "kind": "dense"}
    mamba = {"type": "mamba2", "mlp": ffn,
             "mixer": {"conv": 4, "groups": max(1, heads // 8), "heads": 2 * W // 64, "norm_groups": 1, "state": 128,
                       "vdim": 64}}
    par = {"type": "parallel", "mlp": ffn,
           "mixer": {"left": {"dim": hd, "heads": heads, "kv_heads": max(1, heads // 4), "mask": {"size": 2048},
                              "rot": {"base": 500000.0, "dims": hd // 2}, "scale": hd ** -0.5, "softcap": 50.0,
                              "vdim": hd},
                     "left_scale": 0.8, "right_scale": 1.1,
                     "right": {"decay": _geometric_decays(heads // 2), "dim": hd, "heads": heads // 2, "vdim": hd}}}
    lin = {"type": "lightning", "mlp": ffn,
           "mixer": {"decay": _geometric_decays(heads), "dim": hd, "heads": heads, "vdim": hd}}
    layers = [mamba, mamba, par, lin] * groups
    cfg = Config(name=key, vocab_size=vocab, width=W, eps=1e-5, layers=[json.loads(json.dumps(l)) for l in layers],
                 loop=None)
    cfg.validate()
    return cfg


# ---- weights ----------------------------------------------------------------------------------------------------------


class _Layer:
    """Device tensors of one layer in the layout the kernels read (fused where several matrices share an input)."""

    def __init__(self) -> None:
        self.kind = ""
        self.norm1 = self.norm1b = self.norm2 = self.norm2b = None
        self.w_in = self.w_o = None          # mixer: every projection of the mixer's input, stacked; output projection
        self.mix_norm = None                 # lightning / mamba2 / parallel.right
        self.decay = None                    # fp32 [heads] (lightning, parallel.right)
        self.conv = self.conv_b = self.dt_bias = self.a_log = self.skip = None       # mamba2
        self.bq = self.bk = self.bv = self.q_norm = self.k_norm = None               # parallel.left
        self.w_gu = self.w_down = None       # feed-forward: gate / up stacked (or interleaved, see `gu_interleaved`)
        self.gu_interleaved = False


class Weights:
    def __init__(self, cfg: Config, device: torch.device, dtype: torch.dtype):
        self.cfg, self.device, self.dtype = cfg, device, dtype
        self.embed = self.head = self.final_norm = self.loop_in = self.loop_step = None
        self.layers: List[_Layer] = []
        self.tp_size, self.tp_rank = 1, 0

    def nbytes(self) -> int:
        n = 0
        for t in [self.embed, self.head, self.final_norm, self.loop_in, self.loop_step] + [
                v for l in self.layers for v in vars(l).values()]:
            if isinstance(t, torch.Tensor):
                n += t.numel() * t.element_size()
        return n

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
        g = torch.Generator(device=device).manual_seed(1000 * seed + 7)

        class _Gen:
            def has(self, name):
                return name in shapes

            def shape(self, name):
                return shapes[name]

            def full(self, name):
                sh = shapes[name]
                leaf = name.rsplit(".", 1)[-1]
                if len(sh) == 2 and leaf != "conv" and name != "loop.step":
                    return torch.randn(sh, generator=g, device=device) * (sh[1] ** -0.5)
                if leaf == "conv":
                    return torch.randn(sh, generator=g, device=device) * 0.3
                if leaf.startswith("norm") or name.endswith(".norm"):
                    return 1.0 + 0.1 * torch.randn(sh, generator=g, device=device)
                if leaf == "A_log":
                    return torch.log(1.0 + 3.0 * torch.rand(sh, generator=g, device=device))
                if leaf == "dt_bias":
                    return -2.0 + torch.randn(sh, generator=g, device=device)
                if leaf == "D":
                    return 1.0 + 0.1 * torch.randn(sh, generator=g, device=device)
                return 0.1 * torch.randn(sh, generator=g, device=device)

        shapes = cfg.tensor_shapes()
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

        def lightning(l: _Layer, p: str, c: dict):
            return [get(p + "q"), get(p + "k"), get(p + "v"), get(p + "g")]

        W = cfg.width
        w.embed, w.head, w.final_norm = dev(get("embed")), dev(get("head")), dev(get("final.norm"))
        if cfg.loop:
            w.loop_in, w.loop_step = dev(get("loop.in")), dev(get("loop.step"))
        for i, spec in enumerate(cfg.layers):
            p, c, l = f"l{i}.", spec["mixer"], _Layer()
            l.kind = spec["type"]
            l.norm1, l.norm1b = dev(get(p + "norm1")), dev(get(p + "norm1b"))
            m = p + "mix."
            if l.kind == "lightning":
                l.w_in = dev(torch.cat(lightning(l, m, c), 0))
                l.w_o, l.mix_norm, l.decay = dev(get(m + "o")), dev(get(m + "norm")), f32(c["decay"])
            elif l.kind == "mamba2":
                l.w_in, l.w_o, l.mix_norm = dev(get(m + "in")), dev(get(m + "o")), dev(get(m + "norm"))
                l.conv, l.conv_b = dev(get(m + "conv")), dev(get(m + "conv.b"))
                l.dt_bias, l.a_log, l.skip = dev(get(m + "dt_bias")), dev(get(m + "A_log")), f32(get(m + "D").float())
            else:
                a = m + "left."
                l.w_in = dev(torch.cat([get(a + "q"), get(a + "k"), get(a + "v"), get(a + "g")] +
                                       lightning(l, m + "right.", c["right"]), 0))
                l.bq, l.bk, l.bv = dev(get(a + "q.b")), dev(get(a + "k.b")), dev(get(a + "v.b"))
                l.q_norm, l.k_norm = dev(get(a + "q.norm")), dev(get(a + "k.norm"))
                l.w_o = dev(torch.cat([get(a + "o"), get(m + "right.o")], 1))   # [left heads ; right heads] -> width
                l.mix_norm, l.decay = dev(get(m + "right.norm")), f32(c["right"]["decay"])
            if spec.get("mlp") is not None:
                F = spec["mlp"]["ff"]
                l.norm2, l.norm2b = dev(get(p + "norm2")), dev(get(p + "norm2b"))
                gate, up = get(p + "mlp.gate"), get(p + "mlp.up")
                if _use_tc(dtype, W) and F % 64 == 0:
                    from ..weights import interleave_gate_up

                    l.w_gu, l.gu_interleaved = dev(interleave_gate_up(gate, up)), True   # SwiGLU in the GEMM epilogue
                else:
                    l.w_gu = dev(torch.cat([gate, up], 0))
                l.w_down = dev(get(p + "mlp.down"))
            w.layers.append(l)
        return w


# ---- the layer program ------------------------------------------------------------------------------------------------


class Program:
    needs_seq_view = True     # kernels walk the step sequence by sequence (ModelRunner._stage_seq)
    graph_safe = True         # a sequence staged with no rows and no page slot is skipped by every stateful kernel

    def __init__(self, r) -> None:
        self.r = r
        cfg: Config = r.m
        w: Weights = r.w
        e = r.e
        self.cfg, self.w = cfg, w
        if e.tp_size != 1:
            raise ValueError("Safisun runs on one GPU per replica (no tensor-parallel split of the state mixers)")
        xt = w.dtype
        self.dt = _cabi.DT_F32 if xt == torch.float32 else _cabi.DT_BF16
        self.xt, self.esz = xt, (4 if xt == torch.float32 else 2)
        dev, T, lib = r.dev, r.Tmax, r.lib
        W = cfg.width
        f32 = torch.float32
        runs = cfg.runs()
        self.runs = runs
        # widest intermediate of any layer
        n_in = n_rec = n_mix = n_c = n_h = n_q = n_ff = 1
        for spec in cfg.layers:
            c = spec["mixer"]
            if spec["type"] == "lightning":
                hd, hv = c["heads"] * c["dim"], c["heads"] * c["vdim"]
                n_in, n_rec, n_mix = max(n_in, 2 * hd + 2 * hv), max(n_rec, hv), max(n_mix, hv)
            elif spec["type"] == "mamba2":
                inner, gn = c["heads"] * c["vdim"], c["groups"] * c["state"]
                n_in = max(n_in, 2 * inner + 2 * gn + c["heads"])
                n_rec, n_mix, n_c, n_h = max(n_rec, inner), max(n_mix, inner), max(n_c, inner + 2 * gn), max(n_h, c["heads"])
            else:
                a, b = c["left"], c["right"]
                hd, hv = b["heads"] * b["dim"], b["heads"] * b["vdim"]
                n_a = a["heads"] * a["dim"] + a["kv_heads"] * (a["dim"] + a["vdim"]) + a["heads"]
                n_in = max(n_in, n_a + 2 * hd + 2 * hv)
                n_rec, n_mix, n_q = max(n_rec, hv), max(n_mix, a["heads"] * a["vdim"] + hv), max(n_q, a["heads"] * a["dim"])
            if spec.get("mlp") is not None:
                n_ff = max(n_ff, spec["mlp"]["ff"])
        self.h = torch.zeros(T, W, dtype=f32, device=dev)          # residual stream
        self.y = torch.zeros(T, W, dtype=f32, device=dev)          # a sublayer's output before its post-norm
        self.proj = torch.zeros(T * n_in + 4, dtype=f32, device=dev)   # every projection of the mixer input, fused
        self.rec = torch.zeros(T * n_rec, dtype=f32, device=dev)   # recurrence output
        self.xbc = torch.zeros(T * n_c, dtype=f32, device=dev)
        self.dtb = torch.zeros(2, T * n_h, dtype=f32, device=dev)  # step sizes, decays
        self.gu = torch.zeros(T * 2 * n_ff, dtype=f32, device=dev)
        self.xn_flat = torch.zeros(T * max(W, 2 * W if cfg.loop else W), dtype=xt, device=dev)
        self.mix_flat = torch.zeros(T * n_mix, dtype=xt, device=dev)
        self.q_flat = torch.zeros(T * n_q, dtype=xt, device=dev)
        self.act_flat = torch.zeros(T * n_ff, dtype=xt, device=dev)
        self.xl = torch.zeros(r.Rmax, W, dtype=xt, device=dev)
        self.xn = self.xn_flat[:T * W].view(T, W)
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
            if l.w_gu is not None:
                d["gu"] = _Linear(lib, l.w_gu, self.xn, self.dt)
                d["down"] = _Linear(lib, l.w_down, view(self.act_flat, l.w_down.shape[1]), self.dt)
            self.lin.append(d)
        self.lin_head = _Linear(lib, w.head, self.xl, self.dt)
        self.lin_loop = None
        if cfg.loop:
            self.xcat = self.xn_flat[:T * 2 * W].view(T, 2 * W)
            self.lin_loop = _Linear(lib, w.loop_in, self.xcat, self.dt)

        # ---- pages and state slots: one set per layer RUN (a looped layer has one per pass) ------------------------
        bs = r.bs
        page_bytes = cfg.kv_bytes_per_token(self.esz) * bs
        if e.num_gpu_blocks is not None:
            nb = int(e.num_gpu_blocks)
        elif page_bytes == 0:
            nb = r.MB * r.Smax
        else:
            free, total = torch.cuda.mem_get_info(dev)
            budget = int(total * e.gpu_memory_utilization) - (total - free) - (512 << 20)
            budget -= cfg.state_bytes_per_sequence() * r.Smax
            nb = min(budget // page_bytes, r.MB * r.Smax)
            if nb < r.MB:
                raise RuntimeError(f"KV budget holds {nb} blocks; one sequence of max_model_len needs {r.MB}")
        r.num_blocks = nb
        r.block_bytes = page_bytes
        S = r.Smax
        self.kv: List[Optional[Tuple[torch.Tensor, torch.Tensor]]] = []
        self.state: List[Optional[torch.Tensor]] = []
        self.conv_state: List[Optional[torch.Tensor]] = []
        self.rot: Dict[Tuple[float, int], torch.Tensor] = {}
        for li, _ in runs:
            spec, c = cfg.layers[li], cfg.layers[li]["mixer"]
            kv = st = cs = None
            if spec["type"] == "lightning":
                st = torch.zeros(S, c["heads"], c["dim"], c["vdim"], dtype=f32, device=dev)
            elif spec["type"] == "mamba2":
                st = torch.zeros(S, c["heads"], c["state"], c["vdim"], dtype=f32, device=dev)
                ch = c["heads"] * c["vdim"] + 2 * c["groups"] * c["state"]
                cs = torch.zeros(S, max(1, c["conv"] - 1), ch, dtype=f32, device=dev)
            else:
                a, b = c["left"], c["right"]
                kv = (torch.zeros(nb, a["kv_heads"], bs, a["dim"], dtype=xt, device=dev),
                      torch.zeros(nb, a["kv_heads"], bs, a["vdim"], dtype=xt, device=dev))
                st = torch.zeros(S, b["heads"], b["dim"], b["vdim"], dtype=f32, device=dev)
                rot = a.get("rot") or {}
                key = (float(rot.get("base", 10000.0)), int(rot.get("dims", 0)))
                if key[1] and key not in self.rot:
                    self.rot[key] = rotation_table(key[0], key[1], e.max_model_len, dev)
            self.kv.append(kv)
            self.state.append(st)
            self.conv_state.append(cs)

    # ------------------------------------------------------------------------------------------------------------------
    def _lightning(self, l: _Layer, c: dict, proj: int, ld: int, off: int, state: torch.Tensor, out_ptr: int, ldo: int,
                   scale: float, T: int, n_dec: int, n_seqs: int, fl: int, st: int) -> int:
        """proj columns [off, ...): q | k | v | g of a lightning mixer; writes the normed, gated heads to out."""
        r, lib, ck, dp = self.r, self.r.lib, self.r._ck, self.r._dp
        H, D, V = c["heads"], c["dim"], c["vdim"]
        q, k, v, g = (proj + 4 * (off + o) for o in (0, H * D, 2 * H * D, 2 * H * D + H * V))
        n = self._scan(q, ld, k, ld, v, ld, H, H, D, V, l.decay.data_ptr(), None, None, None, 1, state.data_ptr(),
                       self.rec.data_ptr(), H * V, n_dec, n_seqs - n_dec, fl, st)
        ck(lib.atx_gated_norm(self.rec.data_ptr(), H * V, g, ld, l.mix_norm.data_ptr(), out_ptr, ldo, T, H * V, 1,
                              self.cfg.eps, 0, scale, self.dt, fl, st))
        return n + 1

    def _scan(self, q, ldq, k, ldk, v, ldv, H, G, D, V, decay_head, decay_tok, kscale_tok, skip, act, state, y, ldy,
              n_dec: int, n_pf: int, fl: int, st: int) -> int:
        """The decayed outer-product recurrence of one layer over the step's sequences: single decoded tokens (the first
        n_dec sequences) token by token on the FMA pipe; prompt portions in chunks on the tensor cores when the elements
        are bf16 and the kernel has the key size, else token by token as well."""
        lib, ck, dp = self.r.lib, self.r._ck, self.r._dp
        seqs = (dp["seq_start"], dp["seq_count"], dp["seq_pos0"], dp["seq_slot"])
        chunked = n_pf > 0 and self.xt == torch.bfloat16 and lib.atx_linear_recurrence_chunked_supported(D)
        n_seq = n_dec if chunked else n_dec + n_pf
        n = 0
        if n_seq:
            ck(lib.atx_linear_recurrence(q, ldq, k, ldk, v, ldv, H, G, D, V, decay_head, decay_tok, kscale_tok, skip, act,
                                         state, y, ldy, *seqs, n_seq, fl, st))
            n += 1
        if chunked:
            ck(lib.atx_linear_recurrence_chunked(q, ldq, k, ldk, v, ldv, H, G, D, V, decay_head, decay_tok, kscale_tok,
                                                 skip, act, state, y, ldy, *(p + 4 * n_dec for p in seqs), n_pf, fl, st))
            n += 1
        return n

    def forward(self, T: int, n_dec: int, n_pf: int, n_rows: int) -> int:
        """Issue every kernel of one step on the current stream; returns the launch count. The step's first n_dec
        sequences are single decoded tokens (rows 0 .. n_dec-1), the next n_pf are prompt portions."""
        r, cfg, w = self.r, self.cfg, self.w
        n_seqs = n_dec + n_pf
        lib, ck, dp, fl, dt = r.lib, r._ck, r._dp, r.flags, self.dt
        st = torch.cuda.current_stream().cuda_stream
        W, V, eps = cfg.width, cfg.vocab_size, cfg.eps
        h, y, xn = self.h.data_ptr(), self.y.data_ptr(), self.xn.data_ptr()
        proj = self.proj.data_ptr()
        n = 0
        ck(lib.atx_embed_rows(dp["ids"], w.embed.data_ptr(), h, T, W, V, dt, fl, st))
        n += 1
        pending = None     # post-norm weight of the sublayer output waiting in y
        probe = r.layer_probe
        small = T <= 64    # decode-sized: split-K GEMMs accumulate into buffers that the norm kernels hand back cleared
        if small:
            self.y[:T].zero_()

        def resid(w_pre, out_ptr, vec=None, rows=None, rows_n: int = T, zero_ptr=None, zero_bytes: int = 0) -> None:
            nonlocal n, pending
            have = pending is not None
            ck(lib.atx_resid_norm(h, y if have else None, pending, vec, w_pre, out_ptr, rows, rows_n, W, eps,
                                  1 if (have and rows is None and small) else 0, zero_ptr, zero_bytes, dt, fl, st))
            n += 1
            if rows is None:
                pending = None

        for ri, (li, p) in enumerate(self.runs):
            spec, c, l, lin = cfg.layers[li], cfg.layers[li]["mixer"], w.layers[li], self.lin[li]
            vec = None
            if p is not None and li == cfg.loop["start"]:
                if pending is not None:
                    resid(None, None)
                ck(lib.atx_concat_embed(h, dp["ids"], w.embed.data_ptr(), self.xcat.data_ptr(), T, W, V, dt, fl, st))
                self.lin_loop.run(h, W, T, fl, st)
                n += 2
                vec = w.loop_step.data_ptr() + p * W * self.esz
            ld = l.w_in.shape[0]
            acc = lin["in"].accumulates(T)
            resid(l.norm1.data_ptr(), xn, vec=vec, zero_ptr=proj if acc else None,
                  zero_bytes=(T * ld * 4 + 15) // 16 * 16 if acc else 0)
            lin["in"].run(proj, ld, T, fl, st, zeroed=acc)
            n += 1
            K_o = l.w_o.shape[1]
            mix = self.mix_flat.data_ptr()
            if l.kind == "lightning":
                n += self._lightning(l, c, proj, ld, 0, self.state[ri], mix, K_o, 1.0, T, n_dec, n_seqs, fl, st)
            elif l.kind == "mamba2":
                H, P, N, G, K = c["heads"], c["vdim"], c["state"], c["groups"], c["conv"]
                inner, ch = H * P, H * P + 2 * G * N
                xbc, dts, dec = self.xbc.data_ptr(), self.dtb[0].data_ptr(), self.dtb[1].data_ptr()
                cs = self.conv_state[ri].data_ptr()
                ck(lib.atx_conv_dt(proj, ld, inner, inner + ch, l.conv.data_ptr(), l.conv_b.data_ptr(),
                                   l.dt_bias.data_ptr(), l.a_log.data_ptr(), cs, xbc, dts, dec, dp["tok_seq"],
                                   dp["seq_start"], dp["seq_pos0"], dp["seq_slot"], T, ch, H, K, dt, fl, st))
                ck(lib.atx_conv_state_update(proj, ld, inner, cs, dp["seq_start"], dp["seq_count"], dp["seq_pos0"],
                                             dp["seq_slot"], n_seqs, ch, K, fl, st))
                n += self._scan(xbc + 4 * (inner + G * N), ch, xbc + 4 * inner, ch, xbc, ch, H, G, N, P, None, dec, dts,
                                l.skip.data_ptr(), 0, self.state[ri].data_ptr(), self.rec.data_ptr(), inner, n_dec, n_pf,
                                fl, st)
                ck(lib.atx_gated_norm(self.rec.data_ptr(), inner, proj, ld, l.mix_norm.data_ptr(), mix, K_o, T, inner,
                                      c["norm_groups"], eps, 1, 1.0, dt, fl, st))
                n += 3 if K > 1 else 2
            else:
                a, b = c["left"], c["right"]
                H, G, D, Vd = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
                o_k, o_v, o_g = H * D, H * D + G * D, H * D + G * D + G * Vd
                o_right = o_g + H
                rot = a.get("rot") or {}
                rd = int(rot.get("dims", 0))
                table = self.rot[(float(rot.get("base", 10000.0)), rd)].data_ptr() if rd else None
                kc, vc = self.kv[ri]
                q = self.q_flat.data_ptr()
                ck(lib.atx_qk_prepare(proj, ld, 0, o_k, o_v, l.bq.data_ptr(), l.bk.data_ptr(), l.bv.data_ptr(),
                                      l.q_norm.data_ptr(), l.k_norm.data_ptr(), table, rd, dp["pos"], dp["slots"], q,
                                      kc.data_ptr(), vc.data_ptr(), T, H, G, D, Vd, r.bs, eps, dt, fl, st))
                chunk = int((a.get("mask") or {}).get("size", 0) or 0)
                # prompt portions on the tensor cores where the head sizes have such a kernel; single tokens (and every
                # row otherwise) on the one-warp-per-row kernel
                tc = n_pf > 0 and lib.atx_attn_local_prefill_supported(D, Vd, dt)
                t_rows = n_dec if tc else T
                args = (H, G, D, Vd, r.bs, float(a["scale"]), float(a.get("softcap") or 0.0), chunk, 1,
                        float(c["left_scale"]), dt, fl, st)
                if t_rows:
                    ck(lib.atx_attn_local(q, kc.data_ptr(), vc.data_ptr(), dp["seq_bt"], r.MB, dp["tok_seq"], dp["pos"],
                                          proj + 4 * o_g, ld, mix, K_o, t_rows, *args))
                    n += 1
                if tc:
                    ck(lib.atx_attn_local_prefill(q, kc.data_ptr(), vc.data_ptr(), dp["seq_bt"] + 4 * n_dec * r.MB, r.MB,
                                                  dp["seq_start"] + 4 * n_dec, dp["seq_count"] + 4 * n_dec,
                                                  dp["seq_pos0"] + 4 * n_dec, n_pf, T - n_dec, proj + 4 * o_g, ld, mix,
                                                  K_o, *args))
                    n += 1
                n += 1
                n += self._lightning(l, b, proj, ld, o_right, self.state[ri], mix + H * Vd * self.esz, K_o,
                                     float(c["right_scale"]), T, n_dec, n_seqs, fl, st)
            lin["o"].run(y, W, T, fl, st, zeroed=small)
            n += 1
            pending = l.norm1b.data_ptr()
            if l.w_gu is not None:
                resid(l.norm2.data_ptr(), xn)
                F = l.w_down.shape[1]
                act = self.act_flat.data_ptr()
                if l.gu_interleaved:
                    lin["gu"].run(act, F, T, fl, st, mode=_cabi.GEMM_SWIGLU_BF16)
                    n += 1
                else:
                    lin["gu"].run(self.gu.data_ptr(), 2 * F, T, fl, st)
                    ck(lib.atx_gated_act(self.gu.data_ptr(), act, T, F, dt, fl, st))
                    n += 2
                lin["down"].run(y, W, T, fl, st, zeroed=small)
                n += 1
                pending = l.norm2b.data_ptr()
            if probe is not None:
                resid(None, None)
                probe.append(self.h[:T].clone())
        if n_rows:
            resid(w.final_norm.data_ptr(), self.xl.data_ptr(), rows=dp["rows"], rows_n=n_rows)
            self.lin_head.run(r.logits.data_ptr(), V, n_rows, fl, st)
            ck(lib.atx_sample(r.logits.data_ptr(), V, dp["temps"], dp["top_p"], dp["seeds"], dp["steps"],
                              r.out_ids.data_ptr(), n_rows, V, fl, st))
            n += 2
        return n
