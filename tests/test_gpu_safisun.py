"""The Safisun family on the GPU against the float64 reference (oracle/safisun_ref.py): kernels alone on inputs built
so that a lost key, a wrong block edge or a dropped state shows, and the engine (scheduler, pages, state slots,
runner, kernels) on small random models: whole prompts, token-by-token decoding, portions, mixed batches, reuse of
pages and slots, greedy generation through the ordinary entry point."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import safisun_ref as R

pytestmark = pytest.mark.gpu
F64 = torch.float64
DEV = "cuda:0"


# ---- small models ------------------------------------------------------------------------------------------------------

def lightning_layer(heads=3, dim=8, vdim=12, mlp=None, decay=None):
    return {"type": "lightning", "mlp": mlp,
            "mixer": {"decay": decay or [0.5, 0.9, 0.995][:heads], "dim": dim, "heads": heads, "vdim": vdim}}


def mamba_layer(heads=4, vdim=10, state=8, groups=2, norm_groups=2, conv=3, mlp=None):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups, "state": state, "vdim": vdim}}


def parallel_layer(mlp=None, size=8, rot_dims=8, dim=16, vdim=12, heads=4, kv=2):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": {"dim": dim, "heads": heads, "kv_heads": kv, "mask": {"size": size},
                               "rot": {"base": 100.0, "dims": rot_dims}, "scale": 0.3, "softcap": 5.0, "vdim": vdim},
                      "left_scale": 0.7, "right_scale": 1.3,
                      "right": {"decay": [0.8, 0.97], "dim": 12, "heads": 2, "vdim": 6}}}


def model_cfg(layers, width=64, vocab=96, loop=None):
    return {"architecture": "Safisun", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": layers, "loop": loop}


def loop_model(width=64):
    ff = {"ff": 64, "kind": "dense"}
    return model_cfg([lightning_layer(), mamba_layer(mlp={"ff": 40, "kind": "dense"}), parallel_layer(mlp=ff),
                      lightning_layer(heads=2, dim=16, vdim=8, decay=[0.7, 0.999])],
                     width=width, loop={"start": 1, "stop": 3, "times": 2})


def engine(cfg, wt, dtype="float32", **kw):
    from atx.config import EngineConfig, ModelSource
    from atx.engine import LLMEngine
    from atx.models import safisun

    mcfg = safisun.Config.from_json(cfg)
    xt = torch.float32 if dtype == "float32" else torch.bfloat16
    w = safisun.Weights.from_state_dict(mcfg, wt, torch.device(DEV), xt)
    ecfg = EngineConfig(max_model_len=kw.pop("max_model_len", 256), max_num_seqs=kw.pop("max_num_seqs", 4),
                        max_num_batched_tokens=kw.pop("max_num_batched_tokens", 256),
                        num_gpu_blocks=kw.pop("num_gpu_blocks", 64), enable_prefix_caching=False,
                        enable_cuda_graphs=kw.pop("enable_cuda_graphs", False),
                        async_scheduling=kw.pop("async_scheduling", False), dtype=dtype,
                        max_logit_rows=kw.pop("max_logit_rows", 256), **kw)
    return LLMEngine(ModelSource(mcfg, None, None), ecfg, w)


def tokens(n, vocab=96, seed=0):
    return [int(t) for t in torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed))]


def rel_rows(got, want):
    """Per row: rms(got - want) / rms(want), both with the row mean taken off."""
    got, want = torch.as_tensor(got, dtype=F64), torch.as_tensor(want, dtype=F64)
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt()


def rel(got, want):
    """Worst row of rel_rows."""
    return float(rel_rows(got, want).max())


TOL = {"float32": 2e-5, "bfloat16": 0.15}      # bf16: operand rounding through up to seven layer runs; fp32 is the sharp test


def whole(eng, rid, toks, end=True):
    return eng.feed([(rid, toks, list(range(len(toks))))], [rid] if end else [])


# ---- each mechanism alone, through the engine ------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [64, 96])       # 96: not a multiple of the tensor-core GEMM's K block
@pytest.mark.parametrize("kind", ["lightning", "mamba2", "parallel", "parallel_full", "parallel_tc", "lightning_ffn"])
def test_one_layer_models(kind, width, dtype):
    layer = {"lightning": lightning_layer(), "mamba2": mamba_layer(),
             "parallel": parallel_layer(), "parallel_full": parallel_layer(size=None, rot_dims=16, kv=4),
             "parallel_tc": parallel_layer(size=24, rot_dims=32, dim=64, vdim=64, heads=4, kv=2),   # tensor-core head sizes
             "lightning_ffn": lightning_layer(heads=1, dim=4, vdim=4, decay=[0.9], mlp={"ff": 24, "kind": "dense"})}[kind]
    if kind == "parallel_full":
        layer["mixer"]["left"]["mask"] = None
        layer["mixer"]["left"]["softcap"] = None
    cfg = model_cfg([layer], width=width)
    wt = R.random_checkpoint(cfg, 11)
    toks = tokens(150 if kind == "parallel_tc" else 45, seed=1)
    eng = engine(cfg, wt, dtype)
    got = whole(eng, "a", toks)
    want = R.forward(cfg, wt, toks)
    assert rel(got, want) < TOL[dtype]
    if kind == "parallel_tc":      # portions that start inside a block and inside a 64-row tile, beside a decoded token
        a = eng.feed([("p", toks[:70], list(range(70)))], [])
        b = eng.feed([("p", toks[70:71], [0]), ("q", toks[:131], list(range(131)))], ["q"])
        c = eng.feed([("p", toks[71:], list(range(79)))], ["p"])
        assert rel(np.concatenate([a, b[:1], c]), want) < TOL[dtype] and rel(b[1:], want[:131]) < TOL[dtype]


def test_first_tokens_of_a_sequence():
    cfg = loop_model()
    wt = R.random_checkpoint(cfg, 3)
    eng = engine(cfg, wt)
    for n in (1, 2, 3):
        toks = tokens(n, seed=n)
        assert rel(whole(eng, f"r{n}", toks), R.forward(cfg, wt, toks)) < TOL["float32"]


# ---- the same logits however the tokens are cut ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_token_by_token_and_portions_agree(dtype):
    cfg = loop_model()
    wt = R.random_checkpoint(cfg, 4)
    toks = tokens(70, seed=5)
    want = R.forward(cfg, wt, toks)
    eng = engine(cfg, wt, dtype)
    a = whole(eng, "w", toks)
    b = np.concatenate([eng.feed([("t", toks[i:i + 1], [0])], ["t"] if i == len(toks) - 1 else []) for i in range(len(toks))])
    cuts, parts, at = [2, 3, 16, 1, 7, 2, 9, 1, 1, 17, 2], [], 0
    cuts.append(len(toks) - sum(cuts))
    for n in cuts:
        parts.append(eng.feed([("p", toks[at:at + n], list(range(n)))], ["p"] if at + n == len(toks) else []))
        at += n
    c = np.concatenate(parts)
    for got in (a, b, c):
        assert rel(got, want) < TOL[dtype]
    if dtype == "float32":
        assert rel(b, a) < 1e-5 and rel(c, a) < 1e-5


def test_long_decoding_keeps_its_state():
    cfg = loop_model()
    wt = R.random_checkpoint(cfg, 6)
    toks = tokens(200, seed=7)
    eng = engine(cfg, wt)
    got = [eng.feed([("d", toks[:9], list(range(9)))], [])]
    got += [eng.feed([("d", toks[i:i + 1], [0])], []) for i in range(9, len(toks))]
    assert rel(np.concatenate(got), R.forward(cfg, wt, toks)) < TOL["float32"]


def test_mixed_batches_equal_each_request_alone():
    cfg = loop_model()
    wt = R.random_checkpoint(cfg, 8)
    reqs = {"a": tokens(61, seed=1), "b": tokens(23, seed=2), "c": tokens(40, seed=3), "d": tokens(5, seed=4)}
    want = {k: R.forward(cfg, wt, v) for k, v in reqs.items()}
    # portions of some requests beside single tokens of others; c joins late, d comes and goes in the middle
    steps = [[("a", 17), ("b", 2)], [("a", 1), ("b", 19)], [("a", 30), ("b", 1), ("c", 3)], [("b", 1), ("c", 1), ("d", 5)],
             [("a", 13), ("c", 20)], [("c", 1)], [("c", 15)]]
    eng = engine(cfg, wt, max_num_seqs=4)
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    for step in steps:
        entries, end = [], []
        for k, n in step:
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        out = eng.feed(entries, end)
        o = 0
        for k, n in step:
            got[k].append(out[o:o + n])
            o += n
    assert at == {k: len(v) for k, v in reqs.items()}
    for k in reqs:
        assert rel(np.concatenate(got[k]), want[k]) < TOL["float32"], k
    assert eng.allocator.num_free == eng.allocator.num_blocks and eng.state_slots.num_free == 4


def tensor_core_sized_model():
    """Key sizes the chunked tensor-core recurrence (32 / 64) and the tensor-core attention (64) accept, so that bf16
    prompt portions take those kernels and single tokens the token-by-token ones, on the same pages and state slots."""
    ff = {"ff": 96, "kind": "dense"}
    return model_cfg([mamba_layer(heads=4, vdim=16, state=64, groups=2, norm_groups=2, conv=4, mlp=ff),
                      parallel_layer(mlp=ff, size=24, rot_dims=16, dim=64, vdim=64, heads=4, kv=2),
                      lightning_layer(heads=3, dim=32, vdim=24)], width=128, loop={"start": 0, "stop": 2, "times": 2})


def test_bf16_portions_on_the_tensor_cores_beside_single_tokens():
    """Mixed steps in bf16 where prompt portions run on the chunked recurrence and the tensor-core attention while the
    single tokens beside them run token by token: the per-sequence lists handed to the two kernel families start at
    different offsets of the same step. Portions cross the 64-token chunk of the recurrence and the 24-token block of
    the mask; each request is compared with the float64 reference and with itself run alone."""
    cfg = tensor_core_sized_model()
    wt = R.random_checkpoint(cfg, 15)
    reqs = {"a": tokens(150, seed=1), "b": tokens(90, seed=2), "c": tokens(70, seed=3), "d": tokens(6, seed=5)}
    want = {k: R.forward(cfg, wt, v) for k, v in reqs.items()}
    steps = [[("a", 70), ("b", 2)], [("a", 1), ("b", 65)], [("a", 1), ("b", 1), ("c", 63)], [("a", 64), ("b", 1), ("c", 1),
             ("d", 6)], [("b", 21), ("c", 2), ("a", 1)], [("a", 13), ("c", 4)]]
    eng = engine(cfg, wt, "bfloat16", max_num_seqs=4, max_model_len=160, max_num_batched_tokens=512)
    lib, _ = _lib()
    assert lib.atx_linear_recurrence_chunked_supported(64) and lib.atx_attn_local_prefill_supported(64, 64, 0)
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    for step in steps:
        entries, end = [], []
        for k, n in step:
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        out = eng.feed(entries, end)
        o = 0
        for k, n in step:
            got[k].append(out[o:o + n])
            o += n
    assert at == {k: len(v) for k, v in reqs.items()}
    # A looped model with a norm after every sublayer has rows that magnify bf16 rounding several times over (the
    # float64 reference itself moves by 0.3 on some rows when its weights get bf16-sized noise), so rows are judged
    # together: a wrong offset, slot or page spoils whole requests, not one row in twenty.
    for k in reqs:
        mixed = np.concatenate(got[k])
        alone = whole(eng, k + "-alone", reqs[k])
        for other in (want[k], alone):
            r = rel_rows(mixed, other)
            assert float(r.median()) < 0.04 and float(r.quantile(0.9)) < 0.15 and float(r.max()) < 0.6, (k, r.max())
    assert eng.allocator.num_free == eng.allocator.num_blocks and eng.state_slots.num_free == 4


def test_pages_and_slots_are_reused_without_leaking_state():
    cfg = loop_model()
    wt = R.random_checkpoint(cfg, 9)
    eng = engine(cfg, wt, max_num_seqs=2, num_gpu_blocks=6, max_model_len=96)       # 96 tokens of pages, two slots
    first = tokens(90, seed=1)
    whole(eng, "big", first)                                   # fills every page and leaves a large state in slot 0
    for seed, n in ((2, 33), (3, 50), (4, 17)):
        toks = tokens(n, seed=seed)
        assert rel(whole(eng, f"r{seed}", toks), R.forward(cfg, wt, toks)) < TOL["float32"]
    # a request that starts while another is alive takes the freed slot and freed pages
    a, b, c = tokens(40, seed=5), tokens(30, seed=6), tokens(36, seed=7)
    ab = eng.feed([("a", a[:20], list(range(20))), ("b", b, list(range(30)))], ["b"])
    ga = [ab[:20]]
    assert rel(ab[20:], R.forward(cfg, wt, b)) < TOL["float32"]
    gc = eng.feed([("a", a[20:21], [0]), ("c", c, list(range(36)))], ["c"])
    ga += [gc[:1], eng.feed([("a", a[21:], list(range(19)))], ["a"])]
    assert rel(np.concatenate(ga), R.forward(cfg, wt, a)) < TOL["float32"]
    assert rel(gc[1:], R.forward(cfg, wt, c)) < TOL["float32"]
    with pytest.raises(Exception):
        eng.feed([("x", tokens(97, seed=8), [])], [])          # more pages than the pool has


def test_other_sizes():
    ff = {"ff": 72, "kind": "dense"}
    cfg = model_cfg([mamba_layer(heads=6, vdim=4, state=20, groups=3, norm_groups=1, conv=5, mlp=ff),
                     parallel_layer(size=5, rot_dims=2, dim=6, vdim=40, heads=6, kv=1),
                     lightning_layer(heads=1, dim=40, vdim=3, decay=[0.93])],
                    width=80, vocab=53, loop={"start": 0, "stop": 2, "times": 3})
    wt = R.random_checkpoint(cfg, 12)
    toks = tokens(37, vocab=53, seed=2)
    want = R.forward(cfg, wt, toks)
    for dtype in ("float32", "bfloat16"):
        eng = engine(cfg, wt, dtype)
        got = np.concatenate([eng.feed([("s", toks[:20], list(range(20)))], []),
                              eng.feed([("s", toks[20:22], [0, 1])], [])] +
                             [eng.feed([("s", toks[i:i + 1], [0])], []) for i in range(22, 37)])
        assert rel(got, want) < TOL[dtype], dtype


_FF = {"ff": 72, "kind": "dense"}
ODD_MODELS = {
    "no_loop": lambda: model_cfg([mamba_layer(), parallel_layer(mlp=_FF), lightning_layer()], loop=None),
    "loop_once_over_everything": lambda: model_cfg([mamba_layer(), parallel_layer(mlp=_FF), lightning_layer()],
                                                   loop={"start": 0, "stop": 3, "times": 1}),
    "loop_at_the_tail": lambda: model_cfg([lightning_layer(), mamba_layer(mlp=_FF), parallel_layer()],
                                          loop={"start": 2, "stop": 3, "times": 3}),
    "two_taps_four_groups": lambda: model_cfg([mamba_layer(heads=8, vdim=8, state=16, groups=4, norm_groups=4, conv=2),
                                               lightning_layer()]),
    "one_tap": lambda: model_cfg([mamba_layer(heads=2, vdim=8, state=16, groups=1, norm_groups=1, conv=1, mlp=_FF)]),
    "eight_taps": lambda: model_cfg([mamba_layer(heads=2, vdim=8, state=32, groups=2, norm_groups=1, conv=8, mlp=_FF)]),
    "every_head_its_own_kv_whole_head_rotated": lambda: model_cfg([parallel_layer(heads=4, kv=4, dim=16, vdim=16,
                                                                                  rot_dims=16, size=7)]),
    "blocks_of_one": lambda: model_cfg([parallel_layer(size=1), lightning_layer()]),
    "block_larger_than_the_prompt": lambda: model_cfg([parallel_layer(size=4096, mlp=_FF)]),
    "tensor_core_key_size_other_value_size": lambda: model_cfg([parallel_layer(heads=2, kv=1, dim=128, vdim=64, rot_dims=64,
                                                                               size=40, mlp=_FF)], width=128),
    "value_wider_than_key": lambda: model_cfg([parallel_layer(heads=4, kv=2, dim=64, vdim=128, rot_dims=32, size=100)],
                                              width=128),
    "heads_of_256": lambda: model_cfg([parallel_layer(heads=2, kv=1, dim=256, vdim=32, rot_dims=128, size=33),
                                       lightning_layer(heads=2, dim=256, vdim=16, decay=[0.9, 0.99])], width=128),
    "chunked_scan_96_keys_odd_values": lambda: model_cfg(
        [lightning_layer(heads=2, dim=96, vdim=20, decay=[0.9, 0.999]),
         mamba_layer(heads=6, vdim=12, state=128, groups=3, norm_groups=2, conv=4)], width=128),
    "width_not_a_gemm_block": lambda: model_cfg([mamba_layer(), parallel_layer(mlp=_FF), lightning_layer()], width=72, vocab=77),
    "one_head_one_rotated_pair": lambda: model_cfg([lightning_layer(heads=1, dim=32, vdim=32, decay=[0.97]),
                                                    parallel_layer(heads=1, kv=1, dim=64, vdim=64, rot_dims=2, size=16)]),
}


@pytest.mark.parametrize("name", sorted(ODD_MODELS))
def test_odd_configurations_whole_and_in_portions(name):
    """Sizes on both sides of every kernel's fast path, each in fp32 and bf16: the whole prompt in one step, and cut into
    70 | 2 | 1 | 1 | 64 | 3 | rest (a prompt-sized portion continues from single tokens and the other way round)."""
    cfg = ODD_MODELS[name]()
    wt = R.random_checkpoint(cfg, 3)
    toks = tokens(150, vocab=cfg["vocab"], seed=9)
    want = R.forward(cfg, wt, toks)
    for dtype in ("float32", "bfloat16"):
        eng = engine(cfg, wt, dtype, max_model_len=160, max_num_batched_tokens=512)
        a = whole(eng, "w", toks)
        cuts = [70, 2, 1, 1, 64, 3]
        cuts.append(len(toks) - sum(cuts))
        parts, at = [], 0
        for n in cuts:
            parts.append(eng.feed([("p", toks[at:at + n], list(range(n)))], ["p"] if at + n == len(toks) else []))
            at += n
        b = np.concatenate(parts)
        lim = 3e-5 if dtype == "float32" else 0.3      # bf16 operands through up to seven layer runs; fp32 is the sharp test
        assert np.isfinite(a).all() and np.isfinite(b).all(), dtype
        assert rel(a, want) < lim and rel(b, want) < lim, (dtype, rel(a, want), rel(b, want))
        eng.runner.close()


def drawn_model(rng):
    """A model whose layer order, sizes, constants and looped block are drawn at random from sizes a real model could
    have (key sizes on and off the tensor-core paths, widths on and off the GEMM's block, odd vocabularies)."""
    def decays(h):
        return [rng.choice([0.5, 0.61, 0.82, 0.92, 0.97, 0.988, 0.999, 0.9999]) for _ in range(h)]

    def lightning():
        h = rng.choice([1, 2, 3, 4, 6, 8])
        return {"decay": decays(h), "dim": rng.choice([16, 32, 48, 64, 96, 128]), "heads": h,
                "vdim": rng.choice([16, 24, 32, 48, 64, 128])}

    def mamba():
        g = rng.choice([1, 2, 4])
        h = g * rng.choice([1, 2, 3])
        return {"conv": rng.choice([2, 3, 4, 5]), "groups": g, "heads": h,
                "norm_groups": rng.choice([x for x in (1, 2, 3, 4, 6) if h % x == 0]),
                "state": rng.choice([16, 32, 64, 128]), "vdim": rng.choice([16, 32, 48, 64])}

    def softmax_side():
        kv = rng.choice([1, 2, 4])
        d = rng.choice([32, 64, 96, 128])
        return {"dim": d, "heads": kv * rng.choice([1, 2, 3, 4]), "kv_heads": kv,
                "mask": {"size": rng.choice([16, 32, 48, 64, 100, 128])},
                "rot": {"base": rng.choice([1e4, 5e5, 1e6]), "dims": rng.choice([x for x in (2, 16, 32, 64, 128) if x <= d])},
                "scale": rng.choice([d ** -0.5, 0.05, 0.2]), "softcap": rng.choice([20.0, 30.0, 50.0]),
                "vdim": rng.choice([32, 64, 128, d])}

    def layer(kind):
        mixer = {"lightning": lightning, "mamba2": mamba,
                 "parallel": lambda: {"left": softmax_side(), "left_scale": rng.choice([0.5, 0.8, 1.0]),
                                      "right": lightning(), "right_scale": rng.choice([1.0, 1.1, 0.6])}}[kind]()
        return {"type": kind, "mixer": mixer, "mlp": rng.choice([None, {"ff": rng.choice([128, 192, 320, 500]), "kind": "dense"}])}

    n = rng.randint(3, 6)
    kinds = ["lightning", "mamba2", "parallel"] + [rng.choice(["lightning", "mamba2", "parallel"]) for _ in range(n - 3)]
    rng.shuffle(kinds)
    a = rng.randint(0, n - 1)
    loop = rng.choice([None, {"start": a, "stop": rng.randint(a + 1, n), "times": rng.choice([1, 2, 3])}])
    cfg = model_cfg([layer(k) for k in kinds], width=rng.choice([64, 128, 160, 192, 256, 320]),
                    vocab=rng.choice([256, 320, 500, 1000, 1027]), loop=loop)
    cfg["norm"]["eps"] = rng.choice([1e-5, 1e-6])
    return cfg


@pytest.mark.parametrize("draw", range(8))
def test_drawn_models_whole_cut_and_mixed(draw):
    """Three unequal requests of a drawn model: each whole, the longest in portions with its last tokens one by one, then
    all three in steps where a request may bring a portion, one token or nothing. fp32 is held to rounding on every row;
    bf16 to its typical row (single rows of a random model are ill-conditioned by factors of ten to twenty in both types)."""
    import random
    rng = random.Random(4000 + draw)
    cfg = drawn_model(rng)
    wt = R.random_checkpoint(cfg, 70 + draw)
    V = cfg["vocab"]
    reqs = {"a": tokens(rng.randint(150, 330), V, draw), "b": tokens(rng.randint(70, 200), V, draw + 100),
            "c": tokens(rng.randint(2, 90), V, draw + 200)}
    want = {k: R.forward(cfg, wt, v) for k, v in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        eng = engine(cfg, wt, dtype, max_model_len=384, max_num_batched_tokens=1024, max_logit_rows=1024, num_gpu_blocks=48)
        rows = [rel_rows(eng.feed([(k, v, list(range(len(v))))], [k]), want[k]) for k, v in reqs.items()]
        v, at, parts = reqs["a"], 0, []
        while at < len(v):
            n = 1 if len(v) - at <= 40 else min(rng.choice([2, 3, 7, 64, 65, 100, 130]), len(v) - at - 40)
            parts.append(eng.feed([("a", v[at:at + n], list(range(n)))], ["a"] if at + n == len(v) else []))
            at += n
        rows.append(rel_rows(np.concatenate(parts), want["a"]))
        pos, got, live = {k: 0 for k in reqs}, {k: [] for k in reqs}, ["a", "b", "c"]
        while live:
            entries, end, taken = [], [], []
            for k in list(live):
                if len(live) > 1 and rng.random() < 0.25:
                    continue                                   # left out of this step, goes on later
                n = min(len(reqs[k]) - pos[k], rng.choice([1, 1, 1, 2, 5, 31, 64, 90]))
                entries.append((k, reqs[k][pos[k]:pos[k] + n], list(range(n))))
                taken.append((k, n))
                pos[k] += n
                if pos[k] == len(reqs[k]):
                    end.append(k)
                    live.remove(k)
            if entries:
                out, o = eng.feed(entries, end), 0
                for k, n in taken:
                    got[k].append(out[o:o + n])
                    o += n
        rows += [rel_rows(np.concatenate(got[k]), want[k]) for k in reqs]
        assert eng.allocator.num_free == eng.allocator.num_blocks and eng.state_slots.num_free == 4
        r = torch.cat(rows)
        assert torch.isfinite(r).all(), dtype
        if dtype == "float32":
            assert float(r.max()) < 1e-4 and float(r.median()) < 5e-6, (float(r.max()), float(r.median()))
        else:
            assert float(r.max()) < 0.6 and float(r.median()) < 0.03, (float(r.max()), float(r.median()))
        eng.runner.close()


# ---- generation through the ordinary entry point ---------------------------------------------------------------------------

@pytest.mark.parametrize("mode", ["plain", "chunked_prefill", "async", "graphs"])
def test_greedy_generation_matches_the_reference(mode):
    from atx.scheduler import SamplingParams

    cfg = loop_model()
    wt = R.random_checkpoint(cfg, 13)
    prompts = [tokens(37, seed=1), tokens(5, seed=2), tokens(64, seed=3)]
    kw = {"plain": {}, "chunked_prefill": {"max_num_batched_tokens": 16}, "async": {"async_scheduling": True},
          "graphs": {"async_scheduling": True, "enable_cuda_graphs": True}}[mode]
    eng = engine(cfg, wt, **kw)
    outs = eng.generate_sync(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        lg = R.forward(cfg, wt, p + o[:-1])[len(p) - 1:]
        top2 = lg.topk(2, dim=-1).values
        for i, tok in enumerate(o):            # teacher-forced: every token is the reference's arg-max (ties aside)
            assert tok == int(lg[i].argmax()) or float(top2[i, 0] - top2[i, 1]) < 1e-4, (mode, i)
    assert eng.allocator.num_free == eng.allocator.num_blocks and eng.state_slots.num_free == eng.state_slots.num_slots


# ---- kernels alone, on inputs where one wrong key or a lost state shows ----------------------------------------------------

def _lib():
    from atx import _cabi

    return _cabi.load(), _cabi


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _st():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("size,n", [(8, 41), (16, 50), (0, 37)])
def test_attention_block_edges_with_dominant_keys(size, n):
    """Every block's first and last key carry a score far above the rest and a value of their own: a query that sees
    one key too many or too few lands on a different value. Rows are also run one at a time (decode form) over pages
    in scrambled order."""
    lib, cabi = _lib()
    H, G, D, Vd, bs = 4, 2, 8, 6, 16
    g = torch.Generator().manual_seed(size + n)
    q = torch.randn(n, H, D, generator=g, dtype=F64)
    k = 0.2 * torch.randn(n, G, D, generator=g, dtype=F64)
    v = torch.randn(n, G, Vd, generator=g, dtype=F64)
    edge = [j for j in range(n) if size and (j % size in (0, size - 1))] or [0, 5, n - 2]
    for j in edge:
        k[j] = 4.0 * torch.sign(torch.randn(G, D, generator=g, dtype=F64))
        v[j] = 10.0 * (1 + edge.index(j))
    q[:, :, :] = q.abs() * torch.sign(k[edge[0]]).repeat_interleave(H // G, dim=0)      # queries lean towards edge keys
    want = R.sink_attention(q, k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1), 0.4, 6.0, size or None)
    nblk = (n + bs - 1) // bs
    table = torch.randperm(nblk + 3, generator=g)[:nblk].tolist()
    kc = torch.full((nblk + 3, G, bs, D), float("nan"), device=DEV)
    vc = torch.full((nblk + 3, G, bs, Vd), float("nan"), device=DEV)
    for j in range(n):
        kc[table[j // bs], :, j % bs] = k[j].float().to(DEV)
        vc[table[j // bs], :, j % bs] = v[j].float().to(DEV)
    bt = _i32([table + [0] * 2])
    qd = q.float().reshape(n, H * D).contiguous().to(DEV)
    out = torch.zeros(n, H * Vd, device=DEV)
    seq_of_row, pos_of_row = _i32([0] * n), _i32(list(range(n)))      # named: a pointer must not outlive its tensor
    rc = lib.atx_attn_local(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), nblk + 2, seq_of_row.data_ptr(),
                            pos_of_row.data_ptr(), None, 0, out.data_ptr(), H * Vd, n, H, G, D, Vd, bs, 0.4, 6.0,
                            size, 1, 1.0, cabi.DT_F32, 0, _st())
    assert rc == 0, lib.atx_last_error()
    torch.cuda.synchronize()
    assert torch.allclose(out.cpu().double().view(n, H, Vd), want, atol=2e-4, rtol=2e-5)
    one = torch.zeros(1, H * Vd, device=DEV)
    seq0 = _i32([0])
    for t in sorted(set(edge + [j + 1 for j in edge if j + 1 < n] + [n - 1])):
        q1, pos1 = qd[t:t + 1].contiguous(), _i32([t])
        rc = lib.atx_attn_local(q1.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), nblk + 2, seq0.data_ptr(),
                                pos1.data_ptr(), None, 0, one.data_ptr(), H * Vd, 1, H, G, D, Vd, bs, 0.4, 6.0, size, 1,
                                1.0, cabi.DT_F32, 0, _st())
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.allclose(one.cpu().double().view(H, Vd), want[t], atol=2e-4, rtol=2e-5), t


@pytest.mark.parametrize("D,size,pos0,n", [(64, 24, 0, 200), (64, 64, 37, 150), (128, 0, 5, 130), (128, 100, 99, 234)])
def test_tensor_core_attention_block_edges_with_dominant_keys(D, size, pos0, n):
    """The prompt-portion kernel on bf16 pages: positions pos0 .. pos0+n-1 are this step's rows (earlier keys are in
    the pages already), block edges carry dominant keys with values of their own, a second short sequence shares the
    launch. Every input is exactly representable in bf16; the probabilities are rounded to bf16 inside the kernel."""
    lib, cabi = _lib()
    H, G, bs, total = 4, 2, 16, pos0 + n
    g = torch.Generator().manual_seed(D + size + n)
    bf = lambda t: t.to(torch.bfloat16).to(F64)
    q = bf(torch.randn(total, H, D, generator=g, dtype=F64))
    k = bf(0.1 * torch.randn(total, G, D, generator=g, dtype=F64))
    v = bf(torch.randn(total, G, D, generator=g, dtype=F64))
    edge = sorted({j for j in range(total) if size and (j % size in (0, size - 1))} | {pos0, max(0, pos0 - 1), 63, 64, 127, 128} & set(range(total)))
    for i, j in enumerate(edge):
        k[j] = bf(0.5 * torch.sign(torch.randn(G, D, generator=g, dtype=F64)))
        v[j] = float(8 * (1 + i % 30))
    q = bf(q.abs() * torch.sign(k[edge[0]]).repeat_interleave(H // G, dim=0))
    want = R.sink_attention(q, k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1), 0.3, 7.0, size or None)
    nblk = (total + bs - 1) // bs
    table = torch.randperm(nblk + 5, generator=g)[:nblk].tolist()
    kc = torch.full((nblk + 5, G, bs, D), float("nan"), device=DEV, dtype=torch.bfloat16)
    vc = torch.full((nblk + 5, G, bs, D), float("nan"), device=DEV, dtype=torch.bfloat16)
    for j in range(total):
        kc[table[j // bs], :, j % bs] = k[j].to(torch.bfloat16).to(DEV)
        vc[table[j // bs], :, j % bs] = v[j].to(torch.bfloat16).to(DEV)
    short = min(9, total)                                   # a second sequence: the first `short` positions, rows first
    bt = _i32([table + [0] * 4, table + [0] * 4])
    rows = list(range(short)) + list(range(pos0, total))
    qd = q[rows].to(torch.bfloat16).reshape(len(rows), H * D).contiguous().to(DEV)
    gate = torch.randn(len(rows), H, generator=g).to(DEV).contiguous()
    out = torch.zeros(len(rows), H * D + 8, device=DEV, dtype=torch.bfloat16)
    s0, sc, sp = _i32([0, short]), _i32([short, n]), _i32([0, pos0])
    assert lib.atx_attn_local_prefill_supported(D, D, cabi.DT_BF16) == 1
    rc = lib.atx_attn_local_prefill(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), nblk + 4, s0.data_ptr(),
                                    sc.data_ptr(), sp.data_ptr(), 2, len(rows), gate.data_ptr(), H, out.data_ptr(), H * D + 8,
                                    H, G, D, D, bs, 0.3, 7.0, size, 1, 0.5, cabi.DT_BF16, 0, _st())
    assert rc == 0, lib.atx_last_error()
    torch.cuda.synchronize()
    got = out[:, :H * D].float().cpu().double().view(len(rows), H, D)
    ref = want[rows] * torch.sigmoid(gate.cpu().double())[:, :, None] * 0.5
    assert float(out[:, H * D:].float().abs().max()) == 0.0
    scale = ref.abs().amax(dim=(1, 2), keepdim=True).clamp(min=1.0)
    assert float(((got - ref).abs() / scale).max()) < 2e-2
    # the same launch as an ordinary softmax: no sink, no cap (rows in a new block meet whole tiles that are masked for them)
    rc = lib.atx_attn_local_prefill(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), nblk + 4, s0.data_ptr(),
                                    sc.data_ptr(), sp.data_ptr(), 2, len(rows), None, 0, out.data_ptr(), H * D + 8,
                                    H, G, D, D, bs, 0.3, 0.0, size, 0, 1.0, cabi.DT_BF16, 0, _st())
    assert rc == 0, lib.atx_last_error()
    torch.cuda.synchronize()
    got = out[:, :H * D].float().cpu().double().view(len(rows), H, D)
    pos = torch.arange(total)
    seen = pos[:, None] >= pos[None, :]
    if size:
        seen = seen & ((pos[:, None] // size) == (pos[None, :] // size))
    sco = torch.einsum("thd,jhd->htj", q, k.repeat_interleave(H // G, 1)) * 0.3
    prob = torch.softmax(sco.masked_fill(~seen[None], float("-inf")), dim=-1)
    ref = torch.einsum("htj,jhv->thv", prob, v.repeat_interleave(H // G, 1))[rows]
    scale = ref.abs().amax(dim=(1, 2), keepdim=True).clamp(min=1.0)
    assert float(((got - ref).abs() / scale).max()) < 2e-2


@pytest.mark.parametrize("per_token", [False, True])
def test_recurrence_remembers_a_far_key_across_steps_and_slots(per_token):
    """One early token has a key and value far larger than the rest and the slowest head barely decays: hundreds of
    tokens later the outputs are still made of it. The sequence is cut into steps of uneven sizes, beside a second
    sequence in another slot, after the slots were filled with garbage."""
    lib, cabi = _lib()
    n, H, G, D, V = 700, 4, 2, 40, 24
    g = torch.Generator().manual_seed(21)
    q, k = torch.randn(n, G, D, generator=g, dtype=F64), torch.randn(n, G, D, generator=g, dtype=F64)
    v = torch.randn(n, H, V, generator=g, dtype=F64)
    k[3] *= 30.0
    v[3] *= 30.0
    q[-50:] = q[-50:].abs() * torch.sign(k[3])
    qh, kh = q.repeat_interleave(H // G, 1), k.repeat_interleave(H // G, 1)
    if per_token:
        dt = 0.01 + 0.05 * torch.rand(n, H, generator=g, dtype=F64)
        rate, skip = torch.tensor([0.01, 0.3, 2.0, 20.0], dtype=F64), torch.tensor([0.5, -1.0, 0.0, 2.0], dtype=F64)
        want = R.selective_scan(v, kh, qh, dt, rate, skip)
        dec_tok = torch.exp(-rate * dt).float().to(DEV).contiguous()
        dt_d, skip_d = dt.float().to(DEV).contiguous(), skip.float().to(DEV)
    else:
        lam = torch.tensor([0.9995, 0.99, 0.9, 0.5], dtype=F64)
        want = R.decayed_linear_attention(qh, kh, v, lam)
        lam_d = lam.float().to(DEV)
    assert want[-1].abs().max() > 50 * want[2].abs().max()          # the far token dominates the end
    other = 17
    qd = torch.cat([q, q[:other]]).float().reshape(-1, G * D).to(DEV)
    state = torch.full((3, H, D, V), 1e30, device=DEV)
    cuts, at, outs = [1, 2, 15, 16, 17, 33, 250, 1, 1, 300], 0, []
    cuts.append(n - sum(cuts))
    for i, c in enumerate(cuts):
        with_other = i == 3                 # the other sequence runs whole beside the fourth portion, rows first
        rows = list(range(at, at + c))
        src = (list(range(other)) if with_other else []) + rows
        idx = torch.tensor(src, device=DEV)
        qs = q.float().reshape(n, G * D).to(DEV)[idx].contiguous()
        ks = k.float().reshape(n, G * D).to(DEV)[idx].contiguous()
        vs = v.float().reshape(n, H * V).to(DEV)[idx].contiguous()
        y = torch.zeros(len(src), H * V, device=DEV)
        seqs = ([(0, other, 0, 0)] if with_other else []) + [(len(src) - c, c, at, 2)]
        a = [_i32([s[j] for s in seqs]) for j in range(4)]
        if per_token:
            dec_rows, dt_rows = dec_tok[idx].contiguous(), dt_d[idx].contiguous()
            rc = lib.atx_linear_recurrence(qs.data_ptr(), G * D, ks.data_ptr(), G * D, vs.data_ptr(), H * V, H, G, D, V, None,
                                           dec_rows.data_ptr(), dt_rows.data_ptr(),
                                           skip_d.data_ptr(), 0, state.data_ptr(), y.data_ptr(), H * V, a[0].data_ptr(),
                                           a[1].data_ptr(), a[2].data_ptr(), a[3].data_ptr(), len(seqs), 0, _st())
        else:
            rc = lib.atx_linear_recurrence(qs.data_ptr(), G * D, ks.data_ptr(), G * D, vs.data_ptr(), H * V, H, G, D, V,
                                           lam_d.data_ptr(), None, None, None, 0, state.data_ptr(), y.data_ptr(), H * V,
                                           a[0].data_ptr(), a[1].data_ptr(), a[2].data_ptr(), a[3].data_ptr(), len(seqs), 0,
                                           _st())
        assert rc == 0, lib.atx_last_error()
        torch.cuda.synchronize()
        if with_other:
            assert torch.allclose(y[:other].cpu().double().view(other, H, V), want[:other], rtol=1e-4, atol=1e-3)
        outs.append(y[len(src) - c:].cpu().double())
        at += c
    got = torch.cat(outs).view(n, H, V)
    scale = want.abs().amax(dim=(1, 2), keepdim=True).clamp(min=1.0)
    assert float(((got - want).abs() / scale).max()) < 2e-4


@pytest.mark.parametrize("per_token,D,V", [(False, 32, 24), (False, 128, 128), (False, 64, 80), (True, 128, 64),
                                            (True, 32, 40), (True, 96, 8)])
def test_chunked_recurrence_matches_the_closed_form_and_shares_its_state_with_the_stepwise_kernel(per_token, D, V):
    """The tensor-core form of the recurrence on the far-key input: portions of uneven sizes (chunk edges inside and at
    the ends of portions, a portion of two tokens), single tokens between them on the token-by-token kernel, the same
    state slot throughout, a second sequence beside one portion, slots filled with garbage first. Operands are bf16
    values, so what remains against the float64 closed form is the rounding of the decayed products. One head decays
    to exactly zero in a single step (per-token case): nothing may turn into NaN."""
    lib, cabi = _lib()
    assert lib.atx_linear_recurrence_chunked_supported(D) == 1 and lib.atx_linear_recurrence_chunked_supported(40) == 0
    n, H, G = 450, 4, 2
    g = torch.Generator().manual_seed(5)
    bf = lambda x: x.to(torch.bfloat16).to(F64)
    q, k = bf(torch.randn(n, G, D, generator=g, dtype=F64)), bf(torch.randn(n, G, D, generator=g, dtype=F64))
    v = bf(torch.randn(n, H, V, generator=g, dtype=F64))
    k[3], v[3] = bf(k[3] * 30.0), bf(v[3] * 30.0)
    q[-50:] = q[-50:].abs() * torch.sign(k[3])
    qh, kh = q.repeat_interleave(H // G, 1), k.repeat_interleave(H // G, 1)
    if per_token:
        dt = (0.01 + 0.05 * torch.rand(n, H, generator=g)).to(F64)
        rate, skip = torch.tensor([0.01, 0.3, 2.0, 1e5], dtype=F64), torch.tensor([0.5, -1.0, 0.0, 2.0], dtype=F64)
        dec = torch.exp(-rate * dt).float()
        assert float(dec[:, 3].max()) == 0.0
        want = R.selective_scan(v, kh, qh, dt, rate, skip)
        dec_d, dt_d, skip_d = dec.to(DEV).contiguous(), dt.float().to(DEV).contiguous(), skip.float().to(DEV)
    else:
        lam = torch.tensor([0.9995, 0.99, 0.9, 0.5], dtype=F64)
        want = R.decayed_linear_attention(qh, kh, v, lam)
        lam_d = lam.float().to(DEV)
    assert want[-1, 0].abs().max() > 20 * want[2, 0].abs().max()          # the far token dominates the end
    other = 70
    qa, ka, va = (x.float().reshape(n, -1).to(DEV) for x in (q, k, v))
    state = torch.full((3, H, D, V), 1e30, device=DEV)
    cuts, at, outs = [2, 62, 1, 64, 65, 1, 1, 127, 3], 0, []
    cuts.append(n - sum(cuts))
    lead = 1 if D in (32, 96) else 4       # unused elements before every row: an odd pitch and 4-byte alignment, or 16
    for i, c in enumerate(cuts):
        with_other = i == 4
        src = (list(range(other)) if with_other else []) + list(range(at, at + c))
        idx = torch.tensor(src, device=DEV)
        # lead 1: the kernel's 4-byte loads; lead 4: its 16-byte loads
        qs, ks, vs = (torch.nn.functional.pad(x[idx], (lead, 0)) for x in (qa, ka, va))
        qp, kp, vp = (x.data_ptr() + 4 * lead for x in (qs, ks, vs))
        lq, lv = G * D + lead, H * V + lead
        y = torch.full((len(src), H * V), float("nan"), device=DEV)
        seqs = ([(0, other, 0, 0)] if with_other else []) + [(len(src) - c, c, at, 2)]
        a = [_i32([s_[j] for s_ in seqs]) for j in range(4)]
        fn = lib.atx_linear_recurrence if c == 1 else lib.atx_linear_recurrence_chunked
        if per_token:
            dr, tr = dec_d[idx].contiguous(), dt_d[idx].contiguous()
            rc = fn(qp, lq, kp, lq, vp, lv, H, G, D, V, None, dr.data_ptr(), tr.data_ptr(), skip_d.data_ptr(), 0,
                    state.data_ptr(), y.data_ptr(), H * V, a[0].data_ptr(), a[1].data_ptr(), a[2].data_ptr(), a[3].data_ptr(),
                    len(seqs), 0, _st())
        else:
            rc = fn(qp, lq, kp, lq, vp, lv, H, G, D, V, lam_d.data_ptr(), None, None, None, 0, state.data_ptr(),
                    y.data_ptr(), H * V, a[0].data_ptr(), a[1].data_ptr(), a[2].data_ptr(), a[3].data_ptr(), len(seqs), 0,
                    _st())
        assert rc == 0, lib.atx_last_error()
        torch.cuda.synchronize()
        outs.append(y.cpu().double())
        at += c
    assert all(bool(torch.isfinite(o).all()) for o in outs)
    scale = want.abs().amax(dim=2, keepdim=True).clamp(min=1.0)
    beside = outs[4][:other].view(other, H, V)
    assert float(((beside - want[:other]).abs() / scale[:other]).max()) < 2e-2
    got = torch.cat([o[-c:] for o, c in zip(outs, cuts)]).view(n, H, V)
    assert float(((got - want).abs() / scale).max()) < 2e-2
    assert float(((got - want).abs() / scale).mean()) < 2e-3


def test_short_convolution_carries_its_window_across_short_steps():
    lib, cabi = _lib()
    n, Cc, H, K = 29, 37, 3, 4
    g = torch.Generator().manual_seed(31)
    x = torch.randn(n, Cc + H + 5, generator=g, dtype=F64)           # [pad | channels | dt] in one row, pitch Cc + H + 5
    taps, bias = torch.randn(Cc, K, generator=g, dtype=F64), torch.randn(Cc, generator=g, dtype=F64)
    dt_bias, a_log = torch.randn(H, generator=g, dtype=F64), torch.randn(H, generator=g, dtype=F64)
    want = R.swish(R.causal_taps(x[:, 5:5 + Cc], taps, bias))
    want_dt = torch.log1p(torch.exp(x[:, 5 + Cc:] + dt_bias))
    want_dec = torch.exp(-torch.exp(a_log) * want_dt)
    xd = x.float().to(DEV).contiguous()
    f = lambda t: t.float().to(DEV).contiguous()
    taps_d, bias_d, dtb_d, al_d = f(taps), f(bias), f(dt_bias), f(a_log)
    state = torch.full((2, K - 1, Cc), 1e30, device=DEV)
    at, outs, dts, decs = 0, [], [], []
    for c in [1, 1, 2, 1, 3, 5, 2, 14]:
        rows = xd[at:at + c].contiguous()
        out, dto, deco = torch.zeros(c, Cc, device=DEV), torch.zeros(c, H, device=DEV), torch.zeros(c, H, device=DEV)
        s0, sc, sp, ss, ts = _i32([0]), _i32([c]), _i32([at]), _i32([1]), _i32([0] * c)
        rc = lib.atx_conv_dt(rows.data_ptr(), Cc + H + 5, 5, 5 + Cc, taps_d.data_ptr(), bias_d.data_ptr(), dtb_d.data_ptr(),
                             al_d.data_ptr(), state.data_ptr(), out.data_ptr(), dto.data_ptr(), deco.data_ptr(),
                             ts.data_ptr(), s0.data_ptr(), sp.data_ptr(), ss.data_ptr(), c, Cc, H, K, cabi.DT_F32, 0, _st())
        assert rc == 0, lib.atx_last_error()
        rc = lib.atx_conv_state_update(rows.data_ptr(), Cc + H + 5, 5, state.data_ptr(), s0.data_ptr(), sc.data_ptr(),
                                       sp.data_ptr(), ss.data_ptr(), 1, Cc, K, 0, _st())
        assert rc == 0
        outs.append(out.cpu().double()), dts.append(dto.cpu().double()), decs.append(deco.cpu().double())
        at += c
    assert at == n
    assert torch.allclose(torch.cat(outs), want, atol=1e-5)
    assert torch.allclose(torch.cat(dts), want_dt, atol=1e-5) and torch.allclose(torch.cat(decs), want_dec, atol=1e-5)


@pytest.mark.parametrize("K", [2, 4, 7])
def test_short_convolution_on_prompt_sized_steps_with_several_sequences(K):
    """Steps of 256 rows and more take the row-tiled kernel: three sequences of uneven length in one step (starting in
    the middle of a tile of rows, one of them shorter than the window), padded rows between them, and a second step
    that continues two of them from the carried window."""
    lib, cabi = _lib()
    Cc, H = 300, 5
    g = torch.Generator().manual_seed(33)
    lens = [131, K - 1 if K > 2 else 1, 210]
    x = [torch.randn(n + 140, Cc + H, generator=g, dtype=F64) for n in lens]
    taps, bias = torch.randn(Cc, K, generator=g, dtype=F64), torch.randn(Cc, generator=g, dtype=F64)
    dt_bias, a_log = torch.randn(H, generator=g, dtype=F64), torch.randn(H, generator=g, dtype=F64)
    want = [R.swish(R.causal_taps(xi[:, :Cc], taps, bias)) for xi in x]
    f = lambda t: t.float().to(DEV).contiguous()
    taps_d, bias_d, dtb_d, al_d = f(taps), f(bias), f(dt_bias), f(a_log)
    state = torch.full((4, K - 1, Cc), 1e30, device=DEV)
    slots = [2, 0, 3]

    def step(parts):           # parts: (sequence, first position, rows); three padded rows after every sequence
        rows, seq_of, starts = [], [], []
        for si, (q, p0, n) in enumerate(parts):
            starts.append(len(seq_of))
            rows.append(x[q][p0:p0 + n])
            rows.append(torch.full((3, Cc + H), float("nan"), dtype=F64))
            seq_of += [si] * n + [-1] * 3
        xd = f(torch.cat(rows))
        T = xd.shape[0]
        assert T >= 256
        out, dto, deco = (torch.zeros(T, w_, device=DEV) for w_ in (Cc, H, H))
        s0, sc = _i32(starts), _i32([n for _, _, n in parts])
        sp, ss, ts = _i32([p0 for _, p0, _ in parts]), _i32([slots[q] for q, _, _ in parts]), _i32(seq_of)
        rc = lib.atx_conv_dt(xd.data_ptr(), Cc + H, 0, Cc, taps_d.data_ptr(), bias_d.data_ptr(), dtb_d.data_ptr(),
                             al_d.data_ptr(), state.data_ptr(), out.data_ptr(), dto.data_ptr(), deco.data_ptr(),
                             ts.data_ptr(), s0.data_ptr(), sp.data_ptr(), ss.data_ptr(), T, Cc, H, K, cabi.DT_F32, 0, _st())
        assert rc == 0, lib.atx_last_error()
        rc = lib.atx_conv_state_update(xd.data_ptr(), Cc + H, 0, state.data_ptr(), s0.data_ptr(), sc.data_ptr(),
                                       sp.data_ptr(), ss.data_ptr(), len(parts), Cc, K, 0, _st())
        assert rc == 0
        torch.cuda.synchronize()
        for (q, p0, n), a in zip(parts, starts):
            assert torch.allclose(out[a:a + n].cpu().double(), want[q][p0:p0 + n], atol=1e-5), (q, p0)
            dt_want = torch.log1p(torch.exp(x[q][p0:p0 + n, Cc:] + dt_bias))
            assert torch.allclose(dto[a:a + n].cpu().double(), dt_want, atol=1e-5)
            assert torch.allclose(deco[a:a + n].cpu().double(), torch.exp(-torch.exp(a_log) * dt_want), atol=1e-5)

    step([(0, 0, lens[0]), (1, 0, lens[1]), (2, 0, lens[2])])
    step([(2, lens[2], 140), (1, lens[1], 1), (0, lens[0], 140)])


def test_fma_gemm_and_norm_kernels_match_their_formulas():
    lib, cabi = _lib()
    g = torch.Generator().manual_seed(41)
    T, N, K = 37, 53, 75
    for xt, dt, tol in ((torch.float32, cabi.DT_F32, 1e-5), (torch.bfloat16, cabi.DT_BF16, 1e-5)):
        w = torch.randn(N, K, generator=g).to(xt).to(DEV)
        x = torch.randn(T, K, generator=g).to(xt).to(DEV)
        out = torch.zeros(T, N + 3, device=DEV)
        rc = lib.atx_gemm_simple(w.data_ptr(), K, x.data_ptr(), K, out.data_ptr(), N + 3, T, N, K, 0, dt, 0, _st())
        assert rc == 0, lib.atx_last_error()
        assert torch.allclose(out[:, :N].cpu().double(), x.cpu().double() @ w.cpu().double().T, atol=1e-4, rtol=tol)
        assert float(out[:, N:].abs().max()) == 0.0
    for W in (70, 72, 1028):      # element-wise; one four-element vector per thread, kept in registers; vectors in a loop
        h, y = torch.randn(T, W, generator=g, dtype=F64), 3.0 * torch.randn(T, W, generator=g, dtype=F64)
        wp, vec, wn = (torch.randn(W, generator=g, dtype=F64) for _ in range(3))
        hd, o = h.float().to(DEV), torch.zeros(T, W, device=DEV)
        f = lambda t: t.float().to(DEV).contiguous()
        yd, wpd, vecd, wnd = f(y), f(wp), f(vec), f(wn)
        rc = lib.atx_resid_norm(hd.data_ptr(), yd.data_ptr(), wpd.data_ptr(), vecd.data_ptr(), wnd.data_ptr(),
                                o.data_ptr(), None, T, W, 1e-5, 1, None, 0, cabi.DT_F32, 0, _st())
        assert rc == 0, lib.atx_last_error()
        h2 = h + R.unit_rms(y, 1e-5) * wp + vec
        assert float(yd.abs().max()) == 0.0        # the sublayer output is handed back cleared
        assert torch.allclose(hd.cpu().double(), h2, atol=1e-5) and torch.allclose(o.cpu().double(), R.unit_rms(h2, 1e-5) * wn, atol=1e-5)
    for n, groups in ((60, 3), (66, 3)):      # groups of 20: four elements per access; of 22: element-wise
        yy, gg, ww = torch.randn(T, n, generator=g, dtype=F64), torch.randn(T, n, generator=g, dtype=F64), torch.randn(n, generator=g, dtype=F64)
        for mode, want in ((0, R.unit_rms(yy, 1e-5) * ww * torch.sigmoid(gg) * 0.7),
                           (1, R.unit_rms((yy * R.swish(gg)).view(T, groups, n // groups), 1e-5).reshape(T, n) * ww * 0.7)):
            o = torch.zeros(T, n, device=DEV)
            yyd, ggd, wwd = f(yy), f(gg), f(ww)
            rc = lib.atx_gated_norm(yyd.data_ptr(), n, ggd.data_ptr(), n, wwd.data_ptr(), o.data_ptr(), n, T, n,
                                    1 if mode == 0 else groups, 1e-5, mode, 0.7, cabi.DT_F32, 0, _st())
            assert rc == 0, lib.atx_last_error()
            assert torch.allclose(o.cpu().double(), want, atol=1e-5), mode
    for W in (70, 72):      # embedding rows: element-wise; four elements per access
        for xt, dt in ((torch.float32, cabi.DT_F32), (torch.bfloat16, cabi.DT_BF16)):
            V = 9
            table = torch.randn(V, W, generator=g).to(xt).to(DEV)
            ids = torch.tensor([3, 0, 8, 8, 5], dtype=torch.int32, device=DEV)
            n = ids.numel()
            out = torch.zeros(n, W, device=DEV)
            rc = lib.atx_embed_rows(ids.data_ptr(), table.data_ptr(), out.data_ptr(), n, W, V, dt, 0, _st())
            assert rc == 0, lib.atx_last_error()
            assert torch.equal(out, table[ids.long()].float())
            hh = torch.randn(n, W, generator=g).to(DEV)
            both = torch.zeros(n, 2 * W, dtype=xt, device=DEV)
            rc = lib.atx_concat_embed(hh.data_ptr(), ids.data_ptr(), table.data_ptr(), both.data_ptr(), n, W, V, dt, 0, _st())
            assert rc == 0, lib.atx_last_error()
            assert torch.equal(both[:, :W], hh.to(xt)) and torch.equal(both[:, W:], table[ids.long()])
