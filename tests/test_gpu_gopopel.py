"""The Gopopel family on the GPU against the float64 reference (oracle/gopopel_ref.py): the engine (scheduler, pages,
runner, kernels) on small random models (whole prompts, token-by-token decoding, portions down to two tokens, mixed
batches, reuse of pages, greedy generation through the ordinary entry point) and kernels alone on inputs built so that a
window that is one key off, a missing sink, a wrong slope or a lost far key shows."""
import numpy as np
import pytest
import torch

from oracle import gopopel_ref as R

pytestmark = pytest.mark.gpu
F64 = torch.float64
DEV = "cuda:0"


# ---- small models ------------------------------------------------------------------------------------------------------

def attention_layer(heads=4, kv=2, dim=8, vdim=12, size=9, v_mix=False, mlp=None, scale=0.35):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"dim": dim, "heads": heads, "kv_heads": kv, "mask": {"size": size}, "scale": scale, "v_mix": v_mix,
                      "vdim": vdim}}


def latent_layer(heads=3, dim=8, rot_dim=4, vdim=10, kv_rank=12, q_rank=16, size=11, rot_dims=None, base=100.0, mlp=None,
                 scale=0.3):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"dim": dim, "heads": heads, "kv_rank": kv_rank, "mask": {"size": size}, "q_rank": q_rank,
                      "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}, "rot_dim": rot_dim,
                      "scale": scale, "vdim": vdim}}


def model_cfg(layers, width=64, vocab=96, embed_scale=3.0, eps=1e-6):
    return {"architecture": "Gopopel", "embedding": {"scale": embed_scale}, "vocab": vocab, "width": width,
            "norm": {"eps": eps}, "layers": layers}


FF = {"ff": 72, "kind": "dense"}


def mixed_model(width=64):
    """Both mixers, three blending layers (the first only records its values), one layer without a feed-forward."""
    return model_cfg([latent_layer(mlp=FF), attention_layer(v_mix=True, mlp=FF), attention_layer(v_mix=True, size=14),
                      latent_layer(heads=2, dim=6, rot_dim=8, rot_dims=4, vdim=16, kv_rank=20, q_rank=24, size=7, mlp=FF),
                      attention_layer(heads=2, kv=2, dim=8, vdim=12, v_mix=True, size=5, mlp={"ff": 40, "kind": "dense"})],
                     width=width)


def engine(cfg, wt, dtype="float32", **kw):
    from atx.config import EngineConfig, ModelSource
    from atx.engine import LLMEngine
    from atx.models import gopopel

    mcfg = gopopel.Config.from_json(cfg)
    xt = torch.float32 if dtype == "float32" else torch.bfloat16
    w = gopopel.Weights.from_state_dict(mcfg, wt, torch.device(DEV), xt)
    ecfg = EngineConfig(max_model_len=kw.pop("max_model_len", 256), max_num_seqs=kw.pop("max_num_seqs", 4),
                        max_num_batched_tokens=kw.pop("max_num_batched_tokens", 256),
                        num_gpu_blocks=kw.pop("num_gpu_blocks", 64),
                        enable_prefix_caching=kw.pop("enable_prefix_caching", False),
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
    return float(rel_rows(got, want).max())


TOL = {"float32": 2e-5, "bfloat16": 0.08}      # bf16: operand rounding through up to five layers; fp32 is the sharp test


def whole(eng, rid, toks, end=True):
    return eng.feed([(rid, toks, list(range(len(toks))))], [rid] if end else [])


def run_steps(eng, reqs, steps):
    """steps: lists of (request, token count); returns the logits of every request in order of its tokens."""
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    for step in steps:
        entries, end = [], []
        for k, n in step:
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        out, o = eng.feed(entries, end), 0
        for k, n in step:
            got[k].append(out[o:o + n])
            o += n
    assert at == {k: len(v) for k, v in reqs.items()}
    return {k: np.concatenate(v) for k, v in got.items()}


# ---- each mechanism alone, through the engine ------------------------------------------------------------------------------

ONE_LAYER = {
    "attention": lambda: attention_layer(),
    "attention_every_head_its_own_kv": lambda: attention_layer(heads=3, kv=3, dim=10, vdim=6, size=200),
    "attention_ffn": lambda: attention_layer(heads=2, kv=1, dim=4, vdim=4, size=3, mlp={"ff": 24, "kind": "dense"}),
    "attention_tensor_core_sizes": lambda: attention_layer(heads=4, kv=2, dim=64, vdim=64, size=70, scale=0.125),
    "attention_between_tile_widths": lambda: attention_layer(heads=2, kv=1, dim=72, vdim=40, size=33, scale=0.12),
    "latent": lambda: latent_layer(),
    "latent_part_of_the_rotated_block_turns": lambda: latent_layer(rot_dim=8, rot_dims=2, size=200),
    "latent_ffn": lambda: latent_layer(heads=1, dim=4, rot_dim=2, vdim=4, kv_rank=6, q_rank=5, size=4, mlp=FF),
    "latent_tensor_core_sizes": lambda: latent_layer(heads=4, dim=32, rot_dim=16, vdim=24, kv_rank=48, q_rank=64, size=70,
                                                     scale=0.14),
    "latent_wide": lambda: latent_layer(heads=2, dim=16, rot_dim=32, vdim=16, kv_rank=160, q_rank=32, size=40, scale=0.1),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [64, 88])       # 88: not a multiple of the tensor-core GEMM's K block
@pytest.mark.parametrize("kind", sorted(ONE_LAYER))
def test_one_layer_models(kind, width, dtype):
    cfg = model_cfg([ONE_LAYER[kind]()], width=width)
    wt = R.random_checkpoint(cfg, 11)
    toks = tokens(150, seed=1)
    eng = engine(cfg, wt, dtype)
    got = whole(eng, "a", toks)
    want = R.forward(cfg, wt, toks)
    assert rel(got, want) < TOL[dtype]
    # portions that start inside a window and inside a 64-row tile, beside a decoded token of another request
    a = eng.feed([("p", toks[:70], list(range(70)))], [])
    b = eng.feed([("p", toks[70:71], [0]), ("q", toks[:131], list(range(131)))], ["q"])
    c = eng.feed([("p", toks[71:], list(range(79)))], ["p"])
    assert rel(np.concatenate([a, b[:1], c]), want) < TOL[dtype] and rel(b[1:], want[:131]) < TOL[dtype]
    eng.runner.close()


def test_first_tokens_of_a_sequence():
    cfg = mixed_model()
    wt = R.random_checkpoint(cfg, 3)
    eng = engine(cfg, wt)
    for n in (1, 2, 3):
        toks = tokens(n, seed=n)
        assert rel(whole(eng, f"r{n}", toks), R.forward(cfg, wt, toks)) < TOL["float32"]


def test_residual_stream_after_every_layer():
    cfg = mixed_model()
    wt = R.random_checkpoint(cfg, 5)
    toks = tokens(40, seed=2)
    res = []
    R.forward(cfg, wt, toks, res)
    eng = engine(cfg, wt)
    eng.runner.layer_probe = []
    whole(eng, "a", toks)
    got = eng.runner.layer_probe
    assert len(got) == len(res)
    for g, w in zip(got, res):
        assert float((g.cpu().double() - w).abs().max()) < 2e-5 * float(w.abs().max())


# ---- the same logits however the tokens are cut ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_token_by_token_and_portions_agree(dtype):
    cfg = mixed_model()
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


def test_long_decoding_lets_every_window_pass_over_decoded_tokens():
    cfg = mixed_model()
    wt = R.random_checkpoint(cfg, 6)
    toks = tokens(200, seed=7)
    eng = engine(cfg, wt)
    got = [eng.feed([("d", toks[:9], list(range(9)))], [])]
    got += [eng.feed([("d", toks[i:i + 1], [0])], []) for i in range(9, len(toks))]
    assert rel(np.concatenate(got), R.forward(cfg, wt, toks)) < TOL["float32"]


def test_mixed_batches_equal_each_request_alone():
    cfg = mixed_model()
    wt = R.random_checkpoint(cfg, 8)
    reqs = {"a": tokens(61, seed=1), "b": tokens(23, seed=2), "c": tokens(40, seed=3), "d": tokens(5, seed=4)}
    want = {k: R.forward(cfg, wt, v) for k, v in reqs.items()}
    # portions of some requests beside single tokens of others; c joins late, d comes and goes in the middle
    steps = [[("a", 17), ("b", 2)], [("a", 1), ("b", 19)], [("a", 30), ("b", 1), ("c", 3)], [("b", 1), ("c", 1), ("d", 5)],
             [("a", 13), ("c", 20)], [("c", 1)], [("c", 15)]]
    for dtype in ("float32", "bfloat16"):
        eng = engine(cfg, wt, dtype, max_num_seqs=4)
        got = run_steps(eng, reqs, steps)
        for k in reqs:
            assert rel(got[k], want[k]) < TOL[dtype], (dtype, k)
        assert eng.allocator.num_free == eng.allocator.num_blocks
        eng.runner.close()


def test_bf16_portions_on_the_tensor_cores_beside_single_tokens():
    """bf16 steps where prompt portions take the tensor-core attention and single tokens beside them the row kernel, on
    the same pages; portions cross 64-row tiles, 16-token pages and both windows."""
    cfg = model_cfg([latent_layer(heads=4, dim=32, rot_dim=16, vdim=24, kv_rank=48, q_rank=64, size=70, scale=0.14, mlp=FF),
                     attention_layer(heads=4, kv=2, dim=64, vdim=32, size=40, scale=0.125, v_mix=True, mlp=FF),
                     attention_layer(heads=4, kv=2, dim=24, vdim=32, size=90, scale=0.2, v_mix=True)], width=128)
    wt = R.random_checkpoint(cfg, 15)
    reqs = {"a": tokens(150, seed=1), "b": tokens(90, seed=2), "c": tokens(70, seed=3), "d": tokens(6, seed=5)}
    want = {k: R.forward(cfg, wt, v) for k, v in reqs.items()}
    steps = [[("a", 70), ("b", 2)], [("a", 1), ("b", 65)], [("a", 1), ("b", 1), ("c", 63)], [("a", 64), ("b", 1), ("c", 1),
             ("d", 6)], [("b", 21), ("c", 2), ("a", 1)], [("a", 13), ("c", 4)]]
    from atx import _cabi
    lib = _cabi.load()
    assert lib.atx_attn_window_prefill_supported(64, 48, 64, 64, 0) and lib.atx_attn_window_prefill_supported(24, 32, 24, 32, 0)
    eng = engine(cfg, wt, "bfloat16", max_num_seqs=4, max_model_len=160, max_num_batched_tokens=512)
    got = run_steps(eng, reqs, steps)
    for k in reqs:
        alone = whole(eng, k + "-alone", reqs[k])
        assert rel(got[k], want[k]) < TOL["bfloat16"] and rel(got[k], alone) < TOL["bfloat16"], k
    assert eng.allocator.num_free == eng.allocator.num_blocks


def test_pages_are_reused_without_leaking_old_keys():
    cfg = mixed_model()
    wt = R.random_checkpoint(cfg, 9)
    eng = engine(cfg, wt, max_num_seqs=2, num_gpu_blocks=6, max_model_len=96)       # 96 tokens of pages
    whole(eng, "big", tokens(90, seed=1))                                          # fills every page
    for seed, n in ((2, 33), (3, 50), (4, 17)):
        toks = tokens(n, seed=seed)
        assert rel(whole(eng, f"r{seed}", toks), R.forward(cfg, wt, toks)) < TOL["float32"]
    # a request that starts while another is alive takes the freed pages
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


ODD_MODELS = {
    "window_of_one": lambda: model_cfg([attention_layer(size=1), latent_layer(size=1)]),
    "windows_larger_than_the_prompt": lambda: model_cfg([latent_layer(size=4096, mlp=FF), attention_layer(size=1000)]),
    "no_blending_anywhere": lambda: model_cfg([attention_layer(mlp=FF), attention_layer(heads=2, kv=1, dim=6, vdim=20)]),
    "one_blending_layer_only_records": lambda: model_cfg([attention_layer(v_mix=True, mlp=FF), attention_layer()]),
    "blending_skips_a_layer": lambda: model_cfg([attention_layer(v_mix=True), attention_layer(mlp=FF),
                                                 latent_layer(), attention_layer(v_mix=True, size=4)]),
    "one_head": lambda: model_cfg([attention_layer(heads=1, kv=1, dim=16, vdim=16), latent_layer(heads=1)]),
    "many_heads_one_kv": lambda: model_cfg([attention_layer(heads=8, kv=1, dim=4, vdim=6, size=20)]),
    "no_embedding_scale_other_eps": lambda: model_cfg([latent_layer(mlp=FF), attention_layer(mlp=FF)], embed_scale=1.0,
                                                      eps=1e-3),
    "width_and_vocabulary_off_every_block": lambda: model_cfg([latent_layer(mlp=FF), attention_layer(mlp=FF)], width=72,
                                                              vocab=77),
    "value_wider_than_key": lambda: model_cfg([attention_layer(heads=4, kv=2, dim=16, vdim=136, size=50),
                                               latent_layer(heads=2, dim=8, rot_dim=8, vdim=96, kv_rank=24, q_rank=40)],
                                              width=128),
    "latent_wider_than_a_tile": lambda: model_cfg([latent_layer(heads=2, dim=24, rot_dim=16, vdim=32, kv_rank=288,
                                                                q_rank=48, size=60, scale=0.05)], width=128),
    "keys_of_256": lambda: model_cfg([attention_layer(heads=2, kv=1, dim=256, vdim=32, size=33, scale=0.06)], width=128),
    "rotation_base_large": lambda: model_cfg([latent_layer(rot_dim=16, base=1e6, size=120, mlp=FF)]),
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
        lim = 3e-5 if dtype == "float32" else 0.1
        assert np.isfinite(a).all() and np.isfinite(b).all(), dtype
        assert rel(a, want) < lim and rel(b, want) < lim, (dtype, rel(a, want), rel(b, want))
        eng.runner.close()


def drawn_model(rng):
    """A model whose layer order, sizes and constants are drawn at random from sizes a real model could have."""
    vshape = (rng.choice([1, 2, 4]), rng.choice([16, 32, 48, 64, 80]))

    def attention():
        mixing = rng.random() < 0.6
        kv, vd = vshape if mixing else (rng.choice([1, 2, 4]), rng.choice([16, 40, 64, 128]))
        d = rng.choice([16, 32, 64, 96, 128])
        return {"dim": d, "heads": kv * rng.choice([1, 2, 3, 4]), "kv_heads": kv,
                "mask": {"size": rng.choice([1, 16, 33, 64, 100, 140, 500])}, "scale": rng.choice([d ** -0.5, 0.05, 0.11]),
                "v_mix": mixing, "vdim": vd}

    def latent():
        r = rng.choice([8, 16, 32, 64])
        d = rng.choice([16, 32, 64])
        return {"dim": d, "heads": rng.choice([1, 2, 4, 6]), "kv_rank": rng.choice([24, 64, 96, 128, 200]),
                "mask": {"size": rng.choice([2, 17, 64, 75, 130, 400])}, "q_rank": rng.choice([32, 64, 96, 192]),
                "rot": {"base": rng.choice([1e2, 1e4, 5e5]), "dims": rng.choice([x for x in (2, 8, 16, 32, 64) if x <= r])},
                "rot_dim": r, "scale": rng.choice([(d + r) ** -0.5, 0.08]), "vdim": rng.choice([16, 32, 80, 128])}

    def layer(kind):
        return {"type": kind, "mixer": attention() if kind == "attention" else latent(),
                "mlp": rng.choice([None, {"ff": rng.choice([128, 192, 320, 500]), "kind": "dense"}])}

    n = rng.randint(2, 6)
    kinds = ["attention", "latent_attention"] + [rng.choice(["attention", "latent_attention"]) for _ in range(n - 2)]
    rng.shuffle(kinds)
    return model_cfg([layer(k) for k in kinds], width=rng.choice([64, 128, 160, 192, 256, 320]),
                     vocab=rng.choice([256, 320, 500, 1000, 1027]), embed_scale=rng.choice([1.0, 4.0, 12.0, 20.0]),
                     eps=rng.choice([1e-5, 1e-6]))


@pytest.mark.parametrize("draw", range(6))
def test_drawn_models_whole_cut_and_mixed(draw):
    """Three unequal requests of a drawn model: each whole, the longest in portions with its last tokens one by one, then
    all three in steps where a request may bring a portion, one token or nothing."""
    import random
    rng = random.Random(7000 + draw)
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
        assert eng.allocator.num_free == eng.allocator.num_blocks
        r = torch.cat(rows)
        assert torch.isfinite(r).all(), dtype
        if dtype == "float32":
            assert float(r.max()) < 5e-5 and float(r.median()) < 5e-6, (float(r.max()), float(r.median()))
        else:
            assert float(r.max()) < 0.2 and float(r.median()) < 0.03, (float(r.max()), float(r.median()))
        eng.runner.close()


# ---- generation through the ordinary entry point ---------------------------------------------------------------------------

@pytest.mark.parametrize("mode", ["plain", "chunked_prefill", "async", "graphs"])
def test_greedy_generation_matches_the_reference(mode):
    from atx.scheduler import SamplingParams

    cfg = mixed_model()
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
    assert eng.allocator.num_free == eng.allocator.num_blocks
    eng.runner.close()


@pytest.mark.parametrize("mode", ["plain", "graphs"])
def test_bf16_greedy_generation_on_the_tensor_core_kernels(mode):
    """Sizes that take the tensor-core attention for prompts and its decode form for generated tokens (also inside a
    captured graph, with padded rows in the batch bucket). bf16 against the float64 reference: a token may differ only
    where the reference's two best logits are closer than the arithmetic's noise."""
    from atx.scheduler import SamplingParams

    ff = {"ff": 128, "kind": "dense"}      # a multiple of the tcgen05 GEMM's block: decode steps run the feed-forward on
    cfg = model_cfg([latent_layer(heads=4, dim=32, rot_dim=16, vdim=24, kv_rank=48, q_rank=64, size=70, scale=0.14, mlp=ff),
                     attention_layer(heads=4, kv=2, dim=64, vdim=32, size=40, scale=0.125, v_mix=True, mlp=ff),
                     attention_layer(heads=6, kv=2, dim=24, vdim=32, size=90, scale=0.2, v_mix=True)], width=128)
    wt = R.random_checkpoint(cfg, 17)      # a second stream beside the mixer (two branches of a captured graph)
    prompts = [tokens(100, seed=1), tokens(5, seed=2), tokens(64, seed=3)]
    kw = {"plain": {}, "graphs": {"async_scheduling": True, "enable_cuda_graphs": True}}[mode]
    eng = engine(cfg, wt, "bfloat16", **kw)
    outs = eng.generate_sync(prompts, SamplingParams(temperature=0.0, max_tokens=60, ignore_eos=True))
    close = 0
    for p, o in zip(prompts, outs):
        assert len(o) == 60
        lg = R.forward(cfg, wt, p + o[:-1])[len(p) - 1:]
        spread = float(lg.std())
        top2 = lg.topk(2, dim=-1).values
        for i, tok in enumerate(o):
            if tok != int(lg[i].argmax()):
                close += 1
                assert float(top2[i, 0] - lg[i, tok]) < 0.15 * spread, (mode, i)
    assert close <= 12
    assert eng.allocator.num_free == eng.allocator.num_blocks
    eng.runner.close()


def test_generation_over_a_cached_prefix_matches_the_reference():
    """Pages of a shared prefix are attached from the block cache instead of being computed again: they hold blended
    values and latent rows, which depend on the token and its position only, so the continuation must not change."""
    from atx.scheduler import SamplingParams

    cfg = mixed_model()
    wt = R.random_checkpoint(cfg, 21)
    common = tokens(50, seed=9)
    prompts = [common + tokens(7, seed=1), common + tokens(12, seed=2), common[:33] + tokens(3, seed=3)]
    eng = engine(cfg, wt, enable_prefix_caching=True)
    outs = [eng.generate_sync([p], SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))[0] for p in prompts]
    assert eng.allocator.hits >= 3 + 2                      # 48 and 32 tokens of full pages were found again
    for p, o in zip(prompts, outs):
        lg = R.forward(cfg, wt, p + o[:-1])[len(p) - 1:]
        top2 = lg.topk(2, dim=-1).values
        for i, tok in enumerate(o):
            assert tok == int(lg[i].argmax()) or float(top2[i, 0] - top2[i, 1]) < 1e-4, i
    eng.runner.close()


def test_named_shape_generates_through_the_registry():
    from atx.config import EngineConfig, resolve_model
    from atx.engine import LLMEngine
    from atx.scheduler import SamplingParams

    src = resolve_model("random:gopopel-tiny:3")
    eng = LLMEngine(src, EngineConfig(max_model_len=256, max_num_seqs=4, max_num_batched_tokens=256, num_gpu_blocks=64,
                                      enable_prefix_caching=False))
    outs = eng.generate_sync([tokens(40, 1024, 1), tokens(3, 1024, 2)], SamplingParams(temperature=0.0, max_tokens=8,
                                                                                      ignore_eos=True))
    assert [len(o) for o in outs] == [8, 8]
    eng.runner.close()


# ---- kernels alone, on inputs where one wrong key shows --------------------------------------------------------------------

def _lib():
    from atx import _cabi

    return _cabi.load(), _cabi


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _st():
    return torch.cuda.current_stream().cuda_stream


def _pages(x, table, bs, row=None, dtype=torch.float32):
    """x [n, G, w] -> pages [blocks, G, bs, row] in the order of `table`, unused slots NaN."""
    n, G, w = x.shape
    row = row or w
    pg = torch.full((max(table) + 2, G, bs, row), float("nan"), device=DEV, dtype=dtype)
    for j in range(n):
        pg[table[j // bs], :, j % bs, :w] = x[j].to(dtype).to(DEV)
    return pg


def _edge_case(n, H, G, D, Vd, window, seed, bf16=False):
    """Queries that lean towards a few dominant keys placed so that, for some query, the dominant key is the last one the
    window keeps and, for the next query, the first one it has lost; every dominant key has a value of its own. Far
    keys: a dominant key hundreds of positions back must not leak into any query outside its window."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=F64)
    bf = (lambda t: t.to(torch.bfloat16).to(F64)) if bf16 else (lambda t: t)
    q = rnd(n, H, D)
    k = 0.1 * rnd(n, G, D)
    v = rnd(n, G, Vd)
    sign = torch.sign(rnd(G, D))
    strong = sorted({0, 1, 15, 16, 17, n // 3, n // 2, n - window - 1, n - window, n - 2} & set(range(n)))
    for i, j in enumerate(strong):
        k[j] = 3.0 * sign
        v[j] = 6.0 * (1 + i)
    q = q.abs() * sign.repeat_interleave(H // G, dim=0)
    return bf(q), bf(k), bf(v), strong


@pytest.mark.parametrize("window,n", [(1, 20), (7, 60), (16, 70), (33, 400), (64, 130), (1000, 90)])
def test_row_attention_window_edges_sink_and_slopes(window, n):
    """The one-warp-per-row kernel in fp32 on the crafted keys: all rows at once, then single rows (the decode form),
    over pages in scrambled order."""
    lib, cabi = _lib()
    H, G, D, Vd, bs = 4, 2, 8, 6, 16
    q, k, v, strong = _edge_case(n, H, G, D, Vd, window, window + n)
    slopes, sinks = R.head_slopes(H), torch.tensor([0.5, -1.0, 2.0, 0.0], dtype=F64)
    want = R.softmax_attention(q, k, v, 0.4, R.window_mask(n, window), slopes, sinks)
    nblk = (n + bs - 1) // bs
    table = torch.randperm(nblk + 3, generator=torch.Generator().manual_seed(n))[:nblk].tolist()
    kc, vc = _pages(k, table, bs), _pages(v, table, bs)
    bt = _i32([table + [0] * 2])
    qd = q.float().reshape(n, H * D).contiguous().to(DEV)
    sl, sk = slopes.float().to(DEV), sinks.float().to(DEV)
    out = torch.zeros(n, H * Vd, device=DEV)
    seq_of_row, pos_of_row = _i32([0] * n), _i32(list(range(n)))
    rc = lib.atx_attn_window(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), D, Vd, bt.data_ptr(), nblk + 2,
                             seq_of_row.data_ptr(), pos_of_row.data_ptr(), None, 0, out.data_ptr(), H * Vd, n, H, G, D, Vd,
                             bs, 0.4, 0.0, 0, window, sl.data_ptr(), sk.data_ptr(), 1, 1.0, cabi.DT_F32, 0, _st())
    assert rc == 0, lib.atx_last_error()
    torch.cuda.synchronize()
    assert torch.allclose(out.cpu().double().view(n, H, Vd), want, atol=2e-4, rtol=2e-5)
    one, seq0 = torch.zeros(1, H * Vd, device=DEV), _i32([0])
    rows = sorted({j + d for j in strong for d in (0, 1, window - 1, window, window + 1) if j + d < n} | {n - 1})
    for t in rows:
        q1, pos1 = qd[t:t + 1].contiguous(), _i32([t])
        rc = lib.atx_attn_window(q1.data_ptr(), kc.data_ptr(), vc.data_ptr(), D, Vd, bt.data_ptr(), nblk + 2,
                                 seq0.data_ptr(), pos1.data_ptr(), None, 0, one.data_ptr(), H * Vd, 1, H, G, D, Vd, bs, 0.4,
                                 0.0, 0, window, sl.data_ptr(), sk.data_ptr(), 1, 1.0, cabi.DT_F32, 0, _st())
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.allclose(one.cpu().double().view(H, Vd), want[t], atol=2e-4, rtol=2e-5), t
    # without the sink and the slopes the same launch is an ordinary windowed softmax: they are not baked in
    rc = lib.atx_attn_window(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), D, Vd, bt.data_ptr(), nblk + 2,
                             seq_of_row.data_ptr(), pos_of_row.data_ptr(), None, 0, out.data_ptr(), H * Vd, n, H, G, D, Vd,
                             bs, 0.4, 0.0, 0, window, None, None, 0, 1.0, cabi.DT_F32, 0, _st())
    assert rc == 0
    torch.cuda.synchronize()
    plain = R.softmax_attention(q, k, v, 0.4, R.window_mask(n, window))
    assert torch.allclose(out.cpu().double().view(n, H, Vd), plain, atol=2e-4, rtol=2e-5)
    assert not torch.allclose(plain, want, atol=1e-2)


@pytest.mark.parametrize("D,Vd,window,pos0,n", [(64, 64, 24, 0, 200), (64, 32, 64, 37, 150), (128, 128, 1, 5, 130),
                                               (96, 48, 100, 99, 234), (128, 96, 65, 63, 300), (200, 120, 300, 0, 140),
                                               (256, 16, 63, 64, 129)])
def test_tensor_core_attention_window_edges_sink_and_slopes(D, Vd, window, pos0, n):
    """The prompt-portion kernel on bf16 pages: positions pos0 .. pos0+n-1 are this step's rows (earlier keys are in the
    pages already), a second short sequence shares the launch, keys and values sit in rows wider than the heads. Inputs
    are exactly representable in bf16; the probabilities are rounded to bf16 inside the kernel."""
    lib, cabi = _lib()
    H, G, bs, total = 4, 2, 16, pos0 + n
    q, k, v, _ = _edge_case(total, H, G, D, Vd, window, D + window + n, bf16=True)
    k = (k * 0.2).to(torch.bfloat16).to(F64)
    slopes, sinks = R.head_slopes(H), torch.tensor([0.5, -1.0, 2.0, 0.0], dtype=F64)
    want = R.softmax_attention(q, k, v, 0.3, R.window_mask(total, window), slopes, sinks)
    nblk = (total + bs - 1) // bs
    table = torch.randperm(nblk + 5, generator=torch.Generator().manual_seed(n))[:nblk].tolist()
    k_row, v_row = D + 8, Vd + 16
    kc = _pages(k, table, bs, k_row, torch.bfloat16)
    vc = _pages(v, table, bs, v_row, torch.bfloat16)
    short = min(9, total)                                   # a second sequence: the first `short` positions, rows first
    width = max(table) + 4
    bt = _i32([table + [0] * (width - len(table))] * 2)
    rows = list(range(short)) + list(range(pos0, total))
    qd = q[rows].to(torch.bfloat16).reshape(len(rows), H * D).contiguous().to(DEV)
    out = torch.zeros(len(rows), H * Vd + 8, device=DEV, dtype=torch.bfloat16)
    s0, sc, sp = _i32([0, short]), _i32([short, n]), _i32([0, pos0])
    sl, sk = slopes.float().to(DEV), sinks.float().to(DEV)
    assert lib.atx_attn_window_prefill_supported(D, Vd, k_row, v_row, cabi.DT_BF16) == 1
    rc = lib.atx_attn_window_prefill(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), k_row, v_row, bt.data_ptr(), width,
                                     s0.data_ptr(), sc.data_ptr(), sp.data_ptr(), 2, len(rows), None, 0, out.data_ptr(),
                                     H * Vd + 8, H, G, D, Vd, bs, 0.3, 0.0, 0, window, sl.data_ptr(), sk.data_ptr(), 1, 1.0,
                                     cabi.DT_BF16, 0, _st())
    assert rc == 0, lib.atx_last_error()
    torch.cuda.synchronize()
    got = out[:, :H * Vd].float().cpu().double().view(len(rows), H, Vd)
    ref = want[rows]
    assert float(out[:, H * Vd:].float().abs().max()) == 0.0
    scale = ref.abs().amax(dim=(1, 2), keepdim=True).clamp(min=1.0)
    assert float(((got - ref).abs() / scale).max()) < 2e-2
    # the row kernel on the same pages agrees (decoded tokens and prompt portions read the same cache)
    o2 = torch.zeros(len(rows), H * Vd, device=DEV, dtype=torch.bfloat16)
    seq_of_row, pos_of_row = _i32([0] * short + [1] * n), _i32(rows)
    rc = lib.atx_attn_window(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), k_row, v_row, bt.data_ptr(), width,
                             seq_of_row.data_ptr(), pos_of_row.data_ptr(), None, 0, o2.data_ptr(), H * Vd, len(rows), H, G,
                             D, Vd, bs, 0.3, 0.0, 0, window, sl.data_ptr(), sk.data_ptr(), 1, 1.0, cabi.DT_BF16, 0, _st())
    assert rc == 0, lib.atx_last_error()
    torch.cuda.synchronize()
    got2 = o2.float().cpu().double().view(len(rows), H, Vd)
    assert float(((got2 - ref).abs() / scale).max()) < 1e-2
    # the decode form (heads of a key/value group as the rows of a tile) on single tokens at and around the edges,
    # the keys in one slice and in several (more slices than some rows have tiles)
    pick = sorted({0, 1, min(63, total - 1), min(64, total - 1), total // 2, total - 2, total - 1} |
                  {p for p in (window - 1, window, window + 1, 2 * window) if 0 <= p < total})
    qd1 = q[pick].to(torch.bfloat16).reshape(len(pick), H * D).contiguous().to(DEV)
    seq1, pos1 = _i32([0] * len(pick)), _i32(pick)
    assert lib.atx_attn_window_decode_supported(H, G, D, Vd, k_row, v_row, cabi.DT_BF16) == 1
    for splits in (1, 3, 7):
        o3 = torch.zeros(len(pick), H * Vd + 8, device=DEV, dtype=torch.bfloat16)
        ws = torch.full((max(2, lib.atx_attn_window_decode_workspace_bytes(len(pick), H, Vd, splits) // 4),), float("nan"),
                        device=DEV)
        rc = lib.atx_attn_window_decode(qd1.data_ptr(), kc.data_ptr(), vc.data_ptr(), k_row, v_row, bt.data_ptr(), width,
                                        seq1.data_ptr(), pos1.data_ptr(), None, 0, o3.data_ptr(), H * Vd + 8, ws.data_ptr(),
                                        ws.numel() * 4, splits, len(pick), H, G, D, Vd, bs, 0.3, 0.0, 0, window,
                                        sl.data_ptr(), sk.data_ptr(), 1, 1.0, cabi.DT_BF16, 0, _st())
        assert rc == 0, lib.atx_last_error()
        torch.cuda.synchronize()
        got3 = o3[:, :H * Vd].float().cpu().double().view(len(pick), H, Vd)
        ref3 = want[pick]
        sc3 = ref3.abs().amax(dim=(1, 2), keepdim=True).clamp(min=1.0)
        assert float(((got3 - ref3).abs() / sc3).max()) < 2e-2, splits
        assert float(o3[:, H * Vd:].float().abs().max()) == 0.0


def test_a_far_key_among_hundreds_is_found_inside_the_window_and_lost_outside():
    """One key 299 positions back dominates every other score. With a window of 300 the last query's output is that key's
    value; with 299 it is not. Keys and values share one page array (rows of [key | spare], the value being the leading
    part of the key row), as latent attention keeps them."""
    lib, cabi = _lib()
    n, H, D, Vd, bs = 320, 2, 24, 16, 16
    g = torch.Generator().manual_seed(1)
    k = 0.05 * torch.randn(n, 1, D, generator=g, dtype=F64)
    far = n - 300
    k[far, 0, :Vd] = 0.0
    k[far, 0, Vd:] = 2.0                                   # the leading Vd entries are the value: a one-hot marker
    k[far, 0, 3] = 1.0
    q = torch.zeros(n, H, D, dtype=F64)
    q[:, :, Vd:] = 4.0
    table = list(range((n + bs - 1) // bs))[::-1]
    pg = _pages(k, table, bs)
    bt = _i32([table])
    qd = q.float().reshape(n, H * D).contiguous().to(DEV)
    seq0, pos1 = _i32([0]), _i32([n - 1])
    for window, seen in ((300, True), (299, False)):
        out = torch.zeros(1, H * Vd, device=DEV)
        q1 = qd[n - 1:n].contiguous()
        rc = lib.atx_attn_window(q1.data_ptr(), pg.data_ptr(), pg.data_ptr(), D, D, bt.data_ptr(), len(table),
                                 seq0.data_ptr(), pos1.data_ptr(), None, 0, out.data_ptr(), H * Vd, 1, H, 1, D, Vd, bs, 1.0,
                                 0.0, 0, window, None, None, 0, 1.0, cabi.DT_F32, 0, _st())
        assert rc == 0, lib.atx_last_error()
        torch.cuda.synchronize()
        want = R.softmax_attention(q, k, k[:, :, :Vd].contiguous(), 1.0, R.window_mask(n, window))[n - 1]
        assert torch.allclose(out.cpu().double().view(H, Vd), want, atol=1e-4)
        assert (float(out[0, 3]) > 0.99) == seen


@pytest.mark.parametrize("D,Vd,pad,qo_off,lp_off,C", [(10, 6, 3, 1, 2, 12), (12, 8, 4, 4, 4, 12), (10, 6, 3, 1, 2, 530),
                                                       (12, 8, 4, 4, 4, 640)])
def test_head_preparation_norms_rotates_blends_and_writes_pages(D, Vd, pad, qo_off, lp_off, C):
    """Sizes and offsets off the four-element path and on it; a wide bottleneck takes a CTA per head instead of a warp."""
    lib, cabi = _lib()
    T, bs = 37, 16
    g = torch.Generator().manual_seed(2)
    H, G, Rr, rd = 3, 2, 8, 4
    ld = H * D + G * Vd + C + Rr + pad
    src = torch.randn(T, ld, generator=g, dtype=F64)
    qw, cw = 1 + 0.1 * torch.randn(D, generator=g, dtype=F64), 1 + 0.1 * torch.randn(C, generator=g, dtype=F64)
    first = torch.randn(T, G, Vd, generator=g, dtype=F64)
    pos = [5 + 3 * t for t in range(T)]
    perm = torch.randperm(T + 11, generator=g)[:T].tolist()              # a page slot per row, scrambled
    from atx.models.common import rotation_table
    table = rotation_table(50.0, rd, 200, torch.device(DEV))
    srcd = src.float().to(DEV).contiguous()
    qo = torch.full((T, H * D + 2 * qo_off), 7.0, device=DEV)
    vpg = torch.full(((T + 11 + bs - 1) // bs, G, bs, Vd), float("nan"), device=DEV)
    lpg = torch.full(((T + 11 + bs - 1) // bs, 1, bs, C + Rr + 2 * lp_off), float("nan"), device=DEV)
    saved = torch.zeros(T, G * Vd, device=DEV)
    qwd, cwd, fd = qw.float().to(DEV), cw.float().to(DEV), first.float().reshape(T, G * Vd).contiguous().to(DEV)
    S = cabi.HeadSeg
    sg = cabi.head_segs(
        S(src_off=0, src_stride=D, heads=H, width=D, norm_dims=D, norm_w=qwd.data_ptr(), dst_kind=cabi.HEAD_DST_ROWS,
          dst=qo.data_ptr(), dst_ld=H * D + 2 * qo_off, dst_off=qo_off, dst_stride=D),
        S(src_off=H * D, src_stride=Vd, heads=G, width=Vd, mix=0.3, mix_src=fd.data_ptr(), save=saved.data_ptr(),
          dst_kind=cabi.HEAD_DST_PAGES, dst=vpg.data_ptr(), dst_off=0, dst_stride=Vd),
        S(src_off=H * D + G * Vd, src_stride=C + Rr, heads=1, width=C + Rr, norm_dims=C, norm_w=cwd.data_ptr(), rot_off=C,
          rot_dims=rd, rot=table.data_ptr(), dst_kind=cabi.HEAD_DST_PAGES, dst=lpg.data_ptr(), dst_off=lp_off,
          dst_stride=C + Rr + 2 * lp_off))
    posd, slotd = _i32(pos), _i32(perm)
    rc = lib.atx_head_prepare(srcd.data_ptr(), ld, sg, 3, posd.data_ptr(), slotd.data_ptr(), T, bs, 1e-4, cabi.DT_F32, 0, _st())
    assert rc == 0, lib.atx_last_error()
    torch.cuda.synchronize()
    wq = R.unit_rms(src[:, :H * D].view(T, H, D), qw, 1e-4)
    assert torch.allclose(qo[:, qo_off:qo_off + H * D].cpu().double().view(T, H, D), wq, atol=1e-5)
    assert float(qo[:, :qo_off].min()) == 7.0 and float(qo[:, qo_off + H * D:].min()) == 7.0
    vraw = src[:, H * D:H * D + G * Vd].view(T, G, Vd)
    assert torch.allclose(saved.cpu().double().view(T, G, Vd), vraw, atol=1e-6)
    lat = src[:, H * D + G * Vd:H * D + G * Vd + C + Rr]
    wl = torch.cat([R.unit_rms(lat[:, :C], cw, 1e-4),
                    R.rotate_pairs(lat[:, C:].contiguous(), rd, 50.0, torch.tensor(pos))], dim=-1)
    for t in range(T):
        b, o = perm[t] // bs, perm[t] % bs
        assert torch.allclose(vpg[b, :, o].cpu().double(), 0.7 * vraw[t] + 0.3 * first[t], atol=1e-5)
        assert torch.allclose(lpg[b, 0, o, lp_off:lp_off + C + Rr].cpu().double(), wl[t], atol=1e-5)
        assert torch.isnan(lpg[b, 0, o, :lp_off]).all() and torch.isnan(lpg[b, 0, o, lp_off + C + Rr:]).all()
    assert int(torch.isfinite(vpg[:, 0, :, 0]).sum()) == T                  # nothing was written anywhere else


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tanh_norm_activation_head_gemm_and_scaled_embedding_match_their_formulas(dtype):
    lib, cabi = _lib()
    xt, dt = (torch.float32, cabi.DT_F32) if dtype == "float32" else (torch.bfloat16, cabi.DT_BF16)
    tol = 1e-5 if dtype == "float32" else 1e-2
    g = torch.Generator().manual_seed(3)
    rt = lambda t: t.to(xt).to(F64)
    for T, W in ((5, 64), (70, 50)):
        x = 3 * torch.randn(T, W, generator=g, dtype=F64)
        w, b = rt(1 + 0.1 * torch.randn(W, generator=g, dtype=F64)), rt(0.1 * torch.randn(W, generator=g, dtype=F64))
        xd, wd, bd = x.float().to(DEV), w.to(xt).to(DEV), b.to(xt).to(DEV)
        out = torch.zeros(T, W, dtype=xt, device=DEV)
        junk = torch.ones(4096, device=DEV)
        rc = lib.atx_tanh_norm(xd.data_ptr(), None, 0.37, wd.data_ptr(), bd.data_ptr(), out.data_ptr(), T, W, junk.data_ptr(),
                               4096 * 4 - 64, dt, 0, _st())
        assert rc == 0, lib.atx_last_error()
        torch.cuda.synchronize()
        assert torch.allclose(out.cpu().double(), R.dyt(x.float().double(), 0.37, w, b), atol=tol, rtol=tol)
        assert float(junk[:4096 - 16].abs().max()) == 0.0 and float(junk[4096 - 16:].min()) == 1.0
        rows = _i32([T - 1, 0, 2])
        o3 = torch.zeros(3, W, dtype=xt, device=DEV)
        assert lib.atx_tanh_norm(xd.data_ptr(), rows.data_ptr(), 0.37, wd.data_ptr(), bd.data_ptr(), o3.data_ptr(), 3, W,
                                 None, 0, dt, 0, _st()) == 0
        torch.cuda.synchronize()
        assert torch.equal(o3.cpu(), out.cpu()[[T - 1, 0, 2]])
        act = torch.zeros(T, W + 2, dtype=xt, device=DEV)
        assert lib.atx_unary_act(xd.data_ptr(), W, act.data_ptr(), W + 2, T, W, cabi.ACT_RELU2, dt, 0, _st()) == 0
        torch.cuda.synchronize()
        assert torch.allclose(act[:, :W].cpu().double(), R.relu_squared(x.float().double()), atol=tol, rtol=tol)
        assert lib.atx_unary_act(xd.data_ptr(), W, act.data_ptr(), W + 2, T, W, cabi.ACT_GELU_TANH, dt, 0, _st()) == 0
        torch.cuda.synchronize()
        z = x.float().double()
        gelu = 0.5 * z * (1 + torch.tanh((2 / torch.pi) ** 0.5 * (z + 0.044715 * z ** 3)))
        assert torch.allclose(act[:, :W].cpu().double(), gelu, atol=tol, rtol=tol)
    # per-head products, fp32 rows in and rows of the element type in, with and without the gate; sizes off and on the
    # eight-element staging path of the tensor-core kernel, a reduction longer than one staged chunk
    for T, H, N, K, xo, xp, wp in ((70, 3, 20, 13, 1, 2, 3), (150, 2, 72, 136, 8, 8, 8)):
        X = rt(torch.randn(T, H * (K + xp) + xo, generator=g, dtype=F64))
        Wm = rt(torch.randn(H * N, K + wp, generator=g, dtype=F64) / K ** 0.5)
        gate = torch.randn(T, H * N + 5, generator=g, dtype=F64)
        ref = torch.einsum("thk,hnk->thn", torch.stack([X[:, xo + h * (K + xp):xo + h * (K + xp) + K] for h in range(H)], 1),
                           Wm[:, :K].view(H, N, K))
        gd, Wd = gate.float().to(DEV), Wm.to(xt).to(DEV)
        for x_f32 in (1, 0):
            Xd = X.float().to(DEV) if x_f32 else X.to(xt).to(DEV)
            for gated, fl in ((False, 0), (True, 0), (True, cabi.FLAG_HEAD_GEMM_FMA)):
                out = torch.zeros(T, 2 + H * (N + 1), dtype=xt, device=DEV)
                rc = lib.atx_head_gemm(Xd.data_ptr(), x_f32, X.shape[1], xo, K + xp, Wd.data_ptr(), K + wp,
                                       gd.data_ptr() if gated else None, H * N + 5, out.data_ptr(), out.shape[1], 2, N + 1, T,
                                       H, N, K, dt, fl, _st())
                assert rc == 0, lib.atx_last_error()
                torch.cuda.synchronize()
                want = ref * torch.sigmoid(gate.float().double()[:, :H * N].view(T, H, N)) if gated else ref
                got = torch.stack([out[:, 2 + h * (N + 1):2 + h * (N + 1) + N] for h in range(H)], 1).cpu().double()
                assert torch.allclose(got, want, atol=10 * tol, rtol=tol), (x_f32, gated, fl)
    # embedding rows times a scale
    V, W = 50, 24
    tab = rt(torch.randn(V, W, generator=g, dtype=F64))
    ids = _i32([3, 49, 0, 7])
    out = torch.zeros(4, W, device=DEV)
    td = tab.to(xt).to(DEV)
    assert lib.atx_embed_rows_scaled(ids.data_ptr(), td.data_ptr(), out.data_ptr(), 4, W, V, 12.5, dt, 0, _st()) == 0
    torch.cuda.synchronize()
    assert torch.allclose(out.cpu().double(), tab[[3, 49, 0, 7]] * 12.5, rtol=1e-6)


@pytest.mark.parametrize("T,N,K", [(5, 256, 512), (64, 200, 1024), (100, 384, 128), (300, 520, 320)])
def test_gemm_with_the_squared_relu_in_its_epilogue(T, N, K):
    """Decode-sized steps cut K over a cluster and sum the parts before the activation; prompt-sized steps take the
    persistent kernel. Operands exactly representable in bf16."""
    lib, cabi = _lib()
    g = torch.Generator().manual_seed(T + N)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    x = torch.zeros(max(T, 16), K, dtype=torch.bfloat16, device=DEV)
    x[:T] = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    out = torch.full((T, N + 8), 3.0, dtype=torch.bfloat16, device=DEV)
    plan = cabi.GemmPlan(w, x)
    plan.run(out, T, cabi.GEMM_RELU2_BF16)
    torch.cuda.synchronize()
    want = R.relu_squared(x[:T].cpu().double() @ w.cpu().double().T)
    assert torch.allclose(out[:, :N].cpu().double(), want, atol=2e-2, rtol=1e-2)
    assert float((out[:, N:].float() - 3.0).abs().max()) == 0.0


@pytest.mark.parametrize("H,G", [(40, 1), (64, 2), (6, 3)])
def test_decode_attention_with_many_heads_on_one_shared_key_value_row(H, G):
    """Latent attention's decode shape: many query heads over one cached row per token whose leading part is the value.
    Tokens of two sequences at different lengths, padded rows between them, slices that some tokens leave empty."""
    lib, cabi = _lib()
    D, Vd, bs, window, n = 72, 40, 16, 150, 333
    g = torch.Generator().manual_seed(H)
    bf = lambda t: t.to(torch.bfloat16).to(F64)
    q = bf(torch.randn(n, H, D, generator=g, dtype=F64))
    k = bf(0.3 * torch.randn(n, G, D, generator=g, dtype=F64))
    want = R.softmax_attention(q, k, k[:, :, :Vd].contiguous(), 0.2, R.window_mask(n, window))
    table = torch.randperm(30, generator=g)[:(n + bs - 1) // bs].tolist()
    pg = _pages(k, table, bs, D, torch.bfloat16)
    bt = _i32([table + [0] * (32 - len(table)), table + [0] * (32 - len(table))])
    pick = [n - 1, 0, 5, 149, 150, 151, 200]
    qd = torch.zeros(len(pick) + 2, H * D, dtype=torch.bfloat16, device=DEV)
    qd[:len(pick)] = q[pick].to(torch.bfloat16).reshape(len(pick), H * D).to(DEV)
    seq = _i32([0, 1, 1, 0, 1, 0, 1, -1, -1])                  # two padded rows at the end
    pos = _i32(pick + [0, 0])
    for splits in (1, 4, 16):
        out = torch.full((len(pick) + 2, H * Vd), 9.0, device=DEV, dtype=torch.bfloat16)
        ws = torch.zeros(max(2, lib.atx_attn_window_decode_workspace_bytes(len(pick) + 2, H, Vd, splits) // 4), device=DEV)
        rc = lib.atx_attn_window_decode(qd.data_ptr(), pg.data_ptr(), pg.data_ptr(), D, D, bt.data_ptr(), 32, seq.data_ptr(),
                                        pos.data_ptr(), None, 0, out.data_ptr(), H * Vd, ws.data_ptr(), ws.numel() * 4, splits,
                                        len(pick) + 2, H, G, D, Vd, bs, 0.2, 0.0, 0, window, None, None, 0, 1.0,
                                        cabi.DT_BF16, 0, _st())
        assert rc == 0, lib.atx_last_error()
        torch.cuda.synchronize()
        got = out[:len(pick)].float().cpu().double().view(len(pick), H, Vd)
        assert float((got - want[pick]).abs().max()) < 2e-2, splits
        assert float((out[len(pick):].float() - 9.0).abs().max()) == 0.0      # padded rows are left alone
