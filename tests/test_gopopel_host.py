"""Host side of the Gopopel family: configuration and registry, checkpoint names, the weight layout the kernels read,
explicit step plans without state slots, and the reference against itself (window and causality, the sink, the distance
penalty, value blending, and latent attention written out in full against its absorbed form). No GPU."""
import json

import pytest
import torch

from oracle import gopopel_ref as R

F64 = torch.float64


def small_cfg(**over):
    cfg = {
        "architecture": "Gopopel", "embedding": {"scale": 5.0}, "vocab": 96, "width": 64, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "latent_attention", "mlp": {"ff": 40, "kind": "dense"},
             "mixer": {"dim": 8, "heads": 3, "kv_rank": 12, "mask": {"size": 11}, "q_rank": 16,
                       "rot": {"base": 100.0, "dims": 4}, "rot_dim": 4, "scale": 0.3, "vdim": 10}},
            {"type": "attention", "mlp": None,
             "mixer": {"dim": 8, "heads": 4, "kv_heads": 2, "mask": {"size": 9}, "scale": 0.35, "v_mix": True, "vdim": 12}},
            {"type": "attention", "mlp": {"ff": 24, "kind": "dense"},
             "mixer": {"dim": 6, "heads": 2, "kv_heads": 2, "mask": {"size": 5}, "scale": 0.4, "v_mix": True, "vdim": 12}},
        ],
    }
    cfg.update(over)
    return cfg


def test_config_is_read_from_json_and_picked_by_architecture(tmp_path):
    from atx.config import model_config_from_json, resolve_model
    from atx.models import gopopel

    cfg = small_cfg()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    m = model_config_from_json(tmp_path / "config.json")
    assert isinstance(m, gopopel.Config) and m.architecture == "Gopopel" and not m.recurrent
    assert (m.vocab_size, m.width, m.eps, m.embed_scale, m.num_hidden_layers) == (96, 64, 1e-5, 5.0, 3)
    assert m.first_mix_layer() == 1
    assert resolve_model(str(tmp_path)).config.tensor_shapes() == m.tensor_shapes()
    with pytest.raises(ValueError):
        gopopel.Config.from_json(dict(cfg, layers=[{"type": "conv", "mixer": {}, "mlp": None}]))
    short = json.loads(json.dumps(cfg))                  # keys with a plain default may be left out
    del short["layers"][0]["mixer"]["rot"]["dims"], short["layers"][2]["mixer"]["kv_heads"]
    ms = gopopel.Config.from_json(short)
    assert ms.layers[0]["mixer"]["rot"]["dims"] == 4 and ms.layers[2]["mixer"]["kv_heads"] == 2
    assert ms.tensor_shapes() == m.tensor_shapes()
    bad = json.loads(json.dumps(cfg))
    bad["layers"][2]["mixer"]["vdim"] = 16          # blending layers must agree on the value shape
    with pytest.raises(ValueError):
        gopopel.Config.from_json(bad)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["mixer"]["rot"]["dims"] = 6    # more rotated dimensions than the rotated part has
    with pytest.raises(ValueError):
        gopopel.Config.from_json(bad)


def test_checkpoint_names_and_shapes_match_the_reference_listing():
    from atx.models import gopopel

    cfg = small_cfg()
    assert gopopel.Config.from_json(cfg).tensor_shapes() == R.checkpoint_shapes(cfg)
    no_mix = json.loads(json.dumps(cfg))
    for l in no_mix["layers"]:
        l["mixer"].pop("v_mix", None)
    shapes = gopopel.Config.from_json(no_mix).tensor_shapes()
    assert shapes == R.checkpoint_shapes(no_mix) and not any(k.endswith("vmix") for k in shapes)


def test_named_bench_shapes_resolve():
    from atx.config import resolve_model

    src = resolve_model("random:gopopel-tiny:3")
    assert src.config.architecture == "Gopopel" and src.random_seed == 3 and src.path is None
    assert [l["type"] for l in src.config.layers] == ["latent_attention", "attention"]
    assert src.config.kv_bytes_per_token() > 0 and src.config.weight_bytes_per_decode_step() > 0
    big = resolve_model("random:gopopel-8b").config
    assert big.width == 4096 and big.num_hidden_layers == 32
    assert resolve_model("random:tiny:1").config.architecture == "llama"


def test_weights_are_laid_out_for_the_kernels():
    """Stacked input projections, the key up-projection transposed per head, scalars as host numbers, slopes as a table."""
    from atx.models import gopopel

    cfg = small_cfg()
    m = gopopel.Config.from_json(cfg)
    wt = R.random_checkpoint(cfg, 1)
    w = gopopel.Weights.from_state_dict(m, wt, torch.device("cpu"), torch.float32)
    lat, a1, a2 = w.layers
    c = cfg["layers"][0]["mixer"]
    H, D, C = c["heads"], c["dim"], c["kv_rank"]
    assert torch.equal(lat.w_in.double(), torch.cat([wt["l0.mix.dq"], wt["l0.mix.dkv"], wt["l0.mix.g"]]).float().double())
    uk = wt["l0.mix.uk"].view(H, D, C)
    assert torch.equal(lat.w_ukt.double().view(H, C, D), uk.transpose(1, 2).float().double())
    assert a1.vmix == 0.0 and a2.vmix == pytest.approx(float(wt["l2.mix.vmix"]))     # the first blending layer only records
    assert torch.allclose(a1.slopes.double(), R.head_slopes(4)) and a1.slopes[-1] == 2.0 ** -8
    assert lat.norm.alpha == pytest.approx(float(wt["l0.norm1.alpha"])) and w.final_norm.w.shape == (64,)
    with pytest.raises(KeyError):
        gopopel.Weights.from_state_dict(m, {k: v for k, v in wt.items() if k != "l1.mix.sink"}, torch.device("cpu"),
                                        torch.float32)
    with pytest.raises(ValueError):
        gopopel.Weights.from_state_dict(m, dict(wt, head=wt["head"][:-1]), torch.device("cpu"), torch.float32)


def test_explicit_step_plans_need_no_state_slot():
    from atx.kv_cache import BlockAllocator
    from atx.scheduler import SamplingParams, Scheduler, Sequence

    alloc = BlockAllocator(8, 16, False)
    sch = Scheduler(alloc, 4, 256, 256, ())
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    a, b = Sequence("a", list(range(41)), sp, alloc), Sequence("b", [1, 2, 3], sp, alloc)
    plan = sch.plan_explicit([(a, 40, [0, 39]), (b, 1, [0])])
    assert plan.decodes == [] and [c.count for c in plan.prefills] == [40, 1]     # a first token is a portion of one
    assert a.state_slot is None and b.state_slot is None
    sch.commit(plan, {})
    plan = sch.plan_explicit([(a, 1, [0]), (b, 2, [])])
    assert [c.seq.request_id for c in plan.decodes] == ["a"] and [c.count for c in plan.prefills] == [2]
    sch.commit(plan, {})
    sch.retire(a), sch.retire(b)
    assert alloc.num_free == alloc.num_blocks


# ---- the reference against itself -----------------------------------------------------------------------------------------

def test_window_mask_keeps_the_row_itself_and_size_minus_one_before_it():
    m = R.window_mask(10, 3)
    assert m[5].tolist() == [False, False, False, True, True, True, False, False, False, False]
    assert m[0].tolist() == [True] + [False] * 9 and m[1].tolist()[:3] == [True, True, False]
    assert R.window_mask(4, 1).int().tolist() == torch.eye(4, dtype=torch.int32).tolist()


def test_sink_takes_weight_without_a_value_and_slopes_favour_near_keys():
    g = torch.Generator().manual_seed(0)
    n, H = 12, 2
    q, k = torch.randn(n, H, 4, generator=g, dtype=F64), torch.randn(n, H, 4, generator=g, dtype=F64)
    v = torch.ones(n, H, 3, dtype=F64)
    seen = R.window_mask(n, n)
    assert torch.allclose(R.softmax_attention(q, k, v, 0.5, seen), torch.ones(n, H, 3, dtype=F64))
    for s in (-2.0, 0.0, 3.0):
        o = R.softmax_attention(q, k, v, 0.5, seen, sinks=torch.tensor([s, s], dtype=F64))
        a = torch.einsum("ihd,jhd->hij", q, k) * 0.5
        den = torch.exp(a.masked_fill(~seen[None], -1e300)).sum(-1)
        assert torch.allclose(o[..., 0], (den / (den + torch.exp(torch.tensor(s, dtype=F64)))).T)
    # equal scores: the weights fall geometrically with distance, by exp(-slope) a step
    z = torch.zeros(n, H, 4, dtype=F64)
    vv = torch.eye(n, dtype=F64)[:, None, :].repeat(1, H, 1)
    o = R.softmax_attention(z, z, vv, 1.0, seen, slopes=R.head_slopes(H))
    assert torch.allclose(o[n - 1, 0, n - 2] / o[n - 1, 0, n - 1], torch.exp(-R.head_slopes(H)[0]))
    assert R.head_slopes(8)[0] == 0.5 and R.head_slopes(8)[-1] == 2.0 ** -8


def test_latent_attention_written_out_equals_its_absorbed_form():
    """What the engine computes: one cached row [latent | rotated key part] per token, queries mapped into the latent's
    coordinates by W_uk^T, values recovered by W_uv after the weighted sum over latents."""
    cfg = small_cfg()
    c = cfg["layers"][0]["mixer"]
    wt = R.random_checkpoint(cfg, 2, round_bf16=False)
    n = 30
    u = torch.randn(n, 64, generator=torch.Generator().manual_seed(1), dtype=F64)
    want = R.latent_attention_mixer(u, c, wt, "l0.mix.", 1e-5)
    H, D, Rr, V, C = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    p = "l0.mix."
    q = R.lin(R.unit_rms(R.lin(u, wt[p + "dq"]), wt[p + "dq.norm"], 1e-5), wt[p + "uq"]).view(n, H, D + Rr)
    dkv = R.lin(u, wt[p + "dkv"])
    row = torch.cat([R.unit_rms(dkv[:, :C], wt[p + "dkv.norm"], 1e-5),
                     R.rotate_pairs(dkv[:, C:].contiguous(), 4, 100.0)], -1)                      # [n, C + R]: the cache
    q_abs = torch.einsum("thd,hdc->thc", q[..., :D], wt[p + "uk"].view(H, D, C))
    q_all = torch.cat([q_abs, R.rotate_pairs(q[..., D:].contiguous(), 4, 100.0)], -1)
    o_lat = R.softmax_attention(q_all, row[:, None, :], row[:, None, :C].contiguous(), c["scale"], R.window_mask(n, 11))
    o = torch.einsum("thc,hvc->thv", o_lat, wt[p + "uv"].view(H, V, C)).reshape(n, H * V)
    got = R.lin(o * torch.sigmoid(R.lin(u, wt[p + "g"])), wt[p + "o"])
    assert torch.allclose(got, want, atol=1e-10)


def test_forward_is_causal_and_blending_reads_the_first_blending_layer():
    cfg = small_cfg()
    wt = R.random_checkpoint(cfg, 3)
    toks = [int(t) for t in torch.randint(0, 96, (40,), generator=torch.Generator().manual_seed(4))]
    full = R.forward(cfg, wt, toks)
    assert torch.allclose(R.forward(cfg, wt, toks[:25]), full[:25], atol=1e-9)
    other = dict(wt)
    other["l1.mix.vmix"] = wt["l1.mix.vmix"] + 0.3          # the first blending layer's factor is not used
    assert torch.equal(R.forward(cfg, other, toks), full)
    other = dict(wt)
    other["l2.mix.vmix"] = wt["l2.mix.vmix"] + 0.3
    assert not torch.allclose(R.forward(cfg, other, toks), full, atol=1e-6)
    far = list(toks)
    far[0] = (far[0] + 1) % 96                              # beyond every window of every layer: 11 + 9 + 5 - 3 positions
    assert torch.allclose(R.forward(cfg, wt, far)[23:], full[23:], atol=1e-9)
    assert not torch.allclose(R.forward(cfg, wt, far)[:8], full[:8], atol=1e-6)
