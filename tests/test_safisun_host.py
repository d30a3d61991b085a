"""Host side of the Safisun family: configuration and registry, layer order, checkpoint names, the state-slot pool,
explicit step plans, and the reference's closed forms against step-by-step recurrences. No GPU."""
import json

import pytest
import torch

from oracle import safisun_ref as R

F64 = torch.float64


def small_cfg(**over):
    cfg = {
        "architecture": "Safisun", "vocab": 96, "width": 64, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "lightning", "mlp": None, "mixer": {"decay": [0.5, 0.9, 0.99], "dim": 8, "heads": 3, "vdim": 12}},
            {"type": "mamba2", "mlp": {"ff": 40, "kind": "dense"},
             "mixer": {"conv": 3, "groups": 2, "heads": 4, "norm_groups": 2, "state": 8, "vdim": 10}},
            {"type": "parallel", "mlp": None,
             "mixer": {"left": {"dim": 16, "heads": 4, "kv_heads": 2, "mask": {"size": 8}, "rot": {"base": 100.0, "dims": 8},
                                "scale": 0.3, "softcap": 5.0, "vdim": 12},
                       "left_scale": 0.7, "right_scale": 1.3,
                       "right": {"decay": [0.8, 0.95], "dim": 12, "heads": 2, "vdim": 6}}},
        ],
        "loop": {"start": 1, "stop": 3, "times": 3},
    }
    cfg.update(over)
    return cfg


def test_config_is_read_from_json_and_picked_by_architecture(tmp_path):
    from atx.config import model_config_from_json, resolve_model
    from atx.models import safisun

    cfg = small_cfg()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    m = model_config_from_json(tmp_path / "config.json")
    assert isinstance(m, safisun.Config) and m.architecture == "Safisun" and m.recurrent
    assert (m.vocab_size, m.width, m.eps) == (96, 64, 1e-5)
    assert m.runs() == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2)] == R.layer_order(cfg)
    assert resolve_model(str(tmp_path)).config.runs() == m.runs()
    no_loop = safisun.Config.from_json(dict(cfg, loop=None))
    assert no_loop.runs() == [(0, None), (1, None), (2, None)]
    with pytest.raises(ValueError):
        safisun.Config.from_json(dict(cfg, layers=[{"type": "conv", "mixer": {}, "mlp": None}]))
    with pytest.raises(ValueError):
        model_config_from_json_bad = dict(cfg, architecture="nope")
        (tmp_path / "config.json").write_text(json.dumps(model_config_from_json_bad))
        model_config_from_json(tmp_path / "config.json")


def test_checkpoint_names_and_shapes_match_the_reference_listing():
    from atx.models import safisun

    for cfg in (small_cfg(), small_cfg(loop=None)):
        assert safisun.Config.from_json(cfg).tensor_shapes() == R.checkpoint_shapes(cfg)


def test_named_bench_shapes_resolve():
    from atx.config import resolve_model

    src = resolve_model("random:safisun-tiny:3")
    assert src.config.architecture == "Safisun" and src.random_seed == 3 and src.path is None
    kinds = [l["type"] for l in src.config.layers]
    assert kinds == ["mamba2", "mamba2", "parallel", "lightning"]
    assert src.config.state_bytes_per_sequence() > 0 and src.config.kv_bytes_per_token() > 0
    assert resolve_model("random:tiny:1").config.architecture == "llama"


def test_state_slot_pool_hands_slots_out_again():
    from atx.kv_cache import StateSlotPool

    pool = StateSlotPool(2)
    a, b = pool.acquire(), pool.acquire()
    assert {a, b} == {0, 1} and pool.acquire() is None and pool.num_free == 0
    pool.release(a)
    assert pool.acquire() == a
    with pytest.raises(RuntimeError):
        pool.release(b), pool.release(b)


def _sched(num_blocks=8, slots=2, max_seqs=4):
    from atx.kv_cache import BlockAllocator, StateSlotPool
    from atx.scheduler import Scheduler

    alloc = BlockAllocator(num_blocks, 16, enable_prefix_caching=False)
    pool = StateSlotPool(slots)
    return Scheduler(alloc, max_seqs, 256, 128, (), state_slots=pool), alloc, pool


def test_explicit_plans_admit_split_and_give_everything_back():
    from atx.kv_cache import OutOfBlocks
    from atx.scheduler import SamplingParams, Sequence, SeqState

    sch, alloc, pool = _sched()
    a = Sequence("a", list(range(40)), SamplingParams(), alloc)
    b = Sequence("b", list(range(5)), SamplingParams(), alloc)
    plan = sch.plan_explicit([(a, 17, [0, 16]), (b, 5, [])])
    assert [c.count for c in plan.prefills] == [17, 5] and not plan.decodes
    assert a.state_slot is not None and b.state_slot is not None and a.state_slot != b.state_slot
    assert len(a.blocks.table) == 2 and len(b.blocks.table) == 1 and alloc.num_free == 5
    sch.commit(plan, {})
    assert (a.num_computed, b.num_computed) == (17, 5) and a.state is SeqState.RUNNING
    b.tokens.append(7)
    plan = sch.plan_explicit([(b, 1, [0]), (a, 2, [1])])        # one token of a started sequence rides with the decodes
    assert [c.seq for c in plan.decodes] == [b] and [c.seq for c in plan.prefills] == [a]
    assert plan.decodes[0].start == 5 and plan.prefills[0].start == 17 and not plan.decodes[0].samples
    sch.commit(plan, {})
    c = Sequence("c", [1, 2, 3], SamplingParams(), alloc)
    with pytest.raises(RuntimeError):
        sch.plan_explicit([(c, 3, [])])                         # both state slots are held
    sch.retire(b)
    assert b.state is SeqState.FINISHED and b.state_slot is None and pool.num_free == 1
    plan = sch.plan_explicit([(c, 3, [2])])
    assert c.state_slot is not None and pool.num_free == 0
    with pytest.raises(ValueError):
        sch.plan_explicit([(a, 30, [])])                        # more tokens than the sequence has
    big = Sequence("big", list(range(100)), SamplingParams(), alloc)
    sch.retire(c)
    with pytest.raises(OutOfBlocks):
        sch.plan_explicit([(big, 100, [])])                     # 7 pages wanted, 6 free: nothing is preempted for it
    sch.retire(a)
    sch.retire(big)
    assert alloc.num_free == alloc.num_blocks and pool.num_free == 2


def test_ordinary_scheduling_takes_and_returns_state_slots():
    from atx.scheduler import SamplingParams, Sequence

    sch, alloc, pool = _sched(num_blocks=16, slots=2)
    seqs = [Sequence(f"s{i}", [1, 2, 3], SamplingParams(max_tokens=1, ignore_eos=True), alloc) for i in range(3)]
    for s in seqs:
        sch.add(s)
    plan = sch.schedule()
    assert [c.seq for c in plan.prefills] == seqs[:2] and pool.num_free == 0      # the third waits for a slot
    sch.commit(plan, {seqs[0].uid: 5, seqs[1].uid: 6})
    assert pool.num_free == 2 and all(s.state_slot is None for s in seqs[:2])    # finished on length: slots returned
    plan = sch.schedule()
    assert [c.seq for c in plan.prefills] == [seqs[2]] and seqs[2].state_slot is not None


# ---- the reference's closed forms against the recurrences they stand for ---------------------------------------------

def test_reference_linear_attention_equals_its_recurrence():
    g = torch.Generator().manual_seed(0)
    n, H, D, V = 23, 3, 5, 4
    q, k, v = (torch.randn(n, H, d, generator=g, dtype=F64) for d in (D, D, V))
    lam = torch.tensor([0.3, 0.9, 0.999], dtype=F64)
    S, want = torch.zeros(H, D, V, dtype=F64), []
    for t in range(n):
        S = lam[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        want.append(torch.einsum("hdv,hd->hv", S, q[t]))
    assert torch.allclose(R.decayed_linear_attention(q, k, v, lam), torch.stack(want), atol=1e-12)


def test_reference_selective_scan_and_taps_equal_their_recurrences():
    g = torch.Generator().manual_seed(1)
    n, H, P, N = 19, 2, 3, 4
    x, b, c = (torch.randn(n, H, d, generator=g, dtype=F64) for d in (P, N, N))
    dt = torch.rand(n, H, generator=g, dtype=F64)
    rate, skip = torch.tensor([0.5, 2.0], dtype=F64), torch.tensor([1.0, -0.5], dtype=F64)
    S, want = torch.zeros(H, N, P, dtype=F64), []
    for t in range(n):
        S = torch.exp(-rate * dt[t])[:, None, None] * S + dt[t][:, None, None] * b[t][:, :, None] * x[t][:, None, :]
        want.append(torch.einsum("hnp,hn->hp", S, c[t]) + skip[:, None] * x[t])
    assert torch.allclose(R.selective_scan(x, b, c, dt, rate, skip), torch.stack(want), atol=1e-12)
    xs, taps, bias = torch.randn(7, 3, generator=g, dtype=F64), torch.randn(3, 4, generator=g, dtype=F64), torch.ones(3, dtype=F64)
    y = R.causal_taps(xs, taps, bias)
    for t in range(7):
        acc = bias.clone()
        for j in range(4):
            if t - j >= 0:
                acc = acc + taps[:, 3 - j] * xs[t - j]
        assert torch.allclose(y[t], acc, atol=1e-12)


def test_reference_forward_is_causal_and_chunk_local():
    cfg = small_cfg()
    wt = R.random_checkpoint(cfg, 5)
    toks = [int(t) for t in torch.randint(0, cfg["vocab"], (30,), generator=torch.Generator().manual_seed(2))]
    full = R.forward(cfg, wt, toks)
    assert torch.allclose(R.forward(cfg, wt, toks[:11]), full[:11], atol=1e-9)
    # attention alone: a key in the previous block of 8 is not seen, the first key of the own block is
    c = cfg["layers"][2]["mixer"]["left"]
    p = "l2.mix.left."
    u = torch.randn(20, cfg["width"], generator=torch.Generator().manual_seed(3), dtype=F64)
    w64 = {k: v.to(F64) for k, v in wt.items()}
    base = R.local_attention(u, c, w64, p, 1e-5)
    u2 = u.clone()
    u2[7] += 1.0
    moved = (R.local_attention(u2, c, w64, p, 1e-5) - base).abs().amax(-1)
    assert moved[7] > 1e-3 and moved[8:].max() < 1e-12       # row 8 opens a new block
    u3 = u.clone()
    u3[8] += 1.0
    moved = (R.local_attention(u3, c, w64, p, 1e-5) - base).abs().amax(-1)
    assert moved[15] > 1e-6 and moved[16:].max() < 1e-12 and moved[:8].max() < 1e-12
