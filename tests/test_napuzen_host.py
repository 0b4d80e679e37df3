"""Host side of the Napuzen family: configuration and registry, checkpoint names, the weight layout the kernels read,
explicit step plans with state slots, the stretched rotation frequencies, and the reference against itself (recurrence =
sum over pairs, window, absorbed = written-out latent attention, clamps, renormalised expert weights, shared latent). No GPU."""
import json
import math

import pytest
import torch

from oracle import napuzen_ref as R

F64 = torch.float64


def small_cfg(**over):
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 3.0, "original": 40, "fast": 4.0, "slow": 0.5}}
    cfg = {
        "architecture": "Napuzen", "canon": {"taps": 4}, "logit_scale": 0.5, "vocab": 96, "width": 64, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "gla", "mlp": {"kind": "dense", "ff": 40, "limit": 2.0},
             "mixer": {"dim": 6, "heads": 3, "vdim": 10, "tau": 4.0}},
            {"type": "latent_attention_2",
             "mlp": {"kind": "moe", "expert": {"ff": 24}, "shared": {"ff": 16}, "router": {"experts": 5, "top": 3, "scale": 1.25}},
             "mixer": {"dim": 8, "heads": 4, "vdim": 12, "kv_rank": 20, "mask": {"size": 9}, "scale": 0.35}},
            {"type": "latent_attention", "mlp": None,
             "mixer": {"dim": 6, "heads": 2, "vdim": 10, "kv_rank": 14, "q_rank": 18, "rot_dim": 4, "rot": rot, "scale": 0.3}},
            {"type": "latent_attention_2", "mlp": {"kind": "dense", "ff": 24, "limit": 0.75},
             "mixer": {"dim": 10, "heads": 6, "vdim": 4, "kv_rank": 20, "kv_from": 1, "mask": {"size": 5}, "scale": 0.3}},
        ],
    }
    cfg.update(over)
    return cfg


def test_config_is_read_from_json_and_picked_by_architecture(tmp_path):
    from atx.config import model_config_from_json, resolve_model
    from atx.models import napuzen

    cfg = small_cfg()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    m = model_config_from_json(tmp_path / "config.json")
    assert isinstance(m, napuzen.Config) and m.architecture == "Napuzen" and m.recurrent
    assert (m.vocab_size, m.width, m.eps, m.taps, m.logit_scale, m.num_hidden_layers) == (96, 64, 1e-5, 4, 0.5, 4)
    assert resolve_model(str(tmp_path)).config.tensor_shapes() == m.tensor_shapes()
    assert m.kv_bytes_per_token(2) == 2 * (20 + 14 + 4)                      # the sharing layer and the gla layer own no pages
    assert m.state_bytes_per_sequence() == 4 * (3 * 64 * 4 + 3 * 6 * 10)     # taps-1 stream rows per layer + the gla state
    with pytest.raises(ValueError):
        napuzen.Config.from_json(dict(cfg, layers=[{"type": "conv", "mixer": {"dim": 1, "heads": 1}, "mlp": None}]))
    for path, value in ((("layers", 3, "mixer", "kv_from"), 3), (("layers", 3, "mixer", "kv_from"), 0),
                        (("layers", 3, "mixer", "kv_from"), 2), (("layers", 3, "mixer", "kv_rank"), 16),
                        (("layers", 2, "mixer", "rot", "dims"), 6), (("layers", 1, "mlp", "router", "top"), 6),
                        (("layers", 0, "mlp", "kind"), "glu"), (("layers", 0, "mixer", "tau"), 0.0),
                        (("layers", 0, "mlp", "limit"), 0.0), (("canon", "taps"), -1)):
        bad = json.loads(json.dumps(cfg))
        d = bad
        for k in path[:-1]:
            d = d[k]
        d[path[-1]] = value
        with pytest.raises(ValueError):
            napuzen.Config.from_json(bad)
    plain = json.loads(json.dumps(cfg))           # what a configuration leaves out does not exist
    del plain["canon"], plain["logit_scale"], plain["layers"][2]["mixer"]["rot"]["scaling"], plain["layers"][1]["mlp"]["shared"]
    mp = napuzen.Config.from_json(plain)
    assert mp.taps == 0 and mp.logit_scale == 1.0 and "l0.canon1" not in mp.tensor_shapes()
    assert "l1.mlp.shared.sg" not in mp.tensor_shapes()


def test_sizes_that_only_the_tensors_give_are_adopted_from_the_checkpoint():
    from atx.models import napuzen

    cfg = small_cfg()
    cfg["layers"][0]["mixer"]["decay_rank"] = 5          # the reference's checkpoint maker reads it; config.json need not have it
    wt = R.random_checkpoint(cfg, 3)
    del cfg["layers"][0]["mixer"]["decay_rank"], cfg["layers"][2]["mixer"]["q_rank"]
    m = napuzen.Config.from_json(cfg)
    w = napuzen.Weights.from_state_dict(m, wt, torch.device("cpu"), torch.float32)
    assert m.layers[0]["mixer"]["decay_rank"] == 5 and m.layers[2]["mixer"]["q_rank"] == 18
    assert w.layers[0].a2.shape == (18, 5) and w.layers[0].w_in.shape == (2 * 18 + 2 * 30 + 5, 64)


def test_checkpoint_names_and_shapes_match_the_reference_listing():
    from atx.models import napuzen

    cfg = small_cfg()
    m = napuzen.Config.from_json(cfg)
    m.adopt_shapes(lambda name: None)
    assert m.tensor_shapes() == R.checkpoint_shapes(cfg)
    names = set(R.checkpoint_shapes(cfg))
    assert "l3.mix.dkv" not in names and "l1.mix.dkv" in names and "l1.mlp.e4.down" in names and "l2.norm2" not in names
    assert "head" not in names and R.checkpoint_shapes(cfg)["l2.mix.dkv"] == (18, 64) and R.checkpoint_shapes(cfg)["l0.canon1"] == (64, 4)


def test_weights_are_stacked_the_way_the_kernels_read_them():
    from atx.models import napuzen

    cfg = small_cfg()
    wt = R.random_checkpoint(cfg, 1)
    m = napuzen.Config.from_json(cfg)
    w = napuzen.Weights.from_state_dict(m, wt, torch.device("cpu"), torch.float32)
    l0, l1, l2, l3 = w.layers
    assert l0.w_in.shape == (18 + 18 + 30 + 30 + 32, 64) and torch.equal(l0.w_in[36:66].double(), wt["l0.mix.v"])
    assert torch.equal(l0.w_in[96:].double(), wt["l0.mix.a1"])
    assert l1.w_in.shape == (32 + 4 + 20, 64) and torch.equal(l1.w_in[32:36].double(), wt["l1.mix.g"])
    assert l3.w_in.shape == (60 + 6, 64) and l3.dkv_norm is None
    assert l2.w_in.shape == (18 + 18, 64) and torch.equal(l2.w_in[18:].double(), wt["l2.mix.dkv"])
    # W_uk per head, transposed: row h * kv_rank + c holds column c of head h's block
    assert l1.w_ukt.shape == (4 * 20, 8) and torch.equal(l1.w_ukt[2 * 20 + 7].double(), wt["l1.mix.uk"][16:24, 7])
    assert l1.w_router.shape == (6, 64) and torch.equal(l1.w_router[5:].double(), wt["l1.mlp.shared.sg"])
    assert l1.w_egu.shape == (5, 48, 64) and torch.equal(l1.w_egu[3, 24:].double(), wt["l1.mlp.e3.up"])
    assert l0.w_gu.shape == (80, 64) and torch.equal(l0.w_gu[40:].double(), wt["l0.mlp.up"])
    assert (l0.ff, l1.ff, l2.ff, l3.ff) == ("dense", "moe", "", "dense")
    sd = dict(wt)
    del sd["l1.mlp.router"]
    with pytest.raises(KeyError):
        napuzen.Weights.from_state_dict(m, sd, torch.device("cpu"), torch.float32)
    with pytest.raises(ValueError):
        napuzen.Weights.from_state_dict(m, dict(wt, **{"l0.mix.norm": torch.zeros(11)}), torch.device("cpu"), torch.float32)


def test_named_shapes_come_through_the_registry():
    from atx.config import resolve_model

    for name, layers in (("napuzen-tiny", 4), ("napuzen-1b", 16), ("napuzen-8b", 32)):
        c = resolve_model(f"random:{name}:1").config
        assert c.architecture == "Napuzen" and c.num_hidden_layers == layers
        assert [l["type"] for l in c.layers[:4]] == ["gla", "latent_attention_2", "latent_attention_2", "latent_attention"]
        assert all(l["mixer"].get("kv_from") == i - 1 for i, l in enumerate(c.layers) if i % 4 == 2)
    assert c.weight_bytes_per_decode_step(2, 8) > c.weight_bytes_per_decode_step(2, 1)     # more tokens reach more experts
    assert c.decode_kv_bytes(10000) < c.decode_kv_bytes(20000)                             # the unwindowed layers grow


def test_explicit_step_plans_take_and_return_state_slots():
    from atx.kv_cache import BlockAllocator, StateSlotPool
    from atx.scheduler import SamplingParams, Scheduler, Sequence

    alloc, slots = BlockAllocator(16, 16, False), StateSlotPool(2)
    sch = Scheduler(alloc, 4, 64, 64, (), state_slots=slots)
    p = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    a, b = Sequence("a", list(range(20)), p, alloc), Sequence("b", list(range(3)), p, alloc)
    plan = sch.plan_explicit([(a, 18, [0]), (b, 3, [])])
    assert {a.state_slot, b.state_slot} == {0, 1} and slots.num_free == 0
    sch.commit(plan, {})
    c = Sequence("c", [1, 2], p, alloc)
    with pytest.raises(RuntimeError):
        sch.plan_explicit([(c, 2, [])])
    sch.retire(b)
    plan = sch.plan_explicit([(a, 1, [0]), (c, 2, [])])
    assert len(plan.decodes) == 1 and len(plan.prefills) == 1 and c.state_slot is not None and slots.num_free == 0


def test_stretched_frequencies_keep_the_fast_pairs_and_divide_the_slow_ones():
    from atx.models.common import stretched_frequencies

    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    fr, mag = R.stretched_frequencies(32, 10000.0, sc)
    plain, one = R.stretched_frequencies(32, 10000.0, None)
    assert one == 1.0 and mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    lo = math.floor(32 * math.log(64 / (2 * math.pi * 8.0)) / (2 * math.log(10000.0)))
    hi = math.ceil(32 * math.log(64 / (2 * math.pi * 1.0)) / (2 * math.log(10000.0)))
    assert 0 <= lo < hi < 16
    assert torch.equal(fr[:lo + 1], plain[:lo + 1]) and torch.allclose(fr[hi:], plain[hi:] / 4.0)
    mid = slice(lo + 1, hi)
    assert bool(((fr[mid] < plain[mid]) & (fr[mid] > plain[mid] / 4.0)).all())
    for dims, base, s in ((32, 10000.0, sc), (8, 50.0, None), (6, 7.0, {"factor": 2.0, "original": 16, "fast": 64.0, "slow": 0.01})):
        got, gm = stretched_frequencies(base, dims, s)
        want, wm = R.stretched_frequencies(dims, base, s)
        assert torch.allclose(torch.tensor(got, dtype=F64), want, rtol=1e-13) and gm == pytest.approx(wm)
    # adjacent pairs turn; the magnitude scales the turned part and nothing else
    x = torch.randn(5, 2, 8, dtype=F64)
    y = R.rotate_pairs(x, R.stretched_frequencies(8, 50.0, None)[0], 1.5)
    assert torch.allclose(y[0], 1.5 * x[0])
    assert torch.allclose(y[..., 0::2] ** 2 + y[..., 1::2] ** 2, 2.25 * (x[..., 0::2] ** 2 + x[..., 1::2] ** 2))


def test_reference_recurrence_equals_its_sum_over_pairs_and_the_window_is_exact():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(13, d, generator=g, dtype=F64) for d in (5, 5, 7))
    a = torch.rand(13, 5, generator=g, dtype=F64) * 0.6 + 0.4
    assert torch.allclose(R.decayed_outer_recurrence(q, k, v, a), R.decayed_outer_closed_form(q, k, v, a))
    a1 = torch.ones(13, 5, dtype=F64)
    assert torch.allclose(R.decayed_outer_recurrence(q, k, v, a1), torch.tril(q @ k.T) @ v)       # no decay: plain linear attention
    vis = R.visible(12, 4)
    assert vis[11].tolist() == [False] * 8 + [True] * 4 and vis[2].tolist() == [True] * 3 + [False] * 9
    assert R.visible(5, 0).tolist() == torch.tril(torch.ones(5, 5)).bool().tolist()
    u = torch.tensor([[1.0, 2.0], [3.0, 5.0], [7.0, 11.0]], dtype=F64)
    w = torch.tensor([[0.5, 2.0], [0.0, 1.0]], dtype=F64)                   # two taps: the row before, the row itself
    assert R.causal_taps(u, w).tolist() == [[2.0, 2.0], [6.5, 5.0], [15.5, 11.0]]
    z = torch.tensor([[-30.0, 0.0, 30.0]], dtype=F64)
    d = R.channel_decay(torch.ones(1, 1, dtype=F64), torch.ones(1, 1, dtype=F64), z.T.clone(), torch.zeros(3, dtype=F64), 2.0)
    assert torch.allclose(d, torch.sigmoid(z) ** 0.5) and float(d[0, 0]) < 1e-6 and float(d[0, 2]) > 0.999999


def test_reference_clamps_routing_and_absorbed_latent_attention():
    g = torch.Generator().manual_seed(1)
    u = torch.randn(6, 8, generator=g, dtype=F64)
    wt = {"f.gate": torch.eye(8, dtype=F64) * 3, "f.up": -torch.eye(8, dtype=F64) * 3, "f.down": torch.eye(8, dtype=F64)}
    y = R.clamped_glu(u, wt, "f.", 1.0)
    gg, vv = (3 * u).clamp(max=1.0), (-3 * u).clamp(-1.0, 1.0)
    assert torch.allclose(y, gg * torch.sigmoid(1.702 * gg) * (vv + 1.0)) and bool((y[3 * u > 1.0] >= 0).all())
    router = torch.randn(5, 8, generator=g, dtype=F64)
    idx, w = R.route(u, router, 2, 1.75)
    s = torch.softmax(u @ router.T, -1)
    assert torch.allclose(w.sum(-1), torch.full((6,), 1.75, dtype=F64)) and torch.equal(idx, s.topk(2, -1).indices)
    assert torch.allclose(w[:, 0] / w[:, 1], s.gather(1, idx)[:, 0] / s.gather(1, idx)[:, 1])
    # absorbed form: (W_uk^T q) . c and W_uv (sum_j p_j c_j) equal keys and values written out per head
    cfg = small_cfg()
    ck = R.random_checkpoint(cfg, 2)
    c, m = cfg["layers"][1]["mixer"], "l1.mix."
    x = torch.randn(17, 64, generator=g, dtype=F64)
    lat = R.latent_of(x, c, ck, m, 1e-5)
    want = R.latent_mixer_2(x, c, ck, m, 1e-5, lat)
    H, D, V, C = 4, 8, 12, 20
    q = (x @ ck[m + "q"].T).view(17, H, D)
    qa = torch.einsum("thd,hdc->thc", q, ck[m + "uk"].view(H, D, C))
    sc = torch.einsum("ihc,jc->hij", qa, lat) * c["scale"]
    sc = sc.masked_fill(~R.visible(17, 9)[None], float("-inf"))
    ol = torch.einsum("hij,jc->ihc", torch.softmax(sc, -1), lat) * torch.sigmoid(x @ ck[m + "g"].T)[:, :, None]
    o = torch.einsum("ihc,hvc->ihv", ol, ck[m + "uv"].view(H, V, C)).reshape(17, H * V)
    assert torch.allclose(o @ ck[m + "o"].T, want)


def test_reference_is_causal_and_a_borrowed_latent_follows_its_source():
    cfg = small_cfg()
    wt = R.random_checkpoint(cfg, 2)
    toks = [int(t) for t in torch.randint(0, 96, (30,), generator=torch.Generator().manual_seed(0))]
    a = R.forward(cfg, wt, toks)
    assert torch.allclose(a[:17], R.forward(cfg, wt, toks[:17]))
    res_a, res_b = [], []
    wt2 = dict(wt, **{"l1.mix.dkv.norm": wt["l1.mix.dkv.norm"] * 1.5})      # layer 3 reads layer 1's latent: it must change too
    R.forward(cfg, wt, toks, res_a), R.forward(cfg, wt2, toks, res_b)
    assert not torch.allclose(res_a[1], res_b[1])
    only3 = [r - p for r, p in zip(res_a[3:], res_a[2:])], [r - p for r, p in zip(res_b[3:], res_b[2:])]
    assert not torch.allclose(only3[0][0], only3[1][0])
    assert a.shape == (30, 96) and torch.allclose(R.forward(dict(cfg, logit_scale=1.0), wt, toks), 2.0 * a)
