"""Host side of the Zonidra family: configuration and registry, checkpoint names, the weight layout the kernels read,
explicit step plans with state slots, the rescaled rotation frequencies, and the reference against itself (visibility,
unnormalised weights, the pair hash, the shift, routing with its correction and identity experts, shared keys). No GPU."""
import json
import math

import pytest
import torch

from oracle import zonidra_ref as R

F64 = torch.float64


def small_cfg(**over):
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 3.0, "low": 1.0, "high": 5.0, "original": 40}}
    cfg = {
        "architecture": "Zonidra", "embedding": {"scale": 5.0, "bigram": {"buckets": 37, "mul_prev": 11, "mul_cur": 5}},
        "vocab": 96, "width": 64, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "attention", "mlp": {"kind": "dense", "ff": 40},
             "mixer": {"dim": 8, "heads": 4, "kv_heads": 2, "mask": {"size": 9, "keep_first": 3}, "rot": rot, "scale": 0.35, "vdim": 12}},
            {"type": "attention",
             "mlp": {"kind": "moe", "expert": {"ff": 24}, "shared": {"ff": 16},
                     "router": {"experts": 5, "identity": 2, "top": 3, "scale": 1.25}},
             "mixer": {"dim": 8, "heads": 6, "kv_heads": 2, "kv_from": 0, "mask": {"size": 5, "keep_first": 0}, "rot": rot,
                       "scale": 0.3, "vdim": 12}},
            {"type": "attention", "mlp": None,
             "mixer": {"dim": 6, "heads": 2, "kv_heads": 2, "mask": {"size": 7, "keep_first": 9}, "scale": 0.4, "vdim": 10}},
        ],
    }
    cfg.update(over)
    return cfg


def test_config_is_read_from_json_and_picked_by_architecture(tmp_path):
    from atx.config import model_config_from_json, resolve_model
    from atx.models import zonidra

    cfg = small_cfg()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    m = model_config_from_json(tmp_path / "config.json")
    assert isinstance(m, zonidra.Config) and m.architecture == "Zonidra" and m.recurrent
    assert (m.vocab_size, m.width, m.eps, m.embed_scale, m.num_hidden_layers) == (96, 64, 1e-5, 5.0, 3)
    assert m.bigram == {"buckets": 37, "mul_prev": 11, "mul_cur": 5}
    assert resolve_model(str(tmp_path)).config.tensor_shapes() == m.tensor_shapes()
    assert m.kv_bytes_per_token(2) == 2 * 2 * (8 + 12) + 2 * 2 * (6 + 10)          # the sharing layer owns no pages
    assert m.state_bytes_per_sequence() == 4 + 3 * 64 * 4
    for bad_layer in ({"type": "conv", "mixer": {}, "mlp": None},):
        with pytest.raises(ValueError):
            zonidra.Config.from_json(dict(cfg, layers=[bad_layer]))
    for path, value in ((("layers", 1, "mixer", "kv_from"), 2), (("layers", 1, "mixer", "kv_from"), 1),
                        (("layers", 1, "mixer", "vdim"), 16), (("layers", 0, "mixer", "rot", "dims"), 10),
                        (("layers", 1, "mlp", "router", "top"), 8), (("layers", 0, "mlp", "kind"), "glu")):
        bad = json.loads(json.dumps(cfg))
        d = bad
        for k in path[:-1]:
            d = d[k]
        d[path[-1]] = value
        with pytest.raises(ValueError):
            zonidra.Config.from_json(bad)
    plain = json.loads(json.dumps(cfg))           # what a configuration leaves out does not exist
    del plain["embedding"]["bigram"], plain["layers"][0]["mixer"]["rot"]["scaling"], plain["layers"][1]["mixer"]["rot"]["scaling"]
    mp = zonidra.Config.from_json(plain)
    assert mp.bigram is None and "bigram" not in mp.tensor_shapes()


def test_checkpoint_names_and_shapes_match_the_reference_listing():
    from atx.models import zonidra

    cfg = small_cfg()
    assert zonidra.Config.from_json(cfg).tensor_shapes() == R.checkpoint_shapes(cfg)
    names = set(R.checkpoint_shapes(cfg))
    assert "l1.mix.k" not in names and "l1.mlp.e4.down" in names and "l1.mlp.shared.sg" in names and "l2.norm2" not in names
    assert R.checkpoint_shapes(cfg)["bigram"] == (38, 64) and R.checkpoint_shapes(cfg)["l1.mlp.router"] == (7, 64)


def test_weights_are_stacked_the_way_the_kernels_read_them():
    from atx.models import zonidra

    cfg = small_cfg()
    wt = R.random_checkpoint(cfg, 1)
    m = zonidra.Config.from_json(cfg)
    w = zonidra.Weights.from_state_dict(m, wt, torch.device("cpu"), torch.float32)
    l0, l1, l2 = w.layers
    assert l0.w_in.shape == (4 * 8 + 2 * 8 + 2 * 12 + 4 * 12, 64) and l1.w_in.shape == (6 * 8 + 6 * 12, 64)
    assert torch.equal(l1.w_in[:48].double(), wt["l1.mix.q"]) and torch.equal(l1.w_in[48:].double(), wt["l1.mix.g"])
    assert torch.equal(l0.w_in[32:48].double(), wt["l0.mix.k"]) and torch.equal(l0.w_in[48:72].double(), wt["l0.mix.v"])
    assert l1.w_router.shape == (8, 64) and torch.equal(l1.w_router[7:].double(), wt["l1.mlp.shared.sg"])
    assert l1.w_egu.shape == (5, 48, 64) and torch.equal(l1.w_egu[3, 24:].double(), wt["l1.mlp.e3.up"])
    assert l1.w_edown.shape == (5, 64, 24) and l0.act.dtype == torch.float32 and l0.pb.dtype == torch.float32
    assert l2.ff == "" and l0.ff == "dense" and l1.ff == "moe"
    sd = dict(wt)
    del sd["l1.mlp.correction"]
    with pytest.raises(KeyError):
        zonidra.Weights.from_state_dict(m, sd, torch.device("cpu"), torch.float32)
    sd = dict(wt, **{"l0.mix.pb": torch.zeros(5)})
    with pytest.raises(ValueError):
        zonidra.Weights.from_state_dict(m, sd, torch.device("cpu"), torch.float32)


def test_named_shapes_come_through_the_registry():
    from atx.config import resolve_model

    for name, layers in (("zonidra-tiny", 2), ("zonidra-1b", 16), ("zonidra-8b", 32)):
        c = resolve_model(f"random:{name}:1").config
        assert c.architecture == "Zonidra" and c.num_hidden_layers == layers
        assert all(l["mixer"].get("kv_from") == i - 1 for i, l in enumerate(c.layers) if i % 2)
    assert c.weight_bytes_per_decode_step(2, 8) > c.weight_bytes_per_decode_step(2, 1)     # more tokens reach more experts


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
    assert slots.num_free == 1
    plan = sch.plan_explicit([(a, 1, [0]), (c, 2, [])])
    assert len(plan.decodes) == 1 and len(plan.prefills) == 1 and c.state_slot is not None and slots.num_free == 0


def test_rescaled_frequencies_keep_stretch_and_interpolate():
    from atx.models.common import wavelength_scaled_frequencies

    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    fr = R.rescaled_frequencies(16, 1000.0, sc)
    plain = R.rescaled_frequencies(16, 1000.0, None)
    wl = 2 * math.pi / plain
    assert torch.equal(fr[wl < 16], plain[wl < 16]) and torch.allclose(fr[wl > 64], plain[wl > 64] / 4.0)
    mid = (wl >= 16) & (wl <= 64)
    assert mid.any() and bool(((fr[mid] < plain[mid]) & (fr[mid] > plain[mid] / 4.0)).all())
    assert torch.allclose(torch.tensor(wavelength_scaled_frequencies(1000.0, 16, sc), dtype=F64), fr, rtol=1e-13)
    assert torch.allclose(torch.tensor(wavelength_scaled_frequencies(1000.0, 16, None), dtype=F64), plain, rtol=1e-13)
    # the pairing: a rotation of element i with element i + dims / 2 keeps the pair's length and leaves the tail alone
    x = torch.randn(5, 2, 12, dtype=F64)
    y = R.rotate_halves(x, 8, R.rescaled_frequencies(8, 50.0, None))
    assert torch.allclose(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose(y[..., :4] ** 2 + y[..., 4:8] ** 2, x[..., :4] ** 2 + x[..., 4:8] ** 2)


def test_reference_visibility_weights_hash_and_shift():
    vis = R.visible(12, 4, 2)
    assert vis[11].tolist() == [True, True] + [False] * 6 + [True] * 4 and vis[3].tolist() == [True] * 4 + [False] * 8
    q, k, v = torch.zeros(3, 1, 2, dtype=F64), torch.zeros(3, 1, 2, dtype=F64), torch.ones(3, 1, 1, dtype=F64)
    out = R.sigmoid_attention(q, k, v, 1.0, torch.zeros(1, dtype=F64), R.visible(3, 3, 0))
    assert out.flatten().tolist() == [0.5, 1.0, 1.5]          # weights of 1/2 each, never normalised
    assert R.bigram_rows([3, 4, 3], 7, 2, 5) == [7, (3 * 2 + 4 * 5) % 7, (4 * 2 + 3 * 5) % 7]
    u = torch.tensor([[1.0, 1.0], [3.0, 5.0]], dtype=F64)
    assert R.token_shift(u, torch.tensor([0.5, 0.0], dtype=F64)).tolist() == [[0.5, 1.0], [2.0, 5.0]]
    z = torch.randn(4, 9, dtype=F64)
    p = R.poly_norm(z, torch.tensor([0.0, 1.0, 0.0, 2.0], dtype=F64), 0.0)
    assert torch.allclose(((p - 2.0) ** 2).mean(-1), torch.ones(4, dtype=F64))


def test_reference_routing_correction_identity_and_shared_keys():
    u = torch.randn(6, 8, dtype=F64)
    router = torch.randn(5, 8, dtype=F64)
    corr = torch.tensor([0.0, 0.0, 0.0, 0.0, 10.0], dtype=F64)        # the correction decides the choice, not the weight
    idx, w = R.route(u, router, corr, 2, 1.5)
    s = torch.softmax(u @ router.T, -1)
    assert (idx[:, 0] == 4).all() and torch.allclose(w[:, 0], 1.5 * s[:, 4])
    cfg = small_cfg()
    wt = R.random_checkpoint(cfg, 2)
    c = cfg["layers"][1]["mlp"]
    wt2 = dict(wt, **{"l1.mlp.correction": torch.tensor([-9.0] * 5 + [9.0, 9.0], dtype=F64)})
    only_ident = dict(c, router=dict(c["router"], top=2), shared=None)
    y = R.expert_mixture(u.repeat(1, 8), only_ident, wt2, "l1.mlp.")
    s = torch.softmax(u.repeat(1, 8) @ wt["l1.mlp.router"].T, -1)
    assert torch.allclose(y, 1.25 * (s[:, 5] + s[:, 6])[:, None] * u.repeat(1, 8))
    toks = [int(t) for t in torch.randint(0, 96, (30,), generator=torch.Generator().manual_seed(0))]
    a = R.forward(cfg, wt, toks)
    wt3 = dict(wt, **{"l0.mix.k": wt["l0.mix.k"] * 1.5})              # layer 1 reads layer 0's keys: it must change too
    res_a, res_b = [], []
    R.forward(cfg, wt, toks, res_a), R.forward(cfg, wt3, toks, res_b)
    assert not torch.allclose(res_a[0], res_b[0])
    b = R.forward(cfg, wt, toks[:17])
    assert torch.allclose(a[:17], b)                                   # causal
