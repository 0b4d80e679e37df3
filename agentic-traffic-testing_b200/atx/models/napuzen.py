"""Napuzen: a decoder-only family whose layers are listed one by one in config.json.

    x_t = embed[token_t]
    x  <- x + rms(mixer(x + taps(x))) w1          taps(x)_t = sum_j c[:, j] x_(t - K + 1 + j): a causal convolution per channel
    x  <- x + rms(ffn(x)) w2                                                                   (ffn optional)
    logits = logit_scale * embed . (rms(x) w_final)

A norm stands only BEHIND each sublayer; the sublayers read the stream itself. Three mixers:

* `gla`: linear attention whose state decays per key channel, S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t / sqrt(dim)
  with a_t = sigmoid(A2 (A1 u) + b)^(1/tau); every head's output is RMS-normed with one weight vector shared by the heads,
  multiplied by silu(W_g u) and projected.
* `latent_attention`: soft-max attention over a cached latent. Queries through a normed bottleneck, per head
  [dim plain | rot_dim rotated]; W_dkv gives [latent (normed) | one rotated key part shared by all heads]; keys W_uk c, values
  W_uv c. Rotation of adjacent pairs with frequencies stretched by pair index and a magnitude on cos / sin.
* `latent_attention_2`: the same without positions: plain queries, a sliding window, sigmoid(W_g u) per head on the output;
  a layer with `kv_from: j` has no W_dkv and reads layer j's cached latent with its own W_uk / W_uv.

Both attention mixers run in the absorbed form: only the latent row is cached, the query of head h becomes W_uk,h^T q_h (plus
its rotated part), attention runs as ONE key/value head shared by all query heads whose value is the row's leading kv_rank
elements, and W_uv,h is applied to the head's result. Prompt portions and decoded tokens take the same path.

The feed-forward is dense, W_down (g sigmoid(1.702 g) (v + 1)) with g = min(W_gate x, limit), v = clamp(W_up x, +-limit), or
a mixture of gated experts: soft-max router, the `top` largest scores chosen, divided by their sum, times router.scale,
plus a shared expert times sigmoid(W_sg x).

State besides the pages, per live sequence (a state slot): the last taps-1 stream rows of every layer (fp32) and the
[heads, dim, vdim] fp32 state of every gla layer.

fp32 whatever the element type: the residual stream, every norm, the convolution's sum, decays and their logarithms, the
recurrence and its state, rotation, attention scores and weights, router, expert weights and the weighted sum. Projections run
in the element type (bf16 on the tcgen05 GEMM and the tensor-core head / expert products, or fp32 on the FMA pipe) with fp32
accumulation.

The program below only issues kernels; scheduling, pages, state slots, staging, sampling and the step loop are the runner's
and the engine's (atx/runner.py, atx/engine.py)."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch

from .. import _cabi
from .common import _Linear, _use_tc, rotation_table_scaled, stretched_frequencies

MIXERS = ("gla", "latent_attention", "latent_attention_2")
GLU_ALPHA = 1.702      # the dense feed-forward's gate is g * sigmoid(GLU_ALPHA * g) ...
GLU_SHIFT = 1.0        # ... times (up + GLU_SHIFT)
DEFAULT_DECAY_RANK = 32

# ---- configuration --------------------------------------------------------------------------------------------------


def _rot_key(c: dict) -> Optional[tuple]:
    rot = c.get("rot") or {}
    dims = int(rot.get("dims", 0) or 0)
    if not dims:
        return None
    sc = rot.get("scaling") or None
    return (float(rot.get("base", 10000.0)), dims,
            tuple(float(sc[k]) for k in ("factor", "original", "fast", "slow")) if sc else None)


@dataclass
class Config:
    name: str = "napuzen"
    vocab_size: int = 0
    width: int = 0
    eps: float = 1e-6
    taps: int = 0                                      # canon.taps: length of the convolution in front of every mixer (0: none)
    logit_scale: float = 1.0
    layers: List[dict] = field(default_factory=list)   # {"type", "mixer", "mlp"} as in config.json
    eos_token_ids: tuple = ()
    bos_token_id: int = 0
    max_position_embeddings: int = 131072    # the design sets no limit; this bounds the server's default max_model_len
    architecture = "Napuzen"
    recurrent = True      # a state slot per sequence: convolution rows of every layer, states of the gla layers

    @classmethod
    def from_json(cls, d: dict, name: str = "napuzen") -> "Config":
        cfg = cls(name=name, vocab_size=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]),
                  taps=int((d.get("canon") or {}).get("taps", 0) or 0), logit_scale=float(d.get("logit_scale", 1.0)),
                  layers=[json.loads(json.dumps(l)) for l in d["layers"]])
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.taps < 0:
            raise ValueError(f"canon.taps={self.taps} must not be negative")
        for i, l in enumerate(self.layers):
            if l["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            c = l["mixer"] = dict(l["mixer"])
            c.setdefault("vdim", c["dim"])
            if l["type"] == "gla":
                if float(c["tau"]) <= 0:
                    raise ValueError(f"layer {i}: tau must be positive")
            elif l["type"] == "latent_attention":
                c.setdefault("rot_dim", 0)
                rk = _rot_key(c)
                if c["rot_dim"] and (rk is None or rk[1] % 2 or rk[1] > c["rot_dim"]):
                    raise ValueError(f"layer {i}: rot.dims must be even and at most rot_dim={c['rot_dim']}")
            else:
                src = c.get("kv_from")
                if src is not None:
                    src = int(src)
                    o = self.layers[src] if 0 <= src < i else None
                    if o is None or o["type"] != "latent_attention_2" or o["mixer"].get("kv_from") is not None:
                        raise ValueError(f"layer {i}: kv_from={src} must name an earlier latent_attention_2 layer with a latent of its own")
                    if int(o["mixer"]["kv_rank"]) != int(c["kv_rank"]):
                        raise ValueError(f"layer {i}: shares layer {src}'s latent but kv_rank differs")
            if int((c.get("mask") or {}).get("size", 0) or 0) < 0:
                raise ValueError(f"layer {i}: negative mask size")
            mlp = l.get("mlp")
            if mlp is not None:
                kind = mlp.get("kind", "dense")
                if kind == "moe":
                    r = mlp["router"]
                    if not 0 < int(r["top"]) <= int(r["experts"]):
                        raise ValueError(f"layer {i}: top={r['top']} of {r['experts']} experts")
                elif kind == "dense":
                    if float(mlp["limit"]) <= 0:
                        raise ValueError(f"layer {i}: limit must be positive")
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")

    def adopt_shapes(self, shape_of) -> None:
        """Sizes that config.json leaves to the tensors: the rank of a gla layer's decay projection (and a latent layer's
        query bottleneck, if it is not given). shape_of(name) -> shape or None."""
        for i, l in enumerate(self.layers):
            c = l["mixer"]
            if l["type"] == "gla" and "decay_rank" not in c:
                sh = shape_of(f"l{i}.mix.a1")
                c["decay_rank"] = int(sh[0]) if sh else DEFAULT_DECAY_RANK
            if l["type"] == "latent_attention" and "q_rank" not in c:
                sh = shape_of(f"l{i}.mix.dq")
                if sh:
                    c["q_rank"] = int(sh[0])

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def tensor_shapes(self) -> Dict[str, Tuple[int, ...]]:
        """Name -> shape of every tensor of a checkpoint of this configuration."""
        W, out = self.width, {}
        out["embed"] = (self.vocab_size, W)
        for i, l in enumerate(self.layers):
            p, c, m = f"l{i}.", l["mixer"], f"l{i}.mix."
            H, D, V = int(c["heads"]), int(c["dim"]), int(c["vdim"])
            out[p + "norm1"] = (W,)
            if self.taps:
                out[p + "canon1"] = (W, self.taps)
            if l["type"] == "gla":
                rk = int(c.get("decay_rank", DEFAULT_DECAY_RANK))
                out.update({m + "q": (H * D, W), m + "k": (H * D, W), m + "v": (H * V, W), m + "g": (H * V, W),
                            m + "o": (W, H * V), m + "norm": (V,), m + "a1": (rk, W), m + "a2": (H * D, rk),
                            m + "a2.b": (H * D,)})
            elif l["type"] == "latent_attention":
                R, C, Q = int(c["rot_dim"]), int(c["kv_rank"]), int(c["q_rank"])
                out.update({m + "dq": (Q, W), m + "dq.norm": (Q,), m + "uq": (H * (D + R), Q), m + "dkv": (C + R, W),
                            m + "dkv.norm": (C,), m + "uk": (H * D, C), m + "uv": (H * V, C), m + "o": (W, H * V)})
            else:
                C = int(c["kv_rank"])
                out.update({m + "q": (H * D, W), m + "uk": (H * D, C), m + "uv": (H * V, C), m + "g": (H, W),
                            m + "o": (W, H * V)})
                if c.get("kv_from") is None:
                    out.update({m + "dkv": (C, W), m + "dkv.norm": (C,)})
            mlp = l.get("mlp")
            if mlp is None:
                continue
            out[p + "norm2"] = (W,)
            f = p + "mlp."
            if mlp.get("kind", "dense") == "dense":
                F = int(mlp["ff"])
                out.update({f + "gate": (F, W), f + "up": (F, W), f + "down": (W, F)})
            else:
                E, F = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
                for e in range(E):
                    out[f"{f}e{e}.gate"], out[f"{f}e{e}.up"], out[f"{f}e{e}.down"] = (F, W), (F, W), (W, F)
                out[f + "router"] = (E, W)
                if mlp.get("shared"):
                    S = int(mlp["shared"]["ff"])
                    out.update({f + "shared.gate": (S, W), f + "shared.up": (S, W), f + "shared.down": (W, S),
                                f + "shared.sg": (1, W)})
        out["final.norm"] = (W,)
        return out

    # ---- bytes, for the benchmarks' rooflines -------------------------------------------------------------------
    def weight_bytes_per_decode_step(self, elem: int = 2, tokens: int = 1) -> int:
        """Weight bytes a decode step of `tokens` tokens streams: every matrix (the embedding table once, as the output
        head); of the routed experts at most tokens * top per layer."""
        n = 0
        for k, v in self.tensor_shapes().items():
            if ".mlp.e" in k:
                continue
            n += math.prod(v)
        for l in self.layers:
            mlp = l.get("mlp")
            if mlp is not None and mlp.get("kind") == "moe":
                r = mlp["router"]
                n += min(int(r["experts"]), tokens * int(r["top"])) * 3 * int(mlp["expert"]["ff"]) * self.width
        return elem * n

    def latent_row(self, i: int) -> int:
        """Elements of a cached row of layer i (0: the layer caches nothing of its own)."""
        l, c = self.layers[i], self.layers[i]["mixer"]
        if l["type"] == "latent_attention":
            return int(c["kv_rank"]) + int(c["rot_dim"])
        if l["type"] == "latent_attention_2" and c.get("kv_from") is None:
            return int(c["kv_rank"])
        return 0

    def kv_bytes_per_token(self, elem: int = 2) -> int:
        return sum(self.latent_row(i) for i in range(len(self.layers))) * elem

    def state_bytes_per_sequence(self) -> int:
        n = max(0, self.taps - 1) * self.width * len(self.layers)
        for l in self.layers:
            if l["type"] == "gla":
                c = l["mixer"]
                n += int(c["heads"]) * int(c["dim"]) * int(c["vdim"])
        return 4 * n

    def decode_kv_bytes(self, ctx: int, elem: int = 2) -> int:
        """Page bytes one decoded token at context length ctx reads: every attention layer its window of latent rows."""
        n = 0
        for i, l in enumerate(self.layers):
            if l["type"] == "gla":
                continue
            c = l["mixer"]
            size = int((c.get("mask") or {}).get("size", 0) or 0)
            src = c.get("kv_from")
            n += (min(ctx, size) if size else ctx) * self.latent_row(i if src is None else int(src)) * elem
        return n


def named_shape(name: str) -> Optional[Config]:
    """`random:napuzen-<size>`: shapes whose layers resemble a real model's, for benchmarks (no checkpoint exists).
    `napuzen-8b` / `napuzen-1b` have the width, feed-forward size, vocabulary and depth of the Llama 8B / 1B shapes; layers
    in the pattern gla + dense feed-forward, windowed latent attention + experts, the same over the previous layer's
    latent + experts, rotated latent attention + dense feed-forward."""
    key = name.lower()
    shapes = {"napuzen-8b": (4096, 14336, 8, 128256), "napuzen-1b": (2048, 8192, 4, 128256),
              "napuzen-tiny": (256, 512, 1, 1024)}     # width, feed-forward, repeats of the 4-layer pattern, vocabulary
    if key not in shapes:
        return None
    W, F, groups, vocab = shapes[key]
    hd = 128 if W >= 4096 else 64
    heads = W // hd
    Fe = max(64, F // 4 // 64 * 64)
    gla = {"dim": 64, "heads": heads, "vdim": hd, "tau": 8.0, "decay_rank": 32}
    lat2 = {"dim": hd, "heads": heads, "vdim": hd, "kv_rank": 128, "scale": hd ** -0.5, "mask": {"size": 2048}}
    lat = {"dim": hd, "heads": heads, "vdim": hd, "kv_rank": 128, "q_rank": W * 3 // 8, "rot_dim": 64,
           "scale": (hd + 64) ** -0.5,
           "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}
    moe = {"kind": "moe", "expert": {"ff": Fe}, "shared": {"ff": Fe}, "router": {"experts": 8, "top": 2, "scale": 1.0}}
    dense = {"kind": "dense", "ff": F, "limit": 7.0}
    layers = []
    for g in range(groups):
        layers.append({"type": "gla", "mixer": dict(gla), "mlp": dict(dense)})
        layers.append({"type": "latent_attention_2", "mixer": dict(lat2), "mlp": dict(moe)})
        layers.append({"type": "latent_attention_2", "mixer": dict(lat2, kv_from=4 * g + 1), "mlp": dict(moe)})
        layers.append({"type": "latent_attention", "mixer": dict(lat), "mlp": dict(dense)})
    cfg = Config(name=key, vocab_size=vocab, width=W, eps=1e-6, taps=4, logit_scale=1.0,
                 layers=json.loads(json.dumps(layers)))
    cfg.validate()
    return cfg


# ---- weights ----------------------------------------------------------------------------------------------------------


class _Layer:
    """Device tensors of one layer in the layout the kernels read (projections that share an input are stacked)."""

    def __init__(self) -> None:
        self.kind = ""
        self.norm1 = self.norm2 = self.canon = None
        self.w_in = self.w_o = None          # gla: [q | k | v | g | a1]; latent: [dq | dkv]; latent 2: [q | g | dkv]
        self.a2 = self.a2_b = self.mix_norm = None                    # gla
        self.dq_norm = self.dkv_norm = self.w_uq = None               # latent bottlenecks
        self.w_ukt = self.w_uv = None        # [heads * kv_rank, dim] (W_uk per head, transposed), [heads * vdim, kv_rank]
        self.ff = ""                         # "", "dense", "moe"
        self.w_gu = self.w_down = None       # dense: [gate rows ; up rows], or in blocks of 64 (gu_interleaved)
        self.gu_interleaved = False
        self.w_router = None                 # [experts (+ 1: the shared expert's gate), width]
        self.w_egu = self.w_edown = None     # [experts, 2 ff, width], [experts, width, ff]
        self.w_sgu = self.w_sdown = None     # shared expert
        self.sgu_interleaved = False
        self.egu_interleaved = False         # gate / up rows of every expert in blocks of 64, as the gated GEMM epilogue reads them


class Weights:
    def __init__(self, cfg: Config, device: torch.device, dtype: torch.dtype):
        self.cfg, self.device, self.dtype = cfg, device, dtype
        self.embed = self.final_norm = None
        self.layers: List[_Layer] = []
        self.tp_size, self.tp_rank = 1, 0

    def nbytes(self) -> int:
        ts = [self.embed, self.final_norm]
        for l in self.layers:
            ts += [v for v in vars(l).values() if isinstance(v, torch.Tensor)]
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
        g = torch.Generator(device=device).manual_seed(1000 * seed + 17)
        cfg.adopt_shapes(lambda name: None)
        shapes = cfg.tensor_shapes()

        class _Gen:
            def has(self, name):
                return name in shapes

            def shape(self, name):
                return shapes[name]

            def full(self, name):
                sh = shapes[name]
                if name.endswith("a2.b"):
                    return 2.0 + torch.randn(sh, generator=g, device=device)
                if name.endswith("canon1"):
                    return 0.3 * torch.randn(sh, generator=g, device=device)
                if len(sh) == 2:
                    return torch.randn(sh, generator=g, device=device) * (sh[1] ** -0.5)
                return 1.0 + 0.1 * torch.randn(sh, generator=g, device=device)

        return cls._from_source(cfg, _Gen(), device, dtype)

    @classmethod
    def _from_source(cls, cfg: Config, src, device: torch.device, dtype: torch.dtype) -> "Weights":
        w = cls(cfg, device, dtype)
        cfg.adopt_shapes(lambda name: tuple(src.shape(name)) if src.has(name) else None)
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

        def gate_up(gate: torch.Tensor, up: torch.Tensor) -> Tuple[torch.Tensor, bool]:
            if _use_tc(dtype, cfg.width) and gate.shape[0] % 64 == 0:
                from ..weights import interleave_gate_up

                return dev(interleave_gate_up(gate, up)), True
            return dev(torch.cat([gate, up], 0)), False

        W = cfg.width
        w.embed, w.final_norm = dev(get("embed")), dev(get("final.norm"))
        for i, spec in enumerate(cfg.layers):
            p, c, l = f"l{i}.", spec["mixer"], _Layer()
            m = p + "mix."
            l.kind = spec["type"]
            l.norm1 = dev(get(p + "norm1"))
            if cfg.taps:
                l.canon = dev(get(p + "canon1"))
            H, D, V = int(c["heads"]), int(c["dim"]), int(c["vdim"])
            if l.kind == "gla":
                l.w_in = dev(torch.cat([get(m + nm) for nm in ("q", "k", "v", "g", "a1")], 0))
                l.a2, l.a2_b, l.mix_norm = dev(get(m + "a2")), dev(get(m + "a2.b")), dev(get(m + "norm"))
            else:
                C = int(c["kv_rank"])
                if l.kind == "latent_attention":
                    l.w_in = dev(torch.cat([get(m + "dq"), get(m + "dkv")], 0))
                    l.dq_norm, l.dkv_norm, l.w_uq = dev(get(m + "dq.norm")), dev(get(m + "dkv.norm")), dev(get(m + "uq"))
                else:
                    own = c.get("kv_from") is None
                    l.w_in = dev(torch.cat([get(m + "q"), get(m + "g")] + ([get(m + "dkv")] if own else []), 0))
                    if own:
                        l.dkv_norm = dev(get(m + "dkv.norm"))
                l.w_ukt = dev(get(m + "uk").reshape(H, D, C).transpose(1, 2).reshape(H * C, D))
                l.w_uv = dev(get(m + "uv"))
            l.w_o = dev(get(m + "o"))
            mlp = spec.get("mlp")
            if mlp is not None:
                l.norm2 = dev(get(p + "norm2"))
                f = p + "mlp."
                if mlp.get("kind", "dense") == "dense":
                    l.ff = "dense"
                    (l.w_gu, l.gu_interleaved), l.w_down = gate_up(get(f + "gate"), get(f + "up")), dev(get(f + "down"))
                else:
                    l.ff = "moe"
                    E, Fe = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
                    l.w_router = dev(torch.cat([get(f + "router")] + ([get(f + "shared.sg")] if mlp.get("shared") else []), 0))
                    pairs = [gate_up(get(f"{f}e{e}.gate"), get(f"{f}e{e}.up")) for e in range(E)]
                    l.egu_interleaved = pairs[0][1]
                    l.w_egu = torch.stack([t for t, _ in pairs], 0).contiguous()
                    l.w_edown = torch.stack([dev(get(f"{f}e{e}.down")) for e in range(E)], 0).contiguous()
                    if mlp.get("shared"):
                        l.w_sgu, l.sgu_interleaved = gate_up(get(f + "shared.gate"), get(f + "shared.up"))
                        l.w_sdown = dev(get(f + "shared.down"))
            w.layers.append(l)
        return w


# ---- the layer program ------------------------------------------------------------------------------------------------


def _pad4(n: int) -> int:
    return (n + 3) // 4 * 4


class Program:
    needs_seq_view = True     # kernels walk the step sequence by sequence (ModelRunner._stage_seq)
    graph_safe = True         # a row staged without a sequence is skipped by every kernel that touches pages or state

    def __init__(self, r) -> None:
        self.r = r
        cfg: Config = r.m
        w: Weights = r.w
        e = r.e
        self.cfg, self.w = cfg, w
        if e.tp_size != 1:
            raise ValueError("Napuzen runs on one GPU per replica")
        xt = w.dtype
        self.dt = _cabi.DT_F32 if xt == torch.float32 else _cabi.DT_BF16
        self.xt, self.esz = xt, (4 if xt == torch.float32 else 2)
        dev, T, lib = r.dev, r.Tmax, r.lib
        W = cfg.width
        f32, i32 = torch.float32, torch.int32
        n_in = n_q2 = n_qb = n_lat = n_mix = n_cq = n_rec = n_dec = 1
        n_up = n_act = n_rl = n_pairs = n_ef = n_exp = 1
        for spec in cfg.layers:
            c = spec["mixer"]
            H, D, V = int(c["heads"]), int(c["dim"]), int(c["vdim"])
            n_mix = max(n_mix, H * V)
            if spec["type"] == "gla":
                n_in = max(n_in, 2 * H * D + 2 * H * V + int(c["decay_rank"]))
                n_rec, n_dec = max(n_rec, H * V), max(n_dec, H * D)
            elif spec["type"] == "latent_attention":
                R, C, Q = int(c["rot_dim"]), int(c["kv_rank"]), int(c["q_rank"])
                n_in, n_q2, n_cq = max(n_in, Q + C + R), max(n_q2, H * (D + R)), max(n_cq, Q)
                n_qb, n_lat = max(n_qb, H * (C + R)), max(n_lat, H * C)
            else:
                C = int(c["kv_rank"])
                n_in = max(n_in, H * D + H + (C if c.get("kv_from") is None else 0))
                n_qb, n_lat = max(n_qb, H * C), max(n_lat, H * C)
            mlp = spec.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind", "dense") == "dense":
                n_up, n_act = max(n_up, 2 * int(mlp["ff"])), max(n_act, int(mlp["ff"]))
            else:
                rt = mlp["router"]
                n_rl = max(n_rl, int(rt["experts"]) + 1)
                n_pairs, n_ef, n_exp = max(n_pairs, int(rt["top"])), max(n_ef, int(mlp["expert"]["ff"])), max(n_exp, int(rt["experts"]))
                if mlp.get("shared"):
                    n_act = max(n_act, int(mlp["shared"]["ff"]))
                    n_up = max(n_up, 2 * int(mlp["shared"]["ff"]))     # gate | up when the epilogue cannot fuse them
        self.h = torch.zeros(T, W, dtype=f32, device=dev)          # residual stream
        self.y = torch.zeros(T, W, dtype=f32, device=dev)          # a sublayer's output before its post-norm
        # fp32 GEMM outputs of a sublayer, back to back so that one pass clears what split-K accumulates into: the mixer's
        # [input projections | expanded queries]; then, in the same space, [feed-forward gate / up | router outputs]
        self.scratch = torch.zeros(T * max(_pad4(n_in) + _pad4(n_q2), _pad4(n_up) + _pad4(n_rl)) + 32, dtype=f32, device=dev)
        self.rec = torch.zeros(T * n_rec, dtype=f32, device=dev)   # recurrence output
        self.ldec = torch.zeros(T * n_dec, dtype=f32, device=dev)  # logarithms of the decays
        self.xn = torch.zeros(T, W, dtype=xt, device=dev)
        self.cq_flat = torch.zeros(T * n_cq, dtype=xt, device=dev)
        self.q_flat = torch.zeros(T * n_qb, dtype=xt, device=dev)
        self.lat_flat = torch.zeros(T * n_lat, dtype=xt, device=dev)
        self.mix_flat = torch.zeros(T * n_mix, dtype=xt, device=dev)
        self.act_flat = torch.zeros(T * n_act, dtype=xt, device=dev)
        self.xl = torch.zeros(r.Rmax, W, dtype=xt, device=dev)
        # mixture of experts: choices, weights, the plan, the experts' hidden rows and outputs per (token, choice) slot
        self.tile_rows = int(lib.atx_moe_tile_rows())
        P = T * n_pairs
        self.max_tiles = max((P + self.tile_rows - 1) // self.tile_rows, (min(P, 64 * n_pairs) + 15) // 16) + n_exp
        self.sel = torch.zeros(P, dtype=i32, device=dev)
        self.wgt = torch.zeros(P, dtype=f32, device=dev)
        self.seg_off = torch.zeros(n_exp + 1, dtype=i32, device=dev)
        self.perm = torch.zeros(P, dtype=i32, device=dev)
        self.slot_of = torch.zeros(P, dtype=i32, device=dev)
        self.tiles = torch.zeros(2 + 2 * self.max_tiles, dtype=i32, device=dev)
        self.eact = torch.zeros(P * n_ef if n_exp > 1 or n_ef > 1 else 1, dtype=xt, device=dev)
        self.big_rows = int(lib.atx_gemm_grouped_tile_rows())
        self.max_big_tiles = (P + self.big_rows - 1) // self.big_rows + n_exp
        grouped = any(l.egu_interleaved for l in w.layers)
        self.xperm = torch.zeros(P if grouped else 1, W, dtype=xt, device=dev)
        self.tiles_big = torch.zeros(2 + 2 * self.max_big_tiles, dtype=i32, device=dev)
        self.ye = torch.zeros(P * W if n_ef > 1 else 1, dtype=f32, device=dev)
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
            if l.ff == "dense":
                d["gu"] = _Linear(lib, l.w_gu, self.xn, self.dt)
                if l.gu_interleaved:     # the clamps and the gate run in the GEMM's epilogue
                    d["gu"].plan.set_gate(GLU_ALPHA, float(spec["mlp"]["limit"]), GLU_SHIFT)
                d["down"] = _Linear(lib, l.w_down, view(self.act_flat, l.w_down.shape[1]), self.dt)
            elif l.ff == "moe":
                d["router"] = _Linear(lib, l.w_router, self.xn, self.dt)
                if l.egu_interleaved:
                    E_, F2, Fe_ = l.w_egu.shape[0], l.w_egu.shape[1], l.w_edown.shape[2]
                    d["egu"] = _cabi.GemmPlan(l.w_egu.view(E_ * F2, W), self.xperm)
                    d["edown"] = _cabi.GemmPlan(l.w_edown.view(E_ * W, Fe_), self.eact[:P * Fe_].view(P, Fe_))
                if l.w_sgu is not None:
                    d["sgu"] = _Linear(lib, l.w_sgu, self.xn, self.dt)
                    d["sdown"] = _Linear(lib, l.w_sdown, view(self.act_flat, l.w_sdown.shape[1]), self.dt)
            self.lin.append(d)
        self.lin_head = _Linear(lib, w.embed, self.xl, self.dt)     # the output head is the embedding table

        # ---- pages: one latent row per token and layer that has a latent of its own; a sharing layer reads its source's
        bs = r.bs
        page_bytes = max(1, cfg.kv_bytes_per_token(self.esz)) * bs
        if e.num_gpu_blocks is not None:
            nb = int(e.num_gpu_blocks)
        else:
            free, total = torch.cuda.mem_get_info(dev)
            budget = int(total * e.gpu_memory_utilization) - (total - free) - (512 << 20)
            budget -= cfg.state_bytes_per_sequence() * r.Smax
            nb = min(budget // page_bytes, r.MB * r.Smax)
            if nb < r.MB:
                raise RuntimeError(f"KV budget holds {nb} blocks; one sequence of max_model_len needs {r.MB}")
        r.num_blocks = nb
        r.block_bytes = page_bytes
        self.pages: List[Optional[torch.Tensor]] = []
        self.rot: Dict[tuple, torch.Tensor] = {}
        for i, spec in enumerate(cfg.layers):
            c = spec["mixer"]
            row = cfg.latent_row(i)
            if row:
                self.pages.append(torch.zeros(nb, 1, bs, row, dtype=xt, device=dev))
            elif spec["type"] == "latent_attention_2":
                self.pages.append(self.pages[int(c["kv_from"])])
            else:
                self.pages.append(None)
            key = _rot_key(c) if spec["type"] == "latent_attention" else None
            if key is not None and key not in self.rot:
                sc = dict(zip(("factor", "original", "fast", "slow"), key[2])) if key[2] else None
                freqs, mag = stretched_frequencies(key[0], key[1], sc)
                self.rot[key] = rotation_table_scaled(freqs, mag, e.max_model_len, dev)
        # ---- state slots: the stream's last taps-1 rows per layer; the recurrent state of every gla layer ------------
        S = r.Smax
        self.conv_state = torch.zeros(len(cfg.layers), S, max(1, cfg.taps - 1), W, dtype=f32, device=dev)
        self.state: List[Optional[torch.Tensor]] = [
            torch.zeros(S, int(sp["mixer"]["heads"]), int(sp["mixer"]["dim"]), int(sp["mixer"]["vdim"]), dtype=f32, device=dev)
            if sp["type"] == "gla" else None for sp in cfg.layers]
        # scratch of the decode attention's key slices: [tokens, heads, slices, value width + 2] fp32
        self.max_splits = 32
        self.sms = torch.cuda.get_device_properties(dev).multi_processor_count
        h_max = max(int(sp["mixer"]["heads"]) for sp in cfg.layers)
        self.split_ws = torch.zeros(max(2, S * h_max * self.max_splits * (128 + 2)), dtype=f32, device=dev)
        self._opts: List[Optional[_cabi.AttnOpts]] = []
        for spec in cfg.layers:
            c = spec["mixer"]
            if spec["type"] == "gla":
                self._opts.append(None)
                continue
            o = _cabi.AttnOpts()
            o.scale, o.softcap, o.out_scale = float(c["scale"]), 0.0, 1.0
            o.chunk, o.window, o.keep_first, o.sink = 0, int((c.get("mask") or {}).get("size", 0) or 0), 0, 0
            o.weight, o.gate_elem = _cabi.ATTN_SOFTMAX, 0
            o.slopes, o.sinks, o.bias = None, None, None
            self._opts.append(o)

    # ------------------------------------------------------------------------------------------------------------------
    def _attend(self, li: int, q: int, row: int, Dk: int, Vd: int, gate, ldg: int, out: int, ldo: int, T: int, n_dec: int,
                n_pf: int) -> int:
        """Attention of the step's rows over their sequences' latent pages (one key/value head of `row` elements shared by
        all query heads; the key is the row's first Dk elements, the value its first Vd): prompt portions on the tensor
        cores where the element type and the sizes have such a kernel; single decoded tokens (and every row otherwise) on
        the decode form of that kernel or on the kernel that gives a warp to each (row, head). Returns the launch count."""
        import ctypes

        r, lib, ck, dp, dt = self.r, self.r.lib, self.r._ck, self.r._dp, self.dt
        H = int(self.cfg.layers[li]["mixer"]["heads"])
        kc = self.pages[li].data_ptr()
        o = self._opts[li]
        po = ctypes.byref(o)
        fl, st = r.flags, torch.cuda.current_stream().cuda_stream
        tc = n_pf > 0 and lib.atx_attn_window_prefill_supported(Dk, Vd, row, row, dt)
        rows = n_dec if tc else T
        n = 0
        if rows and rows == n_dec and lib.atx_attn_window_decode_supported(H, 1, Dk, Vd, row, row, dt):
            keys = min(o.window if o.window else r.e.max_model_len, r.e.max_model_len)
            splits = max(1, min((keys + 63) // 64, self.max_splits, -(-3 * self.sms // rows)))
            ws = self.split_ws
            ck(lib.atx_attn_paged_decode(q, kc, kc, row, row, dp["seq_bt"], r.MB, dp["tok_seq"], dp["pos"], gate, ldg, out, ldo,
                                         ws.data_ptr(), ws.numel() * 4, splits, rows, H, 1, Dk, Vd, r.bs, po, dt, fl, st))
            n += 2 if splits > 1 else 1
        elif rows:
            ck(lib.atx_attn_paged(q, kc, kc, row, row, dp["seq_bt"], r.MB, dp["tok_seq"], dp["pos"], gate, ldg, out, ldo, rows, H,
                                  1, Dk, Vd, r.bs, po, dt, fl, st))
            n += 1
        if tc:
            # rows of the prompt portions start at row n_dec: q, gate and out are passed whole, rows come from seq_start
            ck(lib.atx_attn_paged_prefill(q, kc, kc, row, row, dp["seq_bt"] + 4 * n_dec * r.MB, r.MB, dp["seq_start"] + 4 * n_dec,
                                          dp["seq_count"] + 4 * n_dec, dp["seq_pos0"] + 4 * n_dec, n_pf, T - n_dec, gate, ldg,
                                          out, ldo, H, 1, Dk, Vd, r.bs, po, dt, fl, st))
            n += 1
        return n

    def forward(self, T: int, n_dec: int, n_pf: int, n_rows: int) -> int:
        """Issue every kernel of one step on the current stream; returns the launch count. The step's first n_dec
        sequences are single decoded tokens (rows 0 .. n_dec-1), the next n_pf are prompt portions."""
        r, cfg, w = self.r, self.cfg, self.w
        lib, ck, dp, fl, dt = r.lib, r._ck, r._dp, r.flags, self.dt
        st = torch.cuda.current_stream().cuda_stream
        W, V, eps, bs, K = cfg.width, cfg.vocab_size, cfg.eps, r.bs, cfg.taps
        n_seqs = n_dec + n_pf
        h, y, xn = self.h.data_ptr(), self.y.data_ptr(), self.xn.data_ptr()
        seqs4 = (dp["seq_start"], dp["seq_count"], dp["seq_pos0"], dp["seq_slot"])
        proj = self.scratch.data_ptr()
        up = proj
        n = 0
        ck(lib.atx_embed_rows(dp["ids"], w.embed.data_ptr(), h, T, W, V, dt, fl, st))
        n += 1
        pending = None     # post-norm weight of the sublayer output waiting in y
        probe = r.layer_probe
        small = T <= 64    # decode-sized: split-K GEMMs accumulate into buffers that the norm kernels hand back cleared
        if small:
            self.y[:T].zero_()

        def resid(out_ptr, w_pre=None, out_scale: float = 1.0, rows=None, rows_n: int = T, zero_ptr=None,
                  zero_bytes: int = 0) -> None:
            """h += rms(y) * pending (if a sublayer output waits); out = h, or rms(h) * w_pre, as the element type."""
            nonlocal n, pending
            have = pending is not None
            if not have and out_ptr is None and not zero_bytes:
                return
            ck(lib.atx_resid_norm_out(h, y if have else None, pending if have else None, None, None, w_pre, out_ptr, 0,
                                      out_scale, rows, rows_n, W, eps, 1 if (have and rows is None and small) else 0,
                                      zero_ptr, zero_bytes, dt, fl, st))
            n += 1
            if rows is None:
                pending = None

        seg, segs = _cabi.HeadSeg, _cabi.head_segs
        ROWS, PAGES = _cabi.HEAD_DST_ROWS, _cabi.HEAD_DST_PAGES
        qb, lat, mix, act = (t.data_ptr() for t in (self.q_flat, self.lat_flat, self.mix_flat, self.act_flat))
        for li, (spec, l, lin) in enumerate(zip(cfg.layers, w.layers, self.lin)):
            c = spec["mixer"]
            H, D, Vd = int(c["heads"]), int(c["dim"]), int(c["vdim"])
            ld = l.w_in.shape[0]
            q2 = proj + 4 * _pad4(T * ld)
            n_q2 = lin["uq"].N if "uq" in lin else 0
            acc = lin["in"].accumulates(T)
            # the stream takes the last sublayer's normed output; what the mixer reads is the stream plus its convolution
            resid(None, zero_ptr=proj if acc else None,
                  zero_bytes=(q2 + 4 * T * n_q2 - proj + 15) // 16 * 16 if acc else 0)
            if K:
                cs = self.conv_state[li].data_ptr()
                ck(lib.atx_conv_residual(h, W, l.canon.data_ptr(), cs, xn, W, dp["tok_seq"], dp["seq_start"], dp["seq_pos0"],
                                         dp["seq_slot"], T, W, K, dt, fl, st))
                ck(lib.atx_conv_state_update(h, W, 0, cs, *seqs4, n_seqs, W, K, fl, st))
                n += 2 if K > 1 else 1
            else:
                resid(xn)
            lin["in"].run(proj, ld, T, fl, st, zeroed=acc)
            n += 1
            K_o = l.w_o.shape[1]
            if l.kind == "gla":
                o_k, o_v, o_g, o_a = H * D, 2 * H * D, 2 * H * D + H * Vd, 2 * H * D + 2 * H * Vd
                rk = int(c["decay_rank"])
                ldec, rec = self.ldec.data_ptr(), self.rec.data_ptr()
                ck(lib.atx_lowrank_logdecay(proj + 4 * o_a, ld, l.a2.data_ptr(), l.a2_b.data_ptr(), ldec, H * D, T, H * D, rk,
                                            float(c["tau"]), dt, fl, st))
                # single decoded tokens (the first n_dec sequences) token by token on the FMA pipe; prompt portions in chunks
                # on the tensor cores when the elements are bf16 and the kernel has the key size, else token by token as well
                chunked = n_pf > 0 and dt == _cabi.DT_BF16 and lib.atx_gated_linear_recurrence_chunked_supported(D)
                n_tok = n_dec if chunked else n_seqs
                rargs = (proj, ld, proj + 4 * o_k, ld, proj + 4 * o_v, ld, ldec, H * D, H, D, Vd, float(D) ** -0.5,
                         self.state[li].data_ptr(), rec, H * Vd)
                if n_tok:
                    ck(lib.atx_gated_linear_recurrence(*rargs, *seqs4, n_tok, fl, st))
                if chunked:
                    ck(lib.atx_gated_linear_recurrence_chunked(*rargs, *(p + 4 * n_dec for p in seqs4), n_pf, fl, st))
                    n += 1 if n_tok else 0
                ck(lib.atx_gated_norm_groups(rec, H * Vd, proj + 4 * o_g, ld, l.mix_norm.data_ptr(), 1, mix, K_o, T, H * Vd, H,
                                             eps, 2, 1.0, dt, fl, st))
                n += 3
            elif l.kind == "latent_attention":
                R, C, Q = int(c["rot_dim"]), int(c["kv_rank"]), int(c["q_rank"])
                key = _rot_key(c)
                table = self.rot[key].data_ptr() if key is not None else None
                rd = key[1] if key is not None else 0
                cq = self.cq_flat.data_ptr()
                # the two bottlenecks: normed query latent -> rows; [normed latent | rotated key part] -> the token's page row
                sg = segs(seg(src_off=0, src_stride=Q, heads=1, width=Q, norm_dims=Q, norm_w=l.dq_norm.data_ptr(),
                              dst_kind=ROWS, dst=cq, dst_ld=Q, dst_off=0, dst_stride=Q),
                          seg(src_off=Q, src_stride=C + R, heads=1, width=C + R, norm_dims=C,
                              norm_w=l.dkv_norm.data_ptr(), rot_off=C, rot_dims=rd, rot=table,
                              dst_kind=PAGES, dst=self.pages[li].data_ptr(), dst_off=0, dst_stride=C + R))
                ck(lib.atx_head_prepare(proj, ld, sg, 2, dp["pos"], dp["slots"], T, bs, eps, dt, fl, st))
                lin["uq"].run(q2, n_q2, T, fl, st, zeroed=acc)
                n += 2
                # queries in the latent's coordinates: [W_uk,h^T q_plain | rotated q part] per head
                if R:
                    sg = segs(seg(src_off=D, src_stride=D + R, heads=H, width=R, rot_off=0, rot_dims=rd, rot=table,
                                  dst_kind=ROWS, dst=qb, dst_ld=H * (C + R), dst_off=C, dst_stride=C + R))
                    ck(lib.atx_head_prepare(q2, n_q2, sg, 1, dp["pos"], dp["slots"], T, bs, eps, dt, fl, st))
                    n += 1
                ck(lib.atx_head_gemm(q2, 1, n_q2, 0, D + R, l.w_ukt.data_ptr(), D, None, 0, qb, H * (C + R), 0, C + R, T, H,
                                     C, D, dt, fl, st))
                n += 1 + self._attend(li, qb, C + R, C + R, C, None, 0, lat, H * C, T, n_dec, n_pf)
                ck(lib.atx_head_gemm(lat, 0, H * C, 0, C, l.w_uv.data_ptr(), C, None, 0, mix, K_o, 0, Vd, T, H, Vd, C, dt, fl,
                                     st))
                n += 1
            else:
                C = int(c["kv_rank"])
                if c.get("kv_from") is None:
                    sg = segs(seg(src_off=H * D + H, src_stride=C, heads=1, width=C, norm_dims=C, norm_w=l.dkv_norm.data_ptr(),
                                  dst_kind=PAGES, dst=self.pages[li].data_ptr(), dst_off=0, dst_stride=C))
                    ck(lib.atx_head_prepare(proj, ld, sg, 1, dp["pos"], dp["slots"], T, bs, eps, dt, fl, st))
                    n += 1
                ck(lib.atx_head_gemm(proj, 1, ld, 0, D, l.w_ukt.data_ptr(), D, None, 0, qb, H * C, 0, C, T, H, C, D, dt, fl, st))
                # the gate of a head is linear in its output, so it is applied to the head's sum over latents
                n += 1 + self._attend(li, qb, C, C, C, proj + 4 * H * D, ld, lat, H * C, T, n_dec, n_pf)
                ck(lib.atx_head_gemm(lat, 0, H * C, 0, C, l.w_uv.data_ptr(), C, None, 0, mix, K_o, 0, Vd, T, H, Vd, C, dt, fl,
                                     st))
                n += 1
            lin["o"].run(y, W, T, fl, st, zeroed=small)
            n += 1
            pending = l.norm1.data_ptr()
            if l.ff == "dense":
                mlp = spec["mlp"]
                F = l.w_down.shape[1]
                if l.gu_interleaved:
                    resid(xn)
                    lin["gu"].run(act, F, T, fl, st, mode=_cabi.GEMM_GLU_CLAMP_BF16)
                    n += 1
                else:
                    acc = lin["gu"].accumulates(T)
                    resid(xn, zero_ptr=up if acc else None, zero_bytes=(T * 2 * F * 4 + 15) // 16 * 16 if acc else 0)
                    lin["gu"].run(up, 2 * F, T, fl, st, zeroed=acc)
                    ck(lib.atx_gated_act_clamped(up, act, T, F, GLU_ALPHA, float(mlp["limit"]), GLU_SHIFT, dt, fl, st))
                    n += 2
                lin["down"].run(y, W, T, fl, st, zeroed=small)
                n += 1
                pending = l.norm2.data_ptr()
            elif l.ff == "moe":
                mlp = spec["mlp"]
                rt = mlp["router"]
                E, top, Fe = int(rt["experts"]), int(rt["top"]), int(mlp["expert"]["ff"])
                shared = "sgu" in lin
                Rn = E + (1 if shared else 0)
                Fs = l.w_sdown.shape[1] if shared else 0
                acc = lin["router"].accumulates(T)
                rl = up + 4 * _pad4(T * (0 if (not shared or l.sgu_interleaved) else 2 * Fs))
                z_hi = rl + 4 * T * Rn
                resid(xn, zero_ptr=up if acc else None, zero_bytes=(z_hi - up + 15) // 16 * 16 if acc else 0)
                lin["router"].run(rl, Rn, T, fl, st, zeroed=acc)
                ck(lib.atx_moe_route_opts(rl, Rn, None, E, top, float(rt.get("scale", 1.0)), 1, self.sel.data_ptr(),
                                          self.wgt.data_ptr(), T, fl, st))
                pairs, so, pm, sl = T * top, self.seg_off.data_ptr(), self.perm.data_ptr(), self.slot_of.data_ptr()
                if "egu" in lin and not small:
                    # prompt-sized: gather every expert's rows, then both products on the tcgen05 GEMM over the plan's tiles
                    big, tb = min(self.max_big_tiles, (pairs + self.big_rows - 1) // self.big_rows + E), self.tiles_big.data_ptr()
                    ck(lib.atx_moe_plan(self.sel.data_ptr(), pairs, E, self.big_rows, so, pm, sl, tb, fl, st))
                    ck(lib.atx_moe_gather_rows(xn, W, pm, top, so, E, self.xperm.data_ptr(), W, pairs, W, dt, fl, st))
                    ck(lib.atx_gemm_run_grouped(lin["egu"]._h, self.eact.data_ptr(), Fe, 2 * Fe, _cabi.GEMM_SWIGLU_BF16, so, tb,
                                                big, fl, st))
                    ck(lib.atx_gemm_run_grouped(lin["edown"]._h, self.ye.data_ptr(), W, W, _cabi.GEMM_STORE_F32, so, tb, big, fl,
                                                st))
                    n += 1
                else:
                    ctas = min(E, pairs) * ((Fe + 63) // 64)
                    tr = 16 if (small and dt == _cabi.DT_BF16 and ctas > 2 * self.sms) else self.tile_rows
                    tiles, tl = min(self.max_tiles, (pairs + tr - 1) // tr + E), self.tiles.data_ptr()
                    ck(lib.atx_moe_plan(self.sel.data_ptr(), pairs, E, tr, so, pm, sl, tl, fl, st))
                    ck(lib.atx_moe_expert_gemm(xn, W, pm, top, 1, l.w_egu.data_ptr(), 2 * Fe * W, W, self.eact.data_ptr(), Fe, Fe,
                                               W, 1, 1 if l.egu_interleaved else 0, tr, so, tl, tiles, dt, fl, st))
                    ck(lib.atx_moe_expert_gemm(self.eact.data_ptr(), Fe, None, top, 0, l.w_edown.data_ptr(), W * Fe, Fe,
                                               self.ye.data_ptr(), W, W, Fe, 0, 0, tr, so, tl, tiles, dt, fl, st))
                n += 5
                if shared:
                    if l.sgu_interleaved:
                        lin["sgu"].run(act, Fs, T, fl, st, mode=_cabi.GEMM_SWIGLU_BF16)
                        n += 1
                    else:
                        lin["sgu"].run(up, 2 * Fs, T, fl, st, zeroed=acc)
                        ck(lib.atx_gated_act(up, act, T, Fs, dt, fl, st))
                        n += 2
                    lin["sdown"].run(y, W, T, fl, st, zeroed=small)
                    n += 1
                ck(lib.atx_moe_combine(y, self.ye.data_ptr(), W, xn, self.sel.data_ptr(), self.wgt.data_ptr(),
                                       self.slot_of.data_ptr(), rl + 4 * E if shared else None, Rn, T, W, top, E, dt, fl, st))
                n += 1
                pending = l.norm2.data_ptr()
            if probe is not None:
                resid(None)
                probe.append(self.h[:T].clone())
        if n_rows:
            resid(self.xl.data_ptr(), w_pre=w.final_norm.data_ptr(), out_scale=cfg.logit_scale, rows=dp["rows"], rows_n=n_rows)
            self.lin_head.run(r.logits.data_ptr(), V, n_rows, fl, st)
            ck(lib.atx_sample(r.logits.data_ptr(), V, dp["temps"], dp["top_p"], dp["seeds"], dp["steps"],
                              r.out_ids.data_ptr(), n_rows, V, fl, st))
            n += 2
        return n
