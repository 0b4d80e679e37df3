"""Zonidra: a decoder-only family whose layers are listed one by one in config.json.

    x_t = embed[token_t] * embedding.scale + bigram[hash(token_(t-1), token_t)]       (optional pair table)
    u   = shift(rms(x) w1)          shift(u)_t = u_t + (u_(t-1) - u_t) * mu, per channel, u_(-1) = 0
    x  <- x + ls1 * rms(mixer(u)) w1b
    x  <- x + ls2 * rms(ffn(rms(x) w2)) w2b                                           (ffn optional)
    logits = head . (rms(x) w_final)

The mixer is attention WITHOUT a softmax: a visible key weighs sigmoid(scale q.k + pb_h) by itself and the weights are
not normalised. A query at p sees key j <= p when p - j < mask.size or j < mask.keep_first. Grouped key/value heads, a
value size of its own, rotation of the first rot.dims elements of q and k in pairs half that range apart with
frequencies rescaled by wavelength (rot.scaling), sigmoid(W_g u) on the concatenated heads before the output
projection. A layer with `kv_from: j` has no key/value projections: it attends over layer j's pages with its own queries.

The feed-forward is dense, W_down poly(W_up u) with poly(z) = a z/rms(z) + b z^2/rms(z^2) + c z^3/rms(z^3) + e, or a
mixture of gated experts: soft-max router, the `top` largest of score + correction chosen, weights = score * scale, the
last `identity` router outputs standing for experts that return their input, plus a shared expert times
sigmoid(W_sg u).

State besides the pages, per live sequence (a state slot): the last token id and, per layer, the last normed row.

fp32 whatever the element type: the residual stream, every norm (the polynomial's included), rotation, scores and
weights of the attention, the token shift and its state, router, expert weights and the weighted sum. Projections run
in the element type (bf16 on the tcgen05 GEMM and the tensor-core expert products, or fp32 on the FMA pipe) with fp32
accumulation.

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
from .common import _Linear, _use_tc, rotation_table_for, wavelength_scaled_frequencies

# ---- configuration --------------------------------------------------------------------------------------------------


def _rot_key(c: dict) -> Optional[tuple]:
    rot = c.get("rot") or {}
    dims = int(rot.get("dims", 0) or 0)
    if not dims:
        return None
    sc = rot.get("scaling") or None
    return (float(rot.get("base", 10000.0)), dims,
            tuple(float(sc[k]) for k in ("factor", "low", "high", "original")) if sc else None)


@dataclass
class Config:
    name: str = "zonidra"
    vocab_size: int = 0
    width: int = 0
    eps: float = 1e-5
    embed_scale: float = 1.0
    bigram: Optional[dict] = None                      # {"buckets", "mul_prev", "mul_cur"}
    layers: List[dict] = field(default_factory=list)   # {"type", "mixer", "mlp"} as in config.json
    eos_token_ids: tuple = ()
    bos_token_id: int = 0
    max_position_embeddings: int = 131072    # the design sets no limit; this bounds the server's default max_model_len
    architecture = "Zonidra"
    recurrent = True      # a state slot per sequence: last token, last normed row of every layer

    @classmethod
    def from_json(cls, d: dict, name: str = "zonidra") -> "Config":
        emb = d.get("embedding") or {}
        bg = emb.get("bigram") or None
        cfg = cls(name=name, vocab_size=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]),
                  embed_scale=float(emb.get("scale", 1.0)), bigram={k: int(v) for k, v in bg.items()} if bg else None,
                  layers=[dict(l) for l in d["layers"]])
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.bigram is not None and self.bigram["buckets"] <= 0:
            raise ValueError("embedding.bigram.buckets must be positive")
        for i, l in enumerate(self.layers):
            if l["type"] != "attention":
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            c = l["mixer"] = dict(l["mixer"])
            c.setdefault("kv_heads", c["heads"])
            c.setdefault("vdim", c["dim"])
            if c["heads"] % c["kv_heads"]:
                raise ValueError(f"layer {i}: {c['heads']} heads over {c['kv_heads']} key/value heads")
            rk = _rot_key(c)
            if rk is not None and (rk[1] % 2 or rk[1] > c["dim"]):
                raise ValueError(f"layer {i}: rot.dims={rk[1]} must be even and at most dim={c['dim']}")
            mask = c.get("mask") or {}
            if int(mask.get("size", 0) or 0) < 0 or int(mask.get("keep_first", 0) or 0) < 0:
                raise ValueError(f"layer {i}: negative mask size")
            src = c.get("kv_from")
            if src is not None:
                src = int(src)
                if not 0 <= src < i or self.layers[src]["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from={src} must name an earlier layer with key/value projections")
                o = self.layers[src]["mixer"]
                if (o["kv_heads"], o["dim"], o["vdim"], _rot_key(o)) != (c["kv_heads"], c["dim"], c["vdim"], rk):
                    raise ValueError(f"layer {i}: shares layer {src}'s keys and values but differs in their shape or rotation")
            mlp = l.get("mlp")
            if mlp is not None:
                kind = mlp.get("kind", "dense")
                if kind == "moe":
                    r = mlp["router"]
                    if not 0 < int(r["top"]) <= int(r["experts"]) + int(r.get("identity", 0)):
                        raise ValueError(f"layer {i}: top={r['top']} of {r['experts']} + {r.get('identity', 0)} experts")
                elif kind != "dense":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")

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
        if self.bigram is not None:
            out["bigram"] = (self.bigram["buckets"] + 1, W)
        for i, l in enumerate(self.layers):
            p, c, m = f"l{i}.", l["mixer"], f"l{i}.mix."
            H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
            for nm in ("norm1", "norm1b", "ls1", "shift"):
                out[p + nm] = (W,)
            out[m + "q"] = (H * D, W)
            if c.get("kv_from") is None:
                out[m + "k"], out[m + "v"] = (G * D, W), (G * V, W)
            out[m + "pb"], out[m + "g"], out[m + "o"] = (H,), (H * V, W), (W, H * V)
            mlp = l.get("mlp")
            if mlp is None:
                continue
            for nm in ("norm2", "norm2b", "ls2"):
                out[p + nm] = (W,)
            f = p + "mlp."
            if mlp.get("kind", "dense") == "dense":
                F = int(mlp["ff"])
                out[f + "up"], out[f + "down"], out[f + "act"] = (F, W), (W, F), (4,)
            else:
                r = mlp["router"]
                E, R, F = int(r["experts"]), int(r["experts"]) + int(r.get("identity", 0)), int(mlp["expert"]["ff"])
                for e in range(E):
                    out[f"{f}e{e}.gate"], out[f"{f}e{e}.up"], out[f"{f}e{e}.down"] = (F, W), (F, W), (W, F)
                out[f + "router"], out[f + "correction"] = (R, W), (R,)
                if mlp.get("shared"):
                    S = int(mlp["shared"]["ff"])
                    out[f + "shared.gate"], out[f + "shared.up"], out[f + "shared.down"] = (S, W), (S, W), (W, S)
                    out[f + "shared.sg"] = (1, W)
        out["final.norm"] = (W,)
        out["head"] = (self.vocab_size, W)
        return out

    # ---- bytes, for the benchmarks' rooflines -------------------------------------------------------------------
    def weight_bytes_per_decode_step(self, elem: int = 2, tokens: int = 1) -> int:
        """Weight bytes a decode step of `tokens` tokens streams: everything but the embedding tables; of the routed
        experts at most tokens * top per layer."""
        n = 0
        for k, v in self.tensor_shapes().items():
            if k in ("embed", "bigram") or ".mlp.e" in k:
                continue
            n += math.prod(v)
        for l in self.layers:
            mlp = l.get("mlp")
            if mlp is not None and mlp.get("kind") == "moe":
                r = mlp["router"]
                n += min(int(r["experts"]), tokens * int(r["top"])) * 3 * int(mlp["expert"]["ff"]) * self.width
        return elem * n

    def kv_bytes_per_token(self, elem: int = 2) -> int:
        return sum(l["mixer"]["kv_heads"] * (l["mixer"]["dim"] + l["mixer"]["vdim"]) * elem for l in self.layers
                   if l["mixer"].get("kv_from") is None)

    def state_bytes_per_sequence(self) -> int:
        return 4 + 4 * self.width * len(self.layers)

    def decode_kv_bytes(self, ctx: int, elem: int = 2) -> int:
        """Page bytes one decoded token at context length ctx reads: every layer its window and the kept first keys."""
        n = 0
        for l in self.layers:
            c = l["mixer"]
            mask = c.get("mask") or {}
            size = int(mask.get("size", 0) or 0)
            keys = min(ctx, size + int(mask.get("keep_first", 0) or 0)) if size else ctx
            n += keys * c["kv_heads"] * (c["dim"] + c["vdim"]) * elem
        return n


def named_shape(name: str) -> Optional[Config]:
    """`random:zonidra-<size>`: shapes whose layers resemble a real model's, for benchmarks (no checkpoint exists).
    `zonidra-8b` / `zonidra-1b` have the width, feed-forward size, vocabulary and depth of the Llama 8B / 1B shapes; layers
    alternate (attention with its own keys and values + dense feed-forward) and (attention over the previous layer's keys
    and values + mixture of 8 experts of a quarter of the feed-forward size, 2 chosen, 2 identity outputs, a shared expert)."""
    key = name.lower()
    shapes = {"zonidra-8b": (4096, 14336, 16, 128256), "zonidra-1b": (2048, 8192, 8, 128256),
              "zonidra-tiny": (256, 512, 1, 1024)}     # width, feed-forward, repeats of the 2-layer pattern, vocabulary
    if key not in shapes:
        return None
    W, F, groups, vocab = shapes[key]
    hd = 128 if W >= 4096 else 64
    heads = W // hd
    mixer = {"dim": hd, "heads": heads, "kv_heads": max(1, heads // 4), "vdim": hd, "scale": hd ** -0.5,
             "mask": {"size": 2048, "keep_first": 64},
             "rot": {"base": 500000.0, "dims": hd // 2,
                     "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    Fe = max(64, F // 4 // 64 * 64)
    layers = []
    for g in range(groups):
        layers.append({"type": "attention", "mixer": dict(mixer), "mlp": {"kind": "dense", "ff": F}})
        layers.append({"type": "attention", "mixer": dict(mixer, kv_from=2 * g),
                       "mlp": {"kind": "moe", "expert": {"ff": Fe}, "shared": {"ff": Fe},
                               "router": {"experts": 8, "identity": 2, "top": 2, "scale": 1.0}}})
    cfg = Config(name=key, vocab_size=vocab, width=W, eps=1e-5, embed_scale=1.0,
                 bigram={"buckets": 65521, "mul_prev": 31, "mul_cur": 17}, layers=json.loads(json.dumps(layers)))
    cfg.validate()
    return cfg


# ---- weights ----------------------------------------------------------------------------------------------------------


class _Layer:
    """Device tensors of one layer in the layout the kernels read (projections that share an input are stacked)."""

    def __init__(self) -> None:
        self.norm1 = self.norm1b = self.ls1 = self.shift = None
        self.norm2 = self.norm2b = self.ls2 = None
        self.w_in = self.w_o = None          # [q | k | v | g] (or [q | g] when keys and values are another layer's)
        self.pb = None                       # fp32 [heads]
        self.ff = ""                         # "", "dense", "moe"
        self.w_up = self.w_down = None       # dense
        self.act = None                      # fp32 [4]
        self.w_router = None                 # [router outputs (+ 1: the shared expert's gate), width]
        self.correction = None               # fp32 [router outputs]
        self.w_egu = self.w_edown = None     # [experts, 2 ff, width] (gate rows, then up rows), [experts, width, ff]
        self.w_sgu = self.w_sdown = None     # shared expert
        self.sgu_interleaved = False
        self.egu_interleaved = False         # gate / up rows of every expert in blocks of 64, as the gated GEMM epilogue reads them


class Weights:
    def __init__(self, cfg: Config, device: torch.device, dtype: torch.dtype):
        self.cfg, self.device, self.dtype = cfg, device, dtype
        self.embed = self.head = self.final_norm = self.bigram = None
        self.layers: List[_Layer] = []
        self.tp_size, self.tp_rank = 1, 0

    def nbytes(self) -> int:
        ts = [self.embed, self.head, self.final_norm, self.bigram]
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
        g = torch.Generator(device=device).manual_seed(1000 * seed + 13)
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
                if leaf == "act":
                    return torch.tensor([0.6, 0.3, 0.2, 0.05], device=device)
                if leaf == "pb":
                    return -3.0 + 0.5 * torch.randn(sh, generator=g, device=device)
                if leaf == "correction":
                    return 0.02 * torch.randn(sh, generator=g, device=device)
                if leaf == "shift":
                    return torch.rand(sh, generator=g, device=device)
                if leaf in ("ls1", "ls2"):
                    return 0.5 + 0.1 * torch.randn(sh, generator=g, device=device)
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
            return torch.as_tensor(t).to(device=device, dtype=torch.float32).contiguous()

        W = cfg.width
        w.embed, w.head, w.final_norm = dev(get("embed")), dev(get("head")), dev(get("final.norm"))
        if cfg.bigram is not None:
            w.bigram = dev(get("bigram"))
        for i, spec in enumerate(cfg.layers):
            p, c, l = f"l{i}.", spec["mixer"], _Layer()
            m = p + "mix."
            l.norm1, l.norm1b, l.ls1, l.shift = (dev(get(p + nm)) for nm in ("norm1", "norm1b", "ls1", "shift"))
            parts = [get(m + "q")] + ([get(m + "k"), get(m + "v")] if c.get("kv_from") is None else []) + [get(m + "g")]
            l.w_in, l.w_o, l.pb = dev(torch.cat(parts, 0)), dev(get(m + "o")), f32(get(m + "pb"))
            mlp = spec.get("mlp")
            if mlp is not None:
                l.norm2, l.norm2b, l.ls2 = (dev(get(p + nm)) for nm in ("norm2", "norm2b", "ls2"))
                f = p + "mlp."
                if mlp.get("kind", "dense") == "dense":
                    l.ff = "dense"
                    l.w_up, l.w_down, l.act = dev(get(f + "up")), dev(get(f + "down")), f32(get(f + "act"))
                else:
                    l.ff = "moe"
                    E = int(mlp["router"]["experts"])
                    rows = [get(f + "router")] + ([get(f + "shared.sg")] if mlp.get("shared") else [])
                    l.w_router, l.correction = dev(torch.cat(rows, 0)), f32(get(f + "correction"))
                    Fe = int(mlp["expert"]["ff"])
                    if _use_tc(dtype, W) and Fe % 64 == 0:
                        from ..weights import interleave_gate_up

                        l.egu_interleaved = True
                        l.w_egu = torch.stack([dev(interleave_gate_up(get(f"{f}e{e}.gate"), get(f"{f}e{e}.up")))
                                               for e in range(E)], 0).contiguous()
                    else:
                        l.w_egu = torch.stack([dev(torch.cat([get(f"{f}e{e}.gate"), get(f"{f}e{e}.up")], 0))
                                               for e in range(E)], 0).contiguous()
                    l.w_edown = torch.stack([dev(get(f"{f}e{e}.down")) for e in range(E)], 0).contiguous()
                    if mlp.get("shared"):
                        gate, up = get(f + "shared.gate"), get(f + "shared.up")
                        if _use_tc(dtype, W) and gate.shape[0] % 64 == 0:
                            from ..weights import interleave_gate_up

                            l.w_sgu, l.sgu_interleaved = dev(interleave_gate_up(gate, up)), True
                        else:
                            l.w_sgu = dev(torch.cat([gate, up], 0))
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
            raise ValueError("Zonidra runs on one GPU per replica")
        xt = w.dtype
        self.dt = _cabi.DT_F32 if xt == torch.float32 else _cabi.DT_BF16
        self.xt, self.esz = xt, (4 if xt == torch.float32 else 2)
        dev, T, lib = r.dev, r.Tmax, r.lib
        W = cfg.width
        f32, i32 = torch.float32, torch.int32
        n_in = n_q = n_mix = n_up = n_act = n_rl = n_pairs = n_ef = n_exp = 1
        for spec in cfg.layers:
            c = spec["mixer"]
            H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
            own = c.get("kv_from") is None
            n_in = max(n_in, H * D + (G * (D + V) if own else 0) + H * V)
            n_q, n_mix = max(n_q, H * D), max(n_mix, H * V)
            mlp = spec.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind", "dense") == "dense":
                n_up, n_act = max(n_up, int(mlp["ff"])), max(n_act, int(mlp["ff"]))
            else:
                rt = mlp["router"]
                n_rl = max(n_rl, int(rt["experts"]) + int(rt.get("identity", 0)) + 1)
                n_pairs, n_ef, n_exp = max(n_pairs, int(rt["top"])), max(n_ef, int(mlp["expert"]["ff"])), max(n_exp, int(rt["experts"]))
                if mlp.get("shared"):
                    n_act = max(n_act, int(mlp["shared"]["ff"]))
                    n_up = max(n_up, 2 * int(mlp["shared"]["ff"]))     # gate | up when the epilogue cannot fuse them
        self.h = torch.zeros(T, W, dtype=f32, device=dev)          # residual stream
        self.y = torch.zeros(T, W, dtype=f32, device=dev)          # a sublayer's output before its post-norm
        self.nf = torch.zeros(T, W, dtype=f32, device=dev)         # normed rows before the token shift
        # fp32 GEMM outputs of a sublayer, back to back so that one pass clears what split-K accumulates into: the mixer's
        # input projections; then, in the same space, [feed-forward up projection | router outputs]
        self.scratch = torch.zeros(T * max(_pad4(n_in), _pad4(n_up) + _pad4(n_rl)) + 32, dtype=f32, device=dev)
        self.xn = torch.zeros(T, W, dtype=xt, device=dev)
        self.q_flat = torch.zeros(T * n_q, dtype=xt, device=dev)
        self.mix_flat = torch.zeros(T * n_mix, dtype=xt, device=dev)
        self.act_flat = torch.zeros(T * n_act, dtype=xt, device=dev)
        self.xl = torch.zeros(r.Rmax, W, dtype=xt, device=dev)
        # mixture of experts: choices, weights, the plan, the experts' hidden rows and outputs per (token, choice) slot
        self.tile_rows = int(lib.atx_moe_tile_rows())
        P = T * n_pairs
        # tiles of 64 slots, or of 16 for decode-sized steps (at most 64 tokens): whichever list is longer
        self.max_tiles = max((P + self.tile_rows - 1) // self.tile_rows, (min(P, 64 * n_pairs) + 15) // 16) + n_exp
        self.sel = torch.zeros(P, dtype=i32, device=dev)
        self.wgt = torch.zeros(P, dtype=f32, device=dev)
        self.seg_off = torch.zeros(n_exp + 1, dtype=i32, device=dev)
        self.perm = torch.zeros(P, dtype=i32, device=dev)
        self.slot_of = torch.zeros(P, dtype=i32, device=dev)
        self.tiles = torch.zeros(2 + 2 * self.max_tiles, dtype=i32, device=dev)
        self.eact = torch.zeros(P * n_ef if n_exp > 1 or n_ef > 1 else 1, dtype=xt, device=dev)
        # prompt-sized steps on the tcgen05 GEMM: every expert's input rows back to back, tiles of its own row count
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
            if l.ff == "dense":
                d["up"] = _Linear(lib, l.w_up, self.xn, self.dt)
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
        self.lin_head = _Linear(lib, w.head, self.xl, self.dt)

        # ---- pages: one set per layer that projects keys and values; a sharing layer reads its source's --------------
        bs = r.bs
        page_bytes = cfg.kv_bytes_per_token(self.esz) * bs
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
        self.kv: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self.rot: Dict[tuple, torch.Tensor] = {}
        for spec in cfg.layers:
            c = spec["mixer"]
            src = c.get("kv_from")
            if src is None:
                self.kv.append((torch.zeros(nb, c["kv_heads"], bs, c["dim"], dtype=xt, device=dev),
                                torch.zeros(nb, c["kv_heads"], bs, c["vdim"], dtype=xt, device=dev)))
            else:
                self.kv.append(self.kv[int(src)])
            key = _rot_key(c)
            if key is not None and key not in self.rot:
                sc = dict(zip(("factor", "low", "high", "original"), key[2])) if key[2] else None
                self.rot[key] = rotation_table_for(wavelength_scaled_frequencies(key[0], key[1], sc), e.max_model_len, dev)
        # ---- state slots: the last token and, per layer, the last normed row of every live sequence -----------------
        S = r.Smax
        self.prev_tok = torch.zeros(S, dtype=i32, device=dev)
        self.shift_state = torch.zeros(len(cfg.layers), S, W, dtype=f32, device=dev)
        # scratch of the decode attention's key slices: [tokens, heads, slices, value width + 2] fp32
        self.max_splits = 32
        self.sms = torch.cuda.get_device_properties(dev).multi_processor_count
        h_max = max(spec["mixer"]["heads"] for spec in cfg.layers)
        self.split_ws = torch.zeros(max(2, S * h_max * self.max_splits * (128 + 2)), dtype=f32, device=dev)
        self._opts: List[_cabi.AttnOpts] = []
        for spec, l in zip(cfg.layers, w.layers):
            c = spec["mixer"]
            mask = c.get("mask") or {}
            o = _cabi.AttnOpts()
            o.scale, o.softcap, o.out_scale = float(c["scale"]), 0.0, 1.0
            o.chunk, o.window, o.keep_first, o.sink = 0, int(mask.get("size", 0) or 0), int(mask.get("keep_first", 0) or 0), 0
            if o.window == 0:
                o.keep_first = 0     # no window: every earlier key is visible anyway
            o.weight, o.gate_elem = _cabi.ATTN_SIGMOID, 1
            o.slopes, o.sinks, o.bias = None, None, l.pb.data_ptr()
            self._opts.append(o)

    # ------------------------------------------------------------------------------------------------------------------
    def _attend(self, li: int, q: int, gate: int, ldg: int, out: int, ldo: int, T: int, n_dec: int, n_pf: int) -> int:
        """Attention of the step's rows over their sequences' pages: prompt portions on the tensor cores where the
        element type and the sizes have such a kernel; single decoded tokens (and every row otherwise) on the decode
        form of that kernel or on the kernel that gives a warp to each (row, head). Returns the launch count."""
        import ctypes

        r, lib, ck, dp, dt = self.r, self.r.lib, self.r._ck, self.r._dp, self.dt
        c = self.cfg.layers[li]["mixer"]
        H, G, D, Vd = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
        kc, vc = (t.data_ptr() for t in self.kv[li])
        o = self._opts[li]
        po = ctypes.byref(o)
        fl, st = r.flags, torch.cuda.current_stream().cuda_stream
        tc = n_pf > 0 and lib.atx_attn_window_prefill_supported(D, Vd, D, Vd, dt)
        rows = n_dec if tc else T
        n = 0
        if rows and rows == n_dec and lib.atx_attn_window_decode_supported(H, G, D, Vd, D, Vd, dt):
            keys = min((o.window + o.keep_first) if o.window else r.e.max_model_len, r.e.max_model_len)
            splits = max(1, min((keys + 63) // 64, self.max_splits, -(-3 * self.sms // (rows * G))))
            ws = self.split_ws
            ck(lib.atx_attn_paged_decode(q, kc, vc, D, Vd, dp["seq_bt"], r.MB, dp["tok_seq"], dp["pos"], gate, ldg, out, ldo,
                                         ws.data_ptr(), ws.numel() * 4, splits, rows, H, G, D, Vd, r.bs, po, dt, fl, st))
            n += 2 if splits > 1 else 1
        elif rows:
            ck(lib.atx_attn_paged(q, kc, vc, D, Vd, dp["seq_bt"], r.MB, dp["tok_seq"], dp["pos"], gate, ldg, out, ldo, rows, H,
                                  G, D, Vd, r.bs, po, dt, fl, st))
            n += 1
        if tc:
            # rows of the prompt portions start at row n_dec: q, gate and out are passed whole, rows come from seq_start
            ck(lib.atx_attn_paged_prefill(q, kc, vc, D, Vd, dp["seq_bt"] + 4 * n_dec * r.MB, r.MB, dp["seq_start"] + 4 * n_dec,
                                          dp["seq_count"] + 4 * n_dec, dp["seq_pos0"] + 4 * n_dec, n_pf, T - n_dec, gate, ldg,
                                          out, ldo, H, G, D, Vd, r.bs, po, dt, fl, st))
            n += 1
        return n

    def forward(self, T: int, n_dec: int, n_pf: int, n_rows: int) -> int:
        """Issue every kernel of one step on the current stream; returns the launch count. The step's first n_dec
        sequences are single decoded tokens (rows 0 .. n_dec-1), the next n_pf are prompt portions."""
        r, cfg, w = self.r, self.cfg, self.w
        lib, ck, dp, fl, dt = r.lib, r._ck, r._dp, r.flags, self.dt
        st = torch.cuda.current_stream().cuda_stream
        W, V, eps, bs = cfg.width, cfg.vocab_size, cfg.eps, r.bs
        h, y, nf, xn = self.h.data_ptr(), self.y.data_ptr(), self.nf.data_ptr(), self.xn.data_ptr()
        seqs = (dp["tok_seq"], dp["seq_start"], dp["seq_count"], dp["seq_pos0"], dp["seq_slot"])
        proj = self.scratch.data_ptr()
        up = proj
        n = 0
        if cfg.bigram is not None:
            b = cfg.bigram
            ck(lib.atx_embed_rows_pair(dp["ids"], w.embed.data_ptr(), cfg.embed_scale, w.bigram.data_ptr(), b["buckets"],
                                       b["mul_prev"], b["mul_cur"], self.prev_tok.data_ptr(), *seqs, h, T, W, V, dt, fl, st))
        else:
            ck(lib.atx_embed_rows_scaled(dp["ids"], w.embed.data_ptr(), h, T, W, V, cfg.embed_scale, dt, fl, st))
        n += 1
        pending = None     # (post-norm weight, branch scale) of the sublayer output waiting in y
        probe = r.layer_probe
        small = T <= 64    # decode-sized: split-K GEMMs accumulate into buffers that the norm kernels hand back cleared
        if small:
            self.y[:T].zero_()

        def resid(w_pre, out_ptr, out_f32: int = 0, rows=None, rows_n: int = T, zero_ptr=None, zero_bytes: int = 0) -> None:
            nonlocal n, pending
            have = pending is not None
            ck(lib.atx_resid_norm_scaled(h, y if have else None, pending[0] if have else None,
                                         pending[1] if have else None, None, w_pre, out_ptr, out_f32, rows, rows_n, W, eps,
                                         1 if (have and rows is None and small) else 0, zero_ptr, zero_bytes, dt, fl, st))
            n += 1
            if rows is None:
                pending = None

        seg, segs = _cabi.HeadSeg, _cabi.head_segs
        ROWS, PAGES = _cabi.HEAD_DST_ROWS, _cabi.HEAD_DST_PAGES
        qb, mix, act = self.q_flat.data_ptr(), self.mix_flat.data_ptr(), self.act_flat.data_ptr()
        for li, (spec, l, lin) in enumerate(zip(cfg.layers, w.layers, self.lin)):
            c = spec["mixer"]
            H, G, D, Vd = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
            own = c.get("kv_from") is None
            ld = l.w_in.shape[0]
            acc = lin["in"].accumulates(T)
            resid(l.norm1.data_ptr(), nf, out_f32=1, zero_ptr=proj if acc else None,
                  zero_bytes=(T * ld * 4 + 15) // 16 * 16 if acc else 0)
            ck(lib.atx_token_shift(nf, l.shift.data_ptr(), self.shift_state[li].data_ptr(), *seqs, xn, T, W, dt, fl, st))
            lin["in"].run(proj, ld, T, fl, st, zeroed=acc)
            n += 2
            key = _rot_key(c)
            table = self.rot[key].data_ptr() if key is not None else None
            rd = key[1] if key is not None else 0
            sg = [seg(src_off=0, src_stride=D, heads=H, width=D, rot_off=0, rot_dims=rd, rot=table, rot_half=1,
                      dst_kind=ROWS, dst=qb, dst_ld=H * D, dst_off=0, dst_stride=D)]
            o_g = H * D
            if own:
                kc, vc = self.kv[li]
                sg.append(seg(src_off=H * D, src_stride=D, heads=G, width=D, rot_off=0, rot_dims=rd, rot=table, rot_half=1,
                              dst_kind=PAGES, dst=kc.data_ptr(), dst_off=0, dst_stride=D))
                sg.append(seg(src_off=H * D + G * D, src_stride=Vd, heads=G, width=Vd,
                              dst_kind=PAGES, dst=vc.data_ptr(), dst_off=0, dst_stride=Vd))
                o_g += G * (D + Vd)
            ck(lib.atx_head_prepare(proj, ld, segs(*sg), len(sg), dp["pos"], dp["slots"], T, bs, eps, dt, fl, st))
            K_o = l.w_o.shape[1]
            n += 1 + self._attend(li, qb, proj + 4 * o_g, ld, mix, K_o, T, n_dec, n_pf)
            lin["o"].run(y, W, T, fl, st, zeroed=small)
            n += 1
            pending = (l.norm1b.data_ptr(), l.ls1.data_ptr())
            if l.ff == "dense":
                F = l.w_up.shape[0]
                acc = lin["up"].accumulates(T)
                resid(l.norm2.data_ptr(), xn, zero_ptr=up if acc else None, zero_bytes=(T * F * 4 + 15) // 16 * 16 if acc else 0)
                lin["up"].run(up, F, T, fl, st, zeroed=acc)
                ck(lib.atx_poly_norm_act(up, F, l.act.data_ptr(), act, F, T, F, eps, dt, fl, st))
                lin["down"].run(y, W, T, fl, st, zeroed=small)
                n += 3
                pending = (l.norm2b.data_ptr(), l.ls2.data_ptr())
            elif l.ff == "moe":
                mlp = spec["mlp"]
                rt = mlp["router"]
                E, R, top, Fe = int(rt["experts"]), int(rt["experts"]) + int(rt.get("identity", 0)), int(rt["top"]), int(mlp["expert"]["ff"])
                shared = "sgu" in lin
                Rn = R + (1 if shared else 0)
                Fs = l.w_sdown.shape[1] if shared else 0
                acc = lin["router"].accumulates(T)
                rl = up + 4 * _pad4(T * (0 if (not shared or l.sgu_interleaved) else 2 * Fs))
                z_hi = rl + 4 * T * Rn
                resid(l.norm2.data_ptr(), xn, zero_ptr=up if acc else None, zero_bytes=(z_hi - up + 15) // 16 * 16 if acc else 0)
                lin["router"].run(rl, Rn, T, fl, st, zeroed=acc)
                ck(lib.atx_moe_route(rl, Rn, l.correction.data_ptr(), R, top, float(rt.get("scale", 1.0)), self.sel.data_ptr(),
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
                    # decode-sized bf16 steps (one or two rows per expert): tiles of 16 slots put three CTAs on an SM instead
                    # of two. That pays when two per SM would need a second wave, and costs a little when one wave suffices.
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
                                       self.slot_of.data_ptr(), rl + 4 * R if shared else None, Rn, T, W, top, E, dt, fl, st))
                n += 1
                pending = (l.norm2b.data_ptr(), l.ls2.data_ptr())
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
