"""Slow reference of the Zonidra family in float64 on the CPU, one function per mechanism.

Test infrastructure only: nothing under agentic-traffic-testing_b200/ imports it, and it imports nothing from there.
Every function works on a whole sequence at once ([n, ...] tensors, position = row index) and is written as the
defining sums over all pairs of positions (no pages, no carried state, no tiling, no sorting of tokens by expert).

Notation: n tokens, model width W; `lin(u, M)` = u M^T for a matrix M [out, in]. `cfg` is the parsed config.json of a
model, `wt` maps tensor names to float64 tensors.

The family: x_t = s_emb E[token_t] + B[hash(token_(t-1), token_t)]; every layer is
    u = shift(rms(x) w1);  x <- x + ls1 * (rms(mixer(u)) w1b);   x <- x + ls2 * (rms(ffn(rms(x) w2)) w2b)
with shift(u)_t = u_t + (u_(t-1) - u_t) * mu (u_(-1) = 0). The mixer is attention without a softmax: every visible key
weighs sigmoid(score + bias_h), visible = causal and (inside a sliding window or among the first few positions);
grouped key/value heads, rotation of half-split pairs with rescaled frequencies, a sigmoid gate on the concatenated
heads, and layers that read another layer's keys and values. The feed-forward is dense with a polynomial activation of
unit-rms powers, or a mixture of gated experts (soft-max router, selection with an additive correction, identity
experts, a gated shared expert). logits = head . (rms(x) w_final).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def lin(u: torch.Tensor, m: torch.Tensor) -> torch.Tensor:
    return u @ m.T


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x scaled to unit root-mean-square over the last axis (eps under the root)."""
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def bigram_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """Row of the pair table for every position: a hash of (previous token, token); the first position has no
    predecessor and takes the extra last row."""
    return [buckets if t == 0 else (tokens[t - 1] * mul_prev + tokens[t] * mul_cur) % buckets for t in range(len(tokens))]


def embed(cfg: dict, wt: Dict[str, torch.Tensor], tokens: List[int]) -> torch.Tensor:
    e = cfg.get("embedding") or {}
    x = wt["embed"][tokens] * float(e.get("scale", 1.0))
    bg = e.get("bigram")
    if bg:
        x = x + wt["bigram"][bigram_rows(tokens, int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]))]
    return x


def token_shift(u: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    """u_t + (u_(t-1) - u_t) mu, element by element; the predecessor of position 0 is zero."""
    prev = torch.cat([torch.zeros_like(u[:1]), u[:-1]], 0)
    return u + (prev - u) * mu


def rescaled_frequencies(dims: int, base: float, scaling: Optional[dict]) -> torch.Tensor:
    """f_i = base^(-2i/dims), i < dims/2; with `scaling`, long wavelengths are stretched by `factor`, short ones kept,
    and the band between is interpolated linearly in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wl = 2.0 * math.pi / f
            if wl < orig / high:
                pass
            elif wl > orig / low:
                f = f / factor
            else:
                s = (orig / wl - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_halves(x: torch.Tensor, dims: int, freqs: torch.Tensor) -> torch.Tensor:
    """x [n, heads, d]: element i < dims/2 is paired with element i + dims/2; the pair at position p turns by p f_i.
    Elements from `dims` on pass through."""
    if dims == 0:
        return x
    n, half = x.shape[0], dims // 2
    ang = torch.arange(n, dtype=F64)[:, None] * freqs[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


def visible(n: int, size: int, keep_first: int) -> torch.Tensor:
    """[n, n] bool: query i sees key j when j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def sigmoid_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, bias: torch.Tensor,
                      vis: torch.Tensor) -> torch.Tensor:
    """q [n, H, d], k [n, G, d], v [n, G, e] -> [n, H, e]: out_i = sum_j sigmoid(scale q_i.k_j + bias_h) v_j over the
    visible j. The weights are not normalised."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        w = torch.sigmoid(q[:, h] @ k[:, g].T * scale + bias[h]) * vis
        out[:, h] = w @ v[:, g]
    return out


def attention_keys_values(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], m: str) -> Tuple[torch.Tensor, torch.Tensor]:
    n = u.shape[0]
    G, D, V = int(c["kv_heads"]), int(c["dim"]), int(c["vdim"])
    rot = c.get("rot") or {}
    dims = int(rot.get("dims", 0))
    fr = rescaled_frequencies(dims, float(rot.get("base", 10000.0)), rot.get("scaling")) if dims else None
    k = rotate_halves(lin(u, wt[m + "k"]).view(n, G, D), dims, fr)
    return k, lin(u, wt[m + "v"]).view(n, G, V)


def attention_mixer(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], m: str,
                    kv: Tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    n = u.shape[0]
    H, D = int(c["heads"]), int(c["dim"])
    rot = c.get("rot") or {}
    dims = int(rot.get("dims", 0))
    fr = rescaled_frequencies(dims, float(rot.get("base", 10000.0)), rot.get("scaling")) if dims else None
    q = rotate_halves(lin(u, wt[m + "q"]).view(n, H, D), dims, fr)
    mask = c.get("mask") or {}
    vis = visible(n, int(mask.get("size", 0)) or n, int(mask.get("keep_first", 0)))
    o = sigmoid_attention(q, kv[0], kv[1], float(c["scale"]), wt[m + "pb"], vis).reshape(n, -1)
    return lin(o * torch.sigmoid(lin(u, wt[m + "g"])), wt[m + "o"])


def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """a N(z) + b N(z^2) + c N(z^3) + e with N = unit rms over the row."""
    return coef[0] * unit_rms(z, eps) + coef[1] * unit_rms(z * z, eps) + coef[2] * unit_rms(z * z * z, eps) + coef[3]


def gated_expert(u: torch.Tensor, wt: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    g = lin(u, wt[p + "gate"])
    return lin(g * torch.sigmoid(g) * lin(u, wt[p + "up"]), wt[p + "down"])


def route(u: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int, scale: float
          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chosen experts [n, top] and their weights: soft-max over every router output; the choice ranks score +
    correction, the weight is the plain score times `scale`."""
    s = torch.softmax(lin(u, router), -1)
    idx = torch.topk(s + correction, top, dim=-1).indices
    return idx, torch.gather(s, 1, idx) * scale


def expert_mixture(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    r = c["router"]
    E, ident = int(r["experts"]), int(r.get("identity", 0))
    idx, wgt = route(u, wt[p + "router"], wt[p + "correction"], int(r["top"]), float(r.get("scale", 1.0)))
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for e, a in zip(idx[t].tolist(), wgt[t]):
            # the last `ident` router outputs stand for experts that return their input
            out[t] += a * (u[t] if e >= E else gated_expert(u[t:t + 1], wt, f"{p}e{e}.")[0])
    if c.get("shared"):
        out = out + torch.sigmoid(lin(u, wt[p + "shared.sg"])) * gated_expert(u, wt, p + "shared.")
    return out


def dense_ffn(u: torch.Tensor, wt: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    return lin(poly_norm(lin(u, wt[p + "up"]), wt[p + "act"], eps), wt[p + "down"])


def forward(cfg: dict, wt: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of a whole sequence; `residuals` receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = embed(cfg, wt, tokens)
    kvs: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    for i, l in enumerate(cfg["layers"]):
        p, c = f"l{i}.", l["mixer"]
        if l["type"] != "attention":
            raise ValueError(f"layer {i}: unknown mixer {l['type']!r}")
        u = token_shift(unit_rms(x, eps) * wt[p + "norm1"], wt[p + "shift"])
        src = c.get("kv_from")
        if src is None:
            kvs[i] = attention_keys_values(u, c, wt, p + "mix.")
        y = attention_mixer(u, c, wt, p + "mix.", kvs[i if src is None else int(src)])
        x = x + unit_rms(y, eps) * wt[p + "norm1b"] * wt[p + "ls1"]
        mlp = l.get("mlp")
        if mlp is not None:
            u = unit_rms(x, eps) * wt[p + "norm2"]
            y = dense_ffn(u, wt, p + "mlp.", eps) if mlp.get("kind", "dense") == "dense" else \
                expert_mixture(u, mlp, wt, p + "mlp.")
            x = x + unit_rms(y, eps) * wt[p + "norm2b"] * wt[p + "ls2"]
        if residuals is not None:
            residuals.append(x.clone())
    return lin(unit_rms(x, eps) * wt["final.norm"], wt["head"])


def checkpoint_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
    W, out = int(cfg["width"]), {}
    out["embed"] = (int(cfg["vocab"]), W)
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        out["bigram"] = (int(bg["buckets"]) + 1, W)
    for i, l in enumerate(cfg["layers"]):
        p, c, m = f"l{i}.", l["mixer"], f"l{i}.mix."
        H, G, D, V = int(c["heads"]), int(c["kv_heads"]), int(c["dim"]), int(c["vdim"])
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
            out[f + "up"], out[f + "down"], out[f + "act"] = (int(mlp["ff"]), W), (W, int(mlp["ff"])), (4,)
        else:
            r = mlp["router"]
            E, ident, F = int(r["experts"]), int(r.get("identity", 0)), int(mlp["expert"]["ff"])
            for e in range(E):
                out[f"{f}e{e}.gate"], out[f"{f}e{e}.up"], out[f"{f}e{e}.down"] = (F, W), (F, W), (W, F)
            out[f + "router"], out[f + "correction"] = (E + ident, W), (E + ident,)
            if mlp.get("shared"):
                S = int(mlp["shared"]["ff"])
                out[f + "shared.gate"], out[f + "shared.up"], out[f + "shared.down"] = (S, W), (S, W), (W, S)
                out[f + "shared.sg"] = (1, W)
    out["final.norm"] = (W,)
    out["head"] = (int(cfg["vocab"]), W)
    return out


def random_checkpoint(cfg: dict, seed: int, round_bf16: bool = True) -> Dict[str, torch.Tensor]:
    """Seeded float64 tensors (values representable in bf16 when round_bf16, so that a bf16 engine loads them exactly)."""
    g = torch.Generator().manual_seed(seed)
    wt = {}
    for name, sh in checkpoint_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if len(sh) == 2:
            t = torch.randn(sh, generator=g, dtype=F64) * (sh[1] ** -0.5)
            if name == "embed":
                t = t * 0.3
            elif leaf == "router":
                t = t * 3.0
        elif leaf == "act":
            t = torch.tensor([0.6, 0.3, 0.2, 0.05], dtype=F64) + 0.1 * torch.randn(4, generator=g, dtype=F64)
        elif leaf == "pb":
            t = -2.0 + 0.5 * torch.randn(sh, generator=g, dtype=F64)
        elif leaf == "correction":
            t = 0.05 * torch.randn(sh, generator=g, dtype=F64)
        elif leaf == "shift":
            t = torch.rand(sh, generator=g, dtype=F64)
        elif leaf in ("ls1", "ls2"):
            t = 0.5 + 0.2 * torch.randn(sh, generator=g, dtype=F64)
        else:   # norm weights
            t = 1.0 + 0.1 * torch.randn(sh, generator=g, dtype=F64)
        wt[name] = t.to(torch.bfloat16).to(F64) if round_bf16 else t
    return wt
