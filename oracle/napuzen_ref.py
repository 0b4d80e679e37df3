"""Slow reference of the Napuzen family in float64 on the CPU, one function per mechanism.

Test infrastructure only: nothing under agentic-traffic-testing_b200/ imports it, and it imports nothing from there.
Every function works on a whole sequence at once ([n, ...] tensors, position = row index) and is written as the
defining sums (loops over positions for the recurrence, sums over all pairs of positions for attention; no pages, no
carried state, no chunks, no sorting of tokens by expert).

Notation: n tokens, model width W; `lin(u, M)` = u M^T for a matrix M [out, in]. `cfg` is the parsed config.json of a
model, `wt` maps tensor names to float64 tensors.

The family: x_t = E[token_t]; every layer is
    x <- x + rms(mixer(x + taps(x))) w1;      x <- x + rms(ffn(x)) w2        (ffn optional)
so a norm stands only behind each sublayer and the sublayers read the stream itself; taps() is a short causal
convolution per channel in front of the mixer. Three mixers: a linear-attention recurrence whose state decays per key
channel by a data-dependent factor (`gla`), soft-max attention whose keys and values are expanded from a cached latent,
with a rotated part shared by all heads and stretched rotation frequencies (`latent_attention`), and a second form of it
without positions, under a sliding window, with a sigmoid gate per head and optionally reading another layer's latent
(`latent_attention_2`). The feed-forward is dense with clamped gate and up projections, or a mixture of gated experts
(soft-max router, the chosen scores renormalised, a gated shared expert). logits = logit_scale * E (rms(x) w_final).
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


def causal_taps(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y_t[c] = sum_j w[c, j] u_(t - K + 1 + j)[c] with K = w.shape[1] taps; rows before the sequence are zero."""
    n, K = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(n):
        for j in range(K):
            s = t - K + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def channel_decay(u: torch.Tensor, a1: torch.Tensor, a2: torch.Tensor, b: torch.Tensor, tau: float) -> torch.Tensor:
    """Decay factors in (0, 1), one per key channel and token: sigmoid(A2 (A1 u) + b)^(1/tau)."""
    return torch.sigmoid(lin(lin(u, a1), a2) + b).pow(1.0 / tau)


def decayed_outer_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    """One head. q, k, a: [n, D]; v: [n, V]. S_t = diag(a_t) S_(t-1) + k_t v_t^T (S_(-1) = 0), o_t = S_t^T q_t."""
    n, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(n):
        S = a[t][:, None] * S + k[t][:, None] * v[t][None, :]
        out.append(S.T @ q[t])
    return torch.stack(out, 0)


def decayed_outer_closed_form(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    """The same as a sum over pairs: o_t = sum_(s <= t) (sum_d q_t[d] k_s[d] prod_(s < r <= t) a_r[d]) v_s."""
    n = q.shape[0]
    la = torch.cumsum(torch.log(a), 0)
    out = torch.zeros(n, v.shape[1], dtype=q.dtype)
    for t in range(n):
        for s in range(t + 1):
            out[t] += (q[t] * k[s] * torch.exp(la[t] - la[s])).sum() * v[s]
    return out


def gla_mixer(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], m: str, eps: float) -> torch.Tensor:
    H, D, V = int(c["heads"]), int(c["dim"]), int(c["vdim"])
    n = u.shape[0]
    q = (lin(u, wt[m + "q"]) * D ** -0.5).view(n, H, D)
    k = lin(u, wt[m + "k"]).view(n, H, D)
    v = lin(u, wt[m + "v"]).view(n, H, V)
    a = channel_decay(u, wt[m + "a1"], wt[m + "a2"], wt[m + "a2.b"], float(c["tau"])).view(n, H, D)
    o = torch.stack([decayed_outer_recurrence(q[:, h], k[:, h], v[:, h], a[:, h]) for h in range(H)], 1)
    o = unit_rms(o, eps) * wt[m + "norm"]
    g = lin(u, wt[m + "g"])
    return lin(o.reshape(n, H * V) * (g * torch.sigmoid(g)), wt[m + "o"])


def stretched_frequencies(dims: int, base: float, scaling: Optional[dict]) -> Tuple[torch.Tensor, float]:
    """f_i = base^(-2i/dims), i < dims/2, and the factor on cos and sin. With `scaling` (factor, original, fast, slow):
    the index at which a pair makes t turns over `original` positions is d(t) = dims ln(original / (2 pi t)) / (2 ln base);
    between lo = d(fast) rounded down and hi = d(slow) rounded up the frequency goes linearly from f_i to f_i / factor;
    cos and sin are multiplied by 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=F64)
    f = torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def d(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(d(float(scaling["fast"]))), 0)
    hi = min(math.ceil(d(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, freqs: torch.Tensor, mag: float, pos: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [n, ..., 2 m] with m = len(freqs): the pair (x[2i], x[2i+1]) at position p is turned by p f_i and scaled by mag."""
    n = x.shape[0]
    p = torch.arange(n, dtype=F64) if pos is None else pos.to(F64)
    ang = p[:, None] * freqs[None, :]
    shape = [n] + [1] * (x.dim() - 2) + [freqs.shape[0]]
    co, si = (ang.cos() * mag).view(shape), (ang.sin() * mag).view(shape)
    a, b = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = a * co - b * si
    out[..., 1::2] = b * co + a * si
    return out


def visible(n: int, window: int) -> torch.Tensor:
    """[n, n] bool: query i sees key j when 0 <= i - j (< window, if window > 0)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if window > 0:
        ok = ok & (i - j < window)
    return ok


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int) -> torch.Tensor:
    """q, k: [n, H, D]; v: [n, H, V]. Plain soft-max over the visible keys."""
    n = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~visible(n, window)[None], float("-inf"))
    return torch.einsum("hij,jhv->ihv", torch.softmax(s, -1), v)


def latent_of(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], m: str, eps: float) -> torch.Tensor:
    """What a latent-attention layer caches per token: [normed latent | raw extra rows (the shared key part, unrotated)]."""
    C = int(c["kv_rank"])
    z = lin(u, wt[m + "dkv"])
    return torch.cat([unit_rms(z[:, :C], eps) * wt[m + "dkv.norm"], z[:, C:]], -1)


def latent_mixer(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], m: str, eps: float) -> torch.Tensor:
    """Queries through a normed bottleneck, per head [D plain | R rotated]; keys [W_uk c | shared rotated part]."""
    H, D, R, V, C = (int(c[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    n = u.shape[0]
    cq = unit_rms(lin(u, wt[m + "dq"]), eps) * wt[m + "dq.norm"]
    q = lin(cq, wt[m + "uq"]).view(n, H, D + R)
    lat = latent_of(u, c, wt, m, eps)
    cl, kr = lat[:, :C], lat[:, C:]
    rot = c.get("rot") or {}
    if R:
        f, mag = stretched_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        rd = int(rot["dims"])
        q = torch.cat([q[..., :D], rotate_pairs(q[..., D:D + rd], f, mag), q[..., D + rd:]], -1)
        kr = torch.cat([rotate_pairs(kr[:, :rd], f, mag), kr[:, rd:]], -1)
    k = torch.cat([lin(cl, wt[m + "uk"]).view(n, H, D), kr[:, None, :].expand(n, H, R)], -1)
    v = lin(cl, wt[m + "uv"]).view(n, H, V)
    window = int((c.get("mask") or {}).get("size", 0) or 0)
    o = softmax_attention(q, k, v, float(c["scale"]), window)
    return lin(o.reshape(n, H * V), wt[m + "o"])


def latent_mixer_2(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], m: str, eps: float,
                   lat: torch.Tensor) -> torch.Tensor:
    """No positions; `lat` [n, C] is this layer's latent or the one of the layer it borrows from; a sigmoid gate per head."""
    H, D, V = (int(c[k]) for k in ("heads", "dim", "vdim"))
    n = u.shape[0]
    q = lin(u, wt[m + "q"]).view(n, H, D)
    k = lin(lat, wt[m + "uk"]).view(n, H, D)
    v = lin(lat, wt[m + "uv"]).view(n, H, V)
    window = int((c.get("mask") or {}).get("size", 0) or 0)
    o = softmax_attention(q, k, v, float(c["scale"]), window)
    o = o * torch.sigmoid(lin(u, wt[m + "g"]))[:, :, None]
    return lin(o.reshape(n, H * V), wt[m + "o"])


def clamped_glu(u: torch.Tensor, wt: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    """W_down (g sigmoid(1.702 g) (v + 1)), g = min(W_gate u, limit), v = clamp(W_up u, -limit, limit)."""
    g = lin(u, wt[p + "gate"]).clamp(max=limit)
    v = lin(u, wt[p + "up"]).clamp(-limit, limit)
    return lin(g * torch.sigmoid(1.702 * g) * (v + 1.0), wt[p + "down"])


def gated_expert(u: torch.Tensor, wt: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    g = lin(u, wt[p + "gate"])
    return lin(g * torch.sigmoid(g) * lin(u, wt[p + "up"]), wt[p + "down"])


def route(u: torch.Tensor, router: torch.Tensor, top: int, scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chosen experts [n, top] and their weights: soft-max scores, the `top` largest, divided by their sum, times scale."""
    s = torch.softmax(lin(u, router), -1)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20) * scale


def expert_mixture(u: torch.Tensor, c: dict, wt: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    r = c["router"]
    idx, wgt = route(u, wt[p + "router"], int(r["top"]), float(r.get("scale", 1.0)))
    y = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(idx.shape[1]):
            y[t] += wgt[t, j] * gated_expert(u[t:t + 1], wt, f"{p}e{int(idx[t, j])}.")[0]
    if c.get("shared"):
        y = y + torch.sigmoid(lin(u, wt[p + "shared.sg"])) * gated_expert(u, wt, p + "shared.")
    return y


def forward(cfg: dict, wt: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence; `residuals`, if a list, receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = wt["embed"][tokens]
    latents: Dict[int, torch.Tensor] = {}
    for i, l in enumerate(cfg["layers"]):
        p, c, m = f"l{i}.", l["mixer"], f"l{i}.mix."
        u = x + causal_taps(x, wt[p + "canon1"]) if (p + "canon1") in wt else x
        if l["type"] == "gla":
            y = gla_mixer(u, c, wt, m, eps)
        elif l["type"] == "latent_attention":
            y = latent_mixer(u, c, wt, m, eps)
        elif l["type"] == "latent_attention_2":
            src = c.get("kv_from")
            if src is None:
                latents[i] = latent_of(u, c, wt, m, eps)
            y = latent_mixer_2(u, c, wt, m, eps, latents[i if src is None else int(src)])
        else:
            raise ValueError(l["type"])
        x = x + unit_rms(y, eps) * wt[p + "norm1"]
        mlp = l.get("mlp")
        if mlp is not None:
            if mlp.get("kind", "dense") == "dense":
                y = clamped_glu(x, wt, p + "mlp.", float(mlp["limit"]))
            else:
                y = expert_mixture(x, mlp, wt, p + "mlp.")
            x = x + unit_rms(y, eps) * wt[p + "norm2"]
        if residuals is not None:
            residuals.append(x.clone())
    return lin(unit_rms(x, eps) * wt["final.norm"], wt["embed"]) * float(cfg.get("logit_scale", 1.0))


# ---- checkpoints for tests --------------------------------------------------------------------------------------------


def checkpoint_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
    W, out = int(cfg["width"]), {}
    taps = int((cfg.get("canon") or {}).get("taps", 0) or 0)
    out["embed"] = (int(cfg["vocab"]), W)
    for i, l in enumerate(cfg["layers"]):
        p, c, m = f"l{i}.", l["mixer"], f"l{i}.mix."
        out[p + "norm1"] = (W,)
        if taps:
            out[p + "canon1"] = (W, taps)
        H, D, V = int(c["heads"]), int(c["dim"]), int(c["vdim"])
        if l["type"] == "gla":
            rk = int(c.get("decay_rank", 32))
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
            F = int(mlp["expert"]["ff"])
            for e in range(int(mlp["router"]["experts"])):
                out.update({f"{f}e{e}.gate": (F, W), f"{f}e{e}.up": (F, W), f"{f}e{e}.down": (W, F)})
            out[f + "router"] = (int(mlp["router"]["experts"]), W)
            if mlp.get("shared"):
                S = int(mlp["shared"]["ff"])
                out.update({f + "shared.gate": (S, W), f + "shared.up": (S, W), f + "shared.down": (W, S),
                            f + "shared.sg": (1, W)})
    out["final.norm"] = (W,)
    return out


def random_checkpoint(cfg: dict, seed: int, round_bf16: bool = True) -> Dict[str, torch.Tensor]:
    """Seeded float64 tensors (rounded to bf16 values, so that a bf16 copy of them is exact)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, sh in checkpoint_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if name.endswith("a2.b"):
            t = 2.0 + torch.randn(sh, generator=g, dtype=F64)
        elif name.endswith("canon1"):
            t = 0.3 * torch.randn(sh, generator=g, dtype=F64)
        elif len(sh) == 2:
            t = torch.randn(sh, generator=g, dtype=F64) * (sh[1] ** -0.5) * (2.0 if leaf in ("router", "a2") else 1.0)
        else:
            t = 1.0 + 0.1 * torch.randn(sh, generator=g, dtype=F64)
        out[name] = t.to(torch.bfloat16).to(F64) if round_bf16 else t
    return out
