"""What the layer programs of the layer-list families share: the linear layer that picks a GEMM kernel, and the table of
rotation angles."""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import _cabi


def _use_tc(dtype: torch.dtype, k: int) -> bool:
    return dtype == torch.bfloat16 and k % 64 == 0


class _Linear:
    """out[t, :] = X[t, :] @ W^T (fp32 out): the tcgen05 GEMM when the operands are bf16 and K is a multiple of its
    64-element block, else the FMA-pipe GEMM (fp32 operands, odd reduction sizes)."""

    def __init__(self, lib, w: torch.Tensor, x_buf: torch.Tensor, dt: int):
        self.lib, self.w, self.x, self.dt = lib, w, x_buf, dt
        self.N, self.K = int(w.shape[0]), int(w.shape[1])
        assert x_buf.shape[1] == self.K and x_buf.is_contiguous() and w.is_contiguous()
        self.plan = _cabi.GemmPlan(w, x_buf) if _use_tc(w.dtype, self.K) else None

    def accumulates(self, T: int) -> bool:
        """Decode-sized steps stream the weights once: the tcgen05 GEMM then cuts K over enough CTAs to fill the GPU
        and ADDS its partial sums, so the target has to be zero before the launch."""
        return self.plan is not None and T <= 64

    def run(self, out_ptr: int, ldo: int, T: int, flags: int, st: int, mode: int = _cabi.GEMM_STORE_F32,
            zeroed: bool = False) -> None:
        if self.plan is not None:
            if zeroed and mode == _cabi.GEMM_STORE_F32 and self.accumulates(T):
                rc = self.lib.atx_gemm_run(self.plan._h, out_ptr, ldo, T, _cabi.GEMM_ADD_F32, 0, flags, st)
            else:
                rc = self.lib.atx_gemm_run(self.plan._h, out_ptr, ldo, T, mode, 1 if mode == _cabi.GEMM_STORE_F32 else 0,
                                           flags, st)
        else:
            assert mode in (_cabi.GEMM_STORE_F32, _cabi.GEMM_ADD_F32)
            rc = self.lib.atx_gemm_simple(self.w.data_ptr(), self.K, self.x.data_ptr(), self.K, out_ptr, ldo, T, self.N,
                                          self.K, 1 if mode == _cabi.GEMM_ADD_F32 else 0, self.dt, flags, st)
        if rc != 0:
            raise _cabi.AtxError(f"atx error {rc}: {self.lib.atx_last_error().decode()}")


def rotation_table(base: float, dims: int, max_pos: int, device: torch.device) -> torch.Tensor:
    """[max_pos, dims] fp32: cos then sin of p * base^(-2i/dims), i < dims/2, evaluated in float64 on the host."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * torch.pow(torch.tensor(base, dtype=torch.float64),
                                                                          -2.0 * i / dims)[None, :]
    return torch.cat((ang.cos(), ang.sin()), -1).to(torch.float32).contiguous().to(device)


def wavelength_scaled_frequencies(base: float, dims: int, scaling: Optional[dict]) -> List[float]:
    """f_i = base^(-2i/dims), i < dims/2, rescaled by wavelength l = 2 pi / f (`scaling` = factor, low, high, original; None:
    as they are): f stays where l < original / high, becomes f / factor where l > original / low, and between the two is
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low). Float64 on the host."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wl = 2.0 * math.pi / f
            if wl > orig / low:
                f = f / factor
            elif wl >= orig / high:
                s = (orig / wl - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotation_table_for(freqs: List[float], max_pos: int, device: torch.device) -> torch.Tensor:
    """[max_pos, 2 * len(freqs)] fp32: cos then sin of p * f_i for the given frequencies, evaluated in float64 on the host."""
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * torch.tensor(freqs, dtype=torch.float64)[None, :]
    return torch.cat((ang.cos(), ang.sin()), -1).to(torch.float32).contiguous().to(device)


def stretched_frequencies(base: float, dims: int, scaling: Optional[dict]) -> "tuple[List[float], float]":
    """f_i = base^(-2i/dims), i < dims/2, stretched by pair index (`scaling` = factor, original, fast, slow; None: as they
    are), and the magnitude that multiplies every cosine and sine. A pair that makes t turns over `original` positions has
    the index d(t) = dims ln(original / (2 pi t)) / (2 ln base); with lo = floor(d(fast)) and hi = ceil(d(slow)), clipped to
    [0, dims - 1], the share s_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) of f_i is divided by factor:
    f_i (1 - s_i) + f_i s_i / factor. Magnitude 0.1 ln(factor) + 1. Float64 on the host."""
    freqs = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return freqs, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        s = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * s + f * (1.0 - s))
    return out, 0.1 * math.log(factor) + 1.0


def rotation_table_scaled(freqs: List[float], magnitude: float, max_pos: int, device: torch.device) -> torch.Tensor:
    """rotation_table_for with every cosine and sine multiplied by `magnitude` (the rotation kernels apply the table's
    entries as they are, so a rotated pair comes out scaled)."""
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * torch.tensor(freqs, dtype=torch.float64)[None, :]
    return (torch.cat((ang.cos(), ang.sin()), -1) * magnitude).to(torch.float32).contiguous().to(device)
