"""Seeded synthetic weights with the shapes and value distributions of the benchmark
configurations (no checkpoint exists offline): Q4_0 nibbles U{1..15} (see _q4), block scale
d = fp16(|N(0, 0.02)|), router gate fp32 N(0, 0.02), norm weights 1 + N(0, 0.05).
Planes are laid out exactly as the reference's planar pack (qs plane + d plane,
experts stacked row-wise), generated directly in device memory."""
from __future__ import annotations

import dataclasses

import numpy as np
import torch

H, E, TOPK, I = 2048, 64, 4, 1536


@dataclasses.dataclass
class MoeLayer:
    gate_qs: torch.Tensor   # uint8 [E*I*64*16]
    gate_d: torch.Tensor    # fp16  [E*I*64]
    up_qs: torch.Tensor
    up_d: torch.Tensor
    down_qs: torch.Tensor   # uint8 [E*H*48*16]
    down_d: torch.Tensor
    router: torch.Tensor    # fp32 [E, H]
    rbias: torch.Tensor     # fp32 [E]
    norm_w: torch.Tensor    # fp32 [H]  (ffn_norm)

    def weight_bytes_per_token(self):
        """Bytes one batch-1 token streams through this layer: router + 4 experts' gate, up, down."""
        return E * H * 4 + 2 * TOPK * I * (H // 32) * 18 + TOPK * H * (I // 32) * 18


def _q4(gen, rows, bpr, device):
    # Nibbles are drawn from 1..15 rather than 0..15: (q - 8) is then exactly zero-mean.  With 0..15 every
    # weight carries a -0.5*d bias, a rank-one common mode with gain ~16 per projection; a single layer
    # does not care, but a 40-layer random stack amplifies it until the fp16 "raw sum" field of Q8_1
    # overflows (the range hazard the reference audits on real weights, ref: src/quant.cuh:33-63).
    n = rows * bpr * 16
    lo = torch.randint(1, 16, (n,), dtype=torch.uint8, device=device, generator=gen)
    hi = torch.randint(1, 16, (n,), dtype=torch.uint8, device=device, generator=gen)
    qs = lo | (hi << 4)
    del lo, hi
    d = (torch.randn(rows * bpr, device=device, generator=gen) * 0.02).abs().to(torch.float16)
    return qs, d


def make_layer(seed: int, device="cuda", zipf_s: float = 0.0, n_exp: int = E) -> MoeLayer:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    gq, gd = _q4(gen, n_exp * I, H // 32, device)
    uq, ud = _q4(gen, n_exp * I, H // 32, device)
    dq, dd = _q4(gen, n_exp * H, I // 32, device)
    router = torch.randn(n_exp, H, device=device, generator=gen) * 0.02
    norm_w = 1.0 + 0.05 * torch.randn(H, device=device, generator=gen)
    if zipf_s > 0:
        # load imbalance: the log of a Zipf(s) law over a seeded permutation of the experts, added
        # to the ranking as the selection bias (scaled into the sigmoid's range)
        rng = np.random.default_rng(seed)
        ranks = rng.permutation(n_exp) + 1
        p = 1.0 / ranks.astype(np.float64) ** zipf_s
        lb = np.log(p / p.sum())
        bias = torch.from_numpy((0.05 * (lb - lb.mean())).astype(np.float32)).to(device)
    else:
        bias = 0.01 * torch.randn(n_exp, device=device, generator=gen)
    return MoeLayer(gq, gd, uq, ud, dq, dd, router.contiguous(), bias.contiguous(), norm_w.contiguous())


def make_model(n_layers: int, seed: int = 1234, device="cuda", zipf_s: float = 0.0):
    return [make_layer(seed + 7919 * l, device, zipf_s) for l in range(n_layers)]
