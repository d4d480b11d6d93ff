"""Batch-1 decode of the MoE FFN stack: the host-side call sequence of the reference's
forward() for this path (ref: src/engine.cu:739-811), one C-ABI call per reference kernel:
router_dot -> router_top4 -> gemv_q4_0_exp2 -> swiglu -> moe_down_accum (which also
produces the next layer's quantised, un-normalised activation and its ssq)."""
from __future__ import annotations

import torch

from . import api
from .synth import E, H, I, TOPK


class DecodeStack:
    def __init__(self, layers, device="cuda", pf_bytes=2 << 20):
        self.layers = layers
        self.pf_bytes = pf_bytes
        f32 = dict(dtype=torch.float32, device=device)
        self.x = torch.zeros(H, **f32)
        self.h32 = torch.zeros(H, **f32)
        self.xq = torch.zeros(64 * 36, dtype=torch.uint8, device=device)
        self.ssq = torch.zeros(64, **f32)
        self.logits = torch.zeros(E, **f32)
        self.idx = torch.zeros(TOPK, dtype=torch.int32, device=device)
        self.w = torch.zeros(TOPK, **f32)
        self.gu = torch.zeros(2 * TOPK * I, **f32)
        self.xq2 = torch.zeros(TOPK * (I // 32) * 36, dtype=torch.uint8, device=device)
        self.launches_per_step = 1 + 5 * len(layers)
        self._np = [api.norm_prod(l.norm_w, self.h32, self.xq, self.ssq) for l in layers]
        # fused path: one persistent kernel for the whole stack
        self._descs = [api.moe_layer_desc(l) for l in layers]
        self.layers_dev = api.layer_descs_to_device(self._descs)
        self.sync = torch.zeros(2, dtype=torch.int32, device=device)
        self.sel_idx = torch.zeros(len(layers), TOPK, dtype=torch.int32, device=device)
        self.sel_w = torch.zeros(len(layers), TOPK, **f32)
        self._scratch = api.moe_scratch(self.logits, self.gu, self.sync)

    def step_fused(self, per_layer_launch=False):
        """The same token step through lkb_moe_ffn_decode_stack (one launch) or, with
        per_layer_launch, one lkb_moe_ffn_decode launch per layer."""
        if per_layer_launch:
            for i, d in enumerate(self._descs):
                api.moe_ffn_decode(d, self.x, self.sel_idx[i], self.sel_w[i], None, self._scratch)
        else:
            api.moe_ffn_decode_stack(self.layers_dev, len(self.layers), 0, self.x, self.sel_idx, self.sel_w, None,
                                     self._scratch)

    def status(self):
        """0 unless a bounded device-side wait of the fused kernel expired."""
        return int(self.sync[1].item())

    def step(self):
        """One token through every layer; x is updated in place."""
        L = self.layers
        api.norm_produce(self.x, H, self._np[0])
        for i, l in enumerate(L):
            api.k_router_dot(self.h32, l.router, self.logits, l.rbias, None, None, self.ssq, 1e-5)
            api.k_router_top4(self.logits, l.rbias, self.idx, self.w)
            api.k_gemv_q4_0_exp2(l.gate_qs, l.gate_d, l.up_qs, l.up_d, self.xq, I, H // 32, I, 0, self.idx,
                                 self.gu[:TOPK * I], self.gu[TOPK * I:], self.ssq, 1e-5)
            api.k_swiglu(self.gu[:TOPK * I], self.gu[TOPK * I:], TOPK * I, None, self.xq2,
                         l.down_qs, self.idx, H, I // 32, self.pf_bytes)
            nxt = self._np[i + 1] if i + 1 < len(L) else None
            api.k_moe_down_accum(l.down_qs, l.down_d, self.xq2, H, I // 32, H, I // 32, self.idx, self.w, self.x, nxt)

    def bytes_per_step(self):
        return sum(l.weight_bytes_per_token() + 3 * H * 4 for l in self.layers)
