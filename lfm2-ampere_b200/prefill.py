"""Batched prefill of the MoE FFN stack on one GPU: the host-side call sequence of the
reference's pf_chunk() for this path (ref: src/engine.cu:1170-1241), one C-ABI call per
reference kernel / launcher:
  k_pf_norm(ffn_norm) -> k_pf_router -> k_pf_select -> memset(cnt) -> k_pf_moe_count ->
  k_pf_moe_plan -> k_pf_moe_scatter -> pf_gemm_swiglu (gate|up, a_shift 2, scale inv) ->
  pf_gemm_moe (down, a_shift 0) -> k_pf_moe_combine_norm (next layer's first norm)."""
from __future__ import annotations

import torch

from . import api
from .synth import E, H, I, TOPK


class PrefillStack:
    def __init__(self, layers, m, device="cuda"):
        self.layers, self.m = layers, m
        ns = m * TOPK
        self.ns = ns
        self.max_tiles = ns // 64 + E                       # ref: src/engine.cu:1007
        f32 = dict(dtype=torch.float32, device=device)
        i32 = dict(dtype=torch.int32, device=device)
        self.X = torch.zeros(m, H, **f32)
        self.a_qs = torch.zeros(m, H, dtype=torch.int8, device=device)
        self.a_sc = torch.zeros(m, H // 32, 2, **f32)
        self.inv = torch.zeros(m, **f32)
        self.h32 = torch.zeros(m, H, **f32)
        self.sel = torch.zeros(m, E, **f32)
        self.sig = torch.zeros(m, E, **f32)
        self.idx = torch.zeros(m, TOPK, **i32)
        self.w = torch.zeros(m, TOPK, **f32)
        self.cnt = torch.zeros(E, **i32)
        self.off = torch.zeros(E, **i32)
        self.tiles = torch.zeros(self.max_tiles, 4, **i32)
        self.ntiles = torch.zeros(1, **i32)
        self.perm = torch.zeros(ns, **i32)
        self.a2_qs = torch.zeros(ns, I, dtype=torch.int8, device=device)
        self.a2_sc = torch.zeros(ns, I // 32, 2, **f32)
        self.D = torch.zeros(ns, H, **f32)
        # the combine's fused norm feeds the next layer's mixer in the full model; here it lands in scratch
        self.n_qs = torch.zeros(m, H, dtype=torch.int8, device=device)
        self.n_sc = torch.zeros(m, H // 32, 2, **f32)
        self.n_inv = torch.zeros(m, **f32)
        self.a = api.pf_act(self.a_qs, self.a_sc)
        self.a2 = api.pf_act(self.a2_qs, self.a2_sc)
        self.an = api.pf_act(self.n_qs, self.n_sc)
        self.launches_per_step = 9 * len(layers)        # kernels per layer (the memset is not a kernel)

    def layer(self, i):
        l, m = self.layers[i], self.m
        api.k_pf_norm(self.X, l.norm_w, 0, self.a, self.inv, self.h32, m)
        api.k_pf_router(self.h32, m, l.router, l.rbias, self.inv, self.sel, self.sig)
        api.k_pf_select(self.sel, self.sig, m, self.idx, self.w)
        api.zero_i32(self.cnt, E)
        api.k_pf_moe_count(self.idx, self.ns, self.cnt)
        api.k_pf_moe_plan(self.cnt, self.off, self.tiles, self.ntiles)
        api.k_pf_moe_scatter(self.idx, self.ns, self.off, self.perm)
        g = api.make_pf_gemm([(l.gate_qs, l.gate_d), (l.up_qs, l.up_d)], [I, I, I], I, H // 32, self.a_qs, self.a_sc,
                             exp_stride=I * (H // 32), perm=self.perm, tiles=self.tiles, ntiles=self.ntiles,
                             a_shift=2, scale=self.inv, oqs=self.a2_qs, osc=self.a2_sc, okb=I // 32)
        api.pf_gemm_swiglu(g, self.max_tiles)
        dn = api.make_pf_gemm([(l.down_qs, l.down_d)], [H, H, H], H, I // 32, self.a2_qs, self.a2_sc,
                              exp_stride=H * (I // 32), perm=self.perm, tiles=self.tiles, ntiles=self.ntiles,
                              a_shift=0, out=self.D, out_ld=H)
        api.pf_gemm_moe(dn, self.max_tiles)
        nxt = self.layers[(i + 1) % len(self.layers)]
        api.k_pf_moe_combine_norm(self.X, self.D, self.w, nxt.norm_w, self.an, self.n_inv, m)

    def step(self):
        for i in range(len(self.layers)):
            self.layer(i)

    def macs_per_step(self):
        """Useful multiply-accumulates (slots only, as the reference counts them: tests/test_prefill.cu:634)."""
        return len(self.layers) * self.ns * (2 * I * H + H * I)
