"""Full-model batch-1 decode step: the host-side call sequence of the reference's forward()
(ref: src/engine.cu:480-860) over the C ABI, on a seeded synthetic model with the reference's shapes.

Per token: embedding row (Q6_K) -> 40 layers of [sequence mixer -> MoE FFN] -> output norm folded into the
Q6_K output projection -> argmax, which stores the next token and advances the device-side position.
Sequence mixer of layer i: split-K attention over the fp16 KV cache when i % 4 == 2 (ref: src/engine.cu:310),
else the short gated convolution.  Norms follow the reference's scale-carrying split: whoever produces the
2048 residual values also emits their quantised raw form and sums of squares, the consumer GEMV multiplies by
1/rms; only layer 0's first norm is a kernel of its own (ref: src/engine.cu:510-517).

Everything a step reads is device-resident (token id and position included), so a step is capturable in a
CUDA graph and replays without host involvement.
"""
from __future__ import annotations

import dataclasses

import torch

from . import api
from .synth import E, H, I, TOPK, MoeLayer, _q4, make_layer

N_HEADS, N_KV, HEAD_DIM = 32, 8, 64
CONV_ROWS = 3 * H                      # in_proj emits B | C | X
VOCAB = 65536
SBPR = H // 256


@dataclasses.dataclass
class Mixer:
    is_attn: bool
    attn_norm: torch.Tensor            # fp32 [H], the norm in front of the mixer
    # short convolution (ref: blk.N.shortconv.{in_proj,conv,out_proj})
    in_qs: torch.Tensor = None
    in_d: torch.Tensor = None
    conv_w: torch.Tensor = None        # fp32 [H*3]
    out_qs: torch.Tensor = None        # out_proj (conv) or attn_output (attention), 2048 x 2048
    out_d: torch.Tensor = None
    # attention (ref: blk.N.attn_{q,k,v,output}, attn_{q,k}_norm)
    wq: tuple = None
    wk: tuple = None
    wv: tuple = None
    qnorm: torch.Tensor = None
    knorm: torch.Tensor = None

    def weight_bytes(self):
        blk = 18 * (H // 32)
        return (H + 2 * N_KV * HEAD_DIM + H) * blk if self.is_attn else (CONV_ROWS + H) * blk + 3 * H * 4


@dataclasses.dataclass
class Model:
    mixers: list
    moe: list                          # synth.MoeLayer per layer
    emb: tuple                         # Q6_K planes (ql, qh, sc, d) of the tied embedding / output matrix
    out_norm: torch.Tensor
    theta: float = 1e6                 # the benchmark configuration's RoPE base (the reference model uses 1e7)


def make_q6(gen, rows, device):
    n = rows * SBPR
    ql = torch.randint(0, 256, (n * 128,), dtype=torch.uint8, device=device, generator=gen)
    qh = torch.randint(0, 256, (n * 64,), dtype=torch.uint8, device=device, generator=gen)
    sc = torch.randint(-128, 128, (n * 16,), dtype=torch.int8, device=device, generator=gen)
    d = (torch.rand(n, device=device, generator=gen) * 4e-5).to(torch.float16)
    return ql, qh, sc, d


def make_full_model(n_layers=40, seed=1234, device="cuda", vocab=VOCAB, moe_layers=None):
    """moe_layers: reuse already generated MoE layers (the benchmark shares them with the FFN-stack workload)."""
    gen = torch.Generator(device=device).manual_seed(seed + 1)
    norm = lambda n: (1.0 + 0.05 * torch.randn(n, device=device, generator=gen)).contiguous()
    mixers = []
    for i in range(n_layers):
        if i % 4 == 2:
            mixers.append(Mixer(True, norm(H), wq=_q4(gen, H, H // 32, device), wk=_q4(gen, N_KV * HEAD_DIM, H // 32, device),
                                wv=_q4(gen, N_KV * HEAD_DIM, H // 32, device), qnorm=norm(HEAD_DIM), knorm=norm(HEAD_DIM),
                                **dict(zip(("out_qs", "out_d"), _q4(gen, H, H // 32, device)))))
        else:
            iq, idd = _q4(gen, CONV_ROWS, H // 32, device)
            oq, od = _q4(gen, H, H // 32, device)
            cw = (torch.randn(H * 3, device=device, generator=gen) * 0.1).contiguous()
            mixers.append(Mixer(False, norm(H), in_qs=iq, in_d=idd, conv_w=cw, out_qs=oq, out_d=od))
    moe = moe_layers if moe_layers is not None else [make_layer(seed + 7919 * l, device) for l in range(n_layers)]
    return Model(mixers, moe, make_q6(gen, vocab, device), norm(H))


class DecodeStep:
    """One token per step(); moe_impl 'mega' = all layers in one persistent launch (lkb_decode_layers), 'fused' =
    one persistent launch per MoE layer, 'kernels' = the reference's five launches per MoE layer."""

    def __init__(self, model: Model, max_seq=4352, moe_impl="fused", device="cuda", pf_bytes=2 << 20):
        self.m, self.moe_impl, self.max_seq, self.pf_bytes = model, moe_impl, max_seq, pf_bytes
        f32 = dict(dtype=torch.float32, device=device)
        i32 = dict(dtype=torch.int32, device=device)
        u8 = dict(dtype=torch.uint8, device=device)
        self.vocab = model.emb[3].numel() // SBPR
        self.x, self.h32, self.ssq = torch.zeros(H, **f32), torch.zeros(H, **f32), torch.zeros(64, **f32)
        self.xq = torch.zeros(64 * 36, **u8)                           # mixer-side activation
        self.xqf = torch.zeros(64 * 36, **u8)                          # FFN-side activation: a producer GEMV must not
        #                                         overwrite the blocks its other CTAs still read (ref: src/engine.cu:276-281)
        self.y = torch.zeros(CONV_ROWS, **f32)                         # in_proj output B | C | X
        self.qv, self.kv, self.vv = torch.zeros(H, **f32), torch.zeros(N_KV * HEAD_DIM, **f32), torch.zeros(N_KV * HEAD_DIM, **f32)
        self.part = torch.zeros(N_HEADS * api.ATTN_SPLIT * api.ATTN_PARTW, **f32)
        n_attn = sum(mx.is_attn for mx in model.mixers)
        n_conv = len(model.mixers) - n_attn
        self.kc = torch.zeros(max(1, n_attn), max_seq, N_KV, HEAD_DIM, dtype=torch.float16, device=device)
        self.vc = torch.zeros_like(self.kc)
        self.hist = torch.zeros(max(1, n_conv), 2 * H, **f32)
        self.logits_v = torch.zeros(self.vocab, **f32)
        nb = (self.vocab + 1023) // 1024
        self.am_v, self.am_i = torch.zeros(nb, **f32), torch.zeros(nb, **i32)
        self.d_token, self.d_pos = torch.zeros(1, **i32), torch.zeros(1, **i32)
        # MoE scratch
        self.logits, self.idx, self.w = torch.zeros(E, **f32), torch.zeros(TOPK, **i32), torch.zeros(TOPK, **f32)
        self.gu = torch.zeros(2 * TOPK * I, **f32)
        self.xq2 = torch.zeros(TOPK * (I // 32) * 36, **u8)
        self.sync = torch.zeros(2, **i32)
        self._scratch = api.moe_scratch(self.logits, self.gu, self.sync)
        self._descs = [api.moe_layer_desc(l) for l in model.moe]
        n = len(model.mixers)
        # producer descriptors: what the kernel that completes the residual quantises for its consumer
        self._np_ffn = [api.norm_prod(l.norm_w, self.h32, self.xqf, self.ssq) for l in model.moe]
        nxt = [model.mixers[i + 1].attn_norm if i + 1 < n else model.out_norm for i in range(n)]
        self._np_next = [api.norm_prod(w, None, self.xq, self.ssq) for w in nxt]
        per_moe = 1 if moe_impl == "fused" else 5
        self.launches_per_step = 2 + sum((5 if mx.is_attn else 3) for mx in model.mixers) + per_moe * n + 3
        if moe_impl == "mega":
            self.launches_per_step = 6
            ci = ai = 0
            descs = []
            for mx in model.mixers:
                if mx.is_attn:
                    descs.append(api.mixer_layer_desc(mx, kc=self.kc[ai], vc=self.vc[ai], max_seq=max_seq))
                    ai += 1
                else:
                    descs.append(api.mixer_layer_desc(mx, hist=self.hist[ci]))
                    ci += 1
            self._mx_descs = descs
            self.mixers_dev = api.layer_descs_to_device(descs)
            self.moe_dev = api.layer_descs_to_device(self._descs)
            self.mxbuf = torch.zeros(3072, **f32)
            self._sscratch = api.step_scratch(self.mxbuf, self.part)
            self._np_out = api.norm_prod(model.out_norm, None, self.xq, self.ssq)

    def fill_kv(self, upto, seed=5):
        """Pre-fill the KV caches with N(0,1) up to position `upto` and set the position there."""
        g = torch.Generator(device=self.kc.device).manual_seed(seed)
        self.kc[:, :upto].copy_(torch.randn(self.kc[:, :upto].shape, device=self.kc.device, generator=g).to(torch.float16))
        self.vc[:, :upto].copy_(torch.randn(self.vc[:, :upto].shape, device=self.vc.device, generator=g).to(torch.float16))
        self.d_pos.fill_(upto)

    def bytes_per_step(self, seq_len):
        w = sum(mx.weight_bytes() for mx in self.m.mixers) + sum(l.weight_bytes_per_token() for l in self.m.moe)
        n_attn = sum(mx.is_attn for mx in self.m.mixers)
        return w + self.vocab * SBPR * 210 + n_attn * seq_len * N_KV * HEAD_DIM * 2 * 2

    def status(self):
        return int(self.sync[1].item())

    def step(self):
        m, bpr = self.m, H // 32
        api.k_embed_q6_K(*m.emb, self.d_token, H, self.x)
        api.k_rmsnorm_q8_1(self.x, m.mixers[0].attn_norm, H, 1e-5, None, None, self.xq)     # layer 0 only
        if self.moe_impl == "mega":
            api.decode_layers(self.moe_dev, self.mixers_dev, len(m.mixers), self.x, self.xq, self.d_pos, m.theta,
                              self._np_out, self._scratch, self._sscratch)
            self._tail()
            return
        ci = ai = 0
        for i, (mx, l) in enumerate(zip(m.mixers, m.moe)):
            ssq = None if i == 0 else self.ssq             # layer 0's input is already normalised
            prod = None if self.moe_impl == "fused" else self._np_ffn[i]      # the fused MoE kernel norms x itself
            if mx.is_attn:
                api.k_gemv_q4_0_3(mx.wq[0], mx.wq[1], H, self.qv, mx.wk[0], mx.wk[1], N_KV * HEAD_DIM, self.kv,
                                  mx.wv[0], mx.wv[1], N_KV * HEAD_DIM, self.vv, self.xq, bpr, ssq, 1e-5)
                api.k_qk_norm_rope(self.qv, self.kv, self.vv, mx.qnorm, mx.knorm, self.d_pos, self.kc[ai], self.vc[ai], m.theta)
                api.k_attn_split(self.qv, self.kc[ai], self.vc[ai], self.d_pos, self.part)
                api.k_attn_combine(self.part, self.d_pos, None, self.xq)
                ai += 1
            else:
                api.k_gemv_q4_0(mx.in_qs, mx.in_d, self.xq, CONV_ROWS, bpr, self.y, 0, ssq, 1e-5)
                api.k_shortconv(self.y, mx.conv_w, self.hist[ci], None, self.xq, H)
                ci += 1
            api.k_gemv_q4_0_prod(mx.out_qs, mx.out_d, self.xq, H, bpr, self.x, 1, prod)
            if self.moe_impl == "fused":
                api.moe_ffn_decode(self._descs[i], self.x, None, None, self._np_next[i], self._scratch)
            else:
                api.k_router_dot(self.h32, l.router, self.logits, l.rbias, None, None, self.ssq, 1e-5)
                api.k_router_top4(self.logits, l.rbias, self.idx, self.w)
                api.k_gemv_q4_0_exp2(l.gate_qs, l.gate_d, l.up_qs, l.up_d, self.xqf, I, bpr, I, 0, self.idx,
                                     self.gu[:TOPK * I], self.gu[TOPK * I:], self.ssq, 1e-5)
                api.k_swiglu(self.gu[:TOPK * I], self.gu[TOPK * I:], TOPK * I, None, self.xq2,
                             l.down_qs, self.idx, H, I // 32, self.pf_bytes)
                api.k_moe_down_accum(l.down_qs, l.down_d, self.xq2, H, I // 32, H, I // 32, self.idx, self.w, self.x,
                                     self._np_next[i])
        self._tail()

    def _tail(self):
        api.k_gemv_q6_K(*self.m.emb, self.xq, self.vocab, SBPR, self.logits_v, self.ssq, 1e-5)
        api.k_argmax_part(self.logits_v, self.vocab, self.am_v, self.am_i)
        api.k_argmax_final(self.am_v, self.am_i, self.am_v.numel(), self.d_token, self.d_pos)


class PrefillChunk:
    """Full-model batched prefill of one chunk of m tokens at positions P .. P+m-1: the host-side call sequence of
    the reference's pf_chunk() (ref: src/engine.cu:1024-1250) over the C ABI.  Sequence mixers run as dense
    Q4_0 x Q8_1 GEMMs (tcgen05) around the chunk kernels of lkb_pfmix.cu; the MoE FFN is prefill.PrefillStack's
    layer body, whose fused combine + norm hands the next layer its quantised activation.  Leaves the conv
    histories and KV caches of `state` (a DecodeStep) exactly where decoding continues from."""

    def __init__(self, model: Model, m: int, state: "DecodeStep", device="cuda"):
        from .prefill import PrefillStack
        self.m_, self.model, self.state = m, model, state
        self.moe = PrefillStack(model.moe, m, device)
        f32 = dict(dtype=torch.float32, device=device)
        self.X, self.a_qs, self.a_sc, self.inv = self.moe.X, self.moe.a_qs, self.moe.a_sc, self.moe.inv
        self.a = self.moe.a
        self.Y = torch.zeros(m, CONV_ROWS, **f32)                       # in_proj output, or q|k|v (first 3072 columns' worth)
        self.qh = torch.zeros(m, H, dtype=torch.float16, device=device)
        self.o = torch.zeros(m, H, **f32)
        self.toks = torch.zeros(m, dtype=torch.int32, device=device)
        n_attn = sum(mx.is_attn for mx in model.mixers)
        self.launches_per_step = 1 + 1 + sum((6 if mx.is_attn else 4) for mx in model.mixers) + 9 * len(model.mixers)

    def macs_per_step(self):
        m, n = self.m_, len(self.model.mixers)
        n_attn = sum(mx.is_attn for mx in self.model.mixers)
        dense = (n - n_attn) * (CONV_ROWS + H) * H + n_attn * (H + 2 * N_KV * HEAD_DIM + H) * H
        return m * dense + self.moe.macs_per_step()

    def step(self, P=0):
        m, md, st, moe = self.m_, self.model, self.state, self.moe
        if P < 0 or P + m > st.max_seq:
            raise ValueError(f"chunk [{P}, {P + m}) does not fit the KV cache of {st.max_seq} positions")
        bpr = H // 32
        api.k_pf_embed(*md.emb, self.toks, self.X, H, m)
        norm_ready = False
        ci = ai = 0
        n = len(md.mixers)
        for i, mx in enumerate(md.mixers):
            if not norm_ready:
                api.k_pf_norm(self.X, mx.attn_norm, 1 if i == 0 else 0, self.a, self.inv, None, m)
            scale = None if i == 0 else self.inv
            if mx.is_attn:
                g = api.make_pf_gemm([mx.wq, mx.wk, mx.wv], [H, H + N_KV * HEAD_DIM, H + 2 * N_KV * HEAD_DIM],
                                     H + 2 * N_KV * HEAD_DIM, bpr, self.a_qs, self.a_sc, ntok=m, scale=scale,
                                     out=self.Y, out_ld=H + 2 * N_KV * HEAD_DIM)
                api.pf_gemm_dense(g)
                api.k_pf_qknr(self.Y, mx.qnorm, mx.knorm, P, self.qh, st.kc[ai], st.vc[ai], m, md.theta)
                api.k_pf_attn(self.qh, m, P, st.kc[ai], st.vc[ai], self.o)
                api.k_pf_quant_rows(self.o, H, bpr, self.a, m)
                ai += 1
            else:
                g = api.make_pf_gemm([(mx.in_qs, mx.in_d)], [CONV_ROWS] * 3, CONV_ROWS, bpr, self.a_qs, self.a_sc, ntok=m,
                                     scale=scale, out=self.Y, out_ld=CONV_ROWS)
                api.pf_gemm_dense(g)
                api.k_pf_conv(self.Y, mx.conv_w, st.hist[ci], self.a, m)
                api.k_pf_conv_hist(self.Y, m, st.hist[ci])
                ci += 1
            og = api.make_pf_gemm([(mx.out_qs, mx.out_d)], [H] * 3, H, bpr, self.a_qs, self.a_sc, ntok=m,
                                  out=self.X, out_ld=H, add=1)
            api.pf_gemm_dense(og)
            nxt = md.mixers[i + 1].attn_norm if i + 1 < n else md.out_norm
            moe.layer(i, next_norm_w=nxt, next_act=(self.a, self.inv))
            norm_ready = True
        st.d_pos.fill_(P + m)
