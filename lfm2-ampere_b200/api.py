"""Thin torch-tensor wrappers over the C ABI, named after the reference's kernels.

Each function takes the reference kernel's arguments (device tensors instead of
raw pointers), launches on torch's current CUDA stream through the C entry point
and raises LkbError on a non-zero status.  Nothing here computes anything.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import EpPeers, MixerLayer, MoeLayer, MoeScratch, NormProd, PfAct, PfGemm, StepScratch, check, lib

__all__ = [
    "ptr", "stream", "norm_prod", "pf_act", "make_pf_gemm",
    "k_quantize_q8_1", "k_rmsnorm_q8_1", "norm_produce", "k_gemv_q4_0", "k_gemv_q4_0_prod", "k_gemv_q4_0_3",
    "k_gemv_q4_0_exp2", "k_gemv_q4_0_exp", "k_swiglu", "k_moe_accum4", "k_moe_down_accum", "k_router_dot",
    "k_router_top4", "router_top4_softmax", "block_sumi", "k_pf_norm", "k_pf_quant_rows", "k_pf_swiglu",
    "k_pf_router", "k_pf_router_small", "k_pf_router_tiled", "k_pf_router_select", "k_pf_select", "k_pf_moe_count", "k_pf_moe_plan", "k_pf_moe_scatter",
    "pf_gemm_dense", "pf_gemm_moe", "pf_gemm_swiglu", "k_pf_moe_combine", "k_pf_moe_combine_norm",
    "k_pf_pack_q8_1", "zero_i32", "moe_layer_desc", "moe_scratch", "moe_ffn_decode", "moe_ffn_decode_stack",
    "layer_descs_to_device", "ep_pack_rows", "ep_unpack_rows", "k_pf_moe_combine_norm_gather", "moe_ffn_decode_stack_static", "set_pdl", "pf_gemm_config", "pf_gemm_arith", "pf_gemm_workspace_bytes", "pf_gemm_set_workspace", "sm_count",
    "k_gemv_q6_K", "k_argmax_part", "k_argmax_final", "k_embed_q6_K", "gemv_q6_K_status",
    "k_attn_split", "k_attn_combine", "k_qk_norm_rope", "k_shortconv", "ATTN_SPLIT", "ATTN_PARTW",
    "mixer_layer_desc", "step_scratch", "decode_layers",
    "k_pf_embed", "k_pf_conv", "k_pf_conv_hist", "k_pf_qknr", "k_pf_attn",
    "decode_set_expert_prefetch", "decode_expert_prefetch_hits", "ep_peers", "EP_ROW_BYTES", "ep_set_wait_limit_ms", "ep_route_exchange", "ep_route_experts", "pf_gemm_moe_rows", "pf_gemm_swiglu_packed", "ep_publish_wait", "ep_pack_push", "ep_wait",
]


def ptr(t):
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "device-resident contiguous tensors only"
    return t.data_ptr()


def stream():
    return torch.cuda.current_stream().cuda_stream


def norm_prod(w=None, h32=None, yq8=None, ssq=None):
    """lkb_norm_prod_t from tensors (ref: LKNormProd)."""
    return NormProd(ptr(w), ptr(h32), ptr(yq8), ptr(ssq))


def pf_act(qs, sc):
    return PfAct(ptr(qs), ptr(sc))


def _np(np_):
    return None if np_ is None else C.byref(np_)


def set_pdl(on):
    check(lib.lkb_set_pdl(1 if on else 0))


def pf_gemm_config(cfg):
    check(lib.lkb_pf_gemm_config(int(cfg)))


def pf_gemm_arith(fold):
    check(lib.lkb_pf_gemm_arith(int(fold)))


def pf_gemm_workspace_bytes(max_tiles, k_max):
    n = C.c_size_t(0)
    check(lib.lkb_pf_gemm_workspace_bytes(int(max_tiles), int(k_max), C.byref(n)))
    return n.value


def pf_gemm_set_workspace(buf):
    """Register (or with None unregister) the caller-owned workspace of the grouped tensor-core GEMM."""
    if buf is None:
        check(lib.lkb_pf_gemm_set_workspace(None, 0))
    else:
        check(lib.lkb_pf_gemm_set_workspace(ptr(buf), buf.numel() * buf.element_size()))


def sm_count():
    return lib.lkb_sm_count()


# ------------------------------------------------------------------ decode --
def k_quantize_q8_1(x, y, nblocks):
    check(lib.lkb_quantize_q8_1(ptr(x), ptr(y), nblocks, stream()), "k_quantize_q8_1")


def k_rmsnorm_q8_1(x, w, n, eps, y32, y16, yq8):
    check(lib.lkb_rmsnorm_q8_1(ptr(x), ptr(w), n, eps, ptr(y32), ptr(y16), ptr(yq8), stream()), "k_rmsnorm_q8_1")


def norm_produce(x, n, np_):
    check(lib.lkb_norm_produce(ptr(x), n, C.byref(np_), stream()), "norm_produce")


def k_gemv_q4_0(qs, d, xq, out_rows, bpr, y, add_residual=0, ssq=None, eps=1e-5):
    check(lib.lkb_gemv_q4_0(ptr(qs), ptr(d), ptr(xq), out_rows, bpr, ptr(y), add_residual, ptr(ssq), eps, stream()),
          "k_gemv_q4_0")


def k_gemv_q4_0_prod(qs, d, xq, out_rows, bpr, y, add_residual, np_):
    check(lib.lkb_gemv_q4_0_prod(ptr(qs), ptr(d), ptr(xq), out_rows, bpr, ptr(y), add_residual, _np(np_), stream()),
          "k_gemv_q4_0_prod")


def k_gemv_q4_0_3(qs0, d0, rows0, y0, qs1, d1, rows1, y1, qs2, d2, rows2, y2, xq, bpr, ssq=None, eps=1e-5):
    check(lib.lkb_gemv_q4_0_3(ptr(qs0), ptr(d0), rows0, ptr(y0), ptr(qs1), ptr(d1), rows1, ptr(y1),
                              ptr(qs2), ptr(d2), rows2, ptr(y2), ptr(xq), bpr, ptr(ssq), eps, stream()),
          "k_gemv_q4_0_3")


def k_gemv_q4_0_exp2(qs_a, d_a, qs_b, d_b, xq, out_rows, bpr, rows_per_expert, xq_stride, d_idx, y_a, y_b,
                     ssq=None, eps=1e-5, sel=None, sig=None, idx_out=None, w_out=None):
    check(lib.lkb_gemv_q4_0_exp2(ptr(qs_a), ptr(d_a), ptr(qs_b), ptr(d_b), ptr(xq), out_rows, bpr, rows_per_expert,
                                 xq_stride, ptr(d_idx), ptr(sel), ptr(sig), ptr(idx_out), ptr(w_out),
                                 ptr(y_a), ptr(y_b), ptr(ssq), eps, stream()), "k_gemv_q4_0_exp2")


def k_gemv_q4_0_exp(qs, d, xq, out_rows, bpr, rows_per_expert, xq_stride, d_idx, y):
    check(lib.lkb_gemv_q4_0_exp(ptr(qs), ptr(d), ptr(xq), out_rows, bpr, rows_per_expert, xq_stride, ptr(d_idx),
                                ptr(y), stream()), "k_gemv_q4_0_exp")


def k_swiglu(gate, up, n, out, yq8, pf_qs=None, pf_idx=None, pf_rows_per_expert=0, pf_bpr=0, pf_bytes=0):
    check(lib.lkb_swiglu(ptr(gate), ptr(up), n, ptr(out), ptr(yq8), ptr(pf_qs), ptr(pf_idx), pf_rows_per_expert,
                         pf_bpr, pf_bytes, stream()), "k_swiglu")


def k_moe_accum4(dst, down4, d_w, n, np_=None):
    check(lib.lkb_moe_accum4(ptr(dst), ptr(down4), ptr(d_w), n, _np(np_), stream()), "k_moe_accum4")


def k_moe_down_accum(qs, d, xq, out_rows, bpr, rows_per_expert, xq_stride, d_idx, d_w, dst, np_=None):
    check(lib.lkb_moe_down_accum(ptr(qs), ptr(d), ptr(xq), out_rows, bpr, rows_per_expert, xq_stride, ptr(d_idx),
                                 ptr(d_w), ptr(dst), _np(np_), stream()), "k_moe_down_accum")


def k_router_dot(h, gate_inp, logits, bias=None, sel=None, sig=None, ssq=None, eps=1e-5):
    check(lib.lkb_router_dot(ptr(h), ptr(gate_inp), ptr(logits), ptr(bias), ptr(sel), ptr(sig), ptr(ssq), eps,
                             stream()), "k_router_dot")


def k_router_top4(logits, bias, idx_out, w_out):
    check(lib.lkb_router_top4(ptr(logits), ptr(bias), ptr(idx_out), ptr(w_out), stream()), "k_router_top4")


def router_top4_softmax(logits, bias, idx_out, w_out):
    check(lib.lkb_router_top4_softmax(ptr(logits), ptr(bias), ptr(idx_out), ptr(w_out), stream()),
          "router_top4_softmax")


def block_sumi(qs, xq, rows, bpr, out):
    check(lib.lkb_block_sumi(ptr(qs), ptr(xq), rows, bpr, ptr(out), stream()), "block_sumi")


# ----------------------------------------------------------------- prefill --
def k_pf_norm(X, w, plain, a, inv_out, h32, m):
    check(lib.lkb_pf_norm(ptr(X), ptr(w), plain, a, ptr(inv_out), ptr(h32), m, stream()), "k_pf_norm")


def k_pf_quant_rows(X, ld, kb, a, rows):
    check(lib.lkb_pf_quant_rows(ptr(X), ld, kb, a, rows, stream()), "k_pf_quant_rows")


def k_pf_swiglu(Y, ld, up_off, kb, a, rows):
    check(lib.lkb_pf_swiglu(ptr(Y), ld, up_off, kb, a, rows, stream()), "k_pf_swiglu")


def k_pf_router(H, m, Wr, bias, inv, sel, sig):
    check(lib.lkb_pf_router(ptr(H), m, ptr(Wr), ptr(bias), ptr(inv), ptr(sel), ptr(sig), stream()), "k_pf_router")


def k_pf_router_select(H, m, small_form, Wr, bias, inv, sel, sig, idx, w):
    check(lib.lkb_pf_router_select(ptr(H), m, int(bool(small_form)), ptr(Wr), ptr(bias), ptr(inv), ptr(sel), ptr(sig), ptr(idx), ptr(w),
                                   stream()), "k_pf_router_select")


def k_pf_router_tiled(H, m, Wr, bias, inv, sel, sig):
    check(lib.lkb_pf_router_tiled(ptr(H), m, ptr(Wr), ptr(bias), ptr(inv), ptr(sel), ptr(sig), stream()),
          "k_pf_router_tiled")


def k_pf_router_small(H, m, Wr, bias, inv, sel, sig):
    check(lib.lkb_pf_router_small(ptr(H), m, ptr(Wr), ptr(bias), ptr(inv), ptr(sel), ptr(sig), stream()),
          "k_pf_router_small")


def k_pf_select(sel, sig, m, idx, w):
    check(lib.lkb_pf_select(ptr(sel), ptr(sig), m, ptr(idx), ptr(w), stream()), "k_pf_select")


def k_pf_moe_count(idx, n, cnt):
    check(lib.lkb_pf_moe_count(ptr(idx), n, ptr(cnt), stream()), "k_pf_moe_count")


def zero_i32(p, n):
    check(lib.lkb_zero_i32(ptr(p), n, stream()), "zero_i32")


def k_pf_moe_plan(cnt, off, tiles, ntiles):
    check(lib.lkb_pf_moe_plan(ptr(cnt), ptr(off), ptr(tiles), ptr(ntiles), stream()), "k_pf_moe_plan")


def k_pf_moe_scatter(idx, n, off, perm):
    check(lib.lkb_pf_moe_scatter(ptr(idx), n, ptr(off), ptr(perm), stream()), "k_pf_moe_scatter")


def make_pf_gemm(segs, seg_end, N, bpr, aqs, asc, *, ntok=0, exp_stride=0, perm=None, tiles=None, ntiles=None,
                 a_shift=0, scale=None, out=None, out_ld=0, add=0, oqs=None, osc=None, okb=0):
    """lkb_pf_gemm from tensors; segs = [(qs, d), ...] (1 to 3 stacked weight tensors)."""
    g = PfGemm()
    for i in range(3):
        q, d = segs[min(i, len(segs) - 1)]
        g.qs[i] = ptr(q)
        g.d[i] = ptr(d)
        g.seg_end[i] = seg_end[min(i, len(seg_end) - 1)]
    g.N, g.bpr, g.exp_stride = N, bpr, exp_stride
    g.aqs, g.asc, g.ntok = ptr(aqs), ptr(asc), ntok
    g.perm, g.tiles, g.ntiles = ptr(perm), ptr(tiles), ptr(ntiles)
    g.a_shift, g.scale = a_shift, ptr(scale)
    g.out, g.out_ld, g.add = ptr(out), out_ld, add
    g.oqs, g.osc, g.okb = ptr(oqs), ptr(osc), okb
    return g


def pf_gemm_dense(g):
    check(lib.lkb_pf_gemm_dense(C.byref(g), stream()), "pf_gemm_dense")


def pf_gemm_moe(g, max_tiles):
    check(lib.lkb_pf_gemm_moe(C.byref(g), max_tiles, stream()), "pf_gemm_moe")


def pf_gemm_swiglu(g, max_tiles):
    check(lib.lkb_pf_gemm_swiglu(C.byref(g), max_tiles, stream()), "pf_gemm_swiglu")


def k_pf_moe_combine(X, D, w, m):
    check(lib.lkb_pf_moe_combine(ptr(X), ptr(D), ptr(w), m, stream()), "k_pf_moe_combine")


def k_pf_moe_combine_norm(X, D, w, nw, a, inv_out, m):
    check(lib.lkb_pf_moe_combine_norm(ptr(X), ptr(D), ptr(w), ptr(nw), a, ptr(inv_out), m, stream()),
          "k_pf_moe_combine_norm")


def k_pf_pack_q8_1(a, t, y):
    check(lib.lkb_pf_pack_q8_1(a, t, ptr(y), stream()), "k_pf_pack_q8_1")


# ------------------------------------------------------------ fused decode --
def moe_layer_desc(l, softmax=0):
    """lkb_moe_layer from an object with gate_qs/gate_d/up_qs/up_d/down_qs/down_d/router/rbias/norm_w tensors."""
    return MoeLayer(ptr(l.gate_qs), ptr(l.gate_d), ptr(l.up_qs), ptr(l.up_d), ptr(l.down_qs), ptr(l.down_d),
                    ptr(l.router), ptr(l.rbias), ptr(l.norm_w), softmax)


def layer_descs_to_device(descs):
    """Pack host descriptors into one device byte tensor (the array lkb_moe_ffn_decode_stack walks)."""
    raw = b"".join(bytes(d) for d in descs)
    return torch.frombuffer(bytearray(raw), dtype=torch.uint8).cuda()


def moe_scratch(logits, gu, sync):
    return MoeScratch(ptr(logits), ptr(gu), ptr(sync))


def moe_ffn_decode(desc, x, idx_out, w_out, next_np, scratch):
    check(lib.lkb_moe_ffn_decode(C.byref(desc), ptr(x), ptr(idx_out), ptr(w_out), _np(next_np), C.byref(scratch),
                                 stream()), "moe_ffn_decode")


def moe_ffn_decode_stack(layers_dev, n_layers, softmax, x, idx_out, w_out, next_np, scratch):
    check(lib.lkb_moe_ffn_decode_stack(ptr(layers_dev), n_layers, softmax, ptr(x), ptr(idx_out), ptr(w_out),
                                       _np(next_np), C.byref(scratch), stream()), "moe_ffn_decode_stack")


def moe_ffn_decode_stack_static(layers_dev, n_layers, x, idx_out, w_out, next_np, hidden=2048, inter=1536,
                                n_experts=64, top_k=4, softmax=0):
    """lkb_moe_ffn_decode_stack with the kernel's scratch inside the library (allocates nothing)."""
    check(lib.lkb_moe_ffn_decode_stack_static(ptr(layers_dev), n_layers, hidden, inter, n_experts, top_k, softmax,
                                              ptr(x), ptr(idx_out), ptr(w_out), _np(next_np), stream()),
          "moe_ffn_decode_stack_static")


def decode_set_expert_prefetch(mode):
    """lkb_decode_set_expert_prefetch: bit 0 the MoE stack kernel, bit 1 the whole-step kernel."""
    check(lib.lkb_decode_set_expert_prefetch(int(mode)), "decode_set_expert_prefetch")


def decode_expert_prefetch_hits(scratch, n_layers):
    """(hits, guesses) of the last multi-layer launch on this scratch (waits for the stream)."""
    h, g = C.c_int(0), C.c_int(0)
    check(lib.lkb_decode_expert_prefetch_hits(C.byref(scratch), n_layers, C.byref(h), C.byref(g), stream()),
          "decode_expert_prefetch_hits")
    return h.value, g.value


# ------------------------------------------------- expert-parallel helpers --
EP_ROW_BYTES = 2048 + 512 + 16


def ep_pack_rows(a, inv, idx, send_order, n, experts_per_rank, out, pos):
    check(lib.lkb_ep_pack_rows(a, ptr(inv), ptr(idx), ptr(send_order), n, experts_per_rank, ptr(out), ptr(pos),
                               stream()), "ep_pack_rows")


def ep_unpack_rows(buf, n, a, inv, local_expert):
    check(lib.lkb_ep_unpack_rows(ptr(buf), n, a, ptr(inv), ptr(local_expert), stream()), "ep_unpack_rows")


def k_pf_moe_combine_norm_gather(X, D, pos, w, nw, a, inv_out, m):
    check(lib.lkb_pf_moe_combine_norm_gather(ptr(X), ptr(D), ptr(pos), ptr(w), ptr(nw), a, ptr(inv_out), m, stream()),
          "k_pf_moe_combine_norm_gather")


# ------------------------------------------------ output projection / embedding --
def k_gemv_q6_K(ql, qh, sc, d, xq, out_rows, sbpr, y, ssq=None, eps=1e-5):
    check(lib.lkb_gemv_q6_K(ptr(ql), ptr(qh), ptr(sc), ptr(d), ptr(xq), out_rows, sbpr, ptr(y), ptr(ssq), eps, stream()),
          "k_gemv_q6_K")


def gemv_q6_K_status():
    return lib.lkb_gemv_q6_K_status()


def k_argmax_part(v, n, pv, pi):
    check(lib.lkb_argmax_part(ptr(v), n, ptr(pv), ptr(pi), stream()), "k_argmax_part")


def k_argmax_final(pv, pi, n, d_token, d_pos=None):
    check(lib.lkb_argmax_final(ptr(pv), ptr(pi), n, ptr(d_token), ptr(d_pos), stream()), "k_argmax_final")


def k_embed_q6_K(ql, qh, sc, d, d_token, n, x):
    check(lib.lkb_embed_q6_K(ptr(ql), ptr(qh), ptr(sc), ptr(d), ptr(d_token), n, ptr(x), stream()), "k_embed_q6_K")


# ------------------------------------------------------------ sequence mixers --
ATTN_SPLIT, ATTN_PARTW = 18, 66          # LKB_ATTN_SPLIT / LKB_ATTN_PARTW of include/lkb.h


def k_attn_split(q, kc, vc, d_pos, part):
    check(lib.lkb_attn_split(ptr(q), ptr(kc), ptr(vc), ptr(d_pos), ptr(part), stream()), "k_attn_split")


def k_attn_combine(part, d_pos, out, yq8=None):
    check(lib.lkb_attn_combine(ptr(part), ptr(d_pos), ptr(out), ptr(yq8), stream()), "k_attn_combine")


def k_qk_norm_rope(qf, kf, vf, qn, kn, d_pos, kc, vc, theta=1e7):
    check(lib.lkb_qk_norm_rope(ptr(qf), ptr(kf), ptr(vf), ptr(qn), ptr(kn), ptr(d_pos), ptr(kc), ptr(vc), theta, stream()),
          "k_qk_norm_rope")


def k_shortconv(bcx, conv_w, hist, y, yq8, n, t=0):
    check(lib.lkb_shortconv(ptr(bcx), t, ptr(conv_w), ptr(hist), ptr(y), ptr(yq8), n, stream()), "k_shortconv")


# ------------------------------------------------------------ whole-step kernel --
def mixer_layer_desc(mx, hist=None, kc=None, vc=None, max_seq=0):
    """lkb_mixer_layer from a model.Mixer plus this layer's state (conv history, or KV cache and its capacity in positions)."""
    if mx.is_attn:
        return MixerLayer(1, int(max_seq), ptr(mx.attn_norm), None, None, None, None, ptr(mx.wq[0]), ptr(mx.wq[1]), ptr(mx.wk[0]),
                          ptr(mx.wk[1]), ptr(mx.wv[0]), ptr(mx.wv[1]), ptr(mx.qnorm), ptr(mx.knorm), ptr(kc), ptr(vc),
                          ptr(mx.out_qs), ptr(mx.out_d))
    return MixerLayer(0, 0, ptr(mx.attn_norm), ptr(mx.in_qs), ptr(mx.in_d), ptr(mx.conv_w), ptr(hist), None, None, None,
                      None, None, None, None, None, None, None, ptr(mx.out_qs), ptr(mx.out_d))


def step_scratch(mx, part):
    return StepScratch(ptr(mx), ptr(part))


def decode_layers(moe_dev, mixers_dev, n_layers, x, xq_first, d_pos, theta, next_np, scratch, sscratch):
    check(lib.lkb_decode_layers(ptr(moe_dev), ptr(mixers_dev), n_layers, ptr(x), ptr(xq_first), ptr(d_pos), theta,
                                _np(next_np), C.byref(scratch), C.byref(sscratch), stream()), "decode_layers")


# ------------------------------------------------------------ prefill mixers --
def k_pf_embed(ql, qh, sc, d, toks, x, n, m):
    check(lib.lkb_pf_embed(ptr(ql), ptr(qh), ptr(sc), ptr(d), ptr(toks), ptr(x), n, m, stream()), "k_pf_embed")


def k_pf_conv(Y, cw, hist, a, m):
    check(lib.lkb_pf_conv(ptr(Y), ptr(cw), ptr(hist), a, m, stream()), "k_pf_conv")


def k_pf_conv_hist(Y, m, hist):
    check(lib.lkb_pf_conv_hist(ptr(Y), m, ptr(hist), stream()), "k_pf_conv_hist")


def k_pf_qknr(Y, qn, kn, P, qh, kc, vc, m, theta=1e7):
    check(lib.lkb_pf_qknr(ptr(Y), ptr(qn), ptr(kn), P, ptr(qh), ptr(kc), ptr(vc), m, theta, stream()), "k_pf_qknr")


def k_pf_attn(qh, m, P, kc, vc, o):
    check(lib.lkb_pf_attn(ptr(qh), m, P, ptr(kc), ptr(vc), ptr(o), stream()), "k_pf_attn")


# ------------------------------------------------ expert-parallel exchange over peer memory --
def ep_peers(cmat_ptrs, flag_ptrs, recv_ptrs, dback_ptrs):
    """lkb_ep_peers from four lists of per-rank device addresses (ints)."""
    p = EpPeers()
    for g, (a, b, c_, d) in enumerate(zip(cmat_ptrs, flag_ptrs, recv_ptrs, dback_ptrs)):
        p.cmat[g], p.flags[g], p.recv[g], p.dback[g] = a, b, c_, d
    return p


def ep_route_exchange(idx, n, experts_per_rank, peers, me, G, epoch, send_order, doff, offs, status):
    check(lib.lkb_ep_route_exchange(ptr(idx), n, experts_per_rank, C.byref(peers), me, G, ptr(epoch), ptr(send_order), ptr(doff),
                                    ptr(offs), ptr(status), stream()), "ep_route_exchange")


def ep_route_experts(recv, cap, flags, G, epoch, offs, cnt, off, tiles, ntiles, perm, nrecv_out, status, peers=None, home_rows=None,
                     inv_out=None):
    check(lib.lkb_ep_route_experts(ptr(recv), cap, ptr(flags), G, ptr(epoch), ptr(offs), ptr(cnt), ptr(off), ptr(tiles), ptr(ntiles),
                                   ptr(perm), ptr(nrecv_out), None if peers is None else C.byref(peers), ptr(home_rows), ptr(inv_out),
                                   ptr(status), stream()), "ep_route_experts")


def pf_gemm_swiglu_packed(g, max_tiles, row_pitch):
    check(lib.lkb_pf_gemm_swiglu_packed(C.byref(g), max_tiles, row_pitch, stream()), "pf_gemm_swiglu_packed")


def pf_gemm_moe_rows(g, max_tiles, out_rows):
    check(lib.lkb_pf_gemm_moe_rows(C.byref(g), max_tiles, ptr(out_rows), stream()), "pf_gemm_moe_rows")


def ep_publish_wait(peers, me, G, phase, epoch, flags, status):
    check(lib.lkb_ep_publish_wait(C.byref(peers), me, G, phase, ptr(epoch), ptr(flags), ptr(status), stream()), "ep_publish_wait")


def ep_pack_push(a, inv, idx, send_order, doff, offs, n, experts_per_rank, peers, me, G, epoch, pos, done):
    check(lib.lkb_ep_pack_push(a, ptr(inv), ptr(idx), ptr(send_order), ptr(doff), ptr(offs), n, experts_per_rank, C.byref(peers),
                               me, G, ptr(epoch), ptr(pos), ptr(done), stream()), "ep_pack_push")


def ep_set_wait_limit_ms(ms):
    check(lib.lkb_ep_set_wait_limit_ms(int(ms)), "ep_set_wait_limit_ms")


def ep_wait(flags, phase, G, epoch, status):
    check(lib.lkb_ep_wait(ptr(flags), phase, G, ptr(epoch), ptr(status), stream()), "ep_wait")


