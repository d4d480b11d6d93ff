"""The weight pack the C++ host (host/engine.cpp) loads through LK_PACK: one file, every tensor of a model.Model in
the planar layout the kernels read (Q4_0: qs plane + fp16 d plane, experts stacked row-wise; Q6_K: ql / qh / sc / d
planes), so loading is one read and one host-to-device copy with no repacking at start-up -- the role of the
reference's pack file (ref: src/engine.cu:1276-1277, tools/pack.py), not its byte format.

Layout (little-endian):
    0   8 bytes  magic "LKBPACK1"
    8   u32      n_layers
    12  u32      vocab
    16  f32      rope theta
    20  u32      n_tensors
    24  u32 x 2  reserved
    32  n_tensors entries of 64 bytes: name[48] (NUL padded) | u64 offset | u64 nbytes
    then the tensor bytes, each starting on a 256-byte boundary (offsets are from the start of the file).
Tensor names follow the GGUF names of the reference model: blk.N.attn_norm, blk.N.shortconv.{in_proj,conv,out_proj},
blk.N.attn_{q,k,v,output}, blk.N.attn_{q,k}_norm, blk.N.ffn_norm, blk.N.ffn_gate_inp, blk.N.exp_probs_b,
blk.N.ffn_{gate,up,down}_exps, token_embd, output_norm; quantised tensors carry a plane suffix (.qs .d / .ql .qh .sc .d).
"""
from __future__ import annotations

import struct

import numpy as np
import torch

MAGIC = b"LKBPACK1"
ALIGN = 256


def tensors_of(model):
    """[(name, tensor)] of a model.Model, in file order."""
    out = []
    for i, (mx, l) in enumerate(zip(model.mixers, model.moe)):
        p = f"blk.{i}."
        out.append((p + "attn_norm", mx.attn_norm))
        if mx.is_attn:
            for nm, w in (("attn_q", mx.wq), ("attn_k", mx.wk), ("attn_v", mx.wv), ("attn_output", (mx.out_qs, mx.out_d))):
                out += [(p + nm + ".qs", w[0]), (p + nm + ".d", w[1])]
            out += [(p + "attn_q_norm", mx.qnorm), (p + "attn_k_norm", mx.knorm)]
        else:
            out += [(p + "shortconv.in_proj.qs", mx.in_qs), (p + "shortconv.in_proj.d", mx.in_d),
                    (p + "shortconv.conv", mx.conv_w),
                    (p + "shortconv.out_proj.qs", mx.out_qs), (p + "shortconv.out_proj.d", mx.out_d)]
        out += [(p + "ffn_norm", l.norm_w), (p + "ffn_gate_inp", l.router), (p + "exp_probs_b", l.rbias),
                (p + "ffn_gate_exps.qs", l.gate_qs), (p + "ffn_gate_exps.d", l.gate_d),
                (p + "ffn_up_exps.qs", l.up_qs), (p + "ffn_up_exps.d", l.up_d),
                (p + "ffn_down_exps.qs", l.down_qs), (p + "ffn_down_exps.d", l.down_d)]
    for suf, t in zip(("ql", "qh", "sc", "d"), model.emb):
        out.append(("token_embd." + suf, t))
    out.append(("output_norm", model.out_norm))
    return out


def _bytes(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().cpu().view(torch.uint8).reshape(-1).numpy()


def write_pack(model, path, vocab=None):
    ts = tensors_of(model)
    vocab = vocab if vocab is not None else model.emb[3].numel() // 8          # 8 superblocks of 256 per 2048-wide row
    head = 32 + 64 * len(ts)
    off = (head + ALIGN - 1) // ALIGN * ALIGN
    table = []
    for name, t in ts:
        nb = t.numel() * t.element_size()
        if len(name.encode()) > 47:
            raise ValueError(f"tensor name too long: {name}")
        table.append((name, off, nb))
        off = (off + nb + ALIGN - 1) // ALIGN * ALIGN
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<IIfIII", len(model.mixers), vocab, float(model.theta), len(ts), 0, 0))
        for name, o, nb in table:
            f.write(name.encode().ljust(48, b"\0") + struct.pack("<QQ", o, nb))
        for (name, t), (_, o, nb) in zip(ts, table):
            f.seek(o)
            f.write(_bytes(t).tobytes())
        f.truncate(off)
    return off


def read_table(path):
    """Header and tensor table of a pack: ({n_layers, vocab, theta}, {name: (offset, nbytes)})."""
    with open(path, "rb") as f:
        h = f.read(32)
        if h[:8] != MAGIC:
            raise ValueError("not an LKBPACK1 file")
        n_layers, vocab, theta, n, _, _ = struct.unpack("<IIfIII", h[8:])
        tab = {}
        for _ in range(n):
            e = f.read(64)
            o, nb = struct.unpack("<QQ", e[48:])
            tab[e[:48].rstrip(b"\0").decode()] = (o, nb)
    return dict(n_layers=n_layers, vocab=vocab, theta=theta), tab
