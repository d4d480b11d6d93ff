"""The C++ host (host/engine.cpp): `engine gen <token ids>` / LK_PROMPT_BIN / LK_NGEN / RESULT line, the interface of
the reference's engine for this path (ref: src/engine.cu:1276, 1612-1626, 1729-1734, 1763-1797).

CPU: the binary is built, refuses to start without its pack or its tokens the way the reference does, and the pack
writer's table round-trips.  GPU: the engine's token stream equals the Python call sequence's (model.PrefillChunk in
the same chunks, then model.DecodeStep) on the same seeded model, token for token."""
import os
import pathlib
import struct
import subprocess
import types

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parent.parent
ENGINE = ROOT / "host" / "engine"


@pytest.fixture(scope="module")
def engine():
    subprocess.run(["make", "-C", str(ROOT / "host")], check=True, capture_output=True)
    assert ENGINE.exists()
    return ENGINE


def _run(engine, args, env=None, **kw):
    e = {k: v for k, v in os.environ.items() if not k.startswith("LK_")}
    e.update(env or {})
    return subprocess.run([str(engine)] + args, env=e, capture_output=True, text=True, timeout=600, **kw)


def test_engine_refuses_without_pack_or_tokens(engine, tmp_path):
    r = _run(engine, ["gen", "1", "2"])
    assert r.returncode == 1 and "LK_PACK not set" in r.stderr
    r = _run(engine, ["ppl"], {"LK_PACK": "x"})
    assert r.returncode == 1 and "unknown mode" in r.stderr
    r = _run(engine, ["gen"], {"LK_PACK": "x"})
    assert r.returncode == 1 and "usage" in r.stderr
    bad = tmp_path / "odd.bin"
    bad.write_bytes(b"\x01\x02\x03")
    r = _run(engine, ["gen"], {"LK_PACK": "x", "LK_PROMPT_BIN": str(bad)})
    assert r.returncode == 1 and "int32 blob" in r.stderr
    r = _run(engine, ["gen", "1", "2", "3"], {"LK_PACK": "x", "LK_NGEN": "8", "LK_MAX_SEQ": "4"})
    assert r.returncode == 1 and "LK_MAX_SEQ" in r.stderr


def test_pack_table_round_trip(tmp_path):
    import importlib
    pack = importlib.import_module("lfm2-ampere_b200.pack")
    g = torch.Generator().manual_seed(0)
    u8 = lambda n: torch.randint(0, 256, (n,), dtype=torch.uint8, generator=g)
    f32 = lambda n: torch.randn(n, generator=g)
    f16 = lambda n: torch.randn(n, generator=g).to(torch.float16)
    conv = types.SimpleNamespace(is_attn=False, attn_norm=f32(8), in_qs=u8(48), in_d=f16(3), conv_w=f32(24), out_qs=u8(16), out_d=f16(1))
    attn = types.SimpleNamespace(is_attn=True, attn_norm=f32(8), wq=(u8(16), f16(1)), wk=(u8(16), f16(1)), wv=(u8(16), f16(1)),
                                 out_qs=u8(16), out_d=f16(1), qnorm=f32(4), knorm=f32(4))
    moe = lambda: types.SimpleNamespace(norm_w=f32(8), router=f32(16), rbias=f32(2), gate_qs=u8(32), gate_d=f16(2), up_qs=u8(32),
                                        up_d=f16(2), down_qs=u8(32), down_d=f16(2))
    model = types.SimpleNamespace(mixers=[conv, attn], moe=[moe(), moe()], emb=(u8(128), u8(64), u8(16).view(torch.int8), f16(1)),
                                  out_norm=f32(8), theta=1e6)
    path = tmp_path / "m.pack"
    size = pack.write_pack(model, path, vocab=1)
    assert path.stat().st_size == size
    head, tab = pack.read_table(path)
    assert head["n_layers"] == 2 and head["vocab"] == 1 and head["theta"] == 1e6
    raw = path.read_bytes()
    for name, t in pack.tensors_of(model):
        off, nb = tab[name]
        assert off % 256 == 0 and nb == t.numel() * t.element_size()
        assert raw[off:off + nb] == t.contiguous().view(torch.uint8).numpy().tobytes(), name
    assert "blk.0.shortconv.in_proj.qs" in tab and "blk.1.attn_q.d" in tab and "token_embd.ql" in tab


@pytest.mark.gpu
def test_engine_token_stream_equals_python_call_sequence(engine, tmp_path):
    import importlib
    M = importlib.import_module("lfm2-ampere_b200.model")
    pack = importlib.import_module("lfm2-ampere_b200.pack")
    vocab, n_layers, n_prompt, ngen, chunk = 4096, 3, 41, 6, 32            # conv, conv, attention; chunks of 32 + 8, last token by decode
    model = M.make_full_model(n_layers=n_layers, seed=11, vocab=vocab)
    path = tmp_path / "m.pack"
    pack.write_pack(model, path)
    toks = torch.randint(0, vocab, (n_prompt,), dtype=torch.int32, generator=torch.Generator().manual_seed(5))
    blob = tmp_path / "prompt.bin"
    blob.write_bytes(struct.pack(f"<{n_prompt - 3}i", *toks[3:].tolist()))
    # the first three ids by argv, the rest by LK_PROMPT_BIN (appended, as in the reference)
    r = _run(engine, ["gen"] + [str(int(t)) for t in toks[:3]],
             {"LK_PACK": str(path), "LK_PROMPT_BIN": str(blob), "LK_NGEN": str(ngen), "LK_PF_CHUNK": str(chunk)})
    assert r.returncode == 0, r.stderr
    lines = r.stdout.strip().splitlines()
    got = [int(v) for v in lines[0].split()]
    res = dict(kv.split("=") for kv in lines[-1].split()[1:])
    assert lines[-1].startswith("RESULT ") and int(res["prompt_n"]) == n_prompt and int(res["generated"]) == ngen
    assert int(res["ctx"]) == n_prompt + ngen and res["prefill_mode"] == "batch" and int(res["prefill_batches"]) == 2
    assert float(res["prefill_tok_s"]) > 0 and float(res["tok_s"]) > 0

    st = M.DecodeStep(model, max_seq=n_prompt + ngen + 8, moe_impl="mega")
    nb = n_prompt - 1
    P = 0
    while P < nb:
        m = min(chunk, nb - P)
        pc = M.PrefillChunk(model, m, st)
        pc.toks.copy_(toks[P:P + m].cuda())
        pc.step(P=P)
        torch.cuda.synchronize()
        del pc
        P += m
    st.d_token.copy_(toks[nb:nb + 1].cuda())
    want = []
    for _ in range(ngen):
        st.step()
        want.append(int(st.d_token.item()))
    assert st.status() == 0
    assert got == want
