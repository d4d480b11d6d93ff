"""The allocation-free decode entry point against the ordinary one.  Needs a B200.

lkb_moe_ffn_decode_stack_static is for callers that cannot hand the kernel any scratch memory -- an engine
that spent its whole device budget at start-up, a plug-in inside somebody else's memory pool, a decode loop
that cannot afford the device-wide stall of cudaMalloc.  It must produce exactly what
lkb_moe_ffn_decode_stack produces with caller-provided scratch, call after call, although every call
reuses the same built-in array and finds the previous call's leftovers in it.
(This file sorts last on purpose: a run that stops at the first failure has then run every other test.)
"""
import importlib

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_the_allocating_one_twice(lkb):
    lkb.init(0)
    synth = importlib.import_module("lfm2-ampere_b200.synth")
    decode = importlib.import_module("lfm2-ampere_b200.decode")
    layers = synth.make_model(3, seed=321, zipf_s=1.1)
    st = decode.DecodeStack(layers)
    gen = torch.Generator("cuda").manual_seed(17)
    x0 = torch.randn(2048, device="cuda", generator=gen)
    x1 = torch.randn(2048, device="cuda", generator=gen) * 3.0

    def reference(x_in):
        st.x.copy_(x_in)
        st.step_fused()                               # caller-provided scratch
        torch.cuda.synchronize()
        assert st.status() == 0
        return st.x.clone(), st.sel_idx.clone(), st.sel_w.clone()

    ref0, ref1 = reference(x0), reference(x1)
    idx = torch.full((3, 4), -1, dtype=torch.int32, device="cuda")
    w = torch.full((3, 4), float("nan"), device="cuda")
    # two calls in a row, different inputs, then the first input again: each must match bit for bit
    for x_in, ref in ((x0, ref0), (x1, ref1), (x0, ref0)):
        x = x_in.clone()
        lkb.moe_ffn_decode_stack_static(st.layers_dev, 3, x, idx, w, None)
        torch.cuda.synchronize()
        assert torch.equal(x, ref[0]) and torch.equal(idx, ref[1]) and torch.equal(w, ref[2])
        assert lkb.lib.lkb_moe_ffn_decode_stack_static_status() == 0      # no bounded wait gave up (the word lives in the library)
    # a shape whose scratch does not fit the built-in array is refused, as is a shape the kernel is not built for
    x = x0.clone()
    rc = lkb.lib.lkb_moe_ffn_decode_stack_static(st.layers_dev.data_ptr(), 3, 2048, 1 << 20, 64, 4, 0, x.data_ptr(),
                                                 None, None, None, None)
    assert rc == -10007 and b"scratch" in lkb.lib.lkb_error_string(rc)
    rc = lkb.lib.lkb_moe_ffn_decode_stack_static(st.layers_dev.data_ptr(), 3, 2048, 1024, 64, 4, 0, x.data_ptr(),
                                                 None, None, None, None)
    assert rc == -10001
    assert torch.equal(x, x0)                          # a refused call touches nothing
