"""Expert-parallel prefill on 1, 2, 4 and 8 GPUs == the single-GPU prefill, bit for bit, through both exchanges: NCCL
all-to-all and the peer-memory kernels (the cases above the box's GPU count are skipped; world 1 runs the same kernels
against the rank's own buffers).  The exchange's bounded wait is exercised with a flag that nothing sets."""
import importlib
import os
import socket

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, m, n_layers, out, dispatch):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    lkb = importlib.import_module("lfm2-ampere_b200")
    synth = importlib.import_module("lfm2-ampere_b200.synth")
    prefill = importlib.import_module("lfm2-ampere_b200.prefill")
    lkb.init(rank)
    layers = synth.make_model(n_layers, seed=4242, device=f"cuda:{rank}", zipf_s=1.1)     # same model on every rank
    gen = torch.Generator(device=f"cuda:{rank}").manual_seed(9)
    X = torch.randn(m, 2048, device=f"cuda:{rank}", generator=gen)
    ep = prefill.PrefillStackEP(layers, m, rank, world, device=f"cuda:{rank}", dispatch=dispatch)
    ml = m // world
    ep.X.copy_(X[rank * ml:(rank + 1) * ml])
    ep.step()
    torch.cuda.synchronize()
    if dispatch == "peer":                                   # a second step over the same buffers: flags and epochs carry on
        first = ep.X.clone()
        ep.X.copy_(X[rank * ml:(rank + 1) * ml])
        ep.step()
        torch.cuda.synchronize()
        assert torch.equal(first, ep.X)
        graph = torch.cuda.CUDAGraph()                       # nothing in the step depends on the host: it replays from a graph
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            ep.step()
        for _ in range(2):
            ep.X.copy_(X[rank * ml:(rank + 1) * ml])
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(first, ep.X)
    ref = prefill.PrefillStack(layers, m, device=f"cuda:{rank}")
    ref.X.copy_(X)
    ref.step()
    torch.cuda.synchronize()
    ok = torch.equal(ep.X, ref.X[rank * ml:(rank + 1) * ml]) and bool(torch.isfinite(ep.X).all())
    status = lkb.lib.lkb_pf_gemm_status() | ep.status()
    slots = torch.as_tensor(ep.recv_slots).sum().to(f"cuda:{rank}", torch.int64).reshape(1)
    dist.all_reduce(slots)
    ok = ok and int(slots.item()) == n_layers * m * 4        # every slot of the chunk was computed exactly once
    t = torch.tensor([1 if (ok and status == 0) else 0], device=f"cuda:{rank}")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        open(out, "w").write(str(int(t.item())))
    dist.destroy_process_group()


@pytest.mark.parametrize("dispatch", ["nccl", "peer"])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ep_prefill_bitwise_equals_single_gpu(world, dispatch, tmp_path):
    """world 1 runs the whole exchange chain (routing + count exchange, dispatch rows, plan over received rows, result rows
    written home by the GEMM, flags) against the rank's own buffers: the kernels are exercised on a single-GPU box too."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    out = str(tmp_path / "ok")
    mp.spawn(_worker, args=(world, _free_port(), 512, 2, out, dispatch), nprocs=world, join=True)
    assert open(out).read() == "1"


def test_ep_wait_runs_out_and_reports(lkb):
    """A wait on a flag nobody publishes ends by itself, records its code, and leaves the context usable."""
    lkb.init(0)
    flags = torch.zeros(24, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lkb.ep_set_wait_limit_ms(200)
    try:
        epoch = lambda e: torch.tensor([e], dtype=torch.int32, device="cuda")
        flags[8:10] = 3                                       # phase 1, sources 0 and 1 have published epoch 3
        lkb.ep_wait(flags, 1, 2, epoch(3), status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        lkb.ep_wait(flags, 1, 2, epoch(4), status)                   # epoch 4 never comes
        torch.cuda.synchronize()
        assert int(status.item()) == 3
        lkb.ep_wait(flags, 2, 2, epoch(1), status)                   # a recorded code ends later waits at once, code unchanged
        torch.cuda.synchronize()
        assert int(status.item()) == 3
    finally:
        lkb.ep_set_wait_limit_ms(5000)
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0


def test_one_cta_routing_equals_count_plan_scatter(lkb):
    """lkb_ep_route_experts' plan over received rows == lkb_pf_moe_count / _plan / _scatter on the same keys (bit for
    bit, ragged and skewed), and lkb_ep_route_exchange's send order == the same kernels keyed by owner rank."""
    import numpy as np
    lkb.init(0)
    rng = np.random.default_rng(12)
    i32 = dict(dtype=torch.int32, device="cuda")
    for n, per in ((1, 8), (700, 8), (2048, 8), (5000, 32), (16384, 64)):
        keys = np.minimum(rng.geometric(0.08, size=n) - 1, per - 1).astype(np.int32)        # skewed local expert ids
        # received rows: only the key word (uint4 #160, .y) matters to the routing kernel
        rows = torch.zeros(n, lkb.EP_ROW_BYTES, dtype=torch.uint8, device="cuda")
        rows.view(torch.int32).view(n, lkb.EP_ROW_BYTES // 4)[:, 641] = torch.from_numpy(keys).cuda()
        flags = torch.full((24,), 7, **i32)
        epoch = torch.tensor([7], **i32)
        offs = torch.zeros(4, **i32); offs[3] = n                                            # G = 1: [send, recv, back, n]
        mt = n // 64 + 64
        cnt, off, tiles, nt, perm = (torch.full((64,), -1, **i32), torch.full((64,), -1, **i32), torch.full((mt, 4), -1, **i32),
                                     torch.full((1,), -1, **i32), torch.full((n,), -1, **i32))
        nrecv, status = torch.zeros(1, **i32), torch.zeros(1, **i32)
        lkb.ep_route_experts(rows, n, flags, 1, epoch, offs, cnt, off, tiles, nt, perm, nrecv, status)
        k = torch.from_numpy(keys).cuda()
        c2, o2, t2, n2, p2 = (torch.zeros(64, **i32), torch.full((64,), -1, **i32), torch.full((mt, 4), -1, **i32),
                              torch.full((1,), -1, **i32), torch.full((n,), -1, **i32))
        lkb.k_pf_moe_count(k, n, c2)
        lkb.k_pf_moe_plan(c2, o2, t2, n2)
        lkb.k_pf_moe_scatter(k, n, o2, p2)
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and int(nrecv.item()) == n
        assert torch.equal(cnt, c2) and torch.equal(off, o2) and torch.equal(nt, n2) and torch.equal(perm, p2)
        assert torch.equal(tiles[:int(nt.item())], t2[:int(n2.item())])
