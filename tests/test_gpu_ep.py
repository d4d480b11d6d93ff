"""Expert-parallel prefill on 2+ GPUs == the single-GPU prefill, bit for bit.  Needs >= 2 B200s
(skipped on a single-GPU box)."""
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


def _worker(rank, world, port, m, n_layers, out):
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
    ep = prefill.PrefillStackEP(layers, m, rank, world, device=f"cuda:{rank}")
    ml = m // world
    ep.X.copy_(X[rank * ml:(rank + 1) * ml])
    ep.step()
    torch.cuda.synchronize()
    ref = prefill.PrefillStack(layers, m, device=f"cuda:{rank}")
    ref.X.copy_(X)
    ref.step()
    torch.cuda.synchronize()
    ok = torch.equal(ep.X, ref.X[rank * ml:(rank + 1) * ml]) and bool(torch.isfinite(ep.X).all())
    status = lkb.lib.lkb_pf_gemm_status()
    t = torch.tensor([1 if (ok and status == 0) else 0], device=f"cuda:{rank}")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        open(out, "w").write(str(int(t.item())))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ep_prefill_bitwise_equals_single_gpu(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    out = str(tmp_path / "ok")
    mp.spawn(_worker, args=(world, _free_port(), 512, 2, out), nprocs=world, join=True)
    assert open(out).read() == "1"
