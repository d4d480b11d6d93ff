#!/usr/bin/env python3
"""Benchmark of the Q4_0 x Q8_1 MoE hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline (one JSON line on stdout, rank 0):
  metric  "bs1 decode tok/s": one step = ONE token through the 40-layer MoE-FFN stack of
          the synthetic model (benchmark configuration 1 repeated over 40 distinct layers:
          router -> top-4 -> gate|up GEMV of the 4 chosen experts -> SwiGLU/Q8_1 -> down
          GEMV + weighted sum + residual + next layer's norm quantiser).  13.6 GB of expert
          weights are resident; a step streams 871 MB of them (which experts depends on the
          token), so nothing is served from the 126 MB L2 twice.
  value   tokens/s with inputs resident in HBM (CUDA-event time, max over ranks).
  e2e     the same steps driven through the public API with the token's hidden state
          copied host->device from pinned memory and the result copied back every step.
  roofline  the dominant kernel (MoE gate|up GEMV): algorithmic bytes / its CUDA-event time.
  prefill   4096-token batched prefill through the same 40 layers (configuration 3, Zipf-
          skewed routing): tok/s, grouped-GEMM TMAC/s and tensor-pipe roofline; expert-
          parallel over N GPUs when N > 1.
Decode does not shard (batch 1): with --gpus N each rank runs an independent replica.
Data are seeded synthetic tensors with the configurations' shapes and value distributions.
"""
import argparse
import importlib
import json
import os
import pathlib
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

N_LAYERS = 40
H, E, TOPK, I = 2048, 64, 4, 1536
LAYER_BYTES = E * H * 4 + 2 * TOPK * I * (H // 32) * 18 + TOPK * H * (I // 32) * 18 + 3 * H * 4   # 21,782,528
GATEUP_BYTES = 2 * TOPK * I * (H // 32) * 18 + 64 * 36 + 2 * TOPK * I * 4                          # per launch
# DRAM traffic of the fused decode kernel per MoE layer, from one ncu capture of a 4-layer launch
# (dram__bytes_read.sum + dram__bytes_write.sum = 87,141,120 + 2,562,816 B; it grows in proportion to the layers)
FUSED_TRAFFIC_PER_LAYER = (87141120 + 2562816) / 4
METRIC = "bs1 decode tok/s"
UNIT = "tok/s"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured", d
    return 6650.0, "fallback", {}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.t.join(timeout=2)
        mhz, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                mhz.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


# --------------------------------------------------------------------------- CPU baseline
_HOST_LAYER = {}


def host_layer(seed=4321):
    """One MoE layer on the host with the benchmark's value distributions (numpy, seeded)."""
    if seed in _HOST_LAYER:
        return _HOST_LAYER[seed]
    rng = np.random.default_rng(seed)

    def q4(rows, bpr):
        qs = rng.integers(0, 256, size=(rows, bpr, 16), dtype=np.uint8)
        d = np.abs(rng.normal(0, 0.02, size=(rows, bpr))).astype(np.float16).view(np.uint16)
        return qs, d
    _HOST_LAYER[seed] = dict(gate=q4(E * I, H // 32), up=q4(E * I, H // 32), down=q4(E * H, I // 32),
                             router=(0.02 * rng.standard_normal((E, H))).astype(np.float32),
                             bias=(0.01 * rng.standard_normal(E)).astype(np.float32),
                             nw=(1 + 0.05 * rng.standard_normal(H)).astype(np.float32))
    return _HOST_LAYER[seed]


def cpu_layer_token(orc, L, x):
    """The checker's statement of one batch-1 MoE FFN layer (the reference's CPU-side formulas)."""
    h32, act, ssq = orc.norm_prod(x, L["nw"])
    inv = orc.norm_inv(ssq)
    logits = orc.router_dot(h32, L["router"], ninv=inv)
    sel, sig = orc.router_gate(logits, L["bias"])
    idx, w = orc.router_select(sel, sig)
    g = orc.gemv_q4_0_exp(L["gate"][0], L["gate"][1], act, I, H // 32, I, 0, idx, ninv=inv)
    u = orc.gemv_q4_0_exp(L["up"][0], L["up"][1], act, I, H // 32, I, 0, idx, ninv=inv)
    act2 = orc.quantize_q8_1(orc.swiglu(g, u))
    xo, _, _, _ = orc.moe_down_accum(L["down"][0], L["down"][1], act2, H, I // 32, H, I // 32, idx, w, x, None)
    return xo


def cpu_baseline(target_s=12.0, max_tokens=None):
    orc = importlib.import_module("oracle.lkb_oracle")
    L = host_layer()
    rng = np.random.default_rng(1)
    x = rng.standard_normal(H).astype(np.float32)
    t0 = time.perf_counter()
    x1 = cpu_layer_token(orc, L, x)
    t1 = time.perf_counter() - t0
    n = max(2, int(target_s / max(t1, 1e-4)))
    if max_tokens:
        n = min(n, max_tokens)
    t0 = time.perf_counter()
    for i in range(n):
        x1 = cpu_layer_token(orc, L, x if i % 2 else x1 * 0.5)
    dt = time.perf_counter() - t0
    per_layer = dt / n
    return {"value": 1.0 / (per_layer * N_LAYERS), "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
            "sample": f"{n} MoE-layer passes of one token on the host (the CPU checker's restatement of the "
                      f"reference formulas, OpenMP over rows); {per_layer * 1e3:.2f} ms per layer, x{N_LAYERS} layers per token"}, per_layer


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per = []
    for _ in range(args.warmup):
        cpu_baseline(target_s=0.5)
    t0 = time.perf_counter()
    for _ in range(max(1, args.steps)):
        cb, per_layer = cpu_baseline(target_s=min(20.0, 60.0 / max(1, args.steps)))
        per.append(per_layer)
    wall = time.perf_counter() - t0
    per_layer = float(np.mean(per))
    val = 1.0 / (per_layer * N_LAYERS)
    cb["value"] = val
    out = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_layer * N_LAYERS * 1e3,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xint4->int32, fp32 accumulate",
           "data": "synthetic (seeded; shapes and distributions of the benchmark configuration)",
           "config": {"workload": f"config 1 x {N_LAYERS} layers: batch-1 MoE FFN stack (64 experts, top-4, "
                                  "hidden 2048, inter 1536, Q4_0 weights x Q8_1 activations); each step here is a "
                                  "bounded sample of MoE-layer passes on the host cores",
                      "wall_s": wall},
           "cpu_baseline": cb,
           "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    print(json.dumps(out), flush=True)


# --------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    lkb = importlib.import_module("lfm2-ampere_b200")
    synth = importlib.import_module("lfm2-ampere_b200.synth")
    decode = importlib.import_module("lfm2-ampere_b200.decode")
    prefill = importlib.import_module("lfm2-ampere_b200.prefill")

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for this path "
                         "(use --impl reference for the host-side baseline)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lkb.init(local)
    lkb.set_pdl(not args.no_pdl)
    hbm_peak, peak_kind, _ = peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    layers = synth.make_model(args.layers, seed=1234, zipf_s=1.1)       # the same model on every rank
    stack = decode.DecodeStack(layers)
    rng = np.random.default_rng(99 + rank)
    n_in = 64
    x_host = torch.from_numpy(rng.standard_normal((n_in, H)).astype(np.float32)).pin_memory()
    y_host = torch.empty(H, dtype=torch.float32).pin_memory()
    x_pool = x_host.cuda()
    st = torch.cuda.current_stream()

    # one CUDA graph per step shape: copy-in of a resident input, then the 201 kernels
    fused = args.decode_impl == "fused"
    use_graph = (not args.no_graph) and not fused
    graph = None
    x_in = torch.zeros(H, device="cuda")
    if use_graph:
        stack.x.copy_(x_pool[0])
        stack.step()                                  # warm the launch path before capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            stack.x.copy_(x_in)
            stack.step()

    def one_step(i, e2e=False):
        if e2e:
            x_in.copy_(x_host[i % n_in], non_blocking=True)
        else:
            x_in.copy_(x_pool[i % n_in])
        if graph is not None:
            graph.replay()
        elif fused:
            stack.x.copy_(x_in)
            stack.step_fused()
        else:
            stack.x.copy_(x_in)
            stack.step()
        if e2e:
            y_host.copy_(stack.x, non_blocking=True)
            st.synchronize()

    for i in range(max(3, args.warmup)):
        one_step(i)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        one_step(i)
    ev1.record()
    barrier()
    ms = max_over_ranks(ev0.elapsed_time(ev1))
    clocks = None
    tok_s = world * args.steps / (ms * 1e-3)

    # end to end: host buffers, copies inside the timed region
    for i in range(3):
        one_step(i, e2e=True)
    barrier()
    ev0.record()
    for i in range(args.steps):
        one_step(i, e2e=True)
    ev1.record()
    barrier()
    ms_e2e = max_over_ranks(ev0.elapsed_time(ev1))
    e2e_tok_s = world * args.steps / (ms_e2e * 1e-3)

    if fused and stack.status() != 0:
        raise SystemExit(f"fused decode kernel reported status {stack.status()} (a bounded wait expired)")
    if fused:
        # the dominant kernel IS the step: one launch of k_moe_ffn_stack per token; its CUDA-event
        # duration over the timed region is ms / steps
        k_ms = ms / args.steps
        ach = args.layers * LAYER_BYTES / (k_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": f"k_moe_ffn_stack (persistent, {args.layers} MoE layers per launch)",
                    "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak,
                    "peak_kind": f"of {peak_kind}", "traffic": args.layers * FUSED_TRAFFIC_PER_LAYER,
                    "algorithmic_bytes_per_launch": args.layers * LAYER_BYTES, "avg_launch_ms": k_ms}
        n_launch = args.steps
    else:
        # dominant kernel: MoE gate|up GEMV, CUDA events around every launch of it while the
        # same steps run un-graphed (the graph hides individual launches from events)
        evs = []
        lkb.set_pdl(False)
        for i in range(min(args.steps, 10)):
            stack.x.copy_(x_pool[i % n_in])
            lkb.norm_produce(stack.x, H, stack._np[0])
            for li, l in enumerate(layers):
                lkb.k_router_dot(stack.h32, l.router, stack.logits, l.rbias, None, None, stack.ssq, 1e-5)
                lkb.k_router_top4(stack.logits, l.rbias, stack.idx, stack.w)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                lkb.k_gemv_q4_0_exp2(l.gate_qs, l.gate_d, l.up_qs, l.up_d, stack.xq, I, H // 32, I, 0, stack.idx,
                                     stack.gu[:TOPK * I], stack.gu[TOPK * I:], stack.ssq, 1e-5)
                b.record()
                evs.append((a, b))
                lkb.k_swiglu(stack.gu[:TOPK * I], stack.gu[TOPK * I:], TOPK * I, None, stack.xq2, l.down_qs, stack.idx,
                             H, I // 32, stack.pf_bytes)
                nxt = stack._np[li + 1] if li + 1 < len(layers) else None
                lkb.k_moe_down_accum(l.down_qs, l.down_d, stack.xq2, H, I // 32, H, I // 32, stack.idx, stack.w, stack.x, nxt)
        torch.cuda.synchronize()
        k_ms = float(np.mean([a.elapsed_time(b) for a, b in evs]))
        lkb.set_pdl(not args.no_pdl)
        ach = GATEUP_BYTES / (k_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "k_gemv_multi<2,6> (MoE gate|up GEMV, 8 x 1536 rows x K2048)",
                    "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak,
                    "peak_kind": f"of {peak_kind}", "traffic": None,
                    "algorithmic_bytes_per_launch": GATEUP_BYTES, "avg_launch_ms": k_ms,
                    "whole_step": {"bytes_per_step": args.layers * LAYER_BYTES,
                                   "achieved_GBs": args.layers * LAYER_BYTES / (ms / args.steps * 1e-3) / 1e9,
                                   "frac": args.layers * LAYER_BYTES / (ms / args.steps * 1e-3) / 1e9 / hbm_peak}}
        n_launch = args.steps * stack.launches_per_step

    # ---------------------------------------------------------------- prefill (configuration 3)
    pf = None
    if not args.no_prefill:
        m = args.pf_tokens
        del graph
        ep = world > 1
        ep_note = None
        if ep:
            ps = None
            if args.ep_dispatch == "peer":
                # the peer exchange needs symmetric memory across the ranks; where the platform refuses it, every rank
                # falls back to the NCCL exchange together (both are this library's GPU paths; the line says which ran)
                good = torch.ones(1, device="cuda")
                try:
                    ps = prefill.PrefillStackEP(layers, m, rank, world, dispatch="peer")
                    ps.prepare()
                except Exception as exc:                                     # noqa: BLE001 - reported in the JSON line
                    good.zero_()
                    ep_note = f"peer exchange unavailable ({type(exc).__name__}: {exc}); NCCL exchange used"
                dist.all_reduce(good, op=dist.ReduceOp.MIN)
                if float(good.item()) == 0.0:
                    ps = None
                    args.ep_dispatch = "nccl"
                    ep_note = ep_note or "peer exchange unavailable on another rank; NCCL exchange used"
            if ps is None:
                ps = prefill.PrefillStackEP(layers, m, rank, world, dispatch="nccl")
        else:
            ps = prefill.PrefillStack(layers, m)
        ml = m // world
        Xall = np.random.default_rng(5).standard_normal((m, H)).astype(np.float32)
        Xh = torch.from_numpy(Xall[rank * ml:(rank + 1) * ml].copy()).pin_memory()       # this rank's tokens
        Xd = Xh.cuda()
        Yh = torch.empty(ml, H, dtype=torch.float32).pin_memory()

        pf_graph = None

        def pf_step(e2e=False):
            ps.X.copy_(Xh if e2e else Xd, non_blocking=True)
            if pf_graph is not None:
                pf_graph.replay()
            else:
                ps.step()
            if e2e:
                Yh.copy_(ps.X, non_blocking=True)
                st.synchronize()
        pf_step()
        if (not ep or args.ep_dispatch == "peer") and not args.no_graph:
            # one CUDA graph for the step's launches (the NCCL exchange has a host sync per layer and cannot be captured)
            torch.cuda.synchronize()
            barrier()
            pf_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(pf_graph, capture_error_mode="thread_local"):
                ps.step()
            pf_step()
        barrier()
        ev0.record()
        for _ in range(args.pf_steps):
            pf_step()
        ev1.record()
        barrier()
        pms = max_over_ranks(ev0.elapsed_time(ev1)) / args.pf_steps
        ev0.record()
        for _ in range(args.pf_steps):
            pf_step(e2e=True)
        ev1.record()
        barrier()
        pms_e2e = max_over_ranks(ev0.elapsed_time(ev1)) / args.pf_steps
        gstat = lkb.lib.lkb_pf_gemm_status()
        if gstat != 0:
            raise SystemExit(f"tensor-core GEMM reported status {gstat} (a bounded wait expired)")
        # int8 tensor peak of this GPU, measured with a library GEMM (timing only): MEASURED_PEAKS.json has no int8 figure
        int8_peak = None
        try:
            A8 = torch.randint(-8, 8, (8192, 8192), dtype=torch.int8, device="cuda")
            B8 = torch.randint(-8, 8, (8192, 8192), dtype=torch.int8, device="cuda")
            for _ in range(3):
                torch._int_mm(A8, B8)
            torch.cuda.synchronize()
            best = 1e9
            for _ in range(5):
                ev0.record()
                torch._int_mm(A8, B8)
                ev1.record()
                torch.cuda.synchronize()
                best = min(best, ev0.elapsed_time(ev1))
            int8_peak = 2 * 8192 ** 3 / (best * 1e-3) / 1e12
            del A8, B8
        except Exception:
            int8_peak = None
        macs = args.layers * m * TOPK * (2 * I * H + H * I)
        tmacs = macs / (pms * 1e-3) / 1e12
        if ep:
            est = torch.tensor([ps.status()], device="cuda")
            dist.all_reduce(est, op=dist.ReduceOp.MAX)                       # every rank leaves together
            if int(est.item()) != 0:
                raise SystemExit(f"expert-parallel exchange reported status {int(est.item())} (a bounded wait expired)")
            mine = torch.as_tensor(ps.recv_slots).sum().to("cuda", torch.float64).reshape(1)
            mx, sm = mine.clone(), mine.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            dist.all_reduce(sm, op=dist.ReduceOp.SUM)
            imbalance = float(mx.item() / (sm.item() / world))
            launches = args.pf_steps * ps.launches_per_step * world
        else:
            cnt = ps.cnt.cpu().numpy()
            imbalance = float(cnt.max() / max(1.0, cnt.mean()))
            launches = args.pf_steps * ps.launches_per_step
        pf = {"metric": "4k prefill tok/s (40-layer MoE-FFN stack)", "tokens": m, "value": m / (pms * 1e-3), "unit": UNIT,
              "ms_per_step": pms, "scaling": "strong", "cuda_graph": pf_graph is not None,
              "parallelism": (f"expert-parallel x{world}: {E // world} experts and {ml} tokens per GPU, token all-to-all "
                              "before and after the grouped GEMMs, " + ("NCCL all_to_all_single with one host sync per layer"
                                                                        if args.ep_dispatch == "nccl" else
                                                                        "peer-memory stores over NVLink with device-side flags, no host sync"))
              if ep else "single GPU",
              "e2e": {"value": m / (pms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": m * H * 4,
                      "d2h_bytes_per_step": m * H * 4},
              "gemm_tmacs": tmacs, "note": ep_note,
              ("slots_per_gpu_max_over_mean" if ep else "last_layer_max_over_mean_slots_per_expert"): imbalance,
              "gpu_launches": launches,
              "roofline": {"bound": "tensor", "achieved": 2 * tmacs, "unit": "TOP/s (int8)",
                           "peak": (int8_peak or 4500.0) * world, "frac": 2 * tmacs / ((int8_peak or 4500.0) * world),
                           "peak_kind": (f"of measured here: torch._int_mm 8192^3, best of 5, on rank 0's GPU, x {world} GPUs" if int8_peak else
                                         "of nominal dense int8 (MEASURED_PEAKS.json records no int8 figure)"),
                           "nominal_int8_tops": 4500.0,
                           "note": "the per-block fp32 scale epilogue on the CUDA cores, not the MMA, bounds this kernel"}}

    # ---------------------------------------------------------------- output projection + argmax (decode tail)
    lm = None
    if not args.no_lmhead:
        V, SB, NCOPY = 65536, 8, 3                      # three weight copies in rotation: 330 MB > L2
        gen = torch.Generator(device="cuda").manual_seed(77)
        copies = []
        for _ in range(NCOPY):
            copies.append((torch.randint(0, 256, (V * SB * 128,), dtype=torch.uint8, device="cuda", generator=gen),
                           torch.randint(0, 256, (V * SB * 64,), dtype=torch.uint8, device="cuda", generator=gen),
                           torch.randint(-128, 128, (V * SB * 16,), dtype=torch.int8, device="cuda", generator=gen),
                           (torch.rand(V * SB, device="cuda", generator=gen) * 4e-4).half()))
        xv = torch.randn(H, device="cuda", generator=gen)
        xq8 = torch.empty(H // 32 * 36, dtype=torch.uint8, device="cuda")
        lkb.k_quantize_q8_1(xv, xq8, H // 32)
        yl = torch.empty(V, dtype=torch.float32, device="cuda")
        pv, pi = torch.empty(V // 1024, device="cuda"), torch.empty(V // 1024, dtype=torch.int32, device="cuda")
        tok = torch.zeros(1, dtype=torch.int32, device="cuda")

        def lm_step(i, tail=True):
            lkb.k_gemv_q6_K(*copies[i % NCOPY], xq8, V, SB, yl, None, 0.0)
            if tail:
                lkb.k_argmax_part(yl, V, pv, pi)
                lkb.k_argmax_final(pv, pi, V // 1024, tok, None)
        # Timed as CUDA-graph replays (30 launches per graph) so that the host's launch rate is not in the figure.
        # GEMV alone: no programmatic overlap between launches.  GEMV + argmax chain: with programmatic dependent
        # launch, as the decode loop runs it (the next GEMV's weight stream starts under the argmax kernels).
        res = []
        for tail in (False, True):
            lkb.set_pdl(tail and not args.no_pdl)
            for i in range(3):
                lm_step(i, tail)
            torch.cuda.synchronize()
            gl = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gl):
                for i in range(30):
                    lm_step(i, tail)
            nrep = max(1, args.lm_steps // 30)
            gl.replay()
            barrier()
            ev0.record()
            for _ in range(nrep):
                gl.replay()
            ev1.record()
            barrier()
            res.append(max_over_ranks(ev0.elapsed_time(ev1)) / (30 * nrep))
            del gl
        lkb.set_pdl(False)
        if lkb.gemv_q6_K_status() != 0:
            raise SystemExit("Q6_K streaming GEMV: a bounded wait expired")
        lm_bytes = V * SB * 210 + H // 32 * 36 + V * 4
        gbs = lm_bytes / (res[0] * 1e-3) / 1e9
        lm = {"metric": "lm_head: Q6_K 65536 x 2048 GEMV (+ two-stage argmax)", "gemv_us": res[0] * 1e3,
              "gemv_argmax_us": res[1] * 1e3, "launches_per_token": 3, "cold_cache": f"{NCOPY} weight copies in rotation (330 MB > L2)",
              "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                           "peak_kind": f"of {peak_kind}", "algorithmic_bytes": lm_bytes,
                           "traffic": 114323968 if V == 65536 else None}}   # ncu dram read + write of one launch (profiles/)
        del copies

    # ---------------------------------------------------------------- Q4_0 x Q8_1 GEMV size sweep (configuration 0 and up)
    sweep = None
    if not args.no_sweep:
        gen2 = torch.Generator(device="cuda").manual_seed(9)
        xq_s = torch.empty(H // 32 * 36, dtype=torch.uint8, device="cuda")
        lkb.k_quantize_q8_1(torch.randn(H, device="cuda", generator=gen2), xq_s, H // 32)
        lkb.set_pdl(False)
        sweep = []
        for rows in (2048, 6144, 65536, 262144):
            nbytes = rows * (H // 32) * 18 + H // 32 * 36 + rows * 4
            ncopy = min(160, max(2, (400 << 20) // nbytes + 1))            # rotate >= 400 MB of weights: every launch streams from HBM
            ws = [(torch.randint(0, 256, (rows * (H // 32) * 16,), dtype=torch.uint8, device="cuda", generator=gen2),
                   (torch.rand(rows * (H // 32), device="cuda", generator=gen2) * 0.02).half()) for _ in range(ncopy)]
            ys = torch.empty(rows, device="cuda")
            nl = max(ncopy, 24)
            for i in range(3):
                lkb.k_gemv_q4_0(ws[i % ncopy][0], ws[i % ncopy][1], xq_s, rows, H // 32, ys)
            torch.cuda.synchronize()
            gs = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gs):
                for i in range(nl):
                    lkb.k_gemv_q4_0(ws[i % ncopy][0], ws[i % ncopy][1], xq_s, rows, H // 32, ys)
            gs.replay()
            barrier()
            ev0.record()
            gs.replay()
            ev1.record()
            barrier()
            us = max_over_ranks(ev0.elapsed_time(ev1)) / nl * 1e3
            sweep.append({"rows": rows, "k": H, "bytes": nbytes, "us": us, "GBs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / hbm_peak})
            del ws, gs

    # ---------------------------------------------------------------- full decode step (configuration 2)
    full = None
    if not args.no_full:
        model_mod = importlib.import_module("lfm2-ampere_b200.model")
        ctx = args.ctx
        fm = model_mod.make_full_model(n_layers=args.layers, seed=4321, moe_layers=layers)
        tok_h = torch.zeros(1, dtype=torch.int32).pin_memory()
        out_h = torch.zeros(1, dtype=torch.int32).pin_memory()
        res = {}
        for impl in ("mega", "kernels"):
            ds = model_mod.DecodeStep(fm, max_seq=ctx + 2 * (args.steps + 8) + 8, moe_impl=impl)
            ds.fill_kv(ctx)
            ds.d_token.fill_(11)
            lkb.set_pdl(impl == "kernels" and not args.no_pdl)
            ds.step()                                         # warm the launch path before capture
            torch.cuda.synchronize()
            gf = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gf):
                ds.step()
            ds.d_pos.fill_(ctx)
            for _ in range(3):
                gf.replay()
            barrier()
            ev0.record()
            for _ in range(args.steps):
                gf.replay()
            ev1.record()
            barrier()
            t_dev = max_over_ranks(ev0.elapsed_time(ev1)) / args.steps
            # end to end: the token id arrives from pinned host memory, the chosen token goes back, every step
            ev0.record()
            for i in range(args.steps):
                tok_h[0] = 11 + i
                ds.d_token.copy_(tok_h, non_blocking=True)
                gf.replay()
                out_h.copy_(ds.d_token, non_blocking=True)
                st.synchronize()
            ev1.record()
            barrier()
            t_e2e = max_over_ranks(ev0.elapsed_time(ev1)) / args.steps
            if ds.status() != 0 or lkb.gemv_q6_K_status() != 0:
                raise SystemExit("full decode step: a bounded device-side wait expired")
            res[impl] = (t_dev, t_e2e, ds.launches_per_step, ds.bytes_per_step(ctx))
            del gf, ds
        lkb.set_pdl(False)
        best = min(res, key=lambda k: res[k][0])
        t_dev, t_e2e, nl, nbytes = res[best]
        gbs = nbytes / (t_dev * 1e-3) / 1e9
        full = {"metric": "bs1 decode tok/s, full model step at context %d" % ctx, "value": world * 1e3 / t_dev, "unit": UNIT,
                "ms_per_step": t_dev, "impl": best,
                "by_impl_ms": {k: v[0] for k, v in res.items()},
                "workload": ("embedding row -> %d layers [short conv (3 of 4) | GQA attention 32/8x64 over an fp16 KV cache (1 of 4)] + "
                             "64-expert top-4 MoE FFN -> Q6_K lm_head (vocab 65536) -> argmax; one CUDA graph per token, token id and "
                             "position device-resident; impl mega = all layers in one persistent launch (6 launches per token), "
                             "kernels = one launch per reference kernel with programmatic dependent launch" % args.layers),
                "e2e": {"value": world * 1e3 / t_e2e, "unit": UNIT, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
                "gpu_launches_per_step": nl, "bytes_per_step": nbytes,
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                             "peak_kind": f"of {peak_kind}", "traffic": None},
                "published_reference": {"value": 424.65, "unit": UNIT, "hardware": "RTX 3090 Ti, real weights, context 4096",
                                        "ratio": (1e3 / t_dev) / 424.65,
                                        "note": "the reference's model has vocab 128000 and two dense FFN layers: 1.467 GB per token "
                                                "against %.3f GB here" % (nbytes / 1e9)} if (ctx == 4096 and args.layers == 40) else None}
        del fm

    # ---------------------------------------------------------------- full-model prefill chunk
    fpf = None
    if not args.no_full and not args.no_prefill and world == 1:
        model_mod = importlib.import_module("lfm2-ampere_b200.model")
        m = args.pf_tokens
        fm = model_mod.make_full_model(n_layers=args.layers, seed=4321, moe_layers=layers)
        stt = model_mod.DecodeStep(fm, max_seq=m + 8, moe_impl="kernels")
        pc = model_mod.PrefillChunk(fm, m, stt)
        tok_hm = torch.randint(0, 65536, (m,), dtype=torch.int32).pin_memory()
        nxt_h = torch.zeros(1, dtype=torch.int32).pin_memory()
        pc.toks.copy_(tok_hm)

        def fpf_step(e2e=False):
            if e2e:
                pc.toks.copy_(tok_hm, non_blocking=True)
            stt.hist.zero_()
            pc.step(P=0)
            if e2e:                                            # the new position comes back to the host
                nxt_h.copy_(stt.d_pos, non_blocking=True)
                st.synchronize()
        fpf_step()
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(args.pf_steps):
            fpf_step()
        ev1.record()
        torch.cuda.synchronize()
        t_pf = ev0.elapsed_time(ev1) / args.pf_steps
        ev0.record()
        for _ in range(args.pf_steps):
            fpf_step(e2e=True)
        ev1.record()
        torch.cuda.synchronize()
        t_pf_e2e = ev0.elapsed_time(ev1) / args.pf_steps
        if lkb.lib.lkb_pf_gemm_status() != 0:
            raise SystemExit("full-model prefill: a bounded wait of the tensor-core GEMM expired")
        attn_macs = sum(mx.is_attn for mx in fm.mixers) * 32 * 64 * 2 * (m * (m + 1) // 2)
        fpf = {"metric": "%dk prefill tok/s, full model chunk" % (m // 1024), "tokens": m, "value": m / (t_pf * 1e-3), "unit": UNIT,
               "ms_per_step": t_pf,
               "workload": "embedding rows -> %d layers [dense Q4_0 x Q8_1 GEMMs + chunk conv | causal GQA flash attention] + "
                           "MoE grouped GEMMs; KV caches and conv histories left ready for decoding" % args.layers,
               "e2e": {"value": m / (t_pf_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 4 * m, "d2h_bytes_per_step": 4},
               "gemm_tmacs": pc.macs_per_step() / (t_pf * 1e-3) / 1e12, "attention_tmacs_total": attn_macs / 1e12,
               "gpu_launches_per_step": pc.launches_per_step,
               "published_reference": {"value": 21188.0, "unit": UNIT, "hardware": "RTX 3090 Ti, real weights, 4096 tokens",
                                       "ratio": (m / (t_pf * 1e-3)) / 21188.0} if (m == 4096 and args.layers == 40) else None}
        del pc, stt, fm

    # ---------------------------------------------------------------- long context (configuration 4)
    longc = None
    if args.long_ctx and world == 1 and not args.no_full:
        model_mod = importlib.import_module("lfm2-ampere_b200.model")
        fm = model_mod.make_full_model(n_layers=args.layers, seed=4321, moe_layers=layers)
        LC = 131072
        ds = model_mod.DecodeStep(fm, max_seq=LC + 64, moe_impl="mega")
        # chunked prefill: 32768 tokens in 8192-token chunks, timed per chunk (attention cost grows with the prefix)
        CH = 8192
        pc = model_mod.PrefillChunk(fm, CH, ds)
        pc.toks.copy_(torch.randint(0, 65536, (CH,), dtype=torch.int32, device="cuda"))
        pc.step(P=0)
        ds.hist.zero_()
        torch.cuda.synchronize()
        chunk_ms = []
        ev_all0, ev_all1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev_all0.record()
        for c in range(4):
            ev0.record()
            pc.step(P=c * CH)
            ev1.record()
            torch.cuda.synchronize()
            chunk_ms.append(ev0.elapsed_time(ev1))
        ev_all1.record()
        torch.cuda.synchronize()
        pf32 = 4 * CH / (sum(chunk_ms) * 1e-3)
        del pc
        # decode at 131072 positions of context
        ds.fill_kv(LC)
        ds.d_token.fill_(11)
        ds.step()
        torch.cuda.synchronize()
        gL = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gL):
            ds.step()
        ds.d_pos.fill_(LC)
        for _ in range(3):
            gL.replay()
        torch.cuda.synchronize()
        nst = min(args.steps, 20)
        ev0.record()
        for _ in range(nst):
            gL.replay()
        ev1.record()
        torch.cuda.synchronize()
        t_l = ev0.elapsed_time(ev1) / nst
        nb = ds.bytes_per_step(LC)
        longc = {"decode_ctx_131072": {"value": 1e3 / t_l, "unit": UNIT, "ms_per_step": t_l, "bytes_per_step": nb,
                                       "roofline": {"bound": "hbm", "achieved": nb / (t_l * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                                                    "frac": nb / (t_l * 1e-3) / 1e9 / hbm_peak, "peak_kind": f"of {peak_kind}"},
                                       "published_reference": {"value": 184.94, "unit": UNIT, "hardware": "RTX 3090 Ti, context 131040"}},
                 "prefill_32768_in_8192_chunks": {"value": pf32, "unit": UNIT, "chunk_ms": chunk_ms,
                                                  "published_reference": {"value": 18190.0, "unit": UNIT, "hardware": "RTX 3090 Ti"}}}
        if ds.status() != 0:
            raise SystemExit("long-context decode: a bounded device-side wait expired")
        del gL, ds, fm

    if rank == 0:
        clocks = sampler.stop()          # sampled over every timed region above (decode, e2e, prefill, lm_head, full step)
        cb, _ = cpu_baseline() if world == 1 and not args.no_cpu else (None, None)
        out = {"metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": world, "steps": args.steps,
               "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True,
               "scaling": "weak", "vs_baseline": None, "dtype": "int8xint4->int32, fp32 accumulate",
               "data": "synthetic (seeded; shapes and distributions of the benchmark configurations)",
               "config": {"workload": f"config 1 x {args.layers} layers: batch-1 MoE FFN stack (64 experts, top-4, hidden "
                                      "2048, inter 1536, Q4_0 weights x Q8_1 activations, sigmoid+bias router)",
                          "layers": args.layers, "resident_weight_bytes": args.layers * 339738624,
                          "bytes_per_token": args.layers * LAYER_BYTES,
                          "cold_cache": "each step streams 871 MB of a 13.6 GB weight set (inputs larger than L2)",
                          "parallelism": "replicas" if world > 1 else "single GPU",
                          "decode_impl": args.decode_impl, "cuda_graph": use_graph, "pdl": (not args.no_pdl) and not fused},
               "e2e": {"value": e2e_tok_s, "unit": UNIT, "h2d_bytes_per_step": H * 4, "d2h_bytes_per_step": H * 4},
               "gpu_launches": n_launch,
               "roofline": roofline, "cpu_baseline": cb, "clocks": clocks, "prefill": pf, "lm_head": lm, "gemv_sweep": sweep, "full_step": full, "full_prefill": fpf, "long_context": longc}
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--pf-tokens", type=int, default=4096)
    ap.add_argument("--pf-steps", type=int, default=3)
    ap.add_argument("--ep-dispatch", choices=["nccl", "peer"], default="peer",
                    help="token exchange of the expert-parallel prefill (N > 1): NCCL all-to-all, or this library's peer-memory kernels")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-lmhead", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the GEMV size sweep")
    ap.add_argument("--long-ctx", action="store_true", help="also time decode at 131072 positions of context and a chunked 32768-token prefill")
    ap.add_argument("--no-full", action="store_true", help="skip the full-model decode step (configuration 2)")
    ap.add_argument("--ctx", type=int, default=4096, help="KV positions pre-filled for the full decode step")
    ap.add_argument("--lm-steps", type=int, default=90)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--decode-impl", default="fused", choices=["fused", "kernels"],
                    help="fused: one persistent launch per token (lkb_moe_ffn_decode_stack); "
                         "kernels: the reference's five launches per layer, graph + PDL")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
