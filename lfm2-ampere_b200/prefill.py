"""Batched prefill of the MoE FFN stack on one GPU: the host-side call sequence of the
reference's pf_chunk() for this path (ref: src/engine.cu:1170-1241), one C-ABI call per
reference kernel / launcher:
  k_pf_norm(ffn_norm) -> k_pf_router + k_pf_select (one launch) -> memset(cnt) -> k_pf_moe_count ->
  k_pf_moe_plan -> k_pf_moe_scatter -> pf_gemm_swiglu (gate|up, a_shift 2, scale inv) ->
  pf_gemm_moe (down, a_shift 0) -> k_pf_moe_combine_norm (next layer's first norm)."""
from __future__ import annotations

import torch

from . import api
from .synth import E, H, I, TOPK


def _timed(owner, fn, *args):
    """Run one GEMM entry point; when owner.gemm_events is a list, bracket it with CUDA events on the current stream."""
    ev = getattr(owner, "gemm_events", None)
    if ev is None:
        return fn(*args)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn(*args)
    e1.record()
    ev.append((e0, e1))


class PrefillStack:
    def __init__(self, layers, m, device="cuda"):
        self.layers, self.m = layers, m
        self.gemm_events = None                              # set to a list to time every grouped-GEMM launch
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
        # caller-owned workspace of the grouped GEMM: activation rows in token-tile order (widest: the gate|up input)
        self.gemm_ws = torch.zeros(api.pf_gemm_workspace_bytes(self.max_tiles, H), dtype=torch.uint8, device=device)
        self.launches_per_step = 10 * len(layers)       # kernels per layer (the memset is not a kernel)

    def layer(self, i, next_norm_w=None, next_act=None):
        """One MoE FFN layer over the chunk.  next_norm_w / next_act = (PfAct, inv): where the fused combine + norm
        puts the next consumer's quantised activation (the full model: the next mixer's attn_norm, into the live
        activation buffers); by default the next layer's ffn_norm into scratch."""
        l, m = self.layers[i], self.m
        api.pf_gemm_set_workspace(self.gemm_ws)
        api.k_pf_norm(self.X, l.norm_w, 0, self.a, self.inv, self.h32, m)
        # router + top-4 selection in one launch (the form follows the chunk size: src/engine.cu:1170-1176)
        api.k_pf_router_select(self.h32, m, m <= 256, l.router, l.rbias, self.inv, self.sel, self.sig, self.idx, self.w)
        api.zero_i32(self.cnt, E)
        api.k_pf_moe_count(self.idx, self.ns, self.cnt)
        api.k_pf_moe_plan(self.cnt, self.off, self.tiles, self.ntiles)
        api.k_pf_moe_scatter(self.idx, self.ns, self.off, self.perm)
        g = api.make_pf_gemm([(l.gate_qs, l.gate_d), (l.up_qs, l.up_d)], [I, I, I], I, H // 32, self.a_qs, self.a_sc,
                             exp_stride=I * (H // 32), perm=self.perm, tiles=self.tiles, ntiles=self.ntiles,
                             a_shift=2, scale=self.inv, oqs=self.a2_qs, osc=self.a2_sc, okb=I // 32)
        _timed(self, api.pf_gemm_swiglu, g, self.max_tiles)
        dn = api.make_pf_gemm([(l.down_qs, l.down_d)], [H, H, H], H, I // 32, self.a2_qs, self.a2_sc,
                              exp_stride=H * (I // 32), perm=self.perm, tiles=self.tiles, ntiles=self.ntiles,
                              a_shift=0, out=self.D, out_ld=H)
        _timed(self, api.pf_gemm_moe, dn, self.max_tiles)
        if next_norm_w is None:
            next_norm_w, next_act = self.layers[(i + 1) % len(self.layers)].norm_w, (self.an, self.n_inv)
        api.k_pf_moe_combine_norm(self.X, self.D, self.w, next_norm_w, next_act[0], next_act[1], m)

    def step(self):
        for i in range(len(self.layers)):
            self.layer(i)

    def macs_per_step(self):
        """Useful multiply-accumulates (slots only, as the reference counts them: tests/test_prefill.cu:634)."""
        return len(self.layers) * self.ns * (2 * I * H + H * I)


def shard_layer(l, rank, world):
    """The expert shard [rank*64/world, (rank+1)*64/world) of a layer: contiguous row ranges of the
    stacked *_exps planes (views, no copy).  Router, bias and norm weights are replicated."""
    import copy
    per = E // world
    e0, e1 = rank * per, (rank + 1) * per
    s = copy.copy(l)
    gb, db = I * (H // 32), H * (I // 32)                 # blocks per expert
    s.gate_qs, s.gate_d = l.gate_qs[e0 * gb * 16:e1 * gb * 16], l.gate_d[e0 * gb:e1 * gb]
    s.up_qs, s.up_d = l.up_qs[e0 * gb * 16:e1 * gb * 16], l.up_d[e0 * gb:e1 * gb]
    s.down_qs, s.down_d = l.down_qs[e0 * db * 16:e1 * db * 16], l.down_d[e0 * db:e1 * db]
    return s


class PrefillStackEP:
    """Expert-parallel prefill over torch.distributed (one process per GPU, NCCL).

    Rank r holds tokens [r*m/G, (r+1)*m/G) of the chunk and the experts [r*64/G, (r+1)*64/G) of every
    layer.  Norm, router, selection and the combine run on the token's home rank; the two grouped GEMMs
    run on the expert's owner, fed by a token all-to-all (see ep.py).  Results are bit-identical to
    PrefillStack on one GPU.

    dispatch="nccl": three all_to_all_single calls per layer and one host sync for the split sizes.
    dispatch="peer": the exchange kernels of lkb_ep.cu write rows straight into the owner's buffers in symmetric
    memory (NVLink peer stores + release/acquire flags); counts stay on the device, the host never waits."""

    def __init__(self, layers, m_total, rank, world, device="cuda", group=None, dispatch="nccl"):
        from . import ep as _ep
        self._ep = _ep
        assert m_total % world == 0 and E % world == 0
        if dispatch not in ("nccl", "peer"):
            raise ValueError("dispatch must be 'nccl' or 'peer'")
        if dispatch == "peer" and world > 8:
            raise ValueError("peer dispatch covers one NVSwitch domain: at most 8 ranks")
        self.dispatch = dispatch
        self.rank, self.world, self.group = rank, world, group
        # this library's kernels per layer (memsets, the torch division and NCCL's own kernels not counted)
        self.launches_per_step = (11 if dispatch == "peer" else 15) * len(layers)
        self.layers = layers
        self.shards = [shard_layer(l, rank, world) for l in layers]
        self.m = m_total // world
        self.m_total = m_total
        m, cap = self.m, m_total * TOPK                          # worst case: every slot of the chunk lands here
        self.cap = cap
        self.max_tiles = cap // 64 + E
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
        self.perm = torch.zeros(cap, **i32)
        self.a2_qs = torch.zeros(cap, I, dtype=torch.int8, device=device)
        self.a2_sc = torch.zeros(cap, I // 32, 2, **f32)
        self.D = torch.zeros(cap, H, **f32)
        self.n_qs = torch.zeros(m, H, dtype=torch.int8, device=device)
        self.n_sc = torch.zeros(m, H // 32, 2, **f32)
        self.n_inv = torch.zeros(m, **f32)
        self.a = api.pf_act(self.a_qs, self.a_sc)
        self.an = api.pf_act(self.n_qs, self.n_sc)
        self.recv_slots = []                                     # per layer: slots this rank computed (load balance)
        self.gemm_events = None
        self.gemm_ws = torch.zeros(api.pf_gemm_workspace_bytes(self.max_tiles, H), dtype=torch.uint8, device=device)

    def _alloc_ep(self, device):
        """Buffers of the device-side dispatch (called once)."""
        i32 = dict(dtype=torch.int32, device=device)
        ns = self.m * TOPK
        self.dest = torch.zeros(ns, **i32)
        self.dcnt = torch.zeros(E, **i32)                       # slots per destination rank (first `world` entries)
        self.doff = torch.zeros(E, **i32)
        self.dtiles = torch.zeros(ns // 64 + E, 4, **i32)       # by-product of the plan kernel, unused
        self.dnt = torch.zeros(1, **i32)
        self.send_order = torch.zeros(ns, **i32)
        self.pos = torch.zeros(ns, **i32)
        self.counts = torch.zeros(2, self.world, **i32)         # [0] what I send to each rank, [1] what I receive
        self.counts_host = torch.zeros(2, self.world, dtype=torch.int32).pin_memory()
        if self.dispatch == "peer":
            self._alloc_peer(device)                            # recv_buf and d_back live in symmetric memory
        else:
            self.send_buf = torch.zeros(ns, api.EP_ROW_BYTES, dtype=torch.uint8, device=device)
            self.recv_buf = torch.zeros(self.cap, api.EP_ROW_BYTES, dtype=torch.uint8, device=device)
            self.d_back = torch.zeros(ns, H, dtype=torch.float32, device=device)
        self.r_qs = torch.zeros(self.cap, H, dtype=torch.int8, device=device)
        self.r_sc = torch.zeros(self.cap, H // 32, 2, dtype=torch.float32, device=device)
        self.r_inv = torch.zeros(self.cap, dtype=torch.float32, device=device)
        self.r_le = torch.zeros(self.cap, **i32)
        self.r_act = api.pf_act(self.r_qs, self.r_sc)

    def _alloc_peer(self, device):
        """Symmetric buffers of the peer dispatch (count matrix, flags, receive rows, returned D rows) carved out
        of one allocation, and the per-rank address tables the kernels take."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        G, ns = self.world, self.m * TOPK
        al = lambda n: (n + 255) // 256 * 256
        sizes = [al(4 * G * G), al(4 * 3 * 8), al(self.cap * api.EP_ROW_BYTES), al(ns * H * 4)]
        offs = [0]
        for n in sizes[:-1]:
            offs.append(offs[-1] + n)
        dev = torch.device(device) if not isinstance(device, torch.device) else device
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        self.symm = symm.empty(sum(sizes), dtype=torch.uint8, device=dev)
        self.symm.zero_()
        grp = self.group if self.group is not None else dist.group.WORLD
        self.symm_handle = symm.rendezvous(self.symm, grp)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)                             # nobody publishes a flag before everyone has zeroed
        base = [int(b) for b in self.symm_handle.buffer_ptrs]
        self.peers = api.ep_peers(*[[b + o for b in base] for o in offs])
        cut = lambda k: self.symm[offs[k]:offs[k] + sizes[k]]
        self.flags = cut(1).view(torch.int32)
        self.recv_buf = cut(2)[:self.cap * api.EP_ROW_BYTES].view(self.cap, api.EP_ROW_BYTES)
        self.d_back = cut(3)[:ns * H * 4].view(torch.float32).view(ns, H)
        i32 = dict(dtype=torch.int32, device=dev)
        self.ep_offs = torch.zeros(3 * G + 1, **i32)
        self.ep_status = torch.zeros(1, **i32)
        self.ep_done = torch.zeros(2, **i32)
        self.nrecv = torch.zeros(max(1, len(self.layers)), **i32)
        self.ep_epoch = torch.zeros(1, **i32)                      # advanced on the device, once per layer
        self.home_rows = torch.zeros(self.cap, dtype=torch.int64, device=dev)      # per received row: address of its result row at home

    def prepare(self):
        """Allocate the exchange buffers now (peer dispatch: the symmetric-memory rendezvous, a collective) instead
        of at the first layer call."""
        if not hasattr(self, "send_order"):
            self._alloc_ep(self.X.device)

    def status(self):
        """0, or the code of the exchange wait that ran out (peer dispatch)."""
        return int(self.ep_status.item()) if hasattr(self, "ep_status") else 0

    def _experts_dev(self, li):
        """The two grouped GEMMs over the received rows; the plan (tiles, perm) is already on the device."""
        sh = self.shards[li]
        # the gate|up GEMM's row gather reads the dispatch rows as they arrived (packed: quants | scale pairs | 1/rms, id)
        g = api.make_pf_gemm([(sh.gate_qs, sh.gate_d), (sh.up_qs, sh.up_d)], [I, I, I], I, H // 32, self.recv_buf, self.recv_buf,
                             exp_stride=I * (H // 32), perm=self.perm, tiles=self.tiles, ntiles=self.ntiles,
                             a_shift=0, scale=self.r_inv, oqs=self.a2_qs, osc=self.a2_sc, okb=I // 32)
        _timed(self, api.pf_gemm_swiglu_packed, g, self.max_tiles, api.EP_ROW_BYTES)
        dn = api.make_pf_gemm([(sh.down_qs, sh.down_d)], [H, H, H], H, I // 32, self.a2_qs, self.a2_sc,
                              exp_stride=H * (I // 32), perm=self.perm, tiles=self.tiles, ntiles=self.ntiles,
                              a_shift=0, out=self.D, out_ld=H)
        # result rows go straight into their home ranks' return buffers (NVLink stores from the GEMM's tail warps)
        _timed(self, api.pf_gemm_moe_rows, dn, self.max_tiles, self.home_rows)

    def _exchange_peer(self, i):
        """route + counts -> rows to their owners -> plan + experts -> D rows home, all on the stream."""
        G, ns, per, me = self.world, self.m * TOPK, E // self.world, self.rank
        ep = self.ep_epoch
        api.ep_route_exchange(self.idx, ns, per, self.peers, me, G, ep, self.send_order, self.doff, self.ep_offs, self.ep_status)
        api.ep_pack_push(self.a, self.inv, self.idx, self.send_order, self.doff, self.ep_offs, ns, per, self.peers, me, G, ep,
                         self.pos, self.ep_done[0:])
        api.ep_route_experts(self.recv_buf, self.cap, self.flags, G, ep, self.ep_offs, self.cnt, self.off, self.tiles, self.ntiles,
                             self.perm, self.nrecv[i:i + 1], self.ep_status, self.peers, self.home_rows, self.r_inv)
        self._experts_dev(i)
        api.ep_publish_wait(self.peers, me, G, 2, ep, self.flags, self.ep_status)

    def _experts(self, li, n):
        """count / plan / scatter + the two grouped GEMMs over the n slots received for this rank's experts."""
        sh = self.shards[li]
        if n == 0:
            return
        api.zero_i32(self.cnt, E)
        api.k_pf_moe_count(self.r_le, n, self.cnt)
        api.k_pf_moe_plan(self.cnt, self.off, self.tiles, self.ntiles)
        api.k_pf_moe_scatter(self.r_le, n, self.off, self.perm)
        mt = n // 64 + E
        g = api.make_pf_gemm([(sh.gate_qs, sh.gate_d), (sh.up_qs, sh.up_d)], [I, I, I], I, H // 32, self.r_qs, self.r_sc,
                             exp_stride=I * (H // 32), perm=self.perm, tiles=self.tiles, ntiles=self.ntiles,
                             a_shift=0, scale=self.r_inv, oqs=self.a2_qs, osc=self.a2_sc, okb=I // 32)
        _timed(self, api.pf_gemm_swiglu, g, mt)
        dn = api.make_pf_gemm([(sh.down_qs, sh.down_d)], [H, H, H], H, I // 32, self.a2_qs, self.a2_sc,
                              exp_stride=H * (I // 32), perm=self.perm, tiles=self.tiles, ntiles=self.ntiles,
                              a_shift=0, out=self.D, out_ld=H)
        _timed(self, api.pf_gemm_moe, dn, mt)

    def layer(self, i):
        import torch.distributed as dist
        l, m, G = self.layers[i], self.m, self.world
        ns, per = m * TOPK, E // G
        if not hasattr(self, "send_order"):
            self._alloc_ep(self.X.device)
        api.pf_gemm_set_workspace(self.gemm_ws)
        api.k_pf_norm(self.X, l.norm_w, 0, self.a, self.inv, self.h32, m)
        # the router form follows the CHUNK size, as on one GPU (ref: src/engine.cu:1170-1176)
        api.k_pf_router_select(self.h32, m, self.m_total <= 256, l.router, l.rbias, self.inv, self.sel, self.sig, self.idx, self.w)
        nxt = self.layers[(i + 1) % len(self.layers)]
        if self.dispatch == "peer":
            self._exchange_peer(i)
            api.k_pf_moe_combine_norm_gather(self.X, self.d_back, self.pos, self.w, nxt.norm_w, self.an, self.n_inv, m)
            return
        # slots grouped by destination rank, ascending slot order inside a destination: the same stable
        # count / plan / scatter kernels, keyed by owner rank instead of expert
        torch.div(self.idx.view(-1), per, rounding_mode="floor", out=self.dest)
        api.zero_i32(self.dcnt, E)
        api.k_pf_moe_count(self.dest, ns, self.dcnt)
        api.k_pf_moe_plan(self.dcnt, self.doff, self.dtiles, self.dnt)
        api.k_pf_moe_scatter(self.dest, ns, self.doff, self.send_order)
        self.counts[0].copy_(self.dcnt[:G])
        dist.all_to_all_single(self.counts[1], self.counts[0], group=self.group)
        api.ep_pack_rows(self.a, self.inv, self.idx, self.send_order, ns, per, self.send_buf, self.pos)
        self.counts_host.copy_(self.counts, non_blocking=True)
        torch.cuda.current_stream().synchronize()                 # the one host sync of the layer: split sizes
        sc, rc = self.counts_host[0].tolist(), self.counts_host[1].tolist()
        n = sum(rc)
        dist.all_to_all_single(self.recv_buf[:n], self.send_buf, output_split_sizes=rc, input_split_sizes=sc,
                               group=self.group)
        api.ep_unpack_rows(self.recv_buf, n, self.r_act, self.r_inv, self.r_le)
        self._experts(i, n)
        dist.all_to_all_single(self.d_back, self.D[:n], output_split_sizes=sc, input_split_sizes=rc, group=self.group)
        self.recv_slots.append(n)
        api.k_pf_moe_combine_norm_gather(self.X, self.d_back, self.pos, self.w, nxt.norm_w, self.an, self.n_inv, m)

    def step(self):
        self.recv_slots = []
        for i in range(len(self.layers)):
            self.layer(i)
        if self.dispatch == "peer":
            self.recv_slots = self.nrecv                       # device tensor: read it after the step, if at all
