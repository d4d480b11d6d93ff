"""Expert-parallel prefill: the token all-to-all around the grouped GEMMs.

No counterpart in the reference (it is single-GPU).  With G ranks, rank g owns experts
[g*64/G, (g+1)*64/G) -- a contiguous row range of every *_exps tensor -- and a contiguous
1/G of the chunk's tokens for norm / router / select / combine.

Per layer:  dispatch   every local slot (token t, rank k) sends its planar Q8_1 activation row,
                       its 1/rms and its expert id to the rank owning that expert;
            compute    the owner runs count / plan / scatter and the two grouped GEMMs on what
                       it received (a_shift 0: one activation row per received slot);
            return     the per-slot down-projection rows D (fp32[2048]) travel back and are
                       combined in rank order k = 0..3 on the token's home rank.

Determinism: a rank sends its slots to one destination in ascending slot order and receives in
ascending source-rank order; token ranges are contiguous, so every expert sees its slots in
ascending GLOBAL slot order -- the order of the single-GPU permutation.  Each (slot, row) dot
is evaluated in block order whatever tile it lands in, so outputs are bit-identical to the
single-GPU run.

This module is device-agnostic host logic over torch.distributed (NCCL on GPUs, gloo on CPU
for the tests); the arithmetic is injected as `expert_fn`.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

N_EXPERTS, TOP_K = 64, 4


class EPPlan:
    """Routing tables of one layer on one rank (all tensors on the routing device)."""

    def __init__(self, idx: torch.Tensor, world: int, n_experts: int = N_EXPERTS):
        # idx: [m_loc, 4] int32, global expert ids in rank order
        self.world = world
        per = n_experts // world
        flat = idx.reshape(-1).to(torch.int64)
        dest = flat // per                                        # owning rank of every local slot
        # stable sort by destination: ascending slot order inside each destination
        self.send_order = torch.sort(dest, stable=True).indices   # local slot ids, grouped by destination
        self.send_counts = torch.bincount(dest, minlength=world).tolist()
        self.local_expert = (flat - dest * per)[self.send_order].to(torch.int32)   # expert id on the owner
        self.n_send = int(flat.numel())
        self.recv_counts = None

    def exchange_counts(self, group=None):
        sc = torch.tensor(self.send_counts, dtype=torch.int64, device=self.send_order.device)
        rc = torch.empty_like(sc)
        dist.all_to_all_single(rc, sc, group=group)
        self.recv_counts = rc.tolist()
        return self.recv_counts


def all_to_all_rows(rows: torch.Tensor, send_counts, recv_counts, group=None) -> torch.Tensor:
    """rows [n_send, ...] grouped by destination -> rows received, grouped by source rank ascending."""
    out = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(recv_counts),
                           input_split_sizes=list(send_counts), group=group)
    return out


def ep_moe_layer(idx, payloads, expert_fn, world, group=None, n_experts=N_EXPERTS):
    """One expert-parallel MoE layer around `expert_fn`.

    idx       [m_loc, 4] int32   global expert ids of the local tokens (rank order k = 0..3)
    payloads  list of tensors whose row t belongs to local TOKEN t (activation planes, 1/rms ...)
    expert_fn (local_expert[n_recv] int32, [payload rows per received slot...]) -> D [n_recv, H]
    Returns D [m_loc*4, H] in local slot order (slot = t*4 + k), ready for the rank-order combine.
    """
    plan = EPPlan(idx, world, n_experts)
    plan.exchange_counts(group)
    tok = plan.send_order // TOP_K                                  # token of every slot in send order
    sent = [p.index_select(0, tok) for p in payloads]               # one row per slot, grouped by destination
    recv = [all_to_all_rows(s, plan.send_counts, plan.recv_counts, group) for s in sent]
    le = all_to_all_rows(plan.local_expert, plan.send_counts, plan.recv_counts, group)
    d_recv = expert_fn(le, recv)                                    # [n_recv, H], one row per received slot
    d_back = all_to_all_rows(d_recv, plan.recv_counts, plan.send_counts, group)   # back in send order
    D = torch.empty_like(d_back)
    D.index_copy_(0, plan.send_order, d_back)                       # send order -> slot order
    return D, plan


def peer_offsets(count_matrix, me):
    """Offset tables of the peer-memory exchange on rank `me` (the arithmetic of k_ep_route_exchange in
    csrc/lkb_ep.cu, restated on the host for tests and for callers that plan on the CPU).

    count_matrix[s][g] = rows rank s sends to rank g.  Returns (send_base, recv_off, back_base, n_recv):
      send_base[g]  first row of my block inside rank g's receive buffer   = rows lower ranks send to g
      recv_off[s]   first row of source s inside my receive buffer         = rows lower sources send to me
      back_base[s]  first row of my block inside source s's return buffer  = rows s sends to lower ranks
    Receive buffers are therefore source-ascending, return buffers are in the sender's own send order
    (destination-ascending): exactly what all_to_all_single leaves with these split sizes."""
    C = [list(map(int, row)) for row in count_matrix]
    G = len(C)
    send_base = [sum(C[s][g] for s in range(me)) for g in range(G)]
    recv_off = [sum(C[s][me] for s in range(t)) for t in range(G)]
    back_base = [sum(C[t][g] for g in range(me)) for t in range(G)]
    return send_base, recv_off, back_base, sum(C[s][me] for s in range(G))
