"""Expert parallelism for the MoE FFN: contiguous expert bands per rank, tokens data-parallel,
all-to-all dispatch and combine over `torch.distributed` (NCCL on GPUs, gloo in the CPU tests).

The reference's `ExpertParallelBackend` (crates/infr-vulkan/src/ep.rs:1-53, 454-493) keeps the
tokens replicated, remaps out-of-band expert ids to weight 0 and all-reduces the per-band partial
outputs.  Here each rank owns a slice of the TOKENS as well: it routes its own rows with the full
(replicated) router, sends every (token, expert) pair's row to the rank that owns the expert,
runs its local experts over what it received, returns the results and sums them in rank order.
The sums are the reference's sums (same band partition `[r*E/W, (r+1)*E/W)`, ep.rs:12-14), only
the data movement differs.

The exchange logic is independent of where the math runs: `ExpertParallel` takes three callables
(route / expert rows / combine) so the same code runs with the CUDA library on GPUs and with a
stand-in expert function in the world-size-2 gloo tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    """Bookkeeping of one dispatch: everything the combine needs to undo it."""
    order: torch.Tensor          # [P] pair indices sorted by (destination rank, expert)
    pos_of_pair: torch.Tensor    # [P] i32 position of pair p in the sorted order
    send_splits: list            # rows sent to each rank
    recv_splits: list            # rows received from each rank
    recv_counts: torch.Tensor    # [W, E_local] rows per (source rank, local expert)
    group_order: torch.Tensor    # [n_recv] received-row index for each expert-grouped row
    seg_off: torch.Tensor        # [E_local + 1] i32 offsets of the local experts' segments


class ExpertParallel:
    """route_fn(x) -> (ids [R,k] int32, wts [R,k] f32)
    expert_fn(x_rows [n, ne], seg_off [E_local+1] int32) -> y_rows [n, ne]   (local experts)
    combine_fn(y_sorted [P, ne], pos_of_pair [P] int32, wts [R,k], x [R, ne]) -> out [R, ne]"""

    def __init__(self, n_expert: int, n_used: int, route_fn: Callable, expert_fn: Callable, combine_fn: Callable,
                 group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_expert % self.world:
            raise ValueError(f"n_expert {n_expert} is not a multiple of the world size {self.world}")  # ep.rs:171-176
        self.n_expert, self.n_used, self.e_local = n_expert, n_used, n_expert // self.world
        self.route_fn, self.expert_fn, self.combine_fn = route_fn, expert_fn, combine_fn
        self.check_ids = False

    # -- exchange ---------------------------------------------------------------------------------
    def _a2a(self, out, inp, out_splits=None, in_splits=None):
        if self.world == 1:
            out.copy_(inp)
        else:
            dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group)

    def plan(self, ids: torch.Tensor) -> DispatchPlan:
        """Counts exchange + the permutations of one dispatch.  `ids` [R, k] global expert ids."""
        W, EL = self.world, self.e_local
        flat = ids.reshape(-1).to(torch.int64)
        if self.check_ids and flat.numel() and (int(flat.min()) < 0 or int(flat.max()) >= self.n_expert):
            raise ValueError("expert id out of range")  # (costs a host synchronisation: off by default)
        order = torch.argsort(flat, stable=True)          # expert-ascending = rank-major, expert-minor
        counts = torch.bincount(flat, minlength=self.n_expert).reshape(W, EL)
        recv_counts = torch.empty_like(counts)
        self._a2a(recv_counts, counts, None, None)
        send_splits = counts.sum(1).tolist()
        recv_splits = recv_counts.sum(1).tolist()
        # received rows arrive source-major, expert-minor; the local GEMM wants expert-major
        e_of_row = torch.repeat_interleave(torch.arange(EL, device=ids.device).repeat(W), recv_counts.reshape(-1))
        group_order = torch.argsort(e_of_row, stable=True)
        seg = torch.zeros(EL + 1, dtype=torch.int64, device=ids.device)
        seg[1:] = torch.cumsum(recv_counts.sum(0), 0)
        pos = torch.empty_like(order)
        pos[order] = torch.arange(order.numel(), device=ids.device)
        return DispatchPlan(order, pos.to(torch.int32), send_splits, recv_splits, recv_counts, group_order,
                            seg.to(torch.int32))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x: this rank's token rows [R, ne] (f32).  Returns the MoE FFN output for those rows."""
        ids, wts = self.route_fn(x)
        pl = self.plan(ids)
        ne = x.shape[1]
        # dispatch: one row per (token, expert) pair, grouped by destination rank
        send = x[pl.order // self.n_used].contiguous()
        n_recv = int(sum(pl.recv_splits))
        recv = torch.empty(n_recv, ne, dtype=x.dtype, device=x.device)
        self._a2a(recv, send, pl.recv_splits, pl.send_splits)
        # local experts over the received rows, grouped by expert
        xg = recv[pl.group_order].contiguous()
        yg = self.expert_fn(xg, pl.seg_off)
        if yg.shape != xg.shape:
            raise RuntimeError(f"expert_fn returned {tuple(yg.shape)} for rows {tuple(xg.shape)}")
        y_recv = torch.empty_like(yg)
        y_recv[pl.group_order] = yg
        # return exchange: the mirror image of the dispatch
        y_sorted = torch.empty(send.shape[0], ne, dtype=yg.dtype, device=x.device)
        self._a2a(y_sorted, y_recv, pl.send_splits, pl.recv_splits)
        return self.combine_fn(y_sorted, pl.pos_of_pair, wts, x)


# -------------------------------------------------------------------------------------------------
# CUDA wiring
# -------------------------------------------------------------------------------------------------

class CudaExpertParallelLayer:
    """One MoE layer sharded over the ranks of the default process group, math on the CUDA library.

    `layer` is a devgen.DeviceLayer holding the FULL router and shared expert (replicated) and the
    banks of THIS rank's experts only (`n_local` experts, see devgen.DeviceLayer(..., band=...))."""

    def __init__(self, be, layer, n_expert: int, n_used: int, n_ff: int, ne: int, scale: float = 1.0, gating: int = 0,
                 norm_w: bool = True, n_groups: int = 0, n_groups_used: int = 0):
        from .backend import DType, MoeFfn
        self.be, self.L = be, layer
        self.ne, self.n_ff, self.n_used, self.n_expert = ne, n_ff, n_used, n_expert
        self._MoeFfn, self._DType = MoeFfn, DType
        self.kw = dict(scale=scale, gating=gating, norm_w=norm_w, n_expert_groups=n_groups, n_expert_groups_used=n_groups_used)
        # the index plumbing runs as torch ops: put the library's kernels on the same stream
        s = torch.cuda.current_stream().cuda_stream
        be.set_stream(s if s != 0 else 1)  # 1 = the legacy default stream handle (0 would mean "own stream")
        self.ep = ExpertParallel(n_expert, n_used, self._route, self._experts, self._combine)
        self.has_shared = "sh_gate" in layer.b

    def _route(self, x):
        be, b = self.be, self.L.b
        R = x.shape[0]
        ids = torch.empty(R, self.n_used, dtype=torch.int32, device=x.device)
        wts = torch.empty(R, self.n_used, dtype=torch.float32, device=x.device)
        xb = be.wrap_tensor(x)
        be.moe_route(self._MoeFfn(x=xb, router=b["router"], gate_exps=b["router"], up_exps=b["router"], down_exps=b["router"],
                                  dst=xb, rows=R, ne=self.ne, n_expert=self.n_expert, n_used=self.n_used, n_ff_exp=self.n_ff,
                                  exp_probs_b=b.get("bias"), ids_out=be.wrap_tensor(ids), wts_out=be.wrap_tensor(wts), **self.kw))
        return ids, wts

    def _experts(self, xg, seg_off):
        be, b = self.be, self.L.b
        y = torch.empty_like(xg)
        if xg.shape[0]:
            be.moe_expert_rows(be.wrap_tensor(xg), be.wrap_tensor(seg_off), b["gate"], b["up"], b["down"], be.wrap_tensor(y),
                               xg.shape[0], self.ep.e_local, self.ne, self.n_ff)
        return y

    def _combine(self, y_sorted, pos_of_pair, wts, x):
        be, b = self.be, self.L.b
        R = x.shape[0]
        out = torch.empty(R, self.ne, dtype=torch.float32, device=x.device)
        sh_rows = sh_logit = None
        keep = []
        if self.has_shared:
            # the shared expert is replicated: every rank runs it over its own tokens
            sh = torch.empty_like(x)
            seg = torch.tensor([0, R], dtype=torch.int32, device=x.device)
            xb = be.wrap_tensor(x)
            be.moe_expert_rows(xb, be.wrap_tensor(seg), b["sh_gate"], b["sh_up"], b["sh_down"], be.wrap_tensor(sh), R, 1, self.ne,
                               self.n_ff)
            sh_rows = be.wrap_tensor(sh)
            keep += [sh, seg]
            if "sh_gate_inp" in b:
                gl = torch.empty(R, dtype=torch.float32, device=x.device)
                sh_logit = be.wrap_tensor(gl)
                be.linear(self._DType.F32, b["sh_gate_inp"], xb, sh_logit, R, self.ne, 1)
                keep.append(gl)
        n_y = max(int(y_sorted.shape[0]), 1)
        yb = be.wrap_tensor(y_sorted) if y_sorted.shape[0] else be.wrap_tensor(torch.zeros(1, self.ne, device=x.device))
        be.moe_combine(yb, be.wrap_tensor(pos_of_pair), be.wrap_tensor(wts), be.wrap_tensor(out), R, self.n_used, self.ne, n_y,
                       sh_rows=sh_rows, sh_logit=sh_logit)
        be.sync()  # the temporaries above must outlive the kernels that read them
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.ep.forward(x)
