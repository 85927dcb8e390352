"""Expert parallelism for the MoE FFN: contiguous expert bands per rank, tokens data-parallel,
all-to-all dispatch and combine over `torch.distributed` (NCCL on GPUs, gloo in the CPU tests).

The reference's `ExpertParallelBackend` (crates/infr-vulkan/src/ep.rs:1-53, 454-493) keeps the
tokens replicated, remaps out-of-band expert ids to weight 0 (`moe_ep_band_remap.comp`) and
all-reduces the per-band partial outputs.  Here each rank owns a slice of the TOKENS as well: it
routes its own rows with the full (replicated) router, sends every row once to each rank that owns
at least one of its experts - together with the row's ids and weights - and gets back that rank's
band-limited partial sum (the op with `ep_band` set, exactly the partial the reference all-reduces).
The home rank adds the partials in rank order and then the shared expert.  Same band partition
`[r*E/W, (r+1)*E/W)` (ep.rs:12-14), same sums up to association; only the data movement differs.

The exchange logic is independent of where the math runs: `ExpertParallel` takes three callables
(route / band partial / finish) so the same code runs with the CUDA library on GPUs and with a
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
    tok: torch.Tensor        # [n_send] token row of every sent row, grouped by destination rank
    send_splits: list        # rows sent to each rank
    recv_splits: list        # rows received from each rank


class ExpertParallel:
    """route_fn(x) -> (ids [R,k] int32, wts [R,k] f32)
    band_fn(x_rows [n, ne], ids [n,k] int32 global ids, wts [n,k]) -> [n, ne]: for every row the
        weighted sum over its pairs whose expert lies in THIS rank's band (others contribute 0)
    finish_fn(moe [R, ne], x [R, ne][, prepared]) -> out [R, ne]   (adds what is replicated: the shared expert)"""

    def __init__(self, n_expert: int, n_used: int, route_fn: Callable, band_fn: Callable, finish_fn: Callable,
                 group: Optional[dist.ProcessGroup] = None, prepare_fn: Optional[Callable] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_expert % self.world:
            raise ValueError(f"n_expert {n_expert} is not a multiple of the world size {self.world}")  # ep.rs:171-176
        self.n_expert, self.n_used, self.e_local = n_expert, n_used, n_expert // self.world
        self.route_fn, self.band_fn, self.finish_fn = route_fn, band_fn, finish_fn
        # optional: work on x that needs no exchange (the shared expert), queued before the plan's
        # host synchronisation so that the device is busy meanwhile; its result goes to finish_fn
        self.prepare_fn = prepare_fn
        self.check_ids = False

    @property
    def band(self):
        return self.rank * self.e_local, self.e_local

    # -- exchange ---------------------------------------------------------------------------------
    def _a2a(self, out, inp, out_splits=None, in_splits=None):
        if self.world == 1:
            out.copy_(inp)
        else:
            dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group)

    def plan(self, ids: torch.Tensor) -> DispatchPlan:
        """Which rows go where (one host synchronisation: the split sizes NCCL needs)."""
        W = self.world
        if self.check_ids and ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= self.n_expert):
            raise ValueError("expert id out of range")  # (costs a host synchronisation: off by default)
        dest = torch.div(ids.to(torch.int64).clamp_(0, self.n_expert - 1), self.e_local, rounding_mode="floor")  # [R, k]
        hit = torch.zeros(ids.shape[0], W, dtype=torch.bool, device=ids.device)
        hit.scatter_(1, dest, True)
        counts = hit.sum(0)                                   # rows for each rank
        recv_counts = torch.empty_like(counts)
        self._a2a(recv_counts, counts)
        # (rank, token) pairs that are hit, rank-major and token-minor, without a second
        # synchronisation: a stable sort brings them to the front, the counts say how many
        order = torch.argsort(~hit.t().reshape(-1), stable=True)
        both = torch.stack([counts, recv_counts]).tolist()    # the synchronisation
        tok = (order[:sum(both[0])] % ids.shape[0]).contiguous()
        return DispatchPlan(tok, both[0], both[1])

    # every rank must take the same branch: the choice depends on sizes all ranks share
    static_limit_bytes = 48 << 20

    def forward_static(self, x: torch.Tensor) -> torch.Tensor:
        """The exchange with fixed shapes, for calls whose rows are few enough to send every row to
        every rank: no counts, no host synchronisation, nothing whose size depends on the routing.
        A rank that owns none of a row's experts sees that row with all ids negative and returns
        zeros for it.  Needs the same number of rows on every rank."""
        W, k = self.world, self.n_used
        R, ne = x.shape
        ids, wts = self.route_fn(x)
        prepared = self.prepare_fn(x) if self.prepare_fn is not None else None
        dest = torch.div(ids.clamp(0, self.n_expert - 1), self.e_local, rounding_mode="floor")                # [R, k]
        ranks = torch.arange(W, device=x.device, dtype=dest.dtype).view(W, 1, 1)
        ids_w = torch.where(dest.unsqueeze(0) == ranks, ids.unsqueeze(0), torch.full_like(ids, -1).unsqueeze(0))  # [W, R, k]
        send_m = torch.cat([ids_w.contiguous().view(torch.float32), wts.unsqueeze(0).expand(W, R, k)], 2).reshape(W * R, 2 * k).contiguous()
        send_x = x.unsqueeze(0).expand(W, R, ne).reshape(W * R, ne).contiguous()  # (a one-row expand reshapes to a stride-0 view)
        recv_x = torch.empty_like(send_x)
        recv_m = torch.empty_like(send_m)
        self._a2a(recv_x, send_x)
        self._a2a(recv_m, send_m)
        part = self.band_fn(recv_x, recv_m[:, :k].contiguous().view(torch.int32), recv_m[:, k:].contiguous())
        if part.shape != recv_x.shape:
            raise RuntimeError(f"band_fn returned {tuple(part.shape)} for rows {tuple(recv_x.shape)}")
        back = torch.empty_like(part)
        self._a2a(back, part)
        moe = back.view(W, R, ne)[0].clone()
        for r in range(1, W):  # rank order
            moe += back.view(W, R, ne)[r]
        return self.finish_fn(moe, x) if self.prepare_fn is None else self.finish_fn(moe, x, prepared)

    def forward(self, x: torch.Tensor, rows_equal: bool = False) -> torch.Tensor:
        """x: this rank's token rows [R, ne] (f32).  Returns the MoE FFN output for those rows.
        `rows_equal`: the caller vouches that every rank passes the same number of rows, which
        allows the fixed-shape exchange when it is small enough."""
        if rows_equal and self.world > 1 and self.world * x.shape[0] * x.shape[1] * 4 <= self.static_limit_bytes:
            return self.forward_static(x)
        ids, wts = self.route_fn(x)
        prepared = self.prepare_fn(x) if self.prepare_fn is not None else None
        pl = self.plan(ids)
        ne, k = x.shape[1], self.n_used
        # dispatch: the row, its ids (bit-cast) and its weights, once per destination rank
        send_x = x[pl.tok]
        send_m = torch.cat([ids[pl.tok].view(torch.float32), wts[pl.tok]], 1)
        n_recv = int(sum(pl.recv_splits))
        recv_x = torch.empty(n_recv, ne, dtype=x.dtype, device=x.device)
        recv_m = torch.empty(n_recv, 2 * k, dtype=torch.float32, device=x.device)
        self._a2a(recv_x, send_x, pl.recv_splits, pl.send_splits)
        self._a2a(recv_m, send_m, pl.recv_splits, pl.send_splits)
        # this rank's band over everything it received
        part = self.band_fn(recv_x, recv_m[:, :k].contiguous().view(torch.int32), recv_m[:, k:].contiguous())
        if part.shape != recv_x.shape:
            raise RuntimeError(f"band_fn returned {tuple(part.shape)} for rows {tuple(recv_x.shape)}")
        # return exchange: the mirror image of the dispatch
        back = torch.empty(send_x.shape[0], ne, dtype=part.dtype, device=x.device)
        self._a2a(back, part, pl.send_splits, pl.recv_splits)
        # partial sums added in rank order (a rank's rows are distinct tokens: no colliding adds)
        moe = torch.zeros_like(x)
        o = 0
        for n in pl.send_splits:
            if n:
                moe.index_add_(0, pl.tok[o:o + n], back[o:o + n])
            o += n
        return self.finish_fn(moe, x) if self.prepare_fn is None else self.finish_fn(moe, x, prepared)


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
        self.has_shared = "sh_gate" in layer.b
        self.ep = ExpertParallel(n_expert, n_used, self._route, self._band, self._finish, prepare_fn=self._shared)
        self._keep = []  # tensors the queued kernels still read; released at the start of the next forward

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

    def _band(self, x_rows, ids, wts):
        """The op restricted to this rank's experts: routing is an input (stages 2 + 4 + 8), ids
        are rebased to the local banks and pairs of other ranks marked negative."""
        be, b = self.be, self.L.b
        n = x_rows.shape[0]
        out = torch.empty_like(x_rows)
        if not n:
            return out
        lo, n_local = self.ep.band
        local = ids - lo
        local = torch.where((local >= 0) & (local < n_local), local, torch.full_like(local, -1)).contiguous()
        wts = wts.contiguous()
        be.moe_ffn(self._MoeFfn(x=be.wrap_tensor(x_rows), router=b["router"], gate_exps=b["gate"], up_exps=b["up"], down_exps=b["down"],
                                dst=be.wrap_tensor(out), rows=n, ne=self.ne, n_expert=n_local, n_used=self.n_used, n_ff_exp=self.n_ff,
                                ids_out=be.wrap_tensor(local), wts_out=be.wrap_tensor(wts), stages=14))
        self._keep += [x_rows, local, wts, out]
        return out

    def _shared(self, x):
        """Queues the replicated shared expert over this rank's own tokens: (rows, gate logits)."""
        if not self.has_shared:
            return None
        be, b = self.be, self.L.b
        R = x.shape[0]
        sh = torch.empty_like(x)
        seg = torch.tensor([0, R], dtype=torch.int32, device=x.device)
        xb = be.wrap_tensor(x)
        be.moe_expert_rows(xb, be.wrap_tensor(seg), b["sh_gate"], b["sh_up"], b["sh_down"], be.wrap_tensor(sh), R, 1, self.ne, self.n_ff)
        gl = None
        if "sh_gate_inp" in b:
            gl = torch.empty(R, dtype=torch.float32, device=x.device)
            be.linear(self._DType.F32, b["sh_gate_inp"], xb, be.wrap_tensor(gl), R, self.ne, 1)
        self._keep += [sh, seg, gl]
        return sh, gl

    def _finish(self, moe, x, prepared):
        if prepared is None:
            return moe
        be = self.be
        sh, gl = prepared
        R = x.shape[0]
        out = torch.empty_like(x)
        if gl is not None:
            be.moe_shared_expert_add(be.wrap_tensor(moe), be.wrap_tensor(sh), be.wrap_tensor(gl), be.wrap_tensor(out), R, self.ne)
        else:
            be.add(be.wrap_tensor(moe), be.wrap_tensor(sh), be.wrap_tensor(out), R * self.ne)
        self._keep += [moe, out]
        return out

    def forward(self, x: torch.Tensor, rows_equal: bool = False) -> torch.Tensor:
        # tensors of the previous call are released here: the caching allocator hands their
        # memory out again in stream order, and everything runs on one stream
        keep, self._keep = self._keep, []
        out = self.ep.forward(x, rows_equal=rows_equal)
        del keep
        return out


# -------------------------------------------------------------------------------------------------
# Expert parallelism inside the library (infr_cuda_ep_init + the collective form of infr_cuda_moe_ffn)
# -------------------------------------------------------------------------------------------------

def join_communicator(be, group: Optional[dist.ProcessGroup] = None) -> None:
    """Brings the backend's context into an NCCL communicator of its own, spanning the ranks of the
    (already initialised) torch process group: rank 0 makes the id, the group carries it to the others
    (the role `ncclGetUniqueId` + an out-of-band channel plays for a host without torch)."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    box = [be.ep_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0, group=group)
    be.ep_init(box[0], rank, world)


class LibraryExpertParallelLayer:
    """One MoE layer sharded over the ranks, every step of it inside the C-ABI library: the call
    below is `Backend::execute` of an `Op::MoeFfn` whose `ep_band` is this rank's band, on a context
    that has joined a communicator (`ExpertParallelBackend`, crates/infr-vulkan/src/ep.rs:454-493).

    `layer` holds the full router and shared expert and the banks of THIS rank's experts only
    (devgen.DeviceLayer(..., band=(rank * E / W, E / W)))."""

    def __init__(self, be, layer, n_expert: int, n_used: int, n_ff: int, ne: int, sh_ff: int = 0, **route_kw):
        from .backend import MoeFfn
        self.be, self.L, self._MoeFfn = be, layer, MoeFfn
        world, rank = getattr(be, "ep_world", 1), getattr(be, "ep_rank", 0)
        if n_expert % world:
            raise ValueError(f"n_expert {n_expert} is not a multiple of the world size {world}")  # ep.rs:171-176
        self.band = (rank * (n_expert // world), n_expert // world)
        self.dims = dict(ne=ne, n_expert=n_expert, n_used=n_used, n_ff_exp=n_ff)
        self.sh_ff = sh_ff if "sh_gate" in layer.b else 0
        # formats of the banks (devgen.DeviceLayer.dtypes; Q4_K / Q4_K / Q6_K when the layer does not say)
        from .backend import DType
        gd, ud, dd = getattr(layer, "dtypes", (12, 12, 14))
        self.route_kw = dict(route_kw, gate_dtype=DType(gd), up_dtype=DType(ud), down_dtype=DType(dd))

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, ids_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: this rank's token rows [R, ne] f32 (the same R on every rank).  Collective."""
        be, b = self.be, self.L.b
        out = torch.empty_like(x) if out is None else out
        op = self._MoeFfn(x=be.wrap_tensor(x), dst=be.wrap_tensor(out), rows=x.shape[0], router=b["router"], gate_exps=b["gate"],
                          up_exps=b["up"], down_exps=b["down"], exp_probs_b=b.get("bias"), ep_band=self.band,
                          ids_out=be.wrap_tensor(ids_out) if ids_out is not None else None,
                          sh_gate=b.get("sh_gate") if self.sh_ff else None, sh_up=b.get("sh_up") if self.sh_ff else None,
                          sh_down=b.get("sh_down") if self.sh_ff else None,
                          sh_gate_inp=b.get("sh_gate_inp") if self.sh_ff else None, sh_ff=self.sh_ff, **self.dims, **self.route_kw)
        be.moe_ffn(op)
        return out
