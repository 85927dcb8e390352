"""A stack of MoE FFN sub-layers as the graph builder emits them for a decode step
(crates/infr-llama/src/seam/runner.rs:7999-8176; layer shape pinned in
crates/infr-core/src/fusion.rs:735-737), attention omitted:

    hn     = RmsNorm(hidden, w_l, eps)
    sub    = MoeFfn(hn) (+ shared expert)
    hidden = Add(hidden, sub)

Every op goes through the C ABI; the whole step can be recorded once and replayed
(`Backend::compile` + decode replay)."""
from __future__ import annotations

from typing import List, Optional

import torch

from .backend import CudaBackend, MoeFfn


class MoeStack:
    def __init__(self, be: CudaBackend, layers: List, norm_weights: List[torch.Tensor], rows: int, ne: int, n_expert: int,
                 n_used: int, n_ff: int, sh_ff: int = 0, eps: float = 1e-6, fused: bool = True, **route_kw):
        """fused: fold RmsNorm and the residual Add into the MoE op (the reference's
        RmsNorm->MoeFfn and MoeFfn->Add peepholes, crates/infr-core/src/fusion.rs:17-25) instead of
        running them as kernels of their own."""
        assert len(layers) == len(norm_weights)
        self.be, self.layers, self.rows, self.ne, self.eps = be, layers, rows, ne, eps
        dev = norm_weights[0].device
        self.hidden = torch.zeros(rows, ne, device=dev)
        self.hn = torch.zeros(rows, ne, device=dev)
        self.sub = torch.zeros(rows, ne, device=dev)
        self.ids = torch.zeros(len(layers), rows, n_used, dtype=torch.int32, device=dev)
        self._nw = norm_weights
        self.b_hidden, self.b_hn, self.b_sub = be.wrap_tensor(self.hidden), be.wrap_tensor(self.hn), be.wrap_tensor(self.sub)
        self.b_nw = [be.wrap_tensor(w) for w in norm_weights]
        self.fused = fused
        self.ops = []
        for li, L in enumerate(layers):
            b = L.b
            fuse = dict(x=self.b_hidden, dst=self.b_hidden, norm_weight=self.b_nw[li], norm_eps=eps, residual=self.b_hidden) \
                if fused else dict(x=self.b_hn, dst=self.b_sub)
            self.ops.append(MoeFfn(router=b["router"], gate_exps=b["gate"], up_exps=b["up"], down_exps=b["down"],
                                   rows=rows, ne=ne, n_expert=n_expert, n_used=n_used, n_ff_exp=n_ff,
                                   ids_out=be.wrap_tensor(self.ids[li]), sh_gate=b.get("sh_gate"), sh_up=b.get("sh_up"),
                                   sh_down=b.get("sh_down"), sh_gate_inp=b.get("sh_gate_inp"),
                                   sh_ff=sh_ff if "sh_gate" in b else 0, **fuse, **route_kw))
        self.plan = None

    def layer(self, li: int) -> None:
        """One sub-layer in place on `hidden`."""
        be = self.be
        if self.fused:
            be.moe_ffn(self.ops[li])
            return
        be.rms_norm(self.b_hidden, self.b_nw[li], self.b_hn, self.rows, self.ne, self.eps)
        be.moe_ffn(self.ops[li])
        be.add(self.b_hidden, self.b_sub, self.b_hidden, self.rows * self.ne)

    def step(self) -> None:
        for li in range(len(self.layers)):
            self.layer(li)

    def record(self) -> None:
        self.step()  # scratch sized, kernels loaded
        self.be.sync()
        self.be.graph_begin()
        self.step()
        self.plan = self.be.graph_end()

    def replay(self) -> None:
        self.be.execute(self.plan)
