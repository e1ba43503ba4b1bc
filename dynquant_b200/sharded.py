"""Multi-GPU placement of the two paths that shard: column-sharded dense GEMV and
expert-parallel MoE.  One process per GPU, ``torch.distributed`` for the exchange (NCCL on
GPUs; the same code runs over gloo on CPU in the tests, with the oracle as the compute).

The reference issues no collective itself -- tensor parallelism there is weight placement
only (``integration/vllm_plugin/parameter.py:102-154``) and the gathers are the host
framework's.  Placement rules kept from it: a column shard is a contiguous slab of rows of
``packed`` / ``scales`` / ``offsets`` (rows are independent under group-wise packing,
``docs/format-spec.md:355-358``); experts are contiguous row slabs of a bank.

No kernel here touches a peer's memory; every exchange is a library collective.
"""

from __future__ import annotations

import ctypes
from typing import Callable

import torch
import torch.distributed as dist

from .format import QuantTensor


def column_shard(qt: QuantTensor, rank: int, world: int) -> QuantTensor:
    """Rows ``[rank*N/world, (rank+1)*N/world)`` of a packed tensor (a view)."""
    if qt.num_rows % world:
        raise ValueError(f"{qt.num_rows} rows do not split evenly over {world} ranks")
    per = qt.num_rows // world
    return qt.rows(rank * per, (rank + 1) * per)


def expert_shard(bank: QuantTensor, rows_per_expert: int, num_experts: int, rank: int, world: int) -> QuantTensor:
    """The contiguous experts ``[rank*E/world, (rank+1)*E/world)`` of a bank folded to rows."""
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not split evenly over {world} ranks")
    per = num_experts // world
    return bank.rows(rank * per * rows_per_expert, (rank + 1) * per * rows_per_expert)


class ColumnShardedLinear:
    """``y = x @ W.T`` with ``W``'s rows split over the ranks; ``forward`` returns the full ``y``
    on every rank after an all-gather of the ``[M, N/world]`` pieces."""

    def __init__(self, local: QuantTensor, *, group=None, compute: Callable | None = None) -> None:
        self.local = local
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if compute is None:
            from . import ops

            compute = ops.quantized_matmul
        self.compute = compute

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        piece = self.compute(x, self.local).contiguous()  # [M, N/world]
        m, n_local = piece.shape
        gathered = torch.empty(self.world * m, n_local, dtype=piece.dtype, device=piece.device)
        dist.all_gather_into_tensor(gathered, piece, group=self.group)
        return gathered.view(self.world, m, n_local).permute(1, 0, 2).reshape(m, self.world * n_local)

    __call__ = forward


class ExpertParallelMoE:
    """Expert layer with the experts placed over the ranks (``E/world`` contiguous experts each).

    Every rank owns ``tokens_local`` tokens.  ``forward`` dispatches each token to the ranks
    that own its experts and combines the partial results at the token's home rank:

    * ``mode="all_to_all"`` (default): dispatch all-to-all (token rows + routing), local
      grouped GEMV over the received tokens with foreign experts masked, combine all-to-all,
      sum over source ranks in rank order.  Fixed capacity -- every rank sends its
      ``tokens_local`` rows to every rank -- so no size has to travel to the host first.
    * ``mode="replicated"``: all-gather tokens and routing, local partial sums for all tokens,
      reduce-scatter back.  Fewer messages; same bytes.

    Both produce the same numbers up to the order of the final fp32 sum over ranks.
    """

    def __init__(self, gate_up_local: QuantTensor, down_local: QuantTensor, *, num_experts: int,
                 group=None, compute: Callable | None = None) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not split evenly over {self.world} ranks")
        self.num_experts = num_experts
        self.local_experts = num_experts // self.world
        self.gate_up = gate_up_local
        self.down = down_local
        if compute is None:
            from . import ops

            def compute(x, ids, w, gate_up, down, num_experts):
                return ops.moe_gemv(x, ids, w, gate_up, down, num_experts=num_experts, out_dtype=torch.float32)

        self.compute = compute

    def _localise(self, ids: torch.Tensor) -> torch.Tensor:
        """Global expert ids -> this rank's local numbering, -1 for experts held elsewhere."""
        lo = self.rank * self.local_experts
        local = ids - lo
        return torch.where((local >= 0) & (local < self.local_experts), local, torch.full_like(ids, -1)).to(torch.int32)

    def _local_partial(self, x: torch.Tensor, ids: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return self.compute(x.contiguous(), self._localise(ids).contiguous(), w.contiguous(), self.gate_up,
                            self.down, self.local_experts)

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor, mode: str = "all_to_all") -> torch.Tensor:
        t, h = x.shape
        k = topk_ids.shape[1]
        world = self.world
        if mode == "replicated":
            xs = torch.empty(world * t, h, dtype=x.dtype, device=x.device)
            ids = torch.empty(world * t, k, dtype=topk_ids.dtype, device=x.device)
            ws = torch.empty(world * t, k, dtype=topk_w.dtype, device=x.device)
            dist.all_gather_into_tensor(xs, x.contiguous(), group=self.group)
            dist.all_gather_into_tensor(ids, topk_ids.contiguous(), group=self.group)
            dist.all_gather_into_tensor(ws, topk_w.contiguous(), group=self.group)
            partial = self._local_partial(xs, ids, ws).to(torch.float32)  # [world*t, h]
            if dist.get_backend(self.group) == "gloo":  # no reduce-scatter there: reduce, keep own rows
                dist.all_reduce(partial, group=self.group)
                out = partial[self.rank * t : (self.rank + 1) * t]
            else:
                out = torch.empty(t, h, dtype=torch.float32, device=x.device)
                dist.reduce_scatter_tensor(out, partial.contiguous(), group=self.group)
            return out.to(x.dtype)
        if mode != "all_to_all":
            raise ValueError(mode)
        # dispatch: rank r receives [world, t, ...] = every rank's tokens and routing
        send_x = x.contiguous().unsqueeze(0).expand(world, t, h).contiguous()
        recv_x = torch.empty_like(send_x)
        dist.all_to_all_single(recv_x, send_x, group=self.group)
        send_r = torch.cat([topk_ids.to(torch.float32), topk_w.to(torch.float32)], dim=1)
        send_r = send_r.unsqueeze(0).expand(world, t, 2 * k).contiguous()
        recv_r = torch.empty_like(send_r)
        dist.all_to_all_single(recv_r, send_r, group=self.group)
        ids = recv_r[..., :k].reshape(world * t, k).to(topk_ids.dtype)
        ws = recv_r[..., k:].reshape(world * t, k).contiguous()
        partial = self._local_partial(recv_x.reshape(world * t, h), ids, ws).to(torch.float32)
        # combine: send each source rank its tokens' partial sums, add them up at home in rank order
        back = torch.empty(world, t, h, dtype=torch.float32, device=x.device)
        dist.all_to_all_single(back, partial.reshape(world, t, h).contiguous(), group=self.group)
        out = back[0].clone()
        for r in range(1, world):
            out += back[r]
        return out.to(x.dtype)

    __call__ = forward


class ShardedStepRunner:
    """One decode step of a :class:`~dynquant_b200.workloads.LinearStack` with every module
    column-sharded: local GEMVs from one ``dq_gemv_sequence`` call per stage, then one
    all-gather per stage whose outputs the next stage consumes (o_proj, gate/up, down_proj and
    the lm_head; q/k/v feed attention head-locally and are not gathered)."""

    def __init__(self, stack, m: int, *, rank: int, world: int, device, act_dtype=torch.bfloat16) -> None:
        from . import _lib
        from .ops import _tag, weight_descriptor

        self._lib = _lib
        self.stack, self.m, self.rank, self.world, self.device = stack, m, rank, world, torch.device(device)
        self.local = [column_shard(mod.weight, rank, world) for mod in stack.modules]
        widths = {}
        for mod in stack.modules:
            widths.setdefault(mod.input, mod.weight.in_features)
        gen = torch.Generator(device=self.device).manual_seed(1234)
        self.inputs = {n: torch.randn(m, k, device=self.device, generator=gen).to(act_dtype) for n, k in widths.items()}
        self.pieces = [torch.empty(m, qt.num_rows, dtype=act_dtype, device=self.device) for qt in self.local]
        self.outputs = {mod.name: torch.empty(world * m, qt.num_rows, dtype=act_dtype, device=self.device)
                        for mod, qt in zip(stack.modules, self.local)}
        self._jobs = (_lib.GemvJob * len(self.local))()
        for i, (mod, qt) in enumerate(zip(stack.modules, self.local)):
            job = self._jobs[i]
            job.x = self.inputs[mod.input].data_ptr()
            job.out = self.pieces[i].data_ptr()
            job.bias = None
            job.m, job.out_stride, job.out_col0 = m, qt.num_rows, 0
            job.x_dtype = job.out_dtype = _tag(act_dtype, "x")
            job.weight = weight_descriptor("gemv_sequence", qt.packed, qt.scales, qt.offsets, qt.bits,
                                           qt.geometry.effective_group, qt.in_features)
        self.stages = stack.stages()
        self.launches_per_step = len(self.local)
        self.gathers_per_step = sum(1 for st in self.stages if self._gathered(st))

    def _gathered(self, stage: list[int]) -> bool:
        leaf = self.stack.modules[stage[0]].name.rsplit(".", 1)[-1]
        return leaf not in ("q_proj", "k_proj", "v_proj")

    def run(self) -> None:
        lib = self._lib.load()
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        size = ctypes.sizeof(self._lib.GemvJob)
        for stage in self.stages:
            jobs = ctypes.cast(ctypes.byref(self._jobs, stage[0] * size), ctypes.POINTER(self._lib.GemvJob))
            self._lib.check(lib.dq_gemv_sequence(jobs, len(stage), stream))
            if self._gathered(stage):
                for idx in stage:
                    dist.all_gather_into_tensor(self.outputs[self.stack.modules[idx].name], self.pieces[idx])
