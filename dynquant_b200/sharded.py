"""Multi-GPU placement of the paths that shard: column-sharded (and input-sharded) dense GEMV
and expert-parallel MoE.  One process per GPU, ``torch.distributed`` for the exchange (NCCL on
GPUs; the same code runs over gloo on CPU in the tests, with the oracle as the compute).

The reference issues no collective itself -- tensor parallelism there is weight placement
only (``integration/vllm_plugin/parameter.py:102-154``) and the gathers are the host
framework's.  Placement rules kept from it: a column shard is a contiguous slab of rows of
``packed`` / ``scales`` / ``offsets`` (rows are independent under group-wise packing,
``docs/format-spec.md:355-358``); experts are contiguous row slabs of a bank.

The dense step exchanges over peer memory with the library's own kernels by default
(``dynquant_b200/peer.py``); NCCL is the checked alternative and the expert layer's default.
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


def input_shard(qt: QuantTensor, rank: int, world: int) -> QuantTensor:
    """The slice ``[rank*K/world, (rank+1)*K/world)`` of the INPUT axis of a packed tensor.

    Legal only on group boundaries (reference ``row_parallel_split``,
    ``integration/serving_common/geometry.py:481-551``): a group's words, scale and offset move
    together, so the groups must divide evenly over the ranks and ``in_features`` must be a
    whole number of groups; per-row tensors (one group spanning the row) are refused as there
    (``:513-520``).  The result is a copy: its rows are shorter, so no view of the parent can
    have the parent's layout.
    """
    from dataclasses import replace

    if qt.is_per_row:
        raise ValueError("a per-row-grouped tensor has one group per row and cannot be split along its input axis")
    g = qt.geometry
    if g.num_groups % world or qt.in_features != g.num_groups * qt.group_size:
        raise ValueError(
            f"{g.num_groups} groups of {qt.group_size} over in_features={qt.in_features} do not split on group "
            f"boundaries over {world} ranks"
        )
    per = g.num_groups // world
    words = slice(rank * per * g.words_per_group, (rank + 1) * per * g.words_per_group)
    groups = slice(rank * per, (rank + 1) * per)
    k = per * qt.group_size
    return replace(
        qt,
        packed=qt.packed[:, words].contiguous(),
        scales=qt.scales[:, groups].contiguous(),
        offsets=None if qt.offsets is None else qt.offsets[:, groups].contiguous(),
        in_features=k,
        logical_shape=(qt.num_rows, k),
    )


class InputShardedLinear:
    """``y = x @ W.T`` with ``W``'s input axis split over the ranks (the o_proj / down_proj
    placement of tensor parallelism): every rank holds ``x[:, its slice]``, computes fp32
    partial sums over its slice and the partials are all-reduced.  The sum over ranks is in
    NCCL's order, so unlike the column-sharded layer the result may differ from the
    single-device one in the last fp32 bit."""

    def __init__(self, local: QuantTensor, *, bias: torch.Tensor | None = None, group=None,
                 compute: Callable | None = None) -> None:
        self.local = local
        self.bias = bias
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if compute is None:
            from . import ops

            def compute(x, qt):
                if x.shape[0] > ops.gemv_max_rows():
                    return ops.gemv_row_chunks(x.contiguous(), [qt], out_dtype=torch.float32)
                return ops.gemv_shards(x.contiguous(), [qt], out_dtype=torch.float32)

        self.compute = compute

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        partial = self.compute(x_local, self.local).to(torch.float32).contiguous()  # [M, N], this rank's slice of K
        dist.all_reduce(partial, group=self.group)
        if self.bias is not None:
            partial = partial + self.bias.to(torch.float32)
        return partial.to(x_local.dtype)

    __call__ = forward


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
    * ``mode="peer"``: the replicated scheme with the library's own exchanges over peer memory
      (``peer=`` a :class:`~dynquant_b200.peer.PeerExchange`): one all-gather launch for token rows,
      ids and weights together, the grouped kernels, one reduce-scatter that adds the source ranks in rank
      order -- kernel launches only, so a whole layer can sit in a CUDA graph.

    All produce the same numbers up to the order of the final fp32 sum over ranks.
    """

    def __init__(self, gate_up_local: QuantTensor, down_local: QuantTensor, *, num_experts: int,
                 group=None, compute: Callable | None = None, max_tokens: int = 64, peer=None) -> None:
        self.group = group
        self.peer = peer
        self._takes_global_ids = False
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

            def compute(x, ids, w, gate_up, down, num_experts, first_expert=0):
                return ops.moe_gemv(x, ids, w, gate_up, down, num_experts=num_experts, out_dtype=torch.float32,
                                    first_expert=first_expert)

            self._takes_global_ids = True  # the kernels renumber the ids themselves
        self.compute = compute
        self.max_tokens = max_tokens

    def _localise(self, ids: torch.Tensor) -> torch.Tensor:
        """Global expert ids -> this rank's local numbering.  Experts held elsewhere come out
        negative or >= ``local_experts``, which the grouped kernels skip: one elementwise op."""
        return (ids - self.rank * self.local_experts).to(torch.int32)

    def _local_partial(self, x: torch.Tensor, ids: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Partial sums of this rank's experts for every gathered token, at most ``max_tokens`` tokens
        per call of the grouped kernel (the gathered batch is ``world`` times a rank's own)."""
        limit = self.max_tokens
        if self._takes_global_ids:  # no renumbering pass: the kernels subtract the first local expert
            local, extra = ids.to(torch.int32), {"first_expert": self.rank * self.local_experts}
        else:
            local, extra = self._localise(ids), {}
        if x.shape[0] <= limit:
            return self.compute(x.contiguous(), local.contiguous(), w.contiguous(), self.gate_up, self.down,
                                self.local_experts, **extra)
        parts = [self.compute(x[s : s + limit].contiguous(), local[s : s + limit].contiguous(),
                              w[s : s + limit].contiguous(), self.gate_up, self.down, self.local_experts, **extra)
                 for s in range(0, x.shape[0], limit)]
        return torch.cat(parts)

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
        if mode == "peer":
            if self.peer is None:
                raise ValueError('mode="peer" needs the layer to be built with peer=PeerExchange(...)')
            xs = torch.empty(world * t, h, dtype=x.dtype, device=x.device)
            ids = torch.empty(world * t, k, dtype=topk_ids.dtype, device=x.device)
            ws = torch.empty(world * t, k, dtype=topk_w.dtype, device=x.device)
            pieces = [x.contiguous(), topk_ids.contiguous(), topk_w.contiguous()]
            if all((p.numel() * p.element_size()) % 16 == 0 for p in pieces):
                self.peer.all_gather_parts(pieces, [xs, ids, ws])  # one launch for the three
            else:
                for p, o in zip(pieces, (xs, ids, ws)):
                    self.peer.all_gather(p, o)
            partial = self._local_partial(xs, ids, ws).to(torch.float32).contiguous()  # [world*t, h]
            out = torch.empty(t, h, dtype=x.dtype, device=x.device)
            self.peer.reduce_scatter(partial.view(-1), out)
            return out
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
    """One decode step of a :class:`~dynquant_b200.workloads.LinearStack` on ``world`` GPUs.

    Large modules -- those whose per-rank slab of packed rows is still at least
    ``shard_min_bytes`` -- are column-sharded (row slabs); everything smaller is computed by
    every rank, because exchanging costs more than the whole small GEMV.  A stage (q/k/v,
    gate/up, or a single module) whose modules are all sharded writes its ``[M, rows/world]``
    outputs into one buffer, and that buffer is all-gathered right after the stage:

    * ``exchange="fused"`` (default): the stage's GEMV launch itself stores its output rows into
      every rank's window and ends with a bounded wait for the other ranks' rows
      (``dq_gemv_stage_push``, :class:`~dynquant_b200.peer.PushWindow`): no exchange launch at
      all.  A stage the pushing kernels do not take falls back to ``"peer"`` for that stage;
    * ``exchange="peer"``: the library's own exchange kernels over peer memory
      (:class:`~dynquant_b200.peer.PeerExchange`), enqueued between the stages and captured in
      the step's CUDA graph -- a step is one graph replay, exchanges included;
    * ``exchange="nccl"``: one ``all_gather_into_tensor`` per sharded stage, issued eagerly after
      the graph of local kernels (the checked fallback; NCCL calls are kept out of the capture).
    """

    def __init__(self, stack, m: int, *, rank: int, world: int, device, act_dtype=torch.bfloat16,
                 shard_min_bytes: int = 32 << 20, graph_mode: str | None = "dataflow", exchange: str = "fused",
                 presharded: bool = False) -> None:
        """``presharded``: ``stack`` already holds this rank's row slabs of every module (a set
        too large to generate whole on every rank); every module then counts as sharded."""
        from .stack import StepRunner
        from .workloads import LinearStack, Module

        if exchange not in ("fused", "peer", "nccl"):
            raise ValueError(exchange)
        self.rank, self.world, self.device = rank, world, torch.device(device)
        modules, self.sharded = [], []
        for mod in stack.modules:
            qt = mod.weight
            if presharded:
                modules.append(mod)
                self.sharded.append(mod.name)
            elif world > 1 and qt.num_rows % world == 0 and qt.nbytes // world >= shard_min_bytes:
                modules.append(Module(mod.name, column_shard(qt, rank, world), mod.input))
                self.sharded.append(mod.name)
            else:
                modules.append(mod)
        self.local_stack = LinearStack(stack.name + f"[{rank}/{world}]", stack.hidden, stack.intermediate, modules,
                                       stack.bit_map)
        self.runner = StepRunner(self.local_stack, m, act_dtype=act_dtype, device=self.device, stage_outputs=True)
        self.inputs = self.runner.inputs
        self.outputs = dict(self.runner.outputs)
        # stages whose modules are all sharded exchange their (one) output buffer
        sharded = set(self.sharded)
        self._gathers = {}  # stage index -> (piece [m, cols], full [world, m, cols])
        self._columns = {}  # module name -> (stage index, first column, rows) inside its stage's buffer
        for index, stage in enumerate(self.local_stack.stages()):
            names = [self.local_stack.modules[i].name for i in stage]
            hit = [n in sharded for n in names]
            if any(hit) and not all(hit):
                raise ValueError(f"stage {names} mixes sharded and replicated modules")
            if world > 1 and all(hit):
                piece = self.runner.stage_buffers[index]
                self._gathers[index] = (piece, torch.empty(world, *piece.shape, dtype=piece.dtype, device=self.device))
                col = 0
                for i in stage:
                    rows = self.local_stack.modules[i].weight.num_rows
                    self._columns[self.local_stack.modules[i].name] = (index, col, rows)
                    col += rows
        for name, (index, col, rows) in self._columns.items():
            self.outputs[name] = self._gathers[index][1][:, :, col:col + rows]  # [world, m, rows/world]
        self.gathers_per_step = len(self._gathers)
        self.exchange = exchange if self._gathers else "none"
        self._peer = None
        self._window = None
        self._slot = {}       # stage index -> exchange of the push window
        self._unfused = set()  # stages the pushing kernels refused: exchanged by the peer kernels instead
        if self.exchange in ("peer", "fused"):
            from .peer import PeerExchange

            biggest = max(p.numel() * p.element_size() for p, _ in self._gathers.values())
            self._peer = PeerExchange(-(-biggest // 16) * 16, device=self.device)
        if self.exchange == "fused":
            from .peer import PushWindow

            order = sorted(self._gathers)
            self._slot = {index: k for k, index in enumerate(order)}
            self._window = PushWindow([self._gathers[i][0].numel() * self._gathers[i][0].element_size() for i in order],
                                      device=self.device)
        self.graph_mode = graph_mode
        in_graph = self.exchange in ("peer", "fused") and graph_mode == "dataflow"
        if graph_mode is not None:
            self.runner.capture(graph_mode, after_stage=self._exchange_stage if in_graph else None,
                                launch_stage=self._launch_stage if in_graph and self._window is not None else None)
        else:
            self.runner.count_launches()
        self._exchanges_in_graph = in_graph
        self.launches_per_step = self.runner.launches_per_step
        self.fused_stages = len(self._slot) - len(self._unfused)
        # what the windows hold now (the capture's own warm-up ran no exchange; an eager pass may have)
        self._runs = 0
        self._base_epoch = 0
        if self._window is not None and self.fused_stages:
            first = next(i for i in sorted(self._slot) if i not in self._unfused)
            self._base_epoch = self._window.epoch(self._slot[first])

    def _launch_stage(self, index: int, first: int, count: int) -> bool:
        slot = self._slot.get(index)
        if slot is None or index in self._unfused:
            return False
        if self._window.run_stage(slot, self.runner.jobs_at(first), count):
            return True
        self._unfused.add(index)
        return False

    def _exchange_stage(self, index: int) -> None:
        pair = self._gathers.get(index)
        if pair is None:
            return
        piece, full = pair
        if self._peer is not None:
            self._peer.all_gather(piece, full)
        else:
            dist.all_gather_into_tensor(full, piece)

    def run(self) -> None:
        if self.graph_mode is not None:
            self.runner.replay()
        elif self._window is not None:
            self.runner.run_dataflow(None, self._exchange_stage, self._launch_stage)
        else:
            self.runner.run()
        self._runs += 1
        if not self._exchanges_in_graph and self._window is None:
            for index in self._gathers:
                self._exchange_stage(index)

    def check(self) -> None:
        """Raises if an exchange's bounded wait ran out (exchanges over peer memory only)."""
        if self._peer is not None:
            self._peer.check()
        if self._window is not None:
            self._window.check()

    def full_output(self, name: str) -> torch.Tensor:
        """``[world, m, rows/world]``: every rank's piece of a sharded module's output after the
        last :meth:`run`.  For a stage exchanged by its own launch this is a view into the window
        half the last step wrote (it alternates from step to step)."""
        index, col, rows = self._columns[name]
        if self._window is None or index not in self._slot or index in self._unfused:
            return self.outputs[name]
        piece = self._gathers[index][0]  # this rank's [m, columns] stage buffer: shape and dtype of a piece
        raw = self._window.piece(self._slot[index], self._base_epoch + self._runs)
        nbytes = piece.numel() * piece.element_size()
        return raw[:, :nbytes].view(piece.dtype).view(self.world, *piece.shape)[:, :, col:col + rows]

    def gathered(self, name: str) -> torch.Tensor:
        """The full ``[m, N]`` output of a sharded module, reassembled from the rank-major pieces."""
        full = self.full_output(name)  # [world, m, rows/world]
        return full.permute(1, 0, 2).reshape(full.shape[1], -1)
