"""Run every packed linear module of a decode step from one host call.

The reference runtime issues one Python ``quantized_matmul`` per module per
step (``packages/dynquant-core/src/dynquant/runtime/linear.py:211-212`` ->
``runtime/ops.py:184-231``) and measures 20-45 us of host time per module
around single-digit-microsecond kernels.  ``StepRunner`` keeps the same
per-module semantics -- module ``i`` computes ``x_i @ W_i.T`` into its own
output buffer, in stream order -- but builds the launch list once and replays
it with a single ``dq_gemv_sequence`` call, optionally from a captured CUDA
graph.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from .ops import _stream, _tag, weight_descriptor
from .workloads import LinearStack


class GemvPlan:
    """A job list compiled into ONE persistent kernel (``dq_plan_*`` of the C ABI).

    Same results as ``dq_gemv_sequence`` over the same ``dq_gemv_job`` array; the jobs' tensors
    are referenced, not copied, and must outlive the plan.  ``launch()`` enqueues
    ``info()["launches"]`` kernels on torch's current stream (one persistent kernel per run of
    stages, plus one streaming GEMV per very long matrix) and may be captured in a CUDA graph; ``check()``
    synchronises and raises if a stage's bounded wait ran out.
    """

    def __init__(self, jobs, count: int, device: torch.device):
        lib = _lib.load()
        self.device = torch.device(device)
        need = ctypes.c_int64()
        _lib.check(lib.dq_plan_workspace_bytes(count, ctypes.byref(need)))
        self.workspace = torch.zeros(need.value, dtype=torch.uint8, device=self.device)
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(lib.dq_plan_create(jobs, count, self.workspace.data_ptr(), need.value,
                                          _stream(self.device), ctypes.byref(handle)))
        self._handle = handle
        self._jobs = jobs  # keeps the ctypes array (and through the runner, the tensors) alive

    def launch(self) -> None:
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().dq_plan_launch(self._handle, _stream(self.device)))

    def check(self) -> None:
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().dq_plan_status(self._handle, _stream(self.device)))

    def info(self) -> dict:
        out = _lib.PlanInfo()
        _lib.check(_lib.load().dq_plan_describe(self._handle, ctypes.byref(out)))
        return {name: int(getattr(out, name)) for name, _ in out._fields_}

    def stage_shape(self, stage: int) -> dict:
        kw, cs = ctypes.c_int32(), ctypes.c_int32()
        ctas = (ctypes.c_int32 * 4)()
        _lib.check(_lib.load().dq_plan_stage_shape(self._handle, stage, ctypes.byref(kw), ctypes.byref(cs), ctas))
        return {"k_slices": kw.value, "slot_steps": cs.value, "ctas": [int(c) for c in ctas if c]}

    def set_wait(self, stage: int, wait_target: int, spin_limit: int) -> None:
        """Failure-handling hook (``dq_plan_set_wait``): make a stage wait for a count."""
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().dq_plan_set_wait(self._handle, stage, wait_target, spin_limit, _stream(self.device)))

    def close(self) -> None:
        if self._handle:
            _lib.load().dq_plan_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):  # pragma: no cover - interpreter teardown order
        try:
            self.close()
        except Exception:
            pass


class StepRunner:
    """Pre-built launch list for one decode step over a :class:`LinearStack`.

    ``inputs`` maps an activation name (``"hidden"``, ``"attn"``, ``"inter"``)
    to a resident ``[m, K]`` tensor; every module writes ``outputs[name]``.
    """

    def __init__(self, stack: LinearStack, m: int, *, act_dtype=torch.bfloat16, out_dtype=None, device="cuda",
                 stage_outputs: bool = False):
        """``stage_outputs``: the modules of a stage (q/k/v, gate/up) write side by side into ONE
        ``[m, sum of their rows]`` buffer (``stage_buffers[i]``), so that a sharded runner can
        exchange a stage's output with one call; ``outputs[name]`` is then a column slice of it."""
        self.stack = stack
        self.m = m
        self.device = torch.device(device)
        out_dtype = out_dtype or act_dtype
        widths = {}
        for mod in stack.modules:
            widths.setdefault(mod.input, mod.weight.in_features)
            if widths[mod.input] != mod.weight.in_features:
                raise ValueError(f"{mod.name}: activation {mod.input!r} has two widths")
        gen = torch.Generator(device=self.device).manual_seed(1234)
        self.inputs = {
            name: torch.randn(m, k, device=self.device, generator=gen).to(act_dtype) for name, k in widths.items()
        }
        placement = {}  # module index -> (buffer, row stride, first column)
        self.stage_buffers: list[torch.Tensor] = []
        if stage_outputs:
            for stage in stack.stages():
                total = sum(stack.modules[i].weight.num_rows for i in stage)
                buf = torch.empty(m, total, dtype=out_dtype, device=self.device)
                self.stage_buffers.append(buf)
                col = 0
                for i in stage:
                    placement[i] = (buf, total, col)
                    col += stack.modules[i].weight.num_rows
        else:
            for i, mod in enumerate(stack.modules):
                placement[i] = (torch.empty(m, mod.weight.num_rows, dtype=out_dtype, device=self.device),
                                mod.weight.num_rows, 0)
        self.outputs = {mod.name: placement[i][0][:, placement[i][2]:placement[i][2] + mod.weight.num_rows]
                        for i, mod in enumerate(stack.modules)}
        self._jobs = (_lib.GemvJob * len(stack.modules))()
        for i, mod in enumerate(stack.modules):
            qt = mod.weight
            x = self.inputs[mod.input]
            out, stride, col0 = placement[i]
            job = self._jobs[i]
            job.x = x.data_ptr()
            job.out = out.data_ptr()
            job.bias = None
            job.m = m
            job.out_stride = stride
            job.out_col0 = col0
            job.x_dtype = _tag(act_dtype, "x")
            job.out_dtype = _tag(out_dtype, "out")
            job.weight = weight_descriptor(
                "gemv_sequence", qt.packed, qt.scales, qt.offsets, qt.bits, qt.geometry.effective_group, qt.in_features
            )
        self._graph: torch.cuda.CUDAGraph | None = None
        self._plan: GemvPlan | None = None
        self.launches_per_step = len(stack.modules)  # replaced by the measured count in capture()

    def plan(self) -> GemvPlan:
        """The whole step as one persistent kernel (built on first use).  Raises ``RuntimeError``
        when a module does not meet the plan kernel's requirements."""
        if self._plan is None:
            self._plan = GemvPlan(self._jobs, len(self._jobs), self.device)
        return self._plan

    def run_plan(self) -> None:
        self.plan().launch()

    def run(self) -> None:
        """Enqueue the whole step on torch's current stream, module after module."""
        lib = _lib.load()
        with torch.cuda.device(self.device):
            _lib.check(lib.dq_gemv_sequence(self._jobs, len(self._jobs), _stream(self.device)))

    def count_launches(self) -> int:
        """Run the step once eagerly and record how many kernels it launched."""
        lib = _lib.load()
        before = int(lib.dq_launch_count())
        self.run()
        self.launches_per_step = int(lib.dq_launch_count()) - before
        return self.launches_per_step

    def _run_jobs(self, first: int, count: int) -> None:
        lib = _lib.load()
        jobs = ctypes.cast(ctypes.byref(self._jobs, first * ctypes.sizeof(_lib.GemvJob)), ctypes.POINTER(_lib.GemvJob))
        _lib.check(lib.dq_gemv_sequence(jobs, count, _stream(self.device)))

    def jobs_at(self, first: int):
        """Pointer to job ``first`` of the step's ``dq_gemv_job`` array."""
        return ctypes.cast(ctypes.byref(self._jobs, first * ctypes.sizeof(_lib.GemvJob)), ctypes.POINTER(_lib.GemvJob))

    def run_dataflow(self, side_streams: list[torch.cuda.Stream] | None = None, after_stage=None,
                     launch_stage=None) -> None:
        """Enqueue the step as its dependency graph: stage after stage, the members of a stage
        (q/k/v, gate/up: contiguous jobs reading one activation) in ONE library call, which
        issues them as one fused launch.  Stages whose members are not contiguous fork onto
        ``side_streams``.  ``after_stage(i)`` (optional) is called after stage ``i`` has been
        enqueued -- where a sharded runner enqueues the exchange of that stage's output.
        ``launch_stage(i, first, count)`` (optional) may enqueue stage ``i`` itself (a launch that
        also exchanges the output) and return True; on False the stage is enqueued as usual."""
        main = torch.cuda.current_stream(self.device)
        with torch.cuda.device(self.device):
            for index, stage in enumerate(self.stack.stages()):
                if list(stage) == list(range(stage[0], stage[0] + len(stage))):
                    if launch_stage is not None and launch_stage(index, stage[0], len(stage)):
                        continue
                    self._run_jobs(stage[0], len(stage))
                    if after_stage is not None:
                        after_stage(index)
                    continue
                fork = torch.cuda.Event()
                fork.record(main)
                self._run_jobs(stage[0], 1)
                for idx, side in zip(stage[1:], side_streams or []):
                    side.wait_event(fork)
                    with torch.cuda.stream(side):
                        self._run_jobs(idx, 1)
                    join = torch.cuda.Event()
                    join.record(side)
                    main.wait_event(join)

    def capture(self, mode: str = "dataflow", after_stage=None, launch_stage=None) -> None:
        """Record the step into a CUDA graph (``after_stage``, ``launch_stage``: see
        :meth:`run_dataflow`; dataflow mode only).

        ``"dataflow"``: stages in order, the members of a stage in one fused launch (what a
        decoder layer's dependencies allow).  ``"chain"``: the whole job list in stream order through
        one ``dq_gemv_sequence`` call -- consecutive modules that read the same activation
        (q/k/v, gate/up) leave as one fused launch, the rest one after the other.
        ``"independent"``: no edges at all -- every module's input is resident, nothing
        waits for anything (the regime the reference's per-shape bandwidth table measures).
        ``"plan"``: the same chain of stages as ``"dataflow"`` as ONE persistent kernel
        (:class:`GemvPlan`).
        """
        if mode == "plan":
            self.run_plan()  # builds the plan; first launch outside the capture
            self.plan().check()
        self.run()  # warm: sets per-kernel attributes outside the capture
        torch.cuda.synchronize(self.device)
        lib = _lib.load()
        before = int(lib.dq_launch_count())
        graph = torch.cuda.CUDAGraph()
        sides = [torch.cuda.Stream(self.device) for _ in range(8 if mode == "independent" else 2)]
        with torch.cuda.graph(graph):
            if mode == "chain":
                self.run()
            elif mode == "plan":
                self.run_plan()
            elif mode == "dataflow":
                self.run_dataflow(sides, after_stage, launch_stage)
            elif mode == "independent":
                main = torch.cuda.current_stream(self.device)
                fork = torch.cuda.Event()
                fork.record(main)
                lanes = [main, *sides]
                for s in sides:
                    s.wait_event(fork)
                for i in range(len(self._jobs)):
                    with torch.cuda.stream(lanes[i % len(lanes)]):
                        self._run_jobs(i, 1)
                for s in sides:
                    join = torch.cuda.Event()
                    join.record(s)
                    main.wait_event(join)
            else:
                raise ValueError(mode)
        self._graph = graph
        self.mode = mode
        self.launches_per_step = int(lib.dq_launch_count()) - before  # kernels recorded in the graph

    def replay(self) -> None:
        if self._graph is None:
            raise RuntimeError("capture() first")
        self._graph.replay()

    def capture_with_io(self, host_inputs: dict[str, torch.Tensor], output: str, host_output: torch.Tensor,
                        mode: str = "dataflow") -> None:
        """Record host -> device copies of the activations, the step, and the device -> host
        copy of one module's output into ONE graph: a serving loop that owns pinned staging
        buffers then pays a single graph launch per step instead of one host call per copy.

        ``host_inputs``: pinned CPU tensors, one per entry of ``inputs`` (same shapes and
        dtypes); ``output``: the module whose result is read back into pinned ``host_output``.
        """
        if set(host_inputs) != set(self.inputs):
            raise ValueError(f"host_inputs must cover exactly {sorted(self.inputs)}")
        for name, t in host_inputs.items():
            if not t.is_pinned() or t.shape != self.inputs[name].shape or t.dtype != self.inputs[name].dtype:
                raise ValueError(f"host input {name!r} must be pinned and match the device tensor")
        dev_out = self.outputs[output]
        if not host_output.is_pinned() or host_output.shape != dev_out.shape or host_output.dtype != dev_out.dtype:
            raise ValueError("host_output must be pinned and match the module's output")
        self.run()
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        sides = [torch.cuda.Stream(self.device) for _ in range(2)]
        with torch.cuda.graph(graph):
            for name, t in host_inputs.items():
                self.inputs[name].copy_(t, non_blocking=True)
            if mode == "chain":
                self.run()
            elif mode == "plan":
                self.run_plan()
            elif mode == "dataflow":
                self.run_dataflow(sides)
            else:
                raise ValueError(mode)
            host_output.copy_(dev_out, non_blocking=True)
        self._graph_io = graph

    def replay_with_io(self) -> None:
        """One step including its copies (``capture_with_io``); the caller synchronises the stream."""
        graph = getattr(self, "_graph_io", None)
        if graph is None:
            raise RuntimeError("capture_with_io() first")
        graph.replay()
