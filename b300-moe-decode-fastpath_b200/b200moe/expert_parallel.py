"""Expert-parallel execution of the layer on 1/2/4/8 GPUs of one NVSwitch box.

The reference has no multi-GPU code at all (README.md:206-207); this module is
new.  Experts shard naturally: rank ``r`` of ``N`` owns the contiguous experts
``[r*E/N, (r+1)*E/N)`` and keeps only their weights resident.

One forward:

1. *Dispatch.*  ``tokens="replicated"``: every rank already holds the same
   ``[T,H]`` activations and routes (decode after tensor-parallel attention);
   nothing moves.  ``tokens="sharded"``: every rank holds ``T/N`` tokens; the
   activations, ids and routing weights are all-gathered (at most ~1 MB at
   decode sizes, one NVSwitch hop).
2. *Local experts.*  One ``b200moe_forward`` call with
   ``B200MOE_FLAG_LOCAL_EXPERTS``: the routing kernel subtracts the rank's first
   expert id and silently drops assignments of other ranks, so the rank's
   stable order is the global stable order restricted to its experts; the GEMMs
   stream only the local active experts' weights; the combine kernel stores
   unrounded FP32 sums of the local assignments (``B200MOE_FLAG_F32_OUTPUT``).
3. *Combine.*  The FP32 partial outputs are summed across ranks and rounded to
   BF16 once.  ``transport="p2p"`` does the local combine and the cross-rank sum
   in one kernel of this library over NVLink peer memory
   (``b200moe_ep_combine_reduce``: weighted sum of the rank's rows, store to the
   rank's peer-mapped buffer, publish a flag, bounded wait for the peers' flags,
   plain peer loads of the partial rows of the ranks that own an expert of the
   token, fixed rank-order sum); ``transport="nccl"`` is the unfused baseline
   (combine kernel, all-reduce, cast).  ``sharded`` callers keep their own rows.

Global routing metadata (bit-exact against a single-GPU run) is assembled from
the ranks' local tensors by :meth:`ExpertParallelMoE.global_routing`.

The per-rank compute is injected (``local_forward``) so the host logic above
runs under ``gloo`` on CPUs in the tests; the default is the native kernels and
nothing else -- there is no CPU execution path in the product.
"""

from __future__ import annotations

import ctypes
from typing import Callable

import torch
import torch.distributed as dist

from . import _lib
from .forward import _enqueue, _native_args
from .validation import RoutedMoEShape
from .workspace import B300MoEWorkspace

LocalForward = Callable[..., torch.Tensor]


def expert_range(rank: int, world: int, num_experts: int) -> tuple[int, int]:
    """First expert id and expert count owned by ``rank``."""

    if num_experts % world != 0:
        raise ValueError(f"num_experts={num_experts} must be divisible by the world size {world}")
    per_rank = num_experts // world
    return rank * per_rank, per_rank


class _StepPlan:
    """What a repeated step of one rank needs, remembered after one fully checked forward with
    replicated tokens over peer memory (the counterpart of ``forward._CallPlan``): a later
    forward whose three tensors have the same dtypes, device, layout and width, on the same
    stream and workspace allocation, rewrites the per-call fields of the bound argument
    struct and goes straight to the two library calls of the step.  Anything else takes the
    checked path, which also covers every error case."""

    __slots__ = ("device", "device_index", "allocations", "stream", "stream_ptr", "args",
                 "args_ref", "fn", "flags", "shape_tail")


class ExpertParallelMoE:
    """The MoE decode layer with its experts spread over the ranks of a process group."""

    def __init__(
        self,
        gate_up_local: torch.Tensor,
        down_local: torch.Tensor,
        *,
        num_experts: int,
        top_k: int,
        group: dist.ProcessGroup | None = None,
        local_forward: LocalForward | None = None,
        capacity_tokens: int = 64,
        use_pdl: bool = True,
        transport: str = "nccl",
        fp8_scales: tuple[torch.Tensor, torch.Tensor] | None = None,
        nvfp4_scales: tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
        wait_limit_us: int = 0,
        combine: str = "auto",
    ) -> None:
        """``fp8_scales = (gate_up_scale [E_local, 2I], down_scale [E_local, H])`` marks the two
        weight tensors as E4M3 codes (uint8) of the FP8-weight path (``b200moe.fp8``).
        ``nvfp4_scales = (gate_up_scale [E_local], down_scale [E_local], gate_up_block_scale,
        down_block_scale)`` marks them as packed E2M1 (uint8 ``[E_local, 2I, H/2]`` and
        ``[E_local, H, I/2]``) of the NVFP4 path (``b200moe.nvfp4``: the fields of an
        ``Nvfp4ExpertWeights`` quantised from this rank's experts).
        ``wait_limit_us`` bounds every device-side wait for a peer (0: one second).
        ``combine`` (``transport="p2p"`` only) selects how rows cross the ranks: ``"push"``
        stores flagged rows into the receivers' inboxes (lowest latency; needs
        ``2 * world * capacity_tokens * H * 8`` bytes per rank and a grid that is resident at
        once), ``"pull"`` publishes one flag per rank and lets receivers read the owners' rows
        (any size), ``"auto"`` takes push when both conditions hold and the inbox stays under
        512 MiB."""

        self.wait_limit_us = int(wait_limit_us)

        if fp8_scales is not None and nvfp4_scales is not None:
            raise ValueError("give fp8_scales or nvfp4_scales, not both")
        self.fp8_scales = fp8_scales
        self.nvfp4_scales = nvfp4_scales
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.num_experts = num_experts
        self.top_k = top_k
        self.base, self.local_experts = expert_range(self.rank, self.world, num_experts)
        if gate_up_local.shape[0] != self.local_experts or down_local.shape[0] != self.local_experts:
            raise ValueError(
                f"rank {self.rank} owns {self.local_experts} experts but was given "
                f"{gate_up_local.shape[0]} / {down_local.shape[0]} weight slices"
            )
        self.gate_up = gate_up_local
        self.down = down_local
        # packed E2M1 holds two elements of H per byte
        self.hidden_size = gate_up_local.shape[2] * (2 if nvfp4_scales is not None else 1)
        self.use_pdl = use_pdl
        self._local_forward = local_forward or self._native_local_forward
        self._native = local_forward is None
        self.workspace = (
            B300MoEWorkspace(capacity_tokens=capacity_tokens, device=gate_up_local.device)
            if self._native
            else None
        )
        self._checked = False
        self._last_call = None
        self.last_tokens = 0
        self._plan: _StepPlan | None = None
        self.repeated_steps = 0  # forwards that took the remembered plan
        if transport not in ("nccl", "p2p"):
            raise ValueError("transport must be 'nccl' or 'p2p'")
        if transport == "p2p" and not self._native:
            raise ValueError("transport='p2p' needs the native kernels (CUDA peer memory)")
        self.transport = transport
        self.capacity_tokens = capacity_tokens
        self._epoch = 0
        if combine not in ("auto", "push", "pull"):
            raise ValueError("combine must be 'auto', 'push' or 'pull'")
        self.combine = "pull"
        if transport == "p2p":
            self.combine = self._choose_combine(combine)
            self._setup_peer_memory()

    # ------------------------------------------------------------------ peer memory
    def _inbox_bytes(self) -> int:
        return 2 * self.world * self.capacity_tokens * self.hidden_size * 8

    def _choose_combine(self, wanted: str) -> str:
        """``"push"`` needs every call's grid (tokens x ceil(H / 1024) blocks) resident at once."""

        if wanted == "pull":
            return "pull"
        blocks = ctypes.c_int(0)
        with torch.cuda.device(self.gate_up.device):
            _lib.check(_lib.load().b200moe_ep_push_max_blocks(ctypes.byref(blocks)),
                       "b200moe_ep_push_max_blocks")
        chunks = (self.hidden_size // 8 + 127) // 128
        fits = self.capacity_tokens * chunks <= blocks.value
        if wanted == "push":
            if not fits:
                raise ValueError(
                    f"combine='push' needs capacity_tokens * ceil(H / 1024) <= {blocks.value} "
                    f"blocks on this GPU, got {self.capacity_tokens * chunks}")
            return "push"
        return "push" if fits and self._inbox_bytes() <= (512 << 20) else "pull"

    def _setup_peer_memory(self) -> None:
        """Symmetric (peer-mapped) buffers for the native combine: two FP32 partial-output
        buffers used alternately, and one flag word per rank.  Allocated once; every rank
        maps every other rank's copy into its own address space."""

        import torch.distributed._symmetric_memory as symm_mem

        device = self.gate_up.device
        group = self.group if self.group is not None else dist.group.WORLD
        self._partials = symm_mem.empty(
            (2, self.capacity_tokens, self.hidden_size), dtype=torch.float32, device=device)
        self._flags = symm_mem.empty((_lib.EP_MAX_WORLD,), dtype=torch.int32, device=device)
        self._flags.zero_()
        self._partials.zero_()
        partial_handle = symm_mem.rendezvous(self._partials, group)
        flag_handle = symm_mem.rendezvous(self._flags, group)
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)
        stride = self.capacity_tokens * self.hidden_size * 4
        self._partial_ptrs = [
            (ctypes.c_void_p * self.world)(*[int(ptr) + parity * stride
                                             for ptr in partial_handle.buffer_ptrs])
            for parity in (0, 1)
        ]
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in flag_handle.buffer_ptrs])
        self._inbox = self._inbox_ptrs = None
        if self.combine == "push":
            # flagged rows land here: [epoch parity][source rank][token][H] words of 8 bytes
            self._inbox = symm_mem.empty((self._inbox_bytes() // 4,), dtype=torch.int32,
                                         device=device)
            self._inbox.zero_()
            inbox_handle = symm_mem.rendezvous(self._inbox, group)
            torch.cuda.synchronize(device)
            dist.barrier(group=self.group)
            self._inbox_ptrs = (ctypes.c_void_p * self.world)(
                *[int(p) for p in inbox_handle.buffer_ptrs])
            self._inbox_handle = inbox_handle
        # dispatch of sharded tokens: gathered activations / ids / weights, two sets
        cap, H, K = self.capacity_tokens, self.hidden_size, self.top_k
        self._g_hidden = symm_mem.empty((2, cap, H), dtype=torch.bfloat16, device=device)
        self._g_ids = symm_mem.empty((2, cap, K), dtype=torch.int64, device=device)
        self._g_weights = symm_mem.empty((2, cap, K), dtype=torch.bfloat16, device=device)
        self._g_flags = symm_mem.empty((_lib.EP_MAX_WORLD,), dtype=torch.int32, device=device)
        self._g_flags.zero_()
        self._push_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self._reduce_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self._reduce_args = None
        handles = [symm_mem.rendezvous(t, group)
                   for t in (self._g_hidden, self._g_ids, self._g_weights, self._g_flags)]
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)
        self._g_ptrs = [[int(p) for p in h.buffer_ptrs] for h in handles]
        self._handles = (partial_handle, flag_handle, *handles)

    def _peer_dispatch(self, hidden: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor):
        """Store this rank's token shard into every rank's gathered buffers (one launch of
        peer stores plus a flag), and return this rank's gathered views and the wait tuple
        for the routing kernel."""

        t_local = hidden.shape[0]
        total = t_local * self.world
        if total > self.capacity_tokens:
            raise ValueError(
                f"{total} tokens exceed the peer buffers' capacity ({self.capacity_tokens})")
        parity = self._epoch & 1
        cap, H, K = self.capacity_tokens, self.hidden_size, self.top_k
        row_bytes = (H * 2, K * 8, K * 2)
        arrays = []
        for which in range(3):
            set_bytes = cap * row_bytes[which]
            offset = parity * set_bytes + self.rank * t_local * row_bytes[which]
            arrays.append((ctypes.c_void_p * self.world)(
                *[base + offset for base in self._g_ptrs[which]]))
        flag_array = (ctypes.c_void_p * self.world)(*self._g_ptrs[3])
        args = _lib.B200MoeEpPushArgs()
        args.hidden_states = hidden.data_ptr()
        args.expert_indices = ids.data_ptr()
        args.expert_weights = weights.data_ptr()
        cast = lambda a: ctypes.cast(a, ctypes.POINTER(ctypes.c_void_p))  # noqa: E731
        args.hidden_dst, args.indices_dst, args.weights_dst = (cast(a) for a in arrays)
        args.flag_ptrs = cast(flag_array)
        args.block_counter = self._push_counter.data_ptr()
        args.world, args.rank = self.world, self.rank
        args.tokens_local, args.top_k, args.hidden_size = t_local, K, H
        args.epoch = self._epoch & 0xFFFFFFFF
        code = _enqueue(_lib.load().b200moe_ep_push, args, hidden.device)
        if code:
            _lib.check(code, "b200moe_ep_push")
        gathered = (self._g_hidden[parity][:total], self._g_ids[parity][:total],
                    self._g_weights[parity][:total])
        return gathered, (self._g_flags.data_ptr(), self.world, self._epoch & 0xFFFFFFFF)

    def _peer_reduce(self, tokens: int, parity: int, dtype: torch.dtype,
                     first_token: int = 0, stream_ptr: int | None = None,
                     out: torch.Tensor | None = None) -> torch.Tensor:
        """One launch after the down projection: this rank's combine, publish, wait for the
        peers (bounded), add the owning ranks' partial rows in rank order over NVLink, round
        to BF16.  ``tokens`` rows starting at ``first_token`` are returned."""

        assert self.workspace is not None and self.workspace.scratch is not None
        device = self.gate_up.device
        output = out if out is not None else \
            torch.empty(tokens, self.hidden_size, dtype=dtype, device=device)
        args = self._reduce_args
        if args is None:
            # everything that does not change between forwards is filled in once
            args = _lib.B200MoeEpReduceArgs()
            args.flag_ptrs = ctypes.cast(self._flag_ptrs, ctypes.POINTER(ctypes.c_void_p))
            args.world, args.rank = self.world, self.rank
            args.hidden_size = self.hidden_size
            args.wait_limit_us = self.wait_limit_us
            args.block_counter = self._reduce_counter.data_ptr()
            args.flags = _lib.FLAG_PDL if self.use_pdl else 0
            if self.combine == "push":
                args.flags |= _lib.FLAG_EP_PUSH
                args.inbox_ptrs = ctypes.cast(self._inbox_ptrs, ctypes.POINTER(ctypes.c_void_p))
                args.inbox_cap_tokens = self.capacity_tokens
            self._reduce_args = args
        args.partial_ptrs = ctypes.cast(self._partial_ptrs[parity],
                                        ctypes.POINTER(ctypes.c_void_p))
        args.num_tokens, args.first_token = tokens, first_token
        # sharded callers output `tokens` rows each; replicated callers all of them
        args.tokens_per_rank = tokens if tokens != self.last_tokens else 0
        args.epoch = self._epoch & 0xFFFFFFFF
        args.output = output.data_ptr()
        args.status = self.workspace.scratch.data_ptr()
        layer_args = self._last_call[0]
        lib = _lib.load()
        if stream_ptr is not None:  # a repeated step: device and stream are already checked
            code = lib.b200moe_ep_combine_reduce(ctypes.byref(layer_args), ctypes.byref(args),
                                                 stream_ptr)
            if code:
                _lib.check(code, "b200moe_ep_combine_reduce")
            return output
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        if torch.cuda.current_device() == device.index:
            code = lib.b200moe_ep_combine_reduce(ctypes.byref(layer_args), ctypes.byref(args),
                                                 stream)
        else:
            with torch.cuda.device(device):
                code = lib.b200moe_ep_combine_reduce(ctypes.byref(layer_args),
                                                     ctypes.byref(args), stream)
        if code:
            _lib.check(code, "b200moe_ep_combine_reduce")
        return output

    # ------------------------------------------------------------------ local compute
    def _native_local_forward(
        self, hidden: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
        ep_wait: tuple[int, int, int] | None = None,
    ) -> torch.Tensor:
        """FP32 ``[T,H]`` sum over this rank's assignments, by the sm_100a kernels."""

        if not self._checked:
            self._check_native_inputs(hidden, ids, weights)
            self._checked = True
        assert self.workspace is not None
        p2p = self.transport == "p2p"
        if p2p and hidden.shape[0] > self.capacity_tokens:
            raise ValueError(
                f"{hidden.shape[0]} tokens exceed the peer buffers' capacity "
                f"({self.capacity_tokens}); construct the layer with a larger capacity_tokens")
        # p2p: the forward stops after the down projection; the combine happens inside the
        # cross-rank kernel (_peer_reduce), which writes the peer-mapped partial buffer
        partial, call = local_partial_forward(
            hidden, ids, weights, self.gate_up, self.down, top_k=self.top_k,
            expert_id_base=self.base, num_experts_global=self.num_experts,
            workspace=self.workspace, use_pdl=self.use_pdl, ep_wait=ep_wait,
            fp8_scales=self.fp8_scales, nvfp4_scales=self.nvfp4_scales, skip_combine=p2p,
            ep_wait_limit_us=self.wait_limit_us, after_push=ep_wait is not None,
        )
        self._last_call = call
        return partial

    def run_local_stage(self, name: str) -> None:
        """Re-enqueue one stage of this rank's last local forward (per-stage timing)."""

        args, _keepalive = self._last_call
        fn = getattr(_lib.load(), f"b200moe_{name}")
        _lib.check(_enqueue(fn, args, self.gate_up.device), f"b200moe_{name}")

    def _check_native_inputs(
        self, hidden: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor
    ) -> None:
        """The single-GPU entry point's gates (b300_moe.py:526-550), for one rank's tensors."""

        if hidden.device.type != "cuda":
            raise ValueError("expert-parallel native compute requires CUDA tensors")
        if torch.cuda.get_device_capability(hidden.device) != (10, 0):
            raise RuntimeError("expert-parallel native compute requires compute capability (10, 0)")
        if ids.dtype != torch.int64:
            raise TypeError("expert_indices must have dtype torch.int64")
        quantised = self.fp8_scales is not None or self.nvfp4_scales is not None
        weight_dtype = torch.uint8 if quantised else torch.bfloat16
        for t, want in ((hidden, torch.bfloat16), (weights, torch.bfloat16),
                        (self.gate_up, weight_dtype), (self.down, weight_dtype)):
            if t.dtype != want:
                raise TypeError("native expert-parallel compute requires bfloat16 inputs and "
                                "bfloat16 (or, with fp8_scales / nvfp4_scales, uint8) weights")
        if self.fp8_scales is not None:
            gs, ds = self.fp8_scales
            inter_ = self.gate_up.shape[1] // 2
            if tuple(gs.shape) != (self.local_experts, 2 * inter_) or \
                    tuple(ds.shape) != (self.local_experts, self.hidden_size) or \
                    gs.dtype != torch.float32 or ds.dtype != torch.float32:
                raise ValueError("fp8_scales must be float32 [E_local, 2I] and [E_local, H]")
            if self.hidden_size % 16 or inter_ % 16:
                raise ValueError("the FP8-weight path requires H and I divisible by 16")
        for t in (hidden, ids, weights, self.gate_up, self.down):
            if not t.is_contiguous():
                raise ValueError("all inputs must be contiguous")
            if t.device != hidden.device:
                raise ValueError("all inputs must be on the same device")
        inter = self.gate_up.shape[1] // 2
        if self.hidden_size % 8 or inter % 8:
            raise ValueError("hidden_size and intermediate_size must be divisible by 8")
        packed = 2 if self.nvfp4_scales is not None else 1
        if tuple(self.down.shape) != (self.local_experts, self.hidden_size, inter // packed):
            raise ValueError("down_weight must have shape [E_local, H, I] ([E_local, H, I/2] "
                             "bytes for NVFP4)")
        if self.nvfp4_scales is not None:
            gs, ds, gb, db = self.nvfp4_scales
            if tuple(gs.shape) != (self.local_experts,) or tuple(ds.shape) != (self.local_experts,) \
                    or gs.dtype != torch.float32 or ds.dtype != torch.float32 \
                    or gb.dtype != torch.uint8 or db.dtype != torch.uint8:
                raise ValueError("nvfp4_scales must be (float32 [E_local], float32 [E_local], "
                                 "uint8 block scales, uint8 block scales)")
            if self.hidden_size % 64 or inter % 64:
                raise ValueError("the NVFP4 path requires H and I divisible by 64")
        _lib.load()

    # ------------------------------------------------------------------ repeated steps
    def _remember_step(self) -> None:
        """Keep what the checked forward that just ran established (peer transport,
        replicated tokens)."""

        ws = self.workspace
        if ws is None or self._last_call is None or torch.cuda.is_current_stream_capturing():
            self._plan = None
            return
        device = self.gate_up.device
        plan = _StepPlan()
        plan.device, plan.device_index = device, device.index
        plan.allocations = ws.allocation_count
        plan.stream = torch.cuda.current_stream(device)
        plan.stream_ptr = int(plan.stream.cuda_stream)
        plan.args = self._last_call[0]
        plan.args_ref = ctypes.byref(plan.args)
        plan.fn = _lib.load().b200moe_forward
        plan.flags = int(plan.args.flags)
        plan.shape_tail = tuple(ws._last_shape[1:]) if ws._last_shape else None
        self._plan = plan if plan.shape_tail is not None else None

    def _repeat_step(self, hidden: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                     out: torch.Tensor | None = None) -> torch.Tensor | None:
        """The output of a replicated-token forward that matches the remembered plan, or
        ``None`` (the caller then takes the checked path)."""

        plan, ws = self._plan, self.workspace
        if plan is None or ws is None or hidden.dim() != 2:
            return None
        tokens = hidden.shape[0]
        if (
            hidden.shape[1] != self.hidden_size
            or tuple(ids.shape) != (tokens, self.top_k)
            or weights.shape != ids.shape
            or hidden.dtype is not torch.bfloat16
            or weights.dtype is not torch.bfloat16
            or ids.dtype is not torch.int64
            or hidden.device != plan.device
            or ids.device != plan.device
            or weights.device != plan.device
            or not hidden.is_contiguous()
            or not ids.is_contiguous()
            or not weights.is_contiguous()
            or hidden.requires_grad
            or weights.requires_grad
            or tokens < 1
            or tokens > self.capacity_tokens
            or torch.cuda.current_device() != plan.device_index
        ):
            return None
        with ws._lock:
            if (
                ws._allocations != plan.allocations
                or tokens > ws._tokens
                or ws._last_stream != plan.stream_ptr
                or torch._C._cuda_getCurrentRawStream(plan.device_index) != plan.stream_ptr
                or torch._C._cuda_isCurrentStreamCapturing()
            ):
                return None
            self._epoch += 1
            args = plan.args
            args.hidden_states = hidden.data_ptr()
            args.expert_indices = ids.data_ptr()
            args.expert_weights = weights.data_ptr()
            args.num_tokens = tokens
            args.output = None
            args.flags = plan.flags
            args.expert_id_base = self.base
            args.ep_wait_flags = None
            args.ep_world = 0
            args.ep_epoch = 0
            args.ep_wait_limit_us = 0
            code = plan.fn(plan.args_ref, plan.stream_ptr)
            if code:
                _lib.check(code, "b200moe_forward (expert-parallel rank)")
            ws._reuses += 1
            ws._last_reused = True
            ws._last_shape = (tokens,) + plan.shape_tail
            ws._event.record(plan.stream)
        self._last_call = (args, (hidden, ids, weights, self.gate_up, self.down, None))
        self.last_tokens = tokens
        self.repeated_steps += 1
        return self._peer_reduce(tokens, self._epoch & 1, hidden.dtype, 0, plan.stream_ptr, out)

    # ------------------------------------------------------------------ forward
    def forward(
        self,
        hidden_states: torch.Tensor,
        expert_indices: torch.Tensor,
        expert_weights: torch.Tensor,
        *,
        tokens: str = "replicated",
        check_status: bool = False,
        out: torch.Tensor | None = None,
    ) -> torch.Tensor:
        """Run the layer; returns BF16 ``[T,H]`` for the tokens this rank was given.

        ``out`` (peer transport only): where the cross-rank combine stores this rank's rows
        instead of a fresh tensor -- contiguous, of the inputs' shape and dtype, on this
        rank's GPU or in pinned host memory (the rows then cross PCIe from the kernel and no
        device-to-host copy is needed).

        A peer that does not arrive within the wait limit does not hang the call: the rows
        that needed it come back as zeros and ``B200MOE_STATUS_PEER_TIMEOUT`` is set in the
        workspace status word.  ``check_status=True`` reads that word after the call (one
        synchronisation) and raises ``RuntimeError``; without it, call
        ``self.workspace.raise_for_status()`` before the next forward, whose first kernel
        clears the word."""

        if tokens not in ("replicated", "sharded"):
            raise ValueError("tokens must be 'replicated' or 'sharded'")
        if expert_indices.shape[1] != self.top_k:
            raise ValueError("top_k must match expert_indices.shape[1]")
        if out is not None:
            if self.transport != "p2p":
                raise ValueError("out needs transport='p2p'")
            if not isinstance(out, torch.Tensor) or out.shape != hidden_states.shape or \
                    out.dtype != hidden_states.dtype or not out.is_contiguous() or \
                    not (out.device == hidden_states.device or
                         (out.device.type == "cpu" and out.is_pinned())):
                raise ValueError("out must be a contiguous tensor of the inputs' shape and "
                                 "dtype on this rank's GPU or in pinned host memory")
        if tokens == "replicated" and self._plan is not None:
            output = self._repeat_step(hidden_states, expert_indices, expert_weights, out)
            if output is not None:
                if check_status:
                    self.workspace.raise_for_status()
                return output
        local_tokens = hidden_states.shape[0]
        self._epoch += 1
        sharded = tokens == "sharded" and self.world > 1
        self._plan = None
        ep_wait = None
        if sharded and self.transport == "p2p":
            (hidden_all, ids_all, weights_all), ep_wait = self._peer_dispatch(
                hidden_states.contiguous(), expert_indices.contiguous(),
                expert_weights.contiguous())
        elif sharded:
            hidden_all = self._all_gather(hidden_states)
            ids_all = self._all_gather(expert_indices)
            weights_all = self._all_gather(expert_weights)
        else:
            hidden_all, ids_all, weights_all = hidden_states, expert_indices, expert_weights
        self.last_tokens = hidden_all.shape[0]

        if ep_wait is not None:
            partial = self._local_forward(hidden_all, ids_all, weights_all, ep_wait=ep_wait)
        else:
            partial = self._local_forward(hidden_all, ids_all, weights_all)
        if self.transport == "p2p":
            # a sharded caller only needs its own rows: reduce that slice of every partial
            first = self.rank * local_tokens if sharded else 0
            rows = local_tokens if sharded else hidden_all.shape[0]
            output = self._peer_reduce(rows, self._epoch & 1, hidden_states.dtype, first,
                                       out=out)
            if tokens == "replicated":
                self._remember_step()
            if check_status:
                self.workspace.raise_for_status()
            return output
        if self.world > 1:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
        output = partial.to(hidden_states.dtype)
        if sharded:
            output = output[self.rank * local_tokens:(self.rank + 1) * local_tokens]
        if check_status and self.workspace is not None:
            self.workspace.raise_for_status()
        return output

    def _all_gather(self, tensor: torch.Tensor) -> torch.Tensor:
        out = torch.empty((self.world * tensor.shape[0],) + tuple(tensor.shape[1:]),
                          dtype=tensor.dtype, device=tensor.device)
        dist.all_gather_into_tensor(out, tensor.contiguous(), group=self.group)
        return out

    # ------------------------------------------------------------------ metadata
    def local_routing(self) -> dict[str, torch.Tensor]:
        """This rank's routing tensors of the last forward (native compute only)."""

        assert self.workspace is not None
        rows = self.last_tokens * self.top_k
        b = self.workspace.buffers
        return {
            "expert_counts": b["expert_counts"][: self.local_experts],
            "expert_offsets": b["expert_offsets"][: self.local_experts + 1],
            "permutation": b["permutation"][:rows],
            "reverse_mapping": b["reverse_mapping"][:rows],
        }

    def global_routing(self, local: dict[str, torch.Tensor] | None = None) -> dict[str, torch.Tensor]:
        """Assemble the single-GPU routing tensors from the ranks' local ones.

        Experts are contiguous per rank, so the global expert-major order is rank 0's rows,
        then rank 1's, ...: counts concatenate, offsets are their running sum, a rank's
        permutation entries keep their (global) assignment ids, and an assignment's global
        row is its local row plus the rows of all lower ranks.
        """

        local = local or self.local_routing()
        return assemble_global_routing(local, self.world, self.group)


def local_partial_forward(
    hidden: torch.Tensor,
    ids: torch.Tensor,
    weights: torch.Tensor,
    gate_up_local: torch.Tensor,
    down_local: torch.Tensor,
    *,
    top_k: int,
    expert_id_base: int,
    num_experts_global: int,
    workspace: B300MoEWorkspace,
    use_pdl: bool = True,
    out: torch.Tensor | None = None,
    ep_wait: tuple[int, int, int] | None = None,
    fp8_scales: tuple[torch.Tensor, torch.Tensor] | None = None,
    skip_combine: bool = False,
    ep_wait_limit_us: int = 0,
    nvfp4_scales: tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
    after_push: bool = False,
):
    """One rank's share of the layer: FP32 ``[T,H]`` sum over the assignments whose expert
    id lies in ``[expert_id_base, expert_id_base + E_local)``.

    ``ids`` are GLOBAL expert ids; other ranks' assignments are dropped by the routing
    kernel (``reverse_mapping == -1``).  Returns the partial output and the bound native
    call (argument struct plus the tensors it points to) for per-stage re-runs.
    ``skip_combine`` stops after the down projection (no partial output is produced; the
    caller runs ``b200moe_ep_combine_reduce`` on the returned call).
    """

    tokens, hidden_size = hidden.shape
    local_experts = gate_up_local.shape[0]
    inter = gate_up_local.shape[1] // 2
    shape = RoutedMoEShape(tokens, local_experts, top_k, hidden_size, inter)
    with workspace._lock:
        # public buffers are sized for the global expert count (>= top_k, >= the local share)
        workspace.reserve(
            num_tokens=tokens, num_experts=num_experts_global, top_k=top_k,
            hidden_size=hidden_size, intermediate_size=inter, device=hidden.device,
            dtype=hidden.dtype, backend="b200_bf16", quant_mode="bf16",
        )
        if skip_combine:
            partial = None
        elif out is None:
            partial = torch.empty(tokens, hidden_size, dtype=torch.float32, device=hidden.device)
        else:
            if out.dtype != torch.float32 or tuple(out.shape) != (tokens, hidden_size) or \
                    not out.is_contiguous():
                raise ValueError("out must be a contiguous float32 [T, H] tensor")
            partial = out
        flags = _lib.FLAG_LOCAL_EXPERTS | _lib.FLAG_F32_OUTPUT
        if skip_combine:
            flags |= _lib.FLAG_SKIP_COMBINE
        if use_pdl:
            flags |= _lib.FLAG_PDL
        if fp8_scales is not None:
            flags |= _lib.FLAG_FP8_WEIGHTS
        if nvfp4_scales is not None:
            flags |= _lib.FLAG_NVFP4_WEIGHTS
        args = _native_args(hidden, ids, weights, gate_up_local, down_local, shape, workspace,
                            partial, flags, expert_id_base=expert_id_base)
        if fp8_scales is not None:
            args.gate_up_scale = fp8_scales[0].data_ptr()
            args.down_scale = fp8_scales[1].data_ptr()
        if nvfp4_scales is not None:
            args.gate_up_scale = nvfp4_scales[0].data_ptr()
            args.down_scale = nvfp4_scales[1].data_ptr()
            args.gate_up_block_scale = nvfp4_scales[2].data_ptr()
            args.down_block_scale = nvfp4_scales[3].data_ptr()
        if ep_wait is not None:
            # (device address of this rank's dispatch flags, world size, epoch): the routing
            # kernel waits for every rank's pushed shard before it reads ids or rows
            args.ep_wait_flags, args.ep_world, args.ep_epoch = ep_wait
            args.ep_wait_limit_us = ep_wait_limit_us
            if after_push:
                # the dispatch kernel was enqueued just before this call on the same stream:
                # the routing kernel may start beside it and wait for the flags alone
                args.flags |= _lib.FLAG_EP_AFTER_PUSH
        code = _enqueue(_lib.load().b200moe_forward, args, hidden.device)
        if code:
            _lib.check(code, "b200moe_forward (expert-parallel rank)")
        workspace._record_use()
    return partial, (args, (hidden, ids, weights, gate_up_local, down_local, partial))


def assemble_global_routing(
    local: dict[str, torch.Tensor], world: int, group: dist.ProcessGroup | None = None
) -> dict[str, torch.Tensor]:
    counts_local = local["expert_counts"].contiguous()
    perm_local = local["permutation"].contiguous()
    rev_local = local["reverse_mapping"].contiguous()
    rows = perm_local.numel()
    if world == 1:
        return {k: v.clone() for k, v in local.items()}
    counts = [torch.empty_like(counts_local) for _ in range(world)]
    perms = [torch.empty_like(perm_local) for _ in range(world)]
    revs = [torch.empty_like(rev_local) for _ in range(world)]
    dist.all_gather(counts, counts_local, group=group)
    dist.all_gather(perms, perm_local, group=group)
    dist.all_gather(revs, rev_local, group=group)
    all_counts = torch.cat(counts)
    offsets = torch.cat([all_counts.new_zeros(1), all_counts.cumsum(0)])
    rank_rows = torch.stack([c.sum() for c in counts])
    rank_base = torch.cat([rank_rows.new_zeros(1), rank_rows.cumsum(0)])
    permutation = torch.cat([perms[r][: int(rank_rows[r])] for r in range(world)])
    reverse = torch.full((rows,), -1, dtype=rev_local.dtype, device=rev_local.device)
    for r in range(world):
        mine = revs[r] >= 0
        reverse = torch.where(mine, revs[r] + rank_base[r], reverse)
    return {
        "expert_counts": all_counts,
        "expert_offsets": offsets,
        "permutation": permutation,
        "reverse_mapping": reverse,
    }
