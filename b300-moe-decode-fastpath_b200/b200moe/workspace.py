"""``B300MoEWorkspace``: capacity-backed scratch with the reference's reuse contract.

Contract mirrored from fastpath/b300_moe.py:63-347: a workspace binds to its
first device; a compatible call reuses the allocation (``reuse_count``), a call
with more tokens grows it (at least doubling), a call with another layout
reallocates; reuse across CUDA streams is ordered by one event recorded after
every use; nothing may be allocated while the stream is being captured.  The
twelve public buffers keep the reference's names and dtypes.

Added for the native kernels: one private byte region (split-K partial rows,
low-order activation halves, the device-built schedule, the status word) sized
by ``b200moe_scratch_bytes``.  ``gate_up_output`` is kept as a zero-row buffer:
the [A, 2I] intermediate never exists because SwiGLU runs in the GEMM epilogue.
"""

from __future__ import annotations

import threading
from types import MappingProxyType
from typing import Mapping

import torch

from . import _lib
from .validation import BACKENDS, QUANT_MODES, SUPPORTED_DTYPES, SUPPORTED_TOP_K

_INT64_BUFFERS = frozenset(
    {
        "expert_counts",
        "expert_offsets",
        "permutation",
        "reverse_mapping",
        "permuted_token_indices",
        "permuted_expert_indices",
    }
)
_NATIVE_BACKENDS = ("cutlass_bf16", "b200_bf16")
_SCRATCH_ALIGN = 256


def _device(device: torch.device | str) -> torch.device:
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


class B300MoEWorkspace:
    """Reusable scratch storage for :func:`b300_moe_forward`."""

    def __init__(
        self, capacity_tokens: int = 0, *, device: torch.device | str | None = None
    ) -> None:
        if isinstance(capacity_tokens, bool) or not isinstance(capacity_tokens, int):
            raise TypeError("capacity_tokens must be an integer")
        if capacity_tokens < 0:
            raise ValueError("capacity_tokens must be non-negative")
        self._hint = capacity_tokens
        self._tokens = 0
        self._assignments = 0
        self._device = None if device is None else _device(device)
        self._dtype: torch.dtype | None = None
        self._signature: tuple[object, ...] | None = None
        self._last_shape: tuple[int, int, int, int, int] | None = None
        self._buffers: dict[str, torch.Tensor] = {}
        self._scratch: torch.Tensor | None = None
        self._scratch_base: torch.Tensor | None = None
        self._allocations = 0
        self._reuses = 0
        self._last_reused = False
        self._last_stream: int | None = None
        self._event: torch.cuda.Event | None = None
        self._recorded_streams: set[int] = set()
        self._args_cache: tuple[object, object] | None = None  # bound native argument struct
        self._plan = None  # facts established by the last fully checked forward (forward.py)
        self._lock = threading.RLock()

    # -- read-only state --------------------------------------------------------
    @property
    def device(self) -> torch.device | None:
        return self._device

    @property
    def dtype(self) -> torch.dtype | None:
        return self._dtype

    @property
    def capacity_tokens(self) -> int:
        return max(self._hint, self._tokens)

    @property
    def capacity_assignments(self) -> int:
        return self._assignments

    @property
    def public_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._buffers.values())

    @property
    def private_bytes(self) -> int:
        return 0 if self._scratch is None else self._scratch.numel()

    @property
    def capacity_bytes(self) -> int:
        return self.public_bytes + self.private_bytes

    @property
    def allocation_count(self) -> int:
        return self._allocations

    @property
    def reuse_count(self) -> int:
        return self._reuses

    @property
    def last_reserve_reused(self) -> bool:
        return self._last_reused

    @property
    def shape_signature(self) -> tuple[object, ...] | None:
        return self._signature

    @property
    def last_shape(self) -> tuple[int, int, int, int, int] | None:
        """Last requested ``(T, E, K, H, I)``."""
        return self._last_shape

    @property
    def last_stream(self) -> int | None:
        return self._last_stream

    @property
    def buffers(self) -> Mapping[str, torch.Tensor]:
        return MappingProxyType(self._buffers)

    @property
    def scratch(self) -> torch.Tensor | None:
        """The private byte region handed to the native library (256-byte aligned)."""
        return self._scratch

    def buffer_data_ptrs(self) -> dict[str, int]:
        return {name: t.data_ptr() for name, t in self._buffers.items()}

    # -- status word ----------------------------------------------------------------
    def status(self) -> int:
        """Read the device status word of the last forward (synchronises)."""

        if self._scratch is None:
            return 0
        return int(self._scratch[:4].view(torch.int32).item()) & 0xFFFFFFFF

    TIMELINE_KERNELS = ("routing", "gather", "gate_up", "down", "combine", "ep_reduce")

    def timeline(self) -> dict[str, tuple[float, float]]:
        """Device timeline of the last forward (synchronises): for each kernel the time its
        first block started and its last block finished, in microseconds after the start of
        the routing kernel, from ``%globaltimer`` stamps the kernels leave in the scratch
        region.  ``*_first_data`` is when block 0 of a GEMM saw its first operands arrive.
        A forward in small-call order starts with the gate+up kernel, whose times are then
        negative or near zero, and has no ``gather`` entry."""

        if self._scratch is None:
            return {}
        words = self._scratch[64:64 + 128].view(torch.int64).cpu().tolist()
        origin = words[0]
        result: dict[str, tuple[float, float]] = {}
        for k, name in enumerate(self.TIMELINE_KERNELS):
            start, end = words[2 * k], words[2 * k + 1]
            if end:
                result[name] = ((start - origin) / 1e3, (end - origin) / 1e3)
        for k, name in ((6, "gate_up_first_data"), (7, "down_first_data")):
            if words[2 * k]:
                result[name] = ((words[2 * k] - origin) / 1e3, (words[2 * k] - origin) / 1e3)
        return result

    def raise_for_status(self) -> None:
        """Raise if the last forward reported a device-side condition (synchronises).

        Out-of-range expert ids raise the same ``ValueError`` the reference
        raises on CPU (reference.py:104-105); a pipeline wait that ran out is a
        ``RuntimeError``.
        """

        bits = self.status()
        if bits & _lib.STATUS_BAD_EXPERT_ID:
            raise ValueError("expert_indices contains an out-of-range expert index")
        if bits & (_lib.STATUS_PIPE_TIMEOUT | _lib.STATUS_PEER_TIMEOUT):
            raise RuntimeError(f"a bounded device-side wait gave up (status 0x{bits:x})")

    # -- allocation -------------------------------------------------------------------
    def _allocate(
        self,
        tokens: int,
        num_experts: int,
        top_k: int,
        hidden: int,
        inter: int,
        device: torch.device,
        dtype: torch.dtype,
        backend: str,
    ) -> None:
        rows = tokens * top_k
        native = backend in _NATIVE_BACKENDS
        shapes: dict[str, tuple[int, ...]] = {
            "expert_counts": (num_experts,),
            "expert_offsets": (num_experts + 1,),
            "expert_offsets_i32": (num_experts,),
            "permutation": (rows,),
            "reverse_mapping": (rows,),
            "permuted_token_indices": (rows,),
            "permuted_expert_indices": (rows,),
            "permuted_weights": (rows,),
            "permuted_hidden": (rows, hidden),
            "gate_up_output": (0 if native else rows, 2 * inter),
            "swiglu_output": (rows, inter),
            "expert_output": (rows, hidden),
        }
        buffers: dict[str, torch.Tensor] = {}
        for name, dims in shapes.items():
            if name in _INT64_BUFFERS:
                kind = torch.int64
            elif name == "expert_offsets_i32":
                kind = torch.int32
            else:
                kind = dtype
            buffers[name] = torch.empty(dims, device=device, dtype=kind)
        self._buffers = buffers
        self._scratch = None
        self._scratch_base = None
        self._recorded_streams = set()
        self._args_cache = None
        self._plan = None
        if native and device.type == "cuda":
            need = _lib.scratch_bytes(tokens, top_k, num_experts, hidden, inter)
            base = torch.empty(need + _SCRATCH_ALIGN, device=device, dtype=torch.uint8)
            skew = (-base.data_ptr()) % _SCRATCH_ALIGN
            self._scratch_base = base
            self._scratch = base[skew : skew + need]
            self._scratch[:_SCRATCH_ALIGN].zero_()
        self._tokens = tokens
        self._assignments = rows
        self._dtype = dtype
        self._allocations += 1

    def reserve(
        self,
        *,
        num_tokens: int,
        num_experts: int,
        top_k: int,
        hidden_size: int,
        intermediate_size: int,
        device: torch.device | str,
        dtype: torch.dtype,
        backend: str = "torch",
        quant_mode: str = "none",
    ) -> bool:
        """Make room for one call; return True when the allocation was reused."""

        for name, value in (
            ("num_tokens", num_tokens),
            ("num_experts", num_experts),
            ("top_k", top_k),
            ("hidden_size", hidden_size),
            ("intermediate_size", intermediate_size),
        ):
            if isinstance(value, bool) or not isinstance(value, int):
                raise TypeError(f"{name} must be an integer")
            if value < 1:
                raise ValueError(f"{name} must be positive")
        if top_k not in SUPPORTED_TOP_K:
            raise ValueError("top_k must be one of (1, 2, 4, 8)")
        if top_k > num_experts:
            raise ValueError("top_k must not exceed num_experts")
        if dtype not in SUPPORTED_DTYPES:
            raise TypeError("dtype must be float32, float16, or bfloat16")
        if backend not in BACKENDS:
            raise ValueError("unknown B300 backend")
        if quant_mode not in QUANT_MODES:
            raise ValueError("unknown quant_mode")

        target = _device(device)
        with self._lock:
            if self._device is not None and self._device != target:
                raise ValueError(f"workspace is bound to device {self._device}, got {target}")
            self._device = target
            signature = (
                target,
                dtype,
                num_experts,
                top_k,
                hidden_size,
                intermediate_size,
                # the two names of the native path share one layout
                "b200_bf16" if backend in _NATIVE_BACKENDS else backend,
                quant_mode,
            )
            new_layout = signature != self._signature
            must_allocate = not self._buffers or new_layout or num_tokens > self._tokens

            on_cuda = target.type == "cuda"
            if on_cuda:
                stream = torch.cuda.current_stream(target)
                capturing = torch.cuda.is_current_stream_capturing()
                # Work already queued on this same stream is ordered by the stream itself;
                # the event is only needed when the previous use was on another stream.  A
                # capturing stream must not wait on work outside its graph (CUDA rejects the
                # dependency); the caller synchronises before starting a capture.
                if (
                    self._event is not None
                    and not capturing
                    and self._last_stream != int(stream.cuda_stream)
                ):
                    stream.wait_event(self._event)
                if self._event is None:
                    if capturing:
                        raise RuntimeError(
                            "workspace event cannot be created during CUDA graph capture; "
                            "call reserve before capture"
                        )
                    self._event = torch.cuda.Event(blocking=False)
                    self._event.record(stream)
                if must_allocate and capturing:
                    raise RuntimeError(
                        "workspace capacity/layout cannot change during CUDA graph capture; "
                        "call reserve before capture"
                    )

            if must_allocate:
                capacity = max(self._hint, num_tokens)
                if not new_layout:
                    capacity = max(capacity, 2 * self._tokens, 1)
                self._allocate(
                    capacity,
                    num_experts,
                    top_k,
                    hidden_size,
                    intermediate_size,
                    target,
                    dtype,
                    backend,
                )
                self._signature = signature
            else:
                self._reuses += 1
            self._last_shape = (num_tokens, num_experts, top_k, hidden_size, intermediate_size)
            self._last_reused = not must_allocate
            if on_cuda:
                self._last_stream = int(stream.cuda_stream)
                self._record_streams(stream)
            else:
                self._last_stream = None
            return self._last_reused

    def _record_streams(self, stream: "torch.cuda.Stream") -> None:
        # One record per (allocation, stream) is enough: the caching allocator keeps the
        # stream in the block's set until the block is freed.
        key = int(stream.cuda_stream)
        if key in self._recorded_streams:
            return
        self._recorded_streams.add(key)
        for tensor in self._buffers.values():
            tensor.record_stream(stream)
        if self._scratch_base is not None:
            self._scratch_base.record_stream(stream)

    def _record_use(self) -> None:
        """Record the completion event after the kernels (and metadata clones) of one call."""

        if self._device is None or self._device.type != "cuda":
            return
        if self._event is None:
            raise RuntimeError("workspace completion event is missing; call reserve before use")
        stream = torch.cuda.current_stream(self._device)
        # An event recorded while the stream is being captured belongs to the graph and
        # cannot order later eager work; inside a capture the graph's own edges order reuse.
        if not torch.cuda.is_current_stream_capturing():
            self._event.record(stream)
        self._last_stream = int(stream.cuda_stream)
        self._record_streams(stream)
