"""The Python face of the collective: a constructor, two calls and an output allocator.

Everything that survives a call (windows, cached plans, the lend pool) lives in the C++ runtime
(csrc/runtime/group.cc). What stays here has no C++ equivalent: resolving the process group,
the comm stream, and wrapping async results in ``AsyncCollectiveTensor``.

Parity: python/fast_ulysses/group.py:35-286 of the reference, same methods and keyword
arguments. Added on top: ``device="cpu"`` selects a CPU/gloo backend that runs the same plan
through ``all_to_all_single`` (for plumbing tests without a GPU); ``check()`` surfaces a
handshake that ran out of time as an exception instead of a hang; ``barrier()`` is the
device-side cross-rank barrier on its own.
"""

from __future__ import annotations

import warnings

import torch
import torch.distributed as dist

from .. import _C  # noqa: F401  (registers torch.ops.fast_ulysses_b200)

_OPS = torch.ops.fast_ulysses_b200


class CompletedHandle:
    """Returned by the async call when there is no work registry to bind the completion event to
    (and always on the CPU backend, which completes before returning). ``wait()`` only unwraps."""

    def __init__(self, tensor: torch.Tensor) -> None:
        self._tensor = tensor

    def wait(self) -> torch.Tensor:
        return self._tensor

    def __repr__(self) -> str:
        return f"CompletedHandle({tuple(self._tensor.shape)}, {self._tensor.dtype})"


class UlyssesGroup:
    """Ulysses all-to-all ``(b, s_local, n_global, d) <-> (b, s_global, n_local, d)`` over one
    NVLink domain, moved by an SM-driven sm_100a kernel with fused handshakes.

    Construction is collective over ``process_group``. Windows are allocated on the first call
    that needs one and cached, so every rank must issue the same sequence of shapes.
    """

    def __init__(
        self,
        process_group: dist.ProcessGroup | None = None,
        device: torch.device | str | int | None = None,
        *,
        require_nvlink: bool = True,
        timeout_ms: int = 10_000,
    ) -> None:
        """
        Args:
            process_group: the group to run over; ``None`` uses ``dist.group.WORLD``. Without an
                initialised default group and with no group given, a single-rank group is built.
            device: this rank's device. A CUDA device (or ``None`` for the current one) selects
                the NVLink backend; ``"cpu"`` selects the CPU/gloo backend.
            require_nvlink: refuse a group whose GPUs are not all NVLink-joined.
            timeout_ms: bound on every device-side cross-rank wait; a wait that runs out is
                reported by ``check()``.
        """
        self._destroyed = True  # so that __del__ is safe if anything below throws
        if process_group is None and not dist.is_initialized():
            self.pg = None
            self.rank, self.world_size, name = 0, 1, "fu_single"
        else:
            pg = process_group if process_group is not None else dist.group.WORLD
            self.pg = pg
            self.rank = dist.get_rank(pg)
            self.world_size = dist.get_world_size(pg)
            name = pg.group_name

        if device is None:
            device = torch.device("cuda")
        device = torch.device(device) if not isinstance(device, int) else torch.device("cuda", device)
        if device.type not in ("cuda", "cpu"):
            raise ValueError(f"device must be a CUDA device or 'cpu', got {device}")
        if device.type == "cuda":
            if device.index is None:
                device = torch.device("cuda", torch.cuda.current_device())
            torch.cuda.set_device(device)
        self.device = device

        if device.type == "cuda" and require_nvlink and self.world_size > 1:
            self._require_nvlink()

        if device.type == "cuda" and self.world_size > 1:
            import torch.distributed._symmetric_memory as symm_mem

            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                symm_mem.enable_symm_mem_for_group(name)

        index = int(device.index) if device.type == "cuda" else -1
        self._handle = torch.classes.fast_ulysses_b200.UlyssesGroup(name, int(self.rank), int(self.world_size), index)
        self._handle.set_timeout_ms(int(timeout_ms))
        self._comm_stream = None
        if device.type == "cuda":
            # The async call runs here; the sync call stays on the caller's stream. The two are not
            # ordered against each other, which is why the runtime gives them separate windows.
            _, greatest = torch.cuda.Stream.priority_range()
            self._comm_stream = torch.cuda.Stream(device=device, priority=greatest)
        self._destroyed = False
        self._fp8_window: dict = {}

    # ------------------------------------------------------------------------------------------
    def _require_nvlink(self) -> None:
        """Every rank checks the same device list, so all of them accept or refuse together."""
        local = torch.tensor([self.device.index], dtype=torch.int64, device=self.device)
        gathered = [torch.zeros_like(local) for _ in range(self.world_size)]
        dist.all_gather(gathered, local, group=self.pg)
        devices = [int(t.item()) for t in gathered]
        if len(set(devices)) != len(devices):
            return  # several ranks on one GPU: not a topology this check can judge
        problem = _C.check_nvlink(devices)
        if problem:
            raise RuntimeError(problem)

    # ------------------------------------------------------------------------------------------
    def all_to_all_4d(
        self,
        x: torch.Tensor,
        *,
        mode: int = 0,
        out: torch.Tensor | None = None,
        seq_splits: list[int] | None = None,
        head_splits: list[int] | None = None,
    ) -> torch.Tensor:
        """mode 0 scatters heads and gathers sequence; mode 1 is the inverse.

        Returns a tensor the caller owns. ``out`` from ``empty_output()`` is written by the peers
        directly (no copy-out); any other contiguous tensor of the output shape is copied into.
        ``seq_splits[p]`` / ``head_splits[p]`` are rank p's shards: both or neither, identical on
        every rank. Differentiable (the backward is the other mode with the same splits) unless
        ``out=`` is given.

        Ownership of the returned tensor. By default the result lives in one of three pooled
        symmetric buffers that the peers wrote directly; it behaves like any tensor (views keep it
        alive, it survives ``destroy()``), and its buffer returns to the pool when the last
        reference is dropped. Two rules follow from the memory not belonging to the caching
        allocator: ``Tensor.record_stream()`` has NO effect on it, and a later call on the same
        group may hand the buffer to the peers again as soon as the tensor is dropped. Readers
        queued on the stream that made the call (and on the stream of the next call) are ordered
        automatically; a reader on any other stream must be ordered by the caller before the
        tensor is dropped (``torch.cuda.current_stream().wait_stream(side)``), or the pool
        switched off on every rank with ``set_output_pool(False)``, which restores window +
        copy-out into an ordinary allocation.
        """
        if out is None:
            return _OPS.all_to_all_4d(self._handle, x, mode, seq_splits, head_splits)
        if torch.is_grad_enabled() and x.requires_grad:
            raise RuntimeError(
                "all_to_all_4d(out=...) does not support autograd: the out-variant mutates a buffer you "
                "own and has no backward, so the gradient would be dropped without an error. Drop out=, "
                "or run under torch.no_grad()."
            )
        _OPS.all_to_all_4d_out(self._handle, x, mode, seq_splits, head_splits, out)
        return out

    def all_to_all_4d_async(
        self,
        x: torch.Tensor,
        *,
        mode: int = 0,
        out: torch.Tensor | None = None,
        seq_splits: list[int] | None = None,
        head_splits: list[int] | None = None,
        lend: bool = False,
        stage: bool = True,
    ):
        """``all_to_all_4d`` on the group's high-priority comm stream, returning immediately.

        The result is an ``AsyncCollectiveTensor``: ``.wait()``, or its first use by an aten op,
        makes the caller's stream wait on the comm stream GPU-side. ``lend=True`` returns one of
        four windows the group rotates through (no copy-out, at most four results alive at once).
        Not differentiable.

        ``x`` may be overwritten or freed the moment this returns: by default the call first takes
        a private copy of ``x`` on the caller's stream (``stage=True``, the reference's contract,
        src/group.cc:320-404 there). ``stage=False`` skips that copy and lets the kernel read ``x``
        in place on the comm stream: freeing ``x`` is still safe (the caching allocator is told
        about the cross-stream use), but writing into ``x`` on the caller's stream before waiting
        on the result is then a race the library cannot see.
        """
        if out is not None and lend:
            raise ValueError(
                "all_to_all_4d_async takes out= or lend=True, not both: each is a way to the zero-copy "
                "path, one with a buffer you own and one with a window the group lends."
            )
        if torch.is_grad_enabled() and x.requires_grad:
            raise RuntimeError(
                "all_to_all_4d_async does not support autograd: its result is an AsyncCollectiveTensor, "
                "which is a leaf, so the gradient would be dropped without an error. Use all_to_all_4d()."
            )
        if self.device.type == "cpu":
            y = self.all_to_all_4d(x, mode=mode, out=out, seq_splits=seq_splits, head_splits=head_splits)
            return CompletedHandle(y)

        from torch.distributed._functional_collectives import AsyncCollectiveTensor

        if stage:
            x = x.clone()
        caller = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self._comm_stream):
            if out is None:
                y = _OPS.all_to_all_4d_staged(
                    self._handle, x, mode, seq_splits, head_splits, caller.stream_id, caller.device_index, lend
                )
            else:
                _OPS.all_to_all_4d_staged_out(
                    self._handle, x, mode, seq_splits, head_splits, out, caller.stream_id, caller.device_index
                )
                y = out
        registered = _C.register_stream_completion(y, self._comm_stream.cuda_stream)
        y.record_stream(self._comm_stream)
        y.record_stream(caller)
        return AsyncCollectiveTensor(y) if registered else CompletedHandle(y)

    def empty_output(
        self,
        x: torch.Tensor,
        *,
        mode: int = 0,
        seq_splits: list[int] | None = None,
        head_splits: list[int] | None = None,
    ) -> torch.Tensor:
        """A buffer shaped like this call's output, in symmetric memory. Passing it back as
        ``out=`` makes the peers write it directly. COLLECTIVE: allocate outside the loop."""
        return _OPS.empty_output(self._handle, x, mode, seq_splits, head_splits)

    def _timed(
        self,
        x: torch.Tensor,
        *,
        mode: int = 0,
        seq_splits: list[int] | None = None,
        head_splits: list[int] | None = None,
    ) -> tuple[torch.Tensor, dict[str, float]]:
        """BENCHMARKS ONLY: the copying call with the kernel's own per-phase device timestamps."""
        out, stages = _OPS.all_to_all_4d_timed(self._handle, x, mode, seq_splits, head_splits)
        names = ("barrier_in", "transfer", "barrier_out", "copy_out")
        return out, dict(zip(names, (float(v) for v in stages), strict=True))

    # ------------------------------------------------------------------------------------------
    def barrier(self, *, async_window: bool = False) -> None:
        """Device-side cross-rank barrier on the current stream (bounded wait, see ``check``)."""
        if self.device.type == "cpu":
            if self.pg is not None:
                dist.barrier(group=self.pg)
            return
        self._handle.barrier(1 if async_window else 0)

    def check(self) -> None:
        """Synchronises, then raises if any device-side handshake of this group ran out of time."""
        self._handle.check()

    def set_output_pool(self, enabled: bool) -> None:
        """Whether ``all_to_all_4d(x)`` returns a pooled symmetric buffer that the peers write
        directly (default, no copy-out) or a fresh tensor filled by a copy out of the window.
        Call it with the same value on every rank, between collectives."""
        if self.device.type != "cpu":
            self._handle.set_output_pool(bool(enabled))

    def set_async_transport(self, transport: str) -> None:
        """How ``all_to_all_4d_async`` moves its payload from now on.

        ``"kernel"`` (default): the same persistent kernel as the synchronous call, on a third of
        the SMs. Fastest on its own, but a GEMM running beside it loses those SMs, and a
        persistent GEMM with a fixed tile schedule finishes later by about the whole exchange.
        ``"copy_engine"``: the routes go to the copy engines (one pitched copy per peer and batch)
        between two one-warp handshake kernels, as in the reference (src/transfer.cu:68-126): no
        SM is held while the payload moves, so compute beside the call keeps the device.
        A local choice; ranks may differ (both transports speak the same handshake)."""
        if transport not in ("kernel", "copy_engine"):
            raise ValueError(f"transport must be 'kernel' or 'copy_engine', got {transport!r}")
        if self.device.type != "cpu":
            self._handle.set_async_copy_engine(transport == "copy_engine")

    def destroy(self) -> None:
        """Release the group's windows. Collective. Buffers from ``empty_output()`` are yours."""
        if self._destroyed:
            return
        if self._comm_stream is not None:
            self._comm_stream.synchronize()
        if self.pg is not None and self.world_size > 1:
            dist.barrier(group=self.pg)
        self._handle.destroy()
        self._fp8_window = {}  # the fp8 exchange's cached symmetric window (ops/fp8.py) goes with the group
        self._destroyed = True

    def __del__(self) -> None:
        if not getattr(self, "_destroyed", True) and self._comm_stream is not None:
            try:
                self._comm_stream.synchronize()
            except Exception:
                pass
