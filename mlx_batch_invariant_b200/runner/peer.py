"""Feature-slice all-gather over peer memory for the sharded decoder (host side of ``bi_push_gather``).

Every rank allocates one block of device memory through the library (``bi_peer_alloc``: a CUDA IPC handle
can name it), sends the handle to the other ranks over the process group, and maps theirs. A gather is
then one kernel launch per rank that stores the local slice into every rank's destination and shakes
hands through flag words (``csrc/peer.cu``); the result is already in ``[rows, world * f]`` order.

Destination buffers rotate: a peer can be one gather ahead of the slowest rank, never two, so three
buffers are enough in a straight run. A captured CUDA graph replays a fixed sequence of ``n`` gathers;
the rotation modulus is then chosen so that the last gather of one replay and the first of the next
use different buffers (``set_cycle``).
"""

from __future__ import annotations

import ctypes

import torch

from .. import _lib

NBUF = 7          # allocated destinations; 3, 4, 5 or 7 of them are cycled through


def pick_cycle(n: int, mod: int, calls: int) -> tuple[int, int]:
    """Rotation (modulus, call counter) for a sequence of n gathers that will be replayed back to back.

    The buffer of call c is c % modulus. The modulus is the smallest of 3, 4, 5, 7 for which the last gather of
    one replay and the first of the next use different buffers (n % modulus != 1), and the counter is
    re-based so that the first gather of the sequence does not reuse the buffer of the gather before it."""
    if n == 1:
        raise RuntimeError("a replayed sequence of ONE gather would reuse one destination buffer every replay, which a "
                           "peer that is one gather ahead may still be writing: capture at least two gathers per replay, "
                           "or run the step eagerly")
    prev = (calls - 1) % mod if calls else -1
    for m in (3, 4, 5, 7):
        if n % m != 1:
            return m, prev + 1
    raise RuntimeError(f"no buffer rotation for a cycle of {n} gathers")


class PeerUnavailable(RuntimeError):
    """Some pair of ranks cannot map each other's memory; raised on every rank of the group together."""


class _Raw:
    """A device pointer as something torch.as_tensor can wrap (no copy, no ownership)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PushGather:
    def __init__(self, group, rank: int, world: int, device: torch.device, max_bytes: int):
        import torch.distributed as dist
        self.rank, self.world, self.dev = rank, world, device
        self.lib = _lib.load()
        self.cap = (max_bytes + 255) // 256 * 256                 # bytes of one gathered destination
        total = NBUF * self.cap + 256                             # + the flag array (uint32[world])
        with torch.cuda.device(device):
            base = ctypes.c_void_p()
            _lib.check(self.lib.bi_peer_alloc(ctypes.byref(base), total))
            handle = ctypes.create_string_buffer(64)
            _lib.check(self.lib.bi_peer_export(base, handle))
            handles = [None] * world
            dist.all_gather_object(handles, handle.raw, group=group)
            self.bases, failure = [], None
            for r in range(world):
                if r == rank:
                    self.bases.append(base.value)
                    continue
                p = ctypes.c_void_p()
                try:
                    _lib.check(self.lib.bi_peer_open(handles[r], ctypes.byref(p)))
                except _lib.KernelError as e:           # no peer mapping to rank r from here (no NVLink / IPC between the two)
                    failure = failure or f"rank {rank} cannot map rank {r}'s buffer: {e}"
                self.bases.append(p.value)
            # Every rank must reach the same conclusion, or the ones that succeeded would wait for the others forever.
            outcomes = [None] * world
            dist.all_gather_object(outcomes, failure, group=group)
            if any(outcomes):
                for r, b in enumerate(self.bases):
                    if r != rank and b:
                        self.lib.bi_peer_close(ctypes.c_void_p(b))
                self.lib.bi_peer_free(base)
                raise PeerUnavailable("; ".join(v for v in outcomes if v))
            self.own = [torch.as_tensor(_Raw(base.value + b * self.cap, self.cap), device=device) for b in range(NBUF)]
            self.counters = torch.zeros(2, dtype=torch.int32, device=device)
        self.calls = 0
        self.mod = 3
        dist.barrier(group=group)                                 # every rank has mapped every buffer

    def fits(self, rows: int, row_bytes: int) -> bool:
        return rows * row_bytes * self.world <= self.cap and row_bytes % 16 == 0

    def set_cycle(self, n: int) -> None:
        """A sequence of n gathers is about to be replayed back to back: pick the rotation modulus. One captured
        sequence per PushGather: capturing a second one re-bases the rotation under the graph already recorded,
        so build a new PushGather (a new ShardedDecoder) for a second graph."""
        if getattr(self, "_cycle_set", False):
            raise RuntimeError("this PushGather already serves a captured sequence of gathers; a second capture needs its own")
        self._cycle_set = True
        self.mod, self.calls = pick_cycle(n, self.mod, self.calls)

    def _slot(self):
        """Destination and flag pointer tables of the next gather, and its buffer index."""
        b = self.calls % self.mod
        self.calls += 1
        arr = ctypes.c_void_p * self.world
        return b, arr(*[base + b * self.cap for base in self.bases]), arr(*[base + NBUF * self.cap for base in self.bases])

    def awaiting(self):
        """What a consumer kernel needs to wait for the gather just issued with wait=False: this rank's flag
        array, the device word holding the gather's epoch, rank and world (the trailing arguments of the
        *_awaiting entry points)."""
        return (self.bases[self.rank] + NBUF * self.cap, self.counters.data_ptr() + 4, self.rank, self.world)

    def sink(self, rows: int, cols: int, dtype: torch.dtype, wait: bool = True):
        """The next gather, for a kernel that pushes its own output (``push=`` of the matmuls and of decode
        attention): returns (push arguments, the local [rows, world * cols] destination). The kernel given the
        arguments is the gather: it must be launched next on the stream. wait=False: see gather()."""
        b, dst, flags = self._slot()
        n = rows * cols * torch.empty(0, dtype=dtype).element_size() * self.world
        view = self.own[b][:n].view(dtype).view(rows, self.world * cols)
        return (dst, flags, self.counters.data_ptr(), self.rank, self.world, int(wait)), view

    def gather_swiglu(self, gate_up: torch.Tensor, wait: bool = True) -> torch.Tensor:
        """gate_up[rows, 2F] of this rank -> swiglu of every rank's slice, [rows, world * F]: the gate is computed
        while the slice is pushed (one launch; same bits as swiglu followed by gather). wait=False: see gather()."""
        rows, f2 = gate_up.shape
        F = f2 // 2
        b, dst, flags = self._slot()
        status = _lib.status_word(self.dev)
        _lib.check(self.lib.bi_push_gather_swiglu(gate_up.data_ptr(), dst, flags, self.counters.data_ptr(), rows, F,
                                                  _lib.DTYPE_CODE[gate_up.dtype], self.rank, self.world, int(wait), status.data_ptr(),
                                                  _lib.stream_ptr(self.dev)))
        n = rows * F * gate_up.element_size() * self.world
        return self.own[b][:n].view(gate_up.dtype).view(rows, self.world * F)

    def gather(self, local: torch.Tensor, wait: bool = True) -> torch.Tensor:
        """local[rows, f] (contiguous) -> [rows, world * f], rank-major along the feature axis. wait=False: the
        kernel does not wait for the peers' slices; the NEXT kernel on the stream that reads the result must be
        an *_awaiting one given ``self.awaiting()``."""
        rows, f = local.shape
        row_bytes = f * local.element_size()
        b, dst, flags = self._slot()
        status = _lib.status_word(self.dev)
        _lib.check(self.lib.bi_push_gather(local.data_ptr(), dst, flags, self.counters.data_ptr(), rows, row_bytes,
                                           self.rank, self.world, int(wait), status.data_ptr(), _lib.stream_ptr(self.dev)))
        n = rows * row_bytes * self.world
        return self.own[b][:n].view(local.dtype).view(rows, self.world * f)
