"""Peer windows: persistent halo buffers every rank of the node can store into.

The reference moves halo rows through its transport's grouped send / recv
(python/tiga/distributed/nccl.py:256-284 of walkerchi/TIGA-lang; python/tiga/distributed/transport.py:
1060-1133 pack, 446-574 reverse).  With all ranks on one NVSwitch node the rows need not pass
through a pack buffer and a library copy: the sender's row mover (``tgb_rows_gather``) stores the rows
it gathers straight into the receiver's ghost buffer, whose address it holds through CUDA IPC, and a
one-element all-reduce on the communication stream tells every rank that all stores of a wave have
been issued and completed.  No kernel of this package ever waits on another GPU: ordering is by
streams and by that collective only.

A window is a ring of ``slots`` buffers per rank (one forward call uses one slot and keeps it until
its backward has read it).  Everything here is collective: all ranks create windows and acquire
slots in the same order, which holds because they run the same program.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _native


def _export(tensor: torch.Tensor):
    handle = (ctypes.c_ubyte * 64)()
    offset = ctypes.c_uint64()
    _native.check(_native.lib().tgb_peer_export(tensor.data_ptr(), handle, ctypes.byref(offset)), "tgb_peer_export")
    return bytes(handle), int(offset.value)


class PeerWindow:
    """``slots`` buffers of ``slot_bytes`` on this rank plus the addresses of every peer's buffers.

    ``layout`` is a small picklable description this rank publishes with its buffer (where a peer's
    rows go inside a slot); ``peer_layout[p]`` is what rank p published."""

    def __init__(self, transport, device, slot_bytes: int, slots: int, layout):
        self.transport = transport
        self.rank, self.world = transport.rank, transport.world_size
        self.slots = int(slots)
        self.slot_bytes = (int(slot_bytes) + 255) // 256 * 256
        self.local = torch.empty(max(self.slot_bytes * self.slots, 256), dtype=torch.uint8, device=device)
        handle, offset = _export(self.local)
        published = [None] * self.world
        dist.all_gather_object(published, (handle, offset, self.slot_bytes, layout), group=transport.group)
        self.peer_layout = [entry[3] for entry in published]
        self.peer_slot_bytes = [entry[2] for entry in published]
        self._mapped = []
        self.peer_base = []
        lib = _native.lib()
        for peer, (peer_handle, peer_offset, _, _) in enumerate(published):
            if peer == self.rank:
                self.peer_base.append(self.local.data_ptr())
                continue
            buffer = (ctypes.c_ubyte * 64).from_buffer_copy(peer_handle)
            mapped = ctypes.c_uint64()
            with torch.cuda.device(device):
                _native.check(lib.tgb_peer_open(buffer, ctypes.byref(mapped)), "tgb_peer_open")
            self._mapped.append(int(mapped.value))
            self.peer_base.append(int(mapped.value) + peer_offset)
        self._next = 0
        self.busy = [False] * self.slots                 # a forward holds its slot until its backward is done
        self.released = [None] * self.slots              # event on the compute stream: this rank's last read

    def address(self, peer: int, slot: int, byte_offset: int = 0) -> int:
        return self.peer_base[peer] + slot * self.peer_slot_bytes[peer] + byte_offset

    def view(self, slot: int, shape, dtype=torch.float32) -> torch.Tensor:
        count = 1
        for extent in shape:
            count *= extent
        start = slot * self.slot_bytes
        return self.local[start:start + count * torch.empty(0, dtype=dtype).element_size()].view(dtype).reshape(shape)

    def acquire(self) -> int | None:
        """Next slot of the ring, or None when it is still held (the caller then takes another path).
        Deterministic across ranks: they all make the same calls in the same order."""
        slot = self._next
        if self.busy[slot]:
            return None
        self._next = (slot + 1) % self.slots
        self.busy[slot] = True
        return slot

    def release(self, slot: int, stream) -> None:
        self.released[slot] = stream.record_event()
        self.busy[slot] = False

    def close(self) -> None:
        lib = _native.lib()
        for mapped in self._mapped:
            lib.tgb_peer_close(mapped)
        self._mapped = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class PushSignals:
    """Stream-ordered "everyone has got this far" on the communication stream: a one-element
    all-reduce.  Issued after a rank's stores of a wave, its completion on a rank means that every
    rank has finished the stores it enqueued before its own call."""

    def __init__(self, transport, device):
        self.transport = transport
        self.token = torch.zeros(1, dtype=torch.float32, device=device)

    def barrier(self) -> None:
        dist.all_reduce(self.token, op=dist.ReduceOp.SUM, group=self.transport.group)


def push_rows(rows: torch.Tensor, ids: torch.Tensor, address: int) -> None:
    """packed rows ``rows[ids]`` written at ``address`` (a peer's or this rank's device memory)."""
    with torch.cuda.device(rows.device):
        _native.check(_native.lib().tgb_rows_gather(rows.data_ptr(), ids.data_ptr(), address, ids.numel(),
                                                    rows.shape[1], torch.cuda.current_stream(rows.device).cuda_stream),
                      "tgb_rows_gather")


def push_block(block: torch.Tensor, address: int) -> None:
    """A contiguous block copied to ``address``."""
    with torch.cuda.device(block.device):
        _native.check(_native.lib().tgb_peer_copy(address, block.data_ptr(), block.numel() * block.element_size(),
                                                  torch.cuda.current_stream(block.device).cuda_stream),
                      "tgb_peer_copy")


__all__ = ["PeerWindow", "PushSignals", "push_block", "push_rows"]
