"""KV transport over the GPUs' copy engines: an alternative to the NCCL send / receive pairs behind
`GroupCoordinator.p2p_*` (core/group_coordinate.py:643-668 of the reference) for one node.

Why: a KV hop through NCCL point-to-point runs as a kernel on both GPUs.  It needs SMs the attention
kernel would use (an attention CTA fills an SM, so a transfer CTA takes a whole one), and one pair of
ranks moves a chunk at a fraction of what the link can do.  A peer-to-peer `cudaMemcpyAsync` into memory
of the consumer that is mapped into the owner's process (CUDA IPC) is executed by a copy engine: no SM,
full NVLink rate per pair.

How: `PeerCopyGroup` wraps a process group and keeps, per (tag, hop, payload index), TWO receive buffers on
every rank (uses alternate between them), exported once to all peers.  A hop is requested by the consumer
and pushed by the owner:

    consumer, when it posts the receive:  record FREED[b] on its compute stream (whatever read buffer b
              before is queued ahead of it)  ->  post the request (sequence number, b) for that owner
    owner     copy stream:  wait(FREED[b])  ->  wait(payload produced)  ->  peer copy into the consumer's
              buffer b  ->  record READY (interprocess event)  ->  post the sequence number
    consumer  compute stream, before the attention launch that reads the buffer:  wait(READY)

Stream waits on an interprocess event only see records made BEFORE the wait call, so each record is
followed by a host-side sequence number in shared memory and each wait call is preceded by a bounded host
wait for that number: a peer that never posts makes the caller raise after `timeout_s`, it never leaves a
stream waiting on the device for something that will not come.  No kernel spins on anything.

The wrapper has the same p2p interface the attention objects use (`p2p_isend(tensor, dst, slot=...)`,
`p2p_irecv(src, out, slot=...)`, `p2p_commit_batch`, `p2p_wait_batch`) plus `p2p_prepare`, which creates
the slots of a call shape on first use (collective); `p2p_irecv` returns the slot the data will land in
(not `out`).  Everything else is forwarded to the wrapped group.  Mapping and copies go through the C ABI
(dtb_ipc_export_mem / dtb_ipc_open_mem / dtb_peer_copy_async); events are torch's interprocess events.
"""
import time
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..logger import init_logger

logger = init_logger(__name__)


class TransportTimeout(RuntimeError):
    pass


class _Slot:
    """Receive buffers of one (tag, hop, payload index) on THIS rank: two, used alternately."""
    __slots__ = ("index", "uses", "bufs", "freed", "ready_from", "recv_uses")

    def __init__(self, index: int, n: int):
        self.index = index            # row in the shared counter table
        self.uses = 0                 # receives posted into this slot so far (any source): picks the buffer
        self.bufs = None              # [2] tensors
        self.freed = None             # [2] events: everything that read the buffer before has been queued
        self.ready_from = [None] * n  # per source rank: [2] events the source records behind its copy
        self.recv_uses = [0] * n      # per source rank: receives posted from it


class _Remote:
    """What this rank knows about a peer's slot: where its two buffers are mapped here, the peer's FREED
    events and this rank's own READY events for it."""
    __slots__ = ("index", "addr", "freed", "ready", "sends")

    def __init__(self, index: int):
        self.index = index
        self.addr = None              # [2] addresses of the peer's buffers in this process
        self.freed = None             # [2] the peer's events, opened here
        self.ready = None             # [2] events this rank records behind a copy into the peer's buffer
        self.sends = 0                # copies made into this peer's slot so far


class PeerCopyGroup:
    MAX_CHANNELS = 256
    # p2p_wait_batch queues nothing but event waits on the caller's stream (the copies run on the owner's copy stream)
    wait_is_event_only = True

    def __init__(self, group, timeout_s: float = 120.0):
        self.inner = group
        self.world_size = group.world_size
        self.rank_in_group = group.rank_in_group
        self.ranks = group.ranks
        self.device = group.device
        self.local_rank = getattr(group, "local_rank", 0)
        self.unique_name = getattr(group, "unique_name", "group") + "+peer"
        self.timeout_s = timeout_s
        self._ops: List[Tuple] = []
        self._slots: Dict[Tuple, _Slot] = {}        # (tag, hop, i) -> this rank's receive buffers
        self._remote: Dict[Tuple, _Remote] = {}     # (dst, tag, hop, i) -> the peer's
        self._shape: Dict[Tuple, Tuple] = {}        # (tag, hop, i) -> (shape, dtype) the buffers were made for
        self._n_channels = 0
        self._mapped: Dict[bytes, int] = {}         # IPC handle -> base address of the mapping in this process
        self._copy_stream = self._new_stream()
        # counters[owner, consumer, row] = (copies the owner has posted READY for, receives the consumer has
        # requested from that owner, buffer of the latest request); rows are handed out in the order slot
        # kinds are first seen, which is the same on all ranks.
        self._counters = self._shared_counters()

    # ------------------------------------------------------------------ platform hooks (CUDA + CUDA IPC)
    def _new_stream(self):
        return torch.cuda.Stream(device=self.device)

    def _current_stream(self):
        return torch.cuda.current_stream(self.device)

    def _alloc(self, shape, dtype) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype, device=self.device)

    def _export_tensor(self, t: torch.Tensor):
        """(IPC handle of the allocation that holds t, byte offset of t in it)."""
        import ctypes
        from .. import _capi
        handle = (ctypes.c_ubyte * 64)()
        off = ctypes.c_int64(0)
        _capi.check(_capi.load().dtb_ipc_export_mem(t.data_ptr(), handle, ctypes.byref(off)), "dtb_ipc_export_mem")
        return (bytes(handle), int(off.value))

    def _import_tensor(self, handle) -> int:
        """Address, in this process, of the peer buffer behind `handle` (mappings are opened once per allocation)."""
        import ctypes
        from .. import _capi
        raw, off = handle
        base = self._mapped.get(raw)
        if base is None:
            out = ctypes.c_void_p(0)
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(raw)
            _capi.check(_capi.load().dtb_ipc_open_mem(buf, ctypes.byref(out)), "dtb_ipc_open_mem")
            base = self._mapped[raw] = int(out.value)
        return base + off

    def _copy(self, dst, src: torch.Tensor, stream):
        """One asynchronous copy of src into the peer buffer dst on `stream` (a copy engine executes it)."""
        from .. import _capi
        if not src.is_contiguous():
            raise RuntimeError("PeerCopyGroup sends contiguous tensors only")
        _capi.check(_capi.load().dtb_peer_copy_async(dst, src.data_ptr(), src.numel() * src.element_size(),
                                                     stream.cuda_stream), "dtb_peer_copy_async")

    def _new_event(self):
        return torch.cuda.Event(enable_timing=False, interprocess=True)

    def _export_event(self, ev):
        return ev.ipc_handle()

    def _import_event(self, handle):
        # opened under THIS rank's device: no context is created on the peer's GPU
        return torch.cuda.Event.from_ipc_handle(self.device, handle)

    def _exchange(self, obj) -> list:
        import torch.distributed as dist
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self.inner.cpu_group)
        return out

    def _shared_counters(self) -> np.ndarray:
        """int64 [N, N, MAX_CHANNELS, 4] in shared memory, created by group rank 0."""
        from multiprocessing import shared_memory
        n = self.world_size
        nbytes = n * n * self.MAX_CHANNELS * 4 * 8
        if self.rank_in_group == 0:
            shm = shared_memory.SharedMemory(create=True, size=nbytes)
            np.ndarray((nbytes // 8,), dtype=np.int64, buffer=shm.buf)[:] = 0
            names = self._exchange(shm.name)
        else:
            names = self._exchange(None)
            shm = shared_memory.SharedMemory(name=names[0])
            try:        # this process only attached: the creator unlinks the segment, nobody else should try to
                from multiprocessing import resource_tracker
                resource_tracker.unregister(shm._name, "shared_memory")
            except Exception:
                pass
        self._shm = shm
        self._shm_owner = self.rank_in_group == 0
        return np.ndarray((n, n, self.MAX_CHANNELS, 4), dtype=np.int64, buffer=shm.buf)

    # ------------------------------------------------------------------ slots
    def _ensure_slots(self, tag: str, hop: int, i: int, like: torch.Tensor):
        """Create (or re-create after a shape change) this rank's buffers for (tag, hop, i) and learn every
        peer's.  Collective over the group: all ranks reach it at the same call, since they run the same plan
        on equally shaped chunks."""
        key = (tag, hop, i)
        want = (tuple(like.shape), like.dtype)
        if self._shape.get(key) == want:
            return
        me, n = self.rank_in_group, self.world_size
        slot = self._slots.get(key)
        if slot is None:
            if self._n_channels >= self.MAX_CHANNELS:
                raise RuntimeError("PeerCopyGroup: more slot kinds than counter rows")
            slot = self._slots[key] = _Slot(self._n_channels, n)
            self._n_channels += 1
            slot.freed = [self._new_event() for _ in range(2)]
        else:
            # A new shape for a known slot: counts, events and counter rows carry on, only the buffers are
            # replaced -- once every rank's copies into the old ones have completed.
            self._copy_stream.synchronize()
            self._current_stream().synchronize()
            self.inner.barrier()
        self._shape[key] = want
        slot.bufs = [self._alloc(*want) for _ in range(2)]
        ready = {}
        for dst in range(n):
            if dst == me:
                continue
            rem = self._remote.get((dst,) + key)
            if rem is None:
                rem = self._remote[(dst,) + key] = _Remote(slot.index)
                rem.ready = [self._new_event() for _ in range(2)]
            ready[dst] = [self._export_event(e) for e in rem.ready]
        mine = ([self._export_tensor(t) for t in slot.bufs], [self._export_event(e) for e in slot.freed], ready)
        everyone = self._exchange(mine)
        for peer in range(n):
            if peer == me:
                continue
            bufs_h, freed_h, ready_h = everyone[peer]
            rem = self._remote[(peer,) + key]
            rem.addr = [self._import_tensor(h) for h in bufs_h]
            rem.freed = [self._import_event(h) for h in freed_h]
            slot.ready_from[peer] = [self._import_event(h) for h in ready_h[me]]

    # ------------------------------------------------------------------ point to point
    def p2p_prepare(self, tag: str, payload, n_hops: int):
        """Make sure slots exist for every hop and payload tensor of a call shaped like `payload`.
        Collective over the group (a cheap look-up after the first call with a shape); every rank calls it
        with the same arguments before it queues the hops of a layer call."""
        for hop in range(n_hops):
            for i, t in enumerate(payload):
                self._ensure_slots(tag, hop, i, t)

    def p2p_isend(self, tensor: torch.Tensor, dst: Optional[int] = None, slot: Optional[Tuple[str, int, int]] = None):
        if dst is None:
            dst = (self.rank_in_group + 1) % self.world_size
        assert slot is not None, "PeerCopyGroup needs the slot a tensor is sent into"
        self._ops.append(("send", dst, slot, tensor))

    def p2p_irecv(self, size=None, dtype=None, src: Optional[int] = None, out: Optional[torch.Tensor] = None,
                  slot: Optional[Tuple[str, int, int]] = None):
        if src is None:
            src = (self.rank_in_group - 1) % self.world_size
        assert slot is not None, "PeerCopyGroup needs the slot a tensor is received into"
        sl = self._slots[slot]
        b = sl.uses & 1
        sl.uses += 1
        seq = sl.recv_uses[src] = sl.recv_uses[src] + 1
        self._ops.append(("recv", src, sl, b, seq))
        return sl.bufs[b]

    def _host_wait(self, cell: np.ndarray, col: int, at_least: int, what: str):
        if cell[col] >= at_least:
            return
        t0 = time.monotonic()
        spins = 0
        while cell[col] < at_least:
            spins += 1
            if spins > 200:
                time.sleep(0)              # let the other ranks' threads / processes run
            if time.monotonic() - t0 > self.timeout_s:
                raise TransportTimeout(f"{self.unique_name}: {what} not posted within {self.timeout_s} s "
                                       f"(have {int(cell[col])}, need {at_least})")

    def p2p_commit_batch(self):
        """Post the queued receives (requests to their owners), then start the queued sends (peer copies on
        the copy stream).  Returns a handle for the receives."""
        me = self.rank_in_group
        ops, self._ops = self._ops, []
        cur = self._current_stream()
        recvs = [op for op in ops if op[0] == "recv"]
        for _, src, sl, b, seq in recvs:
            sl.freed[b].record(cur)                      # behind every kernel queued so far that read buffer b
            cell = self._counters[src, me, sl.index]
            cell[2] = b
            cell[1] = seq                                # the request: visible to the owner from here on
        sends = [op for op in ops if op[0] == "send"]
        if sends:
            produced = self._new_local_event()
            produced.record(cur)
            for _, dst, slot, tensor in sends:
                rem = self._remote[(dst,) + tuple(slot)]
                rem.sends += 1
                cell = self._counters[me, dst, rem.index]
                self._host_wait(cell, 1, rem.sends, f"request {rem.sends} for slot {slot} by rank {dst}")
                b = int(cell[2])
                self._copy_stream.wait_event(rem.freed[b])
                self._copy_stream.wait_event(produced)
                self._copy(rem.addr[b], tensor, self._copy_stream)
                rem.ready[b].record(self._copy_stream)
                cell[0] = rem.sends
                self._keep_alive(tensor)
        return recvs

    def p2p_wait_batch(self, recvs):
        me = self.rank_in_group
        cur = self._current_stream()
        for _, src, sl, b, seq in recvs or []:
            self._host_wait(self._counters[src, me, sl.index], 0, seq, f"chunk {seq} from rank {src}")
            cur.wait_event(sl.ready_from[src][b])

    def _new_local_event(self):
        return torch.cuda.Event(enable_timing=False)

    def _keep_alive(self, tensor: torch.Tensor):
        # the copy stream reads it; the caching allocator must not hand its memory out before that
        tensor.record_stream(self._copy_stream)

    # one-batch form of the reference interface
    def p2p_commit(self):
        self._pending = self.p2p_commit_batch()

    def p2p_wait(self):
        self.p2p_wait_batch(self._pending)
        self._pending = None

    # ------------------------------------------------------------------ everything else
    def __getattr__(self, name):
        return getattr(self.inner, name)

    def close(self):
        for base in getattr(self, "_mapped", {}).values():
            from .. import _capi
            _capi.load().dtb_ipc_close_mem(base)
        self._mapped = {}
        shm = getattr(self, "_shm", None)
        if shm is not None:
            shm.close()
            if self._shm_owner:
                try:
                    shm.unlink()
                except FileNotFoundError:
                    pass
            self._shm = None
