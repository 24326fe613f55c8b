"""N logical ranks of a sequence-parallel group inside ONE process: a test-side stand-in for
GroupCoordinator whose transport is a set of in-memory mailboxes.

Every logical rank runs in its own Python thread with its own group object, its own attention objects
and its own cache, exactly as a process would; `p2p_isend` puts a tensor reference into the mailbox of
the (source, destination) pair, `p2p_wait_batch` copies it into the receiver's slot with `out.copy_()`
on the current stream.  All threads launch on the same stream of the same device, so the device
executes the ranks' kernels in the order the host issued them and no cross-stream events are needed.
With this group the whole reuse path -- cached blocks, first-KV exchange, accumulate into a stored
block, re-blocking merges, pair maps, the Ulysses exchange -- runs on real kernels on a single GPU.

The interface is the subset of core/group_coordinate.py (reference and this package) that the
attention path uses: world_size, rank_in_group, ranks, device, p2p_isend / p2p_irecv /
p2p_commit_batch / p2p_wait_batch (and the one-batch p2p_commit / p2p_wait), all_to_all_single,
all_to_all, all_gather, all_reduce, barrier.
"""
import threading
from typing import Callable, List, Optional

import torch


class LoopbackFabric:
    def __init__(self, world: int, timeout_s: float = 120.0):
        self.world = world
        self.timeout_s = timeout_s
        self.cv = threading.Condition()
        self.mail = {}            # (src, dst, sequence) -> tensor posted by src
        self.consumed = set()     # (src, dst, sequence) whose copy has been queued by dst
        self.coll = {}            # (kind, sequence) -> {rank: tensor}
        self.failure: Optional[BaseException] = None
        self._barrier = threading.Barrier(world)

    def group(self, rank: int, device=None) -> "LoopbackGroup":
        return LoopbackGroup(self, rank, device)

    def abort(self, exc: BaseException):
        with self.cv:
            if self.failure is None:
                self.failure = exc
            self.cv.notify_all()
        self._barrier.abort()

    def wait_for(self, predicate: Callable[[], bool], what: str):
        """Block (condition held by the caller) until predicate() or a failure elsewhere."""
        ok = self.cv.wait_for(lambda: predicate() or self.failure is not None, timeout=self.timeout_s)
        if self.failure is not None:
            raise RuntimeError(f"another logical rank failed: {self.failure!r}")
        if not ok:
            raise TimeoutError(f"loopback transport: {what} did not happen within {self.timeout_s} s")

    def barrier(self):
        try:
            self._barrier.wait(timeout=self.timeout_s)
        except threading.BrokenBarrierError:
            raise RuntimeError(f"loopback barrier broken: {self.failure!r}")


class LoopbackGroup:
    def __init__(self, fabric: LoopbackFabric, rank: int, device=None):
        self.fabric = fabric
        self.world_size = fabric.world
        self.rank_in_group = rank
        self.ranks = list(range(fabric.world))
        self.local_rank = 0
        self.unique_name = f"loopback{rank}"
        self.device = device if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self._send_seq = [0] * fabric.world      # next sequence number towards each destination
        self._recv_seq = [0] * fabric.world      # next sequence number from each source
        self._ops = []
        self._reqs = None
        self._coll_seq = 0

    # ------------------------------------------------------------------ point to point
    def p2p_isend(self, tensor: torch.Tensor, dst: Optional[int] = None, slot=None):
        if dst is None:
            dst = (self.rank_in_group + 1) % self.world_size
        key = (self.rank_in_group, dst, self._send_seq[dst])
        self._send_seq[dst] += 1
        self._ops.append(("send", key, tensor))

    def p2p_irecv(self, size=None, dtype=None, src: Optional[int] = None, out: Optional[torch.Tensor] = None, slot=None):
        if src is None:
            src = (self.rank_in_group - 1) % self.world_size
        tensor = out if out is not None else torch.empty(size, dtype=dtype, device=self.device)
        key = (src, self.rank_in_group, self._recv_seq[src])
        self._recv_seq[src] += 1
        self._ops.append(("recv", key, tensor))
        return tensor

    def p2p_commit_batch(self):
        ops, self._ops = self._ops, []
        f = self.fabric
        with f.cv:
            for kind, key, tensor in ops:
                if kind == "send":
                    f.mail[key] = tensor
            f.cv.notify_all()
        return ops

    def p2p_wait_batch(self, ops):
        """Receives first (they depend only on the peers having posted), then wait until every send of
        the batch has been picked up, so the sender's tensors stay untouched until they were copied."""
        f = self.fabric
        if ops:
            try:                                   # the CPU engine's op record, when a test has switched it on
                from tests.cpu_engine import log_op
                log_op("wait")
            except ImportError:
                pass
        for kind, key, tensor in ops or []:
            if kind != "recv":
                continue
            with f.cv:
                f.wait_for(lambda: key in f.mail, f"send {key}")
                src_tensor = f.mail.pop(key)
            tensor.copy_(src_tensor)
            with f.cv:
                f.consumed.add(key)
                f.cv.notify_all()
        for kind, key, tensor in ops or []:
            if kind != "send":
                continue
            with f.cv:
                f.wait_for(lambda: key in f.consumed, f"pick-up of {key}")
                f.consumed.discard(key)

    def p2p_commit(self):
        assert self._reqs is None, "a point-to-point batch is already in flight"
        self._reqs = self.p2p_commit_batch()

    def p2p_wait(self):
        self.p2p_wait_batch(self._reqs)
        self._reqs = None

    # ------------------------------------------------------------------ collectives
    def _exchange(self, kind: str, tensor: torch.Tensor) -> List[torch.Tensor]:
        """Every rank deposits one tensor; returns all of them in rank order once complete."""
        f = self.fabric
        key = (kind, self._coll_seq)
        self._coll_seq += 1
        self._last_key = key
        with f.cv:
            f.coll.setdefault(key, {})[self.rank_in_group] = tensor
            f.cv.notify_all()
            f.wait_for(lambda: len(f.coll[key]) == self.world_size, f"collective {key}")
            parts = [f.coll[key][r] for r in range(self.world_size)]
        return parts

    def _done(self):
        # nobody's deposit may be released before every rank has queued its copies
        self.fabric.barrier()
        with self.fabric.cv:
            self.fabric.coll.pop(self._last_key, None)

    def all_to_all_single(self, output: torch.Tensor, input_: torch.Tensor):
        parts = self._exchange("a2a", input_)
        for src, p in enumerate(parts):
            output[src].copy_(p[self.rank_in_group])
        self._done()

    def all_to_all(self, input_: torch.Tensor, scatter_dim: int = 2, gather_dim: int = 1) -> torch.Tensor:
        if self.world_size == 1:
            return input_
        parts = self._exchange("a2a_t", input_)
        mine = [torch.tensor_split(p, self.world_size, scatter_dim)[self.rank_in_group] for p in parts]
        out = torch.cat(mine, dim=gather_dim).contiguous()
        self._done()
        return out

    def all_gather(self, input_: torch.Tensor, dim: int = -1, split: bool = False):
        if self.world_size == 1:
            return [input_] if split else input_
        parts = [p.clone() for p in self._exchange("gather", input_)]
        self._done()
        if split:
            return parts
        return torch.cat(parts, dim=dim)

    def all_reduce(self, input_: torch.Tensor) -> torch.Tensor:
        parts = self._exchange("reduce", input_.clone())
        total = torch.stack(parts).sum(0)
        self._done()
        input_.copy_(total)
        return input_

    def barrier(self):
        self.fabric.barrier()


def run_ranks(world: int, body: Callable[[int, LoopbackGroup, LoopbackFabric], object], timeout_s: float = 120.0,
              prepare: Optional[Callable[[int, LoopbackGroup], object]] = None):
    """Run body(rank, group, fabric) on `world` threads; returns the list of results, or raises the
    first exception any rank raised.  `prepare(rank, group)`, if given, runs for every rank in the calling
    thread before the threads start (anything that draws from the process-wide random generator belongs
    there); its result is left in group.context."""
    fabric = LoopbackFabric(world, timeout_s)
    results = [None] * world
    errors = []
    device = torch.cuda.current_device() if torch.cuda.is_available() else None
    groups = [fabric.group(r) for r in range(world)]
    for r, g in enumerate(groups):
        g.context = prepare(r, g) if prepare is not None else None

    def target(r):
        try:
            if device is not None:
                torch.cuda.set_device(device)
            results[r] = body(r, groups[r], fabric)
        except BaseException as e:  # noqa: BLE001 - surfaced to the caller below
            errors.append((r, e))
            fabric.abort(e)

    threads = [threading.Thread(target=target, args=(r,), daemon=True) for r in range(world)]
    for th in threads:
        th.start()
    for th in threads:
        th.join(timeout_s * 4)
    if errors:
        raise errors[0][1]          # the first one raised; later ones are its echoes on other ranks
    if any(th.is_alive() for th in threads):
        raise TimeoutError("a logical rank is still running")
    return results


def stepped(fabric: LoopbackFabric, rank: int, t: int):
    """All ranks enter denoising step t together: the step index is a process-wide global that every
    attention call reads on entry."""
    from ditango_b200.utils import update_timestep
    fabric.barrier()
    if rank == 0:
        update_timestep(t)
    fabric.barrier()


# ---------------------------------------------------------------------------------------------------
# The copy-engine transport (ditango_b200/core/peer_transport.py) on threads: same protocol code --
# requests, sequence numbers, buffer alternation, bounded host waits -- with the platform hooks (device
# memory, CUDA IPC, interprocess events, the shared counter table) replaced by in-process stand-ins.
class _NullEvent:
    def record(self, stream=None):
        pass


class _NullStream:
    def wait_event(self, ev):
        pass

    def synchronize(self):
        pass


def thread_peer_group(group: "LoopbackGroup", timeout_s: float = 30.0):
    """PeerCopyGroup over a LoopbackGroup with CPU tensors: buffers are shared by reference, copies are
    synchronous `copy_` calls, events are no-ops (every operation has completed when the host call returns)."""
    import numpy as np
    from ditango_b200.core.peer_transport import PeerCopyGroup

    fabric = group.fabric

    class ThreadPeerGroup(PeerCopyGroup):
        def _new_stream(self):
            return _NullStream()

        def _current_stream(self):
            return _NullStream()

        def _alloc(self, shape, dtype):
            return torch.empty(shape, dtype=dtype)

        def _export_tensor(self, t):
            return t

        def _import_tensor(self, handle):
            return handle

        def _copy(self, dst, src, stream):
            dst.copy_(src)

        def _new_event(self):
            return _NullEvent()

        def _new_local_event(self):
            return _NullEvent()

        def _export_event(self, ev):
            return ev

        def _import_event(self, handle):
            return handle

        def _keep_alive(self, tensor):
            pass

        def _exchange(self, obj):
            return _exchange_objects(self.inner, obj)

        def _shared_counters(self):
            with fabric.cv:
                table = getattr(fabric, "peer_counters", None)
                if table is None:
                    n = fabric.world
                    table = fabric.peer_counters = np.zeros((n, n, self.MAX_CHANNELS, 4), dtype=np.int64)
            self._shm = None
            return table

    return ThreadPeerGroup(group, timeout_s=timeout_s)


def _exchange_objects(group: "LoopbackGroup", obj):
    """all_gather_object among the logical ranks."""
    f = group.fabric
    key = ("obj", group._coll_seq)
    group._coll_seq += 1
    with f.cv:
        f.coll.setdefault(key, {})[group.rank_in_group] = obj
        f.cv.notify_all()
        f.wait_for(lambda: len(f.coll[key]) == group.world_size, f"object exchange {key}")
        parts = [f.coll[key][r] for r in range(group.world_size)]
    f.barrier()
    with f.cv:
        f.coll.pop(key, None)
    return parts
