"""Process-group wrapper with the reference's GroupCoordinator interface
(core/group_coordinate.py of the reference): one device group (NCCL on GPUs, gloo on CPU ranks) plus
one gloo group per coordinator, group-local ranks, and the collectives the attention path uses --
batched point-to-point (`p2p_isend / p2p_irecv / p2p_commit / p2p_wait`, :643-668), `all_to_all`
(:281-286), `all_gather` (:159-184), `all_reduce`, `barrier` (:609-616)."""
from typing import List, Optional

import torch
import torch.distributed as dist


class GroupCoordinator:
    # p2p_wait_batch only makes the current stream wait for events (torch's Work.wait on NCCL requests): no kernel
    # or copy of the transport is queued between the caller's own launches.  proAttention reads this.
    wait_is_event_only = True

    def __init__(self, group_ranks: List[List[int]], local_rank: int, torch_distributed_backend: str,
                 group_name: Optional[str] = None):
        self.unique_name = group_name or "anonymous"
        self.rank = dist.get_rank()
        self.local_rank = local_rank
        self.device_group = None
        self.cpu_group = None
        self.p2p_ops = []
        self.p2p_reqs = None
        pg_options = None
        if torch_distributed_backend == "nccl":
            # NCCL's transfer kernels run on a high-priority stream: when an SM frees up they are placed
            # ahead of the attention kernel's remaining CTAs, so a KV hop overlaps the attention on
            # the chunk that is already here instead of queueing behind it.
            pg_options = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        for ranks in group_ranks:
            device_group = dist.new_group(ranks, backend=torch_distributed_backend, pg_options=pg_options)
            cpu_group = dist.new_group(ranks, backend="gloo")
            if self.rank in ranks:
                self.ranks = list(ranks)
                self.world_size = len(ranks)
                self.rank_in_group = ranks.index(self.rank)
                self.device_group = device_group
                self.cpu_group = cpu_group
        assert self.cpu_group is not None and self.device_group is not None
        on_gpu = torch_distributed_backend != "gloo" and torch.cuda.is_available()
        self.device = torch.device(f"cuda:{local_rank}") if on_gpu else torch.device("cpu")

    @property
    def first_rank(self):
        return self.ranks[0]

    @property
    def last_rank(self):
        return self.ranks[-1]

    @property
    def is_first_rank(self):
        return self.rank == self.first_rank

    @property
    def is_last_rank(self):
        return self.rank == self.last_rank

    @property
    def next_rank(self):
        return self.ranks[(self.rank_in_group + 1) % self.world_size]

    @property
    def prev_rank(self):
        return self.ranks[(self.rank_in_group - 1) % self.world_size]

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, input_: torch.Tensor) -> torch.Tensor:
        if self.world_size > 1:
            dist.all_reduce(input_, group=self.device_group)
        return input_

    def all_gather(self, input_: torch.Tensor, dim: int = -1, split: bool = False):
        if self.world_size == 1:
            return input_
        if dim < 0:
            dim += input_.dim()
        out = torch.empty((self.world_size,) + tuple(input_.shape), dtype=input_.dtype, device=input_.device)
        flat = out.view((self.world_size * input_.shape[0],) + tuple(input_.shape[1:])) if input_.dim() > 0 else out
        dist.all_gather_into_tensor(flat, input_.contiguous(), group=self.device_group)
        if split:
            return [out[i] for i in range(self.world_size)]
        if dim != 0:
            out = out.movedim(0, dim)
        shape = list(input_.shape)
        shape[dim] *= self.world_size
        return out.reshape(shape)

    def all_to_all(self, input_: torch.Tensor, scatter_dim: int = 2, gather_dim: int = 1) -> torch.Tensor:
        """Rank r receives the r-th split (along scatter_dim) of every rank's tensor, concatenated
        along gather_dim in rank order."""
        if self.world_size == 1:
            return input_
        parts = torch.tensor_split(input_, self.world_size, scatter_dim)
        if all(p.shape == parts[0].shape for p in parts):
            send = torch.stack(parts)                       # one packed buffer, one equal-split exchange
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=self.device_group)
            return torch.cat(list(recv.unbind(0)), dim=gather_dim).contiguous()
        ins = [t.contiguous() for t in parts]
        outs = [torch.empty_like(t) for t in ins]
        dist.all_to_all(outs, ins, group=self.device_group)
        return torch.cat(outs, dim=gather_dim).contiguous()

    def all_to_all_single(self, output: torch.Tensor, input_: torch.Tensor):
        """Equal-split all-to-all on pre-packed buffers: slice i of dim 0 goes to group rank i."""
        return dist.all_to_all_single(output, input_, group=self.device_group)

    def barrier(self):
        dist.barrier(group=self.cpu_group)

    # ------------------------------------------------------------------ batched point-to-point
    def p2p_isend(self, tensor: torch.Tensor, dst: Optional[int] = None, slot=None):
        """`slot` names the receive buffer on the consumer (tag, hop, payload index); NCCL matches sends and
        receives by order and ignores it."""
        if dst is None:
            dst = (self.rank_in_group + 1) % self.world_size
        self.p2p_ops.append(dist.P2POp(dist.isend, tensor, self.ranks[dst], self.device_group))

    def p2p_irecv(self, size=None, dtype=None, src: Optional[int] = None, out: Optional[torch.Tensor] = None, slot=None):
        """Queue a receive from group rank `src`.  `out` receives in place (persistent slot); without
        it a tensor of `size`/`dtype` is allocated, as the reference does on every hop."""
        if src is None:
            src = (self.rank_in_group - 1) % self.world_size
        tensor = out if out is not None else torch.empty(size, dtype=dtype, device=self.device)
        self.p2p_ops.append(dist.P2POp(dist.irecv, tensor, self.ranks[src], self.device_group))
        return tensor

    def p2p_commit(self):
        assert self.p2p_reqs is None, "a point-to-point batch is already in flight"
        self.p2p_reqs = dist.batch_isend_irecv(self.p2p_ops) if self.p2p_ops else []

    def p2p_wait(self):
        for req in self.p2p_reqs or []:
            req.wait()
        self.p2p_ops.clear()
        self.p2p_reqs = None

    # Several batches in flight at once (not in the reference): every hop of a layer call is posted
    # up front as its own batch and waited for just before the attention launch that consumes it.
    def p2p_commit_batch(self):
        """Launch the queued operations as one batch and return its handle; other batches may be in flight."""
        reqs = dist.batch_isend_irecv(self.p2p_ops) if self.p2p_ops else []
        self.p2p_ops = []
        return reqs

    @staticmethod
    def p2p_wait_batch(reqs):
        for req in reqs or []:
            req.wait()

    def destroy(self):
        for g in (self.device_group, self.cpu_group):
            if g is not None:
                dist.destroy_process_group(g)
        self.device_group = self.cpu_group = None


class SingleRankGroup:
    """Stand-in for a group of one (no process group needed): what the attention objects get when
    the job runs on a single GPU."""
    world_size = 1
    rank_in_group = 0
    ranks = [0]
    local_rank = 0

    def __init__(self, device=None):
        self.device = device if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))

    def all_reduce(self, x):
        return x

    def all_gather(self, x, dim=-1, split=False):
        return [x] if split else x

    def all_to_all(self, x, scatter_dim=2, gather_dim=1):
        return x

    def barrier(self):
        pass

    def p2p_commit_batch(self):
        return []

    @staticmethod
    def p2p_wait_batch(reqs):
        return None
