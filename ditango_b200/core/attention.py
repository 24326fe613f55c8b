"""Sequence-parallel attention with cached partial states: the per-layer object the model adapters
call (`proAttention(layer_id, isp_group).attn(q, k, v)` / `.varlen_attn(...)`).

Same contract as the reference's core/attention.py: inputs are this rank's contiguous bf16 chunk
[B,S_loc,H,D] (or packed [T,H,D] with cu_seqlens), the result is a new fp32 tensor of that shape, the
step index comes from the global set by the pipeline, the stride of (step, layer) from the global
schedule, and every rank of the group must call in the same order.

What is different underneath:
  * partial attention runs in the sm_100a kernel; a block's fresh chunks are folded into ONE fp32
    state by the kernel's accumulate epilogue instead of per-chunk merges (utils.py:24-84 of the
    reference, called at core/attention.py:144, :193-196);
  * cached blocks, the own chunk and the fresh block are combined by one N-way merge launch
    (reference: a chain of pairwise merges at :110-116 and :213);
  * KV chunks go owner -> consumer directly, K and V (and cu_seqlens) of a hop in one NCCL group; all
    hops of a call are posted up front into persistent per-hop slots and each is waited for just
    before the launch that reads it; no clone before a send (reference: :51);
  * the first-KV exchange is decided at block level; the reference decides it at chunk level
    (:120), which makes it address itself and count its own chunk twice after some stride
    transitions.  On schedules without such self-sends both give the same result.
"""
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed

from .. import ops as _engine
from .._capi import LSE_BSH
from ..logger import init_logger
from ..timer import get_timer
from ..utils import get_timestep
from .cache import proCache
from .config import get_config
from .redundancy_map import get_redundancy_map
from .schedule import StepPlan, plan_pair_step, plan_step

logger = init_logger(__name__)

# One receive slot per (group, hop, payload index), shared by all layers that use the group: layers run
# one after another on ONE stream, and a layer call has at most group-size hops in flight.  Two
# attention objects of the same group driven from different streams would race on these slots.
# A slot follows the latest shape it was asked for; buffers of shapes no longer in use are dropped.
_SLOTS: Dict[Tuple, torch.Tensor] = {}


def _slot(group, tag: str, index: int, like: torch.Tensor) -> torch.Tensor:
    key = (id(group), tag, index)
    buf = _SLOTS.get(key)
    if buf is None or buf.shape != like.shape or buf.dtype != like.dtype or buf.device != like.device:
        buf = torch.empty_like(like, memory_format=torch.contiguous_format)
        _SLOTS[key] = buf
    return buf


def release_receive_slots(group=None):
    """Drop the receive buffers of `group` (all groups when None)."""
    if group is None:
        _SLOTS.clear()
        return
    for key in [k for k in _SLOTS if k[0] == id(group)]:
        del _SLOTS[key]


# Denoising step at which the device status word was last polled by this process (see _run).
_STATUS_POLL = {"step": None}


class proAttention:
    # How the hops of one call are batched for the transport ("single" or "doubling", see _post_hops).
    # Class-wide default; every rank of a group must agree.
    hop_grouping = "single"
    # dtype of the returned tensor.  float32 is the reference's contract (its callers cast to bf16 right
    # away: executor/cogvideox/attention_processor.py:80, executor/step/attentions.py:98); with
    # torch.bfloat16 the cast is fused into the last kernel of the call and the fp32 copy is never written.
    output_dtype = torch.float32
    # dtype of the values of cached block states (the reference keeps fp32: utils.py:76); bfloat16 halves
    # the cache's footprint and read traffic.  lse stays fp32.
    cache_dtype = torch.float32
    # Overlapping attention launches.  The chunks of a call are attended by one launch each; every launch ends
    # in a partly filled wave and is followed by a launch gap.  A launch made with overlap_previous starts while
    # the attention launch before it is finishing (ops.flash_partial); that is allowed when only event waits /
    # records were queued on the stream since that launch.
    #   "auto"  overlap where it was measured to pay: launches of less than OVERLAP_MAX_FLOPS (short ones, where
    #           gap and tail are a visible share; long D = 128 launches run at the board's power cap, where the
    #           idle tail is what lets the clock recover, and lose about 1 %), and only on transports whose wait
    #           for an incoming chunk is an event wait (the group says so: `wait_is_event_only`);
    #   True    overlap every launch that may.  On a transport that copies on the compute stream when it waits,
    #           the own chunk is attended first, then ALL incoming chunks are waited for, then the remaining
    #           launches go back to back;
    #   False   never.
    # Every rank of a group must agree.  Results are bit-identical in all three.
    chain_launches = "auto"
    OVERLAP_MAX_FLOPS = 5.0e11

    def __init__(self, layer_id: int, isp_group):
        self.group = isp_group
        self.isp_size = self.group.world_size
        self.global_rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else 0
        self.local_chunk_id = self.group.rank_in_group
        self.layer_id = layer_id
        self.target_chunk_id = 0
        # chunk pointer of every rank of the group for this layer; all ranks keep the same copy
        self._pointers = [0] * self.isp_size
        cfg = get_config()
        if cfg is not None and getattr(cfg, "cache_dtype", None) in ("bf16", "bfloat16"):
            self.cache_dtype = torch.bfloat16
        if cfg is not None and getattr(cfg, "output_dtype", None) in ("bf16", "bfloat16"):
            self.output_dtype = torch.bfloat16
        # Partial states, cached states and their merges keep lse as [B,S,H] ([T,H] packed): one lse per
        # (token, head) row in the order the value rows are stored, so the merge kernel reads it without
        # index arithmetic.  Only `last_lse` is presented as [B,H,S], what flash_attn returns.
        self.cache = proCache(isp_size=self.isp_size, layer_id=layer_id, store_dtype=self.cache_dtype,
                              lse_layout=LSE_BSH)
        self.use_ditango = bool(cfg.use_ditango) if cfg is not None else True
        self.small_ring_stride = 8
        self.measure_memory = False
        self.measure_comm = False
        # per-pair reuse maps (RedundancyMap.set_pair_map): cached state per source chunk, and which
        # chunks every rank of the group holds (all ranks keep the same copy)
        self._chunk_states: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._have = [set() for _ in range(self.isp_size)]
        self._last_lse: Optional[torch.Tensor] = None      # [B,S,H] / [T,H] of the last result
        self.stats = dict(calls=0, chunks_attended=0, chunks_received=0, bytes_received=0,
                          cached_blocks_merged=0, merge_launches=0, overlapped_launches=0)
        self._comm_events: List[Tuple[torch.cuda.Event, torch.cuda.Event]] = []
        # True while the operation queued last on the compute stream by this object is an attention launch
        # (what overlap_previous requires of its predecessor)
        self._chain_open = False

    @property
    def last_lse(self) -> Optional[torch.Tensor]:
        """Log-sum-exp of the last result as [B,H,S] (packed: [H,T]), the layout flash_attn returns."""
        return None if self._last_lse is None else self._last_lse.transpose(-1, -2)

    def _finish(self, own, others):
        """Combine the own-chunk state with all other states of the call into the result: one merge launch
        (in place in the own state's fp32 buffer), or none when there is nothing to merge."""
        want_bf16 = self.output_dtype == torch.bfloat16
        if others:
            res16 = torch.empty(own[0].shape, dtype=torch.bfloat16, device=own[0].device) if want_bf16 else None
            out, lse = _engine.merge_states([(own[0], own[1], LSE_BSH)] + others, out=own[0], lse_out=own[1],
                                            lse_out_layout=LSE_BSH, out_bf16=res16, fp32_out=not want_bf16)
            self.stats["merge_launches"] += 1
            return (res16 if want_bf16 else out), lse
        out, lse = own
        if want_bf16 and out.dtype != torch.bfloat16:
            # every chunk was folded into the fp32 state by the attention kernel: one cast pass
            res16 = torch.empty(out.shape, dtype=torch.bfloat16, device=out.device)
            _engine.merge_states([(out, lse, LSE_BSH)], out=out, want_lse=False, out_bf16=res16, fp32_out=False)
            self.stats["merge_launches"] += 1
            out = res16
        return out, lse

    # ------------------------------------------------------------------ transport
    def _queue_hop(self, plan: StepPlan, hop: int, payload: Tuple[torch.Tensor, ...]):
        """Queue this rank's sends of its own chunk and its receive for `hop`; returns the received
        tensors (None when nothing arrives in this hop)."""
        me = self.local_chunk_id
        src = plan.recv_from(me, hop)
        recv = None
        for dst in plan.send_to(me, hop):
            for i, t in enumerate(payload):
                self.group.p2p_isend(t, dst=dst, slot=("kv", hop, i))
        if src is not None:
            own_buffers = hasattr(self.group, "p2p_prepare")     # the transport lands the data in buffers of its own
            recv = tuple(self.group.p2p_irecv(src=src, out=None if own_buffers else _slot(self.group, f"kv{i}", hop, t),
                                              slot=("kv", hop, i)) for i, t in enumerate(payload))
            self.stats["chunks_received"] += 1
            self.stats["bytes_received"] += sum(t.numel() * t.element_size() for t in payload)
        return recv

    def _post_hops(self, plan: StepPlan, n_hops: int, payload: Tuple[torch.Tensor, ...]):
        """Post every hop of this call.  Returns one (received tensors or None, batch handle or None)
        per hop; the handle sits on the first hop of its batch and covers the hops up to the next handle.

        hop_grouping "single": one batch per hop -- a batch is one NCCL group, and the groups of a
        process group run one after another, each moving one chunk per rank at the rate of one peer pair.
        "doubling": batches of 1, 2, 4, ... hops -- the first chunk still arrives as early as possible,
        later batches pull from several peers at once.  Every rank of the group must use the same setting."""
        prepare = getattr(self.group, "p2p_prepare", None)
        if prepare is not None:              # transports that keep their own receive buffers (peer_transport.py)
            prepare("kv", payload, self.isp_size)
        posted, size, hop = [], 1, 0
        while hop < n_hops:
            end = min(n_hops, hop + size)
            recvs = [self._queue_hop(plan, h, payload) for h in range(hop, end)]
            handle = self.group.p2p_commit_batch()
            posted.extend((r, handle if i == 0 else None) for i, r in enumerate(recvs))
            hop = end
            if self.hop_grouping == "doubling":
                size *= 2
        return posted

    def _wait_hop(self, handle):
        if handle is None:          # covered by the batch of an earlier hop
            return
        if not getattr(self.group, "wait_is_event_only", False):
            self._chain_open = False    # the transport's copy now sits behind the last launch
        if self.measure_comm and torch.cuda.is_available():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            self.group.p2p_wait_batch(handle)
            b.record()
            self._comm_events.append((a, b))
        else:
            self.group.p2p_wait_batch(handle)

    def _chain_mode(self) -> Tuple[bool, bool]:
        """(launches may overlap, own chunk first and all waits before the other launches)."""
        mode = self.chain_launches
        event_only = bool(getattr(self.group, "wait_is_event_only", False))
        if mode == "auto":
            return event_only, False
        return bool(mode), bool(mode) and not event_only

    def _attend(self, chain: bool, query, kk, vv, **kw):
        """One attention launch; with `chain` it overlaps the previous one when that was an attention launch of
        this object and no kernel or copy was queued on the stream since."""
        if chain and self._chain_open and (self.chain_launches != "auto" or
                                           4.0 * query.numel() * kk.shape[-3] < self.OVERLAP_MAX_FLOPS):
            kw["overlap_previous"] = True
        self.stats["chunks_attended"] += 1
        self.stats["overlapped_launches"] += int("overlap_previous" in kw)
        res = _engine.flash_partial(query, kk, vv, lse_layout=LSE_BSH, **kw)
        self._chain_open = True
        return res

    def exposed_comm_ms(self, reset: bool = True) -> float:
        """Time the compute stream spent blocked on incoming KV since the last reset."""
        if not self._comm_events:
            return 0.0
        torch.cuda.synchronize()
        total = sum(a.elapsed_time(b) for a, b in self._comm_events)
        if reset:
            self._comm_events = []
        return total

    # ------------------------------------------------------------------ per-pair reuse (extension)
    def _run_pairs(self, flags, query, key, value, cu_q=None, cu_kv=None, max_q=None, max_kv=None):
        """One call under a per-pair reuse map: own chunk always fresh; every other chunk either from
        this rank's per-chunk cache or fetched from its owner and recomputed, as flags[src][me] says."""
        N, me = self.isp_size, self.local_chunk_id
        packed = cu_q is not None
        payload = (key, value, cu_kv) if packed else (key, value)

        chain, reorder = self._chain_mode()
        self._chain_open = False

        def attend(kv, keep=False):
            kw = {}
            if packed:
                kw = dict(cu_seqlens_q=cu_q, cu_seqlens_k=kv[2], max_seqlen_q=max_q, max_seqlen_k=max_kv)
            return self._attend(chain, query, kv[0], kv[1], out_dtype=self.cache_dtype if keep else torch.float32, **kw)

        plan = plan_pair_step(N, flags, self._have)
        posted = self._post_hops(plan, plan.n_hops, payload)
        own = attend(payload)
        if reorder:
            for hop in range(plan.n_hops):
                self._wait_hop(posted[hop][1])
        for hop in range(plan.n_hops):
            current, handle = posted[hop]
            if not reorder:
                self._wait_hop(handle)
            if current is not None:
                self._chunk_states[plan.ranks[me].owners[hop]] = attend(current, keep=True)
        self._chain_open = False
        others = [(o, l, LSE_BSH) for src in ((me + i) % N for i in range(1, N))
                  for o, l in (self._chunk_states.get(src, (None, None)),) if l is not None]
        self.stats["cached_blocks_merged"] += len(others) - len(plan.ranks[me].owners)
        out, lse = self._finish(own, others)
        self._last_lse = lse
        self.stats["calls"] += 1
        return out

    # ------------------------------------------------------------------ the call
    def _run(self, query, key, value, cu_q=None, cu_kv=None, max_q=None, max_kv=None):
        N, me = self.isp_size, self.local_chunk_id
        rmap = get_redundancy_map()
        t = get_timestep()
        if _STATUS_POLL["step"] != t:
            # Once per denoising step: a kernel whose bounded wait ran out leaves a sticky code in the
            # device status word and every later launch skips its work, so results from then on would be
            # garbage behind a zero return code.  The poll never blocks: it tests the copy made one
            # step earlier and queues the next one.
            _STATUS_POLL["step"] = t
            _engine.poll_status()
        flags = rmap.pair_flags(t, self.layer_id) if N > 1 else None
        if flags is not None:
            return self._run_pairs(flags, query, key, value, cu_q, cu_kv, max_q, max_kv)
        stride = rmap.get_curr_isp_stride(t, self.layer_id)
        next_stride = rmap.get_next_isp_stride(t, self.layer_id)
        if t == 0:
            self.cache.set_block_size_mb(value)
        if not self.cache.pass_memory_check(next_stride, self.layer_id):
            next_stride = N
        assert N % stride == 0, f"Does not support this ISP stride {stride} for SP size {N}"
        if stride > self.small_ring_stride and self.use_ditango:
            # the reference switches to a two-level ring here (groups larger than one node)
            assert stride % self.small_ring_stride == 0, \
                f"Does not support this ISP stride {stride} for overlap ring strategy"

        plan = plan_step(N, stride, self._pointers)
        mine = plan.ranks[me]
        nblk = N // stride
        packed = cu_q is not None
        payload = (key, value, cu_kv) if packed else (key, value)
        keep_chunks = stride == N and next_stride != N        # fine-grained store after a full refresh
        keep_block = stride != N and next_stride != N

        chain, reorder = self._chain_mode()
        chain, reorder = chain and N > 1, reorder and N > 1
        self._chain_open = False

        def attend(kv, into=None, dtype=torch.float32):
            kk, vv = kv[0], kv[1]
            kw = {}
            if packed:
                kw = dict(cu_seqlens_q=cu_q, cu_seqlens_k=kv[2], max_seqlen_q=max_q, max_seqlen_k=max_kv)
            if into is None:
                return self._attend(chain, query, kk, vv, out_dtype=dtype, **kw)
            return self._attend(chain, query, kk, vv, out=into[0], lse=into[1], accumulate=True, **kw)

        # 1. cached blocks (every block but the target one)
        states = []
        if stride != N:
            for i in range(nblk - 1):
                o, l = self.cache.get_block((mine.target_block + 1 + i) % nblk)
                if l is not None:
                    states.append((o, l, LSE_BSH))
            self.stats["cached_blocks_merged"] += len(states)

        # 2. every hop of this call is posted now, each into its own slot: chunks travel owner ->
        #    consumer, so the hops do not depend on one another and the link streams them while the
        #    attention kernels work through the chunks already here.
        posted = self._post_hops(plan, stride, payload) if N > 1 else [(None, None)] * stride
        # A single rank with nothing to merge gets its bf16 result straight from the attention kernel.
        direct16 = N == 1 and self.output_dtype == torch.bfloat16 and not rmap.is_auto_setting()
        own = None
        if mine.own_first or reorder:
            # target block is a foreign one: own chunk first, overlapping hop 0.  Reordered launches: always first,
            # so that the transfers run under it and every wait sits in front of the launches that overlap.
            own = attend(payload)
        if reorder:
            for hop in range(stride):
                self._wait_hop(posted[hop][1])

        # 3. the target block's chunks.  A state that goes to the cache without further accumulation is
        #    written by the attention kernel in the cache's dtype: no cast pass afterwards.
        fresh = None
        chunk_states = []
        fresh_chunks = sum(1 for o in mine.owners if o != me)
        for hop in range(stride):
            current, handle = posted[hop]
            if not reorder:
                self._wait_hop(handle)
            if mine.owners[hop] == me:
                if own is None:            # (reordered launches attended it before the waits)
                    own = attend(payload, dtype=torch.bfloat16 if direct16 else torch.float32)
            elif keep_chunks:
                st = attend(current, dtype=self.cache_dtype)
                if st[0].dtype != self.cache.store_dtype:
                    self._chain_open = False           # store_block converts: a kernel behind the launch
                self.cache.store_block(mine.owners[hop], st[0], st[1])
                chunk_states.append((st[0], st[1], LSE_BSH))
            elif keep_block:
                fresh = attend(current, into=fresh, dtype=self.cache_dtype if fresh_chunks == 1 else torch.float32)
            else:
                own = attend(current, into=own)          # nothing is kept: fold into the result

        self._chain_open = False

        # 4. store the fresh block, combine everything in one pass
        if fresh is not None:
            self.cache.store_block(mine.target_block, fresh[0], fresh[1])
            chunk_states.append((self.cache.out_block_cache[mine.target_block], fresh[1], LSE_BSH))
        out, lse = self._finish(own, states + chunk_states)

        # 5. pointers and cache layout for the next step
        self._pointers = plan.pointers_after
        self.target_chunk_id = self._pointers[me]
        self.cache.update_cache_blocks(next_stride, self.target_chunk_id // next_stride)
        self._last_lse = lse
        self.stats["calls"] += 1
        rmap.record_out_redundancy(timestep=t, layer_id=self.layer_id, curr_out=out)
        return out

    @get_timer("oAttn")
    def attn(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
        """query, key, value: [B, S_loc, H, D] -> fp32 [B, S_loc, H, D]."""
        return self._run(query, key, value)

    @get_timer("varlen oAttn")
    def varlen_attn(self, query, key, value, cu_seqlens_q=None, cu_seqlens_kv=None,
                    max_seqlen_q=None, max_seqlen_kv=None, batch_size=1) -> torch.Tensor:
        """Packed variant: query, key, value [T, H, D]; the KV owner's cu_seqlens travels with its K,V."""
        if cu_seqlens_q is None and cu_seqlens_kv is None and max_seqlen_q is None and max_seqlen_kv is None:
            logger.warning("cu_seqlens_q not provided, using normal attention instead.")
            return self.attn(query, key, value)
        return self._run(query, key, value, cu_q=cu_seqlens_q, cu_kv=cu_seqlens_kv,
                         max_q=max_seqlen_q, max_kv=max_seqlen_kv)
