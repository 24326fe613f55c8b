"""CPU oracle for DiTango's sequence-parallel attention path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain fp32 torch-CPU arithmetic, what the reference computes on
its ring / cached-ring / Ulysses attention path.  It is the checker that the parity tests,
the smoke test and the CPU-baseline leg of the benchmark compare the CUDA path against; the
product package never imports it.

Parity pin: the reference ships no tests or golden vectors for this path.  The oracle is
pinned against outputs of the reference itself, executed on CPU/gloo ranks with its
third-party flash-attention call replaced by softmax(QK^T/sqrt(D))V + logsumexp; those
outputs are stored under tests/golden/ together with the generating script
(tests/golden/make_golden.py), and tests/test_oracle_golden.py replays them.

Reference locations restated here (paths relative to the reference project root):
  * partial attention of one Q chunk against one KV chunk, returning (out, lse[B,H,Sq]):
    the `flash_attn_func(..., return_attn_probs=True)` call sites core/attention.py:137-143,
    185-191 and the varlen sites :314-324, :366-376 (third-party `flash_attn==2.7.0.post2`,
    requirements.txt:4 -- standard scaled-dot-product softmax attention, scale 1/sqrt(D)).
  * merge of two partial softmax states: utils.py:24-84 (`update_out_and_lse`).
  * per-layer block store and re-blocking: core/cache.py:9-84 (`proCache`).
  * (step, layer) -> stride lookup: core/redundancy_map.py:49-87; transition legaliser
    :281-326; redundancy -> divider quantiser :199-279.
  * the ring / reuse state machine: core/attention.py:73-237 (dense) and :239-419 (varlen).
  * Ulysses head/sequence all-to-all attention: baseline/ulysses.py:51-124 with
    core/group_coordinate.py:281-286.
  * the drift metric of the redundancy-profiling pass: utils.py:202-267 (`rel_l1`).

All ranks of a group are simulated inside one process: each rank runs the state machine in
its own thread and point-to-point messages travel through in-memory mailboxes, so the order
of sends, receives, partial attentions, merges and cache updates is the reference's.
"""
from __future__ import annotations

import math
import queue
import threading
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# Partial attention (what the reference gets from flash_attn) and the state merge
# --------------------------------------------------------------------------------------

def partial_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                      softmax_scale: Optional[float] = None,
                      out_dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention of q [B,Sq,H,D] against one KV chunk k,v [B,Sk,H,D].

    Returns (out [B,Sq,H,D] in `out_dtype` (default: q's dtype, as flash_attn does),
    lse [B,H,Sq] fp32 in natural-log units).  core/attention.py:137-143.
    """
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
    qf, kf, vf = q.float(), k.float(), v.float()
    scores = torch.einsum("bqhd,bkhd->bhqk", qf, kf) * scale
    lse = torch.logsumexp(scores, dim=-1)
    probs = torch.exp(scores - lse.unsqueeze(-1))
    out = torch.einsum("bhqk,bkhd->bqhd", probs, vf)
    return out.to(out_dtype if out_dtype is not None else q.dtype), lse


def partial_attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                             cu_q: Sequence[int], cu_k: Sequence[int],
                             softmax_scale: Optional[float] = None,
                             out_dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Packed variant: q [Tq,H,D], k,v [Tk,H,D]; segment i of q attends segment i of k.

    Returns (out [Tq,H,D], lse [H,Tq]).  Rows of an empty key segment get out=0, lse=-inf.
    Tokens of q beyond cu_q[-1] are left at out=0, lse=-inf.  core/attention.py:314-324.
    """
    cu_q = [int(x) for x in cu_q]
    cu_k = [int(x) for x in cu_k]
    T, H, D = q.shape
    odt = out_dtype if out_dtype is not None else q.dtype
    out = torch.zeros(T, H, D, dtype=odt)
    lse = torch.full((H, T), float("-inf"), dtype=torch.float32)
    for i in range(len(cu_q) - 1):
        q0, q1, k0, k1 = cu_q[i], cu_q[i + 1], cu_k[i], cu_k[i + 1]
        if q1 <= q0 or k1 <= k0:
            continue
        o, l = partial_attention(q[None, q0:q1], k[None, k0:k1], v[None, k0:k1], softmax_scale, odt)
        out[q0:q1] = o[0]
        lse[:, q0:q1] = l[0]
    return out, lse


def _as_row_lse(lse: torch.Tensor) -> torch.Tensor:
    """[..., H, S] -> [..., S, H, 1] (the layout the merged state is kept in)."""
    return lse.transpose(-2, -1).unsqueeze(-1)


def merge_states(out: Optional[torch.Tensor], lse: Optional[torch.Tensor],
                 block_out: torch.Tensor, block_lse: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(out, lse) (+) (block_out, block_lse), utils.py:44-84.

    `lse` and `block_lse` may each be given as [..,H,S] or [..,S,H,1]; the result's lse is
    [..,S,H,1] and its out is fp32.  First call (out is None) just adopts the block.
    """
    if block_lse.shape[-1] == 1:
        block_lse = block_lse.squeeze(-1).transpose(-1, -2)
    if lse is not None and lse.shape[-1] != 1:
        lse = _as_row_lse(lse)
    if out is None:
        return block_out.to(torch.float32), _as_row_lse(block_lse)
    b_out = block_out.to(torch.float32)
    b_lse = _as_row_lse(block_lse)
    # utils.py:38-39
    new_out = out - torch.sigmoid(b_lse - lse) * (out - b_out)
    new_lse = lse - F.logsigmoid(lse - b_lse)
    return new_out, new_lse


def merge_states_exact(states: Sequence[Tuple[torch.Tensor, torch.Tensor]]) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp64 N-way merge with explicit max subtraction: the mathematical value every merge
    order converges to.  lse inputs are [B,H,S]; returns (out fp64 [B,S,H,D], lse fp64 [B,H,S])."""
    lses = torch.stack([s[1].double() for s in states])                     # [n,B,H,S]
    m = lses.max(dim=0).values
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(lses - m_safe)                                             # [n,B,H,S]
    tot = w.sum(dim=0)
    acc = 0
    for i, (o, _) in enumerate(states):
        acc = acc + o.double() * w[i].transpose(-2, -1).unsqueeze(-1)
    tot_row = tot.transpose(-2, -1).unsqueeze(-1)
    out = torch.where(tot_row > 0, acc / tot_row.clamp_min(1e-300), torch.zeros_like(acc))
    return out, m_safe + torch.log(tot)


# --------------------------------------------------------------------------------------
# Stride schedule
# --------------------------------------------------------------------------------------

def quantise_redundancy(redundancy: np.ndarray, world: int,
                        percentages: Sequence[float], dividers: Sequence[int]) -> np.ndarray:
    """Relative-L1 drift map [T,L] -> divider map [T,L].  core/redundancy_map.py:199-279."""
    T, L = redundancy.shape
    out = np.ones((T, L), dtype=np.int64)
    nz = redundancy[redundancy > 0]
    if nz.size == 0:
        return out
    cuts = [np.percentile(nz, p) for p in percentages]
    for t in range(T - 1):                                   # the last row stays 1 (:244-246)
        for l in range(L):
            r = float(redundancy[t, l])
            if r <= 0:
                continue
            if r < cuts[0]:
                d = dividers[0]
            elif r < cuts[1]:
                d = dividers[1]
            elif r < cuts[2]:
                d = dividers[2]
            else:
                d = dividers[3]
            if world < d:
                d = world
            elif world % d != 0:
                pick = 1
                for cand in sorted(dividers):
                    if world % cand == 0 and cand <= d:
                        pick = cand
                        break
                d = pick
            out[t, l] = int(d)
    return out


def refine_dividers(dividers: np.ndarray) -> np.ndarray:
    """Legalise transitions per layer; first three and last two steps run at divider 1.
    core/redundancy_map.py:281-326 (row 0 is never visited there and stays as given)."""
    d = dividers.copy()
    T, L = d.shape
    for l in range(L):
        for t in range(1, T):
            if t < 3 or t > T - 3:
                d[t, l] = 1
                continue
            prev, cur = d[t - 1, l], d[t, l]
            if prev == 1 or cur <= prev:
                continue
            d[t, l] = 1
    return d


def stride_now(dividers: np.ndarray, world: int, t: int, l: int) -> int:
    """core/redundancy_map.py:49-67."""
    dv = int(dividers[t, l])
    if world < dv:
        return 1
    assert world % dv == 0, f"divider {dv} does not divide group size {world}"
    return max(world // dv, 1)


def stride_next(dividers: np.ndarray, world: int, t: int, l: int) -> int:
    """core/redundancy_map.py:69-87."""
    if t == dividers.shape[0] - 1:
        return world
    dv = int(dividers[t + 1, l])
    if world < dv:
        return 1
    assert world % dv == 0
    return world // dv


def replay_pointers(dividers_col: Sequence[int], world: int) -> List[Dict]:
    """Integer-only replay of one layer's pointer logic for every rank
    (core/attention.py:100-134, :203-214).  Returns, per step, a dict with the stride and
    per-rank lists `target_block`, `first_kv_from` (rank or None), `self_send` (bool)."""
    ptr = [r // world for r in range(world)]           # core/attention.py:27
    T = len(dividers_col)
    div = np.asarray(dividers_col, dtype=np.int64).reshape(T, 1)
    trace = []
    for t in range(T):
        s = stride_now(div, world, t, 0)
        d = world // s
        rec = dict(stride=s, target_block=[], first_kv_from=[], self_send=[], pointer_before=list(ptr))
        for r in range(world):
            lb, tb = r // s, ptr[r] // s
            if s == world:
                ptr[r] = r
            src = None
            if ptr[r] != r:
                src = tb * s + r % s
            rec["target_block"].append(tb)
            rec["first_kv_from"].append(src)
            rec["self_send"].append(src == r)
            # a full refresh advances the pointer once per chunk, `world` times in all
            ptr[r] = (ptr[r] + (world if s == world else s)) % world
        rec["pointer_after"] = list(ptr)
        trace.append(rec)
    return trace


def screen_self_sends(dividers: np.ndarray, world: int) -> np.ndarray:
    """Reset to divider 1 every (step, layer) cell at which the reference would post a
    send to itself (its first-KV exchange fires on a chunk-level test, core/attention.py:120,
    while the peer is chosen at block level, :123-128).  Returns a new map."""
    d = dividers.copy()
    T, L = d.shape
    for l in range(L):
        while True:
            tr = replay_pointers(d[:, l], world)
            bad = [t for t, rec in enumerate(tr) if any(rec["self_send"])]
            if not bad:
                break
            d[bad[0], l] = 1
    return d


# --------------------------------------------------------------------------------------
# Block store (core/cache.py)
# --------------------------------------------------------------------------------------

class BlockStore:
    """Per-layer list of cached (out fp32 [B,S,H,D], lse fp32 [B,H,S]) block states."""

    def __init__(self, world: int):
        self.world = world
        self.slots: List[Optional[Tuple[torch.Tensor, torch.Tensor]]] = [None] * world

    def get(self, i: int):
        return self.slots[i]

    def put(self, i: int, out: torch.Tensor, lse: torch.Tensor):
        self.slots[i] = (out, lse)

    def reblock(self, next_stride: int, next_target_block: int):
        """core/cache.py:49-72 (with _merge_blocks :28-46)."""
        if next_stride == self.world:
            self.slots = [None] * self.world
            return
        n_new = self.world // next_stride
        assert n_new <= len(self.slots), "cache cannot be split into finer blocks"
        if n_new != len(self.slots):
            per = len(self.slots) // n_new
            merged = []
            for i in range(n_new):
                o, l = None, None
                for j in range(per):
                    st = self.slots[i * per + j]
                    if st is None:
                        continue
                    o, l = merge_states(o, l, st[0], st[1])
                merged.append(None if o is None else (o, l))
            self.slots = merged
        self.slots[next_target_block] = None


# --------------------------------------------------------------------------------------
# In-process message passing between simulated ranks
# --------------------------------------------------------------------------------------

class Mailboxes:
    def __init__(self, world: int):
        self.q = {(s, d): queue.Queue() for s in range(world) for d in range(world)}

    def send(self, src: int, dst: int, payload):
        self.q[(src, dst)].put(payload)

    def recv(self, src: int, dst: int, timeout: float = 120.0):
        return self.q[(src, dst)].get(timeout=timeout)


@dataclass
class RankLayerState:
    """What one rank keeps per layer across steps (core/attention.py:21-34)."""
    world: int
    rank: int
    pointer: int = 0
    store: BlockStore = None
    log: List[Tuple] = field(default_factory=list)

    def __post_init__(self):
        self.pointer = self.rank // self.world
        if self.store is None:
            self.store = BlockStore(self.world)


def ring_attention_rank_step(state: RankLayerState, mail: Mailboxes, t: int,
                             stride: int, next_stride: int,
                             q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                             cu_q=None, cu_kv=None,
                             partial_dtype: Optional[torch.dtype] = None,
                             block_level_first_kv: bool = False) -> torch.Tensor:
    """One call of the reference's per-layer attention on one rank.

    Dense when cu_q is None (q,k,v [B,S_loc,H,D], core/attention.py:73-237); packed otherwise
    (q,k,v [T,H,D] with cu_q / cu_kv int lists, the kv list travelling with its K,V,
    core/attention.py:239-419).  Returns the merged fp32 output.

    `block_level_first_kv=True` replaces the chunk-level test of core/attention.py:120 by the
    block-level one (no first-KV exchange when the target block is the rank's own block); on
    schedules without self-sends both are the same.
    """
    N, r = state.world, state.rank
    varlen = cu_q is not None

    def attend(kk, vv, ckv):
        if varlen:
            return partial_attention_varlen(q, kk, vv, cu_q, ckv, out_dtype=partial_dtype)
        return partial_attention(q, kk, vv, out_dtype=partial_dtype)

    assert N % stride == 0
    nblk = N // stride
    local_block = r // stride
    target_block = state.pointer // stride
    out = lse = None

    # 1. cached blocks (core/attention.py:106-116)
    if stride == N:
        state.pointer = r
    else:
        for i in range(nblk - 1):
            b = (target_block + 1 + i) % nblk
            st = state.store.get(b)
            state.log.append(("get", t, b, st is not None))
            if st is not None:
                out, lse = merge_states(out, lse, st[0], st[1])

    # 2. first KV chunk of a foreign target block (core/attention.py:119-145)
    need_first = (target_block != local_block) if block_level_first_kv else (state.pointer != r)
    if need_first:
        hop = (target_block - local_block) % nblk
        send_block = (local_block - hop) % nblk
        inner = r % stride
        src = target_block * stride + inner
        dst = send_block * stride + inner
        mail.send(r, dst, (k, v, cu_kv))
        bo, bl = attend(k, v, cu_kv)
        state.log.append(("attend", t, r))
        out, lse = merge_states(out, lse, bo, bl)
        k, v, cu_kv = mail.recv(src, r)
        kv_owner = src
    else:
        kv_owner = r

    # 3. ring inside the rank's own block (core/attention.py:147-201); groups of <= 8 ranks
    #    never take the two-level ring branch.
    n_update = 1 if stride == N else stride
    off = r // stride * stride
    nxt = (r - 1) % stride + off
    prv = (r + 1) % stride + off
    fresh_o = fresh_l = None
    done = 0
    for step in range(stride):
        if step + 1 != stride:
            mail.send(r, nxt, (k, v, cu_kv, kv_owner))
        bo, bl = attend(k, v, cu_kv)
        state.log.append(("attend", t, kv_owner))
        if local_block == target_block and step == 0:
            out, lse = merge_states(out, lse, bo, bl)
        else:
            fresh_o, fresh_l = merge_states(fresh_o, fresh_l, bo, bl)
        done += 1
        if step + 1 != stride:
            k, v, cu_kv, kv_owner = mail.recv(prv, r)
        # 4. block finished (core/attention.py:203-217)
        if done == n_update:
            if fresh_l is not None:
                fresh_l = fresh_l.squeeze(-1).transpose(-1, -2)
                if next_stride != N:
                    slot = state.pointer if stride == N else target_block
                    state.store.put(slot, fresh_o, fresh_l)
                    state.log.append(("put", t, slot))
                out, lse = merge_states(out, lse, fresh_o, fresh_l)
            state.pointer = (state.pointer + done) % N
            fresh_o = fresh_l = None
            done = 0

    # 5. re-block the store for the next step (core/attention.py:219-220)
    state.store.reblock(next_stride, state.pointer // next_stride)
    state.last_lse = lse
    return out


def run_ring_group(world: int, dividers_col: Sequence[int],
                   qkv_per_step: Sequence[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]],
                   partial_dtype: Optional[torch.dtype] = None,
                   block_level_first_kv: bool = False,
                   cu_per_rank: Optional[Sequence[Sequence[int]]] = None,
                   states: Optional[List[RankLayerState]] = None,
                   t0: int = 0) -> Tuple[List[List[torch.Tensor]], List[RankLayerState]]:
    """Run one layer for len(qkv_per_step) steps on `world` simulated ranks.

    qkv_per_step[t] = global (q, k, v), each [B,S,H,D]; rank r owns rows
    [r*S/world, (r+1)*S/world).  With `cu_per_rank` (one cu_seqlens list per rank, relative
    to the rank's packed tokens) the packed path is used on q[0], k[0], v[0] of each rank.
    Returns (outs[t][r], states).
    """
    T = len(qkv_per_step)
    div = np.asarray(dividers_col, dtype=np.int64).reshape(-1, 1)
    if states is None:
        states = [RankLayerState(world, r) for r in range(world)]
    mail = Mailboxes(world)
    outs: List[List[torch.Tensor]] = [[None] * world for _ in range(T)]
    errors: List[BaseException] = []

    def worker(r: int):
        try:
            for i in range(T):
                t = t0 + i
                q, k, v = qkv_per_step[i]
                S = q.shape[1]
                lo, hi = r * S // world, (r + 1) * S // world
                ql, kl, vl = q[:, lo:hi].contiguous(), k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous()
                s, ns = stride_now(div, world, t, 0), stride_next(div, world, t, 0)
                if cu_per_rank is not None:
                    cu = list(cu_per_rank[r])
                    outs[i][r] = ring_attention_rank_step(states[r], mail, t, s, ns, ql[0], kl[0], vl[0],
                                                          cu_q=cu, cu_kv=cu, partial_dtype=partial_dtype,
                                                          block_level_first_kv=block_level_first_kv)
                else:
                    outs[i][r] = ring_attention_rank_step(states[r], mail, t, s, ns, ql, kl, vl,
                                                          partial_dtype=partial_dtype,
                                                          block_level_first_kv=block_level_first_kv)
        except BaseException as e:  # surfaced to the caller below
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(r,), daemon=True) for r in range(world)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    if errors:
        raise errors[0]
    return outs, states


# --------------------------------------------------------------------------------------
# Generalised per-chunk reuse (pair maps).  NOT in the reference: its schedule can only express
# pair maps that follow from a stride and a rotating pointer.  Here every (source chunk, consumer
# rank) pair carries its own flag per step: a flagged pair takes the partial state the consumer
# computed for that chunk the last time it was fresh; an unflagged pair -- or a flagged one that
# was never computed -- is recomputed from the current step's tensors.  On pair maps expanded from
# a stride schedule this gives the reference's result up to fp32 rounding (tested).
# --------------------------------------------------------------------------------------

def run_pair_map_group(world: int, reusable: np.ndarray,
                       qkv_per_step: Sequence[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]],
                       partial_dtype: Optional[torch.dtype] = None) -> List[List[torch.Tensor]]:
    """reusable[t, src, dst] bool; qkv_per_step[t] = global (q, k, v) [B,S,H,D].  Returns outs[t][dst]
    (fp32 [B,S_loc,H,D]): own chunk first, then the other chunks in ring order (dst+1, dst+2, ...)."""
    T = len(qkv_per_step)
    cache: List[Dict[int, Tuple[torch.Tensor, torch.Tensor]]] = [dict() for _ in range(world)]
    outs: List[List[torch.Tensor]] = []
    for t in range(T):
        q, k, v = qkv_per_step[t]
        S = q.shape[1]
        sl = [slice(r * S // world, (r + 1) * S // world) for r in range(world)]
        row = []
        for dst in range(world):
            ql = q[:, sl[dst]]
            o, l = partial_attention(ql, k[:, sl[dst]], v[:, sl[dst]], out_dtype=partial_dtype)
            out, lse = merge_states(None, None, o, l)
            for step in range(1, world):
                src = (dst + step) % world
                if not (bool(reusable[t, src, dst]) and src in cache[dst]):
                    o, l = partial_attention(ql, k[:, sl[src]], v[:, sl[src]], out_dtype=partial_dtype)
                    cache[dst][src] = (o.float(), l)
                co, cl = cache[dst][src]
                out, lse = merge_states(out, lse, co, cl)
            row.append(out)
        outs.append(row)
    return outs


def pair_map_from_dividers(dividers_col: Sequence[int], world: int) -> np.ndarray:
    """The reusable[t, src, dst] view of one layer's stride schedule (pointer replay)."""
    tr = replay_pointers(dividers_col, world)
    out = np.zeros((len(tr), world, world), dtype=bool)
    for t, rec in enumerate(tr):
        s = rec["stride"]
        if s == world:
            continue
        for dst in range(world):
            for src in range(world):
                out[t, src, dst] = src != dst and src // s != rec["target_block"][dst]
    return out


# --------------------------------------------------------------------------------------
# Ulysses (baseline/ulysses.py:51-124)
# --------------------------------------------------------------------------------------

def all_to_all_views(shards: Sequence[torch.Tensor], scatter_dim: int, gather_dim: int) -> List[torch.Tensor]:
    """What every rank holds after GroupCoordinator.all_to_all (core/group_coordinate.py:281-286):
    rank r gets cat over source ranks j of the r-th split (along scatter_dim) of shards[j]."""
    world = len(shards)
    pieces = [torch.tensor_split(x, world, scatter_dim) for x in shards]
    return [torch.cat([pieces[j][r] for j in range(world)], dim=gather_dim).contiguous() for r in range(world)]


def ulysses_attention(q_shards, k_shards, v_shards) -> List[torch.Tensor]:
    """q/k/v_shards[r]: [B,S_loc,H,D] of rank r.  Returns per-rank output [B,S_loc,H,D] in the
    input dtype: head/sequence transpose, full-sequence attention on H/world heads, transpose back."""
    world = len(q_shards)
    B, S_loc, H, D = q_shards[0].shape
    flat = lambda xs: [x.reshape(B, S_loc, H * D) for x in xs]
    qf = all_to_all_views(flat(q_shards), 2, 1)
    kf = all_to_all_views(flat(k_shards), 2, 1)
    vf = all_to_all_views(flat(v_shards), 2, 1)
    Hn = H // world
    outs = []
    for r in range(world):
        o, _ = partial_attention(qf[r].view(B, -1, Hn, D), kf[r].view(B, -1, Hn, D), vf[r].view(B, -1, Hn, D),
                                 softmax_scale=1.0 / math.sqrt(D))
        outs.append(o.reshape(B, -1, Hn * D))
    back = all_to_all_views(outs, 1, 2)
    return [x.view(B, S_loc, H, D) for x in back]


# --------------------------------------------------------------------------------------
# Redundancy profiling metric (utils.py:202-267 of the reference)
# --------------------------------------------------------------------------------------

def rel_l1(new: torch.Tensor, ori: torch.Tensor) -> float:
    """Relative L1 drift of `new` against `ori` over the positions where neither is NaN:
    mean|new - ori| / (mean|ori| + 1e-8); mean|new| when mean|ori| < 1e-6; inf when no position is
    valid or the result is not finite.  fp64 accumulation."""
    valid = ~(torch.isnan(new) | torch.isnan(ori))
    if not bool(valid.any()):
        return float("inf")
    n, o = new[valid].double(), ori[valid].double()
    ori_mean = o.abs().mean().item()
    if ori_mean < 1e-6:
        return n.abs().mean().item()
    val = (n - o).abs().mean().item() / (ori_mean + 1e-8)
    return val if math.isfinite(val) else float("inf")


# --------------------------------------------------------------------------------------
# Synthetic workloads shared by tests and the benchmark's CPU leg
# --------------------------------------------------------------------------------------

def drifting_qkv(B: int, S: int, H: int, D: int, steps: int, seed: int = 0, drift: float = 0.05,
                 dtype: torch.dtype = torch.float32, rms_norm_qk: bool = False):
    """Step 0: Q,K,V ~ N(0,1) from `seed`; each later step adds N(0, drift^2) to the previous
    step's tensors (order Q,K,V).  With rms_norm_qk, Q and K are RMS-normalised over D after
    the drift.  Yields `steps` tuples of [B,S,H,D] tensors in `dtype`."""
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, S, H, D, generator=g) for _ in range(3))
    res = []
    for t in range(steps):
        if t > 0:
            q, k, v = (x + drift * torch.randn(B, S, H, D, generator=g) for x in (q, k, v))
        qq, kk = q, k
        if rms_norm_qk:
            qq = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + 1e-6)
            kk = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + 1e-6)
        res.append((qq.to(dtype), kk.to(dtype), v.to(dtype)))
    return res


def bernoulli_dividers(steps: int, layers: int, world: int, p: float, seed: int = 0) -> np.ndarray:
    """Reference-expressible random schedule: per cell Bernoulli(p) picks reuse; a reuse cell
    takes a divider drawn uniformly from {2,4,8} that divides `world`; step 0 never reuses.
    The map is then legalised and screened for self-sends."""
    rng = np.random.RandomState(seed)
    choices = [d for d in (2, 4, 8) if d <= world and world % d == 0]
    div = np.ones((steps, layers), dtype=np.int64)
    if choices:
        for t in range(1, steps):
            for l in range(layers):
                if rng.rand() < p:
                    div[t, l] = choices[rng.randint(len(choices))]
    div = refine_dividers(div)
    return screen_self_sends(div, world)
