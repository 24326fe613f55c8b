"""Integer planning of one attention call: which KV chunks each rank of the group attends fresh,
in which order, and who sends what to whom.

The reference moves KV chunks around a ring inside the rank's block (core/attention.py:160-201 of
the reference) after an optional first exchange with the target block (:119-145).  Which chunk a
rank holds at which ring step is a pure function of (group size, stride, chunk pointers), so it is
computed here for ALL ranks at once; every chunk then travels straight from its owner to each
consumer (NVSwitch gives every pair full bandwidth, so forwarding buys nothing and would chain
the hops).  All ranks run the same arithmetic and therefore agree on the send/receive pairs.
"""
from dataclasses import dataclass
from typing import List, Optional


@dataclass
class RankPlan:
    target_block: int
    local_block: int
    own_first: bool            # own chunk is attended before hop 0 (target block is a foreign block)
    owners: List[int]          # chunk owner attended at hop i (== rank itself: the own chunk)


@dataclass
class StepPlan:
    stride: int
    ranks: List[RankPlan]
    pointers_after: List[int]

    @property
    def n_hops(self) -> int:
        return max(len(p.owners) for p in self.ranks)

    def recv_from(self, rank: int, hop: int) -> Optional[int]:
        owners = self.ranks[rank].owners
        if hop >= len(owners) or owners[hop] == rank:
            return None
        return owners[hop]

    def send_to(self, rank: int, hop: int) -> List[int]:
        return [r for r, p in enumerate(self.ranks) if r != rank and hop < len(p.owners) and p.owners[hop] == rank]


def plan_step(world: int, stride: int, pointers: List[int]) -> StepPlan:
    """pointers[r] = rank r's chunk pointer before the call (core/attention.py:27, :107-108, :214)."""
    assert world % stride == 0, f"Does not support this ISP stride {stride} for SP size {world}"
    plans, after = [], []
    for r in range(world):
        ptr = r if stride == world else pointers[r]
        lb, tb = r // stride, ptr // stride
        inner = r % stride
        owners = [tb * stride + (inner + i) % stride for i in range(stride)]
        plans.append(RankPlan(target_block=tb, local_block=lb, own_first=(tb != lb), owners=owners))
        after.append((ptr + (world if stride == world else stride)) % world)
    return StepPlan(stride=stride, ranks=plans, pointers_after=after)


def plan_pair_step(world: int, reusable, have: List[set]) -> StepPlan:
    """Planning for a per-pair reuse map (an extension; the reference cannot express it).

    reusable[src][dst]: consumer `dst` may take chunk `src` from its cache this step; have[dst]: the
    chunks `dst` holds a cached state for.  A pair is fetched and recomputed when it is not flagged, or
    flagged but never computed.  Each consumer walks the other chunks in ring order (dst+1, dst+2, ...);
    its h-th fetch is hop h.  `have` is updated in place.  A hop is no longer a permutation: a rank may
    serve several consumers in one hop, and ranks need different numbers of hops.
    """
    plans = []
    for dst in range(world):
        fetch = []
        for step in range(1, world):
            src = (dst + step) % world
            if not (reusable[src][dst] and src in have[dst]):
                fetch.append(src)
        plans.append(RankPlan(target_block=-1, local_block=-1, own_first=True, owners=fetch))
    for dst, p in enumerate(plans):
        have[dst].update(p.owners)
    return StepPlan(stride=0, ranks=plans, pointers_after=[])
