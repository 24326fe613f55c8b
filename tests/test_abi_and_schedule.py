"""CPU checks: the C-ABI library exports every symbol the header declares; the integer planner
agrees with the oracle's replay of the reference's pointer logic; schedule quantiser / legaliser
agree with the oracle's restatement."""
import os
import re

import numpy as np
import pytest
import torch

from oracle import ring_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from ditango_b200 import _build, _capi
    _build.build()
    with open(os.path.join(ROOT, "include", "ditango_b200.h")) as f:
        declared = set(re.findall(r"DTB_API\s+[\w\s\*]+?\b(dtb_\w+)\s*\(", f.read()))
    assert declared and declared == set(_capi.EXPORTS)
    lib = _capi.load()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.dtb_version() >= 100


def test_rejected_arguments_do_not_need_a_gpu():
    from ditango_b200 import _capi
    lib = _capi.load()
    rc = lib.dtb_flash_fwd(None, None, None, 0, 0, 0, None, 0, 0, None, 0, 0, None, None, 1, 1, 1, 1, 1, 1, 64, 1.0, None)
    assert rc == -1 and b"null" in lib.dtb_last_error()
    rc = lib.dtb_flash_fwd_ex(None, None, None, 0, 0, 0, None, 0, 0, None, 0, 0, None, None, 1, 1, 1, 1, 1, 1, 64, 1.0, 6, None)
    assert rc == -1 and b"launch flag" in lib.dtb_last_error()


def test_cpu_tensors_are_refused_without_fallback():
    from ditango_b200 import ops
    from ditango_b200._capi import ExtensionError
    q = torch.zeros(1, 8, 1, 64, dtype=torch.bfloat16)
    with pytest.raises(ExtensionError):
        ops.flash_partial(q, q, q)


@pytest.mark.parametrize("world,div", [(2, [1, 2, 2, 1]), (4, [1, 4, 4, 2, 2, 2, 1]), (8, [1, 1, 1, 8, 8, 8, 8, 4, 4, 2, 2, 1, 1]),
                                       (4, [1, 1, 1, 4, 4, 2, 2, 1, 1])])
def test_planner_matches_pointer_replay(world, div):
    from ditango_b200.core.schedule import plan_step
    tr = O.replay_pointers(div, world)
    ptr = [0] * world
    dm = np.asarray(div).reshape(-1, 1)
    for t in range(len(div)):
        s = O.stride_now(dm, world, t, 0)
        plan = plan_step(world, s, ptr)
        assert [p.target_block for p in plan.ranks] == tr[t]["target_block"]
        for r in range(world):
            src = tr[t]["first_kv_from"][r]
            assert plan.ranks[r].own_first == (src is not None)
            if src is not None:
                assert plan.ranks[r].owners[0] == src
            # every hop is a permutation: each rank sends its chunk to at most one consumer per hop
            for hop in range(s):
                assert len(plan.send_to(r, hop)) <= 1
                got = plan.recv_from(r, hop)
                if got is not None:
                    assert r in plan.send_to(got, hop)
        ptr = plan.pointers_after
        assert ptr == tr[t]["pointer_after"]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_planner_on_random_legal_schedules(world):
    """Sixty random schedules per group size, drawn like the benchmark's (Bernoulli reuse, a random legal divider),
    legalised and screened by the package's own RedundancyMap: at every step the planner's target blocks, first-KV
    sources and pointers equal the integer replay of the reference's state machine, every hop is a partial
    permutation, and every rank attends each chunk of its target block exactly once."""
    from ditango_b200.core.schedule import plan_step
    rng = np.random.RandomState(100 + world)
    legal = [d for d in (2, 4, 8) if d <= world]
    for case in range(60):
        T = int(rng.randint(4, 14))
        div = np.ones((T, 1), dtype=np.int64)
        for t in range(1, T):
            if rng.rand() < 0.65:
                div[t, 0] = legal[rng.randint(len(legal))]
        rm = _rm(T, 1, world)
        rm.divider_map = torch.from_numpy(div)
        rm._refine_divider_map()
        rm.screen_self_sends()
        col = [int(x) for x in rm.get_map()[:, 0].tolist()]
        tr = O.replay_pointers(col, world)
        ptr = [0] * world
        dm = np.asarray(col).reshape(-1, 1)
        for t in range(T):
            s = O.stride_now(dm, world, t, 0)
            plan = plan_step(world, s, ptr)
            assert [p.target_block for p in plan.ranks] == tr[t]["target_block"], (case, col, t)
            assert not any(tr[t]["self_send"]), (case, col, t)
            for r in range(world):
                src = tr[t]["first_kv_from"][r]
                assert plan.ranks[r].own_first == (src is not None)
                tb = plan.ranks[r].target_block
                want = set(range(tb * s, tb * s + s)) - ({r} if plan.ranks[r].own_first else set())
                assert sorted(plan.ranks[r].owners) == sorted(want | ({r} if not plan.ranks[r].own_first else set())), (case, col, t, r)
                for hop in range(s):
                    assert len(plan.send_to(r, hop)) <= 1
                    got = plan.recv_from(r, hop)
                    if got is not None:
                        assert r in plan.send_to(got, hop) and got == plan.ranks[r].owners[hop]
            ptr = plan.pointers_after
            assert ptr == tr[t]["pointer_after"], (case, col, t)


def _rm(T, L, world):
    from ditango_b200.core.redundancy_map import RedundancyMap

    class A:
        num_inference_steps, num_layers = T, L
    return RedundancyMap(A(), world_size=world)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_quantiser_and_legaliser_match_oracle(world):
    rng = np.random.RandomState(world)
    red = np.abs(rng.randn(20, 6)).astype(np.float32)
    red[0] = 0
    rm = _rm(20, 6, world)
    rm.redundancy_map = torch.from_numpy(red)
    rm.generate_divider_map_from_redundancy([0, 40, 90], [8, 4, 2, 1])
    want = O.quantise_redundancy(red.astype(np.float64), world, [0, 40, 90], [8, 4, 2, 1])
    assert np.array_equal(rm.divider_map.numpy(), want)
    rm._refine_divider_map()
    want = O.refine_dividers(want)
    assert np.array_equal(rm.divider_map.numpy(), want)
    for t in range(20):
        for l in range(6):
            assert rm.get_curr_isp_stride(t, l) == O.stride_now(want, world, t, l)
            assert rm.get_next_isp_stride(t, l) == O.stride_next(want, world, t, l)
    rm.screen_self_sends()
    assert np.array_equal(rm.divider_map.numpy(), O.screen_self_sends(want, world))
    for l in range(6):
        assert not any(any(rec["self_send"]) for rec in rm.replay_layer(l))


def test_plain_ring_when_divider_set_is_degenerate():
    rm = _rm(6, 2, 4)
    rm.redundancy_map = torch.rand(6, 2) + 0.1
    rm.generate_divider_map_from_redundancy([20, 50, 80], [1])
    assert int(rm.divider_map.max()) == 1
    assert rm.get_curr_isp_stride(3, 1) == 4


def test_pair_map_expansion():
    rm = _rm(7, 1, 4)
    for t, d in enumerate([1, 4, 4, 2, 2, 2, 1]):
        rm.divider_map[t, 0] = d
    pm = rm.pair_map(0)
    assert not pm[0].any() and not pm[6].any()
    # step 1, stride 1: rank 1's pointer is on its own chunk -> everything else comes from cache
    assert pm[1, :, 1].tolist() == [True, False, True, True]
    # step 2: pointer on chunk 2 -> chunks 0 and 3 reused, 2 fetched
    assert pm[2, :, 1].tolist() == [True, False, False, True]


def test_config_switches():
    from ditango_b200.core.config import DiTangoConfig
    c = DiTangoConfig(None, make_output_dir=False)
    assert c.use_ditango and c.stride_dividers == [8, 4, 2, 1]
    c.num_layers = 3
    assert c.config["num_layers"] == 3
    with pytest.raises(AttributeError):
        _ = c.nope


def test_split_and_unpad_roundtrip():
    from ditango_b200.utils import remove_padding_after_gather, split_tensor_uneven
    x = torch.arange(2 * 10 * 3, dtype=torch.float32).view(2, 10, 3)
    parts = split_tensor_uneven(x, 4, dim=1, tensor_name="x")
    assert all(p.shape[1] == 3 for p in parts)
    back = remove_padding_after_gather(torch.cat(parts, dim=1), "x")
    assert torch.equal(back, x)


def test_uneven_shard_segment_table_and_single_rank_gather():
    from ditango_b200.core.group_coordinate import SingleRankGroup
    from ditango_b200.utils import gather_sequence_shards, uneven_shard_cu_seqlens, uneven_shard_lengths
    assert uneven_shard_lengths(66, 4) == [17, 17, 16, 16]
    assert uneven_shard_lengths(64, 4) == [16, 16, 16, 16]
    cu, longest = uneven_shard_cu_seqlens(66, 4, rank=2, batch_size=2)
    assert cu.dtype == torch.int32 and cu.tolist() == [0, 16, 17, 33, 34] and longest == 17
    cu, _ = uneven_shard_cu_seqlens(66, 4, rank=0, batch_size=1)
    assert cu.tolist() == [0, 17, 17]                      # no pad on this rank: empty second segment
    x = torch.arange(24, dtype=torch.float32).view(1, 12, 2)
    assert torch.equal(gather_sequence_shards(SingleRankGroup(torch.device("cpu")), x, 12), x)
