"""CPU unit tests of the host-side modules: the schedule against known answers computed by the
reference's own RedundancyMap code on its shipped maps (tests/golden/schedules.npz, made by
tests/golden/make_schedule_golden.py), config files, the memory guard, timers, init_ditango on gloo."""
import os
import types

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp
import yaml

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "schedules.npz"))
MODELS = sorted({k.split("__")[0] for k in GOLD.files})


def _args(T, L, **kw):
    return types.SimpleNamespace(num_inference_steps=T, num_layers=L, **kw)


def test_known_models_present():
    assert MODELS == ["cogvideox_5b", "hunyuanvideo", "stepvideo"]
    assert GOLD["cogvideox_5b__map"].shape == (50, 42) and GOLD["hunyuanvideo__map"].shape == (50, 60)


@pytest.mark.parametrize("model", MODELS)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_schedule_matches_reference_on_shipped_maps(model, world):
    from ditango_b200.core.redundancy_map import RedundancyMap
    red = GOLD[f"{model}__map"]
    T, L = red.shape
    rm = RedundancyMap(_args(T, L), world_size=world)
    rm.redundancy_map = torch.from_numpy(red.copy())
    rm.generate_divider_map_from_redundancy(GOLD[f"{model}__percentiles"].tolist(), GOLD[f"{model}__dividers"].tolist())
    rm._refine_divider_map()
    assert np.array_equal(rm.divider_map.numpy(), GOLD[f"{model}__div_n{world}"])
    got = np.array([[rm.get_curr_isp_stride(t, l) for l in range(L)] for t in range(T)])
    nxt = np.array([[rm.get_next_isp_stride(t, l) for l in range(L)] for t in range(T)])
    assert np.array_equal(got, GOLD[f"{model}__stride_n{world}"])
    assert np.array_equal(nxt, GOLD[f"{model}__next_n{world}"])


def test_divider_histograms_of_the_shipped_maps():
    want = {("cogvideox_5b", 4): {1: 381, 2: 946, 4: 773}, ("cogvideox_5b", 2): {1: 340, 2: 1760},
            ("hunyuanvideo", 8): {1: 560, 2: 1379, 4: 1061}, ("stepvideo", 8): {1: 472, 2: 1928}}
    for (model, world), hist in want.items():
        u, c = np.unique(GOLD[f"{model}__div_n{world}"], return_counts=True)
        assert dict(zip(u.tolist(), c.tolist())) == hist


def test_init_redundancy_map_loads_the_default_file(tmp_path):
    from ditango_b200.core import redundancy_map as rmod
    red = GOLD["stepvideo__map"]
    T, L = red.shape
    d = tmp_path / "configs" / "stepvideo"
    d.mkdir(parents=True)
    torch.save(torch.from_numpy(red.copy()), d / f"redundancy_map_{T}_{L}.pt")
    args = _args(T, L, ditango_base=str(tmp_path), model_name="stepvideo", use_pab=False,
                 stride_percentiles=[0, 0, 90], stride_dividers=[8, 4, 2, 1])
    rmod.destroy_redundancy_map()
    rm = rmod.init_redundancy_map(args, world_size=8)
    try:
        assert np.array_equal(rm.divider_map.numpy(), GOLD["stepvideo__div_n8"])
        assert rmod.get_redundancy_map() is rm and not rmod.is_preprocessing()
        with pytest.raises(AssertionError):
            rmod.init_redundancy_map(args, world_size=8)
    finally:
        rmod.destroy_redundancy_map()


def test_self_send_screen_on_shipped_maps():
    """The shipped CogVideoX / HunyuanVideo maps make the reference exchange KV with itself after some
    stride transitions; the screened schedule has no such cell and never reuses more than the original."""
    from ditango_b200.core.redundancy_map import RedundancyMap
    red = GOLD["hunyuanvideo__map"]
    T, L = red.shape
    rm = RedundancyMap(_args(T, L), world_size=8)
    rm.divider_map = torch.from_numpy(GOLD["hunyuanvideo__div_n8"].copy())
    before = sum(any(rec["self_send"]) for l in range(L) for rec in rm.replay_layer(l))
    assert before > 0
    changed = rm.screen_self_sends()
    assert changed > 0
    assert all(not any(rec["self_send"]) for l in range(L) for rec in rm.replay_layer(l))
    assert (rm.divider_map.numpy() <= GOLD["hunyuanvideo__div_n8"]).all()


def test_config_file_switches(tmp_path):
    from ditango_b200.core.config import get_config, init_config
    path = tmp_path / "config.yaml"
    path.write_text(yaml.dump({"model-name": "hunyuanvideo", "num-layers": 60, "num-inference-steps": 50,
                               "use-ditango": False, "use-ulysses": True, "stride-percentiles": [0, 40, 90],
                               "output-fn": str(tmp_path / "out"), "tag": "t"}))
    cfg = init_config(str(path))
    assert get_config() is cfg
    assert cfg.model_name == "hunyuanvideo" and cfg.use_ulysses and not cfg.use_ditango
    assert cfg.stride_dividers == [1]                     # plain ring outside use-ditango
    assert os.path.isdir(cfg.output_dir)
    path.write_text(yaml.dump({"do-preprocess": True, "use-ditango": True, "output-fn": str(tmp_path / "out")}))
    cfg = init_config(str(path), make_output_dir=False)
    assert not cfg.use_ditango and not cfg.use_ulysses


def test_memory_guard_degrades_to_full_stride(monkeypatch):
    from ditango_b200.core.cache import proCache
    c = proCache(isp_size=4, layer_id=0)
    c.set_block_size_mb(torch.empty(1, 1024, 8, 64))
    assert abs(c.block_size_mb - 1024 * 8 * 65 * 4 / 2 ** 20) < 1e-9
    assert c.pass_memory_check(4, 0)                      # full stride never caches
    c.memory_constraint = 1e9
    assert c.pass_memory_check(1, 0)
    c.memory_constraint = c.block_size_mb * 2.5           # room for two more blocks only
    assert not c.pass_memory_check(1, 0)                  # stride 1 would need four
    c.out_block_cache[0] = torch.zeros(1)
    c.out_block_cache[1] = torch.zeros(1)
    assert c.pass_memory_check(2, 0)                      # two blocks already held


def test_cache_reblocking_bookkeeping(monkeypatch):
    from tests import cpu_engine
    import ditango_b200.core.cache as cache_mod
    monkeypatch.setattr(cache_mod, "_engine", cpu_engine)
    from ditango_b200.core.cache import proCache
    c = proCache(isp_size=4, layer_id=0)
    g = torch.Generator().manual_seed(0)
    for i in (0, 2, 3):
        c.store_block(i, torch.randn(1, 8, 2, 16, generator=g), torch.randn(1, 2, 8, generator=g))
    c.update_cache_blocks(new_isp_stride=2, next_target_block_id=0)
    assert c.curr_block_num == 2 and c.out_block_cache[0] is None and c.out_block_cache[1] is not None
    with pytest.raises(AssertionError):
        c.update_cache_blocks(new_isp_stride=1, next_target_block_id=0)   # cannot split blocks again
    c.update_cache_blocks(new_isp_stride=4, next_target_block_id=0)
    assert c.out_block_cache == [None] * 4


def test_timers_collect_regions():
    from ditango_b200 import timer
    timer.init_timer(enable=True)

    @timer.get_timer("unit-region")
    def work():
        return sum(range(1000))
    for _ in range(3):
        work()
    with timer.get_timer("unit-ctx"):
        pass
    stats = timer.TimerManager.statistics()
    assert stats["unit-region"]["samples"] == 3 and stats["unit-ctx"]["samples"] == 1
    timer.disable_timing()
    work()
    assert timer.TimerManager.statistics()["unit-region"]["samples"] == 3
    assert not timer.is_timing_enabled()


def _init_worker(rank, world, port, cfg_path, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world), RANK=str(rank),
                      LOCAL_RANK=str(rank))
    from ditango_b200.compat import install_as_ditango
    install_as_ditango()
    from ditango.core.initialize import init_ditango, is_ditango_initialized   # the reference's import paths
    from ditango.core.parallel_state import get_isp_group, get_usp_group, get_world_group
    from ditango.core.redundancy_map import get_redundancy_map
    init_ditango(cfg_path, backend="gloo")
    g = get_isp_group()
    ret[rank] = (is_ditango_initialized(), g.world_size, g.rank_in_group, get_usp_group().ranks,
                 get_world_group().world_size, get_redundancy_map().base_weight,
                 int(get_redundancy_map().divider_map.max()))
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


def test_init_ditango_under_the_reference_package_name(tmp_path):
    red = GOLD["cogvideox_5b__map"]
    d = tmp_path / "configs" / "cogvideox-5b"
    d.mkdir(parents=True)
    torch.save(torch.from_numpy(red.copy()), d / "redundancy_map_50_42.pt")
    cfg = tmp_path / "config.yaml"
    cfg.write_text(yaml.dump({"model-name": "cogvideox-5b", "ditango-base": str(tmp_path), "num-layers": 42,
                              "num-inference-steps": 50, "use-ditango": True, "stride-dividers": [8, 4, 2, 1],
                              "stride-percentiles": [0, 40, 90], "output-fn": str(tmp_path / "out")}))
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_init_worker, args=(2, 29871, str(cfg), ret), nprocs=2, join=True)
    for r in range(2):
        assert ret[r] == (True, 2, r, [0, 1], 2, 2, 2)


def test_schedule_lookup_sees_writes_through_any_alias_of_the_divider_tensor():
    """`rm.get_map()[t, l] = d` and writes through a reference held from earlier take effect on the next
    lookup, as in the reference, where every lookup reads the tensor (core/redundancy_map.py:49-87)."""
    from ditango_b200.core import redundancy_map as rmod
    from ditango_b200.core.config import init_config
    cfg = init_config(None, make_output_dir=False)
    cfg.num_layers, cfg.num_inference_steps = 2, 4
    rmod.destroy_redundancy_map()
    rm = rmod.init_redundancy_map(cfg, world_size=4)
    held = rm.divider_map
    assert rm.get_curr_isp_stride(1, 0) == 4
    rm.get_map()[1, 0] = 2
    assert rm.get_curr_isp_stride(1, 0) == 2
    held[2, 1] = 4
    assert rm.get_curr_isp_stride(2, 1) == 1 and rm.get_next_isp_stride(1, 1) == 1
    rmod.destroy_redundancy_map()


def test_cpu_profiling_branch_follows_the_reference_drift_metric():
    """NaN positions masked, mean|cur| when the previous output is ~0, inf when nothing is valid
    (utils.py:202-267); and switching profiling on by assignment works."""
    import math
    import torch
    from oracle import ring_oracle as O
    from ditango_b200.core import redundancy_map as rmod
    from ditango_b200.core.config import init_config
    from ditango_b200.utils import rel_l1
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(1000, generator=g), torch.randn(1000, generator=g)
    a[3] = float("nan")
    b[7] = float("nan")
    assert abs(rel_l1(a, b) - O.rel_l1(a, b)) < 1e-12
    assert abs(rel_l1(a, torch.zeros(1000)) - O.rel_l1(a, torch.zeros(1000))) < 1e-12
    assert math.isinf(rel_l1(torch.full((4,), float("nan")), torch.ones(4)))
    cfg = init_config(None, make_output_dir=False)
    cfg.num_layers, cfg.num_inference_steps = 1, 3
    rmod.destroy_redundancy_map()
    rm = rmod.init_redundancy_map(cfg, world_size=1)
    rm.auto_setting = True                      # not through enable_auto_setting()
    x = torch.randn(2, 8, 2, 4, generator=g)
    y = x + 0.1 * torch.randn(2, 8, 2, 4, generator=g)
    y[0, 0, 0, 0] = float("nan")
    rm.record_out_redundancy(0, 0, x)
    rm.record_out_redundancy(1, 0, y)
    assert abs(rm.redundancy_map[1, 0].item() - O.rel_l1(y, x)) < 1e-6
    rmod.destroy_redundancy_map()


def test_receive_buffers_are_per_group_and_follow_the_latest_shape():
    import torch
    from ditango_b200.core import attention as A

    class G:
        pass
    g1, g2 = G(), G()
    x = torch.zeros(2, 3)
    a = A._slot(g1, "kv0", 0, x)
    assert A._slot(g1, "kv0", 0, x) is a and A._slot(g2, "kv0", 0, x) is not a
    b = A._slot(g1, "kv0", 0, torch.zeros(4, 3))
    assert b.shape == (4, 3) and sum(1 for k in A._SLOTS if k[0] == id(g1)) == 1      # the old shape is dropped
    A.release_receive_slots(g1)
    assert not any(k[0] == id(g1) for k in A._SLOTS) and any(k[0] == id(g2) for k in A._SLOTS)
    A.release_receive_slots()
