"""GPU parity of the whole attention path (public API -> C ABI -> sm_100a kernels) against the CPU
oracle on the same seeded bf16 inputs and the same stride schedule.  Tolerances: fp32 output built
from bf16 inputs <= 2e-2 max-abs / 1e-3 mean-abs, lse <= 1e-3.  Multi-rank cases need that many GPUs
and are skipped otherwise."""
import pytest
import torch
import torch.multiprocessing as mp

from oracle import ring_oracle as O
from tests import _dist_workers as W

pytestmark = pytest.mark.gpu
_PORT = [29810]


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _single_layer(steps):
    from ditango_b200.core import redundancy_map as rmod
    from ditango_b200.core.attention import proAttention
    from ditango_b200.core.config import init_config
    from ditango_b200.core.group_coordinate import SingleRankGroup
    cfg = init_config(None, make_output_dir=False)
    cfg.num_layers, cfg.num_inference_steps = 1, steps
    rmod.destroy_redundancy_map()
    rmod.init_redundancy_map(cfg, world_size=1)
    return proAttention(0, SingleRankGroup())


@pytest.mark.parametrize("B,S,H,D", [(1, 1024, 4, 64), (2, 2222, 3, 64), (1, 1861, 3, 128)])
def test_single_rank_attention_over_steps(B, S, H, D):
    from ditango_b200 import ops
    from ditango_b200.utils import update_timestep
    layer = _single_layer(3)
    data = O.drifting_qkv(B, S, H, D, 3, seed=0, dtype=torch.bfloat16)
    for t, (q, k, v) in enumerate(data):
        update_timestep(t)
        out = layer.attn(q.cuda(), k.cuda(), v.cuda())
        ref, ref_lse = O.partial_attention(q, k, v, out_dtype=torch.float32)
        e = (out.cpu() - ref).abs()
        assert out.dtype == torch.float32 and out.shape == q.shape
        assert e.max() <= 2e-2 and e.mean() <= 1e-3
        assert (layer.last_lse.cpu() - ref_lse).abs().max() <= 1e-3
    assert ops.read_status() == 0


def test_single_rank_packed_attention():
    from ditango_b200.utils import update_timestep
    layer = _single_layer(1)
    H, D = 2, 128
    cu = [0, 700, 768]
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(768, H, D, generator=g).to(torch.bfloat16) for _ in range(3))
    update_timestep(0)
    cu_t = torch.tensor(cu, dtype=torch.int32).cuda()
    out = layer.varlen_attn(q.cuda(), k.cuda(), v.cuda(), cu_seqlens_q=cu_t, cu_seqlens_kv=cu_t,
                            max_seqlen_q=768, max_seqlen_kv=768)
    ref, _ = O.partial_attention_varlen(q, k, v, cu, cu, out_dtype=torch.float32)
    e = (out.cpu() - ref).abs()
    assert e.max() <= 2e-2 and e.mean() <= 1e-3


def test_update_out_and_lse_public_helper():
    from ditango_b200.utils import update_out_and_lse
    g = torch.Generator().manual_seed(4)
    B, S, H, D = 2, 40, 2, 64
    o1, o2 = torch.randn(B, S, H, D, generator=g), torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    l1, l2 = torch.randn(B, H, S, generator=g), torch.randn(B, H, S, generator=g)
    out, lse = update_out_and_lse(None, None, o1.cuda(), l1.cuda())
    out, lse = update_out_and_lse(out, lse, o2.cuda(), l2.cuda())
    ro, rl = O.merge_states(*O.merge_states(None, None, o1, l1), o2, l2)
    assert lse.shape == (B, S, H, 1)
    assert (out.cpu() - ro).abs().max() < 1e-5 and (lse.cpu() - rl).abs().max() < 1e-5


def _spawn(world, case):
    _PORT[0] += 1
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(W.gpu_ring_worker, args=(world, _PORT[0], case, ret), nprocs=world, join=True)
    return dict(ret)


CASES = {
    2: dict(B=1, S=1024, H=4, D=64, seed=0, drift=0.05, dividers=[1, 2, 2, 1], ulysses=True),
    4: dict(B=2, S=1200, H=4, D=128, seed=1, drift=0.05, dividers=[1, 4, 4, 2, 2, 2, 1], ulysses=True),
    8: dict(B=1, S=2048, H=8, D=64, seed=2, drift=0.05, dividers=[1, 1, 1, 8, 8, 8, 8, 4, 4, 2, 2, 1, 1], ulysses=True),
}


@pytest.mark.parametrize("world,grouping,transport", [(2, "single", "nccl"), (4, "single", "nccl"), (8, "single", "nccl"),
                                                     (4, "doubling", "nccl"), (8, "doubling", "nccl"),
                                                     (2, "single", "peer"), (4, "single", "peer"), (8, "single", "peer")])
def test_ring_attention_multi_gpu_matches_oracle(world, grouping, transport):
    """transport "peer": KV chunks pushed by peer-to-peer copies into CUDA-IPC-mapped buffers of the consumer
    (core/peer_transport.py) instead of NCCL send / receive."""
    if _ngpu() < world:
        pytest.skip(f"needs {world} GPUs")
    case = dict(CASES[world], hop_grouping=grouping, transport=transport)
    ret = _spawn(world, case)
    data = O.drifting_qkv(case["B"], case["S"], case["H"], case["D"], len(case["dividers"]), seed=case["seed"],
                          drift=case["drift"], dtype=torch.bfloat16)
    ref, _ = O.run_ring_group(world, case["dividers"], data)
    for r in range(world):
        outs, stats, uly, status = ret[r]
        assert status == 0
        for t in range(len(case["dividers"])):
            e = (outs[t] - ref[t][r]).abs()
            assert e.max() <= 2e-2 and e.mean() <= 1e-3, (world, r, t, e.max().item(), e.mean().item())
    S, lo = case["S"], case["S"] // world
    q, k, v = data[0]
    full, _ = O.partial_attention(q, k, v, out_dtype=torch.float32)
    for r in range(world):
        e = (ret[r][2] - full[:, r * lo:(r + 1) * lo]).abs()
        assert e.max() <= 2e-2 and e.mean() <= 1.5e-3, ("ulysses", r, e.max().item(), e.mean().item())


def test_packed_ring_two_gpus():
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    case = dict(B=1, S=512, H=2, D=128, seed=4, drift=0.05, dividers=[1, 1, 2, 2, 1], cu=[[0, 230, 256], [0, 256, 256]])
    ret = _spawn(2, case)
    data = O.drifting_qkv(1, 512, 2, 128, 5, seed=4, drift=0.05, dtype=torch.bfloat16)
    ref, _ = O.run_ring_group(2, case["dividers"], data, cu_per_rank=case["cu"])
    for r in range(2):
        valid = case["cu"][r][1]
        for t in range(5):
            e = (ret[r][0][t][0, :valid] - ref[t][r][:valid]).abs()
            assert e.max() <= 2e-2 and e.mean() <= 1e-3


def test_uneven_shards_with_masked_pad_two_gpus():
    """257 tokens on 2 ranks (129 + 128 padded to 129): pad tokens sit in a segment of their own and are
    dropped by the gather; the result is full attention over the real tokens."""
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    case = dict(B=2, S=257, H=2, D=128, seed=13)
    _PORT[0] += 1
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(W.gpu_uneven_worker, args=(2, _PORT[0], case, ret), nprocs=2, join=True)
    g = torch.Generator().manual_seed(13)
    q, k, v = (torch.randn(2, 257, 2, 128, generator=g).to(torch.bfloat16) for _ in range(3))
    full, _ = O.partial_attention(q, k, v, out_dtype=torch.float32)
    for r in range(2):
        out, status = ret[r]
        assert status == 0
        e = (out - full).abs()
        assert e.max() <= 2e-2 and e.mean() <= 1e-3, (r, e.max().item(), e.mean().item())


def test_profiling_mode_records_drift_on_device():
    """RedundancyMap in profiling mode: full stride everywhere, drift of consecutive outputs added
    to the map by the device kernel, equal to the reference's rel_l1 of those outputs."""
    from ditango_b200.core import redundancy_map as rmod
    from ditango_b200.utils import update_timestep
    layer = _single_layer(3)
    rm = rmod.get_redundancy_map()
    rm.enable_auto_setting()
    data = O.drifting_qkv(1, 700, 2, 64, 3, seed=5, dtype=torch.bfloat16)
    outs = []
    for t, (q, k, v) in enumerate(data):
        update_timestep(t)
        outs.append(layer.attn(q.cuda(), k.cuda(), v.cuda()).cpu())
    rm.finish_auto_setting()
    assert rm.redundancy_map[0, 0] == 0
    for t in (1, 2):
        want = O.rel_l1(outs[t], outs[t - 1])
        assert abs(rm.redundancy_map[t, 0].item() - want) <= 1e-5 * max(1.0, want)
    assert not rm.is_auto_setting()


@pytest.mark.parametrize("world", [2, 4])
def test_pair_map_attention_multi_gpu(world):
    """Per-pair Bernoulli(0.6) reuse map (an extension beyond the reference's stride schedule) against the
    generalised oracle."""
    if _ngpu() < world:
        pytest.skip(f"needs {world} GPUs")
    import numpy as np
    T = 5
    rng = np.random.RandomState(3)
    reusable = rng.rand(T, world, world) < 0.6
    reusable[0] = False
    case = dict(T=T, B=2, S=300 * world, H=2, D=64, seed=6, drift=0.05, reusable=reusable.tolist())
    _PORT[0] += 1
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(W.gpu_pair_worker, args=(world, _PORT[0], case, ret), nprocs=world, join=True)
    data = O.drifting_qkv(2, 300 * world, 2, 64, T, seed=6, drift=0.05, dtype=torch.bfloat16)
    want = O.run_pair_map_group(world, reusable, data)
    for r in range(world):
        outs, stats, status = ret[r]
        assert status == 0
        for t in range(T):
            e = (outs[t] - want[t][r]).abs()
            assert e.max() <= 2e-2 and e.mean() <= 1e-3
