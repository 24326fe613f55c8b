"""Worker bodies for the multi-process CPU tests (spawned with torch.multiprocessing)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _setup(rank, world, port):
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world), RANK=str(rank),
                      LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    from tests import cpu_engine
    cpu_engine.install()
    from ditango_b200.core import parallel_state as ps
    from ditango_b200.core.config import init_config
    cfg = init_config(None, make_output_dir=False)
    ps.init_distributed_environment(world_size=world, rank=rank, local_rank=rank, backend="gloo")
    c, u, i = ps.generate_parallel_groups(world, do_cfg_guidance=False, sparse_type="full")
    ps.init_model_parallel(cfg_group_ranks=c, usp_group_ranks=u, iosp_dict=i)
    return cfg, ps


def ring_worker(rank, world, port, case, ret):
    cfg, ps = _setup(rank, world, port)
    from ditango_b200.core.attention import proAttention
    from ditango_b200.core.redundancy_map import init_redundancy_map
    from ditango_b200.utils import update_timestep
    from oracle.ring_oracle import drifting_qkv
    div = case["dividers"]
    cfg.num_layers, cfg.num_inference_steps = 1, len(div)
    rm = init_redundancy_map(cfg)
    for t, d in enumerate(div):
        rm.divider_map[t, 0] = d
    layer = proAttention(0, ps.get_isp_group())
    layer.hop_grouping = case.get("hop_grouping", "single")
    B, S, H, D = case["B"], case["S"], case["H"], case["D"]
    data = drifting_qkv(B, S, H, D, len(div), seed=case["seed"], drift=case["drift"])
    outs = []
    for t in range(len(div)):
        update_timestep(t)
        q, k, v = data[t]
        lo, hi = rank * S // world, (rank + 1) * S // world
        ql, kl, vl = (x[:, lo:hi].contiguous() for x in (q, k, v))
        if case.get("cu") is not None:
            cu = torch.tensor(case["cu"][rank], dtype=torch.int32)
            o = layer.varlen_attn(ql[0], kl[0], vl[0], cu_seqlens_q=cu, cu_seqlens_kv=cu,
                                  max_seqlen_q=hi - lo, max_seqlen_kv=hi - lo)[None]
        else:
            o = layer.attn(ql, kl, vl)
        outs.append(o.clone())
    ret[rank] = (torch.stack(outs), dict(layer.stats))
    dist.barrier()
    dist.destroy_process_group()


def uneven_worker(rank, world, port, case, ret):
    """Uneven sequence shards: zero-padded as the reference does, with and without the pad masked."""
    cfg, ps = _setup(rank, world, port)
    from ditango_b200.core.attention import proAttention
    from ditango_b200.core.redundancy_map import init_redundancy_map
    from ditango_b200.utils import (gather_sequence_shards, split_tensor_uneven, uneven_shard_cu_seqlens,
                                    update_timestep)
    cfg.num_layers, cfg.num_inference_steps = 2, 1
    init_redundancy_map(cfg)
    update_timestep(0)
    group = ps.get_isp_group()
    B, S, H, D = case["B"], case["S"], case["H"], case["D"]
    g = torch.Generator().manual_seed(case["seed"])
    q, k, v = (torch.randn(B, S, H, D, generator=g) for _ in range(3))
    ql, kl, vl = (split_tensor_uneven(x, world, dim=1)[rank].contiguous() for x in (q, k, v))
    shard = ql.shape[1]
    cu, max_len = uneven_shard_cu_seqlens(S, world, rank, batch_size=B)
    masked = proAttention(0, group).varlen_attn(ql.reshape(B * shard, H, D), kl.reshape(B * shard, H, D),
                                                vl.reshape(B * shard, H, D), cu_seqlens_q=cu, cu_seqlens_kv=cu,
                                                max_seqlen_q=max_len, max_seqlen_kv=max_len, batch_size=B)
    masked = gather_sequence_shards(group, masked.reshape(B, shard, H, D), S, dim=1)
    padded = gather_sequence_shards(group, proAttention(1, group).attn(ql, kl, vl), S, dim=1)
    ret[rank] = (masked, padded)
    dist.barrier()
    dist.destroy_process_group()


def ulysses_worker(rank, world, port, case, ret):
    cfg, ps = _setup(rank, world, port)
    from ditango_b200.baseline.ulysses import ulysses_attention
    B, S, H, D = case["B"], case["S"], case["H"], case["D"]
    g = torch.Generator().manual_seed(case["seed"])
    q, k, v = (torch.randn(B, S, H, D, generator=g) for _ in range(3))
    lo, hi = rank * S // world, (rank + 1) * S // world
    out = ulysses_attention(q[:, lo:hi].contiguous(), k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(),
                            group=ps.get_isp_group())
    ret[rank] = out.float()
    dist.barrier()
    dist.destroy_process_group()


def collectives_worker(rank, world, port, ret):
    cfg, ps = _setup(rank, world, port)
    g = ps.get_isp_group()
    x = torch.arange(2 * 3 * 4, dtype=torch.float32).view(2, 3, 4) + 100 * rank
    res = dict(
        a2a=g.all_to_all(x, scatter_dim=2, gather_dim=1),
        gather=g.all_gather(x, dim=1),
        reduce=g.all_reduce(x.clone()),
        ranks=(g.world_size, g.rank_in_group, g.ranks),
    )
    buf = torch.empty(3)
    g.p2p_isend(torch.full((3,), float(rank)), dst=(rank + 1) % world)
    got = g.p2p_irecv(src=(rank - 1) % world, out=buf)
    g.p2p_commit()
    g.p2p_wait()
    res["p2p"] = got.clone()
    ret[rank] = res
    dist.barrier()
    dist.destroy_process_group()


def gpu_ring_worker(rank, world, port, case, ret):
    """NCCL ranks, one GPU each, real kernels: proAttention on bf16 inputs."""
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world), RANK=str(rank),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    from ditango_b200 import ops
    from ditango_b200.core import parallel_state as ps
    from ditango_b200.core.attention import proAttention
    from ditango_b200.core.config import init_config
    from ditango_b200.core.redundancy_map import init_redundancy_map
    from ditango_b200.baseline.ulysses import ulysses_attention
    from ditango_b200.utils import update_timestep
    from oracle.ring_oracle import drifting_qkv
    cfg = init_config(None, make_output_dir=False)
    ps.init_distributed_environment(world_size=world, rank=rank, local_rank=rank, backend="nccl")
    c, u, i = ps.generate_parallel_groups(world, do_cfg_guidance=False, sparse_type="full")
    ps.init_model_parallel(cfg_group_ranks=c, usp_group_ranks=u, iosp_dict=i)
    div = case["dividers"]
    cfg.num_layers, cfg.num_inference_steps = 1, len(div)
    rm = init_redundancy_map(cfg)
    for t, d in enumerate(div):
        rm.divider_map[t, 0] = d
    group = ps.get_isp_group()
    if case.get("transport") == "peer":
        from ditango_b200.core.peer_transport import PeerCopyGroup
        group = PeerCopyGroup(group, timeout_s=60.0)
    layer = proAttention(0, group)
    layer.hop_grouping = case.get("hop_grouping", "single")
    B, S, H, D = case["B"], case["S"], case["H"], case["D"]
    data = drifting_qkv(B, S, H, D, len(div), seed=case["seed"], drift=case["drift"], dtype=torch.bfloat16)
    lo, hi = rank * S // world, (rank + 1) * S // world
    outs = []
    for t in range(len(div)):
        update_timestep(t)
        ql, kl, vl = (x[:, lo:hi].contiguous().cuda() for x in data[t])
        if case.get("cu") is not None:
            cu = torch.tensor(case["cu"][rank], dtype=torch.int32).cuda()
            o = layer.varlen_attn(ql[0], kl[0], vl[0], cu_seqlens_q=cu, cu_seqlens_kv=cu,
                                  max_seqlen_q=hi - lo, max_seqlen_kv=hi - lo)[None]
        else:
            o = layer.attn(ql, kl, vl)
        outs.append(o.float().cpu())
    uly = None
    if case.get("ulysses"):
        ql, kl, vl = (x[:, lo:hi].contiguous().cuda() for x in data[0])
        uly = ulysses_attention(ql, kl, vl, group=ps.get_isp_group()).float().cpu()
    status = ops.read_status()
    ret[rank] = (torch.stack(outs), dict(layer.stats), uly, status)
    dist.barrier()
    if case.get("transport") == "peer":
        group.close()
    dist.destroy_process_group()


def gpu_uneven_worker(rank, world, port, case, ret):
    """NCCL ranks, real kernels: uneven shards with the pad in a segment of its own, gathered pad-free."""
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world), RANK=str(rank),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    from ditango_b200 import ops
    from ditango_b200.core import parallel_state as ps
    from ditango_b200.core.attention import proAttention
    from ditango_b200.core.config import init_config
    from ditango_b200.core.redundancy_map import init_redundancy_map
    from ditango_b200.utils import (gather_sequence_shards, split_tensor_uneven, uneven_shard_cu_seqlens,
                                    update_timestep)
    cfg = init_config(None, make_output_dir=False)
    ps.init_distributed_environment(world_size=world, rank=rank, local_rank=rank, backend="nccl")
    c, u, i = ps.generate_parallel_groups(world, do_cfg_guidance=False, sparse_type="full")
    ps.init_model_parallel(cfg_group_ranks=c, usp_group_ranks=u, iosp_dict=i)
    cfg.num_layers, cfg.num_inference_steps = 1, 1
    init_redundancy_map(cfg)
    update_timestep(0)
    group = ps.get_isp_group()
    B, S, H, D = case["B"], case["S"], case["H"], case["D"]
    g = torch.Generator().manual_seed(case["seed"])
    q, k, v = (torch.randn(B, S, H, D, generator=g).to(torch.bfloat16) for _ in range(3))
    ql, kl, vl = (split_tensor_uneven(x, world, dim=1)[rank].contiguous().cuda() for x in (q, k, v))
    shard = ql.shape[1]
    cu, max_len = uneven_shard_cu_seqlens(S, world, rank, batch_size=B, device="cuda")
    out = proAttention(0, group).varlen_attn(ql.reshape(B * shard, H, D), kl.reshape(B * shard, H, D),
                                             vl.reshape(B * shard, H, D), cu_seqlens_q=cu, cu_seqlens_kv=cu,
                                             max_seqlen_q=max_len, max_seqlen_kv=max_len, batch_size=B)
    out = gather_sequence_shards(group, out.reshape(B, shard, H, D), S, dim=1)
    ret[rank] = (out.float().cpu(), ops.read_status())
    dist.barrier()
    dist.destroy_process_group()


def dit_worker(rank, world, port, mode, ret):
    """Tiny CogVideoX-shaped DiT on gloo ranks with the CPU engine: output must not depend on the
    number of ranks the sequence is sharded over."""
    cfg_, ps = _setup(rank, world, port)
    from tests import cpu_engine
    import ditango_b200.executor.cogvideox_dit as M
    M._engine = cpu_engine
    from ditango_b200.core.redundancy_map import init_redundancy_map
    cfg_.num_layers, cfg_.num_inference_steps = 2, 3
    init_redundancy_map(cfg_)
    dcfg = M.DiTConfig(num_layers=2, num_heads=4, head_dim=16, in_channels=4, patch_size=2, text_dim=32, time_dim=16,
                       frames=2, height=8, width=8, text_len=8)
    torch.manual_seed(0)
    model = M.CogVideoXDiT(dcfg, ps.get_isp_group(), mode=mode)
    g = torch.Generator().manual_seed(1)
    lat = torch.randn(1, 2, 4, 8, 8, generator=g)
    txt_c, txt_u = torch.randn(1, 8, 32, generator=g), torch.randn(1, 8, 32, generator=g)
    out = M.denoise(model, lat, txt_c, txt_u, num_steps=2)
    ret[rank] = out
    dist.barrier()
    dist.destroy_process_group()


def pair_worker(rank, world, port, case, ret):
    """proAttention under a per-pair reuse map on gloo ranks (CPU engine)."""
    cfg, ps = _setup(rank, world, port)
    import numpy as np
    from ditango_b200.core.attention import proAttention
    from ditango_b200.core.redundancy_map import init_redundancy_map
    from ditango_b200.utils import update_timestep
    from oracle.ring_oracle import drifting_qkv
    T = case["T"]
    cfg.num_layers, cfg.num_inference_steps = 1, T
    rm = init_redundancy_map(cfg)
    rm.set_pair_map(np.asarray(case["reusable"], dtype=bool)[:, None])      # [T, 1, N, N]
    layer = proAttention(0, ps.get_isp_group())
    layer.hop_grouping = case.get("hop_grouping", "single")
    B, S, H, D = case["B"], case["S"], case["H"], case["D"]
    data = drifting_qkv(B, S, H, D, T, seed=case["seed"], drift=case["drift"])
    outs = []
    for t in range(T):
        update_timestep(t)
        q, k, v = data[t]
        lo, hi = rank * S // world, (rank + 1) * S // world
        outs.append(layer.attn(*(x[:, lo:hi].contiguous() for x in (q, k, v))).clone())
    ret[rank] = (torch.stack(outs), dict(layer.stats))
    dist.barrier()
    dist.destroy_process_group()


def gpu_pair_worker(rank, world, port, case, ret):
    """NCCL ranks, real kernels, per-pair reuse map."""
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world), RANK=str(rank),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    import numpy as np
    from ditango_b200 import ops
    from ditango_b200.core import parallel_state as ps
    from ditango_b200.core.attention import proAttention
    from ditango_b200.core.config import init_config
    from ditango_b200.core.redundancy_map import init_redundancy_map
    from ditango_b200.utils import update_timestep
    from oracle.ring_oracle import drifting_qkv
    cfg = init_config(None, make_output_dir=False)
    ps.init_distributed_environment(world_size=world, rank=rank, local_rank=rank, backend="nccl")
    c, u, i = ps.generate_parallel_groups(world, do_cfg_guidance=False, sparse_type="full")
    ps.init_model_parallel(cfg_group_ranks=c, usp_group_ranks=u, iosp_dict=i)
    T = case["T"]
    cfg.num_layers, cfg.num_inference_steps = 1, T
    rm = init_redundancy_map(cfg)
    rm.set_pair_map(np.asarray(case["reusable"], dtype=bool)[:, None])
    layer = proAttention(0, ps.get_isp_group())
    B, S, H, D = case["B"], case["S"], case["H"], case["D"]
    data = drifting_qkv(B, S, H, D, T, seed=case["seed"], drift=case["drift"], dtype=torch.bfloat16)
    lo, hi = rank * S // world, (rank + 1) * S // world
    outs = []
    for t in range(T):
        update_timestep(t)
        outs.append(layer.attn(*(x[:, lo:hi].contiguous().cuda() for x in data[t])).float().cpu())
    ret[rank] = (torch.stack(outs), dict(layer.stats), ops.read_status())
    dist.barrier()
    dist.destroy_process_group()
