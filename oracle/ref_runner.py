"""Times the REFERENCE's own per-layer attention object (the copy made by oracle/make_ref.py) on CPU/gloo
ranks of this host.  BENCHMARK INFRASTRUCTURE ONLY: the product never imports this.

The reference's hot path runs unmodified (core/attention.py:73-237 of the reference: proAttention.attn);
only what cannot exist on a CPU box is replaced, the same four shims tests/golden/make_golden.py uses:
matplotlib -> stub modules; torch.cuda.get_device_properties / memory_allocated (core/cache.py:22,123) ->
fakes; flash_attn_func (a GPU-only third-party wheel) -> fp32 softmax(QK^T/sqrt(D))V + logsumexp on the
host cores; the copy exposed as package `ditango`.
"""
import math
import os
import sys
import tempfile
import time
import types

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
REFPKG = os.path.join(HERE, "_ref")
_FLOPS = [0.0]


def available() -> bool:
    return os.path.exists(os.path.join(REFPKG, "ditango", "core", "attention.py"))


def _cpu_flash(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, return_attn_probs=False, **kw):
    scale = softmax_scale or 1.0 / math.sqrt(q.shape[-1])
    _FLOPS[0] += 4.0 * q.shape[0] * q.shape[2] * q.shape[1] * k.shape[1] * q.shape[3]
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    lse = torch.logsumexp(s, dim=-1)
    o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.float()).to(q.dtype)
    return (o, lse, None) if return_attn_probs else o


def _cpu_flash_varlen(q, k, v, cu_q, cu_k, max_q, max_k, dropout_p=0.0, softmax_scale=None, causal=False,
                      return_attn_probs=False, **kw):
    """Packed counterpart of _cpu_flash: segment i of q against segment i of k; rows of an empty pairing keep
    out = 0, lse = -inf."""
    T, H, _ = q.shape
    out = torch.zeros_like(q)
    lse = torch.full((H, T), float("-inf"))
    cq, ck = cu_q.tolist(), cu_k.tolist()
    for i in range(len(cq) - 1):
        if cq[i + 1] > cq[i] and ck[i + 1] > ck[i]:
            o, l, _ = _cpu_flash(q[None, cq[i]:cq[i + 1]], k[None, ck[i]:ck[i + 1]], v[None, ck[i]:ck[i + 1]],
                                 softmax_scale=softmax_scale, return_attn_probs=True)
            out[cq[i]:cq[i + 1]] = o[0]
            lse[:, cq[i]:cq[i + 1]] = l[0]
    return (out, lse, None) if return_attn_probs else out


def _worker(rank, world, case, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world),
                      RANK=str(rank), LOCAL_RANK=str(rank))
    os.chdir(tempfile.mkdtemp(prefix="ditango_ref_"))          # init_config() makes ./result/<tag>_<ts>
    m, mpp = types.ModuleType("matplotlib"), types.ModuleType("matplotlib.pyplot")
    m.pyplot = mpp
    sys.modules["matplotlib"], sys.modules["matplotlib.pyplot"] = m, mpp
    sys.path.insert(0, REFPKG)

    class _Props:
        total_memory = 180 * 2 ** 30
    torch.cuda.get_device_properties = lambda i: _Props()
    torch.cuda.memory_allocated = lambda *a, **k: 0
    torch.set_num_threads(max(1, (os.cpu_count() or 8) // world))

    import ditango.core.attention as A
    A.flash_attn_func = _cpu_flash
    A.flash_attn_varlen_func = _cpu_flash_varlen
    from ditango.core import parallel_state as ps
    from ditango.core.config import init_config
    from ditango.core.redundancy_map import get_redundancy_map, init_redundancy_map
    from ditango.utils import update_timestep

    div = case["dividers"]
    cfg = init_config(None)
    cfg.num_layers, cfg.num_inference_steps = 1, len(div)
    ps.init_distributed_environment(world_size=world, rank=rank, local_rank=rank, backend="gloo")
    c, u, i = ps.generate_parallel_groups(world, do_cfg_guidance=False, sparse_type="full")
    ps.init_model_parallel(cfg_group_ranks=c, usp_group_ranks=u, iosp_dict=i)
    init_redundancy_map(cfg)
    rm = get_redundancy_map()
    for t, d in enumerate(div):
        rm.divider_map[t, 0] = d
    layer = A.proAttention(0, ps.get_isp_group())
    B, S, H, D = case["B"], case["S"], case["H"], case["D"]
    g = torch.Generator().manual_seed(case.get("seed", 0) * 1000 + rank)
    dt = torch.bfloat16 if case.get("bf16", True) else torch.float32
    lo = S // world
    data = case.get("data")          # optional: per step (q, k, v) of the WHOLE sequence, sliced here by rank
    outs = [] if case.get("collect") else None
    if data is None:
        q, k, v = (torch.randn(B, lo, H, D, generator=g) for _ in range(3))
    seconds = 0.0
    for t in range(len(div)):
        if data is not None:
            q, k, v = (x[:, rank * lo:(rank + 1) * lo].contiguous() for x in data[t])
        elif t > 0:
            q, k, v = (x + case.get("drift", 0.05) * torch.randn(x.shape, generator=g) for x in (q, k, v))
        qq, kk = q, k
        if case.get("rms"):
            qq = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + 1e-6)
            kk = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + 1e-6)
        args = (qq.to(dt), kk.to(dt), v.to(dt))
        update_timestep(t)
        dist.barrier()
        t0 = time.perf_counter()
        if case.get("cu") is not None:       # packed: this rank's segment table, batch of one
            cu = torch.tensor(case["cu"][rank], dtype=torch.int32)
            o = layer.varlen_attn(args[0][0], args[1][0], args[2][0], cu_seqlens_q=cu, cu_seqlens_kv=cu,
                                  max_seqlen_q=lo, max_seqlen_kv=lo, batch_size=1)[None]
        else:
            o = layer.attn(*args)
        dist.barrier()
        seconds += time.perf_counter() - t0
        if outs is not None:
            outs.append(o.float().numpy().copy())
    ret[rank] = (seconds, _FLOPS[0], outs)
    dist.barrier()
    dist.destroy_process_group()


def time_reference(world, case, port=29790, limit_s=600.0):
    """Runs the reference's proAttention.attn for len(case['dividers']) steps of one layer on `world` gloo
    ranks (world >= 2: the reference has no attention group at one rank).  Returns
    dict(seconds, flops, steps, cores); with case["collect"] also the reference's outputs per rank and step
    (case["data"], per step (q, k, v) of the whole sequence, then replaces the harness's own random inputs)."""
    assert world >= 2 and available()
    mgr = mp.Manager()
    ret = mgr.dict()
    # The ranks are CPU processes: hide any GPU from them (the reference would otherwise put its receive
    # buffers on cuda:<rank>), and keep a launcher's rendezvous variables out of their environment.
    # (TORCHELASTIC_USE_AGENT_STORE would make rank 0 of the CPU group look for the launcher's store instead of
    # opening its own.)
    names = ["CUDA_VISIBLE_DEVICES", "MASTER_ADDR", "MASTER_PORT", "WORLD_SIZE", "RANK", "LOCAL_RANK",
             "LOCAL_WORLD_SIZE", "GROUP_RANK", "GROUP_WORLD_SIZE", "ROLE_RANK", "ROLE_WORLD_SIZE", "OMP_NUM_THREADS"]
    names += [k for k in os.environ if k.startswith("TORCHELASTIC_")]
    saved = {k: os.environ.get(k) for k in names}
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    for k in saved:
        if k != "CUDA_VISIBLE_DEVICES":
            os.environ.pop(k, None)
    try:
        ctx = mp.spawn(_worker, args=(world, case, port + int(time.time()) % 97, ret), nprocs=world, join=False)
        deadline = time.time() + limit_s
        while not ctx.join(timeout=5.0):
            if time.time() > deadline:
                for p in ctx.processes:          # the exact children started above
                    if p.is_alive():
                        p.terminate()
                raise TimeoutError(f"the reference's CPU ranks did not finish within {limit_s:.0f} s")
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    secs = max(ret[r][0] for r in range(world))
    flops = sum(ret[r][1] for r in range(world))
    res = dict(seconds=secs, flops=flops, steps=len(case["dividers"]), cores=os.cpu_count() or 1)
    if case.get("collect"):
        res["outputs"] = [ret[r][2] for r in range(world)]       # [rank][step] -> numpy [B, S_loc, H, D]
    return res
