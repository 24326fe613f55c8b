"""Generate tests/golden/*.npz by EXECUTING THE REFERENCE on CPU/gloo ranks.

Run where the reference (chen-yy20/ditango) is checked out:

    python tests/golden/make_golden.py --ref /path/to/reference

The reference's per-layer attention object (`proAttention.attn` / `.varlen_attn`) is driven
unmodified; only what cannot exist on a CPU box is shimmed:
  * `matplotlib` (imported by core/redundancy_map.py, not installed) -> empty stub modules;
  * `torch.cuda.get_device_properties` / `memory_allocated` (core/cache.py:22,123) -> fakes;
  * `flash_attn_func` / `flash_attn_varlen_func` (GPU-only third-party wheel) -> fp32
    softmax(QK^T/sqrt(D))V + logsumexp written here (NOT the oracle's implementation);
  * the reference directory is exposed as package `ditango` through a symlink in a temp dir.

Every case stores the reference's fp32 outputs per step and rank (optionally row-subsampled)
plus fp64 checksums of the full tensors, and the seeds / schedule needed to regenerate the
inputs with oracle.ring_oracle.drifting_qkv.  The committed .npz files are what
tests/test_oracle_golden.py replays; this script itself needs the reference and is never run
by the tests.
"""
import argparse
import math
import os
import sys
import tempfile
import types

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))


def _cpu_flash(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, return_attn_probs=False, **kw):
    scale = softmax_scale or 1.0 / math.sqrt(q.shape[-1])
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    lse = torch.logsumexp(s, dim=-1)
    o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.float()).to(q.dtype)
    return (o, lse, None) if return_attn_probs else o


def _cpu_flash_varlen(q, k, v, cu_q, cu_k, max_q, max_k, dropout_p=0.0, softmax_scale=None,
                      causal=False, return_attn_probs=False, **kw):
    T, H, D = q.shape
    out = torch.zeros_like(q)
    lse = torch.full((H, T), float("-inf"))
    cq, ck = cu_q.tolist(), cu_k.tolist()
    for i in range(len(cq) - 1):
        if cq[i + 1] <= cq[i] or ck[i + 1] <= ck[i]:
            continue
        o, l, _ = _cpu_flash(q[None, cq[i]:cq[i + 1]], k[None, ck[i]:ck[i + 1]], v[None, ck[i]:ck[i + 1]],
                             softmax_scale=softmax_scale, return_attn_probs=True)
        out[cq[i]:cq[i + 1]] = o[0]
        lse[:, cq[i]:cq[i + 1]] = l[0]
    return (out, lse, None) if return_attn_probs else out


def _worker(rank, world, case, refpkg, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world),
                      RANK=str(rank), LOCAL_RANK=str(rank))
    scratch = tempfile.mkdtemp(prefix="ditango_golden_")
    os.chdir(scratch)                       # init_config() mkdirs ./result/<tag>_<ts>
    m, mpp = types.ModuleType("matplotlib"), types.ModuleType("matplotlib.pyplot")
    m.pyplot = mpp
    sys.modules["matplotlib"], sys.modules["matplotlib.pyplot"] = m, mpp
    sys.path.insert(0, refpkg)
    sys.path.insert(0, REPO)

    class _Props:
        total_memory = 180 * 2 ** 30
    torch.cuda.get_device_properties = lambda i: _Props()
    torch.cuda.memory_allocated = lambda *a, **k: 0
    torch.set_num_threads(max(1, (os.cpu_count() or 8) // world))

    import ditango.core.attention as A
    A.flash_attn_func = _cpu_flash
    A.flash_attn_varlen_func = _cpu_flash_varlen
    from ditango.core.config import init_config
    from ditango.core import parallel_state as ps
    from ditango.core.redundancy_map import init_redundancy_map, get_redundancy_map
    from ditango.utils import update_timestep
    from oracle.ring_oracle import drifting_qkv

    T = len(case["dividers"])
    cfg = init_config(None)
    cfg.num_layers = 1
    cfg.num_inference_steps = T
    ps.init_distributed_environment(world_size=world, rank=rank, local_rank=rank, backend="gloo")
    c, u, i = ps.generate_parallel_groups(world, do_cfg_guidance=False, sparse_type="full")
    ps.init_model_parallel(cfg_group_ranks=c, usp_group_ranks=u, iosp_dict=i)
    init_redundancy_map(cfg)
    rm = get_redundancy_map()
    for t, d in enumerate(case["dividers"]):
        rm.divider_map[t, 0] = d

    layer = A.proAttention(0, ps.get_isp_group())
    events = []
    cache = layer.cache
    _put, _get = cache.store_block, cache.get_block

    def put(bid, o, l):
        events.append(("put", int(cur_t[0]), int(bid)))
        return _put(bid, o, l)

    def get(bid):
        o, l = _get(bid)
        events.append(("get", int(cur_t[0]), int(bid), l is not None))
        return o, l
    cache.store_block, cache.get_block = put, get
    cur_t = [0]

    B, S, H, D = case["B"], case["S"], case["H"], case["D"]
    data = drifting_qkv(B, S, H, D, T, seed=case["seed"], drift=case["drift"])
    outs = []
    for t in range(T):
        cur_t[0] = t
        update_timestep(t)
        q, k, v = data[t]
        lo, hi = rank * S // world, (rank + 1) * S // world
        ql, kl, vl = (x[:, lo:hi].contiguous() for x in (q, k, v))
        if case.get("cu") is not None:
            cu = torch.tensor(case["cu"][rank], dtype=torch.int32)
            mx = int(hi - lo)
            o = layer.varlen_attn(ql[0], kl[0], vl[0], cu_seqlens_q=cu, cu_seqlens_kv=cu,
                                  max_seqlen_q=mx, max_seqlen_kv=mx, batch_size=1)
            o = o[None]
        else:
            o = layer.attn(ql, kl, vl)
        outs.append(o.float().clone())
    ret[rank] = (torch.stack(outs).numpy(), events)
    dist.barrier()
    dist.destroy_process_group()


CASES = {
    # Benchmark configuration 1 (the CPU-runnable case): two ranks, B1 H4 S1024 D64 fp32, 4 steps, Bernoulli(0.5) reuse with
    # step 0 full -> dividers 1,2,2,1 is one draw of it that exercises both transitions.
    "cfg1_n2": dict(world=2, B=1, S=1024, H=4, D=64, seed=0, drift=0.05, dividers=[1, 2, 2, 1], row_step=16),
    # The seven-step schedule whose state-machine trace is known (strides 4,1,1,2,2,2,4).
    "trace_n4": dict(world=4, B=1, S=128, H=2, D=32, seed=1, drift=0.05, dividers=[1, 4, 4, 2, 2, 2, 1], row_step=1),
    # Batch of two, zero drift (cached states stay exact), legal 4->2->1 descent.
    "batch2_n4": dict(world=4, B=2, S=64, H=3, D=16, seed=2, drift=0.0, dividers=[1, 1, 1, 4, 4, 2, 2, 1, 1], row_step=1),
    # Eight ranks through dividers 8,4,2.
    "n8": dict(world=8, B=1, S=256, H=2, D=16, seed=3, drift=0.05,
               dividers=[1, 1, 1, 8, 8, 8, 8, 4, 4, 2, 2, 1, 1], row_step=1),
    # Packed path: per-rank (valid, pad) segment pairs of different lengths.
    "varlen_n4": dict(world=4, B=1, S=192, H=2, D=32, seed=4, drift=0.05, dividers=[1, 1, 2, 2, 1],
                      cu=[[0, 43, 48], [0, 39, 48], [0, 48, 48], [0, 45, 48]], row_step=1),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("DITANGO_REFERENCE", "reference"),
                    help="checkout of chen-yy20/ditango")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    refpkg = tempfile.mkdtemp(prefix="ditango_refpkg_")
    os.symlink(os.path.abspath(args.ref), os.path.join(refpkg, "ditango"))
    sys.path.insert(0, REPO)
    port = 29610
    for name, case in CASES.items():
        if args.only and name != args.only:
            continue
        world = case["world"]
        mgr = mp.Manager()
        ret = mgr.dict()
        port += 1
        mp.spawn(_worker, args=(world, case, refpkg, port, ret), nprocs=world, join=True)
        outs = np.stack([ret[r][0] for r in range(world)], axis=1)          # [T, world, B, S_loc, H, D]
        rs = case["row_step"]
        payload = dict(
            out=outs[:, :, :, ::rs].astype(np.float32),
            checksum=outs.astype(np.float64).sum(axis=(2, 3, 4, 5)),
            abs_checksum=np.abs(outs.astype(np.float64)).sum(axis=(2, 3, 4, 5)),
            dividers=np.asarray(case["dividers"], dtype=np.int64),
            meta=np.asarray([case["world"], case["B"], case["S"], case["H"], case["D"], case["seed"], rs], dtype=np.int64),
            drift=np.asarray(case["drift"], dtype=np.float64),
            events_rank1=np.asarray([list(e) + [0] * (4 - len(e)) if not isinstance(e[0], str) else
                                     [{"put": 0, "get": 1}[e[0]]] + [int(x) for x in e[1:]] + [0] * (4 - len(e))
                                     for e in ret[min(1, world - 1)][1]], dtype=np.int64).reshape(-1, 4),
        )
        if case.get("cu") is not None:
            payload["cu"] = np.asarray(case["cu"], dtype=np.int64)
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **payload)
        print(f"{name}: out {payload['out'].shape} -> {path} ({os.path.getsize(path) / 1024:.0f} KiB)")


if __name__ == "__main__":
    main()
