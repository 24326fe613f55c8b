#!/usr/bin/env python
"""Benchmark of the sequence-parallel attention path on N B200s of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload hunyuan|cogvideox|stepvideo]
                    [--mode ditango|ring|ulysses] [--impl ours|reference]

One step = one denoising step = one call of every layer's attention object (proAttention.attn, or
ulysses_attention) on that step's Q/K/V.  Synthetic inputs of the named model's attention shape:
step-0 Q,K,V ~ N(0,1), every later step adds N(0, 0.05^2) (HunyuanVideo: Q and K RMS-normalised);
the same tensors feed every layer, each layer keeping its own cache and pointer.  The sequence is
sharded over the N ranks (strong scaling); the redundancy schedule is Bernoulli(p) per (step, layer)
drawn from seed 0, legalised and screened, with the first three steps at full stride.

Rank 0 prints ONE JSON line.  `value` counts the FLOPs the kernels executed (4*B*H*Sq*Sk*D per
chunk pair), summed over ranks, divided by the max-over-ranks device time; `e2e` is the same metric
with every layer's inputs copied from pinned host memory and its output copied back inside the
timed region.  `--impl reference` times the CPU restatement of the reference's path (oracle/) on
the host cores on a bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B, H, D, S, layers, steps, reuse probability, rms-normalised q/k
    "hunyuan": dict(B=1, H=24, D=128, S=119056, layers=60, steps=50, p=0.7, rms=True,
                    desc="HunyuanVideo 720p attention shape (33x45x80 video + 256 text tokens)"),
    "cogvideox": dict(B=2, H=48, D=64, S=17776, layers=42, steps=50, p=0.6, rms=False,
                      desc="CogVideoX-5B self-attention shape (13x30x45 video + 226 text tokens)"),
    "stepvideo": dict(B=2, H=48, D=128, S=54808, layers=48, steps=50, p=0.5, rms=False,
                      desc="Stepvideo-T2V self-attention shape (26x34x62 tokens)"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(tensor=float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 1401.5))),
                    tensor_burst=float(d.get("bf16_tflops", 1669.0)), hbm=float(d.get("hbm_gbs", 6544.3)),
                    source="measured")
    return dict(tensor=1400.0, tensor_burst=1590.0, hbm=6650.0, source="fallback")


def flash_dram_traffic(B, S_q, H, D):
    """DRAM bytes of one flash launch on a square chunk pair, scaled from the ncu captures under
    profiles/ (dram__bytes_read.sum + dram__bytes_write.sum): 423.2 MB at B1 S14882 H24 D128 and
    517.1 MB at B2 S8888 H48 D64.  K and V of a head stay in L2 while its query tiles run, so traffic
    follows the tensor sizes (tokens x heads x head_dim), not the FLOPs."""
    ref = {128: (423.2e6, 1 * 14882 * 24 * 128), 64: (517.1e6, 2 * 8888 * 48 * 64)}[D]
    return ref[0] * (B * S_q * H * D) / ref[1]


def draw_dividers(steps, layers, world, p, seed=0):
    """Bernoulli(p) reuse per (step, layer); a reuse cell takes a divider drawn uniformly from
    {2,4,8} that divides the group size; step 0 is a full refresh."""
    rng = np.random.RandomState(seed)
    choices = [d for d in (2, 4, 8) if d <= world and world % d == 0]
    div = np.ones((steps, layers), dtype=np.int64)
    if choices:
        for t in range(1, steps):
            for l in range(layers):
                if rng.rand() < p:
                    div[t, l] = choices[rng.randint(len(choices))]
    return div


def draw_pair_map(workload, steps, layers, world, p, seed=0):
    """Per-pair reuse map reusable[t, l, src, dst] as the benchmark specification words it: Bernoulli(p) per (step, layer,
    source chunk, consumer) with step 0 all-fresh; for stepvideo the structured map "chunks more than
    two ring hops away are reusable after step 10"."""
    r = np.zeros((steps, layers, world, world), dtype=bool)
    if workload == "stepvideo":
        for src in range(world):
            for dst in range(world):
                if min((src - dst) % world, (dst - src) % world) > 2:
                    r[11:, :, src, dst] = True
    else:
        r = np.random.RandomState(seed).rand(steps, layers, world, world) < p
        r[0] = False
    for i in range(world):
        r[:, :, i, i] = False
    return r


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


# ------------------------------------------------------------------------------------------ ours
def make_inputs(w, rank, world, device, seed=0):
    B, H, D, S = w["B"], w["H"], w["D"], w["S"]
    S_loc = S // world
    g = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
    raw = [torch.randn(B, S_loc, H, D, generator=g, device=device, dtype=torch.float32) for _ in range(3)]
    return raw, g


def step_inputs(raw, gen, w, first):
    """Apply the per-step drift in place and return this step's bf16 q, k, v."""
    if not first:
        for x in raw:
            x.add_(torch.randn(x.shape, generator=gen, device=x.device, dtype=x.dtype), alpha=0.05)
    q, k, v = raw
    if w["rms"]:
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + 1e-6)
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + 1e-6)
    return q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)


# Miniature parity cases per group size: schedules that walk through full refresh, every divider the
# group size admits, re-blocking and the return to full stride.
PARITY_CASES = {
    2: dict(B=1, S=1024, H=4, D=64, seed=0, drift=0.05, dividers=[1, 2, 2, 1]),
    4: dict(B=2, S=1200, H=4, D=128, seed=1, drift=0.05, dividers=[1, 4, 4, 2, 2, 2, 1]),
    8: dict(B=1, S=2048, H=8, D=64, seed=2, drift=0.05, dividers=[1, 1, 1, 8, 8, 8, 8, 4, 4, 2, 2, 1, 1]),
}


def parity_miniature(world, rank, group, device):
    """Before anything is timed: the attention path on this job's real process group (NCCL) against the
    CPU oracle on a small seeded case -- ring with cached reuse over a schedule through every divider,
    and the Ulysses exchange.  The oracle is the checker only.  Returns this rank's worst errors."""
    from oracle import ring_oracle as O
    from ditango_b200 import ops
    from ditango_b200.baseline.ulysses import ulysses_attention
    from ditango_b200.core import redundancy_map as rmod
    from ditango_b200.core.attention import proAttention
    from ditango_b200.core.config import get_config
    from ditango_b200.utils import update_timestep
    case = PARITY_CASES.get(world)
    if case is None:
        return None
    cfg = get_config()
    keep = (cfg.num_layers, cfg.num_inference_steps)
    div = case["dividers"]
    cfg.num_layers, cfg.num_inference_steps = 1, len(div)
    rmod.destroy_redundancy_map()
    rm = rmod.init_redundancy_map(cfg, world_size=world)
    for t, d in enumerate(div):
        rm.divider_map[t, 0] = d
    layer = proAttention(0, group)
    B, S, H, D = case["B"], case["S"], case["H"], case["D"]
    data = O.drifting_qkv(B, S, H, D, len(div), seed=case["seed"], drift=case["drift"], dtype=torch.bfloat16)
    ref, states = O.run_ring_group(world, div, data)
    lo, hi = rank * S // world, (rank + 1) * S // world
    worst = dict(max_abs=0.0, mean_abs=0.0, lse_max=0.0, ulysses_max_abs=0.0)
    for t in range(len(div)):
        update_timestep(t)
        out = layer.attn(*(x[:, lo:hi].contiguous().to(device) for x in data[t])).float().cpu()
        e = (out - ref[t][rank]).abs()
        worst["max_abs"] = max(worst["max_abs"], e.max().item())
        worst["mean_abs"] = max(worst["mean_abs"], e.mean().item())
    got_lse = layer.last_lse.float().cpu().transpose(-1, -2).unsqueeze(-1)
    worst["lse_max"] = (got_lse - states[rank].last_lse).abs().max().item()
    q, k, v = data[0]
    full, _ = O.partial_attention(q, k, v, out_dtype=torch.float32)
    uly = ulysses_attention(*(x[:, lo:hi].contiguous().to(device) for x in (q, k, v)), group=group).float().cpu()
    worst["ulysses_max_abs"] = (uly - full[:, lo:hi]).abs().max().item()
    worst["status"] = float(ops.read_status())
    del layer
    rmod.destroy_redundancy_map()
    cfg.num_layers, cfg.num_inference_steps = keep
    update_timestep(0)
    return worst


def run_ours(args):
    import torch.distributed as dist
    from ditango_b200 import _capi, ops
    from ditango_b200.core import parallel_state as ps
    from ditango_b200.core.attention import proAttention, release_receive_slots
    from ditango_b200.core.config import init_config
    from ditango_b200.core.group_coordinate import SingleRankGroup
    from ditango_b200.core.redundancy_map import init_redundancy_map
    from ditango_b200.baseline.ulysses import ulysses_attention
    from ditango_b200.utils import update_timestep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    _capi.check(_capi.load().dtb_device_supported(), "dtb_device_supported")
    w = dict(WORKLOADS[args.workload])
    if args.layers:
        w["layers"] = args.layers
    if w["S"] % world or (args.mode == "ulysses" and w["H"] % world):
        raise SystemExit(f"workload {args.workload} does not shard over {world} ranks")

    cfg = init_config(None, make_output_dir=False)
    cfg.num_layers, cfg.num_inference_steps = w["layers"], w["steps"]
    cfg.use_ditango = args.mode == "ditango"
    if world > 1:
        ps.init_distributed_environment(world_size=world, rank=rank, local_rank=local_rank, backend="nccl")
        c, u, i = ps.generate_parallel_groups(world, do_cfg_guidance=False, sparse_type="full")
        ps.init_model_parallel(cfg_group_ranks=c, usp_group_ranks=u, iosp_dict=i)
        group = ps.get_isp_group()
        if args.transport == "peer":
            from ditango_b200.core.peer_transport import PeerCopyGroup
            group = PeerCopyGroup(group)
    else:
        group = SingleRankGroup(device)
    parity = None
    if world > 1 and not args.no_parity:
        mine = parity_miniature(world, rank, group, device)
        if mine is not None:
            keys = ["max_abs", "mean_abs", "lse_max", "ulysses_max_abs", "status"]
            tp = torch.tensor([mine[k] for k in keys], device=device, dtype=torch.float64)
            dist.all_reduce(tp, op=dist.ReduceOp.MAX)
            parity = {k: float(f"{x:.3e}") for k, x in zip(keys, tp.tolist())}
            parity["case"] = (f"proAttention.attn on this job's own group (transport {args.transport}) vs the CPU "
                              "oracle, max over ranks and steps: " + json.dumps(PARITY_CASES[world]))
            parity["within_tolerance"] = bool(parity["max_abs"] <= 2e-2 and parity["mean_abs"] <= 1e-3
                                              and parity["lse_max"] <= 1e-3 and parity["ulysses_max_abs"] <= 2e-2
                                              and parity["status"] == 0)
    rm = init_redundancy_map(cfg, world_size=world)
    reuse_cells = 0
    if args.mode == "ditango" and world > 1 and args.schedule == "pairs":
        rm.set_pair_map(draw_pair_map(args.workload, w["steps"], w["layers"], world, w["p"]))
    elif args.mode == "ditango" and world > 1:
        rm.divider_map = torch.from_numpy(draw_dividers(w["steps"], w["layers"], world, w["p"]))
        rm._refine_divider_map()
        rm.screen_self_sends()
    proAttention.hop_grouping = args.hop_grouping
    proAttention.chain_launches = {"auto": "auto", "on": True, "off": False}[args.chain]
    layers = [proAttention(l, group) for l in range(w["layers"])]
    raw, gen = make_inputs(w, rank, world, device)
    B, H, D, S = w["B"], w["H"], w["D"], w["S"]
    S_loc = S // world

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    t0 = args.first_step if (args.schedule == "pairs" and args.mode == "ditango") else 0

    def one_step(t, qkv, out_sink=None):
        update_timestep((t0 + t) % w["steps"])
        q, k, v = qkv
        last = None
        for l in range(w["layers"]):
            if args.mode == "ulysses":
                last = ulysses_attention(q, k, v, group=group)
            else:
                last = layers[l].attn(q, k, v)
        return last

    # ---------------------------------------------------------------- device-resident timing
    total_steps = args.warmup + args.steps
    for t in range(args.warmup):
        one_step(t, step_inputs(raw, gen, w, first=(t == 0)))
    # Inputs of the timed steps are produced before the clock starts and stay resident in HBM; when
    # K steps of inputs would not fit a 24 GB budget the prepared steps are cycled.
    step_bytes = 3 * B * S_loc * H * D * 2
    n_prepared = max(1, min(args.steps, int(24e9 // step_bytes)))
    prepared = [step_inputs(raw, gen, w, first=False) for _ in range(n_prepared)]
    barrier()
    status = ops.read_status()
    if status != 0:
        raise SystemExit(f"kernel status {status} during warm-up")
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ops.LaunchLog.reset(with_events=True)
    for L in layers:
        L.measure_comm = world > 1
        L.exposed_comm_ms()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    rx_before = sum(L.stats["bytes_received"] for L in layers)
    barrier()
    ev0.record()
    for t in range(args.warmup, total_steps):
        one_step(t, prepared[(t - args.warmup) % n_prepared])
    ev1.record()
    barrier()
    elapsed_ms = ev0.elapsed_time(ev1)
    rx_timed = sum(L.stats["bytes_received"] for L in layers) - rx_before
    if args.mode == "ulysses" and world > 1:
        # q, k, v out and the result back: (N-1)/N of each leaves the rank per layer call
        rx_timed = int(4 * (world - 1) / world * B * S_loc * H * D * 2) * w["layers"] * args.steps
    clocks = sampler.stop() if rank == 0 else None
    launches = ops.LaunchLog.count
    overlapped_here = ops.LaunchLog.overlapped
    flash_ms = [a.elapsed_time(b) for a, b, _ in ops.LaunchLog.events]
    flash_flops = [f for _, _, f in ops.LaunchLog.events]
    exposed_ms = sum(L.exposed_comm_ms() for L in layers)
    ops.LaunchLog.reset(with_events=False)
    for L in layers:
        L.measure_comm = False
    status = ops.read_status()
    if status != 0:
        raise SystemExit(f"kernel status {status} in the timed region")

    # ---------------------------------------------------------------- end-to-end (host buffers)
    # What a caller with host-resident activations pays per layer call: q and K||V (one buffer, two copies
    # instead of three) go pinned host -> device, the result comes back as bf16 -- the dtype the
    # reference's callers cast to at once (executor/cogvideox/attention_processor.py:80) -- with the cast
    # fused into the last kernel of the call (proAttention.output_dtype).
    e2e_steps = args.steps
    q, k, v = prepared[0]
    host_q = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    host_kv = torch.empty((2,) + tuple(k.shape), dtype=k.dtype).pin_memory()
    host_q.copy_(q)
    host_kv[0].copy_(k)
    host_kv[1].copy_(v)
    host_out = torch.empty(q.shape, dtype=torch.bfloat16).pin_memory()
    # Two device input slots: the copies of layer l+1 run on a copy stream while layer l computes;
    # results leave on a second copy stream.  Every byte still crosses PCIe inside the timed region.
    dev_q = [torch.empty_like(q) for _ in range(2)]
    dev_kv = [torch.empty((2,) + tuple(k.shape), dtype=k.dtype, device=device) for _ in range(2)]
    h2d = (host_q.numel() * host_q.element_size() + host_kv.numel() * host_kv.element_size()) * w["layers"]
    d2h = host_out.numel() * host_out.element_size() * w["layers"]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    for L in layers:
        L.output_dtype = torch.bfloat16

    def e2e_step(t):
        update_timestep((t0 + t) % w["steps"])
        main = torch.cuda.current_stream()

        def fetch(l):
            slot = l & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_free[slot])
                dev_q[slot].copy_(host_q, non_blocking=True)
                dev_kv[slot].copy_(host_kv, non_blocking=True)
                ev_in[slot].record(s_in)
        for slot in range(2):
            ev_free[slot].record(main)
        fetch(0)
        for l in range(w["layers"]):
            slot = l & 1
            if l + 1 < w["layers"]:
                fetch(l + 1)
            main.wait_event(ev_in[slot])
            qkv = (dev_q[slot], dev_kv[slot][0], dev_kv[slot][1])
            o = ulysses_attention(*qkv, group=group) if args.mode == "ulysses" else layers[l].attn(*qkv)
            ev_free[slot].record(main)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                host_out.copy_(o, non_blocking=True)
                o.record_stream(s_out)
        main.wait_stream(s_out)
    t_next = total_steps
    e2e_step(t_next)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ops.LaunchLog.reset(with_events=True)
    e0.record()
    for i in range(e2e_steps):
        e2e_step(t_next + 1 + i)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    e2e_flops = sum(f for _, _, f in ops.LaunchLog.events)
    ops.LaunchLog.reset(with_events=False)
    for L in layers:
        L.output_dtype = torch.float32

    # Host-side ceiling of that region: all ranks move the same bytes host <-> device at once with no
    # kernels in between (both directions concurrently, as the e2e region does).
    barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(2, min(w["layers"], 8))
    c0.record()
    for _ in range(reps):
        with torch.cuda.stream(s_in):
            dev_q[0].copy_(host_q, non_blocking=True)
            dev_kv[0].copy_(host_kv, non_blocking=True)
        with torch.cuda.stream(s_out):
            host_out.copy_(dev_q[1], non_blocking=True)
    torch.cuda.current_stream().wait_stream(s_in)
    torch.cuda.current_stream().wait_stream(s_out)
    c1.record()
    barrier()
    copy_ms = c0.elapsed_time(c1) / reps * w["layers"]       # per step, copies only

    # ---------------------------------------------------------------- plain ring, same steps
    # The comparison behind "exposed communication vs plain ring attention": the same code with an all-ones
    # divider map (every step a full refresh, every chunk fetched and attended; core/config.py:58-59 of the
    # reference makes that the behaviour of every mode but use-ditango).  Fresh layer objects, nothing cached.
    plain = None
    if world > 1 and args.mode == "ditango" and not args.no_plain_ring:
        stats_keep = [dict(L.stats) for L in layers]
        del layers
        release_receive_slots()
        torch.cuda.empty_cache()
        rm.set_pair_map(None)
        rm.divider_map = torch.ones(w["steps"], w["layers"], dtype=torch.long)
        ring_layers = [proAttention(l, group) for l in range(w["layers"])]

        def ring_step(t, qkv):
            update_timestep(t % w["steps"])
            for L in ring_layers:
                L.attn(*qkv)
        for t in range(min(args.warmup, 2)):
            ring_step(t, prepared[t % n_prepared])
        for L in ring_layers:
            L.measure_comm = True
            L.exposed_comm_ms()
        barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for t in range(args.steps):
            ring_step(2 + t, prepared[t % n_prepared])
        r1.record()
        barrier()
        plain = [r0.elapsed_time(r1), sum(L.exposed_comm_ms() for L in ring_layers)]
        layers = ring_layers
        if ops.read_status() != 0:
            raise SystemExit("kernel status non-zero in the plain-ring pass")
    else:
        stats_keep = [dict(L.stats) for L in layers]

    # ---------------------------------------------------------------- reduce over ranks
    stats = torch.tensor([elapsed_ms, e2e_ms, exposed_ms, copy_ms] + (plain if plain is not None else [0.0, 0.0]),
                         device=device, dtype=torch.float64)
    sums = torch.tensor([sum(flash_flops), e2e_flops, sum(flash_ms), float(len(flash_ms)), float(launches), float(overlapped_here)],
                        device=device, dtype=torch.float64)
    # whole-path roofline of this rank's timed steps: the slower of its MMA work at the measured bf16 peak
    # and its received KV bytes at the measured peer-copy bandwidth (770 GB/s per direction on this pool)
    pk = measured_peaks()
    roof = torch.tensor([max(sum(flash_flops) / (pk["tensor"] * 1e12), rx_timed / 770e9) * 1e3,
                         sum(flash_flops) / (pk["tensor"] * 1e12) * 1e3, rx_timed / 770e9 * 1e3],
                        device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
        dist.all_reduce(roof, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, exposed_ms, copy_ms, plain_ms, plain_exposed_ms = stats.tolist()
    tot_flops, tot_e2e_flops, tot_flash_ms, n_flash, tot_launches, overlapped = sums.tolist()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(w, 1, sample_seq=args.cpu_seq, min_seconds=10.0)
    if rank == 0:
        peaks = measured_peaks()
        value = tot_flops / (elapsed_ms * 1e-3) / 1e12
        per_launch_tflops = (tot_flops / n_flash) / (tot_flash_ms / n_flash * 1e-3) / 1e12 if n_flash else 0.0
        full_flops = 4.0 * B * H * float(S) * S * D * w["layers"] * args.steps
        line = {
            "metric": "attention TFLOP/s (executed FLOPs, whole job) and ms per denoising step",
            "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(elapsed_ms / args.steps, 3), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {w['desc']}; B={B} H={H} D={D} S={S}, {w['layers']} layers/step, "
                                   f"mode={args.mode}, sequence sharded over {world} rank(s)",
                       "mode": args.mode, "global_batch": B, "seq_len": S, "layers_per_step": w["layers"],
                       "l2": "inputs larger than L2 (Q,K,V of one layer call exceed 126 MB)",
                       "reuse_probability": w["p"] if (args.mode == "ditango" and world > 1) else 0.0,
                       "schedule": args.schedule if (args.mode == "ditango" and world > 1) else "none",
                       "hop_grouping": args.hop_grouping if (args.mode != "ulysses" and world > 1) else "none",
                       "transport": args.transport if (args.mode != "ulysses" and world > 1) else "none",
                       "chain_launches": args.chain if (args.mode != "ulysses" and world > 1) else "none"},
            "algorithmic_tflops_full_attention": round(full_flops / (elapsed_ms * 1e-3) / 1e12, 2),
            "exposed_comm_ms_per_step": round(exposed_ms / args.steps, 3),
            "pct_of_bf16_peak": round(100.0 * value / world / peaks["tensor_burst"], 2),
            "roofline": {"bound": "tensor", "achieved": round(per_launch_tflops, 2), "peak": peaks["tensor"],
                         "unit": "TFLOP/s", "frac": round(per_launch_tflops / peaks["tensor"], 4),
                         "peak_kind": f"{peaks['source']} sustained bf16 cuBLAS GEMM; burst {peaks['tensor_burst']}",
                         "kernel": f"flash_fwd_row_kernel<{D}>" if D == 128 else f"flash_fwd_pair_kernel<{D}>",
                         "launches_timed": int(n_flash),
                         "timed_unit": "one launch (a launch that overlaps the one before it: from that launch's end to its own)",
                         "overlapped_launches": int(overlapped),
                         "traffic": round(flash_dram_traffic(B, S_loc, H, D)),
                         "traffic_kind": "bytes per launch, scaled by tensor size from the ncu capture of a smaller chunk pair"},
            "clocks": clocks,
            "path_roofline": {"t_roof_ms_per_step": round(roof[0].item() / args.steps, 3),
                              "mma_ms_per_step": round(roof[1].item() / args.steps, 3),
                              "kv_transfer_ms_per_step": round(roof[2].item() / args.steps, 3),
                              "frac": round(roof[0].item() / elapsed_ms, 4),
                              "formula": "max over ranks of max(executed FLOPs / sustained bf16 peak, KV bytes received / 770 GB/s)"},
            "e2e": {"value": round(tot_e2e_flops / (e2e_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                    "ms_per_step": round(e2e_ms / e2e_steps, 3),
                    "h2d_bytes_per_step": int(h2d) * world, "d2h_bytes_per_step": int(d2h) * world,
                    "result_dtype": "bf16 (cast fused into the last kernel of each call)",
                    "host_copy_ms_per_step": round(copy_ms, 3),
                    "host_copy_gbs": round((h2d + d2h) * world / (copy_ms * 1e-3) / 1e9, 1),
                    "host_copy_kind": "the region's copies alone, all ranks at once, no kernels: the floor the "
                                      "host side sets for an e2e step"},
            "gpu_launches": int(tot_launches),
        }
        if parity is not None:
            line["parity"] = parity
        if plain_ms > 0:
            line["plain_ring"] = {"ms_per_step": round(plain_ms / args.steps, 3),
                                  "exposed_comm_ms_per_step": round(plain_exposed_ms / args.steps, 3),
                                  "kind": "same code, all-ones divider map (every chunk fetched and attended every step)"}
            line["exposed_comm_ratio_plain_over_ditango"] = round(plain_exposed_ms / max(exposed_ms, 1e-6), 2)
            line["step_time_ratio_plain_over_ditango"] = round(plain_ms / elapsed_ms, 3)
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        if hasattr(group, "close"):
            group.close()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------- CPU legs
def cpu_baseline(w, world, sample_seq=None, steps=1, min_seconds=0.0):
    """Times the CPU restatement of the reference's path (oracle/) on the host cores: one layer call
    per step on a sequence of `sample_seq` tokens per rank (same B, H, D), ranks simulated as
    threads of one process."""
    from oracle import ring_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(max(1, cores // world))
    B, H, D = w["B"], w["H"], w["D"]
    s_loc = max(256, (sample_seq or 4096) // world)      # the sample keeps ~sample_seq tokens in all
    S = s_loc * world
    data = O.drifting_qkv(B, S, H, D, 1, seed=0, dtype=torch.bfloat16, rms_norm_qk=w["rms"])
    t0 = time.perf_counter()
    flops, calls = 0.0, 0
    while calls < steps or (min_seconds and time.perf_counter() - t0 < min_seconds):
        q, k, v = data[0]
        if world == 1:
            for h0 in range(0, H, 4):         # head groups keep the score matrix under ~2 GB
                O.partial_attention(q[:, :, h0:h0 + 4], k[:, :, h0:h0 + 4], v[:, :, h0:h0 + 4])
        else:
            O.run_ring_group(world, [1], data, partial_dtype=torch.bfloat16)
        flops += 4.0 * B * H * float(S) * S * D
        calls += 1
    dt = time.perf_counter() - t0
    return {"value": round(flops / dt / 1e12, 4), "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "seconds": round(dt, 2),
            "sample": f"{calls} layer call(s) of the oracle at B={B} H={H} D={D} S={S} ({world} simulated rank(s)); "
                      f"full workload is S={w['S']} x {w['layers']} layers per step"}


def reference_sample_schedule(world, p, steps=8, seed=0):
    """Dividers of one layer for a `steps`-step sample: Bernoulli(p) reuse drawn like the GPU arm's
    schedule, legalised, screened, with the first step a full refresh."""
    from ditango_b200.core.config import init_config
    from ditango_b200.core import redundancy_map as rmod
    cfg = init_config(None, make_output_dir=False)
    cfg.num_layers, cfg.num_inference_steps = 1, steps
    rmod.destroy_redundancy_map()
    rm = rmod.init_redundancy_map(cfg, world_size=world)
    div = draw_dividers(steps, 1, world, p, seed=seed)
    for t in range(1, steps):          # a divider may only fall, or restart from 1 (core/redundancy_map.py:281-326)
        if div[t - 1, 0] != 1 and div[t, 0] > div[t - 1, 0]:
            div[t, 0] = 1
    rm.divider_map = torch.from_numpy(div)
    rm.screen_self_sends()
    out = [int(x) for x in rm.get_map()[:, 0].tolist()]
    rmod.destroy_redundancy_map()
    return out


def executed_reference(w, world, sample_seq, mode):
    """The reference's own proAttention.attn (the copy under oracle/_ref, made by oracle/make_ref.py) on
    `world` gloo ranks of this host, one layer, a few steps of the workload's schedule at a reduced
    sequence length.  None when the copy is absent or the group has one rank (the reference has no
    attention group then)."""
    from oracle import ref_runner as R
    if world < 2 or not R.available():
        return None
    B, H, D = w["B"], w["H"], w["D"]
    s_loc = max(256, (sample_seq or 4096) // world)
    div = reference_sample_schedule(world, w["p"]) if mode == "ditango" else [1] * 4
    case = dict(B=B, S=s_loc * world, H=H, D=D, dividers=div, rms=w["rms"], bf16=True)
    r = R.time_reference(world, case)
    return {"value": round(r["flops"] / r["seconds"] / 1e12, 4), "unit": "TFLOP/s", "cores": r["cores"], "kind": "reference",
            "seconds": round(r["seconds"], 2),
            "sample": f"the reference's proAttention.attn, unmodified, on {world} gloo ranks of this host (its GPU-only "
                      f"flash_attn call replaced by fp32 softmax arithmetic on the host cores): 1 layer x {len(div)} steps, "
                      f"dividers {div}, B={B} H={H} D={D} S={s_loc * world}; full workload is S={w['S']} x {w['layers']} layers per step"}


def config1_reference():
    """Benchmark configuration 1 at full size on the executed reference: 2 gloo ranks, B1 H4 S1024 D64 fp32,
    4 steps, dividers 1,2,2,1 (one Bernoulli(0.5) draw with step 0 a full refresh)."""
    from oracle import ref_runner as R
    if not R.available():
        return None
    r = R.time_reference(2, dict(B=1, S=1024, H=4, D=64, dividers=[1, 2, 2, 1], bf16=False, seed=0), port=29890)
    return {"ms_per_step": round(r["seconds"] / r["steps"] * 1e3, 2), "tflops": round(r["flops"] / r["seconds"] / 1e12, 4),
            "ranks": 2, "cores": r["cores"], "kind": "reference",
            "config": "B=1 H=4 S=1024 D=64 fp32, 4 steps, dividers [1,2,2,1], one layer"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = dict(WORKLOADS[args.workload])
    t_all = []
    executed_failed = None
    for i in range(args.warmup + args.steps):
        cpu = None
        if executed_failed is None:
            try:
                cpu = executed_reference(w, args.gpus, args.cpu_seq, args.mode)
            except Exception as e:  # noqa: BLE001 - the arm still reports, on the port, and says why
                executed_failed = f"{type(e).__name__}: {str(e).strip().splitlines()[-1][:200] if str(e).strip() else ''}"
        if cpu is None:
            cpu = cpu_baseline(w, args.gpus, sample_seq=args.cpu_seq, steps=1, min_seconds=4.0)
        if i >= args.warmup:
            t_all.append(cpu)
    t_all = [c for c in t_all if c["kind"] == t_all[-1]["kind"]]
    value = statistics.mean(c["value"] for c in t_all)
    cpu = dict(t_all[-1], value=round(value, 4))
    if executed_failed is not None:
        cpu["executed_reference_failed"] = executed_failed
    try:
        c1 = config1_reference()
    except Exception as e:  # noqa: BLE001
        c1 = None
        cpu["config1_failed"] = f"{type(e).__name__}"
    if c1 is not None:
        cpu["config1"] = c1
    B, H, D, S = w["B"], w["H"], w["D"], w["S"]
    full_step_flops = 4.0 * B * H * float(S) * S * D * w["layers"]
    line = {
        "impl": "reference", "metric": "attention TFLOP/s (executed FLOPs, whole job) and ms per denoising step",
        "value": round(value, 4), "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(full_step_flops / (value * 1e12) * 1e3, 1),
        "ms_per_step_kind": "extrapolated from the sample's FLOP rate to one full-attention step of the workload",
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 inputs, fp32 arithmetic",
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: {w['desc']}; B={B} H={H} D={D} S={S}, {w['layers']} layers/step",
                   "mode": args.mode if cpu["kind"] == "reference" else "ring", "global_batch": B, "seq_len": S,
                   "layers_per_step": w["layers"]},
        "cpu_baseline": cpu,
        "e2e": {"value": round(value, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_dit(args):
    """Benchmark configuration 5: random-init CogVideoX-5B-shaped DiT (42 layers, hidden 3072, 48 x 64 heads),
    latent 13x60x90x16 + 226 text tokens, classifier-free guidance in-batch (B = 2), bf16; one step =
    one denoising step of the whole model.  Prints ms per step and exposed communication."""
    import torch.distributed as dist
    from ditango_b200 import _capi, ops
    from ditango_b200.core import parallel_state as ps
    from ditango_b200.core.attention import proAttention
    from ditango_b200.core.config import init_config
    from ditango_b200.core.group_coordinate import SingleRankGroup
    from ditango_b200.core.redundancy_map import init_redundancy_map
    from ditango_b200.executor.cogvideox_dit import CogVideoXDiT, DiTConfig, denoise

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    _capi.check(_capi.load().dtb_device_supported(), "dtb_device_supported")
    dcfg = DiTConfig()
    if args.layers:
        dcfg.num_layers = args.layers
    steps_total = 50
    cfg = init_config(None, make_output_dir=False)
    cfg.num_layers, cfg.num_inference_steps = dcfg.num_layers, steps_total
    cfg.use_ditango, cfg.use_ulysses = args.mode == "ditango", args.mode == "ulysses"
    if world > 1:
        ps.init_distributed_environment(world_size=world, rank=rank, local_rank=local_rank, backend="nccl")
        c, u, i = ps.generate_parallel_groups(world, do_cfg_guidance=False, sparse_type="full")
        ps.init_model_parallel(cfg_group_ranks=c, usp_group_ranks=u, iosp_dict=i)
        group = ps.get_isp_group()
        if args.transport == "peer" and args.mode != "ulysses":
            from ditango_b200.core.peer_transport import PeerCopyGroup
            group = PeerCopyGroup(group)
    else:
        group = SingleRankGroup(device)
    rm = init_redundancy_map(cfg, world_size=world)
    if args.mode == "ditango" and world > 1:
        rm.divider_map = torch.from_numpy(draw_dividers(steps_total, dcfg.num_layers, world, 0.6))
        rm._refine_divider_map()
        rm.screen_self_sends()
    torch.manual_seed(0)
    proAttention.hop_grouping = args.hop_grouping
    proAttention.chain_launches = {"auto": "auto", "on": True, "off": False}[args.chain]
    with torch.device(device):
        model = CogVideoXDiT(dcfg, group, mode=args.mode).to(torch.bfloat16)
    g = torch.Generator(device=device).manual_seed(0)
    latents = torch.randn(1, dcfg.frames, dcfg.in_channels, dcfg.height, dcfg.width, generator=g, device=device,
                          dtype=torch.float32).to(torch.bfloat16)
    text_c = torch.randn(1, dcfg.text_len, dcfg.text_dim, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    text_u = torch.randn(1, dcfg.text_len, dcfg.text_dim, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    layers = [b.attention for b in model.blocks if b.attention is not None]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    latents = denoise(model, latents, text_c, text_u, num_steps=args.warmup, first_step=0)
    barrier()
    for L in layers:
        L.measure_comm = world > 1
        L.exposed_comm_ms()
    ops.LaunchLog.reset(with_events=True)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    latents = denoise(model, latents, text_c, text_u, num_steps=args.steps, first_step=args.warmup)
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    flash_ms = sum(a.elapsed_time(b) for a, b, _ in ops.LaunchLog.events)
    flash_flops = sum(f for _, _, f in ops.LaunchLog.events)
    n_flash = len(ops.LaunchLog.events)
    launches = ops.LaunchLog.count
    exposed = sum(L.exposed_comm_ms() for L in layers)
    status = ops.read_status()
    stats = torch.tensor([ms, exposed, flash_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms, exposed, flash_ms = stats.tolist()
    if rank == 0:
        print(json.dumps({
            "metric": "ms per denoising step, random-init CogVideoX-5B-shaped DiT", "value": round(ms / args.steps, 3),
            "unit": "ms/step", "higher_is_better": False, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "dtype": "bf16", "data": "synthetic", "scaling": "strong",
            "config": {"workload": f"cogvideox-dit: {dcfg.num_layers} layers, hidden {dcfg.dim}, {dcfg.num_heads}x{dcfg.head_dim} heads, "
                                   f"{dcfg.video_tokens}+{dcfg.text_len} tokens, CFG batch 2, mode={args.mode}", "mode": args.mode,
                       "transport": args.transport if args.mode != "ulysses" else "none"},
            "exposed_comm_ms_per_step": round(exposed / args.steps, 3),
            "attention_kernel_ms_per_step": round(flash_ms / args.steps, 3),
            "attention_kernel_tflops": round(flash_flops / max(flash_ms, 1e-9) / 1e9, 1),
            "flash_launches": n_flash, "gpu_launches": launches, "kernel_status": status,
            "finite": bool(torch.isfinite(latents.float()).all().item())}), flush=True)
    if world > 1:
        dist.barrier()
        if hasattr(group, "close"):
            group.close()
        dist.destroy_process_group()


def run_micro(args):
    """Single-kernel timing on one GPU (also the small case the ncu captures under profiles/ use):
    one chunk pair of the workload at S/shard tokens (`flash`), an n-state merge at that shape
    (`merge`), or the Ulysses re-layout copy (`copy`).  Prints one JSON line."""
    from ditango_b200 import ops
    torch.cuda.set_device(0)
    w = WORKLOADS[args.workload]
    B, H, D, S = w["B"], w["H"], w["D"], w["S"] // args.shard
    peaks = measured_peaks()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape, dt=torch.float32: torch.randn(*shape, generator=g, device=dev, dtype=torch.float32).to(dt)
    if args.micro == "flash":
        q, k, v = (rnd(B, S, H, D, dt=torch.bfloat16) for _ in range(3))
        out = torch.empty(B, S, H, D, device=dev, dtype=torch.float32)
        lse = torch.empty(B, H, S, device=dev, dtype=torch.float32)
        fn = lambda: ops.flash_partial(q, k, v, out=out, lse=lse)
        work, unit, peak, bound = 4.0 * B * H * S * S * D, "TFLOP/s", peaks["tensor_burst"], "tensor"
    elif args.micro == "chain":
        # One layer call's worth of foreign chunks: n launches folded into one state, first without and then with
        # each launch allowed to overlap the end of the one before it.
        n = args.states
        q = rnd(B, S, H, D, dt=torch.bfloat16)
        kv = [(rnd(B, S, H, D, dt=torch.bfloat16), rnd(B, S, H, D, dt=torch.bfloat16)) for _ in range(n)]
        out = torch.empty(B, S, H, D, device=dev, dtype=torch.float32)
        lse = torch.empty(B, S, H, device=dev, dtype=torch.float32)

        # An event recorded long ago on another stream: waiting for it between two launches is what a transport's
        # "chunk has arrived" wait looks like to the compute stream when the chunk is already there.
        side = torch.cuda.Stream()
        landed = torch.cuda.Event()
        with torch.cuda.stream(side):
            landed.record()
        side.synchronize()
        cur = torch.cuda.current_stream()

        def chain(overlap, between=None):
            ops.flash_partial(q, kv[0][0], kv[0][1], out=out, lse=lse, lse_layout=ops.LSE_BSH)
            for kk, vv in kv[1:]:
                if between == "wait":
                    cur.wait_event(landed)
                elif between == "record":
                    torch.cuda.Event().record()
                ops.flash_partial(q, kk, vv, out=out, lse=lse, accumulate=True, lse_layout=ops.LSE_BSH,
                                  overlap_previous=overlap)
        res, ref, same = {}, None, True
        for name, overlap, between in (("separate", False, None), ("overlapped", True, None),
                                       ("overlapped_event_wait_between", True, "wait"),
                                       ("overlapped_event_record_between", True, "record")):
            for _ in range(max(1, args.warmup)):
                chain(overlap, between)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(max(1, args.steps)):
                chain(overlap, between)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / max(1, args.steps)
            res[name] = {"ms": round(ms, 4), "tflops": round(4.0 * B * H * S * S * D * n / (ms * 1e-3) / 1e12, 1)}
            if ref is None:
                ref = (out.clone(), lse.clone())
            same = same and bool(torch.equal(ref[0], out) and torch.equal(ref[1], lse))
        print(json.dumps({"micro": "chain", "workload": args.workload, "shape": dict(B=B, S=S, H=H, D=D), "launches": n,
                          **res, "speedup": round(res["separate"]["ms"] / res["overlapped"]["ms"], 4),
                          "bit_identical": same, "peak_burst": peaks["tensor_burst"], "status": ops.read_status()}), flush=True)
        return
    elif args.micro == "merge":
        n = args.states
        lay = ops.LSE_BSH if args.lse_layout == "bsh" else ops.LSE_BHS
        st = [(rnd(B, S, H, D), rnd(B, S, H) if lay == ops.LSE_BSH else rnd(B, H, S), lay) for _ in range(n)]
        fn = lambda: ops.merge_states(st, out=st[0][0], lse_out=st[0][1], lse_out_layout=lay)
        work, unit, peak, bound = float((n + 1) * B * S * H * (D * 4 + 4)), "GB/s", peaks["hbm"], "hbm"
    else:
        N = 8
        x = [rnd(B, S, H, D, dt=torch.bfloat16) for _ in range(3)]
        y = [torch.empty(N, B, S, H // N, D, device=dev, dtype=torch.bfloat16) for _ in range(3)]
        C = (H // N) * D * 2
        fn = lambda: ops.copy_chunks(list(zip(x, y)), C, (N, B, S), (C, S * H * D * 2, H * D * 2), (B * S * C, S * C, C))
        work, unit, peak, bound = float(2 * 3 * B * S * H * D * 2), "GB/s", peaks["hbm"], "hbm"
    for _ in range(max(1, args.warmup)):
        fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(max(1, args.steps)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    ms = statistics.mean(a.elapsed_time(b) for a, b in evs)
    rate = work / (ms * 1e-3) / (1e12 if bound == "tensor" else 1e9)
    print(json.dumps({"micro": args.micro, "workload": args.workload, "shape": dict(B=B, S=S, H=H, D=D),
                      "states": args.states if args.micro == "merge" else None,
                      "lse_layout": args.lse_layout if args.micro == "merge" else None, "ms": round(ms, 4),
                      "achieved": round(rate, 1), "unit": unit, "peak": peak, "frac": round(rate / peak, 4),
                      "status": ops.read_status()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="hunyuan", choices=sorted(WORKLOADS) + ["cogvideox-dit"])
    ap.add_argument("--mode", default="ditango", choices=["ditango", "ring", "ulysses"])
    ap.add_argument("--layers", type=int, default=0, help="override layers per step (debugging only)")
    ap.add_argument("--first-step", type=int, default=0,
                    help="--schedule pairs: denoising-step index of the first (warm-up) step; a per-pair cache "
                         "fills itself from any starting point, the stride schedule must start at step 0")
    ap.add_argument("--schedule", default="stride", choices=["stride", "pairs"],
                    help="ditango mode: stride schedule (what the reference can express) or a per-pair reuse map")
    ap.add_argument("--hop-grouping", default="single", choices=["single", "doubling"],
                    help="transport batches per call: one per hop, or batches of 1, 2, 4, ... hops")
    ap.add_argument("--transport", default="peer", choices=["nccl", "peer"],
                    help="KV hops by copy-engine copies into IPC-mapped buffers of the consumer (default: no SM is taken "
                         "from the attention kernel, full link rate per pair), or by NCCL send/receive")
    ap.add_argument("--chain", default="auto", choices=["auto", "on", "off"],
                    help="attention launches of one layer call that overlap the end of the launch before them "
                         "(proAttention.chain_launches): auto = launches below 5e11 FLOP, on = all, off = none")
    ap.add_argument("--cpu-seq", type=int, default=4096, help="tokens per rank of the CPU sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the parity miniature that runs before the warm-up at N > 1")
    ap.add_argument("--no-plain-ring", action="store_true", help="skip the plain-ring comparison pass at N > 1")
    ap.add_argument("--micro", default=None, choices=["flash", "merge", "copy", "chain"], help="time one kernel and exit")
    ap.add_argument("--shard", type=int, default=8, help="--micro: tokens = S / shard")
    ap.add_argument("--states", type=int, default=4, help="--micro merge: number of states; --micro chain: launches per chain")
    ap.add_argument("--lse-layout", default="bsh", choices=["bsh", "bhs"],
                    help="--micro merge: lse as [B,S,H] (what the attention path keeps internally) or [B,H,S]")
    args = ap.parse_args()
    if args.micro:
        return run_micro(args)
    if args.workload == "cogvideox-dit":
        return run_dit(args)
    if args.warmup < 3 and args.impl == "ours":
        print("warning: fewer than 3 warm-up steps", file=sys.stderr)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
