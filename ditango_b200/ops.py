"""Tensor-level wrappers over the C ABI: torch tensors in, kernel launches on the current stream.

These are the only places arithmetic happens on the attention path; they raise when the
extension is missing or an argument is not a CUDA tensor of the expected kind.
"""
import ctypes
import math
from typing import Optional, Sequence, Tuple

import torch

from . import _capi
from ._capi import DTB_BF16, DTB_F32, LSE_BHS, LSE_BSH


class LaunchLog:
    """Optional accounting of kernel launches made through this module.  `count` always runs; with
    `events` enabled every flash launch is bracketed by two CUDA events on the launching stream so
    a benchmark can read per-launch device time and the FLOPs each launch executed.  (An event between two
    launches does not keep the second from overlapping the first; for a launch that overlaps its predecessor the
    pair then reads "end of the previous launch to end of this one", so the durations of a chain still add up to
    the chain's time.)"""
    count = 0
    events = None            # list of (start_event, end_event, flops) while enabled
    overlapped = 0           # flash launches made with overlap_previous

    @classmethod
    def reset(cls, with_events: bool = False):
        cls.count = 0
        cls.overlapped = 0
        cls.events = [] if with_events else None


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _capi.ExtensionError("ditango_b200 kernels take CUDA tensors only")


def _tok_stride(x: torch.Tensor) -> int:
    """Elements between consecutive tokens of a [..., H, D] tensor whose (H, D) block is dense and
    whose leading dims are laid out as one flat token axis."""
    if x.stride(-1) != 1 or x.stride(-2) != x.shape[-1]:
        raise _capi.ExtensionError("head and channel dims must be contiguous")
    ts = x.stride(-3)
    for d in range(x.dim() - 4, -1, -1):
        if x.shape[d] != 1 and x.stride(d) != x.stride(d + 1) * x.shape[d + 1]:
            raise _capi.ExtensionError("leading dims must flatten into one token axis")
    return ts


def read_status() -> int:
    """Synchronise the current stream and return (then clear) the device status word."""
    return _capi.load().dtb_read_status(_stream_ptr())


_STATUS_WATCH = {}      # device index -> [pinned int32 word, event behind the copy in flight or None]


def poll_status():
    """Non-blocking look at the device status word, for the hot path.  Each call tests the copy of
    the word that the previous call queued (if it has landed) and queues the next copy behind the
    work already on the current stream; it raises ExtensionError when a kernel reported that a bounded
    wait ran out -- from that point on launches skip their work and results are not valid.  The
    report therefore comes at most one poll late.  `read_status()` clears the word."""
    lib = _capi.load()
    dev = torch.cuda.current_device()
    watch = _STATUS_WATCH.get(dev)
    if watch is None:
        watch = _STATUS_WATCH[dev] = [torch.zeros(1, dtype=torch.int32).pin_memory(), None]
    host, pending = watch
    if pending is not None:
        if not pending.query():
            return                       # the earlier copy is still behind queued work
        watch[1] = None
        code = int(host[0])
        if code != 0:
            raise _capi.ExtensionError(
                f"a kernel gave up on a bounded wait (device status {code}); launches since then skipped "
                "their work -- results are not valid; read_status() clears the word")
    _capi.check(lib.dtb_peek_status_async(host.data_ptr(), _stream_ptr()), "dtb_peek_status_async")
    ev = torch.cuda.Event()
    ev.record()
    watch[1] = ev


def post_status(code: int):
    """Set the device status word from the host (ordered on the current stream): kernels in flight give
    up their bounded waits and later launches skip their work until read_status() clears it."""
    _capi.check(_capi.load().dtb_post_status(int(code), _stream_ptr()), "dtb_post_status")


def flash_partial(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
                  out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
                  accumulate: bool = False, out_dtype: torch.dtype = torch.float32,
                  lse_layout: int = LSE_BHS, softmax_scale: Optional[float] = None,
                  cu_seqlens_q: Optional[torch.Tensor] = None, cu_seqlens_k: Optional[torch.Tensor] = None,
                  max_seqlen_q: Optional[int] = None, max_seqlen_k: Optional[int] = None,
                  overlap_previous: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention state of q against one KV chunk.

    Dense: q [B,Sq,H,D], k,v [B,Sk,H,D] bf16.  Packed (cu_seqlens given): q [Tq,H,D], k,v [Tk,H,D].
    Returns (out, lse); with accumulate=True the chunk's state is merged into the given fp32
    (out, lse) in place.  lse is [B,H,Sq] / [H,Tq] (LSE_BHS) or [B,Sq,H] / [Tq,H] (LSE_BSH).

    overlap_previous=True lets the launch start while the launch queued just before it on the current stream
    is finishing (DTB_LAUNCH_OVERLAP_PREVIOUS).  Only pass it when the last kernel or copy queued on the
    stream was another flash_partial call -- event waits and event records in between are fine, they neither
    write memory nor keep the launches from overlapping -- and when q, k, v, cu_seqlens were not written by
    that call; (out, lse) may be the state that call wrote.
    """
    lib = _capi.load()
    _need_cuda(q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k)
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise _capi.ExtensionError("q, k, v must be bfloat16")
    packed = cu_seqlens_q is not None
    H, D = q.shape[-2], q.shape[-1]
    if packed:
        if q.dim() != 3:
            raise _capi.ExtensionError("packed q must be [T,H,D]")
        Tq, Tk = q.shape[0], k.shape[0]
        nseg = cu_seqlens_q.numel() - 1
        sq = int(max_seqlen_q if max_seqlen_q is not None else Tq)
        sk = int(max_seqlen_k if max_seqlen_k is not None else Tk)
        if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_k.dtype != torch.int32:
            raise _capi.ExtensionError("cu_seqlens must be int32")
        lse_shape = (H, Tq) if lse_layout == LSE_BHS else (Tq, H)
    else:
        if q.dim() != 4:
            raise _capi.ExtensionError("dense q must be [B,S,H,D]")
        B, sq = q.shape[0], q.shape[1]
        sk = k.shape[1]
        nseg, Tq, Tk = B, B * sq, B * sk
        lse_shape = (B, H, sq) if lse_layout == LSE_BHS else (B, sq, H)
    if accumulate:
        if out is None or lse is None or out.dtype != torch.float32:
            raise _capi.ExtensionError("accumulate needs an existing fp32 (out, lse) state")
    if out is None:
        out = torch.empty(q.shape, dtype=out_dtype, device=q.device)
    if lse is None:
        lse = torch.empty(lse_shape, dtype=torch.float32, device=q.device)
    if tuple(lse.shape) != tuple(lse_shape) or not lse.is_contiguous() or lse.dtype != torch.float32:
        raise _capi.ExtensionError(f"lse must be a contiguous fp32 tensor of shape {lse_shape}")
    if out.shape != q.shape:
        raise _capi.ExtensionError("out must have q's shape")
    odt = DTB_F32 if out.dtype == torch.float32 else DTB_BF16
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise _capi.ExtensionError("out must be float32 or bfloat16")
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    # dense: every query row meets every key row of its sequence; packed: upper bound by maxima
    flops = 4.0 * nseg * H * sq * sk * D
    ev = None
    if LaunchLog.events is not None:
        ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        ev[0].record()
    rc = lib.dtb_flash_fwd_ex(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), _tok_stride(q), _tok_stride(k), _tok_stride(v),
        out.data_ptr(), odt, _tok_stride(out), lse.data_ptr(), lse_layout, int(accumulate),
        cu_seqlens_q.data_ptr() if packed else None, cu_seqlens_k.data_ptr() if packed else None,
        nseg, sq, sk, Tq, Tk, H, D, scale, _capi.LAUNCH_OVERLAP_PREVIOUS if overlap_previous else 0, _stream_ptr())
    _capi.check(rc, "dtb_flash_fwd_ex")
    LaunchLog.count += 1
    LaunchLog.overlapped += int(bool(overlap_previous))
    if ev is not None:
        ev[1].record()
        LaunchLog.events.append((ev[0], ev[1], flops))
    return out, lse


def merge_states(states: Sequence[Tuple[torch.Tensor, torch.Tensor, int]], *,
                 out: Optional[torch.Tensor] = None, lse_out: Optional[torch.Tensor] = None,
                 lse_out_layout: int = LSE_BSH, out_bf16: Optional[torch.Tensor] = None,
                 want_lse: bool = True, fp32_out: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """One-pass merge of partial states.  states[i] = (out_i [B,S,H,D] fp32|bf16 contiguous,
    lse_i fp32 contiguous, layout_i).  Returns (out fp32 [B,S,H,D], lse_out or None).  With
    fp32_out=False only the bf16 copy `out_bf16` is written and returned in place of `out`."""
    lib = _capi.load()
    n = len(states)
    o0 = states[0][0]
    if o0.dim() == 3:
        B, (S, H, D) = 1, o0.shape
    else:
        B, S, H, D = o0.shape
    outs = (ctypes.c_void_p * n)()
    lses = (ctypes.c_void_p * n)()
    dts = (ctypes.c_int * n)()
    lays = (ctypes.c_int * n)()
    for i, (o, l, lay) in enumerate(states):
        _need_cuda(o, l)
        if not o.is_contiguous() or not l.is_contiguous() or o.shape != o0.shape:
            raise _capi.ExtensionError("states must be contiguous and of one shape")
        if l.dtype != torch.float32 or l.numel() != B * S * H:
            raise _capi.ExtensionError("lse must be fp32 with B*S*H entries")
        outs[i], lses[i] = o.data_ptr(), l.data_ptr()
        dts[i] = DTB_F32 if o.dtype == torch.float32 else DTB_BF16
        lays[i] = lay
    if not fp32_out:
        if out_bf16 is None:
            raise _capi.ExtensionError("fp32_out=False needs out_bf16")
        out = None
    elif out is None:
        out = torch.empty(o0.shape, dtype=torch.float32, device=o0.device)
    if out_bf16 is not None and (out_bf16.dtype != torch.bfloat16 or out_bf16.shape != o0.shape
                                 or not out_bf16.is_contiguous()):
        raise _capi.ExtensionError("out_bf16 must be a contiguous bfloat16 tensor of the states' shape")
    if not want_lse:
        lse_out = None
    if want_lse and lse_out is None:
        shape = ((B, S, H) if lse_out_layout == LSE_BSH else (B, H, S)) if o0.dim() == 4 else \
                ((S, H) if lse_out_layout == LSE_BSH else (H, S))
        lse_out = torch.empty(shape, dtype=torch.float32, device=o0.device)
    rc = lib.dtb_merge_states(
        n, outs, dts, lses, lays, out.data_ptr() if out is not None else None,
        lse_out.data_ptr() if lse_out is not None else None,
        lse_out_layout, out_bf16.data_ptr() if out_bf16 is not None else None, B, S, H, D, _stream_ptr())
    _capi.check(rc, "dtb_merge_states")
    LaunchLog.count += 1
    return (out if out is not None else out_bf16), lse_out


def copy_chunks(pairs: Sequence[Tuple[torch.Tensor, torch.Tensor]], chunk_bytes: int,
                extents: Tuple[int, int, int], src_strides: Tuple[int, int, int],
                dst_strides: Tuple[int, int, int]):
    """Strided chunk copy src -> dst for up to four tensor pairs in one launch (byte strides)."""
    lib = _capi.load()
    n = len(pairs)
    srcs = (ctypes.c_void_p * n)()
    dsts = (ctypes.c_void_p * n)()
    for i, (s, d) in enumerate(pairs):
        _need_cuda(s, d)
        srcs[i], dsts[i] = s.data_ptr(), d.data_ptr()
    rc = lib.dtb_copy_chunks(n, srcs, dsts, chunk_bytes, *extents, *src_strides, *dst_strides, _stream_ptr())
    _capi.check(rc, "dtb_copy_chunks")
    LaunchLog.count += 1


_DRIFT_SCRATCH = {}


def drift_accumulate(cur: torch.Tensor, prev: torch.Tensor, accum: torch.Tensor,
                     scratch: Optional[torch.Tensor] = None):
    """accum (one fp32 element on the device) += relative L1 drift of `cur` against `prev`
    (fp32, same number of elements), without a host round trip.  `scratch` defaults to a per-device
    buffer kept by this module and grown on demand."""
    lib = _capi.load()
    _need_cuda(cur, prev, accum, scratch)
    if cur.dtype != torch.float32 or prev.dtype != torch.float32 or accum.dtype != torch.float32:
        raise _capi.ExtensionError("drift_accumulate takes fp32 tensors")
    if cur.numel() != prev.numel() or accum.numel() != 1:
        raise _capi.ExtensionError("cur and prev must have equal sizes; accum must hold one element")
    cur, prev = cur.contiguous(), prev.contiguous()
    n = cur.numel()
    need = lib.dtb_drift_scratch_bytes(n)
    if scratch is None:
        key = cur.device
        scratch = _DRIFT_SCRATCH.get(key)
        if scratch is None or scratch.numel() < need:
            scratch = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=cur.device)
            _DRIFT_SCRATCH[key] = scratch
    rc = lib.dtb_drift_accumulate(cur.data_ptr(), prev.data_ptr(), n, accum.data_ptr(), scratch.data_ptr(),
                                  scratch.numel(), _stream_ptr())
    _capi.check(rc, "dtb_drift_accumulate")
    LaunchLog.count += 1
