"""CPU stand-in for ditango_b200.ops, built on the oracle's arithmetic.  TEST-ONLY: the host-side
control plane (schedule, cache, transport order) is exercised on gloo ranks without a GPU by
swapping this in for the kernel wrappers.  The product package never imports it."""

import torch

from oracle import ring_oracle as O

LSE_BHS, LSE_BSH = 0, 1

# Per-thread record of what a rank queued on its (imaginary) stream, for tests of the launch-overlap
# contract: ("flash", overlap_previous) for attention launches, (kind, None) for everything else.  A
# transport stand-in reports its waits with log_op("wait").
OP_LOG = None            # dict thread id -> list while enabled


def log_op(kind, flag=None):
    if OP_LOG is not None:
        import threading
        OP_LOG.setdefault(threading.get_ident(), []).append((kind, flag))


def _to_bhs(lse, layout):
    return lse if layout == LSE_BHS else lse.transpose(-1, -2)


def flash_partial(q, k, v, *, out=None, lse=None, accumulate=False, out_dtype=torch.float32, lse_layout=LSE_BHS,
                  softmax_scale=None, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=None, max_seqlen_k=None,
                  overlap_previous=False):
    log_op("flash", bool(overlap_previous))
    if cu_seqlens_q is not None:
        o, l = O.partial_attention_varlen(q, k, v, cu_seqlens_q.tolist(), cu_seqlens_k.tolist(),
                                          softmax_scale=softmax_scale, out_dtype=torch.float32)
    else:
        o, l = O.partial_attention(q, k, v, softmax_scale=softmax_scale, out_dtype=torch.float32)
    if accumulate:
        mo, ml = O.merge_states(out, _to_bhs(lse, lse_layout), o, l)
        ml = ml.squeeze(-1)                      # [..,S,H]
        out.copy_(mo)
        lse.copy_(ml if lse_layout == LSE_BSH else ml.transpose(-1, -2))
        return out, lse
    res_l = l if lse_layout == LSE_BHS else l.transpose(-1, -2).contiguous()
    if out is not None:
        out.copy_(o.to(out.dtype))
        lse.copy_(res_l)
        return out, lse
    return o.to(out_dtype), res_l.contiguous()


def merge_states(states, *, out=None, lse_out=None, lse_out_layout=LSE_BSH, out_bf16=None, want_lse=True,
                 fp32_out=True):
    log_op("merge")
    o = l = None
    for so, sl, lay in states:
        o, l = O.merge_states(o, l, so.clone(), _to_bhs(sl, lay).clone())
    l = l.squeeze(-1)                            # [..,S,H]
    res_l = l if lse_out_layout == LSE_BSH else l.transpose(-1, -2)
    if not fp32_out:
        out_bf16.copy_(o.to(torch.bfloat16))
        if lse_out is not None:
            lse_out.copy_(res_l)
            res_l = lse_out
        return out_bf16, (res_l.contiguous() if want_lse else None)
    if out is not None:
        out.copy_(o)
        o = out
    if lse_out is not None:
        lse_out.copy_(res_l)
        res_l = lse_out
    if out_bf16 is not None:
        out_bf16.copy_(o.to(torch.bfloat16))
    return o, (res_l.contiguous() if want_lse else None)


def copy_chunks(pairs, chunk_bytes, extents, src_strides, dst_strides):
    log_op("copy")
    n0, n1, n2 = extents
    for src, dst in pairs:
        # raw-pointer semantics: offsets may reach beyond the given view into its buffer
        sb = torch.empty(0, dtype=torch.uint8).set_(src.untyped_storage())[src.storage_offset() * src.element_size():]
        db = torch.empty(0, dtype=torch.uint8).set_(dst.untyped_storage())[dst.storage_offset() * dst.element_size():]
        for i0 in range(n0):
            for i1 in range(n1):
                for i2 in range(n2):
                    so = i0 * src_strides[0] + i1 * src_strides[1] + i2 * src_strides[2]
                    do = i0 * dst_strides[0] + i1 * dst_strides[1] + i2 * dst_strides[2]
                    db[do:do + chunk_bytes] = sb[so:so + chunk_bytes]


def poll_status():
    return None


def _modules():
    import ditango_b200.core.attention as A
    import ditango_b200.core.cache as C
    import ditango_b200.utils as U
    import ditango_b200.baseline.ulysses as UL
    return (A, C, U, UL)


def install():
    """Point every module of the package that launches kernels at this stand-in."""
    import sys
    me = sys.modules[__name__]
    for m in _modules():
        m._engine = me


def uninstall():
    """Point them back at the kernel wrappers (for test processes that also run GPU tests)."""
    import ditango_b200.ops as real
    for m in _modules():
        m._engine = real
