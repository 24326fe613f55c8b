"""Ulysses attention: head <-> sequence all-to-all around full-sequence attention on H/N heads.

Mirrors baseline/ulysses.py of the reference (`use-ulysses`): there q, k, v of the video and text
streams go through six list-form all-to-alls (:51-62), one full-sequence flash call (:99-113) and two
reverse all-to-alls (:121-124), each all-to-all wrapped in tensor_split + contiguous + cat copies
(core/group_coordinate.py:281-286).  Here the three tensors are re-laid-out by ONE strided-copy launch
into a send buffer, exchanged by ONE equal-split all-to-all, and unpacked by one launch; the way back
is one launch + one all-to-all + one launch.
"""
import math
from typing import Optional, Sequence, Tuple

import torch

from .. import ops as _engine
from ..core.parallel_state import get_isp_group, get_usp_group
from ..logger import init_logger
from ..timer import get_timer

logger = init_logger(__name__)


def heads_to_sequence(tensors: Sequence[torch.Tensor], group) -> Tuple[torch.Tensor, ...]:
    """Each x [B,S_loc,H,D] (this rank's tokens, all heads) -> [B,N*S_loc,H/N,D] (all tokens, this
    rank's head group), the effect of all_to_all(scatter_dim=heads, gather_dim=sequence)."""
    N = group.world_size
    if N == 1:
        return tuple(tensors)
    x0 = tensors[0]
    B, S, H, D = x0.shape
    assert H % N == 0, f"{H} heads do not split over {N} ranks"
    Hn, n = H // N, len(tensors)
    C = Hn * D * x0.element_size()
    send = torch.empty(N, n, B, S, Hn, D, dtype=x0.dtype, device=x0.device)
    _engine.copy_chunks([(x.contiguous(), send[0, i]) for i, x in enumerate(tensors)], C, (N, B, S),
                        (C, S * H * D * x0.element_size(), H * D * x0.element_size()),
                        (n * B * S * C, S * C, C))
    recv = torch.empty_like(send)
    group.all_to_all_single(recv, send)
    outs = tuple(torch.empty(B, N * S, Hn, D, dtype=x0.dtype, device=x0.device) for _ in range(n))
    _engine.copy_chunks([(recv[0, i], outs[i]) for i in range(n)], S * C, (N, B, 1),
                        (n * B * S * C, S * C, 0), (S * C, N * S * C, 0))
    return outs


def sequence_to_heads(x: torch.Tensor, group) -> torch.Tensor:
    """x [B,N*S_loc,H/N,D] -> [B,S_loc,H,D]: the reverse exchange."""
    N = group.world_size
    if N == 1:
        return x
    B, S_all, Hn, D = x.shape
    S = S_all // N
    C = Hn * D * x.element_size()
    send = torch.empty(N, B, S, Hn, D, dtype=x.dtype, device=x.device)
    _engine.copy_chunks([(x.contiguous(), send)], S * C, (N, B, 1), (S * C, N * S * C, 0), (B * S * C, S * C, 0))
    recv = torch.empty_like(send)
    group.all_to_all_single(recv, send)
    out = torch.empty(B, S, N * Hn, D, dtype=x.dtype, device=x.device)
    _engine.copy_chunks([(recv, out)], C, (N, B, S), (B * S * C, S * C, C), (C, S * N * C, N * C))
    return out


@get_timer("ulyssesAttn")
def ulysses_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, group=None,
                      softmax_scale: Optional[float] = None) -> torch.Tensor:
    """query, key, value: this rank's [B,S_loc,H,D] bf16 -> attention output [B,S_loc,H,D] bf16 over
    the whole sequence of the group."""
    group = group if group is not None else get_isp_group()
    D = query.shape[-1]
    with get_timer("A2A_1"):
        q, k, v = heads_to_sequence((query, key, value), group)
    out, _ = _engine.flash_partial(q, k, v, out_dtype=torch.bfloat16,
                                   softmax_scale=softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D))
    with get_timer("A2A_2"):
        return sequence_to_heads(out, group)


class CVX_UlyssesAttnProcessor:
    """Attention processor for CogVideoX-style blocks (`attn` provides to_q/to_k/to_v, optional
    norm_q/norm_k, to_out and `heads`).  Text tokens are placed before video tokens, rotary
    embedding (a callable `rotary_fn(x [B,H,S,D], image_rotary_emb)`) is applied to the video part
    with the unsharded tables, as in baseline/ulysses.py:66-91 of the reference."""

    def __init__(self, layer_id=-1, rotary_fn=None):
        self.layer_id = layer_id
        self.rotary_fn = rotary_fn
        g = get_usp_group()
        self.world_size, self.rank = (g.world_size, g.rank_in_group) if g.world_size > 1 else (1, 0)

    def __call__(self, attn, hidden_states, encoder_hidden_states, attention_mask=None, image_rotary_emb=None):
        group = get_isp_group()
        N = group.world_size
        B = hidden_states.shape[0]
        assert attn.heads % N == 0
        H, Hn = attn.heads, attn.heads // N

        def proj(x):
            return [f(x).view(B, x.shape[1], H, -1) for f in (attn.to_q, attn.to_k, attn.to_v)]
        q, k, v = heads_to_sequence(proj(hidden_states), group)
        eq, ek, ev = heads_to_sequence(proj(encoder_hidden_states), group)
        text_len = eq.shape[1]
        q, k, v = (torch.cat([a, b], dim=1) for a, b in ((eq, q), (ek, k), (ev, v)))
        if getattr(attn, "norm_q", None) is not None:
            q = attn.norm_q(q)
        if getattr(attn, "norm_k", None) is not None:
            k = attn.norm_k(k)
        if image_rotary_emb is not None:
            if self.rotary_fn is None:
                raise RuntimeError("image_rotary_emb given but no rotary_fn configured")
            q[:, text_len:] = self.rotary_fn(q[:, text_len:].transpose(1, 2), image_rotary_emb).transpose(1, 2)
            k[:, text_len:] = self.rotary_fn(k[:, text_len:].transpose(1, 2), image_rotary_emb).transpose(1, 2)
        D = q.shape[-1]
        out, _ = _engine.flash_partial(q.contiguous(), k.contiguous(), v.contiguous(), out_dtype=torch.bfloat16,
                                       softmax_scale=1.0 / math.sqrt(D))
        enc, vid = out[:, :text_len], out[:, text_len:]
        vid = sequence_to_heads(vid.contiguous(), group).flatten(2)
        enc = sequence_to_heads(enc.contiguous(), group).flatten(2)
        vid, enc = attn.to_out[1](attn.to_out[0](vid)), attn.to_out[1](attn.to_out[0](enc))
        return vid, enc
