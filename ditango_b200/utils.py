"""Shared helpers with the reference's names (utils.py of the reference):
the global denoising-step index (:15-21), the two-state merge `update_out_and_lse` (:24-84) and the
zero-padded sequence sharding helpers (:86-167), plus two helpers the reference lacks that keep the pad
tokens out of attention (`uneven_shard_cu_seqlens`) and out of the gathered result (`gather_sequence_shards`)."""
from typing import Dict, List, Optional, Tuple

import torch

from . import ops as _engine
from ._capi import LSE_BHS, LSE_BSH

_PADDING_DICT: Dict[str, List[int]] = {}
_TIMESTEP: int = 0


def get_timestep() -> int:
    return _TIMESTEP


def update_timestep(timestep: int) -> None:
    global _TIMESTEP
    _TIMESTEP = timestep


def update_out_and_lse(out: Optional[torch.Tensor], lse: Optional[torch.Tensor],
                       block_out: torch.Tensor, block_lse: torch.Tensor,
                       slice_=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(out, lse) (+) (block_out, block_lse) with the reference's conventions (utils.py:44-84):
    `lse` is [..,S,H,1] (or [..,H,S]), `block_lse` is [..,H,S] (or [..,S,H,1]); the result is
    (fp32 out, lse [..,S,H,1]).  The first call (out is None) adopts the block.  One fused kernel
    launch instead of the reference's chain of elementwise ops."""
    if slice_ is not None:
        if out is None:
            raise RuntimeError("first update_out_and_lse should not pass slice_ args")
        so, sl = update_out_and_lse(out[slice_].contiguous(), lse[slice_].contiguous(), block_out, block_lse)
        out[slice_], lse[slice_] = so, sl
        return out, lse
    if block_lse.shape[-1] == 1 and block_lse.dim() == block_out.dim():
        b_lse, b_lay = block_lse.squeeze(-1).contiguous(), LSE_BSH
    else:
        b_lse, b_lay = block_lse.contiguous(), LSE_BHS
    states = []
    if out is not None:
        if lse.shape[-1] == 1 and lse.dim() == out.dim():
            a_lse, a_lay = lse.squeeze(-1).contiguous(), LSE_BSH
        else:
            a_lse, a_lay = lse.contiguous(), LSE_BHS
        states.append((out.contiguous(), a_lse, a_lay))
    states.append((block_out.contiguous(), b_lse, b_lay))
    new_out, new_lse = _engine.merge_states(states, lse_out_layout=LSE_BSH)
    return new_out, new_lse.unsqueeze(-1)


def rel_l1(new_tensor: torch.Tensor, ori_tensor: torch.Tensor) -> float:
    """Relative L1 drift of `new_tensor` against `ori_tensor` with the reference's conventions
    (utils.py:202-267): positions where either value is NaN are left out; mean|new - ori| /
    (mean|ori| + 1e-8); mean|new| when mean|ori| < 1e-6; +inf when no position is valid or the
    result is not finite.  Host-side form for tensors that live on the CPU (profiling on gloo ranks);
    on a GPU the profiling pass uses the device kernel behind ops.drift_accumulate instead."""
    valid = ~(torch.isnan(new_tensor) | torch.isnan(ori_tensor))
    if not bool(valid.any()):
        return float("inf")
    n, o = new_tensor[valid].double(), ori_tensor[valid].double()
    ori_mean = float(o.abs().mean())
    if ori_mean < 1e-6:
        return float(n.abs().mean())
    val = float((n - o).abs().mean()) / (ori_mean + 1e-8)
    return val if val == val and val not in (float("inf"), float("-inf")) else float("inf")


def split_tensor_uneven(tensor: torch.Tensor, world_size: int, dim: int = 1,
                        tensor_name: Optional[str] = None) -> List[torch.Tensor]:
    """Split `dim` into world_size shards of equal length ceil(len/world_size); the first
    len % world_size shards hold one real element more, the others are zero-padded at the end
    (utils.py:86-136).  Pad sizes are remembered under `tensor_name`."""
    n = tensor.shape[dim]
    base, rem = divmod(n, world_size)
    target = base + (1 if rem else 0)
    shards, pads, start = [], [], 0
    for i in range(world_size):
        length = base + (1 if i < rem else 0)
        piece = tensor.narrow(dim, start, length)
        pad = target - length
        if pad:
            shape = list(piece.shape)
            shape[dim] = pad
            piece = torch.cat([piece, piece.new_zeros(shape)], dim=dim)
        shards.append(piece)
        pads.append(pad)
        start += length
    if tensor_name is not None:
        _PADDING_DICT[tensor_name] = pads
    return shards


def get_padding_dict() -> Dict[str, List[int]]:
    return _PADDING_DICT


def remove_padding_after_gather(tensor: torch.Tensor, tensor_name: str) -> torch.Tensor:
    """Drop the pad rows (dim 1) that split_tensor_uneven added, after an all-gather of the shards
    (utils.py:142-167)."""
    if tensor_name not in _PADDING_DICT:
        return tensor
    pads = _PADDING_DICT[tensor_name]
    seg = tensor.size(1) // len(pads)
    if not any(pads):
        return tensor
    keep = torch.cat([torch.arange(r * seg, (r + 1) * seg - p, device=tensor.device) for r, p in enumerate(pads)])
    return tensor.index_select(1, keep)


def uneven_shard_lengths(total_len: int, world_size: int) -> List[int]:
    """Real tokens per shard for the split of split_tensor_uneven."""
    base, rem = divmod(total_len, world_size)
    return [base + (1 if i < rem else 0) for i in range(world_size)]


def uneven_shard_cu_seqlens(total_len: int, world_size: int, rank: int, batch_size: int = 1,
                            device=None) -> Tuple[torch.Tensor, int]:
    """Segment table that keeps the zero pad of an uneven shard out of attention.

    The reference pads short shards with zero tokens which then act as real keys in every layer
    (utils.py:117-127; nothing masks them).  Fed to `proAttention.varlen_attn` as cu_seqlens_q and
    cu_seqlens_kv of the packed shard `[batch * shard_len, H, D]`, this table puts each sample's real
    tokens in one segment and its pad tokens in another, so real queries see real keys only -- the same
    device the HunyuanVideo adapter uses for masked text (hunyuan_transformer.py:789-792).
    Returns (int32 cu_seqlens of length 2*batch + 1, max segment length)."""
    lengths = uneven_shard_lengths(total_len, world_size)
    shard = max(lengths)
    valid = lengths[rank]
    cu = [0]
    for b in range(batch_size):
        cu += [b * shard + valid, (b + 1) * shard]
    return torch.tensor(cu, dtype=torch.int32, device=device), shard


def gather_sequence_shards(group, local: torch.Tensor, total_len: int, dim: int = 1) -> torch.Tensor:
    """All-gather equal-length (padded) shards along `dim` and return exactly total_len positions: one
    all_gather_into_tensor, then one narrow copy per rank that skips its pad (what
    remove_padding_after_gather does through the name dictionary, utils.py:142-167)."""
    world = group.world_size
    if world == 1:
        return local.narrow(dim, 0, total_len)
    parts = group.all_gather(local, dim=0, split=True)
    lengths = uneven_shard_lengths(total_len, world)
    shape = list(local.shape)
    shape[dim] = total_len
    out = local.new_empty(shape)
    start = 0
    for part, n in zip(parts, lengths):
        out.narrow(dim, start, n).copy_(part.narrow(dim, 0, n))
        start += n
    return out
