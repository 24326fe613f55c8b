"""Per-layer store of cached partial-attention block states, resident in HBM.

Mirrors the reference's proCache (core/cache.py of the reference): a list of slots, one per block at
the current stride, each holding the fp32 (out [B,S,H,D], lse [B,H,S]) state of "all chunks of that
block" as last computed; `update_cache_blocks` re-blocks the list when the next step uses a coarser
stride (:49-72) and empties the slot that will be recomputed.  Differences: re-blocking merges all
member slots of a new block in ONE kernel pass (the reference chains pairwise merges, :28-46); the
block size used by the memory guard is computed from shapes (the reference allocates a zero block to
measure it, :89-101); slots may optionally hold bf16 `out` to halve the footprint.
"""
from typing import List, Optional, Tuple

import torch

from .. import ops as _engine
from .._capi import LSE_BHS
from ..logger import init_logger
from ..utils import get_timestep

logger = init_logger(__name__)

State = Tuple[torch.Tensor, torch.Tensor]


def _device_total_mb() -> float:
    if torch.cuda.is_available():
        return torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory / (1024 * 1024)
    return float("inf")


class proCache:
    def __init__(self, isp_size: int, layer_id: int, store_dtype: torch.dtype = torch.float32,
                 lse_layout: int = LSE_BHS):
        self.isp_size = isp_size
        self.curr_isp_stride = isp_size
        self.curr_block_num = isp_size
        self.layer_id = layer_id
        self.store_dtype = store_dtype
        self.lse_layout = lse_layout          # layout of every lse handed to store_block ([B,H,S] or [B,S,H])
        self.out_block_cache: List[Optional[torch.Tensor]] = [None] * isp_size
        self.lse_block_cache: List[Optional[torch.Tensor]] = [None] * isp_size
        self.block_size_mb: Optional[float] = None
        self.memory_constraint = 0.72 * _device_total_mb()

    # ------------------------------------------------------------------ slots
    def get_block(self, block_id: int) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        if block_id >= len(self.out_block_cache):
            logger.error(f"{get_timestep()} | Cache is not ready but trying to get cached value.")
        return self.out_block_cache[block_id], self.lse_block_cache[block_id]

    def store_block(self, block_id: int, out: torch.Tensor, lse: torch.Tensor):
        if out.dtype != self.store_dtype:
            out = out.to(self.store_dtype)
        self.out_block_cache[block_id] = out
        self.lse_block_cache[block_id] = lse

    def clear(self):
        logger.warning("============== Clear oCache =================")

    def _reset(self, n: int):
        self.out_block_cache = [None] * n
        self.lse_block_cache = [None] * n

    def _merge_blocks(self, new_block_num: int):
        assert self.curr_block_num % new_block_num == 0, f"Invalid block number {new_block_num} for merging."
        per = self.curr_block_num // new_block_num
        outs: List[Optional[torch.Tensor]] = [None] * new_block_num
        lses: List[Optional[torch.Tensor]] = [None] * new_block_num
        for i in range(new_block_num):
            members = [(self.out_block_cache[j], self.lse_block_cache[j], self.lse_layout)
                       for j in range(i * per, (i + 1) * per) if self.lse_block_cache[j] is not None]
            if not members:
                continue
            if len(members) == 1:
                outs[i], lses[i] = members[0][0], members[0][1]
                continue
            if self.store_dtype == torch.bfloat16:
                # the merged block leaves the kernel as bf16; no fp32 copy is written
                o = torch.empty(members[0][0].shape, dtype=torch.bfloat16, device=members[0][0].device)
                _, l = _engine.merge_states(members, lse_out_layout=self.lse_layout, out_bf16=o, fp32_out=False)
            else:
                o, l = _engine.merge_states(members, lse_out_layout=self.lse_layout)
            outs[i], lses[i] = o, l
        self.out_block_cache, self.lse_block_cache = outs, lses

    def update_cache_blocks(self, new_isp_stride: int, next_target_block_id: int):
        if new_isp_stride == self.isp_size:
            self.curr_isp_stride = self.curr_block_num = self.isp_size
            self._reset(self.isp_size)
        elif new_isp_stride == 0:
            self.curr_isp_stride, self.curr_block_num = 0, 1
            self._reset(1)
        else:
            new_block_num = self.isp_size // new_isp_stride
            assert new_block_num <= self.curr_block_num, "Invalid ISP stride."
            self.curr_isp_stride = new_isp_stride
            if new_block_num != self.curr_block_num:
                self._merge_blocks(new_block_num)
                self.curr_block_num = new_block_num
            self.out_block_cache[next_target_block_id] = None
            self.lse_block_cache[next_target_block_id] = None

    # ------------------------------------------------------------------ memory guard
    def set_block_size_mb(self, tensor: torch.Tensor) -> float:
        """Size of one cached block for a chunk shaped like `tensor` ([.., H, D]): fp32 values plus
        one fp32 lse per row, i.e. the bytes of a [.., H, D+1] fp32 tensor."""
        if self.block_size_mb is None:
            rows = tensor.numel() // tensor.shape[-1]
            self.block_size_mb = rows * (tensor.shape[-1] + 1) * 4 / (1024 ** 2)
        return self.block_size_mb

    def pass_memory_check(self, next_isp_stride: int, layer_id: int) -> bool:
        """False when growing the cache to the block count of `next_isp_stride` would push allocated
        device memory past 72 % of HBM (core/cache.py:103-128); the caller then keeps nothing."""
        if next_isp_stride == self.isp_size or self.block_size_mb is None:
            return True
        active = sum(1 for b in self.out_block_cache if b is not None)
        predicted = self.isp_size // next_isp_stride
        if predicted <= active:
            return True
        add_mb = self.block_size_mb * (predicted - active)
        cur_mb = torch.cuda.memory_allocated() / (1024 * 1024) if torch.cuda.is_available() else 0.0
        if cur_mb + add_mb > self.memory_constraint:
            logger.warning(f"T{get_timestep()}L{layer_id} | Memory check failed: {cur_mb + add_mb:.0f} MB > "
                           f"{self.memory_constraint:.0f} MB, setting stride {next_isp_stride} to {self.isp_size}")
            return False
        return True

    def cached_bytes(self) -> int:
        n = 0
        for o, l in zip(self.out_block_cache, self.lse_block_cache):
            if o is not None:
                n += o.numel() * o.element_size() + l.numel() * l.element_size()
        return n

    def report_cache_status(self, layer_id: int):
        filled = ["O" if o is not None else "X" for o in self.out_block_cache]
        logger.info(f"===== Cache Status: Layer {layer_id}, Timestep {get_timestep()} | stride {self.curr_isp_stride} | "
                    f"blocks [{' '.join(filled)}] | {self.cached_bytes() / 2**20:.1f} MB =====")
