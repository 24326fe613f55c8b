"""(step, layer) -> ISP stride schedule.

Mirrors the reference's RedundancyMap (core/redundancy_map.py of the reference): a float drift map
[T,L] (relative L1 distance between consecutive-step layer outputs) is quantised into a divider in
{8,4,2,1} per cell (:199-279), legalised so that a layer's divider only ever falls or restarts from
1 (:281-326), and looked up on the hot path as stride = group_size // divider (:49-87).
The lookup tables are plain Python ints, so the hot path does no tensor `.item()` calls.

Beyond the reference: `screen_self_sends()` resets the cells at which the reference's first-KV
exchange would address the sending rank itself, and `pair_map()` expands the schedule into the
boolean reusable[t, src, dst] view of one layer.
"""
import os
from typing import List, Optional

import numpy as np
import torch

from ..logger import init_logger
from .config import get_config
from .parallel_state import get_usp_group

logger = init_logger(__name__)


class RedundancyMap:
    def __init__(self, args, world_size: Optional[int] = None):
        self.num_timesteps = int(args.num_inference_steps)
        self.num_layers = int(args.num_layers)
        self.base_weight = int(world_size) if world_size is not None else get_usp_group().world_size
        self.stride_divider = [8, 4, 2, 1]
        self.map_percentage = [20, 50, 80]
        self.auto_setting = False
        self.calc_round = 0
        self.prev_out = [None] * self.num_layers
        self.redundancy_map: Optional[torch.Tensor] = None
        self._divider_map = self._init_map()
        self._table = None
        self._table_version = -1
        self._device_map = None          # [T,L] fp32 on the GPU while profiling there
        self.pair_reuse = None           # per-pair reuse map, see set_pair_map

    # The divider map stays a torch long tensor, as callers of the reference index and assign it
    # directly (`rm.divider_map[t, l] = d`); the int lookup table is rebuilt lazily after writes.
    @property
    def divider_map(self) -> torch.Tensor:
        self._table = None
        return self._divider_map

    @divider_map.setter
    def divider_map(self, value: torch.Tensor):
        self._divider_map = value
        self._table = None

    def _init_map(self) -> torch.Tensor:
        return torch.ones(self.num_timesteps, self.num_layers, dtype=torch.long)

    # ------------------------------------------------------------------ per-pair reuse (extension)
    def set_pair_map(self, reusable):
        """Switch the schedule to a per-pair reuse map reusable[t, l, src, dst] (bool array-like,
        [steps, layers, N, N]) or back to the stride schedule (None).  The reference has no such map:
        its (src, dst) pattern always follows from a stride and a rotating pointer.  With a pair map set,
        every attention object keeps one cached state per source chunk and refreshes exactly the pairs
        that are not flagged (or were never computed)."""
        if reusable is None:
            self.pair_reuse = None
            return
        arr = np.asarray(reusable, dtype=bool)
        N = self.base_weight
        assert arr.shape == (self.num_timesteps, self.num_layers, N, N), \
            f"pair map must be [steps, layers, {N}, {N}], got {arr.shape}"
        self.pair_reuse = arr

    def pair_flags(self, timestep: int, layer_id: int):
        """reusable[src][dst] of one cell as nested lists, or None when the stride schedule is active."""
        pr = self.pair_reuse
        if pr is None or self.auto_setting:
            return None
        return pr[timestep, layer_id].tolist()

    def _dividers(self) -> List[List[int]]:
        # The table is rebuilt after any in-place write to the tensor, whichever alias the caller wrote
        # through (`rm.divider_map[t, l] = d`, `rm.get_map()[t, l] = d`, a reference kept from earlier):
        # torch counts in-place writes per tensor.  In the reference every lookup reads the tensor.
        version = self._divider_map._version
        if self._table is None or self._table_version != version:
            self._table = self._divider_map.tolist()
            self._table_version = version
        return self._table

    def is_auto_setting(self) -> bool:
        return self.auto_setting

    def get_curr_isp_stride(self, timestep: int, layer_id: int) -> int:
        if self.auto_setting:
            return self.base_weight
        divider = self._dividers()[timestep][layer_id]
        if self.base_weight < divider:
            return 1
        assert self.base_weight % divider == 0, f"Invalid divider {divider} for base weight {self.base_weight}"
        return max(self.base_weight // divider, 1)

    def get_next_isp_stride(self, timestep: int, layer_id: int) -> int:
        if self.auto_setting or timestep == self.num_timesteps - 1:
            return self.base_weight
        divider = self._dividers()[timestep + 1][layer_id]
        if self.base_weight < divider:
            return 1
        assert self.base_weight % divider == 0, f"Invalid divider {divider} for base weight {self.base_weight}"
        return self.base_weight // divider

    def get_map(self) -> torch.Tensor:
        return self._divider_map

    def reset_map(self):
        self.divider_map = self._init_map()

    # ------------------------------------------------------------------ quantiser + legaliser
    def generate_divider_map_from_redundancy(self, custom_percentages=None, custom_dividers=None):
        if self.redundancy_map is None:
            logger.warning("Cannot generate divider map: no redundancy data available")
            return None
        percentages = list(custom_percentages) if custom_percentages is not None else self.map_percentage
        dividers = list(custom_dividers) if custom_dividers is not None else self.stride_divider
        red = self.redundancy_map.detach().cpu().numpy().astype(np.float64)
        nz = red[red > 0]
        if nz.size == 0:
            logger.warning("No non-zero redundancy values found, keeping default divider map")
            return None
        if len(dividers) < 4 or len(percentages) < 3:
            # A divider set like [1] (every mode but use_ditango) cannot be quantised against three
            # thresholds; the reference ends up with its all-ones map in that case: plain ring.
            self.divider_map = self._init_map()
            return None
        cuts = [float(np.percentile(nz, p)) for p in percentages]
        world = self.base_weight
        out = np.ones((self.num_timesteps, self.num_layers), dtype=np.int64)
        for t in range(self.num_timesteps - 1):
            for l in range(self.num_layers):
                r = red[t, l]
                if r <= 0:
                    continue
                d = dividers[0] if r < cuts[0] else dividers[1] if r < cuts[1] else dividers[2] if r < cuts[2] else dividers[3]
                if world < d:
                    d = world
                elif world % d != 0:
                    d = next((c for c in sorted(dividers) if world % c == 0 and c <= d), 1)
                out[t, l] = int(d)
        self.divider_map = torch.from_numpy(out)
        return cuts

    def _refine_divider_map(self) -> int:
        d = self._divider_map.clone()
        T, L = d.shape
        tab = d.tolist()
        for l in range(L):
            for t in range(1, T):
                if t < 3 or t > T - 3:
                    tab[t][l] = 1
                    continue
                if tab[t - 1][l] == 1 or tab[t][l] <= tab[t - 1][l]:
                    continue
                tab[t][l] = 1
        new = torch.tensor(tab, dtype=torch.long)
        changes = int((new != self._divider_map).sum().item())
        self.divider_map = new
        return changes

    # ------------------------------------------------------------------ pointer replay helpers
    def replay_layer(self, layer_id: int):
        """Integer replay of every rank's chunk pointer through all steps of one layer.  Returns a
        list (per step) of dicts: stride, target_block[r], self_send[r]."""
        N = self.base_weight
        ptr = [0] * N
        trace = []
        for t in range(self.num_timesteps):
            s = self.get_curr_isp_stride(t, layer_id)
            rec = dict(stride=s, target_block=[], self_send=[])
            for r in range(N):
                if s == N:
                    ptr[r] = r
                tb = ptr[r] // s
                rec["target_block"].append(tb)
                rec["self_send"].append(ptr[r] != r and tb * s + r % s == r)
                ptr[r] = (ptr[r] + (N if s == N else s)) % N
            trace.append(rec)
        return trace

    def screen_self_sends(self) -> int:
        """Reset to divider 1 (full refresh) the cells at which a rank's pointer is off its own chunk
        while its target block is its own block -- there the reference would exchange KV with
        itself and count its own chunk twice.  Returns the number of cells changed."""
        changed = 0
        for l in range(self.num_layers):
            while True:
                bad = next((t for t, rec in enumerate(self.replay_layer(l)) if any(rec["self_send"])), None)
                if bad is None:
                    break
                self.divider_map[bad, l] = 1
                changed += 1
        return changed

    def pair_map(self, layer_id: int) -> np.ndarray:
        """reusable[t, src, dst]: True when rank dst takes chunk src's contribution from its cache at
        step t instead of fetching and recomputing it."""
        N = self.base_weight
        out = np.zeros((self.num_timesteps, N, N), dtype=bool)
        for t, rec in enumerate(self.replay_layer(layer_id)):
            s = rec["stride"]
            if s == N:
                continue
            for dst in range(N):
                for src in range(N):
                    out[t, src, dst] = src != dst and src // s != rec["target_block"][dst]
        return out

    # ------------------------------------------------------------------ profiling mode
    def enable_auto_setting(self):
        self.auto_setting = True
        self.redundancy_map = torch.zeros(self.num_timesteps, self.num_layers, dtype=torch.float)
        self._device_map = None
        self.prev_out = [None] * self.num_layers

    def record_out_redundancy(self, timestep: int, layer_id: int, curr_out: torch.Tensor):
        """Profiling only (core/redundancy_map.py:174-197): add the relative L1 drift of this layer's
        output against the previous step's to cell (timestep, layer).  On the device the sums, the
        ratio and the accumulation happen in one kernel with no host round trip; the map is brought
        back by finish_auto_setting()."""
        if not self.auto_setting:
            return
        if self.redundancy_map is None:      # auto_setting switched on by assignment, as reference-era code may
            self.redundancy_map = torch.zeros(self.num_timesteps, self.num_layers, dtype=torch.float)
        prev = self.prev_out[layer_id]
        if prev is not None:
            if curr_out.is_cuda:
                from .. import ops
                if self._device_map is None:
                    self._device_map = torch.zeros(self.num_timesteps, self.num_layers, dtype=torch.float32,
                                                   device=curr_out.device)
                ops.drift_accumulate(curr_out.float(), prev.float(), self._device_map[timestep, layer_id])
            else:
                from ..utils import rel_l1
                self.redundancy_map[timestep, layer_id] += rel_l1(curr_out, prev)
        self.prev_out[layer_id] = curr_out

    def _collect_device_map(self):
        if self._device_map is not None:
            self.redundancy_map = self.redundancy_map + self._device_map.cpu()
            self._device_map = None

    def finished_one_round(self):
        self.calc_round += 1
        self.prev_out = [None] * self.num_layers

    def finish_auto_setting(self):
        if not self.auto_setting:
            return
        self._collect_device_map()
        if torch.distributed.is_initialized() and self.redundancy_map is not None:
            dev = get_usp_group().device
            red = self.redundancy_map.to(dev)
            torch.distributed.all_reduce(red, op=torch.distributed.ReduceOp.SUM)
            self.redundancy_map = (red / torch.distributed.get_world_size()).cpu()
        self.auto_setting = False
        self.prev_out = [None] * self.num_layers

    def stride_grid(self) -> str:
        world = self.base_weight
        d = torch.clamp_max(self._divider_map, world)
        return "\n".join(" ".join(f"{int(world // x):2d}" for x in row) for row in d.tolist())


_redundancy_map: Optional[RedundancyMap] = None


def init_redundancy_map(args, redun_map_path=None, custom_percentages=None, custom_dividers=None,
                        world_size: Optional[int] = None) -> RedundancyMap:
    """Build the process-wide schedule (core/redundancy_map.py:662-748): load
    <ditango_base>/configs/<model_name>/redundancy_map_<T>_<L>.pt when present, quantise with the
    configured percentiles / dividers, legalise; otherwise every cell is a full refresh."""
    global _redundancy_map
    assert _redundancy_map is None, "Stride map is already initialized"
    rm = RedundancyMap(args, world_size=world_size)
    _redundancy_map = rm
    if custom_percentages is None and hasattr(args, "stride_percentiles"):
        custom_percentages = args.stride_percentiles
    if custom_dividers is None and hasattr(args, "stride_dividers"):
        custom_dividers = args.stride_dividers
    if getattr(args, "use_pab", False):
        return rm
    if redun_map_path is None:
        default = os.path.join(f"{args.ditango_base}/configs/{args.model_name}/",
                               f"redundancy_map_{args.num_inference_steps}_{args.num_layers}.pt")
        if os.path.exists(default):
            redun_map_path = default
        else:
            logger.warning(f"No pre-computed redundancy map found at default location: {default}, "
                           "Using full stride map instead")
    if redun_map_path is not None and os.path.exists(redun_map_path):
        try:
            loaded = torch.load(redun_map_path, map_location="cpu")
            if tuple(loaded.shape) == (rm.num_timesteps, rm.num_layers):
                rm.redundancy_map = loaded
                rm.generate_divider_map_from_redundancy(custom_percentages, custom_dividers)
                rm._refine_divider_map()
            else:
                logger.warning(f"Loaded map dimensions {tuple(loaded.shape)} don't match required dimensions "
                               f"({rm.num_timesteps}, {rm.num_layers}). Using default map instead.")
        except Exception as e:  # an unreadable file degrades to the default map, as in the reference
            logger.warning(f"Failed to load redundancy map: {e}. Using default map instead.")
    return rm


def get_redundancy_map() -> Optional[RedundancyMap]:
    return _redundancy_map


def destroy_redundancy_map():
    global _redundancy_map
    _redundancy_map = None


def is_preprocessing() -> bool:
    return _redundancy_map is not None and _redundancy_map.is_auto_setting()


def save_redundancy_map(path=None, override=False):
    """Persist the float drift map as a plain fp32 [T,L] tensor, the reference's file format."""
    rm, cfg = get_redundancy_map(), get_config()
    if rm is None or rm.redundancy_map is None:
        return None
    if path is None:
        path = os.path.join(f"{cfg.ditango_base}/configs/{cfg.model_name}/",
                            f"redundancy_map_{cfg.num_inference_steps}_{cfg.num_layers}.pt")
    if os.path.exists(path) and not override:
        return None
    os.makedirs(os.path.dirname(path), exist_ok=True)
    torch.save(rm.redundancy_map.float().cpu(), path)
    return path


def redundancy_preprocess(*args, **kwargs):
    """Offline profiling driver of the reference (core/redundancy_map.py:863-900): it runs a model
    pipeline over a prompt list to fill the drift map.  Model pipelines are outside this package;
    callers drive `enable_auto_setting()` / `finish_auto_setting()` themselves."""
    raise NotImplementedError("redundancy_preprocess needs a model pipeline; use RedundancyMap.enable_auto_setting() "
                              "around your own denoising loop and finish_auto_setting() afterwards")
