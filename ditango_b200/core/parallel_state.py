"""Process-group registry with the reference's getters (core/parallel_state.py of the reference):
world / DP / CFG / USP groups and the inner/outer sequence-parallel pair per stride.  With the only
live setting of the reference (sparse_type 'full') the inner group (ISP) is the whole USP group and
every outer group (OSP) is a single rank."""
import os
from math import gcd
from typing import Dict, List, Optional, Tuple, Union

import torch
import torch.distributed as dist

from ..logger import init_logger
from .group_coordinate import GroupCoordinator

logger = init_logger(__name__)

_WORLD: Optional[GroupCoordinator] = None
_DP: Optional[GroupCoordinator] = None
_CFG: Optional[GroupCoordinator] = None
_USP: Optional[GroupCoordinator] = None
_IOSP_GROUP_DICT: Optional[Dict[int, Dict[str, GroupCoordinator]]] = None


def get_world_group() -> GroupCoordinator:
    assert _WORLD is not None, "world group is not initialized"
    return _WORLD


def get_dp_group() -> GroupCoordinator:
    assert _DP is not None, "data parallel group is not initialized"
    return _DP


def get_cfg_group() -> GroupCoordinator:
    assert _CFG is not None, "classifier free guidance parallel group is not initialized"
    return _CFG


def get_usp_group() -> GroupCoordinator:
    assert _USP is not None, "Unified sequence parallel group is not initialized"
    return _USP


def get_iosp_group(stride: Optional[int] = None) -> Tuple[GroupCoordinator, GroupCoordinator]:
    assert _IOSP_GROUP_DICT is not None, "IOSP groups are not initialized"
    if stride is None:
        assert len(_IOSP_GROUP_DICT) == 1, "Found more than 1 iosp group pair, need to provide stride"
        groups = next(iter(_IOSP_GROUP_DICT.values()))
    else:
        assert stride in _IOSP_GROUP_DICT, f"No IOSP groups found for stride={stride}"
        groups = _IOSP_GROUP_DICT[stride]
    return groups["osp"], groups["isp"]


def get_isp_group(stride: Optional[int] = None) -> GroupCoordinator:
    return get_iosp_group(stride)[1]


def get_osp_group(stride: Optional[int] = None) -> GroupCoordinator:
    return get_iosp_group(stride)[0]


def init_distributed_environment(world_size: int = -1, rank: int = -1, distributed_init_method: str = "env://",
                                 local_rank: int = -1, backend: str = "nccl"):
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl" and torch.cuda.is_available() and local_rank >= 0:
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, init_method=distributed_init_method, world_size=world_size,
                                rank=rank, **kw)
    if local_rank == -1:
        local_rank = int(os.environ.get("LOCAL_RANK", "0")) if distributed_init_method == "env://" else rank
    global _WORLD
    if _WORLD is None:
        _WORLD = GroupCoordinator([list(range(dist.get_world_size()))], local_rank, backend, group_name="world")
    else:
        assert _WORLD.world_size == dist.get_world_size(), "world group already initialized with a different world size"


def generate_parallel_groups(world_size: int, do_cfg_guidance: bool = True,
                             sparse_type: Union[List, str, None] = "full"):
    """Rank lists for the CFG, USP and (OSP, ISP) groups (core/parallel_state.py:129-208).
    With CFG parallelism the world splits into halves [0, w/2) and [w/2, w) that pair up as
    (i, i + w/2); otherwise one USP group holds every rank."""
    if world_size < 1:
        raise ValueError("World size must be positive")
    if isinstance(sparse_type, str):
        assert sparse_type in ("full", "sequential"), f"Sparse type can only be 'full' or 'sequential'! Found {sparse_type}."
    if isinstance(sparse_type, list):
        strides = list(sparse_type)
    elif sparse_type == "full":
        strides = [world_size // 2] if do_cfg_guidance else [world_size]
    else:
        strides = [1]
    iosp: Dict[int, Tuple] = {}
    if world_size == 1:
        for s in strides:
            iosp[s] = (None, None)
        return None, None, iosp
    if do_cfg_guidance:
        half = world_size // 2
        usp = [list(range(half)), list(range(half, world_size))]
        cfg = [[i, i + half] for i in range(half)]
    else:
        usp, cfg = [list(range(world_size))], None
    usp_size = len(usp[0])
    for s in strides:
        assert s % usp_size == 0 or usp_size % s == 0, f"Does not support stride={s} but usp_size={usp_size}"
        isp_size = gcd(usp_size, s)
        osp_size = usp_size // isp_size
        osp_groups, isp_groups = [], []
        for ranks in usp:
            osp_groups += [ranks[i:i + osp_size] for i in range(0, usp_size, osp_size)]
            isp_groups += [ranks[i::osp_size] for i in range(osp_size)]
        iosp[s] = (osp_groups, isp_groups)
    return cfg, usp, iosp


def init_model_parallel(dp_group_ranks=None, cfg_group_ranks=None, usp_group_ranks=None, iosp_dict=None,
                        backend: Optional[str] = None):
    assert dist.is_initialized()
    world_size = dist.get_world_size()
    backend = backend or dist.get_backend(get_world_group().device_group)
    singles = [[r] for r in range(world_size)]
    local_rank = get_world_group().local_rank
    global _DP, _CFG, _USP, _IOSP_GROUP_DICT
    assert _DP is None and _CFG is None and _USP is None, "model parallel groups are already initialized"
    _DP = GroupCoordinator(dp_group_ranks or singles, local_rank, backend, group_name="dp")
    if cfg_group_ranks is not None:
        assert all(len(g) <= 2 for g in cfg_group_ranks), "cfg_size can only be 1 or 2"
    _CFG = GroupCoordinator(cfg_group_ranks or singles, local_rank, backend, group_name="cfg")
    usp_group_ranks = usp_group_ranks or singles
    _USP = GroupCoordinator(usp_group_ranks, local_rank, backend, group_name="usp")
    if iosp_dict is not None:
        assert _IOSP_GROUP_DICT is None, "iosp sequence parallel group is already initialized"
        _IOSP_GROUP_DICT = {}
        for n, (osp_ranks, isp_ranks) in iosp_dict.items():
            _IOSP_GROUP_DICT[n] = {
                "osp": GroupCoordinator(osp_ranks or singles, local_rank, backend, group_name=f"osp_{n}"),
                "isp": GroupCoordinator(isp_ranks or usp_group_ranks, local_rank, backend, group_name=f"isp_{n}"),
            }


def destroy_model_parallel():
    global _DP, _CFG, _USP, _IOSP_GROUP_DICT
    for g in (_DP, _CFG, _USP):
        if g:
            g.destroy()
    if _IOSP_GROUP_DICT:
        for pair in _IOSP_GROUP_DICT.values():
            for g in pair.values():
                g.destroy()
    _DP = _CFG = _USP = _IOSP_GROUP_DICT = None


def destroy_distributed_environment():
    global _WORLD
    if _WORLD:
        _WORLD.destroy()
    _WORLD = None
    if dist.is_initialized():
        dist.destroy_process_group()
