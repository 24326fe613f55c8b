"""`init_ditango(config_path)`: config -> process groups -> stride schedule -> timers, in the order
of the reference's core/initialize.py:17-66."""
import torch

from ..logger import init_logger
from ..timer import init_timer
from .config import init_config, print_config
from .parallel_state import (generate_parallel_groups, get_world_group, init_distributed_environment,
                             init_model_parallel)
from .redundancy_map import init_redundancy_map

logger = init_logger(__name__)
USE_DITANGO = False


def init_ditango(config_path: str = None, backend: str = "nccl"):
    from ..baseline.cache import init_easy_cache, init_fusion_cache
    from .. import _capi

    config = init_config(config_path)
    if backend == "nccl":
        torch.cuda.set_device(config.local_rank)
        _capi.check(_capi.load().dtb_device_supported(), "dtb_device_supported")
    init_distributed_environment(world_size=config.world_size, rank=config.rank, local_rank=config.local_rank,
                                 backend=backend)
    print_config()
    cfg_ranks, usp_ranks, iosp = generate_parallel_groups(config.world_size, do_cfg_guidance=config.do_cfg_parallel,
                                                          sparse_type="full")
    init_model_parallel(cfg_group_ranks=cfg_ranks, usp_group_ranks=usp_ranks, iosp_dict=iosp)
    rm = init_redundancy_map(config)
    if get_world_group().rank == 0:
        logger.info("===== DiTango Stride Map =====\n" + rm.stride_grid() + "\n=================================")
    if config.use_distrifusion:
        init_fusion_cache()
    elif config.use_pab:
        init_easy_cache()
    if config.enable_timing:
        init_timer(enable=False)      # pipelines switch timing on after the warm-up steps
    global USE_DITANGO
    USE_DITANGO = True
    logger.info(f"RANK {config.rank} - Initialized DiTango")


def is_ditango_initialized() -> bool:
    return USE_DITANGO
