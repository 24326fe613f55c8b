"""Run configuration with the reference's keys, precedence and globals (core/config.py:8-143 of the
reference): YAML keys with dashes become attributes with underscores; WORLD_SIZE / RANK /
LOCAL_RANK come from the environment; `do_preprocess` switches every mode off; without
`use_ditango` the divider set collapses to [1] (plain ring)."""
import copy
import os
import time
from pathlib import Path

import yaml

_DEFAULTS = {
    "model_name": "cogvideox1.5-5b",
    "ditango_base": "./ditango",
    "output_fn": "./result",
    "tag": "test",
    "num_layers": 42,
    "num_inference_steps": 5,
    "seed": 42,
    "enable_timing": False,
    "do_preprocess": False,
    "do_cfg_parallel": False,
    "use_ditango": True,
    "use_ulysses": False,
    "use_distrifusion": False,
    "use_pab": False,
    "stride_dividers": [8, 4, 2, 1],
    "stride_percentiles": [20, 50, 80],
}


class DiTangoConfig:
    def __init__(self, config_path=None, make_output_dir: bool = True):
        object.__setattr__(self, "config", copy.deepcopy(_DEFAULTS))
        if config_path is not None:
            self.load_from_file(config_path)
        c = self.config
        if c["do_preprocess"]:
            c["use_ditango"] = c["use_ulysses"] = c["use_distrifusion"] = c["use_pab"] = False
        if not c["use_ditango"]:
            c["stride_dividers"] = [1]
        stamp = time.strftime("%Y%m%d_%H%M")
        c["output_dir"] = os.path.join(c["output_fn"], f"{c['tag']}_{stamp}")
        if make_output_dir:
            os.makedirs(c["output_dir"], exist_ok=True)
        c["world_size"] = int(os.getenv("WORLD_SIZE", "1"))
        c["rank"] = int(os.getenv("RANK", "0"))
        c["local_rank"] = int(os.getenv("LOCAL_RANK", "0"))

    def load_from_file(self, config_path):
        path = Path(config_path)
        if not path.exists():
            print(f"Warning: Config file {path} for DiTango not found. Using default values.")
            return
        with open(path, "r") as f:
            for key, value in (yaml.safe_load(f) or {}).items():
                self.config[key.replace("-", "_")] = value

    def __getattr__(self, name):
        cfg = object.__getattribute__(self, "config")
        if name in cfg:
            return cfg[name]
        raise AttributeError(f"'DiTangoConfig' object has no attribute '{name}'")

    def __setattr__(self, name, value):
        self.config[name] = value

    def to_dict(self):
        return copy.deepcopy(self.config)

    def save_to_file(self, file_path):
        with open(file_path, "w") as f:
            yaml.dump(self.config, f, default_flow_style=False)


DITANGO_CONFIG = None


def init_config(config_path, make_output_dir: bool = True):
    global DITANGO_CONFIG
    DITANGO_CONFIG = DiTangoConfig(config_path=config_path, make_output_dir=make_output_dir)
    return DITANGO_CONFIG


def get_config():
    return DITANGO_CONFIG


def print_config():
    import torch.distributed as dist
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        print("\n===== DiTango Configuration =====", flush=True)
        for k, v in get_config().to_dict().items():
            print(f"{k}: {v}", flush=True)
        print("\n=================================", flush=True)
