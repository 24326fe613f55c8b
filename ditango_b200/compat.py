"""Make this package importable under the reference's name.

The reference's executors import `ditango.core.attention`, `ditango.utils`, `ditango.timer`, ...
(absolute imports of a package called `ditango`).  `install_as_ditango()` registers this package's
modules under those names, so `sample_video.py` and the model adapters run unchanged on top of the
sm_100a kernels."""
import importlib
import sys

_MODULES = (
    "", "utils", "timer", "logger", "core", "core.attention", "core.cache", "core.config",
    "core.group_coordinate", "core.initialize", "core.parallel_state", "core.redundancy_map",
    "baseline", "baseline.cache", "baseline.ulysses",
)


def install_as_ditango(name: str = "ditango"):
    for sub in _MODULES:
        mod = importlib.import_module("ditango_b200" + ("." + sub if sub else ""))
        sys.modules[name + ("." + sub if sub else "")] = mod
    return sys.modules[name]
