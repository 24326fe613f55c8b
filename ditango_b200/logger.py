"""Logging set-up with the reference's interface (logger.py:12-14, :80-93 of the reference):
`init_logger(name)`, level from LOG_LEVEL, optional per-process files under LOG_DIR."""
import logging
import os
import sys

_FORMAT = "%(levelname)s %(asctime)s [%(filename)s:%(lineno)d] %(message)s"
_configured = False


def _configure_root():
    global _configured
    if _configured:
        return
    root = logging.getLogger("ditango_b200")
    root.setLevel(getattr(logging, os.environ.get("LOG_LEVEL", "INFO").upper(), logging.INFO))
    h = logging.StreamHandler(sys.stdout)
    h.setFormatter(logging.Formatter(_FORMAT, datefmt="%m-%d %H:%M:%S"))
    root.addHandler(h)
    log_dir = os.environ.get("LOG_DIR")
    if log_dir:
        os.makedirs(log_dir, exist_ok=True)
        fh = logging.FileHandler(os.path.join(log_dir, f"ditango_{os.getpid()}.log"))
        fh.setFormatter(logging.Formatter(_FORMAT, datefmt="%m-%d %H:%M:%S"))
        root.addHandler(fh)
    root.propagate = False
    _configured = True


def init_logger(name: str) -> logging.Logger:
    _configure_root()
    short = name.split(".", 1)[1] if name.startswith(("ditango_b200.", "ditango.")) else name
    return logging.getLogger("ditango_b200." + short)
