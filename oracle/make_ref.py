"""Recipe for oracle/_ref/: a runnable copy of the REFERENCE's own attention path, for timing it on host
cores and for checking the oracle against it.  TEST / BENCHMARK INFRASTRUCTURE ONLY -- nothing in the
product package imports anything from oracle/.

    python oracle/make_ref.py --ref /path/to/chen-yy20/ditango

copies the reference's package files that its per-layer attention object needs (core/*.py, utils.py,
logger.py, timer.py, the empty __init__.py files) into oracle/_ref/ditango/, unmodified.  oracle/_ref/ is
git-ignored: the copy is a build output that lives beside the library's own built files, never part of
this repository's history.  oracle/ref_runner.py drives the copy on CPU/gloo ranks with the same four
shims tests/golden/make_golden.py uses.  Without a reference checkout the recipe does nothing and the
benchmark falls back to timing the oracle port.
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref", "ditango")
FILES = ["__init__.py", "utils.py", "logger.py", "timer.py",
         "core/__init__.py", "core/attention.py", "core/cache.py", "core/config.py", "core/group_coordinate.py",
         "core/initialize.py", "core/parallel_state.py", "core/redundancy_map.py"]


def make(ref: str) -> bool:
    if not os.path.isdir(os.path.join(ref, "core")):
        return False
    for rel in FILES:
        src = os.path.join(ref, rel)
        if not os.path.exists(src):
            continue
        dst = os.path.join(DEST, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(src, dst)
    return True


def available() -> bool:
    return os.path.exists(os.path.join(DEST, "core", "attention.py"))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("DITANGO_REFERENCE", "/root/reference"))
    a = ap.parse_args()
    ok = make(a.ref)
    print(f"oracle/_ref/ditango {'written from ' + a.ref if ok else 'NOT written: no reference checkout at ' + a.ref}")
    sys.exit(0)
