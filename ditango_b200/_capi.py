"""ctypes binding of libditango_b200.so (C ABI declared in include/ditango_b200.h).

The library is the only compute path of this package.  If it has not been built, or the current
device is not compute capability 10.x, calls raise; nothing falls back to PyTorch arithmetic.
"""
import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p, POINTER

# DITANGO_B200_LIB points at a library built elsewhere (same ABI); default: the in-tree build.
_LIB_PATH = os.environ.get("DITANGO_B200_LIB") or os.path.join(
    os.path.dirname(os.path.abspath(__file__)), "lib", "libditango_b200.so")
_lib = None

DTB_F32, DTB_BF16 = 0, 1
LSE_BHS, LSE_BSH = 0, 1
MERGE_MAX_STATES = 16
LAUNCH_OVERLAP_PREVIOUS = 1

EXPORTS = (
    "dtb_version", "dtb_last_error", "dtb_device_supported", "dtb_read_status",
    "dtb_peek_status_async", "dtb_post_status",
    "dtb_ipc_export_mem", "dtb_ipc_open_mem", "dtb_ipc_close_mem", "dtb_peer_copy_async",
    "dtb_flash_fwd", "dtb_flash_fwd_ex", "dtb_merge_states", "dtb_copy_chunks",
    "dtb_drift_scratch_bytes", "dtb_drift_accumulate",
    "dtb_drift_noalloc_max_elements", "dtb_drift_accumulate_noalloc",
)


class ExtensionError(RuntimeError):
    pass


def lib_path() -> str:
    return _LIB_PATH


def load():
    """Load the shared library (once) and declare prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise ExtensionError(
            f"{_LIB_PATH} is missing: build it with `python -m ditango_b200._build` "
            "(there is no CPU or PyTorch fallback for the attention kernels)")
    lib = ctypes.CDLL(_LIB_PATH)
    lib.dtb_version.restype = c_int
    lib.dtb_last_error.restype = c_char_p
    lib.dtb_device_supported.restype = c_int
    lib.dtb_read_status.restype = c_int
    lib.dtb_read_status.argtypes = [c_void_p]
    lib.dtb_peek_status_async.restype = c_int
    lib.dtb_peek_status_async.argtypes = [c_void_p, c_void_p]
    lib.dtb_post_status.restype = c_int
    lib.dtb_post_status.argtypes = [c_int, c_void_p]
    lib.dtb_ipc_export_mem.restype = c_int
    lib.dtb_ipc_export_mem.argtypes = [c_void_p, c_void_p, POINTER(c_int64)]
    lib.dtb_ipc_open_mem.restype = c_int
    lib.dtb_ipc_open_mem.argtypes = [c_void_p, POINTER(c_void_p)]
    lib.dtb_ipc_close_mem.restype = c_int
    lib.dtb_ipc_close_mem.argtypes = [c_void_p]
    lib.dtb_peer_copy_async.restype = c_int
    lib.dtb_peer_copy_async.argtypes = [c_void_p, c_void_p, c_int64, c_void_p]
    lib.dtb_flash_fwd.restype = c_int
    lib.dtb_flash_fwd.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
        c_void_p, c_int, c_int64, c_void_p, c_int, c_int,
        c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64,
        c_int, c_int, c_float, c_void_p]
    lib.dtb_flash_fwd_ex.restype = c_int
    lib.dtb_flash_fwd_ex.argtypes = lib.dtb_flash_fwd.argtypes[:-1] + [c_int, c_void_p]
    lib.dtb_merge_states.restype = c_int
    lib.dtb_merge_states.argtypes = [
        c_int, POINTER(c_void_p), POINTER(c_int), POINTER(c_void_p), POINTER(c_int),
        c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    lib.dtb_copy_chunks.restype = c_int
    lib.dtb_copy_chunks.argtypes = [
        c_int, POINTER(c_void_p), POINTER(c_void_p), c_int64, c_int64, c_int64, c_int64,
        c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p]
    lib.dtb_drift_scratch_bytes.restype = c_int64
    lib.dtb_drift_scratch_bytes.argtypes = [c_int64]
    lib.dtb_drift_accumulate.restype = c_int
    lib.dtb_drift_accumulate.argtypes = [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p]
    lib.dtb_drift_noalloc_max_elements.restype = c_int64
    lib.dtb_drift_accumulate_noalloc.restype = c_int
    lib.dtb_drift_accumulate_noalloc.argtypes = [c_void_p, c_void_p, c_int64, c_void_p, c_void_p]
    _lib = lib
    return lib


def check(rc: int, what: str):
    if rc != 0:
        msg = load().dtb_last_error().decode()
        raise ExtensionError(f"{what} failed (status {rc}): {msg}")
