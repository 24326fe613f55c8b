"""Entry points of the reference's baseline caches (baseline/cache.py of the reference) that model
code imports unconditionally.  The DistriFusion and PAB baselines themselves are competing methods,
not part of the sequence-parallel attention path, and are not provided."""
_FUSION_CACHE = None
_EASY_CACHE = None


def init_fusion_cache():
    raise NotImplementedError("the DistriFusion baseline (use-distrifusion) is not part of this package")


def init_easy_cache():
    raise NotImplementedError("the PAB baseline (use-pab) is not part of this package")


def get_fusion_cache():
    return _FUSION_CACHE


def get_easy_cache():
    return _EASY_CACHE


def clear_cache():
    """Between prompts the reference clears its baseline caches here; the block cache of the
    attention path resets itself because step 0 always runs at full stride."""
    return None
