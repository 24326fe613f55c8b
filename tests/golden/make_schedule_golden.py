"""Generate tests/golden/schedules.npz from the reference's shipped redundancy maps.

    python tests/golden/make_schedule_golden.py [--ref /path/to/reference]

For each model config of the reference (configs/<model>/redundancy_map_<T>_<L>.pt with the
stride-dividers / stride-percentiles of its config.yaml) the reference's OWN RedundancyMap code
(core/redundancy_map.py: generate_divider_map_from_redundancy + _refine_divider_map) is run for
group sizes 2, 4 and 8; the float map and the resulting divider maps are stored.  Needs the
reference checked out; never run by the tests.
"""
import argparse
import os
import sys
import tempfile
import types

import numpy as np
import torch
import yaml

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("DITANGO_REFERENCE", "reference"),
                    help="checkout of chen-yy20/ditango")
    args = ap.parse_args()
    m, mpp = types.ModuleType("matplotlib"), types.ModuleType("matplotlib.pyplot")
    m.pyplot = mpp
    sys.modules["matplotlib"], sys.modules["matplotlib.pyplot"] = m, mpp
    refpkg = tempfile.mkdtemp(prefix="ditango_refpkg_")
    os.symlink(os.path.abspath(args.ref), os.path.join(refpkg, "ditango"))
    sys.path.insert(0, refpkg)
    import ditango.core.redundancy_map as R

    payload = {}
    for model in sorted(os.listdir(os.path.join(args.ref, "configs"))):
        cdir = os.path.join(args.ref, "configs", model)
        with open(os.path.join(cdir, "config.yaml")) as f:
            cfg = {k.replace("-", "_"): v for k, v in yaml.safe_load(f).items()}
        T, L = int(cfg["num_inference_steps"]), int(cfg["num_layers"])
        path = os.path.join(cdir, f"redundancy_map_{T}_{L}.pt")
        red = torch.load(path, map_location="cpu")
        key = model.replace("-", "_").replace(".", "_")
        payload[f"{key}__map"] = red.numpy().astype(np.float32)
        payload[f"{key}__percentiles"] = np.asarray(cfg["stride_percentiles"], dtype=np.float64)
        payload[f"{key}__dividers"] = np.asarray(cfg["stride_dividers"], dtype=np.int64)
        for world in (2, 4, 8):
            R.get_usp_group = lambda w=world: types.SimpleNamespace(world_size=w)
            a = types.SimpleNamespace(num_inference_steps=T, num_layers=L)
            rm = R.RedundancyMap(a)
            rm.redundancy_map = red.clone()
            rm.generate_divider_map_from_redundancy(custom_percentages=cfg["stride_percentiles"],
                                                    custom_dividers=cfg["stride_dividers"])
            rm._refine_divider_map()
            dm = rm.divider_map.numpy().astype(np.int64)
            payload[f"{key}__div_n{world}"] = dm
            strides = np.array([[rm.get_curr_isp_stride(t, l) for l in range(L)] for t in range(T)], dtype=np.int64)
            nxt = np.array([[rm.get_next_isp_stride(t, l) for l in range(L)] for t in range(T)], dtype=np.int64)
            payload[f"{key}__stride_n{world}"] = strides
            payload[f"{key}__next_n{world}"] = nxt
            u, c = np.unique(dm, return_counts=True)
            print(model, world, dict(zip(u.tolist(), c.tolist())))
    out = os.path.join(HERE, "schedules.npz")
    np.savez_compressed(out, **payload)
    print(out, os.path.getsize(out) // 1024, "KiB")


if __name__ == "__main__":
    main()
