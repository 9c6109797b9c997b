"""Generates tests/golden/ref_model.json and ref_model_run.npz from the reference's own Python package.

The reference's model.py and sparseconvnet/*.py are imported as they are (its compiled extension
`sparseconvnet.SCN`, which cannot be built here, is replaced by a placeholder: constructing the modules never
calls into it).  Stored:
  ref_model.json     the state_dict keys and shapes of model.Naive_UNet and its module tree (class names, the
                     constructor-derived attributes of every layer), i.e. the topology a drop-in must reproduce
  ref_model_run.npz  what the CPU oracle computes when it walks THAT module tree (weights re-drawn from seeds
                     by name, see seeded_state) on a small seeded scene: a full frame and an incremental frame
Tests build the product's model the same way, load the same seeded weights and must get the same results.

Run from the repository root (needs the reference tree):  python tests/golden/make_golden_model.py
"""
import json
import os
import sys
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REFERENCE = "/root/reference"

ATTRS = ("nIn", "nOut", "nPlanes", "eps", "momentum", "leakiness", "affine", "mode", "dimension", "dilated_rate",
         "in_features", "out_features")


def seeded_state(state_dict_shapes):
    """name -> float32 array: every tensor re-drawn from a seed derived from its name, scaled so that activations
    stay O(1) through the network (weights ~ N(0, 2/fan_in), BatchNorm scale in [0.5, 1.5], variance in [0.5, 1.5])."""
    out = {}
    for name, shape in state_dict_shapes.items():
        rng = np.random.RandomState(zlib.crc32(name.encode()) & 0x7FFFFFFF)
        if name.endswith("num_batches_tracked"):
            continue
        if name.endswith("running_var"):
            a = rng.rand(*shape) + 0.5
        elif name.endswith("running_mean"):
            a = rng.randn(*shape) * 0.1
        elif len(shape) == 1 and name.endswith("weight"):
            a = rng.rand(*shape) + 0.5
        elif len(shape) == 1:
            a = rng.randn(*shape) * 0.1
        else:  # [volume, nIn, nOut] convolution, [nIn, nOut] 1x1 convolution, [out, in] torch Linear
            fan_in = shape[0] * shape[1] if len(shape) == 3 else shape[1] if "linear" in name else shape[0]
            a = rng.randn(*shape) * (2.0 / fan_in) ** 0.5
        out[name] = a.astype(np.float32)
    return out


def small_scene():
    sys.path.insert(0, os.path.join(ROOT, "ins-conv_b200"))
    from insconv import synth
    rng = np.random.RandomState(5)
    coords = np.concatenate([synth.box_surface((70, 66, 68), (100, 90, 84)), synth.sphere_surface((120, 110, 100), 12)], 0)
    coords = coords[rng.permutation(coords.shape[0])]
    feats = rng.uniform(-1, 1, size=(coords.shape[0], 3)).astype(np.float32)
    new = np.concatenate([synth.sphere_surface((96, 92, 88), 6), coords[rng.randint(0, coords.shape[0], 40)]], 0)
    new_feats = rng.uniform(-1, 1, size=(new.shape[0], 3)).astype(np.float32)
    return coords, feats, new, new_feats


def tree(module):
    d = {"class": type(module).__name__}
    for a in ATTRS:
        if hasattr(module, a) and isinstance(getattr(module, a), (int, float, bool)):
            d[a] = getattr(module, a)
    for a in ("filter_size", "filter_stride", "spatial_size"):
        if hasattr(module, a):
            d[a] = [int(v) for v in getattr(module, a)]
    kids = [tree(c) for c in module.children()]
    if kids:
        d["children"] = kids
    return d


def main():
    from unittest import mock
    sys.path.insert(0, REFERENCE)
    sys.modules["sparseconvnet.SCN"] = mock.MagicMock(name="SCN")  # the reference's extension: never called here
    import torch
    import model  # the reference's model.py
    net = model.Naive_UNet({"dimension": 3, "full_scale": 4096}).eval()
    shapes = {k: list(v.shape) for k, v in net.state_dict().items()}
    with open(os.path.join(HERE, "ref_model.json"), "w") as f:
        json.dump({"state_dict": shapes, "tree": tree(net)}, f, indent=0, sort_keys=True)
    net.load_state_dict({k: torch.from_numpy(v) for k, v in seeded_state(shapes).items()}, strict=False)
    sys.path.insert(0, ROOT)
    from oracle.scn_graph import GraphRunner
    coords, feats, new, new_feats = small_scene()
    run = GraphRunner(net)
    full = run([torch.from_numpy(coords), torch.from_numpy(feats)])
    inc = run([torch.from_numpy(new), torch.from_numpy(new_feats)], True)
    np.savez_compressed(os.path.join(HERE, "ref_model_run.npz"), full=full.numpy(), incremental=inc.numpy())
    print("parameters", sum(int(np.prod(s)) for s in shapes.values()), "full", tuple(full.shape), "incremental", tuple(inc.shape),
          "max|full|", float(full.abs().max()))


if __name__ == "__main__":
    main()
