"""Generates tests/golden/c1_small.npz: a small seeded boxes-and-spheres scene (config 1's generator on a
48^3 grid) with the oracle's site numbering, rulebooks and one 8->8 submanifold convolution.  The reference
itself cannot run in this environment, so the fixture freezes the oracle: any later change of the oracle's
behaviour shows up as a diff against these arrays.  Run from the repository root:
    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "ins-conv_b200"))

from insconv import synth  # noqa: E402
from oracle import scn_oracle as O  # noqa: E402


def main():
    rng = np.random.RandomState(42)
    parts = [synth.box_surface((4, 5, 6), (20, 18, 15)), synth.sphere_surface((30, 30, 28), 9),
             synth.box_surface((10, 25, 30), (22, 40, 41))]
    coords = np.concatenate(parts, 0)
    coords = coords[rng.permutation(coords.shape[0])]  # duplicates kept on purpose
    g = O.Grid(coords)
    rules = O.ssc_rules(g)
    _, crules = O.conv2_rules(g)
    feats = rng.randn(g.n, 8).astype(np.float32)
    weight = synth.kaiming_uniform(rng, 27, 8, 8)
    out = O.conv_forward(feats, weight, rules, g.n).numpy()
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "c1_small.npz"), coords=coords,
                        site_coords=g.coords, src_row=g.src_row, ssc_counts=np.array([len(r) for r in rules]),
                        ssc_pairs=np.concatenate(rules, 0), conv_pairs=np.concatenate(crules, 0), feats=feats,
                        weight=weight, ssc_out=out)
    print("sites", g.n, "pairs", sum(len(r) for r in rules))


if __name__ == "__main__":
    main()
