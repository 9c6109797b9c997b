"""Generates tests/golden/ref_*.npz: outputs of the REFERENCE ITSELF on seeded inputs.

The reference (THU-luvision/INS-Conv) is compiled for the host by oracle/build_ref.py and driven through
oracle/scn_ref.py; what this script stores is what the reference's own Metadata, rulebook builders and
cuda_* operators produced.  The library only exists where the reference tree is present, so the vectors are
committed and both the CPU suite (oracle against them) and the GPU suite (CUDA path against them) read the
files.  Inputs are not stored: tests regenerate them from the seeds with insconv.synth and check a digest.

  ref_c1.npz      BASELINE configs[0]: one SubmanifoldConvolution 16->16 fp32, no bias, on the seeded
                  boxes-and-spheres scene (seed 3: 50,208 voxels in a 128^3 grid), Kaiming-uniform weights
  ref_c2.npz      configs[1], the part the reference has semantics for (insert + re-draw; it has no
                  deletion): frame t+1's new points through Incre_InputLayer and Incre_SubmanifoldConvolution
  ref_labels.npz  label fusion: Result<3> (default cap and cap 3) and ResultOfWeight<3> after the seeded frames of
                  tests/labels_cases.py -- labels of every scene voxel after each frame, confidences, after
                  finalize and after set
  ref_chain.npz   InputLayer -> SSC 16->32 -> BatchNormReLU -> Convolution 32->96 /2 -> SSC 96->96 ->
                  Deconvolution 96->32 -> OutputLayer, full frame then incremental frame, every operator the
                  reference's (the network of __graft_entry__.smoke())

Large arrays are stored as a SHA-256 digest (integer results: bit-exact comparison needs nothing more) or as
every STEP-th row plus float64 column sums of the whole tensor (fp32 results).

Run from the repository root:  python tests/golden/make_golden_ref.py
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "ins-conv_b200"))

from insconv import synth  # noqa: E402

STEP = 16
C1_SEED = 3


def digest(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), dtype=np.uint8).copy()


def rules_digest(rules):
    """SHA-256 over the offsets' (input,output) int32 pairs concatenated in offset order."""
    return digest(np.concatenate([np.asarray(r, np.int32).reshape(-1, 2) for r in rules], 0))


def sample(x):
    x = np.asarray(x, np.float32)
    return {"rows": x[::STEP].copy(), "colsum": x.astype(np.float64).sum(0), "shape": np.array(x.shape)}


def put(d, name, x):
    for k, v in sample(x).items():
        d["%s_%s" % (name, k)] = v


def c1_inputs():
    coords = synth.boxes_and_spheres(C1_SEED)
    rng = np.random.RandomState(C1_SEED)
    feats = rng.randn(coords.shape[0], 16).astype(np.float32)
    weight = synth.kaiming_uniform(rng, 27, 16, 16)
    return coords, feats, weight


def chain_params():
    rng = np.random.RandomState(77)
    p = {"w1": (rng.randn(27, 16, 32) * (2.0 / 16 / 27) ** 0.5).astype(np.float32),
         "w2": (rng.randn(8, 32, 96) * (2.0 / 32 / 8) ** 0.5).astype(np.float32),
         "w3": (rng.randn(27, 96, 96) * (2.0 / 96 / 27) ** 0.5).astype(np.float32),
         "w4": (rng.randn(8, 96, 32) * (2.0 / 96 / 8) ** 0.5).astype(np.float32),
         "mean": (rng.randn(32) * 0.1).astype(np.float32), "var": (rng.rand(32) + 0.5).astype(np.float32),
         "gamma": (rng.rand(32) + 0.5).astype(np.float32), "beta": (rng.randn(32) * 0.1).astype(np.float32)}
    return p


def main():
    from oracle import build_ref
    if build_ref.build() is None:
        raise SystemExit("the reference tree is not present: nothing to generate from")
    from oracle import scn_ref as R

    # ---- configs[0] ----
    coords, feats, weight = c1_inputs()
    m = R.Metadata()
    vox = R.input_layer(m, 128, coords, feats, 1, 4)
    rules = m.ssc_rulebook(128)
    out, _ = R.ssc(m, 128, vox, weight)
    d = {"seed": np.array(C1_SEED), "coords_digest": digest(coords), "n_active": np.array(m.n_active(128)),
         "site_coords_digest": digest(m.spatial_locations(128)), "ssc_counts": np.array([len(r) for r in rules]),
         "ssc_pairs_digest": rules_digest(rules)}
    put(d, "out", out)
    crules = m.conv_rulebook(128)
    d["conv_counts"] = np.array([len(r) for r in crules])
    d["conv_pairs_digest"] = rules_digest(crules)
    d["coarse_coords_digest"] = digest(m.spatial_locations(64))
    np.savez_compressed(os.path.join(HERE, "ref_c1.npz"), **d)
    print("ref_c1: %d voxels, %d pairs" % (m.n_active(128), sum(len(r) for r in rules)))

    # ---- configs[1], insert + re-draw ----
    nf = synth.next_frame(coords, feats, C1_SEED)
    m1 = R.Metadata()
    res = R.incre_input_layer(m1, 128, nf["new_coords"], nf["new_feats"], 1, 4, m, vox)
    irules = m1.incre_ssc_rulebook(m, 128)
    res_out, _ = R.incre_ssc(m1, 128, res, weight, None, m, vox)
    d = {"seed": np.array(C1_SEED), "new_coords_digest": digest(nf["new_coords"]), "n_active": np.array(m1.n_active(128)),
         "site_coords_digest": digest(m1.spatial_locations(128)), "pre_exist_digest": digest(m1.pre_exist(m, 128)),
         "ssc_pairs_digest": rules_digest(m1.ssc_rulebook(128)), "incre_counts": np.array([len(r) for r in irules]),
         "incre_pairs_digest": rules_digest(irules), "input_residual": res, "ssc_residual": res_out}
    np.savez_compressed(os.path.join(HERE, "ref_c2.npz"), **d)
    print("ref_c2: %d changed voxels, %d incremental pairs" % (m1.n_active(128), sum(len(r) for r in irules)))

    # ---- chain: full frame, then incremental frame (what the reference's Python modules would call) ----
    coords0 = synth.boxes_and_spheres(0)
    rng = np.random.RandomState(0)
    feats0 = rng.randn(coords0.shape[0], 16).astype(np.float32)
    nf = synth.next_frame(coords0, feats0, 0)
    p = chain_params()
    bn = (p["mean"], p["var"], p["gamma"], p["beta"], 1e-4, 0.0)
    m0 = R.Metadata()
    v0 = R.input_layer(m0, 128, coords0, feats0, 1, 4)
    a = R.ssc(m0, 128, v0, p["w1"])[0]
    b = R.bn(a, *bn)
    c = R.conv(m0, 128, b, p["w2"])[0]
    e_in = R.ssc(m0, 64, c, p["w3"])[0]
    e = R.deconv(m0, 64, e_in, p["w4"])[0]
    full = R.output_layer(m0, e)
    m1 = R.Metadata()
    r0 = R.incre_input_layer(m1, 128, nf["new_coords"], nf["new_feats"], 1, 4, m0, v0)
    ra = R.incre_ssc(m1, 128, r0, p["w1"], None, m0, v0)[0]
    rb = R.incre_bn(ra, *bn, m1, m0, b, a, 128)
    rc = R.conv(m1, 128, rb, p["w2"], None, incremental=True)[0]
    rd = R.incre_ssc(m1, 64, rc, p["w3"], None, m0, c)[0]
    re = R.incre_deconv(m1, 64, rd, p["w4"], None, m0, e_in)[0]
    inc = R.incre_output_layer(m1, re, m0, e)
    d = {"coords_digest": digest(coords0), "new_coords_digest": digest(nf["new_coords"])}
    put(d, "full", full)
    d["incremental"] = inc
    for name, x in (("after_ssc1", a), ("after_bn", b), ("after_conv", c), ("after_ssc2", e_in), ("after_deconv", e)):
        d[name + "_colsum"] = np.asarray(x, np.float64).sum(0)
    np.savez_compressed(os.path.join(HERE, "ref_chain.npz"), **d)
    print("ref_chain: full %s, incremental %s" % (full.shape, inc.shape))

    # ---- label fusion: the reference's Result<3> / ResultOfWeight<3> on seeded frames of scores ----
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from labels_cases import frames
    d = {}
    for name, maximum in (("default", 0.7), ("cap3", 3.0)):
        scene, fr = frames(0)
        r = R.Result(maximum)
        per_frame = []
        for ps, sc in fr:
            r.update(ps, sc)
            per_frame.append(r.multiQuery(scene).astype(np.int8))
        d[name + "_labels_after_each_frame"] = np.stack(per_frame)
        d[name + "_confidence"] = np.array([r.confidence(*[int(v) for v in p]) for p in scene], np.float32)
        d[name + "_size"] = np.array(r.size())
        r.finalize(scene[::3])
        d[name + "_labels_after_finalize"] = r.multiQuery(scene).astype(np.int8)
        r.set(scene[:50], fr[0][1][:50])
        d[name + "_labels_after_set"] = r.multiQuery(scene).astype(np.int8)
    w = R.ResultOfWeight()
    for ps, sc in fr:
        w.update(ps, sc)
    d["weight_labels"] = w.multiQuery(scene).astype(np.int8)
    d["scene_digest"] = digest(scene)
    np.savez_compressed(os.path.join(HERE, "ref_labels.npz"), **d)
    print("ref_labels: %d voxels, %d frames" % (scene.shape[0], len(fr)))


if __name__ == "__main__":
    main()
