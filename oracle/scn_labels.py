"""CPU restatement of the reference's label fusion.  TEST INFRASTRUCTURE ONLY (see oracle/scn_oracle.py).

Result<3> (Metadata/resultHash.h:22-138): voxel -> (label, confidence), and ResultOfWeight<3>
(resultHash.h:141-218): voxel -> score vector.  Plain Python dictionaries keyed by (x, y, z); rows of one call
are applied in row order, which is what the reference's loops do when they run on one thread.  Pinned against the
reference's own classes compiled for the host (tests/test_oracle_vs_reference.py).
"""
import numpy as np


class Result(object):
    def __init__(self, maximum=0.7):
        # the reference declares `int maximum` and initialises it from the float argument (resultHash.h:24-29):
        # the default 0.7 is held as 0
        self.maximum = float(int(maximum))
        self.result = {}

    def set(self, ps, label):
        """resultHash.h:37-50: label = argmax, confidence 0, whatever was there."""
        ps, label = np.asarray(ps), np.asarray(label, np.float32)
        if ps.ndim == 1:
            ps, label = ps[None], label[None]
        for p, row in zip(ps, label):
            self.result[tuple(int(v) for v in p[:3])] = (int(np.argmax(row)), np.float32(0))

    def update(self, ps, label):
        """resultHash.h:52-98.  First pass: which rows name a voxel that is already in the table (a voxel named twice
        in one call is "already there" for its second row).  Second pass, in row order: new -> (argmax, max score);
        same label -> confidence = min(maximum, confidence + score); other label -> confidence -= score, and below
        zero the label flips and the confidence changes sign."""
        ps, label = np.asarray(ps), np.asarray(label, np.float32)
        val = np.argmax(label, 1)
        best = label[np.arange(label.shape[0]), val]
        pre = []
        for p in ps:
            k = tuple(int(v) for v in p[:3])
            pre.append(k in self.result)
            self.result.setdefault(k, (0, np.float32(0)))
        for i, p in enumerate(ps):
            k = tuple(int(v) for v in p[:3])
            if not pre[i]:
                self.result[k] = (int(val[i]), np.float32(best[i]))
                continue
            lab, conf = self.result[k]
            if lab == int(val[i]):
                conf = np.float32(min(np.float32(self.maximum), np.float32(conf + best[i])))
            else:
                conf = np.float32(conf - best[i])
            if conf < 0:
                lab, conf = int(val[i]), np.float32(-conf)
            self.result[k] = (lab, conf)

    def multiQuery(self, ps):
        return np.array([self.result.get(tuple(int(v) for v in p[:3]), (-1, 0))[0] for p in np.asarray(ps)], np.int64)

    def query(self, p):
        return int(self.multiQuery(np.asarray(p)[None])[0])

    def get_all_points_labels(self):
        return np.array([list(k) + [v[0]] for k, v in self.result.items()], np.int64).reshape(-1, 4)

    def finalize(self, points):
        keep = {tuple(int(v) for v in p[:3]) for p in np.asarray(points)}
        self.result = {k: v for k, v in self.result.items() if k in keep}

    def clear(self):
        self.result = {}


class ResultOfWeight(object):
    def __init__(self):
        self.result = {}

    def update(self, ps, label):
        """resultHash.h:146-158: new -> the row; known -> 0.5 * old + row."""
        for p, row in zip(np.asarray(ps), np.asarray(label, np.float32)):
            k = tuple(int(v) for v in p[:3])
            old = self.result.get(k)
            self.result[k] = row.copy() if old is None else (old * np.float32(0.5) + row).astype(np.float32)

    def multiQuery(self, ps):
        out = []
        for p in np.asarray(ps):
            v = self.result.get(tuple(int(x) for x in p[:3]))
            out.append(-1 if v is None else int(np.argmax(v)))
        return np.array(out, np.int64)

    def query(self, p):
        return int(self.multiQuery(np.asarray(p)[None])[0])

    def get_all_points_labels(self):
        return np.array([list(k) + [int(np.argmax(v))] for k, v in self.result.items()], np.int64).reshape(-1, 4)

    def finalize(self, points):
        keep = {tuple(int(v) for v in p[:3]) for p in np.asarray(points)}
        self.result = {k: v for k, v in self.result.items() if k in keep}

    def clear(self):
        self.result = {}
