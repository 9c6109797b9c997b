"""Runs a sparseconvnet module tree on the CPU oracle.  TEST INFRASTRUCTURE ONLY (see scn_oracle.py).

The walker reads the structure and the parameters of an already-built module tree (the product's
`sparseconvnet` modules, e.g. the Naive_UNet of the reference's model.py:9-26) and evaluates it with
the oracle's grids, rulebooks and torch-CPU feature math; it never calls the product's kernels.
Modules are recognised by class name so that this file does not import the product package.

Incremental frames follow the reference's semantics (sparseconvnet/*.py `increment=True` branches and
the Incre_* host functions): the state saved by the last full frame is kept per module in `self.saved`.
"""
import numpy as np
import torch

from . import scn_oracle as O


class OMeta(object):
    """Per-frame grids by spatial size, plus stride-2 rulebooks (the oracle's Metadata)."""

    def __init__(self):
        self.grids = {}
        self.conv_rules = {}
        self.ssc_rules = {}
        self.input_size = None

    def ssc(self, size):
        if size not in self.ssc_rules:
            self.ssc_rules[size] = O.ssc_rules(self.grids[size])
        return self.ssc_rules[size]

    def getSpatialLocations(self, size):
        """[n,4] (x,y,z,batch) of the sites of a scale, in row order (Metadata::getSpatialLocations)."""
        return torch.from_numpy(self.grids[tuple(int(v) for v in size)].coords.copy())

    def coarse(self, in_size, out_size):
        key = (in_size, out_size)
        if key not in self.conv_rules:
            g, r = O.conv2_rules(self.grids[in_size])
            self.grids.setdefault(out_size, g)
            self.conv_rules[key] = r
        return self.grids[out_size], self.conv_rules[key]


class OTensor(object):
    def __init__(self, feats, meta, size):
        self.features, self.metadata, self.spatial_size = feats, meta, size


def _p(module, name):
    t = getattr(module, name, None)
    return None if t is None else t.detach().cpu().float()


def _size(t):
    return tuple(int(v) for v in t)


class GraphRunner(object):
    def __init__(self, root, post=None):
        """post(module, output): optional callback run on the output of every SubmanifoldConvolution and
        Convolution (the multi-GPU slab tests exchange halo rows there)."""
        self.root = root
        self.saved = {}
        self.post = post

    def __call__(self, inputs, increment=False):
        return self._run(self.root, inputs, increment)

    def _run(self, m, x, inc):
        name = type(m).__name__
        fn = getattr(self, "_" + name, None)
        if fn is None:
            for base in type(m).__mro__:
                fn = getattr(self, "_" + base.__name__, None)
                if fn is not None:
                    break
        if fn is None:
            raise NotImplementedError("oracle has no rule for module " + name)
        return fn(m, x, inc)

    # ---- containers ----------------------------------------------------------------------------
    def _Sequential(self, m, x, inc):
        for child in m:
            x = self._run(child, x, inc)
        return x

    def _ConcatTable(self, m, x, inc):
        return [self._run(child, x, inc) for child in m]

    def _AddTable(self, m, x, inc):
        return OTensor(sum(t.features for t in x), x[0].metadata, x[0].spatial_size)

    def _JoinTable(self, m, x, inc):
        return OTensor(torch.cat([t.features for t in x], 1), x[0].metadata, x[0].spatial_size)

    def _Identity(self, m, x, inc):
        return x

    def _Linear(self, m, x, inc):
        return torch.nn.functional.linear(x, _p(m, "weight"), _p(m, "bias"))

    def _Naive_UNet(self, m, x, inc):
        return self._run(m.linear, self._run(m.sparseModel, x, inc), inc)

    # ---- layers --------------------------------------------------------------------------------
    def _InputLayer(self, m, x, inc):
        coords = torch.as_tensor(x[0]).cpu().numpy()
        feats = torch.as_tensor(x[1]).cpu().float()
        size = _size(m.spatial_size)
        meta = OMeta()
        g = O.Grid(coords)
        meta.grids[size] = g
        meta.input_size = size
        if not inc:
            out = OTensor(O.input_forward(feats, g, m.mode), meta, size)
            self.saved[id(m)] = out
        else:
            pre = self.saved[id(m)]
            out = OTensor(O.incre_input_forward(feats, g, m.mode, pre.metadata.grids[size], pre.features), meta, size)
        return out

    def _OutputLayer(self, m, x, inc):
        g = x.metadata.grids[x.metadata.input_size]
        if not inc:
            self.saved[id(m)] = x
            return O.output_forward(x.features, g)
        pre = self.saved[id(m)]
        return O.incre_output_forward(x.features, g, pre.metadata.grids[pre.metadata.input_size], pre.features)

    def _SubmanifoldConvolution(self, m, x, inc):
        g = x.metadata.grids[x.spatial_size]
        w, b = _p(m, "weight"), _p(m, "bias")
        if not inc:
            self.saved[id(m)] = x
            out = O.conv_forward(x.features, w, x.metadata.ssc(x.spatial_size), g.n, b)
        else:
            pre = self.saved[id(m)]
            pg = pre.metadata.grids[x.spatial_size]
            key = ("incre", x.spatial_size)
            if key not in x.metadata.ssc_rules:
                x.metadata.ssc_rules[key] = O.incre_ssc_rules(g, pg)
            out = O.conv_forward(x.features, w, x.metadata.ssc(x.spatial_size), g.n, b)
            out = O.conv_forward(pre.features, w, x.metadata.ssc_rules[key], g.n, out=out)
        res = OTensor(out, x.metadata, x.spatial_size)
        if self.post:
            self.post(m, res)
        return res

    def _Convolution(self, m, x, inc):
        out_size = tuple((s - int(f)) // int(st) + 1 for s, f, st in zip(x.spatial_size, m.filter_size, m.filter_stride))
        coarse, rules = x.metadata.coarse(x.spatial_size, out_size)
        out = O.conv_forward(x.features, _p(m, "weight"), rules, coarse.n, _p(m, "bias"))
        res = OTensor(out, x.metadata, out_size)
        if self.post:
            self.post(m, res)
        return res

    def _Deconvolution(self, m, x, inc):
        out_size = tuple((s - 1) * int(st) + int(f) for s, f, st in zip(x.spatial_size, m.filter_size, m.filter_stride))
        fine = x.metadata.grids[out_size]
        coarse, rules = x.metadata.coarse(out_size, x.spatial_size)
        w, b = _p(m, "weight"), _p(m, "bias")
        if not inc:
            self.saved[id(m)] = x
            out = O.conv_forward(x.features, w, rules, fine.n, b, reverse=True)
        else:
            pre = self.saved[id(m)]
            out = O.incre_deconv_forward(x.features, w, fine, coarse, rules, pre.metadata.grids[out_size],
                                         pre.metadata.grids[x.spatial_size], pre.features, b)
        return OTensor(out, x.metadata, out_size)

    def _BatchNormalization(self, m, x, inc):
        args = (_p(m, "running_mean"), _p(m, "running_var"), _p(m, "weight"), _p(m, "bias"), m.eps, m.leakiness)
        if not inc:
            out = O.bn_forward(x.features, *args)
            self.saved[id(m)] = (x, out)
        else:
            pre_in, pre_out = self.saved[id(m)]
            out = O.incre_bn_forward(x.features, *args, x.metadata.grids[x.spatial_size],
                                     pre_in.metadata.grids[x.spatial_size], pre_out, pre_in.features)
        return OTensor(out, x.metadata, x.spatial_size)

    def _NetworkInNetwork(self, m, x, inc):
        return OTensor(O.nin_forward(x.features, _p(m, "weight"), _p(m, "bias")), x.metadata, x.spatial_size)
