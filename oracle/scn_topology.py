"""Parameter-holding stand-ins for the reference's Python modules, for the CPU oracle.  TEST INFRASTRUCTURE ONLY.

oracle.scn_graph.GraphRunner evaluates a module tree by class name.  The product's `sparseconvnet` package builds
such a tree, but importing it loads the CUDA library; the timed CPU baseline and the topology checks want a tree
that owes nothing to the product.  These classes carry the constructor arguments, parameter shapes and
initialisation of the reference's modules and compute nothing:
  SubmanifoldConvolution  sparseconvnet/submanifoldConvolution.py:18-33   weight [volume, nIn, nOut], N(0, 2/(nIn*volume))
  Convolution / Deconvolution  sparseconvnet/convolution.py:13-30, deconvolution.py:13-30
  BatchNormalization (+ReLU / LeakyReLU)  sparseconvnet/batchNormalization.py:13-45 (eps 1e-4, momentum 0.9)
  NetworkInNetwork  sparseconvnet/networkInNetwork.py:57-70
  InputLayer / OutputLayer  sparseconvnet/ioLayers.py:15-50, 84-100
  Sequential / ConcatTable / AddTable / JoinTable / Identity  sparseconvnet/sequential.py, tables.py, identity.py
  UNet  sparseconvnet/networkArchitectures.py:202-300;  Naive_UNet  model.py:9-26
tests/test_golden_ref.py checks the tree built here against the one the reference's own package builds
(tests/golden/ref_model.json).
"""
import torch
from torch.nn import Module, Parameter


def _long3(v):
    return torch.full((3,), int(v), dtype=torch.int64) if isinstance(v, int) else torch.tensor(list(v), dtype=torch.int64)


class Sequential(torch.nn.Sequential):
    def add(self, module):
        self._modules[str(len(self._modules))] = module
        return self


class ConcatTable(Sequential):
    pass


class AddTable(Sequential):
    pass


class JoinTable(Sequential):
    pass


class Identity(Module):
    pass


class _Conv(Module):
    def __init__(self, dimension, nIn, nOut, filter_size, filter_stride, bias):
        Module.__init__(self)
        self.dimension, self.nIn, self.nOut = dimension, nIn, nOut
        self.filter_size = _long3(filter_size)
        if filter_stride is not None:
            self.filter_stride = _long3(filter_stride)
        volume = int(self.filter_size.prod())
        self.weight = Parameter(torch.empty(volume, nIn, nOut).normal_(0, (2.0 / nIn / volume) ** 0.5))
        if bias:
            self.bias = Parameter(torch.zeros(nOut))


class SubmanifoldConvolution(_Conv):
    def __init__(self, dimension, nIn, nOut, filter_size, bias, dilated_rate=1):
        _Conv.__init__(self, dimension, nIn, nOut, filter_size, None, bias)
        self.dilated_rate = dilated_rate


class Convolution(_Conv):
    pass


class Deconvolution(_Conv):
    pass


class BatchNormalization(Module):
    def __init__(self, nPlanes, eps=1e-4, momentum=0.9, affine=True, leakiness=1):
        Module.__init__(self)
        self.nPlanes, self.eps, self.momentum, self.affine, self.leakiness = nPlanes, eps, momentum, affine, leakiness
        self.register_buffer("running_mean", torch.zeros(nPlanes))
        self.register_buffer("running_var", torch.ones(nPlanes))
        if affine:
            self.weight = Parameter(torch.ones(nPlanes))
            self.bias = Parameter(torch.zeros(nPlanes))


class BatchNormReLU(BatchNormalization):
    def __init__(self, nPlanes, eps=1e-4, momentum=0.9):
        BatchNormalization.__init__(self, nPlanes, eps, momentum, True, 0)


class BatchNormLeakyReLU(BatchNormalization):
    def __init__(self, nPlanes, eps=1e-4, momentum=0.9, leakiness=0.333):
        BatchNormalization.__init__(self, nPlanes, eps, momentum, True, leakiness)


class NetworkInNetwork(Module):
    def __init__(self, nIn, nOut, bias):
        Module.__init__(self)
        self.nIn, self.nOut = nIn, nOut
        self.weight = Parameter(torch.empty(nIn, nOut).normal_(0, (2.0 / nIn) ** 0.5))
        if bias:
            self.bias = Parameter(torch.zeros(nOut))


class InputLayer(Module):
    def __init__(self, dimension, spatial_size, mode=3):
        Module.__init__(self)
        self.dimension, self.mode = dimension, mode
        self.spatial_size = _long3(spatial_size)


class OutputLayer(Module):
    def __init__(self, dimension):
        Module.__init__(self)
        self.dimension = dimension


def UNet(dimension, reps, nPlanes, residual_blocks=False, downsample=(2, 2), leakiness=0):
    """networkArchitectures.py:202-300: per level `reps` blocks, then (if deeper levels exist) identity joined with
    BN -> Convolution/2 -> deeper level -> BN -> Deconvolution, then `reps` blocks on the joined planes."""
    def block(m, a, b):
        if residual_blocks:
            m.add(ConcatTable().add(Identity() if a == b else NetworkInNetwork(a, b, False)).add(
                Sequential().add(BatchNormLeakyReLU(a, leakiness=leakiness)).add(SubmanifoldConvolution(dimension, a, b, 3, False))
                .add(BatchNormLeakyReLU(b, leakiness=leakiness)).add(SubmanifoldConvolution(dimension, b, b, 3, False))))
            m.add(AddTable())
        else:
            m.add(Sequential().add(BatchNormLeakyReLU(a, leakiness=leakiness)).add(SubmanifoldConvolution(dimension, a, b, 3, False)))

    def level(planes):
        m = Sequential()
        for _ in range(reps):
            block(m, planes[0], planes[0])
        if len(planes) > 1:
            m.add(ConcatTable().add(Identity()).add(
                Sequential().add(BatchNormLeakyReLU(planes[0], leakiness=leakiness))
                .add(Convolution(dimension, planes[0], planes[1], downsample[0], downsample[1], False))
                .add(level(planes[1:]))
                .add(BatchNormLeakyReLU(planes[1], leakiness=leakiness))
                .add(Deconvolution(dimension, planes[1], planes[0], downsample[0], downsample[1], False))))
            m.add(JoinTable())
            for i in range(reps):
                block(m, planes[0] * (2 if i == 0 else 1), planes[0])
        return m

    return level(list(nPlanes))


class Naive_UNet(Module):
    """model.py:9-26."""

    def __init__(self, dimension=3, full_scale=4096, m=32, classes=20):
        Module.__init__(self)
        self.sparseModel = Sequential().add(InputLayer(dimension, full_scale, mode=4)).add(
            SubmanifoldConvolution(dimension, 3, m, 3, False)).add(
            UNet(dimension, 2, [m, 2 * m, 3 * m, 4 * m, 5 * m, 6 * m, 7 * m], True)).add(BatchNormReLU(m)).add(
            OutputLayer(dimension))
        self.linear = torch.nn.Linear(m, classes)
