"""The operator modules of the UNet inference path.

Each module mirrors the constructor arguments, parameter shapes, initialisation and forward contract
of its reference counterpart:
  SubmanifoldConvolution  sparseconvnet/submanifoldConvolution.py:18-81
  Convolution             sparseconvnet/convolution.py:13-84
  Deconvolution           sparseconvnet/deconvolution.py:13-106
  BatchNormalization      sparseconvnet/batchNormalization.py:13-110
  NetworkInNetwork        sparseconvnet/networkInNetwork.py:57-88
  InputLayer/OutputLayer  sparseconvnet/ioLayers.py:15-117
`forward(input, increment=False)`: a full frame (increment False) computes on every site and keeps what
the next incremental frames need (`save_meta`, `save_input_feats`, `save_output`, `save_input`); an
incremental frame computes residuals on the sites touched by the new points only.  The modules are
inference only: the operators do not record autograd history, whatever the grad mode.
"""
import weakref

import torch
from torch.nn import Module, Parameter

import sparseconvnet
from . import SCN
from .metadata import Metadata
from .tensor import SparseConvNetTensor
from .utils import toLongTensor, optionalTensor, _precision

_NONE = torch.empty(0)
# [callable or None]: run on the result of every full-frame SubmanifoldConvolution and Convolution (the layers whose
# rows depend on neighbouring sites); a scene split over several GPUs exchanges its halo rows here
# (sparseconvnet.set_halo_exchange, insconv.slab)
halo_exchange = [None]


def _halo(t):
    if halo_exchange[0] is not None:
        halo_exchange[0](t)
    return t


def _keep(module, **state):
    """Stores per-frame state on a module without torch.nn.Module.__setattr__ (which walks the parameter,
    buffer and sub-module tables on every assignment and is the slowest thing a layer call would do)."""
    module.__dict__.update(state)


def _residual(input, increment):
    """True when this call is a residual (reference-style incremental) update.  In the exact incremental mode
    the InputLayer hands down the whole merged scene and every layer runs its full-frame path instead."""
    if isinstance(input, (list, tuple)):
        input = input[0]
    return bool(increment) and not getattr(input, "recompute_all", False)


def _packed(module):
    """The tensor-core kernels read weights transposed.  The copy is made once per weight version and kept on the
    module (keyed on the Parameter object, its version counter and its address), instead of once per call."""
    if _precision[0] == "fp32":
        return _NONE
    w = module._parameters["weight"]
    c = module.__dict__.get("_pack_cache")
    if c is not None and c[0] is w and c[1] == w._version and c[2] == w.data_ptr():
        return c[3]
    p = SCN.pack_weights(w) if w.is_cuda else _NONE
    module.__dict__["_pack_cache"] = (w, w._version, w.data_ptr(), p)
    return p


def _packed_for(module, features):
    """The weight pack that goes with these feature rows: fp16 fragments for fp16 rows (written by a BatchNorm in
    'fp16' precision), else the tf32 pack."""
    if features.dtype != torch.float16:
        return _packed(module)
    w = module._parameters["weight"]
    c = module.__dict__.get("_pack_cache_h")
    if c is not None and c[0] is w and c[1] == w._version and c[2] == w.data_ptr():
        return c[3]
    p = SCN.pack_weights_f16(w)
    module.__dict__["_pack_cache_h"] = (w, w._version, w.data_ptr(), p)
    return p


def takes_half_rows(module):
    """True for a convolution module whose shape has an fp16 gather-GEMM kernel (planes multiples of 32, at most
    224 out: warp-level kernel for 32/64 planes, tcgen05 kernel above)."""
    return isinstance(module, (SubmanifoldConvolution, Convolution, Deconvolution)) and \
        module.nIn % 32 == 0 and module.nOut % 32 == 0 and 32 <= module.nOut <= 224 and module.nIn >= 32 and \
        not hasattr(module, "bias")


def bn_affine(bn):
    """(scale, shift) with which an inference BatchNorm is y = x * scale + shift: scale = gamma / sqrt(var + eps),
    shift = beta - mean * scale.  Made once per version of the module's parameters and statistics."""
    w, b = bn._parameters.get("weight"), bn._parameters.get("bias")
    m, v = bn._buffers["running_mean"], bn._buffers["running_var"]
    key = (m._version, v._version, m.data_ptr(), v.data_ptr(), None if w is None else (w._version, w.data_ptr()),
           None if b is None else (b._version, b.data_ptr()))
    c = bn.__dict__.get("_affine_cache")
    if c is not None and c[0] == key:
        return c[1], c[2]
    with torch.no_grad():
        scale = torch.rsqrt(v + bn.eps)
        if w is not None:
            scale = scale * w
        shift = -m * scale
        if b is not None:
            shift = shift + b
    bn.__dict__["_affine_cache"] = (key, scale.contiguous(), shift.contiguous())
    return bn.__dict__["_affine_cache"][1:]


def _fused_bn_args(module, fuse_bn, features, residual=False):
    """Arguments for a convolution whose epilogue also applies `fuse_bn` (the BatchNorm + ReLU behind it) and writes
    the result as fp16 rows: possible when the convolution itself reads fp16 rows (its kernels carry that epilogue).
    residual: the incremental form, which reads the rows the saved frame's BatchNorm read (fp32) and wrote (fp16)."""
    if fuse_bn is None or features.dtype != torch.float16 or not takes_half_rows(module):
        return None
    if residual:
        so, si = fuse_bn.__dict__.get("save_output"), fuse_bn.__dict__.get("save_input")
        if so is None or si is None or so.features.dtype != torch.float16 or si.features.dtype != torch.float32 or \
                si.features.numel() == 0 or fuse_bn.training:
            return None
    scale, shift = bn_affine(fuse_bn)
    return scale, shift, float(fuse_bn.leakiness), features.new_empty(0, dtype=torch.float16)


def _saved_bn_rows(fuse_bn):
    """(rows the saved frame's BatchNorm read, rows it wrote): operands of the incremental fused BatchNorm."""
    return fuse_bn.save_input.features, fuse_bn.save_output.features


def _finish_fused(conv_out, fuse_bn, bn_rows):
    """What BatchNormalization.forward would have done: the tensor it returns and the state it keeps."""
    normed = conv_out.like(bn_rows)
    _keep(fuse_bn, save_output=normed, save_input=conv_out)
    conv_out.bn_ready = (fuse_bn, normed)
    return conv_out


_wide_rows = {}  # id(fp16 tensor) -> (weak reference to it, its fp32 copy)


def _f32(module, t):
    """Saved fp16 rows as fp32, for the residual operators (they read fp32).  Widened once per saved tensor: a
    BatchNorm's saved output and the saved input of the convolution behind it are the same tensor."""
    if t.dtype != torch.float16:
        return t
    hit = _wide_rows.get(id(t))
    if hit is not None and hit[0]() is t:
        return hit[1]
    key = id(t)
    wide = t.float()
    _wide_rows[key] = (weakref.ref(t, lambda _, key=key: _wide_rows.pop(key, None)), wide)
    return wide


def _residual_rows(module, rows, saved):
    """(residual rows, saved rows, weight pack) for an incremental convolution.  In 'fp16' precision the BatchNorm in
    front hands over the residual as fp16 rows and the saved frame kept its input as fp16 rows: both go to the fp16
    kernels as they are.  Mixed types (a saved frame from another precision) are widened to fp32."""
    if rows.dtype == torch.float16 and saved.dtype == torch.float16:
        return rows, saved, _packed_for(module, rows)
    if rows.dtype == torch.float16:
        rows = rows.float()
    return rows, _f32(module, saved), _packed(module)


def _count(madds, out):
    sparseconvnet.forward_pass_multiplyAdd_count += madds
    sparseconvnet.forward_pass_hidden_states += out.nelement()


def _size_repr(name, n_in, n_out, size, stride=None):
    s = "%s %d->%d C%s" % (name, n_in, n_out, "x".join(str(int(v)) for v in size) if size.max() != size.min() else int(size[0]))
    if stride is not None:
        s += "/%s" % ("x".join(str(int(v)) for v in stride) if stride.max() != stride.min() else int(stride[0]))
    return s


class SubmanifoldConvolution(Module):
    def __init__(self, dimension, nIn, nOut, filter_size, bias, dilated_rate=1):
        Module.__init__(self)
        self.dimension, self.nIn, self.nOut = dimension, nIn, nOut
        self.filter_size = toLongTensor(dimension, filter_size)
        self.filter_volume = int(self.filter_size.prod().item())
        self.dilated_rate = dilated_rate
        std = (2.0 / nIn / self.filter_volume) ** 0.5
        self.weight = Parameter(torch.empty(self.filter_volume, nIn, nOut).normal_(0, std))
        if bias:
            self.bias = Parameter(torch.zeros(nOut))

    def forward(self, input, increment=False, addend=None, fuse_bn=None, raw_needed=True):
        """addend (no bias) = features [nActive, nOut] added to the result in the kernel's epilogue (the residual sum of
        a ResNet block); fuse_bn = the BatchNormalization module that consumes this output: when this convolution reads
        fp16 rows, its epilogue also writes fuse_bn's result as fp16 rows (picked up by that module without a kernel of
        its own) -- on a residual frame the incremental form of it, against the rows the saved frame's BatchNorm read and
        wrote; raw_needed = False (full frames): nothing else reads the fp32 result, it is not stored."""
        assert input.features.nelement() == 0 or input.features.size(1) == self.nIn, (self.nIn, self.nOut, input)
        out = input.features.new_empty(0, dtype=torch.float32)
        if not _residual(input, increment):
            fused = _fused_bn_args(self, fuse_bn, input.features)
            skip_raw = fused is not None and not raw_needed
            madds = SCN.SubmanifoldConvolution_updateOutput(
                input.spatial_size, self.filter_size, input.metadata, input.features, out, self._parameters["weight"],
                optionalTensor(self, "bias"), self.dilated_rate, _packed_for(self, input.features),
                _NONE if addend is None else addend, *(fused if fused else (_NONE, _NONE, 0.0, _NONE)), skip_raw)
            _keep(self, save_meta=input.metadata, save_input_feats=input.features)
            _count(madds, out)
            res = input.like(out)
            return _halo(_finish_fused(res, fuse_bn, fused[3]) if fused else res)
        rows, saved, packed = _residual_rows(self, input.features, self.save_input_feats)
        fused = _fused_bn_args(self, fuse_bn, rows, True)
        fold = addend is not None and "bias" not in self._parameters
        madds = SCN.Incre_SubmanifoldConvolution_updateOutput(
            input.spatial_size, self.filter_size, input.metadata, rows, out, self._parameters["weight"],
            optionalTensor(self, "bias"), self.save_meta, saved, packed, addend if fold else _NONE,
            *(fused if fused else (_NONE, _NONE, 0.0, _NONE)), *(_saved_bn_rows(fuse_bn) if fused else (_NONE, _NONE)))
        _count(madds, out)
        res = input.like(out if addend is None or fold else out + addend)
        if fused:  # the incremental BatchNorm's result: picked up by that module, which keeps no state on residual frames
            res.bn_ready = (fuse_bn, input.like(fused[3]))
        return res

    def input_spatial_size(self, out_size):
        return out_size

    def __repr__(self):
        return _size_repr("SubmanifoldConvolution", self.nIn, self.nOut, self.filter_size)


ValidConvolution = SubmanifoldConvolution


class _Strided(Module):
    def __init__(self, dimension, nIn, nOut, filter_size, filter_stride, bias):
        Module.__init__(self)
        self.dimension, self.nIn, self.nOut = dimension, nIn, nOut
        self.filter_size = toLongTensor(dimension, filter_size)
        self.filter_stride = toLongTensor(dimension, filter_stride)
        self.filter_volume = int(self.filter_size.prod().item())
        std = (2.0 / nIn / self.filter_volume) ** 0.5
        self.weight = Parameter(torch.empty(self.filter_volume, nIn, nOut).normal_(0, std))
        if bias:
            self.bias = Parameter(torch.zeros(nOut))


class Convolution(_Strided):
    def forward(self, input, increment=False, fuse_bn=None):
        """fuse_bn: as for SubmanifoldConvolution (full frames, fp16 rows in)."""
        assert input.features.nelement() == 0 or input.features.size(1) == self.nIn
        out_size = torch.div(input.spatial_size - self.filter_size, self.filter_stride, rounding_mode="floor") + 1
        assert ((out_size - 1) * self.filter_stride + self.filter_size == input.spatial_size).all(), \
            (input.spatial_size, out_size, self.filter_size, self.filter_stride)
        out = input.features.new_empty(0, dtype=torch.float32)
        residual = _residual(input, increment)
        fused = _fused_bn_args(self, fuse_bn, input.features, residual)
        bn_args = fused if fused else (_NONE, _NONE, 0.0, _NONE)
        if residual:
            madds = SCN.Incre_Convolution_updateOutput(
                input.spatial_size, out_size, self.filter_size, self.filter_stride, input.metadata, input.features, out,
                self._parameters["weight"], optionalTensor(self, "bias"), _packed_for(self, input.features),
                fuse_bn.save_output.metadata if fused else None, *bn_args,
                *(_saved_bn_rows(fuse_bn) if fused else (_NONE, _NONE)))
        else:
            madds = SCN.Convolution_updateOutput(
                input.spatial_size, out_size, self.filter_size, self.filter_stride, input.metadata, input.features, out,
                self._parameters["weight"], optionalTensor(self, "bias"), _packed_for(self, input.features), *bn_args, False)
        _count(madds, out)
        res = input.like(out, out_size)
        if residual:
            if fused:
                res.bn_ready = (fuse_bn, res.like(fused[3]))
            return res
        res = _finish_fused(res, fuse_bn, fused[3]) if fused else res
        return _halo(res)

    def input_spatial_size(self, out_size):
        return (out_size - 1) * self.filter_stride + self.filter_size

    def __repr__(self):
        return _size_repr("Convolution", self.nIn, self.nOut, self.filter_size, self.filter_stride)


class Deconvolution(_Strided):
    def forward(self, input, increment=False):
        assert input.features.nelement() == 0 or input.features.size(1) == self.nIn
        out_size = (input.spatial_size - 1) * self.filter_stride + self.filter_size
        out = input.features.new_empty(0, dtype=torch.float32)
        if not _residual(input, increment):
            madds = SCN.Deconvolution_updateOutput(
                input.spatial_size, out_size, self.filter_size, self.filter_stride, input.metadata, input.features,
                out, self._parameters["weight"], optionalTensor(self, "bias"), _packed_for(self, input.features))
            _keep(self, save_meta=input.metadata, save_input_feats=input.features)
        else:
            rows, saved, packed = _residual_rows(self, input.features, self.save_input_feats)
            madds = SCN.Incre_Deconvolution_updateOutput(
                input.spatial_size, out_size, self.filter_size, self.filter_stride, input.metadata, rows,
                out, self._parameters["weight"], optionalTensor(self, "bias"), self.save_meta, saved, packed)
        _count(madds, out)
        return input.like(out, out_size)

    def input_spatial_size(self, out_size):
        in_size = torch.div(out_size - self.filter_size, self.filter_stride, rounding_mode="floor") + 1
        assert ((in_size - 1) * self.filter_stride + self.filter_size == out_size).all()
        return in_size

    def __repr__(self):
        return _size_repr("Deconvolution", self.nIn, self.nOut, self.filter_size, self.filter_stride)


class BatchNormalization(Module):
    """leakiness: 0 = ReLU, (0,1) = leaky ReLU, 1 = no activation, applied in the same kernel."""

    def __init__(self, nPlanes, eps=1e-4, momentum=0.9, affine=True, leakiness=1):
        Module.__init__(self)
        self.nPlanes, self.eps, self.momentum, self.affine, self.leakiness = nPlanes, eps, momentum, affine, leakiness
        self.register_buffer("running_mean", torch.zeros(nPlanes))
        self.register_buffer("running_var", torch.ones(nPlanes))
        if affine:
            self.weight = Parameter(torch.ones(nPlanes))
            self.bias = Parameter(torch.zeros(nPlanes))

    def forward(self, input, increment=False, half_rows=False):
        """half_rows ('fp16' precision, full frames, running statistics): the result is written as fp16 rows; a
        Sequential asks for it when the next module is a convolution that reads fp16 rows."""
        assert input.features.nelement() == 0 or input.features.size(1) == self.nPlanes, \
            (self.nPlanes, input.features.shape)
        residual = _residual(input, increment)
        ready = input.bn_ready
        if ready is not None and ready[0] is self and not self.training:
            return ready[1]  # the convolution in front of this module already wrote this module's result (and state)
        half_rows = half_rows and not self.training and self.nPlanes % 8 == 0
        if residual:  # fp16 residual rows when the saved frame's output was written as fp16 rows and its input was kept
            half_rows = half_rows and self.save_output.features.dtype == torch.float16 and \
                self.save_input.features.dtype == torch.float32 and self.save_input.features.numel() > 0
        feats = input.features
        out = feats.new_empty(0, dtype=torch.float16 if half_rows else torch.float32)
        mean, var = self._buffers["running_mean"], self._buffers["running_var"]
        if not residual:
            # the batch-statistics outputs are only written in training mode
            scratch = feats.new_empty(0) if self.training else _NONE
            SCN.BatchNormalization_updateOutput(
                feats, out, scratch, feats.new_empty(0) if self.training else _NONE, mean, var,
                optionalTensor(self, "weight"), optionalTensor(self, "bias"), self.eps, self.momentum, self.training,
                self.leakiness)
            _keep(self, save_output=input.like(out), save_input=input)
        else:
            SCN.Incre_BatchNormalization_updateOutput(
                feats, out, _NONE, _NONE, mean, var,
                optionalTensor(self, "weight"), optionalTensor(self, "bias"), self.eps, self.momentum, self.training,
                self.leakiness, input.metadata, self.save_output.metadata,
                self.save_output.features if half_rows else _f32(self, self.save_output.features),
                self.save_input.features, input.spatial_size)
        return input.like(out)

    def input_spatial_size(self, out_size):
        return out_size

    def __repr__(self):
        return "%s(%d,eps=%g,momentum=%g,affine=%s,leakiness=%g)" % (
            type(self).__name__, self.nPlanes, self.eps, self.momentum, self.affine, self.leakiness)


class BatchNormReLU(BatchNormalization):
    def __init__(self, nPlanes, eps=1e-4, momentum=0.9):
        BatchNormalization.__init__(self, nPlanes, eps, momentum, True, 0)


class BatchNormLeakyReLU(BatchNormalization):
    def __init__(self, nPlanes, eps=1e-4, momentum=0.9, leakiness=0.333):
        BatchNormalization.__init__(self, nPlanes, eps, momentum, True, leakiness)


class NetworkInNetwork(Module):
    """1x1 convolution; linear, so the incremental frame applies it to the residual rows as is."""

    def __init__(self, nIn, nOut, bias):
        Module.__init__(self)
        self.nIn, self.nOut = nIn, nOut
        self.weight = Parameter(torch.empty(nIn, nOut).normal_(0, (2.0 / nIn) ** 0.5))
        if bias:
            self.bias = Parameter(torch.zeros(nOut))

    def forward(self, input, increment=False):
        assert input.features.nelement() == 0 or input.features.size(1) == self.nIn, (self.nIn, input.features.shape)
        out = input.features.new_empty(0)
        madds = SCN.NetworkInNetwork_updateOutput(input.features, out, self.weight, optionalTensor(self, "bias"),
                                                  _packed(self))
        _count(madds, out)
        return input.like(out)

    def input_spatial_size(self, out_size):
        return out_size

    def __repr__(self):
        return "NetworkInNetwork%d->%d" % (self.nIn, self.nOut)


class InputLayer(Module):
    """(coords, features[, batch_size]) -> SparseConvNetTensor.

    coords: LongTensor N x 3 (one sample) or N x 4 (last column = batch index), on the CPU or on the GPU
    (a CUDA tensor is hashed in place, without a trip through the host).  mode 3 sums and mode 4 averages
    the features of points that share a voxel; other modes are not part of the GPU grid path.
    """

    def __init__(self, dimension, spatial_size, mode=3, normal_guide_scale=10240):
        Module.__init__(self)
        self.dimension = dimension
        self.spatial_size = toLongTensor(dimension, spatial_size)
        self.mode = mode
        self.normal_guide_scale = normal_guide_scale
        self.device = None

    def to(self, device):
        self.device = device
        return self

    def forward(self, input, increment=False):
        """increment: False = full frame; True = the reference's residual update (insert-only, the changed set is
        not dilated, results are approximate by design); "exact" = the frame's points are merged into the scene
        kept from the last full or exact frame (after any delete_voxels / replace_voxels edits) and the network
        recomputes the merged scene, so the result equals a full recompute and the kept scene advances."""
        assert len(input) >= 2, len(input)
        coords, feats = input[0], input[1]
        batch_size = int(input[2]) if len(input) > 2 else 0
        if not feats.is_cuda:
            feats = feats.to(self.device if self.device else "cuda")
        feats = feats.float()
        output = SparseConvNetTensor(metadata=Metadata(self.dimension), spatial_size=self.spatial_size)
        # The previous frame's metadata hands on what this network asked of it beyond the input scale (neighbour maps,
        # stride-2 levels: built by this frame's input layer right away, before feature kernels are queued) and the
        # bounding box it measured (this frame's grid is laid out for it without a round trip to measure its own).
        # Kept per InputLayer, i.e. per network; full and incremental frames each inherit from their own kind.
        kind = "_last_meta_inc" if (increment and increment != "exact") else "_last_meta"
        last = self.__dict__.get(kind)
        if last is not None:
            output.metadata.inherit(last)
        self.__dict__[kind] = output.metadata
        out = feats.new_empty(0)
        if increment == "exact":
            assert self.mode == 4, "the exact incremental mode keeps per-voxel means (InputLayer mode 4)"
            # The kept scene is per-VOXEL state -- coordinates, feature sum, point count -- so its size is the
            # scene's, however many frames have been merged.  The frame's points are appended to the voxel list and
            # the input layer sums (mode 3) features and counts per site: sites of the merged scene, their sums and
            # counts in one pass; the network sees the means.
            scene_c, scene_s, scene_n = self._scene(feats.device)
            coords = coords.to(feats.device).long()
            if coords.shape[1] != scene_c.shape[1]:  # batch column on one side only: batch 0
                pad = lambda c: c if c.shape[1] == 4 else torch.cat([c, c.new_zeros(c.shape[0], 1)], 1)
                coords, scene_c = pad(coords), pad(scene_c)
            n_old, n_new, planes = scene_c.shape[0], coords.shape[0], feats.shape[1]
            merged = torch.empty(n_old + n_new, planes + 1, dtype=torch.float32, device=feats.device)
            merged[:n_old, :planes] = scene_s
            merged[:n_old, planes] = scene_n
            merged[n_old:, :planes] = feats
            merged[n_old:, planes] = 1.0
            SCN.InputLayer_updateOutput(output.metadata, self.spatial_size, torch.cat([scene_c, coords], 0), merged, out,
                                        batch_size, 3)
            sums, counts = out[:, :planes], out[:, planes]
            output.features = sums / counts[:, None]
            output.metadata.setSiteCounts(counts.round().int())  # a later residual frame weights these means correctly
            output.recompute_all = True
            output.new_points = (n_old, n_new)
            sites = output.metadata.getSpatialLocationsDevice(self.spatial_size).t()[:, :scene_c.shape[1]].long()
            _keep(self, save_output=output, _scene_state=(sites.contiguous(), sums.contiguous(), counts.contiguous()),
                  _scene_points=None)
        elif not increment:
            SCN.InputLayer_updateOutput(output.metadata, self.spatial_size, coords, feats, out, batch_size, self.mode)
            output.features = out
            # the scene of the exact mode starts as this frame's points (one point each); they are only turned into
            # voxel state when an exact frame or an edit asks for it
            _keep(self, save_output=output, _scene_points=(coords, feats), _scene_state=None)
        else:
            SCN.Incre_InputLayer_updateOutput(output.metadata, self.spatial_size, coords, feats, out, batch_size,
                                              self.mode, self.save_output.metadata, self.save_output.features)
            output.features = out
        return output

    def _scene(self, device):
        """(coordinates [V, 3|4] int64, feature sums [V, planes], point counts [V]) of the kept scene."""
        state = self.__dict__.get("_scene_state")
        if state is None:
            pts = self.__dict__.get("_scene_points")
            assert pts is not None, "no frame has been run yet"
            c, f = pts
            f = f.to(device).float()
            state = (c.to(device).long(), f, torch.ones(f.shape[0], dtype=torch.float32, device=device))
            _keep(self, _scene_state=state, _scene_points=None)
        return state

    @property
    def scene_coords(self):
        """Coordinates of the kept scene's entries (voxels once an exact frame has merged them)."""
        return self._scene(self.save_output.features.device)[0]

    @staticmethod
    def _voxel_keys(coords):
        """The library's own key: batch << 48 | z << 32 | y << 16 | x (coordinates up to 65534, batch up to 32766)."""
        c = coords.long()
        assert c.numel() == 0 or (int(c.min()) >= 0 and int(c[:, :3].max()) <= 65534), "coordinate outside the key range"
        k = (c[:, 2] << 32) | (c[:, 1] << 16) | c[:, 0]
        if c.shape[1] > 3:
            assert int(c[:, 3].max()) <= 32766, "batch index outside the key range"
            k = k | (c[:, 3] << 48)
        return k

    def delete_voxels(self, coords):
        """Removes the given voxels from the kept scene (effective at the next exact frame).  The reference has no
        deletion; here a deleted voxel simply is no longer part of the scene."""
        c, s, n = self._scene(self.save_output.features.device)
        coords = coords.to(c.device).long()
        if coords.shape[1] != c.shape[1]:
            coords = coords[:, :3] if c.shape[1] == 3 else torch.cat([coords, coords.new_zeros(coords.shape[0], 1)], 1)
        keep = ~torch.isin(self._voxel_keys(c), self._voxel_keys(coords))
        _keep(self, _scene_state=(c[keep], s[keep], n[keep]))

    def replace_voxels(self, coords, feats):
        """Replaces the content of the given voxels by one point each carrying `feats` (a re-drawn feature)."""
        self.delete_voxels(coords)
        c, s, n = self._scene(self.save_output.features.device)
        coords = coords.to(c.device).long()
        if coords.shape[1] != c.shape[1]:
            coords = coords[:, :3] if c.shape[1] == 3 else torch.cat([coords, coords.new_zeros(coords.shape[0], 1)], 1)
        feats = feats.to(s.device).float()
        _keep(self, _scene_state=(torch.cat([c, coords], 0), torch.cat([s, feats], 0),
                                  torch.cat([n, n.new_ones(coords.shape[0])], 0)))


class OutputLayer(Module):
    """SparseConvNetTensor -> N x planes tensor, one row per input point of the InputLayer."""

    def __init__(self, dimension):
        Module.__init__(self)
        self.dimension = dimension

    def forward(self, input, increment=False):
        out = input.features.new_empty(0)
        if not _residual(input, increment):
            SCN.OutputLayer_updateOutput(input.metadata, input.features, out)
            _keep(self, save_input_feats=input.features, save_meta=input.metadata)
            if increment and input.new_points is not None:  # exact mode: rows of this frame's own points
                first, count = input.new_points
                out = out[first:first + count]
        else:
            SCN.Incre_OutputLayer_updateOutput(input.metadata, input.features, out, self.save_meta,
                                               self.save_input_feats)
        return out
