"""Graph glue: Sequential, ConcatTable, AddTable, JoinTable, Identity
(reference: sparseconvnet/sequential.py:9-25, tables.py:13-55, identity.py:10-15)."""
import torch

from .tensor import SparseConvNetTensor
from .utils import _precision


# [True]: in 'fp16' precision full frames fold BatchNorm + ReLU and residual sums into the epilogue of the convolution
# in front of them (sparseconvnet.set_epilogue_fusion)
fuse_epilogues = [True]
# [True]: full frames keep what the reference-style incremental frames read later (every BatchNorm's fp32 input).
# False: a convolution whose only consumer is a fused BatchNorm does not store its fp32 result at all.
keep_state = [True]


class _Container(torch.nn.Sequential):
    def add(self, module):
        self._modules[str(len(self._modules))] = module
        self.__dict__.pop("_half_plan", None)
        self.__dict__.pop("_fuse_plan", None)
        return self


def _run(module, input, increment):
    """module(input, increment) without torch.nn.Module.__call__'s bookkeeping when no hook is installed."""
    if module._forward_hooks or module._forward_pre_hooks:
        return module(input, increment)
    return module.forward(input, increment)


def _hooked(module):
    return bool(module._forward_hooks or module._forward_pre_hooks)


def _bn_consumer(module, after):
    """The BatchNormalization that consumes, as fp16 rows for a convolution right behind it, whatever is handed to
    `module` (`after`: the module that follows `module` in its Sequential) -- or None.  A ConcatTable hands its input to
    every child: the BatchNorm of one Sequential child counts when the other children pass the input on untouched or
    read it as fp32 (Identity, NetworkInNetwork)."""
    from .layers import BatchNormalization, NetworkInNetwork, takes_half_rows
    if isinstance(module, BatchNormalization):
        ok = after is not None and takes_half_rows(after) and not module.training and not _hooked(module) and \
            not _hooked(after) and module.nPlanes % 8 == 0
        return module if ok else None
    if isinstance(module, Sequential):
        mods = list(module._modules.values())
        return _bn_consumer(mods[0], mods[1] if len(mods) > 1 else None) if mods and not _hooked(module) else None
    if isinstance(module, ConcatTable) and not _hooked(module):
        found = None
        for child in module._modules.values():
            if isinstance(child, (Identity, NetworkInNetwork)):
                continue
            bn = _bn_consumer(child, None) if isinstance(child, Sequential) else None
            if bn is None or found is not None:
                return None
            found = bn
        return found
    return None


class Sequential(_Container):
    def forward(self, input, increment=False, next_bn=None, addend=None):
        """next_bn / addend are used by an enclosing container in 'fp16' precision: next_bn = the BatchNormalization
        that consumes this container's output (its result is then formed in the epilogue of the last convolution here),
        addend = features added to the output of the last convolution here (the shortcut of a residual block)."""
        if _precision[0] != "fp16":
            for module in self._modules.values():
                input = _run(module, input, increment)
            return input if addend is None else input.like(input.features + addend)
        from .layers import _residual
        # The same plan serves residual (reference-style incremental) frames: there the fused BatchNorm is the
        # incremental one (every convolution checks that the saved frame left what it needs, else it runs unfused)
        # and the residual of a block's shortcut is added in the branch's last convolution.
        if self.training or not fuse_epilogues[0] or (_residual(input, increment) and not keep_state[0]):
            return self._forward_half_rows(input, increment, addend)
        # 'fp16' precision, full frame: besides BatchNorms that hand fp16 rows to the convolution behind them, (1) a
        # convolution that reads fp16 rows forms the result of the BatchNorm that consumes its output in its own
        # epilogue, (2) the sum of a residual block [ConcatTable(shortcut, branch), AddTable] is formed in the epilogue
        # of the branch's last convolution.  What consumes what depends on the module tree alone: worked out once.
        plan = self.__dict__.get("_fuse_plan")
        if plan is None or plan[0] != len(self._modules):
            plan = (len(self._modules), self._make_plan())
            self.__dict__["_fuse_plan"] = plan
        mods, steps = plan[1]
        n = len(mods)
        i = 0
        while i < n:
            kind, consumer = steps[i]
            module = mods[i]
            last = i == n - 1 or (kind == "block" and i == n - 2)
            if last and consumer is None:
                consumer = next_bn
            extra_add = addend if last else None
            if kind == "block":  # [ConcatTable(shortcut, branch), AddTable]: the branch's last convolution adds the shortcut
                shortcut = _run(module._modules["0"], input, increment)
                add = shortcut.features if extra_add is None else shortcut.features + extra_add
                input = module._modules["1"].forward(input, increment, consumer, add)
                i += 2
                continue
            if kind == "conv":
                kw = {"fuse_bn": consumer}
                if consumer is not None and not keep_state[0] and i + 1 < n and mods[i + 1] is consumer and hasattr(module, "dilated_rate"):
                    kw["raw_needed"] = False
                if extra_add is not None and kind == "conv" and hasattr(module, "dilated_rate") and "bias" not in module._parameters:
                    kw["addend"] = extra_add
                    extra_add = None
                input = module.forward(input, increment, **kw)
            elif kind == "seq":
                input = module.forward(input, increment, consumer, extra_add)
                extra_add = None
            elif kind == "bn_half":
                input = module.forward(input, increment, True)
            elif kind == "join":
                input = module.forward(input, increment, consumer)
            else:
                input = _run(module, input, increment)
            if extra_add is not None:
                input = input.like(input.features + extra_add)
            i += 1
        return input

    def _make_plan(self):
        from .layers import BatchNormalization, Convolution, SubmanifoldConvolution, takes_half_rows
        mods = list(self._modules.values())
        n = len(mods)
        steps = []
        for i, m in enumerate(mods):
            after = mods[i + 1] if i + 1 < n else None
            after2 = mods[i + 2] if i + 2 < n else None
            if isinstance(m, ConcatTable) and isinstance(after, AddTable) and len(m._modules) == 2 and \
                    isinstance(m._modules["1"], Sequential) and not (_hooked(m) or _hooked(after) or _hooked(m._modules["1"])):
                steps.append(("block", _bn_consumer(after2, mods[i + 3] if i + 3 < n else None) if after2 is not None else None))
            elif isinstance(m, (SubmanifoldConvolution, Convolution)) and takes_half_rows(m) and not _hooked(m):
                steps.append(("conv", _bn_consumer(after, after2) if after is not None else None))
            elif isinstance(m, Sequential) and not _hooked(m):
                steps.append(("seq", _bn_consumer(after, after2) if after is not None else None))
            elif isinstance(m, BatchNormalization) and after is not None and takes_half_rows(after) and \
                    not (_hooked(m) or after._forward_pre_hooks):
                steps.append(("bn_half", None))
            elif isinstance(m, JoinTable) and not _hooked(m):  # its BatchNorm consumer is applied while the planes are joined
                steps.append(("join", _bn_consumer(after, after2) if after is not None else None))
            else:
                steps.append(("plain", None))
        return mods, steps

    def _forward_half_rows(self, input, increment, addend=None):
        # a BatchNorm directly in front of a convolution with an fp16 kernel writes fp16 rows for it.
        # Which modules those are depends on the module list alone and is worked out once.
        plan = self.__dict__.get("_half_plan")
        if plan is None or plan[0] != len(self._modules):
            from .layers import BatchNormalization, takes_half_rows
            mods = list(self._modules.values())
            plan = (len(mods), [isinstance(m, BatchNormalization) and i + 1 < len(mods) and takes_half_rows(mods[i + 1])
                                for i, m in enumerate(mods)], mods)
            self.__dict__["_half_plan"] = plan
        mods = plan[2]
        for i, half in enumerate(plan[1]):
            module = mods[i]
            if half and not (module._forward_hooks or module._forward_pre_hooks or mods[i + 1]._forward_pre_hooks):
                input = module.forward(input, increment, True)
            else:
                input = _run(module, input, increment)
        return input if addend is None else input.like(input.features + addend)

    def input_spatial_size(self, out_size):
        for module in reversed(list(self)):
            out_size = module.input_spatial_size(out_size)
        return out_size


class ConcatTable(_Container):
    """Feeds the same input to every child and returns the list of results."""

    def forward(self, input, increment=False):
        return [_run(module, input, increment) for module in self._modules.values()]

    def input_spatial_size(self, out_size):
        return self._modules["0"].input_spatial_size(out_size)


class AddTable(_Container):
    """Sums the features of a list of tensors living on the same sites."""

    def forward(self, input, increment=False):
        feats = input[0].features
        for t in input[1:]:
            feats = feats + t.features
        return input[0].like(feats)

    def input_spatial_size(self, out_size):
        return out_size


class JoinTable(_Container):
    """Concatenates the feature planes of a list of tensors living on the same sites."""

    def forward(self, input, increment=False, fuse_bn=None):
        """fuse_bn ('fp16' precision, full frames): the BatchNormalization that consumes the joined tensor in front of a
        convolution that reads fp16 rows; its result is then written in the same pass as the concatenation."""
        if fuse_bn is not None and len(input) == 2:
            from .layers import SCN, _finish_fused, _residual, bn_affine
            a, b = input[0].features, input[1].features
            if not _residual(input, increment) and not fuse_bn.training and a.is_cuda and a.dtype == torch.float32 and \
                    b.dtype == torch.float32 and a.dim() == 2 and b.dim() == 2 and a.size(0) == b.size(0) and a.size(0) > 0 and \
                    a.size(1) % 4 == 0 and b.size(1) % 4 == 0 and a.size(1) + b.size(1) == fuse_bn.nPlanes:
                scale, shift = bn_affine(fuse_bn)
                joined, rows = a.new_empty(0), a.new_empty(0, dtype=torch.float16)
                SCN.JoinTable_BatchNormalization_updateOutput(a, b, joined, scale, shift, float(fuse_bn.leakiness), rows)
                return _finish_fused(input[0].like(joined), fuse_bn, rows)
        return input[0].like(torch.cat([t.features for t in input], 1))

    def input_spatial_size(self, out_size):
        return out_size


class Identity(torch.nn.Module):
    def forward(self, input, increment=False):
        return input

    def input_spatial_size(self, out_size):
        return out_size
