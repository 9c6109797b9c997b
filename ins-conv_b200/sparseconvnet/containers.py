"""Graph glue: Sequential, ConcatTable, AddTable, JoinTable, Identity
(reference: sparseconvnet/sequential.py:9-25, tables.py:13-55, identity.py:10-15)."""
import torch

from .tensor import SparseConvNetTensor
from .utils import _precision


class _Container(torch.nn.Sequential):
    def add(self, module):
        self._modules[str(len(self._modules))] = module
        self.__dict__.pop("_half_plan", None)
        return self


def _run(module, input, increment):
    """module(input, increment) without torch.nn.Module.__call__'s bookkeeping when no hook is installed."""
    if module._forward_hooks or module._forward_pre_hooks:
        return module(input, increment)
    return module.forward(input, increment)


class Sequential(_Container):
    def forward(self, input, increment=False):
        if _precision[0] != "fp16":
            for module in self._modules.values():
                input = _run(module, input, increment)
            return input
        # 'fp16' precision: a BatchNorm directly in front of a convolution with an fp16 kernel writes fp16 rows for it.
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
        return input

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

    def forward(self, input, increment=False):
        return input[0].like(torch.cat([t.features for t in input], 1))

    def input_spatial_size(self, out_size):
        return out_size


class Identity(torch.nn.Module):
    def forward(self, input, increment=False):
        return input

    def input_spatial_size(self, out_size):
        return out_size
