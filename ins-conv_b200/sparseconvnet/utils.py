"""Small helpers shared by the modules (reference: sparseconvnet/utils.py:13-28)."""
import torch

from . import SCN


_EMPTY = torch.empty(0)


def toLongTensor(dimension, x):
    """int, list/tuple or LongTensor -> CPU LongTensor of `dimension` entries."""
    if isinstance(x, torch.Tensor):
        return x.to(dtype=torch.int64, device="cpu")
    if isinstance(x, (list, tuple)):
        assert len(x) == dimension
        return torch.tensor(list(x), dtype=torch.int64)
    return torch.full((dimension,), int(x), dtype=torch.int64)


def optionalTensor(module, name):
    """The named attribute, or an empty tensor ('no bias' convention of the operator interface)."""
    t = module._parameters.get(name)  # direct table lookup: a missing attribute on a Module is slow to discover
    return t if t is not None else _EMPTY


def set_precision(p):
    """'fp32' (default, bit-for-bit deterministic FFMA), 'tf32' (tensor cores reading the fp32 features as tf32), or
    'fp16' (as tf32, and a BatchNorm directly in front of a convolution with 32 or 64 planes on both sides hands it
    fp16 rows: half the bytes to gather, 11 significant bits instead of tf32's 10)."""
    SCN.set_precision(p)
    _precision[0] = SCN.get_precision()


def get_precision():
    return SCN.get_precision()


# what set_precision() last selected: the modules read this mirror on every call instead of asking the extension
_precision = [SCN.get_precision()]
