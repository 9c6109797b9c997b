"""Factory for the per-scene Metadata object (reference: sparseconvnet/metadata.py:16-17)."""
from . import SCN


def Metadata(dim):
    if dim != 3:
        raise NotImplementedError("only dimension 3 is built (the INS-Conv hot path); got %d" % dim)
    return SCN.Metadata_3()
