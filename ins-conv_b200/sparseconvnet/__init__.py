"""sparseconvnet -- the Python operator modules of the INS-Conv hot path on the B200 library.

The public names and call conventions are those of the reference package (THU-luvision/INS-Conv,
sparseconvnet/__init__.py): `import sparseconvnet as scn`, every module's forward takes
`(input, increment=False)`, full frames stash the state the incremental frames need.  Only the
modules the UNet inference path uses exist here; the compute lives in the `sparseconvnet.SCN`
torch extension, which forwards to libinsconv_b200.so.  There is no CPU path.
"""
forward_pass_multiplyAdd_count = 0
forward_pass_hidden_states = 0

import torch  # noqa: E402,F401  (the extension creates tensors while it loads: torch has to be initialised first)

from . import SCN  # noqa: E402  (the compiled extension; importing fails loudly when it is not built)
from .tensor import SparseConvNetTensor  # noqa: E402
from .metadata import Metadata  # noqa: E402
from .containers import Sequential, ConcatTable, AddTable, JoinTable, Identity  # noqa: E402
from .layers import (SubmanifoldConvolution, ValidConvolution, Convolution, Deconvolution,  # noqa: E402
                     BatchNormalization, BatchNormReLU, BatchNormLeakyReLU, NetworkInNetwork,
                     InputLayer, OutputLayer)
from .nets import UNet  # noqa: E402
from .utils import toLongTensor, optionalTensor, set_precision, get_precision  # noqa: E402


def set_epilogue_fusion(on):
    """In 'fp16' precision a full frame folds BatchNorm + ReLU and the sums of residual blocks into the epilogue of
    the convolution in front of them (default on).  Results are the same to rounding; off runs every module as a
    kernel of its own."""
    from . import containers
    containers.fuse_epilogues[0] = bool(on)


def set_halo_exchange(fn):
    """fn(SparseConvNetTensor) is run on the result of every full-frame SubmanifoldConvolution and Convolution, or None
    to switch it off.  One scene split over several GPUs restores its halo rows here (insconv.slab.SlabExchange)."""
    from . import layers
    layers.halo_exchange[0] = fn


def overlap_grid_build(on):
    """on: the grid builds of the following full frames (InputLayer: site ranking, coarse scales, rulebook maps) run on a
    stream of their own, so that the build of frame t + 1 overlaps the last layers of frame t and the host, which waits
    for the site counts, is not held up by frame t.  The call records "inputs ready" on the current stream: the builds
    wait for the work queued on it so far and for nothing later, so the coordinates of the frames that follow must be
    complete at that point (resident in device memory; call again after queueing new copies).  off (default): builds run
    on the current stream like everything else."""
    SCN.overlap_grid_build(bool(on))


def set_incremental_state(on):
    """Full frames keep the state that reference-style incremental frames (increment=True) read later (default on).
    Off is for pure full-frame inference: a convolution whose output only feeds a BatchNorm fused into its epilogue then
    stores the normalised fp16 rows alone; an incremental frame after such a full frame raises."""
    from . import containers
    containers.keep_state[0] = bool(on)
