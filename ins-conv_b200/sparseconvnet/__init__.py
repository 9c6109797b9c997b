"""sparseconvnet -- the Python operator modules of the INS-Conv hot path on the B200 library.

The public names and call conventions are those of the reference package (THU-luvision/INS-Conv,
sparseconvnet/__init__.py): `import sparseconvnet as scn`, every module's forward takes
`(input, increment=False)`, full frames stash the state the incremental frames need.  Only the
modules the UNet inference path uses exist here; the compute lives in the `sparseconvnet.SCN`
torch extension, which forwards to libinsconv_b200.so.  There is no CPU path.
"""
forward_pass_multiplyAdd_count = 0
forward_pass_hidden_states = 0

from . import SCN  # noqa: E402  (the compiled extension; importing fails loudly when it is not built)
from .tensor import SparseConvNetTensor  # noqa: E402
from .metadata import Metadata  # noqa: E402
from .containers import Sequential, ConcatTable, AddTable, JoinTable, Identity  # noqa: E402
from .layers import (SubmanifoldConvolution, ValidConvolution, Convolution, Deconvolution,  # noqa: E402
                     BatchNormalization, BatchNormReLU, BatchNormLeakyReLU, NetworkInNetwork,
                     InputLayer, OutputLayer)
from .nets import UNet  # noqa: E402
from .utils import toLongTensor, optionalTensor, set_precision, get_precision  # noqa: E402
