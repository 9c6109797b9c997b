"""The torch extension refuses tensors that do not fit the grid an operator would index them by: a wrong row count,
a wrong plane count or a parameter left on the CPU raises a Python exception before any kernel is launched (the
reference exits the process or reads out of bounds in these cases)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_mismatched_tensors_raise_instead_of_reaching_a_kernel(cuda):
    import sparseconvnet as scn
    from insconv import synth
    SCN = scn.SCN
    coords = torch.from_numpy(synth.boxes_and_spheres(0)).to(cuda)
    feats = torch.randn(coords.shape[0], 16, device=cuda)
    m = scn.Metadata(3)
    size, half = torch.tensor([128, 128, 128]), torch.tensor([64, 64, 64])
    two, three = torch.tensor([2, 2, 2]), torch.tensor([3, 3, 3])
    vox = feats.new_empty(0)
    SCN.InputLayer_updateOutput(m, size, coords, feats, vox, 0, 4)
    n = vox.shape[0]
    w27, w8 = torch.randn(27, 16, 32, device=cuda), torch.randn(8, 16, 32, device=cuda)
    empty = torch.empty(0)
    out = feats.new_empty(0)
    SCN.Convolution_updateOutput(size, half, two, two, m, vox, out, w8, empty)  # builds the coarse scale
    n_coarse = out.shape[0]
    bad_rows = torch.randn(n - 7, 16, device=cuda)
    bad_planes = torch.randn(n, 24, device=cuda)
    cases = [
        lambda: SCN.SubmanifoldConvolution_updateOutput(size, three, m, bad_rows, out, w27, empty, 1),
        lambda: SCN.SubmanifoldConvolution_updateOutput(size, three, m, bad_planes, out, w27, empty, 1),
        lambda: SCN.SubmanifoldConvolution_updateOutput(size, three, m, vox, out, w27, torch.zeros(32), 1),  # CPU bias
        lambda: SCN.SubmanifoldConvolution_updateOutput(size, three, m, vox, out, w27, torch.zeros(31, device=cuda), 1),
        lambda: SCN.Convolution_updateOutput(size, half, two, two, m, bad_rows, out, w8, empty),
        lambda: SCN.Convolution_updateOutput(size, half, two, two, m, bad_planes, out, w8, empty),
        lambda: SCN.Convolution_updateOutput(half, torch.tensor([32, 32, 32]), two, two, m, vox, out, w8, empty),  # other scale
        lambda: SCN.Deconvolution_updateOutput(half, size, two, two, m, vox, out, torch.randn(8, 16, 8, device=cuda), empty),
        lambda: SCN.Deconvolution_updateOutput(half, size, two, two, m, torch.randn(n_coarse, 5, device=cuda), out,
                                               torch.randn(8, 16, 8, device=cuda), empty),
        lambda: SCN.NetworkInNetwork_updateOutput(vox, out, torch.randn(24, 8, device=cuda), empty),
        lambda: SCN.BatchNormalization_updateOutput(vox, out, empty, empty, torch.zeros(16), torch.ones(16, device=cuda), empty,
                                                    empty, 1e-4, 0.9, False, 0.0),  # running mean on the CPU
        lambda: SCN.BatchNormalization_updateOutput(vox, out, empty, empty, torch.zeros(8, device=cuda),
                                                    torch.ones(8, device=cuda), empty, empty, 1e-4, 0.9, False, 0.0),
        lambda: SCN.OutputLayer_updateOutput(m, bad_rows, out),
    ]
    for i, case in enumerate(cases):
        with pytest.raises(RuntimeError):
            case()
    # and the context is intact: a correct call still works
    SCN.SubmanifoldConvolution_updateOutput(size, three, m, vox, out, w27, empty, 1)
    torch.cuda.synchronize()
    SCN.check_errors()
    assert out.shape == (n, 32) and bool(torch.isfinite(out).all())
