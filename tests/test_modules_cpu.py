"""Host-side logic of the Python modules that needs no GPU: which BatchNorms hand fp16 rows to the convolution
behind them in the 'fp16' precision, and the bookkeeping around it."""
import torch

import sparseconvnet as scn
from sparseconvnet.layers import takes_half_rows, _f32



def test_which_convolutions_take_half_rows():
    yes = [scn.SubmanifoldConvolution(3, 32, 32, 3, False), scn.Convolution(3, 32, 64, 2, 2, False),
           scn.Deconvolution(3, 64, 32, 2, 2, False), scn.SubmanifoldConvolution(3, 96, 96, 3, False),
           scn.SubmanifoldConvolution(3, 224, 224, 3, False), scn.SubmanifoldConvolution(3, 448, 224, 3, False)]
    no = [scn.SubmanifoldConvolution(3, 3, 32, 3, False),        # first layer: 3 planes
          scn.SubmanifoldConvolution(3, 16, 16, 3, False),       # below 32 planes
          scn.SubmanifoldConvolution(3, 32, 32, 3, True),        # has a bias
          scn.SubmanifoldConvolution(3, 256, 256, 3, False),     # more than 224 output planes
          scn.SubmanifoldConvolution(3, 48, 32, 3, False),       # not a multiple of 32
          scn.NetworkInNetwork(64, 32, False), scn.BatchNormReLU(32), scn.Identity()]
    assert all(takes_half_rows(m) for m in yes)
    assert not any(takes_half_rows(m) for m in no)


def test_unet_plan_marks_every_batchnorm_in_front_of_a_convolution():
    # the UNet of the reference's model.py: 65 BatchNorms, all but the last one sit directly in front of a
    # convolution with an fp16 kernel
    net = scn.Sequential().add(scn.SubmanifoldConvolution(3, 3, 32, 3, False)).add(
        scn.UNet(3, 2, [32, 64, 96, 128, 160, 192, 224], residual_blocks=True)).add(scn.BatchNormReLU(32))
    marked = total = 0
    for seq in [m for m in net.modules() if isinstance(m, scn.Sequential)]:
        mods = list(seq._modules.values())
        for i, m in enumerate(mods):
            if isinstance(m, scn.BatchNormalization):
                total += 1
                marked += int(i + 1 < len(mods) and takes_half_rows(mods[i + 1]))
    assert total == 65 and marked == 64


def test_widened_rows_are_shared_and_released():
    owner = scn.Identity()
    t = torch.arange(6, dtype=torch.float16).reshape(2, 3)
    a, b = _f32(owner, t), _f32(scn.Identity(), t)
    assert a is b and a.dtype == torch.float32 and torch.equal(a, t.float())
    f = torch.ones(2, 2)
    assert _f32(owner, f) is f  # fp32 rows pass through
    from sparseconvnet import layers
    before = len(layers._wide_rows)
    del t, a, b
    assert len(layers._wide_rows) == before - 1


def test_precision_names():
    scn.set_precision("fp16")
    try:
        assert scn.get_precision() == "fp16"
    finally:
        scn.set_precision("fp32")
    assert scn.get_precision() == "fp32"
    try:
        scn.set_precision("bf16")
    except RuntimeError as e:
        assert "precision" in str(e)
    else:
        raise AssertionError("an unknown precision must be refused")
