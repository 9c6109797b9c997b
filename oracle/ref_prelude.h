// First thing in the translation unit that build_ref.py assembles: everything the reference's sources
// expect to find already declared.  TEST INFRASTRUCTURE (see build_ref.py).
#pragma once
#include <ATen/ATen.h>
#include <torch/types.h>
#include <torch/extension.h>  // Metadata/resultHash.h includes it; it must be seen before CUDA is redefined below
#include <cassert>
#include <iostream>
#include <memory>
#include "ref_emu.h"    // CUDA launch / runtime / intrinsics on the host

// "CUDA tensors" of the reference's host code are CPU tensors here: at::CUDA(type) and torch::kCUDA name the CPU.
#define CUDA CPU
#define kCUDA kCPU

// The reference targets PyTorch 1.1, where dividing an integer tensor by an integer stays integral (truncating
// division); today's `/` would return floats.  One place relies on it: coarse coordinates = fine coordinates / 2
// (Metadata/ConvolutionRules.h:370).  An exact-match overload restores the old meaning for integer tensors.
namespace at {
inline Tensor operator/(const Tensor &a, int b) {
  return isIntegralType(a.scalar_type(), false) ? at::div(a, b, "trunc") : at::div(a, b);
}
}  // namespace at
