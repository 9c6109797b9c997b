"""Host-side helpers of the B200 sparse-convolution library.

  insconv.cabi   ctypes binding of the C ABI declared in include/insconv_b200.h
  insconv.synth  seeded synthetic scenes (the workloads of the benchmark and the parity tests)
"""
