"""CPU oracle of the Loopback read path. TEST INFRASTRUCTURE, NOT PRODUCT.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import this package; the CUDA library and the
`loopback_b200` package never do (and have no CPU fallback).

Two independent restatements of the reference algorithm live here, both pinned against tensors produced by the
unmodified reference (tests/golden/):
  * `c_oracle`  -- ctypes binding of lb_oracle.c (fp32 / fp64, OpenMP; forward, analytic backward, whole chains);
  * `torch_oracle` -- a differentiable torch-CPU restatement (gradients come from autograd).
"""
