"""Seeded input generators shared by make_golden.py (which runs the reference on them) and the tests (which run the
oracle and the CUDA path on them). Everything is drawn on the CPU with torch.Generator, so a case is a pure
function of its arguments; every fixture stores a checksum of its inputs so a changed RNG fails loudly."""
from __future__ import annotations

import torch

# benchmark configuration 1: fp32, B=2, T=256, d=768, K=4, R=4, lambda=0.25, eps=1e-6, seed 0
CFG1 = dict(b=2, t=256, d=768, K=4, R=4, beta=0.75, eps=1e-6, sigma_h0=1.0, sigma_d=0.5, sigma_q=0.02, seed=0)
# tokens of configuration 1 whose full read states are stored in the fixture
CFG1_TOKENS = (0, 1, 2, 3, 100, 255, 256, 257, 300, 383, 384, 450, 509, 510, 511, 77)


def chain_inputs(b, t, d, K, R, seed, sigma_h0=1.0, sigma_d=0.5, sigma_q=0.02, dtype=torch.float32, **_):
    """h0 [b,t,d], D [N,b,t,d] (the block updates), Q [N-1,d] (queries), G [N,b,t,d] (upstream gradients)."""
    g = torch.Generator().manual_seed(seed)
    N = K * R
    h0 = (torch.randn(b, t, d, generator=g) * sigma_h0).to(dtype)
    D = (torch.randn(N, b, t, d, generator=g) * sigma_d).to(dtype)
    Q = torch.randn(max(N - 1, 1), d, generator=g) * sigma_q
    G = torch.randn(N, b, t, d, generator=g)
    return h0, D, Q, G


def read_inputs(b, t, d, n, dtype, seed, zero_query=False):
    """One read's inputs, in the style of the reference's kernel test (tests/test_fused_dattn.py:35-45):
    per-source scales 0.5 + 0.1 i, a sizeable query, random prior in [0.1, 1), installed coefficients = prior +
    noise, upstream gradients for both outputs."""
    g = torch.Generator().manual_seed(seed)
    deltas = [(torch.randn(b, t, d, generator=g) * (0.5 + 0.1 * i)).to(dtype) for i in range(n)]
    proposal = torch.randn(b, t, d, generator=g).to(dtype)
    h0 = torch.randn(b, t, d, generator=g).to(dtype)
    q = torch.zeros(d) if zero_query else torch.randn(d, generator=g) * 0.3
    prior = torch.rand(n - 1, generator=g) * 0.9 + 0.1
    coeffs = prior.view(1, 1, -1) + 0.2 * torch.randn(b, t, n - 1, generator=g)
    up = torch.randn(b, t, d, generator=g)
    up2 = torch.randn(b, t, n, generator=g)
    return deltas, proposal, h0, q, prior, coeffs, up, up2


def checksum(*tensors) -> float:
    """Order-sensitive fp64 checksum of the inputs."""
    acc = 0.0
    for k, x in enumerate(tensors):
        xf = x.detach().double().flatten()
        w = torch.arange(1, xf.numel() + 1, dtype=torch.float64).remainder(977.0) + 1.0
        acc += (k + 1) * float((xf * w).sum())
    return acc


# single-read fixture cases: (name, b, t, d, n, dtype, seed, boundary)
READ_CASES = (
    ("f32_n2_in", 1, 5, 64, 2, "float32", 11, False),
    ("f32_n3_bd", 2, 3, 64, 3, "float32", 12, True),
    ("f32_n8_in", 1, 7, 128, 8, "float32", 13, False),
    ("f32_n8_bd", 1, 7, 128, 8, "float32", 14, True),
    ("f32_n20_bd", 1, 4, 192, 20, "float32", 15, True),
    ("bf16_n4_bd", 2, 8, 128, 4, "bfloat16", 21, True),
    ("bf16_n16_bd", 1, 9, 256, 16, "bfloat16", 22, True),
    ("bf16_n16_in", 1, 9, 256, 16, "bfloat16", 23, False),
)

# chain fixture cases: (name, b, t, d, K, R, dtype, seed, with_grad)
CHAIN_CASES = (
    ("f32_k3r2", 1, 7, 64, 3, 2, "float32", 31, True),
    ("f32_k2r3", 2, 3, 64, 2, 3, "float32", 32, True),
    ("f32_k4r4", 1, 5, 128, 4, 4, "float32", 33, True),
    ("bf16_k3r3", 1, 6, 128, 3, 3, "bfloat16", 34, True),
    ("f32_k5r16_clamp", 1, 3, 64, 5, 16, "float32", 35, False),   # prior falls below the 1e-8 clamp
)
