"""loopback_b200: Loopback's depth-attention residual read, its update write and their backward as hand-written
sm_100a CUDA kernels behind a C ABI, with the reference's `fused_dattn` entry points on top.

    from loopback_b200 import fused_dattn          # drop-in for the reference module of the same name
    from loopback_b200.cell import LoopDeltaAttnRes  # the read cell (same `combine` as the reference models)
"""
__version__ = "0.1.0"
