"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

Generated on the CPU with a fixed generator and then moved, so that the CPU checker and the GPU see
identical bits. These stand in for the LAMBADA activations / OPT weights the reference evaluates on.
"""
import torch


def c1(Q=64, R=256, D=2048, seed=123):
    """Config 1: queries ~N(0,1) fp32, keys ~N(0,0.02) fp32."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(Q, D, generator=g, dtype=torch.float32)
    k = torch.randn(R, D, generator=g, dtype=torch.float32) * 0.02
    return q, k


def fc1(Q=512, R=8192, D=2048, seed=123, dtype=torch.float16):
    """FC1-like: activations ~N(0,1) with 1% outliers x20 (fp16), weights ~N(0,0.02)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(Q, D, generator=g, dtype=torch.float32)
    mask = torch.rand(Q, D, generator=g) < 0.01
    q = torch.where(mask, q * 20.0, q).to(dtype)
    k = torch.randn(R, D, generator=g, dtype=torch.float32) * 0.02
    return q, k


def fc2(Q=512, R=2048, D=8192, seed=123, dtype=torch.float16):
    """FC2-like: activations relu(N(0,1)) (about half zeros, fp16), weights ~N(0,0.02)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.relu(torch.randn(Q, D, generator=g, dtype=torch.float32)).to(dtype)
    k = torch.randn(R, D, generator=g, dtype=torch.float32) * 0.02
    return q, k


def edge_rows(D=512, dtype=torch.float32):
    """Rows that hit the corners of the quantiser: ties, zeros, clamps, huge and tiny magnitudes."""
    rows = []
    base = torch.zeros(D)
    rows.append(base.clone())                                            # all zero: shift 0, all slices empty
    r = base.clone(); r[::2] = 0.005; r[1::2] = -0.005; rows.append(r)   # exact .5 ties after x100
    r = base.clone(); r[:] = 0.635; r[7] = -0.645; rows.append(r)        # 63.5 / -64.5: rounding at the clamp edge
    r = base.clone(); r[0] = 1.0e4; r[1] = -1.0e4; r[2:] = 0.37; rows.append(r)      # big outliers: large shift
    r = base.clone(); r[:256] = 3.0e38; r[256:] = -3.0e38; rows.append(r)            # saturating magnitudes
    r = torch.linspace(-0.7, 0.7, D); rows.append(r)                     # dense sweep through every 7-bit level
    r = base.clone(); r[-1] = -0.64; rows.append(r)                      # lone negative at the end: -64 exactly
    r = base.clone(); r[:] = 1.27; r[300] = 1.275; rows.append(r)        # 127 / 127.5: shift boundary 2^7
    x = torch.stack(rows)
    if dtype != torch.float32:
        x = x.clamp(-6.0e4, 6.0e4).to(dtype)
    return x
