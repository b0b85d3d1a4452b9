"""Shared helpers of the GPU parity tests."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# tolerances of the parity contract: bf16 max-abs 2e-2 / max-rel 1e-2, fp32 1e-4
TOL = {torch.bfloat16: (2e-2, 1e-2), torch.float32: (1e-4, 1e-4)}


def golden(name):
    d = np.load(os.path.join(GOLDEN, name))
    return {k: torch.from_numpy(d[k]) for k in d.files}


def check(x, ref, dtype, what="", scale=1.0):
    """|x - ref| <= atol*scale + rtol*|ref| elementwise; infinities must coincide."""
    atol, rtol = TOL[dtype]
    x = x.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert x.shape == ref.shape, f"{what}: shape {tuple(x.shape)} vs {tuple(ref.shape)}"
    fin = torch.isfinite(ref)
    assert torch.equal(fin, torch.isfinite(x)), f"{what}: non-finite pattern differs"
    err = (x[fin] - ref[fin]).abs()
    bound = atol * scale + rtol * ref[fin].abs()
    bad = err > bound
    assert not bool(bad.any()), (f"{what}: {int(bad.sum())} of {err.numel()} outside tolerance, "
                                 f"max err {float(err.max()):.3e}")


def cuda(t, dtype=None):
    t = t.cuda()
    return t.to(dtype) if (dtype is not None and t.is_floating_point()) else t


def rms_ratio(x, ref):
    x, ref = x.detach().float().cpu(), ref.detach().float().cpu()
    return float((x - ref).square().mean().sqrt() / ref.square().mean().sqrt().clamp_min(1e-30))
