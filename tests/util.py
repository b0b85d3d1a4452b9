"""Shared helpers of the GPU parity tests."""
import atexit
import json
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# tolerances of the parity contract: bf16 max-abs 2e-2 / max-rel 1e-2, fp32 1e-4
CONTRACT = {torch.bfloat16: (2e-2, 1e-2), torch.float32: (1e-4, 1e-4)}
# what the tests enforce: half the contract in bf16 and a tenth of it in fp32 (the worst error observed over the
# whole suite is 0.46 of the bf16 bound below and 0.12 of the fp32 one)
TOL = {torch.bfloat16: (1e-2, 5e-3), torch.float32: (1e-5, 1e-5)}


def golden(name):
    d = np.load(os.path.join(GOLDEN, name))
    return {k: torch.from_numpy(d[k]) for k in d.files}


_observed = []


def _dump_observed():
    path = os.environ.get("HILS_PARITY_LOG")
    if path and _observed:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "a") as f:
            for rec in _observed:
                f.write(json.dumps(rec) + "\n")


atexit.register(_dump_observed)


def check(x, ref, dtype, what="", scale=None):
    """The one tolerance rule of the parity tests:

        |x - ref| <= atol * s + rtol * |ref|   elementwise,   s = max(1, max|ref|) over the tensor

    with (atol, rtol) = TOL[dtype], tighter than the contract's (2e-2, 1e-2) for bf16 and 1e-4 for fp32.  Outputs of the path are O(1), where
    this is the contract's max-abs / max-rel bound as it stands; gradients are sums over thousands of products
    and can be much larger than 1, where the absolute part is taken relative to the tensor's largest entry.
    `scale`, where a test passes it, multiplies s and is stated with its reason at the call.
    Infinities must coincide.  With HILS_PARITY_LOG set, the worst observed error of every call is appended to
    that file (one JSON object per call)."""
    atol, rtol = TOL[dtype]
    x = x.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert x.shape == ref.shape, f"{what}: shape {tuple(x.shape)} vs {tuple(ref.shape)}"
    fin = torch.isfinite(ref)
    assert torch.equal(fin, torch.isfinite(x)), f"{what}: non-finite pattern differs"
    if not bool(fin.any()):
        return
    err = (x[fin] - ref[fin]).abs()
    mag = float(ref[fin].abs().max())
    s = max(1.0, mag) * (1.0 if scale is None else float(scale))
    bound = atol * s + rtol * ref[fin].abs()
    worst = float((err / bound).max())
    _observed.append({"what": what, "dtype": str(dtype).replace("torch.", ""), "max_abs_err": float(err.max()),
                      "max_abs_ref": mag, "err_over_bound": worst, "n": int(err.numel()),
                      "test": os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0]})
    bad = err > bound
    assert not bool(bad.any()), (f"{what}: {int(bad.sum())} of {err.numel()} outside tolerance, "
                                 f"max err {float(err.max()):.3e} (max |ref| {mag:.3e}, worst err/bound {worst:.2f})")


def cuda(t, dtype=None):
    t = t.cuda()
    return t.to(dtype) if (dtype is not None and t.is_floating_point()) else t


def rms_ratio(x, ref):
    x, ref = x.detach().float().cpu(), ref.detach().float().cpu()
    return float((x - ref).square().mean().sqrt() / ref.square().mean().sqrt().clamp_min(1e-30))
