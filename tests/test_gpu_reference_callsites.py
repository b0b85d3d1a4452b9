"""The drop-in boundary through the REFERENCE'S OWN call sites.

`install_into_reference()` registers this package's ops under the module paths the reference imports from
(`ops.hils_fwd_bwd_head`, `ops.topk_head_softmax`, ...).  These tests then load two reference files by path:
  models/NaiveBSA/naive_bsa_kernel.py   imports the ops lazily inside `naive_bsa_kernel` (:169-171)
  models/FlashHiLS/hils_attention.py    binds them at import and in `HiLSAttention.__init__` (:9-10, :264-267)
and run the reference's code on top of the B200 kernels.  The files are looked for under $HILS_REFERENCE_ROOT,
baseline/_ref/ (filled by baseline/install_reference.py); the tests skip when neither has them.
Needs a B200.
"""
import importlib.util
import os
import sys
import types

import pytest
import torch

from oracle import hils_oracle as orc
from tests.util import check, golden

pytestmark = pytest.mark.gpu
BF, F32 = torch.bfloat16, torch.float32
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_file(rel):
    for base in (os.environ.get("HILS_REFERENCE_ROOT"), os.path.join(ROOT, "baseline", "_ref")):
        if base and os.path.exists(os.path.join(base, rel)):
            return os.path.join(base, rel)
    pytest.skip(f"reference file {rel} not available on this machine")


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture()
def bound_ops():
    """This package's ops under the reference's module names; removed again afterwards."""
    from hils_attention_b200.attention import install_into_reference
    before = {n: sys.modules.get(n) for n in list(sys.modules) if n == "ops" or n.startswith("ops.")}
    install_into_reference()
    yield
    for n in [n for n in sys.modules if n == "ops" or n.startswith("ops.")]:
        del sys.modules[n]
    sys.modules.update({n: m for n, m in before.items() if m is not None})


@pytest.mark.parametrize("tag", ["mha", "gqa", "lmk"])
def test_reference_naive_bsa_kernel_runs_on_these_ops(bound_ops, tag):
    """The reference's `naive_bsa_kernel`, unmodified, with its lazy `from ops... import` resolved here, reproduces
    the dense naive-BSA goldens (fp32), and so does this package's own `naive_bsa_kernel`."""
    from hils_attention_b200.naive_bsa import naive_bsa_kernel as ours
    ref_mod = _load(_reference_file("models/NaiveBSA/naive_bsa_kernel.py"), "_ref_naive_bsa_kernel_callsite")
    g = golden(f"bsa_{tag}.npz")
    S, W, K, ml = [int(x) for x in g["args"]]
    q, k, v = g["q"].cuda(), g["k"].cuda(), g["v"].cuda()
    o_ref_code = ref_mod.naive_bsa_kernel(q, k, v, chunk_size=S, window_size=W, topk=K, mask_last_token=bool(ml))
    o_ours, aux = ours(q, k, v, chunk_size=S, window_size=W, topk=K, mask_last_token=bool(ml), return_aux=True)
    check(o_ours, g["o"], F32, "package naive_bsa_kernel vs golden")
    check(aux["log_Z"].permute(0, 2, 1, 3), g["log_z"], F32, "log_Z vs golden")
    # the reference's torch.topk may pick non-candidates (weight 0, any id) for rows with fewer than K candidates, and
    # breaks ties as it likes: compare on rows whose K candidates exist
    n_cand = torch.isfinite(aux["score_pool"]).sum(-1)                               # (B,L,h_kv)
    rows = (n_cand >= K).repeat_interleave(q.shape[2] // k.shape[2], dim=2)
    check(o_ref_code[rows], g["o"].cuda()[rows], F32, "reference naive_bsa_kernel on these ops vs golden")


class _RMSNorm(torch.nn.Module):
    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (self.weight * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype))


def _veomni_stub():
    class _Logger:
        def __getattr__(self, name):
            return lambda *a, **k: None
    veomni = types.ModuleType("veomni")
    utils = types.ModuleType("veomni.utils")
    logging = types.ModuleType("veomni.utils.logging")
    logging.get_logger = lambda *a, **k: _Logger()
    import_utils = types.ModuleType("veomni.utils.import_utils")
    import_utils.is_liger_kernel_available = lambda: False
    utils.logging, utils.import_utils = logging, import_utils
    veomni.utils = utils
    return {"veomni": veomni, "veomni.utils": utils, "veomni.utils.logging": logging,
            "veomni.utils.import_utils": import_utils}


def test_reference_attention_module_runs_on_these_ops(bound_ops):
    """The reference's `HiLSAttention` (projections, norms, the whole forward) with the B200 ops bound by its own
    imports: forward and backward equal this package's `HiLSAttentionCore` fed with the module's own q, k, v, and the
    attention output agrees with the oracle chain where the selections agree."""
    from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore
    path = _reference_file("models/FlashHiLS/hils_attention.py")
    stubs = _veomni_stub()
    saved = {n: sys.modules.get(n) for n in stubs}
    sys.modules.update(stubs)
    try:
        mod = _load(path, "_ref_hils_attention_callsite")
    finally:
        for n, m in saved.items():
            if m is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = m
    B, L, hq, hk, D, S, W, K = 1, 1024, 4, 2, 64, 64, 128, 4
    cfg = types.SimpleNamespace(hidden_size=hq * D, num_attention_heads=hq, num_key_value_heads=hk, hils_topk=K,
                                chunk_size=S, sliding_window=W, hils_sliding_window=W, enable_softmax1=False,
                                num_hidden_layers=1, enable_lmk_q_proj=False, apply_hils_rope=False)
    torch.manual_seed(3)
    attn = mod.HiLSAttention(cfg, layer_idx=0, norm_cls=_RMSNorm).cuda().to(BF).train()
    hidden = torch.randn(B, L, hq * D, device="cuda").to(BF).requires_grad_(True)
    out, _ = attn(hidden, position_embeddings=(None, None))
    do = torch.randn_like(out)
    out.backward(do)
    g_ref = hidden.grad.clone()
    # the same chain through this package's module, fed with the reference module's own projections
    hidden2 = hidden.detach().clone().requires_grad_(True)
    q, k, v, lmk_q = attn._project_qkv(hidden2)
    core = HiLSAttentionCore(HiLSAttentionConfig(hq, hk, K, S, W)).train()
    o_core, aux = core(q, k, v, lmk_q, return_aux=True)
    out2 = attn.o_proj(o_core.reshape(B, L, hq * D))
    check(out, out2, BF, "reference module vs HiLSAttentionCore: output")
    out2.backward(do)
    check(g_ref, hidden2.grad, BF, "reference module vs HiLSAttentionCore: d hidden")
    # and against the oracle chain on the module's q, k, v
    qc, kc, vc = (t.detach().cpu() for t in (q, k, v))
    ref, raux = orc.hils_attention_chain(qc, kc, vc, qc, chunk_size=S, window_size=W, topk=K, return_aux=True)
    same = (aux["indices"].cpu() == raux["indices"]).all(-1)
    assert same.float().mean().item() >= 0.99
    rows = same.repeat_interleave(hq // hk, dim=2)
    check(o_core.detach().cpu()[rows], ref[rows], BF, "module attention output vs oracle")
