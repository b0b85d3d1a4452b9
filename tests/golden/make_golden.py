"""Generate the golden fixtures in this directory by running the reference's OWN PyTorch
functions on seeded CPU inputs.

Usage (needs the reference checkout; the fixtures themselves are committed, so tests never
need it):   python tests/golden/make_golden.py /path/to/HiLS-Attention

Reference functions executed:
  ops/chunk_attn_pool_tilelang.py   chunk_attn_pool_ref
  ops/topk_head_softmax.py          ref_softmax_topk_max_pooling
  ops/hils_fwd_bwd_head.py          hils_torch_ref
  models/NaiveBSA/naive_bsa_kernel.py  exact_chunk_log_z      (loaded by file path)
  models/NaiveBSA/naive_bsa_ref.py     naive_bsa_attention    (loaded by file path)
  models/FlashHiLS/modeling_olmo_hils.py  rms_norm            (its source text is compiled on its own:
                                                               the module imports packages absent here)
  ops/rope_tilelang_fp32.py         rotate_half_torch, with the torch formula of that file's test
Each fixture stores the inputs (fp32 arrays; bf16 cases hold bf16-representable values),
the call's scalar arguments and the reference outputs / autograd gradients.
"""
import importlib.util
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _np(t):
    return t.detach().float().numpy() if t.is_floating_point() else t.detach().numpy()


def _bf(t):
    return t.to(torch.bfloat16).float()


def main(ref_root):
    sys.path.insert(0, ref_root)
    from ops.chunk_attn_pool_tilelang import chunk_attn_pool_ref
    from ops.topk_head_softmax import ref_softmax_topk_max_pooling
    from ops.hils_fwd_bwd_head import hils_torch_ref
    bsa_k = _load(os.path.join(ref_root, "models/NaiveBSA/naive_bsa_kernel.py"), "_ref_naive_bsa_kernel")
    bsa_r = _load(os.path.join(ref_root, "models/NaiveBSA/naive_bsa_ref.py"), "_ref_naive_bsa_ref")

    # ---- pool: forward (bf16-valued inputs) + fp32 autograd gradients ----------------
    for tag, (B, N, H, D, S) in {"a": (1, 6, 2, 64, 64), "b": (2, 3, 1, 128, 32)}.items():
        g = torch.Generator().manual_seed(100 + ord(tag))
        mu = _bf(torch.randn(B, N, H, D, generator=g)).requires_grad_(True)
        kc = _bf(torch.randn(B, N, S, H, D, generator=g)).requires_grad_(True)
        gk = _bf(torch.randn(B, N, H, D, generator=g))
        gb = torch.randn(B, N, H, generator=g)
        lk, lb = chunk_attn_pool_ref(mu, kc, 1.0 / math.sqrt(D))
        (lk * gk).sum().add((lb * gb).sum()).backward()
        np.savez_compressed(os.path.join(HERE, f"pool_{tag}.npz"), mu_q=_np(mu), k_chunked=_np(kc),
                            g_lmk_k=_np(gk), g_lmk_b=_np(gb), lmk_k=_np(lk), lmk_b=_np(lb),
                            d_mu_q=_np(mu.grad), d_k=_np(kc.grad))

    # ---- selection ---------------------------------------------------------------------
    cases = {
        # tag: B, L, N, h_kv, G, D, K, S, W, q_offset, bias, per_qhead, gumbel
        "shared": (1, 640, 10, 2, 2, 64, 4, 64, 64, 0, False, False, True),
        "bias_pq": (2, 512, 8, 1, 4, 32, 4, 64, 128, 0, True, True, False),
        "decode": (1, 3, 16, 2, 1, 64, 8, 64, 64, 1021, True, False, False),
        "ragged": (1, 333, 5, 1, 2, 64, 8, 64, 64, 0, False, False, False),
    }
    for tag, (B, L, N, hk, G, D, K, S, W, qo, use_b, pq, gum) in cases.items():
        g = torch.Generator().manual_seed(200 + len(tag))
        q = _bf(torch.randn(B, L, hk, G, D, generator=g))
        lm = _bf(torch.randn(B, N, hk * G if pq else hk, D, generator=g))
        lse = torch.randn(B, L, hk * G, generator=g) + 3.0
        bias = torch.randn(B, N, hk * G, generator=g) if use_b else None
        gn = None
        if gum:
            u = torch.rand(1, 1, hk * G, N, generator=g).clamp_(1e-20, 1 - 1e-7)
            gn = -torch.log(-torch.log(u))
        idx, sc = ref_softmax_topk_max_pooling(q, lm, lse, K, S, W, is_causal=True, q_offset=qo,
                                               bias=bias, gumbel_noise=gn)
        out = dict(q=_np(q), lmks=_np(lm), lse_swa=_np(lse), indices=_np(idx.to(torch.int32)),
                   scores=_np(sc), args=np.array([K, S, W, qo], dtype=np.int64))
        if use_b:
            out["bias"] = _np(bias)
        if gum:
            out["gumbel"] = _np(gn)
        np.savez_compressed(os.path.join(HERE, f"topk_{tag}.npz"), **out)

    # ---- sparse attention: fp32 forward + gradients ------------------------------------
    for tag, (B, L, T, H, HQ, D, K, S) in {"a": (1, 256, 256, 1, 2, 64, 4, 32),
                                           "kvlong": (1, 96, 160, 2, 2, 32, 4, 32)}.items():
        g = torch.Generator().manual_seed(300 + ord(tag[0]))
        nblk = T // S
        idx = torch.full((B, L, H, K), -1, dtype=torch.int32)
        for t in range(L):
            mb = min((t + (T - L)) // S + 1, nblk)
            ns = min(K, mb)
            for h in range(H):
                idx[:, t, h, :ns] = torch.randperm(mb, generator=g)[:ns].sort()[0].to(torch.int32)
        q = torch.randn(B, L, HQ, D, generator=g).requires_grad_(True)
        k = torch.randn(B, T, H, D, generator=g).requires_grad_(True)
        v = torch.randn(B, T, H, D, generator=g).requires_grad_(True)
        logit = torch.randn(B, L, HQ, K, generator=g)
        logit.masked_fill_(idx.repeat_interleave(HQ // H, dim=2) == -1, float("-inf"))
        w = torch.nan_to_num(torch.softmax(logit, -1), 0.0).requires_grad_(True)
        do = torch.randn(B, L, HQ, D, generator=g)
        o = hils_torch_ref(q, k, v, w, idx, chunk_size=S, sm_scale=1.0 / math.sqrt(D), block_q=1,
                           mask_last_token=True)
        o.backward(do)
        np.savez_compressed(os.path.join(HERE, f"sparse_{tag}.npz"), q=_np(q), k=_np(k), v=_np(v),
                            w=_np(w), indices=_np(idx), do=_np(do), o=_np(o), dq=_np(q.grad),
                            dk=_np(k.grad), dv=_np(v.grad), dw=_np(w.grad),
                            args=np.array([S], dtype=np.int64))

    # ---- exact chunk log Z ---------------------------------------------------------------
    for tag, (B, L, hq, hk, D, S, W) in {"a": (1, 300, 2, 1, 32, 32, 64),
                                         "b": (1, 256, 2, 2, 64, 64, 64)}.items():
        g = torch.Generator().manual_seed(400 + ord(tag))
        q = torch.randn(B, L, hq, D, generator=g)
        k = torch.randn(B, L, hk, D, generator=g)
        lz = bsa_k.exact_chunk_log_z(q, k, chunk_size=S, window_size=W, sm_scale=1.0 / math.sqrt(D))
        np.savez_compressed(os.path.join(HERE, f"logz_{tag}.npz"), q=_np(q), k=_np(k), log_z=_np(lz),
                            args=np.array([S, W], dtype=np.int64))

    # ---- whole naive block-sparse attention (dense reference) -----------------------------
    for tag, (B, L, hq, hk, D, S, W, K, ml) in {"mha": (1, 384, 2, 2, 32, 32, 64, 4, False),
                                                "gqa": (2, 250, 4, 2, 32, 32, 96, 4, False),
                                                "lmk": (1, 256, 2, 1, 32, 32, 64, 2, True)}.items():
        g = torch.Generator().manual_seed(500 + ord(tag[0]))
        q = torch.randn(B, L, hq, D, generator=g)
        k = torch.randn(B, L, hk, D, generator=g)
        v = torch.randn(B, L, hk, D, generator=g)
        o, aux = bsa_r.naive_bsa_attention(q, k, v, chunk_size=S, window_size=W, topk=K,
                                           mask_last_token=ml, return_aux=True)
        np.savez_compressed(os.path.join(HERE, f"bsa_{tag}.npz"), q=_np(q), k=_np(k), v=_np(v), o=_np(o),
                            lse_swa=_np(aux["log_Z_swa"]), log_z=_np(aux["log_Z_chunk"]),
                            args=np.array([S, W, K, int(ml)], dtype=np.int64))
    norm_rope_fixtures(ref_root)
    print("golden fixtures written to", HERE)


def _function_from_source(path, name):
    """Compile ONE top-level function of a reference file from its source text (for modules whose
    imports are not installed here) and return it."""
    import ast
    src = open(path).read()
    node = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == name)
    ns = {"torch": torch}
    exec(compile(ast.Module(body=[node], type_ignores=[]), path, "exec"), ns)
    return ns[name]


def norm_rope_fixtures(ref_root):
    """Per-head RMSNorm (the reference's rms_norm) followed by the rotary embedding (the reference's
    rotate_half_torch in the formula of its own test), forward and autograd gradients."""
    sys.path.insert(0, ref_root)
    from ops.rope_tilelang_fp32 import rotate_half_torch
    rms_norm = _function_from_source(os.path.join(ref_root, "models/FlashHiLS/modeling_olmo_hils.py"), "rms_norm")
    for tag, (B, L, H, D, shared, cs_fp32, dt) in {"a": (2, 40, 3, 64, True, False, torch.bfloat16),
                                                   "b": (1, 33, 2, 128, False, True, torch.bfloat16),
                                                   "c": (1, 20, 2, 64, True, True, torch.float32)}.items():
        g = torch.Generator().manual_seed(600 + ord(tag))
        x = torch.randn(B, L, H, D, generator=g).to(dt)
        w = (1.0 + 0.2 * torch.randn(D, generator=g)).to(dt)
        freqs = torch.randn(1 if shared else B, L, D // 2, generator=g)
        emb = torch.cat((freqs, freqs), dim=-1)
        cs_dt = torch.float32 if cs_fp32 else torch.bfloat16
        cos, sin = emb.cos().to(cs_dt), emb.sin().to(cs_dt)
        do = torch.randn(B, L, H, D, generator=g).to(dt)
        # fp32 leaves for the gradients, values representable in dt
        xl, wl = x.float().requires_grad_(True), w.float().requires_grad_(True)
        y = rms_norm(xl.to(dt), wl.to(dt), 1e-6)                                   # (B,L,H,D) in dt
        yr = y.transpose(1, 2).float()                                             # (B,H,L,D)
        out = ((yr * cos.float().unsqueeze(1)) + (rotate_half_torch(yr) * sin.float().unsqueeze(1))) \
            .transpose(1, 2).contiguous().to(dt)
        out_norm_only = y.detach().clone()
        rope_only = ((x.transpose(1, 2).float() * cos.float().unsqueeze(1))
                     + (rotate_half_torch(x.transpose(1, 2).float()) * sin.float().unsqueeze(1))) \
            .transpose(1, 2).contiguous().to(dt)
        out.backward(do)
        np.savez_compressed(os.path.join(HERE, f"normrope_{tag}.npz"), x=_np(x), w=_np(w), cos=_np(cos), sin=_np(sin),
                            do=_np(do), out=_np(out), out_norm_only=_np(out_norm_only), out_rope_only=_np(rope_only),
                            dx=_np(xl.grad), dw=_np(wl.grad),
                            args=np.array([int(dt == torch.bfloat16), int(cs_fp32)], dtype=np.int64))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/HiLS-Attention")
    main(sys.argv[1])
