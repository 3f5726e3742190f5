"""Generates tests/golden/*.pt by running the REFERENCE's own PyTorch code on seeded inputs
(CPU).  Run in a container that has the reference tree:

    python tests/golden/make_golden.py <reference root>      (or YIRAGE_REFERENCE_ROOT=...)

Only the reference classes/functions are executed here; nothing from this repository's
oracle is involved, so the fixtures pin the oracle from outside.  Two sources:

  * demo/llama3/models/modeling_llama3.py is imported as a module (RMSNorm, MLP, rotary
    tables, naive attention);
  * the torch restatements the reference's own kernel tests compare against
    (tests/runtime_python/test_paged_attention.py: rotate_half, apply_rotary_pos_emb, rmsnorm,
    torch_paged_attention; test_multitoken_paged_attention.py:
    torch_multitoken_paged_attention; test_decoding_w_norm.py: attention_decode).  Those
    scripts import a pybind extension and allocate on "cuda" at import, so the function
    definitions are taken out of the files (ast) and run on CPU; the module-level constants
    they read (page_size, head_dim, qo_heads, ...) are set as in the scripts.

Shapes are reduced versions of the BASELINE.json configs (same distributions and seeds) to
keep the files small.
"""
import ast
import contextlib
import io
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

OUT = os.path.dirname(os.path.abspath(__file__))


def load_defs(path, names, **consts):
    """The named top-level function definitions of a reference test script, compiled from the
    file itself into a namespace holding the script's module-level constants."""
    with open(path) as f:
        tree = ast.parse(f.read(), filename=path)
    ns = {"torch": torch, "np": np, "F": F}
    ns.update(consts)
    found = set()
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            exec(compile(ast.Module(body=[node], type_ignores=[]), path, "exec"), ns)
            found.add(node.name)
    missing = set(names) - found
    if missing:
        raise RuntimeError(f"{path}: no definition of {sorted(missing)}")
    return ns


def kernel_test_fixtures(ref_root):
    tdir = os.path.join(ref_root, "tests", "runtime_python")
    QO, KV, D, PS, MP = 4, 1, 128, 64, 16
    bf = torch.bfloat16
    consts = dict(qo_heads=QO, kv_heads=KV, head_dim=D, page_size=PS, max_num_pages=MP,
                  device="cpu", dtype=bf)
    pa = load_defs(os.path.join(tdir, "test_paged_attention.py"),
                   ["rotate_half", "apply_rotary_pos_emb", "rmsnorm", "torch_paged_attention"], **consts)
    mt = load_defs(os.path.join(tdir, "test_multitoken_paged_attention.py"),
                   ["rotate_half", "apply_rotary_pos_emb", "rmsnorm",
                    "torch_multitoken_paged_attention"], prompt_len=0, max_tokens=4, **consts)

    # --- rotate-half RoPE application (test_paged_attention.py:18-34).  Random cos/sin whose
    #     two halves differ (as the reference test draws them) pin which table entry each
    #     output element uses; the real Llama-3 tables are covered by rope_tables.pt.
    g = torch.Generator().manual_seed(11)
    T = 6
    q = torch.randn(T, 8, D, generator=g).to(bf)
    k = torch.randn(T, 2, D, generator=g).to(bf)
    cos = torch.randn(T, D, generator=g).to(bf)
    sin = torch.randn(T, D, generator=g).to(bf)
    qe, ke = pa["apply_rotary_pos_emb"](q, k, cos, sin, unsqueeze_dim=1)
    torch.save({"q": q, "k": k, "cos": cos, "sin": sin, "q_out": qe, "k_out": ke},
               os.path.join(OUT, "rope_apply.pt"))

    # --- one-token paged attention (test_paged_attention.py:48-94): page-boundary lengths,
    #     a last page exactly full, a seeded page permutation; with and without q/k RMSNorm
    g = torch.Generator().manual_seed(12)
    cases = []
    perm = torch.randperm(MP, generator=g).to(torch.int32)
    all_cos = torch.randn(1100, D, generator=g).to(bf)
    all_sin = torch.randn(1100, D, generator=g).to(bf)
    for seq_len, qk_norm in [(1, False), (63, False), (64, False), (65, False), (128, False),
                             (200, False), (513, False), (64, True), (65, True), (200, True)]:
        kc = torch.randn(MP, PS, KV * D, generator=g).to(bf)
        vc = torch.randn(MP, PS, KV * D, generator=g).to(bf)
        qkv = torch.randn(QO + 2 * KV, D, generator=g).to(bf)
        page, off = int(perm[(seq_len - 1) // PS]), (seq_len - 1) % PS
        kc[page, off] = qkv[QO]
        vc[page, off] = qkv[QO + 1]
        qw = (torch.randn(1, D, generator=g) * 0.2 + 1.0).to(bf)
        kw = (torch.randn(1, D, generator=g) * 0.2 + 1.0).to(bf)
        k_after = kc.clone()
        out = pa["torch_paged_attention"](qkv[:QO].unsqueeze(1), k_after, vc.clone(), perm, seq_len,
                                          qk_norm, True, qw, kw, all_cos[seq_len].unsqueeze(0),
                                          all_sin[seq_len].unsqueeze(0), 1e-5)
        # the fixture keeps the request's rows only (position order); the test scatters them
        # back into pages `perm`
        rows = [(int(perm[p // PS]), p % PS) for p in range(seq_len)]
        kflat = torch.stack([kc[a, b] for a, b in rows])
        vflat = torch.stack([vc[a, b] for a, b in rows])
        cases.append({"seq_len": seq_len, "qk_norm": qk_norm, "qkv": qkv, "k_rows": kflat, "v_rows": vflat,
                      "q_norm_w": qw, "k_norm_w": kw, "eps": 1e-5, "cos_row": all_cos[seq_len].clone(),
                      "sin_row": all_sin[seq_len].clone(),
                      "k_new_after": k_after[page, off].clone(), "out": out.squeeze(1).clone()})
    torch.save({"pages": perm, "page_size": PS, "cases": cases},
               os.path.join(OUT, "paged_attention_decode.pt"))

    # --- several new tokens of one request (test_multitoken_paged_attention.py:51-122):
    #     in-place K update in the page and the causal window among the new tokens.  The
    #     reference function writes the new K into the last page only, so the cases keep the
    #     new tokens inside it.
    g = torch.Generator().manual_seed(13)
    cases = []
    for cached, ntok, qk_norm in [(8, 4, False), (0, 5, False), (60, 4, False), (64, 8, False),
                                  (130, 3, False), (8, 4, True), (70, 8, True)]:
        seq_len = cached + ntok
        npages = (seq_len + PS - 1) // PS
        perm = torch.randperm(MP, generator=g).to(torch.int32)
        kc = torch.randn(MP, PS, KV * D, generator=g).to(bf)
        vc = torch.randn(MP, PS, KV * D, generator=g).to(bf)
        qkv = torch.randn(ntok, (QO + 2 * KV) * D, generator=g).to(bf)
        for t in range(ntok):
            p = cached + t
            kc[int(perm[p // PS]), p % PS] = qkv[t, QO * D:(QO + 1) * D]
            vc[int(perm[p // PS]), p % PS] = qkv[t, (QO + 1) * D:]
        cos = torch.randn(seq_len + 1, D, generator=g).to(bf)
        sin = torch.randn(seq_len + 1, D, generator=g).to(bf)
        qw = (torch.randn(1, D, generator=g) * 0.2 + 1.0).to(bf)
        kw = (torch.randn(1, D, generator=g) * 0.2 + 1.0).to(bf)
        last_len = (seq_len - 1) % PS + 1
        assert last_len >= ntok
        mt["prompt_len"] = cached          # the script's mask reads this module constant
        k_after = kc.clone()
        with contextlib.redirect_stdout(io.StringIO()):
            out = mt["torch_multitoken_paged_attention"](
                qkv[:, :QO * D].reshape(ntok, QO, D), k_after, vc.clone(),
                torch.tensor([0, npages], dtype=torch.int32), perm,
                torch.tensor([last_len], dtype=torch.int32), 0, ntok, qk_norm, True, qw, kw,
                cos, sin, eps=1e-5)
        rows = [(int(perm[p // PS]), p % PS) for p in range(seq_len)]
        cases.append({"cached": cached, "num_tokens": ntok, "qk_norm": qk_norm, "qkv": qkv,
                      "pages": perm[:npages].clone(),
                      "k_rows": torch.stack([kc[a, b] for a, b in rows]),
                      "v_rows": torch.stack([vc[a, b] for a, b in rows]), "cos": cos, "sin": sin,
                      "q_norm_w": qw, "k_norm_w": kw, "eps": 1e-5,
                      "k_rows_after": torch.stack([k_after[a, b] for a, b in rows]),
                      "out": out.reshape(ntok, QO, D).clone()})
    torch.save({"page_size": PS, "cases": cases}, os.path.join(OUT, "paged_attention_multitoken.pt"))

    # --- decode attention with q/k RMSNorm over a contiguous cache
    #     (test_decoding_w_norm.py:38-72: rmsnorm, attention_decode)
    dn = load_defs(os.path.join(tdir, "test_decoding_w_norm.py"),
                   ["rotate_half", "apply_rotary_pos_emb", "rmsnorm", "attention_decode"],
                   q_heads=4, k_heads=1, v_heads=1, head_dim=D, device="cpu", dtype=bf)
    g = torch.Generator().manual_seed(14)
    cases = []
    for valid in (1, 17, 64, 130):
        kc = torch.randn(1, valid, D, generator=g).to(bf)
        vc = torch.randn(1, valid, D, generator=g).to(bf)
        q = torch.randn(4, 1, D, generator=g).to(bf)
        qw = (torch.randn(1, D, generator=g) * 0.2 + 1.0).to(bf)
        kw = (torch.randn(1, D, generator=g) * 0.2 + 1.0).to(bf)
        cos = torch.randn(1, D, generator=g).to(bf)
        sin = torch.randn(1, D, generator=g).to(bf)
        k_after = kc.clone()
        out = dn["attention_decode"](q, k_after, vc, valid, qw, kw, 1e-5, cos, sin)
        cases.append({"valid_len": valid, "q": q[:, 0].clone(), "k_cache": kc[0].clone(),
                      "v_cache": vc[0].clone(), "q_norm_w": qw, "k_norm_w": kw, "eps": 1e-5,
                      "cos": cos[0].clone(), "sin": sin[0].clone(),
                      "k_new_after": k_after[0, valid - 1].clone(), "out": out.reshape(4, D).clone()})
    torch.save({"cases": cases}, os.path.join(OUT, "decode_attention_qknorm.pt"))


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "demo", "llama3"))
    from models.configuration_llama3 import Llama3Config
    from models.modeling_llama3 import (Llama3MLP, Llama3RMSNorm, Llama3RotaryEmbedding,
                                        naive_attention)

    # --- RMSNorm (modeling_llama3.py:38-52), config-1 distribution, bf16 like the model
    g = torch.Generator().manual_seed(0)
    x = torch.randn(8, 4096, generator=g).to(torch.bfloat16)
    w = (torch.randn(4096, generator=g) * 0.1 + 1.0).to(torch.bfloat16)
    for eps, tag in ((1e-6, "eps1e-6"), (1e-5, "eps1e-5")):
        norm = Llama3RMSNorm(4096, eps=eps).to(torch.bfloat16)
        with torch.no_grad():
            norm.weight.copy_(w)
            y = norm(x)
        torch.save({"x": x, "w": w, "eps": eps, "y": y}, os.path.join(OUT, f"rmsnorm_{tag}.pt"))

    # --- gated MLP (modeling_llama3.py:91-111), config-2 distribution at reduced width
    g = torch.Generator().manual_seed(1)
    cfg = Llama3Config(hidden_size=256, intermediate_size=448, num_hidden_layers=1,
                       num_attention_heads=2, num_key_value_heads=1)
    mlp = Llama3MLP(cfg, world_size=1).to(torch.bfloat16)
    with torch.no_grad():
        for p in (mlp.gate_proj.weight, mlp.up_proj.weight, mlp.down_proj.weight):
            p.copy_((torch.randn(p.shape, generator=g) * 0.02).to(torch.bfloat16))
        xm = torch.randn(8, 256, generator=g).to(torch.bfloat16)
        ym = mlp(torch.nn.Identity(), xm)
    torch.save({"x": xm, "gate": mlp.gate_proj.weight.detach().clone(),
                "up": mlp.up_proj.weight.detach().clone(),
                "down": mlp.down_proj.weight.detach().clone(), "y": ym},
               os.path.join(OUT, "gated_mlp.pt"))

    # --- rotary tables (modeling_llama3.py:54-89): Llama-3 theta, head_dim 128
    #     The class cannot be constructed with the transformers release installed here (its
    #     __init__ looks up ROPE_INIT_FUNCTIONS["default"], which that release no longer has),
    #     so the instance is made without __init__ and given the inverse frequencies of the
    #     default rope init of transformers (1 / theta^(arange(0, d, 2) / d)); the table
    #     construction itself (forward, :71-89) is the reference's code.
    cfg8 = Llama3Config()
    rot = Llama3RotaryEmbedding.__new__(Llama3RotaryEmbedding)
    torch.nn.Module.__init__(rot)
    d = cfg8.head_dim if getattr(cfg8, "head_dim", None) else cfg8.hidden_size // cfg8.num_attention_heads
    rot.inv_freq = 1.0 / (cfg8.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
    rot.attention_scaling = 1.0
    pos = torch.arange(4160)[None, :]
    cos, sin = rot(pos)
    torch.save({"theta": cfg8.rope_theta, "head_dim": d,
                "positions": torch.tensor([0, 1, 63, 64, 511, 4096, 4159]),
                "cos": cos[0, [0, 1, 63, 64, 511, 4096, 4159]].clone(),
                "sin": sin[0, [0, 1, 63, 64, 511, 4096, 4159]].clone()},
               os.path.join(OUT, "rope_tables.pt"))

    # --- decode attention (modeling_llama3.py:114-135): config-3 layout (32 q / 8 kv heads,
    #     head_dim 128) at context 200; one query token, non-causal over the whole cache
    g = torch.Generator().manual_seed(2)
    ctx = 200
    kc = torch.randn(1, 1, ctx, 8, 128, generator=g).to(torch.bfloat16)
    vc = torch.randn(1, 1, ctx, 8, 128, generator=g).to(torch.bfloat16)
    q = torch.randn(1, 32, 128, generator=g).to(torch.bfloat16)
    with torch.no_grad():
        o = naive_attention(q, kc, vc, ctx, 0, False, True)
    torch.save({"q": q, "k": kc[0, 0].clone(), "v": vc[0, 0].clone(), "out": o},
               os.path.join(OUT, "decode_attention.pt"))
    #     and a 5-token causal prefill chunk (is_causal=True path, :227-236)
    q5 = torch.randn(5, 32, 128, generator=g).to(torch.bfloat16)
    with torch.no_grad():
        o5 = naive_attention(q5, kc, vc, 5, 0, True, True)
    torch.save({"q": q5, "k": kc[0, 0, :5].clone(), "v": vc[0, 0, :5].clone(), "out": o5},
               os.path.join(OUT, "prefill_attention.pt"))
    kernel_test_fixtures(ref_root)
    print("golden fixtures written to", OUT)


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("YIRAGE_REFERENCE_ROOT")
    if not root:
        raise SystemExit("usage: make_golden.py <reference root>  (or set YIRAGE_REFERENCE_ROOT)")
    main(root)
