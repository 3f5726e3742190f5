"""Generates tests/golden/*.pt by running the REFERENCE's own PyTorch model code on seeded
inputs (CPU).  Run in a container that has the reference tree:

    python tests/golden/make_golden.py /root/reference

Only the reference classes/functions are executed here; nothing from this repository's
oracle is involved, so the fixtures pin the oracle from outside.  Shapes are reduced
versions of the BASELINE.json configs (same distributions and seeds) to keep the files
small.
"""
import os
import sys

import torch

OUT = os.path.dirname(os.path.abspath(__file__))


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
    print("golden fixtures written to", OUT)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
