"""The reference's own demo script (demo/llama3/demo.py) builds its Llama graph against this
package through `import yirage`, unchanged.  Runs only where the reference tree is mounted
(it is not on the GPU box); no GPU needed: tensors live on the CPU and compile() goes
through the host-only handle, so every builder call, shape check and the native graph
validation are exercised."""
import importlib.util
import json
import os
import sys
import types

import pytest
import torch

# where the reference tree is mounted: YIRAGE_REFERENCE_ROOT, else <parent of the repo>/reference
REF = os.environ.get("YIRAGE_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
DEMO = os.path.join(REF, "demo", "llama3", "demo.py")

pytestmark = pytest.mark.skipif(not os.path.exists(DEMO), reason="reference tree not mounted")


def fake_llama(hidden, inter, layers, hq, hkv, vocab, max_pages, page_size):
    """Object with the attributes the demo reads from Llama3ForCausalLM."""
    d = 128
    bf = dict(dtype=torch.bfloat16)
    lin = lambda o, i: types.SimpleNamespace(weight=torch.zeros(o, i, **bf))
    norm = lambda: types.SimpleNamespace(weight=torch.ones(hidden, **bf))
    layer_list = []
    for _ in range(layers):
        layer_list.append(types.SimpleNamespace(
            input_layernorm=norm(), post_attention_layernorm=norm(),
            self_attn=types.SimpleNamespace(q_proj=lin(hq * d, hidden), k_proj=lin(hkv * d, hidden),
                                            v_proj=lin(hkv * d, hidden), o_proj=lin(hidden, hq * d)),
            mlp=types.SimpleNamespace(gate_proj=lin(inter, hidden), up_proj=lin(inter, hidden),
                                      down_proj=lin(hidden, inter))))
    kv = tuple(torch.zeros(layers, max_pages, page_size, hkv, d, **bf) for _ in range(2))
    cfg = types.SimpleNamespace(hidden_size=hidden, intermediate_size=inter, vocab_size=vocab,
                                num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d)
    return types.SimpleNamespace(
        config=cfg, lm_head=lin(vocab, hidden),
        model=types.SimpleNamespace(layers=layer_list, kv_cache=kv, norm=norm(),
                                    embed_tokens=types.SimpleNamespace(weight=torch.zeros(vocab, hidden, **bf))))


def test_reference_demo_builds_its_graph_unchanged(monkeypatch, tmp_path, native_lib):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    monkeypatch.syspath_prepend(root)
    monkeypatch.syspath_prepend(os.path.join(REF, "demo", "llama3"))
    monkeypatch.chdir(tmp_path)
    spec = importlib.util.spec_from_file_location("ref_llama3_demo", DEMO)
    demo = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(demo)                    # the file itself, not a copy

    import yirage as yr
    from yirage_b200.persistent_kernel import PersistentKernel
    # the only stand-ins: no GPU here, so "cuda" allocations land on the CPU, the SM count
    # comes from a B200, and compile() validates on a host-only handle
    for fn in ("zeros", "empty", "full"):
        real = getattr(torch, fn)
        monkeypatch.setattr(torch, fn, (lambda real: lambda *a, **k: real(*a, **{**k, "device": "cpu"}))(real))
    monkeypatch.setattr(yr, "get_configurations_from_gpu", lambda rank: (128, 80))
    real_compile = PersistentKernel.compile
    monkeypatch.setattr(PersistentKernel, "compile", lambda self, **kw: real_compile(self, dry_run=True))

    args = types.SimpleNamespace(
        profiling=False, trace_name="", spec_decode=None, ngram_size=3, spec_length=3,
        max_seq_length=512, max_num_batched_requests=4, max_num_batched_tokens=8, page_size=4096,
        max_num_pages=16, use_cutlass_kernel=True, output_dir=None)           # the demo's defaults
    # Llama-3-8B widths (the demo's grid heuristics assume them), two layers
    model = fake_llama(4096, 14336, 2, 32, 8, 128256, args.max_num_pages, args.page_size)
    cos = torch.zeros(1, 32768, 128, dtype=torch.bfloat16)
    input_data = {
        "tokens": torch.zeros(4, 512, dtype=torch.long), "prompt_lengths": torch.full((4,), 20, dtype=torch.int),
        "position_embeddings": (cos, cos.clone()),
        "input_tokens": torch.zeros(8, 1, dtype=torch.long), "output_tokens": torch.zeros(8, 1, dtype=torch.long),
        "step": torch.zeros(4, dtype=torch.int32), "num_new_tokens": torch.ones(4, dtype=torch.int32)}
    ypk = demo.build_yirage_graph(model, args, world_size=1, rank=0, input_data=input_data,
                                  eos_token_id_for_yirage=128009)
    assert isinstance(ypk, PersistentKernel) and ypk._is_compiled
    kinds = [o.kind for o in ypk.lower().ops]
    assert kinds == ["embed"] + ["linear", "attention", "linear", "linear", "linear"] * 2 + \
        ["linear", "argmax_partial", "argmax_reduce"]
    # the files the demo writes from generate_task_graph()
    j = json.load(open(tmp_path / "task_graph_0.json"))
    assert len(j["all_tasks"]) == ypk.lower().num_tasks
    assert os.path.exists(tmp_path / "kernel_0.cu")
    ypk.finalize()
