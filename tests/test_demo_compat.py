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


QWEN_DEMO = os.path.join(REF, "demo", "qwen3", "demo.py")


class _Built(Exception):
    """Raised by the patched compile(): the script has built its graph; what follows needs a GPU."""
    def __init__(self, ypk):
        self.ypk = ypk


def fake_qwen3(hidden, inter, layers, hq, hkv, vocab, max_pages, page_size):
    m = fake_llama(hidden, inter, layers, hq, hkv, vocab, max_pages, page_size)
    for layer in m.model.layers:
        layer.self_attn.q_norm = types.SimpleNamespace(weight=torch.ones(128, dtype=torch.bfloat16))
        layer.self_attn.k_norm = types.SimpleNamespace(weight=torch.ones(128, dtype=torch.bfloat16))
    m.config.eos_token_id = 151645
    m.device = "cpu"
    m.to = lambda *_a, **_k: m
    cos = torch.zeros(1, 32768, 128, dtype=torch.bfloat16)
    m.model.rotary_emb = lambda positions: (cos, cos.clone())
    return m


@pytest.mark.skipif(not os.path.exists(QWEN_DEMO), reason="reference tree not mounted")
@pytest.mark.parametrize("spec", [None, "promptlookup"])
def test_reference_qwen3_demo_builds_its_graph_unchanged(monkeypatch, tmp_path, native_lib, spec):
    """demo/qwen3/demo.py is a flat script: it is run as __main__, unchanged, with stand-ins for
    what is not on this machine (the Hugging Face model and tokenizer, a GPU).  It builds the
    dense Qwen3 graph (q/k norm inside attention) and, with --spec-decode promptlookup, the
    draft and verification operators through the reference's own dispatcher calls."""
    import runpy
    import transformers
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    monkeypatch.syspath_prepend(root)
    monkeypatch.chdir(tmp_path)
    model = fake_qwen3(4096, 12288, 2, 32, 8, 151936, 16, 4096)
    models = types.ModuleType("models")
    mq = types.ModuleType("models.modeling_qwen3")
    mq.Qwen3ForCausalLM = types.SimpleNamespace(from_pretrained=lambda *a, **k: model)
    models.modeling_qwen3 = mq
    monkeypatch.setitem(sys.modules, "models", models)
    monkeypatch.setitem(sys.modules, "models.modeling_qwen3", mq)

    class Tok:
        def apply_chat_template(self, messages, **kw):
            return "prompt"
        def __call__(self, texts, **kw):
            enc = types.SimpleNamespace(input_ids=torch.arange(3, 24).unsqueeze(0))
            enc.to = lambda *_a, **_k: enc
            return enc
    monkeypatch.setattr(transformers, "AutoTokenizer", types.SimpleNamespace(from_pretrained=lambda *a, **k: Tok()))

    import yirage as yr
    from yirage_b200.persistent_kernel import PersistentKernel
    for fn in ("zeros", "empty", "full"):
        real = getattr(torch, fn)
        monkeypatch.setattr(torch, fn, (lambda real: lambda *a, **k: real(*a, **{**k, "device": "cpu"}))(real))
    monkeypatch.setattr(torch.cuda, "set_device", lambda *_a, **_k: None)
    monkeypatch.setattr(torch.cuda, "Event", lambda *_a, **_k: types.SimpleNamespace())
    monkeypatch.setattr(yr, "get_configurations_from_gpu", lambda rank: (128, 80))
    real_compile = PersistentKernel.compile

    def compile_and_stop(self, **kw):
        real_compile(self, dry_run=True)
        raise _Built(self)
    monkeypatch.setattr(PersistentKernel, "compile", compile_and_stop)
    argv = [QWEN_DEMO, "--use-yirage", "--max-num-batched-requests", "2"]
    if spec:
        # the script's grids for the spec_length + 1 tokens of its request assume that many slots
        argv = [QWEN_DEMO, "--use-yirage", "--max-num-batched-requests", "1", "--max-num-batched-tokens", "6",
                "--spec-decode", spec, "--ngram-size", "3", "--spec-length", "5"]
    monkeypatch.setattr(sys, "argv", argv)
    try:
        with pytest.raises(_Built) as built:
            runpy.run_path(QWEN_DEMO, run_name="__main__")          # the file itself
    finally:
        torch.set_default_dtype(torch.float32)                  # the script switches it to bf16
    ypk = built.value.ypk
    assert ypk._is_compiled
    g = ypk.lower()
    kinds = [o.kind for o in g.ops]
    layer = ["linear", "attention", "linear", "linear", "linear"]
    head = ["ngram_partial", "ngram_global", "embed"] if spec else ["embed"]
    tail = ["linear", "argmax_partial", "argmax_reduce"] + (["verify"] if spec else [])
    assert kinds == head + layer * 2 + tail
    from yirage_b200 import _native as N
    att = [t for t in g.tasks if t.type == N.TASK_ATTENTION]
    assert att and all(t.flags & N.F_QK_NORM for t in att)
    assert os.path.exists(tmp_path / "task_graph_0.json")
    ypk.finalize()
