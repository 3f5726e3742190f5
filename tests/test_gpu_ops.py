"""Parity of the task kernels against the CPU oracle, through the PersistentKernel surface
and the C ABI, one operator per graph.  Tolerance: max-abs 2e-2 + relative 1e-2 against
the fp32 oracle on the same bf16/fp16 inputs; ids and indices bit-exact."""
import pytest
import torch

import yirage_b200 as yr
from oracle import decode_oracle as O
from tests.util import assert_close, onepass_kernel, randn

pytestmark = pytest.mark.gpu


def run_linear(B, K, Nrows, *, norm=False, residual=False, dtype=torch.bfloat16, seed=0,
               eps=1e-6, max_tokens=8, tensor_core=None):
    x = randn((max_tokens, K), seed, 1.0, dtype)
    w = randn((Nrows, K), seed + 1, 0.02, dtype)
    nw = randn((K,), seed + 2, 0.1, dtype, mean=1.0)
    res = randn((max_tokens, Nrows), seed + 3, 1.0, dtype)
    ypk = onepass_kernel(max_tokens)
    ydt = yr.bfloat16 if dtype == torch.bfloat16 else yr.float16
    xt = ypk.attach_input(x, "x")
    wt = ypk.attach_input(w, "w")
    out = torch.zeros(max_tokens, Nrows, dtype=dtype, device="cuda")
    ot = ypk.attach_input(out, "out")
    src = xt
    grid = max(g for g in range(1, Nrows // 64 + 1) if Nrows % g == 0)
    if norm:
        nwt = ypk.attach_input(nw, "nw")
        tmp = ypk.new_tensor(dims=(max_tokens, K), dtype=ydt, name="normed")
        ypk.rmsnorm_layer(xt, nwt, tmp, (max_tokens, 1, 1), (128, 1, 1), eps=eps)
        src = tmp
    if residual:
        rt = ypk.attach_input(res, "res")
        ypk.linear_with_residual_layer(src, wt, rt, ot, (grid, 1, 1), (128, 1, 1))
    else:
        ypk.linear_layer(src, wt, ot, (grid, 1, 1), (128, 1, 1))
    ypk.compile()
    ypk(batch=B)
    torch.cuda.synchronize()
    if tensor_core is not None:
        ran = ypk.status().tensor_core_tasks
        assert (ran > 0) == tensor_core, f"tensor-core LINEAR tasks: {ran}"
    xin = x[:B].cpu()
    if norm:
        xin = O.rmsnorm(xin, nw.cpu(), eps)
    want = O.linear(xin, w.cpu(), res[:B].cpu() if residual else None)
    assert_close(out[:B], want, f"linear B={B} K={K} N={Nrows} norm={norm} res={residual}")
    assert torch.all(out[B:] == 0), "rows beyond the batch must stay untouched"
    ypk.finalize()


@pytest.mark.parametrize("B", [1, 2, 3, 5, 8])
def test_linear_plain(B):
    run_linear(B, 512, 320)


@pytest.mark.parametrize("B,K,N", [(1, 4096, 4096), (8, 4096, 4096), (4, 1792, 256), (1, 14336, 296)])
def test_linear_shapes(B, K, N):
    run_linear(B, K, N, seed=3)


def test_linear_rmsnorm_fused_cfg1_fp16():
    # BASELINE config 1: X [8,4096] fp16 ~N(0,1), norm weight ~N(1,0.1), eps 1e-6,
    # W [4096,4096] fp16 ~N(0,0.02)
    run_linear(8, 4096, 4096, norm=True, dtype=torch.float16, seed=0, eps=1e-6)


@pytest.mark.parametrize("B", [1, 8])
def test_linear_norm_residual(B):
    run_linear(B, 1024, 512, norm=True, residual=True, seed=5, eps=1e-5)


def test_linear_batch_above_eight_odd_k_blocks(monkeypatch):
    """K of five 64-column k-blocks, split along K unevenly: on the tensor cores and, with
    them switched off, as one pass of 16 tokens."""
    run_linear(11, 320, 192, max_tokens=16, seed=9, tensor_core=True)
    monkeypatch.setenv("YPK_TENSOR_CORE", "never")
    run_linear(11, 320, 192, max_tokens=16, seed=9, tensor_core=False)


@pytest.mark.parametrize("B,K,N,norm,res,dtype", [
    (9, 512, 192, False, False, torch.bfloat16),
    (16, 4096, 4096, True, False, torch.float16),
    (17, 1024, 520, True, True, torch.bfloat16),      # 16 + 1
    (40, 1792, 250, False, True, torch.bfloat16),     # 16 + 16 + 8, odd row slabs
    (64, 14336, 296, True, True, torch.bfloat16),     # 14 chunks of K
    (12, 64, 64, True, False, torch.bfloat16),        # K below one stage
])
def test_linear_sixteen_tokens_per_pass(B, K, N, norm, res, dtype, monkeypatch):
    """More than 8 tokens on the GEMV path: 16 per pass, K in chunks of a ring stage, running
    sums in registers."""
    monkeypatch.setenv("YPK_TENSOR_CORE", "never")
    run_linear(B, K, N, norm=norm, residual=res, dtype=dtype, seed=B, eps=1e-5, max_tokens=64,
               tensor_core=False)


@pytest.mark.parametrize("B,K,N,norm,res,dtype", [
    (9, 512, 192, False, False, torch.bfloat16),
    (11, 512, 200, True, False, torch.bfloat16),
    (16, 4096, 4096, True, False, torch.float16),
    (33, 1024, 520, True, True, torch.bfloat16),
    (48, 1792, 256, False, True, torch.bfloat16),
    (64, 4096, 1000, False, False, torch.bfloat16),
    (64, 14336, 296, True, True, torch.bfloat16),
])
def test_linear_tensor_core_path(B, K, N, norm, res, dtype, monkeypatch):
    """9..64 tokens: tcgen05.mma with TMEM accumulators, TMA-staged weights."""
    monkeypatch.setenv("YPK_TENSOR_CORE", "always")   # these slabs are too small to win on cost
    run_linear(B, K, N, norm=norm, residual=res, dtype=dtype, seed=B, eps=1e-5, max_tokens=64,
               tensor_core=True)


def test_linear_small_batches_in_a_large_batch_graph():
    """A graph of up to 64 tokens run with few: 3..8 tokens still take the tensor cores (its
    operators are cut for them), one or two tokens the GEMV passes."""
    run_linear(8, 512, 192, max_tokens=64, seed=4, tensor_core=True)
    run_linear(3, 1024, 520, max_tokens=64, seed=5, norm=True, residual=True, tensor_core=True)
    run_linear(2, 512, 192, max_tokens=64, seed=6, tensor_core=False)
    run_linear(1, 4096, 4096, max_tokens=64, seed=7, residual=True, tensor_core=False)


@pytest.mark.parametrize("B,H,I,tc", [(1, 512, 1024, "always"), (8, 4096, 1792, "always"),
                                      (3, 1024, 2048, "always"), (16, 1024, 2048, "always"),
                                      (40, 512, 1024, "always"), (64, 4096, 1792, "always"),
                                      (16, 1024, 2048, "never"), (33, 4096, 1792, "never"),
                                      # BASELINE config 2 at its stated size, batch 8 and 64,
                                      # both LINEAR paths for the 64-token case
                                      (8, 4096, 14336, "auto"), (64, 4096, 14336, "always"),
                                      (64, 4096, 14336, "never"), (16, 4096, 14336, "auto")])
def test_gated_mlp_fused(B, H, I, tc, monkeypatch):
    """rmsnorm -> linear(gate|up) -> silu_mul -> linear(down)+residual, the MLP half of a
    layer (BASELINE config 2, at reduced width and at its full 4096 x 14336); more than 8
    tokens can take the tcgen05 path."""
    MT = 8 if B <= 8 else 64
    monkeypatch.setenv("YPK_TENSOR_CORE", tc)
    x = randn((MT, H), 1)
    nw = randn((H,), 2, 0.1, mean=1.0)
    wg, wu = randn((I, H), 3, 0.02), randn((I, H), 4, 0.02)
    wd = randn((H, I), 5, 0.02)
    ypk = onepass_kernel(MT)
    xt, nwt = ypk.attach_input(x, "x"), ypk.attach_input(nw, "nw")
    wgt, wut, wdt = ypk.attach_input(wg, "wg"), ypk.attach_input(wu, "wu"), ypk.attach_input(wd, "wd")
    out = torch.zeros(MT, H, dtype=torch.bfloat16, device="cuda")
    ot = ypk.attach_input(out, "out")
    normed = ypk.new_tensor(dims=(MT, H), name="normed")
    mid = ypk.new_tensor(dims=(MT, 2 * I), name="mid")
    act = ypk.new_tensor(dims=(MT, I), name="act")
    groups = 8
    wgu = ypk.shuffle_tensors([wgt, wut], 0, groups, "wgu")
    ypk.rmsnorm_layer(xt, nwt, normed, (MT, 1, 1), (128, 1, 1), eps=1e-5)
    ypk.linear_layer(normed, wgu, mid, (2 * groups, 1, 1), (128, 1, 1))
    ypk.silu_mul_layer(mid, act, (groups, 1, 1), (128, 1, 1))
    ypk.linear_with_residual_layer(act, wdt, xt, ot, (H // 64, 1, 1), (128, 1, 1))
    ypk.compile()
    # gate/up + silu fuse; the norm folds into the projection in graphs of at most 8 tokens
    # and stays an operator of its own beyond (the tensor-core path takes its tokens by TMA)
    assert [o.kind for o in ypk.lower().ops] == (["linear", "linear"] if MT <= 8 else
                                                 ["rmsnorm", "linear", "linear"])
    ypk(batch=B)
    torch.cuda.synchronize()
    if tc != "auto":
        assert (ypk.status().tensor_core_tasks > 0) == (B > 8 and tc == "always")
    xc = x[:B].cpu()
    h = O.rmsnorm(xc, nw.cpu(), 1e-5)
    want = xc.float() + O.gated_mlp(h, wg.cpu(), wu.cpu(), wd.cpu())
    if I < 8192:
        assert_close(out[:B], want, f"gated mlp B={B}")
    else:
        # 14336-term dot products over an activation that was rounded to bf16 three times: the
        # reference's own bf16 pipeline (the oracle rounding every operator output) is itself
        # outside the tolerance against fp32 here; the device must be no further from fp32
        # than that pipeline is, give or take a quarter
        pipe = xc.float() + O.gated_mlp(O.rmsnorm(xc, nw.cpu(), 1e-5, "bf16"), wg.cpu(), wu.cpu(),
                                        wd.cpu(), rounding="bf16")
        _, _, ref_ratio = O.within_tolerance(pipe, want)
        _, max_abs, dev_ratio = O.within_tolerance(out[:B].float().cpu(), want)
        assert dev_ratio <= 1.25 * max(ref_ratio, 1.0), \
            f"gated mlp B={B}: {dev_ratio:.2f}x the tolerance from fp32 (max abs {max_abs:.4f}), " \
            f"the bf16 pipeline {ref_ratio:.2f}x"
    ypk.finalize()


def test_unfused_rmsnorm_and_silu_mul_tasks():
    """A norm whose output is read twice and a silu_mul on a plain tensor cannot fuse and run
    as their own tasks."""
    MT, H, groups = 4, 512, 4
    x = randn((MT, H), 11)
    nw = randn((H,), 12, 0.1, mean=1.0)
    ypk = onepass_kernel(MT)
    xt, nwt = ypk.attach_input(x, "x"), ypk.attach_input(nw, "nw")
    normed_t = torch.zeros(MT, H, dtype=torch.bfloat16, device="cuda")
    act_t = torch.zeros(MT, H // 2, dtype=torch.bfloat16, device="cuda")
    normed, act = ypk.attach_input(normed_t, "normed"), ypk.attach_input(act_t, "act")
    ypk.rmsnorm_layer(xt, nwt, normed, (MT, 1, 1), (128, 1, 1), eps=1e-6)
    ypk.silu_mul_layer(normed, act, (groups, 1, 1), (128, 1, 1))
    ypk.compile()
    ypk(batch=3)
    torch.cuda.synchronize()
    want_n = O.rmsnorm(x[:3].cpu(), nw.cpu(), 1e-6, "bf16")
    assert_close(normed_t[:3], want_n, "rmsnorm task")
    gs = H // 2 // groups
    v = normed_t[:3].cpu().float().view(3, groups, 2, gs)
    want_a = O.silu_mul(v[:, :, 0], v[:, :, 1], "bf16").reshape(3, -1)
    assert_close(act_t[:3], want_a, "silu_mul task")
    ypk.finalize()


def test_embedding_gather_is_bit_exact():
    MT, V, H = 8, 1000, 1024
    table = randn((V, H), 21, 0.02)
    ids = torch.tensor([[5], [999], [0], [-1], [17], [17], [3], [512]], dtype=torch.int64, device="cuda")
    out = torch.full((MT, H), 7.0, dtype=torch.bfloat16, device="cuda")
    ypk = onepass_kernel(MT)
    ypk.embed_layer(ypk.attach_input(ids, "ids"), ypk.attach_input(table, "table"),
                    ypk.attach_input(out, "out"), (1, 1, 1), (128, 1, 1), input_source=1)
    ypk.compile()
    ypk(batch=6)
    torch.cuda.synchronize()
    want = table[ids[:6, 0].clamp(min=0)].clone()
    want[3] = 0  # negative id -> zeros
    assert torch.equal(out[:6], want)
    assert torch.all(out[6:] == 7.0)
    ypk.finalize()


def test_argmax_is_bit_exact_with_planted_and_tied_maxima():
    MT, V, parts = 8, 4096, 128
    logits = randn((MT, V), 31)
    logits[0, 4095] = 100.0            # last column
    logits[1, 0] = 100.0               # first column
    logits[2, 77] = logits[2, 3000] = 50.0   # tie across chunks: lowest index wins
    logits[3, 1024] = logits[3, 1025] = 60.0  # tie inside a chunk
    logits[4] = -5.0                   # all equal
    pv = torch.zeros(MT, parts, dtype=torch.bfloat16, device="cuda")
    pi = torch.zeros(MT, parts, dtype=torch.int64, device="cuda")
    out = torch.full((MT, 1), -1, dtype=torch.int64, device="cuda")
    ypk = onepass_kernel(MT)
    lt, pvt, pit = ypk.attach_input(logits, "logits"), ypk.attach_input(pv, "pv"), ypk.attach_input(pi, "pi")
    ot = ypk.attach_input(out, "out")
    ypk.argmax_partial_layer(lt, (pvt, pit), (parts, 1, 1), (128, 1, 1))
    ypk.argmax_reduce_layer((pvt, pit), ot, (1, 1, 1), (128, 1, 1))
    ypk.compile()
    ypk(batch=MT)
    torch.cuda.synchronize()
    want = O.argmax_lowest(logits.cpu().float())
    assert out[:, 0].cpu().tolist() == want.tolist()
    assert want.tolist()[:5] == [4095, 0, 77, 1024, 0]
    ypk.finalize()


def test_kernel_graph_surface_rmsnorm_matmul_config1():
    """benchmark/rmsnorm.py through yirage.new_kernel_graph(): X [8,4096] fp16 ~N(0,1),
    W [4096,4096] fp16 ~N(0,0.02) stored [K,N]; rms_norm without weight or epsilon."""
    import yirage as yr_alias
    graph = yr_alias.new_kernel_graph()
    X = graph.new_input(dims=(8, 4096), dtype=yr_alias.float16)
    W = graph.new_input(dims=(4096, 4096), dtype=yr_alias.float16)
    graph.mark_output(graph.matmul(graph.rms_norm(X, normalized_shape=(4096,)), W))
    run = graph.superoptimize(config="mlp", backend="cuda", warmup_iters=1, profile_iters=1)
    x = randn((8, 4096), 0, 1.0, torch.float16)
    w = randn((4096, 4096), 1, 0.02, torch.float16)
    out = run(inputs=[x, w])[0]
    out2 = run(inputs=[x, w])[0]          # second call reuses the loaded graph
    torch.cuda.synchronize()
    want = O.linear(O.rmsnorm(x.cpu(), None, 0.0), w.cpu().t())
    assert_close(out, want, "kernel-graph rms_norm->matmul")
    assert out2.data_ptr() == out.data_ptr()


@pytest.mark.parametrize("B", [8, 64])
def test_kernel_graph_surface_gated_mlp_config2(B):
    """benchmark/gated_mlp.py: mul(silu(X.W1), X.W2) at reduced width, batch 8 and 64."""
    import yirage as yr_alias
    H, I = 1024, 1792
    graph = yr_alias.new_kernel_graph()
    X = graph.new_input(dims=(B, H), dtype=yr_alias.bfloat16)
    W1 = graph.new_input(dims=(H, I), dtype=yr_alias.bfloat16)
    W2 = graph.new_input(dims=(H, I), dtype=yr_alias.bfloat16)
    graph.mark_output(graph.mul(graph.silu(graph.matmul(X, W1)), graph.matmul(X, W2)))
    run = graph.superoptimize(config="mlp")
    x, w1, w2 = randn((B, H), 1), randn((H, I), 2, 0.02), randn((H, I), 3, 0.02)
    out = run(inputs=[x, w1, w2])[0]
    torch.cuda.synchronize()
    want = O.silu_mul(O.linear(x.cpu(), w1.cpu().t()), O.linear(x.cpu(), w2.cpu().t()))
    assert_close(out, want, f"kernel-graph gated mlp B={B}")


def test_embedding_id_beyond_the_table_gives_zeros():
    """A sampled id can lie in the zero-padded tail of the lm_head, past the last row of the
    embedding table: the gather must not read there."""
    MT, V, H = 8, 1000, 1024
    table = randn((V, H), 21, 0.02)
    ids = torch.tensor([[999], [1000], [1 << 40], [0], [5000], [7], [0], [0]], dtype=torch.int64, device="cuda")
    out = torch.full((MT, H), 7.0, dtype=torch.bfloat16, device="cuda")
    ypk = onepass_kernel(MT)
    ypk.embed_layer(ypk.attach_input(ids, "ids"), ypk.attach_input(table, "table"),
                    ypk.attach_input(out, "out"), (1, 1, 1), (128, 1, 1), input_source=1)
    ypk.compile()
    ypk(batch=6)
    torch.cuda.synchronize()
    want = torch.zeros(6, H, dtype=torch.bfloat16, device="cuda")
    for b, i in enumerate([999, None, None, 0, None, 7]):
        if i is not None:
            want[b] = table[i]
    assert torch.equal(out[:6], want)
    ypk.finalize()


def test_argmax_ignores_the_padded_vocabulary_tail():
    """All real logits negative, the padded columns hold 0.0 (zero rows of the lm_head): the
    sampled id must be the arg-max over the real vocabulary (torch.argmax on the unpadded
    columns), not a padded column."""
    MT, V, VPAD, parts = 8, 3000, 4096, 128
    logits = -(randn((MT, VPAD), 41).abs()) - 0.5
    logits[:, V:] = 0.0
    logits[5, V - 1] = -0.01           # the last real column wins in one row
    pv = torch.zeros(MT, parts, dtype=torch.bfloat16, device="cuda")
    pi = torch.zeros(MT, parts, dtype=torch.int64, device="cuda")
    out = torch.full((MT, 1), -1, dtype=torch.int64, device="cuda")
    ypk = onepass_kernel(MT)
    lt, pvt, pit = ypk.attach_input(logits, "logits"), ypk.attach_input(pv, "pv"), ypk.attach_input(pi, "pi")
    ypk.argmax_partial_layer(lt, (pvt, pit), (parts, 1, 1), (128, 1, 1), valid_cols=V)
    ypk.argmax_reduce_layer((pvt, pit), ypk.attach_input(out, "out"), (1, 1, 1), (128, 1, 1))
    ypk.compile()
    ypk(batch=MT)
    torch.cuda.synchronize()
    want = torch.argmax(logits[:, :V].float().cpu(), dim=-1)
    assert out[:, 0].cpu().tolist() == want.tolist()
    assert int(out[5, 0]) == V - 1 and int(out.max()) < V
    ypk.finalize()


def test_argmax_planted_maximum_as_the_reference_test_does():
    """tests/runtime_python/test_argmax.py of the reference: 6 rows of 153600 bf16 logits, 96
    chunks, the largest bf16 planted at a known column per row; the ids must match exactly."""
    rows, V, parts = 6, 153600, 96
    logits = randn((8, V), 51)
    g = torch.Generator().manual_seed(51)
    planted = torch.randint(0, V, (rows,), generator=g).tolist()
    for r, c in enumerate(planted):
        logits[r, c] = 65504.0
    pv = torch.zeros(8, parts, dtype=torch.bfloat16, device="cuda")
    pi = torch.zeros(8, parts, dtype=torch.int64, device="cuda")
    out = torch.full((8, 1), -1, dtype=torch.int64, device="cuda")
    ypk = onepass_kernel(8)
    ypk.argmax_partial_layer(ypk.attach_input(logits, "logits"),
                             (ypk.attach_input(pv, "pv"), ypk.attach_input(pi, "pi")), (parts, 1, 1), (128, 1, 1))
    ypk.argmax_reduce_layer((ypk.kn_graph.cygraph.tensors[1], ypk.kn_graph.cygraph.tensors[2]),
                            ypk.attach_input(out, "out"), (1, 1, 1), (128, 1, 1))
    ypk.compile()
    ypk(batch=rows)
    torch.cuda.synchronize()
    assert out[:rows, 0].cpu().tolist() == planted
    ypk.finalize()
