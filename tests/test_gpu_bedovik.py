"""Bedovik on CUDA: the sm_100a kernels (generic latent attention, the tcgen05 multi-query kernels on the latent cache,
router, gathered and dense experts, Dynamic Tanh, CUDA-core GEMM) against the plain float64 oracle.

float32 runs everything in true 32-bit (tight tolerance); bfloat16 is what serving uses (tolerance of 16-bit rounding).
"""
import pytest
import torch

import bedovik_oracle as oracle
import test_bedovik_cpu as cases
from llmss_b200 import ops
from llmss_b200.utils.checkpoint import bedovik_config

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16
MODES = [pytest.param(F32, 3e-4, id="f32"), pytest.param(BF16, 8e-2, id="bf16")]

# ranks the tcgen05 multi-query kernels take (64 / 128 / 256) with few, odd and many heads, beside ranks only the generic
# kernel takes; experts with enough tokens for the dense form
cases.CONFIGS["tc_ranks"] = bedovik_config(128, 211, 320, [cases.L(True, 1, 16, 16, 64, 8, 2, 2, 1, 32), cases.L(False, 5, 16, 24, 128, 8, 3, 4, 2, 32),
                                                           cases.L(True, 8, 32, 16, 256), cases.L(False, 2, 8, 8, 48, 4, 2, 1, 1, 16)], loop=(1, 3, 2))
cases.CONFIGS["odd_sizes"] = bedovik_config(72, 83, 320, [cases.L(True, 3, 6, 10, 18, 6, 2, 3, 2, 9), cases.L(False, 7, 4, 5, 33, 5, 5, 1, 1, 7)], loop=(0, 1, 2))


def test_loaded_library_is_the_in_tree_one():
    from llmss_b200.ops import _lib

    _lib.load()
    assert _lib.LOADED_FROM.endswith("llmss_b200/_C/libllmss_b200.so")


@pytest.mark.parametrize("dtype,tol", MODES)
def test_mechanisms(dtype, tol):
    cases.test_experts_op("cuda", dtype, max(tol, 1e-5) if dtype == F32 else 3e-2)
    for E, top, groups, keep in [(8, 3, 4, 2), (6, 2, 3, 3), (4, 1, 1, 1), (12, 4, 3, 2), (5, 5, 1, 1), (64, 6, 8, 3), (96, 8, 4, 1), (256, 8, 8, 4)]:
        cases.test_router_op(E, top, groups, keep, "cuda")
    torch.manual_seed(0)
    r, a, b = (torch.randn(9, 40, device="cuda") for _ in range(3))
    w, bias, s1, s2 = (torch.randn(40, device="cuda").to(dtype) for _ in range(4))
    y, r2 = ops.dyt_residual(r, 0.6, w, bias, a, s1, b, s2, out_dtype=dtype)
    want_r = r.double() + s1.double() * a.double() + s2.double() * b.double()
    cases.close(r2, want_r.cpu(), 1e-5)
    cases.close(y, oracle.dyt(want_r, 0.6, w.double(), bias.double()).cpu(), 1e-5 if dtype == F32 else 2e-2)


@pytest.mark.parametrize("dtype,tol", MODES)
@pytest.mark.parametrize("sizes", [(40, 3, 8, 12, 24), (64, 5, 16, 8, 64), (64, 2, 32, 32, 128), (96, 9, 8, 16, 256), (64, 20, 8, 8, 300),
                                   (64, 16, 8, 8, 128), (64, 32, 8, 8, 64), (64, 32, 8, 8, 128), (64, 7, 8, 8, 128), (64, 12, 8, 8, 256),
                                   (64, 8, 8, 8, 256), (64, 64, 8, 8, 64)])
def test_latent_attention_kernels(dtype, tol, sizes):
    many_heads = sizes[1] >= 12      # the oracle loops over heads in Python: fewer cuttings there
    for chunks in (([5, 2, 17, 1, 1, 9, 2, 40],) if many_heads else ([77], [1] * 40, [5, 2, 17, 1, 1, 9, 2, 40], [64, 64, 3])):
        for gated in ((True,) if many_heads else (True, False)):
            cases.test_latent_attention_ops(gated, chunks, "cuda", dtype, tol, sizes)


@pytest.mark.parametrize("dtype,tol", [pytest.param(F32, 1e-3, id="f32"), pytest.param(BF16, 3e-2, id="bf16")])
@pytest.mark.parametrize("R,bs", [(24, 16), (64, 64), (128, 64), (256, 16), (40, 64)])
def test_far_keys_and_page_borders(dtype, tol, R, bs):
    for far in (0, 3, 15, 16, 63, 64, 65, 127, 128, 255, 256, 320, 398, 399):
        for q_len in (1, 2, 9):
            cases.test_one_key_stands_out(far, q_len, "cuda", dtype, R, bs, tol)
    # a context long enough for the decode kernels to split the key range and merge the partial softmaxes
    for far in (0, 255, 256, 257, 511, 512, 700, 1023, 1024, 1099):
        for q_len in (1, 5):
            cases.test_one_key_stands_out(far, q_len, "cuda", dtype, R, bs, tol, ctx=1100)
    cases.test_window_edges_of_causality("cuda", dtype, 2e-3 if dtype == F32 else 3e-2)


@pytest.mark.parametrize("dtype,tol", MODES)
@pytest.mark.parametrize("name", ["mid_loop", "no_loop", "all_loop", "one_pass", "tc_ranks", "odd_sizes"])
def test_model_whole_prompt(tmp_path, dtype, tol, name):
    cases.test_whole_prompt_and_residual_stream(tmp_path, name, "cuda", dtype, tol)


@pytest.mark.parametrize("dtype,tol", MODES)
def test_model_schedules(tmp_path, dtype, tol):
    cases.test_decode_token_by_token_and_portions(tmp_path / "a", "cuda", dtype, tol)
    cases.test_first_tokens(tmp_path / "b", "cuda", dtype, tol)
    cases.test_unequal_batch_equals_each_alone(tmp_path / "c", "cuda", dtype, tol)
    cases.test_pages_and_slots_are_reused(tmp_path / "d", "cuda", dtype, tol)
    cases.test_long_decode(tmp_path / "e", "cuda", dtype, tol)


@pytest.mark.parametrize("dtype,tol", MODES)
def test_tensor_core_paths_through_the_engine(tmp_path, dtype, tol):
    """Ranks 64 / 128 / 256 on 64-token pages: decode, portions over context and mixed batches run on the tcgen05 kernels in
    16-bit; long portions take the dense expert form (threshold lowered so that this small case reaches it)."""
    from llmss_b200.models import blocks

    old, blocks._DENSE_MIN = blocks._DENSE_MIN, 48
    old_g, blocks._GROUPED_ROWS = blocks._GROUPED_ROWS, 16      # portions of 64 tokens and more: grouped experts
    old_f, blocks._FORCE_GROUPED = blocks._FORCE_GROUPED, True
    try:
        cfg, W, eng = cases.build(tmp_path, "tc_ranks", "cuda", dtype)
        assert eng.runner.block_size == 64
        toks = cases.tokens_for(cfg, 150, 7)
        want, _ = oracle.forward(cfg, W, toks)
        few = 0.03 if dtype == BF16 else 0.0     # share of positions a flipped near-tie of the router may move
        for sizes in ([150], [100, 1], [2, 62, 1, 63, 3, 2, 17], [64, 64, 22], [1]):
            cases.close(cases.feed_in_portions(eng, tuple(sizes), toks, sizes), want, tol, few)
        other = cases.tokens_for(cfg, 90, 8)
        o1 = eng.feed([("p", toks[:70], list(range(70))), ("q", other[:60], list(range(60)))], [])
        o2 = eng.feed([("p", toks[70:71], [0]), ("q", other[60:], list(range(30)))], ["p", "q"])
        cases.close(torch.cat([o1[:70], o2[:1]]), want[:71], tol, few)
        cases.close(torch.cat([o1[70:], o2[1:]]), oracle.forward(cfg, W, other)[0], tol, few)
    finally:
        blocks._DENSE_MIN, blocks._GROUPED_ROWS, blocks._FORCE_GROUPED = old, old_g, old_f


@pytest.mark.parametrize("dtype,tol", [pytest.param(BF16, 3e-2, id="bf16"), pytest.param(torch.float16, 1e-2, id="f16")])
def test_expert_forms_agree(dtype, tol):
    """The three execution forms of the routed experts (per-token gather, dense with zero weights, grouped by expert) against
    the oracle on the same inputs."""
    from llmss_b200.models import blocks

    torch.manual_seed(0)
    T, W, F, E, top = 300, 64, 32, 8, 2
    ups = [(torch.randn(F, W) * W ** -0.5).to(dtype) for _ in range(E)]
    downs = [(torch.randn(W, F) * F ** -0.5).to(dtype) for _ in range(E)]
    ff = blocks.RoutedExperts(E, top, 4, 2, 1.5, F)
    ff.w_up, ff.w_down, ff.z_off = torch.stack(ups).cuda(), torch.cat(downs, dim=1).contiguous().cuda(), 0
    h = torch.randn(T, W).to(dtype)
    z = 2.0 * torch.randn(T, E)
    want = []
    for t in range(T):
        chosen, w = oracle.route(z[t].double(), top, 4, 2, 1.5)
        want.append(oracle.experts(h[t].double(), chosen, w, [u.double() for u in ups], [d.double() for d in downs]))
    want = torch.stack(want)
    keep = blocks._GROUPED_ROWS, blocks._DENSE_MIN, blocks._FORCE_GROUPED
    blocks._FORCE_GROUPED = True
    try:
        for form, (g, d) in {"gather": (10 ** 9, 10 ** 9), "dense": (10 ** 9, 1), "grouped": (1, 1)}.items():
            blocks._GROUPED_ROWS, blocks._DENSE_MIN = g, d
            cases.close(ff.forward(h.cuda(), z.cuda()), want, tol)
    finally:
        blocks._GROUPED_ROWS, blocks._DENSE_MIN, blocks._FORCE_GROUPED = keep


def test_greedy_generation_with_decode_graphs(tmp_path):
    """Engine.generate: admission, packed prefill, CUDA-graph decode steps and the sampler kernel, in true 32-bit so that the
    tokens are comparable with the oracle's."""
    for name in ("mid_loop", "tc_ranks"):
        cases.test_greedy_generation_through_the_scheduler(tmp_path / name, name, "cuda", F32, graph=True)


def test_bfloat16_generation_runs_on_graphs(tmp_path):
    from llmss_b200.engine.runner import SamplingParams
    from llmss_b200.ops import _lib

    cfg, W, eng = cases.build(tmp_path, "tc_ranks", "cuda", BF16, graph=True, max_seq_len=128)
    n0 = _lib.LAUNCHES["count"]
    prompts = [cases.tokens_for(cfg, n, 90 + n) for n in (7, 30, 2)]
    out = eng.generate(prompts, SamplingParams(max_new_tokens=16, is_greedy=True))
    assert all(len(o) == 16 for o in out) and eng.runner.stats["graph_replays"] > 0 and _lib.LAUNCHES["count"] > n0
    # teacher-forcing the generated tokens gives logits whose argmax is (almost always) the next generated token
    seq = prompts[1] + out[1]
    lg = eng.feed([("chk", seq, list(range(len(prompts[1]) - 1, len(seq) - 1)))], ["chk"])
    agree = (lg.argmax(-1).cpu() == torch.tensor(out[1])).float().mean().item()
    assert agree >= 0.8


@pytest.mark.parametrize("dtype,tol", [pytest.param("float32", 3e-4, id="f32"), pytest.param("bfloat16", 8e-2, id="bf16")])
def test_trace_runner_on_cuda(tmp_path, dtype, tol):
    cases.run_trace_runner(tmp_path, {}, dtype, tol)
