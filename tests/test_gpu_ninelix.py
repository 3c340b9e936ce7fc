"""Ninelix on CUDA: the recurrence scan, token shift, short convolution, grouped gated norm, post-norm residual, biased
attention and gated experts kernels against the plain float64 oracle.

float32 runs everything in true 32-bit (tight tolerance); bfloat16 is what serving uses (tolerance of 16-bit rounding).
"""
import pytest
import torch

import ninelix_oracle as oracle
import test_ninelix_cpu as cases
from llmss_b200 import ops
from llmss_b200.utils.checkpoint import ninelix_config

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16
MODES = [pytest.param(F32, 3e-4, id="f32"), pytest.param(BF16, 8e-2, id="bf16")]

# sizes the kernels tile differently: key sizes over several 16-row strips, value sizes over a warp, many heads per group,
# more value channels than one block holds, widths that fit the tensor-core GEMM's 16-byte rules
cases.CONFIGS["wide"] = ninelix_config(128, 211, [
    {"type": "wkv", "heads": 2, "dim": 64, "lora": 16, "mlp": {"kind": "moe", "experts": 8, "top": 2, "ff": 32}},
    {"type": "parallel", "left": cases.attn(heads=12, kv_heads=1, dim=40, vdim=72, conv=4, bias_max=100, buckets=14),
     "right": cases.ssd(heads=4, vdim=32, state=40, groups=2, norm_groups=4, conv=4), "mlp": {"kind": "dense", "ff": 256}},
    {"type": "lightning", "heads": 2, "dim": 136, "vdim": 24, "mlp": None},
    {"type": "lightning", "heads": 1, "dim": 48, "vdim": 136, "mlp": None},
    {"type": "parallel", "left": cases.attn(heads=4, kv_heads=2, dim=128, vdim=64, conv=3, bias_max=70, buckets=8),
     "right": cases.ssd(heads=2, vdim=64, state=128, groups=1, norm_groups=1, conv=4), "mlp": None}], buckets=101)


def test_loaded_library_is_the_in_tree_one():
    from llmss_b200.ops import _lib

    _lib.load()
    assert _lib.LOADED_FROM.endswith("llmss_b200/_C/libllmss_b200.so")


def test_mechanisms():
    for taps in (1, 2, 3, 4, 6, 8):
        cases.test_causal_conv_op(taps, "cuda")
    for E, top in [(8, 2), (5, 1), (3, 3), (64, 6)]:
        cases.test_router_is_softmax_over_the_chosen_logits(E, top, "cuda")
    cases.test_gated_experts_op("cuda", F32, 1e-5)
    cases.test_gated_experts_op("cuda", BF16, 3e-2)


@pytest.mark.parametrize("kind,dk,dv,heads,qk_heads,read_before", [(0, 16, 16, 2, 2, False), (0, 136, 24, 2, 2, False), (1, 40, 32, 4, 2, False),
                                                                   (1, 128, 64, 2, 1, False), (2, 48, 48, 3, 3, True), (2, 64, 64, 2, 2, True),
                                                                   (2, 20, 136, 1, 1, True), (1, 300, 8, 2, 2, False)])
@pytest.mark.parametrize("chunked", [False, True])
def test_linear_scan_kernel_against_the_plain_recurrence(kind, dk, dv, heads, qk_heads, read_before, chunked, device="cuda"):
    """Portions of 1, 2 and more rows of two sequences, states carried in slots that held other values before.  ``chunked``:
    portions of 17 tokens and more run in two passes over 16-token chunks (chunk states and decay products in scratch)."""
    if device == "cuda":
        from llmss_b200.ops import cuda_impl as cu

        keep = cu._SCAN_CHUNK, cu._SCAN_CHUNK_MIN
        cu._SCAN_CHUNK, cu._SCAN_CHUNK_MIN = (16, 17) if chunked else (128, 1 << 30)
        try:
            _scan_case(kind, dk, dv, heads, qk_heads, read_before, device)
        finally:
            cu._SCAN_CHUNK, cu._SCAN_CHUNK_MIN = keep
    else:
        _scan_case(kind, dk, dv, heads, qk_heads, read_before, device)


def _scan_case(kind, dk, dv, heads, qk_heads, read_before, device):
    torch.manual_seed(dk + dv)
    n = [85, 45]
    rep = heads // qk_heads
    mk = lambda T, c: torch.randn(T, c, dtype=torch.float64) * 0.5
    data, head_decay = [], torch.rand(heads, dtype=torch.float64)
    for T in n:
        q, k, v = mk(T, qk_heads * dk), mk(T, qk_heads * dk), mk(T, heads * dv)
        dec = {0: head_decay, 1: -torch.rand(T, heads, dtype=torch.float64),
               2: -torch.rand(T, heads * dk, dtype=torch.float64)}[kind]
        c = torch.rand(T, heads, dtype=torch.float64) + 0.5
        data.append((q, k, v, dec, c))
    u = torch.randn(heads, dk, dtype=torch.float64) * 0.3
    want = []
    for (q, k, v, dec, c), T in zip(data, n):
        out = torch.zeros(T, heads, dv, dtype=torch.float64)
        for h in range(heads):
            S = torch.zeros(dk, dv, dtype=torch.float64)
            g = h // rep
            for t in range(T):
                a = dec[h] if kind == 0 else torch.exp(dec[t, h]) if kind == 1 else torch.exp(dec[t, h * dk:(h + 1) * dk])[:, None]
                kv = torch.outer(k[t, g * dk:(g + 1) * dk], c[t, h] * v[t, h * dv:(h + 1) * dv])
                if read_before:
                    out[t, h] = (S + u[h][:, None] * kv).T @ q[t, g * dk:(g + 1) * dk]
                    S = a * S + kv
                else:
                    S = a * S + kv
                    out[t, h] = S.T @ q[t, g * dk:(g + 1) * dk]
        want.append(out.reshape(T, heads * dv))
    state = torch.full((3, heads, dk, dv), 3.0, device=device)
    got, at = [[], []], [0, 0]
    f = lambda x: x.float().to(device)
    for sizes in ([1, 4], [2, 1], [1, 1], [49, 2], [16, 33], [40, 10]):
        live = [i for i in (0, 1) if sizes[i] > 0 and at[i] < n[i]]
        if not live:
            continue
        lens = [min(sizes[i], n[i] - at[i]) for i in live]
        batch = cases.fake_batch(lens, [at[i] for i in live], [2 - i for i in live], device, bs=64)
        cat = lambda j: torch.cat([data[i][j][at[i]:at[i] + m] for i, m in zip(live, lens)])
        dec = f(data[0][3]) if kind == 0 else f(cat(3))
        o = ops.linear_scan(f(cat(0)), f(cat(1)), f(cat(2)), dec, kind, batch, state, heads, qk_heads, dk, dv,
                            bonus=f(u) if read_before else None, v_scale=f(cat(4)), read_before=read_before).cpu()
        p = 0
        for i, m in zip(live, lens):
            got[i].append(o[p:p + m])
            at[i] += m
            p += m
    for i in (0, 1):
        assert at[i] == n[i]
        cases.close(torch.cat(got[i]), want[i], 2e-4)


@pytest.mark.parametrize("dtype,tol", MODES)
@pytest.mark.parametrize("name", ["wkv", "lightning", "parallel", "dense", "moe", "mixed", "edges", "wide"])
def test_model_whole_prompt(tmp_path, dtype, tol, name):
    cases.test_whole_prompt_and_residual_stream(tmp_path, name, "cuda", dtype, tol)


@pytest.mark.parametrize("dtype,tol", MODES)
def test_model_schedules(tmp_path, dtype, tol):
    for name in ("mixed", "edges", "wide"):
        cases.test_decode_token_by_token_and_portions(tmp_path / name, name, "cuda", dtype, tol)
    cases.test_unequal_batches_against_each_alone(tmp_path / "b", "cuda", dtype, tol)
    cases.test_first_tokens(tmp_path / "c", "cuda", dtype, tol)
    cases.test_long_decoding(tmp_path / "d", "cuda", dtype, tol)


@pytest.mark.parametrize("dtype,tol", MODES)
def test_model_pages_slots_far_keys(tmp_path, dtype, tol):
    cases.test_pages_and_slots_are_used_again(tmp_path / "a", "cuda", dtype, tol)
    cases.test_far_keys_bucket_edges_and_page_borders(tmp_path / "b", "cuda", dtype, tol if dtype == F32 else 0.15)
    cases.test_model_call_with_a_past(tmp_path / "c", "cuda", dtype, tol)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("graph", [False, True])
def test_generation(tmp_path, dtype, graph):
    """Engine.generate with and without CUDA-graph decode steps (padded batch rows are inert: slot -1)."""
    cases.test_greedy_generation_through_engine_and_cli(tmp_path, "cuda", dtype, graph)


def test_cuda_equals_cpu_engine_on_a_replayed_schedule(tmp_path):
    """The same mixed schedule through the CPU ops and through the kernels, true 32-bit."""
    cfg, W, cpu = cases.build(tmp_path / "a", "wide", "cpu", F32)
    _, _, gpu = cases.build(tmp_path / "b", "wide", "cuda", F32)
    reqs = {k: cases.tokens_for(cfg, n, 90 + n) for k, n in (("a", 130), ("b", 70), ("c", 3))}
    plan = [[("a", 65), ("c", 1)], [("a", 1), ("b", 64), ("c", 2)], [("a", 63), ("b", 1)], [("a", 1), ("b", 5)]]
    at = {k: 0 for k in reqs}
    for step in plan:
        entries = []
        for k, n in step:
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
        cases.close(gpu.feed(entries), cpu.feed(entries), 3e-4)


# key = value size 64 / 128 / 256 in 16-bit: the tensor-core flash kernel with the distance table and the gate; its
# tables end inside and beyond the context
cases.CONFIGS["tc_sizes"] = ninelix_config(128, 173, [
    {"type": "parallel", "left": cases.attn(heads=4, kv_heads=2, dim=64, vdim=64, conv=3, bias_max=50, buckets=12),
     "right": cases.ssd(heads=2, vdim=16, state=16, groups=1, norm_groups=1, conv=2), "mlp": {"kind": "dense", "ff": 128}},
    {"type": "parallel", "left": cases.attn(heads=2, kv_heads=1, dim=128, vdim=128, conv=2, bias_max=400, buckets=20),
     "right": cases.ssd(heads=2, vdim=16, state=16, groups=2, norm_groups=2, conv=2), "mlp": None},
    {"type": "parallel", "left": cases.attn(heads=3, kv_heads=3, dim=256, vdim=256, conv=2, bias_max=9, buckets=6),
     "right": cases.ssd(heads=2, vdim=16, state=16, groups=2, norm_groups=1, conv=3), "mlp": None}], buckets=37)


@pytest.mark.parametrize("d,hq,hkv,n_dist", [(64, 4, 2, 30), (128, 8, 2, 200), (256, 2, 1, 7), (128, 3, 3, 1)])
def test_biased_attention_kernels_agree_with_the_plain_formula(d, hq, hkv, n_dist):
    """Both CUDA forms (tensor-core flash kernel, generic kernel) on the same pages: a whole prompt, a portion over context,
    single tokens; keys at distances inside, on and beyond the table's end and across page borders."""
    from llmss_b200.engine.batch import BatchInput
    from llmss_b200.ops import cuda_impl as cu

    torch.manual_seed(d + hq)
    bs, dev = 64, "cuda"
    lens, ctxs = [150, 9, 1, 1], [0, 130, 139, 64]
    nblk = 4
    tables = [[1 + i * nblk + j for j in range(nblk)] for i in range(len(lens))]
    batch = BatchInput.build([[0] * n for n in lens], ctxs, tables, bs, dev, max_blocks=nblk)
    T = sum(lens)
    q = torch.randn(T, hq * d, device=dev).to(BF16)
    kc = torch.randn(1 + len(lens) * nblk, hkv, bs, d, device=dev).to(BF16)
    vc = torch.randn(1 + len(lens) * nblk, hkv, bs, d, device=dev).to(BF16)
    bias = (2.0 * torch.randn(hq, n_dist, device=dev)).contiguous()
    gate = torch.randn(T, hq + 3, device=dev)[:, 1:hq + 1]
    scale = 2.0 * d ** -0.5
    want = torch.zeros(T, hq, d, dtype=torch.float64)
    row = 0
    for i, (n, c) in enumerate(zip(lens, ctxs)):
        L = c + n
        k = kc[tables[i]].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :L].double().cpu()
        v = vc[tables[i]].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :L].double().cpu()
        for r in range(n):
            p = c + r
            for h in range(hq):
                g = h // (hq // hkv)
                s = (k[g, :p + 1] @ q[row, h * d:(h + 1) * d].double().cpu()) * scale
                s = s + torch.stack([bias[h, min(p - j, n_dist - 1)].double().cpu() for j in range(p + 1)])
                want[row, h] = (torch.softmax(s, 0)[:, None] * v[g, :p + 1]).sum(0) / (1.0 + torch.exp(-gate[row, h].double().cpu()))
            row += 1
    assert cu.attention_bias_uses_tc(BF16, d, d, bs, scale)
    got_tc = ops.attention_bias(q, kc, vc, batch, hq, hkv, d, d, scale, bias, gate=gate, out_dtype=BF16)
    cu._BIAS_TC = False
    try:
        got_generic = ops.attention_bias(q, kc, vc, batch, hq, hkv, d, d, scale, bias, gate=gate, out_dtype=BF16)
    finally:
        cu._BIAS_TC = True
    # 16-bit outputs of values several times the spread the error is measured against
    cases.close(got_generic, want.reshape(T, -1), 6e-2)
    cases.close(got_tc, want.reshape(T, -1), 6e-2)


def test_model_on_the_tensor_core_attention(tmp_path):
    cases.test_whole_prompt_and_residual_stream(tmp_path / "a", "tc_sizes", "cuda", BF16, 8e-2)
    cases.test_decode_token_by_token_and_portions(tmp_path / "b", "tc_sizes", "cuda", BF16, 8e-2)
    cases.test_whole_prompt_and_residual_stream(tmp_path / "c", "tc_sizes", "cuda", F32, 3e-4)


cases.CONFIGS["long"] = ninelix_config(128, 199, [
    {"type": "wkv", "heads": 2, "dim": 64, "lora": 8, "mlp": None},
    {"type": "parallel", "left": cases.attn(heads=4, kv_heads=2, dim=64, vdim=64, conv=3, bias_max=300, buckets=16),
     "right": cases.ssd(heads=4, vdim=24, state=40, groups=2, norm_groups=2, conv=4), "mlp": {"kind": "dense", "ff": 128}},
    {"type": "lightning", "heads": 2, "dim": 128, "vdim": 72, "mlp": None},
    {"type": "parallel", "left": cases.attn(heads=3, kv_heads=1, dim=40, vdim=24, conv=2, bias_max=900, buckets=24),
     "right": cases.ssd(heads=2, vdim=64, state=128, groups=1, norm_groups=1, conv=2), "mlp": None}], buckets=53)


@pytest.mark.parametrize("dtype,tol", [pytest.param(F32, 5e-4, id="f32"), pytest.param(BF16, 0.12, id="bf16")])
def test_long_prompt_in_portions_equals_the_cpu_engine(tmp_path, dtype, tol):
    """700 tokens: portions long enough for the two-pass recurrence (and one just under its threshold), a single token between
    them, attention over a dozen pages with the distance table ending inside and beyond the context -- against the same model
    on the CPU ops fed in one piece."""
    cfg, W, cpu = cases.build(tmp_path / "a", "long", "cpu", F32, max_seq_len=1024)
    _, _, gpu = cases.build(tmp_path / "b", "long", "cuda", dtype, max_seq_len=1024)
    toks = cases.tokens_for(cfg, 700, 21)
    want = cases.feed_in_portions(cpu, "w", toks, [700])
    got = cases.feed_in_portions(gpu, "p", toks, [300, 1, 257, 142])
    cases.close(got, want, tol)
    got = cases.feed_in_portions(gpu, "q", toks, [255, 445])
    cases.close(got, want, tol)
