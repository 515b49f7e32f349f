"""GPU parity tests: every operator through the C ABI (raw pointers, caller-allocated
outputs) against the CPU oracle and the reference-made golden fixtures.

Tolerances: reshape_and_cache and add_rms_norm's residual output are bit-exact; the other
fp16 results are within rtol 1e-2 / atol 1e-3 of the fp32-accumulating golden.
"""
import numpy as np
import pytest
import torch

import decode_workloads as wl
from conftest import bits, f16, knob
from oracle import decode_ops_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
RTOL, ATOL = 1e-2, 1e-3


def close(got, want, rtol=RTOL, atol=ATOL):
    torch.testing.assert_close(got.cpu().float(), want.float(), rtol=rtol, atol=atol)


# ------------------------------------------------------------------ add_rms_norm
def run_add_rms_norm(cabi, x, r, w, eps):
    xd, rd, wd = x.to(DEV), r.to(DEV), w.to(DEV)
    y = torch.full_like(xd, float("nan"))
    s = torch.full_like(xd, float("nan"))
    cabi.add_rms_norm(xd, rd, wd, eps, y, s)
    torch.cuda.synchronize()
    return y.cpu(), s.cpu()


def test_add_rms_norm_golden(cabi, golden):
    z = golden("add_rms_norm")
    for i in range(int(z["n"])):
        y, s = run_add_rms_norm(cabi, f16(z[f"x{i}"]), f16(z[f"r{i}"]), f16(z[f"w{i}"]), float(z[f"eps{i}"]))
        assert np.array_equal(bits(s), z[f"s{i}"])
        close(y, f16(z[f"y{i}"]))


@pytest.mark.parametrize("tokens,hidden", [(1, 64), (7, 128), (33, 1088), (257, 4096), (5, 8192),
                                           (3, 16384), (2, 65536), (2, 65600)])
def test_add_rms_norm_shapes(cabi, tokens, hidden):
    d = wl.add_rms_norm_inputs(tokens, hidden, seed=tokens + hidden)
    y, s = run_add_rms_norm(cabi, d["x"], d["residual"], d["weight"], d["eps"])
    ey, es = oracle.add_rms_norm(d["x"], d["residual"], d["weight"], d["eps"])
    assert torch.equal(s, es)
    close(y, ey)


def test_add_rms_norm_benchmark_size_and_api(cabi, ops):
    d = wl.add_rms_norm_inputs()
    ey, es = oracle.add_rms_norm(d["x"], d["residual"], d["weight"], d["eps"])
    y, s = ops.add_rms_norm(d["x"].to(DEV), d["residual"].to(DEV), d["weight"].to(DEV), d["eps"])
    assert torch.equal(s.cpu(), es)
    close(y, ey)
    # large-magnitude rows must not overflow the fp32 sum of squares
    big = (d["x"][:4] * 200).half()
    y, s = run_add_rms_norm(cabi, big, big, d["weight"], 1e-6)
    ey, es = oracle.add_rms_norm(big, big, d["weight"], 1e-6)
    assert torch.equal(s, es)
    close(y, ey)


# ------------------------------------------------------------------ swiglu
def run_swiglu(cabi, x):
    xd = x.to(DEV)
    y = torch.full((x.shape[0], x.shape[1] // 2), float("nan"), dtype=torch.float16, device=DEV)
    cabi.swiglu(xd, y)
    torch.cuda.synchronize()
    return y.cpu()


def test_swiglu_golden(cabi, golden):
    z = golden("swiglu")
    for i in range(int(z["n"])):
        close(run_swiglu(cabi, f16(z[f"x{i}"])), f16(z[f"y{i}"]))


@pytest.mark.parametrize("tokens,d", [(1, 32), (5, 96), (1031, 192), (64, 14336), (3, 100000 * 32 // 32)])
def test_swiglu_shapes(cabi, tokens, d):
    if d % 32:
        d = d // 32 * 32
    x = (torch.randn(tokens, 2 * d, generator=torch.Generator().manual_seed(d)) * 4).half()
    close(run_swiglu(cabi, x), oracle.swiglu(x))


def test_swiglu_extreme_values_and_api(ops):
    x = torch.tensor([[-65504.0, -30.0, -1.0, 0.0, 1.0, 30.0, 200.0, 65504.0] * 8] * 2).half()
    x = torch.cat([x, torch.ones_like(x)], dim=1)  # gate = values, up = 1
    y = ops.swiglu(x.to(DEV)).cpu()
    close(y, oracle.swiglu(x))
    assert torch.isfinite(y[:, :-1].float()).all()


# ------------------------------------------------------------------ rope
def run_rope(cabi, q, k, pos, cos, sin):
    oq = torch.full_like(q, float("nan"), device=DEV)
    ok = torch.full_like(k, float("nan"), device=DEV)
    cabi.rope(q.to(DEV), k.to(DEV), pos.to(DEV), cos.to(DEV), sin.to(DEV), oq, ok)
    torch.cuda.synchronize()
    return oq.cpu(), ok.cpu()


def test_rope_golden(cabi, golden):
    z = golden("rope")
    for i in range(int(z["n"])):
        oq, ok = run_rope(cabi, f16(z[f"q{i}"]), f16(z[f"k{i}"]), torch.from_numpy(z[f"pos{i}"]),
                          f16(z[f"cos{i}"]), f16(z[f"sin{i}"]))
        # fp32 evaluation of the reference's fn_naive, one rounding
        close(oq, torch.from_numpy(z[f"oq32_{i}"]))
        close(ok, torch.from_numpy(z[f"ok32_{i}"]))
        # and the fp16 evaluation the reference itself runs
        close(oq, f16(z[f"oq{i}"]))
        close(ok, f16(z[f"ok{i}"]))


@pytest.mark.parametrize("tokens,hq,hkv,d", [(1, 1, 1, 16), (9, 4, 4, 64), (256, 32, 8, 128), (17, 28, 4, 256)])
def test_rope_shapes(cabi, ops, tokens, hq, hkv, d):
    w = wl.rope_inputs(tokens, hq, hkv, d, min_pos=0, max_pos=300, seed=tokens)
    eq, ek = oracle.rope(w["q"], w["k"], w["position_ids"], w["cos_cache"], w["sin_cache"])
    oq, ok = run_rope(cabi, w["q"], w["k"], w["position_ids"], w["cos_cache"], w["sin_cache"])
    close(oq, eq)
    close(ok, ek)
    aq, ak = ops.rope(*(w[n].to(DEV) for n in ("q", "k", "position_ids", "cos_cache", "sin_cache")))
    assert torch.equal(aq.cpu(), oq) and torch.equal(ak.cpu(), ok)


# ------------------------------------------------------------------ reshape_and_cache
def test_reshape_and_cache_reference_case(cabi, ops, golden):
    z = golden("reshape_and_cache")
    shape = tuple(int(v) for v in z["shape0"])
    kc = torch.zeros(shape, dtype=torch.float16, device=DEV)
    vc = torch.zeros(shape, dtype=torch.float16, device=DEV)
    cabi.reshape_and_cache(f16(z["key0"]).to(DEV), f16(z["value0"]).to(DEV), kc, vc,
                           torch.from_numpy(z["slots0"]).to(DEV), cabi.KV_LAYOUT_NZ)
    torch.cuda.synchronize()
    for cache, vals in ((kc, z["kc0"]), (vc, z["vc0"])):
        flat = bits(cache).reshape(-1)
        assert np.array_equal(flat[z["idx0"]], vals)
        assert np.count_nonzero(flat) == np.count_nonzero(vals)
    # key-only form through the Python API: value cache must stay zero
    kc.zero_()
    vc.zero_()
    ops.reshape_and_cache(f16(z["key1"]).to(DEV), None, kc, None, torch.from_numpy(z["slots1"]).to(DEV))
    torch.cuda.synchronize()
    flat = bits(kc).reshape(-1)
    assert np.array_equal(flat[z["idx1"]], z["kc1"]) and np.count_nonzero(flat) == np.count_nonzero(z["kc1"])
    assert not vc.any()


def test_reshape_and_cache_small_dense_golden(cabi, golden):
    z = golden("reshape_and_cache")
    shape = tuple(int(v) for v in z["shape2"])
    kc = torch.zeros(shape, dtype=torch.float16, device=DEV)
    vc = torch.zeros(shape, dtype=torch.float16, device=DEV)
    cabi.reshape_and_cache(f16(z["key2"]).to(DEV), f16(z["value2"]).to(DEV), kc, vc,
                           torch.from_numpy(z["slots2"]).to(DEV), cabi.KV_LAYOUT_NZ)
    assert np.array_equal(bits(kc), z["kc2_dense"]) and np.array_equal(bits(vc), z["vc2_dense"])


@pytest.mark.parametrize("layout", [wl.KV_LAYOUT_NHD, wl.KV_LAYOUT_NZ])
@pytest.mark.parametrize("tokens,hkv,d,blocks,p", [(2048, 8, 128, 4096, 128), (37, 2, 64, 9, 16),
                                                   (5, 1, 24, 4, 8), (64, 3, 40, 16, 32)])
def test_reshape_and_cache_vs_oracle(cabi, layout, tokens, hkv, d, blocks, p):
    if layout == wl.KV_LAYOUT_NZ and (hkv * d) % 16:
        pytest.skip("NZ layout needs a row that is a multiple of 16")
    w = wl.reshape_and_cache_inputs(tokens, hkv, d, blocks, p, layout, seed=tokens)
    slots = w["slot_indices"].clone()
    if tokens > 4:  # some slots the kernel must skip
        slots[1] = -1
        slots[3] = blocks * p
        slots[4] = -7
    pattern = (torch.arange(int(np.prod(w["cache_shape"])), dtype=torch.int32) % 1021).short()
    kc_cpu = pattern.view(torch.float16).view(w["cache_shape"]).clone()
    vc_cpu = (pattern + 1).view(torch.float16).view(w["cache_shape"]).clone()
    kc, vc = kc_cpu.to(DEV), vc_cpu.to(DEV)
    cabi.reshape_and_cache(w["key"].to(DEV), w["value"].to(DEV), kc, vc, slots.to(DEV), layout)
    torch.cuda.synchronize()
    oracle.reshape_and_cache(w["key"], kc_cpu, slots, w["value"], vc_cpu, layout)
    assert np.array_equal(bits(kc), bits(kc_cpu))
    assert np.array_equal(bits(vc), bits(vc_cpu))


# ------------------------------------------------------------------ paged_attention
def run_paged_attention(cabi, w):
    q = w["q"].to(DEV)
    kc, vc = w["key_cache"].to(DEV), w["value_cache"].to(DEV)
    out = torch.full_like(q, float("nan"))
    n = cabi.paged_attention_workspace_size(q.shape[0], q.shape[1], w["kv_heads"], q.shape[2],
                                            w["block_size"], w["block_tables"].shape[1])
    ws = torch.empty(max(n, 1), dtype=torch.uint8, device=DEV)
    cabi.paged_attention(q, kc, vc, w["block_tables"].to(DEV), w["context_lens"].to(DEV), out,
                         w["kv_heads"], w["block_size"], w["layout"], ws if n else None)
    torch.cuda.synchronize()
    assert cabi.pipeline_status() == 0
    return out.cpu()


@pytest.mark.parametrize("layout", [wl.KV_LAYOUT_NHD, wl.KV_LAYOUT_NZ])
@pytest.mark.parametrize("heads,kv_heads,d,p", [(28, 4, 128, 128), (32, 8, 128, 128), (8, 8, 64, 16),
                                                (16, 1, 128, 32), (12, 4, 256, 16), (4, 2, 32, 8),
                                                (40, 2, 128, 64)])
def test_paged_attention_ragged(cabi, layout, heads, kv_heads, d, p):
    lens = [1, 0, p, p + 1, 3 * p - 1, 517, 1300, 2048, 5]
    blocks = sum((l + p - 1) // p for l in lens) + 3
    w = wl.paged_attention_inputs(heads=heads, kv_heads=kv_heads, head_dim=d, block_size=p,
                                  blocks=blocks, layout=layout, context_lens=lens, seed=heads + d)
    # poison every cache position beyond each sequence's length: a correct kernel never lets
    # them reach the output
    w = poison_unused(w)
    want = oracle.paged_attention(clean(w["q"]), w["key_cache_clean"], w["value_cache_clean"],
                                  w["block_tables"], w["context_lens"], layout)
    got = run_paged_attention(cabi, w)
    close(got, want)
    assert not got[1].any()  # context_len 0 -> zeros


def clean(t):
    return t


def poison_unused(w):
    """NaN-fill all cache tokens that no sequence owns (tails of last pages, spare pages)."""
    layout, p = w["layout"], w["block_size"]
    kc, vc = w["key_cache"], w["value_cache"]
    pages = kc.shape[0]
    used = torch.zeros(pages, p, dtype=torch.bool)
    for b, L in enumerate(w["context_lens"].tolist()):
        for i in range((L + p - 1) // p):
            pg = int(w["block_tables"][b, i])
            used[pg, : min(p, L - i * p)] = True
    w = dict(w)
    w["key_cache_clean"], w["value_cache_clean"] = kc, vc
    kp, vp = kc.clone(), vc.clone()
    if layout == wl.KV_LAYOUT_NHD:
        kp[~used] = float("nan")
        vp[~used] = float("nan")
    else:
        m = (~used)[:, None, :, None].expand_as(kp)
        kp[m] = float("nan")
        vp[m] = float("nan")
    w["key_cache"], w["value_cache"] = kp, vp
    return w


def test_paged_attention_benchmark_shape_reduced(cabi, ops):
    """The benchmark's GQA configuration (28 q / 4 kv heads, D 128, pages of 128) on 12 sequences."""
    w = wl.paged_attention_inputs(bs=12, blocks=12 * 64, seed=33)
    want = oracle.paged_attention(w["q"], w["key_cache"], w["value_cache"], w["block_tables"],
                                  w["context_lens"])
    got = run_paged_attention(cabi, w)
    close(got, want)
    api = ops.paged_attention(w["q"].to(DEV), w["key_cache"].to(DEV), w["value_cache"].to(DEV),
                              w["block_tables"].to(DEV), w["context_lens"].to(DEV))
    assert torch.equal(api.cpu(), got)


def test_paged_attention_long_context_split(cabi):
    """One long sequence next to short ones: many chunks for one, a single chunk for others."""
    w = wl.paged_attention_inputs(heads=32, kv_heads=8, context_lens=[16385, 7, 129, 4096],
                                  blocks=200, seed=9)
    want = oracle.paged_attention(w["q"], w["key_cache"], w["value_cache"], w["block_tables"],
                                  w["context_lens"])
    close(run_paged_attention(cabi, w), want)


def test_paged_attention_workspace_too_small(cabi):
    w = wl.paged_attention_inputs(bs=2, blocks=200, seed=1)
    q = w["q"].to(DEV)
    with pytest.raises(cabi.B200OpsError) as e:
        cabi.paged_attention(q, w["key_cache"].to(DEV), w["value_cache"].to(DEV),
                             w["block_tables"].to(DEV), w["context_lens"].to(DEV),
                             torch.empty_like(q), 4, 128, wl.KV_LAYOUT_NHD,
                             torch.empty(16, dtype=torch.uint8, device=DEV))
    assert e.value.code == cabi.EWORKSPACE


# ------------------------------------------------------------------ grouped_matmul
def run_grouped_matmul(cabi, x, w_storage, gl, fill=float("nan"), split_k=True):
    """With split_k the call gets the workspace the size query asks for (if any)."""
    y = torch.full((x.shape[0], w_storage.shape[1]), fill, dtype=torch.float16, device=DEV)
    e, n, k = w_storage.shape
    nbytes = cabi.grouped_matmul_workspace_size(x.shape[0], k, e, n) if split_k else 0
    ws = torch.full((nbytes,), 0xAB, dtype=torch.uint8, device=DEV) if nbytes else None
    cabi.grouped_matmul(x.to(DEV), w_storage.to(DEV), gl.to(DEV), y, ws)
    torch.cuda.synchronize()
    assert cabi.pipeline_status() == 0
    return y.cpu()


def test_grouped_matmul_golden(cabi, golden):
    z = golden("grouped_matmul")
    for i in range(int(z["n"])):
        y = run_grouped_matmul(cabi, f16(z[f"x{i}"]), f16(z[f"w{i}"]), torch.from_numpy(z[f"gl{i}"]))
        close(y, f16(z[f"y{i}"]))


@pytest.mark.parametrize("counts,k,n", [
    ([128], 64, 64),                       # one exact tile
    ([1], 64, 64),                         # a single row
    ([300, 0, 1, 129, 70], 256, 320),      # M tails, an empty group, N tail (320 = 256 + 64)
    ([5, 250, 3, 0, 0, 77, 128, 256], 512, 1024),
    ([1000], 1024, 768),                   # plain NT GEMM (one group)
    ([17] * 128, 128, 192),                # many experts, uniform
    ([0, 0, 40], 64, 128),                 # leading empty groups
])
def test_grouped_matmul_vs_oracle(cabi, counts, k, n):
    g = torch.Generator().manual_seed(sum(counts) + k + n)
    m = sum(counts)
    x = torch.randn(m, k, generator=g).half()
    w_storage = (torch.randn(len(counts), n, k, generator=g) * 0.05).half()
    gl = torch.tensor(counts).cumsum(0).to(torch.int64)
    want = oracle.grouped_matmul(x, w_storage.transpose(1, 2), gl)
    close(run_grouped_matmul(cabi, x, w_storage, gl), want)


def test_grouped_matmul_rows_past_last_group_untouched_and_api(cabi, ops):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(200, 128, generator=g).half()
    w_storage = (torch.randn(3, 192, 128, generator=g) * 0.05).half()
    gl = torch.tensor([50, 50, 130], dtype=torch.int64)  # rows 130..199 belong to no group
    y = run_grouped_matmul(cabi, x, w_storage, gl, fill=7.0)
    want = oracle.grouped_matmul(x, w_storage.transpose(1, 2), gl)
    close(y[:130], want[:130])
    assert (y[130:] == 7.0).all()
    api = ops.grouped_matmul(x.to(DEV), w_storage.to(DEV).transpose(1, 2), gl.to(DEV)).cpu()
    assert torch.equal(api[:130], y[:130])


def test_grouped_matmul_moe_shape_sampled_rows(cabi):
    """Expert count, hidden size and routing skew of the MoE benchmark at a reduced row
    count and N; all rows are checked."""
    w = wl.grouped_matmul_inputs(rows=1536, k=4096, n=1024, experts=8, seed=11)
    want = oracle.grouped_matmul(w["x"], w["w_storage"].transpose(1, 2), w["group_list"])
    close(run_grouped_matmul(cabi, w["x"], w["w_storage"], w["group_list"]), want)


def test_paged_attention_benchmark_size_all_paths_agree(cabi, monkeypatch):
    """Full benchmark batch (64 sequences, lengths U[512, 8192], 8192 pages): the split-context
    TMA kernel, the general kernel and the CPU oracle."""
    w = wl.paged_attention_inputs()
    knob(monkeypatch, "B200OPS_PA_MODE", "1")
    chunked = run_paged_attention(cabi, w)
    knob(monkeypatch, "B200OPS_PA_MODE", "2")
    general = run_paged_attention(cabi, w)
    knob(monkeypatch, "B200OPS_PA_MODE", None)
    close(chunked, general)
    want = oracle.paged_attention(w["q"], w["key_cache"], w["value_cache"], w["block_tables"],
                                  w["context_lens"])
    close(chunked, want)


@pytest.mark.parametrize("layout", [wl.KV_LAYOUT_NHD, wl.KV_LAYOUT_NZ])
@pytest.mark.parametrize("stages", ["2", "4", "6"])
@pytest.mark.parametrize("chunk", ["128", "2048"])
def test_paged_attention_split_context_path_pipeline_depths(cabi, monkeypatch, stages, chunk, layout):
    """The TMA path on both cache layouts, every ring depth, short and long chunks, with NaN in
    every cache token that no sequence owns."""
    knob(monkeypatch, "B200OPS_PA_MODE", "1")
    knob(monkeypatch, "B200OPS_PA_STAGES", stages)
    knob(monkeypatch, "B200OPS_PA_CHUNK_TOKENS", chunk)
    lens = [1, 63, 64, 65, 127, 128, 129, 1000, 4097, 0, 2048]
    w = wl.paged_attention_inputs(heads=32, kv_heads=4, context_lens=lens, blocks=80, seed=int(stages),
                                  layout=layout)
    w = poison_unused(w)
    want = oracle.paged_attention(w["q"], w["key_cache_clean"], w["value_cache_clean"],
                                  w["block_tables"], w["context_lens"])
    close(run_paged_attention(cabi, w), want)


@pytest.mark.parametrize("heads,kv_heads,page,lens", [
    (28, 4, 128, [1, 63, 64, 65, 127, 128, 129, 1000, 4097, 0, 2048]),
    (32, 8, 64, [0, 0, 5, 0, 700, 64, 0]),                 # empty sequences in every position
    (16, 1, 256, [33000]),                                 # one long sequence spread over all CTAs
    (64, 4, 128, [3000] * 3 + [17] * 40),                  # group of 16 (upper MMA rows in use)
    (8, 8, 128, list(range(1, 400, 7))),                   # many short sequences, group 1
    (8, 2, 64, [(i * 37) % 300 for i in range(700)]),      # a large batch of short sequences
])
def test_paged_attention_ragged_batches(cabi, heads, kv_heads, page, lens):
    blocks = sum((l + page - 1) // page for l in lens) + 2
    w = wl.paged_attention_inputs(heads=heads, kv_heads=kv_heads, block_size=page, context_lens=lens,
                                  blocks=blocks, seed=heads + page)
    w = poison_unused(w)
    want = oracle.paged_attention(w["q"], w["key_cache_clean"], w["value_cache_clean"],
                                  w["block_tables"], w["context_lens"])
    close(run_paged_attention(cabi, w), want)


@pytest.mark.parametrize("counts,k,n", [
    ([40, 0, 3, 90, 7, 64, 1, 128], 14336, 4096),  # expert down projection at decode size
    ([70], 14336, 4096),               # one expert per GPU: 16 tiles -> 9 k-slices each
    ([100], 8192, 320),                # N tail with split-K
    ([130], 8192, 256),                # two m-tiles, the second one a tail
    ([256], 16384, 1024),              # dense projection with a long K
])
def test_grouped_matmul_split_k(cabi, monkeypatch, counts, k, n):
    knob(monkeypatch, "B200OPS_GMM_KSPLIT", "0")  # single-group shapes would take the cluster path
    g = torch.Generator().manual_seed(sum(counts) + k)
    m = sum(counts)
    x = torch.randn(m, k, generator=g).half()
    w_storage = (torch.randn(len(counts), n, k, generator=g) * 0.03).half()
    gl = torch.tensor(counts).cumsum(0).to(torch.int64)
    assert cabi.grouped_matmul_workspace_size(m, k, len(counts), n) > 0
    want = oracle.grouped_matmul(x, w_storage.transpose(1, 2), gl)
    split = run_grouped_matmul(cabi, x, w_storage, gl, split_k=True)
    plain = run_grouped_matmul(cabi, x, w_storage, gl, split_k=False)
    close(split, want)
    close(plain, want)
    # twice in a row on the same workspace contents: the call resets its own counters
    close(run_grouped_matmul(cabi, x, w_storage, gl, split_k=True), want)


@pytest.mark.parametrize("counts,k,n", [
    ([100], 4096, 6144),          # decode-size QKV projection: 96 narrow tiles, one per CTA
    ([32], 4096, 4096),           # output projection at 32 tokens
    ([128], 64, 64),              # smallest narrow problem
    ([10] * 8, 512, 4096),        # several groups: 512 narrow tiles, several per CTA
    ([3, 0, 60, 1, 64], 1024, 2304),  # ragged groups, empty group, N not a multiple of 256
])
def test_grouped_matmul_narrow_tiles(cabi, monkeypatch, counts, k, n):
    """At most 128 rows in total and few output columns: the 128 x 64 tile configuration
    (reached by single-group shapes only when the cluster split-K path is switched off)."""
    knob(monkeypatch, "B200OPS_GMM_KSPLIT", "0")
    g = torch.Generator().manual_seed(sum(counts) + k + n)
    m = sum(counts)
    x = torch.randn(m, k, generator=g).half()
    w_storage = (torch.randn(len(counts), n, k, generator=g) * 0.05).half()
    gl = torch.tensor(counts).cumsum(0).to(torch.int64)
    want = oracle.grouped_matmul(x, w_storage.transpose(1, 2), gl)
    close(run_grouped_matmul(cabi, x, w_storage, gl), want)


@pytest.mark.parametrize("counts,k,n", [
    ([128], 64, 64),                        # smallest: CTA 1 of the pair has no rows at all
    ([256], 128, 256),                      # exactly one full pair
    ([300, 0, 1, 129, 70], 256, 320),       # odd m-tile counts, an empty group, N tail (256 + 64)
    ([5, 250, 3, 0, 0, 77, 128, 256], 512, 1024),
    ([1000], 1024, 768),                    # one group: 4 pairs x 3 n-tiles
    ([17] * 128, 128, 192),                 # many experts, every pair half empty
    ([0, 0, 40], 64, 128),                  # leading empty groups; second half of w past N
    ([700, 900, 3000], 2048, 1536),         # several items per cluster, long k loop (ring wraps)
])
def test_grouped_matmul_cta_pairs(cabi, monkeypatch, counts, k, n):
    """The CTA-pair kernel (two CTAs per 256-row MMA), forced for shapes of every kind; the
    single-CTA kernel on the same inputs must give the same bits (same fp32 sums, same order)."""
    g = torch.Generator().manual_seed(sum(counts) + k + n)
    m = sum(counts)
    x = torch.randn(m, k, generator=g).half()
    w_storage = (torch.randn(len(counts), n, k, generator=g) * 0.05).half()
    gl = torch.tensor(counts).cumsum(0).to(torch.int64)
    want = oracle.grouped_matmul(x, w_storage.transpose(1, 2), gl)
    knob(monkeypatch, "B200OPS_GMM_PAIR", "2")
    pairs = run_grouped_matmul(cabi, x, w_storage, gl, fill=3.0, split_k=False)
    knob(monkeypatch, "B200OPS_GMM_PAIR", "0")
    single = run_grouped_matmul(cabi, x, w_storage, gl, fill=3.0, split_k=False)
    close(pairs, want)
    assert torch.equal(pairs, single)


def test_grouped_matmul_cta_pairs_engage_at_benchmark_scale(cabi, monkeypatch):
    """A problem of several tile waves takes the pair kernel by default; sampled rows of every
    group are checked against the oracle, all rows against the single-CTA kernel."""
    w = wl.grouped_matmul_inputs(rows=8192, k=1024, n=4096, experts=8, seed=12)
    knob(monkeypatch, "B200OPS_GMM_PAIR", None)
    auto = run_grouped_matmul(cabi, w["x"], w["w_storage"], w["group_list"])
    knob(monkeypatch, "B200OPS_GMM_PAIR", "0")
    single = run_grouped_matmul(cabi, w["x"], w["w_storage"], w["group_list"], split_k=False)  # tile by tile
    assert torch.equal(auto, single)
    rows = torch.arange(0, 8192, 61)
    ends = w["group_list"]
    expert = torch.searchsorted(ends, rows, right=True)
    want = torch.stack([(w["x"][r].float() @ w["w_storage"][e].float().T) for r, e in zip(rows, expert)])
    close(auto[rows], want.half())


@pytest.mark.parametrize("counts,k,n", [
    ([256], 4096, 6144),     # QKV projection of a 256-row decode batch: 48 tiles x 3 CTAs
    ([256], 4096, 4096),     # output projection: 32 tiles x 4
    ([32], 4096, 6144),      # 32 rows: 24 tiles x 6
    ([32], 4096, 4096),      # 16 tiles x 8 (the largest cluster)
    ([200], 1024, 320),      # second m-tile a tail, N tail (256 + 64), 4 k-blocks per CTA
    ([1], 512, 64),          # one row, one tile, two CTAs
    ([70], 14336, 4096),     # long K
    ([129], 960, 2048),      # 15 k-blocks over 3 CTAs: uneven slices
])
def test_grouped_matmul_cluster_split_k(cabi, monkeypatch, counts, k, n):
    """Dense decode-size projections: the CTAs of a cluster share one output tile and reduce
    their k-slices through distributed shared memory."""
    g = torch.Generator().manual_seed(sum(counts) + k + n)
    m = sum(counts)
    x = torch.randn(m, k, generator=g).half()
    w_storage = (torch.randn(1, n, k, generator=g) * 0.05).half()
    gl = torch.tensor(counts).cumsum(0).to(torch.int64)
    want = oracle.grouped_matmul(x, w_storage.transpose(1, 2), gl)
    knob(monkeypatch, "B200OPS_GMM_KSPLIT", None)
    got = run_grouped_matmul(cabi, x, w_storage, gl, fill=5.0, split_k=False)
    close(got, want)
    again = run_grouped_matmul(cabi, x, w_storage, gl, fill=5.0, split_k=False)
    assert torch.equal(got, again)  # fixed summation order: bitwise repeatable
    knob(monkeypatch, "B200OPS_GMM_SHORT", "0")  # full activation tiles also for up to 80 rows: the same bits
    assert torch.equal(run_grouped_matmul(cabi, x, w_storage, gl, fill=5.0, split_k=False), got)
    knob(monkeypatch, "B200OPS_GMM_SHORT", None)
    knob(monkeypatch, "B200OPS_GMM_KSPLIT", "0")
    close(run_grouped_matmul(cabi, x, w_storage, gl, fill=5.0, split_k=False), want)


@pytest.mark.parametrize("counts,k,n", [
    ([64] * 8, 512, 512),              # a decode batch: every group fits the short activation tile
    ([80, 1, 0, 79, 33], 1024, 768),   # the limit itself, a single row, an empty group; 16 k-blocks wrap the 5-stage ring
    ([81, 3], 512, 512),               # one row too many: the launch keeps the full tile
    ([40, 70], 8192, 512),             # short tiles together with split-K through the workspace
    ([17] * 100, 256, 256),            # a hundred small groups
])
def test_grouped_matmul_short_activation_tiles(cabi, monkeypatch, counts, k, n):
    """When no group has more than 80 rows the kernel loads 80-row activation tiles into a
    five-stage ring; the products are the same, in the same order: bit-equal to the full tile."""
    g = torch.Generator().manual_seed(sum(counts) + k + n)
    m = sum(counts)
    x = torch.randn(m + 40, k, generator=g).half()  # rows past the last group: read by boxes, never used
    w_storage = (torch.randn(len(counts), n, k, generator=g) * 0.05).half()
    gl = torch.tensor(counts).cumsum(0).to(torch.int64)
    want = oracle.grouped_matmul(x, w_storage.transpose(1, 2), gl)
    knob(monkeypatch, "B200OPS_GMM_SHORT", None)
    got = run_grouped_matmul(cabi, x, w_storage, gl, fill=5.0)
    close(got[:m], want[:m])
    assert (got[m:] == 5.0).all()
    knob(monkeypatch, "B200OPS_GMM_SHORT", "0")
    full = run_grouped_matmul(cabi, x, w_storage, gl, fill=5.0)
    assert torch.equal(got, full)
    # the same with SwiGLU in the epilogue
    xd, wd, gld = x.to(DEV), w_storage.to(DEV), gl.to(DEV)
    fused_full = torch.full((m + 40, n // 2), 3.0, dtype=torch.float16, device=DEV)
    cabi.grouped_matmul_swiglu(xd, wd, gld, fused_full)
    knob(monkeypatch, "B200OPS_GMM_SHORT", None)
    fused = torch.full((m + 40, n // 2), 3.0, dtype=torch.float16, device=DEV)
    cabi.grouped_matmul_swiglu(xd, wd, gld, fused)
    torch.cuda.synchronize()
    assert cabi.pipeline_status() == 0
    assert torch.equal(fused, fused_full)
    close(fused[:m].cpu(), oracle.swiglu(want[:m]))


def test_grouped_matmul_cluster_split_k_fewer_rows_than_the_bound(cabi):
    """group_list may end before num_tokens: clusters whose tile does not exist do nothing, rows
    past the group's end stay untouched."""
    g = torch.Generator().manual_seed(77)
    x = torch.randn(256, 2048, generator=g).half()
    w_storage = (torch.randn(1, 1024, 2048, generator=g) * 0.05).half()
    gl = torch.tensor([100], dtype=torch.int64)
    want = oracle.grouped_matmul(x, w_storage.transpose(1, 2), gl)
    got = run_grouped_matmul(cabi, x, w_storage, gl, fill=9.0, split_k=False)
    close(got[:100], want[:100])
    assert (got[100:] == 9.0).all()


@pytest.mark.parametrize("pair_mode", ["0", "2"])  # single-CTA kernel / CTA-pair kernel
@pytest.mark.parametrize("counts,k,d", [
    ([128], 64, 64),                         # one tile, half of it columns
    ([300, 0, 1, 129, 70], 256, 192),        # M tails, an empty group, d = 128 + 64 (a column tail)
    ([40, 3, 90, 7], 512, 1024),             # decode-size groups
    ([700, 900, 300], 1024, 1408),           # several tiles per CTA; d = 11 * 128
])
def test_grouped_matmul_swiglu_equals_the_two_operators(cabi, monkeypatch, counts, k, d, pair_mode):
    """SwiGLU in the GEMM's epilogue: the same bits as grouped_matmul followed by swiglu (the
    accumulators are rounded to fp16 in between, as the intermediate tensor would be)."""
    knob(monkeypatch, "B200OPS_GMM_PAIR", pair_mode)
    g = torch.Generator().manual_seed(sum(counts) + k + d)
    m = sum(counts)
    x = torch.randn(m, k, generator=g).half().to(DEV)
    w_storage = (torch.randn(len(counts), 2 * d, k, generator=g) * 0.05).half().to(DEV)
    gl = torch.tensor(counts).cumsum(0).to(torch.int64).to(DEV)
    gu = torch.zeros(m, 2 * d, dtype=torch.float16, device=DEV)
    cabi.grouped_matmul(x, w_storage, gl, gu, None)
    two_step = torch.empty(m, d, dtype=torch.float16, device=DEV)
    cabi.swiglu(gu, two_step)
    fused = torch.full((m, d), 3.0, dtype=torch.float16, device=DEV)
    cabi.grouped_matmul_swiglu(x, w_storage, gl, fused)
    torch.cuda.synchronize()
    assert cabi.pipeline_status() == 0
    assert torch.equal(fused, two_step)
    want = oracle.swiglu(oracle.grouped_matmul(x.cpu(), w_storage.cpu().transpose(1, 2), gl.cpu()))
    close(fused.cpu(), want)


def test_grouped_matmul_swiglu_rejects_odd_widths(cabi):
    x = torch.zeros(4, 64, dtype=torch.float16, device=DEV)
    w = torch.zeros(1, 192, 64, dtype=torch.float16, device=DEV)  # d = 96: not a multiple of 64
    gl = torch.tensor([4], dtype=torch.int64, device=DEV)
    with pytest.raises(cabi.B200OpsError) as e:
        cabi.grouped_matmul_swiglu(x, w, gl, torch.zeros(4, 96, dtype=torch.float16, device=DEV))
    assert e.value.code == cabi.EINVAL


@pytest.mark.parametrize("rows", [0, 64, 80, 81, 100, 128, 300, 512])
def test_grouped_matmul_cluster_split_k_loose_row_bound(cabi, monkeypatch, rows):
    """One expert, a 512-row buffer, K = 8192: the cluster size is chosen for one m-tile of rows;
    clusters of m-tiles without rows leave at once, those with rows run as further waves.  The
    kernel reads the row count first and loads short activation tiles for up to 80 rows: the
    same products in the same order."""
    g = torch.Generator().manual_seed(rows + 5)
    x = torch.randn(512, 8192, generator=g).half()
    w_storage = (torch.randn(1, 512, 8192, generator=g) * 0.03).half()
    gl = torch.tensor([rows], dtype=torch.int64)
    want = oracle.grouped_matmul(x, w_storage.transpose(1, 2), gl)
    got = run_grouped_matmul(cabi, x, w_storage, gl, fill=9.0, split_k=True)
    close(got[:rows], want[:rows])
    assert (got[rows:] == 9.0).all()
    knob(monkeypatch, "B200OPS_GMM_SHORT", "0")
    assert torch.equal(run_grouped_matmul(cabi, x, w_storage, gl, fill=9.0, split_k=True), got)


def test_paged_attention_nz_layout_fast_and_general_paths_agree(cabi, monkeypatch):
    """The reference's own cache layout [blocks, Hkv*D/16, P, 16] at a 16-sequence slice of the
    benchmark batch with 16 query heads per kv head: TMA path, general path and the oracle."""
    w = wl.paged_attention_inputs(bs=16, heads=32, kv_heads=2, blocks=16 * 64, layout=wl.KV_LAYOUT_NZ, seed=13)
    knob(monkeypatch, "B200OPS_PA_MODE", "1")
    fast = run_paged_attention(cabi, w)
    knob(monkeypatch, "B200OPS_PA_MODE", "2")
    general = run_paged_attention(cabi, w)
    knob(monkeypatch, "B200OPS_PA_MODE", None)
    close(fast, general)
    close(fast, oracle.paged_attention(w["q"], w["key_cache"], w["value_cache"], w["block_tables"],
                                       w["context_lens"]))


@pytest.mark.parametrize("m,k,n", [(128, 128, 128), (257, 256, 256), (32, 4096, 6144), (3000, 512, 768)])
def test_dense_matmul_api(ops, m, k, n):
    """The dense NT product of the reference's earlier interface (benchmark/test_matmul.py: seed 0,
    x [m, k] and w [n, k] ~ N(0, 1), atol = rtol = 1e-3 there against an fp16 torch product; here
    against the fp32-accumulated product, with the operator tolerance)."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(m, k, generator=g).half()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).half()
    y = ops.matmul(x.to(DEV), w.to(DEV)).cpu()
    close(y, (x.float() @ w.float().T).half())
    with pytest.raises(RuntimeError):
        ops.matmul(x.to(DEV), w.to(DEV)[:, : k // 2])


@pytest.mark.parametrize("page", [16, 32])
@pytest.mark.parametrize("chunk", ["", "64", "1000"])
def test_paged_attention_small_pages_take_the_tma_path(cabi, monkeypatch, page, chunk):
    """Pages shorter than the 64-token tile (the common 16 and 32): a tile is assembled from 4 or 2
    pages.  NaN in every cache token no sequence owns; TMA path against the general path and the
    oracle; chunk lengths that are and are not multiples of the tile."""
    if chunk:
        knob(monkeypatch, "B200OPS_PA_CHUNK_TOKENS", chunk)
    lens = [1, 15, 16, 17, 63, 64, 65, 100, 1000, 4097, 0, 2500, page * 3]
    blocks = sum((l + page - 1) // page for l in lens) + 5
    w = wl.paged_attention_inputs(heads=28, kv_heads=4, block_size=page, context_lens=lens, blocks=blocks,
                                  seed=page + len(chunk))
    w = poison_unused(w)
    want = oracle.paged_attention(w["q"], w["key_cache_clean"], w["value_cache_clean"],
                                  w["block_tables"], w["context_lens"])
    knob(monkeypatch, "B200OPS_PA_MODE", "1")
    fast = run_paged_attention(cabi, w)
    knob(monkeypatch, "B200OPS_PA_MODE", "2")
    general = run_paged_attention(cabi, w)
    close(fast, want)
    close(general, want)


@pytest.mark.parametrize("layout", [wl.KV_LAYOUT_NHD, wl.KV_LAYOUT_NZ])
def test_paged_attention_wide_block_table_and_long_sequences(cabi, monkeypatch, layout):
    """A block table padded far beyond the contexts (as a graph-replaying host passes it) and
    sequences long enough that the chunk count per sequence is capped, so that they take longer
    chunks than the short ones in the same batch.  TMA path, general path and oracle."""
    knob(monkeypatch, "B200OPS_PA_CHUNK_TOKENS", "128")  # small base chunk: the cap engages early
    lens = [40000, 1, 129, 5000, 0, 128 * 8 * 7 + 3, 20011]
    page = 128
    blocks = sum((l + page - 1) // page for l in lens) + 4
    w = wl.paged_attention_inputs(heads=16, kv_heads=2, block_size=page, context_lens=lens, blocks=blocks,
                                  layout=layout, seed=41)
    wide = torch.zeros(len(lens), 2048, dtype=torch.int32)  # capacity 262144 tokens
    wide[:, : w["block_tables"].shape[1]] = w["block_tables"]
    want = oracle.paged_attention(w["q"], w["key_cache"], w["value_cache"], w["block_tables"], w["context_lens"])
    w = dict(w, block_tables=wide)
    knob(monkeypatch, "B200OPS_PA_MODE", "1")
    fast = run_paged_attention(cabi, w)
    knob(monkeypatch, "B200OPS_PA_MODE", "2")
    general = run_paged_attention(cabi, w)
    close(fast, want)
    close(general, want)


# ---------------------------------------------------------------------------------------
# Benchmark-size grouped GEMMs, the repeated-slot rule, invalid block-table entries, matmul
def _sampled_rows(ends, per_group=32):
    """First, last and evenly spaced rows of every non-empty group, with their expert."""
    rows, experts, lo = [], [], 0
    for e, hi in enumerate(ends):
        if hi > lo:
            pick = sorted(set([lo, hi - 1] + [lo + (hi - lo) * i // per_group for i in range(per_group)]))
            rows.extend(pick)
            experts.extend([e] * len(pick))
        lo = hi
    return rows, experts


@pytest.mark.parametrize("which,k,n,seed", [("gate_up", 4096, 28672, 4), ("down", 14336, 4096, 5)])
def test_grouped_matmul_benchmark_size(cabi, which, k, n, seed):
    """The two grouped GEMMs at the size the benchmark times (8192 rows in 8 skewed groups, weight
    tensors of 0.9 and 0.5 G elements): at least 256 rows spread over every group, the first and
    the last row of each group among them, against the fp32 product of the same fp16 operands
    (tolerance convention of the reference's own check, benchmark/test_grouped_matmul.py:52-60:
    assert_close on the fp16 result; rtol 1e-2 / atol 1e-3 as for every fp16 operator here)."""
    w = wl.grouped_matmul_inputs(rows=8192, k=k, n=n, seed=seed)
    y = run_grouped_matmul(cabi, w["x"], w["w_storage"], w["group_list"])
    rows, experts = _sampled_rows(w["group_list"].tolist())
    assert len(rows) >= 256
    x32 = w["x"][rows].float()
    want = torch.empty(len(rows), n)
    for e in sorted(set(experts)):
        sel = [i for i, ee in enumerate(experts) if ee == e]
        want[sel] = x32[sel] @ w["w_storage"][e].float().T
    close(y[rows], want.half())
    assert torch.isfinite(y.float()).all()


@pytest.mark.parametrize("layout", [wl.KV_LAYOUT_NHD, wl.KV_LAYOUT_NZ])
@pytest.mark.parametrize("tokens,hkv,d", [(2048, 8, 128), (23, 2, 64), (9, 1, 24), (40, 3, 40), (7, 1, 12), (2047, 4, 128)])
def test_reshape_and_cache_repeated_slot_keeps_the_later_token(cabi, layout, tokens, hkv, d):
    """The reference walks the tokens in order (reshape_and_cache_ex.cpp:47-61), so when several
    tokens name one slot the last of them stays.  Every kernel form (row per warp, 16-byte
    vectors, single elements) is covered by the head sizes."""
    if layout == wl.KV_LAYOUT_NZ and (hkv * d) % 16 != 0:
        pytest.skip("the NZ cache holds rows in chunks of 16 elements")
    blocks, p = 12, 16
    c = wl.reshape_and_cache_inputs(tokens, hkv, d, blocks=max(blocks, tokens // p + 2), block_size=p,
                                    layout=layout, seed=tokens)
    slots = c["slot_indices"].clone()
    g = torch.Generator().manual_seed(tokens + d)
    dup = torch.randperm(tokens, generator=g)[: max(2, tokens // 3)]
    slots[dup] = int(slots[dup[0]])     # a third of the batch piles onto one slot ...
    slots[tokens // 2] = int(slots[0])  # ... and one more pair
    last = {}
    for t, s_ in enumerate(slots.tolist()):
        last[s_] = t
    keep = torch.tensor([last[s_] == t for t, s_ in enumerate(slots.tolist())])
    only_last = torch.where(keep, slots, torch.full_like(slots, -1))
    kc = torch.full(c["cache_shape"], 3.0, dtype=torch.float16)
    vc = torch.full(c["cache_shape"], 4.0, dtype=torch.float16)
    ekc, evc = kc.clone(), vc.clone()
    oracle.reshape_and_cache(c["key"], ekc, only_last, c["value"], evc, layout=layout)
    kd, vd = kc.to(DEV), vc.to(DEV)
    cabi.reshape_and_cache(c["key"].to(DEV), c["value"].to(DEV), kd, vd, slots.to(DEV), layout)
    torch.cuda.synchronize()
    assert torch.equal(kd.cpu(), ekc) and torch.equal(vd.cpu(), evc)


@pytest.mark.parametrize("layout,page", [(wl.KV_LAYOUT_NHD, 128), (wl.KV_LAYOUT_NHD, 16), (wl.KV_LAYOUT_NZ, 64)])
def test_paged_attention_invalid_block_table_entry_is_left_out(cabi, monkeypatch, layout, page):
    """A block-table entry outside [0, num_pages) inside a sequence's context names no page: its
    tokens take no part, on the TMA path and on the general path alike.  Expected value: the
    same sequence with that page removed from its table."""
    lens = [5 * page + 7, 3 * page, 9 * page + 1]
    w = wl.paged_attention_inputs(heads=8, kv_heads=2, block_size=page, context_lens=lens, blocks=40, seed=page,
                                  layout=layout)
    bad = w["block_tables"].clone()
    bad[0, 2] = -1
    bad[1, 0] = 40          # == num_pages
    bad[2, 4] = 1 << 30
    ref_table = w["block_tables"].clone()
    ref_lens = w["context_lens"].clone()
    for b, col in ((0, 2), (1, 0), (2, 4)):
        ref_table[b, col:-1] = w["block_tables"][b, col + 1:]
        ref_lens[b] -= page
    want = oracle.paged_attention(w["q"], w["key_cache"], w["value_cache"], ref_table, ref_lens)
    w_bad = dict(w, block_tables=bad)
    knob(monkeypatch, "B200OPS_PA_MODE", "1")
    fast = run_paged_attention(cabi, w_bad)
    knob(monkeypatch, "B200OPS_PA_MODE", "2")
    general = run_paged_attention(cabi, w_bad)
    close(fast, want)
    close(general, want)


@pytest.mark.parametrize("m,k,n", [(128, 128, 128), (256, 4096, 6144), (1, 64, 64), (37, 100, 72), (300, 257, 65),
                                   (5, 8, 3), (2100, 512, 768)])
def test_matmul_c_abi_any_shape(cabi, m, k, n):
    """b200ops_matmul replaces the reference's matmul_impl (_csrc/ffi.cpp:71-75), which takes any
    m, n, k (its multiple-of-64 check is commented out, :423-424): tensor-core path for k and n
    multiples of 64, plain tiled kernel otherwise; same torch golden as benchmark/test_matmul.py."""
    g = torch.Generator().manual_seed(m + k + n)
    x = torch.randn(m, k, generator=g).half()
    w = (torch.randn(n, k, generator=g) * 0.1).half()
    y = torch.full((m, n), float("nan"), dtype=torch.float16, device=DEV)
    cabi.matmul(x.to(DEV), w.to(DEV), y)
    torch.cuda.synchronize()
    assert cabi.pipeline_status() == 0
    close(y.cpu(), (x.float() @ w.float().T).half())


@pytest.mark.parametrize("counts,k,n", [
    ([350, 340, 410], 14336, 4096),      # 160 tiles on 148 SMs: the 12 tiles of the second wave are cut in four
    ([380, 390, 400], 14336, 4096),      # 176 tiles: 28 cut
    ([200] * 4, 14336, 4096),            # 128 tiles, nearly a full wave: cutting would save too little, stays whole
    ([64] * 8, 14336, 4096),             # decode down projection: one m-tile per expert, stays whole
    ([40, 0, 3, 90, 7, 64, 1, 128], 8192, 1024),  # fewer tiles than half the SMs, long k: split-K proper
    ([200, 100], 8192, 320),             # N tail (320 = 256 + 64) in cut tiles
    ([1024], 1024, 256 * 146),           # 7.9 waves of a short k: stays whole
])
def test_grouped_matmul_balanced_schedule(cabi, counts, k, n):
    """With a workspace the kernel cuts the (tile, k-block) units into equal ranges per SM; tiles
    cut by a range boundary are summed from partial tiles.  Against the oracle, and against the
    same call without a workspace (tile by tile): the two may differ in the last bit only."""
    g = torch.Generator().manual_seed(sum(counts) + k)
    m = sum(counts)
    x = torch.randn(m, k, generator=g).half()
    w_storage = (torch.randn(len(counts), n, k, generator=g) * 0.03).half()
    gl = torch.tensor(counts).cumsum(0).to(torch.int64)
    assert cabi.grouped_matmul_workspace_size(m, k, len(counts), n) > 0
    balanced = run_grouped_matmul(cabi, x, w_storage, gl, fill=5.0)
    by_tiles = run_grouped_matmul(cabi, x, w_storage, gl, fill=5.0, split_k=False)
    again = run_grouped_matmul(cabi, x, w_storage, gl, fill=5.0)
    assert torch.equal(balanced, again)  # repeatable bit for bit
    close(balanced, by_tiles)
    rows, experts = _sampled_rows(gl.tolist(), per_group=24)
    want = torch.stack([x[r].float() @ w_storage[e].float().T for r, e in zip(rows, experts)])
    close(balanced[rows], want.half())


@pytest.mark.parametrize("counts,k,d", [([300] * 3, 14336, 1024), ([64] * 8, 4096, 2048), ([1, 127, 129], 8192, 640)])
def test_grouped_matmul_swiglu_balanced_schedule(cabi, counts, k, d):
    """The fused gate/up form under the balanced schedule: the CTA that sums a cut tile applies
    SwiGLU to the rounded sums.  Against grouped_matmul followed by swiglu (whose 256-column
    tiles are cut at other k-blocks, so single sums may differ in the last bit) and the oracle."""
    g = torch.Generator().manual_seed(sum(counts) + d)
    m = sum(counts)
    x = torch.randn(m, k, generator=g).half().to(DEV)
    w = (torch.randn(len(counts), 2 * d, k, generator=g) * 0.03).half().to(DEV)
    gl = torch.tensor(counts).cumsum(0).to(torch.int64).to(DEV)
    nbytes = cabi.grouped_matmul_workspace_size(m, k, len(counts), 2 * d)
    assert nbytes > 0
    ws = torch.full((nbytes,), 0xCD, dtype=torch.uint8, device=DEV)
    fused = torch.full((m, d), float("nan"), dtype=torch.float16, device=DEV)
    cabi.grouped_matmul_swiglu(x, w, gl, fused, ws)
    h = torch.empty(m, 2 * d, dtype=torch.float16, device=DEV)
    cabi.grouped_matmul(x, w, gl, h, ws)
    two = torch.empty(m, d, dtype=torch.float16, device=DEV)
    cabi.swiglu(h, two)
    torch.cuda.synchronize()
    assert cabi.pipeline_status() == 0
    close(fused.cpu(), two.cpu())
    assert float((fused == two).float().mean()) > 0.9  # single roundings flip where the fp32 sums differ in the last bit
    want = oracle.swiglu(oracle.grouped_matmul(x.cpu(), w.cpu().transpose(1, 2), gl.cpu()))
    close(fused.cpu(), want)
