"""The CPU oracle against fixtures produced by the reference's own golden code
(tests/golden/make_golden.py).  Runs without a GPU."""
import numpy as np
import torch

from conftest import bits, f16
from oracle import decode_ops_oracle as oracle


def test_add_rms_norm_matches_reference_golden(golden):
    z = golden("add_rms_norm")
    for i in range(int(z["n"])):
        y, s = oracle.add_rms_norm(f16(z[f"x{i}"]), f16(z[f"r{i}"]), f16(z[f"w{i}"]), float(z[f"eps{i}"]))
        assert np.array_equal(bits(y), z[f"y{i}"])
        assert np.array_equal(bits(s), z[f"s{i}"])


def test_swiglu_matches_reference_golden(golden):
    z = golden("swiglu")
    for i in range(int(z["n"])):
        assert np.array_equal(bits(oracle.swiglu(f16(z[f"x{i}"]))), z[f"y{i}"])


def test_grouped_matmul_matches_reference_golden(golden):
    # The reference golden multiplies in fp16 on CPU and asserts atol = rtol = 1e-3
    # (benchmark/test_grouped_matmul.py:60); the oracle accumulates in fp32.
    z = golden("grouped_matmul")
    for i in range(int(z["n"])):
        w = f16(z[f"w{i}"]).transpose(1, 2)
        y = oracle.grouped_matmul(f16(z[f"x{i}"]), w, torch.from_numpy(z[f"gl{i}"]))
        torch.testing.assert_close(y, f16(z[f"y{i}"]), atol=1e-3, rtol=1e-3)


def test_rope_matches_reference_golden(golden):
    z = golden("rope")
    for i in range(int(z["n"])):
        args = (f16(z[f"q{i}"]), f16(z[f"k{i}"]), torch.from_numpy(z[f"pos{i}"]),
                f16(z[f"cos{i}"]), f16(z[f"sin{i}"]))
        oq, ok = oracle.rope(*args)
        # fn_naive evaluated in fp32 on the same fp16 inputs, rounded once: bit-exact.
        assert np.array_equal(bits(oq), bits(torch.from_numpy(z[f"oq32_{i}"]).half()))
        assert np.array_equal(bits(ok), bits(torch.from_numpy(z[f"ok32_{i}"]).half()))
        # fn_naive as the reference runs it (fp16 arithmetic, three roundings).
        torch.testing.assert_close(oq, f16(z[f"oq{i}"]), atol=1e-3, rtol=1e-2)
        torch.testing.assert_close(ok, f16(z[f"ok{i}"]), atol=1e-3, rtol=1e-2)


def test_cos_sin_cache_recipe():
    cos, sin = oracle.cos_sin_cache(64, 128)
    assert cos.shape == (64, 64) and cos.dtype == torch.float16
    assert float(cos[0, 0]) == 1.0 and float(sin[0, 0]) == 0.0
    assert abs(float(cos[1, 0]) - 0.5403) < 1e-3


def _sparse_expect(shape, idx, vals):
    flat = np.zeros(int(np.prod(shape)), dtype=np.uint16)
    flat[idx] = vals
    return flat


def test_reshape_and_cache_reference_case(golden):
    """The reference script's own case: seed 42, slots [6,134,212,290], cache [583,64,128,16]."""
    z = golden("reshape_and_cache")
    shape = tuple(int(v) for v in z["shape0"])
    kc = torch.zeros(shape, dtype=torch.float16)
    vc = torch.zeros(shape, dtype=torch.float16)
    oracle.reshape_and_cache(f16(z["key0"]), kc, torch.from_numpy(z["slots0"]), f16(z["value0"]), vc)
    assert np.array_equal(bits(kc).reshape(-1), _sparse_expect(shape, z["idx0"], z["kc0"]))
    assert np.array_equal(bits(vc).reshape(-1), _sparse_expect(shape, z["idx0"], z["vc0"]))
    # key-only form: the value cache stays untouched
    kc = torch.zeros(shape, dtype=torch.float16)
    vc = torch.zeros(shape, dtype=torch.float16)
    oracle.reshape_and_cache(f16(z["key1"]), kc, torch.from_numpy(z["slots1"]), None, vc)
    assert np.array_equal(bits(kc).reshape(-1), _sparse_expect(shape, z["idx1"], z["kc1"]))
    assert not vc.any()


def test_reshape_and_cache_small_dense_case(golden):
    z = golden("reshape_and_cache")
    shape = tuple(int(v) for v in z["shape2"])
    kc = torch.zeros(shape, dtype=torch.float16)
    vc = torch.zeros(shape, dtype=torch.float16)
    oracle.reshape_and_cache(f16(z["key2"]), kc, torch.from_numpy(z["slots2"]), f16(z["value2"]), vc)
    assert np.array_equal(bits(kc), z["kc2_dense"])
    assert np.array_equal(bits(vc), z["vc2_dense"])


def test_reshape_and_cache_skips_invalid_slots_and_nhd_layout():
    g = torch.Generator().manual_seed(0)
    key = torch.randn(5, 2, 32, generator=g).half()
    val = torch.randn(5, 2, 32, generator=g).half()
    slots = torch.tensor([3, -1, 40, 39, 7], dtype=torch.int32)  # 40 is out of range (capacity 40)
    kc = torch.zeros(5, 8, 2, 32, dtype=torch.float16)
    vc = torch.zeros_like(kc)
    oracle.reshape_and_cache(key, kc, slots, val, vc)
    flat = kc.view(40, 2, 32)
    for t, s in enumerate(slots.tolist()):
        if 0 <= s < 40:
            assert torch.equal(flat[s], key[t])
    assert int((flat.abs().sum((1, 2)) > 0).sum()) == 3


def test_paged_attention_layouts_agree_and_match_dense_softmax():
    g = torch.Generator().manual_seed(1)
    bs, hq, hkv, d, p, pages = 3, 8, 2, 64, 16, 12
    lens = torch.tensor([37, 1, 64], dtype=torch.int32)
    k_nhd = torch.randn(pages, p, hkv, d, generator=g).half()
    v_nhd = torch.randn(pages, p, hkv, d, generator=g).half()
    table = torch.tensor([[5, 2, 9, 0], [7, 0, 0, 0], [1, 3, 4, 6]], dtype=torch.int32)
    q = torch.randn(bs, hq, d, generator=g).half()
    out = oracle.paged_attention(q, k_nhd, v_nhd, table, lens)
    # NZ copies of the same caches: [pages, Hkv*D/16, P, 16]
    to_nz = lambda c: c.reshape(pages, p, hkv * d // 16, 16).permute(0, 2, 1, 3).contiguous()
    out_nz = oracle.paged_attention(q, to_nz(k_nhd), to_nz(v_nhd), table, lens)
    assert torch.equal(out, out_nz)
    # dense check for sequence 0, head 5 (kv head 1)
    L = 37
    toks = torch.cat([k_nhd[pg] for pg in table[0, :3].tolist()])[:L, 1].float()
    vals = torch.cat([v_nhd[pg] for pg in table[0, :3].tolist()])[:L, 1].float()
    s = (q[0, 5].float() @ toks.T) / 8.0
    ref = torch.softmax(s, 0) @ vals
    torch.testing.assert_close(out[0, 5].float(), ref, atol=1e-3, rtol=1e-2)


def test_c_oracle_agrees_with_python_oracle():
    """oracle/reshape_and_cache_oracle.c (plain C) against the torch restatement."""
    import ctypes
    import subprocess
    from pathlib import Path

    odir = Path(oracle.__file__).resolve().parent
    subprocess.run(["make", "-s", "-C", str(odir)], check=True)
    lib = ctypes.CDLL(str(odir / "liboracle.so"))
    g = torch.Generator().manual_seed(3)
    key = torch.randn(40, 4, 32, generator=g).half()
    val = torch.randn(40, 4, 32, generator=g).half()
    slots = torch.randperm(8 * 16, generator=g)[:40].int()
    slots[5], slots[6] = -3, 8 * 16
    for nhd, shape in ((1, (8, 16, 4, 32)), (0, (8, 8, 16, 16))):
        kc = torch.zeros(shape, dtype=torch.float16)
        vc = torch.zeros(shape, dtype=torch.float16)
        ek, ev = kc.clone(), vc.clone()
        oracle.reshape_and_cache(key, ek, slots, val, ev, oracle.KV_LAYOUT_NHD if nhd else oracle.KV_LAYOUT_NZ)
        P = shape[1] if nhd else shape[2]
        C = 0 if nhd else shape[1]
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        lib.oracle_reshape_and_cache(p(key), p(val), p(kc), p(vc), p(slots), ctypes.c_int64(40),
                                     ctypes.c_int64(128), ctypes.c_int64(8), ctypes.c_int64(C),
                                     ctypes.c_int64(P), ctypes.c_int(nhd))
        assert np.array_equal(bits(kc), bits(ek)) and np.array_equal(bits(vc), bits(ev))


def test_head_rms_norm_is_add_rms_norm_without_residual():
    """The per-head q/k normalisation is pinned through the add_rms_norm golden: with a zero
    residual both must give the same bits, row by row (one head per row)."""
    g = torch.Generator().manual_seed(9)
    x = torch.randn(7, 5, 128, generator=g).half()
    w = (1 + 0.1 * torch.randn(128, generator=g)).half()
    got = oracle.head_rms_norm(x, w, 1e-6)
    want, _ = oracle.add_rms_norm(x.view(-1, 128), torch.zeros(35, 128, dtype=torch.float16), w, 1e-6)
    assert torch.equal(got.view(-1, 128), want)


def test_paged_attention_oracle_against_an_independent_statement():
    """The attention oracle has no reference golden to pin it (the reference's kernel is
    unfinished and its check calls a third-party NPU library), so this does not pin it either.
    It removes one risk: that oracle and kernel share one author's misreading.  A second
    statement of decode attention written differently -- gather each sequence's pages into a
    dense [kv_heads, L, D] tensor and call torch's scaled_dot_product_attention in fp32 with
    grouped-query broadcasting -- must agree with the oracle on the benchmark recipe (64
    sequences, 28 query / 4 kv heads, lengths U[512, 8192], random distinct pages), on both
    cache layouts."""
    import torch.nn.functional as F

    import decode_workloads as wl
    from oracle import decode_ops_oracle as oracle

    for layout in (wl.KV_LAYOUT_NHD, wl.KV_LAYOUT_NZ):
        w = wl.paged_attention_inputs(blocks=2400, layout=layout, seed=3)
        got = oracle.paged_attention(w["q"], w["key_cache"], w["value_cache"], w["block_tables"],
                                     w["context_lens"])
        kc, vc = w["key_cache"], w["value_cache"]
        if layout == wl.KV_LAYOUT_NZ:  # [pages, Hkv*D/16, P, 16] -> [pages, P, Hkv, D]
            pages, chunks, p, _ = kc.shape
            kc = kc.permute(0, 2, 1, 3).reshape(pages, p, 4, 128)
            vc = vc.permute(0, 2, 1, 3).reshape(pages, p, 4, 128)
        want = torch.empty_like(w["q"])
        for b in range(w["q"].shape[0]):
            n = int(w["context_lens"][b])
            ids = w["block_tables"][b, : (n + 127) // 128].long()
            k = kc[ids].reshape(-1, 4, 128)[:n].permute(1, 0, 2).float()   # [Hkv, L, D]
            v = vc[ids].reshape(-1, 4, 128)[:n].permute(1, 0, 2).float()
            q = w["q"][b].float()[:, None, :]                              # [Hq, 1, D]
            o = F.scaled_dot_product_attention(q[None], k[None], v[None], enable_gqa=True)
            want[b] = o[0, :, 0, :].half()
        torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=1e-3)
