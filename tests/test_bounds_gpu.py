"""Out-of-bounds guard: every operator writes its outputs into the middle of a larger buffer
whose margins hold a canary pattern; the margins must be intact afterwards."""
import ctypes

import pytest
import torch

from conftest import knob

import decode_workloads as wl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GUARD = 4096  # halfs on each side
CANARY = 0x7B3C  # an ordinary fp16 bit pattern unlikely to be produced by accident


class Guarded:
    """A tensor carved out of a canary-filled buffer."""

    def __init__(self, shape, dtype=torch.float16):
        n = 1
        for s in shape:
            n *= s
        self.raw = torch.full((n + 2 * GUARD,), CANARY, dtype=torch.int16, device=DEV)
        self.t = self.raw[GUARD:GUARD + n].view(dtype).view(shape)
        self.n = n

    def intact(self):
        return bool((self.raw[:GUARD] == CANARY).all()) and bool((self.raw[GUARD + self.n:] == CANARY).all())


def test_elementwise_ops_stay_inside_their_outputs(cabi):
    d = wl.add_rms_norm_inputs(37, 1088, seed=1)
    y, s = Guarded((37, 1088)), Guarded((37, 1088))
    cabi.add_rms_norm(d["x"].to(DEV), d["residual"].to(DEV), d["weight"].to(DEV), 1e-6, y.t, s.t)
    x = wl.swiglu_inputs(19, 96)["x"].to(DEV)
    o = Guarded((19, 96))
    cabi.swiglu(x, o.t)
    r = wl.rope_inputs(23, 5, 3, 64, 0, 100, seed=2)
    oq, ok = Guarded((23, 5, 64)), Guarded((23, 3, 64))
    cabi.rope(r["q"].to(DEV), r["k"].to(DEV), r["position_ids"].to(DEV), r["cos_cache"].to(DEV),
              r["sin_cache"].to(DEV), oq.t, ok.t)
    torch.cuda.synchronize()
    for g in (y, s, o, oq, ok):
        assert g.intact()
        assert not bool((g.t.view(torch.int16) == CANARY).all())  # and the output itself was written


@pytest.mark.parametrize("layout", [wl.KV_LAYOUT_NHD, wl.KV_LAYOUT_NZ])
def test_reshape_and_cache_stays_inside_the_caches(cabi, layout):
    c = wl.reshape_and_cache_inputs(33, 2, 64, 5, 16, layout, seed=3)
    slots = c["slot_indices"].clone()
    slots[0], slots[1], slots[2] = 79, 0, -1  # last slot, first slot, skipped
    kc, vc = Guarded(c["cache_shape"]), Guarded(c["cache_shape"])
    cabi.reshape_and_cache(c["key"].to(DEV), c["value"].to(DEV), kc.t, vc.t, slots.to(DEV), layout)
    torch.cuda.synchronize()
    assert kc.intact() and vc.intact()


def test_attention_and_gemm_stay_inside_their_outputs(cabi):
    a = wl.paged_attention_inputs(heads=28, kv_heads=4, context_lens=[700, 1, 2049, 128, 0], blocks=30, seed=4)
    q = a["q"].to(DEV)
    out = Guarded(tuple(q.shape))
    n = cabi.paged_attention_workspace_size(q.shape[0], 28, 4, 128, 128, a["block_tables"].shape[1])
    ws = Guarded((n // 2,))
    cabi.paged_attention(q, a["key_cache"].to(DEV), a["value_cache"].to(DEV), a["block_tables"].to(DEV),
                         a["context_lens"].to(DEV), out.t, 4, 128, wl.KV_LAYOUT_NHD, ws.t.view(torch.uint8))
    g = wl.grouped_matmul_inputs(rows=301, k=256, n=320, experts=5, seed=6)
    y = Guarded((301, 320))
    cabi.grouped_matmul(g["x"].to(DEV), g["w_storage"].to(DEV), g["group_list"].to(DEV), y.t)
    # split-K: partial tiles and counters must stay inside the workspace
    g2 = wl.grouped_matmul_inputs(rows=70, k=8192, n=256, experts=1, seed=7)
    nb = cabi.grouped_matmul_workspace_size(70, 8192, 1, 256)
    assert nb > 0
    ws2, y2 = Guarded((nb // 2,)), Guarded((70, 256))
    cabi.grouped_matmul(g2["x"].to(DEV), g2["w_storage"].to(DEV), g2["group_list"].to(DEV), y2.t,
                        ws2.t.view(torch.uint8))
    torch.cuda.synchronize()
    assert cabi.pipeline_status() == 0
    for buf in (out, ws, y, ws2, y2):
        assert buf.intact()


@pytest.mark.parametrize("ksplit", ["1", "0"])  # cluster split-K / split-K through the workspace
def test_split_k_paths_stay_inside_their_outputs(cabi, monkeypatch, ksplit):
    knob(monkeypatch, "B200OPS_GMM_KSPLIT", ksplit)
    g2 = wl.grouped_matmul_inputs(rows=70, k=8192, n=320, experts=1, seed=7)
    nb = cabi.grouped_matmul_workspace_size(70, 8192, 1, 320)
    assert nb > 0
    ws2, y2 = Guarded((nb // 2,)), Guarded((70, 320))
    cabi.grouped_matmul(g2["x"].to(DEV), g2["w_storage"].to(DEV), g2["group_list"].to(DEV), y2.t,
                        ws2.t.view(torch.uint8))
    torch.cuda.synchronize()
    assert cabi.pipeline_status() == 0
    assert ws2.intact() and y2.intact()
    assert not bool((y2.t.view(torch.int16) == CANARY).all())


@pytest.mark.parametrize("pairs", ["0", "2"])  # single-CTA kernel / CTA-pair kernel
def test_pair_and_swiglu_epilogues_stay_inside_their_outputs(cabi, monkeypatch, pairs):
    knob(monkeypatch, "B200OPS_GMM_PAIR", pairs)
    g = wl.grouped_matmul_inputs(rows=301, k=256, n=384, experts=5, seed=6)
    x, w, gl = g["x"].to(DEV), g["w_storage"].to(DEV), g["group_list"].to(DEV)
    y, act = Guarded((301, 384)), Guarded((301, 192))
    cabi.grouped_matmul(x, w, gl, y.t)
    cabi.grouped_matmul_swiglu(x, w, gl, act.t)
    torch.cuda.synchronize()
    assert cabi.pipeline_status() == 0
    assert y.intact() and act.intact()
    assert not bool((act.t.view(torch.int16) == CANARY).all())


def test_print_info_reports_the_device(cabi):
    buf = ctypes.create_string_buffer(2048)
    cabi.check(cabi.load().b200ops_print_info(0, buf, 2048))
    text = buf.value.decode()
    assert "SMs:" in text and "L2:" in text and torch.cuda.get_device_name(0).split()[-1] in text
    assert cabi.load().b200ops_print_info(9999, None, 0) == cabi.ECUDA
