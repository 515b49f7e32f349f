"""Generate the golden fixtures in this directory by running the REFERENCE'S OWN golden code.

Run once where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

Nothing here is needed at test time: the tests read only the .npz files this script
writes.  The reference's golden functions are executed unmodified:
  * add_rms_norm_cpu, swiglu_cpu, reference_reshape_and_cache are imported from their
    `__main__`-guarded scripts (benchmark/test_add_rms_norm.py, test_swiglu.py,
    test_reshape_and_cache.py) with stub modules standing in for the Ascend-only imports;
  * grouped_matmul_ref (benchmark/test_grouped_matmul.py:6-23) and the nested fn_naive
    (benchmark/test_graph.py:347-367) sit in files that touch an NPU at import time, so their
    FunctionDef nodes are lifted out of the parsed source and compiled on their own.
fp16 arrays are stored as uint16 bit patterns so that comparisons can be bit-exact.
"""
from __future__ import annotations

import ast
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _stub_ascend_modules():
    for name in ("torch_npu", "ascend910a_extras", "ascend910a_extras.ops", "ascend910a_extras.graph"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["ascend910a_extras"].ops = sys.modules["ascend910a_extras.ops"]


def _import_script(path: Path):
    spec = importlib.util.spec_from_file_location("ref_" + path.stem, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _lift_function(path: Path, name: str):
    """Compile one (possibly nested) function definition of `path` by itself."""
    tree = ast.parse(path.read_text())
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == name:
            module = ast.Module(body=[node], type_ignores=[])
            ns = {"torch": torch}
            exec(compile(module, str(path), "exec"), ns)
            return ns[name]
    raise KeyError(f"{name} not found in {path}")


def bits(t: torch.Tensor) -> np.ndarray:
    assert t.dtype == torch.float16
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main(ref_root: Path):
    _stub_ascend_modules()
    bench = ref_root / "benchmark"
    add_rms_norm_cpu = _import_script(bench / "test_add_rms_norm.py").add_rms_norm_cpu
    swiglu_cpu = _import_script(bench / "test_swiglu.py").swiglu_cpu
    reference_reshape_and_cache = _import_script(
        bench / "test_reshape_and_cache.py").reference_reshape_and_cache
    grouped_matmul_ref = _lift_function(bench / "test_grouped_matmul.py", "grouped_matmul_ref")
    fn_naive = _lift_function(bench / "test_graph.py", "fn_naive")

    # ---- add_rms_norm: shapes incl. the minimum hidden size and a non-power-of-two one ----
    out = {}
    for i, (t, h, eps) in enumerate([(8, 256, 1e-6), (3, 64, 1e-5), (5, 1088, 1e-6)]):
        g = torch.Generator().manual_seed(100 + i)
        x = torch.randn(t, h, generator=g).half()
        r = torch.randn(t, h, generator=g).half()
        w = torch.randn(h, generator=g).half()
        y, s = add_rms_norm_cpu(x, r, w, eps)
        out.update({f"x{i}": bits(x), f"r{i}": bits(r), f"w{i}": bits(w), f"eps{i}": np.float32(eps),
                    f"y{i}": bits(y), f"s{i}": bits(s)})
    out["n"] = np.int64(3)
    np.savez_compressed(HERE / "add_rms_norm.npz", **out)

    # ---- swiglu: the reference script's width (2*192) and a wider one ----
    out = {}
    for i, (t, two_d) in enumerate([(16, 384), (4, 64), (3, 1280)]):
        g = torch.Generator().manual_seed(200 + i)
        x = (torch.randn(t, two_d, generator=g) * 3).half()
        out.update({f"x{i}": bits(x), f"y{i}": bits(swiglu_cpu(x))})
    out["n"] = np.int64(3)
    np.savez_compressed(HERE / "swiglu.npz", **out)

    # ---- grouped_matmul: small E with an empty group; w built as the reference script does ----
    out = {}
    for i, (m, k, n, counts) in enumerate([(96, 128, 64, [40, 0, 17, 39]), (70, 64, 192, [70]),
                                           (33, 192, 128, [1, 2, 30])]):
        g = torch.Generator().manual_seed(300 + i)
        x = torch.randn(m, k, generator=g).half()
        w_storage = (torch.randn(len(counts), n, k, generator=g) * 0.1).half()
        w = w_storage.transpose(1, 2)
        gl = torch.tensor(counts).cumsum(0).to(torch.int64)
        y = grouped_matmul_ref(x, w, gl)  # fp16 matmul on CPU, as in the reference script
        out.update({f"x{i}": bits(x), f"w{i}": bits(w_storage), f"gl{i}": gl.numpy(), f"y{i}": bits(y)})
    out["n"] = np.int64(3)
    np.savez_compressed(HERE / "grouped_matmul.npz", **out)

    # ---- rope: the reference test's head configuration with a short cos/sin table ----
    out = {}
    for i, (bs, hq, hkv, d, max_pos) in enumerate([(4, 32, 8, 128, 96), (3, 4, 1, 64, 40)]):
        g = torch.Generator().manual_seed(400 + i)
        inv_freq = 1.0 / (1000000 ** (torch.arange(0, d, 2).float() / d))
        freqs = torch.einsum("i,j->ij", torch.arange(max_pos, dtype=torch.float), inv_freq)
        cos, sin = freqs.cos().half().contiguous(), freqs.sin().half().contiguous()
        q = torch.randn(bs, hq, d, generator=g).half()
        k = torch.randn(bs, hkv, d, generator=g).half()
        pos = torch.randint(0, max_pos, (bs,), generator=g, dtype=torch.int32)
        oq, ok = fn_naive(q, k, pos.long(), cos, sin)  # fp16 arithmetic, as the reference runs it
        oq32, ok32 = fn_naive(q.float(), k.float(), pos.long(), cos.float(), sin.float())
        out.update({f"q{i}": bits(q), f"k{i}": bits(k), f"pos{i}": pos.numpy(), f"cos{i}": bits(cos),
                    f"sin{i}": bits(sin), f"oq{i}": bits(oq), f"ok{i}": bits(ok),
                    f"oq32_{i}": oq32.numpy(), f"ok32_{i}": ok32.numpy()})
    out["n"] = np.int64(2)
    np.savez_compressed(HERE / "rope.npz", **out)

    # ---- reshape_and_cache: the reference script's exact case (seed 42, slots 6/134/212/290,
    #      cache [583, 64, 128, 16]) stored sparsely, plus a small dense case ----
    out = {}
    torch.manual_seed(42)
    slots = torch.tensor([6, 134, 212, 290], dtype=torch.int32)
    key = torch.randn(4, 8, 128, dtype=torch.float16)
    value = torch.randn(4, 8, 128, dtype=torch.float16)
    shape = (583, 64, 128, 16)
    kc = torch.zeros(*shape, dtype=torch.float16)
    vc = torch.zeros(*shape, dtype=torch.float16)
    reference_reshape_and_cache(key, kc, slots, value, vc)
    kb, vb = bits(kc).reshape(-1), bits(vc).reshape(-1)
    touched = np.nonzero(kb | vb)[0]
    out.update({"key0": bits(key), "value0": bits(value), "slots0": slots.numpy(),
                "shape0": np.array(shape, dtype=np.int64), "idx0": touched.astype(np.int64),
                "kc0": kb[touched], "vc0": vb[touched]})
    key2 = torch.randn(4, 8, 128, dtype=torch.float16)
    kc2 = torch.zeros(*shape, dtype=torch.float16)
    reference_reshape_and_cache(key2, kc2, slots)  # key-only form
    kb2 = bits(kc2).reshape(-1)
    t2 = np.nonzero(kb2)[0]
    out.update({"key1": bits(key2), "slots1": slots.numpy(), "shape1": np.array(shape, dtype=np.int64),
                "idx1": t2.astype(np.int64), "kc1": kb2[t2]})
    g = torch.Generator().manual_seed(500)
    key3 = torch.randn(6, 2, 64, generator=g).half()
    value3 = torch.randn(6, 2, 64, generator=g).half()
    shape3 = (5, 8, 16, 16)
    slots3 = torch.tensor([79, 0, 17, 33, 64, 15], dtype=torch.int32)
    kc3 = torch.zeros(*shape3, dtype=torch.float16)
    vc3 = torch.zeros(*shape3, dtype=torch.float16)
    reference_reshape_and_cache(key3, kc3, slots3, value3, vc3)
    out.update({"key2": bits(key3), "value2": bits(value3), "slots2": slots3.numpy(),
                "shape2": np.array(shape3, dtype=np.int64), "kc2_dense": bits(kc3), "vc2_dense": bits(vc3)})
    np.savez_compressed(HERE / "reshape_and_cache.npz", **out)
    print("wrote", *sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <checkout of the reference project>")
    main(Path(sys.argv[1]))
