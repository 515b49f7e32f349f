"""The package installs with pip and imports from the installed copy with no path edits
(counterpart of the reference's `pip install -e .`, setup.py:122-176 / pyproject.toml:1-12)."""
import os
import shutil
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent


def test_pip_install_then_import_from_site_packages(tmp_path):
    site = tmp_path / "site"
    # pip builds inside the directory it is given: install from a copy so that the source tree
    # gets no build/ or egg-info folders (with second copies of the shared objects in them).
    # The copy keeps the tree's shape (the C header sits beside the package directory) and the
    # object files of the in-tree build, so an up-to-date tree installs without recompiling.
    src = tmp_path / "tree" / "ascend-ops_b200"
    shutil.copytree(REPO / "include", tmp_path / "tree" / "include")

    def leave_out(folder, names):
        if Path(folder).name == "build":  # keep the object files, not an earlier pip build
            return [n for n in names if n.startswith(("lib", "bdist"))]
        return [n for n in names if n.endswith(".egg-info") or n == "__pycache__"]

    shutil.copytree(REPO / "ascend-ops_b200", src, ignore=leave_out)
    r = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                        "--quiet", "--target", str(site), str(src)],
                       capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert (site / "ascend910a_extras" / "lib" / "libb200ops.so").exists()
    code = ("import ascend910a_extras, ascend910a_extras.ops as ops, moe_decode_layer, moe_parallel;"
            "from ascend910a_extras import cabi;"
            "assert cabi.load().b200ops_version() >= 200;"
            "print(ascend910a_extras.__file__)")
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    env["PYTHONPATH"] = str(site)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(tmp_path), env=env,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert str(site) in r.stdout  # the installed copy, not the source tree
