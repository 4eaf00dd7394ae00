"""Puts the unmodified reference (CodeMan62/lily) under ``baseline/_ref`` for ``bench.py --impl reference``.

    python baseline/install_reference.py [SOURCE_CHECKOUT]

Without an argument the checkout is looked for in ``$LILY_REFERENCE_SRC`` and then in a folder
named ``reference`` beside this repository.

First the offline ``pip install --target baseline/_ref`` is tried.  The reference's build backend
(hatchling) is not among the offline wheels, so that fails here; the fallback then does by hand what
that backend would do for this project, whose ``pyproject.toml`` says
``[tool.hatch.build.targets.wheel] packages = ["lily"]``: the ``lily`` package tree, with its
``csrc`` folder of CUDA sources, is copied as it is.  Nothing is edited.  What happened is written to
``baseline/_ref/INSTALL.txt``.

With ``--prebuild`` the reference's own CUDA extension is also compiled for sm_100 by its own loader
(``LILY_CUDA_BUILD_ONLY=1``, lily/layers/quantization/cuda_ops.py:39-65) into
``baseline/_ref/_cuda_build``, so that the benchmark box has less to compile.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
WHEELHOUSE = os.environ.get("LILY_WHEELHOUSE", "/opt/wheelhouse")


def find_source(given: Optional[str] = None) -> Optional[str]:
    candidates = [given, os.environ.get("LILY_REFERENCE_SRC"),
                  os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in candidates:
        if c and os.path.isfile(os.path.join(c, "lily", "engine.py")):
            return os.path.abspath(c)
    return None


def installed() -> bool:
    return os.path.isfile(os.path.join(DEST, "lily", "engine.py"))


def _pip(source: str) -> str:
    """The offline install as an installer would run it; returns "" on success, else the last line of its output."""
    with tempfile.TemporaryDirectory() as tmp:
        copy = os.path.join(tmp, "src")                  # the build may write into the tree: give it a copy
        shutil.copytree(source, copy, ignore=shutil.ignore_patterns(".git", "__pycache__"))
        for extra in ([], ["--no-deps"]):
            cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--find-links",
                   WHEELHOUSE, "--target", DEST, *extra, copy]
            try:
                done = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
            except (OSError, subprocess.TimeoutExpired) as exc:
                return f"{type(exc).__name__}: {exc}"
            if done.returncode == 0 and installed():
                return ""
        lines = [ln.strip() for ln in (done.stdout + done.stderr).splitlines() if ln.strip()]
        errors = [ln for ln in lines if "Error" in ln or "error:" in ln.lower()]
        return (errors or lines or [f"pip exited with {done.returncode}"])[-1]


def install(source: Optional[str] = None, force: bool = False) -> str:
    """Returns a one-line account of how the reference got to ``baseline/_ref`` (raises if it did not)."""
    note_path = os.path.join(DEST, "INSTALL.txt")
    if installed() and not force:
        return open(note_path).read().strip() if os.path.isfile(note_path) else "already present"
    src = find_source(source)
    if src is None:
        raise FileNotFoundError("no checkout of the reference found (argument, $LILY_REFERENCE_SRC, ../reference)")
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    os.makedirs(DEST)
    problem = _pip(src)
    if problem:
        if os.path.isdir(DEST):
            shutil.rmtree(DEST)
        os.makedirs(DEST)
        shutil.copytree(os.path.join(src, "lily"), os.path.join(DEST, "lily"),
                        ignore=shutil.ignore_patterns("__pycache__"))
        note = f"pip install failed ({problem}); copied the lily package tree unchanged, as its wheel would hold it"
    else:
        note = "pip install --target succeeded"
    with open(note_path, "w") as f:
        f.write(note + "\n")
    return note


def prebuild_cuda() -> str:
    """Compiles the reference's CUDA extension with the reference's own loader, without a GPU."""
    env = dict(os.environ, LILY_CUDA_BUILD_ONLY="1", TORCH_CUDA_ARCH_LIST="10.0",
               LILY_CUDA_BUILD_DIR=os.path.join(DEST, "_cuda_build"), PYTHONPATH=DEST, HF_HUB_OFFLINE="1")
    code = ("from lily.layers.quantization import cuda_ops as c; import sys; "
            "sys.exit(0 if c.available() else 1)")
    done = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=3600)
    tail = [ln for ln in (done.stderr + done.stdout).splitlines() if ln.strip()][-1:] or [""]
    if done.returncode == 0:
        # ninja rebuilds when the sources' paths change: remember under which name of this folder they were compiled
        with open(os.path.join(DEST, "_cuda_build", "BUILT_AT"), "w") as f:
            f.write(DEST + "\n")
        return "built"
    return f"not built: {tail[0]}"


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(install(args[0] if args else None, force="--force" in sys.argv))
    if "--prebuild" in sys.argv:
        print("cuda extension:", prebuild_cuda())
