"""Builds ``oracle/_ref/``: the reference package itself, CPU path only, as a second checker (test infrastructure).

What it makes (all under ``oracle/_ref/``, which git ignores; nothing of it is product code):

* ``site/falkon/...``  -- the reference installed by pip from a scratch copy of its checkout, with
  ``NO_BUILD_EXT=1`` (pure Python; the reference's own switch for "do not compile at install time");
* ``site/falkon/c_ext/_C.so`` -- the reference's C++ extension, CPU sources only, compiled from the sources where
  they lie in the checkout by the reference's own JIT recipe (``falkon/c_ext/_backend.py``: torch's cpp_extension
  ``load`` over ``ops/cpu/*.cpp``, ``ops/autograd/*.cpp``, ``ops/*.cpp``, ``*.cpp``) with ``nvcc`` hidden from
  PATH, so that neither CUDA sources nor CUDA libraries enter the build.

With it ``import falkon`` works from ``oracle/_ref/site`` on a machine that has no reference checkout (the
built tree travels with the repository snapshot), and the tests / ``bench.py --impl reference`` can run the
reference's own ``Kernel.mmv`` / ``Kernel.dmmv`` / ``FalkonConjugateGradient`` with
``FalkonOptions(use_cpu=True, keops_active="no")``.

Usage:  python oracle/build_ref.py [--src <reference checkout>] [--force]
The checkout is looked for in $FALKON_REFERENCE_SRC, else in a directory ``reference`` beside the repository.
"""
import argparse
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF_DIR = os.path.join(HERE, "_ref")
SITE_DIR = os.path.join(REF_DIR, "site")


def default_source() -> str:
    return os.environ.get("FALKON_REFERENCE_SRC") or os.path.join(os.path.dirname(ROOT), "reference")


def site_dir() -> str:
    return SITE_DIR


def is_built() -> bool:
    return os.path.exists(os.path.join(SITE_DIR, "falkon", "c_ext", "_C.so"))


def _env_without_nvcc() -> dict:
    env = dict(os.environ)
    keep = [p for p in env.get("PATH", "").split(os.pathsep) if p and not os.path.exists(os.path.join(p, "nvcc"))]
    env["PATH"] = os.pathsep.join(keep)
    return env


def build_ref(src: str = None, force: bool = False, verbose: bool = True) -> str:
    """Returns the directory to put on sys.path.  Raises RuntimeError with the failing step's output."""
    src = src or default_source()
    if is_built() and not force:
        return SITE_DIR
    if not os.path.isdir(os.path.join(src, "falkon")):
        raise RuntimeError(f"no reference checkout at {src}")
    if os.path.isdir(REF_DIR):
        shutil.rmtree(REF_DIR)
    os.makedirs(SITE_DIR)
    with tempfile.TemporaryDirectory(prefix="flk_ref_") as tmp:
        # 1. pure-Python install (pip wants a writable source tree: install from a scratch copy)
        work = os.path.join(tmp, "src")
        shutil.copytree(src, work, ignore=shutil.ignore_patterns(".git", "__pycache__", "*.egg-info", "build"))
        env = _env_without_nvcc()
        env["NO_BUILD_EXT"] = "1"
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", SITE_DIR, work]
        res = subprocess.run(cmd, env=env, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"pip install of the reference failed:\n{res.stdout[-2000:]}\n{res.stderr[-2000:]}")
        # 2. the CPU extension, by the reference's own JIT recipe over its sources in place
        ext_dir = os.path.join(tmp, "ext")
        env = _env_without_nvcc()
        env["TORCH_EXTENSIONS_DIR"] = ext_dir
        env["PYTHONPATH"] = src
        env["PYTHONDONTWRITEBYTECODE"] = "1"
        res = subprocess.run([sys.executable, "-c", "import falkon.c_ext._backend"], env=env, capture_output=True, text=True,
                             cwd=tmp)
        built = os.path.join(ext_dir, "falkon.c_ext._C", "falkon.c_ext._C.so")
        if res.returncode != 0 or not os.path.exists(built):
            raise RuntimeError(f"JIT build of the reference's CPU extension failed:\n{res.stdout[-2000:]}\n"
                               f"{res.stderr[-2000:]}")
        shutil.copyfile(built, os.path.join(SITE_DIR, "falkon", "c_ext", "_C.so"))
    # 3. check: the installed copy imports and computes, away from the checkout
    env = dict(os.environ)
    env["PYTHONPATH"] = SITE_DIR
    probe = ("import torch, falkon; from falkon.kernels import GaussianKernel; from falkon import FalkonOptions; "
             "k = GaussianKernel(1.0, opt=FalkonOptions(use_cpu=True, keops_active='no')); "
             "print(tuple(k.dmmv(torch.ones(8, 3), torch.ones(2, 3), torch.ones(2, 1), None).shape))")
    res = subprocess.run([sys.executable, "-c", probe], env=env, capture_output=True, text=True, cwd=REF_DIR)
    if res.returncode != 0 or "(2, 1)" not in res.stdout:
        raise RuntimeError(f"the installed reference does not run:\n{res.stdout[-2000:]}\n{res.stderr[-2000:]}")
    if verbose:
        print(f"reference built into {SITE_DIR}")
    return SITE_DIR


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=None)
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    build_ref(args.src, args.force)


if __name__ == "__main__":
    main()
