"""Builder and loader of the sm_100a native runtime.

The extension is compiled IN-TREE for ``sm_100a`` only and imported from the
package directory; importing :mod:`ep_xpress_b200` itself never compiles and
never initialises CUDA (same rule as the reference, ep_xpress/__init__.py:13-20
and ep_xpress/native.py:20-205, which JIT-builds on first use). Unlike the
reference there is no build-time ablation matrix: kernel variants are runtime
template selections inside one binary, so every rank of a group always runs the
same protocol and the build identity below is only a safety net.
"""

from __future__ import annotations

import hashlib
import importlib.machinery
import importlib.util
import os
import shutil
import sys
import threading
from pathlib import Path

_PACKAGE = Path(__file__).resolve().parent
_CSRC = _PACKAGE / "csrc"
_NAME = "_epx_native"
_SOURCES = ("engine.cpp", "heap.cpp", "moe_bindings.cpp", "host_ring.cpp", "dispatch_sm100.cu", "combine_sm100.cu", "expert_ops.cu",
            "moe_gemm_sm100.cu", "moe_noalloc.cu")
_HEADERS = ("epx_layout.h", "epx_device.cuh", "epx_launch.h", "heap.h", "moe_gemm.h", "moe_noalloc.h")
_ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
_lock = threading.Lock()
_module = None


def sources():
    return [str(_CSRC / name) for name in _SOURCES]


def library_path() -> Path:
    return _PACKAGE / f"{_NAME}.so"


def build_identity() -> str:
    """Hash of the native sources; part of the bootstrap signature."""
    digest = hashlib.blake2b(digest_size=8)
    for name in sorted(_SOURCES + _HEADERS):
        digest.update(name.encode())
        digest.update((_CSRC / name).read_bytes())
    return digest.hexdigest()


def _stamp_path() -> Path:
    return _PACKAGE / f"{_NAME}.stamp"


def is_built() -> bool:
    stamp = _stamp_path()
    return library_path().exists() and stamp.exists() and stamp.read_text().strip() == build_identity()


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile the extension for sm_100a into the package directory.

    Works without a GPU (nvcc cross-compiles). Safe to call repeatedly: an
    up-to-date library is kept.
    """
    with _lock:
        if not force and is_built():
            return library_path()
        from torch.utils import cpp_extension

        build_dir = _PACKAGE / "_build"
        build_dir.mkdir(exist_ok=True)
        cuda_flags = ["-O3", "-lineinfo", "-std=c++17", *_ARCH_FLAGS, "--expt-relaxed-constexpr"]
        previous = os.environ.get("TORCH_CUDA_ARCH_LIST")
        os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
        try:
            cpp_extension.load(
                name=_NAME,
                sources=sources(),
                extra_cflags=["-O3", "-std=c++17"],
                extra_cuda_cflags=cuda_flags,
                extra_include_paths=[str(_CSRC)],
                build_directory=str(build_dir),
                verbose=verbose,
                is_python_module=False,
            )
        finally:
            if previous is None:
                os.environ.pop("TORCH_CUDA_ARCH_LIST", None)
            else:
                os.environ["TORCH_CUDA_ARCH_LIST"] = previous
        shutil.copyfile(build_dir / f"{_NAME}.so", library_path())
        _stamp_path().write_text(build_identity() + "\n")
        return library_path()


def load():
    """Import the prebuilt runtime; build it first only if a compiler is present.

    Raises instead of falling back to a PyTorch path: on a GPU machine a missing
    native runtime must be loud.
    """
    global _module
    with _lock:
        if _module is not None:
            return _module
    if not library_path().exists():
        if shutil.which("nvcc") is None:
            raise RuntimeError(
                "ep_xpress_b200 native runtime is not built and nvcc is unavailable; "
                "run `python -c 'import __graft_entry__ as g; g.build()'` on a machine with the CUDA toolkit")
        build()
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    with _lock:
        if _module is None:
            loader = importlib.machinery.ExtensionFileLoader(_NAME, str(library_path()))
            spec = importlib.util.spec_from_file_location(_NAME, str(library_path()), loader=loader)
            module = importlib.util.module_from_spec(spec)
            loader.exec_module(module)
            sys.modules.setdefault(f"ep_xpress_b200.{_NAME}", module)
            _module = module
        return _module
