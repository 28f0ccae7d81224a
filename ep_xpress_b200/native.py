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
            "moe_gemm_sm100.cu", "moe_noalloc.cu", "host_helpers.cu")
_HEADERS = ("epx_layout.h", "epx_device.cuh", "epx_launch.h", "heap.h", "moe_gemm.h", "moe_noalloc.h", "host_helpers.h")
_ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
_lock = threading.Lock()
_module = None
_loaded_identity = ""


def sources():
    return [str(_CSRC / name) for name in _SOURCES]


def library_path() -> Path:
    return _PACKAGE / f"{_NAME}.so"


def source_identity() -> str:
    """Hash of the native sources in the tree."""
    digest = hashlib.blake2b(digest_size=8)
    for name in sorted(_SOURCES + _HEADERS):
        digest.update(name.encode())
        digest.update((_CSRC / name).read_bytes())
    return digest.hexdigest()


def _stamp_path() -> Path:
    return _PACKAGE / f"{_NAME}.stamp"


def binary_identity() -> str:
    """Source hash the library file on disk was built from ("" when there is none). The stamp is
    written right after the library, so it names the binary, not the tree."""
    stamp = _stamp_path()
    if not (library_path().exists() and stamp.exists()):
        return ""
    return stamp.read_text().strip()


def build_identity() -> str:
    """Identity of the native build this process runs: part of the bootstrap signature, so that
    ranks with different binaries refuse to form a group (the reference puts its extension's
    build name there, ep_xpress/host_sm.py:360-366). `load()` only ever imports a library whose
    stamp matches the sources, hence this is the stamp of the loaded binary."""
    return _loaded_identity or binary_identity() or source_identity()


def is_built() -> bool:
    return binary_identity() == source_identity()


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile the extension for sm_100a into the package directory.

    Works without a GPU (nvcc cross-compiles). Safe to call repeatedly: an
    up-to-date library is kept.
    """
    import fcntl
    with _lock, open(_PACKAGE / f"{_NAME}.lock", "w") as guard:
        fcntl.flock(guard, fcntl.LOCK_EX)      # one builder per tree: the ranks of a job share it
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
        _stamp_path().unlink(missing_ok=True)
        shutil.copyfile(build_dir / f"{_NAME}.so", library_path())
        _stamp_path().write_text(source_identity() + "\n")
        return library_path()


def load():
    """Import the runtime built from EXACTLY the sources in the tree.

    A library whose stamp differs from the sources (edited sources, a binary copied from
    elsewhere) is never imported: it is rebuilt when a compiler is present, otherwise the call
    fails. Raises instead of falling back to a PyTorch path: on a GPU machine a missing native
    runtime must be loud.
    """
    global _module, _loaded_identity
    with _lock:
        if _module is not None:
            return _module
    if not is_built():
        if shutil.which("nvcc") is None:
            raise RuntimeError(
                "ep_xpress_b200 native runtime is missing or was built from other sources than the ones in "
                "this tree, and nvcc is unavailable; run `python -c 'import __graft_entry__ as g; g.build()'` "
                "on a machine with the CUDA toolkit")
        build()
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    with _lock:
        if _module is None:
            _loaded_identity = binary_identity()
            loader = importlib.machinery.ExtensionFileLoader(_NAME, str(library_path()))
            spec = importlib.util.spec_from_file_location(_NAME, str(library_path()), loader=loader)
            module = importlib.util.module_from_spec(spec)
            loader.exec_module(module)
            sys.modules.setdefault(f"ep_xpress_b200.{_NAME}", module)
            _module = module
        return _module
