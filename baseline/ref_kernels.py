"""The reference's own Triton launchers, loaded from its installed copy under ``baseline/_ref``.

``baseline/_ref`` is the UNMODIFIED reference package, installed once with

    cp -r <reference checkout> /tmp/ref_copy
    python -m pip install --no-index --no-build-isolation --no-deps \
        --find-links /opt/wheelhouse --target baseline/_ref /tmp/ref_copy

(``--no-deps``: torch, triton, scipy and vllm are already in the image; the copy under /tmp because
the build writes an egg-info directory into the source tree).  The folder is not under version
control.  The reference and this repository's package share the import name ``rotorquant_vllm``,
so the Triton modules -- which import only ``torch`` and ``triton`` -- are loaded by file path
under private module names.  Used by ``bench.py`` (the GPU-kernel baseline the new kernels are
timed beside) and by one GPU test (the INT8 prefill error of both kernels against exact attention).
"""

from __future__ import annotations

import importlib.util
import os
import sys

_ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "rotorquant_vllm", "triton")

_FILES = {
    "fused_paged_rq_decode": "fused_paged_rq_decode.py",
    "fused_paged_rq_int8_prefill": "fused_paged_rq_int8_prefill.py",
    "iso_compress": "isoquant_compress.py",
    "planar_compress": "planarquant_compress.py",
    "iso_decompress": "isoquant_decompress.py",
    "planar_decompress": "planarquant_decompress.py",
}


def available() -> bool:
    return os.path.isdir(_ROOT)


def load(name: str):
    """The reference launcher ``name`` (one of the keys of ``_FILES``)."""
    if name not in _FILES:
        raise KeyError(name)
    path = os.path.join(_ROOT, _FILES[name])
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path}: install the reference under baseline/_ref first (see this module's docstring)")
    mod_name = "rq_reference_" + _FILES[name][:-3]
    mod = sys.modules.get(mod_name)
    if mod is None:
        spec = importlib.util.spec_from_file_location(mod_name, path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[mod_name] = mod
        spec.loader.exec_module(mod)
    return getattr(mod, name)
