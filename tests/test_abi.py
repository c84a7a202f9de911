"""The C-ABI library builds without a GPU, loads, and exports every symbol the header declares."""
import ctypes
from pathlib import Path
import re

import pytest

from tilecadence_b200 import cuda_runtime

HEADER = Path(__file__).resolve().parents[1] / "include" / "tilecadence_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return set(re.findall(r"\b(tc_[a-z0-9_]+)\s*\(", text))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    assert {"tc_prefill_forward_out", "tc_prefill_workspace_spec", "tc_prefill_resources", "tc_decode_forward_out",
            "tc_decode_workspace_spec", "tc_decode_resources", "tc_decode_partial_out", "tc_combine_partials",
            "tc_last_error", "tc_abi_version", "tc_device_status"} <= names


def test_library_exports_every_declared_symbol(library):
    raw = ctypes.CDLL(str(library.path))
    for name in declared_symbols():
        assert hasattr(raw, name), f"{name} is declared in the header but not exported"
        assert name in library.SIGNATURES, f"{name} has no ctypes signature in cuda_runtime.Library"
    assert library.handle.tc_abi_version() == 1


def test_phase_libraries_export_only_their_phase(tmp_path):
    from tilecadence_b200.operator import emit

    emit("decode", tmp_path / "decode")
    path, identity = cuda_runtime.compile_directory(tmp_path / "decode")
    phase_library = cuda_runtime.load_library(path)
    assert phase_library.has("tc_decode_") and not phase_library.has("tc_prefill_")
    assert identity["target"] == "sm_100a" and "config.cuh" in identity["source_sha256"]
    assert cuda_runtime.ops_for(phase_library).phase == "decode"
    with pytest.raises(RuntimeError, match="another phase"):
        phase_library.call("tc_prefill_workspace_spec")


@pytest.mark.parametrize("module,symbol", [("trace_decode", "tc_debug_trace"),
                                           ("trace_prefill", "tc_debug_prefill_trace"),
                                           ("trace_project", "tc_debug_project_trace")])
def test_time_line_builds_are_libraries_of_their_own(library, module, symbol):
    """The TC_TRACE switch makes a separate library that exports the table reader; the shipped one never does."""
    import importlib

    path = importlib.import_module(f"tilecadence_b200.{module}").build()
    assert Path(path) != Path(library.path)
    assert hasattr(ctypes.CDLL(str(path)), symbol)
    assert not hasattr(ctypes.CDLL(str(library.path)), symbol)


def test_calls_fail_loudly_without_a_b200(library):
    """No CPU fallback: on a machine without an sm_100 device the entry points return an error."""
    import torch

    if torch.cuda.is_available() and torch.cuda.get_device_capability(0)[0] == 10:
        pytest.skip("a B200 is present; the failure path needs a machine without one")
    spec = (ctypes.c_int64 * 3)()
    with pytest.raises(RuntimeError, match="tc_decode_workspace_spec"):
        library.call("tc_decode_workspace_spec", 0, 1, 32768, 8, 0, 1, 1, spec)
    with pytest.raises(RuntimeError):
        cuda_runtime.cuda_device("cuda:0")


def test_build_cuda_rejects_directories_without_cuda(tmp_path):
    (tmp_path / "empty").mkdir()
    with pytest.raises(ValueError, match="No generated CUDA translation unit"):
        cuda_runtime.compile_directory(tmp_path / "empty")
