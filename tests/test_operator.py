"""Emitter: solved offsets reach the CUDA template (reference ``tests/test_operator.py:9-19``)."""
from pathlib import Path
import subprocess
import sys

import pytest

from tilecadence_b200.operator import OFFSETS, emit
from tilecadence_b200.placement import HANDOFFS, replay


@pytest.mark.parametrize("phase", ("prefill", "decode"))
def test_solved_offsets_reach_the_cuda_template(tmp_path: Path, phase: str):
    placement = emit(phase, tmp_path / phase)
    config = (tmp_path / phase / "config.cuh").read_text()
    offsets = {name: value["offset_bytes"] for name, value in placement["regions"].items()}
    for name, macro in OFFSETS[phase].items():
        assert f"#define {macro} {offsets[name]}\n" in config
    first, second = offsets
    offsets[second] = offsets[first]
    with pytest.raises(ValueError, match="overlap"):
        replay(HANDOFFS[phase], offsets)


def test_emit_is_self_contained_and_never_overwrites(tmp_path: Path):
    target = tmp_path / "decode"
    emit("decode", target)
    names = {path.name for path in target.iterdir()}
    assert {"config.cuh", "placement.json", "decode_sm100.cu", "tc_ptx.cuh", "tc_host.cuh", "tc_abi.cu",
            "tilecadence_b200.h"} <= names
    with pytest.raises(FileExistsError):
        emit("decode", target)
    with pytest.raises(ValueError, match="Unknown operator"):
        emit("combine", tmp_path / "x")


def test_operator_cli(tmp_path: Path):
    out = tmp_path / "cli"
    subprocess.run([sys.executable, "-m", "tilecadence_b200.operator", "--phase", "prefill", "--out", str(out)],
                   check=True, cwd=Path(__file__).resolve().parents[1])
    assert "#define PREFILL_LSE_HEAD1_OFFSET_BYTES 66048\n" in (out / "config.cuh").read_text()


def test_emitted_default_matches_the_tree(tmp_path: Path):
    """The solved offsets are the template defaults, so the in-tree build is the emitted schedule."""
    from tilecadence_b200.cuda_runtime import CSRC

    for phase in ("prefill", "decode"):
        emit(phase, tmp_path / phase)
        assert (tmp_path / phase / "config.cuh").read_text() == (CSRC / phase / "config.cuh").read_text()
