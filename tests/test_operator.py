"""Emitter: solved offsets reach the CUDA template (reference ``tests/test_operator.py:9-19``)."""
from pathlib import Path
import subprocess
import sys

import pytest

from tilecadence_b200.operator import OFFSETS, emit
from tilecadence_b200.placement import HANDOFFS, replay


def defines_of(text):
    """{macro: value} for every ``#define NAME <integer>`` line of a header."""
    found = {}
    for line in text.splitlines():
        words = line.split()
        if len(words) == 3 and words[0] == "#define" and words[2].lstrip("-").isdigit():
            found[words[1]] = int(words[2])
    return found


@pytest.mark.parametrize("phase", sorted(OFFSETS))
def test_emitted_config_carries_the_solved_offsets(tmp_path, phase):
    """What the reference's ``tests/test_operator.py:9-19`` pins: every region's solved offset is the value
    of its macro in the emitted ``config.cuh``, and a placement that puts two regions on the same bytes is
    rejected by ``replay`` with an "overlap" error."""
    directory = tmp_path / "emitted" / phase
    solved = emit(phase, directory)
    macros = defines_of((directory / "config.cuh").read_text())
    placed = {}
    for region, macro in OFFSETS[phase].items():
        placed[region] = solved["regions"][region]["offset_bytes"]
        assert macros[macro] == placed[region]
    assert set(placed) == set(solved["regions"])
    replay(HANDOFFS[phase], placed)  # the solved placement itself is accepted
    regions = list(placed)
    collided = dict(placed)
    collided[regions[1]] = collided[regions[0]]
    with pytest.raises(ValueError, match="overlap"):
        replay(HANDOFFS[phase], collided)


def test_emitted_prefill_config_carries_the_tensor_memory_map(tmp_path: Path):
    """The prefill kernel's tensor-memory columns come from the planner the way its LSE offsets do."""
    import json

    from tilecadence_b200.operator import TMEM_ALLOCATION, TMEM_COLUMNS
    from tilecadence_b200.placement import TMEM_MAPS, replay_tmem

    emit("prefill", tmp_path / "prefill")
    macros = defines_of((tmp_path / "prefill" / "config.cuh").read_text())
    solved = json.loads((tmp_path / "prefill" / "tmem_placement.json").read_text())
    columns = {}
    for region, macro in TMEM_COLUMNS["prefill"].items():
        columns[region] = solved["regions"][region]["offset_columns"]
        assert macros[macro] == columns[region]
    assert macros[TMEM_ALLOCATION["prefill"]] == solved["allocation_columns"] == 512
    replay_tmem(TMEM_MAPS["prefill"], columns)
    source = (tmp_path / "prefill" / "prefill_sm100.cu").read_text()
    for macro in list(TMEM_COLUMNS["prefill"].values()) + [TMEM_ALLOCATION["prefill"]]:
        assert macro in source  # the kernel reads its map from the emitted macros, not from constants of its own
    emit("decode", tmp_path / "decode")
    assert not (tmp_path / "decode" / "tmem_placement.json").exists()  # the decode kernel uses no tensor memory


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
