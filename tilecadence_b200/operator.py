"""Turn a solved handoff into a buildable source directory for the prefill or the decode kernel.

Public surface and behaviour follow ``tilecadence/operator.py`` (``OFFSETS`` :13-18, ``emit`` :21-38,
command line :41-46): the phase's handoff is solved, each region's byte offset replaces the value of
one macro in that phase's ``config.cuh``, every other source file is copied unchanged, and the solver's
answer is stored as ``placement.json``. For the prefill kernel the tensor-memory map is solved as well
(``placement.solve_tmem``): the first column of every tile and the allocation size replace their macros
in the same ``config.cuh`` and the answer is stored as ``tmem_placement.json``. An existing output directory is an error. What is written here
is self-contained (kernel, PTX helpers, host plumbing, C-ABI header): it is exactly what
:func:`tilecadence_b200.cuda_runtime.build_cuda` compiles.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

from . import placement as _placement
from .cuda_runtime import staged_sources

#: region name -> macro that carries its offset, per phase (the reference's names, so that emitted
#: configurations stay readable side by side).
OFFSETS = {
    "prefill": {
        "head0_lse": "PREFILL_LSE_HEAD0_OFFSET_BYTES",
        "head1_lse": "PREFILL_LSE_HEAD1_OFFSET_BYTES",
    },
    "decode": {
        "output_tile": "AB_DECODE_O_OFFSET_BYTES",
        "row_lse": "AB_DECODE_LSE_OFFSET_BYTES",
    },
}

#: tensor-memory tile -> macro that carries its first column, per phase (no counterpart in the reference,
#: whose kernels have no tensor memory). ``TMEM_ALLOCATION`` names the macro of the allocation size.
TMEM_COLUMNS = {
    "prefill": {
        "score_head0": "PREFILL_TMEM_S_HEAD0_COLUMN",
        "score_head1": "PREFILL_TMEM_S_HEAD1_COLUMN",
        "probability_head0": "PREFILL_TMEM_P_HEAD0_COLUMN",
        "probability_head1": "PREFILL_TMEM_P_HEAD1_COLUMN",
        "output_head0": "PREFILL_TMEM_O_HEAD0_COLUMN",
        "output_head1": "PREFILL_TMEM_O_HEAD1_COLUMN",
    },
}
TMEM_ALLOCATION = {"prefill": "PREFILL_TMEM_ALLOCATION_COLUMNS"}

CONFIG_NAME = "config.cuh"


def _with_macro_values(text: str, values: dict[str, int]) -> str:
    """``text`` with the integer after ``#define NAME`` replaced for every NAME in ``values``.

    Each name must be defined exactly once, on a line of its own, with an unsigned decimal value.
    """
    seen = dict.fromkeys(values, 0)
    lines = text.split("\n")
    for index, line in enumerate(lines):
        words = line.split()
        if len(words) == 3 and words[0] == "#define" and words[1] in values and words[2].isdigit() \
                and line == " ".join(words):
            lines[index] = f"#define {words[1]} {values[words[1]]}"
            seen[words[1]] += 1
    for name, count in seen.items():
        if count != 1:
            raise ValueError(f"Expected exactly one template definition of {name}")
    return "\n".join(lines)


def emit(phase: str, out: Path) -> dict:
    """Solve ``phase``'s handoff and write the source directory ``out``; returns the placement."""
    macros = OFFSETS.get(phase)
    if macros is None:
        raise ValueError(f"Unknown operator: {phase}")
    solved = _placement.solve(_placement.HANDOFFS[phase])
    sources = staged_sources(phase)
    values = {macro: int(solved["regions"][region]["offset_bytes"]) for region, macro in macros.items()}
    tensor_memory = None
    if phase in TMEM_COLUMNS:
        tensor_memory = _placement.solve_tmem(_placement.TMEM_MAPS[phase])
        for region, macro in TMEM_COLUMNS[phase].items():
            values[macro] = int(tensor_memory["regions"][region]["offset_columns"])
        values[TMEM_ALLOCATION[phase]] = int(tensor_memory["allocation_columns"])
    config = _with_macro_values(sources[CONFIG_NAME].read_text(encoding="utf-8"), values)

    target = Path(out)
    target.mkdir(parents=True, exist_ok=False)
    for name, source in sources.items():
        destination = target / name
        if name == CONFIG_NAME:
            destination.write_text(config, encoding="utf-8", newline="\n")
        else:
            destination.write_bytes(source.read_bytes())
    (target / "placement.json").write_text(json.dumps(solved, indent=2) + "\n", encoding="utf-8")
    if tensor_memory is not None:
        (target / "tmem_placement.json").write_text(json.dumps(tensor_memory, indent=2) + "\n", encoding="utf-8")
    return solved


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--phase", required=True, choices=sorted(OFFSETS))
    parser.add_argument("--out", required=True, type=Path)
    arguments = parser.parse_args(argv)
    emit(arguments.phase, arguments.out)


if __name__ == "__main__":
    main()
