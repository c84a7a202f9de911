"""Emit the prefill or decode schedule with solved shared-memory offsets.

Same behaviour as ``tilecadence/operator.py`` (``OFFSETS`` :13-18, ``emit`` :21-38, CLI :41-46):
solve the phase's handoff, rewrite exactly one ``#define <MACRO> <n>`` per region in the phase's
``config.cuh``, copy the remaining template files next to it and write ``placement.json``. The
output directory must not exist. The emitted directory is self-contained (kernel, PTX helpers,
host plumbing and the C-ABI header) and is what :func:`tilecadence_b200.cuda_runtime.build_cuda`
compiles.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path
import re
import shutil

from .cuda_runtime import staged_sources
from .placement import HANDOFFS, solve


OFFSETS = {
    "prefill": {"head0_lse": "PREFILL_LSE_HEAD0_OFFSET_BYTES",
                "head1_lse": "PREFILL_LSE_HEAD1_OFFSET_BYTES"},
    "decode": {"output_tile": "AB_DECODE_O_OFFSET_BYTES",
               "row_lse": "AB_DECODE_LSE_OFFSET_BYTES"},
}


def emit(phase: str, out: Path) -> dict:
    if phase not in OFFSETS:
        raise ValueError(f"Unknown operator: {phase}")
    placement = solve(HANDOFFS[phase])
    template = staged_sources(phase)
    config = template["config.cuh"].read_text(encoding="utf-8")
    for region, macro in OFFSETS[phase].items():
        offset = placement["regions"][region]["offset_bytes"]
        config, count = re.subn(rf"^#define {macro} \d+$", f"#define {macro} {offset}", config, flags=re.M)
        if count != 1:
            raise ValueError(f"Expected exactly one template definition of {macro}")
    out = Path(out)
    out.mkdir(parents=True, exist_ok=False)
    for name, path in template.items():
        if name != "config.cuh":
            shutil.copyfile(path, out / name)
    (out / "config.cuh").write_text(config, encoding="utf-8", newline="\n")
    (out / "placement.json").write_text(json.dumps(placement, indent=2) + "\n", encoding="utf-8")
    return placement


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--phase", choices=OFFSETS, required=True)
    parser.add_argument("--out", type=Path, required=True)
    args = parser.parse_args()
    emit(args.phase, args.out)


if __name__ == "__main__":
    main()
