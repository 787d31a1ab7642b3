"""The split-K cost model of the down projection, evaluated on the host.

``choose_down_splits`` (csrc/common.cuh) is shared by the routing kernel and the host; it was
fitted to sweeps of forced split factors on a B200.  This test compiles it for the host and
pins its choice for the measured cases, each of which was within a few percent of the best
forced factor -- a guard against refits that help one shape and silently cost another.
"""

from __future__ import annotations

import shutil
import subprocess
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
CSRC = REPO / "b300-moe-decode-fastpath_b200" / "csrc"

# (units, K blocks, rows per segment rounded to 16) -> split factor; 296 resident blocks
MEASURED = [
    ((32, 224, 16), 7), ((64, 224, 16), 4), ((96, 224, 16), 3), ((128, 224, 16), 2),
    ((160, 224, 16), 5), ((192, 224, 16), 3), ((224, 224, 16), 1), ((256, 224, 16), 1),
    ((288, 224, 16), 1), ((320, 224, 16), 5), ((384, 224, 16), 3), ((448, 224, 16), 3),
    ((184, 45, 16), 3), ((184, 45, 32), 1), ((184, 45, 64), 1),      # H = I = 2880
    ((112, 32, 16), 2), ((224, 32, 16), 1), ((336, 32, 16), 2),      # H = 7168, I = 2048
    ((3304, 32, 16), 1),                                              # many experts: never split
    ((64, 112, 16), 4), ((256, 112, 16), 1),                         # FP8 weights: 128-element K blocks
    ((256, 224, 64), 1),
]


def test_split_model_keeps_its_measured_choices(tmp_path) -> None:
    if shutil.which("nvcc") is None:
        pytest.skip("no nvcc")
    rows = ",".join(f"{{{u},{k},{r}}}" for (u, k, r), _ in MEASURED)
    source = tmp_path / "split_model.cu"
    source.write_text(
        '#include <cstdio>\n#include "common.cuh"\n'
        "int main() {\n"
        f"  const int cases[][3] = {{{rows}}};\n"
        "  for (auto& c : cases)\n"
        '    printf("%d\\n", b200moe::choose_down_splits(c[0], 296, c[1], c[2]));\n'
        '  printf("%d %d %d %d %d\\n", b200moe::rows16_of(2, 2), b200moe::rows16_of(136, 8),\n'
        "         b200moe::rows16_of(504, 8), b200moe::rows16_of(0, 0), b200moe::rows16_of(4000, 2));\n"
        "  return 0;\n}\n"
    )
    binary = tmp_path / "split_model"
    subprocess.run(["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", str(CSRC),
                    "-I", str(REPO / "include"), "-o", str(binary), str(source)],
                   check=True, capture_output=True)
    lines = subprocess.run([str(binary)], check=True, capture_output=True, text=True).stdout.split("\n")
    got = [int(x) for x in lines[: len(MEASURED)]]
    assert got == [want for _, want in MEASURED]
    assert lines[len(MEASURED)].split() == ["16", "32", "64", "16", "128"]
