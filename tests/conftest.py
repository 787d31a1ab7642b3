"""Shared test plumbing: import paths, the ``gpu`` marker, golden-fixture loading."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
PACKAGE_DIR = REPO / "b300-moe-decode-fastpath_b200"
for entry in (str(PACKAGE_DIR), str(REPO)):
    if entry not in sys.path:
        sys.path.insert(0, entry)

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a CUDA device of compute capability 10.0")


def _from_bits(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


class GoldenCase:
    """One case of a golden group: BF16 inputs plus the reference's FP32 results."""

    def __init__(self, group: str, data, index: int) -> None:
        p = f"case{index}_"
        self.group = group
        self.label = f"{group}:{str(data[p + 'label'])}"
        self.num_experts, self.hidden_size, self.intermediate_size = (int(v) for v in data["dims"])
        self.gate_up_weight = _from_bits(data["gate_up_weight"])
        self.down_weight = _from_bits(data["down_weight"])
        self.hidden = _from_bits(data[p + "hidden"])
        self.ids = torch.from_numpy(data[p + "ids"].copy())
        self.weights = _from_bits(data[p + "weights"])
        self.top_k = int(self.ids.shape[1])
        self.output_fp32 = torch.from_numpy(data[p + "output_fp32"].copy())
        self.routing = {
            key: torch.from_numpy(data[p + key].copy())
            for key in ("permutation", "reverse_mapping", "expert_counts", "expert_offsets")
        }

    def inputs(self, device: str = "cpu"):
        return tuple(
            t.to(device)
            for t in (self.hidden, self.ids, self.weights, self.gate_up_weight, self.down_weight)
        )


def load_golden_cases() -> list[GoldenCase]:
    cases: list[GoldenCase] = []
    for path in sorted(GOLDEN_DIR.glob("golden_*.npz")):
        data = np.load(path)
        if "dims" not in data.files:
            continue  # not a layer fixture (the router fixture has its own loader)
        group = path.stem.removeprefix("golden_")
        for index in range(int(data["num_cases"][0])):
            cases.append(GoldenCase(group, data, index))
    return cases


def load_router_cases() -> list[dict]:
    """Router fixtures: logits plus the reference's top-k ids and softmax weights."""

    data = np.load(GOLDEN_DIR / "golden_router.npz")
    cases = []
    for index in range(int(data["num_cases"][0])):
        for tag in ("f32", "bf16"):
            p = f"case{index}_{tag}_"
            if tag == "f32":
                logits = torch.from_numpy(data[p + "logits"].copy())
                weights = torch.from_numpy(data[p + "weights"].copy())
            else:
                logits = _from_bits(data[p + "logits"])
                weights = _from_bits(data[p + "weights"])
            ids = torch.from_numpy(data[p + "ids"].copy())
            cases.append({"label": f"router{index}_{tag}_T{ids.shape[0]}_E{logits.shape[1]}"
                                   f"_K{ids.shape[1]}",
                          "logits": logits, "ids": ids, "weights": weights})
    return cases


GOLDEN_CASES = load_golden_cases()
ROUTER_CASES = load_router_cases()


@pytest.fixture(scope="session")
def cuda_device() -> torch.device:
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    return torch.device("cuda", 0)
