"""Generate the golden fixtures in this directory by running the reference itself.

    python tests/golden/make_golden.py /path/to/b300-moe-decode-fastpath

The reference's pure-PyTorch backend (``fastpath.b300_moe_forward(...,
backend="torch")``) imports and runs on a CPU.  This script feeds it small,
seeded BF16-representable inputs (as FP32 tensors, so its arithmetic is the
"FP32 reference on identical inputs"), and stores inputs, outputs and routing
tensors.  The fixtures pin ``oracle/moe_oracle.py`` and are replayed through
the CUDA kernels by the GPU tests.  Nothing at test time needs the reference.

File format (``.npz``): per group one set of expert weights shared by several
cases.  BF16 tensors are stored as their raw 16-bit patterns (uint16).
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def bf16_bits(x: torch.Tensor) -> np.ndarray:
    return x.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def main() -> int:
    if len(sys.argv) != 2:
        print(__doc__)
        return 2
    sys.path.insert(0, sys.argv[1])
    from baseline.routing import generate_router_logits, topk_routing  # type: ignore
    from fastpath import b300_moe_forward  # type: ignore

    def run_reference(hidden, ids, weights, gate_up, down, experts, top_k):
        out, meta = b300_moe_forward(
            hidden.float(),
            ids,
            weights.float(),
            gate_up.float(),
            down.float(),
            num_experts=experts,
            top_k=top_k,
            backend="torch",
            quant_mode="none",
            return_metadata=True,
        )
        return out, meta

    groups = {
        # name: (E, H, I, std, seed, [(T, K, workload)])
        # the shape and workloads of the reference's own CUDA suite
        # (tests/test_goal_1b_cuda.py:54-136): E=16, H=32, I=48
        "e16_h32_i48": (16, 32, 48, None, 100, [
            (1, 1, "uniform"), (1, 8, "hotspot"), (2, 2, "zipf"), (7, 4, "uniform"),
            (16, 2, "hotspot"), (32, 8, "zipf"), (64, 8, "uniform"), (64, 1, "hotspot"),
            (5, 2, "same_expert_twice"), (24, 4, "duplicates"), (16, 2, "single_expert"),
        ]),
        # H and I multiples of 8 but not of 64 or 128: K tails and M tails
        "e4_h72_i200": (4, 72, 200, None, 200, [
            (3, 2, "uniform"), (17, 4, "zipf"), (63, 4, "duplicates"), (40, 1, "single_expert"),
        ]),
        # more than 128 rows in one expert (segments split) and many empty experts
        "e32_h32_i64": (32, 32, 64, None, 300, [
            (64, 8, "single_expert"), (64, 4, "hotspot"), (1, 2, "uniform"), (33, 8, "zipf"),
        ]),
    }

    for name, (E, H, I, std, seed, cases) in groups.items():
        g = torch.Generator().manual_seed(seed)
        s_in = H ** -0.5 if std is None else std
        s_dn = I ** -0.5 if std is None else std
        gate_up = (torch.randn(E, 2 * I, H, generator=g) * s_in).to(torch.bfloat16)
        down = (torch.randn(E, H, I, generator=g) * s_dn).to(torch.bfloat16)
        payload: dict[str, np.ndarray] = {
            "gate_up_weight": bf16_bits(gate_up),
            "down_weight": bf16_bits(down),
            "dims": np.array([E, H, I], np.int64),
            "num_cases": np.array([len(cases)], np.int64),
        }
        for index, (T, K, workload) in enumerate(cases):
            hidden = torch.randn(T, H, generator=g).to(torch.bfloat16)
            case_seed = seed + 10 * index + 1
            if workload in ("uniform", "hotspot", "zipf"):
                logits = generate_router_logits(T, E, K, workload, case_seed, dtype=torch.float32)
                ids, weights = topk_routing(logits, K)
                weights = weights.to(torch.bfloat16)
            elif workload == "same_expert_twice":
                ids = torch.full((T, K), 3, dtype=torch.int64)
                weights = torch.randn(T, K, generator=g).to(torch.bfloat16)  # negatives too
            elif workload == "duplicates":
                ids = torch.randint(0, E, (T, K), generator=g)
                weights = (torch.randn(T, K, generator=g) * 2).to(torch.bfloat16)
            elif workload == "single_expert":
                base = 5 if E > 5 else 1
                ids = torch.full((T, K), base, dtype=torch.int64)
                weights = torch.softmax(torch.randn(T, K, generator=g), -1).to(torch.bfloat16)
                if K <= E and K > 1:
                    # every token to the same K experts, distinct per slot
                    ids = torch.arange(base, base + K, dtype=torch.int64).remainder(E).expand(T, K).clone()
                    if name == "e32_h32_i64" and T * K >= 256:
                        ids = torch.full((T, K), base, dtype=torch.int64)  # 512 rows in one expert
            else:
                raise ValueError(workload)
            ids = ids.contiguous()
            out, meta = run_reference(hidden, ids, weights, gate_up, down, E, K)
            p = f"case{index}_"
            payload[p + "hidden"] = bf16_bits(hidden)
            payload[p + "ids"] = ids.numpy().astype(np.int64)
            payload[p + "weights"] = bf16_bits(weights)
            payload[p + "output_fp32"] = out.numpy().astype(np.float32)
            payload[p + "permutation"] = meta["permutation"].numpy()
            payload[p + "reverse_mapping"] = meta["reverse_mapping"].numpy()
            payload[p + "expert_counts"] = meta["expert_counts"].numpy()
            payload[p + "expert_offsets"] = meta["expert_offsets"].numpy()
            payload[p + "label"] = np.array(f"T={T},K={K},{workload}")
        np.savez_compressed(HERE / f"golden_{name}.npz", **payload)
        print("wrote", name, {k: v.shape for k, v in payload.items() if k.startswith("case0")})
    # router front end: the reference's generators and its topk_routing, FP32 and BF16 logits
    router: dict[str, np.ndarray] = {}
    specs = [(1, 8, 1, "uniform"), (7, 16, 2, "hotspot"), (64, 64, 8, "zipf"),
             (33, 256, 8, "uniform"), (64, 128, 4, "hotspot")]
    for index, (T, E, K, workload) in enumerate(specs):
        logits = generate_router_logits(T, E, K, workload, 500 + index, dtype=torch.float32)
        for tag, cast in (("f32", logits), ("bf16", logits.to(torch.bfloat16))):
            ids, weights = topk_routing(cast, K)
            p = f"case{index}_{tag}_"
            router[p + "logits"] = logits.numpy() if tag == "f32" else bf16_bits(cast)
            router[p + "ids"] = ids.numpy()
            router[p + "weights"] = weights.numpy() if tag == "f32" else bf16_bits(weights)
    router["num_cases"] = np.array([len(specs)], np.int64)
    np.savez_compressed(HERE / "golden_router.npz", **router)
    print("wrote router", len(specs))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
