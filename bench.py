"""Benchmark of the MoE decode layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1): the Mixtral-8x7B-shaped BF16 decode layer -- H=4096, I=14336,
E=8, top_k=2, T swept over {1,2,4,8,16,32,64}, activations ~N(0,1), weights
~N(0,0.02), uniform distinct routing, softmax routing weights.  One *step* is
one pass of the layer at every T of the sweep (seven forwards).  The reported
metric is the layer's P50 latency in microseconds, averaged over the sweep;
per-T and per-stage P50/P90/P99 and the achieved expert-weight HBM bandwidth are
attached to the same JSON line.

Timing protocol (the reference's, benchmark/timing.py:32-80, with an L2 flush
added): W warm-up steps, then K timed steps; every forward is bracketed by its
own CUDA-event pair on the launching stream, and before each forward a 256 MiB
buffer is written and a second one read, so no weight byte is served from the
126 MB L2 and no dirty line of the flush is written back under the timed kernels.
Percentiles use linear interpolation on the sorted samples (timing.py:23-29).
``total`` is ``b300_moe_forward``'s work only; the reference's ``total_us`` also
contains the router's top-k (benchmark_goal_1b.py:530-546), which is outside
this layer.

``--impl reference`` times the reference's own pure-PyTorch path
(``fastpath.b300_moe_forward(..., backend="torch")``) on the host CPU cores, same
workload, same metric, when an unmodified copy of the reference package lies in
``baseline/_ref`` (made by ``python bench.py --prepare-reference`` where the
reference checkout is available; the directory is not part of the repository's
history).  Without that copy it times the restatement in ``oracle/moe_oracle.py``
and says so (``cpu_baseline.kind`` = ``"port"``).

With N > 1 the layer runs expert-parallel; before anything is timed every token
layout and transport is checked against the FP32 oracle and the assembled
routing tensors against ``group_tokens`` (``parity`` in the JSON line; a miss
ends the run with a non-zero exit code).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
for entry in (str(REPO / "b300-moe-decode-fastpath_b200"), str(REPO)):
    if entry not in sys.path:
        sys.path.insert(0, entry)

import torch  # noqa: E402

SWEEP = (1, 2, 4, 8, 16, 32, 64)
HIDDEN, INTER, EXPERTS, TOP_K = 4096, 14336, 8, 2
ROUTING, WEIGHT_KIND = "uniform", "softmax"
WORKLOAD = "mixtral_8x7b_bf16_decode_layer_H4096_I14336_E8_K2_T1-64"
METRIC = "moe_layer_decode_p50_us_mean_over_T1_2_4_8_16_32_64"

# The default (and the only configuration the driver's line is quoted on) is the
# Mixtral-shaped sweep.  The others are the remaining benchmark configurations, run by
# hand with --config.
CONFIGS = {
    "mixtral": dict(hidden=4096, inter=14336, experts=8, top_k=2, sweep=(1, 2, 4, 8, 16, 32, 64),
                    routing="uniform", weight_kind="softmax"),
    "wide": dict(hidden=4096, inter=14336, experts=64, top_k=8, sweep=(64,),
                 routing="zipf", weight_kind="raw"),
    # the wide layer cut to 16 experts: same tiles, rows per expert and routing law, a fourth
    # of the weights (multi-GPU parity runs)
    "wide_e16": dict(hidden=4096, inter=14336, experts=16, top_k=8, sweep=(64,),
                     routing="zipf", weight_kind="raw"),
    "deepseek": dict(hidden=7168, inter=2048, experts=256, top_k=8, sweep=(1, 8, 32, 64),
                     routing="uniform", weight_kind="softmax"),
    "deepseek_hotspot": dict(hidden=7168, inter=2048, experts=256, top_k=8, sweep=(1, 8, 32, 64),
                             routing="hotspot", weight_kind="softmax"),
    "irregular": dict(hidden=2880, inter=2880, experts=32, top_k=8, sweep=(1, 3, 17, 63),
                      routing="concentrated", weight_kind="softmax"),
}


def apply_config(name: str) -> None:
    global SWEEP, HIDDEN, INTER, EXPERTS, TOP_K, ROUTING, WEIGHT_KIND, WORKLOAD, METRIC
    c = CONFIGS[name]
    HIDDEN, INTER, EXPERTS, TOP_K = c["hidden"], c["inter"], c["experts"], c["top_k"]
    SWEEP, ROUTING, WEIGHT_KIND = c["sweep"], c["routing"], c["weight_kind"]
    if name != "mixtral":
        tokens = "_".join(str(t) for t in SWEEP)
        WORKLOAD = (f"{name}_bf16_decode_layer_H{HIDDEN}_I{INTER}_E{EXPERTS}_K{TOP_K}_"
                    f"{ROUTING}_T{tokens}")
        METRIC = f"moe_layer_decode_p50_us_mean_over_T{tokens}"
L2_FLUSH_BYTES = 256 << 20
# End-to-end runs: outputs up to this size are stored into pinned host memory by the combine
# kernel itself (out=); larger ones go through a device-to-host copy, which the copy engine
# moves faster than a kernel's stores (measured: 512 KB at T=64 takes 2.5 us longer that way,
# 64 KB at T=8 takes 8 us less).
DIRECT_OUT_BYTES = 256 << 10
L2_POLICY = ("flushed before every timed forward: 256 MiB written, then 256 MiB read to push the "
             "dirty lines out; every forward also streams >= 352 MB of weights (> 126 MB L2)")
FALLBACK_HBM_GBS = 6650.0
STAGE_NAMES = ("routing", "gather", "gate_up_swiglu", "down", "combine")
PARITY_BAR = 2e-2  # max |y - y_ref| <= 2e-2 x rms(y_ref) against the FP32 oracle
# DRAM traffic of one launch of the dominant kernel, from the ncu captures summarised under
# profiles/: a small data file next to the summaries, keyed by kernel and tagged with the
# hash of the kernel source the capture was taken from.
TRAFFIC_FILE = REPO / "profiles" / "dram_traffic.json"
CSRC = REPO / "b300-moe-decode-fastpath_b200" / "csrc"


def source_hash(names: list[str]) -> str:
    import hashlib

    digest = hashlib.sha256()
    for name in names:
        digest.update((CSRC / name).read_bytes())
    return digest.hexdigest()[:16]


def measured_traffic(key: str) -> tuple[int | None, str]:
    """``dram__bytes_read.sum + dram__bytes_write.sum`` per launch for ``key``, or None
    (with the reason) when no capture is recorded or the kernel source has changed since."""

    try:
        entry = json.loads(TRAFFIC_FILE.read_text())[key]
    except (OSError, KeyError, ValueError):
        return None, "no ncu capture recorded for this kernel and workload"
    try:
        current = source_hash(entry["sources"])
    except OSError:
        return None, "kernel sources not found"
    if current != entry["source_hash"]:
        return None, (f"kernel source changed since the capture ({entry['source_hash']} -> "
                      f"{current}); re-capture and update profiles/dram_traffic.json")
    return int(entry["dram_bytes_read"]) + int(entry["dram_bytes_write"]), entry["summary"]


def percentile(sorted_values: list[float], q: float) -> float:
    if not sorted_values:
        return float("nan")
    pos = (len(sorted_values) - 1) * q
    lo = int(math.floor(pos))
    hi = min(lo + 1, len(sorted_values) - 1)
    return sorted_values[lo] + (sorted_values[hi] - sorted_values[lo]) * (pos - lo)


def summary(samples_us: list[float]) -> dict[str, float]:
    s = sorted(samples_us)
    return {
        "p50": round(percentile(s, 0.50), 2),
        "p90": round(percentile(s, 0.90), 2),
        "p99": round(percentile(s, 0.99), 2),
    }


def measured_peak_gbs() -> tuple[float, str]:
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, device_index: int) -> None:
        self.device_index = device_index
        self.proc: subprocess.Popen | None = None
        self.file = None
        self._thread = None
        self._stop = None
        self._nvml_samples: list[tuple[float, int]] = []
        self._nvml_max = None

    # NVML in a background thread is the primary source (a sample every 20 ms, no process
    # start-up inside a timed region that may last well under a second); nvidia-smi -lms is
    # the fall-back when the NVML binding is missing.  Both only read.
    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid)
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.device_index)

    def _nvml_read(self, pynvml, handle) -> None:
        clock = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
        reader = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(
            pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons")
        self._nvml_samples.append((float(clock), int(reader(handle))))

    def start(self) -> None:
        import threading

        try:
            pynvml, handle = self._nvml_handle()
            self._nvml_max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self._stop = threading.Event()

            def loop() -> None:
                while not self._stop.is_set():
                    try:
                        self._nvml_read(pynvml, handle)
                    except Exception:
                        return
                    self._stop.wait(0.02)

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
            return
        except Exception:
            self._thread = None
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.file, stderr=subprocess.DEVNULL,
            )
        except OSError:
            self.proc = None

    def _stop_nvml(self) -> dict[str, object]:
        self._stop.set()
        self._thread.join(timeout=2)
        # NVML's reason bits (nvml.h): sw_power_cap 0x4, hw_slowdown 0x8,
        # sw_thermal_slowdown 0x20, hw_thermal_slowdown 0x40
        bits = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20,
                "hw_thermal_slowdown": 0x40}
        clocks = sorted(c for c, _ in self._nvml_samples)
        reasons = sorted(name for name, bit in bits.items()
                         if any(mask & bit for _, mask in self._nvml_samples))
        return {
            "sm_mhz": percentile(clocks, 0.5) if clocks else None,
            "sm_max_mhz": self._nvml_max,
            "samples": len(clocks),
            "source": "nvml, 20 ms period",
            "reasons": reasons,
        }

    def stop(self) -> dict[str, object]:
        if self._thread is not None:
            return self._stop_nvml()
        if self.proc is None or self.file is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        clocks, max_clock, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        clocks.sort()
        return {
            "sm_mhz": percentile(clocks, 0.5) if clocks else None,
            "sm_max_mhz": max_clock,
            "samples": len(clocks),
            "source": "nvidia-smi -lms 100",
            "reasons": sorted(reasons),
        }


WEIGHT_ELEMENT_BYTES = 2  # 1 with --weights fp8
WEIGHT_FORMAT = "bf16"    # "fp8" / "nvfp4" with --weights


def weight_bytes(active_experts: int) -> dict[str, int]:
    """Algorithmic expert-weight bytes one forward must stream from HBM."""

    if WEIGHT_FORMAT == "nvfp4":
        # packed E2M1 (half a byte) + one E4M3 scale per 16 elements + one FP32 per matrix
        gate_up = active_experts * (2 * HIDDEN * INTER // 2 + 2 * HIDDEN * INTER // 16 + 4)
        down = active_experts * (HIDDEN * INTER // 2 + HIDDEN * INTER // 16 + 4)
        return {"gate_up": gate_up, "down": down, "total": gate_up + down}
    gate_up = active_experts * 2 * HIDDEN * INTER * WEIGHT_ELEMENT_BYTES  # [2I,H] per expert
    down = active_experts * HIDDEN * INTER * WEIGHT_ELEMENT_BYTES         # [H,I] per expert
    if WEIGHT_ELEMENT_BYTES == 1:  # + one FP32 scale per weight row
        gate_up += active_experts * 2 * INTER * 4
        down += active_experts * HIDDEN * 4
    return {"gate_up": gate_up, "down": down, "total": gate_up + down}


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if n_gpus > 1 and world > 1:
        import torch.distributed as dist

        # The product path crosses ranks with plain peer loads and stores of its own kernels;
        # NCCL serves the unfused baseline and the set-up only.  Its in-switch reduction is
        # left off unless the caller asks for it, so that no buffer of this process is bound
        # to an NVLink multicast object (every number in profiles/ was measured this way).
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return rank, world, local, dist
    return 0, 1, local if world > 1 else 0, None


# -----------------------------------------------------------------------------
# our arm
# -----------------------------------------------------------------------------
def library_gemm_baseline(case, gate_up, down, flush_l2, reps: int) -> dict[str, object]:
    """The two GEMMs as the reference's compiled path runs them, on this GPU.

    The reference calls PyTorch's BF16 grouped GEMM (csrc/grouped_gemm_sm103.cu:47-52) or
    a loop of ``torch.matmul(..., out=)`` over the active experts
    (fastpath/gemm_dispatch.py:100-150); its own GEMM-only comparison
    (results/b300_goal1b_20260720/step4_02_gemm_only.py:187-209) times exactly these two.
    They are library kernels, timed here only to be reported beside this library's stages:
    same permuted rows, same weights, same L2 flush, one CUDA-event pair per launch group.
    """

    ws = case["workspace"]
    rows = case["dev"][1].numel()
    buffers = ws.buffers
    x = buffers["permuted_hidden"][:rows]
    offsets = buffers["expert_offsets"][: EXPERTS + 1].to("cpu").tolist()  # outside the timed region
    ends_i32 = buffers["expert_offsets"][1: EXPERTS + 1].to(torch.int32)
    act = buffers["swiglu_output"][:rows]
    gu_out = torch.empty(rows, 2 * INTER, dtype=torch.bfloat16, device=x.device)
    dn_out = torch.empty(rows, HIDDEN, dtype=torch.bfloat16, device=x.device)
    active = [(e, offsets[e], offsets[e + 1]) for e in range(EXPERTS) if offsets[e + 1] > offsets[e]]

    def grouped(a, w):
        return torch._grouped_mm(a, w.transpose(1, 2), offs=ends_i32)

    def per_expert(a, w, out):
        for e, lo, hi in active:
            torch.matmul(a[lo:hi], w[e].t(), out=out[lo:hi])

    variants = {
        "grouped_mm": {"gate_up": lambda: grouped(x, gate_up), "down": lambda: grouped(act, down)},
        "per_expert_matmul": {"gate_up": lambda: per_expert(x, gate_up, gu_out),
                              "down": lambda: per_expert(act, down, dn_out)},
    }
    report: dict[str, object] = {}
    for name, stages in variants.items():
        entry: dict[str, object] = {}
        for stage, fn in stages.items():
            try:
                for _ in range(3):
                    fn()
                pairs = []
                for _ in range(reps):
                    flush_l2()
                    a = torch.cuda.Event(enable_timing=True)
                    b = torch.cuda.Event(enable_timing=True)
                    a.record()
                    fn()
                    b.record()
                    pairs.append((a, b))
                torch.cuda.synchronize(x.device)
                entry[stage] = summary([a.elapsed_time(b) * 1e3 for a, b in pairs])
            except (RuntimeError, AttributeError, TypeError) as error:
                entry[stage] = {"unavailable": str(error).splitlines()[0][:200]}
        report[name] = entry
    return report


# Column names of the reference's result files (benchmark/benchmark_goal_1b.py:77-122), so
# tooling written for those files reads this benchmark's output unchanged.
REFERENCE_CSV_FIELDS = (
    "backend_set_requested", "requested_backend", "actual_backend", "device", "gpu_name",
    "gpu_capability", "architecture", "dtype", "workload", "num_tokens", "num_experts", "top_k",
    "hidden_size", "intermediate_size", "quant_mode", "used_fallback", "gemm_policy",
    "gate_up_gemm_strategy", "down_gemm_strategy", "stage", "stage_status", "measurement",
    "samples", "p50_us", "p90_us", "p99_us", "cold_start_us", "cold_start_scope", "warmup",
    "repetitions", "timing_method", "weights_prepared_outside_timing", "torch_version",
    "torch_cuda_version", "torch_arch_list", "cuda_toolkit_version",
    "cuda_toolkit_version_source", "cutlass_version", "cutlass_version_source", "cutlass_path",
    "wrapper_compiled_architecture", "grouped_gemm_provider",
    "grouped_gemm_provider_architecture", "pytorch_cxx_version",
)
# reference stage name -> key of this benchmark's per-T record
REFERENCE_CSV_STAGES = (
    ("routing_us", "routing"), ("permutation_us", "permutation"), ("quantization_us", None),
    ("gate_up_gemm_us", "gate_up"), ("swiglu_us", "swiglu"), ("down_gemm_us", "down"),
    ("combine_us", "combine"), ("total_us", "total"),
)


def write_reference_csv(path: str, result: dict[str, object], args, device) -> int:
    """One row per (T, stage) in the reference's CSV schema; returns the row count.

    ``quantization_us`` is ``not_applicable`` (BF16 inputs are consumed as they are, as in
    benchmark_goal_1b.py:601-606) and ``swiglu_us`` is 0 with status ``fused_in_gate_up``:
    the activation runs in the gate+up kernel's epilogue and has no launch of its own.
    ``total_us`` is the layer call only; the reference's also holds the router's top-k.
    """

    import csv

    from b200moe import build_info

    info = build_info()
    props = torch.cuda.get_device_properties(device)
    common = {
        "backend_set_requested": "cutlass_bf16",
        "requested_backend": "cutlass_bf16",
        "actual_backend": "cutlass_bf16",
        "device": str(device),
        "gpu_name": props.name,
        "gpu_capability": f"{props.major}.{props.minor}",
        "architecture": "sm_100a",
        "dtype": "bfloat16",
        "workload": ROUTING,
        "num_experts": EXPERTS,
        "top_k": TOP_K,
        "hidden_size": HIDDEN,
        "intermediate_size": INTER,
        "quant_mode": "bf16",
        "used_fallback": "false",
        "gemm_policy": "auto",
        "gate_up_gemm_strategy": "grouped",
        "down_gemm_strategy": "grouped",
        "measurement": "steady_state",
        "cold_start_scope": "first_forward_after_input_setup",
        "warmup": args.warmup,
        "repetitions": args.steps,
        "timing_method": "cuda_events",
        "weights_prepared_outside_timing": "true",
        "torch_version": torch.__version__,
        "torch_cuda_version": str(torch.version.cuda),
        "torch_arch_list": ",".join(torch.cuda.get_arch_list()),
        "cuda_toolkit_version": str(info.get("cuda_runtime_version", "unavailable")),
        "cuda_toolkit_version_source": "extension_cudart_header",
        "cutlass_version": "not_used",
        "cutlass_version_source": "not_used",
        "cutlass_path": "not_used",
        "wrapper_compiled_architecture": str(info.get("compiled_architecture", "sm_100a")),
        "grouped_gemm_provider": str(info.get("bf16_grouped_gemm_provider", "unavailable")),
        "grouped_gemm_provider_architecture": str(info.get("compiled_architecture", "sm_100a")),
        "pytorch_cxx_version": "not_linked",
    }
    rows = []
    for T, record in result["per_T"].items():
        for stage, key in REFERENCE_CSV_STAGES:
            if key is None:
                stats, status, samples = {"p50": 0.0, "p90": 0.0, "p99": 0.0}, "not_applicable", args.steps
            elif key == "total":
                stats, status, samples = record["total_us"], "measured", args.steps
            else:
                stats = record["stages_us"][key]
                status = stats.get("status", "measured")
                samples = record.get("stage_samples", args.steps)
            rows.append(common | {
                "num_tokens": T,
                "stage": stage,
                "stage_status": status,
                "samples": samples,
                "p50_us": f"{stats.get('p50', 0.0):.9f}",
                "p90_us": f"{stats.get('p90', 0.0):.9f}",
                "p99_us": f"{stats.get('p99', 0.0):.9f}",
                "cold_start_us": f"{record.get('cold_start_us', 0.0):.9f}",
            })
    out = Path(path)
    out.parent.mkdir(parents=True, exist_ok=True)
    with out.open("w", newline="", encoding="utf-8") as handle:
        writer = csv.DictWriter(handle, fieldnames=REFERENCE_CSV_FIELDS)
        writer.writeheader()
        writer.writerows(rows)
    return len(rows)


# -----------------------------------------------------------------------------
# parity, checked outside every timed region (the oracle is the checker, never the path)
# -----------------------------------------------------------------------------
def _parity_tokens(T: int, num_experts: int) -> list[int]:
    """All tokens when the FP32 oracle of the whole layer fits the host (the 8-expert
    layer), else three of them (the oracle then needs only the experts those route to)."""

    if num_experts * HIDDEN * INTER <= 8 * 4096 * 14336:
        return list(range(T))
    return sorted({0, T // 2, T - 1})


def _oracle_rows(hidden, ids, weights, tokens, expert_weights):
    """FP32 oracle rows for ``tokens``; ``expert_weights`` maps expert id -> (gate_up, down)
    CPU tensors and must hold every expert those tokens route to."""

    from oracle import moe_oracle

    picked = ids[tokens]
    experts = sorted({int(e) for e in picked.reshape(-1).tolist()})
    remap = {e: i for i, e in enumerate(experts)}
    small_ids = torch.tensor([[remap[int(e)] for e in row] for row in picked.tolist()],
                             dtype=torch.int64)
    gate_up = torch.stack([expert_weights[e][0] for e in experts])
    down = torch.stack([expert_weights[e][1] for e in experts])
    ref, _ = moe_oracle.routed_moe(hidden[tokens], small_ids, weights[tokens], gate_up, down,
                                   num_experts=len(experts), top_k=picked.shape[1])
    return ref


def single_gpu_parity(forward, cases, gate_up_cpu, down_cpu, sweep) -> dict[str, object]:
    """The timed call at the smallest and the largest T against the FP32 oracle."""

    from oracle import moe_oracle

    experts = {e: (gate_up_cpu[e], down_cpu[e]) for e in range(gate_up_cpu.shape[0])}
    detail, worst, floor = {}, 0.0, 0.0
    for T in sorted({sweep[0], sweep[-1]}):
        out = forward(T)
        torch.cuda.synchronize(out.device)
        hidden, ids, weights = cases[T]["host"]
        tokens = _parity_tokens(T, len(experts))
        ref = _oracle_rows(hidden, ids, weights, tokens, experts)
        err = moe_oracle.relative_max_error(out[tokens].float().cpu(), ref)
        detail[str(T)] = {"err_over_rms": round(err, 5), "floor": round(moe_oracle.bf16_floor(ref), 5),
                          "tokens_checked": len(tokens)}
        worst = max(worst, err)
        floor = max(floor, detail[str(T)]["floor"])
    return {"err_over_rms": round(worst, 5), "floor": floor, "bar": PARITY_BAR,
            "status": 0 if worst <= PARITY_BAR else 1,
            "oracle": "oracle/moe_oracle.routed_moe (FP32) on the same seeded inputs",
            "per_T": detail}


def expert_parallel_parity(engines, cases, gate_up, down, base, count, rank, world, device,
                           dist, fp8_scales) -> dict[str, object]:
    """Every token layout and transport of the N-GPU layer against the FP32 oracle, and the
    assembled routing tensors bit-exact against ``group_tokens``; rank 0 judges.

    The oracle needs the weights of the experts the checked tokens route to: their owners
    broadcast them once (BF16, as resident; FP8 weights are dequantised first, so the
    oracle sees what the kernels multiply by)."""

    import numpy as np

    from oracle import moe_oracle

    if fp8_scales is not None:
        from b200moe import dequantize_rows_fp8  # E4M3 value * row scale, as BF16

        gate_up = dequantize_rows_fp8(gate_up, fp8_scales[0])
        down = dequantize_rows_fp8(down, fp8_scales[1])
    checked_T = sorted({SWEEP[0], SWEEP[-1]})
    tokens = {T: _parity_tokens(T, EXPERTS) for T in checked_T}
    needed = sorted({int(e) for T in checked_T
                     for e in cases[T]["host"][1][tokens[T]].reshape(-1).tolist()})
    expert_weights = {}
    gu_buf = torch.empty_like(gate_up[0])
    dn_buf = torch.empty_like(down[0])
    for e in needed:
        owner = e // count
        if owner == rank:
            gu_buf.copy_(gate_up[e - base])
            dn_buf.copy_(down[e - base])
        dist.broadcast(gu_buf, src=owner)
        dist.broadcast(dn_buf, src=owner)
        if rank == 0:
            expert_weights[e] = (gu_buf.cpu(), dn_buf.cpu())
    report = {"replicated_err_over_rms": 0.0, "sharded_err_over_rms": 0.0, "floor": 0.0,
              "routing_bit_exact": True, "bar": PARITY_BAR, "status": 0,
              "oracle": "oracle/moe_oracle.routed_moe (FP32) and group_tokens on the same "
                        "seeded inputs; rank 0 judges every rank's rows",
              "checked": {}}
    for T in checked_T:
        hidden, ids, weights = cases[T]["host"]
        ref = want = None
        if rank == 0:
            ref = _oracle_rows(hidden, ids, weights, tokens[T], expert_weights)
            want = moe_oracle.group_tokens(ids, EXPERTS)
            report["floor"] = max(report["floor"], round(moe_oracle.bf16_floor(ref), 5))
        for name, engine in engines.items():
            out = engine.forward(*cases[T]["dev"], tokens="replicated")
            assembled = engine.global_routing()
            # every rank's replicated output goes to rank 0: all of them must pass
            gathered = [torch.empty_like(out) for _ in range(world)]
            dist.all_gather(gathered, out.contiguous())
            entry = {}
            if rank == 0:
                errs = [moe_oracle.relative_max_error(g[tokens[T]].float().cpu(), ref)
                        for g in gathered]
                entry["replicated"] = round(max(errs), 5)
                entry["ranks_identical"] = all(torch.equal(g, gathered[0]) for g in gathered)
                exact = all(np.array_equal(assembled[key].cpu().numpy(), getattr(want, key))
                            for key in ("expert_counts", "expert_offsets", "permutation",
                                        "reverse_mapping"))
                entry["routing_bit_exact"] = bool(exact)
                report["routing_bit_exact"] &= bool(exact)
                report["replicated_err_over_rms"] = max(report["replicated_err_over_rms"],
                                                        entry["replicated"])
            if T % world == 0:
                per = T // world
                shard = tuple(t[rank * per:(rank + 1) * per].contiguous()
                              for t in cases[T]["dev"])
                mine = engine.forward(*shard, tokens="sharded")
                rows = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(rows, mine.contiguous())
                if rank == 0:
                    whole = torch.cat(rows)
                    entry["sharded"] = round(moe_oracle.relative_max_error(
                        whole[tokens[T]].float().cpu(), ref), 5)
                    report["sharded_err_over_rms"] = max(report["sharded_err_over_rms"],
                                                         entry["sharded"])
            status = int(engine.workspace.status()) if engine.workspace is not None else 0
            flag = torch.tensor([status], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            entry["device_status"] = int(flag.item())
            report["checked"][f"T{T}_{name}"] = entry
            if entry["device_status"] != 0:
                report["status"] = 2
    if rank == 0:
        ok = (report["replicated_err_over_rms"] <= PARITY_BAR
              and report["sharded_err_over_rms"] <= PARITY_BAR and report["routing_bit_exact"]
              and all(e.get("ranks_identical", True) for e in report["checked"].values()))
        if not ok and report["status"] == 0:
            report["status"] = 1
    verdict = torch.tensor([report["status"]], device=device)
    dist.broadcast(verdict, src=0)
    report["status"] = int(verdict.item())
    return report


def packed_step_inputs(hidden, ids, weights, device):
    """One step's inputs as views into ONE pinned host buffer and ONE device buffer of the
    same layout, so that the end-to-end path moves them with a single host-to-device copy
    (three separate copies of a few KB each cost three DMA start-ups).  Returns
    ``(host_pack, dev_pack, host_views, dev_views)``; the views are ``(hidden, ids, weights)``
    with the alignment the kernels need (hidden 256 bytes, ids 8 bytes)."""

    def carve(buffer):
        views, offset = [], 0
        for t in (hidden, ids, weights):
            nbytes = t.numel() * t.element_size()
            views.append(buffer[offset:offset + nbytes].view(t.dtype).view(t.shape))
            offset += (nbytes + 255) // 256 * 256
        return tuple(views)

    total = sum((t.numel() * t.element_size() + 255) // 256 * 256 for t in (hidden, ids, weights))
    host_pack = torch.empty(total, dtype=torch.uint8).pin_memory()
    dev_pack = torch.empty(total, dtype=torch.uint8, device=device)
    host_views = carve(host_pack)
    for view, t in zip(host_views, (hidden, ids, weights)):
        view.copy_(t)
    return host_pack, dev_pack, host_views, carve(dev_pack)


def run_timeline(args: argparse.Namespace) -> dict[str, object]:
    """Device timeline of one forward per T from the kernels' own ``%globaltimer`` stamps.

    Every kernel of the library stamps when its first block started and when its last block
    finished, and the GEMMs when block 0 had its first complete operand stage
    (``B300MoEWorkspace.timeline()``); values are microseconds after the start of the routing
    kernel (negative for a kernel that started before it), medians of 11 forwards with L2
    flushed before each.  ``event_us`` is the CUDA-event time around the same forward.  A
    diagnosis aid: nothing here enters the benchmark line.
    """

    from b200moe import (B300MoEWorkspace, StagedLayer, quantize_expert_weights_fp8,
                         quantize_expert_weights_nvfp4, workloads)

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    sweep = tuple(args.only_tokens) if args.only_tokens else SWEEP
    gate_up, down = workloads.make_expert_weights(EXPERTS, HIDDEN, INTER, seed=1236, std=0.02,
                                                  device=device)
    extra: dict[str, object] = {}
    if args.weights == "fp8":
        extra["fp8_weights"] = quantize_expert_weights_fp8(gate_up, down)
    elif args.weights == "nvfp4":
        extra["nvfp4_weights"] = quantize_expert_weights_nvfp4(gate_up, down)
    if extra:
        gate_up = down = None
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    drain = torch.zeros(L2_FLUSH_BYTES // 4, dtype=torch.float32, device=device)
    rows = {}
    for T in sweep:
        dev = (workloads.make_hidden(T, HIDDEN, seed=1234).to(device),
               workloads.make_routing(T, EXPERTS, TOP_K, ROUTING, 1235).to(device),
               workloads.make_routing_weights(T, TOP_K, WEIGHT_KIND, 1235).to(device))
        layer = StagedLayer(*dev, gate_up, down, num_experts=EXPERTS, top_k=TOP_K,
                            workspace=B300MoEWorkspace(capacity_tokens=max(sweep), device=device),
                            **extra)
        for _ in range(3):
            layer.forward()
        torch.cuda.synchronize(device)
        timelines, events = [], []
        for _ in range(11):
            flush.fill_(1)
            drain.sum()
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record()
            layer.forward()
            b.record()
            torch.cuda.synchronize(device)
            events.append(a.elapsed_time(b) * 1e3)
            timelines.append(layer.workspace.timeline())
        median = lambda xs: sorted(xs)[len(xs) // 2]  # noqa: E731
        rows[str(T)] = {
            "event_us": round(median(events), 1),
            **{key: [round(median([t[key][0] for t in timelines]), 1),
                     round(median([t[key][1] for t in timelines]), 1)]
               for key in timelines[0]},
        }
    return {"timeline_us_after_routing_start": rows, "weights": args.weights,
            "config": {"workload": WORKLOAD}}


def run_ours(args: argparse.Namespace) -> dict[str, object]:
    from b200moe import (B300MoEWorkspace, StagedLayer, b300_moe_forward,
                         b300_moe_forward_pinned, workloads)

    rank, world, local, dist = dist_setup(args.gpus)
    if world > 1:
        return run_ours_expert_parallel(args, rank, world, local, dist)

    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    sweep = tuple(args.only_tokens) if args.only_tokens else SWEEP
    gate_up, down = workloads.make_expert_weights(
        EXPERTS, HIDDEN, INTER, seed=1236, std=0.02, device=device
    )
    fp8 = None
    if args.weights == "fp8":
        # quantised once, outside every timed region (weights are prepared at load time)
        from b200moe import b300_moe_forward_fp8, quantize_expert_weights_fp8

        global WEIGHT_ELEMENT_BYTES
        WEIGHT_ELEMENT_BYTES = 1
        fp8 = quantize_expert_weights_fp8(gate_up, down)
        torch.cuda.synchronize(device)
    nvfp4 = None
    if args.weights == "nvfp4":
        from b200moe import b300_moe_forward_nvfp4, quantize_expert_weights_nvfp4

        global WEIGHT_FORMAT
        WEIGHT_FORMAT = "nvfp4"
        nvfp4 = quantize_expert_weights_nvfp4(gate_up, down)
        torch.cuda.synchronize(device)
    quantised = fp8 is not None or nvfp4 is not None
    tag = "fp8" if fp8 is not None else "nvfp4" if nvfp4 is not None else None
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    drain = torch.zeros(L2_FLUSH_BYTES // 4, dtype=torch.float32, device=device)

    def flush_l2() -> None:
        # Write a buffer twice the size of L2, then read another one: the read pushes the
        # dirty lines of the write out to HBM, so their write-back does not overlap (and
        # slow down) the timed kernels that follow.
        flush.fill_(1)
        drain.sum()

    cases = {}
    for T in sweep:
        hidden = workloads.make_hidden(T, HIDDEN, seed=1234)
        ids = workloads.make_routing(T, EXPERTS, TOP_K, ROUTING, 1235)
        weights = workloads.make_routing_weights(T, TOP_K, WEIGHT_KIND, 1235)
        host_pack, dev_pack, host, stage_in = packed_step_inputs(hidden, ids, weights, device)
        dev = tuple(t.to(device) for t in host)
        cases[T] = {
            "host": host,
            "dev": dev,
            "host_pack": host_pack,
            "dev_pack": dev_pack,
            "stage_in": stage_in,
            "workspace": B300MoEWorkspace(capacity_tokens=max(sweep), device=device),
            "active": int(torch.unique(ids).numel()),
            "host_out": torch.empty(T, HIDDEN, dtype=torch.bfloat16).pin_memory(),
        }

    def layer_call(inputs, workspace, out=None) -> torch.Tensor:
        if nvfp4 is not None:
            return b300_moe_forward_nvfp4(*inputs, nvfp4, num_experts=EXPERTS, top_k=TOP_K,
                                          workspace=workspace, out=out)
        if fp8 is not None:
            return b300_moe_forward_fp8(*inputs, fp8, num_experts=EXPERTS, top_k=TOP_K,
                                        workspace=workspace, out=out)
        return b300_moe_forward(*inputs, gate_up, down, num_experts=EXPERTS, top_k=TOP_K,
                                backend="cutlass_bf16", workspace=workspace, out=out)

    def forward(T: int) -> torch.Tensor:
        c = cases[T]
        return layer_call(c["dev"], c["workspace"])

    def forward_e2e(T: int) -> torch.Tensor:
        c = cases[T]
        c["dev_pack"].copy_(c["host_pack"], non_blocking=True)  # one copy: all three inputs
        if c["host_out"].numel() * 2 <= DIRECT_OUT_BYTES:
            # the combine kernel stores the result rows straight into the pinned host buffer
            return layer_call(c["stage_in"], c["workspace"], out=c["host_out"])
        out = layer_call(c["stage_in"], c["workspace"])
        c["host_out"].copy_(out, non_blocking=True)
        return out

    def forward_pinned(T: int) -> torch.Tensor:
        if quantised:  # timed for BF16 weights only
            return forward_e2e(T)
        # same end-to-end work without staging copies: the kernels read the pinned host
        # inputs and write the pinned host output themselves
        c = cases[T]
        return b300_moe_forward_pinned(*c["host"], gate_up, down, num_experts=EXPERTS,
                                       top_k=TOP_K, workspace=c["workspace"], out=c["host_out"])

    def timed_pass(fn, steps: int) -> dict[int, list[float]]:
        events = {T: [] for T in sweep}
        for _ in range(steps):
            for T in sweep:
                flush_l2()
                start = torch.cuda.Event(enable_timing=True)
                stop = torch.cuda.Event(enable_timing=True)
                start.record()
                fn(T)
                stop.record()
                events[T].append((start, stop))
        torch.cuda.synchronize(device)
        return {T: [a.elapsed_time(b) * 1e3 for a, b in pairs] for T, pairs in events.items()}

    # cold start: the very first forward of each case (tensor maps encoded, caches cold)
    cold_us = {}
    for T in sweep:
        torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        forward(T)
        torch.cuda.synchronize(device)
        cold_us[T] = (time.perf_counter() - t0) * 1e6

    # warm-up (untimed), then the timed region bracketed by synchronisation
    timed_pass(forward, args.warmup)
    timed_pass(forward_e2e, min(args.warmup, 3))
    torch.cuda.synchronize(device)
    sampler = ClockSampler(local)
    sampler.start()
    wall0 = time.perf_counter()
    samples = timed_pass(forward, args.steps)
    torch.cuda.synchronize(device)
    wall1 = time.perf_counter()
    clocks = sampler.stop()
    e2e_samples = timed_pass(forward_e2e, args.steps)
    torch.cuda.synchronize(device)
    # what the end-to-end path left in host memory is what the device path returns
    for T in sweep:
        if not torch.equal(cases[T]["host_out"], forward(T).cpu()):
            raise SystemExit(f"end-to-end output in host memory differs from the device path at T={T}")
    timed_pass(forward_pinned, 3)
    pinned_samples = timed_pass(forward_pinned, args.steps)
    torch.cuda.synchronize(device)

    # the same forward captured once in a CUDA graph and replayed (how decode loops usually
    # run it): no Python and no per-kernel launch call inside the timed region
    graph_samples = {}
    for T in sweep:
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize(device)
        with torch.cuda.graph(graph):
            forward(T)
        pairs = []
        for _ in range(max(10, min(args.steps, 50))):
            flush_l2()
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            pairs.append((a, b))
        torch.cuda.synchronize(device)
        graph_samples[T] = [a.elapsed_time(b) * 1e3 for a, b in pairs]
        del graph

    # host cost of one call: the time the call takes to return with an empty launch queue
    # (a synchronise before every call, so that no launch waits for queue space behind
    # earlier forwards); median of 30
    host_us = {}
    for T in sweep:
        forward(T)
        times = []
        for _ in range(30):
            torch.cuda.synchronize(device)
            t0 = time.perf_counter_ns()
            forward(T)
            times.append((time.perf_counter_ns() - t0) / 1e3)
        host_us[T] = percentile(sorted(times), 0.5)
    torch.cuda.synchronize(device)

    # per-stage timing through the staged C-ABI entry points (isolated launches)
    peak, peak_kind = measured_peak_gbs()
    per_t: dict[str, object] = {}
    stage_reps = max(10, min(args.steps, 50))
    for T in sweep:
        c = cases[T]
        layer = StagedLayer(*c["dev"], gate_up, down, num_experts=EXPERTS, top_k=TOP_K,
                            workspace=c["workspace"], use_pdl=False, fp8_weights=fp8,
                            nvfp4_weights=nvfp4)
        layer.forward()
        stage_us: dict[str, dict[str, float]] = {}
        for name in STAGE_NAMES:
            pairs = []
            for _ in range(stage_reps):
                flush_l2()
                a = torch.cuda.Event(enable_timing=True)
                b = torch.cuda.Event(enable_timing=True)
                a.record()
                layer.run_stage(name)
                b.record()
                pairs.append((a, b))
            torch.cuda.synchronize(device)
            stage_us[name] = summary([a.elapsed_time(b) * 1e3 for a, b in pairs])
        total = summary(samples[T])
        wb = weight_bytes(c["active"])
        per_t[str(T)] = {
            "active_experts": c["active"],
            "total_us": total,
            "e2e_us": summary(e2e_samples[T]),
            "e2e_pinned_io_us": summary(pinned_samples[T]),
            "graph_replay_us": summary(graph_samples[T]),
            "host_enqueue_us": round(host_us[T], 1),
            "cold_start_us": round(cold_us[T], 1),
            "stage_samples": stage_reps,
            "stages_us": {
                "routing": stage_us["routing"],
                "permutation": stage_us["gather"],
                "gate_up": stage_us["gate_up_swiglu"],
                "swiglu": {"p50": 0.0, "status": "fused_in_gate_up"},
                "down": stage_us["down"],
                "combine": stage_us["combine"],
            },
            "weight_bytes": wb["total"],
            "layer_weight_gbs": round(wb["total"] / total["p50"] / 1e3, 1),
            "layer_frac_of_peak": round(wb["total"] / total["p50"] / 1e3 / peak, 3),
            "gate_up_gbs": round(wb["gate_up"] / stage_us["gate_up_swiglu"]["p50"] / 1e3, 1),
            "down_gbs": round(wb["down"] / stage_us["down"]["p50"] / 1e3, 1),
        }
        if args.library_gemm_baseline and not quantised:
            per_t[str(T)]["library_gemm_us"] = library_gemm_baseline(
                c, gate_up, down, flush_l2, stage_reps)

    p50s = [per_t[str(T)]["total_us"]["p50"] for T in sweep]
    e2e_p50s = [per_t[str(T)]["e2e_us"]["p50"] for T in sweep]
    value = sum(p50s) / len(p50s)
    step_ms = sum(sum(samples[T]) for T in sweep) / args.steps / 1e3

    # roofline of the dominant kernel (gate+up GEMM, 2/3 of the weight bytes) at T=1
    t1 = per_t[str(sweep[0])]
    gu_bytes = weight_bytes(t1["active_experts"])["gate_up"] + 2 * t1["active_experts"] * (
        HIDDEN * 2 + 2 * INTER * 2)  # + token rows in, hi/lo activations out (tiny)
    kernel_name = ("grouped_gemm_fp8_kernel<gate_up> (tcgen05 kind::f8f6f4, SwiGLU epilogue)"
                   if fp8 is not None else
                   "grouped_gemm_nvfp4_kernel<gate_up> (tcgen05 kind::mxf4nvf4 block-scaled, "
                   "SwiGLU epilogue)" if nvfp4 is not None else
                   "grouped_gemm_kernel<gate_up> (tcgen05, SwiGLU epilogue)")
    gu_us = [t1["stages_us"]["gate_up"]["p50"]]
    achieved = gu_bytes / gu_us[0] / 1e3
    roofline = {
        "kernel": f"{kernel_name}, T={sweep[0]}",
        "bound": "hbm",
        "achieved": round(achieved, 1),
        "peak": peak,
        "peak_kind": f"of {peak_kind}",
        "unit": "GB/s",
        "frac": round(achieved / peak, 3),
        "algorithmic_bytes": gu_bytes,
        "frac_of_8000": round(achieved / 8000.0, 3),
    }
    # the captures are of the Mixtral-shaped layer at T=1 (two active experts)
    if args.config == "mixtral" and sweep[0] == 1:
        roofline["traffic"], roofline["traffic_source"] = measured_traffic(
            f"gate_up_mixtral_T1_{tag or 'bf16'}")
    else:
        roofline["traffic"], roofline["traffic_source"] = None, "captured for the mixtral T=1 case only"

    h2d = sum(cases[T]["host_pack"].numel() for T in sweep)
    d2h = sum(cases[T]["host_out"].numel() * 2 for T in sweep)
    result = {
        "metric": METRIC if not quantised else METRIC + f"_{tag}_weights",
        "value": round(value, 2),
        "unit": "us",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(step_ms, 4),
        "wall_ms_per_step": round((wall1 - wall0) * 1e3 / args.steps, 4),
        "higher_is_better": False,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": ("bf16" if not quantised else
                  "fp8_e4m3 weights x bf16 activations, fp32 accumulate" if fp8 is not None else
                  "nvfp4 weights (e2m1, e4m3 block scales) x bf16 activations, fp32 accumulate"),
        "data": "synthetic",
        "config": {
            "workload": WORKLOAD if not quantised else WORKLOAD.replace("_bf16_", f"_{tag}w_"),
            "tokens": list(sweep),
            "step": "one forward at each T of the sweep",
        },
        "l2_policy": L2_POLICY,
        "e2e": {
            "value": round(sum(e2e_p50s) / len(e2e_p50s), 2),
            "unit": "us",
            "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h,
            "what": ("the layer call with the step's activations, routes and routing weights "
                     "copied in from one pinned host buffer (a single host-to-device copy) "
                     "inside the timed region; outputs of at most 256 KB are stored into pinned "
                     "host memory by the combine kernel itself (out=pinned host tensor: the "
                     "d2h bytes cross PCIe inside the kernel), larger ones copied out; expert "
                     "weights resident"),
        },
        "e2e_pinned_io": {
            "value": round(sum(per_t[str(T)]["e2e_pinned_io_us"]["p50"] for T in sweep)
                           / len(sweep), 2),
            "unit": "us",
            "what": "b300_moe_forward_pinned: the same host-resident inputs and output, read and "
                    "written by the kernels directly over PCIe (no staging copies)",
        },
        # BF16: five kernels, four for calls of at most 32 assignments; quantised weights: six
        "gpu_launches": (6 * len(sweep) if quantised else
                         sum(4 if T * TOP_K <= 32 else 5 for T in sweep)) * args.steps,
        "clocks": clocks,
        "roofline": roofline,
        "per_T": per_t,
    }
    if not quantised and not args.no_fp8_extra:
        # the same sweep with NVFP4 expert weights (the reference's cutlass_nvfp4 name)
        try:
            from b200moe import _lib as native, b300_moe_forward_nvfp4, quantize_expert_weights_nvfp4

            if not native.load().b200moe_nvfp4_available():
                raise RuntimeError("the library reports nvfp4_available = 0")
            nw = quantize_expert_weights_nvfp4(gate_up, down)
            torch.cuda.synchronize(device)

            def forward_nvfp4(T: int) -> torch.Tensor:
                c = cases[T]
                return b300_moe_forward_nvfp4(*c["dev"], nw, num_experts=EXPERTS, top_k=TOP_K,
                                              workspace=c["workspace"])

            timed_pass(forward_nvfp4, 3)
            nv_samples = timed_pass(forward_nvfp4, max(10, min(args.steps, 30)))
            nv_p50 = {str(T): summary(nv_samples[T])["p50"] for T in sweep}
            nv_mean = sum(nv_p50.values()) / len(nv_p50)
            result["nvfp4_weights"] = {
                "what": "b300_moe_forward_nvfp4 (backend name cutlass_nvfp4): E2M1 expert weights "
                        "with E4M3 block scales, BF16 activations, same inputs and protocol",
                "value": round(nv_mean, 2),
                "unit": "us",
                "per_T_p50_us": nv_p50,
                "speedup_over_bf16": round(value / nv_mean, 3),
                "weight_bytes_ratio": round(nw.nbytes / (gate_up.numel() * 2 + down.numel() * 2), 4),
            }
            del nw
        except Exception as error:  # never let the extra line break the contract line
            result["nvfp4_weights"] = {"unavailable": f"{type(error).__name__}: {error}"[:200]}
    if fp8 is None and nvfp4 is None and not args.no_fp8_extra:
        # the same sweep with FP8 (E4M3) expert weights, reported beside the BF16 line
        # (a separate entry point and a different weight format: not part of `value`)
        try:
            from b200moe import b300_moe_forward_fp8, quantize_expert_weights_fp8

            fw = quantize_expert_weights_fp8(gate_up, down)
            torch.cuda.synchronize(device)

            def forward_fp8(T: int) -> torch.Tensor:
                c = cases[T]
                return b300_moe_forward_fp8(*c["dev"], fw, num_experts=EXPERTS, top_k=TOP_K,
                                            workspace=c["workspace"])

            timed_pass(forward_fp8, 3)
            fp8_samples = timed_pass(forward_fp8, max(10, min(args.steps, 30)))
            fp8_p50 = {str(T): summary(fp8_samples[T])["p50"] for T in sweep}
            fp8_mean = sum(fp8_p50.values()) / len(fp8_p50)
            result["fp8_weights"] = {
                "what": "b300_moe_forward_fp8: E4M3 expert weights (one FP32 scale per weight "
                        "row), BF16 activations, same inputs, same timing protocol",
                "value": round(fp8_mean, 2),
                "unit": "us",
                "per_T_p50_us": fp8_p50,
                "speedup_over_bf16": round(value / fp8_mean, 3),
                "weight_bytes_ratio": 0.5,
            }
            del fw
        except Exception as error:  # never let the extra line break the contract line
            result["fp8_weights"] = {"unavailable": f"{type(error).__name__}: {error}"[:200]}
    if not args.no_cpu_baseline:
        gate_up_cpu, down_cpu = gate_up.cpu(), down.cpu()
        result["parity"] = single_gpu_parity(forward, cases, gate_up_cpu, down_cpu, sweep)
        result["cpu_baseline"] = cpu_baseline(gate_up_cpu, down_cpu, cases, budget_s=20.0)
        if result["parity"]["status"] != 0:
            print(json.dumps(result), flush=True)
            raise SystemExit(3)
    if args.csv:
        result["csv"] = {"path": args.csv,
                         "rows": write_reference_csv(args.csv, result, args, device)}
    return result


def run_ours_expert_parallel(args, rank: int, world: int, local: int, dist):
    """N > 1: the same layer with its 8 experts sharded over the ranks (E/N per rank).

    Tokens are replicated on every rank (decode after tensor-parallel attention); each rank
    streams only its own active experts' weights and the FP32 partial outputs are summed by
    an all-reduce.  Total work is fixed as N grows (strong scaling): the metric is still the
    layer's P50 latency, now the maximum over ranks of every sample.
    """

    from b200moe import workloads
    from b200moe.expert_parallel import ExpertParallelMoE, expert_range

    device = torch.device("cuda", local)
    base, count = expert_range(rank, world, EXPERTS)
    gate_up, down = workloads.make_expert_weights(count, HIDDEN, INTER, seed=1236 + rank,
                                                  std=0.02, device=device)
    fp8_scales = None
    if args.weights == "nvfp4":
        # ExpertParallelMoE takes NVFP4 weights (nvfp4_scales=...; tests/test_gpu_nvfp4.py), but
        # this benchmark's N-GPU parity step has no NVFP4 leg: refuse rather than time BF16
        raise SystemExit("bench.py --gpus N > 1 supports --weights bf16 and fp8 only")
    if args.weights == "fp8":
        # each rank quantises its own experts once, outside every timed region
        from b200moe import quantize_expert_weights_fp8

        global WEIGHT_ELEMENT_BYTES
        WEIGHT_ELEMENT_BYTES = 1
        fw = quantize_expert_weights_fp8(gate_up, down)
        gate_up, down, fp8_scales = fw.gate_up_q, fw.down_q, (fw.gate_up_scale, fw.down_scale)
        torch.cuda.synchronize(device)
    baseline = ExpertParallelMoE(gate_up, down, num_experts=EXPERTS, top_k=TOP_K,
                                 capacity_tokens=max(SWEEP), transport="nccl",
                                 fp8_scales=fp8_scales)
    transport, transport_note = args.ep_transport, None
    layer = baseline
    if transport == "p2p":
        try:
            layer = ExpertParallelMoE(gate_up, down, num_experts=EXPERTS, top_k=TOP_K,
                                      capacity_tokens=max(SWEEP), transport="p2p",
                                      fp8_scales=fp8_scales)
        except Exception as error:  # peer mapping unavailable on this box: say so, use NCCL
            transport, transport_note = "nccl", f"p2p setup failed: {type(error).__name__}: {error}"
        agree = torch.tensor([1 if transport == "p2p" else 0], device=device)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if int(agree.item()) == 0 and transport == "p2p":
            transport, transport_note, layer = "nccl", "p2p setup failed on another rank", baseline
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    drain = torch.zeros(L2_FLUSH_BYTES // 4, dtype=torch.float32, device=device)
    cases = {}
    for T in SWEEP:
        host_pack, dev_pack, host, stage_in = packed_step_inputs(
            workloads.make_hidden(T, HIDDEN, seed=1234),
            workloads.make_routing(T, EXPERTS, TOP_K, ROUTING, 1235),
            workloads.make_routing_weights(T, TOP_K, WEIGHT_KIND, 1235), device)
        dev = tuple(t.to(device) for t in host)
        ids = host[1]
        local_active = int(torch.unique(ids[(ids >= base) & (ids < base + count)]).numel())
        cases[T] = {"host": host, "dev": dev, "stage_in": stage_in, "host_pack": host_pack,
                    "dev_pack": dev_pack,
                    "host_out": torch.empty(T, HIDDEN, dtype=torch.bfloat16).pin_memory(),
                    "local_active": local_active}

    # parity first, outside every timed region: both transports, both token layouts
    engines = {"nccl": baseline}
    if layer is not baseline:
        engines["p2p"] = layer
    parity = expert_parallel_parity(engines, cases, gate_up, down, base, count, rank, world,
                                    device, dist, fp8_scales)
    if parity["status"] != 0:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "n_gpus": world, "parity": parity,
                              "error": "parity check failed; nothing was timed"}), flush=True)
        dist.barrier()
        raise SystemExit(3)
    if args.parity_only:
        return None if rank != 0 else {"metric": METRIC, "n_gpus": world,
                                       "config": {"workload": WORKLOAD, "tokens": list(SWEEP)},
                                       "parity": parity}

    def forward(T):
        return layer.forward(*cases[T]["dev"], tokens="replicated")

    def forward_e2e(T):
        c = cases[T]
        c["dev_pack"].copy_(c["host_pack"], non_blocking=True)  # one copy: all three inputs
        if layer.transport == "p2p" and c["host_out"].numel() * 2 <= DIRECT_OUT_BYTES:
            # the combine kernel stores this rank's rows straight into the pinned host buffer
            return layer.forward(*c["stage_in"], tokens="replicated", out=c["host_out"])
        out = layer.forward(*c["stage_in"], tokens="replicated")
        c["host_out"].copy_(out, non_blocking=True)
        return out

    def timed_pass(fn, steps):
        events = {T: [] for T in SWEEP}
        for _ in range(steps):
            for T in SWEEP:
                flush.fill_(1)
                drain.sum()
                a = torch.cuda.Event(enable_timing=True)
                b = torch.cuda.Event(enable_timing=True)
                a.record()
                fn(T)
                b.record()
                events[T].append((a, b))
        torch.cuda.synchronize(device)
        return {T: [a.elapsed_time(b) * 1e3 for a, b in pairs] for T, pairs in events.items()}

    def max_over_ranks(samples):
        flat = torch.tensor([samples[T] for T in SWEEP], dtype=torch.float64, device=device)
        dist.all_reduce(flat, op=dist.ReduceOp.MAX)
        return {T: flat[i].tolist() for i, T in enumerate(SWEEP)}

    timed_pass(forward, args.warmup)
    timed_pass(forward_e2e, min(args.warmup, 3))
    dist.barrier()
    torch.cuda.synchronize(device)
    sampler = ClockSampler(local)
    sampler.start()
    wall0 = time.perf_counter()
    samples = timed_pass(forward, args.steps)
    dist.barrier()
    torch.cuda.synchronize(device)
    wall1 = time.perf_counter()
    clocks = sampler.stop()
    e2e_samples = timed_pass(forward_e2e, args.steps)
    torch.cuda.synchronize(device)
    # what the end-to-end path left in host memory is what the device path returns
    for T in SWEEP:
        if not torch.equal(cases[T]["host_out"], forward(T).cpu()):
            raise SystemExit(f"end-to-end output in host memory differs from the device path at T={T}")
    samples = max_over_ranks(samples)
    e2e_samples = max_over_ranks(e2e_samples)
    # the unfused baseline (NCCL all-reduce + cast) on the same inputs, for comparison
    nccl_samples = None
    if layer is not baseline:
        def forward_nccl(T):
            return baseline.forward(*cases[T]["dev"], tokens="replicated")

        timed_pass(forward_nccl, 3)
        nccl_samples = max_over_ranks(timed_pass(forward_nccl, max(5, args.steps // 2)))

    # Sharded tokens (data-parallel attention in front of the layer): each rank holds T/N
    # tokens, stores its shard into every rank's gathered buffers over NVLink (one launch of
    # peer stores + a flag), computes its experts' share for all T tokens and reduces only
    # its own T/N output rows.  Timed for every T of the sweep that divides evenly.
    sharded_T = [T for T in SWEEP if T % world == 0]
    sharded_samples, sharded_nccl_samples = {}, {}
    if sharded_T:
        def shard(T):
            lo, hi = rank * (T // world), (rank + 1) * (T // world)
            return tuple(t[lo:hi].contiguous() for t in cases[T]["dev"])

        shards = {T: shard(T) for T in sharded_T}

        def timed_sharded(engine, steps):
            events = {T: [] for T in sharded_T}
            for _ in range(steps):
                for T in sharded_T:
                    flush.fill_(1)
                    drain.sum()
                    a = torch.cuda.Event(enable_timing=True)
                    b = torch.cuda.Event(enable_timing=True)
                    a.record()
                    engine.forward(*shards[T], tokens="sharded")
                    b.record()
                    events[T].append((a, b))
            torch.cuda.synchronize(device)
            flat = torch.tensor([[a.elapsed_time(b) * 1e3 for a, b in events[T]]
                                 for T in sharded_T], dtype=torch.float64, device=device)
            dist.all_reduce(flat, op=dist.ReduceOp.MAX)
            return {T: flat[i].tolist() for i, T in enumerate(sharded_T)}

        timed_sharded(layer, 3)
        sharded_samples = timed_sharded(layer, args.steps)
        if layer is not baseline:
            timed_sharded(baseline, 3)
            sharded_nccl_samples = timed_sharded(baseline, max(5, args.steps // 2))

    host_us = {}
    for T in SWEEP:
        forward(T)
        times = []
        for _ in range(30):
            torch.cuda.synchronize(device)
            dist.barrier()  # keep the ranks together: a forward waits for its peers
            t0 = time.perf_counter_ns()
            forward(T)
            times.append((time.perf_counter_ns() - t0) / 1e3)
        host_us[T] = percentile(sorted(times), 0.5)
    torch.cuda.synchronize(device)

    # per-rank stage timing of the dominant kernel at the largest T (all local experts active)
    T_big = SWEEP[-1]
    forward(T_big)
    stage_pairs = []
    for _ in range(20):
        flush.fill_(1)
        drain.sum()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        layer.run_local_stage("gate_up_swiglu")
        b.record()
        stage_pairs.append((a, b))
    torch.cuda.synchronize(device)
    gu_us = summary([a.elapsed_time(b) * 1e3 for a, b in stage_pairs])["p50"]
    active_counts = torch.tensor([[cases[T]["local_active"] for T in SWEEP]], device=device)
    gathered = [torch.empty_like(active_counts) for _ in range(world)]
    dist.all_gather(gathered, active_counts)
    active_by_rank = torch.cat(gathered).tolist()
    gu_t = torch.tensor([gu_us], dtype=torch.float64, device=device)
    dist.all_reduce(gu_t, op=dist.ReduceOp.MAX)
    if rank != 0:
        return None

    peak, peak_kind = measured_peak_gbs()
    per_t = {}
    for i, T in enumerate(SWEEP):
        total = summary(samples[T])
        busiest = max(r[i] for r in active_by_rank)
        per_t[str(T)] = {
            "total_us": total,
            "e2e_us": summary(e2e_samples[T]),
            "host_enqueue_us_rank0": round(host_us[T], 1),
            "active_experts_per_rank": [r[i] for r in active_by_rank],
            "busiest_rank_weight_bytes": weight_bytes(busiest)["total"],
            "busiest_rank_weight_gbs": round(weight_bytes(busiest)["total"] / total["p50"] / 1e3, 1),
        }
        if nccl_samples is not None:
            per_t[str(T)]["nccl_allreduce_baseline_us"] = summary(nccl_samples[T])
        if T in sharded_samples:
            per_t[str(T)]["sharded_tokens_us"] = summary(sharded_samples[T])
        if T in sharded_nccl_samples:
            per_t[str(T)]["sharded_tokens_nccl_baseline_us"] = summary(sharded_nccl_samples[T])
    p50s = [per_t[str(T)]["total_us"]["p50"] for T in SWEEP]
    e2e_p50s = [per_t[str(T)]["e2e_us"]["p50"] for T in SWEEP]
    gu_bytes = weight_bytes(max(r[-1] for r in active_by_rank))["gate_up"]
    achieved = gu_bytes / float(gu_t.item()) / 1e3
    h2d = sum(cases[T]["host_pack"].numel() for T in SWEEP)
    d2h = sum(cases[T]["host_out"].numel() * 2 for T in SWEEP)
    return {
        "metric": METRIC if fp8_scales is None else METRIC + "_fp8_weights",
        "value": round(sum(p50s) / len(p50s), 2),
        "unit": "us",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(sum(sum(samples[T]) for T in SWEEP) / args.steps / 1e3, 4),
        "wall_ms_per_step": round((wall1 - wall0) * 1e3 / args.steps, 4),
        "higher_is_better": False,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "bf16" if fp8_scales is None else "fp8_e4m3 weights x bf16 activations, fp32 accumulate",
        "data": "synthetic",
        "config": {
            "workload": WORKLOAD if fp8_scales is None else WORKLOAD.replace("_bf16_", "_fp8w_"),
            "tokens": list(SWEEP),
            "step": "one forward at each T of the sweep",
        },
        "parallelism": {
            "kind": f"expert-parallel ep{world}: {EXPERTS // world} experts per rank, tokens "
                    "replicated, rows combined and reduced across ranks by "
                    + ("one peer-memory kernel over NVLink (b200moe_ep_combine_reduce)"
                       if transport == "p2p" else "combine kernel + NCCL all-reduce + cast"),
            "transport": transport,
            "transport_note": transport_note,
            "sample": "every sample is the max over ranks",
        },
        "l2_policy": L2_POLICY,
        "parity": parity,
        "e2e": {"value": round(sum(e2e_p50s) / len(e2e_p50s), 2), "unit": "us",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "what": "ExpertParallelMoE.forward with the step's inputs copied in from one "
                        "pinned host buffer (a single copy) inside the timed region, per rank; "
                        + ("outputs of at most 256 KB are stored into pinned host memory by "
                           "the cross-rank combine kernel itself (out=), larger ones copied out"
                           if transport == "p2p" else
                           "the output copied out inside the timed region")},
        "gpu_launches": ((6 if transport == "p2p" else 5) + (1 if fp8_scales is not None else 0))
                        * len(SWEEP) * args.steps * world,
        "clocks": clocks,
        "roofline": {
            "kernel": f"grouped_gemm_kernel<gate_up> on the busiest rank, T={T_big}",
            "bound": "hbm", "achieved": round(achieved, 1), "peak": peak,
            "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": round(achieved / peak, 3),
            "algorithmic_bytes": gu_bytes, "traffic": None,
        },
        "per_T": per_t,
    }


# -----------------------------------------------------------------------------
# CPU arms: the reference's torch backend on the host cores
# -----------------------------------------------------------------------------
REFERENCE_COPY = REPO / "baseline" / "_ref"
REFERENCE_PACKAGES = ("fastpath", "baseline")


def prepare_reference(source: str) -> str:
    """Copy the reference's two pure-Python packages, unmodified, into ``baseline/_ref``.

    The directory is listed in ``.gitignore`` (it is not this repository's code) but travels
    with the working tree, so ``--impl reference`` can import the real reference on a
    machine that has no checkout of it.  Returns a one-line description of what was done.
    """

    import shutil

    root = Path(source)
    missing = [name for name in REFERENCE_PACKAGES if not (root / name / "__init__.py").exists()]
    if missing:
        return f"not prepared: {root} has no {', '.join(missing)} package"
    REFERENCE_COPY.mkdir(parents=True, exist_ok=True)
    for name in REFERENCE_PACKAGES:
        target = REFERENCE_COPY / name
        if target.exists():
            shutil.rmtree(target)
        shutil.copytree(root / name, target, ignore=shutil.ignore_patterns("__pycache__", "*.so"))
    return f"copied {', '.join(REFERENCE_PACKAGES)} from {root} to {REFERENCE_COPY}"


def reference_forward():
    """``(callable, kind, note)``: the reference's ``b300_moe_forward`` from ``baseline/_ref``
    when that copy exists (kind ``"reference"``), else the oracle's restatement of the same
    torch path (kind ``"port"``)."""

    if (REFERENCE_COPY / "fastpath" / "__init__.py").exists():
        try:
            if str(REFERENCE_COPY) not in sys.path:
                sys.path.insert(0, str(REFERENCE_COPY))
            import fastpath  # the reference package, unmodified

            def run(hidden, ids, weights, gate_up, down):
                return fastpath.b300_moe_forward(hidden, ids, weights, gate_up, down,
                                                 num_experts=EXPERTS, top_k=TOP_K,
                                                 backend="torch")

            return run, "reference", ("fastpath.b300_moe_forward(backend='torch') imported from "
                                      "baseline/_ref (unmodified copy of the reference package)")
        except Exception as error:  # say why, then time the restatement
            note = f"baseline/_ref could not be imported ({type(error).__name__}: {error}); "
    else:
        note = "no baseline/_ref on this machine; "
    from oracle import moe_oracle

    def run_port(hidden, ids, weights, gate_up, down):
        out, _ = moe_oracle.routed_moe(hidden, ids, weights, gate_up, down, num_experts=EXPERTS,
                                       top_k=TOP_K, compute_dtype=torch.bfloat16)
        return out

    return run_port, "port", note + "timed the restatement in oracle/moe_oracle.py"


def host_threads() -> int:
    """All the cores this process may run on (torchrun exports OMP_NUM_THREADS=1)."""

    try:
        count = max(1, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        count = max(1, os.cpu_count() or 1)
    try:
        torch.set_num_threads(count)
    except RuntimeError:
        pass
    return torch.get_num_threads()


def time_cpu_path(run, cases_host, gate_up_cpu, down_cpu, warmup: int, reps: int,
                  budget_s: float | None = None) -> tuple[dict[int, list[float]], float]:
    """The one timing loop of both CPU legs: ``warmup`` untimed passes over the sweep, then
    ``reps`` timed passes (``time.perf_counter_ns`` around each forward).  Returns the
    samples in microseconds per T and the wall time of the timed passes."""

    for _ in range(warmup):
        for T in cases_host:
            run(*cases_host[T], gate_up_cpu, down_cpu)
    samples: dict[int, list[float]] = {T: [] for T in cases_host}
    start = time.perf_counter()
    for _ in range(reps):
        for T in cases_host:
            t0 = time.perf_counter_ns()
            run(*cases_host[T], gate_up_cpu, down_cpu)
            samples[T].append((time.perf_counter_ns() - t0) / 1e3)
        if budget_s is not None and time.perf_counter() - start > budget_s:
            break
    return samples, time.perf_counter() - start


def cpu_baseline(gate_up_cpu, down_cpu, cases, budget_s: float) -> dict[str, object]:
    """The reference's BF16 torch path on the host cores, bounded sample (our arm's leg)."""

    run, kind, note = reference_forward()
    cores = host_threads()
    cases_host = {T: tuple(t.clone() for t in cases[T]["host"]) for T in cases}
    samples, _ = time_cpu_path(run, cases_host, gate_up_cpu, down_cpu, warmup=2, reps=5,
                               budget_s=budget_s)
    per_t = {str(T): round(percentile(sorted(v), 0.5), 1) for T, v in samples.items() if v}
    done = list(per_t.values())
    return {
        "value": round(sum(done) / len(done), 1),
        "unit": "us",
        "cores": cores,
        "host_cpus": os.cpu_count(),
        "kind": kind,
        "note": note,
        "sample": f"2 warm-up + up to 5 forwards at each T in {sorted(int(k) for k in per_t)} of "
                  "the same workload (BF16 tensors, the reference's torch backend), "
                  f"bounded to {budget_s:.0f} s",
        "per_T_p50_us": per_t,
    }


def run_reference(args: argparse.Namespace) -> dict[str, object] | None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    from b200moe import workloads

    run, kind, note = reference_forward()
    cores = host_threads()
    gate_up, down = workloads.make_expert_weights(EXPERTS, HIDDEN, INTER, seed=1236, std=0.02,
                                                  device="cpu")
    cases = {}
    for T in SWEEP:
        cases[T] = (workloads.make_hidden(T, HIDDEN, seed=1234),
                    workloads.make_routing(T, EXPERTS, TOP_K, ROUTING, 1235),
                    workloads.make_routing_weights(T, TOP_K, WEIGHT_KIND, 1235))
    samples, wall = time_cpu_path(run, cases, gate_up, down, warmup=max(args.warmup, 1),
                                  reps=args.steps)
    p50s = [percentile(sorted(samples[T]), 0.5) for T in SWEEP]
    value = round(sum(p50s) / len(p50s), 1)
    sample = ("every T of the sweep, whole workload, BF16 tensors through the reference's torch "
              "backend on the host CPU")
    return {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": "us",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(wall * 1e3 / args.steps, 3),
        "higher_is_better": False,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens": list(SWEEP),
                   "step": "one forward at each T of the sweep"},
        "cpu_baseline": {"value": value, "unit": "us", "cores": cores, "kind": kind,
                         "note": note, "sample": sample},
        "e2e": {"value": value, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "per_T_p50_us": {str(T): round(p, 1) for T, p in zip(SWEEP, p50s)},
    }


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=None)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--config", choices=tuple(CONFIGS), default="mixtral",
                        help="benchmark configuration (default: the Mixtral-shaped sweep)")
    parser.add_argument("--ep-transport", choices=("p2p", "nccl"), default="p2p",
                        help="N > 1: combine over NVLink peer memory (default) or NCCL")
    parser.add_argument("--only-tokens", type=int, nargs="*", default=None,
                        help="restrict the sweep (profiling runs); the default is the full sweep")
    parser.add_argument("--weights", choices=("bf16", "fp8", "nvfp4"), default="bf16",
                        help="bf16 (default, the configuration the metric is quoted on) or "
                             "fp8: E4M3 expert weights (b300_moe_forward_fp8 / fp8_scales)")
    parser.add_argument("--no-fp8-extra", action="store_true",
                        help="N=1, BF16 run: skip the extra FP8-weight sweep reported as `fp8_weights`")
    parser.add_argument("--csv", default=None,
                        help="N=1: also write per-stage rows in the reference's CSV schema")
    parser.add_argument("--library-gemm-baseline", action="store_true",
                        help="N=1: also time torch._grouped_mm and the per-expert matmul loop "
                             "(the library GEMMs the reference's compiled path calls)")
    parser.add_argument("--parity-only", action="store_true",
                        help="N > 1: run the parity check of every token layout and transport "
                             "against the oracle, print it and exit without timing anything")
    parser.add_argument("--timeline", action="store_true",
                        help="N=1: print the device timeline of one forward per T (in-kernel "
                             "timer stamps) instead of the benchmark line")
    parser.add_argument("--prepare-reference", nargs="?", const="/root/reference", default=None,
                        metavar="CHECKOUT",
                        help="copy the reference's fastpath/ and baseline/ packages from CHECKOUT "
                             "into baseline/_ref (for --impl reference) and exit")
    args = parser.parse_args()
    if args.prepare_reference is not None:
        print(prepare_reference(args.prepare_reference))
        return 0
    apply_config(args.config)
    if args.weights != "bf16":
        args.no_cpu_baseline = True  # the CPU legs run the reference's BF16 layer
    if args.config in ("wide", "wide_e16", "deepseek", "deepseek_hotspot"):
        args.no_cpu_baseline = True  # ~21 GiB of weights: the CPU port is not timed on these
    if args.timeline:
        print(json.dumps(run_timeline(args)), flush=True)
        return 0
    if args.impl == "reference":
        args.steps = 3 if args.steps is None else args.steps
        args.warmup = 1 if args.warmup is None else args.warmup
        result = run_reference(args)
    else:
        args.steps = 100 if args.steps is None else args.steps
        args.warmup = 10 if args.warmup is None else max(args.warmup, 3)
        result = run_ours(args)
    if result is not None:
        print(json.dumps(result), flush=True)
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
