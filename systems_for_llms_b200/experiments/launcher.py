"""Host-side launcher: payload manifest, preflight, test gate, study, evidence.

The reference ships its studies to rented GPUs through Modal
(distributed/run_modal.py:21-355, scripts/modal_pilot.py).  There is no network
here, so this launcher runs the same pipeline on the machine it is started on
(locally, or on a GPU box through whatever transports the tree there):

    prepare_payload   explicit file list with hashes; symlinks and missing files
                      are refused, nothing outside the list is shipped
    validate_options  stage / GPU count / timeout sanity, GPU-minute estimate
    preflight         GPU count, native bf16, names, memory, capability, peer
                      access matrix, ``nvidia-smi topo -m`` (diagnostics that fail
                      are recorded as warnings, never fatal)
    run_gate          the full test suite with a junit report; any failure,
                      error or skip stops the launch (zero skips required on a
                      GPU host)
    run_stage         ``distributed_plan.run_plan`` for the chosen stage
    collect_evidence  JSON / JSONL files and bounded log tails, never tensors,
                      with path-traversal checks

``run_pipeline`` strings these together and writes ``launch-summary.json``.
"""

from __future__ import annotations

import argparse
import json
import subprocess
import sys
import time
import xml.etree.ElementTree as ElementTree
from pathlib import Path

from . import common
from . import distributed_plan as planner

PAYLOAD_PATTERNS = ("systems_for_llms_b200/**/*.py", "systems_for_llms_b200/csrc/*",
                    "llmlab/**/*.py", "llmdist/**/*.py", "attention_lab/**/*.py", "configs/*.json",
                    "tests/**/*.py", "bench.py", "__graft_entry__.py")
LOG_TAIL_BYTES = 16000
EVIDENCE_SUFFIXES = (".json", ".jsonl")

PREFLIGHT_SCRIPT = r"""
import json, subprocess, sys
import torch

expected = int(sys.argv[2])
found = torch.cuda.device_count()
if found < expected:
    raise RuntimeError(f"Expected at least {expected} CUDA GPUs; found {found}")
warnings, devices = [], []
for index in range(expected):
    torch.cuda.set_device(index)
    if not torch.cuda.is_bf16_supported(including_emulation=False):
        raise RuntimeError(f"GPU {index} lacks native BF16 support")
    props = torch.cuda.get_device_properties(index)
    devices.append({"index": index, "name": props.name,
                    "uuid": str(getattr(props, "uuid", "unavailable")),
                    "memory_bytes": props.total_memory,
                    "capability": list(torch.cuda.get_device_capability(index))})


def query(command):
    try:
        done = subprocess.run(command, capture_output=True, text=True, timeout=30)
        status = "completed" if done.returncode == 0 else "unavailable"
        report = {"command": command, "status": status, "returncode": done.returncode,
                  "stdout": done.stdout, "stderr": done.stderr}
    except subprocess.TimeoutExpired as error:
        report = {"command": command, "status": "timeout", "returncode": None,
                  "stdout": "", "stderr": str(error)}
    except OSError as error:
        report = {"command": command, "status": "unavailable", "returncode": None,
                  "stdout": "", "stderr": str(error)}
    if report["status"] != "completed":
        warnings.append(" ".join(command) + ": " + report["status"])
    return report


topology = query(["nvidia-smi", "topo", "-m"])
identities = query(["nvidia-smi", "--query-gpu=uuid,name,pci.bus_id", "--format=csv,noheader"])
peers = []
for i in range(expected):
    row = []
    for j in range(expected):
        try:
            row.append(True if i == j else bool(torch.cuda.can_device_access_peer(i, j)))
        except RuntimeError as error:
            row.append(None)
            warnings.append(f"Peer-access query {i}->{j} unavailable: {error}")
    peers.append(row)
report = {"devices": devices, "torch": torch.__version__, "cuda": torch.version.cuda,
          "peer_access": peers,
          "nvidia_smi_topology": topology["stdout"] if topology["status"] == "completed" else None,
          "nvidia_smi_identities": identities["stdout"] if identities["status"] == "completed" else None,
          "nvidia_smi_diagnostics": {"topology": topology, "identities": identities},
          "warnings": warnings}
with open(sys.argv[1], "w") as handle:
    json.dump(report, handle, indent=2)
print(json.dumps({"devices": devices, "warnings": warnings}, indent=2))
"""


def prepare_payload(root: Path = common.REPO_ROOT, patterns=PAYLOAD_PATTERNS) -> dict:
    """Explicit manifest of what a launch ships: relative path -> sha256."""
    root = Path(root).resolve()
    files = {}
    for pattern in patterns:
        matches = sorted(root.glob(pattern))
        if not matches and "*" not in pattern:
            raise FileNotFoundError(f"payload file is missing: {pattern}")
        for path in matches:
            if path.is_dir() or "__pycache__" in path.parts or path.suffix in (".so", ".o"):
                continue
            if path.is_symlink():
                raise ValueError(f"payload must not contain symlinks: {path}")
            files[str(path.relative_to(root))] = common.file_sha256(path)
    if not files:
        raise ValueError("payload is empty")
    return {"format_version": 1, "root": str(root), "file_count": len(files), "files": files,
            "payload_sha256": common.json_sha256(files)}


def verify_payload(manifest: dict, root: Path | None = None) -> None:
    root = Path(root or manifest["root"])
    for relative, digest in manifest["files"].items():
        path = root / relative
        if not path.is_file() or common.file_sha256(path) != digest:
            raise ValueError(f"source changed after the payload was frozen: {relative}")


def validate_options(options: dict) -> dict:
    stage = options.get("stage")
    if stage not in planner.STAGES:
        raise ValueError(f"stage must be one of {', '.join(planner.STAGES)}")
    gpus = options.get("gpus")
    if type(gpus) is not int or gpus not in (1, 2, 4, 8):
        raise ValueError("gpus must be 1, 2, 4 or 8")
    plan = planner.build_plan(stage)
    if gpus < plan["required_gpus"]:
        raise ValueError(f"stage {stage} needs {plan['required_gpus']} GPUs")
    timeout = options.get("timeout_seconds", 3600)
    if not common.is_finite(timeout, positive=True):
        raise ValueError("timeout_seconds must be finite and positive")
    if options.get("device", "cuda") not in ("cuda", "cpu"):
        raise ValueError("device must be cuda or cpu")
    return {"stage": stage, "gpus": gpus, "timeout_seconds": float(timeout),
            "device": options.get("device", "cuda"), "skip_tests": bool(options.get("skip_tests")),
            "plan": plan, "estimate": cost_estimate(plan, gpus)}


def cost_estimate(plan: dict, gpus: int) -> dict:
    """Upper bound on GPU-minutes: every case at its timeout on all allocated GPUs."""
    worst = sum(case["timeout_seconds"] for case in plan["cases"])
    return {"cases": len(plan["cases"]), "allocated_gpus": gpus,
            "worst_case_wall_minutes": worst / 60, "worst_case_gpu_minutes": worst * gpus / 60,
            "scope": "per-case timeouts only; excludes setup, tests and evidence collection"}


def preflight(output: Path, gpus: int) -> dict:
    script = output / "preflight.py"
    script.write_text(PREFLIGHT_SCRIPT)
    report_path = output / "preflight.json"
    done = subprocess.run([sys.executable, str(script), str(report_path), str(gpus)],
                          capture_output=True, text=True, timeout=300)
    if done.returncode != 0:
        raise RuntimeError("preflight failed: " + done.stderr[-2000:])
    return common.read_json(report_path)


def parse_junit(path: Path) -> dict:
    root = ElementTree.parse(path).getroot()
    suites = [root] if root.tag == "testsuite" else list(root.iter("testsuite"))
    report = {"tests": 0, "failures": 0, "errors": 0, "skipped": 0, "nonpassing": []}
    for suite in suites:
        for key in ("tests", "failures", "errors", "skipped"):
            report[key] += int(suite.get(key, 0))
        for case in suite.iter("testcase"):
            for tag in ("failure", "error", "skipped"):
                if case.find(tag) is not None:
                    report["nonpassing"].append({"name": case.get("name"),
                                                 "class": case.get("classname"), "status": tag})
    report["passed"] = report["tests"] - report["failures"] - report["errors"] - report["skipped"]
    return report


def run_gate(output: Path, *, device: str, timeout: float) -> dict:
    """Full test suite; on a GPU host nothing may be skipped."""
    junit = output / "tests.xml"
    marker = [] if device == "cuda" else ["-m", "not gpu"]
    command = [sys.executable, "-m", "pytest", "tests", "-q", f"--junitxml={junit}", *marker]
    record = common.run_case(command, log_path=output / "tests.log", timeout=timeout,
                             cwd=common.REPO_ROOT, env=common.child_environment())
    report = parse_junit(junit) if junit.exists() else {"tests": 0, "failures": 1, "errors": 0,
                                                        "skipped": 0, "nonpassing": []}
    report["returncode"] = record["returncode"]
    clean = record["status"] == "completed" and report["failures"] == report["errors"] == 0
    if device == "cuda":
        clean = clean and report["skipped"] == 0
    report["gate"] = "passed" if clean else "failed"
    return report


def collect_evidence(run_dir: Path, *, log_tail_bytes: int = LOG_TAIL_BYTES) -> dict:
    """Small text artefacts only (JSON, JSONL, log tails); checkpoints stay behind."""
    run_dir = Path(run_dir).resolve()
    files, logs = {}, {}
    for path in sorted(run_dir.rglob("*")):
        if not path.is_file() or path.is_symlink():
            continue
        resolved = path.resolve()
        if run_dir not in resolved.parents:
            raise ValueError(f"evidence path escapes the run directory: {path}")
        relative = str(path.relative_to(run_dir))
        if path.suffix in EVIDENCE_SUFFIXES and path.stat().st_size <= 8 << 20:
            files[relative] = path.read_text(errors="replace")
        elif path.suffix == ".log":
            data = path.read_bytes()
            logs[relative] = {"bytes": len(data),
                              "tail": data[-log_tail_bytes:].decode(errors="replace")}
    return {"format_version": 1, "files": files, "logs": logs,
            "evidence_sha256": common.json_sha256({"files": files, "logs": logs})}


def run_pipeline(options: dict, base_config: dict, output: Path) -> dict:
    """preflight -> test gate -> stage; writes ``launch-summary.json``."""
    options = validate_options(options)
    output = Path(output)
    output.mkdir(parents=True, exist_ok=False)
    started = time.monotonic()
    manifest = prepare_payload()
    common.write_json(output / "payload.json", manifest)
    summary = {"format_version": 1, "stage": options["stage"], "gpus": options["gpus"],
               "payload_sha256": manifest["payload_sha256"], "estimate": options["estimate"],
               "status": "running"}
    try:
        if options["device"] == "cuda":
            summary["preflight"] = preflight(output, options["gpus"])
        if not options["skip_tests"]:
            summary["tests"] = run_gate(output, device=options["device"],
                                        timeout=options["timeout_seconds"])
            if summary["tests"]["gate"] != "passed":
                raise RuntimeError("test gate failed; the study was not started")
        verify_payload(manifest)
        aggregate = planner.run_plan(options["plan"], base_config, output / "study",
                                     device=options["device"], allocated_gpus=options["gpus"])
        summary["study_status"] = aggregate["status"]
        summary["status"] = "completed" if aggregate["status"] == "completed" else "failed"
    except Exception as error:
        summary["status"] = "failed"
        summary["error"] = str(error)
    summary["wall_seconds"] = time.monotonic() - started
    common.write_json(output / "launch-summary.json", summary)
    common.write_json(output / "evidence.json", collect_evidence(output))
    return summary


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--stage", choices=planner.STAGES, default="smoke")
    parser.add_argument("--gpus", type=int, default=2)
    parser.add_argument("--config", type=Path, required=True)
    parser.add_argument("--output-dir", type=Path, required=True)
    parser.add_argument("--device", choices=["cuda", "cpu"], default="cuda")
    parser.add_argument("--timeout-seconds", type=float, default=3600)
    parser.add_argument("--skip-tests", action="store_true")
    parser.add_argument("--execute", action="store_true",
                        help="without this flag only the validated options are printed")
    args = parser.parse_args()
    options = {"stage": args.stage, "gpus": args.gpus, "device": args.device,
               "timeout_seconds": args.timeout_seconds, "skip_tests": args.skip_tests}
    checked = validate_options(options)
    if not args.execute:
        print(json.dumps({k: v for k, v in checked.items() if k != "plan"}, indent=2))
        return
    summary = run_pipeline(options, common.read_json(args.config), args.output_dir)
    print(json.dumps({"status": summary["status"], "error": summary.get("error")}, indent=2))
    if summary["status"] != "completed":
        raise SystemExit(1)


if __name__ == "__main__":
    main()
