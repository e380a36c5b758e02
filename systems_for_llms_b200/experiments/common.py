"""Utilities shared by the experiment planners, executors and analysers.

Plans are JSON documents that carry their own hash; cases run as subprocesses
with a timeout and a process-group kill; evidence files are written atomically
and never overwritten.  These conventions come from the reference's harness
(src/llmlab/pilot.py, distributed/run_experiments.py) and are collected here so
every planner in this package behaves the same way.
"""

from __future__ import annotations

import hashlib
import json
import math
import os
import signal
import subprocess
import time
from pathlib import Path

REPO_ROOT = Path(__file__).resolve().parents[2]


def json_sha256(value) -> str:
    return hashlib.sha256(json.dumps(value, sort_keys=True, allow_nan=False).encode()).hexdigest()


def file_sha256(path: str | Path) -> str:
    digest = hashlib.sha256()
    with open(path, "rb") as handle:
        while block := handle.read(1 << 20):
            digest.update(block)
    return digest.hexdigest()


def write_json(path: str | Path, value, *, exclusive: bool = False) -> None:
    """Atomic write; ``exclusive`` refuses to replace an existing file."""
    path = Path(path)
    if exclusive and path.exists():
        raise FileExistsError(f"refusing to overwrite {path}")
    temporary = path.with_name(path.name + ".tmp")
    temporary.write_text(json.dumps(value, indent=2, allow_nan=False) + "\n")
    os.replace(temporary, path)


def read_json(path: str | Path):
    return json.loads(Path(path).read_text())


def read_jsonl(path: str | Path) -> list[dict]:
    return [json.loads(line) for line in Path(path).read_text().splitlines() if line.strip()]


def is_finite(value, *, positive: bool = False, nonnegative: bool = False) -> bool:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
        return False
    if positive and value <= 0:
        return False
    return not (nonnegative and value < 0)


def percentile_linear(values: list[float], fraction: float) -> float:
    """Linear interpolation at ``fraction * (n - 1)`` (the reference's p90 rule)."""
    ordered = sorted(values)
    position = fraction * (len(ordered) - 1)
    low, high = math.floor(position), math.ceil(position)
    return ordered[low] + (ordered[high] - ordered[low]) * (position - low)


def geometric_mean(values: list[float]) -> float:
    return math.exp(sum(math.log(v) for v in values) / len(values))


def seal(document: dict, key: str = "plan_sha256") -> dict:
    """Adds the hash of everything else under ``key``."""
    body = {k: v for k, v in document.items() if k != key}
    document[key] = json_sha256(body)
    return document


def verify_seal(document: dict, key: str = "plan_sha256") -> bool:
    body = {k: v for k, v in document.items() if k != key}
    return document.get(key) == json_sha256(body)


def classify_failure(text: str) -> str:
    lowered = text.lower()
    if "out of memory" in lowered or "outofmemoryerror" in lowered:
        return "oom"
    if "illegal memory access" in lowered or "device-side assert" in lowered:
        return "device_fault"
    return "process_error"


def run_case(command: list[str], *, log_path: Path, timeout: float, cwd: Path | None = None,
             env: dict | None = None) -> dict:
    """Runs one case in its own process group; on timeout the whole group gets
    SIGTERM, then SIGKILL.  Returns status / returncode / wall time / error."""
    started = time.perf_counter()
    record = {"command": command, "status": "running", "returncode": None}
    with open(log_path, "w") as log:
        try:
            process = subprocess.Popen(command, cwd=cwd, env=env, stdout=log,
                                       stderr=subprocess.STDOUT, start_new_session=True)
        except OSError as error:
            record.update(status="failed", error=str(error),
                          wall_seconds=time.perf_counter() - started)
            return record
        try:
            code = process.wait(timeout=timeout)
            record.update(status="completed" if code == 0 else "failed", returncode=code)
            if code:
                record["error"] = f"process exited with code {code}; see {log_path.name}"
        except subprocess.TimeoutExpired:
            stop_group(process)
            record.update(status="timeout", error=f"case exceeded {timeout} seconds")
    record["wall_seconds"] = time.perf_counter() - started
    if record["status"] == "failed":
        try:
            tail = Path(log_path).read_text(errors="replace")[-4000:]
        except OSError:
            tail = ""
        record["failure_kind"] = classify_failure(record.get("error", "") + tail)
    elif record["status"] == "timeout":
        record["failure_kind"] = "timeout"
    return record


def stop_group(process: subprocess.Popen, grace: float = 5.0) -> None:
    """Terminate exactly the process group this process started."""
    try:
        os.killpg(process.pid, signal.SIGTERM)
    except ProcessLookupError:
        return
    try:
        process.wait(timeout=grace)
    except subprocess.TimeoutExpired:
        try:
            os.killpg(process.pid, signal.SIGKILL)
        except ProcessLookupError:
            pass
        process.wait()


def child_environment(extra: dict | None = None) -> dict:
    env = os.environ.copy()
    env["PYTHONDONTWRITEBYTECODE"] = "1"
    env["PYTHONPATH"] = str(REPO_ROOT) + os.pathsep + env.get("PYTHONPATH", "")
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    if extra:
        env.update(extra)
    return env
