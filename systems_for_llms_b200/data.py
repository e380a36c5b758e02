"""Token data: synthetic or memory-mapped ``.npy`` arrays, identities and batching.

Behaviour follows the reference (src/llmlab/data.py:18-56): two arrays (train,
valid), a sha256 identity per array plus tokenizer file hashes, range checks,
and windows of ``context_length + 1`` tokens split into inputs and next-token
targets.  On CUDA the windows are staged in pinned host memory and copied
asynchronously, so the host-to-device transfer overlaps the previous
microbatch's kernels instead of blocking on a pageable copy.
"""

from __future__ import annotations

import hashlib
from pathlib import Path

import numpy as np
import torch

from .config import TrainConfig


def file_sha256(path: str | Path) -> str:
    digest = hashlib.sha256()
    with open(path, "rb") as handle:
        while chunk := handle.read(1 << 20):
            digest.update(chunk)
    return digest.hexdigest()


def _array_identity(array: np.ndarray, digest: str) -> dict:
    return {"sha256": digest, "tokens": len(array), "dtype": str(array.dtype)}


def load_data(config: TrainConfig) -> tuple[np.ndarray, np.ndarray, dict]:
    """Returns ``(train_tokens, valid_tokens, identity)``."""
    if config.data.kind == "synthetic":
        generator = np.random.default_rng(config.seed)
        arrays = []
        for _ in ("train", "valid"):
            arrays.append(generator.integers(0, config.model.vocab_size,
                                             size=config.data.synthetic_tokens, dtype=np.int64))
        identities = [_array_identity(a, hashlib.sha256(a.tobytes()).hexdigest()) for a in arrays]
    else:
        locations = (config.data.train_path, config.data.valid_path)
        arrays = [np.load(location, mmap_mode="r", allow_pickle=False) for location in locations]
        identities = [_array_identity(a, file_sha256(location))
                      for a, location in zip(arrays, locations)]
    for array in arrays:
        if array.ndim != 1 or not np.issubdtype(array.dtype, np.integer):
            raise ValueError("token data must be a one-dimensional integer array")
        if len(array) <= config.model.context_length:
            raise ValueError("token data must exceed the context length")
        if array.min() < 0 or array.max() >= config.model.vocab_size:
            raise ValueError("token ID outside model vocabulary")
    tokenizer = [{"name": Path(item).name, "sha256": file_sha256(item)}
                 for item in config.data.tokenizer_files]
    identity = {"kind": config.data.kind, "train": identities[0], "valid": identities[1],
                "tokenizer_files": tokenizer}
    return arrays[0], arrays[1], identity


def gather_windows(data: np.ndarray, starts, context_length: int) -> torch.Tensor:
    """Host tensor ``[len(starts), context_length + 1]`` of int64 token windows."""
    starts = np.asarray(starts, dtype=np.int64)
    offsets = np.arange(context_length + 1, dtype=np.int64)
    windows = np.asarray(data[starts[:, None] + offsets[None, :]], dtype=np.int64)
    return torch.from_numpy(windows)


def batch_at(data: np.ndarray, starts, context_length: int,
             device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Inputs and next-token targets for the windows beginning at ``starts``."""
    tokens = gather_windows(data, starts, context_length)
    device = torch.device(device)
    if device.type == "cuda":
        tokens = tokens.pin_memory().to(device, non_blocking=True)
    else:
        tokens = tokens.to(device)
    return tokens[:, :-1], tokens[:, 1:]


def sample_batch(data: np.ndarray, config: TrainConfig, generator: torch.Generator,
                 device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    starts = torch.randint(len(data) - config.model.context_length, (config.batch_size,),
                           generator=generator).tolist()
    return batch_at(data, starts, config.model.context_length, device)
