"""Wire helpers of the generate endpoints: log-prob flooring and compact packing of routed-expert indices
(reference: skyrl/backends/skyrl_train/inference_servers/generate_wire.py:22-106)."""

from __future__ import annotations

import base64
import math
from typing import Any, Dict, Iterable, List, Optional, Tuple

import numpy as np

CLAMPED_LOGPROB = -9999.0
_DTYPES = {"uint8": np.dtype("uint8"), "uint16": np.dtype("uint16"), "int32": np.dtype("int32")}


def build_logprobs_content(logprobs: Iterable[Optional[float]]) -> Tuple[List[Dict[str, float]], int]:
    """``logprobs.content`` entries; missing, NaN and infinite values are floored. Returns (content, n_clamped)."""
    content, clamped = [], 0
    for lp in logprobs:
        if lp is None or not math.isfinite(lp):
            lp = CLAMPED_LOGPROB
            clamped += 1
        content.append({"logprob": float(lp)})
    return content, clamped


def compact_routed_expert_indices(arr: Any) -> np.ndarray:
    """``[tokens, layers, top_k]`` integer array in the narrowest canonical dtype."""
    for m in ("detach", "cpu", "numpy"):
        op = getattr(arr, m, None)
        if callable(op):
            arr = op()
    if not isinstance(arr, np.ndarray):
        raise TypeError("routed expert indices must be an array, not nested lists")
    if arr.ndim != 3 or arr.dtype.kind not in "iu":
        raise ValueError(f"routed expert indices must be a 3-D integer array, got {arr.dtype} with shape {arr.shape}")
    if arr.size and arr.min() < 0:
        raise ValueError("routed expert indices must be non-negative")
    hi = int(arr.max()) if arr.size else 0
    dt = np.uint8 if hi < 256 else (np.uint16 if hi < 65536 else np.int32)
    return np.ascontiguousarray(arr.astype(dt, copy=False))


def pack_routed_experts(arr: Any) -> Dict[str, Any]:
    c = compact_routed_expert_indices(arr)
    return {"data": base64.b64encode(memoryview(c)).decode("ascii"), "shape": list(c.shape), "dtype": c.dtype.name}


def decode_packed_routed_experts(payload: Dict[str, Any]) -> np.ndarray:
    if not isinstance(payload, dict):
        raise TypeError("packed routed expert indices must be an object")
    try:
        dt = _DTYPES[payload["dtype"]]
        shape = tuple(payload["shape"])
        data = base64.b64decode(payload["data"], validate=True)
    except (KeyError, TypeError, ValueError) as e:
        raise ValueError("invalid packed routed_experts payload") from e
    if len(shape) != 3 or any((not isinstance(d, (int, np.integer))) or isinstance(d, bool) or d < 0 for d in shape):
        raise ValueError(f"invalid packed routed_experts shape: {shape}")
    if len(data) != math.prod(shape) * dt.itemsize:
        raise ValueError(f"packed routed_experts has {len(data)} bytes, expected {math.prod(shape) * dt.itemsize}")
    out = np.frombuffer(data, dtype=dt).reshape(shape)
    if compact_routed_expert_indices(out).dtype != dt:
        raise ValueError(f"packed routed_experts uses non-canonical dtype {dt.name}")
    return out
