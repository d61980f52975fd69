"""Shared helpers of the test-suite: tolerance rule, tiny model builders, oracle/engine runners."""
from __future__ import annotations

import json
from typing import List, Sequence

import numpy as np

# Parity bar for floating point (stated by the build's north star): 1e-4 relative per output.  Outputs
# near zero (softmax tails) get a floor of 1e-3 of the largest reference magnitude; the reference's own
# load-time self test uses 1e-4 absolute (import_model.hpp:2005-2009).
REL_TOL = 1e-4
FLOOR = 1e-3


def assert_close(got: np.ndarray, want: np.ndarray, what: str = "", rel: float = REL_TOL) -> None:
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all() or not np.isfinite(want).all(), f"{what}: non-finite output"
    scale = np.maximum(np.abs(want), FLOOR * max(float(np.abs(want).max()), 1e-30))
    err = np.abs(got.astype(np.float64) - want.astype(np.float64)) / scale
    worst = float(err.max()) if err.size else 0.0
    assert worst <= rel, f"{what}: max relative error {worst:.3e} > {rel:.1e} (max abs {float(np.abs(got - want).max()):.3e})"


def model_text(model_json: dict) -> str:
    return json.dumps(model_json, allow_nan=False, separators=(",", ":"))


def oracle_outputs(text: str, samples: Sequence[Sequence[np.ndarray]], threads: int = 8) -> List[List[np.ndarray]]:
    from oracle import OracleModel
    return OracleModel(json_text=text).predict_multi(samples, threads=threads)
