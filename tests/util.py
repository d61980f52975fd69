"""Shared helpers of the test-suite: tolerance rule, tiny model builders, oracle/engine runners."""
from __future__ import annotations

import json
from typing import List, Sequence

import numpy as np

# Parity bar for floating point: 1e-4 relative per output.  The rounding noise of a dot product does not
# shrink when its terms cancel, so an output whose magnitude lies below the RMS magnitude of its tensor
# is measured against that RMS instead of against itself (two correct fp32 implementations that sum in
# different orders, such as the oracle and Eigen, differ by more than 1e-4 of such outputs).  The
# reference's own load-time self test uses 1e-4 absolute (import_model.hpp:2005-2009); it is exercised
# through the embedded tests of the golden fixtures.
REL_TOL = 1e-4


def assert_close(got: np.ndarray, want: np.ndarray, what: str = "", rel: float = REL_TOL) -> None:
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all() or not np.isfinite(want).all(), f"{what}: non-finite output"
    rms = float(np.sqrt(np.mean(np.square(want.astype(np.float64))))) if want.size else 0.0
    scale = np.maximum(np.abs(want), max(rms, 1e-30))
    err = np.abs(got.astype(np.float64) - want.astype(np.float64)) / scale
    worst = float(err.max()) if err.size else 0.0
    assert worst <= rel, f"{what}: max relative error {worst:.3e} > {rel:.1e} (max abs {float(np.abs(got - want).max()):.3e})"


def model_text(model_json: dict) -> str:
    return json.dumps(model_json, allow_nan=False, separators=(",", ":"))


def oracle_outputs(text: str, samples: Sequence[Sequence[np.ndarray]], threads: int = 8) -> List[List[np.ndarray]]:
    from oracle import OracleModel
    return OracleModel(json_text=text).predict_multi(samples, threads=threads)


def worst_relative(got: np.ndarray, truth: np.ndarray) -> float:
    """Largest error of `got` against `truth` under the rule of assert_close (relative, with the RMS of the tensor as floor)."""
    t = truth.astype(np.float64)
    rms = float(np.sqrt(np.mean(np.square(t)))) if t.size else 0.0
    scale = np.maximum(np.abs(t), max(rms, 1e-30))
    err = np.abs(got.astype(np.float64) - t) / scale
    return float(err.max()) if err.size else 0.0


def arbiter_outputs(text: str, samples: Sequence[Sequence[np.ndarray]], threads: int = 8) -> List[List[np.ndarray]]:
    """The same model through the double-precision build of the oracle (float64 arrays)."""
    from oracle import OracleModel
    return OracleModel(json_text=text, double=True).predict_multi(samples, threads=threads)
