"""Error bookkeeping shared by the GPU parity tests.

Bounds (max-abs against the f32 oracle):

* f32 inputs: 1e-4 for outputs and every gradient.
* 16-bit inputs, outputs and dq/dk/dv of the benchmark configurations: 2e-2 absolute.
* 16-bit shared-bias gradient: 2e-2 * max(1, max|reference|).  The gradient is a sum over all pair rows and is
  returned in the 16-bit bias type, so its own rounding is 2^-9 relative to each value; with hundreds of rows the
  values exceed 1 and an absolute 2e-2 would sit below one unit in the last place of the result.  Absolute and
  relative-to-maximum errors are both recorded.

When the environment variable OOPS_PARITY_REPORT names a file, every recorded comparison is written there as JSON
at the end of the session.
"""

from __future__ import annotations

import json
import os
from typing import Dict

import torch

REPORT: Dict[str, dict] = {}


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double().cpu() - b.double().cpu()).abs().max())


def check(label: str, got: torch.Tensor, want: torch.Tensor, atol: float, *, relative_to_max: bool = False) -> float:
    """Assert ``max|got - want| <= atol`` (times ``max(1, max|want|)`` when ``relative_to_max``) and record it."""
    assert got.shape == want.shape, (label, got.shape, want.shape)
    error = max_abs(got, want)
    peak = float(want.double().abs().max())
    bound = atol * max(1.0, peak) if relative_to_max else atol
    REPORT[label] = dict(max_abs=error, reference_max=peak, relative_to_max=error / peak if peak > 0 else 0.0, bound=bound)
    assert torch.isfinite(got.float()).all(), f"{label}: non-finite values"
    assert error <= bound, f"{label}: max-abs error {error:.3e} > {bound:.3e} (reference max {peak:.3e})"
    return error


def write_report() -> None:
    path = os.environ.get("OOPS_PARITY_REPORT")
    if path and REPORT:
        with open(path, "w") as handle:
            json.dump(REPORT, handle, indent=1, sort_keys=True)
