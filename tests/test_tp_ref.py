"""Cross-check of the slice planner (library and oracle) against the reference's own header,
compiled into oracle/_ref/tp_plan_ref by oracle/Makefile.  Skipped where that binary is absent."""

import os
import subprocess

import numpy as np
import pytest

import tyloquant_b200 as T
from conftest import ROOT
from oracle import mfq_oracle as O

BIN = os.path.join(ROOT, "oracle", "_ref", "tp_plan_ref")


@pytest.mark.skipif(not os.path.exists(BIN), reason="reference planner checker not built")
def test_planner_agrees_with_reference_header():
    rng = np.random.default_rng(5)
    for _ in range(150):
        n = int(rng.integers(1, 9))
        gran = int(rng.choice([1, 8, 24, 128, 384]))
        extent = int(rng.integers(max(1, n * gran - 2 * gran), n * gran * 30 + 1))
        weights = [] if rng.random() < 0.5 else [round(float(x), 3) for x in rng.uniform(0.1, 4.0, n)]
        out = subprocess.run([BIN, str(extent), str(gran), str(n)] + [repr(w) for w in weights], capture_output=True,
                             text=True, check=True).stdout.strip().split("\n")
        devs = list(range(n))
        if out[0].startswith("throw"):
            with pytest.raises(ValueError):
                O.tp_plan(extent, gran, devs, weights)
            with pytest.raises(T.MfqbError):
                T.plan_tensor_parallel_slices(extent, gran, devs, weights)
            continue
        ref = [tuple(int(v) for v in line.split()) for line in out[:n]]
        mine = T.plan_tensor_parallel_slices(extent, gran, devs, weights)
        assert [(b, e) for _, b, e in mine] == ref
        assert [(b, e) for _, b, e in O.tp_plan(extent, gran, devs, weights)] == ref
        if out[n] == "valid":
            T.validate_tensor_parallel_slices(mine, extent, gran)
        else:
            with pytest.raises(T.MfqbError):
                T.validate_tensor_parallel_slices(mine, extent, gran)
