"""The scratch pools filled with NaN bytes before every evaluation (the reference's PET_WS_POISON, include/pet/kokkos.hpp):
nothing may change. An evaluation that read a value nobody wrote would pass or fail by what the memory last held."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
WORKER = Path(__file__).with_name("poison_worker.py")


def run_worker(tmp_path, name, env_over):
    env = dict(os.environ, PET_GRAPHS="0", **env_over)
    for k in ("PET_WS_POISON", "PET_B200_WS_POISON"):
        if k not in env_over:
            env.pop(k, None)
    out = tmp_path / f"{name}.npz"
    r = subprocess.run([sys.executable, str(WORKER), str(tmp_path / name), str(out)], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "POISON_WORKER_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])
    return np.load(out)


def test_poisoned_pools_change_no_bit(lib_path, tmp_path):
    plain = run_worker(tmp_path, "plain", {})
    poisoned = run_worker(tmp_path, "poisoned", {"PET_B200_WS_POISON": "1"})
    assert sorted(plain.files) == sorted(poisoned.files) and len(plain.files) > 60
    for k in plain.files:
        assert np.isfinite(poisoned[k]).all(), k
        assert np.array_equal(plain[k], poisoned[k]), (k, np.abs(plain[k] - poisoned[k]).max())
