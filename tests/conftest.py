import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def lib_path():
    """The in-tree CUDA library; built here if absent (nvcc cross-compiles without a GPU)."""
    from pet_kokkos_b200 import build
    p = build.OUT
    if not p.exists():
        build.build()
    return p


@pytest.fixture(scope="session")
def models(tmp_path_factory):
    """Seeded random-init checkpoints, written once per session: name -> (json, safetensors)."""
    from pet_kokkos_b200 import checkpoint as ck
    d = tmp_path_factory.mktemp("models")
    made = {}

    def get(shape, featurizer="feedforward", init="n002", seed=0):
        key = (shape, featurizer, init, seed)
        if key not in made:
            made[key] = ck.write_random_checkpoint(d / f"{shape}_{featurizer}_{init}_{seed}", shape, featurizer,
                                                   seed=seed, init=init)
        return made[key]
    return get


@pytest.fixture(scope="session")
def reference():
    """The reference's own evaluator compiled for the host (oracle/reference_lib.py): built here when a checkout
    of the reference is at hand, used prebuilt otherwise, and the test skipped where there is neither."""
    from oracle import reference_lib
    if not reference_lib.build():
        pytest.skip("the reference library is not built and no reference checkout is present")
    return reference_lib


@pytest.fixture(scope="session")
def has_gpu():
    import torch
    return torch.cuda.is_available()
