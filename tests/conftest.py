import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on the GPU box")


@pytest.fixture(autouse=True)
def fresh_slab_mode_history():
    """Every test starts with the default slab mode: what earlier tests' passes recomputed must not pick the mode of
    this one (the policy remembers shapes for the life of the process)."""
    from linear_cross_entropy_loss_b200 import ops

    ops.slab_mode_policy.history.clear()
    yield


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(ROOT / "tests" / "golden" / "lce_golden.npz")


def golden_case(golden, name):
    """Inputs (float64 numpy), options and expected outputs of one golden case."""
    import numpy as np

    N, H, V, ign = (int(v) for v in golden[f"{name}/meta"])
    zreg, scale = (float(v) for v in golden[f"{name}/opts"])
    seed = int(golden[f"{name}/inputs"][0])
    x = golden[f"inputs{seed}/xq"].astype(np.float64)[:N] / 64.0
    W = golden[f"inputs{seed}/wq"].astype(np.float64) / 512.0
    return dict(
        N=N, H=H, V=V, ignore_index=ign, z_regularization=zreg, logit_scale=scale, x=x, W=W,
        y=golden[f"{name}/y"], scalars=golden[f"{name}/scalars"], dx=golden[f"{name}/dx"],
        dW_rows=golden[f"{name}/dW_rows"], dW_rowsum=golden[f"{name}/dW_rowsum"],
        dW_colsum=golden[f"{name}/dW_colsum"],
    )


GOLDEN_CASES = ["plain", "ignore", "all_options", "big_scale"]
