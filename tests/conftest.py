import glob
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on a B200")


GLUE_GOLDEN = "glue_refs"  # norms and token shift (tests/golden/make_golden_glue.py); the rest are attention cases


def golden_names():
    names = sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))
    return [n for n in names if n != GLUE_GOLDEN]


def load_glue_golden():
    """Fixture produced by tests/golden/make_golden_glue.py: upstream's reference norm functions on CPU and
    its token-shift Triton kernels in Triton's CPU interpreter (fp16)."""
    z = np.load(os.path.join(GOLDEN_DIR, GLUE_GOLDEN + ".npz"))
    return {k: (torch.from_numpy(np.ascontiguousarray(z[k])) if z[k].ndim else z[k].item()) for k in z.files}


def load_golden(name):
    """Fixture produced by tests/golden/make_golden.py: upstream's Triton kernels run in
    Triton's CPU interpreter (fp16, 128x128 blocks)."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    rec = {k: z[k] for k in z.files}
    out = {}
    for k, v in rec.items():
        if k == "sm_scale":
            out[k] = float(v)
        else:
            out[k] = torch.from_numpy(np.ascontiguousarray(v))
    out.setdefault("seq_start", None)
    out.setdefault("threshold", None)
    out.setdefault("start_index", None)
    return out


@pytest.fixture(params=golden_names())
def golden(request):
    rec = load_golden(request.param)
    rec["name"] = request.param
    return rec
