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


GLUE_GOLDEN = "glue_refs"  # norms and token shift (tests/golden/make_golden_glue.py)
INDEX_GOLDEN = "index_scans"  # pruning index arrays of upstream's scan kernels (tests/golden/make_golden_index.py)
CE_GOLDEN = "cross_entropy"  # upstream's fused cross-entropy kernels (tests/golden/make_golden_ce.py)
# every other .npz is an attention case


def golden_names():
    names = sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))
    return [n for n in names if n not in (GLUE_GOLDEN, INDEX_GOLDEN, CE_GOLDEN)]


def load_ce_golden():
    """Fixture produced by tests/golden/make_golden_ce.py: upstream's cross_entropy_loss (its Triton kernels in
    the CPU interpreter).  Returns {case: dict(logits, labels, dloss, losses, z_losses, dlogits, args)}."""
    z = np.load(os.path.join(GOLDEN_DIR, CE_GOLDEN + ".npz"))
    cases = {}
    for key in z.files:
        case, field = key.split("/")
        cases.setdefault(case, {})[field] = torch.from_numpy(np.ascontiguousarray(z[key]))
    return cases


def load_index_golden():
    """Fixture produced by tests/golden/make_golden_index.py: upstream's _find_start_index_kernel and
    _find_end_index_kernel launched directly (Triton's CPU interpreter) on torch.cumsum prefix sums.
    Returns {case: dict(shape=(B,H,M,N,BM,BN), log_fgate, threshold, start_index, end_index)}."""
    z = np.load(os.path.join(GOLDEN_DIR, INDEX_GOLDEN + ".npz"))
    cases = {}
    for key in z.files:
        case, field = key.split("/")
        cases.setdefault(case, {})[field] = z[key]
    for rec in cases.values():
        rec["shape"] = tuple(int(x) for x in rec["shape"])
    return cases


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


def upstream_ops():
    """The upstream project's own operator module (forgetting_transformer.ops.forgetting_attention) for
    head-to-head GPU tests, or None when no copy is installed.  Looked for in $FOX_REFERENCE_SRC (the directory
    holding the ``forgetting_transformer`` package), then in ``baseline/_ref`` of this checkout (where
    ``pip install --target baseline/_ref <upstream>`` puts it; git-ignored).  Its three block-size hooks, which
    upstream documents as overridable and which raise on sm_100, are pinned to 128 x 128 tiles so that the
    pruning index arrays of both sides live on the same grid."""
    import importlib
    for cand in (os.environ.get("FOX_REFERENCE_SRC"), os.path.join(ROOT, "baseline", "_ref")):
        if cand and os.path.isdir(os.path.join(cand, "forgetting_transformer")):
            if cand not in sys.path:
                sys.path.insert(0, cand)
            sys.dont_write_bytecode = True
            mod = importlib.import_module("forgetting_transformer.ops.forgetting_attention")
            # The forward grid defines start_index and stays 128 x 128.  At head dim 128 Triton's sm_100 lowering
            # of the backward kernels with 128 x 128 tiles needs more shared memory (two stages) and more tensor
            # memory (576 of 512 columns) than the SM has, so they run on upstream's own H100 tile for the key side
            # and a 128 x 64 tile for the query side; backward tiles only decide which nearly-empty tiles are
            # skipped (each carries less than e^threshold of a row's mass).
            mod.get_fwd_config = lambda B, H, M, N, D, causal: (128, 128, 2 if D <= 64 else 1, 8)
            mod.get_bwd_kv_config = lambda B, H, M, N, D, causal: (128, 128, 2, 8) if D <= 64 else (64, 64, 2, 4)
            mod.get_bwd_q_config = lambda B, H, M, N, D, causal: (128, 128, 2, 8) if D <= 64 else (128, 64, 2, 8)
            return mod
    return None
