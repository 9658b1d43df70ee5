import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with `-m gpu`")


def pytest_collection_modifyitems(config, items):
    # GPU tests are skipped (not failed) where no GPU is visible and the run did not ask for them
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# ---- tolerance of the floating-point parity tests -------------------------------------------------
# 16-bit kernels against the fp32 oracle on identical inputs: max abs error <= 2e-2 and max relative
# error <= 1e-2, the relative error taken over elements with |ref| > REL_FLOOR * max|ref| (below that
# floor an element is rounding noise of the sums that produced it).
ABS_TOL = 2e-2
REL_TOL = 1e-2
REL_FLOOR = 1e-3


# fp16 outputs below 2^-14 are subnormal with an absolute spacing of 2^-24: under this magnitude even
# exact rounding misses REL_TOL, so such elements are judged by the absolute tolerance only
FP16_REL_MIN = 2.0 ** -24 / REL_TOL * 2


def parity_errors(got, ref, rel_floor=REL_FLOOR):
    fp16_out = got.dtype == torch.float16
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    d = (got - ref).abs()
    floor = rel_floor * ref.abs().max().item()
    if fp16_out:
        floor = max(floor, FP16_REL_MIN)
    m = ref.abs() > floor
    rel = (d[m] / ref.abs()[m]).max().item() if m.any() else 0.0
    return d.max().item(), rel


# Every comparison is also recorded (max abs error, max relative error at the 1e-3 and at the 0.1 floor) and, when
# GPU tests ran, written as JSON lines to PARITY_LOG at the end of the session: the measured errors behind the
# pass / fail verdicts.  `config` groups records of one benchmark configuration.
PARITY_RECORDS = []
PARITY_LOG = os.environ.get("TRINITY_PARITY_LOG", os.path.join(ROOT, "test_out", "parity_errors.jsonl"))


def record(kind, what, config=None, **fields):
    PARITY_RECORDS.append(dict(kind=kind, what=what, config=config, **fields))


def assert_parity(got, ref, what="", abs_tol=ABS_TOL, rel_tol=REL_TOL, rel_floor=REL_FLOOR, config=None):
    a, r = parity_errors(got, ref, rel_floor)
    if got.is_cuda:
        _, r3 = parity_errors(got, ref, 1e-3)
        _, r1 = parity_errors(got, ref, 1e-1)
        record("parity", what, config, max_abs=a, max_rel_floor_1em3=r3, max_rel_floor_1em1=r1, abs_tol=abs_tol,
               rel_tol=rel_tol, rel_floor=rel_floor, max_ref=float(ref.detach().abs().max()), n=int(ref.numel()))
        print(f"[parity] {what}: max abs {a:.3e}, max rel {r3:.3e} above 1e-3*max, {r1:.3e} above 0.1*max")
    assert a <= abs_tol and r <= rel_tol, f"{what}: max abs {a:.3e} (tol {abs_tol}), max rel {r:.3e} (tol {rel_tol})"
    return a, r


def pytest_sessionfinish(session, exitstatus):
    if not PARITY_RECORDS:
        return
    import json
    try:
        os.makedirs(os.path.dirname(PARITY_LOG), exist_ok=True)
        with open(PARITY_LOG, "w") as f:
            for rec in PARITY_RECORDS:
                f.write(json.dumps(rec) + "\n")
    except OSError:
        pass
