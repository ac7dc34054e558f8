"""Error metrics shared by the GPU parity tests.

Every comparison checks three numbers, so that a defect confined to a few rows cannot hide behind
the norm of a large tensor: the global relative L2 error, the largest relative L2 error of any one
sequence (jagged tensors), and the largest element-wise error in units of the largest reference
element.  When ``B200_HSTU_PARITY_REPORT`` names a file, each comparison appends its measured
numbers to it as one JSON line (the test run then doubles as a measurement)."""

import json
import os

from oracle import hstu_oracle as O

# half-precision kernels against the fp32 oracle on the same (already rounded) inputs
HALF_TOL = 1e-2        # global relative L2
HALF_SEQ_TOL = 1e-2    # worst single sequence (measured: 5e-3 on a one-token sequence)
HALF_MAX_TOL = 1e-2    # max |error| / max |reference| (measured: 6e-3)
# fp32 kernels against fp32 fixtures: accumulation order only
F32_TOL = 2e-4
F32_SEQ_TOL = 5e-4
F32_MAX_TOL = 5e-4


def _note(name, rec):
    path = os.environ.get("B200_HSTU_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(dict(name=str(name), **rec)) + "\n")


def check(name, got, ref, seq_offsets=None, tol=HALF_TOL, seq_tol=HALF_SEQ_TOL, max_tol=HALF_MAX_TOL):
    """Assert that ``got`` matches ``ref`` in all three metrics; returns the global error."""
    e = O.rel_l2(got, ref)
    rec = {"rel_l2": e, "tol": tol}
    ok = e < tol
    if seq_offsets is not None:
        es = O.per_sequence_rel_l2(got, ref, seq_offsets)
        rec.update(seq_rel_l2=es, seq_tol=seq_tol)
        ok = ok and es < seq_tol
    em = O.max_abs_ratio(got, ref)
    rec.update(max_abs_ratio=em, max_tol=max_tol)
    ok = ok and em < max_tol
    _note(name, rec)
    assert ok, (name, rec)
    return e


def check_f32(name, got, ref, seq_offsets=None):
    return check(name, got, ref, seq_offsets, F32_TOL, F32_SEQ_TOL, F32_MAX_TOL)


def check_vs_bf16_reference(name, got, ref32, ref16, tol=HALF_TOL, slack=1.25):
    """For a chain of 16-bit stages: ``got`` must be within ``tol`` of the fp32 oracle, or - where
    the reference's own arithmetic in that precision (the oracle run in bf16, rounding between the
    stages where the reference rounds) is itself further away - no further than ``slack`` times
    that distance.  Both distances are recorded."""
    e = O.rel_l2(got, ref32)
    e_ref = O.rel_l2(ref16, ref32)
    bound = max(tol, slack * e_ref)
    _note(name, {"rel_l2": e, "tol": tol, "bf16_reference_rel_l2": e_ref, "bound": bound})
    assert e < bound, (name, e, e_ref)
    return e, e_ref
