"""Shared helpers of the GPU parity tests: the error metric and seeded input builders."""
import os

import numpy as np


def max_rel_err(got, want):
    """max_i |got_i - want_i| / max(|want_i|, rms(want)): element-wise relative error with the
    denominator floored at the tensor's RMS, so that entries which cancel to ~0 are judged against the
    typical magnitude of the tensor instead of against themselves."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    rms = float(np.sqrt(np.mean(want * want))) if want.size else 0.0
    den = np.maximum(np.abs(want), max(rms, 1e-30))
    return float(np.max(np.abs(got - want) / den)) if want.size else 0.0


def dot_rel_err(got, want, absdot):
    """max_i |got_i - want_i| / absdot_i, where absdot_i is the same contraction evaluated on the
    absolute values of the operands (sum_j |a_ij||b_j|, plus |bias|): the relative error of a dot product
    in the sense of its forward error bound.  For a sum without cancellation it is the plain relative
    error; where terms cancel, the error is judged against the magnitude of what was summed.  This is the
    metric the 1e-4 (3xTF32) and 2e-3 (TF32) tolerances are stated on."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    den = np.maximum(np.asarray(absdot, np.float64), 1e-30)
    err = float(np.max(np.abs(got - want) / den)) if want.size else 0.0
    test = os.environ.get("PYTEST_CURRENT_TEST")
    if test and want.size:          # every contraction comparison of the suite also reports the stricter element-wise metric
        _note(test.split(" ")[0], err, survey_rel_err(got, want))
    return err


def survey_rel_err(got, want):
    """max_i |got_i - want_i| / max(|want_i|, 1e-3 * max_j |want_j|): the element-wise relative error with the
    denominator floored at a thousandth of the tensor's largest magnitude.  Far stricter than dot_rel_err where the terms of
    a contraction cancel (an output element near zero is judged against at most 1e-3 of the largest output, whatever was
    summed to get it), so it is reported next to dot_rel_err and bounded by what was measured, see PARITY_BOUNDS."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    if not want.size:
        return 0.0
    floor = 1e-3 * float(np.max(np.abs(want)))
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), max(floor, 1e-30))))


# every comparison of a contraction also lands here: name -> (dot_rel_err or None, survey_rel_err); conftest.py writes the
# collected numbers to the file named by B200CONV_PARITY_REPORT at the end of the session
PARITY_REPORT = {}


def _note(name, d, s):
    old = PARITY_REPORT.get(name)
    if old:
        d = old[0] if d is None else (d if old[0] is None else max(d, old[0]))
        s = max(s, old[1])
    PARITY_REPORT[name] = (d, s)


def record_parity(name, got, want, absdot=None):
    """Records (and returns) both error figures of one named comparison."""
    d = dot_rel_err(got, want, absdot) if absdot is not None else None
    s = survey_rel_err(got, want)
    _note(name, d, s)
    return d, s


TOL_X3 = 1e-4      # 3xTF32 against the fp32 CPU oracle
TOL_TF32 = 2e-3    # plain TF32


def conv_inputs(seed, B, C, H, W, K, k, s, p, dist="cfg"):
    """Seeded inputs in the manner of the headline configurations: image U[-1,1], He-normal weights,
    N(0,1) upstream delta, small random bias."""
    r = np.random.default_rng(seed)
    x = r.uniform(-1, 1, (B, C, H, W)).astype(np.float32)
    wt = r.normal(0, np.sqrt(2.0 / (C * k * k)), (1, 1, K, C * k * k)).astype(np.float32)
    b = r.normal(0, 0.1, (1, K, 1, 1)).astype(np.float32)
    oy, ox = (H - k + 2 * p) // s + 1, (W - k + 2 * p) // s + 1
    d = r.normal(0, 1, (B, K, oy, ox)).astype(np.float32)
    return x, wt, b, d
