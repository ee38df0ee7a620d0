"""Shared helpers of the GPU parity tests: the error metric and seeded input builders."""
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
    return float(np.max(np.abs(got - want) / den)) if want.size else 0.0


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
