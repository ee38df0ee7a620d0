"""Generates the committed golden fixtures of the convolution hot path.

  reference_kat.npz   inputs and expected outputs of the reference's own known-answer tests
                      (cuda/ctensortest.cu.h; line ranges cited per case below).  The expected
                      values are transcribed from that file as data and are ALSO recomputed here by
                      the compiled reference CPU backend; generation fails if the two disagree.
  seeded_cases.npz    seeded random cases (stride, padding, W-broadcast, pooling ties ...) whose
                      outputs come from the compiled reference CPU backend (oracle/_ref/libref.so).

Run in a container that has the reference tree:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import Oracle  # noqa: E402


def kat_cases(ref):
    out = {}
    B = 10
    # --- ctensortest.cu.h:77-166  ForwardConvolution, 3x3x3 image, two 2x2x3 kernels, s1 p0
    img = np.arange(1, 28, dtype=np.float32).reshape(1, 3, 3, 3).repeat(B, 0)
    ker = np.stack([np.arange(1, 13), np.arange(12, 0, -1)]).astype(np.float32).reshape(1, 2, 12)
    exp = np.array([1245, 1323, 1479, 1557, 627, 705, 861, 939], np.float32).reshape(1, 2, 2, 2).repeat(B, 0)
    got = ref.conv_forward(img, ker, np.zeros((1, 2), np.float32), 2, 2, 1, 1, 0, 0)
    assert np.array_equal(got, exp)
    out.update(fwd_image=img, fwd_kernel=ker, fwd_expected=exp)
    # --- ctensortest.cu.h:310-410  CreateDeltaWeightAndBias, 7x7 image, 4x4 delta, 5x5 kernel, s2 p2
    img = np.arange(1, 50, dtype=np.float32).reshape(1, 1, 7, 7).repeat(B, 0)
    dl = np.arange(1, 17, dtype=np.float32).reshape(1, 1, 4, 4).repeat(B, 0)
    exp = np.array([2031, 2130, 2746, 1968, 2058, 2724, 2823, 3628, 2598, 2688, 3448, 3556, 4560, 3256, 3352,
                    1860, 1923, 2428, 1698, 1752, 2301, 2364, 2974, 2076, 2130], np.float32).reshape(1, 1, 25).repeat(B, 0)
    dk, db = ref.conv_wgrad(np.zeros((B, 1, 25), np.float32), np.zeros((B, 1), np.float32), img, dl, 5, 5, 2, 2, 2, 2)
    assert np.array_equal(dk, exp)
    out.update(wgrad_s2_image=img, wgrad_s2_delta=dl, wgrad_s2_expected=exp, wgrad_s2_dbias=db)
    # --- ctensortest.cu.h:415-535  CreateDeltaWeightAndBias, 4x4 image, 2x2 delta, 3x3 per-sample kernels, s1 p0
    img = np.array([4, 5, 8, 7, 1, 8, 8, 8, 3, 6, 6, 4, 6, 5, 7, 8], np.float32).reshape(1, 1, 4, 4).repeat(B, 0)
    dl = np.array([2, 1, 4, 4], np.float32).reshape(1, 1, 2, 2).repeat(B, 0)
    exp = np.array([49, 82, 87, 46, 72, 64, 56, 66, 76], np.float32).reshape(1, 1, 9).repeat(B, 0)
    dk, db = ref.conv_wgrad(np.zeros((B, 1, 9), np.float32), np.zeros((B, 1), np.float32), img, dl, 3, 3, 1, 1, 0, 0)
    assert np.array_equal(dk, exp)
    out.update(wgrad_s1_image=img, wgrad_s1_delta=dl, wgrad_s1_expected=exp, wgrad_s1_dbias=db)
    # --- ctensortest.cu.h:541-652  BackwardConvolution, 4x4 delta -> 7x7, 5x5 kernel, s2 p2
    ker = np.arange(1, 26, dtype=np.float32).reshape(1, 1, 25)
    dl = np.arange(1, 17, dtype=np.float32).reshape(1, 1, 4, 4).repeat(B, 0)
    exp = np.array([56, 70, 124, 102, 172, 134, 156, 126, 140, 244, 192, 322, 244, 266, 233, 266, 450, 344, 567, 422, 467,
                    318, 348, 556, 400, 634, 452, 490, 521, 578, 918, 656, 1035, 734, 803, 510, 556, 868, 608, 946, 660, 714,
                    740, 786, 1228, 858, 1336, 930, 984], np.float32).reshape(1, 1, 7, 7).repeat(B, 0)
    got = ref.conv_backward(dl, ker, np.zeros((1, 1), np.float32), (1, 7, 7), 5, 5, 2, 2, 2, 2)
    assert np.array_equal(got, exp)
    out.update(bwd_kernel=ker, bwd_delta=dl, bwd_expected=exp)
    # --- ctensortest.cu.h:803-841  batched 2x2 Mul incl. W-broadcast on either side
    a = np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 2, 2).repeat(B, 0)
    exp = np.array([7, 10, 15, 22], np.float32).reshape(1, 1, 2, 2).repeat(B, 0)
    for l, r in ((a, a), (a[:1], a), (a, a[:1])):
        assert np.array_equal(ref.mul(l, r), exp)
    out.update(mul_a=a, mul_expected=exp)
    # --- ctensortest.cu.h:172-305  ForwardConvolution with stride and padding: the reference test
    # builds inputs but checks nothing; the expected tensor here is the reference CPU output.
    img = np.arange(1, 76, dtype=np.float32).reshape(1, 3, 5, 5).repeat(B, 0)
    ker = np.stack([np.arange(1, 28), np.arange(27, 0, -1)]).astype(np.float32).reshape(1, 2, 27)
    out.update(fwd_s2_image=img, fwd_s2_kernel=ker,
               fwd_s2_expected=ref.conv_forward(img, ker, np.zeros((1, 2), np.float32), 3, 3, 2, 2, 1, 1))
    return out


SEEDED = [
    # name, B, C, H, W, K, k, s, p
    ("c3x3", 4, 8, 12, 12, 16, 3, 1, 1),
    ("c4x4s2", 3, 6, 16, 16, 8, 4, 2, 1),
    ("c5x5s2", 2, 3, 11, 9, 5, 5, 2, 2),
    ("c1x1", 2, 7, 5, 6, 3, 1, 1, 0),
]


def seeded_cases(ref):
    out = {}
    for name, B, Cc, H, W, K, k, s, p in SEEDED:
        r = np.random.default_rng(sum(map(ord, name)))
        x = r.uniform(-1, 1, (B, Cc, H, W)).astype(np.float32)
        wt = r.normal(0, np.sqrt(2.0 / (Cc * k * k)), (1, K, Cc * k * k)).astype(np.float32)
        b = r.normal(0, 0.5, (1, K)).astype(np.float32)
        y = ref.conv_forward(x, wt, b, k, k, s, s, p, p)
        d = r.normal(0, 1, y.shape).astype(np.float32)
        dx = ref.conv_backward(d, wt, np.zeros((1, K), np.float32), (Cc, H, W), k, k, s, s, p, p)
        dk, db = ref.conv_wgrad(np.zeros((B, K, Cc * k * k), np.float32), np.zeros((B, K), np.float32), x, d, k, k, s, s, p, p)
        out.update({f"{name}_cfg": np.array([B, Cc, H, W, K, k, s, p]), f"{name}_x": x, f"{name}_w": wt, f"{name}_b": b,
                    f"{name}_y": y, f"{name}_d": d, f"{name}_dx": dx, f"{name}_dk": dk, f"{name}_db": db})
    r = np.random.default_rng(99)
    px = r.integers(-3, 4, (2, 3, 8, 8)).astype(np.float32)
    mo, mp = ref.maxpool(px, 2, 2)
    md = r.normal(0, 1, mo.shape).astype(np.float32)
    out.update(pool_x=px, pool_out=mo, pool_pos=mp, pool_delta=md, pool_back=ref.maxpool_backward(md, mp, 2, 2))
    u = r.normal(0, 1, (2, 3, 4, 5)).astype(np.float32)
    out.update(up_x=u, up_out=ref.upsample(u, 2, 2), down_out=ref.downsample(ref.upsample(u, 2, 2), 2, 2))
    a = r.normal(0, 1, (6, 1, 40, 33)).astype(np.float32)
    bb = r.normal(0, 1, (1, 1, 33, 17)).astype(np.float32)
    c = r.normal(0, 1, (6, 1, 40, 9)).astype(np.float32)
    out.update(gemm_a=a, gemm_b=bb, gemm_c=c, gemm_mul=ref.mul(a, bb), gemm_tmul=ref.tmul(a, c))
    # batch normalisation (the reference's tensor routines in the layer's order) and the reference's VAE output layer object
    bx = r.normal(1.5, 2.0, (16, 3, 4, 5)).astype(np.float32)
    bg, bb_ = r.normal(1, 0.2, (3, 4, 5)).astype(np.float32), r.normal(0, 0.3, (3, 4, 5)).astype(np.float32)
    f = ref.bn_forward(bx, bg, bb_, 0.9, 1e-6, np.zeros((3, 4, 5), np.float32), np.ones((3, 4, 5), np.float32))
    bdy = r.normal(0, 1, bx.shape).astype(np.float32)
    bdx, bdg, bdb = ref.bn_backward(bdy, f["xhat"], f["ivar"], bg)
    out.update(bn_x=bx, bn_gamma=bg, bn_beta=bb_, bn_dy=bdy, bn_dx=bdx, bn_dgamma=bdg, bn_dbeta=bdb,
               **{"bn_" + k: v for k, v in f.items()})
    vmu = r.normal(0, 1, (6, 1, 40, 1)).astype(np.float32)
    vlv = r.normal(0, 4, (6, 1, 40, 1)).astype(np.float32)
    vlv[0, 0, :4, 0] = [11, -11, 10, -10]
    vd = r.normal(0, 1, vmu.shape).astype(np.float32)
    vz, veps, vdmu, vdlv = ref.vae_layer(vmu, vlv, vd, 0.25)
    out.update(vae_mu=vmu, vae_logvar=vlv, vae_delta=vd, vae_eps=veps, vae_z=vz, vae_dmu=vdmu, vae_dlogvar=vdlv, vae_kl_speed=np.float32(0.25))
    xs = np.linspace(-35, 35, 141).astype(np.float32).reshape(1, 1, 1, -1)
    out["act_x"] = xs
    for f in Oracle.FUNCS:
        out[f"act_{f}"] = ref.activation(xs, f)
        out[f"dact_{f}"] = ref.activation(xs, f, True)
    return out


if __name__ == "__main__":
    ref = Oracle("reference")
    np.savez_compressed(os.path.join(HERE, "reference_kat.npz"), **kat_cases(ref))
    np.savez_compressed(os.path.join(HERE, "seeded_cases.npz"), **seeded_cases(ref))
    for f in ("reference_kat.npz", "seeded_cases.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
