"""The oracle's gain / leaf-weight restatement against the reference's own
src/core/gain.cu compiled for the host (``make -C oracle ref``): bit-exact."""
import ctypes
import os

import numpy as np
import pytest

from oracle import oracle as orc

REF = os.path.join(os.path.dirname(orc.__file__), "_ref", "libref_gain.so")
pytestmark = pytest.mark.skipif(not os.path.exists(REF), reason="oracle/_ref not built")


def _ref():
    L = ctypes.CDLL(REF)
    f, d, u64, u32, vp = ctypes.c_float, ctypes.c_double, ctypes.c_uint64, ctypes.c_uint, ctypes.c_void_p
    for name, args in (("gain_f", [f, f, u64, u64, vp]), ("gain_d", [d, d, u64, u64, vp]),
                       ("gain_f2", [f, f, f, f, u64, u64, vp]), ("gain_d2", [d, d, d, d, u64, u64, vp]),
                       ("weight_f", [f, u32, vp]), ("weight_d", [d, u32, vp]),
                       ("weight_f2", [f, f, u32, vp]), ("weight_d2", [d, d, u32, vp])):
        fn = getattr(L, "ref_" + name)
        fn.restype = f
        fn.argtypes = args
    return L


PARAMS = [dict(), dict(lambda_=1.0, hess=1.0, min_leaf_size=1),
          dict(lambda_=0.5, alpha=0.3, hess=2.0, min_leaf_size=3, gamma_absolute=0.1),
          dict(lambda_=1.0, alpha=1.0, max_leaf_weight=0.05, gamma_relative=0.01, hess=0.5)]


@pytest.mark.parametrize("kw", PARAMS)
def test_gain_and_weight_bit_exact(kw):
    R, O = _ref(), orc.lib()
    p = orc.gain_params(**kw)
    pp = ctypes.byref(p)
    rng = np.random.default_rng(7)
    for _ in range(4000):
        tc = int(rng.integers(1, 5000))
        lc = int(rng.integers(0, tc + 1))
        scale = float(10 ** rng.uniform(-3, 3))
        lx, rx = rng.normal(0, scale, 2)
        ly, ry = np.abs(rng.normal(0, scale * 0.3, 2))
        tx, ty = lx + rx, ly + ry
        for a, b in ((R.ref_gain_d2(lx, ly, tx, ty, lc, tc, pp), O.orc_gain_d2(lx, ly, tx, ty, lc, tc, pp)),
                     (R.ref_gain_f2(lx, ly, tx, ty, lc, tc, pp), O.orc_gain_f2(lx, ly, tx, ty, lc, tc, pp)),
                     (R.ref_gain_d(lx, tx, lc, tc, pp), O.orc_gain_d(lx, tx, lc, tc, pp)),
                     (R.ref_gain_f(lx, tx, lc, tc, pp), O.orc_gain_f(lx, tx, lc, tc, pp)),
                     (R.ref_weight_d2(lx, ly, lc, pp), O.orc_weight_d2(lx, ly, lc, pp)),
                     (R.ref_weight_f2(lx, ly, lc, pp), O.orc_weight_f2(lx, ly, lc, pp)),
                     (R.ref_weight_d(lx, lc, pp), O.orc_weight_d(lx, lc, pp)),
                     (R.ref_weight_f(lx, lc, pp), O.orc_weight_f(lx, lc, pp))):
            assert np.float32(a).tobytes() == np.float32(b).tobytes(), (a, b, lx, ly, tx, ty, lc, tc)
