"""LayerNorm, AdaptiveRMSNorm and ModulatedLayerNorm kernels against the CPU restatement (device/cpu/layernorm/compute.go)."""
import numpy as np
import pytest

import oracle as O
from gpu_util import dev, empty, host

pytestmark = pytest.mark.gpu
ES = {O.F32: 4, O.F16: 2, O.BF16: 2}


def close(dt, got, want):
    if dt == O.F32:
        # the shift / bias is added last, so outputs near zero come from cancellation: the error is bounded relative to the
        # size of the terms, max(1, |want|), not to the result itself
        err = np.abs(got.astype(np.float64) - want.astype(np.float64)) / np.maximum(1.0, np.abs(want.astype(np.float64)))
        assert err.max() <= 1e-5
    else:
        # same arithmetic, different summation order: one unit in the last place of the storage type at the size of the
        # terms (outputs near zero come from cancellation against the shift / bias), and nearly all outputs bit-equal
        g, w = O.to_f32(got, dt).astype(np.float64), O.to_f32(want, dt).astype(np.float64)
        ulp = 2.0 ** -7 if dt == O.BF16 else 2.0 ** -10
        assert (np.abs(g - w) <= ulp * np.maximum(1.0, np.abs(w))).all()
        assert (got != want).mean() < 0.02


@pytest.mark.parametrize("dt", [O.F32, O.BF16, O.F16])
@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 7), (33, 768), (16, 4096), (5, 10000)])
def test_layernorm(dt, rows, cols):
    import puter_b200

    d = puter_b200.Device()
    rng = np.random.default_rng(rows * cols)
    x = O.from_f32((rng.standard_normal((rows, cols)) * 2 + 0.3).astype(np.float32), dt)
    g = O.from_f32(rng.uniform(0.5, 1.5, cols).astype(np.float32), dt)
    b = O.from_f32(rng.standard_normal(cols).astype(np.float32), dt)
    want = O.layernorm(dt, x, g, b)
    out = empty(rows * cols * ES[dt])
    d.LayerNorm(dev(x), dev(g), dev(b), out, rows, cols, dt)
    close(dt, host(out, O.np_dtype(dt), (rows, cols)), want)


@pytest.mark.parametrize("dt", [O.F32, O.BF16, O.F16])
@pytest.mark.parametrize("pad", [0, 5])  # 0: 16-byte vector path, 5: modulation rows unaligned -> scalar path
@pytest.mark.parametrize("rows,cols,rpb", [(4, 64, 2), (12, 1536, 4), (6, 4096, 6)])
def test_adaptive_rmsnorm(dt, rows, cols, rpb, pad):
    import puter_b200

    d = puter_b200.Device()
    rng = np.random.default_rng(rows + cols)
    mod_cols = 2 * cols + pad
    x = O.from_f32(rng.standard_normal((rows, cols)).astype(np.float32), dt)
    mod = O.from_f32((rng.standard_normal((rows // rpb, mod_cols)) * 0.2).astype(np.float32), dt)
    want = O.adaptive_rmsnorm(dt, x, mod, rpb, mod_cols, 1e-6)
    out = empty(rows * cols * ES[dt])
    d.AdaptiveRMSNorm(puter_b200.RMSNormConfig(1e-6), dev(x), dev(mod), out, rows, cols, rpb, mod_cols, dt)
    close(dt, host(out, O.np_dtype(dt), (rows, cols)), want)


@pytest.mark.parametrize("dt", [O.F32, O.BF16, O.F16])
@pytest.mark.parametrize("pad", [0, 3])
@pytest.mark.parametrize("rows,cols,rpb,set_index", [(4, 64, 2, 0), (12, 1536, 4, 1), (6, 4096, 3, 2)])
def test_modulated_layernorm(dt, rows, cols, rpb, set_index, pad):
    import puter_b200

    d = puter_b200.Device()
    rng = np.random.default_rng(rows + cols + set_index)
    mod_cols = (set_index * 3 + 2) * cols + pad
    x = O.from_f32((rng.standard_normal((rows, cols)) + 0.5).astype(np.float32), dt)
    mod = O.from_f32((rng.standard_normal((rows // rpb, mod_cols)) * 0.2).astype(np.float32), dt)
    want = O.modulated_layernorm(dt, x, mod, rpb, mod_cols, 1e-6, set_index)
    out = empty(rows * cols * ES[dt])
    d.ModulatedLayerNorm(puter_b200.ModulatedLayerNormConfig(1e-6, set_index), dev(x), dev(mod), out, rows, cols, rpb, mod_cols, dt)
    close(dt, host(out, O.np_dtype(dt), (rows, cols)), want)


def test_validation_errors_match_the_cpu_panics():
    import puter_b200

    d = puter_b200.Device()
    x = dev(np.zeros((4, 8), np.float32))
    mod = dev(np.zeros((2, 16), np.float32))
    out = empty(4 * 8 * 4)
    with pytest.raises(puter_b200.DeviceError):  # rows not divisible by rowsPerBatch
        d.AdaptiveRMSNorm(puter_b200.RMSNormConfig(1e-6), x, mod, out, 4, 8, 3, 16, O.F32)
    with pytest.raises(puter_b200.DeviceError):  # modulation width too small for set 1
        d.ModulatedLayerNorm(puter_b200.ModulatedLayerNormConfig(1e-6, 1), x, mod, out, 4, 8, 2, 16, O.F32)
    with pytest.raises(puter_b200.DeviceError):  # epsilon must be positive
        d.AdaptiveRMSNorm(puter_b200.RMSNormConfig(0.0), x, mod, out, 4, 8, 2, 16, O.F32)
