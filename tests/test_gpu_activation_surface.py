"""The rest of device.Activation and the shape / fused-norm entries on the GPU, through the C ABI, against the CPU oracle:
every unary activation with a bridge op code (float32 formulas; 16-bit lookup-table semantics on every bit pattern), SeGLU and
LinGLU, row Softmax / LogSoftmax, LastToken, and the catalog's fused layernorm + add."""
import numpy as np
import pytest

import oracle as O
from gpu_util import dev, empty, host, rel_err, ulp16_diff

pytestmark = pytest.mark.gpu
ES = {O.F32: 4, O.F16: 2, O.BF16: 2}
TRANSCENDENTAL_LIBM = {"Gelu"}  # erf comes from two math libraries (glibc on the CPU, libdevice on the GPU)


@pytest.fixture(scope="module")
def d():
    import puter_b200

    O.build()
    return puter_b200.Device()


def _method(name):
    return "ReLU" if name == "Relu" else name


@pytest.mark.parametrize("name", sorted(O.UNARY_CODES))
def test_unary_f32_every_activation(d, name):
    code = O.UNARY_CODES[name]
    rng = np.random.default_rng(code)
    x = np.concatenate([(rng.standard_normal(8192) * 4).astype(np.float32),
                        np.array([0.0, -0.0, 1.0, -1.0, 3.0, -3.0, 6.0, -6.0, 20.0, 20.5, -20.5, 88.0, -88.0, 100.0, -100.0, 1e-30, -1e-30,
                                  4.92, -4.92, 5.0, 1e30, -1e30, np.inf, -np.inf], np.float32)])
    want = O.unary(code, O.F32, x)
    out = empty(x.size * 4)
    getattr(d, _method(name))(out, dev(x), x.size, O.F32)
    got = host(out, np.float32)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    if name in TRANSCENDENTAL_LIBM:
        assert np.allclose(got[ok], want[ok], rtol=1e-5, atol=1e-9)
    else:
        assert np.array_equal(got[ok].view(np.uint32), want[ok].view(np.uint32)), name


@pytest.mark.parametrize("dt", [O.BF16, O.F16])
@pytest.mark.parametrize("name", ["Silu", "Relu", "Gelu"])
def test_unary_16bit_large_input_equals_the_table_path(d, name, dt):
    """From 4 Mi elements on, the 16-bit unary activations read their table from shared memory (a different kernel): its result
    must be, element for element, what the small-input kernel returns for the same bit pattern."""
    n = (1 << 22) + 8 * 1000 + 5  # vector body, a second half-round for some threads, and a ragged tail
    rng = np.random.default_rng(len(name) + dt)
    x = rng.integers(0, 65536, n, dtype=np.uint32).astype(np.uint16)
    x[:65536] = np.arange(65536, dtype=np.uint16)
    table_out = empty(65536 * 2)
    getattr(d, _method(name))(table_out, dev(np.arange(65536, dtype=np.uint16)), 65536, dt)
    table = host(table_out, np.uint16)
    out = empty(n * 2)
    getattr(d, _method(name))(out, dev(x), n, dt)
    assert np.array_equal(host(out, np.uint16), table[x])
    assert d.take_error() == 0


@pytest.mark.parametrize("dt", [O.BF16, O.F16])
@pytest.mark.parametrize("name", sorted(O.UNARY_CODES))
def test_unary_16bit_tables_every_pattern(d, name, dt):
    code = O.UNARY_CODES[name]
    x = np.arange(65536, dtype=np.uint16)
    want = O.unary(code, dt, x)
    out = empty(65536 * 2)
    getattr(d, _method(name))(out, dev(x), 65536, dt)
    got = host(out, np.uint16)
    wn, gn = np.isnan(O.to_f32(want, dt)), np.isnan(O.to_f32(got, dt))
    assert np.array_equal(wn, gn), name
    if name in TRANSCENDENTAL_LIBM:
        assert np.allclose(O.to_f32(got[~wn], dt), O.to_f32(want[~wn], dt), rtol=1e-2, atol=1e-9)
        assert (ulp16_diff(got[~wn], want[~wn]) > 0).mean() < 1e-3
    else:
        assert np.array_equal(got[~wn], want[~wn]), (name, int((got[~wn] != want[~wn]).sum()))


@pytest.mark.parametrize("name,code", [("SeGLU", O.SEGLU), ("LinGLU", O.LINGLU)])
@pytest.mark.parametrize("dt", [O.F32, O.BF16, O.F16])
def test_seglu_linglu(d, name, code, dt):
    rng = np.random.default_rng(code)
    n, batch, half = 8192 + 3, 5, 72
    g = O.from_f32(rng.standard_normal(n).astype(np.float32) * 3, dt)
    u = O.from_f32(rng.standard_normal(n).astype(np.float32), dt)
    out = empty(n * ES[dt])
    getattr(d, name + "Tensors")(out, dev(g), dev(u), n, dt)
    want = O.gated_tensors(code, dt, g, u)
    assert np.array_equal(host(out, want.dtype).view(np.uint8), want.view(np.uint8))
    packed = O.from_f32(rng.standard_normal((batch, 2 * half)).astype(np.float32), dt)
    out = empty(batch * half * ES[dt])
    getattr(d, name)(out, dev(packed), batch, half, dt)
    want = O.gated_packed(code, dt, packed, batch, half)
    assert np.array_equal(host(out, want.dtype, want.shape).view(np.uint8), want.view(np.uint8))


@pytest.mark.parametrize("log", [False, True])
@pytest.mark.parametrize("dt", [O.F32, O.BF16, O.F16])
@pytest.mark.parametrize("rows,cols", [(1, 1), (1, 7), (3, 1000), (64, 4096), (700, 1024), (5, 32768), (2, 100003), (9, 32000)])
def test_row_softmax(d, dt, rows, cols, log):
    rng = np.random.default_rng(rows * 31 + cols)
    x = O.from_f32((rng.standard_normal((rows, cols)) * 3).astype(np.float32), dt)
    want = O.softmax_rows(dt, x, log)
    out = empty(rows * cols * ES[dt])
    d.SoftmaxRows(out, dev(x), rows, cols, dt, log=log)
    got = host(out, want.dtype, want.shape)
    assert d.take_error() == 0
    if dt == O.F32:
        # same formula, tree sum instead of the reference's sequential float32 sum, whose own rounding error grows with the
        # row length: 1e-5 relative up to 4096 columns, scaled by cols / 4096 beyond.  Log-softmax outputs are
        # differences of terms of size |x - max| and log(sum): the bound is relative to max(1, |result|).
        tol = 1e-5 * max(1.0, cols / 4096.0)
        if log:
            err = np.abs(got.astype(np.float64) - want.astype(np.float64)) / np.maximum(1.0, np.abs(want.astype(np.float64)))
            assert err.max() <= tol
        else:
            assert rel_err(got, want) <= tol
            assert np.abs(got.sum(axis=1) - 1).max() <= 1e-4
    else:
        # one unit in the last place; how many results sit close enough to a rounding boundary to flip grows with the
        # difference between the two float32 sums, hence with the row length
        assert ulp16_diff(got, want).max() <= 1 and (got != want).mean() < 0.02 * max(1.0, cols / 4096.0)


def test_softmax_one_vector_like_the_go_method(d):
    rng = np.random.default_rng(1)
    x = rng.standard_normal(5000).astype(np.float32)
    out = empty(x.size * 4)
    d.Softmax(out, dev(x), x.size, O.F32)
    assert rel_err(host(out, np.float32), O.softmax_rows(O.F32, x[None, :])[0]) <= 1e-5
    d.LogSoftmax(out, dev(x), x.size, O.F32)
    want = O.softmax_rows(O.F32, x[None, :], True)[0]
    assert (np.abs(host(out, np.float32) - want) / np.maximum(1.0, np.abs(want))).max() <= 1e-5
    d.Softmax(dev(x), dev(x), 0, O.F32)  # zero elements: a silent no-op


def test_last_token_known_answers(d):
    # execution/shape_intrinsic_test.go:53-88: [2, 3, 2] -> [[5, 6], [50, 60]]
    x = np.array([1, 2, 3, 4, 5, 6, 10, 20, 30, 40, 50, 60], np.float32)
    out = empty(16)
    d.LastToken(dev(x), out, 2, 3, 2, O.F32)
    assert host(out, np.float32).tolist() == [5, 6, 50, 60]
    # execution/bind_test.go:1201-1239: a [6, 4] allocation of which N = 3 rows are live -> the live final row
    x = np.array([1, 2, 3, 4, 9, 9, 9, 9, 5, 6, 7, 8] + [0] * 12, np.float32)
    out = empty(16)
    d.IntrinsicLastToken(dev(x), out, 3, 16, 16, O.F32)
    assert host(out, np.float32).tolist() == [5, 6, 7, 8]


@pytest.mark.parametrize("dt,batch,seq,hidden", [(O.BF16, 64, 17, 4096), (O.F32, 3, 5, 7), (O.F16, 4, 1, 33), (O.E4M3, 2, 9, 160)])
def test_last_token_random(d, dt, batch, seq, hidden):
    rng = np.random.default_rng(seq)
    es = {O.F32: 4, O.BF16: 2, O.F16: 2, O.E4M3: 1}[dt]
    raw = rng.integers(0, 256, batch * seq * hidden * es, dtype=np.uint8)
    x = raw.view({4: np.uint32, 2: np.uint16, 1: np.uint8}[es]).reshape(batch, seq, hidden)
    out = empty(batch * hidden * es)
    d.LastToken(dev(x), out, batch, seq, hidden, dt)
    assert np.array_equal(host(out, x.dtype, (batch, hidden)), O.last_token(x, batch, seq, hidden))
    assert np.array_equal(O.last_token(x, batch, seq, hidden), x[:, -1, :])


@pytest.mark.parametrize("dt", [O.F32, O.BF16, O.F16])
@pytest.mark.parametrize("rows,cols", [(3, 7), (33, 768), (64, 4096), (5, 10000)])
def test_layernorm_residual_equals_layernorm_then_add(d, dt, rows, cols):
    from test_gpu_layernorm import close

    rng = np.random.default_rng(rows * cols + 1)
    x = O.from_f32((rng.standard_normal((rows, cols)) * 2 + 0.3).astype(np.float32), dt)
    g = O.from_f32(rng.uniform(0.5, 1.5, cols).astype(np.float32), dt)
    b = O.from_f32(rng.standard_normal(cols).astype(np.float32), dt)
    r = O.from_f32(rng.standard_normal((rows, cols)).astype(np.float32), dt)
    ln = O.layernorm(dt, x, g, b)
    want = O.binary(O.ADD, dt, ln, r)
    out = empty(rows * cols * ES[dt])
    d.LayerNormResidual(dev(x), dev(g), dev(b), dev(r), out, rows, cols, dt)
    got = host(out, O.np_dtype(dt), (rows, cols))
    if dt == O.F32:
        close(dt, got, want)
    else:
        # the LayerNorm term carries the one-unit-in-the-last-place difference of its summation order; the add can cancel it
        # against the residual, so the bound is at the size of the terms, not of the sum
        gf, wf = O.to_f32(got, dt).astype(np.float64), O.to_f32(want, dt).astype(np.float64)
        size = np.maximum(1.0, np.maximum(np.abs(O.to_f32(ln, dt)), np.abs(wf)))
        assert (np.abs(gf - wf) <= 2 * (2.0 ** -7 if dt == O.BF16 else 2.0 ** -10) * size).all()
        assert (got != want).mean() < 0.03
    # the fused entry and the two separate device ops give the same bits
    ln, two = empty(rows * cols * ES[dt]), empty(rows * cols * ES[dt])
    d.LayerNorm(dev(x), dev(g), dev(b), ln, rows, cols, dt)
    d.Add(two, ln, dev(r), rows * cols, dt)
    assert np.array_equal(host(two, O.np_dtype(dt), (rows, cols)), got)
    assert d.take_error() == 0
