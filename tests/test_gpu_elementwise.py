"""GPU parity: converters, activations, elementwise, norms, RoPE, paged KV — through the C ABI vs the CPU oracle."""
import numpy as np
import pytest

import oracle as O
from gpu_util import dev, empty, host, rel_err, ulp16_diff

pytestmark = pytest.mark.gpu

LENGTHS = [1, 7, 64, 1024, 8192]  # device/cpu/parity/parity.go:10
ES = {O.F32: 4, O.F16: 2, O.BF16: 2, O.E4M3: 1, O.E5M2: 1}


@pytest.fixture(scope="module")
def d():
    import puter_b200

    O.build()
    return puter_b200.Device()


def specials_f32():
    bits = [0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00000, 0x7F800001, 0xFFBFFFFF, 0x00000001,
            0x807FFFFF, 0x00800000, 0x7F7FFFFF, 0xFF7FFFFF, 0x477FE000, 0x477FF000, 0x47800000, 0x33000000, 0x33000001,
            0x32FFFFFF, 0x43E00000, 0x43E80000, 0x43E80001, 0x3F808000, 0x3F818000, 0x3F800001, 0x38800000, 0x387FC000]
    ties = [(e << 23) | (m << 16) | 0x8000 for e in range(1, 255, 7) for m in range(0, 128, 5)]
    return np.array(bits + ties, dtype=np.uint32).view(np.float32)


@pytest.mark.parametrize("src_dt,dst_dt", [(O.BF16, O.F32), (O.F16, O.F32), (O.E4M3, O.F32), (O.E5M2, O.F32), (O.F32, O.BF16),
                                           (O.F32, O.F16), (O.F32, O.E4M3), (O.F32, O.E5M2)])
def test_convert_bit_exact(d, src_dt, dst_dt):
    rng = np.random.default_rng(20 + src_dt * 7 + dst_dt)
    if src_dt == O.F32:
        src = rng.integers(0, 2**32, (1 << 22) + 5, dtype=np.uint64).astype(np.uint32).view(np.float32)
        sp = specials_f32()
        src[: sp.size] = sp
    elif ES[src_dt] == 2:
        src = np.tile(np.arange(65536, dtype=np.uint16), 17)[: 65536 * 16 + 3]  # every pattern, ragged tail
    else:
        src = np.tile(np.arange(256, dtype=np.uint8), 4099)[: 256 * 4096 + 9]
    want = O.convert(src, src_dt, dst_dt)
    out = empty(src.size * ES[dst_dt])
    d.Convert(out, dev(src), src.size, dst_dt, src_dt)
    got = host(out, want.dtype)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


def test_convert_unaligned_and_tiny(d):
    for n in (1, 3, 17):
        src = np.arange(n, dtype=np.float32) * 0.37 - 1
        base = dev(np.concatenate([np.zeros(1, np.float32), src]))
        out = empty(n * 2 + 2)
        d.Convert(out[2:], base[4:], n, O.BF16, O.F32)
        assert np.array_equal(host(out[2:], np.uint16), O.convert(src, O.F32, O.BF16))


def test_convert_host_matches_and_checks_lengths(d):
    import puter_b200

    rng = np.random.default_rng(21)
    src = rng.integers(0, 2**32, (1 << 20) + 11, dtype=np.uint64).astype(np.uint32).view(np.float32)
    dst = np.zeros(src.size, np.uint16)
    d.ConvertHost(dst, src, O.BF16, O.F32)
    assert np.array_equal(dst, O.convert(src, O.F32, O.BF16))
    back = np.zeros(src.size, np.float32)
    d.ConvertHost(back, dst, O.F32, O.BF16)
    assert np.array_equal(back.view(np.uint32), O.convert(dst, O.BF16, O.F32).view(np.uint32))
    with pytest.raises(puter_b200.DeviceError) as e:  # convert.ErrLenMismatch
        d.ConvertHost(np.zeros(5, np.uint16), src[:6], O.BF16, O.F32)
    assert e.value.code == -2 and "length" in e.value.message


@pytest.mark.parametrize("op,code", [("Silu", O.SILU), ("Gelu", O.GELU), ("GeluTanh", O.GELU_TANH), ("Sigmoid", O.SIGMOID),
                                     ("Tanh", O.TANH), ("Relu", O.RELU)])
@pytest.mark.parametrize("n", LENGTHS)
def test_unary_f32(d, op, code, n):
    rng = np.random.default_rng(n + code)
    x = (rng.standard_normal(n) * 4).astype(np.float32)
    x[:1] = 0
    want = O.unary(code, O.F32, x)
    out = empty(n * 4)
    getattr(d, op)(out, dev(x), n, O.F32)
    got = host(out, np.float32)
    if op == "Gelu":  # erf comes from two math libraries; 1 + erf(x) cancels for very negative x
        assert np.allclose(got, want, rtol=1e-5, atol=1e-9)
    else:
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("op,code", [("Silu", O.SILU), ("Gelu", O.GELU), ("GeluTanh", O.GELU_TANH)])
@pytest.mark.parametrize("dt", [O.BF16, O.F16])
def test_unary_16bit_lut_every_pattern(d, op, code, dt):
    x = np.arange(65536, dtype=np.uint16)
    want = O.unary(code, dt, x)
    out = empty(65536 * 2)
    getattr(d, op)(out, dev(x), 65536, dt)
    got = host(out, np.uint16)
    nan = np.isnan(O.to_f32(want, dt))
    diff = ulp16_diff(got[~nan], want[~nan])
    if op == "Gelu":  # two erf implementations: equal except where 1 + erf(x) cancels (x << 0) or on rounding ties
        gf, wf = O.to_f32(got[~nan], dt), O.to_f32(want[~nan], dt)
        assert np.allclose(gf, wf, rtol=1e-2, atol=1e-9)
    else:
        assert diff.max() == 0, (op, int(diff.max()), int((diff > 0).sum()))
    assert (diff > 0).mean() < 1e-3


GATED = [("SwiGLU", O.SWIGLU), ("GeGLU", O.GEGLU), ("GLU", O.GLU), ("ReGLU", O.REGLU), ("SiGLU", O.SIGLU), ("GeGLUTanh", O.GEGLU_TANH)]


@pytest.mark.parametrize("name,code", GATED)
@pytest.mark.parametrize("dt", [O.F32, O.BF16, O.F16])
@pytest.mark.parametrize("n", [7, 1024, 8192 + 3])
def test_gated_tensors(d, name, code, dt, n):
    rng = np.random.default_rng(n + code)
    g = O.from_f32(rng.standard_normal(n).astype(np.float32) * 3, dt)
    u = O.from_f32(rng.standard_normal(n).astype(np.float32), dt)
    want = O.gated_tensors(code, dt, g, u)
    out = empty(n * ES[dt])
    getattr(d, name + "Tensors")(out, dev(g), dev(u), n, dt)
    got = host(out, want.dtype)
    if name == "GeGLU":
        assert rel_err(O.to_f32(got, dt), O.to_f32(want, dt)) <= (1e-6 if dt == O.F32 else 1e-2)
    elif name == "SwiGLU" and dt != O.F32:
        # 16-bit SwiGLU: at most one unit in the last place.  f16 evaluates the reference polynomial with fused multiply-adds
        # (differs rarely); bf16 takes the exponential from the special-function unit, which is closer to exp than the
        # reference's polynomial (about 2e-6 relative apart): results within that distance of a bf16 rounding boundary flip
        diff = ulp16_diff(got, want)
        assert diff.max() <= 1 and (diff > 0).mean() <= (3e-3 if dt == O.BF16 else 1e-3)
    else:
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


@pytest.mark.parametrize("dt", [O.F32, O.BF16])
@pytest.mark.parametrize("batch,half", [(1, 7), (5, 64), (3, 1376)])
def test_swiglu_packed(d, dt, batch, half):
    rng = np.random.default_rng(batch * half)
    packed = O.from_f32(rng.standard_normal((batch, 2 * half)).astype(np.float32), dt)
    want = O.gated_packed(O.SWIGLU, dt, packed, batch, half)
    out = empty(batch * half * ES[dt])
    d.SwiGLU(out, dev(packed), batch, half, dt)
    got = host(out, want.dtype).reshape(batch, half)
    if dt == O.F32 or half % 8:  # float32 and the element-at-a-time path are bit-identical to the reference
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8))
    else:
        diff = ulp16_diff(got, want)
        assert diff.max() <= 1 and (diff > 0).mean() <= 3e-3  # bf16: exponential from the special-function unit (see above)


@pytest.mark.parametrize("op,code", [("Add", O.ADD), ("Sub", O.SUB), ("Mul", O.MUL), ("Div", O.DIV), ("Max", O.MAX), ("Min", O.MIN)])
@pytest.mark.parametrize("dt", [O.F32, O.BF16, O.F16])
def test_binary(d, op, code, dt):
    n = 8192 + 5
    rng = np.random.default_rng(code)
    a = O.from_f32(rng.standard_normal(n).astype(np.float32), dt)
    b = O.from_f32(rng.standard_normal(n).astype(np.float32) + 0.1, dt)
    want = O.binary(code, dt, a, b)
    out = empty(n * ES[dt])
    getattr(d, op)(out, dev(a), dev(b), n, dt)
    assert np.array_equal(host(out, want.dtype).view(np.uint8), want.view(np.uint8))


def test_zero_size_is_a_silent_noop(d):
    out = empty(16)
    d.Add(out, out, out, 0, O.F32)
    d.Silu(out, out, 0, O.BF16)
    d.RMSNorm(__import__("puter_b200").RMSNormConfig(1e-5), out, out, out, 0, 4, O.F32)
    assert bool((out.cpu() == 0xAB).all())


@pytest.mark.parametrize("dt", [O.F32, O.BF16, O.F16])
@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 7), (128, 512), (5, 4096), (2, 8192 * 2 + 8), (4, 100)])
def test_rmsnorm(d, dt, rows, cols):
    import puter_b200

    rng = np.random.default_rng(rows * cols)
    x = O.from_f32(rng.standard_normal((rows, cols)).astype(np.float32), dt)
    g = O.from_f32(rng.uniform(0.5, 1.5, cols).astype(np.float32), dt)
    eps = 1e-5
    want = O.rmsnorm(dt, x, g, eps)
    out = empty(rows * cols * ES[dt])
    d.RMSNorm(puter_b200.RMSNormConfig(eps), dev(x), dev(g), out, rows, cols, dt)
    got = host(out, want.dtype, (rows, cols))
    if dt == O.F32:
        assert rel_err(got, want) <= 1e-6
    else:
        # the float32 row sum is a tree instead of a sequential loop: a row may land on the other side of a
        # 16-bit rounding boundary of the sum, which moves its outputs by at most one unit in the last place
        diff = ulp16_diff(got, want)
        assert diff.max() <= 1
        assert (diff.max(axis=1) > 0).mean() <= 0.34 or rows < 8


def test_rmsnorm_rejects_bad_epsilon(d):
    import puter_b200

    x = dev(np.ones(8, np.float32))
    with pytest.raises(puter_b200.DeviceError) as e:
        d.RMSNorm(puter_b200.RMSNormConfig(0.0), x, x, x, 2, 4, O.F32)
    assert e.value.code == -2 and "epsilon must be positive" in e.value.message


def test_gated_residual_known_answers(d):
    # execution/math_gated_residual_intrinsic_test.go:17-65
    res = np.arange(1, 13, dtype=np.float32)
    br = np.ones(12, np.float32)
    mod = np.array([0, 0, 0, 0, 0, 0, 0.5, 1, 2, 0, 0, 0, 0, 0, 0, 3, 4, 5], np.float32)
    out = empty(48)
    d.GatedResidual(dev(res), dev(br), dev(mod), out, 4, 3, 2, 9, 0, O.F32)
    assert host(out, np.float32).tolist() == [1.5, 3, 5, 4.5, 6, 8, 10, 12, 14, 13, 15, 17]


@pytest.mark.parametrize("dt", [O.F32, O.BF16, O.F16])
@pytest.mark.parametrize("rows,cols,rpb,sets,set_", [(8, 3, 4, 2, 1), (64, 256, 16, 1, 0), (33, 1024, 11, 3, 2)])
def test_gated_residual(d, dt, rows, cols, rpb, sets, set_):
    import puter_b200

    rng = np.random.default_rng(rows + cols)
    batches = (rows + rpb - 1) // rpb
    mod_cols = sets * 3 * cols
    res = O.from_f32(rng.standard_normal(rows * cols).astype(np.float32), dt)
    br = O.from_f32(rng.standard_normal(rows * cols).astype(np.float32), dt)
    mod = O.from_f32(rng.uniform(0, 1, batches * mod_cols).astype(np.float32), dt)
    want = O.gated_residual(dt, res, br, mod, rows, cols, rpb, mod_cols, set_)
    out = empty(rows * cols * ES[dt])
    d.GatedResidual(dev(res), dev(br), dev(mod), out, rows, cols, rpb, mod_cols, set_, dt)
    assert np.array_equal(host(out, want.dtype).view(np.uint8), want.view(np.uint8))
    with pytest.raises(puter_b200.DeviceError):  # modulation too narrow for the set
        d.GatedResidual(dev(res), dev(br), dev(mod), out, rows, cols, rpb, mod_cols, sets, dt)


@pytest.mark.parametrize("dt", [O.BF16, O.F32])
def test_fused_add_rmsnorm_gated_residual_equals_unfused_ops(d, dt):
    import puter_b200

    rows, cols, rpb = 96, 1024, 32
    rng = np.random.default_rng(3)
    x = O.from_f32(rng.standard_normal((rows, cols)).astype(np.float32), dt)
    r = O.from_f32(rng.standard_normal((rows, cols)).astype(np.float32), dt)
    br = O.from_f32(rng.standard_normal((rows, cols)).astype(np.float32), dt)
    g = O.from_f32(rng.uniform(0.5, 1.5, cols).astype(np.float32), dt)
    mod = O.from_f32(rng.uniform(0, 1, (rows // rpb) * 3 * cols).astype(np.float32), dt)
    h = O.binary(O.ADD, dt, x, r)
    n = O.rmsnorm(dt, h.reshape(rows, cols), g, 1e-6)
    gr = O.gated_residual(dt, h, br, mod, rows, cols, rpb, 3 * cols, 0)
    ho, no, go = (empty(rows * cols * ES[dt]) for _ in range(3))
    d.AddRMSNormGatedResidual(puter_b200.RMSNormConfig(1e-6), dev(x), dev(r), dev(g), dev(br), dev(mod), ho, no, go, rows, cols, rpb,
                              3 * cols, 0, dt)
    assert np.array_equal(host(ho, h.dtype).view(np.uint8), h.ravel().view(np.uint8))
    assert np.array_equal(host(go, gr.dtype).view(np.uint8), gr.ravel().view(np.uint8))
    if dt == O.F32:
        assert rel_err(host(no, np.float32), n) <= 1e-6
    else:
        assert ulp16_diff(host(no, np.uint16), n.ravel()).max() <= 1


@pytest.mark.parametrize("dt,cols", [(O.BF16, 16384), (O.F32, 8192), (O.BF16, 1024), (O.F16, 4100)])
@pytest.mark.parametrize("inplace", [False, True])
def test_fused_and_plain_rmsnorm_long_rows_in_place_and_out_of_place(d, dt, cols, inplace):
    """Rows longer than the register cache of the row kernel (more than 8192 16-bit / 4096 float32 columns) take its second
    pass over memory; with the residual stream updated in place (hOut = x) that pass must not add the residual twice."""
    import puter_b200

    rows, rpb = 12, 4
    rng = np.random.default_rng(cols)
    x = O.from_f32(rng.standard_normal((rows, cols)).astype(np.float32), dt)
    r = O.from_f32(rng.standard_normal((rows, cols)).astype(np.float32), dt)
    br = O.from_f32(rng.standard_normal((rows, cols)).astype(np.float32), dt)
    g = O.from_f32(rng.uniform(0.5, 1.5, cols).astype(np.float32), dt)
    mod = O.from_f32(rng.uniform(0, 1, (rows // rpb) * 3 * cols).astype(np.float32), dt)
    h = O.binary(O.ADD, dt, x, r)
    n = O.rmsnorm(dt, h.reshape(rows, cols), g, 1e-6)
    gr = O.gated_residual(dt, h, br, mod, rows, cols, rpb, 3 * cols, 0)
    xd, rd = dev(x), dev(r)
    ho = xd if inplace else empty(x.nbytes)
    go = rd if inplace else empty(x.nbytes)   # the gated output reuses the residual's buffer
    no = empty(x.nbytes)
    d.AddRMSNormGatedResidual(puter_b200.RMSNormConfig(1e-6), xd, rd, dev(g), dev(br), dev(mod), ho, no, go, rows, cols, rpb, 3 * cols, 0, dt)
    assert np.array_equal(host(ho, h.dtype).view(np.uint8), h.ravel().view(np.uint8))
    assert np.array_equal(host(go, gr.dtype).view(np.uint8), gr.ravel().view(np.uint8))
    if dt == O.F32:
        assert rel_err(host(no, np.float32), n) <= 1e-6
    else:
        assert ulp16_diff(host(no, np.uint16), n.ravel()).max() <= 1
    # plain RMSNorm, output over its input
    xd = dev(h)
    out = xd if inplace else empty(x.nbytes)
    d.RMSNorm(puter_b200.RMSNormConfig(1e-6), xd, dev(g), out, rows, cols, dt)
    if dt == O.F32:
        assert rel_err(host(out, np.float32), n) <= 1e-6
    else:
        assert ulp16_diff(host(out, np.uint16), n.ravel()).max() <= 1


def test_rmsnorm_refuses_overlaps_it_cannot_run_in_place(d):
    import puter_b200

    rows, cols = 4, 256
    buf = dev(np.zeros(rows * cols * 2 + 64, np.float32))
    x, shifted = buf[:rows * cols * 4], buf[64:64 + rows * cols * 4]
    g = dev(np.ones(cols, np.float32))
    cfg = puter_b200.RMSNormConfig(1e-6)
    with pytest.raises(puter_b200.DeviceError) as e:  # partial overlap of input and output
        d.RMSNorm(cfg, x, g, shifted, rows, cols, O.F32)
    assert e.value.code == -2
    r = dev(np.zeros(rows * cols, np.float32))
    o = empty(rows * cols * 4)
    with pytest.raises(puter_b200.DeviceError) as e:  # two outputs in one buffer
        d.AddRMSNormGatedResidual(cfg, x, r, g, None, None, o, o, None, rows, cols, 0, 0, 0, O.F32)
    assert e.value.code == -2


ROPE_CASES = [dict(base=10000.0, start=0, mode=0, scaling=0, factor=1.0, low=0.0, high=0.0, orig_ctx=0),
              dict(base=10000.0, start=5, mode=1, scaling=0, factor=1.0, low=0.0, high=0.0, orig_ctx=0),
              dict(base=500000.0, start=3, mode=1, scaling=1, factor=32.0, low=1.0, high=4.0, orig_ctx=8192),
              dict(base=500000.0, start=0, mode=0, scaling=1, factor=8.0, low=1.0, high=4.0, orig_ctx=8192)]


@pytest.mark.parametrize("dt", [O.F32, O.BF16, O.F16])
@pytest.mark.parametrize("cfg", ROPE_CASES)
@pytest.mark.parametrize("seq,heads,dim", [(1, 1, 2), (7, 2, 8), (64, 3, 64), (1024, 2, 128), (130, 5, 6)])
def test_rope(d, dt, cfg, seq, heads, dim):
    import puter_b200

    rng = np.random.default_rng(seq * dim)
    x = O.from_f32(((rng.random(seq * heads * dim) - 0.5) * 4).astype(np.float32), dt)
    want = O.rope(dt, x, seq, heads, dim, **cfg)
    out = empty(x.size * ES[dt])
    rc = puter_b200.RoPEConfig(cfg["base"], cfg["start"], cfg["mode"], cfg["scaling"], cfg["factor"], cfg["low"], cfg["high"], cfg["orig_ctx"])
    d.RoPE(rc, dev(x), out, seq, heads, dim, dt)
    got = host(out, want.dtype)
    if dt == O.F32:
        # cos/sin come from two float64 math libraries; after the cast to float32 they agree except on rare ties
        assert np.abs(got - want).max() <= 1e-5 * max(1.0, float(np.abs(want).max()))
        assert (got.view(np.uint32) != want.view(np.uint32)).mean() < 1e-3
    else:
        assert ulp16_diff(got, want).max() <= 1
        assert (got != want).mean() < 1e-3


def test_rope_validation_and_noop(d):
    import puter_b200

    x = dev(np.ones(16, np.float32))
    out = empty(64)
    d.RoPE(puter_b200.RoPEConfig(), x, out, 2, 1, 7, O.F32)  # odd head dimension: no-op (device/cpu/rope/compute.go:17-19)
    assert bool((out.cpu() == 0xAB).all())
    with pytest.raises(puter_b200.DeviceError) as e:
        d.RoPE(puter_b200.RoPEConfig(BaseFreq=0.0), x, out, 2, 1, 8, O.F32)
    assert "base frequency must be positive" in e.value.message
    with pytest.raises(puter_b200.DeviceError):
        d.RoPE(puter_b200.RoPEConfig(Scaling=1, ScalingFactor=8.0, LowFreqFactor=4.0, HighFreqFactor=1.0, OriginalContext=8192), x, out,
               2, 1, 8, O.F32)


def test_rope_pairs(d):
    import puter_b200

    rng = np.random.default_rng(9)
    half = 37
    x = rng.standard_normal(2 * half).astype(np.float32)
    c = rng.standard_normal(half).astype(np.float32)
    s = rng.standard_normal(half).astype(np.float32)
    out = empty(8 * half)
    d.RoPEPairs(out, dev(x), dev(c), dev(s), half, O.F32)
    assert np.array_equal(host(out, np.float32).view(np.uint32), O.rope_pairs(x, c, s).view(np.uint32))
    with pytest.raises(puter_b200.DeviceError):
        d.RoPEPairs(out, dev(x), dev(c), dev(s), half, O.BF16)


def test_page_write_gather_known_answer(d):
    # execution/page_intrinsic_test.go:15-72,403-470
    storage = dev(np.zeros(12, np.float32))
    d.KVPageWrite(storage, dev(np.array([7, 8], np.float32)), dev(np.array([1, 1], np.int32)), dev(np.array([0, 1], np.int32)), storage,
                  3, 2, 1, 2, 6, O.F32)
    flat = host(storage, np.float32)
    assert flat[8] == 7 and flat[9] == 8 and flat.sum() == 15
    out = empty(8)
    d.KVPageGather(storage, dev(np.array([1], np.int32)), out, 3, 2, 1, 2, 6, O.F32)
    assert host(out, np.float32).tolist() == [7, 8]


@pytest.mark.parametrize("n", LENGTHS)
@pytest.mark.parametrize("dt,inner", [(O.F32, 8), (O.BF16, 8), (O.F16, 8), (O.BF16, 1024), (O.E4M3, 1024), (O.F32, 3)])
def test_page_roundtrip_and_oracle_equality(d, n, dt, inner):
    # device/cpu/shape/page_parity_test.go:59-118 (P=4, inner=8) plus KV-cache-sized rows
    rng = np.random.default_rng(n + inner)
    page_size = 4
    pages = (n + page_size - 1) // page_size + 2
    npdt = O.np_dtype(dt)
    vals = rng.integers(0, 256, (n, inner * ES[dt]), dtype=np.uint8).view(npdt)
    perm = rng.permutation(pages).astype(np.int32)
    ids = perm[np.arange(n) // page_size]
    offs = (np.arange(n) % page_size).astype(np.int32)
    storage0 = rng.integers(0, 256, pages * page_size * inner * ES[dt], dtype=np.uint8).view(npdt)
    want_storage = O.page_write(dt, storage0, vals, ids, offs, pages, page_size, inner)
    st = dev(storage0)
    out_st = empty(storage0.nbytes)
    d.KVPageWrite(st, dev(vals), dev(ids), dev(offs), out_st, pages, page_size, inner, n, 0, dt)  # functional form
    same = lambda a, b: np.array_equal(np.ascontiguousarray(a).view(np.uint8), np.ascontiguousarray(b).view(np.uint8))  # NaN-proof
    assert same(host(out_st, npdt), want_storage)
    assert same(host(st, npdt), storage0)
    d.KVPageWrite(st, dev(vals), dev(ids), dev(offs), st, pages, page_size, inner, n, 0, dt)  # in place
    assert same(host(st, npdt), want_storage)
    out = empty(n * inner * ES[dt])
    d.KVPageGather(st, dev(perm), out, pages, page_size, inner, n, 0, dt)
    got = host(out, npdt, (n, inner))
    assert same(got, vals)
    assert same(got, O.page_gather(dt, want_storage, perm, pages, page_size, inner, n))
    assert d.take_error() == 0


def test_page_ops_flag_bad_ids_without_touching_memory(d):
    storage = dev(np.zeros(4 * 2 * 4, np.float32))
    vals = dev(np.ones(2 * 4, np.float32))
    d.KVPageWrite(storage, vals, dev(np.array([9, -1], np.int32)), dev(np.array([0, 0], np.int32)), storage, 4, 2, 4, 2, 0, O.F32)
    assert d.take_error() == 1
    assert host(storage, np.float32).sum() == 0
    out = empty(2 * 16)
    d.KVPageGather(storage, dev(np.array([7], np.int32)), out, 4, 2, 4, 2, 0, O.F32)
    assert d.take_error() == 1
    assert d.take_error() == 0
