"""Parity of the CUDA int8 weight-only projection with the CPU oracle, through the C ABI (needs a B200).

The reference has no int8 x int8 -> int32 contraction on this path (activations are never int8); its projection
is (cast(x) @ cast(codes)) * scale with bf16-exact products and an f32 accumulate
(ir/.../inference/HfDecoderGraph.kt:625-655).  Two bars:
  - wherever the f32 accumulation is exact (integer-valued activations, partial sums below 2^24) the result must
    be the exact integer dot product, bit for bit, whatever the summation order;
  - otherwise rel 1e-2 / abs 2e-3 against the oracle on normalised activations and weights whose outputs are of order 1
    (uniform codes under small scales, or N(0, 0.02) weights quantized by the reference's rule).  The row-vector kernel and the bf16 tensor-core kernel differ from
    the oracle only in the f32 summation order (~1e-6 relative).  The int8 tensor-core kernel (17 to 128 rows) carries
    each activation row as 16-bit fixed point under a power-of-two row step s: its error is bounded by
    (s / 2) * scale[n] * sum_k |codes[k, n]|, checked below on rows with outlier channels.
The order-faithful kernel must equal the oracle bit for bit on any input.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from tlaloc_b200 import ops as o

    return o


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def model_like_weights(rng, k, n):
    """A projection weight as a checkpoint holds it, [out, in] ~ N(0, 0.02), through the reference's INT8 rule."""
    return oracle.quantize_int8((rng.standard_normal((n, k)) * 0.02).astype(np.float32))


def make(rng, m, k, n, x_int=False, unit_outputs=False):
    """The operator sweep's inputs: uniform codes, scales U(0.001, 0.02), N(0, 1) activations (outputs of rms ~60), or
    integer activations for the exactness cases.  `unit_outputs` divides the scales by 64 so that the outputs are of
    order 1, as a model's projections are: the cases that also run the int8 tensor-core form use it, because that
    form's absolute error scales with the output (see the error-bound test) while the abs 2e-3 bar does not."""
    codes = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
    scales = (rng.uniform(0.001, 0.02, size=n) / (64.0 if unit_outputs else 1.0)).astype(np.float32)
    if x_int:
        x = rng.integers(-8, 9, size=(m, k)).astype(np.float32)
    else:
        x = oracle.snap_bf16(rng.standard_normal((m, k)).astype(np.float32))
    return x, codes, scales


def close(got, want):
    err = np.abs(got - want)
    assert np.all(err <= 2e-3 + 1e-2 * np.abs(want)), err.max()
    return err.max()


@pytest.mark.parametrize("m", [1, 3, 8, 16, 17, 32])
@pytest.mark.parametrize("k,n", [(4096, 4096), (1024, 14336), (14336, 1024), (256, 688), (688, 256), (256, 1024), (2048, 4112)])
def test_integer_activations_give_the_exact_integer_dot_product(m, k, n):
    rng = np.random.default_rng(m * 7 + k + n)
    x, codes, _ = make(rng, m, k, n, x_int=True)
    want = (x.astype(np.float64) @ codes.astype(np.float64)).astype(np.float32)  # exact integers; |sum| <= 14336*8*127 < 2^24
    got = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), None)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), want)
    # power-of-two scales keep it exact too, and an f32 x is cast to bf16 on the way in
    scales = np.exp2(rng.integers(-8, -2, size=n)).astype(np.float32)
    got = ops().int8_gemm(dev(x), dev(codes), dev(scales))
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), want * scales[None, :])


@pytest.mark.parametrize("i8_mma", [True, False])
@pytest.mark.parametrize("m", [17, 33, 64, 100, 128, 256, 300])
@pytest.mark.parametrize("k,n", [(4096, 4096), (1024, 14336), (14336, 1024), (256, 688), (688, 256), (2048, 4112), (64, 256), (8240, 1296)])
def test_batched_rows_on_the_tensor_core_kernel_are_exact_on_integer_activations(m, k, n, i8_mma):
    """17 rows and more take a tcgen05 kernel: the bf16 form (int8 -> bf16 in shared memory) or, with `i8_mma` and up to
    128 rows, the int8 form (codes by TMA, activations as two int8 planes); accumulators in TMEM either way.
    K = 688 is not a multiple of 16, which the int8 form needs: those cases run the bf16 form twice."""
    from tlaloc_b200 import _native as N

    rng = np.random.default_rng(m * 11 + k + n)
    x, codes, _ = make(rng, m, k, n, x_int=True)
    want = (x.astype(np.float64) @ codes.astype(np.float64)).astype(np.float32)  # exact: every partial sum is an integer below 2^53
    scales = np.exp2(rng.integers(-8, -2, size=n)).astype(np.float32)
    res = rng.integers(-50, 50, size=(m, n)).astype(np.float32)
    got = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales), residual=dev(res), i8_mma=i8_mma)
    torch.cuda.synchronize()
    assert N.lib().tlaloc_b200_device_status() == 0
    assert np.array_equal(got.cpu().numpy(), want * scales[None, :] + res)


@pytest.mark.parametrize("i8_mma", [True, False])
@pytest.mark.parametrize("m", [64, 256])
def test_batched_rows_against_the_oracle(m, i8_mma):
    rng = np.random.default_rng(8)
    k, n = 4096, 14336
    x, codes, scales = make(rng, m, k, n, unit_outputs=i8_mma)
    want = oracle.proj_int8(x, codes, scales, round_x_bf16=True, threads=8)
    got = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales), i8_mma=i8_mma)
    torch.cuda.synchronize()
    worst = close(got.cpu().numpy(), want)
    assert worst <= 1e-4 * max(1.0, np.abs(want).max())
    # declaring the weights constant only moves their first loads ahead of the dependency wait: same bits
    again = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales), weights_const=True, i8_mma=i8_mma)
    torch.cuda.synchronize()
    assert torch.equal(again, got)


@pytest.mark.parametrize("m", [1, 8, 32])
@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 14336), (14336, 4096)])
def test_sweep_shapes_against_the_oracle(m, k, n):
    rng = np.random.default_rng(3)
    x, codes, scales = make(rng, m, k, n)
    want = oracle.proj_int8(x, codes, scales, round_x_bf16=True, threads=8)
    got = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales))
    torch.cuda.synchronize()
    worst = close(got.cpu().numpy(), want)
    assert worst <= 1e-4 * max(1.0, np.abs(want).max())


def test_vocabulary_head_shape_against_the_oracle():
    rng = np.random.default_rng(4)
    m, k, n = 8, 4096, 128256
    x, codes, scales = make(rng, m, k, n)
    want = oracle.proj_int8(x, codes, scales, round_x_bf16=True, threads=8)
    got = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales))
    torch.cuda.synchronize()
    close(got.cpu().numpy(), want)


def test_more_than_32_rows_residual_and_bf16_output():
    rng = np.random.default_rng(5)
    m, k, n = 70, 1024, 2048
    x, codes, scales = make(rng, m, k, n)
    res = rng.standard_normal((m, n)).astype(np.float32)
    want = oracle.proj_int8(x, codes, scales, round_x_bf16=True, threads=8) + res
    got = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales), residual=dev(res))
    torch.cuda.synchronize()
    close(got.cpu().numpy(), want)
    got_b = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales), residual=dev(res), out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    assert np.array_equal(got_b.float().cpu().numpy(), oracle.snap_bf16(got.cpu().numpy()))


@pytest.mark.parametrize("m,k,n", [(1, 8, 11), (2, 8, 8), (5, 37, 11), (4, 256, 688), (3, 300, 130)])
def test_order_faithful_kernel_is_bit_identical_to_the_oracle(m, k, n):
    rng = np.random.default_rng(k * n)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[0, min(3, k - 1)] = 0.0
    codes = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
    scales = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
    for round_x in (True, False):
        want = oracle.proj_int8(x, codes, scales, round_x_bf16=round_x)
        got = ops().int8_gemm(dev(x), dev(codes), dev(scales), exact=True, x_f32_exact=not round_x)
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy(), want)
    w = rng.standard_normal((k, n)).astype(np.float32)
    got = ops().dense_gemm_exact(dev(x), dev(w))
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), oracle.matmul_f32(x, w))
    wb = oracle.snap_bf16(w)
    got = ops().dense_gemm_exact(dev(x), dev(wb, torch.bfloat16))
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), oracle.matmul_f32(oracle.snap_bf16(x), wb))


def test_quantized_weights_round_trip_like_the_reference_identity():
    """int8 graph == graph of dequantized weights to 4.7e-6 relative (docs/CAPABILITIES.md:113), on the GPU path."""
    rng = np.random.default_rng(6)
    w = (rng.standard_normal((1024, 512)) * 0.02).astype(np.float32)  # [out, in]
    codes, scales = oracle.quantize_int8(w)
    x = oracle.snap_bf16(rng.standard_normal((4, 512)).astype(np.float32))
    got = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales)).cpu().numpy()
    deq = codes.astype(np.float32) * scales[None, :]
    want = (x.astype(np.float64) @ deq.astype(np.float64)).astype(np.float32)
    assert np.abs(got - want).max() <= 4.7e-6 * max(1.0, np.abs(want).max()) * 4
    assert np.abs(deq.T - w).max() <= np.abs(w).max() / 127.0 * 0.5 + 1e-9


def _exact_want_on_device(x, codes, scales, res):
    """The exact integer dot products in float64 on the device (sums of integers below 2^53 are exact in any order),
    column block by column block, narrowed to f32 and scaled like the kernel's epilogue."""
    tx = torch.from_numpy(x).to(DEV).double()
    out = torch.empty((x.shape[0], codes.shape[1]), dtype=torch.float32, device=DEV)
    tc = torch.from_numpy(codes).to(DEV)
    for c0 in range(0, codes.shape[1], 8192):
        out[:, c0:c0 + 8192] = (tx @ tc[:, c0:c0 + 8192].double()).float()
    out = out * torch.from_numpy(scales).to(DEV)[None, :]
    if res is not None:
        out = out + torch.from_numpy(res).to(DEV)
    return out, tc


# The projections of the 70B-shape decode step at batch 128 (K x N: q|k|v, o, gate|up, down), the shards one of eight
# tensor-parallel ranks holds, and the vocabulary head.
STEP_SHAPES = [(8192, 10240), (8192, 8192), (8192, 57344), (28672, 8192),
               (8192, 1280), (1024, 8192), (8192, 7168), (3584, 8192)]


@pytest.mark.parametrize("i8_mma", [True, False])
@pytest.mark.parametrize("k,n", STEP_SHAPES)
def test_decode_step_shapes_at_128_rows(k, n, i8_mma):
    """Exact on integer activations over the whole output; against the oracle on a sample of rows for N(0,1) ones;
    on the int8 and on the bf16 form of the tensor-core kernel."""
    from tlaloc_b200 import _native as N

    m = 128
    rng = np.random.default_rng(k + n)
    codes = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
    span = 4 if k > 16384 else 8  # keeps every partial sum an integer below 2^24
    x = rng.integers(-span, span + 1, size=(m, k)).astype(np.float32)
    scales = np.exp2(rng.integers(-8, -2, size=n)).astype(np.float32)
    res = rng.integers(-50, 50, size=(m, n)).astype(np.float32)
    want, tc = _exact_want_on_device(x, codes, scales, res)
    got = ops().int8_gemm(dev(x, torch.bfloat16), tc, dev(scales), residual=dev(res), weights_const=True, i8_mma=i8_mma)
    torch.cuda.synchronize()
    assert N.lib().tlaloc_b200_device_status() == 0
    assert torch.equal(got, want)
    xn = oracle.snap_bf16(rng.standard_normal((m, k)).astype(np.float32))
    sc = (rng.uniform(0.001, 0.02, size=n) / (64.0 if i8_mma else 1.0)).astype(np.float32)  # int8 form: outputs of order 1
    got = ops().int8_gemm(dev(xn, torch.bfloat16), tc, dev(sc), i8_mma=i8_mma).cpu().numpy()
    rows = [0, 77, 127]
    wantn = oracle.proj_int8(xn[rows], codes, sc, round_x_bf16=True, threads=oracle.host_threads())
    worst = close(got[rows], wantn)
    assert worst <= 1e-4 * max(1.0, np.abs(wantn).max())


@pytest.mark.parametrize("m", [1, 32, 256])
def test_vocabulary_head_shape_at_1_32_and_256_rows(m):
    from tlaloc_b200 import _native as N

    k, n = 4096, 128256
    rng = np.random.default_rng(m)
    codes = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
    x = rng.integers(-8, 9, size=(m, k)).astype(np.float32)
    scales = np.exp2(rng.integers(-8, -2, size=n)).astype(np.float32)
    want, tc = _exact_want_on_device(x, codes, scales, None)
    got = ops().int8_gemm(dev(x, torch.bfloat16), tc, dev(scales))
    torch.cuda.synchronize()
    assert N.lib().tlaloc_b200_device_status() == 0
    assert torch.equal(got, want)
    xn = oracle.snap_bf16(rng.standard_normal((m, k)).astype(np.float32))
    sc = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
    got = ops().int8_gemm(dev(xn, torch.bfloat16), tc, dev(sc)).cpu().numpy()
    rows = sorted({0, m // 2, m - 1})
    wantn = oracle.proj_int8(xn[rows], codes, sc, round_x_bf16=True, threads=oracle.host_threads())
    close(got[rows], wantn)


def test_views_off_a_16_byte_boundary_take_the_order_faithful_kernel():
    """x + 4 elements or a weight matrix that starts at an odd byte must not reach the 16-byte copies of the fast
    kernels: the call falls back and still agrees with the oracle (bit for bit: it is the order-faithful kernel)."""
    rng = np.random.default_rng(12)
    m, k, n = 8, 512, 1024
    x, codes, scales = make(rng, m, k, n)
    want = oracle.proj_int8(x, codes, scales, round_x_bf16=True)
    xbuf = torch.zeros((m * k + 4,), dtype=torch.bfloat16, device=DEV)
    xv = xbuf[4:].view(m, k)  # starts 8 bytes into the allocation
    xv.copy_(dev(x, torch.bfloat16))
    assert xv.data_ptr() % 16 == 8
    got = ops().int8_gemm(xv, dev(codes), dev(scales))
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), want)
    cbuf = torch.zeros((k * n + 1,), dtype=torch.int8, device=DEV)
    cv = cbuf[1:].view(k, n)  # starts one byte into the allocation
    cv.copy_(dev(codes))
    for rows in (m, 64):  # the row-vector kernel's range and the tensor-core kernel's
        xr = oracle.snap_bf16(rng.standard_normal((rows, k)).astype(np.float32))
        got = ops().int8_gemm(dev(xr, torch.bfloat16), cv, dev(scales))
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy(), oracle.proj_int8(xr, codes, scales, round_x_bf16=True))
    with pytest.raises(ValueError, match="INT8_PROJ out"):
        ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales), out=torch.empty((m, n + 16), device=DEV))


@pytest.mark.parametrize("m", [8, 64])
def test_every_code_value_converts_exactly(m):
    """All 256 byte values as weights (-128, which the quantizer never emits, included): one-hot activations
    read each code back, on the row-vector kernel and on the tensor-core kernel."""
    k, n = 256, 256
    codes = np.zeros((k, n), np.int8)
    for j in range(n):
        codes[:, j] = np.roll(np.arange(-128, 128), j).astype(np.int8)
    x = np.zeros((m, k), np.float32)
    for i in range(m):
        x[i, (5 * i) % k] = 1.0
        x[i, (7 * i + 3) % k] += 2.0
    want = x.astype(np.float64) @ codes.astype(np.float64)
    got = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), None)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), want.astype(np.float32))


@pytest.mark.parametrize("i8_mma", [True, False])
@pytest.mark.parametrize("m,k,n2", [(128, 512, 512), (64, 4096, 2048), (33, 256, 256), (200, 1024, 7168), (128, 8192, 1024), (256, 688, 512), (8, 512, 512)])
def test_gate_up_projection_with_swiglu_in_the_epilogue(m, k, n2, i8_mma):
    """tlaloc_b200_int8_gemm_swiglu against the two-step path (gate|up projection, then the SwiGLU kernel) on the same
    weights: the same f32 sums meet the same SiLU arithmetic, so the results are bit-equal on the bf16 tensor-core
    kernel and within f32 rounding of the K slices' partial sums on the int8 one; and against the oracle.  Shapes cover
    one and several K slices per tile, one and two accumulators, and (8 rows) the order-faithful fallback."""
    from tlaloc_b200 import _native as N
    from tlaloc_b200 import sharding

    rng = np.random.default_rng(m + k + n2)
    f = n2 // 2
    x = oracle.snap_bf16(rng.standard_normal((m, k)).astype(np.float32))
    gate, up = model_like_weights(rng, k, f), model_like_weights(rng, k, f)
    codes, scales = sharding.interleave_gate_up(gate, up)
    got = ops().int8_gemm_swiglu(dev(x, torch.bfloat16), dev(codes), dev(scales), out_dtype=torch.float32, i8_mma=i8_mma)
    torch.cuda.synchronize()
    assert N.lib().tlaloc_b200_device_status() == 0
    g = ops().int8_gemm(dev(x, torch.bfloat16), dev(gate[0]), dev(gate[1]), i8_mma=i8_mma)
    u = ops().int8_gemm(dev(x, torch.bfloat16), dev(up[0]), dev(up[1]), i8_mma=i8_mma)
    two_step = ops().swiglu(g, u)
    torch.cuda.synchronize()
    want = oracle.swiglu(oracle.proj_int8(x, gate[0], gate[1], threads=8), oracle.proj_int8(x, up[0], up[1], threads=8))
    close(got.cpu().numpy(), want)
    if m > 32 and (not i8_mma or m > 128 or k % 16):
        assert torch.equal(got, two_step)
    elif m > 32:
        assert torch.allclose(got, two_step, rtol=1e-5, atol=1e-6)
    got_b = ops().int8_gemm_swiglu(dev(x, torch.bfloat16), dev(codes), dev(scales), i8_mma=i8_mma)
    assert got_b.dtype == torch.bfloat16 and np.array_equal(got_b.float().cpu().numpy(), oracle.snap_bf16(got.cpu().numpy()))


def _row_steps(x):
    """The int8 kernel's power-of-two row step: the smallest 2^e with max|x[m, :]| / 2^e <= 127 * 256."""
    amax = np.abs(x).max(axis=1).astype(np.float64)
    e = np.ceil(np.log2(np.maximum(amax, 1e-300) / (127.0 * 256.0)))
    return np.where(amax > 0, np.exp2(e), 1.0)


@pytest.mark.parametrize("m,k,n", [(128, 4096, 4096), (17, 8192, 1280), (100, 2064, 1296)])
def test_int8_tensor_core_kernel_stays_inside_its_error_bound_on_outlier_channels(m, k, n):
    """Rows whose largest magnitudes sit in a few channels 60 times the rest (what RMSNorm gains do to a model's
    activations): the int8 form rounds the small elements to multiples of the row step s, so every output is within
    (s / 2) * scale[n] * sum_k |codes[k, n]| of the exact product (plus the f32 rounding of the result); the bf16 form
    on the same inputs is within f32 summation error."""
    rng = np.random.default_rng(m + k + n)
    codes, scales = model_like_weights(rng, k, n)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[:, ::97] *= 60.0
    x = oracle.snap_bf16(x)
    exact = (torch.from_numpy(x).to(DEV).double() @ torch.from_numpy(codes).to(DEV).double()).cpu().numpy() * scales[None, :].astype(np.float64)
    got = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales), i8_mma=True).double().cpu().numpy()
    bound = 0.5 * _row_steps(x)[:, None] * (scales.astype(np.float64) * np.abs(codes.astype(np.float64)).sum(axis=0))[None, :]
    err = np.abs(got - exact)
    assert np.all(err <= bound + 4e-7 * np.abs(exact) + 1e-30), float((err - bound).max())
    assert err.max() > 0  # the bound is not vacuous: these rows do lose bits
    assert np.sqrt((err ** 2).mean()) <= 1e-3 * np.sqrt((exact ** 2).mean())
    got_bf = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales)).double().cpu().numpy()
    assert np.sqrt(((got_bf - exact) ** 2).mean()) <= 1e-5 * np.sqrt((exact ** 2).mean())


def test_int8_tensor_core_kernel_rows_with_infinity_or_nan_come_out_nan_and_leave_the_others_alone():
    rng = np.random.default_rng(21)
    m, k, n = 40, 512, 512
    x, codes, scales = make(rng, m, k, n)
    clean = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales), i8_mma=True).cpu().numpy()
    x[3, 17] = np.inf
    x[9, 400] = np.nan
    got = ops().int8_gemm(dev(x, torch.bfloat16), dev(codes), dev(scales), i8_mma=True).cpu().numpy()
    assert np.isnan(got[3]).all() and np.isnan(got[9]).all()
    keep = [r for r in range(m) if r not in (3, 9)]
    assert np.array_equal(got[keep], clean[keep])
    # all-zero rows and an f32 x (rounded to bf16 on the way in, like the other kernels)
    x = oracle.snap_bf16(rng.standard_normal((m, k)).astype(np.float32))
    x[5] = 0.0
    xf = x + rng.uniform(-1e-4, 1e-4, size=x.shape).astype(np.float32) * (x != 0)
    a = ops().int8_gemm(dev(oracle.snap_bf16(xf), torch.bfloat16), dev(codes), dev(scales), i8_mma=True)
    b = ops().int8_gemm(dev(xf), dev(codes), dev(scales), i8_mma=True)
    torch.cuda.synchronize()
    assert torch.equal(a, b) and not a[5].any()


@pytest.mark.parametrize("rows,n", [(128, 8192), (40, 512), (17, 16384), (64, 4096)])
def test_rmsnorm_writes_the_planes_the_projections_quantizer_would(rows, n):
    """tlaloc_b200_rmsnorm_planes leaves, beside the bf16 rows, the activation planes of the int8 tensor-core projection
    that consumes them: bit for bit what that projection's own quantizer launch writes for the same rows (hi, lo and the
    row steps), so the projection called with x_planes gives the same bits with one launch less.  16384 columns take the
    two-launch fallback (the row does not fit the registers)."""
    from tlaloc_b200 import _native as N

    rng = np.random.default_rng(rows + n)
    x = rng.standard_normal((rows, n)).astype(np.float32) * 3.0
    x[1] = 0.0
    gain = rng.uniform(0.5, 1.5, size=n).astype(np.float32)
    k, nn = n, 512
    codes = rng.integers(-127, 128, size=(k, nn), dtype=np.int8)
    scales = (rng.uniform(0.001, 0.02, size=nn) / 64.0).astype(np.float32)
    o = ops()
    nbytes = o.int8_gemm_scratch_bytes(rows, n, 0)
    scr_a = torch.zeros((nbytes + 3) // 4, dtype=torch.float32, device=DEV)
    scr_b = torch.zeros_like(scr_a)
    plain = o.rmsnorm(dev(x), dev(gain), 1e-5, out_dtype=torch.bfloat16)
    hn = o.rmsnorm(dev(x), dev(gain), 1e-5, planes=scr_a)
    assert torch.equal(hn, plain)
    before = N.lib().tlaloc_b200_launch_count()
    y_a = o.int8_gemm(hn, dev(codes), dev(scales), scratch=scr_a, i8_mma=True, x_planes=True)
    assert N.lib().tlaloc_b200_launch_count() - before == 1
    y_b = o.int8_gemm(hn, dev(codes), dev(scales), scratch=scr_b, i8_mma=True)  # quantizer + projection
    torch.cuda.synchronize()
    used = (2 * rows * n + 4 * rows) // 4
    assert torch.equal(scr_a[:used].view(torch.int32), scr_b[:used].view(torch.int32))
    assert torch.equal(y_a, y_b)
    want = oracle.proj_int8(hn.float().cpu().numpy(), codes, scales, threads=8)
    close(y_a.cpu().numpy(), want)


def test_activation_planes_match_their_definition():
    """The quantizer's output against a numpy restatement of its rule: s = the smallest power of two with max|x| / s <=
    127 * 256, q = rint(x / s) (ties to even), hi = floor((q + 128) / 256), lo = q - 256 hi; bit for bit, on rows with
    outlier channels, a zero row, a tiny row and a row whose largest magnitude sits just below a power of two."""
    rng = np.random.default_rng(77)
    m, k = 48, 2048
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[:, ::61] *= 50.0
    x[2] = 0.0
    x[3] *= 1e-30
    x[4, 7] = np.float32(255.0 / 256.0 * 64.0)  # 0.99609375 * 2^6: the step must move up one power of two
    x[4, 8:] *= 0.01
    x = oracle.snap_bf16(x)
    o = ops()
    scr = torch.zeros((o.int8_gemm_scratch_bytes(m, k, 0) + 3) // 4, dtype=torch.float32, device=DEV)
    o.int8_gemm(dev(x, torch.bfloat16), torch.zeros((k, 256), dtype=torch.int8, device=DEV), None, scratch=scr, i8_mma=True)
    torch.cuda.synchronize()
    raw = scr.view(torch.int8)
    hi = raw[:m * k].view(m, k).cpu().numpy().astype(np.int64)
    lo = raw[m * k:2 * m * k].view(m, k).cpu().numpy().astype(np.int64)
    steps = scr[(2 * m * k) // 4:(2 * m * k) // 4 + m].cpu().numpy().astype(np.float64)
    want_steps = _row_steps(x)
    want_steps[3] = max(want_steps[3], 2.0 ** -126)  # the step's exponent stops at the smallest normal f32
    assert np.array_equal(steps, want_steps)
    q = np.rint(x.astype(np.float64) / want_steps[:, None]).astype(np.int64)
    want_hi = (q + 128) >> 8
    assert np.array_equal(hi, want_hi) and np.array_equal(lo, q - 256 * want_hi)
    assert np.abs(hi).max() <= 127 and lo.min() >= -128 and lo.max() <= 127
    assert np.array_equal((256 * hi + lo)[4, 7] * steps[4], np.float64(x[4, 7]))  # exact where the row's bits allow
