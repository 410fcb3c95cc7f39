"""GPU parity for the dense f16/bf16 GEMM (mircuda_dense_*) and the int4-g128 W4A16 op."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def assert_close(actual: torch.Tensor, expected: torch.Tensor, what: str):
    actual, expected = actual.double().cpu(), expected.double().cpu()
    assert torch.isfinite(actual).all(), what
    scale = expected.abs().max().clamp_min(1e-30)
    assert (actual - expected).abs().max() <= 1e-2 * scale, what
    assert (actual - expected).norm() <= 5e-3 * expected.norm().clamp_min(1e-30), what


def run_dense(stream, a, b, c, spec, alpha, beta):
    from mircuda_b200 import dense
    plan = dense.DenseMatmulPlan(stream, spec)
    torch.cuda.synchronize()
    plan.execute(stream, a.reshape(-1), b.reshape(-1), c.view(-1), alpha, beta)
    stream.synchronize()
    plan.close()
    return c


@pytest.mark.parametrize("m", [1, 128])
def test_dense_bf16_golden(cuda_stream, m):
    """tests/cutlass/dense/mod.rs:22-26 (run_bf16): ones x ones, N = K = 128 -> 128."""
    from mircuda_b200 import dense
    a = torch.ones(m, 128, dtype=torch.bfloat16, device="cuda")
    b = torch.ones(128, 128, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros(m, 128, dtype=torch.bfloat16, device="cuda")
    run_dense(cuda_stream, a, b, c, dense.DenseMatmulSpec(m, 128, 128), 1.0, 0.0)
    assert (c.float() == 128.0).all()


def test_dense_bf16_wide_decode_golden(cuda_stream):
    """tests/cutlass/dense/mod.rs:28-40: M = 1, N = 8192, K = 128."""
    from mircuda_b200 import dense
    a = torch.ones(1, 128, dtype=torch.bfloat16, device="cuda")
    b = torch.ones(8192, 128, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros(1, 8192, dtype=torch.bfloat16, device="cuda")
    run_dense(cuda_stream, a, b, c, dense.DenseMatmulSpec(1, 8192, 128), 1.0, 0.0)
    assert (c.float() == 128.0).all()


def test_dense_bf16_fp32_output_golden(cuda_stream):
    """tests/cutlass/dense/mod.rs:42-58: the f32 result must not be rounded to bf16."""
    from mircuda_b200 import dense
    a = torch.full((1, 128), 0.1, dtype=torch.bfloat16, device="cuda")
    b = torch.full((128, 128), 0.1, dtype=torch.bfloat16, device="cuda")
    c = torch.full((1, 128), float("nan"), dtype=torch.float32, device="cuda")
    run_dense(cuda_stream, a, b, c, dense.DenseMatmulSpec(1, 128, 128, torch.bfloat16, torch.float32), 1.0, 0.0)
    assert torch.isfinite(c).all() and (c - c[0, 0]).abs().max() < 1.2e-7
    assert abs(float(c[0, 0]) - float(c[0, 0].to(torch.bfloat16))) > 1.2e-7


def test_dense_bf16_unaligned_golden(cuda_stream):
    """tests/cutlass/dense/mod.rs:60-72: M=2, N=4, K=3, alpha = beta = 1 on ones -> 4."""
    from mircuda_b200 import dense
    a = torch.ones(2, 3, dtype=torch.bfloat16, device="cuda")
    b = torch.ones(4, 3, dtype=torch.bfloat16, device="cuda")
    c = torch.ones(2, 4, dtype=torch.bfloat16, device="cuda")
    run_dense(cuda_stream, a, b, c, dense.DenseMatmulSpec(2, 4, 3), 1.0, 1.0)
    assert (c.float() == 4.0).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k,alpha,beta", [(256, 512, 1024, 1.0, 0.0), (300, 328, 200, 0.5, 0.25),
                                              (5, 1000, 64, 1.0, 0.0), (129, 264, 136, 1.0, 1.0)])
def test_dense_random(cuda_stream, dtype, m, n, k, alpha, beta):
    from mircuda_b200 import dense
    generator = torch.Generator(device="cuda").manual_seed(8100 + m)
    a = torch.randn(m, k, generator=generator, device="cuda").to(dtype)
    b = (torch.randn(n, k, generator=generator, device="cuda") * 0.05).to(dtype)
    c0 = torch.randn(m, n, generator=generator, device="cuda").to(dtype)
    expected = alpha * (a.double() @ b.double().T) + beta * c0.double()
    c = c0.clone()
    run_dense(cuda_stream, a, b, c, dense.DenseMatmulSpec(m, n, k, dtype), alpha, beta)
    assert_close(c, expected, f"dense {dtype} {m}x{n}x{k}")


def run_w4a16(stream, x, packed, scales, m, n, k):
    from mircuda_b200 import dense
    out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    plan = dense.W4A16Plan(stream, dense.W4A16Spec(m, n, k))
    torch.cuda.synchronize()
    for _ in range(2):
        plan.execute(stream, x.view(-1), packed.view(-1), scales.view(-1), out.view(-1))
    stream.synchronize()
    plan.close()
    return out


def assert_w4a16_matches_oracle(out, x, packed, scales, what):
    import oracle
    expected = oracle.w4a16_int4(x.cpu().numpy(), packed.cpu().numpy(), scales.cpu().numpy())
    assert_close(out, torch.from_numpy(expected.astype(np.float32)), what)


@pytest.fixture(params=["stream", "ring"])
def w4a16_kernel(request, monkeypatch):
    """Decode kernels behind mircuda_b200_w4a16_*: the persistent streaming kernel (n % 16 == 0,
    k % 2048 == 0, m <= 16; other shapes fall to the ring kernel) and the TMA-ring kernel."""
    monkeypatch.setenv("MIRCUDA_B200_W4A16", request.param)
    return request.param


@pytest.mark.parametrize("m,n,k", [(1, 512, 1024), (4, 1000, 512), (8, 200, 128), (16, 640, 2048),
                                   (9, 4096, 4096), (256, 512, 1024), (40, 264, 384),
                                   (1, 4096, 4096), (3, 2384, 2048), (8, 160, 6144), (12, 1024, 6144),
                                   (16, 48, 4096)])
def test_w4a16_random(cuda_stream, w4a16_kernel, m, n, k):
    """Device quantiser (bit-exact against the oracle's) and the product against the oracle's
    (q - 8) * scale restatement, sys/native/marlin/vendor/dequant.h:107-216."""
    import oracle
    from mircuda_b200 import dense
    generator = torch.Generator(device="cuda").manual_seed(8200 + m)
    weight = torch.randn(n, k, generator=generator, device="cuda") * 0.02
    packed, scales = dense.quantize_int4(weight)
    oracle_packed, oracle_scales = oracle.int4_g128_quantize(weight.cpu().numpy())
    assert np.array_equal(scales.cpu().numpy().view(np.uint16), oracle_scales.view(np.uint16))
    assert np.array_equal(packed.cpu().numpy(), oracle_packed)
    x = torch.randn(m, k, generator=generator, device="cuda").to(torch.float16)
    out = run_w4a16(cuda_stream, x, packed, scales, m, n, k)
    assert_w4a16_matches_oracle(out, x, packed, scales, f"w4a16 {m}x{n}x{k}")


@pytest.mark.parametrize("m", [1, 16, 256])
@pytest.mark.parametrize("n,k", [(14336, 4096), (4096, 14336)])
def test_w4a16_benchmark_shapes(cuda_stream, w4a16_kernel, m, n, k):
    """The Marlin-style W4A16 shapes the throughput is quoted on: K=4096 x N=14336 and
    K=14336 x N=4096, weights ~N(0, 0.02) quantised by the oracle (symmetric zero point 8,
    group 128, f16 scales = max|w|/7), f16 activations ~N(0, 1) at M in {1, 16, 256}."""
    import oracle
    rng = np.random.default_rng(4000 + n // 64 + m)
    weight = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    packed_host, scales_host = oracle.int4_g128_quantize(weight)
    x_host = rng.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    packed = torch.from_numpy(packed_host).cuda()
    scales = torch.from_numpy(scales_host).cuda()
    x = torch.from_numpy(x_host).cuda()
    out = run_w4a16(cuda_stream, x, packed, scales, m, n, k)
    expected = oracle.w4a16_int4(x_host, packed_host, scales_host)
    assert_close(out, torch.from_numpy(expected.astype(np.float32)), f"w4a16 {m}x{n}x{k}")


@pytest.mark.parametrize("prefill", ["fused", "single", "expand"])
@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (40, 264, 384), (17, 8, 128), (300, 1000, 2176),
                                   (128, 256, 128), (129, 776, 4096), (64, 264, 8192)])
def test_w4a16_prefill_kernels(cuda_stream, monkeypatch, prefill, m, n, k):
    """M > 16: the fused GEMM (packed weights expanded inside the kernel; CTA pairs above 128 tokens
    by default, single CTAs with `single`) and the two-launch form
    (expansion into an f16 workspace, then the dense GEMM), ragged in M and N, one and many scale
    groups along K, with and without K ranges met through fp32 partial sums (the last two
    shapes); both must produce the oracle's product."""
    monkeypatch.setenv("MIRCUDA_B200_W4A16_PREFILL", prefill)
    from mircuda_b200 import dense
    generator = torch.Generator(device="cuda").manual_seed(8300 + m)
    weight = torch.randn(n, k, generator=generator, device="cuda") * 0.02
    packed, scales = dense.quantize_int4(weight)
    x = torch.randn(m, k, generator=generator, device="cuda").to(torch.float16)
    out = run_w4a16(cuda_stream, x, packed, scales, m, n, k)
    assert_w4a16_matches_oracle(out, x, packed, scales, f"w4a16 {prefill} {m}x{n}x{k}")
    # other activations through a fresh plan (every plan runs twice: cached tensor maps)
    x2 = torch.randn(m, k, generator=generator, device="cuda").to(torch.float16)
    out2 = run_w4a16(cuda_stream, x2, packed, scales, m, n, k)
    assert_w4a16_matches_oracle(out2, x2, packed, scales, f"w4a16 {prefill} {m}x{n}x{k} (second)")


def test_w4a16_nibble_order(cuda_stream):
    """Only even-k codes differ from the zero point: exposes a swapped nibble order."""
    from mircuda_b200 import dense
    n, k = 128, 128
    packed = torch.full((n, k // 2), 0x89, dtype=torch.uint8, device="cuda")   # even k: +1, odd k: 0
    scales = torch.ones(n, 1, dtype=torch.float16, device="cuda")
    x = torch.arange(k, dtype=torch.float32, device="cuda").to(torch.float16).view(1, k)
    out = torch.zeros(1, n, dtype=torch.float16, device="cuda")
    plan = dense.W4A16Plan(cuda_stream, dense.W4A16Spec(1, n, k))
    torch.cuda.synchronize()
    plan.execute(cuda_stream, x.view(-1), packed.view(-1), scales.view(-1), out.view(-1))
    cuda_stream.synchronize()
    plan.close()
    assert (out.float() == float(sum(range(0, k, 2)))).all()


def test_fp8_vector_golden(cuda_stream):
    """blockwise_fp8_vector_produces_bf16 (tests/cutlass/fp8.rs:12-34): ones, unit scales -> 128."""
    from mircuda_b200 import dense
    n = k = 128
    x = torch.full((k,), 0x38, dtype=torch.uint8, device="cuda")
    w = torch.full((n * k,), 0x38, dtype=torch.uint8, device="cuda")
    ones = torch.ones(1, dtype=torch.float32, device="cuda")
    out = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    plan = dense.BlockwiseFp8VectorPlan(cuda_stream, dense.BlockwiseFp8VectorSpec(n, k))
    torch.cuda.synchronize()
    plan.execute(cuda_stream, x, ones, w, ones.clone(), out)
    cuda_stream.synchronize()
    plan.close()
    assert (out.float() == 128.0).all()


def test_fp8_vector_random(cuda_stream):
    import oracle
    from mircuda_b200 import dense
    n, k = 1152, 2048
    rng = np.random.default_rng(515)
    x = rng.integers(0, 256, size=k, dtype=np.uint8)
    w = rng.integers(0, 256, size=(n, k), dtype=np.uint8)
    x[(x & 0x7F) == 0x7F] = 0x38
    w[(w & 0x7F) == 0x7F] = 0x38
    sa = rng.uniform(0.5, 2.0, size=k // 128).astype(np.float32)
    sb = rng.uniform(0.01, 0.05, size=(k // 128, n // 128)).astype(np.float32)   # [block, n / 128]
    table = oracle.e4m3_table().astype(np.float64)
    products = (table[w].reshape(n, k // 128, 128) * table[x].reshape(1, k // 128, 128)).sum(axis=2)
    expected = (products * sa[None, :] * sb.T.repeat(128, axis=0)).sum(axis=1)
    out = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    plan = dense.BlockwiseFp8VectorPlan(cuda_stream, dense.BlockwiseFp8VectorSpec(n, k))
    torch.cuda.synchronize()
    plan.execute(cuda_stream, torch.from_numpy(x).cuda(), torch.from_numpy(sa).cuda(),
                 torch.from_numpy(w.reshape(-1)).cuda(), torch.from_numpy(sb.reshape(-1)).cuda(), out)
    cuda_stream.synchronize()
    plan.close()
    assert_close(out, torch.from_numpy(expected), "blockwise fp8 vector")


def _run_scaled_fp8(cuda_stream, m, n, k, x, w, sa, sb, bias, scale_dtype, tile=0):
    from mircuda_b200 import dense
    spec = dense.ScaledFp8Spec(m, k, n, scale_dtype, "tensor" if len(sb) == 1 else "output_channel",
                               bias is not None, tile)
    out = torch.zeros(m * n, dtype=torch.bfloat16, device="cuda")
    device_bias = None if bias is None else torch.from_numpy(bias.view(np.int16)).view(torch.bfloat16).cuda()
    device_sb = torch.from_numpy(sb).cuda().to(scale_dtype)
    operands = (torch.from_numpy(x.reshape(-1)).cuda(), torch.from_numpy(w.reshape(-1)).cuda(),
                torch.from_numpy(sa).cuda(), device_sb, device_bias, out)
    plan = dense.ScaledFp8Plan(cuda_stream, spec)
    assert plan.workspace_bytes() == 0
    torch.cuda.synchronize()
    execute = plan.execute_f32_scales if scale_dtype == torch.float32 else plan.execute_bf16_scales
    for _ in range(2):
        execute(cuda_stream, *operands)
    cuda_stream.synchronize()
    plan.close()
    return out.view(m, n), device_sb.float().cpu().numpy()


@pytest.mark.parametrize("tile", [0, 1])
def test_scaled_fp8_goldens(cuda_stream, tile):
    """tests/cutlass/scaled_fp8.rs:9-71: both of the reference's cases, bit for bit."""
    ones_x = np.full(16, 0x38, dtype=np.uint8)
    ones_w = np.full(256, 0x38, dtype=np.uint8)
    channel = np.arange(1, 17, dtype=np.float32) / 16.0
    import oracle
    bias = oracle.f32_to_bf16(np.ones(16, dtype=np.float32))
    out, _ = _run_scaled_fp8(cuda_stream, 1, 16, 16, ones_x, ones_w, np.float32([0.5]), channel, bias,
                             torch.float32, tile)
    assert (out.float().cpu().numpy().reshape(-1) == (8.0 * channel + 1.0).astype(np.float32)).all()
    out, _ = _run_scaled_fp8(cuda_stream, 1, 16, 16, ones_x, ones_w, np.float32([0.5]),
                             np.float32([0.25]), None, torch.float32, tile)
    assert (out.float() == 2.0).all()


@pytest.mark.parametrize("m,n,k,channel,with_bias,scale_dtype", [
    (1, 1024, 4096, True, True, torch.float32),
    (5, 48, 80, True, False, torch.bfloat16),         # ragged K (not a multiple of 64), small N
    (8, 2048, 1040, False, True, torch.float32),
    (13, 512, 2048, True, True, torch.bfloat16),      # second token half, partly filled
    (16, 1024, 4096, False, False, torch.float32),
    (17, 272, 144, True, True, torch.float32),        # tcgen05 path: ragged M, N, K tiles
    (200, 1024, 1024, True, True, torch.bfloat16),
    (512, 2048, 4096, False, False, torch.float32),
])
def test_scaled_fp8_random(cuda_stream, m, n, k, channel, with_bias, scale_dtype):
    import oracle
    rng = np.random.default_rng(m * 7919 + n + k)
    x = rng.integers(0, 256, size=(m, k), dtype=np.uint8)
    w = rng.integers(0, 256, size=(n, k), dtype=np.uint8)
    # No NaN codes, and magnitudes kept below 2^4 so that sums stay far inside fp32 / bf16 range.
    for codes in (x, w):
        codes[(codes & 0x7F) >= 0x60] &= 0x9F
    sa = rng.uniform(0.5, 2.0, size=m).astype(np.float32)
    sb = rng.uniform(0.01, 0.05, size=n if channel else 1).astype(np.float32)
    bias = oracle.f32_to_bf16(rng.normal(0, 2.0, size=n).astype(np.float32)) if with_bias else None
    out, used_sb = _run_scaled_fp8(cuda_stream, m, n, k, x, w, sa, sb, bias, scale_dtype)
    expected = oracle.scaled_fp8(x, w, sa, used_sb, bias, m, n, k)
    actual = out.view(torch.int16).cpu().numpy().view(np.uint16)
    stats = oracle.compare_bf16(actual, expected)
    assert stats["max_rel_to_max"] <= 1e-2 and stats["rel_frobenius"] <= 5e-3, stats
