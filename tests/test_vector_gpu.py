"""GPU parity for the decode paths: dense GEMV, FP4 x FP4 GEMV, bf16 x NVFP4 skinny GEMM,
NVFP4 quantizer and weight-only MXFP8 — through the C ABI, against the CPU oracle and, where
it was built, against the reference's own kernels compiled from its sources."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close_bf16, bf16_bits, from_bf16_bits, seeded_bf16, u8

pytestmark = pytest.mark.gpu


def random_fp4(rows, k, seed):
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 256, size=(rows, k // 2), dtype=np.uint8)
    scale_values = rng.integers(0x20, 0x48, size=(rows, k // 16), dtype=np.uint8)  # 2^-3 .. 4
    scales = np.zeros(oracle.fp4_scale_bytes(rows, k), dtype=np.uint8)
    scales[oracle.fp4_scale_offsets(rows, k)] = scale_values
    return codes, scales


# ------------------------------------------------------------------------------- dense GEMV

@pytest.mark.parametrize("n,k", [(4096, 4096), (37, 264), (100, 1000), (5, 7), (6144, 2560)])
@pytest.mark.parametrize("data_type", [0, 1])
def test_dense_vector(cuda_stream, n, k, data_type):
    from mircuda_b200 import plans
    dtype = torch.bfloat16 if data_type else torch.float16
    generator = torch.Generator().manual_seed(n * 7 + k)
    x = torch.randn(k, generator=generator).to(dtype).cuda()
    w = (torch.randn(n, k, generator=generator) * 0.02).to(dtype).cuda()
    y = torch.randn(n, generator=generator).to(dtype).cuda()
    expected_input = y.clone()
    plan = plans.DenseVectorPlan(cuda_stream, plans.DenseVectorSpec(n, k, data_type))
    torch.cuda.synchronize()
    plan.execute(cuda_stream, x, w.view(-1), y, alpha=1.5, beta=0.25)
    cuda_stream.synchronize()
    view = torch.int16
    expected = oracle.dense_vector(
        data_type, x.view(view).cpu().numpy().view(np.uint16), w.view(view).cpu().numpy().view(np.uint16),
        expected_input.view(view).cpu().numpy().view(np.uint16), n, k, 1.5, 0.25)
    actual = y.view(view).cpu().numpy().view(np.uint16)
    if data_type:
        assert_close_bf16(actual, expected, f"dense bf16 {n}x{k}")
    else:
        a = actual.view(np.float16).astype(np.float64)
        e = expected.view(np.float16).astype(np.float64)
        assert np.max(np.abs(a - e)) <= 1e-2 * np.max(np.abs(e))
    path = oracle.ref_library("vector")
    if path is not None:
        # The reference's own kernel (sys/native/dense_vector_sm120.cu:147-175, compiled from
        # its source for sm_100a), same inputs, through its own entry points.
        library = ctypes.CDLL(str(path))
        raw = ctypes.c_void_p()
        stream = ctypes.c_void_p(cuda_stream.cuda_stream)
        assert library.mircuda_dense_vector_create(data_type, n, k, stream, ctypes.byref(raw)) == 0
        reference_y = expected_input.clone()
        torch.cuda.synchronize()
        library.mircuda_dense_vector_execute.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_float] * 2
        assert library.mircuda_dense_vector_execute(
            raw, stream, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
            ctypes.c_void_p(reference_y.data_ptr()), ctypes.c_float(1.5), ctypes.c_float(0.25)) == 0
        cuda_stream.synchronize()
        library.mircuda_dense_vector_destroy.argtypes = [ctypes.c_void_p]
        library.mircuda_dense_vector_destroy(raw)
        reference_bits = reference_y.view(view).cpu().numpy().view(np.uint16)
        # pins the restatement (different summation order, so a tolerance) and this library
        if data_type:
            assert_close_bf16(expected, reference_bits, f"oracle vs reference dense kernel {n}x{k}")
            assert_close_bf16(actual, reference_bits, f"dense bf16 vs reference kernel {n}x{k}")
        else:
            r = reference_bits.view(np.float16).astype(np.float64)
            e = expected.view(np.float16).astype(np.float64)
            assert np.max(np.abs(e - r)) <= 1e-2 * np.max(np.abs(r))
            assert np.max(np.abs(a - r)) <= 1e-2 * np.max(np.abs(r))
    # beta = 0 must not read the output (NaN-prefilled, reference idiom tests/cutlass/grouped/bf16.rs:28)
    y2 = torch.full((n,), float("nan"), dtype=dtype, device="cuda")
    torch.cuda.synchronize()
    plan.execute(cuda_stream, x, w.view(-1), y2, alpha=1.0, beta=0.0)
    cuda_stream.synchronize()
    assert not torch.isnan(y2).any()
    plan.close()


# --------------------------------------------------------------------------- FP4 x FP4 GEMV

def run_fp4_vector(stream, x, xs, w, ws, n, k, alpha):
    from mircuda_b200 import plans
    plan = plans.BlockScaledFp4VectorPlan(stream, plans.BlockScaledFp4VectorSpec(n, k))
    args = [u8(x.reshape(-1)), u8(xs), u8(w.reshape(-1)), u8(ws)]
    out = torch.full((n,), float("nan"), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    for _ in range(2):                     # twice: the cross-slice counters must reset themselves
        plan.execute(stream, *args, out, alpha)
    stream.synchronize()
    plan.close()
    return bf16_bits(out)


@pytest.fixture(params=["stream", "tensor", "simt"])
def fp4_vector_kernel(request, monkeypatch):
    """The implementations behind mircuda_fp4_vector_*: the persistent streaming kernel (default
    where n % 128 == 0 and k % 2048 == 0; other shapes fall to the two below), the tcgen05 kernel
    (large weights) and the CUDA-core kernel; the override is read when a plan is created."""
    monkeypatch.setenv("MIRCUDA_B200_FP4_VECTOR", request.param)
    return request.param


def test_fp4_vector_golden(cuda_stream, fp4_vector_kernel):
    """tests/cutlass/fp4/vector.rs:11-30 — all 0x22 / 0x38, N=704, K=2816 -> 2816.0."""
    n, k = 704, 2816
    x = np.full(k // 2, 0x22, np.uint8)
    xs = np.full(oracle.fp4_scale_bytes(1, k), 0x38, np.uint8)
    w = np.full((n, k // 2), 0x22, np.uint8)
    ws = np.full(oracle.fp4_scale_bytes(n, k), 0x38, np.uint8)
    out = run_fp4_vector(cuda_stream, x, xs, w, ws, n, k, 1.0)
    assert (oracle.bf16_to_f32(out) == 2816.0).all()


@pytest.mark.parametrize("n,k", [(4096, 4096), (200, 448), (129, 64), (2048, 2816), (24576, 4096),
                                 (4096, 12288), (128, 192), (6144, 4096), (256, 2048), (1152, 6144)])
def test_fp4_vector_random(cuda_stream, fp4_vector_kernel, n, k):
    x, xs = random_fp4(1, k, 11)
    w, ws = random_fp4(n, k, 12)
    expected = oracle.fp4_vector(x, xs, w, ws, n, k, 0.5)
    actual = run_fp4_vector(cuda_stream, x, xs, w, ws, n, k, 0.5)
    assert_close_bf16(actual, expected, f"fp4 vector {n}x{k}")
    path = oracle.ref_library("vector")
    if path is not None:                   # the reference's own kernel, same inputs
        library = ctypes.CDLL(str(path))
        raw = ctypes.c_void_p()
        stream = ctypes.c_void_p(cuda_stream.cuda_stream)
        assert library.mircuda_fp4_vector_create(n, k, stream, ctypes.byref(raw)) == 0
        tensors = [u8(x.reshape(-1)), u8(xs), u8(w.reshape(-1)), u8(ws)]
        out = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        library.mircuda_fp4_vector_execute.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_float]
        assert library.mircuda_fp4_vector_execute(
            raw, stream, *[ctypes.c_void_p(t.data_ptr()) for t in tensors],
            ctypes.c_void_p(out.data_ptr()), ctypes.c_float(0.5)) == 0
        cuda_stream.synchronize()
        library.mircuda_fp4_vector_destroy.argtypes = [ctypes.c_void_p]
        library.mircuda_fp4_vector_destroy(raw)
        assert_close_bf16(actual, bf16_bits(out), f"fp4 vector vs reference kernel {n}x{k}")


# ------------------------------------------------------------------ bf16 x NVFP4 skinny GEMM

@pytest.fixture(params=["stream", "ring", "direct"])
def nvfp4_vector_kernel(request, monkeypatch):
    """The kernels behind mircuda_b200_nvfp4_vector_*: the persistent streaming kernel (shapes
    with whole 128-row scale tiles and K a multiple of 2048; other shapes fall to the direct
    kernel), weights through a TMA-fed shared-memory ring, or loaded straight from global
    memory; the choice is read when a plan is created."""
    monkeypatch.setenv("MIRCUDA_B200_NVFP4_VECTOR", request.param)
    return request.param


@pytest.mark.parametrize("m,n,k", [
    (m, n, k) for n, k in [(4096, 4096), (200, 448), (129, 64), (6144, 1024)] for m in [1, 4, 8, 3]
] + [
    # Shapes whose row tiles are shared between CTAs in every way: a CTA's share of the
    # units starts and ends inside tiles, and covers whole tiles in between.
    (8, 24576, 4096), (1, 24576, 4096), (8, 4096, 12288), (2, 12160, 2112),
    # Every form of the streaming kernel: one CTA per tile (K = 2048, 6144) or a CTA pair
    # (K = 4096, 8192, 12288), one to three K chunks per warp, fewer tiles than CTA pairs,
    # an odd and an even number of tiles per pair, the four benchmark shapes.
    (1, 256, 2048), (5, 6144, 6144), (8, 128, 8192), (1, 4096, 12288), (4, 6144, 4096),
    (2, 2432, 4096), (7, 1152, 8192),
])
def test_nvfp4_vector_random(cuda_stream, nvfp4_vector_kernel, m, n, k):
    from mircuda_b200 import plans
    w, ws = random_fp4(n, k, 21)
    x = seeded_bf16((m, k), 1.0, 3000 + m)
    global_scale = 0.37
    expected = oracle.nvfp4_gemv_bf16(bf16_bits(x), w, ws, n, k, global_scale)
    plan = plans.NvFp4VectorPlan(cuda_stream, plans.NvFp4VectorSpec(m, n, k))
    wd, wsd = u8(w.reshape(-1)), u8(ws)
    out = torch.full((m * n,), float("nan"), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    for _ in range(2):
        plan.execute(cuda_stream, x.view(-1), wd, wsd, out, global_scale)
    cuda_stream.synchronize()
    plan.close()
    assert_close_bf16(bf16_bits(out).reshape(m, n), expected, f"nvfp4 vector m={m} {n}x{k}")


def test_nvfp4_vector_nibble_order(cuda_stream, nvfp4_vector_kernel):
    """Asymmetric pattern: only even-k codes are non-zero, activations differ per k."""
    from mircuda_b200 import plans
    n, k = 128, 64
    w = np.zeros((n, k // 2), np.uint8)
    w[:, :] = 0x02                                      # even k = 1.0 (low nibble), odd k = 0
    ws = np.zeros(oracle.fp4_scale_bytes(n, k), np.uint8)
    ws[oracle.fp4_scale_offsets(n, k)] = 0x38
    x = torch.arange(k, dtype=torch.float32).to(torch.bfloat16).cuda().view(1, k)
    plan = plans.NvFp4VectorPlan(cuda_stream, plans.NvFp4VectorSpec(1, n, k))
    out = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    plan.execute(cuda_stream, x.view(-1), u8(w.reshape(-1)), u8(ws), out, 1.0)
    cuda_stream.synchronize()
    assert (out.float() == float(sum(range(0, k, 2)))).all()
    plan.close()


# ------------------------------------------------------------------------- NVFP4 quantizer

@pytest.mark.parametrize("rows,k,std", [(128, 1024, 0.02), (5, 64, 1.0), (300, 448, 3.0)])
def test_nvfp4_quantizer_bit_exact(cuda_stream, rows, k, std):
    from mircuda_b200 import plans
    values = seeded_bf16((rows, k), std, 4000 + rows)
    torch.cuda.synchronize()
    codes, scales, global_scale = plans.nvfp4_quantize_bf16(cuda_stream, values)
    cuda_stream.synchronize()
    expected_codes, expected_scales, expected_global = oracle.nvfp4_quantize(bf16_bits(values))
    assert np.float32(global_scale.item()) == np.float32(expected_global)
    assert np.array_equal(scales.cpu().numpy(), expected_scales)
    assert np.array_equal(codes.cpu().numpy(), expected_codes)


def test_nvfp4_quantizer_zero_tensor(cuda_stream):
    from mircuda_b200 import plans
    values = torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    codes, scales, global_scale = plans.nvfp4_quantize_bf16(cuda_stream, values)
    cuda_stream.synchronize()
    assert global_scale.item() == 1.0 and not codes.any() and not scales.any()


# --------------------------------------------------------------------- weight-only MXFP8

def test_weight_only_golden(cuda_stream):
    """tests/mxfp8/matmul.rs:7-33."""
    from mircuda_b200 import plans
    x = torch.tensor([[float(t)] * 32 for t in range(1, 6)], dtype=torch.bfloat16, device="cuda")
    words = torch.tensor([0x38383838] * 8 + [0xB0B0B0B0 - (1 << 32)] * 8, dtype=torch.int32, device="cuda")
    scales = torch.tensor([127, 128], dtype=torch.uint8, device="cuda")
    out = torch.zeros(10, dtype=torch.bfloat16, device="cuda")
    operation = plans.MxFp8Matmul(plans.MxFp8Spec(5, 32, 2))
    torch.cuda.synchronize()
    operation.execute(cuda_stream, x.view(-1), words, scales, out)
    cuda_stream.synchronize()
    expected = [v for t in range(1, 6) for v in (32.0 * t, -32.0 * t)]
    assert out.float().cpu().tolist() == expected


@pytest.mark.parametrize("tokens,k,n", [(1, 4096, 512), (5, 1024, 300), (3, 96, 17), (5, 1024, 304), (8, 4096, 64),
                                        (3, 128, 16), (2, 12288, 256), (9, 1024, 64), (7, 1152, 48), (2, 1024, 64),
                                        (1, 12288, 32)])
def test_weight_only_random(cuda_stream, tokens, k, n):
    from mircuda_b200 import plans
    w = seeded_bf16((n, k), 0.02, 5000)
    codes, swizzled = oracle.mxfp8_quantize(bf16_bits(w))
    row_major = swizzled[oracle.scale_offsets(n, k // 32)]
    x = seeded_bf16((tokens, k), 1.0, 5001)
    expected = oracle.mxfp8_bf16_matmul(bf16_bits(x), codes.view(np.uint32), row_major)
    out = torch.zeros(tokens * n, dtype=torch.bfloat16, device="cuda")
    operation = plans.MxFp8Matmul(plans.MxFp8Spec(tokens, k, n))
    cd, sd = u8(codes.reshape(-1)), u8(row_major.reshape(-1))
    torch.cuda.synchronize()
    operation.execute(cuda_stream, x.view(-1), cd, sd, out)
    cuda_stream.synchronize()
    assert_close_bf16(bf16_bits(out), expected.reshape(-1), f"weight-only {tokens}x{k}x{n}")
    path = oracle.ref_library("device")
    if path is not None:
        library = ctypes.CDLL(str(path))
        ref_out = torch.zeros(tokens * n, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        assert library.ref_mxfp8_bf16(
            ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(cd.data_ptr()), ctypes.c_void_p(sd.data_ptr()),
            ctypes.c_void_p(ref_out.data_ptr()), ctypes.c_uint32(tokens), ctypes.c_uint32(k),
            ctypes.c_uint32(n), ctypes.c_int(0), ctypes.c_void_p(cuda_stream.cuda_stream)) == 0
        cuda_stream.synchronize()
        assert_close_bf16(bf16_bits(out), bf16_bits(ref_out), "weight-only vs reference kernel")
