"""GPU parity for the Marlin-layout NVFP4 dense projection (tokens <= 16), end to end through
the C ABI: canonical NVFP4 weights -> repack + scale preparation on the device -> execute,
compared with the oracle's dequantize-then-matmul. The reference ships no test that executes
this entry point; numerics follow sys/native/marlin/vendor/dense_template.h:1655-1658."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from oracle import marlin
from helpers import assert_close_bf16, bf16_bits, seeded_bf16, u8

pytestmark = pytest.mark.gpu


def pointer(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


@pytest.fixture(params=["stream", "tiles"])
def dense_kernel(request, monkeypatch):
    """Both kernels behind the entry point: the streaming one (default where N % 64 == 0 and
    K % 512 == 0) and the tile kernel (every other shape, or by environment variable)."""
    monkeypatch.setenv("MIRCUDA_B200_MARLIN_DENSE", request.param)
    return request.param


@pytest.mark.parametrize("tokens", [1, 8, 13, 16])
@pytest.mark.parametrize("n,k", [(4096, 4096), (128, 64), (6144, 1024), (24576, 2048), (192, 1104),
                                 (4096, 12288), (6144, 4096), (64, 512), (24576, 4096), (9472, 1536)])
def test_marlin_nvfp4_dense(cuda_stream, dense_kernel, tokens, n, k):
    if dense_kernel == "tiles" and n * k > 24576 * 2048:
        pytest.skip("the large shapes are there for the streaming kernel's K splits")
    from mircuda_b200 import _lib
    library = _lib.load()
    stream = ctypes.c_void_p(cuda_stream.cuda_stream)
    rng = np.random.default_rng(n + k)
    codes = rng.integers(0, 256, size=n * k // 2, dtype=np.uint8)
    scales = rng.integers(0x28, 0x48, size=n * k // 16, dtype=np.uint8)      # 2^-2 .. 4
    global_scale = np.array([0.013], dtype=np.float32)
    x = seeded_bf16((tokens, k), 1.0, 8000 + tokens)

    d_codes, d_scales = u8(codes), u8(scales)
    d_global = torch.from_numpy(global_scale).cuda()
    packed = torch.zeros(n * k // 2, dtype=torch.uint8, device="cuda")
    prepared = torch.zeros(n * k // 16, dtype=torch.uint8, device="cuda")
    prepared_global = torch.zeros(1, dtype=torch.float32, device="cuda")
    maximum = torch.zeros(1, dtype=torch.int32, device="cuda")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    temporary = torch.zeros(sms * 4096, dtype=torch.float32, device="cuda")
    locks = torch.zeros(sms, dtype=torch.int32, device="cuda")
    out = torch.full((tokens * n,), float("nan"), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    assert library.mircuda_marlin_nvfp4_repack(stream, pointer(d_codes), pointer(packed), 1, n, k) == 0
    assert library.mircuda_marlin_nvfp4_prepare_scales(
        stream, pointer(d_scales), None, pointer(d_global), pointer(prepared),
        pointer(prepared_global), pointer(maximum), 1, n, k) == 0
    # The streaming kernel may read the prepared weights before the kernel directly in front of
    # it on the stream has completed (the entry point's documented contract): finish preparing.
    cuda_stream.synchronize()
    for _ in range(2):                                   # twice: locks must return to zero
        assert library.mircuda_marlin_nvfp4_dense_execute(
            stream, pointer(x), pointer(packed), pointer(out), pointer(temporary), pointer(prepared),
            ctypes.cast(prepared_global.data_ptr(), ctypes.c_void_p), tokens, n, k, 0,
            pointer(locks), False) == 0
    cuda_stream.synchronize()
    assert not locks.any()

    expected_packed = marlin.repack(codes, 1, n, k)
    expected_codes, expected_globals, factor = marlin.nvfp4_scales(scales, None, global_scale, 1, n, k)
    assert np.array_equal(packed.cpu().numpy().view(np.uint32), expected_packed)
    assert np.array_equal(prepared.cpu().numpy(), expected_codes)
    weights = marlin.dequantize_packed_nvfp4(expected_packed, expected_codes, 1, n, k)[0]
    product = (oracle.bf16_to_f32(bf16_bits(x)).astype(np.float64) @ weights.T.astype(np.float64))
    product *= float(expected_globals[0]) * 2.0 ** -126
    expected = oracle.f32_to_bf16(product.astype(np.float32))
    assert_close_bf16(bf16_bits(out).reshape(tokens, n), expected, f"marlin dense {tokens}x{n}x{k}")
    # and the same answer as the plain dequantize-then-matmul on the canonical tensors
    plain = oracle.nvfp4_dequantize_rowmajor(codes.reshape(n, k // 2), scales.reshape(n, k // 16), k) \
        if hasattr(oracle, "nvfp4_dequantize_rowmajor") else None
    if plain is not None:
        reference = oracle.f32_to_bf16(
            ((oracle.bf16_to_f32(bf16_bits(x)) @ plain.T) * global_scale[0]).astype(np.float32))
        assert_close_bf16(bf16_bits(out).reshape(tokens, n), reference, "vs canonical tensors")
