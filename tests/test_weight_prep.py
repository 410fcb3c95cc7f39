"""Prepared-weight container (CPU) and the preparation itself (GPU): a prepared file holds the
same bytes the library's entry points produce when called directly, survives a save / load
round trip bit for bit, and dequantises back to the weights within the format's step."""
import struct

import numpy as np
import pytest
import torch


def _sample():
    from mircuda_b200 import weight_prep
    generator = torch.Generator().manual_seed(5)
    first = weight_prep.PreparedWeight("int4_g128", 8, 256, {
        "codes": torch.randint(0, 256, (8, 128), dtype=torch.uint8, generator=generator),
        "scales": torch.rand(8, 2, generator=generator).to(torch.float16)})
    second = weight_prep.PreparedWeight("int4_g128", 16, 128, {
        "codes": torch.randint(0, 256, (16, 64), dtype=torch.uint8, generator=generator),
        "scales": torch.rand(16, 1, generator=generator).to(torch.float16)})
    return {"layers.0.q": first, "layers.0.k": second}


def test_container_round_trip(tmp_path):
    from mircuda_b200 import weight_prep
    weights = _sample()
    path = tmp_path / "w.mirw"
    weight_prep.save(path, weights)
    loaded = weight_prep.load(path)
    assert list(loaded) == list(weights)
    for name, prepared in weights.items():
        assert (loaded[name].format, loaded[name].n, loaded[name].k) == (prepared.format, prepared.n, prepared.k)
        for part, tensor in prepared.tensors.items():
            assert loaded[name].tensors[part].dtype == tensor.dtype
            assert torch.equal(loaded[name].tensors[part], tensor)


def test_container_refuses_unknown_layouts(tmp_path):
    from mircuda_b200 import weight_prep
    path = tmp_path / "w.mirw"
    weight_prep.save(path, _sample())
    raw = bytearray(path.read_bytes())
    assert raw[:8] == weight_prep.MAGIC
    newer = bytearray(raw)
    newer[8:12] = struct.pack("<I", weight_prep.LAYOUT_VERSION + 1)
    (tmp_path / "newer.mirw").write_bytes(newer)
    with pytest.raises(weight_prep.UnknownLayout):
        weight_prep.load(tmp_path / "newer.mirw")
    (tmp_path / "other.mirw").write_bytes(b"something else entirely")
    with pytest.raises(weight_prep.UnknownLayout):
        weight_prep.load(tmp_path / "other.mirw")
    (tmp_path / "short.mirw").write_bytes(raw[:len(raw) - 64])
    with pytest.raises(weight_prep.UnknownLayout):
        weight_prep.load(tmp_path / "short.mirw")
    mixed = _sample()
    mixed["layers.0.k"].format = "nvfp4"
    with pytest.raises(ValueError):
        weight_prep.save(tmp_path / "mixed.mirw", mixed)


def _weight(n, k, seed):
    generator = torch.Generator().manual_seed(seed)
    return (torch.randn(n, k, generator=generator) * 0.05).to(torch.bfloat16).cuda()


@pytest.mark.gpu
def test_prepare_mxfp8_and_nvfp4_match_the_oracle(cuda_stream, tmp_path):
    import oracle
    from helpers import bf16_bits
    from mircuda_b200 import weight_prep
    n, k = 256, 512
    weight = _weight(n, k, 21)
    prepared = weight_prep.prepare(cuda_stream, weight, "mxfp8")
    codes, scales = oracle.mxfp8_quantize(bf16_bits(weight))
    assert np.array_equal(prepared.tensors["codes"].cpu().numpy(), codes.reshape(n, k))
    assert np.array_equal(prepared.tensors["scales"].cpu().numpy(), scales)

    prepared = weight_prep.prepare(cuda_stream, weight, "nvfp4")
    codes, scales, global_scale = oracle.nvfp4_quantize(bf16_bits(weight))
    assert np.array_equal(prepared.tensors["codes"].cpu().numpy().reshape(-1), codes.reshape(-1))
    assert np.array_equal(prepared.tensors["scales"].cpu().numpy(), scales)
    assert float(prepared.tensors["global_scale"].item()) == float(global_scale)
    path = tmp_path / "nvfp4.mirw"
    weight_prep.save(path, {"w": prepared})
    loaded = weight_prep.load(path, "cuda")["w"]
    for part, tensor in prepared.tensors.items():
        assert torch.equal(loaded.tensors[part], tensor)
    restored = oracle.nvfp4_dequantize(codes, scales, k) * global_scale
    original = weight.float().cpu().numpy()
    assert np.linalg.norm(restored - original) <= 0.12 * np.linalg.norm(original)


@pytest.mark.gpu
@pytest.mark.parametrize("tokens", [1, 8])
def test_prepared_marlin_weights_run(cuda_stream, tokens):
    """The Marlin file's tiles, scales and global feed mircuda_marlin_nvfp4_dense_execute and
    give the product of the activations with the dequantised NVFP4 weights."""
    import ctypes

    import oracle
    from helpers import assert_close_bf16, bf16_bits, seeded_bf16
    from mircuda_b200 import _lib, weight_prep
    n, k = 256, 512
    weight = _weight(n, k, 22)
    prepared = weight_prep.prepare(cuda_stream, weight, "marlin_nvfp4")
    plain = weight_prep.prepare(cuda_stream, weight, "nvfp4")
    x = seeded_bf16((tokens, k), 1.0, 99 + tokens)
    library = _lib.load()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    temporary = torch.zeros(sms * 4096, dtype=torch.float32, device="cuda")
    locks = torch.zeros(sms, dtype=torch.int32, device="cuda")
    out = torch.full((tokens * n,), float("nan"), dtype=torch.bfloat16, device="cuda")
    pointer = lambda tensor: ctypes.c_void_p(tensor.data_ptr())
    torch.cuda.synchronize()
    assert library.mircuda_marlin_nvfp4_dense_execute(
        ctypes.c_void_p(cuda_stream.cuda_stream), pointer(x), pointer(prepared.tensors["tiles"]),
        pointer(out), pointer(temporary), pointer(prepared.tensors["scales"]),
        pointer(prepared.tensors["global_scale"]), tokens, n, k, 0, pointer(locks), False) == 0
    cuda_stream.synchronize()
    weights = oracle.nvfp4_dequantize(plain.tensors["codes"].cpu().numpy(),
                                      plain.tensors["scales"].cpu().numpy(), k)
    product = oracle.bf16_to_f32(bf16_bits(x)).astype(np.float64) @ weights.T.astype(np.float64)
    product *= float(plain.tensors["global_scale"].item())
    assert_close_bf16(bf16_bits(out).reshape(tokens, n), oracle.f32_to_bf16(product.astype(np.float32)),
                      "prepared marlin weights")


@pytest.mark.gpu
def test_prepare_int4_runs_through_the_w4a16_plan(cuda_stream):
    from mircuda_b200 import dense, weight_prep
    n, k = 256, 512
    weight = _weight(n, k, 23)
    prepared = weight_prep.prepare(cuda_stream, weight, "int4_g128")
    packed, scales = dense.quantize_int4(weight)
    assert torch.equal(prepared.tensors["codes"], packed) and torch.equal(prepared.tensors["scales"], scales)
    with pytest.raises(Exception):
        weight_prep.prepare(cuda_stream, weight[:, :100], "int4_g128")
