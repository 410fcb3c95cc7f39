"""GPU parity for the routed weight-only MXFP8 projection and the MXFP8 embedding lookup."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close_bf16, bf16_bits, seeded_bf16, u8

pytestmark = pytest.mark.gpu


def bf16(value):
    return int(oracle.f32_to_bf16(np.array([value], dtype=np.float32))[0])


def pointer(tensor):
    return ctypes.c_void_p(tensor.data_ptr()) if tensor is not None else None


def gathered(stream, x, words, scales, bias, selected, matrices, rows, columns, per_input):
    from mircuda_b200 import _lib
    library = _lib.load()
    assignments = len(selected)
    d = dict(x=torch.from_numpy(x.view(np.int16)).cuda().view(torch.bfloat16),
             w=torch.from_numpy(words.view(np.int32)).cuda(), s=u8(scales),
             b=None if bias is None else torch.from_numpy(bias.view(np.int16)).cuda().view(torch.bfloat16),
             sel=torch.from_numpy(np.asarray(selected, np.uint32).view(np.int32)).cuda())
    out = torch.full((assignments * rows,), float("nan"), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    assert library.mircuda_b200_mxfp8_bf16_gathered(
        pointer(d["x"]), pointer(d["w"]), pointer(d["s"]), pointer(d["b"]), pointer(d["sel"]),
        pointer(out), assignments, matrices, rows, columns, per_input,
        ctypes.c_void_p(stream.cuda_stream)) == 0
    stream.synchronize()
    return bf16_bits(out).reshape(assignments, rows)


def test_gathered_golden(cuda_stream):
    """tests/mxfp8/gathered.rs:5-69: two matrices of two rows, one input row routed to both."""
    x = np.full((1, 32), bf16(1.0), dtype=np.uint16)
    words = np.array([0x38383838] * 8 + [0xB0B0B0B0] * 8 + [0x38383838] * 8 + [0xB0B0B0B0] * 8,
                     dtype=np.uint32)
    scales = np.array([127, 127, 128, 128], dtype=np.uint8)
    bias = np.array([bf16(v) for v in (1.0, 2.0, 3.0, 4.0)], dtype=np.uint16)
    plain = gathered(cuda_stream, x, words, scales, None, [1, 0], 2, 2, 32, 2)
    assert plain.reshape(-1).tolist() == [bf16(v) for v in (64.0, -32.0, 32.0, -16.0)]
    biased = gathered(cuda_stream, x, words, scales, bias, [1, 0], 2, 2, 32, 2)
    assert biased.reshape(-1).tolist() == [bf16(v) for v in (67.0, -28.0, 33.0, -14.0)]
    skipped = gathered(cuda_stream, x, words, scales, None, [5, 0], 2, 2, 32, 2)
    assert skipped[0].tolist() == [0, 0]


@pytest.mark.parametrize("inputs,per_input,matrices,rows,columns", [(3, 4, 6, 96, 512), (1, 8, 16, 200, 2048),
                                                                    (5, 1, 2, 33, 96)])
def test_gathered_random(cuda_stream, inputs, per_input, matrices, rows, columns):
    rng = np.random.default_rng(900 + rows)
    x = bf16_bits(seeded_bf16((inputs, columns), 1.0, 9000 + rows))
    codes = rng.integers(0, 256, size=(matrices * rows, columns), dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x38                      # no NaN codes
    scales = rng.integers(120, 132, size=matrices * rows * columns // 32, dtype=np.uint8)
    bias = bf16_bits(seeded_bf16((matrices * rows,), 1.0, 9100))
    selected = rng.integers(0, matrices, size=inputs * per_input).astype(np.uint32)
    selected[0] = matrices + 3
    words = codes.reshape(-1).view(np.uint32)
    expected = oracle.mxfp8_bf16_gathered(x, words, scales, bias, selected, matrices, rows, columns, per_input)
    actual = gathered(cuda_stream, x, words, scales, bias, selected, matrices, rows, columns, per_input)
    assert (actual[0] == 0).all()
    assert_close_bf16(actual, expected, f"gathered {inputs}x{per_input} {rows}x{columns}")


def embedding(stream, words, scales, selected, start, tokens, vocab, hidden, output_scale, fill):
    from mircuda_b200 import _lib
    library = _lib.load()
    d_words = torch.from_numpy(words.view(np.int32)).cuda()
    d_selected = torch.from_numpy(np.asarray(selected, np.uint32).view(np.int32)).cuda()
    d_scales = u8(scales)
    out = torch.full((tokens * hidden,), fill, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    assert library.mircuda_b200_mxfp8_embedding_bf16(
        pointer(d_words), pointer(d_scales), pointer(d_selected), pointer(out), start, tokens, vocab,
        hidden, ctypes.c_float(output_scale), ctypes.c_void_p(stream.cuda_stream)) == 0
    stream.synchronize()
    return bf16_bits(out).reshape(tokens, hidden)


def test_embedding_golden(cuda_stream):
    """tests/mxfp8/quantize.rs:48-79: rows selected [1, 0] -> -1.0 then 1.0."""
    words = np.array([0x38383838] * 8 + [0xB0B0B0B0] * 8, dtype=np.uint32)
    scales = np.array([127, 128], dtype=np.uint8)
    result = embedding(cuda_stream, words, scales, [1, 0], 0, 2, 2, 32, 1.0, 0.0)
    assert (result[0] == bf16(-1.0)).all() and (result[1] == bf16(1.0)).all()


def test_embedding_random_bit_exact(cuda_stream):
    rng = np.random.default_rng(77)
    vocab, hidden, tokens, start = 300, 1024, 37, 5
    codes = rng.integers(0, 256, size=(vocab, hidden), dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x38
    scales = rng.integers(110, 140, size=vocab * hidden // 32, dtype=np.uint8)
    selected = rng.integers(0, vocab, size=start + tokens).astype(np.uint32)
    selected[start + 3] = vocab + 9                           # left untouched
    words = codes.reshape(-1).view(np.uint32)
    before = np.full((tokens, hidden), bf16(7.0), dtype=np.uint16)
    expected = oracle.mxfp8_embedding(words, scales, selected, start, tokens, vocab, hidden, 0.37,
                                      output=before.copy())
    actual = embedding(cuda_stream, words, scales, selected, start, tokens, vocab, hidden, 0.37, 7.0)
    assert np.array_equal(actual, expected)
