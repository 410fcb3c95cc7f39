"""The numpy restatement of the Marlin layouts against independent scalar loops that follow
the host references in the reference's tests line by line. No GPU needed."""
import numpy as np

from oracle import marlin

EXPERTS, N, K = 2, 64, 64


def canonical_weights():
    raw = np.zeros(EXPERTS * N * K // 2, dtype=np.uint8)
    for expert in range(EXPERTS):
        for n in range(N):
            for k in range(0, K, 2):
                low = (expert * 7 + n * 3 + k) & 15
                high = (expert * 7 + n * 3 + k + 1) & 15
                raw[expert * N * K // 2 + n * K // 2 + k // 2] = low | high << 4
    return raw


def scalar_repack(raw, padded_n, padded_k, interleaved):
    """tests/marlin/padded.rs:127-161 with source_row from :194-203 (identity when not
    interleaved)."""
    def source_row(n):
        if not interleaved:
            return n if n < N else None
        physical, logical = padded_n // 2, N // 2
        unit, up = (n, 0) if n < physical else (n - physical, 1)
        return unit * 2 + up if unit < logical else None

    def value(expert, n, k):
        row = source_row(n)
        if row is None or k >= K:
            return 0
        return (int(raw[(expert * N + row) * (K // 2) + k // 2]) >> ((k & 1) * 4)) & 15

    tiles_n, tiles_k = padded_n // 64, padded_k // 16
    output = np.zeros(EXPERTS * tiles_n * tiles_k * 128, dtype=np.uint32)
    for expert in range(EXPERTS):
        for tile_k in range(tiles_k):
            for tile_n in range(tiles_n):
                for lane in range(32):
                    for warp in range(4):
                        n = tile_n * 64 + warp * 16 + lane // 4
                        k = tile_k * 16 + (lane % 4) * 2
                        values = [value(expert, n, k), value(expert, n, k + 1), value(expert, n, k + 8),
                                  value(expert, n, k + 9), value(expert, n + 8, k), value(expert, n + 8, k + 1),
                                  value(expert, n + 8, k + 8), value(expert, n + 8, k + 9)]
                        packed = 0
                        for shift, index in enumerate([0, 2, 4, 6, 1, 3, 5, 7]):
                            packed |= values[index] << (shift * 4)
                        tile = (expert * tiles_k + tile_k) * tiles_n + tile_n
                        output[tile * 128 + lane * 4 + warp] = packed
    return output


def test_repack_matches_scalar_reference():
    raw = canonical_weights()
    assert np.array_equal(marlin.repack(raw, EXPERTS, N, K), scalar_repack(raw, N, K, False))
    assert np.array_equal(marlin.repack(raw, EXPERTS, N, K, N, K, interleaved=True),
                          scalar_repack(raw, N, K, True))
    assert np.array_equal(marlin.repack(raw, EXPERTS, 128, 128, N, K, interleaved=True),
                          scalar_repack(raw, 128, 128, True))


def test_scale_destination_is_a_permutation_of_each_64_run():
    destination = marlin.scale_destination(np.arange(192))
    for chunk in range(3):
        assert sorted(destination[chunk * 64:(chunk + 1) * 64].tolist()) == list(range(chunk * 64, chunk * 64 + 64))
    # one thread's eight scales (rows g, g+8 of four 16-row quarters) are eight adjacent bytes
    for g in range(8):
        rows = [16 * w + g + 8 * h for w in range(4) for h in range(2)]
        assert sorted(marlin.scale_destination(np.array(rows)).tolist()) == list(range(8 * g, 8 * g + 8))


def test_packed_dequantize_round_trip():
    rng = np.random.default_rng(0)
    experts, n, k = 2, 128, 64
    raw = rng.integers(0, 256, experts * n * k // 2, dtype=np.uint8)
    scales = rng.integers(0x30, 0x48, experts * n * k // 16, dtype=np.uint8)
    globals_ = np.ones(experts, dtype=np.float32)
    packed = marlin.repack(raw, experts, n, k)
    codes, out_globals, factor = marlin.nvfp4_scales(scales, None, globals_, experts, n, k)
    restored = marlin.dequantize_packed_nvfp4(packed, codes, experts, n, k)
    import oracle
    nibbles = marlin.unpack_nibbles(raw, experts, n, k)
    expected = oracle.e2m1_table()[nibbles] * np.repeat(
        oracle.e4m3_table()[scales.reshape(experts, n, k // 16)], 16, axis=2)
    assert np.allclose(restored, expected * factor * 128.0)
    assert np.allclose(out_globals, 2.0 ** 119 / factor)


def test_routes_reference():
    selected = np.array([1, 0, 1, 1, 5, 0], dtype=np.uint32)
    sorted_rows, expert_ids, total, offsets = marlin.routes(selected, 3, 2)
    assert offsets.tolist() == [0, 2, 6] and total == 6
    assert sorted_rows[:6].tolist() == [1, 5, 0, 2, 3, 6]          # 6 = padding marker
    assert expert_ids[:3].tolist() == [0, 1, 1]
