"""CSF packed block-scale storage: the reference's own host tests, restated.

crates/cuda-kernels/tests/csf_scale_storage.rs (codec cases at :17-61, vector cases at
:258-312, decode helper `decode_one_six` at :392-407).
"""
import numpy as np
import pytest

from oracle import oracle as o


def _decode_one_six(p, rows, k, row, kg):
    tiles = (rows + 127) // 128 * (k // 128)
    stride = len(p) // tiles
    nbytes = (stride - 768) // 128
    t = row // 128 * (k // 128) + kg // 8
    r = row % 128
    at = t * stride + (r // 16) * 96 + (r % 8) * 12 + (r % 16 // 8) * 3 + (kg % 8 // 4) * 6
    word = int(p[at]) | (int(p[at + 1]) << 8) | (int(p[at + 2]) << 16)
    q = (word >> ((kg % 4) * 6)) & 63
    at = t * stride + 768 + r * nbytes
    if nbytes == 1:
        return q | (((int(p[at]) >> (kg % 8)) & 1) << 6)
    return q | (((int(p[at + kg % 8 // 4]) >> ((kg % 4) * 2)) & 3) << 6)


@pytest.mark.parametrize("rows,k", [(128, 128), (129, 256), (256, 2048)])
def test_matrix_codec_exact(rows, k):
    groups = k // 16
    logical = np.zeros(rows * groups, np.uint8)
    for i in range(rows * groups):
        row, col = divmod(i, groups)
        m = row % 5
        if m == 0:
            v = 32 + col % 8
        elif m == 1:
            v = 47 if col % 8 == 7 else 32
        elif m == 2:
            v = 48 if col % 8 == 7 else 32
        elif m == 3:
            v = (row + col * 37) % 256
        else:
            v = 0
        logical[i] = v
    enc = o.csf_encode(logical, rows, k)
    body = enc[128:]
    padded = (rows + 127) // 128 * 128
    step = 7 if rows * groups > 4096 else 1
    for row in range(0, padded, step):
        for kg in range(groups):
            want = logical[row * groups + kg] if row < rows else 0
            assert _decode_one_six(body, padded, k, row, kg) == want
    # scale_at agrees with the test-side decoder for in-range groups
    for g in range(0, rows * groups, 13):
        assert o.lib().orc_csf_scale_at(enc.ctypes.data_as(__import__("ctypes").POINTER(__import__("ctypes").c_uint8)), g) == logical[g]
    # header: k, rows, log2(k/16), 6 + mask bytes (2 here: values >= 128 present)
    assert int.from_bytes(enc[0:4].tobytes(), "little") == k
    assert int.from_bytes(enc[4:8].tobytes(), "little") == rows
    assert enc[8] == (k // 16).bit_length() - 1 and enc[9] == 8


def test_positive_scales_use_one_mask_byte_and_896_byte_tiles():
    rows, k = 256, 768 * 1 + 0
    k = 768
    raw = (np.arange(rows * k // 16) * 7 % 0x79).astype(np.uint8)
    enc = o.csf_encode(raw, rows, k)
    assert len(enc) == o.csf_encoded_len(rows, k) == 128 + 2 * 6 * 896
    assert enc[9] == 7 and enc[8] == 4  # 48 groups per row: trailing zeros of 48
    assert np.array_equal(o.csf_decode(enc, raw.size), raw)
    assert np.array_equal(o.csf_decode_matrix(enc, rows, k), raw)


def test_compact_vectors_preserve_all_scale_bytes():
    for length in [16, 128, 256, 2048, 6144]:
        source = (np.arange(length // 16) * 37 % 256).astype(np.uint8)
        k = 1 << (max(length, 128) - 1).bit_length()
        enc = o.csf_encode(source, 1, k)
        assert len(enc) == o.csf_encoded_len(1, k)
        assert np.array_equal(o.csf_decode(enc, source.size), source)


def test_mixed_zero_scale_bytes_stay_exact():
    for values in ([0, 96, 101, 0, 112, 96, 101, 0], [0, 1, 63, 0, 1, 63, 0, 0],
                   [0, 127, 127, 0, 127, 0, 127, 0], [0, 1, 127, 0, 1, 127, 0, 1]):
        enc = o.csf_encode(np.array(values, np.uint8), 1, 128)
        assert list(o.csf_decode(enc, 8)) == values


def test_every_high_bit_mask():
    for mask in range(256):
        values = [((i * 7 + mask) % 64) | (((mask >> i) & 1) << 6) for i in range(8)]
        enc = o.csf_encode(np.array(values, np.uint8), 1, 128)
        assert list(o.csf_decode(enc, 8)) == values
        # the same eight codes as one matrix record (row 0 of a 128x128 tile)
        raw = np.zeros(128 * 8, np.uint8)
        raw[:8] = values
        m = o.csf_encode(raw, 128, 128)
        assert list(o.csf_decode(m, 8)) == values


def test_preconditions():
    with pytest.raises(ValueError):
        o.csf_encode(np.zeros(4, np.uint8), 2, 64)  # k must be a multiple of 128
    with pytest.raises(ValueError):
        o.csf_encode(np.zeros(100, np.uint8), 2, 128)  # raw longer than rows*k/16
