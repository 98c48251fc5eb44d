"""The bit arithmetic of the MXFP4 expansion, restated in numpy and checked against the plain
dequantisation for every code and a range of scales (no GPU).

Device side (csrc/mxfp4.cu, csrc/grouped_gemm_pair.cu): the loader stores the eight nibbles of
every packed 32-bit word as e0 e2 e4 e6 | e1 e3 e5 e7; the kernel picks a pair of elements with
one mask, makes both shifted copies of the two nibbles with one multiply, keeps sign and
magnitude bits with one mask - a bf16 pair whose values are code * 2^-126 - and multiplies by
2^(scale - 1) in bf16."""
import numpy as np

import helpers  # noqa: F401  (puts the package on the path under its importable name)
from gpt_oss_b200 import synth


def _reorder(words):
    """e0 e1 ... e7 (element k at bits 4k) -> e0 e2 e4 e6 | e1 e3 e5 e7."""
    out = np.zeros_like(words)
    for pos, k in enumerate([0, 2, 4, 6, 1, 3, 5, 7]):
        out |= ((words >> np.uint32(4 * k)) & np.uint32(0xF)) << np.uint32(4 * pos)
    return out


def _bf16_bits_to_f32(bits16):
    return (bits16.astype(np.uint32) << np.uint32(16)).view(np.float32)


def _expand_word(w, scale_byte):
    """One reordered word -> its 8 values, the way the kernel's lanes compute them."""
    w8 = w >> np.uint32(8)
    raws = [
        ((w & np.uint32(0x000F000F)) * np.uint32(0x1040)) & np.uint32(0x81C081C0),
        ((w & np.uint32(0x00F000F0)) * np.uint32(0x104)) & np.uint32(0x81C081C0),
        ((w8 & np.uint32(0x000F000F)) * np.uint32(0x1040)) & np.uint32(0x81C081C0),
        ((w8 & np.uint32(0x00F000F0)) * np.uint32(0x104)) & np.uint32(0x81C081C0),
    ]
    s1 = min(int(scale_byte), 128)
    mul = np.float32(2.0) ** np.float32(s1 - 1)             # the bf16 (s1 + 126) << 7
    vals = []
    for r in raws:
        lo = _bf16_bits_to_f32(np.uint16(r & np.uint32(0xFFFF)))   # code * 2^-126, maybe subnormal
        hi = _bf16_bits_to_f32(np.uint16(r >> np.uint32(16)))
        for v in (lo, hi):
            p = np.float32(np.float64(v) * np.float64(mul))        # exact: a power of two
            if scale_byte > 128:
                p = np.float32(np.float64(p) * 2.0 ** (int(scale_byte) - 128))
            vals.append(p)
    return np.array(vals, dtype=np.float32)


def test_every_code_and_scale_expands_to_the_dequantised_value():
    rng = np.random.default_rng(0)
    # 64 rows of 32 codes: all 256 byte values appear in every position of a word
    blocks = np.concatenate([np.arange(256, dtype=np.uint8).repeat(16).reshape(256, 16),
                             rng.integers(0, 256, size=(64, 16), dtype=np.uint8)])
    for scale in (90, 100, 119, 123, 126, 127, 128, 129, 131):
        scales = np.full((blocks.shape[0], 1), scale, dtype=np.uint8)
        want = synth.mxfp4_dequant(blocks, scales)          # [rows, 32]
        words = blocks.view(np.uint32)                      # [rows, 4], little endian: element k at bits 4k
        got = np.stack([np.concatenate([_expand_word(_reorder(w), scale) for w in row])
                        for row in words])
        np.testing.assert_array_equal(got, want.astype(np.float32))


def test_the_multiply_cannot_mix_the_two_nibbles():
    for n0 in range(16):
        for n1 in range(16):
            u = np.uint32(n0 | (n1 << 16))
            r = (u * np.uint32(0x1040)) & np.uint32(0x81C081C0)
            want = ((n0 & 7) << 6) | ((n0 & 8) << 12) | (((n1 & 7) << 6 | (n1 & 8) << 12) << 16)
            assert int(r) == want
            r2 = ((u << np.uint32(4)) * np.uint32(0x104)) & np.uint32(0x81C081C0)
            assert int(r2) == want
