"""Independent packers for the GGUF block formats (test helpers).

They are the inverse of the decode rules the reference states (quantization.cpp:338-357 for
the Q4_K 6-bit scale/min packing, :558-593 for the Q6_K bit planes) and build the
known-answer blocks of the reference's own tests from their stated field values.
"""
from __future__ import annotations

import struct

import numpy as np


def q4k_block(d_bits: int, dmin_bits: int, scales, minima, nibbles) -> np.ndarray:
    block = np.zeros(144, np.uint8)
    block[0:2] = np.frombuffer(struct.pack("<H", d_bits), np.uint8)
    block[2:4] = np.frombuffer(struct.pack("<H", dmin_bits), np.uint8)
    packed = block[4:16]
    for g in range(4):
        packed[g] = scales[g] | ((scales[g + 4] >> 4) << 6)
        packed[g + 4] = minima[g] | ((minima[g + 4] >> 4) << 6)
        packed[g + 8] = (scales[g + 4] & 15) | ((minima[g + 4] & 15) << 4)
    q = block[16:]
    for chunk in range(4):
        for i in range(32):
            q[chunk * 32 + i] = nibbles[64 * chunk + i] | (nibbles[64 * chunk + 32 + i] << 4)
    return block


def q6k_block(d_bits: int, scales, quants) -> np.ndarray:
    """quants are the stored 6-bit codes (value + 32), scales signed int8."""
    block = np.zeros(210, np.uint8)
    for half in range(2):
        for lane in range(32):
            q = [quants[half * 128 + quarter * 32 + lane] for quarter in range(4)]
            block[half * 64 + lane] = (q[0] & 15) | ((q[2] & 15) << 4)
            block[half * 64 + 32 + lane] = (q[1] & 15) | ((q[3] & 15) << 4)
            block[128 + half * 32 + lane] = sum((q[quarter] >> 4) << (quarter * 2) for quarter in range(4))
    block[192:208] = np.array(scales, np.int8).view(np.uint8)
    block[208:210] = np.frombuffer(struct.pack("<H", d_bits), np.uint8)
    return block


def q80_block(d_bits: int, values) -> np.ndarray:
    block = np.zeros(34, np.uint8)
    block[0:2] = np.frombuffer(struct.pack("<H", d_bits), np.uint8)
    block[2:] = np.array(values, np.int8).view(np.uint8)
    return block


def f16_bits(value: float) -> int:
    return int(np.array([value], np.float16).view(np.uint16)[0])


# ---- the reference's known-answer blocks ----

def reference_q8_0_kat():
    """tests/tensor/tensor_tests.cpp:474-503: scale 0x3800 = 0.5."""
    raw = bytes([0x00, 0x38, 0x00, 0x02, 0xFE, 0x7F, 0x80, 0x04, 0x06, 0x08, 0x0A, 0x0C, 0x0E, 0x10, 0x12, 0x14,
                 0x16, 0x18, 0x1A, 0x1C, 0x1E, 0x20, 0x22, 0x24, 0x26, 0x28, 0x2A, 0x2C, 0x2E, 0x30, 0x32, 0x34,
                 0x36, 0x38])
    expected = {0: 0.0, 1: 1.0, 2: -1.0, 3: 63.5, 4: -64.0}
    return np.frombuffer(raw, np.uint8).copy(), expected


def reference_q4_k_kat():
    """tests/support/tensor_test_support.cpp:223-241 with the expectations of
    tests/tensor/tensor_tests.cpp:539-559,658-676: d = 1.0, dmin = 0.5."""
    scales, minima, nibbles = [0] * 8, [0] * 8, [0] * 256
    scales[0], minima[0] = 2, 1
    scales[1], minima[1] = 3, 2
    scales[4], minima[4] = 6, 5
    nibbles[0], nibbles[31], nibbles[32], nibbles[63], nibbles[128] = 4, 15, 5, 6, 7
    block = q4k_block(0x3C00, 0x3800, scales, minima, nibbles)
    expected = {0: 7.5, 32: 14.0, 128: 39.5, 31: 29.5, 63: 17.0}
    x = np.zeros(256, np.float32)
    x[0], x[32], x[128] = 1.0, 2.0, -1.0
    return block, expected, x, -4.0


def reference_q6_k_kat():
    """tests/support/tensor_test_support.cpp:243-262 with the expectations of
    tests/tensor/tensor_tests.cpp:678-721: d = 0.5."""
    scales = [0] * 16
    scales[0], scales[1], scales[2], scales[4], scales[8] = 2, 3, -3, 4, -2
    values = [0] * 256            # stored code = value + 32; untouched elements hold code 0 = value -32
    codes = [0] * 256
    for index, value in ((0, -32), (31, 31), (32, -1), (64, 5), (128, 7)):
        codes[index] = value + 32
    del values
    block = q6k_block(0x3800, scales, codes)
    expected = {0: -32.0, 32: 1.5, 64: 10.0, 31: 46.5, 128: -7.0}
    x = np.zeros(256, np.float32)
    x[0], x[32], x[64], x[128] = 1.0, 2.0, -1.0, 3.0
    return block, expected, x, -60.0
