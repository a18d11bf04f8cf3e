"""Writes tests/golden/known_answers.json.

The reference cannot be executed here (Rust workspace, no toolchain), so the golden
vectors are the reference's own known-answer tests, read as text: each case rebuilds
the block bytes the cited test builds and records the closed-form values that test
asserts (value per element range, with the tolerance the test uses; 0 = exact).
Nothing in this script calls the oracle or the CUDA library, so the fixture pins both.

Run:  python tests/golden/make_golden.py
"""
import json
import os

import numpy as np


def f16(v: float) -> bytes:
    return np.float16(v).tobytes()


cases = []


def add(name, fmt, data, num_elements, expect, cite, scales=None):
    cases.append({
        "name": name, "fmt": fmt, "bytes": bytes(data).hex(), "num_elements": num_elements,
        "scales": bytes(scales).hex() if scales is not None else None,
        "expect": [{"start": s, "end": e, "value": v, "tol": t} for (s, e, v, t) in expect],
        "cite": cite,
    })


# ---- Q8_0 -----------------------------------------------------------------
b = bytearray(34)
for i in range(32):
    b[2 + i] = 42
add("q8_0_zero_scale", "Q8_0", b, 32, [(0, 32, 0.0, 0.0)], "crates/nn-gguf/src/dequant.rs:699-715")

# ---- Q4_0 -----------------------------------------------------------------
b = bytearray(18)
b[0:2] = f16(1.0)
for i in range(16):
    b[2 + i] = 0x88
add("q4_0_centered", "Q4_0", b, 32, [(0, 32, 0.0, 1e-6)], "crates/nn-gguf/src/dequant.rs:717-734")

# ---- Q4_K (nn-gguf) -------------------------------------------------------
b = bytearray(144)
for i in range(4, 16):
    b[i] = 0xFF
for i in range(16, 144):
    b[i] = 0xAB
add("q4_k_zero_d_dmin", "Q4_K", b, 256, [(0, 256, 0.0, 0.0)], "crates/nn-gguf/src/dequant.rs:750-770")

b = bytearray(144)
b[0:2] = f16(1.0)
b[4] = 0x02
for i in range(16):
    b[16 + i] = 0x33
add("q4_k_known_values", "Q4_K", b, 256, [(0, 32, 6.0, 1e-4), (32, 256, 0.0, 1e-6)],
    "crates/nn-gguf/src/dequant.rs:772-818")

b = bytearray(144)
b[0:2] = f16(1.0)
b[2:4] = f16(0.5)
b[4] = 0x01
b[8] = 0x04
add("q4_k_with_dmin", "Q4_K", b, 256, [(0, 32, -2.0, 1e-3)], "crates/nn-gguf/src/dequant.rs:820-852")

# high two scale bits: the Q5_K test exercises the same 12-byte packing
# (low nibble 3, high crumb 2 -> scale 35); with d = 1 and q = 1 in sub-block 0
# the nn-gguf Q4_K decoder must give 35.
b = bytearray(144)
b[0:2] = f16(1.0)
b[4] = 0x03
b[12] = 0x02
for i in range(16):
    b[16 + i] = 0x11
add("q4_k_high_scale_bits", "Q4_K", b, 256, [(0, 32, 35.0, 0.0), (32, 256, 0.0, 0.0)],
    "crates/nn-gguf/src/dequant.rs:2118-2149 (packing shared with Q4_K, :353-377)")

# ---- Q6_K -----------------------------------------------------------------
b = bytearray(210)
for i in range(192):
    b[i] = 0xAB
for i in range(192, 208):
    b[i] = 0x7F
add("q6_k_zero_d", "Q6_K", b, 256, [(0, 256, 0.0, 0.0)], "crates/nn-gguf/src/dequant.rs:1165-1182")

b = bytearray(210)
b[208:210] = f16(1.0)
for i in range(192):
    b[i] = 0xFF
add("q6_k_zero_scales", "Q6_K", b, 256, [(0, 256, 0.0, 0.0)], "crates/nn-gguf/src/dequant.rs:1184-1201")

b = bytearray(210)
b[208:210] = f16(1.0)
for i in range(192, 208):
    b[i] = 1
for i in range(128, 192):
    b[i] = 0xAA
add("q6_k_centered_q32", "Q6_K", b, 256, [(0, 256, 0.0, 1e-4)], "crates/nn-gguf/src/dequant.rs:1203-1227")

b = bytearray(210)
b[208:210] = f16(0.5)
b[192] = 2
for i in range(8):
    b[i] = 0x33
for i in range(4):
    b[128 + i] = 0xAA
add("q6_k_known_values", "Q6_K", b, 256, [(0, 16, 3.0, 1e-3), (16, 256, 0.0, 1e-4)],
    "crates/nn-gguf/src/dequant.rs:1229-1281")

b = bytearray(210)
b[208:210] = f16(1.0)
b[192] = 0xFD
for i in range(8):
    b[i] = 0x11
for i in range(4):
    b[128 + i] = 0xAA
add("q6_k_negative_scale", "Q6_K", b, 256, [(0, 16, -3.0, 1e-3)], "crates/nn-gguf/src/dequant.rs:1283-1314")

b = bytearray(420)
b[208:210] = f16(1.0)
b[210 + 208:210 + 210] = f16(2.0)
add("q6_k_two_blocks", "Q6_K", b, 512, [(0, 512, 0.0, 0.0)], "crates/nn-gguf/src/dequant.rs:1316-1334")

b = bytearray(210)
b[208:210] = f16(0.5)
b[192] = 4
for i in range(8):
    b[i] = 0xFF
for i in range(4):
    b[128 + i] = 0xFF
add("q6_k_max_quant", "Q6_K", b, 256, [(0, 16, 62.0, 1e-2), (16, 256, 0.0, 1e-4)],
    "crates/nn-gguf/src/dequant.rs:1336-1374")

b = bytearray(210)
b[208:210] = f16(1.0)
b[192] = 2
add("q6_k_min_quant", "Q6_K", b, 256, [(0, 16, -64.0, 1e-2)], "crates/nn-gguf/src/dequant.rs:1376-1399")

# ---- MXFP4 ----------------------------------------------------------------
# E2M1 table through each decoder at scale 1 (e = 127): codes 0..15 then zeros.
codes = list(range(16)) + [0] * 16
lut = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
packed_low_even = bytearray(16)
packed_high_even = bytearray(16)
for i in range(0, 32, 2):
    packed_low_even[i // 2] = codes[i] | (codes[i + 1] << 4)
    packed_high_even[i // 2] = (codes[i] << 4) | codes[i + 1]
exp_lut = [(i, i + 1, lut[i], 0.0) for i in range(16)] + [(16, 32, 0.0, 0.0)]
add("mxfp4_core_e2m1_table", "MXFP4_CORE", bytes([127]) + bytes(packed_low_even), 32, exp_lut,
    "crates/nn-core/src/layers/quantized/mxfp4.rs:60; mxfp4_tests.rs:259-283")
add("mxfp4_gptoss_lut", "MXFP4_GPTOSS", packed_high_even, 32, exp_lut,
    "crates/nn-gptoss/src/quantize.rs:271-289", scales=bytes([127]))
add("mxfp4_split_lut", "MXFP4_SPLIT", packed_low_even, 32, exp_lut,
    "crates/nn-metal/src/mxfp4_gemm_msl.rs:94-101,124-145", scales=bytes([127]))
# block scale: e = 127 -> 1, 128 -> 2, 126 -> 0.5 (code 2 = 1.0 in element 0)
one = bytearray(16)
one[0] = 0x02
one_hi = bytearray(16)
one_hi[0] = 0x20
for e, v in ((127, 1.0), (128, 2.0), (126, 0.5)):
    add(f"mxfp4_core_scale_e{e}", "MXFP4_CORE", bytes([e]) + bytes(one), 32, [(0, 1, v, 0.0), (1, 32, 0.0, 0.0)],
        "crates/nn-core/src/layers/quantized/mxfp4_tests.rs:293-304")
    add(f"mxfp4_gptoss_scale_e{e}", "MXFP4_GPTOSS", one_hi, 32, [(0, 1, v, 0.0), (1, 32, 0.0, 0.0)],
        "crates/nn-gptoss/src/quantize.rs:373-377", scales=bytes([e]))

# ---- Q5_0 / Q5_1 ----------------------------------------------------------
D = "crates/nn-gguf/src/dequant.rs:"
add("q5_0_zero_scale", "Q5_0", bytearray(22), 32, [(0, 32, 0.0, 0.0)], D + "898-907")
b = bytearray(22)
b[0:2] = f16(1.0)
b[2:6] = b"\xff" * 4
add("q5_0_centered", "Q5_0", b, 32, [(0, 32, 0.0, 1e-4)], D + "909-928")
b = bytearray(22)
b[0:2] = f16(0.5)
b[6:22] = b"\x55" * 16
add("q5_0_known_values", "Q5_0", b, 32, [(0, 32, -5.5, 1e-3)], D + "930-951")
b = bytearray(44)
b[0:2] = f16(1.0)
b[22:24] = f16(2.0)
add("q5_0_two_blocks", "Q5_0", b, 64, [(0, 32, -16.0, 1e-3), (32, 64, -32.0, 1e-3)], D + "953-984")
b = bytearray(22)
b[0:2] = f16(1.0)
b[2:6] = (0xAAAAAAAA).to_bytes(4, "little")
add("q5_0_mixed_high_bits", "Q5_0", b, 32,
    [(i, i + 1, -16.0 if i % 2 == 0 else 0.0, 1e-3) for i in range(32)], D + "986-1023")

b = bytearray(24)
b[2:4] = f16(3.0)
b[8:24] = b"\xaa" * 16
add("q5_1_zero_scale", "Q5_1", b, 32, [(0, 32, 3.0, 1e-3)], D + "1027-1042")
b = bytearray(24)
b[0:2] = f16(1.0)
b[4:8] = b"\xff" * 4
b[8:24] = b"\x77" * 16
add("q5_1_known_values", "Q5_1", b, 32, [(0, 32, 23.0, 1e-2)], D + "1044-1070")
b = bytearray(24)
b[0:2] = f16(0.5)
b[2:4] = f16(10.0)
add("q5_1_with_minimum", "Q5_1", b, 32, [(0, 32, 10.0, 1e-2)], D + "1072-1092")
b = bytearray(48)
b[0:2] = f16(1.0)
b[24:26] = f16(1.0)
b[26:28] = f16(5.0)
add("q5_1_two_blocks", "Q5_1", b, 64, [(0, 32, 0.0, 1e-3), (32, 64, 5.0, 1e-2)], D + "1094-1127")
b = bytearray(24)
b[0:2] = f16(1.0)
b[4:8] = b"\xff" * 4
b[8:24] = b"\xff" * 16
add("q5_1_max_quant", "Q5_1", b, 32, [(0, 32, 31.0, 1e-2)], D + "1129-1155")

# ---- Q2_K -----------------------------------------------------------------
b = bytearray(84)
b[0:80] = b"\xff" * 80
add("q2_k_zero_d_dmin", "Q2_K", b, 256, [(0, 256, 0.0, 0.0)], D + "1410-1427")
b = bytearray(84)
b[80:82] = f16(1.0)
b[0] = 0x03
b[16:20] = b"\xaa" * 4
add("q2_k_known_values", "Q2_K", b, 256, [(0, 16, 6.0, 1e-3), (16, 256, 0.0, 1e-6)], D + "1429-1470")
b = bytearray(84)
b[80:82] = f16(1.0)
b[82:84] = f16(0.5)
b[0] = 0x41
add("q2_k_with_dmin", "Q2_K", b, 256, [(0, 16, -2.0, 1e-3), (16, 256, 0.0, 1e-6)], D + "1472-1510")
b = bytearray(84)
b[80:82] = f16(2.0)
b[82:84] = f16(1.0)
b[0] = 0xFF
b[16:20] = b"\xff" * 4
add("q2_k_max_quant", "Q2_K", b, 256, [(0, 16, 75.0, 1e-1)], D + "1512-1542")
b = bytearray(168)
b[80:82] = f16(1.0)
b[84 + 80:84 + 82] = f16(1.0)
add("q2_k_two_blocks", "Q2_K", b, 512, [(0, 512, 0.0, 0.0)], D + "1544-1561")

# ---- Q3_K -----------------------------------------------------------------
b = bytearray(110)
b[0:108] = b"\xff" * 108
add("q3_k_zero_d", "Q3_K", b, 256, [(0, 256, 0.0, 0.0)], D + "1571-1585")


def q3k_unit_scales(d):
    b = bytearray(110)
    b[108:110] = f16(d)
    b[96:104] = b"\x11" * 8     # low nibbles 1
    b[104:108] = b"\xaa" * 4    # high crumbs 2 -> 1 | 2 << 4 = 33 -> scale +1
    return b


b = q3k_unit_scales(1.0)
b[0:32] = b"\xff" * 32
add("q3_k_centered_q4", "Q3_K", b, 256, [(0, 256, 0.0, 1e-4)], D + "1587-1621")
b = bytearray(110)
b[108:110] = f16(0.5)
b[96] = 0x01
b[104] = 0x02
b[0] = b[1] = 0xFF
b[32:36] = b"\x55" * 4
add("q3_k_known_values", "Q3_K", b, 256, [(0, 16, 0.5, 1e-3)], D + "1623-1670")
b = bytearray(110)
b[108:110] = f16(1.0)
add("q3_k_zero_scales_nonzero_d", "Q3_K", b, 256, [(0, 256, 128.0, 1e-1)], D + "1672-1690")
b = q3k_unit_scales(1.0)
b[0:32] = b"\xff" * 32
b[32:96] = b"\xff" * 64
add("q3_k_all_q3_max", "Q3_K", b, 256, [(0, 256, 3.0, 1e-3)], D + "1692-1726")
b = bytearray(110)
b[108:110] = f16(0.5)
b[96:104] = b"\x22" * 8
b[104:108] = b"\xaa" * 4
add("q3_k_all_q3_min", "Q3_K", b, 256, [(0, 256, -4.0, 1e-3)], D + "1728-1760")
b = bytearray(110)
b[108:110] = f16(1.0)
b[96] = 0x0F
b[104] = 0x01
b[0] = b[1] = 0xFF
b[32:36] = b"\x55" * 4
add("q3_k_negative_scale", "Q3_K", b, 256, [(0, 16, -1.0, 1e-3)], D + "1762-1794")
b = bytearray(220)
b[0:108] = b"\xab" * 108
b[110:218] = b"\xcd" * 108
add("q3_k_two_blocks", "Q3_K", b, 512, [(0, 512, 0.0, 0.0)], D + "1796-1811")
b = bytearray(110)
b[108:110] = f16(1.0)
b[96] = 0x01
b[104] = 0x02
b[1] = 0xFF
add("q3_k_mixed_high_bits", "Q3_K", b, 256, [(0, 8, -4.0, 1e-3), (8, 16, 0.0, 1e-3)], D + "1813-1853")

# ---- Q5_K -----------------------------------------------------------------
b = bytearray(176)
b[4:176] = b"\xff" * 172
add("q5_k_zero_d_dmin", "Q5_K", b, 256, [(0, 256, 0.0, 0.0)], D + "1863-1877")
b = bytearray(176)
b[0:2] = f16(1.0)
b[4] = 0x02
b[48:64] = b"\x33" * 16
add("q5_k_known_values", "Q5_K", b, 256, [(0, 32, 6.0, 1e-3), (32, 256, 0.0, 1e-6)], D + "1879-1921")
b = bytearray(176)
b[0:2] = f16(1.0)
b[2:4] = f16(0.5)
b[4] = 0x01
b[8] = 0x04
add("q5_k_with_dmin", "Q5_K", b, 256, [(0, 32, -2.0, 1e-3)], D + "1923-1954")
b = bytearray(176)
b[0:2] = f16(1.0)
b[4] = 0x01
b[16:48] = b"\xff" * 32
add("q5_k_with_high_bit", "Q5_K", b, 256, [(0, 32, 16.0, 1e-3)], D + "1956-1988")
b = bytearray(176)
b[0:2] = f16(0.5)
b[4] = 0x04
b[16:48] = b"\xff" * 32
b[48:176] = b"\xff" * 128
add("q5_k_max_quant", "Q5_K", b, 256, [(0, 32, 62.0, 1e-1)], D + "1990-2024")
b = bytearray(176)
b[0:2] = f16(1.0)
b[4] = 0x01
b[17] = 0xFF
add("q5_k_mixed_high_bits", "Q5_K", b, 256, [(0, 8, 0.0, 1e-4), (8, 16, 16.0, 1e-3), (16, 32, 0.0, 1e-4)], D + "2026-2065")
b = bytearray(352)
b[0:2] = f16(1.0)
b[176:178] = f16(2.0)
add("q5_k_two_blocks", "Q5_K", b, 512, [(0, 512, 0.0, 0.0)], D + "2067-2083")
b = bytearray(176)
b[0:2] = f16(1.0)
b[2:4] = f16(1.0)
b[4] = 0x02
b[8] = 0x03
add("q5_k_scale_packing", "Q5_K", b, 256, [(0, 32, -3.0, 1e-3)], D + "2087-2116")
b = bytearray(176)
b[0:2] = f16(0.1)
b[4] = 0x03
b[12] = 0x02
b[48:64] = b"\x11" * 16
add("q5_k_high_scale_bits", "Q5_K", b, 256, [(0, 32, float(np.float32(np.float16(0.1)) * np.float32(35.0)), 1e-2)],
    D + "2118-2145")

# ---- fused nn-core product (Q8_0 / Q4_0): weight rows all equal ------------
matmul = []


def q8_block(scale, q):
    return f16(scale) + bytes([q & 0xFF] * 32)


def q4_0_block(scale, nib):
    return f16(scale) + bytes([nib | (nib << 4)] * 16)


def add_mm(name, fmt, block, n, k, x_rows, bias, expect, tol, cite):
    matmul.append({"name": name, "fmt": fmt, "bytes": (block * (n * (k // 32))).hex(), "n": n, "k": k,
                   "x": x_rows, "bias": bias, "expect": expect, "tol": tol, "cite": cite})


add_mm("q8_0_known_values", "Q8_0", q8_block(0.5, 2), 2, 32, [[1.0] * 32], None, [[32.0, 32.0]], 0.5,
       "crates/nn-core/src/dyn_tensor/quantized_matmul_tests.rs:150-165")
add_mm("q8_0_identity_like", "Q8_0", q8_block(1.0, 1), 1, 32, [[1.0] * 32, [2.0] * 32], None, [[32.0], [64.0]],
       0.5, "crates/nn-core/src/dyn_tensor/quantized_matmul_tests.rs:167-198")
add_mm("q8_0_batch_4d", "Q8_0", q8_block(1.0, 1), 3, 32, [[2.0] * 32] * 4, None, [[64.0] * 3] * 4, 1.0,
       "crates/nn-core/src/dyn_tensor/quantized_matmul_tests.rs:296-317")
add_mm("linear_with_bias", "Q8_0", q8_block(1.0, 1), 2, 32, [[1.0] * 32], [10.0, 20.0], [[42.0, 52.0]], 1.0,
       "crates/nn-core/src/dyn_tensor/quantized_matmul_tests.rs:323-350")
add_mm("linear_batched_with_bias", "Q8_0", q8_block(1.0, 1), 3, 32, [[0.5] * 32] * 2, [100.0, 200.0, 300.0],
       [[116.0, 216.0, 316.0]] * 2, 1.0, "crates/nn-core/src/dyn_tensor/quantized_matmul_tests.rs:383-414")
add_mm("q8_0_multi_block", "Q8_0", q8_block(1.0, 1), 2, 64, [[1.0] * 64], None, [[64.0, 64.0]], 1.0,
       "crates/nn-core/src/dyn_tensor/quantized_matmul_tests.rs:528-546")
add_mm("q4_0_known_values", "Q4_0", q4_0_block(1.0, 9), 2, 32, [[1.0] * 32], None, [[32.0, 32.0]], 0.5,
       "crates/nn-core/src/dyn_tensor/quantized_matmul_tests.rs:88-105")
add_mm("q4_0_zero_weight", "Q4_0", q4_0_block(2.0, 8), 4, 32, [[42.0] * 32] * 3, None, [[0.0] * 4] * 3, 1e-6,
       "crates/nn-core/src/dyn_tensor/quantized_matmul_tests.rs:107-125")
add_mm("q4_0_negative_values", "Q4_0", q4_0_block(0.5, 4), 1, 32, [[1.0] * 32], None, [[-64.0]], 1.0,
       "crates/nn-core/src/dyn_tensor/quantized_matmul_tests.rs:127-144")
add_mm("q4_0_multi_block", "Q4_0", q4_0_block(1.0, 9), 1, 96, [[1.0] * 96] * 2, None, [[96.0], [96.0]], 1.0,
       "crates/nn-core/src/dyn_tensor/quantized_matmul_tests.rs:548-566")

out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "known_answers.json")
with open(out, "w") as f:
    json.dump({"dequant": cases, "matmul": matmul}, f, indent=1)
print(f"wrote {out}: {len(cases)} dequant cases, {len(matmul)} matmul cases")
