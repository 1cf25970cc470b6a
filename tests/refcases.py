"""Known-answer cases restated from the FFAI reference's own unit tests.

Each builder re-derives the inputs from the formulas written in the cited test
(values, not code) and computes the expected result with plain numpy in float64,
independently of the C oracle.  Paths are relative to the FFAI project.
"""
from __future__ import annotations

import numpy as np


def trunc_bf16(a):
    """bf16 by truncation, as the reference's GEMV tests build their inputs
    (``bitPattern >> 16``; Tests/FFAITests/Ops/QuantizedOpsTests.swift:221-223)."""
    bits = np.asarray(a, dtype=np.float32).view(np.uint32)
    return (bits >> 16).astype(np.uint16)


def rne_bf16(a):
    """bf16 by round-to-nearest-even (MoEBgemmBm64MppTests.swift:68-72)."""
    bits = np.asarray(a, dtype=np.float32).view(np.uint32)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_f32(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ── byte-wise pack helpers, restating QuantizedOpsTests.swift:33-124 ──

def _bytes_to_u32(by):
    by = np.asarray(by, dtype=np.uint8).reshape(-1, 4).astype(np.uint32)
    return by[:, 0] | (by[:, 1] << 8) | (by[:, 2] << 16) | (by[:, 3] << 24)


def pack8_4bit(q):        # pack8, :33-39
    w = 0
    for i in range(8):
        w |= (int(q[i]) & 0xF) << (4 * i)
    return np.array([w], dtype=np.uint32)


def pack4_bytes(q):       # pack4Bytes, :42-47
    w = 0
    for i in range(4):
        w |= (int(q[i]) & 0xFF) << (8 * i)
    return np.array([w], dtype=np.uint32)


def pack16_2bit(q):       # pack16Twobit, :50-55
    w = 0
    for i in range(16):
        w |= (int(q[i]) & 0x3) << (2 * i)
    return np.array([w], dtype=np.uint32)


def pack16_6bit(q):       # pack16Sixbit, :58-71
    by = [0] * 12
    for p in range(4):
        v0, v1, v2, v3 = (int(q[p * 4 + j]) & 0x3F for j in range(4))
        by[p * 3 + 0] = (v0 | ((v1 & 0x03) << 6)) & 0xFF
        by[p * 3 + 1] = (((v1 >> 2) & 0x0F) | ((v2 & 0x0F) << 4)) & 0xFF
        by[p * 3 + 2] = (((v2 >> 4) & 0x03) | ((v3 & 0x3F) << 2)) & 0xFF
    return _bytes_to_u32(by)


def pack32_3bit(q):       # pack32Threebit, :75-88
    by = [0] * 12
    for c in range(4):
        v = [int(q[c * 8 + j]) & 0x07 for j in range(8)]
        by[c * 3 + 0] = (v[0] | (v[1] << 3) | ((v[2] & 0x03) << 6)) & 0xFF
        by[c * 3 + 1] = (((v[2] >> 2) & 0x01) | (v[3] << 1) | (v[4] << 4) | ((v[5] & 0x01) << 7)) & 0xFF
        by[c * 3 + 2] = (((v[5] >> 1) & 0x03) | (v[6] << 2) | (v[7] << 5)) & 0xFF
    return _bytes_to_u32(by)


def pack32_5bit(q):       # pack32Fivebit, :92-109
    by = [0] * 20
    for c in range(4):
        v = [int(q[c * 8 + j]) & 0x1F for j in range(8)]
        by[c * 5 + 0] = (v[0] | ((v[1] & 0x07) << 5)) & 0xFF
        by[c * 5 + 1] = (((v[1] >> 3) & 0x03) | ((v[2] & 0x1F) << 2) | ((v[3] & 0x01) << 7)) & 0xFF
        by[c * 5 + 2] = (((v[3] >> 1) & 0x0F) | ((v[4] & 0x0F) << 4)) & 0xFF
        by[c * 5 + 3] = (((v[4] >> 4) & 0x01) | ((v[5] & 0x1F) << 1) | ((v[6] & 0x03) << 6)) & 0xFF
        by[c * 5 + 4] = (((v[6] >> 2) & 0x07) | ((v[7] & 0x1F) << 3)) & 0xFF
    return _bytes_to_u32(by)


REF_PACKERS = {2: (16, pack16_2bit), 3: (32, pack32_3bit), 4: (8, pack8_4bit), 5: (32, pack32_5bit),
               6: (16, pack16_6bit), 8: (4, pack4_bytes)}


def ref_pack_row(q, bits):
    chunk, fn = REF_PACKERS[bits]
    return np.concatenate([fn(q[i:i + chunk]) for i in range(0, len(q), chunk)])


# ── per-bit-width dequant GEMV cases ──

class GemvCase:
    def __init__(self, name, bits, gs, q, scales_f32, biases_f32, x_f32, trunc=True):
        self.name, self.bits, self.gs = name, bits, gs
        self.out_dim, self.in_dim = q.shape
        conv = trunc_bf16 if trunc else rne_bf16
        self.q = q
        self.weight = np.stack([ref_pack_row(q[r], bits) for r in range(q.shape[0])])
        self.scales = conv(scales_f32).reshape(self.out_dim, self.in_dim // gs)
        self.biases = conv(biases_f32).reshape(self.out_dim, self.in_dim // gs)
        self.x = conv(x_f32)
        s = np.repeat(bf16_f32(self.scales).astype(np.float64), gs, axis=1)
        b = np.repeat(bf16_f32(self.biases).astype(np.float64), gs, axis=1)
        self.expected = ((q.astype(np.float64) * s + b) * bf16_f32(self.x).astype(np.float64)).sum(axis=1)


def gemv_cases():
    cases = []
    # realShapeRoundTrip — QuantizedOpsTests.swift:126-193 (4-bit, gs 64, 4x128)
    o, n, gs = 4, 128, 64
    q = np.array([[(i + r * 7) % 16 for i in range(n)] for r in range(o)], dtype=np.uint32)
    g = o * (n // gs)
    cases.append(GemvCase("int4_gs64_4x128", 4, gs, q, (np.arange(g) + 1) * 0.01, np.arange(g) * -0.005,
                          np.arange(n) * 0.1 - 6.4, trunc=False))
    # roundTripInt6Bf16 — :195-262
    o, n, gs = 2, 64, 64
    q = np.array([[(i + r * 11) & 0x3F for i in range(n)] for r in range(o)], dtype=np.uint32)
    cases.append(GemvCase("int6_gs64_2x64", 6, gs, q, (np.arange(o) + 1) * 0.05, np.arange(o) * -0.1,
                          np.arange(n) * 0.1 - 3.2))
    # runDequantGemvCheck — :264-363 (3-, 2-, 5-bit)
    for bits, mask in ((3, 0x07), (2, 0x03), (5, 0x1F)):
        q = np.array([[(i + r * 7) & mask for i in range(n)] for r in range(o)], dtype=np.uint32)
        cases.append(GemvCase(f"int{bits}_gs64_2x64", bits, gs, q, (np.arange(o) + 1) * 0.04,
                              np.arange(o) * -0.07, np.arange(n) * 0.1 - 3.2))
    # roundTripInt8Bf16 — :365-438
    o, n, gs = 2, 128, 64
    g = o * (n // gs)
    q = np.array([[(i + r * 13) & 0xFF for i in range(n)] for r in range(o)], dtype=np.uint32)
    cases.append(GemvCase("int8_gs64_2x128", 8, gs, q, (np.arange(g) + 1) * 0.001, np.arange(g) * -0.0005,
                          np.arange(n) * 0.1 - 6.4))
    return cases


# ── grouped GEMM integer-hash cases — MoEBgemmBm64MppTests.swift:159-336 ──

class GroupedCase:
    def __init__(self, name, E, M, N, K, gs, seedW, seedS, seedB, seedX, sparse):
        self.name, self.E, self.M, self.N, self.K, self.gs = name, E, M, N, K, gs
        if sparse:   # :166-172
            idx = sorted((r * (E // max(M, 1))) % E for r in range(M))
        else:        # :174-176
            idx = [r // (M // E) for r in range(M)]
        self.indices = np.array(idx, dtype=np.uint32)
        total = E * N * K
        i = np.arange(total, dtype=np.int64)
        q = ((i * seedW + 3) & 0xF).astype(np.uint32)            # :180-183
        self.q = q.reshape(E, N, K)
        qq = self.q.reshape(E, N, K // 8, 8).astype(np.uint32)
        w = np.zeros((E, N, K // 8), dtype=np.uint32)
        for j in range(8):
            w |= qq[..., j] << np.uint32(4 * j)                 # pack8 (low nibble first)
        self.weight = w
        g = np.arange(E * N * (K // gs), dtype=np.int64)
        s = (0.005 + 0.001 * ((g * seedS) % 137).astype(np.float32) / np.float32(137.0)).astype(np.float32)   # :196
        b = (-0.02 + 0.005 * ((g * seedB) % 149).astype(np.float32) / np.float32(149.0)).astype(np.float32)   # :197
        xi = np.arange(M * K, dtype=np.int64)
        x = (0.05 * ((xi * seedX) % 223).astype(np.float32) / np.float32(223.0) - 0.025).astype(np.float32)  # :204
        self.scales = rne_bf16(s).reshape(E, N, K // gs)
        self.biases = rne_bf16(b).reshape(E, N, K // gs)
        self.x = rne_bf16(x).reshape(M, K)

    def expected(self):
        """float64 dequant matmul on the bf16-rounded operands."""
        s = np.repeat(bf16_f32(self.scales).astype(np.float64), self.gs, axis=2)
        b = np.repeat(bf16_f32(self.biases).astype(np.float64), self.gs, axis=2)
        xf = bf16_f32(self.x).astype(np.float64)
        out = np.zeros((self.M, self.N))
        for e in np.unique(self.indices):
            rows = np.nonzero(self.indices == e)[0]
            w = self.q[e].astype(np.float64) * s[e] + b[e]
            out[rows] = xf[rows] @ w.T
        return out


def grouped_cases(include_large=True):
    cases = [
        GroupedCase("clean_tile", 4, 64, 64, 64, 32, 7, 19, 29, 37, False),       # :284-294
        GroupedCase("multi_tile", 8, 128, 128, 128, 64, 11, 23, 31, 41, False),   # :296-308
    ]
    if include_large:
        cases += [
            GroupedCase("qwen36_gate_up", 128, 64, 768, 2048, 64, 13, 19, 23, 29, True),  # :310-325
            GroupedCase("qwen36_down", 128, 64, 2048, 768, 64, 17, 31, 37, 43, True),     # :327-340
        ]
    return cases


# ── router cases — Tests/FFAITests/Benchmark/MoELayerTests.swift:33-111,
#    Tests/FFAITests/Ops/QuantizedOpsTests.swift:999-1027, LFM2TextTests.swift:119-150 ──
# (logits, k, gating_mode, norm, expert_bias, expected indices (ordered or set), expected weights or None, tol)
ROUTER_CASES = [
    ("softmaxThenTopK_norm", [1, 3, 2, 0], 2, 0, 1, None, [1, 2], [0.73107, 0.26893], 1e-4, True),
    ("softmaxThenTopK_raw", [1, 3, 2, 0], 2, 0, 0, None, [1, 2], [0.64391, 0.23688], 1e-4, True),
    ("topKThenSoftmax", [1, 3, 2, 0], 2, 1, 1, None, [1, 2], [0.73106, 0.26894], 1e-4, True),
    ("ties_lower_index", [5, 5, 5, 5], 2, 1, 1, None, [0, 1], [0.5, 0.5], 1e-5, True),
    ("k_equals_E", [0, 1, 2], 3, 0, 1, None, [0, 1, 2], None, 0, False),
    ("gpu_router_1534", [1, 5, 3, 4], 2, 0, 1, None, [1, 3], None, 0, False),
    ("lfm2_expert_bias", [1, 3, 2, 0], 2, 0, 1, [0.5, 0, 0, 0.5], [0, 1], None, 0, False),
]


def four_expert_layer(with_shared: bool):
    """MoELayerTests.swift:150-265: 4 experts, top-2, scalar weights, x = 2.

    The reference test uses hidden = intermediate = 1 with dense fp32 projections.
    The quantized block needs hidden and intermediate to be multiples of 64, so the
    scalars are embedded: x = [2, 0, 0, ...]; a projection with scalar weight `a` has
    q = 0 everywhere and group bias `a` on its row 0 (other rows bias 0).  The
    routed/shared arithmetic is then exactly the reference's scalar chain.
    Returns (arrays dict, spec kwargs, x_f32[64], expected scalar at out[0]).
    """
    H = I = 64
    E = 4
    gate_w = np.zeros((E, H), dtype=np.float32)
    gate_w[:, 0] = [0.5, 1.5, 1.0, 0.0]
    gW, uW, dW = [0.1, 0.7, 0.3, 0.9], [1.0, 0.5, 2.0, 0.4], [0.2, 1.1, 0.6, 0.8]

    def proj(vals, n):
        w = np.zeros((n, 64, 64 * 4 // 32), dtype=np.uint32)
        s = np.zeros((n, 64, 1), dtype=np.float32)
        b = np.zeros((n, 64, 1), dtype=np.float32)
        b[:, 0, 0] = vals
        return w, rne_bf16(s).reshape(n, 64, 1), rne_bf16(b).reshape(n, 64, 1)

    arrays = {"gate.weight": gate_w}
    for name, vals in (("gate_proj", gW), ("up_proj", uW), ("down_proj", dW)):
        w, s, b = proj(vals, E)
        arrays[f"experts.{name}.weight"], arrays[f"experts.{name}.scales"], arrays[f"experts.{name}.biases"] = w, s, b
    sg, su, sd = 0.4, 0.6, 1.5
    if with_shared:
        for name, val in (("gate_proj", sg), ("up_proj", su), ("down_proj", sd)):
            w, s, b = proj([val], 1)
            arrays[f"shared_expert.{name}.weight"], arrays[f"shared_expert.{name}.scales"], arrays[f"shared_expert.{name}.biases"] = w, s, b
    x = np.zeros(H, dtype=np.float32)
    x[0] = 2.0

    def bf(v):
        return float(bf16_f32(rne_bf16(np.array([v], dtype=np.float32)))[0])

    def swiglu_ref(g, u, d):   # MoELayerTests.swift:127-131
        gx = bf(g) * 2.0
        silu = gx * (1.0 / (1.0 + np.exp(-gx)))
        return bf(d) * (silu * (bf(u) * 2.0))

    w1, w2 = 0.73107, 0.26893
    expected = w1 * swiglu_ref(gW[1], uW[1], dW[1]) + w2 * swiglu_ref(gW[2], uW[2], dW[2])
    if with_shared:
        expected += swiglu_ref(sg, su, sd)
    return arrays, x, expected
