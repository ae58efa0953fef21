"""The reference's in-file test fixtures, regenerated from their formulas, and the
"want" values its tests compute — written independently of the oracle (plain numpy /
Python, f64 where the reference uses f64), so the oracle can be pinned against them.

Each function names the reference test it reproduces (path relative to the reference
project root).
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def f16_round(x) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16)


def round_half_away(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    return np.where(x >= 0, np.floor(x + F32(0.5)), np.ceil(x - F32(0.5))).astype(np.float32)


def quantize_a_block_np(a32: np.ndarray):
    """matmul_q_i8.quantizeABlock (src/aion/backend/cpu/kernels/matmul_q_i8.zig:187-203), numpy f32."""
    a32 = np.asarray(a32, dtype=np.float32)
    amax = np.max(np.abs(a32)).astype(np.float32)
    if amax == 0:
        return np.zeros(32, dtype=np.int8), F32(0)
    scale = F32(amax / F32(127.0))
    inv = F32(F32(127.0) / amax)
    q = np.clip(round_half_away(a32 * inv), -127, 127).astype(np.int8)
    return q, scale


def pack_q8_block_np(v32: np.ndarray) -> bytes:
    """quantize.packQ8Block (src/aion/storage/quantize.zig:81-103), numpy f32."""
    v32 = np.asarray(v32, dtype=np.float32)
    absmax = np.max(np.abs(v32)).astype(np.float32)
    scale = F32(1.0) if absmax == 0 else F32(absmax / F32(127.0))
    s16 = np.float16(scale)
    eff = F32(s16)
    inv = F32(0) if (absmax == 0 or eff == 0) else F32(F32(1.0) / eff)
    q = np.clip(round_half_away(v32 * inv), -128, 127).astype(np.int8)
    return s16.tobytes() + q.tobytes()


def pack_q4_block_np(v32: np.ndarray) -> bytes:
    """quantizeQ4_0FromF32Block32 (src/aion/backend/cpu/test_cpu_kernels.zig:490-523), numpy f32."""
    v32 = np.asarray(v32, dtype=np.float32)
    absmax = np.max(np.abs(v32)).astype(np.float32)
    scale = F32(1.0) if absmax == 0 else F32(absmax / F32(7.0))
    s16 = np.float16(scale)
    q = np.clip(round_half_away(v32 / scale), -8, 7).astype(np.int32) + 8
    nib = bytearray(16)
    for t in range(32):
        if t % 2 == 0:
            nib[t >> 1] |= int(q[t]) & 0x0F
        else:
            nib[t >> 1] |= (int(q[t]) & 0x0F) << 4
    return s16.tobytes() + bytes(nib)


# --- src/aion/storage/quantize.zig:105-137 --------------------------------------------
def quantize_zig_q8_kn():
    K, N = 64, 5
    vals = (np.array([(i % 17) - 8 for i in range(K * N)], dtype=np.float32) * F32(0.1)).reshape(K, N)
    expect = bytearray()
    for b in range(K // 32):
        for j in range(N):
            expect += pack_q8_block_np(vals[b * 32:(b + 1) * 32, j])
    return vals, np.frombuffer(bytes(expect), dtype=np.uint8)


# --- src/aion/backend/cpu/kernels/matvec_q.zig:176-219 ---------------------------------
def matvec_q_chunk_case():
    m, n, k = 2, 5, 8192 + 64
    blocks = k // 32
    a = (np.array([(i % 37) - 18 for i in range(m * k)], dtype=np.float32) * F32(0.01)).reshape(m, k)
    b = bytearray()
    s = np.float16(0.02).tobytes()
    for bi in range(blocks * n):
        b += s + bytes(((bi * 5 + t * 3) & 0xFF) for t in range(32))
    return m, n, k, a, np.frombuffer(bytes(b), dtype=np.uint8)


def int8_reference_f64(a: np.ndarray, b: np.ndarray, m: int, n: int, k: int, *, nt: bool, bb: int = 34) -> np.ndarray:
    """The f64 "want" of the reference's matvec / NT / weight_layout tests: the library's
    activation quantizer, exact integer dot, f64 scaling (src/aion/backend/cpu/kernels/matvec_q.zig:198-219)."""
    blocks = k // 32
    want = np.zeros((m, n), dtype=np.float64)
    raw = np.asarray(b, dtype=np.uint8)
    for r in range(m):
        aq = np.zeros((blocks, 32), dtype=np.int64)
        asc = np.zeros(blocks, dtype=np.float64)
        for kb in range(blocks):
            q, s = quantize_a_block_np(a[r, kb * 32:(kb + 1) * 32])
            aq[kb] = q
            asc[kb] = float(s)
        for c in range(n):
            acc = 0.0
            for kb in range(blocks):
                off = ((c * blocks + kb) if nt else (kb * n + c)) * bb
                bs = float(raw[off:off + 2].view(np.float16)[0])
                if bb == 34:
                    wq = raw[off + 2:off + 34].view(np.int8).astype(np.int64)
                else:
                    by = raw[off + 2:off + 18].astype(np.int64)
                    wq = np.empty(32, dtype=np.int64)
                    wq[0::2] = (by & 0x0F) - 8
                    wq[1::2] = (by >> 4) - 8
                acc += asc[kb] * bs * float(np.dot(aq[kb], wq))
            want[r, c] = acc
    return want


# --- src/aion/backend/cpu/kernels/matmul_nt_q.zig:587-637 ------------------------------
def nt_grouped_case(group_rows: int, m: int):
    k = 96
    blocks = k // 32
    n = 2 * group_rows
    rows = bytearray()
    for bi in range(n * blocks):
        sc = np.float16(np.float16(1 + bi % 3) * np.float16(0.01))
        rows += sc.tobytes() + bytes(((bi * 29 + t * 7) & 0xFF) for t in range(32))
    a = (np.array([(i % 19) - 9 for i in range(m * k)], dtype=np.float32) * F32(0.03)).reshape(m, k)
    return m, n, k, a, np.frombuffer(bytes(rows), dtype=np.uint8)


def relayout_map_np(order_group: int, chunk: int, n: int, k: int, src: np.ndarray) -> np.ndarray:
    """QuantBlockOrder placement as the reference's relayout test spells it
    (src/aion/graph/opt/test_opt.zig:946-959), from a ROW-MAJOR [n, k] source."""
    blocks = k // 32
    W = order_group
    out = np.zeros_like(src)
    for r in range(n):
        for kb in range(blocks):
            blk = src[(r * blocks + kb) * 34:(r * blocks + kb) * 34 + 34]
            seg = ((r // W) * blocks + kb) * W * 34
            lane = r % W
            out[seg + 2 * lane:seg + 2 * lane + 2] = blk[0:2]
            for c in range(32 // chunk):
                o = seg + 2 * W + (c * W + lane) * chunk
                out[o:o + chunk] = blk[2 + chunk * c:2 + chunk * c + chunk]
    return out


# --- src/aion/graph/opt/test_opt.zig:1106-1175 -----------------------------------------
def weight_layout_arith_case(m: int):
    k, n = 128, 96
    seed = 12345
    a = np.zeros(m * k, dtype=np.float32)
    for i in range(m * k):
        seed = (seed * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        a[i] = F32(F32((seed >> 33) % 2000) - F32(1000.0)) * F32(0.0005)
    w = (np.array([((i + 1) % 23) - 11 for i in range(k * n)], dtype=np.float32) * F32(0.07)).reshape(k, n)
    return m, n, k, a.reshape(m, k), w


# --- src/aion/backend/cpu/test_cpu_backend.zig:2879-3012 -------------------------------
def nt_backend_case():
    m, k, n = 3, 64, 5
    b_ref = np.zeros((n, k), dtype=np.float32)
    for row in range(n):
        rs = F32(row + 1) * F32(0.0625)
        b_ref[row] = (np.arange(k, dtype=np.float32) - F32(32)) * rs
    packed = bytearray()
    deq_b = np.zeros((n, k), dtype=np.float32)
    for row in range(n):
        absmax = np.max(np.abs(b_ref[row])).astype(np.float32)
        scale = F32(1.0) if absmax == 0 else F32(absmax / F32(127.0))
        inv = F32(0) if absmax == 0 else F32(F32(1.0) / scale)
        s16 = np.float16(scale)
        for blk in range(k // 32):
            q = np.clip(round_half_away(b_ref[row, blk * 32:(blk + 1) * 32] * inv), -128, 127).astype(np.int8)
            packed += s16.tobytes() + q.tobytes()
            deq_b[row, blk * 32:(blk + 1) * 32] = q.astype(np.float32) * F32(s16)
    a = ((np.arange(m * k, dtype=np.float32) - F32(50)) * F32(0.01)).reshape(m, k)
    deq_a = np.zeros_like(a)
    for mi in range(m):
        for blk in range(k // 32):
            q, s = quantize_a_block_np(a[mi, blk * 32:(blk + 1) * 32])
            deq_a[mi, blk * 32:(blk + 1) * 32] = q.astype(np.float32) * s
    c_ref = deq_a.astype(np.float64) @ deq_b.astype(np.float64).T
    return m, n, k, a, np.frombuffer(bytes(packed), dtype=np.uint8), c_ref


# --- attention ------------------------------------------------------------------------
def window_keys(left: int, right: int, chunk: int, q_pos: int, kv_end: int):
    """AttentionWindow.keys (src/aion/graph/graph.zig:160-167)."""
    anchor = (q_pos // chunk) * chunk if chunk > 0 else q_pos
    span = chunk if chunk > 0 else 1
    lo = anchor - min(anchor, left)
    hi = min(kv_end, anchor + span + right)
    return lo, hi


def cached_gqa_ref(q, k, v, positions, end_index, scale, left, right, chunk, soft_cap):
    """cachedGqaRefF32 (src/aion/backend/cpu/test_cpu_backend.zig:4806-4900): exact exp / tanh,
    f32 online softmax. q [B,L,Hq,Dk], k [B,T,Hkv,Dk], v [B,T,Hkv,Dv] as f32."""
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    B, L, Hq, Dk = q.shape
    _, T, Hkv, _ = k.shape
    Dv = v.shape[3]
    g = Hq // Hkv
    out = np.zeros((B, L, Hq, Dv), dtype=np.float32)
    for b in range(B):
        end = max(int(end_index[b]), 0)
        for l in range(L):
            pos = max(int(positions[b, l]), 0)
            lo, hi = window_keys(left, right, chunk, pos, end)
            for h in range(Hq):
                m_state, l_state = -np.inf, F32(0)
                acc = np.zeros(Dv, dtype=np.float32)
                for t in range(lo, hi):
                    dot = F32(0)
                    for i in range(Dk):
                        dot = F32(dot + q[b, l, h, i] * k[b, t, h // g, i])
                    logit = F32(dot * F32(scale))
                    if soft_cap > 0:
                        logit = F32(float(F32(soft_cap)) * np.tanh(float(F32(logit / F32(soft_cap)))))
                    m_new = max(m_state, logit)
                    rescale = F32(0) if m_state == -np.inf else F32(np.exp(float(F32(m_state - m_new))))
                    p_new = F32(np.exp(float(F32(logit - m_new))))
                    acc = acc * rescale + v[b, t, h // g] * p_new
                    l_state = F32(l_state * rescale + p_new)
                    m_state = m_new
                if l_state > 0:
                    acc = acc * F32(F32(1.0) / l_state)
                out[b, l, h] = acc
    return out


def gqa_case_f32():
    """src/aion/backend/cpu/test_cpu_backend.zig:4906-4950: B=1 L=2 Hq=4 Hkv=2 T=6 Dk=3 Dv=2."""
    B, L, Hq, Hkv, T, Dk, Dv = 1, 2, 4, 2, 6, 3, 2
    q = (np.array([(i % 17) - 8 for i in range(B * L * Hq * Dk)], dtype=np.float32) * F32(0.07)).reshape(B, L, Hq, Dk)
    k = (np.array([(i % 19) - 9 for i in range(B * T * Hkv * Dk)], dtype=np.float32) * F32(0.05)).reshape(B, T, Hkv, Dk)
    v = (np.array([(i % 23) - 11 for i in range(B * T * Hkv * Dv)], dtype=np.float32) * F32(0.06)).reshape(B, T, Hkv, Dv)
    pos = np.array([[4, 5]], dtype=np.int32)
    end = np.array([6], dtype=np.int32)
    return q, k, v, pos, end, dict(scale=0.5, left=2, right=0, chunk=0, soft_cap=1.75)


def api_attention_case():
    """src/aion/api/test_api.zig:3256-3330: zero q/k, exact window averages."""
    q = np.zeros((1, 2, 4, 2), dtype=np.float32)
    k = np.zeros((1, 6, 2, 2), dtype=np.float32)
    v = np.zeros((1, 6, 2, 1), dtype=np.float32)
    for t in range(6):
        v[0, t, 0, 0] = t + 1
        v[0, t, 1, 0] = (t + 1) * 10
    pos = np.array([[4, 5]], dtype=np.int32)
    end = np.array([6], dtype=np.int32)
    expected = np.array([4, 4, 40, 40, 5, 5, 50, 50], dtype=np.float32).reshape(1, 2, 4, 1)
    return q, k, v, pos, end, dict(scale=1.0, left=2, right=0, chunk=0, soft_cap=0.0), expected


# --- seeded synthetic inputs with the benchmark's distributions -------------------------
def synth_weights(n_rows: int, n_cols: int, seed: int = 1234) -> np.ndarray:
    return (np.random.default_rng(seed).standard_normal((n_rows, n_cols)) * 0.02).astype(np.float32)


def synth_acts(m: int, k: int, seed: int = 5678) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((m, k)).astype(np.float32)


def rel_l2(got: np.ndarray, want: np.ndarray) -> float:
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    den = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / (den if den > 0 else 1.0))
