"""Input generators the reference's own tests carry, restated so the parity tests read like them."""
import numpy as np


def pseudo(n: int, seed: int) -> np.ndarray:
    """ir/src/commonTest/.../passes/PagedAttentionTest.kt:75-81 (also KptxPagedAttentionKernelTest.kt:96-102):
    a 32-bit signed LCG, s = s*1103515245 + 12345 with wrap-around, value (((s>>>16)&0x7fff)/32768f - 0.5f)*2f."""
    out = np.empty(n, dtype=np.float32)
    s = seed & 0xFFFFFFFF
    for i in range(n):
        s = (s * 1103515245 + 12345) & 0xFFFFFFFF
        out[i] = (np.float32(((s >> 16) & 0x7FFF)) / np.float32(32768.0) - np.float32(0.5)) * np.float32(2.0)
    return out


def lcg_weights(seed: int, n: int) -> np.ndarray:
    """maestro/.../serving/ReferenceDecodeGraph.kt:71-77: s = s*1664525 + 1013904223 mod 2^32,
    w = float32((s>>>8) / 2^24) - 0.5f."""
    out = np.empty(n, dtype=np.float32)
    s = seed & 0xFFFFFFFF
    for i in range(n):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32((s >> 8) / float(1 << 24)) - np.float32(0.5)
    return out


def dense_twin(q, kc, vc, table, lens, scale, window=None):
    """PagedAttentionTest.kt:91-145 denseReference: gather the pages into a contiguous window, then plain
    attention over the live prefix in float64.  q [R,H,D], pools [P,bs,Hkv,D], table [R,M]."""
    R, H, D = q.shape
    P, bs, Hkv, _ = kc.shape
    M = table.shape[1]
    group = H // Hkv
    out = np.zeros((R, H, D), dtype=np.float32)
    for s in range(R):
        ln = int(lens[s])
        first = 0 if window is None else max(0, ln - window)
        kwin = np.concatenate([kc[table[s, b]] for b in range(M)], axis=0).astype(np.float64)  # [ctx,Hkv,D]
        vwin = np.concatenate([vc[table[s, b]] for b in range(M)], axis=0).astype(np.float64)
        for h in range(H):
            kv = h // group
            if ln - first <= 0:
                continue
            logits = (kwin[first:ln, kv] @ q[s, h].astype(np.float64)) * scale
            e = np.exp(logits - logits.max())
            p = e / e.sum()
            out[s, h] = (p[:, None] * vwin[first:ln, kv]).sum(axis=0).astype(np.float32)
    return out
