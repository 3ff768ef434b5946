"""The lane-to-element mapping of the mma.sync decode-attention kernels, checked on the CPU against an
emulation of the m16n8k16 fragment layout of the PTX ISA (lane = 4 g + tq):
  A (16x16): a0 = A[g][2tq, 2tq+1], a1 = A[g+8][same], a2 = A[g][2tq+8, 2tq+9], a3 = A[g+8][same]
  B (16x8) : b0 = B[2tq, 2tq+1][g], b1 = B[2tq+8, 2tq+9][g]
  D (16x8) : c0 = D[g][2tq], c1 = D[g][2tq+1], c2 = D[g+8][2tq], c3 = D[g+8][2tq+1]
The kernels themselves are tested on the GPU; this pins the index arithmetic they are built on."""
import numpy as np


def mma(a_regs, b_regs):
    """a_regs[lane] = four pairs, b_regs[lane] = two pairs -> per-lane (c0, c1, c2, c3)."""
    A, B = np.zeros((16, 16)), np.zeros((16, 8))
    for lane in range(32):
        g, tq = lane >> 2, lane & 3
        A[g, 2 * tq:2 * tq + 2] = a_regs[lane][0]
        A[g + 8, 2 * tq:2 * tq + 2] = a_regs[lane][1]
        A[g, 2 * tq + 8:2 * tq + 10] = a_regs[lane][2]
        A[g + 8, 2 * tq + 8:2 * tq + 10] = a_regs[lane][3]
        B[2 * tq:2 * tq + 2, g] = b_regs[lane][0]
        B[2 * tq + 8:2 * tq + 10, g] = b_regs[lane][1]
    D = A @ B
    return np.array([[D[l >> 2, 2 * (l & 3)], D[l >> 2, 2 * (l & 3) + 1],
                      D[(l >> 2) + 8, 2 * (l & 3)], D[(l >> 2) + 8, 2 * (l & 3) + 1]]
                     for l in range(32)])


def test_attention_rows_carry_high_and_low_parts():
    """flash_decode_mma_kernel: rows 0..7 of A hold the high part of q (of P), rows 8..15 the low
    part; the two halves of an accumulator add up inside one lane."""
    rng = np.random.default_rng(1)
    G, HD, KEYS = 4, 32, 16
    q = rng.standard_normal((G, HD))
    kmat = rng.standard_normal((KEYS, HD))
    qh = np.round(q * 32) / 32
    ql = q - qh
    s = np.zeros((32, 2, 4))                      # [lane][key block of 8][c0..c3]
    for ks in range(HD // 16):
        a = []
        for lane in range(32):
            g, tq = lane >> 2, lane & 3
            d0 = ks * 16 + tq * 2
            hi = qh[g] if g < G else np.zeros(HD)
            lo = ql[g] if g < G else np.zeros(HD)
            a.append([hi[d0:d0 + 2], lo[d0:d0 + 2], hi[d0 + 8:d0 + 10], lo[d0 + 8:d0 + 10]])
        for nb in range(2):                       # B = K^T: B[k = dim][n = key]
            b = []
            for lane in range(32):
                g, tq = lane >> 2, lane & 3
                key, d0 = nb * 8 + g, ks * 16 + tq * 2
                b.append([kmat[key, d0:d0 + 2], kmat[key, d0 + 8:d0 + 10]])
            s[:, nb] += mma(a, b)
    ref = q @ kmat.T
    for lane in range(32):
        g, tq = lane >> 2, lane & 3
        if g >= G:
            continue
        for nb in range(2):
            got = [s[lane, nb, 0] + s[lane, nb, 2], s[lane, nb, 1] + s[lane, nb, 3]]
            want = ref[g, nb * 8 + tq * 2: nb * 8 + tq * 2 + 2]
            assert np.abs(np.array(got) - want).max() < 1e-12


def test_decode_attention_tiles_cover_every_key_exactly_once():
    """flash_decode_mma_kernel: splits, 128-key tiles, 16 keys per warp, masks past the slice."""
    for kv_len in (1, 15, 16, 127, 128, 129, 333, 1500, 8193):
        for n_splits in (1, 4, 7, 18, 36):
            seen = np.zeros(kv_len, dtype=np.int32)
            per = (kv_len + n_splits - 1) // n_splits
            for split in range(n_splits):
                k0 = split * per
                k1 = min(kv_len, k0 + per)
                ntiles = (k1 - k0 + 127) // 128 if k1 > k0 else 0
                for t in range(ntiles):
                    row0 = k0 + t * 128
                    for warp in range(8):
                        key0 = row0 + warp * 16
                        if key0 >= k1:
                            continue
                        for e in range(16):
                            if key0 + e < k1:             # the kernel masks the others to -inf
                                seen[key0 + e] += 1
            assert (seen == 1).all(), (kv_len, n_splits)
