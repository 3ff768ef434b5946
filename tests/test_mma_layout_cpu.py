"""The lane-to-element mappings of the two mma.sync kernels, checked on the CPU against an
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


def test_gemv_mapping_visits_every_weight_once():
    """gemv_mma_kernel: lane (g, tq) loads 16 consecutive weights of rows g and g + 8 per 64-column
    step and uses them in storage order; column 0 / 1 of B carry the high / low part of x."""
    rng = np.random.default_rng(0)
    K = 256
    W, x = rng.standard_normal((16, K)), rng.standard_normal(K)
    xh = np.round(x * 64) / 64
    xl = x - xh                                   # any exact high + low split
    acc = np.zeros((32, 4))
    for u in range(K // 64):
        def chunk(row, lane):
            k = u * 64 + (lane & 3) * 16
            return W[row, k:k + 16]
        for m in range(4):                        # MMA m: elements 4m .. 4m+3 of the lane's 16
            a, b = [], []
            for lane in range(32):
                g, tq = lane >> 2, lane & 3
                ra, rb = chunk(g, lane), chunk(g + 8, lane)
                a.append([ra[4 * m:4 * m + 2], rb[4 * m:4 * m + 2],
                          ra[4 * m + 2:4 * m + 4], rb[4 * m + 2:4 * m + 4]])
                col = xh if g == 0 else xl if g == 1 else np.zeros(K)
                xs = col[u * 64 + tq * 16: u * 64 + tq * 16 + 16]
                b.append([xs[4 * m:4 * m + 2], xs[4 * m + 2:4 * m + 4]])
            acc += mma(a, b)
    y = np.zeros(16)
    for lane in range(0, 32, 4):                  # tq == 0 holds columns 0 and 1
        y[lane >> 2] = acc[lane][0] + acc[lane][1]
        y[(lane >> 2) + 8] = acc[lane][2] + acc[lane][3]
    assert np.abs(y - W @ x).max() < 1e-12


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
