"""The index arithmetic of the two mma.sync decode kernels (``decode_splitkv_mma_kernel``,
``small_m_linear_mma_kernel`` in ``csrc/decode_sm100.cu``), restated on the host and checked against plain matrix
products: the XOR-swizzled staging of 16-byte pieces, the row addresses handed to ``ldmatrix`` (plain and
transposed), and the way the fragments are paired with the operands of ``mma.m16n8k16``. Runs without a GPU; the
numerics of the kernels themselves are covered by ``test_gpu_inference.py``."""
import numpy as np

PIECE = 8  # bf16 elements in a 16-byte piece


def stage(tile_rows, row_bytes, src):
    """cp.async staging: piece ``ch`` of row ``row`` goes to byte offset ``row * row_bytes + ((ch ^ (row & 7)) << 4)``.
    ``src (rows, cols)``; returns the shared-memory image as a dict offset -> 8 elements."""
    smem = {}
    for row in range(tile_rows):
        for ch in range(src.shape[1] // PIECE):
            smem[row * row_bytes + ((ch ^ (row & 7)) << 4)] = src[row, ch * PIECE:(ch + 1) * PIECE]
    return smem


def ldmatrix_x4(smem, lane_addr, trans=False):
    """Four 8x8 matrices; lanes 8m..8m+7 give the row addresses of matrix m. Thread (g, t) = (lane // 4, lane % 4)
    receives elements [g][2t], [g][2t+1] of every matrix (of its transpose with ``trans``). Returns ``r[lane][m]`` as
    pairs."""
    mats = [np.stack([smem[lane_addr[8 * m + i]] for i in range(8)]) for m in range(4)]
    out = {}
    for lane in range(32):
        g, t = lane // 4, lane % 4
        out[lane] = [(mt.T if trans else mt)[g, 2 * t:2 * t + 2] for mt in mats]
    return out


def mma_16816_top(acc, a0, a2, b0, b1):
    """acc[lane] = (d0, d1) of row g, columns 2t, 2t+1. A row g: a0 covers k = 2t, 2t+1, a2 covers k = 2t+8, 2t+9 (rows
    8..15 are zero); B column n = g of the giving lane: b0 covers k = 2t, 2t+1, b1 covers k = 2t+8, 2t+9."""
    A = np.zeros((16, 16))
    B = np.zeros((16, 8))
    for lane in range(32):
        g, t = lane // 4, lane % 4
        A[g, 2 * t:2 * t + 2] = a0[lane]
        A[g, 2 * t + 8:2 * t + 10] = a2[lane]
        B[2 * t:2 * t + 2, g] = b0[lane]
        B[2 * t + 8:2 * t + 10, g] = b1[lane]
    D = A @ B
    for lane in range(32):
        g, t = lane // 4, lane % 4
        acc[lane] = acc[lane] + D[g, 2 * t:2 * t + 2]


def test_attention_chunk_matches_q_kt_and_p_v():
    rng = np.random.default_rng(0)
    for D in (64, 128):
        RB = D * 2
        q = rng.integers(-3, 4, (8, D)).astype(float)
        k = rng.integers(-3, 4, (16, D)).astype(float)
        v = rng.integers(-3, 4, (16, D)).astype(float)
        kt, vt = stage(16, RB, k), stage(16, RB, v)
        # ---- S = Q K^T, two n-tiles of 8 cache rows
        s = [{lane: np.zeros(2) for lane in range(32)} for _ in range(2)]
        for ks in range(D // 16):
            a0 = {lane: q[lane // 4, 16 * ks + 2 * (lane % 4):16 * ks + 2 * (lane % 4) + 2] for lane in range(32)}
            a2 = {lane: q[lane // 4, 16 * ks + 8 + 2 * (lane % 4):16 * ks + 10 + 2 * (lane % 4)] for lane in range(32)}
            addr = {}
            for lane in range(32):
                mat, rr = lane >> 3, lane & 7
                row, ch = rr + 8 * (mat >> 1), 2 * ks + (mat & 1)
                addr[lane] = row * RB + ((ch ^ (row & 7)) << 4)
            bf = ldmatrix_x4(kt, addr)
            mma_16816_top(s[0], a0, a2, {l: bf[l][0] for l in bf}, {l: bf[l][1] for l in bf})
            mma_16816_top(s[1], a0, a2, {l: bf[l][2] for l in bf}, {l: bf[l][3] for l in bf})
        want = q @ k.T
        for nt in range(2):
            for lane in range(32):
                g, t = lane // 4, lane % 4
                assert np.array_equal(s[nt][lane], want[g, 8 * nt + 2 * t:8 * nt + 2 * t + 2])
        # ---- O = P V with P taken from the S fragments (a0: cache rows 2t, 2t+1; a2: rows 8 + 2t, +1)
        p = want  # any 8 x 16 matrix will do; use the scores themselves
        a0 = {lane: p[lane // 4, 2 * (lane % 4):2 * (lane % 4) + 2] for lane in range(32)}
        a2 = {lane: p[lane // 4, 8 + 2 * (lane % 4):10 + 2 * (lane % 4)] for lane in range(32)}
        o = [{lane: np.zeros(2) for lane in range(32)} for _ in range(D // 8)]
        for j in range(D // 16):
            addr = {}
            for lane in range(32):
                mat, rr = lane >> 3, lane & 7
                row, ch = rr + 8 * (mat & 1), 2 * j + (mat >> 1)
                addr[lane] = row * RB + ((ch ^ (row & 7)) << 4)
            bf = ldmatrix_x4(vt, addr, trans=True)
            mma_16816_top(o[2 * j], a0, a2, {l: bf[l][0] for l in bf}, {l: bf[l][1] for l in bf})
            mma_16816_top(o[2 * j + 1], a0, a2, {l: bf[l][2] for l in bf}, {l: bf[l][3] for l in bf})
        want_o = p @ v
        for j in range(D // 8):
            for lane in range(32):
                g, t = lane // 4, lane % 4
                assert np.array_equal(o[j][lane], want_o[g, 8 * j + 2 * t:8 * j + 2 * t + 2])


def test_linear_chunk_matches_x_wt():
    rng = np.random.default_rng(1)
    KC, RB = 128, 256
    x = rng.integers(-3, 4, (8, KC)).astype(float)   # eight x rows (rows >= M are zero-filled by the kernel)
    w = rng.integers(-3, 4, (16, KC)).astype(float)  # sixteen weight rows = output columns
    wt, xt = stage(16, RB, w), stage(8, RB, x)
    acc = [{lane: np.zeros(2) for lane in range(32)} for _ in range(2)]
    for ks2 in range(KC // 32):
        addr = {}
        for lane in range(32):
            mat, rr = lane >> 3, lane & 7
            ch = 4 * ks2 + mat
            addr[lane] = rr * RB + ((ch ^ (rr & 7)) << 4)
        af = ldmatrix_x4(xt, addr)
        for h in range(2):
            addr = {}
            for lane in range(32):
                mat, rr = lane >> 3, lane & 7
                row, ch = rr + 8 * (mat >> 1), 2 * (2 * ks2 + h) + (mat & 1)
                addr[lane] = row * RB + ((ch ^ (row & 7)) << 4)
            bf = ldmatrix_x4(wt, addr)
            a0, a2 = {l: af[l][2 * h] for l in af}, {l: af[l][2 * h + 1] for l in af}
            mma_16816_top(acc[0], a0, a2, {l: bf[l][0] for l in bf}, {l: bf[l][1] for l in bf})
            mma_16816_top(acc[1], a0, a2, {l: bf[l][2] for l in bf}, {l: bf[l][3] for l in bf})
    want = x @ w.T
    for nt in range(2):
        for lane in range(32):
            g, t = lane // 4, lane % 4
            assert np.array_equal(acc[nt][lane], want[g, 8 * nt + 2 * t:8 * nt + 2 * t + 2])


def test_swizzle_keeps_the_eight_rows_of_an_ldmatrix_on_different_banks():
    """The eight 16-byte rows of one 8x8 matrix must fall into eight different 16-byte bank groups of a 128-byte
    line, for every piece index, or ldmatrix serialises."""
    for row_bytes in (128, 256):
        for ch in range(row_bytes // 16):
            for base_row in (0, 8):
                groups = {((base_row + r) * row_bytes + ((ch ^ ((base_row + r) & 7)) << 4)) % 128 // 16 for r in range(8)}
                assert len(groups) == 8
