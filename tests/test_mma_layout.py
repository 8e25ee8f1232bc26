"""CPU: index arithmetic of the warp-MMA small-batch kernel (shrew_b200/csrc/gemv_mma.cu).

The kernel permutes k inside each 64-wide block so that every lane can feed
mma.sync.m16n8k16 from one contiguous 16-byte run of codes.  This test replays the kernel's
per-lane loads, builds the A (16x16) and B (16x8) operands exactly as the PTX fragment
layout of m16n8k16 defines them (A: a0=(g, 2t..2t+1) a1=(g+8, 2t..) a2=(g, 2t+8..)
a3=(g+8, 2t+8..); B: b0=(2t..2t+1, g) b1=(2t+8.., g); D: d0,d1=(g, 2t..2t+1)
d2,d3=(g+8, 2t..2t+1), g = lane/4, t = lane%4), multiplies them, and checks the scattered
accumulators against x @ W^T — i.e. that operand slots pair the same k on both sides and
that the epilogue's (tile, block, lane, register) -> (token, channel) map is right."""
import numpy as np
import pytest

KWARPS, NB = 8, 2


def emulate(q, x, mt16, gated_up=None):
    N, K = q.shape
    M = x.shape[0]
    kchan = 8 if gated_up is not None else 8 * NB
    out = np.zeros((M, N), dtype=np.float64)
    out_up = np.zeros((M, N), dtype=np.float64)
    for cta in range((N + kchan - 1) // kchan):
        n0 = cta * kchan
        acc = np.zeros((KWARPS, mt16, NB, 32, 4))
        for warp in range(KWARPS):
            for kb in range(warp, K // 64, KWARPS):
                koff = kb * 64
                wv = np.zeros((NB, 32, 16))
                al = np.zeros((mt16, 32, 16))
                ah = np.zeros((mt16, 32, 16))
                for lane in range(32):
                    g, t = lane >> 2, lane & 3
                    for nb in range(NB):
                        n = min(n0 + (0 if gated_up is not None else nb * 8) + g, N - 1)
                        src = gated_up if (gated_up is not None and nb == 1) else q
                        wv[nb, lane] = src[n, koff + 16 * t: koff + 16 * t + 16]
                    for mt in range(mt16):
                        m = mt * 16 + g
                        if m < M:
                            al[mt, lane] = x[m, koff + 16 * t: koff + 16 * t + 16]
                        if m + 8 < M:
                            ah[mt, lane] = x[m + 8, koff + 16 * t: koff + 16 * t + 16]
                for nb in range(NB):
                    for j in range(4):
                        B = np.zeros((16, 8))
                        for lane in range(32):
                            g, t = lane >> 2, lane & 3
                            for e in range(2):
                                B[2 * t + e, g] = wv[nb, lane, 4 * j + e]          # b0
                                B[2 * t + 8 + e, g] = wv[nb, lane, 4 * j + 2 + e]  # b1
                        for mt in range(mt16):
                            A = np.zeros((16, 16))
                            for lane in range(32):
                                g, t = lane >> 2, lane & 3
                                for e in range(2):
                                    A[g, 2 * t + e] = al[mt, lane, 4 * j + e]              # a0 = al word 2j
                                    A[g + 8, 2 * t + e] = ah[mt, lane, 4 * j + e]          # a1 = ah word 2j
                                    A[g, 2 * t + 8 + e] = al[mt, lane, 4 * j + 2 + e]      # a2 = al word 2j+1
                                    A[g + 8, 2 * t + 8 + e] = ah[mt, lane, 4 * j + 2 + e]  # a3 = ah word 2j+1
                            D = A @ B
                            for lane in range(32):
                                g, t = lane >> 2, lane & 3
                                acc[warp, mt, nb, lane, 0] += D[g, 2 * t]
                                acc[warp, mt, nb, lane, 1] += D[g, 2 * t + 1]
                                acc[warp, mt, nb, lane, 2] += D[g + 8, 2 * t]
                                acc[warp, mt, nb, lane, 3] += D[g + 8, 2 * t + 1]
        red = acc.sum(axis=0)
        out_blocks = 1 if gated_up is not None else NB
        for i in range(mt16 * out_blocks * 4 * 32):
            ln, r, rest = i & 31, (i >> 5) & 3, i >> 7
            nb, mt = rest % out_blocks, rest // out_blocks
            m = mt * 16 + (ln >> 2) + (8 if (r & 2) else 0)
            n = n0 + nb * 8 + 2 * (ln & 3) + (r & 1)
            if m >= M or n >= N:
                continue
            if gated_up is not None:
                out[m, n] = red[mt, 0, ln, r]
                out_up[m, n] = red[mt, 1, ln, r]
            else:
                out[m, n] = red[mt, nb, ln, r]
    return (out, out_up) if gated_up is not None else out


@pytest.mark.parametrize("M,N,K,mt16", [(1, 16, 64, 1), (5, 40, 128, 1), (16, 35, 640, 1), (23, 24, 192, 2), (50, 17, 1024, 4)])
def test_kernel_indexing_reproduces_the_product(M, N, K, mt16):
    rng = np.random.default_rng(M * 100 + N)
    q = rng.integers(-127, 128, size=(N, K)).astype(np.float64)
    x = rng.integers(-8, 9, size=(M, K)).astype(np.float64)  # small integers: every sum is exact
    np.testing.assert_array_equal(emulate(q, x, mt16), x @ q.T)


def test_gated_blocks_pair_gate_and_up_rows():
    rng = np.random.default_rng(3)
    M, N, K = 9, 21, 256
    qg = rng.integers(-127, 128, size=(N, K)).astype(np.float64)
    qu = rng.integers(-127, 128, size=(N, K)).astype(np.float64)
    x = rng.integers(-8, 9, size=(M, K)).astype(np.float64)
    g, u = emulate(qg, x, 1, gated_up=qu)
    np.testing.assert_array_equal(g, x @ qg.T)
    np.testing.assert_array_equal(u, x @ qu.T)
