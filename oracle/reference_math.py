"""CPU restatement (numpy) of the reference's validation math. TEST INFRASTRUCTURE ONLY.

This module is the oracle that the CUDA kernels are checked against. Only tests, the smoke
check and the bench's cpu-baseline / reference arm may import it; no product code path does.

The reference (VisionSystemsInc/nervanagpu) cannot run here: its kernels are Maxwell SASS and
its host code needs PyCUDA. What it does provide is numpy code that defines the expected
results, inline in its benchmark scripts and its one unit test. Each function below follows
that code and names it:

  gemm        benchmarks/gemm_test.py:52-59, benchmarks/gemm_test2.py:52-59 (np.dot on fp32
              copies, .T for transposed operands); inputs quantised to fp16 first as
              benchmarks/batched_dot_test.py:38-40; epilogue order alpha -> relu -> + beta*C
              -> round from nervanagpu/nervanagpu.py:960-965 and
              kernels/sass/hgemm_common_128x128.sass:183-272.
  conv        benchmarks/conv_test.py:53-55 (slicable), :72 (zero pad row), :99-130
              (pixel_indices), :147-167 (the three np.dot lines); output dims
              nervanagpu/layers.py:297-301.
  pool        benchmarks/pool_test.py:45-56, :71-104 (pixel_indices), :117-140 (first-hit
              np.argmax, bprop += at the argmax, finfo.min pad row).
  elementwise nervanagpu/tests/test_tensor.py:46-57 (compute in fp32; integers np.around +
              clip; cast), mean/var per nervanagpu/nervanagpu.py:1191-1208.
  stochastic  nervanagpu/float_ew.py:126-130,181-201 and hgemm_common_128x128.sass:281-343:
  rounding    add a uniform below one target ulp to the magnitude, truncate toward zero, so
              the result is one of the two neighbours of the fp32 value.

Pinning: the reference stores no golden files and seeds nothing. Its known-answer cases (all
ones GEMM == k, all zeros == 0: kernels/C_interface/test.cu:27-55,70 and
benchmarks/gemm_test2.py:30-43; ones switches in conv_test.py:58-61) and its own unit-test
recipe are reproduced in tests/test_oracle.py; stochastic rounding has no reference test
(parity unpinned for that mode; checked by the neighbour + unbiasedness properties).
"""
from math import ceil

import numpy as np


# ---------------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------------
def gemm(A, B, a_t=False, b_t=False, alpha=1.0, beta=0.0, relu=False, C=None):
    """fp32 result of relu?(alpha * op(A) @ op(B)) + beta * C before the final rounding."""
    a = np.asarray(A, dtype=np.float32)
    b = np.asarray(B, dtype=np.float32)
    if a_t:
        a = a.T
    if b_t:
        b = b.T
    c = np.dot(a, b) * np.float32(alpha)
    if relu:
        c = np.maximum(c, np.float32(0))
    if beta != 0.0:
        c = c + np.float32(beta) * np.asarray(C, dtype=np.float32)
    return c.astype(np.float32)


def gemm_abs(A, B, a_t=False, b_t=False):
    """|op(A)| @ |op(B)|: scale of the rounding-error bound of a length-k dot product."""
    return gemm(np.abs(np.asarray(A, np.float32)), np.abs(np.asarray(B, np.float32)), a_t, b_t)


# ---------------------------------------------------------------------------------------------
# convolution
# ---------------------------------------------------------------------------------------------
class ConvDims(object):
    """Shape bookkeeping of ConvLayer (nervanagpu/layers.py:281-325)."""

    def __init__(self, N, C, K, D=1, H=1, W=1, T=1, R=1, S=1, pad_d=0, pad_h=0, pad_w=0,
                 str_d=1, str_h=1, str_w=1):
        self.N, self.C, self.K = N, C, K
        self.DHW = (D, H, W)
        self.TRS = (T, R, S)
        self.padding = (pad_d, pad_h, pad_w)
        self.strides = (str_d, str_h, str_w)
        M = int(ceil(float(D - T + 1 + 2 * pad_d) / str_d))
        P = int(ceil(float(H - R + 1 + 2 * pad_h) / str_h))
        Q = int(ceil(float(W - S + 1 + 2 * pad_w) / str_w))
        self.MPQ = (M, P, Q)
        self.dimI = (C, D, H, W, N)
        self.dimF = (C, T, R, S, K)
        self.dimO = (K, M, P, Q, N)
        self.flops = M * P * Q * K * N * C * T * R * S * 2.0


def _slicable(dim, pad=0):
    """Collapse all but the last dimension; optionally one extra padding row (conv_test.py:53-55)."""
    rows = 1
    for d in dim[:-1]:
        rows *= d
    return (rows + pad, dim[-1])


def _conv_pixel_rows(cd, mt, pr, qs):
    """Row numbers (c,z,y,x) of the collapsed input that one output pixel reads, in (c,t,r,s)
    order; out-of-image taps point at the padding row (conv_test.py:99-130)."""
    T, R, S = cd.TRS
    D, H, W = cd.DHW
    C = cd.C
    HW, DHW = H * W, D * H * W
    pad_row = C * DHW
    rows = []
    for c in range(C):
        for t in range(T):
            z = mt + t
            z_ok = 0 <= z < D
            for r in range(R):
                y = pr + r
                y_ok = z_ok and 0 <= y < H
                for s in range(S):
                    x = qs + s
                    if y_ok and 0 <= x < W:
                        rows.append(c * DHW + z * HW + y * W + x)
                    else:
                        rows.append(pad_row)
    return rows


def _conv_pixels(cd):
    M, P, Q = cd.MPQ
    pad_d, pad_h, pad_w = cd.padding
    str_d, str_h, str_w = cd.strides
    for m in range(M):
        for p in range(P):
            for q in range(Q):
                yield m, p, q, _conv_pixel_rows(cd, m * str_d - pad_d, p * str_h - pad_h, q * str_w - pad_w)


def _padded_input(cd, I):
    buf = np.zeros(_slicable(cd.dimI, 1), dtype=np.float32)
    buf[:-1, :] = np.asarray(I, dtype=np.float32).reshape(_slicable(cd.dimI))
    return buf


def conv_fprop(cd, I, F, alpha=1.0, relu=False):
    """Per-pixel loop of conv_test.py:147-161: O[:,m,p,q,:] = F2d.T @ I2d[rows]."""
    I2 = _padded_input(cd, I)
    F2 = np.asarray(F, dtype=np.float32).reshape(_slicable(cd.dimF))
    O = np.zeros(cd.dimO, dtype=np.float32)
    for m, p, q, rows in _conv_pixels(cd):
        O[:, m, p, q, :] = np.dot(F2.T, I2[rows, :])
    O *= np.float32(alpha)
    if relu:
        O = np.maximum(O, np.float32(0))
    return O


def conv_bprop(cd, F, E, alpha=1.0):
    """conv_test.py:163-164: gradI2d[rows] += F2d @ E[:,m,p,q,:]."""
    F2 = np.asarray(F, dtype=np.float32).reshape(_slicable(cd.dimF))
    E = np.asarray(E, dtype=np.float32).reshape(cd.dimO)
    B = np.zeros(_slicable(cd.dimI, 1), dtype=np.float32)
    for m, p, q, rows in _conv_pixels(cd):
        # rows of one pixel are distinct except for the shared padding row, which is dropped
        np.add.at(B, rows, np.dot(F2, E[:, m, p, q, :]))
    return (B[:-1, :] * np.float32(alpha)).reshape(cd.dimI)


def conv_update(cd, I, E, alpha=1.0):
    """conv_test.py:166-167: gradF2d += I2d[rows] @ E[:,m,p,q,:].T."""
    I2 = _padded_input(cd, I)
    E = np.asarray(E, dtype=np.float32).reshape(cd.dimO)
    U = np.zeros(_slicable(cd.dimF), dtype=np.float32)
    for m, p, q, rows in _conv_pixels(cd):
        U += np.dot(I2[rows, :], E[:, m, p, q, :].T)
    return (U * np.float32(alpha)).reshape(cd.dimF)


# Large temporaries of the vectorised variants. A timing loop that repeats the same shapes may
# switch the cache on (keep_workspaces(True)) so that the buffers are allocated, and their pages
# touched, once instead of on every call; the arithmetic is the same either way.
_WORKSPACES = None


def keep_workspaces(on):
    global _WORKSPACES
    _WORKSPACES = {} if on else None


def _workspace(tag, shape, zero=False):
    if _WORKSPACES is None:
        return np.zeros(shape, dtype=np.float32) if zero else np.empty(shape, dtype=np.float32)
    key = (tag,) + tuple(shape)
    buf = _WORKSPACES.get(key)
    if buf is None:
        buf = _WORKSPACES[key] = np.zeros(shape, dtype=np.float32)
    elif zero:
        buf.fill(0)
    return buf


def _im2col(cd, I):
    """All pixels at once: (C*T*R*S, M*P*Q*N) patch matrix, zero outside the image."""
    C, D, H, W, N = cd.dimI
    T, R, S = cd.TRS
    M, P, Q = cd.MPQ
    pad_d, pad_h, pad_w = cd.padding
    str_d, str_h, str_w = cd.strides
    Ip = _workspace("padded", (C, D + 2 * pad_d + str_d, H + 2 * pad_h + str_h, W + 2 * pad_w + str_w, N), zero=True)
    Ip[:, pad_d:pad_d + D, pad_h:pad_h + H, pad_w:pad_w + W, :] = np.asarray(I, dtype=np.float32).reshape(cd.dimI)
    col = _workspace("col", (C, T, R, S, M, P, Q, N))
    for t in range(T):
        for r in range(R):
            for s in range(S):
                col[:, t, r, s] = Ip[:, t:t + M * str_d:str_d, r:r + P * str_h:str_h, s:s + Q * str_w:str_w, :]
    return col.reshape(C * T * R * S, M * P * Q * N)


def conv_fprop_fast(cd, I, F, alpha=1.0, relu=False):
    """Vectorised variant (one matmul) for the large configurations; the same sums as
    conv_fprop in a different association order. Cross-checked against it in tests."""
    col = _im2col(cd, I)
    F2 = np.asarray(F, dtype=np.float32).reshape(_slicable(cd.dimF))
    O = np.dot(F2.T, col).reshape(cd.dimO) * np.float32(alpha)
    if relu:
        O = np.maximum(O, np.float32(0))
    return O


def conv_update_fast(cd, I, E, alpha=1.0):
    col = _im2col(cd, I)
    E2 = np.asarray(E, dtype=np.float32).reshape(cd.K, -1)
    return (np.dot(col, E2.T) * np.float32(alpha)).reshape(cd.dimF)


def conv_bprop_fast(cd, F, E, alpha=1.0):
    C, D, H, W, N = cd.dimI
    T, R, S = cd.TRS
    M, P, Q = cd.MPQ
    pad_d, pad_h, pad_w = cd.padding
    str_d, str_h, str_w = cd.strides
    F2 = np.asarray(F, dtype=np.float32).reshape(_slicable(cd.dimF))
    E2 = np.asarray(E, dtype=np.float32).reshape(cd.K, -1)
    colg = np.dot(F2, E2, out=_workspace("col", (C * T * R * S, M * P * Q * N))).reshape(C, T, R, S, M, P, Q, N)
    Bp = _workspace("padded", (C, D + 2 * pad_d + str_d, H + 2 * pad_h + str_h, W + 2 * pad_w + str_w, N), zero=True)
    for t in range(T):
        for r in range(R):
            for s in range(S):
                Bp[:, t:t + M * str_d:str_d, r:r + P * str_h:str_h, s:s + Q * str_w:str_w, :] += colg[:, t, r, s]
    return Bp[:, pad_d:pad_d + D, pad_h:pad_h + H, pad_w:pad_w + W, :] * np.float32(alpha)   # (a copy)


# ---------------------------------------------------------------------------------------------
# convolution at sampled positions (for shapes whose whole im2col matrix would not fit in memory)
# ---------------------------------------------------------------------------------------------
def conv_pixel_rows_np(cd, mt, pr, qs):
    """_conv_pixel_rows without the Python loops: the same (c,t,r,s)-ordered row numbers, taps
    outside the image pointing at the padding row (conv_test.py:99-130)."""
    T, R, S = cd.TRS
    D, H, W = cd.DHW
    C = cd.C
    z = (mt + np.arange(T))[:, None, None]
    y = (pr + np.arange(R))[None, :, None]
    x = (qs + np.arange(S))[None, None, :]
    ok = (z >= 0) & (z < D) & (y >= 0) & (y < H) & (x >= 0) & (x < W)
    rows = np.where(ok, z * (H * W) + y * W + x, -1)
    full = np.arange(C)[:, None, None, None] * (D * H * W) + rows[None]
    full = np.where(rows[None] >= 0, full, C * D * H * W)
    return full.reshape(-1)


def conv_fprop_pixels(cd, I, F, pixels, alpha=1.0, relu=False, absolute=False):
    """The per-pixel arithmetic of conv_test.py:147-161 at the output pixels `pixels`, a list of
    (m, p, q): returns an array (len(pixels), K, N) with O[:, m, p, q, :] of each. With
    `absolute` the operands are replaced by their magnitudes (scale of the rounding-error bound)."""
    I2 = _padded_input(cd, I)
    F2 = np.asarray(F, dtype=np.float32).reshape(_slicable(cd.dimF))
    if absolute:
        I2, F2 = np.abs(I2), np.abs(F2)
    pad_d, pad_h, pad_w = cd.padding
    str_d, str_h, str_w = cd.strides
    out = np.empty((len(pixels), cd.K, cd.N), dtype=np.float32)
    for i, (m, p, q) in enumerate(pixels):
        rows = conv_pixel_rows_np(cd, m * str_d - pad_d, p * str_h - pad_h, q * str_w - pad_w)
        out[i] = np.dot(F2.T, I2[rows, :])
    out *= np.float32(alpha)
    if relu:
        out = np.maximum(out, np.float32(0))
    return out


def conv_bprop_pixels(cd, F, E, positions, alpha=1.0, absolute=False):
    """Input gradient at the input positions `positions`, a list of (z, y, x): the sum that the
    scatter of conv_test.py:163-164 leaves there, gathered: every output pixel (m,p,q) and tap
    (t,r,s) with m*str_d - pad_d + t == z (and likewise y, x) adds F[:, t,r,s, :] @ E[:, m,p,q, :].
    Returns (len(positions), C, N)."""
    T, R, S = cd.TRS
    M, P, Q = cd.MPQ
    pad_d, pad_h, pad_w = cd.padding
    str_d, str_h, str_w = cd.strides
    F4 = np.asarray(F, dtype=np.float32).reshape(cd.C, T * R * S, cd.K)
    E2 = np.asarray(E, dtype=np.float32).reshape(cd.K, M * P * Q, cd.N)
    if absolute:
        F4, E2 = np.abs(F4), np.abs(E2)
    out = np.zeros((len(positions), cd.C, cd.N), dtype=np.float32)
    for i, (z, y, x) in enumerate(positions):
        taps, pix = [], []
        for t in range(T):
            mz = z + pad_d - t
            if mz < 0 or mz % str_d or mz // str_d >= M:
                continue
            for r in range(R):
                py = y + pad_h - r
                if py < 0 or py % str_h or py // str_h >= P:
                    continue
                for s in range(S):
                    qx = x + pad_w - s
                    if qx < 0 or qx % str_w or qx // str_w >= Q:
                        continue
                    taps.append((t * R + r) * S + s)
                    pix.append(((mz // str_d) * P + py // str_h) * Q + qx // str_w)
        if taps:
            Fs = F4[:, taps, :].reshape(cd.C, -1)                       # (C, taps*K)
            Es = E2[:, pix, :].transpose(1, 0, 2).reshape(-1, cd.N)     # (taps*K, N)
            out[i] = np.dot(Fs, Es)
    return out * np.float32(alpha)


def conv_update_taps(cd, I, E, taps, alpha=1.0, absolute=False, dtype=np.float32):
    """Weight gradient of the filter taps `taps`, a list of (t, r, s): the sum over all output
    pixels of conv_test.py:166-167 restricted to those taps. Returns (len(taps), C, K).
    `dtype=np.float64` sums in double precision: over millions of terms the fp32 sum of the
    reference's np.dot carries a rounding error of its own of about 1e-4 relative."""
    C, D, H, W, N = cd.dimI
    M, P, Q = cd.MPQ
    pad_d, pad_h, pad_w = cd.padding
    str_d, str_h, str_w = cd.strides
    Ip = np.zeros((C, D + 2 * pad_d + str_d, H + 2 * pad_h + str_h, W + 2 * pad_w + str_w, N), dtype=dtype)
    Ip[:, pad_d:pad_d + D, pad_h:pad_h + H, pad_w:pad_w + W, :] = np.asarray(I, dtype=dtype).reshape(cd.dimI)
    E2 = np.asarray(E, dtype=dtype).reshape(cd.K, -1)
    if absolute:
        Ip, E2 = np.abs(Ip), np.abs(E2)
    out = np.empty((len(taps), C, cd.K), dtype=dtype)
    for i, (t, r, s) in enumerate(taps):
        sl = Ip[:, t:t + M * str_d:str_d, r:r + P * str_h:str_h, s:s + Q * str_w:str_w, :].reshape(C, -1)
        out[i] = np.dot(sl, E2.T)
    return (out * dtype(alpha)).astype(np.float32)


# ---------------------------------------------------------------------------------------------
# pooling
# ---------------------------------------------------------------------------------------------
class PoolDims(object):
    """Shape bookkeeping of PoolLayer (nervanagpu/layers.py:542-584)."""

    def __init__(self, N, C, D=1, H=1, W=1, J=1, T=1, R=1, S=1, pad_j=0, pad_d=0, pad_h=0, pad_w=0,
                 str_j=None, str_d=None, str_h=None, str_w=None):
        str_j = J if str_j is None else str_j
        str_d = T if str_d is None else str_d
        str_h = R if str_h is None else str_h
        str_w = S if str_w is None else str_w
        self.N, self.C = N, C
        self.DHW = (D, H, W)
        self.JTRS = (J, T, R, S)
        self.padding = (pad_j, pad_d, pad_h, pad_w)
        self.strides = (str_j, str_d, str_h, str_w)
        K = int(ceil(float(C - J + 1 + 2 * pad_j) / str_j))
        M = int(ceil(float(D - T + 1 + 2 * pad_d) / str_d))
        P = int(ceil(float(H - R + 1 + 2 * pad_h) / str_h))
        Q = int(ceil(float(W - S + 1 + 2 * pad_w) / str_w))
        self.K = K
        self.MPQ = (M, P, Q)
        self.dimI = (C, D, H, W, N)
        self.dimO = (K, M, P, Q, N)


def _pool_pixel_rows(pd, kj, mt, pr, qs):
    C = pd.C
    J, T, R, S = pd.JTRS
    D, H, W = pd.DHW
    HW, DHW = H * W, D * H * W
    pad_row = C * DHW
    rows = []
    for j in range(J):
        c = kj + j
        c_ok = 0 <= c < C
        for t in range(T):
            z = mt + t
            z_ok = c_ok and 0 <= z < D
            for r in range(R):
                y = pr + r
                y_ok = z_ok and 0 <= y < H
                for s in range(S):
                    x = qs + s
                    rows.append(c * DHW + z * HW + y * W + x if (y_ok and 0 <= x < W) else pad_row)
    return rows


def pool_max(pd, I, E=None):
    """Max-pool forward, and backward when E is given (pool_test.py:117-140).

    Returns (O, gradI). The padding row holds finfo.min so it never wins; np.argmax returns the
    first maximum in (j,t,r,s) order. gradI accumulates E (the reference script passes its own
    output as E) in fp32, window after window in (k,m,p,q) order."""
    N = pd.N
    I2 = np.empty(_slicable(pd.dimI, 1), dtype=np.float32)
    I2[:-1, :] = np.asarray(I, dtype=np.float32).reshape(_slicable(pd.dimI))
    I2[-1, :] = np.finfo(np.float32).min
    O = np.empty(pd.dimO, dtype=np.float32)
    B = np.zeros(_slicable(pd.dimI, 1), dtype=np.float32)
    if E is not None:
        E = np.asarray(E, dtype=np.float32).reshape(pd.dimO)
    M, P, Q = pd.MPQ
    pad_j, pad_d, pad_h, pad_w = pd.padding
    str_j, str_d, str_h, str_w = pd.strides
    cols = np.arange(N)
    for k in range(pd.K):
        for m in range(M):
            for p in range(P):
                for q in range(Q):
                    rows = np.array(_pool_pixel_rows(pd, k * str_j - pad_j, m * str_d - pad_d,
                                                     p * str_h - pad_h, q * str_w - pad_w))
                    window = I2[rows, :]
                    O[k, m, p, q, :] = np.max(window, axis=0)
                    if E is not None:
                        hit = rows[np.argmax(window, axis=0)]
                        B[hit, cols] += E[k, m, p, q, :]
    gradI = B[:-1, :].reshape(pd.dimI) if E is not None else None
    return O, gradI


def pool_max_fast(pd, I, E=None):
    """pool_max for the large configurations: the same windows in the same (m,p,q) order, all
    feature maps of a window position at once. Needs windows that do not overlap along the
    feature-map axis (J == 1, or J == str_j with no padding and C a multiple of J), so that the
    order in which the maps are visited cannot change any sum. Cross-checked against pool_max."""
    J, T, R, S = pd.JTRS
    C, D, H, W, N = pd.dimI
    pad_j, pad_d, pad_h, pad_w = pd.padding
    str_j, str_d, str_h, str_w = pd.strides
    assert (J == 1 and str_j == 1 and pad_j == 0) or (J == str_j and pad_j == 0 and C % J == 0)
    K = pd.K
    M, P, Q = pd.MPQ
    I6 = np.asarray(I, dtype=np.float32).reshape(K, J, D, H, W, N)
    O = np.empty(pd.dimO, dtype=np.float32)
    B = np.zeros((K, J, D, H, W, N), dtype=np.float32) if E is not None else None
    if E is not None:
        E = np.asarray(E, dtype=np.float32).reshape(pd.dimO)
    kk = np.arange(K)[:, None]
    nn = np.arange(N)[None, :]
    for m in range(M):
        z0, z1 = max(m * str_d - pad_d, 0), min(m * str_d - pad_d + T, D)
        for p in range(P):
            y0, y1 = max(p * str_h - pad_h, 0), min(p * str_h - pad_h + R, H)
            for q in range(Q):
                x0, x1 = max(q * str_w - pad_w, 0), min(q * str_w - pad_w + S, W)
                tz, ty, tx = z1 - z0, y1 - y0, x1 - x0
                win = I6[:, :, z0:z1, y0:y1, x0:x1, :].reshape(K, J * tz * ty * tx, N)
                if win.shape[1] == 0:
                    O[:, m, p, q, :] = np.finfo(np.float32).min
                    continue
                O[:, m, p, q, :] = win.max(axis=1)
                if E is not None:
                    hit = win.argmax(axis=1)                      # first maximum in (j,t,r,s) order
                    j, rem = np.divmod(hit, tz * ty * tx)
                    dz, rem = np.divmod(rem, ty * tx)
                    dy, dx = np.divmod(rem, tx)
                    B[kk, j, z0 + dz, y0 + dy, x0 + dx, nn] += E[:, m, p, q, :]
    gradI = B.reshape(pd.dimI) if E is not None else None
    return O, gradI


def pool_avg_l2(pd, I, op, E=None):
    """Average / L2 pooling forward as the reference's numpy model defines them
    (benchmarks/pool_test.py:141-146): np.mean, and np.sqrt(np.sum(x**2)), over ALL J*T*R*S window
    positions, positions outside the tensor reading the zero padding row (pool_test.py:57-58,100-101).

    The reference has no backward pass for these ops ("bprop not implemented yet", pool_test.py:140);
    when E is given this returns the derivative of the forward definition: gradI += E / (J*T*R*S)
    for avg, gradI += E * I / O for l2 with O as the forward pass stored it (rounded to `O_dtype`
    of pd, default fp16) and nothing where O is 0. Accumulation in fp32, windows in (k,m,p,q) order.
    Returns (O, gradI)."""
    assert op in ("avg", "l2")
    I2 = np.zeros(_slicable(pd.dimI, 1), dtype=np.float32)
    I2[:-1, :] = np.asarray(I, dtype=np.float32).reshape(_slicable(pd.dimI))
    O = np.empty(pd.dimO, dtype=np.float32)
    B = np.zeros(_slicable(pd.dimI, 1), dtype=np.float32)
    if E is not None:
        E = np.asarray(E, dtype=np.float32).reshape(pd.dimO)
    out_dtype = getattr(pd, "O_dtype", np.float16)
    M, P, Q = pd.MPQ
    pad_j, pad_d, pad_h, pad_w = pd.padding
    str_j, str_d, str_h, str_w = pd.strides
    for k in range(pd.K):
        for m in range(M):
            for p in range(P):
                for q in range(Q):
                    rows = np.array(_pool_pixel_rows(pd, k * str_j - pad_j, m * str_d - pad_d,
                                                     p * str_h - pad_h, q * str_w - pad_w))
                    window = I2[rows, :]
                    if op == "avg":
                        O[k, m, p, q, :] = np.mean(window, axis=0)
                    else:
                        O[k, m, p, q, :] = np.sqrt(np.sum(window ** 2, axis=0))
                    if E is not None:
                        if op == "avg":
                            contrib = np.broadcast_to(E[k, m, p, q, :] / np.float32(len(rows)), window.shape)
                        else:
                            norm = O[k, m, p, q, :].astype(out_dtype).astype(np.float32)
                            safe = np.where(norm > 0, norm, np.float32(1))
                            contrib = np.where(norm > 0, E[k, m, p, q, :] * window / safe, np.float32(0))
                        np.add.at(B, rows, contrib.astype(np.float32))
    B[-1, :] = 0
    gradI = B[:-1, :].reshape(pd.dimI) if E is not None else None
    return O, gradI


# ---------------------------------------------------------------------------------------------
# element-wise
# ---------------------------------------------------------------------------------------------
def cast_result(x, dtype):
    """Final store of an element-wise kernel as the reference test models it
    (tests/test_tensor.py:50-53): integers round to nearest (ties to even) and saturate."""
    dtype = np.dtype(dtype)
    x = np.asarray(x, dtype=np.float32)
    if dtype.kind in "iu":
        info = np.iinfo(dtype)
        x = np.around(x).clip(info.min, info.max)
    return x.astype(dtype)


def batch_norm(A, eps=1e-3, axis=1):
    """(A - mean(A,axis)) / sqrt(var(A,axis) + eps) with population variance, the README
    expression built from NervanaGPU.mean / var (nervanagpu/nervanagpu.py:1191-1208)."""
    a = np.asarray(A, dtype=np.float32)
    mean = a.sum(axis=axis, keepdims=True, dtype=np.float32) * np.float32(1.0 / a.shape[axis])
    d = a - mean
    var = (d * d).sum(axis=axis, keepdims=True, dtype=np.float32) * np.float32(1.0 / a.shape[axis])
    return (d / np.sqrt(var + np.float32(eps))).astype(np.float32)


# ---------------------------------------------------------------------------------------------
# stochastic rounding
# ---------------------------------------------------------------------------------------------
def fp16_neighbours(x, mantissa_bits=10):
    """The two values a stochastic rounding of fp32 `x` to fp16 with `mantissa_bits` kept may
    return: truncation toward zero and the next value away from zero (equal when x is exact)."""
    x = np.asarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    drop = np.uint32(23 - mantissa_bits)
    mask = np.uint32((1 << int(drop)) - 1)
    lo_bits = bits & ~mask
    exact = (bits & mask) == 0
    hi_bits = np.where(exact, lo_bits, lo_bits + (mask + np.uint32(1)))
    lo = lo_bits.view(np.float32)
    hi = hi_bits.view(np.float32)
    # below the fp16 normal range the spacing is fixed at 2^-24 (times dropped mantissa bits)
    ulp = np.float32(2.0 ** (-24 + 10 - mantissa_bits))
    sub = np.abs(x) < np.float32(2.0 ** -14)
    mag = np.abs(x)
    lo_s = np.copysign(np.floor(mag / ulp) * ulp, x).astype(np.float32)
    hi_s = np.copysign(np.where(np.floor(mag / ulp) * ulp == mag, mag, np.floor(mag / ulp) * ulp + ulp), x).astype(np.float32)
    lo = np.where(sub, lo_s, lo)
    hi = np.where(sub, hi_s, hi)
    # truncation never produces infinity from a finite value: clamp at the largest fp16
    big = np.float32(65504.0)
    return np.clip(lo, -big, big).astype(np.float16), np.clip(hi, -big, big).astype(np.float16)
