"""float64 NumPy statement of conv2d and its gradients, plus the per-output operand norms the parity
tolerances are scaled by.  Test infrastructure only (like the rest of this package): it is never on the product path.

Every output of the three products is a dot product; the path's tolerance is stated per output as a fraction
of (norm of the one operand's terms) x (norm of the other's), exactly as for a GEMM's ||a_row|| ||b_col||:

  y [n,o,h,w]  = <window of x at (n,h,w), w[o]>                  terms: (c, kh, kw)
  dx[n,c,h,w]  = <dy values whose windows cover (h,w), w[:,c]>   terms: (o, kh, kw)
  dw[o,c,i,j]  = <dy[:,o], x shifted by tap (i,j) in channel c>  terms: (n, oh, ow)
"""
import numpy as np


def out_size(h, w, kh, kw, stride, padding):
    return (h + 2 * padding[0] - kh) // stride[0] + 1, (w + 2 * padding[1] - kw) // stride[1] + 1


def _windows(x64, kh, kw, stride, padding):
    """View [n, c, oh, ow, kh, kw] of the zero-padded input."""
    n, c, h, w = x64.shape
    oh, ow = out_size(h, w, kh, kw, stride, padding)
    xp = np.pad(x64, ((0, 0), (0, 0), (padding[0], padding[0]), (padding[1], padding[1])))
    v = np.lib.stride_tricks.sliding_window_view(xp, (kh, kw), axis=(2, 3))
    return v[:, :, ::stride[0], ::stride[1]][:, :, :oh, :ow]


def forward(x, w, bias, stride, padding):
    x64, w64 = x.astype(np.float64), w.astype(np.float64)
    win = _windows(x64, w.shape[2], w.shape[3], stride, padding)
    y = np.einsum("nchwij,ocij->nohw", win, w64, optimize=True)
    if bias is not None:
        y = y + bias.astype(np.float64)[None, :, None, None]
    return y


def grad_input(dy, w, xshape, stride, padding):
    n, c, h, wd = xshape
    co, _, kh, kw = w.shape
    oh, ow = dy.shape[2], dy.shape[3]
    dy64, w64 = dy.astype(np.float64), w.astype(np.float64)
    dxp = np.zeros((n, c, h + 2 * padding[0], wd + 2 * padding[1]))
    for i in range(kh):
        for j in range(kw):
            dxp[:, :, i:i + stride[0] * oh:stride[0], j:j + stride[1] * ow:stride[1]] += np.einsum(
                "nohw,oc->nchw", dy64, w64[:, :, i, j], optimize=True)
    return dxp[:, :, padding[0]:padding[0] + h, padding[1]:padding[1] + wd]


def grad_weight(dy, x, wshape, stride, padding):
    win = _windows(x.astype(np.float64), wshape[2], wshape[3], stride, padding)
    return np.einsum("nohw,nchwij->ocij", dy.astype(np.float64), win, optimize=True)


def forward_norms(x, w, stride, padding):
    """||window of x|| [n,1,oh,ow] times ||w[o]|| [1,o,1,1]."""
    win = _windows(x.astype(np.float64) ** 2, w.shape[2], w.shape[3], stride, padding)
    pn = np.sqrt(win.sum(axis=(1, 4, 5)))
    wn = np.linalg.norm(w.astype(np.float64).reshape(w.shape[0], -1), axis=1)
    return pn[:, None, :, :] * wn[None, :, None, None]


def grad_input_norms(dy, w, xshape, stride, padding):
    """||dy values that reach input pixel (n,h,w)|| [n,1,h,w] times ||w[:,c]|| [1,c,1,1]."""
    co, c, kh, kw = w.shape
    ones = np.ones((co, 1, kh, kw))
    dn = np.sqrt(grad_input(dy.astype(np.float64) ** 2, ones, (xshape[0], 1, xshape[2], xshape[3]), stride, padding))
    wn = np.sqrt((w.astype(np.float64) ** 2).sum(axis=(0, 2, 3)))
    return dn * wn[None, :, None, None]


def grad_weight_norms(dy, x, wshape, stride, padding):
    """||dy[:,o]|| [o,1,1,1] times ||x seen through tap (c,i,j)|| [1,c,kh,kw]."""
    dn = np.sqrt((dy.astype(np.float64) ** 2).sum(axis=(0, 2, 3)))
    ones = np.ones((dy.shape[0], 1, dy.shape[2], dy.shape[3]))
    xn = np.sqrt(grad_weight(ones, x.astype(np.float64) ** 2, (1,) + tuple(wshape[1:]), stride, padding))
    return dn[:, None, None, None] * xn


# ---- single outputs of a stride-1 layer, for sizes where the full f64 tensors are impractical.
# Each returns (value, norm product), both float64.

def sample_forward(x, w, bias, pad, n, o, h, wd):
    c, kh, kw = w.shape[1:]
    H, W = x.shape[2:]
    h0, w0 = h - pad[0], wd - pad[1]
    ys, xs = slice(max(h0, 0), min(h0 + kh, H)), slice(max(w0, 0), min(w0 + kw, W))
    a = x[n, :, ys, xs].astype(np.float64)
    b = w[o, :, ys.start - h0:ys.stop - h0, xs.start - w0:xs.stop - w0].astype(np.float64)
    v = float((a * b).sum()) + (float(bias[o]) if bias is not None else 0.0)
    return v, float(np.sqrt((a * a).sum()) * np.linalg.norm(w[o].astype(np.float64)))


def sample_grad_input(dy, w, pad, n, c, h, wd):
    co, _, kh, kw = w.shape
    OH, OW = dy.shape[2:]
    # dy[n, o, h + p - i, wd + p - j] * w[o, c, i, j]
    acc, sq = 0.0, 0.0
    for i in range(kh):
        oy = h + pad[0] - i
        if oy < 0 or oy >= OH:
            continue
        for j in range(kw):
            ox = wd + pad[1] - j
            if ox < 0 or ox >= OW:
                continue
            g = dy[n, :, oy, ox].astype(np.float64)
            acc += float((g * w[:, c, i, j].astype(np.float64)).sum())
            sq += float((g * g).sum())
    return acc, float(np.sqrt(sq) * np.sqrt((w[:, c].astype(np.float64) ** 2).sum()))


def sample_grad_weight(dy, x, pad, o, c, i, j):
    OH, OW = dy.shape[2:]
    H, W = x.shape[2:]
    # dy[n, o, oy, ox] * x[n, c, oy + i - p, ox + j - p] over the valid (oy, ox)
    oy0, oy1 = max(0, pad[0] - i), min(OH, H + pad[0] - i)
    ox0, ox1 = max(0, pad[1] - j), min(OW, W + pad[1] - j)
    g = dy[:, o, oy0:oy1, ox0:ox1].astype(np.float64)
    a = x[:, c, oy0 + i - pad[0]:oy1 + i - pad[0], ox0 + j - pad[1]:ox1 + j - pad[1]].astype(np.float64)
    return float((g * a).sum()), float(np.sqrt((dy[:, o].astype(np.float64) ** 2).sum()) * np.sqrt((a * a).sum()))
