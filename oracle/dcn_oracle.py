"""CPU restatement of (modulated) deformable 2-D convolution, forward and backward.

TEST INFRASTRUCTURE ONLY: imported by tests/ and by bench.py's CPU-baseline leg, never by the
product path.

The reference computes the operator on the NPU (kernels/deformable_conv2d/op_kernel/
deformable_conv2d.cpp:223-420: positions = base grid + offsets, floor, bilinear weights
(optionally times the mask), four-corner gather into `offset_output`, then a matmul with the
weights per group; kernels/deformable_conv2d/op_kernel/deformable_conv2d_grad.cpp for the
gradients) and pins it against mmcv's deform_conv2d / modulated_deform_conv2d on CPU
(tests/torch/test_deformable_conv2d.py:24-37, tests/torch/test_modulated_deformable_conv2d.py).
mmcv is not available here; this file restates the published algorithm (Dai et al. 2017,
Zhu et al. 2019, as implemented by mmcv and torchvision):

    p        = (ho*stride_h - pad_h + i*dil_h + dy,  wo*stride_w - pad_w + j*dil_w + dx)
    sample   = bilinear(x[n, c], p), zero for p outside (-1, H) x (-1, W), corners outside
               the image read as zero
    col      = sample * mask
    out      = sum over (c in group, i, j) of weight[co, c, i, j] * col  (+ bias)

Offset channels are ordered (deformable group, tap, (dy, dx)); mask channels (deformable
group, tap). Layout is NCHW like the Python-level API. Arithmetic is float64.
Parity pin: tests/golden/dcn_golden.npz, produced by torchvision.ops.deform_conv2d on CPU
(tests/golden/make_dcn_golden.py).
"""
import numpy as np


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def out_size(size, k, stride, pad, dil):
    return (size + 2 * pad - (dil * (k - 1) + 1)) // stride + 1


def _positions(offset, i, j, dg, K, kw, Ho, Wo, stride, padding, dilation):
    k = i * kw + j
    base_y = (np.arange(Ho) * stride[0] - padding[0] + i * dilation[0])[None, :, None]
    base_x = (np.arange(Wo) * stride[1] - padding[1] + j * dilation[1])[None, None, :]
    py = base_y + offset[:, dg * 2 * K + 2 * k]
    px = base_x + offset[:, dg * 2 * K + 2 * k + 1]
    return py, px


def _corners(py, px, H, W):
    """Floor corner, fractions, validity of the sample and of each corner."""
    valid = (py > -1) & (px > -1) & (py < H) & (px < W)
    y0 = np.floor(np.where(valid, py, 0)).astype(np.int64)
    x0 = np.floor(np.where(valid, px, 0)).astype(np.int64)
    lh = np.where(valid, py - y0, 0.0)
    lw = np.where(valid, px - x0, 0.0)
    hh, hw = 1 - lh, 1 - lw
    ok = [valid & (y0 >= 0) & (x0 >= 0), valid & (y0 >= 0) & (x0 + 1 <= W - 1),
          valid & (y0 + 1 <= H - 1) & (x0 >= 0), valid & (y0 + 1 <= H - 1) & (x0 + 1 <= W - 1)]
    ys = [y0, y0, y0 + 1, y0 + 1]
    xs = [x0, x0 + 1, x0, x0 + 1]
    wts = [hh * hw, hh * lw, lh * hw, lh * lw]
    return valid, ys, xs, ok, wts, (lh, lw, hh, hw)


def _gather(xg, ys, xs, ok, H, W):
    """xg [N, Cd, H, W] -> four arrays [N, Cd, Ho, Wo] of corner values (0 where missing)."""
    N = xg.shape[0]
    n_idx = np.arange(N)[:, None, None]
    vals = []
    for y, x, m in zip(ys, xs, ok):
        yc, xc = np.clip(y, 0, H - 1), np.clip(x, 0, W - 1)
        v = xg[n_idx, :, yc, xc]            # [N, Ho, Wo, Cd]
        v = np.where(m[..., None], v, 0.0)
        vals.append(np.moveaxis(v, -1, 1))   # [N, Cd, Ho, Wo]
    return vals


def columns(x, offset, mask, kernel, stride=1, padding=0, dilation=1, deform_groups=1):
    """cols[n, c, k, ho, wo]: the sampled (and modulated) input, the reference's offset_output."""
    x = np.asarray(x, np.float64)
    offset = np.asarray(offset, np.float64)
    stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
    kh, kw = kernel
    N, C, H, W = x.shape
    Ho, Wo = offset.shape[2], offset.shape[3]
    K, Cd = kh * kw, C // deform_groups
    cols = np.zeros((N, C, K, Ho, Wo))
    for dg in range(deform_groups):
        xg = x[:, dg * Cd:(dg + 1) * Cd]
        for i in range(kh):
            for j in range(kw):
                k = i * kw + j
                py, px = _positions(offset, i, j, dg, K, kw, Ho, Wo, stride, padding, dilation)
                _, ys, xs, ok, wts, _ = _corners(py, px, H, W)
                vals = _gather(xg, ys, xs, ok, H, W)
                s = sum(w[:, None] * v for w, v in zip(wts, vals))
                if mask is not None:
                    s = s * np.asarray(mask, np.float64)[:, dg * K + k][:, None]
                cols[:, dg * Cd:(dg + 1) * Cd, k] = s
    return cols


def forward(x, offset, mask, weight, bias=None, stride=1, padding=0, dilation=1, groups=1,
            deform_groups=1):
    """out [N, Co, Ho, Wo] (float64)."""
    weight = np.asarray(weight, np.float64)
    Co, Cg, kh, kw = weight.shape
    cols = columns(x, offset, mask, (kh, kw), stride, padding, dilation, deform_groups)
    N, C, K, Ho, Wo = cols.shape
    cg = cols.reshape(N, groups, Cg, K, Ho, Wo)
    wg = weight.reshape(groups, Co // groups, Cg, K)
    out = np.einsum("ngckhw,gock->ngohw", cg, wg).reshape(N, Co, Ho, Wo)
    if bias is not None:
        out = out + np.asarray(bias, np.float64)[None, :, None, None]
    return out


def backward(x, offset, mask, weight, grad_out, stride=1, padding=0, dilation=1, groups=1,
             deform_groups=1):
    """-> grad_x, grad_offset, grad_mask (None without mask), grad_weight, grad_bias."""
    x = np.asarray(x, np.float64)
    offset = np.asarray(offset, np.float64)
    weight = np.asarray(weight, np.float64)
    grad_out = np.asarray(grad_out, np.float64)
    if mask is not None:
        mask = np.asarray(mask, np.float64)
    stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
    Co, Cg, kh, kw = weight.shape
    N, C, H, W = x.shape
    Ho, Wo = offset.shape[2], offset.shape[3]
    K, Cd = kh * kw, C // deform_groups

    cols = columns(x, offset, mask, (kh, kw), stride, padding, dilation, deform_groups)
    go = grad_out.reshape(N, groups, Co // groups, Ho, Wo)
    wg = weight.reshape(groups, Co // groups, Cg, K)
    grad_weight = np.einsum("ngohw,ngckhw->gock", go, cols.reshape(N, groups, Cg, K, Ho, Wo))
    grad_weight = grad_weight.reshape(Co, Cg, kh, kw)
    grad_cols = np.einsum("ngohw,gock->ngckhw", go, wg).reshape(N, C, K, Ho, Wo)
    grad_bias = grad_out.sum(axis=(0, 2, 3))

    grad_x = np.zeros_like(x)
    grad_offset = np.zeros_like(offset)
    grad_mask = None if mask is None else np.zeros_like(mask)
    n_idx = np.arange(N)[:, None, None]
    for dg in range(deform_groups):
        cs = slice(dg * Cd, (dg + 1) * Cd)
        xg = x[:, cs]
        for i in range(kh):
            for j in range(kw):
                k = i * kw + j
                py, px = _positions(offset, i, j, dg, K, kw, Ho, Wo, stride, padding, dilation)
                _, ys, xs, ok, wts, (lh, lw, hh, hw) = _corners(py, px, H, W)
                v1, v2, v3, v4 = _gather(xg, ys, xs, ok, H, W)
                gc = grad_cols[:, cs, k]                         # [N, Cd, Ho, Wo]
                m = 1.0 if mask is None else mask[:, dg * K + k][:, None]
                gcm = gc * m
                if mask is not None:
                    sample = sum(w[:, None] * v for w, v in zip(wts, (v1, v2, v3, v4)))
                    grad_mask[:, dg * K + k] = (gc * sample).sum(axis=1)
                d_dy = hw[:, None] * (v3 - v1) + lw[:, None] * (v4 - v2)
                d_dx = hh[:, None] * (v2 - v1) + lh[:, None] * (v4 - v3)
                grad_offset[:, dg * 2 * K + 2 * k] = (gcm * d_dy).sum(axis=1)
                grad_offset[:, dg * 2 * K + 2 * k + 1] = (gcm * d_dx).sum(axis=1)
                for y, xx, okc, w in zip(ys, xs, ok, wts):
                    contrib = np.moveaxis(gcm * w[:, None], 1, -1)   # [N, Ho, Wo, Cd]
                    contrib = np.where(okc[..., None], contrib, 0.0)
                    yc, xc = np.clip(y, 0, H - 1), np.clip(xx, 0, W - 1)
                    flat = (np.broadcast_to(n_idx, y.shape) * H + yc) * W + xc
                    acc = np.zeros((N * H * W, Cd))
                    np.add.at(acc, flat.reshape(-1), contrib.reshape(-1, Cd))
                    grad_x[:, cs] += np.moveaxis(acc.reshape(N, H, W, Cd), -1, 1)
    return grad_x, grad_offset, grad_mask, grad_weight, grad_bias
