"""The reference's CPU implementation of the path, restated. TEST INFRASTRUCTURE ONLY.

The reference checks its operator against a pure-PyTorch golden: per level,
``grid_sample`` (bilinear, zero padding, align_corners=False) of the level's
value map at ``2 * loc - 1``, multiplied by the attention weights and summed
over levels and points; gradients come from autograd
(tests/torch/test_multi_scale_deformable_attn.py:34-76). This module states the
same computation with its own tensor bookkeeping. It is the CPU baseline that
the benchmark times ("port" of the reference's CPU path) and a second,
independent checker next to the C oracle.
"""
import torch
import torch.nn.functional as F


def msda_forward(value, shapes, loc, attn):
    """value [B,K,H,D], shapes [L,2] (H,W), loc [B,Q,H,L,P,2], attn [B,Q,H,L,P] -> [B,Q,H*D]."""
    B, K, H, D = value.shape
    _, Q, _, L, P, _ = loc.shape
    sizes = [int(h) * int(w) for h, w in shapes.tolist()]
    # [B, K, H, D] -> [B*H, D, K]: one image batch entry per (batch, head)
    maps = value.permute(0, 2, 3, 1).reshape(B * H, D, K)
    # [B, Q, H, L, P, 2] -> [L, B*H, Q, P, 2] in grid_sample's [-1, 1] convention
    grids = (2.0 * loc - 1.0).permute(3, 0, 2, 1, 4, 5).reshape(L, B * H, Q, P, 2)
    sampled = []
    begin = 0
    for lvl, (h, w) in enumerate(shapes.tolist()):
        img = maps[:, :, begin:begin + sizes[lvl]].reshape(B * H, D, int(h), int(w))
        begin += sizes[lvl]
        sampled.append(F.grid_sample(img, grids[lvl], mode="bilinear", padding_mode="zeros",
                                     align_corners=False))      # [B*H, D, Q, P]
    stacked = torch.stack(sampled, dim=3)                        # [B*H, D, Q, L, P]
    wts = attn.permute(0, 2, 1, 3, 4).reshape(B * H, 1, Q, L, P)
    out = (stacked * wts).sum(dim=(3, 4))                        # [B*H, D, Q]
    return out.reshape(B, H * D, Q).transpose(1, 2).contiguous()


def msda_forward_backward(value, shapes, loc, attn, grad_out):
    """Returns (out, grad_value, grad_loc, grad_attn), all detached, in the inputs' dtype."""
    value = value.detach().clone().requires_grad_(True)
    loc = loc.detach().clone().requires_grad_(True)
    attn = attn.detach().clone().requires_grad_(True)
    out = msda_forward(value, shapes, loc, attn)
    out.backward(grad_out)
    return out.detach(), value.grad, loc.grad, attn.grad


def da_forward(feat, shapes, starts, loc, wts):
    """Deformable aggregation restated with grid_sample, independent of the C oracle; used to
    cross-check the oracle's backward through autograd.
    feat [B,F,C]; shapes [cams,scales,2] (h,w); starts [cams,scales]; loc [B,A,Pts,cams,2] (w,h)
    in (0,1); wts [B,A,Pts,cams,scales,G] -> out [B,A,C]."""
    B, Fk, C = feat.shape
    _, A, Pts, cams, scales, G = wts.shape
    inside = ((loc > 0) & (loc < 1)).all(-1)                      # [B,A,Pts,cams]
    out = feat.new_zeros(B, A, C)
    for cam in range(cams):
        grid = (2.0 * loc[:, :, :, cam] - 1.0)                     # [B,A,Pts,2]
        for sc in range(scales):
            h, w = int(shapes[cam, sc, 0]), int(shapes[cam, sc, 1])
            st = int(starts[cam, sc])
            img = feat[:, st:st + h * w].reshape(B, h, w, C).permute(0, 3, 1, 2)
            val = F.grid_sample(img, grid, mode="bilinear", padding_mode="zeros",
                                align_corners=False)                # [B,C,A,Pts]
            wt = wts[:, :, :, cam, sc]                              # [B,A,Pts,G]
            wt = wt.repeat_interleave(C // G, dim=-1).permute(0, 3, 1, 2)
            mask = inside[:, :, :, cam].unsqueeze(1).to(val.dtype)
            out = out + (val * wt * mask).sum(-1).transpose(1, 2)
    return out
