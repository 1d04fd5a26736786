"""ROIAlign and the suppression core of non-maximum suppression on the sm_100a kernels (``detection.cu``)."""
import torch

from . import lib, ptr, stream_ptr, count_launch, check
from ._util import dt


def roi_align_supported(data, rois):
    return (data.is_cuda and data.dim() == 4 and data.dtype in (torch.float32, torch.float16, torch.bfloat16)
            and rois.dim() == 2 and rois.shape[1] == 5 and rois.device == data.device and data.numel() > 0)


class _ROIAlign(torch.autograd.Function):
    @staticmethod
    def forward(ctx, data, rois, pooled, scale, sample_ratio, position_sensitive, aligned):
        data = data.contiguous()
        rois = rois.to(data.dtype).contiguous()
        N, CI, H, W = data.shape
        R = rois.shape[0]
        PH, PW = pooled
        C = CI // (PH * PW) if position_sensitive else CI
        out = torch.empty((R, C, PH, PW), dtype=data.dtype, device=data.device)
        if R:
            check(lib().mxb_roi_align_forward(dt(data), ptr(data), ptr(rois), ptr(out), R, CI, H, W, PH, PW, float(scale),
                                              int(sample_ratio), int(bool(position_sensitive)), int(bool(aligned)),
                                              stream_ptr(data.device)), 'roi_align_forward')
            count_launch(1)
        ctx.save_for_backward(rois)
        ctx.geom = (tuple(data.shape), data.dtype, pooled, scale, sample_ratio, position_sensitive, aligned)
        return out

    @staticmethod
    def backward(ctx, dout):
        rois, = ctx.saved_tensors
        shape, dtype, (PH, PW), scale, sample_ratio, position_sensitive, aligned = ctx.geom
        N, CI, H, W = shape
        ddata = torch.zeros(shape, dtype=torch.float32, device=dout.device)
        R = rois.shape[0]
        if R:
            dout = dout.to(dtype).contiguous()
            check(lib().mxb_roi_align_backward(dt(dout), ptr(dout), ptr(rois), ptr(ddata), R, CI, H, W, PH, PW, float(scale),
                                               int(sample_ratio), int(bool(position_sensitive)), int(bool(aligned)),
                                               stream_ptr(dout.device)), 'roi_align_backward')
            count_launch(1)
        return ddata.to(dtype), None, None, None, None, None, None


def roi_align(data, rois, pooled_size, spatial_scale, sample_ratio, position_sensitive, aligned):
    return _ROIAlign.apply(data, rois, tuple(int(v) for v in pooled_size), float(spatial_scale), int(sample_ratio),
                           bool(position_sensitive), bool(aligned))


def nms_keep(boxes, thresh, ids=None, max_keep=0, plus_one=False):
    """Keep flags (bool [n]) of greedy suppression over `boxes` [n, 4] (corner format, already in descending score
    order): a box is dropped when an earlier kept box overlaps it by more than `thresh` (and, with `ids`, has the
    same class).  At most `max_keep` boxes are kept when that is positive."""
    n = boxes.shape[0]
    if n == 0:
        return torch.zeros(0, dtype=torch.bool, device=boxes.device)
    L = lib()
    b = boxes.detach().float().contiguous()
    i = ids.detach().float().contiguous() if ids is not None else None
    words = L.mxb_nms_words(n)
    mask = torch.empty(n * words, dtype=torch.int64, device=boxes.device)
    keep = torch.empty(n, dtype=torch.uint8, device=boxes.device)
    check(L.mxb_nms(ptr(b), ptr(i), ptr(mask), ptr(keep), n, float(thresh), 1.0 if plus_one else 0.0, int(max_keep),
                    stream_ptr(boxes.device)), 'nms')
    count_launch(2)
    return keep.bool()
