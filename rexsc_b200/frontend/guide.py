"""Opt-in helper for the float "guide" convolutions of the reference's conv2d_generic.

The reference computes the guide of an SC layer as two convolutions of the same activation, one with the positive and
one with the negative part of the weights (utils_functional.py:1199-1200, 1210-1211):

    w_pos = weight.clamp(0, 100);  w_neg = -(weight.clamp(-100, 0))
    conv_pos_normal = F.conv2d(activation, w_pos, padding=(0, 0), stride=stride)
    conv_neg_normal = F.conv2d(activation, w_neg, padding=(0, 0), stride=stride)

:func:`guide_conv_pair` returns the same two tensors from ONE convolution with the filters stacked along the output
channels, so the activation is read once in the forward pass and once more in each backward pass instead of twice.
Using it means editing those two lines of the front end, which is why it is not part of the drop-in modules:

    conv_pos_normal, conv_neg_normal = rexsc_b200.frontend.guide.guide_conv_pair(activation, weight, stride)

Autograd flows through it as through the two-convolution form (the clamps are recomputed from ``weight``).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def guide_conv_pair(activation: torch.Tensor, weight: torch.Tensor, stride, padding=(0, 0)):
    """(F.conv2d(activation, weight.clamp(0, 100)), F.conv2d(activation, -(weight.clamp(-100, 0)))) computed by a single
    convolution.  The two results are the two halves of one tensor along the channel dimension."""
    c_out = weight.size(0)
    stacked = torch.cat([weight.clamp(0, 100), -(weight.clamp(-100, 0))], dim=0)
    if activation.dim() == 4 and activation.is_contiguous(memory_format=torch.channels_last) \
            and not activation.is_contiguous():
        stacked = stacked.contiguous(memory_format=torch.channels_last)
    out = F.conv2d(activation.to(stacked.dtype), stacked, padding=padding, stride=stride)
    return out[:, :c_out], out[:, c_out:]
