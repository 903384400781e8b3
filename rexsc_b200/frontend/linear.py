"""Opt-in replacement of the per-bit torch loop of the reference's ``linear_generic`` (utils_functional.py:955-1082).

With ``generator='lfsr'`` and shared generators (the defaults ``Linear_Or`` uses, utils_class.py:183-208) that function
simulates an SC fully-connected layer bit by bit: ``bit_length`` rounds of three elementwise LFSR steps, three
comparisons and two ``F.linear`` calls on 0/1 tensors, then a mean over the rounds.  The SC linear op of this library
computes the same counts in one call when its weight generators are seeded the way ``lfsr_init`` seeds them
(utils_functional.py:147-165: positive weights at offset 67, negative ones at 37, inputs at 0; the extension's own
linear op uses 13 for both, sc_cuda_matmul.cu:77-78):

* the quantisation precision is the stream length (``prec = bit_length``, :978-979), the LFSR the one of that length
  (``lfsr_cont``, :254-271) stepped before every comparison;
* ``value * prec > state`` on a non-integer product equals ``ceil(value * prec) > state``, the extension's rule.  The
  extension also saturates at ``prec - 1``; the torch loop does not (its weight clamp uses the default ``prec`` of 128,
  :972, its activations are not clamped), so a magnitude above ``(bit_length - 1) / bit_length`` -- which 7-bit
  operands reach only with streams shorter than 128 bits -- keeps its last stream bit there and loses it here;
* ``F.linear(a_bit, w_bit).sign()`` summed over the rounds is OR-1 accumulation, ``forward='full_bin'`` plain counting.

:func:`linear_generic_sc` returns what ``linear_generic`` returns (same guide expression for the backward pass, same
values in ``.data``) for operands up to ``(bit_length - 1) / bit_length`` in magnitude -- ``Linear_Or`` quantises both
to 7 bits before the call, so its default 128-bit streams always qualify.  Using
it means replacing the call in ``Linear_Or.forward``; the drop-in extension modules cannot do that by themselves.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops

WEIGHT_SEEDS = (67, 37)  # WEIGHT_POS_SEED, WEIGHT_NEG_SEED of utils_functional.py:147-148
_PLAIN_COUNT = 51200     # an OR-n with n above any dot-product length counts plainly
_NO_PROG_LOAD = (7, 8, 1)


def linear_generic_sc(activation: torch.Tensor, weight: torch.Tensor, bit_length: int = 128, forward: str = "full_or",
                      value_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """``linear_generic(activation, weight, bit_length=bit_length, forward=forward, generator='lfsr')`` with the SC
    part computed by ``linear_generic_general_acc``.  ``value_dtype`` is the dtype of the SC values that overwrite the
    guide's data (the reference's ``compute_type``, float16)."""
    if forward not in ("full_or", "full_bin"):
        raise ValueError("linear_generic_sc: forward must be 'full_or' or 'full_bin'")
    if activation.dim() != 2 or weight.dim() != 2:
        raise ValueError("linear_generic_sc: expected activation [B, C] and weight [Co, C]")
    bin_config = 0 if forward == "full_or" else _PLAIN_COUNT
    pos, neg = ops.linear_generic_general_acc(activation.data, weight.data, _NO_PROG_LOAD, int(bit_length), -1,
                                              bin_config, 1, False, False, weight_seeds=WEIGHT_SEEDS)
    # floating-point forward pass that guides back-propagation (utils_functional.py:1050-1061)
    w_pos = weight.clamp(0, 100)
    w_neg = -(weight.clamp(-100, 0))
    activation = activation.to(w_pos.dtype)
    if forward == "full_or":
        guide_pos = 1 - torch.exp(-F.linear(activation, w_pos))
        guide_neg = 1 - torch.exp(-F.linear(activation, w_neg))
    else:
        guide_pos = F.linear(activation, w_pos)
        guide_neg = F.linear(activation, w_neg)
    # the SC result overwrites the values (:1066-1073): mean over the rounds = count / bit_length
    guide_pos.data = (pos.to(torch.float32) / bit_length).to(value_dtype)
    guide_neg.data = (neg.to(torch.float32) / bit_length).to(value_dtype)
    return guide_pos - guide_neg
