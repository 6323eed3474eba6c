"""Autograd boundary of the GCN layer: same classes, call signatures and
return values as the reference's ``gcn_conv.py`` (EPPGCN/gcn_conv.py:7-65),
running on this package's native ``GNNAdvisor`` module.
"""
import math

import torch

from . import load_gnnadvisor
from .param import *  # noqa: F401,F403  (the reference re-exports its bags the same way)

GNNA = load_gnnadvisor()


class GNNAFunction(torch.autograd.Function):
    """``X' = Â (X W)`` with the backward restricted to the prepared path.

    forward  (EPPGCN/gcn_conv.py:9-29): calls ``GNNA.forward``; on the first
             iteration of the ``map``/``constant`` modes it also runs this
             layer's execution-path marking step.
    backward (EPPGCN/gcn_conv.py:31-39): calls ``GNNA.ours_backward`` with the
             bag filled by the preparation; gradients flow to X and W only.
    """

    @staticmethod
    def forward(ctx, X, weight, inputInfo, maskInfo, backInfo, isFirstIter, isBackModeNet):
        ctx.save_for_backward(X, weight)
        ctx.inputInfo, ctx.backInfo = inputInfo, backInfo
        ctx.partSize, ctx.dimWorker, ctx.warpPerBlock = (
            inputInfo.partSize, inputInfo.dimWorker, inputInfo.warpPerBlock)
        out = GNNA.forward(X, weight, inputInfo.row_pointers, inputInfo.column_index, inputInfo.degrees,
                           inputInfo.partPtr, inputInfo.part2Node,
                           inputInfo.partSize, inputInfo.dimWorker, inputInfo.warpPerBlock)[0]
        if isFirstIter and not isBackModeNet:
            GNNA.mask_forward(inputInfo.part2Node, inputInfo.partPtr, inputInfo.column_index,
                              maskInfo.src_mask, maskInfo.ngh_mask, maskInfo.backEdgeMask, maskInfo.node_degs,
                              maskInfo.num_layers, maskInfo.layer, maskInfo.blockx, maskInfo.blocky)
        return out

    @staticmethod
    def backward(ctx, d_output):
        X, weight = ctx.saved_tensors
        b = ctx.backInfo
        args = (d_output, X, weight, b.id, b.partPointer, b.edgeList, b.degrees, b.partSize, b.numParts, b.layer,
                b.blockx, b.blocky)
        if not ctx.needs_input_grad[0] and hasattr(GNNA, "ours_backward_weight_only"):
            # the input is the feature matrix (first layer): its gradient, an [N, Din] product the
            # reference computes regardless (EPPGCN_kernel.cu:614), is never used
            return None, GNNA.ours_backward_weight_only(*args)[1], None, None, None, None, None
        d_input, d_weight = GNNA.ours_backward(*args)
        return d_input, d_weight, None, None, None, None, None


class GCNConv(torch.nn.Module):
    """One graph convolution; ``weights`` is ``[input_dim, output_dim]`` drawn
    from U(-1/sqrt(output_dim), 1/sqrt(output_dim)) (EPPGCN/gcn_conv.py:44-49)."""

    def __init__(self, input_dim, output_dim):
        super().__init__()
        self.weights = torch.nn.Parameter(torch.empty(input_dim, output_dim))
        self.reset_parameters()

    def reset_parameters(self):
        bound = 1.0 / math.sqrt(self.weights.size(1))
        with torch.no_grad():
            self.weights.uniform_(-bound, bound)

    def print_time(self):
        GNNA.print_time()

    def clear_time(self):
        GNNA.clear_time()

    def forward(self, X, inputInfo, maskInfo, backInfo, isFirstIter, isBackModeNet):
        """X: node embeddings ``[num_nodes, input_dim]``; the three bags come
        from :mod:`eppgcn_b200.param`."""
        return GNNAFunction.apply(X, self.weights, inputInfo, maskInfo, backInfo, isFirstIter, isBackModeNet)
