"""The CPU GCN path timed as the baseline: fp32 ``torch.sparse`` CSR SpMM on
all host cores.  TEST / BASELINE INFRASTRUCTURE ONLY -- nothing in the shipped
package imports this.

The reference has no CPU implementation of its CUDA operators; its README
compares against framework SpMM.  PyG / torch-sparse are not installed in
this environment, so ``torch.sparse.mm`` on a CSR tensor stands in.  The
matrix carries the edge weight ``deg[r] * deg[c]`` that the reference's
kernels compute on the fly (EPPGCN_kernel.cu:269, :660-661).
"""
import numpy as np
import torch


def normalised_csr(graph) -> torch.Tensor:
    """``diag(d) A diag(d)`` with ``d = rsqrt(row nnz)`` as a float32 CSR tensor."""
    deg = np.maximum(np.diff(graph.indptr), 1).astype(np.float32)
    d = (1.0 / np.sqrt(deg)).astype(np.float32)
    rows = np.repeat(np.arange(graph.num_nodes), np.diff(graph.indptr))
    vals = d[rows] * d[graph.indices]
    return torch.sparse_csr_tensor(torch.from_numpy(graph.indptr.astype(np.int64)),
                                   torch.from_numpy(graph.indices.astype(np.int64)),
                                   torch.from_numpy(vals), size=(graph.num_nodes, graph.num_nodes))


def aggregation_epoch(a_csr: torch.Tensor, mats):
    """The aggregations of one epoch: ``A @ M`` for every matrix handed in
    (two forward, two backward for a 2-layer GCN; the graph is symmetric, so
    the backward uses the same matrix)."""
    return [torch.sparse.mm(a_csr, m) for m in mats]


def gcn_epoch(a_csr, x, weights, y, train_mask, optimizer):
    """One full training epoch of the dense-update / sparse-aggregate GCN
    (EPPGCN/gcn_main.py:225-265) with autograd on the CPU."""
    optimizer.zero_grad()
    h = x
    for i, w in enumerate(weights):
        h = torch.sparse.mm(a_csr, h @ w)
        if i < len(weights) - 1:
            h = torch.relu(h)
    loss = torch.nn.functional.nll_loss(torch.log_softmax(h, 1)[train_mask], y[train_mask])
    loss.backward()
    optimizer.step()
    return loss
