"""CPU restatement of EPPGCN's aggregation hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA kernels: only the tests, the smoke
check and the benchmark's CPU-baseline leg may import it.  Nothing in the
shipped package routes through it.

Parity status: the reference holds no tests, golden vectors or fixtures for
this path, so the restatement is pinned in two other ways: (1) every function
exists twice, as a pure-Python loop that follows the reference kernel line by
line (``*_loops``, small inputs) and as vectorised numpy (any size), and the
two must agree exactly; (2) on a GPU box the reference's own extension, built
unmodified from its sources into ``oracle/_ref``, is run on the same seeded
inputs inside its valid range and must agree with this file (bit-exact for
integer outputs, within the float tolerance for aggregations).

Each function cites the reference code it restates, by path inside the
reference project.
"""
from __future__ import annotations

import math

import numpy as np
import scipy.sparse as sp

RTOL = 1e-5     # float aggregations are compared with |a-b| <= ATOL + RTOL*|b|
ATOL = 1e-6


# --------------------------------------------------------------------------
# neighbour-group partition (host)                      EPPGCN.cpp:186-227
# --------------------------------------------------------------------------
def build_part(part_size: int, indptr: np.ndarray, reference_quirk: bool = False):
    """``(partPtr[P+1], part2Node[P])``: every vertex is cut into
    ``ceil(deg/part_size)`` groups of consecutive edges (EPPGCN.cpp:195-225).

    The reference writes the closing pointer ``partPtr[P]`` only while it
    handles the last vertex (EPPGCN.cpp:222-223), so a graph whose last vertex
    has no edges keeps 0 there and silently drops its final group.  The
    intended value ``indptr[N]`` is returned unless ``reference_quirk``.
    The reference returns float32 tensors (EPPGCN.cpp:205-206), exact only
    below 2**24; int32 is returned here.
    """
    if part_size < 1:
        raise ValueError("partSize must be >= 1")
    indptr = np.asarray(indptr, dtype=np.int64)
    deg = np.diff(indptr)
    nparts = (deg + part_size - 1) // part_size
    P = int(nparts.sum())
    part2node = np.repeat(np.arange(deg.shape[0], dtype=np.int64), nparts)
    first = np.zeros(deg.shape[0] + 1, dtype=np.int64)
    np.cumsum(nparts, out=first[1:])
    k = np.arange(P, dtype=np.int64) - first[part2node]
    part_ptr = np.zeros(P + 1, dtype=np.int64)
    part_ptr[:P] = indptr[part2node] + k * part_size
    if not (reference_quirk and (deg.shape[0] == 0 or deg[-1] == 0)):
        part_ptr[P] = indptr[-1]
    return part_ptr.astype(np.int32), part2node.astype(np.int32)


def build_part_loops(part_size: int, indptr, reference_quirk: bool = False):
    """Line-by-line form of EPPGCN.cpp:191-226."""
    n = len(indptr) - 1
    ptr, node = [], []
    closing = 0
    for i in range(n):
        deg = indptr[i + 1] - indptr[i]
        cnt = deg // part_size + (1 if deg % part_size else 0)
        for pid in range(cnt):
            beg = indptr[i] + pid * part_size
            end = min(beg + part_size, indptr[i + 1])
            ptr.append(beg)
            node.append(i)
            if i == n - 1 and end == indptr[i + 1]:
                closing = end
    if not reference_quirk:
        closing = indptr[n] if n >= 0 else 0
    ptr.append(closing)
    return np.asarray(ptr, dtype=np.int32), np.asarray(node, dtype=np.int32)


# --------------------------------------------------------------------------
# execution-path marking                         EPPGCN_kernel.cu:351-388
# --------------------------------------------------------------------------
def _group_edges(ids, part_pointer):
    """Edge positions covered by the groups and the row of each."""
    part_pointer = np.asarray(part_pointer, dtype=np.int64)
    P = len(ids)
    size = np.maximum(part_pointer[1:P + 1] - part_pointer[:P], 0)
    grp = np.repeat(np.arange(P, dtype=np.int64), size)
    start = np.zeros(P + 1, dtype=np.int64)
    np.cumsum(size, out=start[1:])
    pos = part_pointer[grp] + (np.arange(grp.shape[0], dtype=np.int64) - start[grp])
    return pos, np.asarray(ids, dtype=np.int64)[grp]


def mask_forward(ids, part_pointer, edge_list, src_mask, ngh_mask, back_edge_mask,
                 node_degs, num_layers: int, layer: int):
    """In place, as EPPGCN_kernel.cu:363-387: for every edge ``e`` of every
    group (row ``r``, column ``c``): when this is not the last preparation
    step and ``src_mask[r]``, mark ``ngh_mask[r]`` and ``ngh_mask[c]``; when
    ``src_mask[c]``, record ``back_edge_mask[e] = r``; ``node_degs[r]`` grows
    by the number of recorded edges.  ``ngh_mask`` is an empty array in the
    last step (EPPGCN/gcn_main.py:133) and is not touched."""
    pos, row = _group_edges(ids, part_pointer)
    col = np.asarray(edge_list, dtype=np.int64)[pos]
    if layer != num_layers:
        sel = src_mask[row]
        ngh_mask[row[sel]] = True
        ngh_mask[col[sel]] = True
    act = src_mask[col]
    back_edge_mask[pos[act]] = row[act]
    node_degs += np.bincount(row[act], minlength=node_degs.shape[0]).astype(node_degs.dtype)


def mask_forward_loops(ids, part_pointer, edge_list, src_mask, ngh_mask, back_edge_mask,
                       node_degs, num_layers: int, layer: int):
    last = layer == num_layers
    for p in range(len(ids)):
        r = int(ids[p])
        start = int(part_pointer[p])
        count = 0
        for i in range(int(part_pointer[p + 1]) - start):
            c = int(edge_list[start + i])
            if not last and src_mask[r]:
                ngh_mask[r] = True
                ngh_mask[c] = True
            if src_mask[c]:
                back_edge_mask[start + i] = r
                count += 1
        node_degs[r] += count


# --------------------------------------------------------------------------
# compaction of the marked edges          cuCompactor.cu:360-463, EPPGCN.cpp:282-296
# --------------------------------------------------------------------------
def compact_back_edge(edge_mask, column_index):
    """Stable filter of ``(edge_mask[e], column_index[e])`` over
    ``edge_mask[e] != -1`` (predicate cuCompactor.cu:367, scatter :412-416).
    Returns ``(id[E], edge_list[E], valid_len)``, both zero padded
    (EPPGCN.cpp:288-289)."""
    edge_mask = np.asarray(edge_mask)
    keep = edge_mask != -1
    n = int(keep.sum())
    ids = np.zeros_like(edge_mask)
    cols = np.zeros_like(np.asarray(column_index))
    ids[:n] = edge_mask[keep]
    cols[:n] = np.asarray(column_index)[keep]
    return ids, cols, n


def compact_back_edge_loops(edge_mask, column_index):
    ids = [0] * len(edge_mask)
    cols = [0] * len(edge_mask)
    n = 0
    for e in range(len(edge_mask)):
        if edge_mask[e] != -1:
            ids[n] = int(edge_mask[e])
            cols[n] = int(column_index[e])
            n += 1
    return np.asarray(ids, dtype=np.int32), np.asarray(cols, dtype=np.int32), n


# --------------------------------------------------------------------------
# splitting active rows into parts   cuCompactor.cu:514-619, :42-48, EPPGCN.cpp:327-346
# --------------------------------------------------------------------------
def split_back_part(node_deg, num_edges: int, part_size: int, out_len: int | None = None):
    """``(part_pointer[out_len], num_parts)``; ``out_len`` defaults to the
    reference's ``num_edges`` (EPPGCN.cpp:335-336).  Every vertex with
    ``node_deg > 0`` contributes, in vertex order, ``ceil(deg/part_size)``
    part sizes ``part_size, ..., part_size, remainder`` (cuCompactor.cu:566-572);
    ``part_pointer`` is the exclusive scan of those sizes over
    ``num_parts + 1`` entries (cuCompactor.cu:42-48), zero beyond.

    The reference counts parts per vertex in 10 bits and per warp in 11 bits
    (cuCompactor.cu:500,527,549); :func:`split_reference_valid` tells whether
    an input lies inside that range.  This function is exact for any int32
    input.  An entry that would fall at index ``out_len`` (with the
    reference's length: only when ``num_parts == num_edges``, where the
    reference writes one element past its buffer) is dropped; the operator
    module of this repository allocates ``num_edges + 1`` entries so the closing
    pointer always exists.
    """
    if part_size < 1:
        raise ValueError("back part size must be >= 1")
    deg = np.asarray(node_deg, dtype=np.int64)
    deg = np.where(deg > 0, deg, 0)
    cnt = (deg + part_size - 1) // part_size
    num_parts = int(cnt.sum())
    owner = np.repeat(np.arange(deg.shape[0], dtype=np.int64), cnt)
    first = np.zeros(deg.shape[0] + 1, dtype=np.int64)
    np.cumsum(cnt, out=first[1:])
    edge0 = np.zeros(deg.shape[0] + 1, dtype=np.int64)
    np.cumsum(deg, out=edge0[1:])
    k = np.arange(num_parts, dtype=np.int64) - first[owner]
    full = np.zeros(num_parts + 1, dtype=np.int64)
    full[:num_parts] = edge0[owner] + k * part_size
    full[num_parts] = edge0[-1]
    out_len = num_edges if out_len is None else out_len
    out = np.zeros(out_len, dtype=np.int32)
    m = min(num_parts + 1, out_len)
    out[:m] = full[:m]
    return out, num_parts


def split_back_part_loops(node_deg, num_edges: int, part_size: int):
    sizes = []
    for d in node_deg:
        d = int(d)
        if d > 0:
            cnt = (d + part_size - 1) // part_size
            for i in range(cnt):
                sizes.append(d - i * part_size if i + 1 == cnt else part_size)
    num_parts = len(sizes)
    out = [0] * num_edges
    run = 0
    for j in range(num_parts + 1):
        if j < num_edges:
            out[j] = run
        if j < num_parts:
            run += sizes[j]
    return np.asarray(out, dtype=np.int32), num_parts


def split_reference_valid(node_deg, part_size: int) -> bool:
    """True when the reference's bit-sliced counters cannot overflow:
    at most 1023 parts per vertex and at most 2047 per 32 consecutive
    vertices (cuCompactor.cu:500,527,549)."""
    deg = np.maximum(np.asarray(node_deg, dtype=np.int64), 0)
    cnt = (deg + part_size - 1) // part_size
    if cnt.size == 0:
        return True
    if cnt.max() > 1023:
        return False
    pad = (-cnt.size) % 32
    warp = np.concatenate([cnt, np.zeros(pad, dtype=np.int64)]).reshape(-1, 32).sum(1)
    return bool(warp.max() <= 2047)


def count_nonzero(node_deg) -> int:
    """cuCompactor.cu:638-678."""
    return int(np.count_nonzero(np.asarray(node_deg)))


def _c_round(x: float) -> int:
    return int(math.copysign(math.floor(abs(x) + 0.5), x))


def get_map_back_part_size(node_deg, valid_len: int) -> int:
    """Linear model of EPPGCN.cpp:304-310 in double precision, C ``round``.
    The result is not clamped (it goes non-positive on large graphs); callers
    clamp."""
    valid_node = count_nonzero(node_deg)
    if valid_node == 0:
        raise ZeroDivisionError("no active vertex")
    valid_degree = 1.0 * valid_len / valid_node
    return _c_round(0.65538 + 1.67431e-5 * valid_node + -2.24342e-6 * valid_len
                    + 0.63641 * valid_degree)


def bucket_back_part_size(valid_len: int, valid_node: int) -> int:
    """Degree-bucket rule of EPPGCN.cpp:243-258 (integer average degree).
    Returns 0 for an average of 512 or more, as the reference leaves it."""
    d = valid_len // valid_node
    if d < 4:
        return 4
    if d < 16:
        return 8
    if d < 64:
        return 16
    if d < 256:
        return 32
    if d < 512:
        return 64
    return 0


def get_ginfo(node_deg, valid_len: int) -> np.ndarray:
    """Degree histogram features, EPPGCN.cpp:348-386.  The last bucket also
    receives vertices of degree 0 (the ``else`` branch at :373)."""
    deg = np.asarray(node_deg, dtype=np.int64)
    valid = int(np.count_nonzero(deg))
    edges = [(1, 5), (5, 10), (10, 20), (20, 40), (40, 80), (80, 160)]
    hist = [int(((deg >= lo) & (deg < hi)).sum()) for lo, hi in edges]
    hist.append(int(deg.shape[0] - sum(hist)))
    out = np.zeros(10, dtype=np.float32)
    out[0] = valid * 1.0 / 10000
    out[1] = valid_len * 1.0 / 10000
    out[2] = 1.0 * valid_len / valid
    for i, h in enumerate(hist):
        out[3 + i] = float(np.float32(h)) * 1.0 / valid
    return out


# --------------------------------------------------------------------------
# aggregations in float64
# --------------------------------------------------------------------------
def spmm_forward(indptr, indices, degrees, feat):
    """``out[r] = sum_e (deg[r]*deg[col[e]]) * feat[col[e]]`` over the CSR row
    (EPPGCN_kernel.cu:263-293) in float64.  ``feat`` is the post-update matrix
    ``X @ W`` (EPPGCN_kernel.cu:142)."""
    n = len(indptr) - 1
    d = np.asarray(degrees, dtype=np.float64)
    a = sp.csr_matrix((np.ones(len(indices)), np.asarray(indices), np.asarray(indptr)),
                      shape=(n, n))
    return d[:, None] * (a @ (d[:, None] * np.asarray(feat, dtype=np.float64)))


def spmm_forward_loops(indptr, indices, degrees, feat):
    n = len(indptr) - 1
    feat = np.asarray(feat, dtype=np.float64)
    out = np.zeros((n, feat.shape[1]))
    for r in range(n):
        for e in range(indptr[r], indptr[r + 1]):
            c = indices[e]
            out[r] += float(degrees[r]) * float(degrees[c]) * feat[c]
    return out


def ours_backward_aggregate(ids, part_pointer, edge_list, degrees, d_out, num_parts: int):
    """Compacted backward aggregation, EPPGCN_kernel.cu:640-668, float64:
    part ``p`` adds ``sum_e deg[r]*deg[c_e] * d_out[c_e]`` to row
    ``r = ids[part_pointer[p]]`` of a zero matrix shaped like ``d_out``."""
    d_out = np.asarray(d_out, dtype=np.float64)
    n = d_out.shape[0]
    valid = int(part_pointer[num_parts]) if num_parts > 0 else 0
    rows = np.asarray(ids[:valid], dtype=np.int64)
    cols = np.asarray(edge_list[:valid], dtype=np.int64)
    d = np.asarray(degrees, dtype=np.float64)
    a = sp.coo_matrix((d[rows] * d[cols], (rows, cols)), shape=(n, n)).tocsr()
    return a @ d_out


def ours_backward_aggregate_loops(ids, part_pointer, edge_list, degrees, d_out, num_parts: int):
    d_out = np.asarray(d_out, dtype=np.float64)
    out = np.zeros_like(d_out)
    for p in range(num_parts):
        start = int(part_pointer[p])
        r = int(ids[start])
        for i in range(int(part_pointer[p + 1]) - start):
            c = int(edge_list[start + i])
            out[r] += float(degrees[r]) * float(degrees[c]) * d_out[c]
    return out


def spmm_rows(indptr, indices, rows, feat, row_scale=None):
    """The aggregation of selected rows only, in float64: ``out[i] = row_scale[rows[i]] * sum of
    feat[c] over the edges (rows[i], c)``.  ``feat`` rows carry whatever source-side factor the
    caller folded in.  Same sums as EPPGCN_kernel.cu:263-293 for a subset of the rows; lets a
    checker look at a sample of a graph that is too large for the full product."""
    n = len(indptr) - 1
    a = sp.csr_matrix((np.ones(len(indices), dtype=np.float64), indices, indptr), shape=(n, feat.shape[0]))
    out = a[np.asarray(rows)] @ np.asarray(feat, dtype=np.float64)
    if row_scale is not None:
        out = out * np.asarray(row_scale, dtype=np.float64)[np.asarray(rows)][:, None]
    return out


def spmm_rows_from_pairs(row_ids, cols, num_rows, rows, feat, row_scale=None):
    """As :func:`spmm_rows` for an edge list given as (row id, source) pairs -- the compacted path
    ``(id[e], edgeList[e])`` of EPPGCN_kernel.cu:654-668 -- instead of a CSR."""
    a = sp.coo_matrix((np.ones(len(cols), dtype=np.float64), (np.asarray(row_ids), np.asarray(cols))),
                      shape=(num_rows, feat.shape[0])).tocsr()
    out = a[np.asarray(rows)] @ np.asarray(feat, dtype=np.float64)
    if row_scale is not None:
        out = out * np.asarray(row_scale, dtype=np.float64)[np.asarray(rows)][:, None]
    return out


def gcn_layer_forward(x, w, indptr, indices, degrees):
    """Whole ``forward`` operator (EPPGCN_kernel.cu:142-184) in float64."""
    return spmm_forward(indptr, indices, degrees,
                        np.asarray(x, dtype=np.float64) @ np.asarray(w, dtype=np.float64))


def gcn_layer_backward(d_out, x, w, ids, part_pointer, edge_list, degrees, num_parts):
    """Whole ``ours_backward`` operator (EPPGCN_kernel.cu:562-623) in float64:
    ``d' = aggregate(d_out)``, ``d_input = d' @ W.T``, ``d_weight = X.T @ d'``."""
    dp = ours_backward_aggregate(ids, part_pointer, edge_list, degrees, d_out, num_parts)
    return dp @ np.asarray(w, dtype=np.float64).T, np.asarray(x, dtype=np.float64).T @ dp, dp


# --------------------------------------------------------------------------
# the one-time preparation as the training script sequences it
# --------------------------------------------------------------------------
def prepare_execution_path(indptr, indices, train_mask, num_layers: int, part_size: int,
                           back_sizes):
    """Runs mask -> compact -> split for every layer in the order of
    EPPGCN/gcn_main.py:130-176: preparation step ``k`` (1-based) reads the
    train mask (k=1) or the previous neighbour mask, writes
    ``edge_masks[L-k]``/``node_degs[L-k]``, and feeds the backward of
    convolution ``L-k+1``.  ``back_sizes[i]`` is the backward part size of
    convolution ``i+1``.  Returns one dict per convolution."""
    n, e = len(indptr) - 1, len(indices)
    part_ptr, part2node = build_part(part_size, indptr)
    ngh = [np.zeros(n, dtype=bool) for _ in range(num_layers - 1)]
    edge_masks = [np.full(e, -1, dtype=np.int32) for _ in range(num_layers)]
    node_degs = [np.zeros(n, dtype=np.int32) for _ in range(num_layers)]
    empty = np.zeros(0, dtype=bool)
    for i in range(num_layers):
        src = np.asarray(train_mask, dtype=bool) if i == 0 else ngh[i - 1]
        dst = ngh[i] if i < num_layers - 1 else empty
        mask_forward(part2node, part_ptr, indices, src, dst,
                     edge_masks[num_layers - 1 - i], node_degs[num_layers - 1 - i],
                     num_layers, i + 1)
    out = []
    for i in range(num_layers):
        ids, cols, valid = compact_back_edge(edge_masks[i], indices)
        pp, nparts = split_back_part(node_degs[i], e, back_sizes[i], out_len=e + 1)
        out.append(dict(id=ids, edgeList=cols, valid_len=valid, partPointer=pp,
                        numParts=nparts, partSize=back_sizes[i], node_degs=node_degs[i],
                        edge_mask=edge_masks[i]))
    return out, ngh
