"""ctypes binding of ``libeppgcn_b200.so`` (declared in ``include/eppgcn_b200.h``).

This is the thin layer the tests and the benchmark use to drive the C-ABI
directly with torch tensors as device buffers.  There is no CPU fallback: a
missing library, or a device entry point given a non-CUDA tensor, raises.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# EPPGCN_B200_DEBUG_BOUNDS=1 selects the bounds-checking build of the library
# (``python -m eppgcn_b200.build --debug-bounds``), see eppgcn_debug_status.
DEBUG_BOUNDS = os.environ.get("EPPGCN_B200_DEBUG_BOUNDS", "") not in ("", "0")
LIB_PATH = os.path.join(_HERE, "libeppgcn_b200_debug.so" if DEBUG_BOUNDS else "libeppgcn_b200.so")

EPP_OK, EPP_ERR_BAD_ARG, EPP_ERR_CUDA, EPP_ERR_SCAN_TIMEOUT, EPP_ERR_TOO_LARGE, EPP_ERR_PEER_TIMEOUT = range(6)

_P, _I, _LL, _SZ = C.c_void_p, C.c_int, C.c_longlong, C.c_size_t

# name -> (restype, argtypes); mirrors include/eppgcn_b200.h one to one.
SIGNATURES = {
    "eppgcn_version": (_I, []),
    "eppgcn_status_string": (C.c_char_p, [_I]),
    "eppgcn_last_error": (C.c_char_p, []),
    "eppgcn_spmm_forward": (_I, [_P, _LL, _P, _LL, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "eppgcn_spmm_backward_compacted": (_I, [_P, _LL, _P, _LL, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "eppgcn_tile_plan_bytes": (_SZ, [_LL, _I, _I]),
    "eppgcn_tile_plan_from_csr": (_I, [_P, _P, _SZ, _P, _P, _I, _LL, _I, _P]),
    "eppgcn_tile_plan_from_ids": (_I, [_P, _P, _SZ, _P, _P, _LL, _I, _I, _P]),
    "eppgcn_pack_scaled_rows": (_I, [_P, _LL, _P, _LL, _P, _P, _I, _I, _P]),
    "eppgcn_tile_plan_destroy": (None, [_P]),
    "eppgcn_tile_plan_info": (_I, [_P, _P]),
    "eppgcn_spmm_tiles": (_I, [_P, _LL, _P, _LL, _P, _P, _I, _P]),
    "eppgcn_spmm_tiles_add": (_I, [_P, _LL, _P, _LL, _P, _P, _I, _P]),
    "eppgcn_debug_status": (_I, [_P, _I]),
    "eppgcn_update_scaled": (_I, [_P, _LL, _P, _LL, _P, _LL, _P, _I, _I, _I, _I, _P]),
    "eppgcn_weight_grad": (_I, [_P, _P, _LL, _P, _LL, _I, _I, _I, _P]),
    "eppgcn_weight_grad_rows": (_I, [_P, _P, _LL, _P, _LL, _P, _I, _I, _I, _P]),
    "eppgcn_tile_plan_active_rows": (_I, [_P, _P, _P]),
    "eppgcn_mask_forward": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "eppgcn_compact_scratch_bytes": (_SZ, [_I]),
    "eppgcn_compact_mask": (_I, [_P, _P, _P, _P, _I, _P, _SZ, _P, _P, _I, _P]),
    "eppgcn_compact_mask_static": (_I, [_P, _P, _P, _P, _I, _P, _P, _P]),
    "eppgcn_split_scratch_bytes": (_SZ, [_I]),
    "eppgcn_split_parts": (_I, [_P, _I, _I, _P, _I, _P, _SZ, _P, _P, _I, _P]),
    "eppgcn_build_part_scratch_bytes": (_SZ, [_I]),
    "eppgcn_build_part": (_I, [_P, _I, _I, _P, _I, _P, _I, _P, _SZ, _P, _P, _I, _P]),
    "eppgcn_count_nonzero": (_I, [_P, _I, _P, _P]),
    "eppgcn_push_rows": (_I, [_P, _LL, _P, _P, _P, _P, _LL, _I, _I, _LL, _P]),
    "eppgcn_peer_barrier": (_I, [_P, _I, _I, C.c_uint, _LL, _P, _P]),
    "eppgcn_peer_barrier_counted": (_I, [_P, _I, _I, _P, _LL, _P, _P]),
    "eppgcn_push_rows_signal": (_I, [_P, _LL, _P, _P, _P, _P, _LL, _I, _I, _I, _P, _P, _P, _P]),
    "eppgcn_bump_counter": (_I, [_P, _P]),
    "eppgcn_wait_landed": (_I, [_P, C.c_uint, _P, _LL, _P, _P]),
    "eppgcn_build_part_host": (_I, [_I, _P, _I, _P, _P, C.POINTER(_LL)]),
    "eppgcn_map_back_part_size": (_I, [_I, _I, C.POINTER(_I)]),
    "eppgcn_bucket_back_part_size": (_I, [_I, _I, C.POINTER(_I)]),
    "eppgcn_get_ginfo_host": (_I, [_P, _I, _I, _P]),
    "eppgcn_timing_enable": (_I, [_I]),
    "eppgcn_time_begin": (_I, [_P]),
    "eppgcn_time_end": (_I, [_I, _I, _I, _P]),
    "eppgcn_time_read": (_I, [_P]),
    "eppgcn_print_time": (_I, []),
    "eppgcn_clear_time": (_I, []),
}

_lib = None


class EppError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"eppgcn_b200 status {status}: {message}")
        self.status = status


def lib() -> C.CDLL:
    """Loads the library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: run `python -m eppgcn_b200.build` (there is no CPU fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int):
    if status != EPP_OK:
        l = lib()
        raise EppError(status, f"{l.eppgcn_status_string(status).decode()}: {l.eppgcn_last_error().decode()}")


def _dev(t: torch.Tensor | None, dtype, name: str):
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _row_stride(t: torch.Tensor, name: str) -> int:
    if t.dim() != 2 or not t.is_cuda or t.dtype != torch.float32 or (t.size(1) > 1 and t.stride(1) != 1):
        raise RuntimeError(f"{name} must be a 2-D fp32 CUDA tensor with unit column stride")
    return t.stride(0) if t.size(0) > 1 else max(t.stride(0), t.size(1))


def _out_rows(t: torch.Tensor, n: int, dim: int, name: str) -> int:
    """Address of an ``[n, dim]`` fp32 result whose rows may be a column block of a wider matrix."""
    _row_stride(t, name)
    if t.size(0) < n or t.size(1) != dim:
        raise RuntimeError(f"{name} must be [{n}, {dim}], got {list(t.shape)}")
    return t.data_ptr()


def update_scaled(x, w, scale=None, pad_to=8):
    """``scale[:, None] * (x @ w)`` as a view ``[N, dout]`` of a buffer whose
    row stride is ``dout`` rounded up to ``pad_to`` floats."""
    n, k = x.shape
    dout = w.size(1)
    ld = (dout + pad_to - 1) // pad_to * pad_to
    full = torch.empty(n, ld, device=x.device, dtype=torch.float32)
    check(lib().eppgcn_update_scaled(
        full.data_ptr(), ld, x.data_ptr(), _row_stride(x, "x"), _dev(w, torch.float32, "w"), dout,
        None if scale is None else _dev(scale, torch.float32, "scale"), n, k, dout, ld - dout, _stream()))
    return full[:, :dout]


def weight_grad(x, d, plan=None):
    """``x.T @ d`` for a tall ``x [N, k]`` and ``d [N, dout]``; with a tile ``plan`` only over the
    rows that have edges in it (the other rows of ``d`` are zero by construction)."""
    k, dout = x.size(1), d.size(1)
    dw = torch.empty(k, dout, device=x.device, dtype=torch.float32)
    if plan is None:
        check(lib().eppgcn_weight_grad(dw.data_ptr(), x.data_ptr(), _row_stride(x, "x"), d.data_ptr(),
                                       _row_stride(d, "d"), x.size(0), k, dout, _stream()))
        return dw
    rows, count = _P(), _I()
    check(lib().eppgcn_tile_plan_active_rows(plan._handle, C.byref(rows), C.byref(count)))
    check(lib().eppgcn_weight_grad_rows(dw.data_ptr(), x.data_ptr(), _row_stride(x, "x"), d.data_ptr(),
                                        _row_stride(d, "d"), rows, count.value, k, dout, _stream()))
    return dw


def spmm_forward(feat, row_ptr, col_idx, degrees, part_ptr, part2node, part_size=0, dim_worker=32,
                 warp_per_block=8, out=None, deg_row=None, prescaled=False):
    """``out = diag(deg_row) A diag(degrees) feat`` over the CSR; ``feat`` may
    have a padded row stride.  ``prescaled``: the rows of ``feat`` already carry
    ``degrees[col]`` and the kernel skips that gather."""
    n = row_ptr.numel() - 1
    dim = feat.size(1)
    ld = _row_stride(feat, "feat")
    if out is None:
        out = torch.empty(n, dim, device=feat.device, dtype=torch.float32)
    deg_row = degrees if deg_row is None else deg_row
    check(lib().eppgcn_spmm_forward(
        _out_rows(out, n, dim, "out"), _row_stride(out, "out"), feat.data_ptr(), ld,
        _dev(row_ptr, torch.int32, "row_ptr"), _dev(col_idx, torch.int32, "col_idx"),
        _dev(deg_row, torch.float32, "deg_row"), None if prescaled else _dev(degrees, torch.float32, "degrees"),
        _dev(part_ptr, torch.int32, "part_ptr"), _dev(part2node, torch.int32, "part2node"),
        n, dim, part2node.numel(), part_size, dim_worker, warp_per_block, _stream()))
    return out


def spmm_backward_compacted(d_out, ids, part_ptr, edge_list, degrees, num_parts, part_size=0,
                            blockx=4, blocky=16, out=None, deg_row=None, num_rows=None):
    n = d_out.size(0) if num_rows is None else num_rows
    dim = d_out.size(1)
    ld = _row_stride(d_out, "d_out")
    if out is None:
        out = torch.empty(n, dim, device=d_out.device, dtype=torch.float32)
    deg_row = degrees if deg_row is None else deg_row
    check(lib().eppgcn_spmm_backward_compacted(
        _out_rows(out, n, dim, "d_in"), _row_stride(out, "d_in"), d_out.data_ptr(), ld,
        _dev(ids, torch.int32, "ids"), _dev(part_ptr, torch.int32, "part_ptr"),
        _dev(edge_list, torch.int32, "edge_list"),
        _dev(deg_row, torch.float32, "deg_row"), _dev(degrees, torch.float32, "degrees"),
        n, dim, int(num_parts), part_size, blockx, blocky, _stream()))
    return out


class TilePlan:
    """Plan of the tiled aggregation (``eppgcn_tile_plan_*``): the rows of an edge
    list sorted into length classes, with the plan's own padded copy of the
    source ids.  Owns the device buffer and the host handle."""

    INFO = ("edges", "rows", "slots", "pieces", "nonempty_rows", "cleared_rows", "atomic_rows",
            "clears_whole_result")

    def __init__(self, handle, buf):
        self._handle, self._buf = handle, buf
        out = (_LL * 8)()
        check(lib().eppgcn_tile_plan_info(handle, out))
        self.info = dict(zip(self.INFO, [int(v) for v in out]))

    @staticmethod
    def _buffer(device, num_edges, num_rows, num_sources):
        nbytes = lib().eppgcn_tile_plan_bytes(int(num_edges), int(num_rows), int(num_sources))
        return torch.empty((nbytes + 7) // 8, dtype=torch.int64, device=device), nbytes

    @classmethod
    def from_csr(cls, row_ptr, col_idx, num_sources=None):
        """Forward plan: row ``r`` owns edges ``[row_ptr[r], row_ptr[r+1])`` of ``col_idx``;
        ``num_sources`` rows in the source matrix (default: a square graph)."""
        num_rows, num_edges = row_ptr.numel() - 1, col_idx.numel()
        num_sources = num_rows if num_sources is None else num_sources
        buf, nbytes = cls._buffer(row_ptr.device, num_edges, num_rows, num_sources)
        handle = _P()
        check(lib().eppgcn_tile_plan_from_csr(C.byref(handle), buf.data_ptr(), nbytes,
                                              _dev(row_ptr, torch.int32, "row_ptr"),
                                              _dev(col_idx, torch.int32, "col_idx"), num_rows, num_edges,
                                              int(num_sources), _stream()))
        return cls(handle, buf)

    @classmethod
    def from_ids(cls, ids, col_idx, num_edges, num_rows, num_sources=None):
        """Backward plan: ``ids[e]`` is the row and ``col_idx[e]`` the source of compacted edge ``e < num_edges``."""
        num_sources = num_rows if num_sources is None else num_sources
        buf, nbytes = cls._buffer(ids.device, num_edges, num_rows, num_sources)
        handle = _P()
        check(lib().eppgcn_tile_plan_from_ids(C.byref(handle), buf.data_ptr(), nbytes, _dev(ids, torch.int32, "ids"),
                                              _dev(col_idx, torch.int32, "col_idx"), int(num_edges), int(num_rows),
                                              int(num_sources), _stream()))
        return cls(handle, buf)

    def __del__(self):
        if getattr(self, "_handle", None) and _lib is not None:
            _lib.eppgcn_tile_plan_destroy(self._handle)
            self._handle = None


def pack_scaled_rows(x, scale, plan=None, out=None, pad_to=8):
    """``scale[:, None] * x`` into a buffer whose row stride is the width rounded up to
    ``pad_to`` floats; with ``plan`` only the rows its edges name are written."""
    n, dim = x.shape
    if out is None:
        ld = (dim + pad_to - 1) // pad_to * pad_to
        out = torch.empty(n, ld, device=x.device, dtype=torch.float32)[:, :dim]
    check(lib().eppgcn_pack_scaled_rows(out.data_ptr(), _row_stride(out, "out"), x.data_ptr(), _row_stride(x, "x"),
                                        None if scale is None else _dev(scale, torch.float32, "scale"),
                                        None if plan is None else plan._handle, n, dim, _stream()))
    return out


def debug_status(reset=True):
    """``(code, value, limit, tile)`` of the bounds-checking build: code 0 nothing found, 1 source id,
    2 row id out of range, -1 not a bounds-checking build."""
    out = (_I * 4)()
    check(lib().eppgcn_debug_status(out, 1 if reset else 0))
    return tuple(out)


def spmm_tiles(src, plan, row_scale=None, out=None):
    """``out[r] = row_scale[r] * sum_e src[col_idx[e]]`` over the rows of ``plan``;
    ``src`` rows already carry their source-side factor and may be padded."""
    n = plan.info["rows"]
    dim = src.size(1)
    ld = _row_stride(src, "src")
    if out is None:
        out = torch.empty(n, dim, device=src.device, dtype=torch.float32)
    check(lib().eppgcn_spmm_tiles(
        _out_rows(out, n, dim, "out"), _row_stride(out, "out"), src.data_ptr(), ld, plan._handle,
        None if row_scale is None else _dev(row_scale, torch.float32, "row_scale"), dim, _stream()))
    return out


def spmm_tiles_add(src, plan, row_scale, out):
    """Adds ``row_scale[r] * sum_e src[col_idx[e]]`` over the rows of ``plan`` to ``out``."""
    n = plan.info["rows"]
    dim = src.size(1)
    check(lib().eppgcn_spmm_tiles_add(
        _out_rows(out, n, dim, "out"), _row_stride(out, "out"), src.data_ptr(), _row_stride(src, "src"), plan._handle,
        None if row_scale is None else _dev(row_scale, torch.float32, "row_scale"), dim, _stream()))
    return out


def mask_forward(ids, part_ptr, edge_list, src_mask, ngh_mask, back_edge_mask, node_degs,
                 num_layers, layer, blockx=4, blocky=16, row_offset=0):
    is_last = int(layer == num_layers)
    ngh = None if (ngh_mask is None or ngh_mask.numel() == 0) else _dev(ngh_mask, torch.bool, "ngh_mask")
    check(lib().eppgcn_mask_forward(
        _dev(ids, torch.int32, "id"), _dev(part_ptr, torch.int32, "partPointer"),
        _dev(edge_list, torch.int32, "edgeList"), _dev(src_mask, torch.bool, "src_mask"), ngh,
        _dev(back_edge_mask, torch.int32, "backEdgeMask"), _dev(node_degs, torch.int32, "node_degs"),
        ids.numel(), is_last, row_offset, blockx, blocky, _stream()))


def _finish(counter: torch.Tensor) -> tuple[int, int]:
    """Reads the (result, status) pair a scan entry point left on the device."""
    vals = counter.cpu()          # synchronises with the producing stream
    if int(vals[1]) != EPP_OK:
        raise EppError(int(vals[1]), lib().eppgcn_status_string(int(vals[1])).decode())
    return int(vals[0]), int(vals[1])


def compact_mask(edge_mask, col_idx, mode=0):
    """Returns ``(id[E], edge_list[E], valid_len)``; the trailing entries are zero."""
    length = edge_mask.numel()
    dev = edge_mask.device
    out_id = torch.empty_like(edge_mask)
    out_edge = torch.empty_like(col_idx)
    nbytes = lib().eppgcn_compact_scratch_bytes(length)
    scratch = torch.empty((nbytes + 7) // 8, dtype=torch.int64, device=dev)
    counter = torch.empty(2, dtype=torch.int32, device=dev)
    check(lib().eppgcn_compact_mask(
        _dev(edge_mask, torch.int32, "edge_mask"), _dev(col_idx, torch.int32, "column_index"),
        out_id.data_ptr(), out_edge.data_ptr(), length, scratch.data_ptr(), nbytes,
        counter.data_ptr(), counter.data_ptr() + 4, mode, _stream()))
    valid, _ = _finish(counter)
    return out_id, out_edge, valid


def compact_mask_static(edge_mask, col_idx, out_id, out_edge, counter):
    """Compaction through the entry point that allocates nothing.  The caller
    owns every buffer: ``out_id``/``out_edge`` (length of the input) and
    ``counter`` (two int32: kept count, status).  Returns the kept count after
    synchronising with the stream."""
    check(lib().eppgcn_compact_mask_static(
        _dev(edge_mask, torch.int32, "edge_mask"), _dev(col_idx, torch.int32, "column_index"),
        _dev(out_id, torch.int32, "out_id"), _dev(out_edge, torch.int32, "out_edge"), edge_mask.numel(),
        _dev(counter, torch.int32, "counter"), counter.data_ptr() + 4, _stream()))
    valid, _ = _finish(counter)
    return valid


def split_parts(node_deg, num_edges, part_size, mode=0, out_len=None):
    """Returns ``(part_pointer[out_len], num_parts)``; ``out_len`` defaults to
    ``num_edges + 1`` so the closing pointer always fits."""
    n = node_deg.numel()
    dev = node_deg.device
    out_len = num_edges + 1 if out_len is None else out_len
    out = torch.empty(out_len, dtype=torch.int32, device=dev)
    nbytes = lib().eppgcn_split_scratch_bytes(n)
    scratch = torch.empty((nbytes + 7) // 8, dtype=torch.int64, device=dev)
    counter = torch.empty(2, dtype=torch.int32, device=dev)
    check(lib().eppgcn_split_parts(
        _dev(node_deg, torch.int32, "node_deg"), n, int(part_size), out.data_ptr(), out_len,
        scratch.data_ptr(), nbytes, counter.data_ptr(), counter.data_ptr() + 4, mode, _stream()))
    parts, _ = _finish(counter)
    return out, parts


def build_part_device(part_size: int, row_ptr: torch.Tensor, num_edges: int | None = None, mode=0):
    """Neighbour groups of a CSR whose row pointer lives on the device: returns
    ``(part_ptr[P+1], part2node[P])`` as int32 CUDA tensors, equal to what
    :func:`build_part` returns for the same row pointer on the host."""
    n = row_ptr.numel() - 1
    dev = row_ptr.device
    if num_edges is None:
        num_edges = int(row_ptr[-1].item())
    cap = num_edges // max(int(part_size), 1) + n + 1
    part_ptr = torch.empty(cap + 1, dtype=torch.int32, device=dev)
    part2node = torch.empty(cap, dtype=torch.int32, device=dev)
    nbytes = lib().eppgcn_build_part_scratch_bytes(n)
    scratch = torch.empty((nbytes + 7) // 8, dtype=torch.int64, device=dev)
    counter = torch.empty(2, dtype=torch.int32, device=dev)
    check(lib().eppgcn_build_part(_dev(row_ptr, torch.int32, "row_ptr"), n, int(part_size), part_ptr.data_ptr(),
                                  cap + 1, part2node.data_ptr(), cap, scratch.data_ptr(), nbytes,
                                  counter.data_ptr(), counter.data_ptr() + 4, mode, _stream()))
    parts, _ = _finish(counter)
    return part_ptr[:parts + 1].clone(), part2node[:parts].clone()


def push_rows(rows, send_idx, send_ptr, peer_base, peer_first_row, peer_ld, dim=None, start_row=0):
    """Gathers ``rows[send_idx[j]]`` and stores them into other ranks' buffers
    (``peer_base``: their addresses as mapped into this process).  ``send_ptr``,
    ``peer_base`` and ``peer_first_row`` are Python sequences of length
    ``world + 1``, ``world`` and ``world``; ``start_row`` is the send-list entry
    the kernel begins with (it wraps around)."""
    world = len(peer_base)
    dim = rows.size(1) if dim is None else dim
    sp = (_LL * (world + 1))(*[int(v) for v in send_ptr])
    pb = (_P * world)(*[int(v) if v else None for v in peer_base])
    fr = (_LL * world)(*[int(v) for v in peer_first_row])
    check(lib().eppgcn_push_rows(rows.data_ptr(), _row_stride(rows, "rows"), _dev(send_idx, torch.int32, "send_idx"),
                                 sp, pb, fr, int(peer_ld), int(dim), world, int(start_row), _stream()))


def push_rows_signal(rows, send_idx, send_ptr, peer_base, peer_first_row, peer_ld, rank, peer_landed, epoch, done,
                     dim=None):
    """:func:`push_rows` served peer by peer, each peer's word ``rank`` of its "landed" array
    (``peer_landed``: addresses as mapped into this process) set to ``epoch[0]`` once its rows are
    stored; ``epoch`` and ``done`` (16 zeroed words of scratch) are int32 device tensors."""
    world = len(peer_base)
    dim = rows.size(1) if dim is None else dim
    sp = (_LL * (world + 1))(*[int(v) for v in send_ptr])
    pb = (_P * world)(*[int(v) if v else None for v in peer_base])
    fr = (_LL * world)(*[int(v) for v in peer_first_row])
    pl = (_P * world)(*[int(v) if v else None for v in peer_landed])
    check(lib().eppgcn_push_rows_signal(rows.data_ptr(), _row_stride(rows, "rows"), _dev(send_idx, torch.int32, "send_idx"),
                                        sp, pb, fr, int(peer_ld), int(dim), world, int(rank), pl,
                                        _dev(epoch, torch.int32, "epoch"), _dev(done, torch.int32, "done"), _stream()))


def bump_counter(counter):
    """Adds one to an int32 device word, in stream order."""
    check(lib().eppgcn_bump_counter(_dev(counter, torch.int32, "counter"), _stream()))


def wait_landed(landed, owners, epoch, status, max_polls=4_000_000):
    """Makes the stream wait (bounded) until ``landed[r] >= epoch[0]`` for every rank ``r`` in ``owners``;
    int32 device tensors, see ``eppgcn_wait_landed``."""
    mask = 0
    for r in owners:
        mask |= 1 << int(r)
    check(lib().eppgcn_wait_landed(_dev(landed, torch.int32, "landed"), mask, _dev(epoch, torch.int32, "epoch"),
                                   int(max_polls), _dev(status, torch.int32, "status"), _stream()))


def peer_barrier(peer_flags, rank, value, status, max_polls=4_000_000):
    """Enqueues barrier number ``value`` over the ranks whose flag arrays
    (addresses as mapped into this process) are ``peer_flags``; ``status`` is a
    device int32 that receives ``EPP_ERR_PEER_TIMEOUT`` if a wait runs out."""
    world = len(peer_flags)
    pf = (_P * world)(*[int(v) for v in peer_flags])
    check(lib().eppgcn_peer_barrier(pf, int(rank), world, int(value) & 0xffffffff, int(max_polls),
                                    _dev(status, torch.int32, "status"), _stream()))


def peer_barrier_counted(peer_flags, rank, counter, status, max_polls=4_000_000):
    """Enqueues the next barrier of the sequence ``counter`` (a device int32 word, zero before the
    first barrier) numbers; see :func:`peer_barrier`.  Can be captured into a CUDA graph."""
    world = len(peer_flags)
    pf = (_P * world)(*[int(v) for v in peer_flags])
    check(lib().eppgcn_peer_barrier_counted(pf, int(rank), world, _dev(counter, torch.int32, "counter"), int(max_polls),
                                            _dev(status, torch.int32, "status"), _stream()))


def count_nonzero(values) -> int:
    counter = torch.empty(1, dtype=torch.int32, device=values.device)
    check(lib().eppgcn_count_nonzero(_dev(values, torch.int32, "values"), values.numel(),
                                     counter.data_ptr(), _stream()))
    return int(counter.item())


def build_part(part_size: int, indptr: torch.Tensor):
    """Host partition; ``indptr`` is a CPU int32 tensor."""
    if indptr.is_cuda or indptr.dtype != torch.int32:
        raise RuntimeError("indptr must be a CPU int32 tensor")
    indptr = indptr.contiguous()
    n = indptr.numel() - 1
    total = _LL(0)
    check(lib().eppgcn_build_part_host(part_size, indptr.data_ptr(), n, None, None, C.byref(total)))
    part_ptr = torch.empty(total.value + 1, dtype=torch.int32)
    part2node = torch.empty(total.value, dtype=torch.int32)
    check(lib().eppgcn_build_part_host(part_size, indptr.data_ptr(), n, part_ptr.data_ptr(),
                                       part2node.data_ptr(), C.byref(total)))
    return part_ptr, part2node


def map_back_part_size(valid_node: int, valid_len: int) -> int:
    v = _I(0)
    check(lib().eppgcn_map_back_part_size(valid_node, valid_len, C.byref(v)))
    return v.value


def bucket_back_part_size(valid_node: int, valid_len: int) -> int:
    v = _I(0)
    check(lib().eppgcn_bucket_back_part_size(valid_node, valid_len, C.byref(v)))
    return v.value


def get_ginfo(node_deg: torch.Tensor, valid_len: int) -> torch.Tensor:
    if node_deg.is_cuda or node_deg.dtype != torch.int32:
        raise RuntimeError("node_deg must be a CPU int32 tensor")
    node_deg = node_deg.contiguous()
    out = torch.zeros(10, dtype=torch.float32)
    check(lib().eppgcn_get_ginfo_host(node_deg.data_ptr(), node_deg.numel(), valid_len, out.data_ptr()))
    return out


def time_read() -> list[float]:
    out = (C.c_float * 11)()
    check(lib().eppgcn_time_read(out))
    return list(out)
