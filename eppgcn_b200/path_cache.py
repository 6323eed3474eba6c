"""Prepared execution paths on disk.

The preparation (one ``mask_forward`` per layer, compaction, part splitting)
depends only on the graph, the train mask, the layer count and the part-size
rule; the reference repeats it at every start (EPPGCN/gcn_main.py:147-168).
``save`` writes what ``ours_backward`` needs per layer -- the valid prefixes of
``id`` and ``edgeList``, the closed ``partPointer``, the part size and count --
under a fingerprint of those inputs; ``load`` returns it only when the
fingerprint matches, so a stale file is never used.
"""
from __future__ import annotations

import hashlib
import os
import zipfile

import numpy as np
import torch

FORMAT = 1


def fingerprint(row_pointers, column_index, train_mask, num_layers: int, part_size: int, backsize_mode: str,
                backsize: int) -> str:
    """SHA-256 over the CSR, the train mask and the knobs the path depends on."""
    h = hashlib.sha256()
    h.update(f"{FORMAT}|{int(num_layers)}|{int(part_size)}|{backsize_mode}|{int(backsize)}|".encode())
    for t, dtype in ((row_pointers, np.int32), (column_index, np.int32), (train_mask, np.bool_)):
        a = np.ascontiguousarray(t.detach().cpu().numpy().astype(dtype, copy=False))
        h.update(str(a.shape[0]).encode() + b"|")
        h.update(a.tobytes())
    return h.hexdigest()


def file_name(directory: str, fp: str) -> str:
    return os.path.join(directory, f"eppgcn_path_{fp[:24]}.npz")


def save(directory: str, fp: str, back_props) -> str:
    """``back_props``: per layer an object with ``id, edgeList, partPointer,
    partSize, numParts`` and ``valid_len`` (``backInputProperty`` after
    ``fillProperty``).  Written atomically."""
    os.makedirs(directory, exist_ok=True)
    arrays = {"fingerprint": np.frombuffer(fp.encode(), dtype=np.uint8), "layers": np.int64(len(back_props))}
    for i, p in enumerate(back_props):
        valid, parts = int(p.valid_len), int(p.numParts)
        arrays[f"id{i}"] = p.id[:valid].detach().cpu().numpy().astype(np.int32, copy=False)
        arrays[f"edge{i}"] = p.edgeList[:valid].detach().cpu().numpy().astype(np.int32, copy=False)
        arrays[f"ptr{i}"] = p.partPointer[:parts + 1].detach().cpu().numpy().astype(np.int32, copy=False)
        arrays[f"meta{i}"] = np.array([int(p.partSize), parts, valid], dtype=np.int64)
    path = file_name(directory, fp)
    tmp = path + f".tmp{os.getpid()}.npz"
    np.savez(tmp, **arrays)
    os.replace(tmp, path)
    return path


def load(directory: str, fp: str, device="cpu"):
    """Per layer ``dict(id, edgeList, partPointer, partSize, numParts,
    valid_len)`` with tensors on ``device``, or ``None`` when there is no
    usable file for this fingerprint."""
    path = file_name(directory, fp)
    if not os.path.exists(path):
        return None
    try:
        with np.load(path) as z:
            if bytes(z["fingerprint"]).decode() != fp:
                return None
            out = []
            for i in range(int(z["layers"])):
                part_size, parts, valid = (int(v) for v in z[f"meta{i}"])
                ids, edges, ptr = z[f"id{i}"], z[f"edge{i}"], z[f"ptr{i}"]
                if ids.shape[0] != valid or edges.shape[0] != valid or ptr.shape[0] != parts + 1:
                    return None
                if parts and (int(ptr[0]) != 0 or int(ptr[-1]) != valid):
                    return None
                out.append(dict(id=torch.from_numpy(ids.copy()).to(device),
                                edgeList=torch.from_numpy(edges.copy()).to(device),
                                partPointer=torch.from_numpy(ptr.copy()).to(device),
                                partSize=part_size, numParts=parts, valid_len=valid))
            return out
    except (OSError, KeyError, ValueError, EOFError, zipfile.BadZipFile):
        return None                                   # unreadable or damaged: prepare again
