"""Generates the golden vectors under tests/golden/ by running the REFERENCE's
own operators (the unmodified extension built by oracle/build_ref.py) on small
seeded inputs.

  python tests/golden/make_golden.py            # CPU operators -> ref_cpu_ops.npz
  python tests/golden/make_golden.py --gpu      # on a GPU box: CUDA operators -> ref_gpu_ops.npz
  python tests/golden/make_golden.py --gpu --copy-to DIR     # ... and a copy of the file into DIR

Inputs are regenerated from seeds by ``golden_inputs()``; only the reference's
outputs are stored.  Cases stay inside the reference's valid range: at most
1023 parts per vertex, offsets below 2**24, last vertex with an edge.
"""
import os
import shutil
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.ref_loader import load_reference          # noqa: E402
from tests.helpers import degrees_of, random_csr      # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

CPU_CASES = [dict(n=60, avg_deg=3.0, seed=1, empty_frac=0.2, ps=3),
             dict(n=500, avg_deg=9.0, seed=2, hubs=2, hub_deg=400, ps=9),
             dict(n=40, avg_deg=1.0, seed=3, empty_frac=0.5, ps=1)]
GPU_CASE = dict(n=600, avg_deg=6.0, seed=7, empty_frac=0.1, hubs=2, hub_deg=500, self_loops=True)
GPU_LAYERS, GPU_PART, GPU_BACK, GPU_DIMS = 2, 6, 4, (16, 22)


def golden_inputs():
    """Seeded inputs of the GPU case: graph, degrees (both conventions), train mask, X, W per layer."""
    indptr, indices = random_csr(**GPU_CASE)
    if indptr[-1] == indptr[-2]:
        raise AssertionError("last vertex must have an edge (reference build_part quirk)")
    n = len(indptr) - 1
    rng = np.random.Generator(np.random.PCG64(123))
    train = rng.random(n) < 0.1
    x = rng.standard_normal((n, 12)).astype(np.float32)
    ws = [rng.uniform(-0.25, 0.25, (12, GPU_DIMS[0])).astype(np.float32),
          rng.uniform(-0.25, 0.25, (GPU_DIMS[0], GPU_DIMS[1])).astype(np.float32)]
    d_outs = [rng.standard_normal((n, d)).astype(np.float32) for d in GPU_DIMS]
    return dict(indptr=indptr, indices=indices, train=train, x=x, ws=ws, d_outs=d_outs,
                deg_rsqrt=degrees_of(indptr, "rsqrt"), deg_sqrt=degrees_of(indptr, "sqrt"))


def make_cpu(ref):
    out = {}
    for i, c in enumerate(CPU_CASES):
        c = dict(c)
        ps = c.pop("ps")
        indptr, _ = random_csr(**c)
        pp, p2n = ref.build_part(ps, torch.from_numpy(indptr))
        out[f"build_part_{i}_ptr"] = pp.numpy()          # float32, as the reference returns it
        out[f"build_part_{i}_node"] = p2n.numpy()
        deg = np.diff(indptr).astype(np.int32)
        out[f"ginfo_{i}"] = ref.get_ginfo(torch.from_numpy(deg), int(deg.sum())).numpy()
    np.savez_compressed(os.path.join(HERE, "ref_cpu_ops.npz"), **out)
    print("wrote ref_cpu_ops.npz", sorted(out))


def make_gpu(ref):
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = golden_inputs()
    n, e = len(g["indptr"]) - 1, len(g["indices"])
    cu = lambda a, dt=None: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    pp, p2n = ref.build_part(GPU_PART, torch.from_numpy(g["indptr"]))
    pp, p2n = pp.int().to(dev), p2n.int().to(dev)
    row, col = cu(g["indptr"]), cu(g["indices"])
    out = {}
    # preparation chain, EPPGCN/gcn_main.py:130-168
    ngh = [torch.zeros(n, dtype=torch.bool, device=dev) for _ in range(GPU_LAYERS - 1)]
    ems = [torch.full((e,), -1, dtype=torch.int32, device=dev) for _ in range(GPU_LAYERS)]
    nds = [torch.zeros(n, dtype=torch.int32, device=dev) for _ in range(GPU_LAYERS)]
    empty = torch.zeros(0, dtype=torch.bool, device=dev)
    for i in range(GPU_LAYERS):
        src = cu(g["train"]) if i == 0 else ngh[i - 1]
        dst = ngh[i] if i < GPU_LAYERS - 1 else empty
        ref.mask_forward(p2n, pp, col, src, dst, ems[GPU_LAYERS - 1 - i], nds[GPU_LAYERS - 1 - i],
                         GPU_LAYERS, i + 1, 4, 16)
    torch.cuda.synchronize()
    for i in range(GPU_LAYERS - 1):
        out[f"ngh_mask_{i}"] = ngh[i].cpu().numpy()
    paths = []
    for i in range(GPU_LAYERS):
        out[f"edge_mask_{i}"] = ems[i].cpu().numpy()
        out[f"node_degs_{i}"] = nds[i].cpu().numpy()
        ids, edges, info = ref.compact_back_edge(ems[i], col)
        valid = int(info[0].item())
        out[f"compact_id_{i}"], out[f"compact_edge_{i}"] = ids.cpu().numpy(), edges.cpu().numpy()
        out[f"valid_len_{i}"] = np.int64(valid)
        out[f"map_size_{i}"] = np.int64(ref.get_map_back_part_size(nds[i], valid))
        ppb, pinfo = ref.split_back_part(nds[i], e, GPU_BACK)
        out[f"part_pointer_{i}"] = ppb.cpu().numpy()
        out[f"num_parts_{i}"] = np.int64(int(pinfo[0].item()))
        paths.append((ids, ppb, edges, int(pinfo[0].item())))
        bb = ref.build_back_part(ems[i], col, nds[i], 0, 16)
        out[f"bbp_part_pointer_{i}"] = bb[2].cpu().numpy()
        out[f"bbp_info_{i}"] = bb[3].cpu().numpy()
    # operators, both degree conventions
    for conv in ("rsqrt", "sqrt"):
        deg = cu(g[f"deg_{conv}"])
        h = cu(g["x"])
        for i in range(GPU_LAYERS):
            w = cu(g["ws"][i])
            y = ref.forward(h, w, row, col, deg, pp, p2n, GPU_PART, min(GPU_DIMS[i], 32), 4)[0]
            out[f"forward_{conv}_{i}"] = y.cpu().numpy()
            ids, ppb, edges, nparts = paths[i]
            d_in, d_w = ref.ours_backward(cu(g["d_outs"][i]), h, w, ids, ppb, edges, deg, GPU_BACK, nparts,
                                          i + 1, 4, 16)
            out[f"ours_backward_{conv}_{i}_dinput"] = d_in.cpu().numpy()
            out[f"ours_backward_{conv}_{i}_dweight"] = d_w.cpu().numpy()
            d_in, d_w = ref.backward(cu(g["d_outs"][i]), h, w, row, col, deg, pp, p2n, GPU_PART,
                                     min(GPU_DIMS[i], 32), 4)
            out[f"backward_{conv}_{i}_dinput"] = d_in.cpu().numpy()
            h = torch.relu(y)
    torch.cuda.synchronize()
    path = os.path.join(HERE, "ref_gpu_ops.npz")
    np.savez_compressed(path, **out)
    if "--copy-to" in sys.argv:
        target = sys.argv[sys.argv.index("--copy-to") + 1]
        os.makedirs(target, exist_ok=True)
        shutil.copy(path, os.path.join(target, "ref_gpu_ops.npz"))
    print("wrote ref_gpu_ops.npz", len(out), "arrays", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    ref = load_reference()
    if ref is None:
        raise SystemExit("oracle/_ref holds no reference build: run python oracle/build_ref.py")
    make_gpu(ref) if "--gpu" in sys.argv else make_cpu(ref)
