"""Knobs and property bags of the GCN layer, attribute-compatible with the
reference's ``param.py`` (EPPGCN/param.py:6-24, :28-148, :171-200).

The reference file cannot be imported as shipped (a stray token at
EPPGCN/param.py:25 raises NameError), so the three bags and ``getBlockSize``
are provided here with the same constructor arguments and attribute names.
The CUDA kernels in this package treat ``dimWorker``, ``warpPerBlock``,
``blockx`` and ``blocky`` as hints: any legal value gives the same result.
"""
from __future__ import annotations

# (exclusive upper bound of dim, blockx, blocky)   -- EPPGCN/param.py:6-24
_BLOCK_SHAPES = ((8, 2, 32), (32, 4, 16), (96, 8, 8), (192, 16, 4), (512, 32, 2))


def getBlockSize(dim):
    """Launch shape the reference picks for the mask and backward kernels."""
    for bound, bx, by in _BLOCK_SHAPES:
        if dim < bound:
            return (bx, by)
    return (32, 2)


class inputProperty(object):
    """Forward-pass bag: CSR, degrees, neighbour groups and launch knobs."""

    MAX_warpPerBlock = 8

    def __init__(self, row_pointers=None, column_index=None, degrees=None,
                 partSize=None, dimWorker=None, warpPerBlock=None,
                 sharedMem=None, hiddenDim=None, dataset_obj=None,
                 manual_mode=True, verbose=False):
        if dataset_obj is None:
            raise ValueError("Dataset object MUST SET !!!")
        self.dataset_obj = dataset_obj
        self.row_pointers, self.column_index, self.degrees = row_pointers, column_index, degrees
        self.num_nodes = dataset_obj.num_nodes
        self.avgNodeDegree = dataset_obj.avg_degree
        self.avgEdgeSpan = dataset_obj.avg_edgeSpan
        self.inputDim = dataset_obj.num_features
        self.hiddenDim = hiddenDim

        self.partSize, self.dimWorker, self.warpPerBlock = partSize, dimWorker, warpPerBlock
        self.dimWorker_input = self.dimWorker_hidden = dimWorker
        self.warpPerBlock_input = self.warpPerBlock_hidden = warpPerBlock

        self.manual_mode, self.verbose_flag = manual_mode, verbose
        self.state_set_input = False
        self.share_memory = (100 if sharedMem is None else sharedMem) * 0.4     # KB, EPPGCN/param.py:65
        self.gap_smem = 100
        self.partPtr = self.part2Node = None

    def _log(self, text):
        if self.verbose_flag:
            print(text)

    def decider(self):
        """Same rules as EPPGCN/param.py:73-127.  The group size always
        becomes ``int(average degree)`` (:80), whatever was passed in; a graph
        with fewer edges than vertices would get 0 there, which no group
        builder accepts, so it is raised to 1 here."""
        self.partSize = max(int(self.avgNodeDegree), 1)
        ps4 = self.partSize * 4
        gap4 = self.gap_smem * 4
        est_in = self.MAX_warpPerBlock * (ps4 + self.inputDim * 4 + gap4) / 1e3
        est_hid = self.MAX_warpPerBlock * (ps4 + self.hiddenDim + gap4) / 1e3      # sic, :89
        smem_in, smem_hid = min(est_in, self.share_memory), min(est_hid, self.share_memory)
        self._log("input-layer shared memory (KB): {:.3f} -> {:.3f}".format(est_in, smem_in))
        self._log("hidden-layer shared memory (KB): {:.3f} -> {:.3f}".format(est_hid, smem_hid))
        self.warpPerBlock_input = min(int(smem_in * 1e3 / (ps4 + self.inputDim * 4)), self.MAX_warpPerBlock)
        self.warpPerBlock_hidden = min(int(smem_hid * 1e3 / (ps4 + self.hiddenDim * 4)), self.MAX_warpPerBlock)
        self.dimWorker_input = min(self.inputDim, 32)
        self.dimWorker_hidden = min(self.hiddenDim, 32)
        self._log("\n=> AUTO Decider Complete !!!\n")

    def set_input(self):
        """Switch the launch knobs to the first layer's."""
        self.dimWorker, self.warpPerBlock = self.dimWorker_input, self.warpPerBlock_input
        self.state_set_input = True
        return self

    def set_hidden(self):
        """Switch the launch knobs to the hidden layers'."""
        self.dimWorker, self.warpPerBlock = self.dimWorker_hidden, self.warpPerBlock_hidden
        self.state_set_input = False
        return self

    def print_param(self):
        if not self.verbose_flag:
            return
        tag = "{} {}".format("manual" if self.manual_mode else "auto",
                             "INPUT" if self.state_set_input else "HIDDEN")
        for key in ("partSize", "dimWorker", "warpPerBlock"):
            print("# {} {}: {}".format(tag, key, getattr(self, key)))


class maskInputProperty(object):
    """Arguments of one execution-path preparation step (EPPGCN/param.py:171-180)."""

    def __init__(self, src_mask=None, ngh_mask=None, backEdgeMask=None, node_degs=None,
                 num_layers=None, layer=None, dim=None):
        self.src_mask, self.ngh_mask = src_mask, ngh_mask
        self.backEdgeMask, self.node_degs = backEdgeMask, node_degs
        self.num_layers, self.layer, self.dim = num_layers, layer, dim
        self.blockx, self.blocky = getBlockSize(dim)


class backInputProperty(object):
    """Prepared execution path of one layer's backward (EPPGCN/param.py:182-200)."""

    def __init__(self, id=None, partPointer=None, edgeList=None, degrees=None,
                 partSize=None, numParts=None, dim=None, layer=None):
        self.degrees, self.dim, self.layer = degrees, dim, layer
        self.blockx, self.blocky = getBlockSize(dim)
        self.fillProperty(id, partPointer, edgeList, partSize, numParts)

    def fillProperty(self, id=None, partPointer=None, edgeList=None, partSize=None, numParts=None):
        self.id, self.partPointer, self.edgeList = id, partPointer, edgeList
        self.partSize, self.numParts = partSize, numParts
