"""Replica tables: for every global node id the list of (rank, local slot) copies.

Mirrors starrygl/cache/replica_table.py (``CSRReplicaTable`` :3-82, ``UVACSRReplicaTable`` :86-175,
``build_replica_table`` :178-215).  ``lookup`` on CUDA tensors is one pair of kernels
(row lengths + scan, then expansion) with a single read-back of the total, instead of the reference's
chain of ``repeat_interleave`` / ``cumsum`` temporaries.
"""
import torch

from .. import ops


class CSRReplicaTable:
    def __init__(self, indptr: torch.Tensor, indices: torch.Tensor, locs: torch.Tensor,
                 device: torch.device = torch.device('cpu')):
        self.indptr = indptr
        self.indices = indices
        self.locs = locs
        self.device = indptr.device

    def to(self, device):
        return CSRReplicaTable(self.indptr.to(device), self.indices.to(device), self.locs.to(device))

    def lookup(self, batch_ids: torch.Tensor, max_replicas_per_node: int = 0):
        """-> (src_indices, target_ranks, target_locs): row k of the batch repeated once per replica.

        The table has to live on the GPU (``.to(device)``).  ``max_replicas_per_node`` bounds the output size
        without a read-back; 0 means "number of ranks seen in the table" (computed once).
        """
        if not self.indptr.is_cuda:
            raise RuntimeError("CSRReplicaTable.lookup runs on the GPU: move the table with .to(device) first")
        batch_ids = batch_ids.to(self.device)
        if max_replicas_per_node <= 0:
            if not hasattr(self, "_max_rep"):
                self._max_rep = int((self.indptr[1:] - self.indptr[:-1]).max().item()) if self.indptr.numel() > 1 else 0
            max_replicas_per_node = self._max_rep
        cap = batch_ids.numel() * max(max_replicas_per_node, 1)
        st = ops.StatusWord(self.device)
        src, rk, lc, offs = ops.replica_lookup(self.indptr, self.indices, self.locs, batch_ids, cap, status=st)
        total = int(offs[-1].item())
        st.check("replica lookup")
        if total == 0:
            e = torch.empty(0, dtype=torch.long, device=self.device)
            return e, e.clone(), e.clone()
        return src[:total], rk[:total], lc[:total]


class UVACSRReplicaTable(CSRReplicaTable):
    """Row pointer on the GPU, replica lists in pinned host memory that the lookup kernels read in place
    (the reference stages them through a host ``index_select``; the GPU addresses pinned memory directly)."""

    def __init__(self, indptr: torch.Tensor, indices: torch.Tensor, locs: torch.Tensor = None,
                 max_batch_size_estimate=100000):
        if locs is None:
            raise ValueError("UVACSRReplicaTable needs the replica slots (locs)")
        dev = torch.device("cuda", torch.cuda.current_device())
        super().__init__(indptr.to(dev), indices.cpu().contiguous().pin_memory(), locs.cpu().contiguous().pin_memory())
        self.device = dev


def build_replica_table(num_nodes, partition_book, num_parts, type=None):
    """CSR over node id of (rank, local slot), sorted by (node, rank, slot); one-time set-up on the host."""
    trip = []
    for part in range(num_parts):
        nodes = partition_book[part]
        nodes = torch.as_tensor(nodes, dtype=torch.long)
        trip.append(torch.stack((nodes, torch.full_like(nodes, part), torch.arange(nodes.shape[0], dtype=torch.long))))
    all_pairs = torch.cat(trip, dim=1) if trip else torch.empty((3, 0), dtype=torch.long)
    u = all_pairs.unique(dim=1)
    indptr = torch.zeros(num_nodes + 1, dtype=torch.long)
    indptr[1:] = torch.cumsum(u[0].bincount(minlength=num_nodes), dim=0)
    if type == 'UVA':
        return UVACSRReplicaTable(indptr=indptr, indices=u[1].contiguous(), locs=u[2].contiguous(),
                                  max_batch_size_estimate=int(0.2 * num_nodes))
    return CSRReplicaTable(indptr=indptr, indices=u[1].contiguous(), locs=u[2].contiguous())
