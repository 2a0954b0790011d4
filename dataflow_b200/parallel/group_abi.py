"""The collective face every group object offers to block code, whatever moves the bytes underneath.

``ctx.groups[name]`` is one of ``DpGroup`` / ``TpGroup`` / ``EpGroup`` (in-process ranks: fused peer-memory kernels where
they exist, ``torch.distributed`` otherwise), ``service.peer.nm.HostGroupHandle`` (daemon fleet on CPU) or
``service.peer.ncclcomm.NcclComm`` (daemon fleet on GPUs).  All of them answer

    all_reduce(t)            sum in place, every rank
    broadcast(t, root)       root's values everywhere, in place
    reduce(t, root)          sum lands in root's tensor; the other ranks' tensors are left as they were
    all_gather(own, full)    full = concatenation of every rank's ``own``, rank order
    reduce_scatter(full, out) out = this rank's slice of the element-wise sum of every rank's ``full``
    check()                  raise what a kernel or a peer reported since the last call

so an executable written against this list runs under every launcher.  This mixin supplies the list through the process
group of the in-process ranks; classes override what they do better (``DpGroup.rs_adamw``, ``TpGroup.ag_gemm``, ...).
Role parity: reference ``src/dataflow/runtime/groups.py`` (GroupHandle: allreduce / broadcast / reduce / reduce_scatter /
all_gather).
"""
from __future__ import annotations


class GroupCollectives:
    """Needs ``rank``, ``world`` and ``pg`` (a ``torch.distributed`` group or ``None`` for the whole job) on the instance."""

    def _dist(self):
        import torch.distributed as dist
        return dist if (dist.is_available() and dist.is_initialized() and self.world > 1) else None

    def _global(self, group_rank: int) -> int:
        dist = self._dist()
        pg = getattr(self, "pg", None)
        return dist.get_global_rank(pg, group_rank) if (dist is not None and pg is not None) else group_rank

    def all_reduce(self, t):
        dist = self._dist()
        if dist is not None:
            dist.all_reduce(t, group=getattr(self, "pg", None))
        return t

    def broadcast(self, t, root: int = 0):
        dist = self._dist()
        if dist is not None:
            dist.broadcast(t, src=self._global(root), group=getattr(self, "pg", None))
        return t

    def reduce(self, t, root: int = 0):
        dist = self._dist()
        if dist is not None:
            keep = None if self.rank == root else t.clone()
            dist.reduce(t, dst=self._global(root), group=getattr(self, "pg", None))
            if keep is not None:
                t.copy_(keep)             # the library leaves non-root buffers unspecified; this ABI leaves them untouched
        return t

    def all_gather(self, own, full):
        dist = self._dist()
        if dist is None:
            full.reshape(-1)[: own.numel()].copy_(own.reshape(-1))
            return full
        dist.all_gather_into_tensor(full.reshape(-1), own.reshape(-1).contiguous(), group=getattr(self, "pg", None))
        return full

    def reduce_scatter(self, full, out):
        dist = self._dist()
        if dist is None:
            out.reshape(-1).copy_(full.reshape(-1)[: out.numel()])
            return out
        dist.reduce_scatter_tensor(out.reshape(-1), full.reshape(-1).contiguous(), group=getattr(self, "pg", None))
        return out
