"""Replica-to-replica memory for the data-parallel update (`tb200_dp_update`).

The fused update reads every replica's gradients and writes every replica's parameters from inside one
kernel, so both flat buffers must be memory every GPU of the node can address: a symmetric allocation
(the same size at the same offset on every rank), exchanged once at set-up.  torch's symmetric-memory
allocator provides exactly that -- peer mappings of every rank's buffer and, where the GPUs sit behind an
NVSwitch, an NVLink multicast mapping -- and is used here for the allocation and the exchange of handles
only; the kernel that moves the data is the library's own.
"""
from . import lib


class ReplicaLink:
    """The parameter and gradient buffers of one replica, addressable by all replicas, and the signal pads
    the ranks meet on.  Create it on every rank at the same point (it is a collective), keep it alive as
    long as any launch that uses it may still run, and let every rank reach `close()`."""

    def __init__(self, torch, elements, group=None, multimem=True):
        import torch.distributed._symmetric_memory as symm
        dist = torch.distributed
        self.torch = torch
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 16:
            raise ValueError("tb200_dp_update takes at most 16 replicas")
        bf = torch.bfloat16
        dev = torch.device("cuda", torch.cuda.current_device())
        self.elements = (elements + 7) // 8 * 8
        self.params = symm.empty(self.elements, dtype=bf, device=dev)
        self.grads = symm.empty(self.elements, dtype=bf, device=dev)
        self.signals = symm.empty(lib.dp_signal_bytes() // 4, dtype=torch.int32, device=dev)
        self.params.zero_()
        self.grads.zero_()
        self.signals.zero_()
        self.state = torch.zeros(lib.dp_state_bytes() // 4, dtype=torch.int32, device=dev)
        self._handles = [symm.rendezvous(t, group) for t in (self.params, self.grads, self.signals)]
        hp, hg, hs = self._handles
        self.param_ptrs, self.grad_ptrs, self.signal_ptrs = list(hp.buffer_ptrs), list(hg.buffer_ptrs), list(hs.buffer_ptrs)
        mc_p, mc_g = int(hp.multicast_ptr or 0), int(hg.multicast_ptr or 0)
        self.multimem = bool(multimem and mc_p and mc_g)
        self.param_mc, self.grad_mc = (mc_p, mc_g) if self.multimem else (0, 0)
        torch.cuda.synchronize()
        dist.barrier(group)        # every rank's pads are zero before anyone signals

    def desc(self, first, last, alpha, blocks=0):
        """The descriptor of the update of elements [first, last) of the flat buffers."""
        off = 2 * first
        return lib.dp_desc(self.rank, self.world, last - first, alpha,
                           [p + off for p in self.grad_ptrs], [p + off for p in self.param_ptrs], self.signal_ptrs,
                           self.state.data_ptr(), self.grad_mc + off if self.multimem else 0,
                           self.param_mc + off if self.multimem else 0, blocks)

    def close(self):
        """Every rank's launches done, then the mappings go: call it on every rank, none leaving early."""
        torch = self.torch
        torch.cuda.synchronize()
        torch.distributed.barrier()
        self._handles = None
        self.params = self.grads = self.signals = None
