"""Gradient reduce-scatter over peer memory for ranks that are one process per GPU on one node.

FSDP2 hands a unit's gradients (bf16) to `fsdp::chunk_cat`, which upcasts them into an fp32 rank-major staging
buffer, and then reduce-scatters that buffer in fp32. Here the override of `chunk_cat` packs the gradients, still
bf16, into a staging buffer every peer has mapped (CUDA IPC), and the reduce-scatter hook - after a barrier on its
stream - launches q3_reduce_scatter_pull: each rank reads its rows of every peer's staging buffer over NVLink, adds
them in fp32 in rank order and writes its fp32 shard. The result is the fp32 reduce-scatter of the upcast gradients,
bit for bit what NCCL's sum gives on two ranks and the same fixed-order fp32 sum on more; 2 bytes per element cross
the links instead of 4, and the fp32 staging buffer is never written or read.

Ordering. Packing, barrier and pull of every unit run on FSDP's reduce-scatter stream, in that order, and the two
staging slots alternate: when rank A packs unit k+2 into the slot unit k used, A has passed the barrier of unit k+1,
which no rank enters before it has finished pulling unit k. No kernel waits on a flag written by another GPU; the
barrier is a one-element all-reduce of the collective library on the same stream.

What the reference has in this place: hand-written pull kernels over IPC mappings in its collectives
(qwen3_triton/runtime/collectives.py:139-203, `reduce_scatter(..., lossless_bf16=...)`) behind the same FSDP2 hook.
"""
import ctypes

import torch
import torch.distributed as dist

from .. import _abi


class PeerGradientReducer:
    SLOTS = 2

    @classmethod
    def create(cls, group, device, capacity_elements):
        """A reducer, or None on every rank when some rank could not allocate or map the staging buffers (ranks on
        different nodes, peer access unavailable): the callers then stay on the collective backend."""
        try:
            reducer = cls(group, device, capacity_elements)
        except (RuntimeError, ValueError) as error:
            import warnings
            warnings.warn('peer-memory gradient reduction unavailable: %s' % error)
            reducer = None
        return reducer if reducer is not None and reducer.usable else None

    def __init__(self, group, device, capacity_elements):
        """`capacity_elements`: the largest number of (padded) gradient elements one FSDP unit hands over. Collective:
        every rank of `group` takes part in the handle exchange even if its own allocation failed; `usable` is the
        same on all ranks afterwards."""
        self.group, self.device = group, torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world not in (2, 4, 8):
            raise ValueError('Peer reduce-scatter supports 2, 4 or 8 ranks on one node')
        self.capacity = (int(capacity_elements) + 8 * self.world - 1) // (8 * self.world) * (8 * self.world)
        lib = _abi.lib()
        self.own, self.peers, self.tables = [], [], []
        failure = None
        with torch.cuda.device(self.device):
            for _ in range(self.SLOTS):
                ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
                if failure is None and lib.q3_peer_alloc(self.capacity * 2, ctypes.byref(ptr), handle) != 0:
                    failure = 'allocation'
                handles = [None] * self.world
                dist.all_gather_object(handles, handle.raw if failure is None else None, group=group)
                mapped = []
                for r in range(self.world):
                    if r == self.rank:
                        mapped.append(ptr.value)
                        continue
                    peer = ctypes.c_void_p()
                    if failure is None and (handles[r] is None or lib.q3_peer_open(handles[r], ctypes.byref(peer)) != 0):
                        failure = 'mapping the buffer of rank %d' % r
                    mapped.append(peer.value)
                self.own.append(ptr.value)
                self.peers.append(mapped)
                self.tables.append((ctypes.c_void_p * self.world)(*[m or 0 for m in mapped]))
        verdicts = [None] * self.world
        dist.all_gather_object(verdicts, failure, group=group)
        self.usable = all(v is None for v in verdicts)
        self.closed = False
        if not self.usable:
            self.flag = None
            self.close()
            return
        self.flag = torch.zeros(1, device=self.device)
        self.next_slot = 0
        self.pending = {}           # data_ptr of FSDP's fp32 reduce-scatter input -> (slot, columns, dtype)
        self.units = 0

    # -- called from the chunk_cat override, on the reduce-scatter stream
    def stage(self, tensors, out, launch, plan):
        """Pack `tensors` (one 16-bit dtype) as [world, columns] into the next staging slot; `out` is the fp32 buffer
        FSDP believes it fills. Returns False (nothing done) if the unit does not fit."""
        rows, cols = plan([tuple(t.shape) for t in tensors], [t.data_ptr() for t in tensors], self.own[self.next_slot],
                          2, self.world)
        if cols * self.world > self.capacity or cols != out.shape[1] or cols % 8:
            return False
        slot = self.next_slot
        self.next_slot = (slot + 1) % self.SLOTS
        launch(rows, tensors[0].dtype, tensors[0].dtype, self.device)
        self.pending[out.data_ptr()] = (slot, cols, tensors[0].dtype)
        return True

    # -- called from the reduce-scatter hook, on the reduce-scatter stream
    def staged(self, input_tensor):
        return input_tensor.data_ptr() in self.pending

    def reduce(self, input_tensor, output_tensor, scale):
        """`input_tensor` is a buffer whose gradients were staged: barrier, then pull this rank's rows, times `scale`."""
        slot, cols, dtype = self.pending.pop(input_tensor.data_ptr())
        if output_tensor.numel() != cols or output_tensor.dtype != torch.float32 or not output_tensor.is_contiguous():
            raise ValueError('Reduce-scatter output does not match the staged gradients')
        dist.all_reduce(self.flag, group=self.group)        # every rank's pack precedes its all-reduce on this stream
        _abi.call('q3_reduce_scatter_pull', self.tables[slot], self.world, output_tensor.data_ptr(), self.rank * cols,
                  cols, float(scale), _abi.dt(dtype), _abi.stream())
        self.units += 1

    def close(self):
        if self.closed:
            return
        self.closed = True
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)                        # nobody unmaps while a peer may still be reading
        lib = _abi.lib()
        with torch.cuda.device(self.device):
            for slot in range(len(self.peers)):
                for r, address in enumerate(self.peers[slot]):
                    if r != self.rank and address:
                        lib.q3_peer_close(ctypes.c_void_p(address))
            dist.barrier(group=self.group)
            for address in self.own:
                if address:
                    lib.q3_peer_free(ctypes.c_void_p(address))
