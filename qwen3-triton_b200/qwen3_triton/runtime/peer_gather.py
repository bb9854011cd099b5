"""Parameter all-gather through the copy engines, for ranks that are one process per GPU on one node.

FSDP2 asks its all-gather hook for the rank-major output buffer ([world, shard] elements), copies this rank's shards
into row `rank` of it, and calls the hook to fill the other rows. With the collective library that is a kernel which
occupies SMs for as long as the transfer lasts, beside the forward GEMMs. Here the output buffers are slots of a small
ring of device buffers that every peer has mapped (CUDA IPC); after a barrier on the all-gather stream, row r of the
output is one `cudaMemcpyAsync` from rank r's mapped slot - a copy-engine transfer over NVLink that takes no SM at all.
What a rank reads from a peer is the row the peer wrote itself (its own shards), at the same offset of the same slot.

Slots. `allocate` hands out slot (k mod SLOTS) for the k-th buffer; the tensor made over a slot keeps a small owner
object alive, and when FSDP drops the buffer (after its copy-out) the owner records an event on the stream that is
current then and marks the slot free; the next user of the slot makes its stream wait for that event. A peer cannot
still be reading a slot when its owner writes it again: the copies of use u are queued on the peer's all-gather stream
before the peer's barrier of use u+1, and the owner reaches use u+SLOTS only after it has passed that barrier.
A request that does not fit, or finds its slot still held, gets an ordinary buffer and the collective library's
all-gather (every rank takes the same decision: same program, same sizes, same lifetimes).

What the reference has in this place: its all_gather over IPC-mapped buffers with pull kernels
(qwen3_triton/runtime/collectives.py:88-137) behind the same FSDP2 hook (runtime/fsdp.py:15-24).
"""
import ctypes

import torch
import torch.distributed as dist

from .. import _abi


class _SlotOwner:
    """Presents `nbytes` of a slot to torch through the CUDA array interface; torch keeps it alive with the storage."""

    def __init__(self, ring, index, nbytes):
        self.ring, self.index = ring, index
        self.__cuda_array_interface__ = dict(shape=(nbytes,), typestr='|u1', data=(ring.own[index], False), version=2,
                                             strides=None)

    def __del__(self):
        try:
            event = torch.cuda.Event()
            event.record()                 # FSDP drops the buffer on the stream that ran its copy-out
            self.ring.free_events[self.index] = event
        except Exception:                  # interpreter shutdown
            pass
        self.ring.held[self.index] = False


class PeerAllGather:
    SLOTS = 4

    @classmethod
    def create(cls, group, device, capacity_bytes):
        """A gatherer, or None on every rank when some rank could not allocate or map the slots."""
        try:
            gatherer = cls(group, device, capacity_bytes)
        except (RuntimeError, ValueError) as error:
            import warnings
            warnings.warn('copy-engine all-gather unavailable: %s' % error)
            return None
        return gatherer if gatherer.usable else None

    def __init__(self, group, device, capacity_bytes):
        self.group, self.device = group, torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.capacity = (int(capacity_bytes) + 255) // 256 * 256
        lib = _abi.lib()
        self.own, self.peers = [], []
        failure = None
        with torch.cuda.device(self.device):
            for _ in range(self.SLOTS):
                ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
                if failure is None and lib.q3_peer_alloc(self.capacity, ctypes.byref(ptr), handle) != 0:
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
        verdicts = [None] * self.world
        dist.all_gather_object(verdicts, failure, group=group)
        self.usable = all(v is None for v in verdicts)
        self.closed = False
        self.held = [False] * self.SLOTS
        self.free_events = [None] * self.SLOTS
        self.next_slot = 0
        self.by_pointer = {}
        self.gathers = 0
        self.delivered = 0
        self.direct = False          # set by runtime/fsdp.py:configure when the unshard wrapper delivers the pieces
        self.deferred = None
        self.flag = None
        if not self.usable:
            self.close()
            return
        self.flag = torch.zeros(1, device=self.device)
        self.by_pointer = {address: index for index, address in enumerate(self.own)}

    # -- FSDP's allocate hook
    def allocate(self, size, dtype, device):
        """A tensor of `size` over the next slot, or None (too large, slot still held, another device)."""
        numel = 1
        for n in size:
            numel *= int(n)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        index = self.next_slot
        if (self.closed or torch.device(device) != self.device or nbytes == 0 or nbytes > self.capacity
                or self.held[index]):
            return None
        self.next_slot = (index + 1) % self.SLOTS
        self.held[index] = True
        event, self.free_events[index] = self.free_events[index], None
        if event is not None:
            torch.cuda.current_stream(self.device).wait_event(event)
        raw = torch.as_tensor(_SlotOwner(self, index, nbytes), device=self.device)
        return raw.view(dtype).view(tuple(size))

    # -- FSDP's all-gather hook, on the all-gather stream
    def gather(self, output_tensor, input_tensor):
        """Fill the other ranks' rows of `output_tensor` if it lives in a slot (True), else do nothing (False)."""
        index = self.by_pointer.get(output_tensor.data_ptr())
        if index is None:
            return False
        row = input_tensor.numel() * input_tensor.element_size()
        if (input_tensor.data_ptr() != output_tensor.data_ptr() + self.rank * row
                or output_tensor.numel() * output_tensor.element_size() != row * self.world):
            raise ValueError('All-gather input must be this rank\'s row of the output buffer')
        dist.all_reduce(self.flag, group=self.group)       # every rank's row is written before anyone reads it
        self.gathers += 1
        if self.direct:
            # the rows are not copied here: `deliver` (called by the wrapper of FSDP2's unshard, which knows the unit's
            # parameter tensors) sends every piece straight to its parameter
            self.deferred = dict(index=index, row=row, output=output_tensor.data_ptr(),
                                 stream=torch.cuda.current_stream(self.device), itemsize=input_tensor.element_size())
            return True
        self._copy_rows(index, row, output_tensor.data_ptr(), _abi.stream())
        return True

    def _copy_rows(self, index, row, output, stream):
        for step in range(1, self.world):
            r = (self.rank + step) % self.world             # ranks start on different peers
            _abi.call('q3_peer_copy', output + r * row, self.peers[index][r] + r * row, row, stream)

    def deliver(self, split_sizes, outs):
        """Finish the all-gather whose barrier `gather` has just issued. `outs[i]`: the contiguous tensor of
        world x split_sizes[i] elements FSDP2 would fill by splitting the rank-major buffer. Every rank's piece of
        every parameter goes there directly (one copy-engine transfer each, this rank's own pieces included), on the
        all-gather stream; returns the event behind the last copy - the rank-major buffer then needs no split-copy.
        If the tensors are not what the row layout implies, the rows are copied into the rank-major buffer instead
        and None is returned (FSDP2 splits as usual)."""
        d, self.deferred = self.deferred, None
        if d is None:
            return None
        itemsize, row, index = d['itemsize'], d['row'], d['index']
        sizes = [int(n) for n in split_sizes]
        fits = (len(outs) == len(sizes) and sum(sizes) * itemsize == row
                and all(o.is_contiguous() and o.element_size() == itemsize and o.numel() == self.world * n
                        for o, n in zip(outs, sizes)))
        with torch.cuda.stream(d['stream']):
            if not fits:
                self._copy_rows(index, row, d['output'], _abi.stream())
                return None
            count = len(sizes) * self.world
            dst, src, nbytes = (ctypes.c_void_p * count)(), (ctypes.c_void_p * count)(), (ctypes.c_int64 * count)()
            k, offset = 0, 0
            for o, n in zip(outs, sizes):
                piece = n * itemsize
                for step in range(self.world):
                    r = (self.rank + step) % self.world
                    dst[k] = o.data_ptr() + r * piece
                    src[k] = self.peers[index][r] + r * row + offset
                    nbytes[k] = piece
                    k += 1
                offset += piece
            _abi.call('q3_peer_copy_many', dst, src, nbytes, count, _abi.stream())
            event = torch.cuda.Event()
            event.record()
        self.delivered += 1
        return event

    def close(self):
        if self.closed:
            return
        self.closed = True
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)                       # nobody unmaps while a peer may still be reading
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
