"""Gradient reduce-scatter over peer memory for ranks that are one process per GPU on one node.

FSDP2 hands a unit's gradients (bf16) to `fsdp::chunk_cat`, which upcasts them into an fp32 rank-major staging
buffer, and then reduce-scatters that buffer in fp32. Here the override of `chunk_cat` packs the gradients, still
bf16, into a staging buffer every peer has mapped (CUDA IPC), and the reduce-scatter hook - after a barrier on its
stream - launches q3_reduce_scatter_pull: each rank reads its rows of every peer's staging buffer over NVLink, adds
them in fp32 in rank order and writes its fp32 shard. The result is the fp32 reduce-scatter of the upcast gradients,
bit for bit what NCCL's sum gives on two ranks and the same fixed-order fp32 sum on more; 2 bytes per element cross
the links instead of 4, and the fp32 staging buffer is never written or read.

Gradients born in the staging buffer (`register_units`, optional). The fused decoder layer's backward can write its
weight gradients straight into the unit's staging slot: each parameter has a fixed home (parameters one after the
other, every one contiguous, so the views are ordinary gradient tensors that autograd adopts without a copy). The
`chunk_cat` override then finds the gradients already in place and packs nothing (the few that are not - norm weights
produced by other kernels - are copied to their homes), and the reduce-scatter hook pulls parameter by parameter:
rank r's piece of parameter p is rows [r d0/W, (r+1) d0/W) of p's home in every peer's slot. That removes the pack
pass (2 + 2 bytes per gradient element of HBM traffic beside the backward GEMMs).

Ordering. Barrier and pull of every unit run on FSDP's reduce-scatter stream (the pack too, where there is one), and
three staging slots rotate. A slot is written again - by the pack on the reduce-scatter stream or by the backward
GEMMs on the compute stream - only after the event recorded behind the barrier of the unit AFTER its previous user:
no rank enters that barrier before it has finished pulling the previous user's gradients. No kernel waits on a flag
written by another GPU; the barrier is a one-element all-reduce of the collective library on the same stream.

What the reference has in this place: hand-written pull kernels over IPC mappings in its collectives
(qwen3_triton/runtime/collectives.py:139-203, `reduce_scatter(..., lossless_bf16=...)`) behind the same FSDP2 hook.
"""
import ctypes

import torch
import torch.distributed as dist

from .. import _abi


class PeerGradientReducer:
    SLOTS = 3

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
        # room for every parameter's home to start on a 16-byte boundary
        self.capacity = (int(capacity_elements) + 4096 + 8 * self.world - 1) // (8 * self.world) * (8 * self.world)
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
        self.pending = {}           # data_ptr of FSDP's fp32 reduce-scatter input -> staged unit
        self.units = 0
        self.free_after = [None] * self.SLOTS    # event to wait for before a slot is written again
        self.previous_slot = None                # slot of the unit whose barrier came last
        # gradients born in the staging buffer
        self.layouts = []                        # per registered FSDP unit: homes of its parameters
        self.home_of = {}                        # (id(module), parameter name) -> (layout index, position in it)
        self.claimed = {}                        # layout index -> slot, from the first gradient view to the reduce
        self.handed = set()                      # (layout index, position) given out since the unit's slot was claimed
        self.slot_views = None                   # one 16-bit tensor per slot over the staging memory
        self.born_in_place = 0
        self.copied_home = 0

    # -- slots
    def _claim(self):
        """Next slot of the rotation; the current stream waits until every rank is done with its previous content."""
        slot = self.next_slot
        self.next_slot = (slot + 1) % self.SLOTS
        event, self.free_after[slot] = self.free_after[slot], None
        if event is not None:
            torch.cuda.current_stream(self.device).wait_event(event)
        return slot

    # -- gradients born in the staging buffer
    def register_units(self, model):
        """Give every parameter of every FSDP unit of `model` a home in the unit's staging slot. Returns the number of
        units registered (units with a parameter that would need padding, or not sharded on dim 0, are left out and
        keep the pack path)."""
        from torch.distributed.fsdp import FSDPModule

        class _Memory:
            def __init__(self, address, elements):
                self.__cuda_array_interface__ = dict(shape=(elements,), typestr='<i2', data=(address, False), version=2,
                                                     strides=None)

        if self.slot_views is None:
            self.slot_views = [torch.as_tensor(_Memory(address, self.capacity), device=self.device)
                               for address in self.own]
        for module in model.modules():
            if not isinstance(module, FSDPModule):
                continue
            group = module._get_fsdp_state()._fsdp_param_group
            if group is None:
                continue
            homes, offset, usable = [], 0, True
            for fsdp_param in group.fsdp_params:
                shape = tuple(fsdp_param._orig_size)
                numel = 1
                for d in shape:
                    numel *= d
                first = shape[0] if shape else 1
                piece = numel // self.world
                if (not shape or first % self.world or piece % 8 or fsdp_param.fsdp_placement.dim != 0
                        or fsdp_param._module_info.shared_modules):
                    usable = False
                    break
                info = fsdp_param._module_info
                homes.append(dict(key=(id(info.module), info.param_name), shape=shape, numel=numel, piece=piece,
                                  home=offset))
                offset += (numel + 7) // 8 * 8
            if not usable or not homes or offset > self.capacity:
                continue
            index = len(self.layouts)
            columns, out_offsets = 0, []
            for h in homes:
                out_offsets.append(columns)
                columns += h['piece']
            self.layouts.append(dict(homes=homes, columns=columns, out_offsets=out_offsets,
                                     signature=tuple(h['shape'] for h in homes)))
            for position, h in enumerate(homes):
                self.home_of[h['key']] = (index, position)
        return len(self.layouts)

    def home(self, module, name='weight'):
        """Opaque handle of a parameter's home (for `gradient_view`), or None if the parameter has none."""
        return self.home_of.get((id(module), name))

    def gradient_view(self, handle, dtype):
        """A contiguous tensor of the parameter's shape inside the staging slot its unit uses in this backward pass, or
        None. Called from the backward of the layer that produces the gradient, on the compute stream."""
        if handle is None or self.closed or dtype not in (torch.bfloat16, torch.float16):
            return None
        index, position = handle
        if (index, position) in self.handed:
            # a second backward pass before the unit was reduced (gradient accumulation): the home holds the first
            # pass's gradient, which autograd is about to add to - the new one needs memory of its own
            return None
        slot = self.claimed.get(index)
        if slot is None:
            slot = self.claimed[index] = self._claim()
        self.handed.add((index, position))
        h = self.layouts[index]['homes'][position]
        return self.slot_views[slot][h['home']:h['home'] + h['numel']].view(dtype).view(h['shape'])

    def _layout_of(self, tensors):
        """The registered unit these gradients belong to: the one some of them already live in, else one with the
        same list of shapes (units with equal shapes have equal layouts)."""
        if not self.layouts:
            return None
        signature = tuple(tuple(t.shape) for t in tensors)
        for index, slot in self.claimed.items():
            layout = self.layouts[index]
            if layout['signature'] != signature:
                continue
            base = self.own[slot]
            if any(t.data_ptr() == base + 2 * h['home'] for t, h in zip(tensors, layout['homes'])):
                return index
        for index, layout in enumerate(self.layouts):
            if layout['signature'] == signature and index not in self.claimed:
                return index
        return None

    # -- called from the chunk_cat override, on the reduce-scatter stream
    def stage(self, tensors, out, launch, plan):
        """Make the unit's 16-bit gradients readable by the peers; `out` is the fp32 buffer FSDP believes it fills.
        Returns False (nothing done) if the unit does not fit."""
        index = self._layout_of(tensors)
        if index is not None and self.layouts[index]['columns'] == out.shape[1]:
            layout = self.layouts[index]
            slot = self.claimed.pop(index, None)
            self.handed = {key for key in self.handed if key[0] != index}
            if slot is None:
                slot = self._claim()
            base = self.own[slot]
            rows = []
            for t, h in zip(tensors, layout['homes']):
                if t.data_ptr() == base + 2 * h['home']:
                    self.born_in_place += 1
                else:                        # produced elsewhere (norm weights): one plain copy to its home
                    rows.append((t.data_ptr(), base + 2 * h['home'], 1, h['numel'], h['numel'], h['numel'], h['numel']))
                    self.copied_home += 1
            if rows:
                launch(rows, tensors[0].dtype, tensors[0].dtype, self.device)
            self.pending[out.data_ptr()] = ('homes', slot, index, tensors[0].dtype)
            return True
        # rank-major pack of whatever FSDP hands over (also of gradients that were born in a slot: a unit whose list
        # of gradients is not the registered one, e.g. a parameter without gradient; that slot was never offered to the
        # peers and needs no release)
        self.claimed.clear()
        self.handed.clear()
        rows, cols = plan([tuple(t.shape) for t in tensors], [t.data_ptr() for t in tensors], 0, 2, self.world)
        if cols * self.world > self.capacity or cols != out.shape[1] or cols % 8:
            return False
        slot = self._claim()
        rows, cols = plan([tuple(t.shape) for t in tensors], [t.data_ptr() for t in tensors], self.own[slot], 2,
                          self.world)
        launch(rows, tensors[0].dtype, tensors[0].dtype, self.device)
        self.pending[out.data_ptr()] = ('rows', slot, cols, tensors[0].dtype)
        return True

    # -- called from the reduce-scatter hook, on the reduce-scatter stream
    def staged(self, input_tensor):
        return input_tensor.data_ptr() in self.pending

    def reduce(self, input_tensor, output_tensor, scale):
        """`input_tensor` is a buffer whose gradients were staged: barrier, then pull this rank's part, times `scale`."""
        kind, slot, what, dtype = self.pending.pop(input_tensor.data_ptr())
        if output_tensor.dtype != torch.float32 or not output_tensor.is_contiguous():
            raise ValueError('Reduce-scatter output must be contiguous fp32')
        dist.all_reduce(self.flag, group=self.group)        # every rank's gradients are in place before its all-reduce
        event = torch.cuda.Event()
        event.record()
        if self.previous_slot is not None:
            # every rank has entered this barrier, so every rank has finished pulling the previous unit
            self.free_after[self.previous_slot] = event
        self.previous_slot = slot
        stream, table = _abi.stream(), self.tables[slot]
        if kind == 'rows':
            cols = what
            if output_tensor.numel() != cols:
                raise ValueError('Reduce-scatter output does not match the staged gradients')
            _abi.call('q3_reduce_scatter_pull', table, self.world, output_tensor.data_ptr(), self.rank * cols, cols,
                      float(scale), _abi.dt(dtype), stream)
        else:
            layout = self.layouts[what]
            if output_tensor.numel() != layout['columns']:
                raise ValueError('Reduce-scatter output does not match the staged gradients')
            for h, out_offset in zip(layout['homes'], layout['out_offsets']):
                _abi.call('q3_reduce_scatter_pull', table, self.world, output_tensor.data_ptr() + 4 * out_offset,
                          h['home'] + self.rank * h['piece'], h['piece'], float(scale), _abi.dt(dtype), stream)
        self.units += 1

    def close(self):
        if self.closed:
            return
        self.closed = True
        from .. import fused
        if fused.GradientHomes.provider is self:
            fused.GradientHomes.provider = None
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
