"""FSDP2 communication hooks: the bf16 parameter all-gather and the fp32 gradient reduce-scatter go through
the runtime's collective backend on FSDP's own communication streams.

Same surface as the reference qwen3_triton/runtime/fsdp.py:15-46: `TritonAllGather(communication)`,
`TritonReduceScatter(communication)` implementing FSDP2's `AllGather` / `ReduceScatter` protocol
(`allocate(size, *, dtype, device)` + `__call__(output, input, group[, op], async_op=False)`, asynchronous
handles rejected: FSDP orders the calls with stream events), and `configure(model, communication)`, which
installs them on every FSDPModule. Any world size; the reference is fixed to ranks [0,1,2,3].
"""
import torch
import torch.distributed as dist
from torch.distributed.fsdp import FSDPModule
from torch.distributed.fsdp._fully_shard._fsdp_api import AllGather, ReduceScatter


class _Allocation:
    def allocate(self, size, *, dtype, device):
        return torch.empty(tuple(size), device=device, dtype=dtype)


def _largest_unit(model, world):
    """(elements, bytes in the unit's all-gather dtype) of the largest FSDP unit, parameters padded to the world size
    along their first dimension."""
    elements = nbytes = 0
    for module in model.modules():
        if not isinstance(module, FSDPModule):
            continue
        group = module._get_fsdp_state()._fsdp_param_group
        if group is None:
            continue
        total = total_bytes = 0
        for fsdp_param in group.fsdp_params:
            shape = tuple(fsdp_param._orig_size)
            first = shape[0] if shape else 1
            rest = 1
            for d in shape[1:]:
                rest *= d
            padded = -(-first // world) * world * rest
            policy = getattr(group, 'mp_policy', None)
            dtype = (policy.param_dtype if policy is not None else None) or fsdp_param.sharded_param.dtype
            total += padded
            total_bytes += padded * torch.empty((), dtype=dtype).element_size()
        elements, nbytes = max(elements, total), max(nbytes, total_bytes)
    return elements, nbytes


def _same_group(group, communication):
    return dist.get_process_group_ranks(group) == dist.get_process_group_ranks(communication.group)


class TritonAllGather(_Allocation, AllGather):
    def __init__(self, communication, peer_gather=None):
        self.communication = communication
        self.peer_gather = peer_gather         # runtime/peer_gather.py: output buffers peers can read, copy-engine pulls
        self.calls = 0
        self.peer_calls = 0

    def allocate(self, size, *, dtype, device):
        if self.peer_gather is not None:
            buffer = self.peer_gather.allocate(tuple(size), dtype, device)
            if buffer is not None:
                return buffer
        return torch.empty(tuple(size), device=device, dtype=dtype)

    def __call__(self, output_tensor, input_tensor, group, async_op=False):
        if async_op:
            raise ValueError('Stream/event ordered FSDP calls required')
        if not _same_group(group, self.communication):
            raise ValueError('FSDP mesh and communicator group differ')
        self.calls += 1
        if self.peer_gather is not None and self.peer_gather.gather(output_tensor, input_tensor):
            self.peer_calls += 1
            return
        self.communication.all_gather(output_tensor, input_tensor)


class TritonReduceScatter(_Allocation, ReduceScatter):
    def __init__(self, communication, peer_reducer=None):
        self.communication = communication
        self.peer_reducer = peer_reducer       # runtime/peer_reduce.py: gradients staged as bf16, pulled over NVLink
        self.before_reduce = None              # e.g. TritonAdamW.step_pending: runs on the reduce-scatter stream
        self.calls = 0
        self.peer_calls = 0

    def __call__(self, output_tensor, input_tensor, group, op, async_op=False):
        if async_op:
            raise ValueError('Stream/event ordered FSDP calls required')
        if not _same_group(group, self.communication):
            raise ValueError('FSDP mesh and communicator group differ')
        if op == dist.ReduceOp.AVG:
            operation = 'avg'
        elif op == dist.ReduceOp.SUM:
            operation = 'sum'
        else:
            raise ValueError('FSDP SUM/AVG only')
        self.calls += 1
        if self.before_reduce is not None:
            # the gradient shards of the units reduced before this one are assigned by now, and the kernels that wrote
            # them are earlier on this stream
            self.before_reduce()
        if self.peer_reducer is not None and self.peer_reducer.staged(input_tensor):
            if operation != 'avg':
                # with a gradient divide factor FSDP scales its fp32 buffer before a SUM; that buffer was never filled
                raise ValueError('peer_memory_reduce supports the AVG gradient reduction only')
            self.peer_reducer.reduce(input_tensor, output_tensor, 1.0 / self.communication.world)
            self.peer_calls += 1
            return
        self.communication.reduce_scatter(output_tensor, input_tensor, operation, lossless_bf16=True)


def largest_unit_elements(model, world):
    """Upper bound of the padded gradient elements one FSDP unit reduces."""
    return _largest_unit(model, world)[0]


def configure(model, communication, *, pack_kernels=True, pack_gradients_off_compute_stream=False,
              peer_memory_reduce=False, copy_engine_gather=False, early_copy_out=False,
              gradients_in_staging=False, gather_into_parameters=False):
    """Install the comm hooks on every FSDP unit and (by default) the pack/unpack kernels of runtime/ops.py.
    `pack_gradients_off_compute_stream`: run the reduce-scatter copy-in on FSDP's reduce-scatter stream.
    `peer_memory_reduce`: reduce gradients with the pull kernel over peer memory (runtime/peer_reduce.py; one node,
    2 / 4 / 8 ranks, implies the copy-in on the reduce-scatter stream); the returned dict holds the reducer under
    'peer_reducer' - call its close() before the process group is destroyed. If any rank cannot allocate or map
    the staging buffers, every rank falls back to the collective backend and 'peer_reducer' is None.
    `copy_engine_gather`: all-gather the parameters with copy-engine transfers from buffers the peers have mapped
    (runtime/peer_gather.py; one node); 'peer_gather' in the returned dict, same close() rule and fallback.
    `gradients_in_staging` (with `peer_memory_reduce`): the fused decoder layers write their weight gradients straight
    into the staging buffer the reduction reads, so nothing is packed ('gradient_homes' in the returned dict = number
    of FSDP units set up that way; process-wide: qwen3_triton.fused.GradientHomes).
    `gather_into_parameters` (with `copy_engine_gather`): every rank's piece of every parameter is copied straight
    into the parameter's tensor (one copy-engine transfer each), so FSDP2's split-copy of the rank-major buffer has
    nothing to do; needs the unshard wrapper of runtime/early_copy_out.py ('gather_into_parameters' in the result).
    `early_copy_out`: split-copy the gathered parameters on a side stream as soon as their all-gather is issued
    (runtime/early_copy_out.py; process-wide, needs the pack kernels); 'early_copy_out' in the returned dict tells
    whether it is active."""
    reducer = None
    if peer_memory_reduce:
        if not pack_kernels:
            raise ValueError('peer_memory_reduce needs the pack kernels')
        from .peer_reduce import PeerGradientReducer
        device = torch.device('cuda', torch.cuda.current_device())
        reducer = PeerGradientReducer.create(communication.group, device,
                                             largest_unit_elements(model, communication.world))
    from .. import fused
    homes = 0
    if reducer is not None and gradients_in_staging:
        homes = reducer.register_units(model)
    fused.GradientHomes.provider = reducer if homes else None
    if pack_kernels:
        from .ops import (install_fsdp_pack_kernels, pack_gradients_on_reduce_scatter_stream,
                          reduce_gradients_over_peer_memory)
        install_fsdp_pack_kernels()
        pack_gradients_on_reduce_scatter_stream(model if (pack_gradients_off_compute_stream or reducer) else None)
        reduce_gradients_over_peer_memory(reducer)
    early = False
    if pack_kernels:
        from . import early_copy_out as eco
        early = eco.enable(bool(early_copy_out) and eco.install())
    gatherer = None
    if copy_engine_gather:
        from .peer_gather import PeerAllGather
        device = torch.device('cuda', torch.cuda.current_device())
        gatherer = PeerAllGather.create(communication.group, device, _largest_unit(model, communication.world)[1])
    direct = False
    if pack_kernels:
        direct = eco.deliver_through(gatherer if (gather_into_parameters and gatherer is not None and eco.install())
                                     else None)
    ag = TritonAllGather(communication, gatherer)
    rs = TritonReduceScatter(communication, reducer)
    count = 0
    for module in model.modules():
        if isinstance(module, FSDPModule):
            module.set_custom_all_gather(ag)
            module.set_custom_reduce_scatter(rs)
            count += 1
    if not count:
        raise ValueError('No FSDP units to configure')
    return dict(all_gather=ag, reduce_scatter=rs, units=count, peer_reducer=reducer, peer_gather=gatherer,
                early_copy_out=early, gradient_homes=homes, gather_into_parameters=direct)
