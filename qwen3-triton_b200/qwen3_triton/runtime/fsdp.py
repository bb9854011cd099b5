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


def _same_group(group, communication):
    return dist.get_process_group_ranks(group) == dist.get_process_group_ranks(communication.group)


class TritonAllGather(_Allocation, AllGather):
    def __init__(self, communication):
        self.communication = communication
        self.calls = 0

    def __call__(self, output_tensor, input_tensor, group, async_op=False):
        if async_op:
            raise ValueError('Stream/event ordered FSDP calls required')
        if not _same_group(group, self.communication):
            raise ValueError('FSDP mesh and communicator group differ')
        self.communication.all_gather(output_tensor, input_tensor)
        self.calls += 1


class TritonReduceScatter(_Allocation, ReduceScatter):
    def __init__(self, communication):
        self.communication = communication
        self.calls = 0

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
        self.communication.reduce_scatter(output_tensor, input_tensor, operation, lossless_bf16=True)
        self.calls += 1


def configure(model, communication, *, pack_kernels=True, pack_gradients_off_compute_stream=False):
    """Install the comm hooks on every FSDP unit and (by default) the pack/unpack kernels of runtime/ops.py.
    `pack_gradients_off_compute_stream`: run the reduce-scatter copy-in on FSDP's reduce-scatter stream."""
    if pack_kernels:
        from .ops import install_fsdp_pack_kernels, pack_gradients_on_reduce_scatter_stream
        install_fsdp_pack_kernels()
        pack_gradients_on_reduce_scatter_stream(model if pack_gradients_off_compute_stream else None)
    ag = TritonAllGather(communication)
    rs = TritonReduceScatter(communication)
    count = 0
    for module in model.modules():
        if isinstance(module, FSDPModule):
            module.set_custom_all_gather(ag)
            module.set_custom_reduce_scatter(rs)
            count += 1
    if not count:
        raise ValueError('No FSDP units to configure')
    return dict(all_gather=ag, reduce_scatter=rs, units=count)
