"""Collective backend for the training runtime: NCCL (over NVLink / NVSwitch) through torch.distributed.

Same method surface as the reference's peer-memory communicator `TritonCollectives`
(qwen3_triton/runtime/collectives.py:139-203): all_gather(output, source), reduce_scatter(output, source, op,
lossless_bf16=...), all_reduce(tensor, op), all_to_all(output, source), barrier(), close(), report(). The
reference moves the bytes with hand-written Triton pull kernels over CUDA-IPC mappings between exactly four
PCIe GPUs; on an NVSwitch box the transport is NCCL, any world size, launched on whatever stream is current
(FSDP2 calls these from its all-gather / reduce-scatter streams). Payloads cross the wire in their own dtype:
bf16 parameters, fp32 gradients.
"""
import torch
import torch.distributed as dist

_OPS = {'sum': dist.ReduceOp.SUM, 'avg': dist.ReduceOp.AVG, 'max': dist.ReduceOp.MAX, 'min': dist.ReduceOp.MIN}
_DTYPES = (torch.bfloat16, torch.float32, torch.float64, torch.int64, torch.int32, torch.float16)


class NcclCollectives:
    def __init__(self, *, group=None):
        if not dist.is_initialized():
            raise RuntimeError('torch.distributed must be initialised first')
        self.group = dist.group.WORLD if group is None else group
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.backend = dist.get_backend(self.group)
        self.closed = False
        self.calls = dict(gather=0, scatter=0, reduce=0, alltoall=0, barrier=0)
        self.bytes = dict(gather=0, scatter=0, reduce=0, alltoall=0)

    def _check(self, output, source):
        if self.closed:
            raise RuntimeError('Closed communicator')
        if (source.device != output.device or not source.is_contiguous() or not output.is_contiguous()
                or source.dtype not in _DTYPES):
            raise ValueError('Supported contiguous same-device tensors required')

    def all_gather(self, output, source):
        self._check(output, source)
        if output.numel() != self.world * source.numel() or output.dtype != source.dtype:
            raise ValueError('World-size-times gather output of the same dtype required')
        dist.all_gather_into_tensor(output, source, group=self.group)
        self.calls['gather'] += 1
        self.bytes['gather'] += output.numel() * output.element_size()
        return output

    def reduce_scatter(self, output, source, op='avg', *, lossless_bf16=False):
        self._check(output, source)
        if source.numel() != self.world * output.numel() or output.dtype != source.dtype:
            raise ValueError('World-size-times reduce-scatter input of the same dtype required')
        if op not in _OPS or (op == 'avg' and not output.dtype.is_floating_point):
            raise ValueError('Supported reduction required')
        # lossless_bf16 asks the reference transport to ship fp32 gradients as bf16 when that is exact; NCCL
        # over NVLink carries the fp32 payload as is, so the flag changes nothing here.
        if self.backend == 'gloo':
            # gloo has no reduce-scatter and no AVG: all-reduce a copy and keep this rank's slice (CPU tests)
            full = source.clone()
            dist.all_reduce(full, op=_OPS['sum' if op == 'avg' else op], group=self.group)
            if op == 'avg':
                full /= self.world
            output.copy_(full.view(self.world, -1)[self.rank].view_as(output))
        else:
            dist.reduce_scatter_tensor(output, source, op=_OPS[op], group=self.group)
        self.calls['scatter'] += 1
        self.bytes['scatter'] += source.numel() * source.element_size()
        return output

    def all_reduce(self, tensor, op='sum'):
        self._check(tensor, tensor)
        if op not in _OPS:
            raise ValueError('Supported reduction required')
        if op == 'avg' and self.backend == 'gloo':
            dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self.group)
            tensor /= self.world
        else:
            dist.all_reduce(tensor, op=_OPS[op], group=self.group)
        self.calls['reduce'] += 1
        self.bytes['reduce'] += tensor.numel() * tensor.element_size()
        return tensor

    def all_to_all(self, output, source):
        self._check(output, source)
        if source.numel() != output.numel() or source.numel() % self.world or source.dtype != output.dtype:
            raise ValueError('Equal all-to-all blocks required')
        dist.all_to_all_single(output, source, group=self.group)
        self.calls['alltoall'] += 1
        self.bytes['alltoall'] += source.numel() * source.element_size()
        return output

    def barrier(self):
        if self.closed:
            raise RuntimeError('Closed communicator')
        dist.barrier(group=self.group)
        self.calls['barrier'] += 1

    def close(self):
        self.closed = True

    def report(self):
        return dict(complete=True, backend=self.backend, world=self.world, calls=dict(self.calls), bytes=dict(self.bytes))


TritonCollectives = NcclCollectives   # the reference's class name, for call sites that construct it
