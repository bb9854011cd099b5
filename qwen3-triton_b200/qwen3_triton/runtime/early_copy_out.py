"""Split-copy of gathered parameters ahead of time, off the compute stream.

FSDP2 turns the rank-major all-gather buffer into per-parameter tensors (`fsdp::split_with_sizes_copy`) when a unit is
about to run, on the compute stream: about 8 ms per step of Qwen3-8B that nothing overlaps, whatever the number of
GPUs. With all-gathers issued one or two units ahead, the buffer is complete long before it is needed. This module
wraps `FSDPParamGroup.unshard`: right after a unit's all-gather has been issued it allocates the unit's parameter
tensors (the same calls FSDP2 makes later, which then find them allocated) and runs the split-copy on a stream of
its own, ordered after the all-gather's event; the `split_with_sizes_copy` override (runtime/ops.py) recognises the
buffer when FSDP2's own copy-out arrives, makes the compute stream wait for that early copy and copies nothing.

Stream safety. The parameter tensors are allocated while the compute stream is current, so their memory may have been
released by compute work that is still queued; the copy stream therefore waits for the compute stream's work queued
up to the allocation before it writes, and the tensors are marked as used by the copy stream before FSDP2 can free
them. The all-gather buffer stays alive in FSDP2's hands until its own copy-out call has returned.

This reaches into torch 2.11's FSDP2 internals (`_fsdp_param_group.FSDPParamGroup.unshard`, `AllGatherResult`,
`FSDPParam.init_all_gather_outputs / alloc_all_gather_outputs`); `install()` checks that they are there and does
nothing otherwise. The reference leaves the copy where FSDP2 puts it (qwen3_triton/runtime/ops.py:116-127).
"""
import torch

_state = dict(installed=False, enabled=False, stream=None, done={}, copies=0, original=None, gatherer=None,
              delivered=0)


def pending_event(all_gather_output):
    """The event of an early copy of this buffer (and forget it), or None."""
    return _state['done'].pop(all_gather_output.data_ptr(), None)


def statistics():
    return dict(enabled=_state['enabled'], early_copies=_state['copies'], direct_deliveries=_state['delivered'])


def deliver_through(gatherer):
    """With a runtime/peer_gather.py:PeerAllGather given here (and the wrapper installed), an all-gather is finished by
    the wrapper: every rank's piece of every parameter is copied straight into the parameter's tensor, and FSDP2's
    split-copy finds nothing left to do. None: back to rank-major rows and a split-copy."""
    if _state['gatherer'] is not None:
        _state['gatherer'].direct = False
    _state['gatherer'] = gatherer if (gatherer is not None and _state['installed']) else None
    if _state['gatherer'] is not None:
        _state['gatherer'].direct = True
    return _state['gatherer'] is not None


def enable(flag=True):
    _state['enabled'] = bool(flag) and _state['installed']
    if not _state['enabled']:
        _state['done'].clear()
    return _state['enabled']


def install():
    """Wrap FSDPParamGroup.unshard once. Returns True if the early copy-out is available."""
    if _state['installed']:
        return True
    try:
        from torch.distributed.fsdp._fully_shard import _fsdp_param_group as pg
        from torch.distributed.fsdp._fully_shard._fsdp_param import FSDPParam
        group_class = pg.FSDPParamGroup
        needed = (hasattr(group_class, 'unshard') and hasattr(group_class, 'wait_for_unshard')
                  and hasattr(FSDPParam, 'init_all_gather_outputs') and hasattr(FSDPParam, 'alloc_all_gather_outputs'))
    except Exception:
        needed = False
    if not needed:
        return False
    original = group_class.unshard

    def unshard(self, async_op=False):
        had_result = self._all_gather_result is not None
        original(self, async_op)
        gatherer = _state['gatherer']
        if gatherer is not None and gatherer.deferred is not None:
            _deliver_now(self, gatherer)          # must run: the hook left the rows of this all-gather uncopied
        elif _state['enabled'] and not had_result:
            try:
                _copy_out_now(self)
            except Exception:
                enable(False)          # anything unexpected: leave the copy to FSDP2 from here on
                raise

    group_class.unshard = unshard
    _state['original'] = original
    _state['installed'] = True
    return True


def _outputs_of(group, result, world, device):
    """The unit's parameter tensors, allocated now (FSDP2's copy-out makes the same calls later and finds them)."""
    outs = []
    for numels, dtypes, fsdp_param in zip(result.param_all_gather_input_numels, result.param_all_gather_input_dtypes,
                                          group.fsdp_params):
        fsdp_param.init_all_gather_outputs(numels, dtypes, world, device, force_recreate=False)
        fsdp_param.alloc_all_gather_outputs()
        outs.extend(fsdp_param.all_gather_outputs)
    return outs


def _deliver_now(group, gatherer):
    result = group._all_gather_result
    stream = gatherer.deferred['stream']
    output = result.all_gather_output if result is not None else None
    usable = (result is not None and result.all_gather_event is not None and result.all_gather_work is None
              and output.data_ptr() == gatherer.deferred['output']
              and all(p.fsdp_placement.dim == 0 for p in group.fsdp_params))
    if not usable:
        event = gatherer.deliver([], [None])          # rows into the rank-major buffer
        if result is not None:
            with torch.cuda.stream(stream):
                group._all_gather_result = result._replace(all_gather_event=stream.record_event())
        return
    world = group._all_gather_process_group.size()
    outs = _outputs_of(group, result, world, output.device)
    compute = torch.cuda.current_stream(output.device)
    if stream != compute:
        stream.wait_stream(compute)                   # the outputs' memory is free in compute-stream order only
    event = gatherer.deliver(list(result.all_gather_input_split_sizes), outs)
    if event is None:                                 # rows copied instead: FSDP2 splits them, after this event
        with torch.cuda.stream(stream):
            group._all_gather_result = result._replace(all_gather_event=stream.record_event())
        return
    for t in outs:
        t.record_stream(stream)
    group._all_gather_result = result._replace(all_gather_event=event)
    _state['done'][output.data_ptr()] = event         # the split-copy override: nothing left to copy
    _state['delivered'] += 1


def _copy_out_now(group):
    from .ops import launch_split_copy
    result = group._all_gather_result
    if result is None or result.all_gather_event is None or result.all_gather_work is not None:
        return
    output = result.all_gather_output
    _state['done'].pop(output.data_ptr(), None)      # nothing left over from an earlier buffer at this address
    if not output.is_cuda or not result.all_gather_input_split_sizes:
        return
    world = group._all_gather_process_group.size()
    if world < 2 or any(p.fsdp_placement.dim != 0 for p in group.fsdp_params):
        return
    outs = _outputs_of(group, result, world, output.device)
    views = [t.view(world, -1) for t in outs]
    compute = torch.cuda.current_stream(output.device)
    stream = _state['stream']
    if stream is None or stream.device != output.device:
        stream = _state['stream'] = torch.cuda.Stream(device=output.device)
    stream.wait_stream(compute)                      # the outputs' memory is free in compute-stream order only
    stream.wait_event(result.all_gather_event)
    with torch.cuda.stream(stream):
        if not launch_split_copy(output.view(world, -1), list(result.all_gather_input_split_sizes), views):
            return                                   # shapes the kernel does not take: FSDP2 copies as usual
        event = torch.cuda.Event()
        event.record()
    for t in outs:
        t.record_stream(stream)
    _state['done'][output.data_ptr()] = event
    _state['copies'] += 1
