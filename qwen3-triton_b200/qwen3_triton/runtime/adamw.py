"""FP32 multi-tensor AdamW for local Tensor / DTensor shards: one kernel launch per parameter group.

The Python Optimizer keeps parameter-group and state bookkeeping; step counters, bias corrections,
moments, decoupled decay and the parameter update run in the q3_adamw_multi kernels. Same surface as the
reference qwen3_triton/runtime/adamw.py:64-159 (class name kept so call sites do not change): state keys
`step` (fp32 0-d tensor on the device), `exp_avg`, `exp_avg_sq`; rejects non-fp32 tensors and GradScaler;
bumps autograd version counters after the in-place update.
"""
import copy
from typing import NamedTuple

import torch

from .. import _abi


def local(tensor):
    return tensor.to_local() if hasattr(tensor, 'to_local') else tensor


STATE_KEYS = ('step', 'exp_avg', 'exp_avg_sq')
UNSUPPORTED_MODES = ('amsgrad', 'maximize', 'differentiable', 'capturable')


class _Row(NamedTuple):
    """One parameter's line of the device pointer table (q3_adamw_multi / q3_adamw_multi_mp column order)."""
    param: int
    grad: int            # fp32 gradient, or 0 when a low-precision gradient is given
    exp_avg: int
    exp_avg_sq: int
    step: int
    numel: int
    first_block: int
    lowp_grad: int = 0   # bf16/fp16 gradient read directly (single-GPU mixed precision)
    lowp_copy: int = 0   # bf16/fp16 working copy refreshed in the same pass
    lowp_dtype: int = 0


def _fp32_cuda_contiguous(t):
    return t.dtype == torch.float32 and t.is_cuda and t.is_contiguous()


class TritonAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-5, betas=(.9, .999), eps=1e-8, weight_decay=.01, *, block=4096):
        if not 0 <= lr or not 0 <= eps or not 0 <= weight_decay or not all(0 <= b < 1 for b in betas):
            raise ValueError('Invalid AdamW scalar configuration')
        if block not in (1024, 2048, 4096, 8192, 16384):
            raise ValueError('Explicit supported block required')
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.block = block
        self.kernel_steps = 0
        self._tables = {}
        self._pending_streams, self._pending_calls = [], 0

    # ------------------------------------------------------------------------------------------ restore
    def _checked_entry(self, parameter, entry):
        """The (step, exp_avg, exp_avg_sq) tensors of one checkpoint entry, validated against the local shard."""
        if set(entry) != set(STATE_KEYS):
            raise ValueError('Expected plain FP32 AdamW checkpoint state')
        shard = local(parameter)
        tensors = []
        for key in STATE_KEYS:
            t = local(entry[key])
            if t.dtype != torch.float32 or not t.is_contiguous():
                raise ValueError('Contiguous FP32 checkpoint state required before upload')
            if t.numel() != 1 if key == 'step' else t.shape != shard.shape:
                raise ValueError('Local checkpoint shape differs')
            if t.device.type != 'cpu' and t.device != shard.device:
                raise ValueError('Load CPU or same-device local shards only')
            tensors.append(t)
        return tensors

    def load_state_dict(self, state_dict):
        """Restore in two passes: first check the whole checkpoint against the current groups and shards without
        touching the device, then copy tensor by tensor into the buffers this optimizer already holds (allocating
        only what is missing). The stock Optimizer.load_state_dict builds a complete second state on the device
        before dropping the old one - a transient extra copy of both moments (reference
        qwen3_triton/runtime/adamw.py:76-115 avoids the same thing)."""
        state_dict = dict(state_dict)
        for hook in self._optimizer_load_state_dict_pre_hooks.values():
            state_dict = hook(self, state_dict) or state_dict
        saved_groups = copy.deepcopy(state_dict['param_groups'])
        if [len(g['params']) for g in saved_groups] != [len(g['params']) for g in self.param_groups]:
            raise ValueError('Optimizer checkpoint group layout differs')
        pending, groups = [], []
        for saved, current in zip(saved_groups, self.param_groups):
            if any(saved.get(mode) for mode in UNSUPPORTED_MODES):
                raise ValueError('Unsupported optimizer checkpoint mode')
            groups.append({**saved, 'params': current['params']})
            for saved_id, parameter in zip(saved['params'], current['params']):
                entry = state_dict['state'].get(saved_id)
                if entry:
                    pending.append((parameter, self._checked_entry(parameter, entry)))
        restored, touched = {}, []
        for parameter, tensors in pending:
            device = local(parameter).device
            held = self.state.get(parameter, {})
            slot = {}
            for key, source in zip(STATE_KEYS, tensors):
                buffer = local(held[key]) if key in held else None
                reusable = (buffer is not None and buffer.shape == source.shape and buffer.device == device
                            and buffer.dtype == torch.float32)
                if not reusable:
                    buffer = torch.empty(source.shape, device=device, dtype=torch.float32)
                buffer.copy_(source)
                slot[key] = buffer
                touched.append(buffer)
            restored[parameter] = slot
        if touched:
            torch.autograd.graph.increment_version(touched)
        self.__setstate__({'state': restored, 'param_groups': groups})
        self._tables = {}
        for hook in self._optimizer_load_state_dict_post_hooks.values():
            hook(self)

    # ------------------------------------------------------------------------------------------ step
    def _state_for(self, parameter, shard):
        state = self.state[parameter]
        if not state:
            state['step'] = torch.zeros((), device=shard.device, dtype=torch.float32)
            state['exp_avg'] = torch.zeros(shard.shape, device=shard.device, dtype=torch.float32)
            state['exp_avg_sq'] = torch.zeros(shard.shape, device=shard.device, dtype=torch.float32)
        m, v, step = local(state['exp_avg']), local(state['exp_avg_sq']), state['step']
        if (m.shape != shard.shape or v.shape != shard.shape or m.dtype != torch.float32 or v.dtype != torch.float32
                or step.dtype != torch.float32 or step.numel() != 1 or step.device != shard.device):
            raise ValueError('Invalid local FP32 AdamW state')
        return m, v, step

    def _rows_of(self, parameters):
        """(table rows, total blocks, device, tensors the kernel will modify) for the parameters that have a gradient."""
        rows, touched, blocks, device = [], [], 0, None
        for parameter in parameters:
            low_g = getattr(parameter, 'q3_lowp_grad', None)      # set by runtime/mixed_precision.py
            low_p = getattr(parameter, 'q3_lowp_copy', None)
            if parameter.grad is None and low_g is None:
                continue
            shard = local(parameter)
            grad = local(parameter.grad) if low_g is None else None
            if not _fp32_cuda_contiguous(shard) or (grad is not None and (
                    not _fp32_cuda_contiguous(grad) or grad.device != shard.device or grad.shape != shard.shape
                    or grad.is_sparse)):
                raise ValueError('Matching contiguous local CUDA FP32 parameter/gradient required')
            for low in (low_g, low_p):
                if low is not None and (low.dtype not in (torch.bfloat16, torch.float16) or low.shape != shard.shape
                                        or low.device != shard.device or not low.is_contiguous()):
                    raise ValueError('Low-precision gradient / working copy must match the FP32 parameter')
            if device not in (None, shard.device):
                raise ValueError('One CUDA device per group')
            device = shard.device
            if not shard.numel():
                continue
            m, v, step = self._state_for(parameter, shard)
            low = low_g if low_g is not None else low_p
            rows.append(_Row(shard.data_ptr(), grad.data_ptr() if grad is not None else 0, m.data_ptr(), v.data_ptr(),
                             step.data_ptr(), shard.numel(), blocks, _abi.ptr(low_g) or 0, _abi.ptr(low_p) or 0,
                             _abi.dt(low.dtype) if low is not None else 0))
            blocks += -(-shard.numel() // self.block)
            touched += [parameter, m, v, step] + ([shard] if shard is not parameter else [])
        return rows, blocks, device, touched

    def _device_table(self, index, rows, columns, device):
        """Pointer table and per-tensor coefficient scratch on the device; rebuilt only when a pointer changed
        (gradients re-allocated). The upload goes through a pinned buffer and is asynchronous on the launching
        stream, so that a changed pointer never stalls the host behind that stream's queued work."""
        key = tuple(r[:columns] for r in rows)
        cached = self._tables.get(index)
        if cached is None or cached['key'] != key:
            if cached is None or cached['meta'].shape != (len(rows), columns):
                cached = self._tables[index] = dict(
                    host=torch.empty((len(rows), columns), dtype=torch.int64, pin_memory=True),
                    meta=torch.empty((len(rows), columns), dtype=torch.int64, device=device),
                    coeff=torch.empty((len(rows), 3), device=device, dtype=torch.float32), uploaded=None)
            if cached['uploaded'] is not None:
                cached['uploaded'].synchronize()           # the previous upload has long finished reading `host`
            cached['host'].copy_(torch.tensor(key, dtype=torch.int64))
            cached['meta'].copy_(cached['host'], non_blocking=True)
            cached['uploaded'] = torch.cuda.Event()
            cached['uploaded'].record()
            cached['key'] = key
        return cached['meta'], cached['coeff']

    def _launch(self, index, group, parameters):
        """One kernel launch on the current stream over those of `parameters` that have a gradient."""
        rows, blocks, device, touched = self._rows_of(parameters)
        if not rows:
            return
        low_dtypes = {r.lowp_dtype for r in rows if r.lowp_dtype}
        if len(low_dtypes) > 1:
            raise ValueError('One low-precision dtype per group')
        beta1, beta2 = group['betas']
        scalars = (float(group['lr']), float(beta1), float(beta2), float(group['weight_decay']), float(group['eps']))
        if low_dtypes:
            meta, coeff = self._device_table(index, rows, 9, device)
            every_row_both = int(all(r.lowp_grad and r.lowp_copy for r in rows))
            _abi.call('q3_adamw_multi_mp', meta.data_ptr(), coeff.data_ptr(), len(rows), blocks, self.block,
                      low_dtypes.pop(), every_row_both, *scalars, _abi.stream())
        else:
            meta, coeff = self._device_table(index, rows, 7, device)
            _abi.call('q3_adamw_multi', meta.data_ptr(), coeff.data_ptr(), len(rows), blocks, self.block, *scalars,
                      _abi.stream())
        torch.autograd.graph.increment_version(touched)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if getattr(self, 'grad_scale', None) is not None or getattr(self, 'found_inf', None) is not None:
            raise ValueError('GradScaler is not supported by this explicit BF16/FP32 path')
        for index, group in enumerate(self.param_groups):
            self._launch(index, group, group['params'])
        early = getattr(self, '_early', None)
        if early is not None:
            early.join()
        for stream in self._pending_streams:
            torch.cuda.current_stream(stream.device).wait_stream(stream)
        self._pending_streams, self._pending_calls = [], 0
        self.kernel_steps += 1
        return loss

    @torch.no_grad()
    def step_pending(self, eligible=None):
        """Update, on the current stream, every parameter (of `eligible`, a collection of parameters, if given) that
        has a gradient right now, and drop those gradients. Only for parameters whose gradient is complete as soon as
        it exists (used once in the model), which holds for the shards FSDP assigns after a reduce-scatter. The
        next `step()` updates the rest and makes its stream wait for this one. For sharded training: called from the
        gradient reduce-scatter hook (runtime/fsdp.py, `before_reduce`), it updates the shards of the units reduced
        so far on the reduce-scatter stream, beside the backward pass of the units still to come. Same result as
        `step()` alone (see step_during_backward); same restrictions (one backward per step, no clipping)."""
        current = torch.cuda.current_stream()
        launched = False
        if eligible is not None and not isinstance(eligible, (set, frozenset)):
            eligible = {id(p) for p in eligible}
        for index, group in enumerate(self.param_groups):
            ready = [p for p in group['params'] if p.grad is not None and (eligible is None or id(p) in eligible)]
            if not ready:
                continue
            self._launch(('pending', self._pending_calls, index), group, ready)
            for parameter in ready:
                local(parameter.grad).record_stream(current)
                parameter.grad = None
            launched = True
        if launched:
            self._pending_calls += 1
            if all(current != s for s in self._pending_streams):
                self._pending_streams.append(current)
        return launched

    # ------------------------------------------------------------------------------ update during backward
    def step_during_backward(self, buckets, gradient_of=None):
        """Update each bucket of parameters on a side stream as soon as the backward pass has produced the bucket's
        last gradient, so that the update (bound by HBM bandwidth) runs beside the remaining backward GEMMs (bound by
        the tensor cores) instead of after them. `step()` then updates whatever is left (parameters in no bucket, or
        a bucket the backward pass did not complete) and makes the current stream wait for the side stream.

        `buckets`: lists of this optimizer's parameters, e.g. one per decoder layer; every member must get a
        gradient in every backward pass. `gradient_of(parameter)` returns the tensor whose `.grad` autograd fills for
        that parameter (the bf16 working copy under runtime/mixed_precision.py; default: the parameter itself) -
        when it is another tensor, its gradient is handed over as the parameter's `q3_lowp_grad` and cleared.

        The result is the one `step()` alone gives: per-parameter step counters live on the device, the kernel is
        elementwise, and a bucket is launched only after its last gradient is complete. Do not use with gradient
        accumulation over several backward passes or with gradient clipping (both need all gradients first);
        `early.enabled = False` on the returned object suspends it. The reference steps after backward only
        (qwen3_triton/runtime/adamw.py:117-159)."""
        if getattr(self, '_early', None) is not None:
            raise ValueError('step_during_backward was already set up')
        self._early = _EarlySteps(self, buckets, gradient_of or (lambda parameter: parameter))
        return self._early


class _EarlySteps:
    def __init__(self, optimizer, buckets, gradient_of):
        self.optimizer = optimizer
        self.enabled = True
        self.stream = None
        self.launched = 0
        self.handles = []
        group_of = {id(p): (i, g) for i, g in enumerate(optimizer.param_groups) for p in g['params']}
        seen = set()
        for number, bucket in enumerate(buckets):
            bucket = list(bucket)
            if not bucket:
                continue
            groups = {group_of[id(p)][0] if id(p) in group_of else None for p in bucket}
            if None in groups or len(groups) != 1:
                raise ValueError('A bucket holds parameters of one parameter group of this optimizer')
            if any(id(p) in seen for p in bucket):
                raise ValueError('A parameter belongs to one bucket')
            seen.update(id(p) for p in bucket)
            index, group = group_of[id(bucket[0])]
            state = dict(parameters=bucket, sources=[gradient_of(p) for p in bucket], waiting=len(bucket), group=group,
                         key=('early', number, index))
            for source in state['sources']:
                if not source.requires_grad:
                    raise ValueError('Every member of a bucket must receive a gradient')
                self.handles.append(source.register_post_accumulate_grad_hook(self._hook(state)))

    def _hook(self, state):
        def fire(_):
            if not self.enabled:
                return
            state['waiting'] -= 1
            if state['waiting'] == 0:
                state['waiting'] = len(state['parameters'])
                self._launch(state)
        return fire

    @torch.no_grad()
    def _launch(self, state):
        current = torch.cuda.current_stream()
        if self.stream is None or self.stream.device != current.device:
            self.stream = torch.cuda.Stream(device=current.device)
        for parameter, source in zip(state['parameters'], state['sources']):
            if source is not parameter:
                gradient = source.grad
                parameter.q3_lowp_grad = gradient if gradient.is_contiguous() else gradient.contiguous()
                source.grad = None
        self.stream.wait_stream(current)            # every gradient of the bucket was produced by work queued so far
        with torch.cuda.stream(self.stream):
            self.optimizer._launch(state['key'], state['group'], state['parameters'])
        for parameter, source in zip(state['parameters'], state['sources']):
            # the side stream still reads the gradient: keep its memory from being handed out before that
            if source is not parameter:
                parameter.q3_lowp_grad.record_stream(self.stream)
                parameter.q3_lowp_grad = None
            elif parameter.grad is not None:
                local(parameter.grad).record_stream(self.stream)
                parameter.grad = None
        self.launched += 1

    def join(self):
        if self.stream is not None:
            torch.cuda.current_stream(self.stream.device).wait_stream(self.stream)

    def remove(self):
        for handle in self.handles:
            handle.remove()
        self.handles = []
        self.join()
        self.optimizer._early = None


AdamW = TritonAdamW
