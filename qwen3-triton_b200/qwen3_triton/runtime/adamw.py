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

    def _rows_of(self, group):
        """(table rows, total blocks, device, tensors the kernel will modify) for the parameters that have a gradient."""
        rows, touched, blocks, device = [], [], 0, None
        for parameter in group['params']:
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
        (gradients re-allocated), since uploading it costs a synchronising copy."""
        key = tuple(r[:columns] for r in rows)
        cached = self._tables.get(index)
        if cached is None or cached[0] != key:
            meta = torch.tensor(key, dtype=torch.int64).to(device)
            coeff = torch.empty((len(rows), 3), device=device, dtype=torch.float32)
            cached = self._tables[index] = (key, meta, coeff)
        return cached[1], cached[2]

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if getattr(self, 'grad_scale', None) is not None or getattr(self, 'found_inf', None) is not None:
            raise ValueError('GradScaler is not supported by this explicit BF16/FP32 path')
        for index, group in enumerate(self.param_groups):
            rows, blocks, device, touched = self._rows_of(group)
            if not rows:
                continue
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
        self.kernel_steps += 1
        return loss


AdamW = TritonAdamW
