"""FP32 multi-tensor AdamW for local Tensor / DTensor shards: one kernel launch per parameter group.

The Python Optimizer keeps parameter-group and state bookkeeping; step counters, bias corrections,
moments, decoupled decay and the parameter update run in the q3_adamw_multi kernels. Same surface as the
reference qwen3_triton/runtime/adamw.py:64-159 (class name kept so call sites do not change): state keys
`step` (fp32 0-d tensor on the device), `exp_avg`, `exp_avg_sq`; rejects non-fp32 tensors and GradScaler;
bumps autograd version counters after the in-place update.
"""
import copy
from collections import defaultdict

import torch

from .. import _abi


def local(tensor):
    return tensor.to_local() if hasattr(tensor, 'to_local') else tensor


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

    def load_state_dict(self, state_dict):
        # Validate first, then reuse the existing device buffers and upload one tensor at a time, so a
        # restore never holds a second copy of the moments on the device.
        state_dict = state_dict.copy()
        for hook in self._optimizer_load_state_dict_pre_hooks.values():
            changed = hook(self, state_dict)
            if changed is not None:
                state_dict = changed
        saved_groups = copy.deepcopy(state_dict['param_groups'])
        if len(saved_groups) != len(self.param_groups) or any(
                len(a['params']) != len(b['params']) for a, b in zip(saved_groups, self.param_groups)):
            raise ValueError('Optimizer checkpoint group layout differs')
        specifications = []
        groups = []
        for saved, current in zip(saved_groups, self.param_groups):
            if any(saved.get(key, False) for key in ['amsgrad', 'maximize', 'differentiable', 'capturable']):
                raise ValueError('Unsupported optimizer checkpoint mode')
            groups.append(dict(saved, params=current['params']))
            for saved_id, parameter in zip(saved['params'], current['params']):
                source_state = state_dict['state'].get(saved_id, {})
                if not source_state:
                    continue
                if set(source_state) != {'step', 'exp_avg', 'exp_avg_sq'}:
                    raise ValueError('Expected plain FP32 AdamW checkpoint state')
                p = local(parameter)
                for key in ['step', 'exp_avg', 'exp_avg_sq']:
                    source = local(source_state[key])
                    if source.dtype != torch.float32 or not source.is_contiguous():
                        raise ValueError('Contiguous FP32 checkpoint state required before upload')
                    if (key == 'step' and source.numel() != 1) or (key != 'step' and source.shape != p.shape):
                        raise ValueError('Local checkpoint shape differs')
                    if source.device.type != 'cpu' and source.device != p.device:
                        raise ValueError('Load CPU or same-device local shards only')
                specifications.append((parameter, source_state))
        restored = defaultdict(dict)
        versions = []
        for parameter, sources in specifications:
            p = local(parameter)
            previous = self.state.get(parameter, {})
            for key in ['step', 'exp_avg', 'exp_avg_sq']:
                source = local(sources[key])
                target = local(previous[key]) if key in previous else None
                if target is None or target.shape != source.shape or target.device != p.device or target.dtype != torch.float32:
                    target = torch.empty(source.shape, device=p.device, dtype=torch.float32)
                target.copy_(source)
                restored[parameter][key] = target
                versions.append(target)
        if versions:
            torch.autograd.graph.increment_version(versions)
        self.__setstate__(dict(state=restored, param_groups=groups))
        self._tables = {}
        for hook in self._optimizer_load_state_dict_post_hooks.values():
            hook(self)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if getattr(self, 'grad_scale', None) is not None or getattr(self, 'found_inf', None) is not None:
            raise ValueError('GradScaler is not supported by this explicit BF16/FP32 path')
        for index, group in enumerate(self.param_groups):
            rows = []
            blocks = 0
            device = None
            changed = []
            mixed = False
            for parameter in group['params']:
                # single-GPU mixed precision (runtime/mixed_precision.py): a bf16 gradient to read directly and/or
                # a bf16 working copy to refresh in the same pass
                low_g = getattr(parameter, 'q3_lowp_grad', None)
                low_p = getattr(parameter, 'q3_lowp_copy', None)
                if parameter.grad is None and low_g is None:
                    continue
                p = local(parameter)
                g = local(parameter.grad) if low_g is None else None
                if g is not None and (g.dtype != torch.float32 or p.device != g.device or not g.is_contiguous()
                                      or p.shape != g.shape or g.is_sparse):
                    raise ValueError('Matching contiguous local CUDA FP32 parameter/gradient required')
                if p.dtype != torch.float32 or not p.is_cuda or not p.is_contiguous():
                    raise ValueError('Matching contiguous local CUDA FP32 parameter/gradient required')
                for low in (low_g, low_p):
                    if low is not None and (low.dtype not in (torch.bfloat16, torch.float16) or low.shape != p.shape
                                            or low.device != p.device or not low.is_contiguous()):
                        raise ValueError('Low-precision gradient / working copy must match the FP32 parameter')
                mixed = mixed or low_g is not None or low_p is not None
                if device is not None and device != p.device:
                    raise ValueError('One CUDA device per group')
                device = p.device
                if not p.numel():
                    continue
                state = self.state[parameter]
                if not state:
                    state['step'] = torch.zeros((), device=device, dtype=torch.float32)
                    state['exp_avg'] = torch.zeros(p.shape, device=device, dtype=torch.float32)
                    state['exp_avg_sq'] = torch.zeros(p.shape, device=device, dtype=torch.float32)
                m, v = local(state['exp_avg']), local(state['exp_avg_sq'])
                step = state['step']
                if (m.shape != p.shape or v.shape != p.shape or m.dtype != torch.float32 or v.dtype != torch.float32
                        or step.dtype != torch.float32 or step.numel() != 1 or step.device != device):
                    raise ValueError('Invalid local FP32 AdamW state')
                rows.append((p.data_ptr(), g.data_ptr() if g is not None else 0, m.data_ptr(), v.data_ptr(), step.data_ptr(),
                             p.numel(), blocks, low_g.data_ptr() if low_g is not None else 0,
                             low_p.data_ptr() if low_p is not None else 0,
                             _abi.dt((low_g if low_g is not None else low_p).dtype) if (low_g is not None or low_p is not None) else 0))
                blocks += -(-p.numel() // self.block)
                changed.extend([parameter, m, v, step])
                if p is not parameter:
                    changed.append(p)
            if not rows:
                continue
            # The pointer table only changes when gradients are re-allocated; cache the device copy.
            lowp = {r[9] for r in rows if r[9]}
            if len(lowp) > 1:
                raise ValueError('One low-precision dtype per group')
            rows = [r[:9] if mixed else r[:7] for r in rows]
            key = tuple(rows)
            cached = self._tables.get(index)
            if cached is None or cached[0] != key:
                cpu = torch.tensor(rows, dtype=torch.int64)
                meta = torch.empty(cpu.shape, device=device, dtype=torch.int64)
                meta.copy_(cpu)
                coeff = torch.empty((len(rows), 3), device=device, dtype=torch.float32)
                cached = (key, meta, coeff)
                self._tables[index] = cached
            _, meta, coeff = cached
            b1, b2 = group['betas']
            if mixed:
                _abi.call('q3_adamw_multi_mp', meta.data_ptr(), coeff.data_ptr(), len(rows), blocks, self.block,
                          lowp.pop(), int(all(row[7] and row[8] for row in rows)), float(group['lr']), float(b1),
                          float(b2), float(group['weight_decay']), float(group['eps']), _abi.stream())
            else:
                _abi.call('q3_adamw_multi', meta.data_ptr(), coeff.data_ptr(), len(rows), blocks, self.block,
                          float(group['lr']), float(b1), float(b2), float(group['weight_decay']), float(group['eps']),
                          _abi.stream())
            torch.autograd.graph.increment_version(changed)
        self.kernel_steps += 1
        return loss


AdamW = TritonAdamW
