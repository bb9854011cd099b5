"""Single-GPU mixed precision: fp32 master parameters, bf16 working copies, fp32 gradients.

On one GPU there is no FSDP unit to do the casts, so this does what FSDP2's MixedPrecisionPolicy
(param_dtype=bf16, reduce_dtype=fp32) does around its collectives (reference training/fsdp/official.py:24):
before forward the fp32 master weights are cast into persistent bf16 tensors the model computes with; after
backward the bf16 gradients are upcast into the fp32 `.grad` of the masters, which the optimizer updates.
Both casts are q3_cast kernel launches.
"""
import torch

from .. import _abi


class MasterWeights:
    def __init__(self, model, compute_dtype=torch.bfloat16):
        """`model` holds fp32 parameters on the GPU. They become the masters; the model's parameters are
        replaced by compute-dtype tensors of the same shapes."""
        self.model = model
        self.compute_dtype = compute_dtype
        self.masters = []
        self.working = []
        seen = {}
        for module in model.modules():
            for name, p in list(module._parameters.items()):
                if p is None:
                    continue
                if id(p) in seen:                      # tied weights share one master
                    module._parameters[name] = seen[id(p)]
                    continue
                if p.dtype != torch.float32 or not p.is_cuda:
                    raise ValueError('fp32 CUDA parameters required')
                master = torch.nn.Parameter(p.detach())
                work = torch.nn.Parameter(torch.empty_like(p, dtype=compute_dtype), requires_grad=p.requires_grad)
                module._parameters[name] = work
                seen[id(p)] = work
                self.masters.append(master)
                self.working.append(work)
        self.fused = False
        self.sync_working()

    def fuse_into_optimizer(self):
        """Let TritonAdamW read the bf16 gradients directly and refresh the bf16 working copies in its own pass:
        after this, `sync_working()` and `collect_grads()` launch nothing."""
        self.fused = True
        for m, w in zip(self.masters, self.working):
            m.q3_lowp_copy = w.data
        return self

    def parameters(self):
        return self.masters

    def masters_of(self, module):
        """The fp32 masters of `module`'s (working) parameters, in `module.parameters()` order."""
        master_of = {id(w): m for m, w in zip(self.masters, self.working)}
        return [master_of[id(w)] for w in module.parameters() if id(w) in master_of]

    def working_of(self, master):
        """The working copy autograd fills the gradient of (TritonAdamW.step_during_backward's `gradient_of`)."""
        if not hasattr(self, '_working_of'):
            self._working_of = {id(m): w for m, w in zip(self.masters, self.working)}
        return self._working_of[id(master)]

    def release_grads(self):
        """Drop the low-precision gradients handed to the optimizer (call after optimizer.step()): otherwise they stay
        alive through the next backward, next to the new ones."""
        for m in self.masters:
            m.q3_lowp_grad = None

    @torch.no_grad()
    def sync_working(self):
        """master (fp32) -> working (bf16)."""
        if self.fused and getattr(self, '_synced_once', False):
            return
        self._synced_once = True
        for m, w in zip(self.masters, self.working):
            _abi.call('q3_cast', m.data_ptr(), _abi.Q3_F32, w.data_ptr(), _abi.dt(self.compute_dtype), m.numel(),
                      _abi.stream())

    @torch.no_grad()
    def collect_grads(self):
        """working.grad (bf16) -> master.grad (fp32); frees the bf16 gradient."""
        if self.fused:
            for m, w in zip(self.masters, self.working):
                m.q3_lowp_grad = w.grad.contiguous() if w.grad is not None else None
                w.grad = None
            return
        for m, w in zip(self.masters, self.working):
            if w.grad is None:
                m.grad = None
                continue
            if m.grad is None:
                m.grad = torch.empty_like(m)
            g = w.grad.contiguous()
            _abi.call('q3_cast', g.data_ptr(), _abi.dt(g.dtype), m.grad.data_ptr(), _abi.Q3_F32, g.numel(), _abi.stream())
            w.grad = None
