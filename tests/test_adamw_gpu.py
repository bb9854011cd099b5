"""Multi-tensor AdamW against the fp64 oracle and torch.optim.AdamW: non-zero initial moments, skipped and
zero gradients, odd tensor sizes, state_dict round trip, fp32-only enforcement."""
import pytest
import torch

import recipe
from oracle import ops as O

pytestmark = pytest.mark.gpu
HYPER = dict(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
SIZES = [(1,), (7,), (1031,), (4099,), (128, 130), (4096,), (3, 4097)]


def make_params(seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(*s, generator=g) for s in SIZES]


def test_matches_fp64_oracle_over_steps():
    from qwen3_triton.runtime.adamw import TritonAdamW
    cpu = make_params(1)
    params = [torch.nn.Parameter(p.clone().cuda()) for p in cpu]
    opt = TritonAdamW(params, **HYPER)
    ref = [(p.clone(), torch.zeros_like(p), torch.zeros_like(p)) for p in cpu]
    g = torch.Generator().manual_seed(2)
    steps = [0] * len(cpu)
    for it in range(1, 9):
        for i, p in enumerate(params):
            if i == 1 and it % 2 == 0:
                p.grad = None                       # skipped gradient: state must not advance
                continue
            grad = torch.zeros_like(cpu[i]) if (i == 2 and it == 3) else torch.randn(cpu[i].shape, generator=g) * 1e-2
            p.grad = grad.cuda()
            steps[i] += 1
            pp, m, v = ref[i]
            ref[i] = O.adamw_step(pp, grad, m, v, steps[i], HYPER['lr'], *HYPER['betas'], HYPER['eps'], HYPER['weight_decay'])
        opt.step()
    for i, p in enumerate(params):
        st = opt.state[p]
        assert float(st['step']) == steps[i] and st['step'].dtype == torch.float32 and st['step'].ndim == 0
        # AdamW state within 1e-5 (stated tolerance); observed differences are a few fp32 ulps
        torch.testing.assert_close(p.detach().cpu(), ref[i][0], rtol=1e-5, atol=1e-7)
        torch.testing.assert_close(st['exp_avg'].cpu(), ref[i][1], rtol=1e-5, atol=1e-9)
        torch.testing.assert_close(st['exp_avg_sq'].cpu(), ref[i][2], rtol=1e-5, atol=1e-12)


def test_matches_torch_adamw_and_state_dict_roundtrip():
    from qwen3_triton.runtime.adamw import TritonAdamW
    cpu = make_params(3)
    a = [torch.nn.Parameter(p.clone().cuda()) for p in cpu]
    b = [torch.nn.Parameter(p.clone()) for p in cpu]
    oa, ob = TritonAdamW(a, **HYPER), torch.optim.AdamW(b, **HYPER)
    g = torch.Generator().manual_seed(4)
    for it in range(6):
        for pa, pb in zip(a, b):
            grad = torch.randn(pb.shape, generator=g) * 1e-2
            pa.grad, pb.grad = grad.cuda(), grad.clone()
        oa.step()
        ob.step()
        if it == 2:                                   # save -> CPU -> restore into a fresh optimizer
            saved = {'state': {k: {n: t.detach().cpu().clone() for n, t in s.items()} for k, s in oa.state_dict()['state'].items()},
                     'param_groups': oa.state_dict()['param_groups']}
            oa = TritonAdamW(a, **HYPER)
            oa.load_state_dict(saved)
    for pa, pb in zip(a, b):
        torch.testing.assert_close(pa.detach().cpu(), pb.detach(), rtol=1e-5, atol=1e-7)
    assert oa.kernel_steps == 3


def test_rejects_bf16_and_gradscaler():
    from qwen3_triton.runtime.adamw import TritonAdamW
    p = torch.nn.Parameter(torch.zeros(8, device='cuda', dtype=torch.bfloat16))
    p.grad = torch.zeros_like(p)
    with pytest.raises(ValueError):
        TritonAdamW([p]).step()
    q = torch.nn.Parameter(torch.zeros(8, device='cuda'))
    q.grad = torch.zeros_like(q)
    opt = TritonAdamW([q])
    opt.grad_scale = torch.ones(1)
    with pytest.raises(ValueError):
        opt.step()


def test_version_counter_bumped():
    from qwen3_triton.runtime.adamw import TritonAdamW
    p = torch.nn.Parameter(torch.ones(64, device='cuda'))
    p.grad = torch.ones_like(p)
    before = p._version
    TritonAdamW([p]).step()
    assert p._version > before


def test_mixed_precision_fusion_is_bit_identical_to_separate_cast_passes():
    """bf16 gradients read directly + bf16 working copy written by the optimizer kernel == upcast pass, fp32
    AdamW, downcast pass."""
    from qwen3_triton.runtime.adamw import TritonAdamW
    from qwen3_triton.runtime.mixed_precision import MasterWeights

    def build():
        torch.manual_seed(7)
        net = torch.nn.Sequential(torch.nn.Linear(130, 257, bias=False), torch.nn.Linear(257, 64, bias=False)).cuda()
        mw = MasterWeights(net)
        return net, mw, TritonAdamW(mw.parameters(), **HYPER)

    net_a, mw_a, opt_a = build()
    net_b, mw_b, opt_b = build()
    mw_b.fuse_into_optimizer()
    g = torch.Generator().manual_seed(8)
    for _ in range(4):
        grads = [torch.randn(w.shape, generator=g).to(torch.bfloat16).cuda() * 1e-2 for w in mw_a.working]
        for mw, opt in ((mw_a, opt_a), (mw_b, opt_b)):
            mw.sync_working()
            for w, gr in zip(mw.working, grads):
                w.grad = gr.clone()
            mw.collect_grads()
            opt.step()
        mw_a.sync_working()
    for ma, mb, wa, wb in zip(mw_a.masters, mw_b.masters, mw_a.working, mw_b.working):
        assert torch.equal(ma, mb), float((ma - mb).abs().max())
        assert torch.equal(wa, wb) and wb.dtype == torch.bfloat16, float((wa.float() - wb.float()).abs().max())


@pytest.mark.parametrize('mixed', [True, False])
def test_updates_during_backward_equal_a_step_after_backward(mixed):
    """Buckets updated on a side stream as soon as their last gradient exists, the rest by step(): bit-identical
    parameters, moments and step counters to updating everything after backward - with bf16 working copies
    (gradients handed over from the working copies) and with plain fp32 parameters."""
    from qwen3_triton.runtime.adamw import TritonAdamW
    from qwen3_triton.runtime.mixed_precision import MasterWeights

    def build(early):
        torch.manual_seed(11)
        blocks = [torch.nn.Sequential(torch.nn.Linear(256, 384, bias=False), torch.nn.Linear(384, 256, bias=False))
                  for _ in range(3)]
        net = torch.nn.Sequential(*blocks, torch.nn.Linear(256, 32, bias=False)).cuda()
        if mixed:
            mw = MasterWeights(net).fuse_into_optimizer()
            opt = TritonAdamW(mw.parameters(), **HYPER)
            if early:
                handle = opt.step_during_backward([mw.masters_of(b) for b in blocks], mw.working_of)
        else:
            mw = None
            opt = TritonAdamW(net.parameters(), **HYPER)
            if early:
                handle = opt.step_during_backward([list(b.parameters()) for b in blocks])
        return net, mw, opt, (handle if early else None)

    def run(early):
        net, mw, opt, handle = build(early)
        g = torch.Generator().manual_seed(12)
        for _ in range(4):
            x = torch.randn(64, 256, generator=g).cuda()
            if mixed:
                mw.sync_working()
                net(x.to(torch.bfloat16)).float().square().mean().backward()
                mw.collect_grads()
                opt.step()
                mw.release_grads()
            else:
                net(x).square().mean().backward()
                opt.step()
                opt.zero_grad(set_to_none=True)
        torch.cuda.synchronize()
        if early:
            assert handle.launched == 4 * 3
        params = mw.masters if mixed else list(net.parameters())
        state = [(opt.state[p]['step'].clone(), opt.state[p]['exp_avg'].clone(), opt.state[p]['exp_avg_sq'].clone())
                 for p in params]
        return [p.detach().clone() for p in params], state, ([w.detach().clone() for w in mw.working] if mixed else [])

    late, early = run(False), run(True)
    for a, b in zip(late[0], early[0]):
        assert torch.equal(a, b)
    for sa, sb in zip(late[1], early[1]):
        assert all(torch.equal(x, y) for x, y in zip(sa, sb))
        assert float(sa[0]) == 4.0
    for a, b in zip(late[2], early[2]):
        assert torch.equal(a, b)


def test_step_pending_on_another_stream_then_step_equals_one_step():
    """step_pending(eligible) updates the eligible parameters that have a gradient on the current (side) stream and
    drops those gradients; step() updates the rest and waits for that stream: the same state as one step()."""
    from qwen3_triton.runtime.adamw import TritonAdamW

    def build():
        g = torch.Generator().manual_seed(21)
        params = [torch.nn.Parameter(torch.randn(s, generator=g).cuda()) for s in ((300, 70), (1024,), (64, 64), (5,))]
        return params, TritonAdamW(params, **HYPER)

    (pa, oa), (pb, ob) = build(), build()
    side = torch.cuda.Stream()
    g = torch.Generator().manual_seed(22)
    for _ in range(3):
        grads = [torch.randn(p.shape, generator=g).cuda() * 1e-2 for p in pa]
        for p, q, gr in zip(pa, pb, grads):
            p.grad, q.grad = gr.clone(), gr.clone()
        oa.step()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            assert ob.step_pending(pb[:2]) is True           # only the first two are eligible
            assert ob.step_pending(pb[:2]) is False          # nothing left with a gradient among them
        assert pb[0].grad is None and pb[1].grad is None and pb[2].grad is not None
        ob.step()
        ob.zero_grad(set_to_none=True)
        oa.zero_grad(set_to_none=True)
    torch.cuda.synchronize()
    for p, q in zip(pa, pb):
        assert torch.equal(p, q)
        for key in ('step', 'exp_avg', 'exp_avg_sq'):
            assert torch.equal(oa.state[p][key], ob.state[q][key]), key
        assert float(oa.state[p]['step']) == 3.0
