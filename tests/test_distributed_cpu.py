"""Host-side logic of the multi-GPU path on CPU: the collective backend and the FSDP2 hook objects with two
gloo ranks, the checkpoint / retention policy helpers, and the vocabulary-parallel statistics algebra."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent

WORKER = textwrap.dedent('''
    import sys, torch, torch.distributed as dist
    sys.path.insert(0, r"%s")
    from qwen3_triton.runtime.collectives import NcclCollectives, TritonCollectives
    from qwen3_triton.runtime.fsdp import TritonAllGather, TritonReduceScatter
    dist.init_process_group("gloo")
    r, w = dist.get_rank(), dist.get_world_size()
    comm = NcclCollectives()
    assert TritonCollectives is NcclCollectives and comm.world == 2
    # all-gather: every coordinate against the expected value, several sizes and dtypes
    for dtype in (torch.bfloat16, torch.float32, torch.int64):
        for n in (1, 7, 1031):
            src = (torch.arange(n) + 1000 * r).to(dtype)
            out = torch.empty(w * n, dtype=dtype)
            comm.all_gather(out, src)
            exp = torch.cat([(torch.arange(n) + 1000 * k).to(dtype) for k in range(w)])
            assert torch.equal(out, exp), (dtype, n)
    # reduce-scatter avg / sum in fp32
    for op in ("avg", "sum"):
        src = torch.arange(8, dtype=torch.float32) * (r + 1)
        out = torch.empty(4)
        comm.reduce_scatter(out, src, op)
        full = torch.arange(8, dtype=torch.float32) * 3 / (2 if op == "avg" else 1)
        assert torch.allclose(out, full.view(2, 4)[r]), op
    t = torch.tensor([float(r), 5.0 - r]); comm.all_reduce(t, "max"); assert t.tolist() == [1.0, 5.0]
    a = torch.arange(4.) + 10 * r; b = torch.empty(4); comm.all_to_all(b, a)
    assert b.tolist() == [0. + 2 * r, 1. + 2 * r, 10. + 2 * r, 11. + 2 * r]
    # FSDP2 hook protocol
    ag, rs = TritonAllGather(comm), TritonReduceScatter(comm)
    buf = ag.allocate((6,), dtype=torch.bfloat16, device=torch.device("cpu"))
    ag(buf, torch.full((3,), float(r), dtype=torch.bfloat16), dist.group.WORLD)
    assert buf.tolist() == [0, 0, 0, 1, 1, 1] and ag.calls == 1
    out = torch.empty(2); rs(out, torch.ones(4) * (r + 1), dist.group.WORLD, dist.ReduceOp.AVG)
    assert out.tolist() == [1.5, 1.5]
    for bad in (lambda: ag(buf, buf[:3], dist.group.WORLD, async_op=True),
                lambda: rs(out, torch.ones(4), dist.group.WORLD, dist.ReduceOp.MAX),
                lambda: comm.all_gather(torch.empty(5), torch.ones(2)),
                lambda: comm.reduce_scatter(torch.empty(2), torch.ones(4), "median")):
        try:
            bad(); raise SystemExit("expected ValueError")
        except ValueError:
            pass
    rep = comm.report(); assert rep["calls"]["gather"] == 10 and rep["world"] == 2
    comm.close()
    try:
        comm.barrier(); raise SystemExit("closed communicator must refuse")
    except RuntimeError:
        pass
    dist.barrier(); dist.destroy_process_group(); sys.stdout.write("rank" + str(r) + "ok" + chr(10)); sys.stdout.flush()
''') % str(ROOT / "qwen3-triton_b200")


def test_collectives_and_fsdp_hooks_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, OMP_NUM_THREADS="1")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)], capture_output=True,
                         text=True, timeout=240, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "rank0ok" in res.stdout and "rank1ok" in res.stdout


def test_checkpoint_and_retention_policy_helpers():
    from qwen3_triton.training.sharding import canonical_parameter_name, checkpoint_layer_indices
    assert checkpoint_layer_indices(4, every=1) == (0, 1, 2, 3)
    assert checkpoint_layer_indices(5, every=2) == (0, 2, 4)
    assert checkpoint_layer_indices(3, all_layers=True) == (0, 1, 2)
    assert checkpoint_layer_indices(3) == ()
    with pytest.raises(ValueError):
        checkpoint_layer_indices(3, all_layers=True, every=1)
    with pytest.raises(ValueError):
        checkpoint_layer_indices(0)
    assert canonical_parameter_name('model.layers.0._checkpoint_wrapped_module.mlp.up_proj.weight') == 'model.layers.0.mlp.up_proj.weight'


def test_vocab_parallel_statistics_algebra():
    """The two-all-reduce scheme (MAX of shard LSEs, then SUM of exp(lse_local - max) and of the owned target
    logit) reproduces the full cross-entropy: checked here with plain tensors standing in for the ranks."""
    g = torch.Generator().manual_seed(0)
    n, V, W = 9, 40, 4
    logits, labels = torch.randn(n, V, generator=g) * 3, torch.randint(0, V, (n,), generator=g)
    shards = logits.view(n, W, V // W)
    lse_local = torch.logsumexp(shards, dim=2)                      # [n, W]
    owner = labels // (V // W)
    target = torch.stack([torch.where(owner == r, shards[torch.arange(n), r, labels % (V // W)], torch.zeros(n)) for r in range(W)], 1)
    maximum = lse_local.max(dim=1).values                             # all-reduce MAX
    packed = torch.stack([torch.exp(lse_local - maximum[:, None]).sum(1), target.sum(1)])   # all-reduce SUM
    lse = maximum + torch.log(packed[0])
    loss = (lse - packed[1]).mean()
    torch.testing.assert_close(loss, torch.nn.functional.cross_entropy(logits, labels))


def test_fsdp_pack_plans_against_reference_semantics():
    """The table builders of runtime/ops.py, executed by a plain-Python interpreter of the table, reproduce
    torch's own all_gather copy-in, split_with_sizes_copy and _chunk_cat on CPU tensors."""
    import ctypes
    from qwen3_triton.runtime import ops

    def run(table, src_dtype, dst_dtype):
        for src, dst, r, c, ss, ds, valid, _vec in table:
            s = torch.frombuffer((ctypes.c_char * (max(valid, 1) * src_dtype.itemsize)).from_address(src), dtype=src_dtype)
            n_dst = (r - 1) * ds + c
            d = torch.frombuffer((ctypes.c_char * (n_dst * dst_dtype.itemsize)).from_address(dst), dtype=dst_dtype)
            for i in range(r):
                for j in range(c):
                    k = i * ss + j
                    d[i * ds + j] = s[k].to(dst_dtype) if k < valid else 0

    g = torch.Generator().manual_seed(0)
    world, rank = 4, 2
    shards = [torch.randn(n, generator=g) for n in (5, 12, 1)]
    out = torch.zeros(world * 18, dtype=torch.bfloat16)
    table, total = ops.finalize(ops.plan_copy_in([5, 12, 1], out.data_ptr(), 2, rank, [t.data_ptr() for t in shards]))
    run(table, torch.float32, torch.bfloat16)
    assert total == 18 and torch.equal(out[36:54], torch.cat(shards).to(torch.bfloat16)) and out[:36].abs().sum() == 0

    gathered = torch.randn(world, 18, generator=g).to(torch.bfloat16)
    outs = [torch.zeros(world, n, dtype=torch.bfloat16) for n in (5, 12, 1)]
    table, _ = ops.finalize(ops.plan_split(gathered.data_ptr(), 2, world, [5, 12, 1], [o.data_ptr() for o in outs]))
    run(table, torch.bfloat16, torch.bfloat16)
    for o, ref in zip(outs, torch.split(gathered, [5, 12, 1], dim=1)):
        assert torch.equal(o, ref)

    grads = [torch.randn(s, generator=g).to(torch.bfloat16) for s in ((6, 3), (5, 2), (9,), (1, 4))]   # 5, 9, 1 need padding
    rows, cols = ops.plan_chunk_cat([tuple(t.shape) for t in grads], [t.data_ptr() for t in grads], 0, 4, world)
    ref = torch.zeros(world, cols)
    torch._chunk_cat([t.float() for t in grads], 0, world, out=ref)
    got = torch.full((world, cols), float('nan'))
    rows, _ = ops.plan_chunk_cat([tuple(t.shape) for t in grads], [t.data_ptr() for t in grads], got.data_ptr(), 4, world)
    table, _ = ops.finalize(rows)
    run(table, torch.bfloat16, torch.float32)
    assert torch.equal(got, ref)


def test_peer_reduce_layout_bf16_staging_then_ordered_fp32_sum():
    """The data path of the peer-memory gradient reduction, restated on the CPU: every rank packs its bf16 gradients
    with the chunk-cat table into a [world, columns] bf16 staging buffer; rank r's result is the fp32 sum, in rank
    order, of row r of every rank's buffer, times 1/world. It must equal what FSDP2 computes: chunk-cat with upcast
    into fp32, then an averaging reduce-scatter (here: the mean over ranks of row r)."""
    import ctypes
    from qwen3_triton.runtime import ops

    def run(table, src_dtype, dst_dtype):
        for src, dst, r, c, ss, ds, valid, _vec in table:
            s = torch.frombuffer((ctypes.c_char * (max(valid, 1) * src_dtype.itemsize)).from_address(src), dtype=src_dtype)
            d = torch.frombuffer((ctypes.c_char * (((r - 1) * ds + c) * dst_dtype.itemsize)).from_address(dst), dtype=dst_dtype)
            for i in range(r):
                for j in range(c):
                    k = i * ss + j
                    d[i * ds + j] = s[k].to(dst_dtype) if k < valid else 0

    world = 4
    shapes = ((8, 3), (6, 2), (9,), (4, 4))                      # 6 and 9 rows need padding to the world size
    g = torch.Generator().manual_seed(3)
    grads = [[torch.randn(s, generator=g).to(torch.bfloat16) for s in shapes] for _ in range(world)]
    staged, reference = [], []
    for rank_grads in grads:
        _, cols = ops.plan_chunk_cat([tuple(t.shape) for t in rank_grads], [t.data_ptr() for t in rank_grads], 0, 2, world)
        buf = torch.full((world, cols), float('nan'), dtype=torch.bfloat16)
        rows, _ = ops.plan_chunk_cat([tuple(t.shape) for t in rank_grads], [t.data_ptr() for t in rank_grads],
                                     buf.data_ptr(), 2, world)
        run(ops.finalize(rows)[0], torch.bfloat16, torch.bfloat16)
        staged.append(buf)
        ref = torch.zeros(world, cols)
        torch._chunk_cat([t.float() for t in rank_grads], 0, world, out=ref)
        reference.append(ref)
    for r in range(world):
        pulled = torch.zeros(staged[0].shape[1])
        for buf in staged:                                        # rank order, fp32 accumulation
            pulled = pulled + buf[r].float()
        pulled = pulled * (1.0 / world)
        want = torch.stack([ref[r] for ref in reference]).sum(0) / world
        torch.testing.assert_close(pulled, want, rtol=1e-6, atol=1e-7)
        assert not torch.isnan(pulled).any()


def test_unshard_wrapper_finds_the_fsdp2_internals_it_needs():
    """runtime/early_copy_out.py reaches into FSDP2 (FSDPParamGroup.unshard, FSDPParam.init/alloc_all_gather_outputs,
    AllGatherResult as a named tuple with an `all_gather_event` field). With this torch they must be there; the wrapper
    is installed once, is inactive until enabled, and delivers nothing without a gatherer."""
    from torch.distributed.fsdp._fully_shard._fsdp_collectives import AllGatherResult
    from torch.distributed.fsdp._fully_shard._fsdp_param_group import FSDPParamGroup
    from qwen3_triton.runtime import early_copy_out as eco
    before = FSDPParamGroup.unshard
    assert eco.install() is True
    wrapped = FSDPParamGroup.unshard
    assert eco.install() is True and FSDPParamGroup.unshard is wrapped          # idempotent
    assert wrapped is not before
    stats = eco.statistics()
    assert stats['enabled'] is False and stats['early_copies'] == 0 and stats['direct_deliveries'] == 0
    assert eco.deliver_through(None) is False
    assert {'all_gather_output', 'all_gather_event', 'all_gather_work', 'param_all_gather_input_numels',
            'param_all_gather_input_dtypes', 'all_gather_input_split_sizes'} <= set(AllGatherResult._fields)
    assert eco.pending_event(torch.zeros(1)) is None
