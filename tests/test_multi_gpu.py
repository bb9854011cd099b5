"""Two ranks on two GPUs (skipped on a single-GPU box): the vocabulary-parallel embedding against the full lookup
and the averaged full gradient; one training step of a small fused-layer model under FSDP2, with the embedding
gathered by FSDP and kept vocabulary-parallel, against an UNSHARDED copy of the same model run on the concatenated
batch of both ranks (loss of each rank's tokens, and the rank's shards of the embedding, lm_head and a decoder
matrix gradient, which FSDP averages over ranks); and the two sharded forms against each other (same loss, same
embedding-gradient shard, same loss after AdamW); and the gradient reduce-scatter by the pull kernel over peer memory
against the NCCL fp32 reduce-scatter (every shard bit-identical on two ranks). What the reference checks with its CPU-gathered fp64 average
(scripts/check_triton_fsdp_v14.py:22-100)."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu

WORKER = textwrap.dedent('''
    import os, sys, types, torch, torch.distributed as dist
    sys.path.insert(0, r"%s")
    from qwen3_triton import _abi, model_for_variant
    from qwen3_triton.runtime.adamw import TritonAdamW
    from qwen3_triton.runtime.collectives import NcclCollectives
    from qwen3_triton.runtime.fsdp import configure
    from qwen3_triton.training.sharding import shard_vocab_loss_model
    from qwen3_triton.training.vocab_parallel import VocabParallelEmbedding
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)

    # 1. vocabulary-parallel embedding
    V, H, T = 1024, 256, 700
    g = torch.Generator().manual_seed(5)
    full = torch.randn(V, H, generator=g)
    ids_all = torch.randint(0, V, (world, 2, T // 2), generator=g)
    ids_all[:, 0, :50] = 511                                  # repeated token on a shard edge
    dy_all = torch.randn(world, 2, T // 2, H, generator=g).to(torch.bfloat16)
    emb = VocabParallelEmbedding(full)
    y = emb(ids_all[rank].to(dev))
    assert torch.equal(y.cpu(), full.to(torch.bfloat16)[ids_all[rank]])
    y.backward(dy_all[rank].to(dev))
    ref = torch.zeros(V, H, dtype=torch.float64).index_add_(0, ids_all.view(-1), dy_all.double().view(-1, H)) / world
    rows = V // world
    torch.testing.assert_close(emb.weight.grad.double().cpu(), ref[rank * rows:(rank + 1) * rows], rtol=1e-5, atol=1e-5)

    # 2. one FSDP2 step, embedding gathered by FSDP vs vocabulary-parallel
    cfg = types.SimpleNamespace(model_type="qwen3", hidden_act="silu", attention_dropout=0.0, attention_bias=False,
                                use_sliding_window=False, rope_scaling=None, vocab_size=1024, hidden_size=256,
                                intermediate_size=512, num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=1,
                                head_dim=128, max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=1e6,
                                initializer_range=0.02, tie_word_embeddings=False, use_cache=False)
    all_ids = [torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(100 + r)) for r in range(world)]
    ids = all_ids[rank].to(dev)
    # unsharded yardstick: same seed -> same weights, bf16 compute, the global batch in one process
    torch.manual_seed(1234)
    with torch.device(dev):
        whole = model_for_variant(cfg, "b200_fused")
    whole = whole.to(dev, torch.bfloat16)     # also moves the rotary frequencies, which are built on the CPU
    whole.model.set_recompute("selective")
    mine = float(whole(ids, labels=ids).loss)
    whole(torch.cat(all_ids).to(dev), labels=torch.cat(all_ids).to(dev)).loss.backward()
    yard = {n: p.grad.float().cpu() for n, p in whole.named_parameters()}
    del whole

    def shard_of(name, t):
        rows = yard[name].shape[0] // world
        return yard[name][rank * rows:(rank + 1) * rows], (t.to_local() if hasattr(t, "to_local") else t).float().cpu()

    results = []
    for vp in (False, True):
        torch.manual_seed(1234)
        with torch.device(dev):
            model = model_for_variant(cfg, "b200_fused")
        comm = NcclCollectives()
        model = shard_vocab_loss_model(model, keep_full_layers=4, checkpoint_every=1, skip_embedding_backward_gather=True,
                                       fused_vocab_dw=True, communication=None, checkpoint_mode="selective",
                                       layers_per_unit=[1, 1, 2], vocab_parallel_embedding=vp)
        configure(model, comm)
        opt = TritonAdamW([p for p in model.parameters()], lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
        out = model(ids, labels=ids)
        out.loss.backward()
        assert abs(float(out.loss) - mine) / mine < 1e-3, (float(out.loss), mine)
        named = dict(model.named_parameters())
        for name in ("model.embed_tokens.weight", "lm_head.weight", "model.layers.2.mlp.down_proj.weight",
                     "model.layers.0.self_attn.k_proj.weight", "model.norm.weight"):
            want, got = shard_of(name, named[name].grad)
            rel = float((got - want).norm() / want.norm())
            sys.stdout.write("rank%%d vp=%%s %%s rel_l2 %%.3e" %% (rank, vp, name, rel) + chr(10))
            assert rel < 2e-2, (name, rel)
        w = model.model.embed_tokens.weight
        grad = w.grad.to_local() if hasattr(w.grad, "to_local") else w.grad
        opt.step()
        opt.zero_grad(set_to_none=True)
        loss2 = model(ids, labels=ids).loss
        results.append((float(out.loss), grad.float().cpu().clone(), float(loss2)))
        assert _abi.read_status() == 0
    (l0, g0, s0), (l1, g1, s1) = results
    assert abs(l0 - l1) / abs(l0) < 1e-3, (l0, l1)
    assert abs(s0 - s1) / abs(s0) < 2e-3, (s0, s1)
    assert s0 < l0
    rel = float((g0 - g1).norm() / g0.norm())
    assert rel < 2e-2, rel

    # 3. the same step with parameters gathered by copy-engine pulls, split-copied ahead of time on a side stream, and
    #    gradients reduced by the pull kernel over peer memory: on two ranks the fp32 sum of the two upcast bf16 gradients has one possible value, so every gradient
    #    shard equals the NCCL path's bit for bit
    shards, losses = [], []
    for peer in (False, True, "homes"):
        torch.manual_seed(1234)
        with torch.device(dev):
            model = model_for_variant(cfg, "b200_fused")
        comm = NcclCollectives()
        model = shard_vocab_loss_model(model, keep_full_layers=4, checkpoint_every=1, skip_embedding_backward_gather=True,
                                       fused_vocab_dw=True, communication=None, checkpoint_mode="selective",
                                       layers_per_unit=[1, 1, 2], vocab_parallel_embedding=True)
        hooks = configure(model, comm, peer_memory_reduce=bool(peer), copy_engine_gather=bool(peer),
                          early_copy_out=peer is True, gradients_in_staging=peer == "homes",
                          gather_into_parameters=peer == "homes")
        assert hooks["gather_into_parameters"] == (peer == "homes")
        assert hooks["early_copy_out"] == (peer is True)
        assert (hooks["gradient_homes"] > 0) == (peer == "homes")
        for _ in range(3):                                   # three steps: both staging slots reused several times
            model.zero_grad(set_to_none=True)
            model(ids, labels=ids).loss.backward()
        torch.cuda.synchronize()
        shards.append({n: (q.grad.to_local() if hasattr(q.grad, "to_local") else q.grad).float().cpu().clone()
                       for n, q in model.named_parameters()})
        rs, ag = hooks["reduce_scatter"], hooks["all_gather"]
        assert rs.calls > 0 and rs.peer_calls == (rs.calls if peer else 0), (rs.calls, rs.peer_calls)
        assert ag.calls > 0 and ag.peer_calls == (ag.calls if peer else 0), (ag.calls, ag.peer_calls)
        losses.append(float(model(ids, labels=ids).loss))   # one more forward: gathered parameters are the same
        for key in ("peer_gather", "peer_reducer"):
            if hooks[key] is not None:
                hooks[key].close()
        if peer is True:
            from qwen3_triton.runtime import early_copy_out
            assert early_copy_out.statistics()["early_copies"] >= 4 * 3      # every unit, every step
        if peer == "homes":
            # the seven matrices of each of the 4 layers are written by their GEMMs into the staging buffer, 3 steps
            assert hooks["peer_reducer"].born_in_place == 3 * 4 * 7, hooks["peer_reducer"].born_in_place
            assert hooks["peer_reducer"].copied_home > 0               # norm weights are copied to their homes
            # every all-gather delivered its pieces straight into the parameter tensors
            assert hooks["peer_gather"].delivered == hooks["all_gather"].peer_calls > 0
        configure(model, comm)                               # leaves no reducer installed behind, early copy-out off
        assert _abi.read_status() == 0
    for other in shards[1:]:
        for name, want in shards[0].items():
            assert torch.equal(want, other[name]), name
    assert losses[0] == losses[1] == losses[2], losses  # parameters gathered by copy engines: the same bits
    sys.stdout.write("rank%%d peer-memory reduce equals NCCL on %%d tensors" %% (rank, len(shards[0])) + chr(10))
    dist.barrier(); dist.destroy_process_group()
    sys.stdout.write("rank" + str(rank) + "ok" + chr(10)); sys.stdout.flush()
''') % str(ROOT / "qwen3-triton_b200")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_vocab_parallel_embedding_and_fsdp_step(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMP_NUM_THREADS="1")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29621", str(script)], capture_output=True,
                         text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-5000:]
    assert "rank0ok" in res.stdout and "rank1ok" in res.stdout
