#!/usr/bin/env python
"""Training-step throughput of the Qwen3-8B-shaped hot path on B200, one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1: BASELINE config 4 - a 4-layer slice of the Qwen3-8B architecture (hidden 4096, 32/8 heads, head_dim 128,
intermediate 12288, vocab 151936, untied lm_head), bf16 compute with fp32 master weights, microbatch 4 x 2048,
forward + cross-entropy + backward + AdamW every step, synthetic uniform token ids, weights ~ N(0, 0.02).
N > 1 (launched with torch.distributed.run): the full 36-layer model under FSDP2, microbatch 1 x 2048 per GPU.

`value` = tokens/s over all GPUs with the token ids already resident in HBM; `e2e.value` = the same step driven
with pinned-host ids copied in and the loss read back every step. `--impl reference` times the CPU oracle
restatement of the reference's model on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "qwen3-triton_b200"))
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "train_tokens_per_s"
UNIT = "tokens/s"

# kernels launched by one call of each C-ABI entry (for the gpu_launches claim)
LAUNCHES = {"q3_rmsnorm_bwd": 2, "q3_add_rmsnorm_bwd": 2, "q3_norm_rope_bwd": 2, "q3_adamw_multi": 2, "q3_ce_fwd": 2,
            "q3_attn_bwd": 3, "q3_vce_finish": 2, "q3_embedding_bwd": 2, "q3_embedding_shard_bwd": 2,
            "q3_qk_norm_rope_bwd": 3}


GEMM_ENTRIES = ("q3_gemm", "q3_gemm_acc", "q3_gate_up_swiglu_fwd", "q3_linear_fwd_grouped", "q3_linear_dgrad_grouped",
                "q3_linear_wgrad_grouped", "q3_down_dgrad_swiglu_bwd")


def gemm_flops_of(name, a):
    """FLOPs of one call of a GEMM entry point from its recorded arguments (0 for anything else)."""
    if name in ("q3_gemm", "q3_gemm_acc"):
        return 2.0 * a[7] * a[8] * a[9]
    if name == "q3_gate_up_swiglu_fwd":
        return 4.0 * a[6] * a[7] * a[8]
    if name == "q3_down_dgrad_swiglu_bwd":
        return 2.0 * a[6] * a[7] * a[8]
    if name in ("q3_linear_fwd_grouped", "q3_linear_dgrad_grouped", "q3_linear_wgrad_grouped"):
        return 2.0 * a[5] * a[6] * sum(a[3][i] for i in range(a[4]))
    return 0.0


def slice_config(layers):
    from qwen3_triton import Qwen3Config
    return Qwen3Config(num_hidden_layers=layers)


def model_flops_per_token(cfg, seq):
    """Model FLOPs per token for fwd+bwd (3x forward), no recompute: 2*matmul params + causal attention."""
    c = cfg
    layer = (c.hidden_size * c.head_dim * (2 * c.num_attention_heads + 2 * c.num_key_value_heads)
             + 3 * c.hidden_size * c.intermediate_size)
    fwd = c.num_hidden_layers * (2 * layer + 2 * seq * c.head_dim * c.num_attention_heads) + 2 * c.hidden_size * c.vocab_size
    return 3 * fwd


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        self.path = ROOT / "gpurun_out" / f"clocks_bench_{index}.csv"
        try:
            self.path.parent.mkdir(exist_ok=True)
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=self.fh,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.path.read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return data.get("bf16_tflops_sustained", 1395.4), data.get("hbm_gbs", 6540.8), "measured"
    return 1400.0, 6650.0, "fallback"


# ---------------------------------------------------------------------------------------- CPU reference arm
def cpu_reference_step_tokens_per_s(layers, sample_tokens, steps, warmup):
    """The oracle restatement of the reference's CPU model (same architecture, fp32, torch CPU kernels on all
    host threads): forward + CE + backward + AdamW on a bounded sample of `sample_tokens` tokens per step."""
    from oracle.model import OracleQwen3
    torch.set_num_threads(os.cpu_count() or 1)
    cfg = slice_config(layers)
    model = OracleQwen3(cfg, seed=1)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)
    gen = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab_size, (1, sample_tokens), generator=gen)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        opt.zero_grad(set_to_none=True)
        loss, _ = model(ids, ids)
        loss.backward()
        opt.step()
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    return sample_tokens / sec, sec


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    layers = 4
    sample = 128
    steps, warmup = max(1, min(args.steps, 3)), 1
    tps, sec = cpu_reference_step_tokens_per_s(layers, sample, steps, warmup)
    cores = os.cpu_count() or 1
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "qwen3-8b 4-layer slice fwd+bwd+AdamW (CPU sample 1x%d tokens)" % sample,
                       "note": "the CPU arm always times the 4-layer slice (BASELINE config 4); the full 36-layer model "
                               "of config 5 needs ~130 GB of host memory for fp32 weights, gradients and moments and "
                               "would run about 9x fewer tokens/s, so at N>1 this line is an upper bound for the CPU"},
            "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"oracle model, 4 layers, 1 x {sample} tokens per step, median of {steps}"},
            "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------- GPU arm
class Counter:
    """Counts C-ABI calls / kernel launches and, when `profile` is on, times every call with CUDA events."""

    def __init__(self):
        from qwen3_triton import _abi
        self.abi = _abi
        self.orig = _abi.call
        self.launches = 0
        self.profile = False
        self.records = []
        _abi.call = self
        # modules bound `call` through the module object, so patching the attribute is enough

    def __call__(self, name, *a):
        self.launches += LAUNCHES.get(name, 1)
        if self.profile:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            self.orig(name, *a)
            e.record()
            self.records.append((name, a, s, e))
        else:
            self.orig(name, *a)


def build_single_gpu(cfg, device):
    from qwen3_triton import model_for_variant
    from qwen3_triton.runtime.adamw import TritonAdamW
    from qwen3_triton.runtime.mixed_precision import MasterWeights
    torch.manual_seed(20261114)
    with torch.device(device):
        model = model_for_variant(cfg, os.environ.get("Q3_BENCH_VARIANT", "b200_fused"))
    model.to(device)   # buffers created on the CPU on purpose (rotary frequencies) move here
    if hasattr(model, "fused_loss"):
        # "1": hidden -> loss without logits in HBM (one extra logits GEMM in backward; measured 8 ms slower per step here)
        model.fused_loss = os.environ.get("Q3_BENCH_FUSED_LOSS", "0") == "1"
    masters = MasterWeights(model).fuse_into_optimizer()
    opt = TritonAdamW(masters.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1, block=16384)
    return model, masters, opt


def run_ours(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        return run_fsdp(args)
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    counter = Counter()
    # N=1 workload: the full 36-layer Qwen3-8B at the per-GPU microbatch of config 5 (1 x 2048) when it fits this GPU
    # (fp32 masters + moments 98 GB, bf16 working copies and gradients 33 GB, activations 6 GB), else the 4-layer
    # slice of config 4 (4 x 2048). Q3_BENCH_N1 = "full" | "slice" forces one.
    choice = os.environ.get("Q3_BENCH_N1", "auto")
    free_gib = torch.cuda.mem_get_info(device)[0] / 2 ** 30
    want_full = choice == "full" or (choice == "auto" and free_gib >= 160)
    model = masters = opt = None
    if want_full:
        layers, batch, seq = 36, 1, 2048
        try:
            cfg = slice_config(layers)
            model, masters, opt = build_single_gpu(cfg, device)
        except torch.cuda.OutOfMemoryError:
            model = masters = opt = None
            import gc
            gc.collect()
            torch.cuda.empty_cache()
    if model is None:
        layers, batch, seq = 4, 4, 2048
        cfg = slice_config(layers)
        model, masters, opt = build_single_gpu(cfg, device)
    gen = torch.Generator().manual_seed(3)
    nbatches = args.warmup + args.steps
    host_ids = [torch.randint(0, cfg.vocab_size, (batch, seq), generator=gen).pin_memory() for _ in range(min(nbatches, 8))]
    dev_ids = [h.to(device) for h in host_ids]

    def step(ids):
        masters.sync_working()
        out = model(ids, labels=ids)
        out.loss.backward()
        masters.collect_grads()
        opt.step()
        masters.release_grads()
        return out.loss

    for i in range(args.warmup):
        step(dev_ids[i % len(dev_ids)])
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    counter.launches = 0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(args.steps):
        loss = step(dev_ids[i % len(dev_ids)])
    end.record()
    torch.cuda.synchronize()
    launches = counter.launches
    ms = start.elapsed_time(end) / args.steps
    tokens = batch * seq
    value = tokens / (ms * 1e-3)

    # end to end: pinned host ids copied in, loss read back, every step
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(args.steps):
        ids = host_ids[i % len(host_ids)].to(device, non_blocking=True)
        last = float(step(ids).item())
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop()

    # per-kernel census of one more step with CUDA events around every C-ABI call
    counter.profile = True
    step(dev_ids[0])
    torch.cuda.synchronize()
    counter.profile = False
    by_name = {}
    gemm_flops = 0.0
    for name, a, s, e in counter.records:
        t = s.elapsed_time(e)
        by_name[name] = by_name.get(name, 0.0) + t
        gemm_flops += gemm_flops_of(name, a)
    gemm_ms = sum(by_name.get(n, 0.0) for n in GEMM_ENTRIES)
    peak_tf, _, peak_kind = measured_peaks()
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    total_ms = sum(by_name.values())
    census = {k: round(v, 3) for k, v in sorted(by_name.items(), key=lambda kv: -kv[1])}

    flops_tok = model_flops_per_token(cfg, seq)
    mfu = value * flops_tok / (peak_tf * 1e12)
    if os.environ.get("Q3_BENCH_SKIP_CPU"):     # profiling runs under ncu skip the host-side baseline leg
        cpu_tps = None
    else:
        cpu_tps, _ = cpu_reference_step_tokens_per_s(layers, 128, 1, 1)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": ("qwen3-8b full 36-layer model on one GPU, fwd+bwd+AdamW, microbatch 1x2048 (the per-GPU "
                                "workload of BASELINE config 5, no sharding)" if layers == 36 else
                                "qwen3-8b 4-layer slice fwd+bwd+AdamW, microbatch 4x2048 (BASELINE config 4)"),
                   "global_batch": batch, "seq_len": seq, "parallelism": "single",
                   "l2": "inputs+weights >> L2 (%d GB bf16 weights)" % (16 if layers == 36 else 4),
                   "attention_path": "see kernel census", "mfu_of_%s_peak" % peak_kind: mfu, "last_loss": last,
                   "peak_memory_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": batch * seq * 8,
                "d2h_bytes_per_step": 4},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "gemm_tc_kernel (all GEMM entry points of a step: q3_gemm, q3_linear_*_grouped, q3_gate_up_swiglu_fwd)",
                     "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                     "peak_kind": peak_kind + " bf16_tflops_sustained", "traffic": None,
                     "gemm_ms_per_step": gemm_ms, "all_kernels_ms_per_step": total_ms, "census_ms": census},
        "cpu_baseline": {"value": cpu_tps, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                         "sample": "oracle model, 4 layers, 1 x 128 tokens, one timed step after one warm-up"},
    }
    print(json.dumps(line), flush=True)


def census(counter):
    by_name, gemm_flops = {}, 0.0
    shapes = {}
    for name, a, s, e in counter.records:
        by_name[name] = by_name.get(name, 0.0) + s.elapsed_time(e)
        if name in ("q3_gemm", "q3_gemm_acc"):
            key = (a[7], a[8], a[9], "A:%s B:%s" % ("K" if a[2] == 1 else "MN", "K" if a[4] == 1 else "MN"))
            cnt, tot = shapes.get(key, (0, 0.0))
            shapes[key] = (cnt + 1, tot + s.elapsed_time(e))
        gemm_flops += gemm_flops_of(name, a)
    if os.environ.get("Q3_BENCH_PROFILE"):
        for (m, n, k, lay), (cnt, tot) in sorted(shapes.items(), key=lambda kv: -kv[1][1]):
            sys.stderr.write("gemm %6d x %6d x %6d %-10s n=%3d total %8.3f ms avg %8.1f us %7.1f TFLOP/s\n" % (
                m, n, k, lay, cnt, tot, tot / cnt * 1e3, 2.0 * m * n * k * cnt / tot / 1e9))
    gemm_ms = sum(by_name.get(n, 0.0) for n in GEMM_ENTRIES)
    return by_name, gemm_flops, gemm_ms


def unit_sizes(layers):
    """FSDP unit sizes for the decoder layers. Default: units of 4 layers, but the first four layers as 1+1+2, so that
    the all-gather that cannot hide (the first) and the reduce-scatter that cannot hide (the last) are small.
    Q3_BENCH_LAYERS_PER_UNIT = an integer (uniform) or a comma-separated list that sums to the layer count."""
    spec = os.environ.get("Q3_BENCH_LAYERS_PER_UNIT", "")
    if "," in spec:
        return [int(v) for v in spec.split(",")]
    if spec:
        return int(spec)
    if layers < 8:
        return 1
    sizes = [1, 1, 2]
    rest = layers - 4
    sizes += [4] * (rest // 4)
    if rest % 4:
        sizes.append(rest % 4)
    return sizes


def run_fsdp(args):
    """N > 1: BASELINE config 5 - the full 36-layer model under FSDP2 (one process per GPU, NCCL), bf16 parameter
    all-gather, fp32 gradient reduce-scatter, vocabulary-parallel lm_head + cross-entropy, per-layer activation
    recomputation, microbatch 1 x 2048 per GPU, AdamW every step."""
    import torch.distributed as dist
    from qwen3_triton import model_for_variant
    from qwen3_triton.runtime.adamw import TritonAdamW
    from qwen3_triton.runtime.collectives import NcclCollectives
    from qwen3_triton.runtime.fsdp import configure
    from qwen3_triton.training.sharding import shard_vocab_loss_model

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    counter = Counter()
    layers = int(os.environ.get("Q3_BENCH_LAYERS", "36"))
    batch, seq = 1, 2048
    cfg = slice_config(layers)
    torch.manual_seed(20261114)            # same weights on every rank
    with torch.device(device):
        model = model_for_variant(cfg, os.environ.get("Q3_BENCH_VARIANT", "b200_fused"))
    comm = NcclCollectives()
    # the vocabulary-parallel head and embedding talk over their own communicator, so that their small collectives on
    # the compute stream do not queue behind FSDP's reduce-scatters on the same NCCL communicator
    vocab_comm = NcclCollectives(group=dist.new_group()) if os.environ.get("Q3_BENCH_VP_GROUP", "1") == "1" else None
    # activation recomputation: 'none' keeps every layer's activations (about 5 GB at 2048 tokens per GPU, nothing on
    # a 180 GB part); 'selective' / 'full' are the memory-saving modes
    ckpt = os.environ.get("Q3_BENCH_CHECKPOINT", "none")
    model = shard_vocab_loss_model(model, keep_full_layers=layers, checkpoint_every=1,
                                   skip_embedding_backward_gather=True, fused_vocab_dw=True, communication=vocab_comm,
                                   checkpoint_mode=ckpt, layers_per_unit=unit_sizes(layers),
                                   vocab_parallel_embedding=os.environ.get("Q3_BENCH_VP_EMBEDDING", "1") == "1",
                                   forward_prefetch=int(os.environ.get("Q3_BENCH_FORWARD_PREFETCH", "2")))
    model.lm_head.fused = os.environ.get("Q3_BENCH_FUSED_LOSS", "0") == "1"
    hooks = configure(model, comm, pack_gradients_off_compute_stream=os.environ.get("Q3_BENCH_PACK_SIDE", "0") == "1")
    decoder = [p for n, p in model.named_parameters() if not n.startswith("lm_head.")]
    opt = TritonAdamW([dict(params=decoder), dict(params=[model.lm_head.weight])], lr=1e-4, betas=(0.9, 0.95),
                      weight_decay=0.1, block=16384)
    gen = torch.Generator().manual_seed(100 + rank)
    host_ids = [torch.randint(0, cfg.vocab_size, (batch, seq), generator=gen).pin_memory() for _ in range(8)]
    dev_ids = [h.to(device) for h in host_ids]

    def step(ids):
        opt.zero_grad(set_to_none=True)
        out = model(ids, labels=ids)
        out.loss.backward()
        opt.step()
        return out.loss

    for i in range(args.warmup):
        step(dev_ids[i % len(dev_ids)])
    torch.cuda.synchronize()
    dist.barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    counter.launches = 0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(args.steps):
        step(dev_ids[i % len(dev_ids)])
    end.record()
    torch.cuda.synchronize()
    dist.barrier()
    launches = counter.launches
    t = torch.tensor([start.elapsed_time(end) / args.steps], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())

    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        ids = host_ids[i % len(host_ids)].to(device, non_blocking=True)
        last = float(step(ids).item())
    torch.cuda.synchronize()
    t = torch.tensor([(time.perf_counter() - t0) * 1e3 / args.steps], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    clocks = sampler.stop() if sampler else None

    if os.environ.get("Q3_BENCH_PROFILE") and rank == 0:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            step(dev_ids[0])
            torch.cuda.synchronize()
        sys.stderr.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=25, max_name_column_width=70) + "\n")
        (ROOT / "gpurun_out").mkdir(exist_ok=True)
        prof.export_chrome_trace(str(ROOT / "gpurun_out" / "trace_rank0.json"))
    elif os.environ.get("Q3_BENCH_PROFILE"):
        step(dev_ids[0])
    counter.profile = True
    step(dev_ids[0])
    torch.cuda.synchronize()
    counter.profile = False
    by_name, gemm_flops, gemm_ms = census(counter)
    dist.barrier()
    if rank == 0:
        peak_tf, _, peak_kind = measured_peaks()
        achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
        tokens = batch * seq * world
        value = tokens / (ms * 1e-3)
        mfu = (value / world) * model_flops_per_token(cfg, seq) / (peak_tf * 1e12)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "qwen3-8b %d layers under FSDP2, microbatch 1x2048 per GPU, vocab-parallel head%s, "
                                   "%s activation recompute, AdamW (BASELINE config 5)" % (
                                       layers, " and embedding" if os.environ.get("Q3_BENCH_VP_EMBEDDING", "1") == "1" else "", ckpt),
                       "global_batch": batch * world, "seq_len": seq, "parallelism": "fsdp%d" % world,
                       "l2": "weights and activations >> L2", "mfu_of_%s_peak_per_gpu" % peak_kind: mfu,
                       "tokens_per_s_per_gpu": value / world, "last_loss": last,
                       "peak_memory_gb_rank0": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
                       "fsdp_units": hooks["units"], "collectives": comm.report()},
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": batch * seq * 8 * world,
                    "d2h_bytes_per_step": 4 * world},
            "gpu_launches": launches, "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "gemm_tc_kernel (all GEMM entry points of a step, rank 0: q3_gemm, q3_linear_*_grouped, q3_gate_up_swiglu_fwd)",
                         "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                         "peak_kind": peak_kind + " bf16_tflops_sustained", "traffic": None, "gemm_ms_per_step": gemm_ms,
                         "all_kernels_ms_per_step": sum(by_name.values()),
                         "census_ms": {k: round(v, 3) for k, v in sorted(by_name.items(), key=lambda kv: -kv[1])}},
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    run_ours(args)


if __name__ == "__main__":
    main()
