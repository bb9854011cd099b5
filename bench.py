#!/usr/bin/env python
"""Training-step throughput of the Qwen3-8B-shaped hot path on B200, one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--out DIR]

Workload (metric: training tokens per second, Qwen3-8B shapes, microbatch 1 x 2048 tokens per GPU, forward +
cross-entropy + backward + AdamW every step, bf16 compute with fp32 master weights and moments, seeded synthetic
token ids, weights ~ N(0, 0.02)):
  N = 1  the full 36-layer model on one GPU, unsharded (falls back to a 4-layer slice at 4 x 2048 when the GPU
         has less than 160 GiB free);
  N > 1  (launched with torch.distributed.run) the same model under FSDP2: bf16 parameter all-gather (copy-engine
         transfers from peer-mapped buffers; Q3_BENCH_CE_GATHER=0: NCCL), fp32 gradient reduce-scatter (one pull
         kernel over peer memory per unit, weight gradients written by their GEMMs straight into its staging buffer;
         Q3_BENCH_PEER_REDUCE=0: NCCL), vocabulary-parallel lm_head + cross-entropy, per-layer activation
         recomputation ("full", the contract configuration; the "selective" and "none" policies are timed after it
         and reported under config.other_recompute_policies).
The loss head never writes the [tokens, vocab] logits (Q3_BENCH_FUSED_LOSS=0 selects the materialising head).

`value` = tokens/s over all GPUs with the token ids already resident in HBM; `e2e.value` = the same step driven
through the public model API with pinned-host ids copied in and the loss read back every step. `--impl reference`
times the CPU restatement of the reference's model (oracle/) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
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
            "q3_qk_norm_rope_bwd": 3, "q3_attn_bwd_bshd": 3, "q3_adamw_multi_mp": 2,
            "q3_peer_copy": 0, "q3_peer_copy_many": 0}      # copy-engine transfers are not kernels

GEMM_ENTRIES = ("q3_gemm", "q3_gemm_acc", "q3_gemm_acc_f32", "q3_gate_up_swiglu_fwd", "q3_linear_fwd_grouped",
                "q3_linear_dgrad_grouped", "q3_linear_wgrad_grouped", "q3_down_dgrad_swiglu_bwd", "q3_linear_ce_stats",
                "q3_linear_ce_grad")

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum, one ncu capture per shape) divided by the algorithmic
# bytes (operands read once + result written once) of the GEMM shapes of one training step at 2048 tokens; the source
# table with the full command is profiles/gemm_tc_kernel_step_shapes_dram.md. Used for roofline.traffic.
DRAM_OVER_ALGORITHMIC = 1.214
DRAM_RATIO_SOURCE = "profiles/gemm_tc_kernel_step_shapes_dram.md"


def gemm_work_of(name, a):
    """(FLOPs, algorithmic bytes) of one call of a GEMM entry point from its recorded arguments."""
    def dense(m, n, k, out_bytes=2):
        return 2.0 * m * n * k, 2.0 * (m * k + n * k) + out_bytes * m * n
    if name in ("q3_gemm", "q3_gemm_acc"):
        return dense(a[7], a[8], a[9], 4 if a[11] == 0 else 2)
    if name == "q3_gemm_acc_f32":
        return dense(a[7], a[8], a[9], 8)
    if name == "q3_gate_up_swiglu_fwd":
        m, n, k = a[6], a[7], a[8]
        return 4.0 * m * n * k, 2.0 * (m * k + 2 * n * k) + 6.0 * m * n
    if name == "q3_down_dgrad_swiglu_bwd":
        m, i, h = a[6], a[7], a[8]
        return 2.0 * m * i * h, 2.0 * (m * h + i * h) + 8.0 * m * i
    if name in ("q3_linear_fwd_grouped", "q3_linear_dgrad_grouped", "q3_linear_wgrad_grouped"):
        m, k, total = a[5], a[6], sum(a[3][i] for i in range(a[4]))
        return 2.0 * m * k * total, 2.0 * (m * k + total * k + m * total)
    if name == "q3_linear_ce_stats":
        m, v, k = a[6], a[7], a[8]
        return 2.0 * m * v * k, 2.0 * (m * k + v * k)
    if name == "q3_linear_ce_grad":
        m, v, k = a[7], a[8], a[9]
        return dense(m, v, k)
    return 0.0, 0.0


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
    """nvidia-smi clock / throttle-reason samples every 200 ms while the timed region runs (read-only query)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index, out_dir):
        self.proc = None
        self.path = Path(out_dir) / f"clocks_gpu{index}.csv"
        try:
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
def _median_ms(fn, warmup, runs):
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(runs):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return statistics.median(times) * 1e3


def cpu_model_step_ms(cfg, batch, seq, warmup, runs, adamw=None):
    """One forward + CE + backward + AdamW step of the restated reference CPU model (fp32, all host threads)."""
    from oracle.model import OracleQwen3
    model = OracleQwen3(cfg, seed=1)
    opt = torch.optim.AdamW(model.parameters(), **(adamw or dict(lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)))
    ids = torch.randint(0, cfg.vocab_size, (batch, seq), generator=torch.Generator().manual_seed(2))

    def step():
        opt.zero_grad(set_to_none=True)
        loss, _ = model(ids, ids)
        loss.backward()
        opt.step()
    return _median_ms(step, warmup, runs)


def cpu_workload_baseline(layers, sample_tokens, warmup=3, runs=5):
    """tokens/s of the `layers`-layer Qwen3-8B-shaped model on the host, from a bounded sample: steps of a 2-layer and
    of a 4-layer slice at 1 x `sample_tokens` tokens give the per-layer and the embedding+head cost per step, from which
    the step of the full depth follows (4 layers: measured directly)."""
    torch.set_num_threads(os.cpu_count() or 1)
    t4 = cpu_model_step_ms(slice_config(4), 1, sample_tokens, warmup, runs)
    if layers == 4:
        return sample_tokens / (t4 * 1e-3), t4, f"4 layers, 1 x {sample_tokens} tokens per step, {warmup} warm-ups, median of {runs}"
    t2 = cpu_model_step_ms(slice_config(2), 1, sample_tokens, warmup, runs)
    per_layer = max((t4 - t2) / 2.0, 0.0)
    full = (t2 - 2.0 * per_layer) + layers * per_layer
    note = (f"{layers}-layer step extrapolated from measured 2- and 4-layer slices at 1 x {sample_tokens} tokens "
            f"({t2:.0f} ms, {t4:.0f} ms: {per_layer:.0f} ms per layer + {t2 - 2 * per_layer:.0f} ms embedding/head/optimizer rest), "
            f"{warmup} warm-ups, median of {runs}; the 4-layer slice alone gives {sample_tokens / (t4 * 1e-3):.1f} tokens/s")
    return sample_tokens / (full * 1e-3), full, note


def cpu_operator_baselines(warmup=1, runs=3):
    """The reference's CPU operators (restated in oracle/ops.py, fp32, all host threads) at the operator-sweep and
    attention shapes, each on a stated slice; and the tiny two-layer decoder's full training step."""
    from types import SimpleNamespace
    from oracle import ops as O
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(4)
    r = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    T = 4096                                    # a quarter of the 16384-token sweep
    out = []

    def add(name, shape, fn, note=""):
        out.append({"op": name, "shape": shape, "ms": round(_median_ms(fn, warmup, runs), 3), "note": note})

    tiny = SimpleNamespace(vocab_size=2048, hidden_size=256, intermediate_size=688, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=1e6,
                           initializer_range=0.02)
    ms = cpu_model_step_ms(tiny, 2, 128, 3, 5)
    out.append({"op": "tiny decoder full step (2 layers, hidden 256, vocab 2048, fp32)", "shape": "batch 2 x seq 128",
                "ms": round(ms, 3), "note": "%.0f tokens/s; 3 warm-ups, median of 5" % (256 / (ms * 1e-3))})
    x, w, dy = r(T, 4096), torch.ones(4096), r(T, 4096)
    add("rms_norm fwd", f"[{T},4096]", lambda: O.rms_norm(x, w), "1/4 of 16384 tokens")
    add("rms_norm bwd", f"[{T},4096]", lambda: O.rms_norm_backward(x, w, dy), "1/4 of 16384 tokens")
    q, k = r(1, T, 32, 128), r(1, T, 8, 128)
    wq, wk = torch.ones(128), torch.ones(128)
    pos = torch.arange(T)[None]
    inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2).float() / 128))
    ang = pos[..., None].float() * inv
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    add("qk_norm_rope fwd", f"q [1,{T},32,128] k [1,{T},8,128]",
        lambda: (O.norm_rope(q, wq, cos, sin), O.norm_rope(k, wk, cos, sin)), "1/4 of 16384 tokens")
    gate, up = r(T, 12288), r(T, 12288)
    add("swiglu fwd", f"[{T},12288] x2", lambda: O.swiglu(gate, up), "1/4 of 16384 tokens")
    aq, ak, av, ado = r(1, 4, 4096, 128), r(1, 1, 4096, 128), r(1, 1, 4096, 128), r(1, 4, 4096, 128)
    add("attention fwd", "B1 Hq4 Hkv1 S4096 D128", lambda: O.attention(aq, ak, av), "one query-head group = 1/32 of B4 Hq32 S4096")
    add("attention bwd", "B1 Hq4 Hkv1 S4096 D128", lambda: O.attention_backward(aq, ak, av, ado), "1/32 of B4 Hq32 S4096")
    a, b = r(2048, 4096), r(4096, 4096)
    add("linear fwd (q_proj)", "2048 x 4096 x 4096", lambda: O.linear(a, b))
    logits, labels = r(1, 1024, 151936), torch.randint(0, 151936, (1, 1024), generator=g)
    add("cross-entropy fwd", "[1024,151936] fp32 logits", lambda: O.causal_cross_entropy(logits, labels), "1/16 of 16384 tokens")
    n = 4096 * 12288
    p = torch.nn.Parameter(r(n))
    p.grad = r(n) * 1e-3
    opt = torch.optim.AdamW([p], lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)
    add("AdamW step", f"{n} fp32 parameters", opt.step, "one gate_proj matrix = 1/163 of 8.19e9 parameters")
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    layers, sample = 36, 128
    warmup, runs = 3, max(5, min(args.steps, 7))
    tps, ms, note = cpu_workload_baseline(layers, sample, warmup, runs)
    cores = os.cpu_count() or 1
    extra = None if os.environ.get("Q3_BENCH_SKIP_CPU_OPS") else cpu_operator_baselines()
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": runs,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "qwen3-8b full 36-layer model, fwd+bwd+AdamW, microbatch 1x2048 per GPU "
                                   "(CPU arm: restated reference model on the host cores, bounded sample)",
                       "global_batch": args.gpus, "seq_len": 2048, "parallelism": "cpu",
                       "note": "a step of the full model at 2048 tokens needs about 130 GB of host memory and minutes "
                               "per step on the CPU, so the arm times 1 x %d-token steps of 2- and 4-layer slices and "
                               "extrapolates the depth; tokens/s is per host, not multiplied by the GPU count" % sample},
            "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": note, "extra": extra},
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


def census(counter):
    """Per-entry-point time of the recorded step and the GEMM totals (ms, FLOPs, algorithmic bytes)."""
    by_name, flops, nbytes, shapes = {}, 0.0, 0.0, {}
    for name, a, s, e in counter.records:
        t = s.elapsed_time(e)
        by_name[name] = by_name.get(name, 0.0) + t
        f, b = gemm_work_of(name, a)
        flops += f
        nbytes += b
        if name in ("q3_gemm", "q3_gemm_acc"):
            key = (a[7], a[8], a[9], "A:%s B:%s" % ("K" if a[2] == 1 else "MN", "K" if a[4] == 1 else "MN"))
            cnt, tot = shapes.get(key, (0, 0.0))
            shapes[key] = (cnt + 1, tot + t)
    if os.environ.get("Q3_BENCH_PROFILE"):
        for (m, n, k, lay), (cnt, tot) in sorted(shapes.items(), key=lambda kv: -kv[1][1]):
            sys.stderr.write("gemm %6d x %6d x %6d %-10s n=%3d total %8.3f ms avg %8.1f us %7.1f TFLOP/s\n" % (
                m, n, k, lay, cnt, tot, tot / cnt * 1e3, 2.0 * m * n * k * cnt / tot / 1e9))
    gemm_ms = sum(by_name.get(n, 0.0) for n in GEMM_ENTRIES)
    trace = os.environ.get("Q3_BENCH_TRACE")
    if trace and counter.records:
        # timeline of the census step: entry point, start (ms after the first call, same stream only) and duration
        first = counter.records[0][2]
        with open("%s.rank%s" % (trace, os.environ.get("RANK", "0")), "w") as f:
            for name, a, s, e in counter.records:
                try:
                    f.write("%s %.4f %.4f\n" % (name, first.elapsed_time(s), s.elapsed_time(e)))
                except Exception:
                    f.write("%s nan %.4f\n" % (name, s.elapsed_time(e)))
    return by_name, flops, nbytes, gemm_ms


def roofline_of(counter):
    by_name, flops, nbytes, gemm_ms = census(counter)
    peak_tf, _, peak_kind = measured_peaks()
    achieved = flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    return {"bound": "tensor",
            "kernel": "gemm_tc_kernel (every GEMM entry point of one step: q3_gemm*, q3_linear_*_grouped, "
                      "q3_gate_up_swiglu_fwd, q3_down_dgrad_swiglu_bwd, q3_linear_ce_*)",
            "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
            "peak_kind": peak_kind + " bf16_tflops_sustained",
            "traffic": nbytes * DRAM_OVER_ALGORITHMIC,
            "traffic_note": "bytes per step over all GEMM launches: algorithmic bytes (operands once + result once) "
                            "x %.2f, the DRAM/algorithmic ratio ncu measured on the step's GEMM shapes (%s)" % (
                                DRAM_OVER_ALGORITHMIC, DRAM_RATIO_SOURCE),
            "algorithmic_bytes_per_step": nbytes, "flops_per_step": flops, "gemm_ms_per_step": gemm_ms,
            "all_kernels_ms_per_step": sum(by_name.values()),
            "census_ms": {k: round(v, 3) for k, v in sorted(by_name.items(), key=lambda kv: -kv[1])}}


def build_single_gpu(cfg, device):
    from qwen3_triton import model_for_variant
    from qwen3_triton.runtime.adamw import TritonAdamW
    from qwen3_triton.runtime.mixed_precision import MasterWeights
    torch.manual_seed(20261114)
    with torch.device(device):
        model = model_for_variant(cfg, os.environ.get("Q3_BENCH_VARIANT", "b200_fused"))
    model.to(device)   # buffers created on the CPU on purpose (rotary frequencies) move here
    if hasattr(model, "fused_loss"):
        # hidden -> loss without the [tokens, vocab] logits in HBM ("0": materialise them, one GEMM less in backward)
        model.fused_loss = os.environ.get("Q3_BENCH_FUSED_LOSS", "1") == "1"
    masters = MasterWeights(model).fuse_into_optimizer()
    opt = TritonAdamW(masters.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1, block=16384)
    if os.environ.get("Q3_BENCH_EARLY_ADAMW", "0") == "1":
        # each decoder layer is updated on a side stream as soon as its backward is complete, beside the GEMMs of the
        # layers below it; embedding, final norm and head are updated by opt.step()
        opt.step_during_backward([masters.masters_of(layer) for layer in model.model.layers], masters.working_of)
    return model, masters, opt


def run_ours(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        return run_fsdp(args)
    from qwen3_triton import _abi
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    counter = Counter()
    # the full model fits one B200: fp32 masters + moments 98 GB, bf16 working copies and gradients 33 GB, activations 6 GB
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
    sampler = ClockSampler(0, args.out)
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
    status = _abi.read_status()          # a kernel that gave up or saw a bad label would have left its bit here

    # end to end: pinned host ids copied in, loss read back, every step
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(args.steps):
        ids = host_ids[i % len(host_ids)].to(device, non_blocking=True)
        last = float(step(ids).item())
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop()
    status |= _abi.read_status()

    # per-kernel census of one more step with CUDA events around every C-ABI call
    counter.profile = True
    step(dev_ids[0])
    torch.cuda.synchronize()
    counter.profile = False
    roofline = roofline_of(counter)
    peak_tf, _, peak_kind = measured_peaks()
    mfu = value * model_flops_per_token(cfg, seq) / (peak_tf * 1e12)
    if os.environ.get("Q3_BENCH_SKIP_CPU"):     # profiling runs under ncu skip the host-side baseline leg
        cpu = {"value": None, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port", "sample": "skipped"}
    else:
        cpu_tps, _, note = cpu_workload_baseline(layers, 128)
        cpu = {"value": cpu_tps, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port", "sample": note,
               "extra": None if os.environ.get("Q3_BENCH_SKIP_CPU_OPS") else cpu_operator_baselines()}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": ("qwen3-8b full 36-layer model on one GPU, fwd+bwd+AdamW, microbatch 1x2048 (the per-GPU "
                                "workload of the multi-GPU runs, unsharded)" if layers == 36 else
                                "qwen3-8b 4-layer slice fwd+bwd+AdamW, microbatch 4x2048"),
                   "global_batch": batch, "seq_len": seq, "parallelism": "single",
                   "l2": "inputs+weights >> L2 (%d GB bf16 weights)" % (16 if layers == 36 else 4),
                   "loss_head": "no logits in memory" if getattr(model, "fused_loss", False) else "materialised logits",
                   "adamw": ("decoder layers updated during backward on a side stream (%d bucket launches so far), "
                             "embedding / final norm / head after backward" % opt._early.launched
                             if getattr(opt, "_early", None) is not None else "after backward"),
                   "mfu_of_%s_peak" % peak_kind: mfu, "last_loss": last, "device_status": status,
                   "peak_memory_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": batch * seq * 8,
                "d2h_bytes_per_step": 4},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": roofline,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)
    if status:
        raise SystemExit("device status word is not clean: %d (see include/q3b200.h, Q3_STATUS_*)" % status)


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


PARITY_PARAMS = ("model.layers.0.self_attn.q_proj.weight", "model.layers.%d.mlp.down_proj.weight",
                 "model.layers.%d.mlp.gate_proj.weight", "lm_head.weight")


def unsharded_yardstick(cfg, device, all_ids, rank, world, names):
    """Loss and this rank's gradient rows of `names` from ONE unsharded bf16 copy of the model run on the
    concatenated batch of all ranks (what FSDP's averaged gradients must equal). Built from the same seed as the
    sharded model, freed before that one is built."""
    from qwen3_triton import model_for_variant
    torch.manual_seed(20261114)
    with torch.device(device):
        whole = model_for_variant(cfg, "b200_fused")
    whole = whole.to(device=device, dtype=torch.bfloat16)
    whole.model.set_recompute("full")
    whole.fused_loss = True
    ids = torch.cat(all_ids).to(device)
    loss = whole(ids, labels=ids).loss
    loss.backward()
    named = dict(whole.named_parameters())
    shards = {}
    for name in names:
        g = named[name].grad
        rows = g.shape[0] // world
        shards[name] = g[rank * rows:(rank + 1) * rows].float().clone()
    value = float(loss)
    del whole, named, loss
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return value, shards


def run_fsdp(args):
    """N > 1: the full 36-layer model under FSDP2 (one process per GPU, NCCL), bf16 parameter all-gather, fp32
    gradient reduce-scatter, vocabulary-parallel lm_head + cross-entropy and embedding, microbatch 1 x 2048 per GPU,
    AdamW every step; per-layer activation recomputation for the headline number, the lighter policies after it."""
    import torch.distributed as dist
    from qwen3_triton import _abi, model_for_variant
    from qwen3_triton.runtime.adamw import TritonAdamW
    from qwen3_triton.runtime.collectives import NcclCollectives
    from qwen3_triton.runtime.fsdp import configure
    from qwen3_triton.training.sharding import shard_vocab_loss_model

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    pg_options = None
    max_ctas = int(os.environ.get("Q3_BENCH_NCCL_MAX_CTAS", "0"))
    if max_ctas > 0:
        # fewer NCCL CTAs leave more SMs (and HBM bandwidth) to the GEMMs the collectives run beside
        pg_options = dist.ProcessGroupNCCL.Options()
        pg_options.config.max_ctas = max_ctas
        pg_options.config.min_ctas = min(max_ctas, int(os.environ.get("Q3_BENCH_NCCL_MIN_CTAS", "1")))
    dist.init_process_group("nccl", device_id=device, pg_options=pg_options)
    counter = Counter()
    layers = int(os.environ.get("Q3_BENCH_LAYERS", "36"))
    batch, seq = 1, 2048
    cfg = slice_config(layers)
    host_ids = [[torch.randint(0, cfg.vocab_size, (batch, seq), generator=torch.Generator().manual_seed(100 * (k + 1) + r))
                 for r in range(world)] for k in range(8)]

    parity = None
    names = [n % (layers // 2 if i == 1 else layers - 1) if "%d" in n else n for i, n in enumerate(PARITY_PARAMS)]
    if os.environ.get("Q3_BENCH_PARITY", "1") == "1":
        yard_loss, yard = unsharded_yardstick(cfg, device, host_ids[0], rank, world, names)

    torch.manual_seed(20261114)            # same weights on every rank
    with torch.device(device):
        model = model_for_variant(cfg, os.environ.get("Q3_BENCH_VARIANT", "b200_fused"))
    comm = NcclCollectives()
    # the vocabulary-parallel head and embedding talk over their own communicator, so that their small collectives on
    # the compute stream do not queue behind FSDP's reduce-scatters on the same NCCL communicator
    vocab_comm = NcclCollectives(group=dist.new_group()) if os.environ.get("Q3_BENCH_VP_GROUP", "1") == "1" else None
    policies = [p for p in os.environ.get("Q3_BENCH_CHECKPOINT", "full,selective,none").split(",") if p]
    model = shard_vocab_loss_model(model, keep_full_layers=layers, checkpoint_every=1,
                                   skip_embedding_backward_gather=True, fused_vocab_dw=True, communication=vocab_comm,
                                   checkpoint_mode=policies[0], layers_per_unit=unit_sizes(layers),
                                   vocab_parallel_embedding=os.environ.get("Q3_BENCH_VP_EMBEDDING", "1") == "1",
                                   forward_prefetch=int(os.environ.get("Q3_BENCH_FORWARD_PREFETCH", "2")))
    model.lm_head.fused = os.environ.get("Q3_BENCH_FUSED_LOSS", "1") == "1"
    # gradients reduced by the pull kernel over peer memory (bf16 on the links, fp32 sums) unless Q3_BENCH_PEER_REDUCE=0
    peer_reduce = os.environ.get("Q3_BENCH_PEER_REDUCE", "1") == "1" and world in (2, 4, 8)
    hooks = configure(model, comm, pack_gradients_off_compute_stream=os.environ.get("Q3_BENCH_PACK_SIDE", "0") == "1",
                      peer_memory_reduce=peer_reduce,
                      copy_engine_gather=os.environ.get("Q3_BENCH_CE_GATHER", "1") == "1",
                      early_copy_out=os.environ.get("Q3_BENCH_EARLY_COPY_OUT", "0") == "1",
                      gradients_in_staging=os.environ.get("Q3_BENCH_GRAD_HOMES", "1") == "1",
                      gather_into_parameters=os.environ.get("Q3_BENCH_DIRECT_GATHER", "0") == "1")
    peer_reduce = hooks["peer_reducer"] is not None        # False on every rank if the mappings could not be made
    decoder = [p for n, p in model.named_parameters() if not n.startswith("lm_head.")]
    opt = TritonAdamW([dict(params=decoder), dict(params=[model.lm_head.weight])], lr=1e-4, betas=(0.9, 0.95),
                      weight_decay=0.1, block=16384)
    pinned = [k[rank].pin_memory() for k in host_ids]
    dev_ids = [h.to(device) for h in pinned]

    def set_policy(policy):
        for layer in model.model.layers:
            layer.recompute = {"full": 2, "selective": 1, "none": 0}[policy]

    def step(ids):
        opt.zero_grad(set_to_none=True)
        out = model(ids, labels=ids)
        out.loss.backward()
        opt.step()
        return out.loss

    if os.environ.get("Q3_BENCH_PARITY", "1") == "1":
        # First step of the sharded model on the same global batch, before any update: the mean of the ranks' losses
        # against the unsharded loss, and the reduce-scattered (rank-averaged) gradient shards against the unsharded
        # gradient rows. Worst value over ranks.
        opt.zero_grad(set_to_none=True)
        out = model(dev_ids[0], labels=dev_ids[0])
        out.loss.backward()
        mean_loss = out.loss.detach().float().clone()
        dist.all_reduce(mean_loss, op=dist.ReduceOp.AVG)
        named = dict(model.named_parameters())
        rel = torch.zeros(len(names), device=device)
        ratio = torch.zeros(len(names), device=device)
        for i, name in enumerate(names):
            g = named[name].grad
            g = (g.to_local() if hasattr(g, "to_local") else g).float()
            rel[i] = (g - yard[name]).norm() / yard[name].norm()
            ratio[i] = g.norm() / yard[name].norm()
        dist.all_reduce(rel, op=dist.ReduceOp.MAX)
        dist.all_reduce(ratio, op=dist.ReduceOp.MAX)
        parity = {"loss": abs(float(mean_loss) - yard_loss) / abs(yard_loss), "grads": float(rel.max()),
                  "grads_by_tensor": {n: round(float(v), 5) for n, v in zip(names, rel)},
                  "grad_norm_ratio_by_tensor": {n: round(float(v), 4) for n, v in zip(names, ratio)},
                  "what": "first step vs one unsharded bf16 model on the concatenated %d x 2048 batch: relative loss "
                          "difference; relative L2 (worst over ranks) of this rank's gradient shard of each tensor" % world}
        del yard, named
        opt.zero_grad(set_to_none=True)

    early_adamw = os.environ.get("Q3_BENCH_EARLY_ADAMW", "0") == "1"
    if early_adamw:
        # the shards of the units reduced so far (and the head's weight) are updated on the reduce-scatter stream at
        # the next unit's reduce-scatter, beside the backward pass of the units still to come; opt.step() does the rest
        eligible = frozenset(id(p) for n, p in model.named_parameters()
                             if n.startswith("model.layers.") or n.startswith("lm_head."))
        hooks["reduce_scatter"].before_reduce = lambda: opt.step_pending(eligible)

    def timed(policy, steps, warmup):
        set_policy(policy)
        for i in range(warmup):
            step(dev_ids[i % len(dev_ids)])
        torch.cuda.synchronize()
        dist.barrier()
        counter.launches = 0
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for i in range(steps):
            step(dev_ids[i % len(dev_ids)])
        end.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([start.elapsed_time(end) / steps], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), counter.launches

    sampler = ClockSampler(local, args.out) if rank == 0 else None
    ms, launches = timed(policies[0], args.steps, args.warmup)
    status = _abi.read_status()

    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        ids = pinned[i % len(pinned)].to(device, non_blocking=True)
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
        prof.export_chrome_trace(str(Path(args.out) / "trace_rank0.json"))
    elif os.environ.get("Q3_BENCH_PROFILE"):
        step(dev_ids[0])
    counter.profile = True
    step(dev_ids[0])
    torch.cuda.synchronize()
    counter.profile = False
    roofline = roofline_of(counter)
    peak_memory = round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)
    dist.barrier()

    others = {}
    short = max(3, min(args.steps, 6))
    for policy in policies[1:]:
        other_ms, _ = timed(policy, short, 2)
        others[policy] = other_ms
    status |= _abi.read_status()
    bad = torch.tensor([status], device=device)
    dist.all_reduce(bad, op=dist.ReduceOp.MAX)     # any non-zero word on any rank fails the run
    status = int(bad.item())

    if rank == 0:
        peak_tf, _, peak_kind = measured_peaks()
        tokens = batch * seq * world
        value = tokens / (ms * 1e-3)
        flops_tok = model_flops_per_token(cfg, seq)
        mfu = (value / world) * flops_tok / (peak_tf * 1e12)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "qwen3-8b %d layers under FSDP2, microbatch 1x2048 per GPU, vocab-parallel head%s, "
                                   "%s activation recomputation per layer, AdamW every step" % (
                                       layers, " and embedding" if os.environ.get("Q3_BENCH_VP_EMBEDDING", "1") == "1" else "",
                                       policies[0]),
                       "global_batch": batch * world, "seq_len": seq, "parallelism": "fsdp%d" % world,
                       "l2": "weights and activations >> L2",
                       "loss_head": "no logits in memory" if model.lm_head.fused else "materialised logits shard",
                       "mfu_of_%s_peak_per_gpu" % peak_kind: mfu, "mfu_basis": "model FLOPs (recomputed forward not counted)",
                       "tokens_per_s_per_gpu": value / world, "last_loss": last, "device_status": status,
                       "parity_step1_rel": parity,
                       "other_recompute_policies": {p: {"ms_per_step": v, "tokens_per_s": tokens / (v * 1e-3),
                                                        "mfu_of_%s_peak_per_gpu" % peak_kind:
                                                            (tokens / world / (v * 1e-3)) * flops_tok / (peak_tf * 1e12),
                                                        "steps": short} for p, v in others.items()},
                       "peak_memory_gb_rank0": peak_memory, "nccl_max_ctas": max_ctas or "default",
                       "adamw": ("shards of reduced units updated during backward on the reduce-scatter stream, "
                                 "the rest after backward" if early_adamw else "after backward"),
                       "parameter_gather": ("copy-engine pulls from peer-mapped buffers (%d of %d all-gather calls)" % (
                                                hooks["all_gather"].peer_calls, hooks["all_gather"].calls)
                                            if hooks["peer_gather"] is not None else "NCCL all-gather"),
                       "parameter_copy_out": ("none: pieces gathered straight into the parameters"
                                              if hooks["gather_into_parameters"] else
                                              "ahead of time on a side stream" if hooks["early_copy_out"]
                                              else "on the compute stream (FSDP2's place)"),
                       "gradient_pack": ("%d of %d weight gradients written by their GEMMs into the staging buffer, "
                                         "%d copied there" % (hooks["peer_reducer"].born_in_place,
                                                              hooks["peer_reducer"].born_in_place
                                                              + hooks["peer_reducer"].copied_home,
                                                              hooks["peer_reducer"].copied_home)
                                         if hooks["gradient_homes"] else "one pack kernel per FSDP unit"),
                       "gradient_reduce": ("pull kernel over peer memory, bf16 on the links, fp32 sums in rank order "
                                           "(%d of %d reduce-scatter calls)" % (hooks["reduce_scatter"].peer_calls,
                                                                                hooks["reduce_scatter"].calls)
                                           if peer_reduce else "NCCL fp32 reduce-scatter"),
                       "fsdp_units": hooks["units"], "collectives": comm.report()},
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": batch * seq * 8 * world,
                    "d2h_bytes_per_step": 4 * world},
            "gpu_launches": launches, "clocks": clocks,
            "roofline": roofline,
        }
        print(json.dumps(line), flush=True)
    if hooks["peer_gather"] is not None:
        hooks["peer_gather"].close()
    if hooks["peer_reducer"] is not None:
        hooks["peer_reducer"].close()
    dist.destroy_process_group()
    if status:
        raise SystemExit("device status word is not clean: %d (see include/q3b200.h, Q3_STATUS_*)" % status)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--out", default=None, help="directory for the clock samples (default: a temporary directory)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    if args.out is None:
        with tempfile.TemporaryDirectory(prefix="q3bench_") as tmp:
            args.out = tmp
            return run_ours(args)
    Path(args.out).mkdir(parents=True, exist_ok=True)
    run_ours(args)


if __name__ == "__main__":
    main()
