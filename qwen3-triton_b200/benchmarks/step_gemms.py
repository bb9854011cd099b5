#!/usr/bin/env python
"""The GEMM launches of one training step at Qwen3-8B shapes, in launch order: one decoder layer plus the loss head.

    python qwen3-triton_b200/benchmarks/step_gemms.py [--tokens 2048] [--json out.json]

Builds a 1-layer model with the 8B widths (hidden 4096, 32/8 heads of 128, MLP 12288, vocabulary 151936), runs one
warm-up step and one recorded forward + backward through the fused decoder layer and the no-logits loss head, and
prints every tensor-core GEMM entry point called in the recorded step with its FLOPs, its algorithmic bytes (operands
read once, result written once) and its CUDA-event time. The launch order is deterministic, so a profiler capture of
the same command (`-k regex:gemm_tc_kernel`, skipping the warm-up step's launches) lines up with this list row by row:
that is how the DRAM bytes per GEMM shape behind the roofline `traffic` figure are obtained. A full step of the
36-layer model repeats the layer rows 36 times.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import torch  # noqa: E402

from qwen3_triton import Qwen3Config, _abi, model_for_variant  # noqa: E402

GEMMS = {"q3_gemm", "q3_gemm_acc", "q3_gemm_acc_f32", "q3_gate_up_swiglu_fwd", "q3_linear_fwd_grouped",
         "q3_linear_dgrad_grouped", "q3_linear_wgrad_grouped", "q3_down_dgrad_swiglu_bwd", "q3_linear_ce_stats",
         "q3_linear_ce_grad"}


def work(name, a):
    """(description, FLOPs, algorithmic bytes) of one GEMM entry-point call."""
    def dense(m, n, k, out_bytes):
        return 2.0 * m * n * k, 2.0 * (m * k + n * k) + out_bytes * m * n
    if name in ("q3_gemm", "q3_gemm_acc"):
        lay = "A:%s B:%s" % ("K" if a[2] == 1 else "MN", "K" if a[4] == 1 else "MN")
        return (f"{a[7]}x{a[8]}x{a[9]} {lay} out={'f32' if a[11] == 0 else '16b'}",) + dense(a[7], a[8], a[9], 4 if a[11] == 0 else 2)
    if name == "q3_gemm_acc_f32":
        return (f"{a[7]}x{a[8]}x{a[9]} += f32",) + dense(a[7], a[8], a[9], 8)
    if name == "q3_gate_up_swiglu_fwd":
        m, n, k = a[6], a[7], a[8]
        return f"{m}x(2x{n})x{k} gate|up", 4.0 * m * n * k, 2.0 * (m * k + 2 * n * k) + 6.0 * m * n
    if name == "q3_down_dgrad_swiglu_bwd":
        m, i, h = a[6], a[7], a[8]
        return f"{m}x{i}x{h} dY->dG,dU", 2.0 * m * i * h, 2.0 * (m * h + i * h) + 8.0 * m * i
    if name.endswith("_grouped"):
        m, k, sizes = a[5], a[6], [a[3][i] for i in range(a[4])]
        return f"M={m} K={k} group={sizes}", 2.0 * m * k * sum(sizes), 2.0 * (m * k + sum(sizes) * k + m * sum(sizes))
    if name == "q3_linear_ce_stats":
        m, v, k = a[6], a[7], a[8]
        return f"{m}x{v}x{k} logits->stats", 2.0 * m * v * k, 2.0 * (m * k + v * k)
    m, v, k = a[7], a[8], a[9]
    return (f"{m}x{v}x{k} logits->dZ",) + dense(m, v, k, 2)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    torch.manual_seed(0)
    cfg = Qwen3Config(num_hidden_layers=1)
    with torch.device("cuda"):
        model = model_for_variant(cfg, "b200_fused")
    model = model.to("cuda", torch.bfloat16)
    model.fused_loss = True
    ids = torch.randint(0, cfg.vocab_size, (1, a.tokens), device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    records = []
    orig = _abi.call

    def recording(name, *args):
        if name not in GEMMS:
            return orig(name, *args)
        flush.zero_()                      # operands come from HBM, as they do between the layers of a real step
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        orig(name, *args)
        e.record()
        records.append((name, args, s, e))

    def step():
        model.zero_grad(set_to_none=True)
        model(ids, labels=ids).loss.backward()

    step()                                 # warm-up: module loading, allocator, tensor-map driver entry point
    torch.cuda.synchronize()
    _abi.call = recording
    step()
    torch.cuda.synchronize()
    _abi.call = orig
    rows = []
    for name, args, s, e in records:
        what, flops, nbytes = work(name, args)
        ms = s.elapsed_time(e)
        rows.append({"entry": name, "shape": what, "flops": flops, "algorithmic_bytes": nbytes, "ms": ms})
        print(f"{len(rows):3d} {name:26s} {what:44s} {ms * 1e3:8.1f} us {flops / ms / 1e9:8.1f} TFLOP/s {nbytes / 1e6:9.1f} MB")
    assert _abi.read_status() == 0
    if a.json:
        Path(a.json).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
